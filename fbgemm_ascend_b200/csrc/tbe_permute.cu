// permute_pooled_embs for B200: column-block permutation of a [B, total_D] matrix.
//
// Replaces aclnnPermutePooledEmbs (reference: permute_pooled_embs.cpp:62-105 and
// v220/op_kernel/permute_pooled_embs_kernel.h:140-211).  Pure copy, bounded by HBM
// bandwidth: 2 * B * total_D * elem_bytes per call.
//
// One thread owns one 16-byte vector of output columns for kRows consecutive
// rows: it finds the output feature holding its first column once (binary search
// of inv_offset_dim_list), then issues kRows independent 16-byte loads and
// stores.  A vector that straddles two features, or whose source is not 16-byte
// aligned, is copied element by element instead, so any dims are accepted and
// the host never has to read the lists (the reference syncs on them at
// permute_pooled_embs.cpp:82-92).  Zero-width features are skipped.
#include "tbe_common.cuh"

namespace tbe {
namespace {

constexpr int kRows = 8;
constexpr int kThreads = 256;

struct PermuteParams {
    const char* in;
    char* out;
    const int64_t* off;       // offset_dim_list      [T+1]
    const int64_t* perm;      // permute_list         [T]
    const int64_t* inv_off;   // inv_offset_dim_list  [T+1]
    int32_t* error_flag;
    int64_t B;
    int64_t total_D;
    int64_t in_stride;        // bytes
    int64_t out_stride;       // bytes
    int64_t blk_cols;         // source columns per block (total_D when the source is one matrix)
    int64_t blk_stride;       // bytes between consecutive source blocks
    int32_t T;
    int32_t esz;
    bool vec_ok;              // bases and strides are 16-byte aligned
};

// Largest i in [0, T) with inv_off[i] <= c (c < inv_off[T]).
__device__ __forceinline__ int find_feature(const int64_t* inv_off, int T, int64_t c)
{
    int lo = 0, hi = T;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(inv_off + mid) <= c) lo = mid;
        else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(kThreads) permute_pooled_embs_kernel(const PermuteParams p)
{
    const int ve = 16 / p.esz;   // elements per 16-byte vector
    const int64_t vec = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t c0 = vec * ve;
    if (c0 >= p.total_D) return;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kRows;
    const int nrows = static_cast<int>(min(static_cast<int64_t>(kRows), p.B - row0));

    int i = find_feature(p.inv_off, p.T, c0);
    const int64_t seg_lo = __ldg(p.inv_off + i);
    const int64_t seg_hi = __ldg(p.inv_off + i + 1);
    const int64_t pi = __ldg(p.perm + i);
    const bool pi_ok = pi >= 0 && pi < p.T;
    const int64_t src_c0 = pi_ok ? __ldg(p.off + pi) + (c0 - seg_lo) : 0;
    // Source column c lives in block c / blk_cols at column c % blk_cols.
    const int64_t blk0 = src_c0 / p.blk_cols;
    const int64_t in_blk0 = src_c0 - blk0 * p.blk_cols;

    if (p.vec_ok && pi_ok && c0 + ve <= seg_hi && c0 + ve <= p.total_D && ((in_blk0 * p.esz) & 15) == 0 &&
        in_blk0 + ve <= p.blk_cols) {
        const char* src = p.in + blk0 * p.blk_stride + row0 * p.in_stride + in_blk0 * p.esz;
        char* dst = p.out + row0 * p.out_stride + c0 * p.esz;
        uint4 v[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (r < nrows) v[r] = ldg16(src + r * p.in_stride);
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (r < nrows) *reinterpret_cast<uint4*>(dst + r * p.out_stride) = v[r];
        return;
    }

    // Element-wise: walk the (possibly several) features this vector touches.
    const int64_t c_end = min(c0 + ve, p.total_D);
    for (int64_t c = c0; c < c_end; ++c) {
        while (i + 1 < p.T && c >= __ldg(p.inv_off + i + 1)) ++i;
        const int64_t q = __ldg(p.perm + i);
        if (q < 0 || q >= p.T) {
            if (p.error_flag) atomicOr(p.error_flag, 1);
            continue;
        }
        const int64_t sc = __ldg(p.off + q) + (c - __ldg(p.inv_off + i));
        for (int r = 0; r < nrows; ++r) {
            const int64_t sb = sc / p.blk_cols;
            const char* s = p.in + sb * p.blk_stride + (row0 + r) * p.in_stride + (sc - sb * p.blk_cols) * p.esz;
            char* d = p.out + (row0 + r) * p.out_stride + c * p.esz;
            if (p.esz == 4) *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s);
            else *reinterpret_cast<uint16_t*>(d) = *reinterpret_cast<const uint16_t*>(s);
        }
    }
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_b200_permute_pooled_embs_blocked(const void* pooled_embs, int64_t B, int64_t total_D, int32_t elem_bytes,
                                                    int64_t in_stride, int64_t out_stride, int64_t block_cols,
                                                    int64_t block_stride, const int64_t* offset_dim_list,
                                                    const int64_t* permute_list, const int64_t* inv_offset_dim_list,
                                                    int32_t T, void* output, int32_t* error_flag, tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (elem_bytes != 2 && elem_bytes != 4)
        return fail(TBE_B200_ERR_UNSUPPORTED, "permute_pooled_embs: elem_bytes must be 2 or 4, got %d", elem_bytes);
    if (T <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_pooled_embs: T must be positive, got %d", T);
    if (B < 0 || total_D < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_pooled_embs: negative size");
    if (B == 0 || total_D == 0) return TBE_B200_OK;
    if (!pooled_embs || !output || !offset_dim_list || !permute_list || !inv_offset_dim_list)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_pooled_embs: a required pointer is NULL");
    if (block_cols <= 0 || block_cols > total_D) block_cols = total_D;
    if (in_stride < block_cols || out_stride < total_D)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_pooled_embs: row stride smaller than the row width");

    PermuteParams p;
    p.in = static_cast<const char*>(pooled_embs);
    p.out = static_cast<char*>(output);
    p.off = offset_dim_list;
    p.perm = permute_list;
    p.inv_off = inv_offset_dim_list;
    p.error_flag = error_flag;
    p.B = B;
    p.total_D = total_D;
    p.in_stride = in_stride * elem_bytes;
    p.out_stride = out_stride * elem_bytes;
    p.blk_cols = block_cols;
    p.blk_stride = block_stride * elem_bytes;
    p.T = T;
    p.esz = elem_bytes;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(pooled_embs) | reinterpret_cast<uintptr_t>(output) |
                 static_cast<uint64_t>(p.in_stride) | static_cast<uint64_t>(p.out_stride) |
                 static_cast<uint64_t>(p.blk_stride)) & 15) == 0;

    const int ve = 16 / elem_bytes;
    const int64_t nvec = (total_D + ve - 1) / ve;
    const int64_t gx = (nvec + kThreads - 1) / kThreads;
    const int64_t gy = (B + kRows - 1) / kRows;
    if (gx > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "permute_pooled_embs: total_D too large");
    // grid.y is limited to 65535: cover taller inputs with several launches.
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t max_gy = 65535;
    for (int64_t y0 = 0; y0 < gy; y0 += max_gy) {
        PermuteParams q = p;
        const int64_t rows_done = y0 * kRows;
        q.in = p.in + rows_done * p.in_stride;
        q.out = p.out + rows_done * p.out_stride;
        q.B = B - rows_done;
        const int64_t this_gy = (gy - y0 < max_gy) ? (gy - y0) : max_gy;
        if (this_gy < max_gy) { /* last launch keeps q.B as the remaining rows */ }
        else q.B = max_gy * kRows;
        permute_pooled_embs_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(this_gy)), kThreads, 0, s>>>(q);
    }
    return check_launch("permute_pooled_embs_kernel");
}

extern "C" int tbe_b200_permute_pooled_embs(const void* pooled_embs, int64_t B, int64_t total_D, int32_t elem_bytes,
                                            int64_t in_stride, int64_t out_stride, const int64_t* offset_dim_list,
                                            const int64_t* permute_list, const int64_t* inv_offset_dim_list, int32_t T,
                                            void* output, int32_t* error_flag, tbe_b200_stream_t stream)
{
    return tbe_b200_permute_pooled_embs_blocked(pooled_embs, B, total_D, elem_bytes, in_stride, out_stride, total_D, 0,
                                                offset_dim_list, permute_list, inv_offset_dim_list, T, output, error_flag,
                                                stream);
}
