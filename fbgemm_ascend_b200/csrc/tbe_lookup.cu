// Quantized table-batched-embedding lookup for B200 (sm_100a).
//
// Replaces the device side of int_nbit_split_embedding_codegen_lookup_function
// (reference: c310/op_kernel/int_nbit_split_embedding_pooling_kernel.h:44-394 and
// int_nbit_split_embedding_nobag_kernel.h:31-398).  The path is a gather and a
// reduction bounded by HBM/L2 bandwidth, so there is no tensor-core work here.
//
// Pooled kernel, one warp per bag (t, b):
//   * the warp reads up to 32 of the bag's indices (and per-sample weights) with one
//     coalesced load and hands them out with shuffles;
//   * LPR lanes (2..32, a power of two chosen from the row width) cooperate on one
//     row, so 32/LPR rows of the bag are fetched concurrently, each lane with one
//     16-byte (INT8/FP8/FP16/FP32) or 8-byte (INT4) load; rows are dequantised in
//     registers with the row's fp16 scale/bias and accumulated in fp32, 16
//     accumulators per lane;
//   * INT8/INT4 rows start with a 4-byte header, which shifts the payload off the
//     16-byte grid.  The lane that loads the header chunk has 4 (INT8) or 8 (INT4)
//     free slots; when D is a multiple of 16 they take the row's last elements,
//     which would otherwise need one more lane.  D = 16*LPR rows then keep every
//     lane busy with exactly 16 elements;
//   * the per-group partial sums are combined with a reduce-scatter over
//     shuffles, after which every lane owns 16*LPR/32 finished elements and
//     stores them (8- or 16-byte stores);
//   * rows of any other shape (row_alignment 1, odd D, INT2, unaligned tables)
//     take a byte-wise path with the same results.
#include <stdarg.h>
#include <stdio.h>

#include "tbe_common.cuh"

namespace tbe {

namespace {

constexpr unsigned kFull = 0xffffffffu;

struct LookupParams {
    const uint8_t* dev_weights;
    const int64_t* weights_offsets;
    const uint8_t* weights_tys;
    const int32_t* D_offsets;
    const void* indices;
    const void* offsets;
    const float* pw;
    void* output;
    const int64_t* out_cols;
    void* const* dests;
    int32_t* error_flag;
    int64_t B;
    int64_t num_bags;
    int64_t out_stride;
    int64_t rows_per_dest;
    int32_t T;
    uint32_t B32;        // B when T*B < 2^32, else 0
    int32_t pooling_mode;
    int32_t out_ty;
    int32_t row_alignment;
    uint32_t fp8_shift;  // 16 + exponent bits
    float fp8_mult;      // 2^(127 - bias)
};

__host__ __device__ inline int64_t row_bytes_of(int ty, int D, int align)
{
    int64_t b;
    switch (ty) {
        case TBE_B200_FP32: b = 4ll * D; break;
        case TBE_B200_FP16: b = 2ll * D; break;
        case TBE_B200_BF16: b = 2ll * D; break;
        case TBE_B200_FP8: b = D; break;
        case TBE_B200_INT8: b = D + 4ll; break;
        case TBE_B200_INT4: b = (D + 1) / 2 + 4ll; break;
        case TBE_B200_INT2: b = (D + 3) / 4 + 4ll; break;
        default: return 0;
    }
    if (align > 1) b = (b + align - 1) / align * align;
    return b;
}

// ---- output ----------------------------------------------------------------

// Converts and stores N (1, 2 or 4) consecutive finished elements.  `p` points at
// the first of them in the output, already offset; `vec` says the address is
// aligned for one N-wide store.
template <int N>
__device__ __forceinline__ void store_out(void* seg, int e0, const float* v, int out_ty, bool vec)
{
    if (out_ty == TBE_B200_FP32) {
        float* p = static_cast<float*>(seg) + e0;
        if (N == 4 && vec) {
            st_stream16(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                                      __float_as_uint(v[3])));
        } else if (N == 2 && vec) {
            st_stream8(p, make_uint2(__float_as_uint(v[0]), __float_as_uint(v[1])));
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j) p[j] = v[j];
        }
    } else {
        uint32_t h[N];
#pragma unroll
        for (int j = 0; j < N; ++j) h[j] = (out_ty == TBE_B200_FP16) ? f32_to_f16_bits(v[j]) : f32_to_bf16_bits(v[j]);
        unsigned short* p = static_cast<unsigned short*>(seg) + e0;
        if (N == 4 && vec) {
            st_stream8(p, make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16)));
        } else if (N == 2 && vec) {
            st_stream4(p, h[0] | (h[1] << 16));
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j) p[j] = static_cast<unsigned short>(h[j]);
        }
    }
}

// ---- per-type row access ---------------------------------------------------
//
// Every lane owns 16 accumulator "slots".  A path says which bytes a lane loads
// for a row (load), how they add into the slots (accum), and which element of
// the row a slot stands for (elem).  `unit` is the lane's position among the
// 16-slot units of the row: unit = block * LPR + k.

struct LaneCtx {
    int unit;        // 16-slot unit handled by this lane in the current block
    int D;           // elements per row
    bool active;     // this unit exists in the row
    bool wrap;       // INT8/INT4 header lane that also takes the row's tail
    bool first_blk;  // block 0: the header chunk is held by lane k == 0 of the group
    uint32_t fp8_shift;
    float fp8_mult;
};

template <int TY>
struct Path;

template <>
struct Path<TBE_B200_INT8> {
    struct Regs {
        uint4 v;
        uint32_t hdr;
    };
    static constexpr bool kHasHeader = true;
    // 16-byte chunks of the row: chunk c covers elements [16c - 4, 16c + 12).
    static __device__ __forceinline__ int units(int D, bool wrap) { return wrap ? D / 16 : (D + 4 + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int D) { return (D & 15) == 0; }
    static __device__ __forceinline__ void load(Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
    {
        r.v = make_uint4(0u, 0u, 0u, 0u);
        r.hdr = 0u;
        if (ok && cx.active) r.v = ldg16(row + cx.unit * 16);
        if (ok && cx.wrap) r.hdr = ldg4(row + cx.D);            // tail: elements D-4 .. D-1
        else if (ok && !cx.first_blk) r.hdr = ldg4(row);        // later blocks fetch the header directly
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(Regs& r, const LaneCtx& cx, float w, float (&acc)[16], float& bias_acc)
    {
        uint32_t hdr = r.hdr;
        if (cx.first_blk) {
            hdr = __shfl_sync(kFull, r.v.x, 0, LPR);
            if (cx.wrap) r.v.x = r.hdr;
        }
        const float s = half_bits_to_float(hdr & 0xffffu) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), w, bias_acc);
        const uint32_t words[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float q = static_cast<float>((words[i] >> (8 * j)) & 0xffu);
                acc[4 * i + j] = fmaf(q, s, acc[4 * i + j]);
            }
        }
    }
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot, int /*LPR*/)
    {
        if (cx.wrap && slot < 4) return cx.D - 4 + slot;
        return 16 * cx.unit - 4 + slot;
    }
};

template <>
struct Path<TBE_B200_INT4> {
    struct Regs {
        uint2 v;
        uint32_t hdr;
    };
    static constexpr bool kHasHeader = true;
    // 8-byte chunks: chunk c covers elements [16c - 8, 16c + 8).
    static __device__ __forceinline__ int units(int D, bool wrap) { return wrap ? D / 16 : (D / 2 + 4 + 7) / 8; }
    static __device__ __forceinline__ bool can_wrap(int D) { return (D & 15) == 0; }
    static __device__ __forceinline__ void load(Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
    {
        r.v = make_uint2(0u, 0u);
        r.hdr = 0u;
        if (ok && cx.active) r.v = ldg8(row + cx.unit * 8);
        if (ok && cx.wrap) r.hdr = ldg4(row + cx.D / 2);        // tail: elements D-8 .. D-1
        else if (ok && !cx.first_blk) r.hdr = ldg4(row);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(Regs& r, const LaneCtx& cx, float w, float (&acc)[16], float& bias_acc)
    {
        uint32_t hdr = r.hdr;
        if (cx.first_blk) {
            hdr = __shfl_sync(kFull, r.v.x, 0, LPR);
            if (cx.wrap) r.v.x = r.hdr;
        }
        const float s = half_bits_to_float(hdr & 0xffffu) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), w, bias_acc);
        const uint32_t words[2] = {r.v.x, r.v.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float q = static_cast<float>((words[i] >> (4 * j)) & 0xfu);
                acc[8 * i + j] = fmaf(q, s, acc[8 * i + j]);
            }
        }
    }
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot, int /*LPR*/)
    {
        if (cx.wrap && slot < 8) return cx.D - 8 + slot;
        return 16 * cx.unit - 8 + slot;
    }
};

template <>
struct Path<TBE_B200_FP8> {
    struct Regs {
        uint4 v;
    };
    static constexpr bool kHasHeader = false;
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    static __device__ __forceinline__ void load(Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
    {
        r.v = make_uint4(0u, 0u, 0u, 0u);
        if (ok && cx.active) r.v = ldg16(row + cx.unit * 16);
    }
    // Byte -> fp32 by bit placement: ((b & 0x7f) << (16 + ebits)) as a float, times
    // 2^(127 - bias), sign bit or'ed in (reference: c310/op_kernel/common.h:120-167).
    template <int LPR>
    static __device__ __forceinline__ void accum(Regs& r, const LaneCtx& cx, float w, float (&acc)[16], float&)
    {
        const uint32_t words[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t b = (words[i] >> (8 * j)) & 0xffu;
                const float mag = __uint_as_float((b & 0x7fu) << cx.fp8_shift) * cx.fp8_mult;
                const float val = __uint_as_float(__float_as_uint(mag) | ((b & 0x80u) << 24));
                acc[4 * i + j] = fmaf(w, val, acc[4 * i + j]);
            }
        }
    }
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot, int) { return 16 * cx.unit + slot; }
};

template <>
struct Path<TBE_B200_FP16> {
    struct Regs {
        uint4 a, b;
    };
    static constexpr bool kHasHeader = false;
    // A unit is two 16-byte chunks LPR chunks apart, so that one load instruction of
    // a group covers LPR*16 contiguous bytes: with blk = unit / LPR and k = unit % LPR,
    // chunk_a = 2*blk*LPR + k, chunk_b = chunk_a + LPR; a chunk is 8 elements.
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    template <int LPR>
    static __device__ __forceinline__ int chunk_a(int unit) { return 2 * (unit / LPR) * LPR + (unit % LPR); }
    template <int LPR>
    static __device__ __forceinline__ void load_l(Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
    {
        r.a = make_uint4(0u, 0u, 0u, 0u);
        r.b = make_uint4(0u, 0u, 0u, 0u);
        const int ca = chunk_a<LPR>(cx.unit);
        if (ok && cx.active && ca * 8 < cx.D) r.a = ldg16(row + ca * 16);
        if (ok && cx.active && (ca + LPR) * 8 < cx.D) r.b = ldg16(row + (ca + LPR) * 16);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(Regs& r, const LaneCtx&, float w, float (&acc)[16], float&)
    {
        const uint32_t words[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[2 * i] = fmaf(w, half_bits_to_float(words[i] & 0xffffu), acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, half_bits_to_float(words[i] >> 16), acc[2 * i + 1]);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ int elem_l(const LaneCtx& cx, int slot)
    {
        const int ca = chunk_a<LPR>(cx.unit);
        return slot < 8 ? 8 * ca + slot : 8 * (ca + LPR) + slot - 8;
    }
};

template <>
struct Path<TBE_B200_FP32> {
    struct Regs {
        uint4 v[4];
    };
    static constexpr bool kHasHeader = false;
    // A unit is four 16-byte chunks, LPR chunks apart: chunk_m = 4*blk*LPR + m*LPR + k.
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    template <int LPR>
    static __device__ __forceinline__ int chunk0(int unit) { return 4 * (unit / LPR) * LPR + (unit % LPR); }
    template <int LPR>
    static __device__ __forceinline__ void load_l(Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
    {
        const int c0 = chunk0<LPR>(cx.unit);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            r.v[m] = make_uint4(0u, 0u, 0u, 0u);
            if (ok && cx.active && (c0 + m * LPR) * 4 < cx.D) r.v[m] = ldg16(row + (c0 + m * LPR) * 16);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(Regs& r, const LaneCtx&, float w, float (&acc)[16], float&)
    {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            acc[4 * m + 0] = fmaf(w, __uint_as_float(r.v[m].x), acc[4 * m + 0]);
            acc[4 * m + 1] = fmaf(w, __uint_as_float(r.v[m].y), acc[4 * m + 1]);
            acc[4 * m + 2] = fmaf(w, __uint_as_float(r.v[m].z), acc[4 * m + 2]);
            acc[4 * m + 3] = fmaf(w, __uint_as_float(r.v[m].w), acc[4 * m + 3]);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ int elem_l(const LaneCtx& cx, int slot)
    {
        return 4 * (chunk0<LPR>(cx.unit) + (slot >> 2) * LPR) + (slot & 3);
    }
};

template <int TY, int LPR>
__device__ __forceinline__ void path_load(typename Path<TY>::Regs& r, const uint8_t* row, const LaneCtx& cx, bool ok)
{
    if constexpr (TY == TBE_B200_FP16 || TY == TBE_B200_FP32) Path<TY>::template load_l<LPR>(r, row, cx, ok);
    else Path<TY>::load(r, row, cx, ok);
}

template <int TY, int LPR>
__device__ __forceinline__ int path_elem(const LaneCtx& cx, int slot)
{
    if constexpr (TY == TBE_B200_FP16 || TY == TBE_B200_FP32) return Path<TY>::template elem_l<LPR>(cx, slot);
    else return Path<TY>::elem(cx, slot, LPR);
}

// One halving step of the cross-group reduce-scatter: lanes `dist` apart swap the
// half of their N live values that the other one keeps.
template <int N>
__device__ __forceinline__ void halve(float (&a)[16], int dist, bool upper)
{
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
        const float send = upper ? a[j] : a[j + N / 2];
        const float keep = upper ? a[j + N / 2] : a[j];
        a[j] = keep + __shfl_xor_sync(kFull, send, dist);
    }
}

struct BagInfo {
    const uint8_t* table;   // first row of the table
    int64_t stride;         // bytes per row
    int64_t start;          // first position of the bag in indices
    int L;                  // rows in the bag
    int D;
    void* seg;              // output address of element 0 of the bag
    float mean_mul;         // 1/L for MEAN, else 1
    bool seg_aligned;       // seg is 16-byte aligned
};

// Pools one bag whose rows are 16-byte aligned with a 16-byte-multiple stride.
template <int TY, int LPR, typename IdxT>
__device__ __forceinline__ void pool_bag(const LookupParams& p, const BagInfo& bag, int lane)
{
    using P = Path<TY>;
    constexpr int RPI = kWarp / LPR;            // rows in flight per pass of the warp
    constexpr int NF = 16 / RPI;                // finished slots per lane after the reduce-scatter
    constexpr int UNROLL = (TY == TBE_B200_FP32) ? 1 : 2;
    const int k = lane % LPR;
    const int g = lane / LPR;
    const IdxT* indices = static_cast<const IdxT*>(p.indices) + bag.start;
    const float* pw = p.pw ? p.pw + bag.start : nullptr;
    const bool wrap_row = P::can_wrap(bag.D);
    const int nunits = P::units(bag.D, wrap_row);

    for (int ublk = 0; ublk < nunits; ublk += LPR) {
        LaneCtx cx;
        cx.unit = ublk + k;
        cx.D = bag.D;
        // FP16/FP32 units interleave their chunks, so those paths bound-check per chunk instead.
        cx.active = (TY == TBE_B200_FP16 || TY == TBE_B200_FP32) ? true : (cx.unit < nunits);
        cx.first_blk = (ublk == 0);
        cx.wrap = wrap_row && cx.unit == 0;
        cx.fp8_shift = p.fp8_shift;
        cx.fp8_mult = p.fp8_mult;

        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
        float bias_acc = 0.0f;

        for (int base = 0; base < bag.L; base += kWarp) {
            const int nb = min(kWarp, bag.L - base);
            int64_t my_idx = -1;
            float my_w = 1.0f;
            if (lane < nb) {
                my_idx = static_cast<int64_t>(ld_stream(indices + base + lane));
                if (pw) my_w = ld_stream(pw + base + lane);
                if (my_idx < -1 && p.error_flag) atomicOr(p.error_flag, 1);
            }
            const int npass = (nb + RPI - 1) / RPI;
            for (int pass = 0; pass < npass; pass += UNROLL) {
                typename P::Regs regs[UNROLL];
                float w[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int r = (pass + u) * RPI + g;
                    int64_t idx;
                    if constexpr (sizeof(IdxT) == 8) {
                        const uint32_t lo = __shfl_sync(kFull, static_cast<uint32_t>(my_idx), r & 31);
                        const uint32_t hi = __shfl_sync(kFull, static_cast<uint32_t>(my_idx >> 32), r & 31);
                        idx = static_cast<int64_t>((static_cast<uint64_t>(hi) << 32) | lo);
                    } else {
                        idx = static_cast<int64_t>(__shfl_sync(kFull, static_cast<int32_t>(my_idx), r & 31));
                    }
                    w[u] = __shfl_sync(kFull, my_w, r & 31);
                    const bool ok = (r < nb) && (idx >= 0);
                    if (!ok) w[u] = 0.0f;
                    path_load<TY, LPR>(regs[u], bag.table + idx * bag.stride, cx, ok);
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) P::template accum<LPR>(regs[u], cx, w[u], acc, bias_acc);
            }
        }

        // Combine the RPI groups: after this every lane holds NF finished slots,
        // slots [slot_base, slot_base + NF) of its unit.
        int slot_base = 0;
        if constexpr (RPI >= 2) { const bool up = (lane >> 4) & 1; halve<16>(acc, 16, up); slot_base += up ? 8 : 0; }
        if constexpr (RPI >= 4) { const bool up = (lane >> 3) & 1; halve<8>(acc, 8, up); slot_base += up ? 4 : 0; }
        if constexpr (RPI >= 8) { const bool up = (lane >> 2) & 1; halve<4>(acc, 4, up); slot_base += up ? 2 : 0; }
        if constexpr (RPI >= 16) { const bool up = (lane >> 1) & 1; halve<2>(acc, 2, up); slot_base += up ? 1 : 0; }
        if constexpr (P::kHasHeader) {
#pragma unroll
            for (int d = LPR; d < kWarp; d <<= 1) bias_acc += __shfl_xor_sync(kFull, bias_acc, d);
        }

        if (cx.active) {
            constexpr int W = NF >= 4 ? 4 : NF;   // elements per store
#pragma unroll
            for (int q = 0; q < NF / W; ++q) {
                const int slot = slot_base + q * W;
                const int e0 = path_elem<TY, LPR>(cx, slot);
                if (e0 >= 0 && e0 < bag.D) {
                    float v[W];
#pragma unroll
                    for (int j = 0; j < W; ++j) v[j] = (acc[q * W + j] + bias_acc) * bag.mean_mul;
                    store_out<W>(bag.seg, e0, v, p.out_ty, bag.seg_aligned);
                }
            }
        }
    }
}

template <int TY, typename IdxT>
__device__ __forceinline__ void pool_bag_by_width(const LookupParams& p, const BagInfo& bag, int lane)
{
    const bool wrap = Path<TY>::can_wrap(bag.D);
    const int nunits = Path<TY>::units(bag.D, wrap);
    if (nunits <= 2) pool_bag<TY, 2, IdxT>(p, bag, lane);
    else if (nunits <= 4) pool_bag<TY, 4, IdxT>(p, bag, lane);
    else if (nunits <= 8) pool_bag<TY, 8, IdxT>(p, bag, lane);
    else if (nunits <= 16) pool_bag<TY, 16, IdxT>(p, bag, lane);
    else pool_bag<TY, 32, IdxT>(p, bag, lane);
}

// ---- byte-wise path (any alignment, any D, every type) ----------------------

__device__ __forceinline__ float decode_elem(const uint8_t* row, int ty, int e, float scale, float bias,
                                             uint32_t fp8_shift, float fp8_mult)
{
    switch (ty) {
        case TBE_B200_INT8: return fmaf(static_cast<float>(row[4 + e]), scale, bias);
        case TBE_B200_INT4: return fmaf(static_cast<float>((row[4 + (e >> 1)] >> ((e & 1) * 4)) & 0xf), scale, bias);
        case TBE_B200_INT2: return fmaf(static_cast<float>((row[4 + (e >> 2)] >> ((e & 3) * 2)) & 0x3), scale, bias);
        case TBE_B200_FP8: {
            const uint32_t b = row[e];
            const float mag = __uint_as_float((b & 0x7fu) << fp8_shift) * fp8_mult;
            return __uint_as_float(__float_as_uint(mag) | ((b & 0x80u) << 24));
        }
        case TBE_B200_FP16: return half_bits_to_float(row[2 * e] | (static_cast<uint32_t>(row[2 * e + 1]) << 8));
        case TBE_B200_BF16:
            return __uint_as_float((row[2 * e] | (static_cast<uint32_t>(row[2 * e + 1]) << 8)) << 16);
        default: {
            const uint32_t u = row[4 * e] | (static_cast<uint32_t>(row[4 * e + 1]) << 8) |
                               (static_cast<uint32_t>(row[4 * e + 2]) << 16) | (static_cast<uint32_t>(row[4 * e + 3]) << 24);
            return __uint_as_float(u);
        }
    }
}

__device__ __forceinline__ void read_header(const uint8_t* row, int ty, float& scale, float& bias)
{
    scale = 1.0f;
    bias = 0.0f;
    if (ty == TBE_B200_INT8 || ty == TBE_B200_INT4 || ty == TBE_B200_INT2) {
        scale = half_bits_to_float(row[0] | (static_cast<uint32_t>(row[1]) << 8));
        bias = half_bits_to_float(row[2] | (static_cast<uint32_t>(row[3]) << 8));
    }
}

__device__ __forceinline__ void store_scalar(void* seg, int e, float v, int out_ty)
{
    if (out_ty == TBE_B200_FP32) static_cast<float*>(seg)[e] = v;
    else static_cast<unsigned short*>(seg)[e] =
        static_cast<unsigned short>(out_ty == TBE_B200_FP16 ? f32_to_f16_bits(v) : f32_to_bf16_bits(v));
}

constexpr int kByteAcc = 4;   // accumulators per lane in the byte-wise path

template <typename IdxT>
__device__ __noinline__ void pool_bag_bytewise(const IdxT* indices, const float* pw, int32_t* error_flag,
                                               const uint8_t* table, int64_t stride, int L, int D, void* seg,
                                               float mean_mul, int ty, int out_ty, uint32_t fp8_shift,
                                               float fp8_mult, int lane)
{
    for (int e_blk = 0; e_blk < D; e_blk += kByteAcc * kWarp) {
        float acc[kByteAcc];
#pragma unroll
        for (int j = 0; j < kByteAcc; ++j) acc[j] = 0.0f;
        for (int n = 0; n < L; ++n) {
            const int64_t idx = static_cast<int64_t>(indices[n]);
            if (idx < 0) {
                if (idx < -1 && lane == 0 && error_flag) atomicOr(error_flag, 1);
                continue;
            }
            const float w = pw ? pw[n] : 1.0f;
            const uint8_t* row = table + idx * stride;
            float scale, bias;
            read_header(row, ty, scale, bias);
#pragma unroll
            for (int j = 0; j < kByteAcc; ++j) {
                const int e = e_blk + j * kWarp + lane;
                if (e < D) acc[j] = fmaf(w, decode_elem(row, ty, e, scale, bias, fp8_shift, fp8_mult), acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < kByteAcc; ++j) {
            const int e = e_blk + j * kWarp + lane;
            if (e < D) store_scalar(seg, e, acc[j] * mean_mul, out_ty);
        }
    }
}

// ---- kernels -----------------------------------------------------------------

constexpr int kWarpsPerBlock = 4;
constexpr int kMinBlocksPerSM = 8;   // caps the pooled kernel at 64 registers: 32 resident warps per SM

template <typename IdxT>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, kMinBlocksPerSM)
tbe_pooled_kernel(const LookupParams p)
{
    const int lane = threadIdx.x & 31;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (i >= p.num_bags) return;
    int t;
    int64_t b;
    if (p.B32) {
        t = static_cast<int>(static_cast<uint32_t>(i) / p.B32);
        b = static_cast<uint32_t>(i) - static_cast<uint32_t>(t) * p.B32;
    } else {
        t = static_cast<int>(i / p.B);
        b = i - static_cast<int64_t>(t) * p.B;
    }
    const int ty = p.weights_tys[t];
    const int d0 = p.D_offsets[t];
    const int D = p.D_offsets[t + 1] - d0;
    const int64_t woff = p.weights_offsets[t];
    const IdxT* offsets = static_cast<const IdxT*>(p.offsets);
    const int64_t start = static_cast<int64_t>(offsets[i]);
    const int64_t end = static_cast<int64_t>(offsets[i + 1]);

    BagInfo bag;
    bag.table = p.dev_weights + woff;
    bag.stride = row_bytes_of(ty, D, p.row_alignment);
    bag.start = start;
    bag.L = static_cast<int>(end - start);
    bag.D = D;
    bag.mean_mul = (p.pooling_mode == TBE_B200_POOL_MEAN && bag.L > 0) ? 1.0f / static_cast<float>(bag.L) : 1.0f;
    const int64_t col = p.out_cols ? p.out_cols[t] : static_cast<int64_t>(d0);
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    char* dst;
    int64_t brow = b;
    if (p.dests) {
        const int64_t which = b / p.rows_per_dest;
        brow = b - which * p.rows_per_dest;
        dst = static_cast<char*>(p.dests[which]);
    } else {
        dst = static_cast<char*>(p.output);
    }
    bag.seg = dst + (brow * p.out_stride + col) * esz;
    bag.seg_aligned = (reinterpret_cast<uintptr_t>(bag.seg) & 15) == 0;
    if (D <= 0) return;

    const bool rows_aligned = ((reinterpret_cast<uintptr_t>(bag.table) | static_cast<uint64_t>(bag.stride)) & 15) == 0;
    if (rows_aligned && (D & 3) == 0) {
        switch (ty) {
            case TBE_B200_INT8: pool_bag_by_width<TBE_B200_INT8, IdxT>(p, bag, lane); return;
            case TBE_B200_INT4: pool_bag_by_width<TBE_B200_INT4, IdxT>(p, bag, lane); return;
            case TBE_B200_FP8: pool_bag_by_width<TBE_B200_FP8, IdxT>(p, bag, lane); return;
            case TBE_B200_FP16:
                if ((D & 7) == 0) { pool_bag_by_width<TBE_B200_FP16, IdxT>(p, bag, lane); return; }
                break;
            case TBE_B200_FP32: pool_bag_by_width<TBE_B200_FP32, IdxT>(p, bag, lane); return;
            default: break;
        }
    }
    pool_bag_bytewise<IdxT>(static_cast<const IdxT*>(p.indices) + bag.start, p.pw ? p.pw + bag.start : nullptr,
                            p.error_flag, bag.table, bag.stride, bag.L, bag.D, bag.seg, bag.mean_mul, ty, p.out_ty,
                            p.fp8_shift, p.fp8_mult, lane);
}

// Pooling NONE: one warp per position n of `indices`; row n of the output gets the
// dequantised row, zero-filled from D_t up to max_D.  Table of position n: the t with offsets[t*B] <= n < offsets[(t+1)*B].
template <typename IdxT>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
tbe_nobag_kernel(const LookupParams p, int64_t num_indices, int max_D)
{
    const int lane = threadIdx.x & 31;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (n >= num_indices) return;
    const IdxT* offsets = static_cast<const IdxT*>(p.offsets);
    // Binary search over the T+1 table boundaries offsets[t*B].
    int lo = 0, hi = p.T;   // invariant: boundary(lo) <= n < boundary(hi)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(offsets[static_cast<int64_t>(mid) * p.B]) <= n) lo = mid;
        else hi = mid;
    }
    const int t = lo;
    const int ty = p.weights_tys[t];
    const int D = p.D_offsets[t + 1] - p.D_offsets[t];
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    void* seg = static_cast<char*>(p.output) + n * p.out_stride * esz;
    const int64_t idx = static_cast<int64_t>(static_cast<const IdxT*>(p.indices)[n]);
    if (idx < 0) {
        if (idx < -1 && lane == 0 && p.error_flag) atomicOr(p.error_flag, 1);
        for (int e = lane; e < max(D, max_D); e += kWarp) store_scalar(seg, e, 0.0f, p.out_ty);
        return;
    }
    const int64_t stride = row_bytes_of(ty, D, p.row_alignment);
    const uint8_t* row = p.dev_weights + p.weights_offsets[t] + idx * stride;
    float scale, bias;
    read_header(row, ty, scale, bias);
    for (int e = lane; e < D; e += kWarp)
        store_scalar(seg, e, decode_elem(row, ty, e, scale, bias, p.fp8_shift, p.fp8_mult), p.out_ty);
    for (int e = D + lane; e < max_D; e += kWarp) store_scalar(seg, e, 0.0f, p.out_ty);
}

}  // namespace

}  // namespace tbe

extern "C" int tbe_b200_int_nbit_lookup(const tbe_b200_lookup_args* a, tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (!a) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: args is NULL");
    if (a->T <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: T must be positive, got %d", a->T);
    if (a->B < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: B must be non-negative");
    if (a->index_bits != 32 && a->index_bits != 64)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: index_bits must be 32 or 64, got %d", a->index_bits);
    if (a->pooling_mode < TBE_B200_POOL_SUM || a->pooling_mode > TBE_B200_POOL_NONE)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: pooling_mode must be 0 (SUM), 1 (MEAN) or 2 (NONE), got %d",
                    a->pooling_mode);
    if (a->output_dtype != TBE_B200_FP32 && a->output_dtype != TBE_B200_FP16 && a->output_dtype != TBE_B200_BF16)
        return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: output_dtype %d is not supported (0 FP32, 1 FP16, 5 BF16)",
                    a->output_dtype);
    if (!a->dev_weights || !a->weights_offsets || !a->weights_tys || !a->D_offsets || !a->offsets || !a->output)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: a required pointer is NULL");
    if (a->num_indices > 0 && !a->indices) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: indices is NULL");
    if (a->row_alignment < 1) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: row_alignment must be >= 1");
    if (a->dest_outputs && a->rows_per_dest <= 0)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "lookup: rows_per_dest must be positive with dest_outputs");

    LookupParams p;
    p.dev_weights = a->dev_weights;
    p.weights_offsets = a->weights_offsets;
    p.weights_tys = a->weights_tys;
    p.D_offsets = a->D_offsets;
    p.indices = a->indices;
    p.offsets = a->offsets;
    p.pw = a->indice_weights;
    p.output = a->output;
    p.out_cols = a->output_col_offsets;
    p.dests = a->dest_outputs;
    p.error_flag = a->error_flag;
    p.B = a->B;
    p.num_bags = static_cast<int64_t>(a->T) * a->B;
    p.out_stride = a->output_stride;
    p.rows_per_dest = a->rows_per_dest;
    p.T = a->T;
    p.B32 = (p.num_bags < (1ll << 32) && a->B > 0) ? static_cast<uint32_t>(a->B) : 0u;
    p.pooling_mode = a->pooling_mode;
    p.out_ty = a->output_dtype;
    p.row_alignment = a->row_alignment;
    const int ebits = a->fp8_exponent_bits > 0 ? a->fp8_exponent_bits : 4;
    const int ebias = a->fp8_exponent_bias >= 0 ? a->fp8_exponent_bias : 7;
    p.fp8_shift = static_cast<uint32_t>(16 + ebits);
    const uint32_t mult_bits = static_cast<uint32_t>(254 - ebias) << 23;
    memcpy(&p.fp8_mult, &mult_bits, 4);

    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (a->pooling_mode == TBE_B200_POOL_NONE) {
        if (a->num_indices <= 0) return TBE_B200_OK;
        const int64_t blocks = (a->num_indices + kWarpsPerBlock - 1) / kWarpsPerBlock;
        if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: too many indices for one launch");
        if (a->index_bits == 32)
            tbe_nobag_kernel<int32_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p, a->num_indices, a->max_D);
        else
            tbe_nobag_kernel<int64_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p, a->num_indices, a->max_D);
        return check_launch("tbe_nobag_kernel");
    }
    if (p.num_bags == 0) return TBE_B200_OK;
    const int64_t blocks = (p.num_bags + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: T*B too large for one launch");
    if (a->index_bits == 32)
        tbe_pooled_kernel<int32_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p);
    else
        tbe_pooled_kernel<int64_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p);
    return check_launch("tbe_pooled_kernel");
}
