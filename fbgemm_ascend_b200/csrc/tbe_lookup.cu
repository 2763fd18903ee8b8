// Quantized table-batched-embedding lookup for B200 (sm_100a).
//
// Replaces the device side of int_nbit_split_embedding_codegen_lookup_function
// (reference: c310/op_kernel/int_nbit_split_embedding_pooling_kernel.h:44-394 and
// int_nbit_split_embedding_nobag_kernel.h:31-398).  The path is a gather and a
// reduction bounded by HBM/L2 bandwidth, so there is no tensor-core work here.
//
// Pooled kernel (SUM / MEAN), in three tiers chosen per table:
//   * aligned rows of INT8 / INT4 / FP8 / FP16 / FP32 with D a multiple of 16 up to 512 (pool_run_staged): LPR lanes
//     share a row, 16 fp32 accumulators per lane, so a warp has 32/LPR lane groups; the groups pool that many
//     consecutive bags side by side (or split one long bag and reduce-scatter at the end).  Rows reach shared
//     memory by one bulk asynchronous copy each (cp.async.bulk, completion on an mbarrier), up to 32 per warp in
//     flight; they are dequantised with the row's fp16 scale/bias (codes -> exact fp16 by a magic constant, then
//     fp16 x fp16 + fp32 mixed FMA) and accumulated in fp32.  INT8/INT4 rows start with a 4-byte header, which
//     shifts the payload off the 16-byte grid; the lane that reads the header chunk has 4 / 8 free slots, which
//     take the row's last elements, so D = 16*LPR rows keep every lane busy with exactly 16 elements;
//   * other aligned shapes (pool_bag): one warp per bag, cp.async staging in chunks, cross-group reduce-scatter;
//   * anything else (row_alignment 1, odd D, INT2 or BF16 rows, unaligned tables): a byte-wise path.
// Sequence mode (pooling NONE): tbe_nobag_kernel, 64 consecutive positions per warp.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

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
    int64_t num_indices;
    int64_t out_stride;
    int64_t rows_per_dest;
    int64_t span;        // bags per warp
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
// Every lane owns 16 accumulator "slots".  A path says which bytes a lane fetches
// for a row (issue), how the fetched bytes add into the slots (accum), and which
// element of the row a slot stands for (elem).  `unit` is the lane's position
// among the 16-slot units of the row: unit = block * LPR + k.
//
// Rows are fetched with cp.async straight into shared memory, never through
// registers: each lane has private staging slots (one per pass of a chunk, two
// chunks deep), so the rows of two chunks are in flight per warp while the
// accumulators and addresses are all the registers a lane needs.  A lane reads
// back only what it fetched itself, so no warp barrier is involved.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16-byte asynchronous copy global -> shared, L2 only; `bytes` = 16, or 0 to write zeros without reading.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint4 lds16(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds8(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds4(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

// ---- dequantisation arithmetic ------------------------------------------------
//
// Integer -> float conversion instructions run at 16 lanes per clock per SM on sm_100a, which
// would cap a 128-element INT8 row at 8 cycles.  Codes are therefore turned into exact fp16 values
// with one byte permute (or mask) and one half2 subtract per pair -- 0x6400 | q is the half 1024 + q
// -- and accumulated with the sm_100 mixed-precision FMA (fp16 * fp16 + fp32 -> fp32): the row scale
// is stored as fp16, so code * scale is formed exactly and added to the fp32 accumulator with a
// single rounding, as an fp32 FMA would.  With per-sample weights the scale is no longer an fp16
// value; the codes are then widened to fp32 and an fp32 FMA with w * scale is used.

// d = a(fp16) * b(fp16) + d(fp32), one rounding.  a, b: fp16 bit patterns in the low 16 bits.
__device__ __forceinline__ void mixed_fma(float& d, uint32_t a, uint32_t b)
{
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(d) : "h"(static_cast<unsigned short>(a)), "h"(static_cast<unsigned short>(b)));
}

// Two exact fp16 values (as a half2 bit pattern) from two codes already or'ed into the mantissas of
// the half2 `magic` (0x6400: 1024, 0x5400: 64 with the code in mantissa bits 4..7).
__device__ __forceinline__ uint32_t codes_to_half2(uint32_t packed, uint32_t magic)
{
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&packed), *reinterpret_cast<const __half2*>(&magic));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// acc[0..1] += pair (half2 bits) * scale: mixed FMA with the fp16 scale, or fp32 FMA with `ws`.
__device__ __forceinline__ void add_pair(float& a0, float& a1, uint32_t pair, uint32_t scale_h, float ws, bool weighted)
{
    if (!weighted) {
        mixed_fma(a0, pair & 0xffffu, scale_h);
        mixed_fma(a1, pair >> 16, scale_h);
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pair));
        a0 = fmaf(f.x, ws, a0);
        a1 = fmaf(f.y, ws, a1);
    }
}

// The same with the choice made at compile time and the two halves split inside one asm block.
template <bool WEIGHTED>
__device__ __forceinline__ void add_pair_t(float& a0, float& a1, uint32_t pair, unsigned short scale_h, float ws)
{
    if constexpr (!WEIGHTED) {
        asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; fma.rn.f32.f16 %0, l, %3, %0; fma.rn.f32.f16 %1, h, %3, %1; }"
            : "+f"(a0), "+f"(a1)
            : "r"(pair), "h"(scale_h));
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pair));
        a0 = fmaf(f.x, ws, a0);
        a1 = fmaf(f.y, ws, a1);
    }
}

// Staging memory of one warp: two chunk buffers of kChunkBytes (a lane's slot for pass u is at
// (u*32 + lane) * slot_bytes) and, for header types, one 4-byte side slot per (buffer, pass, lane).
constexpr int kChunkBytes = 2048;
constexpr int kMaxPasses = 8;
constexpr int kSideBytes = 2 * kMaxPasses * kWarp * 4;
constexpr int kWarpSmemBytes = 2 * kChunkBytes + kSideBytes;

struct LaneCtx {
    int unit;        // 16-slot unit handled by this lane in the current block
    int D;           // elements per row
    int k;           // lane index within its row group
    bool active;     // this unit exists in the row
    bool wrap;       // INT8/INT4 header lane that also takes the row's tail
    bool first_blk;  // block 0: the header is the first word of unit 0
    bool weighted;   // per-sample weights are in use
    uint32_t fp8_shift;
    float fp8_mult;
};

template <int TY>
struct Path;

template <>
struct Path<TBE_B200_INT8> {
    static constexpr bool kHasHeader = true;
    static constexpr int kSlotBytes = 16;
    static constexpr int kPasses = 4;   // passes per chunk (x 32 lanes x 16 B = 2 KB)
    // 16-byte chunks of the row: chunk c covers elements [16c - 4, 16c + 12).
    static __device__ __forceinline__ int units(int D, bool wrap) { return wrap ? D / 16 : (D + 4 + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int D) { return (D & 15) == 0; }
    // The side slot of the header lane gets the row's tail (elements D-4 .. D-1) when the row
    // wraps, and the header itself in the later blocks of a wide row.
    template <int LPR>
    static __device__ __forceinline__ void issue(uint32_t slot, uint32_t side, const uint8_t* row, const uint8_t* safe,
                                                 const LaneCtx& cx, bool ok)
    {
        if (cx.active) cp_async16(slot, ok ? row + cx.unit * 16 : safe, ok ? 16 : 0);
        if (cx.k == 0 && (cx.wrap || !cx.first_blk)) cp_async4(side, ok ? row + (cx.wrap ? cx.D : 0) : safe, ok ? 4 : 0);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(uint32_t slot, uint32_t side, const LaneCtx& cx, float w, float (&acc)[16],
                                                 float& bias_acc)
    {
        uint4 v = cx.active ? lds16(slot) : make_uint4(0u, 0u, 0u, 0u);
        uint32_t hdr = v.x;
        if (cx.k == 0 && (cx.wrap || !cx.first_blk)) {
            const uint32_t s = lds4(side);
            if (cx.wrap) v.x = s; else hdr = s;
        }
        hdr = __shfl_sync(kFull, hdr, 0, LPR);
        // A row that must not be added has zero-filled data and header, so its scale and bias are 0.
        const uint32_t scale_h = hdr & 0xffffu;
        const float ws = half_bits_to_float(scale_h) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), cx.weighted ? w : 1.0f, bias_acc);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // bytes (q0, 0x64, q1, 0x64) = half2(1024 + q0, 1024 + q1)
            const uint32_t lo = codes_to_half2(__byte_perm(words[i], 0x64646464u, 0x4140), 0x64006400u);
            const uint32_t hi = codes_to_half2(__byte_perm(words[i], 0x64646464u, 0x4342), 0x64006400u);
            add_pair(acc[4 * i + 0], acc[4 * i + 1], lo, scale_h, ws, cx.weighted);
            add_pair(acc[4 * i + 2], acc[4 * i + 3], hi, scale_h, ws, cx.weighted);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot)
    {
        if (cx.wrap && slot < 4) return cx.D - 4 + slot;
        return 16 * cx.unit - 4 + slot;
    }
};

template <>
struct Path<TBE_B200_INT4> {
    static constexpr bool kHasHeader = true;
    static constexpr int kSlotBytes = 8;
    static constexpr int kPasses = 8;   // x 32 lanes x 8 B = 2 KB
    // 8-byte chunks: chunk c covers elements [16c - 8, 16c + 8).
    static __device__ __forceinline__ int units(int D, bool wrap) { return wrap ? D / 16 : (D / 2 + 4 + 7) / 8; }
    static __device__ __forceinline__ bool can_wrap(int D) { return (D & 15) == 0; }
    template <int LPR>
    static __device__ __forceinline__ void issue(uint32_t slot, uint32_t side, const uint8_t* row, const uint8_t* safe,
                                                 const LaneCtx& cx, bool ok)
    {
        if (cx.active) cp_async8(slot, ok ? row + cx.unit * 8 : safe, ok ? 8 : 0);
        if (cx.k == 0 && (cx.wrap || !cx.first_blk)) cp_async4(side, ok ? row + (cx.wrap ? cx.D / 2 : 0) : safe, ok ? 4 : 0);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(uint32_t slot, uint32_t side, const LaneCtx& cx, float w, float (&acc)[16],
                                                 float& bias_acc)
    {
        uint2 v = cx.active ? lds8(slot) : make_uint2(0u, 0u);
        uint32_t hdr = v.x;
        if (cx.k == 0 && (cx.wrap || !cx.first_blk)) {
            const uint32_t s = lds4(side);
            if (cx.wrap) v.x = s; else hdr = s;
        }
        hdr = __shfl_sync(kFull, hdr, 0, LPR);
        const uint32_t scale_h = hdr & 0xffffu;
        const float ws = half_bits_to_float(scale_h) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), cx.weighted ? w : 1.0f, bias_acc);
        const uint32_t words[2] = {v.x, v.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            // nibble pairs (j, j + 4) sit 16 bits apart: mask them into two half mantissas at once.
            // 0x6400 | n = 1024 + n; 0x5400 | (n << 4) = 64 + n.
            const uint32_t x = words[i], y = words[i] >> 8;
            const uint32_t p0 = codes_to_half2((x & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 0, 4
            const uint32_t p1 = codes_to_half2((x & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 1, 5
            const uint32_t p2 = codes_to_half2((y & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 2, 6
            const uint32_t p3 = codes_to_half2((y & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 3, 7
            add_pair(acc[8 * i + 0], acc[8 * i + 4], p0, scale_h, ws, cx.weighted);
            add_pair(acc[8 * i + 1], acc[8 * i + 5], p1, scale_h, ws, cx.weighted);
            add_pair(acc[8 * i + 2], acc[8 * i + 6], p2, scale_h, ws, cx.weighted);
            add_pair(acc[8 * i + 3], acc[8 * i + 7], p3, scale_h, ws, cx.weighted);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot)
    {
        if (cx.wrap && slot < 8) return cx.D - 8 + slot;
        return 16 * cx.unit - 8 + slot;
    }
};

template <>
struct Path<TBE_B200_FP8> {
    static constexpr bool kHasHeader = false;
    static constexpr int kSlotBytes = 16;
    static constexpr int kPasses = 4;
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    template <int LPR>
    static __device__ __forceinline__ void issue(uint32_t slot, uint32_t, const uint8_t* row, const uint8_t* safe,
                                                 const LaneCtx& cx, bool ok)
    {
        if (cx.active) cp_async16(slot, ok ? row + cx.unit * 16 : safe, ok ? 16 : 0);
    }
    // Byte -> fp32 by bit placement: ((b & 0x7f) << (16 + ebits)) as a float, times
    // 2^(127 - bias), sign bit or'ed in (reference: c310/op_kernel/common.h:120-167).
    template <int LPR>
    static __device__ __forceinline__ void accum(uint32_t slot, uint32_t, const LaneCtx& cx, float w, float (&acc)[16], float&)
    {
        const uint4 v = cx.active ? lds16(slot) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
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
    template <int LPR>
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot) { return 16 * cx.unit + slot; }
};

template <>
struct Path<TBE_B200_FP16> {
    static constexpr bool kHasHeader = false;
    static constexpr int kSlotBytes = 32;
    static constexpr int kPasses = 2;
    // A unit is two 16-byte chunks LPR chunks apart, so that one copy instruction of a group covers
    // LPR*16 contiguous bytes: with blk = unit / LPR and k = unit % LPR, chunk_a = 2*blk*LPR + k,
    // chunk_b = chunk_a + LPR; a chunk is 8 elements.  Bounds are checked per chunk.
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    template <int LPR>
    static __device__ __forceinline__ int chunk_a(int unit) { return 2 * (unit / LPR) * LPR + (unit % LPR); }
    template <int LPR>
    static __device__ __forceinline__ void issue(uint32_t slot, uint32_t, const uint8_t* row, const uint8_t* safe,
                                                 const LaneCtx& cx, bool ok)
    {
        const int ca = chunk_a<LPR>(cx.unit);
        if (ca * 8 < cx.D) cp_async16(slot, ok ? row + ca * 16 : safe, ok ? 16 : 0);
        if ((ca + LPR) * 8 < cx.D) cp_async16(slot + 16, ok ? row + (ca + LPR) * 16 : safe, ok ? 16 : 0);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(uint32_t slot, uint32_t, const LaneCtx& cx, float w, float (&acc)[16], float&)
    {
        const int ca = chunk_a<LPR>(cx.unit);
        const uint4 a = (ca * 8 < cx.D) ? lds16(slot) : make_uint4(0u, 0u, 0u, 0u);
        const uint4 b = ((ca + LPR) * 8 < cx.D) ? lds16(slot + 16) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        // unweighted: value * 1.0 + acc in one mixed FMA (rows not to be added are zero-filled)
#pragma unroll
        for (int i = 0; i < 8; ++i) add_pair(acc[2 * i], acc[2 * i + 1], words[i], 0x3c00u, w, cx.weighted);
    }
    template <int LPR>
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot)
    {
        const int ca = chunk_a<LPR>(cx.unit);
        return slot < 8 ? 8 * ca + slot : 8 * (ca + LPR) + slot - 8;
    }
};

template <>
struct Path<TBE_B200_FP32> {
    static constexpr bool kHasHeader = false;
    static constexpr int kSlotBytes = 64;
    static constexpr int kPasses = 1;
    // A unit is four 16-byte chunks, LPR chunks apart: chunk_m = 4*blk*LPR + m*LPR + k.
    static __device__ __forceinline__ int units(int D, bool) { return (D + 15) / 16; }
    static __device__ __forceinline__ bool can_wrap(int) { return false; }
    template <int LPR>
    static __device__ __forceinline__ int chunk0(int unit) { return 4 * (unit / LPR) * LPR + (unit % LPR); }
    template <int LPR>
    static __device__ __forceinline__ void issue(uint32_t slot, uint32_t, const uint8_t* row, const uint8_t* safe,
                                                 const LaneCtx& cx, bool ok)
    {
        const int c0 = chunk0<LPR>(cx.unit);
#pragma unroll
        for (int m = 0; m < 4; ++m)
            if ((c0 + m * LPR) * 4 < cx.D) cp_async16(slot + 16 * m, ok ? row + (c0 + m * LPR) * 16 : safe, ok ? 16 : 0);
    }
    template <int LPR>
    static __device__ __forceinline__ void accum(uint32_t slot, uint32_t, const LaneCtx& cx, float w, float (&acc)[16], float&)
    {
        const int c0 = chunk0<LPR>(cx.unit);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const uint4 v = ((c0 + m * LPR) * 4 < cx.D) ? lds16(slot + 16 * m) : make_uint4(0u, 0u, 0u, 0u);
            acc[4 * m + 0] = fmaf(w, __uint_as_float(v.x), acc[4 * m + 0]);
            acc[4 * m + 1] = fmaf(w, __uint_as_float(v.y), acc[4 * m + 1]);
            acc[4 * m + 2] = fmaf(w, __uint_as_float(v.z), acc[4 * m + 2]);
            acc[4 * m + 3] = fmaf(w, __uint_as_float(v.w), acc[4 * m + 3]);
        }
    }
    template <int LPR>
    static __device__ __forceinline__ int elem(const LaneCtx& cx, int slot)
    {
        return 4 * (chunk0<LPR>(cx.unit) + (slot >> 2) * LPR) + (slot & 3);
    }
};

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

// Up to 32 consecutive indices and weights of a bag, one per lane.  Indices are narrowed to 32 bits:
// a row number outside [-1, 2^31) is reported through the error flag and treated as -1 (skipped).
struct BagHead {
    int32_t idx;   // -1 beyond the bag
    float w;
};

template <typename IdxT>
__device__ __forceinline__ BagHead load_batch(const IdxT* indices, const float* pw, int n, int lane, int32_t* error_flag)
{
    BagHead h;
    h.idx = -1;
    h.w = 1.0f;
    if (lane < n) {
        const IdxT v = __ldg(indices + lane);
        const bool bad = (v < static_cast<IdxT>(-1)) || (sizeof(IdxT) == 8 && static_cast<int64_t>(v) > 0x7fffffffll);
        h.idx = bad ? -1 : static_cast<int32_t>(v);
        if (bad && error_flag) atomicOr(error_flag, 1);
        if (pw) h.w = __ldg(pw + lane);
    }
    return h;
}

// Pools one bag whose rows are 16-byte aligned with a 16-byte-multiple stride.
// `head` holds the bag's first 32 indices/weights; `wsm` is the warp's staging memory.
template <int TY, int LPR, typename IdxT>
__device__ __forceinline__ void pool_bag(const LookupParams& p, const BagInfo& bag, const BagHead& head, int lane,
                                         uint32_t wsm)
{
    using P = Path<TY>;
    constexpr int RPI = kWarp / LPR;                                   // rows per pass of the warp
    constexpr int UC = (P::kPasses < kWarp / RPI) ? P::kPasses : (kWarp / RPI);   // passes per chunk
    constexpr int RC = UC * RPI;                                       // rows per chunk (divides 32)
    constexpr int NF = 16 / RPI;                                       // finished slots per lane after the reduce-scatter
    static_assert(UC * kWarp * P::kSlotBytes <= kChunkBytes && UC <= kMaxPasses, "chunk does not fit its buffer");
    const int k = lane % LPR;
    const int g = lane / LPR;
    const IdxT* indices = static_cast<const IdxT*>(p.indices) + bag.start;
    const float* pw = p.pw ? p.pw + bag.start : nullptr;
    const bool wrap_row = P::can_wrap(bag.D);
    const int nunits = P::units(bag.D, wrap_row);
    const int nchunks = (bag.L + RC - 1) / RC;
    const uint32_t slot0 = wsm + lane * P::kSlotBytes;
    const uint32_t side0 = wsm + 2 * kChunkBytes + g * 4;

    for (int ublk = 0; ublk < nunits; ublk += LPR) {
        LaneCtx cx;
        cx.unit = ublk + k;
        cx.D = bag.D;
        cx.k = k;
        // FP16/FP32 units interleave their chunks, so those paths bound-check per chunk instead.
        cx.active = (TY == TBE_B200_FP16 || TY == TBE_B200_FP32) ? true : (cx.unit < nunits);
        cx.first_blk = (ublk == 0);
        cx.wrap = wrap_row && cx.unit == 0;
        cx.weighted = p.pw != nullptr;
        cx.fp8_shift = p.fp8_shift;
        cx.fp8_mult = p.fp8_mult;

        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
        float bias_acc = 0.0f;

        // The 32 indices the lanes currently hold cover rows [batch0, batch0 + 32) of the bag.
        int batch0 = 0;
        int32_t my_idx = head.idx;
        float my_w = head.w;
        float w_buf0 = 0.0f, w_buf1 = 0.0f;   // per staging buffer: weight of row (chunk start + lane), 0 if not to be added

        auto issue_chunk = [&](int c) {
            const int row0 = c * RC;
            if (row0 >= batch0 + kWarp) {
                batch0 += kWarp;
                const BagHead nb = load_batch<IdxT>(indices + batch0, pw ? pw + batch0 : nullptr, bag.L - batch0, lane,
                                                    cx.first_blk ? p.error_flag : nullptr);
                my_idx = nb.idx;
                my_w = nb.w;
            }
            const uint32_t slot = slot0 + (c & 1) * kChunkBytes;
            const uint32_t side = side0 + (c & 1) * (kMaxPasses * 16 * 4);
            const int rel0 = row0 - batch0;   // position of the chunk's first row among the 32 held indices
#pragma unroll 1
            for (int u = 0; u < UC; ++u) {
                const int r = rel0 + u * RPI + g;
                const int32_t idx = __shfl_sync(kFull, my_idx, r & 31);
                const bool ok = (row0 + u * RPI + g < bag.L) && (idx >= 0);
                P::template issue<LPR>(slot + u * kWarp * P::kSlotBytes, side + u * 16 * 4,
                                       bag.table + static_cast<int64_t>(idx) * bag.stride, bag.table, cx, ok);
            }
            cp_async_commit();
            if (cx.weighted) {
                // weight of row (row0 + lane) for the lanes that stand for a row of this chunk
                const int32_t li = __shfl_sync(kFull, my_idx, (rel0 + lane) & 31);
                float lw = __shfl_sync(kFull, my_w, (rel0 + lane) & 31);
                if (lane >= RC || row0 + lane >= bag.L || li < 0) lw = 0.0f;
                if (c & 1) w_buf1 = lw; else w_buf0 = lw;
            }
        };

        if (nchunks > 0) issue_chunk(0);
        if (nchunks > 1) issue_chunk(1);
        for (int c = 0; c < nchunks; ++c) {
            if (c + 1 < nchunks) cp_async_wait<1>(); else cp_async_wait<0>();
            const uint32_t slot = slot0 + (c & 1) * kChunkBytes;
            const uint32_t side = side0 + (c & 1) * (kMaxPasses * 16 * 4);
            const float wb = (c & 1) ? w_buf1 : w_buf0;
#pragma unroll 1
            for (int u = 0; u < UC; ++u) {
                // Unweighted: rows that are not to be added are zero-filled, so every row can use weight 1.
                const float w = cx.weighted ? __shfl_sync(kFull, wb, u * RPI + g) : 1.0f;
                P::template accum<LPR>(slot + u * kWarp * P::kSlotBytes, side + u * 16 * 4, cx, w, acc, bias_acc);
            }
            if (c + 2 < nchunks) issue_chunk(c + 2);
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
                const int e0 = P::template elem<LPR>(cx, slot);
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
__device__ __forceinline__ void pool_bag_by_width(const LookupParams& p, const BagInfo& bag, const BagHead& head, int lane,
                                                  uint32_t wsm)
{
    const bool wrap = Path<TY>::can_wrap(bag.D);
    const int nunits = Path<TY>::units(bag.D, wrap);
    if (nunits <= 2) pool_bag<TY, 2, IdxT>(p, bag, head, lane, wsm);
    else if (nunits <= 4) pool_bag<TY, 4, IdxT>(p, bag, head, lane, wsm);
    else if (nunits <= 8) pool_bag<TY, 8, IdxT>(p, bag, head, lane, wsm);
    else if (nunits <= 16) pool_bag<TY, 16, IdxT>(p, bag, head, lane, wsm);
    else pool_bag<TY, 32, IdxT>(p, bag, head, lane, wsm);
}

// Description of the table a bag belongs to; reloaded only when the warp moves on to another table.
struct TableMeta {
    const uint8_t* table;   // first row
    int64_t stride;         // bytes per row
    int64_t col;            // output column of the table
    int32_t ty;
    int32_t D;
    bool rows_aligned;      // table start and row stride are multiples of 16 bytes
};

__device__ __forceinline__ TableMeta load_meta(const LookupParams& p, int t)
{
    TableMeta m;
    m.ty = p.weights_tys[t];
    const int d0 = p.D_offsets[t];
    m.D = p.D_offsets[t + 1] - d0;
    m.table = p.dev_weights + p.weights_offsets[t];
    m.col = p.out_cols ? p.out_cols[t] : static_cast<int64_t>(d0);
    m.stride = row_bytes_of(m.ty, m.D, p.row_alignment);
    m.rows_aligned = ((reinterpret_cast<uintptr_t>(m.table) | static_cast<uint64_t>(m.stride)) & 15) == 0;
    return m;
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

// ---- the common shapes: rows staged in shared memory by bulk copies, groups of lanes --------
//
// One bulk asynchronous copy (cp.async.bulk, executed by the copy engine of the SM) moves a whole row
// from global to shared memory; its completion is counted on an mbarrier.  Every lane of a warp issues
// the copy of a different row, so up to 32 rows per warp are in flight with one instruction and no
// register holds data that is still on its way.  Source, destination and size are multiples of 16
// bytes by construction (aligned tables, padded row stride).

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// Orders this thread's earlier shared-memory accesses before its later asynchronous copies.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Waits for the phase with the given parity.  The wait is bounded: false after kWaitTries polls.
constexpr int kWaitTries = 1 << 22;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (int t = 0; t < kWaitTries; ++t) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (done) return true;
    }
    return false;
}

// Adds one INT8 / INT4 row chunk to a lane's 16 slots.  `w0` is the lane's first payload word (the row's tail
// on the header lane), words[1..] the rest of its chunk, `hdr` the row header (fp16 scale, fp16 bias; zero
// for a row that is not to be added).
template <int TY, bool WEIGHTED, bool FOLD>
__device__ __forceinline__ void accum_header_row(uint32_t w0, const uint32_t (&words)[4], uint32_t hdr, float w, float (&acc)[16],
                                                 float& bias_acc, float& scale_acc)
{
    constexpr bool k8 = (TY == TBE_B200_INT8);
    const unsigned short scale_h = static_cast<unsigned short>(hdr & 0xffffu);
    float ws = 0.0f;
    if constexpr (WEIGHTED) {
        ws = half_bits_to_float(scale_h) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), w, bias_acc);
    } else {
        bias_acc += half_bits_to_float(hdr >> 16);
        if constexpr (FOLD) scale_acc += half_bits_to_float(scale_h);
    }
    if (k8) {
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const uint32_t c = (i4 == 0) ? w0 : words[i4];
            // bytes 0 and 2, then bytes 1 and 3, placed in the mantissas of half2(1024, 1024)
            uint32_t even = (c & 0x00FF00FFu) | 0x64006400u;
            uint32_t odd = __byte_perm(c, 0x64646464u, 0x4341);
            if constexpr (!FOLD) {
                even = codes_to_half2(even, 0x64006400u);
                odd = codes_to_half2(odd, 0x64006400u);
            }
            add_pair_t<WEIGHTED>(acc[4 * i4 + 0], acc[4 * i4 + 2], even, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[4 * i4 + 1], acc[4 * i4 + 3], odd, scale_h, ws);
        }
    } else {
#pragma unroll
        for (int i2 = 0; i2 < 2; ++i2) {
            const uint32_t c = (i2 == 0) ? w0 : words[i2];
            const uint32_t y = c >> 8;
            // nibble pairs (j, j + 4) sit 16 bits apart: 0x6400 | n = 1024 + n; 0x5400 | (n << 4) = 64 + n
            const uint32_t p0 = codes_to_half2((c & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 0, 4
            const uint32_t p1 = codes_to_half2((c & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 1, 5
            const uint32_t p2 = codes_to_half2((y & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 2, 6
            const uint32_t p3 = codes_to_half2((y & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 3, 7
            add_pair_t<WEIGHTED>(acc[8 * i2 + 0], acc[8 * i2 + 4], p0, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i2 + 1], acc[8 * i2 + 5], p1, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i2 + 2], acc[8 * i2 + 6], p2, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i2 + 3], acc[8 * i2 + 7], p3, scale_h, ws);
        }
    }
}

// Output address of element 0 of bag `b` of the table at column `col`, when the result is scattered
// over per-destination buffers (bag b belongs to destination b / rows_per_dest).
__device__ __forceinline__ char* dest_segment(const LookupParams& p, int64_t b, int64_t col, int esz)
{
    int64_t which, rem;
    if (p.B32) {
        const uint32_t w = static_cast<uint32_t>(b) / static_cast<uint32_t>(p.rows_per_dest);
        which = w;
        rem = static_cast<uint32_t>(b) - w * static_cast<uint32_t>(p.rows_per_dest);
    } else {
        which = b / p.rows_per_dest;
        rem = b - which * p.rows_per_dest;
    }
    return static_cast<char*>(p.dests[which]) + (rem * p.out_stride + col) * esz;
}

constexpr int kStageBytes = kWarpSmemBytes;   // row slots of one warp

// A run of consecutive bags of ONE table whose rows are D = 16 * n <= 512 elements, 16-byte aligned.
// LPR lanes share a row, 16 elements per lane, so a warp has G = 32 / LPR lane groups, and every group
// walks its OWN range of the index array:
//   * normally the groups pool G consecutive bags side by side.  Nothing is exchanged between lanes when
//     a bag is finished -- a lane simply stores its 16 elements -- and all the per-bag work (offsets,
//     lengths, addresses, conversion, stores) is done for G bags by one instruction stream;
//   * when the G bags differ too much in length (or fewer than G are left), the warp takes a single bag
//     and splits its rows over the groups instead; the groups' partial sums are then combined with a
//     reduce-scatter over shuffles.  Both forms share the row loop.
// The row loop works in rounds of R rows per group (R * G <= 32 rows, as many as the warp's staging
// memory holds).  Lane k < R of a group reads the index of the group's k-th row of the round and issues
// that row's bulk copy into slot k*G + g (a lane whose row is not to be added -- index -1, or past the
// group's range -- clears the slot's header, or the whole slot for a type without header, instead).
// When the round's rows have landed the group reads them back, one per pass: 16 (INT4: 8) bytes per
// lane, the header word by broadcast, and for INT8/INT4 the row's last 4 / 8 elements, which the lane
// that owns the header chunk takes into the slots the header leaves free.  Interleaving the slots by
// group keeps the G header words of a pass in different banks.  The indices of a round are requested
// one round ahead, so only the first index load of a step is exposed.  (Two rounds of rows in flight per
// warp, half the rows each, measured slower: the kernel is bound by instruction issue, and shorter
// rounds mean more per-round work.)
// FOLD (INT8, unweighted, 16-bit output): the subtraction of the magic constant that turns a code into
// an fp16 value is skipped, (1024 + q) * scale is accumulated, and 1024 * sum(scale) is removed again at
// least every 32 rows, which keeps the partial sums small enough for the extra term not to cost
// precision that a 16-bit result could show.
// Returns false when a wait for staged rows ran out (reported through the error flag, bit 1).
template <int TY, int LPR, typename IdxT, bool WEIGHTED, bool FOLD>
__device__ __noinline__ bool pool_run_staged(const LookupParams& p, const TableMeta& m, int64_t i0, int64_t i1, int64_t b0,
                                             int lane, uint32_t wsm, uint32_t bar, uint32_t& parity)
{
    static_assert(!FOLD || (TY == TBE_B200_INT8 && !WEIGHTED), "the folded form is for unweighted INT8 pooling");
    constexpr bool kHdr = (TY == TBE_B200_INT8 || TY == TBE_B200_INT4);
    constexpr bool k8 = (TY == TBE_B200_INT8);
    constexpr int CH = (TY == TBE_B200_INT4) ? 8 : 16;                 // bytes per chunk read by a lane
    constexpr int NCH = (TY == TBE_B200_FP16) ? 2 : (TY == TBE_B200_FP32) ? 4 : 1;   // chunks per lane and row
    constexpr int EPC = 16 / NCH;                      // elements per chunk
    constexpr int HS = k8 ? 4 : (TY == TBE_B200_INT4 ? 8 : 0);         // slots of the header lane that hold the row's tail
    constexpr int G = kWarp / LPR;                     // lane groups = rows per pass of the warp
    constexpr int LOG_G = G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3;
    constexpr int NF = 16 / G;                         // split form: finished slots per lane after the reduce-scatter
    constexpr int WS = NF >= 4 ? 4 : NF;               // split form: elements per store
    static_assert(G <= 8, "at least 4 lanes per row");
    const int k = lane % LPR;
    const int g = lane / LPR;
    const int D = m.D;
    const int nunits = D / 16;
    const bool head_lane = kHdr && (k == 0);
    const bool active = k < nunits;                    // lanes past the row's last unit have nothing to add (D < 16 * LPR)
    const uint32_t stride = static_cast<uint32_t>(m.stride);
    const uint32_t copy_bytes = static_cast<uint32_t>(row_bytes_of(TY, D, 16));   // the row without its alignment padding
    const int R = min(LPR, (kStageBytes / static_cast<int>(copy_bytes)) >> LOG_G);   // rows per group and round (>= 1)
    const uint32_t own_slot = wsm + static_cast<uint32_t>(k * G + g) * copy_bytes;   // the slot this lane fills (k < R)
    const uint32_t read0 = wsm + static_cast<uint32_t>(g) * copy_bytes + (active ? k * CH : 0);   // pass 0, chunk 0
    const uint32_t pass_pitch = G * copy_bytes;
    // INT8/INT4: the extra word of a pass is the row's tail for the header lane and the header for the others.
    const uint32_t extra0 = wsm + static_cast<uint32_t>(g) * copy_bytes + (head_lane ? (k8 ? D : D / 2) : 0);
    const IdxT* offs = static_cast<const IdxT*>(p.offsets) + i0;
    const IdxT* indices = static_cast<const IdxT*>(p.indices);
    const int nb = static_cast<int>(i1 - i0);
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    const int64_t row_bytes = p.out_stride * esz;
    const bool mean = p.pooling_mode == TBE_B200_POOL_MEAN;
    char* out_run = nullptr;               // output address of (bag b0, first column of this table)
    bool vec_ok = false;
    if (!p.dests) {
        out_run = static_cast<char*>(p.output) + m.col * esz + b0 * row_bytes;
        vec_ok = ((reinterpret_cast<uintptr_t>(out_run) | static_cast<uint64_t>(row_bytes)) & 15) == 0;
    }
    // Element a slot stands for.  Chunk c = k + (slot / EPC) * nunits of the row holds EPC elements; INT8/INT4
    // chunks are shifted by the header (unit k covers elements [16k - HS, 16k + 16 - HS)), and the header
    // lane's first HS slots are the row's last HS elements.
    auto elem_of = [&](int slot) -> int {
        if constexpr (kHdr) return (head_lane && slot < HS) ? (D - HS + slot) : (16 * k - HS + slot);
        else return EPC * (k + (slot / EPC) * nunits) + (slot % EPC);
    };
    // Split form: which of its 16 slots a lane ends up with.
    int slot_base = 0;
    if constexpr (G >= 2) slot_base += ((lane >> 4) & 1) ? 8 : 0;
    if constexpr (G >= 4) slot_base += ((lane >> 3) & 1) ? 4 : 0;
    if constexpr (G >= 8) slot_base += ((lane >> 2) & 1) ? 2 : 0;

    for (int j = 0; j < nb;) {
        // Group g looks at bag j + g (an empty one past the end of the run).
        const int64_t o0 = static_cast<int64_t>(__ldg(offs + min(j + g, nb)));
        const int64_t o1 = static_cast<int64_t>(__ldg(offs + min(j + g + 1, nb)));
        const int Lg = static_cast<int>(o1 - o0);
        int maxL = Lg, sumL = Lg;
#pragma unroll
        for (int d = LPR; d < kWarp; d <<= 1) {
            maxL = max(maxL, __shfl_xor_sync(kFull, maxL, d));
            sumL += __shfl_xor_sync(kFull, sumL, d);
        }
        // Side by side costs max(L) passes; one bag at a time costs about L / G + 4 passes per bag.
        const int bags_here = min(G, nb - j);
        const bool split = (G > 1) && (maxL + 2 > (sumL >> LOG_G) + 4 * bags_here);
        int64_t lo = o0;      // this group's rows are indices[lo .. lo + n)
        int n = Lg;
        int maxn = maxL;      // rows of the longest group
        int Lbag = Lg;        // length of the bag this lane contributes to
        if (split) {
            Lbag = __shfl_sync(kFull, Lg, 0);
            const int64_t start = __shfl_sync(kFull, o0, 0);
            const int per = (Lbag + G - 1) >> LOG_G;
            const int a = min(Lbag, g * per);
            lo = start + a;
            n = min(Lbag, a + per) - a;
            maxn = per;
        }
        const IdxT* ip = indices + lo + k;
        const float* wp = WEIGHTED ? p.pw + lo + k : nullptr;
        const int nrounds = (maxn + R - 1) / R;

        // Lane k < R of the group takes row r*R + k of round r.  The raw index is kept as loaded and only
        // looked at when the round is issued, one iteration later, so the load has that long to arrive.
        auto load_raw = [&](int r, IdxT& raw, float& w) {
            raw = static_cast<IdxT>(-1);
            w = 0.0f;
            if (k < R && r * R + k < n) {
                raw = __ldg(ip + r * R);
                if constexpr (WEIGHTED) w = __ldg(wp + r * R);
            }
        };
        // Index narrowed to 32 bits, -1 = nothing to add.
        auto narrow = [&](IdxT raw) -> int32_t {
            const bool bad = (raw < static_cast<IdxT>(-1)) || (sizeof(IdxT) == 8 && static_cast<int64_t>(raw) > 0x7fffffffll);
            if (bad) {
                if (p.error_flag) atomicOr(p.error_flag, 1);
                return -1;
            }
            return static_cast<int32_t>(raw);
        };
        // Starts a round: the copy of this lane's row into its slot, or a cleared slot.
        auto issue = [&](int32_t idx) {
            const uint32_t slot = own_slot;
            const uint32_t sbar = bar;
            // The reads of the previous round (by every lane) come before the writes of this round.
            __syncwarp();
            fence_async_smem();
            if (idx >= 0) {
                mbar_arrive_expect(sbar, copy_bytes);
                bulk_copy_row(slot, m.table + static_cast<uint64_t>(static_cast<uint32_t>(idx)) * stride, copy_bytes, sbar);
            } else {
                if (k < R) {
                    if constexpr (kHdr) {
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(slot), "r"(0u) : "memory");
                    } else {
                        for (uint32_t o = 0; o < copy_bytes; o += 16)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(slot + o), "r"(0u) : "memory");
                    }
                }
                mbar_arrive(sbar);
            }
        };

        float acc[16];
#pragma unroll
        for (int s = 0; s < 16; ++s) acc[s] = 0.0f;
        float bias_acc = 0.0f;
        float scale_acc = 0.0f;   // sum of the row scales since the last fold (FOLD only)
        int since_fold = 0;
        (void)scale_acc;
        (void)since_fold;

        IdxT raw_next;
        float w_cur = 0.0f, w_next = 0.0f;
        if (nrounds > 0) {
            IdxT raw0;
            load_raw(0, raw0, w_cur);
            load_raw(1, raw_next, w_next);
            const int32_t idx0 = narrow(raw0);
            if (idx0 < 0) w_cur = 0.0f;
            issue(idx0);
        }
#pragma unroll 1
        for (int r = 0; r < nrounds; ++r) {
            if (!mbar_wait(bar, parity)) {
                if (p.error_flag) atomicOr(p.error_flag, 2);
                return false;
            }
            parity ^= 1u;

            const int cnt = min(R, maxn - r * R);
            uint32_t rd = read0, ex = extra0;
#pragma unroll 1
            for (int u = 0; u < cnt; ++u, rd += pass_pitch, ex += pass_pitch) {
                float w = 1.0f;
                if constexpr (WEIGHTED) w = __shfl_sync(kFull, w_cur, u, LPR);
                if constexpr (kHdr) {
                    uint32_t words[4] = {0u, 0u, 0u, 0u};
                    if (k8) {
                        const uint4 v = lds16(rd);
                        words[0] = v.x; words[1] = v.y; words[2] = v.z; words[3] = v.w;
                    } else {
                        const uint2 v = lds8(rd);
                        words[0] = v.x; words[1] = v.y;
                    }
                    const uint32_t x = lds4(ex);
                    const uint32_t hdr = head_lane ? words[0] : x;
                    const uint32_t w0 = head_lane ? x : words[0];
                    accum_header_row<TY, WEIGHTED, FOLD>(w0, words, hdr, w, acc, bias_acc, scale_acc);
                } else if constexpr (TY == TBE_B200_FP8) {
                    // byte -> fp32 by bit placement: ((b & 0x7f) << (16 + ebits)) as a float, times 2^(127 - bias),
                    // sign bit or'ed in (reference: c310/op_kernel/common.h:120-167)
                    const uint4 v = lds16(rd);
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
#pragma unroll
                        for (int b4 = 0; b4 < 4; ++b4) {
                            const uint32_t by = (words[i4] >> (8 * b4)) & 0xffu;
                            const float mag = __uint_as_float((by & 0x7fu) << p.fp8_shift) * p.fp8_mult;
                            const float val = __uint_as_float(__float_as_uint(mag) | ((by & 0x80u) << 24));
                            acc[4 * i4 + b4] = fmaf(w, val, acc[4 * i4 + b4]);
                        }
                    }
                } else if constexpr (TY == TBE_B200_FP16) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint4 v = lds16(rd + c * nunits * 16);
                        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                        // unweighted: value * 1.0 + acc in one mixed FMA
#pragma unroll
                        for (int i4 = 0; i4 < 4; ++i4)
                            add_pair_t<WEIGHTED>(acc[8 * c + 2 * i4], acc[8 * c + 2 * i4 + 1], words[i4], 0x3c00u, w);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 v = lds16(rd + c * nunits * 16);
                        acc[4 * c + 0] = fmaf(w, __uint_as_float(v.x), acc[4 * c + 0]);
                        acc[4 * c + 1] = fmaf(w, __uint_as_float(v.y), acc[4 * c + 1]);
                        acc[4 * c + 2] = fmaf(w, __uint_as_float(v.z), acc[4 * c + 2]);
                        acc[4 * c + 3] = fmaf(w, __uint_as_float(v.w), acc[4 * c + 3]);
                    }
                }
            }
            if constexpr (FOLD) {
                since_fold += cnt;
                if (since_fold >= 32) {
#pragma unroll
                    for (int s = 0; s < 16; ++s) acc[s] = fmaf(-1024.0f, scale_acc, acc[s]);
                    scale_acc = 0.0f;
                    since_fold = 0;
                }
            }
            if (r + 1 < nrounds) {
                // The next round's rows go out (its indices were requested a round ago), then the request for
                // the indices of the round after it.
                const int32_t idx1 = narrow(raw_next);
                w_cur = (idx1 >= 0) ? w_next : 0.0f;
                issue(idx1);
                load_raw(r + 2, raw_next, w_next);
            }
        }
        // What is left of the folded offset goes out with the biases.
        if constexpr (FOLD) bias_acc = fmaf(-1024.0f, scale_acc, bias_acc);
        const float mean_mul = (mean && Lbag > 0) ? 1.0f / static_cast<float>(Lbag) : 1.0f;

        if (!split) {
            // Every group stores its own bag: slots [4q, 4q + 4) of a lane are 4 consecutive elements.
            const int64_t bag = j + g;
            char* seg = p.dests ? dest_segment(p, b0 + bag, m.col, esz) : out_run + bag * row_bytes;
            const bool vec = p.dests ? (reinterpret_cast<uintptr_t>(seg) & 15) == 0 : vec_ok;
            bool stored = false;
            if constexpr (FOLD) {
                // Unweighted INT8 with a 16-bit output (the only instantiation that carries this code: compiled into
                // the others it cost the INT4 and fp32-output shapes 4 % through register allocation alone).  A
                // lane's 16 elements start 4 elements before a 32-byte boundary.  Its first 4 go to the lane below
                // (the header lane's, the row's tail, to the last lane), after which every lane owns elements
                // [16k, 16k + 16): two aligned 16-byte stores, whole sectors, instead of four 8-byte ones that share
                // sectors with the neighbours.
                if (vec) {
                    uint32_t h[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float lo16 = (acc[2 * q] + bias_acc) * mean_mul, hi16 = (acc[2 * q + 1] + bias_acc) * mean_mul;
                        h[q] = (p.out_ty == TBE_B200_FP16) ? (f32_to_f16_bits(lo16) | (f32_to_f16_bits(hi16) << 16))
                                                           : (f32_to_bf16_bits(lo16) | (f32_to_bf16_bits(hi16) << 16));
                    }
                    const int from = (k + 1 == nunits) ? 0 : k + 1;
                    const uint32_t up0 = __shfl_sync(kFull, h[0], from, LPR);
                    const uint32_t up1 = __shfl_sync(kFull, h[1], from, LPR);
                    if (active && bag < nb) {
                        st_stream16(seg + 32 * k, make_uint4(h[2], h[3], h[4], h[5]));
                        st_stream16(seg + 32 * k + 16, make_uint4(h[6], h[7], up0, up1));
                    }
                    stored = true;
                }
            }
            if (!stored && active && bag < nb) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float v[4];
#pragma unroll
                    for (int s = 0; s < 4; ++s) v[s] = (acc[4 * q + s] + bias_acc) * mean_mul;
                    store_out<4>(seg, elem_of(4 * q), v, p.out_ty, vec);
                }
            }
            j += G;
        } else {
            // One bag over all groups: reduce-scatter the partial sums, add the pooled biases, store.
            if constexpr (G >= 2) halve<16>(acc, 16, (lane >> 4) & 1);
            if constexpr (G >= 4) halve<8>(acc, 8, (lane >> 3) & 1);
            if constexpr (G >= 8) halve<4>(acc, 4, (lane >> 2) & 1);
            if constexpr (kHdr) {
#pragma unroll
                for (int d = LPR; d < kWarp; d <<= 1) bias_acc += __shfl_xor_sync(kFull, bias_acc, d);
            }
            char* seg = p.dests ? dest_segment(p, b0 + j, m.col, esz) : out_run + static_cast<int64_t>(j) * row_bytes;
            const bool vec = p.dests ? (reinterpret_cast<uintptr_t>(seg) & 15) == 0 : vec_ok;
            if (active) {
#pragma unroll
                for (int q = 0; q < NF / WS; ++q) {
                    float v[WS];
#pragma unroll
                    for (int s = 0; s < WS; ++s) v[s] = (acc[q * WS + s] + bias_acc) * mean_mul;
                    store_out<WS>(seg, elem_of(slot_base + q * WS), v, p.out_ty, vec);
                }
            }
            j += 1;
        }
    }
    return true;
}

// A run of bags of one table through the general per-bag code.
template <typename IdxT>
__device__ __forceinline__ void pool_run_general(const LookupParams& p, const TableMeta& m, int64_t i0, int64_t i1, int64_t b,
                                                 int lane, uint32_t wsm)
{
    const IdxT* offsets = static_cast<const IdxT*>(p.offsets);
    const IdxT* indices = static_cast<const IdxT*>(p.indices);
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    int64_t start = static_cast<int64_t>(offsets[i0]);
    for (int64_t i = i0; i < i1; ++i, ++b) {
        const int64_t end = static_cast<int64_t>(offsets[i + 1]);
        const int L = static_cast<int>(end - start);
        BagInfo bag;
        bag.table = m.table;
        bag.stride = m.stride;
        bag.start = start;
        bag.L = L;
        bag.D = m.D;
        bag.mean_mul = (p.pooling_mode == TBE_B200_POOL_MEAN && L > 0) ? 1.0f / static_cast<float>(L) : 1.0f;
        char* dst;
        int64_t brow = b;
        if (p.dests) {
            const int64_t which = b / p.rows_per_dest;
            brow = b - which * p.rows_per_dest;
            dst = static_cast<char*>(p.dests[which]);
        } else {
            dst = static_cast<char*>(p.output);
        }
        bag.seg = dst + (brow * p.out_stride + m.col) * esz;
        bag.seg_aligned = (reinterpret_cast<uintptr_t>(bag.seg) & 15) == 0;
        bool done = false;
        if (m.rows_aligned && (m.D & 3) == 0) {
            const BagHead head = load_batch<IdxT>(indices + start, p.pw ? p.pw + start : nullptr, min(L, kWarp), lane, p.error_flag);
            done = true;
            switch (m.ty) {
                case TBE_B200_INT8: pool_bag_by_width<TBE_B200_INT8, IdxT>(p, bag, head, lane, wsm); break;
                case TBE_B200_INT4: pool_bag_by_width<TBE_B200_INT4, IdxT>(p, bag, head, lane, wsm); break;
                case TBE_B200_FP8: pool_bag_by_width<TBE_B200_FP8, IdxT>(p, bag, head, lane, wsm); break;
                case TBE_B200_FP16:
                    if ((m.D & 7) == 0) pool_bag_by_width<TBE_B200_FP16, IdxT>(p, bag, head, lane, wsm);
                    else done = false;
                    break;
                case TBE_B200_FP32: pool_bag_by_width<TBE_B200_FP32, IdxT>(p, bag, head, lane, wsm); break;
                default: done = false; break;
            }
        }
        if (!done)
            pool_bag_bytewise<IdxT>(indices + start, p.pw ? p.pw + start : nullptr, p.error_flag, bag.table, bag.stride, L,
                                    m.D, bag.seg, bag.mean_mul, m.ty, p.out_ty, p.fp8_shift, p.fp8_mult, lane);
        start = end;
    }
}

template <int TY, typename IdxT, bool WEIGHTED, bool FOLD>
__device__ __forceinline__ bool pool_run_staged_by_width(const LookupParams& p, const TableMeta& m, int64_t i0, int64_t i1,
                                                         int64_t b, int lane, uint32_t wsm, uint32_t bar, uint32_t& parity)
{
    const int nunits = m.D / 16;
    if (nunits <= 4) return pool_run_staged<TY, 4, IdxT, WEIGHTED, FOLD>(p, m, i0, i1, b, lane, wsm, bar, parity);
    if (nunits <= 8) return pool_run_staged<TY, 8, IdxT, WEIGHTED, FOLD>(p, m, i0, i1, b, lane, wsm, bar, parity);
    if (nunits <= 16) return pool_run_staged<TY, 16, IdxT, WEIGHTED, FOLD>(p, m, i0, i1, b, lane, wsm, bar, parity);
    return pool_run_staged<TY, 32, IdxT, WEIGHTED, FOLD>(p, m, i0, i1, b, lane, wsm, bar, parity);
}

template <typename IdxT, bool WEIGHTED>
__device__ __forceinline__ bool pool_run_staged_by_type(const LookupParams& p, const TableMeta& m, int64_t i0, int64_t i1,
                                                        int64_t b, int lane, uint32_t wsm, uint32_t bar, uint32_t& parity)
{
    switch (m.ty) {
        case TBE_B200_INT8:
            if constexpr (!WEIGHTED) {
                if (p.out_ty != TBE_B200_FP32)
                    return pool_run_staged_by_width<TBE_B200_INT8, IdxT, false, true>(p, m, i0, i1, b, lane, wsm, bar, parity);
            }
            return pool_run_staged_by_width<TBE_B200_INT8, IdxT, WEIGHTED, false>(p, m, i0, i1, b, lane, wsm, bar, parity);
        case TBE_B200_INT4: return pool_run_staged_by_width<TBE_B200_INT4, IdxT, WEIGHTED, false>(p, m, i0, i1, b, lane, wsm, bar, parity);
        case TBE_B200_FP8: return pool_run_staged_by_width<TBE_B200_FP8, IdxT, WEIGHTED, false>(p, m, i0, i1, b, lane, wsm, bar, parity);
        case TBE_B200_FP16: return pool_run_staged_by_width<TBE_B200_FP16, IdxT, WEIGHTED, false>(p, m, i0, i1, b, lane, wsm, bar, parity);
        default: return pool_run_staged_by_width<TBE_B200_FP32, IdxT, WEIGHTED, false>(p, m, i0, i1, b, lane, wsm, bar, parity);
    }
}

// ---- kernels -----------------------------------------------------------------

constexpr int kWarpsPerBlock = 4;
constexpr int kMinBlocksPerSM = 8;   // 32 resident warps per SM: 64 registers and 6 KB of staging memory per warp

// The T*B bags (bag i = t*B + b) are cut into spans of `span` consecutive bags, one span per warp, so a
// warp walks `offsets`, `indices` and the per-sample weights front to back.  A span is processed as runs
// of consecutive bags of one table: the table's description is read once per run and the run is handed
// to the code specialised for its row shape.
template <typename IdxT, int MINB>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, MINB)
tbe_pooled_kernel(const __grid_constant__ LookupParams p)
{
    __shared__ __align__(128) uint8_t smem[kWarpsPerBlock * kWarpSmemBytes];
    __shared__ __align__(8) uint64_t bars[kWarpsPerBlock];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t wsm = smem_u32(smem) + warp * kWarpSmemBytes;
    const uint32_t bar = smem_u32(&bars[warp]);
    const int64_t gw = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
    const int64_t span_lo = gw * p.span;
    const int64_t span_hi = min(p.num_bags, span_lo + p.span);
    if (span_lo >= span_hi) return;
    // The span's first offsets are needed right after the table description: ask for their line(s) now, so the two
    // latencies overlap.
    if (lane < 2) {
        const IdxT* o = static_cast<const IdxT*>(p.offsets) + (lane == 0 ? span_lo : span_hi);
        asm volatile("prefetch.global.L1 [%0];" ::"l"(o));
    }
    // One mbarrier per warp; every lane arrives once per round of staged rows.
    if (lane == 0) mbar_init(bar, kWarp);
    __syncwarp();
    uint32_t parity = 0;

    int t;
    int64_t b;
    if (p.B32) {
        t = static_cast<int>(static_cast<uint32_t>(span_lo) / p.B32);
        b = static_cast<uint32_t>(span_lo) - static_cast<uint32_t>(t) * p.B32;
    } else {
        t = static_cast<int>(span_lo / p.B);
        b = span_lo - static_cast<int64_t>(t) * p.B;
    }
    const bool weighted = p.pw != nullptr;

    for (int64_t i = span_lo; i < span_hi;) {
        const int64_t run_end = min(span_hi, i + (p.B - b));   // the bags left in table t, or in the span
        const TableMeta m = load_meta(p, t);
        if (m.D > 0) {
            const bool staged = m.rows_aligned && (m.D & 15) == 0 && m.D <= 512 && m.stride < (1ll << 32) &&
                                (m.ty == TBE_B200_INT8 || m.ty == TBE_B200_INT4 || m.ty == TBE_B200_FP8 ||
                                 m.ty == TBE_B200_FP16 || m.ty == TBE_B200_FP32);
            if (staged) {
                const bool ok = weighted ? pool_run_staged_by_type<IdxT, true>(p, m, i, run_end, b, lane, wsm, bar, parity)
                                         : pool_run_staged_by_type<IdxT, false>(p, m, i, run_end, b, lane, wsm, bar, parity);
                if (!ok) return;   // a bounded wait ran out; the error flag says so
            } else {
                pool_run_general<IdxT>(p, m, i, run_end, b, lane, wsm);
            }
        }
        b += run_end - i;
        i = run_end;
        if (b == p.B) {
            b = 0;
            ++t;
        }
    }
}

// ---- pooling NONE (sequence mode) --------------------------------------------------------------
//
// Row n of the output gets the dequantised row indices[n] of the table that position n belongs to (the t with
// offsets[t*B] <= n < offsets[(t+1)*B]), zero-filled from D_t up to max_D.  A warp takes kNobagChunk consecutive
// positions: the table is found once by binary search and then followed, and G = 32 / LPR rows are handled per
// pass, LPR lanes per row, 16 elements per lane, with the same chunk-to-element mapping as the pooled path.
// Nothing is accumulated, so rows go straight to registers; value = code * scale + bias in one mixed FMA.

constexpr int kNobagChunk = 64;

// One position through the byte-wise decoder (any type, alignment and width).
template <typename IdxT>
__device__ __noinline__ void nobag_position_bytewise(const LookupParams& p, const TableMeta& m, const IdxT* indices, int64_t n, int max_D,
                                                     int lane)
{
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    void* seg = static_cast<char*>(p.output) + n * p.out_stride * esz;
    const int64_t idx = static_cast<int64_t>(indices[n]);
    if (idx < 0) {
        if (idx < -1 && lane == 0 && p.error_flag) atomicOr(p.error_flag, 1);
        for (int e = lane; e < max(m.D, max_D); e += kWarp) store_scalar(seg, e, 0.0f, p.out_ty);
        return;
    }
    const uint8_t* row = m.table + idx * m.stride;
    float scale, bias;
    read_header(row, m.ty, scale, bias);
    for (int e = lane; e < m.D; e += kWarp)
        store_scalar(seg, e, decode_elem(row, m.ty, e, scale, bias, p.fp8_shift, p.fp8_mult), p.out_ty);
    for (int e = m.D + lane; e < max_D; e += kWarp) store_scalar(seg, e, 0.0f, p.out_ty);
}

// `cnt` consecutive positions [n, n + cnt) of one table with aligned rows of D = 16 * units <= 512 elements.
template <int TY, int LPR, typename IdxT>
__device__ __forceinline__ void nobag_rows(const LookupParams& p, const TableMeta& m, const IdxT* indices, int64_t n, int cnt, int max_D,
                                           int lane)
{
    constexpr bool kHdr = (TY == TBE_B200_INT8 || TY == TBE_B200_INT4);
    constexpr bool k8 = (TY == TBE_B200_INT8);
    constexpr int CH = (TY == TBE_B200_INT4) ? 8 : 16;
    constexpr int NCH = (TY == TBE_B200_FP16) ? 2 : (TY == TBE_B200_FP32) ? 4 : 1;
    constexpr int EPC = 16 / NCH;
    constexpr int HS = k8 ? 4 : (TY == TBE_B200_INT4 ? 8 : 0);
    constexpr int G = kWarp / LPR;
    const int k = lane % LPR, g = lane / LPR;
    const int D = m.D, nunits = D / 16;
    const bool head_lane = kHdr && k == 0;
    const bool active = k < nunits;
    const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
    for (int r0 = 0; r0 < cnt; r0 += G) {
        const bool mine = r0 + g < cnt;
        int64_t idx = -1;
        if (mine) {
            idx = static_cast<int64_t>(__ldg(indices + n + r0 + g));
            if ((idx < -1 || idx > 0x7fffffffll) && k == 0 && p.error_flag) atomicOr(p.error_flag, 1);
            if (idx > 0x7fffffffll) idx = -1;
        }
        const bool ok = idx >= 0;
        const uint8_t* row = m.table + (ok ? idx : 0) * m.stride;
        uint32_t words[4 * NCH];
#pragma unroll
        for (int c = 0; c < 4 * NCH; ++c) words[c] = 0u;
        uint32_t tail = 0u;
        if (ok && active) {
            if constexpr (TY == TBE_B200_INT4) {
                const uint2 v = ldg8(row + k * 8);
                words[0] = v.x; words[1] = v.y;
            } else {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const uint4 v = ldg16(row + 16 * (k + c * nunits));
                    words[4 * c + 0] = v.x; words[4 * c + 1] = v.y; words[4 * c + 2] = v.z; words[4 * c + 3] = v.w;
                }
            }
            if (head_lane) tail = ldg4(row + (k8 ? D : D / 2));
        }
        float v[16];
        if constexpr (kHdr) {
            const uint32_t hdr = __shfl_sync(kFull, words[0], 0, LPR);   // zero for a row that is not read
            const uint32_t w0 = head_lane ? tail : words[0];
            const unsigned short scale_h = static_cast<unsigned short>(hdr & 0xffffu);
            const float bias = half_bits_to_float(hdr >> 16);
#pragma unroll
            for (int s = 0; s < 16; ++s) v[s] = bias;
            if (k8) {
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const uint32_t c = (i4 == 0) ? w0 : words[i4];
                    const uint32_t even = codes_to_half2((c & 0x00FF00FFu) | 0x64006400u, 0x64006400u);
                    const uint32_t odd = codes_to_half2(__byte_perm(c, 0x64646464u, 0x4341), 0x64006400u);
                    add_pair_t<false>(v[4 * i4 + 0], v[4 * i4 + 2], even, scale_h, 0.0f);
                    add_pair_t<false>(v[4 * i4 + 1], v[4 * i4 + 3], odd, scale_h, 0.0f);
                }
            } else {
#pragma unroll
                for (int i2 = 0; i2 < 2; ++i2) {
                    const uint32_t c = (i2 == 0) ? w0 : words[i2];
                    const uint32_t y = c >> 8;
                    const uint32_t p0 = codes_to_half2((c & 0x000F000Fu) | 0x64006400u, 0x64006400u);
                    const uint32_t p1 = codes_to_half2((c & 0x00F000F0u) | 0x54005400u, 0x54005400u);
                    const uint32_t p2 = codes_to_half2((y & 0x000F000Fu) | 0x64006400u, 0x64006400u);
                    const uint32_t p3 = codes_to_half2((y & 0x00F000F0u) | 0x54005400u, 0x54005400u);
                    add_pair_t<false>(v[8 * i2 + 0], v[8 * i2 + 4], p0, scale_h, 0.0f);
                    add_pair_t<false>(v[8 * i2 + 1], v[8 * i2 + 5], p1, scale_h, 0.0f);
                    add_pair_t<false>(v[8 * i2 + 2], v[8 * i2 + 6], p2, scale_h, 0.0f);
                    add_pair_t<false>(v[8 * i2 + 3], v[8 * i2 + 7], p3, scale_h, 0.0f);
                }
            }
        } else if constexpr (TY == TBE_B200_FP8) {
#pragma unroll
            for (int s = 0; s < 16; ++s) {
                const uint32_t by = (words[s >> 2] >> (8 * (s & 3))) & 0xffu;
                const float mag = __uint_as_float((by & 0x7fu) << p.fp8_shift) * p.fp8_mult;
                v[s] = __uint_as_float(__float_as_uint(mag) | ((by & 0x80u) << 24));
            }
        } else if constexpr (TY == TBE_B200_FP16) {
#pragma unroll
            for (int s = 0; s < 16; ++s) v[s] = half_bits_to_float((words[s >> 1] >> (16 * (s & 1))) & 0xffffu);
        } else {
#pragma unroll
            for (int s = 0; s < 16; ++s) v[s] = __uint_as_float(words[s]);
        }
        if (mine) {
            char* seg = static_cast<char*>(p.output) + (n + r0 + g) * p.out_stride * esz;
            const bool vec = ((reinterpret_cast<uintptr_t>(seg)) & 15) == 0;
            if (active) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int slot = 4 * q;
                    int e0;
                    if constexpr (kHdr) e0 = (head_lane && slot < HS) ? (D - HS + slot) : (16 * k - HS + slot);
                    else e0 = EPC * (k + (slot / EPC) * nunits) + (slot % EPC);
                    store_out<4>(seg, e0, &v[slot], p.out_ty, vec);
                }
            }
            for (int e = D + k; e < max_D; e += LPR) store_scalar(seg, e, 0.0f, p.out_ty);
        }
    }
}

template <int TY, typename IdxT>
__device__ __forceinline__ void nobag_rows_by_width(const LookupParams& p, const TableMeta& m, const IdxT* indices, int64_t n, int cnt,
                                                    int max_D, int lane)
{
    const int nunits = m.D / 16;
    if (nunits <= 4) nobag_rows<TY, 4, IdxT>(p, m, indices, n, cnt, max_D, lane);
    else if (nunits <= 8) nobag_rows<TY, 8, IdxT>(p, m, indices, n, cnt, max_D, lane);
    else if (nunits <= 16) nobag_rows<TY, 16, IdxT>(p, m, indices, n, cnt, max_D, lane);
    else nobag_rows<TY, 32, IdxT>(p, m, indices, n, cnt, max_D, lane);
}

template <typename IdxT>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
tbe_nobag_kernel(const __grid_constant__ LookupParams p, int64_t num_indices, int max_D)
{
    const int lane = threadIdx.x & 31;
    const int64_t gw = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    int64_t n = gw * kNobagChunk;
    const int64_t n_end = min(num_indices, n + kNobagChunk);
    if (n >= n_end) return;
    const IdxT* offsets = static_cast<const IdxT*>(p.offsets);
    const IdxT* indices = static_cast<const IdxT*>(p.indices);
    // Binary search over the T+1 table boundaries offsets[t*B]: the table of the chunk's first position.
    int lo = 0, hi = p.T;   // invariant: boundary(lo) <= n < boundary(hi)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(offsets[static_cast<int64_t>(mid) * p.B]) <= n) lo = mid;
        else hi = mid;
    }
    int t = lo;
    while (n < n_end) {
        // positions [n, stop) belong to table t (skip tables without positions)
        int64_t stop = static_cast<int64_t>(offsets[static_cast<int64_t>(t + 1) * p.B]);
        while (stop <= n && t + 1 < p.T) {
            ++t;
            stop = static_cast<int64_t>(offsets[static_cast<int64_t>(t + 1) * p.B]);
        }
        stop = (t + 1 >= p.T) ? n_end : min(stop, n_end);
        if (stop <= n) stop = n_end;   // offsets that do not cover every position: the last table takes the rest
        const TableMeta m = load_meta(p, t);
        const int cnt = static_cast<int>(stop - n);
        const bool fast = m.rows_aligned && m.D > 0 && (m.D & 15) == 0 && m.D <= 512;
        bool done = fast;
        if (fast) {
            switch (m.ty) {
                case TBE_B200_INT8: nobag_rows_by_width<TBE_B200_INT8, IdxT>(p, m, indices, n, cnt, max_D, lane); break;
                case TBE_B200_INT4: nobag_rows_by_width<TBE_B200_INT4, IdxT>(p, m, indices, n, cnt, max_D, lane); break;
                case TBE_B200_FP8: nobag_rows_by_width<TBE_B200_FP8, IdxT>(p, m, indices, n, cnt, max_D, lane); break;
                case TBE_B200_FP16: nobag_rows_by_width<TBE_B200_FP16, IdxT>(p, m, indices, n, cnt, max_D, lane); break;
                case TBE_B200_FP32: nobag_rows_by_width<TBE_B200_FP32, IdxT>(p, m, indices, n, cnt, max_D, lane); break;
                default: done = false; break;
            }
        }
        if (!done)
            for (int64_t q = n; q < stop; ++q) nobag_position_bytewise<IdxT>(p, m, indices, q, max_D, lane);
        n = stop;
    }
}

constexpr int kSpanLarge = 16;   // bags per warp when there is plenty of work; a multiple of every group count

template <typename IdxT, int MINB>
int launch_pooled(LookupParams p, int max_D, cudaStream_t s)
{
    static int resident = 0;   // blocks that fit on one SM (occupancy query, once)
    if (resident == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, tbe_pooled_kernel<IdxT, MINB>, kWarpsPerBlock * kWarp, 0) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = MINB;
        }
        resident = n;
    }
    // Plenty of bags: fixed spans, as many blocks as that takes; the hardware block scheduler evens out the
    // load.  Otherwise one span per resident warp, rounded up to the number of bags a warp pools side by
    // side for rows of max_D elements, so that a warp's last step is not a mostly idle one.
    const int64_t slots = static_cast<int64_t>(sm_count()) * resident * kWarpsPerBlock;
    if (p.num_bags >= slots * kSpanLarge) {
        p.span = kSpanLarge;
    } else {
        int lpr = 2;
        while (lpr < 32 && lpr * 16 < max_D) lpr <<= 1;
        const int64_t grain = kWarp / lpr;
        const int64_t per = (p.num_bags + slots - 1) / slots;
        p.span = per < grain ? per : grain;
    }
    const int64_t warps = (p.num_bags + p.span - 1) / p.span;
    const int64_t blocks = (warps + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: too many bags for one launch");
    tbe_pooled_kernel<IdxT, MINB><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p);
    return check_launch("tbe_pooled_kernel");
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
    p.num_indices = a->num_indices;
    p.out_stride = a->output_stride;
    p.rows_per_dest = a->rows_per_dest;
    p.span = 1;
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
        const int64_t chunks = (a->num_indices + kNobagChunk - 1) / kNobagChunk;
        const int64_t blocks = (chunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
        if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: too many indices for one launch");
        if (a->index_bits == 32)
            tbe_nobag_kernel<int32_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p, a->num_indices, a->max_D);
        else
            tbe_nobag_kernel<int64_t><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, 0, s>>>(p, a->num_indices, a->max_D);
        return check_launch("tbe_nobag_kernel");
    }
    if (p.num_bags == 0) return TBE_B200_OK;
    return a->index_bits == 32 ? launch_pooled<int32_t, kMinBlocksPerSM>(p, a->max_D, s)
                               : launch_pooled<int64_t, kMinBlocksPerSM>(p, a->max_D, s);
}
