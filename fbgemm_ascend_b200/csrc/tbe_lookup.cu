// Quantized table-batched-embedding lookup for B200 (sm_100a).
//
// Replaces the device side of int_nbit_split_embedding_codegen_lookup_function
// (reference: c310/op_kernel/int_nbit_split_embedding_pooling_kernel.h:44-394 and
// int_nbit_split_embedding_nobag_kernel.h:31-398).  The path is a gather and a
// reduction bounded by HBM/L2 bandwidth, so there is no tensor-core work here.
//
// Pooled kernel (SUM / MEAN), in three tiers chosen per table:
//   * aligned rows of INT8 / INT4 / FP8 / FP16 / FP32 with D a multiple of 16 up to 512 (pool_run_stream): LPR lanes
//     share a row, 16 fp32 accumulators per lane, so a warp has 32/LPR lane groups.  The rows of a warp's bags are
//     cut into equal ranges, one per group, and every group streams its range through a small ring in shared
//     memory: asynchronous 16-byte copies through L1 (which holds the hot head of a Zipf-distributed table), several
//     rows per group in flight, consumed in order; bags that straddle two ranges are combined through shared memory.  Rows are dequantised
//     with the row's fp16 scale/bias (codes -> exact fp16 by a magic constant, then fp16 x fp16 + fp32 mixed FMA)
//     and accumulated in fp32.  INT8/INT4 rows start with a 4-byte header, which shifts the payload off the
//     16-byte grid; the lane that reads the header chunk has 4 / 8 free slots, which take the row's last
//     elements, so D = 16*LPR rows keep every lane busy with exactly 16 elements;
//   * other aligned shapes (pool_bag; only in the build of the kernel for wide tables): one warp per bag, cp.async
//     staging in chunks, cross-group reduce-scatter;
//   * anything else (row_alignment 1, odd D, INT2 or BF16 rows, unaligned tables): a byte-wise path.
// Sequence mode (pooling NONE): tbe_nobag_kernel, 64 consecutive positions per warp.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>

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
    int64_t dev_weights_bytes;   // size of dev_weights, 0 = unknown
    int32_t idx64;       // indices and offsets are 64-bit
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
// The same through L1 (the line stays cached for the rows that are fetched again and again).
__device__ __forceinline__ void cp_async16_ca(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
#ifdef TBE_L2_HINTS
// Experiment (TBE_L2_HINTS builds only): the row copies carry an L2 evict-last policy.  Measured on benchmark
// configurations 2 and 4 (scaled): L2 hit rate, DRAM bytes and kernel time all unchanged (31.8 -> 31.9 % and
// 45.5 -> 45.5 %; the hottest rows never reach L2, they hit L1, and the rest of the Zipf head stays in L2 anyway),
// so the plain form is what is built.
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void cp_async16_ca_hint(uint32_t dst, const void* src, int bytes, uint64_t pol)
{
    asm volatile("cp.async.ca.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(bytes), "l"(pol) : "memory");
}
#endif
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
    int64_t avail;          // bytes of the table: a row that would end past them is skipped
};

// Up to 32 consecutive indices and weights of a bag, one per lane.  Indices are narrowed to 32 bits:
// a row number outside [-1, 2^31) is reported through the error flag and treated as -1 (skipped).
struct BagHead {
    int32_t idx;   // -1 beyond the bag
    float w;
};

template <typename IdxT>
__device__ __forceinline__ BagHead load_batch(const IdxT* indices, const float* pw, int n, int lane, int32_t* error_flag,
                                              int64_t stride, int64_t avail)
{
    BagHead h;
    h.idx = -1;
    h.w = 1.0f;
    if (lane < n) {
        const int64_t v = static_cast<int64_t>(__ldg(indices + lane));
        const bool bad = (v < -1) || (v > 0x7fffffffll);
        const bool past = !bad && v >= 0 && static_cast<uint64_t>(v + 1) * static_cast<uint64_t>(stride) > static_cast<uint64_t>(avail);
        h.idx = (bad || past) ? -1 : static_cast<int32_t>(v);
        if ((bad || past) && error_flag) atomicOr(error_flag, bad ? 1 : 4);
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
                                                    cx.first_blk ? p.error_flag : nullptr, bag.stride, bag.avail);
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
    int64_t avail;          // bytes of dev_weights the table's rows may occupy (a row past them is not read)
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
    // The table ends where the next one starts (tables laid out in order) or, failing that, where dev_weights ends.
    m.avail = 0x7fffffffffffffffll;
    if (p.dev_weights_bytes > 0) {
        const int64_t start = p.weights_offsets[t];
        int64_t end = p.dev_weights_bytes;
        if (t + 1 < p.T) {
            const int64_t next = p.weights_offsets[t + 1];
            if (next > start && next < end) end = next;
        }
        m.avail = end > start ? end - start : 0;
    }
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
                                               float fp8_mult, int lane, int64_t avail)
{
    for (int e_blk = 0; e_blk < D; e_blk += kByteAcc * kWarp) {
        float acc[kByteAcc];
#pragma unroll
        for (int j = 0; j < kByteAcc; ++j) acc[j] = 0.0f;
        for (int n = 0; n < L; ++n) {
            const int64_t idx = static_cast<int64_t>(indices[n]);
            if (idx < 0) {
                if (idx < -1 && lane == 0 && error_flag && e_blk == 0) atomicOr(error_flag, 1);
                continue;
            }
            if (idx > 0x7fffffffll || static_cast<uint64_t>(idx + 1) * static_cast<uint64_t>(stride) > static_cast<uint64_t>(avail)) {
                if (lane == 0 && error_flag && e_blk == 0) atomicOr(error_flag, idx > 0x7fffffffll ? 1 : 4);
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

// ---- the common shapes: rows streamed through a shared-memory ring, groups of lanes -----------------

// Zeros that stand in for a row that must not be added: zero payload, and for INT8 / INT4 a zero header (scale 0, bias 0).
__device__ __align__(16) const uint8_t g_zero_row[2048] = {0};

// Read-once streams (indices, per-sample weights): not kept in L1.
__device__ __forceinline__ int32_t ld_once32(const void* p) { return ld_stream(static_cast<const int32_t*>(p)); }
__device__ __forceinline__ float ld_once_f32(const void* p) { return ld_stream(static_cast<const float*>(p)); }
__device__ __forceinline__ uint2 ld_once_2x32(const void* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void sts16(uint32_t a, float x, float y, float z, float w)
{
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void sts4(uint32_t a, int32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ float4 lds16f(uint32_t a)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ int32_t lds4i(uint32_t a)
{
    int32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}

// The header of an INT8 / INT4 row (fp16 scale, fp16 bias; zero for a row that is not to be added): adds the bias
// (and, in the folded form, the scale) to the bag's running sums and returns the scale's fp16 bits; `ws` is
// scale * w for the weighted form.
template <bool WEIGHTED, bool FOLD>
__device__ __forceinline__ unsigned short accum_header(uint32_t hdr, float w, float& ws, float& bias_acc, float& scale_acc)
{
    const unsigned short scale_h = static_cast<unsigned short>(hdr & 0xffffu);
    ws = 0.0f;
    if constexpr (WEIGHTED) {
        ws = half_bits_to_float(scale_h) * w;
        bias_acc = fmaf(half_bits_to_float(hdr >> 16), w, bias_acc);
    } else {
        bias_acc += half_bits_to_float(hdr >> 16);
        if constexpr (FOLD) scale_acc += half_bits_to_float(scale_h);
    }
    return scale_h;
}

// Adds NW 32-bit words of INT8 (4 per word) or INT4 (8 per word) codes, times the row scale, to consecutive slots
// of `acc` (a compile-time position inside the lane's accumulators).
template <int TY, bool WEIGHTED, bool FOLD, int NW>
__device__ __forceinline__ void accum_codes(const uint32_t (&words)[NW], unsigned short scale_h, float ws, float* acc)
{
    if constexpr (TY == TBE_B200_INT8 && FOLD) {
        // One byte permute per code builds the register the mixed FMA wants: its two fp16 operands side by side,
        // (1024 + q) below (bytes q, 0x64) and the row scale above.  With the operands in two registers the compiler
        // spends a move per FMA to bring them together (measured: 16 moves for 16 FMAs, none in this form).
        const uint32_t y = (static_cast<uint32_t>(scale_h) << 16) | 0x6400u;
#pragma unroll
        for (int i = 0; i < NW; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t x = __byte_perm(words[i], y, 0x7650u | j);
                asm("{ .reg .b16 l, h; mov.b32 {l, h}, %1; fma.rn.f32.f16 %0, l, h, %0; }" : "+f"(acc[4 * i + j]) : "r"(x));
            }
        }
    } else if constexpr (TY == TBE_B200_INT8) {
#pragma unroll
        for (int i = 0; i < NW; ++i) {
            const uint32_t c = words[i];
            // bytes 0 and 2, then bytes 1 and 3, placed in the mantissas of half2(1024, 1024)
            uint32_t even = (c & 0x00FF00FFu) | 0x64006400u;
            uint32_t odd = __byte_perm(c, 0x64646464u, 0x4341);
            if constexpr (!FOLD) {
                even = codes_to_half2(even, 0x64006400u);
                odd = codes_to_half2(odd, 0x64006400u);
            }
            add_pair_t<WEIGHTED>(acc[4 * i + 0], acc[4 * i + 2], even, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[4 * i + 1], acc[4 * i + 3], odd, scale_h, ws);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NW; ++i) {
            const uint32_t c = words[i];
            const uint32_t y = c >> 8;
            // nibble pairs (j, j + 4) sit 16 bits apart: 0x6400 | n = 1024 + n; 0x5400 | (n << 4) = 64 + n
            const uint32_t p0 = codes_to_half2((c & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 0, 4
            const uint32_t p1 = codes_to_half2((c & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 1, 5
            const uint32_t p2 = codes_to_half2((y & 0x000F000Fu) | 0x64006400u, 0x64006400u);   // nibbles 2, 6
            const uint32_t p3 = codes_to_half2((y & 0x00F000F0u) | 0x54005400u, 0x54005400u);   // nibbles 3, 7
            add_pair_t<WEIGHTED>(acc[8 * i + 0], acc[8 * i + 4], p0, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i + 1], acc[8 * i + 5], p1, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i + 2], acc[8 * i + 6], p2, scale_h, ws);
            add_pair_t<WEIGHTED>(acc[8 * i + 3], acc[8 * i + 7], p3, scale_h, ws);
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

// Shared memory of one warp in the streaming kernel: the partial sums that lane groups hand to one another
// (up to 32 floats per lane), the run's bag offsets, and the ring of rows in flight.
constexpr int kPartBytes = kWarp * 128;
constexpr int kMaxRunBags = 31;                        // bags of one run: their nb + 1 offsets are held one per lane
constexpr int kRelBytes = 144;                         // (kMaxRunBags + 1) offsets, rounded to 16 bytes
#ifndef TBE_RING_BYTES
#define TBE_RING_BYTES 4352                            // four stages of rows with up to 32 bytes per lane
#endif
#ifndef TBE_MAX_STAGES
#define TBE_MAX_STAGES 4
#endif
constexpr int kRingBytes = TBE_RING_BYTES;
constexpr int kStreamSmemBytes = kPartBytes + kRelBytes + kRingBytes;

__host__ __device__ constexpr int floor_pow2(int x) { return x >= 8 ? 8 : x >= 4 ? 4 : x >= 2 ? 2 : 1; }
__host__ __device__ constexpr int min3(int a, int b, int c) { return a < b ? (a < c ? a : c) : (b < c ? b : c); }

// A run of nb <= kMaxRunBags consecutive bags of ONE table whose rows are D = 16 * n <= 512 elements, 16-byte
// aligned.  LPR lanes share a row, 16 elements per lane, so a warp has G = 32 / LPR lane groups.
//
// Work split.  The run's rows -- positions [R0, R1) of `indices` -- are cut into G equal ranges, one per
// group, whatever the bag lengths are, so the groups finish together.  A group walks its range row by row
// and keeps the sum of the bag it is in; when the walk reaches the end of a bag the group stores the bag
// and starts the next one (a divergent branch, taken once per bag and group).  A bag that straddles a range
// boundary is summed in pieces: the group in whose range the bag STARTS owns it; every later group that holds
// a piece writes its partial sum to shared memory, and the owner adds those pieces at the end of the run.
// Empty bags are written (zeros) by the group whose walk passes their position.
//
// Row fetch.  Lane k of a group reads the index of the group's row c * LPR + k (chunk c of the range; the indices
// of a chunk are requested two chunks ahead).  Rows travel through a ring of NS stages in the warp's shared memory:
// in step q the group consumes row q - NS out of stage q mod NS and then requests row q into the same stage with
// asynchronous copies (cp.async through L1, 16 bytes per lane, completion counted per step with commit / wait
// groups), so NS rows per group are in flight all the time, whatever the compiler does with registers -- a ring of
// registers filled by ordinary loads measured twice as slow, because a warp has only six scoreboards and a row
// about to be consumed ended up waiting for loads that had just been issued.  A lane reads back only the bytes it
// copied itself, so no barrier is involved.  A row that is not to be added (index -1, out of range, past the end
// of the group's range) is zero-filled in the stage without being read.
//
// FOLD (INT8, unweighted, 16-bit output): the subtraction of the magic constant that turns a code into an fp16
// value is skipped, (1024 + q) * scale is accumulated, and 1024 * sum(scale) is removed again at least every
// 32 rows, which keeps the partial sums small enough for the extra term not to cost precision that a 16-bit
// result could show.
template <int TY, int LPR, int EPL, bool WEIGHTED, bool FOLD>
__device__ __noinline__ void pool_run_stream(const LookupParams& p, const TableMeta& m, int64_t i0, int nb, int64_t b0, int lane,
                                             uint32_t wsm)
{
    static_assert(!FOLD || (TY == TBE_B200_INT8 && !WEIGHTED), "the folded form is for unweighted INT8 pooling");
    static_assert(EPL == 16 || (EPL == 32 && (TY == TBE_B200_INT8 || TY == TBE_B200_INT4)), "32 elements per lane: INT8 / INT4 only");
    constexpr bool kHdr = (TY == TBE_B200_INT8 || TY == TBE_B200_INT4);
    constexpr bool k8 = (TY == TBE_B200_INT8);
    // A lane holds NCH chunks of CH bytes of a row; chunk c is unit k + c * nunits of the row (a unit = UE elements),
    // so one copy instruction of a group covers nunits * CH contiguous bytes.
    constexpr int NCH = (TY == TBE_B200_FP16) ? 2 : (TY == TBE_B200_FP32) ? 4 : (k8 ? EPL / 16 : 1);
    constexpr int CH = (TY == TBE_B200_INT4) ? EPL / 2 : 16;           // bytes per chunk
    constexpr int UE = EPL / NCH;                      // elements per unit
    constexpr int HS = k8 ? 4 : (TY == TBE_B200_INT4 ? 8 : 0);         // slots of the header lane that hold the row's tail
    constexpr int G = kWarp / LPR;                     // lane groups
    constexpr int LOG_G = G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3;
    constexpr int LANEB = CH * NCH;                                    // bytes of a row that one lane holds
    constexpr int STAGE = kWarp * LANEB + (kHdr ? 32 : 0);             // one row per group, and the groups' tail words
    constexpr int NS = floor_pow2(min3(kRingBytes / STAGE, LPR, TBE_MAX_STAGES));   // stages of the ring (rows in flight per group)
    static_assert(NS >= 1 && NS * STAGE <= kRingBytes, "the ring does not fit");
    static_assert(G <= 8, "at least 4 lanes per row");
    const int k = lane % LPR;
    const int g = lane / LPR;
    const unsigned gmask = (LPR == 32) ? kFull : (((1u << (LPR & 31)) - 1u) << (g * LPR));
    const int D = m.D;
    const int nunits = D / EPL;                        // lanes that hold a piece of the row
    const bool head_lane = kHdr && (k == 0);
    const bool act = k < nunits;                       // lanes past the row's last unit have nothing to add (D < EPL * LPR)
    const uint32_t stride = static_cast<uint32_t>(m.stride);
    const uint8_t* lane_base = m.table + k * CH;
    const uint32_t tail_off = k8 ? D : D / 2;          // header lane (k = 0): where the row's last HS elements are
    const uint32_t chunk_step = static_cast<uint32_t>(nunits) * CH;    // distance between a lane's chunks
    const uint8_t* zero_base = g_zero_row + k * 16;
    const bool idx64 = p.idx64 != 0;
    const int isz = idx64 ? 8 : 4;
    const uint32_t sm_rel = wsm + kPartBytes;

    // The run's nb + 1 offsets, one per lane, relative to the first one.
    int64_t off = 0;
    if (lane <= nb) {
        const char* op = static_cast<const char*>(p.offsets) + (i0 + lane) * isz;
        off = idx64 ? __ldg(reinterpret_cast<const int64_t*>(op)) : static_cast<int64_t>(__ldg(reinterpret_cast<const int32_t*>(op)));
    }
    int64_t R0 = __shfl_sync(kFull, off, 0);
    int64_t R1 = __shfl_sync(kFull, off, nb);
    if (R0 < 0 || R1 < R0 || R1 > p.num_indices || R1 - R0 > 0x7fffffffll) {
        // Offsets that do not describe positions of `indices`: nothing is read through them; the run's bags are
        // written as empty ones (zeros), so that the output is defined, and the condition is reported.
        if (p.error_flag && lane == 0) atomicOr(p.error_flag, 8);
        off = R0 = R1 = 0;
    }
    const int n = static_cast<int>(R1 - R0);
    const int rel = static_cast<int>(min(max(off - R0, static_cast<int64_t>(0)), static_cast<int64_t>(n)));
    __syncwarp();                                      // the previous run's reads of this memory are over
    if (lane <= nb) sts4(sm_rel + 4 * lane, rel);
    __syncwarp();

    // This group's range of rows, and the bag its first row is in.
    const int per = (n + G - 1) >> LOG_G;
    const int lo = min(n, g * per);
    const int hi = min(n, lo + per);
    int cur = 0;
    if constexpr (G > 1) {
#pragma unroll
        for (int gg = 1; gg < G; ++gg) {
            const int lo_gg = min(n, gg * per);
            const unsigned started = __ballot_sync(kFull, lane >= 1 && lane <= nb && rel <= lo_gg);
            if (g == gg) cur = __popc(started);
        }
    }
    const bool active = (g == 0) || (lo < hi);         // group 0 also writes the empty bags at the front of the run
    int bag_start = lds4i(sm_rel + 4 * cur);
    int bag_end = (active && cur < nb) ? lds4i(sm_rel + 4 * (cur + 1)) : -1;
    int pos = lo;

    // Element a slot stands for: slot s belongs to the lane's chunk s / UE, which is unit k + (s / UE) * nunits of the
    // row.  INT8 / INT4 units are shifted by the header (unit u covers elements [UE * u - HS, UE * u + UE - HS)), and
    // the header lane's first HS slots are the row's last HS elements.
    auto elem_of = [&](int slot) -> int {
        if (kHdr && head_lane && slot < HS) return D - HS + slot;
        return UE * (k + (slot / UE) * nunits) - HS + (slot % UE);
    };

    float acc[EPL];
#pragma unroll
    for (int s = 0; s < EPL; ++s) acc[s] = 0.0f;
    float bias_acc = 0.0f;
    float scale_acc = 0.0f;   // sum of the row scales since the last fold (FOLD only)
    int since_fold = 0;
    (void)scale_acc;
    (void)since_fold;

    // Stores the finished bag `bag` of L rows (acc + bias_acc, times 1/L for MEAN).  Executed by whole groups.
    auto store_bag = [&](int bag, int L) {
        const float mm = (p.pooling_mode == TBE_B200_POOL_MEAN && L > 0) ? 1.0f / static_cast<float>(L) : 1.0f;
        const float bm = bias_acc * mm;
        // (computed here, once per bag, rather than kept in registers across the row loop)
        const int esz = (p.out_ty == TBE_B200_FP32) ? 4 : 2;
        char* seg = p.dests ? dest_segment(p, b0 + bag, m.col, esz)
                            : static_cast<char*>(p.output) + ((b0 + bag) * p.out_stride + m.col) * esz;
        const bool vec = (reinterpret_cast<uintptr_t>(seg) & 15) == 0;
        bool stored = false;
        if constexpr (FOLD) {
            // Unweighted INT8 with a 16-bit output.  A unit's 16 elements start 4 elements before a 32-byte boundary.
            // Its first 4 go to the unit before it (unit 0's, the row's tail, to the last unit), after which every
            // unit is 16 elements from a 32-byte boundary on: two aligned 16-byte stores, whole sectors.  The unit after
            // lane k's chunk c is lane k + 1's chunk c, or, for the last lane, lane 0's NEXT chunk.  `vec` is the same
            // for all lanes of the group, so the group takes the shuffles together.
            if (vec) {
                uint32_t h[EPL / 2];
#pragma unroll
                for (int q = 0; q < EPL / 2; ++q) {
                    const float lo16 = fmaf(acc[2 * q], mm, bm), hi16 = fmaf(acc[2 * q + 1], mm, bm);
                    if (p.out_ty == TBE_B200_FP16) {
                        const __half2 hh = __floats2half2_rn(lo16, hi16);
                        h[q] = *reinterpret_cast<const uint32_t*>(&hh);
                    } else {
                        const __nv_bfloat162 bb = __floats2bfloat162_rn(lo16, hi16);
                        h[q] = *reinterpret_cast<const uint32_t*>(&bb);
                    }
                }
                const int from = (k + 1 == nunits) ? 0 : k + 1;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const int cn = (c + 1) % NCH;
                    const uint32_t s0 = (k == 0) ? h[8 * cn] : h[8 * c];
                    const uint32_t s1 = (k == 0) ? h[8 * cn + 1] : h[8 * c + 1];
                    const uint32_t up0 = __shfl_sync(gmask, s0, from, LPR);
                    const uint32_t up1 = __shfl_sync(gmask, s1, from, LPR);
                    if (act) {
                        char* dst = seg + 32 * (k + c * nunits);
                        st_stream16(dst, make_uint4(h[8 * c + 2], h[8 * c + 3], h[8 * c + 4], h[8 * c + 5]));
                        st_stream16(dst + 16, make_uint4(h[8 * c + 6], h[8 * c + 7], up0, up1));
                    }
                }
                stored = true;
            }
        }
        if (!stored && act) {
#pragma unroll
            for (int q = 0; q < EPL / 4; ++q) {
                float v[4];
#pragma unroll
                for (int s = 0; s < 4; ++s) v[s] = fmaf(acc[4 * q + s], mm, bm);
                store_out<4>(seg, elem_of(4 * q), v, p.out_ty, vec);
            }
        }
    };
    // Hands this group's piece of a bag that started in an earlier group's range to that bag's owner.
    auto write_partial = [&]() {
#pragma unroll
        for (int q = 0; q < EPL / 4; ++q)
            sts16(wsm + static_cast<uint32_t>(q * kWarp + lane) * 16u, acc[4 * q + 0] + bias_acc, acc[4 * q + 1] + bias_acc,
                  acc[4 * q + 2] + bias_acc, acc[4 * q + 3] + bias_acc);
    };
    // Finishes every bag that ends at the group's position (the one being summed, then the empty ones after it).
    auto drain = [&]() {
        while (pos == bag_end) {
            if constexpr (FOLD) {
                bias_acc = fmaf(-1024.0f, scale_acc, bias_acc);
                scale_acc = 0.0f;
            }
            if (bag_start < lo) write_partial();
            else store_bag(cur, bag_end - bag_start);
#pragma unroll
            for (int s = 0; s < EPL; ++s) acc[s] = 0.0f;
            bias_acc = 0.0f;
            ++cur;
            bag_start = bag_end;
            bag_end = (cur < nb) ? lds4i(sm_rel + 4 * (cur + 1)) : -1;
        }
    };
    drain();

    // Index stream of the group: lane k reads the index (and weight) of row c * LPR + k of the range (chunk c).
    const char* ipb = static_cast<const char*>(p.indices) + (R0 + lo + k) * isz;
    const float* wpb = WEIGHTED ? p.pw + R0 + lo + k : nullptr;
    // The index is kept exactly as loaded (one or two 32-bit words; nothing is computed from it before `narrow` looks
    // at it two chunks later: even a sign extension right after the load would make the warp wait for the load).
    auto load_raw = [&](int c, uint2& raw, float& w) {
        raw = make_uint2(0xffffffffu, 0xffffffffu);
        w = 0.0f;
        if (lo + c * LPR + k < hi) {
            const char* ip = ipb + static_cast<int64_t>(c) * (LPR * isz);
            if (idx64) raw = ld_once_2x32(ip);
            else raw.x = static_cast<uint32_t>(ld_once32(ip));
            if constexpr (WEIGHTED) w = ld_once_f32(wpb + c * LPR);
        }
    };
    // Row number narrowed to 32 bits; -1 = nothing to add.  A row outside [-1, 2^31) or past the end of the
    // table is reported and skipped.  `max_rows` (once per run) folds both limits into one unsigned compare.
    const uint64_t rows_avail = static_cast<uint64_t>(m.avail) / stride;
    const uint64_t max_rows = rows_avail < 0x80000000ull ? rows_avail : 0x80000000ull;
    auto narrow = [&](uint2 words) -> int32_t {
        const int64_t raw = idx64 ? static_cast<int64_t>((static_cast<uint64_t>(words.y) << 32) | words.x)
                                  : static_cast<int64_t>(static_cast<int32_t>(words.x));
        if (static_cast<uint64_t>(raw) >= max_rows) {          // -1 and every other negative number included
            if (raw != -1 && p.error_flag) atomicOr(p.error_flag, (raw < 0 || raw > 0x7fffffffll) ? 1 : 4);
            return -1;
        }
        return static_cast<int32_t>(raw);
    };

    // The ring of rows in flight: stage s holds one row per group; a lane copies and reads back its own chunk(s)
    // only (chunk c of lane l at (c * 32 + l) * 16), the header lane also the group's tail word.
#ifdef TBE_L2_HINTS
    const uint64_t row_policy = l2_policy_evict_last();
#endif
    const uint32_t ring = wsm + kPartBytes + kRelBytes;
    const uint32_t my_main = ring + static_cast<uint32_t>(lane) * CH;   // chunk c of lane l at (c * 32 + l) * CH
    const uint32_t my_tail = ring + kWarp * LANEB + static_cast<uint32_t>(g) * 4u;
    // Requests row `idx` of the table into stage `st` (byte offset): asynchronous copies through L1, zero-filled
    // without reading for a row that is not to be added.
    auto request = [&](uint32_t st, int32_t idx) {
        const bool ok = act && idx >= 0;   // the lanes past the row's last unit zero-fill their slots as well
        const uint8_t* src = ok ? lane_base + static_cast<uint64_t>(static_cast<uint32_t>(idx)) * stride : zero_base;
        const int sz = ok ? CH : 0;
        if constexpr (CH == 8) {
            cp_async8(my_main + st, src, sz);
        } else {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
#ifdef TBE_L2_HINTS
                cp_async16_ca_hint(my_main + st + c * (kWarp * 16), src + c * chunk_step, sz, row_policy);
#else
                cp_async16_ca(my_main + st + c * (kWarp * 16), src + c * chunk_step, sz);
#endif
            }
        }
        if constexpr (kHdr) {
            if (head_lane) cp_async4(my_tail + st, src + tail_off, ok ? 4 : 0);   // (zero_base + tail_off is still inside the zeros)
        }
        cp_async_commit();
    };
    // Adds the row in stage `st`, with weight w.
    auto consume = [&](uint32_t st, float w) {
        constexpr int NW = LANEB / 4;      // 32-bit words of the row in this lane
        uint32_t r[NW];
        if constexpr (CH == 8) {
            const uint2 v = lds8(my_main + st);
            r[0] = v.x;
            r[1] = v.y;
        } else {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const uint4 v = lds16(my_main + st + c * (kWarp * 16));
                r[4 * c + 0] = v.x;
                r[4 * c + 1] = v.y;
                r[4 * c + 2] = v.z;
                r[4 * c + 3] = v.w;
            }
        }
        if constexpr (kHdr) {
            const uint32_t hdr = __shfl_sync(kFull, r[0], 0, LPR);   // zero for a row that was not copied
            if (head_lane) r[0] = lds4(my_tail + st);                // the header lane's first HS slots: the row's tail
            float ws;
            const unsigned short scale_h = accum_header<WEIGHTED, FOLD>(hdr, w, ws, bias_acc, scale_acc);
            accum_codes<TY, WEIGHTED, FOLD, NW>(r, scale_h, ws, acc);
        } else if constexpr (TY == TBE_B200_FP8) {
            // byte -> fp32 by bit placement: ((b & 0x7f) << (16 + ebits)) as a float, times 2^(127 - bias),
            // sign bit or'ed in (reference: c310/op_kernel/common.h:120-167)
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
#pragma unroll
                for (int b4 = 0; b4 < 4; ++b4) {
                    const uint32_t by = (r[i4] >> (8 * b4)) & 0xffu;
                    const float mag = __uint_as_float((by & 0x7fu) << p.fp8_shift) * p.fp8_mult;
                    const float val = __uint_as_float(__float_as_uint(mag) | ((by & 0x80u) << 24));
                    acc[4 * i4 + b4] = fmaf(w, val, acc[4 * i4 + b4]);
                }
            }
        } else if constexpr (TY == TBE_B200_FP16) {
            // unweighted: value * 1.0 + acc in one mixed FMA
#pragma unroll
            for (int i8 = 0; i8 < 8; ++i8) add_pair_t<WEIGHTED>(acc[2 * i8], acc[2 * i8 + 1], r[i8], 0x3c00u, w);
        } else {
#pragma unroll
            for (int s = 0; s < 16; ++s) acc[s] = fmaf(w, __uint_as_float(r[s]), acc[s]);
        }
    };

    // Step q requests row q of the range and consumes row q - NS (copied NS steps ago into the same stage), so NS rows
    // per group are in flight; rows per .. per + NS - 1 do not exist and only drain the ring.  The step loop is kept
    // rolled on purpose: unrolled over the stages (constant stage addresses, one copy of the end-of-bag code per stage)
    // it measured 5-10 % slower, and twice as slow with eight stages -- the loop no longer fits the instruction cache.
    const int total = per + NS;
    uint2 raw_a, raw_b;                    // the indices of the next chunk and of the one after it, as loaded
    float w_a = 0.0f, w_b = 0.0f;
    int32_t idx_c;                         // lane k: index of row c * LPR + k of the chunk being requested
    float w_c = 0.0f, w_prev = 0.0f;       // weights of the chunk being requested / of the one before it
    {
        uint2 raw0;
        load_raw(0, raw0, w_c);
        load_raw(1, raw_a, w_a);
        load_raw(2, raw_b, w_b);
        idx_c = narrow(raw0);
        if (idx_c < 0) w_c = 0.0f;
    }
    int q = 0;
#pragma unroll 1
    for (int c = 0; q < total; ++c) {
        if (c > 0) {
            w_prev = w_c;
            idx_c = narrow(raw_a);
            w_c = (idx_c >= 0) ? w_a : 0.0f;
            raw_a = raw_b;
            w_a = w_b;
            load_raw(c + 2, raw_b, w_b);
        }
        const int u_end = min(LPR, total - q);
#pragma unroll 1
        for (int u = 0; u < u_end; ++u, ++q) {
            const uint32_t st = static_cast<uint32_t>(q & (NS - 1)) * STAGE;
            if (q >= NS) {
                float w = 1.0f;
                if constexpr (WEIGHTED) w = __shfl_sync(kFull, u >= NS ? w_c : w_prev, (u - NS) & (LPR - 1), LPR);
                cp_async_wait<NS - 1>();
                consume(st, w);
                pos = min(pos + 1, hi);
                if (pos == bag_end) drain();
            }
            request(st, __shfl_sync(kFull, idx_c, u, LPR));
        }
        if constexpr (FOLD) {
            since_fold += u_end;
            if (since_fold + LPR > 32) {
#pragma unroll
                for (int s = 0; s < EPL; ++s) acc[s] = fmaf(-1024.0f, scale_acc, acc[s]);
                scale_acc = 0.0f;
                since_fold = 0;
            }
        }
    }
    cp_async_wait<0>();                    // nothing of this run is still on its way when the ring is handed on

    // A bag that the range ended in the middle of: a piece for its owner, or, when it started in this range, the
    // owner's own piece, completed with the pieces of the groups after it.
    const bool open = active && bag_end >= 0 && bag_start < pos && pos < bag_end;
    if (open) {
        if constexpr (FOLD) {
            bias_acc = fmaf(-1024.0f, scale_acc, bias_acc);
            scale_acc = 0.0f;
        }
        if (bag_start < lo) write_partial();
    }
    __syncwarp();
    if (open && bag_start >= lo) {
        for (int gg = g + 1; gg < G && gg * per < bag_end; ++gg) {
#pragma unroll
            for (int q = 0; q < EPL / 4; ++q) {
                const float4 v = lds16f(wsm + static_cast<uint32_t>(q * kWarp + gg * LPR + k) * 16u);
                acc[4 * q + 0] += v.x;
                acc[4 * q + 1] += v.y;
                acc[4 * q + 2] += v.z;
                acc[4 * q + 3] += v.w;
            }
        }
        store_bag(cur, bag_end - bag_start);
    }
}

template <int TY, bool WEIGHTED, bool FOLD>
__device__ __forceinline__ void pool_run_stream_by_width(const LookupParams& p, const TableMeta& m, int64_t i0, int nb, int64_t b,
                                                         int lane, uint32_t wsm)
{
    // INT8 / INT4 rows of 128 elements or more that divide into 32-element pieces: 32 elements per lane, so that twice
    // as many bags share a warp and the per-row work that does not depend on the width is shared twice as widely.
    if constexpr (TY == TBE_B200_INT8 || TY == TBE_B200_INT4) {
        if (m.D >= 128 && (m.D & 31) == 0) {
            const int n32 = m.D / 32;
            if (n32 <= 4) pool_run_stream<TY, 4, 32, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
            else if (n32 <= 8) pool_run_stream<TY, 8, 32, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
            else pool_run_stream<TY, 16, 32, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
            return;
        }
    }
    const int nunits = m.D / 16;
    if (nunits <= 4) pool_run_stream<TY, 4, 16, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
    else if (nunits <= 8) pool_run_stream<TY, 8, 16, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
    else if (nunits <= 16) pool_run_stream<TY, 16, 16, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
    else pool_run_stream<TY, 32, 16, WEIGHTED, FOLD>(p, m, i0, nb, b, lane, wsm);
}

template <bool WEIGHTED>
__device__ __forceinline__ void pool_run_stream_by_type(const LookupParams& p, const TableMeta& m, int64_t i0, int nb, int64_t b,
                                                        int lane, uint32_t wsm)
{
    switch (m.ty) {
        case TBE_B200_INT8:
            if constexpr (!WEIGHTED) {
                if (p.out_ty != TBE_B200_FP32) {
                    pool_run_stream_by_width<TBE_B200_INT8, false, true>(p, m, i0, nb, b, lane, wsm);
                    return;
                }
            }
            pool_run_stream_by_width<TBE_B200_INT8, WEIGHTED, false>(p, m, i0, nb, b, lane, wsm);
            return;
        case TBE_B200_INT4: pool_run_stream_by_width<TBE_B200_INT4, WEIGHTED, false>(p, m, i0, nb, b, lane, wsm); return;
        case TBE_B200_FP8: pool_run_stream_by_width<TBE_B200_FP8, WEIGHTED, false>(p, m, i0, nb, b, lane, wsm); return;
        case TBE_B200_FP16: pool_run_stream_by_width<TBE_B200_FP16, WEIGHTED, false>(p, m, i0, nb, b, lane, wsm); return;
        default: pool_run_stream_by_width<TBE_B200_FP32, WEIGHTED, false>(p, m, i0, nb, b, lane, wsm); return;
    }
}


// A run of bags of one table through the general per-bag code.
template <typename IdxT, bool STAGING>
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
        bag.avail = m.avail;
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
        if (STAGING && m.rows_aligned && (m.D & 3) == 0 && L >= 0 && start >= 0 && end <= p.num_indices) {
            const BagHead head = load_batch<IdxT>(indices + start, p.pw ? p.pw + start : nullptr, min(L, kWarp), lane, p.error_flag,
                                                  m.stride, m.avail);
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
        if (!done) {
            // positions outside `indices` are not read: the bag is written as if it were empty, and reported
            const bool sane = L >= 0 && start >= 0 && end <= p.num_indices;
            if (!sane && lane == 0 && p.error_flag) atomicOr(p.error_flag, 8);
            pool_bag_bytewise<IdxT>(indices + start, p.pw ? p.pw + start : nullptr, p.error_flag, bag.table, bag.stride, sane ? L : 0,
                                    m.D, bag.seg, bag.mean_mul, m.ty, p.out_ty, p.fp8_shift, p.fp8_mult, lane, m.avail);
        }
        start = end;
    }
}

// ---- kernels -----------------------------------------------------------------

// Warps per block.  With 8 (two blocks per SM) or 16 (one) the warps of an SM work on fewer tables at a time, which
// helps launches whose tables differ in type or width (their loops compete for the instruction cache): measured
// +4.5 % / +2.7 % on benchmark configuration 3 and +1.6 % / +0.4 % on configuration 5, but -0.9 % / -4.6 % on the
// single-shape configuration 4 (a finished block leaves its SM emptier for longer), so 4 it is.
#ifndef TBE_WARPS_PER_BLOCK
#define TBE_WARPS_PER_BLOCK 4
#endif
constexpr int kWarpsPerBlock = TBE_WARPS_PER_BLOCK;
#ifndef TBE_SPAN_LARGE
#define TBE_SPAN_LARGE 31
#endif
#ifndef TBE_STREAM_BLOCKS_PER_SM
#define TBE_STREAM_BLOCKS_PER_SM (16 / TBE_WARPS_PER_BLOCK)   // 16 resident warps per SM at up to 128 registers (32 accumulators per lane); measured best
#endif
constexpr int kStreamBlocksPerSM = TBE_STREAM_BLOCKS_PER_SM;
constexpr int kWideBlocksPerSM = 32 / TBE_WARPS_PER_BLOCK;

// The T*B bags (bag i = t*B + b) are cut into spans of `span` consecutive bags, one span per warp, so a
// warp walks `offsets`, `indices` and the per-sample weights front to back.  A span is processed as runs
// of consecutive bags of one table: the table's description is read once per run and the run is handed
// to the code specialised for its row shape.
// Two builds of the kernel share this outline.  WIDE = false is the one for the common shapes: every table with
// aligned rows of D = 16 * n <= 512 elements goes through the register streams (little shared memory, so most of
// the SM's memory is L1 for the hot rows), anything else through the byte-wise path.  WIDE = true is launched when
// the widest table has more than 512 elements or a width that is not a multiple of 16: aligned shapes use the
// cp.async staging of pool_bag there.
template <typename IdxT, bool WIDE>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp, WIDE ? kWideBlocksPerSM : kStreamBlocksPerSM)
tbe_pooled_kernel(const __grid_constant__ LookupParams p)
{
    constexpr int kSmemPerWarp = WIDE ? kWarpSmemBytes : kStreamSmemBytes;
    extern __shared__ __align__(128) uint8_t smem[];      // kWarpsPerBlock * kSmemPerWarp bytes, given at launch
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t wsm = smem_u32(smem) + warp * kSmemPerWarp;
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
    // The last offset has to be the number of indices (the reference kernel asserts the same:
    // c310/op_kernel/int_nbit_split_embedding_pooling_kernel.h:149-150); here it is reported, not trapped.
    if (gw == 0 && lane == 0 && p.error_flag) {
        if (static_cast<int64_t>(static_cast<const IdxT*>(p.offsets)[p.num_bags]) != p.num_indices) atomicOr(p.error_flag, 8);
    }

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
            bool done = false;
            if constexpr (!WIDE) {
                const bool stream = m.rows_aligned && (m.D & 15) == 0 && m.D <= 512 && m.stride < (1ll << 32) &&
                                    (m.ty == TBE_B200_INT8 || m.ty == TBE_B200_INT4 || m.ty == TBE_B200_FP8 ||
                                     m.ty == TBE_B200_FP16 || m.ty == TBE_B200_FP32);
                if (stream) {
                    const int nb = static_cast<int>(run_end - i);   // <= span <= kMaxRunBags
                    if (weighted) pool_run_stream_by_type<true>(p, m, i, nb, b, lane, wsm);
                    else pool_run_stream_by_type<false>(p, m, i, nb, b, lane, wsm);
                    done = true;
                }
            }
            if (!done) pool_run_general<IdxT, WIDE>(p, m, i, run_end, b, lane, wsm);
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
    const bool bad = idx < -1 || idx > 0x7fffffffll;
    const bool past = !bad && idx >= 0 && static_cast<uint64_t>(idx + 1) * static_cast<uint64_t>(m.stride) > static_cast<uint64_t>(m.avail);
    if (idx < 0 || bad || past) {
        if ((bad || past) && lane == 0 && p.error_flag) atomicOr(p.error_flag, bad ? 1 : 4);
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

// Four consecutive output elements of a row image in shared memory (e0 a multiple of 4).
__device__ __forceinline__ void stage_out4(uint8_t* row_image, int e0, const float* v, int out_ty)
{
    if (out_ty == TBE_B200_FP32) {
        *reinterpret_cast<float4*>(row_image + e0 * 4) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = (out_ty == TBE_B200_FP16) ? f32_to_f16_bits(v[j]) : f32_to_bf16_bits(v[j]);
        *reinterpret_cast<uint2*>(row_image + e0 * 2) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    }
}

constexpr int kNobagStageBytes = 2048;   // the G rows of one step: at most 512 elements of 4 bytes

// `cnt` consecutive positions [n, n + cnt) of one table with aligned rows of D = 16 * units <= 512 elements.
// A lane's 16 decoded elements start 4 (INT8) or 8 (INT4) elements before a 16-element boundary, so stored from
// registers they are 8-byte pieces 32 bytes apart: every 32-byte sector of the output -- which is larger than the
// input here -- is written in part by several instructions.  With a 16-byte aligned output the G rows of a step are
// put together in the warp's `stage` area and leave as whole 16-byte pieces, consecutive from lane to lane.
template <int TY, int LPR, typename IdxT>
__device__ __forceinline__ void nobag_rows(const LookupParams& p, const TableMeta& m, const IdxT* indices, int64_t n, int cnt, int max_D,
                                           int lane, uint8_t* stage)
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
    const int row_out_bytes = D * esz, pieces_per_row = row_out_bytes / 16;
    const int piece_shift = (pieces_per_row & (pieces_per_row - 1)) == 0 ? __ffs(pieces_per_row) - 1 : -1;   // power of two: no division
    const bool staged = (reinterpret_cast<uintptr_t>(p.output) & 15) == 0 && (p.out_stride * esz) % 16 == 0;   // warp-uniform
    // The warp's positions are narrowed and checked once (lane l holds positions l and l + 32), then taken U steps of
    // G rows at a time: the row loads of all U steps are issued before the first row is decoded, so U * G rows per warp
    // are in flight instead of G.
    constexpr int U = (NCH == 1) ? 4 : (NCH == 2 ? 2 : 1);
    auto checked = [&](int pos) -> int32_t {
        if (pos >= cnt) return -1;
        int64_t idx = static_cast<int64_t>(__ldg(indices + n + pos));
        if ((idx < -1 || idx > 0x7fffffffll) && p.error_flag) atomicOr(p.error_flag, 1);
        if (idx > 0x7fffffffll || idx < 0) return -1;
        if (static_cast<uint64_t>(idx + 1) * static_cast<uint64_t>(m.stride) > static_cast<uint64_t>(m.avail)) {
            if (p.error_flag) atomicOr(p.error_flag, 4);
            return -1;
        }
        return static_cast<int32_t>(idx);
    };
    const int32_t idx_lo = checked(lane), idx_hi = checked(lane + 32);
    for (int r0 = 0; r0 < cnt; r0 += G * U) {
        uint32_t words_u[U][4 * NCH];
        uint32_t tail_u[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pos = r0 + u * G + g;
            const int32_t a = __shfl_sync(kFull, idx_lo, pos & 31), b = __shfl_sync(kFull, idx_hi, pos & 31);
            const int32_t idx = pos < 32 ? a : (pos < 64 ? b : -1);
            const bool ok = idx >= 0;
            const uint8_t* row = m.table + static_cast<int64_t>(ok ? idx : 0) * m.stride;
#pragma unroll
            for (int c = 0; c < 4 * NCH; ++c) words_u[u][c] = 0u;
            tail_u[u] = 0u;
            if (ok && active) {
                if constexpr (TY == TBE_B200_INT4) {
                    const uint2 v = ldg8(row + k * 8);
                    words_u[u][0] = v.x; words_u[u][1] = v.y;
                } else {
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        const uint4 v = ldg16(row + 16 * (k + c * nunits));
                        words_u[u][4 * c + 0] = v.x; words_u[u][4 * c + 1] = v.y; words_u[u][4 * c + 2] = v.z; words_u[u][4 * c + 3] = v.w;
                    }
                }
                if (head_lane) tail_u[u] = ldg4(row + (k8 ? D : D / 2));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
        const uint32_t* words = words_u[u];
        const uint32_t tail = tail_u[u];
        const int pos = r0 + u * G + g;
        const bool mine = pos < cnt;
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
        if (staged) {
            if (active) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int slot = 4 * q;
                    int e0;
                    if constexpr (kHdr) e0 = (head_lane && slot < HS) ? (D - HS + slot) : (16 * k - HS + slot);
                    else e0 = EPC * (k + (slot / EPC) * nunits) + (slot % EPC);
                    stage_out4(stage + g * row_out_bytes, e0, &v[slot], p.out_ty);
                }
            }
            __syncwarp();
            for (int c = lane; c < G * pieces_per_row; c += kWarp) {
                const int row = piece_shift >= 0 ? (c >> piece_shift) : c / pieces_per_row, piece = c - row * pieces_per_row;
                const int rpos = r0 + u * G + row;
                if (rpos < cnt)
                    st_stream16(static_cast<char*>(p.output) + (n + rpos) * p.out_stride * esz + 16 * piece,
                                *reinterpret_cast<const uint4*>(stage + row * row_out_bytes + 16 * piece));
            }
            __syncwarp();
            if (mine) {
                char* seg = static_cast<char*>(p.output) + (n + pos) * p.out_stride * esz;
                for (int e = D + k; e < max_D; e += LPR) store_scalar(seg, e, 0.0f, p.out_ty);
            }
        } else if (mine) {
            char* seg = static_cast<char*>(p.output) + (n + pos) * p.out_stride * esz;
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
}

template <int TY, typename IdxT>
__device__ __forceinline__ void nobag_rows_by_width(const LookupParams& p, const TableMeta& m, const IdxT* indices, int64_t n, int cnt,
                                                    int max_D, int lane, uint8_t* stage)
{
    const int nunits = m.D / 16;
    if (nunits <= 4) nobag_rows<TY, 4, IdxT>(p, m, indices, n, cnt, max_D, lane, stage);
    else if (nunits <= 8) nobag_rows<TY, 8, IdxT>(p, m, indices, n, cnt, max_D, lane, stage);
    else if (nunits <= 16) nobag_rows<TY, 16, IdxT>(p, m, indices, n, cnt, max_D, lane, stage);
    else nobag_rows<TY, 32, IdxT>(p, m, indices, n, cnt, max_D, lane, stage);
}

template <typename IdxT>
__global__ void __launch_bounds__(kWarpsPerBlock* kWarp)
tbe_nobag_kernel(const __grid_constant__ LookupParams p, int64_t num_indices, int max_D)
{
    __shared__ __align__(16) uint8_t stage_all[kWarpsPerBlock][kNobagStageBytes];
    uint8_t* stage = stage_all[threadIdx.x >> 5];
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
                case TBE_B200_INT8: nobag_rows_by_width<TBE_B200_INT8, IdxT>(p, m, indices, n, cnt, max_D, lane, stage); break;
                case TBE_B200_INT4: nobag_rows_by_width<TBE_B200_INT4, IdxT>(p, m, indices, n, cnt, max_D, lane, stage); break;
                case TBE_B200_FP8: nobag_rows_by_width<TBE_B200_FP8, IdxT>(p, m, indices, n, cnt, max_D, lane, stage); break;
                case TBE_B200_FP16: nobag_rows_by_width<TBE_B200_FP16, IdxT>(p, m, indices, n, cnt, max_D, lane, stage); break;
                case TBE_B200_FP32: nobag_rows_by_width<TBE_B200_FP32, IdxT>(p, m, indices, n, cnt, max_D, lane, stage); break;
                default: done = false; break;
            }
        }
        if (!done)
            for (int64_t q = n; q < stop; ++q) nobag_position_bytewise<IdxT>(p, m, indices, q, max_D, lane);
        n = stop;
    }
}

constexpr int kSpanLarge = TBE_SPAN_LARGE;   // bags per warp when there is plenty of work: the more, the fewer bags straddle lane groups

// Blocks of a kernel that fit on one SM of the current device (occupancy query, once per device and kernel).
template <typename Kernel>
int resident_blocks(Kernel kernel, int variant, int fallback, int smem_bytes = 0)
{
    constexpr int kMaxDev = 64, kVariants = 4;
    static std::atomic<int> cached[kMaxDev][kVariants];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return fallback;
    int n = cached[dev][variant].load(std::memory_order_relaxed);
    if (n == 0) {
        if (smem_bytes > 48 * 1024) (void)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kWarpsPerBlock * kWarp, smem_bytes) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = fallback;
        }
        cached[dev][variant].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Environment switches, read once: TBE_B200_L2_POLICY (0 = nothing, the default; 2 = access-policy window, see
// apply_l2_window) and TBE_B200_SPAN (bags per warp, for experiments; 0 = automatic).
int env_int(const char* name, int dflt)
{
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}
int l2_policy_mode()
{
    static const int mode = env_int("TBE_B200_L2_POLICY", 0);
    return mode;
}

// TBE_B200_L2_POLICY=2: an access-policy window over dev_weights on the caller's stream, with part of L2 set aside for
// persisting lines (per-context state that ends with the process).  Off by default: the hot rows of a table are
// scattered over it, so the window cannot single them out (it keeps a random fraction of the table's lines), and it
// measured 3-6 % slower with the L2 hit rate unchanged.
void apply_l2_window(const void* base, int64_t bytes, cudaStream_t s)
{
    static std::atomic<int> prepared[64];
    int dev = 0;
    if (bytes <= 0 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    int max_window = 0, max_persist = 0;
    cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev);
    cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev);
    if (max_window <= 0 || max_persist <= 0) return;
    if (prepared[dev].exchange(1) == 0) (void)cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, static_cast<size_t>(max_persist));
    cudaStreamAttrValue attr{};
    const size_t win = static_cast<size_t>(bytes < max_window ? bytes : max_window);
    attr.accessPolicyWindow.base_ptr = const_cast<void*>(base);
    attr.accessPolicyWindow.num_bytes = win;
    const float ratio = static_cast<float>(max_persist) / static_cast<float>(win);
    attr.accessPolicyWindow.hitRatio = ratio < 1.0f ? ratio : 1.0f;
    attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    (void)cudaStreamSetAttribute(s, cudaStreamAttributeAccessPolicyWindow, &attr);
    (void)cudaGetLastError();
}
int forced_span()
{
    static const int span = env_int("TBE_B200_SPAN", 0);
    return span;
}

template <typename IdxT, bool WIDE>
int launch_pooled(LookupParams p, cudaStream_t s)
{
    constexpr int kSmemBytes = kWarpsPerBlock * (WIDE ? kWarpSmemBytes : kStreamSmemBytes);
    const int resident = resident_blocks(tbe_pooled_kernel<IdxT, WIDE>, (sizeof(IdxT) == 8 ? 2 : 0) + (WIDE ? 1 : 0),
                                         WIDE ? kWideBlocksPerSM : kStreamBlocksPerSM, kSmemBytes);
    // Plenty of bags: fixed spans, as many blocks as that takes; the hardware block scheduler evens out the load.
    // Otherwise the spans are sized so that the warps fill a whole number of waves of resident warps.
    const int64_t slots = static_cast<int64_t>(sm_count()) * resident * kWarpsPerBlock;
    const int64_t waves = (p.num_bags + slots * kSpanLarge - 1) / (slots * kSpanLarge);
    if (waves >= 4) {
        p.span = kSpanLarge;
    } else {
        const int64_t per = (p.num_bags + slots * waves - 1) / (slots * waves);
        p.span = per < 1 ? 1 : (per > kSpanLarge ? kSpanLarge : per);
    }
    const int fs = forced_span();
    if (fs > 0) p.span = fs > kMaxRunBags ? kMaxRunBags : fs;
    const int64_t warps = (p.num_bags + p.span - 1) / p.span;
    const int64_t blocks = (warps + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "lookup: too many bags for one launch");
    tbe_pooled_kernel<IdxT, WIDE><<<static_cast<unsigned>(blocks), kWarpsPerBlock * kWarp, kSmemBytes, s>>>(p);
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
    p.dev_weights_bytes = a->dev_weights_bytes > 0 ? a->dev_weights_bytes : 0;
    p.idx64 = a->index_bits == 64 ? 1 : 0;
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
    if (l2_policy_mode() == 2) apply_l2_window(a->dev_weights, a->dev_weights_bytes, s);
    // The widest table decides which build of the kernel runs (max_D is the caller's, like the reference's max_*_D).
    const bool wide = a->max_D > 512 || (a->max_D & 15) != 0;
    if (a->index_bits == 32) return wide ? launch_pooled<int32_t, true>(p, s) : launch_pooled<int32_t, false>(p, s);
    return wide ? launch_pooled<int64_t, true>(p, s) : launch_pooled<int64_t, false>(p, s);
}
