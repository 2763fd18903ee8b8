// Rowwise quantizers / dequantizers and table-row packing for B200.
//
//   FloatToFused8BitRowwiseQuantized / Fused8BitRowwiseQuantizedToFloat
//   FloatToFusedNBitRowwiseQuantizedSBHalf / FusedNBitRowwiseQuantizedSBHalfToFloat
//
// These operators are not defined in the reference tree; it inherits them from
// fbgemm_gpu (fbgemm_ascend/__init__.py:9).  Their byte layout must be bit-exact,
// so the arithmetic below is written without fused multiply-adds where the CPU
// definition has none, with IEEE division, and with round-to-nearest-even.
//
// All kernels are HBM-bound streaming passes: a group of LPR lanes owns a row,
// finds min/max with shuffles (first pass over the row), then re-reads the row
// (L1/L2-resident by then) and writes the codes.
#include "tbe_common.cuh"

namespace tbe {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kThreads = 256;

template <typename InT>
__device__ __forceinline__ float load_in(const InT* p);
template <>
__device__ __forceinline__ float load_in<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_in<__half>(const __half* p) { return __half2float(__ldg(p)); }

// Writes the 4-byte row header (two fp16 bit patterns) at `o`.  `h` is first pinned in a 32-bit
// register: byte stores fed straight from the 16-bit result of the float->half conversion came out
// with a zero low byte on sm_100a (CUDA 12.9), while the same stores from a 32-bit value are correct.
__device__ __forceinline__ void store_header(uint8_t* o, uint32_t lo16, uint32_t hi16)
{
    uint32_t h = (lo16 & 0xffffu) | (hi16 << 16);
    asm volatile("" : "+r"(h));
    if ((reinterpret_cast<uintptr_t>(o) & 3) == 0) {
        *reinterpret_cast<uint32_t*>(o) = h;
    } else {
        o[0] = static_cast<uint8_t>(h & 0xffu);
        o[1] = static_cast<uint8_t>((h >> 8) & 0xffu);
        o[2] = static_cast<uint8_t>((h >> 16) & 0xffu);
        o[3] = static_cast<uint8_t>(h >> 24);
    }
}

template <int LPR>
__device__ __forceinline__ void group_minmax(float& mn, float& mx)
{
#pragma unroll
    for (int d = LPR / 2; d >= 1; d >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(kFull, mn, d));
        mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, d));
    }
}

// Row min/max over D elements, LPR lanes per row.  The comparisons reproduce a
// sequential `if (x < mn) mn = x` scan for finite inputs.
template <int LPR, typename InT>
__device__ __forceinline__ void row_minmax(const InT* x, int64_t D, int k, bool vec4, float& mn, float& mx)
{
    mn = __int_as_float(0x7f800000);
    mx = __int_as_float(0xff800000);
    if (vec4) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int64_t v = k; v < D / 4; v += LPR) {
            const float4 f = __ldg(x4 + v);
            mn = fminf(fminf(mn, f.x), fminf(f.y, fminf(f.z, f.w)));
            mx = fmaxf(fmaxf(mx, f.x), fmaxf(f.y, fmaxf(f.z, f.w)));
        }
    } else {
        for (int64_t c = k; c < D; c += LPR) {
            const float f = load_in<InT>(x + c);
            mn = fminf(mn, f);
            mx = fmaxf(mx, f);
        }
    }
    group_minmax<LPR>(mn, mx);
    if (D == 0) { mn = 0.0f; mx = 0.0f; }
}

// ---- 8-bit -------------------------------------------------------------------
//
// TABLE == false: out row = [D codes][fp32 scale][fp32 bias], stride D + 8.
// TABLE == true : out row = [fp16 scale][fp16 bias][D codes], stride row_bytes
//                 (the table-batched layout), padding zeroed.
template <int LPR, typename InT, bool TABLE>
__global__ void __launch_bounds__(kThreads)
quantize_8bit_kernel(const InT* __restrict__ in, int64_t N, int64_t D, uint8_t* __restrict__ out, int64_t out_stride)
{
    constexpr int RPB = kThreads / LPR;
    const int k = threadIdx.x % LPR;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / LPR;
    // Whole groups leave together (LPR divides 32), so shuffles below stay convergent per group;
    // rows past N still run the shuffles with no memory access.
    const bool live = r < N;
    const InT* x = in + (live ? r : 0) * D;
    const bool in_vec4 = sizeof(InT) == 4 && (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    float mn, mx;
    row_minmax<LPR, InT>(x, live ? D : 0, k, in_vec4, mn, mx);
    if (!live) return;
    const float range = mx - mn;
    const float scale = __fdiv_rn(range, 255.0f);
    const float inv = __fdiv_rn(255.0f, __fadd_rn(range, 1e-8f));
    uint8_t* o = out + r * out_stride;
    uint8_t* codes = TABLE ? o + 4 : o;
    const bool out_vec4 = in_vec4 && (out_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 3) == 0);
    if (out_vec4) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int64_t v = k; v < D / 4; v += LPR) {
            const float4 f = __ldg(x4 + v);
            const uint32_t q0 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(f.x, mn), inv))) & 0xffu;
            const uint32_t q1 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(f.y, mn), inv))) & 0xffu;
            const uint32_t q2 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(f.z, mn), inv))) & 0xffu;
            const uint32_t q3 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(f.w, mn), inv))) & 0xffu;
            *reinterpret_cast<uint32_t*>(codes + 4 * v) = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
        }
    } else {
        for (int64_t c = k; c < D; c += LPR) {
            const float f = load_in<InT>(x + c);
            codes[c] = static_cast<uint8_t>(__float2int_rn(__fmul_rn(__fsub_rn(f, mn), inv)));
        }
    }
    if (TABLE) {
        if (k == 0) store_header(o, f32_to_f16_bits(scale), f32_to_f16_bits(mn));
        for (int64_t c = 4 + D + k; c < out_stride; c += LPR) o[c] = 0;
    } else if (k == 0) {
        const uint32_t sb[2] = {__float_as_uint(scale), __float_as_uint(mn)};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[D + j] = (sb[j >> 2] >> (8 * (j & 3))) & 0xff;
    }
}

// The common 8-bit shapes, batched: fp32 rows of D = 4 * n <= 512 elements, 16-byte aligned.  A warp takes ROWS
// rows at a time and keeps them in registers (VPL float4 per lane and row), so the loads of all ROWS rows are in
// flight together and nothing is read twice; a fixed grid strides over the rows.  Same arithmetic as
// quantize_8bit_kernel, hence the same bytes.
//
// STAGED (D <= 128, rows of at most kStagedStride bytes, 16-byte aligned output): the warp builds the image of its
// ROWS output rows in shared memory and writes it out as whole 16-byte pieces -- the rows of one step are contiguous
// in the output -- instead of one 4-byte store per lane and row plus separate header and padding stores.
constexpr int kStagedStride = 144;
template <bool TABLE, int VPL, int ROWS, bool STAGED = false>
__global__ void __launch_bounds__(kThreads)
quantize_8bit_batched_kernel(const float* __restrict__ in, int64_t N, int64_t D, uint8_t* __restrict__ out, int64_t out_stride)
{
    __shared__ __align__(16) uint8_t staged[STAGED ? kThreads / 32 : 1][STAGED ? ROWS * kStagedStride : 16];
    uint8_t* img = staged[STAGED ? (threadIdx.x >> 5) : 0];
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const int nvec = static_cast<int>(D / 4);
    const float4* in4 = reinterpret_cast<const float4*>(in);
    if (STAGED && TABLE) {
        // the padding behind the codes is the same for every row this warp will ever stage: cleared once
        for (int j = 0; j < ROWS; ++j)
            for (int c = 4 + static_cast<int>(D) + lane; c < static_cast<int>(out_stride); c += 32) img[j * out_stride + c] = 0;
    }
    for (int64_t r0 = warp * ROWS; r0 < N; r0 += nwarps * ROWS) {
        float4 f[ROWS][VPL];
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
            for (int v = 0; v < VPL; ++v)
                if (r0 + j < N && lane + 32 * v < nvec) f[j][v] = __ldg(in4 + (r0 + j) * nvec + lane + 32 * v);
        float mn_r[ROWS], mx_r[ROWS];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll
            for (int v = 0; v < VPL; ++v)
                if (r0 + j < N && lane + 32 * v < nvec) {
                    mn = fminf(fminf(mn, f[j][v].x), fminf(f[j][v].y, fminf(f[j][v].z, f[j][v].w)));
                    mx = fmaxf(fmaxf(mx, f[j][v].x), fmaxf(f[j][v].y, fmaxf(f[j][v].z, f[j][v].w)));
                }
            // whole-warp min / max in one instruction each (sm_100a reduces fp32 across the warp in hardware)
            asm volatile("redux.sync.min.f32 %0, %0, 0xffffffff;" : "+f"(mn));
            asm volatile("redux.sync.max.f32 %0, %0, 0xffffffff;" : "+f"(mx));
            mn_r[j] = mn;
            mx_r[j] = mx;
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            if (r0 + j >= N) continue;
            const float mn = mn_r[j];
            // (doing the two divisions of the ROWS rows in different lanes at once and handing the results round by
            // shuffle was measured 3 % slower than repeating them here)
            const float range = mx_r[j] - mn;
            const float scale = __fdiv_rn(range, 255.0f);
            const float inv = __fdiv_rn(255.0f, __fadd_rn(range, 1e-8f));
            uint8_t* o = STAGED ? img + j * out_stride : out + (r0 + j) * out_stride;
            uint8_t* codes = TABLE ? o + 4 : o;
#pragma unroll
            for (int v = 0; v < VPL; ++v)
                if (lane + 32 * v < nvec) {
                    const float4 x = f[j][v];
                    const uint32_t q0 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(x.x, mn), inv))) & 0xffu;
                    const uint32_t q1 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(x.y, mn), inv))) & 0xffu;
                    const uint32_t q2 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(x.z, mn), inv))) & 0xffu;
                    const uint32_t q3 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(x.w, mn), inv))) & 0xffu;
                    *reinterpret_cast<uint32_t*>(codes + 4 * (lane + 32 * v)) = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
                }
            if (TABLE) {
                if (STAGED) {
                    if (lane == 0) *reinterpret_cast<uint32_t*>(o) = (f32_to_f16_bits(scale) & 0xffffu) | (f32_to_f16_bits(mn) << 16);
                } else {
                    if (lane == 0) store_header(o, f32_to_f16_bits(scale), f32_to_f16_bits(mn));
                    for (int64_t c = 4 + D + lane; c < out_stride; c += 32) o[c] = 0;
                }
            } else if (lane == 0) {
                // D is a multiple of 4 and rows are 4-byte aligned here
                *reinterpret_cast<uint32_t*>(o + D) = __float_as_uint(scale);
                *reinterpret_cast<uint32_t*>(o + D + 4) = __float_as_uint(mn);
            }
        }
        if (STAGED) {
            __syncwarp();
            const int64_t rows = (N - r0 < ROWS) ? N - r0 : ROWS;
            const int bytes = static_cast<int>(rows * out_stride);
            uint8_t* dst = out + r0 * out_stride;                  // 16-byte aligned: r0 is a multiple of 4, the stride of 4
            for (int c = lane * 16; c + 16 <= bytes; c += 32 * 16)
                *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(img + c);
            for (int c = (bytes & ~15) + lane; c < bytes; c += 32) dst[c] = img[c];
            __syncwarp();
        }
    }
}

// The same for D = 8 * n <= 256 with EIGHT elements per lane: LPR lanes share a row, 32 / LPR rows per pass, four passes of
// loads in flight, so the per-row work that does not depend on the width (the two divisions, the header, the
// reduction, the bounds checks) is issued once for 32 / LPR rows instead of once per row -- the kernel is bound by
// instruction issue, not by memory.  The warp's 4 * 32 / LPR output rows are staged in shared memory and leave as whole
// 16-byte pieces.  Same arithmetic, hence the same bytes.
constexpr int kStaged8Bytes = 2304;      // 16 rows of 144 bytes
template <bool TABLE, int LPR>
__global__ void __launch_bounds__(kThreads)
quantize_8bit_wide_kernel(const float* __restrict__ in, int64_t N, int64_t D, uint8_t* __restrict__ out, int64_t out_stride)
{
    constexpr int RPP = 32 / LPR, PASSES = 4, R = RPP * PASSES;
    __shared__ __align__(16) uint8_t staged[kThreads / 32][kStaged8Bytes];
    uint8_t* img = staged[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31, k = lane % LPR, g = lane / LPR;
    const int nunits = static_cast<int>(D / 8), stride = static_cast<int>(out_stride), Di = static_cast<int>(D);
    const bool active = k < nunits;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const float4* in4 = reinterpret_cast<const float4*>(in);
    if (TABLE) {
        for (int r = 0; r < R; ++r)
            for (int c = 4 + Di + lane; c < stride; c += 32) img[r * stride + c] = 0;     // padding: cleared once
    }
    for (int64_t r0 = warp * R; r0 < N; r0 += nwarps * R) {
        float4 a[PASSES], b[PASSES];
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t row = r0 + p * RPP + g;
            if (row < N && active) {
                a[p] = __ldg(in4 + row * (2 * nunits) + 2 * k);
                b[p] = __ldg(in4 + row * (2 * nunits) + 2 * k + 1);
            }
        }
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t row = r0 + p * RPP + g;
            const bool live = row < N && active;
            float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
            if (live) {
                mn = fminf(fminf(fminf(a[p].x, a[p].y), fminf(a[p].z, a[p].w)), fminf(fminf(b[p].x, b[p].y), fminf(b[p].z, b[p].w)));
                mx = fmaxf(fmaxf(fmaxf(a[p].x, a[p].y), fmaxf(a[p].z, a[p].w)), fmaxf(fmaxf(b[p].x, b[p].y), fmaxf(b[p].z, b[p].w)));
            }
#pragma unroll
            for (int d = LPR / 2; d > 0; d >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, d));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            }
            if (!live) continue;
            const float range = mx - mn;
            const float scale = __fdiv_rn(range, 255.0f);
            const float inv = __fdiv_rn(255.0f, __fadd_rn(range, 1e-8f));
            const float x[8] = {a[p].x, a[p].y, a[p].z, a[p].w, b[p].x, b[p].y, b[p].z, b[p].w};
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j)
                w[j >> 2] |= (static_cast<uint32_t>(__float2int_rn(__fmul_rn(__fsub_rn(x[j], mn), inv))) & 0xffu) << (8 * (j & 3));
            uint8_t* o = img + (p * RPP + g) * stride;
            uint8_t* codes = (TABLE ? o + 4 : o) + 8 * k;        // 4-byte aligned (table rows) or 8-byte aligned
            *reinterpret_cast<uint32_t*>(codes) = w[0];
            *reinterpret_cast<uint32_t*>(codes + 4) = w[1];
            if (k == 0) {
                if (TABLE) {
                    *reinterpret_cast<uint32_t*>(o) = (f32_to_f16_bits(scale) & 0xffffu) | (f32_to_f16_bits(mn) << 16);
                } else {
                    *reinterpret_cast<uint32_t*>(o + Di) = __float_as_uint(scale);
                    *reinterpret_cast<uint32_t*>(o + Di + 4) = __float_as_uint(mn);
                }
            }
        }
        __syncwarp();
        const int64_t rows = (N - r0 < R) ? N - r0 : R;
        const int bytes = static_cast<int>(rows) * stride;
        uint8_t* dst = out + r0 * out_stride;                  // 16-byte aligned: r0 is a multiple of R >= 4, the stride of 4
        for (int c = lane * 16; c + 16 <= bytes; c += 32 * 16)
            *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(img + c);
        for (int c = (bytes & ~15) + lane; c < bytes; c += 32) dst[c] = img[c];
        __syncwarp();
    }
}

// 8-bit rows back to fp32, batched the same way: D = 4 * n <= 512, ROWS rows per warp in flight.
template <int VPL, int ROWS>
__global__ void __launch_bounds__(kThreads)
dequantize_8bit_batched_kernel(const uint8_t* __restrict__ in, int64_t N, int64_t Dq, float* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t D = Dq - 8;
    const int nvec = static_cast<int>(D / 4);
    for (int64_t r0 = warp * ROWS; r0 < N; r0 += nwarps * ROWS) {
        uint32_t w[ROWS][VPL];
        uint32_t sb[ROWS][2];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            if (r0 + j >= N) continue;
            const uint8_t* q = in + (r0 + j) * Dq;
#pragma unroll
            for (int v = 0; v < VPL; ++v)
                if (lane + 32 * v < nvec) w[j][v] = ldg4(q + 4 * (lane + 32 * v));
            sb[j][0] = ldg4(q + D);
            sb[j][1] = ldg4(q + D + 4);
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            if (r0 + j >= N) continue;
            const float scale = __uint_as_float(sb[j][0]), bias = __uint_as_float(sb[j][1]);
            float4* o = reinterpret_cast<float4*>(out + (r0 + j) * D);
#pragma unroll
            for (int v = 0; v < VPL; ++v)
                if (lane + 32 * v < nvec) {
                    const uint32_t x = w[j][v];
                    float4 f;
                    f.x = fmaf(static_cast<float>(x & 0xffu), scale, bias);
                    f.y = fmaf(static_cast<float>((x >> 8) & 0xffu), scale, bias);
                    f.z = fmaf(static_cast<float>((x >> 16) & 0xffu), scale, bias);
                    f.w = fmaf(static_cast<float>(x >> 24), scale, bias);
                    o[lane + 32 * v] = f;
                }
        }
    }
}

template <typename OutT>
__device__ __forceinline__ void store_deq(OutT* p, float v);
template <>
__device__ __forceinline__ void store_deq<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_deq<__half>(__half* p, float v) { *p = __float2half_rn(v); }

template <int LPR, typename OutT>
__global__ void __launch_bounds__(kThreads)
dequantize_8bit_kernel(const uint8_t* __restrict__ in, int64_t N, int64_t Dq, OutT* __restrict__ out)
{
    constexpr int RPB = kThreads / LPR;
    const int k = threadIdx.x % LPR;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / LPR;
    if (r >= N) return;
    const int64_t D = Dq - 8;
    const uint8_t* q = in + r * Dq;
    uint32_t sb[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) sb[j >> 2] |= static_cast<uint32_t>(__ldg(q + D + j)) << (8 * (j & 3));
    const float scale = __uint_as_float(sb[0]), bias = __uint_as_float(sb[1]);
    OutT* o = out + r * D;
    const bool vec = sizeof(OutT) == 4 && (Dq % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    if (vec) {
        for (int64_t v = k; v < D / 4; v += LPR) {
            const uint32_t w = ldg4(q + 4 * v);
            float4 f;
            f.x = fmaf(static_cast<float>(w & 0xffu), scale, bias);
            f.y = fmaf(static_cast<float>((w >> 8) & 0xffu), scale, bias);
            f.z = fmaf(static_cast<float>((w >> 16) & 0xffu), scale, bias);
            f.w = fmaf(static_cast<float>(w >> 24), scale, bias);
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + 4 * v) = f;
        }
    } else {
        for (int64_t c = k; c < D; c += LPR) store_deq<OutT>(o + c, fmaf(static_cast<float>(__ldg(q + c)), scale, bias));
    }
}

// ---- 2- and 4-bit ------------------------------------------------------------
//
// TABLE == false: out row = [codes][fp16 scale][fp16 bias], stride pbytes + 4.
// TABLE == true : out row = [fp16 scale][fp16 bias][codes], stride row_bytes.
template <int LPR, int BITS, bool TABLE>
__global__ void __launch_bounds__(kThreads)
quantize_nbit_kernel(const float* __restrict__ in, int64_t N, int64_t D, uint8_t* __restrict__ out, int64_t out_stride)
{
    constexpr int RPB = kThreads / LPR;
    constexpr int PER = 8 / BITS;
    constexpr int QMAX = (1 << BITS) - 1;
    const int k = threadIdx.x % LPR;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * RPB + threadIdx.x / LPR;
    const bool live = r < N;
    const float* x = in + (live ? r : 0) * D;
    const bool in_vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    float mn, mx;
    row_minmax<LPR, float>(x, live ? D : 0, k, in_vec4, mn, mx);
    if (!live) return;
    const __half bias_h = __float2half_rn(mn);
    const float bias = __half2float(bias_h);
    const float range = __fsub_rn(mx, bias);
    float scale = (range == 0.0f) ? 1.0f : __fdiv_rn(range, static_cast<float>(QMAX));
    __half scale_h = __float2half_rn(scale);
    scale = __half2float(scale_h);
    if (scale == 0.0f) {
        scale = 1.0f;
        scale_h = __float2half_rn(1.0f);
    }
    float inv = __fdiv_rn(1.0f, scale);
    if (isinf(inv)) {
        scale_h = __float2half_rn(1.0f);
        inv = 1.0f;
    }
    const int64_t pbytes = (D + PER - 1) / PER;
    uint8_t* o = out + r * out_stride;
    uint8_t* codes = TABLE ? o + 4 : o;
    for (int64_t b = k; b < pbytes; b += LPR) {
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int64_t c = b * PER + j;
            if (c < D) {
                int q = __float2int_rn(__fmul_rn(__fsub_rn(__ldg(x + c), bias), inv));
                q = max(0, min(QMAX, q));
                byte |= static_cast<uint32_t>(q) << (j * BITS);
            }
        }
        codes[b] = static_cast<uint8_t>(byte);
    }
    if (k == 0) {
        store_header(TABLE ? o : o + pbytes, __half_as_ushort(scale_h), __half_as_ushort(bias_h));
    }
    if (TABLE)
        for (int64_t c = 4 + pbytes + k; c < out_stride; c += LPR) o[c] = 0;
}

// The common 4- and 2-bit shapes, batched like the 8-bit ones: fp32 rows of D = n * 32 / BITS elements (one 32-bit word
// of codes per lane: 8 or 16 elements), 16-byte aligned input and output.  LPR lanes share a row, 32 / LPR rows per
// pass, PASSES passes of loads in flight per warp; the warp builds the image of its PASSES * 32 / LPR output rows --
// contiguous in the output -- in shared memory and writes it as whole 16-byte pieces.  Same arithmetic as
// quantize_nbit_kernel, hence the same bytes.
constexpr int kStaged4Bytes = 1280;
template <bool TABLE, int LPR, int BITS>
__global__ void __launch_bounds__(kThreads)
quantize_nbit_batched_kernel(const float* __restrict__ in, int64_t N, int64_t D, uint8_t* __restrict__ out, int64_t out_stride)
{
    constexpr int EL = 32 / BITS;                 // elements per lane and row: one word of codes
    constexpr int VL = EL / 4;                    // float4 per lane and row
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int RPP = 32 / LPR, PASSES = (BITS == 4) ? 4 : 2, R = RPP * PASSES;
    __shared__ __align__(16) uint8_t staged[kThreads / 32][kStaged4Bytes];
    uint8_t* img = staged[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31, k = lane % LPR, g = lane / LPR;
    const int nunits = static_cast<int>(D / EL), pbytes = static_cast<int>(D * BITS / 8), stride = static_cast<int>(out_stride);
    const bool active = k < nunits;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const float4* in4 = reinterpret_cast<const float4*>(in);
    if (TABLE) {
        // the padding behind the codes is the same for every row this warp will ever stage: cleared once
        for (int r = 0; r < R; ++r)
            for (int c = 4 + pbytes + lane; c < stride; c += 32) img[r * stride + c] = 0;
    }
    for (int64_t r0 = warp * R; r0 < N; r0 += nwarps * R) {
        float4 x4[PASSES][VL];
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t row = r0 + p * RPP + g;
            if (row < N && active) {
#pragma unroll
                for (int v = 0; v < VL; ++v) x4[p][v] = __ldg(in4 + row * (VL * nunits) + VL * k + v);
            }
        }
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t row = r0 + p * RPP + g;
            const bool live = row < N && active;
            float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
            if (live) {
#pragma unroll
                for (int v = 0; v < VL; ++v) {
                    mn = fminf(mn, fminf(fminf(x4[p][v].x, x4[p][v].y), fminf(x4[p][v].z, x4[p][v].w)));
                    mx = fmaxf(mx, fmaxf(fmaxf(x4[p][v].x, x4[p][v].y), fmaxf(x4[p][v].z, x4[p][v].w)));
                }
            }
#pragma unroll
            for (int d = LPR / 2; d > 0; d >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, d));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            }
            if (!live) continue;
            const __half bias_h = __float2half_rn(mn);
            const float bias = __half2float(bias_h);
            const float range = __fsub_rn(mx, bias);
            float scale = (range == 0.0f) ? 1.0f : __fdiv_rn(range, static_cast<float>(QMAX));
            __half scale_h = __float2half_rn(scale);
            scale = __half2float(scale_h);
            if (scale == 0.0f) {
                scale = 1.0f;
                scale_h = __float2half_rn(1.0f);
            }
            float inv = __fdiv_rn(1.0f, scale);
            if (isinf(inv)) {
                scale_h = __float2half_rn(1.0f);
                inv = 1.0f;
            }
            uint32_t word = 0;
#pragma unroll
            for (int v = 0; v < VL; ++v) {
                const float x[4] = {x4[p][v].x, x4[p][v].y, x4[p][v].z, x4[p][v].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int q = __float2int_rn(__fmul_rn(__fsub_rn(x[j], bias), inv));
                    q = max(0, min(QMAX, q));
                    word |= static_cast<uint32_t>(q) << (BITS * (4 * v + j));
                }
            }
            uint8_t* o = img + (p * RPP + g) * stride;
            *reinterpret_cast<uint32_t*>(o + (TABLE ? 4 : 0) + 4 * k) = word;
            if (k == 0)
                *reinterpret_cast<uint32_t*>(o + (TABLE ? 0 : pbytes)) =
                    static_cast<uint32_t>(__half_as_ushort(scale_h)) | (static_cast<uint32_t>(__half_as_ushort(bias_h)) << 16);
        }
        __syncwarp();
        const int64_t rows = (N - r0 < R) ? N - r0 : R;
        const int bytes = static_cast<int>(rows) * stride;
        uint8_t* dst = out + r0 * out_stride;                  // 16-byte aligned: r0 is a multiple of R >= 4 (or 2 rows of a
                                                               // stride that is a multiple of 8), the stride of 4
        for (int c = lane * 16; c + 16 <= bytes; c += 32 * 16)
            *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(img + c);
        for (int c = (bytes & ~15) + lane; c < bytes; c += 32) dst[c] = img[c];
        __syncwarp();
    }
}

template <int BITS>
__global__ void __launch_bounds__(kThreads)
dequantize_nbit_kernel(const uint8_t* __restrict__ in, int64_t N, int64_t Dq, float* __restrict__ out)
{
    constexpr int PER = 8 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    if (r >= N) return;
    const int64_t pbytes = Dq - 4;
    const int64_t D = pbytes * PER;
    const uint8_t* q = in + r * Dq;
    const float scale = half_bits_to_float(__ldg(q + pbytes) | (static_cast<uint32_t>(__ldg(q + pbytes + 1)) << 8));
    const float bias = half_bits_to_float(__ldg(q + pbytes + 2) | (static_cast<uint32_t>(__ldg(q + pbytes + 3)) << 8));
    float* o = out + r * D;
    for (int64_t c = lane; c < D; c += 32) {
        const uint32_t v = (__ldg(q + c / PER) >> ((c % PER) * BITS)) & MASK;
        o[c] = fmaf(static_cast<float>(v), scale, bias);
    }
}

// 4-bit rows back to fp32, batched: D a multiple of 8, rows 4-byte aligned.  LPR lanes share a row; a lane turns one
// 16-bit half of a payload word (4 codes) into ONE float4 store, so that a store instruction of the warp writes
// consecutive 16-byte pieces (whole sectors; two float4 per lane, 32 bytes apart from lane to lane, measured at 0.60
// of the copy bandwidth).  PASSES passes of 32 / LPR rows are in flight per warp.
template <int LPR, int VPL, int PASSES>
__global__ void __launch_bounds__(kThreads)
dequantize_4bit_batched_kernel(const uint8_t* __restrict__ in, int64_t N, int64_t Dq, float* __restrict__ out)
{
    constexpr int RPP = 32 / LPR;          // rows per pass
    constexpr int RPS = RPP * PASSES;      // rows per warp and step
    const int lane = threadIdx.x & 31;
    const int k = lane % LPR, g = lane / LPR;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t pbytes = Dq - 4;
    const int64_t D = pbytes * 2;
    const int nhalves = static_cast<int>(pbytes / 2);      // float4 pieces of an output row
    for (int64_t r0 = warp * RPS; r0 < N; r0 += nwarps * RPS) {
        uint32_t w[PASSES][VPL], hdr[PASSES];
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int64_t r = r0 + j * RPP + g;
            if (r >= N) continue;
            const uint8_t* q = in + r * Dq;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int h = k + LPR * v;
                if (h < nhalves) w[j][v] = ldg4(q + 4 * (h >> 1));
            }
            hdr[j] = ldg4(q + pbytes);
        }
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int64_t r = r0 + j * RPP + g;
            if (r >= N) continue;
            const float scale = half_bits_to_float(hdr[j] & 0xffffu), bias = half_bits_to_float(hdr[j] >> 16);
            float4* o = reinterpret_cast<float4*>(out + r * D);
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int h = k + LPR * v;
                if (h < nhalves) {
                    const uint32_t x = w[j][v] >> ((h & 1) * 16);
                    float4 a;
                    a.x = fmaf(static_cast<float>(x & 15u), scale, bias);
                    a.y = fmaf(static_cast<float>((x >> 4) & 15u), scale, bias);
                    a.z = fmaf(static_cast<float>((x >> 8) & 15u), scale, bias);
                    a.w = fmaf(static_cast<float>((x >> 12) & 15u), scale, bias);
                    o[h] = a;
                }
            }
        }
    }
}

// ---- packing quantizer output into table rows ----------------------------------

template <int SRC_BITS>
__global__ void __launch_bounds__(kThreads)
pack_rows_kernel(const uint8_t* __restrict__ fused, int64_t N, int64_t pbytes, int64_t row_bytes, uint8_t* __restrict__ rows)
{
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    if (r >= N) return;
    constexpr int TAIL = SRC_BITS == 8 ? 8 : 4;
    const uint8_t* f = fused + r * (pbytes + TAIL);
    uint8_t* o = rows + r * row_bytes;
    if (lane == 0) {
        uint32_t h;
        if (SRC_BITS == 8) {
            uint32_t sb[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j) sb[j >> 2] |= static_cast<uint32_t>(__ldg(f + pbytes + j)) << (8 * (j & 3));
            h = (f32_to_f16_bits(__uint_as_float(sb[0])) & 0xffffu) | (f32_to_f16_bits(__uint_as_float(sb[1])) << 16);
        } else {
            h = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) h |= static_cast<uint32_t>(__ldg(f + pbytes + j)) << (8 * j);
        }
        store_header(o, h & 0xffffu, h >> 16);
    }
    for (int64_t c = lane; c < pbytes; c += 32) o[4 + c] = __ldg(f + c);
    for (int64_t c = 4 + pbytes + lane; c < row_bytes; c += 32) o[c] = 0;
}

// fp32 [N, D] -> fp16 table rows (no header), stride row_bytes, padding zeroed.
__global__ void __launch_bounds__(kThreads)
cast_fp16_rows_kernel(const float* __restrict__ in, int64_t N, int64_t D, int64_t row_bytes, uint8_t* __restrict__ rows)
{
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    if (r >= N) return;
    const float* x = in + r * D;
    uint8_t* o = rows + r * row_bytes;
    const bool even = (reinterpret_cast<uintptr_t>(o) & 1) == 0;
    for (int64_t c = lane; c < D; c += 32) {
        uint32_t h = f32_to_f16_bits(__ldg(x + c));
        asm volatile("" : "+r"(h));   // see store_header
        if (even) {
            *reinterpret_cast<unsigned short*>(o + 2 * c) = static_cast<unsigned short>(h);
        } else {
            o[2 * c] = static_cast<uint8_t>(h & 0xffu);
            o[2 * c + 1] = static_cast<uint8_t>((h >> 8) & 0xffu);
        }
    }
    for (int64_t c = 2 * D + lane; c < row_bytes; c += 32) o[c] = 0;
}

template <typename K, typename... A>
int launch_rows(K kernel, int lpr, int64_t N, cudaStream_t s, const char* name, A... args)
{
    if (N <= 0) return TBE_B200_OK;
    const int64_t rpb = kThreads / lpr;
    const int64_t blocks = (N + rpb - 1) / rpb;
    if (blocks > 0x7fffffffll) return fail(TBE_B200_ERR_UNSUPPORTED, "%s: too many rows for one launch", name);
    kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(args...);
    return check_launch(name);
}

}  // namespace

// Shared by the two public 8-bit quantizer entry points.
int quantize_8bit_impl(const void* input, int in_is_half, int64_t N, int64_t D, uint8_t* out, int64_t out_stride,
                       bool table, cudaStream_t s)
{
    // fp32 rows of the common widths take the batched kernel
    if (!in_is_half && D >= 32 && D <= 512 && D % 4 == 0 && (reinterpret_cast<uintptr_t>(input) & 15) == 0 && out_stride % 4 == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 3) == 0 && N > 0) {
        const float* x = static_cast<const float*>(input);
        const int64_t groups = (N + 3) / 4;                                  // at most 4 rows per warp and step
        const int64_t want = (groups + kThreads / 32 - 1) / (kThreads / 32);
        const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
        const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
#define TBE_Q8B(TAB, VPL, ROWS) quantize_8bit_batched_kernel<TAB, VPL, ROWS><<<blocks, kThreads, 0, s>>>(x, N, D, out, out_stride)
        // D a multiple of 8 up to 256, 16-byte aligned output: eight elements per lane, several rows per pass
        if (D % 8 == 0 && D <= 256 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_stride >= D + (table ? 4 : 8)) {
            const int64_t units = D / 8;
            const int lanes = (units <= 4) ? 4 : (units <= 8) ? 8 : (units <= 16) ? 16 : 32;
            const int64_t rows_per_warp = 4 * (32 / lanes);
            if (rows_per_warp * out_stride <= kStaged8Bytes) {
                const int64_t groups8 = (N + rows_per_warp - 1) / rows_per_warp;
                const int64_t want8 = (groups8 + kThreads / 32 - 1) / (kThreads / 32);
                const unsigned blocks8 = static_cast<unsigned>(want8 < cap ? want8 : cap);
#define TBE_Q8W(TAB, LANES) quantize_8bit_wide_kernel<TAB, LANES><<<blocks8, kThreads, 0, s>>>(x, N, D, out, out_stride)
                if (table) { if (lanes == 4) TBE_Q8W(true, 4); else if (lanes == 8) TBE_Q8W(true, 8); else if (lanes == 16) TBE_Q8W(true, 16); else TBE_Q8W(true, 32); }
                else { if (lanes == 4) TBE_Q8W(false, 4); else if (lanes == 8) TBE_Q8W(false, 8); else if (lanes == 16) TBE_Q8W(false, 16); else TBE_Q8W(false, 32); }
#undef TBE_Q8W
                return check_launch("quantize_8bit_wide_kernel");
            }
        }
        const bool staged = D <= 128 && out_stride <= kStagedStride && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        if (staged) {
            if (table) quantize_8bit_batched_kernel<true, 1, 4, true><<<blocks, kThreads, 0, s>>>(x, N, D, out, out_stride);
            else quantize_8bit_batched_kernel<false, 1, 4, true><<<blocks, kThreads, 0, s>>>(x, N, D, out, out_stride);
        } else if (table) { if (D <= 128) TBE_Q8B(true, 1, 4); else if (D <= 256) TBE_Q8B(true, 2, 2); else TBE_Q8B(true, 4, 1); }
        else { if (D <= 128) TBE_Q8B(false, 1, 4); else if (D <= 256) TBE_Q8B(false, 2, 2); else TBE_Q8B(false, 4, 1); }
#undef TBE_Q8B
        return check_launch("quantize_8bit_batched_kernel");
    }
    const int lpr = (D <= 64) ? 8 : 32;
#define TBE_Q8(LPR, T, TAB) \
    return launch_rows(quantize_8bit_kernel<LPR, T, TAB>, LPR, N, s, "quantize_8bit_kernel", static_cast<const T*>(input), N, D, out, out_stride)
    if (in_is_half) {
        if (table) { if (lpr == 8) TBE_Q8(8, __half, true); else TBE_Q8(32, __half, true); }
        else { if (lpr == 8) TBE_Q8(8, __half, false); else TBE_Q8(32, __half, false); }
    } else {
        if (table) { if (lpr == 8) TBE_Q8(8, float, true); else TBE_Q8(32, float, true); }
        else { if (lpr == 8) TBE_Q8(8, float, false); else TBE_Q8(32, float, false); }
    }
#undef TBE_Q8
}

int quantize_nbit_impl(int bit_rate, const float* input, int64_t N, int64_t D, uint8_t* out, int64_t out_stride,
                       bool table, cudaStream_t s)
{
    // fp32 rows of the common widths take the batched kernel
    const int el = 32 / bit_rate;                                  // elements per 32-bit word of codes
    if ((bit_rate == 4 || bit_rate == 2) && D >= 4 * el && D <= 32 * el && D % el == 0 && N > 0 &&
        (reinterpret_cast<uintptr_t>(input) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_stride % 4 == 0 &&
        out_stride >= D * bit_rate / 8 + 4) {
        const int64_t units = D / el;
        const int lanes = (units <= 4) ? 4 : (units <= 8) ? 8 : (units <= 16) ? 16 : 32;
        const int64_t rows_per_warp = (bit_rate == 4 ? 4 : 2) * (32 / lanes);
        // the rows of a warp and step must start on a 16-byte boundary and fit the staging area
        if (rows_per_warp * out_stride <= kStaged4Bytes && (rows_per_warp * out_stride) % 16 == 0) {
            const int64_t groups = (N + rows_per_warp - 1) / rows_per_warp;
            const int64_t want = (groups + kThreads / 32 - 1) / (kThreads / 32);
            const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
            const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
#define TBE_QNB(TAB, LANES, BITS) quantize_nbit_batched_kernel<TAB, LANES, BITS><<<blocks, kThreads, 0, s>>>(input, N, D, out, out_stride)
#define TBE_QNB_LANES(TAB, BITS)                                      \
    do {                                                              \
        if (lanes == 4) TBE_QNB(TAB, 4, BITS);                        \
        else if (lanes == 8) TBE_QNB(TAB, 8, BITS);                   \
        else if (lanes == 16) TBE_QNB(TAB, 16, BITS);                 \
        else TBE_QNB(TAB, 32, BITS);                                  \
    } while (0)
            if (bit_rate == 4) { if (table) TBE_QNB_LANES(true, 4); else TBE_QNB_LANES(false, 4); }
            else { if (table) TBE_QNB_LANES(true, 2); else TBE_QNB_LANES(false, 2); }
#undef TBE_QNB_LANES
#undef TBE_QNB
            return check_launch("quantize_nbit_batched_kernel");
        }
    }
    const int lpr = (D <= 128) ? 8 : 32;
#define TBE_QN(LPR, BITS, TAB) \
    return launch_rows(quantize_nbit_kernel<LPR, BITS, TAB>, LPR, N, s, "quantize_nbit_kernel", input, N, D, out, out_stride)
    if (bit_rate == 4) {
        if (table) { if (lpr == 8) TBE_QN(8, 4, true); else TBE_QN(32, 4, true); }
        else { if (lpr == 8) TBE_QN(8, 4, false); else TBE_QN(32, 4, false); }
    } else {
        if (table) { if (lpr == 8) TBE_QN(8, 2, true); else TBE_QN(32, 2, true); }
        else { if (lpr == 8) TBE_QN(8, 2, false); else TBE_QN(32, 2, false); }
    }
#undef TBE_QN
}

}  // namespace tbe

using namespace tbe;

extern "C" int tbe_b200_quantize_8bit_rowwise(const void* input, int32_t in_is_half, int64_t nrows, int64_t ncols,
                                              uint8_t* output, tbe_b200_stream_t stream)
{
    if (nrows < 0 || ncols < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_8bit_rowwise: negative size");
    if (nrows > 0 && (!input || !output)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_8bit_rowwise: NULL pointer");
    return quantize_8bit_impl(input, in_is_half, nrows, ncols, output, ncols + 8, false, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tbe_b200_dequantize_8bit_rowwise(const uint8_t* input, int64_t nrows, int64_t ncols_q, void* output,
                                                int32_t out_is_half, tbe_b200_stream_t stream)
{
    if (nrows < 0 || ncols_q < 8)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "dequantize_8bit_rowwise: rows need at least the 8 scale/bias bytes");
    if (nrows > 0 && (!input || !output)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "dequantize_8bit_rowwise: NULL pointer");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t D = ncols_q - 8;
    if (!out_is_half && D >= 32 && D <= 512 && D % 4 == 0 && (reinterpret_cast<uintptr_t>(input) & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(output) & 15) == 0 && nrows > 0) {
        const int64_t groups = (nrows + 3) / 4;
        const int64_t want = (groups + kThreads / 32 - 1) / (kThreads / 32);
        const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
        const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
        float* o = static_cast<float*>(output);
        if (D <= 128) dequantize_8bit_batched_kernel<1, 4><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, o);
        else if (D <= 256) dequantize_8bit_batched_kernel<2, 2><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, o);
        else dequantize_8bit_batched_kernel<4, 1><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, o);
        return check_launch("dequantize_8bit_batched_kernel");
    }
    const int lpr = (ncols_q - 8 <= 64) ? 8 : 32;
    if (out_is_half) {
        if (lpr == 8) return launch_rows(dequantize_8bit_kernel<8, __half>, 8, nrows, s, "dequantize_8bit_kernel", input, nrows, ncols_q, static_cast<__half*>(output));
        return launch_rows(dequantize_8bit_kernel<32, __half>, 32, nrows, s, "dequantize_8bit_kernel", input, nrows, ncols_q, static_cast<__half*>(output));
    }
    if (lpr == 8) return launch_rows(dequantize_8bit_kernel<8, float>, 8, nrows, s, "dequantize_8bit_kernel", input, nrows, ncols_q, static_cast<float*>(output));
    return launch_rows(dequantize_8bit_kernel<32, float>, 32, nrows, s, "dequantize_8bit_kernel", input, nrows, ncols_q, static_cast<float*>(output));
}

extern "C" int tbe_b200_quantize_nbit_rowwise_sbhalf(int32_t bit_rate, const float* input, int64_t nrows, int64_t ncols,
                                                     uint8_t* output, tbe_b200_stream_t stream)
{
    if (bit_rate != 2 && bit_rate != 4)
        return fail(TBE_B200_ERR_UNSUPPORTED, "quantize_nbit_rowwise_sbhalf: bit_rate must be 2 or 4, got %d", bit_rate);
    if (nrows < 0 || ncols < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_nbit_rowwise_sbhalf: negative size");
    if (nrows > 0 && (!input || !output)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_nbit_rowwise_sbhalf: NULL pointer");
    const int per = 8 / bit_rate;
    return quantize_nbit_impl(bit_rate, input, nrows, ncols, output, (ncols + per - 1) / per + 4, false,
                              reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tbe_b200_dequantize_nbit_rowwise_sbhalf(int32_t bit_rate, const uint8_t* input, int64_t nrows,
                                                       int64_t ncols_q, float* output, tbe_b200_stream_t stream)
{
    if (bit_rate != 2 && bit_rate != 4)
        return fail(TBE_B200_ERR_UNSUPPORTED, "dequantize_nbit_rowwise_sbhalf: bit_rate must be 2 or 4, got %d", bit_rate);
    if (nrows < 0 || ncols_q < 4)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "dequantize_nbit_rowwise_sbhalf: rows need at least the 4 scale/bias bytes");
    if (nrows > 0 && (!input || !output)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "dequantize_nbit_rowwise_sbhalf: NULL pointer");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t pb = ncols_q - 4;
    if (bit_rate == 4 && pb >= 16 && pb % 4 == 0 && pb <= 512 && (reinterpret_cast<uintptr_t>(input) & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(output) & 15) == 0 && nrows > 0) {
        const int64_t want = (nrows + 8 * (kThreads / 32) - 1) / (8 * (kThreads / 32));
        const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
        const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
        if (pb <= 32) dequantize_4bit_batched_kernel<16, 1, 4><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, output);
        else if (pb <= 64) dequantize_4bit_batched_kernel<32, 1, 4><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, output);
        else if (pb <= 128) dequantize_4bit_batched_kernel<32, 2, 4><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, output);
        else dequantize_4bit_batched_kernel<32, 8, 2><<<blocks, kThreads, 0, s>>>(input, nrows, ncols_q, output);
        return check_launch("dequantize_4bit_batched_kernel");
    }
    if (bit_rate == 4) return launch_rows(dequantize_nbit_kernel<4>, 32, nrows, s, "dequantize_nbit_kernel", input, nrows, ncols_q, output);
    return launch_rows(dequantize_nbit_kernel<2>, 32, nrows, s, "dequantize_nbit_kernel", input, nrows, ncols_q, output);
}

extern "C" int tbe_b200_pack_table_rows(int32_t src_bits, const uint8_t* fused, int64_t nrows, int64_t ncols,
                                        int64_t row_bytes, uint8_t* rows, tbe_b200_stream_t stream)
{
    if (src_bits != 8 && src_bits != 4 && src_bits != 2)
        return fail(TBE_B200_ERR_UNSUPPORTED, "pack_table_rows: src_bits must be 8, 4 or 2, got %d", src_bits);
    if (nrows < 0 || ncols < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "pack_table_rows: negative size");
    const int per = 8 / src_bits;
    const int64_t pbytes = (ncols + per - 1) / per;
    if (row_bytes < pbytes + 4) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "pack_table_rows: row_bytes %lld too small for %lld payload bytes + header",
                                            (long long)row_bytes, (long long)pbytes);
    if (nrows > 0 && (!fused || !rows)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "pack_table_rows: NULL pointer");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (src_bits == 8) return launch_rows(pack_rows_kernel<8>, 32, nrows, s, "pack_rows_kernel", fused, nrows, pbytes, row_bytes, rows);
    return launch_rows(pack_rows_kernel<4>, 32, nrows, s, "pack_rows_kernel", fused, nrows, pbytes, row_bytes, rows);
}

extern "C" int tbe_b200_quantize_to_table_rows(int32_t weight_ty, const float* input, int64_t nrows, int64_t ncols,
                                               int64_t row_bytes, uint8_t* rows, tbe_b200_stream_t stream)
{
    if (nrows < 0 || ncols < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_to_table_rows: negative size");
    if (nrows > 0 && (!input || !rows)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_to_table_rows: NULL pointer");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int64_t need;
    switch (weight_ty) {
        case TBE_B200_INT8: need = ncols + 4; break;
        case TBE_B200_INT4: need = (ncols + 1) / 2 + 4; break;
        case TBE_B200_INT2: need = (ncols + 3) / 4 + 4; break;
        case TBE_B200_FP16: need = 2 * ncols; break;
        default:
            return fail(TBE_B200_ERR_UNSUPPORTED, "quantize_to_table_rows: weight type %d (supported: FP16, INT8, INT4, INT2)", weight_ty);
    }
    if (row_bytes < need)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "quantize_to_table_rows: row_bytes %lld smaller than the %lld bytes a row needs",
                    (long long)row_bytes, (long long)need);
    if (weight_ty == TBE_B200_INT8) return quantize_8bit_impl(input, 0, nrows, ncols, rows, row_bytes, true, s);
    if (weight_ty == TBE_B200_INT4) return quantize_nbit_impl(4, input, nrows, ncols, rows, row_bytes, true, s);
    if (weight_ty == TBE_B200_INT2) return quantize_nbit_impl(2, input, nrows, ncols, rows, row_bytes, true, s);
    return launch_rows(cast_fp16_rows_kernel, 32, nrows, s, "cast_fp16_rows_kernel", input, nrows, ncols, row_bytes, rows);
}
