// Shared helpers for the tbe_b200 CUDA library: error reporting, cached device
// properties, small device-side load/store and conversion primitives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tbe_b200.h"

namespace tbe {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);

// cudaGetLastError() after a launch -> status.
int check_launch(const char* what);

// Number of SMs of the current device (cached per device).
int sm_count();

constexpr int kWarp = 32;

__device__ __forceinline__ uint4 ldg16(const void* p)
{
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint2 ldg8(const void* p)
{
    return __ldg(reinterpret_cast<const uint2*>(p));
}
__device__ __forceinline__ uint32_t ldg4(const void* p)
{
    return __ldg(reinterpret_cast<const uint32_t*>(p));
}

// Streaming (read-once) loads: do not keep the line in L1, mark it first to go in L2.
__device__ __forceinline__ int32_t ld_stream(const int32_t* p)
{
    int32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ int64_t ld_stream(const int64_t* p)
{
    int64_t v;
    asm volatile("ld.global.nc.L1::no_allocate.b64 %0, [%1];" : "=l"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_stream(const float* p)
{
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// Streaming stores (output is written once and not re-read by this kernel).
__device__ __forceinline__ void st_stream16(void* p, uint4 v)
{
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void st_stream8(void* p, uint2 v)
{
    asm volatile("st.global.cs.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream4(void* p, uint32_t v)
{
    asm volatile("st.global.cs.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16)
{
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

// fp32 -> 16-bit output patterns, round-to-nearest-even.
__device__ __forceinline__ uint32_t f32_to_f16_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v)
{
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

}  // namespace tbe
