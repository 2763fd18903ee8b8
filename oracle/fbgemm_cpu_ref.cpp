/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * Harness over the FBGEMM CPU kernels that ship inside libtorch_cpu.so (public
 * headers: torch/include/fbgemm/FbgemmEmbedding.h, QuantUtils.h).  FBGEMM is the
 * CPU library that the reference's golden path is built on: the reference's
 * tests compare against fbgemm_gpu's CPU operators
 * (bench/tbe_inference/.../test_int_nbit_split_embedding_codegen_lookup_function.py:322-349),
 * and fbgemm_gpu itself (requirements.txt:4) is not installable here.  This file
 * drives those kernels in the table-batched layout the way the upstream CPU
 * operator does: one EmbeddingSpMDM call per (table, batch chunk) with
 * input = dev_weights + weights_offsets[t], input_stride = row bytes,
 * output_stride = total_D, scale_bias_last = false, OpenMP across the calls.
 *
 * It is the strongest pin for oracle/tbe_oracle.c and the "reference" CPU
 * baseline the benchmark times.  Only tests, the smoke test and the benchmark's
 * CPU leg load it; the GPU library never does.
 *
 * Build: see oracle/Makefile (g++ -std=c++17 against the torch include/lib dirs;
 * output oracle/_ref/libfbgemm_cpu_ref.so).
 */
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "fbgemm/FbgemmEmbedding.h"
#include "fbgemm/QuantUtils.h"

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

enum { TY_FP32 = 0, TY_FP16 = 1, TY_INT8 = 2, TY_INT4 = 3, TY_INT2 = 4, TY_BF16 = 5, TY_FP8 = 6 };
enum { POOL_SUM = 0, POOL_MEAN = 1, POOL_NONE = 2 };

int64_t row_bytes(int ty, int64_t D, int64_t align)
{
    int64_t b;
    switch (ty) {
        case TY_FP32: b = 4 * D; break;
        case TY_FP16: b = 2 * D; break;
        case TY_FP8: b = D; break;
        case TY_INT8: b = D + 4; break;
        case TY_INT4: b = (D + 1) / 2 + 4; break;
        case TY_INT2: b = (D + 3) / 4 + 4; break;
        default: return -1;
    }
    if (align > 1) b = (b + align - 1) / align * align;
    return b;
}

template <typename InT, typename IdxT, typename OutT>
using Kern = typename fbgemm::EmbeddingSpMDMKernelSignature<InT, IdxT, IdxT, OutT>::Type;

/* One generated kernel per distinct (type, D, flags); generation JIT-compiles. */
template <typename InT, typename IdxT, typename OutT>
Kern<InT, IdxT, OutT> make_kernel(int ty, int64_t D, bool weighted, bool mean, bool nobag, bool bf16_out,
                                  int64_t out_stride, int64_t in_stride, int ebits, int ebias)
{
    if constexpr (std::is_same<InT, uint8_t>::value) {
        if (ty == TY_INT8) {
            return fbgemm::GenerateEmbeddingSpMDMWithStrides<uint8_t, IdxT, IdxT, OutT>(
                D, weighted, mean, /*prefetch=*/16, /*is_weight_positional=*/false, /*use_offsets=*/true,
                out_stride, in_stride, /*scale_bias_last=*/false, nobag, bf16_out, false);
        }
        if (ty == TY_FP8) {
            if constexpr (!std::is_same<OutT, uint8_t>::value) {
                return fbgemm::GenerateEmbeddingSpMDMFP8WithStrides<IdxT, IdxT, OutT>(
                    D, mean, false, true, out_stride, in_stride, ebits, ebias, bf16_out);
            }
        }
        return fbgemm::GenerateEmbeddingSpMDMNBitWithStrides<IdxT, IdxT, OutT>(
            ty == TY_INT4 ? 4 : 2, D, weighted, mean, 16, false, true, out_stride, in_stride,
            /*scale_bias_last=*/false, bf16_out, nobag, -1);
    } else {
        return fbgemm::GenerateEmbeddingSpMDMWithStrides<InT, IdxT, IdxT, OutT>(
            D, weighted, mean, 16, false, true, out_stride,
            in_stride / (int64_t)sizeof(InT), /*scale_bias_last=*/false, nobag, bf16_out, false);
    }
}

template <typename IdxT, typename OutT>
int64_t lookup_typed(const uint8_t* dev_weights, int64_t dev_weights_bytes, const int64_t* weights_offsets,
                     const uint8_t* weights_tys, const int32_t* D_offsets, int64_t T, int64_t B,
                     const IdxT* indices, const IdxT* offsets, const float* indice_weights, int pooling_mode,
                     bool bf16_out, int64_t row_alignment, int ebits, int ebias, OutT* out, int64_t out_stride)
{
    const bool mean = pooling_mode == POOL_MEAN;
    const bool weighted = indice_weights != nullptr;
    /* FP8 weighted pooling has no generated-kernel flag; the caller never asks for it. */
    std::vector<Kern<uint8_t, IdxT, OutT>> k8(T);
    std::vector<Kern<uint16_t, IdxT, OutT>> k16(T);
    std::vector<Kern<float, IdxT, OutT>> k32(T);
    std::vector<int64_t> rb(T), nrows(T);
    for (int64_t t = 0; t < T; ++t) {
        const int ty = weights_tys[t];
        const int64_t D = D_offsets[t + 1] - D_offsets[t];
        rb[t] = row_bytes(ty, D, row_alignment);
        if (rb[t] <= 0) return -1000 - t;
        const int64_t end = (t + 1 < T) ? weights_offsets[t + 1] : dev_weights_bytes;
        int64_t span = end - weights_offsets[t];
        if (span < 0) span = dev_weights_bytes - weights_offsets[t];
        nrows[t] = span / rb[t];
        if (ty == TY_FP16) k16[t] = make_kernel<uint16_t, IdxT, OutT>(ty, D, weighted, mean, false, bf16_out, out_stride, rb[t], 0, 0);
        else if (ty == TY_FP32) k32[t] = make_kernel<float, IdxT, OutT>(ty, D, weighted, mean, false, bf16_out, out_stride, rb[t], 0, 0);
        else k8[t] = make_kernel<uint8_t, IdxT, OutT>(ty, D, weighted, mean, false, bf16_out, out_stride, rb[t], ebits, ebias);
    }
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    int64_t chunks_per_table = (nthreads * 4 + T - 1) / T;
    if (chunks_per_table < 1) chunks_per_table = 1;
    int64_t chunk = (B + chunks_per_table - 1) / chunks_per_table;
    if (chunk < 1) chunk = 1;
    chunks_per_table = (B + chunk - 1) / chunk;
    int64_t status = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < T * chunks_per_table; ++job) {
        const int64_t t = job / chunks_per_table;
        const int64_t b0 = (job % chunks_per_table) * chunk;
        const int64_t nb = (b0 + chunk <= B) ? chunk : (B - b0);
        const int ty = weights_tys[t];
        const IdxT* off = offsets + t * B + b0;
        const int64_t first = off[0];
        const int64_t index_size = off[nb] - first;
        const uint8_t* w = dev_weights + weights_offsets[t];
        const float* pw = weighted ? indice_weights + first : nullptr;
        OutT* o = out + b0 * out_stride + D_offsets[t];
        bool ok;
        if (ty == TY_FP16) ok = k16[t](nb, index_size, nrows[t], (const uint16_t*)w, indices + first, off, pw, o);
        else if (ty == TY_FP32) ok = k32[t](nb, index_size, nrows[t], (const float*)w, indices + first, off, pw, o);
        else ok = k8[t](nb, index_size, nrows[t], w, indices + first, off, pw, o);
        if (!ok) {
#pragma omp critical
            status = -(1 + job);
        }
    }
    return status;
}

}  // namespace

extern "C" {

void fbr_quantize_8bit_rowwise(const float* in, int64_t N, int64_t D, uint8_t* out)
{
    fbgemm::FloatOrHalfToFused8BitRowwiseQuantizedSBFloat<float>(in, (size_t)N, (int)D, out);
}

void fbr_dequantize_8bit_rowwise(const uint8_t* in, int64_t N, int64_t Dq, float* out)
{
    fbgemm::Fused8BitRowwiseQuantizedSBFloatToFloatOrHalf<float>(in, (size_t)N, (int)Dq, out);
}

void fbr_quantize_nbit_rowwise_sbhalf(int bit_rate, const float* in, int64_t N, int64_t D, uint8_t* out)
{
    fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf<float>(bit_rate, in, (size_t)N, (int)D, out);
}

void fbr_dequantize_nbit_rowwise_sbhalf(int bit_rate, const uint8_t* in, int64_t N, int64_t Dq, float* out)
{
    fbgemm::FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf<float>(bit_rate, in, (size_t)N, (int)Dq, out);
}

/*
 * Same argument meaning as orc_tbe_lookup in tbe_oracle.c, plus the byte size of
 * dev_weights (the FBGEMM kernels bounds-check indices against the row count).
 * Pooled modes only.  out_ty: 0 fp32, 1 fp16, 5 bf16.
 * Returns 0, or a negative value if a kernel rejected an index.
 */
int64_t fbr_tbe_lookup(const uint8_t* dev_weights, int64_t dev_weights_bytes, const int64_t* weights_offsets,
                       const uint8_t* weights_tys, const int32_t* D_offsets, int64_t T, int64_t B,
                       int64_t total_D, const void* indices, const void* offsets, int idx_bits,
                       const float* indice_weights, int pooling_mode, int out_ty, int64_t row_alignment,
                       int fp8_ebits, int fp8_ebias, void* out, int64_t out_stride)
{
    (void)total_D;
    if (pooling_mode == POOL_NONE) return -2;
#define CALL(IdxT, OutT, BF)                                                                                   \
    return lookup_typed<IdxT, OutT>(dev_weights, dev_weights_bytes, weights_offsets, weights_tys, D_offsets, T, \
                                    B, (const IdxT*)indices, (const IdxT*)offsets, indice_weights,             \
                                    pooling_mode, BF, row_alignment, fp8_ebits, fp8_ebias, (OutT*)out,         \
                                    out_stride)
    if (idx_bits == 32) {
        if (out_ty == 0) CALL(int32_t, float, false);
        if (out_ty == 1) CALL(int32_t, uint16_t, false);
        if (out_ty == 5) CALL(int32_t, uint16_t, true);
    } else {
        if (out_ty == 0) CALL(int64_t, float, false);
        if (out_ty == 1) CALL(int64_t, uint16_t, false);
        if (out_ty == 5) CALL(int64_t, uint16_t, true);
    }
#undef CALL
    return -3;
}

int fbr_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
