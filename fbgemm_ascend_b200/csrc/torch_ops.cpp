// PyTorch operator registrations: the `torch.ops.fbgemm.*` surface of the
// quantized TBE inference path, dispatched to CUDA and implemented by the C ABI
// of libtbe_b200.so (include/tbe_b200.h).
//
// This file takes the place of the reference's adapter layer
//   src/tbe_inference/int_nbit_split_embedding_codegen_lookup_function/
//       int_nbit_split_embedding_codegen_lookup_function.cpp:55-176
//   src/pooled_embedding_ops/permute_pooled_embs/permute_pooled_embs.cpp:25-121
// and of the launch shim EXEC_NPU_CMD (src/common/pytorch_npu_helper.hpp:536-585):
// same operator names, argument order, defaults, checks and error type
// (c10::Error -> RuntimeError), but no host synchronisation and no CPU fallback.
//
// The reference relies on `import fbgemm_gpu` for the operator schemas.  Here a
// schema is defined only when nobody has defined it yet, so the library also
// loads next to a real fbgemm_gpu.
#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/library.h>

#include <algorithm>
#include <optional>
#include <tuple>
#include <vector>

#include "tbe_b200.h"

namespace {

using at::Tensor;

tbe_b200_stream_t current_stream() { return reinterpret_cast<tbe_b200_stream_t>(c10::cuda::getCurrentCUDAStream().stream()); }

void check_status(int rc, const char* op)
{
    TORCH_CHECK(rc == TBE_B200_OK, op, " failed (status ", rc, "): ", tbe_b200_last_error());
}

void check_cuda(const Tensor& t, const char* name)
{
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor; this library has no CPU path");
}

// SparseType -> dtype of the output tensor
// (int_nbit_split_embedding_codegen_lookup_function.cpp:37-52).
at::ScalarType sparse_type_to_scalar_type(int64_t output_dtype)
{
    switch (output_dtype) {
        case TBE_B200_FP32: return at::kFloat;
        case TBE_B200_FP16: return at::kHalf;
        case TBE_B200_INT8: return at::kByte;
        case TBE_B200_BF16: return at::kBFloat16;
        default:
            TORCH_CHECK(false, "Unsupported output_dtype: ", output_dtype,
                        ". Supported: 0(FP32), 1(FP16), 2(INT8), 5(BF16)");
    }
}

Tensor int_nbit_split_embedding_codegen_lookup_function_cuda(
    Tensor dev_weights, Tensor uvm_weights, Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys,
    Tensor D_offsets, const int64_t total_D, const int64_t max_int2_D, const int64_t max_int4_D,
    const int64_t max_int8_D, const int64_t max_float16_D, const int64_t max_float32_D, Tensor indices, Tensor offsets,
    const int64_t pooling_mode, std::optional<Tensor> indice_weights, const int64_t output_dtype,
    std::optional<Tensor> lxu_cache_weights, std::optional<Tensor> lxu_cache_locations,
    const std::optional<int64_t> row_alignment, const std::optional<int64_t> max_float8_D,
    const std::optional<int64_t> fp8_exponent_bits, const std::optional<int64_t> fp8_exponent_bias)
{
    (void)uvm_weights; (void)weights_placements; (void)lxu_cache_weights; (void)lxu_cache_locations;  // reserved
    check_cuda(dev_weights, "dev_weights");
    check_cuda(indices, "indices");
    check_cuda(offsets, "offsets");
    const c10::cuda::CUDAGuard guard(dev_weights.device());

    const int64_t T = weights_offsets.size(0);
    const int64_t total_len = indices.numel();
    const int64_t max_float8 = max_float8_D.value_or(0);
    const int64_t row_align = row_alignment.value_or(16);
    const int64_t max_D = std::max({max_int2_D, max_int4_D, max_int8_D, max_float8, max_float16_D, max_float32_D});

    std::optional<Tensor> weights;
    if (indice_weights && indice_weights->defined() && indice_weights->numel() > 0) {
        weights = indice_weights->to(dev_weights.device(), at::kFloat).contiguous();
    }
    Tensor offs = offsets.scalar_type() != indices.scalar_type() ? offsets.toType(indices.scalar_type()) : offsets;

    TORCH_CHECK(T > 0, "weights_offsets size must be great than 0.");
    TORCH_CHECK(total_len > 0, "indices can not be empty tensor.");
    TORCH_CHECK(offs.size(0) > 1, "offsets dim_0 must be great than 1.");
    TORCH_CHECK(weights_tys.size(0) == T, "weights_tys size must equal weights_offsets size.");
    TORCH_CHECK(D_offsets.numel() == T + 1, "D_offsets must have T+1 elements.");
    TORCH_CHECK(indices.scalar_type() == at::kInt || indices.scalar_type() == at::kLong, "indices must be int32 or int64");
    TORCH_CHECK(pooling_mode >= 0 && pooling_mode <= 2, "pooling_mode must be 0 (SUM), 1 (MEAN) or 2 (NONE), got ",
                pooling_mode);
    TORCH_CHECK(dev_weights.scalar_type() == at::kByte, "dev_weights must be uint8");
    if (weights) TORCH_CHECK(weights->numel() == total_len, "indice_weights size must equal indices size.");
    const at::ScalarType out_type = sparse_type_to_scalar_type(output_dtype);
    TORCH_CHECK(output_dtype != TBE_B200_INT8, "INT8 output_dtype is not supported by this device kernel.");

    const auto dev = dev_weights.device();
    Tensor w_dev = dev_weights.contiguous();
    Tensor w_off = weights_offsets.to(dev, at::kLong).contiguous();
    Tensor w_tys = weights_tys.to(dev, at::kByte).contiguous();
    Tensor d_off = D_offsets.to(dev, at::kInt).contiguous();
    Tensor idx = indices.contiguous();
    offs = offs.contiguous();

    tbe_b200_lookup_args a{};
    a.dev_weights = w_dev.data_ptr<uint8_t>();
    a.dev_weights_bytes = w_dev.numel();
    a.weights_offsets = w_off.data_ptr<int64_t>();
    a.weights_tys = w_tys.data_ptr<uint8_t>();
    a.D_offsets = d_off.data_ptr<int32_t>();
    a.T = static_cast<int32_t>(T);
    a.total_D = total_D;
    a.max_D = static_cast<int32_t>(max_D);
    a.indices = idx.data_ptr();
    a.offsets = offs.data_ptr();
    a.index_bits = idx.scalar_type() == at::kInt ? 32 : 64;
    a.num_indices = total_len;
    a.indice_weights = weights ? weights->data_ptr<float>() : nullptr;
    a.pooling_mode = static_cast<int32_t>(pooling_mode);
    a.output_dtype = static_cast<int32_t>(output_dtype);
    a.row_alignment = static_cast<int32_t>(row_align);
    a.fp8_exponent_bits = static_cast<int32_t>(fp8_exponent_bits.value_or(-1));
    a.fp8_exponent_bias = static_cast<int32_t>(fp8_exponent_bias.value_or(-1));

    Tensor output;
    if (pooling_mode == TBE_B200_POOL_NONE) {
        // Sequence mode: one output row per index, max_D wide
        // (int_nbit_split_embedding_codegen_lookup_function.cpp:132-146).
        a.B = (offs.numel() - 1) / T;
        output = at::empty({total_len, max_D}, dev_weights.options().dtype(out_type));
        a.output_stride = max_D;
    } else {
        const int64_t rem = (offs.size(0) - 1) % T;
        TORCH_CHECK(rem == 0, "offset size = ", offs.size(0), " is incorrect for feature count = ", T);
        a.B = (offs.size(0) - 1) / T;
        // The kernel writes every element, zeros for empty bags included, so no memset pass.
        output = at::empty({a.B, total_D}, dev_weights.options().dtype(out_type));
        a.output_stride = total_D;
    }
    a.output = output.data_ptr();
    check_status(tbe_b200_int_nbit_lookup(&a, current_stream()), "int_nbit_split_embedding_codegen_lookup_function");
    return output;
}

// ---- rowwise quantizers (upstream fbgemm operators; fbgemm_ascend/__init__.py:9) --

Tensor as_rows(const Tensor& t, int64_t& nrows, int64_t& ncols, const char* op)
{
    TORCH_CHECK(t.dim() >= 1, op, ": input must have at least one dimension");
    Tensor c = t.contiguous();
    ncols = c.size(-1);
    nrows = ncols > 0 ? c.numel() / ncols : 0;
    return c;
}

std::vector<int64_t> with_last(const Tensor& t, int64_t last)
{
    std::vector<int64_t> s = t.sizes().vec();
    s.back() = last;
    return s;
}

Tensor float_or_half_to_fused8bit(const Tensor& input, bool half, const char* op)
{
    check_cuda(input, "input");
    TORCH_CHECK(input.scalar_type() == (half ? at::kHalf : at::kFloat), op, ": input dtype mismatch");
    const c10::cuda::CUDAGuard guard(input.device());
    int64_t n, d;
    Tensor x = as_rows(input, n, d, op);
    Tensor out = at::empty(with_last(x, d + 8), x.options().dtype(at::kByte));
    check_status(tbe_b200_quantize_8bit_rowwise(x.data_ptr(), half ? 1 : 0, n, d, out.data_ptr<uint8_t>(), current_stream()), op);
    return out;
}

Tensor float_to_fused8bit(const Tensor& input) { return float_or_half_to_fused8bit(input, false, "FloatToFused8BitRowwiseQuantized"); }
Tensor half_to_fused8bit(const Tensor& input) { return float_or_half_to_fused8bit(input, true, "HalfToFused8BitRowwiseQuantized"); }

Tensor fused8bit_to_float_or_half(const Tensor& input, bool half, const char* op)
{
    check_cuda(input, "input");
    TORCH_CHECK(input.scalar_type() == at::kByte, op, ": input must be uint8");
    const c10::cuda::CUDAGuard guard(input.device());
    int64_t n, dq;
    Tensor q = as_rows(input, n, dq, op);
    TORCH_CHECK(dq >= 8, op, ": rows must hold at least the 8 scale/bias bytes");
    Tensor out = at::empty(with_last(q, dq - 8), q.options().dtype(half ? at::kHalf : at::kFloat));
    check_status(tbe_b200_dequantize_8bit_rowwise(q.data_ptr<uint8_t>(), n, dq, out.data_ptr(), half ? 1 : 0, current_stream()), op);
    return out;
}

Tensor fused8bit_to_float(const Tensor& input) { return fused8bit_to_float_or_half(input, false, "Fused8BitRowwiseQuantizedToFloat"); }
Tensor fused8bit_to_half(const Tensor& input) { return fused8bit_to_float_or_half(input, true, "Fused8BitRowwiseQuantizedToHalf"); }

Tensor float_to_fused_nbit_sbhalf(const Tensor& input, const int64_t bit_rate)
{
    const char* op = "FloatToFusedNBitRowwiseQuantizedSBHalf";
    check_cuda(input, "input");
    TORCH_CHECK(input.scalar_type() == at::kFloat, op, ": input must be float32");
    TORCH_CHECK(bit_rate == 2 || bit_rate == 4, op, ": bit_rate must be 2 or 4");
    const c10::cuda::CUDAGuard guard(input.device());
    int64_t n, d;
    Tensor x = as_rows(input, n, d, op);
    const int64_t per = 8 / bit_rate;
    TORCH_CHECK(d % per == 0, op, ": the last dimension must be a multiple of ", per);
    Tensor out = at::empty(with_last(x, d / per + 4), x.options().dtype(at::kByte));
    check_status(tbe_b200_quantize_nbit_rowwise_sbhalf(static_cast<int32_t>(bit_rate), x.data_ptr<float>(), n, d,
                                                       out.data_ptr<uint8_t>(), current_stream()), op);
    return out;
}

Tensor fused_nbit_sbhalf_to_float(const Tensor& input, const int64_t bit_rate)
{
    const char* op = "FusedNBitRowwiseQuantizedSBHalfToFloat";
    check_cuda(input, "input");
    TORCH_CHECK(input.scalar_type() == at::kByte, op, ": input must be uint8");
    TORCH_CHECK(bit_rate == 2 || bit_rate == 4, op, ": bit_rate must be 2 or 4");
    const c10::cuda::CUDAGuard guard(input.device());
    int64_t n, dq;
    Tensor q = as_rows(input, n, dq, op);
    TORCH_CHECK(dq >= 4, op, ": rows must hold at least the 4 scale/bias bytes");
    Tensor out = at::empty(with_last(q, (dq - 4) * (8 / bit_rate)), q.options().dtype(at::kFloat));
    check_status(tbe_b200_dequantize_nbit_rowwise_sbhalf(static_cast<int32_t>(bit_rate), q.data_ptr<uint8_t>(), n, dq,
                                                         out.data_ptr<float>(), current_stream()), op);
    return out;
}

// fp32 [E, D] -> table rows uint8 [E, row_bytes] of weight type `weight_ty` (library-specific helper).
Tensor quantize_to_table_rows(const Tensor& input, const int64_t weight_ty, const int64_t row_bytes)
{
    const char* op = "quantize_to_table_rows";
    check_cuda(input, "input");
    TORCH_CHECK(input.scalar_type() == at::kFloat && input.dim() == 2, op, ": input must be a float32 matrix");
    const c10::cuda::CUDAGuard guard(input.device());
    Tensor x = input.contiguous();
    Tensor out = at::empty({x.size(0), row_bytes}, x.options().dtype(at::kByte));
    check_status(tbe_b200_quantize_to_table_rows(static_cast<int32_t>(weight_ty), x.data_ptr<float>(), x.size(0), x.size(1),
                                                 row_bytes, out.data_ptr<uint8_t>(), current_stream()), op);
    return out;
}

Tensor pack_table_rows(const Tensor& fused, const int64_t src_bits, const int64_t ncols, const int64_t row_bytes)
{
    const char* op = "pack_table_rows";
    check_cuda(fused, "fused");
    TORCH_CHECK(fused.scalar_type() == at::kByte && fused.dim() == 2, op, ": fused must be a uint8 matrix");
    const c10::cuda::CUDAGuard guard(fused.device());
    Tensor f = fused.contiguous();
    Tensor out = at::empty({f.size(0), row_bytes}, f.options());
    check_status(tbe_b200_pack_table_rows(static_cast<int32_t>(src_bits), f.data_ptr<uint8_t>(), f.size(0), ncols, row_bytes,
                                          out.data_ptr<uint8_t>(), current_stream()), op);
    return out;
}

// ---- permute_pooled_embs ------------------------------------------------------

// Same checks, order and messages as validate_permute_pooled_embs_inputs
// (permute_pooled_embs.cpp:25-60).
void validate_permute_pooled_embs_inputs(const Tensor& pooled_embs, const Tensor& offset_dim_list,
                                         const Tensor& permute_list, const Tensor& inv_offset_dim_list)
{
    TORCH_CHECK(pooled_embs.dim() >= 2, "pooled_embs must be at least 2-D");
    TORCH_CHECK(offset_dim_list.scalar_type() == at::ScalarType::Long, "offset_dim_list must be int64");
    TORCH_CHECK(permute_list.scalar_type() == at::ScalarType::Long, "permute_list must be int64");
    TORCH_CHECK(inv_offset_dim_list.scalar_type() == at::ScalarType::Long, "inv_offset_dim_list must be int64");
    const auto T = permute_list.numel();
    TORCH_CHECK(offset_dim_list.numel() == T + 1, "offset_dim_list must have T+1 elements");
    TORCH_CHECK(inv_offset_dim_list.numel() == T + 1, "inv_offset_dim_list must have T+1 elements");
    TORCH_CHECK(pooled_embs.scalar_type() == at::ScalarType::Float || pooled_embs.scalar_type() == at::ScalarType::Half ||
                    pooled_embs.scalar_type() == at::ScalarType::BFloat16,
                "pooled_embs must be float32, float16, or bfloat16");
    TORCH_CHECK(pooled_embs.numel() > 0, "pooled_embs must not be empty");
    TORCH_CHECK(offset_dim_list.numel() > 0, "offset_dim_list must not be empty");
    TORCH_CHECK(permute_list.numel() > 0, "permute_list must not be empty");
    TORCH_CHECK(inv_offset_dim_list.numel() > 0, "inv_offset_dim_list must not be empty");
    check_cuda(pooled_embs, "pooled_embs");
}

Tensor permute_pooled_embs_cuda(const Tensor& pooled_embs, const Tensor& offset_dim_list, const Tensor& permute_list,
                                const Tensor& inv_offset_dim_list, const Tensor& inv_permute_list)
{
    (void)inv_permute_list;  // not used by the forward (permute_pooled_embs.cpp:69)
    validate_permute_pooled_embs_inputs(pooled_embs, offset_dim_list, permute_list, inv_offset_dim_list);
    const c10::cuda::CUDAGuard guard(pooled_embs.device());
    const auto dev = pooled_embs.device();
    Tensor in = pooled_embs.contiguous();
    Tensor off = offset_dim_list.to(dev).contiguous();
    Tensor perm = permute_list.to(dev).contiguous();
    Tensor inv_off = inv_offset_dim_list.to(dev).contiguous();
    Tensor out = at::empty_like(in);
    const int64_t total_D = in.size(-1);
    const int64_t B = in.numel() / total_D;
    check_status(tbe_b200_permute_pooled_embs(in.data_ptr(), B, total_D, static_cast<int32_t>(in.element_size()), total_D,
                                              total_D, off.data_ptr<int64_t>(), perm.data_ptr<int64_t>(),
                                              inv_off.data_ptr<int64_t>(), static_cast<int32_t>(perm.numel()),
                                              out.data_ptr(), nullptr, current_stream()),
                 "permute_pooled_embs");
    return out;
}

// Differentiable wrapper: the backward is the same permutation with the inverse
// lists (what the upstream module calls as permute_pooled_embs_auto_grad,
// bench/pooled_embedding/permute_pooled_embs/permute_pooled_embedding_modules.py:135).
class PermutePooledEmbsFunction : public torch::autograd::Function<PermutePooledEmbsFunction> {
public:
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& pooled_embs, const Tensor& offset_dim_list,
                          const Tensor& permute_list, const Tensor& inv_offset_dim_list, const Tensor& inv_permute_list)
    {
        ctx->save_for_backward({offset_dim_list, permute_list, inv_offset_dim_list, inv_permute_list});
        at::AutoDispatchBelowADInplaceOrView g;
        return permute_pooled_embs_cuda(pooled_embs, offset_dim_list, permute_list, inv_offset_dim_list, inv_permute_list);
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grad)
    {
        const auto saved = ctx->get_saved_variables();
        Tensor g = permute_pooled_embs_cuda(grad[0], saved[2], saved[3], saved[0], saved[1]);
        return {g, Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

Tensor permute_pooled_embs_auto_grad(const Tensor& pooled_embs, const Tensor& offset_dim_list, const Tensor& permute_list,
                                     const Tensor& inv_offset_dim_list, const Tensor& inv_permute_list)
{
    return PermutePooledEmbsFunction::apply(pooled_embs, offset_dim_list, permute_list, inv_offset_dim_list, inv_permute_list);
}

// ---- lengths -> offsets (asynchronous_complete_cumsum.cpp:14-57) -------------------------------

Tensor asynchronous_complete_cumsum_cuda(const Tensor& offset)
{
    check_cuda(offset, "offset");
    TORCH_CHECK(offset.dim() == 1, "offset must be 1D");
    TORCH_CHECK(offset.scalar_type() == at::kInt || offset.scalar_type() == at::kLong, "offset must be int32 or int64");
    const c10::cuda::CUDAGuard guard(offset.device());
    const Tensor in = offset.contiguous();
    const int64_t n = in.size(0);
    Tensor out = at::empty({n + 1}, in.options());
    const int64_t need = tbe_b200_complete_cumsum_scratch_bytes(n);
    Tensor scratch = at::empty({need}, in.options().dtype(at::kByte));   // caching-allocator blocks are 512-byte aligned
    check_status(tbe_b200_complete_cumsum(n ? in.data_ptr() : nullptr, n, in.scalar_type() == at::kInt ? 32 : 64, out.data_ptr(),
                                          need ? scratch.data_ptr() : nullptr, need, current_stream()),
                 "asynchronous_complete_cumsum");
    return out;
}

Tensor asynchronous_inclusive_cumsum_cuda(const Tensor& offset)
{
    if (offset.numel() == 0) return at::empty_like(offset);
    const Tensor all = asynchronous_complete_cumsum_cuda(offset);
    return all.narrow(0, 1, all.size(0) - 1);
}

Tensor asynchronous_exclusive_cumsum_cuda(const Tensor& offset)
{
    if (offset.numel() == 0) return at::empty_like(offset);
    const Tensor all = asynchronous_complete_cumsum_cuda(offset);
    return all.narrow(0, 0, all.size(0) - 1);
}

// ---- jagged request reordered by table (permute2d_sparse_data.cpp:45-150, permute1d_sparse_data.cpp:81-165) ----

using SparseTuple = std::tuple<Tensor, Tensor, std::optional<Tensor>>;

// lengths2d is [T_in, B]; the caller reshapes the returned lengths.
SparseTuple permute_sparse_common(const Tensor& permute, const Tensor& lengths2d, const Tensor& values,
                                  const std::optional<Tensor>& weights, const std::optional<int64_t>& permuted_lengths_sum,
                                  const char* op)
{
    check_cuda(permute, "permute");
    check_cuda(lengths2d, "lengths");
    check_cuda(values, "values");
    TORCH_CHECK(permute.dim() == 1, "permute must be 1D");
    TORCH_CHECK(permute.scalar_type() == at::kInt, "permute must be int32");
    TORCH_CHECK(lengths2d.scalar_type() == at::kInt || lengths2d.scalar_type() == at::kLong, "lengths must be int32 or int64");
    if (weights.has_value()) {
        check_cuda(*weights, "weights");
        TORCH_CHECK(weights->dim() == 1 || weights->dim() == 2, "weights must be 1D [L] or 2D [L, D]");
        TORCH_CHECK(weights->size(0) == values.size(0), "weights and values length mismatch: ", weights->size(0), " vs ", values.size(0));
    }
    if (permuted_lengths_sum.has_value())
        TORCH_CHECK(*permuted_lengths_sum >= 0, "permuted_lengths_sum must be non-negative, got ", *permuted_lengths_sum);
    const c10::cuda::CUDAGuard guard(values.device());
    const Tensor perm = permute.contiguous();
    const Tensor len = lengths2d.contiguous();
    const Tensor val = values.contiguous();
    const int64_t T_out = perm.size(0), T_in = len.size(0), B = len.size(1);
    if (T_in == 0 || B == 0 || T_out == 0)
        return SparseTuple(len.clone(), val.clone(), weights.has_value() ? std::make_optional(weights->contiguous().clone()) : std::nullopt);
    Tensor out_len = at::empty({T_out, B}, len.options());
    const int64_t sbytes = tbe_b200_permute_2d_sparse_scratch_bytes(T_in, T_out);
    Tensor scratch = at::empty({sbytes / 8}, len.options().dtype(at::kLong));
    check_status(tbe_b200_permute_2d_sparse_offsets(perm.data_ptr<int32_t>(), T_out, len.data_ptr(), len.scalar_type() == at::kInt ? 32 : 64,
                                                    T_in, B, out_len.data_ptr(), scratch.data_ptr(), sbytes, nullptr, current_stream()),
                 op);
    // Without permuted_lengths_sum the output size has to be read back, as in the reference (.item(), :106-112).
    const int64_t total = permuted_lengths_sum.has_value() ? *permuted_lengths_sum : scratch[sbytes / 8 - 1].item<int64_t>();
    Tensor out_val = at::empty({total}, val.options());
    std::optional<Tensor> out_w;
    Tensor w;
    int64_t w_row_bytes = 0;
    if (weights.has_value()) {
        w = weights->contiguous();
        const int64_t cols = w.dim() == 2 ? w.size(1) : 1;
        w_row_bytes = cols * w.element_size();
        out_w = w.dim() == 2 ? at::empty({total, cols}, w.options()) : at::empty({total}, w.options());
    }
    if (total > 0)
        check_status(tbe_b200_permute_2d_sparse_copy(perm.data_ptr<int32_t>(), T_out, T_in, val.data_ptr(), val.element_size(),
                                                     weights.has_value() ? w.data_ptr() : nullptr, w_row_bytes, out_val.data_ptr(),
                                                     out_w.has_value() ? out_w->data_ptr() : nullptr, total, scratch.data_ptr(),
                                                     current_stream()),
                     op);
    return SparseTuple(out_len, out_val, out_w);
}

SparseTuple permute_2d_sparse_data_cuda(const Tensor& permute, const Tensor& lengths, const Tensor& values,
                                        const std::optional<Tensor>& weights, std::optional<c10::SymInt> permuted_lengths_sum)
{
    TORCH_CHECK(lengths.dim() == 2, "lengths must be 2D");
    std::optional<int64_t> sum;
    if (permuted_lengths_sum.has_value()) sum = permuted_lengths_sum->guard_int(__FILE__, __LINE__);
    return permute_sparse_common(permute, lengths, values, weights, sum, "permute_2D_sparse_data");
}

SparseTuple permute_2d_sparse_data_input1d_cuda(const Tensor& permute, const Tensor& lengths, const Tensor& values, int64_t stride,
                                                const std::optional<Tensor>& weights, std::optional<c10::SymInt> permuted_lengths_sum)
{
    TORCH_CHECK(lengths.dim() == 1, "lengths must be 1D");
    TORCH_CHECK(stride > 0 && lengths.numel() % stride == 0, "lengths of ", lengths.numel(), " elements do not split into rows of ", stride);
    std::optional<int64_t> sum;
    if (permuted_lengths_sum.has_value()) sum = permuted_lengths_sum->guard_int(__FILE__, __LINE__);
    auto r = permute_sparse_common(permute, lengths.view({-1, stride}), values, weights, sum, "permute_2D_sparse_data_input1D");
    return SparseTuple(std::get<0>(r).view({-1}), std::get<1>(r), std::get<2>(r));
}

SparseTuple permute_1d_sparse_data_cuda(const Tensor& permute, const Tensor& lengths, const Tensor& values,
                                        const std::optional<Tensor>& weights, std::optional<c10::SymInt> permuted_lengths_sum)
{
    TORCH_CHECK(permute.dim() == 1, "permute must be 1D");
    TORCH_CHECK(lengths.dim() == 1, "lengths must be 1D");
    TORCH_CHECK(values.dim() == 1, "values must be 1D");
    if (weights.has_value()) TORCH_CHECK(weights->numel() > 0 || values.numel() == 0, "weights must not be empty");
    std::optional<int64_t> sum;
    if (permuted_lengths_sum.has_value()) sum = permuted_lengths_sum->guard_int(__FILE__, __LINE__);
    auto r = permute_sparse_common(permute, lengths.view({-1, 1}), values, weights, sum, "permute_1D_sparse_data");
    return SparseTuple(std::get<0>(r).view({-1}), std::get<1>(r), std::get<2>(r));
}

bool has_schema(const char* qualified_name)
{
    return c10::Dispatcher::singleton().findSchema({qualified_name, ""}).has_value();
}

void def_if_absent(torch::Library& m, const char* ns, const char* name, const char* schema)
{
    const std::string q = std::string(ns) + "::" + name;
    if (!has_schema(q.c_str())) m.def(schema);
}

void def_sparse_schemas(torch::Library& m, const char* ns)
{
    def_if_absent(m, ns, "asynchronous_complete_cumsum", "asynchronous_complete_cumsum(Tensor offset) -> Tensor");
    def_if_absent(m, ns, "asynchronous_inclusive_cumsum", "asynchronous_inclusive_cumsum(Tensor offset) -> Tensor");
    def_if_absent(m, ns, "asynchronous_exclusive_cumsum", "asynchronous_exclusive_cumsum(Tensor offset) -> Tensor");
    def_if_absent(m, ns, "permute_2D_sparse_data",
                  "permute_2D_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)");
    def_if_absent(m, ns, "permute_sparse_data",
                  "permute_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)");
    def_if_absent(m, ns, "permute_2D_sparse_data_input1D",
                  "permute_2D_sparse_data_input1D(Tensor permute, Tensor lengths, Tensor values, int stride, Tensor? weights=None, "
                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)");
    def_if_absent(m, ns, "permute_1D_sparse_data",
                  "permute_1D_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights=None, "
                  "SymInt? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)");
}

void impl_sparse(torch::Library& m)
{
    m.impl("asynchronous_complete_cumsum", TORCH_FN(asynchronous_complete_cumsum_cuda));
    m.impl("asynchronous_inclusive_cumsum", TORCH_FN(asynchronous_inclusive_cumsum_cuda));
    m.impl("asynchronous_exclusive_cumsum", TORCH_FN(asynchronous_exclusive_cumsum_cuda));
    m.impl("permute_2D_sparse_data", TORCH_FN(permute_2d_sparse_data_cuda));
    m.impl("permute_sparse_data", TORCH_FN(permute_2d_sparse_data_cuda));
    m.impl("permute_2D_sparse_data_input1D", TORCH_FN(permute_2d_sparse_data_input1d_cuda));
    m.impl("permute_1D_sparse_data", TORCH_FN(permute_1d_sparse_data_cuda));
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(fbgemm, m)
{
    def_if_absent(m, "fbgemm", "int_nbit_split_embedding_codegen_lookup_function",
                  "int_nbit_split_embedding_codegen_lookup_function(Tensor dev_weights, Tensor uvm_weights, "
                  "Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys, Tensor D_offsets, int total_D, "
                  "int max_int2_D, int max_int4_D, int max_int8_D, int max_float16_D, int max_float32_D, Tensor indices, "
                  "Tensor offsets, int pooling_mode, Tensor? indice_weights, int output_dtype=1, "
                  "Tensor? lxu_cache_weights=None, Tensor? lxu_cache_locations=None, int? row_alignment=None, "
                  "int? max_float8_D=0, int? fp8_exponent_bits=-1, int? fp8_exponent_bias=-1) -> Tensor");
    def_if_absent(m, "fbgemm", "FloatToFused8BitRowwiseQuantized", "FloatToFused8BitRowwiseQuantized(Tensor t) -> Tensor");
    def_if_absent(m, "fbgemm", "HalfToFused8BitRowwiseQuantized", "HalfToFused8BitRowwiseQuantized(Tensor t) -> Tensor");
    def_if_absent(m, "fbgemm", "Fused8BitRowwiseQuantizedToFloat", "Fused8BitRowwiseQuantizedToFloat(Tensor input) -> Tensor");
    def_if_absent(m, "fbgemm", "Fused8BitRowwiseQuantizedToHalf", "Fused8BitRowwiseQuantizedToHalf(Tensor input) -> Tensor");
    def_if_absent(m, "fbgemm", "FloatToFusedNBitRowwiseQuantizedSBHalf",
                  "FloatToFusedNBitRowwiseQuantizedSBHalf(Tensor input, int bit_rate) -> Tensor");
    def_if_absent(m, "fbgemm", "FusedNBitRowwiseQuantizedSBHalfToFloat",
                  "FusedNBitRowwiseQuantizedSBHalfToFloat(Tensor input, int bit_rate) -> Tensor");
    def_if_absent(m, "fbgemm", "permute_pooled_embs",
                  "permute_pooled_embs(Tensor pooled_embs, Tensor offset_dim_list, Tensor permute_list, "
                  "Tensor inv_offset_dim_list, Tensor inv_permute_list) -> Tensor");
    def_if_absent(m, "fbgemm", "permute_pooled_embs_auto_grad",
                  "permute_pooled_embs_auto_grad(Tensor pooled_embs, Tensor offset_dim_list, Tensor permute_list, "
                  "Tensor inv_offset_dim_list, Tensor inv_permute_list) -> Tensor");
    def_sparse_schemas(m, "fbgemm");
}

TORCH_LIBRARY_IMPL(fbgemm, CUDA, m)
{
    impl_sparse(m);
    m.impl("int_nbit_split_embedding_codegen_lookup_function", TORCH_FN(int_nbit_split_embedding_codegen_lookup_function_cuda));
    m.impl("FloatToFused8BitRowwiseQuantized", TORCH_FN(float_to_fused8bit));
    m.impl("HalfToFused8BitRowwiseQuantized", TORCH_FN(half_to_fused8bit));
    m.impl("Fused8BitRowwiseQuantizedToFloat", TORCH_FN(fused8bit_to_float));
    m.impl("Fused8BitRowwiseQuantizedToHalf", TORCH_FN(fused8bit_to_half));
    m.impl("FloatToFusedNBitRowwiseQuantizedSBHalf", TORCH_FN(float_to_fused_nbit_sbhalf));
    m.impl("FusedNBitRowwiseQuantizedSBHalfToFloat", TORCH_FN(fused_nbit_sbhalf_to_float));
    m.impl("permute_pooled_embs", TORCH_FN(permute_pooled_embs_cuda));
}

TORCH_LIBRARY_IMPL(fbgemm, Autograd, m)
{
    m.impl("permute_pooled_embs_auto_grad", TORCH_FN(permute_pooled_embs_auto_grad));
}

// The reference also exposes these operators under its own namespace
// (permute_pooled_embs.cpp:107-117, asynchronous_complete_cumsum.cpp:55-67, permute2d_sparse_data.cpp:152-175).
TORCH_LIBRARY_FRAGMENT(mxrec, m)
{
    def_sparse_schemas(m, "mxrec");
    def_if_absent(m, "mxrec", "permute_pooled_embs",
                  "permute_pooled_embs(Tensor pooled_embs, Tensor offset_dim_list, Tensor permute_list, "
                  "Tensor inv_offset_dim_list, Tensor inv_permute_list) -> Tensor");
}

TORCH_LIBRARY_IMPL(mxrec, CUDA, m)
{
    m.impl("permute_pooled_embs", TORCH_FN(permute_pooled_embs_cuda));
    impl_sparse(m);
}

// Helpers with no upstream counterpart.
TORCH_LIBRARY_FRAGMENT(tbe_b200, m)
{
    m.def("quantize_to_table_rows(Tensor input, int weight_ty, int row_bytes) -> Tensor");
    m.def("pack_table_rows(Tensor fused, int src_bits, int ncols, int row_bytes) -> Tensor");
}

TORCH_LIBRARY_IMPL(tbe_b200, CUDA, m)
{
    m.impl("quantize_to_table_rows", TORCH_FN(quantize_to_table_rows));
    m.impl("pack_table_rows", TORCH_FN(pack_table_rows));
}
