/*
 * tbe_b200 -- C ABI of the B200 (sm_100a) quantized table-batched-embedding
 * inference library (libtbe_b200.so).
 *
 * This is the boundary a host framework binds to.  It plays the role that the
 * per-operator C entry points of libcust_opapi.so play in the reference
 * (aclnn<Op>GetWorkspaceSize + aclnn<Op>, looked up and called by EXEC_NPU_CMD,
 * src/common/pytorch_npu_helper.hpp:536-585): plain pointers and sizes in, an int
 * status out, work enqueued asynchronously on the stream the caller names.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the current CUDA device unless the
 *     comment says "host".  The library never allocates, frees or synchronises.
 *   - Every call returns TBE_B200_OK (0) or a negative tbe_b200_status; the
 *     message of the last failure on the calling thread is tbe_b200_last_error().
 *   - Calls are re-entrant and may be issued from any thread (the only state kept between calls is a
 *     per-device cache of device properties, updated atomically).
 *   - `stream` is a cudaStream_t (0 = the default stream).
 */
#ifndef TBE_B200_H_
#define TBE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tbe_b200_stream_t;

typedef enum {
    TBE_B200_OK = 0,
    TBE_B200_ERR_INVALID_ARGUMENT = -1,
    TBE_B200_ERR_UNSUPPORTED = -2,
    TBE_B200_ERR_CUDA = -3
} tbe_b200_status;

/* Weight / output element types: SparseType of
 * int_nbit_split_embedding_codegen_lookup_function.cpp:24-33. */
typedef enum {
    TBE_B200_FP32 = 0,
    TBE_B200_FP16 = 1,
    TBE_B200_INT8 = 2,
    TBE_B200_INT4 = 3,
    TBE_B200_INT2 = 4,
    TBE_B200_BF16 = 5,
    TBE_B200_FP8 = 6
} tbe_b200_sparse_type;

/* PoolingMode of int_nbit_split_embedding_codegen_lookup_function.cpp:18-22. */
typedef enum { TBE_B200_POOL_SUM = 0, TBE_B200_POOL_MEAN = 1, TBE_B200_POOL_NONE = 2 } tbe_b200_pooling_mode;

/*
 * Arguments of the pooled / sequence lookup.  Replaces the argument list that
 * int_nbit_split_embedding_codegen_lookup_function_npu hands to
 * aclnnIntNbitSplitEmbeddingCodegenLookupFunction
 * (int_nbit_split_embedding_codegen_lookup_function.cpp:139-165) together with the
 * tiling data the host computes for it
 * (c310/op_host/int_nbit_split_embedding_codegen_lookup_function_tiling.h:20-43).
 *
 * Geometry: T tables, B bags per table; bag i = t*B + b owns
 * indices[offsets[i] .. offsets[i+1]); table t starts at byte weights_offsets[t]
 * of dev_weights; a row of table t is
 *   [fp16 scale][fp16 bias][payload]   for INT8 / INT4 / INT2
 *   [payload]                          for FP32 / FP16 / FP8
 * padded to a multiple of row_alignment bytes; D_t = D_offsets[t+1]-D_offsets[t].
 *
 * Pooled modes write bag (t, b) to
 *   dst(b) + (b % rows_per_dest) * output_stride + col(t)
 * where col(t) = output_col_offsets ? output_col_offsets[t] : D_offsets[t] and
 * dst(b) = dest_outputs ? dest_outputs[b / rows_per_dest] : output (in which
 * case rows_per_dest is ignored and b is used as is).  The two optional fields
 * let one launch pool, scatter the batch over several destination buffers
 * (peer GPUs' memory included) and place each table at its final, permuted
 * column in one pass; leave them NULL for the plain operator.
 * An empty bag writes zeros.  Index -1 contributes nothing but counts in MEAN.
 *
 * Pooling NONE writes row n of `indices` to output + n*output_stride, D_t
 * elements wide.
 */
typedef struct {
    const uint8_t* dev_weights;         /* all tables, flat bytes */
    int64_t dev_weights_bytes;          /* size of dev_weights; 0 = unknown.  When known, a row that would end past
                                           its table (the next table's start, or the end of dev_weights) is skipped */
    const int64_t* weights_offsets;     /* [T] byte offset of each table */
    const uint8_t* weights_tys;         /* [T] tbe_b200_sparse_type per table */
    const int32_t* D_offsets;           /* [T+1] prefix sum of the tables' D */
    int32_t T;
    int64_t B;
    int64_t total_D;                    /* D_offsets[T] */
    int32_t max_D;                      /* max over tables of D_t (host-known; sizes the launch) */
    const void* indices;                /* [N] int32 or int64 */
    const void* offsets;                /* [T*B+1], same width as indices */
    int32_t index_bits;                 /* 32 or 64 */
    int64_t num_indices;                /* N */
    const float* indice_weights;        /* [N] per-sample weights, or NULL */
    int32_t pooling_mode;               /* tbe_b200_pooling_mode */
    int32_t output_dtype;               /* TBE_B200_FP32 / FP16 / BF16 */
    int32_t row_alignment;              /* bytes; the operator's default is 16 */
    int32_t fp8_exponent_bits;          /* FP8 tables only */
    int32_t fp8_exponent_bias;          /* FP8 tables only */
    void* output;                       /* [B, output_stride] (pooled) or [N, output_stride] (NONE) */
    int64_t output_stride;              /* elements between consecutive output rows */
    const int64_t* output_col_offsets;  /* [T] or NULL (pooled modes) */
    void* const* dest_outputs;          /* [ceil(B / rows_per_dest)] device array of base pointers, or NULL */
    int64_t rows_per_dest;              /* used only with dest_outputs */
    int32_t* error_flag;                /* optional device word, or'ed with
                                             1  an index outside [-1, 2^31) was met (that row is skipped),
                                             4  an index at or past the end of its table was met (dev_weights_bytes
                                                known; the row is skipped like -1 and never read),
                                             8  offsets[T*B] != num_indices, or offsets that point outside
                                                `indices` (such bags are not read and come out as empty ones);
                                           NULL = no reporting (the checks that skip rows are made all the same) */
} tbe_b200_lookup_args;

/* Pooled (SUM / MEAN) or sequence (NONE) lookup over fused INT8 / INT4 / INT2 /
 * FP16 / FP32 / FP8 rows; fp32 accumulation; output cast round-to-nearest-even.
 * Replaces aclnnIntNbitSplitEmbeddingCodegenLookupFunction
 * (c310/op_kernel/int_nbit_split_embedding_codegen_lookup_function.cpp:58-89). */
int tbe_b200_int_nbit_lookup(const tbe_b200_lookup_args* args, tbe_b200_stream_t stream);

/* FloatToFused8BitRowwiseQuantized: fp32 (or fp16 when in_is_half) [nrows, ncols]
 * -> uint8 [nrows, ncols + 8]: codes, fp32 scale, fp32 bias.  Upstream fbgemm op
 * that the reference inherits through `import fbgemm_gpu`
 * (fbgemm_ascend/__init__.py:9). */
int tbe_b200_quantize_8bit_rowwise(const void* input, int32_t in_is_half, int64_t nrows, int64_t ncols,
                                   uint8_t* output, tbe_b200_stream_t stream);

/* Fused8BitRowwiseQuantizedToFloat (or ...ToHalf when out_is_half):
 * uint8 [nrows, ncols_q] -> [nrows, ncols_q - 8]. */
int tbe_b200_dequantize_8bit_rowwise(const uint8_t* input, int64_t nrows, int64_t ncols_q, void* output,
                                     int32_t out_is_half, tbe_b200_stream_t stream);

/* FloatToFusedNBitRowwiseQuantizedSBHalf, bit_rate 2 or 4: fp32 [nrows, ncols] ->
 * uint8 [nrows, ncols*bit_rate/8 + 4]: packed codes, fp16 scale, fp16 bias. */
int tbe_b200_quantize_nbit_rowwise_sbhalf(int32_t bit_rate, const float* input, int64_t nrows, int64_t ncols,
                                          uint8_t* output, tbe_b200_stream_t stream);

/* FusedNBitRowwiseQuantizedSBHalfToFloat: inverse of the above. */
int tbe_b200_dequantize_nbit_rowwise_sbhalf(int32_t bit_rate, const uint8_t* input, int64_t nrows,
                                            int64_t ncols_q, float* output, tbe_b200_stream_t stream);

/* Turn quantizer output rows into table rows: move the scale/bias pair to the
 * front as fp16 (8-bit rows: fp32 -> fp16 round-to-nearest-even; n-bit rows:
 * already fp16) and pad each row to row_bytes.  src_bits 8, 4 or 2.  This is the
 * layout step the upstream inference module performs when weights are assigned
 * (exercised by the reference through split_embedding_weights(),
 * test_int_nbit_split_embedding_codegen_lookup_function.py:144-156). */
int tbe_b200_pack_table_rows(int32_t src_bits, const uint8_t* fused, int64_t nrows, int64_t ncols,
                             int64_t row_bytes, uint8_t* rows, tbe_b200_stream_t stream);

/* Quantize fp32 [nrows, ncols] straight into table rows of weight type
 * weight_ty (INT8, INT4, INT2: quantizer + header-first packing in one pass, same
 * bytes as the quantizer followed by tbe_b200_pack_table_rows; FP16: a
 * round-to-nearest-even cast), row stride row_bytes, padding zeroed.  For building
 * tables too large to hold the intermediate quantizer output. */
int tbe_b200_quantize_to_table_rows(int32_t weight_ty, const float* input, int64_t nrows, int64_t ncols,
                                    int64_t row_bytes, uint8_t* rows, tbe_b200_stream_t stream);

/* permute_pooled_embs: out[:, inv_offset_dim_list[i] .. inv_offset_dim_list[i+1]) =
 * in[:, offset_dim_list[p] .. offset_dim_list[p+1]), p = permute_list[i].
 * Replaces aclnnPermutePooledEmbs (permute_pooled_embs.cpp:100-101; kernel
 * v220/op_kernel/permute_pooled_embs_kernel.h:173-211).  elem_bytes 2 or 4.
 * in_stride / out_stride: elements between consecutive rows.  A permute entry
 * outside [0, T) copies nothing for that feature and sets *error_flag (if given). */
int tbe_b200_permute_pooled_embs(const void* pooled_embs, int64_t B, int64_t total_D, int32_t elem_bytes,
                                 int64_t in_stride, int64_t out_stride, const int64_t* offset_dim_list,
                                 const int64_t* permute_list, const int64_t* inv_offset_dim_list, int32_t T,
                                 void* output, int32_t* error_flag, tbe_b200_stream_t stream);

/* The same permutation over a source that is held as consecutive column blocks:
 * source column c is read from
 *   pooled_embs + (c / block_cols) * block_stride + row * in_stride + c % block_cols
 * (elements).  This is the layout an all-to-all of pooled rows leaves behind (one
 * [B, block_cols] block per sending rank), so the exchange buffer is permuted into
 * feature order without first being concatenated.  No counterpart in the reference,
 * which has no multi-device code. */
int tbe_b200_permute_pooled_embs_blocked(const void* pooled_embs, int64_t B, int64_t total_D, int32_t elem_bytes,
                                         int64_t in_stride, int64_t out_stride, int64_t block_cols,
                                         int64_t block_stride, const int64_t* offset_dim_list,
                                         const int64_t* permute_list, const int64_t* inv_offset_dim_list, int32_t T,
                                         void* output, int32_t* error_flag, tbe_b200_stream_t stream);

/* ---- producers of the lookup's inputs -------------------------------------------------------- */

/* Complete cumulative sum: out[0] = 0, out[i + 1] = in[0] + ... + in[i]; `in` has n elements of
 * index_bits (32 or 64) bits, `out` n + 1 of the same type (sums wrap like the integer type does).
 * Replaces aclnnAsynchronousCompleteCumsum, reached from asynchronous_complete_cumsum_npu
 * (src/sparse_ops/asynchronous_complete_cumsum/asynchronous_complete_cumsum.cpp:14-37); the inclusive and
 * exclusive forms (:39-57) are views of this result.  Inputs longer than 8192 elements need scratch:
 * tbe_b200_complete_cumsum_scratch_bytes(n) bytes of device memory (0 for short inputs, then scratch may be
 * NULL; 16 bytes per 8192 elements otherwise), 8-byte aligned, overwritten by the call.  The call puts one small
 * memset of the scratch and one kernel on the stream; the input is read once.  Two calls that may overlap need
 * separate scratch. */
int64_t tbe_b200_complete_cumsum_scratch_bytes(int64_t n);
int tbe_b200_complete_cumsum(const void* in, int64_t n, int index_bits, void* out, void* scratch, int64_t scratch_bytes,
                             tbe_b200_stream_t stream);

/* Complete cumulative sum that allocates nothing and takes no scratch from the caller.  It has no counterpart
 * in the reference.  It exists for hosts that cannot hand the library any extra device memory at call time:
 * a serving process that reserved the whole GPU for its tables at start-up and never calls the CUDA allocator
 * again (an allocation there can fail, or stall every stream of the device while it runs), or a runtime whose
 * memory arena is owned by another component.  The per-tile sums go into a 64 KB array that is part of the
 * library image; every GPU that loads the library holds those 64 KB until the process exits.
 *   - n may be at most tbe_b200_complete_cumsum_static_max_elements() (16 777 216); a longer input is refused
 *     with TBE_B200_ERR_UNSUPPORTED and a message that names the limit.
 *   - The first call on each device looks the array's device address up once, with that device current; make
 *     that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps what the last call left there.  Nothing in it has
 *     to start at zero, but two calls whose kernels can run at the same time (different streams, no ordering
 *     between them) race on it: order them, or give one of them tbe_b200_complete_cumsum with its own scratch.
 * Same result as tbe_b200_complete_cumsum, bit for bit. */
int64_t tbe_b200_complete_cumsum_static_max_elements(void);
int tbe_b200_complete_cumsum_static(const void* in, int64_t n, int index_bits, void* out, tbe_b200_stream_t stream);

/* Reordering of a jagged request by table; replaces aclnnPermute2dSparseData, reached from
 * permute2d_sparse_data_impl_npu (src/sparse_ops/permute2d_sparse_data/permute2d_sparse_data.cpp:45-150) and, with
 * B = 1, permute1d_sparse_data_impl_npu (permute1d_sparse_data.cpp:81-165).  `lengths` is [T_in, B] (int32 or
 * int64); table t owns the next sum(lengths[t, :]) entries of `values` (and rows of `weights`).  Output table i
 * is input table permute[i] (int32; entries may repeat, T_out need not equal T_in):
 *     out_lengths[i, :] = lengths[permute[i], :]
 *     out_values  = values of table permute[0], then of permute[1], ...     (weights alike)
 * Two calls, so that a caller that does not know the output size can read it in between:
 *   _offsets  fills out_lengths and the scratch: seg_len[T_in], in_off[T_in + 1], out_off[T_out + 1], all
 *             int64; out_off[T_out] (the last word) is the number of output values.
 *   _copy     moves min(out_capacity, out_off[T_out]) values of value_bytes each, and as many weight rows of
 *             weight_row_bytes (weights may be NULL), using the scratch the first call left.
 * scratch: tbe_b200_permute_2d_sparse_scratch_bytes(T_in, T_out) bytes of device memory, 8-byte aligned.
 * A permute entry outside [0, T_in) stands for an empty table and sets *error_flag (if given). */
int64_t tbe_b200_permute_2d_sparse_scratch_bytes(int64_t T_in, int64_t T_out);
int tbe_b200_permute_2d_sparse_offsets(const int32_t* permute, int64_t T_out, const void* lengths, int lengths_bits,
                                       int64_t T_in, int64_t B, void* out_lengths, void* scratch, int64_t scratch_bytes,
                                       int32_t* error_flag, tbe_b200_stream_t stream);
int tbe_b200_permute_2d_sparse_copy(const int32_t* permute, int64_t T_out, int64_t T_in, const void* values,
                                    int64_t value_bytes, const void* weights, int64_t weight_row_bytes, void* out_values,
                                    void* out_weights, int64_t out_capacity, const void* scratch,
                                    tbe_b200_stream_t stream);

/* The copy step with several output buffers (no counterpart in the reference, which has no multi-device code): output
 * table i belongs to destination i / tables_per_dest, and the values of a destination's tables land one after the
 * other from dest_bases[destination] on.  dest_bases is a device array of T_out / tables_per_dest addresses, each
 * 16-byte aligned and writable from this GPU -- local memory or a peer's (the stores then cross NVLink; this is how
 * the index all-to-all in front of a table-wise sharded lookup is folded into the permute).  A destination takes at
 * most dest_capacity values; values beyond are dropped and bit 2 is or'ed into *error_flag (if given).  total_hint
 * is an upper bound of the number of values (it sizes the grid; the input size will do).  `scratch` is what
 * tbe_b200_permute_2d_sparse_offsets left.  Completion at a peer is the caller's business
 * (tbe_b200_signal_peers / tbe_b200_wait_flags on the same stream). */
int tbe_b200_permute_2d_sparse_copy_to_dests(const int32_t* permute, int64_t T_out, int64_t T_in, const void* values,
                                             int64_t value_bytes, const int64_t* dest_bases, int64_t tables_per_dest,
                                             int64_t dest_capacity, int64_t total_hint, const void* scratch,
                                             int32_t* error_flag, tbe_b200_stream_t stream);

/* ---- step flags of a table-wise sharded lookup (one process per GPU) ---------------------------- */

/* A rank tells its peers that the pooled rows it stored into their output buffers for step `value` are in place:
 * it writes `value` to peer_flags[r][my_rank] for every rank r (its own included).  peer_flags is a DEVICE array of
 * `world` pointers, each to a peer-mapped array of `world` int64 flags in rank r's memory.  Enqueue it on the stream
 * of the lookup, after the lookup: the flag is ordered after everything the GPU wrote before this call (release at
 * system scope).  Plain peer stores; no multicast.  The reference has no multi-device code and no counterpart. */
int tbe_b200_signal_peers(int64_t* const* peer_flags, int32_t world, int32_t my_rank, int64_t value,
                          tbe_b200_stream_t stream);

/* Waits on the device until flags[r] >= value for every r < world (flags: this rank's own array, written by the
 * peers' tbe_b200_signal_peers).  The wait is bounded: a flag that is not up after max_polls polls (about a
 * microsecond apart) sets bit 16 of *error_flag (if given) and the kernel returns, so the stream always drains;
 * the caller reads the word to learn that a peer is late or gone.  No counterpart in the reference. */
int tbe_b200_wait_flags(const int64_t* flags, int32_t world, int64_t value, int64_t max_polls, int32_t* error_flag,
                        tbe_b200_stream_t stream);

/* Message of the last failure on the calling thread ("" if none).  Host pointer,
 * valid until the next failing call on the same thread. */
const char* tbe_b200_last_error(void);

/* Library version, major*10000 + minor*100 + patch. */
int tbe_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* TBE_B200_H_ */
