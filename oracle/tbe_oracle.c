/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * Plain-C restatement of the CPU semantics of the quantized table-batched-
 * embedding (TBE) inference path, used only as the checker in tests, in the
 * smoke test and as the timed "port" CPU baseline of the benchmark.  The GPU
 * library never links, loads or calls anything in this file.
 *
 * The arithmetic of this path lives in a third-party dependency of the
 * reference (fbgemm_gpu 1.2.0+cpu, requirements.txt:4; imported at
 * fbgemm_ascend/__init__.py:9), which is not vendored.  The functions below
 * restate its published algorithm; each one names the reference call site
 * whose behaviour it stands for.  Parity is pinned (tests/test_oracle_pins.py)
 * against
 *   - the FBGEMM CPU kernels that ship inside libtorch_cpu.so
 *     (oracle/fbgemm_cpu_ref.cpp), the library the upstream CPU op is built on,
 *   - torch.ops.quantized.embedding_bag_{byte,4bit}_{prepack,unpack,
 *     rowwise_offsets}, built on the same library,
 *   - the known-answer vectors of the reference's own permute tests
 *     (bench/pooled_embedding/permute_pooled_embs/permute_pooled_embedding_test.py:79-86,
 *      permute_pooled_embedding_modules.py:45-80).
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- scalar type conversions (IEEE round-to-nearest-even) ---------------- */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

uint16_t orc_f32_to_f16(float f)
{
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) {                       /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x38800000u) {                        /* subnormal half or zero */
        if (absx < 0x33000000u) return (uint16_t)sign;      /* < 2^-25 -> 0 */
        int e = (int)(absx >> 23);                   /* biased exponent, 102..112 */
        uint32_t man = (absx & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;                         /* 14..24 */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t r = absx - 0x38000000u;                 /* rebias 127 -> 15 */
    uint32_t q = r >> 13;
    uint32_t rem = r & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        float v = (float)m * (1.0f / 16777216.0f);   /* m * 2^-24, exact */
        return (sign ? -v : v);
    }
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

uint16_t orc_f32_to_bf16(float f)
{
    uint32_t x = f32_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

float orc_bf16_to_f32(uint16_t h) { return bits_f32(((uint32_t)h) << 16); }

/* ---- rowwise quantizers --------------------------------------------------- */

/*
 * FloatToFused8BitRowwiseQuantized: fp32 [N, D] -> uint8 [N, D + 8]; each row is
 * D quantized bytes, then fp32 scale, then fp32 bias.  The op is not defined in
 * the reference tree; it reaches users through `import fbgemm_gpu`
 * (fbgemm_ascend/__init__.py:9).  Arithmetic: bias = row min, scale =
 * (max - min) / 255, q = rint((x - min) * (255 / (max - min + 1e-8))), all fp32.
 */
void orc_quantize_8bit_rowwise(const float* in, int64_t N, int64_t D, uint8_t* out)
{
    const int64_t ostride = D + 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const float* x = in + r * D;
        uint8_t* o = out + r * ostride;
        float mn = 0.0f, mx = 0.0f;
        if (D > 0) {
            mn = x[0]; mx = x[0];
            for (int64_t c = 1; c < D; ++c) {
                if (x[c] < mn) mn = x[c];
                if (x[c] > mx) mx = x[c];
            }
        }
        const float range = mx - mn;
        const float scale = range / 255.0f;
        const float inv = 255.0f / (range + 1e-8f);
        for (int64_t c = 0; c < D; ++c) {
            o[c] = (uint8_t)lrintf((x[c] - mn) * inv);
        }
        memcpy(o + D, &scale, 4);
        memcpy(o + D + 4, &mn, 4);
    }
}

/*
 * Fused8BitRowwiseQuantizedToFloat: uint8 [N, D + 8] -> fp32 [N, D];
 * x = fma(q, scale, bias).
 */
void orc_dequantize_8bit_rowwise(const uint8_t* in, int64_t N, int64_t Dq, float* out)
{
    const int64_t D = Dq - 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const uint8_t* q = in + r * Dq;
        float scale, bias;
        memcpy(&scale, q + D, 4);
        memcpy(&bias, q + D + 4, 4);
        for (int64_t c = 0; c < D; ++c) out[r * D + c] = fmaf((float)q[c], scale, bias);
    }
}

/*
 * FloatToFusedNBitRowwiseQuantizedSBHalf (bit_rate 2 or 4): fp32 [N, D] ->
 * uint8 [N, D*bit_rate/8 + 4]; packed codes (element j of a byte sits at bit
 * (j % per_byte) * bit_rate), then fp16 scale, then fp16 bias.  Needed to build
 * INT4 tables; upstream op, same provenance as the 8-bit one.
 */
void orc_quantize_nbit_rowwise_sbhalf(int bit_rate, const float* in, int64_t N, int64_t D, uint8_t* out)
{
    const int per_byte = 8 / bit_rate;
    const int64_t pbytes = (D + per_byte - 1) / per_byte;
    const int64_t ostride = pbytes + 4;
    const int qmax = (1 << bit_rate) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const float* x = in + r * D;
        uint8_t* o = out + r * ostride;
        float mn = 0.0f, mx = 0.0f;
        if (D > 0) {
            mn = x[0]; mx = x[0];
            for (int64_t c = 1; c < D; ++c) {
                if (x[c] < mn) mn = x[c];
                if (x[c] > mx) mx = x[c];
            }
        }
        uint16_t bias_h = orc_f32_to_f16(mn);
        const float bias = orc_f16_to_f32(bias_h);
        const float range = mx - bias;
        float scale = (range == 0.0f) ? 1.0f : range / (float)qmax;
        uint16_t scale_h = orc_f32_to_f16(scale);
        scale = orc_f16_to_f32(scale_h);
        if (scale == 0.0f) {
            scale = 1.0f;
            scale_h = orc_f32_to_f16(1.0f);
        }
        float inv = 1.0f / scale;
        if (isinf(inv)) {
            scale = 1.0f;
            scale_h = orc_f32_to_f16(1.0f);
            inv = 1.0f;
        }
        memset(o, 0, (size_t)pbytes);
        for (int64_t c = 0; c < D; ++c) {
            long q = lrintf((x[c] - bias) * inv);
            if (q < 0) q = 0;
            if (q > qmax) q = qmax;
            o[c / per_byte] |= (uint8_t)(q << ((c % per_byte) * bit_rate));
        }
        memcpy(o + pbytes, &scale_h, 2);
        memcpy(o + pbytes + 2, &bias_h, 2);
    }
}

void orc_dequantize_nbit_rowwise_sbhalf(int bit_rate, const uint8_t* in, int64_t N, int64_t Dq, float* out)
{
    const int per_byte = 8 / bit_rate;
    const int64_t pbytes = Dq - 4;
    const int64_t D = pbytes * per_byte;
    const int mask = (1 << bit_rate) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const uint8_t* q = in + r * Dq;
        uint16_t sh, bh;
        memcpy(&sh, q + pbytes, 2);
        memcpy(&bh, q + pbytes + 2, 2);
        const float scale = orc_f16_to_f32(sh), bias = orc_f16_to_f32(bh);
        for (int64_t c = 0; c < D; ++c) {
            int v = (q[c / per_byte] >> ((c % per_byte) * bit_rate)) & mask;
            out[r * D + c] = fmaf((float)v, scale, bias);
        }
    }
}

/* ---- TBE row geometry ----------------------------------------------------- */

enum { ORC_FP32 = 0, ORC_FP16 = 1, ORC_INT8 = 2, ORC_INT4 = 3, ORC_INT2 = 4, ORC_BF16 = 5, ORC_FP8 = 6 };
enum { ORC_SUM = 0, ORC_MEAN = 1, ORC_NONE = 2 };

/*
 * Bytes of one row of a table: header (fp16 scale + fp16 bias for the integer
 * types) + payload, rounded up to row_alignment.  SparseType values follow
 * int_nbit_split_embedding_codegen_lookup_function.cpp:24-33; the FP8 rule
 * (payload only, padded) is int_nbit_split_embedding_pooling_kernel.h:241.
 */
int64_t orc_row_bytes(int ty, int64_t D, int64_t row_alignment)
{
    int64_t b;
    switch (ty) {
        case ORC_FP32: b = 4 * D; break;
        case ORC_FP16: b = 2 * D; break;
        case ORC_BF16: b = 2 * D; break;
        case ORC_FP8:  b = D; break;
        case ORC_INT8: b = D + 4; break;
        case ORC_INT4: b = (D + 1) / 2 + 4; break;
        case ORC_INT2: b = (D + 3) / 4 + 4; break;
        default: return -1;
    }
    if (row_alignment > 1) b = (b + row_alignment - 1) / row_alignment * row_alignment;
    return b;
}

/*
 * FP8 byte -> fp32 with a configurable exponent width and bias, by bit
 * placement: body = (b & 0x7f) << (16 + ebits) reinterpreted as fp32, times
 * 2^(127 - bias) (encoded as (254 - bias) << 23), then the sign bit or'ed in.
 * Restates c310/op_kernel/common.h:120-167 (InitFp8Params, FP8U8ToFP32Bitpack).
 */
float orc_fp8_to_f32(uint8_t b, int ebits, int ebias)
{
    uint32_t body = ((uint32_t)(b & 0x7f)) << (16 + ebits);
    float mult = bits_f32(((uint32_t)(254 - ebias)) << 23);
    float v = bits_f32(body) * mult;
    return bits_f32(f32_bits(v) | (((uint32_t)(b & 0x80)) << 24));
}

static inline void row_to_f32(const uint8_t* row, int ty, int64_t D, int ebits, int ebias, float* v)
{
    switch (ty) {
        case ORC_FP32: memcpy(v, row, (size_t)(4 * D)); break;
        case ORC_FP16:
            for (int64_t j = 0; j < D; ++j) { uint16_t h; memcpy(&h, row + 2 * j, 2); v[j] = orc_f16_to_f32(h); }
            break;
        case ORC_BF16:
            for (int64_t j = 0; j < D; ++j) { uint16_t h; memcpy(&h, row + 2 * j, 2); v[j] = orc_bf16_to_f32(h); }
            break;
        case ORC_FP8:
            for (int64_t j = 0; j < D; ++j) v[j] = orc_fp8_to_f32(row[j], ebits, ebias);
            break;
        default: {
            uint16_t sh, bh;
            memcpy(&sh, row, 2);
            memcpy(&bh, row + 2, 2);
            const float scale = orc_f16_to_f32(sh), bias = orc_f16_to_f32(bh);
            const uint8_t* p = row + 4;
            if (ty == ORC_INT8) {
                for (int64_t j = 0; j < D; ++j) v[j] = fmaf((float)p[j], scale, bias);
            } else if (ty == ORC_INT4) {
                for (int64_t j = 0; j < D; ++j) v[j] = fmaf((float)((p[j >> 1] >> ((j & 1) * 4)) & 0xf), scale, bias);
            } else {
                for (int64_t j = 0; j < D; ++j) v[j] = fmaf((float)((p[j >> 2] >> ((j & 3) * 2)) & 0x3), scale, bias);
            }
        }
    }
}

static inline void store_out(void* out, int64_t pos, int out_ty, float v)
{
    if (out_ty == ORC_FP32) ((float*)out)[pos] = v;
    else if (out_ty == ORC_FP16) ((uint16_t*)out)[pos] = orc_f32_to_f16(v);
    else ((uint16_t*)out)[pos] = orc_f32_to_bf16(v);
}

/*
 * int_nbit_split_embedding_codegen_lookup_function, CPU semantics.
 *
 * Geometry follows the reference: bag i = t*B + b (table-major), its rows are
 * indices[offsets[i] .. offsets[i+1]), table t starts at byte weights_offsets[t]
 * of dev_weights, the result goes to out[b, D_offsets[t] .. D_offsets[t+1])
 * (int_nbit_split_embedding_pooling_kernel.h:44-85), an empty bag leaves zeros
 * (:65-69), MEAN multiplies by 1/L (:355,307-310), output is cast with
 * round-to-nearest-even (:319-342).  Row decoding for INT8/INT4/INT2/FP16/FP32
 * is the upstream TBE format (header first, fp16 scale/bias); accumulation is
 * fp32 in bag order: acc = acc + fma(q, scale, bias); with per-sample weights
 * acc = fma(q, w*scale, acc + w*bias) for integer rows and acc = fma(w, value, acc)
 * for float rows.  Index -1 (a pruned row) contributes zero
 * but still counts in L.  Pooling NONE writes row n of the indices to
 * out[n, 0 .. D) (int_nbit_split_embedding_nobag_kernel.h:31-398).
 *
 * idx_bits: 32 or 64 (indices and offsets share it, as after
 * int_nbit_split_embedding_codegen_lookup_function.cpp:110-113).
 * Returns 0, or -(1+i) if bag i holds an index < -1.
 */
int64_t orc_tbe_lookup(
    const uint8_t* dev_weights, const int64_t* weights_offsets, const uint8_t* weights_tys,
    const int32_t* D_offsets, int64_t T, int64_t B, int64_t total_D,
    const void* indices, const void* offsets, int idx_bits,
    const float* indice_weights, int pooling_mode, int out_ty, int64_t row_alignment,
    int fp8_ebits, int fp8_ebias, void* out, int64_t out_stride, int64_t max_D)
{
    const int32_t* i32 = (const int32_t*)indices;
    const int64_t* i64 = (const int64_t*)indices;
    const int32_t* o32 = (const int32_t*)offsets;
    const int64_t* o64 = (const int64_t*)offsets;
    int64_t status = 0;

    if (pooling_mode == ORC_NONE) {
#pragma omp parallel
        {
            float* v = (float*)__builtin_alloca((size_t)(max_D > 0 ? max_D : 1) * sizeof(float));
#pragma omp for schedule(static)
            for (int64_t t = 0; t < T; ++t) {
                const int ty = weights_tys[t];
                const int64_t D = D_offsets[t + 1] - D_offsets[t];
                const int64_t rb = orc_row_bytes(ty, D, row_alignment);
                const int64_t s = (idx_bits == 32) ? o32[t * B] : o64[t * B];
                const int64_t e = (idx_bits == 32) ? o32[(t + 1) * B] : o64[(t + 1) * B];
                for (int64_t n = s; n < e; ++n) {
                    const int64_t idx = (idx_bits == 32) ? i32[n] : i64[n];
                    if (idx < 0) {
                        for (int64_t j = 0; j < D; ++j) store_out(out, n * out_stride + j, out_ty, 0.0f);
                        continue;
                    }
                    row_to_f32(dev_weights + weights_offsets[t] + idx * rb, ty, D, fp8_ebits, fp8_ebias, v);
                    for (int64_t j = 0; j < D; ++j) store_out(out, n * out_stride + j, out_ty, v[j]);
                }
            }
        }
        return 0;
    }

#pragma omp parallel
    {
        float* v = (float*)__builtin_alloca((size_t)(max_D > 0 ? max_D : 1) * 2 * sizeof(float));
        float* acc = v + (max_D > 0 ? max_D : 1);
#pragma omp for schedule(dynamic, 64)
        for (int64_t i = 0; i < T * B; ++i) {
            const int64_t t = i / B, b = i % B;
            const int ty = weights_tys[t];
            const int64_t D = D_offsets[t + 1] - D_offsets[t];
            const int64_t rb = orc_row_bytes(ty, D, row_alignment);
            const int64_t s = (idx_bits == 32) ? o32[i] : o64[i];
            const int64_t e = (idx_bits == 32) ? o32[i + 1] : o64[i + 1];
            for (int64_t j = 0; j < D; ++j) acc[j] = 0.0f;
            for (int64_t n = s; n < e; ++n) {
                const int64_t idx = (idx_bits == 32) ? i32[n] : i64[n];
                if (idx == -1) continue;
                if (idx < -1) {
#pragma omp critical
                    status = -(1 + i);
                    continue;
                }
                const uint8_t* row = dev_weights + weights_offsets[t] + idx * rb;
                if (indice_weights && (ty == ORC_INT8 || ty == ORC_INT4 || ty == ORC_INT2)) {
                    /* Weighted integer rows fold the weight into scale and bias first:
                       acc = fma(q, w*scale, acc + w*bias).  This factoring reproduces the
                       FBGEMM CPU kernels bit for bit (tests/test_oracle_pins.py). */
                    uint16_t sh, bh;
                    memcpy(&sh, row, 2);
                    memcpy(&bh, row + 2, 2);
                    const float w = indice_weights[n];
                    const float ws = w * orc_f16_to_f32(sh), wb = w * orc_f16_to_f32(bh);
                    const uint8_t* p = row + 4;
                    for (int64_t j = 0; j < D; ++j) {
                        int q;
                        if (ty == ORC_INT8) q = p[j];
                        else if (ty == ORC_INT4) q = (p[j >> 1] >> ((j & 1) * 4)) & 0xf;
                        else q = (p[j >> 2] >> ((j & 3) * 2)) & 0x3;
                        acc[j] = fmaf((float)q, ws, acc[j] + wb);
                    }
                    continue;
                }
                row_to_f32(row, ty, D, fp8_ebits, fp8_ebias, v);
                if (indice_weights) {
                    const float w = indice_weights[n];
                    for (int64_t j = 0; j < D; ++j) acc[j] = fmaf(w, v[j], acc[j]);
                } else {
                    for (int64_t j = 0; j < D; ++j) acc[j] = acc[j] + v[j];
                }
            }
            if (pooling_mode == ORC_MEAN && e > s) {
                const float inv = 1.0f / (float)(e - s);
                for (int64_t j = 0; j < D; ++j) acc[j] *= inv;
            }
            const int64_t base = b * out_stride + D_offsets[t];
            for (int64_t j = 0; j < D; ++j) store_out(out, base + j, out_ty, acc[j]);
        }
    }
    return status;
}

/*
 * permute_pooled_embs: out[:, inv_offset_dim_list[i] .. inv_offset_dim_list[i+1]) =
 * in[:, offset_dim_list[p] .. offset_dim_list[p+1]) with p = permute_list[i]
 * (permute_pooled_embs.cpp:87-98; kernel permute_pooled_embs_kernel.h:173-211).
 * Byte-typed, so any element size.  Returns 0, or -1 for a bad permute entry
 * (the reference raises at permute_pooled_embs.cpp:90-91).
 */
int orc_permute_pooled_embs(
    const void* in, int64_t B, int64_t total_D, int64_t elem_bytes,
    const int64_t* offset_dim_list, const int64_t* permute_list,
    const int64_t* inv_offset_dim_list, int64_t T, void* out)
{
    for (int64_t i = 0; i < T; ++i) {
        if (permute_list[i] < 0 || permute_list[i] >= T) return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        const uint8_t* src = (const uint8_t*)in + b * total_D * elem_bytes;
        uint8_t* dst = (uint8_t*)out + b * total_D * elem_bytes;
        for (int64_t i = 0; i < T; ++i) {
            const int64_t p = permute_list[i];
            const int64_t len = offset_dim_list[p + 1] - offset_dim_list[p];
            memcpy(dst + inv_offset_dim_list[i] * elem_bytes, src + offset_dim_list[p] * elem_bytes,
                   (size_t)(len * elem_bytes));
        }
    }
    return 0;
}

/*
 * Helper for building tables in tests: turn fused 8-bit rows ([D bytes][fp32
 * scale][fp32 bias]) into TBE INT8 rows ([fp16 scale][fp16 bias][D bytes], padded
 * to row_bytes), converting scale and bias fp32 -> fp16 with RNE.  This is the
 * two-step construction that the benchmark configurations describe ("128 int8
 * bytes plus an fp16 scale and fp16 bias, produced by
 * FloatToFused8BitRowwiseQuantized").
 */
void orc_pack_int8_rows(const uint8_t* fused, int64_t N, int64_t D, int64_t row_bytes, uint8_t* rows)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const uint8_t* f = fused + r * (D + 8);
        uint8_t* o = rows + r * row_bytes;
        float scale, bias;
        memcpy(&scale, f + D, 4);
        memcpy(&bias, f + D + 4, 4);
        uint16_t sh = orc_f32_to_f16(scale), bh = orc_f32_to_f16(bias);
        memcpy(o, &sh, 2);
        memcpy(o + 2, &bh, 2);
        memcpy(o + 4, f, (size_t)D);
        if (row_bytes > D + 4) memset(o + 4 + D, 0, (size_t)(row_bytes - D - 4));
    }
}

/* N-bit SBHalf rows ([codes][fp16 scale][fp16 bias]) -> TBE rows (header first). */
void orc_pack_nbit_rows(const uint8_t* fused, int64_t N, int64_t pbytes, int64_t row_bytes, uint8_t* rows)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const uint8_t* f = fused + r * (pbytes + 4);
        uint8_t* o = rows + r * row_bytes;
        memcpy(o, f + pbytes, 4);
        memcpy(o + 4, f, (size_t)pbytes);
        if (row_bytes > pbytes + 4) memset(o + 4 + pbytes, 0, (size_t)(row_bytes - pbytes - 4));
    }
}

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
