/*
 * CPU oracle for the NVFP4 + multi-LoRA linear path.  TEST INFRASTRUCTURE ONLY — see
 * atlas_oracle.h.  Plain C; OpenMP only spreads independent output rows over host cores
 * (each output element is still one sequential scalar loop).
 *
 * Reference paths below are relative to the reference project root.
 */
#include "atlas_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------ */
/* scalar codecs                                                                        */
/* ------------------------------------------------------------------------------------ */

/* kernels/gb10/common/dequant_nvfp4_bf16.cu:26-29 (same table: w4a16_gemm.cu:31-34,
 * crates/spark-runtime/src/cutlass/tests/mod.rs:156-161). bit 3 = sign. */
static const float E2M1_LUT[16] = {
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f,
};

float orc_e2m1_decode(uint32_t nibble) { return E2M1_LUT[nibble & 0xF]; }

static float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_as_u32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* kernels/gb10/common/dequant_nvfp4_bf16.cu:34-46; the normal branch is written with the
 * bit construction of quantize_bf16_to_nvfp4.cu:213-226 (identical values). */
float orc_e4m3_decode(uint8_t b) {
    uint32_t sign = (b >> 7) & 1u, e = (b >> 3) & 0xFu, m = b & 0x7u;
    float v;
    if (e == 0u) v = (float)m * 0.001953125f;
    else if (e == 15u && m == 7u) v = 0.0f;
    else v = u32_as_f32(((e + 120u) << 23) | (m << 20));
    return sign ? -v : v;
}

/* kernels/gb10/common/quantize_bf16_to_nvfp4.cu:42-103 (software float -> E4M3: saturate at
 * 448, mantissa rounded half-up with carry, subnormals via round(|v|*512)). */
uint8_t orc_e4m3_encode(float v) {
    uint32_t bits = f32_as_u32(v);
    uint32_t sign = (bits >> 31) & 1u;
    if ((bits & 0x7FFFFFFFu) == 0u) return (uint8_t)(sign << 7);
    float absv = fabsf(v);
    if (absv > 448.0f) absv = 448.0f;
    bits = f32_as_u32(absv);
    int f32_exp = (int)((bits >> 23) & 0xFF) - 127;
    uint32_t f32_man = bits & 0x7FFFFFu;
    if (f32_exp < -9) return (uint8_t)(sign << 7);
    if (f32_exp < -6) {
        int man = (int)(absv * 512.0f + 0.5f);
        if (man > 7) man = 7;
        if (man < 0) man = 0;
        return (uint8_t)((sign << 7) | (uint32_t)man);
    }
    int e = f32_exp + 7;
    uint32_t man;
    if (e < 1) e = 1;
    if (e > 15) { e = 15; man = 6; }
    else {
        man = (f32_man + (1u << 19)) >> 20;
        if (man > 7) {
            man = 0; e++;
            if (e > 15) { e = 15; man = 6; }
        }
    }
    return (uint8_t)((sign << 7) | ((uint32_t)e << 3) | man);
}

/* Unsigned E4M3 with round-to-nearest-even and saturation to 448: the conversion the
 * CUTLASS scale-factor type performs in crates/spark-runtime/cuda/cutlass_nvfp4_gemm.cu:146
 * (third-party numeric type; restated from the OCP FP8 definition). */
static uint8_t e4m3_encode_rne(float v) {
    if (!(v > 0.0f)) return 0;
    if (v >= 448.0f) return 0x7E;
    /* candidates: nearest representable, ties to even mantissa */
    int ex; float fr = frexpf(v, &ex);      /* v = fr * 2^ex, fr in [0.5,1) */
    int e = ex - 1;                           /* v = (2fr) * 2^e, 2fr in [1,2) */
    if (e < -6) {                             /* subnormal grid 2^-9 */
        float q = v * 512.0f;
        float r = rintf(q);                   /* ties-to-even under default rounding */
        if (r >= 8.0f) return 0x08;
        return (uint8_t)r;
    }
    float q = (2.0f * fr - 1.0f) * 8.0f;      /* mantissa in [0,8) */
    float r = rintf(q);
    int m = (int)r;
    if (m == 8) { m = 0; e++; }
    if (e > 8) return 0x7E;
    if (e == 8 && m == 7) return 0x7E;
    return (uint8_t)(((e + 7) << 3) | m);
}

/* kernels/gb10/common/quantize_bf16_to_nvfp4.cu:109-124 (same bins:
 * crates/spark-runtime/src/cutlass/tests/mod.rs:164-185). */
uint32_t orc_e2m1_quantize(float v) {
    float a = fabsf(v);
    uint32_t sign = (v < 0.0f) ? 8u : 0u, idx;
    if (a <= 0.25f) idx = 0; else if (a <= 0.75f) idx = 1; else if (a <= 1.25f) idx = 2;
    else if (a <= 1.75f) idx = 3; else if (a <= 2.5f) idx = 4; else if (a <= 3.5f) idx = 5;
    else if (a <= 5.0f) idx = 6; else idx = 7;
    return sign | idx;
}

/* crates/spark-model/examples/lora_apply_microtest.rs:49-56 */
uint16_t orc_f32_to_bf16(float f) {
    uint32_t bits = f32_as_u32(f);
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}
float orc_bf16_to_f32(uint16_t b) { return u32_as_f32((uint32_t)b << 16); }

/* ------------------------------------------------------------------------------------ */
/* PRNG: crates/spark-model/examples/lora_apply_microtest.rs:31-44                       */
/* ------------------------------------------------------------------------------------ */
uint64_t orc_splitmix64_next(uint64_t *s) {
    *s += 0x9E3779B97F4A7C15ull;
    uint64_t z = *s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
float orc_rng_uniform(uint64_t *s, float lo, float hi) {
    float u = (float)(orc_splitmix64_next(s) >> 40) / (float)(1ull << 24);
    return lo + u * (hi - lo);
}
/* crates/spark-runtime/src/cutlass/tests/mod.rs:204-214 */
float orc_gen_val(uint64_t seed) {
    uint64_t x = seed * 0x9E3779B97F4A7C15ull + 0x123456789ABCDEF0ull;
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)(x >> 40) / (float)(1ull << 24) - 0.5f;
}

/* ------------------------------------------------------------------------------------ */
/* NVFP4 tensors                                                                        */
/* ------------------------------------------------------------------------------------ */

/* kernels/gb10/common/dequant_nvfp4_bf16.cu:50-73 */
void orc_dequant_nvfp4_to_bf16(const uint8_t *packed, const uint8_t *scales, uint16_t *out,
                               float g, uint32_t N, uint32_t K) {
#pragma omp parallel for schedule(static)
    for (long row = 0; row < (long)N; row++) {
        const uint8_t *rp = packed + (size_t)row * (K / 2);
        const uint8_t *rs = scales + (size_t)row * (K / 16);
        uint16_t *ro = out + (size_t)row * K;
        for (uint32_t col = 0; col < K; col++) {
            float s = orc_e4m3_decode(rs[col / 16]) * g;
            uint8_t byte = rp[col >> 1];
            uint32_t nib = (col & 1u) ? ((byte >> 4) & 0xFu) : (byte & 0xFu);
            ro[col] = orc_f32_to_bf16(E2M1_LUT[nib] * s);
        }
    }
}

void orc_dequant_nvfp4_to_f32(const uint8_t *packed, const uint8_t *scales, float *out,
                              float g, uint32_t N, uint32_t K) {
#pragma omp parallel for schedule(static)
    for (long row = 0; row < (long)N; row++) {
        const uint8_t *rp = packed + (size_t)row * (K / 2);
        const uint8_t *rs = scales + (size_t)row * (K / 16);
        float *ro = out + (size_t)row * K;
        for (uint32_t col = 0; col < K; col++) {
            float s = orc_e4m3_decode(rs[col / 16]) * g;
            uint8_t byte = rp[col >> 1];
            uint32_t nib = (col & 1u) ? ((byte >> 4) & 0xFu) : (byte & 0xFu);
            ro[col] = E2M1_LUT[nib] * s;
        }
    }
}

/* kernels/gb10/common/quantize_bf16_to_nvfp4.cu:131-167 */
float orc_nvfp4_global_absmax(const uint16_t *in, size_t total) {
    float m = 0.0f;
    for (size_t i = 0; i < total; i++) {
        float v = fabsf(orc_bf16_to_f32(in[i]));
        if (v > m) m = v;
    }
    return m;
}

/* kernels/gb10/common/quantize_bf16_to_nvfp4.cu:176-243 */
void orc_quantize_bf16_to_nvfp4(const uint16_t *in, uint8_t *packed, uint8_t *scales,
                                float scale2, uint32_t N, uint32_t K) {
    float inv_scale2 = (scale2 > 0.0f) ? (1.0f / scale2) : 0.0f;
    uint32_t groups = K / 16;
#pragma omp parallel for schedule(static)
    for (long row = 0; row < (long)N; row++) {
        const uint16_t *ri = in + (size_t)row * K;
        uint8_t *rp = packed + (size_t)row * (K / 2);
        uint8_t *rs = scales + (size_t)row * groups;
        for (uint32_t g = 0; g < groups; g++) {
            uint32_t base = g * 16;
            float gmax = 0.0f;
            for (int i = 0; i < 16; i++) {
                float v = fabsf(orc_bf16_to_f32(ri[base + i]));
                if (v > gmax) gmax = v;
            }
            float f8 = (gmax > 0.0f) ? (gmax * inv_scale2 / 6.0f) : 0.0f;
            uint8_t byte = orc_e4m3_encode(f8);
            rs[g] = byte;
            float eff = orc_e4m3_decode(byte) * scale2;
            float inv_eff = (eff > 0.0f) ? (1.0f / eff) : 0.0f;
            for (int i = 0; i < 16; i += 2) {
                uint32_t n0 = orc_e2m1_quantize(orc_bf16_to_f32(ri[base + i]) * inv_eff);
                uint32_t n1 = orc_e2m1_quantize(orc_bf16_to_f32(ri[base + i + 1]) * inv_eff);
                rp[g * 8 + i / 2] = (uint8_t)((n1 << 4) | (n0 & 0xF));
            }
        }
    }
}

/* crates/spark-runtime/cuda/cutlass_nvfp4_gemm.cu:125-162 (scales written row-major here;
 * the reference scatters them through the MMA scale-factor layout, which is data movement) */
void orc_act_quant_max6(const uint16_t *in, uint8_t *packed, uint8_t *scales, uint32_t M, uint32_t K) {
    uint32_t groups = K / 16;
#pragma omp parallel for schedule(static)
    for (long row = 0; row < (long)M; row++) {
        for (uint32_t g = 0; g < groups; g++) {
            const uint16_t *p = in + (size_t)row * K + g * 16;
            float mx = 0.0f;
            for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(orc_bf16_to_f32(p[i])));
            float scale = mx > 0.0f ? mx / 6.0f : 1.0f;
            uint8_t sf = e4m3_encode_rne(scale);
            scales[(size_t)row * groups + g] = sf;
            float dec = orc_e4m3_decode(sf);
            float inv = dec > 0.0f ? 1.0f / dec : 0.0f;
            for (int i = 0; i < 16; i += 2) {
                uint32_t n0 = orc_e2m1_quantize(orc_bf16_to_f32(p[i]) * inv);
                uint32_t n1 = orc_e2m1_quantize(orc_bf16_to_f32(p[i + 1]) * inv);
                packed[(size_t)row * (K / 2) + g * 8 + i / 2] = (uint8_t)(n0 | (n1 << 4));
            }
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* routing / registry math                                                              */
/* ------------------------------------------------------------------------------------ */

/* crates/spark-model/src/lora/slot_math.rs:50-62 */
void orc_build_seq_slot_host(const int32_t *slots, size_t n, size_t padded_n, int32_t active, int32_t *out) {
    for (size_t i = 0; i < padded_n; i++) {
        if (i < n) { int32_t s = slots[i]; out[i] = (s >= 0) ? s : active; }
        else out[i] = -1;
    }
}

/* crates/spark-model/src/lora/slot_math.rs:83-90; -1 encodes None */
int32_t orc_routed_prefill_slot_of(int32_t adapter_slot, size_t active, size_t num_slots) {
    size_t resolved = adapter_slot >= 0 ? (size_t)adapter_slot : active;
    return (resolved != active && resolved < num_slots) ? (int32_t)resolved : -1;
}

/* crates/atlas-core/src/config/parsers/lora.rs:70-77 */
float orc_peft_scaling(double alpha, size_t r, int use_rslora) {
    return use_rslora ? (float)(alpha / sqrt((double)r)) : (float)(alpha / (double)r);
}

/* crates/spark-model/src/lora/types.rs:62-74 */
void orc_module_dims(const orc_model_dims *c, int module, size_t *out_dim, size_t *in_dim) {
    size_t h = c->hidden_size, qd = (size_t)c->num_attention_heads * c->head_dim;
    size_t kvd = (size_t)c->num_key_value_heads * c->head_dim;
    switch (module) {
        case 0: *out_dim = (c->attn_gated ? 2 : 1) * qd; *in_dim = h; break;
        case 1: case 2: *out_dim = kvd; *in_dim = h; break;
        case 3: *out_dim = h; *in_dim = qd; break;
        case 4: case 5: *out_dim = c->intermediate_size; *in_dim = h; break;
        default: *out_dim = h; *in_dim = c->intermediate_size; break;
    }
}

/* crates/spark-model/src/lora/slot_math.rs:109-122 */
size_t orc_pool_slot_bytes(const orc_model_dims *c, size_t max_rank) {
    size_t per_layer = 0;
    for (int m = 0; m < 7; m++) {
        size_t o, i; orc_module_dims(c, m, &o, &i);
        per_layer += (max_rank * i + o * max_rank) * 2;
    }
    return per_layer * c->num_full_attention_layers;
}

/* crates/spark-model/src/lora/slot_math.rs:139-162 */
int orc_module_slot_offsets(const orc_model_dims *c, size_t max_rank, size_t layer_ordinal,
                            int module, size_t *a_off, size_t *b_off) {
    size_t off = 0;
    for (size_t l = 0; l < c->num_full_attention_layers; l++) {
        for (int m = 0; m < 7; m++) {
            size_t o, i; orc_module_dims(c, m, &o, &i);
            size_t a = off, b = off + max_rank * i * 2;
            off = b + o * max_rank * 2;
            if (l == layer_ordinal && m == module) { *a_off = a; *b_off = b; return 1; }
        }
    }
    return 0;
}

/* crates/spark-model/src/lora/loading.rs:166-186 */
void orc_pack_pair(const uint16_t *a, const uint16_t *b, size_t r, size_t in_dim, size_t out_dim,
                   size_t max_rank, uint16_t *a_pool, uint16_t *b_pool) {
    memset(a_pool, 0, max_rank * in_dim * 2);
    memcpy(a_pool, a, r * in_dim * 2);
    memset(b_pool, 0, out_dim * max_rank * 2);
    for (size_t row = 0; row < out_dim; row++) memcpy(b_pool + row * max_rank, b + row * r, r * 2);
}

/* ------------------------------------------------------------------------------------ */
/* LoRA apply with the reference's rounding boundaries                                  */
/* ------------------------------------------------------------------------------------ */

/* One routed row.  Stage roundings: xa -> BF16, delta -> BF16, then
 * out = bf16(f32(out) + scale * f32(delta_bf16))
 * (crates/spark-model/examples/lora_apply_microtest.rs:185-207 for the two products,
 *  kernels/gb10/common/lora_bgmv.cu:214-223 for the fold).  Contraction runs over
 * max_rank (pads are zero), as kernels/gb10/common/lora_bgmv.cu:27-29 requires. */
static void lora_row_staged(const uint16_t *xr, const uint16_t *A, const uint16_t *B, float scale,
                            uint16_t *out, uint16_t *xa, uint16_t *delta_or_null,
                            uint32_t k_in, uint32_t n_out, uint32_t max_rank) {
    for (uint32_t j = 0; j < max_rank; j++) {
        float acc = 0.0f;
        const uint16_t *ar = A + (size_t)j * k_in;
        for (uint32_t k = 0; k < k_in; k++) acc += orc_bf16_to_f32(xr[k]) * orc_bf16_to_f32(ar[k]);
        xa[j] = orc_f32_to_bf16(acc);
    }
    for (uint32_t o = 0; o < n_out; o++) {
        float acc = 0.0f;
        const uint16_t *br = B + (size_t)o * max_rank;
        for (uint32_t j = 0; j < max_rank; j++) acc += orc_bf16_to_f32(xa[j]) * orc_bf16_to_f32(br[j]);
        uint16_t dbf = orc_f32_to_bf16(acc);
        if (delta_or_null) delta_or_null[o] = dbf;
        out[o] = orc_f32_to_bf16(orc_bf16_to_f32(out[o]) + scale * orc_bf16_to_f32(dbf));
    }
}

/* crates/spark-model/src/layers/ops/lora_delta.rs:269-314 + kernels/gb10/common/lora_bgmv.cu:50-225.
 * Rows with seq_slot < 0, or whose slot has a NULL A or B entry, are left untouched
 * (lora_bgmv.cu:60-65,150-155); their xa row is not written. */
void orc_lora_bgmv_staged(const uint16_t *x, const int32_t *seq_slot,
                          const uint16_t *const *a_ptrs, const uint16_t *const *b_ptrs,
                          const float *scale_table, uint32_t max_loras,
                          uint16_t *base_out, uint16_t *xa,
                          uint32_t n, uint32_t k_in, uint32_t n_out, uint32_t max_rank,
                          uint32_t x_row_stride, uint32_t out_row_stride) {
#pragma omp parallel for schedule(dynamic, 1)
    for (long row = 0; row < (long)n; row++) {
        int32_t s = seq_slot[row];
        if (s < 0 || (uint32_t)s >= max_loras) continue;
        if (!a_ptrs[s] || !b_ptrs[s]) continue;
        lora_row_staged(x + (size_t)row * x_row_stride, a_ptrs[s], b_ptrs[s], scale_table[s],
                        base_out + (size_t)row * out_row_stride, xa + (size_t)row * max_rank, NULL,
                        k_in, n_out, max_rank);
    }
}

/* crates/spark-model/src/layers/ops/lora_delta.rs:145-235 */
void orc_lora_delta_staged(const uint16_t *x, const uint16_t *a, const uint16_t *b, float scale,
                           uint16_t *base_out, uint16_t *xa, uint16_t *delta,
                           uint32_t m, uint32_t k_in, uint32_t n_out, uint32_t max_rank) {
#pragma omp parallel for schedule(dynamic, 1)
    for (long row = 0; row < (long)m; row++) {
        lora_row_staged(x + (size_t)row * k_in, a, b, scale, base_out + (size_t)row * n_out,
                        xa + (size_t)row * max_rank, delta ? delta + (size_t)row * n_out : NULL,
                        k_in, n_out, max_rank);
    }
}

/* ------------------------------------------------------------------------------------ */
/* base linear                                                                          */
/* ------------------------------------------------------------------------------------ */

/* kernels/gb10/common/w4a16_gemm.cu:87-180: each weight = bf16(LUT * e4m3 * scale2) (line
 * 152-153), FP32 accumulate, BF16 out.  The E4M3 decode there is the hardware cast, which
 * differs from orc_e4m3_decode only on the NaN byte; inputs never carry it. */
void orc_w4a16_gemm_bf16w(const uint16_t *a, const uint8_t *packed, const uint8_t *scales, float scale2,
                          uint16_t *c, uint32_t M, uint32_t N, uint32_t K) {
#pragma omp parallel
    {
        float *w = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (long n = 0; n < (long)N; n++) {
            const uint8_t *rp = packed + (size_t)n * (K / 2);
            const uint8_t *rs = scales + (size_t)n * (K / 16);
            for (uint32_t k = 0; k < K; k++) {
                uint8_t byte = rp[k >> 1];
                uint32_t nib = (k & 1u) ? (byte >> 4) : (byte & 0xFu);
                float dq = E2M1_LUT[nib] * orc_e4m3_decode(rs[k / 16]) * scale2;
                w[k] = orc_bf16_to_f32(orc_f32_to_bf16(dq));
            }
            for (uint32_t m = 0; m < M; m++) {
                const uint16_t *ar = a + (size_t)m * K;
                float acc = 0.0f;
                for (uint32_t k = 0; k < K; k++) acc += orc_bf16_to_f32(ar[k]) * w[k];
                c[(size_t)m * N + n] = orc_f32_to_bf16(acc);
            }
        }
        free(w);
    }
}

/* kernels/gb10/common/dense_gemm_tc.cu:23-145 (C = A * B^T, BF16 in, FP32 acc, BF16 out) */
void orc_dense_gemm_bf16(const uint16_t *a, const uint16_t *w, uint16_t *c, uint32_t M, uint32_t N, uint32_t K) {
#pragma omp parallel for schedule(static)
    for (long n = 0; n < (long)N; n++) {
        const uint16_t *wr = w + (size_t)n * K;
        for (uint32_t m = 0; m < M; m++) {
            const uint16_t *ar = a + (size_t)m * K;
            float acc = 0.0f;
            for (uint32_t k = 0; k < K; k++) acc += orc_bf16_to_f32(ar[k]) * orc_bf16_to_f32(wr[k]);
            c[(size_t)m * N + n] = orc_f32_to_bf16(acc);
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* the fused layer: y = dequant(W) x + scale_s B_s (A_s x), FP32 accumulation, no rounding */
/* ------------------------------------------------------------------------------------ */

static void fused_row_prepare(const orc_fused_args *g, uint32_t row, float *xf, float *t, int *slot_out) {
    const uint16_t *xr = g->x + (size_t)row * g->x_row_stride;
    for (uint32_t k = 0; k < g->K; k++) xf[k] = orc_bf16_to_f32(xr[k]);
    int s = g->seq_slot ? g->seq_slot[row] : -1;
    if (s >= 0 && ((uint32_t)s >= g->max_loras || !g->a_ptrs[s] || !g->b_ptrs[s])) s = -1;
    *slot_out = s;
    if (s >= 0) {
        uint32_t r = g->rank_table ? g->rank_table[s] : g->max_rank;
        if (r > g->max_rank) r = g->max_rank;
        for (uint32_t j = 0; j < g->max_rank; j++) t[j] = 0.0f;
        for (uint32_t j = 0; j < r; j++) {
            const uint16_t *ar = g->a_ptrs[s] + (size_t)j * g->K;
            float acc = 0.0f;
            for (uint32_t k = 0; k < g->K; k++) acc += xf[k] * orc_bf16_to_f32(ar[k]);
            t[j] = acc;
        }
    }
    if (g->act_fp4) {
        /* W4A4 oracle: the base product sees dequant(quant(x)); LoRA shrink above saw exact x.
         * Quantiser = kernels/gb10/common/quantize_bf16_to_nvfp4.cu:176-243 with scale2 = 1
         * (crates/spark-model/src/layers/ops/gemm_fp4.rs:20-40). */
        uint32_t groups = g->K / 16;
        for (uint32_t gi = 0; gi < groups; gi++) {
            float gmax = 0.0f;
            for (int i = 0; i < 16; i++) { float v = fabsf(xf[gi * 16 + i]); if (v > gmax) gmax = v; }
            float f8 = gmax > 0.0f ? gmax / 6.0f : 0.0f;
            float eff = orc_e4m3_decode(orc_e4m3_encode(f8));
            float inv = eff > 0.0f ? 1.0f / eff : 0.0f;
            for (int i = 0; i < 16; i++)
                xf[gi * 16 + i] = E2M1_LUT[orc_e2m1_quantize(xf[gi * 16 + i] * inv)] * eff;
        }
    }
}

static float fused_one(const orc_fused_args *g, const float *xf, const float *t, int s, uint32_t col) {
    float acc = 0.0f;
    if (g->w_bf16) {
        const uint16_t *wr = g->w_bf16 + (size_t)col * g->K;
        for (uint32_t k = 0; k < g->K; k++) acc += xf[k] * orc_bf16_to_f32(wr[k]);
    } else {
        /* group scale factored out of its 16 products, as kernels/gb10/common/w4a16_gemv.cu:121-130 */
        const uint8_t *rp = g->packed + (size_t)col * (g->K / 2);
        const uint8_t *rs = g->scales + (size_t)col * (g->K / 16);
        for (uint32_t gi = 0; gi < g->K / 16; gi++) {
            float part = 0.0f;
            for (int i = 0; i < 16; i++) {
                uint32_t k = gi * 16 + i;
                uint8_t byte = rp[k >> 1];
                uint32_t nib = (k & 1u) ? (byte >> 4) : (byte & 0xFu);
                part += E2M1_LUT[nib] * xf[k];
            }
            acc += orc_e4m3_decode(rs[gi]) * part;
        }
        acc *= g->scale2;
    }
    if (s >= 0) {
        const uint16_t *br = g->b_ptrs[s] + (size_t)col * g->max_rank;
        float d = 0.0f;
        for (uint32_t j = 0; j < g->max_rank; j++) d += t[j] * orc_bf16_to_f32(br[j]);
        acc += g->scale_table[s] * d;
    }
    return acc;
}

void orc_fused_linear_f32(const orc_fused_args *g, const uint32_t *rows, uint32_t nr,
                          const uint32_t *cols, uint32_t nc, float *out) {
    if (!rows) nr = g->M;
    if (!cols) nc = g->N;
#pragma omp parallel
    {
        float *xf = (float *)malloc((size_t)g->K * sizeof(float));
        float *t = (float *)malloc((size_t)(g->max_rank ? g->max_rank : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (long ri = 0; ri < (long)nr; ri++) {
            uint32_t row = rows ? rows[ri] : (uint32_t)ri;
            int s;
            fused_row_prepare(g, row, xf, t, &s);
            for (uint32_t ci = 0; ci < nc; ci++) {
                uint32_t col = cols ? cols[ci] : ci;
                out[(size_t)ri * nc + ci] = fused_one(g, xf, t, s, col);
            }
        }
        free(xf); free(t);
    }
}

/* The reference's launch sequence on this path, on the CPU: base linear with BF16 output
 * (crates/spark-model/src/layers/ops/gemm_dense.rs:258-281 -> w4a16_gemm.cu, or the dense BF16
 * GEMM for an unquantised base), then apply_lora_bgmv in place
 * (crates/spark-model/src/layers/ops/lora_delta.rs:269-314). */
void orc_reference_sequence(const orc_fused_args *g, uint16_t *y, uint16_t *xa, uint32_t out_row_stride) {
    uint16_t *tmp = (uint16_t *)malloc((size_t)g->M * g->N * 2);
    /* contiguous copy of x for the base GEMM */
    uint16_t *xc = (uint16_t *)malloc((size_t)g->M * g->K * 2);
    for (uint32_t m = 0; m < g->M; m++) memcpy(xc + (size_t)m * g->K, g->x + (size_t)m * g->x_row_stride, (size_t)g->K * 2);
    if (g->w_bf16) orc_dense_gemm_bf16(xc, g->w_bf16, tmp, g->M, g->N, g->K);
    else orc_w4a16_gemm_bf16w(xc, g->packed, g->scales, g->scale2, tmp, g->M, g->N, g->K);
    for (uint32_t m = 0; m < g->M; m++) memcpy(y + (size_t)m * out_row_stride, tmp + (size_t)m * g->N, (size_t)g->N * 2);
    free(tmp); free(xc);
    if (g->seq_slot)
        orc_lora_bgmv_staged(g->x, g->seq_slot, g->a_ptrs, g->b_ptrs, g->scale_table, g->max_loras, y, xa,
                             g->M, g->K, g->N, g->max_rank, g->x_row_stride, out_row_stride);
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads the OpenMP loops use from now on (launchers such as torch.distributed.run export OMP_NUM_THREADS=1,
 * which would otherwise silently serialise the timed baseline).  n <= 0: one per online core. */
int orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n <= 0) n = omp_get_num_procs();
    omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* SwiGLU between the gate / up and the down projection, the arithmetic of kernels/gb10/common/moe_silu_mul.cu:14-54
 * (clamped at `limit` when limit > 0: gate from above only, up on both sides) with the per-projection scale folds of
 * kernels/gb10/qwen3.6-27b/nvfp4/nvfp4_mmq.cu:126-139.  FP32; the GPU's fast exponential differs from expf in the last
 * bits, which is why comparisons with this function allow one BF16 ulp. */
static float orc_swiglu(float g, float u, float limit) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return g * (1.0f / (1.0f + expf(-g))) * u;
}

void orc_silu_mul(const uint16_t *gate, const uint16_t *up, float *out_f32, float gate_scale, float up_scale, float limit, size_t total) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)total; i++)
        out_f32[i] = orc_swiglu(orc_bf16_to_f32(gate[i]) * gate_scale, orc_bf16_to_f32(up[i]) * up_scale, limit);
}

/* The activation quantiser of the FP4-activation mode applied to FP32 values (what the fused SwiGLU + quantise kernel
 * does): group of 16, scale byte = software E4M3 encode of max / 6 with tensor scale 1
 * (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:176-243 with scale2 = 1), codes by the E2M1 bins of :109-124. */
void orc_quantize_f32_to_nvfp4_scale1(const float *in, uint8_t *packed, uint8_t *scales, uint32_t M, uint32_t K) {
    uint32_t groups = K / 16;
#pragma omp parallel for schedule(static)
    for (long row = 0; row < (long)M; row++) {
        for (uint32_t g = 0; g < groups; g++) {
            const float *p = in + (size_t)row * K + g * 16;
            float mx = 0.0f;
            for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(p[i]));
            uint8_t sf = orc_e4m3_encode(mx > 0.0f ? mx / 6.0f : 0.0f);
            scales[(size_t)row * groups + g] = sf;
            float dec = orc_e4m3_decode(sf);
            float inv = dec > 0.0f ? 1.0f / dec : 0.0f;
            for (int i = 0; i < 16; i += 2) {
                uint32_t n0 = orc_e2m1_quantize(p[i] * inv);
                uint32_t n1 = orc_e2m1_quantize(p[i + 1] * inv);
                packed[(size_t)row * (K / 2) + g * 8 + i / 2] = (uint8_t)(n0 | (n1 << 4));
            }
        }
    }
}

/* The K side of the fused QKV epilogue, kernels/gb10/common/fused_k_norm_rope_cache.cu:60-141: per (token, kv head)
 * RMS norm in the "(1 + w)" convention, rotary embedding of the pairs (d, d + rotary_dim/2) with the frequency
 * theta^(-2 pair / rotary_dim) evaluated in double, and ONE rounding to BF16 into the paged cache
 * [blocks, block_size, kv_heads, head_dim] at slot_mapping[token] (negative: token skipped).  The sum of squares follows
 * the reference's order: an xor-butterfly over each group of 32 consecutive elements (:84-85), then a butterfly over the
 * group sums padded with zeros (:93-98).  Two library calls differ from the device's by design and bound the agreement
 * to the last FP32 bits (so to a rare flip of the last BF16 bit): 1/sqrtf for the device's rsqrtf, and the host's
 * sinf / cosf. */
static float orc_butterfly32(float *v) {
    for (int o = 16; o > 0; o >>= 1) {
        float n[32];
        for (int l = 0; l < 32; l++) n[l] = v[l] + v[l ^ o];
        memcpy(v, n, sizeof(n));
    }
    return v[0];
}

void orc_k_norm_rope_cache_write(const uint16_t *k_in, size_t in_row_stride, const uint16_t *k_norm_w, const uint32_t *positions,
                                 const int64_t *slot_mapping, uint16_t *k_cache, uint32_t tokens, uint32_t kv_heads,
                                 uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta) {
    for (uint32_t t = 0; t < tokens; t++) {
        int64_t slot = slot_mapping[t];
        if (slot < 0) continue;
        for (uint32_t h = 0; h < kv_heads; h++) {
            const uint16_t *row = k_in + (size_t)t * in_row_stride + (size_t)h * head_dim;
            float x[256], nrm[256], grp[32];
            uint32_t n_grp = (head_dim + 31) / 32;
            for (uint32_t g = 0; g < 32; g++) grp[g] = 0.0f;
            for (uint32_t g = 0; g < n_grp; g++) {
                float v[32];
                for (uint32_t l = 0; l < 32; l++) {
                    uint32_t d = g * 32 + l;
                    x[d < 256 ? d : 255] = d < head_dim ? orc_bf16_to_f32(row[d]) : 0.0f;
                    float e = d < head_dim ? x[d] : 0.0f;
                    v[l] = e * e;
                }
                grp[g] = orc_butterfly32(v);
            }
            float total = orc_butterfly32(grp);
            float rms = 1.0f / sqrtf(total / (float)head_dim + rms_eps);
            for (uint32_t d = 0; d < head_dim; d++) nrm[d] = x[d] * rms * (1.0f + orc_bf16_to_f32(k_norm_w[d]));
            uint32_t half = rotary_dim / 2;
            uint16_t *dst = k_cache + ((size_t)(slot / block_size) * block_size + (size_t)(slot % block_size)) * ((size_t)kv_heads * head_dim) +
                            (size_t)h * head_dim;
            for (uint32_t d = 0; d < head_dim; d++) {
                float out = nrm[d];
                if (d < rotary_dim) {
                    int low = d < half;
                    uint32_t pair = low ? d : d - half;
                    float x0 = low ? nrm[d] : nrm[d - half], x1 = low ? nrm[d + half] : nrm[d];
                    double fe = (double)(2u * pair) / (double)rotary_dim;
                    float freq = (float)(1.0 / pow((double)theta, fe));
                    float angle = (float)positions[t] * freq;
                    float c = cosf(angle), s = sinf(angle);
                    out = low ? (x0 * c - x1 * s) : (x1 * c + x0 * s);
                }
                dst[d] = orc_f32_to_bf16(out);
            }
        }
    }
}

/* The decode-path QKV consumer, kernels/gb10/common/fused_verify_elemwise.cu:78-224: per (token, head) the RMS norm with
 * weight w or (1 + w) (:170-178), the normed head rounded to BF16 (:176-177), the rotation of the pairs (t, t + rotary_dim/2)
 * by angle = position * inv_freq[t] with cosine and sine scaled by the attention factor (:186-194), Q back in place, K into
 * the paged cache, V copied (:104-121).  Sum of squares in the reference's order: thread t squares the packed pair
 * (2t, 2t + 1), butterfly per warp of 32 threads, butterfly over the warp sums (:139-163).  1/sqrtf, sinf, cosf are the
 * host's (see orc_k_norm_rope_cache_write). */
static void orc_norm_rope_head(const uint16_t *x, const uint16_t *w, uint32_t head_dim, uint32_t rotary_dim, float pos,
                               const float *inv_freq, float eps, float factor, int offset_one, uint16_t *dst) {
    float warp_sum[32];
    for (int i = 0; i < 32; i++) warp_sum[i] = 0.0f;
    uint32_t half = head_dim / 2, n_warps = (head_dim + 31) / 32;
    for (uint32_t wi = 0; wi < n_warps && wi < 32; wi++) {
        float v[32];
        for (uint32_t l = 0; l < 32; l++) {
            uint32_t t = wi * 32 + l;
            if (t < half) {
                float a = orc_bf16_to_f32(x[2 * t]), b = orc_bf16_to_f32(x[2 * t + 1]);
                float aa = a * a, bb = b * b;
                v[l] = aa + bb;
            } else v[l] = 0.0f;
        }
        warp_sum[wi] = orc_butterfly32(v);
    }
    float total = orc_butterfly32(warp_sum);
    float rms = 1.0f / sqrtf(total / (float)head_dim + eps);
    uint16_t nb[256];
    for (uint32_t d = 0; d < head_dim; d++) {
        float wf = orc_bf16_to_f32(w[d]);
        float weff = offset_one ? 1.0f + wf : wf;
        float t1 = orc_bf16_to_f32(x[d]) * rms;
        nb[d] = orc_f32_to_bf16(t1 * weff);
    }
    uint32_t pairs = rotary_dim / 2;
    for (uint32_t t = 0; t < head_dim; t++) {
        if (t < pairs) {
            float a = orc_bf16_to_f32(nb[t]), b = orc_bf16_to_f32(nb[t + pairs]);
            float angle = pos * inv_freq[t];
            float c = cosf(angle) * factor, s = sinf(angle) * factor;
            float ac = a * c, bs = b * s, bc = b * c, as = a * s;
            dst[t] = orc_f32_to_bf16(ac - bs);
            dst[t + pairs] = orc_f32_to_bf16(bc + as);
        } else if (t >= rotary_dim) dst[t] = nb[t];
    }
}

void orc_qkv_norm_rope_cache_write(uint16_t *q, size_t q_row_stride, const uint16_t *k_in, const uint16_t *v_in, size_t kv_row_stride,
                                   const uint16_t *q_norm_w, const uint16_t *k_norm_w, const uint32_t *positions, const float *inv_freq,
                                   const int64_t *slot_mapping, uint16_t *k_cache, uint16_t *v_cache, uint32_t tokens, uint32_t q_heads,
                                   uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float eps, float factor,
                                   int offset_one) {
    for (uint32_t t = 0; t < tokens; t++) {
        float pos = (float)positions[t];
        for (uint32_t h = 0; h < q_heads; h++) {
            uint16_t *row = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
            uint16_t tmp[256];
            memcpy(tmp, row, head_dim * 2);
            orc_norm_rope_head(tmp, q_norm_w, head_dim, rotary_dim, pos, inv_freq, eps, factor, offset_one, row);
        }
        int64_t slot = slot_mapping[t];
        if (slot < 0) continue;
        size_t at = ((size_t)(slot / block_size) * block_size + (size_t)(slot % block_size)) * ((size_t)kv_heads * head_dim);
        for (uint32_t h = 0; h < kv_heads; h++) {
            orc_norm_rope_head(k_in + (size_t)t * kv_row_stride + (size_t)h * head_dim, k_norm_w, head_dim, rotary_dim, pos, inv_freq, eps,
                               factor, offset_one, k_cache + at + (size_t)h * head_dim);
            memcpy(v_cache + at + (size_t)h * head_dim, v_in + (size_t)t * kv_row_stride + (size_t)h * head_dim, head_dim * 2);
        }
    }
}
