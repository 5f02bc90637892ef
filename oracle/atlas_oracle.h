/*
 * CPU oracle for the NVFP4 + multi-LoRA linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a scalar restatement, in plain C, of the arithmetic the reference
 * (TheApathy/apathy-atlas) performs on this path.  It is the checker the GPU
 * kernels are compared against; nothing in the shipped library links or calls it.
 * Every function names the reference file:line it follows.
 *
 * Parity pins (checked by tests/test_oracle_golden.py): the E2M1 table, the 256-entry
 * E4M3 table, BF16 round-to-nearest-even vectors, the E2M1 quantiser bins, the
 * `build_seq_slot_host` vectors, the PEFT scaling values and the pool-slot byte golden
 * that the reference's own unit tests hold.  No reference test holds a golden OUTPUT
 * tensor for the combined NVFP4-base + LoRA layer, so the combination itself is
 * "parity unpinned" beyond those parts.
 */
#ifndef ATLAS_ORACLE_H
#define ATLAS_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar codecs -------------------------------------------------------------- */
float    orc_e2m1_decode(uint32_t nibble);
float    orc_e4m3_decode(uint8_t byte);            /* NaN byte (0x7F/0xFF) -> 0 */
uint8_t  orc_e4m3_encode(float v);                 /* reference software encoder */
uint32_t orc_e2m1_quantize(float v);               /* nearest-bin, ties to smaller magnitude */
uint16_t orc_f32_to_bf16(float f);                 /* round-to-nearest-even, NaN quieted */
float    orc_bf16_to_f32(uint16_t b);

/* ---- SplitMix64, as the reference's microtests seed their inputs ----------------- */
uint64_t orc_splitmix64_next(uint64_t *state);
float    orc_rng_uniform(uint64_t *state, float lo, float hi);
float    orc_gen_val(uint64_t seed);

/* ---- NVFP4 tensors --------------------------------------------------------------- */
/* packed [N, K/2] u8 (low nibble = even k), scales [N, K/16] e4m3, out [N, K] */
void orc_dequant_nvfp4_to_bf16(const uint8_t *packed, const uint8_t *scales, uint16_t *out,
                               float combined_global, uint32_t N, uint32_t K);
void orc_dequant_nvfp4_to_f32(const uint8_t *packed, const uint8_t *scales, float *out,
                              float combined_global, uint32_t N, uint32_t K);
void orc_quantize_bf16_to_nvfp4(const uint16_t *in, uint8_t *packed, uint8_t *scales,
                                float scale2, uint32_t N, uint32_t K);
float orc_nvfp4_global_absmax(const uint16_t *in, size_t total);
/* activation quantiser of the CUTLASS path: scale = max/6 -> ue4m3, inv = 1/decoded */
void orc_act_quant_max6(const uint16_t *in, uint8_t *packed, uint8_t *scales, uint32_t M, uint32_t K);

/* ---- routing / registry math ------------------------------------------------------ */
void  orc_build_seq_slot_host(const int32_t *adapter_slots, size_t n, size_t padded_n,
                              int32_t active, int32_t *out);
int32_t orc_routed_prefill_slot_of(int32_t adapter_slot, size_t active, size_t num_slots);
float orc_peft_scaling(double lora_alpha, size_t r, int use_rslora);

typedef struct {
    uint32_t hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, head_dim;
    uint32_t attn_gated;
    uint32_t num_full_attention_layers;
} orc_model_dims;

/* module order q,k,v,o,gate,up,down */
void   orc_module_dims(const orc_model_dims *cfg, int module, size_t *out_dim, size_t *in_dim);
size_t orc_pool_slot_bytes(const orc_model_dims *cfg, size_t max_rank);
/* layer_ordinal counts full-attention layers in ascending order */
int    orc_module_slot_offsets(const orc_model_dims *cfg, size_t max_rank, size_t layer_ordinal,
                               int module, size_t *a_off, size_t *b_off);
/* A [r,in] -> head of [max_rank,in]; B [out,r] -> [out,max_rank], zero padded */
void   orc_pack_pair(const uint16_t *a, const uint16_t *b, size_t r, size_t in_dim, size_t out_dim,
                     size_t max_rank, uint16_t *a_pool, uint16_t *b_pool);

/* ---- LoRA apply with the reference's BF16 rounding boundaries -------------------- */
/* a_ptrs/b_ptrs: host pointers per slot (NULL = slot does not adapt this module) */
void orc_lora_bgmv_staged(const uint16_t *x, const int32_t *seq_slot,
                          const uint16_t *const *a_ptrs, const uint16_t *const *b_ptrs,
                          const float *scale_table, uint32_t max_loras,
                          uint16_t *base_out, uint16_t *xa,
                          uint32_t n, uint32_t k_in, uint32_t n_out, uint32_t max_rank,
                          uint32_t x_row_stride, uint32_t out_row_stride);
void orc_lora_delta_staged(const uint16_t *x, const uint16_t *a, const uint16_t *b, float scale,
                           uint16_t *base_out, uint16_t *xa, uint16_t *delta,
                           uint32_t m, uint32_t k_in, uint32_t n_out, uint32_t max_rank);

/* ---- base linear ------------------------------------------------------------------ */
/* GEMM-path semantics: every weight rounded to BF16 (with scale2 folded) before the product */
void orc_w4a16_gemm_bf16w(const uint16_t *a, const uint8_t *packed, const uint8_t *scales, float scale2,
                          uint16_t *c, uint32_t M, uint32_t N, uint32_t K);
/* dense BF16 base */
void orc_dense_gemm_bf16(const uint16_t *a, const uint16_t *w, uint16_t *c,
                         uint32_t M, uint32_t N, uint32_t K);

/* ---- the fused layer, FP32-accumulated ideal -------------------------------------- */
typedef struct {
    const uint16_t *x;            /* [M, x_row_stride] bf16 */
    uint32_t M, N, K, x_row_stride;
    /* base weight: NVFP4 (packed+scales+scale2) or dense bf16 (w_bf16) */
    const uint8_t *packed, *scales; float scale2;
    const uint16_t *w_bf16;
    /* activation mode: 0 = exact bf16 x, 1 = x quantised to NVFP4 (scale2 = 1) before the base product */
    int act_fp4;
    /* routing */
    const int32_t *seq_slot;      /* [M] or NULL */
    const uint16_t *const *a_ptrs, *const *b_ptrs;
    const float *scale_table;
    const uint32_t *rank_table;   /* optional true ranks */
    uint32_t max_loras, max_rank;
} orc_fused_args;

/* out_f32[i] for i over rows[nr] x cols[nc] (NULL rows/cols = all).  No intermediate rounding. */
void orc_fused_linear_f32(const orc_fused_args *g, const uint32_t *rows, uint32_t nr,
                          const uint32_t *cols, uint32_t nc, float *out_f32);

/* Reference launch sequence on the CPU: base (bf16-rounded weights, bf16 out) then staged bgmv. */
void orc_reference_sequence(const orc_fused_args *g, uint16_t *y, uint16_t *xa, uint32_t out_row_stride);

void orc_k_norm_rope_cache_write(const uint16_t *k_in, size_t in_row_stride, const uint16_t *k_norm_w, const uint32_t *positions,
                                 const int64_t *slot_mapping, uint16_t *k_cache, uint32_t tokens, uint32_t kv_heads,
                                 uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta);
void orc_qkv_norm_rope_cache_write(uint16_t *q, size_t q_row_stride, const uint16_t *k_in, const uint16_t *v_in, size_t kv_row_stride,
                                   const uint16_t *q_norm_w, const uint16_t *k_norm_w, const uint32_t *positions, const float *inv_freq,
                                   const int64_t *slot_mapping, uint16_t *k_cache, uint16_t *v_cache, uint32_t tokens, uint32_t q_heads,
                                   uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float eps, float factor,
                                   int offset_one);
void orc_silu_mul(const uint16_t *gate, const uint16_t *up, float *out_f32, float gate_scale, float up_scale, float limit, size_t total);
void orc_quantize_f32_to_nvfp4_scale1(const float *in, uint8_t *packed, uint8_t *scales, uint32_t M, uint32_t K);
int orc_num_threads(void);
int orc_set_num_threads(int n);   /* n <= 0: one per online core; returns the count in effect */

#ifdef __cplusplus
}
#endif
#endif
