/*
 * atlas_b200 — C ABI of the B200 (sm_100a) NVFP4 + multi-LoRA linear path.
 *
 * Every entry point follows the reference's static-library launcher convention
 * (crates/spark-runtime/src/cutlass.rs:33-168, cuda/cutlass_nvfp4_gemm.cu:242-343):
 * plain pointers and sizes, the CUDA stream as `void*` (0 = legacy default stream),
 * return 0 on success and a negative status otherwise.  All device memory is owned by
 * the caller and must outlive the call; launchers allocate nothing, never synchronise
 * and never read device memory on the host, so they can be captured into a CUDA graph
 * like the reference's launches (crates/spark-model/src/layers/ops/lora_delta.rs:132-137).
 *
 * Status codes
 *      0            success
 *     -1            bad dimensions / unsupported shape
 *     -2            workspace too small
 *     -3            misaligned pointer or stride
 *     -4            null pointer where one is required
 *     -5            limit exceeded (max_loras, max_rank, scratch capacity)
 *     -6            adapter rejected at ingest (named reason in the caller's message buffer)
 *     -7            registry slot busy (sequences in flight)
 *     -10 - e       CUDA runtime error e at launch
 *     -120          library was not built for this GPU architecture
 */
#ifndef ATLAS_B200_H
#define ATLAS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ATLAS_B200_API __attribute__((visibility("default")))
#else
#define ATLAS_B200_API
#endif

#define ATLAS_B200_OK             0
#define ATLAS_B200_ERR_DIMS      (-1)
#define ATLAS_B200_ERR_WORKSPACE (-2)
#define ATLAS_B200_ERR_ALIGN     (-3)
#define ATLAS_B200_ERR_NULL      (-4)
#define ATLAS_B200_ERR_LIMIT     (-5)
#define ATLAS_B200_ERR_REJECT    (-6)   /* adapter ingest: the adapter cannot be applied faithfully; the reason is in the message buffer */
#define ATLAS_B200_ERR_BUSY      (-7)   /* registry: the slot has sequences in flight */
#define ATLAS_B200_ERR_CUDA_BASE (-10)
#define ATLAS_B200_ERR_ARCH      (-120)

/* which kernel family a call dispatched to (launcher audit; see atlas_b200_last_variant) */
#define ATLAS_B200_VARIANT_NONE     0
#define ATLAS_B200_VARIANT_SIMT     1   /* CUDA-core tiles, any shape */
#define ATLAS_B200_VARIANT_TCGEN05  2   /* TMA + tcgen05.mma + TMEM, LoRA expand in the accumulator */

/* flags of atlas_b200_linear_desc.flags */
#define ATLAS_B200_FLAG_FORCE_SIMT     1u   /* always take the CUDA-core path */
#define ATLAS_B200_FLAG_FORCE_TCGEN05  2u   /* fail with -1 instead of falling back */
#define ATLAS_B200_FLAG_STAGED_LORA    4u   /* reference rounding: base->bf16, then shrink/expand/fold in place */
#define ATLAS_B200_FLAG_REUSE_SHRINK   8u   /* tcgen05 path only: lora_t already holds this call's shrink result (same x,
                                               seq_slot, tables and scale2 as the call that wrote it); skip the shrink launch */
#define ATLAS_B200_FLAG_ACT_FP4       16u   /* W4A4: the base product sees x quantised to NVFP4 (group of 16, E4M3 scale =
                                               group max / 6, tensor scale 1) and runs as a block-scaled FP4 x FP4 MMA; the
                                               LoRA term still sees exact x.  The opt-in W4A4 arm of the reference:
                                               crates/spark-model/src/layers/ops/gemm_fp4.rs:20-107 with the activation
                                               quantiser kernels/gb10/common/quantize_bf16_to_nvfp4.cu:176-243.  Needs the
                                               tcgen05 path (-1 where that path does not take the shape; nothing else is
                                               substituted) and `ws` of ATLAS_B200_ACT_FP4_WS_BYTES(m, k) bytes, 256-byte
                                               aligned (-2 / -3 / -4 otherwise).  Weight scale bytes must not carry a sign bit. */
/* Optional scratch that speeds up the LoRA part of the tcgen05 path: with at least this many bytes of `ws`
 * (after the ATLAS_B200_ACT_FP4_WS_BYTES region, rounded up to 256, when that flag is set), 256-byte aligned, and a
 * strided pool declared (b_pool_base / b_slot_stride), the shrink writes the LoRA K-steps' activation tiles there
 * once per call and `lora_t` is left untouched; with less, every CTA builds them from `lora_t`.  Same results. */
#define ATLAS_B200_LORA_WS_BYTES(m, max_loras, max_rank) \
    (((((size_t)(m) + 255) / 256) * 256 + 256) * ((max_loras) < 256 ? (max_loras) : 256) * (((size_t)(max_rank) + 15) / 16) * 32)
#define ATLAS_B200_FLAG_NO_CTA_PAIR   32u   /* tcgen05 path: keep every CTA on its own (no two-CTA MMAs); for comparison runs */
#define ATLAS_B200_FLAG_NO_K_SPLIT    64u   /* tcgen05 path: one CTA per output tile even when that leaves SMs idle; for comparison runs */
#define ATLAS_B200_FLAG_NO_PERSISTENT 128u   /* tcgen05 path: one output tile per CTA even for many-tile shapes; for comparison runs */
#define ATLAS_B200_FLAG_ONE_TILE_PASS 256u   /* tcgen05 path, persistent form, BF16 activations: one 256-token tile per pass instead of two
                                                192-token tiles that share each expanded weight stage (the default from 768 tokens);
                                                for comparison runs */
#define ATLAS_B200_FLAG_ACT_FP4_READY 512u    /* with ATLAS_B200_FLAG_ACT_FP4: `ws` already holds the quantised activations of this call (written by
                                                atlas_b200_silu_mul_quant_nvfp4, or by an earlier call over the same x); the quantiser is skipped */
#define ATLAS_B200_ACT_FP4_WS_BYTES(m, k) \
    ((((size_t)(m) * ((k) / 2) + 255) / 256) * 256 + (size_t)(m) * ((k) / 16))

/* ---------------------------------------------------------------------------------------
 * Routed multi-adapter LoRA delta over n rows:  out[i,:] += scale_s * (x[i,:] A_s^T) B_s^T,
 * s = seq_slot[i]; rows with s < 0, or whose slot has a null A/B table entry, are untouched.
 * Replaces `apply_lora_bgmv` (crates/spark-model/src/layers/ops/lora_delta.rs:269-314) and
 * its two kernels (kernels/gb10/common/lora_bgmv.cu:50-126, :139-225); argument meaning and
 * order follow them, strides are in elements.  Rounding boundaries are the reference's:
 * lora_xa is BF16, the expand result is rounded to BF16 before the scaled fold.
 *   x [n, x_row_stride] bf16   seq_slot [n] i32   a_table/b_table [max_loras] u64 device addresses
 *   scale_table [max_loras] f32   base_out [n, out_row_stride] bf16 (in place)
 *   lora_xa [n, max_rank] bf16 scratch
 * `max_loras` is the length of the three tables; a slot index >= max_loras is treated as
 * "no adapter" and recorded in the device status word. */
ATLAS_B200_API int atlas_b200_lora_bgmv(const void* x, const int32_t* seq_slot,
                         const uint64_t* a_table, const uint64_t* b_table, const float* scale_table,
                         void* base_out, void* lora_xa,
                         uint32_t n, uint32_t k_in, uint32_t n_out, uint32_t max_rank,
                         uint32_t x_row_stride, uint32_t out_row_stride, uint32_t max_loras,
                         void* stream);

/* Single adapter on m contiguous rows: base_out += scale * (x a^T) b^T.
 * Replaces `apply_lora_delta` (crates/spark-model/src/layers/ops/lora_delta.rs:145-235).
 *   a [max_rank, k_in] bf16, b [n_out, max_rank] bf16 (pool layout, zero padded)
 *   lora_xa [m, max_rank] bf16 scratch; lora_delta [m, n_out] bf16 scratch (may be null: the
 *   fold is fused, the buffer is only written when given). */
ATLAS_B200_API int atlas_b200_lora_delta(const void* x, const void* a, const void* b, float scale,
                          void* base_out, void* lora_xa, void* lora_delta,
                          uint32_t m, uint32_t k_in, uint32_t n_out, uint32_t max_rank,
                          void* stream);

/* Base NVFP4 linear  C[M,N] = A[M,K] * dequant(B)^T * scale2  (BF16 in/out, FP32 accumulate).
 * Replaces `w4a16_gemm` / `w4a16_gemv` launchers
 * (crates/spark-model/src/layers/ops/gemm_dense.rs:258-281, quant_dispatch.rs:94-115; kernels
 * kernels/gb10/common/w4a16_gemm.cu:87-180, w4a16_gemv.cu:62-161).
 *   b_packed [N, K/2] u8, low nibble = even k;  b_scale [N, K/16] E4M3;  scale2 by value.
 * `ws` is unused by the current kernels and may be null. */
ATLAS_B200_API int atlas_b200_w4a16_gemm(const void* a_bf16, const void* b_packed, const void* b_scale,
                          float scale2, void* c_bf16, uint32_t m, uint32_t n, uint32_t k,
                          void* ws, size_t ws_bytes, void* stream);

/* Standalone NVFP4 -> BF16 decode, out[n,k] = bf16(E2M1[nib] * (e4m3(scale) * combined_global)).
 * Replaces `dequant_nvfp4_to_bf16` (kernels/gb10/common/dequant_nvfp4_bf16.cu:50-73). */
ATLAS_B200_API int atlas_b200_dequant_nvfp4_to_bf16(const void* packed, const void* scales, void* out_bf16,
                                     float combined_global, uint32_t n, uint32_t k, void* stream);

/* BF16 -> NVFP4 quantiser (per-16 E4M3 scales, E2M1 codes) with a caller-given scale2.
 * Replaces `quantize_bf16_to_nvfp4` (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:176-243). */
ATLAS_B200_API int atlas_b200_quantize_bf16_to_nvfp4(const void* in_bf16, void* packed, void* scales,
                                      float scale2, uint32_t n, uint32_t k, void* stream);

/* The K/V consumer of a fused QKV projection, one launch: for every token with slot_mapping[token] >= 0,
 *   K heads:  k = bf16( rope( x * rsqrt(mean(x^2) + rms_eps) * (1 + w) ) )  into k_cache at the token's paged slot,
 *   V heads:  copied into v_cache at the same slot (v_in NULL: K side only).
 * Replaces `fused_k_norm_rope_cache_write_bf16` (kernels/gb10/common/fused_k_norm_rope_cache.cu:60-141; same FP32
 * arithmetic and summation order, one rounding to BF16, same bits) and the V-side cache write that accompanies it.  Unlike
 * the reference, k_in / v_in need not be contiguous copies: they point at the first K / V column of token 0 inside the fused
 * QKV output and in_row_stride (elements) is that buffer's row stride.
 *   k_norm_weight [head_dim] bf16 ("(1 + w)" convention);  positions [tokens] u32;  slot_mapping [tokens] i64;
 *   k_cache / v_cache [blocks, block_size, kv_heads, head_dim] bf16;  rotary pairs (d, d + rotary_dim/2), frequency
 *   theta^(-2 pair / rotary_dim) evaluated in FP64 as the reference does.
 * head_dim a multiple of 32 up to 256, rotary_dim a multiple of 64 (0: no rotation), else -1. */
ATLAS_B200_API int atlas_b200_kv_norm_rope_cache_write(const void* k_in, const void* v_in, uint32_t in_row_stride, const void* k_norm_weight,
                                        const uint32_t* positions, const long long* slot_mapping, void* k_cache, void* v_cache,
                                        uint32_t tokens, uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size,
                                        float rms_eps, float theta, void* stream);

/* The same with three position streams (MRoPE): rotary pair p is rotated by the temporal, height or width position for
 * p mod 3 = 0, 1, 2.  Replaces `fused_k_norm_rope_mrope_cache_write_bf16` (fused_k_norm_rope_cache.cu:149-243); with
 * pos_h == pos_w == pos_t the result equals atlas_b200_kv_norm_rope_cache_write's. */
ATLAS_B200_API int atlas_b200_kv_norm_mrope_cache_write(const void* k_in, const void* v_in, uint32_t in_row_stride, const void* k_norm_weight,
                                         const uint32_t* pos_t, const uint32_t* pos_h, const uint32_t* pos_w, const long long* slot_mapping,
                                         void* k_cache, void* v_cache, uint32_t tokens, uint32_t kv_heads, uint32_t head_dim,
                                         uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta, void* stream);

/* The K side into an FP8 (E4M3) paged cache, one byte per element: the same chain, then value * inv_scale cast with
 * saturation.  Replaces `fused_k_norm_rope_cache_write_fp8` (fused_k_norm_rope_cache.cu:253-338). */
ATLAS_B200_API int atlas_b200_k_norm_rope_cache_write_fp8(const void* k_in, uint32_t in_row_stride, const void* k_norm_weight, const uint32_t* positions,
                                           const long long* slot_mapping, void* k_cache_fp8, uint32_t tokens, uint32_t kv_heads,
                                           uint32_t head_dim, uint32_t rotary_dim, uint32_t block_size, float rms_eps, float theta,
                                           float inv_scale, void* stream);

/* The decode-path consumer of the fused QKV projection, Q side included, one launch: per token and head
 *   Q heads:  q = rope( bf16( rmsnorm(q) ) ) in place;   K heads: the same chain into k_cache at the token's paged slot;
 *   V heads:  copied into v_cache.  Tokens with slot_mapping < 0 get their Q processed and write no cache.
 * Replaces `fused_qkv_norm_rope_cache_write_bf16` (kernels/gb10/common/fused_verify_elemwise.cu:78-224) with its rounding
 * points (the normed head is rounded to BF16 before the rotation), its rotary form (angle = position * inv_freq[pair] from a
 * table of rotary_dim / 2 floats, cosine and sine multiplied by attention_factor, pairs (t, t + rotary_dim / 2)), its weight
 * convention (norm_offset_one: 1 -> x * rms * (1 + w), 0 -> x * rms * w) and its summation order: same bits.  Unlike the
 * reference, q / k_in / v_in point into the fused QKV output where the projection wrote it: first column of token 0 of each
 * part, with row strides in elements (q_row_stride for q, kv_row_stride for k_in and v_in).
 * head_dim and rotary_dim even, head_dim <= 256 (-1 otherwise); q, k_in and both strides 4-byte aligned (-3). */
ATLAS_B200_API int atlas_b200_qkv_norm_rope_cache_write(void* q, const void* k_in, const void* v_in, uint32_t q_row_stride, uint32_t kv_row_stride,
                                         const void* q_norm_weight, const void* k_norm_weight, const uint32_t* positions,
                                         const float* inv_freq, const long long* slot_mapping, void* k_cache, void* v_cache,
                                         uint32_t tokens, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t rotary_dim,
                                         uint32_t block_size, float rms_eps, float attention_factor, int norm_offset_one, void* stream);

/* First phase of the weight quantiser: *global_max (a device float the caller has zeroed) becomes max |in| over `total`
 * BF16 elements.  Replaces `nvfp4_global_absmax` (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:131-167). */
ATLAS_B200_API int atlas_b200_nvfp4_global_absmax(const void* in_bf16, float* global_max_dev, size_t total, void* stream);
/* scale2 the quantiser uses for a tensor with that maximum: max / (6 * 448) (quantize_bf16_to_nvfp4.cu:174-175). */
ATLAS_B200_API float atlas_b200_nvfp4_scale2_from_absmax(float global_max);
/* The two checkpoint conventions for the per-tensor scale folded into the one multiplier the kernels take (`scale2` /
 * `combined_global`): ModelOpt stores a direct multiplier (weight_scale_2), compressed-tensors a reciprocal
 * (weight_global_scale), 0 mapping to 0 (crates/spark-model/src/weight_map/fp8_lut.rs:46-57). */
ATLAS_B200_API float atlas_b200_nvfp4_combined_global_scale(float stored_scale, int is_reciprocal);

/* SwiGLU between the gate / up and the down projection: out = SiLU(min(g, L)) * clamp(u, -L, L) with g = gate * gate_scale,
 * u = up * up_scale, L = swiglu_limit (0: no clamp); BF16 in, FP32 math with the fast exponential, BF16 out.  Replaces
 * `moe_silu_mul` / `silu_mul_noclamp` (kernels/gb10/common/moe_silu_mul.cu:14-54).  gate, up [m, in_row_stride], out
 * [m, out_row_stride]; k a multiple of 8, strides multiples of 8 elements, pointers 16-byte aligned. */
ATLAS_B200_API int atlas_b200_silu_mul(const void* gate_bf16, const void* up_bf16, void* out_bf16, float gate_scale, float up_scale,
                        float swiglu_limit, uint32_t m, uint32_t k, uint32_t in_row_stride, uint32_t out_row_stride, void* stream);
/* The same product quantised straight to NVFP4 for the down projection's FP4-activation mode, so that the BF16
 * intermediate never reaches memory: the fusion of `nvfp4_silu_mul_quant` (crates/spark-model/src/layers/ops/
 * nvfp4_mmq.rs:126-157), with this library's activation quantiser (group of 16, E4M3(group max / 6), tensor scale 1).
 * `ws` receives what an ATLAS_B200_FLAG_ACT_FP4 call writes there: packed codes [m, k/2], then — 256-byte aligned —
 * scale bytes [m, k/16]; ws_bytes >= ATLAS_B200_ACT_FP4_WS_BYTES(m, k).  The down projection then runs with
 * ATLAS_B200_FLAG_ACT_FP4 | ATLAS_B200_FLAG_ACT_FP4_READY on that `ws` (its x is only read by the LoRA shrink).
 * k a multiple of 16. */
ATLAS_B200_API int atlas_b200_silu_mul_quant_nvfp4(const void* gate_bf16, const void* up_bf16, void* ws, size_t ws_bytes, float gate_scale,
                                    float up_scale, float swiglu_limit, uint32_t m, uint32_t k, uint32_t in_row_stride, void* stream);

/* ---------------------------------------------------------------------------------------
 * The fused layer:  y = dequant_NVFP4(W) x + scale_s B_s (A_s x),  y written once.
 * New relative to the reference, which issues the base GEMM
 * (crates/spark-model/src/layers/ops/gemm_dense.rs:258-453) and then apply_lora_bgmv
 * (lora_delta.rs:269-314) as separate launches over the same tensors; the descriptor
 * carries exactly their arguments.
 */
typedef struct atlas_b200_linear_desc {
    /* activations */
    const void*     x;              /* [m, x_row_stride] bf16 */
    uint32_t        m, k, x_row_stride;
    /* base weight: NVFP4 (w_packed, w_scale, scale2) or, when w_bf16 != NULL, dense bf16 [n, k] */
    uint32_t        n;
    const void*     w_packed;       /* [n, k/2] u8 */
    const void*     w_scale;        /* [n, k/16] e4m3 */
    const void*     w_bf16;         /* [n, k] bf16 or NULL */
    float           scale2;
    uint32_t        flags;
    /* routing (seq_slot == NULL: base linear only) */
    const int32_t*  seq_slot;       /* [m] i32, < 0 = no adapter */
    const uint64_t* a_table;        /* [max_loras] device addresses of A_s [max_rank, k] bf16, 0 = none */
    const uint64_t* b_table;        /* [max_loras] device addresses of B_s [n, max_rank] bf16, 0 = none */
    const float*    scale_table;    /* [max_loras] */
    const uint32_t* rank_table;     /* [max_loras] true ranks, or NULL (= max_rank everywhere) */
    uint32_t        max_loras, max_rank;
    /* output */
    void*           y;              /* [m, out_row_stride] bf16 */
    uint32_t        out_row_stride;
    uint32_t        reserved0;
    /* scratch: shrink result, [m, max_rank] bf16 */
    void*           lora_t;
    void*           ws;             /* scratch of ATLAS_B200_FLAG_ACT_FP4 calls; otherwise unused, may be NULL */
    size_t          ws_bytes;
    /* Optional: the B side of the adapter pool as a strided array.  When b_table[s] ==
     * b_pool_base + s * b_slot_stride for every resident slot s — which is how the reference lays its
     * pool out (slot k at k * pool_slot_bytes, crates/spark-model/src/lora/slot_math.rs:124-137) — pass the
     * base and the stride (bytes, a multiple of 16) and the tcgen05 path fetches B_s tiles by TMA.
     * NULL / 0: B_s is read through b_table with ordinary loads (any placement, slower). */
    const void*     b_pool_base;
    size_t          b_slot_stride;
    /* Optional: tensor-parallel output placement (n_dest == 0: the tile goes to `y` and nothing else).
     * With n_dest = tp >= 1 this call is rank `r`'s column shard (n = N / tp) and stores its [m, n] result
     * directly into columns [y_col_offset, y_col_offset + n) of every rank's gathered row-major buffer:
     * y_dest[i] is rank i's [m, out_row_stride] buffer as mapped into THIS process (CUDA IPC / symmetric
     * memory for i != r), out_row_stride >= N.  The stores replace the all-gather that follows a
     * column-parallel linear (crates/spark-comm/src/nccl_backend/comm_impl.rs:130-145); the caller still
     * synchronises the ranks before reading.  `y` is ignored.  Needs the tcgen05 path and 16-byte aligned
     * rows (buffers 16-byte aligned, out_row_stride and y_col_offset multiples of 8), else -1 / -3. */
    uint32_t        n_dest;
    uint32_t        y_col_offset;
    void*           y_dest[8];
    /* Optional: the A side of the adapter pool as a strided array, the counterpart of b_pool_base / b_slot_stride:
     * a_table[s] == a_pool_base + s * a_slot_stride for every resident slot s (in the reference's pool both strides are
     * pool_slot_bytes).  With it, and max_rank a multiple of 16, the shrink of a prefill batch (m >= 1024) runs on the
     * tcgen05 tensor cores with A_s tiles fetched by TMA.  NULL / 0: A_s is read through a_table (any placement). */
    const void*     a_pool_base;
    size_t          a_slot_stride;
} atlas_b200_linear_desc;

ATLAS_B200_API int atlas_b200_nvfp4_lora_linear(const atlas_b200_linear_desc* desc, void* stream);

/* The shrink of a fused call alone, sharded by tokens over a tensor-parallel group (no counterpart in the reference,
 * which recomputes nothing across ranks because it runs LoRA on one GPU only: crates/spark-server/src/main_modules/
 * serve.rs:364-369).  Column-parallel ranks all need t = A_s x for every token, but x and A_s are replicated, so each
 * rank would otherwise stream the whole of x through the same shrink.  Instead rank r calls this for its rows
 * [row_begin, row_begin + row_count) (row_begin a multiple of 64; row_count 0 = to the end) and the kernel stores the
 * LoRA activation tiles of those rows into ws_dest[0 .. n_dest): the `ws` scratch of every rank's descriptor (its own
 * included), as mapped into this process — plain stores, over NVLink for the peers.  After the ranks have synchronised,
 * every rank runs atlas_b200_nvfp4_lora_linear with ATLAS_B200_FLAG_REUSE_SHRINK on the same descriptor.
 * `desc` must be the descriptor of that later call (same shapes, flags and `ws` layout on every rank; desc->ws is used
 * only to derive where the tiles live inside a scratch buffer).  Needs what the tcgen05 shrink needs: m >= 1024, the
 * strided A and B pools, max_rank a multiple of 16, `ws` of ATLAS_B200_LORA_WS_BYTES; -1 otherwise (the caller then
 * lets every rank run the whole shrink inside the fused call). */
ATLAS_B200_API int atlas_b200_lora_shrink_tiles(const atlas_b200_linear_desc* desc, uint32_t row_begin, uint32_t row_count,
                                 void* const* ws_dest, uint32_t n_dest, void* stream);

/* The fused layer for a caller that must not allocate device memory (no counterpart in the
 * reference, whose callers size their scratch from a buffer arena).  Identical to
 * atlas_b200_nvfp4_lora_linear except that `desc->lora_t` is ignored: the shrink scratch is a fixed
 * array of ATLAS_B200_STATIC_SCRATCH_ELEMS BF16 values (1 MiB) that the library keeps on every GPU
 * it is loaded on until the process exits.  Meant for plug-ins whose host engine owns all device
 * memory, and for call sites where entering the CUDA allocator is forbidden.
 *   - m * max_rank must not exceed ATLAS_B200_STATIC_SCRATCH_ELEMS, else -5 and nothing is launched.
 *   - The first call on each device looks the array's device address up (with that device current);
 *     make that first call outside any stream capture.  Later calls only launch kernels.
 *   - The call itself never calls cudaMalloc / cudaFree or any allocating routine.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  The
 *     kernels overwrite every element they later read, so nothing is cleared between calls; but two
 *     calls whose kernels overlap on the GPU (different streams, or concurrent graph branches) race
 *     on it.  Serialise such calls, or use atlas_b200_nvfp4_lora_linear with a scratch per stream.
 *   - ATLAS_B200_FLAG_REUSE_SHRINK through this entry point reuses whatever the array holds: it is only meaningful when
 *     no other call (of any descriptor, on any stream of the device) has gone through this entry point since the call
 *     whose shrink result is to be reused. */
/* Tensor-parallel exchange as a copy that runs BESIDE the next projection's kernels: the [m, n_cols] BF16 block at `src`
 * (row stride src_row_stride elements; this rank's columns of its own gathered buffer) is stored into the same block of
 * each of the n_dest <= 8 buffers `dest[i]` (row stride dst_row_stride; the peers' gathered buffers as mapped into this
 * process, each already offset to the block's first column).  One small kernel (128 threads per CTA, no shared memory):
 * launched on a second stream after the projection that produced the block, its CTAs share the SMs with the following
 * projection's kernels and its NVLink stores overlap their arithmetic.  Use it where a rank's share of a projection is a
 * single wave of tiles, so that stores issued by the tiles themselves (n_dest > 1 in the descriptor) would all fall at
 * the end of that wave.  Replaces the all-gather after a column-parallel linear
 * (crates/spark-comm/src/nccl_backend/comm_impl.rs:130-145); the caller still synchronises the ranks before reading.
 * n_cols and both strides multiples of 8, all addresses 16-byte aligned (-3 otherwise). */
ATLAS_B200_API int atlas_b200_push_columns(const void* src, uint32_t src_row_stride, void* const* dest, uint32_t n_dest,
                            uint32_t dst_row_stride, uint32_t m, uint32_t n_cols, void* stream);

/* The same exchange carried by the copy engines instead of a kernel: one strided device-to-device copy
 * (cudaMemcpy2DAsync) per destination, no SM involved.  Same arguments as atlas_b200_push_columns, without its alignment
 * rules. */
ATLAS_B200_API int atlas_b200_copy_columns(const void* src, uint32_t src_row_stride, void* const* dest, uint32_t n_dest,
                            uint32_t dst_row_stride, uint32_t m, uint32_t n_cols, void* stream);

#define ATLAS_B200_STATIC_SCRATCH_ELEMS (512u * 1024u)
ATLAS_B200_API int atlas_b200_nvfp4_lora_linear_noalloc(const atlas_b200_linear_desc* desc, void* stream);

/* ---------------------------------------------------------------------------------------
 * Column-parallel sharding (split of N over `tp` ranks), as `shard_quantized_nvfp4`
 * ColumnParallel (crates/spark-model/src/tp_shard/quant_shard.rs:57-90): rank r owns output
 * rows [r*n/tp, (r+1)*n/tp) of W, of its scales, and of every B_s; scale2, A_s, x are
 * replicated.  Returns the row range; -1 when n is not divisible as required. */
ATLAS_B200_API int atlas_b200_column_shard(uint32_t n, uint32_t tp, uint32_t rank, uint32_t* row_begin, uint32_t* row_count);

/* ---------------------------------------------------------------------------------------
 * LoRA registry: slot math and pool layout (host only, no GPU).
 */
typedef struct atlas_b200_model_dims {
    uint32_t hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, head_dim;
    uint32_t attn_gated;                 /* q_proj output is [Q|gate] when set */
    uint32_t num_full_attention_layers;  /* layers that carry LoRA modules */
} atlas_b200_model_dims;

enum { ATLAS_B200_Q = 0, ATLAS_B200_K, ATLAS_B200_V, ATLAS_B200_O, ATLAS_B200_GATE, ATLAS_B200_UP, ATLAS_B200_DOWN,
       ATLAS_B200_NUM_MODULES };

/* `build_seq_slot_host` (crates/spark-model/src/lora/slot_math.rs:50-62) */
ATLAS_B200_API int atlas_b200_build_seq_slot(const int32_t* adapter_slots, size_t n, size_t padded_n, int32_t active, int32_t* out);
/* `routed_prefill_slot_of` (slot_math.rs:83-90); returns the slot or -1 for None */
ATLAS_B200_API int32_t atlas_b200_routed_prefill_slot_of(int32_t adapter_slot, size_t active, size_t num_slots);
/* `PeftAdapterConfig::scaling` (crates/atlas-core/src/config/parsers/lora.rs:70-77) */
ATLAS_B200_API float atlas_b200_peft_scaling(double lora_alpha, size_t r, int use_rslora);
/* `LoraModule::dims` (crates/spark-model/src/lora/types.rs:62-74) */
ATLAS_B200_API int atlas_b200_module_dims(const atlas_b200_model_dims* cfg, int module, size_t* out_dim, size_t* in_dim);
/* `pool_slot_bytes`, `slot_base_offset`, `module_slot_offsets` (slot_math.rs:109-162) */
ATLAS_B200_API size_t atlas_b200_pool_slot_bytes(const atlas_b200_model_dims* cfg, size_t max_rank);
ATLAS_B200_API size_t atlas_b200_slot_base_offset(size_t slot, const atlas_b200_model_dims* cfg, size_t max_rank);
ATLAS_B200_API int atlas_b200_module_slot_offsets(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal,
                                   int module, size_t* a_off, size_t* b_off);
/* One module of `pack_slot` (crates/spark-model/src/lora/loading.rs:160-186) into a host image of
 * the slot: A [r, in] copied to the head of its [max_rank, in] region, B [out, r] row-repacked
 * to stride max_rank; pads zeroed. `slot_image` is the slot's byte image (pool_slot_bytes long). */
ATLAS_B200_API int atlas_b200_pack_module(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal, int module,
                           const void* a_bf16, const void* b_bf16, size_t r, void* slot_image);
/* The per-(layer, module) pointer tables of `load_lora_adapters_multi`'s post-pass
 * (crates/spark-model/src/lora/loading.rs:310-369; one cell of them is what `refresh_slot_tables`,
 * lora/types.rs:338-373, rewrites after a swap).  For module `module` of adapted layer `layer_ordinal`:
 * a_table[s] / b_table[s], s < max_loras, receive the device addresses of slot s's padded A [max_rank, in]
 * and B [out, max_rank] inside a pool whose slot 0 starts at device address `pool_base` — or 0 where
 * present[s] == 0 (slot not packed, or its adapter omits the module).  `present` may be NULL (= every slot).
 * Host arrays in, host arrays out (little-endian u64, the image the reference uploads); no GPU involved.
 * b_table[s] == b_table[0] + s * atlas_b200_pool_slot_bytes(...) for every present slot, so
 * atlas_b200_linear_desc::b_pool_base / b_slot_stride can describe the B side. */
ATLAS_B200_API int atlas_b200_build_route_tables(const atlas_b200_model_dims* cfg, size_t max_rank, size_t layer_ordinal, int module,
                                  uint64_t pool_base, size_t max_loras, const uint8_t* present,
                                  uint64_t* a_table, uint64_t* b_table);
/* `select_victim_slot` (slot_math.rs:25-38): free-first, else least-recently-used idle slot,
 * else -1 (pool full).  Arrays describe the cache region only. */
ATLAS_B200_API int atlas_b200_select_victim_slot(const size_t* slot_index, const uint8_t* filled, const size_t* ref_count,
                                  const uint64_t* last_used, size_t count);


/* ---------------------------------------------------------------------------------------
 * Adapter ingest and the adapter registry (host only, no GPU): PEFT config rules, safetensors -> BF16,
 * key classification, audit, slot packing, routing tables and slot lifecycle.
 */
#define ATLAS_B200_PEFT_MAX_TARGETS 16
#define ATLAS_B200_PEFT_MAX_LAYERS  256
/* Parsed subset of a PEFT adapter_config.json (crates/atlas-core/src/config/parsers/lora.rs:44-78). */
typedef struct atlas_b200_peft_config {
    size_t   r;
    double   lora_alpha;
    int32_t  use_rslora;
    uint32_t n_target_modules;
    char     target_modules[ATLAS_B200_PEFT_MAX_TARGETS][96];   /* verbatim entries (bare names or full paths) */
    int32_t  has_layers_to_transform;
    uint32_t n_layers_to_transform;
    uint32_t layers_to_transform[ATLAS_B200_PEFT_MAX_LAYERS];
} atlas_b200_peft_config;

/* `parse_peft_adapter_config` (crates/atlas-core/src/config/parsers/lora.rs:121-262): hard-fails with the reference's
 * named REJECT(<feature>) reasons — peft_type, use_dora, bias, rank_pattern, alpha_pattern, modules_to_save, use_rslora
 * absent, layers_to_transform malformed, r == 0, lora_alpha, target_modules string / empty / non-string entries, gdn,
 * embedding, unknown_module.  0 on success; ATLAS_B200_ERR_REJECT with the message (NUL terminated, truncated to
 * err_cap) in `err`; ATLAS_B200_ERR_DIMS for a document that is not JSON or lacks r / lora_alpha / target_modules. */
ATLAS_B200_API int atlas_b200_peft_parse(const char* json, size_t len, atlas_b200_peft_config* out, char* err, size_t err_cap);
/* `PeftAdapterConfig::scaling` of a parsed config (lora.rs:70-77). */
ATLAS_B200_API float atlas_b200_peft_config_scaling(const atlas_b200_peft_config* cfg);
/* `classify_key` (crates/spark-model/src/lora/key.rs:53-113): PEFT tensor name -> (global layer index, module, 0 = lora_A /
 * 1 = lora_B).  `full_attention` [num_hidden_layers] flags the layers that carry LoRA (NULL: all of them).
 * ATLAS_B200_ERR_REJECT with the reference's REJECT[...] reason in `err` otherwise. */
ATLAS_B200_API int atlas_b200_classify_key(const char* key, uint32_t num_hidden_layers, const uint8_t* full_attention,
                            uint32_t* layer, int* module, int* ab, char* err, size_t err_cap);
/* `adapter_id_hash` (key.rs:33-47): FNV-1a of the name, the generation folded in when non-zero, never 0. */
ATLAS_B200_API uint64_t atlas_b200_adapter_id_hash(const char* name, uint64_t generation);
/* BF16 (round to nearest even, NaN quieted) of F16 / F32 / BF16 little-endian tensor bytes, the host conversion of
 * `load_adapter_safetensors` (crates/spark-runtime/src/weights/adapter.rs:62-105).  dtype: "F16", "F32" or "BF16". */
ATLAS_B200_API int atlas_b200_convert_to_bf16(const char* dtype, const void* src, size_t n_elems, void* dst_bf16);

/* The registry: `LoraWeights` (crates/spark-model/src/lora/types.rs:120-200) without the device side.  It knows the
 * pool's device base address but never touches the device: packing produces a host image of one slot that the caller
 * uploads to pool_base + slot * slot_bytes, and the table functions produce the host images of the device tables. */
typedef struct atlas_b200_registry atlas_b200_registry;
/* `full_attention` [num_hidden_layers]: layers that carry LoRA modules, ascending = the pool's layer ordinals (NULL:
 * every layer); their count must equal cfg->num_full_attention_layers. */
ATLAS_B200_API int atlas_b200_registry_create(const atlas_b200_model_dims* cfg, uint32_t num_hidden_layers, const uint8_t* full_attention,
                               size_t max_loras, size_t max_rank, uint64_t pool_device_base, atlas_b200_registry** out);
ATLAS_B200_API void atlas_b200_registry_destroy(atlas_b200_registry* reg);
ATLAS_B200_API size_t atlas_b200_registry_slot_bytes(const atlas_b200_registry* reg);
ATLAS_B200_API size_t atlas_b200_registry_pool_bytes(const atlas_b200_registry* reg);
/* Audit and pack one adapter into `slot`: `audit_adapter` + `pack_slot` (crates/spark-model/src/lora/loading.rs:48-230) at
 * load time, `pack_store_into_slot` (loading.rs:401-459) for a slot that is already filled — then the slot must be idle
 * (ATLAS_B200_ERR_BUSY, nothing changed), its generation is bumped and its table cells are refreshed.
 *   config_json / config_len     adapter_config.json
 *   safetensors / st_len         adapter_model.safetensors (F16 / F32 / BF16 tensors; anything else is rejected)
 *   slot_image                   receives the slot's byte image (atlas_b200_registry_slot_bytes long, zero padded)
 * Every rejection of the reference is reproduced by name: the config rules above, REJECT[rank-exceeds-max], the
 * classify_key reasons, duplicate-tensor, empty-adapter, unpaired-tensor, shape-mismatch, unmatched-target. */
ATLAS_B200_API int atlas_b200_registry_load_adapter(atlas_b200_registry* reg, size_t slot, const char* name,
                                     const char* config_json, size_t config_len, const void* safetensors, size_t st_len,
                                     void* slot_image, char* err, size_t err_cap);
/* Slots [0, pinned) are never eviction victims (the start-up adapter set, loading.rs:300-312). */
ATLAS_B200_API int atlas_b200_registry_set_pinned(atlas_b200_registry* reg, size_t pinned);
ATLAS_B200_API int atlas_b200_registry_set_active(atlas_b200_registry* reg, size_t slot);
/* Host images of the device tables: for (global layer, module) the [max_loras] A / B address tables (0 = base only), the
 * scale table and the true-rank table (`load_lora_adapters_multi` post-pass, loading.rs:310-369; `refresh_slot_tables`,
 * types.rs:338-373).  ATLAS_B200_ERR_DIMS for a layer that carries no LoRA. */
ATLAS_B200_API int atlas_b200_registry_route_tables(const atlas_b200_registry* reg, uint32_t layer, int module, uint64_t* a_table, uint64_t* b_table);
ATLAS_B200_API int atlas_b200_registry_scale_table(const atlas_b200_registry* reg, float* out);
ATLAS_B200_API int atlas_b200_registry_rank_table(const atlas_b200_registry* reg, uint32_t* out);
/* Slot lifecycle (types.rs:268-413): acquire resolves `slot` (>= 0: that slot, -1: the active one), takes a reference,
 * stamps the slot as most recently used and returns the resolved index (-1: out of range, nothing taken); release is
 * saturating and ignores -1; touch stamps without taking a reference. */
ATLAS_B200_API int32_t atlas_b200_registry_acquire_slot(atlas_b200_registry* reg, int32_t slot);
ATLAS_B200_API void atlas_b200_registry_release_slot(atlas_b200_registry* reg, int32_t resolved);
ATLAS_B200_API void atlas_b200_registry_touch_slot(atlas_b200_registry* reg, size_t slot);
ATLAS_B200_API size_t atlas_b200_registry_slot_ref_count(const atlas_b200_registry* reg, size_t slot);
ATLAS_B200_API uint64_t atlas_b200_registry_slot_last_used(const atlas_b200_registry* reg, size_t slot);
ATLAS_B200_API uint64_t atlas_b200_registry_slot_generation(const atlas_b200_registry* reg, size_t slot);
ATLAS_B200_API int32_t atlas_b200_registry_slot_of(const atlas_b200_registry* reg, const char* name);
ATLAS_B200_API uint64_t atlas_b200_registry_adapter_id_for_slot(const atlas_b200_registry* reg, int32_t slot);
/* `cache_slot_views` + `select_victim_slot` over the cache region [pinned, max_loras): a never-filled slot first, else
 * the least recently used idle slot, else -1 (every cache slot is busy). */
ATLAS_B200_API int32_t atlas_b200_registry_select_victim(const atlas_b200_registry* reg);

/* ---------------------------------------------------------------------------------------
 * Diagnostics.
 */
/* Device status word: 0 = clean; otherwise the first problem a kernel recorded (out-of-range
 * slot index, a bounded wait that expired).  Synchronises the device; not for use during
 * stream capture.  `clear` != 0 resets it. */
ATLAS_B200_API int atlas_b200_device_status(uint32_t* out_word, int clear);
/* Kernel family chosen by the most recent fused / base call on this thread. */
/* Self-test of the bounded wait every kernel of this library is built on (not on any data path; allocates 12 bytes and
 * synchronises): a one-CTA kernel waits, with the library's wait primitive and a limit of `limit_ns` (<= 0.1 s), on a
 * barrier that nothing arrives on.  The wait must give up, record ATLAS_B200 status 0x100 in the device status word and
 * raise the CTA's abort flag, through which a second waiter leaves; the kernel returns normally.
 * out[0], out[1] = 1 if the first / second waiter gave up, out[2] = nanoseconds the first one waited. */
ATLAS_B200_API int atlas_b200_selftest_bounded_wait(uint64_t limit_ns, uint32_t out[3]);
ATLAS_B200_API int atlas_b200_last_variant(void);
/* Launch shape of the most recent tcgen05 call on this thread (launcher audit, no counterpart in the reference):
 * out[0] = token tile, out[1] = 1 if CTAs were paired for two-CTA MMAs, out[2] = CTAs per output tile (K split),
 * out[3] = 1 if the LoRA activation tiles came from the shrink through `ws`. */
ATLAS_B200_API int atlas_b200_last_launch_shape(uint32_t out[4]);
/* The persistent form of the most recent tcgen05 call on this thread: out[0] = token tiles per pass (0: the call ran one
 * output tile per CTA), out[1] = CTA pairs in the grid. */
ATLAS_B200_API int atlas_b200_last_persistent_shape(uint32_t out[2]);
/* Per-CTA cycle counters of the tcgen05 kernel, the counterpart of the reference's per-phase timers
 * (crates/spark-model/src/layers/qwen3_attention/trait_impl/multi_seq/mod.rs:125-141).  While a device
 * buffer of `n_words` u64 is set (16 words per CTA, CTA index = blockIdx.y * gridDim.x + blockIdx.x) each
 * launch that fits writes, in SM cycles unless noted: [0] low 32 bits: MMA thread waiting for operands,
 * high 32 bits: kernel entry to first MMA wait; [1] CTA lifetime; [2] MMA role total; [3] expansion warps
 * waiting for raw weights; [4] waiting for a free stage; [5] expansion total; [6] LoRA operand build;
 * [7] epilogue; [8]/[9] %globaltimer (ns) at CTA entry / exit; [10]-[12] LoRA operand build: waiting for a free
 * stage, issuing copies, waiting for copies; [13] LoRA K blocks.  Pass NULL to switch it off (default). */
ATLAS_B200_API int atlas_b200_set_profile_buffer(void* device_buffer, size_t n_words);
ATLAS_B200_API const char* atlas_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ATLAS_B200_H */
