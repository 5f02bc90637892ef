// The K/V consumer of a fused QKV projection:  K heads go through the per-head RMS norm (Qwen3's "(1 + w)" form),
// rotary embedding and ONE rounding to BF16 into the paged K cache; V heads are copied into the paged V cache.
//
// The reference does the K side in `fused_k_norm_rope_cache_write_bf16` and, with three position streams (MRoPE: rotary
// pair p takes the temporal, height or width position by p mod 3), `fused_k_norm_rope_mrope_cache_write_bf16`
// (kernels/gb10/common/fused_k_norm_rope_cache.cu:60-141, :149-243; `fused_k_norm_rope_cache_write_fp8`, :253-338, is the
// same chain ending in value * inv_scale cast to E4M3 with saturation: one block of head_dim threads per (token, head), K taken
// from a contiguous [tokens, kv_heads, head_dim] copy) and the V side with a separate cache-write launch.  Here one
// launch covers both and reads K and V where the projection left them — column ranges of the fused QKV output, with
// its row stride — so no contiguous copies are made.  One warp owns one (token, head): lane l holds elements l, l+32,
// l+64, ... of the head, so the sum of squares needs only shuffles and, for rotary_dim a multiple of 64, both
// elements of every rotated pair (d, d + rotary_dim/2) sit in the same lane.
//
// The arithmetic follows the reference operation by operation, in FP32 with every product and sum rounded on its own
// (the reference is built without FMA contraction) and in the reference's summation order — a butterfly over each
// group of 32 consecutive elements, then a butterfly over the group sums — so that the result is the same BF16 bits.
#pragma once

#include <cstdint>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace atlas {

constexpr int KVE_WARPS = 8;                 // (token, head) pairs per CTA
constexpr int KVE_MAX_HEAD_DIM = 256;

struct KvEpilogueParams {
    const uint16_t* k_in;        // first K column of token 0 (BF16), rows `in_row_stride` elements apart
    const uint16_t* v_in;        // first V column of token 0, or nullptr: K side only
    const uint16_t* k_norm_w;    // [head_dim] BF16
    const uint32_t* positions;   // [tokens]
    const uint32_t* positions_h; // MRoPE: the height and width position streams (pair p takes stream p mod 3: t, h, w), or both nullptr
    const uint32_t* positions_w;
    const long long* slot_mapping;   // [tokens], < 0: token skipped
    uint16_t* k_cache;           // [blocks, block_size, kv_heads, head_dim] BF16
    uint16_t* v_cache;           // same layout, or nullptr
    uint32_t tokens, kv_heads, head_dim, rotary_dim, block_size, in_row_stride;
    float rms_eps, theta;
    float fp8_inv_scale;         // != 0: k_cache is an E4M3 cache (one byte per element): value * fp8_inv_scale, saturating cast
};

__device__ __forceinline__ float kve_butterfly(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__global__ void __launch_bounds__(KVE_WARPS * 32)
kv_norm_rope_cache_kernel(const KvEpilogueParams p) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t heads_all = p.kv_heads * (p.v_in ? 2u : 1u);           // K heads, then V heads
    const uint64_t item = uint64_t(blockIdx.x) * KVE_WARPS + warp;
    if (item >= uint64_t(p.tokens) * heads_all) return;
    const uint32_t token = uint32_t(item / heads_all), h = uint32_t(item - uint64_t(token) * heads_all);
    const long long slot = p.slot_mapping[token];
    if (slot < 0) return;                                                  // padding token
    const bool is_v = h >= p.kv_heads;
    const uint32_t head = is_v ? h - p.kv_heads : h;
    const uint32_t n_grp = p.head_dim / 32u;                               // elements per lane (head_dim: a multiple of 32, <= 256)
    const uint16_t* src = (is_v ? p.v_in : p.k_in) + size_t(token) * p.in_row_stride + size_t(head) * p.head_dim;
    const size_t dst_at = (size_t(slot / (long long)p.block_size) * p.block_size + size_t(slot % (long long)p.block_size)) *
                              (size_t(p.kv_heads) * p.head_dim) + size_t(head) * p.head_dim;
    if (is_v) {
        uint16_t* dst = p.v_cache + dst_at;
        for (uint32_t j = 0; j < n_grp; ++j) dst[lane + 32u * j] = src[lane + 32u * j];
        return;
    }
    float x[KVE_MAX_HEAD_DIM / 32];
    float grp[KVE_MAX_HEAD_DIM / 32];
#pragma unroll
    for (uint32_t j = 0; j < uint32_t(KVE_MAX_HEAD_DIM / 32); ++j) {
        if (j < n_grp) {
            x[j] = __uint_as_float(uint32_t(src[lane + 32u * j]) << 16);
            grp[j] = kve_butterfly(__fmul_rn(x[j], x[j]));                 // sum over elements 32 j .. 32 j + 31
        }
    }
    // the group sums as lanes 0 .. n_grp-1 of one more butterfly
    float mine = 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < uint32_t(KVE_MAX_HEAD_DIM / 32); ++j)
        if (j < n_grp && lane == j) mine = grp[j];
    const float total = kve_butterfly(mine);
    const float rms = rsqrtf(__fadd_rn(__fdiv_rn(total, float(p.head_dim)), p.rms_eps));
    float nrm[KVE_MAX_HEAD_DIM / 32] = {};
#pragma unroll
    for (uint32_t j = 0; j < uint32_t(KVE_MAX_HEAD_DIM / 32); ++j)
        if (j < n_grp) {
            const float w = __uint_as_float(uint32_t(p.k_norm_w[lane + 32u * j]) << 16);
            nrm[j] = __fmul_rn(__fmul_rn(x[j], rms), __fadd_rn(1.0f, w));
        }
    const uint32_t half = p.rotary_dim / 2u, half_grp = half / 32u;        // rotary_dim: a multiple of 64
    const float pos_t = float(p.positions[token]);
    const float pos_h = p.positions_h ? float(p.positions_h[token]) : pos_t, pos_w = p.positions_w ? float(p.positions_w[token]) : pos_t;
    uint16_t* dst = p.k_cache + dst_at;
    uint8_t* dst8 = reinterpret_cast<uint8_t*>(p.k_cache) + dst_at;
    const bool fp8 = p.fp8_inv_scale != 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < uint32_t(KVE_MAX_HEAD_DIM / 32); ++j) {
        if (j >= n_grp) continue;
        const uint32_t d = lane + 32u * j;
        float out = nrm[j];
        if (d < p.rotary_dim) {
            const bool low = d < half;
            const uint32_t pair = low ? d : d - half;
            // the pair's two elements are in this lane: groups j and j +- half / 32 (constant indices keep them in registers)
            const uint32_t j0 = low ? j : j - half_grp, j1 = low ? j + half_grp : j;
            float x0 = 0.0f, x1 = 0.0f;
#pragma unroll
            for (uint32_t q = 0; q < uint32_t(KVE_MAX_HEAD_DIM / 32); ++q) {
                if (q == j0) x0 = nrm[q];
                if (q == j1) x1 = nrm[q];
            }
            const double freq_exp = double(2u * pair) / double(p.rotary_dim);
            const float freq = float(1.0 / pow(double(p.theta), freq_exp));
            const uint32_t section = pair % 3u;                            // (all three are the token's position without MRoPE)
            const float angle = __fmul_rn(section == 0u ? pos_t : (section == 1u ? pos_h : pos_w), freq);
            const float c = cosf(angle), s = sinf(angle);
            out = low ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
        }
        if (fp8) dst8[d] = uint8_t(__nv_cvt_float_to_fp8(__fmul_rn(out, p.fp8_inv_scale), __NV_SATFINITE, __NV_E4M3));
        else dst[d] = f32_to_bf16_bits(out);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// The decode-path consumer of the fused QKV projection, Q side included: per (token, head)
//   Q head:  q = rope( bf16( rmsnorm(q) ) )  in place,
//   K head:  the same chain, result into the paged K cache,
//   V head:  copied into the paged V cache,
// with the rounding points and the rotary form of the reference's `fused_qkv_norm_rope_cache_write_bf16`
// (kernels/gb10/common/fused_verify_elemwise.cu:78-224): the normed head is rounded to BF16 before the rotation
// (the chain it replaced stored it), the angle is position * inv_freq[pair] from a table, cosine and sine are scaled by
// the attention factor (YaRN), and the weight is `w` or `1 + w`.  One warp per (token, head), Q, K and V read where the
// projection wrote them (row strides given), the BF16 normed head staged in the warp's own shared-memory strip so that
// a lane can read the partner element of its pair.
//
// Summation order of the reference (one block of head_dim threads, thread t squaring the packed pair (2t, 2t + 1), a
// butterfly per warp, then a butterfly over the warp sums): group g of 64 elements = the reference's warp g, lane l of
// the group = its thread 32 g + l.
// ------------------------------------------------------------------------------------------------------------------
struct QkvEpilogueParams {
    uint16_t* q;                 // first Q column of token 0 (BF16, in/out), rows q_row_stride elements apart
    const uint16_t* k_in;        // first K column of token 0, rows kv_row_stride apart
    const uint16_t* v_in;
    const uint16_t* q_norm_w;    // [head_dim]
    const uint16_t* k_norm_w;    // [head_dim]
    const uint32_t* positions;   // [tokens]
    const float* inv_freq;       // [rotary_dim / 2]
    const long long* slot_mapping;
    uint16_t* k_cache;
    uint16_t* v_cache;
    uint32_t tokens, q_heads, kv_heads, head_dim, rotary_dim, block_size, q_row_stride, kv_row_stride;
    float rms_eps, attention_factor;
    uint32_t norm_offset_one;
};

__global__ void __launch_bounds__(KVE_WARPS * 32)
qkv_norm_rope_cache_kernel(const QkvEpilogueParams p) {
    __shared__ uint16_t normed_s[KVE_WARPS][KVE_MAX_HEAD_DIM];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t roles = p.q_heads + 2u * p.kv_heads;
    const uint64_t item = uint64_t(blockIdx.x) * KVE_WARPS + warp;
    if (item >= uint64_t(p.tokens) * roles) return;
    const uint32_t token = uint32_t(item / roles), role = uint32_t(item - uint64_t(token) * roles);
    const long long slot = p.slot_mapping[token];
    const size_t cache_at = slot < 0 ? 0 : (size_t(slot / (long long)p.block_size) * p.block_size + size_t(slot % (long long)p.block_size)) *
                                               (size_t(p.kv_heads) * p.head_dim);
    if (role >= p.q_heads + p.kv_heads) {                                  // V: a copy
        if (slot < 0) return;
        const uint32_t head = role - p.q_heads - p.kv_heads;
        const uint16_t* src = p.v_in + size_t(token) * p.kv_row_stride + size_t(head) * p.head_dim;
        uint16_t* dst = p.v_cache + cache_at + size_t(head) * p.head_dim;
        for (uint32_t d = lane; d < p.head_dim; d += 32) dst[d] = src[d];
        return;
    }
    const bool is_q = role < p.q_heads;
    const uint32_t head = is_q ? role : role - p.q_heads;
    if (!is_q && slot < 0) return;                                         // (the reference computes and drops it)
    uint16_t* qrow = p.q + size_t(token) * p.q_row_stride + size_t(head) * p.head_dim;
    const uint16_t* x = is_q ? qrow : p.k_in + size_t(token) * p.kv_row_stride + size_t(head) * p.head_dim;
    const uint16_t* w = is_q ? p.q_norm_w : p.k_norm_w;
    const uint32_t n_grp = (p.head_dim + 63u) / 64u;                       // the reference's warps that hold data
    constexpr uint32_t MAX_GRP = KVE_MAX_HEAD_DIM / 64;
    float x0v[MAX_GRP], x1v[MAX_GRP];
    float mine = 0.0f;
#pragma unroll
    for (uint32_t g = 0; g < MAX_GRP; ++g) {
        if (g >= n_grp) continue;
        const uint32_t e = 64u * g + 2u * lane;                            // this lane's packed pair of the group
        float sq = 0.0f;
        x0v[g] = x1v[g] = 0.0f;
        if (e < p.head_dim) {
            const uint32_t pk = *reinterpret_cast<const uint32_t*>(x + e);
            x0v[g] = __uint_as_float(pk << 16);
            x1v[g] = __uint_as_float(pk & 0xFFFF0000u);
            sq = __fadd_rn(__fmul_rn(x0v[g], x0v[g]), __fmul_rn(x1v[g], x1v[g]));
        }
        const float s = kve_butterfly(sq);
        if (lane == g) mine = s;
    }
    const float total = kve_butterfly(mine);
    const float rms = rsqrtf(__fadd_rn(__fdiv_rn(total, float(p.head_dim)), p.rms_eps));
#pragma unroll
    for (uint32_t g = 0; g < MAX_GRP; ++g) {
        if (g >= n_grp) continue;
        const uint32_t e = 64u * g + 2u * lane;
        if (e < p.head_dim) {
            const uint32_t wk = *reinterpret_cast<const uint32_t*>(w + e);
            const float w0 = __uint_as_float(wk << 16), w1 = __uint_as_float(wk & 0xFFFF0000u);
            const float f0 = p.norm_offset_one ? __fadd_rn(1.0f, w0) : w0, f1 = p.norm_offset_one ? __fadd_rn(1.0f, w1) : w1;
            normed_s[warp][e] = f32_to_bf16_bits(__fmul_rn(__fmul_rn(x0v[g], rms), f0));
            normed_s[warp][e + 1] = f32_to_bf16_bits(__fmul_rn(__fmul_rn(x1v[g], rms), f1));
        }
    }
    __syncwarp();
    uint16_t* dst = is_q ? qrow : p.k_cache + cache_at + size_t(head) * p.head_dim;
    const uint32_t pairs = p.rotary_dim / 2u;
    const float pos = float(p.positions[token]);
    for (uint32_t t = lane; t < p.head_dim; t += 32) {
        if (t < pairs) {
            const float a = __uint_as_float(uint32_t(normed_s[warp][t]) << 16);
            const float b = __uint_as_float(uint32_t(normed_s[warp][t + pairs]) << 16);
            const float angle = __fmul_rn(pos, p.inv_freq[t]);
            const float c = __fmul_rn(cosf(angle), p.attention_factor), s = __fmul_rn(sinf(angle), p.attention_factor);
            dst[t] = f32_to_bf16_bits(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
            dst[t + pairs] = f32_to_bf16_bits(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
        } else if (t >= p.rotary_dim) {
            dst[t] = normed_s[warp][t];                                    // channels beyond the rotary part pass through
        }
    }
}

}  // namespace atlas
