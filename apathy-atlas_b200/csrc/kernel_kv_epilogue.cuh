// The K/V consumer of a fused QKV projection:  K heads go through the per-head RMS norm (Qwen3's "(1 + w)" form),
// rotary embedding and ONE rounding to BF16 into the paged K cache; V heads are copied into the paged V cache.
//
// The reference does the K side in `fused_k_norm_rope_cache_write_bf16`
// (kernels/gb10/common/fused_k_norm_rope_cache.cu:60-141: one block of head_dim threads per (token, head), K taken
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
    const long long* slot_mapping;   // [tokens], < 0: token skipped
    uint16_t* k_cache;           // [blocks, block_size, kv_heads, head_dim] BF16
    uint16_t* v_cache;           // same layout, or nullptr
    uint32_t tokens, kv_heads, head_dim, rotary_dim, block_size, in_row_stride;
    float rms_eps, theta;
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
    const float pos = float(p.positions[token]);
    uint16_t* dst = p.k_cache + dst_at;
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
            const float angle = __fmul_rn(pos, freq);
            const float c = cosf(angle), s = sinf(angle);
            out = low ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
        }
        dst[d] = f32_to_bf16_bits(out);
    }
}

}  // namespace atlas
