// The K/V consumer of a fused QKV projection:  K heads go through the per-head RMS norm (Qwen3's "(1 + w)" form),
// rotary embedding and ONE rounding to BF16 into the paged K cache; V heads are copied into the paged V cache.
//
// The reference does the K side in `fused_k_norm_rope_cache_write_bf16` and, with three position streams (MRoPE: rotary
// pair p takes the temporal, height or width position by p mod 3), `fused_k_norm_rope_mrope_cache_write_bf16`
// (kernels/gb10/common/fused_k_norm_rope_cache.cu:60-141, :149-243; `fused_k_norm_rope_cache_write_fp8`, :253-338, is the
// same chain ending in value * inv_scale cast to E4M3 with saturation: one block of head_dim threads per (token, head), K taken
// from a contiguous [tokens, kv_heads, head_dim] copy) and the V side with a separate cache-write launch.  Here one
// launch covers both and reads K and V where the projection left them — column ranges of the fused QKV output, with
// its row stride — so no contiguous copies are made.  A warp takes the heads of one token, one (token, head) at a time:
// lane l holds elements l, l+32, l+64, ... of the head, so the sum of squares needs only shuffles and, for rotary_dim a
// multiple of 64, both elements of every rotated pair (d, d + rotary_dim/2) sit in the same lane.
//
// The arithmetic follows the reference operation by operation, in FP32 with every product and sum rounded on its own
// (the reference is built without FMA contraction) and in the reference's summation order — a butterfly over each
// group of 32 consecutive elements, then a butterfly over the group sums; `kve_group_total` walks the same tree with
// fewer shuffles — so that the result is the same BF16 bits.
#pragma once

#include <cstdint>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace atlas {

constexpr int KVE_WARPS = 8;                 // warps per CTA
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

// The head's sum of squares from N per-lane partial sums (one per group of lanes' elements), bit for bit the two-level
// form: each group summed over the 32 lanes by offsets 16, 8, 4, 2, 1, then the group sums, held by lanes 0 .. N-1 of a
// zero-filled warp, summed the same way (for N = 8 that is ((s0+s4)+(s2+s6)) + ((s1+s5)+(s3+s7)); a zero stands in for a
// group the head does not have).  Addition commutes, so a lane may keep one of two values at a level and pass the other
// one to its partner: N groups take N-1 + (5 - log2 N) + log2 N shuffles instead of 5 (N + 1).  After the first part the
// lane whose bits 16, 8, 4 spell the group's index bits 0, 1, 2 holds that group's sum.
template <uint32_t N>
__device__ __forceinline__ float kve_group_total(float (&s)[N], const uint32_t lane) {
    static_assert(N == 1 || N == 2 || N == 4 || N == 8, "group count");
    constexpr uint32_t FULL = 0xFFFFFFFFu;
    uint32_t o = 16;
    if constexpr (N >= 2) {
        const bool up = (lane & 16u) != 0u;
#pragma unroll
        for (uint32_t k = 0; k < N / 2; ++k) {
            const float keep = up ? s[2 * k + 1] : s[2 * k], send = up ? s[2 * k] : s[2 * k + 1];
            s[k] = __fadd_rn(keep, __shfl_xor_sync(FULL, send, 16));
        }
        o = 8;
    }
    if constexpr (N >= 4) {
        const bool up = (lane & 8u) != 0u;
#pragma unroll
        for (uint32_t k = 0; k < N / 4; ++k) {
            const float keep = up ? s[2 * k + 1] : s[2 * k], send = up ? s[2 * k] : s[2 * k + 1];
            s[k] = __fadd_rn(keep, __shfl_xor_sync(FULL, send, 8));
        }
        o = 4;
    }
    if constexpr (N >= 8) {
        const bool up = (lane & 4u) != 0u;
        const float keep = up ? s[1] : s[0], send = up ? s[0] : s[1];
        s[0] = __fadd_rn(keep, __shfl_xor_sync(FULL, send, 4));
        o = 2;
    }
    float v = s[0];
#pragma unroll
    for (; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, o));
    if constexpr (N >= 8) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, 4));
    if constexpr (N >= 4) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, 8));
    if constexpr (N >= 2) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, 16));
    return v;
}

// total / head_dim rounded to nearest; for a power of two the product with the exact reciprocal is the same number
__device__ __forceinline__ float kve_mean(const float total, const uint32_t head_dim) {
    return (head_dim & (head_dim - 1u)) == 0u ? __fmul_rn(total, __uint_as_float((127u - (31u - __clz(head_dim))) << 23))
                                              : __fdiv_rn(total, float(head_dim));
}

constexpr int KVE_TOKENS = 8;                // tokens per CTA (prefill form)
constexpr int KVE_INFLIGHT = 4;              // heads a warp has loaded before it starts on the first of them

// NG: head_dim / 32 rounded up to 2, 4 or 8 (register arrays sized for the head at hand).  EXACT: head_dim = 32 NG,
// rotary_dim = 64 and a BF16 cache, known when the kernel is compiled (the common shapes): no masked groups, and which
// group holds a pair's other half is a constant.
template <uint32_t NG, bool EXACT>
__global__ void __launch_bounds__(KVE_WARPS * 32)
kv_norm_rope_cache_kernel(KvEpilogueParams p) {
    static_assert(KVE_TOKENS == KVE_WARPS, "one warp per token of the CTA");
    if constexpr (EXACT) { p.head_dim = 32u * NG; p.rotary_dim = 64u; p.fp8_inv_scale = 0.0f; }
    // One CTA per KVE_TOKENS tokens.  The rotation's frequency depends on the pair only and its cosine and sine on
    // (token, pair) only, so the FP64 power is evaluated once per CTA and pair, the two transcendental calls once per
    // token and pair — the reference evaluates all three per element — and every head reads them from shared memory.
    // Same calls on the same arguments: same bits.  The op is a stream; what limits it is the latency of a head's chain
    // (load, group sums, rsqrt, store), so a warp loads KVE_INFLIGHT heads before it works on the first.
    __shared__ float cos_s[KVE_TOKENS][KVE_MAX_HEAD_DIM / 2], sin_s[KVE_TOKENS][KVE_MAX_HEAD_DIM / 2];
    __shared__ float freq_s[KVE_MAX_HEAD_DIM / 2];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t token0 = blockIdx.x * KVE_TOKENS;
    const uint32_t n_tok = min(uint32_t(KVE_TOKENS), p.tokens - token0);
    const uint32_t half = p.rotary_dim / 2u, half_grp = half / 32u;        // rotary_dim: a multiple of 64
    for (uint32_t pair = threadIdx.x; pair < half; pair += KVE_WARPS * 32) {
        const double freq_exp = double(2u * pair) / double(p.rotary_dim);
        freq_s[pair] = float(1.0 / pow(double(p.theta), freq_exp));
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n_tok * half; i += KVE_WARPS * 32) {
        const uint32_t tk = i / half, pair = i - tk * half;
        const uint32_t section = pair % 3u;                                // MRoPE: temporal / height / width stream by pair
        const uint32_t* ps = (section == 0u || !p.positions_h) ? p.positions : (section == 1u ? p.positions_h : p.positions_w);
        const float angle = __fmul_rn(float(ps[token0 + tk]), freq_s[pair]);
        cos_s[tk][pair] = cosf(angle);
        sin_s[tk][pair] = sinf(angle);
    }
    __syncthreads();
    const uint32_t heads_all = p.kv_heads * (p.v_in ? 2u : 1u);           // K heads, then V heads
    const uint32_t n_grp = p.head_dim / 32u;                               // elements per lane (head_dim: a multiple of 32, <= 256)
    const bool fp8 = p.fp8_inv_scale != 0.0f;
    const uint32_t tk = warp;                                              // a warp takes all heads of one token
    if (tk >= n_tok) return;
    const long long slot = p.slot_mapping[token0 + tk];
    if (slot < 0) return;                                                  // padding token
    const uint16_t* const k_tok = p.k_in + size_t(token0 + tk) * p.in_row_stride;
    const uint16_t* const v_tok = p.v_in ? p.v_in + size_t(token0 + tk) * p.in_row_stride : nullptr;
    // page slot / block_size, offset slot % block_size in a cache of [pages, block_size, kv_heads, head_dim]: row `slot`
    const size_t row_at = size_t(slot) * (size_t(p.kv_heads) * p.head_dim);
    for (uint32_t h0 = 0; h0 < heads_all; h0 += KVE_INFLIGHT) {
        uint16_t raw[KVE_INFLIGHT][NG];
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t h = h0 + r;
            if (h >= heads_all) continue;
            const uint16_t* src = h < p.kv_heads ? k_tok + h * p.head_dim : v_tok + (h - p.kv_heads) * p.head_dim;
#pragma unroll
            for (uint32_t j = 0; j < NG; ++j)
                if (j < n_grp) raw[r][j] = src[lane + 32u * j];
        }
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t h = h0 + r;
            if (h >= heads_all) continue;                                  // (warp-uniform)
            const bool is_v = h >= p.kv_heads;
            const uint32_t head = is_v ? h - p.kv_heads : h;
            const size_t dst_at = row_at + head * p.head_dim;
            if (is_v) {
                uint16_t* dst = p.v_cache + dst_at;
#pragma unroll
                for (uint32_t j = 0; j < NG; ++j)
                    if (j < n_grp) dst[lane + 32u * j] = raw[r][j];
                continue;
            }
            float x[NG], sq[NG];
#pragma unroll
            for (uint32_t j = 0; j < NG; ++j) {
                x[j] = j < n_grp ? __uint_as_float(uint32_t(raw[r][j]) << 16) : 0.0f;
                sq[j] = __fmul_rn(x[j], x[j]);                                 // group j = elements 32 j .. 32 j + 31
            }
            const float total = kve_group_total<NG>(sq, lane);
            const float rms = rsqrtf(__fadd_rn(kve_mean(total, p.head_dim), p.rms_eps));
            float nrm[NG] = {};
#pragma unroll
            for (uint32_t j = 0; j < NG; ++j)
                if (j < n_grp) {
                    const float w = __uint_as_float(uint32_t(p.k_norm_w[lane + 32u * j]) << 16);
                    nrm[j] = __fmul_rn(__fmul_rn(x[j], rms), __fadd_rn(1.0f, w));
                }
            uint16_t* dst = p.k_cache + dst_at;
            uint8_t* dst8 = reinterpret_cast<uint8_t*>(p.k_cache) + dst_at;
#pragma unroll
            for (uint32_t j = 0; j < NG; ++j) {
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
                    for (uint32_t q = 0; q < NG; ++q) {
                        if (q == j0) x0 = nrm[q];
                        if (q == j1) x1 = nrm[q];
                    }
                    const float c = cos_s[tk][pair], s = sin_s[tk][pair];
                    out = low ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
                }
                if (fp8) dst8[d] = uint8_t(__nv_cvt_float_to_fp8(__fmul_rn(out, p.fp8_inv_scale), __NV_SATFINITE, __NV_E4M3));
                else dst[d] = f32_to_bf16_bits(out);
            }
        }
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
// projection wrote them (row strides given).  A lane reads the partner element of its pair by one shuffle when
// rotary_dim = 64 (the halves of a pair are then 16 lanes apart in the head's first 64 channels), otherwise from the
// BF16 normed head staged in the warp's own shared-memory strip.
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

// MAX_GRP: head_dim / 64 rounded up to 1, 2 or 4.  EXACT: head_dim = 64 MAX_GRP and rotary_dim = 64 (the common shapes),
// known when the kernel is compiled, so that no lane is masked, a pair's halves meet by one shuffle and the general
// form with its shared-memory strip drops out.
template <uint32_t MAX_GRP, bool EXACT>
__global__ void __launch_bounds__(KVE_WARPS * 32, MAX_GRP == 4 ? 4 : 6)     // (occupancy matters more here than a few held values)
qkv_norm_rope_cache_kernel(QkvEpilogueParams p) {
    if constexpr (EXACT) { p.head_dim = 64u * MAX_GRP; p.rotary_dim = 64u; }
    // one CTA per token; cosine and sine of the token's angles evaluated once for all its heads (see above)
    __shared__ uint16_t normed_s[EXACT ? 1 : KVE_WARPS][EXACT ? 2 : KVE_MAX_HEAD_DIM];
    __shared__ float cos_s[KVE_MAX_HEAD_DIM / 2], sin_s[KVE_MAX_HEAD_DIM / 2];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t token = blockIdx.x;
    const uint32_t pairs = p.rotary_dim / 2u;
    {
        const float pos = float(p.positions[token]);
        for (uint32_t t = threadIdx.x; t < pairs; t += KVE_WARPS * 32) {
            const float angle = __fmul_rn(pos, p.inv_freq[t]);
            cos_s[t] = __fmul_rn(cosf(angle), p.attention_factor);
            sin_s[t] = __fmul_rn(sinf(angle), p.attention_factor);
        }
    }
    __syncthreads();
    const long long slot = p.slot_mapping[token];
    const uint32_t n_grp = EXACT ? MAX_GRP : (p.head_dim + 63u) / 64u;     // the reference's warps that hold data
    const bool in_lanes = EXACT || (p.rotary_dim == 64u && (p.head_dim & 63u) == 0u);
    // in-lane form: this lane's two angles, held for all of the token's heads
    float c0 = 0.0f, s0 = 0.0f, c1 = 0.0f, s1 = 0.0f;
    if (in_lanes) {
        const uint32_t t = (2u * lane) & 31u;
        c0 = cos_s[t], s0 = sin_s[t], c1 = cos_s[t + 1], s1 = sin_s[t + 1];
    }
    uint32_t have = EXACT ? (1u << MAX_GRP) - 1u : 0u;                     // bit g: this lane holds a pair of group g
    if constexpr (!EXACT) {
#pragma unroll
        for (uint32_t g = 0; g < MAX_GRP; ++g)
            if (g < n_grp && 64u * g + 2u * lane < p.head_dim) have |= 1u << g;
    }

    auto load_head = [&](uint32_t (&rw)[MAX_GRP], const uint16_t* x) {
#pragma unroll
        for (uint32_t g = 0; g < MAX_GRP; ++g)
            rw[g] = ((have >> g) & 1u) ? *reinterpret_cast<const uint32_t*>(x + 64u * g + 2u * lane) : 0u;
    };
    // per-head RMS norm, rotation and one rounding of the head held as packed pairs in rw; result to dst
    auto norm_rope_head = [&](const uint32_t (&rw)[MAX_GRP], const uint16_t* w, uint16_t* dst) {
        float x0v[MAX_GRP], x1v[MAX_GRP], sq[MAX_GRP];
#pragma unroll
        for (uint32_t g = 0; g < MAX_GRP; ++g) {                           // (a group the head does not have was loaded as zero)
            x0v[g] = __uint_as_float(rw[g] << 16);
            x1v[g] = __uint_as_float(rw[g] & 0xFFFF0000u);
            sq[g] = __fadd_rn(__fmul_rn(x0v[g], x0v[g]), __fmul_rn(x1v[g], x1v[g]));
        }
        const float total = kve_group_total<MAX_GRP>(sq, lane);
        const float rms = rsqrtf(__fadd_rn(kve_mean(total, p.head_dim), p.rms_eps));
        if (in_lanes) {
            // rotary_dim = 64 over whole 64-channel groups: a pair's two halves sit 16 lanes apart in group 0, so they
            // meet by one shuffle and nothing goes through shared memory; the arithmetic is that of the general form
#pragma unroll
            for (uint32_t g = 0; g < MAX_GRP; ++g) {
                if (g >= n_grp) continue;
                const uint32_t e = 64u * g + 2u * lane;
                const uint32_t wk = *reinterpret_cast<const uint32_t*>(w + e);
                const float w0 = __uint_as_float(wk << 16), w1 = __uint_as_float(wk & 0xFFFF0000u);
                const float f0 = p.norm_offset_one ? __fadd_rn(1.0f, w0) : w0, f1 = p.norm_offset_one ? __fadd_rn(1.0f, w1) : w1;
                const uint32_t own = pack_bf16x2(__fmul_rn(__fmul_rn(x0v[g], rms), f0), __fmul_rn(__fmul_rn(x1v[g], rms), f1));
                uint32_t out = own;
                if (g == 0) {
                    const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, own, 16);
                    const bool low = lane < 16u;
                    const uint32_t first = low ? own : other, second = low ? other : own;   // channels t and t + 32
                    const float a0 = __uint_as_float(first << 16), a1 = __uint_as_float(first & 0xFFFF0000u);
                    const float b0 = __uint_as_float(second << 16), b1 = __uint_as_float(second & 0xFFFF0000u);
                    const float r0 = low ? __fsub_rn(__fmul_rn(a0, c0), __fmul_rn(b0, s0)) : __fadd_rn(__fmul_rn(b0, c0), __fmul_rn(a0, s0));
                    const float r1 = low ? __fsub_rn(__fmul_rn(a1, c1), __fmul_rn(b1, s1)) : __fadd_rn(__fmul_rn(b1, c1), __fmul_rn(a1, s1));
                    out = pack_bf16x2(r0, r1);
                }
                *reinterpret_cast<uint32_t*>(dst + e) = out;
            }
            return;
        }
        if constexpr (EXACT) return;
        __syncwarp();                                                      // the strip's previous head has been read
#pragma unroll
        for (uint32_t g = 0; g < MAX_GRP; ++g) {
            if (!((have >> g) & 1u)) continue;
            const uint32_t e = 64u * g + 2u * lane;
            const uint32_t wk = *reinterpret_cast<const uint32_t*>(w + e);
            const float w0 = __uint_as_float(wk << 16), w1 = __uint_as_float(wk & 0xFFFF0000u);
            const float f0 = p.norm_offset_one ? __fadd_rn(1.0f, w0) : w0, f1 = p.norm_offset_one ? __fadd_rn(1.0f, w1) : w1;
            normed_s[warp][e] = f32_to_bf16_bits(__fmul_rn(__fmul_rn(x0v[g], rms), f0));
            normed_s[warp][e + 1] = f32_to_bf16_bits(__fmul_rn(__fmul_rn(x1v[g], rms), f1));
        }
        __syncwarp();
        for (uint32_t t = lane; t < p.head_dim; t += 32) {
            if (t < pairs) {
                const float a = __uint_as_float(uint32_t(normed_s[warp][t]) << 16);
                const float b = __uint_as_float(uint32_t(normed_s[warp][t + pairs]) << 16);
                const float c = cos_s[t], s = sin_s[t];
                dst[t] = f32_to_bf16_bits(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
                dst[t + pairs] = f32_to_bf16_bits(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
            } else if (t >= p.rotary_dim) {
                dst[t] = normed_s[warp][t];                                // channels beyond the rotary part pass through
            }
        }
    };

    // Q heads, in place: a warp loads KVE_INFLIGHT heads, then works on each
    uint16_t* const q_tok = p.q + size_t(token) * p.q_row_stride;
    for (uint32_t h0 = warp; h0 < p.q_heads; h0 += KVE_WARPS * KVE_INFLIGHT) {
        uint32_t raw[KVE_INFLIGHT][MAX_GRP];
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t head = h0 + r * KVE_WARPS;
            if (head < p.q_heads) load_head(raw[r], q_tok + head * p.head_dim);
        }
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t head = h0 + r * KVE_WARPS;
            if (head < p.q_heads) norm_rope_head(raw[r], p.q_norm_w, q_tok + head * p.head_dim);
        }
    }
    if (slot < 0) return;                                                  // (the reference computes a padding token's K and drops it)
    // K heads into the cache row `slot` (page slot / block_size, offset slot % block_size of [pages, block_size, kv_heads,
    // head_dim]), V heads copied beside them: items 0 .. kv_heads-1 are K, the rest V
    const uint16_t* const k_tok = p.k_in + size_t(token) * p.kv_row_stride;
    const uint16_t* const v_tok = p.v_in + size_t(token) * p.kv_row_stride;
    const size_t cache_at = size_t(slot) * (size_t(p.kv_heads) * p.head_dim);
    for (uint32_t i0 = warp; i0 < 2u * p.kv_heads; i0 += KVE_WARPS * KVE_INFLIGHT) {
        uint32_t raw[KVE_INFLIGHT][MAX_GRP];
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t item = i0 + r * KVE_WARPS;
            if (item < 2u * p.kv_heads)
                load_head(raw[r], item < p.kv_heads ? k_tok + item * p.head_dim : v_tok + (item - p.kv_heads) * p.head_dim);
        }
#pragma unroll
        for (uint32_t r = 0; r < uint32_t(KVE_INFLIGHT); ++r) {
            const uint32_t item = i0 + r * KVE_WARPS;
            if (item >= 2u * p.kv_heads) continue;
            if (item < p.kv_heads) {
                norm_rope_head(raw[r], p.k_norm_w, p.k_cache + cache_at + item * p.head_dim);
            } else {
                uint16_t* dst = p.v_cache + cache_at + (item - p.kv_heads) * p.head_dim;
#pragma unroll
                for (uint32_t g = 0; g < MAX_GRP; ++g)
                    if ((have >> g) & 1u) *reinterpret_cast<uint32_t*>(dst + 64u * g + 2u * lane) = raw[r][g];
            }
        }
    }
}

}  // namespace atlas
