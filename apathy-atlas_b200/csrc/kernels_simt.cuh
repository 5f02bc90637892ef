// CUDA-core kernels: NVFP4 codecs, the grouped LoRA shrink, the staged expand+fold, and a
// shape-agnostic tiled linear.  The shrink is the production shrink for every path; the rest
// serve shapes the tcgen05 path does not take and the reference-rounding ("staged") mode.
#pragma once

#include "common.cuh"

namespace atlas {

// =============================================================================================
// NVFP4 -> BF16 decode.  One block per row, threads stride over 8-element groups.
// out = bf16(E2M1[nib] * (e4m3(scale) * g)), the operation order of
// kernels/gb10/common/dequant_nvfp4_bf16.cu:64-72, so results are bit-identical to it.
// =============================================================================================
__global__ void __launch_bounds__(256)
dequant_nvfp4_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                     uint16_t* __restrict__ out, float g, uint32_t N, uint32_t K) {
    const uint32_t row = blockIdx.x;
    if (row >= N) return;
    const uint8_t* rp = packed + size_t(row) * (K / 2);
    const uint8_t* rs = scales + size_t(row) * (K / 16);
    uint16_t* ro = out + size_t(row) * K;
    for (uint32_t b = threadIdx.x; b < K / 2; b += blockDim.x) {
        const float s = e4m3_decode(rs[b >> 3]) * g;
        const uint32_t byte = rp[b];
        const uint32_t w = uint32_t(f32_to_bf16_bits(e2m1_decode(byte & 0xFu) * s)) |
                           (uint32_t(f32_to_bf16_bits(e2m1_decode(byte >> 4) * s)) << 16);
        reinterpret_cast<uint32_t*>(ro)[b] = w;
    }
}

// =============================================================================================
// BF16 -> NVFP4 quantiser, one thread per 16-element group.
// Software E4M3 encode and E2M1 bins as kernels/gb10/common/quantize_bf16_to_nvfp4.cu:42-124,
// group loop as :197-242.
// =============================================================================================
__device__ __forceinline__ uint32_t e4m3_encode_sw(float v) {
    uint32_t bits = __float_as_uint(v);
    const uint32_t sign = bits >> 31;
    if ((bits & 0x7FFFFFFFu) == 0u) return sign << 7;
    float a = fabsf(v);
    if (a > 448.0f) a = 448.0f;
    bits = __float_as_uint(a);
    const int fe = int((bits >> 23) & 0xFF) - 127;
    const uint32_t fm = bits & 0x7FFFFFu;
    if (fe < -9) return sign << 7;
    if (fe < -6) {
        int man = int(a * 512.0f + 0.5f);
        man = man > 7 ? 7 : (man < 0 ? 0 : man);
        return (sign << 7) | uint32_t(man);
    }
    int e = fe + 7;
    uint32_t man;
    if (e < 1) e = 1;
    if (e > 15) { e = 15; man = 6; }
    else {
        man = (fm + (1u << 19)) >> 20;
        if (man > 7) { man = 0; if (++e > 15) { e = 15; man = 6; } }
    }
    return (sign << 7) | (uint32_t(e) << 3) | man;
}

// E2M1 code of v with the reference's bins (|v| <= .25 -> 0, <= .75 -> .5, <= 1.25 -> 1, <= 1.75 -> 1.5, <= 2.5 -> 2,
// <= 3.5 -> 3, <= 5 -> 4, else 6: ties go to the smaller magnitude, kernels/gb10/common/quantize_bf16_to_nvfp4.cu:109-124).
// From 1 upward E2M1 is "one mantissa bit": adding just under half an ulp of that bit to the FP32 pattern and truncating
// rounds half DOWN, which is exactly the `<=` of the bins (and carries into the exponent at 1.75 and 3.5); the code is
// then twice the unbiased exponent plus the mantissa bit plus 2, clamped to 6.0's code.  Below 1 the two bins are compared
// directly.  Same results as the chain of compares, in half the instructions (the quantiser is bound by instruction issue).
__device__ __forceinline__ uint32_t e2m1_quantize(float v) {
    const uint32_t bits = __float_as_uint(v);
    const uint32_t mag = bits & 0x7FFFFFFFu;
    const float a = __uint_as_float(mag);
    // (mag + 0x1FFFFF) >> 22 = (biased exponent << 1) | mantissa bit, after rounding half down
    int32_t code = int32_t((mag + 0x1FFFFFu) >> 22) - (127 * 2 - 2);
    code = min(max(code, 2), 7);
    uint32_t idx = a <= 0.75f ? (a <= 0.25f ? 0u : 1u) : uint32_t(code);
    if (mag > 0x7F800000u) idx = 7u;                 // NaN compares false everywhere in the chain of bins: the last one
    return (v < 0.0f ? 8u : 0u) | idx;
}

// `in_row_stride` (elements) lets the rows of `in` be spaced wider than K (activations); the outputs
// are dense.  `vec` != 0: rows and outputs are 16-/8-byte aligned, so a group is read with two 128-bit
// loads and its codes leave as one 64-bit store.
__global__ void __launch_bounds__(256)
quantize_nvfp4_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ scales, float scale2, uint32_t N, uint32_t K, uint32_t in_row_stride,
                      uint32_t vec) {
    const uint32_t groups = K / 16;
    const size_t total = size_t(N) * groups;
    const float inv_scale2 = scale2 > 0.0f ? __fdiv_rn(1.0f, scale2) : 0.0f;
    for (size_t gi = size_t(blockIdx.x) * blockDim.x + threadIdx.x; gi < total; gi += size_t(gridDim.x) * blockDim.x) {
        const uint16_t* p = in + (gi / groups) * in_row_stride + (gi % groups) * 16;
        float v[16];
        float gmax = 0.0f;
        if (vec) {
            const uint4 lo = __ldg(reinterpret_cast<const uint4*>(p)), hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(uint32_t(p[i]) << 16);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) gmax = fmaxf(gmax, fabsf(v[i]));
        const float f8 = gmax > 0.0f ? __fdiv_rn(__fmul_rn(gmax, inv_scale2), 6.0f) : 0.0f;
        const uint32_t byte = e4m3_encode_sw(f8);
        scales[gi] = uint8_t(byte);
        const float eff = __fmul_rn(e4m3_decode(byte), scale2);
        const float inv_eff = eff > 0.0f ? __fdiv_rn(1.0f, eff) : 0.0f;
        uint32_t q[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i / 8] |= e2m1_quantize(__fmul_rn(v[i], inv_eff)) << (4 * (i % 8));
        if (vec) {
            *reinterpret_cast<uint2*>(packed + gi * 8) = make_uint2(q[0], q[1]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) packed[gi * 8 + i] = uint8_t(q[i / 4] >> (8 * (i % 4)));
        }
    }
}

// =============================================================================================
// Grouped LoRA shrink:  t[m, j] = f(s) * sum_k x[m,k] * A_s[j,k],  s = seq_slot[m].
//
// One CTA owns (adapter slot s, RT consecutive ranks, a chunk of TC tokens).  It scans the
// chunk's seq_slot entries for rows routed to s, then walks those rows TG at a time: every
// thread keeps a K-slice of the TG x RT partial sums in registers, loading x and A with
// 128-bit accesses, so A_s is fetched from L2/HBM once per CTA and re-served by L1 for later
// row groups instead of once per row as in kernels/gb10/common/lora_bgmv.cu:84-99.
// Partial sums are reduced by warp shuffles, then across the 8 warps through shared memory.
//
// Output rounding: BF16, the reference's lora_xa boundary (lora_bgmv.cu:121-125).
//   f(s) = 1                     (reference semantics: xa unscaled)
//   f(s) = scale_table[s]*post   (fused path: the expand runs inside the MMA accumulator, which
//                                 holds y / (scale2 * 2^8))
// Ranks >= rank_table[s] are written as zero, never skipped: the fused expand multiplies them
// by zero-padded B columns and must not meet uninitialised bits.
// uniform mode (seq_slot == nullptr): every row uses `a_uniform` (apply_lora_delta).
// =============================================================================================
constexpr int SHRINK_RT = 4;      // ranks per CTA
constexpr int SHRINK_TG = 4;      // rows per register pass
constexpr int SHRINK_TC = 256;    // rows scanned per CTA
constexpr int SHRINK_THREADS = 256;

struct ShrinkParams {
    const uint16_t* x;
    const int32_t* seq_slot;        // nullable
    const uint64_t* a_table;
    const uint64_t* b_table;        // nullable; when given, a null B entry also disables the slot
    const float* scale_table;       // used when prescale != 0
    const uint32_t* rank_table;     // nullable
    const uint16_t* a_uniform;      // used when seq_slot == nullptr
    uint16_t* out;                  // [M, max_rank]
    uint32_t M, k_in, max_rank, x_row_stride, max_loras;
    float post;                     // 0 => unscaled output
    uint32_t release_dependents;    // let a programmatic dependent launch start while this grid runs
    // Tile output (tensor-core shrink only; tile_out == nullptr: rows of `out` as above).  The token axis
    // is cut into tiles of `chunk` tokens, each tile into parts of `part_rows` tokens (the whole tile, or
    // halves for CTA pairs).  For every tile, the (slot, 16-rank granule) pairs that occur in it are
    // numbered in ascending (slot, granule) order, and pair number q is written, for part h of tile i, as
    // a complete [part_rows x 16] BF16 block at tile_out + (((i * parts + h) * tile_cap + q) * part_rows) * 16:
    // the shrink result in rows routed to the slot, zeros in every other row, the two 16-byte halves of a
    // row swapped where (row / 4) is odd.  That is the activation operand of one LoRA K-step of the fused
    // kernel exactly as the MMA reads it from shared memory (K-major, 32-byte swizzle), so blocks are
    // fetched as plain bytes and consecutive blocks with one copy.
    uint16_t* tile_out;
    uint32_t tile_cap;              // blocks reserved per tile
    uint32_t chunk;                 // tokens scanned per CTA (<= 256); 0 = 256
    uint32_t part_rows;             // chunk or chunk / 2
    uint32_t ksplit;                // tensor-core shrink: CTAs per cluster sharing K (set by the launcher)
    // Token-sharded tile output (tcgen05 shrink only): the launch covers rows [m_begin, m_begin + m_count) of the batch
    // (m_count == 0: all of it) and writes every block row into n_tile_dest buffers of identical layout —
    // tile_out itself and tile_out_more[0 .. n_tile_dest - 2] (the same scratch on other GPUs, mapped into this process).
    uint32_t m_begin, m_count;
    uint32_t n_tile_dest;           // 0 or 1: tile_out only
    uint16_t* tile_out_more[7];
    // host side only: the A side of the adapter pool as a strided array (0: not known), for the launcher's tensor map
    const void* a_pool_base;
    size_t a_slot_stride;
    // optional diagnostics (tcgen05 shrink only): 16 u64 words per CTA — set-up, K loop, epilogue and total cycles, the
    // producer's and the MMA thread's wait cycles, adapters in the first pass, start time (ns), issue cycles of both
    unsigned long long* profile;
};

__global__ void __launch_bounds__(SHRINK_THREADS)
lora_shrink_grouped_kernel(const ShrinkParams p) {
    __shared__ uint16_t rows[SHRINK_TC];
    __shared__ uint32_t warp_count[SHRINK_THREADS / 32];
    __shared__ float red[SHRINK_THREADS / 32][SHRINK_TG * SHRINK_RT];

    // The fused layer launches its main kernel as a programmatic dependent of this grid; it reads
    // this grid's output only behind its own griddepcontrol.wait, so it may start right away.
    if (p.release_dependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s = blockIdx.x;
    const uint32_t j0 = blockIdx.y * SHRINK_RT;
    const uint32_t m_base = blockIdx.z * SHRINK_TC;

    const uint16_t* A;
    float f = 1.0f;
    uint32_t rank = p.max_rank;
    if (p.seq_slot) {
        const uint64_t a_addr = p.a_table[s];
        if (a_addr == 0ull) return;
        if (p.b_table && p.b_table[s] == 0ull) return;
        A = reinterpret_cast<const uint16_t*>(a_addr);
        if (p.rank_table) rank = min(p.rank_table[s], p.max_rank);
        if (p.post != 0.0f) f = p.scale_table[s] * p.post;
    } else {
        A = p.a_uniform;
    }

    // ---- ordered list of this chunk's rows routed to slot s ----
    uint32_t n_rows;
    {
        const uint32_t m = m_base + tid;
        bool hit = false;
        if (m < p.M) hit = p.seq_slot ? (p.seq_slot[m] == int32_t(s)) : true;
        const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < SHRINK_THREADS / 32; ++w) {
            const uint32_t c = warp_count[w];
            if (w < int(warp)) before += c;
            total += c;
        }
        if (hit) rows[before + __popc(ballot & ((1u << lane) - 1u))] = uint16_t(tid);
        n_rows = total;
        __syncthreads();
    }
    if (n_rows == 0) return;

    const bool vec_ok = (p.k_in % 8 == 0) && (p.x_row_stride % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(A)) % 16 == 0);

    for (uint32_t g0 = 0; g0 < n_rows; g0 += SHRINK_TG) {
        float acc[SHRINK_TG][SHRINK_RT];
#pragma unroll
        for (int t = 0; t < SHRINK_TG; ++t)
#pragma unroll
            for (int r = 0; r < SHRINK_RT; ++r) acc[t][r] = 0.0f;

        const uint16_t* xr[SHRINK_TG];
#pragma unroll
        for (int t = 0; t < SHRINK_TG; ++t) {
            const uint32_t idx = min(g0 + t, n_rows - 1);   // clamp: duplicates are discarded at the store
            xr[t] = p.x + size_t(m_base + rows[idx]) * p.x_row_stride;
        }
        // ranks at or beyond the adapter's true rank contribute zero and are not read
        uint32_t live = 0;
#pragma unroll
        for (int r = 0; r < SHRINK_RT; ++r) if (j0 + r < rank) live = r + 1;

        if (live) {
            if (vec_ok) {
                const uint32_t kv_n = p.k_in / 8;
                for (uint32_t kv = tid; kv < kv_n; kv += SHRINK_THREADS) {
                    uint4 xa[SHRINK_TG];
#pragma unroll
                    for (int t = 0; t < SHRINK_TG; ++t) xa[t] = reinterpret_cast<const uint4*>(xr[t])[kv];
#pragma unroll
                    for (int r = 0; r < SHRINK_RT; ++r) {
                        if (r < int(live)) {
                            const uint4 av = __ldg(reinterpret_cast<const uint4*>(A + size_t(j0 + r) * p.k_in) + kv);
                            const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                            for (int t = 0; t < SHRINK_TG; ++t) {
                                const uint32_t xw[4] = {xa[t].x, xa[t].y, xa[t].z, xa[t].w};
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    acc[t][r] = fmaf(bf16_lo(xw[q]), bf16_lo(aw[q]), acc[t][r]);
                                    acc[t][r] = fmaf(bf16_hi(xw[q]), bf16_hi(aw[q]), acc[t][r]);
                                }
                            }
                        }
                    }
                }
            } else {
                for (uint32_t k = tid; k < p.k_in; k += SHRINK_THREADS) {
#pragma unroll
                    for (int r = 0; r < SHRINK_RT; ++r) {
                        if (r < int(live)) {
                            const float av = __uint_as_float(uint32_t(A[size_t(j0 + r) * p.k_in + k]) << 16);
#pragma unroll
                            for (int t = 0; t < SHRINK_TG; ++t)
                                acc[t][r] = fmaf(__uint_as_float(uint32_t(xr[t][k]) << 16), av, acc[t][r]);
                        }
                    }
                }
            }
        }

        // ---- block reduction of TG*RT partial sums ----
#pragma unroll
        for (int t = 0; t < SHRINK_TG; ++t)
#pragma unroll
            for (int r = 0; r < SHRINK_RT; ++r) {
                float v = acc[t][r];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0) red[warp][t * SHRINK_RT + r] = v;
            }
        __syncthreads();
        if (tid < SHRINK_TG * SHRINK_RT) {
            const uint32_t t = tid / SHRINK_RT, r = tid % SHRINK_RT;
            if (g0 + t < n_rows && j0 + r < p.max_rank) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < SHRINK_THREADS / 32; ++w) v += red[w][tid];
                const uint32_t m = m_base + rows[g0 + t];
                // f == 1 exactly in the unscaled mode, so v * f is v there
                p.out[size_t(m) * p.max_rank + j0 + r] = f32_to_bf16_bits((j0 + r < rank) ? v * f : 0.0f);
            }
        }
        __syncthreads();
    }
}

// =============================================================================================
// Staged expand + fold (reference rounding):
//   delta = bf16(sum_j xa[m,j] * B_s[o,j]);  out[m,o] = bf16(f32(out[m,o]) + scale_s * f32(delta))
// as kernels/gb10/common/lora_bgmv.cu:139-225 (fold order :214-223).  One CTA owns 128 outputs
// x 32 rows; each thread keeps one output column and walks the rows, so B rows are re-served
// by L1 while consecutive rows share an adapter, instead of being re-read per row.
// uniform mode (seq_slot == nullptr) serves apply_lora_delta; `delta_out` (nullable) receives
// the BF16 delta the reference materialises in its lora_delta scratch.
// =============================================================================================
constexpr int EXPAND_OUTS = 128;
constexpr int EXPAND_ROWS = 32;
constexpr int EXPAND_MAX_RANK = 256;

struct ExpandParams {
    const uint16_t* xa;             // [M, max_rank]
    const int32_t* seq_slot;        // nullable
    const uint64_t* a_table;        // nullable; a null A entry also disables the slot
    const uint64_t* b_table;
    const float* scale_table;
    const uint16_t* b_uniform;
    float scale_uniform;
    uint16_t* out;                  // [M, out_row_stride]
    uint16_t* delta_out;            // nullable, [M, n_out]
    uint32_t M, n_out, max_rank, out_row_stride, max_loras;
    uint32_t rows_per_cta;          // 1..EXPAND_ROWS: fewer rows per CTA for small batches, so that the grid still fills the GPU
};

__global__ void __launch_bounds__(EXPAND_OUTS)
lora_expand_fold_kernel(const ExpandParams p) {
    __shared__ float xs[EXPAND_ROWS][EXPAND_MAX_RANK + 1];
    __shared__ int32_t slot_s[EXPAND_ROWS];
    const uint32_t tid = threadIdx.x;
    const uint32_t o = blockIdx.x * EXPAND_OUTS + tid;
    const uint32_t rpc = p.rows_per_cta ? min(p.rows_per_cta, uint32_t(EXPAND_ROWS)) : uint32_t(EXPAND_ROWS);
    const uint32_t m0 = blockIdx.y * rpc;
    const uint32_t nrows = min(rpc, p.M - m0);

    if (tid < EXPAND_ROWS) {
        int32_t s = -1;
        if (tid < nrows) {
            if (!p.seq_slot) s = 0;
            else {
                s = p.seq_slot[m0 + tid];
                if (s >= 0) {
                    if (uint32_t(s) >= p.max_loras) { record_status(STATUS_SLOT_OUT_OF_RANGE); s = -1; }
                    else if (p.b_table[s] == 0ull || (p.a_table && p.a_table[s] == 0ull)) s = -1;
                }
            }
        }
        slot_s[tid] = s;
    }
    __syncthreads();
    for (uint32_t i = tid; i < nrows * p.max_rank; i += EXPAND_OUTS) {
        const uint32_t r = i / p.max_rank, j = i % p.max_rank;
        xs[r][j] = slot_s[r] >= 0 ? __uint_as_float(uint32_t(p.xa[size_t(m0 + r) * p.max_rank + j]) << 16) : 0.0f;
    }
    __syncthreads();
    if (o >= p.n_out) return;

    const bool vec_ok = (p.max_rank % 8 == 0);
    for (uint32_t r = 0; r < nrows; ++r) {
        const int32_t s = slot_s[r];
        if (s < 0) continue;
        const uint16_t* B = p.seq_slot ? reinterpret_cast<const uint16_t*>(p.b_table[s]) : p.b_uniform;
        const float sc = p.seq_slot ? p.scale_table[s] : p.scale_uniform;
        const uint16_t* br = B + size_t(o) * p.max_rank;
        float acc = 0.0f;
        if (vec_ok && (reinterpret_cast<uintptr_t>(br) % 16 == 0)) {
            for (uint32_t jv = 0; jv < p.max_rank / 8; ++jv) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(br) + jv);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc = fmaf(xs[r][jv * 8 + 2 * q], bf16_lo(bw[q]), acc);
                    acc = fmaf(xs[r][jv * 8 + 2 * q + 1], bf16_hi(bw[q]), acc);
                }
            }
        } else {
            for (uint32_t j = 0; j < p.max_rank; ++j)
                acc = fmaf(xs[r][j], __uint_as_float(uint32_t(br[j]) << 16), acc);
        }
        const uint16_t dbf = f32_to_bf16_bits(acc);
        if (p.delta_out) p.delta_out[size_t(m0 + r) * p.n_out + o] = dbf;
        uint16_t* dst = p.out + size_t(m0 + r) * p.out_row_stride + o;
        const float base = __uint_as_float(uint32_t(*dst) << 16);
        *dst = f32_to_bf16_bits(__fadd_rn(base, __fmul_rn(sc, __uint_as_float(uint32_t(dbf) << 16))));
    }
}

// =============================================================================================
// Shape-agnostic tiled linear on CUDA cores:  y[m,f] = bf16(scale2 * sum_k x[m,k] * w[f,k]),
// w decoded to FP32 exactly (E2M1 * E4M3), FP32 accumulation.  64 x 64 output tile, K step 32,
// 256 threads with 4 x 4 outputs each.  Serves shapes the tcgen05 path rejects (K not a
// multiple of 256, unaligned strides) and the dense-BF16 base.
// =============================================================================================
constexpr int SIMT_TM = 64, SIMT_TF = 64, SIMT_TK = 32;

struct SimtLinearParams {
    const uint16_t* x;
    const uint8_t* w_packed;
    const uint8_t* w_scale;
    const uint16_t* w_bf16;     // dense base when non-null
    uint16_t* y;
    uint32_t M, N, K, x_row_stride, out_row_stride;
    float scale2;
};

__global__ void __launch_bounds__(256)
linear_simt_kernel(const SimtLinearParams p) {
    __shared__ float xs[SIMT_TK][SIMT_TM + 4];
    __shared__ float ws[SIMT_TK][SIMT_TF + 4];
    const uint32_t tid = threadIdx.x;
    const uint32_t f0 = blockIdx.x * SIMT_TF, m0 = blockIdx.y * SIMT_TM;
    const uint32_t ty = tid / 16, tx = tid % 16;
    float acc[4][4] = {};

    for (uint32_t k0 = 0; k0 < p.K; k0 += SIMT_TK) {
        {   // x tile: thread -> (row, 8 consecutive k)
            const uint32_t r = tid >> 2, kq = (tid & 3) * 8;
            const uint32_t m = m0 + r;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t k = k0 + kq + i;
                xs[kq + i][r] = (m < p.M && k < p.K) ? __uint_as_float(uint32_t(p.x[size_t(m) * p.x_row_stride + k]) << 16) : 0.0f;
            }
        }
        {   // w tile: thread -> (feature, 8 consecutive k)
            const uint32_t r = tid >> 2, kq = (tid & 3) * 8;
            const uint32_t f = f0 + r, k = k0 + kq;
            if (f < p.N && k < p.K) {
                if (p.w_bf16) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        ws[kq + i][r] = (k + i < p.K) ? __uint_as_float(uint32_t(p.w_bf16[size_t(f) * p.K + k + i]) << 16) : 0.0f;
                } else {
                    const float sc = e4m3_decode(p.w_scale[size_t(f) * (p.K / 16) + k / 16]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t byte = p.w_packed[size_t(f) * (p.K / 2) + k / 2 + i];
                        ws[kq + 2 * i][r] = e2m1_decode(byte & 0xFu) * sc;
                        ws[kq + 2 * i + 1][r] = e2m1_decode(byte >> 4) * sc;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) ws[kq + i][r] = 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SIMT_TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = xs[k][ty * 4 + i]; b[i] = ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t f = f0 + tx * 4 + j;
            if (f < p.N) p.y[size_t(m) * p.out_row_stride + f] = f32_to_bf16_bits(acc[i][j] * p.scale2);
        }
    }
}

}  // namespace atlas
