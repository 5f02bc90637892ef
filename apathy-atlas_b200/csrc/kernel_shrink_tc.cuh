// LoRA shrink for prefill batches on the tcgen05 tensor cores:
//     t[m, j] = f(s) * sum_k x[m,k] * A_s[j,k],   s = seq_slot[m].
//
// lora_shrink_mma_kernel (kernel_shrink_mma.cuh) spreads one (slot, 16 ranks, token tile) over a cluster so that a
// decode batch still has loads in flight on every SM; with thousands of tokens that shape reads every x row once
// per 16 ranks and spends its time in cluster barriers.  Here one CTA owns SHT_ROWS = 64 consecutive tokens and ALL
// ranks of EVERY adapter those tokens use, so x is read from HBM exactly once:
//
//   acc_i[row, j] = sum_k x[row, k] * A_{s_i}[j, k]        one accumulator per adapter s_i that occurs in the CTA's rows,
//                                                          side by side in tensor memory (lanes = rows,
//                                                          rank_pad columns each, at most 512 columns per pass)
//   t[row, :]     = f(s_i) * acc_i[row, :]  where seq_slot[row] == s_i
//
// i.e. the rows are not compacted: every row is multiplied with every adapter present in the CTA (a prefill chunk
// touches one to three) and the epilogue keeps, per row, the accumulator of its own adapter.  The surplus products
// cost nothing next to the memory traffic, and the contraction order of a row does not depend on its neighbours.
//
// Pipeline: a ring of shared-memory stages of 64 K elements — the x tile [64 x 128 B] and one A_s tile
// [rank_pad x 128 B] per present adapter, both in the 128-byte swizzled K-major layout the MMA reads — filled by ONE
// thread with TMA copies (cp.async.bulk.tensor, never multicast): one 2-D box of x and one 3-D box per adapter out
// of the A side of the strided adapter pool [max_loras][max_rank][k_in] (rows past max_rank are filled with zeros),
// so the copies of as many stages as fit are in flight at the cost of a handful of instructions per stage; one
// thread issues tcgen05.mma (M = 128 rows of which 64 are tokens, N = rank_pad, K = 16) per adapter and K step and releases the stage with
// tcgen05.commit.  Afterwards four warps read the accumulators back (lane = row) and write
//   * rows of t [M, max_rank] (routed rows only), or
//   * the masked [part_rows x 16] blocks of ShrinkParams::tile_out, numbered per token tile exactly as the fused
//     kernel numbers its granules — including the all-zero rows of blocks whose adapter occurs elsewhere in the
//     token tile but not in this CTA's rows.
// More adapters than fit into 512 columns are handled by further passes over the same rows.
// Every wait is bounded (1 s); on expiry the kernel records a status and leaves through the common teardown.
#pragma once

#include "kernel_shrink_mma.cuh"
#include "kernel_tc.cuh"

namespace atlas {

constexpr int SHT_THREADS = 256;
constexpr int SHT_ROWS = 64;             // tokens per CTA: half of the UMMA's 128 rows, so that a batch of a few thousand
                                         // tokens still gives every SM a CTA (the stream is bound by how many SMs pull);
                                         // MMA rows 64..127 read whatever follows the x tile in the stage and land in
                                         // accumulator lanes nobody reads
constexpr int SHT_KSTAGE = 64;           // K elements per stage (one 128-byte swizzle row of BF16)
constexpr int SHT_X_BYTES = SHT_ROWS * 128;
constexpr int SHT_MAX_STAGES = 12;
constexpr int SHT_RING_BYTES = 192 * 1024;
constexpr int SHT_MAX_ACC_COLS = 512;
constexpr int SHT_MAX_SLOTS = 32;        // adapters per pass (512 columns / 16 ranks)
constexpr int SHT_SMEM_BYTES = SHT_RING_BYTES + 128 * 128 + 1024;     // + what the MMA's rows 64..127 may touch past the last stage

__global__ void __launch_bounds__(SHT_THREADS, 1)
lora_shrink_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_a, const ShrinkParams p) {
    extern __shared__ uint8_t sht_dyn[];
    __shared__ int32_t slot_row[SHT_ROWS];               // validated slot of each of this CTA's rows (-1 = none)
    __shared__ uint32_t present_c[128];                  // slots that occur in this CTA's rows
    __shared__ uint32_t present_t[2][128];               // slots that occur in the (at most two) token tiles the rows lie in
    __shared__ uint32_t base_t[2][128];                  // granules of the slots in lower bitmap words, per token tile
    __shared__ uint32_t warp_cnt[2][4];
    __shared__ uint16_t cslot[SHT_MAX_SLOTS];            // adapters of the current pass, ascending
    __shared__ uint32_t n_cslot_s, next_word_s, next_bit_s;
    __shared__ uint64_t bars[2 * SHT_MAX_STAGES + 1];
    __shared__ uint32_t tmem_base_s, abort_s;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t m0 = p.m_begin + blockIdx.x * SHT_ROWS;      // (m_begin: a multiple of SHT_ROWS)
    if (m0 >= p.M) return;
    unsigned long long* prof = p.profile ? p.profile + size_t(blockIdx.x) * 8 : nullptr;
    const long long t_start = clock64();
    if (prof && tid == 0) prof[7] = tc::global_timer_ns();
    const uint32_t chunk = p.chunk ? p.chunk : 256u;     // token tile of the fused kernel (tile output only)
    const uint32_t tile_lo = m0 / chunk;                 // first token tile this CTA's rows lie in
    const uint32_t rank_pad = (p.max_rank + 15u) & ~15u; // accumulator columns per adapter
    const uint32_t per_pass = min(uint32_t(SHT_MAX_SLOTS), uint32_t(SHT_MAX_ACC_COLS) / rank_pad);
    const uint32_t ring = (tc::smem_u32(sht_dyn) + 1023u) & ~1023u;
    const uint32_t bar0 = tc::smem_u32(bars);
    volatile uint32_t* abort_flag = &abort_s;
    auto rank_of = [&](uint32_t s) { return p.rank_table ? min(p.rank_table[s], p.max_rank) : p.max_rank; };

    // ---- routing of this CTA's rows and of the token tiles they belong to ----
    if (tid < 128) { present_c[tid] = 0u; present_t[0][tid] = 0u; present_t[1][tid] = 0u; }
    if (tid == 0) { abort_s = 0u; next_word_s = 0u; next_bit_s = 0u; }
    __syncthreads();
    auto valid_slot = [&](uint32_t m) -> int32_t {
        if (m >= p.M) return -1;
        if (!p.seq_slot) return 0;
        int32_t s = p.seq_slot[m];
        if (s < 0) return -1;
        if (uint32_t(s) >= p.max_loras) return -1;                  // recorded by the kernel that consumes t
        if (p.a_table[s] == 0ull || (p.b_table && p.b_table[s] == 0ull)) return -1;
        return s;
    };
    if (tid < SHT_ROWS) {
        const int32_t s = valid_slot(m0 + tid);
        slot_row[tid] = s;
        if (s >= 0) atomicOr(&present_c[uint32_t(s) >> 5], 1u << (uint32_t(s) & 31u));
    }
    if (p.tile_out) {
        for (uint32_t tl = 0; tl < 2; ++tl) {
            const uint32_t t_m0 = (tile_lo + tl) * chunk;
            if (t_m0 >= min(m0 + uint32_t(SHT_ROWS), p.M)) break;
            for (uint32_t i = tid; i < chunk; i += SHT_THREADS) {
                const int32_t s = valid_slot(t_m0 + i);
                if (s >= 0) atomicOr(&present_t[tl][uint32_t(s) >> 5], 1u << (uint32_t(s) & 31u));
            }
        }
        __syncthreads();
        // exclusive prefix, over the 128 bitmap words, of the granules each word's slots contribute (warps 0-3: tile 0, 4-7: tile 1)
        const uint32_t tl = tid >> 7, w = tid & 127u;
        uint32_t cnt = 0;
        for (uint32_t bits = present_t[tl][w]; bits; bits &= bits - 1) cnt += (rank_of(w * 32 + (__ffs(bits) - 1)) + 15u) / 16u;
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= uint32_t(o)) incl += v;
        }
        if (lane == 31) warp_cnt[tl][warp & 3u] = incl;
        __syncthreads();
        uint32_t add = 0;
        for (uint32_t k = 0; k < (warp & 3u); ++k) add += warp_cnt[tl][k];
        base_t[tl][w] = add + incl - cnt;
    }
    // ---- barriers, tensor memory ----
    const uint32_t BAR_FULL = bar0, BAR_EMPTY = bar0 + 8 * SHT_MAX_STAGES, BAR_ACC = bar0 + 16 * SHT_MAX_STAGES;
    if (tid == 0) {
        for (int i = 0; i < SHT_MAX_STAGES; ++i) {
            tc::mbar_init(BAR_FULL + 8 * i, 1);          // the producer's arrival, with the stage's byte count
            tc::mbar_init(BAR_EMPTY + 8 * i, 1);
        }
        tc::mbar_init(BAR_ACC, 1);
        tc::fence_barrier_init();
    }
    if (warp == 4) { tc::tmem_alloc(tc::smem_u32(&tmem_base_s), 512); tc::tmem_relinquish(); }
    if (tid == 0) { tc::tma_prefetch_desc(&map_x); tc::tma_prefetch_desc(&map_a); }
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    const uint32_t tmem_acc = tmem_base_s;
    const long long t_setup = clock64();
    long long t_wait = 0;

    // position of slot s among the granules of token tile tl: granules of all present slots below it
    auto granules_ahead = [&](uint32_t tl, uint32_t s) -> uint32_t {
        uint32_t q = base_t[tl][s >> 5];
        for (uint32_t bits = present_t[tl][s >> 5] & ((1u << (s & 31u)) - 1u); bits; bits &= bits - 1)
            q += (rank_of((s & ~31u) + (__ffs(bits) - 1)) + 15u) / 16u;
        return q;
    };
    // where row `row` of this CTA keeps granule block q: element offset of its 32 bytes inside ShrinkParams::tile_out
    auto block_row = [&](uint32_t row, uint32_t q, uint32_t& swap) -> size_t {
        const uint32_t m = m0 + row, tile = m / chunk, idx = m % chunk;
        const uint32_t part = idx / p.part_rows, r = idx % p.part_rows;
        swap = (r >> 2) & 1u;
        return (((size_t(tile) * (chunk / p.part_rows) + part) * p.tile_cap + q) * p.part_rows + r) * 16;
    };
    // the two 16-byte halves of a block row, to every destination buffer
    auto store_block_row = [&](size_t at, uint32_t swap, const uint4& lo, const uint4& hi) {
        uint4* dst = reinterpret_cast<uint4*>(p.tile_out + at);
        dst[swap] = lo;
        dst[swap ^ 1u] = hi;
        for (uint32_t d = 1; d < p.n_tile_dest; ++d) {
            uint4* peer = reinterpret_cast<uint4*>(p.tile_out_more[d - 1] + at);
            peer[swap] = lo;
            peer[swap ^ 1u] = hi;
        }
    };

    // Parity each role waits for next, one bit per stage: the ring's depth changes from pass to pass (it depends on how
    // many adapters the pass holds), so phases are tracked per barrier rather than derived from a position.
    uint32_t empty_par = 0xFFFFFFFFu;                    // producers: a fresh barrier passes a wait on parity 1
    uint32_t full_par = 0u;                              // MMA thread
    uint32_t acc_phase = 0;
    bool ok = true;
    for (uint32_t pass = 0;; ++pass) {
        // ---- the adapters of this pass: the next `per_pass` set bits of present_c, ascending ----
        if (warp == 0) {
            uint32_t n = 0, w = next_word_s, b = next_bit_s;
            if (lane == 0) {
                while (w < 128 && n < per_pass) {
                    const uint32_t bits = present_c[w] & ~((b >= 32u) ? 0xFFFFFFFFu : ((1u << b) - 1u));
                    if (!bits) { ++w; b = 0; continue; }
                    const uint32_t bit = __ffs(bits) - 1;
                    cslot[n++] = uint16_t(w * 32 + bit);
                    b = bit + 1;
                    if (b >= 32u) { ++w; b = 0; }
                }
                n_cslot_s = n; next_word_s = w; next_bit_s = b;
            }
        }
        __syncthreads();
        const uint32_t n_cs = n_cslot_s;
        if (n_cs == 0 && pass > 0) break;
        const uint32_t n_arows = n_cs * rank_pad;                                    // A rows of a stage (all adapters)
        const uint32_t stage_bytes = SHT_X_BYTES + n_arows * 128u;
        const uint32_t n_stages = min(uint32_t(SHT_MAX_STAGES), uint32_t(SHT_RING_BYTES) / stage_bytes);
        const uint32_t n_ks = p.k_in / SHT_KSTAGE;

        if (n_cs > 0 && warp == 0 && lane == 0) {
            // ================================ TMA producer ================================
            for (uint32_t ks = 0; ok && ks < n_ks; ++ks) {
                const uint32_t s = ks % n_stages;
                const long long w0 = prof ? clock64() : 0;
                ok = tc::mbar_wait(BAR_EMPTY + 8 * s, (empty_par >> s) & 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 20);
                if (prof) t_wait += clock64() - w0;
                if (!ok) break;
                empty_par ^= 1u << s;
                const uint32_t st = ring + s * stage_bytes;
                tc::mbar_arrive_expect_tx(BAR_FULL + 8 * s, stage_bytes);
                // (every CTA walks K in the same order, so a row's result does not depend on how the batch is cut into launches)
                const uint32_t kk = ks;
                tc::tma_load_2d(st, &map_x, int32_t(kk * SHT_KSTAGE), int32_t(m0), BAR_FULL + 8 * s);
                for (uint32_t ci = 0; ci < n_cs; ++ci)
                    tc::tma_load_3d(st + SHT_X_BYTES + ci * rank_pad * 128u, &map_a, int32_t(kk * SHT_KSTAGE), 0, int32_t(cslot[ci]), BAR_FULL + 8 * s);
            }
        } else if (n_cs > 0 && warp == 4 && lane == 0) {
            // ================================ MMA issue ================================
            const uint32_t idesc = tc::make_idesc_bf16(rank_pad, 128u);
            for (uint32_t ks = 0; ok && ks < n_ks; ++ks) {
                const uint32_t s = ks % n_stages;
                const long long w0 = prof ? clock64() : 0;
                ok = tc::mbar_wait(BAR_FULL + 8 * s, (full_par >> s) & 1u, abort_flag, STATUS_WAIT_EXPIRED_MMA, 20);
                if (prof) t_wait += clock64() - w0;
                if (!ok) break;
                full_par ^= 1u << s;
                tc::tcgen05_fence_after();
                const uint32_t st = ring + s * stage_bytes;
                const uint64_t xd = tc::make_kmajor_sw128_desc(st);
                for (uint32_t ci = 0; ci < n_cs; ++ci) {
                    const uint64_t ad = tc::make_kmajor_sw128_desc(st + SHT_X_BYTES + ci * rank_pad * 128u);
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)     // 16 k = 32 bytes along the swizzled 128-byte rows
                        tc::umma_bf16_ss<false>(tmem_acc + ci * rank_pad, xd + 2 * j, ad + 2 * j, idesc, (ks | j) ? 1u : 0u);
                }
                tc::umma_commit<false>(BAR_EMPTY + 8 * s);
            }
            if (ok) tc::umma_commit<false>(BAR_ACC);
        }
        __syncwarp();

        if (warp >= 4) {
            // ================================ epilogue: lane = row ================================
            const uint32_t row = (warp & 3u) * 32 + lane;              // accumulator lane; lanes 64..127 hold nothing
            const bool has_rows = (warp & 3u) * 32 < uint32_t(SHT_ROWS);
            const int32_t my_slot = has_rows ? slot_row[row] : -1;
            const bool row_live = has_rows && m0 + row < p.M;
            if (n_cs > 0) {
                ok = tc::mbar_wait(BAR_ACC, acc_phase, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 200) && ok;
                tc::tcgen05_fence_after();
            }
            if (prof && tid == 128 && pass == 0) { prof[1] = clock64() - t_setup; prof[6] = n_cs; }
            if (ok && has_rows) {
                for (uint32_t ci = 0; ci < n_cs; ++ci) {
                    const uint32_t sl = cslot[ci];
                    const uint32_t rank = rank_of(sl);
                    const float f = (p.post != 0.0f) ? p.scale_table[sl] * p.post : 1.0f;
                    const bool mine = my_slot == int32_t(sl);
                    uint32_t q0 = 0;
                    if (p.tile_out && row_live) q0 = granules_ahead((m0 + row) / chunk - tile_lo, sl);
                    const uint32_t j_end = p.tile_out ? rank : p.max_rank;
                    for (uint32_t j0 = 0; j0 < j_end; j0 += 16) {
                        uint32_t v[16];
                        tc::tmem_ld16(tmem_acc + (((warp & 3u) * 32u) << 16) + ci * rank_pad + j0, v);   // (whole warp: .sync.aligned)
                        tc::tmem_ld_wait();
                        if (!row_live) continue;
                        uint32_t w[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float a = (mine && j0 + 2 * u < rank) ? __uint_as_float(v[2 * u]) * f : 0.0f;
                            const float b = (mine && j0 + 2 * u + 1 < rank) ? __uint_as_float(v[2 * u + 1]) * f : 0.0f;
                            w[u] = pack_bf16x2(a, b);
                        }
                        if (p.tile_out) {
                            const uint32_t q = q0 + j0 / 16;
                            if (q >= p.tile_cap) { record_status(STATUS_TILE_CAPACITY); continue; }
                            uint32_t swap;
                            const size_t at = block_row(row, q, swap);
                            store_block_row(at, swap, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
                        } else if (mine) {
                            uint16_t* dst = p.out + size_t(m0 + row) * p.max_rank + j0;
                            if (j0 + 16 <= p.max_rank && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                                reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                                reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                            } else {
                                for (uint32_t e = 0; e < 16 && j0 + e < p.max_rank; ++e) dst[e] = uint16_t(w[e >> 1] >> (16u * (e & 1u)));
                            }
                        }
                    }
                }
                // blocks of adapters that occur in the row's token tile but not in this CTA's rows: this row is all zeros there
                if (pass == 0 && p.tile_out && row_live) {
                    const uint32_t tl = (m0 + row) / chunk - tile_lo;
                    for (uint32_t wd = 0; wd < 128; ++wd) {
                        uint32_t bits = present_t[tl][wd] & ~present_c[wd];
                        if (!bits) continue;
                        for (; bits; bits &= bits - 1) {
                            const uint32_t sl = wd * 32 + (__ffs(bits) - 1);
                            const uint32_t q0 = granules_ahead(tl, sl), n_gr = (rank_of(sl) + 15u) / 16u;
                            for (uint32_t k = 0; k < n_gr && q0 + k < p.tile_cap; ++k) {
                                uint32_t swap;
                                const size_t at = block_row(row, q0 + k, swap);
                                store_block_row(at, swap, make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u));
                            }
                        }
                    }
                }
            }
            tc::tcgen05_fence_before();
        }
        if (prof && pass == 0) {
            if (tid == 0) prof[3] = t_wait;
            if (tid == 128) prof[4] = t_wait;
        }
        if (n_cs > 0) acc_phase ^= 1u;
        __syncthreads();                                 // every MMA of the pass has completed (the epilogue waited for them): the ring is free
        if (*abort_flag) break;                          // (uniform: read after the barrier)
        if (n_cs < per_pass) break;                      // no adapters left for another pass
    }

    // ---- teardown ----
    tc::tcgen05_fence_before();
    __syncthreads();
    if (prof && tid == 128) {
        const long long t_end = clock64();
        prof[0] = t_setup - t_start;
        prof[5] = t_end - t_start;
        prof[2] = (t_end - t_setup) - (long long)prof[1];
    }
    if (warp == 4) {
        tc::tcgen05_fence_after();
        tc::tmem_dealloc(tmem_acc, 512);
    }
}

}  // namespace atlas
