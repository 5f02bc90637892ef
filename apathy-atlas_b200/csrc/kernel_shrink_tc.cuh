// LoRA shrink for prefill batches on the tcgen05 tensor cores:
//     t[m, j] = f(s) * sum_k x[m,k] * A_s[j,k],   s = seq_slot[m].
//
// lora_shrink_mma_kernel (kernel_shrink_mma.cuh) spreads one (slot, 16 ranks, token tile) over a cluster so that a
// decode batch still has loads in flight on every SM; with thousands of tokens that shape reads every x row once
// per 16 ranks and spends its time in cluster barriers.  Here a cluster of `ksplit` CTAs owns SHT_ROWS = 128
// consecutive tokens and ALL ranks of EVERY adapter those tokens use, so x is read from HBM exactly once:
//
//   acc_i[row, j] = sum_k x[row, k] * A_{s_i}[j, k]        one accumulator per adapter s_i that occurs in the rows,
//                                                          side by side in tensor memory (lanes = rows,
//                                                          rank_pad columns each, at most 512 columns per pass)
//   t[row, :]     = f(s_i) * acc_i[row, :]  where seq_slot[row] == s_i
//
// i.e. the rows are not compacted: every row is multiplied with every adapter present in the CTA (a prefill chunk
// touches one to three) and the epilogue keeps, per row, the accumulator of its own adapter.  The surplus products
// cost nothing next to the memory traffic, and the contraction order of a row does not depend on its neighbours.
//
// What bounds the K loop is the issue rate of these small MMAs (N = rank_pad columns: a 128 x 64 x 16 MMA with both
// operands in shared memory takes ~230 cycles, measured, however few columns it has), not the stream: so the MMA
// covers all 128 rows of the datapath, and the cluster's CTAs each contract a contiguous share of K (CTA z: K blocks
// [z, z+1) * n / ksplit) into their own accumulators.  Afterwards the partial sums are exchanged over distributed
// shared memory: the 16-column granules are dealt out to the CTAs round robin, every CTA sends the granules it does
// not own to their owners, and the owner adds the partials in CTA order 0, 1, ... (its own in its place), so the
// result depends neither on timing nor on which CTA owns a granule.
//
// Pipeline: a ring of shared-memory stages of 64 K elements — the x tile [128 x 128 B] and one A_s tile
// [rank_pad x 128 B] per present adapter, both in the 128-byte swizzled K-major layout the MMA reads — filled by ONE
// thread with TMA copies (cp.async.bulk.tensor, never multicast): one 2-D box of x and one 3-D box per adapter out
// of the A side of the strided adapter pool [max_loras][max_rank][k_in] (rows past max_rank are filled with zeros);
// one thread issues tcgen05.mma (M = 128, N = rank_pad x the adapters that fit into 256 columns, K = 16) per K step and
// releases the stage with tcgen05.commit.  Afterwards all eight warps read the accumulators back (lane = row) and write
//   * rows of t [M, max_rank] (routed rows only), or
//   * the masked [part_rows x 16] blocks of ShrinkParams::tile_out, numbered per token tile exactly as the fused
//     kernel numbers its granules — including the all-zero rows of blocks whose adapter occurs elsewhere in the
//     token tile but not in this CTA's rows.
// More adapters than fit into 512 columns are handled by further passes over the same rows.
// Every wait is bounded (1 s); on expiry the kernel records a status and skips the work that is left, but still
// reaches every cluster barrier (their number depends on the routing data only, which the CTAs of a cluster share).
#pragma once

#include "kernel_shrink_mma.cuh"
#include "kernel_tc.cuh"

namespace atlas {

constexpr int SHT_THREADS = 256;
constexpr int SHT_ROWS = 128;            // tokens per cluster: the UMMA's 128 rows
constexpr int SHT_KSTAGE = 64;           // K elements per stage (one 128-byte swizzle row of BF16)
constexpr int SHT_X_BYTES = SHT_ROWS * 128;
constexpr int SHT_MAX_STAGES = 12;
constexpr int SHT_RING_BYTES = 192 * 1024;   // also the receive area of the partial-sum exchange (<= 3/4 * 32 granules * 8 KB)
constexpr int SHT_MAX_ACC_COLS = 512;
constexpr int SHT_MAX_SLOTS = 32;        // adapters per pass (512 columns / 16 ranks)
constexpr int SHT_MAX_KSPLIT = 4;
constexpr int SHT_SMEM_BYTES = SHT_RING_BYTES + 1024;

__global__ void __launch_bounds__(SHT_THREADS, 1)
lora_shrink_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_a, const ShrinkParams p) {
    extern __shared__ uint8_t sht_dyn[];
    __shared__ int32_t slot_row[SHT_ROWS];               // validated slot of each of this CTA's rows (-1 = none)
    __shared__ uint32_t present_c[128];                  // slots that occur in this CTA's rows
    __shared__ uint32_t present_t[2][128];               // slots that occur in the (at most two) token tiles the rows lie in
    __shared__ uint32_t base_t[2][128];                  // granules of the slots in lower bitmap words, per token tile
    __shared__ uint32_t warp_cnt[2][4];
    __shared__ uint16_t cslot[SHT_MAX_SLOTS];            // adapters of the current pass, ascending
    __shared__ uint16_t cq0[2][SHT_MAX_SLOTS];           // their first granule number in either token tile
    __shared__ uint16_t crank[SHT_MAX_SLOTS];            // their true ranks
    __shared__ float cscale[SHT_MAX_SLOTS];              // and output factors
    __shared__ uint32_t n_cslot_s, next_word_s, next_bit_s;
    __shared__ uint64_t bars[2 * SHT_MAX_STAGES + 1];
    __shared__ uint32_t tmem_base_s, abort_s;

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ksn = p.ksplit ? p.ksplit : 1u;       // CTAs per cluster (consecutive blockIdx.x)
    const uint32_t kz = ksn > 1u ? tc::cluster_cta_rank() : 0u;
    const uint32_t m0 = p.m_begin + (blockIdx.x / ksn) * SHT_ROWS;      // (m_begin: a multiple of 64)
    if (m0 >= p.M) return;                               // (the whole cluster returns)
    unsigned long long* prof = p.profile ? p.profile + size_t(blockIdx.x) * 16 : nullptr;
    const long long t_start = clock64();
    if (prof && tid == 0) prof[7] = tc::global_timer_ns();
    const uint32_t chunk = p.chunk ? p.chunk : 256u;     // token tile of the fused kernel (tile output only; >= 128)
    const uint32_t tile_lo = m0 / chunk;                 // first token tile this CTA's rows lie in
    const uint32_t rank_pad = (p.max_rank + 15u) & ~15u; // accumulator columns per adapter
    const uint32_t gpa = rank_pad / 16u;                 // granules per adapter
    const uint32_t per_pass = min(uint32_t(SHT_MAX_SLOTS), uint32_t(SHT_MAX_ACC_COLS) / rank_pad);
    const uint32_t n_words = (p.max_loras + 31u) >> 5;   // bitmap words in use
    const uint32_t ring = (tc::smem_u32(sht_dyn) + 1023u) & ~1023u;
    const uint8_t* ring_gen = sht_dyn + (ring - tc::smem_u32(sht_dyn));
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
    long long t_wait = 0, t_a = 0, t_b = 0;

    // position of slot s among the granules of token tile tl: granules of all present slots below it
    auto granules_ahead = [&](uint32_t tl, uint32_t s) -> uint32_t {
        uint32_t q = base_t[tl][s >> 5];
        for (uint32_t bits = present_t[tl][s >> 5] & ((1u << (s & 31u)) - 1u); bits; bits &= bits - 1)
            q += (rank_of((s & ~31u) + (__ffs(bits) - 1)) + 15u) / 16u;
        return q;
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

    // this CTA's share of K
    const uint32_t n_ks_all = p.k_in / SHT_KSTAGE;
    const uint32_t ks_lo = kz * n_ks_all / ksn, ks_hi = (kz + 1u) * n_ks_all / ksn;
    const uint32_t n_ks = ks_hi - ks_lo;

    // row of this thread in the accumulators (lane of its warp's quadrant), and which of the quadrant's two warps it is in
    const uint32_t quad = warp & 3u, half = warp >> 2;
    const uint32_t row = quad * 32 + lane;
    const int32_t my_slot = slot_row[row];
    const bool row_live = m0 + row < p.M;
    // where this row's blocks live: block q of the row is at row_at + q * part_rows * 16 elements
    uint32_t tl = 0, swap = 0;
    size_t row_at = 0;
    if (p.tile_out && row_live) {
        const uint32_t m = m0 + row, tile = m / chunk, idx = m - tile * chunk;
        const uint32_t part = idx / p.part_rows, r = idx - part * p.part_rows;
        tl = tile - tile_lo;
        swap = (r >> 2) & 1u;
        row_at = ((size_t(tile) * (chunk / p.part_rows) + part) * p.tile_cap * p.part_rows + r) * 16;
    }
    const size_t q_step = size_t(p.part_rows) * 16;
    // this thread's 16 accumulator columns of granule (ci, j0), or zeros when this CTA contracted nothing
    auto load_granule = [&](uint32_t ci, uint32_t j0, uint32_t (&v)[16]) {
        if (n_ks > 0) {
            tc::tmem_ld16(tmem_acc + ((quad * 32u) << 16) + ci * rank_pad + j0, v);      // (whole warp: .sync.aligned)
            tc::tmem_ld_wait();
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = 0u;
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
                while (w < n_words && n < per_pass) {
                    const uint32_t bits = present_c[w] & ~((b >= 32u) ? 0xFFFFFFFFu : ((1u << b) - 1u));
                    if (!bits) { ++w; b = 0; continue; }
                    const uint32_t bit = __ffs(bits) - 1;
                    cslot[n++] = uint16_t(w * 32 + bit);
                    b = bit + 1;
                    if (b >= 32u) { ++w; b = 0; }
                }
                n_cslot_s = n; next_word_s = w; next_bit_s = b;
            }
            __syncwarp();
            const uint32_t n_sel = n_cslot_s;
            if (lane < n_sel) {
                const uint32_t sl = cslot[lane];
                crank[lane] = uint16_t(rank_of(sl));
                cscale[lane] = (p.post != 0.0f) ? p.scale_table[sl] * p.post : 1.0f;
                if (p.tile_out) {
                    cq0[0][lane] = uint16_t(min(granules_ahead(0, sl), 0xFFFFu));
                    cq0[1][lane] = uint16_t(min(granules_ahead(1, sl), 0xFFFFu));
                }
            }
        }
        __syncthreads();
        if (prof && tid == 128 && pass == 0) prof[11] = clock64() - t_setup;
        const uint32_t n_cs = n_cslot_s;
        if (n_cs == 0 && pass > 0) break;                                            // (uniform over the cluster)
        const uint32_t n_arows = n_cs * rank_pad;                                    // A rows of a stage (all adapters)
        const uint32_t stage_bytes = SHT_X_BYTES + n_arows * 128u;
        const uint32_t n_stages = min(uint32_t(SHT_MAX_STAGES), uint32_t(SHT_RING_BYTES) / stage_bytes);
        const bool have_acc = n_cs > 0 && n_ks > 0;                                  // this CTA's accumulators hold something

        if (have_acc && warp == 0 && lane == 0) {
            // ================================ TMA producer ================================
            for (uint32_t i = 0; ok && i < n_ks; ++i) {
                const uint32_t s = i % n_stages;
                const long long w0 = prof ? clock64() : 0;
                ok = tc::mbar_wait(BAR_EMPTY + 8 * s, (empty_par >> s) & 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 20);
                if (prof) t_wait += clock64() - w0;
                if (!ok) break;
                empty_par ^= 1u << s;
                const uint32_t st = ring + s * stage_bytes;
                const long long i0 = prof ? clock64() : 0;
                tc::mbar_arrive_expect_tx(BAR_FULL + 8 * s, stage_bytes);
                // (K is walked in ascending order by every cluster, so a row's result does not depend on how the batch is cut into launches)
                const int32_t k0 = int32_t((ks_lo + i) * SHT_KSTAGE);
                tc::tma_load_2d(st, &map_x, k0, int32_t(m0), BAR_FULL + 8 * s);
                for (uint32_t ci = 0; ci < n_cs; ++ci)
                    tc::tma_load_3d(st + SHT_X_BYTES + ci * rank_pad * 128u, &map_a, k0, 0, int32_t(cslot[ci]), BAR_FULL + 8 * s);
                if (prof) t_a += clock64() - i0;
            }
        } else if (have_acc && warp == 4 && lane == 0) {
            // ================================ MMA issue ================================
            // The adapters' A tiles lie one after the other in a stage and their accumulators side by side in tensor memory,
            // so one MMA covers as many adapters as fit into 256 columns.
            const uint32_t per_mma = max(1u, 256u / rank_pad);
            for (uint32_t i = 0; ok && i < n_ks; ++i) {
                const uint32_t s = i % n_stages;
                const long long w0 = prof ? clock64() : 0;
                ok = tc::mbar_wait(BAR_FULL + 8 * s, (full_par >> s) & 1u, abort_flag, STATUS_WAIT_EXPIRED_MMA, 20);
                if (prof) t_wait += clock64() - w0;
                if (!ok) break;
                full_par ^= 1u << s;
                const long long i0 = prof ? clock64() : 0;
                tc::tcgen05_fence_after();
                const uint32_t st = ring + s * stage_bytes;
                const uint64_t xd = tc::make_kmajor_sw128_desc(st);
                for (uint32_t c0 = 0; c0 < n_cs; c0 += per_mma) {
                    const uint32_t idesc = tc::make_idesc_bf16(min(per_mma, n_cs - c0) * rank_pad, 128u);
                    const uint64_t ad = tc::make_kmajor_sw128_desc(st + SHT_X_BYTES + c0 * rank_pad * 128u);
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)     // 16 k = 32 bytes along the swizzled 128-byte rows
                        tc::umma_bf16_ss<false>(tmem_acc + c0 * rank_pad, xd + 2 * j, ad + 2 * j, idesc, (i | j) ? 1u : 0u);
                }
                const long long i1 = prof ? clock64() : 0;
                tc::umma_commit<false>(BAR_EMPTY + 8 * s);
                if (prof) { t_a += i1 - i0; t_b += clock64() - i1; }
            }
            if (ok) tc::umma_commit<false>(BAR_ACC);
        }
        __syncwarp();

        // ---- every warp: wait until this CTA's accumulators are complete ----
        if (have_acc) {
            const long long w0 = prof ? clock64() : 0;
            ok = tc::mbar_wait(BAR_ACC, acc_phase, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 200) && ok;
            tc::tcgen05_fence_after();
            if (prof && tid == 128 && pass == 0) prof[12] = clock64() - w0;
        }
        if (prof && tid == 128 && pass == 0) { prof[1] = clock64() - t_setup; prof[6] = n_cs; }
        const uint32_t n_gran = n_cs * gpa;                          // granules of this pass, numbered ci * gpa + j0 / 16
        const uint32_t n_own_max = (n_gran + ksn - 1u) / ksn;        // granules a CTA owns at most
        if (ksn > 1u) {
            // ---- exchange of the partial sums: granule g belongs to CTA g mod ksplit ----
            tc::tcgen05_fence_before();
            tc::cluster_sync_all();                                  // every CTA of the cluster has drained its ring
            tc::tcgen05_fence_after();
            if (__all_sync(0xFFFFFFFFu, ok && *abort_flag == 0u)) {
                for (uint32_t g = half; g < n_gran; g += 2) {        // (warp-uniform)
                    const uint32_t owner = g % ksn;
                    const uint32_t ci = g / gpa, j0 = (g - ci * gpa) * 16;
                    if (owner == kz || j0 >= crank[ci]) continue;
                    uint32_t v[16];
                    load_granule(ci, j0, v);
                    // receive area of the owner: [source (this CTA's place among the owner's peers)][owned granule][row][16 floats]
                    const uint32_t src = kz < owner ? kz : kz - 1u;
                    const uint32_t dst = tc::map_to_cta(ring + ((src * n_own_max + g / ksn) * SHT_ROWS + row) * 64u, owner);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 16u * e), "r"(v[4 * e]), "r"(v[4 * e + 1]),
                                     "r"(v[4 * e + 2]), "r"(v[4 * e + 3]) : "memory");
                }
            }
            tc::tcgen05_fence_before();
            tc::cluster_sync_all();                                  // all partial sums have arrived
            tc::tcgen05_fence_after();
        }

        // ================================ epilogue: lane = row, this CTA's granules ================================
        if (__all_sync(0xFFFFFFFFu, ok && *abort_flag == 0u)) {
            uint32_t n_mine = 0;                                     // owned granules so far: the two warps of a quadrant alternate
            for (uint32_t g = kz; g < n_gran; g += ksn, ++n_mine) {
                if ((n_mine & 1u) != half) continue;
                const uint32_t ci = g / gpa, j0 = (g - ci * gpa) * 16;
                const uint32_t sl = cslot[ci], rank = crank[ci];
                if (j0 >= rank && p.tile_out) continue;              // padding ranks have no block
                float acc[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
                if (j0 < rank) {
                    uint32_t v[16];
                    load_granule(ci, j0, v);
                    // the cluster's partial sums in CTA order, this CTA's own in its place
                    for (uint32_t z = 0; z < ksn; ++z) {
                        if (z == kz) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) acc[e] = (z == 0u) ? __uint_as_float(v[e]) : acc[e] + __uint_as_float(v[e]);
                        } else {
                            const uint32_t src = z < kz ? z : z - 1u;
                            const float4* rp = reinterpret_cast<const float4*>(ring_gen + ((src * n_own_max + g / ksn) * SHT_ROWS + row) * 64u);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float4 r4 = rp[e];
                                if (z == 0u) { acc[4 * e] = r4.x; acc[4 * e + 1] = r4.y; acc[4 * e + 2] = r4.z; acc[4 * e + 3] = r4.w; }
                                else { acc[4 * e] += r4.x; acc[4 * e + 1] += r4.y; acc[4 * e + 2] += r4.z; acc[4 * e + 3] += r4.w; }
                            }
                        }
                    }
                }
                if (!row_live) continue;
                const float f = cscale[ci];
                const bool mine = my_slot == int32_t(sl);
                uint32_t w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float a = (mine && j0 + 2 * u < rank) ? acc[2 * u] * f : 0.0f;
                    const float b = (mine && j0 + 2 * u + 1 < rank) ? acc[2 * u + 1] * f : 0.0f;
                    w[u] = pack_bf16x2(a, b);
                }
                if (p.tile_out) {
                    const uint32_t q = uint32_t(cq0[tl][ci]) + j0 / 16;
                    if (q >= p.tile_cap) { record_status(STATUS_TILE_CAPACITY); continue; }
                    store_block_row(row_at + q * q_step, swap, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
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
            // blocks of adapters that occur in the row's token tile but not in this CTA's rows: this row is all zeros there
            // (written by the cluster's first CTA; the two warps of a quadrant take alternate adapters)
            if (pass == 0 && kz == 0 && p.tile_out && row_live) {
                uint32_t n_seen = 0;
                for (uint32_t wd = 0; wd < n_words; ++wd) {
                    uint32_t bits = present_t[tl][wd] & ~present_c[wd];
                    for (; bits; bits &= bits - 1, ++n_seen) {
                        if ((n_seen & 1u) != half) continue;
                        const uint32_t sl = wd * 32 + (__ffs(bits) - 1);
                        const uint32_t q0 = granules_ahead(tl, sl), n_gr = (rank_of(sl) + 15u) / 16u;
                        for (uint32_t k = 0; k < n_gr && q0 + k < p.tile_cap; ++k)
                            store_block_row(row_at + (q0 + k) * q_step, swap, make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u));
                    }
                }
            }
        }
        tc::tcgen05_fence_before();
        if (prof && pass == 0) {
            if (tid == 0) { prof[3] = t_wait; prof[8] = t_a; }
            if (tid == 128) { prof[4] = t_wait; prof[9] = t_a; prof[10] = t_b; }
        }
        if (have_acc) acc_phase ^= 1u;
        // Every MMA of the pass has completed and every thread is done with the receive area: the ring is free again —
        // cluster-wide, because the next pass's exchange writes into the peers' rings; the receive area was written and
        // read through the generic proxy and is written by TMA next.
        tc::fence_proxy_async();
        if (ksn > 1u) tc::cluster_sync_all(); else __syncthreads();
        if (n_cs < per_pass) break;                      // no adapters left for another pass (uniform over the cluster)
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
