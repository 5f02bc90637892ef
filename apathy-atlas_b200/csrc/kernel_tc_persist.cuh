// Persistent form of the fused NVFP4 + multi-LoRA linear for shapes with many output tiles (prefill batches).
//
// Same arithmetic, operand layouts and accumulation order as nvfp4_lora_linear_tc_kernel (kernel_tc.cuh), so the
// two produce identical bits; what changes is the schedule.  The grid is one cluster of two CTAs per pair of
// SMs, and every pair walks a static list of output tiles (tile t = pair, pair + pairs, ...; consecutive tiles
// share their tokens, so the CTAs running at one moment read the same activation rows out of L2):
//
//   * barriers, tensor memory and tensor-map prefetch are set up once per CTA, not once per tile;
//   * the operand rings (activation tiles, raw weight stages, the expanded weight operand in tensor memory)
//     run straight across tile boundaries: while tile i's last K blocks are multiplied, tile i+1's first
//     stages are already fetched and expanded;
//   * the LoRA K-steps have their own ring of (B_s tile, masked-t tile) stages, fetched by their own producer
//     thread while the base K loop runs, so they are issued back to back after the last base block;
//   * the epilogue is split: four warps first move the accumulator out of tensor memory into a shared-memory
//     tile (BF16, [token][128 features]) and hand the accumulator back to the MMA thread, and only then write
//     the rows to global memory (to every destination buffer), under the next tile's K loop.  The tensor pipe
//     idles only while the accumulator is being drained.
//
// A pass may cover G token tiles of MT tokens at once (G accumulators side by side in tensor memory): every
// expanded weight stage is then multiplied with G activation tiles before it is released, which divides the
// expansion work per multiply-add by G.  (G = 1 and 2 are instantiated; the accumulators of a pass complete
// together and are drained one after the other.)
//
// The shared-memory tile the accumulators are drained into and the LoRA operand ring occupy the SAME bytes:
// the ring is in use from the moment the tile's granule list exists until its last LoRA MMA has completed, the
// drain tile from then until its rows have left, and the next list is only published after that.
//
// Needs: CTA pairs, no K split, 16-byte aligned destination rows, and LoRA operands that both arrive by TMA
// (strided adapter pool + masked-t tiles written by the shrink).  The launcher falls back to the one-tile-per-CTA
// kernel otherwise.
//
// Warp roles (19 warps, 608 threads):
//   warp 0        TMA producer of the base K loop
//   warp 1        TMEM allocation, tcgen05.mma issue (first CTA of the pair issues for both)
//   warps 2-5     accumulator drain; row stores; granule list of the next tile
//   warps 6-13    A16: NVFP4 -> BF16 weight operand into tensor memory; A4: block scales into tensor memory
//   warp 14       TMA producer of the LoRA operand ring
//   warps 15-18   accumulator drain and row stores, with warps 2-5 (two warps per tensor-memory lane quadrant)
// Every wait is bounded as in kernel_tc.cuh; on expiry all roles fall through to the common teardown.
#pragma once

#include "kernel_tc.cuh"

namespace atlas {
namespace tc {

constexpr int P_NUM_THREADS = 32 * 19;
constexpr int P_LORA_WARP = 14;
constexpr int P_EPI_WARP1 = 15;         // second group of four drain / store warps (the first is warps 2-5)
constexpr int P_EPI_WARPS = 8;
constexpr int P_EPI_THREADS = 32 * P_EPI_WARPS;

template <int MT, int G, bool A4> struct PCfg {
    static_assert(MT % 64 == 0 && MT >= 128 && MT <= 256, "token tile of a pass");
    static_assert(!A4 || G == 1, "FP4 activations: one token tile per pass");
    static constexpr int XROWS = MT / 2;                                   // token rows of a tile this CTA stages
    static constexpr int X_TILE_BYTES = XROWS * KB * 2;
    static constexpr int X_STAGE_BYTES = G * X_TILE_BYTES;
    static constexpr int S4_W = 0;
    static constexpr int S4_X = S4_W + RAW_PACKED_BYTES;
    static constexpr int S4_WS = S4_X + XROWS * 128;
    static constexpr int S4_XS = S4_WS + RAW_SCALE_BYTES;
    static constexpr int S4_BYTES = ((S4_XS + MT * 16) + 1023) / 1024 * 1024;
    static constexpr int A_COLS = KB / 2;
    static constexpr int XSF_BLOCKS = MT > 128 ? MT / 128 : 1;
    static constexpr int SF_COLS = 16 + 16 * XSF_BLOCKS;
    static constexpr int ACC_COLS = G * MT;
    // the drain tile: every accumulator of the pass as [token][128 features] BF16; also the LoRA operand ring
    static constexpr int EPI_BYTES = G * MT * 256;
    static constexpr int L_GRAN_A = FT * 32;                               // B_s granule [128 x 16] BF16, SWIZZLE_32B
    static constexpr int L_GRAN_T = XROWS * 32;                            // masked-t granule [XROWS x 16] BF16
    static constexpr int L_STAGE = L_GRAN_A + L_GRAN_T;
    static constexpr int L_STAGES = EPI_BYTES / L_STAGE > 16 ? 16 : EPI_BYTES / L_STAGE;
    // ring depths: what the 227 KB of shared memory and the 512 columns of tensor memory leave
    static constexpr int STAGES = A4 ? 4 : (G == 1 ? 6 : 3);
    static constexpr int RAW_STAGES = A4 ? STAGES : (G == 1 ? 3 : 2);
    static constexpr int TMEM_A_BASE = ACC_COLS;
    static constexpr int TMEM_NEEDED = TMEM_A_BASE + (A4 ? STAGES * SF_COLS : STAGES * A_COLS);
    static constexpr int TMEM_COLS = 512;
    static constexpr int MAX_GRANULES = MT * (MAX_RANK_TC / 16);
    static constexpr int OFF_X = 0;
    static constexpr int OFF_RAWP = OFF_X + STAGES * X_STAGE_BYTES;
    static constexpr int OFF_RAWS = OFF_RAWP + RAW_STAGES * RAW_PACKED_BYTES;
    static constexpr int OFF_EPI = A4 ? STAGES * S4_BYTES : OFF_RAWS + RAW_STAGES * RAW_SCALE_BYTES;
    static constexpr int OFF_SLOT = OFF_EPI + EPI_BYTES;                          // int32[MT]  (scratch of the list build)
    static constexpr int OFF_GRAN = OFF_SLOT + MT * 4;                            // uint16[G][MAX_GRANULES]
    static constexpr int OFF_BITMAP = OFF_GRAN + G * MAX_GRANULES * 2;            // uint32[128]
    static constexpr int OFF_SCAN = OFF_BITMAP + (MAX_LORAS_TC / 32) * 4;         // uint32[8]
    static constexpr int OFF_GCOUNT = OFF_SCAN + 64;                              // uint8[MAX_LORAS_TC]: granules per slot, 0 = slot not usable
    static constexpr int OFF_BAR = OFF_GCOUNT + MAX_LORAS_TC;
    static constexpr int NUM_BARS = 2 * STAGES + 2 * RAW_STAGES + 2 * L_STAGES + 2 * G + 2;
    static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;                       // tmem ptr, abort, n_gran[G]
    static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
    static_assert(OFF_EPI % 1024 == 0, "drain tile / LoRA ring alignment");
    static_assert(L_STAGE % 256 == 0, "LoRA ring stages keep the 32-byte swizzle atom aligned");
    static_assert(TMEM_NEEDED <= 512, "tensor memory budget");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

// additional launch constants of the persistent form (the rest is tc::Params)
struct PParams {
    uint32_t n_fpairs;       // pairs of feature tiles along N
    uint32_t n_passes;       // token passes (G tiles of MT tokens each) along M
    uint32_t n_tiles;        // n_fpairs * n_passes
};

template <int MT, int G, bool A4>
__global__ void __launch_bounds__(P_NUM_THREADS, 1)
nvfp4_lora_linear_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_x,
                                       const __grid_constant__ CUtensorMap map_w,
                                       const __grid_constant__ CUtensorMap map_s,
                                       const __grid_constant__ CUtensorMap map_b,
                                       const __grid_constant__ CUtensorMap map_xs,
                                       const __grid_constant__ CUtensorMap map_t,
                                       const Params p, const PParams pp) {
    using C = PCfg<MT, G, A4>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t x_tile0 = smem_base + C::OFF_X;
    const uint32_t rawp0 = smem_base + C::OFF_RAWP;
    const uint32_t raws0 = smem_base + C::OFF_RAWS;
    const uint32_t epi0 = smem_base + C::OFF_EPI;
    int32_t* slot_arr = reinterpret_cast<int32_t*>(smem_gen + C::OFF_SLOT);
    uint16_t* gran = reinterpret_cast<uint16_t*>(smem_gen + C::OFF_GRAN);
    uint32_t* bitmap = reinterpret_cast<uint32_t*>(smem_gen + C::OFF_BITMAP);
    uint32_t* scan = reinterpret_cast<uint32_t*>(smem_gen + C::OFF_SCAN);
    uint8_t* gcount = smem_gen + C::OFF_GCOUNT;
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    const uint32_t BAR_FULL = bar0;                                     // [STAGES]   operands of a K block -> MMA (first CTA)
    const uint32_t BAR_EMPTY = BAR_FULL + 8 * C::STAGES;                // [STAGES]   MMA -> producers
    const uint32_t BAR_FULL_RAW = BAR_EMPTY + 8 * C::STAGES;            // [RAW_STAGES]
    const uint32_t BAR_EMPTY_RAW = BAR_FULL_RAW + 8 * C::RAW_STAGES;    // [RAW_STAGES]
    const uint32_t BAR_LFULL = BAR_EMPTY_RAW + 8 * C::RAW_STAGES;       // [L_STAGES] LoRA granule operands -> MMA (first CTA)
    const uint32_t BAR_LEMPTY = BAR_LFULL + 8 * C::L_STAGES;            // [L_STAGES]
    const uint32_t BAR_ACC_FULL = BAR_LEMPTY + 8 * C::L_STAGES;         // [G] accumulator complete -> drain
    const uint32_t BAR_ACC_EMPTY = BAR_ACC_FULL + 8 * G;                // [G] accumulator drained -> MMA (first CTA)
    const uint32_t BAR_LIST = BAR_ACC_EMPTY + 8 * G;                    // granule lists of the current pass are published
    const uint32_t BAR_EPI = BAR_LIST + 8;                              // the four drain warps meet here
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + C::OFF_MISC);
    // misc[0] = TMEM base, misc[2] = abort flag, misc[4 + g] = granule count of tile g of the current pass
    volatile uint32_t* abort_flag = misc + 2;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t cta_rank = blockIdx.x & 1u;
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const bool leader = cta_rank == 0u;
    constexpr uint32_t pair_mask = 3u;
    const uint32_t num_kb = A4 ? p.K / KRAW : p.K / KB;                 // pipeline steps of one tile's base K loop
    const uint32_t num_raw = A4 ? num_kb : num_kb / 4u;
    const uint32_t my_tiles = pp.n_tiles > pair ? (pp.n_tiles - pair + n_pairs - 1u) / n_pairs : 0u;
    const bool prof = p.profile != nullptr;
    const long long t_entry = clock64();
    unsigned long long* prof_row = prof ? p.profile + size_t(blockIdx.x) * PROFILE_WORDS : nullptr;

    if (tid == 0) {
        for (int i = 0; i < C::STAGES; ++i) {
            mbar_init(BAR_FULL + 8 * i, 2 * (A4 ? DEQ_GROUP_WARPS / 2 : DEQ_GROUP_WARPS) + 1);
            mbar_init(BAR_EMPTY + 8 * i, 1);
        }
        for (int i = 0; i < C::RAW_STAGES; ++i) {
            mbar_init(BAR_FULL_RAW + 8 * i, 1);
            mbar_init(BAR_EMPTY_RAW + 8 * i, DEQ_WARPS);
        }
        for (int i = 0; i < C::L_STAGES; ++i) {
            mbar_init(BAR_LFULL + 8 * i, 1);
            mbar_init(BAR_LEMPTY + 8 * i, 1);
        }
        for (int g = 0; g < G; ++g) {
            mbar_init(BAR_ACC_FULL + 8 * g, 1);
            mbar_init(BAR_ACC_EMPTY + 8 * g, 2);                         // one arrival per CTA of the pair
        }
        mbar_init(BAR_LIST, 1);
        mbar_init(BAR_EPI, P_EPI_WARPS);
        misc[2] = 0;
        for (int g = 0; g < G; ++g) misc[4 + g] = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc_pair(smem_base + C::OFF_MISC, C::TMEM_COLS); tmem_relinquish_pair(); }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_s);
        if (A4) tma_prefetch_desc(&map_xs);
    }
    if (warp == P_LORA_WARP && lane == 0 && p.seq_slot) {
        tma_prefetch_desc(&map_b);
        tma_prefetch_desc(&map_t);
    }
    if (p.seq_slot) {
        // granules (16 ranks each) every slot contributes to a tile it occurs in; 0 for a slot without both tables' entries
        for (uint32_t sl = tid; sl < p.max_loras; sl += P_NUM_THREADS) {
            const bool usable = p.a_table[sl] != 0ull && p.b_table[sl] != 0ull;
            const uint32_t r = p.rank_table ? min(p.rank_table[sl], p.max_rank) : p.max_rank;
            gcount[sl] = usable ? uint8_t((r + 15u) / 16u) : uint8_t(0);
        }
    }
    tcgen05_fence_before();
    __syncwarp();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t full_at_leader = map_to_cta(BAR_FULL, 0);
    const uint32_t lfull_at_leader = map_to_cta(BAR_LFULL, 0);
    const uint32_t acc_empty_at_leader = map_to_cta(BAR_ACC_EMPTY, 0);
    const uint32_t tmem_acc = misc[0];
    const uint32_t tmem_a0 = tmem_acc + C::TMEM_A_BASE;

    // tile t of this pair: feature pair (fastest) and token pass
    auto tile_fpair = [&](uint32_t i) { return (pair + i * n_pairs) % pp.n_fpairs; };
    auto tile_pass = [&](uint32_t i) { return (pair + i * n_pairs) / pp.n_fpairs; };

    if (warp == 0) {
        // ===================================== TMA producer, base K loop =====================================
        if (lane == 0 && A4) {
            uint32_t s = 0, ph = 0;
            for (uint32_t i = 0; i < my_tiles; ++i) {
                const uint32_t f0 = (tile_fpair(i) * 2u + cta_rank) * FT, m0 = tile_pass(i) * MT;
                const uint32_t rot = tile_fpair(i) % num_kb;
                bool ok = true;
                for (uint32_t it = 0; it < num_kb; ++it) {
                    ok = mbar_wait(BAR_EMPTY + 8 * s, ph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 32);
                    if (!ok) break;
                    const uint32_t st = smem_base + s * C::S4_BYTES;
                    const uint32_t kk = (it + rot) % num_kb;
                    mbar_arrive_expect_tx(BAR_FULL_RAW + 8 * s, RAW_SCALE_BYTES + MT * 16);
                    tma_load_2d(st + C::S4_WS, &map_s, int32_t(kk * (KRAW / 16)), int32_t(f0), BAR_FULL_RAW + 8 * s);
                    tma_load_2d(st + C::S4_XS, &map_xs, int32_t(kk * (KRAW / 16)), int32_t(m0), BAR_FULL_RAW + 8 * s);
                    if (leader) mbar_arrive_expect_tx(BAR_FULL + 8 * s, 2 * (RAW_PACKED_BYTES + C::XROWS * 128));
                    tma_load_2d_pair(st + C::S4_W, &map_w, int32_t(kk * (KRAW / 2)), int32_t(f0), full_at_leader + 8 * s);
                    tma_load_2d_pair(st + C::S4_X, &map_x, int32_t(kk * (KRAW / 2)), int32_t(m0 + cta_rank * C::XROWS), full_at_leader + 8 * s);
                    if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
            }
        }
        if (lane == 0 && !A4) {
            // two rings fed by one thread without blocking on either: activation tiles (one stage per K block, G
            // tiles each) and raw weight stages (codes + scale bytes, one per four K blocks)
            uint32_t xs = 0, xph = 0, rs = 0, rph = 0, spins = 0;
            uint64_t t0 = 0;
            bool dead = false;
            for (uint32_t i = 0; i < my_tiles && !dead; ++i) {
                const uint32_t f0 = (tile_fpair(i) * 2u + cta_rank) * FT, m0 = tile_pass(i) * (MT * G);
                const uint32_t rot_raw = tile_fpair(i) % num_raw;
                uint32_t it = 0, ri = 0;
                while (it < num_kb || ri < num_raw) {
                    bool progressed = false;
                    if (ri < num_raw && mbar_try_wait(BAR_EMPTY_RAW + 8 * rs, rph ^ 1u)) {
                        mbar_arrive_expect_tx(BAR_FULL_RAW + 8 * rs, RAW_PACKED_BYTES + RAW_SCALE_BYTES);
                        const uint32_t rk = (ri + rot_raw) % num_raw;
                        tma_load_2d(rawp0 + rs * RAW_PACKED_BYTES, &map_w, int32_t(rk * (KRAW / 2)), int32_t(f0), BAR_FULL_RAW + 8 * rs);
                        tma_load_2d(raws0 + rs * RAW_SCALE_BYTES, &map_s, int32_t(rk * (KRAW / 16)), int32_t(f0), BAR_FULL_RAW + 8 * rs);
                        ++ri;
                        if (++rs == uint32_t(C::RAW_STAGES)) { rs = 0; rph ^= 1u; }
                        progressed = true;
                    }
                    if (it < num_kb && mbar_try_wait(BAR_EMPTY + 8 * xs, xph ^ 1u)) {
                        if (leader) mbar_arrive_expect_tx(BAR_FULL + 8 * xs, 2 * C::X_STAGE_BYTES);
                        const uint32_t kb = (it + 4u * rot_raw) % num_kb;
#pragma unroll
                        for (uint32_t g = 0; g < uint32_t(G); ++g)
                            tma_load_2d_pair(x_tile0 + xs * C::X_STAGE_BYTES + g * C::X_TILE_BYTES, &map_x, int32_t(kb * KB),
                                             int32_t(m0 + g * MT + cta_rank * C::XROWS), full_at_leader + 8 * xs);
                        ++it;
                        if (++xs == uint32_t(C::STAGES)) { xs = 0; xph ^= 1u; }
                        progressed = true;
                    }
                    if (progressed) {
                        spins = 0;
                        t0 = 0;
                    } else {
                        __nanosleep(64);
                        if ((++spins & 63u) != 0u) continue;
                        if (*abort_flag) { dead = true; break; }
                        const uint64_t now = global_timer_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > WAIT_LIMIT_NS) {
                            record_status(STATUS_WAIT_EXPIRED_PRODUCER);
                            *abort_flag = 1u;
                            dead = true;
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == P_LORA_WARP) {
        // ===================================== TMA producer, LoRA operand ring ===============================
        if (lane == 0 && p.seq_slot) {
            uint32_t ls = 0, lph = 0;
            bool ok = true, waited_for_shrink = false;
            for (uint32_t i = 0; ok && i < my_tiles; ++i) {
                ok = mbar_wait(BAR_LIST, i & 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 64);
                if (!ok) break;
                const uint32_t f0 = (tile_fpair(i) * 2u + cta_rank) * FT;
                for (uint32_t g = 0; ok && g < uint32_t(G); ++g) {
                    const uint32_t n_gran = misc[4 + g];
                    if (n_gran && !waited_for_shrink) {
                        // the masked-t tiles are the shrink grid's output: it must be complete before the first fetch
                        if (p.wait_for_shrink) asm volatile("griddepcontrol.wait;" ::: "memory");
                        waited_for_shrink = true;
                    }
                    const uint32_t t_row0 = ((tile_pass(i) * G + g) * 2u + cta_rank) * p.t_tile_cap * uint32_t(C::L_GRAN_T / 256);
                    for (uint32_t q = 0; q < n_gran; ++q) {
                        ok = mbar_wait(BAR_LEMPTY + 8 * ls, lph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 32);
                        if (!ok) break;
                        const uint32_t base = epi0 + ls * C::L_STAGE;
                        const uint32_t e = gran[g * C::MAX_GRANULES + q];
                        if (leader) mbar_arrive_expect_tx(BAR_LFULL + 8 * ls, 2 * C::L_STAGE);
                        tma_load_3d_pair(base, &map_b, int32_t((e & 3u) * 16u), int32_t(f0), int32_t(e >> 2), lfull_at_leader + 8 * ls);
                        tma_load_2d_pair(base + C::L_GRAN_A, &map_t, 0, int32_t(t_row0 + q * uint32_t(C::L_GRAN_T / 256)), lfull_at_leader + 8 * ls);
                        if (++ls == uint32_t(C::L_STAGES)) { ls = 0; lph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===================================== MMA issuer ====================================================
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_bf16(MT, 256u);
            unsigned long long w_full = 0, w_acc = 0, w_lora = 0, w_head = 0;
            const long long t_begin = prof ? clock64() : 0;
            bool ok = true;
            uint32_t s = 0, ph = 0, ls = 0, lph = 0;
            for (uint32_t i = 0; ok && i < my_tiles; ++i) {
                // the accumulators of the previous pass must have been drained
                for (uint32_t g = 0; ok && g < uint32_t(G); ++g)
                    ok = mbar_wait_timed(BAR_ACC_EMPTY + 8 * g, (i & 1u) ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_acc, MMA_BACKOFF_NS);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned long long w_full_at_pass = w_full;
                uint32_t acc = 0;
                if constexpr (A4) {
                    constexpr uint32_t idesc4 = make_idesc_nvfp4(MT, 256u);
                    for (uint32_t it = 0; it < num_kb; ++it) {
                        ok = mbar_wait_timed(BAR_FULL + 8 * s, ph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_full, MMA_BACKOFF_NS);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t st = smem_base + s * C::S4_BYTES, sf = tmem_a0 + s * C::SF_COLS;
                        const uint64_t wa = make_kmajor_sw128_desc(st + C::S4_W);
                        const uint64_t xb = make_kmajor_sw128_desc(st + C::S4_X);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
                            umma_nvfp4_ss<true>(tmem_acc, wa + 2 * j, xb + 2 * j, idesc4, sf + 4 * j, sf + 16 + 4 * C::XSF_BLOCKS * j, acc | j);
                        umma_commit<true>(BAR_EMPTY + 8 * s, pair_mask);
                        acc = 1u;
                        if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
                    }
                } else {
                    for (uint32_t it = 0; it < num_kb; ++it) {
                        if (prof && it == 4) w_head += w_full - w_full_at_pass;
                        ok = mbar_wait_timed(BAR_FULL + 8 * s, ph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_full, MMA_BACKOFF_NS);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t a_tmem = tmem_a0 + s * C::A_COLS;
#pragma unroll
                        for (uint32_t g = 0; g < uint32_t(G); ++g) {
                            const uint64_t b_desc = make_kmajor_sw128_desc(x_tile0 + s * C::X_STAGE_BYTES + g * C::X_TILE_BYTES);
#pragma unroll
                            for (uint32_t j = 0; j < 4; ++j)
                                umma_bf16_ts<true>(tmem_acc + g * MT, a_tmem + 8 * j, b_desc + 2 * j, idesc, acc | j);
                        }
                        umma_commit<true>(BAR_EMPTY + 8 * s, pair_mask);
                        acc = 1u;
                        if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
                    }
                }
                if (!ok) break;
                // LoRA K-steps: one 16-wide kind::f16 step per granule, operands from their own ring
                if (p.seq_slot) {
                    ok = mbar_wait_timed(BAR_LIST, i & 1u, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_lora, MMA_BACKOFF_NS);
                    if (!ok) break;
                }
                for (uint32_t g = 0; ok && g < uint32_t(G); ++g) {
                    const uint32_t n_gran = p.seq_slot ? misc[4 + g] : 0u;
                    for (uint32_t q = 0; q < n_gran; ++q) {
                        ok = mbar_wait_timed(BAR_LFULL + 8 * ls, lph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_lora, MMA_BACKOFF_NS);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint64_t la = make_kmajor_sw32_desc(epi0 + ls * C::L_STAGE);
                        const uint64_t lb = make_kmajor_sw32_desc(epi0 + ls * C::L_STAGE + C::L_GRAN_A);
                        umma_bf16_ss<true>(tmem_acc + g * MT, la, lb, idesc, 1u);
                        umma_commit<true>(BAR_LEMPTY + 8 * ls, pair_mask);
                        if (++ls == uint32_t(C::L_STAGES)) { ls = 0; lph ^= 1u; }
                    }
                    if (ok) umma_commit<true>(BAR_ACC_FULL + 8 * g, pair_mask);
                }
            }
            if (prof) {
                prof_row[0] = w_full; prof_row[2] = (unsigned long long)(clock64() - t_begin);
                prof_row[10] = w_acc; prof_row[11] = w_lora; prof_row[9] = w_head;
            }
        }
        __syncwarp();
    } else if (warp < DEQ_WARP0 || warp >= P_EPI_WARP1) {
        // ============================ accumulator drain, row stores, granule lists ===========================
        const uint32_t grp = warp < DEQ_WARP0 ? 0u : 1u;                            // which of the two groups of four warps
        const uint32_t te = ((warp < DEQ_WARP0 ? warp - EPI_WARP0 : warp - P_EPI_WARP1 + 4u) << 5) + lane;   // 0..255
        const uint32_t q = warp & 3u;                      // TMEM lane quadrant this warp may read
        uint32_t epi_phase = 0;
        bool ok = true;
        unsigned long long w_accfull = 0, c_drain = 0, c_store = 0, c_list = 0;
        // bounded rendezvous of the eight warps of this role
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_EPI);
            const bool r = mbar_wait(BAR_EPI, epi_phase, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE);
            epi_phase ^= 1u;
            return r;
        };
        // this thread's row of each token tile of pass `pass`: its slot if the row takes a LoRA term, else -1
        auto load_slots = [&](uint32_t pass, int32_t (&out)[G]) {
#pragma unroll
            for (uint32_t g = 0; g < uint32_t(G); ++g) {
                const uint32_t m = (pass * G + g) * MT + te;
                out[g] = (p.seq_slot && te < uint32_t(MT) && m < p.M) ? p.seq_slot[m] : -1;
            }
        };
        // lists of a pass from those slots: for each of its G token tiles the (slot, granule) pairs that occur, slots ascending
        auto build_lists = [&](const int32_t (&slots)[G]) -> bool {
            if (!p.seq_slot) return true;
            for (uint32_t g = 0; g < uint32_t(G); ++g) {
                if (te < 128u) bitmap[te] = 0;
                if (!epi_sync()) return false;
                int32_t sl = slots[g];
                if (sl >= 0) {
                    if (uint32_t(sl) >= p.max_loras) { record_status(STATUS_SLOT_OUT_OF_RANGE); sl = -1; }
                    else if (gcount[sl] == 0) sl = -1;
                }
                if (sl >= 0) atomicOr(&bitmap[uint32_t(sl) >> 5], 1u << (uint32_t(sl) & 31u));
                if (!epi_sync()) return false;
                uint32_t word = 0, cnt = 0, incl = 0;
                if (te < 128u) {                                  // (warps 2-5: one bitmap word = 32 slots per thread)
                    word = bitmap[te];
                    for (uint32_t w = word; w; w &= w - 1) cnt += gcount[te * 32 + (__ffs(w) - 1)];
                    incl = cnt;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                        if (lane >= uint32_t(o)) incl += v;
                    }
                    if (lane == 31) scan[te >> 5] = incl;
                }
                if (!epi_sync()) return false;
                if (te < 128u) {
                    uint32_t base = 0;
                    for (uint32_t w = 0; w < (te >> 5); ++w) base += scan[w];
                    uint32_t pos = base + incl - cnt;
                    for (uint32_t w = word; w; w &= w - 1) {
                        const uint32_t s2 = te * 32 + (__ffs(w) - 1);
                        for (uint32_t k = 0; k < gcount[s2]; ++k) gran[g * C::MAX_GRANULES + pos++] = uint16_t((s2 << 2) | k);
                    }
                    if (te == 0) misc[4 + g] = scan[0] + scan[1] + scan[2] + scan[3];
                }
            }
            return epi_sync();
        };
        (void)slot_arr;
        int32_t next_slots[G];
        if (my_tiles) {
            load_slots(tile_pass(0), next_slots);
            ok = build_lists(next_slots);
            if (ok && te == 0) mbar_arrive(BAR_LIST);
        }
        const float osc = p.out_scale;
        const bool odd = lane & 1u;
        const uint32_t fe = (q * 32u + lane) & ~1u;
        for (uint32_t i = 0; ok && i < my_tiles; ++i) {
            const uint32_t f0 = (tile_fpair(i) * 2u + cta_rank) * FT;
            // the next pass's routing entries travel while this pass's accumulators complete
            if (i + 1 < my_tiles) load_slots(tile_pass(i + 1), next_slots);
            // ---- drain: every accumulator of the pass -> BF16 [token][128 features] in shared memory ----
            for (uint32_t g = 0; ok && g < uint32_t(G); ++g) {
                const long long t_w = prof ? clock64() : 0;
                // all accumulators of a pass complete together; wait for the last one before the first drain, because
                // the drain tile overlays the LoRA operand ring that the later accumulators' K-steps still read
                if (g == 0) {
                    for (uint32_t g2 = 0; ok && g2 < uint32_t(G); ++g2)
                        ok = mbar_wait(BAR_ACC_FULL + 8 * g2, i & 1u, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 256);
                    if (!ok) break;
                }
                tcgen05_fence_after();
                const long long t_d = prof ? clock64() : 0;
                if (prof) w_accfull += (unsigned long long)(t_d - t_w);
                const uint32_t tile = epi0 + g * (MT * 256);
                // The two warps of a quadrant take alternate blocks of 32 token columns.  The next block's tensor-memory
                // loads are issued before the current block is converted and stored, so their latency is not exposed.
                constexpr uint32_t N_BLK = uint32_t(MT) / 64u;
                const uint32_t t_col0 = tmem_acc + ((q * 32u) << 16) + g * MT + grp * 32u;
                uint32_t v[2][2][16];
                tmem_ld16(t_col0, v[0][0]);
                tmem_ld16(t_col0 + 16, v[0][1]);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t blk = 0; blk < N_BLK; ++blk) {
                    const uint32_t cur = blk & 1u;
                    if (blk + 1 < N_BLK) {
                        tmem_ld16(t_col0 + 64 * (blk + 1), v[cur ^ 1u][0]);
                        tmem_ld16(t_col0 + 64 * (blk + 1) + 16, v[cur ^ 1u][1]);
                    }
                    const uint32_t c0 = grp * 32 + 64 * blk;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float a = __uint_as_float(v[cur][h][2 * u]) * osc, b = __uint_as_float(v[cur][h][2 * u + 1]) * osc;
                            const float got = __shfl_xor_sync(0xFFFFFFFFu, odd ? a : b, 1);
                            const uint32_t row = c0 + 16 * h + 2 * u + (odd ? 1u : 0u);
                            const uint32_t w = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);
                            const uint32_t chunk = (fe >> 3) ^ ((row & 1u) << 2);
                            asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + row * 256u + chunk * 16u + (fe & 7u) * 2u), "r"(w) : "memory");
                        }
                    if (blk + 1 < N_BLK) tmem_ld_wait();
                }
                tcgen05_fence_before();
                ok = epi_sync();                              // all of the accumulator is out of tensor memory and in the tile
                if (!ok) break;
                if (te == 0) mbar_arrive_cluster(acc_empty_at_leader + 8 * g);
                if (prof) c_drain += (unsigned long long)(clock64() - t_d);
            }
            if (!ok) break;
            // ---- rows out: 16 threads per row, one 16-byte chunk (8 features) each, to every destination ----
            const long long t_s = prof ? clock64() : 0;
            {
                const uint32_t j = te & 15u;
                const uint32_t f = f0 + j * 8u;
                if (f < p.N) {
                    const bool whole = f + 8u <= p.N;
                    const uint32_t m_base = tile_pass(i) * (MT * G);
                    for (uint32_t row = te >> 4; row < uint32_t(MT * G); row += P_EPI_THREADS >> 4) {
                        const uint32_t m = m_base + row;
                        if (m >= p.M) break;
                        const uint4 val = lds128(epi0 + row * 256u + ((j ^ ((row & 1u) << 2)) << 4));
                        const size_t at = size_t(m) * p.out_row_stride + p.y_col0 + f;
                        for (uint32_t r = 0; r < p.n_dest; ++r) {
                            uint16_t* dst = p.y_dest[r] + at;
                            if (whole) {
                                *reinterpret_cast<uint4*>(dst) = val;
                            } else {
                                const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                                for (uint32_t e = 0; f + e < p.N; ++e) dst[e] = uint16_t(w4[e >> 1] >> (16u * (e & 1u)));
                            }
                        }
                    }
                }
            }
            // the drain tile has been read; order these reads (and the drain's writes) before the TMA writes of the next
            // pass's LoRA operands, which overwrite it once the next list is published
            fence_proxy_async();
            ok = epi_sync();
            if (prof) c_store += (unsigned long long)(clock64() - t_s);
            if (!ok) break;
            if (i + 1 < my_tiles) {
                const long long t_l = prof ? clock64() : 0;
                ok = build_lists(next_slots);
                if (ok && te == 0) mbar_arrive(BAR_LIST);
                if (prof) c_list += (unsigned long long)(clock64() - t_l);
            }
        }
        if (prof && te == 0) { prof_row[7] = c_drain; prof_row[12] = c_store; prof_row[13] = c_list; prof_row[6] = w_accfull; }
    } else {
        // ========================== weight operand (A16) / block scales (A4) into tensor memory ==============
        const uint32_t q = warp & 3u;
        const uint32_t half = ((warp - DEQ_WARP0) >> 2) & 1u;
        const uint32_t row = q * 32 + lane;
        const uint32_t td = tid - DEQ_WARP0 * 32;
        const uint32_t lane_base = (q * 32u) << 16;
        bool ok = true;
        unsigned long long w_raw = 0, w_empty = 0;
        const long long t_begin = clock64();
        uint32_t s = 0, ph = 0, rs = 0, rph = 0;
        if constexpr (A4) {
            uint32_t itg = 0;                                 // K blocks since kernel start: the halves take alternate ones
            for (uint32_t i = 0; ok && i < my_tiles; ++i) {
                for (uint32_t it = 0; ok && it < num_kb; ++it, ++itg) {
                    if ((itg & 1u) != half) {
                        if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
                        continue;
                    }
                    ok = mbar_wait_timed(BAR_FULL_RAW + 8 * s, ph, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_raw);
                    if (!ok) break;
                    const uint32_t st = smem_base + s * C::S4_BYTES;
                    const uint32_t sf = tmem_a0 + lane_base + s * C::SF_COLS;
                    {
                        uint32_t r[16];
                        uint32_t neg = 0;
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            const uint4 v = lds128(st + C::S4_WS + (lane + 32 * c) * 16);
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u) {
                                const uint32_t nan = __vcmpeq4(w[u] & 0x7F7F7F7Fu, 0x7F7F7F7Fu);
                                neg |= w[u] & ~nan;
                                r[4 * u + c] = w[u] & ~nan & 0x7F7F7F7Fu;
                            }
                        }
                        if (neg & 0x80808080u) record_status(STATUS_NEGATIVE_SCALE);
                        tmem_st16(sf, r);
                    }
                    if constexpr (C::XSF_BLOCKS == 1) {
                        uint32_t r[16];
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            const uint32_t xr = lane + 32 * c;
                            uint4 v = make_uint4(0u, 0u, 0u, 0u);
                            if (xr < uint32_t(MT)) v = lds128(st + C::S4_XS + xr * 16);
                            r[c] = v.x; r[4 + c] = v.y; r[8 + c] = v.z; r[12 + c] = v.w;
                        }
                        tmem_st16(sf + 16, r);
                    } else {
                        uint32_t r0[16], r1[16];
#pragma unroll
                        for (uint32_t blk = 0; blk < 2; ++blk)
#pragma unroll
                            for (uint32_t c = 0; c < 4; ++c) {
                                const uint4 v = lds128(st + C::S4_XS + (128 * blk + 32 * c + lane) * 16);
                                r0[4 * blk + c] = v.x; r0[8 + 4 * blk + c] = v.y;
                                r1[4 * blk + c] = v.z; r1[8 + 4 * blk + c] = v.w;
                            }
                        tmem_st16(sf + 16, r0);
                        tmem_st16(sf + 32, r1);
                    }
                    tmem_st_wait();
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(full_at_leader + 8 * s);
                    if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
                }
            }
        } else {
            for (uint32_t i = 0; ok && i < my_tiles; ++i) {
                for (uint32_t ri = 0; ok && ri < num_raw; ++ri) {
                    ok = mbar_wait_timed(BAR_FULL_RAW + 8 * rs, rph, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_raw);
                    if (!ok) break;
                    const uint4 sc4 = lds128(raws0 + rs * RAW_SCALE_BYTES + row * 16);
                    const uint32_t scw[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
#pragma unroll
                    for (uint32_t jr = 0; jr < 4; jr += 2) {
                        uint32_t o[2][16];
#pragma unroll
                        for (uint32_t u = 0; u < 2; ++u) {
                            const uint32_t j = jr + u;
                            const uint4 pk = lds128(rawp0 + rs * RAW_PACKED_BYTES + sw128_off(row, 2 * j + half));
                            const uint32_t pw[4] = {pk.x, pk.y, pk.z, pk.w};
                            const uint32_t scj = j == 0 ? scw[0] : (j == 1 ? scw[1] : (j == 2 ? scw[2] : scw[3]));
                            const uint32_t sbytes = scj >> (16 * half);
                            const uint32_t mul0 = e4m3_to_bf16x2_shifted(sbytes & 0xFFu);
                            const uint32_t mul1 = e4m3_to_bf16x2_shifted((sbytes >> 8) & 0xFFu);
#pragma unroll
                            for (uint32_t qd = 0; qd < 4; ++qd) {
                                uint32_t o4[4];
                                e2m1x8_to_bf16x8(pw[qd], qd < 2 ? mul0 : mul1, o4);
                                o[u][4 * qd] = o4[0]; o[u][4 * qd + 1] = o4[1]; o[u][4 * qd + 2] = o4[2]; o[u][4 * qd + 3] = o4[3];
                            }
                        }
                        const uint32_t s0 = s, ph0 = ph;
                        uint32_t s1 = s0 + 1, ph1 = ph0;
                        if (s1 >= uint32_t(C::STAGES)) { s1 -= C::STAGES; ph1 ^= 1u; }
                        ok = mbar_wait_timed(BAR_EMPTY + 8 * s0, ph0 ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_empty);
                        if (!ok) break;
                        tcgen05_fence_after();
                        tmem_st16(tmem_a0 + lane_base + s0 * C::A_COLS + 16 * half, o[0]);
                        ok = mbar_wait_timed(BAR_EMPTY + 8 * s1, ph1 ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_empty);
                        if (!ok) break;
                        tcgen05_fence_after();
                        tmem_st16(tmem_a0 + lane_base + s1 * C::A_COLS + 16 * half, o[1]);
                        tmem_st_wait();
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive_cluster(full_at_leader + 8 * s0);
                            mbar_arrive_cluster(full_at_leader + 8 * s1);
                        }
                        s = s1 + 1; ph = ph1;
                        if (s >= uint32_t(C::STAGES)) { s -= C::STAGES; ph ^= 1u; }
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR_EMPTY_RAW + 8 * rs);
                    if (++rs == uint32_t(C::RAW_STAGES)) { rs = 0; rph ^= 1u; }
                }
            }
        }
        if (prof && td == 0) {
            prof_row[3] = w_raw; prof_row[4] = w_empty; prof_row[5] = (unsigned long long)(clock64() - t_begin);
        }
    }

    // ========================================= teardown ==========================================
    if (*abort_flag) {
        // give copies that may still be in flight time to land before shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncwarp();
    // (the other CTA's MMAs read this CTA's shared and tensor memory, and its warps arrive on this CTA's barriers)
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_acc, C::TMEM_COLS);
        if (prof && lane == 0) { prof_row[1] = (unsigned long long)(clock64() - t_entry); prof_row[8] = my_tiles; }
    }
}

}  // namespace tc
}  // namespace atlas
