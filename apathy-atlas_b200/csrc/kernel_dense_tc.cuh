// Dense-BF16 base linear on the tcgen05 tensor cores:  y[m, f] = bf16( sum_k x[m,k] * w[f,k] ),  w [N, K] BF16.
//
// The reference routes a dense (unquantised) weight through its BF16 GEMV / GEMM
// (crates/spark-model/src/layers/ops/quant_dispatch.rs:47,83; kernels/gb10/common/dense_gemv_bf16.cu:33-107).  Here it is
// the same orientation as the NVFP4 kernel — 128 output features in the MMA's M (TMEM lanes), a tile of MT tokens in its
// N — with both operands K-major tiles that TMA drops into shared memory (128-byte swizzle) and the MMA reads in place
// (kind::f16, both operands from shared memory); nothing is expanded, no warp touches the operands.
//
// A decode batch has few output tiles (N / 128) and is bound by streaming w: `ks` CTAs along grid z form a cluster and
// each contracts a share of K, so that every SM pulls weights; their FP32 partial tiles are added by the cluster's
// first CTA over distributed shared memory, in rank order (results do not depend on timing).
//
// Roles (6 warps): warp 0 TMA producer · warp 1 TMEM allocation and MMA issue · warps 2-5 epilogue (one per TMEM lane
// quadrant).  Every wait is bounded as in kernel_tc.cuh.
#pragma once

#include "kernel_tc.cuh"

namespace atlas {
namespace tc {

constexpr int D_THREADS = 192;
constexpr int D_W_BYTES = FT * KB * 2;                // one weight stage: [128 features x 64 k] BF16

template <int MT> struct DCfg {
    static constexpr int X_BYTES = MT * KB * 2;
    static constexpr int STAGE_BYTES = D_W_BYTES + ((X_BYTES + 1023) / 1024) * 1024;
    static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
    static constexpr int TMEM_COLS = MT < 32 ? 32 : MT;
    static constexpr int PARTIAL_BYTES = FT * MT * 4;                  // this CTA's FP32 tile, for the split-K reduction
    static constexpr int OFF_BAR = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + (2 * STAGES + 1) * 8 + 64 + 1024;
    static_assert(PARTIAL_BYTES <= STAGES * STAGE_BYTES, "the partial tile re-uses the stage memory");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct DParams {
    uint16_t* y;
    uint32_t M, N, K, out_row_stride, k_split;
};

template <int MT>
__global__ void __launch_bounds__(D_THREADS, 1)
dense_bf16_linear_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const DParams p) {
    using C = DCfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    const uint32_t BAR_FULL = bar0, BAR_EMPTY = bar0 + 8 * C::STAGES, BAR_ACC = bar0 + 16 * C::STAGES;
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + C::OFF_BAR + (2 * C::STAGES + 1) * 8);
    volatile uint32_t* abort_flag = misc + 2;           // misc[0] = TMEM base

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t f0 = blockIdx.x * FT, m0 = blockIdx.y * MT;
    const uint32_t ks = p.k_split, kz = blockIdx.z;
    const uint32_t total_kb = p.K / KB;
    const uint32_t kb_lo = kz * total_kb / ks, kb_hi = (kz + 1u) * total_kb / ks;
    const uint32_t num_kb = kb_hi - kb_lo;

    if (tid == 0) {
        for (int i = 0; i < C::STAGES; ++i) { mbar_init(BAR_FULL + 8 * i, 1); mbar_init(BAR_EMPTY + 8 * i, 1); }
        mbar_init(BAR_ACC, 1);
        misc[2] = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) { tmem_alloc(smem_base + C::OFF_BAR + (2 * C::STAGES + 1) * 8, C::TMEM_COLS); tmem_relinquish(); }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_acc = misc[0];
    bool acc_ready = false;

    if (warp == 0 && lane == 0) {
        uint32_t s = 0, ph = 0;
        for (uint32_t it = 0; it < num_kb; ++it) {
            if (!mbar_wait(BAR_EMPTY + 8 * s, ph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 20)) break;
            const uint32_t st = smem_base + s * C::STAGE_BYTES;
            mbar_arrive_expect_tx(BAR_FULL + 8 * s, D_W_BYTES + C::X_BYTES);
            tma_load_2d(st, &map_w, int32_t((kb_lo + it) * KB), int32_t(f0), BAR_FULL + 8 * s);
            tma_load_2d(st + D_W_BYTES, &map_x, int32_t((kb_lo + it) * KB), int32_t(m0), BAR_FULL + 8 * s);
            if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = make_idesc_bf16(MT, 128u);
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t it = 0; it < num_kb; ++it) {
            ok = mbar_wait(BAR_FULL + 8 * s, ph, abort_flag, STATUS_WAIT_EXPIRED_MMA, 20);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t st = smem_base + s * C::STAGE_BYTES;
            const uint64_t wd = make_kmajor_sw128_desc(st), xd = make_kmajor_sw128_desc(st + D_W_BYTES);
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) umma_bf16_ss<false>(tmem_acc, wd + 2 * j, xd + 2 * j, idesc, (it | j) ? 1u : 0u);
            umma_commit<false>(BAR_EMPTY + 8 * s);
            if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit<false>(BAR_ACC);
    } else if (warp >= 2) {
        // ---- epilogue: lane = feature, TMEM column = token ----
        const uint32_t q = warp & 3u;
        const uint32_t f = f0 + q * 32 + lane;
        if (num_kb == 0 || mbar_wait(BAR_ACC, 0, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 200)) {
            tcgen05_fence_after();
            acc_ready = true;
            for (uint32_t c0 = 0; c0 < uint32_t(MT); c0 += 16) {
                uint32_t v[16];
                if (num_kb) { tmem_ld16(tmem_acc + ((q * 32u) << 16) + c0, v); tmem_ld_wait(); }
                else { for (int i = 0; i < 16; ++i) v[i] = 0u; }
                if (ks == 1) {
                    if (f < p.N) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t m = m0 + c0 + i;
                            if (m < p.M) p.y[size_t(m) * p.out_row_stride + f] = f32_to_bf16_bits(__uint_as_float(v[i]));
                        }
                    }
                } else {
                    // the partial tile [token][128 features] FP32 into this CTA's shared memory (the stages are drained)
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(smem_base + ((c0 + i) * FT + q * 32 + lane) * 4u), "r"(v[i]) : "memory");
                }
            }
        }
    }
    if (ks > 1) {
        tcgen05_fence_before();
        __syncwarp();
        cluster_sync_all();                              // every CTA's partial tile is in its shared memory
        if (kz == 0 && warp >= 2 && acc_ready) {
            const uint32_t te = tid - 64;                // 0..127 = feature within the tile
            const uint32_t f = f0 + te;
            for (uint32_t i = 0; i < uint32_t(MT); ++i) {
                const uint32_t m = m0 + i;
                if (m >= p.M || f >= p.N) continue;
                float acc = 0.0f;
                for (uint32_t z = 0; z < ks; ++z) {
                    uint32_t bits;
                    asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(bits) : "r"(map_to_cta(smem_base + (i * FT + te) * 4u, z)) : "memory");
                    acc += __uint_as_float(bits);
                }
                p.y[size_t(m) * p.out_row_stride + f] = f32_to_bf16_bits(acc);
            }
        }
        __syncwarp();
        cluster_sync_all();                              // the tiles stay alive until they have been read
    }
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_acc, C::TMEM_COLS);
    }
}

}  // namespace tc
}  // namespace atlas
