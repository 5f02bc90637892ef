// The fused NVFP4 + multi-LoRA linear for sm_100a: TMA-staged tiles, tcgen05.mma into a TMEM accumulator,
// and the LoRA expand appended as extra K-steps of the same accumulator so y is written exactly once.
//
// Orientation ("swap-AB"): the MMA's M dimension (128 TMEM lanes per CTA) is a block of 128 OUTPUT
// FEATURES, its N dimension (TMEM columns) a tile of MT TOKENS, MT in {16..256}.  A decode batch
// of 16-64 tokens therefore still fills the 128-lane datapath, and a 256-token tile gives the
// 128 x 256 x 16 instruction shape.
//
//   acc[f, m]  = sum_k  W'[f,k] * x[m,k]                      base, A16: W' = E2M1*E4M3*2^-8 (exact BF16), kind::f16
//                                                             base, A4: E2M1 x E2M1 with E4M3 block scales of both
//                                                             sides in tensor memory, kind::mxf4nvf4.block_scale
//              + sum_g  B_{s_g}[f, j_g..j_g+16) * T_g[m, :]   LoRA: one 16-wide kind::f16 K-step per granule
//   y[m, f]    = bf16(acc[f,m] * scale2 [* 2^8])
//
// A granule g is 16 consecutive ranks of one adapter slot that occurs in the token tile; T_g[m,:]
// is row m of the pre-scaled shrink result t where seq_slot[m] equals the granule's slot and zero
// elsewhere, so adapters never mix across tokens.  Granules are ordered by slot, four to a K block;
// zeros add exactly, so a token's result does not depend on which other tokens share its tile.
// The masked tiles either arrive ready-made from the shrink kernel (Params::t_tile_cap) or are built
// here from t.
//
// Operand placement, A16: the weight operand (MMA "A", 128 features x 16 k per instruction) is written
// by the expansion warps straight into TENSOR MEMORY (tcgen05.st) and read from there by the MMA;
// only the activation operand lives in shared memory.  A4: both operands are the packed tiles in
// shared memory as TMA delivers them; the warps only carry scale bytes to tensor memory.
//
// Launch shapes: one CTA per tile; or pairs of CTAs (clusters of 2 along x) issuing cta_group::2 MMAs
// with half of the activation tile each (Cfg::PAIR); and, times that, k_split CTAs along z sharing one
// tile's contraction and exchanging partial sums over distributed shared memory.
//
// Warp roles (14 warps, 448 threads):
//   warp 0        TMA producer: activation tiles, raw weight stages (packed codes + scale bytes),
//                 LoRA operand tiles, each through its own mbarrier ring
//   warp 1        TMEM allocation, tcgen05.mma issue, tcgen05.commit (in a pair: the first CTA's thread
//                 issues for both)
//   warps 2-5     build the tile's granule list while the main loop runs; then the epilogue
//   warps 6-13    A16: expand raw NVFP4 into the BF16 weight operand (TMEM); A4: scale bytes -> TMEM;
//                 build the LoRA operands where the shrink has not; then join the epilogue:
//                 tcgen05.ld -> scale -> BF16 -> shared-memory tile -> 16-byte row stores
//
// Every mbarrier wait is bounded: on expiry the waiter records a status code, raises the CTA's abort
// flag, and all roles fall through to a common teardown that frees TMEM; cluster barriers are placed
// where every thread of every CTA passes on every path.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace atlas {
namespace tc {

constexpr int FT = 128;              // features per CTA = UMMA M
constexpr int KB = 64;               // K elements per MMA stage (one 128-byte swizzle row of BF16)
constexpr int KRAW = 256;            // K elements per raw weight stage
constexpr int RAW_PACKED_BYTES = FT * (KRAW / 2);    // 16 KiB
constexpr int RAW_SCALE_BYTES = FT * (KRAW / 16);    // 2 KiB
// Expansion warps come in groups of eight (one warp per TMEM quadrant and K half).  With G groups, group
// i expands K blocks i, i+G, ... of each raw stage.  One group measured best: a second group does not
// shorten the K loop (which is bound by shared-memory bandwidth at 256 tokens and by the MMA thread's
// issue rate below) and takes issue slots from the MMA thread.
constexpr int DEQ_GROUPS = 1;
constexpr int DEQ_WARP0 = 6, DEQ_GROUP_WARPS = 8, DEQ_WARPS = 8 * DEQ_GROUPS, DEQ_THREADS = 32 * DEQ_WARPS;
constexpr int NUM_THREADS = 32 * (DEQ_WARP0 + DEQ_WARPS);
constexpr int EPI_WARP0 = 2, EPI_THREADS = 128;
constexpr int EPI_WARPS = 4 + DEQ_WARPS;   // warps that take part in the epilogue: the list warps and the expansion warps
constexpr int MAX_LORAS_TC = 4096;
constexpr int MAX_RANK_TC = 64;
constexpr uint64_t WAIT_LIMIT_NS = 1000000000ull;    // 1 s
constexpr int PROFILE_WORDS = 16;
constexpr int MAX_DEST = 8;            // tensor-parallel ranks whose output buffers one launch can store into
#ifndef MMA_BACKOFF_NS
#define MMA_BACKOFF_NS 32
#endif                    // u64 words per CTA in the optional profile buffer

// A4 = true selects the block-scaled FP4 x FP4 form (activations quantised to NVFP4 by a kernel that
// runs first): both MMA operands are the packed 4-bit tiles exactly as TMA delivers them, the E4M3 block
// scales of both sides are put into tensor memory by the expansion warps, and one pipeline stage covers
// 256 K elements (four K=64 instructions of kind::mxf4nvf4).
//
// PAIR = true runs the kernel as clusters of two CTAs on neighbouring SMs that issue their MMAs together
// (cta_group::2, 256 features x MT tokens per instruction): each CTA still owns 128 features, their
// weight operand and their accumulator, but holds only HALF of the token tile's activation operand in
// shared memory; the tensor cores of the pair exchange the halves.  That halves the shared-memory traffic
// of the activation operand, which is what bounds the single-CTA form at 128 and 256 tokens.
template <int MT, bool A4 = false, bool PAIR = false> struct Cfg {
    static constexpr int XROWS = PAIR ? MT / 2 : MT;                       // token rows of the tile this CTA stages
    static constexpr int X_TILE_BYTES = XROWS * KB * 2;
    // A4: one stage = packed W [128 x 128 B] | packed x [MT x 128 B] | W scale bytes [128 x 16] | x scale bytes [MT x 16]
    static constexpr int S4_W = 0;
    static constexpr int S4_X = S4_W + RAW_PACKED_BYTES;
    static constexpr int S4_WS = S4_X + XROWS * 128;
    static constexpr int S4_XS = S4_WS + RAW_SCALE_BYTES;
    static constexpr int S4_BYTES = ((S4_XS + MT * 16) + 1023) / 1024 * 1024;
    static constexpr int S4_STAGES = (200 * 1024) / S4_BYTES > 8 ? 8 : (200 * 1024) / S4_BYTES;
    static constexpr int STAGES = A4 ? S4_STAGES : (XROWS >= 256 ? 5 : 8);
    // raw weight stages in flight: small token tiles leave shared memory free, and they are the
    // HBM-bound shapes that need many bytes in flight per SM
    static constexpr int RAW_STAGES = A4 ? STAGES : (XROWS >= 256 ? 2 : (XROWS >= 128 ? 4 : 6));
    static constexpr int A_COLS = KB / 2;                                  // TMEM columns of one weight-operand stage
    static constexpr int TMEM_A_BASE = MT < 32 ? 32 : MT;                  // accumulator occupies [0, MT)
    // A4: scale factors in TMEM.  One instruction reads, per operand, 4 scale bytes (one 32-bit column
    // entry) for each of its rows; lane l of every 32-lane quadrant holds rows l, l+32, l+64, l+96 of a
    // 128-row block in 4 consecutive columns.  Per stage: W 4 instructions x 4 columns, then x 4
    // instructions x (4 columns per 128 tokens).
    static constexpr int XSF_BLOCKS = MT > 128 ? MT / 128 : 1;
    static constexpr int SF_COLS = 16 + 16 * XSF_BLOCKS;
    static constexpr int TMEM_NEEDED = TMEM_A_BASE + (A4 ? STAGES * SF_COLS : STAGES * A_COLS);
    static constexpr int TMEM_COLS = TMEM_NEEDED <= 64 ? 64 : TMEM_NEEDED <= 128 ? 128 : TMEM_NEEDED <= 256 ? 256 : 512;
    static constexpr int MAX_GRANULES = MT * (MAX_RANK_TC / 16);
    // shared memory map (offsets from a 1024-byte aligned base)
    static constexpr int OFF_X = 0;
    static constexpr int OFF_RAWP = OFF_X + STAGES * X_TILE_BYTES;
    static constexpr int OFF_RAWS = OFF_RAWP + RAW_STAGES * RAW_PACKED_BYTES;
    static constexpr int STAGING_BASE = A4 ? STAGES * S4_BYTES : OFF_RAWS + RAW_STAGES * RAW_SCALE_BYTES;
    // After the base K loop the whole staging area is re-used for the LoRA K blocks: each block holds up
    // to four granules, each a B_s tile [128 x 16] and a masked-t tile [MT x 16], BF16, K-major, SWIZZLE_32B.
    static constexpr int L_GRAN_A = FT * 32;                                     // one granule of B_s: [128 x 16] BF16
    static constexpr int L_GRAN_T = XROWS * 32;                                  // one granule of masked t: [XROWS x 16] BF16
    static constexpr int L_TILE_A = 4 * L_GRAN_A;
    static constexpr int L_BLOCK = L_TILE_A + 4 * L_GRAN_T;
    static constexpr int L_STAGES = (STAGING_BASE / L_BLOCK) >= 4 ? 4 : ((STAGING_BASE / L_BLOCK) >= 3 ? 3 : 4);
    static constexpr int STAGING_BYTES = STAGING_BASE > L_STAGES * L_BLOCK ? STAGING_BASE : L_STAGES * L_BLOCK;
    static constexpr int OFF_SLOT = STAGING_BYTES;                               // int32[MT]
    static constexpr int OFF_GRAN = OFF_SLOT + MT * 4;                           // uint16[MAX_GRANULES]
    static constexpr int OFF_GRANB = OFF_GRAN + MAX_GRANULES * 2;                // uint64[MAX_GRANULES]: B_s address of the granule
    static constexpr int OFF_BITMAP = OFF_GRANB + MAX_GRANULES * 8;              // uint32[128]
    static constexpr int OFF_SCAN = OFF_BITMAP + (MAX_LORAS_TC / 32) * 4;        // uint32[8]
    static constexpr int OFF_BAR = OFF_SCAN + 64;                                // mbarriers
    static constexpr int NUM_BARS = 2 * STAGES + 2 * RAW_STAGES + 4 + 2 * L_STAGES;
    static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;                      // tmem ptr, n_gran, abort
    static constexpr int SMEM_BYTES = OFF_MISC + 32 + 1024;                      // + alignment slack
    static_assert(!PAIR || MT >= 128, "pairs are built for token tiles of 128 and 256");
    static_assert(TMEM_NEEDED <= 512, "tensor memory budget");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct Params {
    const int32_t* seq_slot;       // nullable: base only
    const uint64_t* a_table;
    const uint64_t* b_table;
    const uint32_t* rank_table;    // nullable
    const uint16_t* t;             // [M, max_rank] pre-scaled shrink result
    uint16_t* y;
    // Output destinations.  One (y itself) normally.  As one column shard of a tensor-parallel layer the
    // kernel can store its tile straight into every rank's gathered [M, out_row_stride] buffer, at columns
    // y_col0 + f: y_dest[r] is rank r's buffer as mapped into this process (peer memory for r != own rank).
    uint16_t* y_dest[MAX_DEST];
    uint32_t n_dest, y_col0;
    uint32_t M, N, K, out_row_stride, max_loras, max_rank;
    float out_scale;               // scale2 * 2^8 (A16) or scale2 (A4)
    uint32_t k_split;              // >= 1: CTAs (clusters along grid z) that share one output tile, each contracting a
                                   //       share of K and of the LoRA K blocks; partial tiles are summed over
                                   //       distributed shared memory
    uint32_t staged_epilogue;      // destination rows allow 16-byte stores: write the tile out through shared memory
    uint32_t t_tile_cap;           // != 0: the shrink wrote masked-t tiles (ShrinkParams::tile_out) with this many blocks
                                   //       reserved per token tile; they are fetched by TMA (map_t) and `t` is not read
    uint32_t b_pool_strided;       // B_s tiles can be fetched by TMA from a [max_loras][N][max_rank] strided pool
    uint32_t wait_for_shrink;      // launched as a programmatic dependent of the shrink: wait before reading t
    unsigned long long* profile;   // nullable: per-CTA wait/busy cycle counters (PROFILE_WORDS per CTA)
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false when the CTA is aborting (this waiter's limit expired, or
// another role raised the flag).  `backoff_ns` > 0 makes a waiter that expects to wait long (the
// epilogue warps during the main loop) sleep between polls: a polling warp otherwise takes issue
// slots and shared-memory bandwidth from the warps that feed the tensor pipe.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code,
                                          uint32_t backoff_ns = 0, uint64_t limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (true) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                record_status(code);
                *abort_flag = 1u;
                return false;
            }
        }
    }
}

// mbar_wait that also adds the cycles spent waiting to `acc` (profiling builds of a launch only)
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t code,
                                                bool timed, unsigned long long& acc, uint32_t backoff_ns = 0) {
    if (!timed) return mbar_wait(bar, parity, abort_flag, code, backoff_ns);
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, abort_flag, code, backoff_ns);
    acc += (unsigned long long)(clock64() - t0);
    return ok;
}

__device__ __forceinline__ void fence_barrier_init();

// Self-test of the bounded wait, in the form every kernel of this library uses it: warp 0 waits for a phase of a
// barrier on which nothing ever arrives, with a short limit; the wait must give up, record `code` in the status word and
// raise the abort flag; warp 1 waits on the same barrier and must leave through the flag (or its own limit).  The kernel
// then returns normally: no trap, the context stays usable.  out[0] = 1 if warp 0's wait returned false, out[1] the same
// for warp 1, out[2] = nanoseconds warp 0 waited.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, uint32_t code, uint32_t* out) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_s;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(b), "r"(1) : "memory");
        abort_s = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile uint32_t* abort_flag = &abort_s;
    if (threadIdx.x == 0) {
        const uint64_t t0 = global_timer_ns();
        const bool ok = mbar_wait(b, 0, abort_flag, code, 32, limit_ns);
        out[0] = ok ? 0u : 1u;
        const uint64_t dt = global_timer_ns() - t0;
        out[2] = uint32_t(dt > 0xFFFFFFFFull ? 0xFFFFFFFFull : dt);
    } else if (threadIdx.x == 32) {
        const bool ok = mbar_wait(b, 0, abort_flag, code + 1u, 64, 4 * limit_ns);
        out[1] = ok ? 0u : 1u;
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Two-CTA form: the data lands in this CTA's shared memory, the bytes are counted on an mbarrier that may
// live in the pair's other CTA (`bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// shared::cluster address of this CTA's shared-memory address `addr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// arrive on an mbarrier given by its shared::cluster address (possibly in the other CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    // (CTA-scope release, as for a local arrive: what the barrier orders here is tensor-memory and async-proxy
    //  traffic, fenced separately; a cluster-scope release measured ~1700 cycles per arrive)
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Two-CTA forms: executed by the same warp of both CTAs of a pair; the same columns are taken in both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]^T, BF16 inputs, FP32 accumulate; one thread issues.
// A: 128 lanes x 8 columns (16 BF16 per lane, two per 32-bit column, even k in the low half).
template <bool PAIR = false>
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    
    }
}
// D[tmem] (+)= A[smem] * B[smem]^T (both operands K-major shared-memory tiles); one thread issues.
template <bool PAIR = false>
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    
    }
}
// D[tmem] (+)= (A * SFA)[smem] * (B * SFB)[smem]^T : E2M1 operands (K = 64 per instruction), one UE4M3
// scale per 16 elements held in tensor memory; one thread issues.
template <bool PAIR = false>
__device__ __forceinline__ void umma_nvfp4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
    
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
    
    }
}
// block-scaled instruction descriptor: A = B = E2M1, UE4M3 scales, both K-major, M = 128, N = n, K = 64
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(uint32_t n, uint32_t m = 128u) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((m >> 4) << 24);
}
// registers -> 32 lanes x N consecutive 32-bit TMEM columns (lane = this warp's quadrant base + laneid)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
// When every MMA issued so far has completed, arrive on mbarrier `bar`; the pair form arrives on the
// barrier at that shared-memory offset in BOTH CTAs of the pair.
template <bool PAIR = false>
__device__ __forceinline__ void umma_commit(uint32_t bar, uint32_t pair_mask = 3u) {
    if constexpr (PAIR) {
        const uint16_t both = uint16_t(pair_mask);     // the pair's two ranks within the cluster
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"(both) : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
}

// 32 lanes x 16 consecutive columns of 32-bit TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// K-major operand tile, 128-byte rows, SWIZZLE_128B: 8-row groups are 1024 bytes apart.
// start address >> 4 | LBO (unused for swizzled K-major, 1) | SBO = 1024 B | version 1 | SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// K-major operand tile of 16 BF16 (32-byte rows), SWIZZLE_32B: 8-row groups are 256 bytes apart.
__device__ __forceinline__ uint64_t make_kmajor_sw32_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(256 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(6) << 61);
}
// byte offset of 16-byte chunk `c` (0..1) of row `r` in a SWIZZLE_32B tile of 32-byte rows
__device__ __forceinline__ uint32_t sw32_off(uint32_t r, uint32_t c) { return r * 32u + ((c ^ ((r >> 2) & 1u)) << 4); }
// kind::f16 instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t n, uint32_t m = 128u) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 16-byte global -> shared copy; src_bytes < 16 zero-fills the remainder (0 = all zeros, nothing read)
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// byte offset of logical 16-byte chunk `c` (0..7) of row `r` in a SWIZZLE_128B tile of 128-byte rows
__device__ __forceinline__ uint32_t sw128_off(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
// Epilogue for one participant: `q` = TMEM lane quadrant of this warp, chunks of 16 token columns
// c = part, part + nparts, ...  Lane pairs exchange values so every thread stores two adjacent
// features (4 bytes) of one token.
template <int MT>
__device__ __forceinline__ void epilogue_columns(const Params& p, uint32_t tmem_acc, uint32_t q, uint32_t lane,
                                                 uint32_t f0, uint32_t m0, uint32_t part, uint32_t nparts) {
    const uint32_t f = f0 + q * 32 + lane;
    const float osc = p.out_scale;
    const bool pair_ok = (p.out_row_stride % 2u == 0u) && ((reinterpret_cast<uintptr_t>(p.y) & 3u) == 0u);
    const bool odd = lane & 1u;
#pragma unroll 1
    for (uint32_t c0 = part * 16; c0 < uint32_t(MT); c0 += nparts * 16) {
        uint32_t v[16];
        tmem_ld16(tmem_acc + ((q * 32u) << 16) + c0, v);
        tmem_ld_wait();
        if (pair_ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = __uint_as_float(v[2 * i]) * osc, b = __uint_as_float(v[2 * i + 1]) * osc;
                const float got = __shfl_xor_sync(0xFFFFFFFFu, odd ? a : b, 1);
                // even lane: token 2i, features (f, f+1); odd lane: token 2i+1, features (f-1, f)
                const uint32_t m = m0 + c0 + 2 * i + (odd ? 1u : 0u);
                const uint32_t fe = f & ~1u;
                const uint32_t w = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);
                if (m < p.M) {
                    if (fe + 1 < p.N) *reinterpret_cast<uint32_t*>(p.y + size_t(m) * p.out_row_stride + fe) = w;
                    else if (fe < p.N) p.y[size_t(m) * p.out_row_stride + fe] = uint16_t(w & 0xFFFFu);
                }
            }
        } else if (f < p.N) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t m = m0 + c0 + i;
                if (m < p.M) p.y[size_t(m) * p.out_row_stride + f] = f32_to_bf16_bits(__uint_as_float(v[i]) * osc);
            }
        }
    }
}

// map_x: activations (A16: BF16 [M, K]; A4: packed codes [M, K/2]); map_w / map_s: packed weight codes and
// their scale bytes; map_b: the strided adapter pool's B side; map_xs: A4 only, activation scale bytes [M, K/16];
// map_t: the shrink's masked-t blocks as rows of 256 bytes, when p.t_tile_cap != 0.
// Epilogue through shared memory: the warps first lay the tile down as [token][128 features] BF16 (256-byte
// rows; the 16-byte chunks of odd rows rotated by four so that the two rows a store instruction touches
// fall into different banks), meet on an mbarrier, then copy whole rows out with 16-byte stores — to every
// destination buffer in turn.  `e_tid` = 0 .. 32 * EPI_WARPS - 1 numbers the participating threads.
// Requires 16-byte aligned destination rows (checked by the caller); returns false if the wait expired.
template <int MT>
__device__ __forceinline__ bool epilogue_staged(const Params& p, uint32_t tmem_acc, uint32_t tile, uint32_t bar_epi,
                                                volatile uint32_t* abort_flag, uint32_t q, uint32_t lane, uint32_t f0,
                                                uint32_t m0, uint32_t part, uint32_t nparts, uint32_t e_tid) {
    const float osc = p.out_scale;
    const bool odd = lane & 1u;
    const uint32_t fe = (q * 32u + lane) & ~1u;                  // even feature of this lane pair, within the tile
#pragma unroll 1
    for (uint32_t c0 = part * 16; c0 < uint32_t(MT); c0 += nparts * 16) {
        uint32_t v[16];
        tmem_ld16(tmem_acc + ((q * 32u) << 16) + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = __uint_as_float(v[2 * i]) * osc, b = __uint_as_float(v[2 * i + 1]) * osc;
            const float got = __shfl_xor_sync(0xFFFFFFFFu, odd ? a : b, 1);
            // even lane: token 2i, features (fe, fe+1); odd lane: token 2i+1, the same two features
            const uint32_t row = c0 + 2 * i + (odd ? 1u : 0u);
            const uint32_t w = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);
            const uint32_t chunk = (fe >> 3) ^ ((row & 1u) << 2);
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + row * 256u + chunk * 16u + (fe & 7u) * 2u), "r"(w) : "memory");
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_epi);
    if (!mbar_wait(bar_epi, 0, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE)) return false;
    // rows out: 16 threads per row, one 16-byte chunk (8 features) each
    const uint32_t j = e_tid & 15u;
    const uint32_t f = f0 + j * 8u;
    if (f >= p.N) return true;
    const bool whole = f + 8u <= p.N;
    for (uint32_t row = e_tid >> 4; row < uint32_t(MT); row += (32u * EPI_WARPS) >> 4) {
        const uint32_t m = m0 + row;
        if (m >= p.M) break;
        const uint4 val = lds128(tile + row * 256u + ((j ^ ((row & 1u) << 2)) << 4));
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
    return true;
}

// Split-K epilogue, first half: this CTA's partial tile goes, 16 token columns at a time, to the CTA of the
// cluster that owns those columns (chunk c belongs to CTA c % ks), as raw FP32 accumulators into that CTA's
// receive area [source CTA][its chunk][column][128 features] at the start of its staging memory.
template <int MT>
__device__ __forceinline__ void split_send(uint32_t tmem_acc, uint32_t recv0, uint32_t ks, uint32_t kz, uint32_t cta_rank,
                                           uint32_t ctas, uint32_t q, uint32_t lane, uint32_t part, uint32_t nparts) {
    const uint32_t lc_n = (uint32_t(MT) / 16u + ks - 1u) / ks;          // chunks an owner can hold per source
    for (uint32_t c = part; c < uint32_t(MT) / 16u; c += nparts) {
        uint32_t v[16];
        tmem_ld16(tmem_acc + ((q * 32u) << 16) + c * 16u, v);
        tmem_ld_wait();
        const uint32_t owner = c % ks, lc = c / ks;
        const uint32_t dst = map_to_cta(recv0 + (((kz * lc_n + lc) * 16u) * 128u + q * 32u + lane) * 4u, cta_rank + ctas * owner);
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i)
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(dst + i * 512u), "r"(v[i]) : "memory");
    }
}

// Second half: the owner adds the ks partial tiles of its columns in source order, scales, converts and stores.
template <int MT>
__device__ __forceinline__ void split_reduce_store(const Params& p, uint32_t recv0, uint32_t ks, uint32_t kz, uint32_t f0,
                                                   uint32_t m0, uint32_t e_tid) {
    const uint32_t lc_n = (uint32_t(MT) / 16u + ks - 1u) / ks;
    const uint32_t n_chunks = uint32_t(MT) / 16u;
    const uint32_t mine = n_chunks > kz ? (n_chunks - kz + ks - 1u) / ks : 0u;      // chunks kz, kz + ks, ...
    const float osc = p.out_scale;
    for (uint32_t unit = e_tid; unit < mine * 256u; unit += 32u * EPI_WARPS) {
        const uint32_t j = unit & 15u, i = (unit >> 4) & 15u, lc = unit >> 8;
        const uint32_t m = m0 + (lc * ks + kz) * 16u + i, f = f0 + j * 8u;
        if (m >= p.M || f >= p.N) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (uint32_t z = 0; z < ks; ++z) {
            const uint32_t at = recv0 + ((((z * lc_n + lc) * 16u + i) * 128u) + j * 8u) * 4u;
            const uint4 a = lds128(at), b = lds128(at + 16u);
            acc[0] += __uint_as_float(a.x); acc[1] += __uint_as_float(a.y); acc[2] += __uint_as_float(a.z); acc[3] += __uint_as_float(a.w);
            acc[4] += __uint_as_float(b.x); acc[5] += __uint_as_float(b.y); acc[6] += __uint_as_float(b.z); acc[7] += __uint_as_float(b.w);
        }
        uint4 val;
        val.x = pack_bf16x2(acc[0] * osc, acc[1] * osc); val.y = pack_bf16x2(acc[2] * osc, acc[3] * osc);
        val.z = pack_bf16x2(acc[4] * osc, acc[5] * osc); val.w = pack_bf16x2(acc[6] * osc, acc[7] * osc);
        const size_t at = size_t(m) * p.out_row_stride + p.y_col0 + f;
        const bool whole = p.staged_epilogue && f + 8u <= p.N;
        for (uint32_t r = 0; r < p.n_dest; ++r) {
            uint16_t* dst = p.y_dest[r] + at;
            if (whole) {
                *reinterpret_cast<uint4*>(dst) = val;
            } else {
                const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                for (uint32_t e = 0; e < 8u && f + e < p.N; ++e) dst[e] = uint16_t(w4[e >> 1] >> (16u * (e & 1u)));
            }
        }
    }
}

template <int MT, bool A4, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
nvfp4_lora_linear_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                            const __grid_constant__ CUtensorMap map_w,
                            const __grid_constant__ CUtensorMap map_s,
                            const __grid_constant__ CUtensorMap map_b,
                            const __grid_constant__ CUtensorMap map_xs,
                            const __grid_constant__ CUtensorMap map_t,
                            const Params p) {
    using C = Cfg<MT, A4, PAIR>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t x_tile0 = smem_base + C::OFF_X;
    const uint32_t rawp0 = smem_base + C::OFF_RAWP;
    const uint32_t raws0 = smem_base + C::OFF_RAWS;
    int32_t* slot_arr = reinterpret_cast<int32_t*>(smem_gen + C::OFF_SLOT);
    uint16_t* gran = reinterpret_cast<uint16_t*>(smem_gen + C::OFF_GRAN);
    unsigned long long* gran_b = reinterpret_cast<unsigned long long*>(smem_gen + C::OFF_GRANB);
    uint32_t* bitmap = reinterpret_cast<uint32_t*>(smem_gen + C::OFF_BITMAP);
    uint32_t* scan = reinterpret_cast<uint32_t*>(smem_gen + C::OFF_SCAN);
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    // FULL[s]: both operands of stage s are in place.  DEQ_GROUP_WARPS + 1 arrivals per phase: the eight
    // expansion warps, plus the TMA producer (with the tile's byte count) for a base K block or one
    // extra arrival by an expansion thread for a LoRA K block, whose activation tile they build.
    const uint32_t BAR_FULL = bar0;                                    // [STAGES] operands -> MMA
    const uint32_t BAR_EMPTY = bar0 + 8 * C::STAGES;                   // [STAGES] MMA -> producers
    const uint32_t BAR_FULL_RAW = bar0 + 16 * C::STAGES;               // [C::RAW_STAGES]
    const uint32_t BAR_EMPTY_RAW = BAR_FULL_RAW + 8 * C::RAW_STAGES;      // [C::RAW_STAGES]
    const uint32_t BAR_ACC = BAR_EMPTY_RAW + 8 * C::RAW_STAGES;           // accumulator complete
    const uint32_t BAR_LIST = BAR_ACC + 8;                             // granule list ready
    const uint32_t BAR_LFULL = BAR_LIST + 8;                           // [L_STAGES] LoRA operands -> MMA
    const uint32_t BAR_LEMPTY = BAR_LFULL + 8 * C::L_STAGES;           // [L_STAGES] MMA -> LoRA operand build
    const uint32_t BAR_DRAINED = BAR_LEMPTY + 8 * C::L_STAGES;         // every expansion warp is done with the staging area
    const uint32_t BAR_EPI = BAR_DRAINED + 8;                          // every epilogue warp has put its part of the tile into shared memory
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + C::OFF_MISC);
    // misc[0] = TMEM base address, misc[1] = granule count, misc[2] = abort flag
    volatile uint32_t* abort_flag = misc + 2;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bool acc_ready = false;                              // split K: this warp saw the accumulator complete
    const uint32_t f0 = blockIdx.x * FT;
    const uint32_t m0 = blockIdx.y * MT;
    constexpr uint32_t CTAS = PAIR ? 2u : 1u;
    const uint32_t ks = p.k_split, kz = blockIdx.z;      // split K: CTAs per output tile, and which of them this is
    // a pair = two CTAs with neighbouring feature tiles (x and x + 1 in a cluster); its first CTA issues the MMAs for both
    const uint32_t cta_rank = PAIR ? (blockIdx.x & 1u) : 0u;
    const uint32_t leader_rank = CTAS * kz;              // rank, within the cluster, of this pair's first CTA
    const uint32_t pair_mask = 3u << (2u * kz);
    const bool leader = cta_rank == 0u;
    const uint32_t mx0 = m0 + cta_rank * C::XROWS;       // first token row whose activations this CTA stages
    // This CTA's share of the contraction (all of it unless p.k_split > 1): whole raw stages of 256 K elements.
    const uint32_t total_kb = A4 ? p.K / KRAW : (p.K + KB - 1) / KB;
    const uint32_t total_raw = A4 ? total_kb : (total_kb + 3u) / 4u;
    const uint32_t raw_lo = kz * total_raw / ks, raw_hi = (kz + 1u) * total_raw / ks;
    const uint32_t kb_lo = A4 ? raw_lo : 4u * raw_lo;
    const uint32_t num_kb = (A4 ? raw_hi : min(4u * raw_hi, total_kb)) - kb_lo;      // pipeline steps of the base K loop
    const bool prof = p.profile != nullptr;
    const long long t_entry = clock64();
    const uint64_t t_entry_ns = prof ? global_timer_ns() : 0;
    unsigned long long* prof_row = prof ? p.profile + (size_t(blockIdx.y) * gridDim.x + blockIdx.x) * PROFILE_WORDS : nullptr;

    if (tid == 0) {
        for (int i = 0; i < C::STAGES; ++i) {
            // A16: every expansion warp of the pair writes part of a stage; A4: the four warps of one half do
            mbar_init(BAR_FULL + 8 * i, CTAS * (A4 ? DEQ_GROUP_WARPS / 2 : DEQ_GROUP_WARPS) + 1);     // used in the pair's first CTA only
            mbar_init(BAR_EMPTY + 8 * i, 1);
        }
        for (int i = 0; i < C::RAW_STAGES; ++i) {
            mbar_init(BAR_FULL_RAW + 8 * i, 1);
            mbar_init(BAR_EMPTY_RAW + 8 * i, DEQ_WARPS);
        }
        mbar_init(BAR_ACC, 1);
        mbar_init(BAR_LIST, 1);
        mbar_init(BAR_DRAINED, DEQ_WARPS);
        mbar_init(BAR_EPI, EPI_WARPS);
        for (int i = 0; i < C::L_STAGES; ++i) {
            mbar_init(BAR_LFULL + 8 * i, p.t_tile_cap ? 1u : CTAS * DEQ_WARPS + 1);
            mbar_init(BAR_LEMPTY + 8 * i, 1);
        }
        misc[1] = 0;
        misc[2] = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) { tmem_alloc_pair(smem_base + C::OFF_MISC, C::TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_base + C::OFF_MISC, C::TMEM_COLS); tmem_relinquish(); }
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_s);
        if (p.b_pool_strided) tma_prefetch_desc(&map_b);
        if (A4) tma_prefetch_desc(&map_xs);
        if (p.t_tile_cap) tma_prefetch_desc(&map_t);
    }
    tcgen05_fence_before();
    __syncwarp();
    // (pair: neither CTA may signal the other's barriers before they are initialised)
    if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
    tcgen05_fence_after();
    // barriers the MMA thread waits on live in the pair's first CTA; everyone else arrives there
    const uint32_t full_at_leader = PAIR ? map_to_cta(BAR_FULL, leader_rank) : BAR_FULL;
    const uint32_t lfull_at_leader = PAIR ? map_to_cta(BAR_LFULL, leader_rank) : BAR_LFULL;
    auto arrive_at_leader = [&](uint32_t bar_at_leader) {
        if constexpr (PAIR) mbar_arrive_cluster(bar_at_leader); else mbar_arrive(bar_at_leader);
    };
    const uint32_t tmem_acc = misc[0];
    const uint32_t tmem_a0 = tmem_acc + C::TMEM_A_BASE;   // A16: weight-operand stages [tmem_a0 + s * A_COLS, + A_COLS);
                                                          // A4: scale-factor stages [tmem_a0 + s * SF_COLS, + SF_COLS)

    if (warp == 0) {
        // ===================================== TMA producer =====================================
        if (lane == 0 && A4) {
            // One ring: a stage's two packed operand tiles complete FULL[s] (which the MMA thread waits
            // on), its two scale-byte tiles FULL_RAW[s] (which the warps that move them to TMEM wait on).
            const uint32_t rot = (blockIdx.x / CTAS) % num_kb;     // (the CTAs of a pair walk K in the same order)
            uint32_t s = 0, ph = 0;
            for (uint32_t it = 0; it < num_kb; ++it) {
                if (!mbar_wait(BAR_EMPTY + 8 * s, ph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 32)) break;
                const uint32_t st = smem_base + s * C::S4_BYTES;
                const uint32_t kk = kb_lo + (it + rot) % num_kb;
                mbar_arrive_expect_tx(BAR_FULL_RAW + 8 * s, RAW_SCALE_BYTES + MT * 16);
                tma_load_2d(st + C::S4_WS, &map_s, int32_t(kk * (KRAW / 16)), int32_t(f0), BAR_FULL_RAW + 8 * s);
                tma_load_2d(st + C::S4_XS, &map_xs, int32_t(kk * (KRAW / 16)), int32_t(m0), BAR_FULL_RAW + 8 * s);
                if (leader) mbar_arrive_expect_tx(BAR_FULL + 8 * s, CTAS * (RAW_PACKED_BYTES + C::XROWS * 128));
                if constexpr (PAIR) {
                    tma_load_2d_pair(st + C::S4_W, &map_w, int32_t(kk * (KRAW / 2)), int32_t(f0), full_at_leader + 8 * s);
                    tma_load_2d_pair(st + C::S4_X, &map_x, int32_t(kk * (KRAW / 2)), int32_t(mx0), full_at_leader + 8 * s);
                } else {
                    tma_load_2d(st + C::S4_W, &map_w, int32_t(kk * (KRAW / 2)), int32_t(f0), BAR_FULL + 8 * s);
                    tma_load_2d(st + C::S4_X, &map_x, int32_t(kk * (KRAW / 2)), int32_t(m0), BAR_FULL + 8 * s);
                }
                if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
            }
        }
        if (lane == 0 && !A4) {
            // One thread feeds two rings without blocking on either: activation tiles (one per K
            // block) and raw weight stages (codes + scale bytes, one per four K blocks), so the
            // weight stream runs ahead of the activation stream.
            // CTAs start their K loop at different K offsets (a rotation in units of one raw stage),
            // so concurrently running CTAs do not all pull the same activation lines at one moment.
            const uint32_t num_raw = (num_kb + 3u) / 4u;
            const uint32_t rot_raw = (num_kb % 4u == 0u) ? ((blockIdx.x / CTAS) % num_raw) : 0u;   // (same for both CTAs of a pair)
            uint32_t it = 0, ri = 0, spins = 0;
            uint64_t t0 = 0;
            while (it < num_kb || ri < num_raw) {
                bool progressed = false;
                if (ri < num_raw) {
                    const uint32_t rs = ri % C::RAW_STAGES, rph = (ri / C::RAW_STAGES) & 1u;
                    if (mbar_try_wait(BAR_EMPTY_RAW + 8 * rs, rph ^ 1u)) {
                        mbar_arrive_expect_tx(BAR_FULL_RAW + 8 * rs, RAW_PACKED_BYTES + RAW_SCALE_BYTES);
                        const uint32_t rk = raw_lo + (ri + rot_raw) % num_raw;
                        tma_load_2d(rawp0 + rs * RAW_PACKED_BYTES, &map_w, int32_t(rk * (KRAW / 2)), int32_t(f0), BAR_FULL_RAW + 8 * rs);
                        tma_load_2d(raws0 + rs * RAW_SCALE_BYTES, &map_s, int32_t(rk * (KRAW / 16)), int32_t(f0), BAR_FULL_RAW + 8 * rs);
                        ++ri;
                        progressed = true;
                    }
                }
                if (it < num_kb) {
                    const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
                    if (mbar_try_wait(BAR_EMPTY + 8 * s, ph ^ 1u)) {
                        if (leader) mbar_arrive_expect_tx(BAR_FULL + 8 * s, CTAS * C::X_TILE_BYTES);
                        const uint32_t kb = kb_lo + (it + 4u * rot_raw) % num_kb;
                        if constexpr (PAIR) tma_load_2d_pair(x_tile0 + s * C::X_TILE_BYTES, &map_x, int32_t(kb * KB), int32_t(mx0), full_at_leader + 8 * s);
                        else tma_load_2d(x_tile0 + s * C::X_TILE_BYTES, &map_x, int32_t(kb * KB), int32_t(m0), BAR_FULL + 8 * s);
                        ++it;
                        progressed = true;
                    }
                }
                if (progressed) {
                    spins = 0;
                    t0 = 0;
                } else {
                    __nanosleep(64);
                    if ((++spins & 63u) != 0u) continue;
                    if (*abort_flag) break;
                    const uint64_t now = global_timer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > WAIT_LIMIT_NS) {
                        record_status(STATUS_WAIT_EXPIRED_PRODUCER);
                        *abort_flag = 1u;
                        break;
                    }
                }
            }
        }
        if (lane == 0) {
            // LoRA K blocks: when the adapter pool is strided, this thread also fetches the B_s tiles
            // (one 3-D TMA per granule), running ahead of the warps that build the masked-t tiles.
            if (p.seq_slot && p.b_pool_strided && !*abort_flag &&
                mbar_wait(BAR_LIST, 0, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 64)) {
                const uint32_t n_gran = misc[1];
                // the staging area may be overwritten once the expansion warps have seen every base MMA finish
                if (n_gran && mbar_wait(BAR_DRAINED, 0, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER, 32)) {
                    // masked-t tiles are the shrink grid's output: it must be complete before they are fetched
                    if (p.t_tile_cap && p.wait_for_shrink) asm volatile("griddepcontrol.wait;" ::: "memory");
                    // this CTA's blocks: [XROWS x 16] BF16 images, C::L_GRAN_T bytes each, consecutive in list order
                    const uint32_t t_row0 = (blockIdx.y * CTAS + cta_rank) * p.t_tile_cap * uint32_t(C::L_GRAN_T / 256);
                    uint32_t ls = 0, lph = 0;
                    for (uint32_t g0 = 4 * kz; g0 < n_gran; g0 += 4 * ks) {      // this CTA's share of the LoRA K blocks
                        if (!mbar_wait(BAR_LEMPTY + 8 * ls, lph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_PRODUCER)) break;
                        const uint32_t ng = min(4u, n_gran - g0);
                        const uint32_t base = x_tile0 + ls * C::L_BLOCK;
                        if (leader) mbar_arrive_expect_tx(BAR_LFULL + 8 * ls, CTAS * ng * (C::L_GRAN_A + (p.t_tile_cap ? C::L_GRAN_T : 0)));
                        for (uint32_t g = 0; g < ng; ++g) {
                            const uint32_t e = gran[g0 + g];
                            if constexpr (PAIR) tma_load_3d_pair(base + g * C::L_GRAN_A, &map_b, int32_t((e & 3u) * 16u), int32_t(f0), int32_t(e >> 2), lfull_at_leader + 8 * ls);
                            else tma_load_3d(base + g * C::L_GRAN_A, &map_b, int32_t((e & 3u) * 16u), int32_t(f0), int32_t(e >> 2), BAR_LFULL + 8 * ls);
                            if (p.t_tile_cap) {
                                const int32_t row = int32_t(t_row0 + (g0 + g) * uint32_t(C::L_GRAN_T / 256));
                                if constexpr (PAIR) tma_load_2d_pair(base + C::L_TILE_A + g * C::L_GRAN_T, &map_t, 0, row, lfull_at_leader + 8 * ls);
                                else tma_load_2d(base + C::L_TILE_A + g * C::L_GRAN_T, &map_t, 0, row, BAR_LFULL + 8 * ls);
                            }
                        }
                        if (++ls == uint32_t(C::L_STAGES)) { ls = 0; lph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===================================== MMA issuer =======================================
        // One thread runs this role.  tcgen05.mma issue blocks once a couple of instructions are
        // queued, so whatever this thread executes between the last MMA of one K block and the
        // first of the next must fit inside that short queue or the tensor pipe drains: the loop
        // carries its stage/phase/operand addresses incrementally and waits on ONE barrier per block.
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_bf16(MT, 128u * CTAS);
            unsigned long long w_full = 0;
            const long long t_begin = prof ? clock64() : 0;
            bool ok = true;
            uint32_t s = 0, ph = 0, acc = 0;
            uint32_t bar_full = BAR_FULL, bar_empty = BAR_EMPTY, a_tmem = tmem_a0;
            uint64_t b_desc = make_kmajor_sw128_desc(x_tile0);
            constexpr uint64_t b_desc_step = uint64_t(C::X_TILE_BYTES >> 4);
            bool ready = false;                              // result of an early look at this block's barrier
            if constexpr (A4) {
                // four K=64 block-scaled instructions per stage; both operands are the packed tiles, the
                // scales sit in this stage's TMEM columns
                constexpr uint32_t idesc4 = make_idesc_nvfp4(MT, 128u * CTAS);
                uint32_t st = smem_base, sf = tmem_a0;
                for (uint32_t it = 0; it < num_kb; ++it) {
                    ok = mbar_wait_timed(bar_full, ph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_full, MMA_BACKOFF_NS);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint64_t wa = make_kmajor_sw128_desc(st + C::S4_W);
                    const uint64_t xb = make_kmajor_sw128_desc(st + C::S4_X);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i)   // 64 k = 32 bytes along the swizzled 128-byte row
                        umma_nvfp4_ss<PAIR>(tmem_acc, wa + 2 * i, xb + 2 * i, idesc4, sf + 4 * i, sf + 16 + 4 * C::XSF_BLOCKS * i, acc | i);
                    umma_commit<PAIR>(bar_empty, pair_mask);
                    acc = 1u;
                    bar_full += 8; bar_empty += 8; st += C::S4_BYTES; sf += C::SF_COLS;
                    if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; bar_full = BAR_FULL; bar_empty = BAR_EMPTY; st = smem_base; sf = tmem_a0; }
                }
            } else
            for (uint32_t it = 0; it < num_kb; ++it) {
                if (!ready) {
                    ok = mbar_wait_timed(bar_full, ph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_full, MMA_BACKOFF_NS);
                    if (!ok) break;
                }
                tcgen05_fence_after();
                // next block's stage / phase / operands
                uint32_t n_full = bar_full + 8, n_empty = bar_empty + 8, n_a = a_tmem + C::A_COLS, n_ph = ph;
                uint64_t n_b = b_desc + b_desc_step;
                if (++s == uint32_t(C::STAGES)) {
                    s = 0; n_ph ^= 1u;
                    n_full = BAR_FULL; n_empty = BAR_EMPTY; n_a = tmem_a0; n_b = b_desc - b_desc_step * (C::STAGES - 1);
                }
                // 16 k per instruction: 8 TMEM columns of A, 32 bytes along the swizzled row of B
                umma_bf16_ts<PAIR>(tmem_acc, a_tmem, b_desc, idesc, acc);
                umma_bf16_ts<PAIR>(tmem_acc, a_tmem + 8, b_desc + 2, idesc, 1u);
                // look at the next block's barrier while the tensor pipe still holds queued work
                ready = mbar_try_wait(n_full, n_ph);
                umma_bf16_ts<PAIR>(tmem_acc, a_tmem + 16, b_desc + 4, idesc, 1u);
                umma_bf16_ts<PAIR>(tmem_acc, a_tmem + 24, b_desc + 6, idesc, 1u);
                umma_commit<PAIR>(bar_empty, pair_mask);
                acc = 1u;
                bar_full = n_full; bar_empty = n_empty; a_tmem = n_a; b_desc = n_b; ph = n_ph;
            }
            ready = false;
            if (prof) { prof_row[14] = (unsigned long long)(clock64() - t_begin); prof_row[15] = w_full; }
            // base K blocks issued; the LoRA K blocks follow once the granule list is known
            if (ok) ok = mbar_wait(BAR_LIST, 0, abort_flag, STATUS_WAIT_EXPIRED_MMA, 32);
            if (ok) {
                // LoRA K blocks: both operands are shared-memory tiles in their own ring
                const uint32_t n_gran = misc[1];
                uint32_t ls = 0, lph = 0;
                for (uint32_t g0 = 4 * kz; g0 < n_gran; g0 += 4 * ks) {
                    ok = mbar_wait_timed(BAR_LFULL + 8 * ls, lph, abort_flag, STATUS_WAIT_EXPIRED_MMA, prof, w_full, MMA_BACKOFF_NS);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t ksteps = min(4u, n_gran - g0);
                    const uint64_t la = make_kmajor_sw32_desc(x_tile0 + ls * C::L_BLOCK);
                    const uint64_t lb_ = make_kmajor_sw32_desc(x_tile0 + ls * C::L_BLOCK + C::L_TILE_A);
                    for (uint32_t k = 0; k < ksteps; ++k)   // one granule = one 16-wide K step with its own pair of tiles
                        umma_bf16_ss<PAIR>(tmem_acc, la + k * (C::L_GRAN_A >> 4), lb_ + k * (C::L_GRAN_T >> 4), idesc, 1u);
                    umma_commit<PAIR>(BAR_LEMPTY + 8 * ls, pair_mask);
                    if (++ls == uint32_t(C::L_STAGES)) { ls = 0; lph ^= 1u; }
                }
            }
            if (ok) umma_commit<PAIR>(BAR_ACC, pair_mask);
            if (prof) { prof_row[0] = w_full + ((unsigned long long)(t_begin - t_entry) << 32); prof_row[2] = (unsigned long long)(clock64() - t_begin); }
        }
        __syncwarp();
    } else if (warp < DEQ_WARP0) {
        // ============================ granule list, then the epilogue ===========================
        const uint32_t te = tid - EPI_WARP0 * 32;          // 0..127
        uint32_t n_gran = 0;
        if (p.seq_slot) {
            bitmap[te] = 0;                                 // 128 words = 4096 slots
            named_bar_sync(1, EPI_THREADS);
            for (uint32_t r = te; r < uint32_t(MT); r += EPI_THREADS) {
                const uint32_t m = m0 + r;
                int32_t s = (m < p.M) ? p.seq_slot[m] : -1;
                if (s >= 0) {
                    if (uint32_t(s) >= p.max_loras) { record_status(STATUS_SLOT_OUT_OF_RANGE); s = -1; }
                    else if (p.a_table[s] == 0ull || p.b_table[s] == 0ull) s = -1;
                }
                slot_arr[r] = s;
                if (s >= 0) atomicOr(&bitmap[uint32_t(s) >> 5], 1u << (uint32_t(s) & 31u));
            }
            named_bar_sync(1, EPI_THREADS);
            // thread te owns slots [32 te, 32 te + 32): count its granules, scan, emit in slot order
            uint32_t word = bitmap[te], cnt = 0;
            for (uint32_t w = word; w; w &= w - 1) {
                const uint32_t s = te * 32 + (__ffs(w) - 1);
                const uint32_t r = p.rank_table ? min(p.rank_table[s], p.max_rank) : p.max_rank;
                cnt += (r + 15u) / 16u;
            }
            uint32_t incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= uint32_t(o)) incl += v;
            }
            if (lane == 31) scan[warp - EPI_WARP0] = incl;
            named_bar_sync(1, EPI_THREADS);
            uint32_t base = 0;
            for (uint32_t w = 0; w < warp - EPI_WARP0; ++w) base += scan[w];
            n_gran = scan[0] + scan[1] + scan[2] + scan[3];
            uint32_t pos = base + incl - cnt;
            for (uint32_t w = word; w; w &= w - 1) {
                const uint32_t s = te * 32 + (__ffs(w) - 1);
                const uint32_t r = p.rank_table ? min(p.rank_table[s], p.max_rank) : p.max_rank;
                const unsigned long long b_addr = p.b_table[s];
                for (uint32_t g = 0; g < (r + 15u) / 16u; ++g) { gran_b[pos] = b_addr; gran[pos++] = uint16_t((s << 2) | g); }
            }
            if (te == 0) misc[1] = n_gran;
            named_bar_sync(1, EPI_THREADS);
            // For every token row: where its slot's granules sit in the list (they are consecutive) and
            // how many there are, packed (pos << 3 | count); 0xFFFF = the row takes no LoRA term.  The
            // slot bitmap is dead by now and its space is re-used.
            uint16_t* row_pg = reinterpret_cast<uint16_t*>(bitmap);
            for (uint32_t r = te; r < uint32_t(MT); r += EPI_THREADS) {
                const int32_t sl = slot_arr[r];
                uint16_t pg = 0xFFFFu;
                if (sl >= 0) {
                    const uint32_t key = uint32_t(sl) << 2;       // first entry >= key is (sl, granule 0)
                    uint32_t lo = 0, hi = n_gran;
                    while (lo < hi) { const uint32_t mid = (lo + hi) >> 1; if (gran[mid] < key) lo = mid + 1; else hi = mid; }
                    const uint32_t rk = p.rank_table ? min(p.rank_table[sl], p.max_rank) : p.max_rank;
                    pg = uint16_t((lo << 3) | ((rk + 15u) / 16u));
                }
                row_pg[r] = pg;
            }
            named_bar_sync(1, EPI_THREADS);
        }
        if (te == 0) mbar_arrive(BAR_LIST);
        // Pull this CTA's rows of every B_s it will need into L2 now, while the base K loop runs:
        // the LoRA K blocks at the end then see L2 latency instead of HBM latency.
        if (n_gran) {
            const uint32_t f = f0 + te;
            if (f < p.N) {
                for (uint32_t g = 0; g < n_gran; ++g) {
                    const uint32_t e = gran[g];
                    const uint16_t* src = reinterpret_cast<const uint16_t*>(gran_b[g]) + size_t(f) * p.max_rank + (e & 3u) * 16u;
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
                }
            }
        }

        // ---- epilogue, shared with the expansion warps: TMEM lane = feature, column = token ----
        if (mbar_wait(BAR_ACC, 0, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 512)) {
            const long long t_epi = clock64();
            tcgen05_fence_after();
            if (ks > 1) acc_ready = true;                   // split K: the tile is finished by the whole cluster, below
            else if (p.staged_epilogue) epilogue_staged<MT>(p, tmem_acc, x_tile0, BAR_EPI, abort_flag, warp & 3u, lane, f0, m0, 0, 1 + DEQ_WARPS / 4, te);
            else epilogue_columns<MT>(p, tmem_acc, warp & 3u, lane, f0, m0, 0, 1 + DEQ_WARPS / 4);
            if (prof && te == 0) prof_row[7] = (unsigned long long)(clock64() - t_epi);
        }
    } else {
        // ========================== NVFP4 -> BF16 weight operand, into TMEM ======================
        // warp w may touch TMEM lanes [32 (w % 4), +32): it owns those 32 features; the two warps
        // of a quadrant split each K block in halves of 32.  K blocks are expanded two at a time so
        // that each warp has two independent dependency chains in flight.
        const uint32_t q = warp & 3u;
        const uint32_t half = ((warp - DEQ_WARP0) >> 2) & 1u;
        const uint32_t grp = (warp - DEQ_WARP0) >> 3;       // expansion group of this warp
        const uint32_t row = q * 32 + lane;
        const uint32_t td = tid - DEQ_WARP0 * 32;
        const uint32_t lane_base = (q * 32u) << 16;
        bool ok = true;
        unsigned long long w_raw = 0, w_empty = 0;
        const long long t_begin = clock64();
        const uint32_t num_raw = (num_kb + 3u) / 4u;
        uint32_t s = grp, ph = 0;                            // stage / phase of this group's next K block
        uint32_t rs = 0, rph = 0;
        if constexpr (A4) {
            // Block scales, shared memory -> registers -> TMEM.  The warp of quadrant q writes lanes
            // [32 q, +32); the MMA wants every quadrant to hold the same 32 x 4-column image (lane l:
            // rows l, l+32, l+64, l+96 of the 128-row block), so the four warps of a half write the same
            // values.  The halves take alternate stages (both operands' scales), so that one stage's
            // load -> store -> wait chain runs under the other's.
            s = 0;
            for (uint32_t it = 0; ok && it < num_kb; ++it) {
                if ((it & 1u) != half) {
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
                        for (uint32_t i = 0; i < 4; ++i) {
                            // a NaN scale byte decodes to zero (as in the scalar decode); the MMA reads
                            // unsigned scales, so a sign bit cannot be honoured: it is reported and dropped
                            const uint32_t nan = __vcmpeq4(w[i] & 0x7F7F7F7Fu, 0x7F7F7F7Fu);
                            neg |= w[i] & ~nan;
                            r[4 * i + c] = w[i] & ~nan & 0x7F7F7F7Fu;
                        }
                    }
                    if (neg & 0x80808080u) record_status(STATUS_NEGATIVE_SCALE);
                    tmem_st16(sf, r);
                }
                if constexpr (C::XSF_BLOCKS == 1) {
                    uint32_t r[16];                           // column = 4 i + c
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c) {
                        const uint32_t row = lane + 32 * c;
                        uint4 v = make_uint4(0u, 0u, 0u, 0u);
                        if (row < uint32_t(MT)) v = lds128(st + C::S4_XS + row * 16);
                        r[c] = v.x; r[4 + c] = v.y; r[8 + c] = v.z; r[12 + c] = v.w;
                    }
                    tmem_st16(sf + 16, r);
                } else {
                    {
                        static_assert(C::XSF_BLOCKS <= 2, "token tiles of at most 256");
                        uint32_t r0[16], r1[16];              // instructions 0,1 and 2,3: column = 8 i + 4 blk + c
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
                }
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) arrive_at_leader(full_at_leader + 8 * s);
                if (++s == uint32_t(C::STAGES)) { s = 0; ph ^= 1u; }
            }
        } else
        for (uint32_t ri = 0; ok && ri < num_raw; ++ri) {
            ok = mbar_wait_timed(BAR_FULL_RAW + 8 * rs, rph, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_raw);
            if (!ok) break;
            const uint4 sc4 = lds128(raws0 + rs * RAW_SCALE_BYTES + row * 16);
            const uint32_t scw[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
#pragma unroll
            for (uint32_t jr = 0; jr < 4; jr += 2 * DEQ_GROUPS) {
                if (ri * 4 + jr + grp >= num_kb) break;
                const bool two = ri * 4 + jr + grp + DEQ_GROUPS < num_kb;
                uint32_t o[2][16];
#pragma unroll
                for (uint32_t u = 0; u < 2; ++u) {
                    const uint32_t j = jr + grp + DEQ_GROUPS * u;       // K block of the raw stage (0..3)
                    // 32 codes of this row: logical chunk 2j + half of the swizzled 128-byte raw row
                    const uint4 pk = lds128(rawp0 + rs * RAW_PACKED_BYTES + sw128_off(row, 2 * j + half));
                    const uint32_t pw[4] = {pk.x, pk.y, pk.z, pk.w};
                    const uint32_t scj = j == 0 ? scw[0] : (j == 1 ? scw[1] : (j == 2 ? scw[2] : scw[3]));
                    const uint32_t sbytes = scj >> (16 * half);          // scale bytes 2*half, 2*half+1 of word j
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
                uint32_t s1 = s0 + DEQ_GROUPS, ph1 = ph0;
                if (s1 >= uint32_t(C::STAGES)) { s1 -= C::STAGES; ph1 ^= 1u; }
                ok = mbar_wait_timed(BAR_EMPTY + 8 * s0, ph0 ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_empty);
                if (!ok) break;
                tcgen05_fence_after();
                // this thread's 32 k of its feature row: 16 columns at 16 * half of the stage
                tmem_st16(tmem_a0 + lane_base + s0 * C::A_COLS + 16 * half, o[0]);
                if (two) {
                    ok = mbar_wait_timed(BAR_EMPTY + 8 * s1, ph1 ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_empty);
                    if (!ok) break;
                    tcgen05_fence_after();
                    tmem_st16(tmem_a0 + lane_base + s1 * C::A_COLS + 16 * half, o[1]);
                }
                tmem_st_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    arrive_at_leader(full_at_leader + 8 * s0);
                    if (two) arrive_at_leader(full_at_leader + 8 * s1);
                }
                s = s1 + DEQ_GROUPS; ph = ph1;
                if (s >= uint32_t(C::STAGES)) { s -= C::STAGES; ph ^= 1u; }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_EMPTY_RAW + 8 * rs);
            if (++rs == uint32_t(C::RAW_STAGES)) { rs = 0; rph ^= 1u; }
        }
        if (prof && td == 0) {
            prof_row[3] = w_raw; prof_row[4] = w_empty; prof_row[5] = (unsigned long long)(clock64() - t_begin);
        }
        const long long t_lora = clock64();

        // ---- LoRA K blocks.  Per granule: a B_s tile [128 features x 16 ranks] and a masked-t tile
        //      [MT tokens x 16] (rows of t where the token is routed to the granule's slot, zero
        //      elsewhere), both in the MMA's SWIZZLE_32B layout, four granules to a block, L_STAGES
        //      blocks in flight.  B_s tiles come by 3-D TMA out of the strided adapter pool (one
        //      tensor map covers every slot); without such a pool they are copied with cp.async like
        //      the t tiles.  No registers hold data, so shared memory alone sets the pipeline depth.
        if (ok) ok = mbar_wait(BAR_LIST, 0, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, 32);
        // t is produced by the shrink grid this kernel may have overtaken: everything above ran
        // without it; from here on its writes must be complete and visible.
        if (p.wait_for_shrink) asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t n_gran = ok ? misc[1] : 0u;
        const uint32_t n_lb = (n_gran + 3u) / 4u;
        s = num_kb % uint32_t(C::STAGES);                    // stage / phase the K block after the last one would take
        ph = (num_kb / uint32_t(C::STAGES)) & 1u;
        if (ok && n_lb > 0) {
            // the staging area is about to be overwritten: every base MMA must have read its x tile,
            // and every expansion warp must be done with the raw weight stages
            {
                uint32_t ss = s, pp = ph;
                for (int i = 0; ok && i < C::STAGES; ++i) {
                    ok = mbar_wait(BAR_EMPTY + 8 * ss, pp ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT);
                    if (++ss == uint32_t(C::STAGES)) { ss = 0; pp ^= 1u; }
                }
            }
            // (an mbarrier rather than bar.sync, so that this wait is bounded like every other one)
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_DRAINED);
            if (ok) ok = mbar_wait(BAR_DRAINED, 0, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT);
        }
        if (ok && n_lb > 0 && !p.t_tile_cap) {
            constexpr uint32_t XR = uint32_t(C::XROWS);     // this CTA builds the tile's token rows [cta_rank * XR, + XR)
            constexpr uint32_t T_TASKS = (XR * 2 + DEQ_THREADS - 1) / DEQ_THREADS;             // per granule
            // Masked-t side.  Task -> (row = task % MT, 16-byte chunk = task / MT): eight neighbouring lanes
            // write eight different swizzled chunks.  A row's slot owns `t_ng` consecutive granules
            // starting at list position `t_pos`, so whether block lb touches the row is arithmetic on lb.
            // All t tiles are zeroed once; afterwards a task only writes where its row is routed to the
            // granule (a copy of 16 bytes of t) or was, the last time the stage was used (zeros again).
            const uint16_t* row_pg = reinterpret_cast<const uint16_t*>(bitmap);
            int32_t t_pos[T_TASKS];
            uint32_t t_ng[T_TASKS];
            const uint16_t* t_src[T_TASKS];
            uint32_t t_dst[T_TASKS];
#pragma unroll
            for (uint32_t u = 0; u < T_TASKS; ++u) {
                const uint32_t task = td + u * DEQ_THREADS;
                const uint32_t r = task & (XR - 1u), hh = task / XR;
                const uint32_t tile_row = cta_rank * XR + r;
                const uint32_t pg = (task < XR * 2 && p.seq_slot) ? row_pg[tile_row] : 0xFFFFu;
                t_ng[u] = pg == 0xFFFFu ? 0u : (pg & 7u);
                t_pos[u] = int32_t(pg >> 3);
                t_src[u] = p.t + size_t(m0 + tile_row) * p.max_rank + 8 * hh;
                t_dst[u] = C::L_TILE_A + r * 32u + ((hh ^ ((r >> 2) & 1u)) << 4);
                // granule columns beyond max_rank do not exist in t: treat as not routed
                if (t_ng[u] && 16 * (t_ng[u] - 1) + 8 * hh >= p.max_rank) t_ng[u] -= 1;
            }
            for (uint32_t i = td; i < uint32_t(C::L_STAGES) * XR * 8u; i += DEQ_THREADS) {
                const uint32_t st_i = i / (XR * 8u), off = (i % (XR * 8u)) * 16u;
                sts128(x_tile0 + st_i * C::L_BLOCK + C::L_TILE_A + off, 0u, 0u, 0u, 0u);
            }
            // B_s side: this thread copies chunk (2 g + a_h) of feature row a_row
            const uint32_t a_row = td & 127u, a_h = (td >> 7) & 1u;    // threads 0..255 copy B_s when it does not come by TMA
            const uint32_t a_dst = sw32_off(a_row, a_h);
            const uint32_t f = f0 + a_row;
            const size_t a_src_off = size_t(f) * p.max_rank + 8 * a_h;
            uint32_t ls = 0, lph = 0;
            unsigned long long w_lempty = 0, w_issue = 0, w_group = 0;
            auto issue_block = [&](uint32_t lb) -> bool {
                if (!mbar_wait_timed(BAR_LEMPTY + 8 * ls, lph ^ 1u, abort_flag, STATUS_WAIT_EXPIRED_DEQUANT, prof, w_lempty)) return false;
                const long long t_i0 = prof ? clock64() : 0;
                const uint32_t base = x_tile0 + ls * C::L_BLOCK;
                const uint32_t ng = min(4u, n_gran - lb * 4);
                // the block's ninth arrival comes from the TMA producer when it fetches B_s, else from here
                if (td == 0 && leader && !p.b_pool_strided) mbar_arrive(BAR_LFULL + 8 * ls);
                if (!p.b_pool_strided)
#pragma unroll
                for (uint32_t g = 0; g < 4; ++g) {
                    if (g < ng) {
                        const uint32_t j0 = (gran[lb * 4 + g] & 3u) * 16u;
                        if (td < 256u) {
                            const bool live = f < p.N && j0 + 8 * a_h < p.max_rank;
                            const uint16_t* src = live ? reinterpret_cast<const uint16_t*>(gran_b[lb * 4 + g]) + a_src_off + j0 : p.t;
                            cp_async_16_zfill(base + g * C::L_GRAN_A + a_dst, src, live ? 16u : 0u);
                        }
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < T_TASKS; ++u) {
                    const int32_t d = int32_t(lb * 4) - t_pos[u];        // granule of the row's slot that block lb starts with
#pragma unroll
                    for (int32_t g = 0; g < 4; ++g) {
                        const uint32_t k = uint32_t(d + g);
                        if (k < t_ng[u]) cp_async_16_zfill(base + g * C::L_GRAN_T + t_dst[u], t_src[u] + 16 * k, 16u);
                        else if (uint32_t(d + g - 4 * C::L_STAGES * int32_t(ks)) < t_ng[u]) sts128(base + g * C::L_GRAN_T + t_dst[u], 0u, 0u, 0u, 0u);
                    }
                }
                if (++ls == uint32_t(C::L_STAGES)) { ls = 0; lph ^= 1u; }
                if (prof) w_issue += (unsigned long long)(clock64() - t_i0);
                return true;
            };
            // one cp.async group per block, issued L_STAGES - 1 blocks ahead (empty groups past the end
            // keep "group index == block index")
            // (this CTA's blocks are kz, kz + ks, ...: local block i is block kz + i * ks of the tile)
            for (uint32_t i = 0; ok && i + 1 < uint32_t(C::L_STAGES); ++i) {
                if (kz + i * ks < n_lb) ok = issue_block(kz + i * ks);
                cp_async_commit();
            }
            // Hand block lb over first, refill afterwards: the refill waits for the MMA to release a
            // stage, and must not stand between finished copies and the MMA that is waiting for them.
            uint32_t cs = 0;
            for (uint32_t i = 0; ok && kz + i * ks < n_lb; ++i) {
                const long long t_g0 = prof ? clock64() : 0;
                cp_async_wait_group<C::L_STAGES - 2>();      // groups 0 .. lb + L_STAGES - 2 are committed: lb is done
                if (prof) w_group += (unsigned long long)(clock64() - t_g0);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) arrive_at_leader(lfull_at_leader + 8 * cs);
                if (++cs == uint32_t(C::L_STAGES)) cs = 0;
                if (kz + (i + C::L_STAGES - 1) * ks < n_lb) ok = issue_block(kz + (i + C::L_STAGES - 1) * ks);
                cp_async_commit();
            }
            cp_async_wait_group<0>();
            if (prof && td == 0) { prof_row[10] = w_lempty; prof_row[11] = w_issue; prof_row[12] = w_group; prof_row[13] = n_lb; }
        }
        if (prof && td == 0) prof_row[6] = (unsigned long long)(clock64() - t_lora);

        // ---- join the epilogue ----
        if (ok && mbar_wait(BAR_ACC, 0, abort_flag, STATUS_WAIT_EXPIRED_EPILOGUE, 64)) {
            tcgen05_fence_after();
            if (ks > 1) acc_ready = true;
            else if (p.staged_epilogue) epilogue_staged<MT>(p, tmem_acc, x_tile0, BAR_EPI, abort_flag, q, lane, f0, m0, 1 + ((warp - DEQ_WARP0) >> 2), 1 + DEQ_WARPS / 4, EPI_THREADS + td);
            else epilogue_columns<MT>(p, tmem_acc, q, lane, f0, m0, 1 + ((warp - DEQ_WARP0) >> 2), 1 + DEQ_WARPS / 4);
        }
    }

    // ================================ split K: the cluster finishes the tile =================================
    if (ks > 1) {
        tcgen05_fence_before();
        __syncwarp();
        cluster_sync_all();                                  // every CTA's MMAs are done: staging areas may receive
        tcgen05_fence_after();
        if (warp >= EPI_WARP0) {
            const uint32_t part = warp < DEQ_WARP0 ? 0u : 1u + ((warp - DEQ_WARP0) >> 2);
            if (acc_ready) split_send<MT>(tmem_acc, x_tile0, ks, kz, cta_rank, CTAS, warp & 3u, lane, part, 1 + DEQ_WARPS / 4);
        }
        __syncwarp();
        cluster_sync_all();                                  // all partial tiles have arrived
        if (warp >= EPI_WARP0 && acc_ready) split_reduce_store<MT>(p, x_tile0, ks, kz, f0, m0, tid - EPI_WARP0 * 32);
    }

    // ========================================= teardown ==========================================
    if (*abort_flag) {
        // give copies that may still be in flight time to land before shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tcgen05_fence_before();
    __syncwarp();
    // (pair: the other CTA's MMAs read this CTA's shared and tensor memory, and its warps arrive on this CTA's barriers)
    if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_acc, C::TMEM_COLS); else tmem_dealloc(tmem_acc, C::TMEM_COLS);
        if (prof && lane == 0) { prof_row[1] = (unsigned long long)(clock64() - t_entry); prof_row[8] = t_entry_ns; prof_row[9] = global_timer_ns(); }
    }
}

}  // namespace tc
}  // namespace atlas
