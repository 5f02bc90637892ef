// Tensor-core LoRA shrink:  t[m, j] = f(s) * sum_k x[m,k] * A_s[j,k],  s = seq_slot[m].
//
// A CLUSTER of 1..SHM_KSPLIT CTAs (4 warps each; ShrinkParams::ksplit, chosen at launch) owns (adapter slot s, 16
// consecutive ranks = one granule of the fused layer, a chunk of tokens = that layer's token tile).  Every CTA
// scans the chunk's seq_slot entries for the rows routed to s and walks them 32 at a time.  K is split in
// interleaved 32-element chunks over the cluster's CTAs and their warps (the op is bound by memory latency, so
// what matters is how many loads are in flight); each warp multiplies its chunks with mma.sync.m16n8k16 (BF16
// in, FP32 accumulate), a CTA adds its four partial tiles in shared memory, and the cluster's first CTA adds
// the CTAs' tiles over distributed shared memory — always in the same order, so results do not depend on timing.
//
// The result goes either to rows of t [M, max_rank], or (ShrinkParams::tile_out) to complete masked blocks in
// the layout the fused kernel's MMA reads, see ShrinkParams.
//
// Operand fragments are loaded straight from global memory with 128-bit loads: the thread with
// (group g, quad lane t) reads 8 consecutive K elements at k = 32*chunk + 8*t of row g (and g+8) of
// x, and of row g of A_s.  Elements 0..3 feed one MMA, 4..7 the next; x and A_s use the same
// assignment, so each K element meets its partner and every 32-byte sector fetched is used in full.
//
// A CTA is small on purpose (128 threads, well under 64 registers): in the fused layer this grid runs
// next to the tcgen05 kernel's CTAs on the same SMs (programmatic dependent launch), and must fit in
// what that kernel leaves free.
//
// Output rounding, rank handling and the uniform mode are those of lora_shrink_grouped_kernel, which
// remains the path for shapes this kernel does not take (K not a multiple of 32, unaligned rows).
#pragma once

#include <cooperative_groups.h>

#include "kernels_simt.cuh"

namespace atlas {
namespace cg = cooperative_groups;

constexpr int SHM_THREADS = 128;
constexpr int SHM_RANKS = 16;     // ranks per CTA (two n-tiles of 8)
constexpr int SHM_TOKENS = 32;    // tokens per pass (two m-tiles of 16)
constexpr int SHM_CHUNK = 256;    // tokens scanned per CTA
constexpr int SHM_KSPLIT = 8;     // CTAs per cluster, splitting K, at most (the launch picks 1, 2, 4 or 8: ShrinkParams::ksplit)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(SHM_THREADS, 8)
lora_shrink_mma_kernel(const ShrinkParams p) {
    __shared__ uint16_t rows[SHM_CHUNK];
    __shared__ float part[SHM_TOKENS][SHM_RANKS];          // this CTA's tile, read by the cluster's first CTA

    if (p.release_dependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t krank = cluster.block_rank();            // this CTA's share of K
    const uint32_t ksplit = p.ksplit;                       // = the cluster's size
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s = blockIdx.x / ksplit;
    const uint32_t j0 = blockIdx.y * SHM_RANKS;
    const uint32_t chunk = p.chunk ? p.chunk : uint32_t(SHM_CHUNK);
    const uint32_t m_base = blockIdx.z * chunk;

    const uint16_t* A;
    float f = 1.0f;
    uint32_t rank = p.max_rank;
    if (p.seq_slot) {
        const uint64_t a_addr = p.a_table[s];
        if (a_addr == 0ull) return;
        if (p.b_table && p.b_table[s] == 0ull) return;
        A = reinterpret_cast<const uint16_t*>(a_addr);
        if (p.rank_table) rank = min(p.rank_table[s], p.max_rank);
        if (p.tile_out && j0 >= rank) return;               // no such granule in any tile's list (whole cluster leaves)
        if (p.post != 0.0f) f = p.scale_table[s] * p.post;
    } else {
        A = p.a_uniform;
    }

    // ---- ordered list of this chunk's rows routed to slot s (two candidates per thread) ----
    uint32_t n_rows;
    bool hit[2];
    {
        uint32_t ballot[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t m = m_base + h * SHM_THREADS + tid;
            hit[h] = (h * SHM_THREADS + tid < chunk) && (m < p.M) && (p.seq_slot ? (p.seq_slot[m] == int32_t(s)) : true);
            ballot[h] = __ballot_sync(0xFFFFFFFFu, hit[h]);
        }
        __shared__ uint32_t cnt[2][SHM_THREADS / 32];
        if (lane == 0) { cnt[0][warp] = __popc(ballot[0]); cnt[1][warp] = __popc(ballot[1]); }
        __syncthreads();
        uint32_t total = 0, before[2] = {0, 0};
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int w = 0; w < SHM_THREADS / 32; ++w) {
                if (h == 0 && w < int(warp)) before[0] += cnt[0][w];
                if (h == 1) { if (w < int(warp)) before[1] += cnt[1][w]; }
                total += cnt[h][w];
            }
        uint32_t first_half = 0;
#pragma unroll
        for (int w = 0; w < SHM_THREADS / 32; ++w) first_half += cnt[0][w];
        if (hit[0]) rows[before[0] + __popc(ballot[0] & ((1u << lane) - 1u))] = uint16_t(tid);
        if (hit[1]) rows[first_half + before[1] + __popc(ballot[1] & ((1u << lane) - 1u))] = uint16_t(SHM_THREADS + tid);
        n_rows = total;
        __syncthreads();
    }
    if (n_rows == 0) return;

    // ranks at or beyond the adapter's true rank are written as zeros and never read
    const bool any_live = j0 < rank;

    // ---- tile output: where this (slot, granule) pair's block goes, and its zero rows ----
    uint16_t* tile = nullptr;
    if (p.tile_out) {
        if (!any_live) return;                               // the pair is not in the tile's list (whole cluster leaves)
        if (krank == 0) {
            // pairs ahead of this one: every granule of every valid slot below s that occurs in the tile
            __shared__ uint32_t present[SHM_THREADS];        // one bit per slot, 32 * 128 = 4096 slots
            __shared__ uint32_t ahead[SHM_THREADS / 32];
            present[tid] = 0u;
            __syncthreads();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t idx = h * SHM_THREADS + tid, m = m_base + idx;
                if (idx < chunk && m < p.M) {
                    const int32_t s2 = p.seq_slot[m];
                    if (s2 >= 0 && uint32_t(s2) < s && p.a_table[s2] != 0ull && (!p.b_table || p.b_table[s2] != 0ull))
                        atomicOr(&present[uint32_t(s2) >> 5], 1u << (uint32_t(s2) & 31u));
                }
            }
            __syncthreads();
            uint32_t cnt = 0;
            for (uint32_t w = present[tid]; w; w &= w - 1) {
                const uint32_t s2 = tid * 32 + (__ffs(w) - 1);
                const uint32_t r2 = p.rank_table ? min(p.rank_table[s2], p.max_rank) : p.max_rank;
                cnt += (r2 + 15u) / 16u;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xFFFFFFFFu, cnt, o);
            if (lane == 0) ahead[warp] = cnt;
            __syncthreads();
            const uint32_t q = ahead[0] + ahead[1] + ahead[2] + ahead[3] + blockIdx.y;
            if (q < p.tile_cap) {
                // part 0's block of this pair; part 1's lies tile_cap blocks further on
                tile = p.tile_out + (size_t(blockIdx.z) * (chunk / p.part_rows) * p.tile_cap + q) * p.part_rows * 16;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t idx = h * SHM_THREADS + tid;
                    if (idx < chunk && !hit[h]) {
                        const uint32_t part = idx / p.part_rows, r = idx % p.part_rows;
                        uint4* z = reinterpret_cast<uint4*>(tile + (size_t(part) * p.tile_cap * p.part_rows + r) * 16);
                        z[0] = make_uint4(0u, 0u, 0u, 0u);
                        z[1] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            } else {
                record_status(STATUS_TILE_CAPACITY);         // cannot happen with a capacity computed as documented
            }
        }
    }
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t n_chunks = p.k_in / 32;
    const bool a_aligned = (reinterpret_cast<uintptr_t>(A) & 15u) == 0;

    for (uint32_t r0 = 0; r0 < n_rows; r0 += SHM_TOKENS) {
        float acc[2][2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;

        if (any_live) {
            // x rows of this thread's fragment positions (clamped: surplus rows are dropped at the store)
            const uint16_t* xr[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t idx = min(r0 + mt * 16 + h * 8 + g, n_rows - 1);
                    xr[mt][h] = p.x + size_t(m_base + rows[idx]) * p.x_row_stride + 8 * t;
                }
            // A_s rows of the two n-tiles (clamped to a valid row; dead ranks are zeroed at the store)
            const uint16_t* ar[2];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) ar[nt] = A + size_t(min(j0 + nt * 8 + g, p.max_rank - 1)) * p.k_in + 8 * t;

#pragma unroll 2
            for (uint32_t c = krank + ksplit * warp; c < n_chunks; c += ksplit * (SHM_THREADS / 32)) {
                uint4 xv[2][2], av[2];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int h = 0; h < 2; ++h) xv[mt][h] = *reinterpret_cast<const uint4*>(xr[mt][h] + c * 32);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    if (a_aligned) av[nt] = __ldg(reinterpret_cast<const uint4*>(ar[nt] + c * 32));
                    else {
                        const uint32_t* q = reinterpret_cast<const uint32_t*>(ar[nt] + c * 32);   // 4-byte aligned at least
                        av[nt] = make_uint4(__ldg(q), __ldg(q + 1), __ldg(q + 2), __ldg(q + 3));
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        mma_bf16_16816(acc[mt][nt], xv[mt][0].x, xv[mt][1].x, xv[mt][0].y, xv[mt][1].y, av[nt].x, av[nt].y);
                        mma_bf16_16816(acc[mt][nt], xv[mt][0].z, xv[mt][1].z, xv[mt][0].w, xv[mt][1].w, av[nt].z, av[nt].w);
                    }
            }
        }
        // ---- add the four warps' partial tiles in warp order (little shared memory: this grid shares
        //      its SMs with a kernel that leaves only a few KB free) ----
#pragma unroll 1
        for (uint32_t w = 0; w < SHM_THREADS / 32; ++w) {
            if (warp == w) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        float* r_lo = &part[mt * 16 + g][nt * 8 + 2 * t];
                        float* r_hi = &part[mt * 16 + g + 8][nt * 8 + 2 * t];
                        if (w == 0) {
                            r_lo[0] = acc[mt][nt][0]; r_lo[1] = acc[mt][nt][1]; r_hi[0] = acc[mt][nt][2]; r_hi[1] = acc[mt][nt][3];
                        } else {
                            r_lo[0] += acc[mt][nt][0]; r_lo[1] += acc[mt][nt][1]; r_hi[0] += acc[mt][nt][2]; r_hi[1] += acc[mt][nt][3];
                        }
                    }
            }
            __syncthreads();
        }
        cluster.sync();                                      // every CTA's tile is in its shared memory
        if (krank == 0) {
            for (uint32_t i = tid; i < SHM_TOKENS * SHM_RANKS; i += SHM_THREADS) {
                const uint32_t tok = i / SHM_RANKS, jr = i % SHM_RANKS;
                if (r0 + tok < n_rows && (p.tile_out || j0 + jr < p.max_rank)) {
                    float v = 0.0f;
                    for (uint32_t r = 0; r < ksplit; ++r) v += cluster.map_shared_rank(&part[0][0], r)[i];
                    const uint16_t bits = f32_to_bf16_bits((j0 + jr < rank) ? v * f : 0.0f);
                    if (p.tile_out) {
                        if (tile) {
                            const uint32_t idx = rows[r0 + tok], part = idx / p.part_rows, r = idx % p.part_rows;
                            tile[(size_t(part) * p.tile_cap * p.part_rows + r) * 16 + (((jr >> 3) ^ ((r >> 2) & 1u)) << 3) + (jr & 7u)] = bits;
                        }
                    }
                    else p.out[size_t(m_base + rows[r0 + tok]) * p.max_rank + j0 + jr] = bits;
                }
            }
        }
        cluster.sync();                                      // tiles stay alive until they have been read
    }
}

}  // namespace atlas
