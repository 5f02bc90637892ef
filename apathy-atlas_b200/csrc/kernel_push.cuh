// Column-block push for column-parallel tensor parallelism: this rank's [m, n_cols] BF16 result block, already in its
// own gathered row-major buffer, is copied into the same columns of every peer's gathered buffer (peer memory mapped
// into this process), each 16-byte chunk read once and stored n_dest times with plain stores over NVLink.
//
// The fused kernels can store their tiles into the peers themselves (n_dest > 1); when a rank's share of a projection
// is a single wave of tiles, those stores all happen at the end of the one wave and nothing is left to hide them
// behind.  This kernel is the other way to overlap: it is small (128 threads, no shared memory), so its CTAs are
// resident next to the CTAs of the NEXT projection's kernels, and it runs on a second stream while they compute.
// It replaces the all-gather that follows a column-parallel linear in the reference
// (crates/spark-comm/src/nccl_backend/comm_impl.rs:130-145).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace atlas {

constexpr int PUSH_THREADS = 128;
constexpr int PUSH_MAX_DEST = 8;

struct PushParams {
    const uint4* src;               // first chunk of the block in the source buffer
    uint4* dst[PUSH_MAX_DEST];      // first chunk of the block in each destination buffer
    uint32_t n_dest;
    uint32_t m, chunks_per_row;     // rows, 16-byte chunks per row of the block
    uint32_t src_row_chunks;        // row strides in 16-byte chunks
    uint32_t dst_row_chunks;
};

// (at most 40 registers: a CTA must fit beside a 608-thread, 96-register CTA of the persistent kernel)
__global__ void __launch_bounds__(PUSH_THREADS, 12)
push_columns_kernel(const PushParams p) {
    const uint64_t total = uint64_t(p.m) * p.chunks_per_row;
    const uint64_t stride = uint64_t(gridDim.x) * PUSH_THREADS;
    uint64_t i = uint64_t(blockIdx.x) * PUSH_THREADS + threadIdx.x;
    // four chunks in flight per thread
    for (; i + 3 * stride < total; i += 4 * stride) {
        uint4 v[4];
        uint64_t at[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t j = i + u * stride;
            const uint32_t r = uint32_t(j / p.chunks_per_row), c = uint32_t(j - uint64_t(r) * p.chunks_per_row);
            v[u] = p.src[uint64_t(r) * p.src_row_chunks + c];
            at[u] = uint64_t(r) * p.dst_row_chunks + c;
        }
#pragma unroll
        for (int d = 0; d < PUSH_MAX_DEST; ++d) {            // (constant indices: the addresses stay in the parameter bank)
            if (uint32_t(d) < p.n_dest) {
#pragma unroll
                for (int u = 0; u < 4; ++u) p.dst[d][at[u]] = v[u];
            }
        }
    }
    for (; i < total; i += stride) {
        const uint32_t r = uint32_t(i / p.chunks_per_row), c = uint32_t(i - uint64_t(r) * p.chunks_per_row);
        const uint4 v = p.src[uint64_t(r) * p.src_row_chunks + c];
#pragma unroll
        for (int d = 0; d < PUSH_MAX_DEST; ++d)
            if (uint32_t(d) < p.n_dest) p.dst[d][uint64_t(r) * p.dst_row_chunks + c] = v;
    }
}

}  // namespace atlas
