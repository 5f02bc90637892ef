// The memory-bound steps either side of the MLP's linears, and the weight quantiser's first phase:
//   nvfp4_global_absmax_kernel   max |x| of a BF16 tensor (kernels/gb10/common/quantize_bf16_to_nvfp4.cu:131-167)
//   silu_mul_kernel              h = SiLU(min(g, L)) * clamp(u, -L, L), BF16 -> BF16, with or without the swiglu limit
//                                (kernels/gb10/common/moe_silu_mul.cu:14-54)
//   silu_mul_quant_nvfp4_kernel  the same h, quantised straight to NVFP4 in the activation layout of the FP4-activation
//                                mode (packed codes [M, K/2], scale bytes [M, K/16]) so that the BF16 h never exists in
//                                HBM — the fusion crates/spark-model/src/layers/ops/nvfp4_mmq.rs:126-157 performs for its
//                                own down arm; quantiser arithmetic is that of quantize_bf16_to_nvfp4.cu:176-243
//                                (group of 16, E4M3(max / 6) through the software encoder, tensor scale 1).
// All three stream their inputs once with 128-bit loads; grids are sized as a multiple of the SM count.
#pragma once

#include "kernels_simt.cuh"

namespace atlas {

__global__ void __launch_bounds__(256)
nvfp4_global_absmax_kernel(const uint16_t* __restrict__ in, float* __restrict__ global_max, size_t total) {
    float local = 0.0f;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t vecs = ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) ? total / 8 : 0;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += stride) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(in) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) local = fmaxf(local, fmaxf(fabsf(bf16_lo(w[k])), fabsf(bf16_hi(w[k]))));
    }
    for (size_t i = vecs * 8 + size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
        local = fmaxf(local, fabsf(__uint_as_float(uint32_t(in[i]) << 16)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xFFFFFFFFu, local, o));
    __shared__ float warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.0f;
        for (int w = 0; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        // non-negative floats order like their bit patterns
        atomicMax(reinterpret_cast<unsigned int*>(global_max), __float_as_uint(m));
    }
}

__device__ __forceinline__ float swiglu(float g, float u, float limit) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return g * (1.0f / (1.0f + __expf(-g))) * u;
}

// rows of gate / up / out may be spaced wider than K (column segments of wider buffers); strides in elements, multiples of 8
__global__ void __launch_bounds__(256)
silu_mul_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up, uint16_t* __restrict__ out, float gate_scale,
                float up_scale, float limit, uint32_t M, uint32_t K, uint32_t in_stride, uint32_t out_stride) {
    const size_t per_row = K / 8, total = size_t(M) * per_row;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const size_t row = i / per_row, c = (i % per_row) * 8;
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate + row * in_stride + c));
        const uint4 uv = __ldg(reinterpret_cast<const uint4*>(up + row * in_stride + c));
        const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w}, u[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            o[k] = pack_bf16x2(swiglu(bf16_lo(g[k]) * gate_scale, bf16_lo(u[k]) * up_scale, limit),
                               swiglu(bf16_hi(g[k]) * gate_scale, bf16_hi(u[k]) * up_scale, limit));
        *reinterpret_cast<uint4*>(out + row * out_stride + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// one thread per group of 16: codes [M, K/2] and scale bytes [M, K/16], both dense
__global__ void __launch_bounds__(256)
silu_mul_quant_nvfp4_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up, uint8_t* __restrict__ packed,
                            uint8_t* __restrict__ scales, float gate_scale, float up_scale, float limit, uint32_t M, uint32_t K,
                            uint32_t in_stride) {
    const size_t groups = K / 16, total = size_t(M) * groups;
    for (size_t gi = size_t(blockIdx.x) * blockDim.x + threadIdx.x; gi < total; gi += size_t(gridDim.x) * blockDim.x) {
        const size_t row = gi / groups, c = (gi % groups) * 16;
        const uint4* gp = reinterpret_cast<const uint4*>(gate + row * in_stride + c);
        const uint4* up4 = reinterpret_cast<const uint4*>(up + row * in_stride + c);
        const uint4 g0 = __ldg(gp), g1 = __ldg(gp + 1), u0 = __ldg(up4), u1 = __ldg(up4 + 1);
        const uint32_t g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const uint32_t u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float v[16];
        float gmax = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            v[2 * k] = swiglu(bf16_lo(g[k]) * gate_scale, bf16_lo(u[k]) * up_scale, limit);
            v[2 * k + 1] = swiglu(bf16_hi(g[k]) * gate_scale, bf16_hi(u[k]) * up_scale, limit);
            gmax = fmaxf(gmax, fmaxf(fabsf(v[2 * k]), fabsf(v[2 * k + 1])));
        }
        // the activation quantiser of the FP4-activation mode: tensor scale 1, scale byte = E4M3(group max / 6)
        const float f8 = gmax > 0.0f ? __fdiv_rn(gmax, 6.0f) : 0.0f;
        const uint32_t byte = e4m3_encode_sw(f8);
        scales[gi] = uint8_t(byte);
        const float eff = e4m3_decode(byte);
        const float inv_eff = eff > 0.0f ? __fdiv_rn(1.0f, eff) : 0.0f;
        uint32_t q[2] = {0u, 0u};
#pragma unroll
        for (int k = 0; k < 16; ++k) q[k / 8] |= e2m1_quantize(__fmul_rn(v[k], inv_eff)) << (4 * (k % 8));
        *reinterpret_cast<uint2*>(packed + gi * 8) = make_uint2(q[0], q[1]);
    }
}

}  // namespace atlas
