// Shared device helpers: BF16 packing, the NVFP4 codecs, the device status word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace atlas {

// ---- device status word -------------------------------------------------------------------
// First problem recorded by any kernel since the last clear (0 = clean).  Kernels never trap:
// they record a code here and carry on in a defined way (treat the row as un-adapted, or
// leave the tile unwritten after a wait that expired).
enum : uint32_t {
    STATUS_OK = 0,
    STATUS_SLOT_OUT_OF_RANGE = 1,   // seq_slot[i] >= max_loras
    STATUS_NEGATIVE_SCALE = 2,      // FP4-activation mode met a weight scale byte with its sign bit set; the sign was dropped
    STATUS_TILE_CAPACITY = 3,       // the shrink met more (slot, granule) pairs in a token tile than its tile output reserves
    STATUS_WAIT_EXPIRED_PRODUCER = 0x100,
    STATUS_WAIT_EXPIRED_DEQUANT = 0x101,
    STATUS_WAIT_EXPIRED_MMA = 0x102,
    STATUS_WAIT_EXPIRED_EPILOGUE = 0x103,
};

__device__ uint32_t g_status_word = 0;

__device__ __forceinline__ void record_status(uint32_t code) { atomicCAS(&g_status_word, 0u, code); }

// ---- BF16 <-> FP32 ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);               // one conversion for the pair, each rounded to nearest even
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ---- E2M1 / E4M3, scalar forms (bit-for-bit the arithmetic of
//      kernels/gb10/common/dequant_nvfp4_bf16.cu:26-46) ---------------------------------------
__device__ __forceinline__ float e2m1_decode(uint32_t nib) {
    // magnitude = {0, .5, 1, 1.5, 2, 3, 4, 6}[nib & 7], bit 3 = sign
    const uint32_t m = nib & 7u;
    // FP32 bits with (m << 22) are 2^(e-127)*(1+mant/2) for e>0 and a subnormal for e==0;
    // multiplying by 2^126 gives the E2M1 value exactly in both cases.
    float v = __uint_as_float(m << 22) * 8.507059173023462e37f;   // 2^126
    return (nib & 8u) ? -v : v;
}

__device__ __forceinline__ float e4m3_decode(uint32_t b) {
    const uint32_t e = (b >> 3) & 0xFu, m = b & 0x7u;
    float v;
    if (e == 0u) v = float(m) * 0.001953125f;
    else if (e == 15u && m == 7u) v = 0.0f;               // the NaN byte decodes to 0
    else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -v : v;
}

// ---- packed BF16x2 multiply (subnormal inputs are honoured: no .ftz) ------------------------
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// E4M3 scale byte -> BF16x2 {f, f} with f = e4m3(byte) * 2^118.
// (byte & 0x7F) << 4 read as BF16 is e4m3 * 2^-120 for normals and subnormals alike.
__device__ __forceinline__ uint32_t e4m3_to_bf16x2_shifted(uint32_t byte) {
    const uint32_t mag = byte & 0x7Fu;
    uint32_t bits = (mag == 0x7Fu) ? 0u : (mag << 4);
    bits |= (byte & 0x80u) << 8;
    uint32_t v = bits | (bits << 16);
    v = bf16x2_mul(v, 0x7B807B80u);   // * 2^120 : exact E4M3 value
    v = bf16x2_mul(v, 0x7A807A80u);   // * 2^118
    return v;
}

// Eight E2M1 codes (element i in bits [4i, 4i+4)) times a BF16x2 multiplier {f, f}
// -> eight BF16 values in element order, as four BF16x2 words.
// With f = scale * 2^118 each output is E2M1 * scale * 2^-8, exact in BF16 (<= 6 significant bits).
__device__ __forceinline__ void e2m1x8_to_bf16x8(uint32_t p, uint32_t mul, uint32_t (&out)[4]) {
    // pair i holds elements (i, i+4): sign to bit 15/31, 3 magnitude bits to bits 6..8 / 22..24
    // (BF16 exponent lsbs + mantissa msb), i.e. value * 2^-126.
    const uint32_t b0 = ((p << 12) & 0x80008000u) | ((p << 6) & 0x01C001C0u);
    const uint32_t b1 = ((p << 8) & 0x80008000u) | ((p << 2) & 0x01C001C0u);
    const uint32_t b2 = ((p << 4) & 0x80008000u) | ((p >> 2) & 0x01C001C0u);
    const uint32_t b3 = (p & 0x80008000u) | ((p >> 6) & 0x01C001C0u);
    const uint32_t h0 = bf16x2_mul(b0, mul), h1 = bf16x2_mul(b1, mul);
    const uint32_t h2 = bf16x2_mul(b2, mul), h3 = bf16x2_mul(b3, mul);
    out[0] = __byte_perm(h0, h1, 0x5410);   // (e0, e1)
    out[1] = __byte_perm(h2, h3, 0x5410);   // (e2, e3)
    out[2] = __byte_perm(h0, h1, 0x7632);   // (e4, e5)
    out[3] = __byte_perm(h2, h3, 0x7632);   // (e6, e7)
}

constexpr float kWeightPreScale = 256.0f;   // 2^8: weights enter the MMA as value * 2^-8

}  // namespace atlas
