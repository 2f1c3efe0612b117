// Block-fixed-point activation planes and the integer block dot product shared by the matrix-vector kernels.
#pragma once

#include "common.cuh"
#include "internal.h"

namespace tb {

// The three byte planes (signed high, unsigned middle and low) of 32 activations, and 2^(e-21): x ~ X * mul with
// X = hi*65536 + mid*256 + lo, |X| <= 2^22.
struct Planes {
    uint32_t hi[8], mid[8], lo[8];
    float mul;
};

__device__ __forceinline__ uint32_t pack_bytes(int x0, int x1, int x2, int x3, uint32_t sel) {
    return __byte_perm(__byte_perm(x0, x1, sel), __byte_perm(x2, x3, sel), 0x5410);
}

// The dot product of 32 weights (two 16-byte chunks, in the order of the planes' words) with a block's planes, as a
// float holding the exact integer sum rounded once.
__device__ __forceinline__ float block_dot(const uint4& a, const uint4& b, const Planes& p) {
    int h = 0, m = 0, l = 0;
    h = dp4a_ss(a.x, p.hi[0], h), m = dp4a_su(a.x, p.mid[0], m), l = dp4a_su(a.x, p.lo[0], l);
    h = dp4a_ss(a.y, p.hi[1], h), m = dp4a_su(a.y, p.mid[1], m), l = dp4a_su(a.y, p.lo[1], l);
    h = dp4a_ss(a.z, p.hi[2], h), m = dp4a_su(a.z, p.mid[2], m), l = dp4a_su(a.z, p.lo[2], l);
    h = dp4a_ss(a.w, p.hi[3], h), m = dp4a_su(a.w, p.mid[3], m), l = dp4a_su(a.w, p.lo[3], l);
    h = dp4a_ss(b.x, p.hi[4], h), m = dp4a_su(b.x, p.mid[4], m), l = dp4a_su(b.x, p.lo[4], l);
    h = dp4a_ss(b.y, p.hi[5], h), m = dp4a_su(b.y, p.mid[5], m), l = dp4a_su(b.y, p.lo[5], l);
    h = dp4a_ss(b.z, p.hi[6], h), m = dp4a_su(b.z, p.mid[6], m), l = dp4a_su(b.z, p.lo[6], l);
    h = dp4a_ss(b.w, p.hi[7], h), m = dp4a_su(b.w, p.mid[7], m), l = dp4a_su(b.w, p.lo[7], l);
    return fmaf(static_cast<float>(h), 65536.0f, static_cast<float>(m * 256 + l));
}

// The same for 32 four-bit weights n - 8 (crates/tachyon/src/quant.rs:60-66: word j holds columns 8j..8j+3 in its low
// nibbles and 8j+4..8j+7 in its high ones): sum n X - 8 sum X, with `sx` the block's sum of X.
__device__ __forceinline__ float block_dot_q4(const uint4& w, const Planes& p, float sx) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    int h = 0;
    uint32_t m = 0, l = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t lo = ww[j] & 0x0F0F0F0Fu, hi = (ww[j] >> 4) & 0x0F0F0F0Fu;
        h = dp4a_su(p.hi[2 * j], lo, h), m = dp4a_uu(p.mid[2 * j], lo, m), l = dp4a_uu(p.lo[2 * j], lo, l);
        h = dp4a_su(p.hi[2 * j + 1], hi, h), m = dp4a_uu(p.mid[2 * j + 1], hi, m), l = dp4a_uu(p.lo[2 * j + 1], hi, l);
    }
    return fmaf(-8.0f, sx, fmaf(static_cast<float>(h), 65536.0f, static_cast<float>(m * 256u + l)));
}

// Sum of a block's 32 fixed-point activations, as a float.
__device__ __forceinline__ float plane_sum(const Planes& p) {
    int h = 0;
    uint32_t m = 0, l = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) h = dp4a_ss(p.hi[k], 0x01010101, h), m = dp4a_uu(p.mid[k], 0x01010101u, m), l = dp4a_uu(p.lo[k], 0x01010101u, l);
    return fmaf(static_cast<float>(h), 65536.0f, static_cast<float>(m * 256u + l));
}

// Used by the generic kernel: planes of 32 values held by one thread.
__device__ __forceinline__ void make_planes(const float (&v)[32], Planes& p) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(v[j]));
    uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);  // biased exponent of the largest magnitude
    const bool zero = eb < 22u;                            // below 2^-105: the block counts as zero
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);  // 2^(21 - e)
    p.mul = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);           // 2^(e - 21)
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int x0 = __float2int_rn(v[4 * k] * sc), x1 = __float2int_rn(v[4 * k + 1] * sc);
        const int x2 = __float2int_rn(v[4 * k + 2] * sc), x3 = __float2int_rn(v[4 * k + 3] * sc);
        p.hi[k] = pack_bytes(x0, x1, x2, x3, 0x0062);
        p.mid[k] = pack_bytes(x0, x1, x2, x3, 0x0051);
        p.lo[k] = pack_bytes(x0, x1, x2, x3, 0x0040);
    }
}

__device__ __forceinline__ void load32_f32(const float* base, float (&v)[32]) {
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float4 t = ld_cg_f4(base + 4 * k);
        v[4 * k] = t.x, v[4 * k + 1] = t.y, v[4 * k + 2] = t.z, v[4 * k + 3] = t.w;
    }
}

__device__ __forceinline__ void load32_f16(const __half* base, float (&v)[32]) {
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint4 t = ld_cg_u4(base + 8 * k);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[8 * k + 2 * j] = f.x, v[8 * k + 2 * j + 1] = f.y;
        }
    }
}

}  // namespace tb
