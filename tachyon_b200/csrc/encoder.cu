// The packed variable-length encoder (ModernBERT shape): kernels and host object.  Counterpart of
// crates/tachyon/src/encoder/run.rs (layers 413-447, batches/tiles 207-221 and 354-373, embeddings 161-175) and of the
// kernels in crates/tachyon/src/ptx/encoder.rs: embed_f16 + norm_f16 (582-668, 761-805), rope_f16 (893-959),
// attend_f16 (961-1215), with the products on the tcgen05 GEMM (gemm.cu; its store modes replace ptx/encoder.rs:418-492).
//
// Sequences are packed back to back without padding: activations are [tokens, width]; attention works per sequence
// through a list of 64-query tiles.  Weights are Q8 (int8 codes + f16 scale per 32) or f16, the embedding table f16; a
// converted model's Q8E matrices (codes + an f32 scale per 64, crates/tachyon/src/quant.rs:107-115) load into the former.
// A batch runs padded to whole tiles of 64 tokens as a CUDA graph recorded once per padded shape (run.rs:379-410).
#include "../../include/tachyon_b200.h"
#include "common.cuh"
#include "internal.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace tb {

namespace {

// ---- layer norm without bias, one block per token -----------------------------------------------------------------------
// y = (x - mean) / sqrt(var + eps) * w.  `ids` given: x is row ids[token] of the f16 table (embedding + its norm).
// Outputs: f32 (optional) and f16 (optional).
__global__ void __launch_bounds__(256) enc_norm_kernel(const float* x, const __half* table, const uint32_t* ids, const float* w, uint32_t h, float eps,
                                                       float* out32, __half* out16) {
    __shared__ float sh[8];
    const uint32_t t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto block_sum = [&](float v) {
        v = warp_sum(v);
        __syncthreads();
        if (lane == 0) sh[warp] = v;
        __syncthreads();
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) s += sh[i];
        return s;
    };
    float v[8];  // h <= 2048
    int cnt = 0;
    float sum = 0.0f;
    for (uint32_t i = tid; i < h; i += 256, cnt++) {
        v[cnt] = ids ? __half2float(table[(size_t)ids[t] * h + i]) : x[(size_t)t * h + i];
        sum += v[cnt];
    }
    const float mean = block_sum(sum) / (float)h;
    float var = 0.0f;
    for (int c = 0; c < cnt; c++) var = fmaf(v[c] - mean, v[c] - mean, var);
    const float rs = rsqrtf(block_sum(var) / (float)h + eps);
    cnt = 0;
    for (uint32_t i = tid; i < h; i += 256, cnt++) {
        const float y = (v[cnt] - mean) * rs * __ldg(w + i);
        if (out32) out32[(size_t)t * h + i] = y;
        if (out16) out16[(size_t)t * h + i] = __float2half_rn(y);
    }
}

// LayerNorm with one warp per token for widths that are multiples of 128 up to 2048: the token stays in registers
// (16-byte loads, two shuffle reductions, no block barrier).  Same arithmetic as enc_norm_kernel.
template <int V>  // float4 per lane: h = 128 V
__global__ void __launch_bounds__(256) enc_norm_warp_kernel(const float* x, const __half* table, const uint32_t* ids, const float* w, float eps, float* out32,
                                                            __half* out16, uint32_t tokens) {
    constexpr uint32_t h = 128 * V;
    const uint32_t t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    float4 v[V];
    if (ids != nullptr) {
        const __half* row = table + (size_t)ids[t] * h;
#pragma unroll
        for (int i = 0; i < V; i++) {
            const uint2 raw = *reinterpret_cast<const uint2*>(row + (i * 32 + lane) * 4);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            v[i] = make_float4(a.x, a.y, b.x, b.y);
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; i++) v[i] = *reinterpret_cast<const float4*>(x + (size_t)t * h + (i * 32 + lane) * 4);
    }
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < V; i++) sum += v[i].x + v[i].y + v[i].z + v[i].w;
    const float mean = warp_sum(sum) / (float)h;
    float var = 0.0f;
#pragma unroll
    for (int i = 0; i < V; i++) {
        v[i].x -= mean, v[i].y -= mean, v[i].z -= mean, v[i].w -= mean;
        var = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, var))));
    }
    const float rs = rsqrtf(warp_sum(var) / (float)h + eps);
#pragma unroll
    for (int i = 0; i < V; i++) {
        const float4 ww = __ldg(reinterpret_cast<const float4*>(w + (i * 32 + lane) * 4));
        const float4 y = make_float4(v[i].x * rs * ww.x, v[i].y * rs * ww.y, v[i].z * rs * ww.z, v[i].w * rs * ww.w);
        if (out32) *reinterpret_cast<float4*>(out32 + (size_t)t * h + (i * 32 + lane) * 4) = y;
        if (out16) {
            const __half2 a = __floats2half2_rn(y.x, y.y), b = __floats2half2_rn(y.z, y.w);
            *reinterpret_cast<uint2*>(out16 + (size_t)t * h + (i * 32 + lane) * 4) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
        }
    }
}
// Picks the warp-per-token kernel where the width allows it.
static void launch_enc_norm(cudaStream_t s, uint32_t T, const float* x, const __half* table, const uint32_t* ids, const float* w, uint32_t h, float eps, float* out32,
                            __half* out16);
// dst row r = src row of the same head with the halves interleaved (r = head d + i: i even -> i / 2, i odd -> d / 2 + i / 2)
// for the first `turned` rows; the rest as they are.  Eight halves a thread.
__global__ void __launch_bounds__(256) enc_pair_rows_kernel(const __half* src, __half* dst, uint32_t rows, uint32_t cols, uint32_t turned, uint32_t d) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x, per_row = cols / 8;
    if (i >= (size_t)rows * per_row) return;
    const uint32_t r = (uint32_t)(i / per_row), c = (uint32_t)(i % per_row), in = r % d;
    const uint32_t from = r < turned ? r - in + ((in & 1u) ? d / 2 + in / 2 : in / 2) : r;
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[(size_t)from * per_row + c];
}

// One warp per token: a lane turns eight pairs at a time (16-byte loads and stores of the low and the high half of a head)
// by the cosines and sines of the token's position from `table` (f32 [positions, d/2, 2]): (a, b) -> (a c - b s, b c + a s),
// a product then one fused multiply-add each, the reference's operations (ptx/encoder.rs:942-956) and so its bits.
__global__ void __launch_bounds__(256) enc_rope_kernel(__half* qkv, const uint32_t* pos, const float2* table, uint32_t h, uint32_t d, uint32_t tokens) {
    const uint32_t t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const uint32_t half_d = d / 2, chunks = half_d / 8, heads = h / d, items = 2 * heads * chunks;  // q and k parts
    const float2* row = table + (size_t)pos[t] * half_d;
    for (uint32_t i = lane; i < items; i += 32) {
        const uint32_t part = i / (heads * chunks), r = i % (heads * chunks), head = r / chunks, j = (r % chunks) * 8;
        __half* base = qkv + (size_t)t * 3 * h + part * h + head * d + j;
        uint4 lo = *reinterpret_cast<const uint4*>(base), hi = *reinterpret_cast<const uint4*>(base + half_d);
        __half2* l2 = reinterpret_cast<__half2*>(&lo);
        __half2* h2 = reinterpret_cast<__half2*>(&hi);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float2 a = __half22float2(l2[e]), b = __half22float2(h2[e]);
            const float4 cs = __ldg(reinterpret_cast<const float4*>(row + j + 2 * e));  // (c0, s0, c1, s1)
            l2[e] = __floats2half2_rn(__fmaf_rn(b.x, -cs.y, __fmul_rn(a.x, cs.x)), __fmaf_rn(b.y, -cs.w, __fmul_rn(a.y, cs.z)));
            h2[e] = __floats2half2_rn(__fmaf_rn(a.x, cs.y, __fmul_rn(b.x, cs.x)), __fmaf_rn(a.y, cs.w, __fmul_rn(b.y, cs.z)));
        }
        *reinterpret_cast<uint4*>(base) = lo;
        *reinterpret_cast<uint4*>(base + half_d) = hi;
    }
}
static void launch_enc_norm(cudaStream_t s, uint32_t T, const float* x, const __half* table, const uint32_t* ids, const float* w, uint32_t h, float eps, float* out32,
                            __half* out16) {
    const uint32_t blocks = (T + 7) / 8;
    switch (h % 128 == 0 ? h / 128 : 0) {
        case 6: enc_norm_warp_kernel<6><<<blocks, 256, 0, s>>>(x, table, ids, w, eps, out32, out16, T); break;   // 768
        case 8: enc_norm_warp_kernel<8><<<blocks, 256, 0, s>>>(x, table, ids, w, eps, out32, out16, T); break;   // 1024
        case 3: enc_norm_warp_kernel<3><<<blocks, 256, 0, s>>>(x, table, ids, w, eps, out32, out16, T); break;   // 384
        case 2: enc_norm_warp_kernel<2><<<blocks, 256, 0, s>>>(x, table, ids, w, eps, out32, out16, T); break;   // 256
        case 1: enc_norm_warp_kernel<1><<<blocks, 256, 0, s>>>(x, table, ids, w, eps, out32, out16, T); break;   // 128
        default: enc_norm_kernel<<<T, 256, 0, s>>>(x, table, ids, w, h, eps, out32, out16);
    }
}

// ---- bidirectional attention over packed sequences -----------------------------------------------------------------------
// A block: one tile of up to 64 queries of one sequence, one head; 4 warps x 16 query rows; keys in tiles of 64.
// Query i sees key j of its sequence when |i - j| <= window (window < 0: all).  `scale` is log2(e) / sqrt(d).  A tile of length
// 0 (an unused slot of a padded batch) does nothing.
constexpr int QT = 64, KT = 64;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
// 2^x by the hardware's approximation; 2^-inf is 0.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int D>
__global__ void __launch_bounds__(128) enc_attend_kernel(const __half* qkv, const uint32_t* tiles, __half* out, uint32_t h, int window, float scale) {
    constexpr int LD = D + 8;
    __shared__ __align__(16) __half Qs[QT * LD];
    __shared__ __align__(16) __half Ks[KT * LD];
    __shared__ __align__(16) __half Vs[KT * LD];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t start = tiles[blockIdx.x * 3], len = tiles[blockIdx.x * 3 + 1], q0 = tiles[blockIdx.x * 3 + 2], head = blockIdx.y;
    const uint32_t nq = min((uint32_t)QT, len - q0);
    const size_t row = (size_t)3 * h;
    for (uint32_t c = tid; c < QT * (D / 8); c += 128) {
        const uint32_t r = c / (D / 8), ch = c % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(qkv + (size_t)(start + q0 + r) * row + head * D + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * LD + ch * 8) = v;
    }
    const uint32_t lo = window < 0 ? 0u : (q0 > (uint32_t)window ? q0 - (uint32_t)window : 0u);
    const uint32_t hi = window < 0 ? len : min(len, q0 + nq + (uint32_t)window);  // exclusive
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; nb++) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const uint32_t ia = q0 + warp * 16 + (lane >> 2), ib = ia + 8;  // the two query positions this lane holds

    for (uint32_t j0 = lo; j0 < hi; j0 += KT) {
        __syncthreads();
        for (uint32_t c = tid; c < KT * (D / 8); c += 128) {
            const uint32_t r = c / (D / 8), ch = c % (D / 8), j = j0 + r;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (j < hi) {
                const __half* src = qkv + (size_t)(start + j) * row + head * D + ch * 8;
                kv = *reinterpret_cast<const uint4*>(src + h);
                vv = *reinterpret_cast<const uint4*>(src + 2 * h);
            }
            *reinterpret_cast<uint4*>(Ks + r * LD + ch * 8) = kv;
            *reinterpret_cast<uint4*>(Vs + r * LD + ch * 8) = vv;
        }
        __syncthreads();
        float sc[KT / 8][4];
#pragma unroll
        for (int nb = 0; nb < KT / 8; nb++) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            uint32_t a[4];
            ldsm_x4(a, Qs + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < KT / 8; nb += 2) {  // two blocks of eight keys per load
                uint32_t b[4];
                ldsm_x4(b, Ks + (nb * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma16816(sc[nb], a, b0);
                mma16816(sc[nb + 1], a, b1);
            }
        }
        float mt[2] = {-INFINITY, -INFINITY};
        // A tile every query of the block sees whole (all its keys exist and lie inside every query's window, and the block
        // has all its 64 queries) needs no mask.
        const bool whole = nq == QT && j0 + KT <= hi && (window < 0 || (j0 + KT - 1 <= q0 + (uint32_t)window && q0 + QT - 1 <= j0 + (uint32_t)window));
        if (whole) {
#pragma unroll
            for (int nb = 0; nb < KT / 8; nb++) {
                sc[nb][0] *= scale, sc[nb][1] *= scale, sc[nb][2] *= scale, sc[nb][3] *= scale;
                mt[0] = fmaxf(mt[0], fmaxf(sc[nb][0], sc[nb][1]));
                mt[1] = fmaxf(mt[1], fmaxf(sc[nb][2], sc[nb][3]));
            }
        } else {
#pragma unroll
            for (int nb = 0; nb < KT / 8; nb++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t j = j0 + nb * 8 + 2 * (lane & 3) + (e & 1), i = (e < 2) ? ia : ib;
                    const bool seen = j < hi && i < len && (window < 0 || (j <= i + (uint32_t)window && i <= j + (uint32_t)window));
                    sc[nb][e] = seen ? sc[nb][e] * scale : -INFINITY;
                    mt[e >> 1] = fmaxf(mt[e >> 1], sc[nb][e]);
                }
            }
        }
        float corr[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 1));
            mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 2));
            const float mn = fmaxf(m_run[r], mt[r]);
            base[r] = fmaxf(mn, -1e30f);               // finite, so a row that has seen nothing yet gets 2^-inf = 0 and no NaN
            corr[r] = ex2_approx(m_run[r] - base[r]);  // 1 when the maximum stays; 0 for a row's first keys (its sums are zeros)
            m_run[r] = mn;
        }
        float lt[2] = {0.0f, 0.0f};
        uint32_t pf[KT / 16][4];
#pragma unroll
        for (int nb = 0; nb < KT / 8; nb++) {
            const float e0 = ex2_approx(sc[nb][0] - base[0]), e1 = ex2_approx(sc[nb][1] - base[0]);
            const float e2 = ex2_approx(sc[nb][2] - base[1]), e3 = ex2_approx(sc[nb][3] - base[1]);
            const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
            lt[0] += __low2float(h01) + __high2float(h01);
            lt[1] += __low2float(h23) + __high2float(h23);
            pf[nb / 2][(nb & 1) * 2] = *reinterpret_cast<const uint32_t*>(&h01);
            pf[nb / 2][(nb & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            lt[r] += __shfl_xor_sync(0xffffffffu, lt[r], 1);
            lt[r] += __shfl_xor_sync(0xffffffffu, lt[r], 2);
            l_run[r] = l_run[r] * corr[r] + lt[r];
        }
        const bool moved = __any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f);  // else the scaling is by one
#pragma unroll
        for (int nb = 0; nb < D / 8; nb += 2) {  // two blocks of eight dimensions per load
            if (moved) {
                o[nb][0] *= corr[0], o[nb][1] *= corr[0], o[nb][2] *= corr[1], o[nb][3] *= corr[1];
                o[nb + 1][0] *= corr[0], o[nb + 1][1] *= corr[0], o[nb + 1][2] *= corr[1], o[nb + 1][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < KT / 16; kk++) {
                uint32_t b[4];
                ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 15)) * LD + (nb + (lane >> 4)) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma16816(o[nb], pf[kk], b0);
                mma16816(o[nb + 1], pf[kk], b1);
            }
        }
    }
    const float inv[2] = {l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f};
#pragma unroll
    for (int nb = 0; nb < D / 8; nb++) {
        const uint32_t col = head * D + nb * 8 + 2 * (lane & 3);
        if (ia < len) *reinterpret_cast<__half2*>(out + (size_t)(start + ia) * h + col) = __floats2half2_rn(o[nb][0] * inv[0], o[nb][1] * inv[0]);
        if (ib < len) *reinterpret_cast<__half2*>(out + (size_t)(start + ib) * h + col) = __floats2half2_rn(o[nb][2] * inv[1], o[nb][3] * inv[1]);
    }
}

// ---- pooling ------------------------------------------------------------------------------------------------------------------
// The sequence's vector (first token, or the mean over its tokens) L2-normalised (max(len, 1e-12), as
// encoder/run.rs:160-173), truncated to `dims` and normalised again when truncated (encoder/text.rs:56-63).
// The mean's sums come in POOL_PARTS parts (a block a part of a sequence's tokens: one block a sequence left most of the
// machine idle over 50 MB of hidden states), which the sequence's block then adds in a fixed order.
constexpr uint32_t POOL_PARTS = 8;

__global__ void __launch_bounds__(256) enc_pool_part_kernel(const float* hidden, const uint32_t* starts, const uint32_t* lens, uint32_t h, float* part) {
    const uint32_t s = blockIdx.x, k = blockIdx.y, start = starts[s], len = lens[s];
    const uint32_t per = (len + POOL_PARTS - 1) / POOL_PARTS, t0 = min(len, k * per), t1 = min(len, t0 + per);
    for (uint32_t i = threadIdx.x; i < h; i += 256) {
        // Four running sums, so that several loads are in flight instead of one.
        const float* col = hidden + (size_t)start * h + i;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        uint32_t t = t0;
#pragma unroll 2
        for (; t + 4 <= t1; t += 4) a0 += col[(size_t)t * h], a1 += col[(size_t)(t + 1) * h], a2 += col[(size_t)(t + 2) * h], a3 += col[(size_t)(t + 3) * h];
        for (; t < t1; t++) a0 += col[(size_t)t * h];
        part[((size_t)s * POOL_PARTS + k) * h + i] = (a0 + a1) + (a2 + a3);
    }
}

__global__ void __launch_bounds__(256) enc_pool_kernel(const float* hidden, const float* part, const uint32_t* starts, const uint32_t* lens, uint32_t h, uint32_t dims,
                                                       int mean, float* out) {
    __shared__ float sh[8];
    __shared__ float vec[2048];
    const uint32_t s = blockIdx.x, start = starts[s], len = lens[s];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto block_sum = [&](float v) {
        v = warp_sum(v);
        __syncthreads();
        if (lane == 0) sh[warp] = v;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) t += sh[i];
        return t;
    };
    float sq = 0.0f;
    for (uint32_t i = tid; i < h; i += 256) {
        float v = 0.0f;
        if (mean) {
            const float* p = part + (size_t)s * POOL_PARTS * h + i;
#pragma unroll
            for (uint32_t k = 0; k < POOL_PARTS; k++) v += p[(size_t)k * h];
            v /= (float)len;
        } else {
            v = hidden[(size_t)start * h + i];
        }
        vec[i] = v;
        sq = fmaf(v, v, sq);
    }
    const float n1 = fmaxf(sqrtf(block_sum(sq)), 1e-12f);
    float sq2 = 0.0f;
    for (uint32_t i = tid; i < dims; i += 256) {
        const float v = vec[i] / n1;
        vec[i] = v;
        sq2 = fmaf(v, v, sq2);
    }
    const float n2 = dims < h ? fmaxf(sqrtf(block_sum(sq2)), 1e-12f) : 1.0f;
    for (uint32_t i = tid; i < dims; i += 256) out[(size_t)s * dims + i] = vec[i] / n2;
}

// A converted model's Q8E scales (f32, one per 64 along a row) as this build's (f16, one per 32): each rounded and stored twice.
__global__ void __launch_bounds__(256) enc_scales_kernel(const float* in, __half* out, size_t n) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const __half v = __float2half_rn(in[i]);
    out[2 * i] = v, out[2 * i + 1] = v;
}

struct EMat {
    int8_t* w = nullptr;
    __half* s = nullptr;
    __half* f16 = nullptr;  // the matrix as f16 [rows, cols] instead, in an allocation of its own (a model too narrow for 8 bits to pay)
    __half* copy = nullptr; // the codes times their scales as f16 [rows, cols], in the arena: what the products read (tb_encoder.use_copy)
    uint32_t rows = 0, cols = 0;
    size_t code_bytes() const { return (size_t)rows * cols; }
    size_t scale_bytes() const { return (size_t)rows * (cols / 32) * 2; }
};

struct ELayer {
    EMat qkv, o, up, down;
    float *attn_norm = nullptr, *mlp_norm = nullptr;
    bool global = false;
};

struct EGraph {
    uint32_t padded = 0, sequences = 0;
    cudaGraphExec_t exec = nullptr;
};

constexpr size_t ENC_GRAPHS = 16;  // shapes kept, the oldest dropped first (encoder/run.rs:20)

}  // namespace

int launch_enc_attend(tb_context* ctx, const __half* qkv, const uint32_t* tiles, __half* out, uint32_t h, uint32_t d, int window, float scale, uint32_t ntiles) {
    if (!qkv || !tiles || !out || ntiles == 0 || h == 0 || (d != 32 && d != 64) || h % d != 0) return fail(OUT_OF_RANGE, "encoder attention: null or empty argument, or heads other than 32 or 64 wide");
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) & 15) return fail(OUT_OF_RANGE, "encoder attention: buffers must be 16-byte aligned");
    if (d == 64) enc_attend_kernel<64><<<dim3(ntiles, h / d), 128, 0, ctx->stream>>>(qkv, tiles, out, h, window, scale);
    else enc_attend_kernel<32><<<dim3(ntiles, h / d), 128, 0, ctx->stream>>>(qkv, tiles, out, h, window, scale);
    TB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace tb

using namespace tb;

struct tb_encoder {
    tb_context* ctx = nullptr;
    tb_encoder_config cfg = {};
    std::vector<uint8_t> global;
    std::vector<ELayer> layers;
    uint32_t cap_tokens = 0, cap_padded = 0, cap_seqs = 0, tokens = 0;
    char* arena = nullptr;
    size_t arena_bytes = 0;
    __half* embed = nullptr;
    float *embed_norm = nullptr, *final_norm = nullptr;
    float2* rope[2] = {nullptr, nullptr};  // cosines and sines [positions, d/2]: global layers', sliding layers'
    float *x = nullptr, *hidden = nullptr, *pooled = nullptr, *pool_part = nullptr;  // pool_part: [sequences][POOL_PARTS][hidden] partial sums of the mean
    __half *a16 = nullptr, *qkv16 = nullptr, *att16 = nullptr, *g16 = nullptr;
    // A batch's inputs, one block on the device and its twin in pinned host memory: ids, positions, tiles, first rows, lengths.
    uint32_t *inputs = nullptr, *stage = nullptr;
    size_t input_words = 0;
    uint32_t *ids = nullptr, *pos = nullptr, *tiles = nullptr, *starts = nullptr, *lens = nullptr;
    bool use_graphs = true, warmed = false;
    // The products read an f16 copy of the 8-bit matrices by TMA instead of converting codes in their loop (2 bytes a weight
    // more; the values are the codes' own, launch_dequant_f16).  Written before a batch when a tensor was loaded since.
    // TACHYON_B200_ENCODER_COPY=0 leaves it out.
    bool use_copy = true, copy_valid = false;
    // The q/k/v product turns the queries and keys in its store (GemmRope): its copy of the matrix has a head's rows j and
    // j + d/2 side by side, so q and k come out with their dimensions in that order, which the dot products do not mind.
    // Off unless TACHYON_B200_ENCODER_ROPE=1: measured over forty batches in a row it loses 3 % (9.97 against 9.66 ms a batch:
    // the table loads and shuffles lengthen an epilogue that is short of issue slots already, and the rotation kernel it
    // saves finds its 100 MB in the L2).
    bool rope_fused = false;
    __half* rope_tmp = nullptr;  // the q/k/v matrix in f16 before its rows are put in that order
    uint32_t tile_q = QT;  // queries a tile of the list holds: 64, or 128 where attention runs on tcgen05 (decided when the encoder is opened)
    std::vector<EGraph> graphs;
};

namespace {

size_t enc_layout(tb_encoder* e, char* base) {
    const tb_encoder_config& c = e->cfg;
    size_t end = 0;
    auto take = [&](size_t bytes) {
        const size_t at = end;
        end += (bytes + 255) / 256 * 256;
        return base + at;
    };
    auto mat = [&](EMat& m, uint32_t rows, uint32_t cols) {
        m.rows = rows, m.cols = cols;
        m.w = reinterpret_cast<int8_t*>(take(m.code_bytes()));
        m.s = reinterpret_cast<__half*>(take(m.scale_bytes()));
        m.copy = e->use_copy ? reinterpret_cast<__half*>(take(2 * m.code_bytes())) : nullptr;
    };
    const uint32_t h = c.hidden, up_rows = c.gated ? 2 * c.inter : c.inter, T = e->cap_padded, S = e->cap_seqs;
    e->embed = reinterpret_cast<__half*>(take((size_t)c.vocab * h * 2));
    e->embed_norm = reinterpret_cast<float*>(take(h * 4));
    e->final_norm = reinterpret_cast<float*>(take(h * 4));
    for (int k = 0; k < 2; k++) e->rope[k] = reinterpret_cast<float2*>(take((size_t)e->cap_tokens * (h / c.heads / 2) * 8));
    for (uint32_t l = 0; l < c.layers; l++) {
        ELayer& L = e->layers[l];
        L.global = e->global[l] != 0;
        L.attn_norm = reinterpret_cast<float*>(take(h * 4));
        L.mlp_norm = reinterpret_cast<float*>(take(h * 4));
        mat(L.qkv, 3 * h, h), mat(L.o, h, h), mat(L.up, up_rows, h), mat(L.down, h, c.inter);
    }
    e->rope_tmp = e->rope_fused ? reinterpret_cast<__half*>(take((size_t)3 * h * h * 2)) : nullptr;
    e->x = reinterpret_cast<float*>(take((size_t)T * h * 4));
    e->hidden = reinterpret_cast<float*>(take((size_t)T * h * 4));
    e->pooled = reinterpret_cast<float*>(take((size_t)S * h * 4));
    e->pool_part = reinterpret_cast<float*>(take((size_t)S * POOL_PARTS * h * 4));
    e->a16 = reinterpret_cast<__half*>(take((size_t)T * h * 2));
    e->qkv16 = reinterpret_cast<__half*>(take((size_t)T * 3 * h * 2));
    e->att16 = reinterpret_cast<__half*>(take((size_t)T * h * 2));
    e->g16 = reinterpret_cast<__half*>(take((size_t)T * c.inter * 2));
    e->input_words = (size_t)2 * T + ((size_t)T / QT + S) * 3 + 2 * (size_t)S;
    e->inputs = reinterpret_cast<uint32_t*>(take(e->input_words * 4));
    return end;
}

// Where each part of a batch's inputs sits in the block at `base` (the device's or the host's).
void enc_inputs(tb_encoder* e, uint32_t* base, uint32_t*& ids, uint32_t*& pos, uint32_t*& tiles, uint32_t*& starts, uint32_t*& lens) {
    const size_t T = e->cap_padded, S = e->cap_seqs;
    ids = base, pos = ids + T, tiles = pos + T, starts = tiles + (T / QT + S) * 3, lens = starts + S;
}

int enc_validate(const tb_encoder_config& c) {
    if (c.hidden == 0 || c.heads == 0 || c.hidden % c.heads != 0) return fail(FORMAT, "encoder: an inconsistent shape");
    const uint32_t d = c.hidden / c.heads;
    if (d != 32 && d != 64) return fail(UNSUPPORTED, "encoder: head size 32 or 64");
    if (c.hidden % 64 != 0 || c.inter % 64 != 0 || c.hidden > 2048) return fail(UNSUPPORTED, "encoder: widths must be multiples of 64, hidden at most 2048");
    if (c.layers == 0 || c.vocab == 0 || c.inter == 0) return fail(OUT_OF_RANGE, "encoder: empty model");
    if (c.dims == 0 || c.dims > c.hidden) return fail(OUT_OF_RANGE, "encoder: dims must be in 1..hidden");
    if (c.gated > 2) return fail(OUT_OF_RANGE, "encoder: gated is 0 (plain GELU), 1 (GELU gate) or 2 (SiLU gate)");
    return OK;
}

struct ENamed {
    void* ptr = nullptr;
    size_t bytes = 0;
    int kind = 0;          // 0 vector or table; 1 codes (.w); 2 f16 scales per 32 (.s); 3 a matrix by its size: Q8E codes or f16; 4 f32 scales per 64 (.scale)
    EMat* mat = nullptr;
    bool gated_up = false;  // the gated MLP's Wi, whose two halves' rows are interleaved on the device
};

bool enc_find(tb_encoder* e, const std::string& name, ENamed& out) {
    const tb_encoder_config& c = e->cfg;
    const size_t hb = (size_t)c.hidden * 4;
    if (name == "embed") return out = {e->embed, (size_t)c.vocab * c.hidden * 2, 0}, true;
    if (name == "embed_norm") return out = {e->embed_norm, hb, 0}, true;
    if (name == "final_norm") return out = {e->final_norm, hb, 0}, true;
    const size_t dot = name.find('.');
    if (dot == std::string::npos || dot == 0) return false;
    uint32_t l = 0;
    for (size_t k = 0; k < dot; k++) {
        if (name[k] < '0' || name[k] > '9') return false;
        l = l * 10 + (uint32_t)(name[k] - '0');
    }
    if (l >= c.layers) return false;
    ELayer& L = e->layers[l];
    const std::string rest = name.substr(dot + 1);
    if (rest == "attn_norm") return out = {L.attn_norm, hb, 0}, true;
    if (rest == "mlp_norm") return out = {L.mlp_norm, hb, 0}, true;
    auto mat = [&](EMat& m, const std::string& suffix, bool gated_up) {
        if (suffix == ".w") out = {m.w, m.code_bytes(), 1, &m, gated_up};
        else if (suffix == ".s") out = {m.s, m.scale_bytes(), 2, &m, gated_up};
        else if (suffix.empty()) out = {nullptr, 0, 3, &m, gated_up};
        else if (suffix == ".scale") out = {m.s, (size_t)m.rows * (m.cols / 64) * 4, 4, &m, gated_up};
        else return false;
        return true;
    };
    if (rest.rfind("qkv", 0) == 0) return mat(L.qkv, rest.substr(3), false);
    if (rest == "o" || rest.rfind("o.", 0) == 0) return mat(L.o, rest.substr(1), false);
    if (rest.rfind("up", 0) == 0) return mat(L.up, rest.substr(2), c.gated != 0);
    if (rest.rfind("down", 0) == 0) return mat(L.down, rest.substr(4), false);
    return false;
}

// One matrix product of the forward pass: the matrix as f16 when it was loaded so, else its codes and scales.
int enc_product(tb_encoder* e, const EMat& m, const __half* a, uint32_t tokens, void* out, int mode) {
    const __half* f16 = m.f16 != nullptr ? m.f16 : (e->copy_valid ? m.copy : nullptr);
    if (f16 != nullptr) return launch_gemm_q8(e->ctx, reinterpret_cast<const int8_t*>(f16), nullptr, a, tokens, m.rows, m.cols, out, mode, 16);
    return launch_gemm_q8(e->ctx, m.w, m.s, a, tokens, m.rows, m.cols, out, mode);
}

// The kernels of the batch in the inputs (Encoder::layers, encoder/run.rs:413-447) over `n` rows (the batch padded to whole
// tiles of 64 tokens: the rows past its tokens hold token 0 at position 0 and belong to no tile), `slots` tiles, `sequences`
// sequences; leaves the last hidden states in `hidden` and the embeddings in `pooled`.
int enc_layers(tb_encoder* e, uint32_t n, uint32_t slots, uint32_t sequences) {
    const tb_encoder_config& c = e->cfg;
    tb_context* ctx = e->ctx;
    cudaStream_t s = ctx->stream;
    const uint32_t h = c.hidden, d = h / c.heads;
    const float scale = 1.4426950408889634f / sqrtf((float)d);
    // embeddings -> norm: x (f32 residual stream) and, since layer 0 has no attention norm, its f16 GEMM input
    launch_enc_norm(s, n, nullptr, e->embed, e->ids, e->embed_norm, h, c.eps, e->x, e->a16);
    for (uint32_t l = 0; l < c.layers; l++) {
        ELayer& L = e->layers[l];
        if (l > 0) launch_enc_norm(s, n, e->x, nullptr, nullptr, L.attn_norm, h, c.eps, nullptr, e->a16);
        if (e->rope_fused) {
            const GemmRope turn{e->rope[L.global ? 0 : 1], e->pos, 2 * h, d};
            TB_TRY(launch_gemm_persistent(ctx, reinterpret_cast<const int8_t*>(L.qkv.copy), nullptr, e->a16, n, 3 * h, h, e->qkv16, 1, 16, nullptr, 0, &turn));
        } else {
            TB_TRY(enc_product(e, L.qkv, e->a16, n, e->qkv16, 1));
            enc_rope_kernel<<<(n + 7) / 8, 256, 0, s>>>(e->qkv16, e->pos, e->rope[L.global ? 0 : 1], h, d, n);
        }
        if (e->tile_q == 128) TB_TRY(launch_enc_attend_tc(ctx, e->qkv16, e->tiles, e->att16, h, L.global ? -1 : (int)c.window, scale, slots, n));
        else TB_TRY(launch_enc_attend(ctx, e->qkv16, e->tiles, e->att16, h, d, L.global ? -1 : (int)c.window, scale, slots));
        TB_TRY(enc_product(e, L.o, e->att16, n, e->x, 3));
        launch_enc_norm(s, n, e->x, nullptr, nullptr, L.mlp_norm, h, c.eps, nullptr, e->a16);
        TB_TRY(enc_product(e, L.up, e->a16, n, e->g16, c.gated == 2 ? 8 : c.gated ? 4 : 5));
        TB_TRY(enc_product(e, L.down, e->g16, n, e->x, 3));
    }
    launch_enc_norm(s, n, e->x, nullptr, nullptr, e->final_norm, h, c.eps, e->hidden, nullptr);
    if (c.mean_pool) enc_pool_part_kernel<<<dim3(sequences, POOL_PARTS), 256, 0, s>>>(e->hidden, e->starts, e->lens, h, e->pool_part);
    enc_pool_kernel<<<sequences, 256, 0, s>>>(e->hidden, e->pool_part, e->starts, e->lens, h, c.dims, c.mean_pool ? 1 : 0, e->pooled);
    TB_CUDA(cudaGetLastError());
    return OK;
}

// One batch (Encoder::encode, encoder/run.rs:379-410): its inputs written and copied, then the kernels, as the graph of the
// batch's padded shape, recorded the first time the shape is seen.
int enc_batch(tb_encoder* e, const uint32_t* ids, const uint32_t* lens, uint32_t sequences, float* out_host) {
    cudaStream_t s = e->ctx->stream;
    if (e->use_copy && !e->copy_valid) {
        for (ELayer& L : e->layers)
            for (EMat* m : {&L.qkv, &L.o, &L.up, &L.down}) {
                const bool pairs = e->rope_fused && m == &L.qkv;
                if (m->f16 == nullptr) TB_TRY(launch_dequant_f16(e->ctx, m->w, m->s, m->rows, m->cols, 8, pairs ? e->rope_tmp : m->copy));
                if (pairs) {
                    const size_t items = (size_t)m->rows * (m->cols / 8);
                    enc_pair_rows_kernel<<<(unsigned)((items + 255) / 256), 256, 0, s>>>(m->f16 ? m->f16 : e->rope_tmp, m->copy, m->rows, m->cols, 2 * e->cfg.hidden,
                                                                                      e->cfg.hidden / e->cfg.heads);
                    TB_CUDA(cudaGetLastError());
                }
            }
        e->copy_valid = true;
    }
    uint32_t *hi, *hp, *ht, *hs, *hl;
    enc_inputs(e, e->stage, hi, hp, ht, hs, hl);
    uint32_t T = 0, tiles = 0;
    for (uint32_t q = 0; q < sequences; q++) {
        hs[q] = T, hl[q] = lens[q];
        for (uint32_t i = 0; i < lens[q]; i++) hi[T + i] = ids[T + i], hp[T + i] = i;
        for (uint32_t q0 = 0; q0 < lens[q]; q0 += e->tile_q, tiles++) ht[3 * tiles] = T, ht[3 * tiles + 1] = lens[q], ht[3 * tiles + 2] = q0;
        T += lens[q];
    }
    const uint32_t n = (T + QT - 1) / QT * QT, slots = n / QT + sequences;
    for (uint32_t i = T; i < n; i++) hi[i] = 0, hp[i] = 0;
    for (uint32_t i = 3 * tiles; i < 3 * slots; i++) ht[i] = 0;
    e->tokens = T;
    TB_CUDA(cudaMemcpyAsync(e->inputs, e->stage, e->input_words * 4, cudaMemcpyHostToDevice, s));
    if (!e->use_graphs) {
        TB_TRY(enc_layers(e, n, slots, sequences));
    } else {
        size_t at = 0;
        while (at < e->graphs.size() && !(e->graphs[at].padded == n && e->graphs[at].sequences == sequences)) at++;
        if (at == e->graphs.size()) {
            if (!e->warmed) {  // every kernel once outside a recording: their first launches set function attributes
                TB_TRY(enc_layers(e, n, slots, sequences));
                e->warmed = true;
            }
            TB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            const int st = enc_layers(e, n, slots, sequences);
            cudaGraph_t graph = nullptr;
            const cudaError_t ec = cudaStreamEndCapture(s, &graph);
            if (st != OK || ec != cudaSuccess) {
                if (graph) cudaGraphDestroy(graph);
                return st != OK ? st : cuda_fail(ec, "tb_encoder_embed: recording the batch");
            }
            EGraph g;
            g.padded = n, g.sequences = sequences;
            const cudaError_t ei = cudaGraphInstantiate(&g.exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ei != cudaSuccess) return cuda_fail(ei, "tb_encoder_embed: cudaGraphInstantiate");
            if (e->graphs.size() == ENC_GRAPHS) {
                cudaGraphExecDestroy(e->graphs.front().exec);
                e->graphs.erase(e->graphs.begin());
            }
            e->graphs.push_back(g);
            at = e->graphs.size() - 1;
        }
        TB_CUDA(cudaGraphLaunch(e->graphs[at].exec, s));
    }
    if (out_host) TB_CUDA(cudaMemcpyAsync(out_host, e->pooled, (size_t)sequences * e->cfg.dims * 4, cudaMemcpyDeviceToHost, s));
    TB_CUDA(cudaStreamSynchronize(s));
    return OK;
}

}  // namespace

extern "C" {

int tb_encoder_open(tb_context* ctx, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, tb_encoder** out) {
    if (!ctx || !cfg || !out || tokens == 0 || sequences == 0) return fail(OUT_OF_RANGE, "tb_encoder_open: null or empty argument");
    *out = nullptr;
    TB_TRY(enc_validate(*cfg));
    tb_encoder* e = new tb_encoder();
    e->ctx = ctx, e->cfg = *cfg, e->cap_tokens = tokens, e->cap_padded = (tokens + QT - 1) / QT * QT, e->cap_seqs = sequences;
    e->global.resize(cfg->layers);
    for (uint32_t l = 0; l < cfg->layers; l++) e->global[l] = cfg->global ? cfg->global[l] : (l % (cfg->global_every ? cfg->global_every : 3) == 0);
    e->cfg.global = nullptr;
    e->layers.resize(cfg->layers);
    const char* env = getenv("TACHYON_B200_ENCODER_GRAPHS");
    e->use_graphs = !(env && env[0] == '0');
    env = getenv("TACHYON_B200_ENCODER_COPY");
    e->use_copy = !(env && env[0] == '0');
    env = getenv("TACHYON_B200_ENCODER_ROPE");
    e->rope_fused = e->use_copy && env && env[0] == '1' && gemm_persistent_supports(3 * cfg->hidden, cfg->hidden, 16) && cfg->hidden % 16 == 0;
    e->tile_q = (ctx->flash_tc && enc_attend_tc_supports(cfg->hidden, cfg->hidden / cfg->heads)) ? 128u : (uint32_t)QT;
    e->arena_bytes = enc_layout(e, nullptr);
    cudaError_t err = cudaSetDevice(ctx->gpu);
    if (err == cudaSuccess) err = cudaMalloc(&e->arena, e->arena_bytes);
    if (err == cudaSuccess) err = cudaMemsetAsync(e->arena, 0, e->arena_bytes, ctx->stream);
    if (err == cudaSuccess) err = cudaMallocHost(&e->stage, e->input_words * 4);
    if (err != cudaSuccess) {
        tb_encoder_close(e);
        return cuda_fail(err, "tb_encoder_open");
    }
    enc_layout(e, e->arena);
    enc_inputs(e, e->inputs, e->ids, e->pos, e->tiles, e->starts, e->lens);
    // RoPE's cosines and sines of every position a sequence can have, in f64 and rounded once (rope_tables, encoder/run.rs:523-537).
    const uint32_t half = cfg->hidden / cfg->heads / 2;
    std::vector<float2> table((size_t)tokens * half);
    for (int k = 0; k < 2; k++) {
        const double theta = (double)(k ? cfg->theta_local : cfg->theta_global);
        for (uint32_t j = 0; j < half; j++) {
            const double f = pow(theta, -2.0 * (double)j / (double)(2 * half));
            for (uint32_t p = 0; p < tokens; p++) table[(size_t)p * half + j] = make_float2((float)cos((double)p * f), (float)sin((double)p * f));
        }
        err = cudaMemcpyAsync(e->rope[k], table.data(), table.size() * 8, cudaMemcpyHostToDevice, ctx->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
        if (err != cudaSuccess) {
            tb_encoder_close(e);
            return cuda_fail(err, "tb_encoder_open: rope tables");
        }
    }
    *out = e;
    return OK;
}

void tb_encoder_close(tb_encoder* e) {
    if (!e) return;
    if (e->ctx && e->ctx->stream) cudaStreamSynchronize(e->ctx->stream);
    for (EGraph& g : e->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    for (ELayer& L : e->layers)
        for (EMat* m : {&L.qkv, &L.o, &L.up, &L.down})
            if (m->f16) cudaFree(m->f16);
    if (e->arena) cudaFree(e->arena);
    if (e->stage) cudaFreeHost(e->stage);
    delete e;
}

int tb_encoder_load(tb_encoder* e, const char* name, const void* data, size_t bytes) {
    if (!e || !name || !data) return fail(OUT_OF_RANGE, "tb_encoder_load: null argument");
    ENamed t;
    if (!enc_find(e, name, t)) return fail(NO_MODEL, std::string("tb_encoder_load: no tensor named ") + name);
    e->copy_valid = false;
    cudaStream_t s = e->ctx->stream;
    TB_CUDA(cudaSetDevice(e->ctx->gpu));
    if (t.kind == 3) {  // a matrix under its plain name: Q8E codes or f16, told apart by the size
        EMat& m = *t.mat;
        if (bytes == m.code_bytes()) {
            t.ptr = m.w, t.bytes = bytes, t.kind = 1;
            if (m.f16) cudaFree(m.f16), m.f16 = nullptr;
        } else if (bytes == 2 * m.code_bytes()) {
            if (!m.f16) TB_CUDA(cudaMalloc(&m.f16, bytes));
            t.ptr = m.f16, t.bytes = bytes;
        } else {
            return fail(FORMAT, std::string("tb_encoder_load: ") + name + " has " + std::to_string(bytes) + " bytes, neither i8 nor f16 of its shape");
        }
    }
    if (bytes != t.bytes) return fail(FORMAT, std::string("tb_encoder_load: ") + name + " has " + std::to_string(bytes) + " bytes, expected " + std::to_string(t.bytes));
    if (t.kind == 0 || (t.kind != 4 && !t.gated_up)) {
        TB_CUDA(cudaMemcpyAsync(t.ptr, data, bytes, cudaMemcpyHostToDevice, s));
        TB_CUDA(cudaStreamSynchronize(s));
        return OK;
    }
    // Through a scratch copy.  The gated MLP's Wi: activation rows, then gate rows in the file; pairs side by side on the
    // device, so that a GEMM tile holds both (Encoder::interleave, encoder/run.rs:449-466).  Q8E scales: rounded to f16,
    // one per 32.
    void *tmp = nullptr, *tmp2 = nullptr;
    TB_CUDA(cudaMalloc(&tmp, bytes));
    cudaError_t err = cudaMemcpyAsync(tmp, data, bytes, cudaMemcpyHostToDevice, s);
    int st = OK;
    const uint32_t inter = e->cfg.inter;
    if (err == cudaSuccess && t.kind == 4) {
        const void* src = tmp;
        if (t.gated_up) {
            err = cudaMalloc(&tmp2, bytes);
            if (err == cudaSuccess) st = launch_interleave_rows(e->ctx, tmp, tmp2, inter, (uint32_t)(bytes / (2 * (size_t)inter)));
            src = tmp2;
        }
        if (err == cudaSuccess && st == OK) {
            const size_t n = bytes / 4;
            enc_scales_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const float*>(src), static_cast<__half*>(t.ptr), n);
            err = cudaGetLastError();
        }
    } else if (err == cudaSuccess) {
        st = launch_interleave_rows(e->ctx, tmp, t.ptr, inter, (uint32_t)(bytes / (2 * (size_t)inter)));
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    cudaFree(tmp);
    if (tmp2) cudaFree(tmp2);
    if (err != cudaSuccess) return cuda_fail(err, "tb_encoder_load");
    return st;
}

// For the file loader: a tensor that is copied to its place as it is (the embedding table, the norms) may arrive in pieces.
int tb_encoder_load_part(tb_encoder* e, const char* name, size_t offset, const void* data, size_t bytes, size_t total) {
    if (!e || !name || !data) return fail(OUT_OF_RANGE, "tb_encoder_load_part: null argument");
    if (offset == 0 && bytes == total) return tb_encoder_load(e, name, data, bytes);
    ENamed t;
    if (!enc_find(e, name, t)) return fail(NO_MODEL, std::string("tb_encoder_load: no tensor named ") + name);
    if (t.kind != 0) return fail(UNSUPPORTED, std::string("tb_encoder_load_part: ") + name + " is rearranged on the way and comes whole");
    if (total != t.bytes) return fail(FORMAT, std::string("tb_encoder_load: ") + name + " has " + std::to_string(total) + " bytes, expected " + std::to_string(t.bytes));
    if (offset > total || bytes > total - offset) return fail(OUT_OF_RANGE, "tb_encoder_load_part: a piece past the tensor's end");
    TB_CUDA(cudaSetDevice(e->ctx->gpu));
    TB_CUDA(cudaMemcpyAsync(static_cast<char*>(t.ptr) + offset, data, bytes, cudaMemcpyHostToDevice, e->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(e->ctx->stream));
    return OK;
}

int tb_encoder_loads_in_parts(tb_encoder* e, const char* name) {
    ENamed t;
    return e && name && enc_find(e, name, t) && t.kind == 0;
}

int tb_encoder_fill_random(tb_encoder* e, uint64_t seed) {
    if (!e) return fail(OUT_OF_RANGE, "null encoder");
    e->copy_valid = false;
    const tb_encoder_config& c = e->cfg;
    tb_context* ctx = e->ctx;
    // Streams: 0 embed (f16 N(0,1)*0.02... as values), 1 embed_norm, 2 final_norm; layer l: 16*(l+1) + {0 qkv.w, 1 qkv.s, 2 o.w, 3 o.s,
    // 4 up.w, 5 up.s, 6 down.w, 7 down.s, 8 attn_norm, 9 mlp_norm}.
    TB_TRY(launch_fill_gauss_f16(ctx, seed, 0, e->embed, (size_t)c.vocab * c.hidden, 1.0f));
    TB_TRY(launch_fill_uniform(ctx, seed, 1, e->embed_norm, c.hidden, 0.5f, 1.5f));
    TB_TRY(launch_fill_uniform(ctx, seed, 2, e->final_norm, c.hidden, 0.5f, 1.5f));
    const float smul = 0.02f / 127.0f;
    void *tw = nullptr, *ts = nullptr;
    if (c.gated) {
        TB_CUDA(cudaMalloc(&tw, e->layers[0].up.code_bytes()));
        TB_CUDA(cudaMalloc(&ts, e->layers[0].up.scale_bytes()));
    }
    int st = OK;
    for (uint32_t l = 0; l < c.layers && st == OK; l++) {
        ELayer& L = e->layers[l];
        const uint64_t b = 16ull * (l + 1);
        auto mat = [&](EMat& m, uint64_t id) -> int {
            TB_TRY(launch_fill_codes(ctx, seed, id, m.w, m.code_bytes()));
            return launch_fill_scales(ctx, seed, id + 1, m.s, m.scale_bytes() / 2, smul);
        };
        st = mat(L.qkv, b);
        if (st == OK) st = mat(L.o, b + 2);
        if (st == OK && c.gated) {
            st = launch_fill_codes(ctx, seed, b + 4, static_cast<int8_t*>(tw), L.up.code_bytes());
            if (st == OK) st = launch_fill_scales(ctx, seed, b + 5, static_cast<__half*>(ts), L.up.scale_bytes() / 2, smul);
            if (st == OK) st = launch_interleave_rows(ctx, tw, L.up.w, c.inter, c.hidden);
            if (st == OK) st = launch_interleave_rows(ctx, ts, L.up.s, c.inter, c.hidden / 32 * 2);
        } else if (st == OK) {
            st = mat(L.up, b + 4);
        }
        if (st == OK) st = mat(L.down, b + 6);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 8, L.attn_norm, c.hidden, 0.5f, 1.5f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 9, L.mlp_norm, c.hidden, 0.5f, 1.5f);
    }
    cudaStreamSynchronize(ctx->stream);
    if (tw) cudaFree(tw);
    if (ts) cudaFree(ts);
    return st;
}

// Encoder::embeddings (encoder/run.rs:161-175): `ids` packed back to back, `lens[s]` tokens per sequence; out (host)
// receives dims floats per sequence.  The sequences go in batches of at most the capacity's tokens (and sequences), in
// order, a batch closed by the first sequence that no longer fits (Encoder::batches, run.rs:207-221).
int tb_encoder_embed(tb_encoder* e, const uint32_t* ids, const uint32_t* lens, uint32_t sequences, float* out_host) {
    if (!e || !ids || !lens || sequences == 0) return fail(OUT_OF_RANGE, "tb_encoder_embed: null or empty argument");
    const tb_encoder_config& c = e->cfg;
    size_t total = 0;
    for (uint32_t q = 0; q < sequences; q++) {
        if (lens[q] == 0) return fail(OUT_OF_RANGE, "tb_encoder_embed: an empty sequence");
        if (lens[q] > e->cap_tokens) return fail(TOO_LONG, "tb_encoder_embed: a sequence of " + std::to_string(lens[q]) + " tokens, more than the " + std::to_string(e->cap_tokens) + " the encoder was opened for");
        total += lens[q];
    }
    for (size_t i = 0; i < total; i++)
        if (ids[i] >= c.vocab) return fail(OUT_OF_RANGE, "tb_encoder_embed: token outside the vocabulary");
    TB_CUDA(cudaSetDevice(e->ctx->gpu));
    uint32_t from = 0, used = 0;
    size_t first = 0;  // of the open batch: its first sequence, its tokens so far, its first token
    for (uint32_t q = 0; q <= sequences; q++) {
        if (q == sequences || used + lens[q] > e->cap_tokens || q - from == e->cap_seqs) {
            TB_TRY(enc_batch(e, ids + first, lens + from, q - from, out_host ? out_host + (size_t)from * c.dims : nullptr));
            first += used, from = q, used = 0;
        }
        if (q < sequences) used += lens[q];
    }
    return OK;
}

int tb_encoder_hidden(tb_encoder* e, float* out_host) {
    if (!e || !out_host) return fail(OUT_OF_RANGE, "tb_encoder_hidden: null argument");
    TB_CUDA(cudaMemcpyAsync(out_host, e->hidden, (size_t)e->tokens * e->cfg.hidden * 4, cudaMemcpyDeviceToHost, e->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(e->ctx->stream));
    return OK;
}

uint32_t tb_encoder_batch_tokens(const tb_encoder* e) { return e ? e->tokens : 0; }

uint32_t tb_encoder_graphs(const tb_encoder* e) { return e ? (uint32_t)e->graphs.size() : 0; }

// Encoder::bytes (encoder/run.rs:144-147): the VRAM it holds, weights, RoPE tables and activations, with the f16 matrices a
// converted model brought.
size_t tb_encoder_bytes(const tb_encoder* e) {
    if (!e) return 0;
    size_t n = e->arena_bytes;
    for (const ELayer& L : e->layers)
        for (const EMat* m : {&L.qkv, &L.o, &L.up, &L.down})
            if (m->f16) n += 2 * m->code_bytes();
    return n;
}

// encoder::footprint (encoder/run.rs:613-619): what tb_encoder_open will take for this shape and capacity, before anything is
// allocated.  `f16_matrices` != 0 adds the layers' matrices in f16, which a converted f16 model loads beside the arena.
int tb_encoder_footprint(tb_context* ctx, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, int f16_matrices, size_t* bytes) {
    if (!ctx || !cfg || !bytes || tokens == 0 || sequences == 0) return fail(OUT_OF_RANGE, "tb_encoder_footprint: null or empty argument");
    TB_TRY(enc_validate(*cfg));
    tb_encoder e;
    e.ctx = ctx, e.cfg = *cfg, e.cap_tokens = tokens, e.cap_padded = (tokens + QT - 1) / QT * QT, e.cap_seqs = sequences;
    e.global.assign(cfg->layers, 0);
    e.layers.resize(cfg->layers);
    const char* env = getenv("TACHYON_B200_ENCODER_COPY");
    e.use_copy = !(env && env[0] == '0');
    env = getenv("TACHYON_B200_ENCODER_ROPE");
    e.rope_fused = e.use_copy && env && env[0] == '1' && gemm_persistent_supports(3 * cfg->hidden, cfg->hidden, 16) && cfg->hidden % 16 == 0;
    *bytes = enc_layout(&e, nullptr);
    if (f16_matrices)
        for (const ELayer& L : e.layers)
            for (const EMat* m : {&L.qkv, &L.o, &L.up, &L.down}) *bytes += 2 * m->code_bytes();
    return OK;
}

}  // extern "C"
