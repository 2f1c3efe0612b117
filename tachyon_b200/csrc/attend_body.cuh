// Decode attention, device side: the shared-memory layout, the per-head helpers and the body one block runs for one
// (key-value head, split) work item.  Used by the stand-alone kernel (attend.cu) and by the fused decode step
// (step.cu), which runs it on the first 256 threads of its blocks.
#pragma once

#include "common.cuh"
#include "internal.h"

namespace tb {
namespace attend {

constexpr int D = 256;        // head size
constexpr int TILE = 64;      // positions per shared-memory tile
constexpr int MAXG = 4;       // query heads per key-value head this kernel is built for
constexpr int THREADS = 256;
constexpr int MIN_SPAN = 16;  // fewest positions worth a block of their own

struct Smem {
    __half k[TILE][D];
    __half v[TILE][D];
    float q[MAXG][D];
    float kf[D], vf[D];          // the new token's key and value
    float p[TILE][MAXG];         // scores, then probabilities
    float corr[MAXG], mrun[MAXG], lrun[MAXG];
    uint64_t bar;
    uint32_t last;
};

// RMS-norm (optional weights), RoPE (optional) of one head held as 8 values per lane: dims 4l..4l+3 and 128+4l..128+4l+3.
__device__ __forceinline__ void norm_rope(float (&x)[8], bool norm, const float* w, const float* freq, uint32_t pos, float eps, int lane) {
    if (norm) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) s = fmaf(x[i], x[i], s);
        const float r = rsqrtf(warp_sum(s) / (float)D + eps);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] *= r;
        if (w != nullptr) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(w + 4 * lane)), b = __ldg(reinterpret_cast<const float4*>(w + 128 + 4 * lane));
            x[0] *= a.x, x[1] *= a.y, x[2] *= a.z, x[3] *= a.w, x[4] *= b.x, x[5] *= b.y, x[6] *= b.z, x[7] *= b.w;
        }
    }
    if (freq != nullptr) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(freq + 4 * lane));
        const float fr[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float s, c;
            sincosf((float)pos * fr[i], &s, &c);
            const float a = x[i], b = x[i + 4];
            x[i] = a * c - b * s;
            x[i + 4] = b * c + a * s;
        }
    }
}

__device__ __forceinline__ void load_head(const float* src, float (&x)[8], int lane) {
    const float4 a = ld_cg_f4(src + 4 * lane), b = ld_cg_f4(src + 128 + 4 * lane);
    x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
}

__device__ __forceinline__ void store_head(float* dst, const float (&x)[8], int lane) {
    *reinterpret_cast<float4*>(dst + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(dst + 128 + 4 * lane) = make_float4(x[4], x[5], x[6], x[7]);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void store_head_f16(__half* dst, const float (&x)[8], int lane) {
    *reinterpret_cast<uint2*>(dst + 4 * lane) = make_uint2(pack_half2(x[0], x[1]), pack_half2(x[2], x[3]));
    *reinterpret_cast<uint2*>(dst + 128 + 4 * lane) = make_uint2(pack_half2(x[4], x[5]), pack_half2(x[6], x[7]));
}

// Synchronises the 256 threads that run the body: the whole block of the stand-alone kernel, or a named barrier of
// the fused step's first eight warps.
template <bool FUSED>
__device__ __forceinline__ void block_sync() {
    if constexpr (FUSED) named_bar_sync(3, THREADS);
    else __syncthreads();
}

// One work item: key-value head `g`, split `sp`.  `phase` is the parity of sm.bar's next completion; the caller keeps
// it across calls that reuse the barrier.  Every return is taken by all 256 threads together.
// How the newest n positions are split over at most `splits` blocks: positions per block.  Spans longer than a tile are
// whole tiles, so that no block is left with a sliver of a second tile.
__device__ __forceinline__ uint32_t split_span(uint32_t n, uint32_t splits) {
    uint32_t span = max((n + splits - 1) / splits, (uint32_t)MIN_SPAN);
    if (span > (uint32_t)TILE) span = (span + TILE - 1) / TILE * TILE;
    return span;
}

// Thread 0's part of loading a tile: rows of ages [a0, a0 + cnt) of key-value head `g` (without the new token's row
// when `has_new`), as one or two contiguous ranges of ring slots, completing on `bar`.
__device__ __forceinline__ void issue_tile(const AttendParams& p, Smem& sm, uint64_t* bar, uint32_t g, uint32_t cur, uint32_t a0, uint32_t cnt,
                                           bool has_new) {
    const uint32_t loaded = has_new ? cnt - 1 : cnt;
    if (loaded == 0) return;
    const uint32_t first = (cur + p.cap - (a0 + cnt - 1)) % p.cap;  // slot of row 0
    const uint32_t head_rows = min(loaded, p.cap - first), tail_rows = loaded - head_rows;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier accesses to the tile's memory precede its refill
    mbar_expect_tx(bar, loaded * D * 2 * 2);
    const __half* kb = p.kc + (size_t)g * p.cap * D;
    const __half* vb = p.vc + (size_t)g * p.cap * D;
    bulk_load(&sm.k[0][0], kb + (size_t)first * D, head_rows * D * 2, bar);
    bulk_load(&sm.v[0][0], vb + (size_t)first * D, head_rows * D * 2, bar);
    if (tail_rows > 0) {
        bulk_load(&sm.k[head_rows][0], kb, tail_rows * D * 2, bar);
        bulk_load(&sm.v[head_rows][0], vb, tail_rows * D * 2, bar);
    }
}

// The first tile of work item (g, sp) at position `pos`: issues its loads (thread 0 calls this; the body is then told
// the tile is already on its way).  Returns false when the item has nothing to load.
__device__ __forceinline__ bool issue_first_tile(const AttendParams& p, Smem& sm, uint64_t* bar, uint32_t g, uint32_t sp, uint32_t pos) {
    const uint32_t n = min(pos + 1, p.window), cur = pos % p.cap;
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    if (sp >= used) return false;
    const uint32_t a_begin = sp * span, a_end = min(n, a_begin + span);
    const uint32_t cnt = min((uint32_t)TILE, a_end - a_begin);
    const bool has_new = p.fresh != 0 && sp == 0;
    if ((has_new ? cnt - 1 : cnt) == 0) return false;
    issue_tile(p, sm, bar, g, cur, a_begin, cnt, has_new);
    return true;
}

template <int G, bool FUSED>
__device__ __forceinline__ void attend_body(const AttendParams& p, Smem& sm, uint64_t* bar, const int tid, const uint32_t g, const uint32_t sp,
                                            const uint32_t pos, const bool preloaded, uint32_t* status, uint32_t& phase) {
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t n = min(pos + 1, p.window), cur = pos % p.cap;
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    if (sp >= used) return;
    const uint32_t a_begin = sp * span, a_end = min(n, a_begin + span);  // ages: 0 is the new token
    const bool fresh_here = p.fresh != 0 && sp == 0;
    const bool norms = p.q_norm != nullptr;
    const float qscale = p.scale * 1.4426950408889634f;  // scores in base 2

    // Queries of the group (warps 0..G-1), the new key (warp G) and value (warp G+1).
    if (warp < G) {
        float x[8];
        load_head(p.qkv + (size_t)(g * G + warp) * D, x, lane);
        norm_rope(x, norms, p.q_norm, p.freq, pos, p.eps, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] *= qscale;
        store_head(sm.q[warp], x, lane);
    } else if (fresh_here && warp == G) {
        float x[8];
        load_head(p.qkv + (size_t)(p.heads + g) * D, x, lane);
        norm_rope(x, norms, p.k_norm, p.freq, pos, p.eps, lane);
        store_head(sm.kf, x, lane);
        store_head_f16(p.kc + ((size_t)g * p.cap + cur) * D, x, lane);
    } else if (fresh_here && warp == G + 1) {
        float x[8];
        load_head(p.qkv + (size_t)(p.heads + p.kv_heads + g) * D, x, lane);
        norm_rope(x, norms, nullptr, nullptr, pos, p.eps, lane);
        store_head(sm.vf, x, lane);
        store_head_f16(p.vc + ((size_t)g * p.cap + cur) * D, x, lane);
    }
    if (tid < G) sm.mrun[tid] = -INFINITY, sm.lrun[tid] = 0.0f;

    float acc[G];
#pragma unroll
    for (int h = 0; h < G; h++) acc[h] = 0.0f;
    bool ok = true;
    for (uint32_t a0 = a_begin; a0 < a_end; a0 += TILE) {
        const uint32_t cnt = min((uint32_t)TILE, a_end - a0);
        // Rows of the tile: row r holds age a0 + cnt - 1 - r, so rows are ascending ring slots.  The new token (age 0)
        // would be the last row of the first tile; it is taken from kf / vf instead and not loaded.
        const bool has_new = fresh_here && a0 == 0;
        const uint32_t loaded = has_new ? cnt - 1 : cnt;
        block_sync<FUSED>();  // the previous tile is no longer read; q, kf, vf, mrun are written
        if (tid == 0 && !(preloaded && a0 == a_begin)) issue_tile(p, sm, bar, g, cur, a0, cnt, has_new);
        if (loaded > 0) {
            if (ok && !mbar_wait(bar, phase)) {
                atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                ok = false;
            }
            phase ^= 1;
        }
        // Scores: one warp per row, a lane holds eight dimensions of the key and of each query.
        float qr[G][8];
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float4 a = *reinterpret_cast<const float4*>(&sm.q[h][8 * lane]), b = *reinterpret_cast<const float4*>(&sm.q[h][8 * lane + 4]);
            qr[h][0] = a.x, qr[h][1] = a.y, qr[h][2] = a.z, qr[h][3] = a.w, qr[h][4] = b.x, qr[h][5] = b.y, qr[h][6] = b.z, qr[h][7] = b.w;
        }
        for (uint32_t r = warp; r < cnt; r += THREADS / 32) {
            float kv[8];
            if (has_new && r == cnt - 1) {
                const float4 a = *reinterpret_cast<const float4*>(&sm.kf[8 * lane]), b = *reinterpret_cast<const float4*>(&sm.kf[8 * lane + 4]);
                kv[0] = a.x, kv[1] = a.y, kv[2] = a.z, kv[3] = a.w, kv[4] = b.x, kv[5] = b.y, kv[6] = b.z, kv[7] = b.w;
            } else {
                const uint4 t = *reinterpret_cast<const uint4*>(&sm.k[r][8 * lane]);
                const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    kv[2 * j] = f.x, kv[2 * j + 1] = f.y;
                }
            }
            float sc[G];
#pragma unroll
            for (int h = 0; h < G; h++) {
                sc[h] = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) sc[h] = fmaf(qr[h][i], kv[i], sc[h]);
            }
            // Reduce the G sums together: the halves (then quarters) of the warp trade values, so head h ends up summed
            // in the lanes whose top bits spell h.
            float v;
            if constexpr (G == 4) {
                const bool b4 = lane & 16, b3 = lane & 8;
                const float k0 = (b4 ? sc[2] : sc[0]) + __shfl_xor_sync(0xffffffffu, b4 ? sc[0] : sc[2], 16);
                const float k1 = (b4 ? sc[3] : sc[1]) + __shfl_xor_sync(0xffffffffu, b4 ? sc[1] : sc[3], 16);
                v = (b3 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, b3 ? k0 : k1, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                if ((lane & 7) == 0) sm.p[r][lane >> 3] = ok ? v : 0.0f;
            } else if constexpr (G == 2) {
                const bool b4 = lane & 16;
                v = (b4 ? sc[1] : sc[0]) + __shfl_xor_sync(0xffffffffu, b4 ? sc[0] : sc[1], 16);
#pragma unroll
                for (int o2 = 8; o2 > 0; o2 >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o2);
                if ((lane & 15) == 0) sm.p[r][lane >> 4] = ok ? v : 0.0f;
            } else {
                v = warp_sum(sc[0]);
                if (lane == 0) sm.p[r][0] = ok ? v : 0.0f;
            }
        }
        block_sync<FUSED>();
        // Softmax statistics: warp h owns query head h.
        if (warp < G) {
            float m = -INFINITY;
            for (uint32_t r = lane; r < cnt; r += 32) m = fmaxf(m, sm.p[r][warp]);
            m = warp_max(m);
            const float mold = sm.mrun[warp], mnew = fmaxf(mold, m);
            float l = 0.0f;
            for (uint32_t r = lane; r < cnt; r += 32) {
                const float e = exp2f(sm.p[r][warp] - mnew);
                sm.p[r][warp] = e;
                l += e;
            }
            l = warp_sum(l);
            if (lane == 0) {
                const float c = exp2f(mold - mnew);  // 0 on the first tile (mold = -inf)
                sm.corr[warp] = c;
                sm.mrun[warp] = mnew;
                sm.lrun[warp] = sm.lrun[warp] * c + l;
            }
        }
        block_sync<FUSED>();
        // Values: one thread per dimension, all heads of the group.
#pragma unroll
        for (int h = 0; h < G; h++) acc[h] *= sm.corr[h];
        for (uint32_t r = 0; r < cnt; r++) {
            const float vv = (has_new && r == cnt - 1) ? sm.vf[tid] : __half2float(sm.v[r][tid]);
#pragma unroll
            for (int h = 0; h < G; h++) acc[h] = fmaf(sm.p[r][h], vv, acc[h]);
        }
    }

    const uint32_t stride = 2 * G + G * D;  // floats per partial: maxima, sums, outputs
    if (p.defer) {
        // The consumer of the output merges the splits itself: leave this split's statistics and sums, nothing else.
        float* mine = p.partial + (size_t)(g * p.splits + sp) * stride;
        if (tid < G) mine[tid] = sm.mrun[tid], mine[G + tid] = sm.lrun[tid];
#pragma unroll
        for (int h = 0; h < G; h++) mine[2 * G + h * D + tid] = acc[h];
        return;
    }
    if (used == 1) {
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float o = acc[h] / sm.lrun[h];
            const size_t at = (size_t)(g * G + h) * D + tid;
            if (p.out_f16) static_cast<__half*>(p.out)[at] = __float2half_rn(o);
            else static_cast<float*>(p.out)[at] = o;
        }
        return;
    }
    float* mine = p.partial + (size_t)(g * p.splits + sp) * stride;
    if (tid < G) mine[tid] = sm.mrun[tid], mine[G + tid] = sm.lrun[tid];
#pragma unroll
    for (int h = 0; h < G; h++) mine[2 * G + h * D + tid] = acc[h];
    __threadfence();
    block_sync<FUSED>();
    if (tid == 0) sm.last = (atomicAdd(p.count + g, 1u) == used - 1) ? 1u : 0u;
    block_sync<FUSED>();
    if (sm.last == 0) return;
    __threadfence();
    // Combine (attend.rs:371-405): weights 2^(m_s - M) over the splits that ran.  Every load of a phase is issued
    // before its first use, so the phases cost one trip to the L2 each, not one per split.
    const float* base = p.partial + (size_t)g * p.splits * stride;
    float* wts = reinterpret_cast<float*>(&sm.k[0][0]);  // [used][G], the tile is no longer needed
    for (uint32_t i = tid; i < used * G; i += THREADS) wts[i] = __ldcg(base + (size_t)(i / G) * stride + i % G);
    block_sync<FUSED>();
    if (warp < G) {
        float M = -INFINITY, L = 0.0f;
        for (uint32_t s2 = lane; s2 < used; s2 += 32) M = fmaxf(M, wts[s2 * G + warp]);
        M = warp_max(M);
        for (uint32_t s2 = lane; s2 < used; s2 += 32) {
            const float wgt = exp2f(wts[s2 * G + warp] - M);
            L = fmaf(wgt, __ldcg(base + (size_t)s2 * stride + G + warp), L);
            wts[s2 * G + warp] = wgt;
        }
        L = warp_sum(L);
        if (lane == 0) sm.lrun[warp] = L;
    }
    block_sync<FUSED>();
    float o[G];
#pragma unroll
    for (int h = 0; h < G; h++) o[h] = 0.0f;
    uint32_t s2 = 0;
    for (; s2 + 4 <= used; s2 += 4) {
        float t[4][G];
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int h = 0; h < G; h++) t[u][h] = __ldcg(base + (size_t)(s2 + u) * stride + 2 * G + h * D + tid);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int h = 0; h < G; h++) o[h] = fmaf(wts[(s2 + u) * G + h], t[u][h], o[h]);
    }
    for (; s2 < used; s2++)
#pragma unroll
        for (int h = 0; h < G; h++) o[h] = fmaf(wts[s2 * G + h], __ldcg(base + (size_t)s2 * stride + 2 * G + h * D + tid), o[h]);
#pragma unroll
    for (int h = 0; h < G; h++) {
        const float r = o[h] / sm.lrun[h];
        const size_t at = (size_t)(g * G + h) * D + tid;
        if (p.out_f16) static_cast<__half*>(p.out)[at] = __float2half_rn(r);
        else static_cast<float*>(p.out)[at] = r;
    }
    if (tid == 0) p.count[g] = 0;
}

}  // namespace attend
}  // namespace tb
