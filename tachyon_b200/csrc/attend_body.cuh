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

constexpr int ROW = D + 8;    // halves between rows of a tile: 16 bytes of padding put eight neighbouring rows on different banks
constexpr int PROW = TILE + 8;  // the same for the transposed probabilities

struct Smem {
    __half k[TILE][ROW];
    __half v[TILE][ROW];
    float q[MAXG][D + 8];        // the queries, scaled (rows padded: the fragment build reads four rows at once); after the last tile the outputs on their way to the old layout
    float kf[D], vf[D];          // the new token's key and value
    float s[2][TILE][8];         // raw scores: [half of the dimensions][row][column]; column h is head h's high part, G + h its low part
    __half pt[8][PROW];          // probabilities, transposed: row h the f16 value of head h's, row G + h what the f16 leaves of it
    float pnew[MAXG];            // probability of the new token's row
    float corr[MAXG], mrun[MAXG], lrun[MAXG];
    uint32_t last;
};

// The stand-alone kernel's shared memory: the above, and what the other blocks of a thread-block cluster write here
// (AttendParams::cluster > 1): every split's maxima and sums, and of every split's outputs the slice of dimensions this
// block merges.  Nothing else may live in these arrays: a neighbour that finishes first writes while this block is still
// at work.
struct ClusterSmem {
    Smem body;
    float xstats[8][2 * MAXG];
    float xacc[MAXG * D];  // [split][head][dimension within the slice of D / cluster]
};

// cos and sin of the position's angle for the four dimension pairs a lane rotates: (4l + i, 128 + 4l + i).  They depend
// on the position alone, so a kernel can have them ready before its input arrives.
struct Trig {
    float c[4], s[4];
};
__device__ __forceinline__ Trig rope_trig(const float* freq, uint32_t pos, int lane, const float* table = nullptr) {
    Trig t;
    if (table != nullptr) {  // the same values, computed once per position when the table was filled
        const float4 c = __ldg(reinterpret_cast<const float4*>(table + (size_t)pos * D + 4 * lane));
        const float4 s = __ldg(reinterpret_cast<const float4*>(table + (size_t)pos * D + D / 2 + 4 * lane));
        t.c[0] = c.x, t.c[1] = c.y, t.c[2] = c.z, t.c[3] = c.w, t.s[0] = s.x, t.s[1] = s.y, t.s[2] = s.z, t.s[3] = s.w;
        return t;
    }
    if (freq == nullptr) {
#pragma unroll
        for (int i = 0; i < 4; i++) t.c[i] = 1.0f, t.s[i] = 0.0f;
        return t;
    }
    const float4 f = __ldg(reinterpret_cast<const float4*>(freq + 4 * lane));
    const float fr[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
    for (int i = 0; i < 4; i++) sincosf((float)pos * fr[i], &t.s[i], &t.c[i]);
    return t;
}

// RMS-norm (optional weights), RoPE (optional) of one head held as 8 values per lane: dims 4l..4l+3 and 128+4l..128+4l+3.
__device__ __forceinline__ void norm_rope(float (&x)[8], bool norm, const float* w, const Trig* trig, float eps, int lane) {
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
    if (trig != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float a = x[i], b = x[i + 4];
            x[i] = a * trig->c[i] - b * trig->s[i];
            x[i + 4] = b * trig->c[i] + a * trig->s[i];
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

// How the newest n positions are split over at most `splits` blocks: positions per block.  Spans longer than a tile are
// whole tiles, so that no block is left with a sliver of a second tile.
__device__ __forceinline__ uint32_t split_span(uint32_t n, uint32_t splits) {
    uint32_t span = max((n + splits - 1) / splits, (uint32_t)MIN_SPAN);
    if (span > (uint32_t)TILE) span = (span + TILE - 1) / TILE * TILE;
    return span;
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// x = hi + lo with both f16: the tensor cores then multiply x to nearly f32 precision in two columns (or rows).
__device__ __forceinline__ void split_f16(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

// The 256 threads' part of loading a tile: rows of ages [a0, a0 + cnt) of key-value head `g` (without the new token's
// row when `has_new`), in 16-byte asynchronous copies into the padded rows.  Rows of the value tile that stay unused
// are cleared: the tensor cores multiply them by zero, which must not meet a NaN left by an earlier tile.
// The caller commits the copies.
__device__ __forceinline__ void load_tile(const AttendParams& p, Smem& sm, uint32_t g, uint32_t cur, uint32_t a0, uint32_t cnt, bool has_new, int tid) {
    const uint32_t loaded = has_new ? cnt - 1 : cnt;
    const uint32_t first = (cur + p.cap - (a0 + cnt - 1)) % p.cap;  // slot of row 0
    const __half* kb = p.kc + (size_t)g * p.cap * D;
    const __half* vb = p.vc + (size_t)g * p.cap * D;
    // Thread t takes 16-byte piece t % 64 (0..31 of the key, 32..63 of the value) of rows t / 64, t / 64 + 4, ...
    const uint32_t j = (uint32_t)tid % 64, piece = (j & 31) * 8;
    const __half* src = (j < 32 ? kb : vb) + piece;
    __half* dst = (j < 32 ? &sm.k[0][0] : &sm.v[0][0]) + piece;
    uint32_t slot = first + (uint32_t)tid / 64;
    if (slot >= p.cap) slot -= p.cap;
#pragma unroll 4
    for (uint32_t r = (uint32_t)tid / 64; r < TILE; r += THREADS / 64) {
        if (r < loaded) cp_async_16(dst + r * ROW, src + (size_t)slot * D);
        else if (j >= 32) *reinterpret_cast<uint4*>(dst + r * ROW) = make_uint4(0u, 0u, 0u, 0u);
        slot += THREADS / 64;
        if (slot >= p.cap) slot -= p.cap;
    }
}

// The first tile of work item (g, sp) at position `pos`, asked for before the rest of the body runs (all 256 threads
// call this and commit; the body is then told the tile is on its way).  Returns false when the item has no tile.
__device__ __forceinline__ bool load_first_tile(const AttendParams& p, Smem& sm, uint32_t g, uint32_t sp, uint32_t pos, int tid) {
    const uint32_t n = min(pos + 1, p.window), cur = pos % p.cap;
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    if (sp >= used) return false;
    const uint32_t a_begin = sp * span, a_end = min(n, a_begin + span);
    const uint32_t cnt = min((uint32_t)TILE, a_end - a_begin);
    load_tile(p, sm, g, cur, a_begin, cnt, p.fresh != 0 && sp == 0, tid);
    cp_async_commit();
    return true;
}

// One work item: key-value head `g`, split `sp`.  Every return is taken by all 256 threads together.
//
// The two products run on the tensor cores (mma.sync m16n8k16, f16 operands, f32 accumulation): a 64-row tile is far
// too little work to be worth anything else, and what matters is how few dependent instructions stand between the
// arrival of the query and the partial result.  The f32 query is split into two f16 numbers (columns h and G + h of
// the scores' B operand), and so are the probabilities (rows h and G + h of the second product's A operand), so
// the only rounding beyond the f32 path's is the accumulation order.  The cache is f16 as it is.
//   scores[row][col] = K[row][:] . q[col][:]      M = 64 rows (four 16-row tiles), N = 8, K = 256: warp w takes
//                                                 row tile w % 4 and dimensions 128 (w / 4) .. + 127
//   out[m][dim]      = P[m][:] . V[:][dim]        M = 16 (2G rows used), N = 256 (warp w: 32 w .. + 31), K = 64 rows
// This part leaves the split's statistics in sm.mrun / sm.lrun and its unnormalised outputs in out[h] (dimension tid of
// head h); false when the split has no positions.
template <int G, bool FUSED>
__device__ __forceinline__ bool attend_partial(const AttendParams& p, Smem& sm, const int tid, const uint32_t g, const uint32_t sp, const uint32_t pos,
                                               const bool preloaded, const Trig& trig, float (&out)[G]) {
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t n = min(pos + 1, p.window), cur = pos % p.cap;
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    if (sp >= used) return false;
    const uint32_t a_begin = sp * span, a_end = min(n, a_begin + span);  // ages: 0 is the new token
    const bool fresh_here = p.fresh != 0 && sp == 0;
    const bool norms = p.q_norm != nullptr;
    const Trig* rot = p.freq != nullptr ? &trig : nullptr;
    const float qscale = p.scale * 1.4426950408889634f;  // scores in base 2

    // Queries of the group (warps 0..G-1), the new key (warp G) and value (warp G+1).
    if (warp < G) {
        float x[8];
        load_head(p.qkv + (size_t)(g * G + warp) * D, x, lane);
        norm_rope(x, norms, p.q_norm, rot, p.eps, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] *= qscale;
        store_head(sm.q[warp], x, lane);
    } else if (fresh_here && warp == G) {
        float x[8];
        load_head(p.qkv + (size_t)(p.heads + g) * D, x, lane);
        norm_rope(x, norms, p.k_norm, rot, p.eps, lane);
        store_head(sm.kf, x, lane);
        store_head_f16(p.kc + ((size_t)g * p.cap + cur) * D, x, lane);
    } else if (fresh_here && warp == G + 1) {
        float x[8];
        load_head(p.qkv + (size_t)(p.heads + p.kv_heads + g) * D, x, lane);
        norm_rope(x, norms, nullptr, nullptr, p.eps, lane);
        store_head(sm.vf, x, lane);
        store_head_f16(p.vc + ((size_t)g * p.cap + cur) * D, x, lane);
    }
    if (tid < G) sm.mrun[tid] = -INFINITY, sm.lrun[tid] = 0.0f;
    // Rows 2G..7 of the transposed probabilities are never written: they are the unused rows of the A operand.
    for (int i = tid; i < 8 * PROW / 2; i += THREADS) reinterpret_cast<uint32_t*>(&sm.pt[0][0])[i] = 0u;
    block_sync<FUSED>();  // q, kf, vf are written

    // The scores' B operand for this warp's half of the dimensions: column c = lane / 4 is the high part of head c
    // (c < G), the low part of head c - G (c < 2G), or nothing; a thread holds dimensions 16 ks + 2 (lane % 4) + {0, 1, 8, 9}.
    const int khalf = warp >> 2, mtile = warp & 3;
    uint32_t qb[8][2];
    {
        const int c = lane >> 2;
        const bool use = c < 2 * G, low = c >= G;
        const float* qh = sm.q[use ? (low ? c - G : c) : 0];
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const int d = khalf * 128 + ks * 16 + 2 * (lane & 3);
            const float2 x0 = *reinterpret_cast<const float2*>(qh + d), x1 = *reinterpret_cast<const float2*>(qh + d + 8);
            __half h0, l0, h1, l1, h2, l2, h3, l3;
            split_f16(x0.x, h0, l0), split_f16(x0.y, h1, l1), split_f16(x1.x, h2, l2), split_f16(x1.y, h3, l3);
            const __half2 b0 = low ? __halves2half2(l0, l1) : __halves2half2(h0, h1), b1 = low ? __halves2half2(l2, l3) : __halves2half2(h2, h3);
            qb[ks][0] = use ? *reinterpret_cast<const uint32_t*>(&b0) : 0u;
            qb[ks][1] = use ? *reinterpret_cast<const uint32_t*>(&b1) : 0u;
        }
    }

    // Outputs: this warp's four 8-dimension tiles; element 0, 1 of each is row lane / 4, dimensions 2 (lane % 4) + {0, 1}.
    float acc[4][4];
#pragma unroll
    for (int t = 0; t < 4; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[t][i] = 0.0f;
    const int orow = lane >> 2;       // row of the second product this thread holds
    const int ohead = orow % G;      // its head (rows >= 2G hold zeros)

    for (uint32_t a0 = a_begin; a0 < a_end; a0 += TILE) {
        const uint32_t cnt = min((uint32_t)TILE, a_end - a0);
        // Rows of the tile: row r holds age a0 + cnt - 1 - r, so rows are ascending ring slots.  The new token (age 0)
        // would be the last row of the first tile; it is taken from kf / vf instead and not loaded.
        const bool has_new = fresh_here && a0 == 0;
        const uint32_t loaded = has_new ? cnt - 1 : cnt;
        if (!(preloaded && a0 == a_begin)) {
            if (a0 != a_begin) block_sync<FUSED>();  // the previous tile is no longer read
            load_tile(p, sm, g, cur, a0, cnt, has_new, tid);
            cp_async_commit();
        }
        cp_async_wait_all();
        block_sync<FUSED>();

        // Scores of 16 rows over 128 dimensions, in two chains of four products.
        {
            float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const __half* base = &sm.k[mtile * 16 + (lane & 15)][khalf * 128 + (lane >> 4) * 8];
#pragma unroll
            for (int ks = 0; ks < 8; ks += 2) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, base + ks * 16);
                ldmatrix_x4(b, base + ks * 16 + 16);
                mma_16816(c0, a[0], a[1], a[2], a[3], qb[ks][0], qb[ks][1]);
                mma_16816(c1, b[0], b[1], b[2], b[3], qb[ks + 1][0], qb[ks + 1][1]);
            }
            float* out = &sm.s[khalf][mtile * 16 + (lane >> 2)][2 * (lane & 3)];
            *reinterpret_cast<float2*>(out) = make_float2(c0[0] + c1[0], c0[1] + c1[1]);
            *reinterpret_cast<float2*>(out + 8 * 8) = make_float2(c0[2] + c1[2], c0[3] + c1[3]);
        }
        block_sync<FUSED>();
        // Softmax statistics: warp h owns query head h; a lane takes rows lane and lane + 32.
        if (warp < G) {
            float fresh_score = 0.0f;
            if (has_new) {  // the new token's key is still f32
                const float4 ka = *reinterpret_cast<const float4*>(&sm.kf[8 * lane]), kb = *reinterpret_cast<const float4*>(&sm.kf[8 * lane + 4]);
                const float4 qa = *reinterpret_cast<const float4*>(&sm.q[warp][8 * lane]), qc = *reinterpret_cast<const float4*>(&sm.q[warp][8 * lane + 4]);
                fresh_score = warp_sum(ka.x * qa.x + ka.y * qa.y + ka.z * qa.z + ka.w * qa.w + kb.x * qc.x + kb.y * qc.y + kb.z * qc.z + kb.w * qc.w);
            }
            float sc[TILE / 32];
            float m = -INFINITY;
#pragma unroll
            for (int u = 0; u < TILE / 32; u++) {
                const uint32_t r = lane + 32 * u;
                float v = -INFINITY;
                if (r < loaded) v = (sm.s[0][r][warp] + sm.s[1][r][warp]) + (sm.s[0][r][G + warp] + sm.s[1][r][G + warp]);
                else if (r < cnt) v = fresh_score;
                sc[u] = v;
                m = fmaxf(m, v);
            }
            m = warp_max(m);
            const float mold = sm.mrun[warp], mnew = fmaxf(mold, m);
            float l = 0.0f;
#pragma unroll
            for (int u = 0; u < TILE / 32; u++) {
                const uint32_t r = lane + 32 * u;
                const float e = r < cnt ? exp2f(sc[u] - mnew) : 0.0f;
                l += e;
                __half hi, lo;
                split_f16(r < loaded ? e : 0.0f, hi, lo);  // the new token's row goes through vf, not through the tile
                sm.pt[warp][r] = hi, sm.pt[G + warp][r] = lo;
                if (has_new && r == cnt - 1) sm.pnew[warp] = e;
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
        // Values.
        {
            const float c = sm.corr[ohead];
#pragma unroll
            for (int t = 0; t < 4; t++) acc[t][0] *= c, acc[t][1] *= c;
#pragma unroll
            for (int ks = 0; ks < TILE / 16; ks++) {
                const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&sm.pt[orow][ks * 16 + 2 * (lane & 3)]);
                const uint32_t pa2 = *reinterpret_cast<const uint32_t*>(&sm.pt[orow][ks * 16 + 8 + 2 * (lane & 3)]);
#pragma unroll
                for (int t = 0; t < 4; t += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, &sm.v[ks * 16 + (lane & 15)][warp * 32 + t * 8 + (lane >> 4) * 8]);
                    mma_16816(acc[t], pa0, 0u, pa2, 0u, b[0], b[1]);
                    mma_16816(acc[t + 1], pa0, 0u, pa2, 0u, b[2], b[3]);
                }
            }
            if (has_new && orow < G) {
                const float pn = sm.pnew[orow];
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const float2 vf = *reinterpret_cast<const float2*>(&sm.vf[warp * 32 + t * 8 + 2 * (lane & 3)]);
                    acc[t][0] = fmaf(pn, vf.x, acc[t][0]), acc[t][1] = fmaf(pn, vf.y, acc[t][1]);
                }
            }
        }
    }
    // High and low rows together, then through shared memory to one thread per dimension with all heads of the group.
    block_sync<FUSED>();  // the queries are no longer read
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const float v0 = acc[t][0] + __shfl_xor_sync(0xffffffffu, acc[t][0], 4 * G);
        const float v1 = acc[t][1] + __shfl_xor_sync(0xffffffffu, acc[t][1], 4 * G);
        if (orow < G) *reinterpret_cast<float2*>(&sm.q[orow][warp * 32 + t * 8 + 2 * (lane & 3)]) = make_float2(v0, v1);
    }
    block_sync<FUSED>();
#pragma unroll
    for (int h = 0; h < G; h++) out[h] = sm.q[h][tid];
    return true;
}

template <int G, bool FUSED>
__device__ __forceinline__ void attend_body(const AttendParams& p, Smem& sm, const int tid, const uint32_t g, const uint32_t sp, const uint32_t pos,
                                            const bool preloaded, const Trig& trig) {
    float out[G];
    if (!attend_partial<G, FUSED>(p, sm, tid, g, sp, pos, preloaded, trig, out)) return;
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t n = min(pos + 1, p.window);
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    constexpr uint32_t HD = attend_header(G);
    const uint32_t stride = HD + G * D;  // floats per partial: maxima, sums (padded), outputs
    if (p.defer) {
        // The consumer of the output merges the splits itself: leave this split's statistics and sums, nothing else.
        float* mine = p.partial + (size_t)(g * p.splits + sp) * stride;
        if (tid < G) mine[tid] = sm.mrun[tid], mine[G + tid] = sm.lrun[tid];
#pragma unroll
        for (int h = 0; h < G; h++) mine[HD + h * D + tid] = out[h];
        return;
    }
    if (used == 1) {
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float o = out[h] / sm.lrun[h];
            const size_t at = (size_t)(g * G + h) * D + tid;
            if (p.out_f16 == 2) q8_store(o, (uint32_t)at, static_cast<int8_t*>(p.out), reinterpret_cast<float2*>(p.out_pairs));
            else if (p.out_f16) static_cast<__half*>(p.out)[at] = __float2half_rn(o);
            else static_cast<float*>(p.out)[at] = o;
        }
        return;
    }
    float* mine = p.partial + (size_t)(g * p.splits + sp) * stride;
    if (tid < G) mine[tid] = sm.mrun[tid], mine[G + tid] = sm.lrun[tid];
#pragma unroll
    for (int h = 0; h < G; h++) mine[HD + h * D + tid] = out[h];
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
            for (int h = 0; h < G; h++) t[u][h] = __ldcg(base + (size_t)(s2 + u) * stride + HD + h * D + tid);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int h = 0; h < G; h++) o[h] = fmaf(wts[(s2 + u) * G + h], t[u][h], o[h]);
    }
    for (; s2 < used; s2++)
#pragma unroll
        for (int h = 0; h < G; h++) o[h] = fmaf(wts[s2 * G + h], __ldcg(base + (size_t)s2 * stride + HD + h * D + tid), o[h]);
#pragma unroll
    for (int h = 0; h < G; h++) {
        const float r = o[h] / sm.lrun[h];
        const size_t at = (size_t)(g * G + h) * D + tid;
        if (p.out_f16 == 2) q8_store(r, (uint32_t)at, static_cast<int8_t*>(p.out), reinterpret_cast<float2*>(p.out_pairs));
        else if (p.out_f16) static_cast<__half*>(p.out)[at] = __float2half_rn(r);
        else static_cast<float*>(p.out)[at] = r;
    }
    if (tid == 0) p.count[g] = 0;
}

// ---- splits merged inside a thread-block cluster ---------------------------------------------------------------------
//
// With AttendParams::cluster = C > 1 the grid is launched in clusters of C blocks along the splits.  The C splits of a
// cluster meet in distributed shared memory instead of global memory: every block sends its maxima and sums to all, and of
// its outputs to each block the slice of D / C dimensions that block merges; after one cluster barrier each block
// combines its slice over the splits (weights 2^(m_s - M), attend.rs:371-405) and writes it to entry (first split / C) of
// `partial`, still unnormalised, with the merged maximum and sum.  The product that follows reads one entry per cluster
// instead of one per split.  A block whose split is empty still takes part: it owns a slice.

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
    cluster_arrive();
    cluster_wait();
}
// Stores v at the address `local` has in block `rank` of the cluster.
__device__ __forceinline__ void st_cluster(const float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int G>
__device__ __forceinline__ void attend_cluster_body(const AttendParams& p, ClusterSmem& cs, const int tid, const uint32_t g, const uint32_t sp, const uint32_t pos,
                                                    const bool preloaded, const Trig& trig) {
    const uint32_t C = p.cluster, rank = cluster_rank(), slice = D / C;
    const uint32_t n = min(pos + 1, p.window);
    const uint32_t span = split_span(n, p.splits);
    const uint32_t used = (n + span - 1) / span;
    const uint32_t first = sp - rank;  // the cluster's first split
    if (first >= used) return;         // a cluster without positions: all of its blocks leave, nobody writes to anybody
    const uint32_t here = min(C, used - first);  // splits of this cluster that have positions
    // A block's shared memory may be written from outside only once the block runs: every block says so here and checks
    // the others right before its first store to them, with its own work in between.
    cluster_arrive();
    float out[G];
#pragma unroll
    for (int h = 0; h < G; h++) out[h] = 0.0f;
    Smem& sm = cs.body;
    const bool active = attend_partial<G, false>(p, sm, tid, g, sp, pos, preloaded, trig, out);
    cluster_wait();
    if (active) {
        if (tid < 2 * G) {
            const float v = tid < G ? sm.mrun[tid] : sm.lrun[tid - G];
            for (uint32_t peer = 0; peer < C; peer++) st_cluster(&cs.xstats[rank][tid], peer, v);
        }
        const uint32_t owner = (uint32_t)tid / slice, dd = (uint32_t)tid % slice;
#pragma unroll
        for (int h = 0; h < G; h++) st_cluster(&cs.xacc[(rank * G + h) * slice + dd], owner, out[h]);
    }
    cluster_sync();
    for (uint32_t idx = (uint32_t)tid; idx < G * slice; idx += THREADS) {  // up to G * D / 2 outputs a block
        const uint32_t h = idx / slice, dd = idx % slice;
        float M = -INFINITY;
        for (uint32_t s = 0; s < here; s++) M = fmaxf(M, cs.xstats[s][h]);
        float L = 0.0f, o = 0.0f;
        for (uint32_t s = 0; s < here; s++) {
            const float wgt = exp2f(cs.xstats[s][h] - M);
            L = fmaf(wgt, cs.xstats[s][G + h], L);
            o = fmaf(wgt, cs.xacc[(s * G + h) * slice + dd], o);
        }
        float* entry = p.partial + (size_t)(g * p.splits + first / C) * (attend_header(G) + G * D);
        entry[attend_header(G) + h * D + rank * slice + dd] = o;
        if (rank == 0 && dd == 0) entry[h] = M, entry[G + h] = L;
    }
}

}  // namespace attend
}  // namespace tb
