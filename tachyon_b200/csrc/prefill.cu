// The kernels around the prefill GEMMs, one chunk of prompt tokens at a time: embedding rows, the residual/RMS-norm
// step per token (quant_q8p / norm_q8p's place, crates/tachyon/src/ptx/mod.rs:253-287, 491-511), query and key/value
// preparation (query_256 and kv_256, ptx/attend.rs:472-556) and causal / sliding-window flash attention over the cache
// ring (flash_256, ptx/flash.rs:326-374).  Attention is 2 % of a prefill's arithmetic; it runs on mma.sync with f16
// operands and f32 softmax and accumulators, the GEMMs (98 %) on tcgen05 (gemm.cu).
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int D = 256;

// ---- embedding rows ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prefill_embed_kernel(const int8_t* w, const __half* s, const uint32_t* tokens, uint32_t cols, float scale, float* out,
                                                            uint32_t wbits) {
    const size_t row = (size_t)tokens[blockIdx.x] * cols;
    float* o = out + (size_t)blockIdx.x * cols;
    if (wbits == 4) {  // the reference's Q4 table (quant.rs:60-66)
        const uint8_t* packed = reinterpret_cast<const uint8_t*>(w);
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
            const size_t at = row + i, g = at / 64, k = at % 64;
            const int n = (packed[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
            o[i] = (float)(n - 8) * __half2float(s[g]) * scale;
        }
        return;
    }
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) o[i] = (float)w[row + i] * __half2float(s[(row + i) / 32]) * scale;
}

// ---- residual + norm, one warp per token, 2048 values (64 per lane) ---------------------------------------------------
// h' = (h + w1 * rmsnorm(y)) * hscale when y is given (h updated in place), x = w2 * rmsnorm(h') as f16, or h' itself
// without w2 (what the per-layer input's gate reads).  A warp keeps its token in registers: sixteen 16-byte loads of h
// and of y in flight per lane and two shuffle reductions, no block barrier.
constexpr int NORM_N = 2048, NORM_V = NORM_N / 128;  // float4 per lane
__global__ void __launch_bounds__(256) prefill_norm_kernel(float* h, const float* y, const float* w1, const float* w2, uint32_t tokens, float eps, float hscale,
                                                           __half* x) {
    const uint32_t token = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();  // the product behind sets itself up meanwhile; it reads x only after its own wait
    pdl_wait();               // h and y come from the kernels in front
    if (token >= tokens) return;
    const size_t base = (size_t)token * NORM_N;
    float4 v[NORM_V];
#pragma unroll
    for (int i = 0; i < NORM_V; i++) v[i] = *reinterpret_cast<const float4*>(h + base + (i * 32 + lane) * 4);
    if (y != nullptr) {
        float4 yy[NORM_V];
#pragma unroll
        for (int i = 0; i < NORM_V; i++) yy[i] = __ldcs(reinterpret_cast<const float4*>(y + base + (i * 32 + lane) * 4));
        float sy = 0.0f;
#pragma unroll
        for (int i = 0; i < NORM_V; i++) sy = fmaf(yy[i].x, yy[i].x, fmaf(yy[i].y, yy[i].y, fmaf(yy[i].z, yy[i].z, fmaf(yy[i].w, yy[i].w, sy))));
        const float ry = rsqrtf(warp_sum(sy) / (float)NORM_N + eps);
#pragma unroll
        for (int i = 0; i < NORM_V; i++) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(w1 + (i * 32 + lane) * 4));
            v[i].x = fmaf(yy[i].x * ry, w.x, v[i].x) * hscale, v[i].y = fmaf(yy[i].y * ry, w.y, v[i].y) * hscale;
            v[i].z = fmaf(yy[i].z * ry, w.z, v[i].z) * hscale, v[i].w = fmaf(yy[i].w * ry, w.w, v[i].w) * hscale;
            *reinterpret_cast<float4*>(h + base + (i * 32 + lane) * 4) = v[i];
        }
    }
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_V; i++) sq = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, sq))));
    const float rh = w2 != nullptr ? rsqrtf(warp_sum(sq) / (float)NORM_N + eps) : 1.0f;
#pragma unroll
    for (int i = 0; i < NORM_V; i++) {
        const float4 w = w2 != nullptr ? __ldg(reinterpret_cast<const float4*>(w2 + (i * 32 + lane) * 4)) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        const __half2 a = __floats2half2_rn(v[i].x * rh * w.x, v[i].y * rh * w.y), b2 = __floats2half2_rn(v[i].z * rh * w.z, v[i].w * rh * w.w);
        *reinterpret_cast<uint2*>(x + base + (i * 32 + lane) * 4) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b2));
    }
}

// ---- q / k / v preparation: one warp per (token, head) -----------------------------------------------------------------
// Queries: norm (weights) + RoPE, times scale*log2(e), f16 [token][head][DH].  Keys: norm (weights) + RoPE -> cache
// slot (pos0 + token) % cap; values: norm without weights -> cache.  The reference's kv_256 / kv_512 and query_256 /
// query_512 (crates/tachyon/src/ptx/attend.rs:472-556) in one launch.  A lane holds dims (DH/64) l .. and their RoPE
// partners DH/2 + (DH/64) l ..
// Which rows of a token's projected vector a launch prepares (the whole of it in the decoder; the key and value rows for
// kv_256 / kv_512 and the query rows for query_256 / query_512 when they are launched by name), the floats from one
// token's vector to the next, and, for the launches by name, the chunk's first position in device memory.
struct QkvRows {
    uint32_t first, count, stride;
    const uint32_t* pos;
};

template <int DH>
__global__ void __launch_bounds__(128) prefill_qkv_kernel(const float* qkv, const float* q_norm, const float* k_norm, const float* freq, __half* q_out,
                                                          __half* kc, __half* vc, uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads,
                                                          float eps, float qscale, QkvRows rows_of) {
    constexpr int H2 = DH / 64, NV = 2 * H2;  // values a lane holds of each half, and in all
    const uint32_t item = blockIdx.x * 4 + (threadIdx.x >> 5), token = item / rows_of.count, r = rows_of.first + item % rows_of.count;
    pdl_launch_dependents();  // the attention kernel behind waits for this one before it reads anything
    pdl_wait();               // the projections come from the product in front
    if (token >= tokens) return;  // the last block's spare warps (nothing below synchronises the block)
    if (rows_of.pos != nullptr) pos0 = __ldg(rows_of.pos);
    const int lane = threadIdx.x & 31;
    const float* src = qkv + (size_t)token * rows_of.stride + (size_t)r * DH;
    float x[NV];
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const float4 t = *reinterpret_cast<const float4*>(src + half * (DH / 2) + H2 * lane + 4 * v);
            x[half * H2 + 4 * v] = t.x, x[half * H2 + 4 * v + 1] = t.y, x[half * H2 + 4 * v + 2] = t.z, x[half * H2 + 4 * v + 3] = t.w;
        }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) ss = fmaf(x[i], x[i], ss);
    const float rn = rsqrtf(warp_sum(ss) / (float)DH + eps);
    const bool is_q = r < heads, is_k = !is_q && r < heads + kv_heads;
    const float* w = is_q ? q_norm : (is_k ? k_norm : nullptr);
#pragma unroll
    for (int i = 0; i < NV; i++) x[i] *= rn * (w ? __ldg(w + (i < H2 ? H2 * lane + i : DH / 2 + H2 * lane + i - H2)) : 1.0f);
    const uint32_t pos = pos0 + token;
    if (is_q || is_k) {
#pragma unroll
        for (int i = 0; i < H2; i++) {
            float sn, cs;
            sincosf((float)pos * __ldg(freq + H2 * lane + i), &sn, &cs);
            const float p = x[i], q = x[i + H2];
            x[i] = p * cs - q * sn;
            x[i + H2] = q * cs + p * sn;
        }
    }
    __half* dst;
    if (is_q) {
#pragma unroll
        for (int i = 0; i < NV; i++) x[i] *= qscale;
        dst = q_out + ((size_t)token * heads + r) * DH;
    } else {
        const uint32_t g = is_k ? r - heads : r - heads - kv_heads;
        dst = (is_k ? kc : vc) + ((size_t)g * cap + pos % cap) * DH;
    }
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const __half2 h0 = __floats2half2_rn(x[half * H2 + 4 * v], x[half * H2 + 4 * v + 1]), h1 = __floats2half2_rn(x[half * H2 + 4 * v + 2], x[half * H2 + 4 * v + 3]);
            *reinterpret_cast<uint2*>(dst + half * (DH / 2) + H2 * lane + 4 * v) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        }
}

// ---- flash attention --------------------------------------------------------------------------------------------------
// The reference's flash_256 / flash_512 (crates/tachyon/src/ptx/flash.rs:1-23).  A block: 16 tokens x the `group` (up
// to 4) query heads of one key-value head.  SPLIT warps share the 16 rows of a head: each scores all the tile's keys
// and sums its 1/SPLIT of the head's width, which keeps a thread's sums in registers at heads of 512 (SPLIT 2; heads
// of 256 run SPLIT 1).  Keys are visited in tiles of 32 positions that start at multiples of 32, so a token's sums do
// not depend on how the prompt was cut into chunks (flash.rs:9-12).  Token at position p sees p - window < j <= p.
constexpr int FT = 16, FK = 32;  // tokens per block, keys per tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
// 16 bytes global -> shared without passing through registers; `bytes` 0 fills the 16 bytes with zeros instead.
__device__ __forceinline__ void cp_async_16_zfill(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// 2^x by the hardware's approximation; 2^-inf is 0.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// What a launch by the reference's kernel name changes (flash.rs:19-22): the chunk's first position comes from device
// memory, the queries carry no log2(e) (the scores are multiplied by `sscale` instead), the output is f32.
struct FlashByName {
    const uint32_t* pos;
    float sscale;  // 1 when the queries are already in base 2
    int out_f32;
};

template <int DH, int SPLIT>
__global__ void __launch_bounds__(128 * SPLIT) prefill_flash_kernel(const __half* q, const __half* kc, const __half* vc, void* out, uint32_t tokens,
                                                                    uint32_t pos0, uint32_t cap, uint32_t window, uint32_t heads, uint32_t kv_heads,
                                                                    FlashByName named) {
    if (named.pos != nullptr) pos0 = __ldg(named.pos);
    constexpr int LDS = DH + 8;        // padded row length in halves
    constexpr int DW = DH / SPLIT;     // dimensions a warp sums
    extern __shared__ __align__(16) uint8_t raw[];
    __half* Qs = reinterpret_cast<__half*>(raw);   // [group * FT][LDS]
    // Block row blockIdx.y takes `group` query heads, all of one key-value head: every head of it, or four of its eight
    // (flash.rs:5-6: block row ctaid.y serves key-value head ctaid.y / group).
    const uint32_t ratio = heads / kv_heads, group = ratio < 4 ? ratio : 4;
    __half* KV = Qs + group * FT * LDS;            // two stages of keys [FK][LDS] then values [FK][LDS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hw = warp / SPLIT, part = warp % SPLIT;  // the head (of the group) this warp serves, and its share of the width
    const uint32_t t0 = blockIdx.x * FT, head0 = blockIdx.y * group, g = head0 / ratio;
    const uint32_t nthreads = group * SPLIT * 32;

    // Queries of this block: row w*16 + i is (head head0 + w, token t0 + i).
    for (uint32_t c = tid; c < group * FT * (DH / 8); c += nthreads) {
        const uint32_t row = c / (DH / 8), ch = c % (DH / 8), w = row / FT, i = row % FT, t = t0 + i;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < tokens) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * heads + head0 + w) * DH + ch * 8);
        *reinterpret_cast<uint4*>(Qs + row * LDS + ch * 8) = v;
    }
    const uint32_t p_first = pos0 + t0, p_last = pos0 + min(t0 + FT, tokens) - 1;
    const uint32_t lo = p_first + 1 > window ? p_first + 1 - window : 0;  // oldest position any token of the block sees
    const uint32_t tile0 = lo / FK * FK;

    float o[DW / 8][4];
#pragma unroll
    for (int nb = 0; nb < DW / 8; nb++) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const uint32_t row_a = lane >> 2, row_b = row_a + 8;                   // the two rows this lane holds
    const uint32_t pa = pos0 + t0 + row_a, pb = pos0 + t0 + row_b;        // their positions

    // Tiles arrive through cp.async, one tile ahead of the products: the copy of tile i + 1 is in flight while tile i is
    // multiplied.  Rows past the block's last position are filled with zeros (stale cache rows could hold anything).
    // A thread copies the same 16 bytes of every (nthreads / (DH / 8))-th row (the block's threads are a multiple of a row's pieces).
    const uint32_t piece = tid % (DH / 8), row0 = tid / (DH / 8), row_step = nthreads / (DH / 8);
    const __half* kbase = kc + (size_t)g * cap * DH + piece * 8;
    const __half* vbase = vc + (size_t)g * cap * DH + piece * 8;
    auto fetch = [&](uint32_t j0, uint32_t stage) {
        __half* Kd = KV + stage * (2 * FK * LDS) + piece * 8;
        __half* Vd = Kd + FK * LDS;
        const uint32_t slot0 = j0 % cap;
        for (uint32_t r = row0; r < FK; r += row_step) {
            const bool live = j0 + r <= p_last;
            uint32_t slot = slot0 + r;
            slot = slot >= cap ? slot % cap : slot;
            const size_t at = live ? (size_t)slot * DH : 0;
            cp_async_16_zfill(Kd + r * LDS, kbase + at, live ? 16u : 0u);
            cp_async_16_zfill(Vd + r * LDS, vbase + at, live ? 16u : 0u);
        }
        cp_async_commit();
    };
    // Tiles every row of the block sees whole need no mask: all keys at or before the first row's position and inside the
    // last row's window.  (A block with rows past the chunk's end always masks.)
    const bool whole_rows = t0 + FT <= tokens;
    fetch(tile0, 0);
    uint32_t stage = 0;
    for (uint32_t j0 = tile0; j0 <= p_last; j0 += FK, stage ^= 1u) {
        cp_async_wait_all();
        __syncthreads();  // this tile is visible to all; the other stage is no longer read (and, first time, Qs is written)
        if (j0 + FK <= p_last) fetch(j0 + FK, stage ^ 1u);
        const __half* Ks = KV + stage * (2 * FK * LDS);
        const __half* Vs = Ks + FK * LDS;
        // Scores S = Q K^T for this warp's 16 rows and the tile's 32 keys.
        float sc[FK / 8][4];
#pragma unroll
        for (int nb = 0; nb < FK / 8; nb++) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f;
#pragma unroll 4
        for (int ks = 0; ks < DH / 16; ks++) {
            uint32_t a[4];
            ldmatrix_x4(a, Qs + (hw * FT + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < FK / 8; nb += 2) {  // two blocks of eight keys per load
                uint32_t b[4];
                ldmatrix_x4(b, Ks + (nb * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma_16816(sc[nb], a, b0);
                mma_16816(sc[nb + 1], a, b1);
            }
        }
        // Mask, running maximum and sums (scores are already in base 2: the queries carry scale*log2(e)).
        float mt[2] = {-INFINITY, -INFINITY};
        if (named.sscale != 1.0f) {
#pragma unroll
            for (int nb = 0; nb < FK / 8; nb++) sc[nb][0] *= named.sscale, sc[nb][1] *= named.sscale, sc[nb][2] *= named.sscale, sc[nb][3] *= named.sscale;
        }
        if (whole_rows && j0 + FK - 1 <= p_first && j0 + window > p_first + FT - 1) {
#pragma unroll
            for (int nb = 0; nb < FK / 8; nb++) {
                mt[0] = fmaxf(mt[0], fmaxf(sc[nb][0], sc[nb][1]));
                mt[1] = fmaxf(mt[1], fmaxf(sc[nb][2], sc[nb][3]));
            }
        } else {
#pragma unroll
            for (int nb = 0; nb < FK / 8; nb++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t j = j0 + nb * 8 + 2 * (lane & 3) + (e & 1), p = (e < 2) ? pa : pb;
                    const bool seen = j <= p && j + window > p && p <= p_last;
                    sc[nb][e] = seen ? sc[nb][e] : -INFINITY;
                    mt[e >> 1] = fmaxf(mt[e >> 1], sc[nb][e]);
                }
            }
        }
        float corr[2], base[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 1));
            mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 2));
            const float mn = fmaxf(m_run[h], mt[h]);
            base[h] = fmaxf(mn, -1e30f);        // finite, so a row that has seen nothing yet gets 2^-inf = 0 and no NaN
            corr[h] = ex2(m_run[h] - base[h]);  // 1 when the maximum stays; 0 for a row's first keys (its sums are zeros)
            m_run[h] = mn;
        }
        float lt[2] = {0.0f, 0.0f};
        uint32_t pfrag[FK / 16][4];
#pragma unroll
        for (int nb = 0; nb < FK / 8; nb++) {
            const float e0 = ex2(sc[nb][0] - base[0]), e1 = ex2(sc[nb][1] - base[0]), e2 = ex2(sc[nb][2] - base[1]), e3 = ex2(sc[nb][3] - base[1]);
            const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
            // the sums use the rounded probabilities, the ones the values are weighted with
            lt[0] += __low2float(h01) + __high2float(h01);
            lt[1] += __low2float(h23) + __high2float(h23);
            pfrag[nb / 2][(nb & 1) * 2] = *reinterpret_cast<const uint32_t*>(&h01);
            pfrag[nb / 2][(nb & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            lt[h] += __shfl_xor_sync(0xffffffffu, lt[h], 1);
            lt[h] += __shfl_xor_sync(0xffffffffu, lt[h], 2);
            l_run[h] = l_run[h] * corr[h] + lt[h];
        }
        // O = O * corr + P V over this warp's share of the width; a tile that moved no maximum of the warp skips the scaling.
        const bool moved = __any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f);
        const __half* Vw = Vs + part * DW;
#pragma unroll
        for (int nb = 0; nb < DW / 8; nb += 2) {  // two blocks of eight dimensions per load
            if (moved) {
                o[nb][0] *= corr[0], o[nb][1] *= corr[0], o[nb][2] *= corr[1], o[nb][3] *= corr[1];
                o[nb + 1][0] *= corr[0], o[nb + 1][1] *= corr[0], o[nb + 1][2] *= corr[1], o[nb + 1][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < FK / 16; kk++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, Vw + (kk * 16 + (lane & 15)) * LDS + (nb + (lane >> 4)) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma_16816(o[nb], pfrag[kk], b0);
                mma_16816(o[nb + 1], pfrag[kk], b1);
            }
        }
    }
    // Normalise and store f16 [token][heads * DH].
    const float inv[2] = {l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f};
    const uint32_t head = head0 + hw;
#pragma unroll
    for (int nb = 0; nb < DW / 8; nb++) {
        const uint32_t col = head * DH + part * DW + nb * 8 + 2 * (lane & 3);
        const size_t at_a = (size_t)(t0 + row_a) * heads * DH + col, at_b = (size_t)(t0 + row_b) * heads * DH + col;
        if (named.out_f32) {
            if (t0 + row_a < tokens) *reinterpret_cast<float2*>(static_cast<float*>(out) + at_a) = make_float2(o[nb][0] * inv[0], o[nb][1] * inv[0]);
            if (t0 + row_b < tokens) *reinterpret_cast<float2*>(static_cast<float*>(out) + at_b) = make_float2(o[nb][2] * inv[1], o[nb][3] * inv[1]);
        } else {
            if (t0 + row_a < tokens) *reinterpret_cast<__half2*>(static_cast<__half*>(out) + at_a) = __floats2half2_rn(o[nb][0] * inv[0], o[nb][1] * inv[0]);
            if (t0 + row_b < tokens) *reinterpret_cast<__half2*>(static_cast<__half*>(out) + at_b) = __floats2half2_rn(o[nb][2] * inv[1], o[nb][3] * inv[1]);
        }
    }
}

}  // namespace

int launch_prefill_embed(tb_context* ctx, const int8_t* w, const __half* s, const uint32_t* tokens, uint32_t n, uint32_t cols, float scale, float* out,
                         uint32_t wbits) {
    prefill_embed_kernel<<<n, 256, 0, ctx->stream>>>(w, s, tokens, cols, scale, out, wbits);
    TB_CUDA(cudaGetLastError());
    return OK;
}

int launch_prefill_norm(tb_context* ctx, float* h, const float* y, const float* w1, const float* w2, uint32_t tokens, uint32_t n, float eps, float hscale,
                        __half* x) {
    if (n != 2048) return fail(UNSUPPORTED, "prefill norm: rows of 2048 values");
    TB_CUDA(launch_kernel(ctx, prefill_norm_kernel, dim3((tokens + 7) / 8), dim3(256), (size_t)0, true, h, y, w1, w2, tokens, eps, hscale, x));
    TB_CUDA(cudaGetLastError());
    return OK;
}

int launch_prefill_qkv(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, __half* q_out, __half* kc, __half* vc,
                       uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float scale, uint32_t head_dim) {
    PrefillRows rows;
    rows.count = heads + 2 * kv_heads, rows.stride = rows.count * head_dim;
    return launch_prefill_rows(ctx, qkv, q_norm, k_norm, freq, q_out, kc, vc, tokens, pos0, cap, heads, kv_heads, eps, scale * 1.4426950408889634f, head_dim, rows);
}

int launch_prefill_rows(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, __half* q_out, __half* kc, __half* vc,
                        uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float qscale, uint32_t head_dim,
                        const PrefillRows& rows) {
    const uint32_t items = tokens * rows.count, blocks = (items + 3) / 4;
    if (head_dim != 256 && head_dim != 512) return fail(UNSUPPORTED, "prefill qkv: heads of 256 or 512");
    if (items == 0) return fail(OUT_OF_RANGE, "prefill qkv: nothing to prepare");
    const QkvRows r{rows.first, rows.count, rows.stride, rows.pos};
    cudaError_t le;
    if (head_dim == 512) le = launch_kernel(ctx, prefill_qkv_kernel<512>, dim3(blocks), dim3(128), (size_t)0, true, qkv, q_norm, k_norm, freq, q_out, kc, vc, tokens, pos0, cap, heads, kv_heads, eps, qscale, r);
    else le = launch_kernel(ctx, prefill_qkv_kernel<256>, dim3(blocks), dim3(128), (size_t)0, true, qkv, q_norm, k_norm, freq, q_out, kc, vc, tokens, pos0, cap, heads, kv_heads, eps, qscale, r);
    TB_CUDA(le);
    TB_CUDA(cudaGetLastError());
    return OK;
}

int launch_prefill_flash(tb_context* ctx, const __half* q, const __half* kc, const __half* vc, void* out, uint32_t tokens, uint32_t pos0, uint32_t cap,
                         uint32_t window, uint32_t heads, uint32_t kv_heads, uint32_t head_dim, const uint32_t* pos_dev, float sscale, int out_f32) {
    if (kv_heads == 0 || heads % kv_heads != 0) return fail(UNSUPPORTED, "prefill attention: heads must be a multiple of kv_heads");
    const uint32_t ratio = heads / kv_heads, group = ratio < 4 ? ratio : 4;  // query heads a block takes
    if (ratio != 1 && ratio != 2 && ratio != 4 && ratio != 8) return fail(UNSUPPORTED, "prefill attention: 1, 2, 4 or 8 query heads per key-value head");
    if (head_dim != 256 && head_dim != 512) return fail(UNSUPPORTED, "prefill attention: heads of 256 or 512");
    if (ctx->flash_tc && prefill_flash_tc_supports(heads, kv_heads, head_dim, cap))
        return launch_prefill_flash_tc(ctx, q, kc, vc, out, tokens, pos0, cap, window, heads, kv_heads, pos_dev, sscale, out_f32);
    // queries, two stages of keys and values; rows padded by 8 halves
    auto bytes = [&](uint32_t grp) { return (size_t)(grp * FT + 4 * FK) * (head_dim + 8) * 2; };
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(prefill_flash_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((4 * FT + 4 * FK) * (256 + 8) * 2)));
        TB_CUDA(cudaFuncSetAttribute(prefill_flash_kernel<512, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((4 * FT + 4 * FK) * (512 + 8) * 2)));
        configured[ctx->gpu & 15] = true;
    }
    const dim3 grid((tokens + FT - 1) / FT, heads / group);
    const FlashByName named{pos_dev, sscale, out_f32};
    if (head_dim == 512) prefill_flash_kernel<512, 2><<<grid, group * 64, bytes(group), ctx->stream>>>(q, kc, vc, out, tokens, pos0, cap, window, heads, kv_heads, named);
    else prefill_flash_kernel<256, 1><<<grid, group * 32, bytes(group), ctx->stream>>>(q, kc, vc, out, tokens, pos0, cap, window, heads, kv_heads, named);
    TB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace tb
