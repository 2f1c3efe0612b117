// The whole decode step as one persistent kernel: every phase of crates/tachyon/src/model/decode.rs:569-592's op list
// (embedding row, per layer qkv / attention / o / gate_up / down, LM head with the greedy pick) runs in the same 148
// resident blocks, separated by grid-wide barriers instead of kernel boundaries.
//
// Why: at 8 TB/s a layer's 118 MB of weights stream in 15 us, and the 177 kernel boundaries of the launch-per-phase
// form (start-up, prologue, drain: 3-4 us each) cost as much as the streaming.  Here the producer warp of each block
// walks the block's slices of ALL the step's matrices in order, through one shared-memory ring, and never takes part in
// a barrier: weights are read-only, so while the consumers wait for the other blocks or rebuild their activation
// planes, the ring keeps filling with the next phase's weights and HBM stays busy.
//
// Blocks wait on one another, so the launch is cooperative (all blocks resident) and every wait is bounded: a block that
// gives up sets the context's status word and every block then skips to the end.
#include "attend_body.cuh"
#include "planes.cuh"

namespace tb {

namespace {

constexpr int CONSUMERS = 16;
constexpr int CTHREADS = CONSUMERS * 32;
constexpr int THREADS = CTHREADS + 32;
constexpr int SEG = 2048;
constexpr int NST = 4;              // ring stages
constexpr int STAGE_W = 32768;      // weight bytes per stage: 16 rows of 2048, 2 rows of 16384
constexpr int STAGE_S = STAGE_W / 16;
constexpr int AREA = 81920;         // attention's tiles, or the planes of a vector longer than 2048

// Shared memory, in this order.
constexpr int OFF_W = 0;
constexpr int OFF_S = OFF_W + NST * STAGE_W;
constexpr int OFF_AREA = OFF_S + NST * STAGE_S;
constexpr int OFF_HI = OFF_AREA + AREA;      // planes of a 2048-long vector: 64 groups x 32 bytes per plane
constexpr int OFF_MID = OFF_HI + 2048;
constexpr int OFF_LO = OFF_MID + 2048;
constexpr int OFF_MUL = OFF_LO + 2048;
constexpr int OFF_FULL = OFF_MUL + 256;
constexpr int OFF_EMPTY = OFF_FULL + NST * 8;
constexpr int OFF_RED = OFF_EMPTY + NST * 8;          // float [2][CONSUMERS]
constexpr int OFF_BESTV = OFF_RED + 2 * CONSUMERS * 4;  // float [2 * CONSUMERS]
constexpr int OFF_BESTI = OFF_BESTV + 2 * CONSUMERS * 4;
constexpr int OFF_SUMS = OFF_BESTI + 2 * CONSUMERS * 4;  // float4 [CONSUMERS]
constexpr int OFF_FLAGS = OFF_SUMS + CONSUMERS * 16;     // uint32: [0] abort, [1] attention's first tile is on its way
constexpr int OFF_PHASE = OFF_FLAGS + 16;                // two descriptors: phase ph lives in slot ph % 2, the next one beside it
constexpr int PHASE_BYTES = ((int)sizeof(StepPhase) + 15) / 16 * 16;
constexpr int SMEM_BYTES = OFF_PHASE + 2 * PHASE_BYTES;
static_assert(sizeof(attend::Smem) <= AREA, "attention's shared memory must fit its area");
static_assert(SMEM_BYTES <= 232448, "over the 227 KiB a block may use");
static_assert(sizeof(StepPhase) % 4 == 0, "descriptors are copied word by word");

struct PlanePtr {
    uint32_t *hi, *mid, *lo;
    float* mul;
};

template <int WPR>
__device__ __forceinline__ PlanePtr plane_ptr(uint8_t* raw) {
    if constexpr (WPR == 1) {
        return {reinterpret_cast<uint32_t*>(raw + OFF_HI), reinterpret_cast<uint32_t*>(raw + OFF_MID), reinterpret_cast<uint32_t*>(raw + OFF_LO),
                reinterpret_cast<float*>(raw + OFF_MUL)};
    } else {
        uint8_t* a = raw + OFF_AREA;
        return {reinterpret_cast<uint32_t*>(a), reinterpret_cast<uint32_t*>(a + WPR * 2048), reinterpret_cast<uint32_t*>(a + 2 * WPR * 2048),
                reinterpret_cast<float*>(a + 3 * WPR * 2048)};
    }
}

// Four consecutive activations -> word `idx` of each plane; the eight lanes sharing a group of 32 agree on its exponent.
__device__ __forceinline__ void store_planes(const PlanePtr& pp, int idx, float v0, float v1, float v2, float v3) {
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);
    const bool zero = eb < 22u;
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);
    const int x0 = __float2int_rn(v0 * sc), x1 = __float2int_rn(v1 * sc), x2 = __float2int_rn(v2 * sc), x3 = __float2int_rn(v3 * sc);
    pp.hi[idx] = pack_bytes(x0, x1, x2, x3, 0x0062);
    pp.mid[idx] = pack_bytes(x0, x1, x2, x3, 0x0051);
    pp.lo[idx] = pack_bytes(x0, x1, x2, x3, 0x0040);
    if ((idx & 7) == 0) pp.mul[idx >> 3] = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);
}

__device__ __forceinline__ void fetch_planes(const PlanePtr& pp, int b, int first, Planes& pl) {
    const uint4* hi = reinterpret_cast<const uint4*>(pp.hi) + b * 2;
    const uint4* mid = reinterpret_cast<const uint4*>(pp.mid) + b * 2;
    const uint4* lo = reinterpret_cast<const uint4*>(pp.lo) + b * 2;
    const uint4 h0 = hi[first], h1 = hi[1 - first], m0 = mid[first], m1 = mid[1 - first], l0 = lo[first], l1 = lo[1 - first];
    pl.hi[0] = h0.x, pl.hi[1] = h0.y, pl.hi[2] = h0.z, pl.hi[3] = h0.w, pl.hi[4] = h1.x, pl.hi[5] = h1.y, pl.hi[6] = h1.z, pl.hi[7] = h1.w;
    pl.mid[0] = m0.x, pl.mid[1] = m0.y, pl.mid[2] = m0.z, pl.mid[3] = m0.w, pl.mid[4] = m1.x, pl.mid[5] = m1.y, pl.mid[6] = m1.z, pl.mid[7] = m1.w;
    pl.lo[0] = l0.x, pl.lo[1] = l0.y, pl.lo[2] = l0.z, pl.lo[3] = l0.w, pl.lo[4] = l1.x, pl.lo[5] = l1.y, pl.lo[6] = l1.z, pl.lo[7] = l1.w;
    pl.mul = pp.mul[b];
}

// The activation vector of a product -> planes, by the 512 consumer threads (same arithmetic as gemv.cu's prologue).
template <int WPR, int XMODE>
__device__ __forceinline__ void build_planes(const GemvParams& p, uint8_t* raw, int t, uint32_t pos, const float4& nw1, const float4& nw2) {
    const PlanePtr pp = plane_ptr<WPR>(raw);
    if constexpr (XMODE == X_F32) {
        float4 f[WPR];
#pragma unroll
        for (int j = 0; j < WPR; j++) f[j] = ld_cg_f4(static_cast<const float*>(p.x) + (size_t)(j * CTHREADS + t) * 4);
#pragma unroll
        for (int j = 0; j < WPR; j++) store_planes(pp, j * CTHREADS + t, f[j].x, f[j].y, f[j].z, f[j].w);
    } else if constexpr (XMODE == X_ATTN) {
        // The vector is attention's output, still split over the blocks that computed it: merge the splits' (maximum,
        // sum, unnormalised output) here, four dimensions per thread, with running-maximum rescaling
        // (crates/tachyon/src/ptx/attend.rs:371-405 does this in the attention kernel's last block).
        static_assert(WPR == 1, "the attention merge is built for 2048 columns");
        const uint32_t G = p.att_heads / p.att_kv, HD = attend_header(G), stride = HD + G * 256;
        const uint32_t head = (uint32_t)t / 64, g = head / G, hh = head % G, d0 = ((uint32_t)t * 4) % 256;
        const uint32_t n = min(pos + 1, p.att_window);  // the step's position, read once at the kernel's start
        const uint32_t span = attend::split_span(n, p.att_splits), used = (n + span - 1) / span;
        const float* base = p.att_partial + (size_t)g * p.att_splits * stride;
        float M = -INFINITY, L = 0.0f;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
        for (uint32_t s2 = 0; s2 < used; s2++) {
            const float* ps = base + (size_t)s2 * stride;
            const float m = ld_cg_f(ps + hh), l = ld_cg_f(ps + G + hh);
            const float4 a = ld_cg_f4(ps + HD + hh * 256 + d0);
            const float Mn = fmaxf(M, m), c = exp2f(M - Mn), w = exp2f(m - Mn);
            L = fmaf(L, c, w * l);
            o.x = fmaf(o.x, c, w * a.x), o.y = fmaf(o.y, c, w * a.y), o.z = fmaf(o.z, c, w * a.z), o.w = fmaf(o.w, c, w * a.w);
            M = Mn;
        }
        const float inv = 1.0f / L;
        store_planes(pp, t, o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    } else {
        static_assert(XMODE != X_NORM || WPR == 1, "the norm prologue is built for 2048 columns");
        const size_t at = (size_t)t * 4;
        const float4 h = ld_cg_f4(p.h + at);
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float sy = 0.0f;
        if (p.yres != nullptr) {
            const float4 y = ld_cg_f4(p.yres + at);
            const float4 w = nw1;
            a = make_float4(y.x * w.x, y.y * w.y, y.z * w.z, y.w * w.w);
            sy = y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
        }
        const float4 w2 = nw2;
        float sh = h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
        float sha = h.x * a.x + h.y * a.y + h.z * a.z + h.w * a.w;
        float sa = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
        float4* sums = reinterpret_cast<float4*>(raw + OFF_SUMS);
        if ((t & 31) == 0) sums[t >> 5] = make_float4(sy, sh, sha, sa);
        named_bar_sync(1, CTHREADS);
        sy = sh = sha = sa = 0.0f;
#pragma unroll
        for (int k = 0; k < CONSUMERS; k++) {
            const float4 q = sums[k];
            sy += q.x, sh += q.y, sha += q.z, sa += q.w;
        }
        const float n = static_cast<float>(p.cols);
        const float ry = p.yres != nullptr ? rsqrtf(sy / n + p.eps) : 0.0f;
        const float hs = p.yres != nullptr ? p.hscale : 1.0f;
        const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
        const float rh = p.w2 != nullptr ? rsqrtf(fmaxf(sq, 0.0f) / n + p.eps) : 1.0f;
        const float v0 = fmaf(a.x, ry, h.x) * hs, v1 = fmaf(a.y, ry, h.y) * hs, v2 = fmaf(a.z, ry, h.z) * hs, v3 = fmaf(a.w, ry, h.w) * hs;
        if (blockIdx.x == 0 && p.h_out != nullptr) *reinterpret_cast<float4*>(p.h_out + at) = make_float4(v0, v1, v2, v3);
        store_planes(pp, t, v0 * rh * w2.x, v1 * rh * w2.y, v2 * rh * w2.z, v3 * rh * w2.w);
    }
}

// The rows [r0, r1) of a product this block owns, and how many ring stages they take.
__device__ __forceinline__ void block_rows(uint32_t rows, uint32_t cols, int epi, uint32_t& r0, uint32_t& r1, uint32_t& nst) {
    const uint32_t unit = epi == EPI_GEGLU ? 2u : 1u, units = rows / unit;
    r0 = static_cast<uint32_t>((uint64_t)units * blockIdx.x / gridDim.x) * unit;
    r1 = static_cast<uint32_t>((uint64_t)units * (blockIdx.x + 1) / gridDim.x) * unit;
    const uint32_t per = STAGE_W / cols;
    nst = (r1 - r0 + per - 1) / per;
}

struct Best {
    float v = -INFINITY;
    uint32_t i = 0xffffffffu;
};

// Consumer side of one product.  `gi` counts the ring stages used so far in the step (it picks slot and parity).
// cols == 2048: a stage holds 16 rows, taken by one half of the warps (two rows a warp) while the other half takes the
// next stage; longer rows: WPR warps share a row and all warps work on every stage.
template <int WPR, int XMODE, int EPI>
__device__ __forceinline__ void gemv_phase(const GemvParams& p, uint8_t* raw, uint32_t& gi, bool& ok, uint32_t* status, Best& best, uint32_t pos, unsigned long long* st,
                                           const float4& nw1, const float4& nw2) {
    constexpr int RPW = WPR == 1 ? 2 : 1;
    constexpr int ROWS = STAGE_W / (WPR * SEG);
    const uint32_t K = p.cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t r0, r1, nst;
    block_rows(p.rows, K, EPI, r0, r1, nst);
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + OFF_FULL);
    uint64_t* empty = reinterpret_cast<uint64_t*>(raw + OFF_EMPTY);

    build_planes<WPR, XMODE>(p, raw, threadIdx.x, pos, nw1, nw2);
    named_bar_sync(1, CTHREADS);
    const int half = WPR == 1 ? warp >> 3 : 0;              // which stages this warp takes when cols == 2048
    const int seg = WPR == 1 ? 0 : warp % WPR;              // the warp's column segment
    const int grp = WPR == 1 ? (warp & 7) : warp / WPR;     // its row group within a stage
    const int first = (lane >> 2) & 1;
    const PlanePtr pp = plane_ptr<WPR>(raw);
    Planes pl[2];
    fetch_planes(pp, seg * 64 + lane, first, pl[0]);
    fetch_planes(pp, seg * 64 + lane + 32, first, pl[1]);
    if (st != nullptr) st[1] = global_ns();

    for (uint32_t i = 0; i < nst; i++) {
        if (WPR == 1 && (int)(i & 1) != half) continue;
        const uint32_t g = gi + i, s = g % NST;
        if (ok && !mbar_wait(&full[s], (g / NST) & 1)) {
            atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
            ok = false;
        }
        const uint32_t row = r0 + i * ROWS + grp * RPW;
        float v[RPW];
#pragma unroll
        for (int j = 0; j < RPW; j++) {
            v[j] = 0.0f;
            if (ok && row + j < r1) {
                const uint8_t* wr = raw + OFF_W + s * STAGE_W + (size_t)(grp * RPW + j) * K + seg * SEG;
                const __half* sr = reinterpret_cast<const __half*>(raw + OFF_S + s * STAGE_S) + (grp * RPW + j) * (K / 32) + seg * 64;
                const uint4 a0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + first) * 16);
                const uint4 b0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + 1 - first) * 16);
                const uint4 a1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + first) * 16);
                const uint4 b1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + 1 - first) * 16);
                const float s0 = __half2float(sr[lane]) * pl[0].mul, s1 = __half2float(sr[lane + 32]) * pl[1].mul;
                v[j] = fmaf(block_dot(a1, b1, pl[1]), s1, block_dot(a0, b0, pl[0]) * s0);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&empty[s], WPR == 1 ? 2 : 1);
        float r;
        uint32_t out_row;
        if constexpr (RPW == 2) {
            const bool upper = lane & 16;
            r = (upper ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, upper ? v[0] : v[1], 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
            out_row = row + (upper ? 1 : 0);
            if constexpr (EPI == EPI_GEGLU) {
                const float up = __shfl_sync(0xffffffffu, r, 16);
                r = gelu_tanh(r) * up;
            }
        } else {
            r = warp_sum(v[0]);
            out_row = row;
        }
        if constexpr (WPR > 1) {
            float* red = reinterpret_cast<float*>(raw + OFF_RED) + (i & 1) * CONSUMERS;
            if (lane == 0) red[warp] = r;
            named_bar_sync(4 + grp, WPR * 32);
            if (seg != 0) continue;
            r = 0.0f;
#pragma unroll
            for (int j = 0; j < WPR; j++) r += red[warp + j];
        }
        const bool writer = (EPI == EPI_GEGLU || RPW == 1) ? lane == 0 : (lane & 15) == 0;
        if (writer && out_row < r1) {
            if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[out_row] = r;
            if constexpr (EPI == EPI_GEGLU) static_cast<float*>(p.y)[out_row / 2] = r;
            if constexpr (EPI == EPI_ARGMAX) {
                if (p.y != nullptr) static_cast<float*>(p.y)[out_row] = r;
                // the two halves of the warps walk the rows interleaved: keep the lower row among equals
                if (r > best.v || (r == best.v && out_row < best.i)) best.v = r, best.i = out_row;
            }
        }
    }
    gi += nst;

    if constexpr (EPI == EPI_ARGMAX) {
        float* sbv = reinterpret_cast<float*>(raw + OFF_BESTV);
        uint32_t* sbi = reinterpret_cast<uint32_t*>(raw + OFF_BESTI);
        if ((lane & 15) == 0) sbv[2 * warp + (lane >> 4)] = best.v, sbi[2 * warp + (lane >> 4)] = best.i;
        named_bar_sync(1, CTHREADS);
        if (threadIdx.x == 0) {
            unsigned long long key = 0;
            for (int j = 0; j < 2 * CONSUMERS; j++) {
                const unsigned long long k = ((unsigned long long)float_key(sbv[j]) << 32) | (0xffffffffu - sbi[j]);
                key = k > key ? k : key;
            }
            atomicMax(p.best, key);
            __threadfence();
            if (atomicAdd(p.count, 1u) == gridDim.x - 1) {
                __threadfence();
                const unsigned long long top = atomicExch(p.best, 0ull);
                const uint32_t token = 0xffffffffu - static_cast<uint32_t>(top);
                const uint32_t position = p.state[0];
                if (p.trace != nullptr) p.trace[position & p.trace_mask] = token;
                p.state[1] = token;
                p.state[0] = position + 1;
                if (p.token_out != nullptr) *p.token_out = token;
                *p.count = 0;
            }
        }
    }
}

__device__ __forceinline__ void run_gemv(const GemvParams& p, uint8_t* raw, uint32_t& gi, bool& ok, uint32_t* status, Best& best, uint32_t pos,
                                         unsigned long long* st, const float4& nw1, const float4& nw2) {
    if (p.cols == 2048) {
        if (p.xmode == X_NORM && p.epi == EPI_F32) gemv_phase<1, X_NORM, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
        else if (p.xmode == X_NORM && p.epi == EPI_GEGLU) gemv_phase<1, X_NORM, EPI_GEGLU>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
        else if (p.xmode == X_NORM && p.epi == EPI_ARGMAX) gemv_phase<1, X_NORM, EPI_ARGMAX>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
        else if (p.xmode == X_ATTN) gemv_phase<1, X_ATTN, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
        else gemv_phase<1, X_F32, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
    } else if (p.cols == 4096) {
        gemv_phase<2, X_F32, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
    } else if (p.cols == 8192) {
        gemv_phase<4, X_F32, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
    } else {
        gemv_phase<8, X_F32, EPI_F32>(p, raw, gi, ok, status, best, pos, st, nw1, nw2);
    }
}

// All blocks have finished the phase before any starts the next: one arrival per block on a counter that only grows
// during a launch.  While thread 0 waits, the other threads copy the next phase's descriptor into shared memory.
// Returns false when this block gave up (two seconds) or another block reported an error.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t target, uint32_t* status, const StepPhase* next, uint8_t* slot, uint8_t* raw) {
    uint32_t* flags = reinterpret_cast<uint32_t*>(raw + OFF_FLAGS);
    named_bar_sync(1, CTHREADS);
    if (threadIdx.x == 0) {
        red_release_add(counter, 1u);  // the block's writes (ordered before this by the barrier above) are released with it
        const unsigned long long start = global_ns();
        for (uint32_t spins = 0; ld_acquire_u32(counter) < target; ++spins) {
            if ((spins & 63u) == 63u) {
                if (ld_acquire_u32(status) != ERR_NONE) {
                    flags[0] = 1;
                    break;
                }
                if (global_ns() - start > WAIT_LIMIT_NS) {
                    atomicCAS(status, ERR_NONE, ERR_GRID);
                    flags[0] = 1;
                    break;
                }
            }
        }
    } else if (next != nullptr) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(next);
        uint32_t* dst = reinterpret_cast<uint32_t*>(slot);
        for (uint32_t i = threadIdx.x - 1; i < sizeof(StepPhase) / 4; i += CTHREADS - 1) dst[i] = __ldg(src + i);
    }
    named_bar_sync(1, CTHREADS);
    return flags[0] == 0;
}

// Walks the ring stages of this block in the order the step consumes them: every product phase, its rows in stage-sized
// pieces.
struct Cursor {
    const StepPhase* phases;
    uint32_t nphases, ph, i, nst, r0, r1, K, per;
    const int8_t* w;
    const __half* s;
    __device__ Cursor(const StepPhase* p, uint32_t n) : phases(p), nphases(n), ph(0), i(0), nst(0) { seek(); }
    __device__ void seek() {
        for (; ph < nphases; ph++) {
            if (__ldg(&phases[ph].kind) != PH_GEMV) continue;
            const GemvParams* gp = &phases[ph].g;
            w = reinterpret_cast<const int8_t*>(__ldg(reinterpret_cast<const unsigned long long*>(&gp->w)));
            s = reinterpret_cast<const __half*>(__ldg(reinterpret_cast<const unsigned long long*>(&gp->s)));
            K = __ldg(&gp->cols);
            block_rows(__ldg(&gp->rows), K, __ldg(&gp->epi), r0, r1, nst);
            per = STAGE_W / K;
            i = 0;
            if (nst > 0) return;
        }
    }
    __device__ bool valid() const { return ph < nphases; }
    __device__ void next() {
        if (++i >= nst) ph++, seek();
    }
    __device__ uint32_t here() const { return min(per, r1 - (r0 + i * per)); }
    __device__ const int8_t* w_ptr() const { return w + (size_t)(r0 + i * per) * K; }
    __device__ const __half* s_ptr() const { return s + (size_t)(r0 + i * per) * (K / 32); }
    __device__ uint32_t w_bytes() const { return here() * K; }
    __device__ uint32_t s_bytes() const { return here() * (K / 16); }
};

__global__ void __launch_bounds__(THREADS, 1) decode_step_kernel(const StepPhase* phases, uint32_t nphases, uint32_t* counter, uint32_t* status,
                                                                     unsigned long long* times, uint32_t ahead, const uint32_t* state) {
    extern __shared__ __align__(128) uint8_t raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + OFF_FULL);
    uint64_t* empty = reinterpret_cast<uint64_t*>(raw + OFF_EMPTY);
    if (threadIdx.x == 0) {
        for (int i = 0; i < NST; i++) mbar_init(&full[i], 1), mbar_init(&empty[i], CONSUMERS);
        reinterpret_cast<uint32_t*>(raw + OFF_FLAGS)[0] = 0;
        reinterpret_cast<uint32_t*>(raw + OFF_FLAGS)[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (uint32_t k = 0; k < 2 && k < nphases; k++)
        if (threadIdx.x < sizeof(StepPhase) / 4)
            reinterpret_cast<uint32_t*>(raw + OFF_PHASE + k * PHASE_BYTES)[threadIdx.x] = __ldg(reinterpret_cast<const uint32_t*>(phases + k) + threadIdx.x);
    __syncthreads();

    if (warp == CONSUMERS) {
        // Producer: this block's slices of every matrix of the step, in order, as far ahead as the ring allows; and,
        // further ahead than the ring reaches, hints to the L2, so that HBM keeps streaming while the consumers sit
        // in the latency-bound phases (barriers, attention, the small matrices).
        // The whole warp walks the same sequence; lane 0 waits and issues the copies, all lanes share the hints (one
        // 128-byte line each per instruction, through the load/store unit so that they do not queue behind the copies).
        Cursor load(phases, nphases), hint(phases, nphases);
        uint32_t gi = 0, hinted = 0;
        bool alive = true;
        // Weights are read once a step: their lines are the first to go, so that hinted lines survive until used.
        const uint64_t stream_once = policy_evict_first();
        while (load.valid() && alive) {
            while (hinted < gi + ahead && hint.valid()) {
                if (hinted >= gi + NST) {  // what the ring itself is about to fetch needs no hint
                    const char* wp = reinterpret_cast<const char*>(hint.w_ptr());
                    const uint32_t wb = hint.w_bytes();
                    for (uint32_t o = lane * 128; o < wb; o += 32 * 128) prefetch_line_l2(wp + o);
                    const char* sp2 = reinterpret_cast<const char*>(hint.s_ptr());
                    const uint32_t sb = hint.s_bytes();
                    for (uint32_t o = lane * 128; o < sb; o += 32 * 128) prefetch_line_l2(sp2 + o);
                }
                hint.next();
                hinted++;
            }
            if (lane == 0) {
                const uint32_t s = gi % NST;
                if (gi >= NST && !mbar_wait(&empty[s], ((gi / NST) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    alive = false;
                } else {
                    mbar_expect_tx(&full[s], load.w_bytes() + load.s_bytes());
                    bulk_load_hint(raw + OFF_W + s * STAGE_W, load.w_ptr(), load.w_bytes(), &full[s], stream_once);
                    bulk_load_hint(raw + OFF_S + s * STAGE_S, load.s_ptr(), load.s_bytes(), &full[s], stream_once);
                }
            }
            alive = __shfl_sync(0xffffffffu, alive, 0);
            load.next();
            gi++;
        }
        return;
    }

    // Consumers.
    attend::Smem& asm_ = *reinterpret_cast<attend::Smem*>(raw + OFF_AREA);
    uint32_t* flags = reinterpret_cast<uint32_t*>(raw + OFF_FLAGS);
    const uint32_t pos = ld_cg_u(state);  // the step's position: only the last phase changes it
    uint32_t gi = 0;
    bool ok = true;
    Best best;
    // Norm weights of the phase about to run: fetched before the barrier in front of it (they are model constants and
    // usually come from HBM), used after it.
    float4 nw1 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), nw2 = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    // Optional timeline (the reference's Decoder::timeline, decode.rs:424-436): the first and the last block stamp
    // %globaltimer at each phase's start, after its planes, at its end and after the barrier behind it.
    const bool stamp = times != nullptr && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1);
    unsigned long long* mine = times + (blockIdx.x == 0 ? 0 : (size_t)nphases * 4);
    for (uint32_t ph = 0; ph < nphases; ph++) {
        const StepPhase& cur = *reinterpret_cast<const StepPhase*>(raw + OFF_PHASE + (ph & 1) * PHASE_BYTES);
        const StepPhase& nxt = *reinterpret_cast<const StepPhase*>(raw + OFF_PHASE + ((ph + 1) & 1) * PHASE_BYTES);
        if (stamp) mine[ph * 4] = global_ns();
        if (cur.kind == PH_EMBED) {
            // Row *token of the table times the scale (crates/tachyon/src/ptx/mod.rs:531-598); one block is plenty.
            if (blockIdx.x == 0) {
                const EmbedParams& e = cur.e;
                const size_t row = (size_t)ld_cg_u(e.token) * e.cols;
                for (uint32_t i = threadIdx.x; i < e.cols; i += CTHREADS) e.out[i] = (float)e.w[row + i] * __half2float(e.s[(row + i) / 32]) * e.scale;
            }
        } else if (cur.kind == PH_GEMV) {
            // When attention comes next, its first tile of keys and values (written by earlier steps) can already be
            // on its way while this product runs: the area it lands in is idle during a 2048-column product.
            if (threadIdx.x < attend::THREADS && ph + 1 < nphases && cur.g.cols == 2048 && nxt.kind == PH_ATTEND) {
                const AttendParams& an = nxt.a;
                bool sent = false;
                if (blockIdx.x < an.kv_heads * an.splits)
                    sent = attend::load_first_tile(an, asm_, blockIdx.x % an.kv_heads, blockIdx.x / an.kv_heads, pos, (int)threadIdx.x);
                if (threadIdx.x == 0) flags[1] = sent ? 1u : 0u;
            }
            run_gemv(cur.g, raw, gi, ok, status, best, pos, stamp ? mine + ph * 4 : nullptr, nw1, nw2);
        } else {
            const AttendParams& a = cur.a;
            const uint32_t items = a.kv_heads * a.splits, group = a.heads / a.kv_heads;
            if (threadIdx.x < attend::THREADS) {
                const attend::Trig trig = attend::rope_trig(a.freq, pos, lane, a.trig);
                for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
                    const bool pre = item == blockIdx.x && flags[1] != 0;
                    attend::block_sync<true>();
                    if (group == 4) attend::attend_body<4, true>(a, asm_, threadIdx.x, item % a.kv_heads, item / a.kv_heads, pos, pre, trig);
                    else if (group == 2) attend::attend_body<2, true>(a, asm_, threadIdx.x, item % a.kv_heads, item / a.kv_heads, pos, pre, trig);
                    else attend::attend_body<1, true>(a, asm_, threadIdx.x, item % a.kv_heads, item / a.kv_heads, pos, pre, trig);
                }
            }
        }
        if (stamp) mine[ph * 4 + 2] = global_ns();
        if (ph + 1 == nphases) break;
        if (nxt.kind == PH_GEMV && nxt.g.xmode == X_NORM) {
            nw1 = nxt.g.yres != nullptr ? __ldg(reinterpret_cast<const float4*>(nxt.g.w1 + (size_t)threadIdx.x * 4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            nw2 = nxt.g.w2 != nullptr ? __ldg(reinterpret_cast<const float4*>(nxt.g.w2 + (size_t)threadIdx.x * 4)) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        }
        // While waiting, the descriptor after the next one replaces this phase's.
        if (!grid_barrier(counter, (ph + 1) * gridDim.x, status, ph + 2 < nphases ? phases + ph + 2 : nullptr, raw + OFF_PHASE + (ph & 1) * PHASE_BYTES, raw)) break;
        if (stamp) mine[ph * 4 + 3] = global_ns();
    }
}

}  // namespace

bool step_supports(const GemvParams& p) {
    if (p.gelu_mul != nullptr) return false;  // the per-layer input's gate: not in the single-kernel step
    if (p.cols == 2048)
        return (p.xmode == X_NORM && (p.epi == EPI_F32 || p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX)) || ((p.xmode == X_F32 || p.xmode == X_ATTN) && p.epi == EPI_F32);
    return (p.cols == 4096 || p.cols == 8192 || p.cols == 16384) && p.xmode == X_F32 && p.epi == EPI_F32;
}

// Ring stages (34 KiB each, per block) the producer hints to the L2 ahead of its loads; TACHYON_B200_AHEAD overrides.
static uint32_t hint_depth() {
    static const uint32_t v = [] {
        const char* e = getenv("TACHYON_B200_AHEAD");
        return (uint32_t)(e ? atoi(e) : 6);
    }();
    return v;
}

int launch_step(tb_context* ctx, const StepPhase* phases, uint32_t n, uint32_t* counter, const uint32_t* state, unsigned long long* times) {
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        int per_sm = 0;
        TB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, THREADS, SMEM_BYTES));
        if (per_sm < 1) return fail(UNSUPPORTED, "fused step: a block does not fit an SM");
        configured[ctx->gpu & 15] = true;
    }
    TB_CUDA(cudaMemsetAsync(counter, 0, 4, ctx->stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctx->sms);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all blocks resident: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, decode_step_kernel, phases, n, counter, ctx->status, times, hint_depth(), state));
    return OK;
}

}  // namespace tb
