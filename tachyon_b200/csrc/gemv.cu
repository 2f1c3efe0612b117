// Q8-weight matrix-vector product for batch-1 decode: y = W x with W int8 [rows, cols] and one f16 scale per 32
// weights along a row.  Replaces the reference's gemv_q4 (crates/tachyon/src/ptx/gemv.rs:156-195) together with the
// small kernels the reference launches around it: the residual/RMS-norm step (norm_q8, ptx/mod.rs:404-511) runs as
// this kernel's prologue, GeGLU (geglu_q8, ptx/mod.rs:376-393) and the greedy pick (sample, ptx/sample.rs:387-417) as
// its epilogues.
//
// Structure (one persistent block per SM, 8 consumer warps + 1 producer warp):
//  * every block owns a contiguous range of rows, so its weights are one contiguous byte range; the producer streams it
//    through a ring of 16 KiB stages with one-dimensional bulk copies (cp.async.bulk) completing on mbarriers.  The
//    weights do not depend on the previous kernel, so the producer starts before griddepcontrol.wait and the ring is
//    full by the time the activations arrive;
//  * the activation vector is split, per block of 32 values, into three byte planes of a 23-bit fixed-point number and a
//    power-of-two multiplier; each consumer warp keeps the planes of its 2048-wide segment in registers, so a weight
//    byte costs 3/4 of a dp4a and no conversion.  Block sums are exact integers, combined in f32 with the weight scale;
//  * lanes reduce with shuffles; warps that share a row (cols > 2048) or a gate/up pair meet on a named barrier.
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int STAGES = 6;
constexpr int STAGE_W = 16384;  // weight bytes per stage
constexpr int STAGE_S = 1024;   // scale bytes per stage (one f16 per 32 weights)
constexpr int CONSUMERS = 8;    // consumer warps
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int SEG = 2048;       // columns one warp covers with its register-resident activation planes

struct Smem {
    uint8_t w[STAGES][STAGE_W];
    uint8_t s[STAGES][STAGE_S];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    float red[2][CONSUMERS];
    float bestv[CONSUMERS];
    uint32_t besti[CONSUMERS];
};

// The three byte planes (signed high, unsigned middle and low) of 32 activations, and 2^(e-21): x ~ X * mul with
// X = hi*65536 + mid*256 + lo, |X| <= 2^22.  Words 0..3 hold values 0..15, words 4..7 values 16..31.
struct Planes {
    uint32_t hi[8], mid[8], lo[8];
    float mul;
};

__device__ __forceinline__ void make_planes(const float (&v)[32], Planes& p, bool swap_halves) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(v[j]));
    uint32_t eb = __float_as_uint(amax) >> 23;  // biased exponent of the largest magnitude
    eb = min(eb, 254u);
    const bool zero = eb < 22u;                 // below 2^-105: the block counts as zero
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);  // 2^(21 - e)
    p.mul = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);           // 2^(e - 21)
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int x0 = __float2int_rn(v[4 * k] * sc), x1 = __float2int_rn(v[4 * k + 1] * sc);
        const int x2 = __float2int_rn(v[4 * k + 2] * sc), x3 = __float2int_rn(v[4 * k + 3] * sc);
        p.hi[k] = __byte_perm(__byte_perm(x0, x1, 0x0062), __byte_perm(x2, x3, 0x0062), 0x5410);
        p.mid[k] = __byte_perm(__byte_perm(x0, x1, 0x0051), __byte_perm(x2, x3, 0x0051), 0x5410);
        p.lo[k] = __byte_perm(__byte_perm(x0, x1, 0x0040), __byte_perm(x2, x3, 0x0040), 0x5410);
    }
    if (swap_halves) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t t;
            t = p.hi[k], p.hi[k] = p.hi[k + 4], p.hi[k + 4] = t;
            t = p.mid[k], p.mid[k] = p.mid[k + 4], p.mid[k + 4] = t;
            t = p.lo[k], p.lo[k] = p.lo[k + 4], p.lo[k + 4] = t;
        }
    }
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

// The activation planes of blocks `b0` and `b0 + 32` of the input vector, for this lane.
template <int XMODE>
__device__ __forceinline__ void load_planes(const GemvParams& p, uint32_t b0, bool swap_halves, bool writer, Planes (&pl)[2]) {
    float v[32];
    if constexpr (XMODE == X_F16) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            load32_f16(static_cast<const __half*>(p.x) + (size_t)(b0 + 32 * i) * 32, v);
            make_planes(v, pl[i], swap_halves);
        }
    } else if constexpr (XMODE == X_F32) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            load32_f32(static_cast<const float*>(p.x) + (size_t)(b0 + 32 * i) * 32, v);
            make_planes(v, pl[i], swap_halves);
        }
    } else {
        // Residual step and RMS-norm over the whole vector (cols == 2048: the warp's lanes hold all of it).
        // Sums in one pass, as the reference does (ptx/mod.rs:24-30): sum y^2, sum h^2, sum h*a, sum a^2 with a = y*w1;
        // mean(h'^2) follows from them.
        const float n = static_cast<float>(p.cols);
        float ry = 0.0f, rh = 1.0f;
        if (p.yres != nullptr || p.w2 != nullptr) {
            float sy = 0.0f, sh = 0.0f, sha = 0.0f, sa = 0.0f;
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const size_t at = (size_t)(b0 + 32 * i) * 32;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float4 h = ld_cg_f4(p.h + at + 4 * k);
                    const float hv[4] = {h.x, h.y, h.z, h.w};
                    float av[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (p.yres != nullptr) {
                        const float4 y = ld_cg_f4(p.yres + at + 4 * k);
                        const float4 w = __ldg(reinterpret_cast<const float4*>(p.w1 + at + 4 * k));
                        av[0] = y.x * w.x, av[1] = y.y * w.y, av[2] = y.z * w.z, av[3] = y.w * w.w;
                        sy += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) sh = fmaf(hv[j], hv[j], sh), sha = fmaf(hv[j], av[j], sha), sa = fmaf(av[j], av[j], sa);
                }
            }
            sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
            if (p.yres != nullptr) ry = rsqrtf(sy / n + p.eps);
            const float hs = p.yres != nullptr ? p.hscale : 1.0f;  // without a residual the state passes through unscaled
            const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
            if (p.w2 != nullptr) rh = rsqrtf(fmaxf(sq, 0.0f) / n + p.eps);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const size_t at = (size_t)(b0 + 32 * i) * 32;
            load32_f32(p.h + at, v);
            if (p.yres != nullptr) {
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float4 y = ld_cg_f4(p.yres + at + 4 * k);
                    const float4 w = __ldg(reinterpret_cast<const float4*>(p.w1 + at + 4 * k));
                    v[4 * k] = fmaf(y.x * ry, w.x, v[4 * k]) * p.hscale;
                    v[4 * k + 1] = fmaf(y.y * ry, w.y, v[4 * k + 1]) * p.hscale;
                    v[4 * k + 2] = fmaf(y.z * ry, w.z, v[4 * k + 2]) * p.hscale;
                    v[4 * k + 3] = fmaf(y.w * ry, w.w, v[4 * k + 3]) * p.hscale;
                }
            }
            if (writer && p.h_out != nullptr) {
#pragma unroll
                for (int k = 0; k < 8; k++) *reinterpret_cast<float4*>(p.h_out + at + 4 * k) = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
            }
            if (p.w2 != nullptr) {
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float4 w = __ldg(reinterpret_cast<const float4*>(p.w2 + at + 4 * k));
                    v[4 * k] *= rh * w.x, v[4 * k + 1] *= rh * w.y, v[4 * k + 2] *= rh * w.z, v[4 * k + 3] *= rh * w.w;
                }
            }
            make_planes(v, pl[i], swap_halves);
        }
    }
}

template <int WPR, int XMODE, int EPI>
__global__ void __launch_bounds__(THREADS, 2) gemv_q8_kernel(const GemvParams p, uint32_t* status) {
    extern __shared__ __align__(128) uint8_t raw[];
    Smem& sm = *reinterpret_cast<Smem*>(raw);
    constexpr int ROWS = CONSUMERS / WPR;                  // rows per stage
    constexpr int UNIT = (EPI == EPI_GEGLU) ? 2 : 1;       // rows that stay in one block
    constexpr int GROUP = (EPI == EPI_GEGLU) ? 2 : WPR;    // warps that produce one output together
    const uint32_t K = p.cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t units = p.rows / UNIT;
    const uint32_t r0 = static_cast<uint32_t>((uint64_t)units * blockIdx.x / gridDim.x) * UNIT;
    const uint32_t r1 = static_cast<uint32_t>((uint64_t)units * (blockIdx.x + 1) / gridDim.x) * UNIT;
    const uint32_t nst = (r1 - r0 + ROWS - 1) / ROWS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) mbar_init(&sm.full[i], 1), mbar_init(&sm.empty[i], CONSUMERS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // Producer: one thread streams this block's rows.  Nothing it reads is written by another kernel.
        if (lane == 0) {
            bool ok = true;
            for (uint32_t i = 0; i < nst && ok; i++) {
                const uint32_t s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&sm.empty[s], ((i / STAGES) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    ok = false;
                    break;
                }
                const uint32_t row = r0 + i * ROWS, here = min((uint32_t)ROWS, r1 - row);
                const uint32_t bw = here * K, bs = here * (K / 16);
                mbar_expect_tx(&sm.full[s], bw + bs);
                bulk_load(sm.w[s], p.w + (size_t)row * K, bw, &sm.full[s]);
                bulk_load(sm.s[s], p.s + (size_t)row * (K / 32), bs, &sm.full[s]);
            }
            pdl_launch_dependents();
        }
        return;
    }

    // Consumers.  Everything below may read what the previous kernel wrote.
    pdl_wait();
    const int seg = warp % WPR, rin = warp / WPR;  // the warp's column segment, and its row within a stage
    const bool sw = (lane >> 2) & 1;               // which 16-byte half of its blocks the lane loads first (bank spread)
    Planes pl[2];
    load_planes<XMODE>(p, (uint32_t)seg * 64 + lane, sw, blockIdx.x == 0 && warp == 0, pl);

    float bestv = -INFINITY;
    uint32_t besti = 0xffffffffu;
    bool ok = true;
    for (uint32_t i = 0; i < nst; i++) {
        const uint32_t s = i % STAGES;
        if (ok && !mbar_wait(&sm.full[s], (i / STAGES) & 1)) {
            atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
            ok = false;
        }
        const uint32_t row = r0 + i * ROWS + rin;
        float v = 0.0f;
        if (ok && row < r1) {
            const uint8_t* wr = sm.w[s] + (size_t)rin * K + seg * SEG;
            const __half* sr = reinterpret_cast<const __half*>(sm.s[s]) + rin * (K / 32) + seg * 64;
            const uint4 a0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + (sw ? 1 : 0)) * 16);
            const uint4 b0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + (sw ? 0 : 1)) * 16);
            const uint4 a1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + (sw ? 1 : 0)) * 16);
            const uint4 b1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + (sw ? 0 : 1)) * 16);
            const float s0 = __half2float(sr[lane]) * pl[0].mul, s1 = __half2float(sr[lane + 32]) * pl[1].mul;
            v = block_dot(a0, b0, pl[0]) * s0;
            v = fmaf(block_dot(a1, b1, pl[1]), s1, v);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[s]);
        v = warp_sum(v);
        if constexpr (GROUP > 1) {
            if (lane == 0) sm.red[i & 1][warp] = v;
            named_bar_sync(1 + warp / GROUP, GROUP * 32);
            if (warp % GROUP != 0) continue;
            if constexpr (EPI == EPI_GEGLU) {
                v = gelu_tanh(sm.red[i & 1][warp]) * sm.red[i & 1][warp + 1];
            } else {
                v = 0.0f;
#pragma unroll
                for (int j = 0; j < GROUP; j++) v += sm.red[i & 1][warp + j];
            }
        }
        if (lane == 0 && row < r1) {
            if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[row] = v;
            if constexpr (EPI == EPI_F16) static_cast<__half*>(p.y)[row] = __float2half_rn(v);
            if constexpr (EPI == EPI_GEGLU) static_cast<float*>(p.y)[row / 2] = v;
            if constexpr (EPI == EPI_ARGMAX) {
                if (p.y != nullptr) static_cast<float*>(p.y)[row] = v;
                if (v > bestv) bestv = v, besti = row;
            }
        }
    }

    if constexpr (EPI == EPI_ARGMAX) {
        // Largest value, lowest row among equals (ptx/sample.rs:91-97): the key orders by value, then by inverted row.
        if (lane == 0) sm.bestv[warp] = bestv, sm.besti[warp] = besti;
        named_bar_sync(15, CONSUMERS * 32);
        if (threadIdx.x == 0) {
            unsigned long long key = 0;
            for (int j = 0; j < CONSUMERS; j++) {
                const unsigned long long k = ((unsigned long long)float_key(sm.bestv[j]) << 32) | (0xffffffffu - sm.besti[j]);
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

// Any shape the staged kernel does not take (cols not a multiple of 2048): one warp per row straight from global
// memory, with the same block arithmetic.
template <int XMODE, int EPI>
__global__ void __launch_bounds__(256) gemv_q8_generic(const GemvParams p) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), nb = p.cols / 32;
    if (row >= p.rows) return;
    float sum = 0.0f;
    for (uint32_t b = lane; b < nb; b += 32) {
        float v[32];
        if constexpr (XMODE == X_F16) load32_f16(static_cast<const __half*>(p.x) + (size_t)b * 32, v);
        else load32_f32(static_cast<const float*>(p.x) + (size_t)b * 32, v);
        Planes pl;
        make_planes(v, pl, false);
        // Rows of a matrix whose width is not a multiple of 16 bytes... cols % 32 == 0, so 16-byte loads stay aligned.
        const uint4* wp = reinterpret_cast<const uint4*>(p.w + (size_t)row * p.cols + (size_t)b * 32);
        const uint4 a = __ldg(wp), c = __ldg(wp + 1);
        sum = fmaf(block_dot(a, c, pl), __half2float(p.s[(size_t)row * nb + b]) * pl.mul, sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) {
        if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[row] = sum;
        else static_cast<__half*>(p.y)[row] = __float2half_rn(sum);
    }
}

template <int WPR, int XMODE, int EPI>
int launch_staged(tb_context* ctx, const GemvParams& p) {
    auto kernel = gemv_q8_kernel<WPR, XMODE, EPI>;
    static bool configured[16] = {};  // per device ordinal
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
        configured[ctx->gpu & 15] = true;
    }
    constexpr uint32_t ROWS = CONSUMERS / WPR;
    constexpr uint32_t UNIT = (EPI == EPI_GEGLU) ? 2 : 1;
    // The argmax epilogue counts blocks, so its grid must not depend on anything but the shape.
    uint32_t grid = (uint32_t)ctx->sms;
    const uint32_t most = (p.rows / UNIT * UNIT + ROWS - 1) / ROWS;
    if (grid > most) grid = most > 0 ? most : 1;
    TB_CUDA(launch_kernel(ctx, kernel, dim3(grid), dim3(THREADS), sizeof(Smem), true, p, ctx->status));
    return OK;
}

template <int WPR>
int dispatch_staged(tb_context* ctx, const GemvParams& p) {
    if (p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX || p.xmode == X_NORM) {
        if constexpr (WPR == 1) {
            if (p.xmode == X_NORM && p.epi == EPI_F32) return launch_staged<1, X_NORM, EPI_F32>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_F16) return launch_staged<1, X_NORM, EPI_F16>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_GEGLU) return launch_staged<1, X_NORM, EPI_GEGLU>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_ARGMAX) return launch_staged<1, X_NORM, EPI_ARGMAX>(ctx, p);
            if (p.xmode == X_F32 && p.epi == EPI_GEGLU) return launch_staged<1, X_F32, EPI_GEGLU>(ctx, p);
            if (p.xmode == X_F32 && p.epi == EPI_ARGMAX) return launch_staged<1, X_F32, EPI_ARGMAX>(ctx, p);
            if (p.xmode == X_F16 && p.epi == EPI_GEGLU) return launch_staged<1, X_F16, EPI_GEGLU>(ctx, p);
            if (p.xmode == X_F16 && p.epi == EPI_ARGMAX) return launch_staged<1, X_F16, EPI_ARGMAX>(ctx, p);
        }
        return fail(UNSUPPORTED, "gemv: the norm prologue, GeGLU and argmax epilogues need cols == 2048");
    }
    if (p.xmode == X_F16 && p.epi == EPI_F32) return launch_staged<WPR, X_F16, EPI_F32>(ctx, p);
    if (p.xmode == X_F16 && p.epi == EPI_F16) return launch_staged<WPR, X_F16, EPI_F16>(ctx, p);
    if (p.xmode == X_F32 && p.epi == EPI_F32) return launch_staged<WPR, X_F32, EPI_F32>(ctx, p);
    if (p.xmode == X_F32 && p.epi == EPI_F16) return launch_staged<WPR, X_F32, EPI_F16>(ctx, p);
    return fail(UNSUPPORTED, "gemv: unknown input or output mode");
}

}  // namespace

size_t gemv_smem_bytes() { return sizeof(Smem); }

int launch_gemv(tb_context* ctx, const GemvParams& p) {
    if (p.rows == 0 || p.cols == 0 || p.cols % 32 != 0) return fail(OUT_OF_RANGE, "gemv: cols must be a positive multiple of 32");
    if (p.w == nullptr || p.s == nullptr) return fail(OUT_OF_RANGE, "gemv: null weights");
    if ((reinterpret_cast<uintptr_t>(p.w) | reinterpret_cast<uintptr_t>(p.s)) & 15) return fail(OUT_OF_RANGE, "gemv: weights and scales must be 16-byte aligned");
    if (p.xmode == X_NORM) {
        if (p.h == nullptr || (p.yres != nullptr && p.w1 == nullptr)) return fail(OUT_OF_RANGE, "gemv: the norm prologue needs h, and w1 with y");
    } else if (p.x == nullptr || (reinterpret_cast<uintptr_t>(p.x) & 15)) {
        return fail(OUT_OF_RANGE, "gemv: the input vector must be present and 16-byte aligned");
    }
    if (p.epi == EPI_GEGLU && p.rows % 2 != 0) return fail(OUT_OF_RANGE, "gemv: GeGLU needs an even number of rows");
    if (p.epi == EPI_ARGMAX && (p.best == nullptr || p.count == nullptr || p.state == nullptr)) return fail(OUT_OF_RANGE, "gemv: argmax needs best, count and state");
    if (p.epi != EPI_ARGMAX && p.y == nullptr) return fail(OUT_OF_RANGE, "gemv: null output");
    switch (p.cols) {
        case 2048: return dispatch_staged<1>(ctx, p);
        case 4096: return dispatch_staged<2>(ctx, p);
        case 8192: return dispatch_staged<4>(ctx, p);
        case 16384: return dispatch_staged<8>(ctx, p);
        default: break;
    }
    if (p.xmode == X_NORM || p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX) return fail(UNSUPPORTED, "gemv: fused prologue/epilogues need cols of 2048");
    const dim3 grid((p.rows + 7) / 8), block(256);
    if (p.xmode == X_F16 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F16, EPI_F32>, grid, block, 0, true, p));
    else if (p.xmode == X_F16 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F16, EPI_F16>, grid, block, 0, true, p));
    else if (p.xmode == X_F32 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F32, EPI_F32>, grid, block, 0, true, p));
    else if (p.xmode == X_F32 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F32, EPI_F16>, grid, block, 0, true, p));
    else return fail(UNSUPPORTED, "gemv: unknown input or output mode");
    return OK;
}

}  // namespace tb
