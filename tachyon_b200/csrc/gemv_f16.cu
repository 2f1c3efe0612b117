// Matrix-vector product with f16 weights: y = W x, W f16 [rows, cols] row-major, f32 accumulation.  The reference keeps
// f16 weights where a model is too small for 8-bit codes to pay (its encoder's gemm_f16, crates/tachyon/src/ptx/
// encoder.rs:498-525, chosen by encoder/convert.rs:26-29); at one token that product is this kernel.  Same prologues and
// outputs as the Q8 product of gemv.cu: the vector as f16 or f32, or the reference's residual / RMS-norm step
// (ptx/mod.rs:24-30) computed on the way in; f32 or f16 out.
//
// HBM-bound and simple: no shared-memory ring.  A warp takes two rows at a time and walks them in pieces of 16 bytes a lane
// (8 weights), four pieces of each row in flight a lane, loads marked as streaming; the vector sits in shared memory as
// f32.  Each weight costs half a conversion and one FMA, far below what the memory system delivers.  Blocks take their
// warps' row pairs round-robin so that every SM streams from the first microsecond to the last.
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int F16_THREADS = 512;
constexpr int F16_WARPS = F16_THREADS / 32;
constexpr int F16_MAX_COLS = 16384;  // the vector as f32 in shared memory: 64 KiB

__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float dot8(const uint4& w, const float* x) {
    const float4 a = *reinterpret_cast<const float4*>(x), b = *reinterpret_cast<const float4*>(x + 4);
    const float2 w0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), w1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    const float2 w2 = __half22float2(*reinterpret_cast<const __half2*>(&w.z)), w3 = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
    float s = w0.x * a.x;
    s = fmaf(w0.y, a.y, s), s = fmaf(w1.x, a.z, s), s = fmaf(w1.y, a.w, s);
    s = fmaf(w2.x, b.x, s), s = fmaf(w2.y, b.y, s), s = fmaf(w3.x, b.z, s), s = fmaf(w3.y, b.w, s);
    return s;
}

// Four 16-byte pieces of either row of a pair, from column c0 on (256 columns apart); pieces past the row's end are zeros.
__device__ __forceinline__ void load_batch(const __half* wa, const __half* wb, uint32_t c0, uint32_t K, uint4 (&a)[4], uint4 (&b)[4]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t c = c0 + j * 256;
        if (c < K) a[j] = ld_stream_u4(wa + c), b[j] = ld_stream_u4(wb + c);
        else a[j] = b[j] = make_uint4(0u, 0u, 0u, 0u);
    }
}

template <int XMODE, int EPI>
__global__ void __launch_bounds__(F16_THREADS, 2) gemv_f16_kernel(const GemvF16Params p) {
    extern __shared__ __align__(16) float xs[];  // [cols], then four sums a warp
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t threads = blockDim.x, nwarps = threads >> 5;
    const uint32_t K = p.cols;
    // The weights depend on no kernel: a warp asks for the first pieces of its first pair of rows before it waits for the
    // kernel in front of this one and before the vector is in shared memory.
    const uint32_t pairs = (p.rows + 1) / 2, stride = gridDim.x * nwarps;
    uint32_t pr = blockIdx.x * nwarps + warp;
    uint4 a[4], b[4];
    if (pr < pairs) {
        const uint32_t r0 = 2 * pr, r1 = min(r0 + 1, p.rows - 1);
        load_batch(p.w + (size_t)r0 * K, p.w + (size_t)r1 * K, lane * 8, K, a, b);
    }
    pdl_wait();
    // The vector.
    if constexpr (XMODE == X_F16) {
        for (uint32_t i = t; i < K / 8; i += threads) {
            const uint4 u = ld_cg_u4(static_cast<const __half*>(p.x) + (size_t)i * 8);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                xs[i * 8 + 2 * j] = f.x, xs[i * 8 + 2 * j + 1] = f.y;
            }
        }
    } else if constexpr (XMODE == X_F32) {
        for (uint32_t i = t; i < K / 4; i += threads) *reinterpret_cast<float4*>(xs + i * 4) = ld_cg_f4(static_cast<const float*>(p.x) + (size_t)i * 4);
    } else {
        // h' = (h + w1 * rmsnorm(y)) * hscale, x = w2 * rmsnorm(h'): one pass of four sums, as gemv.cu's prologue.
        float sy = 0.0f, sh = 0.0f, sha = 0.0f, sa = 0.0f;
        for (uint32_t i = t; i < K; i += threads) {
            const float h = ld_cg_f(p.h + i);
            float av = 0.0f;
            if (p.yres != nullptr) {
                const float y = ld_cg_f(p.yres + i);
                av = y * __ldg(p.w1 + i);
                sy = fmaf(y, y, sy);
            }
            sh = fmaf(h, h, sh), sha = fmaf(h, av, sha), sa = fmaf(av, av, sa);
        }
        sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
        float4* sums = reinterpret_cast<float4*>(xs + K);
        if (lane == 0) sums[warp] = make_float4(sy, sh, sha, sa);
        __syncthreads();
        sy = sh = sha = sa = 0.0f;
        for (uint32_t k = 0; k < nwarps; k++) {
            const float4 q = sums[k];
            sy += q.x, sh += q.y, sha += q.z, sa += q.w;
        }
        const float n = static_cast<float>(K);
        const float ry = p.yres != nullptr ? rsqrtf(sy / n + p.eps) : 0.0f;
        const float hs = p.yres != nullptr ? p.hscale : 1.0f;
        const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
        const float rh = p.w2 != nullptr ? rsqrtf(fmaxf(sq, 0.0f) / n + p.eps) : 1.0f;
        for (uint32_t i = t; i < K; i += threads) {
            const float h = ld_cg_f(p.h + i);
            const float av = p.yres != nullptr ? ld_cg_f(p.yres + i) * __ldg(p.w1 + i) : 0.0f;
            const float v = fmaf(av, ry, h) * hs;
            if (blockIdx.x == 0 && p.h_out != nullptr) p.h_out[i] = v;
            xs[i] = v * rh * (p.w2 != nullptr ? __ldg(p.w2 + i) : 1.0f);
        }
    }
    __syncthreads();
    pdl_launch_dependents();

    // Row pairs, round-robin over all warps of the grid.  The first four pieces of a pair's rows are already on their way
    // when its turn comes: those of the next pair are asked for before this pair's sums are reduced.
    for (; pr < pairs; pr += stride) {
        const uint32_t r0 = 2 * pr, r1 = min(r0 + 1, p.rows - 1);  // a lone last row is read twice
        const __half* wa = p.w + (size_t)r0 * K;
        const __half* wb = p.w + (size_t)r1 * K;
        float sa = 0.0f, sb = 0.0f;
        uint32_t c = lane * 8;
        while (true) {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (c + j * 256 < K) sa += dot8(a[j], xs + c + j * 256), sb += dot8(b[j], xs + c + j * 256);
            c += 4 * 256;
            if (c >= K) break;
            load_batch(wa, wb, c, K, a, b);
        }
        const uint32_t next = pr + stride;
        if (next < pairs) {
            const uint32_t n0 = 2 * next, n1 = min(n0 + 1, p.rows - 1);
            load_batch(p.w + (size_t)n0 * K, p.w + (size_t)n1 * K, lane * 8, K, a, b);
        }
        // Both rows in five exchanges.
        const bool upper = lane & 16;
        float r = (upper ? sb : sa) + __shfl_xor_sync(0xffffffffu, upper ? sa : sb, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        const uint32_t row = r0 + (upper ? 1u : 0u);
        if ((lane & 15) == 0 && row < p.rows && (!upper || r1 != r0)) {
            if constexpr (EPI == EPI_F16) static_cast<__half*>(p.y)[row] = __float2half_rn(r);
            else static_cast<float*>(p.y)[row] = r;
        }
    }
}

// Warps a block (two blocks an SM) for which the last round of row pairs leaves the fewest warps idle.
static uint32_t pick_warps(uint32_t pairs, uint32_t sms) {
    uint32_t best = F16_WARPS;
    double best_eff = 0.0;
    for (uint32_t w = F16_WARPS; w >= 10; w--) {
        const uint64_t slots = (uint64_t)2 * sms * w, rounds = (pairs + slots - 1) / slots;
        const double eff = (double)pairs / (double)(rounds * slots);
        if (eff > best_eff + 1e-9) best_eff = eff, best = w;
    }
    return best;
}

template <int XMODE, int EPI>
int launch_one(tb_context* ctx, const GemvF16Params& p) {
    const size_t smem = (size_t)p.cols * 4 + F16_WARPS * 16;
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(gemv_f16_kernel<XMODE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, F16_MAX_COLS * 4 + F16_WARPS * 16));
        configured[ctx->gpu & 15] = true;
    }
    const uint32_t pairs = (p.rows + 1) / 2;
    const uint32_t warps = pick_warps(pairs, (uint32_t)ctx->sms);
    uint32_t grid = (uint32_t)ctx->sms * 2;  // two blocks an SM
    const uint32_t most = (pairs + warps - 1) / warps;
    if (grid > most) grid = most;
    TB_CUDA(launch_kernel(ctx, gemv_f16_kernel<XMODE, EPI>, dim3(grid), dim3(warps * 32), smem, true, p));
    return OK;
}

}  // namespace

int launch_gemv_f16(tb_context* ctx, const GemvF16Params& p) {
    if (p.rows == 0 || p.cols == 0 || p.cols % 256 != 0 || p.cols > (uint32_t)F16_MAX_COLS) return fail(OUT_OF_RANGE, "gemv_f16: cols must be a multiple of 256, at most 16384");
    if (p.w == nullptr || p.y == nullptr || (reinterpret_cast<uintptr_t>(p.w) & 15)) return fail(OUT_OF_RANGE, "gemv_f16: weights and output must be present, weights 16-byte aligned");
    if (p.xmode == X_NORM) {
        if (p.h == nullptr || (p.yres != nullptr && p.w1 == nullptr)) return fail(OUT_OF_RANGE, "gemv_f16: the norm prologue needs h, and w1 with y");
    } else if (p.x == nullptr || (reinterpret_cast<uintptr_t>(p.x) & 15)) {
        return fail(OUT_OF_RANGE, "gemv_f16: the input vector must be present and 16-byte aligned");
    }
    const bool f16out = p.epi == EPI_F16;
    if (p.epi != EPI_F16 && p.epi != EPI_F32) return fail(UNSUPPORTED, "gemv_f16: f32 or f16 output");
    switch (p.xmode) {
        case X_F16: return f16out ? launch_one<X_F16, EPI_F16>(ctx, p) : launch_one<X_F16, EPI_F32>(ctx, p);
        case X_F32: return f16out ? launch_one<X_F32, EPI_F16>(ctx, p) : launch_one<X_F32, EPI_F32>(ctx, p);
        case X_NORM: return f16out ? launch_one<X_NORM, EPI_F16>(ctx, p) : launch_one<X_NORM, EPI_F32>(ctx, p);
        default: return fail(UNSUPPORTED, "gemv_f16: unknown input mode");
    }
}

}  // namespace tb
