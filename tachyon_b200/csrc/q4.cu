// The reference's own decode formats: Q4 weights (two per byte, an f16 scale per group of 64, crates/tachyon/src/quant.rs:47-82)
// times Q8 activations (i8 codes and [s, s * sum q] per block of 32, quant.rs:93-130), f32 out.
//
//   quant_q8_kernel  = quant_q8   (ptx/mod.rs:191-212, 393-399)
//   geglu_q8_kernel  = geglu_q8   (ptx/mod.rs:376-393): gelu(a) * b in its tanh form, then Q8
//   norm_q8_kernel   = norm_q8    (ptx/mod.rs:404-511): residual step, RMS norms, Q8 of the next input
//   embed_q4_rows    = embed_q4   (ptx/mod.rs:531-598): rows of a Q4 table, one per token
//   gemv_q4_kernel   = gemv_q4    (ptx/gemv.rs:156-195)
//
// Both follow the reference kernels' arithmetic operation by operation, all of it IEEE f32 with round-to-nearest
// (div.rn, mul.rn, fma.rn, cvt.rni) or exact integer sums, so the results are the reference's bit for bit:
//   * a block of 32 activations: d = amax / 127, q = rni(x * (127 / amax)), pair [d, f32(sum q) * d];
//   * a row: lane l of one warp takes the chunks of 32 weights l, l + 32, ... in rising order, each adding
//     fma(fma(ss, -8, f32(sum n q) * sx), f32(scale), sum) to the lane's sum, and the lanes' sums meet in a butterfly
//     with partners 16, 8, 4, 2, 1.
// What differs is how the bytes travel: a producer warp streams each block's rows through a ring of shared-memory
// stages with bulk copies, ahead of the wait for the previous kernel, as the Q8 kernel of gemv.cu does.
#include "common.cuh"
#include "internal.h"

#include <algorithm>

namespace tb {

namespace {

constexpr int CONSUMERS = 16;
constexpr int CTHREADS = CONSUMERS * 32;
constexpr int THREADS = CTHREADS + 32;
constexpr int STAGE_W = 32768;            // bytes of packed weights per stage
constexpr int STAGE_S = STAGE_W / 16;     // their scales: 2 bytes per 32 bytes of weights
constexpr int NST = 6;

struct Layout {
    static constexpr int W = 0;
    static constexpr int S = W + NST * STAGE_W;
    static constexpr int FULL = S + NST * STAGE_S;
    static constexpr int EMPTY = FULL + NST * 8;
    static constexpr int X = EMPTY + NST * 8 + 32;  // the activations: first and second 16 bytes of every chunk, then the pairs
};
static size_t smem_bytes(uint32_t cols) { return (size_t)Layout::X + cols + cols / 4; }

// One warp per 32 values, as the reference's q8 (ptx/mod.rs:191-212).
__global__ void __launch_bounds__(256) quant_q8_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float2* __restrict__ s, uint32_t n) {
    pdl_wait();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;  // n is a multiple of 32: whole warps leave together
    const float v = x[i];
    const float amax = warp_max(fabsf(v));
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int code = __float2int_rn(__fmul_rn(v, inv));
    q[i] = static_cast<int8_t>(code);
    int sum = code;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((i & 31u) == 0) s[i >> 5] = make_float2(d, __fmul_rn(static_cast<float>(sum), d));
}

// Value x of element i -> Q8 (ptx/mod.rs:191-212): every thread of the warp calls this with the warp's 32 consecutive values.
__device__ __forceinline__ void store_q8(float x, uint32_t i, int8_t* q, float2* s) {
    const float amax = warp_max(fabsf(x));
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int code = __float2int_rn(__fmul_rn(x, inv));
    q[i] = static_cast<int8_t>(code);
    int sum = code;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((i & 31u) == 0) s[i >> 5] = make_float2(d, __fmul_rn(static_cast<float>(sum), d));
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
    float y;
    asm("rsqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ptx/mod.rs:376-393: x / (1 + e^(-2u)) * b, u = sqrt(2/pi) (x + 0.044715 x^3), operation by operation.
__global__ void __launch_bounds__(256) geglu_q8_kernel(const float* __restrict__ a, const float* __restrict__ b, int8_t* __restrict__ q, float2* __restrict__ s,
                                                       uint32_t n) {
    pdl_wait();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float x = a[i];
    float t = __fmul_rn(x, x);
    t = __fmaf_rn(t, 0.044714998453855514526f, 1.0f);          // 0f3D372713
    t = __fmul_rn(t, x);
    t = __fmul_rn(t, -2.3022081851959228516f);                 // 0fC0135761 = -2 sqrt(2/pi) log2(e)
    t = __fadd_rn(ex2_approx(t), 1.0f);
    x = __fmul_rn(__fdiv_rn(x, t), b[i]);
    store_q8(x, i, q, s);
}

// Sums of up to four values over a block of eight warps, in every thread, in the order of the reference's block()
// (ptx/mod.rs:153-170): warp butterflies, one slot per warp, lanes 0..7 read the slots, butterflies again.
__device__ __forceinline__ void block_sums4(float (&v)[4], float* red) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 4; k++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[k] = __fadd_rn(v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
    if (lane == 0)
#pragma unroll
        for (int k = 0; k < 4; k++) red[32 * k + warp] = v[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; k++) v[k] = lane < 8 ? red[32 * k + lane] : 0.0f;
#pragma unroll
    for (int k = 0; k < 4; k++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[k] = __fadd_rn(v[k], __shfl_xor_sync(0xffffffffu, v[k], o));
    __syncthreads();
}

// ptx/mod.rs:404-511.  Grid (len / 256, chunks) x 256 threads; every block reads its whole chunk (thread t takes values
// t, t + 256, ...: up to 24), reduces sum y^2, sum h^2, sum h a, sum a^2 (a = w1 y) at once, and writes its own slice
// of the new h and of the Q8 output.
constexpr int NORM_PER_THREAD = 24;
__global__ void __launch_bounds__(256) norm_q8_kernel(const float* __restrict__ h, float* h_out, const float* __restrict__ y, const float* __restrict__ w1,
                                                      const float* __restrict__ w2, int8_t* q, float2* s, uint32_t len, float eps, float scale) {
    __shared__ float red[128];
    pdl_wait();
    const uint32_t th = threadIdx.x, slice = blockIdx.x, base = blockIdx.y * len, own = slice * 256 + th;
    const float n = static_cast<float>(len);
    float hv[NORM_PER_THREAD], yv[NORM_PER_THREAD], av[NORM_PER_THREAD];
#pragma unroll
    for (int k = 0; k < NORM_PER_THREAD; k++) {
        const uint32_t i = th + 256 * k;
        const bool in = i < len;
        hv[k] = in ? h[base + i] : 0.0f;
        yv[k] = (in && y != nullptr) ? y[base + i] : 0.0f;
        av[k] = (in && y != nullptr) ? w1[i] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < NORM_PER_THREAD; k++) av[k] = __fmul_rn(av[k], yv[k]);
    float v[4] = {__fmul_rn(yv[0], yv[0]), __fmul_rn(hv[0], hv[0]), __fmul_rn(hv[0], av[0]), __fmul_rn(av[0], av[0])};
#pragma unroll
    for (int k = 1; k < NORM_PER_THREAD; k++) v[0] = __fmaf_rn(yv[k], yv[k], v[0]);
#pragma unroll
    for (int k = 1; k < NORM_PER_THREAD; k++) v[1] = __fmaf_rn(hv[k], hv[k], v[1]);
#pragma unroll
    for (int k = 1; k < NORM_PER_THREAD; k++) v[2] = __fmaf_rn(hv[k], av[k], v[2]);
#pragma unroll
    for (int k = 1; k < NORM_PER_THREAD; k++) v[3] = __fmaf_rn(av[k], av[k], v[3]);
    block_sums4(v, red);
    float ss = v[0], sh = v[1], su = v[2], uu = v[3];
    float r = rsqrt_approx(__fadd_rn(__fdiv_rn(ss, n), eps));
    if (y != nullptr) {
#pragma unroll
        for (int k = 0; k < NORM_PER_THREAD; k++) {
            hv[k] = __fmul_rn(__fmaf_rn(av[k], r, hv[k]), scale);
            if (slice == (uint32_t)k && th + 256 * k < len) h_out[base + th + 256 * k] = hv[k];
        }
        su = __fadd_rn(su, su);
        su = __fmaf_rn(r, uu, su);
        sh = __fmaf_rn(r, su, sh);
        sh = __fmul_rn(__fmul_rn(sh, scale), scale);
    }
    if (q == nullptr) return;
    r = rsqrt_approx(__fadd_rn(__fdiv_rn(sh, n), eps));
    if (w2 == nullptr) r = 1.0f;
    float x = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_PER_THREAD; k++)
        if (slice == (uint32_t)k) x = hv[k];
    x = __fmul_rn(x, r);
    x = __fmul_rn(x, w2 != nullptr ? w2[own] : 1.0f);
    store_q8(x, base + own, q, s);
}

// ptx/mod.rs:531-598: thread i decodes weight i of row token[blockIdx.y] into row blockIdx.y of the output.
__global__ void __launch_bounds__(256) embed_q4_rows(const uint8_t* __restrict__ w, const __half* __restrict__ s, const uint32_t* __restrict__ token, float* out,
                                                     uint32_t cols, float scale) {
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cols) return;
    const uint32_t tok = token[blockIdx.y], g = i >> 6, k = i & 63;
    const float d = __half2float(s[(size_t)tok * (cols >> 6) + g]);
    const uint32_t byte = w[(size_t)tok * (cols >> 1) + (g << 5) + ((k >> 3) << 2) + (k & 3)];
    const int nib = static_cast<int>((byte >> (((k >> 2) & 1) << 2)) & 15u) - 8;
    out[(size_t)blockIdx.y * cols + i] = __fmul_rn(__fmul_rn(static_cast<float>(nib), d), scale);
}

struct Q4Params {
    const uint8_t* w;      // [rows][cols / 2]
    const __half* ws;      // [rows][cols / 64]
    const int8_t* q;       // [cols]
    const float2* s;       // [cols / 32]
    float* y;              // [rows]
    uint32_t rows, cols;
};

// The sum of 32 nibbles times 32 codes: weight word j holds nibbles 8j..8j+3 low and 8j+4..8j+7 high (quant.rs:60-66).
__device__ __forceinline__ int chunk_dot(const uint4& w, const uint4& a, const uint4& b) {
    int acc = 0;
    acc = dp4a_su(a.x, w.x & 0x0F0F0F0Fu, acc), acc = dp4a_su(a.y, (w.x >> 4) & 0x0F0F0F0Fu, acc);
    acc = dp4a_su(a.z, w.y & 0x0F0F0F0Fu, acc), acc = dp4a_su(a.w, (w.y >> 4) & 0x0F0F0F0Fu, acc);
    acc = dp4a_su(b.x, w.z & 0x0F0F0F0Fu, acc), acc = dp4a_su(b.y, (w.z >> 4) & 0x0F0F0F0Fu, acc);
    acc = dp4a_su(b.z, w.w & 0x0F0F0F0Fu, acc), acc = dp4a_su(b.w, (w.w >> 4) & 0x0F0F0F0Fu, acc);
    return acc;
}
// One chunk's step of a lane's sum (gemv.rs:100-110).
__device__ __forceinline__ float chunk_step(int acc, const float2& sc, float scale, float sum) {
    float f = __fmul_rn(static_cast<float>(acc), sc.x);
    f = __fmaf_rn(sc.y, -8.0f, f);
    return __fmaf_rn(f, scale, sum);
}

// NCH > 0: a lane's NCH chunks of the activations stay in registers (rows of up to 4096 columns); NCH == 0: they are
// read from shared memory chunk by chunk.
template <int NCH>
__global__ void __launch_bounds__(THREADS, 1) gemv_q4_kernel(const Q4Params p, uint32_t* status) {
    extern __shared__ __align__(128) uint8_t raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rb = p.cols / 2;            // bytes per row
    const uint32_t rps = STAGE_W / rb;         // rows per stage: 32 at 2048 columns, 4 at 16384
    const uint32_t r0 = static_cast<uint32_t>((uint64_t)p.rows * blockIdx.x / gridDim.x);
    const uint32_t r1 = static_cast<uint32_t>((uint64_t)p.rows * (blockIdx.x + 1) / gridDim.x);
    const uint32_t nst = (r1 - r0 + rps - 1) / rps;
    // Warps per stage: all sixteen when a stage holds at least sixteen rows, else one per row, the stages going round
    // the groups of warps.
    const uint32_t wps = min(rps, (uint32_t)CONSUMERS), groups = CONSUMERS / wps;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + Layout::FULL);
    uint64_t* empty = reinterpret_cast<uint64_t*>(raw + Layout::EMPTY);
    if (threadIdx.x == 0) {
        for (int i = 0; i < NST; i++) mbar_init(&full[i], 1), mbar_init(&empty[i], wps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // Producer: nothing it reads is written by another kernel.
        if (lane == 0) {
            for (uint32_t i = 0; i < nst; i++) {
                const uint32_t slot = i % NST;
                if (i >= NST && !mbar_wait(&empty[slot], ((i / NST) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                const uint32_t row = r0 + i * rps, here = min(rps, r1 - row);
                const uint32_t bw = here * rb, bs = here * (p.cols / 32);
                mbar_expect_tx(&full[slot], bw + bs);
                bulk_load(raw + Layout::W + slot * STAGE_W, p.w + (size_t)row * rb, bw, &full[slot]);
                bulk_load(raw + Layout::S + slot * STAGE_S, p.ws + (size_t)row * (p.cols / 64), bs, &full[slot]);
            }
            pdl_launch_dependents();
        }
        return;
    }

    // Consumers.  The activations come from the kernel before this one.
    pdl_wait();
    uint4* xlo = reinterpret_cast<uint4*>(raw + Layout::X);
    uint4* xhi = xlo + p.cols / 32;
    float2* xs = reinterpret_cast<float2*>(xhi + p.cols / 32);
    const uint32_t nch = p.cols / 32;
    for (uint32_t i = threadIdx.x; i < nch * 2; i += CTHREADS) {
        const uint4 v = ld_cg_u4(reinterpret_cast<const uint4*>(p.q) + i);
        if (i & 1) xhi[i >> 1] = v;
        else xlo[i >> 1] = v;
    }
    for (uint32_t i = threadIdx.x; i < nch; i += CTHREADS) xs[i] = __ldcg(p.s + i);
    named_bar_sync(1, CTHREADS);
    uint4 ra[NCH > 0 ? NCH : 1], rbb[NCH > 0 ? NCH : 1];
    float2 rs[NCH > 0 ? NCH : 1];
    if constexpr (NCH > 0) {
#pragma unroll
        for (int j = 0; j < NCH; j++) {
            const uint32_t c = lane + 32 * j;
            if (c < nch) ra[j] = xlo[c], rbb[j] = xhi[c], rs[j] = xs[c];
        }
    }

    bool ok = true;
    const uint32_t grp = (uint32_t)warp / wps, wl = (uint32_t)warp % wps;
    for (uint32_t i = grp; i < nst; i += groups) {
        const uint32_t slot = i % NST;
        if (ok && !mbar_wait(&full[slot], (i / NST) & 1)) {
            atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
            ok = false;
        }
        // Two of the warp's rows at a time: each row's sum keeps the reference's order, the two butterflies interleave.
        auto row_sum = [&](uint32_t k) -> float {
            const uint4* wr = reinterpret_cast<const uint4*>(raw + Layout::W + slot * STAGE_W + (size_t)k * rb);
            const __half* sr = reinterpret_cast<const __half*>(raw + Layout::S + slot * STAGE_S) + (size_t)k * (p.cols / 64);
            float sum = 0.0f;
            if constexpr (NCH > 0) {
#pragma unroll
                for (int j = 0; j < NCH; j++) {
                    const uint32_t c = lane + 32 * j;
                    if (c < nch) sum = chunk_step(chunk_dot(wr[c], ra[j], rbb[j]), rs[j], __half2float(sr[c >> 1]), sum);
                }
            } else {
#pragma unroll 2
                for (uint32_t c = lane; c < nch; c += 32) sum = chunk_step(chunk_dot(wr[c], xlo[c], xhi[c]), xs[c], __half2float(sr[c >> 1]), sum);
            }
            return sum;
        };
        for (uint32_t k = wl; k < rps && ok; k += 2 * wps) {
            const uint32_t row = r0 + i * rps + k, k2 = k + wps;
            if (row >= r1) break;
            const bool two = k2 < rps && row + wps < r1;
            float s0 = row_sum(k), s1 = two ? row_sum(k2) : 0.0f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, o));
                s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, o));
            }
            if (lane == 0) {
                p.y[row] = s0;
                if (two) p.y[row + wps] = s1;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
    }
}

// Any other column count (a multiple of 64): one warp per row straight from global memory, the same arithmetic in
// the same order.  The reference's other decode widths (2560, 10240) and its edge shapes take this path.
__global__ void __launch_bounds__(128) gemv_q4_generic(const Q4Params p) {
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * 4 + (threadIdx.x >> 5), nch = p.cols / 32;
    if (row >= p.rows) return;
    const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)row * (p.cols / 2));
    const __half* sr = p.ws + (size_t)row * (p.cols / 64);
    const uint4* xq = reinterpret_cast<const uint4*>(p.q);
    float sum = 0.0f;
    for (uint32_t c = lane; c < nch; c += 32) {
        const uint4 w = __ldcs(wr + c), a = ld_cg_u4(xq + 2 * c), b = ld_cg_u4(xq + 2 * c + 1);
        const float2 sc = __ldcg(p.s + c);
        sum = chunk_step(chunk_dot(w, a, b), sc, __half2float(sr[c >> 1]), sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    if (lane == 0) p.y[row] = sum;
}

// gemv_q4_narrow (ptx/gemv.rs:7-9): rows of at most 256 weights, eight lanes a row (lane l of a row takes chunk l), so a warp
// takes four rows and a block of 128 threads sixteen; the eight sums meet in a butterfly over 4, 2 and 1.
__global__ void __launch_bounds__(128) gemv_q4_narrow_kernel(const Q4Params p) {
    pdl_wait();
    const uint32_t lane = threadIdx.x & 7, row = blockIdx.x * 16 + (threadIdx.x >> 3), nch = p.cols / 32;
    float sum = 0.0f;
    if (row < p.rows && lane < nch) {
        const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)row * (p.cols / 2));
        const uint4* xq = reinterpret_cast<const uint4*>(p.q);
        const uint4 w = __ldcs(wr + lane), a = ld_cg_u4(xq + 2 * lane), b = ld_cg_u4(xq + 2 * lane + 1);
        sum = chunk_step(chunk_dot(w, a, b), __ldcg(p.s + lane), __half2float(p.ws[(size_t)row * (p.cols / 64) + (lane >> 1)]), sum);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    if (lane == 0 && row < p.rows) p.y[row] = sum;
}

}  // namespace

int launch_gemv_q4_narrow(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols) {
    if (!w || !scales || !q || !s || !y) return fail(OUT_OF_RANGE, "gemv_q4_narrow: null argument");
    if (rows == 0 || rows % 4 != 0 || cols == 0 || cols % 64 != 0 || cols > 256) return fail(OUT_OF_RANGE, "gemv_q4_narrow: rows a multiple of 4, columns a multiple of 64 up to 256");
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(q)) & 15) return fail(OUT_OF_RANGE, "gemv_q4_narrow: weights and codes must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(s) & 7) || (reinterpret_cast<uintptr_t>(scales) & 1)) return fail(OUT_OF_RANGE, "gemv_q4_narrow: the pairs must be 8-byte aligned");
    Q4Params p{w, reinterpret_cast<const __half*>(scales), q, reinterpret_cast<const float2*>(s), y, rows, cols};
    TB_CUDA(launch_kernel(ctx, gemv_q4_narrow_kernel, dim3((rows + 15) / 16), dim3(128), 0, true, p));
    return OK;
}

int launch_quant_q8(tb_context* ctx, const float* x, int8_t* q, float* s, uint32_t n) {
    if (!x || !q || !s) return fail(OUT_OF_RANGE, "quant_q8: null argument");
    if (n == 0 || n % 32 != 0) return fail(OUT_OF_RANGE, "quant_q8: the length must be a positive multiple of 32");
    if (reinterpret_cast<uintptr_t>(s) & 7) return fail(OUT_OF_RANGE, "quant_q8: the pairs must be 8-byte aligned");
    TB_CUDA(launch_kernel(ctx, quant_q8_kernel, dim3((n + 255) / 256), dim3(256), 0, true, x, q, reinterpret_cast<float2*>(s), n));
    return OK;
}

int launch_geglu_q8(tb_context* ctx, const float* a, const float* b, int8_t* q, float* s, uint32_t n) {
    if (!a || !b || !q || !s) return fail(OUT_OF_RANGE, "geglu_q8: null argument");
    if (n == 0 || n % 32 != 0) return fail(OUT_OF_RANGE, "geglu_q8: the length must be a positive multiple of 32");
    if (reinterpret_cast<uintptr_t>(s) & 7) return fail(OUT_OF_RANGE, "geglu_q8: the pairs must be 8-byte aligned");
    TB_CUDA(launch_kernel(ctx, geglu_q8_kernel, dim3((n + 255) / 256), dim3(256), 0, true, a, b, q, reinterpret_cast<float2*>(s), n));
    return OK;
}

int launch_norm_q8(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* s, uint32_t len,
                   uint32_t chunks, float eps, float scale) {
    if (!h || chunks == 0) return fail(OUT_OF_RANGE, "norm_q8: null or empty input");
    if (len == 0 || len % 256 != 0 || len > 256 * NORM_PER_THREAD) return fail(OUT_OF_RANGE, "norm_q8: the length must be a multiple of 256 up to 6144");
    if (y && (!w1 || !h_out)) return fail(OUT_OF_RANGE, "norm_q8: a residual needs w1 and h_out");
    if ((q == nullptr) != (s == nullptr) || (reinterpret_cast<uintptr_t>(s) & 7)) return fail(OUT_OF_RANGE, "norm_q8: q and s go together; s 8-byte aligned");
    TB_CUDA(launch_kernel(ctx, norm_q8_kernel, dim3(len / 256, chunks), dim3(256), 0, true, h, h_out, y, w1, w2, q, reinterpret_cast<float2*>(s), len, eps,
                          scale));
    return OK;
}

int launch_embed_q4_rows(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const uint32_t* tokens, uint32_t rows, float* out, uint32_t cols, float scale) {
    if (!w || !scales || !tokens || !out || rows == 0) return fail(OUT_OF_RANGE, "embed_q4: null or empty argument");
    if (cols == 0 || cols % 64 != 0) return fail(OUT_OF_RANGE, "embed_q4: columns must be a positive multiple of 64");
    TB_CUDA(launch_kernel(ctx, embed_q4_rows, dim3((cols + 255) / 256, rows), dim3(256), 0, true, w, reinterpret_cast<const __half*>(scales), tokens, out, cols,
                          scale));
    return OK;
}

int launch_gemv_q4(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols) {
    if (!w || !scales || !q || !s || !y) return fail(OUT_OF_RANGE, "gemv_q4: null argument");
    if (rows == 0 || cols == 0 || cols % 64 != 0) return fail(OUT_OF_RANGE, "gemv_q4: columns must be a positive multiple of 64");
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(q)) & 15)
        return fail(OUT_OF_RANGE, "gemv_q4: weights, scales and codes must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(s) & 7) return fail(OUT_OF_RANGE, "gemv_q4: the pairs must be 8-byte aligned");
    Q4Params p{w, reinterpret_cast<const __half*>(scales), q, reinterpret_cast<const float2*>(s), y, rows, cols};
    // The staged kernel wants whole rows in a stage, stages going round whole groups of warps, and a row's scales
    // (cols / 32 bytes) copied in 16-byte units: a power of two from 512 to 16384 columns.
    if (cols < 512 || cols > 16384 || STAGE_W % (cols / 2) != 0) {
        TB_CUDA(launch_kernel(ctx, gemv_q4_generic, dim3((rows + 3) / 4), dim3(128), 0, true, p));
        return OK;
    }
    const size_t smem = smem_bytes(cols);
    static size_t configured[16] = {};
    if (configured[ctx->gpu & 15] < smem) {
        TB_CUDA(cudaFuncSetAttribute(gemv_q4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(16384)));
        TB_CUDA(cudaFuncSetAttribute(gemv_q4_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(16384)));
        TB_CUDA(cudaFuncSetAttribute(gemv_q4_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(16384)));
        TB_CUDA(cudaFuncSetAttribute(gemv_q4_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(16384)));
        configured[ctx->gpu & 15] = smem_bytes(16384);
    }
    const uint32_t rps = STAGE_W / (cols / 2);
    const uint32_t grid = std::min<uint32_t>((uint32_t)ctx->sms, (rows + rps - 1) / rps);
    if (cols <= 1024) TB_CUDA(launch_kernel(ctx, gemv_q4_kernel<1>, dim3(grid), dim3(THREADS), smem, true, p, ctx->status));
    else if (cols == 2048) TB_CUDA(launch_kernel(ctx, gemv_q4_kernel<2>, dim3(grid), dim3(THREADS), smem, true, p, ctx->status));
    else if (cols == 4096) TB_CUDA(launch_kernel(ctx, gemv_q4_kernel<4>, dim3(grid), dim3(THREADS), smem, true, p, ctx->status));
    else TB_CUDA(launch_kernel(ctx, gemv_q4_kernel<0>, dim3(grid), dim3(THREADS), smem, true, p, ctx->status));
    return OK;
}

}  // namespace tb
