// The reference's prefill formats, by the reference's kernel names, for a caller that drives its own prefill op list
// (crates/tachyon/src/model/prefill.rs:144-196) through tb_launch:
//
//   quant_q8p_kernel  = quant_q8p   (crates/tachyon/src/ptx/mod.rs:217-287): f32 -> Q8P, blocks of 64, pairs [s, z]
//   geglu_q8p_kernel  = geglu_q8p   (ptx/mod.rs:253-307): gelu(a) * b over strided rows, then Q8P
//   norm_q8p_kernel   = norm_q8p    (ptx/mod.rs:404-511 with the Q8P store): the residual / RMS-norm step per token
//   gemm_q4_kernel    = gemm_q4     (ptx/gemm.rs:1-23, 177-205): Q4 weights x Q8P activations -> f32, split over column slices
//   sum_slices_kernel = sum_slices  (ptx/gemm.rs:287-325): the slices added up in order
//
// Q8P (crates/tachyon/src/quant.rs:32, 102-105): per 64 values s = amax / 127, codes rounded to nearest even, and
// z = -8 s sum(q) - MAGIC s with MAGIC = 1.5 * 2^23, so that the product's integer sum i, read as the float MAGIC + i, turns
// into s * sum((n - 8) q) with one fma.  The quantisers repeat the reference's f32 operations in its order (div.rn, mul.rn,
// cvt.rni, fma.rn), so their bytes are the reference's.  The product repeats its per-group arithmetic (integer sums of 64,
// fma(i, s, z), fma(f, d, c), groups in rising order within a slice, ptx/gemm.rs:199-201) on dp4a instead of mma.sync: the
// same sums in the same order, hence the same bits, at the speed of a plain CUDA-core kernel.  The fast prefill product of
// this library is tb_gemm_q4 / tb_gemm_q8 (gemm.cu, tcgen05 on f16 operands); this one exists so that the reference's own op
// list has every name it launches.
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

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

// ptx/mod.rs:217-249: value x of element i as Q8P.  A block of 64 values is two consecutive warps of the thread block, which
// trade their maxima and their sums through shared memory (slot w ^ 1 is the partner's).  Every thread of the block calls
// this (it holds two block barriers); threads with valid == false store nothing.
__device__ __forceinline__ void store_q8p(float x, uint32_t i, bool valid, int8_t* q, float2* s, float* trade) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float amax = warp_max(fabsf(x));
    if (lane == 0) trade[warp] = amax;
    __syncthreads();
    amax = fmaxf(amax, trade[warp ^ 1]);
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int code = __float2int_rn(__fmul_rn(x, inv));
    if (valid) q[i] = static_cast<int8_t>(code);
    int sum = code;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    int* trade_i = reinterpret_cast<int*>(trade) + 16;
    if (lane == 0) trade_i[warp] = sum;
    __syncthreads();
    sum += trade_i[warp ^ 1];
    if ((i & 63u) == 0 && valid) {
        float f = __fmul_rn(static_cast<float>(sum), d);
        f = __fmul_rn(f, -8.0f);
        s[i >> 6] = make_float2(d, __fmaf_rn(d, -12582912.0f, f));
    }
}

__global__ void __launch_bounds__(256) quant_q8p_kernel(const float* __restrict__ x, int8_t* q, float2* s, uint32_t len) {
    __shared__ float trade[32];
    pdl_wait();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    const bool in = i < len;
    store_q8p(in ? x[i] : 0.0f, i, in, q, s, trade);
}

// Value i is row t = i / width, column j: reads a[t sa + j] and b[t sb + j], is stored as value t so + j (ptx/mod.rs:289-307).
__global__ void __launch_bounds__(256) geglu_q8p_kernel(const float* __restrict__ a, const float* __restrict__ b, int8_t* q, float2* s, uint32_t len,
                                                        uint32_t width, uint32_t sa, uint32_t sb, uint32_t so) {
    __shared__ float trade[32];
    pdl_wait();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    const bool in = i < len;
    const uint32_t t = i / width, j = i % width;
    float x = in ? a[(size_t)t * sa + j] : 0.0f;
    const float y = in ? b[(size_t)t * sb + j] : 0.0f;
    // gelu(x) * y as the reference's decoder computes it (ptx/mod.rs:376-390), operation by operation
    float u = __fmul_rn(x, x);
    u = __fmaf_rn(u, 0.044714998453855514526f, 1.0f);
    u = __fmul_rn(u, x);
    u = __fmul_rn(u, -2.3022081851959228516f);
    u = __fadd_rn(ex2_approx(u), 1.0f);
    x = __fmul_rn(__fdiv_rn(x, u), y);
    store_q8p(x, t * so + j, in, q, s, trade);
}

// Sums of four values over the block of eight warps, in every thread, in the order of the reference's block()
// (ptx/mod.rs:153-170); the same helper as norm_q8_kernel's in q4.cu.
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

// norm_q8 with the Q8P store: grid (len / 256, tokens); see norm_q8_kernel in q4.cu for the arithmetic (ptx/mod.rs:404-511).
constexpr int NORM_PER_THREAD = 24;
__global__ void __launch_bounds__(256) norm_q8p_kernel(const float* __restrict__ h, float* h_out, const float* __restrict__ y, const float* __restrict__ w1,
                                                       const float* __restrict__ w2, int8_t* q, float2* s, uint32_t len, float eps, float scale) {
    __shared__ float red[128];
    __shared__ float trade[32];
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
    if (q == nullptr) return;  // the same for every thread of the block
    r = rsqrt_approx(__fadd_rn(__fdiv_rn(sh, n), eps));
    if (w2 == nullptr) r = 1.0f;
    float x = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_PER_THREAD; k++)
        if (slice == (uint32_t)k) x = hv[k];
    x = __fmul_rn(x, r);
    x = __fmul_rn(x, w2 != nullptr ? w2[own] : 1.0f);
    store_q8p(x, base + own, true, q, s, trade);
}

// gemm_q4: a block of 16 x 16 threads computes 16 tokens x 16 rows, thread (ty, tx) token T + ty, row R + tx, over the
// groups of 64 columns of its slice, staged in shared memory group by group (16 tokens x 64 codes + pairs, 16 rows x 32 bytes
// + scales).  Per group: i = sum over 64 of nibble * code (exact), f = fma(float(MAGIC + i), s, z), c = fma(f, d, c).
constexpr int GT = 16;
__global__ void __launch_bounds__(GT* GT) gemm_q4_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ ws, const int8_t* __restrict__ q,
                                                         const float2* __restrict__ s, float* y, uint32_t rows, uint32_t cols, uint32_t tokens) {
    __shared__ __align__(16) uint8_t sq[GT][64 + 16];  // padded rows: sixteen threads read sixteen different rows at once
    __shared__ __align__(16) uint8_t sw[GT][32 + 16];
    __shared__ float2 sp[GT];
    __shared__ float sd[GT];
    pdl_wait();
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4, tid = threadIdx.x;
    const uint32_t T = blockIdx.x * GT, R = blockIdx.y * GT;
    // The slice's columns in turns of 128, as the reference splits them (ptx/gemm.rs:142-150).
    const uint32_t turns = cols >> 7, z = blockIdx.z, Z = gridDim.z;
    const uint32_t g0 = 2 * (turns * z / Z), g1 = 2 * ((turns * z + turns) / Z), groups = cols >> 6;
    float c = 0.0f;
    for (uint32_t g = g0; g < g1; g++) {
        __syncthreads();
        {
            // 16 tokens x 64 bytes = 64 pieces of 16 bytes; 16 rows x 32 bytes = 32 pieces: threads 0..63 and 64..95
            if (tid < 64) {
                const uint32_t t = tid >> 2, piece = tid & 3;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                // the Q8P buffer holds whole tiles of 128 tokens (ptx/gemm.rs:19-20): rows past `tokens` are there and may be read
                v = *reinterpret_cast<const uint4*>(q + (size_t)(T + t) * cols + (size_t)g * 64 + piece * 16);
                *reinterpret_cast<uint4*>(&sq[t][piece * 16]) = v;
            } else if (tid < 96) {
                const uint32_t r = (tid - 64) >> 1, piece = tid & 1;
                *reinterpret_cast<uint4*>(&sw[r][piece * 16]) = *reinterpret_cast<const uint4*>(w + ((size_t)(R + r) * groups + g) * 32 + piece * 16);
            } else if (tid < 112) {
                sp[tid - 96] = s[(size_t)(T + tid - 96) * groups + g];
            } else if (tid < 128) {
                sd[tid - 112] = __half2float(ws[(size_t)(R + tid - 112) * groups + g]);
            }
        }
        __syncthreads();
        int isum = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t word = *reinterpret_cast<const uint32_t*>(&sw[tx][4 * k]);
            const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;  // weights 8k .. 8k+3 and 8k+4 .. 8k+7 (quant.rs:60-66)
            isum = dp4a_su(*reinterpret_cast<const uint32_t*>(&sq[ty][8 * k]), lo, isum);
            isum = dp4a_su(*reinterpret_cast<const uint32_t*>(&sq[ty][8 * k + 4]), hi, isum);
        }
        const float2 pz = sp[ty];
        const float f = __fmaf_rn(__int_as_float(0x4B400000 + isum), pz.x, pz.y);
        c = __fmaf_rn(f, sd[tx], c);
    }
    if (T + ty < tokens) y[(size_t)z * tokens * rows + (size_t)(T + ty) * rows + R + tx] = c;
}

__global__ void __launch_bounds__(256) sum_slices_kernel(float* y, uint32_t len, uint32_t slices) {
    pdl_wait();
    const uint32_t i = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (i >= len) return;
    float4 a = *reinterpret_cast<const float4*>(y + i);
    for (uint32_t z = 1; z < slices; z++) {
        const float4 b = *reinterpret_cast<const float4*>(y + (size_t)z * len + i);
        a.x = __fadd_rn(a.x, b.x), a.y = __fadd_rn(a.y, b.y), a.z = __fadd_rn(a.z, b.z), a.w = __fadd_rn(a.w, b.w);
    }
    *reinterpret_cast<float4*>(y + i) = a;
}

}  // namespace

int launch_quant_q8p(tb_context* ctx, const float* x, int8_t* q, float* s, uint32_t len) {
    if (!x || !q || !s || len == 0) return fail(OUT_OF_RANGE, "quant_q8p: null or empty argument");
    TB_CUDA(launch_kernel(ctx, quant_q8p_kernel, dim3((len + 255) / 256), dim3(256), 0, true, x, q, reinterpret_cast<float2*>(s), len));
    return OK;
}

int launch_geglu_q8p(tb_context* ctx, const float* a, const float* b, int8_t* q, float* s, uint32_t len, uint32_t width, uint32_t sa, uint32_t sb, uint32_t so) {
    if (!a || !b || !q || !s || len == 0 || width == 0 || width % 64 != 0 || so % 64 != 0) return fail(OUT_OF_RANGE, "geglu_q8p: null argument, or rows that are not whole blocks of 64");
    TB_CUDA(launch_kernel(ctx, geglu_q8p_kernel, dim3((len + 255) / 256), dim3(256), 0, true, a, b, q, reinterpret_cast<float2*>(s), len, width, sa, sb, so));
    return OK;
}

int launch_norm_q8p(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* s, uint32_t len,
                    uint32_t tokens, float eps, float scale) {
    if (!h || len == 0 || len % 256 != 0 || len > 256 * NORM_PER_THREAD || tokens == 0 || tokens > 65535) return fail(OUT_OF_RANGE, "norm_q8p: len must be a multiple of 256 up to 6144, tokens 1..65535");
    if (y != nullptr && (!w1 || !h_out)) return fail(OUT_OF_RANGE, "norm_q8p: the residual needs w1 and h_out");
    if ((q == nullptr) != (s == nullptr)) return fail(OUT_OF_RANGE, "norm_q8p: q and s go together");
    TB_CUDA(launch_kernel(ctx, norm_q8p_kernel, dim3(len / 256, tokens), dim3(256), 0, true, h, h_out, y, w1, w2, q, reinterpret_cast<float2*>(s), len, eps, scale));
    return OK;
}

int launch_gemm_q4_ref(tb_context* ctx, const uint8_t* w, const uint16_t* ws, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols,
                       uint32_t tokens, uint32_t slices) {
    if (!w || !ws || !q || !s || !y) return fail(OUT_OF_RANGE, "gemm_q4: null argument");
    if (rows == 0 || rows % 64 != 0 || cols == 0 || cols % 128 != 0 || tokens == 0) return fail(OUT_OF_RANGE, "gemm_q4: rows a multiple of 64, cols of 128 (ptx/gemm.rs:18-20)");
    if (slices == 0 || slices > 8 || slices > cols / 128) return fail(OUT_OF_RANGE, "gemm_q4: 1..8 slices, at most one per 128 columns");
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(q)) & 15) return fail(OUT_OF_RANGE, "gemm_q4: weights and codes must be 16-byte aligned");
    const dim3 grid((tokens + GT - 1) / GT, rows / GT, slices);
    TB_CUDA(launch_kernel(ctx, gemm_q4_kernel, grid, dim3(GT * GT), 0, true, w, reinterpret_cast<const __half*>(ws), q, reinterpret_cast<const float2*>(s), y, rows, cols,
                          tokens));
    return OK;
}

int launch_sum_slices(tb_context* ctx, float* y, uint32_t len, uint32_t slices) {
    if (!y || len == 0 || len % 4 != 0 || slices == 0) return fail(OUT_OF_RANGE, "sum_slices: len a multiple of 4, at least one slice");
    if (reinterpret_cast<uintptr_t>(y) & 15) return fail(OUT_OF_RANGE, "sum_slices: y must be 16-byte aligned");
    TB_CUDA(launch_kernel(ctx, sum_slices_kernel, dim3((len + 1023) / 1024), dim3(256), 0, true, y, len, slices));
    return OK;
}

}  // namespace tb
