// The encoder's small kernels under the reference's names and argument lists (crates/tachyon/src/ptx/encoder.rs:5-38), for a
// caller that drives the encoder launch by launch: quant_f16 (670-743), norm_f16 (580-668), rope_f16 (893-959), embed_f16 /
// gather_rows / add_rows / add_rows_f16 (761-805), gelu_f16 (843-891) and the 8-bit product gemm_q8 on Q8E activations
// (315-375).  Where the reference's arithmetic is a fixed sequence of IEEE operations (quant_f16, rope_f16, the 8-bit
// product's sums) the kernels here follow it operation by operation, so their results have the same bits.
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

// ---- quant_f16: a warp per group of 64 values, two a lane ---------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_f16_kernel(const __half* a, int8_t* q, float* s, uint32_t cols) {
    const uint32_t lane = threadIdx.x & 31, g = blockIdx.x * 8 + (threadIdx.x >> 5), groups = cols >> 6;
    if (g >= groups) return;
    const size_t at = (size_t)blockIdx.y * cols + g * 64 + lane * 2;
    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(a + at));
    float m = fmaxf(fabsf(x.x), fabsf(x.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float inv = m == 0.0f ? 0.0f : __fdiv_rn(127.0f, m);
    const int q0 = __float2int_rn(__fmul_rn(x.x, inv)), q1 = __float2int_rn(__fmul_rn(x.y, inv));
    *reinterpret_cast<uint16_t*>(q + at) = (uint16_t)((q0 & 255) | ((q1 & 255) << 8));
    if (lane == 0) s[(size_t)blockIdx.y * groups + g] = __fdiv_rn(m, 127.0f);
}

// ---- norm_f16: a block per row ------------------------------------------------------------------------------------------
// gamma * (x - mean) / sqrt(var + eps) (+ beta) to a (f16) and, unless null, to xo (f32, may be x).  Two passes over the row
// held in registers (the reference sums the values less the row's first and their squares in one pass: the same quantity).
__global__ void __launch_bounds__(256) norm_f16_kernel(const float* x, const float* gamma, const float* beta, __half* a, float* xo, uint32_t h, float eps) {
    __shared__ float sh[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t row = (size_t)blockIdx.x * h;
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
    float4 v[4];  // h <= 4096
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t c = (i * 256 + tid) * 4;
        v[i] = c < h ? *reinterpret_cast<const float4*>(x + row + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = block_sum(sum) / (float)h;
    float var = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t c = (i * 256 + tid) * 4;
        if (c < h) {
            v[i].x -= mean, v[i].y -= mean, v[i].z -= mean, v[i].w -= mean;
            var = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, var))));
        }
    }
    const float r = 1.0f / sqrtf(block_sum(var) / (float)h + eps);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t c = (i * 256 + tid) * 4;
        if (c >= h) continue;
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + c));
        const float4 b = beta != nullptr ? __ldg(reinterpret_cast<const float4*>(beta + c)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float4 y = make_float4(fmaf(v[i].x * r, g.x, b.x), fmaf(v[i].y * r, g.y, b.y), fmaf(v[i].z * r, g.z, b.z), fmaf(v[i].w * r, g.w, b.w));
        if (xo != nullptr) *reinterpret_cast<float4*>(xo + row + c) = y;
        const __half2 lo = __floats2half2_rn(y.x, y.y), hi = __floats2half2_rn(y.z, y.w);
        *reinterpret_cast<uint2*>(a + row + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

// ---- embed_f16 / add_rows / add_rows_f16 / gather_rows: out[r] (f32 [n, h]) from row idx[r] of a table --------------------
template <bool HALF, bool ADD>
__global__ void __launch_bounds__(256) rows_kernel(const void* table, const uint32_t* idx, float* out, uint32_t h) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x, r = blockIdx.y;
    if (i >= h) return;
    const size_t src = (size_t)idx[r] * h + i, dst = (size_t)r * h + i;
    float v = HALF ? __half2float(static_cast<const __half*>(table)[src]) : static_cast<const float*>(table)[src];
    if (ADD) v += out[dst];
    out[dst] = v;
}

// ---- gelu_f16: gelu(a) * b to f16, from rows [a, b] (gated) or rows of a -----------------------------------------------------
__global__ void __launch_bounds__(256) gelu_f16_kernel(const float* x, __half* out, uint32_t width, uint32_t len, uint32_t gated) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= len) return;
    const uint32_t row = i / width, col = i % width;
    const float* p = x + (size_t)row * (gated ? 2 * width : width) + col;
    out[i] = __float2half_rn(gelu_erf(p[0]) * (gated ? p[width] : 1.0f));
}

// ---- rope_f16: one pair of a query and of a key per thread ------------------------------------------------------------------
// (a, b) = (v[j], v[j + d/2]) of a head become (a c - b s, b c + a s), (c, s) = table[pos][j]: a product then one fused
// multiply-add each, as the reference's (ptx/encoder.rs:942-956).
__global__ void __launch_bounds__(256) rope_f16_kernel(__half* qkv, const float2* table, const uint32_t* pos, uint32_t h, uint32_t d) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x, half_d = d / 2;
    if (i >= h / 2) return;
    const uint32_t tok = blockIdx.y, head = i / half_d, j = i % half_d;
    const float2 cs = __ldg(table + (size_t)pos[tok] * half_d + j);
    __half* q = qkv + (size_t)tok * 3 * h + head * d + j;
#pragma unroll
    for (int part = 0; part < 2; part++, q += h) {
        const float a = __half2float(q[0]), b = __half2float(q[half_d]);
        q[0] = __float2half_rn(__fmaf_rn(b, -cs.y, __fmul_rn(a, cs.x)));
        q[half_d] = __float2half_rn(__fmaf_rn(a, cs.y, __fmul_rn(b, cs.x)));
    }
}

// ---- gemm_q8: Q8E activations x Q8E weights -----------------------------------------------------------------------------------
// y[t, r] = sum over groups of 64 of (integer sum) * sa[t, g] * sw[r, g], each group as the reference's two fused
// multiply-adds on the sum read as the float 12582912 + i (ptx/encoder.rs:354-375): f = fma(M + i, sa, -M sa),
// c = fma(f, sw, c).  A block of 16 x 16 threads takes 64 tokens x 64 rows; thread (ty, tx) holds tokens ty + 16 a and rows
// tx + 16 b.  Rows of a tile sit 68 bytes apart in shared memory, so the sixteen rows a half-warp reads fall in sixteen banks.
constexpr int QT8 = 64, QLD = 17;  // tile edge; words a shared row

__device__ __forceinline__ float act_pair(float gate, float up, uint32_t mode) {
    const float g = mode == 4 ? gelu_erf(gate) : gate / (1.0f + exp2f(-1.4426950408889634f * gate));
    return g * up;
}

__global__ void __launch_bounds__(256) gemm_q8e_kernel(const int8_t* a, const int8_t* w, const float* bias, void* y, uint32_t rows, uint32_t cols, uint32_t tokens,
                                                       uint32_t mode, const float* sa, const float* sw) {
    __shared__ uint32_t as[QT8 * QLD], ws[QT8 * QLD];
    __shared__ float ssa[QT8], ssw[QT8];
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4, groups = cols >> 6;
    const uint32_t t0 = blockIdx.x * QT8, r0 = blockIdx.y * QT8;
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) c[i][j] = 0.0f;
    for (uint32_t g = 0; g < groups; g++) {
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {  // 64 rows of 16 words either tile: a thread copies four words of each
            const uint32_t e = k * 256 + tid, r = e >> 4, kw = e & 15;
            as[r * QLD + kw] = t0 + r < tokens ? *reinterpret_cast<const uint32_t*>(a + ((size_t)(t0 + r) * cols + g * 64 + kw * 4)) : 0u;
            ws[r * QLD + kw] = *reinterpret_cast<const uint32_t*>(w + ((size_t)(r0 + r) * cols + g * 64 + kw * 4));
        }
        if (tid < QT8) ssa[tid] = t0 + tid < tokens ? sa[(size_t)(t0 + tid) * groups + g] : 0.0f;
        else if (tid < 2 * QT8) ssw[tid - QT8] = sw[(size_t)(r0 + tid - QT8) * groups + g];
        __syncthreads();
        int isum[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) isum[i][j] = 0;
#pragma unroll
        for (int kw = 0; kw < 16; kw++) {
            uint32_t av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = as[(ty + 16 * i) * QLD + kw], wv[i] = ws[(tx + 16 * i) * QLD + kw];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) isum[i][j] = __dp4a((int)av[i], (int)wv[j], isum[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float ts = ssa[ty + 16 * i], tz = __fmul_rn(ts, -12582912.0f);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float f = __fmaf_rn(__int_as_float(0x4B400000 + isum[i][j]), ts, tz);
                c[i][j] = __fmaf_rn(f, ssw[tx + 16 * j], c[i][j]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t t = t0 + ty + 16 * i;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t r = r0 + tx + 16 * j;
            float v = c[i][j] + (bias != nullptr ? __ldg(bias + r) : 0.0f);
            const float other = __shfl_xor_sync(0xffffffffu, v, 1);  // the row beside it: lanes tx and tx ^ 1
            if (t >= tokens) continue;
            const size_t at = (size_t)t * rows + r;
            if (mode == 0) static_cast<float*>(y)[at] = v;
            else if (mode == 1) static_cast<float*>(y)[at] += v;
            else if (mode == 2) static_cast<__half*>(y)[at] = __float2half_rn(v);
            else if (mode == 3) static_cast<__half*>(y)[at] = __float2half_rn(fmaxf(v, 0.0f));
            else if ((tx & 1) == 0) static_cast<__half*>(y)[(size_t)t * (rows / 2) + r / 2] = __float2half_rn(act_pair(v, other, mode));
        }
    }
}

}  // namespace

int launch_quant_f16(tb_context* ctx, const __half* a, int8_t* q, float* s, uint32_t cols, uint32_t tokens) {
    if (!a || !q || !s || cols == 0 || cols % 64 != 0 || tokens == 0) return fail(OUT_OF_RANGE, "quant_f16: null or empty argument, or rows not whole groups of 64");
    TB_CUDA(launch_kernel(ctx, quant_f16_kernel, dim3((cols / 64 + 7) / 8, tokens), dim3(256), 0, false, a, q, s, cols));
    return OK;
}

int launch_norm_f16(tb_context* ctx, const float* x, const float* gamma, const float* beta, __half* a, float* xo, uint32_t h, float eps, uint32_t n) {
    if (!x || !gamma || !a || n == 0) return fail(OUT_OF_RANGE, "norm_f16: null or empty argument");
    if (h == 0 || h % 4 != 0 || h > 4096) return fail(OUT_OF_RANGE, "norm_f16: rows of a multiple of 4 values, at most 4096");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(xo)) & 15 ||
        (reinterpret_cast<uintptr_t>(a) & 7))
        return fail(OUT_OF_RANGE, "norm_f16: buffers must be 16-byte aligned");
    TB_CUDA(launch_kernel(ctx, norm_f16_kernel, dim3(n), dim3(256), 0, false, x, gamma, beta, a, xo, h, eps));
    return OK;
}

int launch_rows(tb_context* ctx, int kind, const void* table, const uint32_t* idx, float* out, uint32_t h, uint32_t n) {
    if (!table || !idx || !out || h == 0 || n == 0) return fail(OUT_OF_RANGE, "row kernels: null or empty argument");
    const dim3 grid((h + 255) / 256, n);
    cudaError_t e;
    switch (kind) {
        case 0: e = launch_kernel(ctx, rows_kernel<true, false>, grid, dim3(256), 0, false, table, idx, out, h); break;   // embed_f16
        case 1: e = launch_kernel(ctx, rows_kernel<false, true>, grid, dim3(256), 0, false, table, idx, out, h); break;   // add_rows
        case 2: e = launch_kernel(ctx, rows_kernel<true, true>, grid, dim3(256), 0, false, table, idx, out, h); break;    // add_rows_f16
        default: e = launch_kernel(ctx, rows_kernel<false, false>, grid, dim3(256), 0, false, table, idx, out, h); break; // gather_rows
    }
    TB_CUDA(e);
    return OK;
}

int launch_gelu_f16(tb_context* ctx, const float* x, __half* out, uint32_t width, uint32_t len, uint32_t gated) {
    if (!x || !out || width == 0 || len == 0 || len % width != 0) return fail(OUT_OF_RANGE, "gelu_f16: null or empty argument, or a ragged length");
    TB_CUDA(launch_kernel(ctx, gelu_f16_kernel, dim3((len + 255) / 256), dim3(256), 0, false, x, out, width, len, gated));
    return OK;
}

int launch_rope_f16(tb_context* ctx, __half* qkv, const float* table, const uint32_t* pos, uint32_t h, uint32_t d, uint32_t n) {
    if (!qkv || !table || !pos || n == 0 || d == 0 || d % 2 != 0 || h == 0 || h % d != 0) return fail(OUT_OF_RANGE, "rope_f16: null or empty argument, or a ragged shape");
    if (reinterpret_cast<uintptr_t>(table) & 7) return fail(OUT_OF_RANGE, "rope_f16: the table must be 8-byte aligned");
    TB_CUDA(launch_kernel(ctx, rope_f16_kernel, dim3((h / 2 + 255) / 256, n), dim3(256), 0, false, qkv, reinterpret_cast<const float2*>(table), pos, h, d));
    return OK;
}

int launch_gemm_q8e(tb_context* ctx, const int8_t* a, const int8_t* w, const float* bias, void* y, uint32_t rows, uint32_t cols, uint32_t tokens, uint32_t mode,
                    const float* sa, const float* sw) {
    if (!a || !w || !y || !sa || !sw || tokens == 0) return fail(OUT_OF_RANGE, "gemm_q8: null or empty argument");
    if (rows == 0 || rows % 64 != 0 || cols == 0 || cols % 64 != 0) return fail(OUT_OF_RANGE, "gemm_q8: rows and cols must be multiples of 64");
    if (mode > 5) return fail(OUT_OF_RANGE, "gemm_q8: modes 0 to 5");
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 3) return fail(OUT_OF_RANGE, "gemm_q8: codes must be 4-byte aligned");
    TB_CUDA(launch_kernel(ctx, gemm_q8e_kernel, dim3((tokens + QT8 - 1) / QT8, rows / QT8), dim3(256), 0, false, a, w, bias, y, rows, cols, tokens, mode, sa, sw));
    return OK;
}

}  // namespace tb
