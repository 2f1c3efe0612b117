// The small kernels around the matrix-vector products: embedding-row dequantisation, a stand-alone residual/RMS-norm
// step, the stand-alone greedy sampler and top-k, seeded fills for synthetic models, and the row interleave applied to
// gate/up matrices when a model is loaded.
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

// Dequantises row *token of a Q8 table, times `scale`.  Replaces embed_q4 (crates/tachyon/src/ptx/mod.rs:531-598) for
// this build's Q8 tables.  It triggers its dependents only by finishing, which keeps the chain of early-starting
// kernels behind it ordered after the sampler that wrote the token.
__global__ void __launch_bounds__(256) embed_q8_kernel(const int8_t* w, const __half* s, const uint32_t* token, uint32_t cols, float scale, float* out) {
    pdl_wait();
    const size_t row = (size_t)ld_cg_u(token) * cols;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < cols; i += gridDim.x * blockDim.x)
        out[i] = (float)w[row + i] * __half2float(s[(row + i) / 32]) * scale;
}

// The reference's embed_q4 itself (ptx/mod.rs:531-598): weight k of a group of 64 is nibble k % 8 / 4 of byte
// k / 8 * 4 + k % 4 (quant.rs:60-66), minus 8, times the group's scale.
__global__ void __launch_bounds__(256) embed_q4_kernel(const uint8_t* w, const __half* s, const uint32_t* token, uint32_t cols, float scale, float* out) {
    pdl_wait();
    const size_t row = (size_t)ld_cg_u(token) * cols;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < cols; i += gridDim.x * blockDim.x) {
        const size_t at = row + i, g = at / 64, k = at % 64;
        const int n = (w[g * 32 + k / 8 * 4 + k % 4] >> (k % 8 / 4 * 4)) & 15;
        out[i] = (float)(n - 8) * __half2float(s[g]) * scale;
    }
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (uint32_t i = 0; i < blockDim.x / 32; i++) t += sh[i];
    return t;
}

// h' = (h + w1 * rmsnorm(y)) * hscale when y is given, else h; x = w2 * rmsnorm(h') (or h' without w2).  The stand-alone
// form of the reference's norm_q8 (ptx/mod.rs:404-511) without its Q8 output; the decode step uses the same arithmetic
// as the prologue of the matrix-vector kernel.
__global__ void __launch_bounds__(1024) norm_kernel(const float* h, const float* y, const float* w1, const float* w2, uint32_t n, float eps, float hscale,
                                                    float* h_out, float* x_out) {
    __shared__ float sh[32];
    pdl_wait();
    float sy = 0.0f;
    if (y != nullptr) {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) sy = fmaf(y[i], y[i], sy);
        sy = block_sum(sy, sh);
    }
    const float ry = y != nullptr ? rsqrtf(sy / (float)n + eps) : 0.0f;
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = y != nullptr ? fmaf(y[i] * ry, w1[i], h[i]) * hscale : h[i];
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, sh);
    const float rh = w2 != nullptr ? rsqrtf(sq / (float)n + eps) : 1.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = y != nullptr ? fmaf(y[i] * ry, w1[i], h[i]) * hscale : h[i];
        if (h_out != nullptr) h_out[i] = v;
        if (x_out != nullptr) x_out[i] = w2 != nullptr ? v * rh * w2[i] : v;
    }
}

// The sampler's transform (crates/tachyon/src/ptx/sample.rs:1-27): soft cap, allowed mask, repetition penalty.
__device__ __forceinline__ float transform(float x, uint32_t i, float softcap, float penalty, const uint32_t* seen, const uint32_t* allowed) {
    if (softcap > 0.0f) x = softcap * tanhf(x / softcap);
    if (allowed != nullptr && !((allowed[i >> 5] >> (i & 31)) & 1u)) return -INFINITY;
    if (seen != nullptr && ((seen[i >> 5] >> (i & 31)) & 1u)) x = x > 0.0f ? x / penalty : x * penalty;
    return x;
}

// Greedy pick over transformed logits: largest value, lowest index among equals.  Blocks publish a 64-bit key (value
// order, inverted index) with atomicMax; the last block to finish writes the token and clears the scratch.
__global__ void __launch_bounds__(1024) sample_greedy_kernel(const float* logits, uint32_t vocab, float softcap, float penalty, const uint32_t* seen,
                                                             const uint32_t* allowed, unsigned long long* best, uint32_t* count, uint32_t* state,
                                                             uint32_t* seen_out, uint32_t* token_out) {
    __shared__ unsigned long long sh[32];
    pdl_wait();
    unsigned long long key = 0;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float v = transform(__ldcg(logits + i), i, softcap, penalty, seen, allowed);
        const unsigned long long k = ((unsigned long long)float_key(v) << 32) | (0xffffffffu - i);
        key = k > key ? k : key;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = key;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t i = 1; i < blockDim.x / 32; i++) key = sh[i] > key ? sh[i] : key;
        atomicMax(best, key);
        __threadfence();
        if (atomicAdd(count, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long top = atomicExch(best, 0ull);
            const uint32_t token = 0xffffffffu - (uint32_t)top;
            state[1] = token;
            state[0] = state[0] + 1;
            if (seen_out != nullptr) atomicOr(seen_out + (token >> 5), 1u << (token & 31));
            if (token_out != nullptr) *token_out = token;
            *count = 0;
        }
    }
}

// The k largest logits, largest first, lowest index first among equals: one block, k passes, each taking the largest
// key below the previous pick.  scratch: one 64-bit word.
__global__ void __launch_bounds__(1024) topk_kernel(const float* logits, uint32_t vocab, uint32_t k, uint32_t* idx, float* val) {
    __shared__ unsigned long long sh[32];
    __shared__ unsigned long long limit;
    pdl_wait();
    if (threadIdx.x == 0) limit = ~0ull;
    __syncthreads();
    for (uint32_t round = 0; round < k; round++) {
        const unsigned long long lim = limit;
        unsigned long long key = 0;
        for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned long long c = ((unsigned long long)float_key(__ldcg(logits + i)) << 32) | (0xffffffffu - i);
            if (c < lim && c > key) key = c;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
            key = other > key ? other : key;
        }
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = key;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint32_t i = 1; i < blockDim.x / 32; i++) key = sh[i] > key ? sh[i] : key;
            const uint32_t at = 0xffffffffu - (uint32_t)key;
            idx[round] = at;
            val[round] = at < vocab ? logits[at] : -INFINITY;
            limit = key;
        }
        __syncthreads();
    }
}

// Seeded fills.  The hash and every arithmetic step match the CPU generator bit for bit: only integer operations,
// exactly representable conversions and single correctly-rounded float operations.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ unsigned long long draw(unsigned long long base, unsigned long long i) { return mix64(base + i); }
__device__ __forceinline__ float gauss(unsigned long long base, unsigned long long i) {
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const unsigned long long h = draw(base, 3 * i + j);
        sum += (uint32_t)(h & 0xffff) + (uint32_t)((h >> 16) & 0xffff) + (uint32_t)((h >> 32) & 0xffff) + (uint32_t)(h >> 48);
    }
    return __fmul_rn(__fsub_rn((float)sum, 393210.0f), 1.0f / 65536.0f);
}

__global__ void fill_codes_kernel(unsigned long long base, int8_t* w, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = (int8_t)((int)(draw(base, i) % 255ull) - 127);
}
__global__ void fill_scales_kernel(unsigned long long base, __half* s, size_t n, float mul) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        s[i] = __float2half_rn(__fmul_rn(fabsf(gauss(base, i)), mul));
}
__global__ void fill_gauss_f16_kernel(unsigned long long base, __half* x, size_t n, float mul) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __float2half_rn(__fmul_rn(gauss(base, i), mul));
}
__global__ void fill_uniform_kernel(unsigned long long base, float* x, size_t n, float lo, float step) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __fmaf_rn((float)(draw(base, i) & 0xffff), step, lo);
}

// dst row 2j = src row j, dst row 2j+1 = src row half_rows + j: gate and up rows side by side, so that one block of the
// matrix-vector kernel holds both halves of a GeGLU output.
template <typename V>
__global__ void interleave_rows_kernel(const V* src, V* dst, uint32_t half_rows, uint32_t row_vecs) {
    const size_t total = (size_t)2 * half_rows * row_vecs;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t drow = i / row_vecs, col = i % row_vecs;
        const size_t srow = (drow & 1) ? half_rows + drow / 2 : drow / 2;
        dst[i] = src[srow * row_vecs + col];
    }
}

unsigned long long stream_base(uint64_t seed, uint64_t stream_id) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (stream_id + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint32_t fill_grid(tb_context* ctx, size_t n) {
    const size_t want = (n + 255) / 256, most = (size_t)ctx->sms * 16;
    return (uint32_t)(want < most ? (want ? want : 1) : most);
}

}  // namespace

int launch_embed_q8(tb_context* ctx, const int8_t* w, const __half* s, const uint32_t* token, uint32_t cols, float scale, float* out, uint32_t wbits) {
    if (!w || !s || !token || !out || cols == 0 || cols % 32 != 0 || (wbits == 4 && cols % 64 != 0)) return fail(OUT_OF_RANGE, "embed: bad arguments");
    if (wbits == 4) TB_CUDA(launch_kernel(ctx, embed_q4_kernel, dim3((cols + 255) / 256), dim3(256), 0, true, reinterpret_cast<const uint8_t*>(w), s, token, cols, scale, out));
    else TB_CUDA(launch_kernel(ctx, embed_q8_kernel, dim3((cols + 255) / 256), dim3(256), 0, true, w, s, token, cols, scale, out));
    return OK;
}

int launch_norm(tb_context* ctx, const float* h, const float* y, const float* w1, const float* w2, uint32_t n, float eps, float hscale, float* h_out,
                float* x_out) {
    if (!h || n == 0 || (y && !w1)) return fail(OUT_OF_RANGE, "norm: bad arguments");
    TB_CUDA(launch_kernel(ctx, norm_kernel, dim3(1), dim3(1024), 0, true, h, y, w1, w2, n, eps, hscale, h_out, x_out));
    return OK;
}

int launch_sample(tb_context* ctx, const float* logits, uint32_t vocab, float softcap, float penalty, const uint32_t* seen, const uint32_t* allowed,
                  unsigned long long* best, uint32_t* count, uint32_t* state, uint32_t* seen_out, uint32_t* token_out) {
    if (!logits || !best || !count || !state || vocab == 0) return fail(OUT_OF_RANGE, "sample: bad arguments");
    uint32_t grid = (vocab + 4095) / 4096;
    if (grid > (uint32_t)ctx->sms) grid = (uint32_t)ctx->sms;
    TB_CUDA(launch_kernel(ctx, sample_greedy_kernel, dim3(grid), dim3(1024), 0, true, logits, vocab, softcap, penalty, seen, allowed, best, count, state,
                          seen_out, token_out));
    return OK;
}

int launch_topk(tb_context* ctx, const float* logits, uint32_t vocab, uint32_t k, uint32_t* idx, float* val, unsigned long long*) {
    if (!logits || !idx || !val || vocab == 0 || k == 0 || k > vocab) return fail(OUT_OF_RANGE, "topk: bad arguments");
    TB_CUDA(launch_kernel(ctx, topk_kernel, dim3(1), dim3(1024), 0, true, logits, vocab, k, idx, val));
    return OK;
}

int launch_fill_codes(tb_context* ctx, uint64_t seed, uint64_t stream_id, int8_t* w, size_t n) {
    fill_codes_kernel<<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(stream_base(seed, stream_id), w, n);
    TB_CUDA(cudaGetLastError());
    return OK;
}
int launch_fill_scales(tb_context* ctx, uint64_t seed, uint64_t stream_id, __half* s, size_t n, float mul) {
    fill_scales_kernel<<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(stream_base(seed, stream_id), s, n, mul);
    TB_CUDA(cudaGetLastError());
    return OK;
}
int launch_fill_gauss_f16(tb_context* ctx, uint64_t seed, uint64_t stream_id, __half* x, size_t n, float mul) {
    fill_gauss_f16_kernel<<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(stream_base(seed, stream_id), x, n, mul);
    TB_CUDA(cudaGetLastError());
    return OK;
}
int launch_fill_uniform(tb_context* ctx, uint64_t seed, uint64_t stream_id, float* x, size_t n, float lo, float hi) {
    fill_uniform_kernel<<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(stream_base(seed, stream_id), x, n, lo, (hi - lo) * (1.0f / 65536.0f));
    TB_CUDA(cudaGetLastError());
    return OK;
}
int launch_interleave_rows(tb_context* ctx, const void* src, void* dst, uint32_t half_rows, uint32_t row_bytes) {
    if (row_bytes % 2 != 0) return fail(OUT_OF_RANGE, "interleave: rows must be a multiple of 2 bytes");
    if (row_bytes % 16 == 0) {
        const size_t n = (size_t)2 * half_rows * (row_bytes / 16);
        interleave_rows_kernel<uint4><<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), half_rows, row_bytes / 16);
    } else {
        const size_t n = (size_t)2 * half_rows * (row_bytes / 2);
        interleave_rows_kernel<unsigned short><<<fill_grid(ctx, n), 256, 0, ctx->stream>>>(static_cast<const unsigned short*>(src), static_cast<unsigned short*>(dst),
                                                                                        half_rows, row_bytes / 2);
    }
    TB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace tb
