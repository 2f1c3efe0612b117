// Prefill attention on the fifth-generation tensor cores: flash_256 (crates/tachyon/src/ptx/flash.rs:1-23, 246-251) for heads of
// 256 with four query heads to a key-value head.  Token t of the chunk, at position pos0 + t, attends positions
// p - window < j <= p of the cache ring.  Same results, to the rounding of the probabilities, as prefill.cu's mma.sync kernel,
// which stays for every other shape.
//
// A block takes 32 tokens x the four query heads of one key-value head = 128 query rows (row = 4 * token + head) and walks
// the keys in tiles of 64 positions that start at multiples of 64, so a token's sums do not depend on how the prompt was
// cut into chunks (flash.rs:9-12).  Ten warps:
//   warp 0      one thread issues the TMA loads: the queries once (3-D map over [token][head][256]), then per tile the keys and
//               the values of 64 ring slots (3-D maps over [key-value head][slot][256]), each as four boxes of 64 dimensions
//               in the 128-byte swizzle, two tiles ahead of the products (two stages of keys, two of values);
//   warp 1      allocates tensor memory (two score buffers of 64 columns, the output of 256); one thread issues
//               S = Q K^T (M128 N64 K256: both operands K-major) and O += P V (M128 N256 K64: P K-major from shared memory,
//               V as it lies in the cache, [key][dimension], which is the MN-major form of a B operand);
//   warps 2-9   softmax: two threads own query row r (tensor-memory lane r; warps w and w + 4 read the same quarter of the
//               lanes), one the tile's first 32 keys and the first 128 output dimensions, the other the rest; they trade their
//               maxima through shared memory.  Two passes over the tile's scores with tcgen05.ld (maximum, then exponentials;
//               a half no row of the warp sees is skipped), probabilities rounded to f16 into shared memory in the
//               swizzled K-major layout.  The running maximum only moves when a tile
//               exceeds it by more than 8 (in base 2), so probabilities stay below 2^8 and the output in tensor memory is
//               rescaled (tcgen05.ld, multiply, tcgen05.st) only on those tiles, usually the first one or two.
// The score buffers and the probability buffers alternate, so S of tile i + 1 is multiplied while tile i is in the softmax and
// P V of tile i while tile i + 1 is; keys of tile i + 2 are loaded as soon as S of tile i is done, values as soon as P V of
// tile i is done.  What bounds it, measured by switching parts off: 64 KiB of loads a tile is the SM's rate from the L2
// (0.6 us), the products and the softmax add 0.6 us each when alone and 0.8 together; they share the 224 KiB of
// shared-memory traffic a tile causes (the score product re-reads the 64 KiB of queries every tile).  Every wait is bounded.
#include <cuda.h>

#include <string>

#include "common.cuh"
#include "internal.h"
#include "tc.cuh"

namespace tb {

namespace {

using namespace tc;

constexpr int D = 256, G = 4, TQ = 32, ROWS = TQ * G, KT = 64;
constexpr int CHUNK = ROWS * 128;                          // queries, probabilities: a box of 64 dimensions (128 bytes) x 128 rows
constexpr int KCH = KT * 128, STAGE = 4 * KCH;             // keys, values: a box of 64 dimensions x 64 slots; a tile is four of them
constexpr int OFF_Q = 0, OFF_K = 4 * CHUNK, OFF_V = OFF_K + 2 * STAGE, OFF_P = OFF_V + 2 * STAGE, OFF_BAR = OFF_P + 2 * CHUNK;  // two buffers of probabilities
constexpr int SMEM_BYTES = 1024 + OFF_BAR + 128 + 2 * ROWS * 4;
constexpr int COL_O = 2 * KT;                              // tensor-memory columns: scores at 0 and KT, the output from here
constexpr int THREADS = 320;
static_assert(SMEM_BYTES <= 232448, "over the 227 KiB a block may use");

// kind::f16 instruction descriptors: f32 accumulator, f16 operands, A K-major; N >> 3 at bit 17, M >> 4 at bit 24; bit 16 set
// makes B MN-major.
constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

struct Bars {
    uint64_t q_full, k_full[2], v_full[2], s_full[2], p_ready[2], pv_done[2];
    uint32_t tmem;
    float xch[2][ROWS];  // [half][row]: what a row's two threads trade: each tile their maxima, at the end their sums
};

struct FlashArgs {
    void* out;
    const uint32_t* pos_dev;  // the first position from device memory instead of pos0 (the "flash_256" launch), or null
    uint32_t tokens, pos0, cap, window, heads;
    float sscale;  // factor of the scores (1 when the queries already carry scale * log2 e)
    int out_f32;
};

__global__ void __launch_bounds__(THREADS, 1) prefill_flash_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                                                                      const __grid_constant__ CUtensorMap v_map, const FlashArgs a, uint32_t* status) {
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    Bars& bar = *reinterpret_cast<Bars*>(raw + OFF_BAR);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t t0 = blockIdx.x * TQ, kvh = blockIdx.y;
    pdl_wait();  // the queries, this chunk's keys and values and the position come from the kernels in front
    const uint32_t pos0 = a.pos_dev != nullptr ? __ldg(a.pos_dev) : a.pos0;
    const uint32_t p_first = pos0 + t0, p_last = pos0 + min(t0 + TQ, a.tokens) - 1;
    const uint32_t lo = p_first + 1 > a.window ? p_first + 1 - a.window : 0;  // oldest position any token of the block sees
    const uint32_t tile0 = lo / KT * KT, nt = (p_last - tile0) / KT + 1;

    if (threadIdx.x == 0) {
        mbar_init(&bar.q_full, 1);
        for (int k = 0; k < 2; k++)
            mbar_init(&bar.k_full[k], 1), mbar_init(&bar.v_full[k], 1), mbar_init(&bar.s_full[k], 1), mbar_init(&bar.pv_done[k], 1), mbar_init(&bar.p_ready[k], 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&bar.tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bar.tmem;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bar.q_full, 4 * CHUNK);
            for (int c = 0; c < 4; c++) tma_load_3d(raw + OFF_Q + c * CHUNK, &q_map, 64 * c, (int)(kvh * G), (int)t0, &bar.q_full);
            for (uint32_t i = 0; i < nt; i++) {
                const int slot0 = (int)((tile0 + i * KT) % a.cap);
                const uint32_t st = i & 1, before = ((i - 2) >> 1) & 1;  // the stage, and the parity of the tile that held it last
                // A key stage is free once S of the tile two before is done, a value stage once that tile's P V is done.
                if (i >= 2 && !mbar_wait(&bar.s_full[st], before)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                mbar_expect_tx(&bar.k_full[st], STAGE);
                for (int c = 0; c < 4; c++) tma_load_3d(raw + OFF_K + st * STAGE + c * KCH, &k_map, 64 * c, slot0, (int)kvh, &bar.k_full[st]);
                if (i >= 2 && !mbar_wait(&bar.pv_done[st], before)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                mbar_expect_tx(&bar.v_full[st], STAGE);
                for (int c = 0; c < 4; c++) tma_load_3d(raw + OFF_V + st * STAGE + c * KCH, &v_map, 64 * c, slot0, (int)kvh, &bar.v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t qa = smem_addr(raw + OFF_Q), ka = smem_addr(raw + OFF_K), va = smem_addr(raw + OFF_V), pa = smem_addr(raw + OFF_P);
            auto scores = [&](uint32_t i) {  // S[i & 1] = Q K^T over the 256 dimensions: sixteen products of K = 16
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int k = 0; k < D / 16; k++)
                    mma_f16(tmem + (i & 1) * KT, desc_k_major(qa + (k >> 2) * CHUNK + (k & 3) * 32), desc_k_major(ka + (i & 1) * STAGE + (k >> 2) * KCH + (k & 3) * 32),
                            IDESC_S, k > 0 ? 1u : 0u);
                mma_commit(&bar.s_full[i & 1]);
            };
            bool ok = mbar_wait(&bar.q_full, 0) && mbar_wait(&bar.k_full[0], 0);
            if (ok) scores(0);
            for (uint32_t i = 0; i < nt && ok; i++) {
                if (i + 1 < nt) {
                    ok = mbar_wait(&bar.k_full[(i + 1) & 1], ((i + 1) >> 1) & 1);
                    if (ok) scores(i + 1);
                }
                ok = ok && mbar_wait(&bar.p_ready[i & 1], (i >> 1) & 1) && mbar_wait(&bar.v_full[i & 1], (i >> 1) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int k = 0; k < KT / 16; k++)  // O += P V over the tile's 64 keys: four products of K = 16
                    mma_f16(tmem + COL_O, desc_k_major(pa + (i & 1) * CHUNK + k * 32), desc_mn_major(va + (i & 1) * STAGE + k * 2048, KCH), IDESC_PV,
                            (i > 0 || k > 0) ? 1u : 0u);
                mma_commit(&bar.pv_done[i & 1]);
            }
            if (!ok) atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
        }
    } else {
        // Softmax and epilogue.  This warp reads the tensor-memory lanes of its quarter, warp % 4; a row's two threads (in warps
        // w and w + 4) take the tile's keys 32 half .. + 31 and the output's dimensions 128 half .. + 127.
        const uint32_t quarter = warp & 3, half = (uint32_t)(warp - 2) >> 2, row = 32 * quarter + lane, tl = row / G, head = row % G;
        const uint32_t p = pos0 + t0 + tl;
        const bool valid = t0 + tl < a.tokens;
        const uint32_t lane_addr = (32 * quarter) << 16;
        const uint32_t first_seen = p + 1 > a.window ? p + 1 - a.window : 0;
        float m_used = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (uint32_t i = 0; i < nt; i++) {
            const uint32_t j0 = tile0 + i * KT, sbuf = tmem + lane_addr + (i & 1) * KT + half * 32;
            // A wait that runs out is reported once; the thread then walks the remaining tiles without waiting, so that it still
            // meets its partner at every barrier below.
            if (ok && !mbar_wait(&bar.s_full[i & 1], (i >> 1) & 1)) ok = false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // Key j0 + 32 half + c is seen when c lies in [c_lo, c_hi): at or before this token, inside its window.
            const int k0 = (int)(j0 + 32 * half);
            const int c_lo = valid ? max((int)first_seen - k0, 0) : 32;
            const int c_hi = valid ? min((int)p + 1 - k0, 32) : 0;  // may be <= c_lo: nothing seen
            const bool any = __any_sync(0xffffffffu, c_lo < c_hi);  // whether any row of the warp sees a key of this half
            float mt = -INFINITY;
            if (any) {
                uint32_t r[32];
                tmem_load32(sbuf, r);
#pragma unroll
                for (int e = 0; e < 32; e++)
                    if (e >= c_lo && e < c_hi) mt = fmaxf(mt, __uint_as_float(r[e]));
            }
            bar.xch[half][row] = mt;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (int)quarter) : "memory");  // the row's two threads
            mt = fmaxf(mt, bar.xch[half ^ 1][row]) * a.sscale;  // sscale is positive
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (int)quarter) : "memory");  // both have read: the slots may be written again
            float corr = 1.0f;
            if (mt > m_used + 8.0f) {  // also a row's first keys (m_used = -inf)
                corr = ex2(m_used - mt);  // 0 for the first keys
                m_used = mt;
            }
            const float base = fmaxf(m_used, -1e30f);  // finite, so a row that has seen nothing yet gets 2^-inf = 0 and no NaN
            // The probabilities go where P V of the tile two before read its own: wait for it.
            if (ok && i >= 2 && !mbar_wait(&bar.pv_done[i & 1], ((i - 2) >> 1) & 1)) ok = false;
            float sum = 0.0f;
            uint8_t* prow = raw + OFF_P + (i & 1) * CHUNK + row * 128;  // this thread's half of the row: pieces 4 half .. 4 half + 3
            if (!any) {  // nobody sees these keys: zeros, which P V still multiplies
#pragma unroll
                for (int pc = 0; pc < 4; pc++) *reinterpret_cast<uint4*>(prow + (((half * 4 + pc) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            } else {
                uint32_t r[32];
                tmem_load32(sbuf, r);
#pragma unroll
                for (int pc = 0; pc < 4; pc++) {  // pieces of eight probabilities (16 bytes)
                    uint32_t h[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int c = pc * 8 + 2 * e;
                        const float e0 = (c >= c_lo && c < c_hi) ? ex2(fmaf(__uint_as_float(r[c]), a.sscale, -base)) : 0.0f;
                        const float e1 = (c + 1 >= c_lo && c + 1 < c_hi) ? ex2(fmaf(__uint_as_float(r[c + 1]), a.sscale, -base)) : 0.0f;
                        const __half2 hh = __floats2half2_rn(e0, e1);
                        sum += e0 + e1;  // before the rounding: converting back would cost as much as the exponentials
                        h[e] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    *reinterpret_cast<uint4*>(prow + (((half * 4 + pc) ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                }
            }
            l_run = fmaf(l_run, corr, sum);
            if (i > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // The output must be at rest: P V of the tile before is done.
                if (ok && !mbar_wait(&bar.pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1)) ok = false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int cb = 0; cb < 4; cb++) {
                    uint32_t r[32];
                    const uint32_t at = tmem + lane_addr + COL_O + half * 128 + cb * 32;
                    tmem_load32(at, r);
#pragma unroll
                    for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
                    tmem_store32(at, r);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads P through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar.p_ready[i & 1]);
        }
        if (ok && !mbar_wait(&bar.pv_done[(nt - 1) & 1], ((nt - 1) >> 1) & 1)) ok = false;
        if (!ok) atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        bar.xch[half][row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + (int)quarter) : "memory");
        if (ok) {
            const float l_all = l_run + bar.xch[half ^ 1][row];
            const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
            const size_t at = ((size_t)(t0 + tl) * a.heads + kvh * G + head) * D + half * 128;
            for (int cb = 0; cb < 4; cb++) {
                uint32_t r[32];
                tmem_load32(tmem + lane_addr + COL_O + half * 128 + cb * 32, r);
                if (!valid) continue;
                if (a.out_f32) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at + cb * 32);
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        dst[e] = make_float4(__uint_as_float(r[4 * e]) * inv, __uint_as_float(r[4 * e + 1]) * inv, __uint_as_float(r[4 * e + 2]) * inv,
                                             __uint_as_float(r[4 * e + 3]) * inv);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(a.out) + at + cb * 32);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        uint32_t h[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const __half2 hh = __floats2half2_rn(__uint_as_float(r[8 * e + 2 * k]) * inv, __uint_as_float(r[8 * e + 2 * k + 1]) * inv);
                            h[k] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                        dst[e] = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

}  // namespace

// The shapes this kernel takes: heads of 256, four query heads to a key-value head, a ring of whole tiles.
bool prefill_flash_tc_supports(uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t cap) {
    return head_dim == (uint32_t)D && kv_heads != 0 && heads == (uint32_t)G * kv_heads && cap % KT == 0;
}

int launch_prefill_flash_tc(tb_context* ctx, const __half* q, const __half* kc, const __half* vc, void* out, uint32_t tokens, uint32_t pos0, uint32_t cap,
                            uint32_t window, uint32_t heads, uint32_t kv_heads, const uint32_t* pos_dev, float sscale, int out_f32) {
    tc::EncodeTiled enc = tc::encode_tiled();
    if (!enc) return fail(NO_DRIVER, "prefill attention: the driver does not export cuTensorMapEncodeTiled");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(OUT_OF_RANGE, "prefill attention: buffers must be 16-byte aligned");
    if (tokens == 0 || window == 0 || !(sscale > 0.0f)) return fail(OUT_OF_RANGE, "prefill attention: empty chunk or window, or a scale that is not positive");
    CUtensorMap qm, km, vm;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)D, heads, tokens};
        const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)heads * D * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)TQ}, elem[3] = {1, 1, 1};
        const CUresult r = enc(&qm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(q), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "prefill attention: cuTensorMapEncodeTiled (queries) failed (" + std::to_string((int)r) + ")");
    }
    for (int which = 0; which < 2; which++) {
        const cuuint64_t dims[3] = {(cuuint64_t)D, cap, kv_heads};
        const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)cap * D * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)KT, 1}, elem[3] = {1, 1, 1};
        const CUresult r = enc(which ? &vm : &km, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(which ? vc : kc), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "prefill attention: cuTensorMapEncodeTiled (cache) failed (" + std::to_string((int)r) + ")");
    }
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(prefill_flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[ctx->gpu & 15] = true;
    }
    const FlashArgs a{out, pos_dev, tokens, pos0, cap, window, heads, sscale, out_f32};
    TB_CUDA(launch_kernel(ctx, prefill_flash_tc_kernel, dim3((tokens + TQ - 1) / TQ, kv_heads), dim3(THREADS), (size_t)SMEM_BYTES, true, qm, km, vm, a, ctx->status));
    return OK;
}

}  // namespace tb
