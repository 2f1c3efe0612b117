// The encoder's bidirectional attention on the fifth-generation tensor cores: attend_f16 (crates/tachyon/src/ptx/encoder.rs:
// 961-1215) for heads of 64.  Sequences are packed back to back in qkv (f16 [n][3h], rows [q, k, v]); query i of a sequence
// sees key j of the same sequence when |i - j| <= window, or every key when the layer is global.  Same results, to the
// rounding of the probabilities, as encoder.cu's mma.sync kernel, which stays for heads of 32.
//
// A block takes one tile of up to 128 queries of one sequence and one head (tile list entries [first row, length, first
// query], built on the host; an entry of length 0 is an unused slot) and walks the sequence's keys in tiles of 64 that start
// at multiples of 64 of the sequence, so a sequence's sums do not depend on what it is packed with.  The structure is
// prefill_tc.cu's with one box of 64 dimensions where that has four:
//   warp 0      one thread issues the TMA loads through one 2-D map over qkv: the queries once, then per tile 64 rows of keys
//               and 64 of values, two tiles ahead (rows past the sequence's end are the next sequence's, or zeros past the
//               buffer: the softmax never lets them weigh);
//   warp 1      allocates tensor memory (two score buffers of 64 columns, the output of 64); one thread issues S = Q K^T
//               (M128 N64 K64) and O += P V (M128 N64 K64, V MN-major as it lies in memory);
//   warps 2-9   softmax, two threads a query row (32 keys and 32 output dimensions each), lazy running maximum.
// Two blocks fit an SM (83 KiB of shared memory, 256 columns of tensor memory each).  Every wait is bounded.
#include <cuda.h>

#include <string>

#include "common.cuh"
#include "internal.h"
#include "tc.cuh"

namespace tb {

namespace {

using namespace tc;

constexpr int D = 64, ROWS = 128, KT = 64;
constexpr int QCH = ROWS * 128, KCH = KT * 128;  // a box of 64 dimensions (128 bytes) x 128 queries, or x 64 keys
constexpr int OFF_Q = 0, OFF_K = QCH, OFF_V = OFF_K + 2 * KCH, OFF_P = OFF_V + 2 * KCH, OFF_BAR = OFF_P + 2 * QCH;
constexpr int SMEM_BYTES = 1024 + OFF_BAR + 128 + 2 * ROWS * 4;
constexpr int COL_O = 2 * KT;
constexpr int THREADS = 320;

constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

struct Bars {
    uint64_t q_full, k_full[2], v_full[2], s_full[2], p_ready[2], pv_done[2];
    uint32_t tmem;
    float xch[2][ROWS];  // [half][row]: what a row's two threads trade: each tile their maxima, at the end their sums
};

struct EncArgs {
    __half* out;            // f16 [n][h]
    const uint32_t* tiles;  // [slots][3]: first row of the sequence, its length, the tile's first query
    uint32_t h;
    int window;             // < 0: every key of the sequence
    float sscale;           // log2(e) / sqrt(d)
};

__global__ void __launch_bounds__(THREADS, 2) enc_attend_tc_kernel(const __grid_constant__ CUtensorMap map, const __grid_constant__ CUtensorMap kmap,
                                                                   const EncArgs a, uint32_t* status) {
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    Bars& bar = *reinterpret_cast<Bars*>(raw + OFF_BAR);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t start = a.tiles[blockIdx.x * 3], len = a.tiles[blockIdx.x * 3 + 1], q0 = a.tiles[blockIdx.x * 3 + 2], head = blockIdx.y;
    if (len == 0) return;  // an unused slot of a padded batch: the whole block leaves before it holds anything
    const uint32_t nq = min((uint32_t)ROWS, len - q0);
    // Keys any query of the tile sees: [lo, hi) of the sequence, in tiles that start at multiples of 64.
    const uint32_t lo = a.window < 0 ? 0u : (q0 > (uint32_t)a.window ? q0 - (uint32_t)a.window : 0u);
    const uint32_t hi = a.window < 0 ? len : min(len, q0 + nq + (uint32_t)a.window);
    const uint32_t tile0 = lo / KT * KT, nt = (hi - 1 - tile0) / KT + 1;

    if (threadIdx.x == 0) {
        mbar_init(&bar.q_full, 1);
        for (int k = 0; k < 2; k++)
            mbar_init(&bar.k_full[k], 1), mbar_init(&bar.v_full[k], 1), mbar_init(&bar.s_full[k], 1), mbar_init(&bar.pv_done[k], 1), mbar_init(&bar.p_ready[k], 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&bar.tmem)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bar.tmem;

    if (warp == 0) {
        if (lane == 0) {
            const int qcol = (int)(head * D), kcol = (int)(a.h + head * D), vcol = (int)(2 * a.h + head * D);
            mbar_expect_tx(&bar.q_full, QCH);
            tma_load_2d(raw + OFF_Q, &map, qcol, (int)(start + q0), &bar.q_full);
            for (uint32_t i = 0; i < nt; i++) {
                const int row0 = (int)(start + tile0 + i * KT);
                const uint32_t st = i & 1, before = ((i - 2) >> 1) & 1;
                // A key stage is free once S of the tile two before is done, a value stage once that tile's P V is done.
                if (i >= 2 && !mbar_wait(&bar.s_full[st], before)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                mbar_expect_tx(&bar.k_full[st], KCH);
                tma_load_2d(raw + OFF_K + st * KCH, &kmap, kcol, row0, &bar.k_full[st]);
                if (i >= 2 && !mbar_wait(&bar.pv_done[st], before)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                mbar_expect_tx(&bar.v_full[st], KCH);
                tma_load_2d(raw + OFF_V + st * KCH, &kmap, vcol, row0, &bar.v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t qa = smem_addr(raw + OFF_Q), ka = smem_addr(raw + OFF_K), va = smem_addr(raw + OFF_V), pa = smem_addr(raw + OFF_P);
            auto scores = [&](uint32_t i) {  // S[i & 1] = Q K^T over the 64 dimensions: four products of K = 16
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int k = 0; k < D / 16; k++) mma_f16(tmem + (i & 1) * KT, desc_k_major(qa + k * 32), desc_k_major(ka + (i & 1) * KCH + k * 32), IDESC_S, k > 0 ? 1u : 0u);
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
                for (int k = 0; k < KT / 16; k++)  // O += P V over the tile's 64 keys (one box of 64 dimensions: no second group)
                    mma_f16(tmem + COL_O, desc_k_major(pa + (i & 1) * QCH + k * 32), desc_mn_major(va + (i & 1) * KCH + k * 2048, KCH), IDESC_PV,
                            (i > 0 || k > 0) ? 1u : 0u);
                mma_commit(&bar.pv_done[i & 1]);
            }
            if (!ok) atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
        }
    } else {
        // Softmax and epilogue.  This warp reads the tensor-memory lanes of its quarter, warp % 4; a row's two threads (in warps
        // w and w + 4) take the tile's keys 32 half .. + 31 and the output's dimensions 32 half .. + 31.
        const uint32_t quarter = warp & 3, half = (uint32_t)(warp - 2) >> 2, row = 32 * quarter + lane, qi = q0 + row;
        const bool valid = row < nq;
        const uint32_t lane_addr = (32 * quarter) << 16;
        // Keys of the sequence this query sees: [k_lo, k_hi).
        const int k_lo = a.window < 0 ? 0 : max((int)qi - a.window, 0);
        const int k_hi = a.window < 0 ? (int)len : min((int)len, (int)qi + a.window + 1);
        float m_used = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (uint32_t i = 0; i < nt; i++) {
            const uint32_t sbuf = tmem + lane_addr + (i & 1) * KT + half * 32;
            // A wait that runs out is reported once; the thread then walks the remaining tiles without waiting, so that it still
            // meets its partner at every barrier below.
            if (ok && !mbar_wait(&bar.s_full[i & 1], (i >> 1) & 1)) ok = false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int k0 = (int)(tile0 + i * KT + 32 * half);  // key k0 + c is seen when c lies in [c_lo, c_hi)
            const int c_lo = valid ? max(k_lo - k0, 0) : 32;
            const int c_hi = valid ? min(k_hi - k0, 32) : 0;  // may be <= c_lo: nothing seen
            const bool any = __any_sync(0xffffffffu, c_lo < c_hi);
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
            uint8_t* prow = raw + OFF_P + (i & 1) * QCH + row * 128;  // this thread's half of the row: pieces 4 half .. 4 half + 3
            if (!any) {  // nobody sees these keys: zeros, which P V still multiplies
#pragma unroll
                for (int pc = 0; pc < 4; pc++) *reinterpret_cast<uint4*>(prow + (((half * 4 + pc) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            } else {
                uint32_t r[32];
                tmem_load32(sbuf, r);
#pragma unroll
                for (int pc = 0; pc < 4; pc++) {  // pieces of eight probabilities (16 bytes)
                    uint32_t hw[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int c = pc * 8 + 2 * e;
                        const float e0 = (c >= c_lo && c < c_hi) ? ex2(fmaf(__uint_as_float(r[c]), a.sscale, -base)) : 0.0f;
                        const float e1 = (c + 1 >= c_lo && c + 1 < c_hi) ? ex2(fmaf(__uint_as_float(r[c + 1]), a.sscale, -base)) : 0.0f;
                        const __half2 hh = __floats2half2_rn(e0, e1);
                        sum += e0 + e1;
                        hw[e] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    *reinterpret_cast<uint4*>(prow + (((half * 4 + pc) ^ (row & 7)) << 4)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                }
            }
            l_run = fmaf(l_run, corr, sum);
            if (i > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // The output must be at rest: P V of the tile before is done.
                if (ok && !mbar_wait(&bar.pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1)) ok = false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t r[32];
                const uint32_t at = tmem + lane_addr + COL_O + half * 32;
                tmem_load32(at, r);
#pragma unroll
                for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
                tmem_store32(at, r);
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
            uint32_t r[32];
            tmem_load32(tmem + lane_addr + COL_O + half * 32, r);
            if (valid) {
                uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)(start + qi) * a.h + head * D + half * 32);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    uint32_t hw[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const __half2 hh = __floats2half2_rn(__uint_as_float(r[8 * e + 2 * k]) * inv, __uint_as_float(r[8 * e + 2 * k + 1]) * inv);
                        hw[k] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    dst[e] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
}

}  // namespace

// Heads of 64 and a row pitch TMA takes (whole 16 bytes); qkv and out 16-byte aligned.
bool enc_attend_tc_supports(uint32_t h, uint32_t d) { return d == (uint32_t)D && h % d == 0 && h % 8 == 0; }

int launch_enc_attend_tc(tb_context* ctx, const __half* qkv, const uint32_t* tiles, __half* out, uint32_t h, int window, float scale, uint32_t ntiles,
                         uint32_t rows) {
    tc::EncodeTiled enc = tc::encode_tiled();
    if (!enc) return fail(NO_DRIVER, "encoder attention: the driver does not export cuTensorMapEncodeTiled");
    if (!qkv || !tiles || !out || ntiles == 0 || rows == 0) return fail(OUT_OF_RANGE, "encoder attention: null or empty argument");
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) & 15) return fail(OUT_OF_RANGE, "encoder attention: buffers must be 16-byte aligned");
    if (!(scale > 0.0f)) return fail(OUT_OF_RANGE, "encoder attention: the scale must be positive");
    CUtensorMap qm, km;
    for (int which = 0; which < 2; which++) {  // one tensor, [rows][3h]: boxes of 128 rows (queries) and of 64 (keys, values)
        const cuuint64_t dims[2] = {(cuuint64_t)3 * h, rows};
        const cuuint64_t strides[1] = {(cuuint64_t)3 * h * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)(which ? KT : ROWS)}, elem[2] = {1, 1};
        const CUresult r = enc(which ? &km : &qm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(qkv), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "encoder attention: cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    }
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(enc_attend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[ctx->gpu & 15] = true;
    }
    const EncArgs a{out, tiles, h, window, scale};
    enc_attend_tc_kernel<<<dim3(ntiles, h / D), THREADS, SMEM_BYTES, ctx->stream>>>(qm, km, a, ctx->status);
    TB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace tb
