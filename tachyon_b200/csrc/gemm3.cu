// The prefill / encoder product on pairs of SMs: D[M, N] = A[M, K] (f16) x W[N, K]^T with W quantised, as gemm.cu and
// gemm2.cu compute it, with `tcgen05.mma.cta_group::2`.  Two blocks of a cluster share every product: block r of the
// pair holds 128 token rows of A and dequantises half of the tile's weight rows; one thread of the leading block
// issues MMAs of M 256 that read both blocks' shared memory and leave each block its 128 rows of the accumulator in
// its own tensor memory.  Per FLOP each block copies and dequantises what gemm.cu's 256 x 256 tile does, and half of
// what gemm2.cu's 256 x 128 tile copies of A; the accumulator of 128 x BN fits tensor memory twice, so the epilogue of
// a tile overlaps the products of the next, as in gemm2.cu.
//
// Warps of each block: 0 activation copies, 1 code copies, 2 MMA issue (leading block) or relay (the other block: tells
// the leader when a stage of its shared memory is full), then the dequantising warps, then eight epilogue warps.
// Barriers between the blocks: the relay arrives on the leader's `peer_full`; the leader's commits arrive on both
// blocks' `empty` and `acc_full`; both blocks' epilogue warps arrive on the leader's `acc_empty`.  Every wait is
// bounded; a warp that gives up records it in the context's status word and leaves its loops; the blocks meet at a
// cluster barrier before either exits, so neither reads the other's shared memory after it is gone.
//
// State: results equal the other schedules' on every test shape (tests/test_gemm.py runs both tile widths).  Speed: 660
// to 790 TFLOP/s on the benchmark's long shapes against 990 to 1,000 for gemm2.cu, so launch_gemm_q8 does not pick it
// (TACHYON_B200_GEMM=3 or 4 does).  What the measurements showed on the way: an arrival on the other SM's barrier keeps
// the issuing thread for most of a microsecond (hence several relay lanes, and no such arrival in the dequantising
// loop); a dequantising turn has about half a microsecond of fixed cost (hence several k tiles per turn); more stages
// (4 -> 6) changed nothing.  Not yet understood: the remaining 0.8 us per 64 of K with the leader still waiting for
// full stages.
#include <cuda.h>

#include <string>

#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int BM = 128, BK = 64;  // token rows per block, K per stage
constexpr int ST = 6;             // stages of f16 operands
constexpr int CS = 4;             // stages of codes (at least PER)
constexpr int EW = 8;             // epilogue warps (two per quarter of the accumulator's lanes)
constexpr int PER = 3;            // k tiles a dequantising warp converts per turn
constexpr int RELAYS = 4;         // lanes of the second block's relay warp (fewer than ST)
constexpr int FIRST_DW = 3;

// BN: weight rows of a pair's tile (accumulator columns); each block dequantises BN / 2 of them.
template <int BN>
struct Shape {
    static constexpr int BH = BN / 2;                    // weight rows a block dequantises
    static constexpr int DW = BH / 8;                    // dequantising warps: a thread per (row, quarter of the 64 codes)
    static constexpr int FIRST_EW = FIRST_DW + DW;
    static constexpr int THREADS = 32 * (FIRST_EW + EW);
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BH * BK * 2, C_BYTES = BH * BK;  // per stage; codes at 8 bits
    static constexpr int OFF_A = 0, OFF_B = OFF_A + ST * A_BYTES, OFF_C = OFF_B + ST * B_BYTES, OFF_BAR = OFF_C + CS * C_BYTES;
    static constexpr int SMEM_BYTES = 1024 + OFF_BAR + 512;
    static constexpr uint32_t COLS = 2 * BN;             // tensor memory columns: two accumulators
    // kind::f16, f32 accumulator, K-major A and B, N = BN, M = 256 over the pair
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    static_assert(SMEM_BYTES <= 232448, "over the 227 KiB a block may use");
    static_assert(COLS == 256 || COLS == 512, "tensor memory is allocated in powers of two");
};

enum : uint32_t { ERR_PAIR_TMEM = 5 };  // the two blocks of a pair were given different tensor memory

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {  // K-major, 128-byte rows, SWIZZLE_128B, 1024 bytes between 8-row groups
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this shared address in both blocks of the pair once the products this thread has issued are
// done (one commit signalling both: two commits, one per block, measured no faster and are not how the pair is meant
// to be released).
__device__ __forceinline__ void mma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of this block's shared address `local` in block `cta` of the cluster.
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(cta));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
// mbar_wait for a barrier that another block of the cluster (or a commit of the pair's products) arrives on: acquire at
// cluster scope, and polled with test_wait, which returns at once: try_wait may put the thread to sleep, and an arrival
// from another SM does not wake it before its time is up.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    const unsigned long long start = global_ns();
    for (uint32_t spins = 0;; ++spins) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spins & 255u) == 255u && global_ns() - start > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Four int8 codes (one word) -> four f16 of code * scale: 0x6400 | (code ^ 0x80) is the f16 1024 + code + 128.
__device__ __forceinline__ void dequant4(uint32_t w, __half2 scale, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x80808080u;
    uint32_t a = __byte_perm(x, 0x64646464u, 0x5140), b = __byte_perm(x, 0x64646464u, 0x7362);
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    const __half2 va = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&a), bias), scale), vb = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&b), bias), scale);
    lo = *reinterpret_cast<const uint32_t*>(&va), hi = *reinterpret_cast<const uint32_t*>(&vb);
}
// Eight four-bit weights (quant.rs:60-66: low nibbles are weights 0..3, high nibbles 4..7) -> eight f16 of (n - 8) * scale.
__device__ __forceinline__ void dequant8_q4(uint32_t w, __half2 scale, uint32_t (&out)[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    const __half2 bias = __floats2half2_rn(1032.0f, 1032.0f);
    uint32_t p[4] = {__byte_perm(lo, 0x64646464u, 0x4140), __byte_perm(lo, 0x64646464u, 0x4342), __byte_perm(hi, 0x64646464u, 0x4140),
                     __byte_perm(hi, 0x64646464u, 0x4342)};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p[i]), bias), scale);
        out[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
}

struct Args {
    const __half* s;   // scales [N][K / 32] (8-bit codes) or [N][K / 64] (4-bit)
    void* out;
    uint32_t M, N, K;
    int mode;          // as gemm.cu: 0 f32, 1 f16, 2 GeGLU(tanh) pairs, 3 f32 +=, 4 GeGLU(erf) pairs, 5 GELU(erf) f16
};

struct Bars {
    uint64_t full[ST], peer_full[ST], empty[ST], c_full[CS], c_empty[CS], acc_full[2], acc_empty[2];
    uint32_t tmem;
};

template <int WB, int BN>
__global__ void __launch_bounds__(Shape<BN>::THREADS, 1) gemm_pair_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                                                                          const Args g, uint32_t* status) {
    using S = Shape<BN>;
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    uint8_t *As = raw + S::OFF_A, *Bs = raw + S::OFF_B, *Cs = raw + S::OFF_C;
    Bars& bar = *reinterpret_cast<Bars*>(raw + S::OFF_BAR);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank(), pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t nk = g.K / BK, tiles_m = (g.M + 2 * BM - 1) / (2 * BM), tiles_n = (g.N + BN - 1) / BN, tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        // full: this block's activation copy and its dequantising warps.  peer_full (the leader's): the other block's relay.
        // WB == 16 (f16 weights): this block's half of the weight tile comes by TMA with the activations (warp 0), nothing is
        // converted, and the converting warps join the epilogue.
        for (int i = 0; i < ST; i++) mbar_init(&bar.full[i], WB == 16 ? 1 : S::DW + 1), mbar_init(&bar.peer_full[i], 1), mbar_init(&bar.empty[i], 1);
        for (int i = 0; i < CS; i++) mbar_init(&bar.c_full[i], 1), mbar_init(&bar.c_empty[i], S::DW);
        for (int i = 0; i < 2; i++) mbar_init(&bar.acc_full[i], 1), mbar_init(&bar.acc_empty[i], 2 * (WB == 16 ? S::DW + EW : EW));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {  // one warp of each block of the pair takes part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&bar.tmem)), "r"(S::COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // both blocks' barriers are initialised and both hold their tensor memory
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bar.tmem;
    // The pair's MMAs address one accumulator in both blocks: the two allocations must have come out alike.
    const bool sane = ld_cluster_u32(in_cta(smem_addr(&bar.tmem), rank ^ 1u)) == tmem;
    if (!sane && threadIdx.x == 0) atomicCAS(status, ERR_NONE, ERR_PAIR_TMEM);

    // Tile t of the pair: token tile t % tiles_m (256 rows, 128 per block), weight tile t / tiles_m (BN rows, BN / 2 per block).
    if (!sane) {
        // nothing to do but meet the other block below
    } else if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t t = pair; t < tiles; t += pairs) {
                const uint32_t m0 = (t % tiles_m) * (2 * BM) + rank * BM, n0 = (t / tiles_m) * BN + rank * S::BH;
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % ST;
                    if (it >= ST && !mbar_wait_cluster(&bar.empty[s], ((it / ST) - 1) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                        t = tiles;
                        break;
                    }
                    mbar_expect_tx(&bar.full[s], WB == 16 ? S::A_BYTES + S::B_BYTES : S::A_BYTES);
                    tma_load_2d(As + s * S::A_BYTES, &a_map, (int)(kt * BK), (int)m0, &bar.full[s]);
                    if constexpr (WB == 16) tma_load_2d(Bs + s * S::B_BYTES, &w_map, (int)(kt * BK), (int)n0, &bar.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (WB != 16 && lane == 0) {
            uint32_t ic = 0;
            for (uint32_t t = pair; t < tiles; t += pairs) {
                const uint32_t n0 = (t / tiles_m) * BN + rank * S::BH;
                for (uint32_t kt = 0; kt < nk; kt++, ic++) {
                    const uint32_t c = ic % CS;
                    if (ic >= CS && !mbar_wait(&bar.c_empty[c], ((ic / CS) - 1) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                        t = tiles;
                        break;
                    }
                    mbar_expect_tx(&bar.c_full[c], S::C_BYTES * WB / 8);
                    tma_load_2d(Cs + c * S::C_BYTES, &w_map, (int)(kt * BK * WB / 8), (int)n0, &bar.c_full[c]);
                }
            }
        }
    } else if (warp == 2) {
        if (lane == 0 && rank == 0) {
            // The leader: one MMA of M 256 per 16 of K, reading both blocks' stages.
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (uint32_t t = pair; t < tiles && ok; t += pairs, ti++) {
                const uint32_t b = ti & 1;
                if (ti >= 2 && !mbar_wait_cluster(&bar.acc_empty[b], ((ti >> 1) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % ST;
                    if (!mbar_wait(&bar.full[s], (it / ST) & 1) || !mbar_wait_cluster(&bar.peer_full[s], (it / ST) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a = smem_addr(As + s * S::A_BYTES), bb = smem_addr(Bs + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) mma_pair(tmem + b * BN, smem_desc(a + k * 32), smem_desc(bb + k * 32), S::IDESC, (kt > 0 || k > 0) ? 1u : 0u);
                    mma_commit_both(smem_addr(&bar.empty[s]));  // the stage is free in both blocks
                }
                if (ok) {
                    mma_commit_both(smem_addr(&bar.acc_full[b]));  // arrive when the tile's products have finished, in both blocks
                }
            }
        } else if (rank == 1 && lane < RELAYS) {
            // The relay: tells the leader when stage s of this block (activation rows and dequantised weights) is full.  The
            // dequantising warps arrive on their own block's barrier: a release at cluster scope in their loop measured
            // twice the time per turn.  An arrival at the other SM takes the issuing thread most of a microsecond, more
            // than the products of a k tile, so RELAYS lanes take the k tiles in turn (fewer than ST: when a lane moves on
            // to k tile it + RELAYS, the stage's barrier has long finished the phase before the one it waits for).
            const uint32_t mine = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;  // tiles this pair takes
            for (uint32_t it = lane; it < mine * nk; it += RELAYS) {
                const uint32_t s = it % ST;
                if (!mbar_wait(&bar.full[s], (it / ST) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                    break;
                }
                mbar_arrive_cluster(in_cta(smem_addr(&bar.peer_full[s]), 0));
            }
        }
    } else if (WB != 16 && warp < S::FIRST_EW) {
        // Dequantisation: thread j takes the 16 codes of piece (row j / 4, quarter j % 4) of every stage.
        const int j = threadIdx.x - 32 * FIRST_DW, row = j >> 2, qtr = j & 3;
        constexpr uint32_t GS = WB == 4 ? 8 : 4;               // k tiles one 16-byte load of scales covers
        const uint32_t spr = g.K / (WB == 4 ? 64 : 32);        // scales per row
        uint32_t it = 0, ic = 0;
        bool ok = true;
        for (uint32_t t = pair; t < tiles && ok; t += pairs) {
            const uint32_t n = (t / tiles_m) * BN + rank * S::BH + row;
            const bool live = n < g.N;
            const __half* srow = g.s + (size_t)n * spr;
            auto scales_from = [&](uint32_t kt) -> uint4 {  // the row's eight scales from k tile `kt` on
                const uint32_t at = kt * (WB == 4 ? 1 : 2);
                if (live && at + 8 <= spr && spr % 8 == 0) return __ldg(reinterpret_cast<const uint4*>(srow + at));
                uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (uint32_t e = 0; e < 8; e++)
                    if (live && at + e < spr) w[e >> 1] |= (uint32_t)__half_as_ushort(srow[at + e]) << (16 * (e & 1));
                return make_uint4(w[0], w[1], w[2], w[3]);
            };
            uint4 sc = scales_from(0), sc_next = sc;
            // The codes of k tile `kt` (code stage c) as eight f16 pairs of code * scale.
            auto convert = [&](uint32_t kt, uint32_t c, uint32_t (&v)[8]) {
                if (kt % GS == 0) {
                    if (kt > 0) sc = sc_next;
                    if (kt + GS < nk) sc_next = scales_from(kt + GS);  // one group ahead
                }
                const uint32_t h = WB == 4 ? (kt & 7u) : 2u * (kt & 3u) + (uint32_t)(qtr >> 1);  // which of the eight scales
                const uint32_t word = (h >> 1) == 0 ? sc.x : (h >> 1) == 1 ? sc.y : (h >> 1) == 2 ? sc.z : sc.w;
                const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)((h & 1u) ? (word >> 16) : (word & 0xffffu))));
                if constexpr (WB == 4) {
                    const uint2 cw = *reinterpret_cast<const uint2*>(Cs + c * S::C_BYTES + row * (BK / 2) + qtr * 8);
                    uint32_t a[4], b[4];
                    dequant8_q4(cw.x, s2, a), dequant8_q4(cw.y, s2, b);
#pragma unroll
                    for (int e = 0; e < 4; e++) v[e] = a[e], v[4 + e] = b[e];
                } else {
                    const uint4 cw = *reinterpret_cast<const uint4*>(Cs + c * S::C_BYTES + row * BK + qtr * 16);
                    dequant4(cw.x, s2, v[0], v[1]), dequant4(cw.y, s2, v[2], v[3]), dequant4(cw.z, s2, v[4], v[5]), dequant4(cw.w, s2, v[6], v[7]);
                }
            };
            auto store = [&](uint32_t stage, const uint32_t (&v)[8]) {
                uint8_t* base = Bs + stage * S::B_BYTES + row * 128;
                *reinterpret_cast<uint4*>(base + (((2 * qtr) ^ (row & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<uint4*>(base + (((2 * qtr + 1) ^ (row & 7)) << 4)) = make_uint4(v[4], v[5], v[6], v[7]);
            };
            // PER k tiles a turn: a turn's fixed costs (the waits, the proxy fence, the arrivals) are paid once per PER stages.
            for (uint32_t kt = 0; kt < nk; kt += PER) {
                const uint32_t cnt = min((uint32_t)PER, nk - kt);
                bool got = true;
#pragma unroll
                for (uint32_t i = 0; i < PER; i++)
                    if (i < cnt) got = got && mbar_wait(&bar.c_full[(ic + i) % CS], ((ic + i) / CS) & 1);
                if (!got) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                    ok = false;
                    break;
                }
                uint32_t v[PER][8];
#pragma unroll
                for (uint32_t i = 0; i < PER; i++)
                    if (i < cnt) convert(kt + i, (ic + i) % CS, v[i]);
                __syncwarp();
                if (lane == 0) {  // the codes are in registers
#pragma unroll
                    for (uint32_t i = 0; i < PER; i++)
                        if (i < cnt) mbar_arrive(&bar.c_empty[(ic + i) % CS]);
                }
#pragma unroll
                for (uint32_t i = 0; i < PER; i++)
                    if (i < cnt && it + i >= ST) got = got && mbar_wait_cluster(&bar.empty[(it + i) % ST], (((it + i) / ST) - 1) & 1);
                if (!got) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    ok = false;
                    break;
                }
#pragma unroll
                for (uint32_t i = 0; i < PER; i++)
                    if (i < cnt) store((it + i) % ST, v[i]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor cores read through the async proxy
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (uint32_t i = 0; i < PER; i++)
                        if (i < cnt) mbar_arrive(&bar.full[(it + i) % ST]);
                }
                it += cnt, ic += cnt;
            }
        }
    } else {
        // Epilogue: a warp reads the accumulator lanes (this block's token rows) of its quarter q = warp % 4, 32 columns at
        // a time; the two warps of a quarter take alternate column blocks.
        constexpr int FIRST = WB == 16 ? FIRST_DW : S::FIRST_EW, PARTS = (WB == 16 ? S::DW + EW : EW) / 4;
        const uint32_t q = warp & 3, part = (warp - FIRST) >> 2;
        const uint32_t acc_empty_at_leader[2] = {in_cta(smem_addr(&bar.acc_empty[0]), 0), in_cta(smem_addr(&bar.acc_empty[1]), 0)};
        uint32_t ti = 0;
        for (uint32_t t = pair; t < tiles; t += pairs, ti++) {
            const uint32_t b = ti & 1, m0 = (t % tiles_m) * (2 * BM) + rank * BM, n0 = (t / tiles_m) * BN;
            if (!mbar_wait_cluster(&bar.acc_full[b], (ti >> 1) & 1)) {
                atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int cb = part; cb < BN / 32; cb += PARTS) {
                const uint32_t m = m0 + 32 * q + lane;
                uint32_t r[32];
                tmem_load32(tmem + ((32 * q) << 16) + b * BN + cb * 32, r);
                if (m >= g.M) continue;
                const uint32_t col = n0 + cb * 32;
                if (g.mode == 3) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        if (col + 4 * i < g.N) {
                            float4 x = dst[i];
                            x.x += __uint_as_float(r[4 * i]), x.y += __uint_as_float(r[4 * i + 1]), x.z += __uint_as_float(r[4 * i + 2]), x.w += __uint_as_float(r[4 * i + 3]);
                            dst[i] = x;
                        }
                } else if (g.mode == 0) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        if (col + 4 * i < g.N) dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                } else if (g.mode == 1 || g.mode == 5) {
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t h[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float f0 = __uint_as_float(r[8 * i + 2 * e]), f1 = __uint_as_float(r[8 * i + 2 * e + 1]);
                            if (g.mode == 5) f0 = gelu_erf_lean(f0), f1 = gelu_erf_lean(f1);
                            const __half2 x = __floats2half2_rn(f0, f1);
                            h[e] = *reinterpret_cast<const uint32_t*>(&x);
                        }
                        if (col + 8 * i < g.N) dst[i] = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                } else {
                    // columns (2j, 2j + 1) are (gate_j, up_j): gelu(gate) * up, 16 results per 32 columns
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(g.out) + (size_t)m * (g.N / 2) + col / 2);
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        uint32_t h[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float g0 = __uint_as_float(r[16 * i + 4 * e]), g1 = __uint_as_float(r[16 * i + 4 * e + 2]);
                            const float a0 = (g.mode == 2 ? gelu_tanh(g0) : gelu_erf_lean(g0)) * __uint_as_float(r[16 * i + 4 * e + 1]);
                            const float a1 = (g.mode == 2 ? gelu_tanh(g1) : gelu_erf_lean(g1)) * __uint_as_float(r[16 * i + 4 * e + 3]);
                            const __half2 x = __floats2half2_rn(a0, a1);
                            h[e] = *reinterpret_cast<const uint32_t*>(&x);
                        }
                        if (col + 16 * i < g.N) dst[i] = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_at_leader[b]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // neither block leaves while the other may still read its shared memory or signal its barriers
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(S::COLS) : "memory");
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

template <int WB, int BN>
int launch_pair(tb_context* ctx, const CUtensorMap& amap, const CUtensorMap& wmap, const Args& g, uint32_t tiles) {
    using S = Shape<BN>;
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<WB, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
        configured[ctx->gpu & 15] = true;
    }
    const uint32_t pairs = std::min(tiles, (uint32_t)ctx->sms / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs), cfg.blockDim = dim3(S::THREADS), cfg.dynamicSmemBytes = S::SMEM_BYTES, cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<WB, BN>, amap, wmap, g, ctx->status));
    return OK;
}

}  // namespace

// The shapes this schedule takes: whole 16-byte rows of codes, and none of gemm2.cu's extra output modes.
bool gemm_pair_supports(uint32_t N, uint32_t K, uint32_t wbits, int mode) { return K % BK == 0 && (K * wbits / 8) % 16 == 0 && N > 0 && mode >= 0 && mode <= 5; }

// `narrow` picks the tile of 128 weight rows (half the tensor memory) instead of 256.
int launch_gemm_pair(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                     uint32_t wbits, bool narrow) {
    EncodeTiled enc = encode_tiled();
    if (!enc) return fail(NO_DRIVER, "gemm: the driver does not export cuTensorMapEncodeTiled");
    const uint32_t bn = narrow ? 128u : 256u;
    CUtensorMap amap, wmap;
    {
        const cuuint64_t dims[2] = {K, M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {BK, BM}, elem[2] = {1, 1};
        const CUresult r = enc(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled (activations) failed (" + std::to_string((int)r) + ")");
    }
    {
        const cuuint64_t row = (cuuint64_t)K * wbits / 8;  // bytes of codes (or of f16 weights) per weight row
        const cuuint64_t dims[2] = {wbits == 16 ? (cuuint64_t)K : row, N};
        const cuuint64_t strides[1] = {row};
        const cuuint32_t box[2] = {(cuuint32_t)(wbits == 16 ? BK : BK * wbits / 8), bn / 2}, elem[2] = {1, 1};
        // f16 weights go straight into the operand stage: halves, 128-byte swizzle, like the activations
        const CUresult r = enc(&wmap, wbits == 16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(w), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, wbits == 16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled (codes) failed (" + std::to_string((int)r) + ")");
    }
    const uint32_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + bn - 1) / bn);
    const Args g{s, out, M, N, K, mode};
    if (wbits == 16) return narrow ? launch_pair<16, 128>(ctx, amap, wmap, g, tiles) : launch_pair<16, 256>(ctx, amap, wmap, g, tiles);
    if (wbits == 4) return narrow ? launch_pair<4, 128>(ctx, amap, wmap, g, tiles) : launch_pair<4, 256>(ctx, amap, wmap, g, tiles);
    return narrow ? launch_pair<8, 128>(ctx, amap, wmap, g, tiles) : launch_pair<8, 256>(ctx, amap, wmap, g, tiles);
}

}  // namespace tb
