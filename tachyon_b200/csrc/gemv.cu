// Q8-weight matrix-vector product for batch-1 decode: y = W x with W int8 [rows, cols] and one f16 scale per 32
// weights along a row.  Replaces the reference's gemv_q4 (crates/tachyon/src/ptx/gemv.rs:156-195) together with the
// small kernels the reference launches around it: the residual/RMS-norm step (norm_q8, ptx/mod.rs:404-511) runs as
// this kernel's prologue, GeGLU (geglu_q8, ptx/mod.rs:376-393) and the greedy pick (sample, ptx/sample.rs:387-417) as
// its epilogues.
//
// Structure (one persistent block per SM: 16 consumer warps + 1 producer warp):
//  * every block owns a contiguous range of rows, so its weights are one contiguous byte range; the producer streams it
//    through a ring of stages with one-dimensional bulk copies (cp.async.bulk) completing on mbarriers.  The weights do
//    not depend on the previous kernel, so the producer starts before griddepcontrol.wait; when it has issued its last
//    copy it asks the L2 to fetch the head of the next kernel's weights, so HBM keeps streaming across the boundary;
//  * the activation vector is split once per block, per group of 32 values, into three byte planes of a 23-bit
//    fixed-point number and a power-of-two multiplier, kept in shared memory and then in each warp's registers for
//    its 2048-wide segment: a weight byte costs 3/4 of a dp4a and no conversion.  Block sums are exact integers,
//    combined in f32 with the weight scale;
//  * a warp takes one row (two when cols == 2048, which also puts a gate/up pair in one warp); lanes reduce with
//    shuffles; warps that share a row (cols > 2048) meet on a named barrier.
#include "planes.cuh"

#include <algorithm>

namespace tb {

namespace {

constexpr int CONSUMERS = 16;   // consumer warps
constexpr int CTHREADS = CONSUMERS * 32;
constexpr int THREADS = CTHREADS + 32;
constexpr int SEG = 2048;       // columns one warp covers with its register-resident activation planes
constexpr int SMEM_LIMIT = 230000;

// Rows a warp takes per stage: two, whatever the width (both reduced in one round of five exchanges; with wider rows,
// half as many meetings of the warps that share them).
constexpr int rows_per_warp(int) { return 2; }
// Teams: with rows of 16384 columns the sixteen warps are two row pairs' worth.  Each pair of rows is then a stage of its
// own, and the two groups of eight warps take the stages in turn: one group's meeting and final sum overlap the other's
// products, and the stages are small enough (32 KiB) to be handed out evenly.  Otherwise all warps work on every stage.
constexpr int teams(int wpr) { return wpr == 8 ? 2 : 1; }
constexpr int stage_rows(int wpr) { return CONSUMERS / wpr / teams(wpr) * rows_per_warp(wpr); }
// wb: bits per weight, 8 (one f16 scale per 32) or 4 (the reference's Q4: two weights per byte, one scale per 64).
constexpr int stage_w(int wpr, int wb = 8) { return stage_rows(wpr) * wpr * SEG * wb / 8; }
constexpr int stage_s(int wpr, int wb = 8) { return stage_w(wpr, wb) / 16; }
constexpr int plane_bytes(int wpr) { return wpr * 64 * (96 + 4); }
constexpr int tail_bytes() { return 1024; }  // barriers, reduction slots, stage descriptors (Layout::FULL .. STAGE_CNT), padded
// The most stages a ring holds (a launch may ask for fewer: a short product then leaves the rest of the SM's shared memory
// to the kernels around it).
constexpr int stages(int wpr, int wb = 8) {
    const int n = (SMEM_LIMIT - plane_bytes(wpr) - tail_bytes()) / (stage_w(wpr, wb) + stage_s(wpr, wb));
    return n > 8 ? 8 : n;
}
constexpr int smem_bytes(int wpr, int wb, int nst) { return nst * (stage_w(wpr, wb) + stage_s(wpr, wb)) + plane_bytes(wpr) + tail_bytes(); }

// Shared-memory carve-up, in this order: planes (hi, mid, lo words, multipliers), barriers, reduction slots, stage
// descriptors, then the ring: per stage its weights and behind them its scales.
template <int WPR, int WB = 8>
struct Layout {
    static constexpr int NST_MAX = stages(WPR, WB);
    static constexpr int HI = 0;
    static constexpr int MID = HI + WPR * 64 * 32;
    static constexpr int LO = MID + WPR * 64 * 32;
    static constexpr int MUL = LO + WPR * 64 * 32;
    static constexpr int FULL = MUL + WPR * 64 * 4;
    static constexpr int EMPTY = FULL + 8 * 8;
    static constexpr int RED = EMPTY + 8 * 8;                 // float [2][CONSUMERS][2]
    static constexpr int BESTV = RED + 2 * 2 * CONSUMERS * 4;  // float [2 * CONSUMERS]
    static constexpr int BESTI = BESTV + 2 * CONSUMERS * 4;    // uint32 [2 * CONSUMERS]
    static constexpr int SUMS = BESTI + 2 * CONSUMERS * 4;     // float [CONSUMERS][4]
    static constexpr int STAGE_ROW = SUMS + 4 * CONSUMERS * 4;  // uint32 [8]: first row of the stage's rows
    static constexpr int STAGE_CNT = STAGE_ROW + 8 * 4;         // uint32 [8]: how many rows the stage holds; 0 ends the block's work
    static constexpr int RING = plane_bytes(WPR) + tail_bytes();
    static constexpr int STAGE = stage_w(WPR, WB) + stage_s(WPR, WB);  // a stage: stage_w bytes of weights, then stage_s of scales
    static_assert(STAGE_CNT + 8 * 4 <= RING, "the tail outgrew its bytes");
};

// Four consecutive activations -> one word of each plane.  The eight lanes that share a group of 32 agree on its
// exponent with three exchanges.
template <int WPR, int WB>
__device__ __forceinline__ void store_planes(uint8_t* raw, int idx, float v0, float v1, float v2, float v3) {
    using L = Layout<WPR, WB>;
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);  // biased exponent of the largest magnitude
    const bool zero = eb < 22u;                                  // below 2^-105: the group counts as zero
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);  // 2^(21 - e)
    const int x0 = __float2int_rn(v0 * sc), x1 = __float2int_rn(v1 * sc), x2 = __float2int_rn(v2 * sc), x3 = __float2int_rn(v3 * sc);
    reinterpret_cast<uint32_t*>(raw + L::HI)[idx] = pack_bytes(x0, x1, x2, x3, 0x0062);
    reinterpret_cast<uint32_t*>(raw + L::MID)[idx] = pack_bytes(x0, x1, x2, x3, 0x0051);
    reinterpret_cast<uint32_t*>(raw + L::LO)[idx] = pack_bytes(x0, x1, x2, x3, 0x0040);
    if ((idx & 7) == 0) reinterpret_cast<float*>(raw + L::MUL)[idx >> 3] = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);  // 2^(e - 21)
}

// The block-wide prologue: the 512 consumer threads turn the input vector into planes in shared memory, four
// consecutive values per thread and pass (coalesced), cols / 2048 passes.
template <int WPR, int XMODE, int WB>
__device__ __forceinline__ void build_planes(const GemvParams& p, uint8_t* raw, int t, const float4& nw1, const float4& nw2) {
    using L = Layout<WPR, WB>;
    if constexpr (XMODE == X_F16) {
#pragma unroll
        for (int j = 0; j < WPR; j++) {
            const int idx = j * CTHREADS + t;
            const uint2 u = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __half*>(p.x) + (size_t)idx * 4));
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            store_planes<WPR, WB>(raw, idx, a.x, a.y, b.x, b.y);
        }
    } else if constexpr (XMODE == X_F32) {
        float4 f[WPR];
#pragma unroll
        for (int j = 0; j < WPR; j++) f[j] = ld_cg_f4(static_cast<const float*>(p.x) + (size_t)(j * CTHREADS + t) * 4);
#pragma unroll
        for (int j = 0; j < WPR; j++) store_planes<WPR, WB>(raw, j * CTHREADS + t, f[j].x, f[j].y, f[j].z, f[j].w);
    } else if constexpr (XMODE == X_ATTN) {
        // The vector is attention's output, still split over the blocks that computed it: merge the splits' (maximum,
        // sum, unnormalised output) here, four dimensions per thread, with running-maximum rescaling
        // (crates/tachyon/src/ptx/attend.rs:371-405 does this in the attention kernel's last block).
        static_assert(XMODE != X_ATTN || WPR == 1, "the attention merge is built for 2048 columns");
        const uint32_t G = p.att_heads / p.att_kv, HD = attend_header(G), stride = HD + G * 256;
        const uint32_t head = (uint32_t)t / 64, g = head / G, hh = head % G, d0 = ((uint32_t)t * 4) % 256;
        const uint32_t pos = ld_cg_u(p.att_pos), n = min(pos + 1, p.att_window);
        uint32_t span = max((n + p.att_splits - 1) / p.att_splits, 16u);  // the split rule of the attention kernel
        if (span > 64u) span = (span + 63u) / 64u * 64u;
        // The attention kernel merges att_cluster neighbouring splits itself and leaves one entry for each such group.
        const uint32_t used = ((n + span - 1) / span + p.att_cluster - 1) / p.att_cluster;
        const float* base = p.att_partial + (size_t)g * p.att_splits * stride;
        // A warp's threads share a head.  Lane k fetches split k's maximum and sum, so the statistics of up to 32 splits
        // cost one trip to the L2; the outputs are fetched eight splits at a time, asked for before the statistics so
        // that both are in flight together.  The weights 2^(m_s - M) then go from lane to lane.
        const uint32_t lane = (uint32_t)t & 31u;
        float M = -INFINITY, Lsum = 0.0f;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t s0 = 0; s0 < used; s0 += 32) {
            const uint32_t nch = min(32u, used - s0);
            float wl = 0.0f;
            for (uint32_t b0 = 0; b0 < nch; b0 += 8) {
                float4 a[8];
#pragma unroll
                for (uint32_t k = 0; k < 8; k++)
                    if (b0 + k < nch) a[k] = ld_cg_f4(base + (size_t)(s0 + b0 + k) * stride + HD + hh * 256 + d0);
                if (b0 == 0) {
                    float ml = -INFINITY, ll = 0.0f;
                    if (lane < nch) {
                        const float* ps = base + (size_t)(s0 + lane) * stride;
                        ml = ld_cg_f(ps + hh), ll = ld_cg_f(ps + G + hh);
                    }
                    const float Mn = fmaxf(M, warp_max(ml)), c = exp2f(M - Mn);
                    wl = lane < nch ? exp2f(ml - Mn) : 0.0f;
                    Lsum = fmaf(Lsum, c, warp_sum(wl * ll));
                    o.x *= c, o.y *= c, o.z *= c, o.w *= c;
                    M = Mn;
                }
#pragma unroll
                for (uint32_t k = 0; k < 8; k++) {
                    if (b0 + k < nch) {
                        const float wt = __shfl_sync(0xffffffffu, wl, b0 + k);
                        o.x = fmaf(wt, a[k].x, o.x), o.y = fmaf(wt, a[k].y, o.y), o.z = fmaf(wt, a[k].z, o.z), o.w = fmaf(wt, a[k].w, o.w);
                    }
                }
            }
        }
        const float inv = 1.0f / Lsum;
        store_planes<WPR, WB>(raw, t, o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    } else {
        // Residual step and RMS-norm over the whole vector (cols == 2048, four values per thread).  One pass of sums, as
        // the reference does (ptx/mod.rs:24-30): sum y^2, sum h^2, sum h*a, sum a^2 with a = y*w1; mean(h'^2) follows.
        static_assert(XMODE != X_NORM || WPR == 1, "the norm prologue is built for 2048 columns");
        const size_t at = (size_t)t * 4;
        const float4 h = ld_cg_f4(p.h + at);
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float sy = 0.0f;
        if (p.yres != nullptr) {
            float4 y = ld_cg_f4(p.yres + at);
            if (p.yres2 != nullptr) {
                const float4 y2 = ld_cg_f4(p.yres2 + at);
                y.x += y2.x, y.y += y2.y, y.z += y2.z, y.w += y2.w;
            }
            const float4 w = nw1;
            a = make_float4(y.x * w.x, y.y * w.y, y.z * w.z, y.w * w.w);
            sy = y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
        }
        const float4 w2 = nw2;
        float sh = h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
        float sha = h.x * a.x + h.y * a.y + h.z * a.z + h.w * a.w;
        float sa = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
        float4* sums = reinterpret_cast<float4*>(raw + L::SUMS);
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
        const float hs = p.yres != nullptr ? p.hscale : 1.0f;  // without a residual the state passes through unscaled
        const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
        const float rh = p.w2 != nullptr ? rsqrtf(fmaxf(sq, 0.0f) / n + p.eps) : 1.0f;
        const float v0 = fmaf(a.x, ry, h.x) * hs, v1 = fmaf(a.y, ry, h.y) * hs, v2 = fmaf(a.z, ry, h.z) * hs, v3 = fmaf(a.w, ry, h.w) * hs;
        if (blockIdx.x == 0 && p.h_out != nullptr) *reinterpret_cast<float4*>(p.h_out + at) = make_float4(v0, v1, v2, v3);
        store_planes<WPR, WB>(raw, t, v0 * rh * w2.x, v1 * rh * w2.y, v2 * rh * w2.z, v3 * rh * w2.w);
    }
}

// Planes of block `b` from shared memory; `first` picks which 16-byte half lands in words 0..3 (it matches the
// order the lane loads the weights in, and spreads both loads over all banks).
template <int WPR, int WB>
__device__ __forceinline__ void fetch_planes(const uint8_t* raw, int b, int first, Planes& pl) {
    using L = Layout<WPR, WB>;
    const uint4* hi = reinterpret_cast<const uint4*>(raw + L::HI) + b * 2;
    const uint4* mid = reinterpret_cast<const uint4*>(raw + L::MID) + b * 2;
    const uint4* lo = reinterpret_cast<const uint4*>(raw + L::LO) + b * 2;
    const uint4 h0 = hi[first], h1 = hi[1 - first], m0 = mid[first], m1 = mid[1 - first], l0 = lo[first], l1 = lo[1 - first];
    pl.hi[0] = h0.x, pl.hi[1] = h0.y, pl.hi[2] = h0.z, pl.hi[3] = h0.w, pl.hi[4] = h1.x, pl.hi[5] = h1.y, pl.hi[6] = h1.z, pl.hi[7] = h1.w;
    pl.mid[0] = m0.x, pl.mid[1] = m0.y, pl.mid[2] = m0.z, pl.mid[3] = m0.w, pl.mid[4] = m1.x, pl.mid[5] = m1.y, pl.mid[6] = m1.z, pl.mid[7] = m1.w;
    pl.lo[0] = l0.x, pl.lo[1] = l0.y, pl.lo[2] = l0.z, pl.lo[3] = l0.w, pl.lo[4] = l1.x, pl.lo[5] = l1.y, pl.lo[6] = l1.z, pl.lo[7] = l1.w;
    pl.mul = reinterpret_cast<const float*>(raw + L::MUL)[b];
}

// The kernel's body.  Rows reach a block in one of two ways.  Static: a contiguous range, balanced to one row (small
// matrices, where every SM should get some rows).  Dynamic (p.next != nullptr): stages of ROWS rows are handed out by a
// counter in global memory, the first of each block by its index; blocks that start late or sit far from the memory
// they read take fewer stages, and nobody waits for a slowest block.  The counter and a second word counting finished blocks are zero between launches (the last block clears them).
template <int WPR, int XMODE, int EPI, int WB>
__device__ __forceinline__ void gemv_body(const GemvParams& p, uint32_t* status) {
    extern __shared__ __align__(128) uint8_t raw[];
    using L = Layout<WPR, WB>;
    const uint32_t NST = p.ring;  // stages of this launch's ring (1 .. L::NST_MAX)
    constexpr int RPW = rows_per_warp(WPR);
    constexpr int ROWS = stage_rows(WPR);
    constexpr int TEAMS = teams(WPR);
    constexpr int GPS = CONSUMERS / WPR / TEAMS;  // groups of warps (a group shares a pair of rows) that work on one stage
    constexpr int SW = stage_w(WPR, WB), SS = stage_s(WPR, WB);
    constexpr int GROUP = WB == 8 ? 32 : 64;  // weights per scale
    constexpr int UNIT = (EPI == EPI_GEGLU) ? 2 : 1;  // rows that stay in one block
    static_assert(EPI != EPI_GEGLU || RPW == 2, "a gate/up pair is the two rows of one warp");
    const uint32_t K = p.cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t units = p.rows / UNIT;
    const uint32_t r0 = static_cast<uint32_t>((uint64_t)units * blockIdx.x / gridDim.x) * UNIT;
    const uint32_t r1 = static_cast<uint32_t>((uint64_t)units * (blockIdx.x + 1) / gridDim.x) * UNIT;
    const uint32_t nst = (r1 - r0 + ROWS - 1) / ROWS;
    const bool dynamic = p.next != nullptr;
    const uint32_t nchunks = (p.rows + ROWS - 1) / ROWS;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + L::FULL);
    uint64_t* empty = reinterpret_cast<uint64_t*>(raw + L::EMPTY);
    volatile uint32_t* stage_row = reinterpret_cast<volatile uint32_t*>(raw + L::STAGE_ROW);
    volatile uint32_t* stage_cnt = reinterpret_cast<volatile uint32_t*>(raw + L::STAGE_CNT);

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < NST; i++) mbar_init(&full[i], 1), mbar_init(&empty[i], CONSUMERS / TEAMS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const unsigned long long wait_limit = p.wait_ns != 0 ? p.wait_ns : WAIT_LIMIT_NS;
    if (warp == CONSUMERS) {
        // Producer: one thread streams this block's rows.  Nothing it reads is written by another kernel.
        if (lane == 0 && !p.silent) {
            // This thread's release of the kernel behind this one (at once with p.early, else when the block's last copy is
            // known).  A block counts as having released its dependents once ALL of its threads have said so or have left, so
            // with the consumers silent this only ever matters at the block's end; measured on B200, consumers that also say so
            // at their start let the next kernels move in early but the step as a whole got no faster.
            bool released = p.early != 0;
            if (released) pdl_launch_dependents();
            // The stages after the last one (one for each team) carry a count of zero: the consumers stop there.
            uint32_t chunk = blockIdx.x;  // dynamic: the stage's number among all stages of the matrix
            int ends = 0;
            for (uint32_t i = 0;; i++) {
                const uint32_t s = i % NST;
                uint32_t row, here;
                if (dynamic) {
                    row = chunk * ROWS;
                    here = chunk < nchunks ? min((uint32_t)ROWS, p.rows - row) : 0u;
                } else {
                    row = r0 + i * ROWS;
                    here = i < nst ? min((uint32_t)ROWS, r1 - row) : 0u;
                }
                if (!released && (here == 0 || (!dynamic && i + 1 >= nst))) released = true, pdl_launch_dependents();
                if (i == NST) {
                    // The ring is full and the first stage is not yet free: what comes after the ring, and the head of the next
                    // large matrix, may as well wait in the L2.
                    for (uint32_t k = 0; k < p.l2_ahead; k++) {
                        const uint32_t c = dynamic ? (NST + k) * gridDim.x + blockIdx.x : 0u, far = dynamic ? c * ROWS : r0 + (i + k) * ROWS;
                        if (far < (dynamic ? p.rows : r1)) prefetch_rows_l2(p.w, p.s, far, min((uint32_t)ROWS, (dynamic ? p.rows : r1) - far), K * WB / 8, K / GROUP * 2);
                    }
                    prefetch_stages(p.pf, blockIdx.x);
                }
                if (i >= NST && !mbar_wait(&empty[s], ((i / NST) - 1) & 1, wait_limit)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                stage_row[s] = row, stage_cnt[s] = here;
                if (here == 0) {
                    mbar_arrive(&full[s]);  // nothing to copy: the phase completes on this arrival alone
                    if (++ends == TEAMS) break;
                    continue;
                }
                const uint32_t bw = here * (K * WB / 8), bs = here * (K / GROUP * 2);
                mbar_expect_tx(&full[s], bw + bs);
                bulk_load(raw + L::RING + s * L::STAGE, p.w + (size_t)row * (K * WB / 8), bw, &full[s]);
                bulk_load(raw + L::RING + s * L::STAGE + SW, p.s + (size_t)row * (K / GROUP), bs, &full[s]);
                // The next stage's number, from the counter (the block's first stage is the one with its own index, so that its
                // first copy does not wait for an atomic).  Once the ring is full the atomic is asked for here and first needed
                // after the wait for a free stage, which hides its trip to the L2; a block that starts late finds the counter
                // far along and takes little.
                if (dynamic) chunk = gridDim.x + atomicAdd(p.next, 1u);
            }
            if (dynamic && atomicAdd(p.next + 1, 1u) == gridDim.x - 1) p.next[0] = 0u, p.next[1] = 0u;  // every block has taken its last stage
            if (!released) pdl_launch_dependents();
            // Ask the L2 for what the next kernel's block with this index will stream first.
            prefetch_hint(p.pf, blockIdx.x, gridDim.x);
        }
        return;
    }

    // Consumers.  Everything below may read what the previous kernel wrote.
    // The norm weights are model constants: fetch them (often from HBM, once a step) before waiting for the previous
    // kernel rather than after.
    float4 nw1 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), nw2 = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if constexpr (XMODE == X_NORM) {
        if (p.yres != nullptr) nw1 = __ldg(reinterpret_cast<const float4*>(p.w1 + (size_t)threadIdx.x * 4));
        if (p.w2 != nullptr) nw2 = __ldg(reinterpret_cast<const float4*>(p.w2 + (size_t)threadIdx.x * 4));
    }
    unsigned long long* stamp = nullptr;
    if (p.stamps != nullptr && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) stamp = p.stamps + (blockIdx.x == 0 ? 0 : 4);
    if (stamp) stamp[0] = global_ns();
    pdl_wait();
    if (stamp) stamp[1] = global_ns();
    build_planes<WPR, XMODE, WB>(p, raw, threadIdx.x, nw1, nw2);
    named_bar_sync(1, CTHREADS);
    if (stamp) stamp[2] = global_ns();
    const int seg = warp % WPR;                          // the warp's column segment
    const int team = warp / WPR / GPS, grp = warp / WPR % GPS;  // which stages it takes, and its row pair within them
    // Which 16-byte half of its blocks the lane loads first (bank spread); four-bit weights are read in their order.
    const int first = WB == 8 ? (lane >> 2) & 1 : 0;
    Planes pl[2];
    fetch_planes<WPR, WB>(raw, seg * 64 + lane, first, pl[0]);
    fetch_planes<WPR, WB>(raw, seg * 64 + lane + 32, first, pl[1]);
    float sx[2] = {0.0f, 0.0f};  // four-bit weights are n - 8: the blocks' activation sums, taken eight times off
    if constexpr (WB == 4) sx[0] = plane_sum(pl[0]), sx[1] = plane_sum(pl[1]);

    float bestv = -INFINITY;
    uint32_t besti = 0xffffffffu;
    for (uint32_t i = team;; i += TEAMS) {
        const uint32_t s = i % NST;
        const bool ok = mbar_wait(&full[s], (i / NST) & 1, wait_limit);
        if (!ok) atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);  // the producer's copies never landed: treated as the end of the work
        const uint32_t here = ok ? stage_cnt[s] : 0u;
        // Warps that share rows leave the loop together, through their barrier below (one of them giving up a wait must
        // not leave the others at a barrier); a warp with rows of its own leaves here.
        if constexpr (WPR == 1) {
            if (here == 0) break;
        }
        const uint32_t first_row = stage_row[s], row_end = first_row + here;  // rows of this stage: [first_row, row_end)
        const uint32_t row = first_row + grp * RPW;  // the warp's first row of this stage
        float v[RPW];
#pragma unroll
        for (int j = 0; j < RPW; j++) {
            v[j] = 0.0f;
            if constexpr (WB == 4) {
                if (row + j < row_end) {
                    // The lane's two blocks of 32 columns are 16 bytes each: 32 lane and 1024 + 32 lane of the segment.
                    const uint8_t* wr = raw + L::RING + s * L::STAGE + (size_t)(grp * RPW + j) * (K / 2) + seg * (SEG / 2);
                    const __half* sr = reinterpret_cast<const __half*>(raw + L::RING + s * L::STAGE + SW) + (grp * RPW + j) * (K / 64) + seg * 32;
                    const uint4 w0 = *reinterpret_cast<const uint4*>(wr + lane * 16), w1 = *reinterpret_cast<const uint4*>(wr + 512 + lane * 16);
                    const float s0 = __half2float(sr[lane >> 1]) * pl[0].mul, s1 = __half2float(sr[16 + (lane >> 1)]) * pl[1].mul;
                    v[j] = fmaf(block_dot_q4(w1, pl[1], sx[1]), s1, block_dot_q4(w0, pl[0], sx[0]) * s0);
                }
            } else if (row + j < row_end) {
                const uint8_t* wr = raw + L::RING + s * L::STAGE + (size_t)(grp * RPW + j) * K + seg * SEG;
                const __half* sr = reinterpret_cast<const __half*>(raw + L::RING + s * L::STAGE + SW) + (grp * RPW + j) * (K / 32) + seg * 64;
                const uint4 a0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + first) * 16);
                const uint4 b0 = *reinterpret_cast<const uint4*>(wr + (2 * lane + 1 - first) * 16);
                const uint4 a1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + first) * 16);
                const uint4 b1 = *reinterpret_cast<const uint4*>(wr + 1024 + (2 * lane + 1 - first) * 16);
                const float s0 = __half2float(sr[lane]) * pl[0].mul, s1 = __half2float(sr[lane + 32]) * pl[1].mul;
                v[j] = fmaf(block_dot(a1, b1, pl[1]), s1, block_dot(a0, b0, pl[0]) * s0);
            }
        }
        __syncwarp();
        // Released also when it was an end marker: with a short ring the producer needs the stage again for the next team's.
        if (lane == 0 && ok) mbar_arrive(&empty[s]);
        float r;           // row total: in lane 0 (and, with two rows, the second row's in lane 16)
        uint32_t out_row;  // the row this lane would write
        if constexpr (RPW == 2) {
            // Both rows in five exchanges: the halves of the warp trade one value, then each half reduces its own.
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
            // The warps of a row pair meet: each leaves its two partial sums, the first of them adds them up in order.
            float* red = reinterpret_cast<float*>(raw + L::RED) + ((i / TEAMS) & 1) * CONSUMERS * 2;
            if ((lane & 15) == 0) red[warp * 2 + (lane >> 4)] = r;
            if (named_bar_or(2 + warp / WPR, WPR * 32, here == 0)) break;
            if (seg != 0) continue;
            r = 0.0f;
#pragma unroll
            for (int j = 0; j < WPR; j++) r += red[(warp + j) * 2 + (lane >> 4)];
        }
        const bool writer = (EPI == EPI_GEGLU || RPW == 1) ? lane == 0 : (lane & 15) == 0;
        if (writer && out_row < row_end) {
            if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[out_row] = p.gelu_mul ? gelu_tanh(r) * __ldg(p.gelu_mul + out_row) : r;
            if constexpr (EPI == EPI_F16) static_cast<__half*>(p.y)[out_row] = __float2half_rn(r);
            if constexpr (EPI == EPI_GEGLU) static_cast<float*>(p.y)[out_row / 2] = r;
            if constexpr (EPI == EPI_ARGMAX) {
                if (p.y != nullptr) static_cast<float*>(p.y)[out_row] = r;
                if (r > bestv) bestv = r, besti = out_row;
            }
        }
    }

    if (stamp) stamp[3] = global_ns();
    if constexpr (EPI == EPI_ARGMAX) {
        // Largest value, lowest row among equals (ptx/sample.rs:91-97): the key orders by value, then by inverted row.
        float* sbv = reinterpret_cast<float*>(raw + L::BESTV);
        uint32_t* sbi = reinterpret_cast<uint32_t*>(raw + L::BESTI);
        if ((lane & 15) == 0) sbv[2 * warp + (lane >> 4)] = bestv, sbi[2 * warp + (lane >> 4)] = besti;
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

// The entry point.  At most 80 registers a thread (17 warps: 43,520 of the SM's 65,536), so that a block of the small
// kernel below fits beside one of these: the decode step keeps the next large product's block resident, its ring
// filling, while the short kernels before it run.
template <int WPR, int XMODE, int EPI, int WB = 8>
__global__ void __maxnreg__(80) gemv_q8_kernel(const GemvParams p, uint32_t* status) {
    gemv_body<WPR, XMODE, EPI, WB>(p, status);
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
        make_planes(v, pl);
        // Rows of a matrix whose width is not a multiple of 16 bytes... cols % 32 == 0, so 16-byte loads stay aligned.
        const uint4* wp = reinterpret_cast<const uint4*>(p.w + (size_t)row * p.cols + (size_t)b * 32);
        const uint4 a = __ldg(wp), c = __ldg(wp + 1);
        sum = fmaf(block_dot(a, c, pl), __half2float(p.s[(size_t)row * nb + b]) * pl.mul, sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) {
        if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[row] = p.gelu_mul ? gelu_tanh(sum) * __ldg(p.gelu_mul + row) : sum;
        else static_cast<__half*>(p.y)[row] = __float2half_rn(sum);
    }
}

// The same for four-bit weights (crates/tachyon/src/quant.rs:47-82: a scale per 64 along a row, so cols is a multiple of 64): the
// reference's 256-wide per-layer projections (decode.rs:654-660) and any other width the staged kernel does not take.
template <int XMODE, int EPI>
__global__ void __launch_bounds__(256) gemv_q4x_generic(const GemvParams p) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), nb = p.cols / 32;
    if (row >= p.rows) return;
    const uint8_t* wr = reinterpret_cast<const uint8_t*>(p.w) + (size_t)row * (p.cols / 2);
    float sum = 0.0f;
    for (uint32_t b = lane; b < nb; b += 32) {
        float v[32];
        if constexpr (XMODE == X_F16) load32_f16(static_cast<const __half*>(p.x) + (size_t)b * 32, v);
        else load32_f32(static_cast<const float*>(p.x) + (size_t)b * 32, v);
        Planes pl;
        make_planes(v, pl);
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(wr + (size_t)b * 16));
        sum = fmaf(block_dot_q4(w, pl, plane_sum(pl)), __half2float(p.s[(size_t)row * (nb / 2) + (b >> 1)]) * pl.mul, sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) {
        if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[row] = p.gelu_mul ? gelu_tanh(sum) * __ldg(p.gelu_mul + row) : sum;
        else static_cast<__half*>(p.y)[row] = __float2half_rn(sum);
    }
}

// ---- the small-footprint kernel ---------------------------------------------------------------------------------------
//
// For the short products of a decode step (query/key/value and output projections: a few megabytes over 148 blocks).
// A block of SMALL_WARPS warps takes up to 2 * SMALL_WARPS rows per pass of 2048 columns, straight from global memory
// into registers, no ring and ~7 KiB of shared memory, at most 80 registers a thread: it fits on an SM beside a block
// of the staged kernel.  It releases its dependents at once and loads its first pass of weights before it waits for the
// kernel in front of it, so a chain of such kernels is resident, weights in hand, before its input exists, and the large
// product behind the chain fills its ring while the chain runs.
constexpr int SMALL_WARPS = 8;
constexpr int SMALL_THREADS = SMALL_WARPS * 32;
constexpr int SMALL_ROWS = 2 * SMALL_WARPS;  // rows per pass

struct SmallSmem {
    uint32_t hi[512], mid[512], lo[512];  // planes of 2048 activations, a word per four
    float mul[64];
    float4 sums[SMALL_WARPS];
};

__device__ __forceinline__ void small_store_planes(SmallSmem& sm, int idx, float v0, float v1, float v2, float v3) {
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);
    const bool zero = eb < 22u;
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);
    const int x0 = __float2int_rn(v0 * sc), x1 = __float2int_rn(v1 * sc), x2 = __float2int_rn(v2 * sc), x3 = __float2int_rn(v3 * sc);
    sm.hi[idx] = pack_bytes(x0, x1, x2, x3, 0x0062);
    sm.mid[idx] = pack_bytes(x0, x1, x2, x3, 0x0051);
    sm.lo[idx] = pack_bytes(x0, x1, x2, x3, 0x0040);
    if ((idx & 7) == 0) sm.mul[idx >> 3] = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);
}

__device__ __forceinline__ void small_fetch_planes(const SmallSmem& sm, int b, Planes& pl) {
    const uint4 h0 = reinterpret_cast<const uint4*>(sm.hi)[2 * b], h1 = reinterpret_cast<const uint4*>(sm.hi)[2 * b + 1];
    const uint4 m0 = reinterpret_cast<const uint4*>(sm.mid)[2 * b], m1 = reinterpret_cast<const uint4*>(sm.mid)[2 * b + 1];
    const uint4 l0 = reinterpret_cast<const uint4*>(sm.lo)[2 * b], l1 = reinterpret_cast<const uint4*>(sm.lo)[2 * b + 1];
    pl.hi[0] = h0.x, pl.hi[1] = h0.y, pl.hi[2] = h0.z, pl.hi[3] = h0.w, pl.hi[4] = h1.x, pl.hi[5] = h1.y, pl.hi[6] = h1.z, pl.hi[7] = h1.w;
    pl.mid[0] = m0.x, pl.mid[1] = m0.y, pl.mid[2] = m0.z, pl.mid[3] = m0.w, pl.mid[4] = m1.x, pl.mid[5] = m1.y, pl.mid[6] = m1.z, pl.mid[7] = m1.w;
    pl.lo[0] = l0.x, pl.lo[1] = l0.y, pl.lo[2] = l0.z, pl.lo[3] = l0.w, pl.lo[4] = l1.x, pl.lo[5] = l1.y, pl.lo[6] = l1.z, pl.lo[7] = l1.w;
    pl.mul = sm.mul[b];
}

// A lane's share of two rows: blocks `lane` and `lane + 32` of each (two 16-byte pieces a block), and their scales.
struct SmallRows {
    uint4 w[2][4];
    float s[2][2];
};

__device__ __forceinline__ void small_load_rows(const GemvParams& p, uint32_t row, uint32_t r1, int lane, SmallRows& q) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (row + j < r1) {
            const uint4* wr = reinterpret_cast<const uint4*>(p.w + (size_t)(row + j) * SEG);
            q.w[j][0] = __ldcs(wr + 2 * lane), q.w[j][1] = __ldcs(wr + 2 * lane + 1);
            q.w[j][2] = __ldcs(wr + 64 + 2 * lane), q.w[j][3] = __ldcs(wr + 64 + 2 * lane + 1);
            const __half* sr = p.s + (size_t)(row + j) * (SEG / 32);
            q.s[j][0] = __half2float(__ldcs(sr + lane)), q.s[j][1] = __half2float(__ldcs(sr + lane + 32));
        } else {
            q.w[j][0] = q.w[j][1] = q.w[j][2] = q.w[j][3] = make_uint4(0u, 0u, 0u, 0u);
            q.s[j][0] = q.s[j][1] = 0.0f;
        }
    }
}

template <int XMODE>
__global__ void __launch_bounds__(SMALL_THREADS, 3) gemv_small_kernel(const GemvParams p) {
    __shared__ SmallSmem sm;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t r0 = static_cast<uint32_t>((uint64_t)p.rows * blockIdx.x / gridDim.x);
    const uint32_t r1 = static_cast<uint32_t>((uint64_t)p.rows * (blockIdx.x + 1) / gridDim.x);
    pdl_launch_dependents();  // whatever p.early says: this kernel exists to let the chain behind it start
    SmallRows q;
    small_load_rows(p, r0 + 2 * warp, r1, lane, q);
    // Later passes come through the L2 (asked for now) once the first pass is done with the registers.
    for (uint32_t row = r0 + SMALL_ROWS + 2 * warp; row < r1; row += SMALL_ROWS)
        for (uint32_t j = 0; j < 2 && row + j < r1; j++)
            for (int k = lane; k < SEG / 128; k += 32) prefetch_line_l2(p.w + (size_t)(row + j) * SEG + k * 128);
    unsigned long long* stamp = nullptr;
    if (p.stamps != nullptr && t == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) stamp = p.stamps + (blockIdx.x == 0 ? 0 : 4);
    if (stamp) stamp[0] = global_ns();
    pdl_wait();
    if (stamp) stamp[1] = global_ns();

    // The input vector as planes: virtual thread v of 512 takes values 4v .. 4v + 3; this block's threads take v = t, t + 256.
    if constexpr (XMODE == X_F32) {
        float4 f[2];
#pragma unroll
        for (int k = 0; k < 2; k++) f[k] = ld_cg_f4(static_cast<const float*>(p.x) + (size_t)(k * SMALL_THREADS + t) * 4);
#pragma unroll
        for (int k = 0; k < 2; k++) small_store_planes(sm, k * SMALL_THREADS + t, f[k].x, f[k].y, f[k].z, f[k].w);
    } else if constexpr (XMODE == X_NORM) {
        // The residual step and RMS-norm of gemv_body's prologue (ptx/mod.rs:24-30), two groups of four values a thread.
        float4 h[2], a[2], w2[2];
        float sy = 0.0f, sh = 0.0f, sha = 0.0f, sa = 0.0f;
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const size_t at = (size_t)(k * SMALL_THREADS + t) * 4;
            h[k] = ld_cg_f4(p.h + at);
            a[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (p.yres != nullptr) {
                float4 y = ld_cg_f4(p.yres + at);
                if (p.yres2 != nullptr) {
                    const float4 y2 = ld_cg_f4(p.yres2 + at);
                    y.x += y2.x, y.y += y2.y, y.z += y2.z, y.w += y2.w;
                }
                const float4 w = __ldg(reinterpret_cast<const float4*>(p.w1 + at));
                a[k] = make_float4(y.x * w.x, y.y * w.y, y.z * w.z, y.w * w.w);
                sy += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
            }
            w2[k] = p.w2 != nullptr ? __ldg(reinterpret_cast<const float4*>(p.w2 + at)) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            sh += h[k].x * h[k].x + h[k].y * h[k].y + h[k].z * h[k].z + h[k].w * h[k].w;
            sha += h[k].x * a[k].x + h[k].y * a[k].y + h[k].z * a[k].z + h[k].w * a[k].w;
            sa += a[k].x * a[k].x + a[k].y * a[k].y + a[k].z * a[k].z + a[k].w * a[k].w;
        }
        sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
        if (lane == 0) sm.sums[warp] = make_float4(sy, sh, sha, sa);
        __syncthreads();
        sy = sh = sha = sa = 0.0f;
#pragma unroll
        for (int k = 0; k < SMALL_WARPS; k++) {
            const float4 u = sm.sums[k];
            sy += u.x, sh += u.y, sha += u.z, sa += u.w;
        }
        const float n = static_cast<float>(p.cols);
        const float ry = p.yres != nullptr ? rsqrtf(sy / n + p.eps) : 0.0f;
        const float hs = p.yres != nullptr ? p.hscale : 1.0f;
        const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
        const float rh = p.w2 != nullptr ? rsqrtf(fmaxf(sq, 0.0f) / n + p.eps) : 1.0f;
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const float v0 = fmaf(a[k].x, ry, h[k].x) * hs, v1 = fmaf(a[k].y, ry, h[k].y) * hs, v2 = fmaf(a[k].z, ry, h[k].z) * hs, v3 = fmaf(a[k].w, ry, h[k].w) * hs;
            if (blockIdx.x == 0 && p.h_out != nullptr) *reinterpret_cast<float4*>(p.h_out + (size_t)(k * SMALL_THREADS + t) * 4) = make_float4(v0, v1, v2, v3);
            small_store_planes(sm, k * SMALL_THREADS + t, v0 * rh * w2[k].x, v1 * rh * w2[k].y, v2 * rh * w2[k].z, v3 * rh * w2[k].w);
        }
    } else {
        // X_ATTN: the vector is attention's output, left as one entry (maximum, sum, unnormalised output) per group of
        // att_cluster splits; merge the entries with running-maximum weights (ptx/attend.rs:371-405).
        const uint32_t G = p.att_heads / p.att_kv, HD = attend_header(G), stride = HD + G * 256;
        uint32_t entries = p.att_entries;
        if (entries == 0) {
            const uint32_t pos = ld_cg_u(p.att_pos), n = min(pos + 1, p.att_window);
            uint32_t span = max((n + p.att_splits - 1) / p.att_splits, 16u);  // the split rule of the attention kernel
            if (span > 64u) span = (span + 63u) / 64u * 64u;
            entries = ((n + span - 1) / span + p.att_cluster - 1) / p.att_cluster;
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const uint32_t v = k * SMALL_THREADS + t, head = v / 64, g = head / G, hh = head % G, d0 = (v * 4) % 256;
            const float* base = p.att_partial + (size_t)g * p.att_splits * stride;
            float M = -INFINITY, L = 0.0f;
            float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (uint32_t e0 = 0; e0 < entries; e0 += 4) {
                float4 acc[4];
                float m[4], l[4];
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    m[u] = -INFINITY, l[u] = 0.0f, acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (e0 + u < entries) {
                        const float* ps = base + (size_t)(e0 + u) * stride;
                        m[u] = ld_cg_f(ps + hh), l[u] = ld_cg_f(ps + G + hh), acc[u] = ld_cg_f4(ps + HD + hh * 256 + d0);
                    }
                }
                const float Mn = fmaxf(fmaxf(M, fmaxf(m[0], m[1])), fmaxf(m[2], m[3]));
                const float c = exp2f(M - Mn);  // 0 on the first trip (M = -inf)
                L *= c, o.x *= c, o.y *= c, o.z *= c, o.w *= c;
#pragma unroll
                for (uint32_t u = 0; u < 4; u++) {
                    const float wgt = e0 + u < entries ? exp2f(m[u] - Mn) : 0.0f;
                    L = fmaf(wgt, l[u], L);
                    o.x = fmaf(wgt, acc[u].x, o.x), o.y = fmaf(wgt, acc[u].y, o.y), o.z = fmaf(wgt, acc[u].z, o.z), o.w = fmaf(wgt, acc[u].w, o.w);
                }
                M = Mn;
            }
            const float inv = 1.0f / L;
            small_store_planes(sm, v, o.x * inv, o.y * inv, o.z * inv, o.w * inv);
        }
    }
    __syncthreads();
    if (stamp) stamp[2] = global_ns();

    for (uint32_t base_row = r0; base_row < r1; base_row += SMALL_ROWS) {
        const uint32_t row = base_row + 2 * warp;
        if (base_row != r0) small_load_rows(p, row, r1, lane, q);
        float v[2];
        {
            Planes pl;
            small_fetch_planes(sm, lane, pl);
            v[0] = block_dot(q.w[0][0], q.w[0][1], pl) * (q.s[0][0] * pl.mul);
            v[1] = block_dot(q.w[1][0], q.w[1][1], pl) * (q.s[1][0] * pl.mul);
            small_fetch_planes(sm, lane + 32, pl);
            v[0] = fmaf(block_dot(q.w[0][2], q.w[0][3], pl), q.s[0][1] * pl.mul, v[0]);
            v[1] = fmaf(block_dot(q.w[1][2], q.w[1][3], pl), q.s[1][1] * pl.mul, v[1]);
        }
        const bool upper = lane & 16;
        float r = (upper ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, upper ? v[0] : v[1], 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        const uint32_t out_row = row + (upper ? 1 : 0);
        if ((lane & 15) == 0 && out_row < r1) static_cast<float*>(p.y)[out_row] = r;
    }
    if (stamp) stamp[3] = global_ns();
}

// Whether the small kernel takes this product: eight-bit weights, 2048 columns, f32 out with no extras, and few enough
// rows a block that two passes cover them.
bool small_supports(const GemvParams& p, int sms) {
    if (p.wbits != 8 || p.cols != SEG || p.epi != EPI_F32 || p.gelu_mul != nullptr) return false;
    if (p.xmode != X_F32 && p.xmode != X_NORM && p.xmode != X_ATTN) return false;
    return p.rows <= (uint32_t)sms * 2 * SMALL_ROWS;
}

int launch_small(tb_context* ctx, const GemvParams& p) {
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {  // see launch_staged: the SM's split must leave room for the staged kernel's block
        TB_CUDA(cudaFuncSetAttribute(gemv_small_kernel<X_NORM>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        TB_CUDA(cudaFuncSetAttribute(gemv_small_kernel<X_ATTN>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        TB_CUDA(cudaFuncSetAttribute(gemv_small_kernel<X_F32>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        configured[ctx->gpu & 15] = true;
    }
    uint32_t grid = (uint32_t)ctx->sms;
    const uint32_t most = (p.rows + 1) / 2;
    if (grid > most) grid = most;
    const dim3 g(grid), b(SMALL_THREADS);
    if (p.xmode == X_NORM) TB_CUDA(launch_kernel(ctx, gemv_small_kernel<X_NORM>, g, b, 0, true, p));
    else if (p.xmode == X_ATTN) TB_CUDA(launch_kernel(ctx, gemv_small_kernel<X_ATTN>, g, b, 0, true, p));
    else TB_CUDA(launch_kernel(ctx, gemv_small_kernel<X_F32>, g, b, 0, true, p));
    return OK;
}

template <int WPR, int XMODE, int EPI, int WB = 8>
int launch_staged(tb_context* ctx, const GemvParams& p) {
    auto kernel = gemv_q8_kernel<WPR, XMODE, EPI, WB>;
    using L = Layout<WPR, WB>;
    static bool configured[16] = {};  // per device ordinal
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(WPR, WB, L::NST_MAX)));
        // Whatever a launch's ring needs, the SM is to be split with all it can give to shared memory: a block of another
        // kernel of the step must be able to move in beside this one, and an SM's split cannot change while blocks run on it.
        TB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        configured[ctx->gpu & 15] = true;
    }
    constexpr uint32_t ROWS = stage_rows(WPR);
    constexpr uint32_t UNIT = (EPI == EPI_GEGLU) ? 2 : 1;
    uint32_t grid = (uint32_t)ctx->sms;
    // Small matrices still spread over every SM (a block's stage is then partly empty): they are latency-bound.
    constexpr uint32_t LEAST = UNIT > (uint32_t)rows_per_warp(WPR) ? UNIT : (uint32_t)rows_per_warp(WPR);
    const uint32_t most = (p.rows + LEAST - 1) / LEAST;
    if (grid > most) grid = most > 0 ? most : 1;
    // Matrices of at least two stages a block hand their stages out through a counter; smaller ones are split evenly, and
    // their ring is only as long as a block's share.
    GemvParams q = p;
    q.ring = (uint32_t)L::NST_MAX;
    // (Four-bit stages hold half the bytes, so the counter's trip is paid twice per byte: measured slower there, 1.306 against
    // 1.262 ms a step.)
    if (ctx->dynamic && WB == 8 && (p.rows + ROWS - 1) / ROWS >= 2 * grid) {
        if (q.next == nullptr) q.next = ctx->sched + 2 * (ctx->sched_at++ % 64u);
    } else {
        q.next = nullptr;
        const uint32_t share = ((p.rows / UNIT + grid - 1) / grid) * UNIT;  // the most rows a block gets
        q.ring = std::max(1u, std::min((uint32_t)L::NST_MAX, (share + ROWS - 1) / ROWS));
    }
    TB_CUDA(launch_kernel(ctx, kernel, dim3(grid), dim3(THREADS), smem_bytes(WPR, WB, (int)q.ring), true, q, ctx->status));
    return OK;
}

// Four-bit weights: the combinations a decode step and the plain product use.
template <int WPR>
int dispatch_staged_q4(tb_context* ctx, const GemvParams& p) {
    if constexpr (WPR == 1) {
        if (p.xmode == X_NORM && p.epi == EPI_F32) return launch_staged<1, X_NORM, EPI_F32, 4>(ctx, p);
        if (p.xmode == X_NORM && p.epi == EPI_GEGLU) return launch_staged<1, X_NORM, EPI_GEGLU, 4>(ctx, p);
        if (p.xmode == X_NORM && p.epi == EPI_ARGMAX) return launch_staged<1, X_NORM, EPI_ARGMAX, 4>(ctx, p);
        if (p.xmode == X_ATTN && p.epi == EPI_F32) return launch_staged<1, X_ATTN, EPI_F32, 4>(ctx, p);
    }
    if (p.xmode == X_F32 && p.epi == EPI_F32) return launch_staged<WPR, X_F32, EPI_F32, 4>(ctx, p);
    if (p.xmode == X_F16 && p.epi == EPI_F32) return launch_staged<WPR, X_F16, EPI_F32, 4>(ctx, p);
    return fail(UNSUPPORTED, "gemv: no code path for this prologue and epilogue with four-bit weights");
}

template <int WPR>
int dispatch_staged(tb_context* ctx, const GemvParams& p) {
    if (p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX || p.xmode == X_NORM || p.xmode == X_ATTN) {
        if constexpr (WPR == 1) {
            if (p.xmode == X_NORM && p.epi == EPI_F32) return launch_staged<1, X_NORM, EPI_F32>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_F16) return launch_staged<1, X_NORM, EPI_F16>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_GEGLU) return launch_staged<1, X_NORM, EPI_GEGLU>(ctx, p);
            if (p.xmode == X_NORM && p.epi == EPI_ARGMAX) return launch_staged<1, X_NORM, EPI_ARGMAX>(ctx, p);
            if (p.xmode == X_ATTN && p.epi == EPI_F32) return launch_staged<1, X_ATTN, EPI_F32>(ctx, p);
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

size_t gemv_smem_bytes() { return smem_bytes(1, 8, stages(1)); }

uint32_t gemv_stage_rows(uint32_t cols) { return cols == 2048 ? stage_rows(1) : cols == 4096 ? stage_rows(2) : cols == 8192 ? stage_rows(4) : cols == 16384 ? stage_rows(8) : 0; }

int launch_gemv(tb_context* ctx, const GemvParams& p) {
    if (p.rows == 0 || p.cols == 0 || p.cols % 32 != 0) return fail(OUT_OF_RANGE, "gemv: cols must be a positive multiple of 32");
    if (p.w == nullptr || p.s == nullptr) return fail(OUT_OF_RANGE, "gemv: null weights");
    if ((reinterpret_cast<uintptr_t>(p.w) | reinterpret_cast<uintptr_t>(p.s)) & 15) return fail(OUT_OF_RANGE, "gemv: weights and scales must be 16-byte aligned");
    if (p.xmode == X_NORM) {
        if (p.h == nullptr || (p.yres != nullptr && p.w1 == nullptr)) return fail(OUT_OF_RANGE, "gemv: the norm prologue needs h, and w1 with y");
    } else if (p.xmode == X_ATTN) {
        if (p.att_partial == nullptr || p.att_pos == nullptr || p.att_kv == 0 || p.att_heads % p.att_kv != 0 || p.att_heads * 256 != p.cols)
            return fail(OUT_OF_RANGE, "gemv: the attention-merge prologue needs partials, a position and heads * 256 == cols");
    } else if (p.x == nullptr || (reinterpret_cast<uintptr_t>(p.x) & 15)) {
        return fail(OUT_OF_RANGE, "gemv: the input vector must be present and 16-byte aligned");
    }
    if (p.epi == EPI_GEGLU && p.rows % 2 != 0) return fail(OUT_OF_RANGE, "gemv: GeGLU needs an even number of rows");
    if (p.epi == EPI_ARGMAX && (p.best == nullptr || p.count == nullptr || p.state == nullptr)) return fail(OUT_OF_RANGE, "gemv: argmax needs best, count and state");
    if (p.epi != EPI_ARGMAX && p.y == nullptr) return fail(OUT_OF_RANGE, "gemv: null output");
    if (p.gelu_mul != nullptr && p.epi != EPI_F32) return fail(OUT_OF_RANGE, "gemv: the GELU-times-vector output is f32");
    if (p.wbits != 8 && p.wbits != 4) return fail(OUT_OF_RANGE, "gemv: weights are 8 or 4 bits");
    if (p.xmode == X_ATTN && p.att_cluster == 0) return fail(OUT_OF_RANGE, "gemv: att_cluster must be at least 1");
    if (((p.lean && ctx->lean) || ctx->lean == 2) && small_supports(p, ctx->sms)) return launch_small(ctx, p);
    if (p.wbits == 4) {
        switch (p.cols) {
            case 2048: return dispatch_staged_q4<1>(ctx, p);
            case 4096: return dispatch_staged_q4<2>(ctx, p);
            case 8192: return dispatch_staged_q4<4>(ctx, p);
            case 16384: return dispatch_staged_q4<8>(ctx, p);
            default: break;
        }
        if (p.cols % 64 != 0) return fail(OUT_OF_RANGE, "gemv: four-bit weights come in groups of 64 columns");
        if (p.xmode == X_NORM || p.xmode == X_ATTN || p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX) return fail(UNSUPPORTED, "gemv: fused prologue/epilogues need cols of 2048");
        const dim3 grid4((p.rows + 7) / 8), block4(256);
        if (p.xmode == X_F16 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q4x_generic<X_F16, EPI_F32>, grid4, block4, 0, true, p));
        else if (p.xmode == X_F16 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q4x_generic<X_F16, EPI_F16>, grid4, block4, 0, true, p));
        else if (p.xmode == X_F32 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q4x_generic<X_F32, EPI_F32>, grid4, block4, 0, true, p));
        else if (p.xmode == X_F32 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q4x_generic<X_F32, EPI_F16>, grid4, block4, 0, true, p));
        else return fail(UNSUPPORTED, "gemv: unknown input or output mode");
        return OK;
    }
    switch (p.cols) {
        case 2048: return dispatch_staged<1>(ctx, p);
        case 4096: return dispatch_staged<2>(ctx, p);
        case 8192: return dispatch_staged<4>(ctx, p);
        case 16384: return dispatch_staged<8>(ctx, p);
        default: break;
    }
    if (p.xmode == X_NORM || p.xmode == X_ATTN || p.epi == EPI_GEGLU || p.epi == EPI_ARGMAX) return fail(UNSUPPORTED, "gemv: fused prologue/epilogues need cols of 2048");
    const dim3 grid((p.rows + 7) / 8), block(256);
    if (p.xmode == X_F16 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F16, EPI_F32>, grid, block, 0, true, p));
    else if (p.xmode == X_F16 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F16, EPI_F16>, grid, block, 0, true, p));
    else if (p.xmode == X_F32 && p.epi == EPI_F32) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F32, EPI_F32>, grid, block, 0, true, p));
    else if (p.xmode == X_F32 && p.epi == EPI_F16) TB_CUDA(launch_kernel(ctx, gemv_q8_generic<X_F32, EPI_F16>, grid, block, 0, true, p));
    else return fail(UNSUPPORTED, "gemv: unknown input or output mode");
    return OK;
}

}  // namespace tb
