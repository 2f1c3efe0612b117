// Host-side declarations shared by the library's translation units: the context, launch descriptors of each
// kernel family, and error plumbing.  Nothing here is part of the C ABI (see include/tachyon_b200.h).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

struct tb_context {
    int gpu = 0;
    int sms = 0;
    cudaStream_t stream = nullptr;
    uint32_t* status = nullptr;       // device word: first kernel-side error (tb::ERR_*), 0 when fine
    uint32_t* status_host = nullptr;  // pinned mirror used by tb_status
    // Decoders take their device memory from this pool, which keeps what they free (cuda/mod.rs `alloc_pooled`: a model moved out
    // to make room leaves its VRAM in the pool for the next); tb_context_trim gives it back to the system.
    cudaMemPool_t pool = nullptr;
    bool pdl = true;                  // launch kernels with programmatic stream serialization
    bool prefetch = true;             // give kernels L2 hints about the next kernel's weights
    bool dynamic = true;              // large matrix-vector products hand their stages out through a counter (TACHYON_B200_STATIC=1: never)
    int lean = 1;                     // the small-footprint kernel for short products: 0 never (TACHYON_B200_NO_LEAN=1), 1 where the caller
                                      // marks a product as short (GemvParams::lean), 2 wherever the shape allows (tb_context_set_lean)
    bool early_trigger = true;        // kernels of a decode step release the kernel behind them as they start (TACHYON_B200_LATE_TRIGGER=1: when
                                      // their last copy is issued)
    bool lean_qkv = false;            // the query/key/value product also runs as the small kernel (TACHYON_B200_LEAN_QKV=1)
    uint32_t l2_ahead = 1;            // stages beyond its ring a large product asks the L2 for once the ring is full (TACHYON_B200_L2_AHEAD)
    uint32_t l2_next = 0;             // first stages of the next large product a block asks the L2 for at that point (TACHYON_B200_L2_NEXT)
    bool cluster = true;              // decode attention merges neighbouring splits in thread-block clusters (TACHYON_B200_NO_CLUSTER=1: never)
    uint32_t* sched = nullptr;        // device: 64 pairs of words (next stage, finished blocks) for such products launched outside a decoder
    uint32_t sched_at = 0;            // which pair the next launch takes
    bool attn_block = false;          // a decode layer's attention half as one kernel on clusters of 16 blocks where the layer has its shape (attn_block.cu: measured slower, so off); TACHYON_B200_ATTN_BLOCK=1, tb_context_set_attn_block
    bool gemm_walk = true;            // the one-tile product on f16 weights walks its tiles with one block an SM (gemm.cu); TACHYON_B200_GEMM_WALK=0
    bool gemm_red = true;             // the persistent product's += epilogue as reductions at the L2 (red.global.add.f32) instead of load, add, store; TACHYON_B200_GEMM_RED=0
    bool l2_side = false;             // decode: a side stream asks the L2 for a layer's down projection during the layer's short kernels (TACHYON_B200_L2_SIDE=1)
    bool flash_tc = true;             // prefill attention on tcgen05 where the shape allows (prefill_tc.cu); TACHYON_B200_FLASH=0, tb_context_set_flash
    int gemm_schedule = 0;            // 0: chosen by shape and epilogue; 1..4 force one (TACHYON_B200_GEMM at creation, tb_context_set_gemm_schedule)
};

namespace tb {

// Status codes of the C ABI (mirrors the reference's error enum, crates/tachyon/src/error.rs:8-50).
enum Status : int {
    OK = 0,
    NO_DRIVER = 1,
    UNSUPPORTED_GPU = 2,
    OUT_OF_RANGE = 3,
    CUDA = 4,
    FORMAT = 5,
    TOO_LONG = 6,
    OUT_OF_MEMORY = 7,
    NO_MODEL = 8,
    UNSUPPORTED = 9,
    DEVICE_WAIT = 10,
    IO = 11,
};

int fail(int status, const std::string& what);
// Device memory from the context's pool, in the order of its stream (falls back to cudaMalloc without a pool); and back.
cudaError_t pool_alloc(tb_context* ctx, void** out, size_t bytes);
void pool_free(tb_context* ctx, void* p);
int cuda_fail(cudaError_t e, const char* where);
#define TB_CUDA(call)                                             \
    do {                                                          \
        cudaError_t e_ = (call);                                  \
        if (e_ != cudaSuccess) return ::tb::cuda_fail(e_, #call); \
    } while (0)
#define TB_TRY(call)               \
    do {                           \
        int s_ = (call);           \
        if (s_ != ::tb::OK) return s_; \
    } while (0)

// ---- GEMV ------------------------------------------------------------------------------------------------
enum XMode : int { X_F16 = 0, X_F32 = 1, X_NORM = 2, X_ATTN = 3 };
enum Epilogue : int { EPI_F32 = 0, EPI_F16 = 1, EPI_GEGLU = 2, EPI_ARGMAX = 3 };

// A hint about the matrix a later kernel will stream: that kernel runs `grid` blocks, block b owning the rows
// [units*b/grid, units*(b+1)/grid) * unit with units = rows/unit.  A kernel given the hint asks the L2 for bytes
// [skip, skip + bytes) of each block's range (weights, and the matching scales) once its own loads are issued.
struct Prefetch {
    const int8_t* w = nullptr;
    const __half* s = nullptr;
    uint32_t rows = 0, cols = 0, unit = 1, grid = 1, skip = 0, bytes = 0;
    // The other form of the hint (stages > 0): the later kernel hands out stages of `stage_rows` rows, block b starting
    // with stages b, b + grid, ...; a block given the hint asks the L2 for the first `stages` of those of its own index,
    // row_bytes of weights and srow_bytes of scales a row, as soon as its own ring is full.
    uint32_t stage_rows = 0, stages = 0, row_bytes = 0, srow_bytes = 0;
};

struct GemvParams {
    const int8_t* w = nullptr;    // [rows, cols] codes
    const __half* s = nullptr;    // [rows, cols/32] scales
    uint32_t rows = 0, cols = 0;
    int xmode = X_F16;
    const void* x = nullptr;      // X_F16 / X_F32: the activation vector [cols]
    // X_NORM: x = w2 * rmsnorm(h'), h' = (h + w1 * rmsnorm(y)) * hscale (y may be null: h' = h; w2 may be null: x = h')
    const float* h = nullptr;
    const float* yres = nullptr;
    const float* yres2 = nullptr;  // X_NORM: a second partial product added to yres before anything else (attn_block.cu leaves two)
    const float* w1 = nullptr;
    const float* w2 = nullptr;
    float eps = 1e-6f, hscale = 1.0f;
    float* h_out = nullptr;       // receives h' (written by one block); may be null
    int epi = EPI_F32;
    void* y = nullptr;            // EPI_F32/F16: [rows]; EPI_GEGLU: f32 [rows/2]; EPI_ARGMAX: optional f32 logits [rows]
    const float* gelu_mul = nullptr;  // EPI_F32 only: y[r] = gelu_tanh(sum) * gelu_mul[r] (the per-layer input's gate, decode.rs:654-655)
    // EPI_ARGMAX: the pick is published through `best` (zero between launches) and `count` (zero between launches);
    // the last block writes state[1] = token, state[0] += 1, *token_out (may be null), and clears both.
    unsigned long long* best = nullptr;
    uint32_t* count = nullptr;
    uint32_t* state = nullptr;
    uint32_t* token_out = nullptr;
    uint32_t* trace = nullptr;    // optional: trace[position & trace_mask] = token
    uint32_t trace_mask = 0;
    uint32_t wbits = 8;           // 8: int8 codes, an f16 scale per 32; 4: the reference's Q4, two per byte, a scale per 64
    Prefetch pf;                  // optional hint for the L2
    // Two device words, zero between launches, through which a large product hands out its stages (see gemv_body); null:
    // the launch takes a pair from the context's pool.  Launches that may overlap need pairs of their own.
    uint32_t* next = nullptr;
    // != 0: the product is short and the next kernel in the stream should start as early as possible: run it as the
    // small-footprint kernel (no ring, weights in registers, dependents released at once) when its shape allows.
    uint32_t lean = 0;
    uint32_t ring = 0;            // stages of the shared-memory ring (set by launch_gemv)
    // Self-test of the bounded waits (tb_selftest_wait): the producer posts nothing, so every consumer's wait for its first
    // stage runs out after wait_ns; the kernel must then leave ERR_WAIT_FULL in the status word and return like any other.
    uint32_t silent = 0;
    unsigned long long wait_ns = 0;  // 0: the usual two seconds
    uint32_t early = 0;           // != 0: release the kernel behind this one at once (it waits for this one before it reads anything of it)
    uint32_t l2_ahead = 0;        // stages past the ring to ask the L2 for once the ring is full
    // Optional timeline: 8 words; the first and the last block each leave %globaltimer at entry, after the wait for
    // the previous kernel, after the prologue and at the end.
    unsigned long long* stamps = nullptr;
    // X_ATTN: x is the attention output, merged here from the splits' partial results
    // (layout of AttendParams::partial): x[h*256 + d] = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s.
    const float* att_partial = nullptr;
    const uint32_t* att_pos = nullptr;
    uint32_t att_splits = 1, att_window = 1, att_heads = 8, att_kv = 2;
    uint32_t att_cluster = 1;     // splits merged per entry of att_partial by the attention kernel itself (AttendParams::cluster)
    uint32_t att_entries = 0;     // != 0: att_partial always holds this many entries a key-value head (one cluster covers the window): no need to read the position
};

int launch_gemv(tb_context* ctx, const GemvParams& p);
size_t gemv_smem_bytes();
uint32_t gemv_stage_rows(uint32_t cols);  // rows of a stage of launch_gemv's staged kernel at this width (0: no staged kernel)

// The same product with f16 weights [rows, cols] (gemv_f16.cu): prologues X_F16, X_F32, X_NORM; outputs EPI_F32, EPI_F16.
struct GemvF16Params {
    const __half* w = nullptr;
    uint32_t rows = 0, cols = 0;
    int xmode = X_F16;
    const void* x = nullptr;
    const float* h = nullptr;
    const float* yres = nullptr;
    const float* w1 = nullptr;
    const float* w2 = nullptr;
    float eps = 1e-6f, hscale = 1.0f;
    float* h_out = nullptr;
    int epi = EPI_F32;
    void* y = nullptr;
};
int launch_gemv_f16(tb_context* ctx, const GemvF16Params& p);

// ---- decode attention ----------------------------------------------------------------------------------------
struct AttendParams {
    const float* qkv = nullptr;    // [(heads + 2*kv_heads) * 256] f32: queries, then new keys, then new values
    const float* q_norm = nullptr; // [256] or null (plain mode: no norms)
    const float* k_norm = nullptr;
    const float* freq = nullptr;   // [128] RoPE frequencies or null (no rotation)
    const float* trig = nullptr;   // optional: [positions][256] = cos(pos * freq[0..127]) then sin(...), filled by launch_rope_table
                                   // with the arithmetic the kernel would use; saves the kernel four sincosf per lane
    __half* kc = nullptr;          // [kv_heads][cap][256]
    __half* vc = nullptr;
    const uint32_t* pos = nullptr; // device word: position of the new token
    uint32_t cap = 0, window = 0, fresh = 1, heads = 8, kv_heads = 2;
    float scale = 1.0f, eps = 1e-6f;
    float* partial = nullptr;      // scratch: kv_heads * splits * (2*group + group*256) floats
    uint32_t* count = nullptr;     // kv_heads words, zero between launches
    uint32_t splits = 1;           // blocks per kv head (upper bound on the split actually used)
    void* out = nullptr;           // [heads*256] f32 or f16
    int out_f16 = 0;               // 0: f32, 1: f16, 2: the reference's Q8 (out = i8 codes, out_pairs = [s, s * sum q] per 32)
    float* out_pairs = nullptr;
    Prefetch pf;                   // optional hint for the L2
    unsigned long long* stamps = nullptr;  // optional timeline, as in GemvParams (the third stamp stays zero)
    uint32_t defer = 0;            // != 0: every split only stores its partial; the product that follows merges them (X_ATTN)
    uint32_t early = 0;            // != 0: the position and the older cache rows are final before the previous kernel in the
                                   // stream started, so the first tile may be fetched ahead of griddepcontrol.wait
    uint32_t cluster = 1;          // > 1 (2, 4 or 8, dividing splits; needs defer): blocks of that many neighbouring splits form a
                                   // thread-block cluster and merge their results in distributed shared memory, leaving one entry of
                                   // `partial` per cluster (entry c of a key-value head = its splits c * cluster ...)
};
// An entry of `partial`: the maxima and the sums of the group's query heads, padded to whole 16-byte units so that the
// outputs behind them can be fetched four at a time, then group * 256 unnormalised outputs.
__host__ __device__ constexpr uint32_t attend_header(uint32_t group) { return (2 * group + 3) & ~3u; }
int launch_attend(tb_context* ctx, const AttendParams& p);
size_t attend_partial_floats(uint32_t heads, uint32_t kv_heads, uint32_t splits);
int launch_attend_512(tb_context* ctx, const AttendParams& p);  // heads of 512; up to 8 query heads per key-value head (attend512.cu)
int launch_attend_256_shared(tb_context* ctx, const AttendParams& p);  // heads of 256, the same simple kernel: 8 query heads per key-value head
int launch_attend_static(tb_context* ctx, AttendParams p);  // scratch inside the library; see attend.cu

// ---- the attention half of a decode layer as one kernel (attn_block.cu) ---------------------------------------
struct AttnBlockParams {
    // the residual step and RMS-norm in front of the product: GemvParams' X_NORM fields
    const float* h = nullptr;
    const float* yres = nullptr;   // or null: no residual step (the first layer)
    const float* w1 = nullptr;
    const float* w2 = nullptr;
    float hscale = 1.0f, eps = 1e-6f;
    float* h_out = nullptr;        // or null
    const int8_t* wqkv = nullptr;  // [3072][2048] codes: 8 query heads, 2 key heads, 2 value heads of 256
    const __half* sqkv = nullptr;  // [3072][64]
    const float* q_norm = nullptr; // [256]
    const float* k_norm = nullptr;
    const float* trig = nullptr;   // [positions][256]: cosines then sines (launch_rope_table)
    const uint32_t* pos = nullptr;
    __half* kc = nullptr;          // [2][cap][256]
    __half* vc = nullptr;
    uint32_t cap = 0, window = 0;
    float scale = 1.0f, head_eps = 1e-6f;
    const int8_t* wo = nullptr;    // [2048][2048]
    const __half* so = nullptr;    // [2048][64]
    float* y[2] = {nullptr, nullptr};  // f32 [2048] each: the output projection's partial products over the two groups' columns
    unsigned long long* stamps = nullptr;  // optional timeline, as in GemvParams
    uint32_t stamp_at = 0;         // what the third stamp marks: 0 the planes ready, 1 phase A done, 2 attention done, 3 the merge done
};
// Whether this GPU runs the kernel's two clusters of 16 blocks.
bool attn_block_available(tb_context* ctx);
int launch_attn_block(tb_context* ctx, const AttnBlockParams& p);

// ---- fused decode step ---------------------------------------------------------------------------------------
struct EmbedParams {
    const int8_t* w = nullptr;
    const __half* s = nullptr;
    const uint32_t* token = nullptr;
    uint32_t cols = 0;
    float scale = 1.0f;
    float* out = nullptr;
};
enum PhaseKind : int { PH_EMBED = 0, PH_GEMV = 1, PH_ATTEND = 2 };
// One phase of the fused step: the descriptor the stand-alone kernel of the same kind would be launched with.
struct StepPhase {
    int kind = PH_GEMV;
    EmbedParams e;
    GemvParams g;
    AttendParams a;
};
// Whether the fused step has a code path for this product (shape and fusion).
bool step_supports(const GemvParams& p);
// Launches the fused step over `n` phases (device array); `counter` is a device word the call zeroes first.
// `times` (optional): 2 * n * 4 device words for the first and last block's timeline.
// `state`: the device word holding the step's position.
int launch_step(tb_context* ctx, const StepPhase* phases, uint32_t n, uint32_t* counter, const uint32_t* state, unsigned long long* times = nullptr);

// ---- prefill GEMM (tensor cores) ------------------------------------------------------------------------------
// D[M, N] = A[M, K] (f16) x W[N, K]^T (Q8); mode 0: f32 out, 1: f16 out, 2: GeGLU of column pairs -> f16 [M, N/2].
// mode 6 (the per-layer input's gate in prefill): out f16 [M, N] = gelu_tanh(product) * mul[m * mul_stride + n].
int launch_gemm_q8(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                   uint32_t wbits = 8, const float* mul = nullptr, uint32_t mul_stride = 0, const float* bias = nullptr);

// out f16 [rows, cols] = code * scale exactly as the product's own conversion rounds it (gemm.cu); launch_gemm_q8 with wbits 16
// on the copy gives the product on the codes, with the weight tiles fetched by TMA instead of converted in the loop.
int launch_dequant_f16(tb_context* ctx, const int8_t* w, const __half* s, uint32_t rows, uint32_t cols, uint32_t wbits, __half* out);

// ---- prefill kernels around the GEMMs (prefill.cu) ---------------------------------------------------------------------
int launch_prefill_embed(tb_context* ctx, const int8_t* w, const __half* s, const uint32_t* tokens, uint32_t n, uint32_t cols, float scale, float* out,
                         uint32_t wbits = 8);
int launch_prefill_norm(tb_context* ctx, float* h, const float* y, const float* w1, const float* w2, uint32_t tokens, uint32_t n, float eps, float hscale,
                        __half* x);
int launch_prefill_qkv(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, __half* q_out, __half* kc, __half* vc,
                       uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float scale, uint32_t head_dim = 256);
// The same kernel over some of a token's rows (kv_256 / kv_512: the key and value rows; query_256 / query_512: the query
// rows), `stride` floats from token to token, the first position optionally from device memory; qscale multiplies the queries.
struct PrefillRows {
    uint32_t first = 0, count = 0, stride = 0;
    const uint32_t* pos = nullptr;
};
int launch_prefill_rows(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, __half* q_out, __half* kc, __half* vc,
                        uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float qscale, uint32_t head_dim,
                        const PrefillRows& rows);
// out: f16 (or f32 with out_f32) [tokens][heads * head_dim].  pos_dev: the first position from device memory instead of pos0;
// sscale: factor of the scores (1 when the queries already carry scale * log2(e)).
// The same on tcgen05 (prefill_tc.cu), for the shapes prefill_flash_tc_supports names.
bool prefill_flash_tc_supports(uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t cap);
int launch_prefill_flash_tc(tb_context* ctx, const __half* q, const __half* kc, const __half* vc, void* out, uint32_t tokens, uint32_t pos0, uint32_t cap,
                            uint32_t window, uint32_t heads, uint32_t kv_heads, const uint32_t* pos_dev, float sscale, int out_f32);
int launch_prefill_flash(tb_context* ctx, const __half* q, const __half* kc, const __half* vc, void* out, uint32_t tokens, uint32_t pos0, uint32_t cap,
                         uint32_t window, uint32_t heads, uint32_t kv_heads, uint32_t head_dim = 256, const uint32_t* pos_dev = nullptr, float sscale = 1.0f,
                         int out_f32 = 0);

// ---- small kernels ---------------------------------------------------------------------------------------------
int launch_embed_q8(tb_context* ctx, const int8_t* w, const __half* s, const uint32_t* token, uint32_t cols, float scale, float* out, uint32_t wbits = 8);
int launch_norm(tb_context* ctx, const float* h, const float* y, const float* w1, const float* w2, uint32_t n, float eps, float hscale,
                float* h_out, float* x_out);
int launch_sample(tb_context* ctx, const float* logits, uint32_t vocab, float softcap, float penalty, const uint32_t* seen,
                  const uint32_t* allowed, unsigned long long* best, uint32_t* count, uint32_t* state, uint32_t* seen_out, uint32_t* token_out);
int launch_topk(tb_context* ctx, const float* logits, uint32_t vocab, uint32_t k, uint32_t* idx, float* val, unsigned long long* scratch);
int launch_fill_codes(tb_context* ctx, uint64_t seed, uint64_t stream_id, int8_t* w, size_t n);
int launch_fill_scales(tb_context* ctx, uint64_t seed, uint64_t stream_id, __half* s, size_t n, float mul);
int launch_fill_gauss_f16(tb_context* ctx, uint64_t seed, uint64_t stream_id, __half* x, size_t n, float mul);
int launch_fill_uniform(tb_context* ctx, uint64_t seed, uint64_t stream_id, float* x, size_t n, float lo, float hi);
int launch_interleave_rows(tb_context* ctx, const void* src, void* dst, uint32_t half_rows, uint32_t row_bytes);

// The encoder's kernels by the reference's argument lists (enc_ref.cu, encoder.cu).  kind: 0 embed_f16, 1 add_rows, 2 add_rows_f16,
// 3 gather_rows.  window < 0: every key of the sequence.
int launch_quant_f16(tb_context* ctx, const __half* a, int8_t* q, float* s, uint32_t cols, uint32_t tokens);
int launch_norm_f16(tb_context* ctx, const float* x, const float* gamma, const float* beta, __half* a, float* xo, uint32_t h, float eps, uint32_t n);
int launch_rows(tb_context* ctx, int kind, const void* table, const uint32_t* idx, float* out, uint32_t h, uint32_t n);
int launch_gelu_f16(tb_context* ctx, const float* x, __half* out, uint32_t width, uint32_t len, uint32_t gated);
int launch_rope_f16(tb_context* ctx, __half* qkv, const float* table, const uint32_t* pos, uint32_t h, uint32_t d, uint32_t n);
int launch_gemm_q8e(tb_context* ctx, const int8_t* a, const int8_t* w, const float* bias, void* y, uint32_t rows, uint32_t cols, uint32_t tokens, uint32_t mode,
                    const float* sa, const float* sw);
// Heads of 64 on tcgen05 (enc_attend_tc.cu): tiles of up to 128 queries; `rows` is how many rows qkv holds.
bool enc_attend_tc_supports(uint32_t h, uint32_t d);
int launch_enc_attend_tc(tb_context* ctx, const __half* qkv, const uint32_t* tiles, __half* out, uint32_t h, int window, float scale, uint32_t ntiles,
                         uint32_t rows);
int launch_enc_attend(tb_context* ctx, const __half* qkv, const uint32_t* tiles, __half* out, uint32_t h, uint32_t d, int window, float scale, uint32_t ntiles);

// The reference's own formats (q4.cu): f32 -> Q8 codes and [s, s * sum q] pairs; Q4 weights x Q8 activations.
int launch_quant_q8(tb_context* ctx, const float* x, int8_t* q, float* s, uint32_t n);
int launch_geglu_q8(tb_context* ctx, const float* a, const float* b, int8_t* q, float* s, uint32_t n);
int launch_norm_q8(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* s, uint32_t len,
                   uint32_t chunks, float eps, float scale);
int launch_gemv_q4_narrow(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols);
int launch_embed_q4_rows(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const uint32_t* tokens, uint32_t rows, float* out, uint32_t cols, float scale);
int launch_gemv_q4(tb_context* ctx, const uint8_t* w, const uint16_t* scales, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols);

// The reference's prefill formats by its kernel names (q8p.cu): Q8P quantisers, the Q4 x Q8P product in column slices.
int launch_quant_q8p(tb_context* ctx, const float* x, int8_t* q, float* s, uint32_t len);
int launch_geglu_q8p(tb_context* ctx, const float* a, const float* b, int8_t* q, float* s, uint32_t len, uint32_t width, uint32_t sa, uint32_t sb, uint32_t so);
int launch_norm_q8p(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* s, uint32_t len,
                    uint32_t tokens, float eps, float scale);
int launch_gemm_q4_ref(tb_context* ctx, const uint8_t* w, const uint16_t* ws, const int8_t* q, const float* s, float* y, uint32_t rows, uint32_t cols,
                       uint32_t tokens, uint32_t slices);
int launch_sum_slices(tb_context* ctx, float* y, uint32_t len, uint32_t slices);

// The reference's sampler with draws (sample.cu); cfg: 40 bytes of device memory in the reference's Sampling layout.
int launch_sample_draw(tb_context* ctx, const float* logits, float* work, uint32_t vocab, const void* cfg, uint32_t* state, uint32_t* seen, uint32_t* out,
                       float* partial, uint32_t* count, uint32_t blocks, uint32_t* trace = nullptr, uint32_t trace_mask = 0);

// cos/sin of every (position, frequency): table [positions][256] for AttendParams::trig.
int launch_rope_table(tb_context* ctx, const float* freq, uint32_t positions, float* table);

// The same product on pairs of SMs (gemm3.cu, tcgen05 cta_group::2).
bool gemm_pair_supports(uint32_t N, uint32_t K, uint32_t wbits, int mode);
int launch_gemm_pair(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                     uint32_t wbits, bool narrow);
// The same product as a persistent kernel (gemm2.cu); launch_gemm_q8 validates and dispatches.
bool gemm_persistent_supports(uint32_t N, uint32_t K, uint32_t wbits);
// `rope` (mode 1 only): the outputs of weight rows below `cols` are rotated before they are stored: rows (2j, 2j + 1) of a
// head of `head` rows hold a pair, turned by (c, s) = table[pos[token] * head / 2 + j].  The caller has put a head's rows
// j and j + head / 2 side by side for it (the encoder's q and k rows).
struct GemmRope {
    const float2* table;
    const uint32_t* pos;
    uint32_t cols, head;
};
int launch_gemm_persistent(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                           uint32_t wbits, const float* mul = nullptr, uint32_t mul_stride = 0, const GemmRope* rope = nullptr);

// Launch helper: kernel launch with (optionally) the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(tb_context* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && ctx->pdl) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the grid's blocks grouped into thread-block clusters of `cluster` (1, 1, 1: none).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(tb_context* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, bool pdl, dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl && ctx->pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x, attr[n].val.clusterDim.y = cluster.y, attr[n].val.clusterDim.z = cluster.z;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace tb

// The file loader's way into a model (wpk.cu): a tensor that is copied to its place as it is may arrive in pieces.
struct tb_decoder;
struct tb_encoder;
extern "C" {
int tb_decoder_load_part(tb_decoder* dec, const char* name, size_t offset, const void* data, size_t bytes, size_t total);
int tb_decoder_loads_in_parts(tb_decoder* dec, const char* name);
int tb_encoder_load_part(tb_encoder* enc, const char* name, size_t offset, const void* data, size_t bytes, size_t total);
int tb_encoder_loads_in_parts(tb_encoder* enc, const char* name);
}
