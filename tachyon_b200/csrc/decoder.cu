// The decoder: buffers, the op list of one decode step, its capture into CUDA graphs and the calls that replay it.
// Host-side counterpart of crates/tachyon/src/model/decode.rs (layout 151-181, control 190-204, step 569-592,
// attention 603-618, mlp 631-662, record 525-528, step/start/next_token/stop 305-345) for a model without experts, with
// this build's Q8 weights or the reference's Q4.
//
// One step is 2 + 5 * layers launches:
//   embed -> per layer { qkv (norm prologue) -> attention -> o -> gate_up (residual + norm prologue, GeGLU epilogue) ->
//   down } -> LM head (residual + final norm prologue, greedy pick epilogue).
// With per-layer inputs (Config::per_layer, decode.rs:572-579, 650-660) three more launches open the step (the token's
// row of the per-layer table, the projection of the embedding, their normalised sum for every layer) and two close
// each layer (the gate: residual prologue, GELU times the layer's input; the projection back to the stream).
// The residual additions and every RMS-norm run inside the prologue of the product that consumes them; the token and
// the position live on the device (state = [position, token]) and are advanced by the last kernel, so steps chain
// without the host.
//
// Seeded synthetic models (tb_decoder_fill_random): tensor k of layer i uses generator stream 32*i + k with k =
// 0 qkv.w, 1 qkv.s, 2 o.w, 3 o.s, 4 gate_up.w, 5 gate_up.s (gate rows then up rows), 6 down.w, 7 down.s, 8 q_norm,
// 9 k_norm, 10 input_layernorm, 11 post_attention_layernorm, 12 pre_feedforward_layernorm,
// 13 post_feedforward_layernorm, 14 layer_scalar, 16 per_layer_gate.w, 17 .s, 18 per_layer_proj.w, 19 .s,
// 20 post_per_layer_input_norm; 2^20 embed.w, 2^20+1 embed.s, 2^20+2 norm, 2^20+4 embed_per_layer.w, +5 .s,
// 2^20+6 per_layer_proj.w, +7 .s, 2^20+8 per_layer_norm; caches 2^21 + 2*i (+1).
// Codes are uniform in [-127, 127], scales |N(0,1)|*0.02/127, norm weights uniform in [0.5, 1.5), q/k norm weights in
// [0.15, 0.35), layer scalars in [0.95, 1): a random network with smaller scalars forgets its residual stream within a
// few layers and amplifies rounding differences by five orders of magnitude over 35 layers, which would make any
// comparison with a second implementation meaningless.
#include "../../include/tachyon_b200.h"
#include "common.cuh"
#include "internal.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

using namespace tb;

namespace {

struct Mat {
    int8_t* w = nullptr;
    __half* s = nullptr;
    uint32_t rows = 0, cols = 0;
    uint32_t bits = 8;  // 8: int8 codes, an f16 scale per 32; 4: the reference's Q4 (quant.rs:47-82), a scale per 64
    __half* f16 = nullptr;  // prefill's copy of the matrix as f16 [rows, cols] (settings.prefill_copy), or null
    size_t code_bytes() const { return (size_t)rows * cols * bits / 8; }
    size_t scale_bytes() const { return (size_t)rows * (cols / (bits == 4 ? 64 : 32)) * 2; }
};

struct Layer {
    Mat qkv, o, gate_up, down;
    Mat pl_gate, pl_proj;          // per-layer input: gate [per_layer, hidden], projection [hidden, per_layer]
    float* post_pl = nullptr;      // post_per_layer_input_norm
    float *q_norm = nullptr, *k_norm = nullptr, *input_ln = nullptr, *post_attn = nullptr, *pre_ffn = nullptr, *post_ffn = nullptr;
    float layer_scalar = 1.0f;
    bool global = false;
    int source = -1;  // >= 0: this layer projects no keys or values and attends over that layer's cache
    __half *kc = nullptr, *vc = nullptr;
    uint32_t cap = 0, window = 0, splits = 1;
    uint32_t cluster = 1;  // splits the attention kernel merges in a thread-block cluster before the output projection sees them
    uint32_t dim = 256, kvh = 0;  // head size and key-value heads of this layer's kind (Config::head_dim, Config::kv_heads)
    uint32_t nq = 0, nkv = 0;      // heads * dim, kvh * dim
};

constexpr uint32_t TRACE = 1u << 16;  // tokens remembered by position (a power of two)

}  // namespace

struct tb_decoder {
    tb_context* ctx = nullptr;
    tb_config cfg = {};
    tb_settings settings = {};
    std::vector<uint8_t> global;
    std::vector<Layer> layers;
    Mat embed;
    float* norm = nullptr;
    // Per-layer inputs (Config::per_layer > 0): the table [vocab, layers * per_layer], the projection of the embedding
    // [layers * per_layer, hidden], the norm weights [per_layer]; and the step's buffers for them.
    Mat embed_pl, pl_model_proj;
    float *pl_norm = nullptr, *ple = nullptr, *proj = nullptr, *pli = nullptr, *g2 = nullptr;
    float *pf_ple = nullptr, *pf_proj = nullptr, *pf_pli = nullptr;  // prefill: [chunk][layers * per_layer]: table rows, projections, inputs
    __half* pf_g2 = nullptr;                      // prefill: [chunk][per_layer]
    char* arena = nullptr;
    // settings.prefill_copy: the layers' four large matrices once more as f16, which prefill's products on 256 tokens and more
    // read by TMA instead of converting codes in their loop; decode keeps reading the codes.  Rewritten from the codes when
    // a tensor was loaded since (copy_valid).
    __half* copy = nullptr;
    bool copy_valid = false;
    // A resumed decoder keeps the pinned copy its weights came from (Decoder::shadow_bytes, decode.rs:275-290): parking it again
    // then costs no copy.  Dropped when a tensor is loaded (the copy would be stale) or by tb_decoder_drop_shadow.
    char* shadow = nullptr;
    size_t shadow_bytes = 0;
    cudaEvent_t weights_ready = nullptr;  // while resuming: the weights' copy on its own stream; what reads them for keeps waits for it
    char* host_table = nullptr;  // settings.host_table: the per-layer table, codes then scales, in pinned mapped host memory
    size_t arena_bytes = 0;
    // step buffers
    float *x[2] = {nullptr, nullptr}, *qkv = nullptr, *att = nullptr, *y = nullptr, *g = nullptr, *logits = nullptr, *partial = nullptr;
    float* y2 = nullptr;  // the output projection's second partial product when a layer's attention half runs as one kernel (attn_block.cu)
    uint32_t step_count = 0;  // launches of a step, counted when it was last recorded
    float* freq[2] = {nullptr, nullptr};
    float* trig[2] = {nullptr, nullptr};  // cos/sin of every position for the two frequency sets: [context][256]
    uint32_t *count = nullptr, *state = nullptr, *trace = nullptr;
    uint32_t* sched = nullptr;  // a pair of words per launch of a step: the stage counters of the large products (GemvParams::next)
    unsigned long long* best = nullptr;
    uint32_t* words = nullptr;  // pinned host: [0], [1] the tokens the two graphs write; [2] staging for the token fed in
    cudaGraphExec_t graphs[2] = {nullptr, nullptr};
    // The same step ending in logits + the sampler kernel instead of the fused greedy pick; used while the settings ask
    // for more than the plain largest logit.  The sampler reads its settings from `sampling` on the device.
    cudaGraphExec_t graphs_sampled[2] = {nullptr, nullptr};
    bool sampled = false;       // which pair the next step replays
    bool capture_sampled = false;  // which op list step_ops is recording
    void* sampling = nullptr;   // 40 bytes, ptx/sample.rs:38-78
    float* work = nullptr;      // the sampler's transformed logits
    uint32_t* seen = nullptr;   // bitmap of the tokens generated since the last reset
    float* sample_partial = nullptr;
    uint32_t* sample_count = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    // ctx->l2_side: a second stream on which a small kernel asks the L2 for a layer's down projection while the layer's short
    // kernels run (HBM has nothing else to do then); forked from and joined to the step's stream inside the recorded graph.
    cudaStream_t side = nullptr;
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
    int at = 0;
    bool running = false, built = false;
    uint32_t pos = 0;  // host mirror of the position
    uint32_t launches = 0;
    int final_x = 0;  // which of x[0], x[1] holds the hidden state after the last layer
    // Prefill chunk buffers (settings.chunk tokens): ids, residual stream, f16 GEMM inputs, projections.
    uint32_t* pf_tokens = nullptr;
    float *pf_h = nullptr, *pf_qkv = nullptr, *pf_y = nullptr;
    __half *pf_x = nullptr, *pf_q = nullptr, *pf_att = nullptr, *pf_g = nullptr;
    // The fused step: per graph, the phase table on the device; the grid barrier's counter.
    StepPhase* phase_dev[2] = {nullptr, nullptr};
    uint32_t phase_count = 0;
    uint32_t* grid_counter = nullptr;
    bool fused = false;
    std::vector<StepPhase>* collect = nullptr;  // when set, step_ops records descriptors instead of launching
    unsigned long long* stamps = nullptr;       // when set, launch number i of step_ops stamps its timeline at stamps + 8 * i
    float embed_scale = 1.0f;
};

namespace {

// Head size and key-value heads of the two kinds of layer (0 sliding, 1 global): Config::head_dim, Config::kv_heads.
uint32_t dim_of(const tb_config& c, int kind) { return kind && c.global_head_dim ? c.global_head_dim : c.head_dim; }
uint32_t kvh_of(const tb_config& c, int kind) { return kind && c.global_kv_heads ? c.global_kv_heads : c.kv_heads; }
uint32_t max_nq(const tb_config& c) { return c.heads * std::max(dim_of(c, 0), dim_of(c, 1)); }
uint32_t max_nkv(const tb_config& c) { return std::max(kvh_of(c, 0) * dim_of(c, 0), kvh_of(c, 1) * dim_of(c, 1)); }

float bf16_round(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    b = (b + 0x7fffu + ((b >> 16) & 1u)) & 0xffff0000u;
    memcpy(&v, &b, 4);
    return v;
}

// crates/tachyon/src/ptx/attend.rs:62-65
std::vector<float> rope_freq(float theta, uint32_t d, float fraction) {
    std::vector<float> f(d / 2);
    const uint32_t turned = (uint32_t)(fraction * (float)(d / 2));
    for (uint32_t i = 0; i < d / 2; i++) f[i] = i < turned ? powf(theta, -((float)(2 * i)) / (float)d) : 0.0f;
    return f;
}

int validate(const tb_config& c, const tb_settings& s) {
    if (c.hidden != 2048) return fail(UNSUPPORTED, "decoder: hidden must be 2048 (the width the fused norm prologue is built for)");
    if (c.head_dim != 256) return fail(UNSUPPORTED, "decoder: head_dim must be 256");
    if (c.global_head_dim != 0 && c.global_head_dim != 256 && c.global_head_dim != 512) return fail(UNSUPPORTED, "decoder: global_head_dim must be 256 or 512");
    if (c.global_head_dim == 512 && s.fused) return fail(UNSUPPORTED, "decoder: the single-kernel step has no attention for heads of 512");
    for (int kind = 0; kind < 2; kind++) {
        const uint32_t kvh = kvh_of(c, kind);
        if (c.heads == 0 || kvh == 0 || c.heads % kvh != 0) return fail(UNSUPPORTED, "decoder: heads must be a multiple of kv_heads");
        const uint32_t group = c.heads / kvh;
        if (group != 1 && group != 2 && group != 4 && group != 8) return fail(UNSUPPORTED, "decoder: 1, 2, 4 or 8 query heads per key-value head");
        if (group == 8 && s.fused) return fail(UNSUPPORTED, "decoder: the single-kernel step has no attention for eight query heads to a key-value head");
    }
    const uint32_t qcols = c.heads * c.head_dim;
    if (qcols != 2048 && qcols != 4096 && qcols != 8192 && qcols != 16384 && qcols % 32 != 0) return fail(UNSUPPORTED, "decoder: heads*head_dim must be a multiple of 32");
    if (c.global_head_dim == 512) {
        const uint32_t wide = c.heads * 512;
        if (wide != 2048 && wide != 4096 && wide != 8192 && wide != 16384) return fail(UNSUPPORTED, "decoder: heads*512 must be 2048, 4096, 8192 or 16384");
    }
    if (c.ffn == 0 || c.ffn % 32 != 0) return fail(UNSUPPORTED, "decoder: ffn must be a multiple of 32");
    if (c.per_layer != 0) {
        if (c.per_layer % 256 != 0 || c.per_layer > 6144) return fail(UNSUPPORTED, "decoder: per_layer must be a multiple of 256 up to 6144");
        if (s.fused) return fail(UNSUPPORTED, "decoder: the single-kernel step has no per-layer inputs");
    }
    if (c.layers == 0 || c.vocab == 0 || c.window == 0) return fail(OUT_OF_RANGE, "decoder: empty model");
    if (s.context == 0 || s.context > TRACE) return fail(OUT_OF_RANGE, "decoder: context must be in 1..65536");
    if (c.shared >= c.layers) return fail(OUT_OF_RANGE, "decoder: at least one layer must own its cache");
    if (s.weight_bits != 0 && s.weight_bits != 8 && s.weight_bits != 4) return fail(OUT_OF_RANGE, "decoder: weights are 8 or 4 bits");
    if (s.weight_bits == 4) {
        const uint32_t qc = c.heads * c.head_dim;
        if ((qc != 2048 && qc != 4096 && qc != 8192 && qc != 16384) || (c.ffn != 2048 && c.ffn != 4096 && c.ffn != 8192 && c.ffn != 16384))
            return fail(UNSUPPORTED, "decoder: four-bit weights need heads*head_dim and ffn of 2048, 4096, 8192 or 16384");
        if (s.fused) return fail(UNSUPPORTED, "decoder: the fused step reads eight-bit weights only");
    }
    return OK;
}

struct Taker {
    size_t end = 0;
    size_t take(size_t bytes) {
        const size_t at = end;
        end += (bytes + 255) / 256 * 256;
        return at;
    }
};

// Lays everything out from offset 0 (the reference's `layout`, decode.rs:151-181); with base == nullptr only sizes it.
void layout(tb_decoder* d, char* base) {
    const tb_config& c = d->cfg;
    Taker t;
    auto mat = [&](Mat& m, uint32_t rows, uint32_t cols) {
        m.rows = rows, m.cols = cols, m.bits = d->settings.weight_bits == 4 ? 4 : 8;
        m.w = reinterpret_cast<int8_t*>(base + t.take(m.code_bytes()));
        m.s = reinterpret_cast<__half*>(base + t.take(m.scale_bytes()));
    };
    auto vec = [&](float*& v, size_t n) { v = reinterpret_cast<float*>(base + t.take(n * 4)); };
    mat(d->embed, c.vocab, c.hidden);
    vec(d->norm, c.hidden);
    const uint32_t pl = c.per_layer, plw = c.per_layer * c.layers;
    if (pl) {
        if (d->settings.host_table) {
            // The table stays in pinned, mapped host memory (the reference's host.wpk, decode.rs:477-483): a step reads its
            // token's row from there.  One allocation, codes then scales, made by tb_decoder_open.
            d->embed_pl.rows = c.vocab, d->embed_pl.cols = plw, d->embed_pl.bits = d->settings.weight_bits == 4 ? 4 : 8;
            d->embed_pl.w = reinterpret_cast<int8_t*>(d->host_table);
            d->embed_pl.s = reinterpret_cast<__half*>(d->host_table + (d->embed_pl.code_bytes() + 255) / 256 * 256);
        } else {
            mat(d->embed_pl, c.vocab, plw);
        }
        mat(d->pl_model_proj, plw, c.hidden), vec(d->pl_norm, pl);
    }
    uint32_t max_splits = 1;
    for (uint32_t i = 0; i < c.layers; i++) {
        Layer& L = d->layers[i];
        L.global = d->global[i] != 0;
        // Config::source (model/mod.rs:138-143): a shared layer reuses the last unshared layer of its kind.
        L.source = -1;
        const uint32_t first_shared = c.layers - c.shared;
        if (i >= first_shared)
            for (int j = (int)first_shared - 1; j >= 0; j--)
                if ((d->global[j] != 0) == L.global) {
                    L.source = j;
                    break;
                }
        L.dim = dim_of(c, L.global), L.kvh = kvh_of(c, L.global), L.nq = c.heads * L.dim, L.nkv = L.kvh * L.dim;
        mat(L.qkv, L.nq + (L.source < 0 ? 2 * L.nkv : 0), c.hidden);
        mat(L.o, c.hidden, L.nq);
        mat(L.gate_up, 2 * c.ffn, c.hidden);
        mat(L.down, c.hidden, c.ffn);
        vec(L.q_norm, L.dim), vec(L.k_norm, L.dim);
        vec(L.input_ln, c.hidden), vec(L.post_attn, c.hidden), vec(L.pre_ffn, c.hidden), vec(L.post_ffn, c.hidden);
        if (pl) mat(L.pl_gate, pl, c.hidden), mat(L.pl_proj, c.hidden, pl), vec(L.post_pl, c.hidden);
        // Caches: a global layer keeps `context` positions, a sliding one a ring of window + chunk (decode.rs:152).
        L.window = L.global ? d->settings.context : c.window;
        L.cap = L.global ? d->settings.context : c.window + d->settings.chunk;
        const size_t cache = (size_t)L.kvh * L.cap * L.dim * 2;
        if (L.source >= 0) {
            L.kc = d->layers[L.source].kc, L.vc = d->layers[L.source].vc;
        } else {
            L.kc = reinterpret_cast<__half*>(base + t.take(cache));
            L.vc = reinterpret_cast<__half*>(base + t.take(cache));
        }
        // Blocks per key-value head: spans of about 64 positions, sliding or global (a tile; measured at a context of 2048: 128 for the
        // global layers 1.3157 ms a step, 64 and 96 1.3052, 48 1.3298, 32 1.3641), within the machine.
        static const uint32_t span_global = getenv("TACHYON_B200_SPAN_GLOBAL") ? (uint32_t)atoi(getenv("TACHYON_B200_SPAN_GLOBAL")) : 64u;
        static const uint32_t span_sliding = getenv("TACHYON_B200_SPAN_SLIDING") ? (uint32_t)atoi(getenv("TACHYON_B200_SPAN_SLIDING")) : 64u;
        const uint32_t per = std::max(16u, L.global ? span_global : span_sliding);
        L.splits = (L.window + per - 1) / per;
        const uint32_t most = (uint32_t)(2 * d->ctx->sms) / L.kvh;
        if (L.splits > most) L.splits = most;
        if (L.splits == 0) L.splits = 1;
        // Neighbouring splits meet in a thread-block cluster (attend.cu's kernel, one launch per phase): eight where there
        // are that many, else the largest power of two that divides them.
        L.cluster = 1;
        if (d->ctx->cluster && !d->fused && L.dim == 256 && c.heads != 8 * L.kvh) {
            if (L.splits >= 8) L.splits = std::min((L.splits + 7) / 8 * 8, std::max(most / 8 * 8, 8u)), L.cluster = 8;
            else if (L.splits % 4 == 0) L.cluster = 4;
            else if (L.splits % 2 == 0) L.cluster = 2;
        }
        if (L.splits > max_splits) max_splits = L.splits;
    }
    vec(d->x[0], c.hidden), vec(d->x[1], c.hidden);
    vec(d->qkv, max_nq(c) + 2 * max_nkv(c)), vec(d->att, max_nq(c)), vec(d->y, c.hidden), vec(d->y2, c.hidden), vec(d->g, c.ffn);
    vec(d->logits, c.vocab);
    if (pl) vec(d->ple, plw), vec(d->proj, plw), vec(d->pli, plw), vec(d->g2, pl);
    vec(d->work, c.vocab);
    d->seen = reinterpret_cast<uint32_t*>(base + t.take(((size_t)c.vocab + 31) / 32 * 4));
    d->sampling = base + t.take(64);
    vec(d->sample_partial, (size_t)8 * 1024);
    d->sample_count = reinterpret_cast<uint32_t*>(base + t.take(4));
    // Attention scratch for the larger kind: per key-value head and split the maxima, sums and outputs of its query heads.
    vec(d->partial, (size_t)c.heads * max_splits * (4 + std::max(dim_of(c, 0), dim_of(c, 1))));  // at most attend_header(1) = 4 words a head ahead of its outputs
    vec(d->freq[0], dim_of(c, 0) / 2), vec(d->freq[1], dim_of(c, 1) / 2);
    vec(d->trig[0], (size_t)d->settings.context * 256), vec(d->trig[1], (size_t)d->settings.context * 256);  // heads of 256 only
    d->count = reinterpret_cast<uint32_t*>(base + t.take((size_t)c.heads * 4));
    d->state = reinterpret_cast<uint32_t*>(base + t.take(8));
    d->best = reinterpret_cast<unsigned long long*>(base + t.take(16));
    d->trace = reinterpret_cast<uint32_t*>(base + t.take((size_t)TRACE * 4));
    d->grid_counter = reinterpret_cast<uint32_t*>(base + t.take(4));
    d->sched = reinterpret_cast<uint32_t*>(base + t.take((size_t)(8 + 7 * c.layers) * 8));
    if (d->settings.chunk > 0) {
        const size_t T = d->settings.chunk;
        auto half = [&](__half*& v, size_t n) { v = reinterpret_cast<__half*>(base + t.take(n * 2)); };
        d->pf_tokens = reinterpret_cast<uint32_t*>(base + t.take(T * 4));
        vec(d->pf_h, T * c.hidden), vec(d->pf_qkv, T * (max_nq(c) + 2 * max_nkv(c))), vec(d->pf_y, T * c.hidden);
        half(d->pf_x, T * c.hidden), half(d->pf_q, T * max_nq(c)), half(d->pf_att, T * max_nq(c)), half(d->pf_g, T * c.ffn);
        if (pl) vec(d->pf_ple, T * plw), vec(d->pf_proj, T * plw), vec(d->pf_pli, T * plw), half(d->pf_g2, T * pl);
    }
    d->arena_bytes = t.end;
}

// Bytes of each block's range one L2 hint covers.  Off by default: on B200 the hints measured slower than no hints
// (560 against 663 tokens/s at 192 KiB); TACHYON_B200_PREFETCH_KB turns them on for experiments.
uint32_t prefetch_bytes() {
    static const uint32_t v = [] {
        const char* e = getenv("TACHYON_B200_PREFETCH_KB");
        return (uint32_t)(e ? atoi(e) : 0) * 1024u;
    }();
    return v;
}
#define PF prefetch_bytes()

Prefetch hint(tb_decoder* d, const Mat& m, uint32_t unit, uint32_t skip, uint32_t bytes) {
    Prefetch pf;
    if (!d->ctx->prefetch) return pf;
    pf.w = m.w, pf.s = m.s, pf.rows = m.rows, pf.cols = m.cols, pf.unit = unit, pf.grid = (uint32_t)d->ctx->sms, pf.skip = skip, pf.bytes = bytes;
    return pf;
}

// Asks the L2 for two byte ranges, a thread a piece of 16 KiB (a bulk prefetch: no destination, nothing waits for it).
__global__ void __launch_bounds__(128) l2_prefetch_kernel(const char* a, size_t an, const char* b, size_t bn) {
    constexpr size_t PIECE = 16384;
    const size_t i = (size_t)blockIdx.x * 128 + threadIdx.x, na = (an + PIECE - 1) / PIECE, nb = (bn + PIECE - 1) / PIECE;
    if (i < na) bulk_prefetch_l2(a + i * PIECE, (uint32_t)(an - i * PIECE < PIECE ? an - i * PIECE : PIECE));
    else if (i - na < nb) bulk_prefetch_l2(b + (i - na) * PIECE, (uint32_t)(bn - (i - na) * PIECE < PIECE ? bn - (i - na) * PIECE : PIECE));
}

// Forks the side stream off the step's stream at this point and has it ask the L2 for matrix m.
int side_prefetch(tb_decoder* d, const Mat& m) {
    cudaStream_t s = d->ctx->stream;
    TB_CUDA(cudaEventRecord(d->fork_ev, s));
    TB_CUDA(cudaStreamWaitEvent(d->side, d->fork_ev, 0));
    static const long cap_mb = getenv("TACHYON_B200_L2_SIDE_MB") ? atol(getenv("TACHYON_B200_L2_SIDE_MB")) : -1;  // experiment: how much of it
    size_t an = m.code_bytes(), bn = m.scale_bytes();
    if (cap_mb >= 0 && an > (size_t)cap_mb << 20) bn = bn * ((size_t)cap_mb << 20) / an / 16 * 16, an = (size_t)cap_mb << 20;
    const size_t pieces = (an + 16383) / 16384 + (bn + 16383) / 16384;
    if (pieces == 0) return OK;
    l2_prefetch_kernel<<<(unsigned)((pieces + 127) / 128), 128, 0, d->side>>>(reinterpret_cast<const char*>(m.w), an, reinterpret_cast<const char*>(m.s), bn);
    TB_CUDA(cudaGetLastError());
    return OK;
}

int gemv(tb_decoder* d, const Mat& m, GemvParams p) {
    p.w = m.w, p.s = m.s, p.rows = m.rows, p.cols = m.cols, p.wbits = m.bits;
    p.next = d->sched + 2 * (size_t)d->launches;  // a launch's own pair: neighbouring launches overlap
    p.early = d->ctx->early_trigger ? 1 : 0;
    if (d->stamps) p.stamps = d->stamps + 8 * (size_t)d->launches;
    d->launches++;
    if (d->collect) {
        if (!step_supports(p)) return fail(UNSUPPORTED, "fused step: no code path for this product");
        StepPhase ph;
        ph.kind = PH_GEMV, ph.g = p;
        d->collect->push_back(ph);
        return OK;
    }
    return launch_gemv(d->ctx, p);
}

// The op list of one step (decode.rs:569-592), launched on the context's stream.
int step_ops(tb_decoder* d, uint32_t* token_word) {
    const tb_config& c = d->cfg;
    d->launches = 0;
    int cur = 0;
    if (d->collect) {
        StepPhase ph;
        ph.kind = PH_EMBED;
        ph.e.w = d->embed.w, ph.e.s = d->embed.s, ph.e.token = d->state + 1, ph.e.cols = c.hidden, ph.e.scale = d->embed_scale, ph.e.out = d->x[0];
        d->collect->push_back(ph);
    } else {
        TB_TRY(launch_embed_q8(d->ctx, d->embed.w, d->embed.s, d->state + 1, c.hidden, d->embed_scale, d->x[0], d->embed.bits));
    }
    d->launches++;
    const uint32_t pl = c.per_layer;
    if (pl) {
        // decode.rs:572-579: the token's row of the per-layer table times sqrt(per_layer); the embedding through the
        // per-layer projection; then for every layer (row + w * rmsnorm(projection)) / sqrt(2), the projection's
        // 1 / sqrt(hidden) folded into eps (rmsnorm(c y) is rmsnorm(y) with eps / c^2).
        if (d->collect) return fail(UNSUPPORTED, "fused step: no per-layer inputs");
        TB_TRY(launch_embed_q8(d->ctx, d->embed_pl.w, d->embed_pl.s, d->state + 1, pl * c.layers, sqrtf((float)pl), d->ple, d->embed_pl.bits));
        d->launches++;
        GemvParams pp;
        pp.xmode = X_F32, pp.x = d->x[0], pp.epi = EPI_F32, pp.y = d->proj;
        TB_TRY(gemv(d, d->pl_model_proj, pp));
        TB_TRY(launch_norm_q8(d->ctx, d->ple, d->pli, d->proj, d->pl_norm, nullptr, nullptr, nullptr, pl, c.layers, c.eps * (float)c.hidden, 0.70710678118654752f));
        d->launches++;
    }
    for (uint32_t i = 0; i < c.layers; i++) {
        Layer& L = d->layers[i];
        const bool side = d->ctx->l2_side && d->side != nullptr && !d->collect && !d->fused && L.down.bits == 8;
        if (side) TB_TRY(side_prefetch(d, L.down));  // behind the kernel in front of this layer, beside the layer's short kernels
        // The attention half of the layer as one kernel on two clusters of 16 blocks (attn_block.cu), where the layer has its
        // shape: hidden 2048, 8 query and 2 key-value heads of 256 with a cache of their own, eight-bit matrices.
        const bool block = d->ctx->attn_block && !d->collect && !d->fused && c.hidden == 2048 && c.heads == 8 && L.kvh == 2 && L.dim == 256 && L.source < 0 &&
                           L.qkv.bits == 8 && L.o.bits == 8 && d->trig[L.global ? 1 : 0] != nullptr && attn_block_available(d->ctx);
        if (block) {
            AttnBlockParams b;
            b.h = d->x[cur], b.w2 = L.input_ln, b.eps = c.eps;
            if (i > 0) {
                const Layer& P = d->layers[i - 1];
                b.yres = d->y, b.w1 = pl ? P.post_pl : P.post_ffn, b.hscale = P.layer_scalar, b.h_out = d->x[1 - cur];
                cur = 1 - cur;
            }
            b.wqkv = L.qkv.w, b.sqkv = L.qkv.s, b.q_norm = L.q_norm, b.k_norm = L.k_norm, b.trig = d->trig[L.global ? 1 : 0], b.pos = d->state;
            b.kc = L.kc, b.vc = L.vc, b.cap = L.cap, b.window = L.window, b.scale = c.attn_scale, b.head_eps = c.eps;
            b.wo = L.o.w, b.so = L.o.s, b.y[0] = d->y, b.y[1] = d->y2;
            if (d->stamps) {
                const char* at = getenv("TACHYON_B200_ATTN_BLOCK_STAMP");
                b.stamps = d->stamps + 8 * (size_t)d->launches, b.stamp_at = at ? (uint32_t)atoi(at) : 0u;
            }
            TB_TRY(launch_attn_block(d->ctx, b));
            d->launches++;
        } else {
            GemvParams q;
            q.xmode = X_NORM, q.h = d->x[cur], q.w2 = L.input_ln, q.eps = c.eps;
            if (i > 0) {
                // The previous layer's closing residual: x = (x + post_ffn_norm(down)) * layer_scalar (decode.rs:631-662).
                const Layer& P = d->layers[i - 1];
                q.yres = d->y, q.w1 = pl ? P.post_pl : P.post_ffn, q.hscale = P.layer_scalar, q.h_out = d->x[1 - cur];
                cur = 1 - cur;
            }
            q.epi = EPI_F32, q.y = d->qkv;
            q.lean = d->ctx->lean_qkv ? 1 : 0;
            q.pf = hint(d, L.o, 1, 0, PF);  // what follows attention
            TB_TRY(gemv(d, L.qkv, q));

            AttendParams a;
            a.qkv = d->qkv, a.q_norm = L.q_norm, a.k_norm = L.k_norm, a.freq = d->freq[L.global ? 1 : 0], a.trig = d->trig[L.global ? 1 : 0];
            a.kc = L.kc, a.vc = L.vc, a.pos = d->state, a.cap = L.cap, a.window = L.window, a.fresh = L.source < 0 ? 1 : 0;
            a.heads = c.heads, a.kv_heads = L.kvh, a.scale = c.attn_scale, a.eps = c.eps;
            a.partial = d->partial, a.count = d->count, a.splits = L.splits, a.out = d->att, a.out_f16 = 0;
            a.pf = hint(d, L.gate_up, 2, 0, PF);
            // Heads of 512, or eight query heads to a key-value head: attend512.cu's kernel, which merges its own splits and writes f32 heads.
            const bool wide = L.dim == 512 || c.heads == 8 * L.kvh;
            a.defer = wide ? 0 : 1;  // the o projection merges the splits in its prologue
            // Caches and position are final long before the kernel in front of this one, except in a layer that reads another
            // layer's cache: that layer wrote the newest row during this very step, and with short products between the two
            // nothing but the order of the launches says it has finished.  Such a layer fetches nothing ahead of its wait.
            a.early = (!wide && L.source < 0) ? 1 : 0;
            a.cluster = wide ? 1 : L.cluster;
            if (wide) {
                if (d->collect) return fail(UNSUPPORTED, "fused step: no attention for this layer's heads");
                TB_TRY(L.dim == 512 ? launch_attend_512(d->ctx, a) : launch_attend_256_shared(d->ctx, a));
            } else if (d->collect) {
                StepPhase ph;
                ph.kind = PH_ATTEND, ph.a = a;
                d->collect->push_back(ph);
            } else {
                if (d->stamps) a.stamps = d->stamps + 8 * (size_t)d->launches;
                TB_TRY(launch_attend(d->ctx, a));
            }
            d->launches++;

            GemvParams o;
            o.xmode = X_F32, o.x = d->att, o.epi = EPI_F32, o.y = d->y;
            if (!wide) {
                o.xmode = X_ATTN, o.att_partial = d->partial, o.att_pos = d->state, o.att_splits = L.splits, o.att_window = L.window;
                o.att_heads = c.heads, o.att_kv = L.kvh, o.att_cluster = L.cluster;
            }
            o.lean = 1;  // short: the small kernel, which fits beside the gate/up product's block, so that block fills its ring meanwhile
            if (!wide && L.cluster == L.splits) o.att_entries = 1;  // one cluster covers the window: always one entry
            o.pf = hint(d, L.gate_up, 2, PF, PF);
            TB_TRY(gemv(d, L.o, o));

        }

        GemvParams gu;
        gu.xmode = X_NORM, gu.h = d->x[cur], gu.yres = d->y, gu.w1 = L.post_attn, gu.hscale = 1.0f, gu.w2 = L.pre_ffn, gu.eps = c.eps;
        if (block) gu.yres2 = d->y2;  // the output projection came as two partial products
        gu.h_out = d->x[1 - cur];
        cur = 1 - cur;
        gu.epi = EPI_GEGLU, gu.y = d->g;
        gu.pf = hint(d, L.down, 1, 0, PF);
        gu.l2_ahead = d->ctx->l2_ahead;
        if (d->ctx->l2_next && L.down.bits == 8 && (c.ffn == 2048 || c.ffn == 4096 || c.ffn == 8192 || c.ffn == 16384)) {
            // The head of the down projection (its blocks' first stages: 32 * 2048 / ffn rows each, as launch_gemv cuts them) into the L2 while the
            // short kernels in front of this one run and HBM has nothing else to do.
            Prefetch& pf = gu.pf;
            pf.w = L.down.w, pf.s = L.down.s, pf.rows = L.down.rows, pf.cols = L.down.cols, pf.grid = (uint32_t)d->ctx->sms;
            pf.stage_rows = gemv_stage_rows(c.ffn), pf.stages = d->ctx->l2_next, pf.row_bytes = c.ffn, pf.srow_bytes = c.ffn / 16;
        }
        TB_TRY(gemv(d, L.gate_up, gu));

        GemvParams dn;
        dn.xmode = X_F32, dn.x = d->g, dn.epi = EPI_F32, dn.y = d->y;
        dn.pf = i + 1 < c.layers ? hint(d, d->layers[i + 1].qkv, 1, 0, PF) : hint(d, d->embed, 1, 0, PF);
        TB_TRY(gemv(d, L.down, dn));

        if (pl) {
            // decode.rs:654-658: x += post_ffn_norm(down), unscaled, feeds the gate; gelu(gate) times the layer's input,
            // projected back; the next product's prologue adds post_per_layer_input_norm of it and applies the scalar.
            GemvParams pg;
            pg.xmode = X_NORM, pg.h = d->x[cur], pg.yres = d->y, pg.w1 = L.post_ffn, pg.hscale = 1.0f, pg.w2 = nullptr, pg.eps = c.eps;
            pg.h_out = d->x[1 - cur];
            cur = 1 - cur;
            pg.epi = EPI_F32, pg.y = d->g2, pg.gelu_mul = d->pli + (size_t)i * pl;
            TB_TRY(gemv(d, L.pl_gate, pg));
            GemvParams pj;
            pj.xmode = X_F32, pj.x = d->g2, pj.epi = EPI_F32, pj.y = d->y;
            TB_TRY(gemv(d, L.pl_proj, pj));
        }
    }
    const Layer& P = d->layers[c.layers - 1];
    GemvParams h;
    h.xmode = X_NORM, h.h = d->x[cur], h.yres = d->y, h.w1 = pl ? P.post_pl : P.post_ffn, h.hscale = P.layer_scalar, h.w2 = d->norm, h.eps = c.eps;
    h.h_out = d->x[1 - cur];
    h.epi = EPI_ARGMAX, h.y = d->settings.keep_logits ? d->logits : nullptr;
    h.best = d->best, h.count = reinterpret_cast<uint32_t*>(d->best + 1), h.state = d->state, h.token_out = token_word;
    h.trace = d->trace, h.trace_mask = TRACE - 1;
    h.pf = hint(d, d->layers[0].qkv, 1, 0, PF);  // the next step's first matrix
    if (d->capture_sampled) {
        // decode.rs:588-591: the head's logits, then the sampler, which writes the token and advances the position.
        h.epi = EPI_F32, h.y = d->logits;
        TB_TRY(gemv(d, d->embed, h));
        TB_TRY(launch_sample_draw(d->ctx, d->logits, d->work, c.vocab, d->sampling, d->state, d->seen, token_word, d->sample_partial, d->sample_count, 0,
                                  d->trace, TRACE - 1));
        d->launches++;
    } else {
        TB_TRY(gemv(d, d->embed, h));
    }
    d->final_x = 1 - cur;
    if (d->ctx->l2_side && d->side != nullptr && !d->collect && !d->fused) {  // the side stream joins the step
        TB_CUDA(cudaEventRecord(d->join_ev, d->side));
        TB_CUDA(cudaStreamWaitEvent(d->ctx->stream, d->join_ev, 0));
    }
    if (!d->capture_sampled) d->step_count = d->launches;  // the graphs that end in the sampler have one launch more
    return OK;
}

struct Named {
    void* ptr = nullptr;
    size_t bytes = 0;
    int kind = 0;  // 0 plain, 1 gate_up codes, 2 gate_up scales, 3 layer scalar
    uint32_t layer = 0;
};

bool find_tensor(tb_decoder* d, const std::string& name, Named& out) {
    const tb_config& c = d->cfg;
    auto mat = [&](Mat& m, const std::string& suffix, int gate_up) {
        if (suffix == ".w") out = {m.w, m.code_bytes(), gate_up ? 1 : 0, 0};
        else if (suffix == ".s") out = {m.s, m.scale_bytes(), gate_up ? 2 : 0, 0};
        else return false;
        return true;
    };
    if (c.per_layer && name.rfind("embed_per_layer", 0) == 0) return mat(d->embed_pl, name.substr(15), 0);
    if (c.per_layer && name.rfind("per_layer_proj", 0) == 0) return mat(d->pl_model_proj, name.substr(14), 0);
    if (c.per_layer && name == "per_layer_norm") return out = {d->pl_norm, (size_t)c.per_layer * 4, 0, 0}, true;
    if (name.rfind("embed", 0) == 0) return mat(d->embed, name.substr(5), 0);
    if (name == "norm") return out = {d->norm, (size_t)c.hidden * 4, 0, 0}, true;
    const size_t dot = name.find('.');
    if (dot == std::string::npos || dot == 0) return false;
    uint32_t i = 0;
    for (size_t k = 0; k < dot; k++) {
        if (name[k] < '0' || name[k] > '9') return false;
        i = i * 10 + (uint32_t)(name[k] - '0');
    }
    if (i >= c.layers) return false;
    Layer& L = d->layers[i];
    const std::string rest = name.substr(dot + 1);
    if (c.per_layer && rest.rfind("per_layer_gate", 0) == 0) return mat(L.pl_gate, rest.substr(14), 0);
    if (c.per_layer && rest.rfind("per_layer_proj", 0) == 0) return mat(L.pl_proj, rest.substr(14), 0);
    if (c.per_layer && rest == "post_per_layer_input_norm") return out = {L.post_pl, (size_t)c.hidden * 4, 0, i}, true;
    if (rest.rfind("qkv", 0) == 0) return mat(L.qkv, rest.substr(3), 0);
    if (rest.rfind("o.", 0) == 0) return mat(L.o, rest.substr(1), 0);
    if (rest.rfind("gate_up", 0) == 0) return mat(L.gate_up, rest.substr(7), 1);
    if (rest.rfind("down", 0) == 0) return mat(L.down, rest.substr(4), 0);
    const size_t hb = (size_t)c.hidden * 4, db = (size_t)L.dim * 4;
    if (rest == "q_norm") return out = {L.q_norm, db, 0, i}, true;
    if (rest == "k_norm") return out = {L.k_norm, db, 0, i}, true;
    if (rest == "input_layernorm") return out = {L.input_ln, hb, 0, i}, true;
    if (rest == "post_attention_layernorm") return out = {L.post_attn, hb, 0, i}, true;
    if (rest == "pre_feedforward_layernorm") return out = {L.pre_ffn, hb, 0, i}, true;
    if (rest == "post_feedforward_layernorm") return out = {L.post_ffn, hb, 0, i}, true;
    if (rest == "layer_scalar") return out = {nullptr, 4, 3, i}, true;
    return false;
}

int set_position(tb_decoder* d, uint32_t pos) {
    d->words[2] = pos;
    TB_CUDA(cudaMemcpyAsync(d->state, d->words + 2, 4, cudaMemcpyHostToDevice, d->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
    d->pos = pos;
    return OK;
}

int queue(tb_decoder* d, int g) {
    TB_CUDA(cudaGraphLaunch(d->sampled ? d->graphs_sampled[g] : d->graphs[g], d->ctx->stream));
    TB_CUDA(cudaEventRecord(d->done[g], d->ctx->stream));
    d->pos++;
    return OK;
}

int feed_token(tb_decoder* d, uint32_t token) {
    if (token >= d->cfg.vocab) return fail(OUT_OF_RANGE, "decoder: token outside the vocabulary");
    d->words[2] = token;
    TB_CUDA(cudaMemcpyAsync(d->state + 1, d->words + 2, 4, cudaMemcpyHostToDevice, d->ctx->stream));
    return OK;
}

int ready(tb_decoder* d, uint32_t steps) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    if (!d->built) return fail(NO_MODEL, "decoder: tb_decoder_build has not run");
    if ((uint64_t)d->pos + steps > d->settings.context) return fail(TOO_LONG, "decoder: the sequence would pass the context");
    return OK;
}

// The prefill copy (settings.prefill_copy): room for every layer's qkv, o, gate/up and down matrices as f16.  Automatic
// (0): taken when prefill runs in chunks of 256 tokens and more, the matrices have 8 or 4 bits, and the device keeps a
// quarter of its memory free after it; 2 asks for it whatever is free; 1 leaves it out.
constexpr uint32_t COPY_MIN_TOKENS = 256;

int place_copy(tb_decoder* d) {
    const uint32_t want = d->settings.prefill_copy;
    if (want > 2) return fail(OUT_OF_RANGE, "tb_settings.prefill_copy is 0 (automatic), 1 (none) or 2 (always)");
    const char* env = getenv("TACHYON_B200_PREFILL_COPY");
    if (want == 1 || (want == 0 && env != nullptr && env[0] == '0') || d->settings.chunk == 0 || d->cfg.hidden % 64 != 0 || d->cfg.ffn % 64 != 0) return OK;
    if (want == 0 && d->settings.chunk < COPY_MIN_TOKENS) return OK;
    size_t halves = 0;
    for (Layer& L : d->layers)
        for (Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) halves += ((size_t)m->rows * m->cols + 127) / 128 * 128;
    size_t free_bytes = 0, total = 0;
    TB_CUDA(cudaMemGetInfo(&free_bytes, &total));
    if (want == 0 && (free_bytes < halves * 2 || free_bytes - halves * 2 < total / 4)) return OK;
    const cudaError_t e = pool_alloc(d->ctx, reinterpret_cast<void**>(&d->copy), halves * 2);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (want == 0) return d->copy = nullptr, OK;
        return fail(OUT_OF_MEMORY, "tb_decoder_open: no room for the prefill copy of the weights (" + std::to_string(halves * 2) + " bytes)");
    }
    __half* at = d->copy;
    for (Layer& L : d->layers)
        for (Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) m->f16 = at, at += ((size_t)m->rows * m->cols + 127) / 128 * 128;
    d->copy_valid = false;
    return OK;
}

// Writes the copy from the codes as they are now.
int refresh_copy(tb_decoder* d) {
    if (!d->copy || d->copy_valid) return OK;
    for (Layer& L : d->layers)
        for (Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) TB_TRY(launch_dequant_f16(d->ctx, m->w, m->s, m->rows, m->cols, m->bits, m->f16));
    d->copy_valid = true;
    return OK;
}

// One of prefill's four large products: on the f16 copy from 256 tokens on, on the codes below that.
int prefill_product(tb_decoder* d, const Mat& m, const __half* x, uint32_t tokens, void* out, int mode) {
    if (m.f16 != nullptr && d->copy_valid && tokens >= COPY_MIN_TOKENS)
        return launch_gemm_q8(d->ctx, reinterpret_cast<const int8_t*>(m.f16), nullptr, x, tokens, m.rows, m.cols, out, mode, 16);
    return launch_gemm_q8(d->ctx, m.w, m.s, x, tokens, m.rows, m.cols, out, mode, m.bits);
}

// Every weight tensor in the arena, in the order of the layout (which no setting changes): what parking copies out and
// resuming copies back.  The per-layer table in host memory is not among them (it moves with the parked model as it is).
template <typename F>
void for_each_weight(tb_decoder* d, F&& f) {
    const tb_config& c = d->cfg;
    auto mat = [&](Mat& m) { f(static_cast<void*>(m.w), m.code_bytes()), f(static_cast<void*>(m.s), m.scale_bytes()); };
    auto vec = [&](float* v, size_t n) { f(static_cast<void*>(v), n * 4); };
    mat(d->embed), vec(d->norm, c.hidden);
    if (c.per_layer) {
        if (!d->settings.host_table) mat(d->embed_pl);
        mat(d->pl_model_proj), vec(d->pl_norm, c.per_layer);
    }
    for (Layer& L : d->layers) {
        mat(L.qkv), mat(L.o), mat(L.gate_up), mat(L.down);
        vec(L.q_norm, L.dim), vec(L.k_norm, L.dim), vec(L.input_ln, c.hidden), vec(L.post_attn, c.hidden), vec(L.pre_ffn, c.hidden), vec(L.post_ffn, c.hidden);
        if (c.per_layer) mat(L.pl_gate), mat(L.pl_proj), vec(L.post_pl, c.hidden);
    }
}

size_t weight_bytes(tb_decoder* d) {
    size_t n = 0;
    for_each_weight(d, [&](void*, size_t bytes) { n += (bytes + 255) / 256 * 256; });
    return n;
}

size_t host_table_bytes(const tb_decoder* d) {
    return d->host_table ? (d->embed_pl.code_bytes() + 255) / 256 * 256 + d->embed_pl.scale_bytes() : 0;
}

int open_decoder(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, char* adopt_table, tb_decoder** out);

}  // namespace

extern "C" {

int tb_decoder_open(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, tb_decoder** out) {
    return open_decoder(ctx, cfg, settings, nullptr, out);
}

}  // extern "C"

namespace {

// adopt_table: a per-layer table already in pinned, mapped host memory (a parked model's), taken over instead of a new one.
int open_decoder(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, char* adopt_table, tb_decoder** out) {
    if (!ctx || !cfg || !settings || !out) return fail(OUT_OF_RANGE, "tb_decoder_open: null argument");
    *out = nullptr;
    TB_TRY(validate(*cfg, *settings));
    tb_decoder* d = new tb_decoder();
    d->ctx = ctx, d->cfg = *cfg, d->settings = *settings;
    {
        const char* env = getenv("TACHYON_B200_FUSED");
        d->fused = settings->fused != 0 || (env != nullptr && env[0] == '1' && settings->weight_bits != 4);
    }
    d->global.resize(cfg->layers);
    for (uint32_t i = 0; i < cfg->layers; i++)
        d->global[i] = cfg->global ? cfg->global[i] : (cfg->global_every ? ((i + 1) % cfg->global_every == 0) : 0);
    d->cfg.global = nullptr;
    d->layers.resize(cfg->layers);
    // The embedding's scale is sqrt(hidden) rounded to bfloat16 (decode.rs:571, 689-693).
    d->embed_scale = bf16_round(sqrtf((float)cfg->hidden));
    layout(d, nullptr);
    cudaError_t e = cudaSetDevice(ctx->gpu);
    if (e == cudaSuccess) e = pool_alloc(ctx, reinterpret_cast<void**>(&d->arena), d->arena_bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(d->arena, 0, d->arena_bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaHostAlloc(&d->words, 64, cudaHostAllocMapped);
    if (e == cudaSuccess && cfg->per_layer && settings->host_table) {
        const size_t bytes = (d->embed_pl.code_bytes() + 255) / 256 * 256 + d->embed_pl.scale_bytes();
        if (adopt_table != nullptr) {
            d->host_table = adopt_table;
        } else {
            e = cudaHostAlloc(&d->host_table, bytes, cudaHostAllocMapped);
            if (e == cudaSuccess) memset(d->host_table, 0, bytes);
        }
    }
    for (int g = 0; g < 2 && e == cudaSuccess; g++) e = cudaEventCreateWithFlags(&d->done[g], cudaEventDisableTiming);
    if (e == cudaSuccess && ctx->l2_side) {
        e = cudaStreamCreateWithFlags(&d->side, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&d->fork_ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&d->join_ev, cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        const int s = cuda_fail(e, "tb_decoder_open");
        if (adopt_table != nullptr) d->host_table = nullptr;  // still the caller's
        tb_decoder_close(d);
        return s;
    }
    layout(d, d->arena);
    {
        const int st = place_copy(d);
        if (st != OK) {
            if (adopt_table != nullptr) d->host_table = nullptr;  // still the caller's
        tb_decoder_close(d);
            return st;
        }
    }
    memset(d->words, 0, 64);
    for (int k = 0; k < 2; k++) {
        const std::vector<float> f = rope_freq(k ? cfg->theta_global : cfg->theta_sliding, dim_of(*cfg, k), k ? cfg->fraction_global : 1.0f);
        e = cudaMemcpyAsync(d->freq[k], f.data(), f.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        // The table of cosines and sines by position serves attend.cu's kernel (heads of 256) only.
        if (e == cudaSuccess && dim_of(*cfg, k) == 256 && launch_rope_table(ctx, d->freq[k], d->settings.context, d->trig[k]) != OK) e = cudaErrorUnknown;
        if (e != cudaSuccess) {
            const int s = cuda_fail(e, "tb_decoder_open: rope tables");
            if (adopt_table != nullptr) d->host_table = nullptr;  // still the caller's
        tb_decoder_close(d);
            return s;
        }
    }
    *out = d;
    return OK;
}

}  // namespace

extern "C" {

void tb_decoder_close(tb_decoder* d) {
    if (!d) return;
    if (d->ctx && d->ctx->stream) cudaStreamSynchronize(d->ctx->stream);
    for (int g = 0; g < 2; g++) {
        if (d->graphs[g]) cudaGraphExecDestroy(d->graphs[g]);
        if (d->graphs_sampled[g]) cudaGraphExecDestroy(d->graphs_sampled[g]);
        if (d->done[g]) cudaEventDestroy(d->done[g]);
    }
    for (int g = 0; g < 2; g++)
        if (d->phase_dev[g]) cudaFree(d->phase_dev[g]);
    if (d->fork_ev) cudaEventDestroy(d->fork_ev);
    if (d->join_ev) cudaEventDestroy(d->join_ev);
    if (d->side) cudaStreamDestroy(d->side);
    if (d->arena) pool_free(d->ctx, d->arena);
    if (d->copy) pool_free(d->ctx, d->copy);
    if (d->words) cudaFreeHost(d->words);
    if (d->host_table) cudaFreeHost(d->host_table);
    if (d->shadow) cudaFreeHost(d->shadow);
    delete d;
}

int tb_decoder_load(tb_decoder* d, const char* name, const void* data, size_t bytes) {
    if (!d || !name || !data) return fail(OUT_OF_RANGE, "tb_decoder_load: null argument");
    Named t;
    if (!find_tensor(d, name, t)) return fail(NO_MODEL, std::string("tb_decoder_load: no tensor named ") + name);
    d->copy_valid = false;
    tb_decoder_drop_shadow(d);
    if (bytes != t.bytes) return fail(FORMAT, std::string("tb_decoder_load: ") + name + " has " + std::to_string(bytes) + " bytes, expected " + std::to_string(t.bytes));
    cudaStream_t s = d->ctx->stream;
    if (t.kind == 3) {
        memcpy(&d->layers[t.layer].layer_scalar, data, 4);
        d->built = false;
        return OK;
    }
    if (t.kind == 0) {
        TB_CUDA(cudaMemcpyAsync(t.ptr, data, bytes, cudaMemcpyDefault, s));  // the per-layer table may live in host memory
        TB_CUDA(cudaStreamSynchronize(s));
        return OK;
    }
    // gate_up: gate rows then up rows in the file; pairs (gate_j, up_j) on the device, scattered by strided copies.
    return tb_decoder_load_part(d, name, 0, data, bytes, bytes);
}

// For the file loader: a tensor may arrive in pieces.  One that is copied to its place as it is has each piece written at its
// offset.  The gate/up matrix (gate rows, then up rows in the file; pairs (gate_j, up_j) on the device) has each piece's
// rows scattered by strided copies: file row r goes to device row 2 r, or 2 (r - ffn) + 1 past the first half; a piece
// that starts or ends inside a row has that part copied alone.
int tb_decoder_load_part(tb_decoder* d, const char* name, size_t offset, const void* data, size_t bytes, size_t total) {
    if (!d || !name || !data) return fail(OUT_OF_RANGE, "tb_decoder_load_part: null argument");
    Named t;
    if (!find_tensor(d, name, t)) return fail(NO_MODEL, std::string("tb_decoder_load: no tensor named ") + name);
    if (t.kind == 3 || (offset == 0 && bytes == total && t.kind == 0)) return tb_decoder_load(d, name, data, bytes);
    if (total != t.bytes) return fail(FORMAT, std::string("tb_decoder_load: ") + name + " has " + std::to_string(total) + " bytes, expected " + std::to_string(t.bytes));
    if (offset > total || bytes > total - offset) return fail(OUT_OF_RANGE, "tb_decoder_load_part: a piece past the tensor's end");
    d->copy_valid = false;
    tb_decoder_drop_shadow(d);
    cudaStream_t s = d->ctx->stream;
    char* base = static_cast<char*>(t.ptr);
    const char* src = static_cast<const char*>(data);
    if (t.kind == 0) {
        TB_CUDA(cudaMemcpyAsync(base + offset, src, bytes, cudaMemcpyDefault, s));
    } else {
        const size_t half_rows = d->cfg.ffn, row = total / (2 * half_rows);
        while (bytes > 0) {
            const size_t r = offset / row, in_row = offset % row;
            char* dst = base + (r < half_rows ? 2 * r : 2 * (r - half_rows) + 1) * row;
            size_t n;
            if (in_row != 0 || bytes < row) {
                n = std::min(row - in_row, bytes);
                TB_CUDA(cudaMemcpyAsync(dst + in_row, src, n, cudaMemcpyHostToDevice, s));
            } else {
                const size_t rows = std::min(bytes / row, (r < half_rows ? half_rows : 2 * half_rows) - r);
                n = rows * row;
                TB_CUDA(cudaMemcpy2DAsync(dst, 2 * row, src, row, row, rows, cudaMemcpyHostToDevice, s));
            }
            offset += n, src += n, bytes -= n;
        }
    }
    TB_CUDA(cudaStreamSynchronize(s));
    return OK;
}

int tb_decoder_loads_in_parts(tb_decoder* d, const char* name) {
    Named t;
    return d && name && find_tensor(d, name, t) && t.kind != 3;
}

int tb_decoder_fill_random(tb_decoder* d, uint64_t seed) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    d->copy_valid = false;
    tb_decoder_drop_shadow(d);
    const tb_config& c = d->cfg;
    tb_context* ctx = d->ctx;
    const uint32_t bits = d->embed.bits;
    const float smul = bits == 4 ? 0.02f / 8.0f : 0.02f / 127.0f;  // either way weights of magnitude ~0.02
    auto mat = [&](Mat& m, uint64_t id) -> int {
        TB_TRY(launch_fill_codes(ctx, seed, id, m.w, m.code_bytes()));
        return launch_fill_scales(ctx, seed, id + 1, m.s, m.scale_bytes() / 2, smul);
    };
    TB_TRY(mat(d->embed, 1ull << 20));
    TB_TRY(launch_fill_uniform(ctx, seed, (1ull << 20) + 2, d->norm, c.hidden, 0.5f, 1.5f));
    if (c.per_layer) {
        TB_TRY(mat(d->embed_pl, (1ull << 20) + 4));
        TB_TRY(mat(d->pl_model_proj, (1ull << 20) + 6));
        TB_TRY(launch_fill_uniform(ctx, seed, (1ull << 20) + 8, d->pl_norm, c.per_layer, 0.5f, 1.5f));
    }
    void *tw = nullptr, *ts = nullptr;
    TB_CUDA(cudaMalloc(&tw, d->layers[0].gate_up.code_bytes()));
    TB_CUDA(cudaMalloc(&ts, d->layers[0].gate_up.scale_bytes()));
    int st = OK;
    for (uint32_t i = 0; i < c.layers && st == OK; i++) {
        Layer& L = d->layers[i];
        const uint64_t b = 32ull * i;
        st = mat(L.qkv, b);
        if (st == OK) st = mat(L.o, b + 2);
        if (st == OK) st = launch_fill_codes(ctx, seed, b + 4, static_cast<int8_t*>(tw), L.gate_up.code_bytes());
        if (st == OK) st = launch_fill_scales(ctx, seed, b + 5, static_cast<__half*>(ts), L.gate_up.scale_bytes() / 2, smul);
        if (st == OK) st = launch_interleave_rows(ctx, tw, L.gate_up.w, c.ffn, c.hidden * bits / 8);
        if (st == OK) st = launch_interleave_rows(ctx, ts, L.gate_up.s, c.ffn, c.hidden / (bits == 4 ? 64 : 32) * 2);
        if (st == OK) st = mat(L.down, b + 6);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 8, L.q_norm, L.dim, 0.15f, 0.35f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 9, L.k_norm, L.dim, 0.15f, 0.35f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 10, L.input_ln, c.hidden, 0.5f, 1.5f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 11, L.post_attn, c.hidden, 0.5f, 1.5f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 12, L.pre_ffn, c.hidden, 0.5f, 1.5f);
        if (st == OK) st = launch_fill_uniform(ctx, seed, b + 13, L.post_ffn, c.hidden, 0.5f, 1.5f);
        if (st == OK && c.per_layer) st = mat(L.pl_gate, b + 16);
        if (st == OK && c.per_layer) st = mat(L.pl_proj, b + 18);
        if (st == OK && c.per_layer) st = launch_fill_uniform(ctx, seed, b + 20, L.post_pl, c.hidden, 0.5f, 1.5f);
        if (st == OK) {
            // The scalar comes from the same generator, evaluated through a one-element device fill.
            st = launch_fill_uniform(ctx, seed, b + 14, d->x[0], 1, 0.95f, 1.0f);
            if (st == OK && cudaMemcpyAsync(d->words + 3, d->x[0], 4, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) st = fail(CUDA, "fill: copy");
            if (st == OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = fail(CUDA, "fill: sync");
            if (st == OK) memcpy(&L.layer_scalar, d->words + 3, 4);
        }
    }
    cudaStreamSynchronize(ctx->stream);
    cudaFree(tw);
    cudaFree(ts);
    if (st == OK) TB_CUDA(cudaMemsetAsync(d->x[0], 0, 4, ctx->stream));
    d->built = false;
    return st;
}

int tb_decoder_fill_cache(tb_decoder* d, uint64_t seed, uint32_t positions) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    if (positions > d->settings.context) return fail(TOO_LONG, "tb_decoder_fill_cache: more positions than the context");
    const tb_config& c = d->cfg;
    for (uint32_t i = 0; i < c.layers; i++) {
        Layer& L = d->layers[i];
        if (L.source >= 0) continue;  // a shared layer has no cache of its own
        // Position p lives in slot p % cap; filling whole caches covers every slot a window can reach.
        const size_t n = (size_t)L.kvh * L.cap * L.dim;
        TB_TRY(launch_fill_gauss_f16(d->ctx, seed, (1ull << 21) + 2ull * i, L.kc, n, 1.0f));
        TB_TRY(launch_fill_gauss_f16(d->ctx, seed, (1ull << 21) + 2ull * i + 1, L.vc, n, 1.0f));
    }
    return set_position(d, positions);
}

int tb_decoder_build(tb_decoder* d) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    cudaStream_t s = d->ctx->stream;
    TB_CUDA(cudaStreamSynchronize(s));
    for (int g = 0; g < (d->fused ? 2 : 4); g++) {
        // Graphs 2 and 3 are the pair that ends in the sampler kernel (one launch per phase only).
        cudaGraphExec_t& slot = g < 2 ? d->graphs[g] : d->graphs_sampled[g - 2];
        d->capture_sampled = g >= 2;
        if (slot) cudaGraphExecDestroy(slot), slot = nullptr;
        uint32_t* word = nullptr;
        TB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&word), d->words + (g & 1), 0));
        // The fused step reads its phases from a table on the device, one table per graph (the token word differs).
        if (d->fused) {
            std::vector<StepPhase> table;
            d->collect = &table;
            const int sc = step_ops(d, word);
            d->collect = nullptr;
            TB_TRY(sc);
            d->phase_count = (uint32_t)table.size();
            if (!d->phase_dev[g]) TB_CUDA(cudaMalloc(&d->phase_dev[g], table.size() * sizeof(StepPhase)));
            TB_CUDA(cudaMemcpy(d->phase_dev[g], table.data(), table.size() * sizeof(StepPhase), cudaMemcpyHostToDevice));
        }
        auto run = [&]() -> int { return d->fused ? launch_step(d->ctx, d->phase_dev[g], d->phase_count, d->grid_counter, d->state) : step_ops(d, word); };
        // One uncaptured pass first: it sets each kernel's attributes (not allowed while capturing) and surfaces
        // descriptor errors plainly.  It runs on zeroed state and is followed by a reset.
        if (g == 0 || g == 2) {
            const int first = run();
            if (first != OK) return d->capture_sampled = false, first;
            TB_CUDA(cudaStreamSynchronize(s));
        }
        TB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        const int st = run();
        cudaGraph_t graph = nullptr;
        const cudaError_t e = cudaStreamEndCapture(s, &graph);
        d->capture_sampled = false;
        if (st != OK) {
            if (graph) cudaGraphDestroy(graph);
            return st;
        }
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
        const cudaError_t ei = cudaGraphInstantiate(&slot, graph, 0);
        cudaGraphDestroy(graph);
        if (ei != cudaSuccess) return cuda_fail(ei, "cudaGraphInstantiate");
    }
    // A model on its way back from the host tier writes its prefill copy when a long prompt first asks for it, not here: its
    // return is measured to its first answer, and a short prompt never reads the copy.
    if (!d->weights_ready) TB_TRY(refresh_copy(d));
    d->built = true;
    d->running = false;
    // The uncaptured pass advanced the position and wrote a cache slot; start clean.
    return tb_decoder_reset(d);
}

int tb_decoder_reset(tb_decoder* d) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    if (d->running) TB_TRY(tb_decoder_stop(d));
    TB_CUDA(cudaMemsetAsync(d->state, 0, 8, d->ctx->stream));
    TB_CUDA(cudaMemsetAsync(d->seen, 0, ((size_t)d->cfg.vocab + 31) / 32 * 4, d->ctx->stream));  // a new sequence has seen nothing
    return set_position(d, 0);
}

int tb_decoder_set_sampling(tb_decoder* d, const tb_sampling* s) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_set_sampling: a generation is running; stop it first");
    tb_sampling v = {0.0f, 0.0f, 1.0f, 0.0f, 1.0f, 0u, 0ull, 0ull};  // Sampling::default (sample.rs:58-63)
    if (s) v = *s;
    if (!(v.penalty > 0.0f) || v.temperature < 0.0f || v.softcap < 0.0f) return fail(OUT_OF_RANGE, "tb_decoder_set_sampling: negative temperature or soft cap, or penalty <= 0");
    // The plain largest logit needs no sampler kernel: the LM head picks it (the soft cap is monotonic).
    const bool plain = v.temperature == 0.0f && v.penalty == 1.0f && v.allowed == 0;
    if (!plain && d->fused) return fail(UNSUPPORTED, "tb_decoder_set_sampling: the fused step only picks the largest logit");
    if (!plain && d->cfg.vocab % 4 != 0) return fail(UNSUPPORTED, "tb_decoder_set_sampling: the sampler needs a vocabulary that is a multiple of 4");
    TB_CUDA(cudaMemcpyAsync(d->sampling, &v, sizeof v, cudaMemcpyHostToDevice, d->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(d->ctx->stream));  // `v` is on this stack
    d->sampled = !plain;
    return OK;
}

int tb_decoder_step(tb_decoder* d, uint32_t token, uint32_t* next) {
    TB_TRY(ready(d, 1));
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_step: a generation is running; stop it first");
    TB_TRY(feed_token(d, token));
    TB_TRY(queue(d, 0));
    TB_CUDA(cudaEventSynchronize(d->done[0]));
    if (next) *next = d->words[0];
    return OK;
}

int tb_decoder_start(tb_decoder* d, uint32_t token) {
    TB_TRY(ready(d, 1));
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_start: already running");
    TB_TRY(feed_token(d, token));
    d->at = 0;
    TB_TRY(queue(d, 0));
    d->running = true;
    return OK;
}

int tb_decoder_next_token(tb_decoder* d, uint32_t* token) {
    if (!d || !d->running) return fail(OUT_OF_RANGE, "tb_decoder_next_token: no generation running");
    TB_TRY(ready(d, 1));
    const int g = d->at;
    TB_TRY(queue(d, 1 - g));  // the step on the token being waited for: the GPU never waits for the host
    TB_CUDA(cudaEventSynchronize(d->done[g]));
    d->at = 1 - g;
    if (token) *token = d->words[g];
    return OK;
}

int tb_decoder_stop(tb_decoder* d) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    if (!d->running) return OK;
    TB_CUDA(cudaEventSynchronize(d->done[d->at]));
    d->running = false;
    return OK;
}

int tb_decoder_run(tb_decoder* d, uint32_t token, uint32_t steps, uint32_t* tokens_out) {
    TB_TRY(ready(d, steps));
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_run: a generation is running; stop it first");
    const uint32_t first = d->pos;
    TB_TRY(feed_token(d, token));
    for (uint32_t i = 0; i < steps; i++) TB_TRY(queue(d, (int)(i & 1)));
    if (tokens_out) {
        TB_CUDA(cudaMemcpyAsync(tokens_out, d->trace + first, (size_t)steps * 4, cudaMemcpyDeviceToHost, d->ctx->stream));
        TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
    }
    return OK;
}

// One chunk of prompt tokens through every layer (crates/tachyon/src/model/prefill.rs:124-196): tensor-core GEMMs over
// the chunk, flash attention over the cache ring.  Only what later tokens need is computed: the caches of every layer,
// so the last layer stops after its attention inputs are stored.
static int prefill_chunk(tb_decoder* d, const uint32_t* tokens, uint32_t n, uint32_t pos0) {
    const tb_config& c = d->cfg;
    tb_context* ctx = d->ctx;
    const uint32_t H = c.hidden;
    TB_CUDA(cudaMemcpyAsync(d->pf_tokens, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    TB_TRY(launch_prefill_embed(ctx, d->embed.w, d->embed.s, d->pf_tokens, n, H, d->embed_scale, d->pf_h, d->embed.bits));
    const uint32_t pl = c.per_layer, plw = pl * c.layers;
    if (pl) {
        // Every token's per-layer inputs (decode.rs:572-579 for a chunk): table rows times sqrt(per_layer), the embeddings
        // through the per-layer projection, and (row + w * rmsnorm(projection)) / sqrt(2) per token and layer.
        TB_TRY(launch_prefill_embed(ctx, d->embed_pl.w, d->embed_pl.s, d->pf_tokens, n, plw, sqrtf((float)pl), d->pf_ple, d->embed_pl.bits));
        TB_TRY(launch_prefill_norm(ctx, d->pf_h, nullptr, nullptr, nullptr, n, H, c.eps, 1.0f, d->pf_x));  // the embeddings as f16
        TB_TRY(launch_gemm_q8(ctx, d->pl_model_proj.w, d->pl_model_proj.s, d->pf_x, n, plw, H, d->pf_proj, 0, d->pl_model_proj.bits));
        const uint32_t chunks = n * c.layers;
        for (uint32_t at = 0; at < chunks; at += 32768) {  // the grid's second dimension holds 65535 blocks
            const uint32_t now = std::min(32768u, chunks - at);
            const size_t off = (size_t)at * pl;
            TB_TRY(launch_norm_q8(ctx, d->pf_ple + off, d->pf_pli + off, d->pf_proj + off, d->pl_norm, nullptr, nullptr, nullptr, pl, now, c.eps * (float)H, 0.70710678118654752f));
        }
    }
    for (uint32_t i = 0; i < c.layers; i++) {
        Layer& L = d->layers[i];
        if (i == 0) {
            TB_TRY(launch_prefill_norm(ctx, d->pf_h, nullptr, nullptr, L.input_ln, n, H, c.eps, 1.0f, d->pf_x));
        } else {
            const Layer& P = d->layers[i - 1];
            TB_TRY(launch_prefill_norm(ctx, d->pf_h, d->pf_y, pl ? P.post_pl : P.post_ffn, L.input_ln, n, H, c.eps, P.layer_scalar, d->pf_x));
        }
        TB_TRY(prefill_product(d, L.qkv, d->pf_x, n, d->pf_qkv, 0));
        // A shared layer has query rows only: nothing to append to the cache it reads.
        TB_TRY(launch_prefill_qkv(ctx, d->pf_qkv, L.q_norm, L.k_norm, d->freq[L.global ? 1 : 0], d->pf_q, L.kc, L.vc, n, pos0, L.cap, c.heads,
                                  L.source < 0 ? L.kvh : 0, c.eps, c.attn_scale, L.dim));
        if (i + 1 == c.layers) break;
        TB_TRY(launch_prefill_flash(ctx, d->pf_q, L.kc, L.vc, d->pf_att, n, pos0, L.cap, L.window, c.heads, L.kvh, L.dim));
        TB_TRY(prefill_product(d, L.o, d->pf_att, n, d->pf_y, 0));
        TB_TRY(launch_prefill_norm(ctx, d->pf_h, d->pf_y, L.post_attn, L.pre_ffn, n, H, c.eps, 1.0f, d->pf_x));
        TB_TRY(prefill_product(d, L.gate_up, d->pf_x, n, d->pf_g, 2));
        TB_TRY(prefill_product(d, L.down, d->pf_g, n, d->pf_y, 0));
        if (pl) {
            // decode.rs:654-658 for a chunk: the stream plus the MLP's normed output, unscaled, through the gate; GELU times
            // each token's input of this layer; projected back.  The next layer's norm step adds it.
            TB_TRY(launch_prefill_norm(ctx, d->pf_h, d->pf_y, L.post_ffn, nullptr, n, H, c.eps, 1.0f, d->pf_x));
            TB_TRY(launch_gemm_q8(ctx, L.pl_gate.w, L.pl_gate.s, d->pf_x, n, pl, H, d->pf_g2, 6, L.pl_gate.bits, d->pf_pli + (size_t)i * pl, plw));
            TB_TRY(launch_gemm_q8(ctx, L.pl_proj.w, L.pl_proj.s, d->pf_g2, n, H, pl, d->pf_y, 0, L.pl_proj.bits));
        }
    }
    return OK;
}

int tb_decoder_prefill(tb_decoder* d, const uint32_t* tokens, uint32_t n) {
    TB_TRY(ready(d, n));
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_prefill: a generation is running; stop it first");
    if (n && !tokens) return fail(OUT_OF_RANGE, "tb_decoder_prefill: null tokens");
    for (uint32_t i = 0; i < n; i++)
        if (tokens[i] >= d->cfg.vocab) return fail(OUT_OF_RANGE, "decoder: token outside the vocabulary");
    const char* env = getenv("TACHYON_B200_PREFILL_BY_STEPS");
    const bool by_steps = d->settings.chunk == 0 || d->cfg.ffn % 64 != 0 || (env != nullptr && env[0] == '1');
    if (by_steps) {
        // Without chunk buffers: every prompt token through the decode step; its pick is dropped.  The graphs that end in
        // the greedy pick are used whatever the sampling settings: the sampler marks what it draws as seen, and a prompt
        // must not count as generated text for the repetition penalty (the chunked path and the reference's prefill sample
        // nothing either).
        const bool sampled = d->sampled;
        d->sampled = false;
        int st = OK;
        for (uint32_t i = 0; i < n && st == OK; i++) {
            if (cudaMemcpyAsync(d->state + 1, tokens + i, 4, cudaMemcpyHostToDevice, d->ctx->stream) != cudaSuccess) st = fail(CUDA, "tb_decoder_prefill: copy of a token");
            if (st == OK) st = queue(d, 0);
        }
        d->sampled = sampled;
        TB_TRY(st);
        TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
        return OK;
    }
    if (n >= COPY_MIN_TOKENS) TB_TRY(refresh_copy(d));  // a tensor loaded after tb_decoder_build
    for (uint32_t at = 0; at < n; at += d->settings.chunk) {
        const uint32_t m = n - at < d->settings.chunk ? n - at : d->settings.chunk;
        TB_TRY(prefill_chunk(d, tokens + at, m, d->pos));
        TB_CUDA(cudaStreamSynchronize(d->ctx->stream));  // as the reference: one synchronisation per chunk (decode.rs:346-364)
        TB_TRY(set_position(d, d->pos + m));
    }
    return OK;
}

int tb_decoder_logits(tb_decoder* d, float* host_out) {
    if (!d || !host_out) return fail(OUT_OF_RANGE, "tb_decoder_logits: null argument");
    if (!d->settings.keep_logits) return fail(UNSUPPORTED, "tb_decoder_logits: the decoder was opened without keep_logits");
    TB_CUDA(cudaMemcpyAsync(host_out, d->logits, (size_t)d->cfg.vocab * 4, cudaMemcpyDeviceToHost, d->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
    return OK;
}

int tb_decoder_position(tb_decoder* d, uint32_t* pos) {
    if (!d || !pos) return fail(OUT_OF_RANGE, "tb_decoder_position: null argument");
    TB_CUDA(cudaMemcpyAsync(d->words + 4, d->state, 4, cudaMemcpyDeviceToHost, d->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
    *pos = d->words[4];
    return OK;
}

int tb_decoder_step_bytes(tb_decoder* d, uint64_t* weight_bytes, uint64_t* cache_bytes) {
    if (!d) return fail(OUT_OF_RANGE, "null decoder");
    uint64_t w = d->embed.code_bytes() + d->embed.scale_bytes(), kv = 0;
    for (const Layer& L : d->layers) {
        for (const Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) w += m->code_bytes() + m->scale_bytes();
        if (d->cfg.per_layer) w += L.pl_gate.code_bytes() + L.pl_gate.scale_bytes() + L.pl_proj.code_bytes() + L.pl_proj.scale_bytes();
        const uint64_t n = (uint64_t)d->pos + 1 < L.window ? (uint64_t)d->pos + 1 : L.window;
        kv += 2ull * L.kvh * n * L.dim * 2;
    }
    if (weight_bytes) *weight_bytes = w;
    if (cache_bytes) *cache_bytes = kv;
    return OK;
}

int tb_decoder_step_launches(tb_decoder* d, uint32_t* launches) {
    if (!d || !launches) return fail(OUT_OF_RANGE, "null argument");
    *launches = d->fused ? 1 : (d->step_count ? d->step_count : 2 + 5 * d->cfg.layers);
    return OK;
}

int tb_decoder_timeline(tb_decoder* d, uint32_t token, uint64_t* host_out, uint32_t* phases) {
    TB_TRY(ready(d, 1));
    if (d->running) return fail(OUT_OF_RANGE, "tb_decoder_timeline: a generation is running; stop it first");
    const uint32_t count = d->fused ? d->phase_count : (d->step_count ? d->step_count : 2 + 5 * d->cfg.layers);
    if (phases) *phases = count;
    if (!host_out) return OK;
    const size_t bytes = (size_t)2 * count * 4 * sizeof(unsigned long long);
    cudaStream_t s = d->ctx->stream;
    unsigned long long* dev = nullptr;
    TB_CUDA(cudaMalloc(&dev, bytes));
    cudaError_t e = cudaMemsetAsync(dev, 0, bytes, s);
    int st = OK;
    if (e == cudaSuccess) st = feed_token(d, token);
    if (d->fused) {
        if (e == cudaSuccess && st == OK) st = launch_step(d->ctx, d->phase_dev[0], d->phase_count, d->grid_counter, d->state, dev);
        if (e == cudaSuccess && st == OK) e = cudaMemcpyAsync(host_out, dev, bytes, cudaMemcpyDeviceToHost, s);
    } else if (e == cudaSuccess && st == OK) {
        // One launch per phase: the step is captured once more with every kernel told where to leave its stamps, and
        // replayed as a graph so that the host's launch cost stays out of the picture.  Kernel i's eight words are the
        // first block's four stamps, then the last block's; they are reordered to [block][phase][4] on the way out.
        uint32_t* word = nullptr;
        e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&word), d->words, 0);
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        if (e == cudaSuccess) e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            d->stamps = dev;
            st = step_ops(d, word);
            d->stamps = nullptr;
            e = cudaStreamEndCapture(s, &graph);
        }
        if (e == cudaSuccess && st == OK) e = cudaGraphInstantiate(&exec, graph, 0);
        if (e == cudaSuccess && st == OK) e = cudaGraphLaunch(exec, s);
        std::vector<unsigned long long> raw((size_t)count * 8);
        if (e == cudaSuccess && st == OK) e = cudaMemcpyAsync(raw.data(), dev, bytes, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess && st == OK) e = cudaStreamSynchronize(s);
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        if (e == cudaSuccess && st == OK)
            for (uint32_t i = 0; i < count; i++)
                for (int b = 0; b < 2; b++)
                    for (int k = 0; k < 4; k++) host_out[((size_t)b * count + i) * 4 + k] = raw[(size_t)i * 8 + b * 4 + k];
    }
    if (e == cudaSuccess && st == OK) e = cudaStreamSynchronize(s);
    cudaFree(dev);
    if (e != cudaSuccess) return cuda_fail(e, "tb_decoder_timeline");
    if (st == OK) d->pos++;
    return st;
}

int tb_decoder_hidden(tb_decoder* d, float* host_out) {
    if (!d || !host_out) return fail(OUT_OF_RANGE, "null argument");
    TB_CUDA(cudaMemcpyAsync(host_out, d->x[d->final_x], (size_t)d->cfg.hidden * 4, cudaMemcpyDeviceToHost, d->ctx->stream));
    TB_CUDA(cudaStreamSynchronize(d->ctx->stream));
    return OK;
}

// ---- the host-RAM tier: Decoder::park and Parked::resume (crates/tachyon/src/model/decode.rs:235-247, 452-463) ------------

struct tb_parked {
    tb_context* ctx = nullptr;
    tb_config cfg = {};
    tb_settings settings = {};
    std::vector<uint8_t> global;
    std::vector<float> scalars;  // every layer's layer_scalar (host-side values, as Parked keeps `scalars`)
    char* weights = nullptr;     // pinned: every weight tensor, each from a multiple of 256 bytes, in for_each_weight's order
    size_t weights_bytes = 0;
    char* host_table = nullptr;  // pinned, mapped: the per-layer table, when the decoder kept it there
    size_t table_bytes = 0;
};

size_t tb_decoder_bytes(const tb_decoder* d) {
    if (!d) return 0;
    size_t copy = 0;
    if (d->copy)
        for (const Layer& L : d->layers)
            for (const Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) copy += ((size_t)m->rows * m->cols + 127) / 128 * 128 * 2;
    return d->arena_bytes + copy;
}

size_t tb_decoder_shadow_bytes(const tb_decoder* d) { return d ? d->shadow_bytes : 0; }

void tb_decoder_drop_shadow(tb_decoder* d) {
    if (!d || !d->shadow) return;
    cudaFreeHost(d->shadow);
    d->shadow = nullptr, d->shadow_bytes = 0;
}

size_t tb_decoder_parked_bytes(tb_decoder* d) { return d ? weight_bytes(d) + host_table_bytes(d) : 0; }

int tb_decoder_park(tb_decoder* d, tb_parked** out) {
    if (!d || !out) return fail(OUT_OF_RANGE, "tb_decoder_park: null argument");
    *out = nullptr;
    if (d->running) TB_TRY(tb_decoder_stop(d));
    cudaStream_t s = d->ctx->stream;
    TB_CUDA(cudaStreamSynchronize(s));
    const size_t bytes = weight_bytes(d);
    char* pinned = d->shadow;
    if (pinned == nullptr) {
        const cudaError_t e = cudaHostAlloc(&pinned, bytes, cudaHostAllocDefault);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(OUT_OF_MEMORY, "tb_decoder_park: no pinned memory for the weights (" + std::to_string(bytes) + " bytes)");
        }
        size_t at = 0;
        cudaError_t err = cudaSuccess;
        for_each_weight(d, [&](void* ptr, size_t n) {
            if (err == cudaSuccess) err = cudaMemcpyAsync(pinned + at, ptr, n, cudaMemcpyDeviceToHost, s);
            at += (n + 255) / 256 * 256;
        });
        if (err == cudaSuccess) err = cudaStreamSynchronize(s);
        if (err != cudaSuccess) {
            cudaFreeHost(pinned);
            return cuda_fail(err, "tb_decoder_park");
        }
    }
    tb_parked* p = new tb_parked();
    p->ctx = d->ctx, p->cfg = d->cfg, p->settings = d->settings, p->global = d->global;
    p->cfg.global = nullptr;
    for (const Layer& L : d->layers) p->scalars.push_back(L.layer_scalar);
    p->weights = pinned, p->weights_bytes = bytes;
    p->host_table = d->host_table, p->table_bytes = host_table_bytes(d);
    d->shadow = nullptr, d->shadow_bytes = 0, d->host_table = nullptr;  // theirs now
    tb_decoder_close(d);
    *out = p;
    return OK;
}

size_t tb_parked_bytes(const tb_parked* p) { return p ? p->weights_bytes + p->table_bytes : 0; }

void tb_parked_close(tb_parked* p) {
    if (!p) return;
    if (p->weights) cudaFreeHost(p->weights);
    if (p->host_table) cudaFreeHost(p->host_table);
    delete p;
}

int tb_parked_resume(tb_parked* p, const tb_settings* settings, tb_decoder** out) {
    if (!p || !settings || !out) return fail(OUT_OF_RANGE, "tb_parked_resume: null argument");
    *out = nullptr;
    if ((settings->weight_bits == 4) != (p->settings.weight_bits == 4) || (settings->host_table != 0) != (p->settings.host_table != 0))
        return fail(OUT_OF_RANGE, "tb_parked_resume: the weight format and the place of the per-layer table are the parked model's");
    tb_config cfg = p->cfg;
    cfg.global = p->global.data();
    tb_decoder* d = nullptr;
    TB_TRY(open_decoder(p->ctx, &cfg, settings, p->host_table, &d));
    p->host_table = nullptr, p->table_bytes = 0;  // the decoder's now
    for (size_t i = 0; i < d->layers.size(); i++) d->layers[i].layer_scalar = p->scalars[i];
    // One copy of the weights at the link's speed on a stream of its own, while the step is recorded as tb_decoder_build does
    // (decode.rs:452-463).  The build's trial pass may read weights that have not arrived: its results are thrown away by
    // the reset behind it, and the parked copy stays alive and unwritten until both streams are done.
    cudaStream_t s = d->ctx->stream, cs = nullptr;
    cudaError_t err = cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&d->weights_ready, cudaEventDisableTiming);
    // The arena came from the pool in the order of the context's stream: the copies' stream joins that order first.
    if (err == cudaSuccess) err = cudaEventRecord(d->weights_ready, s);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(cs, d->weights_ready, 0);
    size_t at = 0;
    for_each_weight(d, [&](void* ptr, size_t n) {
        if (err == cudaSuccess) err = cudaMemcpyAsync(ptr, p->weights + at, n, cudaMemcpyHostToDevice, cs);
        at += (n + 255) / 256 * 256;
    });
    if (err == cudaSuccess) err = cudaEventRecord(d->weights_ready, cs);
    int st = err == cudaSuccess ? OK : cuda_fail(err, "tb_parked_resume");
    if (st == OK) st = tb_decoder_build(d);
    if (cs) {
        const cudaError_t e1 = cudaStreamSynchronize(cs), e2 = cudaStreamSynchronize(s);
        if (st == OK && (e1 != cudaSuccess || e2 != cudaSuccess)) st = cuda_fail(e1 != cudaSuccess ? e1 : e2, "tb_parked_resume");
        cudaStreamDestroy(cs);
    }
    if (d->weights_ready) cudaEventDestroy(d->weights_ready), d->weights_ready = nullptr;
    if (st == OK) st = tb_decoder_reset(d);  // whatever the trial pass left behind
    if (st != OK) {
        // Back as it was: the table returns to the parked model, which stays usable.
        p->host_table = d->host_table, p->table_bytes = host_table_bytes(d);
        d->host_table = nullptr;
        tb_decoder_close(d);
        return st;
    }
    d->shadow = p->weights, d->shadow_bytes = p->weights_bytes;  // freeing pinned memory costs about as much as the copy (decode.rs:449-451)
    p->weights = nullptr;
    tb_parked_close(p);
    *out = d;
    return OK;
}

// The device memory a decoder of this shape takes (Engine's `need`, engine.rs:214): the arena and, where the settings ask for
// it (2, or automatic with chunks of 256 tokens and more), the prefill copy.  Nothing is allocated.
int tb_decoder_footprint(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, size_t* bytes) {
    if (!ctx || !cfg || !settings || !bytes) return fail(OUT_OF_RANGE, "tb_decoder_footprint: null argument");
    TB_TRY(validate(*cfg, *settings));
    tb_decoder d;
    d.ctx = ctx, d.cfg = *cfg, d.settings = *settings;
    d.fused = settings->fused != 0;
    d.global.resize(cfg->layers);
    for (uint32_t i = 0; i < cfg->layers; i++)
        d.global[i] = cfg->global ? cfg->global[i] : (cfg->global_every ? ((i + 1) % cfg->global_every == 0) : 0);
    d.cfg.global = nullptr;
    d.layers.resize(cfg->layers);
    layout(&d, nullptr);
    size_t copy = 0;
    const char* env = getenv("TACHYON_B200_PREFILL_COPY");
    const uint32_t want = settings->prefill_copy;
    const bool off = want == 1 || (want == 0 && env != nullptr && env[0] == '0') || settings->chunk == 0 || cfg->hidden % 64 != 0 || cfg->ffn % 64 != 0 ||
                     (want == 0 && settings->chunk < COPY_MIN_TOKENS);
    if (!off)
        for (const Layer& L : d.layers)
            for (const Mat* m : {&L.qkv, &L.o, &L.gate_up, &L.down}) copy += ((size_t)m->rows * m->cols + 127) / 128 * 128 * 2;
    *bytes = d.arena_bytes + copy;
    return OK;
}

}  // extern "C"
