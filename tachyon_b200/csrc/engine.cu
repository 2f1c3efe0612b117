// Model residency: which of the loaded decoders are in VRAM, which are parked in pinned host memory, which are only on disk.
// The rules are the reference engine's (crates/tachyon/src/engine.rs:203-223 load, 243-250 unload, 271-283 tier,
// 309-325 expire, 386-453 resident / room / bring / evict / used / hosted): a VRAM limit and a host-tier limit; a model that
// is asked for comes into VRAM, moving out the least recently used models that may go (not pinned, not the one asked for)
// until it fits; a model moved out is parked in the host tier if it fits there, after freeing the least recently used
// pinned memory (a resident model's kept copy first dropped, a parked model sent to disk), else it goes to disk; a
// keep-alive that has run out sends a model to disk at the next call.  Host code only: the decoders do the GPU work.
// Encoders are held by name too (engine.rs:54-55, 225-232, 244-262): always in VRAM, counted against the limit, dropped when
// their keep-alive runs out; decoders move out to make room for one, an encoder never moves.
// Not here: tokenizer, chat template and towers.
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/tachyon_b200.h"
#include "internal.h"

namespace {

using Clock = std::chrono::steady_clock;

enum Place { AT_VRAM = TB_TIER_VRAM, AT_HOST = TB_TIER_HOST, AT_DISK = TB_TIER_DISK };

struct Model {
    std::string name, weights, host;  // host: the per-layer table's file, or empty
    tb_config cfg = {};
    std::vector<uint8_t> global;
    tb_load load = {};
    size_t need = 0;              // VRAM it takes when resident
    uint64_t used = 0;            // the engine's tick at its last use
    bool ends = false;            // has a keep-alive that can run out
    Clock::time_point until;
    Place at = AT_DISK;
    tb_decoder* dec = nullptr;    // AT_VRAM
    tb_parked* parked = nullptr;  // AT_HOST

    void drop() {
        if (dec) tb_decoder_close(dec), dec = nullptr;
        if (parked) tb_parked_close(parked), parked = nullptr;
        at = AT_DISK;
    }
    // Model::touch (engine.rs:149-153): used now, the keep-alive starts again.
    void touch(uint64_t tick) {
        used = tick;
        ends = load.keep_alive_ms != UINT64_MAX;
        if (ends) until = Clock::now() + std::chrono::milliseconds(load.keep_alive_ms);
    }
    const tb_config* config() {
        cfg.global = global.empty() ? nullptr : global.data();
        return &cfg;
    }
};

// Held (engine.rs:158-168): a loaded encoder, how long it stays after a use, whether it is pinned.
struct Held {
    std::string name;
    tb_encoder* enc = nullptr;
    uint64_t keep_ms = UINT64_MAX;
    bool pin = false, ends = false;
    Clock::time_point until;

    void touch() {
        ends = keep_ms != UINT64_MAX;
        if (ends) until = Clock::now() + std::chrono::milliseconds(keep_ms);
    }
    uint64_t left_ms(Clock::time_point now) const {
        if (!ends || pin) return UINT64_MAX;
        return until > now ? (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(until - now).count() : 0;
    }
};

}  // namespace

struct tb_engine {
    tb_context* ctx = nullptr;
    size_t limits[2] = {0, 0};  // VRAM, host tier
    uint64_t tick = 0;
    std::vector<Model> models;
    std::vector<Held> encoders;

    int held(const char* name) const {
        for (size_t i = 0; i < encoders.size(); i++)
            if (encoders[i].name == name) return (int)i;
        return -1;
    }

    int find(const char* name) const {
        for (size_t i = 0; i < models.size(); i++)
            if (models[i].name == name) return (int)i;
        return -1;
    }
    size_t used() const {
        size_t n = 0;
        for (const Held& h : encoders) n += tb_encoder_bytes(h.enc);
        for (const Model& m : models)
            if (m.at == AT_VRAM) n += m.need;
        return n;
    }
    size_t hosted() const {
        size_t n = 0;
        for (const Model& m : models) n += m.at == AT_HOST ? tb_parked_bytes(m.parked) : m.at == AT_VRAM ? tb_decoder_shadow_bytes(m.dec) : 0;
        return n;
    }

    // engine.rs:420-441
    int evict(size_t i) {
        Model& m = models[i];
        if (m.at != AT_VRAM) return tb::OK;
        const size_t bytes = tb_decoder_parked_bytes(m.dec);
        if (bytes > limits[1]) return m.drop(), tb::OK;
        while (hosted() - tb_decoder_shadow_bytes(m.dec) + bytes > limits[1]) {
            // Something else holds pinned memory: `bytes` alone fits.  The least recently used holder gives way.
            int least = -1;
            for (size_t j = 0; j < models.size(); j++) {
                if (j == i) continue;
                const Model& o = models[j];
                const bool holds = o.at == AT_HOST || (o.at == AT_VRAM && tb_decoder_shadow_bytes(o.dec) > 0);
                if (holds && (least < 0 || o.used < models[least].used)) least = (int)j;
            }
            if (least < 0) break;
            if (models[least].at == AT_VRAM) tb_decoder_drop_shadow(models[least].dec);
            else models[least].drop();
        }
        tb_parked* parked = nullptr;
        const int st = tb_decoder_park(m.dec, &parked);
        if (st != tb::OK) return st;  // the decoder stays where it is
        m.dec = nullptr, m.parked = parked, m.at = AT_HOST;
        return tb::OK;
    }

    // engine.rs:394-404
    int room(size_t need, int keep) {
        while (used() + need > limits[0]) {
            int least = -1;
            for (size_t j = 0; j < models.size(); j++) {
                const Model& o = models[j];
                if ((int)j == keep || o.load.pin || o.at != AT_VRAM) continue;
                if (least < 0 || o.used < models[least].used) least = (int)j;
            }
            if (least < 0) {
                const size_t free_bytes = limits[0] > used() ? limits[0] - used() : 0;
                return tb::fail(tb::OUT_OF_MEMORY, "engine: " + std::to_string(need) + " bytes of VRAM needed, " + std::to_string(free_bytes) + " free of the limit, and nothing may move out");
            }
            const int st = evict((size_t)least);
            if (st != tb::OK) return st;
        }
        return tb::OK;
    }

    // engine.rs:407-415
    int bring(size_t i) {
        Model& m = models[i];
        if (m.at == AT_VRAM) return tb::OK;
        if (m.at == AT_HOST) {
            tb_decoder* dec = nullptr;
            const int st = tb_parked_resume(m.parked, &m.load.settings, &dec);
            if (st != tb::OK) return st;  // still parked
            m.parked = nullptr, m.dec = dec, m.at = AT_VRAM;
            return tb::OK;
        }
        tb_decoder* dec = nullptr;
        int st = tb_decoder_open(ctx, m.config(), &m.load.settings, &dec);
        if (st == tb::OK) st = tb_decoder_load_wpk(dec, m.weights.c_str(), 0);
        if (st == tb::OK && !m.host.empty()) st = tb_decoder_load_wpk(dec, m.host.c_str(), 0);
        if (st == tb::OK) st = tb_decoder_build(dec);
        if (st != tb::OK) {
            if (dec) tb_decoder_close(dec);
            return st;
        }
        m.dec = dec, m.at = AT_VRAM;
        return tb::OK;
    }

    // engine.rs:386-391
    int resident(size_t i) {
        if (models[i].at != AT_VRAM) {
            const int st = room(models[i].need, (int)i);
            if (st != tb::OK) return st;
        }
        return bring(i);
    }

    // engine.rs:309-325
    int expire() {
        const Clock::time_point now = Clock::now();
        bool freed = false;
        for (Model& m : models)
            if (m.at != AT_DISK && !m.load.pin && m.ends && m.until <= now) freed = freed || m.at == AT_VRAM, m.drop();
        for (size_t i = encoders.size(); i-- > 0;)
            if (!encoders[i].pin && encoders[i].ends && encoders[i].until <= now) {
                tb_encoder_close(encoders[i].enc);
                encoders.erase(encoders.begin() + (long)i);
                freed = true;
            }
        return freed ? tb_context_trim(ctx) : tb::OK;  // the VRAM goes back to the system, not only to the pool
    }
};

extern "C" {

int tb_engine_new(tb_context* ctx, size_t vram_limit, size_t host_limit, tb_engine** out) {
    if (!ctx || !out) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_new: null argument");
    *out = nullptr;
    if (vram_limit == 0) {  // 70 % of the GPU's memory (engine.rs:194)
        size_t free_bytes = 0, total = 0;
        TB_CUDA(cudaSetDevice(ctx->gpu));
        TB_CUDA(cudaMemGetInfo(&free_bytes, &total));
        vram_limit = total / 10 * 7;
    }
    if (host_limit == 0) {  // half the machine's RAM (engine.rs:195)
        const long pages = sysconf(_SC_PHYS_PAGES), page = sysconf(_SC_PAGESIZE);
        host_limit = pages > 0 && page > 0 ? (size_t)pages * (size_t)page / 2 : (size_t)8 << 30;
    }
    tb_engine* e = new tb_engine();
    e->ctx = ctx, e->limits[0] = vram_limit, e->limits[1] = host_limit;
    *out = e;
    return tb::OK;
}

void tb_engine_close(tb_engine* e) {
    if (!e) return;
    for (Model& m : e->models) m.drop();
    for (Held& h : e->encoders) tb_encoder_close(h.enc);
    delete e;
}

int tb_engine_unload(tb_engine* e, const char* name, int* was_loaded) {
    if (!e || !name) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_unload: null argument");
    const int i = e->find(name), k = e->held(name);
    if (was_loaded) *was_loaded = i >= 0 || k >= 0;
    if (k >= 0) {
        tb_encoder_close(e->encoders[k].enc);
        e->encoders.erase(e->encoders.begin() + k);
        if (i < 0) return tb_context_trim(e->ctx);
    }
    if (i >= 0) {
        const bool vram = e->models[i].at == AT_VRAM;
        e->models[i].drop();
        e->models.erase(e->models.begin() + i);
        if (vram || k >= 0) return tb_context_trim(e->ctx);  // engine.rs:247-248
    }
    return tb::OK;
}

int tb_engine_expire(tb_engine* e) {
    if (!e) return tb::fail(tb::OUT_OF_RANGE, "null engine");
    return e->expire();
}

int tb_engine_load(tb_engine* e, const char* name, const tb_config* cfg, const tb_load* load, const char* weights_path, const char* host_path) {
    if (!e || !name || !cfg || !load || !weights_path) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_load: null argument");
    tb_engine_unload(e, name, nullptr);
    e->expire();
    Model m;
    m.name = name, m.weights = weights_path, m.host = host_path ? host_path : "";
    m.cfg = *cfg, m.load = *load;
    if (cfg->global) m.global.assign(cfg->global, cfg->global + cfg->layers);
    TB_TRY(tb_decoder_footprint(e->ctx, m.config(), &load->settings, &m.need));
    m.touch(++e->tick);
    e->models.push_back(std::move(m));
    const int st = e->resident(e->models.size() - 1);
    if (st != tb::OK) e->models.back().drop(), e->models.pop_back();
    return st;
}

int tb_engine_decoder(tb_engine* e, const char* name, tb_decoder** out) {
    if (!e || !name || !out) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_decoder: null argument");
    *out = nullptr;
    e->expire();
    const int i = e->find(name);
    if (i < 0) return tb::fail(tb::NO_MODEL, std::string("engine: no model named ") + name);
    TB_TRY(e->resident((size_t)i));
    e->models[i].touch(++e->tick);
    *out = e->models[i].dec;
    return tb::OK;
}

int tb_engine_feed(tb_engine* e, const char* name, const uint32_t* tokens, uint32_t n, uint32_t* first) {
    if (!tokens || n == 0 || !first) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_feed: an empty prompt, or nowhere to put the answer's first token");
    tb_decoder* dec = nullptr;
    TB_TRY(tb_engine_decoder(e, name, &dec));
    TB_TRY(tb_decoder_reset(dec));
    if (n > 1) TB_TRY(tb_decoder_prefill(dec, tokens, n - 1));
    return tb_decoder_step(dec, tokens[n - 1], first);
}

int tb_engine_tier(const tb_engine* e, const char* name, int* tier) {
    if (!e || !name || !tier) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_tier: null argument");
    if (e->held(name) >= 0) return *tier = TB_TIER_VRAM, tb::OK;
    const int i = e->find(name);
    if (i < 0) return tb::fail(tb::NO_MODEL, std::string("engine: no model named ") + name);
    *tier = e->models[i].at;
    return tb::OK;
}

int tb_engine_models(const tb_engine* e, tb_loaded* out, size_t capacity, size_t* count) {
    if (!e || !count || (capacity && !out)) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_models: null argument");
    *count = e->models.size() + e->encoders.size();
    const Clock::time_point now = Clock::now();
    for (size_t i = 0; i < e->models.size() && i < capacity; i++) {
        const Model& m = e->models[i];
        memset(&out[i], 0, sizeof(tb_loaded));
        strncpy(out[i].name, m.name.c_str(), sizeof(out[i].name) - 1);
        out[i].tier = m.at;
        out[i].vram = m.at == AT_VRAM ? m.need : 0;
        out[i].left_ms = UINT64_MAX;
        if (m.ends && !m.load.pin) out[i].left_ms = m.until > now ? (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(m.until - now).count() : 0;
    }
    for (size_t k = 0, i = e->models.size(); k < e->encoders.size() && i < capacity; k++, i++) {  // decoders, then encoders (engine.rs:294)
        const Held& h = e->encoders[k];
        memset(&out[i], 0, sizeof(tb_loaded));
        strncpy(out[i].name, h.name.c_str(), sizeof(out[i].name) - 1);
        out[i].tier = TB_TIER_VRAM;
        out[i].vram = tb_encoder_bytes(h.enc);
        out[i].left_ms = h.left_ms(now);
    }
    return tb::OK;
}

// Engine::load_encoder (engine.rs:225-232): room made by moving decoders out, then the encoder opened from its files and kept as
// asked; one of that name, decoder or encoder, is unloaded first.
int tb_engine_load_encoder(tb_engine* e, const char* name, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, uint64_t keep_alive_ms, int pin,
                           const char* weights_path, const char* host_path) {
    if (!e || !name || !cfg || !weights_path) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_load_encoder: null argument");
    tb_engine_unload(e, name, nullptr);
    e->expire();
    // The layers' matrices come in f16 if the file holds them so: they are allocated beside the arena when loaded.
    int f16 = 0;
    {
        tb_wpk* w = nullptr;
        TB_TRY(tb_wpk_open(weights_path, &w));
        tb_wpk_info info;
        for (uint32_t i = 0; i < tb_wpk_count(w) && !f16; i++)
            if (tb_wpk_tensor(w, i, &info) == tb::OK && info.rank == 2 && info.dtype == 1 && strcmp(info.name, "embed") != 0) f16 = 1;
        tb_wpk_close(w);
    }
    size_t need = 0;
    TB_TRY(tb_encoder_footprint(e->ctx, cfg, tokens, sequences, f16, &need));
    TB_TRY(e->room(need, -1));
    Held h;
    h.name = name, h.keep_ms = keep_alive_ms, h.pin = pin != 0;
    int st = tb_encoder_open(e->ctx, cfg, tokens, sequences, &h.enc);
    if (st == tb::OK) st = tb_encoder_load_wpk(h.enc, weights_path, 0);
    if (st == tb::OK && host_path && host_path[0]) st = tb_encoder_load_wpk(h.enc, host_path, 0);
    if (st != tb::OK) {
        if (h.enc) tb_encoder_close(h.enc);
        return st;
    }
    h.touch();
    e->encoders.push_back(h);
    return tb::OK;
}

// Engine::encoder (engine.rs:244-250): encoder `name`, its keep-alive started again.
int tb_engine_encoder(tb_engine* e, const char* name, tb_encoder** out) {
    if (!e || !name || !out) return tb::fail(tb::OUT_OF_RANGE, "tb_engine_encoder: null argument");
    *out = nullptr;
    e->expire();
    const int k = e->held(name);
    if (k < 0) return tb::fail(tb::NO_MODEL, std::string("engine: no model named ") + name);
    e->encoders[k].touch();
    *out = e->encoders[k].enc;
    return tb::OK;
}

// Engine::embed (engine.rs:258-262) from token ids: the tokenizer stays with the caller.
int tb_engine_embed(tb_engine* e, const char* name, const uint32_t* ids, const uint32_t* lens, uint32_t sequences, float* out_host) {
    tb_encoder* enc = nullptr;
    TB_TRY(tb_engine_encoder(e, name, &enc));
    return tb_encoder_embed(enc, ids, lens, sequences, out_host);
}

int tb_engine_usage(const tb_engine* e, size_t* vram, size_t* host) {
    if (!e) return tb::fail(tb::OUT_OF_RANGE, "null engine");
    if (vram) *vram = e->used();
    if (host) *host = e->hosted();
    return tb::OK;
}

}  // extern "C"
