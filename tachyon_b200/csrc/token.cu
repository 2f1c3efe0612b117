// Text to token ids and back: the reference's tokenizer for Gemma's SentencePiece-style BPE and for Metaspace vocabularies
// (crates/tachyon/src/token/mod.rs:1-11, 97-127, 290-420): spaces become U+2581, the text is cut into characters, characters
// the vocabulary lacks fall back to their UTF-8 bytes (`<0xHH>` tokens), and adjacent tokens merge, lowest-ranked pair first
// (leftmost among equals), until no merge applies.  Text is encoded literally: a special token's text in a prompt stays
// text; special tokens enter by id only, from the chat template (token/chat.rs), so user text cannot forge a turn.
// Read from a Hugging Face tokenizer.json, or from the reference's stored form (`TACHYTOK`, mod.rs:422-455), which this
// file reads and writes word for word so that a converted model's tokenizer.tok loads as it is.  Byte-level BPE (GPT-2's
// scheme, token/bytes.rs: every byte a symbol, the text first cut into pieces by GPT-2's pattern, cl100k's or o200k's, matched
// by hand) and an NFC normalizer (token/unicode.rs) are taken too, the Unicode data generated into unicode_tables.h.  Host code only.
#include <algorithm>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "../../include/tachyon_b200.h"
#include "internal.h"
#include "unicode_tables.h"

namespace {

using tb::fail;

constexpr uint32_t NONE = UINT32_MAX;
constexpr uint32_t META = 1, BYTES = 2, SPLIT = 4, PREPEND = 8, BYTE_LEVEL = 16, CL100K = 32, NFC = 64, O200K = 128;  // mod.rs:25-40
constexpr size_t DIRECT = 0x20000;  // characters with an entry of their own in `chars`: the first two planes
constexpr uint32_t BAR = 0x2581;    // the visible space

// ---- a small JSON reader: enough for tokenizer.json -----------------------------------------------------------------------------
struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double n = 0;
    std::string s;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    const Json* get(const char* key) const {
        if (kind != OBJ) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    const char* str() const { return kind == STR ? s.c_str() : nullptr; }
    bool is(const char* key, const char* want) const {
        const Json* v = get(key);
        return v && v->kind == STR && v->s == want;
    }
    bool flag(const char* key, bool want) const {
        const Json* v = get(key);
        return v && v->kind == BOOL && v->b == want;
    }
};

void put_utf8(std::string& out, uint32_t c) {
    if (c < 0x80) out += (char)c;
    else if (c < 0x800) out += (char)(0xC0 | c >> 6), out += (char)(0x80 | (c & 63));
    else if (c < 0x10000) out += (char)(0xE0 | c >> 12), out += (char)(0x80 | (c >> 6 & 63)), out += (char)(0x80 | (c & 63));
    else out += (char)(0xF0 | c >> 18), out += (char)(0x80 | (c >> 12 & 63)), out += (char)(0x80 | (c >> 6 & 63)), out += (char)(0x80 | (c & 63));
}

struct JsonReader {
    const char *p, *end;
    bool bad = false;

    void space() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    bool eat(char c) {
        space();
        if (p < end && *p == c) return p++, true;
        return false;
    }
    uint32_t hex4() {
        uint32_t v = 0;
        for (int k = 0; k < 4; k++, p++) {
            if (p >= end) return bad = true, 0;
            const char c = *p;
            v = v << 4 | (uint32_t)(c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : (bad = true, 0));
        }
        return v;
    }
    std::string string() {
        std::string out;
        if (!eat('"')) return bad = true, out;
        while (p < end && *p != '"') {
            if (*p != '\\') {
                out += *p++;
                continue;
            }
            if (++p >= end) break;
            const char c = *p++;
            if (c == 'n') out += '\n';
            else if (c == 't') out += '\t';
            else if (c == 'r') out += '\r';
            else if (c == 'b') out += '\b';
            else if (c == 'f') out += '\f';
            else if (c == 'u') {
                uint32_t v = hex4();
                if (v >= 0xD800 && v < 0xDC00 && p + 1 < end && p[0] == '\\' && p[1] == 'u') {  // a surrogate pair
                    p += 2;
                    const uint32_t lo = hex4();
                    v = 0x10000 + ((v - 0xD800) << 10) + (lo - 0xDC00);
                }
                put_utf8(out, v);
            } else out += c;  // quote, backslash, slash
        }
        if (p >= end) return bad = true, out;
        p++;
        return out;
    }
    Json value(int depth = 0) {
        Json j;
        space();
        if (p >= end || depth > 64) return bad = true, j;
        if (*p == '{') {
            p++, j.kind = Json::OBJ;
            if (eat('}')) return j;
            do {
                std::string key = string();
                if (!eat(':')) return bad = true, j;
                j.obj.emplace_back(std::move(key), value(depth + 1));
            } while (!bad && eat(','));
            if (!eat('}')) bad = true;
        } else if (*p == '[') {
            p++, j.kind = Json::ARR;
            if (eat(']')) return j;
            do j.arr.push_back(value(depth + 1));
            while (!bad && eat(','));
            if (!eat(']')) bad = true;
        } else if (*p == '"') {
            j.kind = Json::STR, j.s = string();
        } else if (end - p >= 4 && !strncmp(p, "true", 4)) {
            j.kind = Json::BOOL, j.b = true, p += 4;
        } else if (end - p >= 5 && !strncmp(p, "false", 5)) {
            j.kind = Json::BOOL, p += 5;
        } else if (end - p >= 4 && !strncmp(p, "null", 4)) {
            p += 4;
        } else {
            const char* from = p;
            while (p < end && (strchr("+-.eE", *p) || (*p >= '0' && *p <= '9'))) p++;
            if (p == from) return bad = true, j;
            j.kind = Json::NUM, j.n = atof(std::string(from, p).c_str());
        }
        return j;
    }
};

// One character of UTF-8 at p (p < end): its code point and length; a byte that starts no character is U+FFFD, one byte long.
uint32_t next_char(const uint8_t* p, const uint8_t* end, size_t& len) {
    const uint32_t b = p[0];
    const size_t want = b < 0x80 ? 1 : b >> 5 == 6 ? 2 : b >> 4 == 14 ? 3 : b >> 3 == 30 ? 4 : 0;
    if (want == 0 || (size_t)(end - p) < want) return len = 1, 0xFFFD;
    uint32_t c = want == 1 ? b : b & (0x7Fu >> want);
    for (size_t k = 1; k < want; k++) {
        if (p[k] >> 6 != 2) return len = 1, 0xFFFD;
        c = c << 6 | (p[k] & 63u);
    }
    return len = want, c;
}

}  // namespace

namespace {

// ---- byte-level BPE: the byte a vocabulary character stands for, and the three patterns (token/bytes.rs) ------------------------
bool printable(uint32_t b) { return (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF); }

// Itself if printable, else the nth of the other bytes, written U+0100 + n; -1 if the character stands for no byte.
int byte_of(uint32_t c) {
    if (c < 256) return printable(c) ? (int)c : -1;
    if (c > 323) return -1;
    uint32_t n = c - 256;
    for (uint32_t b = 0; b < 256; b++)
        if (!printable(b) && n-- == 0) return (int)b;
    return -1;
}

uint32_t unicode_entry(uint32_t c) {
    size_t lo = 0, hi = sizeof(tb_unicode::RUNS) / sizeof(tb_unicode::RUNS[0]);
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (tb_unicode::RUNS[mid].last < c) lo = mid + 1;
        else hi = mid;
    }
    return lo < sizeof(tb_unicode::RUNS) / sizeof(tb_unicode::RUNS[0]) && tb_unicode::RUNS[lo].first <= c ? tb_unicode::RUNS[lo].entry : 0;
}

enum Class { LETTER, NUMBER, SPACE, OTHER };
bool is_letter(uint32_t c) { return unicode_entry(c) & 1u; }
bool is_number(uint32_t c) { return (unicode_entry(c) & 2u) != 0; }
bool is_white(uint32_t c) { return (unicode_entry(c) & 4u) != 0; }
uint32_t kind_of(uint32_t c) { return unicode_entry(c) >> 3; }  // to o200k: 1 upper or title, 2 lower, 3 either (modifier, other, mark), 0 none
Class class_of(uint32_t c) {
    const uint32_t e = unicode_entry(c);
    return (e & 1u) ? LETTER : (e & 2u) ? NUMBER : (e & 4u) ? SPACE : OTHER;
}

// ---- Unicode Normalization Form C (token/unicode.rs): canonical decomposition, canonical ordering, canonical composition -----
template <size_t N>
const tb_unicode::Run* find_first(const tb_unicode::Run (&table)[N], uint32_t key) {  // the entry whose `first` is key, or null
    size_t lo = 0, hi = N;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (table[mid].first < key) lo = mid + 1;
        else hi = mid;
    }
    return lo < N && table[lo].first == key ? &table[lo] : nullptr;
}

uint32_t combining_class(uint32_t c) {
    constexpr size_t N = sizeof(tb_unicode::COMBINING) / sizeof(tb_unicode::COMBINING[0]);
    size_t lo = 0, hi = N;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (tb_unicode::COMBINING[mid].last < c) lo = mid + 1;
        else hi = mid;
    }
    return lo < N && tb_unicode::COMBINING[lo].first <= c ? tb_unicode::COMBINING[lo].entry : 0;
}

void decompose(uint32_t c, std::vector<uint32_t>& out) {
    if (c >= 0xAC00 && c <= 0xD7A3) {  // a Hangul syllable: leading consonant, vowel, and maybe a trailing consonant
        const uint32_t s = c - 0xAC00, t = s % 28;
        out.push_back(0x1100 + s / 588), out.push_back(0x1161 + (s % 588) / 28);
        if (t) out.push_back(0x11A7 + t);
        return;
    }
    const tb_unicode::Run* d = c < 0xC0 ? nullptr : find_first(tb_unicode::DECOMPOSE, c);
    if (!d) return out.push_back(c);
    decompose(d->last, out);  // {character, first, second or 0}
    if (d->entry) out.push_back(d->entry);
}

uint32_t compose_pair(uint32_t a, uint32_t b) {
    if (a >= 0x1100 && a < 0x1113 && b >= 0x1161 && b < 0x1176) return 0xAC00 + ((a - 0x1100) * 21 + (b - 0x1161)) * 28;
    if (a >= 0xAC00 && a <= 0xD7A3 && (a - 0xAC00) % 28 == 0 && b > 0x11A7 && b < 0x11C3) return a + (b - 0x11A7);
    constexpr size_t N = sizeof(tb_unicode::COMPOSE) / sizeof(tb_unicode::COMPOSE[0]);
    size_t lo = 0, hi = N;  // {first, second, composite}, sorted by (first, second)
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        const tb_unicode::Run& e = tb_unicode::COMPOSE[mid];
        if (e.first < a || (e.first == a && e.last < b)) lo = mid + 1;
        else hi = mid;
    }
    return lo < N && tb_unicode::COMPOSE[lo].first == a && tb_unicode::COMPOSE[lo].last == b ? tb_unicode::COMPOSE[lo].entry : 0;
}

// The text in NFC, or nothing written and false when it is in NFC already as far as a quick look tells (nothing from U+0300 on).
bool nfc(const uint8_t* p, const uint8_t* end, std::string& out) {
    bool plain = true;
    for (const uint8_t* q = p; q < end && plain; q++) plain = *q < 0xCC;  // U+0300 is CC 80
    if (plain) return false;
    std::vector<uint32_t> cs;
    for (size_t n; p < end; p += n) decompose(next_char(p, end, n), cs);
    for (size_t i = 0; i < cs.size();) {  // canonical ordering: each run of marks sorted by class, equal classes keeping their order
        if (combining_class(cs[i]) == 0) {
            i++;
            continue;
        }
        size_t j = i;
        while (j < cs.size() && combining_class(cs[j]) != 0) j++;
        std::stable_sort(cs.begin() + (long)i, cs.begin() + (long)j, [](uint32_t a, uint32_t b) { return combining_class(a) < combining_class(b); });
        i = j;
    }
    // canonical composition: a character joins the last starter unless a character stands between them whose class is not
    // lower than its own (the marks between are sorted, so the last one's class decides; a starter joins only when adjacent)
    std::vector<uint32_t> r;
    size_t starter = SIZE_MAX;
    uint32_t last_class = 0;
    for (uint32_t c : cs) {
        const uint32_t k = combining_class(c);
        if (starter != SIZE_MAX) {
            const bool blocked = r.size() > starter + 1 && last_class >= k;
            const uint32_t joined = blocked ? 0 : compose_pair(r[starter], c);
            if (joined) {
                r[starter] = joined;
                continue;
            }
        }
        if (k == 0) starter = r.size();
        last_class = k;
        r.push_back(c);
    }
    out.clear();
    for (uint32_t c : r) put_utf8(out, c);
    return true;
}

// A stretch of text as characters; the matchers below give the characters of the pattern's match at i (at least one).
struct Chars {
    std::vector<uint32_t> c;
    size_t n() const { return c.size(); }
    template <typename P>
    size_t run(size_t i, size_t most, P keep) const {
        size_t k = 0;
        while (k < most && i + k < c.size() && keep(c[i + k])) k++;
        return k;
    }
    // 's 't 're 've 'm 'll 'd at i, in any case if `fold`
    size_t contraction(size_t i, bool fold) const {
        if (i + 1 >= c.size() || c[i] != '\'') return 0;
        auto low = [&](size_t j) -> uint32_t { return j < c.size() ? (fold && c[j] >= 'A' && c[j] <= 'Z' ? c[j] + 32 : c[j]) : 0; };
        const uint32_t a = low(i + 1), b = low(i + 2);
        if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
        if (((a == 'r' || a == 'v') && b == 'e') || (a == 'l' && b == 'l')) return 3;
        return 0;
    }
    // \s+(?!\S)|\s+ at i: the run, less its last character when more text follows and the run is longer than one
    size_t spaces(size_t i) const {
        const size_t k = run(i, SIZE_MAX, is_white);
        return (i + k < c.size() && k > 1) ? k - 1 : k;
    }
    size_t gpt2(size_t i) const {
        if (const size_t k = contraction(i, false)) return k;
        const size_t skip = c[i] == ' ' ? 1 : 0;
        if (i + skip < c.size()) {
            const Class first = class_of(c[i + skip]);
            if (first != SPACE) return skip + run(i + skip, SIZE_MAX, [&](uint32_t d) { return class_of(d) == first; });
        }
        return spaces(i);
    }
    // the last alternatives of cl100k and o200k: ` ?[^\s\p{L}\p{N}]+[\r\n]*` (with `slash`, [\r\n/]*) if `symbols`, else
    // \s*[\r\n]+|\s+(?!\S)|\s+
    size_t rest(size_t i, bool symbols, bool slash) const {
        if (symbols) {
            const size_t skip = c[i] == ' ' ? 1 : 0;
            size_t k = skip + run(i + skip, SIZE_MAX, [](uint32_t d) { return class_of(d) == OTHER; });
            return k + run(i + k, SIZE_MAX, [&](uint32_t d) { return d == '\r' || d == '\n' || (slash && d == '/'); });
        }
        const size_t k = run(i, SIZE_MAX, is_white);
        for (size_t j = k; j-- > 0;)
            if (c[i + j] == '\r' || c[i + j] == '\n') return j + 1;
        return spaces(i);
    }
    bool symbol_start(size_t i) const { return class_of(c[i]) == OTHER || (c[i] == ' ' && i + 1 < c.size() && class_of(c[i + 1]) == OTHER); }
    size_t cl100k(size_t i) const {
        if (const size_t k = contraction(i, true)) return k;
        const uint32_t c0 = c[i];
        const Class first = class_of(c0);
        if (first == LETTER) return run(i, SIZE_MAX, is_letter);
        if (first == NUMBER) return run(i, 3, is_number);
        if (c0 != '\r' && c0 != '\n' && i + 1 < c.size() && is_letter(c[i + 1])) return 1 + run(i + 1, SIZE_MAX, is_letter);
        return rest(i, symbol_start(i), false);
    }
    // U*W+ (or with `upper_first`, U+W*) at i, U = upper, title, modifier, other letters and marks, W = lower, modifier, other
    // letters and marks: the longest run of U that W can still follow, then the longest run of W; 0 if it does not match
    size_t word(size_t i, bool upper_first) const {
        size_t len = 0, most = 0;
        while (i + len < c.size() && kind_of(c[i + len]) != 0) len++;
        while (most < len && kind_of(c[i + most]) != 2) most++;
        auto end = [&](size_t a) {
            while (a < len && kind_of(c[i + a]) >= 2) a++;
            return a;
        };
        if (upper_first) return most > 0 ? end(most) : 0;
        for (size_t a = most + 1; a-- > 0;)
            if (end(a) > a) return end(a);
        return 0;
    }
    size_t o200k(size_t i) const {
        const uint32_t c0 = c[i];
        const bool prefix = c0 != '\r' && c0 != '\n' && !is_letter(c0) && !is_number(c0);
        for (int upper_first = 0; upper_first < 2; upper_first++)
            for (int with = prefix ? 1 : 0; with >= 0; with--) {  // each word alternative with its optional first character, then without
                if (i + (size_t)with >= c.size() && with) continue;
                const size_t k = word(i + (size_t)with, upper_first != 0);
                if (k > 0) return (size_t)with + k + contraction(i + (size_t)with + k, true);
            }
        if (is_number(c0)) return run(i, 3, is_number);
        return rest(i, symbol_start(i), true);
    }
};

}  // namespace

// The tables are the stored form's sections (mod.rs:47-78), ready to use as read.
struct tb_tokenizer {
    uint32_t flags = 0, unk = NONE;
    std::vector<uint32_t> offsets{0};  // where each token's text starts in `text`; one more entry than tokens
    std::vector<uint8_t> text;         // every token's text as decoding produces it: U+2581 already a space, byte tokens their byte
    std::vector<uint32_t> special;     // special tokens' ids, sorted
    std::vector<uint32_t> bytes;       // the `<0xHH>` token of each byte
    std::vector<uint32_t> chars;       // the token of each character below DIRECT
    std::vector<uint32_t> rare;        // (character, id) pairs of the single-character tokens above it
    std::vector<uint32_t> joins;       // characters some token joins to a following U+2581: no cut after them
    std::vector<uint32_t> added;       // added tokens that are not special, by first byte then longest first
    std::vector<uint32_t> merges;      // open addressing, entries (left, right, rank, merged)
    std::vector<uint32_t> words;       // open addressing table of tokens by their text (ignore_merges); kept for the stored form
    uint32_t frame[2] = {NONE, NONE};  // the special tokens the post-processor puts before and after a text

    size_t len() const { return offsets.size() - 1; }
    const uint8_t* token(uint32_t id, size_t& n) const {
        if ((size_t)id + 1 >= offsets.size()) return n = 0, text.data();
        n = offsets[id + 1] - offsets[id];
        return text.data() + offsets[id];
    }
    bool is_special(uint32_t id) const { return std::binary_search(special.begin(), special.end(), id); }
    uint32_t char_id(uint32_t c) const {
        if (c < chars.size()) return chars[c];
        for (size_t k = 0; k + 1 < rare.size(); k += 2)
            if (rare[k] == c) return rare[k + 1];
        return NONE;
    }
};

struct tb_detokenizer {
    std::vector<uint8_t> pending;
};

namespace {

size_t slot_of(uint64_t key, size_t mask) { return (size_t)((key * 0x9E3779B97F4A7C15ull) >> 40) & mask; }  // mod.rs:80-82

// Where (a, b) is in the merge table, or the free entry where it belongs.
size_t find_merge(const std::vector<uint32_t>& table, uint32_t a, uint32_t b) {
    const size_t mask = table.size() / 4 - 1;
    size_t i = slot_of((uint64_t)a << 32 | b, mask);
    while (table[4 * i] != NONE && !(table[4 * i] == a && table[4 * i + 1] == b)) i = (i + 1) & mask;
    return 4 * i;
}

uint64_t fnv(const uint8_t* p, size_t n) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (size_t i = 0; i < n; i++) h = (h ^ p[i]) * 0x100000001B3ull;
    return h;
}

size_t pow2_at_least(size_t n) {
    size_t p = 1;
    while (p < n) p <<= 1;
    return p;
}

std::vector<uint32_t> chars_of(const std::string& s) {
    std::vector<uint32_t> out;
    const uint8_t *p = reinterpret_cast<const uint8_t*>(s.data()), *end = p + s.size();
    for (size_t n; p < end; p += n) out.push_back(next_char(p, end, n));
    return out;
}

// Tokenizer::add_token (mod.rs:170-192): the token's decoded text, and its place in the byte and character tables.
void add_token(tb_tokenizer& t, uint32_t id, const std::string& name) {
    if ((t.flags & BYTE_LEVEL) && !t.is_special(id)) {
        // add_byte_token (mod.rs:199-204): a name of byte characters is those bytes; another (an added token's) is its own text
        std::vector<uint8_t> decoded;
        bool all = true;
        for (uint32_t c : chars_of(name)) {
            const int b = byte_of(c);
            all = all && b >= 0;
            decoded.push_back((uint8_t)(b < 0 ? 0 : b));
        }
        if (all && decoded.size() == 1) t.bytes[decoded[0]] = id;
        if (all) t.text.insert(t.text.end(), decoded.begin(), decoded.end());
        else t.text.insert(t.text.end(), name.begin(), name.end());
        t.offsets.push_back((uint32_t)t.text.size());
        return;
    }
    int byte = -1;
    if (name.size() == 6 && !name.compare(0, 3, "<0x") && name[5] == '>') {
        auto hex = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1; };
        const int hi = hex(name[3]), lo = hex(name[4]);
        if (hi >= 0 && lo >= 0) byte = hi * 16 + lo;
    }
    const bool special = t.is_special(id);
    if (byte >= 0 && (t.flags & BYTES) && !special) {
        t.bytes[byte] = id;
        t.text.push_back((uint8_t)byte);
    } else if ((t.flags & META) && !special) {
        for (size_t i = 0; i < name.size();) {
            if (i + 2 < name.size() && (uint8_t)name[i] == 0xE2 && (uint8_t)name[i + 1] == 0x96 && (uint8_t)name[i + 2] == 0x81) t.text.push_back(' '), i += 3;
            else t.text.push_back((uint8_t)name[i++]);
        }
    } else {
        t.text.insert(t.text.end(), name.begin(), name.end());
    }
    t.offsets.push_back((uint32_t)t.text.size());
    const std::vector<uint32_t> cs = chars_of(name);
    if (cs.size() == 1 && !special) {
        if (cs[0] < DIRECT) t.chars[cs[0]] = id;
        else t.rare.push_back(cs[0]), t.rare.push_back(id);
    }
}

struct Added {
    std::string content;
    uint32_t id;
    bool special;
};

// Tokenizer::build (mod.rs:129-168).
int build(tb_tokenizer& t, std::vector<std::pair<std::string, uint32_t>>& vocab, const std::vector<std::pair<std::string, std::string>>& merges,
          std::vector<uint32_t> special, std::vector<uint32_t> plain, const char* unk, uint32_t flags) {
    size_t n = 0;
    for (const auto& v : vocab) n = std::max(n, (size_t)v.second + 1);
    if (n > (1u << 26)) return fail(tb::FORMAT, "tokenizer: a token id beyond 2^26");
    std::vector<std::string> names(n);
    for (const auto& v : vocab) names[v.second] = v.first;
    // name -> id, the last entry of a name winning, by sorting (name, position)
    std::vector<size_t> order(vocab.size());
    for (size_t i = 0; i < order.size(); i++) order[i] = i;
    std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return vocab[a].first != vocab[b].first ? vocab[a].first < vocab[b].first : a < b; });
    auto id_of = [&](const std::string& s) -> uint32_t {
        auto it = std::upper_bound(order.begin(), order.end(), s, [&](const std::string& key, size_t i) { return key < vocab[i].first; });
        if (it == order.begin() || vocab[*(it - 1)].first != s) return NONE;
        return vocab[*(it - 1)].second;
    };
    std::sort(special.begin(), special.end());
    t.flags = flags, t.special = special;
    t.unk = unk ? id_of(unk) : NONE;
    t.bytes.assign(256, NONE), t.chars.assign(DIRECT, NONE);
    t.merges.assign(4 * std::max<size_t>(pow2_at_least(2 * merges.size()), 2), NONE);
    for (size_t id = 0; id < n; id++) add_token(t, (uint32_t)id, names[id]);
    for (size_t id = 0; id < n; id++) {
        if (t.is_special((uint32_t)id)) continue;
        const std::vector<uint32_t> cs = chars_of(names[id]);
        for (size_t k = 0; k + 1 < cs.size(); k++)
            if (cs[k + 1] == BAR && cs[k] != BAR) t.joins.push_back(cs[k]);
    }
    std::sort(t.joins.begin(), t.joins.end());
    t.joins.erase(std::unique(t.joins.begin(), t.joins.end()), t.joins.end());
    // matched (mod.rs:470-476): the added tokens that can match a text, by first byte then longest first; one with U+2581 never does
    for (uint32_t id : plain)
        if (id < n && !names[id].empty() && names[id].find("\xE2\x96\x81") == std::string::npos) t.added.push_back(id);
    std::sort(t.added.begin(), t.added.end(), [&](uint32_t a, uint32_t b) {
        const std::string &x = names[a], &y = names[b];
        if ((uint8_t)x[0] != (uint8_t)y[0]) return (uint8_t)x[0] < (uint8_t)y[0];
        if (x.size() != y.size()) return x.size() > y.size();
        return a < b;
    });
    for (size_t rank = 0; rank < merges.size(); rank++) {
        const std::string &a = merges[rank].first, &b = merges[rank].second;
        const uint32_t ia = id_of(a), ib = id_of(b), iab = id_of(a + b);
        if (ia == NONE || ib == NONE || iab == NONE) return fail(tb::FORMAT, "tokenizer: merge \"" + a + "\" + \"" + b + "\" names an unknown token");
        const size_t at = find_merge(t.merges, ia, ib);
        if (t.merges[at] == NONE) t.merges[at] = ia, t.merges[at + 1] = ib, t.merges[at + 2] = (uint32_t)rank, t.merges[at + 3] = iab;
    }
    return tb::OK;
}

int unsupported(const char* what) { return fail(tb::FORMAT, std::string("tokenizer: ") + what + " is not supported"); }

}  // namespace

namespace {

// Tokenizer::from_json (mod.rs:97-127) for the kinds taken here: BPE with optional byte fallback; no normalizer, or one that
// replaces spaces with U+2581; no pre-tokenizer, Gemma's split on spaces (which never splits once the spaces are U+2581), or
// a Metaspace with U+2581 that may split at every space and prepend one.
int from_json(const char* json, size_t bytes, tb_tokenizer& t) {
    JsonReader r{json, json + bytes};
    const Json doc = r.value();
    if (r.bad || doc.kind != Json::OBJ) return fail(tb::FORMAT, "tokenizer.json: not a JSON object");
    const Json* model = doc.get("model");
    if (!model || !model->is("type", "BPE")) return unsupported("a model other than BPE");
    bool meta = false, nfc_flag = false;
    const Json* norm = doc.get("normalizer");
    if (norm && norm->kind != Json::NUL) {
        if (norm->is("type", "Replace") && norm->is("content", "\xE2\x96\x81")) meta = true;
        else if (norm->is("type", "NFC")) nfc_flag = true;
        else return unsupported("this normalizer");
    }
    uint32_t pre = 0;
    const Json* p = doc.get("pre_tokenizer");
    if (p && p->kind != Json::NUL) {
        const Json* pattern = p->get("pattern");
        // byte_level (mod.rs:498-521): a byte-level pre-tokenizer with GPT-2's pattern, or a split by one of the three patterns
        // (its matches kept) followed by a byte-level one without
        auto level = [&](const Json& q, bool regex) -> uint32_t {
            if (!q.is("type", "ByteLevel") || !q.flag("use_regex", regex)) return 0;
            return BYTE_LEVEL | (q.flag("add_prefix_space", true) ? PREPEND : 0);
        };
        const Json* seq = p->get("pretokenizers");
        if (const uint32_t f = level(*p, true)) pre = f;
        else if (seq && seq->kind == Json::ARR && seq->arr.size() == 2) {
            const Json &split = seq->arr[0], *pat = split.get("pattern");
            const Json* regex = pat ? pat->get("Regex") : nullptr;
            const bool kept = (split.is("behavior", "Removed") && split.flag("invert", true)) || (split.is("behavior", "Isolated") && split.flag("invert", false));
            static const char* const PATTERNS[3] = {
                R"('s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+)",
                R"((?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+)",
                R"([^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+)"};
            int which = -1;
            for (int k = 0; k < 3; k++)
                if (regex && regex->kind == Json::STR && regex->s == PATTERNS[k]) which = k;
            const uint32_t f = level(seq->arr[1], false);
            // (Hugging Face gives a prefix space to every piece of such a split, not to the text: refused rather than encoded otherwise.)
            if (which < 0 || !kept || f == 0 || (f & PREPEND)) return unsupported("this pre-tokenizer");
            pre = f | (which == 1 ? CL100K : which == 2 ? O200K : 0);
        } else if (p->is("type", "ByteLevel") || seq) return unsupported("this pre-tokenizer");
        else if (p->is("type", "Split") && meta && pattern && pattern->is("String", " ")) pre = 0;
        else if (p->is("type", "Metaspace") && p->is("replacement", "\xE2\x96\x81")) {
            pre = META | (p->flag("split", false) ? 0 : SPLIT) | ((p->is("prepend_scheme", "always") || p->is("prepend_scheme", "first")) ? PREPEND : 0);
        } else return unsupported("this pre-tokenizer");
    }
    const bool fallback = model->flag("byte_fallback", true);
    std::vector<std::pair<std::string, uint32_t>> vocab;
    if (const Json* v = model->get("vocab"))
        for (const auto& kv : v->obj) vocab.emplace_back(kv.first, kv.second.kind == Json::NUM ? (uint32_t)kv.second.n : NONE);
    for (const auto& v : vocab)
        if (v.second == NONE) return fail(tb::FORMAT, "tokenizer.json: a token without an id");
    std::vector<uint32_t> special, plain;
    if (const Json* a = doc.get("added_tokens"))
        for (const Json& tok : a->arr) {
            const Json *content = tok.get("content"), *id = tok.get("id");
            if (!id || id->kind != Json::NUM) return fail(tb::FORMAT, "tokenizer.json: an added token without an id");
            vocab.emplace_back(content && content->kind == Json::STR ? content->s : std::string(), (uint32_t)id->n);
            (tok.flag("special", true) ? special : plain).push_back((uint32_t)id->n);
        }
    std::vector<std::pair<std::string, std::string>> merges;
    if (const Json* m = model->get("merges"))
        for (const Json& e : m->arr) {  // ["a", "b"], or "a b" in older files
            if (e.kind == Json::ARR && e.arr.size() >= 2 && e.arr[0].kind == Json::STR && e.arr[1].kind == Json::STR) merges.emplace_back(e.arr[0].s, e.arr[1].s);
            else if (e.kind == Json::STR && e.s.find(' ') != std::string::npos) merges.emplace_back(e.s.substr(0, e.s.find(' ')), e.s.substr(e.s.find(' ') + 1));
        }
    const Json* unk = model->get("unk_token");
    std::vector<uint32_t> skip = special;
    skip.insert(skip.end(), plain.begin(), plain.end());
    TB_TRY(build(t, vocab, merges, special, plain, unk ? unk->str() : nullptr, pre | (meta ? META : 0) | (fallback ? BYTES : 0) | (nfc_flag ? NFC : 0)));
    // frame (mod.rs:528-549): the special tokens a TemplateProcessing post-processor puts before and after a single text
    const Json* post = doc.get("post_processor");
    const Json* tpl = nullptr;
    if (post && post->is("type", "TemplateProcessing")) tpl = post;
    if (!tpl && post)
        if (const Json* all = post->get("processors"))
            for (const Json& q : all->arr)
                if (!tpl && q.is("type", "TemplateProcessing")) tpl = &q;
    if (tpl) {
        auto id = [&](const Json& item) -> uint32_t {
            const Json* st = item.get("SpecialToken");
            const Json* name = st ? st->get("id") : nullptr;
            const Json* table = tpl->get("special_tokens");
            const Json* entry = (name && name->kind == Json::STR && table) ? table->get(name->s.c_str()) : nullptr;
            const Json* ids = entry ? entry->get("ids") : nullptr;
            if (!ids || ids->kind != Json::ARR || ids->arr.size() != 1 || ids->arr[0].kind != Json::NUM) return NONE;
            return (uint32_t)ids->arr[0].n;
        };
        const Json* single = tpl->get("single");
        const std::vector<Json> none;
        const std::vector<Json>& items = single && single->kind == Json::ARR ? single->arr : none;
        size_t at = items.size();
        for (size_t i = 0; i < items.size(); i++)
            if (items[i].get("Sequence")) {
                at = i;
                break;
            }
        if (at == 1) t.frame[0] = id(items[0]);
        if (at < items.size() && items.size() - at - 1 == 1) t.frame[1] = id(items[at + 1]);
    }
    if (model->flag("ignore_merges", true)) {  // index_words (mod.rs:206-218): every token but the added ones, by its text
        t.words.assign(std::max<size_t>(pow2_at_least(2 * t.len()), 2), NONE);
        const size_t mask = t.words.size() - 1;
        for (uint32_t id = 0; id < t.len(); id++) {
            if (std::find(skip.begin(), skip.end(), id) != skip.end()) continue;
            size_t n;
            const uint8_t* s = t.token(id, n);
            size_t i = slot_of(fnv(s, n), mask);
            while (t.words[i] != NONE) i = (i + 1) & mask;
            t.words[i] = id;
        }
    }
    return tb::OK;
}

// ---- encoding -------------------------------------------------------------------------------------------------------------------
struct Work {
    std::vector<uint32_t> ids, next, prev, rank, merged;  // rank, merged: of the symbol's merge with the one after it, NONE if none
    std::vector<uint64_t> heap;  // (rank << 32 | position) of merges that were possible when pushed; checked again when taken
};

// The tokens before merging (mod.rs:393-413): one per character, or per byte of a character the vocabulary lacks.
void symbols(const tb_tokenizer& t, const uint8_t* p, const uint8_t* end, std::vector<uint32_t>& ids) {
    ids.clear();
    for (size_t n; p < end; p += n) {
        uint32_t c = next_char(p, end, n);
        if (c == ' ' && (t.flags & META)) c = BAR;
        const uint32_t id = t.char_id(c);
        if (id != NONE) {
            ids.push_back(id);
            continue;
        }
        uint8_t utf8[4];  // the character's own bytes (a byte that started no character came out as U+FFFD and is spelled so)
        size_t len = 0;
        if (c < 0x80) utf8[len++] = (uint8_t)c;
        else if (c < 0x800) utf8[len++] = (uint8_t)(0xC0 | c >> 6), utf8[len++] = (uint8_t)(0x80 | (c & 63));
        else if (c < 0x10000) utf8[len++] = (uint8_t)(0xE0 | c >> 12), utf8[len++] = (uint8_t)(0x80 | (c >> 6 & 63)), utf8[len++] = (uint8_t)(0x80 | (c & 63));
        else utf8[len++] = (uint8_t)(0xF0 | c >> 18), utf8[len++] = (uint8_t)(0x80 | (c >> 12 & 63)), utf8[len++] = (uint8_t)(0x80 | (c >> 6 & 63)), utf8[len++] = (uint8_t)(0x80 | (c & 63));
        bool all = (t.flags & BYTES) != 0;
        for (size_t k = 0; k < len; k++) all = all && t.bytes[utf8[k]] != NONE;
        if (all)
            for (size_t k = 0; k < len; k++) ids.push_back(t.bytes[utf8[k]]);
        else if (t.unk != NONE && (ids.empty() || ids.back() != t.unk)) ids.push_back(t.unk);
    }
}

// Merges the piece's symbols, lowest-ranked pair first and the leftmost among equals (mod.rs:345-383), and appends what is left.
void merge_all(const tb_tokenizer& t, const uint8_t* p, const uint8_t* end, Work& w, uint32_t* out, size_t cap, size_t& count) {
    if (t.flags & BYTE_LEVEL) {
        w.ids.clear();
        for (; p < end; p++) w.ids.push_back(t.bytes[*p]);
    } else {
        symbols(t, p, end, w.ids);
    }
    const uint32_t n = (uint32_t)w.ids.size();
    if (n == 1) {  // most pieces of a text with many spaces
        if (w.ids[0] != NONE) {
            if (count < cap) out[count] = w.ids[0];
            count++;
        }
        return;
    }
    w.next.resize(n), w.prev.resize(n), w.rank.assign(n, NONE), w.merged.resize(n), w.heap.clear();
    // offer(i): what symbol i and the one after it merge into, kept beside the symbol and put on the heap; an entry taken from
    // the heap counts only while it is still what is kept (a symbol whose pair changed was offered again since)
    auto offer = [&](uint32_t i) {
        if (i >= n) return;
        w.rank[i] = NONE;
        const uint32_t j = w.next[i];
        if (j >= n || w.ids[i] == NONE || w.ids[j] == NONE) return;
        const size_t at = find_merge(t.merges, w.ids[i], w.ids[j]);
        if (t.merges[at] == NONE) return;
        w.rank[i] = t.merges[at + 2], w.merged[i] = t.merges[at + 3];
        w.heap.push_back((uint64_t)w.rank[i] << 32 | i), std::push_heap(w.heap.begin(), w.heap.end(), std::greater<uint64_t>());
    };
    for (uint32_t i = 0; i < n; i++) w.next[i] = i + 1, w.prev[i] = i - 1;  // prev of the first wraps to NONE
    for (uint32_t i = 0; i + 1 < n; i++) offer(i);
    while (!w.heap.empty()) {
        std::pop_heap(w.heap.begin(), w.heap.end(), std::greater<uint64_t>());
        const uint64_t top = w.heap.back();
        w.heap.pop_back();
        const uint32_t i = (uint32_t)top;
        if (w.rank[i] != (uint32_t)(top >> 32)) continue;  // what stood here then is gone
        const uint32_t j = w.next[i];
        w.ids[i] = w.merged[i], w.ids[j] = NONE, w.rank[j] = NONE, w.next[i] = w.next[j];
        if (w.next[i] < n) w.prev[w.next[i]] = i;
        offer(w.prev[i]), offer(i);
    }
    for (uint32_t id : w.ids)
        if (id != NONE) {
            if (count < cap) out[count] = id;
            count++;
        }
}

bool is_join(const tb_tokenizer& t, uint32_t c) { return std::binary_search(t.joins.begin(), t.joins.end(), c); }

// A stretch of text that holds no added token (mod.rs:303-326): U+2581 first if the pre-tokenizer prepends one, then cut before
// each space that follows a character no token joins to a following U+2581 (before every space when the pre-tokenizer splits),
// each piece merged on its own.
void segment(const tb_tokenizer& t, const uint8_t* p, const uint8_t* end, Work& w, uint32_t* out, size_t cap, size_t& count) {
    std::string prefixed;
    // (A byte-level pre-tokenizer prepends its space unless the text starts with one, as Hugging Face does; U+2581 is no space to it.)
    if ((t.flags & PREPEND) && p < end && p[0] != ' ' && ((t.flags & BYTE_LEVEL) || !(end - p >= 3 && p[0] == 0xE2 && p[1] == 0x96 && p[2] == 0x81))) {
        prefixed = ((t.flags & BYTE_LEVEL) ? std::string(" ") : std::string("\xE2\x96\x81")) + std::string(reinterpret_cast<const char*>(p), (size_t)(end - p));
        p = reinterpret_cast<const uint8_t*>(prefixed.data()), end = p + prefixed.size();
    }
    if (t.flags & BYTE_LEVEL) {
        // byte_segment (mod.rs:328-336): each piece its pattern cuts is a token of its own if the model ignores merges for pieces
        // that are tokens, else merged on its own
        Chars cs;
        std::vector<size_t> at;  // where each character starts, and the end
        for (const uint8_t* q = p; q < end;) {
            size_t n;
            cs.c.push_back(next_char(q, end, n));
            at.push_back((size_t)(q - p));
            q += n;
        }
        at.push_back((size_t)(end - p));
        for (size_t i = 0; i < cs.n();) {
            size_t k = (t.flags & O200K) ? cs.o200k(i) : (t.flags & CL100K) ? cs.cl100k(i) : cs.gpt2(i);
            if (k == 0 || i + k > cs.n()) k = 1;
            const uint8_t *from = p + at[i], *to = p + at[i + k];
            uint32_t whole = NONE;
            if (!t.words.empty()) {
                const size_t mask = t.words.size() - 1;
                for (size_t j = slot_of(fnv(from, (size_t)(to - from)), mask); t.words[j] != NONE; j = (j + 1) & mask) {
                    size_t n;
                    const uint8_t* text = t.token(t.words[j], n);
                    if (n == (size_t)(to - from) && !memcmp(text, from, n)) {
                        whole = t.words[j];
                        break;
                    }
                }
            }
            if (whole != NONE) {
                if (count < cap) out[count] = whole;
                count++;
            } else {
                merge_all(t, from, to, w, out, cap, count);
            }
            i += k;
        }
        return;
    }
    const uint8_t *start = p, *at = p;
    uint32_t last = BAR;
    for (size_t n; at < end; at += n) {
        const uint32_t c = next_char(at, end, n);
        const bool space = c == ' ' || c == BAR, joined = last == ' ' || last == BAR || is_join(t, last);
        if (at > start && space && (t.flags & META) && ((t.flags & SPLIT) || !joined)) {
            merge_all(t, start, at, w, out, cap, count);
            start = at;
        }
        last = c;
    }
    if (start < end) merge_all(t, start, end, w, out, cap, count);
}

// Tokenizer::encode (mod.rs:272-301): non-special added tokens are found first, the longest at each place; the text between
// them goes through `segment`.
void encode(const tb_tokenizer& t, const uint8_t* text, size_t bytes, uint32_t* out, size_t cap, size_t& count) {
    Work w;
    std::string normal;
    if ((t.flags & NFC) && nfc(text, text + bytes, normal)) text = reinterpret_cast<const uint8_t*>(normal.data()), bytes = normal.size();
    const uint8_t *end = text + bytes, *from = text, *at = text;
    while (at < end) {
        uint32_t found = NONE;
        size_t len = 0, n;
        // the added tokens that start with this byte, longest first
        auto k = std::partition_point(t.added.begin(), t.added.end(), [&](uint32_t id) { return t.token(id, n)[0] < at[0]; });
        for (; k != t.added.end() && found == NONE; ++k) {
            const uint8_t* s = t.token(*k, n);
            if (s[0] != at[0]) break;
            if (n <= (size_t)(end - at) && !memcmp(s, at, n)) found = *k, len = n;
        }
        if (found != NONE) {
            segment(t, from, at, w, out, cap, count);
            if (count < cap) out[count] = found;
            count++;
            at += len, from = at;
        } else {
            next_char(at, end, n);
            at += n;
        }
    }
    segment(t, from, end, w, out, cap, count);
}

}  // namespace

namespace {

// ---- the stored form (mod.rs:422-455): `TACHYTOK`, then length-prefixed runs of little-endian words -----------------------------
const char TOK_MAGIC[8] = {'T', 'A', 'C', 'H', 'Y', 'T', 'O', 'K'};

std::vector<uint8_t> to_bytes(const tb_tokenizer& t) {
    std::vector<uint8_t> out(TOK_MAGIC, TOK_MAGIC + 8);
    auto word = [&](uint32_t v) {
        for (int k = 0; k < 4; k++) out.push_back((uint8_t)(v >> (8 * k)));
    };
    auto section = [&](const std::vector<uint32_t>& s) {
        word((uint32_t)s.size());
        for (uint32_t v : s) word(v);
    };
    std::vector<uint32_t> text((t.text.size() + 3) / 4, 0);
    for (size_t i = 0; i < t.text.size(); i++) text[i / 4] |= (uint32_t)t.text[i] << (8 * (i % 4));
    section({t.flags, t.unk, (uint32_t)t.text.size(), t.frame[0], t.frame[1]});
    section(t.offsets), section(text), section(t.special), section(t.bytes), section(t.chars), section(t.rare), section(t.joins), section(t.added), section(t.merges);
    if (!t.words.empty()) section(t.words);
    return out;
}

int damaged() { return fail(tb::FORMAT, "tokenizer.tok: damaged, or written by an older Tachyon; convert the model again"); }

int from_bytes(const uint8_t* data, size_t bytes, tb_tokenizer& t) {
    if (bytes < 8 || memcmp(data, TOK_MAGIC, 8) != 0) return damaged();
    size_t at = 8;
    const size_t words = (bytes - 8) / 4;  // a trailing part of a word is ignored, as chunks_exact does
    const size_t end = 8 + 4 * words;
    auto word = [&](uint32_t& v) {
        if (at + 4 > end) return false;
        v = (uint32_t)data[at] | (uint32_t)data[at + 1] << 8 | (uint32_t)data[at + 2] << 16 | (uint32_t)data[at + 3] << 24;
        at += 4;
        return true;
    };
    auto section = [&](std::vector<uint32_t>& s) {
        uint32_t n;
        if (!word(n) || (size_t)n > (end - at) / 4) return false;
        s.resize(n);
        for (uint32_t& v : s) word(v);
        return true;
    };
    std::vector<uint32_t> head, text;
    std::vector<uint32_t>* all[10] = {&head, &t.offsets, &text, &t.special, &t.bytes, &t.chars, &t.rare, &t.joins, &t.added, &t.merges};
    for (std::vector<uint32_t>* s : all)
        if (!section(*s)) return damaged();
    if (head.size() < 3 || (size_t)head[2] > 4 * text.size()) return damaged();
    t.text.resize(head[2]);
    for (size_t i = 0; i < t.text.size(); i++) t.text[i] = (uint8_t)(text[i / 4] >> (8 * (i % 4)));
    if (at < end && !section(t.words)) return damaged();  // older files end after the merges, and their head holds no frame
    t.flags = head[0], t.unk = head[1];
    t.frame[0] = head.size() > 3 ? head[3] : NONE, t.frame[1] = head.size() > 4 ? head[4] : NONE;
    const bool sound = !t.offsets.empty() && t.offsets.back() == t.text.size() && t.bytes.size() == 256 && t.chars.size() == DIRECT && t.merges.size() >= 8 &&
                       (t.merges.size() & (t.merges.size() - 1)) == 0 && std::is_sorted(t.offsets.begin(), t.offsets.end()) && t.rare.size() % 2 == 0;
    if (!sound) return damaged();
    // ids the tables name must be tokens, or none: a damaged file must not index outside the text
    const uint32_t n = (uint32_t)t.len();
    auto ok = [&](uint32_t id) { return id == NONE || id < n; };
    bool ids = ok(t.unk) && std::all_of(t.bytes.begin(), t.bytes.end(), ok) && std::all_of(t.chars.begin(), t.chars.end(), ok) && std::all_of(t.added.begin(), t.added.end(), [&](uint32_t id) { return id < n; });
    for (size_t k = 0; k < t.merges.size() && ids; k += 4) ids = t.merges[k] == NONE || (t.merges[k] < n && t.merges[k + 1] < n && t.merges[k + 3] < n);
    for (size_t k = 1; k < t.rare.size() && ids; k += 2) ids = t.rare[k] < n;
    for (uint32_t id : t.added) {
        size_t len;
        t.token(id, len);
        ids = ids && len > 0;
    }
    bool room = false;  // the merge table must have a free entry, or a lookup would never end
    for (size_t k = 0; k < t.merges.size(); k += 4) room = room || t.merges[k] == NONE;
    if (!ids || !room) return damaged();
    if (!t.words.empty()) {
        bool free_entry = false, tokens = true;
        for (uint32_t id : t.words) free_entry = free_entry || id == NONE, tokens = tokens && ok(id);
        if ((t.words.size() & (t.words.size() - 1)) != 0 || !free_entry || !tokens) return damaged();
    }
    return tb::OK;
}

// ---- Detokenizer (mod.rs:603-648): whole characters only; an unfinished character ends as U+FFFD ------------------------------
// The length of the invalid sequence at p (1 to 3 bytes), 0 if the bytes are the start of a character that the input ends
// inside, or the character's length with `good` set: the rule of Rust's str::from_utf8 (Utf8Error::error_len), which the
// reference's text follows.
size_t utf8_step(const uint8_t* p, size_t left, bool& good) {
    good = false;
    const uint8_t b = p[0];
    if (b < 0x80) return good = true, 1;
    size_t want;
    uint8_t lo = 0x80, hi = 0xBF;
    if (b >= 0xC2 && b <= 0xDF) want = 2;
    else if (b >= 0xE0 && b <= 0xEF) want = 3, lo = b == 0xE0 ? 0xA0 : 0x80, hi = b == 0xED ? 0x9F : 0xBF;
    else if (b >= 0xF0 && b <= 0xF4) want = 4, lo = b == 0xF0 ? 0x90 : 0x80, hi = b == 0xF4 ? 0x8F : 0xBF;
    else return 1;
    for (size_t k = 1; k < want; k++) {
        if (k >= left) return 0;
        const uint8_t c = p[k];
        if (k == 1 ? (c < lo || c > hi) : (c < 0x80 || c > 0xBF)) return k;
    }
    return good = true, want;
}

void flush(tb_detokenizer& d, bool end, std::string& out) {
    size_t at = 0;
    const size_t n = d.pending.size();
    while (at < n) {
        bool good;
        size_t step = utf8_step(d.pending.data() + at, n - at, good);
        if (good) {
            out.append(reinterpret_cast<const char*>(d.pending.data() + at), step);
        } else {
            if (step == 0) {
                if (!end) break;
                step = n - at;
            }
            for (size_t k = 0; k < step; k++) out += "\xEF\xBF\xBD";
        }
        at += step;
    }
    d.pending.erase(d.pending.begin(), d.pending.begin() + (long)at);
}

int give(const std::string& text, char* out, size_t capacity, size_t* bytes) {
    if (bytes) *bytes = text.size();
    if (text.size() > capacity) return fail(tb::OUT_OF_RANGE, "the text needs " + std::to_string(text.size()) + " bytes");
    if (!text.empty()) memcpy(out, text.data(), text.size());
    return tb::OK;
}

}  // namespace

namespace {

// ---- Gemma 4's chat template (token/chat.rs:1-16, 124-199), text only: turn markers by id, the messages as text ------------------
bool is_space(uint32_t c) {  // Unicode White_Space, what Rust's str::trim takes off
    return (c >= 9 && c <= 13) || c == 32 || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 || c == 0x2029 || c == 0x202F ||
           c == 0x205F || c == 0x3000;
}

std::string trimmed(const char* text, size_t bytes) {
    const uint8_t *p = reinterpret_cast<const uint8_t*>(text), *end = p + bytes;
    size_t n;
    while (p < end && is_space(next_char(p, end, n))) p += n;
    const uint8_t* last = p;  // one past the last character that is not a space
    for (const uint8_t* q = p; q < end; q += n)
        if (!is_space(next_char(q, end, n))) last = q + n;
    return std::string(reinterpret_cast<const char*>(p), (size_t)(last - p));
}

struct Sink {
    const tb_tokenizer& tok;
    uint32_t* out;
    size_t cap, count = 0;
    void id(uint32_t v) {
        if (count < cap) out[count] = v;
        count++;
    }
    void text(const std::string& s) { encode(tok, reinterpret_cast<const uint8_t*>(s.data()), s.size(), out, cap, count); }
};

uint32_t special_named(const tb_tokenizer& t, const char* text) {
    const size_t want = strlen(text);
    for (uint32_t id : t.special) {
        size_t n;
        const uint8_t* s = t.token(id, n);
        if (n == want && !memcmp(s, text, n)) return id;
    }
    return NONE;
}

}  // namespace

extern "C" {

int tb_tokenizer_from_json(const void* json, size_t bytes, tb_tokenizer** out) {
    if (!json || !out) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_from_json: null argument");
    *out = nullptr;
    tb_tokenizer* t = new tb_tokenizer();
    const int st = from_json(static_cast<const char*>(json), bytes, *t);
    if (st != tb::OK) return delete t, st;
    *out = t;
    return tb::OK;
}

int tb_tokenizer_from_bytes(const void* data, size_t bytes, tb_tokenizer** out) {
    if (!data || !out) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_from_bytes: null argument");
    *out = nullptr;
    tb_tokenizer* t = new tb_tokenizer();
    const int st = from_bytes(static_cast<const uint8_t*>(data), bytes, *t);
    if (st != tb::OK) return delete t, st;
    *out = t;
    return tb::OK;
}

int tb_tokenizer_to_bytes(const tb_tokenizer* tok, void* out, size_t capacity, size_t* bytes) {
    if (!tok || !bytes) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_to_bytes: null argument");
    const std::vector<uint8_t> b = to_bytes(*tok);
    *bytes = b.size();
    if (!out || capacity < b.size()) return capacity == 0 ? tb::OK : fail(tb::OUT_OF_RANGE, "tb_tokenizer_to_bytes: " + std::to_string(b.size()) + " bytes needed");
    memcpy(out, b.data(), b.size());
    return tb::OK;
}

void tb_tokenizer_close(tb_tokenizer* tok) { delete tok; }

size_t tb_tokenizer_len(const tb_tokenizer* tok) { return tok ? tok->len() : 0; }

int tb_tokenizer_encode(const tb_tokenizer* tok, const char* text, size_t bytes, uint32_t* ids, size_t capacity, size_t* count) {
    if (!tok || (!text && bytes) || !count || (!ids && capacity)) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_encode: null argument");
    *count = 0;
    encode(*tok, reinterpret_cast<const uint8_t*>(text), bytes, ids, capacity, *count);
    return *count > capacity && capacity > 0 ? fail(tb::OUT_OF_RANGE, "tb_tokenizer_encode: " + std::to_string(*count) + " tokens, room for " + std::to_string(capacity)) : tb::OK;
}

int tb_tokenizer_token(const tb_tokenizer* tok, uint32_t id, const uint8_t** text, size_t* bytes) {
    if (!tok || !text || !bytes) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_token: null argument");
    if (id >= tok->len()) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_token: no such token");
    *text = tok->token(id, *bytes);
    return tb::OK;
}

int tb_tokenizer_is_special(const tb_tokenizer* tok, uint32_t id) { return tok && tok->is_special(id); }

int tb_tokenizer_special(const tb_tokenizer* tok, const char* text, uint32_t* id) {
    if (!tok || !text || !id) return fail(tb::OUT_OF_RANGE, "tb_tokenizer_special: null argument");
    *id = special_named(*tok, text);
    return *id == NONE ? fail(tb::NO_MODEL, std::string("tokenizer: no special token ") + text) : tb::OK;
}

void tb_tokenizer_frame(const tb_tokenizer* tok, uint32_t* before, uint32_t* after) {
    if (before) *before = tok ? tok->frame[0] : NONE;
    if (after) *after = tok ? tok->frame[1] : NONE;
}

int tb_detokenizer_new(tb_detokenizer** out) {
    if (!out) return fail(tb::OUT_OF_RANGE, "tb_detokenizer_new: null argument");
    *out = new tb_detokenizer();
    return tb::OK;
}

void tb_detokenizer_close(tb_detokenizer* d) { delete d; }

// The text token `id` completes, into out[capacity]; *bytes is its length.  When it does not fit nothing is consumed: the
// token stays pending and the same call with more room gives the text.
int tb_detokenizer_push(tb_detokenizer* d, const tb_tokenizer* tok, uint32_t id, char* out, size_t capacity, size_t* bytes) {
    if (!d || !tok || !bytes || (!out && capacity)) return fail(tb::OUT_OF_RANGE, "tb_detokenizer_push: null argument");
    *bytes = 0;
    if (tok->is_special(id)) return tb::OK;
    const std::vector<uint8_t> before = d->pending;
    size_t n;
    const uint8_t* s = tok->token(id, n);
    d->pending.insert(d->pending.end(), s, s + n);
    std::string text;
    flush(*d, false, text);
    const int st = give(text, out, capacity, bytes);
    if (st != tb::OK) d->pending = before;
    return st;
}

int tb_detokenizer_finish(tb_detokenizer* d, char* out, size_t capacity, size_t* bytes) {
    if (!d || !bytes || (!out && capacity)) return fail(tb::OUT_OF_RANGE, "tb_detokenizer_finish: null argument");
    const std::vector<uint8_t> before = d->pending;
    std::string text;
    flush(*d, true, text);
    const int st = give(text, out, capacity, bytes);
    if (st != tb::OK) d->pending = before;
    return st;
}

int tb_chat_gemma4(const tb_tokenizer* tok, tb_chat* out) {
    if (!tok || !out) return fail(tb::OUT_OF_RANGE, "tb_chat_gemma4: null argument");
    const char* names[4] = {"<bos>", "<|turn>", "<turn|>", "<|think|>"};
    uint32_t ids[4];
    for (int k = 0; k < 4; k++)
        if ((ids[k] = special_named(*tok, names[k])) == NONE) return fail(tb::FORMAT, std::string("tokenizer: no ") + names[k] + " token, not Gemma 4's");
    out->bos = ids[0], out->turn = ids[1], out->end = ids[2], out->think = ids[3];
    out->closed[0] = out->closed[1] = NONE;
    return tb::OK;
}

// Chat::with_template (chat.rs:97-107): some models' templates open the model's turn with an empty thinking block when
// thinking is off; told from the generation prompt of the model's chat_template.jinja.
int tb_chat_with_template(const tb_tokenizer* tok, tb_chat* chat, const char* text, size_t bytes) {
    if (!tok || !chat || (!text && bytes)) return fail(tb::OUT_OF_RANGE, "tb_chat_with_template: null argument");
    const std::string tpl(text ? text : "", bytes);
    const size_t at = tpl.rfind("add_generation_prompt");
    const uint32_t open = special_named(*tok, "<|channel>"), close = special_named(*tok, "<channel|>");
    const bool writes = at != std::string::npos && tpl.find("'<|channel>thought\\n<channel|>'", at) != std::string::npos;
    chat->closed[0] = chat->closed[1] = NONE;
    if (writes && open != NONE && close != NONE) chat->closed[0] = open, chat->closed[1] = close;
    return tb::OK;
}

// Chat::encode (chat.rs:124-163): <bos>, the system turn when there is a system message first or thinking is on, the turns
// (messages trimmed, consecutive model messages sharing one), then the opening of the model's turn.
int tb_chat_encode(const tb_tokenizer* tok, const tb_chat* chat, const tb_message* messages, size_t n, int think, uint32_t* ids, size_t capacity, size_t* count) {
    if (!tok || !chat || (!messages && n) || !count || (!ids && capacity)) return fail(tb::OUT_OF_RANGE, "tb_chat_encode: null argument");
    for (size_t i = 0; i < n; i++)
        if (messages[i].role < TB_ROLE_SYSTEM || messages[i].role > TB_ROLE_MODEL || (!messages[i].text && messages[i].bytes)) return fail(tb::OUT_OF_RANGE, "tb_chat_encode: a message without a role or a text");
    Sink s{*tok, ids, capacity};
    auto close = [&](const std::string& text) { s.text(text), s.id(chat->end), s.text("\n"); };
    s.id(chat->bos);
    size_t first = 0;
    const bool system = n > 0 && messages[0].role == TB_ROLE_SYSTEM;
    if (system || think) {
        s.id(chat->turn);
        std::string text = "system\n";
        if (think) s.text(text), s.id(chat->think), text = "\n";
        if (system) text += trimmed(messages[0].text, messages[0].bytes), first = 1;
        close(text);
    }
    std::string model;
    bool has_model = false;
    auto model_turn = [&] {
        if (has_model) s.id(chat->turn), close("model\n" + model);
        model.clear(), has_model = false;
    };
    for (size_t i = first; i < n; i++) {
        const tb_message& m = messages[i];
        if (m.role == TB_ROLE_MODEL) {
            model += trimmed(m.text, m.bytes), has_model = true;
            continue;
        }
        model_turn();
        s.id(chat->turn);
        close(std::string(m.role == TB_ROLE_SYSTEM ? "system\n" : "user\n") + trimmed(m.text, m.bytes));
    }
    model_turn();
    s.id(chat->turn);
    s.text("model\n");
    if (chat->closed[0] != NONE && !think) s.id(chat->closed[0]), s.text("thought\n"), s.id(chat->closed[1]);
    *count = s.count;
    return s.count > capacity && capacity > 0 ? fail(tb::OUT_OF_RANGE, "tb_chat_encode: " + std::to_string(s.count) + " tokens, room for " + std::to_string(capacity)) : tb::OK;
}

}  // extern "C"
