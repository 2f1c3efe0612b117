// Reader of `.wpk`, the reference's packed weight file (crates/tachyon/src/wpk/mod.rs:6-10, 37-40, 146-213): a 4 KiB
// header (magic, version and tensor count, sizes, CRC32C of the table and of itself), the tensors' bytes each on a
// 4 KiB boundary, and a table with every tensor's name, element type, shape, offset, length and CRC32C.  Host code only:
// a converted model's weights.wpk is opened, checked as Wpk::open checks it, and its tensors handed to the decoder by
// their converted-model names (model/mod.rs:178-286).  Loading streams the file as the reference's loader does
// (wpk/load.rs: reads in flight into pinned staging slots, each uploaded while the other reads proceed): reader threads
// fill a ring of pinned slots with pread, the calling thread uploads them in the file's order.
#include "../../include/tachyon_b200.h"
#include "internal.h"

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

struct tb_wpk {
    int fd = -1;
    uint64_t data_len = 0;
    struct Entry {
        std::string name;
        uint32_t dtype = 0, rank = 0, crc = 0;
        uint64_t shape[8] = {}, offset = 0, len = 0;
    };
    std::vector<Entry> tensors;
};

namespace tb {
namespace {

constexpr uint64_t ALIGN = 4096;   // wpk/mod.rs:37
constexpr size_t HEADER = 48;      // wpk/mod.rs:40
const uint64_t DTYPE_SIZE[6] = {4, 2, 2, 1, 1, 1};  // F32, F16, BF16, F8E4M3, I8, U8 (wpk/mod.rs:62-72)

// CRC32C (Castagnoli, reflected 0x82F63B78), continuing from `crc`: wpk/mod.rs:105-123.
struct CrcTable {
    uint32_t t[8][256];
    CrcTable() {
        for (uint32_t i = 0; i < 256; i++) {
            uint32_t c = i;
            for (int k = 0; k < 8; k++) c = (c >> 1) ^ (0x82F63B78u & (0u - (c & 1u)));
            t[0][i] = c;
        }
        for (uint32_t i = 0; i < 256; i++)
            for (int k = 1; k < 8; k++) t[k][i] = (t[k - 1][i] >> 8) ^ t[0][t[k - 1][i] & 255u];
    }
};

// The processor's own CRC32C instruction where it has one (SSE4.2: CPUID leaf 1, ECX bit 20), as the reference's crc32c
// prefers it over crc32c_soft (wpk/mod.rs:105-123).
bool has_crc_instruction() {
#if defined(__x86_64__)
    static const bool has = [] {
        uint32_t a = 1, b = 0, c = 0, d = 0;
        asm volatile("cpuid" : "+a"(a), "=b"(b), "+c"(c), "=d"(d));
        (void)b, (void)d;
        return (c >> 20 & 1u) != 0;
    }();
    return has;
#else
    return false;
#endif
}

uint32_t crc32c(uint32_t crc, const uint8_t* p, size_t n) {
#if defined(__x86_64__)
    if (has_crc_instruction()) {
        uint64_t c = (uint32_t)~crc;
        for (; n >= 8; p += 8, n -= 8) {
            uint64_t v;
            memcpy(&v, p, 8);
            asm("crc32q %1, %0" : "+r"(c) : "r"(v));
        }
        for (; n > 0; p++, n--) asm("crc32b %1, %0" : "+r"(c) : "r"(*p));
        return ~(uint32_t)c;
    }
#endif
    static const CrcTable tables;  // built once, by whichever thread comes first
    const uint32_t (*table)[256] = tables.t;
    uint32_t c = ~crc;
    while (n >= 8) {  // eight bytes a turn
        uint32_t lo, hi;
        memcpy(&lo, p, 4), memcpy(&hi, p + 4, 4);
        lo ^= c;
        c = table[7][lo & 255u] ^ table[6][(lo >> 8) & 255u] ^ table[5][(lo >> 16) & 255u] ^ table[4][lo >> 24] ^ table[3][hi & 255u] ^
            table[2][(hi >> 8) & 255u] ^ table[1][(hi >> 16) & 255u] ^ table[0][hi >> 24];
        p += 8, n -= 8;
    }
    while (n--) c = (c >> 8) ^ table[0][(c ^ *p++) & 255u];
    return ~c;
}

// CRC32C of a string A B from crc(A), crc(B) and B's length: crc(A) advanced through len(B) zero bytes (the register times
// x^(8 len) modulo the polynomial, by squaring a 32 x 32 matrix over GF(2)), then xor crc(B).  It lets the loader's reader
// threads each check their own piece of a tensor.
uint32_t gf2_times(const uint32_t* mat, uint32_t vec) {
    uint32_t sum = 0;
    for (; vec; vec >>= 1, mat++)
        if (vec & 1u) sum ^= *mat;
    return sum;
}

uint32_t crc32c_combine(uint32_t crc_a, uint32_t crc_b, uint64_t len_b) {
    if (len_b == 0) return crc_a;
    uint32_t even[32], odd[32];
    odd[0] = 0x82F63B78u;  // one zero bit: shift right, the polynomial where a bit falls out
    for (int n = 1; n < 32; n++) odd[n] = 1u << (n - 1);
    auto square = [](uint32_t* to, const uint32_t* from) {
        for (int n = 0; n < 32; n++) to[n] = gf2_times(from, from[n]);
    };
    square(even, odd);  // two zero bits
    square(odd, even);  // four
    do {                // from here each squaring doubles the zero bytes: one, two, four ...
        square(even, odd);
        if (len_b & 1u) crc_a = gf2_times(even, crc_a);
        len_b >>= 1;
        if (len_b == 0) break;
        square(odd, even);
        if (len_b & 1u) crc_a = gf2_times(odd, crc_a);
        len_b >>= 1;
    } while (len_b != 0);
    return crc_a ^ crc_b;
}

// Little-endian fields; past the end it yields zeros and remembers it (the reference's Cursor, wpk/mod.rs:125-144).
struct Cursor {
    const uint8_t* p;
    size_t left;
    bool is_short = false;
    const uint8_t* take(size_t n) {
        if (n > left) {
            is_short = true;
            return nullptr;
        }
        const uint8_t* at = p;
        p += n, left -= n;
        return at;
    }
    uint64_t num(size_t n) {
        const uint8_t* b = take(n);
        uint64_t v = 0;
        if (b)
            for (size_t i = n; i-- > 0;) v = v << 8 | b[i];
        return v;
    }
};

int io_fail(const char* what, const char* path) { return fail(IO, std::string(what) + " " + path + ": " + strerror(errno)); }

bool read_at(int fd, void* dst, size_t n, uint64_t at) {
    uint8_t* out = static_cast<uint8_t*>(dst);
    while (n > 0) {
        const ssize_t got = pread(fd, out, n, (off_t)at);
        if (got <= 0) return false;
        out += got, at += (uint64_t)got, n -= (size_t)got;
    }
    return true;
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" {

uint32_t tb_crc32c(uint32_t crc, const void* data, size_t bytes) { return crc32c(crc, static_cast<const uint8_t*>(data), bytes); }

uint32_t tb_crc32c_combine(uint32_t crc_a, uint32_t crc_b, uint64_t len_b) { return crc32c_combine(crc_a, crc_b, len_b); }

int tb_wpk_open(const char* path, tb_wpk** out) {
    if (!path || !out) return fail(OUT_OF_RANGE, "tb_wpk_open: null argument");
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return io_fail("tb_wpk_open:", path);
    struct stat st = {};
    uint8_t head[HEADER];
    if (fstat(fd, &st) != 0) {
        const int rc = io_fail("tb_wpk_open:", path);
        close(fd);
        return rc;
    }
    if (!read_at(fd, head, HEADER, 0)) {
        const int rc = st.st_size < (off_t)HEADER ? fail(FORMAT, std::string(path) + ": the file ends early") : io_fail("tb_wpk_open:", path);
        close(fd);
        return rc;
    }
    Cursor c{head, HEADER};
    const uint8_t* magic = c.take(8);
    const uint64_t version = c.num(8), data_len = c.num(8), table_at = c.num(8), table_len = c.num(8);
    const uint32_t table_crc = (uint32_t)c.num(4), head_crc = (uint32_t)c.num(4);
    const uint64_t size = (uint64_t)st.st_size;
    // The checks of wpk/mod.rs:196-203, in their order.
    const char* why = nullptr;
    if (memcmp(magic, "TACHYWPK", 8) != 0) why = "not a .wpk file";
    else if (crc32c(0, head, HEADER - 4) != head_crc) why = "the header is corrupt";
    else if ((uint32_t)version != 1u) why = "unsupported version";
    else if (data_len % ALIGN != 0 || table_at != ALIGN + data_len) why = "the data region is malformed";
    else if (table_at + table_len < table_at || table_at + table_len > size) why = "the file is truncated";
    if (why) {
        close(fd);
        return fail(FORMAT, std::string(path) + ": " + why);
    }
    std::vector<uint8_t> table(table_len);
    if (table_len && !read_at(fd, table.data(), table_len, table_at)) {
        close(fd);
        return io_fail("tb_wpk_open: reading the table of", path);
    }
    if (crc32c(0, table.data(), table.size()) != table_crc) {
        close(fd);
        return fail(FORMAT, std::string(path) + ": the tensor table is corrupt");
    }
    tb_wpk* w = new tb_wpk();
    w->fd = fd, w->data_len = data_len;
    Cursor t{table.data(), table.size()};
    const uint64_t count = version >> 32;
    for (uint64_t i = 0; i < count && !why; i++) {
        tb_wpk::Entry e;
        const size_t name_len = (size_t)t.num(2);
        const uint8_t* name = t.take(name_len);
        if (name) e.name.assign(reinterpret_cast<const char*>(name), name_len);
        e.dtype = (uint32_t)t.num(1), e.rank = (uint32_t)t.num(1);
        for (uint32_t k = 0; k < e.rank && k < 8; k++) e.shape[k] = t.num(8);
        e.offset = t.num(8), e.len = t.num(8), e.crc = (uint32_t)t.num(4);
        // wpk/mod.rs:160-167
        uint64_t want = e.dtype < 6 ? DTYPE_SIZE[e.dtype] : 0;
        bool overflow = false;
        for (uint32_t k = 0; k < e.rank && k < 8; k++) {
            if (e.shape[k] != 0 && want > UINT64_MAX / e.shape[k]) overflow = true;
            want *= e.shape[k];
        }
        if (t.is_short) why = "the tensor table is truncated";
        else if (e.dtype >= 6) why = "unknown element type";
        else if (e.rank > 8) why = "more than 8 dimensions";
        else if (e.offset % ALIGN != 0) why = "not 4 KiB aligned";
        else if (overflow || want != e.len) why = "its length does not match its shape";
        else if (e.offset + e.len < e.offset || e.offset + e.len > data_len) why = "it lies outside the data region";
        if (why) {
            const std::string msg = std::string(path) + ": tensor \"" + e.name + "\": " + why;
            tb_wpk_close(w);
            return fail(FORMAT, msg);
        }
        w->tensors.push_back(e);
    }
    if (t.left != 0) {
        tb_wpk_close(w);
        return fail(FORMAT, std::string(path) + ": the tensor table has trailing bytes");
    }
    *out = w;
    return OK;
}

void tb_wpk_close(tb_wpk* w) {
    if (!w) return;
    if (w->fd >= 0) close(w->fd);
    delete w;
}

uint32_t tb_wpk_count(const tb_wpk* w) { return w ? (uint32_t)w->tensors.size() : 0; }

int tb_wpk_tensor(const tb_wpk* w, uint32_t index, tb_wpk_info* out) {
    if (!w || !out || index >= w->tensors.size()) return fail(OUT_OF_RANGE, "tb_wpk_tensor: no such tensor");
    const tb_wpk::Entry& e = w->tensors[index];
    out->name = e.name.c_str(), out->dtype = e.dtype, out->rank = e.rank, out->offset = e.offset, out->bytes = e.len, out->crc32c = e.crc;
    for (int k = 0; k < 8; k++) out->shape[k] = e.shape[k];
    return OK;
}

int tb_wpk_read(const tb_wpk* w, uint32_t index, void* host, size_t bytes, int verify) {
    if (!w || !host || index >= w->tensors.size()) return fail(OUT_OF_RANGE, "tb_wpk_read: no such tensor");
    const tb_wpk::Entry& e = w->tensors[index];
    if (bytes != e.len) return fail(OUT_OF_RANGE, "tb_wpk_read: the buffer does not have the tensor's size");
    if (!read_at(w->fd, host, bytes, ALIGN + e.offset)) return fail(IO, "tb_wpk_read: " + e.name + ": " + (errno ? strerror(errno) : "the file is truncated"));
    if (verify && crc32c(0, static_cast<const uint8_t*>(host), bytes) != e.crc) return fail(FORMAT, "tensor \"" + e.name + "\" is corrupt");  // Wpk::verify
    return OK;
}

}  // extern "C"

namespace {

// The file's tensors into a model, streamed (Loader::to_device, wpk/load.rs:20-60, with threads and pread where that has an
// io_uring): the tensors are cut into pieces of at most a slot, READERS threads read pieces into a ring of DEPTH pinned slots,
// checking each piece's CRC32C if asked, and the calling thread takes the pieces in the file's order, joins the pieces' sums
// into the tensor's, and hands each piece to `put` (name, offset in the tensor, bytes, length, the tensor's length), which
// uploads it.  A tensor that `in_parts` refuses comes as one piece, and the slots are as large as the largest of those.
// TACHYON_B200_LOAD_READERS=0 reads on the calling thread instead (the pieces and the checks are the same);
// TACHYON_B200_LOAD_SLOT_KB sets the size of a piece (a test cuts small tensors with it).
constexpr size_t SLOT_BYTES = (size_t)16 << 20;  // wpk/load.rs:19 CHUNK
constexpr int DEPTH = 12, READERS = 8;

struct Piece {
    uint32_t tensor;
    size_t offset, len;
};

template <typename P, typename F>
int load_all(const char* what, const char* path, int verify, P&& in_parts, F&& put) {
    tb_wpk* w = nullptr;
    TB_TRY(tb_wpk_open(path, &w));
    const char* env = getenv("TACHYON_B200_LOAD_SLOT_KB");
    const size_t SLOT = env && atoll(env) > 0 ? std::max<size_t>(ALIGN, ((size_t)atoll(env) << 10) / ALIGN * ALIGN) : SLOT_BYTES;
    size_t slot = 0;
    std::vector<Piece> pieces;
    for (uint32_t i = 0; i < w->tensors.size(); i++) {
        const tb_wpk::Entry& e = w->tensors[i];
        const size_t len = (size_t)e.len;
        if (len <= SLOT || !in_parts(e.name.c_str())) {
            pieces.push_back({i, 0, len});
            slot = std::max(slot, len);
        } else {
            for (size_t at = 0; at < len; at += SLOT) pieces.push_back({i, at, std::min(SLOT, len - at)});
            slot = std::max(slot, SLOT);
        }
    }
    slot = (slot + ALIGN - 1) / ALIGN * ALIGN;
    const size_t depth = std::min<size_t>(DEPTH, pieces.size());
    char* stage = nullptr;
    if (slot > 0 && cudaMallocHost(reinterpret_cast<void**>(&stage), depth * slot) != cudaSuccess) {
        cudaGetLastError();
        tb_wpk_close(w);
        return fail(OUT_OF_MEMORY, std::string(what) + ": no pinned memory for the staging slots");
    }
    env = getenv("TACHYON_B200_LOAD_READERS");
    const int readers = slot == 0 ? 0 : env ? std::max(0, std::min(16, atoi(env))) : READERS;

    // Piece i lives in slot i % depth: read once piece i - depth has been taken (taken > i - depth), taken once it is read.
    std::mutex m;
    std::condition_variable cv;
    std::vector<uint8_t> read_done(pieces.size(), 0);
    std::vector<uint32_t> sums(pieces.size(), 0);
    size_t taken = 0;
    std::atomic<size_t> next{0};
    bool stop = false;
    int read_errno = 0;
    size_t failed_piece = SIZE_MAX;
    auto read_piece = [&](size_t i) {
        const Piece& pc = pieces[i];
        const tb_wpk::Entry& e = w->tensors[pc.tensor];
        errno = 0;
        return read_at(w->fd, stage + (i % depth) * slot, pc.len, ALIGN + e.offset + pc.offset);
    };
    auto reader = [&] {
        for (;;) {
            const size_t i = next.fetch_add(1);
            if (i >= pieces.size()) return;
            {
                std::unique_lock<std::mutex> lock(m);
                cv.wait(lock, [&] { return stop || taken + depth > i; });
                if (stop) return;
            }
            const bool ok = read_piece(i);
            const int err = errno;
            if (ok && verify) sums[i] = crc32c(0, reinterpret_cast<const uint8_t*>(stage + (i % depth) * slot), pieces[i].len);
            std::lock_guard<std::mutex> lock(m);
            if (!ok && failed_piece == SIZE_MAX) failed_piece = i, read_errno = err;
            read_done[i] = 1;
            cv.notify_all();
        }
    };
    std::vector<std::thread> threads;
    for (int k = 0; k < readers; k++) {
        try {
            threads.emplace_back(reader);
        } catch (...) {  // no more threads to be had: go on with the ones there are, or read on this thread
            break;
        }
    }
    const bool threaded = !threads.empty();

    int st = OK;
    uint32_t crc = 0;
    for (size_t i = 0; i < pieces.size() && st == OK; i++) {
        const Piece& pc = pieces[i];
        const tb_wpk::Entry& e = w->tensors[pc.tensor];
        bool ok = true;
        int err = 0;
        if (!threaded) {
            ok = read_piece(i), err = errno;
        } else {
            std::unique_lock<std::mutex> lock(m);
            cv.wait(lock, [&] { return read_done[i] != 0; });
            if (failed_piece == i) ok = false, err = read_errno;
        }
        const char* data = stage + (i % depth) * slot;
        if (!ok) st = fail(IO, std::string(what) + ": " + e.name + ": " + (err ? strerror(err) : "the file is truncated"));
        if (st == OK && verify) {
            const uint32_t sum = threaded ? sums[i] : crc32c(0, reinterpret_cast<const uint8_t*>(data), pc.len);
            crc = pc.offset == 0 ? sum : crc32c_combine(crc, sum, pc.len);
            if (pc.offset + pc.len == e.len && crc != e.crc) st = fail(FORMAT, "tensor \"" + e.name + "\" is corrupt");  // Wpk::verify
        }
        if (st == OK) st = put(e.name.c_str(), pc.offset, data, pc.len, (size_t)e.len);
        if (threaded) {
            std::lock_guard<std::mutex> lock(m);
            taken = i + 1;
            cv.notify_all();
        }
    }
    {
        std::lock_guard<std::mutex> lock(m);
        stop = true;
        cv.notify_all();
    }
    for (std::thread& t : threads) t.join();
    if (stage) cudaFreeHost(stage);
    tb_wpk_close(w);
    return st;
}

}  // namespace

extern "C" {

int tb_decoder_load_wpk(tb_decoder* dec, const char* path, int verify) {
    if (!dec) return fail(OUT_OF_RANGE, "tb_decoder_load_wpk: null decoder");
    return load_all(
        "tb_decoder_load_wpk", path, verify, [&](const char* name) { return tb_decoder_loads_in_parts(dec, name) != 0; },
        [&](const char* name, size_t offset, const void* data, size_t bytes, size_t total) { return tb_decoder_load_part(dec, name, offset, data, bytes, total); });
}

// An encoder's converted files (encoder/convert.rs: weights.wpk with the layers' matrices and norms, host.wpk with `embed`), each
// tensor under its own name through tb_encoder_load.
int tb_encoder_load_wpk(tb_encoder* enc, const char* path, int verify) {
    if (!enc) return fail(OUT_OF_RANGE, "tb_encoder_load_wpk: null encoder");
    return load_all(
        "tb_encoder_load_wpk", path, verify, [&](const char* name) { return tb_encoder_loads_in_parts(enc, name) != 0; },
        [&](const char* name, size_t offset, const void* data, size_t bytes, size_t total) { return tb_encoder_load_part(enc, name, offset, data, bytes, total); });
}

}  // extern "C"
