// Reader of `.wpk`, the reference's packed weight file (crates/tachyon/src/wpk/mod.rs:6-10, 37-40, 146-213): a 4 KiB
// header (magic, version and tensor count, sizes, CRC32C of the table and of itself), the tensors' bytes each on a
// 4 KiB boundary, and a table with every tensor's name, element type, shape, offset, length and CRC32C.  Host code only:
// a converted model's weights.wpk is opened, checked as Wpk::open checks it, and its tensors handed to the decoder by
// their converted-model names (model/mod.rs:178-286).  The reference's loader streams the file with O_DIRECT into
// pinned memory (wpk/load.rs); this one reads each tensor with pread into a pinned staging buffer.
#include "../../include/tachyon_b200.h"
#include "internal.h"

#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/stat.h>
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

uint32_t crc32c(uint32_t crc, const uint8_t* p, size_t n) {
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

// Every tensor of the file through `load` (name, bytes in pinned memory, length), in the file's order.
template <typename F>
int load_all(const char* what, const char* path, int verify, F&& load) {
    tb_wpk* w = nullptr;
    TB_TRY(tb_wpk_open(path, &w));
    // One pinned staging buffer, as large as the largest tensor: the upload is a straight copy from it.
    size_t most = 0;
    for (const tb_wpk::Entry& e : w->tensors) most = e.len > most ? (size_t)e.len : most;
    void* stage = nullptr;
    if (most > 0 && cudaMallocHost(&stage, most) != cudaSuccess) {
        tb_wpk_close(w);
        return fail(OUT_OF_MEMORY, std::string(what) + ": no pinned memory for the staging buffer");
    }
    int st = OK;
    for (uint32_t i = 0; i < w->tensors.size() && st == OK; i++) {
        const tb_wpk::Entry& e = w->tensors[i];
        st = tb_wpk_read(w, i, stage, (size_t)e.len, verify);
        if (st == OK) st = load(e.name.c_str(), stage, (size_t)e.len);
    }
    if (stage) cudaFreeHost(stage);
    tb_wpk_close(w);
    return st;
}

}  // namespace

extern "C" {

int tb_decoder_load_wpk(tb_decoder* dec, const char* path, int verify) {
    if (!dec) return fail(OUT_OF_RANGE, "tb_decoder_load_wpk: null decoder");
    return load_all("tb_decoder_load_wpk", path, verify, [&](const char* name, const void* data, size_t bytes) { return tb_decoder_load(dec, name, data, bytes); });
}

// An encoder's converted files (encoder/convert.rs: weights.wpk with the layers' matrices and norms, host.wpk with `embed`), each
// tensor under its own name through tb_encoder_load.
int tb_encoder_load_wpk(tb_encoder* enc, const char* path, int verify) {
    if (!enc) return fail(OUT_OF_RANGE, "tb_encoder_load_wpk: null encoder");
    return load_all("tb_encoder_load_wpk", path, verify, [&](const char* name, const void* data, size_t bytes) { return tb_encoder_load(enc, name, data, bytes); });
}

}  // extern "C"
