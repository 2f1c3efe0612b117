"""Writes a `.wpk` the way the reference's Writer does (crates/tachyon/src/wpk/mod.rs:146-187, 270-337): 4 KiB header,
tensors each on a 4 KiB boundary, then the table.  Test infrastructure: the library only reads the format."""
import struct

ALIGN = 4096
DTYPES = {"f32": (0, 4), "f16": (1, 2), "bf16": (2, 2), "f8e4m3": (3, 1), "i8": (4, 1), "u8": (5, 1)}


def crc32c(data: bytes, crc: int = 0) -> int:
    """Bit-at-a-time CRC32C, the reference's crc32c_soft (wpk/mod.rs:121-123); independent of the library's table version."""
    c = ~crc & 0xFFFFFFFF
    for b in data:
        c ^= b
        for _ in range(8):
            c = (c >> 1) ^ (0x82F63B78 & -(c & 1))
    return ~c & 0xFFFFFFFF


def fast_crc32c(data: bytes) -> int:
    """The same value through the library, for tensors of megabytes (the pure-Python loop above pins it on small inputs)."""
    import tachyon_b200 as tb

    return tb.crc32c(data)


def encode(tensors) -> bytes:
    out = b""
    for name, dtype, shape, offset, length, crc in tensors:
        out += struct.pack("<H", len(name)) + name.encode() + bytes([dtype, len(shape)])
        out += b"".join(struct.pack("<Q", v) for v in list(shape) + [offset, length]) + struct.pack("<I", crc)
    return out


def header(count: int, data_len: int, table: bytes) -> bytes:
    head = b"TACHYWPK" + struct.pack("<QQQQ", 1 | count << 32, data_len, ALIGN + data_len, len(table))
    head += struct.pack("<I", crc32c(table))
    head += struct.pack("<I", crc32c(head))
    return head.ljust(ALIGN, b"\0")


def write(path: str, tensors, crc=crc32c) -> None:
    """tensors: [(name, dtype name, shape, bytes)]."""
    data, table = b"", []
    for name, dtype, shape, raw in tensors:
        code, size = DTYPES[dtype]
        n = size
        for d in shape:
            n *= d
        assert n == len(raw), (name, n, len(raw))
        table.append((name, code, shape, len(data), len(raw), crc(raw)))
        data += raw + b"\0" * (-len(raw) % ALIGN)
    t = encode(table)
    with open(path, "wb") as f:
        f.write(header(len(table), len(data), t) + data + t)
