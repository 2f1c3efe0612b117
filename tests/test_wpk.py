"""The `.wpk` reader against files written as the reference writes them; the cases of crates/tachyon/src/wpk/mod.rs:379-470
(check value of CRC32C, round trip, damaged files, bit rot, misaligned tensors).  No GPU: host code only."""
import os
import struct

import numpy as np
import pytest

import tachyon_b200 as tb
import wpk_writer as ww


def sample(tmp_path, name):
    raw = bytes((i * 7 % 251) & 255 for i in range(10_000))  # wpk/mod.rs:357-365
    path = str(tmp_path / f"{name}.wpk")
    ww.write(path, [("embed", "bf16", (50, 100), raw), ("norm", "f32", (3,), raw[:12]), ("packed", "u8", (10, 2, 5), raw[:100])])
    return path, raw


def rejection(path):
    with pytest.raises(tb.Error) as e:
        tb.Wpk(path)
    assert e.value.status == 5, e.value  # TB_FORMAT
    return str(e.value)


def patch(path, at, data):
    with open(path, "r+b") as f:
        f.seek(at)
        f.write(data)


def test_crc32c_matches_the_standard_check_value():
    assert tb.crc32c(b"123456789") == 0xE3069283 == ww.crc32c(b"123456789")
    long = bytes(i & 255 for i in range(1000))
    assert tb.crc32c(long[333:], tb.crc32c(long[:333])) == ww.crc32c(long) == tb.crc32c(long)
    assert tb.crc32c(b"") == 0


def test_checksums_of_pieces_join_into_the_whole(tmp_path):
    rng = np.random.default_rng(5)
    data = rng.integers(0, 256, 300_000, dtype=np.uint8).tobytes()
    whole = tb.crc32c(data)
    for cut in (0, 1, 7, 4096, 150_001, len(data) - 1, len(data)):
        a, b = data[:cut], data[cut:]
        assert tb.crc32c_combine(tb.crc32c(a), tb.crc32c(b), len(b)) == whole, cut
        assert tb.crc32c(b, tb.crc32c(a)) == whole, cut  # continuing gives the same
    three = tb.crc32c_combine(tb.crc32c_combine(tb.crc32c(data[:1000]), tb.crc32c(data[1000:70_000]), 69_000), tb.crc32c(data[70_000:]), len(data) - 70_000)
    assert three == whole
    assert tb.crc32c(data[:5000]) == ww.crc32c(data[:5000]), "the processor's instruction and the bit-at-a-time loop agree"


def test_written_tensors_read_back_aligned(tmp_path):
    path, raw = sample(tmp_path, "roundtrip")
    w = tb.Wpk(path)
    t = w.tensors()
    assert [x[0] for x in t] == ["embed", "norm", "packed"]
    assert all(x[3] % 4096 == 0 for x in t)
    assert t[1][2] == (3,) and t[2][2] == (10, 2, 5)
    assert os.path.getsize(path) == 4096 + 12288 + 2 * 4096 + len(ww.encode([(n, d, s, o, b, c) for n, d, s, o, b, c in t]))
    assert w.read(0).tobytes() == raw and w.read(1).tobytes() == raw[:12] and w.read(2).tobytes() == raw[:100]
    w.close()


def test_damaged_files_are_rejected(tmp_path):
    path, _ = sample(tmp_path, "damaged")
    size = os.path.getsize(path)
    patch(path, size - 1, b"\xff")
    assert "the tensor table is corrupt" in rejection(path)
    patch(path, 9, b"\xff")
    assert "the header is corrupt" in rejection(path)
    os.truncate(path, size - 1)
    why = rejection(path)
    assert "truncated" in why or "corrupt" in why
    patch(path, 0, b"NOTAWPK!")
    assert "not a .wpk file" in rejection(path)
    with open(path, "wb") as f:
        f.write(b"tiny")
    assert "the file ends early" in rejection(path)
    with pytest.raises(tb.Error) as e:
        tb.Wpk(str(tmp_path / "absent.wpk"))
    assert e.value.status == 11  # TB_IO


def test_corrupted_data_fails_verification(tmp_path):
    path, _ = sample(tmp_path, "bitrot")
    patch(path, 4096 + 5000, b"\xff")
    w = tb.Wpk(path)
    with pytest.raises(tb.Error) as e:
        w.read(0)
    assert e.value.status == 5 and '"embed"' in str(e.value)
    assert w.read(0, verify=False).nbytes == 10_000  # loading never touches the bytes with the CPU
    w.read(1)
    w.close()


def test_misaligned_and_mismatched_tensors_are_rejected(tmp_path):
    path = str(tmp_path / "misaligned.wpk")
    table = ww.encode([("w", 5, (8,), 100, 8, 0)])
    with open(path, "wb") as f:
        f.write(ww.header(1, 4096, table) + b"\0" * 4096 + table)
    assert 'tensor "w": not 4 KiB aligned' in rejection(path)
    table = ww.encode([("x", 1, (3,), 0, 5, 0)])  # three f16 are six bytes
    with open(path, "wb") as f:
        f.write(ww.header(1, 4096, table) + b"\0" * 4096 + table)
    assert "its length does not match its shape" in rejection(path)
    table = ww.encode([("y", 5, (8192,), 0, 8192, 0)])
    with open(path, "wb") as f:
        f.write(ww.header(1, 4096, table) + b"\0" * 4096 + table)
    assert "it lies outside the data region" in rejection(path)
    table = ww.encode([("z", 9, (8,), 0, 8, 0)])
    with open(path, "wb") as f:
        f.write(ww.header(1, 4096, table) + b"\0" * 4096 + table)
    assert "unknown element type" in rejection(path)


@pytest.mark.gpu
def test_a_converted_q4_model_loads_from_its_wpk(ctx, tmp_path):
    """weights.wpk as model::convert writes it (model/mod.rs:178-286): `<name>.w` u8 [rows, cols/2], `<name>.s` f16
    [rows, cols/64], vectors f32; the decoder that read the file gives the bits of the one filled on the device."""
    from oracle.model import OracleModel

    cfg = tb.gemma4_e4b_shape(layers=2, ffn=2048, vocab=2048)
    cfg.window, cfg.global_every = 16, 2
    ref = OracleModel(cfg, 31, context=64, chunk=0, weight_bits=4)
    tensors = []
    for name, a in ref.tensors.items():
        kind = "u8" if name.endswith(".w") else "f16" if name.endswith(".s") else "f32"
        a = np.ascontiguousarray(a)
        tensors.append((name, kind, a.shape, a.view(np.uint8).tobytes() if kind != "u8" else a.astype(np.uint8, copy=False).view(np.uint8).tobytes()))
    path = str(tmp_path / "weights.wpk")
    ww.write(path, tensors, crc=ww.fast_crc32c)
    a = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4)
    a.load_wpk(path)
    a.build()
    b = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4)
    b.fill_random(31)
    b.build()
    for token in [5, 99, 2000, 7]:
        assert a.step(token) == b.step(token)
        assert np.array_equal(a.logits(), b.logits())
    # the wrong format is refused by size, an unknown tensor by name
    c = tb.Decoder(ctx, cfg, context=64, weight_bits=8)
    with pytest.raises(tb.Error) as e:
        c.load_wpk(path)
    assert e.value.status == 5
    ww.write(path, [("per_layer_proj.w", "u8", (4,), b"abcd")])
    with pytest.raises(tb.Error) as e:
        a.load_wpk(path)
    assert e.value.status == 8
    a.close(), b.close(), c.close()


@pytest.mark.gpu
def test_a_converted_model_with_per_layer_inputs_loads_from_both_files(ctx, tmp_path):
    """An E-model's directory (model/mod.rs:178-204): weights.wpk with everything that lives in VRAM, host.wpk with the per-layer
    table `embed_per_layer`, which the decoder here keeps where the reference does, in pinned mapped host memory."""
    from oracle.model import OracleModel

    cfg = tb.gemma4_e4b_shape(layers=3, ffn=2048, vocab=2048)
    cfg.window, cfg.global_every, cfg.per_layer = 16, 3, 256
    ref = OracleModel(cfg, 33, context=64, chunk=0, weight_bits=4)
    files = {"weights.wpk": [], "host.wpk": []}
    for name, a in ref.tensors.items():
        kind = "u8" if name.endswith(".w") else "f16" if name.endswith(".s") else "f32"
        a = np.ascontiguousarray(a)
        files["host.wpk" if name.startswith("embed_per_layer") else "weights.wpk"].append((name, kind, a.shape, a.view(np.uint8).tobytes()))
    assert [t[0] for t in files["host.wpk"]] == ["embed_per_layer.w", "embed_per_layer.s"]
    for name, tensors in files.items():
        ww.write(str(tmp_path / name), tensors, crc=ww.fast_crc32c)
    a = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4, host_table=True)
    a.load_wpk(str(tmp_path / "weights.wpk"))
    a.load_wpk(str(tmp_path / "host.wpk"))
    a.build()
    b = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4)
    b.fill_random(33)
    b.build()
    for pos, token in enumerate([5, 99, 2000, 7]):
        assert a.step(token) == b.step(token) == ref.step(token, pos)[0]
        assert np.array_equal(a.logits(), b.logits())
    a.close(), b.close()


@pytest.mark.gpu
@pytest.mark.parametrize("readers", [0, 1, 4])
def test_a_file_streamed_in_pieces_loads_the_same(ctx, tmp_path, monkeypatch, readers):
    """The loader cuts tensors that are copied as they are into pieces of a slot, read ahead into a ring of pinned slots by
    reader threads and uploaded in order (the reference's Loader::to_device, wpk/load.rs:20-60); tensors rearranged on the
    way come whole.  With slots of 8 KiB every matrix of the small model is in pieces: the same bits as the plain load, with
    the checksums checked across pieces, and a flipped byte in the middle of a tensor in pieces is found."""
    from oracle.model import OracleModel

    cfg = tb.gemma4_e4b_shape(layers=3, ffn=2048, vocab=2048)
    cfg.window, cfg.global_every, cfg.per_layer = 16, 3, 256
    ref = OracleModel(cfg, 35, context=64, chunk=0, weight_bits=4)
    files = {"weights.wpk": [], "host.wpk": []}
    for name, a in ref.tensors.items():
        kind = "u8" if name.endswith(".w") else "f16" if name.endswith(".s") else "f32"
        a = np.ascontiguousarray(a)
        files["host.wpk" if name.startswith("embed_per_layer") else "weights.wpk"].append((name, kind, a.shape, a.view(np.uint8).tobytes()))
    for name, tensors in files.items():
        ww.write(str(tmp_path / name), tensors, crc=ww.fast_crc32c)
    plain = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4, host_table=True)
    plain.load_wpk(str(tmp_path / "weights.wpk")), plain.load_wpk(str(tmp_path / "host.wpk"))
    plain.build()
    monkeypatch.setenv("TACHYON_B200_LOAD_SLOT_KB", "8")
    monkeypatch.setenv("TACHYON_B200_LOAD_READERS", str(readers))
    cut = tb.Decoder(ctx, cfg, context=64, keep_logits=True, weight_bits=4, host_table=True)
    cut.load_wpk(str(tmp_path / "weights.wpk")), cut.load_wpk(str(tmp_path / "host.wpk"))
    cut.build()
    for pos, token in enumerate([5, 99, 2000, 7]):
        assert cut.step(token) == plain.step(token) == ref.step(token, pos)[0]
        assert np.array_equal(cut.logits(), plain.logits())
    # a flipped byte in the third piece of the first large tensor
    w = tb.Wpk(str(tmp_path / "weights.wpk"))
    big = next({"name": t[0], "offset": t[3], "bytes": t[4]} for t in w.tensors() if t[4] > 64 << 10 and "gate_up" not in t[0])
    w.close()
    raw = bytearray(open(tmp_path / "weights.wpk", "rb").read())
    raw[4096 + big["offset"] + 20000] ^= 0x40
    open(tmp_path / "damaged.wpk", "wb").write(raw)
    with pytest.raises(tb.Error) as e:
        cut.load_wpk(str(tmp_path / "damaged.wpk"))
    assert e.value.status == 5 and big["name"] in str(e.value)
    cut.load_wpk(str(tmp_path / "damaged.wpk"), verify=False)  # unchecked it loads
    # a file cut short: the read fails, the threads end, the error names the tensor
    open(tmp_path / "short.wpk", "wb").write(bytes(raw[: 4096 + big["offset"] + 30000]))
    with pytest.raises(tb.Error):
        cut.load_wpk(str(tmp_path / "short.wpk"))
    plain.close(), cut.close()
