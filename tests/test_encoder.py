"""The packed variable-length encoder.  CPU: the oracle's forward against PyTorch's hidden states on the reference's tiny
encoder (crates/tachyon/tests/encoder.rs:162-181, bound 1e-4).  GPU: the kernels against the oracle on the same
fixture with Q8 weights (tests/encoder.rs:384-441: f16 path within 2e-2), packing invariance, and the benchmark's
variant (plain GELU FFN, mean pooling, truncated embeddings)."""
import json
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_encoder.npz")


def fixture():
    z = np.load(GOLDEN)
    cfg = json.loads(bytes(z["config_json"]).decode())
    weights = {k: z[k].astype(np.float32) for k in z.files if not k.startswith("case") and k not in ("config_json", "cases")}
    cases = [(z[f"case{i}.ids"], z[f"case{i}.hidden"]) for i in range(int(z["cases"][0]))]
    return cfg, weights, cases


def test_the_oracle_encoder_matches_pytorch():
    cfg, weights, cases = fixture()
    assert (cfg["global"], cfg["window"], int(cfg["theta_global"]), int(cfg["theta_local"])) == ([True, False, False], 8, 160000, 10000)
    for ids, hidden in cases:
        got = oracle.encoder_forward(cfg, weights, ids)
        assert np.abs(got.ravel() - hidden).max() < 1e-4


def quantize(w: np.ndarray):
    """Q8 as this build stores it: per 32 along a row an f16 scale amax/127 and int8 codes; returns codes, scale bits and
    the dequantised matrix (what the GPU multiplies with, up to its f16 rounding of code*scale)."""
    rows, cols = w.shape
    blocks = w.reshape(rows, cols // 32, 32)
    scale = (np.abs(blocks).max(axis=2) / 127.0).astype(np.float16)
    sf = scale.astype(np.float32)
    codes = np.where(sf[..., None] > 0, np.rint(blocks / np.where(sf[..., None] > 0, sf[..., None], 1.0)), 0).clip(-127, 127).astype(np.int8)
    deq = (codes.astype(np.float32) * sf[..., None]).reshape(rows, cols)
    return codes.reshape(rows, cols), scale.view(np.uint16), deq


def build(ctx, cfg, weights, tokens=1024, sequences=16, mean_pool=0, dims=None, fmt="q8"):
    """An encoder with `weights` loaded as this build's Q8 ("q8"), as a converted model's Q8E matrices and f32 scales per 64
    ("q8e", crates/tachyon/src/encoder/convert.rs:8-9) or as its f16 matrices ("f16"); and the weights the GPU then multiplies
    with, as f32."""
    import tachyon_b200 as tb

    glob = np.array([1 if g else 0 for g in cfg["global"]], np.uint8)
    ec = tb.EncoderConfig(hidden=cfg["hidden"], heads=cfg["heads"], inter=cfg["inter"], vocab=cfg["vocab"], layers=len(cfg["global"]), window=cfg["window"],
                          global_=glob.ctypes.data, global_every=0, theta_global=cfg["theta_global"], theta_local=cfg["theta_local"], eps=cfg["eps"],
                          gated=int(cfg.get("gated", 1)), mean_pool=mean_pool, dims=dims or cfg["hidden"])
    enc = tb.Encoder(ctx, ec, tokens=tokens, sequences=sequences)
    deq = dict(weights)
    for name, w in weights.items():
        if w.ndim == 2 and name != "embed" and fmt == "q8e":
            q, sc = oracle.q8e(w)
            enc.load(name, q.reshape(w.shape))
            enc.load(name + ".scale", sc.reshape(w.shape[0], -1))
            # the device keeps the scales as f16
            deq[name] = (q.reshape(w.shape[0], -1, 64).astype(np.float32) * sc.astype(np.float16).astype(np.float32).reshape(w.shape[0], -1, 1)).reshape(w.shape)
        elif w.ndim == 2 and name != "embed" and fmt == "f16":
            enc.load(name, w.astype(np.float16))
            deq[name] = w.astype(np.float16).astype(np.float32)
        elif w.ndim == 2 and name != "embed":
            codes, scales, d = quantize(w)
            enc.load(name + ".w", codes)
            enc.load(name + ".s", scales)
            deq[name] = d
        elif name == "embed":
            enc.load(name, w.astype(np.float16))
            deq[name] = w.astype(np.float16).astype(np.float32)
        else:
            enc.load(name, w.astype(np.float32))
    enc._glob = glob
    return enc, deq


@pytest.mark.gpu
def test_gpu_encoder_matches_the_oracle_on_the_reference_fixture(ctx):
    cfg, weights, cases = fixture()
    enc, deq = build(ctx, cfg, weights)
    for ids, hidden in cases:
        emb = enc.embed([ids])
        got = enc.hidden()
        want = oracle.encoder_forward(cfg, deq, ids)
        assert np.abs(got - want).max() < 2e-2, float(np.abs(got - want).max())
        # and, through the 8-bit weights, still PyTorch's states
        ref = hidden.reshape(len(ids), -1)
        cos = (got * ref).sum(1) / (np.linalg.norm(got, axis=1) * np.linalg.norm(ref, axis=1))
        assert cos.min() > 0.999
        # the embedding is the first token's state, normalised
        first = got[0] / max(np.linalg.norm(got[0]), 1e-12)
        assert np.allclose(emb[0], first, atol=1e-6)
    enc.close()


@pytest.mark.gpu
def test_packing_does_not_change_a_sequence(ctx):
    """Packed with others or alone, a sequence's embedding has the same bits (rows past the tokens are never mixed in)."""
    cfg, weights, _ = fixture()
    enc, _ = build(ctx, cfg, weights)
    rng = np.random.default_rng(3)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (1, 16, 64, 65, 130, 7, 200)]
    packed = enc.embed(seqs)
    for i, q in enumerate(seqs):
        alone = enc.embed([q])
        assert np.array_equal(alone[0], packed[i]), i
    assert np.allclose(np.linalg.norm(packed, axis=1), 1.0, atol=1e-5)
    enc.close()


@pytest.mark.gpu
def test_benchmark_variant_plain_ffn_mean_pool_truncated(ctx):
    """Plain GELU FFN, head size 64, every third layer global, mean pooling, 64 of 256 dimensions kept."""
    rng = np.random.default_rng(11)
    cfg = {"hidden": 256, "heads": 4, "inter": 512, "vocab": 500, "window": 8, "gated": 0, "theta_global": 160000.0, "theta_local": 10000.0, "eps": 1e-5,
           "global": [True, False, False, True]}
    h, inter = cfg["hidden"], cfg["inter"]
    weights = {"embed": rng.standard_normal((cfg["vocab"], h)).astype(np.float32), "embed_norm": rng.uniform(0.5, 1.5, h).astype(np.float32),
               "final_norm": rng.uniform(0.5, 1.5, h).astype(np.float32)}
    for l in range(4):
        if l > 0:
            weights[f"{l}.attn_norm"] = rng.uniform(0.5, 1.5, h).astype(np.float32)
        weights[f"{l}.mlp_norm"] = rng.uniform(0.5, 1.5, h).astype(np.float32)
        for name, shape in (("qkv", (3 * h, h)), ("o", (h, h)), ("up", (inter, h)), ("down", (h, inter))):
            weights[f"{l}.{name}"] = (rng.standard_normal(shape) * 0.05).astype(np.float32)
    enc, deq = build(ctx, cfg, weights, mean_pool=1, dims=64)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (40, 100, 17)]
    got = enc.embed(seqs)
    hidden = enc.hidden()
    at = 0
    for i, q in enumerate(seqs):
        want_h = oracle.encoder_forward(cfg, deq, q)
        assert np.abs(hidden[at:at + len(q)] - want_h).max() < 3e-2, float(np.abs(hidden[at:at + len(q)] - want_h).max())
        v = want_h.mean(0)
        v = v / max(np.linalg.norm(v), 1e-12)
        v = v[:64] / max(np.linalg.norm(v[:64]), 1e-12)
        assert np.abs(got[i] - v).max() < 5e-3
        at += len(q)
    enc.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["q8e", "f16"])
def test_a_converted_encoder_loads_from_its_files(ctx, tmp_path, fmt):
    """weights.wpk (the layers) and host.wpk (`embed`), as the reference's conversion lays them out (encoder/convert.rs:60-110),
    through tb_encoder_load_wpk: the bits of the tensor-by-tensor load; a tensor the encoder does not know is an error."""
    import tachyon_b200 as tb
    import wpk_writer as ww

    cfg, weights, cases = fixture()
    a, _ = build(ctx, cfg, weights, fmt=fmt)
    device, host = [], []
    for name, w in weights.items():
        if name == "embed":
            host.append((name, "f16", list(w.shape), w.astype(np.float16).tobytes()))
        elif w.ndim == 2 and fmt == "q8e":
            q, sc = oracle.q8e(w)
            device.append((name, "i8", list(w.shape), q.astype(np.int8).tobytes()))
            device.append((name + ".scale", "f32", [w.shape[0], w.shape[1] // 64], sc.astype(np.float32).tobytes()))
        elif w.ndim == 2:
            device.append((name, "f16", list(w.shape), w.astype(np.float16).tobytes()))
        else:
            device.append((name, "f32", list(w.shape), w.astype(np.float32).tobytes()))
    ww.write(str(tmp_path / "weights.wpk"), device, crc=ww.fast_crc32c)
    ww.write(str(tmp_path / "host.wpk"), host, crc=ww.fast_crc32c)
    b = tb.Encoder(ctx, a.cfg, tokens=1024, sequences=16)
    b._glob = a._glob
    b.load_wpk(str(tmp_path / "weights.wpk"))
    b.load_wpk(str(tmp_path / "host.wpk"))
    seqs = [ids for ids, _ in cases]
    assert np.array_equal(a.embed(seqs), b.embed(seqs))
    ww.write(str(tmp_path / "odd.wpk"), [("nobody", "f32", [4], np.zeros(4, np.float32).tobytes())])
    with pytest.raises(tb.Error):
        b.load_wpk(str(tmp_path / "odd.wpk"))
    with pytest.raises(tb.Error):
        b.load_wpk(str(tmp_path / "missing.wpk"))
    a.close(), b.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,bound,cosine", [("q8e", 2e-2, 0.9999), ("f16", 1e-2, 0.99999)])
def test_a_converted_models_matrices_load_as_they_are(ctx, fmt, bound, cosine):
    """The tiny encoder with its layers in Q8E or f16, as the reference's conversion writes them (encoder/convert.rs:79-95;
    crates/tachyon/tests/encoder.rs:410-441 wants a cosine of 0.99999 of the f32 reference in Q8 on its own tiny model)."""
    cfg, weights, cases = fixture()
    enc, deq = build(ctx, cfg, weights, fmt=fmt)
    for ids, hidden in cases:
        enc.embed([ids])
        got = enc.hidden()
        want = oracle.encoder_forward(cfg, deq, ids)
        assert np.abs(got - want).max() < bound, float(np.abs(got - want).max())
        ref = hidden.reshape(len(ids), -1)
        cos = (got * ref).sum(1) / (np.linalg.norm(got, axis=1) * np.linalg.norm(ref, axis=1))
        assert cos.min() > cosine, float(cos.min())
    enc.close()


def random_model(rng, h=256, heads=4, inter=512, vocab=500, layers=3, gated=1):
    cfg = {"hidden": h, "heads": heads, "inter": inter, "vocab": vocab, "window": 8, "gated": gated, "theta_global": 160000.0, "theta_local": 10000.0, "eps": 1e-5,
           "global": [l % 3 == 0 for l in range(layers)]}
    weights = {"embed": rng.standard_normal((vocab, h)).astype(np.float32), "embed_norm": rng.uniform(0.5, 1.5, h).astype(np.float32),
               "final_norm": rng.uniform(0.5, 1.5, h).astype(np.float32)}
    for l in range(layers):
        if l > 0:
            weights[f"{l}.attn_norm"] = rng.uniform(0.5, 1.5, h).astype(np.float32)
        weights[f"{l}.mlp_norm"] = rng.uniform(0.5, 1.5, h).astype(np.float32)
        for name, shape in (("qkv", (3 * h, h)), ("o", (h, h)), ("up", ((2 if gated else 1) * inter, h)), ("down", (h, inter))):
            weights[f"{l}.{name}"] = (rng.standard_normal(shape) * 0.05).astype(np.float32)
    return cfg, weights


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["q8", "q8e", "f16"])
def test_a_silu_gate(ctx, fmt):
    """Config::silu (encoder/mod.rs:55-56): the gate is a SiLU, store mode 5 of the up product."""
    rng = np.random.default_rng(21)
    cfg, weights = random_model(rng, gated=2)
    enc, deq = build(ctx, cfg, weights, fmt=fmt)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (33, 90)]
    enc.embed(seqs)
    hidden, at = enc.hidden(), 0
    for q in seqs:
        want = oracle.encoder_forward(cfg, deq, q)
        assert np.abs(hidden[at:at + len(q)] - want).max() < 3e-2, float(np.abs(hidden[at:at + len(q)] - want).max())
        at += len(q)
    # and it is not the GELU gate
    other = oracle.encoder_forward(dict(cfg, gated=1), deq, seqs[0])
    assert np.abs(hidden[:len(seqs[0])] - other).max() > 5e-2
    enc.close()


@pytest.mark.gpu
def test_batches_fill_the_capacity_in_order(ctx):
    """Encoder::batches (encoder/run.rs:207-221): more tokens than the capacity go in several batches, each closed by the
    first sequence that no longer fits; every sequence's embedding has the bits it has alone.  A batch runs as the graph of
    its padded shape (run.rs:379-410), recorded once."""
    import tachyon_b200 as tb

    cfg, weights, _ = fixture()
    enc, _ = build(ctx, cfg, weights, tokens=128, sequences=4)
    rng = np.random.default_rng(5)
    lens = (40, 40, 40, 100, 28, 1, 1, 1, 1, 1, 128)  # batches: [40 40 40] [100 28] [1 1 1 1] (four sequences) [1] [128]
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    got = enc.embed(seqs)
    assert enc.hidden().shape[0] == 128, "the last batch is the last sequence"
    assert enc.graphs() == 5  # padded tokens and sequences: (128, 3), (128, 2), (64, 4), (64, 1), (128, 1)
    assert np.allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-5)
    big, _ = build(ctx, cfg, weights, tokens=1024, sequences=16)
    assert np.array_equal(big.embed(seqs), got), "one batch or five: the same bits"
    big.close()
    enc.close()


@pytest.mark.gpu
def test_a_batchs_graph_gives_the_bits_of_its_kernels(ctx, monkeypatch):
    cfg, weights, _ = fixture()
    rng = np.random.default_rng(6)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (40, 40, 40, 100, 28, 1, 1, 1, 1, 1, 128)]
    enc, _ = build(ctx, cfg, weights, tokens=128, sequences=4)
    got = enc.embed(seqs)
    again = enc.embed(seqs)  # every shape now replays
    assert enc.graphs() == 5
    for i, q in enumerate(seqs):
        assert np.array_equal(enc.embed([q])[0], got[i]), i
    assert np.array_equal(got, again)
    enc.close()
    monkeypatch.setenv("TACHYON_B200_ENCODER_GRAPHS", "0")
    plain, _ = build(ctx, cfg, weights, tokens=128, sequences=4)
    assert np.array_equal(plain.embed(seqs), got) and plain.graphs() == 0
    plain.close()


@pytest.mark.gpu
def test_sixteen_shapes_are_kept(ctx):
    """GRAPHS = 16 (encoder/run.rs:20): the oldest shape is dropped for the seventeenth."""
    cfg, weights, _ = fixture()
    enc, _ = build(ctx, cfg, weights, tokens=1280, sequences=4)
    first = enc.embed([[5] * 10, [6] * 3])
    for n in range(1, 19):
        enc.embed([[7] * (64 * n)])
        assert enc.graphs() == min(n + 1, 16)
    assert np.array_equal(enc.embed([[5] * 10, [6] * 3]), first), "a dropped shape is recorded again"
    enc.close()


@pytest.mark.gpu
def test_encoder_refuses_what_it_cannot_hold(ctx):
    import tachyon_b200 as tb

    cfg, weights, _ = fixture()
    enc, _ = build(ctx, cfg, weights, tokens=64, sequences=2)
    assert enc.embed([[1] * 40, [2] * 40]).shape == (2, cfg["hidden"])  # two batches
    with pytest.raises(tb.Error) as e:
        enc.embed([[1] * 10, [2] * 65])
    assert e.value.status == 6  # TB_TOO_LONG (Error::TooLong, run.rs:208-210)
    with pytest.raises(tb.Error):
        enc.embed([[1], []])
    with pytest.raises(tb.Error):
        enc.embed([[cfg["vocab"]]])
    with pytest.raises(tb.Error) as e:
        enc.load("0.qkv", np.zeros(7, np.int8))
    assert e.value.status == 5
    with pytest.raises(tb.Error) as e:
        enc.load("9.qkv", np.zeros(7, np.int8))
    assert e.value.status == 8
    enc.close()


@pytest.mark.gpu
def test_attention_on_tcgen05_and_on_mma_sync_agree(ctx):
    """An encoder with heads of 64 opened while tb_context_set_flash is 1 (the default) runs its attention on tcgen05, tiles of 128
    queries of a sequence and head; opened under 0, on mma.sync with tiles of 64.  Same hidden states to the rounding of the
    probabilities, on sequences shorter and longer than a tile and past the window, alone or packed."""
    rng = np.random.default_rng(31)
    cfg, weights = random_model(rng, h=256, heads=4, inter=512, layers=4)  # layers 0 and 3 global, 1 and 2 within 8 either way
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (1, 63, 64, 65, 127, 128, 129, 300, 512, 17)]
    hidden = []
    for which in (0, 1):
        ctx.set_flash(which)
        try:
            enc, deq = build(ctx, cfg, weights, tokens=2048, sequences=16)
        finally:
            ctx.set_flash(1)
        emb = enc.embed(seqs)
        hidden.append(enc.hidden())
        if which == 1:
            for i in (0, 4, 7, 8):
                assert np.array_equal(enc.embed([seqs[i]])[0], emb[i]), "packed or alone: the same bits"
        enc.close()
    top = np.abs(hidden[0]).max()
    assert np.abs(hidden[0] - hidden[1]).max() <= 4e-3 * top, float(np.abs(hidden[0] - hidden[1]).max() / top)
    at = 0
    for q in seqs[:8]:
        want = oracle.encoder_forward(cfg, deq, q)
        assert np.abs(hidden[1][at:at + len(q)] - want).max() < 3e-2
        at += len(q)
    assert ctx.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["q8", "f16"])
def test_the_rotation_in_the_products_store_matches_the_kernel_of_its_own(ctx, monkeypatch, fmt):
    """The q/k/v product turns queries and keys as it stores them, from a copy of the matrix with a head's rows j and j + d/2 side
    by side; q and k then have their dimensions in that order, which changes the order of the dot products' sums and nothing
    else.  TACHYON_B200_ENCODER_ROPE=1 switches it on; against the rotation as a kernel of its own on the reference's fixture and on a
    model of heads of 64 with global and sliding layers; a tensor loaded afterwards is paired again."""
    rng = np.random.default_rng(11)
    for cfg, weights in (fixture()[:2], random_model(rng, h=256, heads=4, inter=512, layers=4)):
        monkeypatch.setenv("TACHYON_B200_ENCODER_ROPE", "1")
        fused, _ = build(ctx, cfg, weights, fmt=fmt)
        monkeypatch.delenv("TACHYON_B200_ENCODER_ROPE")
        apart, _ = build(ctx, cfg, weights, fmt=fmt)
        seqs = [list(rng.integers(0, cfg["vocab"], n)) for n in (5, 64, 65, 130, 300, 17)]
        a, b = fused.embed(seqs), apart.embed(seqs)
        assert np.abs(a - b).max() < 2e-3 * max(1.0, np.abs(b).max()), float(np.abs(a - b).max())
        cos = (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1))
        assert cos.min() > 0.99999, float(cos.min())
        # another q/k/v matrix for layer 1: both pick it up
        name = "1.qkv"
        w = (rng.standard_normal(weights[name].shape) * 0.05).astype(np.float32)
        for enc in (fused, apart):
            if fmt == "f16":
                enc.load(name, w.astype(np.float16))
            else:
                codes, scales, _ = quantize(w)
                enc.load(name + ".w", codes), enc.load(name + ".s", scales)
        a2, b2 = fused.embed(seqs), apart.embed(seqs)
        assert np.abs(a2 - b2).max() < 2e-3 * max(1.0, np.abs(b2).max()) and np.abs(a2 - a).max() > 1e-3
        fused.close(), apart.close()
