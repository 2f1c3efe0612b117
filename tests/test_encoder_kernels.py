"""The encoder's kernels through the kernel-launch seam (tb_launch), by the reference's names and argument lists
(crates/tachyon/src/ptx/encoder.rs:5-38), as the reference's own GPU tests drive them: quant_f16 bit-exact against the CPU's
Q8E and the 8-bit product in every mode under each of its three names (crates/tachyon/tests/encoder.rs:320-356), the f16
product in every mode with a bias (tests/encoder.rs:240-302), and the small kernels (norm, rows, GELU, RoPE, attention)."""
import numpy as np
import pytest

import oracle
from util import f16, f16_to_f32, values, values_fast

pytestmark = pytest.mark.gpu

P, U, F = "p", "u", "f"


def erf_as(x):
    """Abramowitz and Stegun 7.1.26 (tests/encoder.rs:51-55)."""
    t = 1.0 / (1.0 + 0.3275911 * np.abs(x))
    y = 1.0 - (((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t * np.exp(-x * x)
    return np.sign(x) * y


def gelu(x):
    return 0.5 * x * (1.0 + erf_as(x / np.sqrt(2.0)))


def silu(x):
    return x / (1.0 + np.exp(-x))


def test_quant_f16_rounds_as_the_cpu_does(ctx):
    cols, tokens = 192, 128
    a16 = f16(values(tokens * cols, 8))
    a16[64:128] = 0  # a group of zeros: scale 0, codes 0
    ad, qd, sd = ctx.upload(a16), ctx.zeros(tokens * cols), ctx.zeros(tokens * cols // 16)
    ctx.launch("quant_f16", (1, tokens, 1), (256, 1, 1), 0, [(P, ad.ptr), (P, qd.ptr), (P, sd.ptr), (U, cols)])
    q, s = oracle.q8e(f16_to_f32(a16))
    assert np.array_equal(qd.download(np.int8, tokens * cols), q), "the GPU's rounding differs from the CPU's"
    assert np.array_equal(sd.download(np.float32, tokens * cols // 64).view(np.uint32), s.view(np.uint32))
    # 20 groups a row: three blocks of eight warps, the last one partly idle
    cols = 1280
    a16 = f16(values_fast(5 * cols, 9) * 30.0)
    ad, qd, sd = ctx.upload(a16), ctx.zeros(5 * cols), ctx.zeros(5 * cols // 16)
    ctx.launch("quant_f16", (3, 5, 1), (256, 1, 1), 0, [(P, ad.ptr), (P, qd.ptr), (P, sd.ptr), (U, cols)])
    q, s = oracle.q8e(f16_to_f32(a16))
    assert np.array_equal(qd.download(np.int8, 5 * cols), q) and np.array_equal(sd.download(np.float32, 5 * cols // 64), s)


def expected(mode, v, base):
    """What store mode `mode` leaves from the sums v [tokens, rows] (ptx/encoder.rs:5-9)."""
    if mode == 0:
        return v
    if mode == 1:
        return v + base
    if mode == 2:
        return v
    if mode == 3:
        return np.maximum(v, 0.0)
    gate = gelu(v[:, 0::2]) if mode == 4 else silu(v[:, 0::2])
    return gate * v[:, 1::2]


def read_back(y, mode, tokens, rows):
    if mode < 2:
        return y.download(np.float32, 128 * rows).reshape(128, rows)[:tokens].astype(np.float64)
    width = rows // 2 if mode >= 4 else rows
    return f16_to_f32(y.download(np.uint16, tokens * width)).reshape(tokens, width).astype(np.float64)


@pytest.mark.parametrize("kernel,blocks,threads", [("gemm_q8", 4, 128), ("gemm_q8_128", 2, 256), ("gemm_q8_tall", 1, 512)])
def test_the_q8_product_matches_the_cpu_in_every_mode(ctx, kernel, blocks, threads):
    rows, cols, tokens = 128, 192, 70
    a = f16_to_f32(f16(values(128 * cols, 8)))
    w, bias = values(rows * cols, 9), values(rows, 11)
    (aq, sa), (wq, sw) = oracle.q8e(a), oracle.q8e(w)
    base = values(128 * rows, 10).reshape(128, rows)
    qb, sb, wb, swb, bb = ctx.upload(aq), ctx.upload(sa), ctx.upload(wq), ctx.upload(sw), ctx.upload(bias)
    for with_bias in (False, True):
        sums = oracle.gemm_q8e(aq[:tokens * cols], sa[:tokens * cols // 64], wq, sw, rows, bias if with_bias else None)
        for mode in range(6):
            y = ctx.upload(base)
            ctx.launch(kernel, (blocks, 1, 1), (threads, 1, 1), 0,
                       [(P, qb.ptr), (P, wb.ptr), (P, bb.ptr if with_bias else 0), (P, y.ptr), (U, rows), (U, cols), (U, tokens), (U, mode), (P, sb.ptr), (P, swb.ptr)])
            got, want = read_back(y, mode, tokens, rows), expected(mode, sums.astype(np.float64), base[:tokens].astype(np.float64))
            assert np.all(np.abs(got - want) <= 1e-3 + 2e-3 * np.abs(want)), (kernel, mode, float(np.abs(got - want).max()))
            if mode == 0:  # the sums themselves: the same operations in the same order, so the same bits
                assert np.array_equal(got.astype(np.float32).view(np.uint32), sums.view(np.uint32)), "the sums differ from the CPU's"
            if mode < 2:
                past = y.download(np.float32, 128 * rows).reshape(128, rows)[tokens:]
                assert np.array_equal(past.view(np.uint32), base[tokens:].view(np.uint32)), "rows past the tokens were written"
    assert ctx.status() == 0


@pytest.mark.parametrize("kernel,blocks,threads", [("gemm_f16", 4, 128), ("gemm_f16_128", 2, 256), ("gemm_f16_tall", 1, 512)])
def test_the_f16_product_matches_the_cpu_in_every_mode(ctx, kernel, blocks, threads):
    rows, tokens = 128, 70
    for cols, seed in ((192, 1), (256, 5)):
        a16, w16 = f16(values(128 * cols, seed)), f16(values(rows * cols, seed + 1))
        bias, base = values(rows, seed + 2), values(128 * rows, seed + 3).reshape(128, rows)
        sums = f16_to_f32(a16).astype(np.float64).reshape(128, cols)[:tokens] @ f16_to_f32(w16).astype(np.float64).reshape(rows, cols).T
        ab, wb, bb = ctx.upload(a16), ctx.upload(w16), ctx.upload(bias)
        for with_bias in (True, False):
            v = sums + (bias.astype(np.float64)[None, :] if with_bias else 0.0)
            for mode in range(6):
                y = ctx.upload(base)
                ctx.launch(kernel, (blocks, 1, 1), (threads, 1, 1), 0,
                           [(P, ab.ptr), (P, wb.ptr), (P, bb.ptr if with_bias else 0), (P, y.ptr), (U, rows), (U, cols), (U, tokens), (U, mode)])
                got, want = read_back(y, mode, tokens, rows), expected(mode, v, base[:tokens].astype(np.float64))
                slack = 1e-3 if mode < 2 else 1e-3 + 2e-3 * np.abs(want)
                assert np.all(np.abs(got - want) <= slack), (kernel, cols, mode, float(np.abs(got - want).max()))
                if mode < 2:
                    past = y.download(np.float32, 128 * rows).reshape(128, rows)[tokens:]
                    assert np.array_equal(past.view(np.uint32), base[tokens:].view(np.uint32)), "rows past the tokens were written"
    assert ctx.status() == 0


@pytest.mark.parametrize("h", [768, 100, 4096])
def test_norm_f16_with_and_without_a_bias(ctx, h):
    n = 9
    x = (values_fast(n * h, h) * 3.0 + 50.0).reshape(n, h)  # a large mean
    gamma, beta = 1.0 + values_fast(h, 1), values_fast(h, 2)
    x64 = x.astype(np.float64)
    norm = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5)
    gd, bd = ctx.upload(gamma), ctx.upload(beta)
    for with_beta, in_place in ((True, True), (False, False), (True, None)):
        want = norm * gamma + (beta if with_beta else 0.0)
        xd, a = ctx.upload(x), ctx.zeros(n * h * 2)
        xo = xd if in_place else ctx.zeros(n * h * 4) if in_place is False else None
        ctx.launch("norm_f16", (n, 1, 1), ((h // 4 + 31) // 32 * 32, 1, 1), 0,
                   [(P, xd.ptr), (P, gd.ptr), (P, bd.ptr if with_beta else 0), (P, a.ptr), (P, xo.ptr if xo else 0), (U, h), (F, 1e-5)])
        got16 = f16_to_f32(a.download(np.uint16, n * h)).reshape(n, h)
        assert np.all(np.abs(got16 - want) <= 2e-3 + 1e-3 * np.abs(want)), float(np.abs(got16 - want).max())
        if xo is not None:
            got32 = xo.download(np.float32, n * h).reshape(n, h)
            assert np.all(np.abs(got32 - want) <= 2e-4), float(np.abs(got32 - want).max())
            assert np.array_equal(f16(got32).reshape(n, h), a.download(np.uint16, n * h).reshape(n, h)), "the f16 copy is the f32 one, rounded"
        else:
            assert np.array_equal(xd.download(np.float32, n * h), x.ravel()), "x is left alone without xo"


def test_the_row_kernels(ctx):
    h, n, rows = 300, 7, 20
    table32, table16 = values_fast(rows * h, 1), f16(values_fast(rows * h, 2))
    idx = np.array([3, 0, 19, 3, 7, 7, 1], np.uint32)
    base = values_fast(n * h, 3)
    t32, t16, idxd = ctx.upload(table32), ctx.upload(table16), ctx.upload(idx)
    grid = ((h + 255) // 256, n, 1)
    for name, table, want in (("embed_f16", t16, f16_to_f32(table16).reshape(rows, h)[idx]), ("gather_rows", t32, table32.reshape(rows, h)[idx]),
                              ("add_rows", t32, base.reshape(n, h) + table32.reshape(rows, h)[idx]),
                              ("add_rows_f16", t16, base.reshape(n, h) + f16_to_f32(table16).reshape(rows, h)[idx])):
        out = ctx.upload(base)
        ctx.launch(name, grid, (256, 1, 1), 0, [(P, table.ptr), (P, idxd.ptr), (P, out.ptr), (U, h)])
        assert np.array_equal(out.download(np.float32, n * h).reshape(n, h), want.astype(np.float32)), name


def test_gelu_f16_plain_and_gated(ctx):
    width, n = 96, 5
    x = values_fast(n * 2 * width, 4) * 4.0
    xd = ctx.upload(x)
    for gated in (0, 1):
        out = ctx.zeros(n * width * 2)
        ctx.launch("gelu_f16", ((n * width + 255) // 256, 1, 1), (256, 1, 1), 0, [(P, xd.ptr), (P, out.ptr), (U, width), (U, n * width), (U, gated)])
        v = x.astype(np.float64)
        want = gelu(v.reshape(n, 2 * width)[:, :width]) * v.reshape(n, 2 * width)[:, width:] if gated else gelu(v[:n * width]).reshape(n, width)
        got = f16_to_f32(out.download(np.uint16, n * width)).reshape(n, width)
        assert np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want)), float(np.abs(got - want).max())


@pytest.mark.parametrize("d", [32, 64])
def test_rope_f16_turns_by_the_table_bit_for_bit(ctx, d):
    h, n, positions = 4 * d, 11, 40
    qkv = f16(values_fast(n * 3 * h, d))
    table = oracle.rope_table(10000.0, positions, d)
    pos = np.array([0, 1, 2, 39, 17, 0, 5, 6, 7, 8, 30], np.uint32)
    qd = ctx.upload(qkv)
    tabled, posd = ctx.upload(table), ctx.upload(pos)
    ctx.launch("rope_f16", ((h // 2 + 255) // 256, n, 1), (256, 1, 1), 0, [(P, qd.ptr), (P, tabled.ptr), (P, posd.ptr), (U, h), (U, d)])
    got = qd.download(np.uint16, n * 3 * h).reshape(n, 3, h // d, d)
    v = f16_to_f32(qkv).reshape(n, 3, h // d, d)
    a, b = v[:, :2, :, :d // 2].astype(np.float64), v[:, :2, :, d // 2:].astype(np.float64)
    c, s = table[pos][:, None, None, :, 0].astype(np.float64), table[pos][:, None, None, :, 1].astype(np.float64)
    # a product rounded to f32, then one fused multiply-add (ptx/encoder.rs:942-956)
    x = (b * -s + (a * c).astype(np.float32).astype(np.float64)).astype(np.float32)
    y = (a * s + (b * c).astype(np.float32).astype(np.float64)).astype(np.float32)
    want = v.copy()
    want[:, :2, :, :d // 2], want[:, :2, :, d // 2:] = x, y
    assert np.array_equal(got, f16(want).reshape(got.shape))
    assert np.array_equal(got[:, 2], qkv.reshape(n, 3, h // d, d)[:, 2]), "the values are left alone"


def attention(q, k, v, window):
    """softmax(q k^T / sqrt(d)) v of one sequence and head in f64, keys within `window` of the query (0: all)."""
    n, d = q.shape
    sc = q @ k.T / np.sqrt(d)
    if window:
        i, j = np.arange(n)[:, None], np.arange(n)[None, :]
        sc = np.where(np.abs(i - j) <= window, sc, -np.inf)
    p = np.exp(sc - sc.max(1, keepdims=True))
    return (p / p.sum(1, keepdims=True)) @ v


@pytest.mark.parametrize("d,kernel", [(64, "attend_f16"), (32, "attend_f16_32")])
@pytest.mark.parametrize("window", [0, 8])
def test_attend_f16_over_packed_sequences(ctx, d, kernel, window):
    heads, lens = 3, [70, 1, 130]
    h, n = heads * d, sum(lens)
    qkv = f16(values_fast(n * 3 * h, 5 + d) * 2.0)
    tiles, start = [], 0
    for ln in lens:
        tiles += [[start, ln, q0] for q0 in range(0, ln, 64)]
        start += ln
    tiles += [[0, 0, 0]] * 2  # unused slots of a padded batch
    td, qd, out = ctx.upload(np.array(tiles, np.uint32)), ctx.upload(qkv), ctx.upload(np.full(n * h, 0x7E00, np.uint16))
    ctx.launch(kernel, (len(tiles), heads, 1), (128, 1, 1), 0, [(P, qd.ptr), (P, out.ptr), (P, td.ptr), (U, h), (U, window), (F, float(np.log2(np.e) / np.sqrt(d)))])
    got = f16_to_f32(out.download(np.uint16, n * h)).reshape(n, heads, d)
    v = f16_to_f32(qkv).astype(np.float64).reshape(n, 3, heads, d)
    start = 0
    for ln in lens:
        for hd in range(heads):
            want = attention(v[start:start + ln, 0, hd], v[start:start + ln, 1, hd], v[start:start + ln, 2, hd], window)
            assert np.abs(got[start:start + ln, hd] - want).max() < 4e-3, (ln, hd)
        start += ln
    assert ctx.status() == 0


def test_the_seam_refuses_ragged_encoder_launches(ctx):
    import tachyon_b200 as tb

    z = ctx.zeros(1 << 16)
    with pytest.raises(tb.Error):
        ctx.launch("quant_f16", (1, 1, 1), (256, 1, 1), 0, [(P, z.ptr)] * 3 + [(U, 100)])  # not whole groups of 64
    with pytest.raises(tb.Error):
        ctx.launch("norm_f16", (1, 1, 1), (256, 1, 1), 0, [(P, z.ptr)] * 5 + [(U, 8192), (F, 1e-5)])  # wider than 4096
    with pytest.raises(tb.Error):
        ctx.launch("gemm_q8", (1, 1, 1), (128, 1, 1), 0, [(P, z.ptr)] * 4 + [(U, 64), (U, 64), (U, 1), (U, 6), (P, z.ptr), (P, z.ptr)])  # mode 6
    with pytest.raises(tb.Error):
        ctx.launch("gemm_f16", (1, 1, 1), (128, 1, 1), 0, [(P, z.ptr)] * 4 + [(U, 96), (U, 64), (U, 1), (U, 0)])  # rows not a multiple of 64
    with pytest.raises(tb.Error):
        ctx.launch("attend_f16", (1, 2, 1), (128, 1, 1), 0, [(P, z.ptr)] * 3 + [(U, 192), (U, 0), (F, 0.18)])  # three heads, two block rows
    with pytest.raises(tb.Error):
        ctx.launch("rope_f16", (1, 1, 1), (256, 1, 1), 0, [(P, z.ptr)] * 3 + [(U, 100), (U, 64)])  # h not whole heads
