"""The reference's prefill formats through the kernel-launch seam (tb_launch), by its kernel names and argument lists:
quant_q8p bit-exact against the CPU layout (crates/tachyon/tests/gemm.rs:72-81), gemm_q4 whole and in column slices with
sum_slices within the reference's own bound (tests/gemm.rs:17, 54-69, 86-101), norm_q8p against norm_q8 on many tokens
and geglu_q8p over strided rows with the padding left alone (tests/prefill.rs:50-99)."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16_to_f32, values, values_fast

pytestmark = pytest.mark.gpu


def launch_quant_q8p(ctx, x, cols):
    """x quantised on the GPU into buffers of whole tiles of 128 tokens of `cols` (tests/gemm.rs:19-32)."""
    padded = -(-(x.size // cols) // 128) * 128 * cols
    xd, q, s = ctx.upload(x), ctx.zeros(padded), ctx.zeros(padded // 8)
    ctx.launch("quant_q8p", (-(-x.size // 256), 1, 1), (256, 1, 1), 0, [("p", xd.ptr), ("p", q.ptr), ("p", s.ptr), ("u", x.size)])
    return q, s, q.download(np.int8, x.size), s.download(np.float32, x.size // 32)


def test_quant_q8p_matches_the_cpu_exactly(ctx):
    x = values(4096, 7)
    x[128:192] = 0.0
    x[300] = 1e-30
    _, _, q, s = launch_quant_q8p(ctx, x, 4096)
    cq, cs = oracle.q8p(x)
    assert np.array_equal(q, cq), "Q8P values differ"
    assert np.array_equal(s.view(np.uint32), cs.ravel().view(np.uint32)), "Q8P scales differ"
    # a length that is not a whole block of 256 threads: threads past the end store nothing
    y = values(64 * 7, 8)
    qd, sd = ctx.alloc(64 * 7 + 64), ctx.alloc(7 * 8 + 8)
    qd.upload(np.full(64 * 7 + 64, 0x55, np.uint8)), sd.upload(np.full(7 * 8 + 8, 0x55, np.uint8))
    yd = ctx.upload(y)
    ctx.launch("quant_q8p", (2, 1, 1), (256, 1, 1), 0, [("p", yd.ptr), ("p", qd.ptr), ("p", sd.ptr), ("u", y.size)])
    cq, cs = oracle.q8p(y)
    assert np.array_equal(qd.download(np.int8, 64 * 7), cq) and np.all(qd.download(np.uint8, 64 * 7 + 64)[64 * 7:] == 0x55)
    assert np.array_equal(sd.download(np.float32, 14).view(np.uint32), cs.ravel().view(np.uint32)) and np.all(sd.download(np.uint8, 64)[56:] == 0x55)


def nibbles(packed, rows, cols):
    """The Q4 codes minus 8 as f64 [rows, cols]: weight j of a group is nibble j % 8 / 4 of byte j / 8 * 4 + j % 4 (quant.rs:60-66)."""
    pk = packed.reshape(-1, 32)
    out = np.zeros((pk.shape[0], 64))
    for j in range(64):
        out[:, j] = (pk[:, j // 8 * 4 + j % 4] >> (j % 8 // 4 * 4)) & 15
    return (out - 8.0).reshape(rows, cols)


@pytest.mark.parametrize("slices", [1, 3])
@pytest.mark.parametrize("rows,cols,tokens", [(64, 128, 1), (128, 2560, 200), (256, 256, 130), (64, 10240, 37), (192, 384, 128)])
def test_gemm_q4_matches_the_reference_on_every_shape(ctx, rows, cols, tokens, slices):
    wf, x = values_fast(rows * cols, 21 + rows + cols), values_fast(tokens * cols, 77 + tokens)
    packed, scales = oracle.q4(wf)
    qd, sd, q, s = launch_quant_q8p(ctx, x, cols)
    slices = min(slices, cols // 128)
    y, wd, wsd = ctx.zeros(slices * tokens * rows * 4), ctx.upload(packed), ctx.upload(scales)  # held until the results are back
    ctx.launch("gemm_q4", (-(-tokens // 128), rows // 64, slices), (128, 1, 1), 0,
               [("p", wd.ptr), ("p", wsd.ptr), ("p", qd.ptr), ("p", sd.ptr), ("p", y.ptr), ("u", rows), ("u", cols), ("u", tokens)])
    n = tokens * rows
    ctx.launch("sum_slices", (-(-n // 1024), 1, 1), (256, 1, 1), 0, [("p", y.ptr), ("u", n), ("u", slices)])
    got = y.download(np.float32, n).reshape(tokens, rows).astype(np.float64)
    # tests/gemm.rs:54-69: per row the sum over groups of d * s * sum (n - 8) q; allowed: 1e-5 of the terms' magnitudes plus two
    # units d * s of each group's integer sum
    nib = nibbles(packed, rows, cols).reshape(rows, cols // 64, 64)
    qg = q.astype(np.float64).reshape(tokens, cols // 64, 64)
    dot = np.einsum("rgk,tgk->trg", nib, qg)
    unit = f16_to_f32(scales).astype(np.float64).reshape(rows, cols // 64)[None, :, :] * s.reshape(tokens, cols // 64, 2)[:, None, :, 0].astype(np.float64)
    want = (unit * dot).sum(2)
    bound = (1e-5 * np.abs(unit * dot) + 2.0 * unit).sum(2)
    assert np.all(np.abs(got - want) <= bound), float((np.abs(got - want) / bound).max())
    assert ctx.status() == 0


def run_norm(ctx, kernel, h, y, w1, w2, length, block):
    hd, ho, yd, w1d, w2d = (ctx.upload(a) for a in (h, h, y, w1, w2))
    q, s = ctx.zeros(h.size), ctx.zeros(h.size // block * 8)
    ctx.launch(kernel, (length // 256, h.size // length, 1), (256, 1, 1), 0,
               [("p", hd.ptr), ("p", ho.ptr), ("p", yd.ptr), ("p", w1d.ptr), ("p", w2d.ptr), ("p", q.ptr), ("p", s.ptr), ("u", length), ("f", 1e-6), ("f", 0.75)])
    return ho.download(np.float32, h.size), q.download(np.int8, h.size), s.download(np.float32, h.size // block * 2)


def check_q8p(q, s, want, slack):
    """tests/prefill.rs:14-30: the dequantised Q8P values are within half a step (plus slack) of what was quantised, and z is
    -8 s sum q - MAGIC s."""
    scale = np.repeat(s[0::2].astype(np.float64), 64)
    assert np.all(np.abs(q.astype(np.float64) * scale - want) <= 0.5 * scale + slack)
    sums = q.astype(np.float64).reshape(-1, 64).sum(1)
    z = -8.0 * s[0::2].astype(np.float64) * sums - 12582912.0 * s[0::2].astype(np.float64)
    assert np.all(np.abs(s[1::2] - z) <= 2e-7 * np.abs(z) + 1e-30)


def test_norm_q8p_matches_norm_q8_on_many_tokens(ctx):
    length, tokens = 2560, 5
    h, y = 20.0 * values_fast(length * tokens, 5), 300.0 * values_fast(length * tokens, 6)
    w1, w2 = 1.0 + values_fast(length, 3), 0.5 + values_fast(length, 4)
    h8, q8, s8 = run_norm(ctx, "norm_q8", h, y, w1, w2, length, 32)
    hp, qp, sp = run_norm(ctx, "norm_q8p", h, y, w1, w2, length, 64)
    assert np.array_equal(hp, h8), "the residual is the same"
    want = q8.astype(np.float64) * np.repeat(s8[0::2].astype(np.float64), 32)
    check_q8p(qp, sp, want, float((0.5 * s8[0::2]).max()))


def test_geglu_q8p_gates_strided_rows(ctx):
    width, tokens = 512, 3
    gate_up, table = 6.0 * values_fast(2 * width * tokens, 1), values_fast(3 * width * tokens, 2)
    gelu = lambda v: 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v ** 3)))
    gu, tbl = gate_up.astype(np.float64).reshape(tokens, 2 * width), table.astype(np.float64).reshape(tokens, 3 * width)
    want = (gelu(gu[:, :width]) * tbl[:, width:2 * width]).ravel()
    a, b = ctx.upload(gate_up), ctx.upload(table)
    for so in (width, width + 64):
        q, s = ctx.zeros(so * tokens), ctx.zeros(so * tokens // 8)
        n = width * tokens
        ctx.launch("geglu_q8p", (-(-n // 256), 1, 1), (256, 1, 1), 0,
                   [("p", a.ptr), ("p", b.ptr + 4 * width), ("p", q.ptr), ("p", s.ptr), ("u", n), ("u", width), ("u", 2 * width), ("u", 3 * width), ("u", so)])
        qv, sv = q.download(np.int8, so * tokens).reshape(tokens, so), s.download(np.float32, so * tokens // 32).reshape(tokens, so // 32)
        check_q8p(qv[:, :width].ravel(), sv[:, :width // 32].ravel(), want, 1e-5)
        if so > width:
            assert not qv[:, width:].any(), "the padding is not written"


def test_the_seam_refuses_what_it_cannot_run(ctx):
    z = ctx.zeros(4096)
    with pytest.raises(tb.Error) as e:
        ctx.launch("gemm_q4", (1, 1, 1), (128, 1, 1), 0, [("p", z.ptr)] * 5 + [("u", 48), ("u", 128), ("u", 1)])  # rows not a multiple of 64
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.launch("gemm_q4", (1, 1, 9), (128, 1, 1), 0, [("p", z.ptr)] * 5 + [("u", 64), ("u", 128), ("u", 1)])  # nine slices
    with pytest.raises(tb.Error):
        ctx.launch("sum_slices", (1, 1, 1), (256, 1, 1), 0, [("p", z.ptr), ("u", 6), ("u", 2)])  # len not a multiple of 4
    with pytest.raises(tb.Error):
        ctx.launch("quant_q8p", (1, 1, 1), (128, 1, 1), 0, [("p", z.ptr)] * 3 + [("u", 64)])  # blocks of 256
