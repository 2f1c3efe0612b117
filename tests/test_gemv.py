"""Q8-weight GEMV on the GPU against the CPU oracle.  Mirrors crates/tachyon/tests/gemv.rs: every shape of a decode
projection plus ragged edge shapes, tolerance 1e-5 * (sum of term magnitudes) + 1e-6 on f32 results."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16, f16_to_f32, q8_weights

pytestmark = pytest.mark.gpu

# (rows, cols): staged kernel at 2048/4096/8192/16384 columns with whole and ragged row counts; the generic kernel for
# the reference's other column counts (tests/gemv.rs:16) and tiny shapes.
SHAPES = [(16384, 2048), (512, 2048), (37, 2048), (5, 2048), (1, 2048), (3072, 2048), (300, 4096), (64, 8192), (2048, 16384), (37, 16384),
          (512, 2560), (256, 10240), (5, 64), (3, 192), (2560, 256), (36, 64)]


def run(ctx, w, s, x, x_dtype, y_dtype):
    rows, cols = w.shape
    wd, sd = ctx.upload(w), ctx.upload(s)
    xd = ctx.upload(f16(x) if x_dtype == tb.F16 else x.astype(np.float32))
    yd = ctx.zeros(rows * 4)
    ctx.gemv_q8(wd, sd, xd, x_dtype, yd, y_dtype, rows, cols)
    return f16_to_f32(yd.download(np.uint16, rows)) if y_dtype == tb.F16 else yd.download(np.float32, rows)


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_gemv_matches_the_oracle_on_every_shape(ctx, rows, cols):
    w, s = q8_weights(rows, cols, 11 + rows + cols)
    x = np.random.default_rng(99 + rows).standard_normal(cols).astype(np.float32)
    xh = f16_to_f32(f16(x))  # the benchmark's activation is f16
    _, exact, bound = oracle.gemv_q8(w, s, xh)
    got = run(ctx, w, s, x, tb.F16, tb.F32)
    assert np.all(np.abs(got.astype(np.float64) - exact) <= 1e-5 * bound + 1e-6), f"{rows}x{cols}: {np.abs(got - exact).max()}"
    # f16 output: the f32 result rounded once
    got16 = run(ctx, w, s, x, tb.F16, tb.F16)
    assert np.all(np.abs(got16.astype(np.float64) - exact) <= 2.0**-10 * np.abs(exact) + 1e-5 * bound + 1e-6)
    # f32 activations take the same path
    got32 = run(ctx, w, s, x, tb.F32, tb.F32)
    _, exact32, bound32 = oracle.gemv_q8(w, s, x)
    assert np.all(np.abs(got32.astype(np.float64) - exact32) <= 1e-5 * bound32 + 1e-6)


def test_gemv_is_deterministic_and_handles_zero_and_tiny_blocks(ctx):
    rows, cols = 777, 2048
    w, s = q8_weights(rows, cols, 5)
    x = np.random.default_rng(6).standard_normal(cols).astype(np.float32)
    x[64:96] = 0.0
    x[100] = 1e-30
    x[200:232] *= 1e-6
    x[300] = 3000.0
    _, exact, bound = oracle.gemv_q8(w, s, x)
    a = run(ctx, w, s, x, tb.F32, tb.F32)
    b = run(ctx, w, s, x, tb.F32, tb.F32)
    assert np.array_equal(a, b)
    assert np.all(np.abs(a.astype(np.float64) - exact) <= 1e-5 * bound + 1e-6)


def test_gemv_is_linear_at_full_size(ctx):
    """A size-independent property at the benchmark's shape: W(x1 + x2) = W x1 + W x2 up to rounding."""
    rows, cols = 16384, 2048
    w, s = q8_weights(rows, cols, 1)
    rng = np.random.default_rng(2)
    x1, x2 = rng.standard_normal(cols).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
    y1, y2, y12 = (run(ctx, w, s, v, tb.F32, tb.F32) for v in (x1, x2, x1 + x2))
    scale = np.abs(y1).max() + np.abs(y2).max()
    assert np.abs(y12 - (y1 + y2)).max() <= 1e-5 * scale


def test_gemv_rejects_bad_descriptors(ctx):
    w, s = q8_weights(8, 64, 0)
    wd, sd, xd, yd = ctx.upload(w), ctx.upload(s), ctx.upload(np.zeros(64, np.float32)), ctx.zeros(64)
    with pytest.raises(tb.Error) as e:
        ctx.gemv_q8(wd, sd, xd, tb.F32, yd, tb.F32, 8, 48)  # cols not a multiple of 32
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.gemv_q8(wd, sd, xd, 7, yd, tb.F32, 8, 64)  # unknown dtype


def test_norm_prologue_and_geglu_epilogue(ctx):
    """norm_q8 + gemv + geglu_q8 in one launch, against the f64 restatement of crates/tachyon/tests/decode.rs:84-97."""
    rows, cols = 2 * 333, 2048
    w, s = q8_weights(rows, cols, 21)
    rng = np.random.default_rng(22)
    h = (20 * rng.uniform(-1, 1, cols)).astype(np.float32)
    y = (300 * rng.uniform(-1, 1, cols)).astype(np.float32)
    w1 = (1 + rng.uniform(-1, 1, cols)).astype(np.float32)
    w2 = (0.5 + rng.uniform(-1, 1, cols)).astype(np.float32)
    for yres, scale, geglu in [(y, 0.75, False), (None, 1.0, False), (y, 1.0, True)]:
        h_want, x_want = oracle.norm_step(h, yres, w1 if yres is not None else None, w2, 1e-6, scale)
        deq = w.astype(np.float64) * np.repeat(f16_to_f32(s).astype(np.float64), 32, axis=1)
        full = deq @ x_want
        bound = np.abs(deq) @ np.abs(x_want)
        bufs = [ctx.upload(a) for a in (w, s, h, y, w1, w2)]
        hout, yout = ctx.zeros(cols * 4), ctx.zeros(rows * 4)
        ctx.gemv_q8_norm(bufs[0], bufs[1], bufs[2], bufs[3] if yres is not None else None, bufs[4] if yres is not None else None, bufs[5], 1e-6, scale,
                         hout, yout, rows, cols, geglu)
        got_h = hout.download(np.float32, cols)
        assert np.all(np.abs(got_h - h_want) <= 1e-5 * np.maximum(np.abs(h_want), 1.0))
        if geglu:
            # the device stores pairs (gate_j, up_j) on adjacent rows
            gate, up = full[0::2], full[1::2]
            want = np.array([oracle.lib().tbo_gelu_tanh(float(a)) for a in gate]) * up
            got = yout.download(np.float32, rows // 2)
            tol = 1e-4 * (np.abs(want) + bound[0::2] * 1e-1 + bound[1::2] * 1e-1) + 1e-5
            assert np.all(np.abs(got - want) <= tol), np.abs(got - want).max()
        else:
            got = yout.download(np.float32, rows)
            assert np.all(np.abs(got - full) <= 2e-5 * bound + 1e-5), np.abs(got - full).max()


def test_argmax_epilogue_picks_the_lowest_index_of_the_largest(ctx):
    rows, cols = 4000, 2048
    w, s = q8_weights(rows, cols, 31)
    w[3000] = w[17]  # two equal rows: the pick must be the lower index when they win
    s[3000] = s[17]
    x = np.random.default_rng(32).standard_normal(cols).astype(np.float32)
    _, exact, bound = oracle.gemv_q8(w, s, x)
    wd, sd, xd = ctx.upload(w), ctx.upload(s), ctx.upload(x)
    logits, scratch, state, out = ctx.zeros(rows * 4), ctx.zeros(16), ctx.zeros(8), ctx.zeros(4)
    for step in (1, 2):  # twice: the scratch must return to zero
        ctx.gemv_q8_argmax(wd, sd, xd, tb.F32, logits, rows, cols, scratch, state, out)
        got = logits.download(np.float32, rows)
        assert np.all(np.abs(got - exact) <= 1e-5 * bound + 1e-6)
        want = int(np.flatnonzero(got == got.max())[0])
        st = state.download(np.uint32, 2)
        assert (int(st[0]), int(st[1])) == (step, want)
        assert int(out.download(np.uint32, 1)[0]) == want
        assert not scratch.download(np.uint32, 4).any()
    # force the tie to win
    boost = x.copy()
    wd2 = w.copy()
    wd2[17] = np.sign(x).astype(np.int8) * 127
    wd2[3000] = wd2[17]
    s2 = s.copy()
    s2[17] = s2[3000] = f16(np.full(cols // 32, 0.01, np.float32))
    ctx.gemv_q8_argmax(ctx.upload(wd2), ctx.upload(s2), xd, tb.F32, None, rows, cols, scratch, state, None)
    assert int(state.download(np.uint32, 2)[1]) == 17


@pytest.mark.parametrize("rows", [2048, 3072, 4736, 100, 17, 1])
def test_the_small_kernel_gives_the_staged_kernels_bits(ctx, rows):
    """tb_context_set_lean(2): products of 2048 columns and few rows a block go through the small-footprint kernel (weights
    straight into registers, no ring).  Same block arithmetic, same order: the same bits with the plain f32 input; with
    the residual/norm prologue the same up to the order of the prologue's sums."""
    cols = 2048
    w, s = q8_weights(rows, cols, 41 + rows)
    rng = np.random.default_rng(rows)
    x = rng.standard_normal(cols).astype(np.float32)
    h, y, w1, w2 = (rng.uniform(-2, 2, cols).astype(np.float32) for _ in range(4))
    outs = []
    for mode in (0, 2):
        ctx.set_lean(mode)
        try:
            plain = run(ctx, w, s, x, tb.F32, tb.F32)
            bufs = [ctx.upload(a) for a in (w, s, h, y, w1, w2)]
            hout, yout = ctx.zeros(cols * 4), ctx.zeros(rows * 4)
            ctx.gemv_q8_norm(bufs[0], bufs[1], bufs[2], bufs[3], bufs[4], bufs[5], 1e-6, 0.75, hout, yout, rows, cols, False)
            hout2, yout2 = ctx.zeros(cols * 4), ctx.zeros(rows * 4)
            ctx.gemv_q8_norm(bufs[0], bufs[1], bufs[2], None, None, None, 1e-6, 1.0, hout2, yout2, rows, cols, False)
            outs.append((plain, yout.download(np.float32, rows), hout.download(np.float32, cols), yout2.download(np.float32, rows)))
        finally:
            ctx.set_lean(1)
    assert np.array_equal(outs[0][0], outs[1][0])
    # with the norm prologue the four sums meet in another order (8 warps of 2 x 4 values, 16 warps of 4): the last bit may differ
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert np.all(np.abs(a - b) <= 2e-6 * np.abs(a).max())
    _, exact, bound = oracle.gemv_q8(w, s, x)
    assert np.all(np.abs(outs[1][0].astype(np.float64) - exact) <= 1e-5 * bound + 1e-6)
    assert ctx.status() == 0


@pytest.mark.parametrize("rows,cols", [(32768, 2048), (2048, 16384), (9999, 2048), (40000, 4096)])
def test_stages_handed_out_by_a_counter_give_the_same_bits(ctx, rows, cols):
    """Large products give their stages of rows to whichever block is free (a counter in device memory); small ones split
    the rows evenly.  Which block computes a row does not change the row: same bits, launch after launch, and the
    counters return to zero (the second launch would otherwise skip rows)."""
    w, s = q8_weights(rows, cols, 51)
    x = np.random.default_rng(52).standard_normal(cols).astype(np.float32)
    ctx.set_dynamic(False)
    try:
        static = run(ctx, w, s, x, tb.F32, tb.F32)
    finally:
        ctx.set_dynamic(True)
    wd, sd, xd, yd = ctx.upload(w), ctx.upload(s), ctx.upload(x), ctx.zeros(rows * 4)
    for _ in range(70):  # more launches than the context has counter pairs
        ctx.gemv_q8(wd, sd, xd, tb.F32, yd, tb.F32, rows, cols)
    assert np.array_equal(yd.download(np.float32, rows), static)
    _, exact, bound = oracle.gemv_q8(w, s, x)
    assert np.all(np.abs(static.astype(np.float64) - exact) <= 1e-5 * bound + 1e-6)
    assert ctx.status() == 0


# ---- f16 weights -------------------------------------------------------------------------------------------------------

F16_SHAPES = [(16384, 2048), (512, 2048), (37, 2048), (5, 2048), (1, 2048), (3072, 2048), (300, 4096), (64, 8192), (2048, 16384), (37, 16384), (512, 2560),
              (256, 10240), (2560, 256), (36, 768)]


@pytest.mark.parametrize("rows,cols", F16_SHAPES)
def test_gemv_f16_matches_the_oracle_on_every_shape(ctx, rows, cols):
    """tb_gemv_f16 on the shapes of tests/gemv.rs:16 (whole and ragged row counts, the benchmark's 16384 x 2048) against the
    f64 product: 1e-5 of the terms' magnitudes for f32 accumulation (tests/gemv.rs:61-67), plus an f16 rounding for f16 out."""
    rng = np.random.default_rng(rows + cols)
    w = f16(rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.02))
    x = rng.standard_normal(cols).astype(np.float32)
    wd, y = ctx.upload(w), ctx.zeros((rows + 2) * 4)
    for x_dtype, xv in ((tb.F32, x), (tb.F16, f16_to_f32(f16(x)))):
        want, bound = oracle.gemv_f16(w, xv)
        xd = ctx.upload(f16(x) if x_dtype == tb.F16 else x)
        y.upload(np.full(rows + 2, 777.0, np.float32))
        ctx.gemv_f16(wd, xd, x_dtype, y, tb.F32, rows, cols)
        got = y.download(np.float32, rows + 2)
        assert np.all(got[rows:] == 777.0), "rows past the matrix were written"
        assert np.all(np.abs(got[:rows] - want) <= 1e-5 * bound + 1e-6), float(np.abs(got[:rows] - want).max())
        ctx.gemv_f16(wd, xd, x_dtype, y, tb.F16, rows, cols)
        got16 = f16_to_f32(y.download(np.uint16, rows))
        assert np.all(np.abs(got16 - want) <= 2.0**-10 * np.abs(want) + 1e-5 * bound + 1e-6)
    assert ctx.status() == 0


def test_gemv_f16_with_the_norm_prologue(ctx):
    rows, cols = 333, 2048
    rng = np.random.default_rng(3)
    w = f16(rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.02))
    h, y, w1, w2 = (20 * rng.uniform(-1, 1, cols)).astype(np.float32), (300 * rng.uniform(-1, 1, cols)).astype(np.float32), (1 + rng.uniform(-1, 1, cols)).astype(
        np.float32), (0.5 + rng.uniform(-1, 1, cols)).astype(np.float32)
    bufs = [ctx.upload(a) for a in (w, h, y, w1, w2)]
    for yres, scale in ((y, 0.75), (None, 1.0)):
        h_want, x_want = oracle.norm_step(h, yres, w1 if yres is not None else None, w2, 1e-6, scale)
        wf = w.view(np.float16).astype(np.float64)
        want, bound = wf @ x_want, np.abs(wf) @ np.abs(x_want)
        hout, yout = ctx.zeros(cols * 4), ctx.zeros(rows * 4)
        ctx.gemv_f16_norm(bufs[0], bufs[1], bufs[2] if yres is not None else None, bufs[3] if yres is not None else None, bufs[4], 1e-6, scale, hout, yout, tb.F32,
                          rows, cols)
        assert np.all(np.abs(hout.download(np.float32, cols) - h_want) <= 1e-5 * np.maximum(np.abs(h_want), 1.0))
        got = yout.download(np.float32, rows)
        assert np.all(np.abs(got - want) <= 2e-5 * bound + 1e-5), float(np.abs(got - want).max())


def test_gemv_f16_rejects_bad_descriptors(ctx):
    z = ctx.zeros(4096)
    with pytest.raises(tb.Error) as e:
        ctx.gemv_f16(z, z, tb.F32, z, tb.F32, 4, 100)  # cols not a multiple of 256
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.gemv_f16(z, z, tb.F32, z, tb.F32, 4, 32768)  # wider than the kernel's shared-memory vector


def test_a_wait_that_runs_out_comes_back_as_a_status():
    """Every device-side wait has a limit.  tb_selftest_wait makes one run out (a block whose producer copies nothing, a limit
    of a millisecond): the kernel returns, the context's status word reads 1 (a wait for a full stage), tb_status says
    TB_DEVICE_WAIT, and after tb_status_clear the same context computes as before.  A context of its own, so the session's
    stays clean."""
    import ctypes as C
    import time

    c = tb.Context(0)
    t0 = time.perf_counter()
    tb.check(c.lib.tb_selftest_wait(c.handle, 1_000_000))
    assert time.perf_counter() - t0 < 1.0
    word = C.c_uint32(0)
    assert c.lib.tb_status(c.handle, C.byref(word)) == 10 and word.value == 1
    assert "bounded wait" in c.lib.tb_last_error().decode()
    tb.check(c.lib.tb_status_clear(c.handle))
    assert c.status() == 0
    rows, cols = 64, 2048
    w, s = q8_weights(rows, cols, 3)
    x = np.random.default_rng(4).standard_normal(cols).astype(np.float32)
    got = run(c, w, s, x, tb.F32, tb.F32)
    _, exact, bound = oracle.gemv_q8(w, s, x)
    assert np.all(np.abs(got.astype(np.float64) - exact) <= 1e-5 * bound + 1e-6)
    assert c.status() == 0
    with pytest.raises(tb.Error):
        tb.check(c.lib.tb_selftest_wait(c.handle, 0))
    c.close()
