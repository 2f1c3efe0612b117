"""The reference's own decode formats: Q8 activation quantisation and the Q4 x Q8 matrix-vector product.

Mirrors crates/tachyon/tests/gemv.rs: `quant_q8_matches_the_cpu_exactly` and `gemv_matches_the_reference_on_every_shape`
(same seeded values, same shapes, same bound `1e-5 * bound + 1e-6` against the f64 product of tests/common/mod.rs:95-112),
plus what this build can add: the oracle repeats the reference kernel's f32 operations in the kernel's order, and the GPU
must give the oracle's bits."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import values, values_fast

# crates/tachyon/tests/gemv.rs:16 and the decode projections of the benchmark's model (staged path: 2048, 4096, 16384 wide).
SHAPES = [(512, 2560), (512, 2048), (512, 4096), (256, 10240), (37, 2560), (5, 64), (3, 192), (2560, 256), (36, 64),
          (3072, 2048), (37, 2048), (1, 2048), (300, 512), (96, 1024), (64, 8192), (2048, 16384), (37, 16384)]


def inputs(rows, cols, i):
    gen = values if rows * cols <= 1 << 16 else values_fast  # the reference's xorshift generator is a Python loop here
    return gen(rows * cols, 11 + i), gen(cols, 99 + i)


@pytest.mark.parametrize("i,shape", list(enumerate(SHAPES[:9] + [(64, 2048), (8, 16384)])))
def test_oracle_kernel_order_meets_the_reference_bound(i, shape):
    """CPU only: the kernel-order restatement stays within the reference test's bound of the f64 product."""
    rows, cols = shape
    wf, x = inputs(rows, cols, i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    q, pairs = oracle.q8(x)
    y = oracle.gemv_q4(packed, scales, q, pairs, rows)
    want, bound = oracle.product_q4(packed, scales, x, rows)
    assert np.all(np.abs(y.astype(np.float64) - want) <= 1e-5 * bound + 1e-6)


@pytest.mark.gpu
def test_quant_q8_matches_the_cpu_exactly(ctx):
    x = values(4096, 7)
    x[64:96] = 0.0
    x[100] = 1e-30
    xd, qd, sd = ctx.upload(x), ctx.zeros(x.size), ctx.zeros(x.size // 32 * 8)
    ctx.quant_q8(xd, x.size, qd, sd)
    cq, cs = oracle.q8(x)
    assert np.array_equal(qd.download(np.int8, x.size), cq), "Q8 values differ"
    assert np.array_equal(sd.download(np.float32, x.size // 16).view(np.uint32), cs.ravel().view(np.uint32)), "Q8 scales differ"


def gpu_gemv(ctx, packed, scales, x, rows):
    cols = x.size
    xd, qd, sd = ctx.upload(x), ctx.zeros(cols), ctx.zeros(cols // 32 * 8)
    ctx.quant_q8(xd, cols, qd, sd)
    wd, wsd, yd = ctx.upload(packed), ctx.upload(scales), ctx.zeros(rows * 4)
    ctx.gemv_q4(wd, wsd, qd, sd, yd, rows, cols)
    return yd.download(np.float32, rows)


@pytest.mark.gpu
@pytest.mark.parametrize("i,shape", list(enumerate(SHAPES)))
def test_gemv_q4_gives_the_reference_kernels_bits_on_every_shape(ctx, i, shape):
    rows, cols = shape
    wf, x = inputs(rows, cols, i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    got = gpu_gemv(ctx, packed, scales, x, rows)
    q, pairs = oracle.q8(x)
    assert np.array_equal(got.view(np.uint32), oracle.gemv_q4(packed, scales, q, pairs, rows).view(np.uint32)), f"{rows}x{cols}"
    want, bound = oracle.product_q4(packed, scales, x, rows)
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * bound + 1e-6)


@pytest.mark.gpu
def test_gemv_q4_stays_close_to_the_unquantized_product(ctx):
    rows, cols = 512, 2560
    wf, x = values_fast(rows * cols, 3), values_fast(cols, 4)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    y = gpu_gemv(ctx, packed, scales, x, rows).astype(np.float64)
    exact = wf.reshape(rows, cols).astype(np.float64) @ x.astype(np.float64)
    assert np.linalg.norm(y - exact) / np.linalg.norm(exact) < 0.15


@pytest.mark.gpu
def test_gemv_q4_rejects_what_it_cannot_run(ctx):
    d = ctx.zeros(4096)
    with pytest.raises(tb.Error):
        ctx.gemv_q4(d, d, d, d, d, 4, 96)  # not whole groups of 64
    with pytest.raises(tb.Error):
        ctx.quant_q8(d, 48, d, d)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(3072, 2048), (37, 2048), (1, 2048), (300, 4096), (64, 8192), (2048, 16384), (37, 16384)])
def test_gemv_q4x_reads_q4_weights_with_an_unrounded_activation(ctx, rows, cols):
    """The decode product on the reference's converted weights: f32 accuracy against the f64 product."""
    wf, x = values_fast(rows * cols, 21 + rows), np.random.default_rng(cols + rows).standard_normal(cols).astype(np.float32)
    x[64:96] = 0.0
    x[100] = 1e-30
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    want, bound = oracle.gemv_q4x(packed, scales, x, rows)
    wd, sd, xd, yd = ctx.upload(packed), ctx.upload(scales), ctx.upload(x), ctx.zeros(rows * 4)
    ctx.gemv_q4x(wd, sd, xd, tb.F32, yd, rows, cols)
    got = yd.download(np.float32, rows)
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * bound + 1e-6), np.abs(got - want).max()
