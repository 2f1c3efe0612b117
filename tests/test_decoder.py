"""The whole decode step on the GPU against the CPU forward pass (crates/tachyon/tests/model.rs:120-164): logits within
tolerance, greedy tokens identical wherever the top-2 gap exceeds it, queued generation equal to single steps."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from oracle.model import OracleModel

pytestmark = pytest.mark.gpu

SEED = 1234


def small_config(layers=3, ffn=2048, vocab=4096, window=16):
    c = tb.gemma4_e4b_shape(layers=layers, ffn=ffn, vocab=vocab)
    c.window, c.global_every = window, 3
    return c


def check_logits(got, want, gap, got_token, want_token):
    scale = np.abs(want).max()
    err = np.abs(got - want).max()
    assert err <= 2e-3 * scale, (err, scale)
    if gap > 4e-3 * scale:  # bit-exact pick once the top-2 gap clears the tolerance
        assert got_token == want_token


@pytest.fixture(scope="module")
def models(ctx):
    cfg = small_config()
    dec = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True)
    dec.fill_random(SEED)
    dec.build()
    ref = OracleModel(cfg, SEED, context=64, chunk=8)
    yield cfg, dec, ref
    dec.close()


def test_steps_match_the_cpu_forward_through_a_ring_wrap(models):
    cfg, dec, ref = models
    dec.reset()
    token = 17
    for pos in range(40):  # window 16, ring 24: wraps; layer 2 is global
        want_token, want_logits, want_hidden = ref.step(token, pos)
        got_token = dec.step(token)
        got_logits = dec.logits()
        capped = cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap)
        order = np.sort(capped)
        check_logits(got_logits, want_logits, order[-1] - order[-2], got_token, want_token)
        hid = dec.hidden()
        assert np.abs(hid - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
        assert dec.position == pos + 1
        token = (pos * 7919 + 13) % cfg.vocab  # a varied prompt: a tied random model would otherwise repeat itself


def test_loaded_tensors_equal_the_device_fill(ctx, models):
    cfg, dec, ref = models
    other = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True)
    for name, a in ref.tensors.items():
        other.load(name, a)
    other.build()
    dec.reset()
    for pos, token in enumerate([5, 99, 4000, 7]):
        assert other.step(token) == dec.step(token)
        assert np.array_equal(other.logits(), dec.logits()), "same bits from uploaded and generated weights"
    with pytest.raises(tb.Error) as e:
        other.load("3.qkv.w", np.zeros(4, np.int8))
    assert e.value.status == 8  # no such tensor
    with pytest.raises(tb.Error) as e:
        other.load("0.qkv.w", np.zeros(4, np.int8))
    assert e.value.status == 5  # wrong size
    other.close()


def test_queued_generation_equals_single_steps(models):
    cfg, dec, ref = models
    dec.reset()
    single = []
    token = 3
    for _ in range(12):
        token = dec.step(token)
        single.append(token)
    dec.reset()
    dec.start(3)
    queued = [dec.next_token() for _ in range(12)]
    dec.stop()
    assert queued == single
    dec.reset()
    chained = dec.run(3, 12)
    assert list(chained) == single
    # the decoder refuses to pass its context
    dec.reset()
    with pytest.raises(tb.Error) as e:
        dec.run(3, 65)
    assert e.value.status == 6


def test_prefill_then_decode_matches_stepping(models):
    """Chunked tensor-core prefill (f16 GEMM inputs) against the token-by-token decode path (crates/tachyon/tests/
    model.rs:173-195: within tolerance of the reference, and independent of how the prompt is cut)."""
    cfg, dec, ref = models
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(30)]  # longer than the window (16) and the ring (24)
    dec.reset()
    for t in prompt[:-1]:
        dec.step(t)
    a = dec.step(prompt[-1])
    la = dec.logits()
    dec.reset()
    dec.prefill(prompt[:-1])
    assert dec.position == len(prompt) - 1
    b = dec.step(prompt[-1])
    lb = dec.logits()
    scale = np.abs(la).max()
    assert np.abs(la - lb).max() <= 1e-2 * scale, float(np.abs(la - lb).max() / scale)
    top = np.sort(la)
    if top[-1] - top[-2] > 2e-2 * scale:
        assert a == b
    # and against the CPU forward
    want = None
    for pos, t in enumerate(prompt):
        _, want, _ = ref.step(t, pos)
    assert np.abs(lb - want).max() <= 1e-2 * np.abs(want).max()


def test_prefill_does_not_depend_on_the_chunking(ctx, models):
    cfg, dec, ref = models
    prompt = [(i * 104729 + 7) % cfg.vocab for i in range(45)]
    outs = []
    for chunk in (8, 32):
        d = tb.Decoder(ctx, cfg, context=64, chunk=chunk, keep_logits=True)
        d.fill_random(SEED)
        d.build()
        d.prefill(prompt[:-1])
        tok = d.step(prompt[-1])
        outs.append((tok, d.logits()))
        d.close()
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]), "chunks of 8 and of 32 must give the same bits"


@pytest.mark.parametrize("bits", [8, 4])
def test_prefill_on_the_f16_copy_of_the_weights_gives_the_same_bits(ctx, bits):
    """tb_settings.prefill_copy: products on 256 tokens and more read an f16 copy of the matrices by TMA; the copy holds the
    values the converting products build, so nothing changes but the speed.  A tensor loaded after the build reaches the copy."""
    cfg = small_config(layers=3, ffn=2048, vocab=2048, window=128)
    prompt = [(i * 104729 + 7) % cfg.vocab for i in range(700)]
    outs = []
    for copy in (1, 2):
        d = tb.Decoder(ctx, cfg, context=1024, chunk=512, keep_logits=True, weight_bits=bits, prefill_copy=copy)
        d.fill_random(SEED)
        d.build()
        if bits == 8:  # after the build: the copy has to follow
            d.load("1.input_layernorm", np.full(cfg.hidden, 1.25, np.float32))
            w = np.random.default_rng(3).integers(-127, 128, size=(cfg.hidden, cfg.ffn), dtype=np.int8)
            d.load("1.down.w", w)
        d.prefill(prompt[:-1])
        tok = d.step(prompt[-1])
        outs.append((tok, d.logits()))
        d.close()
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1])


def test_overlap_off_gives_the_same_bits(ctx, models):
    """Programmatic dependent launch only changes when kernels start, never what they compute."""
    cfg, dec, ref = models
    dec.reset()
    want = list(dec.run(9, 10))
    ctx.set_overlap(False)
    try:
        plain = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=False)
        plain.fill_random(SEED)
        plain.build()
        assert list(plain.run(9, 10)) == want
        plain.close()
    finally:
        ctx.set_overlap(True)


def test_the_attention_half_of_a_layer_as_one_kernel(ctx, models):
    """tb_context_set_attn_block: norm, q/k/v product, attention and output projection of a layer in one kernel on two clusters of
    16 blocks (attn_block.cu).  The same arithmetic up to the order of the sums (the output projection comes as two partial
    products, the window is cut into 16 runs), so it is held to the three launches, which the tests above hold to the CPU
    forward: through a ring wrap, and behind a chunked prefill."""
    cfg, dec, ref = models
    ctx.set_attn_block(True)
    try:
        one = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True)
        one.fill_random(SEED)
        one.build()
    finally:
        ctx.set_attn_block(False)
    if one.step_launches != 2 + 3 * cfg.layers:
        one.close()
        pytest.skip("this GPU does not give the kernel its two clusters of 16 blocks")
    assert dec.step_launches == 2 + 5 * cfg.layers
    dec.reset()
    for pos in range(40):
        token = (pos * 7919 + 13) % cfg.vocab
        assert one.step(token) == dec.step(token)
        a, b = one.logits(), dec.logits()
        assert np.abs(a - b).max() <= 1e-4 * np.abs(b).max()
    # a prompt through prefill, then steps: the caches the chunked path wrote are the ones this kernel reads
    prompt = [(i * 104729 + 7) % cfg.vocab for i in range(21)]
    outs = []
    for d in (one, dec):
        d.reset()
        d.prefill(prompt[:-1])
        t = d.step(prompt[-1])
        seq = [t]
        for _ in range(5):
            seq.append(d.step(seq[-1]))
        outs.append((seq, d.logits()))
    assert outs[0][0] == outs[1][0] and np.abs(outs[0][1] - outs[1][1]).max() <= 1e-4 * np.abs(outs[1][1]).max()
    one.close()


def test_fused_step_equals_one_launch_per_phase(ctx, models):
    """The persistent step kernel runs the same arithmetic as the 2 + 5*layers separate kernels."""
    cfg, dec, ref = models
    assert dec.step_launches == 2 + 5 * cfg.layers
    plain = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True, fused=True)
    plain.fill_random(SEED)
    plain.build()
    assert plain.step_launches == 1
    dec.reset()
    for pos in range(40):  # through the ring's wrap
        token = (pos * 7919 + 13) % cfg.vocab
        assert dec.step(token) == plain.step(token)
        a, b = dec.logits(), plain.logits()
        assert np.abs(a - b).max() <= 1e-4 * np.abs(b).max()  # the splits are merged in a different order
    # Decoder::timeline: four stamps per phase for the first and the last block, in order
    stamps = plain.timeline(7).astype(np.int64)
    assert stamps.shape == (2, 2 + 5 * cfg.layers, 4)
    starts = stamps[0, :, 0]
    assert np.all(np.diff(starts) > 0) and np.all(stamps[0, :, 2] >= starts)
    plain.close()


@pytest.mark.parametrize("fused", [False, True])
def test_benchmark_width_ffn_and_a_prefilled_cache(ctx, fused):
    """One layer at the benchmark's FFN width (down projection over 16384 columns) on a synthetic 100-position cache."""
    cfg = small_config(layers=2, ffn=16384, vocab=2048, window=512)
    cfg.global_every = 2
    dec = tb.Decoder(ctx, cfg, context=256, chunk=0, keep_logits=True, fused=fused)
    dec.fill_random(77)
    dec.build()
    dec.fill_cache(5, 100)
    ref = OracleModel(cfg, 77, context=256, chunk=0)
    ref.fill_cache(5)
    token = 1000
    for pos in range(100, 104):
        want_token, want_logits, _ = ref.step(token, pos)
        got = dec.step(token)
        capped = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
        check_logits(dec.logits(), want_logits, capped[-1] - capped[-2], got, want_token)
        token = want_token
    w, kv = dec.step_bytes()
    assert w == sum(t.nbytes for n, t in ref.tensors.items() if n.endswith((".w", ".s")))
    dec.close()


def test_prefill_at_the_benchmark_width(ctx):
    """Prefill GEMMs at FFN 16384 (K = 16384 in the down projection), a ragged chunk, against the CPU forward."""
    cfg = small_config(layers=2, ffn=16384, vocab=2048, window=32)
    cfg.global_every = 2
    dec = tb.Decoder(ctx, cfg, context=128, chunk=48, keep_logits=True)
    dec.fill_random(91)
    dec.build()
    ref = OracleModel(cfg, 91, context=128, chunk=48)
    prompt = [(i * 31 + 5) % cfg.vocab for i in range(70)]
    dec.prefill(prompt[:-1])
    got_token = dec.step(prompt[-1])
    for pos, t in enumerate(prompt):
        want_token, want, _ = ref.step(t, pos)
    got = dec.logits()
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-2 * scale, float(np.abs(got - want).max() / scale)
    top = np.sort(want)
    if top[-1] - top[-2] > 2e-2 * scale:
        assert got_token == want_token
    dec.close()


def test_q4_weights_step_matches_the_cpu_forward_and_loads_converted_tensors(ctx):
    """TB_WEIGHTS_Q4: the reference's converted matrices (u8 [rows, cols/2] nibbles, f16 [rows, cols/64] scales) as
    they come out of weights.wpk; the same checks as for eight-bit weights, and a prompt through tb_decoder_prefill."""
    cfg = small_config()
    dec = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True, weight_bits=4)
    dec.fill_random(SEED + 4)
    dec.build()
    ref = OracleModel(cfg, SEED + 4, context=64, chunk=8, weight_bits=4)
    token = 17
    for pos in range(28):
        want_token, want_logits, want_hidden = ref.step(token, pos)
        got_token = dec.step(token)
        capped = cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap)
        order = np.sort(capped)
        check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
        assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
        token = (pos * 7919 + 13) % cfg.vocab
    # the same tensors uploaded by name give the same bits as the device fill
    other = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True, weight_bits=4)
    for name, a in ref.tensors.items():
        other.load(name, a)
    other.build()
    dec.reset()
    for token in [5, 99, 4000, 7]:
        assert other.step(token) == dec.step(token)
        assert np.array_equal(other.logits(), dec.logits())
    with pytest.raises(tb.Error) as e:
        other.load("0.qkv.w", np.zeros(3072 * 2048, np.int8))  # the eight-bit size
    assert e.value.status == 5
    # a prompt through the chunked tensor-core prefill (nibbles dequantised in the operand path) against stepping
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(30)]
    dec.reset()
    for t in prompt[:-1]:
        dec.step(t)
    a, la = dec.step(prompt[-1]), dec.logits()
    dec.reset()
    dec.prefill(prompt[:-1])
    b, lb = dec.step(prompt[-1]), dec.logits()
    scale = np.abs(la).max()
    assert np.abs(la - lb).max() <= 4e-3 * scale
    order = np.sort(cfg.softcap * np.tanh(la.astype(np.float64) / cfg.softcap))
    if order[-1] - order[-2] > 8e-3 * scale:
        assert a == b
    with pytest.raises(tb.Error):
        tb.Decoder(ctx, cfg, context=64, fused=True, weight_bits=4)
    dec.close(), other.close()


def test_decoder_draws_with_the_reference_sampler(models):
    """tb_decoder_set_sampling: the step ends in logits + the sampler kernel; its draws are the oracle's for the step's own
    logits, position by position, and the plain setting goes back to the fused pick."""
    cfg, dec, ref = models
    dec.reset()
    dec.set_sampling()
    greedy = [int(t) for t in dec.run(3, 6)]
    dec.reset()
    dec.set_sampling(temperature=6.0, top_k=40, top_p=0.95, penalty=1.2, softcap=cfg.softcap, seed=77)
    token, seen, drawn = 3, np.zeros(cfg.vocab // 32, np.uint32), []
    s = oracle.sampling(softcap=cfg.softcap, temperature=6.0, top_p=0.95, penalty=1.2, top_k=40, seed=77)
    misses = 0
    for pos in range(16):
        got = dec.step(token)
        want, _ = oracle.sample_draw(dec.logits(), s, pos, seen)
        misses += int(got != want)
        seen[got // 32] |= np.uint32(1 << (got % 32))  # the kernel marks what it generated
        drawn.append(got)
        token = got
    assert misses <= 1, (misses, drawn)  # the GPU's approximate exp/log differ from libm in the last bits only
    assert len(set(drawn)) > 3 and drawn[:6] != greedy
    # chained generation under the same settings reproduces the single steps
    dec.reset()
    chained = [int(t) for t in dec.run(3, 16)]
    assert chained == drawn
    dec.set_sampling()
    dec.reset()
    assert [int(t) for t in dec.run(3, 6)] == greedy


def test_shared_key_value_layers_attend_over_their_source_layers_cache(ctx):
    """Config::shared (model/mod.rs:64, 138-143): the last layers have query rows only and read the cache of the last
    earlier layer of their kind; stepping, the chunked prefill and the Q4 format all follow the CPU forward."""
    cfg = small_config(layers=6)
    cfg.global_every, cfg.shared = 3, 3  # layers 3, 4 (sliding) share layer 1's cache, layer 5 (global) layer 2's
    for bits in (8, 4):
        dec = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True, weight_bits=bits)
        dec.fill_random(SEED + bits)
        dec.build()
        ref = OracleModel(cfg, SEED + bits, context=64, chunk=8, weight_bits=bits)
        assert ref.tensors["4.qkv.w"].shape[0] == cfg.heads * cfg.head_dim and ref.tensors["1.qkv.w"].shape[0] == (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim
        token = 17
        for pos in range(30):
            want_token, want_logits, want_hidden = ref.step(token, pos)
            got_token = dec.step(token)
            order = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
            check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
            assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
            token = (pos * 7919 + 13) % cfg.vocab
        prompt = [(i * 7919 + 13) % cfg.vocab for i in range(30)]
        dec.reset()
        for t in prompt[:-1]:
            dec.step(t)
        a, la = dec.step(prompt[-1]), dec.logits()
        dec.reset()
        dec.prefill(prompt[:-1])
        b, lb = dec.step(prompt[-1]), dec.logits()
        scale = np.abs(la).max()
        assert np.abs(la - lb).max() <= 4e-3 * scale
        dec.close()
    with pytest.raises(tb.Error):
        bad = small_config(layers=3)
        bad.shared = 3
        tb.Decoder(ctx, bad, context=64)


@pytest.mark.parametrize("kv,global_dim,global_kv", [(2, 512, 0), (2, 512, 1), (1, 0, 0), (1, 512, 2)])
def test_global_layers_with_heads_of_512(ctx, kv, global_dim, global_kv):
    """Config::head_dim = [256, 512] and Config::kv_heads = [2, 1] (model/mod.rs:34-37, Gemma 4's global layers): wider
    query/key/value and output matrices, a cache of heads of 512, RoPE over a quarter of the head; and eight query heads
    to a key-value head in either kind of layer (E2B).  Stepping, the chunked prefill, the Q4 format and a shared global
    layer follow the CPU forward."""
    cfg = small_config(layers=6)
    cfg.kv_heads = kv
    cfg.global_every, cfg.global_head_dim, cfg.global_kv_heads, cfg.shared = 3, global_dim, global_kv, 2  # layer 5 (global) shares layer 2's cache
    gd = global_dim or 256
    for bits in (8, 4):
        dec = tb.Decoder(ctx, cfg, context=96, chunk=40, keep_logits=True, weight_bits=bits)
        dec.fill_random(SEED + bits)
        dec.build()
        ref = OracleModel(cfg, SEED + bits, context=96, chunk=40, weight_bits=bits)
        kvg = global_kv or cfg.kv_heads
        assert ref.tensors["2.qkv.w"].shape[0] == (cfg.heads + 2 * kvg) * gd and ref.tensors["5.qkv.w"].shape[0] == cfg.heads * gd
        assert ref.tensors["2.q_norm"].size == gd and ref.tensors["1.q_norm"].size == 256
        token = 17
        for pos in range(40):
            want_token, want_logits, want_hidden = ref.step(token, pos)
            got_token = dec.step(token)
            order = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
            check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
            assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
            token = (pos * 7919 + 13) % cfg.vocab
        prompt = [(i * 7919 + 13) % cfg.vocab for i in range(70)]
        dec.reset()
        for t in prompt[:-1]:
            dec.step(t)
        a, la = dec.step(prompt[-1]), dec.logits()
        dec.reset()
        dec.prefill(prompt[:-1])  # two chunks: 40 tokens, then 29
        b, lb = dec.step(prompt[-1]), dec.logits()
        assert np.abs(la - lb).max() <= 4e-3 * np.abs(la).max()
        dec.close()
    with pytest.raises(tb.Error) as e:
        bad = small_config(layers=3)
        bad.global_head_dim = 128
        tb.Decoder(ctx, bad, context=64)
    assert e.value.status == 9


def test_per_layer_inputs(ctx):
    """Config::per_layer (model/mod.rs:38-39; decode.rs:572-579, 650-660): every layer adds a gated projection of its own
    input, built from the token's row of a second table and a projection of the embedding.  Stepping and the chunked
    prefill follow the CPU forward (tests/common/tiny.rs:239-252, 298-301), also with heads of 512 and a shared layer."""
    cfg = small_config(layers=5)
    cfg.per_layer, cfg.global_every, cfg.global_head_dim, cfg.shared = 256, 3, 512, 1
    dec = tb.Decoder(ctx, cfg, context=96, chunk=40, keep_logits=True)
    dec.fill_random(SEED)
    dec.build()
    ref = OracleModel(cfg, SEED, context=96, chunk=40)
    assert ref.tensors["embed_per_layer.w"].shape == (cfg.vocab, 5 * 256) and ref.tensors["3.per_layer_proj.w"].shape == (cfg.hidden, 256)
    token = 17
    for pos in range(30):
        want_token, want_logits, want_hidden = ref.step(token, pos)
        got_token = dec.step(token)
        order = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
        check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
        assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
        token = (pos * 7919 + 13) % cfg.vocab
    # the inputs matter: without them the same weights give another hidden state
    plain = small_config(layers=5)
    plain.global_every, plain.global_head_dim, plain.shared = 3, 512, 1
    other = OracleModel(plain, SEED, context=96, chunk=40)
    assert np.abs(other.step(17, 0)[2] - ref.step(17, 0)[2]).max() > 0.05 * np.abs(want_hidden).max()
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(70)]
    dec.reset()
    for t in prompt[:-1]:
        dec.step(t)
    a, la = dec.step(prompt[-1]), dec.logits()
    dec.reset()
    dec.prefill(prompt[:-1])  # two chunks
    b, lb = dec.step(prompt[-1]), dec.logits()
    assert np.abs(la - lb).max() <= 4e-3 * np.abs(la).max()
    dec.close()


@pytest.mark.parametrize("host_table", [False, True])
def test_per_layer_inputs_in_the_references_q4_with_the_table_in_host_memory(ctx, host_table):
    """A converted E-model (model/mod.rs:196-204): every matrix Q4, the 256-wide per-layer projections included (decode.rs:654-660),
    and the per-layer table either in HBM or where the reference keeps it, in pinned mapped host memory (host.wpk,
    decode.rs:477-483), read a row a step.  Filled from the generators, and loaded tensor by tensor as a converted model's files
    hold them: the same tokens and logits."""
    cfg = small_config(layers=5)
    cfg.per_layer, cfg.global_every, cfg.global_head_dim, cfg.shared = 256, 3, 512, 1
    dec = tb.Decoder(ctx, cfg, context=96, chunk=40, keep_logits=True, weight_bits=4, host_table=host_table)
    dec.fill_random(SEED + 9)
    dec.build()
    ref = OracleModel(cfg, SEED + 9, context=96, chunk=40, weight_bits=4)
    assert ref.tensors["3.per_layer_proj.w"].shape == (cfg.hidden, 128) and ref.tensors["embed_per_layer.s"].shape == (cfg.vocab, 5 * 256 // 64)
    other = tb.Decoder(ctx, cfg, context=96, chunk=40, keep_logits=True, weight_bits=4, host_table=host_table)
    for name, a in ref.tensors.items():
        other.load(name, a)
    other.build()
    token = 17
    for pos in range(12):
        want_token, want_logits, want_hidden = ref.step(token, pos)
        got_token = dec.step(token)
        order = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
        check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
        assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
        assert other.step(token) == got_token and np.array_equal(other.logits(), dec.logits()), "loaded or generated: the same bits"
        token = (pos * 7919 + 13) % cfg.vocab
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(70)]
    dec.reset()
    for t in prompt[:-1]:
        dec.step(t)
    a, la = dec.step(prompt[-1]), dec.logits()
    dec.reset()
    dec.prefill(prompt[:-1])  # two chunks
    b, lb = dec.step(prompt[-1]), dec.logits()
    assert np.abs(la - lb).max() <= 4e-3 * np.abs(la).max()
    dec.close(), other.close()


def test_a_layer_sharing_the_cache_of_the_layer_right_before_it(ctx):
    """The shortest distance between a layer and the layer whose cache it reads (model/mod.rs:138-143 with every layer
    sliding): layer 2 attends over the row layer 1 appended a few short kernels earlier in the same step, so nothing of
    layer 2's attention may be fetched before layer 1's has finished."""
    cfg = small_config(layers=3)
    cfg.global_every, cfg.shared = 0, 1
    dec = tb.Decoder(ctx, cfg, context=64, chunk=8, keep_logits=True)
    dec.fill_random(SEED + 9)
    dec.build()
    ref = OracleModel(cfg, SEED + 9, context=64, chunk=8)
    assert ref.tensors["2.qkv.w"].shape[0] == cfg.heads * cfg.head_dim
    token = 17
    for pos in range(40):
        want_token, want_logits, want_hidden = ref.step(token, pos)
        got_token = dec.step(token)
        order = np.sort(cfg.softcap * np.tanh(want_logits.astype(np.float64) / cfg.softcap))
        check_logits(dec.logits(), want_logits, order[-1] - order[-2], got_token, want_token)
        assert np.abs(dec.hidden() - want_hidden).max() <= 2e-3 * np.abs(want_hidden).max()
        token = (pos * 7919 + 13) % cfg.vocab
    # chained replays, where kernels of neighbouring steps overlap the most, give the same tokens as single steps
    dec.reset()
    single, t = [], 5
    for _ in range(24):
        t = dec.step(t)
        single.append(t)
    dec.reset()
    assert [int(v) for v in dec.run(5, 24)] == single
    dec.close()


def test_a_prompt_fed_step_by_step_does_not_count_as_generated_text(ctx):
    """Without chunk buffers the prompt goes through the decode step token by token.  Those steps must not mark their
    dropped picks as seen: the repetition penalty is about generated tokens (the reference's prefill samples nothing,
    model/prefill.rs:124-141)."""
    cfg = small_config()
    prompt = [(i * 7919 + 13) % cfg.vocab for i in range(20)]
    outs = []
    for settings_first in (True, False):
        dec = tb.Decoder(ctx, cfg, context=64, chunk=0, keep_logits=False)  # chunk 0: the prompt is fed by steps
        dec.fill_random(SEED)
        dec.build()
        if settings_first:
            dec.set_sampling(penalty=1.3, softcap=cfg.softcap)
        dec.prefill(prompt[:-1])
        if not settings_first:
            dec.set_sampling(penalty=1.3, softcap=cfg.softcap)
        outs.append([int(t) for t in dec.run(prompt[-1], 12)])
        dec.close()
    assert outs[0] == outs[1]
