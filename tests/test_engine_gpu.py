"""The engine against the plain implementation, in float32 and in bfloat16:
each request alone and whole; with the last 32 tokens one by one; in batches of
unequal lengths whose shorter requests end earlier, one batch after another so
that slots are used again; long decoding; the first tokens of a sequence.

Errors are measured as max |difference| / max |plain logits|.

Random N(0, 0.02) weights give flat attention, which hides a misplaced key, so
the tests that are about the cache sharpen the attention (helpers.model_folder).
A peaked softmax multiplies an upstream relative error by about the spread of
its scores, in every layer, so rounding noise grows with sharpness and depth:
float32 runs sharpen every layer by 3 (scores spread by about 9), bfloat16
runs sharpen only the last layer, since bfloat16's 8 significant bits start
from 3e-3 per matrix product.

Bounds, with what was measured on a B200 beside them (configurations A to D):
  float32, flat attention         3e-6    (3.3e-7 .. 6.8e-7)
  float32, every layer sharp      1e-3    (4.8e-6 .. 2.6e-5 in unequal batches,
      1.9e-4 at 300 positions: the 32-bit rotation angle is off by up to
      position * 2^-24)
  bfloat16, flat attention        1.5e-2  (2.0e-3 .. 6.2e-3)
  bfloat16, last layer sharp      4e-2    (1.8e-2 .. 2.2e-2 in unequal batches,
      1.9e-2 at 300 positions)
A key read from a wrong place moves a sharpened model's logits by tenths.  On
the float32 path the logits must moreover be bit-equal however the tokens are
cut into steps or batched: every kernel there reduces in an order that does not
depend on the batch, so any difference is a fault of the cache or the batch.
"""

import math

import numpy as np
import pytest
import torch

import helpers
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

F32_TOL = 3e-6
F32_SHARP_TOL = 1e-3
BF16_TOL = 1.5e-2
BF16_SHARP_TOL = 4e-2
FULL_DEPTH_BF16_TOL = 4e-2  # 36 layers at the benchmark model's widths (measured: 2.5e-2)


def tol(dtype, sharp=False):
    if dtype == "float32":
        return F32_SHARP_TOL if sharp else F32_TOL
    return BF16_SHARP_TOL if sharp else BF16_TOL


def sharp_folder(name, seed, dtype):
    if dtype == "float32":
        return helpers.model_folder(name, seed, "float32", sharp=3.0, sharp_layers="all")
    return helpers.model_folder(name, seed, "bfloat16", sharp=3.0, sharp_layers="last")


def stored(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


CASES = [(n, d) for n in ALL for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_and_tail_one_by_one(name, dtype):
    V = ALL[name]["vocab_size"]
    folder = helpers.model_folder(name, 7, stored(dtype))
    eng = helpers.make_engine(folder, dtype, max_tokens=1024)
    for n, seed in ((100, 3), (33, 4)):
        toks = helpers.random_tokens(n, V, seed)
        ref = helpers.plain_logits(folder, toks)
        whole = helpers.run_whole(eng, toks)
        tail = helpers.run_tail_one_by_one(eng, toks, 32)
        assert whole.shape == ref.shape == tail.shape
        assert helpers.rel_err(whole, ref) < tol(dtype)
        assert helpers.rel_err(tail, ref) < tol(dtype)
        if dtype == "float32":
            assert np.array_equal(whole, tail), "float32 logits depend on how tokens are cut"
    assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_early_ends_slot_reuse(name, dtype):
    V = ALL[name]["vocab_size"]
    folder = sharp_folder(name, 7, dtype)
    # fewer slots than requests: batches of 3 follow one another in reused slots
    eng = helpers.make_engine(folder, dtype, max_tokens=64 * 8, max_slots=3)
    lengths = (5, 17, 32, 1, 70, 129, 64, 2, 65)
    reqs = [helpers.random_tokens(n, V, 100 + n) for n in lengths]
    got = helpers.run_batches(eng, reqs, 3, [5, 17, 20, 1, 64])
    alone = helpers.make_engine(folder, dtype, max_tokens=64 * 8)
    for r, g in zip(reqs, got):
        ref = helpers.plain_logits(folder, r)
        assert g.shape == ref.shape
        assert helpers.rel_err(g, ref) < tol(dtype, sharp=True), len(r)
        if dtype == "float32":
            assert np.array_equal(g, helpers.run_whole(alone, r)), "batching changed float32 logits"
    assert eng.cache.slots.held_count == 0
    assert all(g.pool.held_count == 0 for g in eng.cache.kv_groups)


def mirror_logits(folder, tokens, **kw):
    import fp32_mirror
    import plain_model

    cfg, w = plain_model.read_model(folder)
    return fp32_mirror.forward(cfg, w, tokens, **kw)


@pytest.mark.parametrize("name", list(ALL))
def test_float32_logits_equal_the_host_mirror_bit_for_bit(name):
    """The true 32-bit path against a host program that repeats its kernels'
    arithmetic operation by operation (tests/fp32_mirror.py): the same bits at
    every position, for each request whole, with its last 32 tokens one by one,
    and in unequal batches whose slots are used again.  A tolerance would not see
    a last-bit dependence on the batch that two cuttings happen to share; this
    does.  The mirror with one reduction order changed (the norm's sum of squares
    in plain index order) no longer matches, so the comparison is that sharp."""
    V = ALL[name]["vocab_size"]
    flat = helpers.model_folder(name, 7, "float32")
    eng = helpers.make_engine(flat, "float32", max_tokens=1024)
    for n, seed in ((100, 3), (33, 4), (1, 5)):
        toks = helpers.random_tokens(n, V, seed)
        ref = mirror_logits(flat, toks)
        assert np.array_equal(helpers.run_whole(eng, toks), ref), "whole"
        assert np.array_equal(helpers.run_tail_one_by_one(eng, toks, 32), ref), "last 32 one by one"
        if n == 100:
            assert not np.array_equal(mirror_logits(flat, toks, norm_order=1), ref)
    sharp = sharp_folder(name, 7, "float32")
    eng = helpers.make_engine(sharp, "float32", max_tokens=64 * 8, max_slots=3)
    lengths = (5, 17, 32, 1, 70, 129, 64, 2, 65)
    reqs = [helpers.random_tokens(n, V, 100 + n) for n in lengths]
    got = helpers.run_batches(eng, reqs, 3, [5, 17, 20, 1, 64])
    for r, g in zip(reqs, got):
        assert np.array_equal(g, mirror_logits(sharp, r)), f"batched, length {len(r)}"
    assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_requests_cut_into_steps_at_random_places(name, dtype):
    """Seven requests of random lengths through three slots.  Every step takes,
    from each live request, either one token or a chunk of random length, so
    chunks of prompts and single tokens of other requests meet in one step, a
    request's cuts fall anywhere (inside pages, at their edges, at the window's
    edge), requests end at different steps and the next one takes the slot that
    came free.  Every position's logits are asked for.  float32: the bits of the
    host mirror; bfloat16: within the bound of the plain implementation."""
    V = ALL[name]["vocab_size"]
    folder = sharp_folder(name, 7, dtype)
    rng = np.random.default_rng(sum(map(ord, name + dtype)))
    lengths = [int(x) for x in rng.integers(1, 150, size=7)]
    reqs = [helpers.random_tokens(n, V, 300 + i) for i, n in enumerate(lengths)]
    eng = helpers.make_engine(folder, dtype, max_tokens=3 * 192, max_slots=3)
    waiting = list(range(len(reqs)))
    live = {}  # request -> (slot, tokens done)
    got = {i: [] for i in range(len(reqs))}
    steps = 0
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = (eng.open(), 0)
        entries, order = [], []
        for i, (slot, done) in live.items():
            left = len(reqs[i]) - done
            n = 1 if rng.random() < 0.4 else int(rng.integers(1, min(left, 70) + 1))
            entries.append((slot, reqs[i][done:done + n], list(range(n))))
            order.append((i, n))
        out = eng.step(entries).float().cpu().numpy()
        steps += 1
        row = 0
        for i, n in order:
            got[i].append(out[row:row + n])
            row += n
            slot, done = live[i]
            if done + n == len(reqs[i]):
                eng.close(slot)
                del live[i]
            else:
                live[i] = (slot, done + n)
    assert eng.cache.slots.held_count == 0 and steps > 7
    for i, r in enumerate(reqs):
        g = np.concatenate(got[i], axis=0)
        if dtype == "float32":
            ref = mirror_logits(folder, r)
            bad = np.nonzero((g != ref).any(axis=1))[0]
            assert bad.size == 0, f"request {i} of {len(r)} tokens: first differing position {int(bad[0])}"
        else:
            assert helpers.rel_err(g, helpers.plain_logits(folder, r)) < tol(dtype, sharp=True), (i, len(r))


def test_float32_long_decoding_equals_the_host_mirror():
    """300 tokens one by one on the model with sliding layers: page edges, the
    window's edge and pages given back under way, bit for bit."""
    V = ALL["C"]["vocab_size"]
    folder = sharp_folder("C", 11, "float32")
    eng = helpers.make_engine(folder, "float32", max_tokens=512)
    toks = helpers.random_tokens(300, V, 5)
    got = helpers.run_tail_one_by_one(eng, toks, tail=299)
    ref = mirror_logits(folder, toks)
    bad = np.nonzero((got != ref).any(axis=1))[0]
    assert bad.size == 0, f"first differing position {int(bad[0])}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_page_and_window_edges(dtype):
    """300 tokens one by one on the model with sliding layers (window 37):
    crosses four page edges; the window group gives pages back under way."""
    name = "C"
    V = ALL[name]["vocab_size"]
    folder = sharp_folder(name, 11, dtype)
    eng = helpers.make_engine(folder, dtype, max_tokens=512)
    toks = helpers.random_tokens(300, V, 5)
    ref = helpers.plain_logits(folder, toks)
    got = helpers.run_tail_one_by_one(eng, toks, tail=299)
    err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
    assert err.max() < tol(dtype, sharp=True), int(err.argmax())
    wg = [g for g in eng.cache.kv_groups if g.spec.window]
    assert wg and wg[0].pool.held_count == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype):
    V = ALL[name]["vocab_size"]
    folder = helpers.model_folder(name, 7, stored(dtype))
    eng = helpers.make_engine(folder, dtype, max_tokens=256)
    toks = helpers.random_tokens(4, V, 9)
    ref = helpers.plain_logits(folder, toks)
    one = helpers.run_tail_one_by_one(eng, toks, tail=3)  # 1 token, then 1, 1, 1
    assert helpers.rel_err(one, ref) < tol(dtype)
    s = eng.open()
    only_last = eng.step([(s, toks, [3])]).float().cpu().numpy()
    eng.close(s)
    assert only_last.shape == (1, V)
    assert helpers.rel_err(only_last, ref[3:4]) < tol(dtype) * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_step_and_no_wanted_logits(dtype):
    """A step may mix a chunk of one request with one token of another, and
    may ask for no logits at all (it then only fills the cache)."""
    name = "B"
    V = ALL[name]["vocab_size"]
    folder = sharp_folder(name, 7, dtype)
    eng = helpers.make_engine(folder, dtype, max_tokens=512)
    a, b = helpers.random_tokens(90, V, 1), helpers.random_tokens(40, V, 2)
    sa, sb = eng.open(), eng.open()
    out = eng.step([(sa, a[:50], []), (sb, b[:39], [])])
    assert out.shape == (0, V)
    out = eng.step([(sa, a[50:], list(range(40))), (sb, b[39:], [0])]).float().cpu().numpy()
    ra, rb = helpers.plain_logits(folder, a), helpers.plain_logits(folder, b)
    assert helpers.rel_err(out[:40], ra[50:]) < tol(dtype, sharp=True)
    assert helpers.rel_err(out[40:], rb[39:]) < tol(dtype, sharp=True)
    eng.close(sa)
    eng.close(sb)


def test_decode_graphs_equal_eager_steps():
    name = "B"
    V = ALL[name]["vocab_size"]
    folder = helpers.model_folder(name, 7, "bfloat16")
    toks = helpers.random_tokens(80, V, 3)
    a = helpers.run_tail_one_by_one(helpers.make_engine(folder, "bfloat16", use_graphs=False), toks, 40)
    eng = helpers.make_engine(folder, "bfloat16", use_graphs=True)
    b = helpers.run_tail_one_by_one(eng, toks, 40)
    assert eng._graphs and all(g.graph is not None for g in eng._graphs.values())
    assert np.array_equal(a, b)


def test_step_errors_leave_the_cache_as_it_was():
    from reflex_b200 import ContextOverflow, InvalidInput, OutOfMemory

    folder = helpers.model_folder("A", 7, "float32")
    eng = helpers.make_engine(folder, "float32", max_tokens=128)
    s = eng.open()
    with pytest.raises(InvalidInput):
        eng.step([(s, [1, 2, 99999], [0])])
    with pytest.raises(InvalidInput):
        eng.step([(s, [], [])])
    with pytest.raises(InvalidInput):
        eng.step([(s, [1], [1])])
    with pytest.raises(InvalidInput):
        eng.step([(s, [1], [0]), (s, [2], [0])])
    with pytest.raises(OutOfMemory):
        eng.step([(s, [1] * 200, [0])])
    with pytest.raises(ContextOverflow):
        eng.step([(s, [1] * 300, [0])])
    assert eng.length(s) == 0 and all(g.pool.held_count == 0 for g in eng.cache.kv_groups)
    out = eng.step([(s, [1, 2, 3], [2])])
    assert out.shape == (1, 512) and eng.length(s) == 3
    eng.close(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_at_the_benchmark_models_widths(dtype):
    """The tiny configurations keep every size small; here one layer has the
    benchmark model's widths (hidden 4096, 32 query and 8 kv heads of 128,
    feed-forward 12288; the vocabulary cut to 2048 so that the plain
    implementation stays quick), which is where the tensor-core kernels' tile
    cuts, K splits and clusters are what they are in use.  A prompt whole, then
    its last tokens one by one, and a batch of three, against the plain
    implementation.  In 32-bit the bound is the tiny models' bound scaled by the
    square root of the longest reduction (12288 terms here against 320 there):
    sequential 32-bit sums round once per term.  The cuttings still agree bit
    for bit."""
    import shutil
    import tempfile

    import plain_model
    from reflex_b200.weights import write_random_model

    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": 12288, "vocab_size": 2048, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": False, "max_position_embeddings": 4096,
    }
    folder = tempfile.mkdtemp(prefix="rfx_wide_")
    try:
        write_random_model(cfg, 11, folder, stored(dtype))
        eng = helpers.make_engine(folder, dtype, max_tokens=1024)
        pcfg, w = plain_model.read_model(folder)
        toks = helpers.random_tokens(70, 2048, 5)
        ref = plain_model.forward(pcfg, w, toks)
        bound = tol(dtype) * (math.sqrt(12288 / 320) if dtype == "float32" else 1.0)
        whole = helpers.run_whole(eng, toks)
        tail = helpers.run_tail_one_by_one(eng, toks, 6)
        assert helpers.rel_err(whole, ref) < bound
        assert helpers.rel_err(tail, ref) < bound
        if dtype == "float32":
            assert np.array_equal(whole, tail)
        reqs = [toks[:9], toks[9:40], toks[40:]]
        got = helpers.run_batches(eng, reqs, 3, [4, 20, 8])
        for r, g in zip(reqs, got):
            assert helpers.rel_err(g, plain_model.forward(pcfg, w, r)) < bound
        if dtype == "float32":
            import fp32_mirror

            assert np.array_equal(got[0], fp32_mirror.forward(pcfg, w, reqs[0]))
        assert eng.cache.slots.held_count == 0
    finally:
        shutil.rmtree(folder, ignore_errors=True)


def _random_config(seed):
    """A configuration drawn from sizes that strain the kernels' cuts: widths
    that are and are not multiples of 8, head sizes from 16 to 256, groups up
    to 17, windows shorter and longer than a page."""
    import random

    rng = random.Random(seed)
    d = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256])
    nkv = rng.choice([1, 1, 2, 3, 4, 8])
    g = rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 16, 17])
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, 5, 20, 64, 70])
    types = [rng.choice(["full_attention", "sliding_attention"]) if window else "full_attention"
             for _ in range(layers)]
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
        "hidden_size": rng.choice([20, 36, 50, 64, 72, 100, 104, 129, 200, 264, 520, 1032]),
        "num_attention_heads": g * nkv, "num_key_value_heads": nkv, "head_dim": d,
        "intermediate_size": rng.choice([8, 24, 50, 100, 136, 200, 301, 512, 1000]),
        "vocab_size": rng.choice([17, 100, 333, 512, 1001, 4097]),
        "rope_theta": rng.choice([1e4, 1e6, 500.0]), "rms_norm_eps": rng.choice([1e-6, 1e-5, 1e-3]),
        "tie_word_embeddings": rng.choice([True, False]), "max_position_embeddings": 1024,
        "sliding_window": window if "sliding_attention" in types else None, "layer_types": types,
    }


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configurations(seed, dtype):
    """Unequal batches (slots used again) and a tail decoded one by one, for
    configurations drawn at random from a fixed seed, against the plain
    implementation.  The 32-bit bound is a little above the tiny models' (head
    sizes up to 256 and widths up to 1032 make the reductions longer)."""
    import shutil
    import tempfile

    import plain_model
    from reflex_b200.weights import write_random_model

    cfg = _random_config(seed)
    folder = tempfile.mkdtemp(prefix="rfx_rand_")
    try:
        write_random_model(cfg, seed, folder, stored(dtype))
        eng = helpers.make_engine(folder, dtype, max_tokens=4096)
        pcfg, w = plain_model.read_model(folder)
        V = cfg["vocab_size"]
        reqs = [helpers.random_tokens(n, V, n + seed) for n in (2, 100, 64, 37)]
        bound = 5e-6 if dtype == "float32" else BF16_TOL
        got = helpers.run_batches(eng, reqs, 3, [1, 200, 7])
        for r, g in zip(reqs, got):
            assert helpers.rel_err(g, plain_model.forward(pcfg, w, r)) < bound, cfg
        tail = helpers.run_tail_one_by_one(eng, reqs[1], 32)
        assert helpers.rel_err(tail, plain_model.forward(pcfg, w, reqs[1])) < bound, cfg
        if dtype == "float32":
            import fp32_mirror

            for r, g in zip(reqs, got):
                assert np.array_equal(g, fp32_mirror.forward(pcfg, w, r)), cfg
        assert eng.cache.slots.held_count == 0
    finally:
        shutil.rmtree(folder, ignore_errors=True)


# ----------------------------------------------- schedules around the decode graphs
def test_logits_of_two_steps_can_be_held_together():
    """A step's logits belong to the caller: the next replay of the same graph
    does not overwrite them.  With `borrow=True` they are the graph's own
    buffer and the next step does overwrite them, which is what the flag says."""
    V = ALL["B"]["vocab_size"]
    folder = helpers.model_folder("B", 7, "bfloat16")
    eng = helpers.make_engine(folder, "bfloat16", max_tokens=512)
    toks = helpers.random_tokens(40, V, 8)
    ref = helpers.plain_logits(folder, toks)
    s = eng.open()
    eng.step([(s, toks[:30], [])])
    kept = [eng.step([(s, [toks[i]], [0])]) for i in range(30, 40)]  # every step's logits held
    assert any(g.graph is not None for g in eng._graphs.values())
    for i, l in zip(range(30, 40), kept):
        assert helpers.rel_err(l.float().cpu().numpy(), ref[i:i + 1]) < BF16_TOL, i
    eng.close(s)
    s = eng.open()
    eng.step([(s, toks[:30], [])])
    lent = [eng.step([(s, [toks[i]], [0])], borrow=True) for i in range(30, 34)]
    assert lent[-1].data_ptr() == lent[-2].data_ptr()  # the same storage, as documented
    eng.close(s)


def test_wanted_places_other_than_one_per_token_go_the_eager_way():
    """[[0, 0], []] for two decode sequences passes the checks and has as many
    wanted rows as tokens, but is not the captured step's shape."""
    V = ALL["B"]["vocab_size"]
    folder = helpers.model_folder("B", 7, "bfloat16")
    eng = helpers.make_engine(folder, "bfloat16", max_tokens=512)
    a, b = helpers.random_tokens(20, V, 1), helpers.random_tokens(9, V, 2)
    sa, sb = eng.open(), eng.open()
    eng.step([(sa, a[:19], []), (sb, b[:8], [])])
    out = eng.step([(sa, [a[19]], [0, 0]), (sb, [b[8]], [])]).float().cpu().numpy()
    ref = helpers.plain_logits(folder, a)[19:20]
    assert out.shape == (2, V)
    assert helpers.rel_err(out[0:1], ref) < BF16_TOL and helpers.rel_err(out[1:2], ref) < BF16_TOL
    eng.close(sa)
    eng.close(sb)


def test_a_batch_of_64_that_ends_one_request_at_a_time():
    """64 requests decoded together in bfloat16 with graphs on, whose lengths
    make them leave one after another, so the batch shrinks through every size
    from 64 to 1.  Logits of several requests against the plain implementation;
    the number of graphs and the device memory they take stay bounded (they
    share one pool, and a new size captures at once instead of running eager
    warm-up steps)."""
    V = ALL["B"]["vocab_size"]
    folder = helpers.model_folder("B", 7, "bfloat16")
    eng = helpers.make_engine(folder, "bfloat16", max_tokens=64 * 64 * 2, max_graphs=40)
    reqs = [helpers.random_tokens(3 + (i % 5) + i, V, 200 + i) for i in range(64)]  # lengths 3 .. 70, all different
    torch.cuda.synchronize()
    before = torch.cuda.memory_reserved()
    got = helpers.run_batches(eng, reqs, 64, [3])
    grown = torch.cuda.memory_reserved() - before
    assert eng._eager_decodes == 1
    assert len(eng._graphs) <= 40
    assert grown < 256 << 20, f"decode graphs took {grown >> 20} MiB"
    for i in (0, 1, 17, 40, 63):
        assert helpers.rel_err(got[i], helpers.plain_logits(folder, reqs[i])) < BF16_TOL, i
    assert eng.cache.slots.held_count == 0


@pytest.mark.parametrize("n", [65, 100, 128])
def test_decode_batches_above_64_rows(n):
    """More decode rows than the weight-streaming product takes: the step
    leaves the fused path (library products, stand-alone norms) and must give
    the same logits."""
    V = ALL["B"]["vocab_size"]
    folder = helpers.model_folder("B", 7, "bfloat16")
    eng = helpers.make_engine(folder, "bfloat16", max_tokens=64 * n)
    reqs = [helpers.random_tokens(4 + i % 7, V, 300 + i) for i in range(n)]
    got = helpers.run_batches(eng, reqs, n, [2])
    for i in (0, 1, n // 2, n - 1):
        assert helpers.rel_err(got[i], helpers.plain_logits(folder, reqs[i])) < BF16_TOL, i


def test_a_token_id_fed_from_the_device_outside_the_vocabulary_is_reported():
    from reflex_b200 import CudaError

    folder = helpers.model_folder("A", 7, "bfloat16")
    eng = helpers.make_engine(folder, "bfloat16", max_tokens=256)
    s = eng.open()
    eng.step([(s, [1, 2, 3], [2])])
    eng.check_errors()
    bad = torch.tensor([ALL["A"]["vocab_size"] + 5], dtype=torch.int32, device="cuda:0")
    eng.step_decode([s], bad)
    with pytest.raises(CudaError):
        eng.check_errors()
    eng.check_errors()  # reported once, the device stays usable
    out = eng.step([(s, [4], [0])])
    assert bool(torch.isfinite(out).all())
    eng.close(s)


def test_the_benchmark_model_at_full_depth_and_vocabulary():
    """All 36 layers at the benchmark model's sizes with the 151,936-row head, in
    bfloat16, random weights drawn on the device: two short prompts in one
    prefill step, then three decode steps (captured), logits at every fed
    position against the plain implementation, which rebuilds the same weights
    tensor by tensor from (seed, name) and streams one layer at a time.  What
    `bench.py` times is this model; here its output is checked."""
    import gc

    import plain_model
    from reflex_b200.engine import Engine
    from reflex_b200.weights import random_model_on_device
    from reflex_b200.weights.random_init import draw

    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": False, "max_position_embeddings": 40960,
    }
    seed = 0
    lm = random_model_on_device(cfg, seed, torch.bfloat16, "cuda:0")
    eng = Engine(lm, max_tokens=1024)
    V = cfg["vocab_size"]
    seqs_tok = [helpers.random_tokens(5, V, 1), helpers.random_tokens(9, V, 2)]
    n_prompt = [len(t) for t in seqs_tok]
    ids = [eng.open(), eng.open()]
    out = eng.step([(s, t, [len(t) - 1]) for s, t in zip(ids, seqs_tok)])
    got = [[out[i].float().cpu().numpy()] for i in range(2)]
    for _ in range(3):
        nxt = [int(g[-1].argmax()) for g in got]
        for t, n in zip(seqs_tok, nxt):
            t.append(n)
        out = eng.step([(s, [n], [0]) for s, n in zip(ids, nxt)])
        for i in range(2):
            got[i].append(out[i].float().cpu().numpy())
    eng.check_errors()
    assert eng._graphs, "the decode steps were to run as captured graphs"
    for s in ids:
        eng.close(s)
    del eng, lm, out
    gc.collect()
    torch.cuda.empty_cache()

    def tensor(name, shape, role="matrix"):
        # the same (seed, name) draw, made on the device for speed and copied: the host
        # draw gives the same bits (tests/test_upload_gpu.py holds them together)
        dt = torch.float32 if role == "norm" else torch.bfloat16
        return draw(name, shape, role, seed, "cuda:0", dt).float().cpu().numpy()

    H, I, nq, nkv, d = 4096, 12288, 32, 8, 128
    emb = tensor("model.embed_tokens.weight", (V, H), "table")
    hs = [emb[np.array(t)] for t in seqs_tok]  # float32 throughout: the weights stay as they are drawn
    del emb
    for li in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{li}."
        w = {p + "input_layernorm.weight": tensor(p + "input_layernorm.weight", (H,), "norm"),
             p + "post_attention_layernorm.weight": tensor(p + "post_attention_layernorm.weight", (H,), "norm"),
             p + "self_attn.q_norm.weight": tensor(p + "self_attn.q_norm.weight", (d,), "norm"),
             p + "self_attn.k_norm.weight": tensor(p + "self_attn.k_norm.weight", (d,), "norm"),
             p + "self_attn.q_proj.weight": tensor(p + "self_attn.q_proj.weight", (nq * d, H)),
             p + "self_attn.k_proj.weight": tensor(p + "self_attn.k_proj.weight", (nkv * d, H)),
             p + "self_attn.v_proj.weight": tensor(p + "self_attn.v_proj.weight", (nkv * d, H)),
             p + "self_attn.o_proj.weight": tensor(p + "self_attn.o_proj.weight", (H, nq * d)),
             p + "mlp.gate_proj.weight": tensor(p + "mlp.gate_proj.weight", (I, H)),
             p + "mlp.up_proj.weight": tensor(p + "mlp.up_proj.weight", (I, H)),
             p + "mlp.down_proj.weight": tensor(p + "mlp.down_proj.weight", (H, I))}
        hs = [plain_model.decoder_layer(h, w, p, cfg, np.arange(h.shape[0]), None) for h in hs]
    fn = tensor("model.norm.weight", (H,), "norm")
    head = tensor("lm_head.weight", (V, H))
    worst = 0.0
    for i in range(2):
        x = plain_model.rms_norm(hs[i][n_prompt[i] - 1:], fn, cfg["rms_norm_eps"])
        ref = (x.astype(np.float32) @ head.T).astype(np.float64)
        g = np.stack(got[i])
        assert g.shape == ref.shape and np.isfinite(g).all()
        err = helpers.rel_err(g, ref)
        worst = max(worst, err)
        # the greedy choice agrees wherever the plain model's margin is clear of the error
        for r in range(ref.shape[0]):
            top = np.sort(ref[r])[-2:]
            if top[1] - top[0] > 4 * err * np.abs(ref).max():
                assert int(g[r].argmax()) == int(ref[r].argmax())
    print(f"full-depth bfloat16 error {worst:.3e}")
    assert worst < FULL_DEPTH_BF16_TOL, worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_take_their_memory_from_the_engines_workspace(dtype):
    """After the first step of a size has told the workspace how much it needs,
    further steps of that size are served from it entirely (no request falls
    through to the allocator), prefill and eager decode alike, and give the
    same logits as before."""
    V = ALL["B"]["vocab_size"]
    folder = helpers.model_folder("B", 7, stored(dtype))
    eng = helpers.make_engine(folder, dtype, max_tokens=1024, use_graphs=False)
    toks = helpers.random_tokens(90, V, 12)
    first = helpers.run_tail_one_by_one(eng, toks, 8)
    misses = eng.workspace.misses
    assert misses > 0 and eng.workspace.nbytes > 0
    again = helpers.run_tail_one_by_one(eng, toks, 8)
    assert eng.workspace.misses == misses
    assert np.array_equal(first, again)
    assert helpers.rel_err(again, helpers.plain_logits(folder, toks)) < tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_context_across_graph_buckets_and_many_key_splits(dtype):
    """2,000 tokens in one step, then 150 decoded one by one, on the model with
    sliding layers and a head size of 48: the context passes 32 pages, where the
    decode graphs' buckets change from steps of four pages to powers of two and
    a single sequence's keys are split over more CTAs than a cluster holds (the
    combine kernel merges them).  Every decoded position against the plain
    implementation; in 32-bit also bit for bit against the host mirror."""
    cfg = dict(ALL["C"], max_position_embeddings=4096)
    import shutil
    import tempfile

    import plain_model
    from reflex_b200.weights import write_random_model

    folder = tempfile.mkdtemp(prefix="rfx_long_")
    try:
        write_random_model(cfg, 21, folder, stored(dtype))
        eng = helpers.make_engine(folder, dtype, max_tokens=2304)
        toks = helpers.random_tokens(2150, cfg["vocab_size"], 17)
        pcfg, w = plain_model.read_model(folder)
        s = eng.open()
        out = [eng.step([(s, toks[:2000], [1999])]).float().cpu().numpy()]
        for i in range(2000, 2150):
            out.append(eng.step([(s, [toks[i]], [0])]).float().cpu().numpy())
        eng.close(s)
        got = np.concatenate(out, axis=0)
        ref = plain_model.forward(pcfg, w, toks)[1999:]
        err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
        # the 32-bit rotation angle is off by up to position * 2^-24: 1.3e-4 at 2,150 positions
        assert err.max() < (5e-4 if dtype == "float32" else BF16_TOL), int(err.argmax())
        if dtype == "float32":
            import fp32_mirror

            assert np.array_equal(got, fp32_mirror.forward(pcfg, w, toks)[1999:])
        else:
            assert len({k[1] for k in eng._graphs}) >= 2  # more than one context bucket was captured
    finally:
        shutil.rmtree(folder, ignore_errors=True)


def test_a_step_whose_intermediates_pass_two_to_the_31_elements():
    """26 prompts of 4,096 tokens in one step at the benchmark model's widths (two
    layers): 106,496 rows, so the feed-forward's intermediate has 2.6e9 elements
    and every index that multiplies rows by a width must be 64 bits wide.  A
    request's logits in that batch against the same request alone (the library's
    matrix product may pick another algorithm for another number of rows, so a
    last-bit difference is allowed, no more), and a decode step after it."""
    from reflex_b200.engine import Engine
    from reflex_b200.weights import random_model_on_device

    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096,
           "intermediate_size": 12288, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
           "num_hidden_layers": 2, "vocab_size": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
           "tie_word_embeddings": False, "max_position_embeddings": 8192}
    lm = random_model_on_device(cfg, 0, torch.bfloat16, "cuda:0")
    n_seq, L = 26, 4096
    assert n_seq * L * 2 * cfg["intermediate_size"] > 2 ** 31
    eng = Engine(lm, max_tokens=(n_seq + 1) * (L + 64), max_slots=n_seq + 1)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg["vocab_size"], (n_seq, L), generator=g).tolist()
    want = [0, L // 2, L - 1]
    seqs = [eng.open() for _ in prompts]
    big = eng.step([(s, p, want) for s, p in zip(seqs, prompts)]).float().cpu().numpy()
    eng.check_errors()
    assert np.isfinite(big).all()
    for i in (0, 11, n_seq - 1):
        s = eng.open()
        one = eng.step([(s, prompts[i], want)]).float().cpu().numpy()
        eng.close(s)
        assert helpers.rel_err(big[3 * i:3 * i + 3], one) < 1e-4, i
    ids = [int(x) for x in big[2::3].argmax(axis=1)]
    out = eng.step([(s, [t], [0]) for s, t in zip(seqs, ids)]).float().cpu().numpy()
    eng.check_errors()
    assert np.isfinite(out).all()
    for s in seqs:
        eng.close(s)
    del eng, lm
    torch.cuda.empty_cache()
