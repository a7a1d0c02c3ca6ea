"""Generation through the entry points: greedy and sampled generation against
the plain implementation, the command line, and trace replay as a user runs it."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
import plain_model as pm
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_generate(folder, prompt, n, pick):
    cfg, w = pm.read_model(folder)
    seq, out, margins = list(prompt), [], []
    for step in range(n):
        logits = pm.forward(cfg, w, seq)[-1]
        tok = pick(logits, step)
        top2 = np.sort(logits)[-2:]
        margins.append(float(top2[1] - top2[0]))
        out.append(tok)
        seq.append(tok)
    return out, margins


@pytest.mark.parametrize("name,weights", [("A", "f32"), ("B", "f32"), ("B", "bf16"), ("C", "bf16")])
def test_greedy_generation_of_an_unequal_batch(name, weights):
    import reflex_b200

    folder = helpers.model_folder(name, 7, "float32" if weights == "f32" else "bfloat16")
    V = ALL[name]["vocab_size"]
    lengths = (5, 17, 32) if name == "A" else (1, 7, 64, 100, 129)
    n_new = 16 if name == "A" else 24
    prompts = [helpers.random_tokens(n, V, 40 + n) for n in lengths]
    model = reflex_b200.Model.load(folder, weights=weights, max_tokens=4096, max_batch=4)
    got = model.generate(prompts, n_new)
    assert model.last_stats.batches == (1 if name == "A" else 2)
    for p, g in zip(prompts, got):
        assert len(g) == n_new
        want, margins = plain_generate(folder, p, n_new, lambda l, s: pm.argmax_last(l))
        for i, (a, b) in enumerate(zip(g, want)):
            if a != b:
                # only a near tie may differ, and then the sequences part ways
                limit = 1e-5 if weights == "f32" else 2e-2
                assert margins[i] < limit * max(1.0, margins[i]), (len(p), i, a, b, margins[i])
                break
    one = model.generate(prompts[1], 3)
    assert one == got[1][:3]  # alone or in a batch: the same tokens


def test_load_options_as_one_object_and_from_the_environment(monkeypatch):
    import reflex_b200
    from reflex_b200 import EngineOptions, InvalidInput

    folder = helpers.model_folder("A", 7, "float32")
    prompt = helpers.random_tokens(9, ALL["A"]["vocab_size"], 3)
    want, _ = plain_generate(folder, prompt, 4, lambda l, s: pm.argmax_last(l))
    model = reflex_b200.Model.load(folder, options=EngineOptions(weights="f32", max_tokens=256, max_batch=2,
                                                                 use_graphs=False))
    assert model.weights_dtype == "f32" and model.max_batch == 2
    assert model.generate(prompt, 4) == want
    # an argument beside the options wins; the environment fills in when neither names the weights
    assert reflex_b200.Model.load(folder, weights="bf16", options=EngineOptions(weights="f32")).weights_dtype == "bf16"
    monkeypatch.setenv("REFLEX_WEIGHTS", "f32")
    assert reflex_b200.Model.load(folder, max_tokens=256).weights_dtype == "f32"
    with pytest.raises(InvalidInput):
        reflex_b200.Model.load(folder, max_slots=3)


def test_sampled_generation_follows_the_plain_sampler_with_the_same_uniforms():
    import reflex_b200
    from reflex_b200.sampling import uniform

    folder = helpers.model_folder("B", 7, "float32")
    V = ALL["B"]["vocab_size"]
    prompts = [helpers.random_tokens(n, V, 60 + n) for n in (1, 7, 64)]
    model = reflex_b200.Model.load(folder, weights="f32", max_tokens=2048)
    params = reflex_b200.SamplingParams(temperature=0.8, seed=1234, top_k=50, top_p=0.95)
    got = model.generate(prompts, 12, params)
    assert got == model.generate(prompts, 12, params)  # a seed makes it reproducible
    assert got != model.generate(prompts, 12, reflex_b200.SamplingParams(temperature=0.8, seed=99))
    for r, (p, g) in enumerate(zip(prompts, got)):
        want, _ = plain_generate(folder, p, 12, lambda l, s: pm.sample_token(l, 0.8, uniform(1234, r, s), 50, 0.95))
        assert g == want
    alone = model.generate([prompts[2]], 12, params)[0]
    assert len(alone) == 12 and all(0 <= t < V for t in alone)


def test_stop_tokens_and_limits_through_the_entry_point():
    import reflex_b200
    from reflex_b200 import InvalidInput

    folder = helpers.model_folder("A", 7, "float32")
    model = reflex_b200.Model.load(folder, weights="f32", max_tokens=1024)
    prompt = helpers.random_tokens(9, 512, 1)
    free = model.generate(prompt, 10)
    stop = free[3]
    cut = model.generate(prompt, 10, reflex_b200.SamplingParams(stop_token_ids=(stop,)))
    assert cut == free[: free.index(stop) + 1]  # the stop token is kept, then it ends
    with pytest.raises(InvalidInput):
        model.generate(prompt, 0)
    with pytest.raises(InvalidInput):
        model.generate([prompt, []], 2)
    with pytest.raises(reflex_b200.ContextOverflow):
        model.generate(prompt, 250)  # max_position_embeddings is 256


def test_system1_scores_candidates_in_one_step():
    import reflex_b200

    folder = helpers.model_folder("B", 7, "float32")
    cfg, w = pm.read_model(folder)
    model = reflex_b200.Model.load(folder, weights="f32", max_tokens=2048)
    prompt = helpers.random_tokens(11, 1000, 3)
    cands = [[5], [77, 3, 910], [400, 401]]
    steps = model.engine.steps_run
    resp = model.system1_evaluate(prompt, cands, temperature=0.5)
    assert model.engine.steps_run == steps + 1
    scores = []
    for c in cands:
        logits = pm.forward(cfg, w, prompt + c[:-1])
        scores.append(sum(float(logits[len(prompt) - 1 + i, t]) for i, t in enumerate(c)))
    np.testing.assert_allclose([r.score for r in resp.results], scores, rtol=1e-4, atol=1e-5)
    e = np.exp((np.array(scores) - max(scores)) / 0.5)
    np.testing.assert_allclose(resp.probabilities, e / e.sum(), rtol=1e-3)
    assert resp.best_idx == int(np.argmax(scores))
    assert abs(resp.entropy + float((e / e.sum() * np.log2(e / e.sum())).sum())) < 1e-3


@pytest.mark.parametrize("weights,tol", [("f32", 0.0), ("bf16", 1e-4)])
def test_system1_reads_only_the_candidates_rows_of_the_head(weights, tol):
    """The scores come from a product over the candidates' rows of the head
    alone; they equal what the full-vocabulary logits hold at the same places
    (bit for bit in 32-bit, within 1e-4 in bfloat16,
    src/model/system1_tests.rs:14-65)."""
    import reflex_b200

    folder = helpers.model_folder("B", 7, "float32" if weights == "f32" else "bfloat16")
    model = reflex_b200.Model.load(folder, weights=weights, max_tokens=2048)
    prompt = helpers.random_tokens(70, 1000, 4)
    cands = [[5], [77, 3, 910], [400, 401], [999, 0]]
    resp = model.system1_evaluate(prompt, cands)
    P = len(prompt)
    for c, r in zip(cands, resp.results):
        logits = model.forward_prompt(prompt + c[:-1]).cpu().numpy()
        full = sum(float(logits[P - 1 + i, t]) for i, t in enumerate(c))  # summed as the entry point sums
        assert abs(r.score - full) <= tol * max(1.0, abs(full)), (c, r.score, full)


def test_command_line_generate_and_system1():
    folder = helpers.model_folder("A", 7, "float32")
    exe = [sys.executable, os.path.join(ROOT, "bin", "reflex")]
    out = subprocess.run(exe + ["generate", folder, "5,17,3", "--max-tokens", "4", "--weights", "f32",
                                "--prompt-ids", "9,9"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("REFLEX_GENERATE_OK")]
    assert len(lines) == 2 and "num_generated=4" in lines[0] and "weights_dtype=f32" in lines[0]
    ids = [int(t) for t in lines[0].split("token_ids=[")[1].split("]")[0].split(",")]
    want, _ = plain_generate(folder, [5, 17, 3], 4, lambda l, s: pm.argmax_last(l))
    assert ids == want
    out = subprocess.run(exe + ["system1", folder, "5,17,3", "--candidate", "1", "--candidate", "2,3", "--json"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    recs = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert recs[-1]["num_candidates"] == 2 and len(recs) == 3
    bad = subprocess.run(exe + ["generate", folder, "5", "--max-tokens", "0"], capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "error:" in bad.stderr


def test_command_line_smoke_doctor_and_the_top2_probe():
    folder = helpers.model_folder("A", 7, "float32")
    exe = [sys.executable, os.path.join(ROOT, "bin", "reflex")]
    out = subprocess.run(exe + ["smoke"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "REFLEX_SMOKE_OK process_start_to_first_result_ms=" in out.stdout, out.stderr
    out = subprocess.run(exe + ["doctor"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    checks = [l for l in out.stdout.splitlines() if l.startswith("REFLEX_DOCTOR_CHECK")]
    assert any("name=kernel_launch status=pass" in l for l in checks)
    assert out.stdout.strip().splitlines()[-1].startswith("REFLEX_DOCTOR_OK checks_passed=")
    assert subprocess.run(exe + ["doctor", "--what"], capture_output=True, text=True, timeout=300).returncode == 2
    env = dict(os.environ, REFLEX_TOP2_TRACE="1")
    out = subprocess.run(exe + ["generate", folder, "5,17,3", "--max-tokens", "3", "--weights", "f32"],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stderr
    probes = [l for l in out.stderr.splitlines() if l.startswith("REFLEX_TOP2 ")]
    ids = [int(t) for t in out.stdout.split("token_ids=[")[1].split("]")[0].split(",")]
    assert [int(l.split("top1_id=")[1].split()[0]) for l in probes] == ids  # greedy: the top id is the pick


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("B", "bfloat16"), ("A", "float32"), ("C", "bfloat16")])
def test_trace_run_replays_steps_and_writes_logits(name, dtype, tmp_path):
    """bin/trace_run as a subprocess: two requests start together with unequal
    lengths, go on one token a step, the shorter one ends earlier, and a third
    request then starts in the freed slot (the cache holds two requests).  In
    32-bit the files hold the host mirror's bits."""
    V = ALL[name]["vocab_size"]
    folder = helpers.model_folder(name, 7, "float32" if dtype == "float32" else "bfloat16")
    a, b, c = (helpers.random_tokens(n, V, 80 + n) for n in (70, 9, 40))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": list(range(60))},
                                     {"id": "b", "tokens": b[:5], "want": [0, 4]}], "end": []}]
    for i in range(4):
        steps.append({"step": 1 + i, "entries": [{"id": "a", "tokens": [a[60 + i]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + i]], "want": [0]}],
                      "end": ["b"] if i == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "a", "tokens": a[64:70], "want": []}], "end": ["a"]})
    steps.append({"step": 6, "entries": [{"id": "c", "tokens": c, "want": [39]}], "end": ["c"]})
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.split() == [w for i in range(7) for w in ("done", str(i))]
    tol = 3e-6 if dtype == "float32" else 1.5e-2
    ra, rb, rc = (helpers.plain_logits(folder, t) for t in (a, b, c))
    scale = max(np.abs(ra).max(), np.abs(rb).max(), np.abs(rc).max())

    def load(step, rows):
        x = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert x.size == rows * V
        return x.reshape(rows, V)

    x = load(0, 62)
    assert np.abs(x[:60] - ra[:60]).max() < tol * scale
    assert np.abs(x[60:] - rb[[0, 4]]).max() < tol * scale
    for i in range(4):
        x = load(1 + i, 2)
        assert np.abs(x[0] - ra[60 + i]).max() < tol * scale
        assert np.abs(x[1] - rb[5 + i]).max() < tol * scale
    assert not os.path.exists(os.path.join(out_dir, "5.f32"))  # nothing was wanted
    assert np.abs(load(6, 1)[0] - rc[39]).max() < tol * scale
    if dtype == "float32":
        import fp32_mirror

        cfg, w = pm.read_model(folder)
        ma, mc = fp32_mirror.forward(cfg, w, a), fp32_mirror.forward(cfg, w, c)
        assert np.array_equal(load(0, 62)[:60], ma[:60]) and np.array_equal(load(3, 2)[0], ma[62])
        assert np.array_equal(load(6, 1)[0], mc[39])


def test_diagnostics_print_a_decode_steps_timeline():
    """The kernels' own time stamps, read back for a tiny model: one line per
    product of the captured step, in launch order, each later than the last;
    then the attention kernel of each layer, and a CTA's medians per product."""
    import io

    from reflex_b200 import diagnostics
    from tiny_configs import TINY_B

    out = io.StringIO()
    diagnostics.decode_step(batch=2, layers=2, prompt=8, config=dict(TINY_B), out=out)
    tables = out.getvalue().split("\n\n")
    assert len(tables) == 3
    lines = [l.split() for l in tables[0].splitlines()[2:]]
    assert [l[0] for l in lines] == ["qkv", "o", "gate_up", "down"] * 2 + ["head"]
    left = [float(l[-2]) if len(l) > 11 else float(l[-1]) for l in lines]  # released -> left, us
    assert all(0.0 < v < 1000.0 for v in left)
    attention = tables[1].splitlines()
    assert attention[0].split()[0] == "attention" and len(attention) == 1 + 2  # a line per layer
    medians = [l.split()[0] for l in tables[2].splitlines()[1:]]
    assert medians == ["qkv", "o", "gate_up", "down"]


def test_system1_refuses_bad_candidates_and_gives_its_slots_back():
    """A candidate's last id never goes through the step (it only picks a
    logit), so it is checked on the host; and more candidates than free slots
    are refused before any slot is taken."""
    import reflex_b200
    from reflex_b200 import InvalidInput, OutOfMemory

    folder = helpers.model_folder("A", 7, "float32")
    model = reflex_b200.Model.load(folder, weights="f32", max_tokens=1024)
    V = ALL["A"]["vocab_size"]
    for bad in ([1, V], [V + 3], [2, -1]):
        with pytest.raises(InvalidInput):
            model.system1_evaluate([1, 2, 3], [[4, 5], bad])
    assert model.engine.cache.slots.held_count == 0
    small = reflex_b200.Model(model.lm, max_tokens=128)  # two pages: two slots
    with pytest.raises(OutOfMemory):
        small.system1_evaluate([1, 2, 3], [[4], [5], [6]])
    assert small.engine.cache.slots.held_count == 0
    res = model.system1_evaluate([1, 2, 3], [[4, 5], [6]])
    assert len(res.probabilities) == 2


def test_a_device_error_reaches_the_generation_loop_with_the_ids():
    """The device's error word travels to the host with each step's picked ids,
    so the loop learns of a kernel's error without a wait of its own: here a
    bounded wait is made to run out just before a generation call, which must
    raise, give its slots back, and leave the next call working."""
    import reflex_b200
    from reflex_b200 import CudaError, ops

    folder = helpers.model_folder("A", 7, "bfloat16")
    model = reflex_b200.Model.load(folder, weights="bf16", max_tokens=1024)
    good = model.generate([[1, 2, 3], [4, 5]], 5)
    ops.wait_probe(100_000)  # 0.1 ms on a barrier nothing signals: the error word is set
    with pytest.raises(CudaError):
        model.generate([[1, 2, 3], [4, 5]], 5)
    assert model.engine.cache.slots.held_count == 0
    assert model.generate([[1, 2, 3], [4, 5]], 5) == good
