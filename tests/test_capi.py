"""The engine's C interface, driven by a C program (tests/capi/smoke.c) as the
reference's is by ffi-test/smoke_test.c: error codes without a GPU; on a GPU,
generation, steps and scoring compared with the Python entry point."""

import os
import re
import subprocess
import tempfile

import pytest

import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def smoke_program():
    from reflex_b200.capi import build

    lib = build.ensure_built()
    exe = os.path.join(tempfile.mkdtemp(prefix="rfx_capi_"), "smoke")
    cmd = ["gcc", "-O1", "-Wall", "-Werror", f"-I{os.path.dirname(build.HEADER)}",
           os.path.join(ROOT, "tests", "capi", "smoke.c"), "-o", exe,
           f"-L{os.path.dirname(lib)}", "-lreflex_b200_engine", f"-Wl,-rpath,{os.path.dirname(lib)}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def _env():
    env = dict(os.environ)
    env["REFLEX_B200_ROOT"] = ROOT
    return env


def test_error_codes_need_no_gpu(smoke_program):
    res = subprocess.run([smoke_program], capture_output=True, text=True, timeout=300, env=_env())
    assert res.returncode == 0, res.stderr
    assert "RFX_CAPI_ERROR_CODES_OK" in res.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("weights", ["f32", "bf16"])
def test_generate_step_and_score_match_the_python_entry_point(smoke_program, weights):
    import reflex_b200

    folder = helpers.model_folder("B", 7, "float32" if weights == "f32" else "bfloat16")
    res = subprocess.run([smoke_program, folder, weights], capture_output=True, text=True, timeout=600,
                         env=_env())
    assert res.returncode == 0, res.stdout + res.stderr
    assert "RFX_CAPI_OK" in res.stdout
    got = [[int(t) for t in m.group(1).split(",")]
           for m in re.finditer(r"RFX_CAPI_GENERATE seq=\d+ token_ids=\[([\d,]*)\]", res.stdout)]
    model = reflex_b200.Model.load(folder, weights=weights, max_tokens=4096, max_batch=4)
    prompts = [[5, 17, 3, 9], [11, 2]]
    assert got == model.generate(prompts, 6)
    scores = [float(m.group(1)) for m in re.finditer(r"RFX_CAPI_SCORE idx=\d+ score=(\S+)", res.stdout)]
    want = model.system1_evaluate(prompts[0], [[7], [8, 9]], 1.0)
    assert len(scores) == 2
    for a, b in zip(scores, (r.score for r in want.results)):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(b))
    best = int(re.search(r"RFX_CAPI_SCORE_OK best_idx=(\d+)", res.stdout).group(1))
    assert best == want.best_idx


def test_the_ctypes_client_turns_failures_into_the_librarys_exceptions():
    """The same interface from Python through ctypes: a failure comes back as the
    exception its stable category number names, with the C side's message."""
    import reflex_b200
    from reflex_b200.capi.client import CModel

    with pytest.raises(reflex_b200.ReflexError) as e:
        CModel.load("/nonexistent/model/folder")
    assert e.value.code in (1, 10) and "nonexistent" in str(e.value)


@pytest.mark.gpu
def test_the_ctypes_client_generates_scores_and_steps_like_the_python_entry_point():
    import numpy as np

    import reflex_b200
    from reflex_b200.capi.client import CModel

    folder = helpers.model_folder("B", 7, "bfloat16")
    prompts = [[5, 17, 3, 9], [11, 2]]
    model = reflex_b200.Model.load(folder, weights="bf16", max_tokens=4096, max_batch=4)
    with CModel.load(folder, "bf16", 4096, 4) as c:
        assert c.generate(prompts, 6) == model.generate(prompts, 6)
        rows, best, entropy = c.score(prompts[0], [[7], [8, 9]], 1.0)
        want = model.system1_evaluate(prompts[0], [[7], [8, 9]], 1.0)
        assert best == want.best_idx and abs(entropy - want.entropy) < 1e-5
        for (s, p), r, wp in zip(rows, want.results, want.probabilities):
            assert abs(s - r.score) <= 1e-5 * max(1.0, abs(r.score)) and abs(p - wp) < 1e-5
        seq = c.open_sequence()
        logits = np.array(c.step([(seq, prompts[0], [3])]), dtype=np.float32)
        c.close_sequence(seq)
        s2 = model.engine.open()  # the same step through the Python engine: the same kernels, the same bits
        ref = model.engine.step([(s2, prompts[0], [3])]).cpu().numpy()
        model.engine.close(s2)
        assert logits.shape == ref.shape and np.array_equal(logits, ref)
        with pytest.raises(reflex_b200.InvalidInput):
            c.generate(prompts, 0)
