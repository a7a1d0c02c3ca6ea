"""The command line, in the manner of `reflex <subcommand>`
(src/bin/reflex/main.rs:36-50): `generate`, `system1`, `check`, `bench`,
`smoke`, `doctor`, with the reference's option names and meanings where it has
them (src/bin/reflex/generate.rs:186-250, system1.rs:88-107, check.rs:42-78,
bench.rs:50-55, smoke.rs:1-16, doctor.rs:1-40).  A model is a folder (config.json + safetensors) instead of a
GGUF file, and prompts and candidates are comma-separated token ids instead of
text, since this library has no tokenizer.  Results are one `KEY=value` line
per command (`REFLEX_GENERATE_OK ...`), or one JSON line with `--json`; errors
are `error: <message>` and exit code 1 (src/bin/reflex/main.rs:56-59).
"""

from __future__ import annotations

import json
import sys
import time
from typing import List, Optional

USAGE = """usage: reflex <subcommand> ...
  generate <model-dir> [prompt-ids] [--max-tokens N] [--temperature F] [--top-k N] [--top-p F]
           [--seed N] [--stop-ids a,b] [--weights bf16|f32] [--prompt-ids a,b,c]... [--json]
  system1  <model-dir> <prompt-ids> --candidate a,b [--candidate c]... [--temperature T]
           [--weights bf16|f32] [--json]
  check    <model-dir> <prompt-ids> [--max-tokens N] [--reference file] [--tolerance F]
  bench    <model-dir> [--warmup N] [--iters N] [--weights bf16|f32]
  random   <config.json> <out-dir> [--seed N] [--dtype bfloat16|float32]
  smoke    [--json]      one kernel through the whole path: build, load, launch, check
  doctor   [--json]      is this machine set up for the library? (exit 0 / 1 / 2)
prompt-ids and candidates are comma-separated token ids."""

DEFAULT_PROMPT = [1, 2, 3, 4]


def fail(msg: str) -> "NoReturn":
    print(f"error: {msg}", file=sys.stderr)
    sys.exit(1)


def parse_ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(" ", "").split(",") if t != ""]
    except ValueError:
        fail(f"token ids must be comma-separated integers, got {text!r}")


class Args:
    def __init__(self, argv: List[str], flags_with_value, flags_bool):
        self.positional: List[str] = []
        self.values = {}
        self.multi = {}
        self.bools = set()
        it = iter(argv)
        for a in it:
            if a in flags_bool:
                self.bools.add(a)
            elif a in flags_with_value:
                try:
                    v = next(it)
                except StopIteration:
                    fail(f"{a} requires a value")
                self.values[a] = v
                self.multi.setdefault(a, []).append(v)
            elif a.startswith("--"):
                fail(f"unknown option {a}\n{USAGE}")
            else:
                self.positional.append(a)

    def num(self, flag, kind, default):
        if flag not in self.values:
            return default
        try:
            return kind(self.values[flag])
        except ValueError:
            fail(f"{flag} must be a number, got {self.values[flag]!r}")


def resolve_weights(flag: Optional[str], default: str = "bf16") -> str:
    from .api import resolve_weights as resolve
    from .errors import InvalidInput

    try:
        return resolve(flag, default)
    except InvalidInput as e:
        fail(str(e))


def _load(path: str, weights: str, **kw):
    from .api import Model

    t = time.perf_counter()
    model = Model.load(path, weights=weights, **kw)
    return model, (time.perf_counter() - t) * 1000.0


def cmd_generate(argv: List[str], t0: float) -> int:
    from .sampling import SamplingParams

    a = Args(argv, {"--max-tokens", "--temperature", "--top-k", "--top-p", "--seed", "--weights",
                    "--stop-ids", "--prompt-ids"}, {"--json"})
    if not a.positional:
        fail(USAGE)
    path = a.positional[0]
    prompts = [parse_ids(p) for p in a.positional[1:2]] + [parse_ids(p) for p in a.multi.get("--prompt-ids", [])]
    if not prompts:
        prompts = [DEFAULT_PROMPT]
    max_tokens = a.num("--max-tokens", int, 1)  # the reference's default (generate.rs:174)
    if max_tokens == 0:
        fail("--max-tokens must be at least 1")
    sampling = SamplingParams(
        temperature=a.num("--temperature", float, 0.0), top_k=a.num("--top-k", int, None),
        top_p=a.num("--top-p", float, None), seed=a.num("--seed", int, None),
        stop_token_ids=tuple(parse_ids(a.values.get("--stop-ids", ""))))
    model, load_ms = _load(path, resolve_weights(a.values.get("--weights")))
    first = {}
    t_gen = time.perf_counter()

    def on_token(i, tok):
        if not first:
            first["ms"] = (time.perf_counter() - t0) * 1000.0

    outs = model.generate(prompts, max_tokens, sampling, on_token=on_token)
    total_ms = (time.perf_counter() - t0) * 1000.0
    gen_ms = (time.perf_counter() - t_gen) * 1000.0
    for i, ids in enumerate(outs):
        if "--json" in a.bools:
            print(json.dumps({
                "schema_version": 1, "request": i,
                "process_start_to_first_token_ms": first.get("ms", total_ms),
                "process_start_to_last_token_ms": total_ms, "model_load_ms": load_ms,
                "generate_ms": gen_ms, "num_generated": len(ids), "token_id": ids[0],
                "token_ids": ids, "weights_dtype": model.weights_dtype}))
        else:
            print(f"REFLEX_GENERATE_OK request={i} process_start_to_first_token_ms={first.get('ms', total_ms):.3f} "
                  f"process_start_to_last_token_ms={total_ms:.3f} model_load_ms={load_ms:.3f} "
                  f"generate_ms={gen_ms:.3f} num_generated={len(ids)} token_id={ids[0]} "
                  f"token_ids=[{','.join(str(t) for t in ids)}] weights_dtype={model.weights_dtype}")
    return 0


def cmd_system1(argv: List[str], t0: float) -> int:
    a = Args(argv, {"--candidate", "--temperature", "--weights"}, {"--json"})
    if len(a.positional) < 2:
        fail(USAGE)
    cands = [parse_ids(c) for c in a.multi.get("--candidate", [])]
    if not cands:
        fail("system1 requires at least one --candidate")
    model, load_ms = _load(a.positional[0], resolve_weights(a.values.get("--weights")))
    resp = model.system1_evaluate(parse_ids(a.positional[1]), cands, a.num("--temperature", float, 1.0))
    total_ms = (time.perf_counter() - t0) * 1000.0
    for idx, (r, p) in enumerate(zip(resp.results, resp.probabilities)):
        if "--json" in a.bools:
            print(json.dumps({"schema_version": 1, "idx": idx, "token_ids": r.token_ids,
                              "score": r.score, "probability": p}))
        else:
            print(f"REFLEX_SYSTEM1_CANDIDATE_OK idx={idx} token_ids=[{','.join(map(str, r.token_ids))}] "
                  f"score={r.score:.6f} probability={p:.6f}")
    if "--json" in a.bools:
        print(json.dumps({"schema_version": 1, "process_start_to_result_ms": total_ms,
                          "model_load_ms": load_ms, "num_candidates": len(cands),
                          "best_idx": resp.best_idx, "entropy": resp.entropy,
                          "weights_dtype": model.weights_dtype}))
    else:
        print(f"REFLEX_SYSTEM1_OK process_start_to_result_ms={total_ms:.3f} model_load_ms={load_ms:.3f} "
              f"num_candidates={len(cands)} best_idx={resp.best_idx} entropy={resp.entropy:.6f} "
              f"weights_dtype={model.weights_dtype}")
    return 0


def cmd_check(argv: List[str], t0: float) -> int:
    """Greedy ids and the first token's logit checksum against a reference
    file: line 1 comma-separated ids, optional line 2 the checksum; exit 0 on
    a match, 1 on a mismatch, 2 when there is nothing to compare with
    (src/bin/reflex/check.rs:15-30, 160-187, 217-248).  Defaults to f32
    weights, as the reference's `check` does."""
    a = Args(argv, {"--max-tokens", "--reference", "--tolerance", "--weights"}, set())
    if len(a.positional) < 2:
        fail(USAGE)
    model, _ = _load(a.positional[0], resolve_weights(a.values.get("--weights"), default="f32"))
    prompt = parse_ids(a.positional[1])
    n = a.num("--max-tokens", int, 16)
    logits = model.forward_prompt(prompt)[-1].double()
    checksum = float(logits.sum())
    top1 = float(logits.max())
    ids = model.generate(prompt, n)
    print(f"REFLEX_CHECK token_ids=[{','.join(map(str, ids))}] num_generated={len(ids)} "
          f"logit_checksum={checksum:.6f} top1_logit={top1:.6f} vocab_size={logits.numel()} "
          f"weights_dtype={model.weights_dtype}")
    ref = a.values.get("--reference")
    if ref is None:
        return 2
    with open(ref) as f:
        lines = [l.strip() for l in f.read().splitlines() if l.strip()]
    want = parse_ids(lines[0])
    ok = want == ids
    if len(lines) > 1:
        tol = a.num("--tolerance", float, 1e-2)
        want_sum = float(lines[1])
        ok = ok and abs(checksum - want_sum) <= tol * max(1.0, abs(want_sum))
    print("REFLEX_CHECK_OK" if ok else "REFLEX_CHECK_MISMATCH")
    return 0 if ok else 1


def cmd_bench(argv: List[str], t0: float) -> int:
    """Warm prefill latency at three prompt lengths and decode ms/token over 16
    steps (src/bin/reflex/bench.rs:50-55, 298-361)."""
    import statistics

    import torch

    a = Args(argv, {"--warmup", "--iters", "--weights"}, set())
    if not a.positional:
        fail(USAGE)
    model, load_ms = _load(a.positional[0], resolve_weights(a.values.get("--weights")))
    warmup, iters = a.num("--warmup", int, 2), a.num("--iters", int, 5)
    V = model.spec.vocab_size
    g = torch.Generator().manual_seed(0)
    decode_steps = 16
    for length in (24, 96, 384):
        if length + decode_steps + 1 > model.spec.max_positions:
            continue
        prompt = torch.randint(0, V, (length,), generator=g).tolist()
        pre, dec = [], []
        for it in range(warmup + iters):
            torch.cuda.synchronize()
            t = time.perf_counter()
            model.generate(prompt, 1)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            model.generate(prompt, 1 + decode_steps)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            if it >= warmup:
                pre.append((t1 - t) * 1000.0)
                dec.append(((t2 - t1) - (t1 - t)) * 1000.0 / decode_steps)
        p50 = statistics.median(pre)
        d50 = statistics.median(dec)
        print(f"REFLEX_BENCH_OK prompt_tokens={length} prefill_p50_ms={p50:.3f} "
              f"decode_ms_per_token={d50:.3f} tokens_per_sec={1000.0 / d50:.1f} "
              f"weights_dtype={model.weights_dtype}")
    return 0


def cmd_random(argv: List[str], t0: float) -> int:
    from .weights import write_random_model

    a = Args(argv, {"--seed", "--dtype"}, set())
    if len(a.positional) < 2:
        fail(USAGE)
    with open(a.positional[0]) as f:
        cfg = json.load(f)
    out = write_random_model(cfg, a.num("--seed", int, 0), a.positional[1], a.values.get("--dtype", "bfloat16"))
    print(f"REFLEX_RANDOM_OK model_dir={out}")
    return 0


def cmd_smoke(argv: List[str], t0: float) -> int:
    """The first thing to run on a fresh machine: builds (if needed) and loads
    the kernel library, launches one kernel and checks its result; reports the
    time from process start to that first result (src/bin/reflex/smoke.rs:1-16,
    :105)."""
    a = Args(argv, set(), {"--json"})
    import torch

    from . import ops

    if not torch.cuda.is_available():
        fail("smoke: no CUDA device")
    x = torch.arange(1, 65, dtype=torch.float32, device="cuda:0").reshape(1, 64)
    w = torch.ones(64, dtype=torch.float32, device="cuda:0")
    y = ops.rmsnorm(x, w, 0.0, torch.float32)
    want = x / torch.sqrt((x * x).mean())
    ok = bool(torch.allclose(y, want, rtol=1e-6, atol=0))
    ms = (time.perf_counter() - t0) * 1000.0
    if not ok:
        fail("smoke: the kernel's result is wrong")
    if "--json" in a.bools:
        print(json.dumps({"ok": True, "process_start_to_first_result_ms": round(ms, 3)}))
    else:
        print(f"REFLEX_SMOKE_OK process_start_to_first_result_ms={ms:.3f}")
    return 0


def cmd_doctor(argv: List[str], t0: float) -> int:
    """A health report of the GPU and the toolchain, no model involved
    (src/bin/reflex/doctor.rs:1-40): one `REFLEX_DOCTOR_CHECK name= status=
    detail=` line per check, then `REFLEX_DOCTOR_OK` (exit 0; warnings allowed)
    or `REFLEX_DOCTOR_FAIL` (exit 1)."""
    if any(x not in ("--json",) for x in argv):
        print(USAGE, file=sys.stderr)
        return 2
    as_json = "--json" in argv
    checks = []

    def add(name, status, detail):
        checks.append({"name": name, "status": status, "detail": detail})
        if as_json:
            print(json.dumps({"check": name, "status": status, "detail": detail}))
        else:
            print(f"REFLEX_DOCTOR_CHECK name={name} status={status} detail={json.dumps(detail)}")

    import torch

    gpu = torch.cuda.is_available()
    if gpu:
        props = torch.cuda.get_device_properties(0)
        add("cuda_device", "pass", f"{props.name}, {props.total_memory >> 20} MiB, {props.multi_processor_count} SMs")
        cc = f"{props.major}.{props.minor}"
        add("compute_capability", "pass" if (props.major, props.minor) == (10, 0) else "fail",
            f"device {cc}, kernels are built for sm_100a")
    else:
        add("cuda_device", "fail", "no CUDA device is visible")
    try:
        from .csrc import build

        add("compiler", "pass", build.find_nvcc())
    except RuntimeError as e:
        add("compiler", "warn", f"{e} (only needed when the library has to be rebuilt)")
    try:
        from .csrc import build

        add("kernel_library", "pass", build.ensure_built())
    except Exception as e:  # a report, not a crash
        add("kernel_library", "fail", str(e))
    if gpu and checks[-1]["status"] == "pass":
        try:
            from . import ops

            g = torch.Generator().manual_seed(0)
            x = torch.randn(4, 256, generator=g).bfloat16().cuda()
            w = torch.randn(384, 256, generator=g).bfloat16().cuda()
            y = ops.gemm_tc(x, w, torch.float32)
            ops.check_device_errors("cuda:0")
            err = float((y - x.float() @ w.float().T).abs().max())
            add("kernel_launch", "pass" if err < 1e-2 else "fail",
                f"tcgen05 product 4x256x384, largest difference to the library product {err:.2e}")
        except Exception as e:
            add("kernel_launch", "fail", str(e))
        free, total = torch.cuda.mem_get_info(0)
        add("device_memory", "pass" if free > (1 << 30) else "warn", f"{free >> 20} of {total >> 20} MiB free")
    try:
        import pynvml  # noqa: F401

        add("nvml", "pass", "pynvml importable (clocks and power can be sampled)")
    except Exception:
        add("nvml", "warn", "pynvml not importable; nvidia-smi is used for clocks where needed")
    n = {k: sum(c["status"] == k for c in checks) for k in ("pass", "warn", "fail")}
    ok = n["fail"] == 0
    if as_json:
        print(json.dumps({"ok": ok, "checks_passed": n["pass"], "checks_warned": n["warn"], "checks_failed": n["fail"]}))
    else:
        print(f"REFLEX_DOCTOR_{'OK' if ok else 'FAIL'} checks_passed={n['pass']} checks_warned={n['warn']} "
              f"checks_failed={n['fail']}")
    return 0 if ok else 1


def main(argv: Optional[List[str]] = None) -> int:
    t0 = time.perf_counter()
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(USAGE)
        return 0 if argv else 1
    from .errors import ReflexError

    cmds = {"generate": cmd_generate, "system1": cmd_system1, "check": cmd_check,
            "bench": cmd_bench, "random": cmd_random, "smoke": cmd_smoke, "doctor": cmd_doctor}
    if argv[0] not in cmds:
        fail(f"unknown subcommand {argv[0]!r}\n{USAGE}")
    try:
        return cmds[argv[0]](argv[1:], t0)
    except ReflexError as e:
        fail(f"{argv[0]}: {e}")
    except OSError as e:
        fail(f"{argv[0]}: {e}")


if __name__ == "__main__":
    sys.exit(main())
