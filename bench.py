#!/usr/bin/env python3
"""Decode and prefill throughput at Qwen3-8B layer sizes, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--arms 8b,14b,32b]

A "step" is one decode step of a batch of 8 sequences (512-token prompts, the
cache sized for a context of 4,096 per sequence).  W untimed decode steps, then
exactly K timed ones between CUDA events with a synchronize on both sides.
The weights (15 GB a step) are far larger than L2, so nothing is flushed
between steps.  Prints ONE JSON line.

Beside the headline the line holds: `e2e` (the same through the Python entry
point, host tokens in and out), `prefill` (one 2,048-token prompt), `points`
(decode at batch 1 and 64 over 256 steps from 512-token prompts, whatever
--steps is; and, unless --arms leaves them out, the two larger workloads: at
Qwen3-14B sizes 16 prompts of seeded lengths in [64, 2048] and 128 steps
sampled at temperature 0.7 through the entry point; at Qwen3-32B sizes batch 32
from 1,024-token prompts over 256 steps and one 8,192-token prefill, the cache
sized to 8,192 a slot), `points_frac` (each point's fraction of its roofline)
and `finite` (every logit of the last timed step is a finite number).
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False,
    "rope_scaling": None, "use_sliding_window": False, "sliding_window": None,
}
# the other sizes of the family, for runs beyond the default (--shape)
SHAPES = {
    "8b": {},
    "14b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "intermediate_size": 17408},
    "32b": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "intermediate_size": 25600},
}
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
POINT_STEPS = 256  # decode steps of the batch 1 / 64 / 32 points: contexts 512 -> 768, as the workload is stated


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        p = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    return p


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "samples": len(sm), "reasons": sorted(reasons)}


def model_numbers(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    weight_bytes = 2 * (layers * per_layer + V * H)  # every matrix a decode step reads, bf16
    kv_bytes_per_token = layers * 2 * nkv * d * 2
    return per_layer, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, layers, T):
    per_layer, _, _ = model_numbers(cfg, layers)
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    gemm = 2.0 * T * (layers * per_layer + cfg["vocab_size"] * cfg["hidden_size"] * (1.0 / T))
    attn = layers * nq * 2.0 * T * T * d  # causal: QK^T and PV, half of the square each
    return gemm + attn


class Arm:
    """One model size on the device with its engine; freed before the next."""

    def __init__(self, shape, layers, max_tokens, max_batch):
        import torch

        from reflex_b200.api import Model
        from reflex_b200.weights import random_model_on_device

        cfg = dict(QWEN3_8B)
        cfg.update(SHAPES[shape])
        self.full_layers = cfg["num_hidden_layers"]
        self.layers = layers or self.full_layers
        cfg["num_hidden_layers"] = self.layers
        self.cfg, self.shape = cfg, shape
        lm = random_model_on_device(cfg, 0, torch.bfloat16, "cuda:0")
        self.model = Model(lm, max_tokens=max_tokens, max_batch=max_batch)
        self.eng = self.model.engine
        self.V = cfg["vocab_size"]
        self.g = torch.Generator().manual_seed(1)
        _, self.weight_bytes, self.kv_per_tok = model_numbers(cfg, self.layers)

    def free(self):
        import gc

        import torch

        self.model = self.eng = None
        gc.collect()
        torch.cuda.empty_cache()

    def decode_run(self, batch, prompt_len, steps, warmup, sampler=None):
        """Prefill `batch` prompts of `prompt_len` tokens, then warmup + steps
        greedy decode steps fed from the device; returns a dict."""
        import torch

        from reflex_b200 import ops

        eng = self.eng
        prompts = torch.randint(0, self.V, (batch, prompt_len), generator=self.g).tolist()
        seqs = [eng.open() for _ in range(batch)]
        logits = eng.step([(s, p, [prompt_len - 1]) for s, p in zip(seqs, prompts)])
        # the picked ids stay on the device and feed the next step (two buffers in turn)
        ids = [torch.empty((batch,), dtype=torch.int32, device="cuda:0") for _ in range(2)]
        scratch = torch.empty((batch * 128,), dtype=torch.float32, device="cuda:0")
        ops.argmax(logits, out=ids[0], scratch=scratch)
        for i in range(warmup):
            logits = eng.step_decode(seqs, ids[i % 2], borrow=True)
            ops.argmax(logits, out=ids[(i + 1) % 2], scratch=scratch)
        ctx0 = eng.length(seqs[0])
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = sampler.mark() if sampler else 0
        start.record()
        for i in range(warmup, warmup + steps):
            logits = eng.step_decode(seqs, ids[i % 2], borrow=True)
            ops.argmax(logits, out=ids[(i + 1) % 2], scratch=scratch)
        end.record()
        torch.cuda.synchronize()
        t1 = sampler.mark() if sampler else 0
        finite = bool(torch.isfinite(logits).all().item())  # after the timed region
        eng.check_errors()
        ms = start.elapsed_time(end) / steps
        mean_ctx = ctx0 + (steps + 1) / 2.0
        for s in seqs:
            eng.close(s)
        bytes_step = self.weight_bytes + batch * mean_ctx * self.kv_per_tok
        return {"ms": ms, "tok_s": batch * 1000.0 / ms, "mean_ctx": mean_ctx, "marks": (t0, t1),
                "launches": eng.launches_per_decode_step(batch) + 1,  # + the argmax
                "gbs": bytes_step / (ms * 1e-3) / 1e9, "finite": finite}

    def prefill_run(self, tokens, repeats=3):
        """One prompt of `tokens` tokens in one step; the best of `repeats` after a warm-up."""
        import torch

        eng = self.eng
        prompt = torch.randint(0, self.V, (tokens,), generator=self.g).tolist()
        times, finite = [], True
        for i in range(repeats + 1):
            s = eng.open()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            logits = eng.step([(s, prompt, [tokens - 1])])
            b.record()
            torch.cuda.synchronize()
            finite = finite and bool(torch.isfinite(logits).all().item())
            eng.close(s)
            if i >= 1:
                times.append(a.elapsed_time(b))
        eng.check_errors()
        pms = min(times)
        fl = prefill_flops(self.cfg, self.layers, tokens)
        return {"ms": pms, "tok_s": tokens * 1000.0 / pms, "flops": fl, "tflops": fl / (pms * 1e-3) / 1e12,
                "finite": finite}

    def generate_run(self, prompts, new_tokens, sampling=None):
        """Decode tokens a second through the entry point: the time of
        1 + new_tokens tokens a prompt less the time of 1 (the prefill and the
        first pick), host ids in and out."""
        import torch

        m = self.model
        m.generate(prompts, 3, sampling)  # warm: allocations, graphs of the first sizes
        torch.cuda.synchronize()
        ta = time.perf_counter()
        m.generate(prompts, 1, sampling)
        torch.cuda.synchronize()
        tb = time.perf_counter()
        out = m.generate(prompts, 1 + new_tokens, sampling)
        torch.cuda.synchronize()
        tc = time.perf_counter()
        s = (tc - tb) - (tb - ta)
        n = sum(len(o) - 1 for o in out)
        return {"tok_s": n / s, "seconds": s, "tokens": n, "steps": new_tokens}


def main() -> int:
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 decode points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes of the headline (default: Qwen3-8B)")
    ap.add_argument("--arms", default="8b,14b,32b",
                    help="workloads beside the headline: 14b and 32b add their points (default: all)")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens before the decode steps")
    ap.add_argument("--context", type=int, default=CONTEXT, help="cache positions per sequence")
    args = ap.parse_args()
    PROMPT = args.prompt
    CONTEXT = max(args.context, args.prompt + max(args.steps, 0 if args.no_points else POINT_STEPS) + args.warmup + 64)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "lateos-ai/reflex is a Rust crate (no setup.py/pyproject.toml; pip: 'Directory is "
                          "not installable') and no Rust toolchain exists in this image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: --gpus {args.gpus} is not supported (this library is single-GPU)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    arms = [a for a in args.arms.split(",") if a]
    for a in arms:
        if a not in SHAPES:
            print(f"--arms: unknown workload {a!r}; known: {sorted(SHAPES)}")
            return 2

    import torch

    from reflex_b200.engine.batch import layout
    from reflex_b200.sampling import SamplingParams

    pk = peaks()
    torch.cuda.set_device(0)
    max_batch = max(args.batch, 1 if args.no_points else 64)
    arm = Arm(args.shape, args.layers, max_batch * CONTEXT, max_batch)
    cfg, layers = arm.cfg, arm.layers

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    head = arm.decode_run(args.batch, PROMPT, args.steps, args.warmup, sampler)
    clocks = sampler.summary(*head["marks"])
    finite = head["finite"]

    # end to end through the Python entry point: host ids in, host ids out
    prompts = torch.randint(0, arm.V, (args.batch, PROMPT), generator=arm.g).tolist()
    n_e2e = min(args.steps, 128)
    gen = arm.generate_run(prompts, n_e2e)
    _, words = layout(args.batch, args.batch, args.batch)
    e2e = {"value": gen["tok_s"], "unit": "tokens/s", "steps": n_e2e,
           "h2d_bytes_per_step": words * 4, "d2h_bytes_per_step": args.batch * 4}

    out = {
        "metric": f"decode tokens/s at batch {args.batch} (Qwen3-{args.shape.upper()} bf16, {PROMPT}-token prompts, "
                  f"context {CONTEXT})",
        "value": head["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.shape.upper()} layer sizes", "layers": layers, "layers_full_model": arm.full_layers,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"],
            "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "vocab_size": arm.V, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT,
            "mean_context": head["mean_ctx"], "parallelism": "single GPU", "cache_page_tokens": 64,
            "l2": "inputs larger than L2 (15 GB of weights per step), no flush",
            "peaks": pk["source"], "points_steps": POINT_STEPS, "arms": ",".join(arms),
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": head["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["gbs"] / pk["hbm_gbs"], "of": pk["source"]},
    }

    if not args.no_prefill:
        p = arm.prefill_run(PREFILL_TOKENS)
        finite = finite and p["finite"]
        out["prefill"] = {"value": p["tok_s"], "tokens": PREFILL_TOKENS, "ms": p["ms"],
                          "frac": p["tflops"] / pk["bf16_tflops"], "flops": p["flops"],
                          "peak_tflops": pk["bf16_tflops"], "of": pk["source"]}
    points, fracs = {}, {}
    if not args.no_points:
        for b in (1, 64):
            r = arm.decode_run(b, PROMPT, POINT_STEPS, 4)
            finite = finite and r["finite"]
            points[f"decode_b{b}"] = r["tok_s"]
            fracs[f"decode_b{b}"] = r["gbs"] / pk["hbm_gbs"]
        points[f"decode_b{args.batch}"] = head["tok_s"]
        fracs[f"decode_b{args.batch}"] = head["gbs"] / pk["hbm_gbs"]
    arm.free()
    del arm

    if not args.no_points:
        try:
            if "14b" in arms and args.shape == "8b":
                # 16 prompts of seeded lengths in [64, 2048], 128 steps at temperature 0.7, context 4,096
                a14 = Arm("14b", 0, 16 * 4096, 16)
                lens = torch.randint(64, 2049, (16,), generator=torch.Generator().manual_seed(14)).tolist()
                ps = [torch.randint(0, a14.V, (n,), generator=a14.g).tolist() for n in lens]
                r = a14.generate_run(ps, 128, SamplingParams(temperature=0.7, seed=14))
                ctx_sum = sum(n + 1 + 64.5 for n in lens)
                gbs = (a14.weight_bytes + ctx_sum * a14.kv_per_tok) / (r["seconds"] / r["steps"]) / 1e9
                points["qwen3_14b_b16_unequal_t0.7_decode"] = r["tok_s"]
                fracs["qwen3_14b_b16_unequal_t0.7_decode"] = gbs / pk["hbm_gbs"]
                a14.free()
                del a14
            if "32b" in arms and args.shape == "8b":
                # batch 32 from 1,024-token prompts over 256 steps; one 8,192-token prefill; 8,192 a slot
                a32 = Arm("32b", 0, 32 * 8192, 32)
                r = a32.decode_run(32, 1024, POINT_STEPS, 4)
                p = a32.prefill_run(8192, repeats=2)
                finite = finite and r["finite"] and p["finite"]
                points["qwen3_32b_b32_decode"] = r["tok_s"]
                fracs["qwen3_32b_b32_decode"] = r["gbs"] / pk["hbm_gbs"]
                points["qwen3_32b_prefill_8192"] = p["tok_s"]
                fracs["qwen3_32b_prefill_8192"] = p["tflops"] / pk["bf16_tflops"]
                a32.free()
                del a32
        except Exception as e:  # the headline stands; the point that failed says why
            points["error"] = f"{type(e).__name__}: {e}"[:300]
        out["points"] = points
        out["points_frac"] = fracs
    out["finite"] = finite
    sampler.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
