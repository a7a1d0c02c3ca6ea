#!/usr/bin/env python3
"""Decode and prefill throughput at Qwen3-8B layer sizes, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of a batch of 8 sequences (512-token prompts, the
cache sized for a context of 4,096 per sequence).  W untimed decode steps, then
exactly K timed ones between CUDA events with a synchronize on both sides.
The weights (15 GB a step) are far larger than L2, so nothing is flushed
between steps.  Prints ONE JSON line.
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
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes (default: Qwen3-8B)")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens before the decode steps")
    ap.add_argument("--context", type=int, default=CONTEXT, help="cache positions per sequence")
    args = ap.parse_args()
    PROMPT, CONTEXT = args.prompt, max(args.context, args.prompt + args.steps + args.warmup + 64)

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

    import torch

    import reflex_b200
    from reflex_b200 import ops
    from reflex_b200.api import Model
    from reflex_b200.sampling import SamplingParams
    from reflex_b200.weights import random_model_on_device

    cfg = dict(QWEN3_8B)
    cfg.update(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    torch.cuda.set_device(0)
    lm = random_model_on_device(cfg, 0, torch.bfloat16, "cuda:0")
    max_batch = 64 if not args.no_points else args.batch
    model = Model(lm, max_tokens=max(max_batch, args.batch) * CONTEXT, max_batch=max(max_batch, args.batch))
    eng = model.engine
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(1)
    _, weight_bytes, kv_per_tok = model_numbers(cfg, layers)

    def decode_run(batch, steps, warmup, sampler=None):
        """Prefill `batch` prompts of PROMPT tokens, then warmup + steps decode
        steps; returns (ms per step, mean context, launches per step)."""
        prompts = torch.randint(0, V, (batch, PROMPT), generator=g).tolist()
        seqs = [eng.open() for _ in range(batch)]
        logits = eng.step([(s, p, [PROMPT - 1]) for s, p in zip(seqs, prompts)])
        # the picked ids stay on the device and feed the next step (two buffers in turn)
        ids = [torch.empty((batch,), dtype=torch.int32, device="cuda:0") for _ in range(2)]
        scratch = torch.empty((batch * 128,), dtype=torch.float32, device="cuda:0")
        ops.argmax(logits, out=ids[0], scratch=scratch)
        for i in range(warmup):
            logits = eng.step_decode(seqs, ids[i % 2], borrow=True)
            ops.argmax(logits, out=ids[(i + 1) % 2], scratch=scratch)
        launches0 = ops.launch_count()
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
        ms = start.elapsed_time(end) / steps
        mean_ctx = ctx0 + (steps + 1) / 2.0
        for s in seqs:
            eng.close(s)
        per_step = eng.launches_per_decode_step(batch) + 1  # + the argmax
        return ms, mean_ctx, per_step, (t0, t1), ops.launch_count() - launches0

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    ms, mean_ctx, per_step, (t0, t1), _ = decode_run(args.batch, args.steps, args.warmup, sampler)
    clocks = sampler.summary(t0, t1)
    value = args.batch * 1000.0 / ms
    bytes_step = weight_bytes + args.batch * mean_ctx * kv_per_tok
    achieved = bytes_step / (ms * 1e-3) / 1e9

    # end to end through the Python entry point: host ids in, host ids out
    prompts = torch.randint(0, V, (args.batch, PROMPT), generator=g).tolist()
    n_e2e = min(args.steps, 128)
    model.generate(prompts, 4)  # warm
    torch.cuda.synchronize()
    ta = time.perf_counter()
    model.generate(prompts, 1)
    torch.cuda.synchronize()
    tb = time.perf_counter()
    model.generate(prompts, 1 + n_e2e)
    torch.cuda.synchronize()
    tc = time.perf_counter()
    e2e_s = (tc - tb) - (tb - ta)
    from reflex_b200.engine.batch import layout

    _, words = layout(args.batch, args.batch, args.batch)
    e2e = {"value": args.batch * n_e2e / e2e_s, "unit": "tokens/s", "steps": n_e2e,
           "h2d_bytes_per_step": words * 4, "d2h_bytes_per_step": args.batch * 4}

    out = {
        "metric": f"decode tokens/s at batch {args.batch} (Qwen3-{args.shape.upper()} bf16, {PROMPT}-token prompts, "
                  f"context {CONTEXT})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.shape.upper()} layer sizes", "layers": layers, "layers_full_model": full_layers,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"],
            "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "vocab_size": V, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT,
            "mean_context": mean_ctx, "parallelism": "single GPU", "cache_page_tokens": 64,
            "l2": "inputs larger than L2 (15 GB of weights per step), no flush",
            "peaks": pk["source"],
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"]},
    }

    if not args.no_prefill:
        # prefill of one 2,048-token prompt
        prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
        times = []
        for i in range(4):
            s = eng.open()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            eng.step([(s, prompt, [PREFILL_TOKENS - 1])])
            b.record()
            torch.cuda.synchronize()
            eng.close(s)
            if i >= 1:
                times.append(a.elapsed_time(b))
        pms = min(times)
        fl = prefill_flops(cfg, layers, PREFILL_TOKENS)
        out["prefill"] = {"value": PREFILL_TOKENS * 1000.0 / pms, "tokens": PREFILL_TOKENS, "ms": pms,
                          "frac": fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), "flops": fl,
                          "peak_tflops": pk["bf16_tflops"], "of": pk["source"]}
    if not args.no_points:
        points = {}
        for b in (1, 64):
            st = min(args.steps, 64)
            pms_b, _, _, _, _ = decode_run(b, st, 4)
            points[f"decode_b{b}"] = b * 1000.0 / pms_b
        points[f"decode_b{args.batch}"] = value
        out["points"] = points
    sampler.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
