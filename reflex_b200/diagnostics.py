"""Device-side timelines of the kernels a step's time goes to.

Two of the kernels can record `%globaltimer` stamps of chosen moments of a
CTA's life into a buffer (`rfx_gemm_trace`, `rfx_attention_prefill_tc_trace`;
off unless a buffer is given).  This module drives them on random weights of
a configuration's sizes and prints what the stamps say, so that a figure such
as "1.2 us between one kernel's last exit and the next one's release" can be
taken again:

    python -m reflex_b200.diagnostics decode-step [--batch 8] [--layers 3]
    python -m reflex_b200.diagnostics prefill-attention [--tokens 2048]
    python -m reflex_b200.diagnostics decode-attention [--cases 64x640,8x4096]

The third times the decode attention kernel alone with CUDA events, for each
(batch x context) case at every number of key splits, beside the number the
split model (`ops.decode_splits`) picks: the figures that model is fitted to.

The reference times phases of a step with CUDA events
(src/model/prefill_profile.rs:26-59, `REFLEX_PREFILL_PROFILE`); stamps written
by the kernels themselves also show what happens inside and between launches
of a captured graph, where events cannot be placed.
"""

from __future__ import annotations

import argparse
import ctypes
import sys
from typing import Dict, List

import numpy as np
import torch

# Qwen3-8B layer sizes unless --config names a config.json
DEFAULT_CONFIG: Dict = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096,
    "intermediate_size": 12288, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "num_hidden_layers": 36, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
    "tie_word_embeddings": False, "max_position_embeddings": 40960,
}


def _config(path: str) -> Dict:
    if not path:
        return dict(DEFAULT_CONFIG)
    import json

    with open(path, encoding="utf-8") as f:
        return json.load(f)


def decode_step(batch: int, layers: int, prompt: int, config: Dict, out=sys.stdout) -> None:
    """Stamps of the product kernels of one captured decode step, launch by
    launch: when its CTAs entered, when the wait on the kernel before them
    let them go, when their accumulators were complete, when they left."""
    from . import ops
    from .engine import Engine
    from .ops import native
    from .weights import random_model_on_device

    cfg = dict(config)
    cfg["num_hidden_layers"] = layers
    lm = random_model_on_device(cfg, 0, torch.bfloat16, "cuda:0")
    eng = Engine(lm, max_tokens=batch * (prompt + 128))
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg["vocab_size"], (batch, prompt), generator=g).tolist()
    seqs = [eng.open() for _ in range(batch)]
    logits = eng.step([(s, p, [prompt - 1]) for s, p in zip(seqs, prompts)])
    ids = ops.argmax(logits).tolist()
    lib = native.lib()
    lib.rfx_gemm_trace.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    n_launch, n_cta = 4 * layers + 1, 1200
    buf = torch.zeros((n_launch * n_cta * 8,), dtype=torch.int64, device="cuda:0")
    abuf = torch.zeros((layers * n_cta * 12,), dtype=torch.int64, device="cuda:0")
    lib.rfx_attention_decode_trace.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    from .engine.graphs import DecodeGraph

    for i in range(6):
        if i == DecodeGraph.WARMUP:  # this call captures the step's graph: its launches get trace ids from 0
            lib.rfx_gemm_trace(buf.data_ptr(), n_launch, n_cta)
            lib.rfx_attention_decode_trace(abuf.data_ptr(), layers, n_cta)
        logits = eng.step([(s, [t], [0]) for s, t in zip(seqs, ids)])
        ids = ops.argmax(logits).tolist()
    torch.cuda.synchronize()
    lib.rfx_gemm_trace(0, 0, 0)
    lib.rfx_attention_decode_trace(0, 0, 0)
    ta = abuf.cpu().numpy().reshape(layers, n_cta, 12).astype(np.float64)
    t = buf.cpu().numpy().reshape(n_launch, n_cta, 8).astype(np.float64)
    t0 = t[t > 0].min()
    names = ["qkv", "o", "gate_up", "down"]
    print(f"decode step, batch {batch}, context {prompt}+, {layers} layers; times in us from the first stamp "
          "of the last replay", file=out)
    print(f"{'product':8s} {'CTAs':>5s} {'entered':>17s} {'released':>17s} {'sums done':>17s} {'left':>17s} "
          f"{'released->left':>14s} {'gap before':>10s}", file=out)
    prev_exit = None
    for launch in range(n_launch):
        rec = t[launch]
        used = rec[:, 0] > 0
        if not used.any():
            continue
        r = (rec[used] - t0) / 1e3
        name = names[launch % 4] if launch < 4 * layers else "head"
        span = lambda c: f"{r[:, c].min():8.2f}..{r[:, c].max():7.2f}"
        gap = "" if prev_exit is None else f"{r[:, 1].min() - prev_exit:10.2f}"
        print(f"{name:8s} {int(used.sum()):5d} {span(0)} {span(1)} {span(2)} {span(3)} "
              f"{r[:, 3].max() - r[:, 1].min():14.2f} {gap}", file=out)
        prev_exit = r[:, 3].max()
    # the attention kernel between a layer's qkv and o products, in the same clock
    print(f"\n{'attention':9s} {'CTAs':>5s} {'entered':>17s} {'released':>17s} {'query rows':>17s} {'pages done':>17s} "
          f"{'warps merged':>17s} {'left':>17s}", file=out)
    for launch in range(layers):
        rec = ta[launch]
        used = rec[:, 0] > 0
        if not used.any():
            continue
        r = (rec[used] - t0) / 1e3
        span = lambda c: f"{r[:, c].min():8.2f}..{r[:, c].max():7.2f}"
        print(f"{'':9s} {int(used.sum()):5d} {span(0)} {span(1)} {span(2)} {span(3)} {span(4)} {span(6)}", file=out)
    # A CTA's own spans (medians over the CTAs of the layers' launches, us): the
    # main loop, then the epilogue's parts.  With the K dimension split over a
    # cluster: partial rows pushed to their owners, the cluster's barrier, the
    # sum and store; with one CTA a tile: the first 16 columns, the rest.
    print(f"\n{'product':8s} {'main loop':>10s} {'push / first':>13s} {'barrier / rest':>15s} {'sum+store':>10s} "
          f"{'to exit':>8s}   (a CTA's medians)", file=out)
    for k, name in enumerate(names):
        rows = [t[launch][t[launch][:, 0] > 0] for launch in range(k, 4 * layers, 4)]
        rec = np.concatenate([x for x in rows if len(x)], axis=0) if rows else np.zeros((0, 8))
        if not len(rec):
            continue

        def med(a: int, b: int) -> float:
            ok = (rec[:, a] > 0) & (rec[:, b] > 0)
            return float(np.median((rec[:, b] - rec[:, a])[ok]) / 1e3) if ok.any() else float("nan")

        split = bool((rec[:, 6] > 0).any())
        print(f"{name:8s} {med(1, 2):10.2f} {med(2, 4):13.2f} {med(4, 5):15.2f} "
              f"{(med(5, 6) if split else float('nan')):10.2f} {med(6 if split else 5, 3):8.2f}", file=out)
    for s in seqs:
        eng.close(s)


def prefill_attention(tokens: int, config: Dict, out=sys.stdout) -> None:
    """A CTA's life in the tensor-core prefill attention of one prompt: set-up,
    first scores, last page, output, and how long its MMA thread waited for
    keys, probabilities and values and a softmax row for scores."""
    from . import ops
    from .ops import native

    nq, nkv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    dev = "cuda:0"
    pages = (tokens + 63) // 64
    kp = torch.randn(pages, nkv, 64, d, device=dev).bfloat16()
    vp = torch.randn(pages, nkv, 64, d, device=dev).bfloat16()
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    q = torch.randn(tokens, nq * d, device=dev).bfloat16()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    args = (q, kp, vp, table, 64, i32([0]), i32([0]), i32([tokens]), i32([0, tokens]), tokens, nq, nkv, d,
            None, d ** -0.5)
    run = lambda: ops.attention_prefill_tc(*args)
    for _ in range(3):
        run()
    lib = native.lib()
    lib.rfx_attention_prefill_tc_trace.argtypes = [ctypes.c_void_p, ctypes.c_int]
    g = nq // nkv
    n_cta = nkv * ((tokens + 128 // g - 1) // (128 // g))
    buf = torch.zeros((n_cta * 32,), dtype=torch.int64, device=dev)
    lib.rfx_attention_prefill_tc_trace(buf.data_ptr(), n_cta)
    run()
    torch.cuda.synchronize()
    lib.rfx_attention_prefill_tc_trace(0, 0)
    t = buf.cpu().numpy().reshape(n_cta, 32).astype(np.float64)
    ok = (t[:, 0] > 0) & (t[:, 5] > 0)
    idx = np.nonzero(ok)[0]
    t = t[ok]
    r = (t - t[:, 0].min()) / 1e3
    # CTAs are numbered with the kv head fastest and the tile slowest, longest tiles first
    n_tiles = n_cta // nkv
    tile = n_tiles - 1 - idx // nkv
    bq = 128 // g
    n_pages = ((tile + 1) * bq - 1) // 64 + 1
    life = r[:, 5] - r[:, 0]
    fit = np.linalg.lstsq(np.vstack([n_pages, np.ones_like(n_pages)]).T.astype(np.float64), life, rcond=None)[0]
    print(f"prefill attention, one prompt of {tokens} tokens, {nq} query / {nkv} kv heads of {d}: "
          f"{len(idx)} CTAs, first entry to last exit {r[:, 5].max():.1f} us", file=out)
    print(f"a CTA's life = {fit[0]:.2f} us x pages + {fit[1]:.2f} us", file=out)
    for name, a, b in (("entry -> set up", 0, 1), ("set up -> first scores", 1, 2),
                       ("first scores -> last page", 2, 3), ("last page -> output written", 3, 4),
                       ("output written -> exit", 4, 5)):
        dt = r[:, b] - r[:, a]
        print(f"  {name:30s} median {np.median(dt):6.2f} us   90th percentile {np.percentile(dt, 90):6.2f}", file=out)
    pg = n_pages.astype(np.float64)
    for name, col in (("MMA thread waits for K", 8), ("MMA thread waits for P", 9), ("MMA thread waits for V", 10),
                      ("softmax row 0 waits for S", 11)):
        c = t[:, col] / pg
        print(f"  {name:30s} median {np.median(c):6.0f} cycles a page   90th percentile {np.percentile(c, 90):6.0f}",
              file=out)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(10):
        run()
    b.record()
    torch.cuda.synchronize()
    print(f"kernel, CUDA events, mean of 10 back-to-back launches: {a.elapsed_time(b) * 100:.1f} us", file=out)


def decode_attention(cases: List[str], config: Dict, out=sys.stdout, stamps: bool = False) -> None:
    """Microseconds and GB/s of `ops.attention_decode` over a scrambled paged
    cache, per case and number of key splits (20 launches after 3 warm-up
    launches; a case's cache is larger than L2 from 126 MB on)."""
    from . import ops
    from .ops import native

    nq, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    d = config.get("head_dim") or config["hidden_size"] // nq
    dev = "cuda:0"
    for case in cases:
        B, ctx = (int(x) for x in case.lower().split("x"))
        pages_per = (ctx + 63) // 64
        n_pages = B * pages_per
        kp = torch.randn(n_pages, nkv, 64, d, device=dev).bfloat16()
        vp = torch.randn(n_pages, nkv, 64, d, device=dev).bfloat16()
        table = torch.randperm(n_pages, device=dev).int().reshape(B, pages_per)
        q = torch.randn(B, nq * d, device=dev).bfloat16()
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(B, dtype=torch.int32, device=dev)
        cells = []
        for s_ in (1, 2, 4, 8, 16, 32):
            if s_ > pages_per:
                break

            def run():
                ops.attention_decode(q, kp, vp, table, 64, pos, slot, nq, nkv, d, None, d ** -0.5, n_splits=s_)

            for _ in range(3):
                run()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(20):
                run()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) / 20 * 1000
            cells.append(f"{s_} splits {us:7.1f} us {B * ctx * nkv * d * 4 / us / 1e3:5.0f} GB/s")
        pick = ops.decode_splits(B, nq, nkv, pages_per)
        print(f"batch {B:3d} context {ctx:6d} (model picks {pick:2d}): " + " | ".join(cells), file=out)
        if stamps:
            # one more launch with the model's pick, stamped: where a CTA's time goes
            lib = native.lib()
            lib.rfx_attention_decode_trace.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
            n_cta = B * nkv * ((nq // nkv + 7) // 8) * pick
            buf = torch.zeros((n_cta * 12,), dtype=torch.int64, device=dev)
            lib.rfx_attention_decode_trace(buf.data_ptr(), 1, n_cta)
            ops.attention_decode(q, kp, vp, table, 64, pos, slot, nq, nkv, d, None, d ** -0.5, n_splits=pick)
            torch.cuda.synchronize()
            lib.rfx_attention_decode_trace(0, 0, 0)
            t = buf.cpu().numpy().reshape(n_cta, 12).astype(np.float64)
            per = -(-pages_per // pick)
            med = lambda a, b: float(np.median(t[:, b] - t[:, a]) / 1e3)
            print(f"    {n_cta} CTAs of {per} pages: query rows {med(1, 2):.2f} us, pages {med(2, 3):.2f} us "
                  f"({med(2, 3) / per:.2f} a page; thread 0's cycles a page: waiting for it "
                  f"{float(np.median(t[:, 7])) / per:.0f}, issuing later loads {float(np.median(t[:, 8])) / per:.0f}, "
                  f"tile code {float(np.median(t[:, 9])) / per:.0f}), warps' merge {med(3, 4):.2f}, "
                  f"to exit {med(4, 6):.2f}; first entry to last exit {(t[:, 6].max() - t[:, 0].min()) / 1e3:.2f} us",
                  file=out)


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m reflex_b200.diagnostics", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    a = sub.add_parser("decode-step")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--layers", type=int, default=3)
    a.add_argument("--prompt", type=int, default=512)
    a.add_argument("--config", default="", help="a config.json (default: Qwen3-8B layer sizes)")
    b = sub.add_parser("prefill-attention")
    b.add_argument("--tokens", type=int, default=2048)
    b.add_argument("--config", default="", help="a config.json (default: Qwen3-8B layer sizes)")
    c = sub.add_parser("decode-attention")
    c.add_argument("--cases", default="1x640,8x640,64x640,32x1152,64x2048,8x4096,64x4096,8x16384,1x16384",
                   help="batch x context, comma separated")
    c.add_argument("--config", default="", help="a config.json (default: Qwen3-8B layer sizes)")
    c.add_argument("--stamps", action="store_true", help="after each case, where a CTA's time goes (its own stamps)")
    ns = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("error: diagnostics: no CUDA device (there is no CPU path)", file=sys.stderr)
        return 1
    if ns.what == "decode-step":
        decode_step(ns.batch, ns.layers, ns.prompt, _config(ns.config))
    elif ns.what == "decode-attention":
        decode_attention(ns.cases.split(","), _config(ns.config), stamps=ns.stamps)
    else:
        prefill_attention(ns.tokens, _config(ns.config))
    return 0


if __name__ == "__main__":
    sys.exit(main())
