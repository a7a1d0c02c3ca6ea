"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), allocates the
output, and launches on torch's current stream, so the calls order with the
library matrix products and can be captured into a CUDA graph.  Sizes a kernel
does not take are refused with an error that names them.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..errors import CudaError, InvalidInput
import os as _os

from . import native, workspace
from .workspace import new as _new

F32, BF16 = 0, 1


def launch_count() -> int:
    """Kernels of this library launched directly so far (graph replays are
    counted by the engine, which knows how many a captured step holds)."""
    return native.LAUNCHES


def dt_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise InvalidInput(f"kernels take float32 or bfloat16, got {dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: Optional[torch.Tensor], name: str, dtype=None) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise CudaError(f"{name} must live on the GPU (there is no CPU path)")
    if not t.is_contiguous():
        raise InvalidInput(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise InvalidInput(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


# ---------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, scale: float, err_flag: torch.Tensor) -> torch.Tensor:
    """hidden[r] = table[ids[r]] * scale, as float32 [R, H]."""
    V, H = table.shape
    R = ids.numel()
    out = _new((R, H), torch.float32, table.device, keep=True)  # the residual stream: lives for the whole step
    st = native.lib().rfx_embed(
        _chk(table, "table"), dt_code(table.dtype), _chk(ids, "ids", torch.int32), R, H, V,
        float(scale), out.data_ptr(), _chk(err_flag, "err_flag", torch.int32), _stream())
    native.check(st, "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, update_residual: bool = True,
            rows: Optional[torch.Tensor] = None, weight_offset: float = 0.0,
            want_out: bool = True) -> Optional[torch.Tensor]:
    """RMSNorm of the float32 residual stream `x` [R, H], with the residual add
    fused in: t = x (+ delta); x <- t (if `update_residual`, in place);
    returns t * rsqrt(mean(t^2) + eps) * (weight_offset + weight) in
    `out_dtype`.  With `rows` only those rows are read and the output has
    `len(rows)` rows (the residual is then left alone)."""
    R, H = x.shape
    _chk(x, "x", torch.float32)
    r_out = R if rows is None else rows.numel()
    out = _new((r_out, H), out_dtype, x.device) if want_out else None
    x_out = x if (delta is not None and update_residual and rows is None) else None
    st = native.lib().rfx_rmsnorm(
        x.data_ptr(), _chk(delta, "delta"), dt_code(delta.dtype) if delta is not None else 0,
        x_out.data_ptr() if x_out is not None else 0, _chk(weight, "weight", torch.float32),
        float(eps), float(weight_offset), out.data_ptr() if out is not None else 0,
        dt_code(out_dtype), _chk(rows, "rows", torch.int32), r_out, H, _stream())
    native.check(st, f"rmsnorm (H={H})")
    return out


def add_(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a += b with a float32."""
    _chk(a, "a", torch.float32)
    st = native.lib().rfx_add(a.data_ptr(), _chk(b, "b"), dt_code(b.dtype), a.numel(), _stream())
    native.check(st, "add")
    return a


def swiglu(gate_up: torch.Tensor, alternating: bool = False) -> torch.Tensor:
    """[R, 2I] -> silu(gate) * up, [R, I].  A row holds the gates in its first
    half and the ups in its second, or (`alternating`) gate_i at 2i and up_i at
    2i + 1."""
    R, two_i = gate_up.shape
    I = two_i // 2
    out = _new((R, I), gate_up.dtype, gate_up.device)
    st = native.lib().rfx_swiglu(_chk(gate_up, "gate_up"), out.data_ptr(), dt_code(gate_up.dtype),
                                 R, I, 1 if alternating else 0, _stream())
    native.check(st, "swiglu")
    return out


# -------------------------------------------------------------------- linear
def _env_int(name: str, default: int, lo: int = 0, hi: int = 1 << 30) -> int:
    """A run-time switch read once from the environment; a bad value is an
    `InvalidInput`, as the reference treats its own switches
    (src/model/kernels.rs:244-259)."""
    raw = _os.environ.get(name)
    if raw is None or raw == "":
        return default
    try:
        v = int(raw)
    except ValueError:
        raise InvalidInput(f"{name} must be an integer, got {raw!r}") from None
    if not (lo <= v <= hi):
        raise InvalidInput(f"{name} must be between {lo} and {hi}, got {v}")
    return v


def _env_flag(name: str, default: bool) -> bool:
    raw = _os.environ.get(name)
    if raw is None or raw == "":
        return default
    if raw not in ("0", "1"):
        raise InvalidInput(f"{name} must be 0 or 1, got {raw!r}")
    return raw == "1"


# `REFLEX_PREFILL_PROFILE=1`: CUDA events at phase marks of every eager step
# (embed, norm, qkv_gemm, norm_rope, attn, o_proj, ffn_gate_up, ffn_down, head),
# totals per phase printed to stderr after the step; a no-op when off and
# inside graph capture (src/model/prefill_profile.rs:1-18, 26-59).
PROFILE = _env_flag("REFLEX_PREFILL_PROFILE", False)
_prof_events: list = []


def prof_mark(name: str) -> None:
    if not PROFILE or torch.cuda.is_current_stream_capturing():
        return
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _prof_events.append((name, ev))


def prof_report(label: str) -> None:
    """Waits for the device and prints, per phase, the time between each mark
    and the one before it, summed over the step."""
    import sys

    if not PROFILE or len(_prof_events) < 2:
        _prof_events.clear()
        return
    torch.cuda.synchronize()
    totals, order = {}, []
    for (_, e0), (name, e1) in zip(_prof_events, _prof_events[1:]):
        if name not in totals:
            totals[name] = 0.0
            order.append(name)
        totals[name] += e0.elapsed_time(e1)
    whole = _prof_events[0][1].elapsed_time(_prof_events[-1][1])
    for name in order:
        print(f"REFLEX_PREFILL_PROFILE step={label} phase={name} ms={totals[name]:.3f}", file=sys.stderr)
    print(f"REFLEX_PREFILL_PROFILE step={label} phase=total ms={whole:.3f}", file=sys.stderr)
    _prof_events.clear()


GEMV_MAX_ROWS = _env_int("REFLEX_B200_GEMV_MAX_ROWS", 64, 0, 64)  # up to here the weight-streaming tensor-core kernel runs

_ERR = {}


def device_error_word(device) -> torch.Tensor:
    """One int32 word per device that kernels with bounded waits set to a
    non-zero code when a wait ran out."""
    key = torch.device(device).index or 0
    if key not in _ERR:
        _ERR[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _ERR[key]


def check_device_errors(device="cuda:0") -> None:
    """Synchronises; raises if a kernel reported that a bounded wait ran out."""
    code = int(device_error_word(device).item())
    if code:
        device_error_word(device).zero_()
        raise CudaError(f"a kernel reported an error (code {code}: a bounded wait that ran out, or a token "
                        f"id outside the vocabulary); the step's results are not valid")


def wait_probe(limit_ns: int, device="cuda:0") -> None:
    """Launches one block that waits, for at most `limit_ns` (clamped to a
    second), on a barrier nothing signals: the bounded wait runs out and the
    kernel records it in the device's error word, as the tensor-core kernels do
    when a copy or a product never arrives."""
    st = native.lib().rfx_wait_probe(int(limit_ns), device_error_word(device).data_ptr(), _stream())
    native.check(st, "wait_probe")


class NormedInput:
    """Rows that still await their RMSNorm factor: `hb` = bfloat16(h * norm
    weight) and `ssq[r][p]`, `n_part` partial sums of squares of h's row r.  The product
    that consumes them multiplies its row r by 1 / sqrt(sum_p ssq[r][p] / size +
    eps), which is the same as normalising first.  Made by `gemm_tc_residual`."""

    def __init__(self, hb: torch.Tensor, ssq: torch.Tensor, n_part: int, size: int, eps: float):
        self.hb, self.ssq, self.n_part, self.size, self.eps = hb, ssq, n_part, size, eps

    @property
    def shape(self):
        return self.hb.shape

    @property
    def dtype(self):
        return self.hb.dtype


def gemm_tc(x, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32,
            ksplit: int = 0, swiglu_pairs: bool = False, own: bool = False) -> torch.Tensor:
    """The tcgen05/TMA product y = x @ weight.T (bfloat16 in, float32 accumulate).
    With `swiglu_pairs` the weight's rows alternate gate, up and the result is
    silu(gate) * up, [R, N / 2].  `x` may be a `NormedInput`."""
    normed = x if isinstance(x, NormedInput) else None
    if normed is not None:
        x = normed.hb
    R, K = x.shape
    N = weight.shape[0]
    _chk(x, "x", torch.bfloat16)
    _chk(weight, "weight", torch.bfloat16)
    y = _new((R, N // 2 if swiglu_pairs else N), out_dtype, x.device, own=own)
    st = native.lib().rfx_gemm_bf16_tc(
        x.data_ptr(), weight.data_ptr(), y.data_ptr(), dt_code(out_dtype), R, N, K, ksplit,
        1 if swiglu_pairs else 0, normed.ssq.data_ptr() if normed is not None else 0,
        normed.n_part if normed is not None else 0, normed.size if normed is not None else 0,
        float(normed.eps) if normed is not None else 0.0, device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc (R={R}, N={N}, K={K})")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           own: bool = False) -> torch.Tensor:
    """y = x @ weight.T for weight [N, K] row-major.

    float32: this library's own CUDA-core product (no reduced-precision matrix
    mode; each output element reduced over k in index order).
    bfloat16: the weight-streaming tcgen05 kernel for up to GEMV_MAX_ROWS rows
    (decode), the library matrix product (cuBLAS, 32-bit accumulation) above
    that, where the reference uses a library product too
    (src/model/kernels.rs:2518-2561).  The result comes from the step's workspace;
    with `own` it gets memory of its own (what a step hands to its caller)."""
    R, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise InvalidInput(f"linear: x has {K} columns, weight has {K2}")
    if x.dtype != weight.dtype:
        raise InvalidInput(f"linear: x is {x.dtype}, weight is {weight.dtype}")
    if isinstance(x, NormedInput):
        return gemm_tc(x, weight, out_dtype or torch.bfloat16, own=own)
    _chk(x, "x")
    _chk(weight, "weight")
    if x.dtype == torch.float32:
        y = _new((R, N), torch.float32, x.device, own=own)
        st = native.lib().rfx_gemm_f32(x.data_ptr(), weight.data_ptr(), y.data_ptr(), R, N, K, _stream())
        native.check(st, f"gemm_f32 (R={R}, N={N}, K={K})")
        return y
    out_dtype = out_dtype or torch.bfloat16
    if R <= GEMV_MAX_ROWS and K % 8 == 0:
        return gemm_tc(x, weight, out_dtype, own=own)
    y = _new((R, N), out_dtype, x.device, own=own)
    if out_dtype == torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32, out=y)
    return torch.mm(x, weight.t(), out=y)


def gather_dot(x: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """y[j] = x[j] . weight[ids[j]], float32 [P]: row j of `x` against one row of
    the matrix, chosen by id.  Scoring given continuations needs the head's rows
    of a handful of ids, not the whole vocabulary
    (src/kernels_cuda/gemv_gather.cu:10-51).  In 32-bit the bits are those of
    `linear(x, weight)[j, ids[j]]`."""
    P, K = x.shape
    V, K2 = weight.shape
    if K != K2 or ids.numel() != P:
        raise InvalidInput("gather_dot: x [P, K], weight [V, K] and P ids are needed")
    if x.dtype != weight.dtype:
        raise InvalidInput(f"gather_dot: x is {x.dtype}, weight is {weight.dtype}")
    y = torch.empty((P,), dtype=torch.float32, device=x.device)
    st = native.lib().rfx_gather_dot(_chk(x, "x"), _chk(weight, "weight"), dt_code(x.dtype),
                                     _chk(ids, "ids", torch.int32), y.data_ptr(), P, K, V,
                                     device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gather_dot (P={P}, K={K})")
    return y


def gemm_tc_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor,
                     norm_weight: torch.Tensor, norm_offset: float, eps: float, ksplit: int = 0) -> NormedInput:
    """hidden += x @ weight.T in place (float32), and the rows of the new hidden
    as a `NormedInput` for the product after the norm whose weight is given: the
    residual add and the RMSNorm between two products without a launch."""
    import ctypes

    R, K = x.shape
    N = weight.shape[0]
    _chk(x, "x", torch.bfloat16)
    _chk(weight, "weight", torch.bfloat16)
    _chk(hidden, "hidden", torch.float32)
    _chk(norm_weight, "norm_weight", torch.float32)
    if tuple(hidden.shape) != (R, N) or norm_weight.numel() != N:
        raise InvalidInput("gemm_tc_residual: hidden must be [rows, out] and the norm weight [out]")
    hb = _new((R, N), torch.bfloat16, x.device)
    ssq = _new((R * native.lib().rfx_gemm_bf16_tc_max_parts(N),), torch.float32, x.device)
    n_part = ctypes.c_int(0)
    st = native.lib().rfx_gemm_bf16_tc_residual(
        x.data_ptr(), weight.data_ptr(), hidden.data_ptr(), norm_weight.data_ptr(), float(norm_offset),
        hb.data_ptr(), ssq.data_ptr(), ctypes.addressof(n_part), R, N, K, ksplit,
        device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc_residual (R={R}, N={N}, K={K})")
    return NormedInput(hb, ssq, n_part.value, N, eps)


ADDED = object()  # what `linear_residual` returns when it added into `hidden` and began no norm


def linear_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor, next_norm):
    """The fused forms of `hidden += linear(x, weight)`.

    A few bfloat16 rows and an RMSNorm with a plain weight next: the product
    kernel's epilogue adds into `hidden` and begins `next_norm`; returns a
    `NormedInput`.  More bfloat16 rows than that kernel takes: the library
    product accumulates onto the 32-bit `hidden` in place (C = A B + C with
    32-bit C, so the sum is never rounded to bfloat16); returns `ADDED`.
    Otherwise None, and the caller takes the two-launch way."""
    if x.dtype != torch.bfloat16 or not FUSE_NORM:
        return None
    if x.shape[0] > GEMV_MAX_ROWS or x.shape[1] % 8:
        _chk(x, "x")
        _chk(weight, "weight", torch.bfloat16)
        _chk(hidden, "hidden", torch.float32)
        torch.addmm(hidden, x, weight.t(), out_dtype=torch.float32, out=hidden)
        return ADDED
    if next_norm is None or weight.shape[0] % 8:
        return None  # the product that takes these rows streams them by TMA: whole 16-byte units
    w = getattr(next_norm, "weight", None)
    spec = getattr(next_norm, "spec", None)
    if w is None or spec is None or getattr(spec, "kind", None) != "rmsnorm" or w.numel() != weight.shape[0]:
        return None
    return gemm_tc_residual(x, weight, hidden, w, spec.weight_offset, spec.eps)


FUSE_NORM = _env_flag("REFLEX_B200_FUSE_NORM", True)


def linear_swiglu(x: torch.Tensor, weight_pairs: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate.T) * (x @ up.T) for a weight whose rows alternate gate_j,
    up_j; [R, I] in x's dtype.  For a few bfloat16 rows the activation is the
    product kernel's epilogue; otherwise product, then the SwiGLU kernel."""
    R, K = x.shape
    if x.dtype == torch.bfloat16 and R <= GEMV_MAX_ROWS and K % 8 == 0:
        return gemm_tc(x, weight_pairs, torch.bfloat16, swiglu_pairs=True)
    if isinstance(x, NormedInput):
        raise InvalidInput("a NormedInput is only made for sizes the fused product takes")
    return swiglu(linear(x, weight_pairs), alternating=True)


# ----------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, q_weight, k_weight, eps: float, weight_offset: float,
             rotation, row_pos: torch.Tensor, row_slot: torch.Tensor,
             k_pages, v_pages, page_table: torch.Tensor, page_size: int, nq: int, nkv: int,
             head_dim: int, writes_cache: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """Per-head q/k norm, rotary encoding, q out, k and v into the cache.
    `rotation`: a `parts.Rotation` (denominators, rotary_dim, pairing,
    magnitude) or None for no rotary encoding."""
    from ..parts.registry import PAIRINGS

    R = qkv.shape[0]
    rope_denom, rotary_dim, pairing, magnitude = None, 0, 0, 1.0
    if rotation is not None:
        if rotation.pairing not in PAIRINGS:
            raise InvalidInput(f"qkv_post: pairing must be one of {sorted(PAIRINGS)}, got {rotation.pairing!r}")
        rope_denom, rotary_dim = rotation.denominators, int(rotation.rotary_dim)
        pairing, magnitude = PAIRINGS[rotation.pairing], float(rotation.magnitude)
        if rope_denom is not None and rope_denom.numel() != rotary_dim // 2:
            raise InvalidInput("qkv_post: one denominator per rotary pair is needed")
    nkv_in = nkv if writes_cache else 0
    if qkv.shape[1] != (nq + 2 * nkv_in) * head_dim:
        raise InvalidInput("qkv_post: qkv width does not match the head counts")
    q = _new((R, nq * head_dim), out_dtype, qkv.device)
    st = native.lib().rfx_qkv_post(
        _chk(qkv, "qkv"), dt_code(qkv.dtype), qkv.shape[1], _chk(q_weight, "q_norm", torch.float32),
        _chk(k_weight, "k_norm", torch.float32), float(eps), float(weight_offset),
        _chk(rope_denom, "rope_denom", torch.float32), int(rotary_dim),
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32),
        q.data_ptr(), _chk(k_pages, "k_pages"), _chk(v_pages, "v_pages"), dt_code(out_dtype),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size, R, nq, nkv_in,
        nkv, head_dim, pairing, magnitude, _stream())
    native.check(st, f"qkv_post (head_dim={head_dim})")
    return q


def qkv_fused_takes(x, head_dim: int, rotation, qkv_weight: torch.Tensor) -> bool:
    """Whether `qkv_fused` takes this call: a few bfloat16 rows (decode), a head
    size of 64 or 128, and a rotation, if any, over the whole head in half-split
    pairs."""
    rows, K = x.shape
    if not FUSE_QKV or x.dtype != torch.bfloat16 or qkv_weight.dtype != torch.bfloat16:
        return False
    if rows > min(GEMV_MAX_ROWS, FUSE_QKV_ROWS) or K % 8 or head_dim not in (64, 128):
        return False
    if rotation is not None and (rotation.pairing != "half" or rotation.rotary_dim != head_dim
                                 or rotation.denominators is None):
        return False
    return True


def qkv_fused(x, qkv_weight: torch.Tensor, q_weight, k_weight, eps: float, weight_offset: float,
              rotation, row_pos: torch.Tensor, row_slot: torch.Tensor, k_pages, v_pages,
              page_table: torch.Tensor, page_size: int, nq: int, nkv: int, head_dim: int,
              writes_cache: bool) -> torch.Tensor:
    """The q/k/v product of a decode step and what follows it, in one launch:
    per-head q/k norm, rotary encoding, q out (bfloat16 [R, nq * head_dim]), k and
    v into the cache.  `x`: bfloat16 rows or a `NormedInput`.  What `linear` +
    `qkv_post` give, without the launch between them and without the 32-bit
    q/k/v rows in memory."""
    normed = x if isinstance(x, NormedInput) else None
    if normed is not None:
        x = normed.hb
    R, K = x.shape
    nkv_in = nkv if writes_cache else 0
    if qkv_weight.shape[0] != (nq + 2 * nkv_in) * head_dim or qkv_weight.shape[1] != K:
        raise InvalidInput("qkv_fused: the weight's shape does not match the head counts")
    _chk(x, "x", torch.bfloat16)
    _chk(qkv_weight, "qkv_weight", torch.bfloat16)
    denom = None if rotation is None else rotation.denominators
    q = _new((R, nq * head_dim), torch.bfloat16, x.device)
    st = native.lib().rfx_gemm_bf16_tc_qkv(
        x.data_ptr(), qkv_weight.data_ptr(), R, K,
        normed.ssq.data_ptr() if normed is not None else 0, normed.n_part if normed is not None else 0,
        normed.size if normed is not None else 0, float(normed.eps) if normed is not None else 0.0,
        _chk(q_weight, "q_norm", torch.float32), _chk(k_weight, "k_norm", torch.float32), float(eps),
        float(weight_offset), _chk(denom, "rope_denom", torch.float32),
        float(rotation.magnitude) if rotation is not None else 1.0,
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), q.data_ptr(),
        _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size, nq, nkv_in, nkv,
        head_dim, device_error_word(x.device).data_ptr(), _stream())
    native.check(st, f"gemm_bf16_tc_qkv (R={R}, K={K}, head_dim={head_dim})")
    return q


FUSE_QKV = _env_flag("REFLEX_B200_FUSE_QKV", True)
# Up to this many rows the fused form is the faster one (measured on a B200 at
# Qwen3-8B sizes: 2.3 % of a step at batch 1, 0.7 % at batch 8, level at 16, behind
# from 32 on).  With more rows the attention kernel that follows is the
# step's largest after the feed-forward, and it gains more from starting early,
# beside the light `qkv_post` launch, and fetching its cached pages meanwhile,
# than the step gains from one launch less.
FUSE_QKV_ROWS = _env_int("REFLEX_B200_FUSE_QKV_ROWS", 8, 0, 64)


def attention_plain(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    page_table: torch.Tensor, page_size: int, row_pos: torch.Tensor,
                    row_slot: torch.Tensor, nq: int, nkv: int, head_dim: int,
                    window: Optional[int], scale: float) -> torch.Tensor:
    R = q.shape[0]
    out = _new(q.shape, q.dtype, q.device)
    st = native.lib().rfx_attention_plain(
        _chk(q, "q"), _chk(k_pages, "k_pages", q.dtype), _chk(v_pages, "v_pages", q.dtype),
        dt_code(q.dtype), _chk(page_table, "page_table", torch.int32), page_table.shape[1],
        page_size, _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32),
        out.data_ptr(), R, nq, nkv, head_dim, int(window or 0), float(scale), _stream())
    native.check(st, f"attention_plain (head_dim={head_dim})")
    return out


def gemv_simple(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The plain CUDA-core bfloat16 product (one warp per output column); kept
    as the readable counterpart of `gemm_tc` for tests."""
    R, K = x.shape
    N = weight.shape[0]
    y = torch.empty((R, N), dtype=out_dtype, device=x.device)
    st = native.lib().rfx_gemv_bf16(_chk(x, "x", torch.bfloat16), _chk(weight, "weight", torch.bfloat16),
                                    y.data_ptr(), dt_code(out_dtype), R, N, K, _stream())
    native.check(st, f"gemv_bf16 (R={R}, N={N}, K={K})")
    return y


_SM_COUNT = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once."""
    global _SM_COUNT
    if not _SM_COUNT:
        _SM_COUNT = int(native.lib().rfx_sm_count())
    return _SM_COUNT


def decode_splits(n_rows: int, nq: int, nkv: int, max_pages: int = 64) -> int:
    """Key-range splits of the decode kernel for rows whose longest context has
    `max_pages` pages.  A split buys parallelism and costs a CTA's fixed work
    (query load, the warps' merge, the exchange of partials) once more.  Fitted
    to kernel times on a B200 at batches of 1 to 64 and contexts of 640 to
    16,384: two CTAs fit an SM; a CTA walks its pages at 0.6 us a page with an
    SM to itself and 0.85 us beside another (its tile code, not the memory);
    the pages of all CTAs together cannot come faster than the memory gives
    them, 1.35 us per page and CTA slot; a CTA's fixed work is 3 to 4 us; 4 us
    for the launch; the merge 1 us + 0.12 us a split inside a cluster of up to
    8, 5 us in one of 16, 3 us + 0.25 us a split through the combine kernel.
    The smallest estimate wins."""
    forced = _env_int("REFLEX_B200_DECODE_SPLITS", 0, 0, 64)  # tuning aid
    if forced > 0:
        return forced
    ctas = n_rows * nkv * ((nq // nkv + 7) // 8)
    sms = sm_count()
    slots = 2 * sms
    best, best_cost = 1, None
    for s in (1, 2, 4, 8, 16, 32, 64):
        if s > max(1, max_pages):
            break
        n = ctas * s
        per_split = -(-max_pages // s)
        resident = per_split * (0.6 if n <= sms else 0.85) + 4.0
        streaming = n * (per_split * 1.35 + 3.0) / slots
        if s == 1:
            merge = 0.0
        elif s <= 8:
            merge = 1.0 + 0.12 * s
        elif s == 16:
            merge = 5.0
        else:
            merge = 3.0 + 0.25 * s
        cost = 4.0 + max(resident, streaming) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def attention_decode(q, k_pages, v_pages, page_table, page_size, row_pos, row_slot, nq, nkv,
                     head_dim, window, scale, n_splits: Optional[int] = None) -> torch.Tensor:
    """bfloat16 tensor-core attention for rows that are each one query
    position (decode), split over the keys."""
    R = q.shape[0]
    _chk(q, "q", torch.bfloat16)
    if head_dim % 16 or not (16 <= head_dim <= 256):
        raise InvalidInput(f"attention_decode takes head_dim in steps of 16 up to 256, got {head_dim}")
    n_splits = n_splits or decode_splits(R, nq, nkv)
    out = _new(q.shape, q.dtype, q.device)
    # pages of the store, for the kernel's TMA maps: [pages, kv heads, page, head_dim], one piece
    pool_pages = int(k_pages.shape[0]) if (k_pages.dim() == 4 and k_pages.is_contiguous()
                                           and v_pages.is_contiguous() and v_pages.shape == k_pages.shape) else 0
    if CLUSTER_MERGE and n_splits in (2, 4, 8, 16):
        # the splits as one thread-block cluster that merges its partials itself
        st = native.lib().rfx_attention_decode_cluster(
            q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
            _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
            _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), out.data_ptr(),
            R, nq, nkv, head_dim, n_splits, int(window or 0), float(scale), pool_pages,
            device_error_word(q.device).data_ptr(), _stream())
        if st != native.ERR_UNSUPPORTED:
            native.check(st, f"attention_decode_cluster (head_dim={head_dim}, splits={n_splits})")
            return out
    partial = _new((R * nq * n_splits * (head_dim + 2),), torch.float32, q.device) if n_splits > 1 else None
    st = native.lib().rfx_attention_decode(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(row_pos, "row_pos", torch.int32), _chk(row_slot, "row_slot", torch.int32), out.data_ptr(),
        partial.data_ptr() if partial is not None else 0, R, nq, nkv, head_dim, n_splits,
        int(window or 0), float(scale), pool_pages, device_error_word(q.device).data_ptr(), _stream())
    native.check(st, f"attention_decode (head_dim={head_dim}, splits={n_splits})")
    return out


CLUSTER_MERGE = _env_flag("REFLEX_B200_CLUSTER_MERGE", True)


def attention_prefill(q, k_pages, v_pages, page_table, page_size, seq_slot, seq_start, seq_new,
                      seq_row0, max_new: int, nq, nkv, head_dim, window, scale) -> torch.Tensor:
    """bfloat16 tensor-core attention for a packed batch of sequences that
    each bring one or more rows (prefill, chunks, mixed steps)."""
    _chk(q, "q", torch.bfloat16)
    if head_dim % 16 or not (16 <= head_dim <= 256):
        raise InvalidInput(f"attention_prefill takes head_dim in steps of 16 up to 256, got {head_dim}")
    if nq // nkv > 128:
        raise InvalidInput(f"attention_prefill takes up to 128 query heads per kv head, got {nq // nkv}")
    out = _new(q.shape, q.dtype, q.device)
    S = seq_slot.numel()
    st = native.lib().rfx_attention_prefill(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(seq_slot, "seq_slot", torch.int32), _chk(seq_start, "seq_start", torch.int32),
        _chk(seq_new, "seq_new", torch.int32), _chk(seq_row0, "seq_row0", torch.int32), out.data_ptr(),
        S, int(max_new), nq, nkv, head_dim, int(window or 0), float(scale), _stream())
    native.check(st, f"attention_prefill (head_dim={head_dim})")
    return out


def attention_prefill_tc(q, k_pages, v_pages, page_table, page_size, seq_slot, seq_start, seq_new,
                         seq_row0, max_new: int, nq, nkv, head_dim, window, scale) -> torch.Tensor:
    """The tcgen05/TMEM form of `attention_prefill`, for head sizes 64 and 128."""
    _chk(q, "q", torch.bfloat16)
    if head_dim not in (64, 128):
        raise InvalidInput(f"attention_prefill_tc takes head_dim 64 or 128, got {head_dim}")
    if nq // nkv > 128:
        raise InvalidInput(f"attention_prefill_tc takes up to 128 query heads per kv head, got {nq // nkv}")
    out = _new(q.shape, q.dtype, q.device)
    st = native.lib().rfx_attention_prefill_tc(
        q.data_ptr(), _chk(k_pages, "k_pages", torch.bfloat16), _chk(v_pages, "v_pages", torch.bfloat16),
        k_pages.shape[0], _chk(page_table, "page_table", torch.int32), page_table.shape[1], page_size,
        _chk(seq_slot, "seq_slot", torch.int32), _chk(seq_start, "seq_start", torch.int32),
        _chk(seq_new, "seq_new", torch.int32), _chk(seq_row0, "seq_row0", torch.int32), out.data_ptr(),
        seq_slot.numel(), int(max_new), q.shape[0], nq, nkv, head_dim, int(window or 0), float(scale),
        device_error_word(q.device).data_ptr(), _stream())
    native.check(st, f"attention_prefill_tc (head_dim={head_dim})")
    return out


def attention(q, k_pages, v_pages, page_table, page_size, batch, nq, nkv, head_dim, window, scale):
    """Attention of the step's rows over their sequences' cached keys and
    values; picks the kernel for the dtype and the kind of step."""
    fast = q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
    if fast and batch.is_decode:
        pages = -(-min(batch.max_context, window or batch.max_context) // page_size) + (1 if window else 0)
        return attention_decode(q, k_pages, v_pages, page_table, page_size, batch.row_pos,
                                batch.row_slot, nq, nkv, head_dim, window, scale,
                                n_splits=decode_splits(q.shape[0], nq, nkv, pages))
    if fast and nq // nkv <= 128 and head_dim in (64, 128):
        return attention_prefill_tc(q, k_pages, v_pages, page_table, page_size, batch.seq_slot,
                                    batch.seq_start, batch.seq_new, batch.seq_row0, batch.max_new, nq,
                                    nkv, head_dim, window, scale)
    if fast and nq // nkv <= 128:
        return attention_prefill(q, k_pages, v_pages, page_table, page_size, batch.seq_slot,
                                 batch.seq_start, batch.seq_new, batch.seq_row0, batch.max_new, nq,
                                 nkv, head_dim, window, scale)
    return attention_plain(q, k_pages, v_pages, page_table, page_size, batch.row_pos,
                           batch.row_slot, nq, nkv, head_dim, window, scale)


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit per row (ties: the highest index).  `out`
    (int32 [B]) and `scratch` (float32, B * 128) may be given to spare the
    allocations of a call a step."""
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    if scratch is None:
        scratch = torch.empty((B * 64 * 2,), dtype=torch.float32, device=logits.device)
    st = native.lib().rfx_argmax(logits.data_ptr(), V, B, V, _chk(out, "out", torch.int32),
                                 _chk(scratch, "scratch", torch.float32), _stream())
    native.check(st, "argmax")
    return out


def sample_work_bytes(B: int, V: int) -> int:
    """Bytes of working memory `sample` needs for B rows of V entries."""
    return int(native.lib().rfx_sample_work_bytes(int(B), int(V)))


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           work: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token a row: temperature softmax, optional top-k and top-p cuts, and an
    inverse-CDF draw with the row's uniform number.  `scratch` (float32 [B, V])
    and `work` (uint8, `sample_work_bytes(B, V)`) may be given to spare the
    allocations of a call a step."""
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if scratch is None:
        scratch = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    need = sample_work_bytes(B, V)
    if work is None:
        work = torch.empty((need,), dtype=torch.uint8, device=logits.device)
    elif work.numel() < need or work.dtype != torch.uint8:
        raise InvalidInput(f"sample: work must hold {need} bytes")
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _chk(out, "out", torch.int32)
    st = native.lib().rfx_sample(
        logits.data_ptr(), V, B, V, _chk(temperature, "temperature", torch.float32),
        _chk(top_k, "top_k", torch.int32), _chk(top_p, "top_p", torch.float32),
        _chk(uniform, "uniform", torch.float32), _chk(scratch, "scratch", torch.float32),
        _chk(work, "work", torch.uint8), out.data_ptr(), _stream())
    native.check(st, "sample")
    return out
