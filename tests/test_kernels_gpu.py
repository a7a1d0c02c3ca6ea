"""Each kernel alone against a plain float64 reference of the same op, at sizes
other than the engine's tiny models (and at the benchmark's head shapes).
References are the plain implementation's functions or one-line NumPy/torch
formulas; inputs are made so that faults show (a far key that dominates, keys
at a window's edge, scrambled page tables, stale data in unused cache rows)."""

import math

import numpy as np
import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from reflex_b200 import ops as o

    return o


def relerr(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("R,H", [(1, 64), (3, 100), (5, 4096), (2, 5120), (4, 24)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_with_add_gather_and_offset(R, H, out_dtype):
    g = torch.Generator().manual_seed(R * 1000 + H)
    x = torch.randn(R, H, generator=g) * 3
    d = torch.randn(R, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    eps = 1e-5
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    xd = x.to(DEV)
    out = ops().rmsnorm(xd, w.to(DEV), eps, out_dtype)
    assert relerr(out, pm.rms_norm(x.double().numpy(), w.double().numpy(), eps)) < tol
    # fused residual add: the residual is updated in place, in 32-bit
    for delta in (d.to(DEV), d.to(DEV).bfloat16()):
        xd = x.to(DEV).clone()
        out = ops().rmsnorm(xd, w.to(DEV), eps, out_dtype, delta=delta)
        t = x.double().numpy() + delta.double().cpu().numpy()
        assert relerr(xd, t) < 1e-6
        assert relerr(out, pm.rms_norm(t, w.double().numpy(), eps)) < tol
    # gathered rows, residual untouched, and the (1 + w) variant
    rows = torch.tensor([R - 1, 0], dtype=torch.int32, device=DEV)
    xd = x.to(DEV).clone()
    out = ops().rmsnorm(xd, w.to(DEV), eps, out_dtype, delta=d.to(DEV), rows=rows, weight_offset=1.0)
    t = (x + d).double().numpy()[[R - 1, 0]]
    assert relerr(out, pm.rms_norm(t, 1.0 + w.double().numpy(), eps)) < tol
    assert torch.equal(xd.cpu(), x)


@pytest.mark.parametrize("R,H", [(256, 64), (300, 100), (700, 4096), (1500, 5120), (257, 8200)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_of_many_rows(R, H, out_dtype):
    """Many whole rows: the same bits as a gather of every row, and the plain norm."""
    g = torch.Generator().manual_seed(R + H)
    x = torch.randn(R, H, generator=g) * 3
    x[R // 2] *= 50.0  # a row of another scale among its neighbours
    w = 1 + 0.1 * torch.randn(H, generator=g)
    eps = 1e-6
    xd, wd = x.to(DEV), w.to(DEV)
    out = ops().rmsnorm(xd, wd, eps, out_dtype, weight_offset=0.5)
    every = torch.arange(R, dtype=torch.int32, device=DEV)
    one_by_one = ops().rmsnorm(xd, wd, eps, out_dtype, rows=every, weight_offset=0.5)
    assert torch.equal(out, one_by_one)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    ref = pm.rms_norm(x.double().numpy(), 0.5 + w.double().numpy(), eps)
    for r in (0, R // 2, R - 1):
        assert relerr(out[r], ref[r]) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_embed_add(dtype):
    g = torch.Generator().manual_seed(1)
    gu = (torch.randn(7, 2 * 333, generator=g) * 3).to(dtype)
    out = ops().swiglu(gu.to(DEV))
    a, b = gu[:, :333].double().numpy(), gu[:, 333:].double().numpy()
    assert relerr(out, a / (1 + np.exp(-a)) * b) < (1e-6 if dtype == torch.float32 else 5e-3)
    out = ops().swiglu(gu.to(DEV), alternating=True)
    a, b = gu[:, 0::2].double().numpy(), gu[:, 1::2].double().numpy()
    assert relerr(out, a / (1 + np.exp(-a)) * b) < (1e-6 if dtype == torch.float32 else 5e-3)
    table = torch.randn(1000, 96, generator=g).to(dtype)
    ids = torch.tensor([999, 0, 17, 17, 500], dtype=torch.int32)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    e = ops().embed(table.to(DEV), ids.to(DEV), 2.0, flag)
    assert e.dtype == torch.float32
    assert torch.equal(e.cpu(), table[ids.long()].float() * 2.0)
    assert int(flag.item()) == 0
    ops().embed(table.to(DEV), torch.tensor([3, 1000], dtype=torch.int32, device=DEV), 1.0, flag)
    assert int(flag.item()) == 2  # 1 + the row of the bad id
    acc = torch.randn(5, 77, generator=g)
    d = torch.randn(5, 77, generator=g).to(dtype)
    got = ops().add_(acc.to(DEV).clone(), d.to(DEV))
    assert relerr(got, acc.double().numpy() + d.double().numpy()) < 1e-6


# ----------------------------------------------------------------------- linear
@pytest.mark.parametrize("R,N,K", [(1, 7, 5), (3, 1000, 96), (65, 130, 257), (200, 64, 1024), (16, 6144, 512)])
def test_gemm_f32_is_exact_to_rounding_and_row_independent(R, N, K):
    g = torch.Generator().manual_seed(R + N + K)
    x = torch.randn(R, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.05
    y = ops().linear(x.to(DEV), w.to(DEV))
    ref = x.double().numpy() @ w.double().numpy().T
    assert relerr(y, ref) < 5e-7 * math.sqrt(K)
    # a row's result must not depend on what else is in the batch: bit-equal alone
    alone = ops().linear(x[R // 2:R // 2 + 1].to(DEV).contiguous(), w.to(DEV))
    assert torch.equal(alone[0], y[R // 2])


@pytest.mark.parametrize("R,N,K", [(1, 128, 64), (5, 1000, 96), (8, 4096, 4096), (33, 6144, 4096),
                                   (64, 777, 80), (17, 151936, 512), (2, 4096, 12288)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_any_shape(R, N, K, out_dtype):
    g = torch.Generator().manual_seed(R + N + K)
    x = torch.randn(R, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    ref = (x.double() @ w.double().T).numpy()
    tol = 2e-6 * math.sqrt(K) if out_dtype == torch.float32 else 5e-3
    for ks in (0, 1, 2, 4, 8):
        if ks > 1 and (K + 63) // 64 < ks:
            continue
        y = ops().gemm_tc(x.to(DEV), w.to(DEV), out_dtype, ksplit=ks)
        assert relerr(y, ref) < tol, ks
    ops().check_device_errors(DEV)
    simple = ops().gemv_simple(x.to(DEV), w.to(DEV), out_dtype)
    assert relerr(simple, ref) < tol


@pytest.mark.parametrize("R,I,K", [(1, 64, 64), (5, 160, 96), (8, 12288, 4096), (64, 555, 80), (33, 2048, 4096)])
def test_gemm_tc_with_the_swiglu_epilogue(R, I, K):
    g = torch.Generator().manual_seed(R + I + K)
    x = torch.randn(R, K, generator=g).bfloat16()
    gate = (torch.randn(I, K, generator=g) * 0.08).bfloat16()
    up = (torch.randn(I, K, generator=g) * 0.08).bfloat16()
    ref = pm.swiglu(x.double().numpy(), gate.double().numpy(), up.double().numpy(), np.eye(I))
    pairs = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    for ks in (0, 1, 2, 4, 8):
        if ks > 1 and (K + 63) // 64 < ks:
            continue
        y = ops().gemm_tc(x.to(DEV), pairs.to(DEV), torch.bfloat16, ksplit=ks, swiglu_pairs=True)
        assert y.shape == (R, I)
        assert relerr(y, ref) < 8e-3, ks
    assert relerr(ops().linear_swiglu(x.to(DEV), pairs.to(DEV)), ref) < 8e-3
    ops().check_device_errors(DEV)


@pytest.mark.parametrize("R,N,K", [(1, 64, 64), (5, 96, 320), (8, 4096, 4096), (64, 4096, 12288), (17, 1000, 96)])
def test_gemm_tc_residual_add_with_the_norm_folded_into_the_next_product(R, N, K):
    """hidden += x W^T in the product's epilogue, the rows handed on unnormalised
    with partial sums of squares, and the next product scaling its rows by the
    norm factor: against add, RMSNorm, product done one after the other in
    double precision."""
    g = torch.Generator().manual_seed(R + N + K)
    x = torch.randn(R, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    h = torch.randn(R, N, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(N, generator=g)
    w2 = (torch.randn(2 * 24, N, generator=g) * 0.05).bfloat16()
    eps = 1e-5
    for ks in (0, 1, 2, 4, 8):
        if ks > 1 and (K + 63) // 64 < ks:
            continue
        hd = h.to(DEV).clone()
        ni = ops().gemm_tc_residual(x.to(DEV), w.to(DEV), hd, nw.to(DEV), 0.0, eps, ksplit=ks)
        h_ref = h.double().numpy() + x.double().numpy() @ w.double().numpy().T
        assert relerr(hd, h_ref) < 3e-6 * math.sqrt(K)
        assert relerr(ni.hb, h_ref * nw.double().numpy()) < 5e-3
        ssq = ni.ssq[: R * ni.n_part].view(R, ni.n_part).sum(dim=1)
        assert relerr(ssq, (h_ref * h_ref).sum(axis=1)) < 1e-4  # 32-bit h, K products each
        normed = pm.rms_norm(h_ref, nw.double().numpy(), eps)
        y = ops().linear(ni, w2.to(DEV), out_dtype=torch.float32)
        assert relerr(y, normed @ w2.double().numpy().T) < 8e-3, ks
        act = ops().linear_swiglu(ni, w2.to(DEV))
        full = normed @ w2.double().numpy().T
        gt, up = full[:, 0::2], full[:, 1::2]
        assert relerr(act, gt / (1 + np.exp(-gt)) * up) < 1.2e-2, ks
    ops().check_device_errors(DEV)


@pytest.mark.parametrize("R", [1, 8, 64])
def test_the_head_product_with_the_final_norm_folded_in_at_the_benchmark_models_sizes(R):
    """The decode step's last product as the benchmark model runs it: rows that
    await their norm factor (partial sums of squares from the product before)
    against a 151,936 x 4,096 head, with the factor applied in the product's
    prologue; against norm, then product, in double precision."""
    N, K, V = 4096, 1024, 151936
    g = torch.Generator().manual_seed(R)
    x = torch.randn(R, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    h = torch.randn(R, N, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(N, generator=g)
    gd = torch.Generator(device=DEV).manual_seed(R)
    head = (torch.randn(V, N, generator=gd, device=DEV) * 0.02).bfloat16()  # drawn on the device: 622 M numbers
    eps = 1e-6
    hd = h.to(DEV).clone()
    ni = ops().gemm_tc_residual(x.to(DEV), w.to(DEV), hd, nw.to(DEV), 0.0, eps)
    assert ni.n_part > 1  # the sums of squares arrive in parts
    y = ops().linear(ni, head, out_dtype=torch.float32)
    ops().check_device_errors(DEV)
    h_ref = h.double().numpy() + x.double().numpy() @ w.double().numpy().T
    normed = pm.rms_norm(h_ref, nw.double().numpy(), eps)
    ref = (normed.astype(np.float32) @ head.float().cpu().numpy().T).astype(np.float64)  # on the CPU, 32-bit sums
    assert y.shape == (R, V) and relerr(y, ref) < 8e-3


def test_gemm_tc_refuses_what_it_cannot_do():
    from reflex_b200 import CudaError

    x = torch.zeros(2, 100, dtype=torch.bfloat16, device=DEV)  # K = 100 is no multiple of 8
    w = torch.zeros(16, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(CudaError) as e:
        ops().gemm_tc(x, w)
    assert "not supported" in str(e.value)


# ------------------------------------------------------------------- qkv_post
@pytest.mark.parametrize("nq,nkv,d,rd,theta", [(4, 2, 16, 16, 1e4), (6, 1, 32, 32, 1e6), (3, 1, 48, 32, 5e4),
                                               (32, 8, 128, 128, 1e6), (2, 2, 256, 64, 1e4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qkv_post_norm_rope_cache(nq, nkv, d, rd, theta, dtype):
    g = torch.Generator().manual_seed(nq * d)
    R = 6
    positions = [0, 1, 63, 64, 200, 3000]
    slots = [2, 0, 1, 2, 0, 1]
    n_pages, max_pages = 64, 50
    table = torch.randperm(n_pages * 3, generator=g)[: 3 * max_pages].reshape(3, max_pages).int() % n_pages
    # make the (slot, page index) pairs that are used distinct pages
    used = {}
    for s, p in zip(slots, positions):
        used[(s, p // 64)] = len(used)
    for (s, pi), page in used.items():
        table[s, pi] = page
    qkv = torch.randn(R, (nq + 2 * nkv) * d, generator=g) * 2
    qw = 1 + 0.1 * torch.randn(d, generator=g)
    kw = 1 + 0.1 * torch.randn(d, generator=g)
    eps = 1e-6
    k_pages = torch.full((n_pages, nkv, 64, d), 7.0, dtype=dtype, device=DEV)
    v_pages = torch.full((n_pages, nkv, 64, d), 7.0, dtype=dtype, device=DEV)
    denom = torch.pow(torch.tensor(theta, dtype=torch.float64), torch.arange(rd // 2, dtype=torch.float64) * 2 / rd)
    from reflex_b200.parts import Rotation

    q = ops().qkv_post(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, 0.0, Rotation(denom.float().to(DEV), rd),
                       torch.tensor(positions, dtype=torch.int32, device=DEV),
                       torch.tensor(slots, dtype=torch.int32, device=DEV), k_pages, v_pages, table.to(DEV), 64,
                       nq, nkv, d, True, dtype)
    x = qkv.double().numpy()
    pos = np.array(positions)
    qr = pm.rope_neox(pm.rms_norm(x[:, : nq * d].reshape(R, nq, d), qw.double().numpy(), eps), pos, theta, rd)
    kr = pm.rope_neox(pm.rms_norm(x[:, nq * d:(nq + nkv) * d].reshape(R, nkv, d), kw.double().numpy(), eps), pos, theta, rd)
    vr = x[:, (nq + nkv) * d:].reshape(R, nkv, d)
    # 32-bit angles are off by up to position * 2^-24 against double
    tol = 5e-4 if dtype == torch.float32 else 8e-3
    assert relerr(q.reshape(R, nq, d), qr) < tol
    for i, (s, p) in enumerate(zip(slots, positions)):
        page = int(table[s, p // 64])
        assert relerr(k_pages[page, :, p % 64, :], kr[i]) < tol
        assert relerr(v_pages[page, :, p % 64, :], vr[i]) < (1e-6 if dtype == torch.float32 else 5e-3)
    # nothing else in the cache was touched
    touched = torch.zeros(n_pages, 64, dtype=torch.bool)
    for s, p in zip(slots, positions):
        touched[int(table[s, p // 64]), p % 64] = True
    untouched = ~touched[:, None, :, None].expand(n_pages, nkv, 64, d)
    assert bool((k_pages.float().cpu()[untouched] == 7.0).all())
    assert bool((v_pages.float().cpu()[untouched] == 7.0).all())


# ------------------------------------------------------------------ attention
def _paged(seqs, nkv, d, dtype, g, fill=float("nan")):
    """Random K/V for sequences of the given total lengths in a scrambled
    paged store whose unused rows hold `fill` (NaN: reading one shows)."""
    n_pages_per = [(n + 63) // 64 for n in seqs]
    total = sum(n_pages_per) + 5
    perm = torch.randperm(total, generator=g)
    table = torch.full((len(seqs) + 3, max(n_pages_per) + 2), -12345, dtype=torch.int32)
    slots = torch.randperm(len(seqs) + 3, generator=g)[: len(seqs)].tolist()
    k_pages = torch.full((total, nkv, 64, d), fill, dtype=torch.float32)
    v_pages = torch.full((total, nkv, 64, d), fill, dtype=torch.float32)
    ks, vs, o = [], [], 0
    for i, n in enumerate(seqs):
        k = torch.randn(n, nkv, d, generator=g)
        v = torch.randn(n, nkv, d, generator=g)
        for p in range(n_pages_per[i]):
            page = int(perm[o + p])
            table[slots[i], p] = page
            m = min(64, n - p * 64)
            k_pages[page, :, :m] = k[p * 64:p * 64 + m].transpose(0, 1)
            v_pages[page, :, :m] = v[p * 64:p * 64 + m].transpose(0, 1)
        o += n_pages_per[i]
        ks.append(k)
        vs.append(v)
    return slots, table, k_pages.to(dtype), v_pages.to(dtype), ks, vs


def _ref_rows(q, ks, vs, seqs, scale, window, dtype):
    """seqs: (start, n_new) per sequence; q packed [rows, nq, d]."""
    outs, r = [], 0
    for (start, n), k, v in zip(seqs, ks, vs):
        T = start + n
        kk, vv = k.to(dtype).double().numpy(), v.to(dtype).double().numpy()
        qfull = np.zeros((T, q.shape[1], q.shape[2]))
        qfull[start:] = q[r:r + n].to(dtype).double().numpy()
        outs.append(pm.causal_attention(qfull, kk[:T], vv[:T], scale, window, first_row=start)[start:])
        r += n
    return np.concatenate(outs, axis=0)


ATT_CASES = [
    # nq, nkv, d, [(start, n_new)], window
    (4, 2, 16, [(0, 1)], None),
    (4, 2, 16, [(0, 5), (0, 17), (0, 32)], None),
    (6, 1, 32, [(0, 1), (0, 7), (0, 64), (0, 100), (0, 129)], None),
    (3, 1, 48, [(0, 300), (0, 38)], 37),
    (3, 1, 48, [(100, 37), (700, 300)], 37),
    (32, 8, 128, [(1489, 41), (0, 1), (63, 2)], None),
    (7, 7, 80, [(0, 255), (5, 251)], 64),
    (16, 1, 64, [(31, 34)], None),
    (6, 2, 64, [(0, 1), (0, 7), (0, 64), (0, 100), (0, 129)], None),
    (5, 1, 128, [(100, 37), (700, 300)], 37),
    (8, 8, 128, [(0, 200), (60, 9)], None),
]


# every case with every kernel that takes its head size (the tcgen05 kernel: 64 and 128)
ATT_RUNS = [(k,) + c for k in ("plain_f32", "plain_bf16", "prefill_bf16", "prefill_tc_bf16") for c in ATT_CASES
            if k != "prefill_tc_bf16" or c[2] in (64, 128)]


@pytest.mark.parametrize("kernel,nq,nkv,d,seqs,window", ATT_RUNS)
def test_attention_over_the_paged_cache(kernel, nq, nkv, d, seqs, window):
    g = torch.Generator().manual_seed(nq * 31 + d)
    dtype = torch.float32 if kernel == "plain_f32" else torch.bfloat16
    slots, table, kp, vp, ks, vs = _paged([a + b for a, b in seqs], nkv, d, dtype, g)
    R = sum(b for _, b in seqs)
    q = torch.randn(R, nq, d, generator=g) * 1.5
    scale = d ** -0.5
    ref = _ref_rows(q, ks, vs, seqs, scale, window, dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    row_pos = i32([a + j for a, b in seqs for j in range(b)])
    row_slot = i32([slots[i] for i, (a, b) in enumerate(seqs) for _ in range(b)])
    qd = q.reshape(R, nq * d).to(dtype).to(DEV)
    if kernel.startswith("plain"):
        out = ops().attention_plain(qd, kp.to(DEV), vp.to(DEV), table.to(DEV), 64, row_pos, row_slot,
                                    nq, nkv, d, window, scale)
    else:
        row0 = [0]
        for _, b in seqs:
            row0.append(row0[-1] + b)
        fn = ops().attention_prefill_tc if kernel == "prefill_tc_bf16" else ops().attention_prefill
        out = fn(qd, kp.to(DEV), vp.to(DEV), table.to(DEV), 64, i32(slots),
                 i32([a for a, _ in seqs]), i32([b for _, b in seqs]), i32(row0),
                 max(b for _, b in seqs), nq, nkv, d, window, scale)
        ops().check_device_errors(DEV)
    assert not bool(torch.isnan(out.float()).any()), "read a cache row that was never written"
    assert relerr(out.reshape(R, nq, d), ref) < (2e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("nq,nkv,d,ctxs,window,splits", [
    (4, 2, 16, [1, 17, 64, 65], None, None), (6, 1, 32, [100, 129], None, 3), (3, 1, 48, [300, 38, 37], 37, 5),
    (32, 8, 128, [640] * 4, None, None), (32, 8, 128, [1, 63, 64, 4000], None, 16), (40, 2, 256, [999], None, 4),
    (7, 7, 80, [255, 256], 100, 2), (32, 8, 128, [520] * 8, None, 4), (32, 8, 128, [100, 3000], None, 8),
    (20, 1, 64, [130, 64], None, 2), (32, 8, 128, [3840], None, 16), (16, 4, 256, [2000, 5], None, 16),
    # one sequence and long walks
    (32, 8, 128, [3840], None, 8), (32, 8, 128, [8000], None, 16), (8, 2, 64, [2000, 700], None, 4),
    (3, 1, 48, [3000, 38], 1000, 2), (32, 8, 128, [1500], None, 1),
    # head sizes of three 64-column boxes; a window with the pages coming by TMA
    (6, 2, 192, [300, 70], None, 2), (8, 2, 128, [500, 100, 64], 100, 2), (4, 4, 64, [257], 65, None)])
def test_attention_decode_splits(nq, nkv, d, ctxs, window, splits):
    g = torch.Generator().manual_seed(nq + d)
    slots, table, kp, vp, ks, vs = _paged(ctxs, nkv, d, torch.bfloat16, g)
    R = len(ctxs)
    q = torch.randn(R, nq, d, generator=g) * 1.5
    ref = _ref_rows(q, ks, vs, [(c - 1, 1) for c in ctxs], d ** -0.5, window, torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = ops().attention_decode(q.reshape(R, nq * d).bfloat16().to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV),
                                 64, i32([c - 1 for c in ctxs]), i32(slots), nq, nkv, d, window, d ** -0.5,
                                 n_splits=splits)
    assert not bool(torch.isnan(out.float()).any())
    assert relerr(out.reshape(R, nq, d), ref) < 8e-3
    if splits in (2, 4, 8, 16):
        # merged inside a cluster (the default) or by the combine kernel: the same bits
        import reflex_b200.ops as o

        assert o.CLUSTER_MERGE
        o.CLUSTER_MERGE = False
        try:
            two = o.attention_decode(q.reshape(R, nq * d).bfloat16().to(DEV), kp.to(DEV), vp.to(DEV),
                                     table.to(DEV), 64, i32([c - 1 for c in ctxs]), i32(slots), nq, nkv, d,
                                     window, d ** -0.5, n_splits=splits)
        finally:
            o.CLUSTER_MERGE = True
        assert torch.equal(out.view(torch.int16), two.view(torch.int16))


@pytest.mark.parametrize("kernel", ["plain_f32", "plain_bf16", "prefill_bf16", "prefill_tc_bf16", "decode_bf16"])
def test_a_far_key_among_hundreds_and_the_windows_edge(kernel):
    """One key gets a score far above the rest, so the output must be its value
    row; the key sits far back (position 3 of 900), and then exactly at the
    window's edge: visible at i - j = window - 1, gone at i - j = window."""
    nq, nkv, d, n = 4, 2, 64, 900
    dtype = torch.float32 if kernel == "plain_f32" else torch.bfloat16
    g = torch.Generator().manual_seed(5)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for far, window, expect_hit in ((3, None, True), (n - 1 - 99, 100, True), (n - 1 - 100, 100, False)):
        slots, table, kp, vp, ks, vs = _paged([n], nkv, d, torch.float32, g, fill=0.0)
        q = torch.randn(1, nq, d, generator=g) * 0.1
        # plant: key `far` of every kv head is 8 * the unit query direction of head 0 / head 2
        page, tok = int(table[slots[0], far // 64]), far % 64
        for kvh, h in ((0, 0), (1, 2)):
            u = q[0, h] / q[0, h].norm()
            q[0, h] = u * 6.0
            kp[page, kvh, tok] = u * 60.0
        qd = q.reshape(1, nq * d).to(dtype).to(DEV)
        args = (kp.to(dtype).to(DEV), vp.to(dtype).to(DEV), table.to(DEV), 64)
        if kernel.startswith("plain"):
            out = ops().attention_plain(qd, *args, i32([n - 1]), i32(slots), nq, nkv, d, window, d ** -0.5)
        elif kernel == "decode_bf16":
            out = ops().attention_decode(qd, *args, i32([n - 1]), i32(slots), nq, nkv, d, window, d ** -0.5, n_splits=4)
        else:
            fn = ops().attention_prefill_tc if kernel == "prefill_tc_bf16" else ops().attention_prefill
            out = fn(qd, *args, i32(slots), i32([n - 1]), i32([1]), i32([0, 1]), 1, nq, nkv, d, window, d ** -0.5)
        out = out.float().cpu().reshape(nq, d)
        for kvh, h in ((0, 0), (1, 2)):
            target = vp[page, kvh, tok].to(dtype).float()
            close = float((out[h] - target).abs().max()) < 2e-2
            assert close == expect_hit, (far, window, h)


# -------------------------------------------------------------------- sampling
def test_argmax_ties_go_to_the_highest_index():
    g = torch.Generator().manual_seed(3)
    l = torch.randn(5, 151936, generator=g)
    l[1, 77] = l[1, 150000] = 50.0
    l[2, 0] = 60.0
    l[3, -1] = 60.0
    l[4] = 0.0
    got = ops().argmax(l.to(DEV)).tolist()
    assert got == [pm.argmax_last(r.numpy()) for r in l]
    assert got[1] == 150000 and got[2] == 0 and got[3] == 151935 and got[4] == 151935


@pytest.mark.parametrize("V", [1000, 151936])
@pytest.mark.parametrize("top_k,top_p", [(None, None), (1, None), (50, None), (None, 0.9), (40, 0.5), (None, 0.0)])
def test_sampling_matches_the_plain_sampler_given_the_same_uniforms(V, top_k, top_p):
    g = torch.Generator().manual_seed(V + (top_k or 0))
    B = 12
    logits = torch.randn(B, V, generator=g) * 3
    logits[3, 5] = logits[3, 900] = logits[3].max() + 1  # a tie at the top
    u = torch.rand(B, generator=g)
    u[0], u[1] = 0.0, 0.99999994
    T = 0.8
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    got = ops().sample(logits.to(DEV), torch.full((B,), T, device=DEV), u.to(DEV),
                       top_k=i32([top_k] * B) if top_k else None,
                       top_p=torch.full((B,), top_p, device=DEV) if top_p is not None else None).tolist()
    for b in range(B):
        want = pm.sample_token(logits[b].numpy(), T, float(u[b]), top_k, top_p)
        if got[b] != want:
            # parallel sums round differently: accept only a neighbour in the walk
            # whose cumulative boundary lies within rounding of the draw
            p = np.exp((logits[b].double().numpy() - float(logits[b].max())) / T)
            kept = np.sort(np.argsort(-p, kind="stable")[: top_k or V]) if top_p is None else None
            assert kept is not None, (b, got[b], want)
            cum = np.cumsum(p[kept])
            draw = float(u[b]) * cum[-1]
            i_w, i_g = int(np.searchsorted(kept, want)), int(np.searchsorted(kept, got[b]))
            assert abs(i_w - i_g) == 1 and abs(cum[min(i_w, i_g)] - draw) < 1e-5 * cum[-1], (b, got[b], want)
    if top_k == 1 or top_p == 0.0:
        assert got == [int(torch.nonzero(r == r.max())[0]) for r in logits]  # the most probable, lowest index


@pytest.mark.parametrize("B,V", [(450, 151936), (3, 17), (40, 4097), (700, 1000)])
def test_sampling_with_a_cut_of_its_own_in_every_row(B, V):
    """Rows of one call differ in temperature, top-k and top-p (some have none),
    rows are many enough (450 of 151,936) that the vocabulary is cut into larger chunks, a row
    has equal logits at its cut (the lowest indices stay) and one has entries
    of probability zero."""
    g = torch.Generator().manual_seed(B * 7 + V)
    logits = torch.randn(B, V, generator=g) * 3
    ks = [0, 1, 5, 50, V, V + 3, 0, 0]
    ps = [1.0, 1.0, 1.0, 0.9, 0.5, 0.0, 0.3, 0.97]
    ts = [0.8, 0.3, 1.0, 2.5]
    top_k = [ks[b % len(ks)] for b in range(B)]
    top_p = [ps[(b // 2) % len(ps)] for b in range(B)]
    temp = [ts[b % len(ts)] for b in range(B)]
    if V >= 16:
        logits[0, 3:12] = logits[0].max() + 0.5      # nine equal at the top
        top_k[0], top_p[0] = 5, 1.0                    # the cut falls among them
        logits[1, ::2] = float("-inf")                 # probability zero
        top_k[1], top_p[1] = 0, 1.0
    u = torch.rand(B, generator=g)
    u[0] = 0.99999994
    got = ops().sample(logits.to(DEV), torch.tensor(temp, device=DEV), u.to(DEV),
                       top_k=torch.tensor(top_k, dtype=torch.int32, device=DEV),
                       top_p=torch.tensor(top_p, device=DEV)).tolist()
    for b in (range(B) if B * V < 10_000_000 else list(range(16)) + list(range(16, B, 29))):
        k = top_k[b] if 0 < top_k[b] < V else None
        tp = top_p[b] if top_p[b] < 1.0 else None
        row = logits[b].numpy()
        want = pm.sample_token(row, temp[b], float(u[b]), k, tp)
        if got[b] == want:
            continue
        # sums taken in another order round differently: only where the draw lies within
        # rounding of a boundary of the walk may the neighbouring kept entry come out
        p = np.exp((row.astype(np.float64) - float(row.max())) / temp[b])
        order = np.lexsort((np.arange(V), -p))
        n_keep = k or V
        if tp is not None:
            cum = np.cumsum(p[order] / p.sum())
            n_p = int(np.searchsorted(cum, tp, side="left")) + 1
            assert abs(cum[n_p - 1] - tp) > 1e-6, "the cut itself lies within rounding: choose another seed"
            n_keep = min(n_keep, max(1, n_p))
        kept = np.sort(order[:n_keep])
        assert got[b] in kept, (b, got[b], want)
        cum = np.cumsum(p[kept])
        draw = float(u[b]) * cum[-1]
        i_w, i_g = int(np.searchsorted(kept, want)), int(np.searchsorted(kept, got[b]))
        assert abs(i_w - i_g) == 1 and abs(cum[min(i_w, i_g)] - draw) < 1e-5 * cum[-1], (b, got[b], want)
    if V >= 16:
        assert got[0] in range(3, 8)   # of the nine equal entries the five lowest indices are kept
        assert got[1] % 2 == 1


def test_sampling_distribution():
    V, n = 50, 4000
    g = torch.Generator().manual_seed(9)
    row = torch.randn(V, generator=g) * 2
    logits = row.repeat(n, 1).to(DEV)
    u = ((torch.arange(n) + 0.5) / n).to(DEV)
    got = ops().sample(logits, torch.full((n,), 0.7, device=DEV), u).cpu().numpy()
    p = np.exp(row.double().numpy() / 0.7)
    p /= p.sum()
    np.testing.assert_allclose(np.bincount(got, minlength=V) / n, p, atol=1.5e-3)


# ------------------------------------------------------------------ bounded waits


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """One block waits a millisecond on a barrier that nothing signals.  The
    wait gives up, the kernel records it and returns; the host reads the
    device's error word as an exception, once, and later work is right."""
    import helpers
    from reflex_b200.errors import CudaError

    o = ops()
    o.check_device_errors(DEV)
    o.wait_probe(1_000_000, DEV)
    torch.cuda.synchronize()
    with pytest.raises(CudaError, match="bounded wait"):
        o.check_device_errors(DEV)
    o.check_device_errors(DEV)  # reported once, then clear

    engine = helpers.make_engine(helpers.model_folder("A", 7, "bfloat16"), "bfloat16")
    o.wait_probe(1_000_000, DEV)
    with pytest.raises(CudaError, match="bounded wait"):
        engine.check_errors()
    tokens = helpers.random_tokens(40, 512, 3)
    got = helpers.run_whole(engine, tokens)
    engine.check_errors()
    assert helpers.rel_err(got, helpers.plain_logits(helpers.model_folder("A", 7, "bfloat16"), tokens)) < 1.5e-2


# ------------------------------------------ the 32-bit kernels, bit for bit
def _bits_equal(got: torch.Tensor, ref: np.ndarray) -> bool:
    return np.array_equal(got.float().cpu().numpy(), ref)


@pytest.mark.parametrize("R,H", [(1, 64), (3, 100), (5, 4096), (300, 72), (2, 8200)])
def test_f32_rmsnorm_equals_the_host_mirror(R, H):
    import fp32_mirror as mir

    g = torch.Generator().manual_seed(H)
    x, d = torch.randn(R, H, generator=g) * 3, torch.randn(R, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    xd = x.to(DEV).clone()
    out = ops().rmsnorm(xd, w.to(DEV), 1e-5, torch.float32, delta=d.to(DEV), weight_offset=1.0)
    ref, t = mir.rms_norm(x.numpy(), w.numpy(), 1e-5, delta=d.numpy(), w_offset=1.0)
    assert _bits_equal(out, ref) and _bits_equal(xd, t)


@pytest.mark.parametrize("R,N,K", [(1, 7, 5), (65, 130, 257), (3, 1000, 96)])
def test_f32_product_and_swiglu_equal_the_host_mirror(R, N, K):
    import fp32_mirror as mir

    g = torch.Generator().manual_seed(N)
    x, W = torch.randn(R, K, generator=g), torch.randn(N, K, generator=g)
    assert _bits_equal(ops().linear(x.to(DEV), W.to(DEV)), mir.linear(x.numpy(), W.numpy()))
    gu = torch.randn(R, 2 * N, generator=g) * 8
    gu[0, :4] = torch.tensor([100.0, -100.0, 0.0, -0.0])
    got = ops().swiglu(gu.to(DEV))
    assert _bits_equal(got, mir.swiglu_act(gu[:, :N].numpy(), gu[:, N:].numpy()))


@pytest.mark.parametrize("nq,nkv,d,rd,pairing,magnitude", [
    (4, 2, 16, 16, "half", 1.0), (6, 1, 32, 32, "half", 1.0), (3, 1, 48, 32, "half", 1.0),
    (32, 8, 128, 128, "half", 1.0), (5, 5, 80, 80, "consecutive", 1.0), (4, 2, 64, 32, "consecutive", 1.25),
    (2, 1, 256, 256, "half", 0.75)])
def test_f32_qkv_post_equals_the_host_mirror_with_every_pairing(nq, nkv, d, rd, pairing, magnitude):
    """Norm, rotation (both pairings, a magnitude other than 1) and the cache
    write of the 32-bit form, bit for bit; and the bfloat16 form of the same
    call within its rounding of it."""
    import fp32_mirror as mir
    from reflex_b200.parts import Rotation

    g = torch.Generator().manual_seed(nq * 13 + d)
    positions = [0, 1, 63, 64, 200, 3000, 40959]
    R = len(positions)
    qkv = torch.randn(R, (nq + 2 * nkv) * d, generator=g) * 2
    qw, kw = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    denom = mir.rope_denominators(1e6, rd)
    pos_pages = 40960 // 64
    table = torch.arange(pos_pages, dtype=torch.int32).reshape(1, pos_pages) % 8
    # every used page index maps to its own page
    for i, p in enumerate(sorted({p // 64 for p in positions})):
        table[0, p] = i
    rot = Rotation(torch.from_numpy(denom).to(DEV), rd, pairing, magnitude)
    pair = 1 if pairing == "consecutive" else 0
    x = qkv.numpy()
    qr = mir.head_norm_rope(x[:, : nq * d].reshape(R, nq, d), qw.numpy(), 1e-6, denom, rd, positions, pair, magnitude)
    kr = mir.head_norm_rope(x[:, nq * d:(nq + nkv) * d].reshape(R, nkv, d), kw.numpy(), 1e-6, denom, rd, positions,
                            pair, magnitude)
    for dtype in (torch.float32, torch.bfloat16):
        kp = torch.zeros((8, nkv, 64, d), dtype=dtype, device=DEV)
        vp = torch.zeros((8, nkv, 64, d), dtype=dtype, device=DEV)
        q = ops().qkv_post(qkv.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, 0.0, rot,
                           torch.tensor(positions, dtype=torch.int32, device=DEV),
                           torch.zeros(R, dtype=torch.int32, device=DEV), kp, vp, table.to(DEV), 64, nq, nkv, d,
                           True, dtype)
        kgot = torch.stack([kp[int(table[0, p // 64]), :, p % 64] for p in positions])
        vgot = torch.stack([vp[int(table[0, p // 64]), :, p % 64] for p in positions])
        if dtype == torch.float32:
            assert _bits_equal(q.reshape(R, nq, d), qr) and _bits_equal(kgot, kr)
            assert _bits_equal(vgot, x[:, (nq + nkv) * d:].reshape(R, nkv, d))
        else:
            assert relerr(q.reshape(R, nq, d), qr.astype(np.float64)) < 8e-3
            assert relerr(kgot, kr.astype(np.float64)) < 8e-3
    # the rotation is what the formulas say: against the plain model where it has the pairing
    if pairing == "half" and magnitude == 1.0:
        ref = pm.rope_neox(pm.rms_norm(x[:, : nq * d].reshape(R, nq, d).astype(np.float64), qw.double().numpy(), 1e-6),
                           np.array(positions), 1e6, rd)
        assert np.abs(qr - ref).max() < 2e-2  # the 32-bit angle at position 40959
        assert np.abs(qr[:4] - ref[:4]).max() < 2e-5


@pytest.mark.parametrize("nq,nkv,d,T,window", [(4, 2, 16, 70, None), (6, 1, 32, 129, None), (3, 1, 48, 100, 37),
                                                (8, 2, 128, 66, 5), (2, 1, 80, 33, None)])
def test_f32_attention_equals_the_host_mirror(nq, nkv, d, T, window):
    import fp32_mirror as mir

    g = torch.Generator().manual_seed(nq * 31 + d)
    slots, table, kp, vp, ks, vs = _paged([T], nkv, d, torch.float32, g)
    q = torch.randn(T, nq, d, generator=g) * 3
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = ops().attention_plain(q.reshape(T, nq * d).to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV), 64,
                                i32(list(range(T))), i32([slots[0]] * T), nq, nkv, d, window, scale)
    ref = mir.attention(q.numpy(), ks[0].numpy(), vs[0].numpy(), scale, window)
    assert _bits_equal(out.reshape(T, nq, d), ref)


@pytest.mark.parametrize("P,K,V", [(1, 64, 50), (7, 100, 333), (5, 4096, 151936), (40, 1030, 1000)])
def test_gather_dot_reads_the_chosen_rows(P, K, V):
    """The gathered product against the full product at the chosen columns:
    the same bits in 32-bit, 32-bit accumulation of the same products in
    bfloat16; a row id outside the matrix is reported, not read."""
    g = torch.Generator().manual_seed(P + K)
    W = (torch.randn(V, K, generator=g) * 0.05)
    x = torch.randn(P, K, generator=g)
    ids = torch.randint(0, V, (P,), generator=g).int()
    ids[0] = V - 1
    got = ops().gather_dot(x.to(DEV), W.to(DEV), ids.to(DEV)).cpu()
    full = ops().linear(x.to(DEV), W[ids.long()].to(DEV)).cpu()  # [P, P]: the chosen rows only
    assert torch.equal(got, full.diagonal())
    xb, Wb = x.bfloat16(), W.bfloat16()
    got = ops().gather_dot(xb.to(DEV), Wb.to(DEV), ids.to(DEV)).cpu()
    ref = (xb.double() * Wb[ids.long()].double()).sum(dim=1)
    assert relerr(got, ref.numpy()) < 2e-6
    ops().check_device_errors(DEV)
    bad = ids.clone()
    bad[P - 1] = V
    out = ops().gather_dot(x.to(DEV), W.to(DEV), bad.to(DEV)).cpu()
    assert bool(torch.isnan(out[P - 1]))
    from reflex_b200 import CudaError

    with pytest.raises(CudaError):
        ops().check_device_errors(DEV)


@pytest.mark.parametrize("nq,nkv,d,K,R,writes,norm,rope", [
    (32, 8, 128, 4096, 8, True, True, True), (32, 8, 128, 4096, 1, True, True, True),
    (32, 8, 128, 4096, 64, True, True, True), (40, 8, 128, 1024, 33, True, True, True),
    (6, 2, 64, 96, 5, True, True, True), (3, 1, 64, 200, 17, True, True, True),
    (4, 4, 128, 64, 3, False, True, True), (5, 1, 64, 320, 9, True, False, True),
    (2, 2, 128, 128, 16, True, True, False)])
def test_the_qkv_product_finished_per_head_equals_product_then_qkv_post(nq, nkv, d, K, R, writes, norm, rope):
    """The decode step's q/k/v product with the per-head norms, the rotation and
    the cache write as its epilogue, against the product followed by `qkv_post`
    (the same formulas, sums in another order) and against the plain formulas;
    with and without a norm folded into its prologue; untouched cache rows stay."""
    from reflex_b200.parts import Rotation

    g = torch.Generator().manual_seed(nq * 7 + d + R)
    nkv_in = nkv if writes else 0
    N = (nq + 2 * nkv_in) * d
    x = torch.randn(R, K, generator=g).bfloat16()
    W = (torch.randn(N, K, generator=g) * (2.0 / math.sqrt(K))).bfloat16()
    qw = (1 + 0.1 * torch.randn(d, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)) if norm else None
    theta, eps = 1e6, 1e-6
    denom = torch.pow(torch.tensor(theta, dtype=torch.float64), torch.arange(d // 2, dtype=torch.float64) * 2 / d)
    rot = Rotation(denom.float().to(DEV), d) if rope else None
    positions = [(37 * i + 5) % 700 for i in range(R)]
    n_pages = 700 // 64 + 1
    slots = list(range(R))
    table = (torch.arange(R * n_pages, dtype=torch.int32).reshape(R, n_pages))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)

    def run(fused, xin):
        kp = torch.full((R * n_pages, nkv, 64, d), 7.0, dtype=torch.bfloat16, device=DEV)
        vp = torch.full((R * n_pages, nkv, 64, d), 7.0, dtype=torch.bfloat16, device=DEV)
        args = (dev(qw), dev(kw), eps, 0.0, rot, i32(positions), i32(slots), kp, vp, table.to(DEV), 64, nq, nkv, d, writes)
        if fused:
            assert ops().qkv_fused_takes(xin, d, rot, W) == (R <= ops().FUSE_QKV_ROWS)  # the engine's rule
            q = ops().qkv_fused(xin, W.to(DEV), *args)  # the kernel itself takes up to 64 rows
        else:
            qkv = ops().linear(xin, W.to(DEV), out_dtype=torch.float32)
            q = ops().qkv_post(qkv, *args, torch.bfloat16)
        ops().check_device_errors(DEV)
        return q.float().cpu(), kp.float().cpu(), vp.float().cpu()

    q1, k1, v1 = run(True, x.to(DEV))
    q0, k0, v0 = run(False, x.to(DEV))
    scale = float(q0.abs().max())
    assert float((q1 - q0).abs().max()) < 1e-2 * scale
    assert float((k1 - k0).abs().max()) < 1e-2 * max(scale, 7.0) and float((v1 - v0).abs().max()) < 1e-2 * 7.0
    # against the plain formulas
    y = x.double().numpy() @ W.double().numpy().T
    pos = np.array(positions)
    qr = y[:, : nq * d].reshape(R, nq, d)
    if norm:
        qr = pm.rms_norm(qr, qw.double().numpy(), eps)
    if rope:
        qr = pm.rope_neox(qr, pos, theta, d)
    assert relerr(q1.reshape(R, nq, d), qr) < 8e-3
    if writes:
        kr = y[:, nq * d:(nq + nkv) * d].reshape(R, nkv, d)
        if norm:
            kr = pm.rms_norm(kr, kw.double().numpy(), eps)
        if rope:
            kr = pm.rope_neox(kr, pos, theta, d)
        vr = y[:, (nq + nkv) * d:].reshape(R, nkv, d)
        touched = torch.zeros(R * n_pages, 64, dtype=torch.bool)
        for i, p in enumerate(positions):
            page = int(table[i, p // 64])
            assert relerr(k1[page, :, p % 64], kr[i]) < 8e-3 and relerr(v1[page, :, p % 64], vr[i]) < 8e-3
            touched[page, p % 64] = True
        rest = ~touched[:, None, :, None].expand(R * n_pages, nkv, 64, d)
        assert bool((k1[rest] == 7.0).all()) and bool((v1[rest] == 7.0).all())
    # with the input norm folded in: rows that await their factor, from the product before
    if K % 8 == 0 and K >= 64:
        xr = torch.randn(R, 64, generator=g).bfloat16()
        wr = (torch.randn(K, 64, generator=g) * 0.1).bfloat16()
        h = torch.randn(R, K, generator=g) * 2
        nw = 1 + 0.1 * torch.randn(K, generator=g)
        outs = []
        for fused in (True, False):
            ni = ops().gemm_tc_residual(xr.to(DEV), wr.to(DEV), h.to(DEV).clone(), nw.to(DEV), 0.0, 1e-5)
            outs.append(run(fused, ni))
        assert float((outs[0][0] - outs[1][0]).abs().max()) < 1e-2 * float(outs[1][0].abs().max())
        assert float((outs[0][1] - outs[1][1]).abs().max()) < 1e-2 * 7.0
