"""Each part of a layer alone against the plain implementation, the run order as
data (a layer named twice, a layer reading another layer's cache), and a toy
mixer with state of its own that is defined here, registered, built and stepped
without a change to the framework's files."""

import math
import os

import numpy as np
import pytest
import torch

import helpers
import plain_model as pm
from tiny_configs import TINY_B

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def relerr(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else got
    return float(np.abs(got - ref).max() / np.abs(ref).max())


def test_norm_rope_and_mlp_parts():
    from reflex_b200.config.spec import FeedForwardSpec, NormSpec, PositionSpec
    from reflex_b200.parts import FEED_FORWARDS, NORMS, POSITIONS

    g = torch.Generator().manual_seed(0)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 1.2e-2)):
        norm = NORMS.get("rmsnorm")(NormSpec("rmsnorm", 72, 1e-4), dtype, DEV)
        w = 1 + 0.1 * torch.randn(72, generator=g)
        norm.bind({"weight": w.to(dtype)})
        x = torch.randn(5, 72, generator=g)
        out = norm(x.to(DEV))
        assert out.dtype == dtype
        assert relerr(out, pm.rms_norm(x.double().numpy(), w.to(dtype).double().numpy(), 1e-4)) < max(tol, 5e-3 if dtype == torch.bfloat16 else 0)

        spec = FeedForwardSpec("swiglu", hidden_size=72, intermediate_size=136)
        mlp = FEED_FORWARDS.get("swiglu")(spec, dtype, DEV)
        ws = {k: (torch.randn(*i.shape, generator=g) * 0.1).to(dtype) for k, i in mlp.tensor_specs(spec).items()}
        mlp.bind(ws)
        xin = torch.randn(7, 72, generator=g).to(dtype)
        got = mlp.forward(xin.to(DEV))
        assert got.dtype == torch.float32  # the delta joins the 32-bit residual stream
        ref = pm.swiglu(xin.double().numpy(), *(ws[k].double().numpy() for k in ("gate_proj", "up_proj", "down_proj")))
        assert relerr(got, ref) < tol

    rope = POSITIONS.get("rope_neox")(PositionSpec("rope_neox", head_dim=48, rotary_dim=32, theta=5e4), torch.float32, DEV)
    rot = rope.rotation()
    denom, rd = rot.denominators, rot.rotary_dim
    assert rd == 32 and denom.dtype == torch.float32 and rot.pairing == "half" and rot.magnitude == 1.0
    want = np.power(5e4, np.arange(16) * 2.0 / 32)
    np.testing.assert_allclose(denom.cpu().numpy(), want, rtol=1e-7)


def _one_layer_engine(dtype, run_order=None, n_layers=1):
    """TINY_B's sizes with `n_layers` layers and an optional run order."""
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config import RunEntry, spec_from_config_dict
    from reflex_b200.engine import CausalLM, Engine
    from reflex_b200.weights import random_tensors

    cfg = dict(TINY_B, num_hidden_layers=n_layers)
    _, spec = spec_from_config_dict(cfg)
    if run_order is not None:
        spec.run_order = [RunEntry(*r) for r in run_order]
    model = CausalLM(spec, dtype, DEV)
    tensors = dict(random_tensors(spec, 3, torch.float32))
    # sharpen the attention so that the cache matters; in float32 only: a peaked
    # softmax multiplies bfloat16's rounding noise layer after layer
    if dtype == torch.float32:
        for k in tensors:
            if k.endswith(("q_norm.weight", "k_norm.weight")):
                tensors[k] = tensors[k] * 2.5
    if dtype == torch.bfloat16:
        tensors = {k: v.bfloat16() for k, v in tensors.items()}
    model.bind(tensors)
    w = {k: v.double().numpy() for k, v in tensors.items()}
    return cfg, w, Engine(model, max_tokens=512)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_and_block_against_the_plain_layer(dtype):
    """The pre-norm block with its attention and feed-forward, stepped through
    the cache in two chunks, against the plain decoder layer on the whole."""
    cfg, w, eng = _one_layer_engine(dtype)
    toks = helpers.random_tokens(70, cfg["vocab_size"], 1)
    from reflex_b200 import ops
    from reflex_b200.engine.batch import make_batch

    model, cache = eng.model, eng.cache
    s = cache.take_slot()
    hs = []
    for part, start in ((toks[:41], 0), (toks[41:], 41)):
        cache.reserve([(s, len(part))])
        batch = make_batch([part], [s], [start], [[0]], DEV)
        h, pending = model.hidden_states(batch, cache)
        # the last delta is still pending, unless the fused path already added it
        hs.append(h.clone() if pending is None or isinstance(pending, ops.NormedInput)
                  else ops.add_(h.clone(), pending))
        cache.commit([(s, len(part))])
    got = torch.cat(hs)
    h0 = w["model.embed_tokens.weight"][np.array(toks)]
    ref = pm.decoder_layer(h0, w, "model.layers.0.", cfg, np.arange(70), None)
    assert relerr(got, ref) < (3e-6 if dtype == torch.float32 else 1.5e-2)
    cache.give_slot(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_run_order_is_data_a_layer_twice_and_a_shared_cache(dtype):
    """Run order [L0, L1, L0 again with a cache entry of its own, L1 reading the
    keys and values that its first run wrote] against the same order spelled out
    with the plain implementation's parts."""
    order = [(0, 0, True), (1, 1, True), (0, 2, True), (1, 1, False)]
    cfg, w, eng = _one_layer_engine(dtype, run_order=order, n_layers=2)
    assert len(eng.cache.kv_groups) == 1 and len(eng.cache.kv_groups[0].entries) == 3
    toks = helpers.random_tokens(45, cfg["vocab_size"], 2)
    got = helpers.run_tail_one_by_one(eng, toks, tail=20)

    nq, nkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    T = len(toks)
    pos = np.arange(T)
    h = w["model.embed_tokens.weight"][np.array(toks)]
    kv_of_run1 = None
    for layer, _cache, writes in order:
        p = f"model.layers.{layer}."
        x = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = pm.rope_neox(pm.rms_norm((x @ w[p + "self_attn.q_proj.weight"].T).reshape(T, nq, d),
                                     w[p + "self_attn.q_norm.weight"], eps), pos, cfg["rope_theta"], d)
        if writes:
            k = pm.rope_neox(pm.rms_norm((x @ w[p + "self_attn.k_proj.weight"].T).reshape(T, nkv, d),
                                         w[p + "self_attn.k_norm.weight"], eps), pos, cfg["rope_theta"], d)
            v = (x @ w[p + "self_attn.v_proj.weight"].T).reshape(T, nkv, d)
            if layer == 1:
                kv_of_run1 = (k, v)
        else:
            k, v = kv_of_run1
        a = pm.causal_attention(q, k, v, 1 / math.sqrt(d), None).reshape(T, nq * d)
        h = h + a @ w[p + "self_attn.o_proj.weight"].T
        x = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + pm.swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    ref = pm.rms_norm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T
    assert helpers.rel_err(got, ref) < (2e-5 if dtype == torch.float32 else 1.5e-2)


def _toy_ema_class():
    """Registers (once more, harmlessly) and returns a toy mixer: an exponential
    moving average over a sequence's tokens: state [hidden] per sequence, fixed
    size, zero at the start, updated token by token."""
    from reflex_b200.cache import StateSpec
    from reflex_b200.parts import TensorInfo, register_mixer

    @register_mixer("toy_ema")
    class ToyEma:
        # decode steps index the state with the step's device-side slots and never
        # wait for the host, so they may be captured into a CUDA graph
        capturable = True
        fail_after_update = False  # test switch: raise once the state has been changed

        def __init__(self, spec, dtype, device):
            self.spec, self.dtype, self.device = spec, dtype, device
            self.decay = dict(spec.params)["decay"]

        @classmethod
        def tensor_specs(cls, spec):
            return {"mix": TensorInfo((spec.hidden_size, spec.hidden_size), "matrix")}

        def cache_spec(self):
            return StateSpec((self.spec.hidden_size,), "float32")

        def bind(self, tensors):
            self.mix = tensors["mix"].to(self.device, torch.float32)

        def forward(self, x, ctx):
            b = ctx.batch
            xf = x.float()
            if b.is_decode:
                # one row a sequence: the state rows by the device's slot list
                slots = b.row_slot.long()
                state = ctx.state.index_select(0, slots) * self.decay + xf * (1 - self.decay)
                ctx.state.index_copy_(0, slots, state)
                out = state
            else:
                out = torch.empty((x.shape[0], self.spec.hidden_size), dtype=torch.float32, device=x.device)
                for i, slot in enumerate(b.slots):  # each sequence's rows, in order
                    state = ctx.state[slot]
                    for r in range(b.row0[i], b.row0[i + 1]):
                        state.mul_(self.decay).add_(xf[r], alpha=1 - self.decay)
                        out[r] = state
            if ToyEma.fail_after_update:
                raise RuntimeError("toy failure after the state was updated")
            return out @ self.mix.T

    return ToyEma


def _toy_ema_model(dtype):
    """Two layers of the toy mixer with the library's SwiGLU and norms."""
    from reflex_b200.config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec
    from reflex_b200.engine import CausalLM, expected_tensors
    from reflex_b200.weights import random_tensors

    ToyEma = _toy_ema_class()
    H, V = 40, 97
    mixer = MixerSpec("toy_ema", hidden_size=H, names=(("mix", "ema.mix.weight"),), params=(("decay", 0.75),))
    ffn = FeedForwardSpec("swiglu", H, 56, names=(("gate_proj", "ff.g"), ("up_proj", "ff.u"), ("down_proj", "ff.d")))
    layers = [LayerSpec("prenorm", f"blocks.{i}.", mixer, ffn, NormSpec("rmsnorm", H, 1e-5), NormSpec("rmsnorm", H, 1e-5),
                        names=(("mixer_norm", "n1"), ("feed_forward_norm", "n2"))) for i in range(2)]
    spec = ModelSpec("toy", V, H, layers, NormSpec("rmsnorm", H, 1e-5), tie_word_embeddings=True, max_positions=256,
                     embedding_name="emb", final_norm_name="fn")
    assert "blocks.1.ema.mix.weight" in expected_tensors(spec)
    model = CausalLM(spec, dtype, DEV)
    tensors = {k: (v.to(dtype) if v.dim() > 1 else v) for k, v in random_tensors(spec, 1, torch.float32)}
    model.bind(tensors)
    w = {k: v.double().numpy() for k, v in tensors.items()}

    def plain(tokens):
        h = w["emb"][np.array(tokens)]
        for i in range(2):
            p = f"blocks.{i}."
            x = pm.rms_norm(h, w[p + "n1"], 1e-5)
            state, outs = np.zeros(H), []
            for t in range(len(tokens)):
                state = 0.75 * state + 0.25 * x[t]
                outs.append(state)
            h = h + np.stack(outs) @ w[p + "ema.mix.weight"].T
            x = pm.rms_norm(h, w[p + "n2"], 1e-5)
            h = h + pm.swiglu(x, w[p + "ff.g"], w[p + "ff.u"], w[p + "ff.d"])
        return pm.rms_norm(h, w["fn"], 1e-5) @ w["emb"].T

    return model, plain, ToyEma, V


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_toy_mixer_with_state_of_its_own(dtype):
    """Registered from here; config, weights, cache, step and replay take it as
    they take attention: in 32-bit, and in bfloat16 with the defaults, where its
    decode steps are captured into CUDA graphs (it declares `capturable` and
    reads its slots from the step's device-side indices)."""
    import reflex_b200
    from reflex_b200.engine import Engine

    model, plain, _, V = _toy_ema_model(dtype)
    eng = Engine(model, max_tokens=256)
    assert len(eng.cache.state_groups) == 1 and not eng.cache.kv_groups
    assert eng.use_graphs == (dtype == torch.bfloat16)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    reqs = [helpers.random_tokens(n, V, n) for n in (9, 3, 14, 6)]
    got = helpers.run_batches(eng, reqs, 2, [4, 3, 1])  # unequal batches, slots (and state) used again
    for r, g in zip(reqs, got):
        assert helpers.rel_err(g, plain(r)) < tol
    assert eng.cache.slots.held_count == 0
    if dtype == torch.bfloat16:
        assert eng._graphs and any(g.graph is not None for g in eng._graphs.values())
    # through the entry point, defaults: greedy ids against the plain model's
    api = reflex_b200.Model(model, max_tokens=512)
    prompts = [helpers.random_tokens(n, V, 50 + n) for n in (5, 11, 2)]
    outs = api.generate(prompts, 12)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            logits = plain(seq)[-1]
            best = pm.argmax_last(logits)
            assert tok == best or logits[best] - logits[tok] <= 2 * tol * np.abs(logits).max()
            seq.append(tok)


def test_a_failed_step_leaves_fixed_size_state_as_it_was():
    """A mixer that fails after it has updated its state: the step raises, and
    the sequence's state and length are what they were, so the same step run
    again gives what an undisturbed run gives."""
    from reflex_b200.engine import Engine

    model, plain, ToyEma, V = _toy_ema_model(torch.float32)
    eng = Engine(model, max_tokens=256)
    toks = helpers.random_tokens(12, V, 3)
    s = eng.open()
    eng.step([(s, toks[:7], [])])
    before = eng.cache.state_groups[0].data.clone()
    ToyEma.fail_after_update = True
    try:
        with pytest.raises(RuntimeError):
            eng.step([(s, toks[7:], [0])])
    finally:
        ToyEma.fail_after_update = False
    assert eng.length(s) == 7 and torch.equal(eng.cache.state_groups[0].data, before)
    out = eng.step([(s, toks[7:], list(range(5)))]).cpu().numpy()
    eng.close(s)
    assert helpers.rel_err(out, plain(toks)[7:]) < 1e-5


def rope_pairs(t, positions, theta, rotary_dim, factor, magnitude):
    """A rotary encoding with consecutive pairs (2i, 2i + 1), positions divided by
    `factor`, cos and sin times `magnitude` (src/model/config.rs:15-28 for the
    pairing, src/model/kernels.rs:3086-3129 for a magnitude other than 1)."""
    half = rotary_dim // 2
    denom = np.power(float(theta), 2.0 * np.arange(half) / rotary_dim) * factor
    ang = np.asarray(positions, dtype=np.float64)[:, None] / denom[None, :]
    c, s_ = (np.cos(ang) * magnitude)[:, None, :], (np.sin(ang) * magnitude)[:, None, :]
    out = t.copy()
    a, b = t[..., 0:rotary_dim:2], t[..., 1:rotary_dim:2]
    out[..., 0:rotary_dim:2] = a * c - b * s_
    out[..., 1:rotary_dim:2] = a * s_ + b * c
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_parts_chosen_layer_by_layer(dtype):
    """Parts registered from here and chosen layer by layer, in 32-bit and in
    bfloat16 through the entry point with its defaults: a feed-forward that
    routes each row to its best expert of three (router in 32-bit; it waits for
    the host, so it leaves `capturable` out and the engine captures nothing); a
    rotary encoding with consecutive pairs, divided positions and a magnitude
    other than 1; and a block arrangement with sandwich norms (a norm after the
    mixer and after the feed-forward, before the residual add) that reads its
    extra norms from the layer's record.  Layer 0 uses all three with windowed
    attention, layer 1 the library's own parts: one model, different mixers'
    options, feed-forwards and arrangements in different layers."""
    import reflex_b200
    from reflex_b200 import ops
    from reflex_b200.config.spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                                         PositionSpec, names_dict)
    from reflex_b200.engine import CausalLM, Engine
    from reflex_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, Rotation, TensorInfo, register_block,
                                   register_feed_forward, register_position)
    from reflex_b200.weights import random_tensors

    @register_feed_forward("toy_routed")
    class ToyRouted:
        def __init__(self, spec, dtype, device):
            self.spec, self.dtype, self.device = spec, dtype, device
            self.n_experts = dict(spec.params)["experts"]

        @classmethod
        def tensor_specs(cls, spec):
            E, H, I = dict(spec.params)["experts"], spec.hidden_size, spec.intermediate_size
            return {"router": TensorInfo((E, H), "matrix"), "w_in": TensorInfo((E * I, H), "matrix"),
                    "w_out": TensorInfo((E * H, I), "matrix")}

        def bind(self, tensors):
            E, H, I = self.n_experts, self.spec.hidden_size, self.spec.intermediate_size
            self.router = tensors["router"].to(self.device, torch.float32)
            self.w_in = tensors["w_in"].to(self.device, torch.float32).reshape(E, I, H)
            self.w_out = tensors["w_out"].to(self.device, torch.float32).reshape(E, H, I)

        def forward(self, x):
            xf = x.float()
            pick = (xf @ self.router.T).argmax(dim=1)  # router logits and choice in 32-bit
            out = torch.zeros((x.shape[0], self.spec.hidden_size), dtype=torch.float32, device=x.device)
            for e in range(self.n_experts):  # experts in a fixed order
                rows = (pick == e).nonzero()[:, 0]
                if rows.numel():
                    out[rows] = torch.relu(xf[rows] @ self.w_in[e].T) @ self.w_out[e].T
            return out

    @register_position("toy_rope_pairs")
    class ToyPairsRope:
        capturable = True

        def __init__(self, spec, dtype, device):
            self.spec = spec
            p = dict(spec.params)
            half = spec.rotary_dim // 2
            exps = torch.arange(half, dtype=torch.float64) * 2.0 / spec.rotary_dim
            self.denominators = (torch.pow(torch.tensor(spec.theta, dtype=torch.float64), exps) * p["factor"]).float().to(device)
            self.magnitude = p["magnitude"]

        @classmethod
        def tensor_specs(cls, spec):
            return {}

        def bind(self, tensors):
            pass

        def rotation(self):
            return Rotation(self.denominators, self.spec.rotary_dim, "consecutive", self.magnitude)

    @register_block("toy_sandwich")
    class ToySandwich:
        """h += post_mixer_norm(mixer(norm1(h))); h += post_ffn_norm(ffn(norm2(h)))."""

        def __init__(self, spec, dtype, device):
            self.spec = spec
            mk = lambda n: NORMS.get(n.kind)(n, dtype, device)
            self.norm1, self.norm2 = mk(spec.mixer_norm), mk(spec.feed_forward_norm)
            self.extra = {role: mk(n) for role, n in spec.extra_norms}
            self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device)
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)

        @property
        def capturable(self):
            return all(getattr(p, "capturable", False) for p in
                       (self.norm1, self.norm2, self.mixer, self.feed_forward, *self.extra.values()))

        @classmethod
        def tensor_names(cls, spec):
            out, bn = {}, names_dict(spec.names)
            for part, n in (("mixer_norm", spec.mixer_norm), ("feed_forward_norm", spec.feed_forward_norm), *spec.extra_norms):
                out[spec.prefix + bn[part]] = (part, "weight", NORMS.get(n.kind).tensor_specs(n)["weight"])
            for part, sp, reg in (("mixer", spec.mixer, MIXERS), ("feed_forward", spec.feed_forward, FEED_FORWARDS)):
                nd = names_dict(sp.names)
                for role, info in reg.get(sp.kind).tensor_specs(sp).items():
                    out[spec.prefix + nd.get(role, role)] = (part, role, info)
            return out

        def bind(self, by_part):
            self.norm1.bind(by_part["mixer_norm"])
            self.norm2.bind(by_part["feed_forward_norm"])
            for role, n in self.extra.items():
                n.bind(by_part[role])
            self.mixer.bind(by_part["mixer"])
            self.feed_forward.bind(by_part["feed_forward"])

        def forward(self, hidden, pending, ctx):
            x = self.norm1(hidden, delta=pending)  # adds what the block before left, then norms
            a = self.mixer.forward(x, ctx)
            ops.add_(hidden, self.extra["post_mixer_norm"](a.float()))
            x = self.norm2(hidden)
            f = self.feed_forward.forward(x)
            return hidden, self.extra["post_ffn_norm"](f.float())

    H, V, nq, nkv, d, I, E = 48, 101, 3, 1, 32, 40, 3
    theta, factor, magnitude, window, eps = 1e4, 4.0, 1.1, 9, 1e-5
    names = (("q_proj", "att.q"), ("k_proj", "att.k"), ("v_proj", "att.v"), ("o_proj", "att.o"),
             ("q_norm", "att.qn"), ("k_norm", "att.kn"))

    def mixer(position_kind, params, win):
        return MixerSpec("gqa_attention", hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                         scale=d ** -0.5, window=win, qk_norm=NormSpec("rmsnorm", d, eps),
                         position=PositionSpec(position_kind, d, d, theta, params=params), names=names)

    routed = FeedForwardSpec("toy_routed", H, I, names=(("router", "moe.r"), ("w_in", "moe.i"), ("w_out", "moe.o")),
                             params=(("experts", E),))
    dense = FeedForwardSpec("swiglu", H, 56, names=(("gate_proj", "ff.g"), ("up_proj", "ff.u"), ("down_proj", "ff.d")))
    norm = NormSpec("rmsnorm", H, eps)
    lnames = (("mixer_norm", "n1"), ("feed_forward_norm", "n2"))
    layers = [LayerSpec("toy_sandwich", "blocks.0.", mixer("toy_rope_pairs", (("factor", factor), ("magnitude", magnitude)), window),
                        routed, norm, norm, names=lnames + (("post_mixer_norm", "n3"), ("post_ffn_norm", "n4")),
                        extra_norms=(("post_mixer_norm", norm), ("post_ffn_norm", norm))),
              LayerSpec("prenorm", "blocks.1.", mixer("rope_neox", (), None), dense, norm, norm, names=lnames)]
    spec = ModelSpec("toy2", V, H, layers, norm, tie_word_embeddings=False, max_positions=256,
                     embedding_name="emb", final_norm_name="fn", head_name="head")
    model = CausalLM(spec, dtype, DEV)
    tensors = dict(random_tensors(spec, 3, torch.float32))
    # spread the router so that choices are clear of ties, also after bfloat16's rounding
    tensors["blocks.0.moe.r"] = tensors["blocks.0.moe.r"] * 50
    tensors = {k: (v.to(dtype) if v.dim() > 1 else v) for k, v in tensors.items()}
    model.bind(tensors)
    assert not model.capturable
    eng = Engine(model, max_tokens=512)
    assert not eng.use_graphs
    assert len(eng.cache.kv_groups) == 2  # a windowed group and a full one, storage of their own

    w = {k: v.double().numpy() for k, v in tensors.items()}
    margins = []

    def attention(h, p, rope, win):
        T = h.shape[0]
        x = pm.rms_norm(h, w[p + "n1"], eps)
        q = pm.rms_norm((x @ w[p + "att.q"].T).reshape(T, nq, d), w[p + "att.qn"], eps)
        k = pm.rms_norm((x @ w[p + "att.k"].T).reshape(T, nkv, d), w[p + "att.kn"], eps)
        v = (x @ w[p + "att.v"].T).reshape(T, nkv, d)
        q, k = rope(q), rope(k)
        return pm.causal_attention(q, k, v, d ** -0.5, win).reshape(T, nq * d) @ w[p + "att.o"].T

    def plain(tokens):
        T = len(tokens)
        pos = np.arange(T)
        h = w["emb"][np.array(tokens)]
        a = attention(h, "blocks.0.", lambda t: rope_pairs(t, pos, theta, d, factor, magnitude), window)
        h = h + pm.rms_norm(a, w["blocks.0.n3"], eps)
        x = pm.rms_norm(h, w["blocks.0.n2"], eps)
        r = x @ w["blocks.0.moe.r"].T
        top = np.sort(r, axis=1)
        margins.append(float((top[:, -1] - top[:, -2]).min()))
        pick = r.argmax(axis=1)
        w_in, w_out = w["blocks.0.moe.i"].reshape(E, I, H), w["blocks.0.moe.o"].reshape(E, H, I)
        f = np.stack([np.maximum(x[t] @ w_in[pick[t]].T, 0) @ w_out[pick[t]].T for t in range(T)])
        h = h + pm.rms_norm(f, w["blocks.0.n4"], eps)
        h = h + attention(h, "blocks.1.", lambda t: pm.rope_neox(t, pos, theta, d), None)
        x = pm.rms_norm(h, w["blocks.1.n2"], eps)
        h = h + pm.swiglu(x, w["blocks.1.ff.g"], w["blocks.1.ff.u"], w["blocks.1.ff.d"])
        return pm.rms_norm(h, w["fn"], eps) @ w["head"].T

    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    reqs = [helpers.random_tokens(n, V, n) for n in (23, 5, 40, 12)]
    refs = [plain(r) for r in reqs]
    assert min(margins) > 0.05, "a router choice is too close to a tie for bfloat16 to keep"
    got = helpers.run_batches(eng, reqs, 2, [6, 3, 1])
    for ref, g in zip(refs, got):
        assert helpers.rel_err(g, ref) < tol
    whole = helpers.run_whole(eng, reqs[2])
    assert helpers.rel_err(whole, refs[2]) < tol
    assert eng.cache.slots.held_count == 0
    # through the entry point with its defaults
    api = reflex_b200.Model(model, max_tokens=1024)
    outs = api.generate([reqs[1], reqs[3]], 6)
    for p, o in zip((reqs[1], reqs[3]), outs):
        seq = list(p)
        for tok in o:
            logits = plain(seq)[-1]
            best = pm.argmax_last(logits)
            assert tok == best or logits[best] - logits[tok] <= 2 * tol * np.abs(logits).max()
            seq.append(tok)


@pytest.mark.parametrize("weights", ["f32", "bf16"])
def test_a_toy_architecture_from_config_json_to_generation(weights, tmp_path):
    """A whole architecture added from outside the framework: a typed config
    read from its own config.json keys, a builder that turns it into a
    `ModelSpec` (layers that alternate the toy state mixer and attention, a run
    order that names a layer twice), and a registry entry.  The framework's
    files stay as they are: the random-weights mode writes its model folder, the
    loader checks and binds it by tensor name, the cache gives it a state group
    beside a key/value group, and step, generation and candidate scoring run
    it, in both precisions, against a plain forward written here."""
    from dataclasses import dataclass

    import reflex_b200
    from reflex_b200 import CheckpointError
    from reflex_b200 import CheckpointError as ConfigError  # a malformed config.json is a checkpoint error
    from reflex_b200.config import RunEntry, register_architecture
    from reflex_b200.config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors

    _toy_ema_class()

    @dataclass
    class ToyConfig:
        vocab: int
        width: int
        kinds: tuple  # "ema" | "attention" per layer
        heads: int
        kv_heads: int
        head_size: int
        ff: int
        decay: float
        eps: float
        theta: float
        repeat_last: bool

        @classmethod
        def from_dict(cls, d):
            missing = [k for k in ("vocab", "width", "kinds", "ff") if k not in d]
            if missing:
                raise ConfigError(f"toy config.json lacks {missing}")
            return cls(d["vocab"], d["width"], tuple(d["kinds"]), d.get("heads", 2), d.get("kv_heads", 1),
                       d.get("head_size", 64), d["ff"], d.get("decay", 0.5), d.get("eps", 1e-5),
                       d.get("theta", 1e4), bool(d.get("repeat_last", False)))

        def to_dict(self):
            return {"architectures": ["ToyHybridForCausalLM"], "vocab": self.vocab, "width": self.width,
                    "kinds": list(self.kinds), "heads": self.heads, "kv_heads": self.kv_heads,
                    "head_size": self.head_size, "ff": self.ff, "decay": self.decay, "eps": self.eps,
                    "theta": self.theta, "repeat_last": self.repeat_last}

    def build(c: ToyConfig) -> ModelSpec:
        norm = NormSpec("rmsnorm", c.width, c.eps)
        ffn = FeedForwardSpec("swiglu", c.width, c.ff, names=(("gate_proj", "ff.gate"), ("up_proj", "ff.up"), ("down_proj", "ff.down")))
        layers = []
        for i, kind in enumerate(c.kinds):
            if kind == "ema":
                mixer = MixerSpec("toy_ema", hidden_size=c.width, names=(("mix", "ema.mix"),), params=(("decay", c.decay),))
            else:
                mixer = MixerSpec("gqa_attention", hidden_size=c.width, num_heads=c.heads, num_kv_heads=c.kv_heads,
                                  head_dim=c.head_size, scale=c.head_size ** -0.5,
                                  qk_norm=NormSpec("rmsnorm", c.head_size, c.eps),
                                  position=PositionSpec("rope_neox", c.head_size, c.head_size, c.theta),
                                  names=(("q_proj", "att.q"), ("k_proj", "att.k"), ("v_proj", "att.v"), ("o_proj", "att.o"),
                                         ("q_norm", "att.qn"), ("k_norm", "att.kn")))
            layers.append(LayerSpec("prenorm", f"toy.{i}.", mixer, ffn, norm, norm,
                                    names=(("mixer_norm", "n1"), ("feed_forward_norm", "n2"))))
        order = [RunEntry(i, i) for i in range(len(layers))]
        if c.repeat_last:  # the last layer once more, with its own cache entry: weights shared
            order.append(RunEntry(len(layers) - 1, len(layers)))
        return ModelSpec("toy_hybrid", c.vocab, c.width, layers, norm, tie_word_embeddings=False, max_positions=512,
                         embedding_name="toy.emb", final_norm_name="toy.norm", head_name="toy.head", run_order=order,
                         eos_token_ids=())

    register_architecture(("ToyHybridForCausalLM", "toy_hybrid"), ToyConfig.from_dict, build)

    cfg = {"architectures": ["ToyHybridForCausalLM"], "vocab": 211, "width": 72, "kinds": ["ema", "attention", "ema", "attention"],
           "heads": 2, "kv_heads": 1, "head_size": 64, "ff": 104, "decay": 0.6, "repeat_last": True}
    with pytest.raises(ConfigError):
        reflex_b200.config.spec_from_config_dict({"architectures": ["ToyHybridForCausalLM"], "vocab": 5})
    folder = str(tmp_path / "toy")
    write_random_model(cfg, 5, folder, "float32" if weights == "f32" else "bfloat16")
    model = reflex_b200.Model.load(folder, weights=weights, max_tokens=2048)
    eng = model.engine
    assert len(eng.cache.state_groups) == 1 and len(eng.cache.kv_groups) == 1
    assert eng.use_graphs == (weights == "bf16")

    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    w = {k: f.tensor(k).double().numpy() for k in f.keys()}
    f.close()
    H, d, nq, nkv = 72, 64, 2, 1

    def plain(tokens):
        T = len(tokens)
        pos = np.arange(T)
        h = w["toy.emb"][np.array(tokens)]
        for li in (0, 1, 2, 3, 3):
            p = f"toy.{li}."
            x = pm.rms_norm(h, w[p + "n1"], 1e-5)
            if cfg["kinds"][li] == "ema":
                state, outs = np.zeros(H), []
                for t in range(T):
                    state = 0.6 * state + 0.4 * x[t]
                    outs.append(state)
                h = h + np.stack(outs) @ w[p + "ema.mix"].T
            else:
                q = pm.rms_norm((x @ w[p + "att.q"].T).reshape(T, nq, d), w[p + "att.qn"], 1e-5)
                k = pm.rms_norm((x @ w[p + "att.k"].T).reshape(T, nkv, d), w[p + "att.kn"], 1e-5)
                v = (x @ w[p + "att.v"].T).reshape(T, nkv, d)
                q, k = pm.rope_neox(q, pos, 1e4, d), pm.rope_neox(k, pos, 1e4, d)
                h = h + pm.causal_attention(q, k, v, d ** -0.5, None).reshape(T, nq * d) @ w[p + "att.o"].T
            x = pm.rms_norm(h, w[p + "n2"], 1e-5)
            h = h + pm.swiglu(x, w[p + "ff.gate"], w[p + "ff.up"], w[p + "ff.down"])
        return pm.rms_norm(h, w["toy.norm"], 1e-5) @ w["toy.head"].T

    tol = 1e-5 if weights == "f32" else 1.5e-2
    reqs = [helpers.random_tokens(n, 211, 40 + n) for n in (70, 3, 33, 9)]
    got = helpers.run_batches(eng, reqs, 2, [20, 3, 1])
    for r, g in zip(reqs, got):
        assert helpers.rel_err(g, plain(r)) < tol
    assert eng.cache.slots.held_count == 0
    if weights == "bf16":
        assert any(g.graph is not None for g in eng._graphs.values())
    outs = model.generate([reqs[1], reqs[3]], 8)
    for p, o in zip((reqs[1], reqs[3]), outs):
        seq = list(p)
        for tok in o:
            logits = plain(seq)[-1]
            best = pm.argmax_last(logits)
            assert tok == best or logits[best] - logits[tok] <= 2 * tol * np.abs(logits).max()
            seq.append(tok)
    # candidate scoring teacher-forces a continuation: the state mixer sees its tokens in order
    res = model.system1_evaluate(reqs[3], [[5, 6, 7], [100]])
    full = plain(reqs[3] + [5, 6])
    want = float(full[len(reqs[3]) - 1, 5] + full[len(reqs[3]), 6] + full[len(reqs[3]) + 1, 7])
    assert abs(res.results[0].score - want) < 3 * tol * np.abs(full).max()
    # the loader's one error still names what is wrong with this architecture's checkpoint
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = [(k, f.tensor(k).clone()) for k in f.keys() if k != "toy.1.att.qn"] + [("toy.extra", torch.zeros(2))]
    f.close()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(CheckpointError) as e:
        reflex_b200.Model.load(folder, weights=weights)
    assert "toy.1.att.qn" in str(e.value) and "toy.extra" in str(e.value)


def test_a_cache_group_whose_values_are_smaller_than_its_keys():
    """A toy mixer that keeps a compressed value per position: its `KVSpec` asks
    for 32-element keys and 8-element values.  The cache gives it pages of both
    shapes under one page table; it reads and writes them with the step's
    device-side positions and slots, and the model steps like any other."""
    from reflex_b200.cache import KVSpec
    from reflex_b200.config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec
    from reflex_b200.engine import CausalLM, Engine
    from reflex_b200.parts import TensorInfo, register_mixer
    from reflex_b200.weights import random_tensors

    DK, DV = 32, 8

    @register_mixer("toy_latent_attention")
    class ToyLatent:
        """One head; keys [DK], values compressed to [DV] and expanded after the
        weighted sum; plain causal softmax attention."""

        def __init__(self, spec, dtype, device):
            self.spec, self.dtype, self.device = spec, dtype, device

        @classmethod
        def tensor_specs(cls, spec):
            H = spec.hidden_size
            return {"wq": TensorInfo((DK, H), "matrix"), "wk": TensorInfo((DK, H), "matrix"),
                    "wv": TensorInfo((DV, H), "matrix"), "wo": TensorInfo((H, DV), "matrix")}

        def cache_spec(self):
            return KVSpec(1, DK, None, v_head_dim=DV)

        def bind(self, tensors):
            self.w = {k: v.to(self.device, torch.float32) for k, v in tensors.items()}

        def forward(self, x, ctx):
            kv, b = ctx.kv, ctx.batch
            assert kv.k_pages.shape[-1] == DK and kv.v_pages.shape[-1] == DV
            xf = x.float()
            q, k, v = xf @ self.w["wq"].T, xf @ self.w["wk"].T, xf @ self.w["wv"].T
            pos, slot = b.row_pos.long(), b.row_slot.long()
            page = kv.page_table[slot, pos // kv.page_size].long()
            kv.k_pages[page, 0, pos % kv.page_size] = k.to(kv.k_pages.dtype)
            kv.v_pages[page, 0, pos % kv.page_size] = v.to(kv.v_pages.dtype)
            out = torch.empty((x.shape[0], DV), dtype=torch.float32, device=x.device)
            for i, sl in enumerate(b.slots):  # a row at a time: a toy
                for r in range(b.row0[i], b.row0[i + 1]):
                    p = b.starts[i] + (r - b.row0[i])
                    idx = torch.arange(p + 1, device=x.device)
                    pg = kv.page_table[sl, idx // kv.page_size].long()
                    keys = kv.k_pages[pg, 0, idx % kv.page_size].float()
                    vals = kv.v_pages[pg, 0, idx % kv.page_size].float()
                    a = torch.softmax((keys @ q[r]) * DK ** -0.5, dim=0)
                    out[r] = a @ vals
            return out @ self.w["wo"].T

    H, V = 24, 53
    mixer = MixerSpec("toy_latent_attention", hidden_size=H,
                      names=(("wq", "a.q"), ("wk", "a.k"), ("wv", "a.v"), ("wo", "a.o")))
    ffn = FeedForwardSpec("swiglu", H, 40, names=(("gate_proj", "f.g"), ("up_proj", "f.u"), ("down_proj", "f.d")))
    norm = NormSpec("rmsnorm", H, 1e-5)
    layers = [LayerSpec("prenorm", f"l{i}.", mixer, ffn, norm, norm, names=(("mixer_norm", "n1"), ("feed_forward_norm", "n2")))
              for i in range(2)]
    spec = ModelSpec("toy_latent", V, H, layers, norm, tie_word_embeddings=True, max_positions=256,
                     embedding_name="emb", final_norm_name="fn")
    model = CausalLM(spec, torch.float32, DEV)
    tensors = dict(random_tensors(spec, 2, torch.float32))
    for k in tensors:
        if ".a." in k:
            tensors[k] = tensors[k] * 20  # attention that matters
    model.bind(tensors)
    eng = Engine(model, max_tokens=512)
    g = eng.cache.kv_groups[0]
    assert g.k.shape[-1] == DK and g.v.shape[-1] == DV
    w = {k: v.double().numpy() for k, v in tensors.items()}

    def plain(tokens):
        T = len(tokens)
        h = w["emb"][np.array(tokens)]
        for i in range(2):
            p = f"l{i}."
            x = pm.rms_norm(h, w[p + "n1"], 1e-5)
            q, k, v = x @ w[p + "a.q"].T, x @ w[p + "a.k"].T, x @ w[p + "a.v"].T
            a = pm.causal_attention(q[:, None, :], k[:, None, :], np.pad(v, ((0, 0), (0, DK - DV)))[:, None, :],
                                    DK ** -0.5, None)[:, 0, :DV]
            h = h + a @ w[p + "a.o"].T
            x = pm.rms_norm(h, w[p + "n2"], 1e-5)
            h = h + pm.swiglu(x, w[p + "f.g"], w[p + "f.u"], w[p + "f.d"])
        return pm.rms_norm(h, w["fn"], 1e-5) @ w["emb"].T

    reqs = [helpers.random_tokens(n, V, 70 + n) for n in (70, 4, 9)]
    got = helpers.run_batches(eng, reqs, 2, [66, 2, 1])
    for r, gl in zip(reqs, got):
        assert helpers.rel_err(gl, plain(r)) < 2e-5
    assert eng.cache.slots.held_count == 0
