"""Each part alone against its plain function, with sizes of its own; the order list (a layer
named twice, a run that reads another run's cache); and a toy mixer with state of its own that
is defined here, registered, built and stepped without a change to the framework's files."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import util
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def runtime(dtype, page=16):
    from air_b200.parts.base import Runtime
    return Runtime(torch.device("cuda"), DT[dtype], page)


def tensors_for(part, seed, dtype):
    from air_b200.weights.loader import random_tensors
    t = random_tensors(part.tensor_specs(), seed, DT[dtype], device="cpu")
    t = {k: (v * 4 if ("proj.weight" in k or "bias" in k) else v) for k, v in t.items()}   # not all near zero
    return {k: v.to(DT[dtype]) for k, v in t.items()}


def as_np(tensors):
    return {k: v.float().numpy() for k, v in tensors.items()}


def context_for(cache, entries, part=None):
    from air_b200.engine.batch import Entry, build_context
    entries = [Entry(*e) for e in entries]
    for e in entries:
        if e.request not in cache.sequences:
            cache.open(e.request)
    cache.reserve([(e.request, len(e.tokens)) for e in entries])
    ctx = build_context(entries, cache, "cuda", status=torch.zeros(1, dtype=torch.int32, device="cuda"),
                        planners=[part] if part is not None and part.plan_key() is not None else ())
    return ctx, entries


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_part(dtype):
    from air_b200.parts.norm import RMSNorm
    from air_b200.parts.spec import PartSpec
    part = RMSNorm(PartSpec("rms", {"size": 208, "eps": 3e-4}), "n.")
    t = tensors_for(part, 0, dtype)
    part.load({k: v.cuda() for k, v in t.items()}, runtime(dtype))
    h = torch.randn(9, 208, generator=torch.Generator().manual_seed(0))
    out = part.forward(h.cuda(), None)
    want = plain.rms_norm(h.numpy(), as_np(t)["n.weight"], 3e-4)
    assert out.dtype == DT[dtype]
    assert np.abs(out.float().cpu().numpy() - want).max() < (2e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from air_b200.parts.mlp import SwiGLU
    from air_b200.parts.spec import PartSpec
    part = SwiGLU(PartSpec("swiglu", {"hidden": 80, "intermediate": 208}), "f.")
    t = tensors_for(part, 1, dtype)
    part.load({k: v.cuda() for k, v in t.items()}, runtime(dtype))
    x = torch.randn(11, 80, generator=torch.Generator().manual_seed(1)).to(DT[dtype])
    out = part.forward(x.cuda(), None)
    out = out.sum(0) if out.dim() == 3 else out
    n = as_np(t)
    want = plain.swiglu(x.float().numpy(), n["f.gate_proj.weight"], n["f.up_proj.weight"], n["f.down_proj.weight"])
    assert out.dtype == torch.float32
    assert np.abs(out.cpu().numpy() - want).max() < (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max()
    if dtype == "bfloat16":
        # many rows and a residual stream in the context: the output is added into the stream (in 32-bit),
        # nothing is handed on
        from types import SimpleNamespace
        x = torch.randn(150, 80, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
        stream = torch.randn(150, 80, generator=torch.Generator().manual_seed(3))
        h = stream.clone().cuda()
        assert part.forward(x.cuda(), SimpleNamespace(residual=h)) is None
        want = stream.numpy() + plain.swiglu(x.float().numpy(), n["f.gate_proj.weight"], n["f.up_proj.weight"],
                                             n["f.down_proj.weight"])
        assert np.abs(h.cpu().numpy() - want).max() < 2e-2 * np.abs(want).max()
        handed_on = part.forward(x.cuda(), None)            # without a stream: as before
        assert np.abs(stream.numpy() + handed_on.cpu().numpy() - want).max() < 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("heads,kv,d,window", [(6, 2, 48, None), (5, 5, 16, 9), (4, 1, 80, None)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_over_portions(heads, kv, d, window, dtype):
    """The mixer alone, fed a sequence in three portions through a cache of its own, against the
    plain functions on the whole sequence."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.attention import Attention
    from air_b200.parts.spec import PartSpec
    hidden, T, theta = 112, 45, 777.0
    spec = PartSpec("attention", {"hidden": hidden, "heads": heads, "kv_heads": kv, "head_dim": d, "qkv_bias": True,
                                  "window": window,
                                  "position": PartSpec("rope_half", {"rotary_dim": d, "theta": theta,
                                                                     "max_positions": 64})})
    part = Attention(spec, "a.")
    t = tensors_for(part, 2, dtype)
    part.load({k: v.cuda() for k, v in t.items()}, runtime(dtype))
    cache = CacheManager([part.cache_needs()], 16, 8, 2, dtype=DT[dtype], device="cuda")
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    outs, i = [], 0
    for n in (20, 2, 23):
        ctx, entries = context_for(cache, [("r", [0] * n, [])], part)
        y = part.forward(x[i:i + n].cuda(), ctx, cache.views(0), True)
        outs.append((y.sum(0) if y.dim() == 3 else y).cpu())        # partial sums over parts of k are allowed
        cache.commit("r", n)
        i += n
    out = torch.cat(outs).numpy()
    w, xn = as_np(t), x.float().numpy()
    pos = np.arange(T)
    q = plain.rope(plain.linear(xn, w["a.q_proj.weight"], w["a.q_proj.bias"]).reshape(T, heads, d), pos, theta)
    k = plain.rope(plain.linear(xn, w["a.k_proj.weight"], w["a.k_proj.bias"]).reshape(T, kv, d), pos, theta)
    v = plain.linear(xn, w["a.v_proj.weight"], w["a.v_proj.bias"]).reshape(T, kv, d)
    want = plain.linear(plain.attention(q, k, v, window=window).reshape(T, heads * d), w["a.o_proj.weight"])
    assert np.abs(out - want).max() < (1e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()


def test_parts_refuse_impossible_sizes():
    from air_b200.parts.attention import Attention
    from air_b200.parts.spec import PartSpec
    pos = PartSpec("rope_half", {"rotary_dim": 24, "theta": 1e4, "max_positions": 8})
    with pytest.raises(ValueError, match="multiple of 16"):
        Attention(PartSpec("attention", {"hidden": 48, "heads": 2, "kv_heads": 1, "head_dim": 24, "position": pos}))
    with pytest.raises(ValueError, match="multiple of kv_heads"):
        Attention(PartSpec("attention", {"hidden": 48, "heads": 3, "kv_heads": 2, "head_dim": 16, "position": pos}))
    from air_b200.parts import registry
    with pytest.raises(KeyError, match="no mixer of kind"):
        registry.MIXERS.get("nothing")


# ------------------------------------------------------------------ the order list
def engine_with_order(name, order, dtype="float32"):
    import dataclasses
    from air_b200.config import load_config
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.model import Model
    from air_b200.parts import registry
    from air_b200.parts.base import Runtime
    from air_b200.parts.spec import RunStep
    from air_b200.weights.loader import load_tensors
    folder = util.model_folder(name)
    cfg = load_config(folder)
    spec = registry.architecture(cfg.architecture).build_spec(cfg)
    spec = dataclasses.replace(spec, order=tuple(RunStep(l, c) for l, c in order))
    model = Model(spec)
    rt = Runtime(torch.device("cuda"), DT[dtype], 16)
    model.load(load_tensors(folder, model.tensor_specs(), rt.dtype, rt.device), rt)
    return folder, Engine(model, EngineConfig(dtype=DT[dtype], page_tokens=16, max_tokens=256), cfg)


@pytest.mark.parametrize("order", [[(0, None), (1, None), (1, None), (0, None)],      # layers named twice
                                   [(0, None), (1, None), (2, 1), (0, 0)],             # runs that read another run's cache
                                   [(2, None)]])
def test_order_of_runs_is_data(order):
    from air_b200.engine.batch import Entry
    folder, engine = engine_with_order("B", order)
    toks = util.tokens_for("B", 50, 3)
    cfg, tensors = util.plain_model(folder)
    want = plain.forward(cfg, tensors, toks, order=order)
    got = [engine.step([Entry("r", toks[:31], range(31))]).cpu().numpy(),
           engine.step([Entry("r", toks[31:33], range(2))]).cpu().numpy()]
    got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[33:]]
    got = np.concatenate(got)
    assert np.abs(got - want).max() < util.FP32_TOL * max(1.0, np.abs(want).max())
    own = sum(1 for _, c in order if c is None)
    assert sum(len(g.runs) for g in engine.cache.groups) == own


def engine_and_weights(cfg, seed, dtype="float32", **kw):
    """An engine for a registered architecture with random weights drawn on the CPU, and those weights as
    float32 numpy arrays for an oracle written in the test."""
    from air_b200.config import load_config
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.model import Model
    from air_b200.parts import registry
    from air_b200.parts.base import Runtime
    from air_b200.weights.loader import random_tensors
    config = load_config(cfg)
    model = Model(registry.architecture(config.architecture).build_spec(config))
    tensors = random_tensors(model.tensor_specs(), seed, DT[dtype], device="cpu")
    tensors = {k: (v * 3 if v.dim() == 2 and "embed" not in k else v) for k, v in tensors.items()}
    rt = Runtime(torch.device("cuda"), DT[dtype], kw.get("page_tokens", 16),
                 status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    model.load({k: v.cuda() for k, v in tensors.items()}, rt)
    engine = Engine(model, EngineConfig(dtype=DT[dtype], page_tokens=kw.get("page_tokens", 16),
                                        max_tokens=kw.get("max_tokens", 256), max_requests=kw.get("max_requests", 3)),
                    config)
    return engine, as_np(tensors)


@dataclass(frozen=True)
class ToyConfig:
    """The configuration class of the toy architectures below: what config.json would hold for them."""
    architecture: str
    hidden_size: int
    vocab_size: int
    num_hidden_layers: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["architectures"][0], d["hidden_size"], d["vocab_size"], d["num_hidden_layers"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                "vocab_size": self.vocab_size, "num_hidden_layers": self.num_hidden_layers}


def in_portions(engine, a, b):
    """Two requests through the engine in portions, beside each other; returns their logits."""
    from air_b200.engine.batch import Entry
    na, nb = len(a), len(b)
    got_a, got_b = [], []
    got_a.append(engine.step([Entry("a", a[:17], range(17))]).cpu())
    out = engine.step([Entry("a", a[17:19], range(2)), Entry("b", b[:nb - 5], range(nb - 5))]).cpu()
    got_a.append(out[:2]); got_b.append(out[2:])
    pos = 19
    for i in range(5):
        m = min(4, na - 1 - pos)
        out = engine.step([Entry("b", [b[nb - 5 + i]], [0]), Entry("a", a[pos:pos + m], range(m))]).cpu()
        got_b.append(out[:1]); got_a.append(out[1:])
        pos += m
    got_a.append(engine.step([Entry("a", a[pos:], range(na - pos))]).cpu())
    engine.finish("a"); engine.finish("b")
    return torch.cat(got_a).numpy(), torch.cat(got_b).numpy()


# ------------------------------------------------------------------ a toy mixer with state of its own
def attention_spec(hidden, heads, kv, d, bias):
    from air_b200.parts import PartSpec
    return PartSpec("attention", {"hidden": hidden, "heads": heads, "kv_heads": kv, "head_dim": d, "qkv_bias": bias,
                                  "window": None, "position": PartSpec("rope_half", {"rotary_dim": d, "theta": 100.0,
                                                                                     "max_positions": 128})})


def plain_attention(x, w, p, heads, kv, d, theta=100.0):
    """The attention mixer on a whole sequence, from the plain functions."""
    T = x.shape[0]
    pos = np.arange(T)
    q = plain.rope(plain.linear(x, w[p + "q_proj.weight"], w.get(p + "q_proj.bias")).reshape(T, heads, d), pos, theta)
    k = plain.rope(plain.linear(x, w[p + "k_proj.weight"], w.get(p + "k_proj.bias")).reshape(T, kv, d), pos, theta)
    v = plain.linear(x, w[p + "v_proj.weight"], w.get(p + "v_proj.bias")).reshape(T, kv, d)
    return plain.linear(plain.attention(q, k, v).reshape(T, heads * d), w[p + "o_proj.weight"])


def plain_swiglu(x, w, p):
    return plain.swiglu(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])


def test_a_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer that keeps a decaying running sum of its inputs per request (state of fixed size,
    no pages), a new architecture that alternates it with attention, a configuration class for
    it: all defined here.  It is registered, given random weights, and stepped through the
    engine whole, in portions and beside another request, in slots that were used before; every
    result equals a loop over the whole sequence that is written here from the plain functions."""
    from air_b200.engine.batch import Entry
    from air_b200.parts import (Mixer, PartSpec, BlockSpec, ModelSpec, RunStep, SlotState, register_mixer,
                                register_architecture)
    from air_b200.weights.loader import TensorSpec

    @register_mixer("toy_decay")
    class ToyDecay(Mixer):
        def cache_needs(self):
            return (SlotState((self.spec["hidden"],), "float32"),)

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.spec["hidden"],), init="one_plus_normal")]

        def load(self, tensors, rt):
            super().load(tensors, rt)
            self.w = tensors[self.prefix + "mix.weight"].float()

        def forward(self, x, ctx, cache, owns_cache=True):
            (slot_state,) = cache
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for s in range(ctx.num_seqs):
                state = slot_state.state[ctx.slots_host[s]]
                for t in range(ctx.q_start_host[s], ctx.q_start_host[s + 1]):
                    state.mul_(self.spec["decay"]).add_(x[t].float())
                    out[t] = state * self.w
            return out

    hidden, decay = 32, 0.75

    def toy_spec(c):
        norm = PartSpec("rms", {"size": c.hidden_size, "eps": 1e-5})
        att = attention_spec(c.hidden_size, 2, 1, 16, False)
        toy = PartSpec("toy_decay", {"hidden": c.hidden_size, "decay": decay})
        ff = PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 48})
        layers = tuple(BlockSpec("pre_norm", f"model.layers.{i}.",
                                 {"mixer_norm": norm, "mixer": toy if i % 2 == 0 else att,
                                  "feed_forward_norm": norm, "feed_forward": ff})
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), norm, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    def oracle(w, tokens):
        h = plain.embed(w["model.embed_tokens.weight"], np.asarray(tokens))
        for i in range(3):
            p = f"model.layers.{i}."
            x = plain.rms_norm(h, w[p + "mixer_norm.weight"], 1e-5)
            if i % 2 == 0:
                state, a = np.zeros(hidden, dtype=np.float32), np.zeros_like(x)
                for t in range(len(tokens)):
                    state = (state * np.float32(decay) + x[t]).astype(np.float32)
                    a[t] = state * w[p + "mixer.mix.weight"]
            else:
                a = plain_attention(x, w, p + "mixer.", 2, 1, 16)
            h = (h + a).astype(np.float32)
            h = (h + plain_swiglu(plain.rms_norm(h, w[p + "feed_forward_norm.weight"], 1e-5), w,
                                  p + "feed_forward.")).astype(np.float32)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], 1e-5), w["lm_head.weight"])

    register_architecture("ToyDecayForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToyDecayForCausalLM"], "hidden_size": hidden, "vocab_size": 70, "num_hidden_layers": 3}
    engine, w = engine_and_weights(cfg, seed=5)
    assert [type(b.mixer).__name__ for b in engine.model.blocks] == ["ToyDecay", "Attention", "ToyDecay"]
    assert len(engine.cache.groups) == 1 and len(engine.cache._state_tensors) == 2
    assert not engine.use_graphs, "a mixer that reads the batch on the host keeps the step out of CUDA graphs"
    a = [t % 70 for t in util.tokens_for("A", 40, 1)]
    b = [t % 70 for t in util.tokens_for("A", 25, 2)]
    want_a, want_b = oracle(w, a), oracle(w, b)
    tol = 2e-5 * max(1.0, np.abs(want_a).max())
    whole_a = engine.step([Entry("wa", a, range(40))]).cpu().numpy()
    whole_b = engine.step([Entry("wb", b, range(25))]).cpu().numpy()
    engine.finish("wa"); engine.finish("wb")
    assert np.abs(whole_a - want_a).max() < tol and np.abs(whole_b - want_b).max() < tol
    got_a, got_b = in_portions(engine, a, b)         # in slots that were used before: the state starts at zero
    assert np.abs(got_a - want_a).max() < tol and np.abs(got_b - want_b).max() < tol
    assert not np.allclose(want_a[5], want_a[6])
    engine.cache.check()


# ------------------------------------------------------------------ toy parts of the other kinds
def test_a_toy_position_encoding_registers_and_rotates():
    """Another position encoding, defined here: positions divided by a factor, and only the first half
    of a head rotated.  The attention part takes it by name and its kernel reads the table."""
    from air_b200.cache.manager import CacheManager
    from air_b200.parts import PositionEncoding, PartSpec, register_position_encoding
    from air_b200.parts.attention import Attention

    @register_position_encoding("toy_scaled_partial")
    class ToyScaledPartial(PositionEncoding):
        def load(self, tensors, rt):
            super().load(tensors, rt)
            rot, n = int(self.spec["rotary_dim"]), int(self.spec["max_positions"])
            self.rotary_dim = rot
            i = torch.arange(rot // 2, dtype=torch.float64)
            angle = (torch.arange(n, dtype=torch.float64) / self.spec["factor"])[:, None] * \
                (1.0 / torch.pow(torch.tensor(float(self.spec["theta"]), dtype=torch.float64), 2.0 * i / rot))[None, :]
            self._table = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).float().to(rt.device)

        def table(self):
            return self._table

    hidden, heads, kv, d, rot, T, theta, factor = 80, 4, 2, 32, 16, 37, 500.0, 4.0
    spec = PartSpec("attention", {"hidden": hidden, "heads": heads, "kv_heads": kv, "head_dim": d, "qkv_bias": True,
                                  "window": None,
                                  "position": PartSpec("toy_scaled_partial", {"rotary_dim": rot, "theta": theta,
                                                                              "factor": factor, "max_positions": 64})})
    part = Attention(spec, "a.")
    assert type(part.position).__name__ == "ToyScaledPartial"
    t = tensors_for(part, 7, "float32")
    part.load({k: v.cuda() for k, v in t.items()}, runtime("float32"))
    cache = CacheManager([part.cache_needs()], 16, 8, 2, dtype=torch.float32, device="cuda")
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(4))
    outs, i = [], 0
    for n in (30, 1, 6):
        ctx, entries = context_for(cache, [("r", [0] * n, [])])
        y = part.forward(x[i:i + n].cuda(), ctx, cache.views(0), True)
        outs.append((y.sum(0) if y.dim() == 3 else y).cpu())
        cache.commit("r", n)
        i += n
    out = torch.cat(outs).numpy()
    w, xn = as_np(t), x.numpy()
    pos = np.arange(T) / factor

    def rotate(v):       # the first `rot` elements of every head, the rest as they are
        return np.concatenate([plain.rope(v[..., :rot], pos, theta), v[..., rot:]], axis=-1)

    q = rotate(plain.linear(xn, w["a.q_proj.weight"], w["a.q_proj.bias"]).reshape(T, heads, d))
    k = rotate(plain.linear(xn, w["a.k_proj.weight"], w["a.k_proj.bias"]).reshape(T, kv, d))
    v = plain.linear(xn, w["a.v_proj.weight"], w["a.v_proj.bias"]).reshape(T, kv, d)
    want = plain.linear(plain.attention(q, k, v).reshape(T, heads * d), w["a.o_proj.weight"])
    assert np.abs(out - want).max() < 1e-5 * np.abs(want).max()


def test_a_toy_feed_forward_with_routing_registers_builds_and_steps():
    """A feed-forward that sends every token to one of its experts (router logits in 32-bit, the
    largest wins), defined here together with an architecture that has it in every second layer.  It is
    registered, given random weights and stepped through the engine whole, in portions and beside
    another request; every result equals a loop over tokens that is written here."""
    from air_b200.engine.batch import Entry
    from air_b200.parts import (FeedForward, PartSpec, BlockSpec, ModelSpec, RunStep, register_feed_forward,
                                register_architecture)
    from air_b200.weights.loader import TensorSpec

    @register_feed_forward("toy_routed")
    class ToyRouted(FeedForward):
        def tensor_specs(self):
            e, i, n, p = self.spec["hidden"], self.spec["intermediate"], self.spec["experts"], self.prefix
            specs = [TensorSpec(p + "router.weight", (n, e), wide=True)]
            for x in range(n):
                specs += [TensorSpec(p + f"experts.{x}.gate.weight", (i, e)), TensorSpec(p + f"experts.{x}.up.weight", (i, e)),
                          TensorSpec(p + f"experts.{x}.down.weight", (e, i))]
            return specs

        def load(self, tensors, rt):
            super().load(tensors, rt)
            p = self.prefix
            self.router = tensors[p + "router.weight"].float()
            self.experts = [tuple(tensors[p + f"experts.{x}.{n}.weight"].float() for n in ("gate", "up", "down"))
                            for x in range(self.spec["experts"])]
            self.chosen = []

        def forward(self, x, ctx):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(-1)
            self.chosen.append(choice.cpu())
            out = torch.zeros_like(xf)
            for e, (g, u, d) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = xf[rows]
                    out[rows] = (torch.nn.functional.silu(h @ g.T) * (h @ u.T)) @ d.T
            return out

    def toy_spec(c):
        norm = PartSpec("rms", {"size": c.hidden_size, "eps": 1e-5})
        att = attention_spec(c.hidden_size, 3, 3, 16, True)
        dense = PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 40})
        routed = PartSpec("toy_routed", {"hidden": c.hidden_size, "intermediate": 24, "experts": 3})
        layers = tuple(BlockSpec("pre_norm", f"model.layers.{i}.",
                                 {"mixer_norm": norm, "mixer": att, "feed_forward_norm": norm,
                                  "feed_forward": routed if i % 2 else dense})
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), norm, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    def oracle(w, tokens):
        h = plain.embed(w["model.embed_tokens.weight"], np.asarray(tokens))
        for i in range(4):
            p = f"model.layers.{i}."
            a = plain_attention(plain.rms_norm(h, w[p + "mixer_norm.weight"], 1e-5), w, p + "mixer.", 3, 3, 16)
            h = (h + a).astype(np.float32)
            x = plain.rms_norm(h, w[p + "feed_forward_norm.weight"], 1e-5)
            if i % 2:
                f = np.zeros_like(x)
                q = p + "feed_forward."
                for t in range(len(tokens)):           # one token at a time, to the expert with the largest logit
                    e = int(np.argmax(w[q + "router.weight"].astype(np.float64) @ x[t].astype(np.float64)))
                    f[t] = plain.swiglu(x[t:t + 1], w[q + f"experts.{e}.gate.weight"], w[q + f"experts.{e}.up.weight"],
                                        w[q + f"experts.{e}.down.weight"])[0]
            else:
                f = plain_swiglu(x, w, p + "feed_forward.")
            h = (h + f).astype(np.float32)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], 1e-5), w["lm_head.weight"])

    register_architecture("ToyRoutedForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 90, "num_hidden_layers": 4}
    engine, w = engine_and_weights(cfg, seed=8)
    assert [type(b.feed_forward).__name__ for b in engine.model.blocks] == ["SwiGLU", "ToyRouted", "SwiGLU", "ToyRouted"]
    a = [t % 90 for t in util.tokens_for("A", 45, 3)]
    b = [t % 90 for t in util.tokens_for("A", 21, 4)]
    want_a, want_b = oracle(w, a), oracle(w, b)
    tol = 2e-5 * max(1.0, np.abs(want_a).max())
    whole_a = engine.step([Entry("wa", a, range(45))]).cpu().numpy()
    engine.finish("wa")
    assert np.abs(whole_a - want_a).max() < tol
    routed = engine.model.blocks[1].feed_forward
    assert len(torch.cat(routed.chosen).unique()) > 1, "the tokens went to more than one expert"
    got_a, got_b = in_portions(engine, a, b)
    assert np.abs(got_a - want_a).max() < tol and np.abs(got_b - want_b).max() < tol
    engine.cache.check()


# ------------------------------------------------------------------ another arrangement, another kind of cache, the model's options
def test_a_toy_block_with_a_norm_after_each_part():
    """Another arrangement of parts, defined here as a block class alone: a norm before AND after the
    mixer and the feed-forward (six roles instead of four), and a norm of another kind for the outer ones
    (with a bias, written with the base class's add_delta and torch).  The description of the model names
    the roles; nothing in the package knows them."""
    from air_b200.engine.batch import Entry
    from air_b200.parts import (Block, Norm, PartSpec, BlockSpec, ModelSpec, RunStep, register_block, register_norm,
                                register_architecture, registry)
    from air_b200.weights.loader import TensorSpec

    @register_norm("toy_biased_rms")
    class ToyBiasedRMS(Norm):
        def tensor_specs(self):
            n = self.spec["size"]
            return [TensorSpec(self.prefix + "weight", (n,), init="one_plus_normal", wide=True),
                    TensorSpec(self.prefix + "bias", (n,), wide=True)]

        def load(self, tensors, rt):
            super().load(tensors, rt)
            self.w, self.b = tensors[self.prefix + "weight"].float(), tensors[self.prefix + "bias"].float()

        def forward(self, h, delta, rows=None):
            if rows is None:
                x = self.add_delta(h, delta)           # whatever form delta has, the stream is complete now
            else:
                x = self.add_delta(h.clone(), delta)[rows.long()]
            y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.spec["eps"]) * self.w + self.b
            return y.to(self.rt.dtype)

    @register_block("toy_sandwich")
    class ToySandwich(Block):
        def __init__(self, spec):
            super().__init__(spec)
            build = lambda reg, role: reg.get(spec.part(role).kind)(spec.part(role), spec.name(role))
            self.n1, self.n2 = build(registry.NORMS, "before_mixer"), build(registry.NORMS, "after_mixer")
            self.n3, self.n4 = build(registry.NORMS, "before_ff"), build(registry.NORMS, "after_ff")
            self.mixer, self.ff = build(registry.MIXERS, "mixer"), build(registry.FEED_FORWARDS, "ff")

        def parts(self):
            return (self.n1, self.mixer, self.n2, self.n3, self.ff, self.n4)

        def cache_needs(self):
            return self.mixer.cache_needs()

        def forward(self, h, pending, ctx, cache, owns_cache=True):
            ctx.residual = None                          # the parts hand their output on; nothing adds into h itself
            a = self.mixer.forward(self.n1.forward(h, pending), ctx, cache, owns_cache)
            a = self.n2.forward(torch.zeros_like(h), a)  # the norm of the mixer's output alone
            f = self.ff.forward(self.n3.forward(h, a), ctx)
            return h, self.n4.forward(torch.zeros_like(h), f)

    hidden, eps = 64, 1e-5

    def toy_spec(c):
        rms = PartSpec("rms", {"size": c.hidden_size, "eps": eps})
        biased = PartSpec("toy_biased_rms", {"size": c.hidden_size, "eps": eps})
        layers = tuple(BlockSpec("toy_sandwich", f"model.layers.{i}.",
                                 {"before_mixer": biased, "mixer": attention_spec(c.hidden_size, 4, 2, 16, True),
                                  "after_mixer": rms, "before_ff": biased,
                                  "ff": PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 96}),
                                  "after_ff": rms})
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), rms, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    def oracle(w, tokens):
        def biased(x, p):
            x = x.astype(np.float64)
            y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w[p + "weight"] + w[p + "bias"]
            return y.astype(np.float32)

        h = plain.embed(w["model.embed_tokens.weight"], np.asarray(tokens))
        for i in range(2):
            p = f"model.layers.{i}."
            a = plain_attention(biased(h, p + "before_mixer."), w, p + "mixer.", 4, 2, 16)
            h = (h + plain.rms_norm(a, w[p + "after_mixer.weight"], eps)).astype(np.float32)
            f = plain_swiglu(biased(h, p + "before_ff."), w, p + "ff.")
            h = (h + plain.rms_norm(f, w[p + "after_ff.weight"], eps)).astype(np.float32)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

    register_architecture("ToySandwichForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToySandwichForCausalLM"], "hidden_size": hidden, "vocab_size": 75, "num_hidden_layers": 2}
    a = [t % 75 for t in util.tokens_for("A", 40, 5)]
    b = [t % 75 for t in util.tokens_for("A", 23, 6)]
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        engine, w = engine_and_weights(cfg, seed=11, dtype=dtype)
        assert type(engine.model.blocks[0]).__name__ == "ToySandwich"
        want_a, want_b = oracle(w, a), oracle(w, b)
        scale = max(1.0, np.abs(want_a).max())
        whole = engine.step([Entry("w", a, range(40))]).cpu().numpy()
        engine.finish("w")
        assert np.abs(whole - want_a).max() < tol * scale
        got_a, got_b = in_portions(engine, a, b)
        assert np.abs(got_a - want_a).max() < tol * scale and np.abs(got_b - want_b).max() < tol * scale
        engine.cache.check()


def test_a_toy_block_with_mixer_and_feed_forward_side_by_side():
    """A third arrangement, again a block class of the test alone: ONE norm, and the mixer and the feed-forward
    both read its rows; their outputs are added to the stream together (three roles).  Whatever form the two
    outputs have (rows, or partial sums of a split product), the base class's add_delta completes the stream with
    the first and the block hands the second on."""
    from air_b200.engine.batch import Entry
    from air_b200.parts import (Block, Norm, PartSpec, BlockSpec, ModelSpec, RunStep, register_block,
                                register_architecture, registry)

    @register_block("toy_side_by_side")
    class ToySideBySide(Block):
        def __init__(self, spec):
            super().__init__(spec)
            build = lambda reg, role: reg.get(spec.part(role).kind)(spec.part(role), spec.name(role))
            self.norm = build(registry.NORMS, "norm")
            self.mixer, self.ff = build(registry.MIXERS, "mixer"), build(registry.FEED_FORWARDS, "ff")

        def parts(self):
            return (self.norm, self.mixer, self.ff)

        def cache_needs(self):
            return self.mixer.cache_needs()

        def forward(self, h, pending, ctx, cache, owns_cache=True):
            ctx.residual = None
            x = self.norm.forward(h, pending)
            a = self.mixer.forward(x, ctx, cache, owns_cache)
            f = self.ff.forward(x, ctx)
            Norm.add_delta(h, a)
            return h, f

    eps = 1e-6

    def toy_spec(c):
        rms = PartSpec("rms", {"size": c.hidden_size, "eps": eps})
        layers = tuple(BlockSpec("toy_side_by_side", f"model.layers.{i}.",
                                 {"norm": rms, "mixer": attention_spec(c.hidden_size, 6, 3, 16, False),
                                  "ff": PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 80})})
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), rms, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    def oracle(w, tokens):
        h = plain.embed(w["model.embed_tokens.weight"], np.asarray(tokens))
        for i in range(3):
            p = f"model.layers.{i}."
            x = plain.rms_norm(h, w[p + "norm.weight"], eps)
            h = (h + plain_attention(x, w, p + "mixer.", 6, 3, 16) + plain_swiglu(x, w, p + "ff.")).astype(np.float32)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

    register_architecture("ToySideBySideForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToySideBySideForCausalLM"], "hidden_size": 96, "vocab_size": 83, "num_hidden_layers": 3}
    a = [t % 83 for t in util.tokens_for("A", 40, 7)]
    b = [t % 83 for t in util.tokens_for("A", 23, 8)]
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        engine, w = engine_and_weights(cfg, seed=13, dtype=dtype)
        assert type(engine.model.blocks[0]).__name__ == "ToySideBySide"
        want_a, want_b = oracle(w, a), oracle(w, b)
        scale = max(1.0, np.abs(want_a).max())
        whole = engine.step([Entry("w", a, range(40))]).cpu().numpy()
        engine.finish("w")
        assert np.abs(whole - want_a).max() < tol * scale
        got_a, got_b = in_portions(engine, a, b)
        assert np.abs(got_a - want_a).max() < tol * scale and np.abs(got_b - want_b).max() < tol * scale
        engine.cache.check()


def test_a_toy_mixer_that_pages_one_latent_per_token():
    """Another kind of cache, defined here: instead of keys and values a mixer keeps ONE short vector per
    token, in pages of a shape of its own.  The need states the shape; the cache manager, which knows no
    kinds of need, makes the slab, the pool and the block table, gives pages back and hands them out again.
    The mixer writes and reads its pages through the step's block table."""
    from types import SimpleNamespace
    from air_b200.engine.batch import Entry
    from air_b200.parts import (CacheNeed, Mixer, PartSpec, BlockSpec, ModelSpec, RunStep, register_mixer,
                                register_architecture)
    from air_b200.weights.loader import TensorSpec

    @dataclass(frozen=True)
    class PagedLatent(CacheNeed):
        width: int
        window = None
        paged = True

        def page_shape(self, page_tokens):
            return (page_tokens, self.width)

        def element_dtype(self, compute_dtype):
            return torch.float32

        def view(self, tensor, group):
            return SimpleNamespace(latent=tensor, group=group)

    @register_mixer("toy_latent")
    class ToyLatent(Mixer):
        """c_t = W_down x_t is kept; the output at t is W_up applied to the softmax(c_t . c_j)-weighted mean of
        the c_j up to t."""

        def cache_needs(self):
            return (PagedLatent(self.spec["width"]),)

        def tensor_specs(self):
            e, r, p = self.spec["hidden"], self.spec["width"], self.prefix
            return [TensorSpec(p + "down.weight", (r, e)), TensorSpec(p + "up.weight", (e, r))]

        def load(self, tensors, rt):
            super().load(tensors, rt)
            self.down, self.up = tensors[self.prefix + "down.weight"].float(), tensors[self.prefix + "up.weight"].float()

        def forward(self, x, ctx, cache, owns_cache=True):
            (pages,) = cache
            P = pages.latent.shape[1]
            table = ctx.block_tables[pages.group]
            c = x.float() @ self.down.T
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for s in range(ctx.num_seqs):
                slot, q0, q1 = ctx.slots_host[s], ctx.q_start_host[s], ctx.q_start_host[s + 1]
                first = ctx.kv_len_host[s] - (q1 - q0)
                for t in range(q0, q1):
                    p = first + t - q0
                    page = int(table[slot, p // P])
                    assert page >= 0
                    pages.latent[page, p % P] = c[t]
                    blocks = table[slot, : p // P + 1].long()
                    seen = pages.latent[blocks].reshape(-1, c.shape[1])[: p + 1]
                    out[t] = self.up @ (torch.softmax(seen @ c[t], 0) @ seen)
            return out

    hidden, width = 32, 8

    def toy_spec(c):
        norm = PartSpec("rms", {"size": c.hidden_size, "eps": 1e-5})
        layers = tuple(BlockSpec("pre_norm", f"model.layers.{i}.",
                                 {"mixer_norm": norm, "mixer": PartSpec("toy_latent", {"hidden": c.hidden_size, "width": width}),
                                  "feed_forward_norm": norm,
                                  "feed_forward": PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 48})})
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), norm, "model.embed_tokens.weight",
                         "model.norm.", None)

    def oracle(w, tokens):
        h = plain.embed(w["model.embed_tokens.weight"], np.asarray(tokens))
        for i in range(2):
            p = f"model.layers.{i}."
            x = plain.rms_norm(h, w[p + "mixer_norm.weight"], 1e-5).astype(np.float64)
            c = x @ w[p + "mixer.down.weight"].astype(np.float64).T
            a = np.zeros_like(x)
            for t in range(len(tokens)):
                score = c[: t + 1] @ c[t]
                prob = np.exp(score - score.max())
                a[t] = w[p + "mixer.up.weight"].astype(np.float64) @ ((prob / prob.sum()) @ c[: t + 1])
            h = (h + a).astype(np.float32)
            h = (h + plain_swiglu(plain.rms_norm(h, w[p + "feed_forward_norm.weight"], 1e-5), w,
                                  p + "feed_forward.")).astype(np.float32)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"])

    register_architecture("ToyLatentForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToyLatentForCausalLM"], "hidden_size": hidden, "vocab_size": 60, "num_hidden_layers": 2}
    engine, w = engine_and_weights(cfg, seed=13, max_tokens=80)      # five pages of 16: used again below
    view = engine.cache.views(0)[0]
    assert tuple(view.latent.shape) == (5, 16, width) and view.latent.dtype == torch.float32
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].runs == [0, 1]
    a = [t % 60 for t in util.tokens_for("A", 40, 7)]
    b = [t % 60 for t in util.tokens_for("A", 25, 8)]
    want_a, want_b = oracle(w, a), oracle(w, b)
    tol = 3e-5 * max(1.0, np.abs(want_a).max())
    whole = engine.step([Entry("w", a, range(40))]).cpu().numpy()
    engine.finish("w")
    assert np.abs(whole - want_a).max() < tol
    got_a, got_b = in_portions(engine, a, b)
    assert np.abs(got_a - want_a).max() < tol and np.abs(got_b - want_b).max() < tol
    assert engine.cache.groups[0].pool.takes > engine.cache.num_pages, "pages were used again"
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_model_options_that_qwen2_leaves_off(dtype):
    """An embedding multiplier, an output bias, a logit scale and a soft cap are options of the model's
    description (off for Qwen2).  A toy architecture switches them on; the oracle is the plain forward with the
    same four steps written here."""
    from air_b200.config import Qwen2Config
    from air_b200.config.architectures import qwen2_spec
    from air_b200.engine.batch import Entry
    from air_b200.parts import register_architecture
    import dataclasses

    mult, scale, cap = 3.5, 0.25, 1.5

    def toy_spec(c):
        return dataclasses.replace(qwen2_spec(c), embedding_multiplier=mult, output_bias_name="lm_head.bias",
                                   logit_scale=scale, logit_softcap=cap)

    register_architecture("ToyOptionsForCausalLM", Qwen2Config, toy_spec)
    cfg = dict(util.TINY_B, architectures=["ToyOptionsForCausalLM"])
    engine, w = engine_and_weights(cfg, seed=17, dtype=dtype)
    w["lm_head.bias"] = np.linspace(-2, 2, cfg["vocab_size"]).astype(np.float32)
    engine.model.output_bias.copy_(torch.from_numpy(w["lm_head.bias"]))
    tokens = util.tokens_for("B", 37, 9)
    scaled = dict(w)
    scaled["model.embed_tokens.weight"] = (w["model.embed_tokens.weight"] * np.float32(mult)).astype(np.float32)
    base = plain.forward(dict(cfg, tie_word_embeddings=False), scaled, tokens)
    want = cap * np.tanh((base + w["lm_head.bias"]) * scale / cap)
    got = np.concatenate([engine.step([Entry("r", tokens[:20], range(20))]).cpu().numpy()] +
                         [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in tokens[20:]])
    assert np.abs(want).max() > 0.5 * cap, "the cap bites"
    assert np.abs(got - want).max() < (3e-5 if dtype == "float32" else 4e-2) * max(1.0, np.abs(want).max())
