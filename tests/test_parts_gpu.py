"""Each part alone against its plain function, with sizes of its own; the order list (a layer
named twice, a run that reads another run's cache); and a toy mixer with state of its own that
is defined here, registered, built and stepped without a change to the framework's files."""
import math

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


def context_for(cache, entries):
    from air_b200.engine.batch import Entry, build_context
    entries = [Entry(*e) for e in entries]
    for e in entries:
        if e.request not in cache.sequences:
            cache.open(e.request)
    cache.reserve([(e.request, len(e.tokens)) for e in entries])
    ctx = build_context(entries, cache, "cuda", status=torch.zeros(1, dtype=torch.int32, device="cuda"))
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
        ctx, entries = context_for(cache, [("r", [0] * n, [])])
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


# ------------------------------------------------------------------ a toy mixer with state of its own
def test_a_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer that keeps a decaying running sum of its inputs per request (state of fixed size,
    no pages), a new architecture that alternates it with attention, a configuration class for
    it: all defined here.  It is registered, given random weights, and stepped through the
    engine in portions and beside another request; the result equals a whole-sequence loop."""
    from dataclasses import dataclass
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
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

    @dataclass(frozen=True)
    class ToyConfig:
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

    def toy_spec(c):
        norm = PartSpec("rms", {"size": c.hidden_size, "eps": 1e-5})
        att = PartSpec("attention", {"hidden": c.hidden_size, "heads": 2, "kv_heads": 1, "head_dim": 16,
                                     "qkv_bias": False, "window": None,
                                     "position": PartSpec("rope_half", {"rotary_dim": 16, "theta": 100.0,
                                                                        "max_positions": 128})})
        toy = PartSpec("toy_decay", {"hidden": c.hidden_size, "decay": 0.75})
        ff = PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 48})
        layers = tuple(BlockSpec("pre_norm", f"model.layers.{i}.", toy if i % 2 == 0 else att, ff, norm, norm)
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), norm, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    register_architecture("ToyDecayForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToyDecayForCausalLM"], "hidden_size": 32, "vocab_size": 70, "num_hidden_layers": 3}
    engine = Engine.from_random(cfg, seed=5, config=EngineConfig(dtype=torch.float32, page_tokens=16,
                                                                 max_tokens=256, max_requests=3))
    assert [type(b.mixer).__name__ for b in engine.model.blocks] == ["ToyDecay", "Attention", "ToyDecay"]
    assert len(engine.cache.groups) == 1 and len(engine.cache._state_tensors) == 2
    a, b = util.tokens_for("A", 40, 1)[:40], util.tokens_for("A", 25, 2)
    a, b = [t % 70 for t in a], [t % 70 for t in b]
    whole_a = engine.step([Entry("wa", a, range(40))]).cpu()
    whole_b = engine.step([Entry("wb", b, range(25))]).cpu()
    engine.finish("wa"); engine.finish("wb")
    # now in portions, the two requests beside each other, in slots that were used before
    got_a, got_b = [], []
    got_a.append(engine.step([Entry("a", a[:17], range(17))]).cpu())
    out = engine.step([Entry("a", a[17:19], range(2)), Entry("b", b[:20], range(20))]).cpu()
    got_a.append(out[:2]); got_b.append(out[2:])
    for i in range(5):
        out = engine.step([Entry("b", [b[20 + i]], [0]), Entry("a", a[19 + 4 * i:23 + 4 * i], range(4))]).cpu()
        got_b.append(out[:1]); got_a.append(out[1:])
    got_a.append(engine.step([Entry("a", a[39:], [0])]).cpu())
    assert torch.allclose(torch.cat(got_a), whole_a, atol=1e-5, rtol=1e-5)
    assert torch.allclose(torch.cat(got_b), whole_b, atol=1e-5, rtol=1e-5)
    assert not torch.allclose(whole_a[5], whole_a[6])
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
    another request; the part alone equals a loop over tokens."""
    from dataclasses import dataclass
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.parts import (FeedForward, PartSpec, BlockSpec, ModelSpec, RunStep, register_feed_forward,
                                register_architecture)
    from air_b200.weights.loader import TensorSpec

    @register_feed_forward("toy_routed")
    class ToyRouted(FeedForward):
        def tensor_specs(self):
            e, i, n, p = self.spec["hidden"], self.spec["intermediate"], self.spec["experts"], self.prefix
            specs = [TensorSpec(p + "router.weight", (n, e))]
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

    @dataclass(frozen=True)
    class ToyConfig:
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

    def toy_spec(c):
        norm = PartSpec("rms", {"size": c.hidden_size, "eps": 1e-5})
        att = PartSpec("attention", {"hidden": c.hidden_size, "heads": 3, "kv_heads": 3, "head_dim": 16,
                                     "qkv_bias": True, "window": None,
                                     "position": PartSpec("rope_half", {"rotary_dim": 16, "theta": 100.0,
                                                                        "max_positions": 128})})
        dense = PartSpec("swiglu", {"hidden": c.hidden_size, "intermediate": 40})
        routed = PartSpec("toy_routed", {"hidden": c.hidden_size, "intermediate": 24, "experts": 3})
        layers = tuple(BlockSpec("pre_norm", f"model.layers.{i}.", att, routed if i % 2 else dense, norm, norm)
                       for i in range(c.num_hidden_layers))
        return ModelSpec(c.architecture, c.hidden_size, c.vocab_size, 128, layers,
                         tuple(RunStep(i) for i in range(c.num_hidden_layers)), norm, "model.embed_tokens.weight",
                         "model.norm.", "lm_head.weight")

    register_architecture("ToyRoutedForCausalLM", ToyConfig, toy_spec)
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 90, "num_hidden_layers": 4}
    engine = Engine.from_random(cfg, seed=8, config=EngineConfig(dtype=torch.float32, page_tokens=16,
                                                                 max_tokens=256, max_requests=3))
    assert [type(b.feed_forward).__name__ for b in engine.model.blocks] == ["SwiGLU", "ToyRouted", "SwiGLU", "ToyRouted"]
    a = [t % 90 for t in util.tokens_for("A", 45, 3)]
    b = [t % 90 for t in util.tokens_for("A", 21, 4)]
    whole_a = engine.step([Entry("wa", a, range(45))]).cpu()
    whole_b = engine.step([Entry("wb", b, range(21))]).cpu()
    engine.finish("wa"); engine.finish("wb")
    routed = engine.model.blocks[1].feed_forward
    assert len(torch.cat(routed.chosen).unique()) > 1, "the tokens went to more than one expert"
    got_a = [engine.step([Entry("a", a[:20], range(20))]).cpu()]
    out = engine.step([Entry("b", b[:19], range(19)), Entry("a", a[20:22], range(2))]).cpu()
    got_b = [out[:19]]; got_a.append(out[19:])
    out = engine.step([Entry("b", b[19:20], [0]), Entry("a", a[22:], range(23))]).cpu()
    got_b.append(out[:1]); got_a.append(out[1:])
    got_b.append(engine.step([Entry("b", b[20:], [0])]).cpu())
    assert torch.allclose(torch.cat(got_a), whole_a, atol=1e-5, rtol=1e-5)
    assert torch.allclose(torch.cat(got_b), whole_b, atol=1e-5, rtol=1e-5)
    # the part alone: one token at a time gives what the batch gave
    x = torch.randn(9, 48, generator=torch.Generator().manual_seed(1)).cuda()
    together = routed.forward(x, None)
    alone = torch.cat([routed.forward(x[i:i + 1], None) for i in range(9)])
    assert torch.allclose(together, alone, atol=1e-6)
    engine.cache.check()
