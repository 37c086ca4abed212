"""Each part alone against its plain statement, and the generality of the layout: a
toy architecture defined here (a mixer with state of its own, a windowed attention
with adjacent-pair rotation, a layer that runs twice, a layer that reads another
layer's cache) is registered, written as a random model folder, built and stepped
without a change to the framework's files; so is a second one with a feed-forward that
routes tokens to experts and a position encoding of its own, and a third with a norm and a
block arrangement of its own."""

import math
from dataclasses import dataclass
from typing import ClassVar, Tuple

import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def close(got, want, tol, what=""):
    want = want.to(torch.float64).cpu()
    scale = max(float(want.abs().max()), 1e-6)
    err = float((got.to(torch.float64).cpu() - want).abs().max())
    assert err <= tol * scale, f"{what}: error {err:.3e} = {err / scale:.2e} of scale (limit {tol:.0e})"


def rand(*shape, seed=0, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


def make_ctx(rt, cache, segs, tokens=None):
    """A StepContext for segments [(slot, n_tokens)], continuing what each slot holds."""
    from axon_b200.parts import StepContext
    pos, slot_of, seg = [], [], [[], [], [], []]
    at = 0
    for slot, n in segs:
        start = cache.length(slot)
        assert cache.reserve(slot, start + n)
        pos += list(range(start, start + n))
        slot_of += [slot] * n
        for lst, v in zip(seg, (slot, at, n, start + n)):
            lst.append(v)
        at += n
    cache.sync_tables()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ctx = StepContext(rt=rt, n_tokens=at, tokens=i32(tokens if tokens is not None else [0] * at), positions=i32(pos),
                      token_slot=i32(slot_of), seg_slot=seg[0], seg_q_start=seg[1], seg_q_len=seg[2],
                      seg_kv_len=seg[3], segments=i32(seg), host_positions=pos)
    return ctx


def commit(cache, ctx):
    for slot, kv in zip(ctx.seg_slot, ctx.seg_kv_len):
        cache.commit(slot, kv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_head_parts(dtype):
    from axon_b200.parts import PartSpec, Runtime, part_class
    rt = Runtime(dtype, DEV)
    gain = rand(70, seed=1) * 0.1 + 1
    norm = part_class("norm", "rmsnorm")(PartSpec("rmsnorm", {"size": 70, "eps": 1e-3}, {"gain": "g"}), {"gain": gain}, rt, None)
    x = rand(5, 70, seed=2, std=4.0)
    out = torch.empty(5, 70, dtype=dtype, device=DEV)
    norm.forward(x, out)
    close(out, plain.rms_norm(x.double().cpu(), gain.double().cpu(), 1e-3), TOL[dtype], "rmsnorm part")

    table = rand(33, 70, seed=3, dtype=dtype)
    emb = part_class("embedding", "embedding")(PartSpec("embedding", {"vocab_size": 33, "hidden_size": 70}, {"table": "t"}),
                                               {"table": table}, rt, None)
    tok = torch.tensor([32, 0, 7], dtype=torch.int32, device=DEV)
    x3 = torch.empty(3, 70, dtype=torch.float32, device=DEV)
    emb.forward(tok, x3)
    assert torch.equal(x3.cpu(), plain.embed(table.double().cpu(), [32, 0, 7]).float())

    head = part_class("head", "linear_head")(PartSpec("linear_head", {"vocab_size": 33, "hidden_size": 70}, {"weight": "t"}),
                                             {"weight": table}, rt, None)
    h = rand(3, 70, seed=4, dtype=dtype)
    logits = torch.empty(3, 33, dtype=torch.float32, device=DEV)
    head.forward(h, logits)
    close(logits, plain.linear(h.double().cpu(), table.double().cpu()), 2e-5 if dtype == torch.float32 else 1e-2, "head part")


def test_rope_part_tables_are_shared_per_step():
    from axon_b200.cache import PagedCache
    from axon_b200.parts import KvNeed, PartSpec, Runtime, part_class
    rt = Runtime(torch.float32, DEV)
    cache = PagedCache([KvNeed(1, 16)], torch.float32, DEV, page_size=4, max_tokens=64, max_slots=2, max_positions=64)
    s = cache.open()
    ctx = make_ctx(rt, cache, [(s, 6)])
    spec = PartSpec("rope", {"head_dim": 16, "theta": 1e4, "pairing": "half"})
    a = part_class("position", "rope")(spec, {}, rt, None)
    b = part_class("position", "rope")(spec, {}, rt, None)
    other = part_class("position", "rope")(PartSpec("rope", {"head_dim": 16, "theta": 1e6, "pairing": "adjacent", "rot": 8}), {}, rt, None)
    ta, tb, tc = a.rotation(ctx), b.rotation(ctx), other.rotation(ctx)
    assert ta.data_ptr() == tb.data_ptr() and tc.data_ptr() != ta.data_ptr()
    assert ta.shape == (6, 8, 2) and tc.shape == (6, 4, 2) and other.adjacent and other.rot == 8
    ang = torch.arange(6, dtype=torch.float64)[:, None] * torch.tensor([1e4 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64)
    assert float((ta[..., 0].double().cpu() - torch.cos(ang)).abs().max()) < 6e-8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,hd,window", [(4, 2, 16, None), (5, 5, 32, None), (6, 2, 64, 7)])
def test_attention_part_alone(dtype, heads, kv_heads, hd, window):
    """The mixer by itself: whole sequence in one step, then the same sequence in
    portions, against q/k/v + RoPE + attention + o written with the plain functions."""
    from axon_b200.cache import PagedCache
    from axon_b200.parts import PartSpec, Runtime, part_class
    D, T = 72, 29
    rt = Runtime(dtype, DEV)
    spec = PartSpec("attention", {"hidden_size": D, "heads": heads, "kv_heads": kv_heads, "head_dim": hd,
                                  "qkv_bias": True, "out_bias": False, "window": window, "scale": None},
                    {k: k for k in ("q", "k", "v", "o", "q_bias", "k_bias", "v_bias")},
                    {"position": PartSpec("rope", {"head_dim": hd, "theta": 1e4, "pairing": "half"})})
    cls = part_class("mixer", "attention")
    w = {}
    for i, (name, decl) in enumerate(cls.tensors(spec).items()):
        vec = decl.kind == "bias"
        w[name] = rand(*decl.shape, seed=100 + i, std=0.3, dtype=torch.float32 if vec else dtype)
    ref = {k: v.double().cpu() for k, v in w.items()}
    from axon_b200.engine.model import DecoderModel  # noqa: F401  (registers nothing; parts are built directly)
    mixer = cls(spec, dict(w), rt, lambda sub: part_class("position", sub.kind)(sub, {}, rt, None))
    cache = PagedCache([cls.cache_need(spec)], dtype, DEV, page_size=4, max_tokens=64, max_slots=2, max_positions=64,
                       shuffle_seed=3)
    h = rand(T, D, seed=7, dtype=dtype)
    hd64 = h.double().cpu()
    q = plain.linear(hd64, ref["q"], ref["q_bias"]).view(T, heads, hd)
    k = plain.linear(hd64, ref["k"], ref["k_bias"]).view(T, kv_heads, hd)
    v = plain.linear(hd64, ref["v"], ref["v_bias"]).view(T, kv_heads, hd)
    q, k = plain.rope_half(q, range(T), 1e4), plain.rope_half(k, range(T), 1e4)
    want = plain.linear(plain.causal_gqa_attention(q, k, v, window=window).reshape(T, heads * hd), ref["o"])
    for cuts in ([T], [5, 1, 1, 16, 2, 4]):
        s = cache.open()
        x = torch.zeros(T, D, dtype=torch.float32, device=DEV)
        at = 0
        for n in cuts:
            cache.flush()
            ctx = make_ctx(rt, cache, [(s, n)])
            xs = x[at:at + n]
            mixer.forward(h[at:at + n].contiguous(), xs, ctx, cache.view(0), True)
            commit(cache, ctx)
            at += n
        close(x, want, TOL[dtype], f"attention part, cuts {cuts}")
        cache.close(s)
    if window:
        assert cache.manager.held_pages(0) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_and_block(dtype):
    from axon_b200.cache import PagedCache
    from axon_b200.parts import PartSpec, Runtime, part_class
    D, F, T = 48, 100, 9
    rt = Runtime(dtype, DEV)
    fspec = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": F}, {k: k for k in ("gate", "up", "down")})
    fw = {k: rand(*s, seed=10 + i, std=0.2, dtype=dtype) for i, (k, s) in enumerate(
        {"gate": (F, D), "up": (F, D), "down": (D, F)}.items())}
    ffn = part_class("ffn", "swiglu")(fspec, dict(fw), rt, None)
    h = rand(T, D, seed=20, dtype=dtype)
    x0 = rand(T, D, seed=21)
    x = x0.clone()
    ffn.forward(h, x, None)
    want = x0.double().cpu() + plain.swiglu_ffn(h.double().cpu(), *(fw[k].double().cpu() for k in ("gate", "up", "down")))
    close(x, want, TOL[dtype], "swiglu part adds into the residual")


# ---------------------------------------------------------------------------
# A toy architecture, defined and registered here.

def register_toy():
    from axon_b200.config.base import ModelConfig, register_architecture
    from axon_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry, StateNeed, TensorDecl,
                                 register_part)

    @register_part
    class RunningMean(Mixer):
        """out_t = W mean(h_0..h_t): state of fixed size (the running sum and the count)."""
        category, kind = "mixer", "toy_running_mean"

        @classmethod
        def tensors(cls, spec):
            d = spec.params["hidden_size"]
            return {"w": TensorDecl((d, d))}

        @classmethod
        def cache_need(cls, spec):
            return StateNeed((spec.params["hidden_size"] + 1,), "float32")

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            self.w, self.d = tensors["w"], spec.params["hidden_size"]

        def compute(self, h, ctx, state):
            out = torch.empty(h.shape[0], self.d, dtype=torch.float32, device=h.device)
            for slot, at, n in zip(ctx.seg_slot, ctx.seg_q_start, ctx.seg_q_len):
                hs = h[at:at + n].float()
                total = state[slot, :self.d] + torch.cumsum(hs, 0)
                count = state[slot, self.d] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                state[slot, :self.d] = total[-1]
                state[slot, self.d] = count[-1]
                out[at:at + n] = (total / count[:, None]) @ self.w.float().T
            return out

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyForCausalLM"
        model_types: ClassVar[Tuple[str, ...]] = ("toy_test",)
        hidden_size: int = 40
        vocab_size: int = 99
        heads: int = 4
        kv_heads: int = 2
        head_dim: int = 16
        ffn: int = 56
        window: int = 6
        eps: float = 1e-5
        max_positions: int = 96

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg})

    def toy_spec(c):
        norm = lambda name: PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.eps}, {"gain": name})

        def attn(p, window, pairing, theta):
            return PartSpec("attention", {"hidden_size": c.hidden_size, "heads": c.heads, "kv_heads": c.kv_heads,
                                          "head_dim": c.head_dim, "qkv_bias": False, "out_bias": False,
                                          "window": window, "scale": None},
                            {k: f"{p}.{k}" for k in ("q", "k", "v", "o")},
                            {"position": PartSpec("rope", {"head_dim": c.head_dim, "theta": theta, "pairing": pairing})})

        def ffn(p):
            return PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.ffn},
                            {k: f"{p}.{k}" for k in ("gate", "up", "down")})

        def layer(i, mixer):
            return LayerSpec("prenorm", {"norm_mixer": norm(f"l{i}.n1"), "mixer": mixer,
                                         "norm_ffn": norm(f"l{i}.n2"), "ffn": ffn(f"l{i}.ffn")})
        layers = (
            layer(0, attn("l0.attn", c.window, "adjacent", 1e4)),            # windowed, adjacent pairs
            layer(1, PartSpec("toy_running_mean", {"hidden_size": c.hidden_size}, {"w": "l1.mean.w"})),
            layer(2, attn("l2.attn", None, "half", 1e5)),                    # full attention
            layer(3, attn("l3.attn", None, "half", 1e5)),                    # reads layer 2's cache
        )
        # layer 0 runs twice (each run with a cache of its own); the last entry reads entry 3's cache
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2), ScheduleEntry(3, cache_of=3))
        return ModelSpec("ToyForCausalLM", c.hidden_size, c.vocab_size, c.max_positions,
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"table": "embed"}),
                         layers, schedule, norm("final"),
                         PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"weight": "head"}))

    register_architecture(ToyConfig, toy_spec)
    return ToyConfig


def rope_adjacent(v, positions, theta):
    """Pairs (2i, 2i+1) rotate by pos * theta^(-2i/hd)."""
    hd = v.shape[-1]
    freq = torch.tensor([theta ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64)
    ang = torch.tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0::2], v[..., 1::2]
    out = torch.empty_like(v)
    out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
    return out


def toy_plain_forward(c, w, tokens):
    """The toy architecture written with the plain functions, whole sequence, no cache."""
    T = len(tokens)
    pos = list(range(T))
    x = plain.embed(w["embed"], tokens)

    def attn_layer(x, i, window, rope, theta, kv_from=None):
        h = plain.rms_norm(x, w[f"l{i}.n1"], c.eps)
        q = plain.linear(h, w[f"l{i}.attn.q"]).view(T, c.heads, c.head_dim)
        k = plain.linear(h, w[f"l{i}.attn.k"]).view(T, c.kv_heads, c.head_dim)
        v = plain.linear(h, w[f"l{i}.attn.v"]).view(T, c.kv_heads, c.head_dim)
        q, k = rope(q, pos, theta), rope(k, pos, theta)
        kv = (k, v)
        if kv_from is not None:
            k, v = kv_from
        o = plain.causal_gqa_attention(q, k, v, window=window).reshape(T, c.heads * c.head_dim)
        x = x + plain.linear(o, w[f"l{i}.attn.o"])
        return ffn_half(x, i), kv

    def ffn_half(x, i):
        h = plain.rms_norm(x, w[f"l{i}.n2"], c.eps)
        return x + plain.swiglu_ffn(h, w[f"l{i}.ffn.gate"], w[f"l{i}.ffn.up"], w[f"l{i}.ffn.down"])

    x, _ = attn_layer(x, 0, c.window, rope_adjacent, 1e4)
    h = plain.rms_norm(x, w["l1.n1"], c.eps)
    mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    x = ffn_half(x + plain.linear(mean, w["l1.mean.w"]), 1)
    x, _ = attn_layer(x, 0, c.window, rope_adjacent, 1e4)
    x, kv2 = attn_layer(x, 2, None, plain.rope_half, 1e5)
    x, _ = attn_layer(x, 3, None, plain.rope_half, 1e5, kv_from=kv2)
    return plain.linear(plain.rms_norm(x, w["final"], c.eps), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registers_builds_and_steps(tmp_path, dtype):
    from safetensors.torch import load_file

    from axon_b200.engine.build import build_engine
    from axon_b200.engine.replay import Replayer
    from axon_b200.weights import write_random_model, write_safetensors
    ToyConfig = register_toy()
    cfg = ToyConfig()
    folder = str(tmp_path / "toy")
    write_random_model(folder, cfg, seed=5, std=0.12)
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    engine = build_engine(folder, dtype=dtype, page_size=4, max_tokens=192, max_slots=3, max_positions=96, shuffle_seed=2)
    # two groups of pages: the windowed entries (0 and 2) and the full ones (3); a state slab for entry 1
    assert len(engine.cache.groups) == 2 and sorted(len(g.members) for g in engine.cache.groups) == [1, 2]
    assert list(engine.cache.states) == [(1, "mixer")]
    g = torch.Generator().manual_seed(3)
    seqs = {r: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for r, n in (("a", 41), ("b", 23))}
    want = {r: toy_plain_forward(cfg, w, t) for r, t in seqs.items()}
    tol = 2e-5 if dtype == "float32" else 3e-2
    rp = Replayer(engine)
    fed = {"a": 0, "b": 0}

    def entry(r, n):
        t = seqs[r][fed[r]:fed[r] + n]
        e = {"id": r, "tokens": t, "want": list(range(len(t)))}
        fed[r] += len(t)
        return e
    plan = [[("a", 9)], [("a", 1), ("b", 5)], [("a", 2), ("b", 1)], [("b", 17)], [("a", 29)]]
    for k, row in enumerate(plan):
        ents, rows = [], []
        for r, n in row:
            start = fed[r]
            e = entry(r, n)
            ents.append(e)
            rows += [want[r][start + j] for j in range(len(e["tokens"]))]
        got = rp.run_step({"step": k, "entries": ents, "end": [r for r, _ in row if fed[r] == len(seqs[r])]})
        close(got, torch.stack(rows), tol, f"toy architecture, step {k}")
    # the windowed group gave pages back while "a" was still running; everything is free at the end
    engine.cache.flush()
    engine.cache.manager.check()
    for gi in range(len(engine.cache.groups)):
        assert engine.cache.manager.free_pages(gi) == engine.cache.n_pages
    # a second request in the same slot starts from zeroed state
    got = rp.run_step({"step": 9, "entries": [{"id": "c", "tokens": seqs["b"][:7], "want": [6]}], "end": ["c"]})
    close(got, want["b"][6:7], tol, "state is zeroed for a new request")


# ---------------------------------------------------------------------------
# A second toy architecture: a feed-forward that routes each token to one of several experts,
# and a position encoding of its own, both defined here.  Neither declares itself safe for CUDA
# graphs, so its steps run eagerly.

def register_routed_toy():
    from axon_b200.config.base import ModelConfig, register_architecture
    from axon_b200.kernels import linear as kernels_linear
    from axon_b200.parts import FeedForward, LayerSpec, ModelSpec, Part, PartSpec, ScheduleEntry, TensorDecl, register_part

    @register_part
    class StretchedRotary(Part):
        """Pair i of the first ``rot`` elements of a head, (i, i + rot/2), turns by
        ``(pos / stretch) * base^(-i / (rot/2))``; the rest of the head passes unchanged."""
        category, kind = "position", "toy_stretched_rotary"

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            p = spec.params
            self.rot, self.adjacent = int(p["rot"]), False
            self.stretch, self.base = float(p["stretch"]), float(p["base"])

        def rotation(self, ctx):
            key = ("toy_stretched_rotary", self.rot, self.stretch, self.base)
            table = ctx.scratch.get(key)
            if table is None:
                ang = stretched_angles(ctx.host_positions, self.rot, self.stretch, self.base)
                table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().to(self.rt.device)
                ctx.scratch[key] = table
            return table

    @register_part
    class Top1Experts(FeedForward):
        """Router logits ``R h`` in float32; the token goes to the expert with the largest one
        (the first among equals), whose output is ``W_out relu(W_in h)``."""
        category, kind = "ffn", "toy_top1_experts"

        @classmethod
        def tensors(cls, spec):
            p = spec.params
            e, d, f = p["experts"], p["hidden_size"], p["expert_size"]
            return {"router": TensorDecl((e, d)), "w_in": TensorDecl((e * f, d)), "w_out": TensorDecl((e * d, f))}

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            p = spec.params
            self.e, self.d, self.f = int(p["experts"]), int(p["hidden_size"]), int(p["expert_size"])
            self.router = tensors["router"]
            self.w_in = tensors["w_in"].view(self.e, self.f, self.d)
            self.w_out = tensors["w_out"].view(self.e, self.d, self.f)
            self.seen = set()

        def compute(self, h, ctx):
            rt = self.rt
            logits = torch.empty(h.shape[0], self.e, dtype=torch.float32, device=h.device)
            kernels_linear.linear(h, self.router, logits, precise=rt.precise)
            choice = logits.argmax(dim=-1)
            out = torch.zeros(h.shape[0], self.d, dtype=torch.float32, device=h.device)
            for e in range(self.e):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                self.seen.add(e)
                mid = torch.empty(rows.numel(), self.f, dtype=rt.dtype, device=h.device)
                kernels_linear.linear(h[rows].contiguous(), self.w_in[e], mid, precise=rt.precise)
                part = torch.empty(rows.numel(), self.d, dtype=torch.float32, device=h.device)
                kernels_linear.linear(mid.clamp_(min=0), self.w_out[e], part, precise=rt.precise)
                out[rows] = part
            return out

    @dataclass(frozen=True)
    class RoutedToyConfig(ModelConfig):
        architecture: ClassVar[str] = "RoutedToyForCausalLM"
        model_types: ClassVar[Tuple[str, ...]] = ("routed_toy_test",)
        hidden_size: int = 48
        vocab_size: int = 77
        heads: int = 3
        kv_heads: int = 1
        head_dim: int = 32
        rot: int = 12
        stretch: float = 2.5
        base: float = 500.0
        experts: int = 3
        expert_size: int = 24
        layers: int = 2
        eps: float = 1e-6
        max_positions: int = 80

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg})

    def routed_spec(c):
        norm = lambda name: PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.eps}, {"gain": name})

        def layer(i):
            mixer = PartSpec("attention", {"hidden_size": c.hidden_size, "heads": c.heads, "kv_heads": c.kv_heads,
                                           "head_dim": c.head_dim, "qkv_bias": True, "out_bias": False,
                                           "window": None, "scale": None},
                             {k: f"l{i}.attn.{k}" for k in ("q", "k", "v", "o", "q_bias", "k_bias", "v_bias")},
                             {"position": PartSpec("toy_stretched_rotary", {"rot": c.rot, "stretch": c.stretch, "base": c.base})})
            ffn = PartSpec("toy_top1_experts", {"experts": c.experts, "hidden_size": c.hidden_size, "expert_size": c.expert_size},
                           {k: f"l{i}.experts.{k}" for k in ("router", "w_in", "w_out")})
            return LayerSpec("prenorm", {"norm_mixer": norm(f"l{i}.n1"), "mixer": mixer, "norm_ffn": norm(f"l{i}.n2"), "ffn": ffn})
        return ModelSpec("RoutedToyForCausalLM", c.hidden_size, c.vocab_size, c.max_positions,
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"table": "embed"}),
                         tuple(layer(i) for i in range(c.layers)), tuple(ScheduleEntry(i) for i in range(c.layers)),
                         norm("final"),
                         PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"weight": "head"}))

    register_architecture(RoutedToyConfig, routed_spec)
    return RoutedToyConfig


def stretched_angles(positions, rot, stretch, base):
    pairs = rot // 2
    freq = torch.tensor([base ** (-i / pairs) for i in range(pairs)], dtype=torch.float64)
    return torch.tensor(list(positions), dtype=torch.float64)[:, None] / stretch * freq[None, :]


def decisive_routing(c, w):
    """Random routers decide most tokens by a hair, which bfloat16 would turn the other way.  So
    two coordinates of the residual carry two bits of the token id, large against everything a
    layer adds, and each router reads its three logits off those two: every decision has a margin."""
    ids = torch.arange(c.vocab_size)
    w["embed"][:, 0] = 4.0 * (1 - 2 * (ids & 1)).double()
    w["embed"][:, 1] = 4.0 * (1 - 2 * ((ids >> 1) & 1)).double()
    for i in range(c.layers):
        w[f"l{i}.n2"][:2] = 1.0
        r = w[f"l{i}.experts.router"]
        r *= 0.25
        r[0, 0] += 1.0; r[0, 1] += 1.0          # both bits clear
        r[1, 0] += 1.0; r[1, 1] -= 1.0          # the second bit set
        r[2, 0] -= 1.0                          # the first bit set


def routed_plain_forward(c, w, tokens):
    """The routed toy written with the plain functions; also each routed decision's margin
    (largest router logit minus the next) and the experts chosen."""
    T = len(tokens)
    x = plain.embed(w["embed"], tokens)
    ang = stretched_angles(range(T), c.rot, c.stretch, c.base)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def turn(v):
        half = c.rot // 2
        a, b = v[..., :half], v[..., half:c.rot]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., c.rot:]], dim=-1)
    margins, chosen = [], []
    for i in range(c.layers):
        p = f"l{i}.attn."
        h = plain.rms_norm(x, w[f"l{i}.n1"], c.eps)
        q = plain.linear(h, w[p + "q"], w[p + "q_bias"]).view(T, c.heads, c.head_dim)
        k = plain.linear(h, w[p + "k"], w[p + "k_bias"]).view(T, c.kv_heads, c.head_dim)
        v = plain.linear(h, w[p + "v"], w[p + "v_bias"]).view(T, c.kv_heads, c.head_dim)
        o = plain.causal_gqa_attention(turn(q), turn(k), v).reshape(T, c.heads * c.head_dim)
        x = x + plain.linear(o, w[p + "o"])
        h = plain.rms_norm(x, w[f"l{i}.n2"], c.eps)
        logits = plain.linear(h, w[f"l{i}.experts.router"])
        top = torch.sort(logits, dim=-1, descending=True).values
        margins.append(top[:, 0] - top[:, 1])
        choice = logits.argmax(dim=-1)
        chosen.append(choice)
        w_in = w[f"l{i}.experts.w_in"].view(c.experts, c.expert_size, c.hidden_size)
        w_out = w[f"l{i}.experts.w_out"].view(c.experts, c.hidden_size, c.expert_size)
        y = torch.stack([plain.linear(torch.relu(plain.linear(h[t:t + 1], w_in[e])), w_out[e])[0]
                         for t, e in enumerate(choice.tolist())])
        x = x + y
    return plain.linear(plain.rms_norm(x, w["final"], c.eps), w["head"]), torch.stack(margins), torch.stack(chosen)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_position_encoding(tmp_path, dtype):
    from safetensors.torch import load_file

    from axon_b200.engine.build import build_engine
    from axon_b200.engine.replay import Replayer
    from axon_b200.weights import write_random_model, write_safetensors
    cfg = register_routed_toy()()
    folder = str(tmp_path / "routed")
    write_random_model(folder, cfg, seed=11, std=0.12)
    stored = load_file(folder + "/model.safetensors")
    w = {k: v.double() for k, v in stored.items()}
    decisive_routing(cfg, w)
    write_safetensors(folder + "/model.safetensors", {k: v.to(stored[k].dtype) for k, v in w.items()}, {"format": "pt"})
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    g = torch.Generator().manual_seed(4)
    seqs = {r: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for r, n in (("a", 37), ("b", 26))}
    want, margins, chosen = {}, [], []
    for r, t in seqs.items():
        want[r], m, ch = routed_plain_forward(cfg, w, t)
        margins.append(m.flatten()); chosen.append(ch.flatten())
    assert float(torch.cat(margins).min()) > 1.0, "the routing of this test is not decisive"
    assert sorted(set(torch.cat(chosen).tolist())) == list(range(cfg.experts)), "an expert is never chosen"

    engine = build_engine(folder, dtype=dtype, page_size=4, max_tokens=128, max_slots=2, max_positions=cfg.max_positions,
                          shuffle_seed=6)
    assert not engine.model.graph_safe            # parts that say nothing about graphs keep the steps eager
    tol = 2e-5 if dtype == "float32" else 3e-2
    rp, fed = Replayer(engine), {"a": 0, "b": 0}
    plan = [[("a", 11)], [("a", 2), ("b", 7)], [("a", 1), ("b", 1)], [("b", 1), ("a", 1)], [("b", 17)], [("a", 22)]]
    for k, row in enumerate(plan):
        ents, rows = [], []
        for r, n in row:
            t = seqs[r][fed[r]:fed[r] + n]
            ents.append({"id": r, "tokens": t, "want": list(range(len(t)))})
            rows += [want[r][fed[r] + j] for j in range(len(t))]
            fed[r] += len(t)
        got = rp.run_step({"step": k, "entries": ents, "end": [r for r, _ in row if fed[r] == len(seqs[r])]})
        close(got, torch.stack(rows), tol, f"routed toy, step {k}")
    assert fed == {r: len(t) for r, t in seqs.items()}
    for block in engine.model.blocks:
        assert block.ffn.seen == set(range(cfg.experts))
    engine.cache.flush()
    engine.cache.manager.check()


# ---------------------------------------------------------------------------
# A third toy: a norm and a block arrangement of their own, wide enough (512) that the products
# for few rows are split over K and leave their sums to the next reader.  Neither toy part knows
# of owed sums, so their callers have to fold first.

def register_wide_toy():
    from axon_b200.config.base import ModelConfig, register_architecture
    from axon_b200.parts import LayerSpec, ModelSpec, Part, PartSpec, ScheduleEntry, TensorDecl, register_part

    @register_part
    class CenteredNorm(Part):
        """``(x - mean) / sqrt(var + eps) * gain`` over a row."""
        category, kind = "norm", "toy_centered_norm"

        @classmethod
        def tensors(cls, spec):
            return {"gain": TensorDecl((spec.params["size"],), "gain")}

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            self.gain, self.eps = tensors["gain"], float(spec.params["eps"])

        def forward(self, x, out, rows=None):
            src = x if rows is None else x[rows.long()]
            mu = src.mean(-1, keepdim=True)
            var = ((src - mu) ** 2).mean(-1, keepdim=True)
            out.copy_(((src - mu) / torch.sqrt(var + self.eps) * self.gain.float()).to(out.dtype))

    @register_part
    class ParallelBlock(Part):
        """``x += mixer(norm(x)) + ffn(norm(x))``: both read the same normed rows."""
        category, kind = "block", "toy_parallel"
        nested = {"norm": "norm", "mixer": "mixer", "ffn": "ffn"}

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            self.norm, self.mixer, self.ffn = (build(spec.parts[k]) for k in ("norm", "mixer", "ffn"))

        def forward(self, x, ctx, cache, write_cache=True):
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            self.norm.forward(x, h)
            self.mixer.forward(h, x, ctx, cache, write_cache)
            self.ffn.forward(h, x, ctx)

    @dataclass(frozen=True)
    class WideToyConfig(ModelConfig):
        architecture: ClassVar[str] = "WideToyForCausalLM"
        model_types: ClassVar[Tuple[str, ...]] = ("wide_toy_test",)
        hidden_size: int = 512
        vocab_size: int = 131
        heads: int = 4
        kv_heads: int = 2
        head_dim: int = 128
        ffn: int = 1024
        theta: float = 3e4
        eps: float = 1e-4
        max_positions: int = 96

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg})

    def wide_spec(c):
        norm = lambda name: PartSpec("toy_centered_norm", {"size": c.hidden_size, "eps": c.eps}, {"gain": name})

        def attn(p):
            return PartSpec("attention", {"hidden_size": c.hidden_size, "heads": c.heads, "kv_heads": c.kv_heads,
                                          "head_dim": c.head_dim, "qkv_bias": True, "out_bias": False,
                                          "window": None, "scale": None},
                            {k: f"{p}.{k}" for k in ("q", "k", "v", "o", "q_bias", "k_bias", "v_bias")},
                            {"position": PartSpec("rope", {"head_dim": c.head_dim, "theta": c.theta, "pairing": "half"})})

        def ffn(p):
            return PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.ffn},
                            {k: f"{p}.{k}" for k in ("gate", "up", "down")})
        layers = (
            LayerSpec("prenorm", {"norm_mixer": norm("l0.n1"), "mixer": attn("l0.attn"),
                                  "norm_ffn": norm("l0.n2"), "ffn": ffn("l0.ffn")}),
            LayerSpec("toy_parallel", {"norm": norm("l1.n"), "mixer": attn("l1.attn"), "ffn": ffn("l1.ffn")}),
            LayerSpec("prenorm", {"norm_mixer": norm("l2.n1"), "mixer": attn("l2.attn"),
                                  "norm_ffn": norm("l2.n2"), "ffn": ffn("l2.ffn")}),
        )
        return ModelSpec("WideToyForCausalLM", c.hidden_size, c.vocab_size, c.max_positions,
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"table": "embed"}),
                         layers, tuple(ScheduleEntry(i) for i in range(3)), norm("final"),
                         PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"weight": "head"}))

    register_architecture(WideToyConfig, wide_spec)
    return WideToyConfig


def wide_plain_forward(c, w, tokens):
    T = len(tokens)
    pos = list(range(T))

    def norm(x, name):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return (x - mu) / torch.sqrt(var + c.eps) * w[name]

    def attn(h, p):
        q = plain.linear(h, w[p + ".q"], w[p + ".q_bias"]).view(T, c.heads, c.head_dim)
        k = plain.linear(h, w[p + ".k"], w[p + ".k_bias"]).view(T, c.kv_heads, c.head_dim)
        v = plain.linear(h, w[p + ".v"], w[p + ".v_bias"]).view(T, c.kv_heads, c.head_dim)
        q, k = plain.rope_half(q, pos, c.theta), plain.rope_half(k, pos, c.theta)
        o = plain.causal_gqa_attention(q, k, v).reshape(T, c.heads * c.head_dim)
        return plain.linear(o, w[p + ".o"])

    def ffn(h, p):
        return plain.swiglu_ffn(h, w[p + ".gate"], w[p + ".up"], w[p + ".down"])

    def prenorm(x, i):
        x = x + attn(norm(x, f"l{i}.n1"), f"l{i}.attn")
        return x + ffn(norm(x, f"l{i}.n2"), f"l{i}.ffn")
    x = prenorm(plain.embed(w["embed"], tokens), 0)
    h = norm(x, "l1.n")
    x = x + attn(h, "l1.attn") + ffn(h, "l1.ffn")
    x = prenorm(x, 2)
    return plain.linear(norm(x, "final"), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_norm_and_block_between_products_that_leave_sums_owed(tmp_path, dtype, monkeypatch):
    from safetensors.torch import load_file

    from axon_b200.engine.build import build_engine
    from axon_b200.engine.replay import Replayer
    from axon_b200.kernels import fast
    from axon_b200.weights import write_random_model
    cfg = register_wide_toy()()
    folder = str(tmp_path / "wide")
    write_random_model(folder, cfg, seed=21, std=0.04)
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    g = torch.Generator().manual_seed(8)
    seqs = {r: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for r, n in (("a", 45), ("b", 30))}
    want = {r: wide_plain_forward(cfg, w, t) for r, t in seqs.items()}
    # count the products that left their sums to a reader, and the separate folds that paid them
    owed_made, folds_run = [], []
    if dtype == "bfloat16":
        from axon_b200.kernels import ops
        make, fold = fast.PendingFold.__init__, ops.fold_partials

        def counted_init(self, *a, **k):
            owed_made.append(1)
            make(self, *a, **k)

        def counted_fold(pending):
            folds_run.append(1)
            return fold(pending)
        monkeypatch.setattr(fast.PendingFold, "__init__", counted_init)
        monkeypatch.setattr(ops, "fold_partials", counted_fold)
    engine = build_engine(folder, dtype=dtype, page_size=8, max_tokens=160, max_slots=2, max_positions=cfg.max_positions,
                          shuffle_seed=3)
    assert not engine.model.graph_safe
    tol = 2e-5 if dtype == "float32" else 3e-2
    rp, fed = Replayer(engine), {"a": 0, "b": 0}
    plan = [[("a", 13)], [("a", 1), ("b", 9)], [("a", 1), ("b", 1)], [("b", 20)], [("a", 2), ("b", 0)], [("a", 28)]]
    for k, row in enumerate(plan):
        ents, rows = [], []
        for r, n in row:
            if n == 0:
                continue
            t = seqs[r][fed[r]:fed[r] + n]
            ents.append({"id": r, "tokens": t, "want": list(range(len(t)))})
            rows += [want[r][fed[r] + j] for j in range(len(t))]
            fed[r] += len(t)
        got = rp.run_step({"step": k, "entries": ents, "end": [r for r, n in row if n and fed[r] == len(seqs[r])]})
        close(got, torch.stack(rows), tol, f"wide toy, step {k}")
    assert fed == {r: len(t) for r, t in seqs.items()}
    if dtype == "bfloat16":
        assert owed_made, "no product of this model left its sums to a reader: the sizes are too small for the test"
        assert folds_run, "the toy norm's callers never folded for it"


# ---------------------------------------------------------------------------
# A fourth toy: a block that holds TWO cache-keeping parts under names of its own (an attention
# over one latent row per position, kept in a cache with a single plane, beside the mixer with
# fixed-size state), so a layer's cache is a dict by part name and nothing is called "mixer".

def register_latent_toy():
    from axon_b200.config.base import ModelConfig, register_architecture
    from axon_b200.kernels import linear as kernels_linear
    from axon_b200.kernels import ops
    from axon_b200.parts import KvNeed, LayerSpec, Mixer, ModelSpec, Part, PartSpec, ScheduleEntry, TensorDecl, register_part
    register_toy()            # the running-mean mixer is defined there

    @register_part
    class LatentAttention(Mixer):
        """Every position keeps one latent row ``c = W_c h``; head ``i`` scores its query
        ``W_q,i h`` against the latents of positions 0..pos and takes their weighted sum:
        the latent is key and value at once, so the cache has one plane."""
        category, kind = "mixer", "toy_latent_attention"

        @classmethod
        def tensors(cls, spec):
            p = spec.params
            d, h, r = p["hidden_size"], p["heads"], p["latent"]
            return {"qc": TensorDecl(((h + 1) * r, d)), "o": TensorDecl((d, h * r))}

        @classmethod
        def cache_need(cls, spec):
            return KvNeed(1, int(spec.params["latent"]), planes=1)

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            p = spec.params
            self.heads, self.r = int(p["heads"]), int(p["latent"])
            self.w_qc, self.w_o = tensors["qc"], tensors["o"]

        def compute(self, h, ctx, cache):
            rt, n = self.rt, h.shape[0]
            assert cache.planes == 1 and cache.v_dim == self.r
            qc = torch.empty(n, (self.heads + 1) * self.r, dtype=torch.float32, device=h.device)
            kernels_linear.linear(h, self.w_qc, qc, precise=rt.precise)
            q = torch.empty(n, self.heads * self.r, dtype=rt.dtype, device=h.device)
            ops.rope_kv_write(qc, None, ctx.positions, ctx.token_slot, q, cache, self.heads, 0)
            att = torch.empty_like(q)
            kernels_linear.attention(q, cache, ctx, att, self.heads, 1.0 / math.sqrt(self.r), precise=rt.precise)
            out = torch.empty(n, self.w_o.shape[0], dtype=torch.float32, device=h.device)
            kernels_linear.linear(att, self.w_o, out, precise=rt.precise)
            return out

    @register_part
    class TwoMixerBlock(Part):
        """``x += recall(norm(x)) + memory(norm(x))``: two parts that each keep something."""
        category, kind = "block", "toy_two_mixers"
        nested = {"norm": "norm", "recall": "mixer", "memory": "mixer"}

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            self.norm, self.recall, self.memory = (build(spec.parts[k]) for k in ("norm", "recall", "memory"))

        def forward(self, x, ctx, cache, write_cache=True):
            assert sorted(cache) == ["memory", "recall"]
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            self.norm.forward(x, h)
            self.recall.forward(h, x, ctx, cache["recall"], write_cache)
            self.memory.forward(h, x, ctx, cache["memory"], write_cache)

    @dataclass(frozen=True)
    class LatentToyConfig(ModelConfig):
        architecture: ClassVar[str] = "LatentToyForCausalLM"
        model_types: ClassVar[Tuple[str, ...]] = ("latent_toy_test",)
        width: int = 48
        words: int = 61
        heads: int = 3
        latent: int = 24
        depth: int = 2
        eps: float = 1e-5
        longest: int = 64

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg})

    def latent_spec(c):
        norm = lambda name: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps}, {"gain": name})

        def layer(i):
            return LayerSpec("toy_two_mixers", {
                "norm": norm(f"l{i}.n"),
                "recall": PartSpec("toy_latent_attention", {"hidden_size": c.width, "heads": c.heads, "latent": c.latent},
                                   {"qc": f"l{i}.recall.qc", "o": f"l{i}.recall.o"}),
                "memory": PartSpec("toy_running_mean", {"hidden_size": c.width}, {"w": f"l{i}.memory.w"})})
        return ModelSpec("LatentToyForCausalLM", c.width, c.words, c.longest,
                         PartSpec("embedding", {"vocab_size": c.words, "hidden_size": c.width}, {"table": "embed"}),
                         tuple(layer(i) for i in range(c.depth)), tuple(ScheduleEntry(i) for i in range(c.depth)),
                         norm("final"),
                         PartSpec("linear_head", {"vocab_size": c.words, "hidden_size": c.width}, {"weight": "head"}))

    register_architecture(LatentToyConfig, latent_spec)
    return LatentToyConfig


def latent_plain_forward(c, w, tokens):
    T = len(tokens)
    x = plain.embed(w["embed"], tokens)
    for i in range(c.depth):
        h = plain.rms_norm(x, w[f"l{i}.n"], c.eps)
        qc = plain.linear(h, w[f"l{i}.recall.qc"])
        q = qc[:, :c.heads * c.latent].view(T, c.heads, c.latent)
        lat = qc[:, c.heads * c.latent:].view(T, 1, c.latent)
        o = plain.causal_gqa_attention(q, lat, lat).reshape(T, c.heads * c.latent)
        mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
        x = x + plain.linear(o, w[f"l{i}.recall.o"]) + plain.linear(mean, w[f"l{i}.memory.w"])
    return plain.linear(plain.rms_norm(x, w["final"], c.eps), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_block_with_two_cache_keeping_parts_and_a_one_plane_cache(tmp_path, dtype):
    import os
    import subprocess

    from safetensors.torch import load_file

    from axon_b200.engine.build import build_engine
    from axon_b200.engine.replay import Replayer
    from axon_b200.weights import write_random_model
    cfg = register_latent_toy()()
    folder = str(tmp_path / "latent")
    write_random_model(folder, cfg, seed=17, std=0.15)
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    engine = build_engine(folder, dtype=dtype, page_size=8, max_tokens=128, max_slots=2, max_positions=cfg.longest, shuffle_seed=4)
    # one group of pages with a single plane per position and run; a state slab per run
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].need.planes == 1
    assert engine.cache.groups[0].pool.shape == (17, cfg.depth, 8 * cfg.latent)
    assert sorted(engine.cache.states) == [(0, "memory"), (1, "memory")]
    assert engine.cache.parts(0) == ["recall", "memory"] and engine.cache.bytes_per_token() == cfg.depth * cfg.latent * (4 if dtype == "float32" else 2)
    g = torch.Generator().manual_seed(6)
    seqs = {r: torch.randint(0, cfg.words, (n,), generator=g).tolist() for r, n in (("a", 39), ("b", 21))}
    want = {r: latent_plain_forward(cfg, w, t) for r, t in seqs.items()}
    tol = 2e-5 if dtype == "float32" else 3e-2
    rp, fed = Replayer(engine), {"a": 0, "b": 0}
    plan = [[("a", 10)], [("a", 1), ("b", 6)], [("a", 2), ("b", 1)], [("b", 14)], [("a", 26)]]
    for k, row in enumerate(plan):
        ents, rows = [], []
        for r, n in row:
            t = seqs[r][fed[r]:fed[r] + n]
            ents.append({"id": r, "tokens": t, "want": list(range(len(t)))})
            rows += [want[r][fed[r] + j] for j in range(len(t))]
            fed[r] += len(t)
        got = rp.run_step({"step": k, "entries": ents, "end": [r for r, _ in row if fed[r] == len(seqs[r])]})
        close(got, torch.stack(rows), tol, f"latent toy, step {k}")
    engine.cache.flush()
    engine.cache.manager.check()
    assert engine.cache.manager.free_pages(0) == engine.cache.n_pages
    if dtype == "float32":
        # `axon info` prints an architecture it has never heard of from its spec and its own keys
        import io
        from contextlib import redirect_stdout
        from axon_b200 import cli
        buf = io.StringIO()
        with redirect_stdout(buf):
            assert cli.cmd_info(folder) == 0
        text = buf.getvalue()
        assert "LatentToyForCausalLM" in text and "layers 2 (schedule of 2 runs) / dim 48 / vocab 61 / ctx 64" in text
        assert "latent 24" in text and "keys of 24 (one plane) x 1 kv heads" in text and "state [49] float32" in text
        assert "2 x toy_two_mixers(memory: toy_running_mean, norm: rmsnorm, recall: toy_latent_attention)" in text
        assert "l1.recall.qc -> matrix BF16 [96, 48]" in text


# ---------------------------------------------------------------------------
# A part that calls itself safe for CUDA graphs and is not: the capture fails, the engine keeps
# such steps eager from then on, and the results are right all the same (the reference injects
# the failure on the host as well: src/cuda/mod.rs:148-161, src/cuda/qwen2/slots.rs:2629-2700).

def test_a_failed_graph_capture_falls_back_to_eager_steps(tmp_path):
    from safetensors.torch import load_file

    from axon_b200.config.base import ModelConfig, register_architecture
    from axon_b200.engine.build import build_engine
    from axon_b200.engine.step import StepEntry
    from axon_b200.kernels import linear as kernels_linear
    from axon_b200.parts import FeedForward, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl, register_part
    from axon_b200.weights import write_random_model

    @register_part
    class FragileFeedForward(FeedForward):
        """``W_out relu(W_in h)``; claims to be safe for graphs but refuses to run inside a capture."""
        category, kind = "ffn", "toy_fragile_ffn"
        graph_safe = True
        captures_refused = 0

        @classmethod
        def tensors(cls, spec):
            d, f = spec.params["hidden_size"], spec.params["size"]
            return {"w_in": TensorDecl((f, d)), "w_out": TensorDecl((d, f))}

        def __init__(self, spec, tensors, rt, build):
            super().__init__(spec, tensors, rt, build)
            self.w_in, self.w_out = tensors["w_in"], tensors["w_out"]

        def compute(self, h, ctx):
            if torch.cuda.is_current_stream_capturing():
                FragileFeedForward.captures_refused += 1
                raise RuntimeError("this part cannot be captured")
            mid = self.rt.buffer("fragile_mid", (h.shape[0], self.w_in.shape[0]))
            kernels_linear.linear(h, self.w_in, mid, precise=self.rt.precise)
            out = self.rt.buffer("fragile_out", (h.shape[0], self.w_out.shape[0]), torch.float32)
            kernels_linear.linear(mid.clamp_(min=0), self.w_out, out, precise=self.rt.precise)
            return out

    @dataclass(frozen=True)
    class FragileConfig(ModelConfig):
        architecture: ClassVar[str] = "FragileToyForCausalLM"
        model_types: ClassVar[Tuple[str, ...]] = ("fragile_toy_test",)
        hidden_size: int = 64
        vocab_size: int = 90
        size: int = 80
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg})

    def spec_of(c):
        norm = lambda name: PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.eps}, {"gain": name})
        attn = PartSpec("attention", {"hidden_size": c.hidden_size, "heads": 4, "kv_heads": 2, "head_dim": 16,
                                      "qkv_bias": False, "out_bias": False, "window": None, "scale": None},
                        {k: f"attn.{k}" for k in ("q", "k", "v", "o")},
                        {"position": PartSpec("rope", {"head_dim": 16, "theta": 1e4, "pairing": "half"})})
        ffn = PartSpec("toy_fragile_ffn", {"hidden_size": c.hidden_size, "size": c.size}, {"w_in": "ffn.in", "w_out": "ffn.out"})
        layer = LayerSpec("prenorm", {"norm_mixer": norm("n1"), "mixer": attn, "norm_ffn": norm("n2"), "ffn": ffn})
        return ModelSpec("FragileToyForCausalLM", c.hidden_size, c.vocab_size, 64,
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"table": "embed"}),
                         (layer,), (ScheduleEntry(0),), norm("final"),
                         PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}, {"weight": "head"}))

    register_architecture(FragileConfig, spec_of)
    c = FragileConfig()
    folder = str(tmp_path / "fragile")
    write_random_model(folder, c, seed=2, std=0.2)
    w = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    toks = torch.randint(0, c.vocab_size, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    T = len(toks)
    x = plain.embed(w["embed"], toks)
    h = plain.rms_norm(x, w["n1"], c.eps)
    q, k, v = (plain.linear(h, w[f"attn.{n}"]).view(T, heads, 16) for n, heads in (("q", 4), ("k", 2), ("v", 2)))
    pos = list(range(T))
    o = plain.causal_gqa_attention(plain.rope_half(q, pos, 1e4), plain.rope_half(k, pos, 1e4), v).reshape(T, 64)
    x = x + plain.linear(o, w["attn.o"])
    h = plain.rms_norm(x, w["n2"], c.eps)
    x = x + plain.linear(torch.relu(plain.linear(h, w["ffn.in"])), w["ffn.out"])
    want = plain.linear(plain.rms_norm(x, w["final"], c.eps), w["head"])

    for dtype in ("bfloat16", "float32"):
        FragileFeedForward.captures_refused = 0
        engine = build_engine(folder, dtype=dtype, page_size=16, max_tokens=64, max_slots=2, max_positions=64)
        assert engine.cuda_graphs, "every part says it is safe: the engine will try to capture"
        s = engine.open_request()
        got = [engine.step([StepEntry(s, toks[:20], [19])]).double().cpu()]
        for t in range(20, T):
            got.append(engine.step([StepEntry(s, [toks[t]], [0])]).double().cpu())
        assert FragileFeedForward.captures_refused == 1, "one capture was tried and failed"
        assert not engine.cuda_graphs and not engine._graphs, "steps of single tokens stay eager after the failure"
        close(torch.cat(got), want[19:], TOL[torch.float32 if dtype == "float32" else torch.bfloat16], f"{dtype}, after a failed capture")
        # the engine still steps: another request, fed in portions (a portion's capture fails too and is given up)
        s2 = engine.open_request()
        rows = [engine.step([StepEntry(s2, toks[a:a + 5], [4])]).double().cpu() for a in (0, 5, 10)]
        close(torch.cat(rows), want[[4, 9, 14]], TOL[torch.float32 if dtype == "float32" else torch.bfloat16], f"{dtype}, portions")
