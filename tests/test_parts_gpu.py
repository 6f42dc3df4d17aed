"""Each part alone against the plain implementation's function of the same name, and toy parts
defined here (a mixer with state of its own, a feed-forward with routing, another position
encoding) that are registered, built and stepped without touching the package."""
import math
import os

import numpy as np
import pytest
import torch

from tests.helpers import TINY, make_model_dir, random_tokens
from tests.plain import model as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PART_TOL = {"float32": 2e-5, "bfloat16": 0.06}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return make_model_dir(tmp_path_factory.mktemp("parts"), "C")


def _model(folder, dtype):
    from glint_b200.engine.loading import build_engine, load_model
    model = load_model(folder, dtype)
    return model, build_engine(model, 512, num_slots=2, use_graphs=False)


def _ctx(engine, slot, tokens):
    from glint_b200.engine.step import StepContext, StepEntry
    entries = [StepEntry(slot, tokens, [len(tokens) - 1])]
    engine.cache.reserve([(slot, len(tokens))])
    return StepContext(engine.cache, entries, engine._upload, engine._stage)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_one_by_one(folder, dtype):
    model, engine = _model(folder, dtype)
    c, w = plain.read_config(folder), plain.read_weights(folder)
    cfg = TINY["C"][0]
    tokens = random_tokens(45, cfg["vocab_size"], 11)
    tol = PART_TOL[dtype]
    slot = engine.open()
    ctx = _ctx(engine, slot, tokens)
    act = model.rt.dtype
    cpu = lambda t: t.float().cpu()

    # embedding
    x = model.embedding.forward(ctx.token_ids, ctx)
    want_x = plain.embed(w["model.embed_tokens.weight"], tokens, c["hidden"])
    assert (cpu(x) - want_x).abs().max().item() < 1e-5

    block, lw = model.blocks[0], plain.layer_weights(w, 0)
    # norm
    n = block.pre_mixer_norm.forward(x)
    want_n = plain.rms_norm(want_x, lw["in_norm"], c["eps"])
    assert (cpu(n) - want_n).abs().max().item() < tol

    # mixer (attention with its position encoding and cache write), layers 0 (window) and 1 (global)
    for layer in (0, 1):
        blk, lwl = model.blocks[layer], plain.layer_weights(w, layer)
        nin = plain.rms_norm(want_x, lwl["in_norm"], c["eps"])
        y = blk.mixer.forward(nin.to(act).to(DEV), ctx, engine.cache.views[layer], None)
        want_y = plain.attention(nin.to(act).float(), lwl, c, layer)
        assert (cpu(y) - want_y).abs().max().item() < tol * 2, layer

    # feed-forward
    f = torch.randn(45, c["hidden"]) * 0.5
    d = block.feed_forward.forward(f.to(act).to(DEV), ctx)
    want_d = plain.feed_forward(f.to(act).float(), lw)
    assert (cpu(d) - want_d).abs().max().item() < tol * 2

    # head with its soft cap
    rows = torch.randn(3, c["hidden"])
    logits = model.head.forward(rows.to(act).to(DEV), ctx)
    head_w = w["lm_head.weight"]
    want_l = plain.softcap(rows.to(act).float() @ head_w.T, c["final_cap"])
    assert (cpu(logits) - want_l).abs().max().item() < tol * 3

    # whole block, residual updated in place
    xb = want_x.clone().to(DEV)
    model.blocks[2].forward(xb, None, ctx, engine.cache.views[2], None, None, False)
    want_b = plain.block(want_x, plain.layer_weights(w, 2), c, 2)
    assert (cpu(xb) - want_b).abs().max().item() < (1e-4 if dtype == "float32" else 0.15)
    model.rt.check_status()


# ---- a toy mixer with state, defined here, never part of the package -------------------------------------


def _register_toy():
    from glint_b200.cache import SlotStateNeed
    from glint_b200.config import BlockSpec, LayerCall, ModelSpec, PartSpec, register_architecture
    from glint_b200.parts import Part, TensorNeed, register_part

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t ; y_t = s_t W^T.  Its state is one vector per request."""

        def __init__(self, rt, params, tensors):
            super().__init__(rt, params, tensors)
            self.size, self.decay = int(params["size"]), float(params["decay"])

        def cache_need(self):
            return SlotStateNeed((self.size,), torch.float32)

        def needs(self):
            return [TensorNeed(self.names["w"], (self.size, self.size))]

        def bind(self, tensors):
            self.w = tensors[self.names["w"]].float()

        def forward(self, normed, ctx, view, state):
            out = torch.empty(normed.shape, dtype=torch.float32, device=normed.device)
            x = normed.float()
            for i, slot in enumerate(ctx.h_seq_slot):          # tokens of one request are sequential
                s = state[slot]
                for t in range(ctx.h_cu_seqlens[i], ctx.h_cu_seqlens[i + 1]):
                    s = self.decay * s + x[t]
                    out[t] = s @ self.w.T
                state[slot] = s
            return out

    class ToyConfig:
        def __init__(self, obj):
            self.obj = obj

        @classmethod
        def from_dict(cls, obj):
            return cls(obj)

        def to_dict(self):
            return dict(self.obj)

        def model_spec(self):
            o = self.obj
            H, V = o["hidden_size"], o["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "unit_offset": False}, {"weight": name})
            ffn = lambda p: PartSpec("gated", {"hidden_size": H, "intermediate_size": o["intermediate_size"],
                                               "activation": "silu"},
                                     {"gate": p + "gate", "up": p + "up", "down": p + "down"})
            toy = PartSpec("decay_toy", {"size": H, "decay": o["decay"]}, {"w": "layers.0.mix.w"})
            attn = PartSpec("attention", {"hidden_size": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                          "score_multiplier": 0.25, "softcap": None, "window": None,
                                          "position": PartSpec("rope", {"head_dim": 16, "theta": 10000.0})},
                            {"q": "layers.1.q", "k": "layers.1.k", "v": "layers.1.v", "o": "layers.1.o"})
            blocks = [BlockSpec(toy, ffn("layers.0."), pre_mixer_norm=norm("layers.0.n1"), pre_ffn_norm=norm("layers.0.n2")),
                      BlockSpec(attn, ffn("layers.1."), pre_mixer_norm=norm("layers.1.n1"), pre_ffn_norm=norm("layers.1.n2"))]
            # layer 0 runs twice (each run has a state of its own); the last entry reads entry 1's cache
            order = [LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_of=1)]
            return ModelSpec("ToyForCausalLM", V, H, o["max_position_embeddings"],
                             PartSpec("embedding", {"vocab_size": V, "hidden_size": H, "scale": 1.0}, {"table": "embed"}),
                             blocks, order, norm("final_norm"),
                             PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": None, "tie": True},
                                      {"weight": "head", "tied_to": "embed"}))

    register_part("mixer", "decay_toy", DecayMixer)
    register_architecture("ToyForCausalLM", ToyConfig)
    return ToyConfig


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    import json
    from glint_b200.engine.loading import build_engine, load_model
    from glint_b200.engine.step import StepEntry
    from glint_b200.weights import model_needs, random_tensors, write_safetensors
    ToyConfig = _register_toy()
    obj = {"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 97, "intermediate_size": 48,
           "decay": 0.9, "max_position_embeddings": 128}
    folder = str(tmp_path / "toy")
    os.makedirs(folder)
    json.dump(obj, open(os.path.join(folder, "config.json"), "w"))
    tensors = random_tensors(model_needs(ToyConfig(obj)), seed=3, std=0.2, norm_std=1.0, dtype=torch.float32)
    for k in list(tensors):
        if k.endswith("n1") or k.endswith("n2") or k == "final_norm":
            tensors[k] = tensors[k].abs() + 0.5
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)

    model = load_model(folder, "float32")
    assert type(model.blocks[0].mixer).__name__ == "DecayMixer"
    engine = build_engine(model, 256, num_slots=3, use_graphs=False)
    needs, cache_of = model.cache_needs()
    assert [type(n).__name__ for n in needs] == ["SlotStateNeed", "PagedKVNeed", "SlotStateNeed", "PagedKVNeed"]
    assert cache_of == [None, None, None, 1] and len(engine.cache.groups) == 1
    assert engine.cache.states[0].shape == (3, 32) and engine.cache.states[2].shape == (3, 32)
    assert engine.cache.states[0].data_ptr() != engine.cache.states[2].data_ptr()

    toks_a, toks_b = random_tokens(23, 97, 1), random_tokens(17, 97, 2)
    # whole
    s = engine.open()
    whole_a = engine.step([StepEntry(s, toks_a, list(range(23)))]).cpu()
    engine.close(s)
    s = engine.open()
    whole_b = engine.step([StepEntry(s, toks_b, list(range(17)))]).cpu()
    engine.close(s)
    # cut into portions and mixed with the other request; the state must carry across steps and a
    # reused slot must start from zero
    sa, sb = engine.open(), engine.open()
    got_a, got_b = [], []
    got_a.append(engine.step([StepEntry(sa, toks_a[:7], list(range(7)))]).cpu())
    out = engine.step([StepEntry(sb, toks_b[:5], list(range(5))), StepEntry(sa, toks_a[7:9], [0, 1])]).cpu()
    got_b.append(out[:5]); got_a.append(out[5:])
    out = engine.step([StepEntry(sa, toks_a[9:], list(range(14))), StepEntry(sb, toks_b[5:6], [0])]).cpu()
    got_a.append(out[:14]); got_b.append(out[14:])
    got_b.append(engine.step([StepEntry(sb, toks_b[6:], list(range(11)))]).cpu())
    assert (torch.cat(got_a) - whole_a).abs().max().item() < 1e-4
    assert (torch.cat(got_b) - whole_b).abs().max().item() < 1e-4
    assert whole_a.abs().max().item() > 1e-3
    engine.close(sa); engine.close(sb)
    model.rt.check_status()


# ---- a toy feed-forward with routing and a toy position encoding, defined here -----------------------------


def _register_routed_toy():
    from glint_b200.config import BlockSpec, LayerCall, ModelSpec, PartSpec, register_architecture
    from glint_b200.parts import Part, TensorNeed, register_part

    class RoutedFeedForward(Part):
        """Top-1 of E small experts: router logits in 32-bit, y = W2[e] silu(W1[e] x) * gate weight."""

        def __init__(self, rt, params, tensors):
            super().__init__(rt, params, tensors)
            self.H, self.I, self.E = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])

        def needs(self):
            n = self.names
            need = [TensorNeed(n["router"], (self.E, self.H))]
            for e in range(self.E):
                need += [TensorNeed(f"{n['experts']}.{e}.w1", (self.I, self.H)),
                         TensorNeed(f"{n['experts']}.{e}.w2", (self.H, self.I))]
            return need

        def bind(self, tensors):
            n = self.names
            self.router = tensors[n["router"]].float()
            self.w1 = torch.stack([tensors[f"{n['experts']}.{e}.w1"].float() for e in range(self.E)])
            self.w2 = torch.stack([tensors[f"{n['experts']}.{e}.w2"].float() for e in range(self.E)])

        def forward(self, normed, ctx):
            x = normed.float()
            logits = x @ self.router.T                                  # routing is decided in 32-bit
            weight, expert = torch.softmax(logits, dim=-1).max(dim=-1)
            h = torch.nn.functional.silu(torch.einsum("tih,th->ti", self.w1[expert], x))
            return torch.einsum("thi,ti->th", self.w2[expert], h) * weight[:, None]

    class SinusoidOffset(Part):
        """q and k get a sinusoid of the absolute position added (no rotation); v is stored as it is."""

        def __init__(self, rt, params, tensors):
            super().__init__(rt, params, tensors)
            hd = int(params["head_dim"])
            self.freq = (1.0 / (50.0 ** (torch.arange(hd, dtype=torch.float32) / hd))).to(rt.device)
            self.amplitude = float(params["amplitude"])

        def encode_and_store(self, qkv, ctx, q_out, view, nh, nkv, hd):
            T = qkv.shape[0]
            pos = ctx.positions[:T].long()
            add = self.amplitude * torch.sin(pos[:, None].float() * self.freq[None, :])       # [T, hd]
            q = qkv[:, :nh * hd].view(T, nh, hd) + add[:, None, :]
            q_out.copy_(q.reshape(T, nh * hd).to(q_out.dtype))
            if view.writes:
                k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd) + add[:, None, :]
                v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
                table = ctx.block_table(view.group).long()
                pages = table[ctx.token_seq[:T].long(), pos // view.page_size]
                view.k[pages, :, pos % view.page_size] = k.to(view.k.dtype)
                view.v[pages, :, pos % view.page_size] = v.to(view.v.dtype)

    class RoutedToyConfig:
        def __init__(self, obj):
            self.obj = obj

        @classmethod
        def from_dict(cls, obj):
            return cls(obj)

        def to_dict(self):
            return dict(self.obj)

        def model_spec(self):
            o = self.obj
            H, V, hd = o["hidden_size"], o["vocab_size"], 16
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "unit_offset": False}, {"weight": name})
            attn = lambda i, position, window: PartSpec(
                "attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": hd,
                              "score_multiplier": 0.25, "softcap": None, "window": window, "position": position},
                {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
            routed = PartSpec("routed_toy", {"hidden_size": H, "intermediate_size": 24, "experts": o["experts"]},
                              {"router": "l0.router", "experts": "l0.experts"})
            dense = PartSpec("gated", {"hidden_size": H, "intermediate_size": 40, "activation": "gelu_tanh"},
                             {"gate": "l1.gate", "up": "l1.up", "down": "l1.down"})
            blocks = [BlockSpec(attn(0, PartSpec("sinusoid_toy", {"head_dim": hd, "amplitude": 0.7}), None), routed,
                                pre_mixer_norm=norm("l0.n1"), pre_ffn_norm=norm("l0.n2")),
                      BlockSpec(attn(1, PartSpec("rope", {"head_dim": hd, "theta": 10000.0}), 8), dense,
                                pre_mixer_norm=norm("l1.n1"), pre_ffn_norm=norm("l1.n2"))]
            return ModelSpec("RoutedToyForCausalLM", V, H, o["max_position_embeddings"],
                             PartSpec("embedding", {"vocab_size": V, "hidden_size": H, "scale": 1.0}, {"table": "embed"}),
                             blocks, [LayerCall(0), LayerCall(1)], norm("final_norm"),
                             PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": None, "tie": True},
                                      {"weight": "head", "tied_to": "embed"}))

    register_part("feed_forward", "routed_toy", RoutedFeedForward)
    register_part("position", "sinusoid_toy", SinusoidOffset)
    register_architecture("RoutedToyForCausalLM", RoutedToyConfig)
    return RoutedToyConfig


def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    """A feed-forward with routing and another position encoding, both defined in this file: chosen
    layer by layer beside the package's own parts, and the logits do not depend on the cut."""
    import json
    from glint_b200.engine.loading import build_engine, load_model
    from glint_b200.engine.step import StepEntry
    from glint_b200.weights import model_needs, random_tensors, write_safetensors
    Config = _register_routed_toy()
    obj = {"architectures": ["RoutedToyForCausalLM"], "hidden_size": 48, "vocab_size": 131, "experts": 3,
           "max_position_embeddings": 128}
    folder = str(tmp_path / "routed")
    os.makedirs(folder)
    json.dump(obj, open(os.path.join(folder, "config.json"), "w"))
    tensors = random_tensors(model_needs(Config(obj)), seed=5, std=0.2, norm_std=1.0, dtype=torch.float32)
    for k in list(tensors):
        if k.endswith("n1") or k.endswith("n2") or k == "final_norm":
            tensors[k] = tensors[k].abs() + 0.5
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)

    model = load_model(folder, "float32")
    assert type(model.blocks[0].feed_forward).__name__ == "RoutedFeedForward"
    assert type(model.blocks[0].mixer.position).__name__ == "SinusoidOffset"
    assert type(model.blocks[1].mixer.position).__name__ == "Rotary"
    engine = build_engine(model, 256, num_slots=3, use_graphs=False)
    assert len(engine.cache.groups) == 2                       # all keys / a window of 8: pages of their own

    toks_a, toks_b = random_tokens(29, 131, 1), random_tokens(21, 131, 2)
    s = engine.open()
    whole_a = engine.step([StepEntry(s, toks_a, list(range(29)))]).cpu()
    engine.close(s)
    s = engine.open()
    whole_b = engine.step([StepEntry(s, toks_b, list(range(21)))]).cpu()
    engine.close(s)
    sa, sb = engine.open(), engine.open()
    got_a, got_b = [], []
    got_a.append(engine.step([StepEntry(sa, toks_a[:11], list(range(11)))]).cpu())
    out = engine.step([StepEntry(sb, toks_b[:2], [0, 1]), StepEntry(sa, toks_a[11:12], [0])]).cpu()
    got_b.append(out[:2]); got_a.append(out[2:])
    out = engine.step([StepEntry(sa, toks_a[12:], list(range(17))), StepEntry(sb, toks_b[2:20], list(range(18)))]).cpu()
    got_a.append(out[:17]); got_b.append(out[17:])
    got_b.append(engine.step([StepEntry(sb, toks_b[20:], [0])]).cpu())
    assert (torch.cat(got_a) - whole_a).abs().max().item() < 1e-4
    assert (torch.cat(got_b) - whole_b).abs().max().item() < 1e-4
    # the toy position encoding is felt: the same tokens shifted by one position give other logits
    s = engine.open()
    shifted = engine.step([StepEntry(s, [toks_a[0]] + toks_a[:28], list(range(29)))]).cpu()
    engine.close(s)
    assert (shifted[1:] - whole_a[:28]).abs().max().item() > 1e-3
    engine.close(sa); engine.close(sb)
    model.rt.check_status()


def test_runtime_buffers_are_kept_per_role():
    """``Runtime.buffer`` gives the same memory for a role again and again, different memory for
    different roles, and keeps what a role has outgrown (captured launches may point into it)."""
    from glint_b200.runtime import Runtime
    rt = Runtime(DEV, "bfloat16")
    a = rt.buffer("test.a", (8, 64))
    b = rt.buffer("test.b", (8, 64))
    assert a.dtype == torch.bfloat16 and a.shape == (8, 64) and a.data_ptr() != b.data_ptr()
    assert rt.buffer("test.a", (8, 64)) is a                                  # the view itself is kept
    assert rt.buffer("test.a", (4, 64)).data_ptr() == a.data_ptr()            # a smaller value: the same memory
    f = rt.buffer("test.a", (8, 64), torch.float32)
    assert f.dtype == torch.float32 and f.data_ptr() != a.data_ptr()          # another dtype: its own
    a.fill_(3.0)
    big = rt.buffer("test.a", (4096, 64))                                     # outgrown: new memory, the old is kept
    assert big.data_ptr() != a.data_ptr() and any(t.data_ptr() == a.data_ptr() for t in rt._retired)
    big.zero_()
    assert float(a.float().sum()) == 3.0 * 8 * 64
    assert rt.buffer("test.a", (8, 64)).data_ptr() == big.data_ptr()


# ---- another arrangement of a layer and a mixer that caches one latent vector per token, defined here ----------


def _register_parallel_latent_toy():
    from glint_b200.cache import LayerView, PagedNeed
    from glint_b200.config import BlockSpec, LayerCall, ModelSpec, PartSpec, register_architecture
    from glint_b200.parts import Part, TensorNeed, build_part, register_part

    class LatentNeed(PagedNeed):
        """One vector of ``width`` per token and layer, in pages: neither keys nor values."""

        def __init__(self, width):
            self.width = width

        def group_key(self):
            return ("latent", self.width)

        def allocate(self, layers, num_pages, page_size, dtype, device):
            return torch.zeros((layers, num_pages, page_size, self.width), dtype=torch.float32, device=device)

        def view(self, storage, layer):
            v = LayerView()
            v.latent = storage[layer]
            return v

        def bytes_per_token(self, element_size):
            return 4 * self.width

    class LatentMixer(Part):
        """c_t = Wc x_t is cached; y_t = Wo mean(c_0 .. c_t): every token reads every page of its request."""

        def __init__(self, rt, params, tensors):
            super().__init__(rt, params, tensors)
            self.size, self.width = int(params["size"]), int(params["width"])

        def cache_need(self):
            return LatentNeed(self.width)

        def needs(self):
            return [TensorNeed(self.names["c"], (self.width, self.size)), TensorNeed(self.names["o"], (self.size, self.width))]

        def bind(self, tensors):
            self.wc, self.wo = tensors[self.names["c"]].float(), tensors[self.names["o"]].float()

        def forward(self, normed, ctx, view, state):
            T, ps = normed.shape[0], view.page_size
            table = ctx.block_table(view.group).long()
            pos, seq = ctx.positions[:T].long(), ctx.token_seq[:T].long()
            view.latent[table[seq, pos // ps], pos % ps] = normed.float() @ self.wc.T
            out = torch.empty((T, self.size), dtype=torch.float32, device=normed.device)
            for i in range(ctx.num_seqs):
                lo, hi = ctx.h_cu_seqlens[i], ctx.h_cu_seqlens[i + 1]
                upto = ctx.h_seq_start[i] + hi - lo
                at = torch.arange(upto, device=normed.device)
                latents = view.latent[table[i, at // ps], at % ps]                    # [upto, width] through the pages
                means = latents.cumsum(0) / (at + 1)[:, None]
                out[lo:hi] = means[ctx.h_seq_start[i]:] @ self.wo.T
            return out

    class ParallelBlock:
        """x = x + mixer(norm(x)) + scale * feed_forward(norm(x)): one norm, both parts read it."""

        def __init__(self, rt, spec):
            self.rt = rt
            self.mixer = build_part("mixer", spec.mixer, rt)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, rt)
            self.norm = build_part("norm", spec.pre_mixer_norm, rt)
            self.scale = float(spec.params.get("ffn_scale", 1.0))

        def parts(self):
            return [p for p in (self.mixer, getattr(self.mixer, "position", None), self.feed_forward, self.norm) if p is not None]

        def cache_need(self):
            return self.mixer.cache_need()

        def entry_norm(self):
            return self.norm

        def forward(self, x, normed, ctx, view, state, next_norm=None, want_next=False):
            if normed is None:
                normed = self.norm.forward(x)
            y = self.mixer.forward(normed, ctx, view, state)
            d = self.feed_forward.forward(normed, ctx)
            x.add_(y + self.scale * d)
            return next_norm.forward(x) if want_next else None

    class ParallelToyConfig:
        def __init__(self, obj):
            self.obj = obj

        @classmethod
        def from_dict(cls, obj):
            return cls(obj)

        def to_dict(self):
            return dict(self.obj)

        def model_spec(self):
            o = self.obj
            H, V = o["hidden_size"], o["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5, "unit_offset": False}, {"weight": name})
            ffn = lambda p, act: PartSpec("gated", {"hidden_size": H, "intermediate_size": 56, "activation": act},
                                          {"gate": p + "gate", "up": p + "up", "down": p + "down"})
            latent = PartSpec("latent_toy", {"size": H, "width": o["latent_width"]}, {"c": "l0.c", "o": "l0.o"})
            attn = PartSpec("attention", {"hidden_size": H, "num_heads": 2, "num_kv_heads": 2, "head_dim": 16,
                                          "score_multiplier": 0.25, "softcap": 30.0, "window": 8,
                                          "position": PartSpec("rope", {"head_dim": 16, "theta": 10000.0})},
                            {"q": "l1.q", "k": "l1.k", "v": "l1.v", "o": "l1.o"})
            blocks = [BlockSpec(latent, ffn("l0.", "silu"), pre_mixer_norm=norm("l0.n"), kind="parallel_toy",
                                params={"ffn_scale": 0.5}),
                      BlockSpec(attn, ffn("l1.", "gelu_tanh"), pre_mixer_norm=norm("l1.n1"), pre_ffn_norm=norm("l1.n2"))]
            return ModelSpec("ParallelToyForCausalLM", V, H, o["max_position_embeddings"],
                             PartSpec("embedding", {"vocab_size": V, "hidden_size": H, "scale": 1.0}, {"table": "embed"}),
                             blocks, [LayerCall(0), LayerCall(1), LayerCall(0)], norm("final_norm"),
                             PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": None, "tie": True},
                                      {"weight": "head", "tied_to": "embed"}))

    register_part("mixer", "latent_toy", LatentMixer)
    register_part("block", "parallel_toy", ParallelBlock)
    register_architecture("ParallelToyForCausalLM", ParallelToyConfig)
    return ParallelToyConfig


def test_toy_block_kind_and_toy_latent_cache(tmp_path):
    """A layer with a parallel residual and a mixer whose cache is one latent vector per token (pages of its
    own shape, declared by a need class of its own): registered from this file, built, and stepped under cuts
    with a cache so small that pages are used again."""
    import json
    from glint_b200.cache import cache_bytes_per_token
    from glint_b200.engine.loading import build_engine, load_model
    from glint_b200.engine.step import StepEntry
    from glint_b200.weights import model_needs, random_tensors, write_safetensors
    Config = _register_parallel_latent_toy()
    obj = {"architectures": ["ParallelToyForCausalLM"], "hidden_size": 40, "vocab_size": 113, "latent_width": 12,
           "max_position_embeddings": 128}
    folder = str(tmp_path / "parallel")
    os.makedirs(folder)
    json.dump(obj, open(os.path.join(folder, "config.json"), "w"))
    tensors = random_tensors(model_needs(Config(obj)), seed=9, std=0.2, norm_std=1.0, dtype=torch.float32)
    for k in list(tensors):
        if k.endswith(".n") or k.endswith("n1") or k.endswith("n2") or k == "final_norm":
            tensors[k] = tensors[k].abs() + 0.5
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)

    model = load_model(folder, "float32")
    assert type(model.blocks[0]).__name__ == "ParallelBlock" and type(model.blocks[1]).__name__ == "Block"
    engine = build_engine(model, 96, num_slots=3, use_graphs=False)       # 6 pages per group
    needs, cache_of = model.cache_needs()
    assert [type(n).__name__ for n in needs] == ["LatentNeed", "PagedKVNeed", "LatentNeed"]
    names = sorted(g.name for g in engine.cache.groups)
    assert len(names) == 2 and any("latent" in n for n in names)
    latent_group = next(g for g in engine.cache.groups if "latent" in g.name)
    assert latent_group.members == [0, 2] and latent_group.storage.shape == (2, 6, 16, 12)
    assert cache_bytes_per_token(needs, cache_of, 4) == 2 * 4 * 12 + 2 * 2 * 16 * 4

    toks_a, toks_b = random_tokens(37, 113, 1), random_tokens(26, 113, 2)
    whole = {}
    for name, toks in (("a", toks_a), ("b", toks_b)):
        s = engine.open()
        whole[name] = engine.step([StepEntry(s, toks, list(range(len(toks))))]).cpu()
        engine.close(s)
    sa, sb = engine.open(), engine.open()
    got_a, got_b = [], []
    got_a.append(engine.step([StepEntry(sa, toks_a[:13], list(range(13)))]).cpu())
    out = engine.step([StepEntry(sb, toks_b[:2], [0, 1]), StepEntry(sa, toks_a[13:14], [0])]).cpu()
    got_b.append(out[:2]); got_a.append(out[2:])
    out = engine.step([StepEntry(sa, toks_a[14:], list(range(23))), StepEntry(sb, toks_b[2:25], list(range(23)))]).cpu()
    got_a.append(out[:23]); got_b.append(out[23:])
    got_b.append(engine.step([StepEntry(sb, toks_b[25:], [0])]).cpu())
    assert (torch.cat(got_a) - whole["a"]).abs().max().item() < 1e-4
    assert (torch.cat(got_b) - whole["b"]).abs().max().item() < 1e-4
    assert latent_group.pool.reuses > 0
    engine.close(sa); engine.close(sb)
    engine.cache.check_consistency()
    model.rt.check_status()
