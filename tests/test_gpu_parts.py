"""The parts a layer is made of, each alone against the plain implementation's
function for it; a run order that names a layer twice and lets a layer read
another layer's cache; a toy mixer with state of its own that is defined here,
registered, built and stepped without a change to the package; and greedy
generation through the Python entry point."""
from dataclasses import dataclass, replace

import pytest
import torch

import helpers as H
import plain_llama4 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module", params=["A", "B"])
def folder(request, tmp_path_factory):
    return H.write_model(tmp_path_factory.mktemp(f"model{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def ctx(request, folder):
    from spite_b200.config import load_config
    from spite_b200.kernels.cuda import CudaKernels
    from spite_b200.parts import BuildContext
    from spite_b200.weights import load_bound_tensors
    path, name = folder
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[request.param]
    cfg = load_config(path)
    return dict(path=path, name=name, cfg=cfg, plan=cfg.plan(), dtype=dt, tol=TOL[request.param],
                build=BuildContext(CudaKernels(dt, DEV), dt, torch.device(DEV)),
                bound=load_bound_tensors(path, cfg, device=DEV), plain=H._folder_contents(str(path)))


def close(out, ref, tol, what):
    out, ref = out.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(out).all(), what
    err = float((out - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
    assert err <= tol, f"{what}: error {err:.3e} of the output scale exceeds {tol:.1e}"


def bind(part, bound, prefix):
    part.bind({n: bound[f"{prefix}.{n}"] for n in part.param_specs()})
    return part


def whole_batch(n_tokens, storage=None, start=0):
    """One request, `n_tokens` tokens from position `start`, pages 0.. in order."""
    from spite_b200.engine.batch import Segment, build_step_batch
    tables = []
    if storage is not None and storage.n_groups:
        n_pages = -(-(start + n_tokens) // storage.page_size)
        tables = [[list(range(n_pages))] for _ in range(storage.n_groups)]
    return build_step_batch([Segment("r", 0, start, n_tokens, 0, True)], [[0] * n_tokens], [[]], tables, DEV)


def normalised_input(d, T, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, d), generator=g)
    x = x / x.pow(2).mean(-1, keepdim=True).sqrt()
    return x.to(dtype)                      # both sides start from the same rounded values


def test_norm_and_position_parts(ctx):
    from spite_b200.parts import build_part
    cfg, W = ctx["plain"]
    norm = bind(build_part("norm", ctx["plan"].blocks[1].ffn_norm, ctx["build"]), ctx["bound"], "layers.1.ffn_norm")
    g = torch.Generator().manual_seed(3)
    norm.weight.copy_(torch.rand(norm.size, generator=g).to(DEV) + 0.5)
    h = torch.randn((9, cfg["hidden_size"]), generator=g) * 3
    out = torch.empty((9, cfg["hidden_size"]), dtype=ctx["dtype"], device=DEV)
    norm.forward(h.to(DEV), out)
    close(out, plain.rms_norm(h, norm.weight.cpu(), cfg["rms_norm_eps"]), ctx["tol"] / 2, "rms_norm part")
    spec = ctx["plan"].blocks[0].mixer.params["position"]
    pos = build_part("position", spec, ctx["build"])
    ref = plain.rotary_inv_freq(cfg, cfg["head_dim"])
    assert torch.allclose(pos.rotation().inv_freq.cpu(), ref, rtol=1e-6, atol=0) and pos.rotation().pairing == "neighbours"
    nope = next(b for b in ctx["plan"].blocks if b.mixer.params["position"].kind == "no_position")
    assert build_part("position", nope.mixer.params["position"], ctx["build"]).rotation() is None


@pytest.mark.parametrize("kind", ["rotary", "nope"])
def test_attention_part(ctx, kind):
    from spite_b200.cache import CacheStorage
    from spite_b200.parts import build_part
    cfg, W = ctx["plain"]
    L = next(i for i, b in enumerate(ctx["plan"].blocks)
             if (b.mixer.params["position"].kind == "no_position") == (kind == "nope"))
    mixer = bind(build_part("mixer", ctx["plan"].blocks[L].mixer, ctx["build"]), ctx["bound"], f"layers.{L}.mixer")
    T, d = 45, cfg["hidden_size"]
    storage = CacheStorage({0: mixer.cache_request()}, 16, 8, 2, ctx["dtype"], DEV)
    x = normalised_input(d, T, ctx["dtype"], 5)
    h = torch.zeros((T, d), dtype=torch.float32, device=DEV)
    mixer.forward(x.to(DEV), h, whole_batch(T, storage), storage.layer_cache(0, True))
    ref, (k, v) = plain.attention_layer(cfg, plain._strip_prefix(W), L, x.float(), torch.arange(T))
    close(h, ref, ctx["tol"], f"attention part, layer {L}")
    # what it left in the cache is what the plain layer used as keys and values
    cached = storage.kv[0][0]                                       # [2, pages, kv heads, 16, head_dim]
    got_k = cached[0].permute(0, 2, 1, 3).reshape(-1, k.shape[1], k.shape[2])[:T]
    got_v = cached[1].permute(0, 2, 1, 3).reshape(-1, k.shape[1], k.shape[2])[:T]
    close(got_k, k, ctx["tol"], "cached keys")
    close(got_v, v, ctx["tol"], "cached values")


def test_feed_forward_parts(ctx):
    from spite_b200.parts import build_part
    cfg, W = ctx["plain"]
    Wp = plain._strip_prefix(W)
    d = cfg["hidden_size"]
    kinds = {}
    for L, b in enumerate(ctx["plan"].blocks):
        kinds.setdefault(b.ffn.kind, L)
    assert "moe_sigmoid_prescaled" in kinds
    for kind, L in kinds.items():
        ffn = bind(build_part("feed_forward", ctx["plan"].blocks[L].ffn, ctx["build"]), ctx["bound"], f"layers.{L}.ffn")
        x = normalised_input(d, 400, ctx["dtype"], 7)
        if kind.startswith("moe"):
            # keep the rows whose routing no rounding can change
            _, _, margin, _ = plain.route(x.float(), Wp[f"model.layers.{L}.feed_forward.router.weight"].float(), 1)
            x = x[margin > 0.02][:150]
            assert x.shape[0] >= 100
        h = torch.zeros((x.shape[0], d), dtype=torch.float32, device=DEV)
        ffn.forward(x.to(DEV), h, None)
        close(h, plain.feed_forward_layer(cfg, Wp, L, x.float()), ctx["tol"], f"{kind} part")
        if kind.startswith("moe"):
            ids = ffn.last_routing.expert_ids[0].cpu().long()
            ref_ids, _, _, _ = plain.route(x.float(), Wp[f"model.layers.{L}.feed_forward.router.weight"].float(), 1)
            assert torch.equal(ids, ref_ids[:, 0])
            assert len(ids.unique()) > 1


def test_block_part(ctx):
    from spite_b200.cache import CacheStorage
    from spite_b200.parts.base import _REGISTRIES
    cfg, W = ctx["plain"]
    L = 0
    spec = ctx["plan"].blocks[L]
    blk = _REGISTRIES["block"][spec.arrangement](ctx["build"], spec)
    for name, child in blk.children().items():
        bind(child, ctx["bound"], f"layers.{L}.{name}")
    T, d = 30, cfg["hidden_size"]
    toks = H.decisive_tokens(ctx["path"], T, 2, 0.03 if ctx["name"] == "B" else 0.012)
    h0 = plain.embed(plain._strip_prefix(W)["model.embed_tokens.weight"], torch.tensor(toks))
    storage = CacheStorage({0: blk.mixer.cache_request()}, 16, 4, 2, ctx["dtype"], DEV)
    h = h0.to(DEV).clone()
    blk.forward(h, whole_batch(T, storage), storage.layer_cache(0, True))
    ref, _ = plain.block(cfg, plain._strip_prefix(W), L, h0, torch.arange(T))
    close(h, ref, ctx["tol"], "block part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_with_a_repeated_layer_and_a_shared_cache(folder, dtype):
    """Layer 0 runs twice (two caches), layer 1 runs once with its own cache and once more
    reading that cache without writing; the engine must agree with the plain implementation
    run in the same order, whole and cut into steps."""
    from spite_b200.config import LayerCall, load_config
    from spite_b200.engine import Engine, Model
    from spite_b200.weights import load_bound_tensors
    path, name = folder
    cfg = load_config(path)
    order = [(0, 0, True), (1, 1, True), (0, 2, True), (1, 1, False)]
    plan = replace(cfg.plan(), order=tuple(LayerCall(*o) for o in order))
    model = Model(plan, dtype=dtype, device=DEV, config=cfg)
    model.load_params(load_bound_tensors(path, cfg, device=DEV))
    pcfg, W = H._folder_contents(str(path))
    toks = H.random_tokens(pcfg["vocab_size"], 50, 9)
    if dtype == "bfloat16":
        # grow a sequence with clear routing under this run order
        import random
        rng, toks = random.Random(1), []
        while len(toks) < 50:
            cand = toks + [rng.randrange(pcfg["vocab_size"])]
            info = {}
            plain.forward(pcfg, W, cand, collect=info, order=order)
            m = info["router_margins"]
            if m.numel() == 0 or float(m[:, -1].min()) >= (0.03 if name == "B" else 0.012):
                toks = cand
    ref = plain.forward(pcfg, W, toks, order=order)
    assert not torch.allclose(ref, plain.forward(pcfg, W, toks), atol=1e-3)        # the order matters
    eng = Engine(model, cache_tokens=128, page_size=16, max_requests=2)
    whole = eng.step([("w", toks, list(range(50)))]).cpu()
    eng.finish("w")
    parts = [eng.step([("s", toks[:23], list(range(23)))]).cpu()]
    parts += [eng.step([("s", [t], [0])]).cpu() for t in toks[23:]]
    scale = float(ref.abs().max())
    for what, got in (("whole", whole), ("in steps", torch.cat(parts))):
        err = float((got - ref).abs().max()) / scale
        assert err <= TOL[dtype] * (1 if dtype == "float32" else 2), f"{what}: {err:.3e}"


# ---------------------------------------------------------------------------- a toy mixer with state
@dataclass(frozen=True)
class ToyConfig:
    hidden: int = 48
    vocab: int = 97
    decay: float = 0.8

    @classmethod
    def from_dict(cls, d):
        return cls(d.get("hidden", 48), d.get("vocab", 97), d.get("decay", 0.8))

    def plan(self):
        from spite_b200.config import BlockSpec, LayerCall, ModelPlan, PartSpec
        norm = PartSpec("rms_norm", {"size": self.hidden, "eps": 1e-5})
        toy = PartSpec("toy_decaying_sum", {"hidden_size": self.hidden, "decay": self.decay})
        attn = PartSpec("paged_attention", dict(hidden_size=self.hidden, num_heads=3, num_kv_heads=3, head_dim=16,
                                                position=PartSpec("no_position", {}), window=("sliding", 11)))
        ffn = PartSpec("dense_swiglu", {"hidden_size": self.hidden, "intermediate_size": 80})
        def layer(mixer):
            return BlockSpec("prenorm_residual", {"mixer_norm": norm, "mixer": mixer, "ffn_norm": norm, "ffn": ffn})
        blocks = (layer(toy), layer(attn), layer(toy))
        return ModelPlan(self.hidden, self.vocab, blocks, tuple(LayerCall(i, i) for i in range(3)), norm,
                         tie_word_embeddings=True, max_positions=512)


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    """A mixer defined here keeps a decaying sum per request in a fixed-size state slot:
    s_t = decay * s_{t-1} + W_in x_t,  y_t = W_out s_t.  It shares a model with the
    package's attention (sliding window) and is stepped whole, token by token, and mixed
    with another request; all must agree, and with a plain computation of the same model."""
    from spite_b200.cache import FixedState
    from spite_b200.config import config_from_dict, register_architecture
    from spite_b200.engine import Engine, Model
    from spite_b200.parts import Mixer, ParamSpec, register_mixer

    @register_mixer("toy_decaying_sum")
    class ToyDecayingSum(Mixer):
        # nothing below reads device data on the host: a step of single tokens can be captured in a CUDA graph
        graph_safe = True

        def __init__(self, ctx, hidden_size, decay):
            super().__init__(ctx)
            self.d, self.decay = hidden_size, decay

        def param_specs(self):
            return {"w_in": ParamSpec((self.d, self.d)), "w_out": ParamSpec((self.d, self.d))}

        def bind(self, params):
            self.w_in, self.w_out = params["w_in"].float(), params["w_out"].float()

        def cache_request(self):
            return None, FixedState((self.d,), torch.float32)

        def forward(self, x, h, batch, cache):
            if batch.max_seg_len == 1:
                # one token a request: every request's state in one go, by its slot.  A row that pads a
                # captured step is a copy of the first row and writes the same state to the same slot.
                slots = batch.slots.long()
                s = cache.state[slots] * self.decay + x.float() @ self.w_in.T
                cache.state[slots] = s
                h += s @ self.w_out.T
                return
            for seg in batch.segments:                      # a request's tokens in order
                rows = slice(seg.offset, seg.offset + seg.n_tokens)
                u = x[rows].float() @ self.w_in.T
                s = cache.state[seg.slot]
                states = []
                for i in range(seg.n_tokens):
                    s.mul_(self.decay).add_(u[i])
                    states.append(s.clone())
                h[rows] += torch.stack(states) @ self.w_out.T

    register_architecture("ToyStateForTests")(ToyConfig)
    cfg = config_from_dict({"architectures": ["ToyStateForTests"], "hidden": 48, "vocab": 97})
    model = Model.from_config(cfg, dtype="float32", device=DEV).init_random(seed=5, std=0.15)
    assert model.graph_safe()
    specs = model.cache_specs()
    assert specs[0][0] is None and specs[0][1].shape == (48,) and specs[1][1] is None

    # the same model, plainly: whole sequence, no cache
    def plain_toy(tokens):
        T = len(tokens)
        h = model.embed_table[torch.tensor(tokens, device=DEV)].float()
        for blk in model.blocks:
            x = plain.rms_norm(h, blk.mixer_norm.weight, 1e-5)
            if hasattr(blk.mixer, "w_in"):
                u, s, ys = x @ blk.mixer.w_in.T, torch.zeros(48, device=DEV), []
                for i in range(T):
                    s = 0.8 * s + u[i]
                    ys.append(s)
                h = h + torch.stack(ys) @ blk.mixer.w_out.T
            else:
                qkv = (x @ blk.mixer.wqkv.float().T).view(T, 9, 16)
                q, k, v = qkv[:, :3], qkv[:, 3:6], qkv[:, 6:]
                i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
                mask = ((j <= i) & (j > i - 11)).to(DEV)
                h = h + plain.attention(q, k, v, mask).reshape(T, 48) @ blk.mixer.wo.float().T
            x = plain.rms_norm(h, blk.ffn_norm.weight, 1e-5)
            f = blk.ffn.w_gate_up.shape[0] // 2
            gu = x @ blk.ffn.w_gate_up.float().T
            h = h + (plain.silu(gu[:, :f]) * gu[:, f:]) @ blk.ffn.w_down.float().T
        return (plain.rms_norm(h, model.final_norm.weight, 1e-5) @ model.embed_table.float().T).cpu()

    a, b = H.random_tokens(97, 45, 1), H.random_tokens(97, 38, 2)
    ref_a, ref_b = plain_toy(a), plain_toy(b)
    eng = Engine(model, cache_tokens=192, page_size=16, max_requests=3)
    assert eng.cuda_graphs                                  # state slots and captured decode steps go together
    scale = float(ref_a.abs().max())
    whole = eng.step([("a", a, list(range(45)))]).cpu()
    eng.finish("a")
    assert float((whole - ref_a).abs().max()) / scale < 2e-5
    # mixed: a in portions and single tokens beside b; a reuses the slot a just gave back
    got_a, got_b, ia, ib = [], [], 0, 0
    plan = [(7, 5), (2, 1), (1, 9), (12, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 0), (9, 2), (1, 14), (6, 0)]
    for na, nb in plan:
        entries = []
        if na:
            entries.append(("a", a[ia:ia + na], list(range(na))))
        if nb:
            entries.append(("b", b[ib:ib + nb], list(range(nb))))
        out = eng.step(entries).cpu()
        got_a.append(out[:na]); got_b.append(out[na:na + nb])
        ia, ib = ia + na, ib + nb
    assert ia == 45 and ib == 38 and eng.graph_replays >= 4   # the steps of one token each came from a CUDA graph
    assert float((torch.cat(got_a) - ref_a).abs().max()) / scale < 2e-5
    assert float((torch.cat(got_b) - ref_b).abs().max()) / scale < 2e-5
    eng.finish("a"); eng.finish("b")
    eng.cache.check_invariants()


# ---------------------------------------------------------------------------- a toy routed feed-forward, a toy position encoding
@dataclass(frozen=True)
class ToyRoutedConfig:
    hidden: int = 40
    vocab: int = 83

    @classmethod
    def from_dict(cls, d):
        return cls(d.get("hidden", 40), d.get("vocab", 83))

    def plan(self):
        from spite_b200.config import BlockSpec, LayerCall, ModelPlan, PartSpec
        norm = PartSpec("rms_norm", {"size": self.hidden, "eps": 1e-5})
        attn = PartSpec("paged_attention", dict(hidden_size=self.hidden, num_heads=4, num_kv_heads=2, head_dim=12,
                                                position=PartSpec("toy_harmonic_rotation", {"head_dim": 12, "base": 0.37}),
                                                window=("full", 0)))
        ffn = PartSpec("toy_top2_with_bypass", {"hidden_size": self.hidden, "num_experts": 3, "expert_size": 24})
        centered = PartSpec("toy_centered_norm", {"size": self.hidden, "eps": 1e-4})
        blocks = (BlockSpec("prenorm_residual", {"mixer_norm": norm, "mixer": attn, "ffn_norm": centered, "ffn": ffn}),) * 2
        return ModelPlan(self.hidden, self.vocab, blocks, tuple(LayerCall(i, i) for i in range(2)), norm,
                         tie_word_embeddings=True, max_positions=256)


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_are_registered_built_and_stepped():
    """Three more parts defined here: a feed-forward that sends every token to its two best experts of three
    (sigmoid weights on the input, as the kernels apply them) beside an ungated linear bypass, from the kernel
    set's operations alone; a position encoding with harmonic frequencies base / (i + 1); and a norm that
    centres a row before it scales it and adds a bias (device operations of its own, which a CUDA graph takes as
    well).  The model is graph-safe, so its decode steps replay from CUDA graphs; whole prompts, portions and
    single tokens agree with a plain computation of the same model."""
    from spite_b200.config import config_from_dict, register_architecture
    from spite_b200.engine import Engine, Model
    from spite_b200.parts import (FeedForward, Norm, ParamSpec, PositionEncoding, register_feed_forward, register_norm,
                                  register_position)

    @register_norm("toy_centered_norm")
    class ToyCenteredNorm(Norm):
        graph_safe = True

        def __init__(self, ctx, size, eps):
            super().__init__(ctx)
            self.size, self.eps = size, eps

        def param_specs(self):
            return {"weight": ParamSpec((self.size,), "ones"), "bias": ParamSpec((self.size,))}

        def bind(self, params):
            self.weight, self.bias = params["weight"].float().contiguous(), params["bias"].float().contiguous()

        def forward(self, h, out, rows=None):
            x = h if rows is None else h.index_select(0, rows.long())
            x = x - x.mean(dim=1, keepdim=True)
            out.copy_(x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + self.eps) * self.weight + self.bias)
            return out

    @register_position("toy_harmonic_rotation")
    class ToyHarmonicRotation(PositionEncoding):
        graph_safe = True

        def __init__(self, ctx, head_dim, base):
            super().__init__(ctx)
            self._freq = torch.tensor([base / (i + 1) for i in range(head_dim // 2)], dtype=torch.float32,
                                      device=ctx.device)

        def rotation(self):
            from spite_b200.parts import Rotation
            return Rotation(self._freq, "neighbours")

    @register_feed_forward("toy_top2_with_bypass")
    class ToyTop2WithBypass(FeedForward):
        graph_safe = True
        kernel_libraries = ("gemm_simt", "moe")

        def __init__(self, ctx, hidden_size, num_experts, expert_size):
            super().__init__(ctx)
            self.d, self.E, self.f = hidden_size, num_experts, expert_size

        def param_specs(self):
            return {"router": ParamSpec((self.E, self.d)), "gate_up": ParamSpec((self.E, 2 * self.f, self.d)),
                    "down": ParamSpec((self.E, self.d, self.f)), "bypass": ParamSpec((self.d, self.d))}

        def bind(self, params):
            dt = self.ctx.dtype
            self.router = params["router"].float().contiguous()
            self.gate_up, self.down = params["gate_up"].to(dt).contiguous(), params["down"].to(dt).contiguous()
            self.bypass = params["bypass"].to(dt).contiguous()

        def forward(self, x, h, batch):
            k = self.k
            routing = k.moe_route(x, self.router, 2)
            for slot in range(2):
                a = torch.empty((x.shape[0], self.f), dtype=x.dtype, device=x.device)
                k.grouped_linear_swiglu(x, self.gate_up, routing.sorted_rows[slot], routing.offsets[slot],
                                        routing.weights[slot], a)
                k.grouped_linear_accumulate(a, self.down, routing.sorted_rows[slot], routing.offsets[slot], h)
            k.linear(x, self.bypass, h, accumulate=True)

    register_architecture("ToyRoutedForTests")(ToyRoutedConfig)
    cfg = config_from_dict({"architectures": ["ToyRoutedForTests"]})
    model = Model.from_config(cfg, dtype="float32", device=DEV).init_random(seed=9, std=0.2)
    assert model.graph_safe()

    def plain_toy(tokens):
        T = len(tokens)
        h = model.embed_table[torch.tensor(tokens, device=DEV)].float().cpu()
        pos = torch.arange(T)
        for blk in model.blocks:
            m, ff = blk.mixer, blk.ffn
            x = plain.rms_norm(h, blk.mixer_norm.weight.cpu(), 1e-5)
            qkv = (x @ m.wqkv.float().cpu().T).view(T, 8, 12)
            freq = torch.tensor([0.37 / (i + 1) for i in range(6)])
            q, k, v = qkv[:, :4], qkv[:, 4:6], qkv[:, 6:]
            q, k = plain.apply_rotary(q, pos, freq), plain.apply_rotary(k, pos, freq)
            mask = pos[None, :] <= pos[:, None]
            h = h + plain.attention(q, k, v, mask).reshape(T, 48) @ m.wo.float().cpu().T
            x = h - h.mean(dim=1, keepdim=True)
            x = x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-4) * blk.ffn_norm.weight.cpu() + blk.ffn_norm.bias.cpu()
            logits = x @ ff.router.cpu().T
            order = torch.sort(logits, dim=-1, descending=True, stable=True)
            y = x @ ff.bypass.float().cpu().T
            for slot in range(2):
                for t in range(T):
                    e, w = int(order.indices[t, slot]), torch.sigmoid(order.values[t, slot])
                    gu = (x[t] * w) @ ff.gate_up[e].float().cpu().T
                    y[t] += (plain.silu(gu[:24]) * gu[24:]) @ ff.down[e].float().cpu().T
            h = h + y
        return plain.rms_norm(h, model.final_norm.weight.cpu(), 1e-5) @ model.embed_table.float().cpu().T

    a, b = H.random_tokens(83, 45, 3), H.random_tokens(83, 28, 4)
    ref_a, ref_b = plain_toy(a), plain_toy(b)
    scale = float(ref_a.abs().max())
    eng = Engine(model, cache_tokens=192, page_size=16, max_requests=3)
    assert eng.cuda_graphs
    whole = eng.step([("a", a, list(range(45)))]).cpu()
    eng.finish("a")
    assert float((whole - ref_a).abs().max()) / scale < 2e-5
    got_a, got_b, ia, ib = [], [], 0, 0
    for na, nb in [(9, 0), (2, 6), (1, 1), (1, 1), (1, 1), (14, 1), (1, 1), (1, 1), (1, 0), (1, 16), (13, 0)]:
        entries = ([("a", a[ia:ia + na], list(range(na)))] if na else []) + ([("b", b[ib:ib + nb], list(range(nb)))] if nb else [])
        out = eng.step(entries).cpu()
        got_a.append(out[:na]); got_b.append(out[na:na + nb])
        ia, ib = ia + na, ib + nb
    assert ia == 45 and ib == 28 and eng.graph_replays > 0
    assert float((torch.cat(got_a) - ref_a).abs().max()) / scale < 2e-5
    assert float((torch.cat(got_b) - ref_b).abs().max()) / scale < 2e-5
    eng.finish("a"); eng.finish("b")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folder, dtype):
    from spite_b200 import LLM, generate
    path, name = folder
    cfg, W = H._folder_contents(str(path))
    prompts = [H.random_tokens(cfg["vocab_size"], n, s) for s, n in enumerate((48, 5, 20, 33))]
    llm = LLM(path, dtype=dtype, device=DEV, cache_tokens=512, page_size=16, max_requests=3, max_batch_tokens=24)
    got = llm.generate(prompts, max_tokens=12, temperature=0.0)
    assert llm.engine.graph_replays > 0                       # decode steps came from CUDA graphs
    compared = 0
    for p, g in zip(prompts, got):
        assert len(g) == 12
        # Follow the engine's tokens and ask the plain implementation at every position which tokens it could
        # have chosen: in float32 its argmax alone, in bfloat16 every token whose logit lies within 2 % of the
        # logit scale of the maximum (three times the largest error the engine's bfloat16 logits show)
        ids = list(p)
        for i, tok in enumerate(g):
            logits = plain.forward(cfg, W, ids)[-1]
            slack = 0.02 * float(logits.abs().max()) if dtype == "bfloat16" else 0.0
            allowed = torch.nonzero(logits >= logits.max() - slack).flatten().tolist()
            if len(allowed) == 1:
                assert tok == plain.greedy_pick(logits), f"token {i} of prompt of {len(p)}"
                compared += 1
            else:
                assert tok in allowed, f"token {i} of prompt of {len(p)}: {tok} is none of {allowed}"
            ids.append(tok)
    assert compared >= (48 if dtype == "float32" else 12), f"only {compared} of 48 tokens had a clear choice"
    assert generate(path, prompts[1:2], max_tokens=5, temperature=0.0, dtype=dtype, device=DEV,
                    cache_tokens=128, page_size=16, max_requests=2) == [got[1][:5]]
    # the decode steps above were launched ahead of the reading of their ids; the plain loop gives the same
    assert llm.last_counters["steps_ahead"] > 0
    llm.decode_ahead = False
    assert llm.generate(prompts, max_tokens=12, temperature=0.0) == got
    assert llm.last_counters["steps_ahead"] == 0


# ---------------------------------------------------------------------------- another arrangement, another encoding
@dataclass(frozen=True)
class ToySandwichConfig:
    hidden: int = 56
    vocab: int = 91
    head_dim: int = 24
    rotary_dim: int = 16

    @classmethod
    def from_dict(cls, d):
        return cls()

    def to_dict(self):
        return {"architectures": ["ToySandwichForTests"]}

    def plan(self):
        from spite_b200.config import BlockSpec, LayerCall, ModelPlan, PartSpec
        norm = PartSpec("rms_norm", {"size": self.hidden, "eps": 1e-6})
        pos = PartSpec("toy_half_split_partial", {"rotary_dim": self.rotary_dim, "theta": 100.0})
        attn = PartSpec("paged_attention", dict(hidden_size=self.hidden, num_heads=4, num_kv_heads=2, head_dim=self.head_dim,
                                                position=pos, window=("sliding", 13), qk_norm_eps=1e-6,
                                                qk_norm_gain=True, qk_norm_before_rotation=True, softmax_scale=0.3))
        ffn = PartSpec("dense_swiglu", {"hidden_size": self.hidden, "intermediate_size": 72})
        blocks = (BlockSpec("toy_sandwich", {"pre_norm": norm, "mixer": attn, "post_norm": norm}),       # no feed-forward
                  BlockSpec("toy_sandwich", {"pre_norm": norm, "mixer": attn, "post_norm": norm, "ffn": ffn}))
        return ModelPlan(self.hidden, self.vocab, blocks, tuple(LayerCall(i, i) for i in range(2)), norm,
                         tie_word_embeddings=False, max_positions=256, embedding_scale=self.hidden ** 0.5,
                         logit_scale=0.5, logit_softcap=3.0)

    def weight_bindings(self):
        from spite_b200.config import WeightBinding as B
        d, hd = self.hidden, self.head_dim
        out = [B("embed.weight", "tok.weight", (self.vocab, d)), B("head.weight", "out.weight", (d, self.vocab), transform="toy_transpose"),
               B("final_norm.weight", "norm.weight", (d,), init="ones")]
        for L in range(2):
            s, t = f"blk.{L}.", f"layers.{L}."
            out += [B(t + "pre_norm.weight", s + "ln1", (d,), init="ones"), B(t + "post_norm.weight", s + "ln2", (d,), init="ones"),
                    # one fused tensor in the file for q, k and v: the transforms cut it apart
                    B(t + "mixer.q_proj", s + "wqkv", (8 * hd, d), transform="toy_rows_q"),
                    B(t + "mixer.k_proj", s + "wqkv", (8 * hd, d), transform="toy_rows_k"),
                    B(t + "mixer.v_proj", s + "wqkv", (8 * hd, d), transform="toy_rows_v"),
                    B(t + "mixer.o_proj", s + "wo", (d, 4 * hd)),
                    B(t + "mixer.q_norm", s + "qn", (hd,), init="ones"), B(t + "mixer.k_norm", s + "kn", (hd,), init="ones")]
        out += [B("layers.1.ffn.gate_proj", "blk.1.wg", (72, d)), B("layers.1.ffn.up_proj", "blk.1.wu", (72, d)),
                B("layers.1.ffn.down_proj", "blk.1.wd", (d, 72))]
        return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_arrangement_encoding_and_weight_layout_need_no_change_to_the_package(dtype, tmp_path, device=DEV, kernels=None):
    """Registered from here, none of it in the package: a block arrangement with other places than the
    built-in one (a norm before the mixer and one on its output, the feed-forward optional and without a
    norm of its own); a position encoding that pairs the two halves of the first 16 of 24 head elements
    (the pairing of crates/spite-rope/src/lib.rs:78-92); the package's attention told to normalise q and k
    before the rotation with learnt gains; weight transforms that cut a fused q/k/v tensor apart and
    transpose the head; an embedding scale and a logit soft-cap as plan data.  The model is written as a
    folder, loaded by name, stepped in every cut and compared with a plain computation."""
    from spite_b200.config import register_architecture
    from spite_b200.engine import Engine, Model
    from spite_b200.parts import Block, PositionEncoding, Rotation, register_block, register_position
    from spite_b200.weights import register_weight_transform, write_random_model
    cfg = ToySandwichConfig()
    hd, rd = cfg.head_dim, cfg.rotary_dim

    @register_position("toy_half_split_partial")
    class ToyHalfSplitPartial(PositionEncoding):
        graph_safe = True

        def __init__(self, ctx, rotary_dim, theta):
            super().__init__(ctx)
            f = torch.tensor([theta ** (-2.0 * i / rotary_dim) for i in range(rotary_dim // 2)], dtype=torch.float32)
            self._rotation = Rotation(f.to(ctx.device), "halves", rotary_dim)

        def rotation(self):
            return self._rotation

    @register_block("toy_sandwich")
    class ToySandwich(Block):
        """h += post_norm(mixer(pre_norm(h)));  h += ffn(h as it is), if there is one."""
        graph_safe = True
        places = {"pre_norm": "norm", "mixer": "mixer", "post_norm": "norm", "ffn": "feed_forward"}
        optional = ("ffn",)

        def forward(self, h, batch, cache):
            x = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
            self.pre_norm.forward(h, x)
            y = torch.zeros_like(h)                       # the mixer adds its output into what it is given
            self.mixer.forward(x, y, batch, cache)
            z = torch.empty_like(h)
            self.post_norm.forward(y, z)
            h.add_(z)
            if self.ffn is not None:
                self.ffn.forward(h.to(self.ctx.dtype), h, batch)

    register_weight_transform("toy_transpose")(lambda t: t.t().contiguous())
    register_weight_transform("toy_rows_q")(lambda t: t[:4 * hd].contiguous())
    register_weight_transform("toy_rows_k")(lambda t: t[4 * hd:6 * hd].contiguous())
    register_weight_transform("toy_rows_v")(lambda t: t[6 * hd:].contiguous())
    register_architecture("ToySandwichForTests")(ToySandwichConfig)

    folder = write_random_model(tmp_path / "toy", cfg, seed=3, std=0.15)
    W = plain.read_safetensors(folder / "model.safetensors")
    g = torch.Generator().manual_seed(1)
    for name in W:                                         # gains that are not one, so that they show
        if name.endswith(("qn", "kn", "ln1", "ln2")):
            W[name] = (torch.rand(W[name].shape, generator=g) + 0.5).to(torch.bfloat16)
    from spite_b200.weights import save_file
    save_file(W, folder / "model.safetensors")
    model = Model.from_folder(folder, dtype=dtype, device=device, kernels=kernels)
    assert [sorted(b.children()) for b in model.blocks] == [["mixer", "post_norm", "pre_norm"],
                                                            ["ffn", "mixer", "post_norm", "pre_norm"]]
    assert model.graph_safe() or kernels is not None

    def plain_toy(tokens):
        T = len(tokens)
        f = lambda n: W[n].float()
        h = f("tok.weight")[torch.tensor(tokens)] * cfg.hidden ** 0.5
        pos = torch.arange(T)
        freq = torch.tensor([100.0 ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float32)
        ang = pos.float()[:, None] * freq[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

        def rotate(t):                                      # spite-rope/src/lib.rs:83-91 on the first rd elements
            a, b = t[..., :rd // 2], t[..., rd // 2:rd]
            return torch.cat([a * cos - b * sin, a * sin + b * cos, t[..., rd:]], -1)
        for L in range(2):
            s = f"blk.{L}."
            x = plain.rms_norm(h, f(s + "ln1"), 1e-6)
            qkv = (x @ f(s + "wqkv").T).view(T, 8, hd)
            q, k, v = qkv[:, :4], qkv[:, 4:6], qkv[:, 6:]
            q = rotate(plain.rms_norm(q, f(s + "qn"), 1e-6))
            k = rotate(plain.rms_norm(k, f(s + "kn"), 1e-6))
            mask = (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - 13)
            q = q * (0.3 * hd ** 0.5)                        # plain.attention divides by sqrt(head size); the part's scale is 0.3
            y = plain.attention(q, k, v, mask).reshape(T, 4 * hd) @ f(s + "wo").T
            h = h + plain.rms_norm(y, f(s + "ln2"), 1e-6)
            if L == 1:
                h = h + plain.dense_swiglu(h, f(s + "wg"), f(s + "wu"), f(s + "wd"))
        logits = plain.rms_norm(h, f("norm.weight"), 1e-6) @ f("out.weight") * 0.5
        return 3.0 * torch.tanh(logits / 3.0)

    requests = {"a": H.random_tokens(cfg.vocab, 70, 1), "b": H.random_tokens(cfg.vocab, 33, 2), "c": H.random_tokens(cfg.vocab, 9, 3)}
    refs = {r: plain_toy(t) for r, t in requests.items()}
    tol = 2e-5 if dtype == "float32" else 4e-2
    results = {}
    for cut, steps in {"whole": H.steps_whole(requests), "last 20 one by one": H.steps_last_decoded(requests, 20),
                       "portions": H.steps_portions(requests, 2),
                       "mixed": H.steps_mixed(requests, {"a": 50, "b": 20, "c": 2}, 4)}.items():
        eng = Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=16, max_requests=3)
        results[cut] = H.run_steps(eng, steps)
        for (r, p), row in results[cut].items():
            err = float((row - refs[r][p]).abs().max()) / float(refs[r].abs().max())
            assert err <= tol, f"{cut}: request {r!r}, position {p}: error {err:.3e}"
        if cut == "last 20 one by one" and kernels is None:
            assert eng.graph_replays > 0
    if dtype == "float32" and kernels is None:
        H.assert_cuts_identical(results)
