"""Plain, slow Llama 4 text decoder: whole sequences, no cache, float32 on the CPU.

This file is the oracle of the test suite.  It shares no code with the product
package: it parses config.json and model.safetensors by itself and computes
every part with ordinary torch tensor arithmetic, one function per part.

It rests on the formulas of giveen/spite's scalar Llama 4 path; each function
cites the file and lines it restates (paths are relative to that project).  The
project's Rust model code cannot be compiled in an environment without cargo,
so equality with it is argued from the formulas; `tests/golden/` anchors the
parts that its generic C kernel does compute (norm, projections, SwiGLU,
causal attention).

Where the target checkpoint convention differs from that project's GGUF path
(interleaved rotary pairs, llama3 frequency scaling, chunked instead of sliding
local attention, constants read from config.json instead of being hard-coded)
the function says so.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
           "I32": torch.int32, "I64": torch.int64}


# ----------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw tensor bytes."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _DTYPES[info["dtype"]]
        buf = bytearray(raw[base + lo:base + hi])
        t = torch.frombuffer(buf, dtype=dt) if hi > lo else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def read_model_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    cfg = dict(cfg.get("text_config", cfg))
    tensors = read_safetensors(folder / "model.safetensors")
    return cfg, tensors


def _strip_prefix(tensors):
    out = {}
    for k, v in tensors.items():
        if k.startswith("language_model."):
            k = k[len("language_model."):]
        out[k] = v
    return out


# ----------------------------------------------------------------------------
# schedule of layer kinds
# ----------------------------------------------------------------------------
def layer_uses_rope(cfg, layer: int) -> bool:
    """crates/spite-models/src/llama/llama4.rs:155 — `(layer+1) % no_rope_step != 0`.
    There the step is fixed to 4 (llama4.rs:95); here it is config data: either
    the list `no_rope_layers` (1 = rotary layer, 0 = NoPE layer) or the interval
    `no_rope_layer_interval`."""
    lst = cfg.get("no_rope_layers")
    if lst:
        return bool(lst[layer])
    step = int(cfg.get("no_rope_layer_interval", 4))
    return (layer + 1) % step != 0


def layer_is_moe(cfg, layer: int) -> bool:
    """crates/spite-models/src/llama/llama4.rs:44-47 — step > 0 and (layer+1) % step == 0."""
    lst = cfg.get("moe_layers")
    if lst is not None:
        return layer in lst
    step = int(cfg.get("interleave_moe_layer_step", 1))
    return step > 0 and (layer + 1) % step == 0


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def embed(table, token_ids):
    """llama4.rs:118-119 — the token's row of the table, unscaled."""
    return table[token_ids].float()


def rms_norm(x, weight, eps):
    """crates/spite-models/src/dense.rs:175-181 — x * 1/sqrt(mean(x^2)+eps) * w."""
    x = x.float()
    scale = 1.0 / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = x * scale
    return y if weight is None else y * weight.float()


def rotary_inv_freq(cfg, head_dim):
    """crates/spite-rope/src/lib.rs:78-82 — freq_i = theta^(-2i/head_dim).
    The llama3 rescaling of the frequencies (none in that project, which rejects
    files with frequency tensors, llama4.rs:56-62) follows the public rule: long
    wavelengths are divided by `factor`, short ones kept, the band between is
    blended; an empty band (high == low) is skipped."""
    theta = float(cfg.get("rope_theta", 10000.0))
    half = head_dim // 2
    freqs = [theta ** (-2.0 * i / head_dim) for i in range(half)]
    sc = cfg.get("rope_scaling")
    if sc:
        factor = float(sc["factor"])
        low = float(sc.get("low_freq_factor", 1.0))
        high = float(sc.get("high_freq_factor", 4.0))
        orig = float(sc["original_max_position_embeddings"])
        out = []
        for f in freqs:
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                out.append(f)
            elif wavelen > orig / low:
                out.append(f / factor)
            else:
                s = (orig / wavelen - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        freqs = out
    return torch.tensor(freqs, dtype=torch.float64).to(torch.float32)


def apply_rotary(x, positions, inv_freq):
    """crates/spite-rope/src/lib.rs:83-91 — x0' = x0 cos a - x1 sin a,
    x1' = x0 sin a + x1 cos a with a = pos * freq_i, on every head.  That
    project pairs (i, i + head_dim/2); the checkpoint convention targeted here
    pairs neighbours (2i, 2i+1).
    x: [T, heads, head_dim]; positions: [T]."""
    T, H, D = x.shape
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]       # [T, D/2] in float32
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * cos - x1 * sin
    out[..., 1::2] = x0 * sin + x1 * cos
    return out


def qk_norm(x, eps):
    """llama4.rs:161-176 — after the rotation, every head of q and k is
    RMS-normalised with a vector of ones as weight and the model's eps."""
    return rms_norm(x, None, eps)


def temperature_scale(positions, floor_scale, attn_scale):
    """llama4.rs:177-183 — q *= ln(floor((pos+1)/floor_scale) + 1) * attn_scale + 1
    on layers without rotation (constants 8192 and 0.1 there, config data here)."""
    p = positions.to(torch.int64)
    fl = torch.div(p + 1, int(floor_scale), rounding_mode="floor").to(torch.float32)
    return torch.log(fl + 1.0) * float(attn_scale) + 1.0


def visible(positions, chunk):
    """Mask [T, T]: key j is visible to query i.  crates/spite-compute/src/flash_attn.rs:118-121
    gives the causal rule j <= i.  Local layers: llama4.rs:189-197 keeps the last
    `win` rows (a sliding window); the architecture's own rule, used here, keeps the
    keys of the query's chunk: floor(j/C) == floor(i/C)."""
    i = positions[:, None]
    j = positions[None, :]
    m = j <= i
    if chunk is not None:
        m = m & (torch.div(j, chunk, rounding_mode="floor") == torch.div(i, chunk, rounding_mode="floor"))
    return m


def attention(q, k, v, mask):
    """crates/spite-compute/src/flash_attn.rs:111-156 — per query head h with kv
    head h // (nq/nkv): s_j = (q.k_j)/sqrt(head_dim), masked to -inf, p = exp(s - max)
    / max(sum, 1e-30), o = sum_j p_j v_j.
    q: [T, nq, D]; k, v: [T, nkv, D]; mask: [T, T] -> [T, nq, D]."""
    T, nq, D = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        p = p / p.sum(dim=-1, keepdim=True).clamp_min(1e-30)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def silu(g):
    """crates/spite-models/src/moe.rs:203 — g / (1 + exp(-g))."""
    return g / (1.0 + torch.exp(-g))


def dense_swiglu(x, w_gate, w_up, w_down):
    """llama4.rs:257-271 — down( silu(gate x) * (up x) )."""
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def route(x, w_router, top_k):
    """moe.rs:65-66 logits = Wr x; moe.rs:110-123 — pick top-k by raw logit
    (descending, stable: equal logits keep the lower expert id first), weight =
    sigmoid(logit).  Returns ids [T,k], weights [T,k], and the margin between
    the last chosen and the first rejected logit of every token."""
    logits = x @ w_router.float().T                                # [T, E]
    order = torch.sort(logits, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :top_k]
    chosen = order.values[:, :top_k]
    w = 1.0 / (1.0 + torch.exp(-chosen))
    if logits.shape[1] > top_k:
        margin = order.values[:, top_k - 1] - order.values[:, top_k]
    else:
        margin = torch.full((x.shape[0],), float("inf"))
    return ids, w, margin, logits


def routed_experts(x, ids, weights, gate_up, down):
    """moe.rs:172-191 — the token is scaled by its weight *before* the expert,
    up = Wu xw, gate = Wg xw, up *= silu(gate), y = Wd up; outputs of the chosen
    experts are summed without further weighting.
    The checkpoint stores gate_up [E, d, 2f] (gate columns first) and down
    [E, f, d], both input-major."""
    T, d = x.shape
    f = down.shape[1]
    out = torch.zeros(T, d)
    for slot in range(ids.shape[1]):
        for e in ids[:, slot].unique().tolist():
            rows = torch.nonzero(ids[:, slot] == e).flatten()
            xw = x[rows] * weights[rows, slot][:, None]
            gu = xw @ gate_up[e].float()
            a = gu[:, f:] * silu(gu[:, :f])
            out[rows] += a @ down[e].float()
    return out


def shared_expert(x, w_gate, w_up, w_down):
    """llama4.rs:231-256 — on the unscaled token: down( up x * silu(gate x) ), weight 1."""
    return ((x @ w_up.T) * silu(x @ w_gate.T)) @ w_down.T


def lm_head(h, norm_w, head_w, eps):
    """llama4.rs:277-279 — logits = W_out rmsnorm(h)."""
    return rms_norm(h, norm_w, eps) @ head_w.float().T


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------
def _sizes(cfg):
    d = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim") or d // nq
    return d, nq, nkv, hd, float(cfg.get("rms_norm_eps", 1e-5))


def attention_layer(cfg, W, L, x, pos, shared_kv=None):
    """The mixer of layer L on normalised input x [T, d]: llama4.rs:129-207 without the
    residual add.  Returns (output [T, d], (k, v)).  With `shared_kv` the layer reads
    another layer's keys and values instead of making its own."""
    d, nq, nkv, hd, eps = _sizes(cfg)
    T = x.shape[0]
    p = f"model.layers.{L}."
    g = lambda name: W[name].float()
    q = (x @ g(p + "self_attn.q_proj.weight").T).view(T, nq, hd)
    k = (x @ g(p + "self_attn.k_proj.weight").T).view(T, nkv, hd)
    v = (x @ g(p + "self_attn.v_proj.weight").T).view(T, nkv, hd)
    if layer_uses_rope(cfg, L):
        inv_freq = rotary_inv_freq(cfg, hd)
        q = apply_rotary(q, pos, inv_freq)
        k = apply_rotary(k, pos, inv_freq)
        if cfg.get("use_qk_norm", True):
            q, k = qk_norm(q, eps), qk_norm(k, eps)
        mask = visible(pos, cfg.get("attention_chunk_size", 8192))
    else:
        if cfg.get("attn_temperature_tuning", True):
            s = temperature_scale(pos, cfg.get("floor_scale", 8192), cfg.get("attn_scale", 0.1))
            q = q * s[:, None, None]
        mask = visible(pos, None)
    if shared_kv is not None:
        k, v = shared_kv
    o = attention(q, k, v, mask).reshape(T, nq * hd)
    return o @ g(p + "self_attn.o_proj.weight").T, (k, v)


def feed_forward_layer(cfg, W, L, x, margins=None):
    """The feed-forward of layer L on normalised input x: llama4.rs:212-271."""
    p = f"model.layers.{L}."
    g = lambda name: W[name].float()
    if layer_is_moe(cfg, L):
        ids, w, margin, _ = route(x, g(p + "feed_forward.router.weight"), int(cfg.get("num_experts_per_tok", 1)))
        if margins is not None:
            margins.append(margin)
        y = routed_experts(x, ids, w, W[p + "feed_forward.experts.gate_up_proj"],
                           W[p + "feed_forward.experts.down_proj"])
        return y + shared_expert(x, g(p + "feed_forward.shared_expert.gate_proj.weight"),
                                 g(p + "feed_forward.shared_expert.up_proj.weight"),
                                 g(p + "feed_forward.shared_expert.down_proj.weight"))
    return dense_swiglu(x, g(p + "feed_forward.gate_proj.weight"), g(p + "feed_forward.up_proj.weight"),
                        g(p + "feed_forward.down_proj.weight"))


def block(cfg, W, L, h, pos, shared_kv=None, margins=None):
    """One layer on the residual stream: llama4.rs:126-127, 202-211, 272-274."""
    eps = _sizes(cfg)[4]
    p = f"model.layers.{L}."
    o, kv = attention_layer(cfg, W, L, rms_norm(h, W[p + "input_layernorm.weight"].float(), eps), pos, shared_kv)
    h = h + o
    h = h + feed_forward_layer(cfg, W, L, rms_norm(h, W[p + "post_attention_layernorm.weight"].float(), eps), margins)
    return h, kv


def forward(cfg, tensors, token_ids, *, collect=None, order=None):
    """Logits [T, vocab] (float32) of one whole sequence starting at position 0.
    llama4.rs:116-279 restated for all positions at once.
    `collect`, if a dict, receives the per-layer router margins.  `order`, a list of
    (layer, cache id, writes), runs the layers in another order than 0..n-1; a run
    that does not write reads the keys and values of the run that wrote its cache id."""
    W = _strip_prefix(tensors)
    eps = _sizes(cfg)[4]
    tokens = torch.as_tensor(token_ids, dtype=torch.long)
    T = tokens.numel()
    pos = torch.arange(T)
    h = embed(W["model.embed_tokens.weight"], tokens)
    margins, caches = [], {}
    if order is None:
        order = [(L, L, True) for L in range(cfg["num_hidden_layers"])]
    for L, cache_id, writes in order:
        h, kv = block(cfg, W, L, h, pos, None if writes else caches[cache_id], margins)
        if writes:
            caches[cache_id] = kv
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    if collect is not None:
        collect["router_margins"] = torch.stack(margins) if margins else torch.zeros(0, T)
    return lm_head(h, W["model.norm.weight"].float(), head, eps)


def generate_greedy(cfg, tensors, prompt, n_new):
    """crates/spite-executor/src/lib.rs:666-676 with temperature 0: the argmax
    of the last row is appended and the whole sequence is run again."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, tensors, ids)[-1]
        tok = greedy_pick(logits)
        ids.append(tok)
        out.append(tok)
    return out


def greedy_pick(logits) -> int:
    """crates/spite-sampling/src/lib.rs:236-243 — argmax; Rust's `max_by` returns
    the last of equal maxima, i.e. the highest index."""
    m = logits.max()
    idx = torch.nonzero(logits == m).flatten()
    return int(idx[-1])


# ----------------------------------------------------------------------------
# sampling (crates/spite-sampling/src/lib.rs)
# ----------------------------------------------------------------------------
_MASK64 = (1 << 64) - 1


def lcg_next(state: int):
    """lib.rs:343-348 — s = s*6364136223846793005 + 1442695040888963407 (mod 2^64);
    u = (s >> 33) / 2^31."""
    state = (state * 6364136223846793005 + 1442695040888963407) & _MASK64
    return state, float(state >> 33) / 2147483648.0


def process_logits_plain(logits, context, *, temperature, top_k=0, top_p=1.0, min_p=0.0,
                         repetition_penalty=1.0, repeat_last_n=64):
    """lib.rs:273-279 — penalty, temperature, min_p, top_k, top_p, in this order."""
    l = logits.clone().float()
    if abs(repetition_penalty - 1.0) >= 1.1920929e-07:                   # lib.rs:208-231
        window = context if repeat_last_n == 0 or repeat_last_n >= len(context) else context[-repeat_last_n:]
        for t in set(int(x) for x in window):
            if 0 <= t < l.numel():
                l[t] = l[t] / repetition_penalty if l[t] > 0 else l[t] * repetition_penalty
    if temperature > 0:                                                  # lib.rs:117-125
        l = l / temperature
    if min_p > 0:                                                        # lib.rs:178-189
        l[l < l.max() + math.log(min_p)] = float("-inf")
    if top_k and top_k < l.numel():                                      # lib.rs:128-143
        thresh = torch.sort(l, descending=True).values[top_k - 1]
        l[l < thresh] = float("-inf")
    if top_p < 1.0:                                                      # lib.rs:146-174
        order = torch.sort(l, descending=True, stable=True)
        mass = torch.exp(order.values - order.values[0])
        total = mass.sum()
        cum = torch.cumsum(mass, 0) / total
        kept = int(torch.nonzero(cum >= top_p)[0]) + 1 if bool((cum >= top_p).any()) else l.numel()
        l[order.indices[max(kept, 1):]] = float("-inf")
    return l


def sample_plain(logits, context, *, temperature, state=0, **processors):
    """lib.rs:283-296 — the processors, then argmax (temperature <= 0) or a multinomial
    draw against unnormalised masses (lib.rs:247-265).  Returns (token, state)."""
    l = process_logits_plain(logits, context, temperature=temperature, **processors)
    if temperature <= 0:
        return greedy_pick(l), state
    state, u = lcg_next(state)
    mass = torch.exp(l - l.max())
    target = torch.tensor(u, dtype=torch.float32) * mass.sum()
    cum = torch.cumsum(mass, 0)
    hit = torch.nonzero(cum >= target)
    return (int(hit[0]) if hit.numel() else greedy_pick(l)), state
