"""The plain implementation itself: each part against values worked out by hand
from the reference's formulas, and the whole model's structural properties."""
import math

import pytest
import torch

import helpers as H
import plain_llama4 as plain


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    s = 1.0 / math.sqrt((9 + 16) / 2 + 1e-5)
    assert torch.allclose(plain.rms_norm(x, w, 1e-5), torch.tensor([[3 * s * 2, 4 * s * 0.5]]))


def test_rotation_pairs_neighbours_and_keeps_the_norm():
    inv = plain.rotary_inv_freq({"rope_theta": 10000.0}, 4)
    assert torch.allclose(inv, torch.tensor([1.0, 0.01]))
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0]]])
    y = plain.apply_rotary(x, torch.tensor([3]), inv)
    exp = torch.tensor([math.cos(3.0), math.sin(3.0), -2 * math.sin(0.03), 2 * math.cos(0.03)])
    assert torch.allclose(y[0, 0], exp, atol=1e-6)
    assert torch.allclose(plain.apply_rotary(x, torch.tensor([0]), inv), x)
    assert torch.allclose(y.pow(2).sum(), x.pow(2).sum())


def test_llama3_frequency_bands():
    cfg = {"rope_theta": 500000.0, "rope_scaling": dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                         original_max_position_embeddings=64)}
    base = plain.rotary_inv_freq({"rope_theta": 500000.0}, 32).double()
    got = plain.rotary_inv_freq(cfg, 32).double()
    wavelen = 2 * math.pi / base
    short, long_ = wavelen < 64 / 4, wavelen > 64 / 1
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert torch.allclose(got[short], base[short]) and torch.allclose(got[long_], base[long_] / 8)
    mid = ~short & ~long_
    assert ((got[mid] < base[mid]) & (got[mid] > base[mid] / 8)).all()
    # an empty band (high == low) must not divide by zero
    cfg["rope_scaling"].update(low_freq_factor=1.0, high_freq_factor=1.0)
    assert torch.isfinite(plain.rotary_inv_freq(cfg, 32)).all()


def test_temperature_factor_uses_integer_division():
    s = plain.temperature_scale(torch.tensor([0, 14, 15, 30, 31]), 16, 0.1)
    exp = [1.0, 1.0, math.log(2) * 0.1 + 1, math.log(2) * 0.1 + 1, math.log(3) * 0.1 + 1]
    assert torch.allclose(s, torch.tensor(exp))


def test_visible_sets():
    pos = torch.arange(6)
    full = plain.visible(pos, None)
    assert full.tolist() == torch.tril(torch.ones(6, 6)).bool().tolist()
    ch = plain.visible(pos, 4)
    assert ch[3].tolist() == [True, True, True, True, False, False]
    assert ch[4].tolist() == [False, False, False, False, True, False]
    assert ch[5].tolist() == [False, False, False, False, True, True]


def test_attention_single_token_returns_its_value_and_groups_share_kv():
    q, k, v = torch.ones(1, 4, 8), torch.ones(1, 2, 8), torch.arange(16.0).view(1, 2, 8)
    o = plain.attention(q, k, v, torch.ones(1, 1, dtype=torch.bool))
    assert torch.equal(o[0, 0], v[0, 0]) and torch.equal(o[0, 1], v[0, 0]) and torch.equal(o[0, 3], v[0, 1])


def test_router_prefers_the_lower_id_and_does_not_normalise():
    x = torch.tensor([[1.0, 0.0], [0.0, 1.0]])
    w = torch.tensor([[2.0, 0.0], [2.0, 5.0], [-1.0, 5.0]])
    ids, wt, margin, _ = plain.route(x, w, 1)
    assert ids.flatten().tolist() == [0, 1]
    assert torch.allclose(wt.flatten(), torch.sigmoid(torch.tensor([2.0, 5.0])))
    assert margin.tolist() == [0.0, 0.0]
    ids2, wt2, _, _ = plain.route(x, w, 2)
    assert ids2.tolist() == [[0, 1], [1, 2]] and torch.allclose(wt2[0], torch.sigmoid(torch.tensor([2.0, 2.0])))


def test_expert_input_is_scaled_before_the_expert():
    torch.manual_seed(0)
    x = torch.randn(3, 4)
    gu, dn = torch.randn(2, 4, 6), torch.randn(2, 3, 4)
    ids, w = torch.tensor([[1], [0], [1]]), torch.tensor([[0.5], [0.25], [1.0]])
    y = plain.routed_experts(x, ids, w, gu, dn)
    xs = x[0] * 0.5
    g, u = xs @ gu[1][:, :3], xs @ gu[1][:, 3:]
    assert torch.allclose(y[0], (u * g / (1 + torch.exp(-g))) @ dn[1], atol=1e-6)
    assert not torch.allclose(y[0], 0.5 * plain.routed_experts(x, ids, torch.ones(3, 1), gu, dn)[0])


def test_greedy_tie_and_generator():
    assert plain.greedy_pick(torch.tensor([1.0, 3.0, 3.0, 0.0])) == 2
    s, u = plain.lcg_next(0)
    assert s == 1442695040888963407 and u == float(s >> 33) / 2 ** 31
    s2, _ = plain.lcg_next(s)
    assert s2 == (s * 6364136223846793005 + 1442695040888963407) % 2 ** 64
    l = torch.tensor([0.0, 1.0, 2.0, 3.0])
    assert plain.process_logits_plain(l, [], temperature=1.0, top_k=2).tolist()[:2] == [float("-inf")] * 2
    kept = plain.process_logits_plain(l, [], temperature=1.0, top_p=0.6)
    assert torch.isfinite(kept).tolist() == [False, False, False, True]       # 3 alone holds 64 %
    pen = plain.process_logits_plain(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 0], temperature=1.0,
                                     repetition_penalty=2.0, repeat_last_n=0)
    assert pen.tolist() == [1.0, -4.0, 1.0]                                    # once per distinct token


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_model_is_causal_and_chunks_forget(name, tmp_path):
    folder = H.write_model(tmp_path, name)
    cfg, tensors = plain.read_model_folder(folder)
    toks = H.random_tokens(cfg["vocab_size"], 40, 9)
    full = plain.forward(cfg, tensors, toks)
    assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(plain.forward(cfg, tensors, toks[:25]), full[:25], atol=1e-6)
    other = list(toks)
    other[0] = (other[0] + 1) % cfg["vocab_size"]
    changed = plain.forward(cfg, tensors, other)
    assert not torch.allclose(changed[39], full[39], atol=1e-7)     # the global layers still see position 0
    info = {}
    plain.forward(cfg, tensors, toks, collect=info)
    n_moe = sum(plain.layer_is_moe(cfg, L) for L in range(cfg["num_hidden_layers"]))
    assert info["router_margins"].shape == (n_moe, 40)
    assert len(plain.generate_greedy(cfg, tensors, toks[:6], 3)) == 3


def test_parts_match_the_reference_projects_generic_c_kernel():
    """Outputs of giveen/spite's generic C ops (kernels/generic/generic/ops.c: rms_norm, matmul,
    ffn, attention), stored by tests/golden/make_golden.py, against the plain functions."""
    import json
    import sys
    from pathlib import Path
    golden = Path(__file__).parent / "golden"
    sys.path.insert(0, str(golden))
    from make_golden import SIZES as s, golden_inputs
    stored = json.loads((golden / "generic_ops.json").read_text())
    assert stored["sizes"] == s
    g, i = stored["outputs"], golden_inputs(stored["seed"])
    diff = lambda a, b: float((torch.tensor(a) - b).abs().max())
    assert diff(g["rms_norm"], plain.rms_norm(i["x"], i["gain"], s["eps"])) < 2e-6
    assert diff(g["matmul"], i["x"] @ i["w"].T) < 2e-6
    assert diff(g["ffn"], plain.dense_swiglu(i["x"], i["w_gate"], i["w_up"], i["w_down"])) < 5e-6
    cfg = dict(hidden_size=s["d"], num_attention_heads=s["nq"], num_key_value_heads=s["nkv"], head_dim=s["hd"],
               rms_norm_eps=s["eps"], rope_theta=s["theta"], use_qk_norm=True, attention_chunk_size=64,
               no_rope_layers=[1])
    W = {"model.layers.0.self_attn.q_proj.weight": i["wq"], "model.layers.0.self_attn.k_proj.weight": i["wk"],
         "model.layers.0.self_attn.v_proj.weight": i["wv"], "model.layers.0.self_attn.o_proj.weight": i["wo"]}
    out, (k, v) = plain.attention_layer(cfg, W, 0, i["x"], torch.arange(s["T"]))
    assert diff(g["attention"], out) < 5e-6
    assert diff(g["values_row_3"], v[3].reshape(-1)) < 2e-6
