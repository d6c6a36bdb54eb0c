"""safetensors reading and writing, binding by tensor name, the one error that
lists everything wrong, and the random-weights mode."""
import json
import struct

import pytest
import torch

import helpers as H
import plain_llama4 as plain
from spite_b200.config import Llama4Config
from spite_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_bound_tensors,
                                save_file, write_random_model)


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
         "e": torch.empty(0, 4)}
    save_file(t, tmp_path / "x.safetensors", {"k": "v"})
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
        for k, v in t.items():
            got = f.tensor(k)
            assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the test suite's own reader agrees
    back = plain.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(back["a"], t["a"])


def test_safetensors_damage_is_reported(tmp_path):
    p = tmp_path / "x.safetensors"
    save_file({"a": torch.randn(64, 64)}, p)
    raw = p.read_bytes()
    p.write_bytes(raw[:-100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(p)
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)


@pytest.fixture
def model_b(tmp_path):
    return H.write_model(tmp_path / "m", "B"), Llama4Config.from_dict(H.CONFIG_B)


def test_binding_by_name_and_layout(model_b):
    folder, cfg = model_b
    bound = load_bound_tensors(folder, cfg)
    raw = plain.read_safetensors(folder / "model.safetensors")
    assert set(bound) == {b.target for b in cfg.weight_bindings()}
    assert "head.weight" not in bound                                   # tied
    assert torch.equal(bound["layers.1.ffn.experts_gate_up"],
                       raw["model.layers.1.feed_forward.experts.gate_up_proj"].transpose(1, 2))
    assert bound["layers.1.ffn.experts_down"].shape == (8, 96, 64)
    assert torch.equal(bound["layers.0.mixer.q_proj"], raw["model.layers.0.self_attn.q_proj.weight"])
    assert all(t.dtype == torch.bfloat16 for t in bound.values())
    assert float(bound["final_norm.weight"].float().min()) == 1.0


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_b, tmp_path):
    folder, cfg = model_b
    t = plain.read_safetensors(folder / "model.safetensors")
    del t["model.layers.2.self_attn.k_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 96, dtype=torch.bfloat16)
    t["model.layers.3.feed_forward.experts.down_proj"] = torch.zeros(8, 96, 64, dtype=torch.bfloat16)
    t["model.layers.9.mystery"] = torch.zeros(2)
    t["vision_model.patch.weight"] = torch.zeros(2)                     # other towers are ignored
    save_file(t, folder / "model.safetensors")
    with pytest.raises(WeightError) as e:
        load_bound_tensors(folder, cfg)
    err = e.value
    assert [n for n, _ in err.missing] == ["model.layers.2.self_attn.k_proj.weight", "model.norm.weight"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight",
                                                   "model.layers.3.feed_forward.experts.down_proj"]
    assert err.unexpected == ["model.layers.9.mystery"]
    msg = str(err)
    for needle in ("missing tensors (2)", "wrong shapes (2)", "unexpected tensors (1)", "[10, 96]", "[192, 96]"):
        assert needle in msg


def test_missing_file_and_prefix_and_dtypes(model_b, tmp_path):
    folder, cfg = model_b
    with pytest.raises(WeightError, match="neither"):
        load_bound_tensors(tmp_path / "nowhere", cfg)
    t = plain.read_safetensors(folder / "model.safetensors")
    pre = {"language_model." + k: v for k, v in t.items()}
    pre["language_model.model.norm.weight"] = pre["language_model.model.norm.weight"].float() * 1.5
    pre["language_model.model.layers.0.self_attn.q_proj.weight"] = \
        pre["language_model.model.layers.0.self_attn.q_proj.weight"].to(torch.float16)
    save_file(pre, folder / "model.safetensors")
    bound = load_bound_tensors(folder, cfg)
    assert bound["final_norm.weight"].dtype == torch.float32            # stored in 32 bit: stays so
    assert float(bound["final_norm.weight"][0]) == 1.5
    assert bound["layers.0.mixer.q_proj"].dtype == torch.bfloat16       # float16 becomes bfloat16


def test_sharded_checkpoint(model_b):
    folder, cfg = model_b
    t = plain.read_safetensors(folder / "model.safetensors")
    names = sorted(t)
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, folder / "model-00001-of-00002.safetensors")
    save_file({k: t[k] for k in names[half:]}, folder / "model-00002-of-00002.safetensors")
    (folder / "model.safetensors").unlink()
    wm = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, k in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    bound = load_bound_tensors(folder, cfg)
    assert torch.equal(bound["embed.weight"], t["model.embed_tokens.weight"])


def test_random_mode_is_a_function_of_seed_and_name(tmp_path):
    cfg = Llama4Config.from_dict(H.CONFIG_A)
    a = plain.read_safetensors(write_random_model(tmp_path / "a", cfg, seed=3, std=0.02) / "model.safetensors")
    b = plain.read_safetensors(write_random_model(tmp_path / "b", cfg, seed=3, std=0.02) / "model.safetensors")
    c = plain.read_safetensors(write_random_model(tmp_path / "c", cfg, seed=4, std=0.02) / "model.safetensors")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    assert abs(float(a["lm_head.weight"].float().std()) - 0.02) < 2e-3
    assert float(a["model.layers.0.input_layernorm.weight"].float().sum()) == 64
    # a tensor's values do not depend on the other tensors of the model
    cfg6 = Llama4Config.from_dict(dict(H.CONFIG_A, num_hidden_layers=2, no_rope_layer_interval=2))
    d = plain.read_safetensors(write_random_model(tmp_path / "d", cfg6, seed=3, std=0.02) / "model.safetensors")
    assert torch.equal(a["model.layers.1.self_attn.o_proj.weight"], d["model.layers.1.self_attn.o_proj.weight"])
    saved = json.loads((tmp_path / "a" / "config.json").read_text())
    assert saved["architectures"] == ["Llama4ForCausalLM"] and Llama4Config.from_dict(saved) == cfg
