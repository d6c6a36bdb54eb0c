"""The command line (`bin/spite`): what it does without a GPU (writing a random model folder, refusing bad
arguments, saying in one line that it needs a CUDA device), and, on a GPU, `random` followed by `run` as
a user types them, against the plain implementation.  The end-to-end generate test of giveen/spite's own
command line is crates/spite-cli/src/main.rs:994-1013; the flags are main.rs:282-306."""
import json
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers as H
import plain_llama4 as plain

ROOT = Path(__file__).resolve().parent.parent
SPITE = [sys.executable, str(ROOT / "bin" / "spite")]


def spite(*args, **kw):
    return subprocess.run(SPITE + [str(a) for a in args], capture_output=True, text=True, timeout=900, **kw)


def test_random_writes_a_folder_that_the_loader_takes(tmp_path):
    from spite_b200.config import load_config
    from spite_b200.weights import load_bound_tensors
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(H.CONFIG_B))
    out = tmp_path / "model"
    proc = spite("random", "--config", cfg_file, "--out", out, "--seed", 5, "--std", 0.05)
    assert proc.returncode == 0, proc.stderr
    assert "config.json and model.safetensors" in proc.stderr
    config = load_config(out)
    assert config.num_hidden_layers == 6 and config.tie_word_embeddings
    tensors = load_bound_tensors(out, config)
    assert tensors["embed.weight"].shape == (1000, 96) and tensors["embed.weight"].dtype == torch.bfloat16
    assert tensors["layers.1.ffn.experts_gate_up"].shape == (8, 128, 96)
    assert abs(float(tensors["embed.weight"].float().std()) - 0.05) < 0.005
    # the same seed writes the same bytes, another seed does not
    again = tmp_path / "again"
    assert in_process("random", "--config", cfg_file, "--out", again, "--seed", 5, "--std", 0.05)[0] == 0
    assert (again / "model.safetensors").read_bytes() == (out / "model.safetensors").read_bytes()
    other = tmp_path / "other"
    assert in_process("random", "--config", cfg_file, "--out", other, "--seed", 6, "--std", 0.05)[0] == 0
    assert (other / "model.safetensors").read_bytes() != (out / "model.safetensors").read_bytes()
    # a float32 folder keeps float32
    f32 = tmp_path / "f32"
    assert in_process("random", "--config", cfg_file, "--out", f32, "--dtype", "fp32")[0] == 0
    assert load_bound_tensors(f32, config)["embed.weight"].dtype == torch.float32


def in_process(*args):
    """`spite` with these arguments in this process: (exit code, standard error)."""
    import contextlib
    import io
    from spite_b200 import cli
    err = io.StringIO()
    with contextlib.redirect_stderr(err):
        try:
            code = cli.main([str(a) for a in args])
        except SystemExit as e:
            code = e.code if isinstance(e.code, int) else 1
            if not isinstance(e.code, int) and e.code is not None:
                print(e.code, file=err)
    return code, err.getvalue()


def test_argument_errors_are_messages_not_tracebacks(tmp_path):
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(H.CONFIG_A))
    cases = [
        (["run", "-p", "1 2 3"], "one of the arguments -m/--model --random is required"),
        (["run", "-m", "x"], "one of the arguments -p/--prompt"),
        (["run", "-m", "x", "-p", "1", "--prompt-file", "f"], "not allowed with argument"),
        (["run", "-m", "x", "-p", "1", "--max-tokens", "-1"], "--max-tokens must be positive"),
        (["run", "-m", "x", "-p", "1", "--num-pages", "0"], "--num-pages must be positive"),
        (["run", "-m", "x", "-p", "1", "--max-requests", "0"], "--max-requests must be positive"),
        (["run", "-m", "x", "-p", "1", "--dtype", "fp16"], "invalid choice"),
        (["random", "--out", "y"], "--config"),
        (["bench", "-m", "x", "--n-runs", "0"], "--n-runs must be positive"),
        (["frobnicate"], "invalid choice"),
    ]
    for args, message in cases:
        code, err = in_process(*args)
        assert code == 2 and message in err, (args, code, err)
    proc = spite("run", "-m", "x", "-p", "1", "--max-tokens", "-1")          # and once as a program
    assert proc.returncode == 2 and "--max-tokens must be positive" in proc.stderr and "Traceback" not in proc.stderr
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps(dict(H.CONFIG_A, architectures=["NoSuchModel"])))
    code, err = in_process("random", "--config", bad, "--out", tmp_path / "z")
    assert code == 1 and "unknown architecture" in err


@pytest.mark.skipif(torch.cuda.is_available(), reason="this is what happens where there is no GPU")
def test_run_without_a_gpu_says_so_in_one_line(tmp_path):
    path = H.write_model(tmp_path / "A", "A")
    proc = spite("run", "-m", path, "-p", "1 2 3", "--max-tokens", 2)
    assert proc.returncode == 2
    assert proc.stdout == "" and "Traceback" not in proc.stderr
    lines = [l for l in proc.stderr.splitlines() if l.strip()]
    assert len(lines) == 1 and "no CUDA device" in lines[0]
    code, err = in_process("replay", "--model", path, "--out", tmp_path / "o", "--max-tokens", 64)
    assert code == 2 and "no CUDA device" in err


@pytest.mark.gpu
def test_random_then_run_as_a_user_types_them(tmp_path):
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(H.CONFIG_A))
    model = tmp_path / "model"
    assert spite("random", "--config", cfg_file, "--out", model, "--seed", 11).returncode == 0
    cfg, W = plain.read_model_folder(model)
    prompt = H.random_tokens(512, 21, 9)
    proc = spite("run", "-m", model, "-p", " ".join(map(str, prompt)), "--max-tokens", 8, "--temperature", 0,
                 "--dtype", "fp32", "--page-size", 16, "--num-pages", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == plain.generate_greedy(cfg, W, prompt, 8)
    assert re.search(r"^load time    : \d+\.\d\d s$", proc.stderr, re.M)
    assert re.search(r"^generate     : 21 prompt \+ 8 new tokens in \d+\.\d\d s \(\d+\.\d\d tok/s\)$", proc.stderr, re.M)
    # a temperature, a seed for the sampler, the prompt from a file, ids separated by commas
    ids_file = tmp_path / "prompt.txt"
    ids_file.write_text(",".join(map(str, prompt)))
    want, state, ids = [], 77, list(prompt)
    for _ in range(6):
        tok, state = plain.sample_plain(plain.forward(cfg, W, ids)[-1], ids, temperature=0.7, top_p=0.95,
                                        repetition_penalty=1.1, repeat_last_n=64, state=state)
        ids.append(tok)
        want.append(tok)
    proc = spite("run", "-m", model, "--prompt-file", ids_file, "--max-tokens", 6, "--temperature", 0.7,
                 "--sample-seed", 77, "--dtype", "float32", "--max-requests", 2, "--max-batch-tokens", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == want
    # random weights without a folder, a prompt by length; the serving precision
    proc = spite("run", "--random", cfg_file, "--seed", 11, "--prompt-len", 30, "--max-tokens", 5, "--temperature", 0)
    assert proc.returncode == 0 and len(proc.stdout.split()) == 5, proc.stderr[-2000:]
    # errors a user can make
    proc = spite("run", "-m", model, "-p", "5 999999", "--max-tokens", 2)
    assert proc.returncode != 0 and "vocabulary" in proc.stderr and "Traceback" not in proc.stderr
    proc = spite("run", "-m", tmp_path / "nowhere", "-p", "5", "--max-tokens", 2)
    assert proc.returncode == 1 and "Traceback" not in proc.stderr
    # the benchmark report
    proc = spite("bench", "-m", model, "--n-prompt", 40, "--n-tokens", 12, "--n-runs", 2, "--json", "--dtype", "bf16")
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads(proc.stdout)
    assert report["n_runs"] == 2 and report["decode_tps"] > 0 and report["prefill_tps"] > 0 and report["ttft_ms"] > 0
