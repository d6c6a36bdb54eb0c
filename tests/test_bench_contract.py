"""What `bench.py` promises without a GPU: more than one GPU is refused with one line and exit code 2,
the reference arm prints its `unavailable` record and exits 0, a step count that does not fit the
context is refused, and the configuration record of the default run is flat with at most 20 keys."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused():
    p = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "--gpus 2" in p.stdout


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"]


def test_steps_beyond_the_context_are_refused():
    p = run("--steps", "9000")
    assert p.returncode == 2 and "context" in p.stdout


def test_scout_shapes_are_those_of_the_baseline():
    sys.path.insert(0, str(ROOT))
    import bench
    base = json.loads((ROOT / "BASELINE.json").read_text())
    named = json.dumps(base["configs"][2])
    for key in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim", "num_local_experts",
                "intermediate_size", "vocab_size"):
        assert str(bench.SCOUT[key]) in named, key
