"""Anchors for the plain implementation: outputs of giveen/spite's own generic C
kernel (kernels/generic/generic/ops.c) on small seeded inputs.

The project's Llama 4 model code is Rust and cannot be compiled without cargo;
its generic C kernel, the scalar "ground truth" its GPU kernels are verified
against (tools/verify/verify.py), does compile with a C compiler alone.  It
computes four of the parts the plain implementation restates:
  rms_norm   ops.c:58-93      matmul   ops.c:448-465
  ffn        ops.c:136-185    (SwiGLU, accumulates into out)
  attention  ops.c:265-421    (projections, per-head RMS norm, NEOX rotation, KV
                               rows, causal softmax attention, out += Wo att)
This script builds the kernel from a checkout of the project, runs those four ops
and writes their outputs to `generic_ops.json` beside it; `tests/test_plain.py`
compares the plain implementation's functions with the stored numbers.

    python tests/golden/make_golden.py [/path/to/giveen-spite-checkout]

Two identities map the C attention onto the plain attention layer: its rotation
pairs dimension i with i + head_dim/2 where the plain one pairs 2i with 2i+1, which
is the same computation with the rows of Wq and Wk permuted inside each head; and
its weightless norm runs before the rotation where the plain one runs after, which
is equal because a rotation keeps the sum of squares.
"""
from __future__ import annotations

import ctypes as C
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent

SIZES = dict(d=24, nq=4, nkv=2, hd=8, f=20, T=7, theta=10000.0, eps=1e-5)


def golden_inputs(seed: int = 1234) -> dict:
    """The seeded inputs both the script and the test use."""
    g = torch.Generator().manual_seed(seed)
    s = SIZES
    r = lambda *shape: torch.randn(shape, generator=g)
    return dict(x=r(s["T"], s["d"]), gain=torch.rand(s["d"], generator=g) + 0.5,
                w=r(13, s["d"]) * 0.3, w_gate=r(s["f"], s["d"]) * 0.3, w_up=r(s["f"], s["d"]) * 0.3,
                w_down=r(s["d"], s["f"]) * 0.3, wq=r(s["nq"] * s["hd"], s["d"]) * 0.3,
                wk=r(s["nkv"] * s["hd"], s["d"]) * 0.3, wv=r(s["nkv"] * s["hd"], s["d"]) * 0.3,
                wo=r(s["d"], s["nq"] * s["hd"]) * 0.3)


def to_half_split(w: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    """Rows of a q/k projection reordered so that the half-split rotation of the C
    kernel acts on the pairs the neighbour rotation acts on."""
    w = w.view(heads, hd, -1)
    return torch.cat([w[:, 0::2], w[:, 1::2]], dim=1).reshape(heads * hd, -1).contiguous()


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("ne", C.c_uint32 * 4), ("nb", C.c_uint64 * 4), ("kind", C.c_int)]


class Ctx(C.Structure):
    _fields_ = [("n_ctx", C.c_int), ("n_batch", C.c_int), ("n_threads", C.c_int), ("pos", C.c_int),
                ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("gpu_stream", C.c_void_p),
                ("scratchpad", C.c_void_p), ("scratchpad_bytes", C.c_size_t)]


class KvCache(C.Structure):
    _fields_ = [("k", Tensor), ("v", Tensor), ("layer", C.c_int)]


def tensor(t: torch.Tensor) -> Tensor:
    assert t.dtype == torch.float32 and t.is_contiguous()
    rows, cols = (1, t.shape[0]) if t.dim() == 1 else t.shape
    ne = (C.c_uint32 * 4)(cols, rows, 1, 1)
    nb = (C.c_uint64 * 4)(4, 4 * cols, 4 * cols * rows, 4 * cols * rows)
    return Tensor(t.data_ptr(), ne, nb, 0)


def main(ref: Path):
    srcs = [ref / "core/quant.c"] + [ref / "kernels/generic/generic" / n for n in ("ops.c", "linear_attn.c", "kernel.c")]
    with tempfile.TemporaryDirectory() as tmp:
        so = Path(tmp) / "generic.so"
        subprocess.run(["cc", "-std=c11", "-O2", "-fPIC", "-shared", f"-I{ref}", *map(str, srcs), "-lm", "-o", str(so)],
                       check=True)
        lib = C.CDLL(str(so))
        i, s = golden_inputs(), SIZES
        ctx = Ctx(n_ctx=64, n_batch=s["T"], n_threads=1, pos=0, n_heads=s["nq"], n_kv_heads=s["nkv"])
        out = {}

        y = torch.zeros(s["T"], s["d"])
        assert lib.spite_generic_rms_norm(C.byref(tensor(y)), C.byref(tensor(i["x"])), C.byref(tensor(i["gain"])),
                                          C.c_float(s["eps"]), C.byref(ctx)) == 0
        out["rms_norm"] = y.tolist()

        y = torch.zeros(s["T"], 13)
        assert lib.spite_generic_matmul(C.byref(tensor(y)), C.byref(tensor(i["x"])), C.byref(tensor(i["w"])),
                                        C.byref(ctx)) == 0
        out["matmul"] = y.tolist()

        y = torch.zeros(s["T"], s["d"])
        assert lib.spite_generic_ffn(C.byref(tensor(y)), C.byref(tensor(i["x"])), C.byref(tensor(i["w_gate"])),
                                     C.byref(tensor(i["w_up"])), C.byref(tensor(i["w_down"])), 0, C.byref(ctx)) == 0
        out["ffn"] = y.tolist()

        kc, vc = torch.zeros(64, s["nkv"] * s["hd"]), torch.zeros(64, s["nkv"] * s["hd"])
        kv = KvCache(tensor(kc), tensor(vc), 0)
        ones = torch.ones(s["hd"])
        y = torch.zeros(s["T"], s["d"])
        wq = to_half_split(i["wq"], s["nq"], s["hd"])        # named: the C call reads their memory
        wk = to_half_split(i["wk"], s["nkv"], s["hd"])
        rc = lib.spite_generic_attention(
            C.byref(tensor(y)), C.byref(tensor(i["x"])), C.byref(tensor(wq)), C.byref(tensor(wk)),
            C.byref(tensor(i["wv"])), C.byref(tensor(i["wo"])), C.byref(tensor(ones)), C.byref(tensor(ones)),
            C.c_float(s["eps"]), C.byref(kv), C.c_float(s["theta"]), C.byref(ctx))
        assert rc == 0, rc
        out["attention"] = y.tolist()
        out["values_row_3"] = vc[3].tolist()
    (HERE / "generic_ops.json").write_text(json.dumps({"sizes": SIZES, "seed": 1234, "outputs": out}))
    print("wrote", HERE / "generic_ops.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of giveen/spite>")
    main(Path(sys.argv[1]))
