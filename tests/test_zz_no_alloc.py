"""`spite_sample_noalloc`, the sampling entry point for callers that cannot
allocate device memory (inside a stream capture, under a foreign allocator, in a
loop that must not hit cudaMalloc's synchronisation): it keeps its scratch rows in
a fixed array of the library.  The test calls it through its exported C symbol,
as such a caller would, and checks that it returns what the allocating entry
point `spite_sample` returns, on two calls in a row (the second call finds the
first call's leftovers in the shared scratch), and that it refuses a request
larger than its scratch.  The file sorts last so that a run that stops at the
first failure has run every other test before."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


class NoAllocArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("temperature", C.c_void_p), ("top_k", C.c_void_p),
                ("top_p", C.c_void_p), ("min_p", C.c_void_p), ("repetition_penalty", C.c_void_p),
                ("context", C.c_void_p), ("context_offsets", C.c_void_p), ("rng_state", C.c_void_p),
                ("out_tokens", C.c_void_p), ("rows", C.c_int), ("vocab", C.c_int)]


MAX_FLOATS = 2 * 1024 * 1024


def test_no_alloc_sampling_equals_the_allocating_entry_point():
    from spite_b200.kernels import build
    from spite_b200.kernels.cuda import CudaKernels

    dev = "cuda:0"
    torch.cuda.set_device(0)
    lib = build.load("sampling")
    fn = lib.spite_sample_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(NoAllocArgs), C.c_void_p]
    ks = CudaKernels(torch.float32, dev)

    R = 6
    cases = [dict(temperature=0.0), dict(temperature=0.7), dict(temperature=1.0, top_k=7),
             dict(temperature=0.9, top_p=0.8), dict(temperature=1.2, min_p=0.02, repetition_penalty=1.3),
             dict(temperature=1.0, top_k=50, top_p=0.95, repetition_penalty=1.1)]
    col = lambda key, default, dt: torch.tensor([c.get(key, default) for c in cases], dtype=dt, device=dev)
    temperature, top_k = col("temperature", 0.0, torch.float32), col("top_k", 0, torch.int32)
    top_p, min_p = col("top_p", 1.0, torch.float32), col("min_p", 0.0, torch.float32)
    penalty = col("repetition_penalty", 1.0, torch.float32)
    state = torch.tensor([99 + r for r in range(R)], dtype=torch.int64, device=dev)

    # two calls in a row with different vocabularies: the second, smaller one runs on
    # scratch that still holds the first one's rows
    for call, V in enumerate((50000, 1000)):
        g = torch.Generator().manual_seed(call)
        logits = (torch.randn((R, V), generator=g) * 2.0).to(dev)
        context = torch.randint(0, V, (R * 16,), generator=g, dtype=torch.int32).to(dev)
        offsets = torch.arange(0, R * 16 + 1, 16, dtype=torch.int32, device=dev)

        state_a = state.clone()
        want = ks.sample(logits, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                         repetition_penalty=penalty, context=context, context_offsets=offsets,
                         rng_state=state_a)

        state_b = state.clone()
        got = torch.full((R,), -1, dtype=torch.int32, device=dev)
        args = NoAllocArgs(logits=logits.data_ptr(), temperature=temperature.data_ptr(), top_k=top_k.data_ptr(),
                           top_p=top_p.data_ptr(), min_p=min_p.data_ptr(), repetition_penalty=penalty.data_ptr(),
                           context=context.data_ptr(), context_offsets=offsets.data_ptr(),
                           rng_state=state_b.data_ptr(), out_tokens=got.data_ptr(), rows=R, vocab=V)
        reserved_before = torch.cuda.memory_reserved()
        status = fn(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert status == 0
        assert torch.cuda.memory_reserved() == reserved_before       # nothing came from torch's allocator
        assert got.tolist() == want.tolist(), f"call {call}"
        assert state_b.tolist() == state_a.tolist(), f"call {call}: generator states differ"
        state = state_a

    # a request beyond the fixed scratch is refused and writes nothing
    rows, vocab = 3, MAX_FLOATS // 3 + 1
    got = torch.full((rows,), -7, dtype=torch.int32, device=dev)
    small = torch.zeros(8, device=dev)
    args = NoAllocArgs(logits=small.data_ptr(), temperature=small.data_ptr(), top_k=None, top_p=None, min_p=None,
                       repetition_penalty=None, context=None, context_offsets=None,
                       rng_state=state.data_ptr(), out_tokens=got.data_ptr(), rows=rows, vocab=vocab)
    assert fn(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream)) == -2
    torch.cuda.synchronize()
    assert got.tolist() == [-7] * rows
    args.rows, args.vocab = 2, 0
    assert fn(C.byref(args), None) == -1
