"""The contract of the exported C entry points (spite_b200/csrc/common.cuh, after giveen/spite's
core/abi.h:218,365 and tools/verify/verify.py:1974-2059): a malformed call (null pointer, size that
makes no sense) returns -1, a size outside a kernel's domain returns -2, and in both cases nothing
is launched: outputs filled with a canary value keep it.  And the bounded waits: a wait that runs
out makes the kernel return with an error code that the engine turns into `KernelTimeout`, after
which the next call is right."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
CANARY = 96.5          # exact in bfloat16
BAD_ARG, UNSUPPORTED = -1, -2


@pytest.fixture(scope="module")
def libs():
    from spite_b200.kernels import build
    build.ensure_built()
    return {name: build.load(name) for name in build.LIBRARIES}


def canary(shape, dtype=torch.float32):
    return torch.full(shape, CANARY, dtype=dtype, device=DEV)


def untouched(*tensors):
    torch.cuda.synchronize()
    return all(bool((t == (CANARY if t.is_floating_point() else int(CANARY))).all()) for t in tensors)


def ptr(t):
    return C.c_void_p(None if t is None else t.data_ptr())


# ---------------------------------------------------------------------------- products
def gemm_case(M=4, N=64, K=128, dtype=torch.bfloat16):
    from spite_b200.kernels.cuda import GemmParams
    a = torch.ones((max(M, 1), K), dtype=dtype, device=DEV)
    w = torch.ones((N, K), dtype=dtype, device=DEV)
    c = canary((max(M, 1), N), dtype)
    p = GemmParams(A=a.data_ptr(), W=w.data_ptr(), C=c.data_ptr(), a_rows=None, c_rows=None, group_offsets=None,
                   row_scale=None, lda=K, ldc=N, w_group_stride=0, n_groups=1, M=M, N=N, K=K, epilogue=0,
                   scale_by_a_row=0)
    return p, (a, w, c)


def gemm_calls(libs):
    """(name, call(params) -> status) for every product entry point."""
    scratch = torch.zeros(1 << 16, dtype=torch.float32, device=DEV)
    tickets = torch.zeros(1024, dtype=torch.int32, device=DEV)
    return [
        ("gemm_simt", lambda p: libs["gemm_simt"].spite_gemm_simt(1, C.byref(p), None)),
        ("gemm_skinny", lambda p: libs["gemm_skinny"].spite_gemm_skinny(C.byref(p), max(p.M, 1), 148, None)),
        ("gemm_stream", lambda p: libs["gemm_stream"].spite_gemm_stream(
            C.byref(p), min(max(p.M, 1), 16), 1, 0, 296, 74 * 1024, 1, ptr(scratch), C.c_longlong(scratch.numel()),
            ptr(tickets), tickets.numel(), None)),
        ("gemm_tc", lambda p: libs["gemm_tc"].spite_gemm_tc(C.byref(p), 148, None)),
        ("gemm_tc_pair", lambda p: libs["gemm_tc_pair"].spite_gemm_tc_pair(C.byref(p), 74, None)),
    ]


def test_the_experts_product_refuses_malformed_calls(libs):
    lib = libs["gemm_tc_experts"]
    offsets = torch.tensor([0, 2, 4], dtype=torch.int32, device=DEV)

    def case(**kw):
        p, keep = gemm_case(M=4, N=64, K=128)
        p.group_offsets, p.n_groups, p.epilogue, p.w_group_stride = offsets.data_ptr(), 2, 2, 64 * 128
        p.C = canary((4, 64)).data_ptr()
        for k, v in kw.items():
            setattr(p, k, v)
        return p, keep
    for kw, want in ((dict(A=None), BAD_ARG), (dict(W=None), BAD_ARG), (dict(C=None), BAD_ARG), (dict(group_offsets=None), BAD_ARG),
                     (dict(n_groups=0), BAD_ARG), (dict(N=0), BAD_ARG), (dict(K=0), BAD_ARG), (dict(lda=8), BAD_ARG),
                     (dict(epilogue=7), BAD_ARG), (dict(epilogue=0), UNSUPPORTED), (dict(K=100, lda=100), UNSUPPORTED),
                     (dict(w_group_stride=5), UNSUPPORTED), (dict(n_groups=4000), UNSUPPORTED)):
        p, keep = case(**kw)
        assert lib.spite_gemm_tc_experts(C.byref(p), 148, None) == want, kw
    assert lib.spite_gemm_tc_experts(None, 148, None) == BAD_ARG
    p, keep = case()
    assert lib.spite_gemm_tc_experts(C.byref(p), 0, None) == BAD_ARG


@pytest.mark.parametrize("which", range(5))
def test_products_refuse_malformed_calls(libs, which):
    name, call = gemm_calls(libs)[which]
    for field in ("A", "W", "C"):
        p, (a, w, c) = gemm_case()
        setattr(p, field, None)
        assert call(p) == BAD_ARG, f"{name}: null {field}"
        assert untouched(c), f"{name}: wrote although {field} was null"
    for field, value in (("N", 0), ("K", 0), ("M", -1), ("lda", 64), ("ldc", 8), ("n_groups", 0), ("epilogue", 9)):
        p, (a, w, c) = gemm_case()
        setattr(p, field, value)
        assert call(p) == BAD_ARG, f"{name}: {field} = {value}"
        assert untouched(c), f"{name}: wrote although {field} = {value}"
    # a null parameter block
    fn = {"gemm_simt": lambda: libs["gemm_simt"].spite_gemm_simt(1, None, None),
          "gemm_skinny": lambda: libs["gemm_skinny"].spite_gemm_skinny(None, 1, 148, None),
          "gemm_stream": lambda: libs["gemm_stream"].spite_gemm_stream(None, 1, 1, 0, 296, 74 * 1024, 1, None, C.c_longlong(0), None, 0, None),
          "gemm_tc": lambda: libs["gemm_tc"].spite_gemm_tc(None, 148, None),
          "gemm_tc_pair": lambda: libs["gemm_tc_pair"].spite_gemm_tc_pair(None, 74, None)}[name]
    assert fn() == BAD_ARG
    # zero rows: nothing to do, nothing written, status 0
    p, (a, w, c) = gemm_case(M=0)
    assert call(p) == 0 and untouched(c), name


@pytest.mark.parametrize("which", [1, 2, 3, 4])
def test_tensor_core_products_refuse_sizes_outside_their_domain(libs, which):
    """K = 100 is no multiple of 8 (16-byte rows for TMA and vector loads): -2, and the general kernel takes it."""
    name, call = gemm_calls(libs)[which]
    p, (a, w, c) = gemm_case(M=4, N=64, K=100)
    assert call(p) == UNSUPPORTED, name
    assert untouched(c), name
    p, (a, w, c) = gemm_case(M=4, N=64, K=128)
    p.A = a.data_ptr() + 2                                   # a misaligned base
    assert call(p) == UNSUPPORTED, name
    assert untouched(c), name
    assert libs["gemm_simt"].spite_gemm_simt(1, C.byref(gemm_case(M=4, N=64, K=100)[0]), None) == 0


def test_streaming_product_refuses_too_many_rows_and_missing_scratch(libs):
    p, (a, w, c) = gemm_case(M=4, N=64, K=4096)
    lib = libs["gemm_stream"]
    assert lib.spite_gemm_stream(C.byref(p), 33, 1, 0, 296, 74 * 1024, 1, None, C.c_longlong(0), None, 0, None) == UNSUPPORTED
    assert lib.spite_gemm_stream(C.byref(p), 4, 1, 0, 296, 74 * 1024, 4, None, C.c_longlong(0), None, 0, None) == BAD_ARG
    assert lib.spite_gemm_stream(C.byref(p), 4, 1, 0, 0, 74 * 1024, 1, None, C.c_longlong(0), None, 0, None) == BAD_ARG
    assert lib.spite_gemm_stream(C.byref(p), 4, 3, 0, 296, 74 * 1024, 1, None, C.c_longlong(0), None, 0, None) == BAD_ARG       # k slices: 1, 2, 4, 8
    assert untouched(c)
    p, (a, w, c) = gemm_case(M=4, N=64, K=320)                                     # 320 is no multiple of 64 x 2
    assert lib.spite_gemm_stream(C.byref(p), 4, 2, 0, 296, 74 * 1024, 1, None, C.c_longlong(0), None, 0, None) == UNSUPPORTED
    assert untouched(c)
    p, (a, w, c) = gemm_case(M=600, N=64, K=128)
    assert libs["gemm_skinny"].spite_gemm_skinny(C.byref(p), 600, 148, None) == UNSUPPORTED and untouched(c)


# ---------------------------------------------------------------------------- elementwise, router, sampling
def test_elementwise_entry_points(libs):
    lib = libs["elementwise"]
    table = torch.ones((10, 16), dtype=torch.bfloat16, device=DEV)
    toks = torch.zeros(4, dtype=torch.int32, device=DEV)
    h = canary((4, 16))
    for args in ((1, None, ptr(toks), ptr(h), 4, 16, 10, C.c_float(1.0)), (1, ptr(table), None, ptr(h), 4, 16, 10, C.c_float(1.0)),
                 (1, ptr(table), ptr(toks), None, 4, 16, 10, C.c_float(1.0)), (1, ptr(table), ptr(toks), ptr(h), -1, 16, 10, C.c_float(1.0)),
                 (1, ptr(table), ptr(toks), ptr(h), 4, 0, 10, C.c_float(1.0)), (1, ptr(table), ptr(toks), ptr(h), 4, 16, 0, C.c_float(1.0)),
                 (7, ptr(table), ptr(toks), ptr(h), 4, 16, 10, C.c_float(1.0))):
        assert lib.spite_embed(*args, None) == BAD_ARG, args
    assert untouched(h)
    x = torch.ones((4, 16), dtype=torch.float32, device=DEV)
    gain = torch.ones(16, dtype=torch.float32, device=DEV)
    y = canary((4, 16))
    for args in ((0, None, ptr(gain), None, ptr(y), 4, 16, C.c_float(1e-5)), (0, ptr(x), None, None, ptr(y), 4, 16, C.c_float(1e-5)),
                 (0, ptr(x), ptr(gain), None, None, 4, 16, C.c_float(1e-5)), (0, ptr(x), ptr(gain), None, ptr(y), -2, 16, C.c_float(1e-5)),
                 (0, ptr(x), ptr(gain), None, ptr(y), 4, 0, C.c_float(1e-5)), (0, ptr(x), ptr(gain), None, ptr(y), 4, 16, C.c_float(0.0)),
                 (5, ptr(x), ptr(gain), None, ptr(y), 4, 16, C.c_float(1e-5))):
        assert lib.spite_rms_norm(*args, None) == BAD_ARG, args
    assert untouched(y)
    src = torch.ones((4, 16), dtype=torch.bfloat16, device=DEV)
    dst = canary((4, 16), torch.bfloat16)
    idx = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert lib.spite_gather_rows(None, ptr(idx), ptr(dst), 4, C.c_longlong(32), None) == BAD_ARG
    assert lib.spite_gather_rows(ptr(src), ptr(idx), ptr(dst), 4, C.c_longlong(0), None) == BAD_ARG
    assert lib.spite_gather_rows(ptr(src), ptr(idx), ptr(dst), 4, C.c_longlong(20), None) == UNSUPPORTED
    assert untouched(dst)


def test_router_entry_point(libs):
    lib = libs["moe"]
    M, d, E = 4, 32, 6
    x = torch.ones((M, d), dtype=torch.bfloat16, device=DEV)
    w = torch.ones((E, d), dtype=torch.float32, device=DEV)
    ids, rows = canary((1, M), torch.int32), canary((1, M), torch.int32)
    wts, logits, offs = canary((1, M)), canary((M, E)), canary((1, E + 1), torch.int32)

    def call(**kw):
        a = dict(x=ptr(x), w=ptr(w), M=M, d=d, E=E, k=1, ids=ptr(ids), wts=ptr(wts), logits=ptr(logits),
                 offs=ptr(offs), rows=ptr(rows))
        a.update(kw)
        return lib.spite_moe_route(1, a["x"], a["w"], a["M"], a["d"], a["E"], a["k"], a["ids"], a["wts"],
                                   a["logits"], a["offs"], a["rows"], None)
    for kw in (dict(x=None), dict(w=None), dict(ids=None), dict(wts=None), dict(offs=None), dict(rows=None),
               dict(M=-1), dict(d=0), dict(E=0), dict(k=0), dict(k=E + 1)):
        assert call(**kw) == BAD_ARG, kw
    assert call(E=5000) == UNSUPPORTED
    assert untouched(ids, rows, wts, logits, offs)


def test_sampling_entry_points(libs):
    from spite_b200.kernels.cuda import SampleParams
    lib = libs["sampling"]
    R, V = 2, 50
    logits = torch.zeros((R, V), dtype=torch.float32, device=DEV)
    out = canary((R,), torch.int32)
    assert lib.spite_argmax(None, R, V, ptr(out), None) == BAD_ARG
    assert lib.spite_argmax(ptr(logits), R, V, None, None) == BAD_ARG
    assert lib.spite_argmax(ptr(logits), -1, V, ptr(out), None) == BAD_ARG
    assert lib.spite_argmax(ptr(logits), R, 0, ptr(out), None) == BAD_ARG
    work = canary((R, V))
    temp = torch.ones(R, dtype=torch.float32, device=DEV)
    rng = torch.zeros(R, dtype=torch.int64, device=DEV)
    ctx = torch.zeros(4, dtype=torch.int32, device=DEV)

    def params(**kw):
        a = dict(logits=logits.data_ptr(), work=work.data_ptr(), temperature=temp.data_ptr(), top_k=None, top_p=None,
                 min_p=None, repetition_penalty=None, context=None, context_offsets=None,
                 rng_state=rng.data_ptr(), out_tokens=out.data_ptr(), vocab=V)
        a.update(kw)
        return SampleParams(**a)
    for kw in (dict(logits=None), dict(work=None), dict(temperature=None), dict(rng_state=None), dict(out_tokens=None),
               dict(vocab=0), dict(context=ctx.data_ptr())):
        assert lib.spite_sample(C.byref(params(**kw)), R, None) == BAD_ARG, kw
    assert lib.spite_sample(None, R, None) == BAD_ARG
    assert lib.spite_sample(C.byref(params()), -1, None) == BAD_ARG
    assert untouched(out, work) and int(rng.abs().sum()) == 0


# ---------------------------------------------------------------------------- attention
def attention_case(hd=64, nq=4, nkv=2, page=64, M=3):
    from spite_b200.kernels.cuda import (AttentionParams, AttnDecodeExtra, AttnMmaExtra, PagedCache, QkPrepareParams,
                                         StepTokens)
    kv = torch.zeros((2, 4, nkv, page, hd), dtype=torch.bfloat16, device=DEV)
    q = torch.ones((M, nq * hd), dtype=torch.bfloat16, device=DEV)
    qkv = torch.ones((M, (nq + 2 * nkv) * hd), dtype=torch.bfloat16, device=DEV)
    out = canary((M, nq * hd), torch.bfloat16)
    pos = torch.arange(M, dtype=torch.int32, device=DEV)
    seg = torch.zeros(M, dtype=torch.int32, device=DEV)
    table = torch.zeros((1, 4), dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, M], dtype=torch.int32, device=DEV)
    keep = (kv, q, qkv, out, pos, seg, table, cu)
    b = StepTokens(positions=pos.data_ptr(), seg_of_token=seg.data_ptr(), block_table=table.data_ptr(),
                   table_width=4, n_tokens=M)
    c = PagedCache(kv=kv.data_ptr(), v_offset=kv.stride(0), n_pages=4, page_size=page, num_kv_heads=nkv, head_dim=hd)
    p = AttentionParams(q=q.data_ptr(), out=out.data_ptr(), num_heads=nq, window_kind=0, window_size=0,
                        softmax_scale=0.125)
    x = AttnMmaExtra(cu_seqlens=cu.data_ptr(), o_part=None, ml_part=None, n_segments=1, tokens_per_block=1,
                     n_splits=1, seg_min_tokens=0, seg_max_tokens=1 << 30)
    xd = AttnDecodeExtra(cu_seqlens=cu.data_ptr(), partial=None, tickets=None, n_segments=1, tokens_per_block=1,
                         n_splits=1, seg_min_tokens=0, seg_max_tokens=1 << 30, cache_settled=0)
    qp = QkPrepareParams(qkv=qkv.data_ptr(), q_out=out.data_ptr(), inv_freq=None, qk_norm_eps=0.0,
                         temperature_floor=0, temperature_scale=0.0, num_heads=nq, write_cache=1)
    return dict(p=p, b=b, c=c, x=x, xd=xd, qp=qp, out=out, kv=kv, keep=keep)


def attention_calls(libs):
    return [
        ("attention", lambda k: libs["attention"].spite_paged_attention(1, C.byref(k["p"]), C.byref(k["b"]), C.byref(k["c"]), None)),
        ("attention_mma", lambda k: libs["attention_mma"].spite_paged_attention_mma(
            C.byref(k["p"]), C.byref(k["b"]), C.byref(k["c"]), C.byref(k["x"]), 3, None)),
        ("attention_rows", lambda k: libs["attention_rows"].spite_paged_attention_rows(
            C.byref(k["p"]), C.byref(k["b"]), C.byref(k["c"]), C.byref(k["x"]), 1, None)),
        ("attention_tc", lambda k: libs["attention_tc"].spite_paged_attention_tc(
            C.byref(k["p"]), C.byref(k["b"]), C.byref(k["c"]), C.byref(k["x"]), 1, 148, None)),
        ("attention_decode", lambda k: libs["attention_decode"].spite_paged_attention_decode(
            C.byref(k["p"]), C.byref(k["b"]), C.byref(k["c"]), C.byref(k["xd"]), 3, 3, None)),
    ]


@pytest.mark.parametrize("which", range(5))
def test_attention_refuses_malformed_calls(libs, which):
    name, call = attention_calls(libs)[which]
    edits = [("p", "q", None), ("p", "out", None), ("b", "positions", None), ("b", "block_table", None),
             ("c", "kv", None), ("p", "num_heads", 0), ("p", "num_heads", 3), ("p", "window_kind", 5),
             ("b", "table_width", 0), ("b", "n_tokens", -1)]
    if name == "attention_decode":
        edits += [("xd", "cu_seqlens", None), ("xd", "n_segments", 0), ("xd", "tokens_per_block", 0), ("xd", "n_splits", 4)]
    elif name != "attention":
        edits += [("x", "cu_seqlens", None), ("x", "n_segments", 0), ("x", "tokens_per_block", 0)]
    for struct, field, value in edits:
        k = attention_case()
        setattr(k[struct], field, value)
        assert call(k) == BAD_ARG, f"{name}: {struct}.{field} = {value}"
        assert untouched(k["out"]), f"{name}: wrote although {struct}.{field} = {value}"
    k = attention_case()
    k["p"].window_kind, k["p"].window_size = 1, 0                        # a chunk window of no keys
    assert call(k) == BAD_ARG and untouched(k["out"]), name


def test_attention_refuses_sizes_outside_its_domain(libs):
    calls = dict(attention_calls(libs))
    k = attention_case(hd=24)                                          # head size that is no multiple of 16
    for name in ("attention_mma", "attention_rows", "attention_tc", "attention_decode"):
        assert calls[name](k) == UNSUPPORTED and untouched(k["out"]), name
    k = attention_case(hd=32)                                          # the TMA-fed kernels take 64 and 128 only
    for name in ("attention_tc", "attention_decode"):
        assert calls[name](k) == UNSUPPORTED and untouched(k["out"]), name
    k = attention_case(hd=64, page=16)                                 # and pages of a multiple of 64 keys
    for name in ("attention_tc", "attention_decode"):
        assert calls[name](k) == UNSUPPORTED and untouched(k["out"]), name
    k = attention_case(hd=64, nq=34, nkv=2)                            # 17 query heads on a kv head
    for name in ("attention_mma", "attention_rows", "attention_decode"):
        assert calls[name](k) == UNSUPPORTED and untouched(k["out"]), name
    k = attention_case(hd=258)                                         # beyond the general kernel's 256
    assert calls["attention"](k) == UNSUPPORTED and untouched(k["out"])


def test_prepare_refuses_malformed_calls(libs):
    lib = libs["attention"]
    for struct, field, value in (("qp", "qkv", None), ("qp", "q_out", None), ("b", "positions", None),
                                 ("b", "block_table", None), ("c", "kv", None), ("qp", "num_heads", 0)):
        k = attention_case()
        setattr(k[struct], field, value)
        assert lib.spite_qk_prepare(1, C.byref(k["qp"]), C.byref(k["b"]), C.byref(k["c"]), None) == BAD_ARG, (struct, field)
        torch.cuda.synchronize()
        assert untouched(k["out"]) and float(k["kv"].float().abs().sum()) == 0.0
    k = attention_case()
    assert lib.spite_qk_prepare(9, C.byref(k["qp"]), C.byref(k["b"]), C.byref(k["c"]), None) == BAD_ARG
    assert lib.spite_qk_prepare(1, None, C.byref(k["b"]), C.byref(k["c"]), None) == BAD_ARG
    assert untouched(k["out"])


# ---------------------------------------------------------------------------- a wait that runs out
def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_right():
    """The tcgen05 product is told (by its test-only launch argument) that its first stage brings 16 bytes
    more than its copies deliver, and given waits of a few milliseconds: the barrier of that stage never
    completes, the issuing thread's wait runs out, every role of the block leaves through the common exit,
    and the error word says so.  Nothing faults or spins without a limit.  Through the engine the same
    word becomes `KernelTimeout`.  With the defaults back, the same product is right."""
    from spite_b200.engine import Engine, KernelTimeout
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    g = torch.Generator().manual_seed(0)
    x = (torch.randn((256, 512), generator=g)).to(torch.bfloat16).to(DEV)
    w = (torch.randn((384, 512), generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    ref = x.float() @ w.float().T
    out = torch.zeros((256, 384), dtype=torch.bfloat16, device=DEV)
    ks.tc_pair_min_rows = 1 << 30                         # this product on one block a tile (`gemm_tc`)
    assert ks.errors() == {}
    ks.configure_waits("gemm_tc", limit_cycles=4_000_000, extra_tx=16)     # about two milliseconds
    try:
        before = ks.launches_by_library["gemm_tc"]
        ks.linear(x, w, out)
        assert ks.launches_by_library["gemm_tc"] == before + 1
        torch.cuda.synchronize()
    finally:
        ks.configure_waits("gemm_tc")
    errors = ks.errors()
    assert errors.get("gemm_tc") in (1, 2, 3, 4), errors
    assert ks.errors() == {}                              # reading cleared it

    class OneKernelSet:                                   # what `Engine.check` needs of a model
        kernels = ks
    eng = Engine.__new__(Engine)
    eng.model = OneKernelSet()
    ks.configure_waits("gemm_tc", limit_cycles=4_000_000, extra_tx=16)
    try:
        ks.linear(x, w, out)
        torch.cuda.synchronize()
    finally:
        ks.configure_waits("gemm_tc")
    with pytest.raises(KernelTimeout, match="gemm_tc"):
        eng.check()
    eng.check()                                           # reported once
    out.zero_()
    ks.linear(x, w, out)
    torch.cuda.synchronize()
    assert ks.errors() == {}
    err = float((out.float() - ref).abs().max()) / float(ref.abs().max())
    assert err <= 1.2e-2, err
