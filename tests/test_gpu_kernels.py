"""Each CUDA kernel alone against its plain torch restatement (float64 sums),
at sizes other than the engine tests': widths and vocabularies that are no power
of two, head sizes in steps of 16, odd numbers of heads and groups, empty
experts, pages used out of order.  Inputs are built so that a fault shows: one
far key among hundreds carries the attention, windows end inside pages."""
import math

import pytest
import torch

from reference_kernels import TorchReferenceKernels
from spite_b200.cache import LayerCache, Window
from spite_b200.engine.batch import Segment, build_step_batch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 1.2e-2}


@pytest.fixture(scope="module", params=DTYPES, ids=["f32", "bf16"])
def ks(request):
    from spite_b200.kernels.cuda import CudaKernels
    return CudaKernels(request.param, DEV)


def ref_set(dtype):
    return TorchReferenceKernels(dtype, "cpu", acc=torch.float64)


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(out, ref, tol, what=""):
    out, ref = out.detach().cpu().double(), ref.detach().cpu().double()
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    err = float((out - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
    assert err <= tol, f"{what}: error {err:.3e} of the output scale exceeds {tol:.1e}"


# ---------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("V,d,M", [(37, 48, 5), (1000, 200, 33)])
def test_embed(ks, V, d, M):
    table = rnd((V, d), ks.dtype, 1)
    toks = torch.randint(0, V, (M,), dtype=torch.int32)
    toks[0], toks[-1] = 0, V - 1
    out = torch.full((M, d), 7.0, dtype=torch.float32, device=DEV)
    ks.embed(table.to(DEV), toks.to(DEV), out)
    assert torch.equal(out.cpu(), table[toks.long()].float())


@pytest.mark.parametrize("M,d,eps", [(7, 48, 1e-5), (3, 5120, 1e-6), (19, 200, 1e-2)])
def test_rms_norm(ks, M, d, eps):
    h = rnd((M, d), torch.float32, 2, 3.0)
    gain = rnd((d,), torch.float32, 3) + 1.0
    out = torch.empty((M, d), dtype=ks.dtype, device=DEV)
    ks.rms_norm(h.to(DEV), gain.to(DEV), eps, out)
    ref = torch.empty((M, d), dtype=torch.float64)
    ref_set(ks.dtype).rms_norm(h, gain, eps, ref)
    close(out, ref, TOL[ks.dtype], "rms_norm")
    rows = torch.tensor([M - 1, 0, M // 2], dtype=torch.int32)
    out2 = torch.empty((3, d), dtype=ks.dtype, device=DEV)
    ks.rms_norm(h.to(DEV), gain.to(DEV), eps, out2, rows.to(DEV))
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])


# ---------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K", [(1, 40, 48), (5, 1000, 96), (130, 72, 200), (64, 64, 64), (67, 129, 33),
                                   (8, 200, 5120), (64, 96, 2048), (33, 50, 64), (17, 33, 128), (2, 31, 32),
                                   (128, 128, 64), (256, 384, 512), (300, 200, 136), (1000, 520, 1024), (515, 7168, 192), (2048, 264, 320),
                                   (3, 129, 8192), (16, 300, 4096), (1, 40, 64), (9, 1000, 2048)])
def test_linear(ks, M, N, K):
    x, w = rnd((M, K), ks.dtype, 4), rnd((N, K), ks.dtype, 5, 0.2)
    r = ref_set(ks.dtype)
    out = torch.empty((M, N), dtype=ks.dtype, device=DEV)
    streamed = ks.launches_by_library["gemm_stream"]
    ks.linear(x.to(DEV), w.to(DEV), out)
    if ks.dtype == torch.bfloat16 and M <= 16 and K % 64 == 0:
        assert ks.launches_by_library["gemm_stream"] == streamed + 1     # the TMA weight-streaming kernel took it
    ref = torch.empty((M, N), dtype=torch.float64)
    r.linear(x, w, ref)
    close(out, ref, TOL[ks.dtype], "linear")
    # float32 output (logits) and accumulation into the residual stream with a row scale
    out32 = torch.empty((M, N), dtype=torch.float32, device=DEV)
    ks.linear(x.to(DEV), w.to(DEV), out32)
    close(out32, ref, 1e-5 if ks.dtype == torch.float32 else 1e-5 * K, "linear f32 out")
    h = rnd((M, N), torch.float32, 6)
    scale = rnd((M,), torch.float32, 7)
    hd = h.to(DEV).clone()
    ks.linear(x.to(DEV), w.to(DEV), hd, accumulate=True, row_scale=scale.to(DEV))
    ref_h = h.double().clone()
    r.linear(x, w, ref_h, accumulate=True, row_scale=scale)
    close(hd, ref_h, 2e-5, "linear accumulate")
    if hasattr(ks, "gemm_tc_error"):
        assert ks.gemm_tc_error() == 0, "a tensor-core block gave up waiting"


@pytest.mark.parametrize("slices,splits,cluster", [(1, 1, False), (1, 3, False), (2, 1, False), (2, 2, False), (4, 1, False),
                                                   (4, 2, False), (8, 1, False), (8, 2, False),
                                                   (1, 2, True), (1, 3, True), (1, 4, True)])
@pytest.mark.parametrize("M", [1, 7, 13])
def test_streaming_products_with_k_slices_and_k_splits(slices, splits, cluster, M):
    """The weight-streaming kernel with every way of cutting its work: tiles of 128 / slices rows whose k slices
    meet in shared memory, and k splits across blocks, through the scratch in global memory or, as one thread-block
    cluster a tile, through shared memory; plain, SwiGLU, added into float32 with a row scale, and grouped by
    expert.  Widths that are no multiple of a tile; the same bits twice."""
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    ks.stream_force = (slices, splits)
    ks.stream_cluster_max_rows = 16 if cluster else 0
    if M > 8 and slices == 8:
        ks.stream_shape = [ks.stream_shape[0]] * 2            # stages of 16 tokens x 8 slices are 32 KiB: the deeper ring
    r = ref_set(torch.bfloat16)
    N, K, F, E = 200, 1024, 104, 5                            # 1024 = 2 stages of 8 slices
    x, w = rnd((M, K), torch.bfloat16, 4), rnd((N, K), torch.bfloat16, 5, 0.2)
    before = ks.launches_by_library["gemm_stream"]
    outs = []
    for _ in range(2):
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
        ks.linear(x.to(DEV), w.to(DEV), out)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    ref = torch.empty((M, N), dtype=torch.float64)
    r.linear(x, w, ref)
    close(outs[0], ref, TOL[torch.bfloat16], "linear")
    h, scale = rnd((M, N), torch.float32, 6), rnd((M,), torch.float32, 7)
    hd = h.to(DEV).clone()
    ks.linear(x.to(DEV), w.to(DEV), hd, accumulate=True, row_scale=scale.to(DEV))
    ref_h = h.double().clone()
    r.linear(x, w, ref_h, accumulate=True, row_scale=scale)
    close(hd, ref_h, 2e-5, "linear accumulate")
    logits = torch.empty((M, N), dtype=torch.float32, device=DEV)
    ks.linear(x.to(DEV), w.to(DEV), logits)
    close(logits, ref, 1e-5 * K, "linear f32 out")
    launches = 4
    if slices < 8:                                            # SwiGLU tiles of 8 gate and 8 up rows are not built
        wg = rnd((2 * F, K), torch.bfloat16, 9, 0.3)
        a = torch.empty((M, F), dtype=torch.bfloat16, device=DEV)
        ks.linear_swiglu(x.to(DEV), wg.to(DEV), a, row_scale=(scale.abs() + 0.5).to(DEV))
        a_ref = torch.empty((M, F), dtype=torch.float64)
        r.linear_swiglu(x, wg, a_ref, row_scale=scale.abs() + 0.5)
        close(a, a_ref, TOL[torch.bfloat16], "linear_swiglu")
        launches += 1
    # grouped: expert 1 stays empty
    g = torch.Generator().manual_seed(10 + M)
    ids = torch.randint(0, E, (M,), generator=g)
    ids[ids == 1] = 0
    order = torch.sort(ids, stable=True)
    rows = order.indices.to(torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(torch.bincount(ids, minlength=E), 0)
    w_gu, w_d = rnd((E, 2 * F, K), torch.bfloat16, 12, 0.3), rnd((E, K, 128), torch.bfloat16, 13, 0.3)
    tok_scale = torch.rand(M, generator=g) + 0.5
    if slices < 8:
        a = torch.zeros((M, F), dtype=torch.bfloat16, device=DEV)
        ks.grouped_linear_swiglu(x.to(DEV), w_gu.to(DEV), rows.to(DEV), offsets.to(DEV), tok_scale.to(DEV), a)
        a_ref = torch.zeros((M, F), dtype=torch.float64)
        r.grouped_linear_swiglu(x, w_gu, rows, offsets, tok_scale, a_ref)
        close(a, a_ref, TOL[torch.bfloat16], "grouped_linear_swiglu")
        launches += 1
    if 128 % (64 * slices) == 0:                              # the down product's depth here is 128
        a2 = rnd((M, 128), torch.bfloat16, 15)
        h2 = rnd((M, K), torch.float32, 14)
        hd2 = h2.to(DEV).clone()
        ks.grouped_linear_accumulate(a2.to(DEV), w_d.to(DEV), rows.to(DEV), offsets.to(DEV), hd2)
        h2_ref = h2.double().clone()
        r.grouped_linear_accumulate(a2, w_d, rows, offsets, h2_ref)
        close(hd2, h2_ref, 2e-3, "grouped_linear_accumulate")
        launches += 1
    assert ks.launches_by_library["gemm_stream"] == before + launches       # every one of them ran in that kernel
    assert ks.errors() == {}


@pytest.mark.parametrize("slices,splits", [(1, 1), (1, 3), (2, 1), (2, 2)])
@pytest.mark.parametrize("M", [17, 25, 32])
def test_streaming_products_of_up_to_32_rows(slices, splits, M):
    """One-group products of 17 to 32 rows (the dense projections of a larger decode batch) stream their weights
    too, with 32 token columns a tile: plain, SwiGLU with a row scale, float32 out, added into float32."""
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    ks.stream_force = (slices, splits)
    r = ref_set(torch.bfloat16)
    N, K, F = 200, 1024, 104
    x, w = rnd((M, K), torch.bfloat16, 4), rnd((N, K), torch.bfloat16, 5, 0.2)
    before = ks.launches_by_library["gemm_stream"]
    outs = []
    for _ in range(2):
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
        ks.linear(x.to(DEV), w.to(DEV), out)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    ref = torch.empty((M, N), dtype=torch.float64)
    r.linear(x, w, ref)
    close(outs[0], ref, TOL[torch.bfloat16], "linear")
    h, scale = rnd((M, N), torch.float32, 6), rnd((M,), torch.float32, 7)
    hd = h.to(DEV).clone()
    ks.linear(x.to(DEV), w.to(DEV), hd, accumulate=True, row_scale=scale.to(DEV))
    ref_h = h.double().clone()
    r.linear(x, w, ref_h, accumulate=True, row_scale=scale)
    close(hd, ref_h, 2e-5, "linear accumulate")
    logits = torch.empty((M, N), dtype=torch.float32, device=DEV)
    ks.linear(x.to(DEV), w.to(DEV), logits)
    close(logits, ref, 1e-5 * K, "linear f32 out")
    wg = rnd((2 * F, K), torch.bfloat16, 9, 0.3)
    a = torch.empty((M, F), dtype=torch.bfloat16, device=DEV)
    ks.linear_swiglu(x.to(DEV), wg.to(DEV), a, row_scale=(scale.abs() + 0.5).to(DEV))
    a_ref = torch.empty((M, F), dtype=torch.float64)
    r.linear_swiglu(x, wg, a_ref, row_scale=scale.abs() + 0.5)
    close(a, a_ref, TOL[torch.bfloat16], "linear_swiglu")
    assert ks.launches_by_library["gemm_stream"] == before + 5 and ks.errors() == {}


@pytest.mark.parametrize("M,F,K", [(3, 24, 48), (70, 100, 96), (8, 40, 512), (40, 17, 96), (64, 72, 64), (129, 256, 192), (700, 136, 320), (1100, 1000, 128),
                                   (5, 100, 4096), (16, 72, 6144), (12, 200, 128)])
def test_linear_swiglu(ks, M, F, K):
    x, w = rnd((M, K), ks.dtype, 8), rnd((2 * F, K), ks.dtype, 9, 0.3)
    scale = torch.rand(M) + 0.5
    out = torch.empty((M, F), dtype=ks.dtype, device=DEV)
    ks.linear_swiglu(x.to(DEV), w.to(DEV), out, row_scale=scale.to(DEV))
    ref = torch.empty((M, F), dtype=torch.float64)
    ref_set(ks.dtype).linear_swiglu(x, w, ref, row_scale=scale)
    close(out, ref, TOL[ks.dtype], "linear_swiglu")


@pytest.mark.parametrize("M,E,F,K", [(1, 3, 24, 48), (9, 5, 40, 96), (150, 7, 72, 64), (64, 16, 48, 128),
                                     (60, 3, 24, 64), (8, 128, 16, 32), (1500, 16, 160, 256), (300, 4, 128, 72),
                                     (7, 5, 40, 4096), (16, 9, 72, 128), (1, 3, 2048, 64), (8, 16, 100, 6144), (4, 3, 4096, 64),
                                     (1700, 3, 160, 256), (2100, 4, 72, 64), (18000, 35, 48, 64),
                                     # groups of few rows at prompt lengths: the kernel with the weights as the 128-row
                                     # operand; one group far larger than the rest (cut into token tiles), widths and
                                     # depths that are no multiple of a tile
                                     (2048, 16, 256, 512), (4096, 128, 136, 192), (700, 9, 200, 328), (520, 5, 128, 64)])
def test_grouped_products(ks, M, E, F, K):
    """Tokens sorted by expert, some experts empty; SwiGLU in, scatter-add out."""
    g = torch.Generator().manual_seed(10)
    ids = torch.randint(0, E, (M,), generator=g)
    ids[ids == 1] = 0                                   # expert 1 stays empty
    if M in (700, 520):
        ids[:M - 200] = E - 1                           # one group with most of the tokens
    order = torch.sort(ids, stable=True)
    rows = order.indices.to(torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(torch.bincount(ids, minlength=E), 0)
    x = rnd((M, K), ks.dtype, 11)
    w_gu, w_d = rnd((E, 2 * F, K), ks.dtype, 12, 0.3), rnd((E, K, F), ks.dtype, 13, 0.3)
    scale = torch.rand(M, generator=g) + 0.5
    r = ref_set(ks.dtype)
    a = torch.zeros((M, F), dtype=ks.dtype, device=DEV)
    swapped = ks.launches_by_library["gemm_tc_experts"]
    ks.grouped_linear_swiglu(x.to(DEV), w_gu.to(DEV), rows.to(DEV), offsets.to(DEV), scale.to(DEV), a)
    if ks.dtype == torch.bfloat16 and 16 < M <= 64 * E and K % 8 == 0:
        assert ks.launches_by_library["gemm_tc_experts"] == swapped + 1   # few rows a group: the weights are the 128-row operand
    a_ref = torch.zeros((M, F), dtype=torch.float64)
    r.grouped_linear_swiglu(x, w_gu, rows, offsets, scale, a_ref)
    close(a, a_ref, TOL[ks.dtype], "grouped_linear_swiglu")
    h = rnd((M, K), torch.float32, 14)
    hd = h.to(DEV).clone()
    if M in (4096, 700, 520) and ks.dtype == torch.bfloat16:
        # the down product with swapped operands too, whatever the sizes (a group of 300 to 500 rows is cut in two)
        ks.tc_experts_max_group_rows, ks.tc_experts_down_min_groups = 256, 1
    swapped = ks.launches_by_library["gemm_tc_experts"]
    ks.grouped_linear_accumulate(a, w_d.to(DEV), rows.to(DEV), offsets.to(DEV), hd)
    if M in (4096, 700, 520) and ks.dtype == torch.bfloat16:
        assert ks.launches_by_library["gemm_tc_experts"] == swapped + 1
    ks.tc_experts_max_group_rows, ks.tc_experts_down_min_groups = 64, 64
    h_ref = h.double().clone()
    r.grouped_linear_accumulate(a.cpu(), w_d, rows, offsets, h_ref)
    close(hd, h_ref, 2e-5 if ks.dtype == torch.float32 else 2e-3, "grouped_linear_accumulate")


# ---------------------------------------------------------------------------- attention
def make_batch(seg_specs, page_size, n_pages, seed, device):
    """seg_specs: [(start_pos, n_tokens)]; pages are dealt out of order."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    segs, tables, toks, off = [], [], [], 0
    for s, (start, n) in enumerate(seg_specs):
        n_pg = -(-(start + n) // page_size)
        tables.append([perm.pop() for _ in range(n_pg)])
        segs.append(Segment(s, s, start, n, off, start == 0))
        toks.append([0] * n)
        off += n
    return build_step_batch(segs, toks, [[] for _ in segs], [tables], device), tables


def fill_cache(kv, tables, seg_specs, k_all, v_all, page_size):
    """Write keys/values of positions [0, start) of every segment (the earlier steps)."""
    for s, (start, n) in enumerate(seg_specs):
        for p in range(start):
            page = tables[s][p // page_size]
            kv[0, page, :, p % page_size, :] = k_all[s][p]
            kv[1, page, :, p % page_size, :] = v_all[s][p]


@pytest.mark.parametrize("nq,nkv,hd,rope,norm,temp", [
    (4, 2, 16, "neighbours", "after", False), (6, 1, 32, "neighbours", None, False), (5, 5, 48, None, None, True),
    (40, 8, 128, "neighbours", "after", False), (3, 1, 256, None, None, False),
    # what other encodings need of the same kernel: the two halves of a head pair up, only the first
    # elements of a head rotate, the norm runs before the rotation, the norm has gains
    (4, 2, 16, "halves", "after", False), (6, 2, 64, "halves", "before+gain", False),
    (8, 2, 128, "halves:64", "after+gain", False), (5, 1, 48, "neighbours:24", "before", True),
    (3, 3, 256, "halves", None, False), (2, 1, 80, "neighbours:40", "after+gain", False)])
def test_qk_prepare(ks, nq, nkv, hd, rope, norm, temp):
    from spite_b200.parts import QkNorm, Rotation
    P, n_pages = 16, 12
    specs = [(0, 19), (30, 1), (15, 3)]
    batch, tables = make_batch(specs, P, n_pages, 20, DEV)
    cpu_batch, _ = make_batch(specs, P, n_pages, 20, "cpu")
    M = batch.n_tokens
    qkv = rnd((M, (nq + 2 * nkv) * hd), ks.dtype, 21)

    def pieces(device):
        rotation = qk_norm = None
        if rope:
            pairing, _, rd = rope.partition(":")
            rd = int(rd) if rd else hd
            inv_freq = torch.tensor([10000.0 ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float32)
            rotation = Rotation(inv_freq.to(device), pairing, rd if rd != hd else None)
        if norm:
            gains = [(rnd((hd,), torch.float32, 30 + i) + 1.5).to(device) if "gain" in norm else None for i in range(2)]
            qk_norm = QkNorm(1e-5, norm.startswith("before"), gains[0], gains[1])
        return dict(num_heads=nq, rotation=rotation, qk_norm=qk_norm, temperature=(8, 0.25) if temp else None)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=ks.dtype, device=DEV)
    q = torch.empty((M, nq * hd), dtype=ks.dtype, device=DEV)
    ks.qk_prepare(qkv.to(DEV), q, batch, LayerCache(0, kv, None, P, True), **pieces(DEV))
    kv_ref = torch.zeros((2, n_pages, nkv, P, hd), dtype=torch.float64)
    q_ref = torch.empty((M, nq * hd), dtype=torch.float64)
    ref_set(ks.dtype).qk_prepare(qkv, q_ref, cpu_batch, LayerCache(0, kv_ref, None, P, True), **pieces("cpu"))
    close(q, q_ref, TOL[ks.dtype], "q")
    close(kv, kv_ref, TOL[ks.dtype], "cache")
    # a run that only reads the cache writes nothing
    kv2 = torch.zeros_like(kv)
    ks.qk_prepare(qkv.to(DEV), q, batch, LayerCache(0, kv2, None, P, False), **pieces(DEV))
    assert not kv2.any()


def test_qk_prepare_halves_is_the_rotation_of_spite_rope(ks):
    """`pairing="halves"` against the formula of crates/spite-rope/src/lib.rs:78-92 written out with loops:
    for i < head_dim/2: freq = theta^(-2i/head_dim), a = pos * freq,
    x[i] <- x[i] cos a - x[i + half] sin a,  x[i + half] <- x[i] sin a + x[i + half] cos a."""
    from spite_b200.parts import Rotation
    nq, nkv, hd, P, theta = 3, 1, 32, 16, 10000.0
    batch, _ = make_batch([(5, 4)], P, 4, 4, DEV)
    M = batch.n_tokens
    qkv = rnd((M, (nq + 2 * nkv) * hd), ks.dtype, 5)
    inv_freq = torch.tensor([theta ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float32)
    kv = torch.zeros((2, 4, nkv, P, hd), dtype=ks.dtype, device=DEV)
    q = torch.empty((M, nq * hd), dtype=ks.dtype, device=DEV)
    ks.qk_prepare(qkv.to(DEV), q, batch, LayerCache(0, kv, None, P, True), num_heads=nq,
                  rotation=Rotation(inv_freq.to(DEV), "halves"), qk_norm=None, temperature=None)
    x = qkv.double().view(M, nq + 2 * nkv, hd)
    want = torch.empty((M, nq, hd), dtype=torch.float64)
    half = hd // 2
    for t in range(M):
        pos = 5 + t
        for h in range(nq):
            for i in range(half):
                a = pos * theta ** (-2.0 * i / hd)
                x0, x1 = float(x[t, h, i]), float(x[t, h, i + half])
                want[t, h, i] = x0 * math.cos(a) - x1 * math.sin(a)
                want[t, h, i + half] = x0 * math.sin(a) + x1 * math.cos(a)
    close(q.view(M, nq, hd), want, TOL[ks.dtype], "half-split rotation")


@pytest.mark.parametrize("nq,nkv,hd,window,P", [
    (4, 2, 16, ("full", 0), 16), (6, 1, 32, ("chunk", 16), 16), (5, 5, 48, ("chunk", 40), 16),
    (40, 8, 128, ("full", 0), 64), (10, 2, 128, ("chunk", 96), 64), (3, 1, 256, ("sliding", 37), 16),
    (8, 2, 64, ("full", 0), 16), (4, 2, 16, ("full", 0), 32), (6, 1, 32, ("chunk", 16), 32),
    (5, 5, 48, ("chunk", 40), 32), (8, 2, 64, ("sliding", 50), 32), (16, 1, 80, ("sliding", 37), 32),
    (12, 4, 112, ("full", 0), 64)])
def test_paged_attention(ks, nq, nkv, hd, window, P):
    """Segments of different kinds in one call: a long prompt portion that crosses
    window and page edges, single tokens deep in a context, a first token."""
    win = Window(*window)
    specs = [(0, 70), (300, 1), (95, 34), (0, 1), (63, 2)]
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 3
    batch, tables = make_batch(specs, P, n_pages, 30, DEV)
    cpu_batch, _ = make_batch(specs, P, n_pages, 30, "cpu")
    M = batch.n_tokens
    g = torch.Generator().manual_seed(31)
    k_all = [torch.randn((s + n, nkv, hd), generator=g) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g)
    # one far key carries the attention of the deep single token: its query is aligned with it
    far = 7 if win.kind == "full" else win.lowest_visible(300) + 1
    q[70] = 0.0
    q[70, :, :] = k_all[1][far, 0, :] * (16.0 / math.sqrt(hd))
    kv_ref = torch.zeros((2, n_pages, nkv, P, hd), dtype=ks.dtype)
    fill = [(s + n, 0) for s, n in specs]                 # all keys of the step are cached before it runs
    fill_cache(kv_ref, tables, fill, [k.to(ks.dtype) for k in k_all], [v.to(ks.dtype) for v in v_all], P)
    qd = q.reshape(M, nq * hd).to(ks.dtype)
    out = torch.empty((M, nq * hd), dtype=ks.dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(qd.to(DEV), out, batch, LayerCache(0, kv_ref.to(DEV), None, P, False),
                       num_heads=nq, window=win, softmax_scale=scale)
    ref = torch.empty((M, nq * hd), dtype=torch.float64)
    ref_set(ks.dtype).paged_attention(qd, ref, cpu_batch, LayerCache(0, kv_ref, None, P, False),
                                      num_heads=nq, window=win, softmax_scale=scale)
    close(out, ref, TOL[ks.dtype], f"attention {window}")
    # the far key must dominate row 70 of head 0, else the test would not see a lost key
    w_far = torch.softmax((k_all[1][win.lowest_visible(300):301, 0].to(ks.dtype).double()
                           @ qd[70, :hd].double()) * scale, 0)
    assert float(w_far[far - win.lowest_visible(300)]) > 0.5


@pytest.mark.parametrize("nq,nkv,hd,window,P", [
    (40, 8, 128, ("full", 0), 64), (40, 8, 128, ("chunk", 8192), 64), (10, 2, 128, ("chunk", 1000), 64),
    (6, 1, 64, ("sliding", 777), 64), (16, 1, 128, ("full", 0), 128), (3, 3, 64, ("chunk", 96), 64),
    (32, 2, 64, ("full", 0), 64)])
def test_paged_attention_decode(nq, nkv, hd, window, P):
    """Decoded tokens deep in long contexts on the TMA-fed decode kernel: dozens of key splits merged by the
    block that comes last, a window that starts and ends inside a 64-key tile, pages behind the window given
    back (and poisoned), requests of very different lengths in one call, a first token, two-token portions
    (several tokens in one block), and one far key among thousands that carries a row's attention."""
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    win = Window(*window)
    specs = [(8191, 1), (5000, 1), (0, 1), (63, 1), (64, 2), (3000, 2), (129, 1), (1023, 1)]
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 5
    batch, tables = make_batch(specs, P, n_pages, 50, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(51)
    k_all = [torch.randn((s + n, nkv, hd), generator=g).to(torch.bfloat16) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g).to(torch.bfloat16) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g)
    far = 11 if win.kind == "full" else win.lowest_visible(8191) + 1
    q[0] = k_all[0][far, 0, :].float() * (16.0 / math.sqrt(hd))       # row 0: the token at position 8191
    q = q.to(torch.bfloat16)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=torch.bfloat16)
    fill_cache(kv, tables, [(s + n, 0) for s, n in specs], k_all, v_all, P)
    bt = batch.block_tables[0]
    for s, (start, n) in enumerate(specs):                           # pages wholly behind the window are gone
        for pg in range(win.lowest_visible(start) // P):
            kv[:, tables[s][pg]] = float("nan")
            bt[s, pg] = -1
    out = torch.empty((M, nq * hd), dtype=torch.bfloat16, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    before = ks.launches_by_library["attention_decode"]
    for _ in range(2):                                               # twice: the tickets must be back at zero
        out.fill_(float("nan"))
        ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, kv.to(DEV), None, P, False),
                           num_heads=nq, window=win, softmax_scale=scale)
        ref = dense_attention_reference(q, k_all, v_all, specs, nq, nkv, win, scale)
        close(out.view(M, nq, hd), ref, TOL[torch.bfloat16], f"decode attention {window}")
    assert ks.launches_by_library["attention_decode"] == before + 2 and ks.errors() == {}
    assert ks.attention_scratch_bytes > 0 or win.kind != "full"       # the keys were split among blocks
    lo = win.lowest_visible(8191)
    w_far = torch.softmax((k_all[0][lo:8192, 0].double() @ q[0, 0].double()) * scale, 0)
    assert float(w_far[far - lo]) > 0.5


def dense_attention_reference(q, k_all, v_all, specs, nq, nkv, win, scale):
    """softmax(q k^T) v per request with a dense mask, float64; q [M, nq, hd] and the keys already rounded."""
    out = torch.empty(q.shape, dtype=torch.float64)
    group, off = nq // nkv, 0
    for s, (start, n) in enumerate(specs):
        pos = torch.arange(start, start + n)
        lo = torch.tensor([win.lowest_visible(int(p)) for p in pos])
        j = torch.arange(start + n)
        mask = (j[None, :] <= pos[:, None]) & (j[None, :] >= lo[:, None])
        for h in range(nq):
            sc = (q[off:off + n, h].double() @ k_all[s][:, h // group].double().T) * scale
            w = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1)
            out[off:off + n, h] = w @ v_all[s][:, h // group].double()
        off += n
    return out


@pytest.mark.parametrize("nq,nkv,hd,window,P", [
    (10, 2, 128, ("full", 0), 64), (8, 8, 128, ("chunk", 128), 64), (6, 1, 64, ("chunk", 96), 64),
    (16, 1, 128, ("sliding", 100), 128), (40, 8, 128, ("chunk", 256), 64), (3, 3, 64, ("full", 0), 128),
    (9, 3, 64, ("chunk", 300), 64), (48, 3, 64, ("chunk", 300), 64), (40, 8, 128, ("chunk", 425), 64)])
def test_paged_attention_tcgen05(nq, nkv, hd, window, P):
    """Prompt portions that go to the tcgen05 kernel: several 128-row tiles per request, portions that
    start deep in a context, windows that end inside a 64-key tile, pages behind the window given back,
    a window's edge several key tiles into a row tile's keys (some of its rows then start late and the
    output is rescaled in the middle of the walk), and a block whose second row tile starts at a window's
    edge more key tiles on than the ring holds (tokens 400-424 and 425-449 with chunks of 425)."""
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    win = Window(*window)
    specs = [(0, 650 if window[1] in (300, 425) else 300), (200, 130), (1000, 64), (0, 1), (517, 40)]
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 5
    batch, tables = make_batch(specs, P, n_pages, 40, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(41)
    k_all = [torch.randn((s + n, nkv, hd), generator=g).to(torch.bfloat16) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g).to(torch.bfloat16) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g)
    # a far key carries the attention of one row deep in the first portion
    far = 3 if win.kind == "full" else win.lowest_visible(290) + 1
    q[290] = k_all[0][far, 0, :].float() * (16.0 / math.sqrt(hd))
    q = q.to(torch.bfloat16)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=torch.bfloat16)
    fill_cache(kv, tables, [(s + n, 0) for s, n in specs], k_all, v_all, P)
    if win.kind != "full":
        # pages that lie wholly behind the window of a portion's first token are given back: the kernel may
        # not read them, so poison what they held and drop them from the table
        bt = batch.block_tables[0]
        for s, (start, n) in enumerate(specs):
            for pg in range(win.lowest_visible(start) // P):
                kv[:, tables[s][pg]] = float("nan")
                bt[s, pg] = -1
    out = torch.empty((M, nq * hd), dtype=torch.bfloat16, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, kv.to(DEV), None, P, False),
                       num_heads=nq, window=win, softmax_scale=scale)
    assert ks.attention_tc_error() == 0
    ref = dense_attention_reference(q, k_all, v_all, specs, nq, nkv, win, scale)
    close(out.view(M, nq, hd), ref, TOL[torch.bfloat16], f"tcgen05 attention {window}")
    lo = win.lowest_visible(290)
    w_far = torch.softmax((k_all[0][lo:291, 0].double() @ q[290, 0].double()) * scale, 0)
    assert float(w_far[far - lo]) > 0.5


@pytest.mark.parametrize("n_tokens,library", [(1, "attention_decode"), (1, "attention_mma"), (9, "attention_rows"),
                                              (60, "attention_tc")])
def test_paged_attention_long_context(n_tokens, library):
    """The last tokens of a 40,000-token context on each bfloat16 attention kernel: thousands of key tiles,
    key splits and their merge for the single token, hundreds of pages in random order."""
    from spite_b200.kernels.cuda import CudaKernels
    ks = CudaKernels(torch.bfloat16, DEV)
    ks.use_decode_attention = library != "attention_mma"
    nq, nkv, hd, P, C = 10, 2, 128, 64, 40000
    n_pages = C // P + 3
    batch, tables = make_batch([(C - n_tokens, n_tokens)], P, n_pages, 50, DEV)
    g = torch.Generator(device=DEV).manual_seed(51)
    kv = torch.randn((2, n_pages, nkv, P, hd), generator=g, device=DEV).to(torch.bfloat16)
    q = torch.randn((n_tokens, nq, hd), generator=g, device=DEV)
    # the first key carries the attention of the last token's first head
    tbl = torch.tensor(tables[0], device=DEV)
    q[-1, 0] = kv[0, tbl[0], 0, 0].float() * (24.0 / math.sqrt(hd))
    q = q.to(torch.bfloat16)
    out = torch.empty((n_tokens, nq * hd), dtype=torch.bfloat16, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(q.reshape(n_tokens, nq * hd), out, batch, LayerCache(0, kv, None, P, False), num_heads=nq,
                       window=Window("full", 0), softmax_scale=scale)
    assert ks.launches_by_library[library] > 0, dict(ks.launches_by_library)
    K = kv[0][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd).double()      # [kv heads, positions, head size]
    V = kv[1][tbl].permute(1, 0, 2, 3).reshape(nkv, -1, hd).double()
    ref = torch.empty((n_tokens, nq, hd), dtype=torch.float64, device=DEV)
    for t in range(n_tokens):
        pos = C - n_tokens + t
        for h in range(nq):
            w = torch.softmax((K[h // (nq // nkv), :pos + 1] @ q[t, h].double()) * scale, 0)
            ref[t, h] = w @ V[h // (nq // nkv), :pos + 1]
            if t == n_tokens - 1 and h == 0:
                assert float(w[0]) > 0.5
    close(out.view(n_tokens, nq, hd), ref, TOL[torch.bfloat16], f"attention over {C} keys ({library})")


# ---------------------------------------------------------------------------- router
@pytest.mark.parametrize("M,d,E,k", [(1, 48, 3, 1), (37, 96, 8, 1), (200, 200, 16, 2), (5, 64, 128, 4)])
def test_moe_route(ks, M, d, E, k):
    x = rnd((M, d), ks.dtype, 40)
    w = rnd((E, d), torch.float32, 41, 0.3)
    if E >= 3:
        w[2] = w[0]                                      # equal logits: the lower expert id wins
    got = ks.moe_route(x.to(DEV), w.to(DEV), k, want_logits=True)
    ref = ref_set(ks.dtype).moe_route(x, w, k, want_logits=True)
    close(got.logits, ref.logits, 1e-5, "router logits")
    # compare choices where float32 rounding cannot change the order
    srt = torch.sort(ref.logits.double(), dim=-1, descending=True).values
    clear = ((srt[:, :-1] - srt[:, 1:])[:, :k].min(dim=1).values > 1e-4) if E > 1 else torch.ones(M, dtype=torch.bool)
    ties = (ref.expert_ids.T.long() == 0).any(1) | (ref.expert_ids.T.long() == 2).any(1)
    keep = clear | ties
    assert torch.equal(got.expert_ids.cpu().T[keep], ref.expert_ids.T[keep])
    assert not (got.expert_ids.cpu() == 2).any() or k > 1
    close(got.weights, ref.weights, 1e-5, "router weights")
    for s in range(k):
        ids = got.expert_ids[s].cpu().long()
        order = torch.sort(ids, stable=True)
        assert torch.equal(got.sorted_rows[s].cpu().long(), order.indices)
        assert got.offsets[s].cpu().tolist() == [0] + torch.cumsum(torch.bincount(ids, minlength=E), 0).tolist()


# ---------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("V", [1000, 16384, 202048, 50001])
def test_argmax_prefers_the_highest_index(ks, V):
    """Rows of 16,384 logits and more are read by a cluster of eight blocks: equal maxima in different blocks'
    parts, at both ends of the row and of a part, a constant row, a row without a finite value."""
    if ks.dtype != torch.float32:
        pytest.skip("logits are float32 in both sets")
    part = -(-V // 8)
    l = rnd((9, V), torch.float32, 50)
    l[0, 17] = l[0, V // 2 + 88] = 9.0
    l[1, V - 1] = 9.0
    l[2, 0] = 9.0
    l[3] = 0.0
    l[4, part - 1] = l[4, part] = 9.0                     # the last of one block's part and the first of the next
    l[5, 3 * part] = l[5, 5] = 9.0
    l[6, 7 * part - 1] = 9.0
    l[7] = -float("inf")
    l[8, 2 * part + 1] = 9.0
    got = ks.argmax(l.to(DEV)).cpu()
    ref = ref_set(torch.float32).argmax(l)
    assert got.tolist() == ref.tolist()
    assert got.tolist() == [V // 2 + 88, V - 1, 0, V - 1, part, 3 * part, 7 * part - 1, V - 1, 2 * part + 1]


@pytest.mark.parametrize("V", [512, 1000, 202048])
def test_sample_matches_the_plain_sampler(ks, V):
    if ks.dtype != torch.float32:
        pytest.skip("logits are float32 in both sets")
    from plain_llama4 import lcg_next, process_logits_plain, sample_plain
    R = 8
    l = rnd((R, V), torch.float32, 51, 2.0)
    cases = [dict(temperature=0.0), dict(temperature=0.7), dict(temperature=1.0, top_k=5),
             dict(temperature=0.9, top_p=0.8), dict(temperature=1.3, min_p=0.05),
             dict(temperature=0.8, repetition_penalty=1.3), dict(temperature=0.0, repetition_penalty=1.5),
             dict(temperature=1.0, top_k=40, top_p=0.95, min_p=0.01, repetition_penalty=1.1)]
    ctx = [torch.randint(0, V, (20,)).tolist() for _ in range(R)]
    for r in range(R):
        ctx[r][0] = int(l[r].argmax())                  # the penalty hits the likeliest token
    state = torch.tensor([1234 + r for r in range(R)], dtype=torch.int64)
    f = lambda key, d, dt: torch.tensor([c.get(key, d) for c in cases], dtype=dt, device=DEV)
    offsets = torch.tensor([20 * r for r in range(R + 1)], dtype=torch.int32, device=DEV)
    context = torch.tensor(sum(ctx, []), dtype=torch.int32, device=DEV)
    for draw in range(3):
        dev_state = state.clone().to(DEV)
        got = ks.sample(l.to(DEV), temperature=f("temperature", 0.0, torch.float32),
                        top_k=f("top_k", 0, torch.int32), top_p=f("top_p", 1.0, torch.float32),
                        min_p=f("min_p", 0.0, torch.float32),
                        repetition_penalty=f("repetition_penalty", 1.0, torch.float32),
                        context=context, context_offsets=offsets, rng_state=dev_state).cpu().tolist()
        new_state = []
        for r, c in enumerate(cases):
            tok, st = sample_plain(l[r], ctx[r], repeat_last_n=0, state=int(state[r]), **c)
            new_state.append(st)
            if got[r] == tok:
                continue
            # float32 running sums in another order may cross the target one token earlier or
            # later; the drawn token must still be the one whose mass interval holds the target
            assert c["temperature"] > 0, f"case {c}: device {got[r]}, plain {tok}"
            proc = process_logits_plain(l[r], ctx[r], repeat_last_n=0, **c).double()
            mass = torch.exp(proc - proc.max())
            cum = torch.cumsum(mass, 0)
            target = lcg_next(int(state[r]) & ((1 << 64) - 1))[1] * float(mass.sum())
            slack = 2e-5 * float(mass.sum())
            lo = float(cum[got[r] - 1]) if got[r] > 0 else 0.0
            assert mass[got[r]] > 0 and lo - slack <= target <= float(cum[got[r]]) + slack, \
                f"draw {draw}, case {c}: device {got[r]}, plain {tok}"
        back = [int(s) & ((1 << 64) - 1) for s in dev_state.cpu().tolist()]
        assert back == new_state
        state = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in new_state], dtype=torch.int64)
