"""How the weight-streaming kernel's work is cut (k slices inside a block, k splits across blocks): the host-side
choice alone, at the shapes it was measured on and at its borders.  The kernel itself with every cut:
test_gpu_kernels.py::test_streaming_products_with_k_slices_and_k_splits."""
import pytest

from spite_b200.kernels.cuda import stream_cut

FEW = dict(slots=296, smem=110 * 1024)        # up to three tokens: two blocks a multiprocessor
MORE = dict(slots=444, smem=74 * 1024)        # more: three


def cut(M, N, K, groups=1, swiglu=False, **kw):
    shape = dict(FEW if M <= 3 else MORE)
    shape.update(kw)
    return stream_cut(M, N, K, groups, swiglu, shape.pop("slots"), shape.pop("smem"), 8 if M <= 8 else 16, **shape)


def test_the_measured_shapes_get_the_cuts_that_were_fastest():
    # eight tokens at Scout's layer shapes: slices, no partial sums through global memory
    assert cut(8, 7168, 5120) == (4, 1)                       # qkv: 224 tiles of 32 rows
    assert cut(8, 5120, 5120) == (8, 1)                       # output projection: 320 tiles of 16 rows
    assert cut(8, 5120, 8192) == (8, 1)                       # shared expert, down
    assert cut(8, 8192, 5120, groups=7, swiglu=True)[1] == 1  # seven experts' gate/up: tiles enough without k splits
    assert cut(8, 5120, 8192, groups=7) == (4, 1)             # (if the caller allows slices for grouped products)
    assert cut(8, 5120, 8192, groups=7, max_slices=1)[0] == 1
    # one token: tiles of 128 rows, k splits that fill 296 blocks about once
    assert cut(1, 7168, 5120) == (1, 5)
    assert cut(1, 5120, 5120) == (1, 7)
    assert cut(1, 8192, 5120, swiglu=True) == (1, 2)
    # the output head has tiles enough as it is
    assert cut(1, 202048, 5120) == (1, 1) and cut(8, 202048, 5120)[1] == 1


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 13, 16])
@pytest.mark.parametrize("N,K,swiglu", [(40, 64, False), (200, 320, False), (104, 1024, True), (5120, 8192, False),
                                        (8192, 5120, True), (129, 4096, False), (16, 64, True)])
@pytest.mark.parametrize("groups", [1, 5])
def test_every_cut_is_one_the_kernel_takes(M, N, K, swiglu, groups):
    slices, splits = cut(M, N, K, groups=min(groups, M), swiglu=swiglu)
    assert slices in (1, 2, 4, 8) and K % (64 * slices) == 0          # a stage is `slices` k blocks of 64
    assert not (swiglu and slices == 8)                                # tiles of 8 gate and 8 up rows are not built
    assert slices == 1 or M >= 4                                       # few rows keep tiles of 128 rows (the function's default)
    stages = K // (64 * slices)
    assert 1 <= splits <= max(1, stages // 4)                          # at least four stages stay together
    nt = 8 if M <= 8 else 16
    smem = (FEW if M <= 3 else MORE)["smem"]
    ring = (smem - 5504 - (8 - 8 // slices) * 64 * nt) // (16384 + max(1024, slices * nt * 128))
    assert ring >= 2                                                   # a ring of at least two stages fits


def test_splits_that_can_be_a_cluster_are_preferred_when_the_caller_offers_clusters():
    assert cut(1, 7168, 5120, cluster_max_splits=4, cluster_cost=9.0) == (1, 4)      # qkv: 224 blocks, 56 clusters of four
    assert cut(1, 5120, 5120, cluster_max_splits=4, cluster_cost=9.0) == (1, 7)      # too few blocks in fours
    assert cut(1, 8192, 5120, swiglu=True, cluster_max_splits=4, cluster_cost=9.0) == (1, 2)
    # never more blocks than are resident at once: 128 tiles in four splits are 512 blocks for 296 places
    assert cut(1, 8192, 5120, swiglu=True, cluster_max_splits=4, cluster_cost=0.0) == (1, 2)


def test_the_costs_move_the_choice():
    assert cut(8, 5120, 5120, max_slices=1)[0] == 1                    # tiles of 128 rows only: k splits again
    assert cut(8, 5120, 5120, max_slices=1)[1] > 1
    assert cut(2, 5120, 5120, slices_min_rows=1)[0] > 1                # slices allowed at two rows
    assert cut(8, 5120, 5120, slice_cost=100.0)[0] == 1                # slices made expensive
    assert cut(1, 5120, 5120, split_item_cost=1000.0) == (1, 1)        # splits made expensive
