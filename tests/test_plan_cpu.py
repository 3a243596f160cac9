"""Host logic of the tensor-core backend's planner (no GPU needed): for a sweep of shapes the
persistent grids fit the machine, shared memory stays under the limit, and the tiling covers the
problem exactly."""
import ctypes

import pytest

from flashlstm_poc_b200 import _build, _lib

SMS, SMEM = 148, 232448  # B200


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _lib.load()


def plan(lib, B, H, training=1, sms=SMS, smem=SMEM):
    info = _lib.TcPlanInfo()
    st = lib.flstm_tc_plan(B, H, training, sms, smem, ctypes.byref(info))
    return st, info


@pytest.mark.parametrize("H", [64, 128, 192, 256, 512, 768, 1024, 2048, 4096])
@pytest.mark.parametrize("B", [1, 8, 32, 64, 200, 256, 2048])
def test_plans_fit_the_machine(lib, B, H):
    st, p = plan(lib, B, H, training=1 if H <= 2048 else 0)
    assert st == 0, lib.flstm_last_error()
    if p.step_path:
        # one output-tiled GEMM launch per step; K = 4H split while tiles are scarce
        assert H % 128 == 0 and p.fwd_grid == 0
        assert p.step_bn_fwd in (64, 128, 256) and p.step_bn_bwd in (128, 256) and (4 * H) % p.step_bn_fwd == 0
        assert H % p.step_bn_bwd == 0 and p.step_splits in (1, 2, 4, 8) and (4 * H // 64) % p.step_splits == 0
        return
    assert p.fwd_tiles_per_group == 1 or H % 128 != 0  # the persistent kernels keep the single-tile shapes
    # forward: co-resident grid, covers all row tiles and all sequences
    assert 1 <= p.fwd_grid <= SMS and p.fwd_smem_bytes <= SMEM
    cta_rows = p.fwd_grid // p.fwd_batch_groups
    assert cta_rows * p.fwd_row_tiles_per_cta == H // 16
    assert p.fwd_batch_groups * p.fwd_tiles_per_group * p.fwd_batch_tile >= B
    assert (H // 64) % p.fwd_chunks_per_stage == 0 and p.fwd_stages >= 1
    if not p.fwd_weights_resident:
        assert H >= 2048 or B >= 128  # small batches keep their W_hh slice in shared memory up to H = 1024
    if H <= 2048:
        assert 1 <= p.bwd_grid <= SMS and p.bwd_smem_bytes <= SMEM
        assert p.bwd_cluster_size in (1, 2, 4) and p.bwd_grid % p.bwd_cluster_size == 0
        assert p.bwd_grid == (H // 64) * p.bwd_cluster_size * p.bwd_batch_groups
        assert ((H // 16) // p.bwd_cluster_size) % p.bwd_chunks_per_stage == 0
        assert p.bwd_batch_groups * p.bwd_tiles_per_group * p.bwd_batch_tile >= B


def test_benchmark_configuration_plan(lib):
    """Config 2 (H=1024, B=64): 64 row tiles x 2 batch halves, resident weights, one whole-tile copy per
    step; BPTT as 32 clusters of 4."""
    st, p = plan(lib, 64, 1024)
    assert st == 0
    assert (p.fwd_grid, p.fwd_batch_tile, p.fwd_batch_groups, p.fwd_tiles_per_group) == (128, 32, 2, 1)
    assert p.fwd_weights_resident == 1 and p.fwd_chunks_per_stage == 16 and p.fwd_stages == 1
    assert (p.bwd_grid, p.bwd_cluster_size, p.bwd_weights_resident) == (128, 4, 1)


@pytest.mark.parametrize("B,H,step", [(64, 1024, 0), (96, 1024, 1), (128, 1024, 0), (160, 1024, 0), (256, 1024, 0),
                                      (512, 1024, 1), (2048, 1024, 1),
                                      (32, 2048, 0), (64, 2048, 0), (128, 2048, 1), (256, 2048, 1), (8, 4096, 0),
                                      (64, 4096, 1), (96, 4096, 1)])
def test_path_choice_follows_the_measured_crossover(lib, B, H, step):
    """Measured on B200: the persistent kernels win while a CTA has one batch tile per step, the per-step GEMM
    launches win from two tiles per CTA on.  Where the row tiles alone fill the machine (H = 2048), 33..64
    sequences are one 64-wide tile, so that shape stays on the persistent kernels (46.5 vs 55.6 ms per step at L=2,
    T=1024); with two row tiles per CTA (H = 4096) the per-step path is faster (75.6 vs 88.6 ms)."""
    st, p = plan(lib, B, H, training=0 if H == 4096 else 1)
    assert st == 0 and p.step_path == step
    if not step and H >= 2048 and B > 32:
        assert p.fwd_batch_tile == 64 and p.fwd_tiles_per_group == 1
    if not step and H == 1024 and B > 128:  # two batch groups side by side, each on one 128-wide tile
        assert (p.fwd_batch_tile, p.fwd_batch_groups, p.fwd_tiles_per_group) == (128, 2, 1)
        assert (p.bwd_batch_tile, p.bwd_batch_groups, p.bwd_tiles_per_group) == (128, 2, 1)


@pytest.mark.parametrize("H", [64, 256, 512, 768, 1024, 1536, 2048, 4096])
def test_persistent_plans_cover_every_sequence(lib, H):
    """Whatever tile width the planner settles on, groups x tiles per group x tile width reaches the whole batch
    (a plan that covered fewer sequences would leave rows of every output unwritten)."""
    for B in list(range(1, 66)) + [95, 96, 97, 127, 128, 129, 160, 192, 255, 256, 257, 512, 1000, 2048]:
        for training in (0, 1):
            st, p = plan(lib, B, H, training=training)
            if st != 0 or p.step_path:
                continue
            assert p.fwd_batch_groups * p.fwd_tiles_per_group * p.fwd_batch_tile >= B, (B, H)
            assert p.fwd_grid <= 148
            if training:
                assert p.bwd_batch_groups * p.bwd_tiles_per_group * p.bwd_batch_tile >= B, (B, H)
                assert p.bwd_grid <= 148


def test_wide_batch_plans(lib):
    """Config 3 (B=256, H=2048): 128 forward tiles of 128 x 128, backward K split 4 ways.
    Config 5 (B=2048, H=1024): 256-wide forward tiles, no K split."""
    st, p = plan(lib, 256, 2048)
    assert st == 0 and (p.step_path, p.step_bn_fwd, p.step_splits) == (1, 128, 4)
    assert p.step_fwd_pair == 1  # 256 sequences: the all-steps forward kernel on CTA pairs
    st, p = plan(lib, 2048, 1024)
    assert st == 0 and (p.step_path, p.step_bn_fwd, p.step_splits, p.step_fwd_pair) == (1, 256, 1, 1)
    # config 3's 2-GPU shard (B=128): 128-wide forward tiles would leave 84 SMs idle -> 128 tiles of 128 x 64
    st, p = plan(lib, 128, 2048)
    assert st == 0 and (p.step_path, p.step_bn_fwd, p.step_splits, p.step_fwd_pair) == (1, 64, 8, 0)
    # the persistent forward kernel pairs neighbouring row tiles whenever their number is even
    st, p = plan(lib, 64, 1024)
    assert st == 0 and (p.step_path, p.fwd_pair, p.fwd_grid) == (0, 1, 128)


def test_unsupported_shapes_are_reported(lib):
    st, _ = plan(lib, 8, 100)
    assert st == 4 and b"multiple of 64" in lib.flstm_last_error()
    st, _ = plan(lib, 8, 1024, smem=16 * 1024)  # a machine with too little shared memory
    assert st == 4
