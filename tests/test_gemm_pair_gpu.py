"""GPU parity for the two-CTA (cta_group::2) kernels: a cluster of two SMs shares each tile."""
import pytest
import torch

from gemm_b200 import ops
from tests.util import gpu_bits_compare, run_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("block_n", [256, 128])
def test_pair_kernels_small(block_n):
    stats, cfg = run_case(512, 512, 512, override=dict(cta_group=2, block_n=block_n, swap=0))
    assert cfg["cta_group"] == 2 and cfg["block_n"] == block_n, cfg


@pytest.mark.parametrize("block_n", [256, 128])
def test_pair_kernels_ragged(block_n):
    ov = dict(cta_group=2, block_n=block_n, swap=0)
    run_case(520, 776, 1352, override=ov)                 # ragged everywhere
    run_case(130, 264, 72, override=ov)                   # second CTA's rows mostly out of range
    run_case(1000, 520, 200, override=ov, col_major=True)


def test_pair_kernels_large():
    for bn in (256, 128):
        run_case(4096, 4096, 4096, override=dict(cta_group=2, block_n=bn, swap=0))
    run_case(8192, 8192, 8192, override=dict(cta_group=2, block_n=256, swap=0))


def test_pair_kernel_is_deterministic():
    from gemm_b200.inputs import make_problem
    A, B = make_problem(2048, 2048, 1024, seed=4)
    dA, dB = A.cuda(), B.cuda()
    ops.set_override(cta_group=2, block_n=256, swap=0)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(10):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        ops.set_override()
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("cta_group,block_n", [(2, 256), (2, 128), (1, 256), (1, 128)])
def test_cut_last_wave_on_every_tma_store_kernel(cta_group, block_n):
    # Force the stream-K treatment of the last, partly filled wave (ragged shape, several waves).
    ov = dict(cta_group=cta_group, block_n=block_n, swap=0, stream_k=1)
    stats, cfg = run_case(3000, 5000, 2048, override=ov)
    assert cfg["stream_k"] == 1 and cfg["cta_group"] == cta_group, cfg
    run_case(1000, 520, 2048, override=ov, col_major=True)


def test_cut_last_wave_is_chosen_for_4096_cube_and_is_deterministic():
    from gemm_b200.inputs import make_problem
    stats, cfg = run_case(4096, 4096, 4096)
    assert (cfg["cta_group"], cfg["block_n"], cfg["stream_k"]) == (2, 256, 1), cfg
    A, B = make_problem(4096, 4096, 2048, seed=6)
    dA, dB = A.cuda(), B.cuda()
    first = ops.matmul(dA, dB).clone()
    assert ops.last_config()["stream_k"] == 1
    for _ in range(10):
        assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


def test_wide_pair_tile_is_the_default_for_8192_cube():
    stats, cfg = run_case(8192, 8192, 8192)
    assert (cfg["cta_group"], cfg["block_n"], cfg["stages"]) == (2, 512, 4), cfg


@pytest.mark.parametrize("shape", [(512, 1024, 512), (520, 776, 1352), (130, 264, 72),
                                   (1000, 1544, 200), (4096, 4096, 1024)])
def test_wide_pair_tile_ragged(shape):
    # 256 x 512 tile: both TMEM accumulators belong to one tile; ragged rows, columns and K,
    # a second half that is partly or wholly out of range, several tiles per CTA pair.
    stats, cfg = run_case(*shape, tuning={"wide_tile": 1})
    assert cfg["block_n"] == 512 and cfg["cta_group"] == 2, cfg
    run_case(*shape, tuning={"wide_tile": 1}, col_major=True)


@pytest.mark.parametrize("prologue", [1, 2, 3])
@pytest.mark.parametrize("shape", [(2048, 4096, 64), (2048, 4096, 128), (2104, 4104, 192),
                                   (2048, 4096, 320), (4096, 8192, 2048)])
def test_wide_pair_tile_hand_over(shape, prologue):
    # Several tiles per CTA pair, so every hand-over path runs: tiles of one to a few k-blocks
    # (shorter than the half-0 prologue and than the early notice to the epilogue warps) and
    # long ones, with each prologue length.
    stats, cfg = run_case(*shape, tuning={"wide_tile": 1, "wide_tile_prologue": prologue})
    assert cfg["block_n"] == 512 and cfg["cta_group"] == 2, cfg


def test_wide_pair_tile_is_deterministic_and_never_wide_when_switched_off():
    from gemm_b200.inputs import make_problem
    A, B = make_problem(2048, 4096, 1024, seed=14)
    dA, dB = A.cuda(), B.cuda()
    ops.set_tuning("wide_tile", 1)
    # K walked forwards by every tile (the default alternates the direction from wave to wave,
    # and the two kernels have different waves), so that both sum every element in the same order.
    ops.set_tuning("k_direction_alternates", 0)
    try:
        first = ops.matmul(dA, dB).clone()
        assert ops.last_config()["block_n"] == 512
        for _ in range(10):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
        ops.set_tuning("wide_tile", 0)
        other = ops.matmul(dA, dB)
        assert ops.last_config()["block_n"] <= 256
        # with the default direction rule the narrower kernel (two waves) still repeats itself
        ops.set_tuning("k_direction_alternates", -1)
        again = ops.matmul(dA, dB).clone()
        for _ in range(4):
            assert torch.equal(again.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        ops.set_tuning("wide_tile", -1)
        ops.set_tuning("k_direction_alternates", -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    # same k order per element in both kernels -> identical bits
    assert torch.equal(first.view(torch.int16), other.view(torch.int16))
    s = gpu_bits_compare(again, first)
    assert s["max_ulp"] <= 1 and s["near_zero_ok"] and s["bit_equal_frac"] >= 0.98, s


@pytest.mark.parametrize("shape", [(4096, 8192, 256), (8192, 8192, 1024), (5000, 3000, 640),
                                   (16384, 4096, 512)])
def test_wave_pacing_changes_neither_bits_nor_much_time(shape):
    # Workers wait for each other at the start of every wave (an arrival counter in global
    # memory that must be back at zero after every launch).  Forced on, also for short waves:
    # same bits as without it, launch after launch, and no launch that sits out its time-outs.
    from gemm_b200.inputs import make_problem
    A, B = make_problem(*shape, seed=21)
    dA, dB = A.cuda(), B.cuda()

    out_buf = torch.empty((shape[0], shape[1]), dtype=torch.bfloat16, device="cuda")

    def timed(n):
        # every launch between its own pair of events; the median, so that one stall of the
        # machine (another process, a clock change) does not decide the comparison
        times = []
        for _ in range(n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = ops.matmul(dA, dB, out=out_buf)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
        return out.clone(), sorted(times)[len(times) // 2]

    ops.set_tuning("wave_pacing", 0)
    try:
        plain, _ = timed(3)
        plain, t_plain = timed(10)
        ops.set_tuning("wave_pacing", 1)
        paced, _ = timed(3)
        paced, t_paced = timed(10)
    finally:
        ops.set_tuning("wave_pacing", -1)
    assert torch.equal(plain.view(torch.int16), paced.view(torch.int16))
    assert ops.device_status()[0] == 0
    assert t_paced <= 2.0 * t_plain + 0.1, (t_plain, t_paced)
    run_case(*shape, tuning={"wave_pacing": 1})


@pytest.mark.parametrize("shape", [(4096, 8192, 256), (8192, 4096, 1096), (5000, 3000, 640),
                                   (2048, 2048, 8192)])
def test_alternating_k_direction(shape):
    # Odd waves fetch their k-blocks last to first (ragged last k-block included); the MMA warp
    # does not know.  Parity with the oracle and the same bits launch after launch.
    from gemm_b200.inputs import make_problem
    stats, cfg = run_case(*shape, tuning={"k_direction_alternates": 1})
    run_case(*shape, tuning={"k_direction_alternates": 1}, col_major=True)
    A, B = make_problem(*shape, seed=33)
    dA, dB = A.cuda(), B.cuda()
    ops.set_tuning("k_direction_alternates", 1)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(4):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        ops.set_tuning("k_direction_alternates", -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
