"""GPU parity tests proper: the CUDA path through the C ABI against the CPU oracle.

Tolerances (oracle.assert_parity): allclose rtol=1e-2/atol=1e-2 vs the fp32-accumulated product,
relative Frobenius error <= 3e-3, >= 98 % of elements bit-equal to the RNE-rounded oracle, none
more than 1 bf16 ulp away.
"""
import numpy as np
import pytest
import torch

from gemm_b200 import ops
from gemm_b200.inputs import make_problem
from oracle import oracle
from tests.util import run_case

pytestmark = pytest.mark.gpu


# ---- the benchmark configurations ------------------------------------------------------------
def test_config_512_cube_row_and_column_major():
    run_case(512, 512, 512)
    run_case(512, 512, 512, col_major=True)


def test_config_4096_cube():
    run_case(4096, 4096, 4096)


def test_config_8192_cube():
    run_case(8192, 8192, 8192)


@pytest.mark.parametrize("M", [16, 32, 64, 128])
def test_config_decode_shapes(M):
    stats, cfg = run_case(M, 28672, 8192)
    assert cfg["swap"] == 1, cfg
    # one wave of whole tall tiles (200 rows of B per CTA), one CTA per SM on 144 SMs; from 64
    # columns on the CTAs work in pairs that share the small operand
    group = 2 if M >= 64 else 1
    stages = 7 if M <= 64 else 6
    assert (cfg["stream_k"], cfg["ctas"], cfg["tiles"], cfg["stages"], cfg["cta_group"]) == \
        (0, 144, 144 // group, stages, group), cfg
    # the finished tile leaves as one TMA box; M=128 also with the operands' roles exchanged
    assert ops.last_store_path() == (2 if M > 64 else 1)
    if group == 2:
        stats, cfg = run_case(M, 28672, 8192, override=dict(cta_group=1))
        assert (cfg["stream_k"], cfg["ctas"], cfg["tiles"], cfg["cta_group"]) == (0, 144, 144, 1), cfg
    # the other one-wave plan: 224 tiles of 128 rows, two CTAs to an SM
    stats, cfg = run_case(M, 28672, 8192, tuning={"two_ctas_per_sm": 1})
    half = 5 if M <= 32 else (4 if M <= 64 else 3)
    assert (cfg["stream_k"], cfg["ctas"], cfg["stages"]) == (0, 224, half), cfg
    stats, cfg = run_case(M, 28672, 8192, tuning={"two_ctas_per_sm": 0})   # stream-K over 148 CTAs
    assert (cfg["stream_k"], cfg["ctas"]) == (1, 148), cfg
    run_case(M, 28672, 8192, col_major=True)


@pytest.mark.parametrize("shape", [(16, 28672, 8192), (8, 19000, 1024), (24, 30000, 2048),
                                   (64, 28672, 4096), (40, 20008, 1536), (1, 30000, 1024),
                                   (100, 20000, 2048), (128, 28672, 1024), (128, 257, 1024),
                                   (72, 511, 1088), (16, 30784, 1024), (48, 30001, 1024)])
def test_tall_tiles_whole_wave(shape):
    # 136 to 208 rows of the long operand per CTA (its even share of the rows, a multiple of 8),
    # two accumulators sharing the short operand (forced, so that shapes the launcher would not
    # pick on its own run too): ragged rows (a second block that is partly or wholly out of
    # range), ragged K, both layouts, launch-to-launch determinism.
    stats, cfg = run_case(*shape, tuning={"two_ctas_per_sm": 2})
    rows = shape[1]
    per_cta = max(136, (-(-rows // 148) + 7) // 8 * 8)
    group = cfg["cta_group"]
    assert group == (2 if shape[0] > 32 else 1), cfg
    assert cfg["stream_k"] == 0 and cfg["tiles"] == -(-rows // (per_cta * group)), cfg
    assert cfg["ctas"] == cfg["tiles"] * group and cfg["stages"] in (5, 6, 7), cfg
    if group == 2:   # the same tiles on single CTAs
        stats, cfg = run_case(*shape, tuning={"two_ctas_per_sm": 2}, override=dict(cta_group=1))
        assert cfg["cta_group"] == 1 and cfg["ctas"] == cfg["tiles"] == -(-rows // per_cta), cfg
    run_case(*shape, tuning={"two_ctas_per_sm": 2}, col_major=True)
    A, B = make_problem(*shape, seed=6)
    dA, dB = A.cuda(), B.cuda()
    ops.set_tuning("two_ctas_per_sm", 2)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(4):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        ops.set_tuning("two_ctas_per_sm", -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("shape", [(128, 28672, 2048), (96, 20008, 1024), (65, 29600, 1024),
                                   (64, 28672, 1024), (16, 28672, 1024), (24, 20008, 1024),
                                   (100, 30784, 1024), (96, 20008, 1000), (128, 19000, 8192),
                                   (128, 19048, 1024), (80, 18952, 1024)])
def test_tall_tile_store_paths_agree(shape):
    # A tall tile with a transposed bf16 result (row-major C, operands swapped) has three ways
    # out: staged whole in the idle operand ring and stored by the TMA unit as one box (the
    # default); the same with the operands' roles exchanged in the MMA, which the pair kernel of
    # 128 columns does by default (the accumulator is then the transpose, one row of A per lane);
    # and 16-byte stores from registers (what calls with unaligned outputs fall back to).
    # All three must agree with the oracle and, bit for bit, with one another: every element
    # sums the same products in the same k order.  Shapes: full and ragged last tiles (the TMA
    # unit clips the box at the matrix edge; 20008 rows leave the last pair 136 + 16 of them),
    # fewer rows of A than the pair's 2 x 64 (65: one row in the second CTA), a K that ends inside
    # a k-block, tiles of the smallest height (19000 rows: 136 per CTA, a second MMA block of 8;
    # 19048: 141 tiles, the last pair's second CTA has no rows at all; 18952: a last tile of 48).
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=17)
    dA, dB = A.cuda(), B.cuda()
    want = oracle.gemm_fp32(A, B)
    outs = {}
    for mode in (-1, 4, 3):
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.set_tuning("two_ctas_per_sm", mode)
        try:
            ops.matmul(dA, dB, out=C)
            cfg = ops.last_config()
            path = ops.last_store_path()
        finally:
            ops.set_tuning("two_ctas_per_sm", -1)
        torch.cuda.synchronize()
        assert ops.device_status()[0] == 0, (mode, cfg)
        assert cfg["stream_k"] == 0 and cfg["ctas"] == cfg["tiles"] * cfg["cta_group"], cfg
        assert cfg["cta_group"] == (2 if M > 32 else 1), cfg
        assert path == {-1: 2 if M > 64 else 1, 4: 1, 3: 0}[mode], (mode, path, cfg)
        oracle.assert_parity(C, want, f"tall tile store mode {mode} {shape} {cfg}")
        outs[mode] = C
    for mode in (4, 3):
        assert torch.equal(outs[-1].view(torch.int16), outs[mode].view(torch.int16)), mode


@pytest.mark.parametrize("shape", [(16, 28672, 8192), (8, 19000, 1024), (24, 30000, 2048),
                                   (64, 28672, 4096), (40, 20008, 1536), (1, 37000, 1024),
                                   (100, 20000, 2048), (128, 28672, 1024)])
def test_two_ctas_per_sm_whole_tiles(shape):
    # Half-size rings, every tile resident at once (forced, so that the 64-column kernel and
    # shapes the launcher would not pick on its own run too); ragged rows and K, both layouts,
    # and the stream-K plan of the same shape must give the same bits where no tile is cut
    # differently - checked against the oracle, and launch to launch for determinism.
    stats, cfg = run_case(*shape, tuning={"two_ctas_per_sm": 1})
    assert cfg["stream_k"] == 0 and cfg["ctas"] == cfg["tiles"] and cfg["stages"] in (3, 4, 5), cfg
    run_case(*shape, tuning={"two_ctas_per_sm": 1}, col_major=True)
    A, B = make_problem(*shape, seed=5)
    dA, dB = A.cuda(), B.cuda()
    ops.set_tuning("two_ctas_per_sm", 1)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(4):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        ops.set_tuning("two_ctas_per_sm", -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


# ---- edges the reference cannot handle (it needs multiples of 64, nemgemmV03.cu:375) ----------
SMALL = [1, 8, 17, 64, 100, 128, 129, 200, 256, 300]


@pytest.mark.parametrize("K", [8, 64, 72, 200, 512])
def test_ragged_shape_sweep(K):
    rng = np.random.default_rng(K)
    pairs = [(m, n) for m in SMALL for n in SMALL]
    picks = rng.choice(len(pairs), size=14, replace=False)
    for i in picks:
        m, n = pairs[i]
        run_case(m, n, K, seed=1000 + int(i))
        run_case(m, n, K, seed=2000 + int(i), col_major=True)


@pytest.mark.parametrize("block_n,stream_k", [(256, 0), (128, 0), (128, 1), (64, 0), (64, 1),
                                              (32, 0), (32, 1), (16, 0), (16, 1)])
@pytest.mark.parametrize("swap", [0, 1])
def test_every_single_cta_kernel(block_n, stream_k, swap):
    # 520 x 776 x 1352: ragged in every dimension, several tiles, K not a multiple of 64.
    ov = dict(cta_group=1, block_n=block_n, swap=swap, stream_k=stream_k)
    stats, cfg = run_case(520, 776, 1352, override=ov)
    # 256-wide tiles exist with the TMA-store epilogue only; direct stores cap at 128 columns
    want = block_n if (block_n < 256 or (swap == 0 and stream_k == 0)) else 128
    assert cfg["block_n"] == want and cfg["swap"] == swap, cfg
    run_case(520, 776, 1352, override=ov, col_major=True)


def test_tma_store_kernels_on_aligned_output():
    for bn in (256, 128):
        stats, cfg = run_case(640, 1024, 704, override=dict(cta_group=1, block_n=bn, swap=0))
        assert cfg["block_n"] == bn and cfg["stages"] in (4, 6)


def test_stream_k_with_few_ctas_has_many_contributors():
    # 3 tiles of 128 rows, 64 k-blocks, 7 CTAs -> ranges cut tiles in several places.
    for ctas in (2, 5, 7, 148):
        ov = dict(cta_group=1, block_n=32, swap=1, stream_k=1, max_ctas=ctas)
        run_case(24, 384, 4096, override=ov)


def test_raster_group_heights():
    for g in (1, 3, 8, 64):
        run_case(1408, 1280, 256, override=dict(group_m=g))


def test_unscaled_operands_like_the_reference_driver():
    # benchmark.py:10-11: N(0,1) operands at 1024^3, outputs of magnitude ~32.
    run_case(1024, 1024, 1024, scale_by_k=False, col_major=True)


def test_padded_leading_dimensions():
    M, N, K = 300, 264, 328
    A, B = make_problem(M, N, K, seed=77)
    big_a = torch.zeros(M, K + 40, dtype=torch.bfloat16, device="cuda")
    big_b = torch.zeros(N, K + 8, dtype=torch.bfloat16, device="cuda")
    big_a[:, :K] = A.cuda()
    big_b[:, :K] = B.cuda()
    big_a[:, K:] = 7.0  # must never be read
    big_b[:, K:] = -9.0
    big_c = torch.full((M, N + 24), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = ops.matmul(big_a[:, :K], big_b[:, :K], out=big_c[:, :N])
    torch.cuda.synchronize()
    oracle.assert_parity(out, oracle.gemm_fp32(A, B), "padded lda/ldb/ldc")
    assert torch.isnan(big_c[:, N:]).all(), "columns beyond N were written"


def test_unaligned_row_pitch_of_c_uses_direct_stores():
    M, N, K = 257, 250, 128   # ldc = 250: not a multiple of 8 -> no TMA store
    stats, cfg = run_case(M, N, K)
    run_case(M, N, K, col_major=True)


def test_guard_bands_around_c_stay_untouched():
    M, N, K = 200, 328, 192
    A, B = make_problem(M, N, K, seed=5)
    pad = 4096
    flat = torch.full((pad + M * N + pad,), float("nan"), dtype=torch.bfloat16, device="cuda")
    flat[:pad] = 123.0
    flat[pad + M * N:] = 321.0
    C = flat[pad:pad + M * N].view(M, N)
    ops.matmul(A.cuda(), B.cuda(), out=C)
    torch.cuda.synchronize()
    assert (flat[:pad] == 123.0).all() and (flat[pad + M * N:] == 321.0).all()
    oracle.assert_parity(C, oracle.gemm_fp32(A, B), "guard bands")


def test_repeated_launches_are_bit_identical():
    for (M, N, K) in [(1024, 1536, 2048), (64, 28672, 8192)]:
        A, B = make_problem(M, N, K, seed=8)
        dA, dB = A.cuda(), B.cuda()
        first = ops.matmul(dA, dB).clone()
        for _ in range(10):
            again = ops.matmul(dA, dB)
            assert torch.equal(first.view(torch.int16), again.view(torch.int16))
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


def test_k_zero_writes_zeros_and_empty_is_a_noop():
    A = torch.zeros(8, 0, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(16, 0, dtype=torch.bfloat16, device="cuda")
    out = torch.full((8, 16), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.matmul(A, B, out=out)
    torch.cuda.synchronize()
    assert (out == 0).all()
    ops.matmul(torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda"),
               torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda"))


def test_unsupported_k_raises():
    A = torch.zeros(8, 12, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(8, 12, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.NeoGemmError) as e:
        ops.matmul(A, B)
    assert e.value.code == 2


def test_host_entry_point_round_trip():
    M, N, K = 384, 520, 256
    A, B = make_problem(M, N, K, seed=21)
    C = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    ops.matmul_host(A.pin_memory(), B.pin_memory(), C)
    oracle.assert_parity(C, oracle.gemm_fp32(A, B), "host entry")
    Cc = torch.empty(N, M, dtype=torch.bfloat16)
    ops.matmul_host(A, B, Cc, col_major=True)   # pageable memory works too
    oracle.assert_parity(Cc.t(), oracle.gemm_fp32(A, B), "host entry column-major")


def test_host_entry_point_pipelines_large_operands():
    # More than 1024 stored rows: the upload goes in row chunks, one product launch per chunk,
    # results return while the next chunk is still going up.  Ragged last chunk on purpose.
    M, N, K = 4000, 1032, 520
    A, B = make_problem(M, N, K, seed=23)
    ref = oracle.gemm_fp32(A, B)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    ops.matmul_host(A.pin_memory(), B.pin_memory(), C)
    oracle.assert_parity(C, ref, "host entry, chunked rows of A")
    Cc = torch.full((N, M), float("nan"), dtype=torch.bfloat16).pin_memory()
    ops.matmul_host(A.pin_memory(), B.pin_memory(), Cc, col_major=True)   # chunks run over B
    oracle.assert_parity(Cc.t(), ref, "host entry column-major, chunked rows of B")
    assert ops.device_status()[0] == 0


def test_runs_on_a_side_stream():
    A, B = make_problem(512, 768, 512, seed=31)
    dA, dB = A.cuda(), B.cuda()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        out = ops.matmul(dA, dB)
    s.synchronize()
    oracle.assert_parity(out, oracle.gemm_fp32(A, B), "side stream")


def test_linear_layout():
    x = (torch.randn(3, 5, 256, generator=torch.Generator().manual_seed(2)) / 16).to(torch.bfloat16)
    w = (torch.randn(136, 256, generator=torch.Generator().manual_seed(3)) / 16).to(torch.bfloat16)
    y = ops.linear(x.cuda(), w.cuda())
    assert y.shape == (3, 5, 136)
    oracle.assert_parity(y.reshape(-1, 136), oracle.gemm_fp32(x.reshape(-1, 256), w), "linear")


def test_golden_fixtures_on_the_gpu():
    import glob, os
    files = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "gemm_*.npz")))
    assert files
    for f in files:
        z = np.load(f)
        A = torch.from_numpy(z["A_bits"]).view(torch.bfloat16)
        B = torch.from_numpy(z["B_bits"]).view(torch.bfloat16)
        want = torch.from_numpy(z["C_bits"]).view(torch.bfloat16)
        got = ops.matmul(A.cuda(), B.cuda()).cpu()
        s = oracle.compare(got, want.float())
        # the fixture is already rounded, so compare bf16 to bf16: at most one ulp apart
        assert s["max_ulp"] <= 1 and s["near_zero_ok"] and s["bit_equal_frac"] >= 0.98, (f, s)


def test_torch_extension_module_matches_reference_usage():
    # The flow of the reference's benchmark.py:10-25 with the extension built by setup.py.
    neoGEMM = pytest.importorskip("neoGEMM")
    M, N, K = 1024, 1024, 1024
    A, B = make_problem(M, N, K, seed=41, scale_by_k=False)
    tA, tB = A.cuda(), B.cuda()
    tC = torch.zeros(M, N, device="cuda").to(torch.bfloat16)
    assert neoGEMM.neoGemmV1(tA, tB, tC) is None
    tC = tC.t()
    torch.cuda.synchronize()
    oracle.assert_parity(tC, oracle.gemm_fp32(A, B), "neoGEMM.neoGemmV1")
    tC2 = torch.zeros(M, N, device="cuda").to(torch.bfloat16)
    neoGEMM.neogemm(A=tA, B=tB, C=tC2)
    assert torch.equal(tC2.t().contiguous().view(torch.int16), tC.contiguous().view(torch.int16))
    oracle.assert_parity(neoGEMM.matmul(tA, tB), oracle.gemm_fp32(A, B), "neoGEMM.matmul")
    with pytest.raises(RuntimeError):
        neoGEMM.neoGemmV1(tA.float(), tB, tC2)


def test_device_status_is_clean_after_all_of_the_above():
    torch.cuda.synchronize()
    assert ops.device_status() == (0, 0, 0, 0)


@pytest.mark.parametrize("case", [
    ((16, 3584, 8192), None, None),            # default: one run-time piece per tile
    ((64, 3584, 4096), 2, None),
    ((128, 2048, 8192), 4, None),
    ((24, 1000, 4096), 3, 5),                  # ragged tiles, few CTAs, many claims each
    ((32, 28672, 8192), 1, None),
])
def test_dynamic_tail_pool(case):
    # The last k-blocks of every tile are claimed at run time; who computes them varies from
    # launch to launch, the bits must not.
    (M, N, K), pieces, ctas = case
    tuning = {"two_ctas_per_sm": 0}
    if pieces is not None:
        tuning["dynamic_pieces_per_tile"] = pieces
    ov = dict(stream_k=1, swap=1, max_ctas=ctas) if ctas else None
    stats, cfg = run_case(M, N, K, tuning=tuning, override=ov)
    assert cfg["stream_k"] == 1 and cfg["swap"] == 1, cfg
    A, B = make_problem(M, N, K, seed=99)
    dA, dB = A.cuda(), B.cuda()
    for key, value in tuning.items():
        ops.set_tuning(key, value)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(8):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    finally:
        for key in tuning:
            ops.set_tuning(key, -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


def test_bounded_wait_expires_into_an_error_code_and_the_library_recovers():
    # Failure detection without a fault: a wait on a barrier nothing completes must run out,
    # leave an error record, make later launches fail loudly - and clearing the record must bring
    # everything back, on the same CUDA context.
    import ctypes
    from gemm_b200._lib import lib
    lib.neogemm_debug_wait_expiry.restype = ctypes.c_int
    lib.neogemm_debug_wait_expiry.argtypes = [ctypes.c_uint, ctypes.POINTER(ctypes.c_ulonglong)]
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    waited = ctypes.c_ulonglong(0)
    assert lib.neogemm_debug_wait_expiry(2000, ctypes.byref(waited)) == 0      # 2 ms limit
    assert 2_000_000 <= waited.value < 50_000_000, waited.value
    code, cta, segment, aux = ops.device_status()
    assert (code, cta, segment, aux) == (4, 0, -1, -1)
    A, B = make_problem(128, 128, 64, seed=1)
    with pytest.raises(ops.NeoGemmError) as e:
        ops.matmul(A.cuda(), B.cuda())
    assert e.value.code == 5            # NEOGEMM_ERR_DEVICE_TIMEOUT: sticky until cleared
    ops.clear_device_status()
    assert ops.device_status() == (0, 0, 0, 0)
    run_case(128, 128, 64)              # same context, same library: works again


@pytest.mark.parametrize("shape", [(512, 512, 8192), (256, 256, 4096), (300, 520, 4104)])
def test_handful_of_tiles_under_long_k(shape):
    # with the two-pass split-K switched off: 64-column direct-store tiles, last arriver sums
    stats, cfg = run_case(*shape, tuning={"two_pass_split_k": 0})
    assert (cfg["block_n"], cfg["stream_k"]) == (64, 1), cfg
    run_case(*shape, col_major=True, tuning={"two_pass_split_k": 0})


@pytest.mark.parametrize("shape", [(1024, 1024, 8192), (512, 512, 8192), (256, 256, 4096),
                                   (300, 520, 4104), (1536, 1024, 3072), (1000, 1016, 2056),
                                   (640, 2048, 4096)])
def test_two_pass_split_k(shape):
    # Few wide tiles under a long K: every tile cut into k-chunks, partials summed, rounded and
    # stored by the reduction kernel behind the GEMM.  Ragged edges, both layouts, and the same
    # bits launch after launch.
    stats, cfg = run_case(*shape)
    picked = shape in ((1024, 1024, 8192), (512, 512, 8192), (256, 256, 4096), (300, 520, 4104))
    if picked:   # the launcher cuts these on its own; the others only where forced below
        assert cfg["stream_k"] == 1 and cfg["ctas"] > cfg["tiles"] * cfg["cta_group"], cfg
    run_case(*shape, col_major=True)
    A, B = make_problem(*shape, seed=9)
    dA, dB = A.cuda(), B.cuda()
    first = ops.matmul(dA, dB).clone()
    for _ in range(4):
        assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
    # forced for every TMA-store kernel family
    for ov in (dict(cta_group=1, block_n=256), dict(cta_group=1, block_n=128),
               dict(cta_group=2, block_n=128), dict(cta_group=2, block_n=256)):
        stats, cfg = run_case(*shape, override=dict(stream_k=1, **ov))
        if cfg["tiles"] * 2 <= 148 // cfg["cta_group"] and shape[2] >= 1024:
            assert cfg["stream_k"] == 1, cfg
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


def test_cuda_graph_replays_of_every_launch_kind():
    # A captured graph of back-to-back launches (data-parallel, cut last wave, two-pass split-K
    # with its reduction kernel, tall tiles, stream-K) where each launch's set-up overlaps the
    # previous kernel's tail: replays must give the oracle's result every time, and a chained
    # pair (the second product reads the first one's output) must see complete data.
    shapes = [(1024, 768, 512), (4096, 4096, 1024), (1024, 1024, 4096), (48, 20000, 1024),
              (16, 3584, 2048)]
    problems = [make_problem(*s, seed=30 + i) for i, s in enumerate(shapes)]
    dev = [(a.cuda(), b.cuda()) for a, b in problems]
    outs = [torch.empty((s[0], s[1]), dtype=torch.bfloat16, device="cuda") for s in shapes]
    # chain: D = (A0 B0^T) W^T with W [256, 768]
    W = (torch.randn(256, 768, generator=torch.Generator().manual_seed(5)) / 768 ** 0.5) \
        .to(torch.bfloat16)
    dW = W.cuda()
    chained = torch.empty((1024, 256), dtype=torch.bfloat16, device="cuda")

    def launches():
        for (dA, dB), out in zip(dev, outs):
            ops.matmul(dA, dB, out=out)
        ops.matmul(outs[0], dW, out=chained)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launches()                       # workspace, attributes, tensor maps: before the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launches()
    for replay in range(3):
        for out in outs:
            out.fill_(float("nan"))
        chained.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.device_status()[0] == 0
        for s, (A, B), out in zip(shapes, problems, outs):
            oracle.assert_parity(out, oracle.gemm_fp32(A, B), f"graph replay {replay} {s}")
        oracle.assert_parity(chained, oracle.gemm_fp32(outs[0].cpu(), W),
                             f"chained product, replay {replay}")


@pytest.mark.parametrize("shape", [(512, 512, 512), (1024, 1024, 1024), (520, 776, 264),
                                   (300, 1000, 1352), (128, 136, 64), (1024, 768, 512),
                                   (640, 1024, 704), (200, 328, 72)])
def test_narrow_tiles_for_small_problems(shape):
    # 128 x 64 TMA-store tiles (eight ring slots): picked when 128 x 128 tiles would leave half of
    # the SMs idle, forced here for the rest; both layouts, ragged edges, fp32 result, repeats.
    stats, wide = run_case(*shape, tuning={"narrow_tiles": 0})
    assert wide["block_n"] >= 128 or wide["swap"] == 1, wide
    stats, cfg = run_case(*shape, tuning={"narrow_tiles": 1})
    if (wide["cta_group"], wide["block_n"], wide["swap"]) == (1, 128, 0):
        assert (cfg["cta_group"], cfg["block_n"], cfg["stages"]) == (1, 64, 8), cfg
    else:   # another kernel family was the choice: the knob leaves it alone
        assert cfg["block_n"] == wide["block_n"], (cfg, wide)
    run_case(*shape, tuning={"narrow_tiles": 1}, col_major=True)
    A, B = make_problem(*shape, seed=12)
    dA, dB = A.cuda(), B.cuda()
    ops.set_tuning("narrow_tiles", 1)
    try:
        first = ops.matmul(dA, dB).clone()
        for _ in range(4):
            assert torch.equal(first.view(torch.int16), ops.matmul(dA, dB).view(torch.int16))
        out32 = ops.matmul_fused(dA, dB, out_dtype=torch.float32)
        assert torch.equal(out32.to(torch.bfloat16).view(torch.int16), first.view(torch.int16))
    finally:
        ops.set_tuning("narrow_tiles", -1)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0


def test_small_benchmark_shape_takes_narrow_tiles():
    stats, cfg = run_case(512, 512, 512)
    assert (cfg["block_n"], cfg["ctas"]) == (64, 32), cfg
