"""GPU parity of (batched) GEMM through the C ABI against the CPU oracle (the compiled reference when
it is present, else the C restatement), on seeded inputs at sizes the oracle finishes in seconds."""
import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi, workloads
from intel_gaudi3_software_b200.abi import make_tensor as T
import util
from golden.make_golden import GEMM_CASES

pytestmark = pytest.mark.gpu


def run_case(calc, oracle, M, N, K, op=abi.OP_AB, batch=(), x_batch=None, w_batch=None, seed=0, x_pitch=0, o_pitch=0):
    rng = np.random.default_rng(seed)
    tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
    xb_dims = list(batch if x_batch is None else x_batch)
    wb_dims = list(batch if w_batch is None else w_batch)
    xs = ([M, K] if tA else [K, M]) + xb_dims
    ws = ([K, N] if tB else [N, K]) + wb_dims
    os_ = [N, M] + list(batch)
    xstr = None
    if x_pitch:
        xstr = [1, xs[0] + x_pitch]
        for d in range(2, len(xs)):
            xstr.append(xstr[-1] * xs[d - 1])
    ostr = None
    if o_pitch:
        ostr = [1, N + o_pitch]
        for d in range(2, len(os_)):
            ostr.append(ostr[-1] * os_[d - 1])
    nx = (xstr[-1] * xs[-1]) if xstr else int(np.prod(xs))
    no = (ostr[-1] * os_[-1]) if ostr else int(np.prod(os_))
    xb, wb = util.gen_bf16(rng, nx), util.gen_bf16(rng, int(np.prod(ws)))
    x, w = T(xb, abi.BF16, xs, xstr), T(wb, abi.BF16, ws)
    o1, o2 = np.full(no, 7.0, np.float32), np.full(no, 7.0, np.float32)
    calc.do_batch_gemm(T(o1, abi.FP32, os_, ostr), x, w, op)
    assert oracle.bgemm(T(o2, abi.FP32, os_, ostr), x, w, op) == 0
    # tolerance scale: sum|a||b| <= K since |a|,|b| <= 1; use the exact per-element bound where cheap
    d = np.abs(o1.astype(np.float64) - o2.astype(np.float64))
    assert d.max() <= util.ACC_TOL * K, (M, N, K, op, d.max())
    # and tighter, against the typical magnitude: mean sum|ab| ~ K/4 for U[-1,1]
    assert d.max() <= util.ACC_TOL * K / 4
    if o_pitch:  # holes of a strided output stay untouched
        rows = o1.reshape(-1, N + o_pitch)
        assert (rows[:, N:] == 7.0).all()
    return o1, o2


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 512), (256, 512, 128), (100, 72, 40), (1, 5, 5), (5, 1, 5),
                                   (7, 9, 1), (129, 257, 65), (384, 640, 1000), (64, 64, 8192)])
def test_shapes(calc, best_oracle, M, N, K):
    run_case(calc, best_oracle, M, N, K)


KERNEL_VARIANTS = {
    "pair, four epilogue warps": {"pair": 1, "epi_groups": 1},
    "pair, eight epilogue warps": {"pair": 1, "epi_groups": 2},
    "pair, split-K": {"pair": 1, "split_k": 3},
    "pair, 224-wide tiles": {"pair": 1, "tile_n": 224},
    "pair, 160-wide tiles, eight epilogue warps": {"pair": 1, "tile_n": 160, "epi_groups": 2},
    "pair, 96-wide tiles": {"pair": 1, "tile_n": 96},
    "pair, stream-K tail": {"pair": 1, "split_k": 1, "stream_k": 1},
    "pair, stream-K tail, eight epilogue warps, direct stores": {"pair": 1, "split_k": 1, "stream_k": 1, "epi_groups": 2, "tma_store": 0},
    "single CTA, 256 wide": {"pair": 0},
    "single CTA, 128 wide": {"block_n": 128},
    "single CTA, no TMA stores": {"pair": 0, "tma_store": 0},
}


@pytest.mark.parametrize("variant", sorted(KERNEL_VARIANTS))
def test_every_kernel_variant_matches_the_oracle(calc, best_oracle, variant):
    """The tile geometry is picked per problem; the context's tuning knobs force each form on the same problems."""
    knobs = KERNEL_VARIANTS[variant]
    try:
        for k, v in knobs.items():
            calc.set_option(k, v)
        run_case(calc, best_oracle, 512, 768, 520, abi.OP_AB, seed=3)
        run_case(calc, best_oracle, 300, 260, 200, abi.OP_ABT, seed=4)
        run_case(calc, best_oracle, 256, 256, 96, abi.OP_ATB, batch=(3, 2), w_batch=(1, 2), seed=5)
        run_case(calc, best_oracle, 384, 520, 72, abi.OP_ATBT, o_pitch=8, seed=6)
    finally:
        for k in knobs:
            calc.set_option(k, -1)


@pytest.mark.parametrize("M,N,K,op,batch", [(512, 768, 2048, abi.OP_AB, ()), (1024, 512, 1536, abi.OP_ATB, ()), (300, 700, 1100, abi.OP_ABT, ()),
                                             (256, 256, 1024, abi.OP_AB, (3,)), (2560, 2048, 1024, abi.OP_AB, ())])
def test_stream_k_tail(calc, best_oracle, M, N, K, op, batch):
    """Tiles of a ragged last wave are cut along K into slices that go round the CTA pairs; the pair with a tile's first slice
    adds the others' partial sums: against the oracle, equal run to run, and within the accumulation tolerance of the uncut
    launch. The last shape has whole tiles (80 on 74 pairs) besides the cut ones."""
    try:
        calc.set_option("pair", 1)
        calc.set_option("split_k", 1)
        calc.set_option("stream_k", 1)
        cut, _ = run_case(calc, best_oracle, M, N, K, op, batch=batch, seed=11)
        again, _ = run_case(calc, best_oracle, M, N, K, op, batch=batch, seed=11)
        calc.set_option("stream_k", 0)
        whole, _ = run_case(calc, best_oracle, M, N, K, op, batch=batch, seed=11)
    finally:
        calc.set_option("pair", -1)
        calc.set_option("split_k", -1)
        calc.set_option("stream_k", -1)
    assert (cut.view(np.uint32) == again.view(np.uint32)).all()
    assert (cut != whole).any()        # the summation order differs, so some last bits do
    assert np.abs(cut.astype(np.float64) - whole).max() <= util.ACC_TOL * K / 4


def test_stream_k_tail_at_the_sharded_headline_shape(calc):
    """1024 x 8192 x 8192 fp8 -> bf16 (one rank's rows of the 8192^3 product on eight GPUs): 128 tiles on 74 pairs, the last
    54 cut into four slices each. Against the uncut launch: bf16 outputs equal or one step apart."""
    rng = np.random.default_rng(5)
    M, N, K = 1024, 8192, 8192
    a = workloads.quantise_fp8(rng.standard_normal(M * K).astype(np.float32), abi.FP8_143, 7)
    b = workloads.quantise_fp8(rng.standard_normal(N * K).astype(np.float32), abi.FP8_143, 7)
    outs = []
    for knob in (1, 0):
        calc.set_option("stream_k", knob)
        calc.set_option("host_pipeline", 0)   # one launch over all 1024 rows, not a pipeline of row blocks
        try:
            o = np.zeros(M * N, np.uint16)
            calc.do_batch_gemm(T(o, abi.BF16, [N, M]), T(a, abi.FP8_143, [K, M], fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL),
                               T(b, abi.FP8_143, [K, N], fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL), abi.OP_ABT,
                               cast=abi.make_cast_params(abi.RM_NE))
            outs.append(o)
        finally:
            calc.set_option("stream_k", -1)
            calc.set_option("host_pipeline", -1)
    cut, whole = (workloads.bf16_to_f32(o) for o in outs)
    differ = outs[0] != outs[1]
    assert 0 < differ.mean() < 0.02, differ.mean()
    # one bf16 step apart at most (values next to zero may differ in sign: an absolute allowance far below the outputs' spread)
    assert (np.abs(cut - whole) <= np.maximum(np.abs(cut), np.abs(whole)) * 2.0 ** -7 + 1e-4 * whole.std()).all()


@pytest.mark.parametrize("op", [abi.OP_AB, abi.OP_ABT, abi.OP_ATB, abi.OP_ATBT])
def test_operand_orientations(calc, best_oracle, op):
    run_case(calc, best_oracle, 256, 384, 192, op)
    run_case(calc, best_oracle, 136, 72, 104, op, seed=1)
    run_case(calc, best_oracle, 61, 35, 77, op, seed=2)  # rows not 16-byte aligned: repacked on the device


@pytest.mark.parametrize("op", [abi.OP_AB, abi.OP_ABT, abi.OP_ATB, abi.OP_ATBT])
def test_batched_with_broadcast_and_strides(calc, best_oracle, op):
    run_case(calc, best_oracle, 64, 128, 64, op, batch=(3, 2))
    run_case(calc, best_oracle, 40, 24, 72, op, batch=(3, 2, 2), x_batch=(3, 1, 2), w_batch=(1, 2, 2), seed=3)
    run_case(calc, best_oracle, 40, 24, 72, op, batch=(2,), seed=4, x_pitch=8, o_pitch=4)
    run_case(calc, best_oracle, 13, 10, 21, op, batch=(3, 2, 2), x_batch=(3, 1, 2), w_batch=(1, 2, 2), seed=5, x_pitch=3, o_pitch=2)


def test_golden_bf16_all_chip_models(calc, golden):
    """The committed outputs of the reference for its three chip models: the GPU must be within the
    accumulator tolerance of each (the models differ from one another by less than that)."""
    for i, (M, N, K, op, batch) in enumerate(GEMM_CASES):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xs = ([M, K] if tA else [K, M]) + list(batch)
        ws = ([K, N] if tB else [N, K]) + list(batch)
        for chip in (0, 1, 2):
            c = pkg.Calculator(chip=chip)
            o = np.zeros(golden["gemm%d_chip%d" % (i, chip)].size, np.float32)
            c.do_batch_gemm(T(o, abi.FP32, [N, M] + list(batch)), T(golden["gemm%d_x" % i], abi.BF16, xs), T(golden["gemm%d_w" % i], abi.BF16, ws), op)
            c.close()
            assert np.abs(o - golden["gemm%d_chip%d" % (i, chip)]).max() <= util.ACC_TOL * K / 4, (i, chip)


def test_known_answers(calc, port):
    # mme/tests/unit_tests/mme_unit_test.cpp:67-172: 1x5 . 5x1 of tens = 500 (fp32 and bf16), 5x5 = 250
    ten = np.full(5, 10.0, np.float32)
    y = np.zeros(1, np.float32)
    calc.do_batch_gemm(T(y, abi.FP32, [1, 1]), T(ten, abi.FP32, [5, 1]), T(ten, abi.FP32, [1, 5]), abi.OP_AB)
    assert y[0] == 500.0
    tb = port.fp32_to_bf16(ten)
    calc.do_batch_gemm(T(y, abi.FP32, [1, 1]), T(tb, abi.BF16, [5, 1]), T(tb, abi.BF16, [1, 5]), abi.OP_AB)
    assert y[0] == 500.0
    a, b = np.full(25, 10.0, np.float32), np.full(25, 5.0, np.float32)
    acc = np.zeros(25, np.float32)
    calc.do_batch_gemm(T(acc, abi.FP32, [5, 5]), T(a, abi.FP32_IEEE, [5, 5]), T(b, abi.FP32_IEEE, [5, 5]), abi.OP_AB)
    assert (acc == 250.0).all()
    out = np.zeros(25, np.uint16)
    calc.do_batch_gemm(T(out, abi.BF16, [5, 5]), T(port.fp32_to_bf16(a), abi.BF16, [5, 5]), T(port.fp32_to_bf16(b), abi.BF16, [5, 5]),
                       abi.OP_AB, abi.make_cast_params())
    assert (util.bf16_to_f32(out) == 250.0).all()
    # fp8 two-element dot products (:425-447, :498-519)
    for dt, ew, bias, va, vb in ((abi.FP8_143, 4, 7, 0.25, -0.5), (abi.FP8_152, 5, 15, 0.5, -0.5)):
        xa = np.repeat(port.fp32_to_fp8(np.array([va], np.float32), ew, bias), 2)
        xb = np.repeat(port.fp32_to_fp8(np.array([vb], np.float32), ew, bias), 2)
        calc.do_batch_gemm(T(y, abi.FP32, [1, 1]), T(xa, dt, [2, 1], fp_bias=bias), T(xb, dt, [1, 2], fp_bias=bias), abi.OP_AB)
        assert y[0] == np.float32(2 * va * vb)


FP8_CASES = [(9, 9, 7, 7, 2, 2), (9, 9, 7, 11, 2, 2), (9, 9, 3, 15, 2, 2), (10, 9, 15, 7, 0, 2), (9, 10, 3, 20, 2, 0),
             (10, 10, 15, 1, 0, 0), (9, 9, 15, 15, 0, 0), (9, 9, 7, 7, 1, 1), (10, 10, 15, 15, 1, 2), (9, 10, 11, 30, 0, 1)]


@pytest.mark.parametrize("tx,tw,bx,bw,mx,mw", FP8_CASES)
def test_fp8_all_formats_biases_and_infnan_modes(calc, best_oracle, port, tx, tw, bx, bw, mx, mw):
    """Random code bytes (every code occurs, including the ones that mean Inf/NaN in some modes)."""
    rng = np.random.default_rng(tx * 100 + bw)
    M, N, K = 96, 160, 320
    xb, wb = rng.integers(0, 256, M * K).astype(np.uint8), rng.integers(0, 256, K * N).astype(np.uint8)
    for tame in (True, False):
        if tame:  # clear the top exponent bit: finite, moderate values
            xa, wa = xb & 0xBF, wb & 0xBF
        else:
            xa, wa = xb, wb
        x, w = T(xa, tx, [K, M], fp_bias=bx, inf_nan_mode=mx), T(wa, tw, [N, K], fp_bias=bw, inf_nan_mode=mw)
        o, r = np.zeros(M * N, np.float32), np.zeros(M * N, np.float32)
        calc.do_batch_gemm(T(o, abi.FP32, [N, M]), x, w, abi.OP_AB)
        assert best_oracle.bgemm(T(r, abi.FP32, [N, M]), x, w, abi.OP_AB) == 0
        assert (np.isnan(o) == np.isnan(r)).all()
        fin = np.isfinite(r)
        assert (np.isinf(o) == np.isinf(r))[~np.isnan(r)].all() or not tame
        xf, wf = util.decode(xa, tx, bx, mx, port).reshape(M, K), util.decode(wa, tw, bw, mw, port).reshape(K, N)
        sabs = np.abs(np.nan_to_num(xf, nan=0, posinf=0, neginf=0)).astype(np.float64) @ np.abs(np.nan_to_num(wf, nan=0, posinf=0, neginf=0)).astype(np.float64)
        ok = fin.reshape(M, N) & np.isfinite(o).reshape(M, N)
        err = util.acc_error(np.where(ok, o.reshape(M, N), 0), np.where(ok, r.reshape(M, N), 0), sabs)
        assert err <= util.ACC_TOL, (tame, err)


def test_foreign_code_decision_stays_on_the_device(calc, best_oracle, port):
    """fp8_143 in the reference's default 'full' Inf/NaN convention holds codes (0x78 ...) that the tensor cores would read
    as numbers. Whether a tensor holds one is found by a scan ON the stream, and both forms of the GEMM are enqueued behind
    it: a call on device tensors must return while work enqueued before it is still running (no host round trip), and both
    outcomes must match the oracle."""
    import time
    rng = np.random.default_rng(77)
    M, N, K = 512, 512, 512
    kw = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_FULL)
    clean = (rng.integers(0, 256, M * K).astype(np.uint8) & 0xBF, rng.integers(0, 256, K * N).astype(np.uint8) & 0xBF)
    dirty = (clean[0].copy(), clean[1].copy())
    dirty[0][12345] = 0x78          # +Inf in this convention, 256 to the tensor cores
    dirty[1][54321] = 0x7D          # NaN in this convention
    # long-running work on the same stream: a bit-exact GEMM on the CUDA cores
    big = 3072
    bx, bw, bo = calc.to_device(rng.integers(0, 120, big * big).astype(np.uint8)), calc.to_device(rng.integers(0, 120, big * big).astype(np.uint8)), calc.alloc(big * big * 4)
    kn = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL, mem_space=abi.MEM_DEVICE)
    for xa, wa in (clean, dirty):
        dx, dw, do = calc.to_device(xa), calc.to_device(wa), calc.alloc(M * N * 4)
        # warm-up: the first call of a shape may grow the context's scratch arena (an allocation synchronises the device)
        calc.do_batch_gemm(T(do.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), T(dx.ptr, abi.FP8_143, [K, M], mem_space=abi.MEM_DEVICE, **kw),
                           T(dw.ptr, abi.FP8_143, [N, K], mem_space=abi.MEM_DEVICE, **kw), abi.OP_AB)
        calc.sync()
        calc.set_accumulation(abi.ACC_CHIP_EXACT)
        try:
            t0 = time.perf_counter()
            calc.do_batch_gemm(T(bo.ptr, abi.FP32, [big, big], mem_space=abi.MEM_DEVICE), T(bx.ptr, abi.FP8_143, [big, big], **kn),
                               T(bw.ptr, abi.FP8_143, [big, big], **kn), abi.OP_AB)
        finally:
            calc.set_accumulation(abi.ACC_TENSOR_CORE)
        calc.do_batch_gemm(T(do.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), T(dx.ptr, abi.FP8_143, [K, M], mem_space=abi.MEM_DEVICE, **kw),
                           T(dw.ptr, abi.FP8_143, [N, K], mem_space=abi.MEM_DEVICE, **kw), abi.OP_AB)
        t_enqueued = time.perf_counter() - t0
        calc.sync(30_000_000_000)
        t_done = time.perf_counter() - t0
        assert t_done > 0.02 and t_enqueued < 0.5 * t_done, (t_enqueued, t_done)   # the call came back long before the stream drained
        o = do.download(np.float32)
        r = np.zeros(M * N, np.float32)
        assert best_oracle.bgemm(T(r, abi.FP32, [N, M]), T(xa, abi.FP8_143, [K, M], **kw), T(wa, abi.FP8_143, [N, K], **kw), abi.OP_AB) == 0
        assert (np.isnan(o) == np.isnan(r)).all() and (np.isinf(o) == np.isinf(r)).all()
        fin = np.isfinite(r)
        xf, wf = util.decode(xa, abi.FP8_143, 7, 0, port).reshape(M, K), util.decode(wa, abi.FP8_143, 7, 0, port).reshape(K, N)
        sabs = np.abs(np.nan_to_num(xf, nan=0, posinf=0, neginf=0)).astype(np.float64) @ np.abs(np.nan_to_num(wf, nan=0, posinf=0, neginf=0)).astype(np.float64)
        assert util.acc_error(np.where(fin, o, 0).reshape(M, N), np.where(fin, r, 0).reshape(M, N), sabs) <= util.ACC_TOL
        for b in (dx, dw, do):
            b.free()
    assert np.isnan(o).any() and np.isinf(o).any()      # the second pass did go through the decoded form
    for b in (bx, bw, bo):
        b.free()


def test_fp8_same_type_is_bit_identical_to_the_reference_model(calc, best_oracle, port):
    """fp8 x fp8 products are exact in fp32 and short sums stay exact: for in-range values the
    tensor-core accumulation and the reference's tree agree bit for bit at K = 128 (the attention-shaped batch)."""
    rng = np.random.default_rng(8)
    M, N, K = 128, 256, 128
    xb, wb = util.gen_fp8(rng, M * K, port), util.gen_fp8(rng, K * N, port)
    x, w = T(xb, abi.FP8_143, [K, M], fp_bias=7, inf_nan_mode=2), T(wb, abi.FP8_143, [K, N], fp_bias=7, inf_nan_mode=2)
    o, r = np.zeros(M * N, np.float32), np.zeros(M * N, np.float32)
    calc.do_batch_gemm(T(o, abi.FP32, [N, M]), x, w, abi.OP_ABT)
    assert best_oracle.bgemm(T(r, abi.FP32, [N, M]), x, w, abi.OP_ABT) == 0
    assert (np.abs(o - r) <= util.ACC_TOL * 448 * 448 * K).all()
    assert (o.view(np.uint32) == r.view(np.uint32)).mean() > 0.99


def test_fp32_and_tf32_operands_against_golden(calc, golden):
    M, N, K = 16, 24, 40
    xf, wf = golden["f32gemm_x"], golden["f32gemm_w"]
    sabs = util.sum_abs_products(xf.reshape(M, K), wf.reshape(K, N))
    for dt, nm, tol in ((abi.FP32, "fp32", util.ACC_TOL), (abi.TF32, "tf32", util.ACC_TOL)):
        o = np.zeros(M * N, np.float32)
        calc.do_batch_gemm(T(o, abi.FP32, [N, M]), T(xf, dt, [K, M]), T(wf, dt, [N, K]), abi.OP_AB)
        assert util.acc_error(o.reshape(M, N), golden["f32gemm_" + nm].reshape(M, N), sabs) <= tol, nm


def test_fused_cast_matches_unfused(calc, port):
    """bgemm with cast parameters == bgemm to fp32 followed by doActivation, for every output type
    and deterministic rounding mode (same accumulator bits, same cast code)."""
    rng = np.random.default_rng(12)
    M, N, K = 200, 264, 136
    xb, wb = util.gen_bf16(rng, M * K), util.gen_bf16(rng, K * N)
    x, w = T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K])
    acc = np.zeros(M * N, np.float32)
    calc.do_batch_gemm(T(acc, abi.FP32, [N, M]), x, w, abi.OP_AB)
    for od, bias, mode in ((abi.BF16, 0, 0), (abi.FP8_143, 7, 2), (abi.FP8_152, 15, 0), (abi.FP32, 0, 0)):
        for rm in (0, 1, 2, 3, 6):
            for relu in (0, 1):
                cp = abi.make_cast_params(rm, relu, clip_fp=True)
                fused = np.zeros(M * N, abi.NP_DTYPE[od])
                calc.do_batch_gemm(T(fused, od, [N, M], fp_bias=bias, inf_nan_mode=mode), x, w, abi.OP_AB, cp)
                two = np.zeros(M * N, abi.NP_DTYPE[od])
                calc.do_activation(T(two, od, [N, M], fp_bias=bias, inf_nan_mode=mode), T(acc.copy(), abi.FP32, [N, M]), cp)
                assert (fused.view(np.uint8) == two.view(np.uint8)).all(), (od, rm, relu)
    # counter-based stochastic rounding: the fused epilogue draws the words the cast kernel draws, at a stream position
    # that is a multiple of four (one Philox block per four elements) and at one that is not; flush flags on and off
    for od, bias, mode in ((abi.BF16, 0, 0), (abi.FP8_143, 7, 2), (abi.FP8_143, 3, 0), (abi.FP8_152, 15, 0), (abi.FP8_152, 30, 1)):
        for rm in (abi.RM_SR, abi.RM_SR_NE_DNORM):
            for offset, clip, ftz, sftz in ((0, 0, 0, 0), (17, 1, 0, 0), (8, 1, 1, 0), (4, 0, 0, 1)):
                cp = abi.make_cast_params(rm, clip_fp=bool(clip), flush_denorms=bool(ftz), stochastic_ftz_fp8=bool(sftz), rng_kind=abi.RNG_PHILOX,
                                          rng_seed=77, rng_offset=offset)
                fused = np.zeros(M * N, abi.NP_DTYPE[od])
                calc.do_batch_gemm(T(fused, od, [N, M], fp_bias=bias, inf_nan_mode=mode), x, w, abi.OP_AB, cp)
                two = np.zeros(M * N, abi.NP_DTYPE[od])
                calc.do_activation(T(two, od, [N, M], fp_bias=bias, inf_nan_mode=mode), T(acc.copy(), abi.FP32, [N, M]), cp)
                assert (fused.view(np.uint8) == two.view(np.uint8)).all(), (od, bias, mode, rm, offset, clip, ftz, sftz)
    # LFSR stochastic rounding through bgemm == the reference's sequential order
    cp = abi.make_cast_params(abi.RM_SR, clip_fp=True)
    calc.set_lfsr(np.arange(2, 258, dtype=np.uint32), 37)
    fused = np.zeros(M * N, np.uint16)
    calc.do_batch_gemm(T(fused, abi.BF16, [N, M]), x, w, abi.OP_AB, cp)
    want = np.zeros(M * N, np.uint16)
    rc, _ = port.activation(T(want, abi.BF16, [N, M]), T(acc.copy(), abi.FP32, [N, M]), cp, np.arange(2, 258, dtype=np.uint32), 37)
    assert rc == 0 and (fused == want).all()


def test_fused_cast_over_the_whole_range(calc, port):
    """The epilogue's straight-line casts against the oracle's cast of the same accumulators, on products that span every
    binade of the fp8 formats: vanishing values, subnormals, the top binade, overflow, infinities and NaN in one tile."""
    rng = np.random.default_rng(14)
    M, N, K = 256, 512, 64
    # one non-zero product per output: x row i holds 2^(i % 80 - 50) (+ sign), w is a random mantissa pattern
    xf = np.zeros((M, K), np.float32)
    xf[np.arange(M), np.arange(M) % K] = np.ldexp(1.0, (np.arange(M) % 80) - 50) * np.where(np.arange(M) & 1, -1, 1)
    wf = rng.uniform(1.0, 2.0, (K, N)).astype(np.float32)
    wf[:, 7] = 3.0e38      # times 2^k, k > 0: overflows fp32, the accumulator is an infinity
    wf[:, 9] = np.nan
    wf[:, 11] = 0.0
    xb = (xf.view(np.uint32) >> 16).astype(np.uint16).ravel()
    wb = (wf.view(np.uint32) >> 16).astype(np.uint16).ravel()
    x, w = T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K])
    acc = np.zeros(M * N, np.float32)
    calc.do_batch_gemm(T(acc, abi.FP32, [N, M]), x, w, abi.OP_AB)
    bits = acc.view(np.uint32)
    assert np.isinf(acc).any() and np.isnan(acc).any() and (acc == 0).any()
    relu_bits = np.where((bits >> 31).astype(bool) | np.isnan(acc), np.uint32(0), bits)
    rnd = np.zeros(M * N, np.uint32)
    formats = ((abi.BF16, 0, 0, 0), (abi.FP8_143, 4, 7, 2), (abi.FP8_143, 4, 3, 2), (abi.FP8_143, 4, 11, 2), (abi.FP8_143, 4, 7, 0), (abi.FP8_143, 4, 3, 0), (abi.FP8_143, 4, 9, 1),
               (abi.FP8_143, 4, 15, 1), (abi.FP8_152, 5, 15, 0), (abi.FP8_152, 5, 30, 0), (abi.FP8_152, 5, 1, 0), (abi.FP8_152, 5, 1, 2))
    for od, ew, bias, mode in formats:
        for rm in (0, 1, 2, 3, 6):
            for clip, cii, relu in ((0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)):
                cp = abi.make_cast_params(rm, relu=bool(relu), clip_fp=bool(clip), clip_inf_in=bool(cii))
                fused = np.zeros(M * N, abi.NP_DTYPE[od])
                calc.do_batch_gemm(T(fused, od, [N, M], fp_bias=bias, inf_nan_mode=mode), x, w, abi.OP_AB, cp)
                src = relu_bits if relu else bits
                if od == abi.BF16:
                    want = port.fp32_to_bf16(src, rm, rnd, clip, 0, cii)
                else:
                    want = port.fp32_to_fp8(src, ew, bias, rm, rnd, 0, clip, cii, 0, mode)
                bad = np.flatnonzero(fused != want)
                assert bad.size == 0, (od, bias, mode, rm, clip, cii, relu, [(hex(src[i]), hex(fused[i]), hex(want[i])) for i in bad[:6]])


def test_zero_common_dim_and_errors(calc):
    y = np.full(6, 5.0, np.float32)
    e = np.zeros(1, np.uint16)
    calc.do_batch_gemm(T(y, abi.FP32, [3, 2]), T(e, abi.BF16, [0, 2]), T(e, abi.BF16, [3, 0]), abi.OP_AB)
    assert (y == 0).all()
    a = np.zeros(64, np.uint16)
    with pytest.raises(pkg.MmeError):  # common dims differ
        calc.do_batch_gemm(T(y, abi.FP32, [3, 2]), T(a, abi.BF16, [4, 2]), T(a, abi.BF16, [3, 5]), abi.OP_AB)
    with pytest.raises(pkg.MmeError):  # batch dims do not match
        calc.do_batch_gemm(T(np.zeros(24, np.float32), abi.FP32, [3, 2, 4]), T(a, abi.BF16, [4, 2, 3]), T(a, abi.BF16, [3, 4]), abi.OP_AB)
    with pytest.raises(pkg.MmeError) as ei:  # integer types are outside this backend: error, never a CPU path
        calc.do_batch_gemm(T(y, abi.FP32, [3, 2]), T(a, 2, [4, 2]), T(a, 2, [3, 4]), abi.OP_AB)
    assert ei.value.status == abi.ERR_UNSUPPORTED
    with pytest.raises(pkg.MmeError):  # bf16 x fp8 cannot be mixed (the reference asserts too)
        calc.do_batch_gemm(T(y, abi.FP32, [3, 2]), T(a, abi.BF16, [4, 2]), T(a, abi.FP8_143, [3, 4]), abi.OP_AB)
    # the context stays usable after errors
    ten = np.full(5, 10.0, np.float32)
    o = np.zeros(1, np.float32)
    calc.do_batch_gemm(T(o, abi.FP32, [1, 1]), T(ten, abi.FP32, [5, 1]), T(ten, abi.FP32, [1, 5]), abi.OP_AB)
    assert o[0] == 500.0


def test_device_resident_tensors(calc, best_oracle):
    rng = np.random.default_rng(21)
    M, N, K = 256, 256, 256
    xb, wb = util.gen_bf16(rng, M * K), util.gen_bf16(rng, K * N)
    dx, dw, do = calc.to_device(xb), calc.to_device(wb), calc.alloc(M * N * 4)
    calc.do_batch_gemm(T(do.ptr, abi.FP32, [N, M], mem_space=1), T(dx.ptr, abi.BF16, [K, M], mem_space=1),
                       T(dw.ptr, abi.BF16, [N, K], mem_space=1), abi.OP_AB)
    calc.sync(5_000_000_000)
    o = do.download(np.float32)
    r = np.zeros(M * N, np.float32)
    assert best_oracle.bgemm(T(r, abi.FP32, [N, M]), T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K]), abi.OP_AB) == 0
    assert np.abs(o - r).max() <= util.ACC_TOL * K / 4
    for b in (dx, dw, do):
        b.free()


def test_large_host_tensor_gemm_runs_pipelined_and_matches_device_path(calc):
    """Host-tensor GEMMs above 32 MiB upload / multiply / download in row blocks on three streams; every
    output row must be bit-identical to the single-launch device path (same reduction per row)."""
    rng = np.random.default_rng(33)
    M, N, K = 4352, 2048, 2048   # 17 tiles of rows: the last row block is ragged
    xb, wb = util.gen_bf16(rng, M * K), util.gen_bf16(rng, K * N)
    for op, ws in ((abi.OP_AB, [N, K]), (abi.OP_ABT, [K, N])):
        host = np.zeros(M * N, np.uint16)
        cp = abi.make_cast_params(abi.RM_SR, clip_fp=True, rng_kind=abi.RNG_PHILOX, rng_seed=3, rng_offset=17)
        calc.do_batch_gemm(T(host, abi.BF16, [N, M]), T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, ws), op, cp)
        dx, dw, do = calc.to_device(xb), calc.to_device(wb), calc.alloc(M * N * 2)
        calc.do_batch_gemm(T(do.ptr, abi.BF16, [N, M], mem_space=1), T(dx.ptr, abi.BF16, [K, M], mem_space=1),
                           T(dw.ptr, abi.BF16, ws, mem_space=1), op, cp)
        calc.sync(10_000_000_000)
        assert (host == do.download(np.uint16)).all(), op
        for b in (dx, dw, do):
            b.free()
