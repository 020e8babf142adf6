"""The tensor-core kernel through its raw C-ABI entry point (odla_b200_conv_umma) against an
integer-exact / float64 numpy evaluation: shape sweep with ragged tiles, strides, paddings, channel
tails, every swizzle width, int32 accumulators bit-exact, requantised int8 outputs bit-exact."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def conv_ref(x, w, R, S, stride, pad, P, Q, acc_dtype):
    """x [N,H,W,C], w [K, R*S*C] -> [N,P,Q,K] accumulated in acc_dtype."""
    N, H, W, Cc = x.shape
    K = w.shape[0]
    xp = np.pad(x.astype(acc_dtype), ((0, 0), (pad, pad + stride), (pad, pad + stride), (0, 0)))
    out = np.zeros((N, P, Q, K), acc_dtype)
    wk = w.astype(acc_dtype).reshape(K, R, S, Cc)
    for r in range(R):
        for s in range(S):
            patch = xp[:, r:r + (P - 1) * stride + 1:stride, s:s + (Q - 1) * stride + 1:stride, :]
            out += np.einsum("npqc,kc->npqk", patch, wk[:, r, s, :])
    return out


SHAPES = [  # N, H, W, C, K, R, stride, pad
    (2, 14, 14, 64, 64, 3, 1, 1), (1, 7, 7, 512, 512, 3, 1, 1), (3, 28, 28, 128, 128, 3, 2, 1), (2, 56, 56, 64, 256, 1, 1, 0),
    (2, 28, 28, 256, 512, 1, 2, 0), (1, 9, 11, 32, 40, 3, 1, 1), (2, 5, 5, 16, 8, 3, 1, 1), (1, 13, 13, 24, 255, 1, 1, 0),
    (1, 1, 300, 72, 10, 1, 1, 0), (5, 7, 7, 160, 96, 3, 2, 1), (1, 17, 17, 64, 64, 5, 1, 2), (4, 8, 8, 200, 130, 1, 1, 0),
    # whole 256-row tiles with more than 128 output channels: the CTA-pair (cta_group::2) path, one and several tiles per pair,
    # and a last column tile whose second half lies entirely past K
    (4, 16, 16, 128, 512, 3, 1, 1), (2, 16, 8, 64, 256, 1, 1, 0), (8, 16, 16, 96, 384, 3, 2, 1), (64, 16, 16, 64, 256, 1, 1, 0),
    (4, 8, 8, 64, 64, 3, 1, 1), (16, 8, 8, 256, 128, 1, 1, 0),
    # a few whole output rows fill a tile: rectangular tiles fed by tiled 4-d loads (stride 1 and 2, 3x3 and strided 1x1, 108..128 rows)
    (2, 56, 56, 64, 64, 3, 1, 1), (2, 28, 28, 128, 128, 3, 1, 1), (2, 56, 56, 64, 128, 3, 2, 1), (2, 56, 56, 256, 512, 1, 2, 0), (2, 36, 36, 64, 64, 3, 1, 1),
]


@pytest.fixture
def every_layer_on_pairs(monkeypatch):
    """Lowers the CTA-pair thresholds so that every shape with whole 256-row tiles takes the cta_group::2 kernel."""
    monkeypatch.setenv("ODLA_B200_PAIR_MIN_BN", "64")
    monkeypatch.setenv("ODLA_B200_PAIR_MIN_KB", "1")
    monkeypatch.setenv("ODLA_B200_PAIR_S8", "1")


@pytest.mark.parametrize("shape", [s for s in SHAPES if (s[0] * ((s[1] + 2 * s[7] - s[5]) // s[6] + 1) * ((s[2] + 2 * s[7] - s[5]) // s[6] + 1)) % 256 == 0])
@pytest.mark.parametrize("dtype", ["f16", "s8"])
def test_conv_umma_on_cta_pairs(odla, gpu_lib, shape, dtype, every_layer_on_pairs):
    test_conv_umma_matches_numpy(odla, gpu_lib, shape, dtype)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16", "s8"])
def test_conv_umma_matches_numpy(odla, gpu_lib, shape, dtype):
    N, H, W, Cc, K, R, stride, pad = shape
    if dtype == "s8" and (Cc % 16 or Cc < 32):
        pytest.skip("int8 rows must be 16-byte multiples of at least 32 bytes for TMA")
    P, Q = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - R) // stride + 1
    rng = np.random.default_rng(hash(shape) % 2**31)
    if dtype == "s8":
        x = rng.integers(-128, 128, (N, H, W, Cc), dtype=np.int8)
        w = rng.integers(-127, 128, (K, R * R * Cc), dtype=np.int8)
        xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        y = torch.zeros((N, P, Q, K), dtype=torch.int32, device="cuda")
        d = odla.ConvDesc(n=N, h=H, w=W, c=Cc, k=K, r=R, s=R, stride_h=stride, stride_w=stride, pad_top=pad, pad_left=pad, p=P, q=Q, dtype=2, out_kind=3,
                          res_kind=0, act=0, alpha=0, res_scale=1, out_scale=1)
        assert gpu_lib.b200_conv_umma(C.byref(d), xt.data_ptr(), wt.data_ptr(), None, None, None, y.data_ptr(), None) == 0
        want = conv_ref(x, w, R, R, stride, pad, P, Q, np.int64).astype(np.int32)
        assert np.array_equal(y.cpu().numpy(), want)
        return
    tdt = torch.float16 if dtype == "f16" else torch.bfloat16
    xt = torch.from_numpy(rng.standard_normal((N, H, W, Cc)).astype(np.float32)).to(tdt).cuda()
    wt = torch.from_numpy((rng.standard_normal((K, R * R * Cc)) / np.sqrt(R * R * Cc)).astype(np.float32)).to(tdt).cuda()
    y = torch.zeros((N, P, Q, K), dtype=torch.float32, device="cuda")
    d = odla.ConvDesc(n=N, h=H, w=W, c=Cc, k=K, r=R, s=R, stride_h=stride, stride_w=stride, pad_top=pad, pad_left=pad, p=P, q=Q, dtype=0 if dtype == "f16" else 1,
                      out_kind=1, res_kind=0, act=0, alpha=0, res_scale=1, out_scale=1)
    assert gpu_lib.b200_conv_umma(C.byref(d), xt.data_ptr(), wt.data_ptr(), None, None, None, y.data_ptr(), None) == 0
    want = conv_ref(xt.float().cpu().numpy(), wt.float().cpu().numpy(), R, R, stride, pad, P, Q, np.float64)
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=0, atol=2e-3)   # fp32 accumulation of exact products


@pytest.mark.parametrize("dims", [(3, 14, 128, 96), (4, 16, 128, 256)])   # the second has whole 256-row tiles: CTA pairs
@pytest.mark.parametrize("multiply", [0, 1])
def test_conv_umma_int8_requant_epilogue_is_bit_exact(odla, gpu_lib, multiply, dims, every_layer_on_pairs):
    N, H, Cc, K = dims
    rng = np.random.default_rng(9)
    x = rng.integers(-128, 128, (N, H, H, Cc), dtype=np.int8)
    w = rng.integers(-127, 128, (K, 9 * Cc), dtype=np.int8)
    res = rng.integers(-128, 128, (N, H, H, K), dtype=np.int8)
    mul = rng.uniform(1e-4, 5e-4, K).astype(np.float32)
    add = rng.standard_normal(K).astype(np.float32)
    rs, os_ = np.float32(0.037), np.float32(0.021)
    t = [torch.from_numpy(a).cuda() for a in (x, w, res, mul, add)]
    y = torch.zeros((N, H, H, K), dtype=torch.int8, device="cuda")
    d = odla.ConvDesc(n=N, h=H, w=H, c=Cc, k=K, r=3, s=3, stride_h=1, stride_w=1, pad_top=1, pad_left=1, p=H, q=H, dtype=2, out_kind=2, res_kind=2, act=1,
                      alpha=0, res_scale=float(rs), out_scale=float(os_), out_multiply=multiply)
    assert gpu_lib.b200_conv_umma(C.byref(d), t[0].data_ptr(), t[1].data_ptr(), t[3].data_ptr(), t[4].data_ptr(), t[2].data_ptr(), y.data_ptr(), None) == 0
    acc = conv_ref(x, w, 3, 3, 1, 1, H, H, np.int64)
    v = acc.astype(np.float32) * mul          # every step rounds to fp32 separately, like the kernel's *_rn intrinsics
    v = v + add
    v = v + res.astype(np.float32) * rs
    v = np.maximum(v, np.float32(0))
    # division like the reference's odla_Quantize, or the requantisation form: times fl(1/s)
    scaled = v * (np.float32(1.0) / os_) if multiply else v / os_
    q = np.clip(np.rint(scaled), -128, 127).astype(np.int8)
    assert np.array_equal(y.cpu().numpy(), q)


def test_conv_umma_rejects_what_tma_cannot_address(odla, gpu_lib):
    d = odla.ConvDesc(n=1, h=8, w=8, c=3, k=8, r=3, s=3, stride_h=1, stride_w=1, pad_top=1, pad_left=1, p=8, q=8, dtype=0, out_kind=1, res_kind=0, act=0,
                      alpha=0, res_scale=1, out_scale=1)
    x = torch.zeros(8 * 8 * 3, dtype=torch.float16, device="cuda")
    assert gpu_lib.b200_conv_umma(C.byref(d), x.data_ptr(), x.data_ptr(), None, None, None, x.data_ptr(), None) == -1   # 3 channels: rows are not 16-byte multiples


def test_a_bounded_wait_that_runs_out_reports_a_timeout_and_the_next_launch_is_correct(odla, gpu_lib, monkeypatch):
    """The failure path of the tensor-core kernel, without faulting anything: a test hook makes the producer of one
    CTA leave a pipeline stage unarmed, the MMA lane's wait on that stage gives up after a short limit (a few hundred
    attempts instead of ~2^18), the CTA raises its abort flag, every role falls through to the common exit (tensor
    memory released, copies drained) and the entry point returns -3 -- the code odla_ExecuteComputation turns into
    ODLA_TIMEOUT.  The context stays usable: the same launch without the hook then gives the exact result."""
    N, H, W, Cc, K, R = 2, 14, 14, 64, 64, 3
    rng = np.random.default_rng(4)
    x = rng.integers(-128, 128, (N, H, W, Cc), dtype=np.int8)
    w = rng.integers(-127, 128, (K, R * R * Cc), dtype=np.int8)
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = torch.zeros((N, H, W, K), dtype=torch.int32, device="cuda")
    d = odla.ConvDesc(n=N, h=H, w=W, c=Cc, k=K, r=R, s=R, stride_h=1, stride_w=1, pad_top=1, pad_left=1, p=H, q=W, dtype=2, out_kind=3,
                      res_kind=0, act=0, alpha=0, res_scale=1, out_scale=1)
    monkeypatch.setenv("ODLA_B200_TEST_SPIN_LIMIT", "256")
    monkeypatch.setenv("ODLA_B200_TEST_SKIP_STAGE", "1")
    assert gpu_lib.b200_conv_umma(C.byref(d), xt.data_ptr(), wt.data_ptr(), None, None, None, y.data_ptr(), None) == -3
    monkeypatch.delenv("ODLA_B200_TEST_SKIP_STAGE")
    monkeypatch.delenv("ODLA_B200_TEST_SPIN_LIMIT")
    torch.cuda.synchronize()
    y.zero_()
    assert gpu_lib.b200_conv_umma(C.byref(d), xt.data_ptr(), wt.data_ptr(), None, None, None, y.data_ptr(), None) == 0
    assert np.array_equal(y.cpu().numpy(), conv_ref(x, w, R, R, 1, 1, H, W, np.int64).astype(np.int32))


def test_timeout_through_the_graph_path(odla, gpu_lib, ref, monkeypatch):
    """The same hook under odla_ExecuteComputation: the execute returns ODLA_TIMEOUT (the status word travels back with
    the outputs), and a computation planned afterwards without the hook runs and matches the oracle."""
    import blocks
    monkeypatch.setenv("ODLA_B200_TEST_SPIN_LIMIT", "256")
    monkeypatch.setenv("ODLA_B200_TEST_SKIP_STAGE", "1")
    gpu_lib.SetLogLevel(0)
    try:
        g = odla.Graph(gpu_lib, "timeout", fp16=True)
        x = g.Argument("x", (2, 14, 14, 64))
        wgt = (np.random.default_rng(1).standard_normal((3, 3, 64, 64)) * 0.05).astype(np.float32)
        g.Output(g.Conv(x, odla.CHANNELS_LAST, 1, g.Constant("w", wgt), odla.SIO, (1, 1), (1, 1), (1, 1), (1, 1), None, (2, 14, 14, 64), "y"))
        xin = np.zeros((2, 14, 14, 64), np.float32)
        yout = np.zeros((2, 14, 14, 64), np.float32)
        g.bind_input("x", xin.ctypes.data)
        g.bind_output("y", yout.ctypes.data)
        assert g.execute() == odla.TIMEOUT
        g.close()
    finally:
        gpu_lib.SetLogLevel(3)
    monkeypatch.delenv("ODLA_B200_TEST_SKIP_STAGE")
    monkeypatch.delenv("ODLA_B200_TEST_SPIN_LIMIT")
    blocks.check_block(odla, gpu_lib, ref, mode="fp16", batch=2, hw=14, cin=64, cout=64)
