"""Operator parity on the GPU: each ODLA op is built on libodla_b200.so and on the CPU oracle
platform from the same seeded inputs, through the C ABI, and compared.  fp32 graphs must agree to
1e-4 (the reference's own unit-test threshold, tests/unittests/run_test.py:383); integer and
data-movement results must be identical."""
import numpy as np
import pytest

import blocks

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(1234)


def run_both(odla, lib, ref, build, inputs, fp16=False):
    outs = []
    for L in (lib, ref):
        g = odla.Graph(L, "t", fp16=(fp16 and L is lib))
        build(g)
        outs.append(g.run(inputs))
        g.close()
    return outs


def close(got, want, tol=1e-4):
    for k in want:
        if want[k].dtype.kind in "iu":
            assert np.array_equal(got[k], want[k]), k
        else:
            err = float(np.abs(got[k].astype(np.float64) - want[k]).max()) if want[k].size else 0.0
            assert err <= tol * max(1.0, float(np.abs(want[k]).max()) if want[k].size else 1.0), "%s: %g" % (k, err)


def test_known_answer_add_add(odla, gpu_lib):
    g = odla.Graph(gpu_lib, "add")
    a, b = g.Argument("a", (3,)), g.Argument("b", (3,))
    g.Output(g.Add(g.Add(a, b, "t"), g.Constant("c", np.array([4, 5, 6], np.float32)), "out"))
    out = g.run({"a": np.array([1, 2, 3], np.float32), "b": np.array([1, 2, 3], np.float32)})["out"]
    assert out.tolist() == [6.0, 9.0, 12.0]
    # binding once and executing again must work; rebinding too
    assert g.execute() == 0
    g.close()


@pytest.mark.parametrize("N,H,W,C,K,R,stride,pad", [(2, 8, 8, 3, 5, 3, 1, 1), (1, 9, 7, 4, 6, 3, 2, 1), (1, 12, 12, 3, 8, 7, 2, 3), (3, 5, 5, 2, 3, 1, 1, 0),
                                                    (1, 1, 1, 7, 9, 1, 1, 0)])
def test_conv_fp32_nhwc(odla, gpu_lib, ref, N, H, W, C, K, R, stride, pad):
    P, Q = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - R) // stride + 1
    w = RNG.standard_normal((R, R, C, K)).astype(np.float32)
    bias = RNG.standard_normal((K,)).astype(np.float32)

    def build(g):
        x = g.Argument("x", (N, H, W, C))
        y = g.Conv(x, odla.CHANNELS_LAST, 1, g.Constant("w", w), odla.SIO, (stride, stride), (1, 1), (pad, pad), (pad, pad), g.Constant("b", bias), (N, P, Q, K), "y")
        g.Output(y)
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.standard_normal((N, H, W, C)).astype(np.float32)})
    close(got, want)


def test_conv_fp32_nchw_and_groups(odla, gpu_lib, ref):
    N, C, H, K = 2, 4, 6, 6
    w = RNG.standard_normal((K, C // 2, 3, 3)).astype(np.float32)

    def build(g):
        x = g.Argument("x", (N, C, H, H))
        g.Output(g.Conv(x, odla.CHANNELS_FIRST, 2, g.Constant("w", w), odla.OIS, (1, 1), (1, 1), (1, 1), (1, 1), None, (N, K, H, H), "y"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.standard_normal((N, C, H, H)).astype(np.float32)})
    close(got, want)


@pytest.mark.parametrize("ta,tb,cshape", [(0, 0, (5,)), (0, 1, (1,)), (1, 0, (4, 5)), (0, 0, None)])
def test_gemm_fp32(odla, gpu_lib, ref, ta, tb, cshape):
    M, Kd, Nn = 4, 7, 5
    B = RNG.standard_normal((Nn, Kd) if tb else (Kd, Nn)).astype(np.float32)
    Cm = RNG.standard_normal(cshape).astype(np.float32) if cshape else None

    def build(g):
        a = g.Argument("a", (Kd, M) if ta else (M, Kd))
        g.Output(g.Gemm(a, ta, g.Constant("b", B), tb, 0.5, 2.0, g.Constant("c", Cm) if Cm is not None else None, (M, Nn), "y"))
    got, want = run_both(odla, gpu_lib, ref, build, {"a": RNG.standard_normal((Kd, M) if ta else (M, Kd)).astype(np.float32)})
    close(got, want)


def test_batched_gemm_two_runtime_operands(odla, gpu_lib, ref):
    def build(g):
        a, b = g.Argument("a", (2, 3, 4, 6)), g.Argument("b", (2, 3, 5, 6))
        g.Output(g.Gemm(a, 0, b, 1, 1.0, 0.0, None, (2, 3, 4, 5), "y"))
    ins = {"a": RNG.standard_normal((2, 3, 4, 6)).astype(np.float32), "b": RNG.standard_normal((2, 3, 5, 6)).astype(np.float32)}
    got, want = run_both(odla, gpu_lib, ref, build, ins)
    close(got, want)


@pytest.mark.parametrize("is_max", [True, False])
@pytest.mark.parametrize("N,H,C,R,stride,pad", [(2, 8, 3, 3, 2, 1), (1, 7, 4, 2, 2, 0), (1, 6, 8, 3, 1, 1)])
def test_pooling(odla, gpu_lib, ref, is_max, N, H, C, R, stride, pad):
    P = (H + 2 * pad - R) // stride + 1

    def build(g):
        x = g.Argument("x", (N, H, H, C))
        if is_max:
            g.Output(g.MaxPool(x, odla.CHANNELS_LAST, (R, R), (stride, stride), (pad, pad), (pad, pad), (N, P, P, C), "y"))
        else:
            g.Output(g.AveragePool(x, odla.CHANNELS_LAST, (R, R), (stride, stride), (pad, pad), (pad, pad), False, (N, P, P, C), "y"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.standard_normal((N, H, H, C)).astype(np.float32)})
    close(got, want, 1e-6)


def test_maxpool_int8_is_exact(odla, gpu_lib, ref):
    def build(g):
        x = g.Argument("x", (2, 9, 9, 32), odla.INT8)
        g.Output(g.MaxPool(x, odla.CHANNELS_LAST, (3, 3), (2, 2), (1, 1), (1, 1), (2, 5, 5, 32), "y"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.integers(-128, 128, (2, 9, 9, 32), dtype=np.int8)})
    close(got, want)


def test_batchnorm_and_unary_family(odla, gpu_lib, ref):
    C = 6
    mean, var = RNG.standard_normal(C).astype(np.float32), RNG.uniform(0.5, 1.5, C).astype(np.float32)
    sc, of = RNG.standard_normal(C).astype(np.float32), RNG.standard_normal(C).astype(np.float32)

    def build(g):
        x = g.Argument("x", (2, 4, 4, C))
        y = g.BatchNormalization(x, odla.CHANNELS_LAST, g.Constant("m", mean), g.Constant("v", var), 1e-5, g.Constant("s", sc), g.Constant("o", of), "bn")
        g.Output(y)
        g.Output(g.Relu(x, "relu"))
        g.Output(g.LeakyRelu(x, 0.1, "leaky"))
        g.Output(g.Clamp(x, -0.5, 0.7, "clamp"))
        g.Output(g.Gelu(x, False, "gelu"))
        g.Output(g.Gelu(x, True, "gelu_tanh"))
        g.Output(g.Erf(x, "erf"))
        g.Output(g.Sigmoid(x, "sigmoid"))
        g.Output(g.Tanh(x, "tanh"))
        g.Output(g.Exp(x, "exp"))
        g.Output(g.Abs(x, "abs"))
        g.Output(g.Neg(x, "neg"))
        g.Output(g.Round(x, "round"))
        p = g.Abs(x, "pos")
        g.Output(g.Sqrt(p, "sqrt"))
        g.Output(g.Log(g.Add(p, g.Constant("one", np.array([1.0], np.float32)), "p1"), "log"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.standard_normal((2, 4, 4, C)).astype(np.float32)})
    close(got, want, 2e-5)
    assert np.array_equal(got["relu"], want["relu"]) and np.array_equal(got["round"], want["round"])


def test_binary_broadcasting(odla, gpu_lib, ref):
    def build(g):
        a, b = g.Argument("a", (2, 3, 1, 5)), g.Argument("b", (3, 4, 1))
        g.Output(g.Add(a, b, "add"))
        g.Output(g.Sub(a, b, "sub"))
        g.Output(g.Mul(a, b, "mul"))
        g.Output(g.Div(a, g.Constant("c", np.array([[2.0], [4.0], [8.0], [0.5]], np.float32)), "div"))
    ins = {"a": RNG.standard_normal((2, 3, 1, 5)).astype(np.float32), "b": RNG.standard_normal((3, 4, 1)).astype(np.float32)}
    got, want = run_both(odla, gpu_lib, ref, build, ins)
    for k in want:
        assert np.array_equal(got[k], want[k]), k   # one correctly rounded operation per element


@pytest.mark.parametrize("axis", [-1, 1])
def test_softmax_and_logsoftmax(odla, gpu_lib, ref, axis):
    def build(g):
        x = g.Argument("x", (3, 7, 33))
        g.Output(g.Softmax(x, axis, "sm"))
        g.Output(g.LogSoftmax(x, axis, "lsm"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": (RNG.standard_normal((3, 7, 33)) * 4).astype(np.float32)})
    close(got, want, 1e-5)


def test_reduce_mean_layernorm(odla, gpu_lib, ref):
    gam, bet = RNG.standard_normal(48).astype(np.float32), RNG.standard_normal(48).astype(np.float32)

    def build(g):
        x = g.Argument("x", (2, 7, 7, 48))
        g.Output(g.ReduceMean(x, (1, 2), True, (2, 1, 1, 48), "gap"))
        g.Output(g.ReduceMean(x, (3,), True, (2, 7, 7, 1), "last"))
        g.Output(g.LayerNorm(x, (-1,), 1e-5, g.Constant("g", gam), g.Constant("b", bet), "ln"))
    got, want = run_both(odla, gpu_lib, ref, build, {"x": RNG.standard_normal((2, 7, 7, 48)).astype(np.float32)})
    assert np.array_equal(got["gap"], want["gap"])      # same order of additions and divisions as the reference
    assert np.array_equal(got["last"], want["last"])
    close({"ln": got["ln"]}, {"ln": want["ln"]}, 2e-5)


def test_quantize_dequantize_semantics(odla, gpu_lib, ref):
    scales = RNG.uniform(0.01, 0.2, 6).astype(np.float32)
    zp = np.array([3], np.int32)

    def build(g):
        x = g.Argument("x", (4, 5, 6))
        s = g.Constant("s", np.array([0.05], np.float32))
        q = g.Quantize(x, s, None, 0, odla.INT8, "q")
        g.Output(q)
        g.Output(g.Dequantize(q, s, None, 0, odla.FLOAT32, "dq"))
        qa = g.Quantize(x, g.Constant("sa", scales), None, 2, odla.INT8, "q_axis")
        g.Output(qa)
        g.Output(g.Dequantize(qa, g.Constant("sa2", scales), None, 2, odla.FLOAT32, "dq_axis"))
        g.Output(g.Quantize(x, s, g.Constant("zp", zp), 0, odla.UINT8, "q_u8"))
    x = (RNG.standard_normal((4, 5, 6)) * 3).astype(np.float32)
    x.flat[:6] = [0.025, 0.075, -0.025, 100.0, -100.0, 0.125]   # ties and saturation
    got, want = run_both(odla, gpu_lib, ref, build, {"x": x})
    for k in want:
        assert np.array_equal(got[k], want[k]), k


def test_data_movement_ops(odla, gpu_lib, ref):
    table = RNG.standard_normal((11, 8)).astype(np.float32)

    def build(g):
        x = g.Argument("x", (2, 3, 4, 8))
        idx = g.Argument("idx", (2, 5), odla.INT32)
        g.Output(g.Transpose(x, (0, 2, 1, 3), (2, 4, 3, 8), "tr"))
        g.Output(g.Reshape(x, (2, 12, 8), "rs"))
        g.Output(g.Concat([x, x, x], 3, (2, 3, 4, 24), "cat"))
        g.Output(g.Resize(x, (2, 6, 8, 8), "up"))
        g.Output(g.Slice(x, (0, 1, 0, 2), (2, 3, 4, 8), (1, 1, 2, 3), (2, 2, 2, 2), "sl"))
        g.Output(g.Gather(g.Constant("table", table), idx, 0, (2, 5, 8), "ga"))
        g.Output(g.Cast(idx, odla.FLOAT32, "cast"))
    ins = {"x": RNG.standard_normal((2, 3, 4, 8)).astype(np.float32), "idx": RNG.integers(0, 11, (2, 5), dtype=np.int32)}
    got, want = run_both(odla, gpu_lib, ref, build, ins)
    for k in want:
        assert np.array_equal(got[k], want[k]), k


@pytest.mark.parametrize("fp16", [False, True])
def test_transposes_against_numpy(odla, gpu_lib, fp16):
    """Every kind of move the library has: last two axes swapped (shared-memory tiles, ragged edges), inner axis kept
    (16-byte units), a general permutation, in fp32 and in two-byte storage."""
    x = RNG.standard_normal((3, 37, 70)).astype(np.float32)
    y = RNG.standard_normal((2, 5, 6, 16)).astype(np.float32)

    def build(g):
        a = g.Argument("x", (3, 37, 70))
        b = g.Argument("y", (2, 5, 6, 16))
        g.Output(g.Transpose(a, (0, 2, 1), (3, 70, 37), "t_last2"))
        g.Output(g.Transpose(a, (2, 1, 0), (70, 37, 3), "t_rev"))
        g.Output(g.Transpose(b, (0, 2, 1, 3), (2, 6, 5, 16), "t_heads"))
        g.Output(g.Transpose(b, (0, 3, 1, 2), (2, 16, 5, 6), "t_nchw"))
    g = odla.Graph(gpu_lib, "tr", fp16=fp16)
    build(g)
    got = g.run({"x": x, "y": y})
    g.close()
    if fp16:
        x, y = x.astype(np.float16).astype(np.float32), y.astype(np.float16).astype(np.float32)
    want = {"t_last2": x.transpose(0, 2, 1), "t_rev": x.transpose(2, 1, 0), "t_heads": y.transpose(0, 2, 1, 3), "t_nchw": y.transpose(0, 3, 1, 2)}
    for k, v in want.items():
        assert np.array_equal(got[k], v), k


def test_empty_batch_dimension_is_handled(odla, gpu_lib):
    g = odla.Graph(gpu_lib, "empty")
    x = g.Argument("x", (0, 8))
    g.Output(g.Relu(x, "y"))
    out = g.run({"x": np.zeros((0, 8), np.float32)})
    assert out["y"].shape == (0, 8)
    g.close()


@pytest.mark.parametrize("mode", ["fp32", "fp16", "bf16", "int8"])
@pytest.mark.parametrize("k,stride,cin,cout,hw,act", [(3, 1, 64, 64, 14, "relu"), (1, 1, 64, 256, 14, "relu"), (3, 2, 128, 128, 28, "relu"), (1, 2, 256, 512, 14, "relu"),
                                                      (3, 1, 32, 64, 13, "leaky"), (3, 1, 48, 24, 9, "relu")])
def test_fused_block(odla, gpu_lib, ref, mode, k, stride, cin, cout, hw, act):
    """conv + per-channel add + residual add + activation (+ requantise): one fused launch on the
    tensor cores for fp16 / bf16 / int8, bit-exact for int8."""
    expect = None if mode == "fp32" else "conv_umma"
    desc = blocks.check_block(odla, gpu_lib, ref, mode, 3, hw, cin, cout, k=k, stride=stride, seed=k + stride + cin, act=act, expect_op=expect)
    if mode != "fp32":
        assert desc.count("\n  ") <= 4   # quantise launches for the two inputs + one fused launch (+ none for the epilogue ops)
