"""The CPU oracle is pinned before it is trusted: against the reference's own known-answer test,
against golden vectors produced by the reference's runtime/generic kernels (tests/golden), and,
when the reference-compiled kernels are present, against them directly."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "ref_kernels.npz"))
f32p, i64 = C.POINTER(C.c_float), C.c_int64


def fp(a):
    return a.ctypes.data_as(f32p)


def test_known_answer_add_add(odla, ref):
    # tests/compile/test_cxx_gen.cc:48-50 in the reference: {1,2,3}+{1,2,3}+{4,5,6} = {6,9,12}
    g = odla.Graph(ref, "add")
    a, b = g.Argument("a", (3,)), g.Argument("b", (3,))
    c = g.Constant("c", np.array([4, 5, 6], np.float32))
    g.Output(g.Add(g.Add(a, b, "t"), c, "out"))
    out = g.run({"a": np.array([1, 2, 3], np.float32), "b": np.array([1, 2, 3], np.float32)})["out"]
    assert out.tolist() == [6.0, 9.0, 12.0]
    g.close()


@pytest.mark.parametrize("i", range(5))
def test_conv_restatement_matches_reference_vectors(ref, i):
    N, H, W, Cc, K, R, S, st, pad, P, Q = (int(v) for v in GOLD["conv%d_geom" % i])
    x, w, want = GOLD["conv%d_x" % i], GOLD["conv%d_w" % i], GOLD["conv%d_y" % i]
    y = np.zeros_like(want)
    ref.dll.ora_conv2d_f32(fp(y), fp(x), fp(w), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(K), i64(R), i64(S), i64(st), i64(st), i64(pad),
                           i64(pad), i64(1), C.c_int(1), i64(0), i64(N * P))
    assert np.array_equal(y, want)  # same summation order, no contraction: bit-exact


@pytest.mark.parametrize("i", range(3))
def test_maxpool_restatement_matches_reference_vectors(ref, i):
    N, H, W, Cc, R, st, pad, P, Q = (int(v) for v in GOLD["pool%d_geom" % i])
    x, want = GOLD["pool%d_x" % i], GOLD["pool%d_y" % i]
    y = np.zeros_like(want)
    ref.dll.ora_maxpool_f32(fp(y), fp(x), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(R), i64(R), i64(st), i64(st), i64(pad), i64(pad), C.c_int(1))
    assert np.array_equal(y, want)


@pytest.mark.parametrize("i", range(3))
def test_gemm_restatement_matches_reference_vectors(ref, i):
    A, B, Cm, want = GOLD["gemm%d_a" % i], GOLD["gemm%d_b" % i], GOLD["gemm%d_c" % i], GOLD["gemm%d_y" % i]
    ta, tb = (int(v) for v in GOLD["gemm%d_t" % i])
    M, Nn = want.shape
    Kd = A.shape[0] if ta else A.shape[1]
    y = np.zeros_like(want)
    ref.dll.ora_matmul_f32(fp(y), fp(A), fp(B), i64(M), i64(Nn), i64(Kd), C.c_int(ta), C.c_int(tb))
    ref.dll.ora_gemm_finish_f32(fp(y), fp(Cm), i64(M), i64(Nn), i64(Nn), C.c_float(0.5), C.c_float(2.0))
    assert np.array_equal(y, want)


def test_softmax_relu_batchnorm_match_reference_vectors(ref):
    x, want = GOLD["softmax_x"], GOLD["softmax_y"]
    y = np.zeros_like(x)
    ref.dll.ora_softmax_f32(fp(y), fp(x), i64(12), i64(10), i64(1), C.c_int(0))
    assert np.array_equal(y, want)
    x, want = GOLD["relu_x"], GOLD["relu_y"]
    y = np.zeros_like(x)
    ref.dll.ora_unary_f32(C.c_int(0), fp(y), fp(x), i64(x.size), C.c_float(0), C.c_float(0))
    assert np.array_equal(y, want)
    x, want = GOLD["bn_x"], GOLD["bn_y"]
    y = np.zeros_like(x)
    ref.dll.ora_batchnorm_f32(fp(y), fp(x), fp(GOLD["bn_mean"]), fp(GOLD["bn_var"]), fp(GOLD["bn_sc"]), fp(GOLD["bn_off"]), C.c_float(1), C.c_float(0),
                              C.c_float(1e-5), i64(18), i64(4), i64(1))
    np.testing.assert_allclose(y, want, rtol=0, atol=1e-6)


def test_reference_compiled_kernels_agree_when_present(odla, ref):
    """With oracle/_ref built from the reference's sources the platform routes conv / pool /
    softmax / matmul / relu through them; the restatement must give the same graph result."""
    path = os.path.join(ROOT, "oracle", "_ref", "libhalo_rt_generic.so")
    if not os.path.exists(path):
        pytest.skip("reference-compiled kernels not built here")
    assert ref.cpuref_UsesReference() == 1
    rl = C.CDLL(path)
    rng = np.random.default_rng(5)
    N, H, W, Cc, K, R, st, pad = 3, 11, 13, 5, 7, 3, 2, 1
    P, Q = (H + 2 * pad - R) // st + 1, (W + 2 * pad - R) // st + 1
    x = rng.standard_normal((N, H, W, Cc)).astype(np.float32)
    w = rng.standard_normal((R, R, Cc, K)).astype(np.float32)
    a, b = np.zeros((N, P, Q, K), np.float32), np.zeros((N, P, Q, K), np.float32)
    rl._sn_rt_conv2d_f32_nhwc(fp(a), fp(x), fp(w), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(K), i64(R), i64(R), i64(st), i64(st), i64(pad), i64(pad),
                              i64(pad), i64(pad))
    ref.dll.ora_conv2d_f32(fp(b), fp(x), fp(w), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(K), i64(R), i64(R), i64(st), i64(st), i64(pad), i64(pad),
                           i64(1), C.c_int(1), i64(0), i64(N * P))
    assert np.array_equal(a, b)


def test_quantize_is_divide_round_half_even_saturate(odla, ref):
    # ODLA/platforms/dnnl/odla_dnnl_quantization.cc:61-90: cast_sat(rne(x / scale) + zp)
    g = odla.Graph(ref, "q")
    x = g.Argument("x", (8,))
    s = g.Constant("s", np.array([0.5], np.float32))
    q = g.Quantize(x, s, None, 0, odla.INT8, "q")
    d = g.Dequantize(q, s, None, 0, odla.FLOAT32, "d")
    g.Output(q)
    g.Output(d)
    xs = np.array([0.25, 0.75, 1.25, -0.25, -0.75, 100.0, -100.0, 0.2], np.float32)
    out = g.run({"x": xs})
    assert out["q"].tolist() == [0, 2, 2, 0, -2, 127, -128, 0]   # ties go to even, then saturate
    assert np.array_equal(out["d"], out["q"].astype(np.float32) * np.float32(0.5))
    g.close()


def test_int8_conv_rule_exact_integers(odla, ref):
    """Conv(Dequantize(int8), Dequantize(int8 per-channel)) = float(int32 acc) * fl(s_x*s_w[k])."""
    rng = np.random.default_rng(3)
    N, H, Cc, K = 2, 6, 16, 8
    xq = rng.integers(-128, 128, (N, H, H, Cc), dtype=np.int8)
    wq = rng.integers(-127, 128, (3, 3, Cc, K), dtype=np.int8)
    sx, sw = np.float32(0.031), rng.uniform(0.001, 0.01, K).astype(np.float32)
    g = odla.Graph(ref, "c")
    x = g.Argument("x", xq.shape, odla.INT8)
    xd = g.Dequantize(x, g.Constant("sx", np.array([sx])), None, 0, odla.FLOAT32, "xd")
    wd = g.Dequantize(g.Constant("wq", wq), g.Constant("sw", sw), None, 3, odla.FLOAT32, "wd")
    y = g.Conv(xd, odla.CHANNELS_LAST, 1, wd, odla.SIO, (1, 1), (1, 1), (1, 1), (1, 1), None, (N, H, H, K), "y")
    g.Output(y)
    got = g.run({"x": xq})["y"]
    acc = np.zeros((N, H, H, K), np.int64)
    xp = np.pad(xq.astype(np.int64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    for r in range(3):
        for s in range(3):
            acc += np.einsum("nhwc,ck->nhwk", xp[:, r:r + H, s:s + H, :], wq[r, s].astype(np.int64))
    n = ref.cpuref_GetAccumulators(g.comp, b"y", None, 0)
    buf = np.zeros(n, np.int32)
    ref.cpuref_GetAccumulators(g.comp, b"y", buf.ctypes.data, n)
    assert np.array_equal(buf.reshape(acc.shape), acc.astype(np.int32))
    want = acc.astype(np.float32) * (sx * sw).astype(np.float32)
    assert np.array_equal(got, want)
    g.close()


def test_reduce_mean_is_axis_by_axis(odla, ref):
    # runtime/generic/common/reduce.cc:24-59: each axis summed in order, then divided by its extent
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 7, 7, 5)).astype(np.float32)
    g = odla.Graph(ref, "r")
    a = g.Argument("x", x.shape)
    g.Output(g.ReduceMean(a, (1, 2), True, (2, 1, 1, 5), "m"))
    got = g.run({"x": x})["m"]
    t = np.zeros((2, 7, 5), np.float32)
    for h in range(7):
        t = (t + x[:, h]) if h else x[:, 0].copy()
    t = t / np.float32(7)
    u = t[:, 0].copy()
    for w in range(1, 7):
        u = u + t[:, w]
    u = u / np.float32(7)
    assert np.array_equal(got.reshape(2, 5), u)
    g.close()


def test_layernorm_gelu_avgpool_against_numpy(odla, ref):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((4, 6, 32)).astype(np.float32)
    gam, bet = rng.standard_normal(32).astype(np.float32), rng.standard_normal(32).astype(np.float32)
    g = odla.Graph(ref, "l")
    a = g.Argument("x", x.shape)
    g.Output(g.LayerNorm(a, (-1,), 1e-5, g.Constant("g", gam), g.Constant("b", bet), "ln"))
    g.Output(g.Gelu(a, False, "gelu"))
    out = g.run({"x": x})
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    np.testing.assert_allclose(out["ln"], (x - mu) / np.sqrt(var + 1e-5) * gam + bet, atol=2e-5)
    from math import erf
    want = np.vectorize(lambda v: 0.5 * v * (1 + erf(v / np.sqrt(2))))(x.astype(np.float64))
    np.testing.assert_allclose(out["gelu"], want, atol=1e-6)
    g.close()
    x = rng.standard_normal((1, 5, 5, 3)).astype(np.float32)
    g = odla.Graph(ref, "p")
    a = g.Argument("x", x.shape)
    g.Output(g.AveragePool(a, odla.CHANNELS_LAST, (3, 3), (2, 2), (1, 1), (1, 1), False, (1, 3, 3, 3), "ap"))
    got = g.run({"x": x})["ap"]
    # corner window sees 2x2 valid pixels: the mean excludes the padding
    np.testing.assert_allclose(got[0, 0, 0], x[0, :2, :2].reshape(-1, 3).mean(0), atol=1e-6)
    g.close()


def test_requantisation_multiplies_by_the_reciprocal(odla, ref):
    """Quantize of a value that comes from int32 accumulators is sat(rne(x * fl(1/s))); the same
    Quantize applied to an ordinary float tensor divides like the reference."""
    rng = np.random.default_rng(8)
    xq = rng.integers(-128, 128, (1, 4, 4, 32), dtype=np.int8)
    wq = rng.integers(-127, 128, (1, 1, 32, 16), dtype=np.int8)
    sx, sw, sy = np.float32(0.013), np.float32(0.007), np.float32(0.3)
    g = odla.Graph(ref, "rq")
    x = g.Argument("x", xq.shape, odla.INT8)
    f = g.Argument("f", (1, 4, 4, 16), odla.FLOAT32)
    xd = g.Dequantize(x, g.Constant("sx", np.array([sx])), None, 0, odla.FLOAT32, "xd")
    wd = g.Dequantize(g.Constant("wq", wq), g.Constant("sw", np.array([sw])), None, 3, odla.FLOAT32, "wd")
    c = g.Conv(xd, odla.CHANNELS_LAST, 1, wd, odla.SIO, (1, 1), (1, 1), (0, 0), (0, 0), None, (1, 4, 4, 16), "c")
    S = g.Constant("sy", np.array([sy]))
    g.Output(g.Quantize(g.Relu(c, "r"), S, None, 0, odla.INT8, "q_acc"))
    g.Output(g.Quantize(f, S, None, 0, odla.INT8, "q_plain"))
    g.Output(c)
    fv = (rng.standard_normal((1, 4, 4, 16)) * 20).astype(np.float32)
    out = g.run({"x": xq, "f": fv})
    conv = out["c"]
    inv = np.float32(1.0) / sy
    assert np.array_equal(out["q_acc"], np.clip(np.rint(np.maximum(conv, 0) * inv), -128, 127).astype(np.int8))
    assert np.array_equal(out["q_plain"], np.clip(np.rint(fv / sy), -128, 127).astype(np.int8))
    g.close()
