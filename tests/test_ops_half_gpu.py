"""The two-byte (fp16 / bf16) vector kernels one op at a time.  ODLA_FP16_MODE / ODLA_BF16_MODE keep the API in fp32 and
store every tensor in the two-byte type on the device, so the expectation is: round the inputs to that type, compute the
op in float64, round once to the type.  Data movement and max-pool must then be identical; arithmetic ops may differ by
the rounding of an fp32 intermediate, i.e. one unit in the last place of the two-byte result."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(77)
NHWC = 1  # ODLA_CHANNELS_LAST


def to_type(x, mode):
    """Round-to-nearest-even to fp16 or bf16, returned as float32."""
    x = np.asarray(x, np.float32)
    if mode == "fp16":
        return x.astype(np.float16).astype(np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(x.shape)


def ulp(mode):
    return 2.0 ** -10 if mode == "fp16" else 2.0 ** -7


def graph(odla, lib, mode, name="half"):
    return odla.Graph(lib, name, fp16=(mode == "fp16"), bf16=(mode == "bf16"))


def assert_within_ulps(got, want64, mode, n=1.0, floor=0.0):
    """|got - want| <= n units in the last place of the two-byte type at |want| (plus an absolute floor)."""
    want = np.asarray(want64, np.float64)
    floor = max(floor, 2.0 ** -14 if mode == "fp16" else 2.0 ** -126)   # below that the type's spacing is constant
    tol = n * ulp(mode) * np.maximum(np.abs(want), floor) + 1e-30
    err = np.abs(got.astype(np.float64) - want)
    bad = err > tol
    assert not bad.any(), "%d of %d outside %g ulp, worst %g at want %g" % (bad.sum(), bad.size, n, err[bad].max(), want[bad][err[bad].argmax()])


# rows of 8, 16 and 32 lanes, one to eight 16-byte pieces per lane, a ragged number of pieces per lane (1000 / 8 = 125),
# and widths the vector kernels refuse (not a multiple of 8; longer than 2048) that take the generic row kernels
WIDTHS = [8, 64, 128, 136, 256, 512, 768, 1000, 2048, 33, 4096]


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("dim", WIDTHS)
def test_softmax_rows(odla, gpu_lib, mode, dim):
    rows = 37   # not a multiple of the rows a warp or a block covers
    x = to_type(RNG.standard_normal((rows, dim)) * 3, mode)
    g = graph(odla, gpu_lib, mode)
    a = g.Argument("x", (rows, dim))
    g.Output(g.Softmax(a, -1, "sm"))
    g.Output(g.LogSoftmax(a, -1, "lsm"))
    got = g.run({"x": x})
    g.close()
    z = x.astype(np.float64) - x.max(axis=1, keepdims=True)
    e = np.exp(z)
    sm = e / e.sum(axis=1, keepdims=True)
    lsm = z - np.log(e.sum(axis=1, keepdims=True))
    assert_within_ulps(got["sm"], sm, mode, 1.0)
    assert_within_ulps(got["lsm"], lsm, mode, 1.0, floor=1e-3)
    s = got["sm"].astype(np.float64).sum(axis=1)
    assert np.abs(s - 1).max() <= ulp(mode) * math.sqrt(dim) + 1e-3


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("dim", WIDTHS)
def test_layernorm_rows(odla, gpu_lib, mode, dim):
    rows = 21
    x = to_type(RNG.standard_normal((rows, dim)) * 2 + 0.5, mode)
    gam = RNG.uniform(0.5, 1.5, dim).astype(np.float32)
    bet = RNG.standard_normal(dim).astype(np.float32)
    g = graph(odla, gpu_lib, mode)
    a = g.Argument("x", (rows, dim))
    g.Output(g.LayerNorm(a, (-1,), 1e-5, g.Constant("g", gam), g.Constant("b", bet), "ln"))
    got = g.run({"x": x})["ln"]
    g.close()
    x64 = x.astype(np.float64)
    mu = x64.mean(axis=1, keepdims=True)
    var = ((x64 - mu) ** 2).mean(axis=1, keepdims=True)
    want = (x64 - mu) / np.sqrt(var + 1e-5) * gam + bet
    # gamma * normalised + beta cancels for some elements: the bound is one ulp of the larger operand
    mag = np.maximum(np.abs(want), np.abs((x64 - mu) / np.sqrt(var + 1e-5) * gam))
    err = np.abs(got.astype(np.float64) - want)
    assert (err <= ulp(mode) * np.maximum(mag, 1e-2)).all(), float((err / np.maximum(mag, 1e-2)).max() / ulp(mode))


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("N,H,C,R,stride,pad", [(2, 14, 64, 3, 2, 1), (1, 13, 24, 2, 2, 0), (3, 9, 128, 3, 1, 1), (2, 12, 20, 3, 2, 1)])
def test_maxpool_is_exact(odla, gpu_lib, mode, N, H, C, R, stride, pad):
    x = to_type(RNG.standard_normal((N, H, H, C)), mode)
    P = (H + 2 * pad - R) // stride + 1
    g = graph(odla, gpu_lib, mode)
    a = g.Argument("x", (N, H, H, C))
    g.Output(g.MaxPool(a, NHWC, (R, R), (stride, stride), (pad, pad), (pad, pad), (N, P, P, C), "y"))
    got = g.run({"x": x})["y"]
    g.close()
    xp = np.full((N, H + 2 * pad, H + 2 * pad, C), -np.inf, np.float32)
    xp[:, pad:pad + H, pad:pad + H] = x
    want = np.full((N, P, P, C), -np.inf, np.float32)
    for r in range(R):
        for s in range(R):
            want = np.maximum(want, xp[:, r:r + stride * P:stride, s:s + stride * P:stride][:, :P, :P])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("n", [8 * 1024, 8 * 1024 + 5])     # whole 16-byte units, and a ragged tail
def test_unary_family(odla, gpu_lib, mode, n):
    x = to_type(RNG.standard_normal(n) * 2, mode)
    xpos = to_type(np.abs(RNG.standard_normal(n)) + 0.1, mode)
    erf = np.vectorize(math.erf)
    cases = {
        "Relu": (x, lambda v: np.maximum(v, 0)), "Sigmoid": (x, lambda v: 1 / (1 + np.exp(-v))), "Tanh": (x, np.tanh), "Exp": (x, np.exp),
        "Erf": (x, erf), "Abs": (x, np.abs), "Neg": (x, lambda v: -v), "Log": (xpos, np.log), "Sqrt": (xpos, np.sqrt), "Rsqrt": (xpos, lambda v: 1 / np.sqrt(v)),
        "Reciprocal": (xpos, lambda v: 1 / v),
    }
    g = graph(odla, gpu_lib, mode)
    a = g.Argument("x", (n,))
    p = g.Argument("xpos", (n,))
    for name, (src, _) in cases.items():
        g.Output(getattr(g, name)(a if src is x else p, name))
    g.Output(g.LeakyRelu(a, 0.1, "leaky"))
    g.Output(g.Clamp(a, -0.5, 1.25, "clamp"))
    g.Output(g.Gelu(a, 0, "gelu"))
    got = g.run({"x": x, "xpos": xpos})
    g.close()
    for name, (src, f) in cases.items():
        exact = name in ("Relu", "Abs", "Neg")
        want = f(src.astype(np.float64))
        if exact:
            assert np.array_equal(got[name], want.astype(np.float32)), name
        else:
            assert_within_ulps(got[name], want, mode, 1.0, floor=1e-3)
    x64 = x.astype(np.float64)
    assert_within_ulps(got["leaky"], np.where(x64 > 0, x64, 0.1 * x64), mode, 1.0)
    assert np.array_equal(got["clamp"], np.clip(x, -0.5, 1.25))
    assert_within_ulps(got["gelu"], 0.5 * x64 * (1 + erf(x64 / math.sqrt(2))), mode, 1.0, floor=1e-2)


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", [(4, 14, 14, 64), (3, 5, 7)])
def test_binary_same_shape_and_broadcast(odla, gpu_lib, mode, shape):
    a_ = to_type(RNG.standard_normal(shape), mode)
    b_ = to_type(RNG.uniform(0.5, 2.0, shape) * RNG.choice([-1, 1], shape), mode)
    c_ = to_type(RNG.standard_normal(shape[-1]), mode)
    g = graph(odla, gpu_lib, mode)
    a, b = g.Argument("a", shape), g.Argument("b", shape)
    c = g.Constant("c", c_)
    for fn in ("Add", "Sub", "Mul", "Div"):
        g.Output(getattr(g, fn)(a, b, fn))
    g.Output(g.Add(a, c, "add_bias"))
    g.Output(g.Mul(a, c, "mul_scale"))
    got = g.run({"a": a_, "b": b_})
    g.close()
    a64, b64, c64 = a_.astype(np.float64), b_.astype(np.float64), c_.astype(np.float64)
    # one fp32 operation on two-byte operands rounded once to the type: the correctly rounded result (double rounding
    # through fp32 can flip a tie for products and quotients, so those get one unit)
    assert np.array_equal(got["Add"], to_type(a64 + b64, mode))
    assert np.array_equal(got["Sub"], to_type(a64 - b64, mode))
    assert np.array_equal(got["add_bias"], to_type(a64 + c64, mode))
    assert_within_ulps(got["Mul"], a64 * b64, mode, 1.0)
    assert_within_ulps(got["mul_scale"], a64 * c64, mode, 1.0)
    assert_within_ulps(got["Div"], a64 / b64, mode, 1.0)


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
def test_quantize_from_two_byte_storage_matches_the_oracle(odla, gpu_lib, ref, mode):
    """Quantising a two-byte tensor is the fp32 rule applied to the stored value: identical to the CPU oracle given the
    rounded values, including ties and saturation, for a tensor scale and for per-channel scales."""
    shape = (2, 9, 9, 24)
    x = to_type(RNG.standard_normal(shape) * 2, mode)
    x.flat[:6] = to_type([0.025, 0.075, -0.025, 100.0, -100.0, 0.125], mode)
    scales = RNG.uniform(0.01, 0.2, 24).astype(np.float32)

    def build(g):
        a = g.Argument("x", shape)
        g.Output(g.Quantize(a, g.Constant("s", np.array([0.05], np.float32)), None, 0, odla.INT8, "q"))
        g.Output(g.Quantize(a, g.Constant("sa", scales), None, 3, odla.INT8, "q_axis"))
    g = graph(odla, gpu_lib, mode)
    build(g)
    got = g.run({"x": x})
    g.close()
    o = odla.Graph(ref, "oracle")
    build(o)
    want = o.run({"x": x})
    o.close()
    for k in want:
        assert np.array_equal(got[k], want[k]), k


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
def test_reduce_mean_two_byte(odla, gpu_lib, mode):
    """Global average pool on two-byte storage: sums in fp32 in the reference's axis-by-axis order, one rounding at the end."""
    shape = (5, 7, 7, 136)
    x = to_type(RNG.standard_normal(shape) + 0.25, mode)
    g = graph(odla, gpu_lib, mode)
    a = g.Argument("x", shape)
    g.Output(g.ReduceMean(a, (1, 2), True, (5, 1, 1, 136), "gap"))
    got = g.run({"x": x})["gap"]
    g.close()
    t = x[:, 0].copy()
    for h in range(1, 7):
        t = t + x[:, h]
    t = t / np.float32(7)
    u = t[:, 0].copy()
    for w in range(1, 7):
        u = u + t[:, w]
    u = (u / np.float32(7)).reshape(5, 1, 1, 136)
    assert_within_ulps(got, u.astype(np.float64), mode, 0.51)   # the correctly rounded value of the fp32 result


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("S,D", [(128, 64), (256, 64), (128, 32)])
def test_batched_gemm_with_untransposed_right_operand(odla, gpu_lib, mode, S, D, monkeypatch):
    """probabilities [B, H, S, S] x values [B, H, S, D] (attention context): for D = 64 the tensor cores read the values
    as they lie ([k][n], MN-major operand); other widths, or ODLA_B200_NO_N_MAJOR, go through a transposed copy.  Both
    routes issue the same multiply-accumulates in the same order, so they must agree bit for bit, and with float64 to
    the rounding of the two-byte result."""
    Bt, H = 2, 3
    pr = to_type(RNG.uniform(0, 1, (Bt, H, S, S)) / S * 4, mode)
    v = to_type(RNG.standard_normal((Bt, H, S, D)), mode)

    def run():
        g = graph(odla, gpu_lib, mode)
        a, b = g.Argument("p", (Bt, H, S, S)), g.Argument("v", (Bt, H, S, D))
        g.Output(g.Gemm(a, False, b, False, 1.0, 0.0, None, (Bt, H, S, D), "ctx"))
        out = g.run({"p": pr, "v": v})["ctx"]
        desc = g.describe(first_gpu_only=True)
        g.close()
        return out, desc
    got, desc = run()
    if D == 64:
        assert "gemm_umma" in desc
    monkeypatch.setenv("ODLA_B200_NO_N_MAJOR", "1")
    via_copy, _ = run()
    assert np.array_equal(got, via_copy)
    want = np.einsum("bhik,bhkd->bhid", pr.astype(np.float64), v.astype(np.float64))
    assert_within_ulps(got, want, mode, 1.0, floor=0.05)


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
@pytest.mark.parametrize("dim", [64, 768, 2048, 40])
def test_layernorm_writes_the_int8_copy_a_following_quantize_asks_for(odla, gpu_lib, mode, dim, monkeypatch):
    """LayerNorm -> {float consumer, per-tensor Quantize}: the row kernel writes the int8 tensor as well, quantising the
    values as they are stored, so both outputs are identical to the two-launch form (ODLA_B200_NO_LN_QUANT)."""
    rows = 53
    x = to_type(RNG.standard_normal((rows, dim)) * 2 + 0.25, mode)
    gam = RNG.uniform(0.5, 1.5, dim).astype(np.float32)
    bet = RNG.standard_normal(dim).astype(np.float32)

    def run():
        g = graph(odla, gpu_lib, mode)
        a = g.Argument("x", (rows, dim))
        ln = g.LayerNorm(a, (-1,), 1e-5, g.Constant("g", gam), g.Constant("b", bet), "ln")
        g.Output(ln)
        g.Output(g.Quantize(ln, g.Constant("s", np.array([0.03], np.float32)), None, 0, odla.INT8, "q"))
        out = g.run({"x": x})
        desc = g.describe(first_gpu_only=True)
        g.close()
        return out, desc
    fused, desc = run()
    assert "layernorm" in desc and "quantize" not in desc
    monkeypatch.setenv("ODLA_B200_NO_LN_QUANT", "1")
    plain, desc2 = run()
    assert "quantize" in desc2
    assert np.array_equal(fused["ln"], plain["ln"]) and np.array_equal(fused["q"], plain["q"])
    want = np.clip(np.rint(fused["ln"].astype(np.float32) / np.float32(0.03)), -128, 127).astype(np.int8)
    assert np.array_equal(fused["q"], want)
    assert np.abs(fused["q"].astype(int)).max() > 20   # the comparison is not about zeros
