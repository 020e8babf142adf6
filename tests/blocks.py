"""Shared test helper: one bottleneck-style block (3x3 conv + folded-BN add + residual + relu
[+ requantise]) built on two ODLA libraries and compared."""
import numpy as np


def build_block(odla, g, mode, batch, hw, cin, cout, k=3, stride=1, seed=0, act="relu"):
    rng = np.random.default_rng(seed)
    pad = k // 2
    ho = (hw + 2 * pad - k) // stride + 1
    w = (rng.standard_normal((k, k, cin, cout)) * np.sqrt(2.0 / (k * k * cin))).astype(np.float32)
    b = (rng.standard_normal((1, 1, 1, cout)) * 0.1).astype(np.float32)
    NHWC, SIO, F32, I8 = odla.CHANNELS_LAST, odla.SIO, odla.FLOAT32, odla.INT8
    x = g.Argument("x", (batch, hw, hw, cin), F32)
    r = g.Argument("r", (batch, ho, ho, cout), F32)
    B = g.Constant("b", b)
    if mode == "int8":
        sx, sr, sy = np.float32(4.0 / 127), np.float32(4.0 / 127), np.float32(6.0 / 127)
        sw = (np.abs(w.reshape(-1, cout)).max(axis=0) / 127.0).astype(np.float32)
        wq = np.clip(np.rint(w / sw), -127, 127).astype(np.int8)
        Sx, Sr, Sy = (g.Constant(n, np.array([v], np.float32)) for n, v in (("sx", sx), ("sr", sr), ("sy", sy)))
        xq = g.Quantize(x, Sx, None, 0, I8, "xq")
        rq = g.Quantize(r, Sr, None, 0, I8, "rq")
        xd = g.Dequantize(xq, Sx, None, 0, F32, "xd")
        wd = g.Dequantize(g.Constant("wq", wq), g.Constant("sw", sw), None, 3, F32, "wd")
        y = g.Conv(xd, NHWC, 1, wd, SIO, (stride, stride), (1, 1), (pad, pad), (pad, pad), None, (batch, ho, ho, cout), "conv")
        y = g.Add(y, B, "bn")
        y = g.Add(y, g.Dequantize(rq, Sr, None, 0, F32, "rd"), "res")
        y = g.Relu(y, "relu") if act == "relu" else g.LeakyRelu(y, 0.1, "relu")
        y = g.Quantize(y, Sy, None, 0, I8, "y")
    else:
        W = g.Constant("w", w)
        y = g.Conv(x, NHWC, 1, W, SIO, (stride, stride), (1, 1), (pad, pad), (pad, pad), None, (batch, ho, ho, cout), "conv")
        y = g.Add(y, B, "bn")
        y = g.Add(y, r, "res")
        y = g.Relu(y, "y") if act == "relu" else g.LeakyRelu(y, 0.1, "y")
    g.Output(y)
    ins = {"x": rng.standard_normal((batch, hw, hw, cin)).astype(np.float32),
           "r": rng.standard_normal((batch, ho, ho, cout)).astype(np.float32)}
    return ins


def check_block(odla, lib, ref, mode, batch, hw, cin, cout, k=3, stride=1, seed=0, act="relu", expect_op=None):
    outs, desc = [], ""
    for L in (lib, ref):
        g = odla.Graph(L, "block", fp16=(mode == "fp16" and L is lib), bf16=(mode == "bf16" and L is lib))
        ins = build_block(odla, g, "int8" if mode == "int8" else "fp", batch, hw, cin, cout, k, stride, seed, act)
        outs.append(g.run(ins)["y"])
        if L is lib:
            desc = g.describe(first_gpu_only=True)
        g.close()
    if expect_op is not None:
        assert expect_op in desc, "expected a %s launch, plan was:\n%s" % (expect_op, desc)
    got, want = outs
    if mode == "int8":
        bad = int((got != want).sum())
        assert bad == 0, "int8 block not bit-exact: %d of %d differ (max diff %d)\n%s" % (
            bad, got.size, int(np.abs(got.astype(int) - want.astype(int)).max()), desc)
    else:
        tol = {"fp32": 1e-4, "fp16": 3e-2, "bf16": 2e-1}[mode]
        err = float(np.abs(got.astype(np.float32) - want).max())
        scale = float(np.abs(want).max()) + 1e-6
        assert err <= tol * max(1.0, scale), "%s block: max abs err %g (scale %g)\n%s" % (mode, err, scale, desc)
    return desc
