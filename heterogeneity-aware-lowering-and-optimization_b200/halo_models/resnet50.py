"""ResNet-50 v1.5 (stride on the 3x3 of each bottleneck) as an NHWC ODLA graph with random weights.

Emission follows what HALO produces after its default passes: batch normalisation is folded into
the filter and a per-channel ``odla_Add`` (lib/transforms/inst_simplify.cc:1371-1429 in the
reference), the convolution's own bias argument is null, the global pool is ``odla_ReduceMean`` over
the spatial axes and the classifier is ``odla_Gemm`` + ``odla_Softmax``.

The int8 variant is the same graph in quantise/dequantise form: every activation tensor that
crosses a convolution boundary is an int8 value produced by ``odla_Quantize`` (per-tensor symmetric
scale max|x|/127 from a calibration batch), filters are int8 constants with one scale per output
channel, and each consumer reads them through ``odla_Dequantize``.
"""
import numpy as np

from .. import odla

STAGES = [(3, 64, 256, 1), (4, 128, 512, 2), (6, 256, 1024, 2), (3, 512, 2048, 2)]
MAC_PER_IMAGE = 4089184256
EPS = 1e-5


def conv_list():
    """(name, kh, cin, cout, stride, pad) of every convolution in execution order."""
    convs = [("conv1", 7, 3, 64, 2, 3)]
    cin = 64
    for si, (blocks, mid, out, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            p = "s%db%d" % (si + 1, b)
            convs.append((p + "_c1", 1, cin, mid, 1, 0))
            convs.append((p + "_c2", 3, mid, mid, s, 1))
            convs.append((p + "_c3", 1, mid, out, 1, 0))
            if b == 0:
                convs.append((p + "_sc", 1, cin, out, s, 0))
            cin = out
    return convs


def weights(seed=100):
    """He-normal filters (HWIO) with inference batch-norm statistics folded in; fp32."""
    w = {}
    for i, (name, k, cin, cout, _, _) in enumerate(conv_list()):
        rng = np.random.default_rng(seed + i)
        kern = rng.standard_normal((k, k, cin, cout)) * np.sqrt(2.0 / (k * k * cin))
        beta, mean = rng.standard_normal(cout) * 0.1, rng.standard_normal(cout) * 0.1
        var = rng.uniform(0.5, 1.5, cout)
        # gamma = 1, except the last batch-norm of each bottleneck (gamma = 0.25): with gamma = 1 on
        # every residual branch the activations of a random-weight network double in variance per
        # block, reach ~2e4 (the edge of fp16) and saturate the soft-max, which makes any comparison
        # of outputs meaningless.
        gamma = 0.25 if name.endswith("_c3") else 1.0
        scale = gamma / np.sqrt(var + EPS)
        w[name + "_w"] = (kern * scale).astype(np.float32)
        w[name + "_b"] = (beta - mean * scale).astype(np.float32).reshape(1, 1, 1, cout)
    rng = np.random.default_rng(seed + 1000)
    w["fc_w"] = (rng.standard_normal((2048, 1000)) * 0.01).astype(np.float32)
    w["fc_b"] = np.zeros((1000,), np.float32)
    return w


def inputs(batch, seed=None, dtype=np.float32):
    rng = np.random.default_rng(10 + batch if seed is None else seed)
    return {"input": rng.standard_normal((batch, 224, 224, 3)).astype(dtype)}


def _out_hw(h, k, s, p):
    return (h + 2 * p - k) // s + 1


def torch_forward(w, x_nhwc, record=None):
    """fp32 forward on the host with torch, used only to calibrate activation ranges (and as an
    independent cross-check); returns the soft-max output."""
    import torch
    import torch.nn.functional as F

    def rec(name, t):
        if record is not None:
            record[name] = max(record.get(name, 0.0), float(t.abs().max()))

    def conv(x, name, s, p, relu=True, res=None):
        k = torch.from_numpy(np.ascontiguousarray(w[name + "_w"].transpose(3, 2, 0, 1)))
        y = F.conv2d(x, k, stride=s, padding=p) + torch.from_numpy(w[name + "_b"].reshape(1, -1, 1, 1))
        if res is not None:
            y = y + res
        if relu:
            y = F.relu(y)
        rec(name, y)
        return y

    with torch.no_grad():
        x = torch.from_numpy(np.ascontiguousarray(np.asarray(x_nhwc, np.float32).transpose(0, 3, 1, 2)))
        rec("input", x)
        x = conv(x, "conv1", 2, 3)
        x = F.max_pool2d(x, 3, 2, 1)
        for si, (blocks, mid, out, stride) in enumerate(STAGES):
            for b in range(blocks):
                s = stride if b == 0 else 1
                p = "s%db%d" % (si + 1, b)
                sc = conv(x, p + "_sc", s, 0, relu=False) if b == 0 else x
                y = conv(x, p + "_c1", 1, 0)
                y = conv(y, p + "_c2", s, 1)
                x = conv(y, p + "_c3", 1, 0, res=sc)
        x = x.mean(dim=(2, 3))
        rec("pool", x)
        logits = x @ torch.from_numpy(w["fc_w"]) + torch.from_numpy(w["fc_b"])
        return torch.softmax(logits, dim=1).numpy()


def calibrate(w, n_images=32, seed=7):
    """max|x| of every quantised tensor over a calibration batch of N(0,1) images."""
    rng = np.random.default_rng(seed)
    ranges = {}
    for i in range(0, n_images, 8):
        torch_forward(w, rng.standard_normal((min(8, n_images - i), 224, 224, 3)).astype(np.float32), ranges)
    return {k: np.float32(max(v, 1e-6) / 127.0) for k, v in ranges.items()}


def quantize_weights(w):
    """int8 filters with one symmetric scale per output channel (last axis)."""
    q = {}
    for name, a in w.items():
        if not name.endswith("_w"):
            continue
        flat = np.abs(a.reshape(-1, a.shape[-1])).max(axis=0)
        s = (np.maximum(flat, 1e-12) / 127.0).astype(np.float32)
        q[name + "_q"] = np.clip(np.rint(a / s), -127, 127).astype(np.int8)
        q[name + "_s"] = s
    return q


def build(g, batch, w, input_type=odla.FLOAT32, softmax=True):
    """Floating-point graph (fp32 storage, or fp16/bf16 when the Graph was created in that mode)."""
    NHWC, SIO = odla.CHANNELS_LAST, odla.SIO
    x = g.Argument("input", (batch, 224, 224, 3), input_type)
    h = 224

    def conv(x, name, k, cout, s, p, h_in, relu=True, res=None):
        ho = _out_hw(h_in, k, s, p)
        W = g.Constant(name + "_w", w[name + "_w"])
        B = g.Constant(name + "_b", w[name + "_b"])
        y = g.Conv(x, NHWC, 1, W, SIO, (s, s), (1, 1), (p, p), (p, p), None, (batch, ho, ho, cout), name)
        y = g.Add(y, B, name + "_bn")
        if res is not None:
            y = g.Add(y, res, name + "_add")
        if relu:
            y = g.Relu(y, name + "_relu")
        return y, ho

    x, h = conv(x, "conv1", 7, 64, 2, 3, h)
    ho = _out_hw(h, 3, 2, 1)
    x = g.MaxPool(x, NHWC, (3, 3), (2, 2), (1, 1), (1, 1), (batch, ho, ho, 64), "pool1")
    h = ho
    for si, (blocks, mid, out, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            p = "s%db%d" % (si + 1, b)
            sc = x
            if b == 0:
                sc, _ = conv(x, p + "_sc", 1, out, s, 0, h, relu=False)
            y, _ = conv(x, p + "_c1", 1, mid, 1, 0, h)
            y, h2 = conv(y, p + "_c2", 3, mid, s, 1, h)
            x, _ = conv(y, p + "_c3", 1, out, 1, 0, h2, res=sc)
            h = h2
    x = g.ReduceMean(x, (1, 2), True, (batch, 1, 1, 2048), "gap")
    x = g.Reshape(x, (batch, 2048), "flatten")
    Wf, Bf = g.Constant("fc_w", w["fc_w"]), g.Constant("fc_b", w["fc_b"])
    x = g.Gemm(x, False, Wf, False, 1.0, 1.0, Bf, (batch, 1000), "logits")
    if softmax:
        x = g.Softmax(x, -1, "prob")
    g.Output(x)
    return g


def build_int8(g, batch, w, wq, scales, softmax=True, extra_outputs=(), input_type=odla.FLOAT32):
    """Quantise/dequantise form.  `scales` maps tensor name -> per-tensor activation scale."""
    NHWC, SIO = odla.CHANNELS_LAST, odla.SIO
    F32, I8 = odla.FLOAT32, odla.INT8
    x = g.Argument("input", (batch, 224, 224, 3), input_type)
    sc_const = {}

    def scale(name):
        if name not in sc_const:
            sc_const[name] = g.Constant("scale_" + name, np.array([scales[name]], np.float32))
        return sc_const[name]

    xq = g.Quantize(x, scale("input"), None, 0, I8, "input_q")

    def conv(xq, xname, name, k, cout, s, p, h_in, relu=True, res=None):
        ho = _out_hw(h_in, k, s, p)
        xd = g.Dequantize(xq, scale(xname), None, 0, F32, name + "_xdq")
        Wq = g.Constant(name + "_w_q", wq[name + "_w_q"])
        Ws = g.Constant(name + "_w_s", wq[name + "_w_s"])
        wd = g.Dequantize(Wq, Ws, None, 3, F32, name + "_wdq")
        B = g.Constant(name + "_b", w[name + "_b"])
        y = g.Conv(xd, NHWC, 1, wd, SIO, (s, s), (1, 1), (p, p), (p, p), None, (batch, ho, ho, cout), name)
        y = g.Add(y, B, name + "_bn")
        if res is not None:
            rq, rname = res
            rd = g.Dequantize(rq, scale(rname), None, 0, F32, name + "_rdq")
            y = g.Add(y, rd, name + "_add")
        if relu:
            y = g.Relu(y, name + "_relu")
        yq = g.Quantize(y, scale(name), None, 0, I8, name + "_q")
        if name in extra_outputs:
            g.Output(yq)
        return yq, ho

    h = 224
    xq, h = conv(xq, "input", "conv1", 7, 64, 2, 3, h)
    xname = "conv1"
    ho = _out_hw(h, 3, 2, 1)
    xq = g.MaxPool(xq, NHWC, (3, 3), (2, 2), (1, 1), (1, 1), (batch, ho, ho, 64), "pool1")
    h = ho
    for si, (blocks, mid, out, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            p = "s%db%d" % (si + 1, b)
            res = (xq, xname)
            if b == 0:
                rq, _ = conv(xq, xname, p + "_sc", 1, out, s, 0, h, relu=False)
                res = (rq, p + "_sc")
            yq, _ = conv(xq, xname, p + "_c1", 1, mid, 1, 0, h)
            yq, h2 = conv(yq, p + "_c1", p + "_c2", 3, mid, s, 1, h)
            xq, _ = conv(yq, p + "_c2", p + "_c3", 1, out, 1, 0, h2, res=res)
            xname = p + "_c3"
            h = h2
    xd = g.Dequantize(xq, scale(xname), None, 0, F32, "gap_dq")
    x = g.ReduceMean(xd, (1, 2), True, (batch, 1, 1, 2048), "gap")
    x = g.Reshape(x, (batch, 2048), "flatten")
    pq = g.Quantize(x, scale("pool"), None, 0, I8, "pool_q")
    if "pool" in extra_outputs:
        g.Output(pq)
    pd = g.Dequantize(pq, scale("pool"), None, 0, F32, "pool_dq")
    Wq = g.Constant("fc_w_q", wq["fc_w_q"])
    Ws = g.Constant("fc_w_s", wq["fc_w_s"])
    wd = g.Dequantize(Wq, Ws, None, 1, F32, "fc_wdq")
    Bf = g.Constant("fc_b", w["fc_b"])
    x = g.Gemm(pd, False, wd, False, 1.0, 1.0, Bf, (batch, 1000), "logits")
    if softmax:
        x = g.Softmax(x, -1, "prob")
    g.Output(x)
    return g
