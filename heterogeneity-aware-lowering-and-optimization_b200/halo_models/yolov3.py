"""YOLOv3 (Darknet-53 backbone, three detection heads) as an NHWC ODLA graph with random weights.

Shaped like the reference's checked-in HALO output for this network
(models/vision/detection/popart/yolov3_test.cc.popart.cc:1375-1399): every convolution has a null
bias argument and is followed by ``odla_Add`` with the folded batch-norm offset and
``odla_LeakyRelu(0.1)``; residual blocks are a plain ``odla_Add``; the heads use ``odla_Resize``
(nearest, x2) and ``odla_Concat`` on the channel axis; the three outputs are the raw head tensors
(255 channels each, no activation, no NMS)."""
import numpy as np

from .. import odla

MAC_PER_IMAGE_416 = 32932037632
BACKBONE = [(32, 3, 1, 0), (64, 3, 2, 1), (128, 3, 2, 2), (256, 3, 2, 8), (512, 3, 2, 8), (1024, 3, 2, 4)]  # (channels, k, stride, residual blocks)


def conv_specs():
    """(name, k, cin, cout, stride, linear) for the 75 convolutions in build order."""
    specs, cin, idx = [], 3, [0]

    def add(cout, k, stride, c_in, linear=False):
        specs.append(("conv%d" % idx[0], k, c_in, cout, stride, linear))
        idx[0] += 1
        return cout

    for ch, k, s, nres in BACKBONE:
        cin = add(ch, k, s, cin)
        for _ in range(nres):
            add(ch // 2, 1, 1, cin)
            add(ch, 3, 1, ch // 2)
    c = 1024
    for width, extra in ((512, 0), (256, 512), (128, 256)):
        if extra:
            add(width, 1, 1, c)          # branch conv before the upsample
            c = width + extra            # after concat with the backbone route
        for i in range(3):
            c = add(width, 1, 1, c)
            c = add(width * 2, 3, 1, c)
            if i == 2:
                add(255, 1, 1, c, linear=True)
                c = width                # the branch leaves from the last 1x1 (before the final 3x3)
        # note: the loop above emits 1x1,3x3,1x1,3x3,1x1,3x3,out; the branch point is the fifth conv
    return specs


def weights(seed=300):
    w = {}
    for i, (name, k, cin, cout, _, linear) in enumerate(conv_specs()):
        rng = np.random.default_rng(seed + i)
        kern = rng.standard_normal((k, k, cin, cout)) * np.sqrt(2.0 / (k * k * cin)) * (0.5 if not linear else 1.0)
        w[name + "_w"] = kern.astype(np.float32)
        w[name + "_b"] = (rng.standard_normal((1, 1, 1, cout)) * 0.1).astype(np.float32)
    return w


def inputs(batch, size=416, seed=20):
    return {"input": np.random.default_rng(seed + batch).random((batch, size, size, 3), dtype=np.float32)}


def build(g, batch, w, size=416, input_type=odla.FLOAT32):
    NHWC, SIO = odla.CHANNELS_LAST, odla.SIO
    specs = iter(conv_specs())
    x = g.Argument("input", (batch, size, size, 3), input_type)
    state = {"h": size}

    def conv(x, h_in):
        name, k, cin, cout, s, linear = next(specs)
        p = k // 2
        ho = (h_in + 2 * p - k) // s + 1
        W = g.Constant(name + "_w", w[name + "_w"])
        B = g.Constant(name + "_b", w[name + "_b"])
        y = g.Conv(x, NHWC, 1, W, SIO, (s, s), (1, 1), (p, p), (p, p), None, (batch, ho, ho, cout), name)
        y = g.Add(y, B, name + "_bn")
        if not linear:
            y = g.LeakyRelu(y, 0.1, name + "_act")
        return y, ho, cout

    h = size
    routes = {}
    for ch, k, s, nres in BACKBONE:
        x, h, c = conv(x, h)
        for r in range(nres):
            y, _, _ = conv(x, h)
            y, _, _ = conv(y, h)
            x = g.Add(x, y, "res_%d_%d" % (ch, r))
        routes[ch] = (x, h)
    outs = []
    c = 1024
    for width, route in ((512, None), (256, 512), (128, 256)):
        if route:
            x, _, _ = conv(branch, h)
            h *= 2
            x = g.Resize(x, (batch, h, h, width), "up_%d" % width)
            rx, rh = routes[route]
            assert rh == h
            x = g.Concat([x, rx], 3, (batch, h, h, width + route), "cat_%d" % width)
        for i in range(3):
            x, _, _ = conv(x, h)
            if i == 2:
                branch = x
            x, _, _ = conv(x, h)
        y, _, _ = conv(x, h)
        outs.append(y)
    for i, o in enumerate(outs):
        g.Output(o)
    return g
