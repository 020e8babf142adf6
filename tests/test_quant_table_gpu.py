"""Quantisation-table ingestion (ODLA_QUANT_TABLE / ODLA_QUANT_TABLE_SIZE): a float graph plus a table of
value ranges must run exactly like the hand-written Quantize/Dequantize graph with the same scales."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _scale(mn, mx):
    a = np.float32(max(abs(np.float32(mn)), abs(np.float32(mx))))
    return np.float32(a / np.float32(127.0)) if a > 0 else np.float32(1.0)


def _small_net(odla, g, w, ranges=None, transpose_fc=False):
    """conv3x3+bias+relu -> conv1x1+bias + residual -> relu -> mean -> Gemm(+bias).  With `ranges` the
    Quantize/Dequantize nodes are written out by hand, the way the table rewrite is documented to place them."""
    NHWC, SIO, F32, I8 = odla.CHANNELS_LAST, odla.SIO, odla.FLOAT32, odla.INT8
    B, H, C0, C1 = 4, 16, 32, 64

    def q_act(x, name):
        if ranges is None:
            return x
        s = g.Constant(name + "_s", np.array([_scale(*ranges[name])], np.float32))
        return g.Dequantize(g.Quantize(x, s, None, 0, I8, name + "_q"), s, None, 0, F32, name + "_dq")

    def q_w(name, axis, k_first=False):
        a = w[name]
        if ranges is None:
            return g.Constant(name, a)
        m = a.reshape(a.shape[0], -1) if k_first else a.reshape(-1, a.shape[-1]).T          # [K, rest]
        s = np.array([_scale(r.min(initial=0.0), r.max(initial=0.0)) for r in m], np.float32)
        sb = s.reshape((-1,) + (1,) * (a.ndim - 1)) if k_first else s
        aq = np.clip(np.rint(a / sb), -127, 127).astype(np.int8)
        return g.Dequantize(g.Constant(name + "_q", aq), g.Constant(name + "_qs", s), None, axis, F32, name + "_dq")

    x = g.Argument("x", (B, H, H, C0), F32)
    y = g.Conv(q_act(x, "x"), NHWC, 1, q_w("w1", 3), SIO, (1, 1), (1, 1), (1, 1), (1, 1), None, (B, H, H, C1), "c1")
    y = g.Relu(g.Add(y, g.Constant("b1", w["b1"]), "c1_b"), "r1")
    z = g.Conv(q_act(y, "r1"), NHWC, 1, q_w("w2", 3), SIO, (1, 1), (1, 1), (0, 0), (0, 0), None, (B, H, H, C1), "c2")
    z = g.Relu(g.Add(g.Add(z, g.Constant("b2", w["b2"]), "c2_b"), y, "c2_res"), "r2")
    p = g.Reshape(g.ReduceMean(z, (1, 2), True, (B, 1, 1, C1), "gap"), (B, C1), "flat")
    if transpose_fc:
        out = g.Gemm(q_act(p, "flat"), False, q_w("wfc_t", 0, k_first=True), True, 1.0, 1.0, g.Constant("bfc", w["bfc"]), (B, 10), "fc")
    else:
        out = g.Gemm(q_act(p, "flat"), False, q_w("wfc", 1), False, 1.0, 1.0, g.Constant("bfc", w["bfc"]), (B, 10), "fc")
    g.Output(z)
    g.Output(out)
    return g


def _weights():
    rng = np.random.default_rng(5)
    w = {"w1": rng.standard_normal((3, 3, 32, 64)).astype(np.float32) * 0.06, "b1": rng.standard_normal(64).astype(np.float32) * 0.1,
         "w2": rng.standard_normal((1, 1, 64, 64)).astype(np.float32) * 0.12, "b2": rng.standard_normal(64).astype(np.float32) * 0.1,
         "wfc": rng.standard_normal((64, 10)).astype(np.float32) * 0.1, "bfc": rng.standard_normal(10).astype(np.float32) * 0.1}
    w["wfc_t"] = np.ascontiguousarray(w["wfc"].T)
    return w, rng.standard_normal((4, 16, 16, 32)).astype(np.float32)


@pytest.mark.parametrize("transpose_fc", [False, True])
def test_table_equals_handwritten_qdq_graph(odla, gpu_lib, ref, transpose_fc):
    w, x = _weights()
    ranges = {"x": (-3.1, 2.7), "r1": (0.0, 4.5), "flat": (0.0, 1.9)}     # one range deliberately asymmetric
    # the table: one tensor record per activation (ch_idx = -channels), as the reference's profiler script writes it
    records = [(k, -1, 0.0, 0.0, mn, mx) for k, (mn, mx) in ranges.items()]
    g = _small_net(odla, odla.Graph(gpu_lib, "qt"), w, transpose_fc=transpose_fc)
    g.set_quant_table(records)
    got = g.run({"x": x})
    desc = g.describe(first_gpu_only=True)
    g.close()
    # the operands were absorbed: both convolutions and the Gemm run on the int8 tensor-core kernel
    assert desc.count("conv_umma") == 2 and "quantize" in desc
    h = _small_net(odla, odla.Graph(ref, "qt_ref"), w, ranges=ranges, transpose_fc=transpose_fc)
    want = h.run({"x": x})
    h.close()
    f = _small_net(odla, odla.Graph(ref, "qt_f32"), w, transpose_fc=transpose_fc)
    flt = f.run({"x": x})
    f.close()
    for k in ("r2", "fc"):
        assert np.array_equal(got[k], want[k]), (k, float(np.abs(got[k] - want[k]).max()))
        # and int8 really happened: the result differs from the float graph, by quantisation noise only
        d = float(np.abs(got[k] - flt[k]).max())
        assert 0 < d < 1.0, (k, d)


def test_table_with_per_channel_weight_records_and_direct_scale(odla, gpu_lib, ref):
    """Weight ranges given per channel in the table override the constant's own ranges; a record with
    min = max = 0 and a positive scale supplies the scale directly."""
    w, x = _weights()
    rng = np.random.default_rng(11)
    NHWC, SIO, F32, I8 = odla.CHANNELS_LAST, odla.SIO, odla.FLOAT32, odla.INT8
    sx = np.float32(0.031)
    ch_rng = [(-float(a), float(a) * 0.5) for a in (np.abs(w["w1"]).reshape(-1, 64).max(0) * rng.uniform(0.6, 1.0, 64))]
    # a constant's value id is its symbol plus "_" (include/halo/lib/target/generic_cxx/generic_cxx_codegen.h:292-314 in the reference)
    records = [("x", -1, float(sx), 0.0, 0.0, 0.0), ("w1_", -64, 0.0, 0.0, -1.0, 1.0)] + [("w1_", c, 0.0, 0.0, mn, mx) for c, (mn, mx) in enumerate(ch_rng)]

    def net(g, table):
        xa = g.Argument("x", (4, 16, 16, 32), F32)
        if table:
            xin, win = xa, g.Constant("w1", w["w1"])
        else:
            s = g.Constant("x_s", np.array([sx], np.float32))
            xin = g.Dequantize(g.Quantize(xa, s, None, 0, I8, "x_q"), s, None, 0, F32, "x_dq")
            sw = np.array([_scale(mn, mx) for mn, mx in ch_rng], np.float32)
            wq = np.clip(np.rint(w["w1"] / sw), -127, 127).astype(np.int8)     # out-of-range weights saturate
            win = g.Dequantize(g.Constant("w1_q", wq), g.Constant("w1_s", sw), None, 3, F32, "w1_dq")
        y = g.Conv(xin, NHWC, 1, win, SIO, (1, 1), (1, 1), (1, 1), (1, 1), None, (4, 16, 16, 64), "c1")
        g.Output(g.Relu(g.Add(y, g.Constant("b1", w["b1"]), "c1_b"), "r1"))
        return g

    g = net(odla.Graph(gpu_lib, "qt2"), True)
    g.set_quant_table(records)
    got = g.run({"x": x})["r1"]
    g.close()
    h = net(odla.Graph(ref, "qt2_ref"), False)
    want = h.run({"x": x})["r1"]
    h.close()
    assert np.array_equal(got, want), float(np.abs(got - want).max())


def test_resnet50_float_graph_with_table_runs_int8(odla, gpu_lib, models):
    """The fp32 ResNet-50 graph plus a table made from the calibration ranges: every convolution and the
    FC layer run in int8, and the classifier still agrees with the float run."""
    rn = models.resnet50
    w = rn.weights()
    scales = rn.calibrate(w, n_images=8)
    x = rn.inputs(8)
    g = odla.Graph(gpu_lib, "resnet50", fp16=True)
    rn.build(g, 8, w)
    ref_prob = g.run(x)["prob"]
    g.close()
    records = []
    for name, s in scales.items():
        if name.endswith("_sc"):
            continue                     # projection shortcuts feed only the residual additions
        # the stem's range also holds for the max-pool output, which is what the first block reads
        vid = {"input": "input", "pool": "flatten", "conv1": "pool1"}.get(name, name + "_relu")
        a = float(s) * 127.0
        records.append((vid, -1, 0.0, 0.0, -a, a))
    g = odla.Graph(gpu_lib, "resnet50_qt", fp16=True)
    rn.build(g, 8, w)
    g.set_quant_table(records)
    prob = g.run(x)["prob"]
    desc = g.describe(first_gpu_only=True)
    g.close()
    assert desc.count("_qt_q") + desc.count("quantize") >= 16          # activations are quantised ...
    assert np.abs(prob - ref_prob).max() < 0.1                            # ... and the result stays close to the float run
    assert (prob.argmax(1) == ref_prob.argmax(1)).mean() >= 0.75
    cc = g.emit_cc()
    assert "extern const odla_value_quant_info quant_infos[];" in cc and "ODLA_QUANT_TABLE_SIZE" in cc
    assert "quant_infos_size = %d" % len(records) in g.emit_quant_table_c()


def test_range_profiler_matches_host_ranges(odla, gpu_lib, ref):
    """odla_b200_SetRangeProfiling + odla_b200_GetQuantTable: per-value and per-channel min / max of every materialised
    value, accumulated over two calibration executes, against numpy on the oracle's values; halo_pgq's record layout."""
    rng = np.random.default_rng(3)
    w1 = (rng.standard_normal((3, 3, 8, 16)) * 0.2).astype(np.float32)
    b1 = rng.standard_normal((1, 1, 1, 16)).astype(np.float32)
    xs = [rng.standard_normal((2, 10, 10, 8)).astype(np.float32) * s for s in (1.0, 3.0)]

    def net(g):
        x = g.Argument("x", (2, 10, 10, 8))
        y = g.Conv(x, odla.CHANNELS_LAST, 1, g.Constant("w1", w1), odla.SIO, (1, 1), (1, 1), (1, 1), (1, 1), None, (2, 10, 10, 16), "c1")
        r = g.Relu(g.Add(y, g.Constant("b1", b1), "c1_b"), "r1")
        p = g.MaxPool(r, odla.CHANNELS_LAST, (2, 2), (2, 2), (0, 0), (0, 0), (2, 5, 5, 16), "p1")
        g.Output(g.Reshape(p, (2, 400), "flat"))
        g.Output(r)
        return g

    g = net(odla.Graph(gpu_lib, "prof"))
    g.range_profiling(True)
    for x in xs:
        g.run({"x": x})
    table = g.quant_table()
    g.range_profiling(False)
    g.close()
    h = net(odla.Graph(ref, "prof_ref"))
    want = [h.run({"x": x}) for x in xs]
    h.close()
    rec = {}
    for vid, ch, scale, off, mn, mx in table:
        rec.setdefault(vid, []).append((ch, scale, off, mn, mx))
    assert set(rec) == {"x", "r1", "p1", "flat"}                       # c1 and c1_b only exist inside the fused kernel
    r1 = np.concatenate([o["r1"] for o in want])
    for vid, arr in (("x", np.concatenate(xs)), ("r1", r1)):
        head = rec[vid][0]
        assert head[0] == -arr.shape[-1] and head[2] == 0.0
        np.testing.assert_allclose([head[3], head[4]], [arr.min(), arr.max()], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(head[1], max(abs(arr.min()), abs(arr.max())) / 127.0, rtol=1e-5)
        chans = rec[vid][1:]
        assert [c[0] for c in chans] == list(range(arr.shape[-1]))
        np.testing.assert_allclose([c[3] for c in chans], arr.reshape(-1, arr.shape[-1]).min(0), rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose([c[4] for c in chans], arr.reshape(-1, arr.shape[-1]).max(0), rtol=1e-5, atol=1e-6)
    flat = np.concatenate([o["flat"] for o in want])
    assert len(rec["flat"]) == 1 and rec["flat"][0][0] == -1
    np.testing.assert_allclose(rec["flat"][0][4], flat.max(), rtol=1e-5)


def test_resnet50_calibrated_on_the_gpu_runs_int8(odla, gpu_lib, models):
    """Calibration without the host: the float graph profiles its own ranges on a calibration batch, the table goes
    back in through ODLA_QUANT_TABLE, and the int8 plan agrees with the float run."""
    rn = models.resnet50
    w = rn.weights()
    x = rn.inputs(8)
    g = odla.Graph(gpu_lib, "resnet50", fp16=True)
    rn.build(g, 8, w)
    ref_prob = g.run(x)["prob"]
    g.range_profiling(True)
    g.run(rn.inputs(8, seed=77))
    table = g.quant_table()
    g.range_profiling(False)
    g.close()
    ids = {t[0] for t in table}
    assert {"input", "pool1", "s1b0_c1_relu", "s4b2_c3_relu", "flatten"} <= ids
    q = odla.Graph(gpu_lib, "resnet50_qt", fp16=True)
    rn.build(q, 8, w)
    q.set_quant_table(table)
    prob = q.run(x)["prob"]
    desc = q.describe(first_gpu_only=True)
    q.close()
    assert desc.count("_qt_q") + desc.count("quantize") >= 16
    assert np.abs(prob - ref_prob).max() < 0.1
    assert (prob.argmax(1) == ref_prob.argmax(1)).mean() >= 0.75


def _quint8(w):
    """A float constant as -quantize-weights=quint8 leaves it (lib/quantizer/weights_quantizer.cc:84-182 of the reference):
    one scale and one zero point per tensor, q = clamp(round(w / scale + zp), 0, 255)."""
    mn, mx = min(float(w.min()), 0.0), float(w.max())
    scale = np.float32((mx - mn) / 255.0)
    zp = float(np.clip(np.round(0 - mn / scale), 0, 255))
    q = np.clip(np.round(w * np.float32(1.0 / scale) + zp), 0, 255).astype(np.uint8)
    return q, scale, int(zp)


@pytest.mark.parametrize("skew", [0.0, 0.6, -0.9])
def test_asymmetric_uint8_weights_conv_and_gemm_are_bit_exact(odla, gpu_lib, ref, skew):
    """uint8 weights with a zero point (and an int32 bias quantised with s_in * s_w), handed over as the compiler emits
    them -- QUINT8 / INT32 constants plus table records -- against the oracle's hand-written form
    Dequantize(uint8, scale, zp): int32 accumulators of sum x_q * (W_u - zp) and the requantised int8 results bit-equal.
    skew moves the zero point away from 128, which is what needs more than one int8 filter term."""
    rng = np.random.default_rng(int(abs(skew) * 10) + 1)
    F32, I8, U8, I32, NHWC, SIO = odla.FLOAT32, odla.INT8, odla.UINT8, odla.INT32, odla.CHANNELS_LAST, odla.SIO
    x = rng.standard_normal((2, 12, 12, 32)).astype(np.float32)
    w1 = (rng.standard_normal((3, 3, 32, 64)) * 0.1 + skew * 0.1).astype(np.float32)
    w2 = (rng.standard_normal((64, 48)) * 0.1 - skew * 0.1).astype(np.float32)
    (q1, s1, z1), (q2, s2, z2) = _quint8(w1), _quint8(w2)
    sx, sy = np.float32(np.abs(x).max() / 127), np.float32(0.08)
    b1 = np.round(rng.standard_normal(64) * 0.2 / (sx * s1)).astype(np.int32)           # int32 bias, scale s_in * s_w

    def net(g, table):
        xa = g.Argument("x", x.shape, F32)
        if table:
            xin, win, bias = xa, g.Constant("w1", q1), g.Constant("b1", b1)
        else:
            s = g.Constant("x_s", np.array([sx], np.float32))
            xin = g.Dequantize(g.Quantize(xa, s, None, 0, I8, "x_q"), s, None, 0, F32, "x_dq")
            win = g.Dequantize(g.Constant("w1_q", q1), g.Constant("w1_s", np.array([s1], np.float32)), g.Constant("w1_z", np.array([z1], np.int32)), 0, F32, "w1_dq")
            bias = g.Constant("b1_f", (b1.astype(np.float32) * np.float32(sx * s1)).astype(np.float32))
        y = g.Conv(xin, NHWC, 1, win, SIO, (1, 1), (1, 1), (1, 1), (1, 1), bias, (2, 12, 12, 64), "c1")
        r = g.Relu(y, "r1")
        if table:
            flat, w2in = g.Reshape(r, (288, 64), "flat"), g.Constant("w2", q2)
        else:
            s = g.Constant("y_s", np.array([sy], np.float32))
            rq = g.Quantize(g.Reshape(r, (288, 64), "flat"), s, None, 0, I8, "r1_q")     # the Gemm reads Dequantize directly: the integer rule applies
            g.Output(rq)
            flat = g.Dequantize(rq, s, None, 0, F32, "r1_dq")
            w2in = g.Dequantize(g.Constant("w2_q", q2), g.Constant("w2_s", np.array([s2], np.float32)), g.Constant("w2_z", np.array([z2], np.int32)), 0, F32, "w2_dq")
        g.Output(g.Gemm(flat, False, w2in, False, 1.0, 0.0, None, (288, 48), "fc"))
        return g

    g = net(odla.Graph(gpu_lib, "u8"), True)
    # activation records that give the scale itself (min = max = 0), weight records with the compiler's scale and zero point
    g.set_quant_table([("x", -1, float(sx), 0.0, 0.0, 0.0), ("w1_", -1, float(s1), float(z1), 0.0, 0.0), ("w2_", -1, float(s2), float(z2), 0.0, 0.0),
                       ("flat", -1, float(sy), 0.0, 0.0, 0.0)])
    got = g.run({"x": x})["fc"]
    desc = g.describe(first_gpu_only=True)
    g.close()
    h = net(odla.Graph(ref, "u8_ref"), False)
    want = h.run({"x": x})
    h.close()
    assert "conv_umma" in desc and "gemm_umma" in desc
    assert np.array_equal(got, want["fc"]), float(np.abs(got - want["fc"]).max())
    assert int(np.abs(want["r1_q"].astype(int)).max()) > 20
