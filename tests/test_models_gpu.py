"""Whole-graph parity on the GPU: the benchmark networks (MNIST regression, ResNet-50, YOLOv3, BERT) at sizes the CPU oracle finishes in
seconds, the HALO-style model.cc linked against both libraries, multi-GPU sharding, host-side fault
injection, and size-independent properties at the full batch size."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mnist_softmax_regression(odla, gpu_lib, ref, models):
    x = models.mnist.inputs()
    outs = []
    for L, fp16 in ((gpu_lib, False), (ref, False), (gpu_lib, True)):
        g = odla.Graph(L, "mnist_simple", fp16=fp16)
        models.mnist.build(g)
        outs.append(g.run(x)["y"])
        g.close()
    assert np.abs(outs[0] - outs[1]).max() < 1e-5
    assert np.abs(outs[2] - outs[1]).max() < 1e-2 and (outs[2].argmax(1) == outs[1].argmax(1)).mean() >= 0.95


@pytest.fixture(scope="module")
def rn_weights(models):
    return models.resnet50.weights()


@pytest.fixture(scope="module")
def rn_oracle_fp32(odla, ref, models, rn_weights):
    """fp32 oracle outputs (soft-max and logits) for 2 images; ~20 s of CPU work, shared by the tests."""
    rn = models.resnet50
    x = rn.inputs(2)
    g = odla.Graph(ref, "resnet50")
    rn.build(g, 2, rn_weights)
    prob = g.run(x)["prob"]
    n = ref.cpuref_GetValueData(g.comp, b"logits", None, 0)
    logits = np.zeros(n // 4, np.float32)
    ref.cpuref_GetValueData(g.comp, b"logits", logits.ctypes.data, n)
    g.close()
    return x, prob, logits.reshape(2, 1000)


def test_resnet50_fp32_matches_oracle(odla, gpu_lib, models, rn_weights, rn_oracle_fp32):
    x, prob, _ = rn_oracle_fp32
    g = odla.Graph(gpu_lib, "resnet50")
    models.resnet50.build(g, 2, rn_weights)
    got = g.run(x)["prob"]
    g.close()
    assert np.abs(got - prob).max() < 1e-4           # the reference's unit-test threshold
    assert (got.argmax(1) == prob.argmax(1)).all()


@pytest.mark.parametrize("mode", ["fp16", "bf16"])
def test_resnet50_half_precision_within_tolerance(odla, gpu_lib, models, rn_weights, rn_oracle_fp32, mode):
    x, prob, logits = rn_oracle_fp32
    g = odla.Graph(gpu_lib, "resnet50", fp16=(mode == "fp16"), bf16=(mode == "bf16"))
    models.resnet50.build(g, 2, rn_weights)
    got = g.run(x)["prob"]
    desc = g.describe(first_gpu_only=True)
    g.close()
    assert desc.count("conv_umma") >= 52               # everything but (at most) the 3-channel stem runs on the tensor cores
    assert np.abs(got - prob).max() <= 1e-2            # max-abs 1e-2 against the fp32 reference
    assert (got.argmax(1) == prob.argmax(1)).all()     # top-1 agreement
    if mode == "fp16":
        assert np.abs(got - prob).max() <= 2e-3


def test_resnet50_int8_is_bit_exact(odla, gpu_lib, ref, models, rn_weights):
    """Every requantised int8 tensor that leaves a convolution block, the int8 pooled features and
    the final probabilities, for 2 images, against the CPU oracle."""
    rn = models.resnet50
    scales = rn.calibrate(rn_weights, n_images=8)
    wq = rn.quantize_weights(rn_weights)
    taps = ("conv1", "s1b0_sc", "s1b0_c3", "s2b0_c2", "s3b5_c3", "s4b2_c3", "pool")
    x = rn.inputs(2)
    outs = []
    for L in (gpu_lib, ref):
        g = odla.Graph(L, "resnet50_int8")
        rn.build_int8(g, 2, rn_weights, wq, scales, extra_outputs=taps)
        outs.append(g.run(x))
        if L is gpu_lib:
            desc = g.describe(first_gpu_only=True)
        g.close()
    got, want = outs
    assert desc.count("conv_umma") >= 52 and "gemm_umma" in desc
    for k in want:
        if want[k].dtype == np.int8:
            assert np.array_equal(got[k], want[k]), "%s: %d of %d differ" % (k, int((got[k] != want[k]).sum()), want[k].size)
    assert int(np.abs(want["s4b2_c3_q"].astype(int)).max()) > 20     # the tensors are not trivially zero
    assert np.abs(got["prob"] - want["prob"]).max() < 1e-6


def test_full_batch_properties_fp16(odla, gpu_lib, models, rn_weights):
    """At the benchmark batch size (256) the oracle is out of reach; use properties instead: each
    image's result is independent of its batch neighbours and of its position in the batch, and
    probabilities sum to one."""
    rn = models.resnet50
    B = 256
    x = rn.inputs(B)["input"]
    g = odla.Graph(gpu_lib, "resnet50", fp16=True)
    rn.build(g, B, rn_weights)
    a = g.run({"input": x})["prob"]
    perm = np.random.default_rng(0).permutation(B)
    b = g.run({"input": np.ascontiguousarray(x[perm])})["prob"]
    g.close()
    assert np.array_equal(a[perm], b)                      # bitwise: same kernels, same per-row arithmetic
    np.testing.assert_allclose(a.sum(1), 1.0, atol=1e-3)
    g = odla.Graph(gpu_lib, "resnet50", fp16=True)
    rn.build(g, 2, rn_weights)
    c = g.run({"input": np.ascontiguousarray(x[:2])})["prob"]
    g.close()
    assert np.abs(c - a[:2]).max() < 1e-3                  # a different tile decomposition may reorder nothing but the batch rows


def _run_pair(odla, gpu_lib, ref, build, inputs, **gpu_mode):
    outs = []
    for L in (gpu_lib, ref):
        g = odla.Graph(L, "m", **(gpu_mode if L is gpu_lib else {}))
        build(g)
        outs.append(g.run(inputs))
        desc = g.describe(first_gpu_only=True) if L is gpu_lib else None
        if L is gpu_lib:
            d = desc
        g.close()
    return outs[0], outs[1], d


@pytest.mark.parametrize("mode", ["fp32", "fp16"])
def test_yolov3_heads_match_oracle(odla, gpu_lib, ref, models, mode):
    """Darknet-53 + three heads (75 convolutions, LeakyRelu epilogues, residual adds after the
    activation, nearest upsample, channel concat), 96x96 input so the oracle finishes in seconds."""
    yo = models.yolov3
    w = yo.weights()
    x = yo.inputs(2, size=96)
    got, want, desc = _run_pair(odla, gpu_lib, ref, lambda g: yo.build(g, 2, w, size=96), x, fp16=(mode == "fp16"))
    assert [v.shape for v in want.values()] == [(2, 3, 3, 255), (2, 6, 6, 255), (2, 12, 12, 255)]
    if mode == "fp16":
        assert desc.count("conv_umma") == 75 and "resize" in desc and "concat" in desc
        assert desc.count("binary") == 0        # every residual Add was folded into a convolution epilogue
    for k in want:
        scale = float(np.abs(want[k]).max())
        err = float(np.abs(got[k] - want[k]).max())
        assert err <= (1e-4 if mode == "fp32" else 2e-2) * max(scale, 1.0), (k, err, scale)


@pytest.mark.parametrize("mode,cfg", [("fp32", dict(vocab=500, hidden=64, heads=4, ffn=256, layers=2, seq=16)),
                                      ("fp16", dict(vocab=500, hidden=64, heads=4, ffn=256, layers=2, seq=16)),
                                      ("fp16", dict(vocab=30522, hidden=768, heads=12, ffn=3072, layers=1, seq=128))])
def test_bert_encoder_matches_oracle(odla, gpu_lib, ref, models, mode, cfg):
    """Embedding gather, LayerNorm, Q/K/V/out/FFN Gemms with bias (+GELU) epilogues, head split/merge
    transposes, batched score and context Gemms, soft-max; a small configuration in fp32 and fp16
    and one full-width BERT-base layer in fp16."""
    be = models.bert
    w = be.weights(cfg)
    x = be.inputs(cfg, 2)
    got, want, desc = _run_pair(odla, gpu_lib, ref, lambda g: be.build(g, 2, cfg, w), x, fp16=(mode == "fp16"))
    err = float(np.abs(got["encoder_out"] - want["encoder_out"]).max())
    assert err <= (2e-4 if mode == "fp32" else 3e-2), err
    if mode == "fp16":
        # Q/K/V/out/FFN on the tensor-core Gemm; heads of 128 positions x 64 channels take the fused attention launch
        # (scores product, 1/sqrt(d) Mul, soft-max and context product in one), other shapes the separate kernels
        fused_attention = cfg["seq"] == 128 and cfg["hidden"] // cfg["heads"] == 64
        assert desc.count("gemm_umma") == 6 * cfg["layers"] and "layernorm" in desc and "gather" in desc
        assert desc.count("attention") == (cfg["layers"] if fused_attention else 0)
        if fused_attention:
            assert "softmax" not in desc and "binary       l0_scaled" not in desc
        assert "transpose" not in desc                        # head split / merge ride on the Gemm / attention stores


def test_halo_style_model_runs_against_both_libraries(tmp_path, odla, gpu_lib, ref, models):
    """mnist_simple.cc (emitted in the shape of HALO's generator) + its constants object + a main(),
    linked once with -lodla_b200 and once with the oracle platform: same probabilities."""
    g = odla.Graph(ref, "mnist_simple")
    models.mnist.build(g)
    (tmp_path / "model.cc").write_text(g.emit_cc())
    g.write_constants(str(tmp_path / "model.bin"), str(tmp_path / "model.S"))
    g.close()
    x = models.mnist.inputs()["x"]
    x.tofile(tmp_path / "x.bin")
    (tmp_path / "main.cc").write_text(r'''
#include <cstdio>
extern "C" int mnist_simple(const float*, float*);
extern "C" int mnist_simple_fini();
int main(int argc, char** argv) {
  static float x[64 * 784], y[640];
  FILE* f = fopen(argv[1], "rb"); if (!f || fread(x, 4, 64 * 784, f) != 64 * 784) return 2; fclose(f);
  for (int i = 0; i < 2; ++i) if (mnist_simple(x, y) != 0) return 1;     // bind-and-run twice, like a serving loop
  f = fopen(argv[2], "wb"); fwrite(y, 4, 640, f); fclose(f);
  return mnist_simple_fini();
}''')
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-c", str(tmp_path / "model.cc"), "-o", str(tmp_path / "model.o")], check=True)
    subprocess.run(["gcc", "-c", str(tmp_path / "model.S"), "-o", str(tmp_path / "weights.o")], check=True)
    res = {}
    for tag, path in (("b200", gpu_lib.path), ("cpuref", ref.path)):
        d, n = os.path.dirname(path), os.path.basename(path)[3:-3]
        exe = tmp_path / ("app_" + tag)
        subprocess.run(["g++", str(tmp_path / "main.cc"), str(tmp_path / "model.o"), str(tmp_path / "weights.o"), "-o", str(exe), "-L", d, "-l" + n,
                        "-Wl,-rpath," + d], check=True)
        subprocess.run([str(exe), str(tmp_path / "x.bin"), str(tmp_path / (tag + ".out"))], check=True)
        res[tag] = np.fromfile(tmp_path / (tag + ".out"), np.float32)
    assert np.abs(res["b200"] - res["cpuref"]).max() < 1e-5


def test_device_resident_bindings_and_timing(odla, gpu_lib, models):
    import torch
    g = odla.Graph(gpu_lib, "mnist_simple")
    models.mnist.build(g)
    x = models.mnist.inputs()["x"]
    want = g.run({"x": x})["y"]
    xd = torch.from_numpy(x).cuda()
    yd = torch.zeros((64, 10), dtype=torch.float32, device="cuda")
    g.bind_input("x", xd.data_ptr())
    g.bind_output("y", yd.data_ptr())
    assert g.execute() == 0
    assert np.array_equal(yd.cpu().numpy(), want)
    assert g.device_ms() > 0 and g.launches() >= 2
    prof = g.profile(2)
    assert [p["op"] for p in prof] == ["gemm_simt", "softmax"] and all(p["ms"] > 0 for p in prof)
    g.close()


def test_host_side_fault_injection_unwinds_cleanly(odla, gpu_lib, models):
    """A failing copy or launch (made on the host: the n-th call of a site reports an error without
    touching the GPU) must surface as an error status, leave the streams idle, and the next execute
    must succeed with the right answer."""
    g = odla.Graph(gpu_lib, "mnist_simple")
    models.mnist.build(g)
    x = models.mnist.inputs()
    want = g.run(x)["y"]
    gpu_lib.SetLogLevel(0)
    try:
        for site in ("h2d", "launch", "d2h"):
            os.environ["ODLA_B200_INJECT"] = site + "@1"
            with pytest.raises(RuntimeError):
                g.run(x)
            del os.environ["ODLA_B200_INJECT"]
            assert np.array_equal(g.run(x)["y"], want)
    finally:
        os.environ.pop("ODLA_B200_INJECT", None)
        gpu_lib.SetLogLevel(3)
    g.close()


def test_batch_is_sharded_over_every_visible_gpu(odla, gpu_lib, ref, models):
    """With more than one GPU the batch is split into contiguous shards (uneven when it does not
    divide, fewer GPUs than requested when the batch is smaller); results equal the oracle's."""
    n = gpu_lib.b200_DeviceCount()
    x = models.mnist.inputs(batch=11)
    gr = odla.Graph(ref, "m")
    models.mnist.build(gr, batch=11)
    want = gr.run(x)["y"]
    gr.close()
    for want_gpus in sorted({1, min(2, n), n, n + 3}):
        g = odla.Graph(gpu_lib, "m", n_gpus=want_gpus)
        models.mnist.build(g, batch=11)
        got = g.run(x)["y"]
        desc = g.describe()
        g.close()
        assert np.abs(got - want).max() < 1e-5
        assert desc.count("gpu ") == min(want_gpus, n, 11)


@pytest.mark.parametrize("mode,batch", [("int8", 250), ("int8", 5), ("fp16", 64)])
def test_resnet50_sharded_over_the_gpus_equals_one_gpu(odla, gpu_lib, models, rn_weights, mode, batch):
    """One odla_ExecuteComputation shards dim 0 over every visible GPU (uneven shards at 250 images, fewer GPUs than
    visible at 5); each image's result is bit-identical to the single-GPU run: rows are independent and every GPU runs
    the same kernels.  On a one-GPU machine both runs take the same path and the test only checks the plumbing."""
    rn = models.resnet50
    n = gpu_lib.b200_DeviceCount()
    x = rn.inputs(batch, seed=99)
    outs = []
    for gpus in (1, n):
        g = odla.Graph(gpu_lib, "resnet50_" + mode, fp16=(mode == "fp16"), n_gpus=gpus)
        if mode == "int8":
            sc = {k: np.float32(0.05) for k in ["input", "pool"] + [c[0] for c in rn.conv_list()]}
            rn.build_int8(g, batch, rn_weights, rn.quantize_weights(rn_weights), sc, extra_outputs=("s1b0_c3", "s4b2_c3"))
        else:
            rn.build(g, batch, rn_weights)
        outs.append(g.run(x))
        assert g.describe().count("gpu ") == min(gpus, batch)
        shards = g.plan_shards(gpus)
        assert sum(s[2] for s in shards) == batch and len(shards) == min(gpus, batch)
        g.close()
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k]), k


@pytest.mark.parametrize("mode", ["fp16", "int8"])
def test_stored_executable_runs_like_the_original(tmp_path, odla, gpu_lib, models, rn_weights, mode):
    """A ResNet-50 stored after its first execute carries the prepared constants (filters converted and repacked
    K-major); the loaded computation plans from them without converting anything again and returns identical bits."""
    rn = models.resnet50
    x = rn.inputs(4, seed=21)
    g = odla.Graph(gpu_lib, "resnet50", fp16=(mode == "fp16"))
    if mode == "int8":
        sc = {k: np.float32(0.05) for k in ["input", "pool"] + [c[0] for c in rn.conv_list()]}
        rn.build_int8(g, 4, rn_weights, rn.quantize_weights(rn_weights), sc)
    else:
        rn.build(g, 4, rn_weights)
    want = g.run(x)["prob"]
    st = g.prepared_stats()
    assert st["misses"] >= 54 and st["entries"] == st["misses"]     # every convolution filter and the classifier's matrix
    path = str(tmp_path / "resnet50.odlab200")
    g.store(path)
    g.close()
    h = odla.Graph.load(gpu_lib, path)
    got = h.run(x)["prob"]
    st = h.prepared_stats()
    h.close()
    assert st["misses"] == 0 and st["hits"] >= 54
    assert np.array_equal(got, want)


def test_sub_batches_pipeline_one_gpu(odla, gpu_lib, models, rn_weights):
    """ODLA_BATCHES_PER_STEP = S gives every GPU S replicas (own stream and arena) so that copies of one
    sub-batch overlap kernels of another; an image's result does not depend on how the batch was cut."""
    rn = models.resnet50
    x = rn.inputs(6)
    outs, descs = [], []
    for s in (1, 2, 4, 16):
        g = odla.Graph(gpu_lib, "resnet50", fp16=True, n_gpus=1, sub_batches=s)
        rn.build(g, 6, rn_weights)
        outs.append(g.run(x)["prob"])
        descs.append(g.describe())
        g.close()
    assert [d.count("gpu ") for d in descs] == [1, 2, 4, 6]        # never more sub-batches than images
    # inputs are the larger transfer here, so the sub-batches grow (1 : 3 : 9 ...): the exposed first copy is short
    assert "rows [0,1)" in descs[1] and "rows [1,6)" in descs[1] and "rows [0,1)" in descs[2] and "rows [3,6)" in descs[2]
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])


def test_run_batch_size_and_async_execute(odla, gpu_lib, ref, models):
    """ODLA_RUN_BATCH_SIZE runs the first n rows of the recorded batch through a plan of its own (kept for the
    next call); odla_AsyncExecuteComputation returns before the outputs are written and calls back when they are."""
    import threading
    x = models.mnist.inputs(batch=64)["x"]
    gr = odla.Graph(ref, "m")
    models.mnist.build(gr, batch=64)
    want = gr.run({"x": x})["y"]
    gr.close()
    g = odla.Graph(gpu_lib, "m")
    models.mnist.build(g, batch=64)
    for n in (10, 64, 1, 10):
        xin, out = np.ascontiguousarray(x[:n]), np.full((n, 10), -1.0, np.float32)
        g.bind_input("x", xin.ctypes.data)
        g.bind_output("y", out.ctypes.data)
        assert g.set_run_batch(n) == 0
        assert g.execute() == 0
        assert np.abs(out - want[:n]).max() < 1e-5
        shp = odla.Shape()
        gpu_lib.GetRuntimeShape(g.context(), g.value_handle("y"), C.byref(shp))
        assert list(shp.dims[:2]) == [n, 10]
    gpu_lib.SetLogLevel(0)
    assert g.set_run_batch(65) == 0 and g.execute() == odla.INVALID_PARAM      # more rows than were recorded
    gpu_lib.SetLogLevel(3)
    # asynchronous execute with a callback
    assert g.set_run_batch(0) == 0
    out = np.full((64, 10), -1.0, np.float32)
    g.bind_input("x", x.ctypes.data)
    g.bind_output("y", out.ctypes.data)
    done, seen = threading.Event(), []
    assert g.execute_async(lambda arg, status: (seen.append((arg, status)), done.set(), 0)[2], 77) == 0
    assert done.wait(30) and seen == [(77, 0)]
    assert g.wait() == 0 and np.abs(out - want).max() < 1e-5
    # without a callback: the next call on the context waits
    out[:] = -1
    assert g.execute_async() == 0 and g.wait() == 0 and np.abs(out - want).max() < 1e-5
    # the computation may be destroyed before the context, right after an asynchronous execute (the order the
    # reference's PopART test uses): the library waits for the work, the outputs are complete
    out[:] = -1
    assert g.execute_async() == 0
    assert gpu_lib.DestroyComputation(g.comp) == 0
    assert np.abs(out - want).max() < 1e-5
    assert gpu_lib.DestroyContext(g.ctx) == 0
    g.comp, g.ctx = odla._V(), None


def test_two_contexts_in_flight(odla, gpu_lib, models, rn_weights):
    """Two contexts of one computation execute at the same time, each on arenas and streams of its own: results are
    those of the contexts run one after the other, bit for bit, over many overlapping steps with different inputs;
    a third context shares a lane with the first and takes turns with it."""
    rn = models.resnet50
    B = 32
    xs = [rn.inputs(B, seed=s)["input"] for s in (1, 2, 3)]
    g = odla.Graph(gpu_lib, "resnet50", fp16=True, sub_batches=2)
    rn.build(g, B, rn_weights)
    want = [g.run({"input": x})["prob"].copy() for x in xs]
    assert not np.array_equal(want[0], want[1])
    ctxs = [g, g.extra_context(), g.extra_context()]
    outs = [np.full((B, 1000), -1.0, np.float32) for _ in ctxs]
    for c, x, o in zip(ctxs, xs, outs):
        c.bind_input("input", x.ctypes.data)
        c.bind_output("prob", o.ctypes.data)
    for step in range(12):
        for c in ctxs:
            assert c.wait() == 0
            assert c.execute_async() == 0
        if step % 4 == 3:
            for c, o, w in zip(ctxs, outs, want):
                assert c.wait() == 0
                assert np.array_equal(o, w)
                o[:] = -1.0
    for c in ctxs:
        assert c.wait() == 0
    # synchronous executes from two host threads at once
    import threading
    errs = []

    def worker(c, o, w):
        for _ in range(5):
            o[:] = -1.0
            if c.execute() != 0 or not np.array_equal(o, w):
                errs.append(1)
    ts = [threading.Thread(target=worker, args=(c, o, w)) for c, o, w in zip(ctxs, outs, want)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs
    g.close()
