"""Generates the full-size model fixtures under tests/golden/ with the CPU oracle platform.

    make -C oracle all ref && python tests/golden/make_model_golden.py [resnet50_fp32 resnet50_int8 yolov3 bert ...]

Every fixture is produced by oracle/libodla_cpuref.so executing the same graph description the GPU
tests build (halo_models/*), on seeded synthetic inputs, at the real size of the workload:

  resnet50_b32_fp32.npz   ResNet-50 v1.5 @224, batch 32, fp32: probabilities, logits of the first two images.
                          Convolution, max-pool, matmul, soft-max and relu run through the reference's own
                          runtime/generic kernels (oracle/_ref) when that library is present.
  resnet50_b32_int8.npz   the same network in quantise/dequantise form, batch 32: activation scales, a 64-bit
                          hash per image of every tapped int8 tensor, the small tapped tensors of the first two
                          images in full, and the probabilities.
  yolov3_416_b1.npz       YOLOv3 @416, batch 1, fp32 evaluation, the three raw head tensors stored as fp16.
  bert_base_b1.npz        BERT-base encoder (12 layers, S = 128), batch 1: encoder output of the float graph
                          and of the int8-GEMM form (with the activation scales it was built with), as fp16.

The inputs are not stored: the tests regenerate them from the same seeds.  Quantisation scales ARE stored,
because they come from a host-side calibration pass whose last bits depend on the host's BLAS.
"""
import hashlib
import importlib
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG = "heterogeneity-aware-lowering-and-optimization_b200"
sys.path.insert(0, ROOT)

RESNET_TAPS = ("conv1", "s1b0_sc", "s1b0_c3", "s2b0_c2", "s3b5_c3", "s4b2_c3", "pool")
RESNET_FULL_TAPS = ("s2b0_c2", "s3b5_c3", "s4b2_c3", "pool")   # stored in full for the first two images


def image_hashes(a):
    """One 64-bit hash per row of dim 0 (blake2b over the row's bytes)."""
    a = np.ascontiguousarray(a)
    return np.array([int.from_bytes(hashlib.blake2b(a[i].tobytes(), digest_size=8).digest(), "little") for i in range(a.shape[0])], dtype=np.uint64)


def resnet_inputs(rn, batch):
    """The first 32 images are always the batch-32 fixture's images; larger batches append more."""
    x = rn.inputs(32)["input"]
    if batch <= 32:
        return {"input": np.ascontiguousarray(x[:batch])}
    return {"input": np.concatenate([x, rn.inputs(batch - 32, seed=977 + batch)["input"]], axis=0)}


def bert_inputs(be, cfg, batch):
    """Sequence 0 is always the batch-1 fixture's sequence."""
    x = be.inputs(cfg, 1)["input_ids"]
    if batch == 1:
        return {"input_ids": x}
    return {"input_ids": np.concatenate([x, be.inputs(cfg, batch - 1, seed=4242)["input_ids"]], axis=0)}


def main(which):
    pkg = importlib.import_module(PKG)
    odla = pkg.odla
    ref = odla.OdlaLib(os.path.join(ROOT, "oracle", "libodla_cpuref.so"))
    kind = "runtime/generic (reference-compiled)" if ref.cpuref_UsesReference() else "restated"
    rn = importlib.import_module(PKG + ".halo_models.resnet50")
    if "resnet50_fp32" in which:
        t0 = time.time()
        w = rn.weights()
        g = odla.Graph(ref, "resnet50")
        rn.build(g, 32, w)
        prob = g.run(resnet_inputs(rn, 32))["prob"]
        n = ref.cpuref_GetValueData(g.comp, b"logits", None, 0)
        logits = np.zeros(n // 4, np.float32)
        ref.cpuref_GetValueData(g.comp, b"logits", logits.ctypes.data, n)
        g.close()
        np.savez_compressed(os.path.join(HERE, "resnet50_b32_fp32.npz"), prob=prob, logits2=logits.reshape(32, 1000)[:2], kernels=np.array(kind))
        print("resnet50_fp32: %.0f s, top-1 %s" % (time.time() - t0, prob.argmax(1)[:8]))
    if "resnet50_int8" in which:
        t0 = time.time()
        w = rn.weights()
        scales = rn.calibrate(w, n_images=32)
        wq = rn.quantize_weights(w)
        g = odla.Graph(ref, "resnet50_int8")
        rn.build_int8(g, 32, w, wq, scales, extra_outputs=RESNET_TAPS)
        out = g.run(resnet_inputs(rn, 32))
        g.close()
        rec = {"prob": out["prob"], "scale_names": np.array(sorted(scales)), "scale_values": np.array([scales[k] for k in sorted(scales)], np.float32)}
        for t in RESNET_TAPS:
            a = out[t + "_q"]
            assert a.dtype == np.int8
            rec["hash_" + t] = image_hashes(a)
            if t in RESNET_FULL_TAPS:
                rec["full_" + t] = a[:2]
        np.savez_compressed(os.path.join(HERE, "resnet50_b32_int8.npz"), **rec)
        print("resnet50_int8: %.0f s" % (time.time() - t0))
    if "yolov3" in which:
        t0 = time.time()
        yo = importlib.import_module(PKG + ".halo_models.yolov3")
        w = yo.weights()
        g = odla.Graph(ref, "yolov3")
        yo.build(g, 1, w)
        out = g.run(yo.inputs(1))
        g.close()
        np.savez_compressed(os.path.join(HERE, "yolov3_416_b1.npz"), kernels=np.array(kind), **{k: v.astype(np.float16) for k, v in out.items()})
        print("yolov3: %.0f s, heads %s" % (time.time() - t0, {k: v.shape for k, v in out.items()}))
    if "bert" in which:
        t0 = time.time()
        be = importlib.import_module(PKG + ".halo_models.bert")
        cfg = be.BASE
        w = be.weights(cfg)
        q = be.quantize(cfg, w)
        x = bert_inputs(be, cfg, 1)
        rec = {}
        for name, kw in (("float", {}), ("int8", dict(quant=q))):
            g = odla.Graph(ref, "bert_" + name)
            be.build(g, 1, cfg, w, **kw)
            rec["encoder_out_" + name] = g.run(x)["encoder_out"].astype(np.float16)
            g.close()
        acts = sorted(k for k in q if k.startswith("act_"))
        rec["act_names"], rec["act_scales"] = np.array(acts), np.array([q[k] for k in acts], np.float32)
        np.savez_compressed(os.path.join(HERE, "bert_base_b1.npz"), **rec)
        print("bert: %.0f s, |float - int8| max %.4f" % (time.time() - t0, float(np.abs(rec["encoder_out_float"].astype(np.float32) - rec["encoder_out_int8"].astype(np.float32)).max())))


if __name__ == "__main__":
    main(sys.argv[1:] or ["resnet50_fp32", "resnet50_int8", "yolov3", "bert"])
