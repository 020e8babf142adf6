"""odla_NMS and odla_PostProcess on the GPU against the CPU oracle (and, for NMS, against a plain numpy statement of
the ONNX rule): the selected boxes must be the same boxes, in the same order."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def numpy_nms(boxes, scores, max_per_class, iou_thr, score_thr, rows):
    out = -np.ones((rows, 3), np.int64)
    r = 0
    B, C, N = scores.shape
    for b in range(B):
        y1, y2 = np.minimum(boxes[b, :, 0], boxes[b, :, 2]), np.maximum(boxes[b, :, 0], boxes[b, :, 2])
        x1, x2 = np.minimum(boxes[b, :, 1], boxes[b, :, 3]), np.maximum(boxes[b, :, 1], boxes[b, :, 3])
        area = (y2 - y1) * (x2 - x1)
        for c in range(C):
            s = scores[b, c]
            order = [i for i in np.lexsort((np.arange(N), -s)) if s[i] > score_thr]
            kept = []
            for i in order:
                if len(kept) >= max_per_class:
                    break
                ok = True
                for j in kept:
                    ih = np.float32(min(y2[i], y2[j]) - max(y1[i], y1[j]))
                    iw = np.float32(min(x2[i], x2[j]) - max(x1[i], x1[j]))
                    if ih <= 0 or iw <= 0:
                        continue
                    inter = np.float32(ih * iw)
                    uni = np.float32(np.float32(area[i] + area[j]) - inter)
                    if uni > 0 and np.float32(inter / uni) > iou_thr:
                        ok = False
                        break
                if ok:
                    kept.append(i)
                    if r < rows:
                        out[r] = (b, c, i)
                        r += 1
    return out


def random_boxes(rng, B, N, size=416.0):
    c = rng.uniform(0, size, (B, N, 2))
    wh = rng.uniform(8, 120, (B, N, 2))
    b = np.concatenate([c - wh / 2, c + wh / 2], axis=2).astype(np.float32)       # (y1, x1, y2, x2)
    flip = rng.random((B, N)) < 0.2                                                # some boxes with swapped corners
    b[flip] = b[flip][:, [2, 3, 0, 1]]
    return b


@pytest.mark.parametrize("B,C,N,max_out,index_type", [(1, 3, 200, 20, "i32"), (2, 4, 1000, 50, "i64"), (1, 80, 10647, 30, "i32"), (1, 1, 33, 0, "i32")])
def test_nms_selects_the_same_boxes(odla, gpu_lib, ref, B, C, N, max_out, index_type):
    rng = np.random.default_rng(B * 1000 + N)
    boxes = random_boxes(rng, B, N)
    scores = rng.random((B, C, N)).astype(np.float32)
    scores[scores < 0.6] *= 0.1                                     # most candidates fall under the score threshold
    if N > 100:
        scores[0, 0, 5] = scores[0, 0, 17] = np.float32(0.97)       # a tie: the lower index goes first
    rows = (max_out or 8) * C * B
    it = odla.INT32 if index_type == "i32" else odla.INT64
    outs = []
    for L in (gpu_lib, ref):
        g = odla.Graph(L, "nms")
        bx = g.Argument("boxes", boxes.shape)
        sc = g.Argument("scores", scores.shape)
        g.Output(g.NMS(bx, sc, max_out, 0.5, 0.35, rows, "sel", it))
        outs.append(g.run({"boxes": boxes, "scores": scores})["sel"])
        g.close()
    assert np.array_equal(outs[0], outs[1])
    if N <= 1000:
        assert np.array_equal(outs[0].astype(np.int64), numpy_nms(boxes, scores, max_out or rows, np.float32(0.5), np.float32(0.35), rows))
    assert (outs[0][:, 2] >= 0).sum() > 0


@pytest.mark.parametrize("layout,mode", [("nchw", "fp32"), ("nhwc", "fp32"), ("nhwc", "fp16")])
def test_yolo_postprocess_matches_the_oracle(odla, gpu_lib, ref, layout, mode):
    """Random heads with a handful of confident cells: the decoded boxes agree to float tolerance (exp differs in
    the last bit between the GPU and the host) and the same boxes are selected per class."""
    rng = np.random.default_rng(11)
    cls = 80
    heads = {}
    for S in (13, 26, 52):
        h = rng.normal(-6.0, 1.0, (1, S, S, 3 * (cls + 5))).astype(np.float32)      # objectness and classes far below threshold
        h[..., 0:4] = rng.normal(0, 0.5, h[..., 0:4].shape)
        for _ in range(S):                                                           # S confident detections per head
            y, x, a, c = rng.integers(S), rng.integers(S), rng.integers(3), rng.integers(cls)
            base = a * (cls + 5)
            h[0, y, x, base:base + 4] = rng.normal(0, 0.5, 4)
            h[0, y, x, base + 4] = rng.uniform(2, 5)
            h[0, y, x, base + 5 + c] = rng.uniform(2, 5)
        if mode == "fp16":
            h = h.astype(np.float16).astype(np.float32)
        heads[S] = np.ascontiguousarray(h.transpose(0, 3, 1, 2)) if layout == "nchw" else h
    outs = []
    for L in (gpu_lib, ref):
        g = odla.Graph(L, "pp", **({"fp16": mode == "fp16"} if L is gpu_lib else {}))
        w = g.Constant("img_w", np.array([640], np.uint32))
        hh = g.Constant("img_h", np.array([480], np.uint32))
        b = [g.Argument("bb%d" % S, heads[S].shape) for S in (13, 26, 52)]
        info, num = g.PostProcess(w, hh, b[0], b[1], b[2], "det")
        g.Output(info)
        g.Output(num)
        outs.append(g.run({"bb%d" % S: heads[S] for S in (13, 26, 52)}))
        g.close()
    got, want = outs
    assert want["det0"].shape == (80, 63, 5) and want["det1"].shape == (80,)
    assert np.array_equal(got["det1"], want["det1"]) and int(want["det1"].sum()) >= 20
    tol = 1e-3 if mode == "fp32" else 0.5          # pixels; fp16 storage rounds the result
    assert np.abs(got["det0"][..., :4] - want["det0"][..., :4]).max() <= tol
    assert np.abs(got["det0"][..., 4] - want["det0"][..., 4]).max() <= (1e-5 if mode == "fp32" else 2e-3)
