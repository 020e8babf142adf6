"""MNIST soft-max regression exactly as docs/mnist_sample.md:33-39 of the reference shows HALO
emitting it: odla_Gemm(x, W) -> odla_Add(b) -> odla_Softmax."""
import numpy as np

from .. import odla


def weights(seed=2):
    rng = np.random.default_rng(seed)
    return {"W": (rng.standard_normal((784, 10)) * 0.05).astype(np.float32), "b": np.zeros((1, 10), np.float32)}


def inputs(batch=64, seed=1):
    return {"x": np.random.default_rng(seed).random((batch, 784), dtype=np.float32)}


def build(g, batch=64, w=None):
    w = w or weights()
    x = g.Argument("x", (batch, 784), odla.FLOAT32)
    W = g.Constant("W", w["W"])
    b = g.Constant("b", w["b"])
    y = g.Gemm(x, False, W, False, 1.0, 0.0, None, (batch, 10), "MatMul")
    y = g.Add(y, b, "add")
    y = g.Softmax(y, -1, "y")
    g.Output(y)
    return g


MAC_PER_BATCH_ROW = 784 * 10
