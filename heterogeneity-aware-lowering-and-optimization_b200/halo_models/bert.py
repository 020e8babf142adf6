"""BERT encoder (post-LayerNorm, erf GELU) as an ODLA graph with random weights.

Emission follows HALO's rules for transformer graphs: every matmul is ``odla_Gemm`` (MatMul and
BatchMatMul both lower to it, lib/target/generic_cpp/matmul.cc:24-68 in the reference), head
split/merge are ``odla_Reshape`` + ``odla_Transpose``, the embedding lookup is ``odla_Gather``, the
attention scale is an ``odla_Mul`` by a scalar constant, and layer normalisation / GELU arrive as the
fused ``odla_LayerNorm`` / ``odla_Gelu`` calls (the -fuse-layernorm / -fuse-gelu defaults).

``build(..., quant=...)`` emits the int8-GEMM form: the six dense layers of every block (Q, K, V,
attention output, both FFN layers) read their activation through ``odla_Quantize`` ->
``odla_Dequantize`` (one symmetric per-tensor scale, max|x|/127 over a calibration batch) and their
weight through ``odla_Dequantize`` of an int8 constant with one scale per output column; bias, GELU,
residual adds, soft-max and LayerNorm stay floating point.  The two batched attention products
(scores and context) multiply two run-time tensors and stay floating point as well.
``decomposed_layernorm=True`` emits every LayerNorm as the ReduceMean / Sub / Mul / Add / Rsqrt
chain HALO leaves with -fuse-layernorm=false (the pattern lib/transforms/fusion.cc matches)."""
import numpy as np

from .. import odla

BASE = dict(vocab=30522, hidden=768, heads=12, ffn=3072, layers=12, seq=128)
MAC_PER_SEQUENCE_BASE = 11173625856


def weights(cfg, seed=500):
    rng = np.random.default_rng(seed)
    H, F = cfg["hidden"], cfg["ffn"]

    def n(*shape):
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)

    w = {"word_emb": n(cfg["vocab"], H), "pos_emb": n(1, cfg["seq"], H), "emb_ln_g": np.ones(H, np.float32), "emb_ln_b": np.zeros(H, np.float32)}
    for l in range(cfg["layers"]):
        p = "l%d_" % l
        for nm in ("q", "k", "v", "o"):
            w[p + nm + "_w"], w[p + nm + "_b"] = n(H, H), n(H)
        w[p + "f1_w"], w[p + "f1_b"], w[p + "f2_w"], w[p + "f2_b"] = n(H, F), n(F), n(F, H), n(H)
        for nm in ("ln1", "ln2"):
            w[p + nm + "_g"], w[p + nm + "_b"] = np.ones(H, np.float32), np.zeros(H, np.float32)
    return w


def inputs(cfg, batch, seed=40):
    return {"input_ids": np.random.default_rng(seed + batch).integers(0, cfg["vocab"], (batch, cfg["seq"]), dtype=np.int32)}


def _gelu_erf(x):
    from math import erf
    return (0.5 * x * (1.0 + np.vectorize(erf, otypes=[np.float64])(x / np.sqrt(2.0)))).astype(np.float32)


def numpy_forward(cfg, w, ids, record=None):
    """fp32 forward on the host with numpy: calibrates the activation ranges of the int8-GEMM form
    (record[name] = max|x| of every dense layer's input) and serves as an independent cross-check."""
    S, H, NH = cfg["seq"], cfg["hidden"], cfg["heads"]
    D, B = H // NH, ids.shape[0]

    def ln(x, g, b):
        m = x.mean(-1, keepdims=True)
        v = ((x - m) ** 2).mean(-1, keepdims=True)
        return ((x - m) / np.sqrt(v + 1e-12) * g + b).astype(np.float32)

    def rec(name, t):
        if record is not None:
            record[name] = max(record.get(name, 0.0), float(np.abs(t).max()))

    x = ln(w["word_emb"][ids] + w["pos_emb"], w["emb_ln_g"], w["emb_ln_b"]).reshape(B * S, H)
    for l in range(cfg["layers"]):
        p = "l%d_" % l
        rec(p + "x", x)
        q, k, v = (((x @ w[p + n + "_w"]) + w[p + n + "_b"]).reshape(B, S, NH, D).transpose(0, 2, 1, 3) for n in ("q", "k", "v"))
        sc = (q @ k.transpose(0, 1, 3, 2)) * np.float32(1.0 / np.sqrt(D))
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        pr = sc / sc.sum(-1, keepdims=True)
        ctx = (pr @ v).transpose(0, 2, 1, 3).reshape(B * S, H)
        rec(p + "ctx", ctx)
        x = ln(ctx @ w[p + "o_w"] + w[p + "o_b"] + x, w[p + "ln1_g"], w[p + "ln1_b"])
        rec(p + "x1", x)
        f = _gelu_erf(x @ w[p + "f1_w"] + w[p + "f1_b"])
        rec(p + "gelu", f)
        x = ln(f @ w[p + "f2_w"] + w[p + "f2_b"] + x, w[p + "ln2_g"], w[p + "ln2_b"])
    return x.reshape(B, S, H)


def quantize(cfg, w, n_sequences=4, seed=9):
    """The int8-GEMM form's constants: per-tensor activation scales (max|x|/127 over a calibration batch
    of random token ids) and int8 dense weights with one symmetric scale per output column."""
    ranges = {}
    ids = np.random.default_rng(seed).integers(0, cfg["vocab"], (n_sequences, cfg["seq"]), dtype=np.int32)
    numpy_forward(cfg, w, ids, ranges)
    q = {"act_" + k: np.float32(max(v, 1e-6) / 127.0) for k, v in ranges.items()}
    for name, a in w.items():
        if name.endswith("_w") and name[0] == "l" and a.ndim == 2:
            s = (np.maximum(np.abs(a).max(axis=0), 1e-12) / 127.0).astype(np.float32)
            q[name + "_q"] = np.clip(np.rint(a / s), -127, 127).astype(np.int8)
            q[name + "_s"] = s
    return q


def build(g, batch, cfg, w, quant=None, decomposed_layernorm=False):
    B, S, H, NH, F = batch, cfg["seq"], cfg["hidden"], cfg["heads"], cfg["ffn"]
    D = H // NH
    F32, I8 = odla.FLOAT32, odla.INT8

    def layernorm(x, rows, gname, bname, name):
        gc, bc = g.Constant(gname, w[gname]), g.Constant(bname, w[bname])
        if not decomposed_layernorm:
            return g.LayerNorm(x, (-1,), 1e-12, gc, bc, name)
        # mean, centred value, variance, 1/sqrt(var + eps), scale and shift -- one ODLA call each
        dims = tuple(g.shapes[x[0]])
        red = dims[:-1] + (1,)
        mean = g.ReduceMean(x, (len(dims) - 1,), True, red, name + "_mean")
        xc = g.Sub(x, mean, name + "_xc")
        var = g.ReduceMean(g.Mul(xc, xc, name + "_sq"), (len(dims) - 1,), True, red, name + "_var")
        rstd = g.Rsqrt(g.Add(var, g.Constant(name + "_eps", np.array([1e-12], np.float32)), name + "_vareps"), name + "_rstd")
        return g.Add(g.Mul(g.Mul(xc, rstd, name + "_norm"), gc, name + "_scaled"), bc, name)

    ids = g.Argument("input_ids", (B, S), odla.INT32)
    x = g.Gather(g.Constant("word_emb", w["word_emb"]), ids, 0, (B, S, H), "emb")
    x = g.Add(x, g.Constant("pos_emb", w["pos_emb"]), "emb_pos")
    x = layernorm(x, B * S, "emb_ln_g", "emb_ln_b", "emb_ln")
    x = g.Reshape(x, (B * S, H), "emb_2d")
    scale = g.Constant("attn_scale", np.array([1.0 / np.sqrt(D)], np.float32))
    for l in range(cfg["layers"]):
        p = "l%d_" % l

        qcache = {}

        def dense(inp, nm, n_out, act=None):
            bias = g.Constant(p + nm + "_b", w[p + nm + "_b"])
            if quant is None:
                return g.Gemm(inp, False, g.Constant(p + nm + "_w", w[p + nm + "_w"]), False, 1.0, 1.0, bias, (B * S, n_out), p + nm)
            if act not in qcache:   # Q, K and V read the same quantised tensor
                sc = g.Constant(p + act + "_scale", np.array([quant["act_" + p + act]], np.float32))
                qcache[act] = g.Dequantize(g.Quantize(inp, sc, None, 0, I8, p + act + "_q"), sc, None, 0, F32, p + act + "_dq")
            wd = g.Dequantize(g.Constant(p + nm + "_w_q", quant[p + nm + "_w_q"]), g.Constant(p + nm + "_w_s", quant[p + nm + "_w_s"]), None, 1, F32, p + nm + "_wdq")
            return g.Gemm(qcache[act], False, wd, False, 1.0, 1.0, bias, (B * S, n_out), p + nm)

        def heads(t, nm):
            t = g.Reshape(t, (B, S, NH, D), p + nm + "_4d")
            return g.Transpose(t, (0, 2, 1, 3), (B, NH, S, D), p + nm + "_t")

        q, k, v = heads(dense(x, "q", H, "x"), "q"), heads(dense(x, "k", H, "x"), "k"), heads(dense(x, "v", H, "x"), "v")
        sc = g.Gemm(q, False, k, True, 1.0, 0.0, None, (B, NH, S, S), p + "scores")
        sc = g.Mul(sc, scale, p + "scaled")
        pr = g.Softmax(sc, -1, p + "probs")
        ctx = g.Gemm(pr, False, v, False, 1.0, 0.0, None, (B, NH, S, D), p + "ctx")
        ctx = g.Transpose(ctx, (0, 2, 1, 3), (B, S, NH, D), p + "ctx_t")
        ctx = g.Reshape(ctx, (B * S, H), p + "ctx_2d")
        a = g.Add(dense(ctx, "o", H, "ctx"), x, p + "attn_res")
        x = layernorm(a, B * S, p + "ln1_g", p + "ln1_b", p + "ln1")
        f = g.Gelu(dense(x, "f1", F, "x1"), False, p + "gelu")
        f = g.Add(dense(f, "f2", H, "gelu"), x, p + "ffn_res")
        x = layernorm(f, B * S, p + "ln2_g", p + "ln2_b", p + "ln2")
    out = g.Reshape(x, (B, S, H), "encoder_out")
    g.Output(out)
    return g
