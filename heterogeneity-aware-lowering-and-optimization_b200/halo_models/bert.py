"""BERT encoder (post-LayerNorm, erf GELU) as an ODLA graph with random weights.

Emission follows HALO's rules for transformer graphs: every matmul is ``odla_Gemm`` (MatMul and
BatchMatMul both lower to it, lib/target/generic_cpp/matmul.cc:24-68 in the reference), head
split/merge are ``odla_Reshape`` + ``odla_Transpose``, the embedding lookup is ``odla_Gather``, the
attention scale is an ``odla_Mul`` by a scalar constant, and layer normalisation / GELU arrive as the
fused ``odla_LayerNorm`` / ``odla_Gelu`` calls (the -fuse-layernorm / -fuse-gelu defaults)."""
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


def build(g, batch, cfg, w):
    B, S, H, NH, F = batch, cfg["seq"], cfg["hidden"], cfg["heads"], cfg["ffn"]
    D = H // NH
    ids = g.Argument("input_ids", (B, S), odla.INT32)
    x = g.Gather(g.Constant("word_emb", w["word_emb"]), ids, 0, (B, S, H), "emb")
    x = g.Add(x, g.Constant("pos_emb", w["pos_emb"]), "emb_pos")
    x = g.LayerNorm(x, (-1,), 1e-12, g.Constant("emb_ln_g", w["emb_ln_g"]), g.Constant("emb_ln_b", w["emb_ln_b"]), "emb_ln")
    x = g.Reshape(x, (B * S, H), "emb_2d")
    scale = g.Constant("attn_scale", np.array([1.0 / np.sqrt(D)], np.float32))
    for l in range(cfg["layers"]):
        p = "l%d_" % l

        def dense(inp, nm, n_out):
            return g.Gemm(inp, False, g.Constant(p + nm + "_w", w[p + nm + "_w"]), False, 1.0, 1.0, g.Constant(p + nm + "_b", w[p + nm + "_b"]), (B * S, n_out), p + nm)

        def heads(t, nm):
            t = g.Reshape(t, (B, S, NH, D), p + nm + "_4d")
            return g.Transpose(t, (0, 2, 1, 3), (B, NH, S, D), p + nm + "_t")

        q, k, v = heads(dense(x, "q", H), "q"), heads(dense(x, "k", H), "k"), heads(dense(x, "v", H), "v")
        sc = g.Gemm(q, False, k, True, 1.0, 0.0, None, (B, NH, S, S), p + "scores")
        sc = g.Mul(sc, scale, p + "scaled")
        pr = g.Softmax(sc, -1, p + "probs")
        ctx = g.Gemm(pr, False, v, False, 1.0, 0.0, None, (B, NH, S, D), p + "ctx")
        ctx = g.Transpose(ctx, (0, 2, 1, 3), (B, S, NH, D), p + "ctx_t")
        ctx = g.Reshape(ctx, (B * S, H), p + "ctx_2d")
        a = g.Add(dense(ctx, "o", H), x, p + "attn_res")
        x = g.LayerNorm(a, (-1,), 1e-12, g.Constant(p + "ln1_g", w[p + "ln1_g"]), g.Constant(p + "ln1_b", w[p + "ln1_b"]), p + "ln1")
        f = g.Gelu(dense(x, "f1", F), False, p + "gelu")
        f = g.Add(dense(f, "f2", H), x, p + "ffn_res")
        x = g.LayerNorm(f, (-1,), 1e-12, g.Constant(p + "ln2_g", w[p + "ln2_g"]), g.Constant(p + "ln2_b", w[p + "ln2_b"]), p + "ln2")
    out = g.Reshape(x, (B, S, H), "encoder_out")
    g.Output(out)
    return g
