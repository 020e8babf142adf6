"""Generates tests/golden/ref_kernels.npz from the reference's own CPU kernels.

Run on a machine that has the reference tree (oracle/Makefile's REFERENCE variable points to it):
    make -C oracle ref && python tests/golden/make_golden.py
It calls the _sn_rt_* functions of oracle/_ref/libhalo_rt_generic.so (compiled from the reference's
runtime/generic/*.cc) on small seeded inputs and stores inputs and outputs, so the oracle
restatement can be checked against the reference's code on machines where the reference is absent.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libhalo_rt_generic.so"))
f32p, i64 = C.POINTER(C.c_float), C.c_int64


def fp(a):
    return a.ctypes.data_as(f32p)


rng = np.random.default_rng(2024)
out = {}
# convolution NHWC/HWIO: (N,H,W,C,K,R,S,stride,pad)
for i, (N, H, W, Cc, K, R, S, st, pad) in enumerate([(2, 8, 8, 3, 5, 3, 3, 1, 1), (1, 9, 7, 4, 6, 3, 3, 2, 1), (2, 6, 6, 8, 4, 1, 1, 1, 0),
                                                      (1, 12, 12, 3, 8, 7, 7, 2, 3), (1, 5, 5, 2, 3, 3, 3, 2, 0)]):
    P, Q = (H + 2 * pad - R) // st + 1, (W + 2 * pad - S) // st + 1
    x = rng.standard_normal((N, H, W, Cc)).astype(np.float32)
    w = rng.standard_normal((R, S, Cc, K)).astype(np.float32)
    y = np.zeros((N, P, Q, K), np.float32)
    ref._sn_rt_conv2d_f32_nhwc(fp(y), fp(x), fp(w), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(K), i64(R), i64(S), i64(st), i64(st),
                               i64(pad), i64(pad), i64(pad), i64(pad))
    out["conv%d_x" % i], out["conv%d_w" % i], out["conv%d_y" % i] = x, w, y
    out["conv%d_geom" % i] = np.array([N, H, W, Cc, K, R, S, st, pad, P, Q])
# max pooling NHWC
for i, (N, H, W, Cc, R, st, pad) in enumerate([(2, 8, 8, 3, 3, 2, 1), (1, 7, 7, 4, 2, 2, 0), (1, 6, 6, 2, 3, 1, 1)]):
    P, Q = (H + 2 * pad - R) // st + 1, (W + 2 * pad - R) // st + 1
    x = rng.standard_normal((N, H, W, Cc)).astype(np.float32)
    y = np.zeros((N, P, Q, Cc), np.float32)
    ref._sn_rt_poolingmax_f32_nhwc(fp(y), fp(x), i64(N), i64(H), i64(W), i64(Cc), i64(P), i64(Q), i64(R), i64(R), i64(st), i64(st), i64(pad), i64(pad),
                                   i64(pad), i64(pad))
    out["pool%d_x" % i], out["pool%d_y" % i] = x, y
    out["pool%d_geom" % i] = np.array([N, H, W, Cc, R, st, pad, P, Q])
# matmul / gemm
for i, (M, Kd, Nn, ta, tb) in enumerate([(4, 7, 5, 0, 0), (4, 7, 5, 0, 1), (4, 7, 5, 1, 0)]):
    A = rng.standard_normal((Kd, M) if ta else (M, Kd)).astype(np.float32)
    B = rng.standard_normal((Nn, Kd) if tb else (Kd, Nn)).astype(np.float32)
    Cm = rng.standard_normal((Nn,)).astype(np.float32)
    y = np.zeros((M, Nn), np.float32)
    ref._sn_rt_gemm_f32(fp(y), fp(A), fp(B), fp(Cm), i64(A.shape[0]), i64(A.shape[1]), i64(B.shape[0]), i64(B.shape[1]), i64(Nn), C.c_bool(ta), C.c_bool(tb),
                        C.c_float(0.5), C.c_float(2.0))
    out["gemm%d_a" % i], out["gemm%d_b" % i], out["gemm%d_c" % i], out["gemm%d_y" % i] = A, B, Cm, y
    out["gemm%d_t" % i] = np.array([ta, tb])
# softmax over the last axis, relu, batchnorm NHWC, reduce mean
x = rng.standard_normal((3, 4, 10)).astype(np.float32)
y = np.zeros_like(x)
shape = (i64 * 3)(3, 4, 10)
ref._sn_rt_softmax_f32(fp(y), fp(x), shape, C.c_int32(2), C.c_int32(3), i64(x.size))
out["softmax_x"], out["softmax_y"] = x, y
x = rng.standard_normal((50,)).astype(np.float32)
y = np.zeros_like(x)
ref._sn_rt_relu_f32(fp(y), fp(x), i64(x.size))
out["relu_x"], out["relu_y"] = x, y
x = rng.standard_normal((2, 3, 3, 4)).astype(np.float32)
mean, var = rng.standard_normal(4).astype(np.float32), rng.uniform(0.5, 1.5, 4).astype(np.float32)
off, sc = rng.standard_normal(4).astype(np.float32), rng.standard_normal(4).astype(np.float32)
y = np.zeros_like(x)
ref._sn_rt_bn_f32_nhwc(fp(y), fp(x), fp(mean), fp(var), fp(off), fp(sc), i64(2), i64(3), i64(3), i64(4), C.c_bool(False), C.c_bool(False), C.c_float(1e-5),
                       C.c_float(1.0))
out.update(bn_x=x, bn_mean=mean, bn_var=var, bn_off=off, bn_sc=sc, bn_y=y)
np.savez_compressed(os.path.join(HERE, "ref_kernels.npz"), **out)
print("wrote", os.path.join(HERE, "ref_kernels.npz"), len(out), "arrays")
