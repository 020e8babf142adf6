"""odla_b200_reduce_mean_noalloc, the entry point for callers that may not allocate (a runtime that
owns all device memory, a loop that cannot take the allocator's lock): called through the C ABI
twice in a row on different data and compared with what odla_ReduceMean computes through the
graph path for the same inputs.  Both run the same kernels in the same order, so fp32 results
must be identical; the file sorts last so a failure here cannot hide any other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def graph_reduce_mean(odla, lib, x, axes, out_dims, fp16=False):
    g = odla.Graph(lib, "rm", fp16=fp16)
    a = g.Argument("x", x.shape, odla.FLOAT32)
    g.Output(g.ReduceMean(a, axes, True, out_dims, "m"))
    out = g.run({"x": x})["m"]
    g.close()
    return out


def noalloc_reduce_mean(lib, xt, axes, out_dims, dtype_code):
    y = torch.empty(out_dims, dtype=xt.dtype, device="cuda")
    dims = (C.c_longlong * xt.dim())(*xt.shape)
    ax = (C.c_int * len(axes))(*axes)
    rc = lib.b200_reduce_mean_noalloc(xt.data_ptr(), y.data_ptr(), dtype_code, dims, xt.dim(), ax, len(axes), None)
    assert rc == 0
    torch.cuda.synchronize()
    return y


def test_two_calls_in_a_row_match_the_graph_path(odla, gpu_lib):
    rng = np.random.default_rng(77)
    for shape, axes in (((5, 7, 7, 256), (1, 2)), ((3, 6, 10, 64), (1, 2)), ((4, 9, 32), (1,)), ((2, 3, 4, 5), (0, 2, 3))):
        out_dims = tuple(1 if i in axes else d for i, d in enumerate(shape))
        x = rng.standard_normal(shape).astype(np.float32)
        want = graph_reduce_mean(odla, gpu_lib, x, axes, out_dims)
        got = noalloc_reduce_mean(gpu_lib, torch.from_numpy(x).cuda(), axes, out_dims, 0).cpu().numpy()
        assert np.array_equal(got, want), (shape, axes)
    # fp16 storage: compare with the graph in fp16 mode (same kernels, fp32 intermediates)
    x = rng.standard_normal((4, 7, 7, 128)).astype(np.float32)
    want = graph_reduce_mean(odla, gpu_lib, x, (1, 2), (4, 1, 1, 128), fp16=True)
    got = noalloc_reduce_mean(gpu_lib, torch.from_numpy(x).cuda().half(), (1, 2), (4, 1, 1, 128), 1).float().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-3     # the graph converts its fp16 result back to the fp32 API type


def test_sizes_beyond_the_fixed_scratch_are_refused(gpu_lib):
    x = torch.zeros(8, dtype=torch.float32, device="cuda")
    dims = (C.c_longlong * 4)(2048, 7, 7, 2048)     # first-pass intermediate: 2048*7*2048 floats > 1 Mi
    ax = (C.c_int * 2)(1, 2)
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), x.data_ptr(), 0, dims, 4, ax, 2, None) == -1
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), x.data_ptr(), 7, dims, 4, ax, 2, None) == -1   # unknown dtype
