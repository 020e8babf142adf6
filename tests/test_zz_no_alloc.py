"""odla_b200_reduce_mean_noalloc, the entry point for callers that may not allocate (a runtime that
owns all device memory, a loop that cannot take the allocator's lock): called through the C ABI
twice in a row on different data and compared (a) with what odla_ReduceMean computes through the
graph path for the same inputs -- fp32 results must be identical -- and (b) with an axis-by-axis
numpy evaluation in the reference's order (runtime/generic/common/reduce.cc: one axis after the
other, a sequential fp32 sum and one division per axis), so the check stands without the graph path.
The file sorts last so a failure here cannot hide any other test."""
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


def numpy_reduce_mean(x, axes):
    """Axis after axis; along an axis a left-to-right fp32 sum, then one fp32 division."""
    t = x.astype(np.float32)
    for a in axes:
        acc = np.zeros(t.shape[:a] + (1,) + t.shape[a + 1:], np.float32)
        for i in range(t.shape[a]):
            acc = acc + np.take(t, [i], axis=a)
        t = acc / np.float32(t.shape[a])
    return t


def test_two_calls_in_a_row_match_the_graph_path(odla, gpu_lib):
    rng = np.random.default_rng(77)
    for shape, axes in (((5, 7, 7, 256), (1, 2)), ((3, 6, 10, 64), (1, 2)), ((4, 9, 32), (1,)), ((2, 3, 4, 5), (0, 2, 3))):
        out_dims = tuple(1 if i in axes else d for i, d in enumerate(shape))
        x = rng.standard_normal(shape).astype(np.float32)
        want = graph_reduce_mean(odla, gpu_lib, x, axes, out_dims)
        got = noalloc_reduce_mean(gpu_lib, torch.from_numpy(x).cuda(), axes, out_dims, 0).cpu().numpy()
        assert np.array_equal(got, want), (shape, axes)
        assert np.array_equal(got, numpy_reduce_mean(x, axes)), (shape, axes)
    # fp16 storage: compare with the graph in fp16 mode (same kernels, fp32 intermediates)
    x = rng.standard_normal((4, 7, 7, 128)).astype(np.float32)
    want = graph_reduce_mean(odla, gpu_lib, x, (1, 2), (4, 1, 1, 128), fp16=True)
    got = noalloc_reduce_mean(gpu_lib, torch.from_numpy(x).cuda().half(), (1, 2), (4, 1, 1, 128), 1).float().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-3     # the graph converts its fp16 result back to the fp32 API type


def test_bf16_and_two_streams_ordered_by_an_event(gpu_lib):
    """Calls on different streams share the scratch array; with an event between them they may follow each other."""
    rng = np.random.default_rng(78)
    xs = [rng.standard_normal((6, 7, 7, 192)).astype(np.float32) for _ in range(2)]
    xt = [torch.from_numpy(x).cuda().to(torch.bfloat16) for x in xs]
    ys = [torch.empty((6, 1, 1, 192), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    dims, ax = (C.c_longlong * 4)(6, 7, 7, 192), (C.c_int * 2)(1, 2)
    done = torch.cuda.Event()
    assert gpu_lib.b200_reduce_mean_noalloc(xt[0].data_ptr(), ys[0].data_ptr(), 2, dims, 4, ax, 2, streams[0].cuda_stream) == 0
    done.record(streams[0])
    streams[1].wait_event(done)
    assert gpu_lib.b200_reduce_mean_noalloc(xt[1].data_ptr(), ys[1].data_ptr(), 2, dims, 4, ax, 2, streams[1].cuda_stream) == 0
    torch.cuda.synchronize()
    for x, y in zip(xt, ys):
        want = torch.from_numpy(numpy_reduce_mean(x.float().cpu().numpy(), (1, 2))).to(torch.bfloat16)   # fp32 passes, one rounding at the end
        assert torch.equal(y.cpu(), want)


def test_sizes_beyond_the_fixed_scratch_are_refused(gpu_lib):
    x = torch.zeros(8, dtype=torch.float32, device="cuda")
    dims = (C.c_longlong * 4)(2048, 7, 7, 2048)     # first-pass intermediate: 2048*7*2048 floats > 1 Mi
    ax = (C.c_int * 2)(1, 2)
    y = torch.zeros(8, dtype=torch.float32, device="cuda")
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), y.data_ptr(), 0, dims, 4, ax, 2, None) == -1
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), y.data_ptr(), 7, dims, 4, ax, 2, None) == -1   # unknown dtype
    small = (C.c_longlong * 3)(2, 2, 2)
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), y.data_ptr(), 0, small, 3, (C.c_int * 2)(1, 1), 2, None) == -1   # an axis named twice
    assert gpu_lib.b200_reduce_mean_noalloc(x.data_ptr(), x.data_ptr(), 0, small, 3, (C.c_int * 1)(1), 1, None) == -1      # in place
