"""Host-side logic that needs no GPU: graph recording, getters, property bags, error convention,
the Python binding, the model emitters and the bench's multi-rank helpers (gloo, world size 2)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_getters_and_ids(odla, lib, models):
    g = odla.Graph(lib, "mnist_simple")
    models.mnist.build(g)
    n = C.c_uint32()
    assert lib.GetNumOfArgsFromComputation(g.comp, C.byref(n)) == 0 and n.value == 1
    assert lib.GetNumOfOutputsFromComputation(g.comp, C.byref(n)) == 0 and n.value == 1
    v = C.c_void_p()
    assert lib.GetArgFromComputationByIdx(g.comp, 0, C.byref(v)) == 0
    t = odla.ValueType()
    assert lib.GetValueType(v, C.byref(t)) == 0
    assert t.element_type == odla.FLOAT32 and t.shape.size == 2 and list(t.shape.dims[:2]) == [64, 784]
    name = C.c_char_p()
    assert lib.GetValueId(v, C.byref(name)) == 0 and name.value == b"x"
    assert lib.GetOutputFromComputationByIdx(g.comp, 0, C.byref(v)) == 0
    s = odla.Shape()
    assert lib.GetRuntimeShape(None, v, C.byref(s)) == 0 and list(s.dims[:2]) == [64, 10]
    assert lib.GetArgFromComputationByIdx(g.comp, 5, C.byref(v)) == odla.INVALID_PARAM
    g.close()


def test_builder_errors_poison_the_computation(odla, lib):
    """Generated code never checks builder results (generic_cxx_codegen.cc:775-800 in the
    reference), so a bad call returns a non-NULL value and the error surfaces at context time."""
    lib.SetLogLevel(0)
    try:
        g = odla.Graph(lib, "bad")
        x = g.Argument("x", (1, 8, 8, 4))
        w = g.Constant("w", np.zeros((3, 3, 4, 4), np.float32))
        y = g.Conv(x, odla.CHANNELS_LAST, 1, w, odla.SIO, (1, 1), (2, 2), (1, 1), (1, 1), None, (1, 8, 8, 4), "y")  # dilation 2: unsupported
        assert y[1]
        g.Output(g.Relu(y, "r"))
        ctx = C.c_void_p()
        assert lib.CreateContext(C.byref(ctx)) == odla.UNSUPPORTED_OP
        g.close()
        g = odla.Graph(lib, "bad2")
        a, b = g.Argument("a", (2, 3)), g.Argument("b", (4, 5))
        g.Add(a, b, "s")   # shapes do not broadcast
        assert lib.CreateContext(C.byref(ctx)) == odla.INVALID_PARAM
        g.close()
    finally:
        lib.SetLogLevel(3)


def test_items_and_binding_checks(odla, lib):
    g = odla.Graph(lib, "items", fp16=True, n_gpus=2, use_graph=False)
    x = g.Argument("x", (4, 8))
    y = g.Relu(x, "y")
    g.Output(y)
    lib.SetLogLevel(0)
    try:
        assert lib.SetComputationItem(g.comp, 999, None) == odla.FAILURE            # unknown key, like odla_dnnl
        buf = np.zeros((4, 8), np.float32)
        assert lib.BindToArgumentById(b"nope", buf.ctypes.data, g.context()) == odla.INVALID_PARAM
        assert lib.BindToOutput(x[1], buf.ctypes.data, g.context()) == odla.INVALID_PARAM   # not an output
        assert lib.BindToArgument(y[1], buf.ctypes.data, g.context()) == odla.INVALID_PARAM  # not an argument
        assert lib.BindToOutputById(b"y", buf.ctypes.data, g.context()) == 0
    finally:
        lib.SetLogLevel(3)
    g.close()


def test_dynamic_batch_items_leave_one_replica_per_gpu(odla, lib):
    """Generated code for a dynamic-batch model sets ODLA_DYNAMIC_BATCH / MIN / MAX / OPT_BATCH_SIZE
    (generic_cxx_codegen.cc, EmitComputationItems); none of them may turn into sub-batches."""
    g = odla.Graph(lib, "dyn")
    flag, mn, mx, opt = C.c_bool(True), C.c_int(1), C.c_int(64), C.c_int(32)
    for key, val in ((odla.ITEM_DYNAMIC_BATCH, flag), (odla.ITEM_MIN_BATCH_SIZE, mn), (odla.ITEM_MAX_BATCH_SIZE, mx), (odla.ITEM_OPT_BATCH_SIZE, opt)):
        assert lib.SetComputationItem(g.comp, key, C.cast(C.byref(val), C.c_void_p)) == 0
    x = g.Argument("x", (64, 8))
    g.Output(g.Relu(x, "y"))
    assert g.plan_shards(1) == [(0, 0, 64)]
    assert g.plan_shards(4) == [(0, 0, 16), (1, 16, 16), (2, 32, 16), (3, 48, 16)]
    g.close()


@pytest.mark.parametrize("batch,gpus,subs", [(256, 8, 1), (250, 8, 1), (5, 8, 1), (256, 8, 2), (250, 4, 3), (7, 2, 4), (1, 8, 2), (2048, 8, 1)])
def test_shard_arithmetic(odla, lib, batch, gpus, subs):
    """Shards are contiguous, non-empty, sum to the batch, never use more GPUs than rows, and differ by at most
    one row between GPUs; sub-batches split a GPU's share (even, or growing by 3 when inputs dominate)."""
    for wide_input in (False, True):
        g = odla.Graph(lib, "shards", sub_batches=subs)
        x = g.Argument("x", (batch, 4096 if wide_input else 4))
        g.Output(g.Relu(x, "y") if wide_input else g.Relu(g.Concat([x] * 64, 1, (batch, 256), "wide"), "y"))
        shards = g.plan_shards(gpus)
        g.close()
        assert [s[1] for s in shards] == [sum(r[2] for r in shards[:i]) for i in range(len(shards))]
        assert all(s[2] >= 1 for s in shards) and sum(s[2] for s in shards) == batch
        per_gpu = {}
        for d, _, r in shards:
            per_gpu[d] = per_gpu.get(d, 0) + r
        assert len(per_gpu) == min(gpus, batch) and max(per_gpu.values()) - min(per_gpu.values()) <= 1
        assert [s[0] for s in shards] == sorted(s[0] for s in shards)
        assert len(shards) <= len(per_gpu) * subs


def test_constants_that_span_the_batch_keep_the_graph_whole(odla, lib):
    """Binary / Concat / Gemm with a constant operand of full rank whose dim 0 equals the batch cannot be split by rows
    without offsetting the constant: such graphs run as one replica."""
    k = np.arange(8 * 4, dtype=np.float32).reshape(8, 4)
    for build in (lambda g, x: g.Add(x, g.Constant("k", k), "y"),
                  lambda g, x: g.Concat([x, g.Constant("k", k)], 1, (8, 8), "y"),
                  lambda g, x: g.Gemm(x, False, g.Constant("w", np.ones((4, 4), np.float32)), False, 1.0, 1.0, g.Constant("k", k), (8, 4), "y")):
        g = odla.Graph(lib, "spans")
        g.Output(build(g, g.Argument("x", (8, 4))))
        assert g.plan_shards(4) == [(0, 0, 8)]
        g.close()
    # a Gemm's weights are not aligned with the rows even when their first dimension happens to equal the batch
    # (a [2048, 1000] classifier under 2048 images): the graph still splits
    g = odla.Graph(lib, "square_weights")
    g.Output(g.Gemm(g.Argument("x", (8, 8)), False, g.Constant("w", np.ones((8, 4), np.float32)), False, 1.0, 0.0, None, (8, 4), "y"))
    assert len(g.plan_shards(4)) == 4
    g.close()
    g = odla.Graph(lib, "row_const")       # a per-row-broadcast constant ([1, 4]) splits fine
    g.Output(g.Add(g.Argument("x", (8, 4)), g.Constant("k", k[:1]), "y"))
    assert len(g.plan_shards(4)) == 4
    g.close()


def test_executable_file_round_trip(tmp_path, odla, lib, models):
    """odla_StoreExecutable / odla_LoadExecutable need no GPU: the file holds the graph, the constants and the items.
    A loaded computation exposes the same arguments and outputs, stores to the same bytes, and a damaged or foreign
    file is refused."""
    g = odla.Graph(lib, "mnist_simple", fp16=True, n_gpus=2, sub_batches=2)
    models.mnist.build(g)
    a = str(tmp_path / "a.odlab200")
    g.store(a)
    h = odla.Graph.load(lib, a)
    assert h.arg_names == g.arg_names and h.out_names == g.out_names
    assert all(h.shapes[n] == tuple(g.shapes[n]) and h.dtypes[n] == g.dtypes[n] for n in g.arg_names + g.out_names)
    assert h.plan_shards(4) == g.plan_shards(4)          # items travelled: two GPUs, two sub-batches each
    b = str(tmp_path / "b.odlab200")
    h.store(b)
    blob = open(a, "rb").read()
    assert open(b, "rb").read() == blob
    h.close()
    g.close()
    lib.SetLogLevel(0)
    try:
        bad = bytearray(blob)
        bad[len(bad) // 2] ^= 0x40
        (tmp_path / "bad.odlab200").write_bytes(bytes(bad))
        (tmp_path / "foreign.bin").write_bytes(b"ptrt" + bytes(64))
        for name in ("bad.odlab200", "foreign.bin", "missing.odlab200"):
            with pytest.raises(RuntimeError):
                odla.Graph.load(lib, str(tmp_path / name))
    finally:
        lib.SetLogLevel(3)


def test_device_api_every_item_answers(odla, lib):
    # tests/ODLA/device_test.cc:63-89 in the reference: every odla_GetDeviceInfo item returns SUCCESS
    dev = C.c_void_p()
    assert lib.AllocateDevice(None, 0, 0, C.byref(dev)) == 0
    for item in range(13):
        sv = odla.ScalarValue()
        assert lib.GetDeviceInfo(dev, item, C.byref(sv)) == 0, item
    assert lib.SetCurrentDevice(dev) == 0
    assert lib.DestroyDevice(dev) == 0
    assert lib.AllocateDevice(None, 5, 0, C.byref(dev)) != 0   # a Graphcore IPU is not ours


def test_resnet50_description(models):
    rn = models.resnet50
    convs = rn.conv_list()
    assert len(convs) == 53
    by_name = {c[0]: c for c in convs}

    def macs(name, h_in):
        _, k, cin, cout, s, p = by_name[name]
        ho = (h_in + 2 * p - k) // s + 1
        return ho * ho * k * k * cin * cout, ho

    mac, h = macs("conv1", 224)
    h = (h + 2 - 3) // 2 + 1
    for si, (blocks, mid, out, stride) in enumerate(rn.STAGES):
        for b in range(blocks):
            p = "s%db%d" % (si + 1, b)
            if b == 0:
                mac += macs(p + "_sc", h)[0]
            m1, _ = macs(p + "_c1", h)
            m2, h2 = macs(p + "_c2", h)
            m3, _ = macs(p + "_c3", h2)
            mac += m1 + m2 + m3
            h = h2
    mac += 2048 * 1000
    assert mac == rn.MAC_PER_IMAGE == 4089184256
    w = rn.weights()
    assert sum(v.size for k, v in w.items() if k.endswith("_w")) + sum(v.size for k, v in w.items() if k.endswith("_b")) > 25_000_000
    q = rn.quantize_weights(w)
    assert q["conv1_w_q"].dtype == np.int8 and q["conv1_w_s"].shape == (64,)
    assert int(np.abs(q["s2b0_c2_w_q"]).max()) == 127


def test_yolov3_and_bert_descriptions(models):
    yo, be = models.yolov3, models.bert
    specs = yo.conv_specs()
    assert len(specs) == 75 and sum(1 for s in specs if s[5]) == 3
    # MAC count at 416x416: walk the same structure the builder walks
    it = iter(specs)
    mac, h = 0, 416

    def conv(h_in):
        nonlocal mac
        _, k, cin, cout, s, _ = next(it)
        ho = (h_in + 2 * (k // 2) - k) // s + 1
        mac += ho * ho * k * k * cin * cout
        return ho

    for ch, k, s, nres in yo.BACKBONE:
        h = conv(h)
        for _ in range(nres):
            conv(h); conv(h)
    for width, route in ((512, None), (256, 512), (128, 256)):
        if route:
            conv(h)
            h *= 2
        for _ in range(7):
            conv(h)
    assert mac == yo.MAC_PER_IMAGE_416 == 32932037632
    c = be.BASE
    S, H, F, L = c["seq"], c["hidden"], c["ffn"], c["layers"]
    assert L * (3 * S * H * H + 2 * S * S * H + S * H * H + 2 * S * H * F) == be.MAC_PER_SEQUENCE_BASE == 11173625856


def test_emitted_resnet50_cc_follows_halo_rules(odla, lib, models):
    rn = models.resnet50
    w = {k: (v if v.size < 4096 else v) for k, v in rn.weights().items()}
    g = odla.Graph(lib, "resnet50")
    rn.build(g, 2, w)
    text = g.emit_cc()
    g.close()
    assert text.count("odla_Conv(") == 53 and "odla_ReduceMean(" in text and "odla_Gemm(" in text
    assert "nullptr, {.size = 4" in text                      # convolution bias argument is null, the BN offset is a separate Add
    assert '#include <ODLA/odla.h>' in text and "odla_memory_layout::ODLA_SIO" in text
    assert "static odla_computation Comp;" in text and "odla_BindToArgumentById" in text


def test_quant_table_item_and_emission(odla, lib):
    """ODLA_QUANT_TABLE_SIZE / ODLA_QUANT_TABLE are accepted (the ids are copied, the caller's table may go away)
    and the emitted model declares the table the way the reference's code generator does."""
    g = odla.Graph(lib, "qt")
    x = g.Argument("x", (2, 8, 8, 32))
    w = g.Constant("w", np.ones((1, 1, 32, 32), np.float32))
    g.Output(g.Conv(x, odla.CHANNELS_LAST, 1, w, odla.SIO, (1, 1), (1, 1), (0, 0), (0, 0), None, (2, 8, 8, 32), "c"))
    recs = [("x", -1, 0.0, 0.0, -2.0, 2.0), ("w_", -2, 0.0, 0.0, -1.0, 1.0), ("w_", 0, 0.0, 0.0, -1.0, 0.5), ("w_", 1, 0.0, 0.0, -0.5, 1.0)]
    g.set_quant_table(recs)
    cc, tbl = g.emit_cc(), g.emit_quant_table_c()
    g.close()
    assert "extern const odla_value_quant_info quant_infos[];" in cc and "extern const int quant_infos_size;" in cc
    assert cc.index("ODLA_QUANT_TABLE_SIZE") < cc.index("ODLA_QUANT_TABLE, ")      # the size is set before the records
    assert tbl.count(".value_id") == 4 and "const int quant_infos_size = 4;" in tbl and '"w_", .ch_idx = -2' in tbl


def test_two_rank_gloo_timing_helper():
    """bench.py's max-over-ranks aggregation and per-rank sharding, on CPU with gloo."""
    code = r'''
import os, sys
sys.path.insert(0, %r)
import torch.distributed as dist
import bench
dist.init_process_group("gloo")
r = dist.get_rank()
assert bench.max_over_ranks(1.0 + r) == 2.0
assert bench.sum_over_ranks(3) == 6
assert bench.rank_seed(10, r) != bench.rank_seed(10, 1 - r)
dist.barrier()
dist.destroy_process_group()
print("rank", r, "ok")
''' % ROOT
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    procs = []
    for rank in range(2):
        e = dict(env, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err
        assert "ok" in out


def test_async_execute_reports_failure_through_the_callback_without_a_gpu(odla, lib):
    """odla_AsyncExecuteComputation returns at once; the status reaches the caller through the callback and
    odla_b200_WaitContext.  On a box without a CUDA device that status is a failure (there is no CPU fallback)."""
    if lib.b200_DeviceCount() > 0:
        pytest.skip("needs a box without a GPU")
    g = odla.Graph(lib, "async")
    x = g.Argument("x", (4, 8))
    g.Output(g.Relu(x, "y"))
    a, b = np.ones((4, 8), np.float32), np.zeros((4, 8), np.float32)
    lib.SetLogLevel(0)
    try:
        g.bind_input("x", a.ctypes.data)
        g.bind_output("y", b.ctypes.data)
        seen = []
        assert g.set_run_batch(2) == 0 and g.set_run_batch(-1) == odla.FAILURE
        assert g.execute_async(lambda arg, status: seen.append((arg, status)) or 0, 1234) == 0
        assert g.wait() != 0
        assert seen == [(1234, g.wait())]
        # an unbound argument is refused before any thread starts
        h = odla.Graph(lib, "async2")
        h.Output(h.Relu(h.Argument("x", (4, 8)), "y"))
        assert h.execute_async() == odla.INVALID_PARAM
        # destroying the computation before its context is allowed; the context is detached
        ctx = h.context()
        assert lib.DestroyComputation(h.comp) == 0
        buf = np.zeros((4, 8), np.float32)
        assert lib.BindToArgumentById(b"x", buf.ctypes.data, ctx) == odla.INVALID_PARAM
        assert lib.DestroyContext(ctx) == 0
        h.comp, h.ctx = odla._V(), None
    finally:
        lib.SetLogLevel(3)
    g.close()


def test_contexts_are_spread_over_lanes(odla, lib):
    """The first context of a computation takes lane 0, the second a lane of its own, the third shares the less used
    one; destroying a context frees its place.  Nothing here needs a GPU: lanes are built at the first execute."""
    g = odla.Graph(lib, "lanes")
    x = g.Argument("x", (4, 8))
    g.Output(g.Relu(x, "y"))
    g.context()
    assert lib.b200_ContextLane(g.ctx) == 0
    a, b = g.extra_context(), g.extra_context()
    assert (a.lane(), b.lane()) == (1, 0)
    c = g.extra_context()
    assert c.lane() == 1
    a.close()
    c.close()
    d = g.extra_context()
    assert d.lane() == 1
    assert lib.b200_ContextLane(None) == -1
    g.close()
