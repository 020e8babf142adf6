"""ctypes binding of the ODLA C API and a small graph builder on top of it.

The binding mirrors what the reference's own Python caller does
(``python/halo/odla.py:56-177``: create a computation, call ``model_helper``, query arguments and
outputs, bind, execute) and works with any ODLA platform library that exports the ABI declared in
``include/odla_b200.h`` -- libodla_b200.so (the product) and the CPU oracle platform used by the
tests.  ``Graph`` issues one ODLA builder call per method, with the argument order of the C API,
and records the same calls as C++ text so a HALO-style ``model.cc`` can be written out
(``Graph.emit_cc``).
"""
import ctypes as C
import os

import numpy as np

MAX_DIM = 10
MAX_OUTPUTS = 64

# odla_element_type (include/odla_b200.h)
INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64 = range(8)
FLOAT16, BFLOAT16, FLOAT32, FLOAT64, BOOL = 16, 17, 18, 19, 20
# odla_item_type
ITEM_BF16_MODE, ITEM_FP16_MODE, ITEM_PROCESSOR_NUM, ITEM_USE_DATA_TYPE, ITEM_AGGREGATE_OPS = 13, 14, 16, 18, 23
ITEM_QUANT_TABLE, ITEM_QUANT_TABLE_SIZE = 21, 22
ITEM_BATCHES_PER_STEP = 17
ITEM_DYNAMIC_BATCH, ITEM_MIN_BATCH_SIZE, ITEM_MAX_BATCH_SIZE, ITEM_OPT_BATCH_SIZE = 0, 1, 2, 3
ITEM_LOAD_ENGINE_MODE, ITEM_ENABLE_ENGINE_CACHE, ITEM_CACHE_DIR = 19, 24, 25
ITEM_RUN_BATCH_SIZE, ITEM_ASYNC_CALLBACK_FUNC, ITEM_ASYNC_CALLBACK_ARG = 4, 26, 27
ASYNC_CALLBACK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int)   # int (*)(void* arg, odla_status)
# odla_memory_layout
CHANNELS_FIRST, CHANNELS_LAST, SIO, SOI, OIS, IOS = range(6)
# odla_status
SUCCESS, INVALID_PARAM, UNSUPPORTED_OP, TIMEOUT, FAILURE = 0, 3, 7, 8, 14

_NP2ODLA = {np.dtype(np.float32): FLOAT32, np.dtype(np.float16): FLOAT16, np.dtype(np.int8): INT8,
            np.dtype(np.uint8): UINT8, np.dtype(np.int32): INT32, np.dtype(np.int64): INT64, np.dtype(np.uint32): UINT32}
_ODLA2NP = {v: k for k, v in _NP2ODLA.items()}
_CTYPE = {FLOAT32: "float", FLOAT16: "odla_float16", INT8: "signed char", UINT8: "unsigned char",
          INT32: "int", INT64: "long long", UINT32: "unsigned int"}
_ENUM = {FLOAT32: "ODLA_FLOAT32", FLOAT16: "ODLA_FLOAT16", INT8: "ODLA_INT8", UINT8: "ODLA_UINT8",
         INT32: "ODLA_INT32", INT64: "ODLA_INT64", BFLOAT16: "ODLA_BFLOAT16", UINT32: "ODLA_UINT32"}


class Shape(C.Structure):
    _fields_ = [("size", C.c_int32), ("dims", C.c_int64 * MAX_DIM)]


class ValueType(C.Structure):
    _fields_ = [("element_type", C.c_int), ("shape", Shape)]


class Values(C.Structure):
    _fields_ = [("size", C.c_size_t), ("values", C.c_void_p * MAX_OUTPUTS)]


class ScalarValue(C.Structure):
    class _U(C.Union):
        _fields_ = [("i32", C.c_int32), ("u32", C.c_uint32), ("i64", C.c_int64), ("u64", C.c_uint64),
                    ("f32", C.c_float), ("f64", C.c_double), ("s", C.c_char_p)]
    _anonymous_ = ("u",)
    _fields_ = [("data_type", C.c_int), ("u", _U)]


class QuantInfo(C.Structure):
    """odla_value_quant_info (ODLA/include/ODLA/ops/odla_ops_quantization.h:33-41 in the reference)."""
    _fields_ = [("value_id", C.c_char_p), ("ch_idx", C.c_int), ("scale", C.c_float), ("offset", C.c_float), ("min", C.c_float), ("max", C.c_float)]


class ResourceLocation(C.Structure):
    _fields_ = [("location_type", C.c_int), ("location", C.c_void_p), ("size", C.c_uint64)]


class ProfileEntry(C.Structure):
    _fields_ = [("op", C.c_char * 32), ("name", C.c_char * 64), ("total_ms", C.c_double),
                ("launches", C.c_longlong), ("flops", C.c_double), ("bytes", C.c_double)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n", "h", "w", "c", "k", "r", "s", "stride_h", "stride_w", "pad_top",
                                       "pad_left", "p", "q", "dtype", "out_kind", "res_kind", "act")] + \
               [("alpha", C.c_float), ("res_scale", C.c_float), ("out_scale", C.c_float), ("out_multiply", C.c_int)]


def shape(dims):
    s = Shape()
    s.size = len(dims)
    for i, d in enumerate(dims):
        s.dims[i] = int(d)
    return s


def vtype(et, dims):
    t = ValueType()
    t.element_type = et
    t.shape = shape(dims)
    return t


def _u32(vals):
    return (C.c_uint32 * len(vals))(*[int(v) for v in vals])


def _i32(vals):
    return (C.c_int32 * len(vals))(*[int(v) for v in vals])


_V, _ID, _S = C.c_void_p, C.c_char_p, Shape
_U32P, _I32P = C.POINTER(C.c_uint32), C.POINTER(C.c_int32)
# name -> (restype, argtypes); the argument order is the C API's
_SIGNATURES = {
    "odla_CreateComputation": (C.c_int, [C.POINTER(_V)]),
    "odla_DestroyComputation": (C.c_int, [_V]),
    "odla_SetComputationItem": (C.c_int, [_V, C.c_int, _V]),
    "odla_CreateContext": (C.c_int, [C.POINTER(_V)]),
    "odla_DestroyContext": (C.c_int, [_V]),
    "odla_ExecuteComputation": (C.c_int, [_V, _V, C.c_int, _V]),
    "odla_SetContextItem": (C.c_int, [_V, C.c_int, _V]),
    "odla_GetNumOfArgsFromComputation": (C.c_int, [_V, C.POINTER(C.c_uint32)]),
    "odla_GetArgFromComputationByIdx": (C.c_int, [_V, C.c_uint32, C.POINTER(_V)]),
    "odla_GetNumOfOutputsFromComputation": (C.c_int, [_V, C.POINTER(C.c_uint32)]),
    "odla_GetOutputFromComputationByIdx": (C.c_int, [_V, C.c_uint32, C.POINTER(_V)]),
    "odla_GetValueType": (C.c_int, [_V, C.POINTER(ValueType)]),
    "odla_GetValueId": (C.c_int, [_V, C.POINTER(C.c_char_p)]),
    "odla_GetRuntimeShape": (C.c_int, [_V, _V, C.POINTER(Shape)]),
    "odla_SetValueAsOutput": (C.c_int, [_V]),
    "odla_BindToArgument": (C.c_int, [_V, _V, _V]),
    "odla_BindToArgumentById": (C.c_int, [_ID, _V, _V]),
    "odla_BindToOutput": (C.c_int, [_V, _V, _V]),
    "odla_BindToOutputById": (C.c_int, [_ID, _V, _V]),
    "odla_CreateArgument": (_V, [ValueType, _ID]),
    "odla_CreateConstant": (_V, [ValueType, _V, _ID]),
    "odla_Conv": (_V, [_V, C.c_int, C.c_uint32, _V, C.c_int, _U32P, _U32P, _U32P, _U32P, _V, _S, _ID]),
    "odla_Gemm": (_V, [_V, C.c_uint32, _V, C.c_uint32, C.c_float, C.c_float, _V, _S, _ID]),
    "odla_BatchMatMul": (_V, [_V, C.c_uint32, _V, C.c_uint32, _S, _ID]),
    "odla_MaxPool": (_V, [_V, C.c_int, _U32P, _U32P, _U32P, _U32P, _S, _ID]),
    "odla_AveragePool": (_V, [_V, C.c_int, _U32P, _U32P, _U32P, _U32P, C.c_uint32, _S, _ID]),
    "odla_BatchNormalization": (_V, [_V, C.c_int, _V, _V, C.c_float, _V, _V, C.c_float, C.c_float, _ID]),
    "odla_Clamp": (_V, [_V, C.c_float, C.c_float, _ID]),
    "odla_LeakyRelu": (_V, [_V, C.c_float, _ID]),
    "odla_NMS": (_V, [_V, _V, C.c_uint32, C.c_float, C.c_float, ValueType, _ID]),
    "odla_PostProcess": (Values, [_V, _V, _V, _V, _V, _ID]),
    "odla_Gelu": (_V, [_V, C.c_uint32, _ID]),
    "odla_Softmax": (_V, [_V, C.c_int32, _ID]),
    "odla_LogSoftmax": (_V, [_V, C.c_int32, _ID]),
    "odla_ReduceMean": (_V, [_V, C.c_size_t, _U32P, C.c_uint32, _S, _ID]),
    "odla_LayerNorm": (_V, [_V, C.c_int32, _I32P, C.c_float, _V, _V, _ID]),
    "odla_Quantize": (_V, [_V, _V, _V, C.c_int32, C.c_int, _ID]),
    "odla_Dequantize": (_V, [_V, _V, _V, C.c_int32, C.c_int, _ID]),
    "odla_Reshape": (_V, [_V, _S, _ID]),
    "odla_Transpose": (_V, [_V, _S, _S, _ID]),
    "odla_Concat": (_V, [Values, C.c_int32, _S, _ID]),
    "odla_Resize": (_V, [_V, C.c_int, C.c_int, C.c_uint32, _S, _ID]),
    "odla_Gather": (_V, [_V, _V, C.c_int32, _S, _ID]),
    "odla_Slice": (_V, [_V, _I32P, _I32P, _I32P, _S, _ID]),
    "odla_Cast": (_V, [_V, C.c_int, _ID]),
    "odla_GetVersionString": (C.c_char_p, []),
}
_UNARY = ["Relu", "Sigmoid", "Tanh", "Exp", "Log", "Erf", "Sqrt", "Rsqrt", "Abs", "Neg", "Reciprocal", "Round"]
_BINARY = ["Add", "Sub", "Mul", "Div", "Pow", "PRelu"]
for _n in _UNARY:
    _SIGNATURES["odla_" + _n] = (_V, [_V, _ID])
for _n in _BINARY:
    _SIGNATURES["odla_" + _n] = (_V, [_V, _V, _ID])
_OPTIONAL = {
    "odla_AllocateDevice": (C.c_int, [_V, C.c_int, C.c_int32, C.POINTER(_V)]),
    "odla_DestroyDevice": (C.c_int, [_V]),
    "odla_SetCurrentDevice": (C.c_int, [_V]),
    "odla_GetDeviceInfo": (C.c_int, [_V, C.c_int, C.POINTER(ScalarValue)]),
    "odla_SetLogLevel": (C.c_int, [C.c_int]),
    "odla_AllocateHostMemory": (C.c_int, [C.POINTER(_V), C.c_size_t]),
    "odla_FreeHostMemory": (C.c_int, [_V]),
    "odla_AsyncExecuteComputation": (C.c_int, [_V, _V, C.c_int, _V]),
    "odla_b200_WaitContext": (C.c_int, [_V]),
    "odla_b200_ContextLane": (C.c_int, [_V]),
    "odla_b200_DeviceCount": (C.c_int, []),
    "odla_b200_LastExecuteDeviceMs": (C.c_float, [_V]),
    "odla_b200_LastExecuteLaunches": (C.c_longlong, [_V]),
    "odla_b200_SetProfiling": (C.c_int, [_V, C.c_int]),
    "odla_b200_GetProfile": (C.c_int, [_V, C.POINTER(ProfileEntry), C.c_int]),
    "odla_b200_DescribePlan": (C.c_int, [_V, C.c_char_p, C.c_int]),
    "odla_b200_PreparedConstantStats": (None, [_V, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "odla_StoreExecutable": (C.c_int, [ResourceLocation, _V]),
    "odla_LoadExecutable": (C.c_int, [ResourceLocation, _V, C.POINTER(_V)]),
    "odla_CompileComputation": (C.c_int, [_V, _V, C.POINTER(_V)]),
    "odla_b200_SetRangeProfiling": (C.c_int, [_V, C.c_int]),
    "odla_b200_GetQuantTable": (C.c_int, [_V, C.POINTER(QuantInfo), C.c_int]),
    "odla_b200_PlanShards": (C.c_int, [_V, C.c_longlong, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong), C.c_int]),
    "odla_b200_conv_umma": (C.c_int, [C.POINTER(ConvDesc), _V, _V, _V, _V, _V, _V, _V]),
    "odla_b200_attention": (C.c_int, [C.c_int, _V, _V, _V, _V, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _V]),
    "odla_b200_reduce_mean_noalloc": (C.c_int, [_V, _V, C.c_int, C.POINTER(C.c_longlong), C.c_int, C.POINTER(C.c_int), C.c_int, _V]),
    "odla_cpuref_UsesReference": (C.c_int, []),
    "odla_cpuref_Threads": (C.c_int, []),
    "odla_cpuref_GetAccumulators": (C.c_longlong, [_V, C.c_char_p, _V, C.c_longlong]),
    "odla_cpuref_GetValueData": (C.c_longlong, [_V, C.c_char_p, _V, C.c_longlong]),
}


def default_library_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libodla_b200.so")


class OdlaLib:
    """A loaded ODLA platform library with typed entry points."""

    def __init__(self, path=None):
        self.path = path or default_library_path()
        if not os.path.exists(self.path):
            raise FileNotFoundError(
                "%s is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')" % self.path)
        self.dll = C.CDLL(self.path, mode=C.RTLD_LOCAL)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(self.dll, name)
            fn.restype, fn.argtypes = res, args
            setattr(self, name[5:], fn)
        for name, (res, args) in _OPTIONAL.items():
            try:
                fn = getattr(self.dll, name)
            except AttributeError:
                continue
            fn.restype, fn.argtypes = res, args
            setattr(self, name[5:], fn)

    def version(self):
        return self.GetVersionString().decode()


def _cname(name):
    return "".join(ch if ch.isalnum() or ch == "_" else "_" for ch in name)


class Context:
    """A further odla_context of a Graph's computation, with bindings of its own.  libodla_b200 gives the second context
    of a computation its own arenas and streams, so two contexts can be in flight: start one with execute_async()
    while the other still runs and its input copy proceeds under the other's kernels."""

    def __init__(self, graph):
        self.lib, self.comp, self.graph = graph.lib, graph.comp, graph
        self.ctx = _V()
        Graph._check(self.lib.CreateContext(C.byref(self.ctx)), "odla_CreateContext")

    def bind_input(self, name, ptr):
        Graph._check(self.lib.BindToArgumentById(name.encode(), C.c_void_p(ptr), self.ctx), "odla_BindToArgumentById")

    def bind_output(self, name, ptr):
        Graph._check(self.lib.BindToOutputById(name.encode(), C.c_void_p(ptr), self.ctx), "odla_BindToOutputById")

    def execute(self):
        return self.lib.ExecuteComputation(self.comp, self.ctx, 1, None)

    def execute_async(self):
        return self.lib.AsyncExecuteComputation(self.comp, self.ctx, 1, None)

    def wait(self):
        return self.lib.b200_WaitContext(self.ctx)

    def lane(self):
        return self.lib.b200_ContextLane(self.ctx)

    def close(self):
        if self.ctx is not None:
            self.lib.DestroyContext(self.ctx)
            self.ctx = None


class Graph:
    """One ODLA computation under construction.  Methods are named after the ODLA builders."""

    def __init__(self, lib, name="model", fp16=False, bf16=False, n_gpus=None, use_graph=None, sub_batches=None):
        self.lib, self.name = lib, name
        self._keep = []            # numpy constants and name strings must outlive the computation
        self.shapes, self.dtypes, self._handles = {}, {}, {}
        self.cc_consts, self.cc_body, self.cc_items = [], [], []
        self.const_arrays = {}
        self.arg_names, self.out_names = [], []
        self.comp = _V()
        self._check(lib.CreateComputation(C.byref(self.comp)), "odla_CreateComputation")
        self.ctx = None
        if fp16:
            self._item(ITEM_FP16_MODE, C.c_bool(True), "ODLA_FP16_MODE", "bool", "true")
        if bf16:
            self._item(ITEM_BF16_MODE, C.c_int(2), "ODLA_BF16_MODE", "odla_bf16_mode", "BF16_PERFORMACE_MODE")
        if n_gpus is not None:
            self._item(ITEM_PROCESSOR_NUM, C.c_int(n_gpus), "ODLA_PROCESSOR_NUM", "int", str(n_gpus))
        if use_graph is not None:
            self._item(ITEM_AGGREGATE_OPS, C.c_bool(use_graph), "ODLA_AGGREGATE_OPS", "bool", "true" if use_graph else "false")
        if sub_batches is not None:
            self._item(ITEM_BATCHES_PER_STEP, C.c_int(sub_batches), "ODLA_BATCHES_PER_STEP", "int", str(sub_batches))

    # ---- helpers ----
    @staticmethod
    def _check(status, what):
        if status != SUCCESS:
            raise RuntimeError("%s failed with odla_status %d" % (what, status))

    def _item(self, key, cval, key_name, ctype, ctext):
        self._keep.append(cval)
        self._check(self.lib.SetComputationItem(self.comp, key, C.cast(C.byref(cval), _V)), "odla_SetComputationItem")
        var = "item_%d" % len(self.cc_items)
        self.cc_items.append("  %s %s = %s;\n  odla_SetComputationItem(comp, %s, (odla_item_value)&%s);" % (ctype, var, ctext, key_name, var))

    def set_quant_table(self, records):
        """Hands a quantisation table to the computation (ODLA_QUANT_TABLE_SIZE, then ODLA_QUANT_TABLE).
        `records` = [(value_id, ch_idx, scale, offset, min, max), ...] laid out as utils/halo_pgq.py:309-327
        of the reference writes them: one record per value with ch_idx = -channels, then one per channel."""
        arr = (QuantInfo * len(records))()
        for i, (vid, ch, sc, off, mn, mx) in enumerate(records):
            arr[i] = QuantInfo(self._id(vid), int(ch), float(sc), float(off), float(mn), float(mx))
        n = C.c_int(len(records))
        self._keep += [arr, n]
        self._check(self.lib.SetComputationItem(self.comp, ITEM_QUANT_TABLE_SIZE, C.cast(C.byref(n), _V)), "odla_SetComputationItem")
        self._check(self.lib.SetComputationItem(self.comp, ITEM_QUANT_TABLE, C.cast(arr, _V)), "odla_SetComputationItem")
        self.quant_records = list(records)
        # generated code declares the table the way lib/target/generic_cpp/generic_cxx_codegen.cc:110-116 does
        self.cc_items.append("  odla_SetComputationItem(comp, ODLA_QUANT_TABLE_SIZE, (odla_item_value)&quant_infos_size);\n"
                             "  odla_SetComputationItem(comp, ODLA_QUANT_TABLE, (odla_item_value)quant_infos);")

    def emit_quant_table_c(self):
        """The C file utils/halo_pgq.py:309-333 of the reference writes next to the model."""
        fmt = '  {.value_id = (const odla_value_id) "%s", .ch_idx = %d, .scale = %r, .offset = %r, .min = %r, .max = %r},'
        lines = ["#include <ODLA/odla.h>", "const odla_value_quant_info quant_infos[] = {"]
        lines += [fmt % (v, ch, float(sc), float(off), float(mn), float(mx)) for (v, ch, sc, off, mn, mx) in self.quant_records]
        lines += ["};", "const int quant_infos_size = %d;" % len(self.quant_records), ""]
        return "\n".join(lines)

    def _id(self, name):
        b = name.encode()
        self._keep.append(b)
        return b

    def value_handle(self, name):
        """The odla_value behind a value id."""
        return self._handles[name]

    def _reg(self, name, handle, dims, et):
        if not handle:
            raise RuntimeError("builder for '%s' returned NULL" % name)
        self._handles[name] = handle
        self.shapes[name] = tuple(int(d) for d in dims)
        self.dtypes[name] = et
        return (name, handle)

    @staticmethod
    def _h(v):
        return None if v is None else v[1]

    @staticmethod
    def _n(v):
        return "nullptr" if v is None else _cname(v[0])

    @staticmethod
    def _cs(dims):
        return "{.size = %d, .dims = {%s}}" % (len(dims), ", ".join(str(int(d)) for d in dims))

    @staticmethod
    def _ca(vals, ctype="odla_uint32"):
        return "(const %s[]){%s}" % (ctype, ", ".join(str(int(v)) for v in vals))

    def _line(self, name, call):
        self.cc_body.append('  auto %s = %s, (const odla_value_id)"%s");' % (_cname(name), call, name))

    # ---- leaves ----
    def Argument(self, name, dims, et=FLOAT32):
        h = self.lib.CreateArgument(vtype(et, dims), self._id(name))
        self.arg_names.append(name)
        self.cc_body.append('  auto %s = odla_CreateArgument({%s, %s}, (const odla_value_id)("%s"));' % (_cname(name), _ENUM[et], self._cs(dims), name))
        return self._reg(name, h, dims, et)

    def Constant(self, name, array):
        a = np.ascontiguousarray(array)
        et = _NP2ODLA[a.dtype]
        self._keep.append(a)
        dims = a.shape if a.ndim else (1,)
        h = self.lib.CreateConstant(vtype(et, dims), a.ctypes.data_as(_V), self._id(name + "_"))
        sym = _cname(name)
        self.const_arrays[sym] = a
        self.cc_consts.append("extern const %s %s[%d];" % (_CTYPE[et], sym, max(a.size, 1)))
        self.cc_body.append('  auto %s_ = odla_CreateConstant({%s, %s}, %s, (const odla_value_id)"%s_");' % (sym, _ENUM[et], self._cs(dims), sym, sym))
        return self._reg(name + "_", h, dims, et)

    def Output(self, v):
        self._check(self.lib.SetValueAsOutput(v[1]), "odla_SetValueAsOutput")
        self.out_names.append(v[0])
        self.cc_body.append("  odla_SetValueAsOutput(%s);" % _cname(v[0]))

    # ---- ops (argument order of the C API) ----
    def Conv(self, x, layout, group, w, klayout, strides, dilations, pf, pb, bias, out_dims, name):
        h = self.lib.Conv(x[1], layout, group, w[1], klayout, _u32(strides), _u32(dilations), _u32(pf), _u32(pb), self._h(bias), shape(out_dims), self._id(name))
        lay = {CHANNELS_FIRST: "ODLA_CHANNELS_FIRST", CHANNELS_LAST: "ODLA_CHANNELS_LAST", SIO: "ODLA_SIO", OIS: "ODLA_OIS"}
        self._line(name, "odla_Conv(%s, odla_memory_layout::%s, %d, %s, odla_memory_layout::%s, %s, %s, %s, %s, %s, %s" % (
            self._n(x), lay[layout], group, self._n(w), lay[klayout], self._ca(strides), self._ca(dilations), self._ca(pf), self._ca(pb), self._n(bias), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def Gemm(self, a, ta, b, tb, alpha, beta, c, out_dims, name):
        h = self.lib.Gemm(a[1], int(ta), b[1], int(tb), alpha, beta, self._h(c), shape(out_dims), self._id(name))
        self._line(name, "odla_Gemm(%s, %d, %s, %d, %r, %r, %s, %s" % (self._n(a), ta, self._n(b), tb, float(alpha), float(beta), self._n(c), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[a[0]])

    def _pool(self, fn, x, layout, win, strides, pf, pb, out_dims, name, included=None):
        lay = "ODLA_CHANNELS_LAST" if layout == CHANNELS_LAST else "ODLA_CHANNELS_FIRST"
        if included is None:
            h = self.lib.MaxPool(x[1], layout, _u32(win), _u32(strides), _u32(pf), _u32(pb), shape(out_dims), self._id(name))
            extra = ""
        else:
            h = self.lib.AveragePool(x[1], layout, _u32(win), _u32(strides), _u32(pf), _u32(pb), int(included), shape(out_dims), self._id(name))
            extra = "%d, " % int(included)
        self._line(name, "%s(%s, odla_memory_layout::%s, %s, %s, %s, %s, %s%s" % (fn, self._n(x), lay, self._ca(win), self._ca(strides), self._ca(pf), self._ca(pb), extra, self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def MaxPool(self, x, layout, win, strides, pf, pb, out_dims, name):
        return self._pool("odla_MaxPool", x, layout, win, strides, pf, pb, out_dims, name)

    def AveragePool(self, x, layout, win, strides, pf, pb, included, out_dims, name):
        return self._pool("odla_AveragePool", x, layout, win, strides, pf, pb, out_dims, name, included)

    def BatchNormalization(self, x, layout, mean, var, eps, scale, offset, name, scalar_scale=1.0, scalar_offset=0.0):
        h = self.lib.BatchNormalization(x[1], layout, mean[1], var[1], eps, self._h(scale), self._h(offset), scalar_scale, scalar_offset, self._id(name))
        lay = "ODLA_CHANNELS_LAST" if layout == CHANNELS_LAST else "ODLA_CHANNELS_FIRST"
        self._line(name, "odla_BatchNormalization(%s, odla_memory_layout::%s, %s, %s, %r, %s, %s, %r, %r" % (
            self._n(x), lay, self._n(mean), self._n(var), float(eps), self._n(scale), self._n(offset), float(scalar_scale), float(scalar_offset)))
        return self._reg(name, h, self.shapes[x[0]], self.dtypes[x[0]])

    def _unary(self, fn, x, name, *extra):
        h = getattr(self.lib, fn)(x[1], *extra, self._id(name))
        self._line(name, "odla_%s(%s%s" % (fn, self._n(x), "".join(", %r" % e for e in extra)))
        return self._reg(name, h, self.shapes[x[0]], self.dtypes[x[0]])

    def Clamp(self, x, lo, hi, name):
        return self._unary("Clamp", x, name, float(lo), float(hi))

    def LeakyRelu(self, x, alpha, name):
        return self._unary("LeakyRelu", x, name, float(alpha))

    def Gelu(self, x, approx, name):
        return self._unary("Gelu", x, name, int(approx))

    def _binary(self, fn, a, b, name):
        h = getattr(self.lib, fn)(a[1], b[1], self._id(name))
        self._line(name, "odla_%s(%s, %s" % (fn, self._n(a), self._n(b)))
        try:
            dims = np.broadcast_shapes(self.shapes[a[0]], self.shapes[b[0]])
        except ValueError:   # the library records the error; keep building like generated code would
            dims = self.shapes[a[0]]
        return self._reg(name, h, dims, self.dtypes[a[0]])

    def Softmax(self, x, axis, name):
        return self._unary("Softmax", x, name, int(axis))

    def LogSoftmax(self, x, axis, name):
        return self._unary("LogSoftmax", x, name, int(axis))

    def ReduceMean(self, x, axes, keep_dims, out_dims, name):
        h = self.lib.ReduceMean(x[1], len(axes), _u32(axes), int(keep_dims), shape(out_dims), self._id(name))
        self._line(name, "odla_ReduceMean(%s, %d, %s, %d, %s" % (self._n(x), len(axes), self._ca(axes), int(keep_dims), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def LayerNorm(self, x, axes, eps, scale, offset, name):
        h = self.lib.LayerNorm(x[1], len(axes), _i32(axes), eps, self._h(scale), self._h(offset), self._id(name))
        self._line(name, "odla_LayerNorm(%s, %d, %s, %r, %s, %s" % (self._n(x), len(axes), self._ca(axes, "odla_int32"), float(eps), self._n(scale), self._n(offset)))
        return self._reg(name, h, self.shapes[x[0]], self.dtypes[x[0]])

    def Quantize(self, x, scale, zero_point, axis, target, name):
        h = self.lib.Quantize(x[1], scale[1], self._h(zero_point), axis, target, self._id(name))
        self._line(name, "odla_Quantize(%s, %s, %s, %d, %s" % (self._n(x), self._n(scale), self._n(zero_point), axis, _ENUM[target]))
        return self._reg(name, h, self.shapes[x[0]], target)

    def Dequantize(self, x, scale, zero_point, axis, target, name):
        h = self.lib.Dequantize(x[1], scale[1], self._h(zero_point), axis, target, self._id(name))
        self._line(name, "odla_Dequantize(%s, %s, %s, %d, %s" % (self._n(x), self._n(scale), self._n(zero_point), axis, _ENUM[target]))
        return self._reg(name, h, self.shapes[x[0]], target)

    def Reshape(self, x, out_dims, name):
        h = self.lib.Reshape(x[1], shape(out_dims), self._id(name))
        self._line(name, "odla_Reshape(%s, %s" % (self._n(x), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def Transpose(self, x, perm, out_dims, name):
        h = self.lib.Transpose(x[1], shape(perm), shape(out_dims), self._id(name))
        self._line(name, "odla_Transpose(%s, %s, %s" % (self._n(x), self._cs(perm), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def Concat(self, xs, axis, out_dims, name):
        vs = Values()
        vs.size = len(xs)
        for i, x in enumerate(xs):
            vs.values[i] = x[1]
        h = self.lib.Concat(vs, axis, shape(out_dims), self._id(name))
        self._line(name, "odla_Concat((odla_values){.size = %d, .values = {%s}}, %d, %s" % (len(xs), ", ".join(self._n(x) for x in xs), axis, self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[xs[0][0]])

    def Resize(self, x, out_dims, name, interpolation=0, mode=0, axes_mask=0):
        h = self.lib.Resize(x[1], interpolation, mode, axes_mask, shape(out_dims), self._id(name))
        self._line(name, "odla_Resize(%s, ODLA_NEAREST, ODLA_ASSYMMETRIC, %d, %s" % (self._n(x), axes_mask, self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def Gather(self, x, idx, axis, out_dims, name):
        h = self.lib.Gather(x[1], idx[1], axis, shape(out_dims), self._id(name))
        self._line(name, "odla_Gather(%s, %s, %d, %s" % (self._n(x), self._n(idx), axis, self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def Slice(self, x, start, end, stride, out_dims, name):
        h = self.lib.Slice(x[1], _i32(start), _i32(end), _i32(stride), shape(out_dims), self._id(name))
        self._line(name, "odla_Slice(%s, %s, %s, %s, %s" % (self._n(x), self._ca(start, "odla_int32"), self._ca(end, "odla_int32"), self._ca(stride, "odla_int32"), self._cs(out_dims)))
        return self._reg(name, h, out_dims, self.dtypes[x[0]])

    def NMS(self, boxes, scores, max_num_outputs, iou_threshold, score_threshold, out_rows, name, index_type=INT32):
        h = self.lib.NMS(boxes[1], scores[1], int(max_num_outputs), float(iou_threshold), float(score_threshold), vtype(index_type, (out_rows, 3)), self._id(name))
        self._line(name, "odla_NMS(%s, %s, %d, %r, %r, {%s, %s}" % (self._n(boxes), self._n(scores), max_num_outputs, float(iou_threshold), float(score_threshold),
                                                                  _ENUM[index_type], self._cs((out_rows, 3))))
        return self._reg(name, h, (out_rows, 3), index_type)

    def PostProcess(self, img_w, img_h, bb13, bb26, bb52, name):
        """odla_PostProcess returns two values: <name>0 = selected_info [classes, N/169, 5], <name>1 = selected_num [classes]."""
        vs = self.lib.PostProcess(img_w[1], img_h[1], bb13[1], bb26[1], bb52[1], self._id(name))
        dims = self.shapes[bb13[0]]
        ch = dims[1] if dims[2] == dims[3] else dims[3]
        cls = ch // 3 - 5
        self.cc_body.append("  auto %s = odla_PostProcess(%s, %s, %s, %s, %s, (const odla_value_id)\"%s\");" % (
            _cname(name), self._n(img_w), self._n(img_h), self._n(bb13), self._n(bb26), self._n(bb52), name))
        info = self._reg(name + "0", vs.values[0], (cls, 10647 // 169, 5), FLOAT32)
        num = self._reg(name + "1", vs.values[1], (cls,), UINT32)
        return info, num

    def Cast(self, x, target, name):
        h = self.lib.Cast(x[1], target, self._id(name))
        self._line(name, "odla_Cast(%s, %s" % (self._n(x), _ENUM[target]))
        return self._reg(name, h, self.shapes[x[0]], target)

    # ---- run ----
    def context(self):
        if self.ctx is None:
            self.ctx = _V()
            self._check(self.lib.CreateContext(C.byref(self.ctx)), "odla_CreateContext")
        return self.ctx

    def extra_context(self):
        """Another context of this computation (see Context).  odla_CreateContext attaches to the calling thread's
        current computation, i.e. the one created last: call this before building another Graph."""
        self.context()
        c = Context(self)
        self._extra = getattr(self, "_extra", []) + [c]
        return c

    def bind_input(self, name, ptr):
        self._check(self.lib.BindToArgumentById(name.encode(), C.c_void_p(ptr), self.context()), "odla_BindToArgumentById")

    def bind_output(self, name, ptr):
        self._check(self.lib.BindToOutputById(name.encode(), C.c_void_p(ptr), self.context()), "odla_BindToOutputById")

    def execute(self):
        return self.lib.ExecuteComputation(self.comp, self.context(), 1, None)

    def set_run_batch(self, n):
        """ODLA_RUN_BATCH_SIZE: run only the first n rows of the recorded batch (bound buffers hold n rows)."""
        v = C.c_int(n)
        return self.lib.SetContextItem(self.context(), ITEM_RUN_BATCH_SIZE, C.cast(C.byref(v), _V))

    def execute_async(self, callback=None, arg=None):
        """odla_AsyncExecuteComputation; `callback(arg, status)` runs on the library's worker thread when the outputs are written."""
        if callback is not None:
            self._async_cb = ASYNC_CALLBACK(callback)
            self._check(self.lib.SetContextItem(self.context(), ITEM_ASYNC_CALLBACK_FUNC, C.cast(self._async_cb, _V)), "odla_SetContextItem")
            self._check(self.lib.SetContextItem(self.context(), ITEM_ASYNC_CALLBACK_ARG, C.c_void_p(arg)), "odla_SetContextItem")
        return self.lib.AsyncExecuteComputation(self.comp, self.context(), 1, None)

    def wait(self):
        return self.lib.b200_WaitContext(self.context())

    def run(self, inputs):
        """inputs: dict name -> numpy array.  Returns dict output name -> numpy array."""
        keep = []
        for n in self.arg_names:
            a = np.ascontiguousarray(inputs[n])
            if _NP2ODLA[a.dtype] != self.dtypes[n] or tuple(a.shape) != self.shapes[n]:
                raise ValueError("input '%s': expected %s %s" % (n, self.shapes[n], _ODLA2NP[self.dtypes[n]]))
            keep.append(a)
            self.bind_input(n, a.ctypes.data)
        outs = {}
        for n in self.out_names:
            outs[n] = np.empty(self.shapes[n], dtype=_ODLA2NP[self.dtypes[n]])
            self.bind_output(n, outs[n].ctypes.data)
        self._check(self.execute(), "odla_ExecuteComputation")
        return outs

    def device_ms(self):
        return float(self.lib.b200_LastExecuteDeviceMs(self.context()))

    def launches(self):
        return int(self.lib.b200_LastExecuteLaunches(self.context()))

    def range_profiling(self, enabled=True):
        """Accumulate min / max of every materialised value during the following executes (calibration)."""
        self._check(self.lib.b200_SetRangeProfiling(self.context(), 1 if enabled else 0), "odla_b200_SetRangeProfiling")

    def quant_table(self):
        """The ranges collected so far as set_quant_table() records: [(value_id, ch_idx, scale, offset, min, max), ...]."""
        n = self.lib.b200_GetQuantTable(self.context(), None, 0)
        arr = (QuantInfo * max(n, 1))()
        n = self.lib.b200_GetQuantTable(self.context(), arr, n)
        return [(arr[i].value_id.decode(), arr[i].ch_idx, arr[i].scale, arr[i].offset, arr[i].min, arr[i].max) for i in range(n)]

    def plan_shards(self, visible_devices, run_batch=0):
        """[(device, first_row, rows), ...]: how an execute would be split over `visible_devices` GPUs (no GPU needed)."""
        cap = 256
        dev, start, rows = (C.c_int * cap)(), (C.c_longlong * cap)(), (C.c_longlong * cap)()
        n = self.lib.b200_PlanShards(self.comp, run_batch, visible_devices, dev, start, rows, cap)
        return [(dev[i], start[i], rows[i]) for i in range(min(n, cap))]

    def describe(self, first_gpu_only=False):
        """The launch list of every replica ("gpu <d> rows [a,b) ..." header, then one line per launch), or of the
        first replica only -- the lists are identical up to the batch shard."""
        need = self.lib.b200_DescribePlan(self.comp, None, 0)
        buf = C.create_string_buffer(max(need, 1))
        self.lib.b200_DescribePlan(self.comp, buf, need)
        text = buf.value.decode()
        if first_gpu_only:
            second = text.find("\ngpu ", 1)
            if second >= 0:
                text = text[:second + 1]
        return text

    def profile(self, runs=1):
        ctx = self.context()
        self.lib.b200_SetProfiling(ctx, 1)
        try:
            for _ in range(runs):
                self._check(self.execute(), "odla_ExecuteComputation")
            n = self.lib.b200_GetProfile(ctx, None, 0)
            arr = (ProfileEntry * n)()
            self.lib.b200_GetProfile(ctx, arr, n)
        finally:
            self.lib.b200_SetProfiling(ctx, 0)
        return [dict(op=e.op.decode(), name=e.name.decode(), ms=e.total_ms / max(e.launches, 1), launches=e.launches,
                     flops=e.flops, bytes=e.bytes) for e in arr]

    def store(self, path):
        """odla_StoreExecutable: the computation (graph, constants, items, prepared constants) as one file."""
        p = C.create_string_buffer(path.encode())
        self._keep.append(p)
        loc = ResourceLocation(0, C.cast(p, C.c_void_p), 0)
        self._check(self.lib.StoreExecutable(loc, self.comp), "odla_StoreExecutable")

    @classmethod
    def load(cls, lib, path):
        """odla_LoadExecutable: a Graph bound to the computation the file describes; arguments and outputs are
        discovered through the getters, as a program that only has the file would do."""
        g = cls.__new__(cls)
        g.lib, g.name = lib, os.path.basename(path)
        g._keep, g.shapes, g.dtypes, g._handles = [], {}, {}, {}
        g.cc_consts, g.cc_body, g.cc_items, g.const_arrays = [], [], [], {}
        g.arg_names, g.out_names, g.ctx = [], [], None
        p = C.create_string_buffer(path.encode())
        g._keep.append(p)
        exe = _V()
        cls._check(lib.LoadExecutable(ResourceLocation(0, C.cast(p, C.c_void_p), 0), None, C.byref(exe)), "odla_LoadExecutable")
        g.comp = exe
        for count, by_idx, names in ((lib.GetNumOfArgsFromComputation, lib.GetArgFromComputationByIdx, g.arg_names),
                                     (lib.GetNumOfOutputsFromComputation, lib.GetOutputFromComputationByIdx, g.out_names)):
            n = C.c_uint32()
            count(g.comp, C.byref(n))
            for i in range(n.value):
                h, vt, vid = _V(), ValueType(), C.c_char_p()
                by_idx(g.comp, i, C.byref(h))
                lib.GetValueType(h, C.byref(vt))
                lib.GetValueId(h, C.byref(vid))
                name = vid.value.decode()
                names.append(name)
                g._handles[name] = h
                g.shapes[name] = tuple(vt.shape.dims[k] for k in range(vt.shape.size))
                g.dtypes[name] = vt.element_type
        g.context()   # odla_CreateContext attaches to the current computation, which the load just made this one
        return g

    def prepared_stats(self):
        h, m, e = C.c_longlong(), C.c_longlong(), C.c_longlong()
        self.lib.b200_PreparedConstantStats(self.comp, C.byref(h), C.byref(m), C.byref(e))
        return {"hits": h.value, "misses": m.value, "entries": e.value}

    def close(self):
        for c in getattr(self, "_extra", []):
            c.close()
        self._extra = []
        if self.ctx is not None:
            self.lib.DestroyContext(self.ctx)
            self.ctx = None
        if self.comp:
            self.lib.DestroyComputation(self.comp)
            self.comp = _V()

    # ---- HALO-style source ----
    def emit_cc(self):
        """C++ text shaped like the output of HALO's generic C++ code generator
        (lib/target/generic_cpp/generic_cxx_codegen.cc:668-889 in the reference)."""
        fn = _cname(self.name)
        sig_in = ", ".join("const %s %s[%d]" % (_CTYPE[self.dtypes[n]], _cname(n), int(np.prod(self.shapes[n]))) for n in self.arg_names)
        sig_out = ", ".join("%s out_%s[%d]" % (_CTYPE[self.dtypes[n]], _cname(n), int(np.prod(self.shapes[n]))) for n in self.out_names)
        out = ["// HALO-style ODLA model (shape of the generic C++ code generator's output)", "#include <ODLA/odla.h>", ""]
        out += self.cc_consts
        if getattr(self, "quant_records", None):
            out += ['extern "C" {', "extern const odla_value_quant_info quant_infos[];", "extern const int quant_infos_size;", "}", ""]
        out += ['extern "C" {', "int %s(%s, %s);" % (fn, sig_in, sig_out), "int %s_init();" % fn, "int %s_fini();" % fn,
                "int %s_helper(odla_computation comp);" % fn, "};", "static odla_computation Comp;",
                "int %s_helper(odla_computation comp) {" % fn]
        out += self.cc_items + self.cc_body + ["  return ODLA_SUCCESS;", "}",
                "int %s_fini() { if (Comp) { odla_status s = odla_DestroyComputation(Comp); Comp = nullptr; return s; } return ODLA_SUCCESS; }" % fn,
                "int %s_init() {" % fn, "  if (Comp == nullptr) {", "    odla_status s = odla_CreateComputation(&Comp);",
                "    if (s != ODLA_SUCCESS) return s;", "    return %s_helper(Comp);" % fn, "  }", "  return ODLA_SUCCESS;", "}",
                "int %s(%s, %s) {" % (fn, sig_in, sig_out), "  int s = %s_init();" % fn, "  if (s != ODLA_SUCCESS) return s;",
                "  static odla_context Ctx;", "  if (Ctx == nullptr) { s = odla_CreateContext(&Ctx); if (s != ODLA_SUCCESS) return s; }"]
        for n in self.arg_names:
            out.append('  s = odla_BindToArgumentById((const odla_value_id)"%s", %s, Ctx); if (s != ODLA_SUCCESS) return s;' % (n, _cname(n)))
        for n in self.out_names:
            out.append('  s = odla_BindToOutputById((const odla_value_id)"%s", out_%s, Ctx); if (s != ODLA_SUCCESS) return s;' % (n, _cname(n)))
        out += ["  return odla_ExecuteComputation(Comp, Ctx, ODLA_COMPUTE_INFERENCE, nullptr);", "}", ""]
        return "\n".join(out)

    def write_constants(self, bin_path, asm_path):
        """Writes the constants as one raw blob plus an assembler file that gives every constant its
        own global OBJECT symbol -- the role of HALO's ELF constant object
        (lib/target/generic_llvmir/generic_constant_writer.cc:92-194)."""
        off, lines = 0, ['.section .rodata', '.balign 64']
        with open(bin_path, "wb") as f:
            for sym, a in self.const_arrays.items():
                pad = (-off) % 64
                f.write(b"\0" * pad)
                off += pad
                lines += [".globl %s" % sym, ".type %s, @object" % sym, ".size %s, %d" % (sym, a.nbytes), "%s:" % sym,
                          '.incbin "%s", %d, %d' % (os.path.abspath(bin_path), off, a.nbytes), ".balign 64"]
                f.write(a.tobytes())
                off += a.nbytes
        lines.append('.section .note.GNU-stack,"",@progbits')
        with open(asm_path, "w") as f:
            f.write("\n".join(lines) + "\n")


for _n in _UNARY:
    setattr(Graph, _n, (lambda fn: lambda self, x, name: self._unary(fn, x, name))(_n))
for _n in _BINARY:
    setattr(Graph, _n, (lambda fn: lambda self, a, b, name: self._binary(fn, a, b, name))(_n))
