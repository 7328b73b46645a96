"""ctypes binding of libblaze_b200.so: the Blaze_* C API of the host runtime
(host/include/blaze/api/c_api/c_api_predictor.h) plus helpers that write NetDefs in
protobuf text format. Used by tests and bench.py; no computation happens here."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libblaze_b200.so")

_lib = None
vp, cp = C.c_void_p, C.c_char_p
FORWARD_CB = C.CFUNCTYPE(None, C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: build it first (there is no fallback)" % LIB_PATH)
        C.CDLL(os.path.join(HERE, "lib", "libxdlb200.so"), mode=C.RTLD_GLOBAL)
        L = C.CDLL(LIB_PATH)
        L.Blaze_GetLastErrorString.restype = cp
        L.Blaze_B200_AddTable.argtypes = [vp, cp, C.c_int64, C.c_int, C.c_int, vp, vp]
        L.Blaze_B200_LoadModelFromText.argtypes = [vp, cp, C.c_int]
        L.Blaze_B200_LoadSparseModelWeight.argtypes = [vp, cp, cp]
        L.Blaze_PredictorCreate.argtypes = [vp, C.c_int, C.c_int, C.POINTER(vp)]
        L.Blaze_PredictorReshapeInput.argtypes = [vp, cp, C.POINTER(C.c_int), C.c_int]
        L.Blaze_PredictorFeed.argtypes = [vp, cp, vp, C.c_int]
        L.Blaze_PredictorForward.argtypes = [vp]
        L.Blaze_PredictorOutputShape.argtypes = [vp, cp, C.POINTER(C.c_size_t), C.POINTER(C.POINTER(C.c_size_t))]
        L.Blaze_PredictorOutputDataType.argtypes = [vp, cp, C.POINTER(C.c_int)]
        L.Blaze_PredictorOutput.argtypes = [vp, cp, vp, C.c_size_t]
        L.Blaze_PredictorDelete.argtypes = [vp]
        L.Blaze_PredictorManagerDelete.argtypes = [vp]
        L.Blaze_PredictorManagerCreate.argtypes = [C.POINTER(vp)]
        L.Blaze_PredcitorManagerLoadModel.argtypes = [vp, cp, C.c_int]
        L.Blaze_LoadSparseModelWeight.argtypes = [vp, cp]
        L.Blaze_B200_PredictorFeedDevice.argtypes = [vp, cp, vp, C.c_size_t]
        L.Blaze_B200_PredictorOutputDevice.argtypes = [vp, cp, C.POINTER(vp), C.POINTER(C.c_size_t)]
        L.Blaze_B200_PredictorLastLaunchCount.argtypes = [vp, C.POINTER(C.c_int)]
        L.Blaze_PredictorListInputNames.argtypes = [vp, C.POINTER(C.c_size_t), C.POINTER(C.POINTER(cp))]
        L.Blaze_PredictorListOutputNames.argtypes = [vp, C.POINTER(C.c_size_t), C.POINTER(C.POINTER(cp))]
        L.Blaze_InitScheduler.argtypes = [C.c_int] * 6
        L.Blaze_B200_PredictorForwardAsync.argtypes = [vp, FORWARD_CB, vp]
        L.Blaze_B200_PlanBatch.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp]
        L.Blaze_B200_BatchingStats.argtypes = [C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        L.Blaze_B200_ModelOpTypes.argtypes = [vp, C.c_char_p, C.c_size_t]
        L.Blaze_B200_ShardUniqueId.argtypes = [vp]
        L.Blaze_B200_ShardedInit.argtypes = [vp, C.c_int, C.c_int, vp, C.c_int64, C.c_int, C.c_float]
        L.Blaze_B200_AddDeviceShard.argtypes = [vp, cp, C.c_int64, C.c_int, C.c_int, vp, C.c_int64]
        _lib = L
    return _lib


class BlazeError(RuntimeError):
    pass


def _ck(rc):
    if rc != 0:
        raise BlazeError(lib().Blaze_GetLastErrorString().decode())


NP_DTYPE = {1: np.float32, 2: np.int32, 10: np.int64, 12: np.float16}


def init_scheduler(enable_batching, max_batch_size=100, batch_timeout_micros=100, num_threads_for_cpu=4,
                   num_threads_for_cuda=4, num_threads_for_pipe=2):
    """InitScheduler of the predictor API; batching applies to predictors created afterwards."""
    _ck(lib().Blaze_InitScheduler(int(enable_batching), max_batch_size, batch_timeout_micros, num_threads_for_cpu,
                                  num_threads_for_cuda, num_threads_for_pipe))


def plan_batch(rows, max_tasks):
    """Positions of the waiting requests that would run together with request 0; rows[t][j] is the first
    dimension of request t's j-th per-sample input."""
    r = np.ascontiguousarray(rows, np.int64)
    r = r.reshape(len(rows), -1) if len(rows) else np.zeros((0, 1), np.int64)
    picked = np.zeros(max(len(rows), 1), np.int32)
    n = lib().Blaze_B200_PlanBatch(r.ctypes.data, r.shape[0], r.shape[1], max_tasks, picked.ctypes.data)
    if n < 0:
        _ck(n)
    return picked[:n].tolist()


def batching_stats():
    """(merged runs, requests they carried) since the process started."""
    b, t = C.c_int64(), C.c_int64()
    _ck(lib().Blaze_B200_BatchingStats(C.byref(b), C.byref(t)))
    return b.value, t.value


def shard_unique_id():
    buf = C.create_string_buffer(128)
    _ck(lib().Blaze_B200_ShardUniqueId(buf))
    return buf.raw


class PredictorManager:
    def __init__(self):
        self.h = vp()
        _ck(lib().Blaze_PredictorManagerCreate(C.byref(self.h)))
        self._keep = []

    def load_sparse(self, uri=None, type_="b200_sparse_puller"):
        _ck(lib().Blaze_B200_LoadSparseModelWeight(self.h, uri.encode() if uri else None, type_.encode()))

    def add_table(self, name, weights, storage_dtype=12, keys=None):
        w = np.ascontiguousarray(weights, dtype=np.float32)
        k = None if keys is None else np.ascontiguousarray(keys, dtype=np.int64)
        _ck(lib().Blaze_B200_AddTable(self.h, name.encode(), w.shape[0], w.shape[1], storage_dtype, w.ctypes.data,
                                      None if k is None else k.ctypes.data))

    def load_model_text(self, text, optimize=True):
        _ck(lib().Blaze_B200_LoadModelFromText(self.h, text.encode(), int(optimize)))

    def load_model_file(self, path, optimize=True):
        _ck(lib().Blaze_PredcitorManagerLoadModel(self.h, path.encode(), int(optimize)))

    def init_sharded(self, rank, world, unique_id, max_ids_per_step, partial_dtype=12, capacity_factor=2.0):
        """This process is shard `rank` of `world`; loads b200_sharded_sparse_puller."""
        self.load_sparse(None, "b200_sharded_sparse_puller")
        _ck(lib().Blaze_B200_ShardedInit(self.h, rank, world, unique_id, max_ids_per_step, partial_dtype, capacity_factor))

    def add_device_shard(self, name, tensor, dim, storage_dtype=12):
        """A shard already in device memory (a 2-D CUDA tensor, kept alive by the caller)."""
        self._keep.append(tensor)
        _ck(lib().Blaze_B200_AddDeviceShard(self.h, name.encode(), tensor.shape[0], dim, storage_dtype, tensor.data_ptr(),
                                            tensor.stride(0) * tensor.element_size()))

    def op_types(self):
        """Operator types of the loaded model, in execution order (after the fusion passes if they ran)."""
        n = lib().Blaze_B200_ModelOpTypes(self.h, None, 0)
        buf = C.create_string_buffer(n)
        _ck(lib().Blaze_B200_ModelOpTypes(self.h, buf, n))
        return buf.value.decode().split(",") if buf.value else []

    def create_predictor(self, device_type=1, device_id=0):
        h = vp()
        _ck(lib().Blaze_PredictorCreate(self.h, device_type, device_id, C.byref(h)))
        return Predictor(h)

    def close(self):
        if self.h:
            lib().Blaze_PredictorManagerDelete(self.h)
            self.h = None


class Predictor:
    def __init__(self, h):
        self.h = h

    def feed(self, name, array):
        a = np.ascontiguousarray(array)
        shape = (C.c_int * a.ndim)(*a.shape)
        _ck(lib().Blaze_PredictorReshapeInput(self.h, name.encode(), shape, a.ndim))
        _ck(lib().Blaze_PredictorFeed(self.h, name.encode(), a.ctypes.data, a.nbytes))
        return a            # keep alive until Forward: the copy is asynchronous

    def reshape(self, name, shape):
        s = (C.c_int * len(shape))(*shape)
        _ck(lib().Blaze_PredictorReshapeInput(self.h, name.encode(), s, len(shape)))

    def feed_raw(self, name, ptr, nbytes):
        _ck(lib().Blaze_PredictorFeed(self.h, name.encode(), ptr, nbytes))

    def feed_device(self, name, ptr, nbytes):
        _ck(lib().Blaze_B200_PredictorFeedDevice(self.h, name.encode(), ptr, nbytes))

    def forward(self):
        _ck(lib().Blaze_PredictorForward(self.h))

    def forward_async(self, callback):
        """Forward(cb): `callback()` runs when the outputs are ready (on the batch thread when batching is on)."""
        self._cb = FORWARD_CB(lambda _arg: callback())       # kept alive until the next call
        _ck(lib().Blaze_B200_PredictorForwardAsync(self.h, self._cb, None))

    def output_shape(self, name):
        nd, sh = C.c_size_t(), C.POINTER(C.c_size_t)()
        _ck(lib().Blaze_PredictorOutputShape(self.h, name.encode(), C.byref(nd), C.byref(sh)))
        return [sh[i] for i in range(nd.value)]

    def output(self, name, into=None):
        dt = C.c_int()
        _ck(lib().Blaze_PredictorOutputDataType(self.h, name.encode(), C.byref(dt)))
        shape = self.output_shape(name)
        out = into if into is not None else np.empty(shape, NP_DTYPE[dt.value])
        _ck(lib().Blaze_PredictorOutput(self.h, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def output_device(self, name):
        p, n = vp(), C.c_size_t()
        _ck(lib().Blaze_B200_PredictorOutputDevice(self.h, name.encode(), C.byref(p), C.byref(n)))
        return p.value, n.value

    def launches(self):
        n = C.c_int()
        _ck(lib().Blaze_B200_PredictorLastLaunchCount(self.h, C.byref(n)))
        return n.value

    def names(self, which="input"):
        nd, arr = C.c_size_t(), C.POINTER(cp)()
        f = lib().Blaze_PredictorListInputNames if which == "input" else lib().Blaze_PredictorListOutputNames
        _ck(f(self.h, C.byref(nd), C.byref(arr)))
        return [arr[i].decode() for i in range(nd.value)]

    def close(self):
        if self.h:
            lib().Blaze_PredictorDelete(self.h)
            self.h = None


# ---- NetDef text writer -------------------------------------------------------------------------------
def _esc(s):
    return s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n")


def arg_text(name, v):
    out = ['  arg { name: "%s"' % name]
    if isinstance(v, dict):                         # fixture form {"i":..}/{"floats":[..]}
        for k, val in v.items():
            vals = val if isinstance(val, list) else [val]
            for x in vals:
                out.append(' %s: %s' % (k, ('"%s"' % _esc(x)) if k in ("s", "strings") else x))
    elif isinstance(v, bool):
        out.append(" i: %d" % int(v))
    elif isinstance(v, int):
        out.append(" i: %d" % v)
    elif isinstance(v, float):
        out.append(" f: %r" % v)
    elif isinstance(v, str):
        out.append(' s: "%s"' % _esc(v))
    elif isinstance(v, (list, tuple, np.ndarray)):
        a = np.asarray(v)
        key = "ints" if a.dtype.kind in "iu" else "floats"
        out.append(" " + " ".join("%s: %s" % (key, repr(float(x)) if key == "floats" else int(x)) for x in a.ravel()))
    out.append(" }")
    return "".join(out)


def op_text(type_, inputs, outputs, args=None, name=""):
    lines = ['op { type: "%s" name: "%s"' % (type_, name or outputs[0])]
    lines += ['  input: "%s"' % i for i in inputs]
    lines += ['  output: "%s"' % o for o in outputs]
    for k, v in (args or {}).items():
        lines.append(arg_text(k, v))
    lines.append("}")
    return "\n".join(lines)


def constant_text(name, array, dtype):
    a = np.asarray(array)
    return op_text("ConstantFill", [], [name], {"shape": list(a.shape), "dtype": dtype,
                                               "value": a.astype(np.int64 if dtype in (2, 10) else np.float64).ravel()})


def netdef_text(ops, inputs=(), outputs=(), device_type=1, name="net"):
    """inputs: [(name, dtype)], outputs: [(name, dtype)]"""
    parts = ['name: "%s"' % name, 'run_mode: "simple"', "device_option { device_type: %d device_id: 0 }" % device_type]
    parts += ops
    parts += ['external_input { name: "%s" dtype: %d }' % (n, d) for n, d in inputs]
    parts += ['external_output { name: "%s" dtype: %d }' % (n, d) for n, d in outputs]
    return "\n".join(parts) + "\n"


def fixture_to_text(net, device_type=1):
    """A fixture net (tests/golden/blaze_op_fixtures.json) as NetDef text for the CUDA device."""
    ops = [op_text(o["type"], o["input"], o["output"], o["arg"], o["name"]) for o in net["ops"]]
    outs = [(n, e["dtype"] if isinstance(e["dtype"], int) else 1) for n, e in net["expected"].items()]
    return netdef_text(ops, [], outs, device_type)
