"""ctypes front end of the native DataParallelTable (include/cunn_b200_dpt.h, csrc/dpt.cu).

`NativeDataParallelTable` keeps the reference's method names (DataParallelTable.lua): add, threads,
syncParameters, zeroGradParameters, updateParameters, getParameters, plus the pieces the reference does inside
forward / backward and this API exposes as calls of their own: exec (impl:exec), scatter (_distribute), gather
(_concat), bucketReady / reduce (the gradient exchange at the end of __backward), write / read (__write /
__read).  Python only forwards; replicas, streams, worker threads, NCCL and the watchdog live in the library.
"""
import ctypes

from ._lib import lib, check, CunnError

c_int, c_ll, c_void_p, c_size_t, c_float, c_double = (ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_size_t,
                                                     ctypes.c_float, ctypes.c_double)
EXEC_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_int, c_int, c_void_p)


def _decl(name, restype, argtypes):
    f = getattr(lib, name)
    f.restype, f.argtypes = restype, argtypes


_P = c_void_p
_decl("cunn_b200_dpt_slice_range", None, [c_ll, c_int, c_int, ctypes.POINTER(c_ll), ctypes.POINTER(c_ll)])
_decl("cunn_b200_dpt_nccl_load", c_int, [ctypes.c_char_p])
_decl("cunn_b200_dpt_unique_id", c_int, [_P])
_decl("cunn_b200_dpt_create", _P, [c_int, c_int, c_int])
_decl("cunn_b200_dpt_destroy", None, [_P])
_decl("cunn_b200_dpt_add", c_int, [_P, ctypes.POINTER(c_int), c_int, c_ll])
_decl("cunn_b200_dpt_add_rank", c_int, [_P, c_int, c_int, c_int, _P, c_ll])
_decl("cunn_b200_dpt_adopt_comms", c_int, [_P, ctypes.POINTER(_P), c_int])
_decl("cunn_b200_dpt_local_replicas", c_int, [_P])
_decl("cunn_b200_dpt_world", c_int, [_P])
_decl("cunn_b200_dpt_replica_rank", c_int, [_P, c_int])
_decl("cunn_b200_dpt_replica_device", c_int, [_P, c_int])
_decl("cunn_b200_dpt_param_count", c_ll, [_P])
for _n in ("params", "grads", "visible_grads", "stream"):
    _decl("cunn_b200_dpt_" + _n, _P, [_P, c_int])
_decl("cunn_b200_dpt_set_stream", c_int, [_P, c_int, _P])
_decl("cunn_b200_dpt_set_buffers", c_int, [_P, c_int, _P, _P, _P])
_decl("cunn_b200_dpt_threads", c_int, [_P])
_decl("cunn_b200_dpt_exec", c_int, [_P, EXEC_FN, _P])
_decl("cunn_b200_dpt_scatter", c_int, [_P, _P, c_ll, c_size_t, ctypes.POINTER(_P), ctypes.POINTER(c_ll)])
_decl("cunn_b200_dpt_gather", c_int, [_P, ctypes.POINTER(_P), c_ll, c_size_t, _P])
_decl("cunn_b200_dpt_sync_parameters", c_int, [_P])
_decl("cunn_b200_dpt_zero_grad_parameters", c_int, [_P])
_decl("cunn_b200_dpt_update_parameters", c_int, [_P, c_float])
_decl("cunn_b200_dpt_set_buckets", c_int, [_P, ctypes.POINTER(c_ll), c_int])
_decl("cunn_b200_dpt_bucket_ready", c_int, [_P, c_int, c_int])
_decl("cunn_b200_dpt_reduce", c_int, [_P])
_decl("cunn_b200_dpt_watchdog", c_int, [_P, c_double])
_decl("cunn_b200_dpt_file_write", c_int, [ctypes.c_char_p, ctypes.POINTER(c_int), c_int, _P, c_ll, _P, c_ll])
_decl("cunn_b200_dpt_file_info", c_int, [ctypes.c_char_p, ctypes.POINTER(c_int), ctypes.POINTER(c_ll), ctypes.POINTER(c_ll)])
_decl("cunn_b200_dpt_file_read", c_int, [ctypes.c_char_p, c_int, c_int, ctypes.POINTER(c_int), _P, _P])
_decl("cunn_b200_dpt_write", c_int, [_P, ctypes.c_char_p, _P, c_ll])
_decl("cunn_b200_dpt_read_params", c_int, [_P, ctypes.c_char_p, _P])


def slice_range(n, g, i):
    s, c = c_ll(), c_ll()
    lib.cunn_b200_dpt_slice_range(n, g, i, ctypes.byref(s), ctypes.byref(c))
    return s.value, c.value


def unique_id():
    """128 bytes naming a new NCCL clique (made on rank 0, handed to every rank)."""
    buf = ctypes.create_string_buffer(128)
    check(lib.cunn_b200_dpt_unique_id(buf))
    return buf.raw


def file_write(path, gpus, params, extra=b""):
    """params: contiguous float32 numpy array; extra: bytes."""
    import numpy as np
    params = np.ascontiguousarray(params, dtype=np.float32)
    g = (c_int * len(gpus))(*gpus)
    check(lib.cunn_b200_dpt_file_write(path.encode(), g, len(gpus), params.ctypes.data_as(_P), params.size,
                                       ctypes.c_char_p(extra) if extra else None, len(extra)))


def file_read(path, ngpus_wanted=0, gpus_available=0):
    """Returns (gpus, params, extra) with the GPU assignment the reference's __read would produce."""
    import numpy as np
    ng, np_, eb = c_int(), c_ll(), c_ll()
    check(lib.cunn_b200_dpt_file_info(path.encode(), ctypes.byref(ng), ctypes.byref(np_), ctypes.byref(eb)))
    n_out = ngpus_wanted if ngpus_wanted > 0 else ng.value
    gpus = (c_int * max(n_out, 1))()
    params = np.empty(np_.value, np.float32)
    extra = ctypes.create_string_buffer(max(eb.value, 1))
    check(lib.cunn_b200_dpt_file_read(path.encode(), ngpus_wanted, gpus_available, gpus, params.ctypes.data_as(_P), extra))
    return list(gpus)[:n_out], params, extra.raw[:eb.value]


class NativeDataParallelTable:
    def __init__(self, dimension=1, flattenParams=True, usenccl=True):
        # the reference's dimension is 1-based (DataParallelTable.lua:44); the library's is 0-based
        self.h = lib.cunn_b200_dpt_create(dimension - 1, int(flattenParams), int(usenccl))
        if not self.h:
            raise CunnError(lib.cunn_b200_last_error().decode())
        self._cb = None

    def close(self):
        if self.h:
            lib.cunn_b200_dpt_destroy(self.h)
            self.h = None

    # construction
    def add(self, nparams, gpus):
        check(lib.cunn_b200_dpt_add(self.h, (c_int * len(gpus))(*gpus), len(gpus), nparams))
        return self

    def add_rank(self, nparams, device, rank, world, uid=None):
        check(lib.cunn_b200_dpt_add_rank(self.h, device, rank, world, ctypes.c_char_p(uid) if uid else None, nparams))
        return self

    def threads(self):
        check(lib.cunn_b200_dpt_threads(self.h))
        return self

    # introspection
    def size(self):
        return lib.cunn_b200_dpt_world(self.h)

    def local_replicas(self):
        return lib.cunn_b200_dpt_local_replicas(self.h)

    def device(self, i):
        return lib.cunn_b200_dpt_replica_device(self.h, i)

    def rank(self, i):
        return lib.cunn_b200_dpt_replica_rank(self.h, i)

    def param_count(self):
        return lib.cunn_b200_dpt_param_count(self.h)

    def pointers(self, i):
        """(params, local grads, visible grads, stream) of local replica i as integers."""
        return tuple(getattr(lib, "cunn_b200_dpt_" + n)(self.h, i) for n in ("params", "grads", "visible_grads", "stream"))

    def set_stream(self, i, stream):
        check(lib.cunn_b200_dpt_set_stream(self.h, i, stream))

    def set_buffers(self, i, params, local, visible):
        check(lib.cunn_b200_dpt_set_buffers(self.h, i, params, local, visible))

    # running
    def exec(self, fn, ctx=None):
        """fn(replica, device, stream) -> int, run for every local replica (on its worker thread after threads())."""
        cb = EXEC_FN(lambda _ctx, i, dev, stream: int(fn(i, dev, stream) or 0))
        check(lib.cunn_b200_dpt_exec(self.h, cb, None))

    def scatter(self, src_ptr, rows, row_bytes, dst_ptrs):
        n = self.local_replicas()
        out = (c_ll * n)()
        check(lib.cunn_b200_dpt_scatter(self.h, src_ptr, rows, row_bytes, (_P * n)(*dst_ptrs), out))
        return list(out)

    def gather(self, src_ptrs, rows, row_bytes, dst_ptr):
        n = self.local_replicas()
        check(lib.cunn_b200_dpt_gather(self.h, (_P * n)(*src_ptrs), rows, row_bytes, dst_ptr))

    def syncParameters(self):
        check(lib.cunn_b200_dpt_sync_parameters(self.h))

    def zeroGradParameters(self):
        check(lib.cunn_b200_dpt_zero_grad_parameters(self.h))

    def updateParameters(self, lr):
        check(lib.cunn_b200_dpt_update_parameters(self.h, lr))

    def setBuckets(self, ends):
        check(lib.cunn_b200_dpt_set_buckets(self.h, (c_ll * len(ends))(*ends), len(ends)))

    def bucketReady(self, replica, bucket):
        check(lib.cunn_b200_dpt_bucket_ready(self.h, replica, bucket))

    def reduce(self):
        check(lib.cunn_b200_dpt_reduce(self.h))

    def watchdog(self, timeout_seconds):
        check(lib.cunn_b200_dpt_watchdog(self.h, timeout_seconds))

    def adopt_comms(self, comms):
        check(lib.cunn_b200_dpt_adopt_comms(self.h, (_P * len(comms))(*comms), len(comms)))

    def write(self, path, extra=b""):
        check(lib.cunn_b200_dpt_write(self.h, path.encode(), ctypes.c_char_p(extra) if extra else None, len(extra)))

    def read(self, path, extra_bytes=0):
        buf = ctypes.create_string_buffer(max(extra_bytes, 1))
        check(lib.cunn_b200_dpt_read_params(self.h, path.encode(), buf))
        return buf.raw[:extra_bytes]
