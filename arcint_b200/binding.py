"""ctypes binding over libb200q.so (see include/b200q.h for the contract).

Mirrors the C ABI one to one; `Context` adds numpy conveniences used by the tests and
the benchmark (upload, download, tensor descriptors). No compute happens in Python.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

F32, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS, I32 = 0, 2, 8, 12, 13, 14, 20, 23, 26
OP_MUL_MAT, OP_MUL_MAT_ID = 0, 1
OK, UNSUPPORTED, INVALID, CUDA_ERROR, NO_MEMORY, NCCL_ERROR, TIMEOUT, PEER_FAILED = range(8)
_BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_XS: (256, 136), IQ4_NL: (32, 18)}
STATUS_NAMES = ["OK", "UNSUPPORTED", "INVALID", "CUDA_ERROR", "NO_MEMORY", "NCCL_ERROR", "TIMEOUT", "PEER_FAILED"]


def block_size(t):
    return _BLOCK[t][0]


def block_bytes(t):
    return _BLOCK[t][1]


def row_bytes(t, k):
    return k // _BLOCK[t][0] * _BLOCK[t][1]


def tp_unique_id():
    """128-byte communicator id (rank 0 makes it, every rank gets a copy)."""
    buf = (C.c_uint8 * 128)()
    st = lib().b200q_tp_unique_id(buf)
    if st != OK:
        raise B200QError(st, "tp_unique_id")
    return bytes(buf)


def tp_shard(total, unit, nranks, rank):
    """(first, count) of the slice of `total` rank owns, in whole `unit`s."""
    first, count = C.c_int64(), C.c_int64()
    st = lib().b200q_tp_shard(total, unit, nranks, rank, C.byref(first), C.byref(count))
    if st != OK:
        raise B200QError(st, "tp_shard")
    return first.value, count.value


class B200QError(RuntimeError):
    def __init__(self, status, msg=""):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__("b200q: %s %s" % (name, msg))


class Tensor(C.Structure):
    """b200q_tensor: the ggml_tensor fields the path reads."""
    _fields_ = [("type", C.c_int32), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("data", C.c_void_p),
                ("id", C.c_void_p)]

    @staticmethod
    def make(type_, ne, nb, data, ident=None):
        t = Tensor()
        t.id = ident
        t.type = type_
        ne = list(ne) + [1] * (4 - len(ne))
        nb = list(nb)
        while len(nb) < 4:
            nb.append(nb[-1] * ne[len(nb) - 1])
        for i in range(4):
            t.ne[i] = ne[i]
            t.nb[i] = nb[i]
        t.data = data
        return t

    @staticmethod
    def weights(type_, dev_ptr, k, m, n_expert=1):
        rb = row_bytes(type_, k)
        return Tensor.make(type_, [k, m, n_expert, 1], [block_bytes(type_), rb, rb * m, rb * m * n_expert], dev_ptr)

    @staticmethod
    def f32(dev_ptr, ne):
        nb = [4]
        for d in ne[:-1]:
            nb.append(nb[-1] * d)
        return Tensor.make(F32, ne, nb, dev_ptr)


_lib = None


def lib_path():
    return os.path.join(HERE, "lib", "libb200q.so")


def lib():
    """Load libb200q.so. No fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not os.path.exists(p):
        raise ImportError("%s is missing: run `python -m arcint_b200.build` (or __graft_entry__.build())" % p)
    L = C.CDLL(p)
    vp, sz, TP = C.c_void_p, C.c_size_t, C.POINTER(Tensor)
    L.b200q_init.argtypes = [C.POINTER(vp), C.c_int, vp]
    L.b200q_free.argtypes = [vp]
    L.b200q_free.restype = None
    L.b200q_last_error.argtypes = [vp]
    L.b200q_last_error.restype = C.c_char_p
    L.b200q_version.restype = C.c_char_p
    L.b200q_get_stream.argtypes = [vp, C.POINTER(vp)]
    L.b200q_supports.argtypes = [vp, C.c_int, TP, TP, TP, TP]
    L.b200q_mul_mat.argtypes = [vp, TP, TP, TP]
    L.b200q_mul_mat_id.argtypes = [vp, TP, TP, TP, TP]
    L.b200q_graph_begin.argtypes = [vp]
    L.b200q_capture_begin.argtypes = [vp]
    L.b200q_capture_end.argtypes = [vp, C.POINTER(vp)]
    L.b200q_graph_launch.argtypes = [vp, vp]
    L.b200q_graph_free.argtypes = [vp]
    L.b200q_graph_free.restype = None
    L.b200q_tp_unique_id.argtypes = [vp]
    L.b200q_tp_init.argtypes = [vp, vp, C.c_int, C.c_int]
    L.b200q_tp_rank.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.b200q_tp_shard.argtypes = [C.c_int64, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    L.b200q_all_reduce_f32.argtypes = [vp, vp, sz]
    L.b200q_all_gather.argtypes = [vp, vp, vp, sz]
    L.b200q_mul_mat_allreduce.argtypes = [vp, TP, TP, TP]
    L.b200q_all_to_all_v.argtypes = [vp, vp, C.POINTER(sz), C.POINTER(sz), vp, C.POINTER(sz), C.POINTER(sz)]
    L.b200q_tp_check.argtypes = [vp]
    L.b200q_mul_mat_id_ep.argtypes = [vp, TP, TP, TP, TP, C.c_int]
    L.b200q_ep_reserve.argtypes = [vp, C.c_int64, C.c_int64, C.c_int64]
    L.b200q_moe_router.argtypes = [vp, TP, C.c_int, C.c_float, C.c_float, TP, TP]
    L.b200q_moe_ffn.argtypes = [vp, TP, TP, TP, TP, TP, C.c_int, C.c_float, C.c_float, TP, TP, TP]
    L.b200q_mul_mat_noalloc.argtypes = [C.c_int, vp, TP, TP, TP]
    L.b200q_noalloc_last_error.restype = C.c_char_p
    L.b200q_noalloc_device_error.argtypes = [C.c_int, C.POINTER(C.c_int)]
    L.b200q_buffer_alloc.argtypes = [vp, sz, C.POINTER(vp)]
    L.b200q_buffer_free.argtypes = [vp, vp]
    L.b200q_tensor_set.argtypes = [vp, vp, vp, sz]
    L.b200q_tensor_get.argtypes = [vp, vp, vp, sz]
    L.b200q_tensor_stage.argtypes = [vp, vp, vp, sz]
    L.b200q_tensor_fetch.argtypes = [vp, vp, vp, sz]
    L.b200q_tensor_copy.argtypes = [vp, vp, vp, sz]
    L.b200q_synchronize.argtypes = [vp]
    L.b200q_host_alloc.argtypes = [sz, C.POINTER(vp)]
    L.b200q_host_free.argtypes = [vp]
    L.b200q_stats.argtypes = [vp]
    L.b200q_stats.restype = C.c_char_p
    L.b200q_stats_reset.argtypes = [vp]
    L.b200q_stats_reset.restype = None
    L.b200q_timer_start.argtypes = [vp]
    L.b200q_timer_stop.argtypes = [vp, C.POINTER(C.c_float)]
    L.b200q_flush_l2.argtypes = [vp]
    L.b200q_debug_quantize_act.argtypes = [vp, C.c_int, TP, vp, vp, vp]
    L.b200q_debug_dequantize.argtypes = [vp, TP, vp]
    L.b200q_debug_wait_timeout.argtypes = [vp, C.c_uint]
    L.b200q_debug_check_guards.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    _lib = L
    return L


EXPORTS = [
    "b200q_init", "b200q_free", "b200q_last_error", "b200q_get_stream", "b200q_version", "b200q_supports", "b200q_mul_mat",
    "b200q_mul_mat_id", "b200q_graph_begin", "b200q_capture_begin", "b200q_capture_end", "b200q_graph_launch",
    "b200q_graph_free", "b200q_tp_unique_id", "b200q_tp_init", "b200q_tp_rank", "b200q_tp_shard", "b200q_all_reduce_f32",
    "b200q_all_gather", "b200q_mul_mat_allreduce", "b200q_all_to_all_v", "b200q_tp_check", "b200q_mul_mat_id_ep", "b200q_ep_reserve", "b200q_moe_router", "b200q_moe_ffn", "b200q_mul_mat_noalloc", "b200q_noalloc_last_error", "b200q_noalloc_device_error", "b200q_buffer_alloc", "b200q_buffer_free", "b200q_tensor_set",
    "b200q_tensor_get", "b200q_tensor_stage", "b200q_tensor_fetch", "b200q_tensor_copy", "b200q_synchronize", "b200q_host_alloc", "b200q_host_free",
    "b200q_stats", "b200q_stats_reset", "b200q_timer_start", "b200q_timer_stop", "b200q_flush_l2",
    "b200q_debug_quantize_act", "b200q_debug_dequantize", "b200q_debug_wait_timeout", "b200q_debug_check_guards",
]


class PinnedArray:
    """numpy view over page-locked host memory from b200q_host_alloc."""

    def __init__(self, shape, dtype):
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        st = lib().b200q_host_alloc(self.nbytes, C.byref(p))
        if st != OK:
            raise B200QError(st, "host_alloc")
        self.ptr = p.value
        buf = (C.c_uint8 * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib().b200q_host_free(self.ptr)
            self.ptr = None


class Context:
    def __init__(self, device=0, stream=None):
        self.L = lib()
        h = C.c_void_p()
        st = self.L.b200q_init(C.byref(h), device, stream)
        if st != OK:
            raise B200QError(st, "b200q_init(device=%d)" % device)
        self.h = h
        self._bufs = []

    def close(self):
        if self.h:
            for p in self._bufs:
                self.L.b200q_buffer_free(self.h, p)
            self._bufs = []
            self.L.b200q_free(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def check(self, st):
        if st != OK:
            raise B200QError(st, self.L.b200q_last_error(self.h).decode())

    # ---- memory ----
    def alloc(self, nbytes):
        p = C.c_void_p()
        self.check(self.L.b200q_buffer_alloc(self.h, nbytes, C.byref(p)))
        self._bufs.append(p.value)
        return p.value

    def free(self, ptr):
        self._bufs.remove(ptr)
        self.check(self.L.b200q_buffer_free(self.h, ptr))

    def upload(self, arr, dev=None):
        arr = np.ascontiguousarray(arr)
        if dev is None:
            dev = self.alloc(arr.nbytes)
        self.check(self.L.b200q_tensor_set(self.h, dev, arr.ctypes.data, arr.nbytes))
        self.sync()                                   # pageable source: keep it alive until copied
        return dev

    def download(self, dev, shape, dtype):
        out = np.empty(shape, dtype=dtype)
        self.check(self.L.b200q_tensor_get(self.h, out.ctypes.data, dev, out.nbytes))
        self.sync()
        return out

    def set_async(self, dev, host_ptr, nbytes):
        self.check(self.L.b200q_tensor_set(self.h, dev, host_ptr, nbytes))

    def get_async(self, host_ptr, dev, nbytes):
        self.check(self.L.b200q_tensor_get(self.h, host_ptr, dev, nbytes))

    def stage(self, dev, host_ptr, nbytes):
        """host -> device on the copy stream; kernels queued afterwards wait for it"""
        self.check(self.L.b200q_tensor_stage(self.h, dev, host_ptr, nbytes))

    def fetch(self, host_ptr, dev, nbytes):
        """device -> host on the copy stream, after the work queued so far; complete at the next sync()"""
        self.check(self.L.b200q_tensor_fetch(self.h, host_ptr, dev, nbytes))

    def copy(self, dst, src, nbytes):
        self.check(self.L.b200q_tensor_copy(self.h, dst, src, nbytes))

    def sync(self):
        self.check(self.L.b200q_synchronize(self.h))

    def stream(self):
        """The cudaStream_t (as an integer handle) the context enqueues on."""
        p = C.c_void_p()
        self.check(self.L.b200q_get_stream(self.h, C.byref(p)))
        return p.value

    # ---- the op ----
    def graph_begin(self):
        self.check(self.L.b200q_graph_begin(self.h))

    def supports(self, op, src0, src1, ids, dst):
        return self.L.b200q_supports(self.h, op, src0, src1, ids, dst)

    def mul_mat(self, src0, src1, dst):
        self.check(self.L.b200q_mul_mat(self.h, src0, src1, dst))

    def mul_mat_id(self, src0, src1, ids, dst):
        self.check(self.L.b200q_mul_mat_id(self.h, src0, src1, ids, dst))

    def mul_mat_status(self, src0, src1, dst):
        return self.L.b200q_mul_mat(self.h, src0, src1, dst)

    # ---- multi-GPU ----
    def tp_init(self, id_bytes, rank, nranks):
        buf = (C.c_uint8 * 128).from_buffer_copy(id_bytes)
        self.check(self.L.b200q_tp_init(self.h, buf, rank, nranks))

    def all_reduce_f32(self, dev, count):
        self.check(self.L.b200q_all_reduce_f32(self.h, dev, count))

    def mul_mat_allreduce(self, src0, src1, dst):
        self.check(self.L.b200q_mul_mat_allreduce(self.h, src0, src1, dst))

    def all_gather(self, send, recv, bytes_per_rank):
        self.check(self.L.b200q_all_gather(self.h, send, recv, bytes_per_rank))

    def all_to_all_v(self, send, send_off, send_bytes, recv, recv_off, recv_bytes):
        n = len(send_bytes)
        arr = lambda v: (C.c_size_t * n)(*[int(x) for x in v])
        self.check(self.L.b200q_all_to_all_v(self.h, send, arr(send_off), arr(send_bytes), recv, arr(recv_off), arr(recv_bytes)))

    def mul_mat_id_ep(self, src0_local, src1, ids, dst, n_expert_total):
        self.check(self.L.b200q_mul_mat_id_ep(self.h, src0_local, src1, ids, dst, n_expert_total))

    # ---- CUDA graphs ----
    def moe_router(self, logits, n_used, cmin, cmax, ids, weights):
        self.check(self.L.b200q_moe_router(self.h, logits, n_used, cmin, cmax, ids, weights))

    def moe_ffn(self, gate_w, up_w, down_w, x, logits, n_used, cmin, cmax, y, ids_out=None, weights_out=None):
        self.check(self.L.b200q_moe_ffn(self.h, gate_w, up_w, down_w, x, logits, n_used, cmin, cmax, y, ids_out, weights_out))

    def ep_reserve(self, max_pairs, max_k, max_m):
        self.check(self.L.b200q_ep_reserve(self.h, max_pairs, max_k, max_m))

    def capture(self, fn):
        """Record the calls fn() makes on this context into a graph; returns its handle."""
        self.check(self.L.b200q_capture_begin(self.h))
        try:
            fn()
        finally:
            g = C.c_void_p()
            st = self.L.b200q_capture_end(self.h, C.byref(g))
        self.check(st)
        return g

    def graph_launch(self, g):
        self.check(self.L.b200q_graph_launch(self.h, g))

    def graph_free(self, g):
        self.L.b200q_graph_free(g)

    # ---- stats / timing ----
    def stats(self):
        out = {}
        for line in self.L.b200q_stats(self.h).decode().splitlines():
            k, v = line.split("\t")
            out[k] = int(v)
        return out

    def stats_reset(self):
        self.L.b200q_stats_reset(self.h)

    def timer_start(self):
        self.check(self.L.b200q_timer_start(self.h))

    def timer_stop(self):
        ms = C.c_float()
        self.check(self.L.b200q_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        self.check(self.L.b200q_flush_l2(self.h))

    def check_guards(self):
        """(blocks looked at, blocks whose guard words were overwritten); needs B200Q_CANARY=1 at Context creation."""
        blocks, bad = C.c_int(0), C.c_int(0)
        self.check(self.L.b200q_debug_check_guards(self.h, C.byref(blocks), C.byref(bad)))
        return blocks.value, bad.value

    # ---- numpy conveniences for tests ----
    def run_mul_mat(self, type_, w_bytes, k, x):
        """w_bytes uint8 [m, row_bytes]; x f32 [n, k] -> f32 [n, m] (host arrays in, host array out)."""
        m, n = w_bytes.shape[0], x.shape[0]
        dw, dx, dy = self.upload(w_bytes), self.upload(x.astype(np.float32)), self.alloc(max(n * m * 4, 4))
        try:
            self.graph_begin()
            self.mul_mat(Tensor.weights(type_, dw, k, m), Tensor.f32(dx, [k, n]), Tensor.f32(dy, [m, n]))
            return self.download(dy, (n, m), np.float32)
        finally:
            for p in (dw, dx, dy):
                self.free(p)
