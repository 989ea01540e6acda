"""ctypes binding of liblbk.so, the C ABI of the CUDA kernels (see include/lbk.h).

Plays the role of the reference's ``legateboost/library.py`` (which loads ``liblegateboost.so``
and registers its tasks): it finds the shared object next to this file, declares the entry
points and keeps one context per CUDA device.  Nothing here computes on the CPU; a missing
library or device is an error.
"""
import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblbk.so")

LBK_F32, LBK_F64, LBK_I32, LBK_I64 = 0, 1, 2, 3
UNIQUE_ID_BYTES = 128

#: every symbol include/lbk.h declares
EXPORTS = [
    "lbk_version", "lbk_context_create", "lbk_context_destroy", "lbk_last_error", "lbk_context_trim",
    "lbk_context_set_allocator", "lbk_context_pool_bytes",
    "lbk_comm_unique_id", "lbk_comm_init", "lbk_comm_attach_nccl", "lbk_comm_set_callback",
    "lbk_comm_size", "lbk_owned_features", "lbk_selftest_peer_barrier", "lbk_profile_enable", "lbk_profile_histogram_ms", "lbk_profile_histogram_total", "lbk_build_tree", "lbk_sketch_bytes", "lbk_leaf_values", "lbk_update_tree", "lbk_gradient", "lbk_predict", "lbk_split_proposals", "lbk_bin_matrix",
    "lbk_bin_matrix_bytes", "lbk_quantise", "lbk_histogram", "lbk_histogram_noalloc", "lbk_group_rows",
]


ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p)
RELEASE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p)


class LbkError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("lbk error %d: %s" % (code, text))
        self.code = code


class BuildTreeArgs(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("x_dtype", C.c_int32), ("ldx", C.c_int64),
        ("g", C.c_void_p), ("h", C.c_void_p), ("ldg", C.c_int64),
        ("feature_set", C.c_void_p), ("row_offset", C.c_int64), ("n_local_rows", C.c_int64),
        ("n_features", C.c_int32), ("n_outputs", C.c_int32),
        ("max_depth", C.c_int32), ("max_nodes", C.c_int32), ("split_samples", C.c_int32),
        ("seed", C.c_int32), ("dataset_rows", C.c_int64),
        ("l1_regularization", C.c_double), ("l2_regularization", C.c_double),
        ("min_split_gain", C.c_double),
        ("leaf_value", C.c_void_p), ("feature", C.c_void_p), ("split_value", C.c_void_p),
        ("gain", C.c_void_p), ("hessian", C.c_void_p),
        ("stream", C.c_void_p), ("host_buffers", C.c_int32),
        ("trace_node_sums", C.c_void_p), ("trace_hist", C.c_void_p), ("trace_nodes", C.c_int32),
        ("out_total_bins", C.POINTER(C.c_int32)), ("out_leaf", C.c_void_p),
        ("sketch", C.c_void_p), ("sketch_mode", C.c_int32),
    ]


SKETCH_OFF, SKETCH_SAVE, SKETCH_REUSE = 0, 1, 2


class UpdateTreeArgs(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("x_dtype", C.c_int32), ("ldx", C.c_int64),
        ("g", C.c_void_p), ("h", C.c_void_p), ("ldg", C.c_int64),
        ("n_local_rows", C.c_int64), ("n_features", C.c_int32), ("n_outputs", C.c_int32),
        ("max_nodes", C.c_int32), ("feature", C.c_void_p), ("split_value", C.c_void_p),
        ("l1_regularization", C.c_double), ("l2_regularization", C.c_double),
        ("leaf_value", C.c_void_p), ("hessian", C.c_void_p), ("stream", C.c_void_p),
    ]


class PredictArgs(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("x_dtype", C.c_int32), ("ldx", C.c_int64), ("n_rows", C.c_int64),
        ("n_features", C.c_int32), ("n_outputs", C.c_int32), ("n_trees", C.c_int32),
        ("leaf_value", C.POINTER(C.c_void_p)), ("feature", C.POINTER(C.c_void_p)),
        ("split_value", C.POINTER(C.c_void_p)), ("max_nodes", C.POINTER(C.c_int32)),
        ("pred", C.c_void_p), ("ldp", C.c_int64), ("stream", C.c_void_p),
        ("host_buffers", C.c_int32),
    ]


class HistogramArgs(C.Structure):
    _fields_ = [
        ("bins", C.c_void_p), ("bin_bytes", C.c_int32), ("n_rows", C.c_int64),
        ("n_features", C.c_int32), ("row_ptr", C.c_void_p), ("total_bins", C.c_int32),
        ("gpair", C.c_void_p), ("gpair_f32", C.c_void_p), ("n_outputs", C.c_int32),
        ("row_index", C.c_void_p), ("seg", C.c_void_p), ("n_nodes", C.c_int32),
        ("mode", C.c_int32), ("hist", C.c_void_p), ("stream", C.c_void_p),
        ("host_buffers", C.c_int32), ("max_abs", C.c_void_p), ("max_bins", C.c_int32), ("all_reduce", C.c_int32),
        ("pairs_by_position", C.c_int32),
    ]


_lib = None
_lock = threading.Lock()
_contexts = {}


def load():
    """Load liblbk.so.  Raises if it has not been built (run ``python legate-boost_b200/build.py``)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    "liblbk.so is missing at %s: build it with `python legate-boost_b200/build.py` "
                    "(there is no CPU fallback)" % LIB_PATH)
            lib = C.CDLL(LIB_PATH)
            lib.lbk_version.restype = C.c_int
            lib.lbk_context_create.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
            lib.lbk_context_destroy.argtypes = [C.c_void_p]
            lib.lbk_context_destroy.restype = None
            lib.lbk_last_error.argtypes = [C.c_void_p]
            lib.lbk_last_error.restype = C.c_char_p
            lib.lbk_context_trim.argtypes = [C.c_void_p]
            lib.lbk_context_set_allocator.argtypes = [C.c_void_p, ALLOC_FN, RELEASE_FN, C.c_void_p]
            lib.lbk_context_pool_bytes.argtypes = [C.c_void_p, C.POINTER(C.c_size_t)]
            lib.lbk_comm_unique_id.argtypes = [C.c_void_p]
            lib.lbk_comm_init.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
            lib.lbk_comm_attach_nccl.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
            lib.lbk_comm_size.argtypes = [C.c_void_p]
            lib.lbk_owned_features.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
            lib.lbk_selftest_peer_barrier.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
            lib.lbk_profile_enable.argtypes = [C.c_void_p, C.c_int]
            lib.lbk_profile_histogram_ms.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
            lib.lbk_profile_histogram_total.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]
            lib.lbk_build_tree.argtypes = [C.c_void_p, C.POINTER(BuildTreeArgs)]
            lib.lbk_predict.argtypes = [C.c_void_p, C.POINTER(PredictArgs)]
            lib.lbk_histogram.argtypes = [C.c_void_p, C.POINTER(HistogramArgs)]
            lib.lbk_histogram_noalloc.argtypes = [C.c_int, C.POINTER(HistogramArgs)]
            lib.lbk_split_proposals.argtypes = [
                C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int,
                C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]
            lib.lbk_bin_matrix.argtypes = [
                C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_void_p,
                C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
            lib.lbk_sketch_bytes.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int]
            lib.lbk_sketch_bytes.restype = C.c_size_t
            lib.lbk_bin_matrix_bytes.argtypes = [C.c_int64, C.c_int, C.c_int]
            lib.lbk_bin_matrix_bytes.restype = C.c_size_t
            lib.lbk_quantise.argtypes = [
                C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int,
                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
            lib.lbk_leaf_values.argtypes = [
                C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
            lib.lbk_gradient.argtypes = [
                C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_double, C.c_void_p, C.c_void_p,
                C.c_void_p]
            lib.lbk_group_rows.argtypes = [
                C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
            _lib = lib
    return _lib


class Context:
    """One lbk context (scratch pool, status word, optional communicator) for one CUDA device."""

    def __init__(self, device: int):
        self.lib = load()
        self.device = device
        h = C.c_void_p()
        rc = self.lib.lbk_context_create(device, C.byref(h))
        if rc != 0:
            raise LbkError(rc, self.lib.lbk_last_error(None).decode())
        self.handle = h
        self.rank = 0
        self.n_ranks = 1

    def check(self, rc):
        if rc != 0:
            raise LbkError(rc, self.lib.lbk_last_error(self.handle).decode())

    def init_comm(self, id_bytes: bytes, rank: int, n_ranks: int):
        buf = C.create_string_buffer(id_bytes, UNIQUE_ID_BYTES)
        self.check(self.lib.lbk_comm_init(self.handle, buf, rank, n_ranks))
        self.rank, self.n_ranks = rank, n_ranks

    def use_torch_allocator(self, on=True):
        """Route the library's scratch through torch's caching allocator (``lbk_context_set_allocator``):
        every allocation is a uint8 tensor made on the current stream and kept until the library gives
        it back.  ``on=False`` restores the context's own pool."""
        import torch

        if not on:
            self.check(self.lib.lbk_context_set_allocator(self.handle, ALLOC_FN(0), RELEASE_FN(0), None))
            self._held, self._cbs = {}, None
            return
        held = {}
        device = torch.device("cuda", self.device)

        def alloc(user, nbytes, stream):
            try:
                t = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
            except RuntimeError:
                return None
            held[t.data_ptr()] = t
            return t.data_ptr()

        def release(user, ptr, stream):
            held.pop(ptr, None)

        self._held = held
        self._cbs = (ALLOC_FN(alloc), RELEASE_FN(release))  # keep the trampolines alive
        self.check(self.lib.lbk_context_set_allocator(self.handle, self._cbs[0], self._cbs[1], None))

    def pool_bytes(self) -> int:
        v = C.c_size_t(0)
        self.check(self.lib.lbk_context_pool_bytes(self.handle, C.byref(v)))
        return v.value

    def close(self):
        if self.handle:
            self.lib.lbk_context_destroy(self.handle)
            self.handle = None


def owned_features(rank: int, n_ranks: int, n_features: int):
    """[begin, end) of the features a rank owns when they are divided among the ranks."""
    lib = load()
    b, e = C.c_int(0), C.c_int(0)
    rc = lib.lbk_owned_features(rank, n_ranks, n_features, C.byref(b), C.byref(e))
    if rc != 0:
        raise LbkError(rc, lib.lbk_last_error(None).decode())
    return b.value, e.value


def unique_id() -> bytes:
    lib = load()
    buf = C.create_string_buffer(UNIQUE_ID_BYTES)
    rc = lib.lbk_comm_unique_id(buf)
    if rc != 0:
        raise LbkError(rc, lib.lbk_last_error(None).decode())
    return buf.raw


def context(device=None) -> Context:
    """The context of a CUDA device (default: torch's current device), created on first use."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: the tree kernels have no CPU fallback")
    if device is None:
        device = torch.cuda.current_device()
    with _lock:
        ctx = _contexts.get(device)
    if ctx is None:
        ctx = Context(device)
        with _lock:
            _contexts[device] = ctx
    return ctx


def init_distributed(device=None) -> Context:
    """Give the device's context a communicator over torch.distributed's default group: rank 0
    makes the id, every rank receives it, every rank joins (one rank per GPU)."""
    import torch.distributed as dist

    ctx = context(device)
    if not dist.is_initialized() or dist.get_world_size() == 1 or ctx.n_ranks > 1:
        return ctx
    box = [unique_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    ctx.init_comm(box[0], dist.get_rank(), dist.get_world_size())
    return ctx
