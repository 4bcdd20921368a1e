"""ctypes binding of the kernel-level C ABI (include/tbk.h) for callers that hold
device-resident data (torch CUDA tensors).  PyTorch is plumbing here: it owns device
memory and streams; every computation happens in the native library."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from . import _lib

REP_AUTO, REP_SPARSE, REP_ARRAY, REP_REORG = -1, 0, 1, 2
OUT_F32, OUT_I8 = 0, 1
REP_BY_NAME = {"auto": REP_AUTO, "sparse": REP_SPARSE, "gpu_sparse": REP_SPARSE, "array": REP_ARRAY,
               "gpu_array": REP_ARRAY, "reorg": REP_REORG, "gpu_reorg": REP_REORG}


class ForestArraysC(ctypes.Structure):
    _fields_ = [("num_trees", ctypes.c_int64), ("tree_off", ctypes.c_void_p),
                ("left", ctypes.c_void_p), ("right", ctypes.c_void_p),
                ("feat", ctypes.c_void_p), ("thr", ctypes.c_void_p),
                ("class_id", ctypes.c_void_p), ("num_classes", ctypes.c_int32),
                ("transform", ctypes.c_int32), ("initial_value", ctypes.c_double),
                ("num_features", ctypes.c_int32)]


class ScheduleC(ctypes.Structure):
    _fields_ = [("representation", ctypes.c_int32), ("tile_size", ctypes.c_int32),
                ("rows_per_block", ctypes.c_int32), ("rows_per_thread", ctypes.c_int32),
                ("tree_threads", ctypes.c_int32), ("tree_chunks", ctypes.c_int32),
                ("cache_trees", ctypes.c_int32), ("feature_bits", ctypes.c_int32),
                ("reserved", ctypes.c_int32 * 4)]


class ForestInfoC(ctypes.Structure):
    _fields_ = [("num_trees", ctypes.c_int64), ("num_nodes", ctypes.c_int64),
                ("num_groups", ctypes.c_int64), ("packed_bytes", ctypes.c_int64),
                ("max_depth", ctypes.c_int32), ("num_features", ctypes.c_int32),
                ("num_classes", ctypes.c_int32), ("transform", ctypes.c_int32),
                ("device", ctypes.c_int32), ("schedule", ScheduleC),
                ("staged", ctypes.c_int32), ("smem_bytes", ctypes.c_int32),
                ("threads_per_block", ctypes.c_int32), ("reserved", ctypes.c_int32 * 8)]


class TbkError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"tbk status {status}: {message}")
        self.status = status


_bound = False


def lib():
    global _bound
    L = _lib.load()
    if not _bound:
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32
        L.tbk_last_error.restype = ctypes.c_char_p
        L.tbk_forest_create.argtypes = [vp, vp, i32, i64, ctypes.POINTER(vp)]
        L.tbk_forest_free.argtypes = [vp]
        L.tbk_forest_get_info.argtypes = [vp, vp]
        L.tbk_predict.argtypes = [vp, vp, i64, i64, vp, i32, vp]
        L.tbk_predict_noalloc.argtypes = [vp, vp, i64, i64, vp, i32, vp]
        L.tbk_predict_partial.argtypes = [vp, vp, i64, i64, vp, vp]
        L.tbk_finalize.argtypes = [vp, vp, i64, vp, i32, vp]
        L.tbk_predict_leaf_ids.argtypes = [vp, vp, i64, i64, vp, vp]
        L.tbk_predict_host.argtypes = [vp, vp, i64, i64, vp, i32]
        L.tbk_set_timing.argtypes = [vp, i32]
        L.tbk_last_kernel_time_us.argtypes = [vp]
        L.tbk_last_kernel_time_us.restype = i64
        L.tbk_launch_count.argtypes = [vp]
        L.tbk_launch_count.restype = i64
        L.tbk_check_status.argtypes = [vp]
        L.tbk_debug_expire_next_wait.argtypes = [vp]
        L.tbk_host_layout_check.argtypes = [vp, vp, vp, i64, i64, vp, vp, vp]
        L.tbk_plan_launch.argtypes = [i32, i32, i64, i64, i32, vp, i64, i32, i32, i32, vp]
        u64 = ctypes.c_uint64
        L.tbk_image_create.argtypes = [vp, vp, i32, ctypes.POINTER(vp)]
        L.tbk_image_free.argtypes = [vp]
        L.tbk_image_serialize.argtypes = [vp, vp, u64, ctypes.POINTER(u64)]
        L.tbk_image_deserialize.argtypes = [vp, u64, ctypes.POINTER(vp)]
        L.tbk_image_matches.argtypes = [vp, vp, i32]
        L.tbk_forest_create_from_image.argtypes = [vp, vp, i32, i64, ctypes.POINTER(vp)]
        _bound = True
    return L


def _check(rc: int):
    if rc != 0:
        raise TbkError(rc, lib().tbk_last_error().decode())


def forest_arrays_c(f):
    """(struct, keep-alive list) for any object with the flat forest attributes
    (tree_off, left, right, feat, thr, class_id, num_classes, transform,
    initial_value, num_features)."""
    keep = [np.ascontiguousarray(f.tree_off, np.int64), np.ascontiguousarray(f.left, np.int32),
            np.ascontiguousarray(f.right, np.int32), np.ascontiguousarray(f.feat, np.int32),
            np.ascontiguousarray(f.thr, np.float32), np.ascontiguousarray(f.class_id, np.int32)]
    c = ForestArraysC(len(keep[0]) - 1, *[a.ctypes.data for a in keep], int(f.num_classes),
                      int(f.transform), float(f.initial_value), int(f.num_features))
    return c, keep


def make_schedule(representation="sparse", tile_size=1, rows_per_block=0, rows_per_thread=0,
                  tree_threads=0, tree_chunks=0, cache_trees=0, feature_bits=0) -> ScheduleC:
    rep = REP_BY_NAME[representation] if isinstance(representation, str) else int(representation)
    return ScheduleC(rep, tile_size, rows_per_block, rows_per_thread, tree_threads, tree_chunks,
                     cache_trees, feature_bits)


def _torch():
    import torch
    return torch


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        return _torch().cuda.current_stream().cuda_stream
    return stream.cuda_stream


class DeviceForest:
    """A packed forest resident on one GPU (tbk_forest*)."""

    def __init__(self, forest, device: int = 0, batch_hint: int = 0, **schedule):
        c, keep = forest_arrays_c(forest)
        sched = make_schedule(**schedule)
        h = ctypes.c_void_p()
        _check(lib().tbk_forest_create(ctypes.byref(c), ctypes.byref(sched), device, batch_hint,
                                       ctypes.byref(h)))
        self._h = h
        self.device = device
        self.num_trees = forest.num_trees
        self.num_classes = int(forest.num_classes)
        self.num_features = int(forest.num_features)

    @classmethod
    def from_handle(cls, handle: int, device: int, num_trees: int, num_classes: int,
                    num_features: int):
        self = cls.__new__(cls)
        self._h = ctypes.c_void_p(handle)
        self._borrowed = True
        self.device, self.num_trees = device, num_trees
        self.num_classes, self.num_features = num_classes, num_features
        return self

    def close(self):
        if getattr(self, "_h", None) and not getattr(self, "_borrowed", False):
            try:
                lib().tbk_forest_free(self._h)
            except TypeError:      # interpreter shutdown: module globals are already gone
                pass
        self._h = None

    __del__ = close

    def info(self) -> ForestInfoC:
        info = ForestInfoC()
        _check(lib().tbk_forest_get_info(self._h, ctypes.byref(info)))
        return info

    def _rows(self, rows):
        torch = _torch()
        assert rows.is_cuda and rows.dtype == torch.float32 and rows.dim() == 2
        assert rows.stride(1) == 1 and rows.shape[1] == self.num_features
        return rows.data_ptr(), rows.shape[0], rows.stride(0)

    def predict(self, rows, out=None, int8: bool = False, stream=None):
        """rows: CUDA float32 [n, F] (row stride free).  Returns a CUDA tensor [n]."""
        torch = _torch()
        ptr, n, ld = self._rows(rows)
        if out is None:
            out = torch.empty(n, device=rows.device, dtype=torch.int8 if int8 else torch.float32)
        _check(lib().tbk_predict(self._h, ptr, n, ld, out.data_ptr(), OUT_I8 if int8 else OUT_F32,
                                 _stream_ptr(stream)))
        return out

    def predict_partial(self, rows, out=None, stream=None):
        """Raw leaf-value sums [n, max(1, C)] (no initial value / transformation)."""
        torch = _torch()
        ptr, n, ld = self._rows(rows)
        if out is None:
            out = torch.empty((n, max(1, self.num_classes)), device=rows.device, dtype=torch.float32)
        _check(lib().tbk_predict_partial(self._h, ptr, n, ld, out.data_ptr(), _stream_ptr(stream)))
        return out

    def finalize(self, partial, out=None, int8: bool = False, stream=None):
        torch = _torch()
        n = partial.shape[0]
        if out is None:
            out = torch.empty(n, device=partial.device, dtype=torch.int8 if int8 else torch.float32)
        _check(lib().tbk_finalize(self._h, partial.data_ptr(), n, out.data_ptr(),
                                  OUT_I8 if int8 else OUT_F32, _stream_ptr(stream)))
        return out

    def predict_leaf_ids(self, rows, stream=None):
        torch = _torch()
        ptr, n, ld = self._rows(rows)
        out = torch.empty((n, self.num_trees), device=rows.device, dtype=torch.int32)
        _check(lib().tbk_predict_leaf_ids(self._h, ptr, n, ld, out.data_ptr(), _stream_ptr(stream)))
        return out

    def predict_host(self, rows: np.ndarray, out: Optional[np.ndarray] = None, int8: bool = False):
        """rows: host float32 [n, F] (numpy, pageable or pinned).  Copies in, runs, copies out."""
        assert rows.dtype == np.float32 and rows.ndim == 2 and rows.strides[1] == 4
        n, ld = rows.shape[0], rows.strides[0] // 4
        if out is None:
            out = np.empty(n, np.int8 if int8 else np.float32)
        _check(lib().tbk_predict_host(self._h, rows.ctypes.data, n, ld, out.ctypes.data,
                                      OUT_I8 if int8 else OUT_F32))
        return out

    def check_status(self):
        _check(lib().tbk_check_status(self._h))

    def expire_next_wait(self):
        """Failure drill: the next launch's first stage copy is skipped, its wait gives up."""
        _check(lib().tbk_debug_expire_next_wait(self._h))

    def set_timing(self, on: bool):
        _check(lib().tbk_set_timing(self._h, 1 if on else 0))

    def last_kernel_time_us(self) -> int:
        return int(lib().tbk_last_kernel_time_us(self._h))

    def launch_count(self) -> int:
        return int(lib().tbk_launch_count(self._h))


class PackedImage:
    """A packed forest in host memory (tbk_image*): pack once, serialise, upload later."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def pack(cls, forest, smem_limit: int = 0, **schedule):
        c, keep = forest_arrays_c(forest)
        sched = make_schedule(**schedule)
        h = ctypes.c_void_p()
        _check(lib().tbk_image_create(ctypes.byref(c), ctypes.byref(sched), smem_limit, ctypes.byref(h)))
        return cls(h)

    @classmethod
    def from_bytes(cls, data: bytes):
        h = ctypes.c_void_p()
        view = ctypes.c_char_p(data) if isinstance(data, bytes) else (ctypes.c_char * len(data)).from_buffer(data)
        _check(lib().tbk_image_deserialize(ctypes.cast(view, ctypes.c_void_p), len(data), ctypes.byref(h)))
        return cls(h)

    def to_bytes(self):
        """The serialised image (bytes; a bytearray above 64 MiB, to spare a copy)."""
        n = ctypes.c_uint64()
        _check(lib().tbk_image_serialize(self._h, None, 0, ctypes.byref(n)))
        buf = bytearray(n.value)
        view = (ctypes.c_char * n.value).from_buffer(buf)
        _check(lib().tbk_image_serialize(self._h, view, n.value, ctypes.byref(n)))
        del view
        return bytes(buf) if n.value < (1 << 26) else buf

    def matches(self, smem_limit: int = 0, **schedule) -> bool:
        sched = make_schedule(**schedule)
        return bool(lib().tbk_image_matches(self._h, ctypes.byref(sched), smem_limit))

    def upload(self, forest, device: int = 0, batch_hint: int = 0, **schedule) -> "DeviceForest":
        """Uploads the image; `forest` only supplies the sizes the wrapper keeps."""
        sched = make_schedule(**schedule)
        h = ctypes.c_void_p()
        _check(lib().tbk_forest_create_from_image(self._h, ctypes.byref(sched), device, batch_hint,
                                                  ctypes.byref(h)))
        df = DeviceForest.from_handle(h.value, device, forest.num_trees, int(forest.num_classes),
                                      int(forest.num_features))
        df._borrowed = False
        return df

    def close(self):
        if getattr(self, "_h", None):
            try:
                lib().tbk_image_free(self._h)
            except TypeError:
                pass
        self._h = None

    __del__ = close


def host_layout_check(forest, rows: Optional[np.ndarray], **schedule):
    """Packs on the host and interprets the packed buffers on the CPU (layout tests
    only).  Returns (leaf_ids [n, T], sums [n, max(1, C)], info)."""
    c, keep = forest_arrays_c(forest)
    sched = make_schedule(**schedule)
    info = ForestInfoC()
    if rows is None:
        _check(lib().tbk_host_layout_check(ctypes.byref(c), ctypes.byref(sched), None, 0, 0, None,
                                           None, ctypes.byref(info)))
        return None, None, info
    rows = np.ascontiguousarray(rows, np.float32)
    n = rows.shape[0]
    ids = np.full((n, forest.num_trees), -7, np.int32)
    sums = np.empty((n, max(1, int(forest.num_classes))), np.float32)
    _check(lib().tbk_host_layout_check(ctypes.byref(c), ctypes.byref(sched), rows.ctypes.data, n,
                                       rows.shape[1], ids.ctypes.data, sums.ctypes.data,
                                       ctypes.byref(info)))
    return ids, sums, info


def plan_launch(num_features: int, num_classes: int, num_groups: int, max_group_bytes: int,
                n_rows: int, lut_bytes: int = 2, smem_limit: int = 232448, num_sms: int = 148,
                partial_sums: bool = False, **schedule) -> ForestInfoC:
    sched = make_schedule(**schedule)
    info = ForestInfoC()
    _check(lib().tbk_plan_launch(num_features, num_classes, num_groups, max_group_bytes, lut_bytes,
                                 ctypes.byref(sched), n_rows, smem_limit, num_sms,
                                 1 if partial_sums else 0, ctypes.byref(info)))
    return info
