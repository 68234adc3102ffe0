"""ctypes binding of libsgl_b200.so (the C ABI declared in include/sgl_b200.h).

There is no fallback: if the shared library is missing, or a tensor is not on a CUDA device, the call
raises.  ctypes releases the GIL around every foreign call, so the functions here can be driven from
worker threads the way the reference's pybind module is (csrc/srcs/starrygl/export.cu:193-250 uses
``py::gil_scoped_release`` on every heavy binding).
"""
import ctypes as C
import os
import threading

import torch

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "lib", "libsgl_b200.so")

SGL_DEV_BITS = {1: "node id out of range", 2: "timestamp outside the declared window", 4: "row index out of range",
                8: "output capacity exceeded", 16: "device-side wait timed out",
                32: "a peer sent a different number of rows than announced"}
POLICY = {"recent": 0, "uniform": 1}
GATHER_MODE = {"auto": 0, "vec": 1, "bulk": 2}

_lib = None
_lock = threading.Lock()

_vp, _i64, _i32, _u64, _u32, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_uint64, C.c_uint32, C.c_size_t

_SIGNATURES = {
    "sgl_last_error": (C.c_char_p, []),
    "sgl_build_info": (C.c_char_p, []),
    "sgl_radix_sort_ws_bytes": (_sz, [_i64]),
    "sgl_radix_sort_launches": (_i32, [_i64, _i32]),
    "sgl_radix_sort_u64_u32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, C.POINTER(C.c_int), _vp, _sz, _vp]),
    "sgl_tcsr_build_ws_bytes": (_sz, [_i64, _i64]),
    "sgl_tcsr_build": (_i32, [_i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(C.c_int64), _vp, _sz, _vp]),
    "sgl_sample_ws_bytes": (_sz, [_i64]),
    "sgl_sample_layer": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i64, _i32, _u64, _u32,
                                _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "sgl_tcsr_fence_len": (_i64, [_i64, _i64]),
    "sgl_tcsr_fence": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "sgl_sample_layer_fenced": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _i64, _i32, _u64, _u32,
                                       _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "sgl_sample_layer_static": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i32, _u64, _u32,
                                       _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "sgl_sample_gather": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i32, _u64, _u32,
                                 _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _sz, _vp]),
    "sgl_sample_gather_fenced": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i32, _u64, _u32,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _sz, _vp]),
    "sgl_unique_pairs_ws_bytes": (_sz, [_i64]),
    "sgl_unique_pairs": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _vp,
                                _vp, _sz, _vp]),
    "sgl_build_csc_ws_bytes": (_sz, [_i64, _i64]),
    "sgl_build_csc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp,
                             _i32, _vp, _vp, _sz, _vp]),
    "sgl_relabel_nodes_ws_bytes": (_sz, [_i64]),
    "sgl_relabel_nodes": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "sgl_gather_rows": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _vp]),
    "sgl_cache_gather_ws_bytes": (_sz, [_i64]),
    "sgl_cache_gather": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "sgl_scatter_rows": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _vp]),
    "sgl_wire_pitch": (_i64, [_i64, _i32, _i32]),
    "sgl_route_pack": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "sgl_route_unpack": (_i32, [_vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _vp]),
    "sgl_comm_unique_id": (_i32, [C.c_char_p, _sz]),
    "sgl_comm_init": (_i32, [C.POINTER(C.c_void_p), _i32, _i32, C.c_char_p]),
    "sgl_comm_destroy": (_i32, [_vp]),
    "sgl_route_exchange": (_i32, [_vp, _vp, C.POINTER(C.c_int64), _vp, C.POINTER(C.c_int64), _i64, _vp]),
    "sgl_cache_route_step": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), _vp,
                                    _vp, _vp, _i64, _vp, _i32, _vp, _vp]),
    "sgl_p2p_buffer_bytes": (_sz, [_i32, _i32, _i64, _i64]),
    "sgl_p2p_alloc": (_i32, [_sz, C.POINTER(C.c_void_p), C.c_char_p, _sz]),
    "sgl_p2p_open": (_i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "sgl_p2p_close": (_i32, [_vp]),
    "sgl_p2p_free": (_i32, [_vp]),
    "sgl_p2p_route_create": (_i32, [_i32, _i32, _i32, _i64, _i64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "sgl_p2p_route_destroy": (_i32, [_vp]),
    "sgl_p2p_route_send": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, C.POINTER(C.c_int64), _u64, _vp, _vp]),
    "sgl_p2p_route_recv": (_i32, [_vp, C.POINTER(C.c_int64), _vp, _i64, _i64, _i32, _vp, _u64, _vp, _vp]),
    "sgl_densify_time_groups": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "sgl_comm_info": (_i32, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "sgl_init_p2p": (_i32, [C.POINTER(C.c_int), _i32, C.POINTER(C.c_int)]),
    "sgl_route_add_grouped": (_i32, [_vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp]),
    "sgl_shard_gather": (_i32, [_vp, _vp, _i32, _i64, _vp, _i64, _vp, _vp, _vp, _vp]),
    "sgl_p2p_route_configure": (_i32, [_vp, _i64, _i64]),
    "sgl_p2p_route_send_dev": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _u64, _vp, _vp]),
    "sgl_p2p_route_recv_dev": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _vp, _u64, _vp, _vp]),
    "sgl_p2p_route_step": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), _vp, _i64,
                                  _vp, _u64, _vp, _vp]),
    "sgl_route_add_rows": (_i32, [_vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp]),
    "sgl_dist_pack": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "sgl_dist_unpack": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp]),
    "sgl_seeds_ws_bytes": (_sz, [_i64]),
    "sgl_seeds_in_window": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp,
                                   _vp, _vp, _vp, _sz, _vp]),
    "sgl_lower_bound_i64": (_i32, [_vp, _i64, _vp, _i32, _vp, _vp]),
    "sgl_plan_route_ws_bytes": (_sz, [_i64, _i64]),
    "sgl_plan_route": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                              _sz, _vp]),
    "sgl_slice_window_ws_bytes": (_sz, [_i64]),
    "sgl_slice_window": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                _vp, _vp, _vp, _sz, _vp]),
    "sgl_copy_prefix": (_i32, [_i32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "sgl_mail_reduce_ws_bytes": (_sz, [_i64]),
    "sgl_mail_reduce": (_i32, [_vp, _i64, _vp, _i64, _i64, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _sz, _vp]),
    "sgl_mailbox_write": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp]),
    "sgl_graph_capture_begin": (_i32, [_vp]),
    "sgl_graph_capture_end": (_i32, [_vp, C.POINTER(C.c_void_p)]),
    "sgl_graph_launch": (_i32, [_vp, _vp, _vp, _sz, _vp]),
    "sgl_graph_destroy": (_i32, [_vp]),
    "sgl_replica_lookup_ws_bytes": (_sz, [_i64]),
    "sgl_replica_lookup": (_i32, [_vp, _vp, _vp, _i64, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
}


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python starrygl-framework_b200/build.py` "
                        "(there is no CPU or PyTorch fallback for these operators)")
                l = C.CDLL(LIB_PATH)
                for name, (res, args) in _SIGNATURES.items():
                    f = getattr(l, name)
                    f.restype, f.argtypes = res, args
                _lib = l
    return _lib


class SglError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise SglError(f"libsgl_b200 error {rc}: {lib().sgl_last_error().decode()}")


def ptr(t):
    """Device-usable pointer of a tensor (None -> NULL): CUDA memory, or pinned host memory, which the GPU
    addresses directly under unified addressing.  Pageable CPU tensors are refused: there is no CPU path."""
    if t is None:
        return None
    if not t.is_cuda and not t.is_pinned():
        raise SglError("expected a CUDA (or pinned host) tensor: the data path has no CPU implementation")
    if not t.is_contiguous():
        raise SglError("expected a contiguous tensor")
    return t.data_ptr()


def stream_ptr(stream=None):
    s = torch.cuda.current_stream() if stream is None else stream
    return s.cuda_stream


class Workspace:
    """Per-(device, stream) scratch buffer handed to the library; grows geometrically, never shrinks."""

    def __init__(self):
        self._bufs = {}

    def get(self, nbytes, device, stream_id):
        key = (device.index, stream_id)
        b = self._bufs.get(key)
        if b is None or b.numel() < nbytes:
            b = torch.empty(max(int(nbytes * 1.25), 1 << 16), dtype=torch.uint8, device=device)
            self._bufs[key] = b
        return b


WORKSPACE = Workspace()


def workspace(nbytes, device, stream=None):
    sp = stream_ptr(stream)
    b = WORKSPACE.get(nbytes, device, sp)
    return b, b.data_ptr(), b.numel()


def decode_status(v):
    return ", ".join(txt for bit, txt in SGL_DEV_BITS.items() if v & bit) or "ok"
