"""ctypes wrapper of the C oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY: used by the tests, the smoke
check and the benchmark's CPU-baseline leg; never by the shipped package."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_build", "liboracle.so")
_lib = None
I64 = np.int64


def build():
    src = os.path.join(HERE, "oracle.c")
    if not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "_build/liboracle.so"], check=True, capture_output=True)
    return SO


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_sample_layer.restype = C.c_int64
        _lib.orc_cache_gather.restype = C.c_int64
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().orc_num_threads()


def set_threads(n):
    lib().orc_set_threads(int(n))


def tcsr_build(key, nbr, ts, eid, num_nodes):
    key, nbr, ts = (np.ascontiguousarray(a, I64) for a in (key, nbr, ts))
    eid = None if eid is None else np.ascontiguousarray(eid, I64)
    m = len(key)
    indptr = np.empty(num_nodes + 1, I64)
    o = [np.empty(m, I64) for _ in range(4)]
    rc = lib().orc_tcsr_build(C.c_int64(num_nodes), C.c_int64(m), _p(key), _p(nbr), _p(ts), _p(eid), _p(indptr),
                              _p(o[0]), _p(o[1]), _p(o[2]), _p(o[3]))
    if rc:
        raise ValueError("edge key outside [0, num_nodes)")
    return indptr, o[0], o[1], o[2], o[3]


def sample_layer(indptr, nbr, ts, eid, targets, target_ts, fanout, policy=0, *, equal_root_time=False, allowed_offset=-1,
                 keep_root_time=False, seed=0, stream=0, trim=True):
    targets, target_ts = np.ascontiguousarray(targets, I64), np.ascontiguousarray(target_ts, I64)
    n = len(targets)
    cap = max(n * fanout, 1)
    o_n, o_d, o_t, o_e = (np.empty(cap, I64) for _ in range(4))
    o_dt = np.empty(cap, np.float32)
    offs = np.empty(n + 1, I64)
    tot = lib().orc_sample_layer(_p(indptr), _p(nbr), _p(ts), _p(eid), _p(targets), _p(target_ts), C.c_int64(n),
                                 int(fanout), int(policy), int(equal_root_time), C.c_int64(allowed_offset),
                                 int(keep_root_time), C.c_uint64(seed), C.c_uint32(stream), _p(o_n), _p(o_d), _p(o_t),
                                 _p(o_dt), _p(o_e), _p(offs))
    if trim:
        return o_n[:tot], o_d[:tot], o_t[:tot], o_dt[:tot], o_e[:tot], np.diff(offs)
    return o_n, o_d, o_t, o_dt, o_e, offs


def gather_rows(table, idx, out=None):
    table = np.ascontiguousarray(table)
    idx = np.ascontiguousarray(idx, I64)
    if out is None:
        out = np.empty((len(idx),) + table.shape[1:], table.dtype)
    rb = table.strides[0] if table.ndim > 1 else table.itemsize
    lib().orc_gather_rows(_p(table), C.c_int64(table.shape[0]), C.c_int64(rb), _p(idx), C.c_int64(len(idx)), _p(out))
    return out


def cache_gather(cache, hitmap, backing, ids):
    ids = np.ascontiguousarray(ids, I64)
    n = len(ids)
    out = np.empty((n,) + backing.shape[1:], backing.dtype)
    mp, mi = np.empty(max(n, 1), I64), np.empty(max(n, 1), I64)
    nm = lib().orc_cache_gather(_p(cache), _p(hitmap), _p(backing), C.c_int64(backing.strides[0]), _p(ids), C.c_int64(n),
                                _p(out), _p(mp), _p(mi))
    return out, mp[:nm], mi[:nm]
