"""Python mirror of the oneDNN-graph backend C API (``include/dnnl_graph_compiler.h``).

``GraphCompiler.compile(json)`` -> ``Executable``; ``Executable.execute(inputs, outputs)``
takes ``{tensor id: array}`` dictionaries, the way the reference's C API matches
tensors by id (src/dnnl/dnnl_graph_compiler.cpp:64-103).  Arrays may be numpy
arrays / CPU torch tensors (host pointers; staged by the library) or CUDA torch
tensors (device pointers; used in place).  The 3-method surface
(compile / execute / destroy) follows python/gc_mlir/graph_compiler.py:17-45 of
the reference (compile, jit, compile_and_jit) collapsed onto the C API.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

from . import lib as _lib

# dnnl_status_t
SUCCESS, OUT_OF_MEMORY, INVALID_ARGUMENTS, UNIMPLEMENTED = 0, 1, 2, 3
RUNTIME_ERROR, INVALID_GRAPH = 5, 7

_STATUS = {0: "success", 1: "out_of_memory", 2: "invalid_arguments", 3: "unimplemented", 5: "runtime_error",
           7: "invalid_graph"}


class DnnlError(RuntimeError):
    def __init__(self, status: int, msg: str = ""):
        super().__init__(f"dnnl status {status} ({_STATUS.get(status, '?')}) {msg}")
        self.status = status


class Context(C.Structure):
    _fields_ = [("num_threads", C.c_uint32)]


class Tensor(C.Structure):
    _fields_ = [("id", C.c_size_t), ("ndims", C.c_uint8), ("dims", C.POINTER(C.c_int64)), ("data", C.c_void_p)]


class _VersionPart(C.Structure):
    _fields_ = [("major", C.c_uint8), ("minor", C.c_uint8), ("patch", C.c_uint8), ("hash", C.c_char_p)]


class Version(C.Structure):
    _fields_ = [("api_version", _VersionPart), ("gc_version", _VersionPart)]


def _bind():
    l = _lib.load()
    if getattr(l, "_gc_api_bound", False):
        return l
    l.dnnl_graph_compiler_get_version.restype = C.POINTER(Version)
    l.dnnl_graph_compiler_create.argtypes = [C.POINTER(Context), C.POINTER(C.c_void_p)]
    l.dnnl_graph_compiler_create.restype = C.c_int
    l.dnnl_graph_compiler_destroy.argtypes = [C.c_void_p]
    l.dnnl_graph_compiler_destroy.restype = None
    l.dnnl_graph_compiler_compile.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]
    l.dnnl_graph_compiler_compile.restype = C.c_int
    l.dnnl_graph_compiler_destroy_executable.argtypes = [C.c_void_p]
    l.dnnl_graph_compiler_destroy_executable.restype = None
    l.dnnl_graph_compiler_execute.argtypes = [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor)]
    l.dnnl_graph_compiler_execute.restype = C.c_int
    l.gcb200_execute_on_stream.argtypes = [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]
    l.gcb200_execute_on_stream.restype = C.c_int
    l.gcb200_plan_dump.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    l.gcb200_plan_dump.restype = C.c_int
    l.gcb200_plan_arena.argtypes = [C.POINTER(C.c_int64), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.c_int64,
                                    C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    l.gcb200_plan_arena.restype = C.c_int
    l.gcb200_describe_launches.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    l.gcb200_describe_launches.restype = C.c_int
    l.gcb200_guard_check.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    l.gcb200_guard_check.restype = C.c_int
    l.gcb200_guard_selftest.argtypes = [C.c_void_p]
    l.gcb200_guard_selftest.restype = C.c_int
    l._gc_api_bound = True
    return l


def get_version():
    v = _bind().dnnl_graph_compiler_get_version().contents
    return ((v.api_version.major, v.api_version.minor, v.api_version.patch, v.api_version.hash.decode()),
            (v.gc_version.major, v.gc_version.minor, v.gc_version.patch, v.gc_version.hash.decode()))


def _describe(a):
    """-> (data pointer, shape) of a numpy array or torch tensor."""
    if hasattr(a, "data_ptr"):
        return a.data_ptr(), tuple(a.shape)
    return a.ctypes.data, tuple(a.shape)


def _pack(tensors: Dict[int, object], order=None):
    ids = list(tensors.keys()) if order is None else list(order)
    arr = (Tensor * max(len(ids), 1))()
    keep = []
    for i, tid in enumerate(ids):
        ptr, shape = _describe(tensors[tid])
        dims = (C.c_int64 * max(len(shape), 1))(*shape)
        keep.append(dims)
        arr[i] = Tensor(tid, len(shape), dims, ptr)
    return arr, keep


class BoundCall:
    """An execute call with its tensor structs built once: what a C caller does when it runs the same
    partition on the same buffers every step (the structs of dnnl_graph_compiler_execute are plain
    caller-owned memory, src/dnnl/dnnl_graph_compiler.cpp:214-226)."""

    def __init__(self, exe: "Executable", inputs, outputs):
        self._exe = exe
        self._i, self._ki = _pack(inputs)
        self._o, self._ko = _pack(outputs)
        self._bufs = (inputs, outputs)   # keep the arrays alive
        self._fn = _bind().dnnl_graph_compiler_execute

    def run(self) -> None:
        st = self._fn(self._exe._h, self._i, self._o)
        if st != SUCCESS:
            raise DnnlError(st, _lib.load().gcb200_last_error().decode(errors="replace"))


class Executable:
    def __init__(self, handle):
        self._h = handle

    def bind(self, inputs: Dict[int, object], outputs: Dict[int, object]) -> BoundCall:
        """Build the argument structs once; ``.run()`` then only makes the C call."""
        return BoundCall(self, inputs, outputs)

    def execute(self, inputs: Dict[int, object], outputs: Dict[int, object]) -> None:
        """Synchronous, like the reference: results are in ``outputs`` on return."""
        i_arr, k1 = _pack(inputs)
        o_arr, k2 = _pack(outputs)
        st = _bind().dnnl_graph_compiler_execute(self._h, i_arr, o_arr)
        if st != SUCCESS:
            raise DnnlError(st, _lib.load().gcb200_last_error().decode(errors="replace"))

    def execute_on_stream(self, inputs, outputs, stream=None) -> None:
        """Device tensors only: enqueue on ``stream`` (default: torch's current) and return."""
        import torch

        s = C.c_void_p((stream or torch.cuda.current_stream()).cuda_stream)
        i_arr, k1 = _pack(inputs)
        o_arr, k2 = _pack(outputs)
        st = _bind().gcb200_execute_on_stream(self._h, i_arr, o_arr, s)
        if st != SUCCESS:
            raise DnnlError(st, _lib.load().gcb200_last_error().decode(errors="replace"))

    def plan(self) -> str:
        n = C.c_size_t(0)
        _bind().gcb200_plan_dump(self._h, None, 0, C.byref(n))
        buf = C.create_string_buffer(n.value)
        _bind().gcb200_plan_dump(self._h, buf, n.value, None)
        return buf.value.decode()

    def launches(self, sm_count: int = 148) -> str:
        """One line per step: kernel and, for matmuls, the tile configuration chosen for ``sm_count`` SMs."""
        n = C.c_size_t(0)
        _bind().gcb200_describe_launches(self._h, sm_count, None, 0, C.byref(n))
        buf = C.create_string_buffer(n.value)
        _bind().gcb200_describe_launches(self._h, sm_count, buf, n.value, None)
        return buf.value.decode()

    def guard_check(self) -> int:
        """Damaged guard bands of the workspace arena (partitions compiled under GC_B200_GUARD); 0 = intact."""
        n = C.c_int(-1)
        st = _bind().gcb200_guard_check(self._h, C.byref(n))
        if st != 0:
            raise DnnlError(RUNTIME_ERROR, _lib.load().gcb200_last_error().decode(errors="replace"))
        return n.value

    def guard_selftest(self) -> None:
        """Damages one guard band from the host (test hook for the detection)."""
        st = _bind().gcb200_guard_selftest(self._h)
        if st != 0:
            raise DnnlError(RUNTIME_ERROR, _lib.load().gcb200_last_error().decode(errors="replace"))

    def destroy(self):
        if self._h:
            _bind().dnnl_graph_compiler_destroy_executable(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class GraphCompiler:
    def __init__(self, num_threads: int | None = None):
        l = _bind()
        h = C.c_void_p()
        ctx = Context(num_threads) if num_threads is not None else None
        st = l.dnnl_graph_compiler_create(C.byref(ctx) if ctx is not None else None, C.byref(h))
        if st != SUCCESS:
            raise DnnlError(st)
        self._h = h

    def compile(self, graph_json: str) -> Executable:
        h = C.c_void_p()
        st = _bind().dnnl_graph_compiler_compile(self._h, graph_json.encode(), C.byref(h))
        if st != SUCCESS:
            raise DnnlError(st, _lib.load().gcb200_last_error().decode(errors="replace"))
        return Executable(h)

    def destroy(self):
        if self._h:
            _bind().dnnl_graph_compiler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def schedule_memory(traces, alignment=1, hot_first=False, inplace=None):
    """The static memory planner on a raw trace — the interface of the reference's
    ``memoryplan::scheduleMemoryAllocations`` (include/gc/Transforms/StaticMemoryPlanning.h:57-62).

    traces: [(buffer id, size)], size 0 releases.  inplace: {buffer: [(candidate, "free" | "zero_offset"), ...]}.
    Returns (total, {buffer: offset}, {buffer: [reused buffers]})."""
    l = _bind()
    U64 = C.c_uint64
    n = len(traces)
    tb = (U64 * max(n, 1))(*[t[0] for t in traces])
    ts = (U64 * max(n, 1))(*[t[1] for t in traces])
    hb, hc, hk = [], [], []
    for b, cands in (inplace or {}).items():
        for c, kind in cands:
            hb.append(b); hc.append(c); hk.append(1 if kind == "free" else 0)
    nh = len(hb)
    a_hb, a_hc, a_hk = (U64 * max(nh, 1))(*hb), (U64 * max(nh, 1))(*hc), (C.c_int * max(nh, 1))(*hk)
    cap = n + 1
    ob, oo = (U64 * cap)(), (U64 * cap)()
    sb, sr = (U64 * (nh + 1))(), (U64 * (nh + 1))()
    n_out, n_sel, total = C.c_int(cap), C.c_int(nh + 1), U64(0)
    l.gcb200_schedule_memory.argtypes = [C.POINTER(U64), C.POINTER(U64), C.c_int, U64, C.c_int, C.POINTER(U64), C.POINTER(U64),
                                         C.POINTER(C.c_int), C.c_int, C.POINTER(U64), C.POINTER(U64), C.POINTER(C.c_int),
                                         C.POINTER(U64), C.POINTER(U64), C.POINTER(U64), C.POINTER(C.c_int)]
    st = l.gcb200_schedule_memory(tb, ts, n, alignment, int(hot_first), a_hb, a_hc, a_hk, nh, ob, oo, C.byref(n_out),
                                  C.byref(total), sb, sr, C.byref(n_sel))
    if st != 0:
        raise ValueError("bad planner request: " + _lib.load().gcb200_last_error().decode(errors="replace"))
    offsets = {int(ob[i]): int(oo[i]) for i in range(n_out.value)}
    reused: Dict[int, list] = {}
    for i in range(n_sel.value):
        reused.setdefault(int(sb[i]), []).append(int(sr[i]))
    return int(total.value), offsets, reused


def plan_arena(sizes, first, last, align=64):
    """Offsets and total size for buffers live over step ranges [first, last]."""
    n = len(sizes)
    b = (C.c_int64 * n)(*sizes)
    f = (C.c_int * n)(*first)
    la = (C.c_int * n)(*last)
    off = (C.c_int64 * n)()
    tot = C.c_int64(0)
    st = _bind().gcb200_plan_arena(b, f, la, n, align, off, C.byref(tot))
    if st != 0:
        raise ValueError("bad arena request")
    return list(off), tot.value
