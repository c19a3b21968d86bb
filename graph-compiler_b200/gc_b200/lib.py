"""ctypes binding of libGcDnnlApi.so — the only way Python reaches the CUDA kernels.

There is no fallback: if the shared library is missing, or a launcher reports
that no sm_100 device is usable, an exception is raised.  torch is used here
only for device memory (``tensor.data_ptr()``) and the current stream.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libGcDnnlApi.so")

_i64, _u64, _i32, _int, _vp, _f32 = C.c_int64, C.c_uint64, C.c_int32, C.c_int, C.c_void_p, C.c_float


class GcB200Error(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"gc_b200 status {status}: {msg}")
        self.status = status


class MatmulConfig(C.Structure):
    """Mirror of ``gcb200_matmul_config``."""

    _fields_ = [("swapped", _int), ("bn", _int), ("splits", _int), ("stages", _int), ("group_m", _int), ("grid", _int),
                ("pair", _int), ("kpb", _int)]

    def __repr__(self):
        return (f"MatmulConfig(swapped={self.swapped}, bn={self.bn}, splits={self.splits}, stages={self.stages}, "
                f"group_m={self.group_m}, grid={self.grid}, pair={self.pair}, kpb={self.kpb})")


class TpMlpDesc(C.Structure):
    """Mirror of ``gcb200_tp_mlp_desc``."""

    _fields_ = [("world", _int), ("rank", _int), ("batch", _i64), ("layers", _int), ("hidden", C.POINTER(_i64)),
                ("weights", C.POINTER(_vp)), ("biases", C.POINTER(_vp)), ("relu", _int),
                ("recv", C.POINTER(_vp) * 2), ("act", C.POINTER(_vp) * 2), ("signals", C.POINTER(_vp)), ("x_in", C.POINTER(_vp)),
                ("recv_planes", _int)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python graph-compiler_b200/build.py` (there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.gcb200_last_error.restype = C.c_char_p
    sig = {
        "gcb200_device_error": [_vp, C.POINTER(_int)],
        "gcb200_sm_count": [C.POINTER(_int)],
        "gcb200_launch_count": [C.POINTER(_u64)],
        "gcb200_matmul_bf16_splitk_static": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp],
        "gcb200_static_error": [_vp, C.POINTER(_int)],
        "gcb200_attention_bf16": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp],
        "gcb200_matmul_bf16": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp],
        "gcb200_matmul_bf16_cfg": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, C.POINTER(MatmulConfig), _vp],
        "gcb200_matmul_bf16_f32out": [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp],
        "gcb200_matmul_bf16_f32out_push": [_vp, _vp, C.POINTER(_vp), _int, _int, _i64, _i64, _i64, _vp],
        "gcb200_reduce_bias_act_bf16": [_vp, _int, _i64, _vp, _vp, _i64, _i64, _int, _vp],
        "gcb200_matmul_bf16_f32out_scatter": [_vp, _vp, C.POINTER(_vp), _int, _int, _i64, _i64, _i64, _vp],
        "gcb200_matmul_bf16_f32out_push_mc": [_vp, _vp, _vp, _int, _i64, _i64, _i64, _vp],
        "gcb200_matmul_bf16_allgather_mc": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int, _vp],
        "gcb200_matmul_u8s8_allgather_mc": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp],
        "gcb200_matmul_bf16_allgather": [_vp, _vp, _vp, C.POINTER(_vp), _int, _i64, _i64, _i64, _i64, _int, _int, _int, _vp],
        "gcb200_matmul_u8s8_allgather": [_vp, _vp, _vp, _vp, _vp, C.POINTER(_vp), _int, _i64, _i64, _i64, _i64, _int, _vp],
        "gcb200_reduce_slice_broadcast_bf16": [_vp, _int, _i64, _i64, _vp, C.POINTER(_vp), _int, _i64, _int, _vp],
        "gcb200_matmul_u8s8": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp],
        "gcb200_colsum_s8": [_vp, _vp, _i64, _i64, _i32, _vp],
        "gcb200_matmul_f32": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp],
        "gcb200_select_matmul_config": [_i64, _i64, _i64, _int, _int, _int, C.POINTER(MatmulConfig)],
        "gcb200_model_matmul_config": [_i64, _i64, _i64, _int, _int, _int, C.POINTER(MatmulConfig)],
        "gcb200_tune_cache_put": [_i64, _i64, _i64, _int, _int, C.POINTER(MatmulConfig)],
        "gcb200_tune_cache_get": [_i64, _i64, _i64, _int, _int, C.POINTER(MatmulConfig), C.POINTER(_int)],
        "gcb200_tune_cache_load": [C.c_char_p, C.POINTER(_int)],
        "gcb200_tune_cache_save": [C.c_char_p, C.POINTER(_int)],
        "gcb200_tune_cache_erase": [_i64, _i64, _i64, _int, _int],
        "gcb200_tune_cache_clear": [],
        "gcb200_tp_mlp_create": [C.POINTER(TpMlpDesc), C.POINTER(_vp)],
        "gcb200_tp_mlp_destroy": [_vp],
        "gcb200_tp_mlp_describe": [_vp, _int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)],
        "gcb200_tp_mlp_step": [_vp, _vp, _vp, C.POINTER(_vp)],
        "gcb200_tp_mlp_execute": [_vp, _vp, _vp],
        "gcb200_tp_mlp_timeline": [_vp, _vp, _vp, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)],
        "gcb200_tp_mlp_trace": [_vp, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)],
        "gcb200_wait_selftest": [C.c_longlong, _vp],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _int
    lib.dnnl_brgemm_dispatch.restype = _i64
    lib.dnnl_brgemm_dispatch.argtypes = [_i64] * 8 + [_f32, _i64, _i64]
    lib.dnnl_brgemm_tileconfig.restype = None
    lib.dnnl_brgemm_tileconfig.argtypes = [_i64]
    lib.dnnl_brgemm_tilerelease.restype = None
    lib.dnnl_brgemm_execute.restype = None
    lib.dnnl_brgemm_execute.argtypes = [_i64, _vp, _u64, _vp, _u64, _vp, _u64, _int]
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise GcB200Error(status, load().gcb200_last_error().decode(errors="replace"))


def _ptr(t):
    return None if t is None else _vp(t.data_ptr())


def _stream():
    import torch

    return _vp(torch.cuda.current_stream().cuda_stream)


def sm_count() -> int:
    n = _int(0)
    check(load().gcb200_sm_count(C.byref(n)))
    return n.value


def launch_count() -> int:
    n = _u64(0)
    check(load().gcb200_launch_count(C.byref(n)))
    return n.value


def device_error() -> int:
    code = _int(0)
    check(load().gcb200_device_error(_stream(), C.byref(code)))
    return code.value


def select_matmul_config(M, N, K, dtype_bytes=2, out_bytes=2, sms=148) -> MatmulConfig:
    cfg = MatmulConfig()
    check(load().gcb200_select_matmul_config(M, N, K, dtype_bytes, out_bytes, sms, C.byref(cfg)))
    return cfg


def model_matmul_config(M, N, K, dtype_bytes=2, out_bytes=2, sms=148) -> MatmulConfig:
    """The time model's choice, ignoring measured configurations."""
    cfg = MatmulConfig()
    check(load().gcb200_model_matmul_config(M, N, K, dtype_bytes, out_bytes, sms, C.byref(cfg)))
    return cfg


def tune_cache_put(M, N, K, cfg: MatmulConfig, dtype_bytes=2, out_bytes=2):
    check(load().gcb200_tune_cache_put(M, N, K, dtype_bytes, out_bytes, C.byref(cfg)))


def tune_cache_get(M, N, K, dtype_bytes=2, out_bytes=2):
    """The measured configuration recorded for this shape, or None."""
    cfg, found = MatmulConfig(), _int(0)
    check(load().gcb200_tune_cache_get(M, N, K, dtype_bytes, out_bytes, C.byref(cfg), C.byref(found)))
    return cfg if found.value else None


def tune_cache_load(path: str) -> int:
    n = _int(0)
    check(load().gcb200_tune_cache_load(os.fsencode(path), C.byref(n)))
    return n.value


def tune_cache_save(path: str) -> int:
    n = _int(0)
    check(load().gcb200_tune_cache_save(os.fsencode(path), C.byref(n)))
    return n.value


def tune_cache_erase(M, N, K, dtype_bytes=2, out_bytes=2):
    check(load().gcb200_tune_cache_erase(M, N, K, dtype_bytes, out_bytes))


def tune_cache_clear():
    check(load().gcb200_tune_cache_clear())


# ----------------------------------------------------------------------------- launchers on torch CUDA tensors
def matmul_bf16(A, B, bias=None, relu=False, transpose_a=False, transpose_b=False, out=None, cfg: MatmulConfig | None = None):
    """Y = act(bf16(bf16(op(A).op(B)) + bias)) on bf16 CUDA tensors."""
    import torch

    assert A.is_cuda and A.dtype == torch.bfloat16 and A.is_contiguous() and B.is_contiguous()
    K, M = (A.shape if transpose_a else A.shape[::-1])
    N = B.shape[0] if transpose_b else B.shape[1]
    assert (B.shape[1] if transpose_b else B.shape[0]) == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    if cfg is None:
        check(load().gcb200_matmul_bf16(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), M, N, K, int(transpose_a),
                                        int(transpose_b), int(relu), _stream()))
    else:
        check(load().gcb200_matmul_bf16_cfg(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), M, N, K, int(transpose_a),
                                            int(transpose_b), int(relu), C.byref(cfg), _stream()))
    return out


def matmul_bf16_f32out(A, B, transpose_a=False, transpose_b=False, out=None):
    import torch

    K, M = (A.shape if transpose_a else A.shape[::-1])
    N = B.shape[0] if transpose_b else B.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    check(load().gcb200_matmul_bf16_f32out(_ptr(A), _ptr(B), _ptr(out), M, N, K, int(transpose_a), int(transpose_b),
                                           _stream()))
    return out


def matmul_bf16_f32out_push(A, B, peer_ptrs, my_plane: int):
    """f32 partial sums of A.B stored into plane ``my_plane`` of every buffer in ``peer_ptrs`` (ints)."""
    M, K = A.shape
    N = B.shape[1]
    arr = (_vp * len(peer_ptrs))(*peer_ptrs)
    check(load().gcb200_matmul_bf16_f32out_push(_ptr(A), _ptr(B), arr, len(peer_ptrs), my_plane, M, N, K, _stream()))


def matmul_bf16_f32out_push_mc(A, B, mc_ptr: int, my_plane: int):
    """f32 partial sums of A.B stored once, through the multicast address ``mc_ptr``, into plane ``my_plane`` of every rank's buffer."""
    M, K = A.shape
    N = B.shape[1]
    check(load().gcb200_matmul_bf16_f32out_push_mc(_ptr(A), _ptr(B), _vp(mc_ptr), my_plane, M, N, K, _stream()))


def matmul_bf16_allgather_mc(A, B, bias, relu, mc_ptr: int, ldc: int):
    """This rank's column block stored through the multicast address ``mc_ptr`` (the block's first element inside the
    multicast mapping of the [M, ldc] result) into every rank's result."""
    M, K = A.shape
    N = B.shape[1]
    check(load().gcb200_matmul_bf16_allgather_mc(_ptr(A), _ptr(B), _ptr(bias), _vp(mc_ptr), M, N, K, ldc, 0, 0, int(relu), _stream()))


def matmul_u8s8_allgather_mc(A, W, scale, bias, comp, mc_ptr: int, ldc: int):
    M, K = A.shape
    N = W.shape[1]
    check(load().gcb200_matmul_u8s8_allgather_mc(_ptr(A), _ptr(W), _ptr(scale), _ptr(bias), _ptr(comp), _vp(mc_ptr), M, N, K, ldc,
                                                 0, _stream()))


def matmul_bf16_f32out_scatter(A, B, peer_ptrs, my_plane: int):
    """Row block d of the f32 partial sums of A.B goes into plane ``my_plane`` of peer d's buffer [g][M/g][N] only."""
    M, K = A.shape
    N = B.shape[1]
    arr = (_vp * len(peer_ptrs))(*peer_ptrs)
    check(load().gcb200_matmul_bf16_f32out_scatter(_ptr(A), _ptr(B), arr, len(peer_ptrs), my_plane, M, N, K, _stream()))


def matmul_bf16_allgather(A, B, bias, relu, peer_ptrs, ldc: int, transpose_a=False, transpose_b=False):
    """This rank's column block act(A.B + bias) stored by the GEMM epilogue at ``peer_ptrs[d]`` (ints: address of
    the block's first element inside rank d's [M, ldc] bf16 result) of every rank."""
    M = A.shape[1] if transpose_a else A.shape[0]
    K = A.shape[0] if transpose_a else A.shape[1]
    N = B.shape[0] if transpose_b else B.shape[1]
    arr = (_vp * len(peer_ptrs))(*peer_ptrs)
    check(load().gcb200_matmul_bf16_allgather(_ptr(A), _ptr(B), _ptr(bias), arr, len(peer_ptrs), M, N, K, ldc,
                                              int(transpose_a), int(transpose_b), int(relu), _stream()))


def matmul_u8s8_allgather(A, W, scale, bias, comp, peer_ptrs, ldc: int, transpose_b=False):
    """u8 x s8 column block, dequantised f32, stored at ``peer_ptrs[d]`` inside every rank's [M, ldc] f32 result."""
    M, K = A.shape
    N = W.shape[0] if transpose_b else W.shape[1]
    arr = (_vp * len(peer_ptrs))(*peer_ptrs)
    check(load().gcb200_matmul_u8s8_allgather(_ptr(A), _ptr(W), _ptr(scale), _ptr(bias), _ptr(comp), arr, len(peer_ptrs),
                                              M, N, K, ldc, int(transpose_b), _stream()))


def reduce_slice_broadcast_bf16(parts, bias, relu, out_ptrs, row0: int):
    """parts: this rank's f32 [g, rows, N]; the reduced bf16 rows land at row ``row0`` of every buffer in ``out_ptrs``."""
    nparts, rows, N = parts.shape
    arr = (_vp * len(out_ptrs))(*out_ptrs)
    check(load().gcb200_reduce_slice_broadcast_bf16(_ptr(parts), nparts, rows, N, _ptr(bias), arr, len(out_ptrs), row0, int(relu),
                                                    _stream()))


def reduce_bias_act_bf16(parts, bias=None, relu=False, out=None):
    """parts: f32 [nparts, M, N] contiguous."""
    import torch

    nparts, M, N = parts.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=parts.device)
    check(load().gcb200_reduce_bias_act_bf16(_ptr(parts), nparts, M * N, _ptr(bias), _ptr(out), M, N, int(relu), _stream()))
    return out


def colsum_s8(W, zp_a: int):
    import torch

    K, N = W.shape
    comp = torch.empty((N,), dtype=torch.int32, device=W.device)
    check(load().gcb200_colsum_s8(_ptr(W), _ptr(comp), K, N, zp_a, _stream()))
    return comp


def matmul_u8s8(A, W, scale=None, bias=None, comp=None, want_acc=False, transpose_b=False):
    """Returns (out f32 or None, acc s32 or None).  W is [K,N], or [N,K] when transpose_b."""
    import torch

    M, K = A.shape
    N = W.shape[0] if transpose_b else W.shape[1]
    out = torch.empty((M, N), dtype=torch.float32, device=A.device) if scale is not None else None
    acc = torch.empty((M, N), dtype=torch.int32, device=A.device) if (want_acc or out is None) else None
    check(load().gcb200_matmul_u8s8(_ptr(A), _ptr(W), _ptr(scale), _ptr(bias), _ptr(comp), _ptr(out), _ptr(acc), M, N, K,
                                    int(transpose_b), _stream()))
    return out, acc


def matmul_f32(A, B, bias=None, relu=False, transpose_a=False, transpose_b=False):
    import torch

    K, M = (A.shape if transpose_a else A.shape[::-1])
    N = B.shape[0] if transpose_b else B.shape[1]
    out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    check(load().gcb200_matmul_f32(_ptr(A), _ptr(B), _ptr(bias), _ptr(out), M, N, K, int(transpose_a), int(transpose_b),
                                   int(relu), _stream()))
    return out


def attention_bf16(Q, K, V, scale: float, causal: bool = False, out=None):
    """Fused attention on bf16 CUDA tensors [..., S, D] (leading dims are independent units)."""
    import torch

    assert Q.is_contiguous() and K.is_contiguous() and V.is_contiguous() and Q.dtype == torch.bfloat16
    S, D = Q.shape[-2:]
    bh = Q.numel() // (S * D)
    if out is None:
        out = torch.empty_like(Q)
    check(load().gcb200_attention_bf16(_ptr(Q), _ptr(K), _ptr(V), _ptr(out), bh, S, D, float(scale), int(causal), _stream()))
    return out


class TpMlpPlan:
    """Handle of a ``gcb200_tp_mlp`` plan: ``tables`` are lists of integer device addresses indexed by rank
    (``recv0, recv1, act0, act1, signals`` and optionally ``x_in``), ``weights`` / ``biases`` lists of this rank's
    shard addresses (0 / None = no bias).  Creating and describing a plan needs no device."""

    def __init__(self, world, rank, batch, hidden, weights, biases, relu, recv, act, signals, x_in=None, recv_planes=0):
        layers = len(hidden) - 1

        def table(vals):
            return (_vp * len(vals))(*[_vp(int(v)) if v else _vp(None) for v in vals])

        self._keep = [(_i64 * len(hidden))(*hidden), table(weights), table(biases), table(recv[0]), table(recv[1]),
                      table(act[0]), table(act[1]), table(signals), table(x_in) if x_in else None]
        k = self._keep
        d = TpMlpDesc()
        d.world, d.rank, d.batch, d.layers, d.relu = world, rank, batch, layers, int(relu)
        d.hidden = k[0]
        d.weights = C.cast(k[1], C.POINTER(_vp))
        d.biases = C.cast(k[2], C.POINTER(_vp))
        d.recv[0], d.recv[1] = C.cast(k[3], C.POINTER(_vp)), C.cast(k[4], C.POINTER(_vp))
        d.act[0], d.act[1] = C.cast(k[5], C.POINTER(_vp)), C.cast(k[6], C.POINTER(_vp))
        d.signals = C.cast(k[7], C.POINTER(_vp))
        d.x_in = C.cast(k[8], C.POINTER(_vp)) if x_in else C.POINTER(_vp)()
        d.recv_planes = recv_planes
        self._h = _vp(None)
        check(load().gcb200_tp_mlp_create(C.byref(d), C.byref(self._h)))

    def describe(self, sm_count: int = 148) -> str:
        need = C.c_size_t(0)
        check(load().gcb200_tp_mlp_describe(self._h, sm_count, None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        check(load().gcb200_tp_mlp_describe(self._h, sm_count, buf, need.value, None))
        return buf.value.decode()

    def step(self, x_ptr: int, stream=None) -> int:
        """Enqueues one step; returns the device address of this rank's copy of the result."""
        res = _vp(None)
        check(load().gcb200_tp_mlp_step(self._h, _vp(x_ptr), _stream() if stream is None else _vp(stream), C.byref(res)))
        return int(res.value)

    def timeline(self, x_ptr: int, stream=None) -> str:
        """One eagerly launched step with an event behind every launch: one line per kernel, microseconds first."""
        buf = C.create_string_buffer(4096)
        check(load().gcb200_tp_mlp_timeline(self._h, _vp(x_ptr), _stream() if stream is None else _vp(stream), buf, 4096, None))
        return buf.value.decode()

    def trace(self) -> str:
        """Device-side time stamps of the most recent step (needs GC_B200_TP_TRACE=1 before the first step)."""
        buf = C.create_string_buffer(4096)
        check(load().gcb200_tp_mlp_trace(self._h, buf, 4096, None))
        return buf.value.decode()

    def execute(self, x_host_ptr: int, y_host_ptr: int = 0):
        check(load().gcb200_tp_mlp_execute(self._h, _vp(x_host_ptr), _vp(y_host_ptr) if y_host_ptr else _vp(None)))

    def destroy(self):
        if self._h:
            load().gcb200_tp_mlp_destroy(self._h)
            self._h = _vp(None)

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def wait_selftest(limit_cycles: int = 1_000_000):
    """Launches the failure-path self-test kernel (a bounded wait nothing satisfies) on the current stream."""
    check(load().gcb200_wait_selftest(limit_cycles, _stream()))
