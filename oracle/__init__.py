"""CPU oracle — TEST INFRASTRUCTURE, not part of the product.

ctypes bindings over ``liboracle.so`` (the scalar restatement in
``oracle.cpp``) and, when present, ``_ref/libgc_brgemm_naive.so`` (the
reference's own ``BrgemmNaive.cpp`` compiled unmodified by ``oracle/Makefile``).

Only the test-suite, the smoke test and the benchmark's CPU-baseline leg import
this module.  bf16 tensors travel as ``numpy.uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libgc_brgemm_naive.so")

# dnnl_data_type_t codes of the brgemm ABI
DT_F16, DT_BF16, DT_F32, DT_S32, DT_S8, DT_U8 = 1, 2, 3, 4, 5, 6

_i64, _u64, _f32, _int, _vp = C.c_int64, C.c_uint64, C.c_float, C.c_int, C.c_void_p

DISPATCH_FN = C.CFUNCTYPE(_i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _i64, _i64)
EXECUTE_FN = C.CFUNCTYPE(None, _i64, _vp, _u64, _vp, _u64, _vp, _u64, _int)


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference microkernel when its tree is present)."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(
        os.path.join(_HERE, "oracle.cpp")
    ):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    if force or not os.path.exists(_REF):
        subprocess.check_call(["make", "-C", _HERE, "ref"], stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB)
        _lib.gco_f32_to_bf16.restype = C.c_uint16
        _lib.gco_f32_to_bf16.argtypes = [_f32]
        _lib.gco_bf16_to_f32.restype = _f32
        _lib.gco_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.gco_brgemm.restype = _int
        _lib.gco_brgemm.argtypes = [_i64] * 8 + [_f32, _i64, _i64, _vp, _u64, _vp, _u64, _vp, _u64, _int]
        _lib.gco_brgemm_dispatch.restype = _i64
        _lib.gco_brgemm_dispatch.argtypes = [_i64] * 8 + [_f32, _i64, _i64]
        _lib.gco_brgemm_execute.restype = None
        _lib.gco_brgemm_execute.argtypes = [_i64, _vp, _u64, _vp, _u64, _vp, _u64, _int]
        _lib.gco_num_threads.restype = _int
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF)


def ref():
    """The reference's naive brgemm (dnnl_brgemm_dispatch / dnnl_brgemm_execute)."""
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(_REF)
        _ref = C.CDLL(_REF)
        _ref.dnnl_brgemm_dispatch.restype = _i64
        _ref.dnnl_brgemm_dispatch.argtypes = [_i64] * 8 + [_f32, _i64, _i64]
        _ref.dnnl_brgemm_execute.restype = None
        _ref.dnnl_brgemm_execute.argtypes = [_i64, _vp, _u64, _vp, _u64, _vp, _u64, _int]
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


# --------------------------------------------------------------------------- scalars
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().gco_f32_to_bf16_array(_p(x), _p(out), _i64(x.size))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- brgemm
def brgemm(M, N, K, LDA, LDB, LDC, stride_a, stride_b, beta, dtA, dtB, A, A_off, B, B_off, Cbuf, C_off, num,
           backend: str = "port"):
    """Run one brgemm call in place on ``Cbuf``; backend 'port' (restatement) or 'ref'."""
    if backend == "ref":
        r = ref()
        h = r.dnnl_brgemm_dispatch(M, N, K, LDA, LDB, LDC, stride_a, stride_b, beta, dtA, dtB)
        r.dnnl_brgemm_execute(h, _p(A), A_off, _p(B), B_off, _p(Cbuf), C_off, num)
        return 0
    return lib().gco_brgemm(M, N, K, LDA, LDB, LDC, stride_a, stride_b, beta, dtA, dtB, _p(A), A_off, _p(B), B_off,
                            _p(Cbuf), C_off, num)


def pack_vnni(W: np.ndarray, v: int) -> np.ndarray:
    """[K,N] row-major -> VNNI [ceil(K/v), N, v]."""
    W = np.ascontiguousarray(W)
    K, N = W.shape
    out = np.empty(((K + v - 1) // v, N, v), W.dtype)
    lib().gco_pack_vnni(_p(W), _p(out), _i64(K), _i64(N), _i64(N), _int(W.itemsize), _int(v))
    return out


# --------------------------------------------------------------------------- layers
def linear_bf16(A, W, bias=None, relu=False, transA=False, transB=False, return_acc=False):
    """bf16 linear layer; A, W, bias are uint16 bf16 bit patterns.  Returns uint16 [M,N]."""
    A, W, bias = _c(A, np.uint16), _c(W, np.uint16), _c(bias, np.uint16)
    K, M = (A.shape if transA else A.shape[::-1])
    N = W.shape[0] if transB else W.shape[1]
    assert (W.shape[1] if transB else W.shape[0]) == K
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if return_acc else None
    lib().gco_linear_bf16(_p(A), _p(W), _p(bias), _p(Y), _i64(M), _i64(N), _i64(K), _int(transA), _int(transB),
                          _int(relu), _p(acc))
    return (Y, acc) if return_acc else Y


def linear_bf16_brgemm_nest(A, W, bias=None, relu=False, backend="port", return_acc=False):
    """Same layer computed block by block through the brgemm runtime ABI."""
    A, W, bias = _c(A, np.uint16), _c(W, np.uint16), _c(bias, np.uint16)
    M, K = A.shape
    N = W.shape[1]
    Y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if return_acc else None
    d, e = _backend_fns(backend)
    rc = lib().gco_linear_bf16_brgemm_nest(d, e, _p(A), _p(W), _p(bias), _p(Y), _i64(M), _i64(N), _i64(K),
                                           _int(relu), _p(acc))
    assert rc == 0
    return (Y, acc) if return_acc else Y


def _backend_fns(backend):
    if backend == "ref":
        r = ref()
        return C.cast(r.dnnl_brgemm_dispatch, _vp), C.cast(r.dnnl_brgemm_execute, _vp)
    l = lib()
    return C.cast(l.gco_brgemm_dispatch, _vp), C.cast(l.gco_brgemm_execute, _vp)


def reduce_epilogue_bf16(parts, bias=None, relu=False):
    parts = _c(parts, np.float32)
    nparts, M, N = parts.shape
    bias = _c(bias, np.uint16)
    Y = np.empty((M, N), np.uint16)
    lib().gco_reduce_epilogue_bf16(_p(parts), _int(nparts), _p(bias), _p(Y), _i64(M), _i64(N), _int(relu))
    return Y


def matmul_f32(A, B, bias=None, relu=False, transA=False, transB=False):
    A, B, bias = _c(A, np.float32), _c(B, np.float32), _c(bias, np.float32)
    K, M = (A.shape if transA else A.shape[::-1])
    N = B.shape[0] if transB else B.shape[1]
    Y = np.empty((M, N), np.float32)
    lib().gco_matmul_f32(_p(A), _p(B), _p(bias), _p(Y), _i64(M), _i64(N), _i64(K), _int(transA), _int(transB),
                         _int(relu))
    return Y


def linear_u8s8(A, W, scale=None, bias=None, zp_a=0, want_acc=True, want_out=True):
    """Returns (acc s32 [M,N] or None, out f32 [M,N] or None)."""
    A, W = _c(A, np.uint8), _c(W, np.int8)
    scale, bias = _c(scale, np.float32), _c(bias, np.float32)
    M, K = A.shape
    N = W.shape[1]
    acc = np.empty((M, N), np.int32) if want_acc else None
    out = np.empty((M, N), np.float32) if (want_out and scale is not None) else None
    lib().gco_linear_u8s8(_p(A), _p(W), _p(scale), _p(bias), C.c_int32(zp_a), _i64(M), _i64(N), _i64(K), _p(acc),
                          _p(out))
    return acc, out


def linear_u8s8_brgemm_nest(A, W, backend="port"):
    A, W = _c(A, np.uint8), _c(W, np.int8)
    M, K = A.shape
    N = W.shape[1]
    acc = np.empty((M, N), np.int32)
    d, e = _backend_fns(backend)
    rc = lib().gco_linear_u8s8_brgemm_nest(d, e, _p(A), _p(W), _i64(M), _i64(N), _i64(K), _p(acc))
    assert rc == 0
    return acc


def softmax_f32(X):
    X = _c(X, np.float32)
    Y = np.empty_like(X)
    lib().gco_softmax_f32(_p(X), _p(Y), _i64(X.shape[0]), _i64(X.shape[1]))
    return Y


def attention_bf16(Q, K, V, scale, causal=False):
    """Q,K,V: uint16 [..., S, D]; returns uint16 of the same shape."""
    Q, K, V = _c(Q, np.uint16), _c(K, np.uint16), _c(V, np.uint16)
    S, D = Q.shape[-2:]
    BH = Q.size // (S * D)
    O = np.empty_like(Q)
    lib().gco_attention_bf16(_p(Q), _p(K), _p(V), _p(O), _i64(BH), _i64(S), _i64(D), _f32(scale), _int(causal))
    return O


def mlp_bf16(X, weights, biases, relu=True):
    """Chained layers: the bf16 output of layer i is the A operand of layer i+1
    (test/dnnl/resources/mpl.json; test/benchgc/src/benchgc/pattern/mlp.py:113-150)."""
    h = X
    for W, b in zip(weights, biases):
        h = linear_bf16(h, W, b, relu=relu)
    return h


def num_threads() -> int:
    return lib().gco_num_threads()


def set_num_threads(n: int) -> None:
    lib().gco_set_num_threads(_int(n))
