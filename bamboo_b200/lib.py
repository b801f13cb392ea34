"""ctypes binding of libbamboo_b200.so (the C ABI declared in include/bamboo_b200.h).

There is no Python or CPU fallback behind these calls: if the shared library is missing
or a call fails, an exception is raised.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbamboo_b200.so")

EPI_STORE, EPI_BIAS, EPI_BIAS_GELU, EPI_ACCUM_F32, EPI_STORE_F32, EPI_MUL_DGELU, EPI_BIAS_RESIDUAL = range(7)


class BambooNativeError(RuntimeError):
    """A native entry point returned a negative status."""


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("A", ctypes.c_void_p), ("lda", ctypes.c_longlong), ("a_mn_major", ctypes.c_int),
        ("B", ctypes.c_void_p), ("ldb", ctypes.c_longlong), ("b_mn_major", ctypes.c_int),
        ("D", ctypes.c_void_p), ("ldd", ctypes.c_longlong),
        ("epilogue", ctypes.c_int),
        ("bias", ctypes.c_void_p),
        ("D2", ctypes.c_void_p),
        ("aux", ctypes.c_void_p), ("ld_aux", ctypes.c_longlong),
        ("tile_n", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
    ]


_lib = None
_lock = threading.Lock()


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise BambooNativeError(
                f"{LIB_PATH} is missing: build it with `python -m bamboo_b200.csrc.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(LIB_PATH)
        lib.bb_last_error.restype = ctypes.c_char_p
        lib.bb_version.restype = ctypes.c_int
        _lib = lib
    return _lib


def check(rc, what=""):
    if rc < 0:
        msg = load().bb_last_error().decode(errors="replace")
        raise BambooNativeError(f"{what} failed with status {rc}: {msg}")
    return rc


def read_status():
    """Synchronously read-and-clear the device status word (0 = healthy)."""
    out = ctypes.c_int(0)
    check(load().bb_read_status(ctypes.byref(out)), "bb_read_status")
    return out.value


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def gemm(a, b, out, *, a_mn=False, b_mn=False, epilogue=EPI_STORE, bias=None, out2=None, aux=None,
         M=None, N=None, K=None, tile_n=0, max_ctas=0):
    """out[M,N] = op(a)[M,K] @ op(b)[N,K]^T with a fused epilogue; see bb_gemm_bf16.

    ``a`` is [M,K] (or [K,M] when ``a_mn``), ``b`` is [N,K] (or [K,N] when ``b_mn``); 2-D,
    unit inner stride, bf16, on the current CUDA device.
    """
    if M is None:
        M = a.shape[1] if a_mn else a.shape[0]
    if K is None:
        K = a.shape[0] if a_mn else a.shape[1]
    if N is None:
        N = b.shape[1] if b_mn else b.shape[0]
    for t in (a, b, out, bias, out2, aux):
        if t is not None and (not t.is_cuda or t.stride(-1) != 1):
            raise BambooNativeError("gemm operands must be CUDA tensors with unit inner stride")
    d = GemmDesc(M=M, N=N, K=K, A=_ptr(a), lda=a.stride(0), a_mn_major=int(a_mn),
                 B=_ptr(b), ldb=b.stride(0), b_mn_major=int(b_mn), D=_ptr(out), ldd=out.stride(0),
                 epilogue=epilogue, bias=_ptr(bias), D2=_ptr(out2), aux=_ptr(aux),
                 ld_aux=aux.stride(0) if aux is not None else 0, tile_n=tile_n, max_ctas=max_ctas)
    check(load().bb_gemm_bf16(ctypes.byref(d), _stream()), "bb_gemm_bf16")
    return out
