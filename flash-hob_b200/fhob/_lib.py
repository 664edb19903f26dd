"""ctypes binding of libfhob.so (declarations mirror include/fhob.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libfhob.so"

FHOB_BF16, FHOB_F32, FHOB_F16 = 0, 1, 2
DTYPES = {"torch.bfloat16": FHOB_BF16, "torch.float32": FHOB_F32, "torch.float16": FHOB_F16}
IMPL = {"auto": 0, "simt": 1, "tcgen05": 2}
ERR_TIMEOUT, ERR_SMEM_ALIGN = 64, 128

# every symbol include/fhob.h declares
SYMBOLS = (
    "fhob_version", "fhob_strerror", "fhob_last_cuda_error", "fhob_workspace_bytes", "fhob_bwdbwd",
    "fhob_prepass", "fhob_pass1", "fhob_pass2", "fhob_pass12", "fhob_pass3", "fhob_pass4", "fhob_row_stats",
    "fhob_read_status", "fhob_forward", "fhob_backward", "fhob_bwdbwd_static_scratch",
    "fhob_selftest_expired_wait", "fhob_visible_tiles", "fhob_static_scratch_status",
    "fhob_workspace_bytes_problem",
)
STATIC_SCRATCH_MAX_ROWS = 262144


class FhobLayout(C.Structure):
    """Element strides of q, k, v, o, d_o, ddq, ddk, ddv (rows / heads of a batch entry / batch entries) and of lse."""
    _fields_ = [
        ("heads", C.c_int32), ("reserved", C.c_int32),
        ("row", C.c_int64 * 8), ("head", C.c_int64 * 8), ("batch", C.c_int64 * 8),
        ("lse_head", C.c_int64), ("lse_batch", C.c_int64),
    ]


class FhobProblem(C.Structure):
    _fields_ = [
        ("bh", C.c_int32), ("n_q", C.c_int32), ("n_k", C.c_int32), ("d", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("impl", C.c_int32), ("scale", C.c_float),
        ("window", C.c_int32), ("d_v", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
        ("ddq", C.c_void_p), ("ddk", C.c_void_p), ("ddv", C.c_void_p), ("lse", C.c_void_p),
        ("dq2", C.c_void_p), ("dk2", C.c_void_p), ("dv2", C.c_void_p), ("ddo", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("layout", C.POINTER(FhobLayout)),
    ]


_lib = None


def load() -> C.CDLL:
    """Loads the library once.  There is no fallback: a missing build is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python flash-hob_b200/build.py` "
            "(nvcc, sm_100a). The operator has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    P = C.POINTER(FhobProblem)
    lib.fhob_version.restype = C.c_int
    lib.fhob_strerror.restype = C.c_char_p
    lib.fhob_strerror.argtypes = [C.c_int]
    lib.fhob_last_cuda_error.restype = C.c_char_p
    lib.fhob_workspace_bytes.restype = C.c_size_t
    lib.fhob_workspace_bytes.argtypes = [C.c_int32, C.c_int32]
    lib.fhob_workspace_bytes_problem.restype = C.c_size_t
    lib.fhob_workspace_bytes_problem.argtypes = [P]
    for name in ("fhob_bwdbwd", "fhob_prepass", "fhob_pass1", "fhob_pass2", "fhob_pass12", "fhob_pass3", "fhob_pass4",
                 "fhob_read_status", "fhob_bwdbwd_static_scratch"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [P, C.c_void_p]
    lib.fhob_row_stats.restype = C.c_int
    lib.fhob_row_stats.argtypes = [P, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.fhob_backward.restype = C.c_int
    lib.fhob_backward.argtypes = [P, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.fhob_visible_tiles.restype = C.c_int
    lib.fhob_visible_tiles.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.fhob_selftest_expired_wait.restype = C.c_int
    lib.fhob_selftest_expired_wait.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fhob_static_scratch_status.restype = C.c_int
    lib.fhob_static_scratch_status.argtypes = [C.c_void_p]
    lib.fhob_forward.restype = C.c_int
    lib.fhob_forward.argtypes = [P, C.c_void_p, C.c_void_p, C.c_void_p]
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.fhob_strerror(status).decode()
    if status == 5:
        msg += ": " + lib.fhob_last_cuda_error().decode()
    raise RuntimeError(f"{what} failed with status {status}: {msg}")
