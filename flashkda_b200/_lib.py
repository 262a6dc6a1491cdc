"""ctypes binding of the C ABI declared in include/flashkda_b200.h."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libflashkda_b200.so")

FKDA_STATE_BF16, FKDA_STATE_FP32 = 0, 1
ALGO_AUTO, ALGO_TWOPASS, ALGO_TC = 0, 1, 2
PHASE_PREPARE, PHASE_RECURRENCE = 1, 2
# fkda_fwd_params.flags (tests and tuning; 0 in production)
FLAG_NO_DECODE, FLAG_NO_WIDE, FLAG_NO_SLABS, FLAG_NO_SHORT, FLAG_TEST_DROP_PUSH = 1, 2, 4, 8, 16


def flags_seg_chunks(n: int) -> int:
    return (int(n) & 0xff) << 8


def flags_wait_ms(ms: int) -> int:
    return (int(ms) & 0x3fff) << 16
ALGOS = {"auto": ALGO_AUTO, "twopass": ALGO_TWOPASS, "tc": ALGO_TC}


class FwdParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("g", ctypes.c_void_p),
        ("beta", ctypes.c_void_p), ("out", ctypes.c_void_p), ("A_log", ctypes.c_void_p),
        ("dt_bias", ctypes.c_void_p), ("initial_state", ctypes.c_void_p), ("final_state", ctypes.c_void_p),
        ("state_dtype", ctypes.c_int32), ("algo", ctypes.c_int32), ("cu_seqlens", ctypes.c_void_p),
        ("B", ctypes.c_int64), ("T", ctypes.c_int64), ("H", ctypes.c_int64), ("N", ctypes.c_int64),
        ("token_stride", ctypes.c_int64), ("beta_token_stride", ctypes.c_int64),
        ("scale", ctypes.c_float), ("lower_bound", ctypes.c_double),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("phase_mask", ctypes.c_int32), ("flags", ctypes.c_int32),
        ("chunk_states", ctypes.c_void_p), ("chunk_states_every", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


_lib = None


def lib():
    """Loads the CUDA library; there is no fallback implementation, so a missing build is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flashkda_b200.build` "
                "(flashkda_b200 has no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        L.fkda_params_size.restype = ctypes.c_size_t
        if L.fkda_params_size() != ctypes.sizeof(FwdParams):
            raise RuntimeError(f"{LIB_PATH} was built from another revision of include/flashkda_b200.h "
                               f"(struct of {L.fkda_params_size()} bytes, binding has {ctypes.sizeof(FwdParams)}): rebuild it")
        L.fkda_fwd.restype = ctypes.c_int
        L.fkda_fwd.argtypes = [ctypes.POINTER(FwdParams), ctypes.c_void_p]
        L.fkda_workspace_bytes.restype = ctypes.c_size_t
        L.fkda_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32]
        L.fkda_workspace_bytes_for.restype = ctypes.c_size_t
        L.fkda_workspace_bytes_for.argtypes = [ctypes.POINTER(FwdParams)]
        L.fkda_version.restype = ctypes.c_int
        L.fkda_status_string.restype = ctypes.c_char_p
        L.fkda_status_string.argtypes = [ctypes.c_int]
        L.fkda_last_launch_count.restype = ctypes.c_int
        L.fkda_fwd_noalloc.restype = ctypes.c_int
        L.fkda_fwd_noalloc.argtypes = [ctypes.POINTER(FwdParams), ctypes.c_void_p]
        L.fkda_noalloc_scratch_bytes.restype = ctypes.c_size_t
        L.fkda_device_status.restype = ctypes.c_int
        L.fkda_device_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.fkda_cp_fold.restype = ctypes.c_int
        L.fkda_cp_fold.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_void_p]
        _lib = L
    return _lib


def status_string(rc: int) -> str:
    return lib().fkda_status_string(rc).decode()
