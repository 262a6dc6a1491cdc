"""CPU oracle for the KDA forward pass: TEST INFRASTRUCTURE ONLY.

Python front of ``oracle/kda_oracle.c`` (a plain-C restatement of the reference's
``tests/torch_ref.py:124-251``).  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import this package; the shipped library never
does.  The shared object is built with ``make -C oracle`` (``build()`` below does
that on demand).
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libkda_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``kda_oracle.c`` with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "kda_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libkda_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.kda_oracle_fwd.restype = ctypes.c_int
        _lib.kda_oracle_fwd.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p,
                                                                 ctypes.c_void_p, ctypes.c_double, ctypes.c_void_p,
                                                                 ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p] + \
                                        [ctypes.c_int64] * 4 + [ctypes.c_int]
        _lib.kda_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return _load().kda_oracle_num_threads()


def _cpu(t, dtype):
    if t is None:
        return None
    assert t.dtype == dtype, f"expected {dtype}, got {t.dtype}"
    return t.detach().to("cpu").contiguous()


def fwd(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
        cu_seqlens=None, n_threads: int = 0):
    """Same signature and in-place semantics as ``flash_kda.fwd`` (reference
    ``flash_kda/__init__.py:5``), evaluated on the host.  ``out`` and ``final_state``
    must be CPU tensors (they are written in place)."""
    lib = _load()
    bf = torch.bfloat16
    q, k, v, g, beta = (_cpu(t, bf) for t in (q, k, v, g, beta))
    A_log, dt_bias = _cpu(A_log, torch.float32), _cpu(dt_bias, torch.float32)
    assert out.device.type == "cpu" and out.is_contiguous() and out.dtype == bf
    B, T, H, Dd = q.shape
    assert Dd == 128
    state_dtype = 0
    for s in (initial_state, final_state):
        if s is not None and s.dtype == torch.float32:
            state_dtype = 1
    if initial_state is not None:
        initial_state = initial_state.detach().to("cpu").contiguous()
    if final_state is not None:
        assert final_state.device.type == "cpu" and final_state.is_contiguous()
    if cu_seqlens is not None:
        cu = cu_seqlens.detach().to("cpu", torch.int64).contiguous()
        N = cu.numel() - 1
    else:
        cu, N = None, B
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    rc = lib.kda_oracle_fwd(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), float(scale), ptr(out), ptr(A_log),
                            ptr(dt_bias), float(lower_bound), ptr(initial_state), ptr(final_state), state_dtype,
                            ptr(cu), B, T, H, N, int(n_threads))
    if rc != 0:
        raise RuntimeError(f"kda_oracle_fwd failed with status {rc}")


def err_ratio(x, y) -> float:
    """RMSE(x - y) / RMS(x): the reference's relative-error metric (tests/test_fwd.py:13-16)."""
    x, y = x.detach().double().flatten(), y.detach().double().flatten()
    err = (x - y).square().mean().sqrt().item()
    base = x.square().mean().sqrt().item()
    return err / (base + 1e-8)


def max_abs(x, y) -> float:
    return (x.detach().double() - y.detach().double()).abs().max().item() if x.numel() else 0.0
