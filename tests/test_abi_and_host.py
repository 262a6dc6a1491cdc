"""CPU-side checks: the C-ABI library loads and exports what include/*.h declares, and the
host-side operator mirrors the reference's argument checks (csrc/flash_kda.cpp:44-174)."""
import ctypes
import glob
import os
import re

import pytest
import torch

import flashkda_b200
from flashkda_b200 import _lib
from flashkda_b200.synth import Workload, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for hdr in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(hdr).read(), flags=re.S)
        names += re.findall(r"\b(fkda_[a-z_0-9]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_functions()
    assert {"fkda_fwd", "fkda_workspace_bytes", "fkda_version", "fkda_status_string"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"


def test_version_status_and_workspace_size():
    L = _lib.lib()
    assert L.fkda_version() >= 1001
    assert _lib.status_string(0) == "ok"
    assert "NULL" in _lib.status_string(1)
    # same growth law as the reference's get_workspace_size: 13824 B per (head, chunk) record
    a = flashkda_b200.get_workspace_size(8192, 96, 1, algo="twopass")
    b = flashkda_b200.get_workspace_size(8192 + 16, 96, 1, algo="twopass")
    assert b - a == 96 * 13824
    assert flashkda_b200.get_workspace_size(0, 4, 1, algo="twopass") >= 4 * 13824


def test_params_struct_matches_header_layout():
    # 13 pointers/ints of 8 bytes before B..., natural alignment: guards against silent drift
    assert ctypes.sizeof(_lib.FwdParams) == 10 * 8 + 2 * 4 + 8 + 6 * 8 + 4 + 4 + 8 + 8 + 8 + 8 + 8 + 4 + 4
    assert _lib.lib().fkda_params_size() == ctypes.sizeof(_lib.FwdParams)


def test_null_and_shape_errors_without_gpu():
    L = _lib.lib()
    assert L.fkda_fwd(None, None) == 1
    p = _lib.FwdParams(B=0, T=16, H=1, N=1)
    assert L.fkda_fwd(p, None) == 2
    p = _lib.FwdParams(B=1, T=16, H=1, N=1, token_stride=128, beta_token_stride=1, state_dtype=7)
    assert L.fkda_fwd(p, None) == 3
    p = _lib.FwdParams(B=2, T=16, H=1, N=1, token_stride=128, beta_token_stride=1, cu_seqlens=0x1000)
    assert L.fkda_fwd(p, None) == 4
    p = _lib.FwdParams(B=1, T=16, H=1, N=1, token_stride=128, beta_token_stride=1)
    assert L.fkda_fwd(p, None) == 1  # A_log / dt_bias missing


def test_host_checks_reject_cpu_tensors():
    inp = make_inputs(Workload("x", 1, 16, 1))
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        flashkda_b200.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                          A_log=inp["A_log"], dt_bias=inp["dt_bias"], lower_bound=-5.0)


def test_drop_in_module_name():
    import importlib.util
    assert importlib.util.find_spec("flash_kda") is not None
    import flash_kda
    assert flash_kda.fwd is flashkda_b200.fwd
    import inspect
    params = list(inspect.signature(flash_kda.fwd).parameters)
    assert params[:13] == ["q", "k", "v", "g", "beta", "scale", "out", "A_log", "dt_bias", "lower_bound",
                           "initial_state", "final_state", "cu_seqlens"]
