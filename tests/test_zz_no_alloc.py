"""fkda_fwd_noalloc: the entry point for callers that cannot allocate device memory.

Collected last on purpose (file name): it shares one built-in scratch array per GPU with nothing
else in the suite, and a failure here must not hide the results of the other tests.

What it checks: called through the C ABI with inputs and outputs only (no workspace), twice in a
row, the entry point reproduces the output of the ordinary fkda_fwd (which uses a caller-provided
workspace) exactly -- both run the same kernels, so the comparison is bit for bit, well inside the
suite's tolerances -- and it refuses problems that do not fit its fixed scratch.
"""
import ctypes

import pytest
import torch

import flashkda_b200
from flashkda_b200 import _lib
from flashkda_b200.synth import Workload, make_inputs, to_device


def _params(d, algo):
    q = d["q"]
    B, T, H, _ = q.shape
    N = d["cu_seqlens"].numel() - 1 if d["cu_seqlens"] is not None else B
    ptr = lambda t: None if t is None else t.data_ptr()
    fp32 = any(s is not None and s.dtype == torch.float32 for s in (d["initial_state"], d["final_state"]))
    return _lib.FwdParams(
        q=ptr(q), k=ptr(d["k"]), v=ptr(d["v"]), g=ptr(d["g"]), beta=ptr(d["beta"]), out=ptr(d["out"]),
        A_log=ptr(d["A_log"]), dt_bias=ptr(d["dt_bias"]), initial_state=ptr(d["initial_state"]),
        final_state=ptr(d["final_state"]), state_dtype=1 if fp32 else 0, algo=_lib.ALGOS[algo],
        cu_seqlens=ptr(d["cu_seqlens"]), B=B, T=T, H=H, N=N, token_stride=H * 128, beta_token_stride=H,
        scale=float(d["scale"]), lower_bound=float(d["lower_bound"]), workspace=None, workspace_bytes=0)


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["tc", "twopass"])
def test_noalloc_matches_regular_entry_point_twice(algo):
    L = _lib.lib()
    w = Workload("na", 1, 700, 4, state_in="fp32", state_out="fp32", seq_lens=[300, 1, 143, 256])
    inp = make_inputs(w, seed=21)
    # reference result: the ordinary entry point with an allocated workspace
    ref = to_device(inp, "cuda")
    flashkda_b200.fwd(ref["q"], ref["k"], ref["v"], ref["g"], ref["beta"], ref["scale"], ref["out"],
                      A_log=ref["A_log"], dt_bias=ref["dt_bias"], lower_bound=ref["lower_bound"],
                      initial_state=ref["initial_state"], final_state=ref["final_state"],
                      cu_seqlens=ref["cu_seqlens"], algo=algo)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # the second call reuses the scratch the first one left behind
        d = to_device(inp, "cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]   # the driver's count of free device memory (cudaMemGetInfo)
        rc = L.fkda_fwd_noalloc(_params(d, algo), stream)
        assert rc == 0, _lib.status_string(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call == 1:  # (a first call may make the driver load kernel code; the second finds everything in place)
            assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was taken during the call"
        assert L.fkda_device_status(None, stream) == 0   # NULL = the built-in scratch
        assert torch.equal(d["out"], ref["out"]), f"call {call}: out differs"
        assert torch.equal(d["final_state"], ref["final_state"]), f"call {call}: final_state differs"


@pytest.mark.gpu
def test_noalloc_decode_step_of_a_large_batch():
    """A decode step keeps no per-chunk records, so it fits the built-in scratch whatever the batch size."""
    L = _lib.lib()
    w = Workload("nadec", 640, 1, 16, state_in="bf16", state_out="bf16", lower_bound=-1.0)
    inp = make_inputs(w, seed=5)
    ref = to_device(inp, "cuda")
    flashkda_b200.fwd(ref["q"], ref["k"], ref["v"], ref["g"], ref["beta"], ref["scale"], ref["out"],
                      A_log=ref["A_log"], dt_bias=ref["dt_bias"], lower_bound=ref["lower_bound"],
                      initial_state=ref["initial_state"], final_state=ref["final_state"])
    d = to_device(inp, "cuda")
    rc = L.fkda_fwd_noalloc(_params(d, "tc"), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert torch.equal(d["out"], ref["out"]) and torch.equal(d["final_state"], ref["final_state"])


@pytest.mark.gpu
def test_noalloc_rejects_problems_beyond_its_scratch():
    L = _lib.lib()
    w = Workload("big", 1, 16 * 4000, 1)  # 4000 chunk records > the built-in limit
    assert flashkda_b200.get_workspace_size(w.tokens, w.H, 1, algo="tc") > L.fkda_noalloc_scratch_bytes()
    d = to_device(make_inputs(w), "cuda")
    d["out"].fill_(7.0)
    rc = L.fkda_fwd_noalloc(_params(d, "tc"), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 10 and "too large" in _lib.status_string(rc)
    assert bool((d["out"] == 7.0).all()), "nothing may be launched when the problem is refused"


def test_noalloc_symbols_and_limit_without_gpu():
    L = _lib.lib()
    assert L.fkda_noalloc_scratch_bytes() == 32 * 1024 * 1024
    assert L.fkda_fwd_noalloc(None, None) == 1
    p = _lib.FwdParams(B=1, T=16 * 100000, H=8, N=1, algo=_lib.ALGOS["tc"])
    assert L.fkda_fwd_noalloc(p, None) == 10
