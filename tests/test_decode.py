"""Decode step (one token per sequence, fixed batch): the dedicated state read-modify-write kernel
against the CPU oracle and against the general chunked kernels on the same inputs.

Tolerances as in test_gpu_parity.py.  Against the general GPU path the results differ only by the
fp32 summation order of the 128-long dot products (warp shuffles here, tensor core / FMA chains
there), which flips a small fraction of bf16 roundings.
"""
import pytest
import torch

import flashkda_b200
import oracle
from flashkda_b200 import _lib
from flashkda_b200.synth import Workload, make_inputs
from kda_testlib import run_oracle
from test_gpu_parity import check_against, run_gpu

pytestmark = pytest.mark.gpu

STATE_IO = [("in+out", True, True), ("in_only", True, False), ("out_only", False, True), ("none", False, False)]


@pytest.mark.parametrize("B,H", [(1, 1), (3, 4), (64, 8)])
@pytest.mark.parametrize("state_dtype", ["bf16", "fp32"])
@pytest.mark.parametrize("io", STATE_IO, ids=[s[0] for s in STATE_IO])
def test_decode_step_matches_oracle(B, H, state_dtype, io):
    _, has_in, has_out = io
    w = Workload("dec", B, 1, H, state_in=state_dtype if has_in else None, state_out=state_dtype if has_out else None,
                 lower_bound=-2.0)
    inp = make_inputs(w, seed=100 + B + H)
    ref_out, ref_hT = run_oracle(inp)
    out, hT = run_gpu(inp, "tc")
    assert flashkda_b200.last_launch_count() == 1, "one token per sequence must take the one-kernel decode path"
    check_against(out, hT, ref_out, ref_hT)


def test_decode_kernel_matches_general_path():
    w = Workload("decg", 96, 1, 16, state_in="fp32", state_out="fp32", lower_bound=-1.0)
    inp = make_inputs(w, seed=7)
    out_d, hT_d = run_gpu(inp, "tc")
    assert flashkda_b200.last_launch_count() == 1
    out_g, hT_g = run_gpu(inp, "tc", flags=_lib.FLAG_NO_DECODE)
    assert flashkda_b200.last_launch_count() == 2  # prepare + recurrence
    out_c, hT_c = run_gpu(inp, "twopass")
    mism = (out_d != out_g).float().mean().item()
    print(f"decode kernel vs chunked tensor-core path: out mismatch {mism:.3e}, state ratio {oracle.err_ratio(hT_g, hT_d):.3e}")
    for o, s in ((out_g, hT_g), (out_c, hT_c)):
        assert oracle.err_ratio(o, out_d) <= 2e-3
        assert oracle.err_ratio(s, hT_d) <= 1e-3
    assert mism <= 0.05


def test_decode_loop_carries_state():
    """A decode loop feeds the final state of one step back as the initial state of the next.  Doing that in
    place (one buffer as both arguments) must equal doing it through a fresh buffer per step."""
    B, H, steps = 5, 4, 8
    gen = torch.Generator().manual_seed(3)
    state_a = (torch.randn(B, H, 128, 128, generator=gen) * 0.05).cuda()
    state_b = state_a.clone()
    ws = torch.empty(flashkda_b200.get_workspace_size(B, H, B), dtype=torch.uint8, device="cuda")
    for s in range(steps):
        inp = make_inputs(Workload("decl", B, 1, H, lower_bound=-0.5), seed=200 + s)
        d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
        out_a, out_b = torch.zeros_like(d["v"]), torch.zeros_like(d["v"])
        kw = dict(A_log=d["A_log"], dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], workspace=ws)
        flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], out_a, initial_state=state_a,
                          final_state=state_a, **kw)                       # in place
        nxt = torch.empty_like(state_b)
        flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], out_b, initial_state=state_b,
                          final_state=nxt, **kw)                           # through a copy
        state_b = nxt
        assert torch.equal(out_a, out_b)
    assert torch.equal(state_a, state_b)
    assert torch.isfinite(state_a).all()
