"""Fixed batches of short sequences (2 .. 16 tokens each, one chunk per sequence): the fused one-kernel path
against the general chunked kernels on the same inputs (same numerics: bit for bit) and against the CPU oracle.
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


@pytest.mark.parametrize("T", [2, 3, 4, 7, 8, 15, 16])
@pytest.mark.parametrize("state_dtype", ["bf16", "fp32"])
@pytest.mark.parametrize("io", STATE_IO, ids=[s[0] for s in STATE_IO])
def test_short_batch_matches_general_path_and_oracle(T, state_dtype, io):
    _, has_in, has_out = io
    w = Workload("short", 5, T, 3, state_in=state_dtype if has_in else None, state_out=state_dtype if has_out else None,
                 lower_bound=-2.0)
    inp = make_inputs(w, seed=50 + T)
    out_s, hT_s = run_gpu(inp, "tc")
    assert flashkda_b200.last_launch_count() == 1, "2..16 tokens per sequence must take the one-kernel path"
    out_g, hT_g = run_gpu(inp, "tc", flags=_lib.FLAG_NO_SHORT)
    assert flashkda_b200.last_launch_count() == 2
    assert torch.equal(out_s, out_g)
    if has_out:
        assert torch.equal(hT_s, hT_g)
    ref_out, ref_hT = run_oracle(inp)
    check_against(out_s, hT_s, ref_out, ref_hT)


def test_short_batch_many_chains():
    w = Workload("shortmany", 96, 16, 16, state_in="bf16", state_out="bf16", lower_bound=-1.0)
    inp = make_inputs(w, seed=9)
    out_s, hT_s = run_gpu(inp, "tc")
    out_g, hT_g = run_gpu(inp, "tc", flags=_lib.FLAG_NO_SHORT)
    assert torch.equal(out_s, out_g) and torch.equal(hT_s, hT_g)


def test_short_batch_needs_no_records():
    w = Workload("shortws", 64, 8, 8, state_in="fp32", state_out="fp32")
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in make_inputs(w, seed=1).items()}
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")   # the header only
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], A_log=d["A_log"],
                      dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], initial_state=d["initial_state"],
                      final_state=d["final_state"], workspace=ws)
    torch.cuda.synchronize()
    assert flashkda_b200.device_status(ws) == 0 and torch.isfinite(d["out"].float()).all()
