"""Host-memory front end (flashkda_b200.host.fwd_host): same results as the device-tensor call."""
import pytest
import torch

import flashkda_b200
from flashkda_b200.host import fwd_host
from flashkda_b200.synth import Workload, make_inputs, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("varlen", [False, True])
def test_fwd_host_matches_device_call(varlen):
    if varlen:
        w = Workload("hv", 1, 333, 4, state_in="bf16", state_out="bf16", seq_lens=[100, 33, 200])
    else:
        w = Workload("hf", 5, 160, 4, state_in="fp32", state_out="fp32")
    inp = make_inputs(w, seed=8)
    d = to_device(inp, "cuda")
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], d["A_log"], d["dt_bias"],
                      d["lower_bound"], d["initial_state"], d["final_state"], d["cu_seqlens"])
    torch.cuda.synchronize()
    pin = lambda t: None if t is None else t.clone().pin_memory()
    out_h, hT_h = pin(torch.zeros_like(inp["out"])), pin(torch.zeros_like(inp["final_state"]))
    h2d, d2h = fwd_host(pin(inp["q"]), pin(inp["k"]), pin(inp["v"]), pin(inp["g"]), pin(inp["beta"]), inp["scale"], out_h,
                        inp["A_log"], inp["dt_bias"], inp["lower_bound"], pin(inp["initial_state"]), hT_h,
                        inp["cu_seqlens"], device="cuda", slab_sequences=2)
    assert torch.equal(out_h, d["out"].cpu())
    assert torch.equal(hT_h, d["final_state"].cpu())
    assert h2d >= sum(inp[k].numel() * 2 for k in ("q", "k", "v", "g", "beta")) and d2h >= out_h.numel() * 2
