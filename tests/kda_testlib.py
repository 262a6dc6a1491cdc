"""Shared helpers for the test-suite: golden fixture loading, oracle calls, metrics."""
import os

import numpy as np
import torch

import oracle
from flashkda_b200.synth import D, Workload, config, make_inputs, make_reference_test_inputs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Workloads of the committed fixtures (must match tests/golden/make_golden.py).
GOLDEN_CASES = {
    "cfg1": (config("cfg1"), "bench"),
    "varlen_small_bf16": (Workload("varlen_small_bf16", 1, 100, 2, state_in="bf16", state_out="bf16",
                                   seq_lens=[4, 8, 12, 1, 17, 1, 33, 24]), "reftest"),
    "varlen_fp32_out_only": (Workload("varlen_fp32_out_only", 1, 115, 2, state_out="fp32",
                                      seq_lens=[17, 33, 65]), "reftest"),
    "fixed_T37_stateless": (Workload("fixed_T37_stateless", 1, 37, 3), "reftest"),
    "fixed_T64_fp32_inout": (Workload("fixed_T64_fp32_inout", 2, 64, 2, state_in="fp32", state_out="fp32"),
                             "reftest"),
    "fixed_T97_bf16_in_only_lb3": (Workload("fixed_T97_bf16_in_only_lb3", 1, 97, 1, lower_bound=-3.0,
                                            state_in="bf16"), "bench"),
}


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_golden(name):
    """Returns (inputs dict on CPU, golden out bf16, golden final_state bf16-valued or None)."""
    w, style = GOLDEN_CASES[name]
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    inp = make_inputs(w) if style == "bench" else make_reference_test_inputs(w)
    if "in_q" in z.files:
        for key in ("q", "k", "v", "g", "beta"):
            inp[key] = _bf16(z["in_" + key])
        inp["A_log"] = torch.from_numpy(z["in_A_log"].copy())
        inp["dt_bias"] = torch.from_numpy(z["in_dt_bias"].copy())
        if "in_initial_state" in z.files:
            inp["initial_state"] = _bf16(z["in_initial_state"]).to(inp["initial_state"].dtype)
    else:
        chk = int(inp["q"].view(torch.int16).numpy().view(np.uint16).astype(np.uint64).sum())
        assert chk == int(z["q_checksum"]), "seeded input generation drifted from the fixture"
    out = _bf16(z["out"])
    hT = _bf16(z["final_state"]) if "final_state" in z.files else None
    return w, inp, out, hT


def run_oracle(inp):
    """Runs the CPU oracle on (a CPU copy of) ``inp``; returns (out, final_state)."""
    out = torch.zeros(inp["q"].shape, dtype=torch.bfloat16)
    hT = None
    if inp["final_state"] is not None:
        hT = torch.zeros(inp["final_state"].shape, dtype=inp["final_state"].dtype)
    oracle.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], out, inp["A_log"], inp["dt_bias"],
               inp["lower_bound"], initial_state=inp["initial_state"], final_state=hT, cu_seqlens=inp["cu_seqlens"])
    return out, hT


def mismatch_fraction(a, b):
    return (a != b).float().mean().item() if a.numel() else 0.0
