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


# ---- inputs of the cases whose expected outputs were produced on a GPU by the reference's own torch_ref
#      (tests/golden/make_golden_gpu.py); all generated on the CPU from fixed seeds ----

GATE_CASE_NAMES = ["g=-8_bias=0", "g=-4_bias=0", "g=0_bias=0", "g=8_bias=0", "g=U(-8,8)_bias=0", "g=N(0,8)_bias=0",
                   "g=0_bias={-4,4}", "g=0_bias={-8,8}", "g=0_bias=U(-8,8)", "g=0_bias=N(0,8)"]


def gate_case_inputs(index, T=8192):
    """The gate/bias stress sweep of the reference's accuracy test (tests/test_fwd.py:45-68, 315-333): B=1,
    H=1, q/k/v ~ U[0,1), beta ~ N(0,1), A_log = 0, fp32 state ~ N(0,1) in and out, lower bound -5, one of six
    gate fillings with zero bias or one of four bias fillings with zero gate."""
    gen = torch.Generator().manual_seed(42)
    shp = (1, T, 1, D)
    bf = torch.bfloat16
    q = torch.rand(shp, generator=gen).to(bf)
    k = torch.rand(shp, generator=gen).to(bf)
    v = torch.rand(shp, generator=gen).to(bf)
    beta = torch.randn((1, T, 1), generator=gen).to(bf)
    h0 = torch.randn((1, 1, D, D), generator=gen)
    gen2 = torch.Generator().manual_seed(1000 + index)
    g = torch.zeros(shp)
    dt_bias = torch.zeros(1, D)
    if index < 4:
        g.fill_([-8.0, -4.0, 0.0, 8.0][index])
    elif index == 4:
        g.uniform_(-8, 8, generator=gen2)
    elif index == 5:
        g = torch.randn(shp, generator=gen2) * 8
    elif index == 6:
        dt_bias = torch.where(torch.rand(1, D, generator=gen2) < 0.5, torch.tensor(-4.0), torch.tensor(4.0))
    elif index == 7:
        dt_bias = torch.where(torch.rand(1, D, generator=gen2) < 0.5, torch.tensor(-8.0), torch.tensor(8.0))
    elif index == 8:
        dt_bias = torch.zeros(1, D).uniform_(-8, 8, generator=gen2)
    else:
        dt_bias = torch.randn(1, D, generator=gen2) * 8
    return dict(q=q, k=k, v=v, g=g.to(bf), beta=beta, scale=1.0 / D ** 0.5, out=torch.zeros(shp, dtype=bf),
                A_log=torch.zeros(1), dt_bias=dt_bias.float().contiguous(), lower_bound=-5.0, initial_state=h0,
                final_state=torch.zeros(1, 1, D, D), cu_seqlens=None)


# Many-chains case: 8 x 64 = 512 (sequence, head) chains of 64 chunks, more than the 444 chain slots of a B200,
# so the tensor-core recurrence hands chains from segment to segment through its work queue.
MANY_CHAINS = Workload("many_chains", 8, 1024, 64, lower_bound=-3.0, state_in="fp32", state_out="fp32")
MANY_CHAINS_OUT_EVERY = 256    # the fixture keeps token rows t % 256 == 255 of every sequence
MANY_CHAINS_STATE_EVERY = 32   # and the final states of chains (n * H + h) % 32 == 0


def fp64_recurrence(inp):
    """Token-by-token gated delta rule in float64 on the device of ``inp`` (the mathematical definition, no
    chunking, no bf16 roundings): the independent gold the reference's accuracy test uses through FLA's fp64
    recurrent kernel (tests/test_fwd.py:71-104).  B = 1, any H.  Returns (out [1,T,H,128], state [1,H,V,K])."""
    f64 = torch.float64
    q, k, v, g, beta = (inp[x][0].to(f64) for x in ("q", "k", "v", "g", "beta"))  # [T,H,D] / [T,H]
    dev = q.device
    A = torch.exp(inp["A_log"].to(f64)).view(1, -1, 1)
    gate = inp["lower_bound"] * torch.sigmoid(A * (g + inp["dt_bias"].to(f64).unsqueeze(0)))   # natural-log decay
    decay = torch.exp(gate)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    b = torch.sigmoid(beta)
    T, H, _ = q.shape
    S = torch.zeros(H, D, D, dtype=f64, device=dev) if inp["initial_state"] is None else inp["initial_state"][0].to(f64)
    out = torch.empty(T, H, D, dtype=f64, device=dev)
    for t in range(T):
        S = S * decay[t].unsqueeze(1)                              # S[h, v, k] *= exp(gate[k])
        u = v[t] - torch.einsum("hvk,hk->hv", S, k[t])
        S = S + (b[t].unsqueeze(-1) * u).unsqueeze(-1) * k[t].unsqueeze(1)
        out[t] = torch.einsum("hvk,hk->hv", S, q[t]) * inp["scale"]
    return out.unsqueeze(0), S.unsqueeze(0)
