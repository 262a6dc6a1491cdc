"""The CPU oracle against the committed golden fixtures (outputs of the reference's own
torch_ref text executed on the CPU, see tests/golden/make_golden.py).

The oracle uses libm ``tanhf``/``exp2f`` where the fixture generator used torch's
vectorised CPU functions; those differ by one fp32 ulp in about a fifth of the
arguments, which flips a small fraction of bf16 roundings.  The bounds below are
about 3x the measured residual.
"""
import pytest
import torch

import oracle
from kda_testlib import GOLDEN_CASES, load_golden, mismatch_fraction, run_oracle


@pytest.mark.parametrize("name", list(GOLDEN_CASES))
def test_oracle_matches_golden(name):
    w, inp, gold_out, gold_hT = load_golden(name)
    out, hT = run_oracle(inp)
    assert oracle.err_ratio(gold_out, out) <= 1e-3
    assert oracle.max_abs(gold_out, out) <= 6e-4
    assert mismatch_fraction(gold_out, out) <= 0.02
    if gold_hT is not None:
        assert hT is not None
        hTb = hT.to(torch.bfloat16)
        assert torch.equal(hTb.to(hT.dtype), hT), "exported state must be bf16-representable"
        assert oracle.err_ratio(gold_hT.float(), hT.float()) <= 2e-4
        assert mismatch_fraction(gold_hT.float(), hT.float()) <= 2e-3


def test_oracle_zero_length_sequence_passes_state_through():
    """A sequence of length 0 copies initial_state (rounded to bf16) to final_state."""
    from flashkda_b200.synth import Workload, make_inputs
    w = Workload("zl", 1, 20, 2, state_in="fp32", state_out="fp32", seq_lens=[0, 20, 0])
    inp = make_inputs(w)
    out, hT = run_oracle(inp)
    h0 = inp["initial_state"]
    assert torch.equal(hT[0], h0[0].to(torch.bfloat16).float())
    assert torch.equal(hT[2], h0[2].to(torch.bfloat16).float())
    assert not torch.equal(hT[1], h0[1].to(torch.bfloat16).float())


def test_oracle_chained_calls_equal_one_shot():
    """Splitting a sequence at a multiple of 16 and chaining the state reproduces the
    one-shot result bit for bit (the exported state is exactly the on-chip bf16 state)."""
    from flashkda_b200.synth import Workload, make_inputs
    w = Workload("chain", 1, 80, 2, state_in="bf16", state_out="bf16")
    inp = make_inputs(w)
    out_full, hT_full = run_oracle(inp)
    a = dict(inp)
    for key in ("q", "k", "v", "g", "beta"):
        a[key] = inp[key][:, :48].contiguous()
    out_a, hT_a = run_oracle(a)
    b = dict(inp)
    for key in ("q", "k", "v", "g", "beta"):
        b[key] = inp[key][:, 48:].contiguous()
    b["initial_state"] = hT_a
    out_b, hT_b = run_oracle(b)
    assert torch.equal(torch.cat([out_a, out_b], dim=1), out_full)
    assert torch.equal(hT_b, hT_full)


def test_oracle_vs_fp64_recurrence():
    """Independent sanity check of the algorithm: a direct fp64 token-by-token gated
    delta-rule recurrence (no chunking, no low-precision rounding) agrees with the
    oracle at the level the reference reports against FLA's fp64 recurrent kernel
    (tests/test_fwd.py:360: ratio 0.005 on out)."""
    from flashkda_b200.synth import Workload, make_inputs
    w = Workload("gold", 1, 96, 2, state_in="fp32", state_out="fp32")
    inp = make_inputs(w)
    out, hT = run_oracle(inp)
    q, k, v, g, beta = (inp[x][0].double() for x in ("q", "k", "v", "g", "beta"))
    qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    gate = inp["lower_bound"] * torch.sigmoid(torch.exp(inp["A_log"].double())[None, :, None]
                                              * (g + inp["dt_bias"].double()[None]))
    b = torch.sigmoid(beta)
    S = inp["initial_state"][0].double()  # [H, V, K]
    ref = torch.zeros_like(v)
    for t in range(w.T):
        S = S * torch.exp(gate[t])[:, None, :]
        pred = torch.einsum("hvk,hk->hv", S, kn[t])
        S = S + b[t][:, None, None] * torch.einsum("hv,hk->hvk", v[t] - pred, kn[t])
        ref[t] = inp["scale"] * torch.einsum("hvk,hk->hv", S, qn[t])
    assert oracle.err_ratio(ref, out[0].double()) <= 0.01
    assert oracle.err_ratio(S, hT[0].double()) <= 0.01
