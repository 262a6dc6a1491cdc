"""GPU tests at the full sizes of the benchmark configurations and of the reference's own smoke / long tests.

Where the CPU oracle finishes in seconds the whole result is compared with it (cfg2, cfg3, the reference's
T=8192 x H=96 smoke shape, T=131072 x H=1).  At the sizes it cannot reach (cfg4: 16.8 M token-heads, cfg5 and
the reference's T=1 M case) the checks are size-independent properties of the operator:
  * causality: the first tokens of a sequence do not depend on later ones, so a prefix of the full-size result
    equals the oracle run on that prefix alone (parity tolerances);
  * chaining: running a sequence in pieces that are multiples of 16 tokens, handing the state over, equals the
    one-shot run bit for bit;
  * independence: one sequence of a batch equals the same sequence run alone, bit for bit;
  * every exported state value is bf16-representable and finite.
Shape lists: tests/test_fwd.py:222-312 and tests/test_fwd_full.py:212-274 of the reference.
"""
import pytest
import torch

import flashkda_b200
import oracle
from flashkda_b200.synth import Workload, config, make_inputs, make_reference_test_inputs
from kda_testlib import run_oracle
from test_gpu_parity import OUT_MAX_ABS, OUT_RATIO, STATE_RATIO, check_against

pytestmark = pytest.mark.gpu

KEYS = ("q", "k", "v", "g", "beta")


def fwd_dev(inp, **over):
    """One forward on tensors that already live on the GPU; returns nothing (results in place)."""
    d = dict(inp, **over)
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], A_log=d["A_log"],
                      dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], initial_state=d["initial_state"],
                      final_state=d["final_state"], cu_seqlens=d["cu_seqlens"])


def cpu(inp):
    return {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in inp.items()}


def prefix_problem(inp, b, n_tokens, state_out_dtype=None):
    """Sequence ``b`` of a fixed batch cut to its first ``n_tokens`` tokens, as a CPU problem for the oracle."""
    sub = {k: inp[k][b:b + 1, :n_tokens].contiguous().cpu() for k in KEYS}
    sub.update(scale=inp["scale"], A_log=inp["A_log"].cpu(), dt_bias=inp["dt_bias"].cpu(),
               lower_bound=inp["lower_bound"], cu_seqlens=None, out=torch.zeros_like(sub["v"]),
               initial_state=None if inp["initial_state"] is None else inp["initial_state"][b:b + 1].cpu(),
               final_state=None)
    if state_out_dtype is not None:
        H = sub["q"].shape[2]
        sub["final_state"] = torch.zeros(1, H, 128, 128, dtype=state_out_dtype)
    return sub


def test_cfg2_against_oracle():
    inp = make_inputs(config("cfg2"), device="cuda")
    fwd_dev(inp)
    ref_out, ref_hT = run_oracle(cpu(inp))
    check_against(inp["out"].cpu(), None, ref_out, None)


def test_cfg3_against_oracle():
    w = config("cfg3")
    inp = make_inputs(w, device="cuda")
    fwd_dev(inp)
    ref_out, ref_hT = run_oracle(cpu(inp))
    check_against(inp["out"].cpu(), inp["final_state"].cpu(), ref_out, ref_hT)


def test_reference_smoke_shapes_against_oracle():
    """B=1, T=8192, H=96 with the arange-valued bf16 state, and the six-sequence ragged batch, both with the
    reference's input recipe (normalised q/k, U[0,1) A_log and dt_bias)."""
    w = Workload("smoke", 1, 8192, 96, state_in="bf16", state_out="bf16")
    inp = make_reference_test_inputs(w, device="cuda", seed=0)
    fwd_dev(inp)
    ref_out, ref_hT = run_oracle(cpu(inp))
    check_against(inp["out"].cpu(), inp["final_state"].cpu(), ref_out, ref_hT)
    lens = [1300, 547, 2048, 963, 271, 3063]
    w = Workload("smokev", 1, sum(lens), 96, state_in="bf16", state_out="bf16", seq_lens=lens)
    inp = make_reference_test_inputs(w, device="cuda", seed=0)
    fwd_dev(inp)
    ref_out, ref_hT = run_oracle(cpu(inp))
    check_against(inp["out"].cpu(), inp["final_state"].cpu(), ref_out, ref_hT)


def test_long_single_head_against_oracle():
    """T = 131 072, H = 1, bf16 state in and out, fixed and as a one-sequence ragged batch."""
    w = Workload("long", 1, 131072, 1, state_in="bf16", state_out="bf16", lower_bound=-1.0)
    inp = make_inputs(w, device="cuda", seed=5)
    fwd_dev(inp)
    ref_out, ref_hT = run_oracle(cpu(inp))
    check_against(inp["out"].cpu(), inp["final_state"].cpu(), ref_out, ref_hT)
    out_v, hT_v = torch.zeros_like(inp["out"]), torch.zeros_like(inp["final_state"])
    cu = torch.tensor([0, w.T], dtype=torch.int64, device="cuda")
    fwd_dev(inp, out=out_v, final_state=hT_v, cu_seqlens=cu)
    assert torch.equal(out_v, inp["out"]) and torch.equal(hT_v, inp["final_state"])


def test_million_token_sequence_chains_exactly():
    """T = 1 048 576, H = 1 (the reference's longest test) and two sequences of 524 288 as a ragged batch:
    one shot equals four chained quarter-length calls, and equals the two halves as separate calls."""
    T = 1 << 20
    w = Workload("long1m", 1, T, 1, state_in="bf16", state_out="bf16", lower_bound=-0.5)
    inp = make_inputs(w, device="cuda", seed=6)
    fwd_dev(inp)
    assert torch.isfinite(inp["out"].float()).all() and torch.isfinite(inp["final_state"].float()).all()
    # four chained pieces
    out_c = torch.zeros_like(inp["out"])
    state = inp["initial_state"]
    q4 = T // 4
    for i in range(4):
        sl = slice(i * q4, (i + 1) * q4)
        nxt = torch.zeros_like(inp["final_state"])
        piece = {k: inp[k][:, sl].contiguous() for k in KEYS}
        o = torch.zeros_like(piece["v"])
        fwd_dev(dict(inp, **piece), out=o, initial_state=state, final_state=nxt)
        out_c[:, sl] = o
        state = nxt
    assert torch.equal(out_c, inp["out"]) and torch.equal(state, inp["final_state"])
    # the same tokens as two ragged sequences of half the length, zero initial states
    half = T // 2
    cu = torch.tensor([0, half, T], dtype=torch.int64, device="cuda")
    out_v = torch.zeros_like(inp["out"])
    hT_v = torch.zeros(2, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    fwd_dev(inp, out=out_v, initial_state=None, final_state=hT_v, cu_seqlens=cu)
    for j in range(2):
        sl = slice(j * half, (j + 1) * half)
        piece = {k: inp[k][:, sl].contiguous() for k in KEYS}
        o, h = torch.zeros_like(piece["v"]), torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
        fwd_dev(dict(inp, **piece), out=o, initial_state=None, final_state=h)
        assert torch.equal(out_v[:, sl], o) and torch.equal(hT_v[j:j + 1], h)
    # prefix against the oracle
    sub = prefix_problem(inp, 0, 4096)
    ref_out, _ = run_oracle(sub)
    check_against(inp["out"][:, :4096].cpu(), None, ref_out, None)


def test_cfg4_full_size_properties():
    """B=8, T=32768, H=64, fp32 states (21.6 GB of inputs and outputs, 15 GB of workspace)."""
    w = config("cfg4")
    inp = make_inputs(w, device="cuda")
    fwd_dev(inp)
    hT = inp["final_state"]
    assert torch.isfinite(hT).all()
    assert torch.equal(hT.to(torch.bfloat16).to(hT.dtype), hT)
    assert torch.isfinite(inp["out"][::2, ::64].float()).all()
    b = 5
    # independence: sequence b alone (different chain count: other kernel schedule, same numbers)
    one = {k: inp[k][b:b + 1] for k in KEYS}
    o1, h1 = torch.zeros_like(one["v"]), torch.zeros_like(hT[b:b + 1])
    fwd_dev(dict(inp, **one), out=o1, initial_state=inp["initial_state"][b:b + 1], final_state=h1)
    assert torch.equal(o1, inp["out"][b:b + 1]) and torch.equal(h1, hT[b:b + 1])
    # chaining: two halves with the state handed over
    half = w.T // 2
    state = inp["initial_state"][b:b + 1]
    for i in range(2):
        sl = slice(i * half, (i + 1) * half)
        piece = {k: inp[k][b:b + 1, sl].contiguous() for k in KEYS}
        o, nxt = torch.zeros_like(piece["v"]), torch.zeros_like(h1)
        fwd_dev(dict(inp, **piece), out=o, initial_state=state, final_state=nxt)
        assert torch.equal(o, inp["out"][b:b + 1, sl])
        state = nxt
    assert torch.equal(state, hT[b:b + 1])
    # causality: the first 2048 tokens of sequence 2, all 64 heads, against the oracle
    sub = prefix_problem(inp, 2, 2048, state_out_dtype=torch.float32)
    ref_out, ref_hT = run_oracle(sub)
    check_against(inp["out"][2:3, :2048].cpu(), None, ref_out, None)
    del inp
    torch.cuda.empty_cache()


def test_cfg5_full_size_properties():
    """B=1, T=1 048 576, H=32, fp32 final state (43 GB of inputs and outputs, 29 GB of workspace)."""
    w = config("cfg5")
    inp = make_inputs(w, device="cuda")
    fwd_dev(inp)
    hT = inp["final_state"]
    assert torch.isfinite(hT).all() and torch.equal(hT.to(torch.bfloat16).to(hT.dtype), hT)
    # chaining in four pieces (fp32 hand-over states hold bf16-representable values: exact)
    out_c = torch.zeros_like(inp["out"])
    state = None
    q4 = w.T // 4
    for i in range(4):
        sl = slice(i * q4, (i + 1) * q4)
        nxt = torch.zeros_like(hT)
        fwd_dev(dict(inp, **{k: inp[k][:, sl] for k in KEYS}), out=out_c[:, sl], initial_state=state, final_state=nxt)
        state = nxt
    assert torch.equal(state, hT)
    assert torch.equal(out_c, inp["out"])
    # causality: first 4096 tokens against the oracle
    sub = prefix_problem(inp, 0, 4096)
    ref_out, _ = run_oracle(sub)
    check_against(inp["out"][:, :4096].cpu(), None, ref_out, None)
    # the in-GPU sequence split (approximate at piece boundaries) stays within the parity tolerances
    from flashkda_b200 import cp
    out_s, hT_s = torch.zeros_like(inp["out"]), torch.zeros_like(hT)
    cp.fwd_sequence_parallel(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], out_s, inp["A_log"],
                             inp["dt_bias"], inp["lower_bound"], None, hT_s, parts=16)
    assert oracle.err_ratio(hT.cpu(), hT_s.cpu()) <= STATE_RATIO
    assert oracle.err_ratio(inp["out"][:, ::16].cpu(), out_s[:, ::16].cpu()) <= OUT_RATIO
    assert oracle.max_abs(inp["out"][:, ::16].cpu(), out_s[:, ::16].cpu()) <= OUT_MAX_ABS
    del inp
    torch.cuda.empty_cache()
