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


# ---- ragged batches whose sequences all fit one chunk (the device decides: the host sees only the totals) ----
def _ragged_lens(kind):
    g = torch.Generator().manual_seed(11)
    if kind == "1..16":
        return torch.randint(1, 17, (40,), generator=g).tolist()
    if kind == "ones":            # a decode step handed over as a ragged batch
        return [1] * 48
    if kind == "with_empty":
        lens = torch.randint(0, 17, (44,), generator=g).tolist()
        lens[0], lens[5], lens[-1] = 0, 0, 0
        return lens
    if kind == "full":
        return [16] * 36
    raise KeyError(kind)


def _run_ragged(inp, flags=0):
    """Like run_gpu, with a workspace painted beforehand; returns (out, final_state, untouched record bytes?)."""
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    n = d["cu_seqlens"].numel() - 1
    need = flashkda_b200.get_workspace_size(d["q"].shape[1], d["q"].shape[2], n)
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device="cuda")
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], A_log=d["A_log"],
                      dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], initial_state=d["initial_state"],
                      final_state=d["final_state"], cu_seqlens=d["cu_seqlens"], workspace=ws, flags=flags)
    torch.cuda.synchronize()
    assert flashkda_b200.device_status(ws) == 0
    records_untouched = bool((ws[16384:] == 0xAB).all().item())   # header, prefix tables and queue sit in front
    return d["out"].cpu(), None if d["final_state"] is None else d["final_state"].cpu(), records_untouched


@pytest.mark.parametrize("kind", ["1..16", "ones", "with_empty", "full"])
@pytest.mark.parametrize("state_dtype", ["bf16", "fp32"])
def test_ragged_short_batch_matches_general_path_and_oracle(kind, state_dtype):
    lens = _ragged_lens(kind)
    w = Workload("rs", 1, sum(lens), 2, state_in=state_dtype, state_out=state_dtype, lower_bound=-2.0, seq_lens=lens)
    inp = make_inputs(w, seed=21)
    out_s, hT_s, untouched = _run_ragged(inp)
    # prefix, fused kernel, and the two general kernels that return at once; as many tokens as sequences: the decode
    # kernel is enqueued too, and serves the call when every sequence has one token
    assert flashkda_b200.last_launch_count() == (5 if kind == "ones" else 4)
    assert untouched, "neither one-kernel path keeps chunk records"
    out_g, hT_g, untouched_g = _run_ragged(inp, flags=_lib.FLAG_NO_SHORT)
    assert flashkda_b200.last_launch_count() == 3 and not untouched_g
    if kind == "ones":   # the decode kernel sums its dot products in another order (see test_decode.py)
        assert oracle.err_ratio(out_g, out_s) <= 2e-3 and (out_s != out_g).float().mean().item() <= 0.05
        assert oracle.err_ratio(hT_g, hT_s) <= 1e-3
        out_f, hT_f, _ = _run_ragged(inp, flags=_lib.FLAG_NO_DECODE)   # the fused short-sequence kernel instead
        assert flashkda_b200.last_launch_count() == 4
        assert torch.equal(out_f, out_g) and torch.equal(hT_f, hT_g)
    else:
        assert torch.equal(out_s, out_g) and torch.equal(hT_s, hT_g)
    ref_out, ref_hT = run_oracle(inp)
    check_against(out_s, hT_s, ref_out, ref_hT)
    for n, L in enumerate(lens):
        if L == 0:
            assert torch.equal(hT_s[n].float(), inp["initial_state"][n].to(torch.bfloat16).float())


def test_ragged_batch_with_one_longer_sequence_takes_the_general_kernels():
    lens = [3] * 47 + [17]    # 16 tokens per sequence or fewer on average, but not each
    w = Workload("rl", 1, sum(lens), 2, state_in="fp32", state_out="fp32", lower_bound=-2.0, seq_lens=lens)
    inp = make_inputs(w, seed=22)
    out_s, hT_s, untouched = _run_ragged(inp)
    assert flashkda_b200.last_launch_count() == 4 and not untouched
    out_g, hT_g, _ = _run_ragged(inp, flags=_lib.FLAG_NO_SHORT)
    assert torch.equal(out_s, out_g) and torch.equal(hT_s, hT_g)
    ref_out, ref_hT = run_oracle(inp)
    check_against(out_s, hT_s, ref_out, ref_hT)


def test_ragged_short_batch_without_states_and_many_chains():
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1, 17, (300,), generator=g).tolist()
    w = Workload("rm", 1, sum(lens), 8, lower_bound=-1.0, seq_lens=lens)   # 2 400 chains: the segment queue's regime
    inp = make_inputs(w, seed=23)
    out_s, _, _ = _run_ragged(inp)   # (the queue slots of this regime are reset by the host either way)
    assert flashkda_b200.last_launch_count() == 4
    out_g, _, _ = _run_ragged(inp, flags=_lib.FLAG_NO_SHORT)
    assert torch.equal(out_s, out_g)
    ref_out, _ = run_oracle(inp)
    check_against(out_s, None, ref_out, None)


def test_ragged_batch_with_as_many_tokens_as_sequences_but_not_one_each():
    lens = [0, 2] * 20 + [1] * 8   # 48 tokens, 48 sequences: the decode kernel is enqueued and must stand back
    w = Workload("rd", 1, sum(lens), 2, state_in="bf16", state_out="bf16", lower_bound=-2.0, seq_lens=lens)
    inp = make_inputs(w, seed=24)
    out_s, hT_s, untouched = _run_ragged(inp)
    assert flashkda_b200.last_launch_count() == 5 and untouched
    out_g, hT_g, _ = _run_ragged(inp, flags=_lib.FLAG_NO_SHORT)
    assert torch.equal(out_s, out_g) and torch.equal(hT_s, hT_g)


def test_ragged_decode_step_matches_the_fixed_batch_decode_step():
    """cu_seqlens = 0, 1, 2, ... describes the same problem as a fixed batch with T = 1."""
    N, H = 40, 4
    w = Workload("rdf", N, 1, H, state_in="fp32", state_out="fp32", lower_bound=-2.0)
    inp = make_inputs(w, seed=25)
    out_f, hT_f = run_gpu(inp, "tc")
    assert flashkda_b200.last_launch_count() == 1
    rag = dict(inp)
    for k in ("q", "k", "v", "g", "beta", "out"):
        rag[k] = inp[k].reshape(1, N, *inp[k].shape[2:]).clone()
    rag["cu_seqlens"] = torch.arange(N + 1, dtype=torch.int64)
    rag["final_state"] = torch.zeros_like(inp["final_state"])
    out_r, hT_r, untouched = _run_ragged(rag)
    assert flashkda_b200.last_launch_count() == 5 and untouched
    assert torch.equal(out_r.reshape(out_f.shape), out_f) and torch.equal(hT_r, hT_f)
