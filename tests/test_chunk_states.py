"""Export of intermediate states (``chunk_states``): the state of every sequence before each group of chunks.

FLA's ``chunk_kda(..., return_intermediate_states=True)`` returns these for 64-token chunks; the reference
operator has no such output (its FLA backend declines the option, fla/ops/kda/backends/flashkda.py:84-85).
Oracle: the operator itself, called prefix by prefix -- a state exported before token t equals the final
state of a call on the first t tokens (chained calls are bit-exact, see test_gpu_parity.py), so the
comparison is bit for bit.
"""
import pytest
import torch

import flashkda_b200
from flashkda_b200 import _lib
from flashkda_b200.synth import Workload, make_inputs, to_device

pytestmark = pytest.mark.gpu


def _call(d, sl=None, final=None, init=None, cu=None, **kw):
    cut = (lambda x: x) if sl is None else (lambda x: x[:, sl].contiguous())
    q = cut(d["q"])
    out = torch.zeros_like(q)
    flashkda_b200.fwd(q, cut(d["k"]), cut(d["v"]), cut(d["g"]), cut(d["beta"]), d["scale"], out, A_log=d["A_log"],
                      dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], initial_state=init, final_state=final,
                      cu_seqlens=cu, **kw)
    return out


@pytest.mark.parametrize("algo,flags", [("tc", 0), ("tc", _lib.FLAG_NO_WIDE), ("twopass", 0)])
@pytest.mark.parametrize("B,T,H,every", [(2, 200, 3, 4), (1, 1030, 2, 4), (3, 64, 2, 1), (2, 1, 2, 4)])
def test_fixed_batch_states_equal_prefix_runs(B, T, H, every, algo, flags):
    w = Workload("cs", B, T, H, state_in="bf16", state_out="bf16", lower_bound=-1.0)
    d = to_device(make_inputs(w, seed=3), "cuda")
    group = 16 * every
    per = (T + group - 1) // group
    assert flashkda_b200.chunk_states_slots(B, T, every) == B * per
    hs = torch.full((B * per, H, 128, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    out = _call(d, None, d["final_state"], d["initial_state"], algo=algo, flags=flags, chunk_states=hs,
                chunk_states_every=every)
    plain = _call(d, None, torch.zeros_like(d["final_state"]), d["initial_state"], algo=algo, flags=flags)
    assert torch.equal(out, plain), "exporting states must not change the outputs"
    hs = hs.view(B, per, H, 128, 128)
    assert torch.equal(hs[:, 0], d["initial_state"])
    for i in range(1, per):
        st = torch.zeros_like(d["final_state"])
        _call(d, slice(0, i * group), st, d["initial_state"], algo=algo, flags=flags)
        assert torch.equal(hs[:, i], st), f"state before token {i * group}"


@pytest.mark.parametrize("algo,flags", [("tc", 0), ("tc", _lib.FLAG_NO_WIDE), ("twopass", 0)])
def test_ragged_batch_states(algo, flags):
    lens = [130, 1, 64, 0, 200, 17]
    every, group = 4, 64
    w = Workload("csv", 1, sum(lens), 2, state_in="fp32", state_out="fp32", seq_lens=lens, lower_bound=-1.0)
    d = to_device(make_inputs(w, seed=5), "cuda")
    slots = flashkda_b200.chunk_states_slots(1, 0, every, seq_lens=lens)
    assert slots == 3 + 1 + 1 + 0 + 4 + 1
    hs = torch.full((slots, 2, 128, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    _call(d, None, d["final_state"], d["initial_state"], d["cu_seqlens"], algo=algo, flags=flags, chunk_states=hs,
          chunk_states_every=every)
    torch.cuda.synchronize()
    slot, pos = 0, 0
    for n, L in enumerate(lens):
        h0 = d["initial_state"][n:n + 1].contiguous()
        for i in range((L + group - 1) // group):
            if i == 0:
                expect = h0.to(torch.bfloat16)
            else:
                st = torch.zeros_like(h0)
                _call(d, slice(pos, pos + i * group), st, h0, algo=algo, flags=flags)
                expect = st.to(torch.bfloat16)
            assert torch.equal(hs[slot], expect[0]), f"sequence {n}, group {i}"
            slot += 1
        pos += L
    assert slot == slots
