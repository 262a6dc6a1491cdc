"""The give-up path of the device-side waits, and persistent launches that share the GPU.

Every wait inside the kernels (mbarrier, work-queue slot) is bounded: when its limit runs out the kernel
records FKDA_ERR_DEVICE_STATUS in the workspace header, tells the other warpgroups of its CTA, frees its
tensor memory and returns, so the context stays usable.  The first test makes that happen without any fault:
a test-only flag stops finished segments from queueing their follow-ups, so the work queue starves and the
waiters run out a limit shortened to a few milliseconds.  Nothing here traps, faults or waits without bound.
"""
import time

import pytest
import torch

import flashkda_b200
from flashkda_b200 import _lib
from flashkda_b200.synth import Workload, make_inputs, to_device

pytestmark = pytest.mark.gpu


def _call(d, ws, flags=0):
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], A_log=d["A_log"],
                      dt_bias=d["dt_bias"], lower_bound=d["lower_bound"], initial_state=d["initial_state"],
                      final_state=d["final_state"], cu_seqlens=d["cu_seqlens"], algo="tc", workspace=ws, flags=flags)


def _many_chains(seed, n_seq=100, H=5):
    # 500 chains (more than the 444 chain slots of a B200: the segment queue is in use), 10 to 40 chunks each
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(160, 640, (n_seq,), generator=gen).tolist()
    w = Workload("bw", 1, sum(lens), H, state_in="fp32", state_out="fp32", seq_lens=lens, lower_bound=-2.0)
    d = to_device(make_inputs(w, seed=seed), "cuda")
    ws = torch.empty(flashkda_b200.get_workspace_size(w.tokens, w.H, n_seq), dtype=torch.uint8, device="cuda")
    return d, ws


def test_starved_queue_gives_up_cleanly_and_the_next_call_succeeds():
    d, ws = _many_chains(1)
    _call(d, ws)                                   # a normal call: the expected result
    assert flashkda_b200.device_status(ws) == 0
    good_out, good_state = d["out"].clone(), d["final_state"].clone()

    flags = _lib.FLAG_TEST_DROP_PUSH | _lib.flags_wait_ms(5) | _lib.flags_seg_chunks(8)
    t0 = time.perf_counter()
    _call(d, ws, flags)
    status = flashkda_b200.device_status(ws)       # synchronises
    dt = time.perf_counter() - t0
    assert status == 9, "the starved queue must be reported as FKDA_ERR_DEVICE_STATUS"
    assert dt < 2.0, f"the kernel took {dt:.2f} s to give up with a 5 ms limit"

    # the context is intact and the tensor memory was freed: the same call without the hook is correct again
    d["out"].zero_()
    d["final_state"].zero_()
    _call(d, ws, _lib.flags_seg_chunks(8))
    assert flashkda_b200.device_status(ws) == 0
    assert torch.equal(d["out"], good_out) and torch.equal(d["final_state"], good_state)


def test_two_persistent_launches_on_two_streams():
    """Two calls with more chains than chain slots, on two streams at once: the CTAs of the second launch find
    the SMs taken.  First segments are claimed by whichever CTAs run, so neither launch waits for CTAs that
    have not started; both must finish with the results of lone calls and a clean status."""
    probs = [_many_chains(seed) for seed in (2, 3)]
    expect = []
    for d, ws in probs:
        _call(d, ws)
        assert flashkda_b200.device_status(ws) == 0
        expect.append((d["out"].clone(), d["final_state"].clone()))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    limit = _lib.flags_wait_ms(1000)
    for _ in range(5):
        for (d, ws), s in zip(probs, streams):
            d["out"].zero_()
            d["final_state"].zero_()
            s.wait_stream(torch.cuda.current_stream())
        for (d, ws), s in zip(probs, streams):
            with torch.cuda.stream(s):
                _call(d, ws, limit)
        for s in streams:
            s.synchronize()
        for (d, ws), (out, state) in zip(probs, expect):
            assert flashkda_b200.device_status(ws) == 0
            assert torch.equal(d["out"], out) and torch.equal(d["final_state"], state)
