"""The forward pass inside a CUDA graph: with a caller-provided workspace `fwd` allocates nothing and issues
only stream-ordered work (two memsets, the kernels), so it can be captured once and replayed - the
launch-bound regime (short sequences) is where that matters."""
import pytest
import torch

import flashkda_b200
from flashkda_b200.synth import Workload, make_inputs, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T", [(4, 96), (1, 2048)], ids=["short", "slab_pipeline"])
def test_capture_and_replay(B, T):
    """The second shape takes the slab pipeline (few chains, long sequence): its side stream forks from and
    joins back into the captured stream through events."""
    w = Workload("graph", B, T, 4, state_in="fp32", state_out="fp32")
    d = to_device(make_inputs(w, seed=3), "cuda")
    ws = torch.empty(flashkda_b200.get_workspace_size(w.tokens, w.H, w.n_seqs), dtype=torch.uint8, device="cuda")

    def call():
        flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], d["A_log"], d["dt_bias"],
                          d["lower_bound"], d["initial_state"], d["final_state"], None, workspace=ws)

    call()  # eager reference (also the first call per device, outside capture)
    torch.cuda.synchronize()
    ref_out, ref_hT = d["out"].clone(), d["final_state"].clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            call()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        d["out"].zero_()
        d["final_state"].zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(d["out"], ref_out)
        assert torch.equal(d["final_state"], ref_hT)
    # new inputs in the same buffers are picked up by a replay
    d["v"].mul_(0.5)
    graph.replay()
    call_out = d["out"].clone()
    call()
    torch.cuda.synchronize()
    assert torch.equal(call_out, d["out"])


def test_captured_ragged_batch_decides_on_the_device_at_every_replay():
    """A ragged batch with 16 tokens per sequence or fewer on average enqueues the one-kernel paths AND the general
    kernels; which of them serves the call is decided on the device from `cu_seqlens`, so one captured graph stays
    correct when a replay finds other sequence lengths in the same buffer."""
    from flashkda_b200 import _lib
    n_seq, H = 48, 2
    lens_by_case = {"short": [3, 16, 1, 8] * 12, "one_long": [2] * 47 + [30]}
    T_total = 48 * 7 + 4                      # room for every case (the tail of the buffers is unused)
    for lens in lens_by_case.values():
        assert len(lens) == n_seq and sum(lens) <= T_total
    w = Workload("graphr", 1, T_total, H, state_in="fp32", state_out="fp32", lower_bound=-2.0, seq_lens=[T_total - n_seq + 1] + [1] * (n_seq - 1))
    d = to_device(make_inputs(w, seed=4), "cuda")
    cu = torch.zeros(n_seq + 1, dtype=torch.int64, device="cuda")
    ws = torch.empty(flashkda_b200.get_workspace_size(T_total, H, n_seq), dtype=torch.uint8, device="cuda")

    def set_case(name):
        cu[1:] = torch.tensor(lens_by_case[name], dtype=torch.int64).cumsum(0).cuda()

    def call(flags=0):
        flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["out"], d["A_log"], d["dt_bias"],
                          d["lower_bound"], d["initial_state"], d["final_state"], cu, workspace=ws, flags=flags)

    set_case("short")
    call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            call()
    torch.cuda.current_stream().wait_stream(side)
    for name in ("one_long", "short", "one_long"):
        set_case(name)
        used = int(cu[-1].item())
        d["out"].zero_()
        d["final_state"].zero_()
        graph.replay()
        torch.cuda.synchronize()
        got_out, got_hT = d["out"][:, :used].clone(), d["final_state"].clone()
        d["out"].zero_()
        d["final_state"].zero_()
        call(flags=_lib.FLAG_NO_SHORT)        # the general kernels, eagerly
        torch.cuda.synchronize()
        assert flashkda_b200.device_status(ws) == 0
        assert torch.equal(got_out, d["out"][:, :used]) and torch.equal(got_hT, d["final_state"]), name
