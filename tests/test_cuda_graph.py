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
