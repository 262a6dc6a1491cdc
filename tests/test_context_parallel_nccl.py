"""Context parallelism on real GPUs over NCCL (needs >= 2 GPUs; skipped otherwise): sharded runs, with and
without the additional in-GPU sequence split, against the one-shot single-GPU run."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(T, H):
    from flashkda_b200.synth import Workload, make_inputs
    w = Workload("cpn", 1, T, H, lower_bound=-0.02, state_in="fp32", state_out="fp32")
    inp = make_inputs(w, seed=41)
    inp["A_log"] = torch.full_like(inp["A_log"], -3.0)  # weak gates: the transition maps matter
    return inp


def _worker(rank, world, port, T, H, parts, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from flashkda_b200 import cp
    inp = _inputs(T, H)
    per = T // world
    lo, hi = rank * per, (rank + 1) * per
    dev = torch.device("cuda", rank)
    sh = {key: inp[key][:, lo:hi].contiguous().to(dev) for key in ("q", "k", "v", "g", "beta")}
    out = torch.zeros_like(sh["v"])
    hT = torch.zeros_like(inp["final_state"], device=dev)
    cp.fwd_context_parallel(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], inp["scale"], out, inp["A_log"].to(dev),
                            inp["dt_bias"].to(dev), inp["lower_bound"], initial_state=inp["initial_state"].to(dev),
                            final_state=hT, parts=parts)
    torch.cuda.synchronize()
    ret[rank] = (lo, hi, out.cpu(), hT.cpu())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("parts", [1, 4])
def test_context_parallel_nccl(parts):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import flashkda_b200
    from flashkda_b200.synth import to_device
    T, H = 2048 * world, 4
    inp = to_device(_inputs(T, H), "cuda:0")
    one_out, one_hT = torch.zeros_like(inp["out"]), torch.zeros_like(inp["final_state"])
    flashkda_b200.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], one_out, inp["A_log"],
                      inp["dt_bias"], inp["lower_bound"], inp["initial_state"], one_hT)
    torch.cuda.synchronize()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), T, H, parts, ret), nprocs=world, join=True)
    out = torch.zeros_like(one_out).cpu()
    for r in range(world):
        lo, hi, o, hT = ret[r]
        out[:, lo:hi] = o
        assert oracle.err_ratio(one_hT.cpu(), hT) <= 1e-2
    print(f"world {world} parts {parts}: out ratio {oracle.err_ratio(one_out.cpu(), out):.3e}")
    assert oracle.max_abs(one_out.cpu(), out) <= 2e-2
    assert oracle.err_ratio(one_out.cpu(), out) <= 1e-2
