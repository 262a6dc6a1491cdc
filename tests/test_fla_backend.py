"""The second FLA backend (``flashkda_b200.fla_backend``): intermediate states and FLA's context-parallel
convention, which FLA's stock FlashKDA backend declines (fla/ops/kda/backends/flashkda.py:82-85).

CPU part: the context-parallel host logic with gloo ranks and the CPU oracle as operator, contexts built by FLA's
own ``get_cp_cu_seqlens``, against a one-process oracle run on the packed batch.
GPU part: dispatch through ``fla.ops.kda.chunk_kda`` with ``return_intermediate_states=True`` against FLA's
Triton path (its own tolerance for this pair of implementations, tests/test_fwd.py:360), and the states
against prefix runs of the operator itself (bit for bit).
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from flashkda_b200.synth import Workload, make_inputs, to_device
from kda_testlib import run_oracle

fla = pytest.importorskip("fla")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _packed_inputs(lens, H, seed):
    w = Workload("flacp", 1, sum(lens), H, lower_bound=-0.05, seq_lens=lens)
    inp = make_inputs(w, seed=seed)
    inp["A_log"] = torch.full_like(inp["A_log"], -2.5)   # weak gates: the transition maps matter
    return inp


def _cp_worker(rank, world, port, lens, H, seed, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from fla.ops.cp.context import get_cp_cu_seqlens
    from flashkda_b200.fla_backend import fwd_fla_context_parallel
    inp = _packed_inputs(lens, H, seed)
    cu = inp["cu_seqlens"]
    ctx = get_cp_cu_seqlens(cu, cu_seqlens_cpu=cu.clone(), world_size=world, rank=rank, group=dist.group.WORLD)
    part = sum(lens) // world
    sl = lambda x: x[:, rank * part:(rank + 1) * part].contiguous()
    out = torch.zeros_like(sl(inp["v"]))
    fwd_fla_context_parallel(sl(inp["q"]), sl(inp["k"]), sl(inp["v"]), sl(inp["g"]), sl(inp["beta"]), inp["scale"], out,
                             inp["A_log"], inp["dt_bias"], inp["lower_bound"], ctx, fwd_fn=oracle.fwd)
    ret[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,lens", [(2, [100, 300, 50, 190]), (3, [40, 500, 60]), (4, [640]), (2, [320, 320])])
def test_fla_context_parallel_convention_gloo(world, lens):
    H, seed = 2, 11
    inp = _packed_inputs(lens, H, seed)
    ref_out, _ = run_oracle(inp)
    ret = mp.Manager().dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), lens, H, seed, ret), nprocs=world, join=True)
    part = sum(lens) // world
    for r in range(world):
        ref = ref_out[:, r * part:(r + 1) * part]
        assert oracle.max_abs(ref, ret[r]) <= 2e-2
        assert oracle.err_ratio(ref, ret[r]) <= 1e-2, f"rank {r}"


@pytest.mark.gpu
@pytest.mark.parametrize("lens", [None, [200, 64, 1, 300]])
def test_chunk_kda_returns_intermediate_states_through_fla(lens):
    import flashkda_b200
    import flashkda_b200.fla_backend as fb
    from fla.ops.kda import chunk_kda
    fb.register()
    H = 4
    if lens is None:
        w = Workload("flah", 2, 256, H, state_in="fp32", lower_bound=-2.0)
    else:
        w = Workload("flah", 1, sum(lens), H, state_in="fp32", lower_bound=-2.0, seq_lens=lens)
    d = to_device(make_inputs(w, seed=9), "cuda")
    kw = dict(scale=d["scale"], initial_state=d["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
              use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, safe_gate=True, lower_bound=d["lower_bound"],
              transpose_state_layout=True, A_log=d["A_log"], dt_bias=d["dt_bias"].reshape(-1),
              cu_seqlens=d["cu_seqlens"], return_intermediate_states=True)
    try:
        with torch.inference_mode():
            out, hT, h = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], **kw)
    finally:
        # leave FLA's registry as other tests expect it (they watch the stock backend being dispatched)
        from fla.ops.kda.backends import kda_registry
        kda_registry._backends.pop("flashkda_b200", None)
    torch.cuda.synchronize()
    # ours, directly: the same call with exported states
    slots = flashkda_b200.chunk_states_slots(w.B, w.T, 4, seq_lens=lens)
    assert h.shape[0] * h.shape[1] == slots and h.dtype == torch.bfloat16
    out2 = torch.zeros_like(d["v"])
    hT2 = torch.zeros_like(hT)
    hs = torch.zeros(slots, H, 128, 128, dtype=torch.bfloat16, device="cuda")
    flashkda_b200.fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], out2, A_log=d["A_log"], dt_bias=d["dt_bias"],
                      lower_bound=d["lower_bound"], initial_state=d["initial_state"], final_state=hT2,
                      cu_seqlens=d["cu_seqlens"], chunk_states=hs, chunk_states_every=4)
    assert torch.equal(out, out2) and torch.equal(hT, hT2) and torch.equal(h.reshape(hs.shape), hs), \
        "the backend did not serve the call (or changed its results)"
    # the first slot of every sequence is its (bf16-rounded) initial state
    first = 0
    for n in range(d["initial_state"].shape[0]):
        L = w.T if lens is None else lens[n]
        if L > 0:
            assert torch.equal(hs[first], d["initial_state"][n].to(torch.bfloat16))
        first += (L + 63) // 64
