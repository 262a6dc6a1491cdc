"""Context parallelism (one long sequence sharded over ranks): host logic on CPU with gloo process
groups (world sizes 2 and 3, the CPU oracle standing in for the device operator), and the numerics of
the map-and-fold scheme on one GPU with all shards in one process."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from flashkda_b200 import cp
from flashkda_b200.synth import Workload, make_inputs, to_device
from kda_testlib import run_oracle


def _weak_decay_inputs(T, H, seed):
    """Weak gates (A_log = log 0.05, lower_bound -0.02) so that the transition M of a shard is far from
    zero and the fold really matters; strong default gates would hide a wrong M."""
    w = Workload("cp", 1, T, H, lower_bound=-0.02, state_in="fp32", state_out="fp32")
    inp = make_inputs(w, seed=seed)
    inp["A_log"] = torch.full_like(inp["A_log"], -3.0)
    return inp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cp_worker(rank, world, port, T, H, seed, ret, state_dtype=torch.float32):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    inp = _weak_decay_inputs(T, H, seed)
    per = (T // world) // 16 * 16
    lo, hi = rank * per, (T if rank == world - 1 else (rank + 1) * per)
    sh = {key: inp[key][:, lo:hi].contiguous() for key in ("q", "k", "v", "g", "beta")}
    out = torch.zeros_like(sh["v"])
    hT = torch.zeros_like(inp["final_state"])
    cp.fwd_context_parallel(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], inp["scale"], out, inp["A_log"],
                            inp["dt_bias"], inp["lower_bound"], initial_state=inp["initial_state"].to(state_dtype),
                            final_state=hT, fwd_fn=oracle.fwd)
    ret[rank] = (lo, hi, out, hT)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_gloo(world):
    T, H, seed = 400, 2, 31
    inp = _weak_decay_inputs(T, H, seed)
    ref_out, ref_hT = run_oracle(inp)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), T, H, seed, ret), nprocs=world, join=True)
    out = torch.zeros_like(ref_out)
    for r in range(world):
        lo, hi, o, hT = ret[r]
        out[:, lo:hi] = o
        assert oracle.err_ratio(ref_hT, hT) <= 1e-2, f"rank {r} final_state"
    assert oracle.max_abs(ref_out, out) <= 2e-2
    assert oracle.err_ratio(ref_out, out) <= 1e-2
    # rank 0's shard is computed exactly as in the one-shot run
    lo, hi, o, _ = ret[0]
    assert torch.equal(o, ref_out[:, lo:hi])


def test_context_parallel_gloo_bf16_initial_state():
    """A bf16 initial state with an fp32 final state: rank 0 widens it (the maps and folds are fp32), so no rank
    fails an operator dtype check while the others sit in the all-gather."""
    T, H, seed, world = 256, 1, 33, 2
    inp = _weak_decay_inputs(T, H, seed)
    inp["initial_state"] = inp["initial_state"].to(torch.bfloat16).float()   # what the bf16 caller means
    ref_out, ref_hT = run_oracle(inp)
    ret = mp.Manager().dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), T, H, seed, ret, torch.bfloat16), nprocs=world, join=True)
    for r in range(world):
        lo, hi, o, hT = ret[r]
        assert oracle.err_ratio(ref_out[:, lo:hi], o) <= 1e-2
        assert oracle.err_ratio(ref_hT, hT) <= 1e-2


def _bad_shard_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    inp = _weak_decay_inputs(40, 1, 1)      # 40 tokens on every rank: not a multiple of 16
    try:
        cp.fwd_context_parallel(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                                inp["A_log"], inp["dt_bias"], inp["lower_bound"], fwd_fn=oracle.fwd)
        ret[rank] = "no error"
    except RuntimeError as e:
        ret[rank] = str(e)
    dist.barrier()
    dist.destroy_process_group()


def test_bad_shard_length_fails_before_any_collective():
    ret = mp.Manager().dict()
    mp.spawn(_bad_shard_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert "multiple of 16" in ret[0]      # rank 0 is not the last shard: rejected
    assert "another rank" in ret[1]        # the last rank's own shard is fine; it learns of rank 0's verdict


def test_fold_is_needed_with_weak_decay():
    """Sanity of the test itself: dropping the transition M changes the result visibly."""
    inp = _weak_decay_inputs(256, 1, 5)
    half = {key: inp[key][:, 128:].contiguous() for key in ("q", "k", "v", "g", "beta")}
    M, N = cp.shard_maps(oracle.fwd, half["q"], half["k"], half["v"], half["g"], half["beta"], inp["scale"],
                         inp["A_log"], inp["dt_bias"], inp["lower_bound"])
    assert M.abs().max() > 0.05
    S = torch.randn(1, 1, 128, 128) * 0.05
    assert oracle.err_ratio(cp.fold_initial_state(S, [(M, N)]), N) > 1e-2


def test_emulated_shards_match_one_shot_cpu():
    inp = _weak_decay_inputs(512, 2, 9)
    ref_out, ref_hT = run_oracle(inp)
    out = torch.zeros_like(ref_out)
    hT = torch.zeros_like(ref_hT)
    cp.fwd_sharded_emulated(4, inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], out, inp["A_log"],
                            inp["dt_bias"], inp["lower_bound"], inp["initial_state"], hT, fwd_fn=oracle.fwd)
    assert oracle.err_ratio(ref_out, out) <= 1e-2
    assert oracle.err_ratio(ref_hT, hT) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shards", [2, 4, 8])
def test_emulated_shards_match_one_shot_gpu(shards):
    import flashkda_b200
    inp = to_device(_weak_decay_inputs(4096, 4, 17), "cuda")
    one_out, one_hT = torch.zeros_like(inp["out"]), torch.zeros_like(inp["final_state"])
    flashkda_b200.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], one_out, inp["A_log"],
                      inp["dt_bias"], inp["lower_bound"], inp["initial_state"], one_hT)
    out, hT = torch.zeros_like(one_out), torch.zeros_like(one_hT)
    cp.fwd_sharded_emulated(shards, inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], out,
                            inp["A_log"], inp["dt_bias"], inp["lower_bound"], inp["initial_state"], hT)
    torch.cuda.synchronize()
    print(f"shards {shards}: out ratio {oracle.err_ratio(one_out, out):.3e} state ratio {oracle.err_ratio(one_hT, hT):.3e}")
    assert oracle.max_abs(one_out, out) <= 2e-2
    assert oracle.err_ratio(one_out, out) <= 1e-2
    assert oracle.err_ratio(one_hT, hT) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("parts", [2, 8])
def test_sequence_parallel_single_gpu(parts):
    import flashkda_b200
    inp = to_device(_weak_decay_inputs(4096, 4, 23), "cuda")
    one_out, one_hT = torch.zeros_like(inp["out"]), torch.zeros_like(inp["final_state"])
    flashkda_b200.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], one_out, inp["A_log"],
                      inp["dt_bias"], inp["lower_bound"], inp["initial_state"], one_hT)
    out, hT = torch.zeros_like(one_out), torch.zeros_like(one_hT)
    cp.fwd_sequence_parallel(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], out, inp["A_log"],
                             inp["dt_bias"], inp["lower_bound"], inp["initial_state"], hT, parts=parts)
    torch.cuda.synchronize()
    print(f"parts {parts}: out ratio {oracle.err_ratio(one_out, out):.3e} state ratio {oracle.err_ratio(one_hT, hT):.3e}")
    assert oracle.max_abs(one_out, out) <= 2e-2
    assert oracle.err_ratio(one_out, out) <= 1e-2
    assert oracle.err_ratio(one_hT, hT) <= 1e-2


@pytest.mark.gpu
def test_fold_kernel_matches_matmul():
    """The library's own fold (S . M + N per head, fp32 FMAs in a fixed order) against torch's fp32 matmul."""
    g = torch.Generator().manual_seed(0)
    S, M, N = (torch.randn(3, 5, 128, 128, generator=g).cuda() for _ in range(3))
    M = M * 0.1
    for off in (N, None):
        got = cp.fold(S, M, off)
        ref = torch.matmul(S.double(), M.double()) + (0 if off is None else off.double())
        assert got.dtype == torch.float32 and got.shape == S.shape
        assert (got.double() - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    # an identity map leaves the state as it is, bit for bit
    eye = torch.eye(128, device="cuda").expand(3, 5, 128, 128).contiguous()
    assert torch.equal(cp.fold(S, eye), S)
    # the C entry point refuses an output that aliases an input (every CTA reads whole rows of S and all of M)
    from flashkda_b200 import _lib
    rc = _lib.lib().fkda_cp_fold(S.data_ptr(), M.data_ptr(), None, S.data_ptr(), 15, torch.cuda.current_stream().cuda_stream)
    assert rc == 2
