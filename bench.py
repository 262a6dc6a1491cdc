#!/usr/bin/env python
"""Benchmark of the KDA forward pass (tokens/s; one "step" = one forward over the workload).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg4] [--algo auto]

N > 1 is launched with torch.distributed.run (one rank per GPU).  The default is STRONG scaling: the
workload is one fixed problem whose sequences are partitioned over the ranks (cfg4: B = 8 sequences,
8 / N per GPU; every sequence is generated from its own seed, so N = 1 and N = 8 process the same
data); sequences are independent, so there is no data-path collective.  ``--scaling weak`` gives every
rank its own full copy of the workload instead.  Rank 0 prints ONE JSON line.

  value    whole-job tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e      the same through the host-buffer API: pinned host inputs -> H2D -> forward -> D2H
  roofline the whole forward (both kernels back to back): algorithmic bytes / step time vs measured HBM
           peak; per kernel, its OWN bytes (inputs + records it reads and writes) / its launch time
  cpu_baseline  the CPU oracle (a port of the reference's torch_ref numerics) on a bounded sample

--impl reference times the CPU oracle alone (the reference has no CPU implementation of its
own; its torch_ref needs a GPU), with all host threads, on a bounded sample of the workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "kda_fwd_tokens_per_s"
UNIT = "tokens/s"


L2_BYTES = 126e6
FLUSH_BYTES = 512 << 20


def needs_l2_flush(w):
    """Workloads whose tensors could stay in the 126 MB L2 from one step to the next get a 512 MB write between
    timed steps; the larger ones evict themselves."""
    from flashkda_b200.synth import algorithmic_bytes
    return algorithmic_bytes(w) < 4 * L2_BYTES


def config_dict(w, algo, b_per_gpu=None, sharding=None):
    """The workload description both arms print."""
    from flashkda_b200.synth import algorithmic_bytes
    return {"workload": w.name, "B": w.B, "B_per_gpu": w.B if b_per_gpu is None else b_per_gpu, "T": w.T, "H": w.H,
            "K": 128, "V": 128, "chunk": 16,
            "lower_bound": w.lower_bound, "state": w.state_out or w.state_in or "none",
            "varlen_sequences": w.n_seqs if w.seq_lens else 0, "algo": algo,
            "l2_policy": ("L2 flushed between timed steps (512 MB write, outside the timed events)" if needs_l2_flush(w)
                          else "inputs exceed L2 (%.1f GB per step)" % (algorithmic_bytes(w) / 1e9)),
            "sharding": sharding or "independent sequences per GPU, no collective"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--algo", default=None)
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = the workload's sequences are partitioned over the ranks (default); "
                         "weak = every rank runs its own full copy")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--seq-parts", type=int, default=1,
                    help="single GPU, B=1: split the sequence into this many pieces that run side by side "
                         "(flashkda_b200.cp.fwd_sequence_parallel; approximate at piece boundaries)")
    ap.add_argument("--flags", type=int, default=0,
                    help="fkda_fwd_params.flags for the forward calls (profiling aid: 4 = no slab pipeline, so that a "
                         "few-chains forward is two launches)")
    ap.add_argument("--cp-check", action="store_true",
                    help="context-parallel runs: the last rank also runs the whole sequence alone (exact) and reports "
                         "how far its shard of out and the final state are from that")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target duration of the CPU baseline sample")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------
# clocks: sample nvidia-smi during the timed region
# ------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline leg and the --impl reference arm)
# ------------------------------------------------------------------------------------------
def host_threads():
    """Threads the CPU arm uses: every core this process may run on.  Passed to the oracle explicitly, because
    launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their ranks."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample_workload(w, target_seconds):
    """A bounded sample of workload ``w``: one sequence, all H heads, same gate bound and state
    options, with T chosen so that the oracle runs for about ``target_seconds``."""
    import torch
    import oracle
    from flashkda_b200.synth import Workload, make_inputs
    probe = Workload("probe", 1, 256, w.H, lower_bound=w.lower_bound, state_in=w.state_in, state_out=w.state_out)
    inp = make_inputs(probe)
    t0 = time.perf_counter()
    oracle.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"], inp["A_log"],
               inp["dt_bias"], inp["lower_bound"], inp["initial_state"], inp["final_state"], None,
               n_threads=host_threads())
    dt = max(time.perf_counter() - t0, 1e-4)
    T = int(256 * target_seconds / dt) // 16 * 16
    T = max(256, min(T, w.T))
    return Workload(f"{w.name}-cpu-sample", 1, T, w.H, lower_bound=w.lower_bound, state_in=w.state_in,
                    state_out=w.state_out)


def time_oracle(sample, steps, warmup):
    import oracle
    from flashkda_b200.synth import make_inputs
    inp = make_inputs(sample)
    args = (inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"], inp["A_log"],
            inp["dt_bias"], inp["lower_bound"], inp["initial_state"], inp["final_state"], None)
    for _ in range(warmup):
        oracle.fwd(*args, n_threads=host_threads())
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.fwd(*args, n_threads=host_threads())
    dt = (time.perf_counter() - t0) / steps
    return sample.tokens / dt, dt


def run_reference_arm(a):
    """The CPU arm: oracle port of the reference numerics, all host threads, bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import flashkda_b200
    import oracle
    from flashkda_b200.synth import config
    w = config(a.workload)
    total_budget = 120.0  # seconds for the whole steps+warmup run
    per_step = max(0.5, min(a.cpu_seconds, total_budget / max(1, a.steps + a.warmup)))
    sample = cpu_sample_workload(w, per_step)
    tps, dt = time_oracle(sample, a.steps, a.warmup)
    cores = min(host_threads(), sample.H)  # one OpenMP task per (sequence, head) chain
    desc = f"1 sequence x T={sample.T} x H={sample.H} of {w.name} (B={w.B}, T={w.T}, H={w.H})"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if (a.scaling == "strong" and w.seq_lens is None and w.B % max(1, a.gpus) == 0) else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(w, a.algo or flashkda_b200.default_algo()),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_ours(a):
    import torch
    import torch.distributed as dist
    import flashkda_b200
    from flashkda_b200 import _lib
    from flashkda_b200.host import fwd_host
    from flashkda_b200.synth import (algorithmic_bytes, algorithmic_flops, config, make_inputs)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = config(a.workload)
    # One long sequence (cfg5) on several GPUs: context parallel, every rank holds T / N tokens
    # (strong scaling, one all-gather of the per-shard state maps per step).
    cp_mode = w.name == "cfg5" and world > 1
    # whether the ranks share ONE problem (value = its tokens / time) or each run their own copy
    strong = cp_mode or (a.scaling == "strong" and w.seq_lens is None and w.B % world == 0)
    if cp_mode:
        from flashkda_b200 import cp
        from flashkda_b200.synth import Workload
        w_local = Workload("cfg5-shard", 1, w.T // world // 16 * 16, w.H, lower_bound=w.lower_bound,
                           state_out=w.state_out)
        inp = make_inputs(w_local, device=dev, seed=rank)
        head = make_inputs(Workload("cfg5-params", 1, 16, w.H), device=dev, seed=w.seed)   # one set of per-head parameters
        inp["A_log"], inp["dt_bias"] = head["A_log"], head["dt_bias"]
    elif world > 1 and a.scaling == "strong" and w.seq_lens is None and w.B % world == 0:
        # one fixed problem: this rank takes B / N of its sequences (contiguous), no collective on the data path
        from flashkda_b200.synth import Workload, make_inputs_partition
        per = w.B // world
        w_local = Workload(w.name, per, w.T, w.H, lower_bound=w.lower_bound, state_in=w.state_in, state_out=w.state_out)
        inp = make_inputs_partition(w, rank * per, per, device=dev)
    elif world == 1 and w.seq_lens is None:
        from flashkda_b200.synth import make_inputs_partition
        w_local = w
        inp = make_inputs_partition(w, 0, w.B, device=dev)   # the same data as the partitioned runs
    else:
        w_local = w
        inp = make_inputs(w, device=dev, seed=rank)
    algo = a.algo or flashkda_b200.default_algo()
    ws_bytes = flashkda_b200.get_workspace_size(w_local.tokens, w.H, w_local.n_seqs, algo=algo)
    workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)

    validated = [False]

    def step(phase_mask=0):
        if a.seq_parts > 1 and not cp_mode:
            from flashkda_b200 import cp as _cp
            _cp.fwd_sequence_parallel(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                                      inp["A_log"], inp["dt_bias"], inp["lower_bound"], inp["initial_state"],
                                      inp["final_state"], parts=a.seq_parts)
            return
        if cp_mode:
            cp.fwd_context_parallel(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                                    inp["A_log"], inp["dt_bias"], inp["lower_bound"], None, inp["final_state"],
                                    parts=max(1, a.seq_parts), validate=not validated[0])
            validated[0] = True   # the ranks agree on their arguments in the first (warm-up) call only
            return
        flashkda_b200.fwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                          A_log=inp["A_log"], dt_bias=inp["dt_bias"], lower_bound=inp["lower_bound"],
                          initial_state=inp["initial_state"], final_state=inp["final_state"],
                          cu_seqlens=inp["cu_seqlens"], algo=algo, workspace=workspace, phase_mask=phase_mask,
                          flags=a.flags)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(a.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    if needs_l2_flush(w_local):
        # small workload: every step starts from a cold L2; each step has its own pair of events
        flush_buf = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
        pairs = []
        for _ in range(a.steps):
            flush_buf.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            pairs.append((e0, e1))
        barrier()
        ms_total = sum(x.elapsed_time(y) for x, y in pairs)
        del flush_buf
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            step()
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
    launches_per_step = flashkda_b200.last_launch_count()
    clocks = sampler.stop() if rank == 0 else None
    dev_status = flashkda_b200.device_status(workspace)
    assert dev_status == 0, f"device status {dev_status}: a kernel gave up on a bounded wait"
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / a.steps
    job_tokens = w.tokens if (strong and not cp_mode) else world * w_local.tokens   # tokens of the whole job per step
    value = job_tokens / (ms_step * 1e-3)

    # ---- each kernel of the forward alone (CUDA events on the launching stream); the slower one is
    #      the dominant kernel the roofline line describes ----
    # (the tensor-core recurrence has a one-chain-per-CTA variant that the launcher picks when there are no more
    #  (sequence, head) chains than SMs; otherwise the three-chains-per-CTA kernel runs)
    n_seqs = (len(inp["cu_seqlens"]) - 1) if inp.get("cu_seqlens") is not None else w_local.B
    wide = n_seqs * w.H <= torch.cuda.get_device_properties(dev).multi_processor_count
    names = {"twopass": ("fkda::prepare_warp_kernel", "fkda::recurrence_kernel")}.get(
        algo, ("fkda::prepare_warp_kernel", "fkda::recurrence_tc_wide_kernel" if wide else "fkda::recurrence_tc_ts_kernel"))
    kernel_times = {}
    n_phase = 3
    barrier()
    decode = w_local.T == 1 and inp.get("cu_seqlens") is None and algo != "twopass" and not (a.flags & 1)
    short = 2 <= w_local.T <= 16 and inp.get("cu_seqlens") is None and algo != "twopass" and not (a.flags & 8)
    if (decode or short) and not cp_mode and a.seq_parts == 1:
        # at most one chunk per sequence: the library runs ONE kernel (no phases to time apart)
        kernel_name, kernel_ms = ("fkda::decode_kernel" if decode else "fkda::short_kernel"), ms_step
        kernel_times[kernel_name] = ms_step
    elif not cp_mode and a.seq_parts == 1:
        step()
        for name, mask in zip(names, (_lib.PHASE_PREPARE, _lib.PHASE_RECURRENCE)):
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            step(mask)
            torch.cuda.synchronize(dev)
            p0.record()
            for _ in range(n_phase):
                step(mask)
            p1.record()
            torch.cuda.synchronize(dev)
            kernel_times[name] = p0.elapsed_time(p1) / n_phase
        step()  # leave the workspace and outputs consistent
        torch.cuda.synchronize(dev)
        kernel_name = max(kernel_times, key=kernel_times.get)
        kernel_ms = kernel_times[kernel_name]
    else:
        kernel_name = "whole step (several forward calls: sequence split / context parallel)"
        kernel_ms = ms_step

    # ---- context parallel: distance from the exact single-GPU run (optional) ----
    cp_check = None
    if cp_mode and a.cp_check:
        res = [None]
        if rank == world - 1:
            full = [make_inputs(w_local, device=dev, seed=r) for r in range(world)]
            cat = lambda key: torch.cat([f[key] for f in full], dim=1)
            q, k, v, g, beta = (cat(key) for key in ("q", "k", "v", "g", "beta"))
            del full
            out_x = torch.empty_like(v)
            hT_x = torch.zeros_like(inp["final_state"])
            flashkda_b200.fwd(q, k, v, g, beta, inp["scale"], out_x, A_log=inp["A_log"], dt_bias=inp["dt_bias"],
                              lower_bound=inp["lower_bound"], final_state=hT_x)
            torch.cuda.synchronize(dev)
            mine = out_x[:, rank * w_local.T:(rank + 1) * w_local.T].float()
            err = lambda ref, x: ((ref - x).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-8)).item()
            res[0] = {"state_ratio": err(hT_x.float(), inp["final_state"].float()),
                      "out_ratio_last_shard": err(mine, inp["out"].float()),
                      "out_max_abs_last_shard": (mine - inp["out"].float()).abs().max().item(),
                      "against": "one exact forward of all %d tokens on the last rank" % (w_local.T * world)}
            del q, k, v, g, beta, out_x
        dist.broadcast_object_list(res, src=world - 1)
        cp_check = res[0]

    # ---- end to end through the host-buffer API ----
    e2e = None
    if not a.no_e2e and not cp_mode:
        e2e = measure_e2e(a, w_local, inp, dev, world, algo, fwd_host, job_tokens)

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak_gbs, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak_gbs, peak_src = 6650.0, "fallback"
    # Roofline.  Headline: the WHOLE forward of this GPU (all its kernels back to back) on the algorithmic bytes
    # (q, k, v, g, beta read, out written, states in and out).  Beside it every kernel on its OWN bytes: what it must
    # read and write given the two-kernel split (the prepare kernel reads q, k, g, beta and writes the chunk
    # records; the recurrence reads the records and v, writes out, and moves the states).
    alg_bytes = algorithmic_bytes(w_local) * (world if cp_mode else 1)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    th = w_local.tokens * w.H
    units = ((w_local.tokens + 15) // 16) * w.H
    state_bytes = alg_bytes - th * 1282 if not cp_mode else 0
    rec = {"twopass": 13824}.get(algo, 14656)
    own = {"fkda::prepare_warp_kernel": th * 770 + units * rec,
           "fkda::decode_kernel": alg_bytes, "fkda::short_kernel": alg_bytes}
    for n in names[1:]:
        own[n] = units * rec + th * 512 + state_bytes
    tdb = json.load(open(os.path.join(ROOT, "profiles", "traffic.json"))) \
        if os.path.exists(os.path.join(ROOT, "profiles", "traffic.json")) else {}
    per_kernel, traffic = {}, 0.0
    for name, ms in kernel_times.items():
        entry = tdb.get(name, {})
        t_bytes = None
        if entry.get("bytes_per_unit") is not None:  # scaled from the small ncu capture by the (chunk, head) units
            t_bytes = entry["bytes_per_unit"] * units
        elif entry.get("traffic_over_algorithmic") is not None:  # state-bound kernels: scaled by the algorithmic bytes
            t_bytes = entry["traffic_over_algorithmic"] * alg_bytes
        traffic = None if (traffic is None or t_bytes is None) else traffic + t_bytes
        ob = own.get(name)
        per_kernel[name] = {"ms": ms, "own_bytes": ob, "achieved": None if ob is None else ob / (ms * 1e-3) / 1e9,
                            "frac": None if ob is None else ob / (ms * 1e-3) / 1e9 / peak_gbs, "traffic": t_bytes}
    if not kernel_times:
        traffic = None

    cpu = None
    if not a.no_cpu and world == 1:
        import oracle
        sample = cpu_sample_workload(w, a.cpu_seconds)
        tps, dt = time_oracle(sample, 1, 0)
        cpu = {"value": tps, "unit": UNIT, "cores": min(host_threads(), sample.H), "kind": "port",
               "sample": f"1 sequence x T={sample.T} x H={sample.H} of {w.name}, {dt:.1f} s"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": config_dict(w, algo, w_local.B,
                              "context parallel: T/N tokens per GPU, NCCL all-gather of per-shard state maps" if cp_mode
                              else ("one problem, B/N sequences per GPU (contiguous), no collective" if strong else None)),
        "tflops": job_tokens * w.H * (algorithmic_flops(w_local) / max(1, w_local.tokens * w.H)) / (ms_step * 1e-3) / 1e12,
        # per GPU: the forward of this rank's share (all kernels of a step) against the measured copy bandwidth
        "roofline": {"bound": "hbm", "kernel": "whole forward: " + " + ".join(k.split("::")[-1] for k in kernel_times)
                     if kernel_times else kernel_name,
                     "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                     "peak_source": peak_src, "traffic": traffic, "algorithmic_bytes_per_step": alg_bytes,
                     "slowest_kernel": kernel_name, "kernels": per_kernel},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * a.steps, "clocks": clocks,
    }
    if cp_mode:
        line["config"]["pieces_per_gpu"] = max(1, a.seq_parts)
        if cp_check is not None:
            line["cp_check"] = cp_check
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(a, w, inp, dev, world, algo, fwd_host, job_tokens):
    """Pinned host buffers -> device -> forward -> host, every step, through fwd_host."""
    import torch
    import torch.distributed as dist
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    names = ("q", "k", "v", "g", "beta", "out", "initial_state", "final_state")
    need = sum(inp[n].numel() * inp[n].element_size() for n in names if inp[n] is not None)
    ok = torch.tensor([1 if avail >= 2.5 * need * world else 0], dtype=torch.int32, device=dev)
    if world > 1:  # one decision for all ranks (they share the host's memory): a split decision would hang the barrier below
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        return {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "skipped": f"host memory too small to pin {need * world / 1e9:.1f} GB"}
    host = {}
    for n in names:
        if inp[n] is None:
            host[n] = None
            continue
        host[n] = torch.empty(inp[n].shape, dtype=inp[n].dtype, pin_memory=True)
        host[n].copy_(inp[n])
    A_h, dt_h = inp["A_log"].cpu().pin_memory(), inp["dt_bias"].cpu().pin_memory()
    cu_h = None if inp["cu_seqlens"] is None else inp["cu_seqlens"].cpu().pin_memory()
    torch.cuda.synchronize(dev)

    def one():
        return fwd_host(host["q"], host["k"], host["v"], host["g"], host["beta"], inp["scale"], host["out"], A_h,
                        dt_h, inp["lower_bound"], host["initial_state"], host["final_state"], cu_h, device=dev,
                        slab_sequences=1, algo=algo)

    one()  # warm-up (also allocates the staging buffers in the caching allocator)
    steps = max(1, min(a.steps, 3))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        h2d, d2h = one()  # returns after its own copy streams have been joined and synchronised
    ev1.record()
    torch.cuda.synchronize(dev)
    dt = ev0.elapsed_time(ev1) * 1e-3 / steps
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    del host
    return {"value": job_tokens / dt, "unit": UNIT, "h2d_bytes_per_step": int(h2d) * world,
            "d2h_bytes_per_step": int(d2h) * world, "ms_per_step": dt * 1e3, "steps": steps,
            "api": "flashkda_b200.host.fwd_host (pinned host tensors, per-sequence slabs, copy/compute overlap)"}


def main():
    a = parse()
    if a.impl == "reference":
        run_reference_arm(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
