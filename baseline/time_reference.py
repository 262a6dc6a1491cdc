#!/usr/bin/env python
"""Times the reference's own CUDA operator (built by ``baseline/build_reference.py``) beside this
repository's operator on one GPU: same tensors, same CUDA-event loop, same process.

    python baseline/time_reference.py [--out report.json] [--cases cfg2,cfg3,...]

Method (the reference's, benchmarks/bench_fwd.py:8-30): warm-up calls, then one pair of CUDA events per
timed call, mean and min over the calls; both operators go through their Python wrappers, so the
reference's per-call workspace allocation and beta transpose are inside its time, and this repository's
``fwd`` allocates its workspace per call as well (a second column gives it with a caller-held workspace).
Every shape is also timed with a 512 MB write between calls, outside the events ("cold L2").  Outputs of
the two operators are compared on every shape (bf16 mismatch fraction and error ratio).

Sizes: the reference builds its tensor maps from 32-bit element counts (csrc/smxx/fwd_launch.cu:50, 73-77:
``make_shape(H, T_total, D)`` and ``int(n_ht)`` with int operands), so the headline configuration is run at
B = 4 (2^30 elements per tensor) instead of B = 8 (2^31), and compared per token.
"""
import argparse
import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)

import flashkda_b200  # noqa: E402
from flashkda_b200.synth import Workload, config, make_inputs  # noqa: E402

CASES = {
    "cfg2": lambda: config("cfg2"),
    "cfg3": lambda: config("cfg3"),
    "cfg4_B4": lambda: Workload("cfg4_B4", 4, 32768, 64, lower_bound=-3.0, state_in="fp32", state_out="fp32"),
    "cfg4_B1": lambda: Workload("cfg4_B1", 1, 32768, 64, lower_bound=-3.0, state_in="fp32", state_out="fp32"),
    # the shapes of the reference's published tables (BENCHMARK_GB200.md:16-26): fp32 state in and out
    "T8192_H96_fixed": lambda: config("B=1,T=8192,H=96,state=fp32"),
    "T8192_H96_varlen6": lambda: config("H=96,lens=1300+547+2048+963+271+3063,state=fp32"),
    "T8192_H96_1024x8": lambda: config("H=96,lens=1024x8,state=fp32"),
    "T8192_H64_fixed": lambda: config("B=1,T=8192,H=64,state=fp32"),
    "T8192_H64_varlen6": lambda: config("H=64,lens=1300+547+2048+963+271+3063,state=fp32"),
    "T8192_H64_1024x8": lambda: config("H=64,lens=1024x8,state=fp32"),
}


def load_reference():
    so = os.path.join(HERE, "_ref", "flash_kda_C.so")
    if not os.path.exists(so):
        return None
    spec = importlib.util.spec_from_file_location("flash_kda_C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["flash_kda_C"] = mod
    # the reference's own wrapper (flash_kda/__init__.py), loaded under another name so that it does not
    # shadow this repository's top-level ``flash_kda`` module
    spec = importlib.util.spec_from_file_location("flash_kda_reference", os.path.join(HERE, "_ref", "flash_kda", "__init__.py"))
    wrap = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(wrap)
    return wrap.fwd


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in pairs]
    return {"mean_ms": sum(ms) / len(ms), "min_ms": min(ms)}


def err_ratio(ref, x):
    ref, x = ref.double().flatten(), x.double().flatten()
    return ((ref - x).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-8)).item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--cases", default=",".join(CASES))
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    a = ap.parse_args()
    ref_fwd = load_reference()
    dev = torch.device("cuda", 0)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    report = {"reference_built": ref_fwd is not None, "gpu": torch.cuda.get_device_name(0), "cases": {}}
    for name in a.cases.split(","):
        w = CASES[name]()
        inp = make_inputs(w, device=dev, seed=0)
        args = (inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"])
        kw = dict(A_log=inp["A_log"], dt_bias=inp["dt_bias"], lower_bound=inp["lower_bound"],
                  initial_state=inp["initial_state"], cu_seqlens=inp["cu_seqlens"])
        out_o, out_r = torch.zeros_like(inp["v"]), torch.zeros_like(inp["v"])
        hT_o = None if inp["final_state"] is None else torch.zeros_like(inp["final_state"])
        hT_r = None if inp["final_state"] is None else torch.zeros_like(inp["final_state"])
        ws = torch.empty(max(1, flashkda_b200.get_workspace_size(w.tokens, w.H, w.n_seqs)), dtype=torch.uint8, device=dev)
        big = w.tokens * w.H >= (1 << 22)
        iters, warm = (max(5, a.iters // 10), 3) if big else (a.iters, a.warmup)
        ours = lambda: flashkda_b200.fwd(*args, out_o, final_state=hT_o, **kw)
        ours_ws = lambda: flashkda_b200.fwd(*args, out_o, final_state=hT_o, workspace=ws, **kw)
        line = {"tokens": w.tokens, "H": w.H, "sequences": w.n_seqs}
        line["ours"] = {"warm": timed(ours, iters, warm, None), "cold_l2": timed(ours, iters, 2, flush)}
        line["ours_held_workspace"] = {"warm": timed(ours_ws, iters, warm, None), "cold_l2": timed(ours_ws, iters, 2, flush)}
        if ref_fwd is not None:
            with torch.inference_mode():
                ref = lambda: ref_fwd(*args, out_r, final_state=hT_r, **kw)
                line["reference"] = {"warm": timed(ref, iters, warm, None), "cold_l2": timed(ref, iters, 2, flush)}
            line["speedup_warm"] = line["reference"]["warm"]["mean_ms"] / line["ours"]["warm"]["mean_ms"]
            line["speedup_cold_l2"] = line["reference"]["cold_l2"]["mean_ms"] / line["ours"]["cold_l2"]["mean_ms"]
            line["parity_vs_reference_kernel"] = {
                "out_bf16_mismatch": (out_o != out_r).float().mean().item(), "out_ratio": err_ratio(out_r, out_o),
                "out_max_abs": (out_o.float() - out_r.float()).abs().max().item()}
            if hT_o is not None:
                line["parity_vs_reference_kernel"]["state_ratio"] = err_ratio(hT_r, hT_o)
                line["parity_vs_reference_kernel"]["state_mismatch"] = (hT_o != hT_r).float().mean().item()
        report["cases"][name] = line
        print(name, json.dumps(line), flush=True)
        del inp, args, kw, out_o, out_r, hT_o, hT_r, ws
        torch.cuda.empty_cache()
    if a.out:
        json.dump(report, open(a.out, "w"), indent=1)


if __name__ == "__main__":
    main()
