"""Golden outputs produced ON A GPU by the reference's own, unmodified ``tests/torch_ref.py``.

    python tests/golden/make_golden_gpu.py <dir holding torch_ref.py> <output dir> [--compare report.json]

``torch_ref.py`` needs a GPU (it JIT-compiles a ``tanh.approx`` kernel and calls cuBLAS with fp16
accumulation), so this script runs where one is available; its outputs are copied into
``tests/golden/gpu/`` and committed.  The reference's tests hold its CUDA kernel bit-equal to this
function (tests/test_fwd.py:260-261), which makes these files the reference's GPU results.  The file is
imported from the directory given on the command line (for example ``baseline/_ref/tests``, see
``baseline/build_reference.py``); it is never copied into tracked files.

The one adaptation is outside the file: ``ctypes.CDLL('libcublas.so')`` is redirected to the cuBLAS that
ships with the installed torch wheel, because the system-wide library of the CUDA toolkit image does not
load next to it.

Inputs come from fixed CPU seeds (``tests/kda_testlib.py``), so only outputs are stored:

  <case>.npz        the six small fixture cases of tests/golden/*.npz: full ``out`` and ``final_state``
  gate_<i>.npz      gate/bias stress sweep (T = 8192, H = 1): full ``final_state``, every 16th ``out`` row
  many_chains.npz   8 x 1024 tokens x 64 heads, fp32 states: ``out`` rows t % 256 == 255, states of every
                    32nd chain

With ``--compare`` the script also runs this repository's kernels (and the reference's CUDA extension when
``flash_kda_C.so`` sits next to the given directory's parent) on the same inputs and writes error ratios
and bf16 mismatch fractions against torch_ref, in full, to the given JSON file.
"""
import ctypes
import glob
import json
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import kda_testlib as K  # noqa: E402
from flashkda_b200.synth import make_inputs, to_device  # noqa: E402


def import_torch_ref(ref_tests_dir):
    real_cdll = ctypes.CDLL

    def cdll(name, *a, **kw):
        if name == "libcublas.so":
            import nvidia.cublas
            hits = sorted(glob.glob(os.path.join(list(nvidia.cublas.__path__)[0], "lib", "libcublas.so.*")))
            if hits:
                name = hits[0]
        return real_cdll(name, *a, **kw)

    ctypes.CDLL = cdll
    sys.path.insert(0, ref_tests_dir)
    try:
        import torch_ref
    finally:
        ctypes.CDLL = real_cdll
        sys.path.remove(ref_tests_dir)
    return torch_ref.torch_ref


def import_reference_extension(ref_root):
    """The reference's compiled operator (baseline/_ref/flash_kda_C.so), wrapped as its own
    flash_kda/__init__.py wraps it; None when it was not built."""
    so = os.path.join(ref_root, "flash_kda_C.so")
    if not os.path.exists(so):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("flash_kda_C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    def fwd(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
            cu_seqlens=None):
        B, T, H = q.shape[0], q.shape[1], q.shape[2]
        N = cu_seqlens.numel() - 1 if cu_seqlens is not None else B
        ws = torch.empty(mod.get_workspace_size(B * T, H, N), dtype=torch.uint8, device=q.device)
        mod.fwd(q, k, v, g, beta, float(scale), out, ws, A_log, dt_bias, lower_bound, initial_state=initial_state,
                final_state=final_state, cu_seqlens=cu_seqlens)
    return fwd


def bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def err_ratio(ref, x):
    ref, x = ref.double().flatten(), x.double().flatten()
    return ((ref - x).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-8)).item()


def run(fn, d, **kw):
    out = torch.zeros_like(d["v"])
    hT = None if d["final_state"] is None else torch.zeros_like(d["final_state"])
    h0 = None if d["initial_state"] is None else d["initial_state"].clone()
    fn(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], out, A_log=d["A_log"], dt_bias=d["dt_bias"],
       lower_bound=d["lower_bound"], initial_state=h0, final_state=hT, cu_seqlens=d["cu_seqlens"], **kw)
    torch.cuda.synchronize()
    return out, hT


def compare(ref_out, ref_hT, out, hT):
    r = {"out_max_abs": (ref_out.float() - out.float()).abs().max().item(), "out_ratio": err_ratio(ref_out, out),
         "out_bf16_mismatch": (ref_out != out).float().mean().item()}
    if ref_hT is not None:
        r["state_ratio"] = err_ratio(ref_hT, hT)
        r["state_mismatch"] = (ref_hT != hT).float().mean().item()
    return r


def main():
    ref_tests, out_dir = sys.argv[1], sys.argv[2]
    report_path = sys.argv[sys.argv.index("--compare") + 1] if "--compare" in sys.argv else None
    os.makedirs(out_dir, exist_ok=True)
    torch_ref = import_torch_ref(ref_tests)
    ours = ref_ext = None
    if report_path:
        import flashkda_b200
        ours = flashkda_b200.fwd
        ref_ext = import_reference_extension(os.path.dirname(os.path.abspath(ref_tests)))
    report = {}

    def one(name, inp, pack):
        d = to_device(inp, "cuda")
        t0 = time.time()
        with torch.inference_mode():
            ref_out, ref_hT = run(torch_ref, d)
        rec = pack(ref_out, ref_hT)
        rec["q_checksum"] = np.array(int(bits(inp["q"]).astype(np.uint64).sum()))
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **rec)
        line = {"torch_ref_seconds": time.time() - t0}
        if ours is not None:
            for algo in ("tc", "twopass"):
                line["ours_" + algo] = compare(ref_out, ref_hT, *run(ours, d, algo=algo))
        if ref_ext is not None:
            with torch.inference_mode():
                line["reference_kernel"] = compare(ref_out, ref_hT, *run(ref_ext, d))
        report[name] = line
        print(name, json.dumps(line), flush=True)

    def full(ref_out, ref_hT):
        rec = {"out": bits(ref_out)}
        if ref_hT is not None:
            rec["final_state"] = bits(ref_hT.to(torch.bfloat16))   # every exported value is bf16-representable
        return rec

    for name in K.GOLDEN_CASES:
        _, inp, _, _ = K.load_golden(name)
        one(name, inp, full)
    for i in range(len(K.GATE_CASE_NAMES)):
        one("gate_%d" % i, K.gate_case_inputs(i),
            lambda o, h: {"out": bits(o[:, 15::16]), "final_state": bits(h.to(torch.bfloat16))})
    w = K.MANY_CHAINS
    one(w.name, make_inputs(w, seed=77),
        lambda o, h: {"out": bits(o[:, K.MANY_CHAINS_OUT_EVERY - 1::K.MANY_CHAINS_OUT_EVERY]),
                      "final_state": bits(h.reshape(-1, 128, 128)[::K.MANY_CHAINS_STATE_EVERY].to(torch.bfloat16))})
    if report_path:
        json.dump(report, open(report_path, "w"), indent=1)


if __name__ == "__main__":
    main()
