"""Generate the golden fixtures in this directory from the reference's own torch_ref.

Run once, in a container that has the reference checkout, whose path is the one argument:

    python tests/golden/make_golden.py /path/to/reference

No reference source is copied: the text of ``tests/torch_ref.py`` is read from the
checkout and executed from its "Numeric helpers" section on (the part before that
JIT-compiles a CUDA kernel and opens cuBLAS, which needs a GPU).  Three
CPU stand-ins are injected for the GPU-only pieces it then calls:

  sigmoid_ext.sigmoid_tanh_fp32(x)      -> tanh(x/2)/2 + 1/2 in fp32
  matmul_fp16acc(a, b)                  -> (a.float() @ b.float()).half()
  torch.mm(a, b, out_dtype=float32)     -> a.float() @ b.float()

The outputs therefore follow every rounding point of the reference, with exact
instead of approximate ``tanh``.  Fixtures hold inputs and outputs as raw bit
patterns (bf16 as uint16) in compressed ``.npz`` files.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flashkda_b200.synth import Workload, config, make_inputs, make_reference_test_inputs  # noqa: E402


def load_torch_ref(ref_root: str):
    path = os.path.join(ref_root, "tests", "torch_ref.py")
    text = open(path).read()
    marker = "# Numeric helpers"
    start = text.rfind("# ====", 0, text.index(marker))
    body = text[start:]

    class TorchProxy:
        """Forwards to torch, except mm(..., out_dtype=) which has no CPU kernel."""

        def __getattr__(self, name):
            return getattr(torch, name)

        @staticmethod
        def mm(a, b, out_dtype=None):
            if out_dtype is None:
                return torch.mm(a, b)
            return (a.float() @ b.float()).to(out_dtype)

    sigmoid_ext = types.SimpleNamespace(
        sigmoid_tanh_fp32=lambda x: torch.tanh(x.float() * 0.5) * 0.5 + 0.5)
    ns = {"torch": TorchProxy(), "sigmoid_ext": sigmoid_ext,
          "matmul_fp16acc": lambda a, b: (a.float() @ b.float()).half()}
    exec(compile(body, path, "exec"), ns)
    return ns["torch_ref"]


def bits(t):
    if t is None:
        return None
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


# name -> (Workload, input style, store inputs?)
CASES = {
    # the benchmark's CPU-runnable configuration (inputs regenerated from the seed)
    "cfg1": (config("cfg1"), "bench", False),
    # ragged lengths incl. single-token sequences and tails of every residue class
    "varlen_small_bf16": (Workload("varlen_small_bf16", 1, 100, 2, state_in="bf16", state_out="bf16",
                                   seq_lens=[4, 8, 12, 1, 17, 1, 33, 24]), "reftest", True),
    "varlen_fp32_out_only": (Workload("varlen_fp32_out_only", 1, 115, 2, state_out="fp32",
                                      seq_lens=[17, 33, 65]), "reftest", True),
    "fixed_T37_stateless": (Workload("fixed_T37_stateless", 1, 37, 3), "reftest", True),
    "fixed_T64_fp32_inout": (Workload("fixed_T64_fp32_inout", 2, 64, 2, state_in="fp32", state_out="fp32"),
                             "reftest", True),
    "fixed_T97_bf16_in_only_lb3": (Workload("fixed_T97_bf16_in_only_lb3", 1, 97, 1, lower_bound=-3.0,
                                            state_in="bf16"), "bench", True),
}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference/checkout")
    ref_root = sys.argv[1]
    torch_ref = load_torch_ref(ref_root)
    torch.set_num_threads(os.cpu_count())
    for name, (w, style, store_inputs) in CASES.items():
        inp = make_inputs(w) if style == "bench" else make_reference_test_inputs(w)
        torch_ref(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["scale"], inp["out"],
                  A_log=inp["A_log"], dt_bias=inp["dt_bias"], lower_bound=inp["lower_bound"],
                  initial_state=None if inp["initial_state"] is None else inp["initial_state"].clone(),
                  final_state=inp["final_state"], cu_seqlens=inp["cu_seqlens"])
        rec = {"out": bits(inp["out"]), "style": np.array(style),
               "q_checksum": np.array(int(bits(inp["q"]).astype(np.uint64).sum()))}
        if inp["final_state"] is not None:
            # every exported state value is bf16-representable: store bf16 bits
            rec["final_state"] = bits(inp["final_state"].to(torch.bfloat16))
        if store_inputs:
            for key in ("q", "k", "v", "g", "beta", "A_log", "dt_bias"):
                rec["in_" + key] = bits(inp[key])
            if inp["initial_state"] is not None:
                rec["in_initial_state"] = bits(inp["initial_state"].to(torch.bfloat16))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **rec)
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
