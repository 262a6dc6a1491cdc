"""Parity against results the reference itself produced on a GPU.

``tests/golden/gpu/*.npz`` hold the outputs of the reference's unmodified ``tests/torch_ref.py`` run on a
B200 (generator: ``tests/golden/make_golden_gpu.py``); the reference's own tests require its CUDA kernel to
equal that function bit for bit (tests/test_fwd.py:260-261), and the generator's comparison run found the
reference's sm_100a binary equal to it on every one of these cases.  Unlike the CPU oracle, torch_ref on a
GPU uses the same approximate transcendental instructions as the kernels, so there is no modelling gap.

Bars:
  * default tensor-core path: ``torch.equal`` on ``out`` and ``final_state`` -- it issues the reference's
    contractions in the reference's order and reproduced these files bit for bit when they were made; that is
    well inside the stated target (out max-abs 2e-2, final_state 1e-3 relative), which is asserted as well so
    that a failure message says how far off a regression is;
  * CUDA-core path (algo "twopass", kept as the easy-to-audit implementation): sequential fp32 FMA chains
    instead of tensor-core accumulation order; within out max-abs 2e-2 everywhere and within 1e-3 on the state
    except under the saturated gates of the stress sweep (measured up to 3.8e-3 there), bound 6e-3;
  * CPU oracle (no GPU needed): exact tanh/exp2 against the approximate instructions; measured up to 1.3e-3
    on ``out`` and 5.3e-4 on the state for ordinary inputs, up to 9.0e-3 on the state under saturated gates.
    This is why the suite's GPU-vs-CPU-oracle bound is 1e-2 while the GPU-vs-reference bound is equality.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from flashkda_b200.synth import make_inputs
import kda_testlib as K

GPU_DIR = os.path.join(K.GOLDEN_DIR, "gpu")
STATE_RATIO = 1e-3      # the stated target, against the reference's GPU results
OUT_MAX_ABS = 2e-2


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_case(name):
    """(inputs on the CPU, selector of the stored ``out`` rows, selector of the stored states, golden out,
    golden state as bf16 or None)."""
    z = np.load(os.path.join(GPU_DIR, name + ".npz"))
    if name in K.GOLDEN_CASES:
        _, inp, _, _ = K.load_golden(name)
        sel_out, sel_state = (lambda o: o), (lambda h: h)
    elif name.startswith("gate_"):
        inp = K.gate_case_inputs(int(name.split("_")[1]))
        sel_out, sel_state = (lambda o: o[:, 15::16]), (lambda h: h)
    else:
        inp = make_inputs(K.MANY_CHAINS, seed=77)
        sel_out = lambda o: o[:, K.MANY_CHAINS_OUT_EVERY - 1::K.MANY_CHAINS_OUT_EVERY]
        sel_state = lambda h: h.reshape(-1, 128, 128)[::K.MANY_CHAINS_STATE_EVERY]
    chk = int(inp["q"].contiguous().view(torch.int16).numpy().view(np.uint16).astype(np.uint64).sum())
    assert chk == int(z["q_checksum"]), "seeded input generation drifted from the fixture"
    gold_out = _bf16(z["out"])
    gold_state = _bf16(z["final_state"]) if "final_state" in z.files else None
    return inp, sel_out, sel_state, gold_out, gold_state


SMALL = list(K.GOLDEN_CASES)
GATES = ["gate_%d" % i for i in range(len(K.GATE_CASE_NAMES))]


@pytest.mark.parametrize("name", SMALL + GATES)
def test_cpu_oracle_against_reference_gpu_results(name):
    inp, sel_out, sel_state, gold_out, gold_state = load_case(name)
    out, hT = K.run_oracle(inp)
    out = sel_out(out)
    scale = max(1.0, gold_out.float().abs().max().item())
    assert oracle.max_abs(gold_out, out) <= OUT_MAX_ABS * scale
    assert oracle.err_ratio(gold_out.float(), out.float()) <= 6e-3
    if gold_state is not None:
        got = sel_state(hT).float()
        assert oracle.err_ratio(gold_state.float().reshape(got.shape), got) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("name", SMALL + GATES + ["many_chains"])
@pytest.mark.parametrize("algo", ["tc", "twopass"])
def test_kernels_against_reference_gpu_results(name, algo):
    from test_gpu_parity import run_gpu
    inp, sel_out, sel_state, gold_out, gold_state = load_case(name)
    out, hT = run_gpu(inp, algo)
    out = sel_out(out)
    scale = max(1.0, gold_out.float().abs().max().item())
    d_out = oracle.max_abs(gold_out, out)
    mism = (gold_out.reshape(out.shape) != out).float().mean().item()
    r_state = None
    if gold_state is not None:
        got = sel_state(hT).float()
        gold = gold_state.float().reshape(got.shape)
        r_state = oracle.err_ratio(gold, got)
    print(f"{name}/{algo}: out max-abs {d_out:.3e}, bf16 mismatch {mism:.3e}, state ratio {r_state}")
    assert d_out <= OUT_MAX_ABS * scale
    if algo == "tc":
        if r_state is not None:
            assert r_state <= STATE_RATIO
            assert torch.equal(gold, got), f"final_state differs from the reference's GPU result (ratio {r_state:.3e})"
        assert torch.equal(gold_out.reshape(out.shape), out), f"out differs from the reference's GPU result ({mism:.3e})"
    elif r_state is not None:
        assert r_state <= (6e-3 if name.startswith("gate_") else STATE_RATIO)


@pytest.mark.gpu
@pytest.mark.parametrize("index", range(len(K.GATE_CASE_NAMES)))
def test_gate_sweep_against_fp64_recurrence(index):
    """The reference's accuracy test (tests/test_fwd.py:315-363): T = 8192, H = 1, ten gate/bias fillings,
    against a token-by-token float64 recurrence; its bar is 0.005 on ``out`` (RMSE ratio), the state is
    reported (the reference only warns on it; its published figures are 3.1e-3 .. 9.8e-3)."""
    from test_gpu_parity import run_gpu
    from flashkda_b200.synth import to_device
    inp = K.gate_case_inputs(index)
    out, hT = run_gpu(inp, "tc")
    gold_out, gold_state = K.fp64_recurrence(to_device(inp, "cuda"))
    r_out = oracle.err_ratio(gold_out.float().cpu(), out.float())
    r_state = oracle.err_ratio(gold_state.float().cpu(), hT.float())
    print(f"{K.GATE_CASE_NAMES[index]}: out ratio {r_out:.3e}, state ratio {r_state:.3e} vs fp64")
    assert r_out <= 5e-3
    assert r_state <= 2e-2
