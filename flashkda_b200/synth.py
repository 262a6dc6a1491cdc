"""Seeded synthetic inputs for the KDA forward pass.

The reference benchmarks and tests on random tensors only
(benchmarks/bench_fwd.py:53-61, tests/test_fwd_full.py:26-44); there is no
dataset.  ``make_inputs`` produces tensors with the shapes, dtypes and value
distributions of the benchmark configurations; ``make_reference_test_inputs``
reproduces the distribution the reference's own unit tests use (pre-normalised
q/k, uniform A_log/dt_bias, ``arange`` state).
"""
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

D = 128


@dataclass
class Workload:
    """One forward-pass problem: shapes, gate bound, state options, sequence lengths."""
    name: str
    B: int
    T: int
    H: int
    lower_bound: float = -5.0
    state_in: Optional[str] = None      # None | "bf16" | "fp32"
    state_out: Optional[str] = None
    seq_lens: Optional[List[int]] = None  # varlen: B must be 1 and sum == T
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def n_seqs(self) -> int:
        return len(self.seq_lens) if self.seq_lens is not None else self.B

    @property
    def tokens(self) -> int:
        return self.B * self.T


def varlen_lengths(n: int = 64, max_len: int = 4096, seed: int = 0) -> List[int]:
    """Sequence lengths for the ragged batch: ``n`` draws from U[1, max_len], then at
    least three forced to 1 and at least eight to non-multiples of 16."""
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_len + 1, (n,), generator=gen).tolist()
    for i in (3, 17, 40):
        lens[i % n] = 1
    fixed = 0
    for i in range(n):
        if fixed >= 8:
            break
        if lens[i] > 1 and lens[i] % 16 == 0:
            lens[i] += 5
            fixed += 1
    odd = sum(1 for x in lens if x % 16)
    i = 0
    while odd < 8 and i < n:
        if lens[i] % 16 == 0:
            lens[i] += 3
            odd += 1
        i += 1
    return lens


def _parse_lens(txt: str) -> List[int]:
    """``"1300+547+2048"`` or ``"1024x8"`` (eight sequences of 1024 tokens)."""
    txt = txt.replace("x", "*")
    if "*" in txt:
        length, count = txt.split("*")
        return [int(length)] * int(count)
    return [int(x) for x in txt.split("+")]


def config(name: str) -> Workload:
    """The five benchmark configurations, by short name."""
    if name == "cfg1":   # CPU-runnable case
        return Workload("cfg1", B=2, T=256, H=4, lower_bound=-5.0, state_in="fp32", state_out="fp32")
    if name == "cfg2":   # single-GPU dense prefill, stateless
        return Workload("cfg2", B=1, T=8192, H=32, lower_bound=-5.0)
    if name == "cfg3":   # ragged batch of 64 sequences, bf16 state
        lens = varlen_lengths()
        return Workload("cfg3", B=1, T=sum(lens), H=32, lower_bound=-5.0, state_in="bf16", state_out="bf16",
                        seq_lens=lens)
    if name == "cfg4":   # headline throughput case
        return Workload("cfg4", B=8, T=32768, H=64, lower_bound=-3.0, state_in="fp32", state_out="fp32")
    if name == "cfg5":   # one long sequence (context-parallel case)
        return Workload("cfg5", B=1, T=1048576, H=32, lower_bound=-5.0, state_out="fp32")
    if "=" in name:      # ad-hoc shape, e.g. "B=1,T=4096,H=444,state=fp32,lb=-5" or "H=64,lens=1300+547+2048,state=fp32"
        kv = dict(item.split("=") for item in name.split(","))
        st = kv.get("state")
        if "lens" in kv:  # ragged batch: B = 1, T = total tokens
            lens = _parse_lens(kv["lens"])
            return Workload(name, B=1, T=sum(lens), H=int(kv["H"]), lower_bound=float(kv.get("lb", -5.0)),
                            state_in=st, state_out=st, seq_lens=lens)
        return Workload(name, B=int(kv.get("B", 1)), T=int(kv["T"]), H=int(kv["H"]),
                        lower_bound=float(kv.get("lb", -5.0)), state_in=st, state_out=st)
    raise KeyError(name)


_DT = {"bf16": torch.bfloat16, "fp32": torch.float32}


def make_inputs(w: Workload, device="cpu", seed: Optional[int] = None):
    """Benchmark-style inputs: q,k,v,g ~ N(0,1) bf16 (q,k NOT pre-normalised), beta logits
    ~ N(0,1) bf16, A_log = log U[1,16], dt_bias ~ N(0,0.1), state ~ N(0,0.05)."""
    seed = w.seed if seed is None else seed
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    shp = (w.B, w.T, w.H, D)

    def randn_bf16(shape):
        # generated in bf16 directly on the target device: no fp32 staging copy of multi-GB tensors
        return torch.randn(shape, dtype=torch.bfloat16, device=dev, generator=gen)

    q, k, v, g = (randn_bf16(shp) for _ in range(4))
    beta = randn_bf16((w.B, w.T, w.H))
    A_log = torch.log(torch.empty(w.H, dtype=torch.float32, device=dev).uniform_(1.0, 16.0, generator=gen))
    dt_bias = torch.randn(w.H, D, dtype=torch.float32, device=dev, generator=gen) * 0.1
    n = w.n_seqs
    h0 = None
    if w.state_in is not None:
        h0 = (torch.randn(n, w.H, D, D, dtype=torch.float32, device=dev, generator=gen) * 0.05).to(_DT[w.state_in])
    hT = torch.zeros(n, w.H, D, D, dtype=_DT[w.state_out], device=dev) if w.state_out is not None else None
    cu = None
    if w.seq_lens is not None:
        assert w.B == 1 and sum(w.seq_lens) == w.T
        cu = torch.tensor([0] + list(torch.tensor(w.seq_lens).cumsum(0).tolist()), dtype=torch.int64, device=dev)
    return dict(q=q, k=k, v=v, g=g, beta=beta, scale=1.0 / math.sqrt(D), out=torch.zeros_like(v), A_log=A_log,
                dt_bias=dt_bias, lower_bound=w.lower_bound, initial_state=h0, final_state=hT, cu_seqlens=cu)


def make_inputs_partition(w: Workload, first: int, count: int, device="cpu"):
    """Sequences ``first .. first + count - 1`` of the fixed batch ``w`` (one rank's share when the batch is
    partitioned over GPUs).  Every sequence comes from its own seed (``w.seed + 1 + index``) and the per-head
    parameters from ``w.seed``, so any partition of the batch yields the same data."""
    assert w.seq_lens is None and 0 <= first and first + count <= w.B
    one = Workload(w.name, 1, w.T, w.H, lower_bound=w.lower_bound, state_in=w.state_in, state_out=w.state_out)
    parts = [make_inputs(one, device=device, seed=w.seed + 1 + first + i) for i in range(count)]
    head = make_inputs(Workload(w.name, 1, 16, w.H), device=device, seed=w.seed)
    cat = lambda key: None if parts[0][key] is None else torch.cat([p.pop(key) for p in parts], dim=0)
    out = {key: cat(key) for key in ("q", "k", "v", "g", "beta", "out", "initial_state", "final_state")}
    out.update(scale=head["scale"], A_log=head["A_log"], dt_bias=head["dt_bias"], lower_bound=w.lower_bound,
               cu_seqlens=None)
    return out


def make_reference_test_inputs(w: Workload, device="cpu", seed: int = 42):
    """Inputs in the style of the reference's unit tests (tests/test_fwd_full.py:26-44):
    L2-normalised q/k, randn v/g/beta, U[0,1) A_log and dt_bias, arange-valued state."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    shp = (w.B, w.T, w.H, D)
    F = torch.nn.functional
    q = F.normalize(torch.randn(shp, dtype=torch.float32, device=dev, generator=gen), p=2, dim=-1).to(torch.bfloat16)
    k = F.normalize(torch.randn(shp, dtype=torch.float32, device=dev, generator=gen), p=2, dim=-1).to(torch.bfloat16)
    v = torch.randn(shp, dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16)
    g = torch.randn(shp, dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16)
    beta = torch.randn((w.B, w.T, w.H), dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16)
    A_log = torch.rand(w.H, dtype=torch.float32, device=dev, generator=gen)
    dt_bias = torch.rand(w.H, D, dtype=torch.float32, device=dev, generator=gen)
    n = w.n_seqs
    h0 = None
    if w.state_in is not None:
        h0 = torch.arange(n * w.H * D * D, dtype=torch.float32, device=dev).reshape(n, w.H, D, D) \
            .to(torch.bfloat16).to(_DT[w.state_in])
    hT = torch.zeros(n, w.H, D, D, dtype=_DT[w.state_out], device=dev) if w.state_out is not None else None
    cu = None
    if w.seq_lens is not None:
        assert w.B == 1 and sum(w.seq_lens) == w.T
        cu = torch.tensor([0] + list(torch.tensor(w.seq_lens).cumsum(0).tolist()), dtype=torch.int64, device=dev)
    return dict(q=q, k=k, v=v, g=g, beta=beta, scale=1.0 / math.sqrt(D), out=torch.zeros_like(v), A_log=A_log,
                dt_bias=dt_bias, lower_bound=w.lower_bound, initial_state=h0, final_state=hT, cu_seqlens=cu)


def to_device(inp: dict, device) -> dict:
    """Copy every tensor of an input dict to ``device`` (fresh output buffers)."""
    o = {}
    for key, val in inp.items():
        o[key] = val.to(device).clone() if torch.is_tensor(val) else val
    return o


# Algorithmic cost model: per token and head, 4 input rows + 1 output row of 128 bf16 and one
# beta scalar; FLOPs of the chunk-16 formulation (two 16x16x128 products, the 16x16 inverse,
# two state contractions, two 16x16x128 applications, the rank-16 state update).
BYTES_PER_TOKEN_HEAD = 4 * 256 + 2 + 256
FLOPS_PER_TOKEN_HEAD = 117760


def algorithmic_bytes(w: Workload) -> int:
    b = w.tokens * w.H * BYTES_PER_TOKEN_HEAD
    for s in (w.state_in, w.state_out):
        if s is not None:
            b += w.n_seqs * w.H * D * D * (2 if s == "bf16" else 4)
    return b


def algorithmic_flops(w: Workload) -> int:
    return w.tokens * w.H * FLOPS_PER_TOKEN_HEAD
