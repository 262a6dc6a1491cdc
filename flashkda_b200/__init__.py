"""flashkda_b200: Kimi Delta Attention forward for NVIDIA B200 (sm_100a).

Host-side mirror of the reference operator API (``flash_kda/__init__.py:5-41`` and the
checks of ``csrc/flash_kda.cpp:44-174`` in the reference project): the same ``fwd``
signature, argument meaning and error conditions, on top of a C-ABI CUDA library
(``include/flashkda_b200.h``).  There is no CPU path: calling ``fwd`` without the built
library or without CUDA tensors raises.
"""
import os

import torch

from . import _lib

__all__ = ["fwd", "get_workspace_size", "last_launch_count", "default_algo", "device_status", "chunk_states_slots"]

D = 128
_ENV_ALGO = "FLASHKDA_B200_ALGO"


def default_algo() -> str:
    return os.environ.get(_ENV_ALGO, "auto")


def get_workspace_size(T_total: int, H: int, N: int = 1, algo: str = None) -> int:
    """Scratch bytes one ``fwd`` call allocates (reference: ``get_workspace_size``,
    csrc/flash_kda.cpp:5-26)."""
    a = _lib.ALGOS[algo or default_algo()]
    return int(_lib.lib().fkda_workspace_bytes(int(T_total), int(H), int(N), a))


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def fwd(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
        cu_seqlens=None, *, algo: str = None, workspace: torch.Tensor = None, phase_mask: int = 0, flags: int = 0,
        chunk_states: torch.Tensor = None, chunk_states_every: int = 4):
    """FlashKDA forward; writes ``out`` (and ``final_state``) in place and returns ``None``.

    q, k, v, g, out: bf16 ``[B, T, H, 128]``; beta: bf16 ``[B, T, H]`` logits; A_log: fp32
    ``[H]``; dt_bias: fp32 ``[H, 128]``; states: bf16 or fp32 ``[N, H, 128, 128]`` (``[V, K]``
    layout); cu_seqlens: int64 ``[N + 1]`` (then ``B`` must be 1).  Work is enqueued on the
    current CUDA stream of ``q.device`` without synchronising.

    ``algo`` and ``workspace`` are additions to the reference signature: the implementation
    selector (default from ``$FLASHKDA_B200_ALGO`` or "auto") and an optional caller-owned
    uint8 scratch tensor of at least ``get_workspace_size(...)`` bytes.  ``phase_mask`` is a
    measurement aid (see ``fkda_fwd_params.phase_mask``) and ``flags`` selects kernel variants for tests
    (``fkda_fwd_params.flags``); leave both 0.

    ``chunk_states`` (optional, bf16 ``[slots, H, 128, 128]``) receives the state of every sequence before each
    group of ``chunk_states_every`` 16-token chunks (``chunk_states_slots`` gives the slot count); with the default
    of 4 these are the states FLA's ``chunk_kda`` returns as ``h`` for ``return_intermediate_states=True``.

    The call returns without synchronising, so it cannot tell whether a kernel gave up on one of its
    bounded internal waits (possible only when other long-running kernels hold the GPU's SMs for
    seconds); ``device_status(workspace)`` reports that after the stream has been synchronised.
    """
    bf16 = torch.bfloat16
    big = (q, k, v, g, beta, out)
    _check(all(t.is_cuda for t in big), "all tensors must be on CUDA")
    _check(all(t.is_contiguous() for t in big), "all tensors must be contiguous")
    for name, t in zip("q k v g beta out".split(), big):
        _check(t.dtype == bf16, f"{name} must be bfloat16")
    state_fp32 = False
    if initial_state is not None:
        _check(initial_state.is_cuda and initial_state.is_contiguous(), "initial_state must be contiguous CUDA tensor")
        _check(initial_state.dtype in (bf16, torch.float32), "initial_state must be bfloat16 or float32")
        state_fp32 |= initial_state.dtype == torch.float32
    if final_state is not None:
        _check(final_state.is_cuda and final_state.is_contiguous(), "final_state must be contiguous CUDA tensor")
        _check(final_state.dtype in (bf16, torch.float32), "final_state must be bfloat16 or float32")
        state_fp32 |= final_state.dtype == torch.float32
    if initial_state is not None and final_state is not None:
        _check(initial_state.dtype == final_state.dtype, "initial_state and final_state must have the same dtype")
    _check(A_log.is_cuda and A_log.is_contiguous(), "A_log must be contiguous CUDA tensor")
    _check(A_log.dtype == torch.float32, "A_log must be float32")
    _check(dt_bias.is_cuda and dt_bias.is_contiguous(), "dt_bias must be contiguous CUDA tensor")
    _check(dt_bias.dtype == torch.float32, "dt_bias must be float32")
    for name, t in zip("q k v g".split(), (q, k, v, g)):
        _check(t.dim() == 4, f"{name} must be [B, T, H, D]")
    _check(beta.dim() == 3, "beta must be [B, T, H]")
    _check(out.dim() == 4, "out must be [B, T, H, D]")
    B, T, H, Dd = q.shape
    _check(k.shape == q.shape, "k must match q shape")
    _check(v.shape == q.shape, "v must match q shape")
    _check(g.shape == q.shape, "g must match q shape")
    _check(out.shape == q.shape, "out must match q shape")
    _check(tuple(beta.shape) == (B, T, H), "beta must be [B, T, H] matching q")
    _check(A_log.dim() == 1 and A_log.shape[0] == H, "A_log must be [H]")
    _check(dt_bias.dim() == 2 and tuple(dt_bias.shape) == (H, Dd), "dt_bias must be [H, D]")
    _check(Dd == D, "currently only supports D == 128")
    lower_bound = float(lower_bound)
    _check(-5.0 <= lower_bound <= 0.0, "lower_bound must be in [-5.0, 0]")
    dev = q.device
    _check(all(t.device == dev for t in (k, v, g, beta, out, A_log, dt_bias)), "all tensors must be on the same device")
    if cu_seqlens is not None:
        _check(B == 1, "B must be 1 when cu_seqlens is provided")
        _check(cu_seqlens.is_cuda, "cu_seqlens must be on CUDA")
        _check(cu_seqlens.dtype == torch.int64, "cu_seqlens must be int64")
        _check(cu_seqlens.dim() == 1, "cu_seqlens must be 1D")
        N = cu_seqlens.numel() - 1
        _check(N > 0, "cu_seqlens must have at least 2 elements")
        _check(cu_seqlens.is_contiguous(), "cu_seqlens must be contiguous")
    else:
        N = B
    for name, s in (("initial_state", initial_state), ("final_state", final_state)):
        if s is not None:
            _check(s.dim() == 4 and tuple(s.shape) == (N, H, D, D), f"{name} must be [N, H, D, D]")
            _check(s.device == dev, f"{name} must be on the same device as q")

    if chunk_states is not None:
        _check(chunk_states.is_cuda and chunk_states.is_contiguous() and chunk_states.dtype == bf16,
               "chunk_states must be a contiguous CUDA bfloat16 tensor")
        _check(int(chunk_states_every) >= 1, "chunk_states_every must be >= 1")
        _check(cu_seqlens is not None or chunk_states.numel() == chunk_states_slots(B, T, chunk_states_every) * H * D * D,
               "chunk_states must hold B * ceil(T / (16 * every)) slots of [H, 128, 128]")

    L = _lib.lib()
    algo_id = _lib.ALGOS[algo or default_algo()]
    T_total = B * T
    if T_total == 0 and final_state is None:
        return None
    ptr = lambda t: None if t is None else t.data_ptr()
    p = _lib.FwdParams(
        q=ptr(q), k=ptr(k), v=ptr(v), g=ptr(g), beta=ptr(beta), out=ptr(out), A_log=ptr(A_log), dt_bias=ptr(dt_bias),
        initial_state=ptr(initial_state), final_state=ptr(final_state),
        state_dtype=_lib.FKDA_STATE_FP32 if state_fp32 else _lib.FKDA_STATE_BF16, algo=algo_id,
        cu_seqlens=ptr(cu_seqlens), B=B, T=T, H=H, N=N, token_stride=H * D, beta_token_stride=H,
        scale=float(scale), lower_bound=lower_bound, workspace=None, workspace_bytes=0,
        phase_mask=int(phase_mask), flags=int(flags), chunk_states=ptr(chunk_states),
        chunk_states_every=int(chunk_states_every) if chunk_states is not None else 0)
    with torch.cuda.device(dev):
        need = int(L.fkda_workspace_bytes_for(p))  # what this call's path needs (a decode step: 256 bytes)
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    else:
        _check(workspace.is_cuda and workspace.is_contiguous() and workspace.dtype == torch.uint8
               and workspace.numel() >= need, "workspace must be a contiguous CUDA uint8 tensor of sufficient size")
    p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = L.fkda_fwd(p, stream)
    if rc != 0:
        raise RuntimeError(f"fkda_fwd failed: {_lib.status_string(rc)} (status {rc})")
    # `workspace` was allocated on (or handed over for) the current stream, so the caching allocator
    # reuses it in stream order once this reference is dropped
    return None


def chunk_states_slots(B: int, T: int, every: int = 4, seq_lens=None) -> int:
    """Slots a ``chunk_states`` tensor needs: per sequence ``ceil(len / (16 * every))``; pass the lengths of a
    ragged batch as ``seq_lens``."""
    group = 16 * int(every)
    if seq_lens is not None:
        return int(sum((int(x) + group - 1) // group for x in seq_lens))
    return int(B) * ((int(T) + group - 1) // group)


def device_status(workspace: torch.Tensor) -> int:
    """Synchronises the current stream and returns the device status word of the last call that used
    ``workspace`` (0 = ok; see ``fkda_device_status``)."""
    with torch.cuda.device(workspace.device):
        stream = torch.cuda.current_stream(workspace.device).cuda_stream
        return int(_lib.lib().fkda_device_status(workspace.data_ptr(), stream))


def last_launch_count() -> int:
    """Kernels launched by the last successful ``fwd`` on this thread."""
    return int(_lib.lib().fkda_last_launch_count())
