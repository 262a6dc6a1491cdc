"""A flash-linear-attention backend for ``chunk_kda`` that also serves the two options FLA's stock FlashKDA
backend declines: ``return_intermediate_states`` and ``cp_context``.

FLA picks this repository up as the reference operator without any of this: its own ``FlashKDABackend``
imports the top-level module ``flash_kda`` (fla/ops/kda/backends/flashkda.py:90-151), which this repository
provides.  That backend, however, refuses context parallelism and intermediate states before it ever reaches
``flash_kda.fwd`` (flashkda.py:82-85), because the reference operator has neither.  ``register()`` adds a second
backend, tried before the stock one, that accepts the same calls plus those two:

  * ``return_intermediate_states=True``: the kernels export the state of every sequence before each 64-token
    chunk (``chunk_states`` of ``flashkda_b200.fwd``), FLA's ``h`` of shape ``[B, NT, H, 128, 128]``, bf16;
  * ``cp_context``: FLA's context-parallel convention (fla/ops/cp/context.py): the packed tokens are cut into
    equal parts, one per rank; a rank's first sequence may continue one that started on earlier ranks
    (``pre_num_ranks``) and its last may continue on later ranks (``post_num_ranks``).  Every rank that hands a
    sequence on computes the affine map (M, N) of its last local sequence piece, one all-gather moves the maps,
    and a rank folds the maps of the ranks its first sequence came through into that sequence's initial state
    (see ``flashkda_b200.cp``).

Usage::

    import flashkda_b200.fla_backend as fb
    fb.register()            # once per process, before calling fla.ops.kda.chunk_kda
"""
from __future__ import annotations

import torch

D = 128
_CHUNK_STATES_EVERY = 4   # FLA's intermediate states are taken every 64 tokens = 4 chunks of 16


def _stock_checks(q, v, use_gate_in_kernel, use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel,
                  transpose_state_layout, safe_gate):
    """The conditions of FLA's stock FlashKDA verifier that describe the operator itself."""
    if torch.is_grad_enabled():
        return "inference mode only"
    if q.dtype != torch.bfloat16:
        return f"requires bfloat16, got {q.dtype}"
    if q.shape[-1] != D or v.shape[-1] != D:
        return "requires K = V = 128"
    if v.shape[2] != q.shape[2]:
        return "grouped value heads are not supported"
    if not (use_gate_in_kernel and use_qk_l2norm_in_kernel and use_beta_sigmoid_in_kernel):
        return "requires the gate, the q/k L2 norm and the beta sigmoid in the kernel"
    if not transpose_state_layout:
        return "requires transpose_state_layout=True"
    if not safe_gate:
        return "requires safe_gate=True"
    return None


def fwd_fla_context_parallel(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, cp_context, fwd_fn=None):
    """Forward of this rank's part of a packed batch under FLA's context-parallel convention.

    ``q .. out`` hold this rank's tokens (``[1, T_local, H, 128]``); ``cp_context`` carries the local
    ``cu_seqlens``, the process group and how many ranks the first / last local sequence came from / goes on to.
    No initial or final states (FLA's contract for context parallelism).  ``fwd_fn`` (tests: the CPU oracle)
    replaces the device operator; it is called with the reference signature."""
    import torch.distributed as dist
    from . import cp
    if fwd_fn is None:
        from . import fwd as fwd_fn
    group = cp_context.group
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    dev, H = q.device, q.shape[2]
    cu = cp_context.cu_seqlens.to(device=dev, dtype=torch.int64)
    cu_host = (cp_context.cu_seqlens_cpu if cp_context.cu_seqlens_cpu is not None else cp_context.cu_seqlens.cpu()).tolist()
    n_local = len(cu_host) - 1
    pre, post = int(cp_context.pre_num_ranks or 0), int(cp_context.post_num_ranks or 0)

    # 1. the map of my last local sequence piece, if the sequence goes on to later ranks
    payload = torch.zeros(2, 1, H, D, D, dtype=torch.float32, device=dev)
    if post > 0 and n_local > 0:
        a, b = int(cu_host[-2]), int(cu_host[-1])
        sl = lambda x: x[:, a:b]
        M, N = cp.shard_maps(fwd_fn, sl(q), sl(k), sl(v), sl(g), sl(beta), scale, A_log, dt_bias, lower_bound,
                             need_transition=pre > 0 and n_local == 1)   # M only matters when the piece has a past
        if M is not None:
            payload[0].copy_(M)
        payload[1].copy_(N)
    # 2. exchange
    gathered = [torch.empty_like(payload) for _ in range(world)]
    dist.all_gather(gathered, payload, group=group)
    # 3. the state my first sequence arrives with: the rank where it started contributes N (it started from zero
    #    there), every rank in between its whole shard's (M, N)
    h0 = None
    if n_local > 0:
        h0 = torch.zeros(n_local, H, D, D, dtype=torch.float32, device=dev)
        if pre > 0:
            S = gathered[rank - pre][1]
            for j in range(rank - pre + 1, rank):
                S = cp.fold(S, gathered[j][0], gathered[j][1])
            h0[0] = S[0]
    # 4. my tokens, for real
    if n_local > 0:
        fwd_fn(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, h0, None, cu)
    return out


def _make_backend():
    from fla.ops.backends import BaseBackend

    class FlashKDAB200Backend(BaseBackend):
        """flashkda_b200 behind ``fla.ops.kda.chunk_kda``, including intermediate states and context parallelism."""

        backend_type = "flashkda_b200"
        package_name = "flashkda_b200"
        env_var = "FLA_FLASHKDA_B200"
        default_enable = True
        priority = 2   # before the stock FlashKDA backend (3)

        def chunk_kda_verifier(self, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                               use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                               use_beta_sigmoid_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None,
                               safe_gate=False, lower_bound=None, disable_recompute=False,
                               return_intermediate_states=False, cp_context=None, transpose_state_layout=False,
                               **kwargs):
            why = _stock_checks(q, v, use_gate_in_kernel, use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel,
                                transpose_state_layout, safe_gate)
            if why is not None:
                return False, "flashkda_b200: " + why
            if cp_context is not None:
                if return_intermediate_states:
                    return False, "flashkda_b200: intermediate states are not exported under context parallelism"
                if cp_context.group is None:
                    return False, "flashkda_b200: cp_context without a process group"
            return True, None

        def chunk_kda(self, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                      use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
                      cu_seqlens=None, cu_seqlens_cpu=None, safe_gate=False, lower_bound=None,
                      disable_recompute=False, return_intermediate_states=False, cp_context=None,
                      transpose_state_layout=False, A_log=None, dt_bias=None, **kwargs):
            import flashkda_b200
            if scale is None:
                scale = q.shape[-1] ** -0.5
            H = v.shape[2]
            if dt_bias is not None and dt_bias.ndim == 1:
                dt_bias = dt_bias.view(H, -1)
            out = torch.empty_like(v)
            if cp_context is not None:
                # FLA's contract under context parallelism: no initial state, no final state, cu_seqlens from the context
                fwd_fla_context_parallel(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, cp_context)
                return out, None
            N = len(cu_seqlens) - 1 if cu_seqlens is not None else q.shape[0]
            if initial_state is not None:
                initial_state = initial_state.contiguous()
            final_state = torch.empty(N, H, D, D, dtype=torch.float32, device=q.device) if output_final_state else None
            if cu_seqlens is not None and cu_seqlens.dtype != torch.long:
                cu_seqlens = cu_seqlens.to(torch.long)
            h = None
            if return_intermediate_states:
                if cu_seqlens is not None:
                    lens = (cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu())
                    lens = (lens[1:] - lens[:-1]).tolist()
                    slots = flashkda_b200.chunk_states_slots(1, 0, _CHUNK_STATES_EVERY, seq_lens=lens)
                    h = torch.empty(1, slots, H, D, D, dtype=torch.bfloat16, device=q.device)
                else:
                    per = flashkda_b200.chunk_states_slots(1, q.shape[1], _CHUNK_STATES_EVERY)
                    h = torch.empty(q.shape[0], per, H, D, D, dtype=torch.bfloat16, device=q.device)
            flashkda_b200.fwd(q, k, v, g, beta, scale, out, A_log=A_log, dt_bias=dt_bias, lower_bound=lower_bound,
                              initial_state=initial_state, final_state=final_state, cu_seqlens=cu_seqlens,
                              chunk_states=h, chunk_states_every=_CHUNK_STATES_EVERY)
            if return_intermediate_states:
                return out, final_state, h
            return out, final_state

    return FlashKDAB200Backend


def register():
    """Registers the backend with FLA's ``kda`` registry (idempotent); returns the backend instance."""
    from fla.ops.backends import BackendRegistry
    BackendRegistry.ensure_initialized("kda")
    from fla.ops.kda.backends import kda_registry
    existing = kda_registry._backends.get("flashkda_b200")
    if existing is not None:
        return existing
    backend = _make_backend()()
    kda_registry.register(backend)
    return backend
