"""Context parallelism for one long sequence: every rank holds a contiguous shard of the tokens.

The reference has no multi-GPU path (its FLA adapter rejects context parallelism,
fla/ops/kda/backends/flashkda.py:82-83); this module adds one on top of the forward operator.

One chunk of the recurrence is affine in the state: with the state kept as S[V, K],
``S_out = S_in @ M + N`` where the K x K transition ``M`` depends on q-independent chunk data only
(k, g, beta) and ``N`` is linear in v.  A shard composes to one such pair, which the ordinary
forward operator yields directly: ``N`` is the final state of the shard started from zero, ``M`` is
the final state of the same shard run with ``v = 0`` from the identity.  So

  1. rank 0 runs its shard for real (its final state is exact); ranks 1 .. G-2 compute (M_r, N_r):
     the prepare stage once, then two recurrences over the same chunk records (the records depend on
     q, k, g, beta only); the last rank needs no map;
  2. one all-gather (torch.distributed: NCCL over NVLink on GPUs, gloo in CPU tests) of the fp32
     pairs, 2 * H * 128 * 128 * 4 bytes per rank;
  3. every rank folds its predecessors in order, ``S <- S @ M_j + N_j`` (fp32), to get its true
     initial state, then walks its records once more from that state; the last rank's final state is
     the sequence's final state.

Shard boundaries must be multiples of 16 tokens (every shard but the last), so that the chunk grid
of the sharded run equals that of the one-shot run.  The maps carry the bf16 roundings of the
kernel, so the result matches a single-GPU run to the parity tolerances (out max-abs 2e-2, state
RMSE-ratio 1e-2), not bit for bit.
"""
from typing import Callable, List, Optional, Tuple

import torch

D = 128


def shard_maps(fwd_fn: Callable, q, k, v, g, beta, scale, A_log, dt_bias, lower_bound, need_transition=True,
               streams=None) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """(M, N) of one shard, both fp32 ``[1, H, 128, 128]``: ``S_out = S_in @ M + N`` (S as [V, K])."""
    H = q.shape[2]
    dev = q.device
    N = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev)
    M = None
    scratch = torch.empty_like(v)
    if need_transition:
        M = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev)
        eye = torch.eye(D, dtype=torch.float32, device=dev).expand(1, H, D, D).contiguous()
        zero_v = torch.zeros_like(v)
        scratch2 = torch.empty_like(v)
    if streams is not None and need_transition:
        cur = torch.cuda.current_stream(dev)
        s0, s1 = streams
        s0.wait_stream(cur)
        s1.wait_stream(cur)
        with torch.cuda.stream(s0):
            fwd_fn(q, k, v, g, beta, scale, scratch, A_log, dt_bias, lower_bound, None, N, None)
        with torch.cuda.stream(s1):
            fwd_fn(q, k, zero_v, g, beta, scale, scratch2, A_log, dt_bias, lower_bound, eye, M, None)
        cur.wait_stream(s0)
        cur.wait_stream(s1)
        for t in (scratch, scratch2, zero_v, eye):
            t.record_stream(s0)
            t.record_stream(s1)
    else:
        fwd_fn(q, k, v, g, beta, scale, scratch, A_log, dt_bias, lower_bound, None, N, None)
        if need_transition:
            fwd_fn(q, k, zero_v, g, beta, scale, scratch2, A_log, dt_bias, lower_bound, eye, M, None)
    return M, N


def fold(S: torch.Tensor, M: torch.Tensor, N: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``S . M + N`` over the leading dimensions of fp32 ``[..., 128, 128]`` tensors: a state through a shard's map.
    On the device this is the library's own kernel (``fkda_cp_fold``: fp32 FMAs in a fixed order); host tensors
    (the CPU tests, which run the oracle as operator) go through ``torch.matmul``."""
    if not S.is_cuda:
        R = torch.matmul(S, M)
        return R if N is None else R + N
    from . import _lib
    S, M = S.contiguous(), M.contiguous()
    N = None if N is None else N.contiguous()
    assert S.dtype == M.dtype == torch.float32 and S.shape == M.shape and S.shape[-2:] == (D, D)
    out = torch.empty_like(S)
    rc = _lib.lib().fkda_cp_fold(S.data_ptr(), M.data_ptr(), None if N is None else N.data_ptr(), out.data_ptr(),
                                 S.numel() // (D * D), torch.cuda.current_stream(S.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"fkda_cp_fold failed: {_lib.status_string(rc)}")
    return out


def fold_initial_state(first_end_state: torch.Tensor, maps: List[Tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
    """State entering the shard that follows rank 0 and the shards of ``maps`` (in order)."""
    S = first_end_state.to(torch.float32)
    for M, N in maps:
        S = fold(S, M, N)
    return S


def _shard_argument_error(q, k, v, g, beta, out, initial_state, final_state, rank, world):
    if q.dim() != 4 or q.shape[0] != 1:
        return "context parallelism shards ONE sequence: q must be [1, T, H, 128]"
    for name, t in (("k", k), ("v", v), ("g", g), ("out", out)):
        if tuple(t.shape) != tuple(q.shape):
            return f"{name} must match q shape"
    if tuple(beta.shape) != tuple(q.shape[:3]):
        return "beta must be [1, T, H] matching q"
    if rank < world - 1 and q.shape[1] % 16 != 0:
        return "every shard but the last must hold a multiple of 16 tokens"
    H = q.shape[2]
    for name, s in (("initial_state", initial_state), ("final_state", final_state)):
        if s is not None:
            if tuple(s.shape) != (1, H, D, D):
                return f"{name} must be [1, H, 128, 128]"
            if s.dtype not in (torch.bfloat16, torch.float32):
                return f"{name} must be bfloat16 or float32"
    return None


def _check_shard_arguments(q, k, v, g, beta, out, initial_state, final_state, rank, world, group):
    """Argument checks, agreed on by ALL ranks before the data-path collectives: a shard can be wrong on one rank
    only (its length, a state dtype), and a rank that raised alone would leave the others waiting inside the
    all-gather.  One 4-byte all-reduce carries the verdict; every rank raises when any rank found a fault."""
    import torch.distributed as dist
    err = _shard_argument_error(q, k, v, g, beta, out, initial_state, final_state, rank, world)
    if world > 1:
        flag = torch.tensor([0 if err is None else 1], dtype=torch.int32, device=q.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        if int(flag.item()) != 0 and err is None:
            err = "another rank of the group rejected its arguments"
    if err is not None:
        raise RuntimeError(err)


def fwd_context_parallel(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None,
                         final_state=None, group=None, fwd_fn: Callable = None, parts: int = 1, validate: bool = True):
    """Forward over one sequence sharded across the ranks of ``group`` (contiguous shards in rank
    order, B = 1, every shard but the last a multiple of 16 tokens).  ``initial_state`` (bf16 or fp32) is
    used by rank 0; ``final_state`` (optional, any rank, either dtype) receives the state after the last
    token.  Writes this rank's ``out`` in place.

    With the device operator (``fwd_fn`` left None) every rank prepares its chunk records ONCE and runs its
    recurrences over them (the maps ``N`` and ``M``, then the real pass), and ``parts`` > 1 additionally
    splits the rank's shard into that many pieces that run side by side (``SequenceSplit``).  A caller-given
    ``fwd_fn`` (tests: the CPU oracle) is called with the reference signature only.

    ``validate`` (default on): the ranks agree on the validity of their arguments before the data-path collectives
    (one 4-byte all-reduce whose result the host reads, i.e. one host synchronisation per call); a caller that has
    validated its shards once and calls in a hot loop may turn it off."""
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if validate:
        _check_shard_arguments(q, k, v, g, beta, out, initial_state, final_state, rank, world, group)
    H, dev = q.shape[2], q.device
    payload = torch.zeros(2, 1, H, D, D, dtype=torch.float32, device=dev)
    S0 = None if initial_state is None else initial_state.to(torch.float32)   # maps and folds are fp32
    last = world - 1
    src_last = dist.get_global_rank(group, last) if group is not None else last

    def publish_final(end):
        if final_state is not None:
            buf = end.contiguous() if rank == last else torch.empty(1, H, D, D, dtype=torch.float32, device=dev)
            if world > 1:
                dist.broadcast(buf, src=src_last, group=group)
            final_state.copy_(buf.to(final_state.dtype))

    if fwd_fn is None:
        # ---- device operator: chunk records prepared once per rank, reused by every recurrence ----
        if parts > 1 and q.shape[1] % (16 * parts) != 0:
            parts = 1   # (this rank only; the exchange does not depend on how a rank walks its own shard)
        split = SequenceSplit(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, parts)
        end = None
        if world == 1 or rank == 0:
            end = split.finish(S0 if rank == 0 else None, None)   # exact for this shard's true initial state
            payload[1].copy_(end)
        elif rank < last:
            Mt, Nt = split.maps()
            payload[0].copy_(Mt)
            payload[1].copy_(Nt)
        elif parts > 1:
            split.maps(total=False)   # the last rank needs the maps of its own pieces only
        if world > 1:
            gathered = [torch.empty_like(payload) for _ in range(world)]
            dist.all_gather(gathered, payload, group=group)
            if rank > 0:
                S_in = fold_initial_state(gathered[0][1], [(gathered[j][0], gathered[j][1]) for j in range(1, rank)])
                end = split.finish(S_in, None)
        publish_final(end)
        return

    # ---- any operator with the reference signature (CPU tests run the oracle here) ----
    if world == 1:
        fwd_fn(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state, None)
        return
    if rank == 0:
        end = payload[1]
        fwd_fn(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, S0, end, None)
    elif rank < last:
        M, N = shard_maps(fwd_fn, q, k, v, g, beta, scale, A_log, dt_bias, lower_bound, True, None)
        payload[0].copy_(M)
        payload[1].copy_(N)
    gathered = [torch.empty_like(payload) for _ in range(world)]
    dist.all_gather(gathered, payload, group=group)
    last_state = None
    if rank > 0:
        S_in = fold_initial_state(gathered[0][1], [(gathered[j][0], gathered[j][1]) for j in range(1, rank)])
        last_state = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev)
        fwd_fn(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, S_in.contiguous(), last_state, None)
    publish_final(last_state)


def fwd_sharded_emulated(n_shards: int, q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound,
                         initial_state=None, final_state=None, fwd_fn: Callable = None):
    """The same algorithm with all shards in one process (no process group): used to check the
    numerics of the map-and-fold scheme on a single device."""
    if fwd_fn is None:
        from . import fwd as fwd_fn
    T = q.shape[1]
    per = (T // n_shards) // 16 * 16
    bounds = [i * per for i in range(n_shards)] + [T]
    sl = lambda x, i: x[:, bounds[i]:bounds[i + 1]].contiguous()
    H, dev = q.shape[2], q.device
    outs = [torch.empty_like(sl(v, i)) for i in range(n_shards)]
    end0 = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev)
    fwd_fn(sl(q, 0), sl(k, 0), sl(v, 0), sl(g, 0), sl(beta, 0), scale, outs[0], A_log, dt_bias, lower_bound,
           initial_state, end0, None)
    maps = [shard_maps(fwd_fn, sl(q, i), sl(k, i), sl(v, i), sl(g, i), sl(beta, i), scale, A_log, dt_bias,
                       lower_bound) for i in range(1, n_shards - 1)]
    last = end0
    for i in range(1, n_shards):
        S_in = fold_initial_state(end0, maps[:i - 1]).contiguous()
        last = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev)
        fwd_fn(sl(q, i), sl(k, i), sl(v, i), sl(g, i), sl(beta, i), scale, outs[i], A_log, dt_bias, lower_bound,
               S_in, last, None)
    out.copy_(torch.cat(outs, dim=1))
    if final_state is not None:
        final_state.copy_(last.to(final_state.dtype))


class SequenceSplit:
    """One long sequence on ONE GPU, split into ``parts`` contiguous pieces that run side by side.

    A single (sequence, head) chain is serial, so a lone long sequence keeps only H of the GPU's
    hundreds of chain slots busy.  The same map-and-fold scheme as for context parallelism fixes that
    without any communication: view ``[1, T, H, 128]`` as a batch ``[parts, T/parts, H, 128]`` (no
    copy), compute every piece's ``(M, N)`` in two batched calls (``maps``), fold the pieces in order
    and run the batch once more from the true initial states (``finish``).  The prepare stage runs
    once: its records do not depend on v or on the state, so the second and third call reuse the
    workspace (``phase_mask``).  Results agree with the one-shot run to the parity tolerances (piece
    boundaries carry the kernel's bf16 roundings), not bit for bit.  T must be a multiple of 16 * parts.
    """

    def __init__(self, q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, parts: int):
        import flashkda_b200 as F
        B, T, H, _ = q.shape
        assert B == 1 and (parts == 1 or T % (16 * parts) == 0), "T must be a multiple of 16 * parts"
        self.F, self.P, self.H, self.dev = F, parts, H, q.device
        vw = lambda x: x.view(parts, T // parts, *x.shape[2:])
        self.t = (vw(q), vw(k), vw(v), vw(g), vw(beta))
        self.out = vw(out)
        self.args = (A_log, dt_bias, lower_bound)
        self.scale = scale
        self.ws = torch.empty(max(256, F.get_workspace_size(T, H, parts)), dtype=torch.uint8, device=self.dev)
        self.M = self.N = None
        self.prepared = False   # whether self.ws holds the chunk records of this shard

    def _fwd(self, v, h0, hT):
        """One operator call on the batch of pieces; the first one also runs the prepare stage, later ones
        walk the records it left in the workspace."""
        from . import _lib
        qb, kb, _, gb, bb = self.t
        self.F.fwd(qb, kb, v, gb, bb, self.scale, self.out, *self.args, h0, hT, None, workspace=self.ws,
                   phase_mask=_lib.PHASE_RECURRENCE if self.prepared else 0)
        self.prepared = True

    def maps(self, total: bool = True):
        """Per-piece maps (kept) and, with ``total``, the composed map of the whole shard ``(M, N)``."""
        P, H, dev = self.P, self.H, self.dev
        vb = self.t[2]
        self.N = torch.zeros(P, H, D, D, dtype=torch.float32, device=dev)
        self.M = torch.zeros(P, H, D, D, dtype=torch.float32, device=dev)
        eye = torch.eye(D, dtype=torch.float32, device=dev).expand(P, H, D, D).contiguous()
        self._fwd(vb, None, self.N)                       # from zero: N
        self._fwd(torch.zeros_like(vb), eye, self.M)      # v = 0 from the identity: M
        if not total:
            return None, None
        Mt, Nt = self.M[0:1], self.N[0:1]
        for p in range(1, P):
            Nt = fold(Nt, self.M[p:p + 1], self.N[p:p + 1])
            Mt = fold(Mt, self.M[p:p + 1])
        return Mt, Nt

    def finish(self, initial_state=None, final_state=None):
        """Fold the pieces from ``initial_state`` and run the batch for real (writes ``out``); returns the
        state after the last token, fp32 ``[1, H, 128, 128]``."""
        P, H, dev = self.P, self.H, self.dev
        if P > 1 and self.M is None:
            self.maps(total=False)
        S = torch.zeros(1, H, D, D, dtype=torch.float32, device=dev) if initial_state is None \
            else initial_state.to(torch.float32)
        h0 = torch.empty(P, H, D, D, dtype=torch.float32, device=dev)
        for p in range(P):
            h0[p] = S[0]
            if p + 1 < P:
                S = fold(S, self.M[p:p + 1], self.N[p:p + 1])
        hT = torch.zeros(P, H, D, D, dtype=torch.float32, device=dev)
        self._fwd(self.t[2], h0, hT)
        if final_state is not None:
            final_state.copy_(hT[P - 1:P].to(final_state.dtype))
        return hT[P - 1:P]


def fwd_sequence_parallel(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None,
                          final_state=None, parts: int = 8):
    """Single-GPU forward of one long sequence split into ``parts`` pieces (see ``SequenceSplit``)."""
    SequenceSplit(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, parts).finish(initial_state, final_state)
