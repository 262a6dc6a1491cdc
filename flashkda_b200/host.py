"""Host-buffer front end: the forward pass for callers whose tensors live in host memory.

``fwd_host`` takes CPU tensors (pinned memory gives full copy bandwidth), streams them to the
device in slabs of whole sequences, runs ``fwd`` on each slab and streams ``out`` and
``final_state`` back, overlapping copies with compute on separate CUDA streams.  Sequences are
independent, so slabbing over the batch dimension changes no result.
"""
import torch

from . import fwd as _fwd

D = 128


class _Slab:
    """Device staging buffers for one slab of ``b`` sequences."""

    def __init__(self, b, T, H, dev, h0_dtype, hT_dtype):
        bf = torch.bfloat16
        self.q, self.k, self.v, self.g, self.out = (torch.empty(b, T, H, D, dtype=bf, device=dev) for _ in range(5))
        self.beta = torch.empty(b, T, H, dtype=bf, device=dev)
        self.h0 = torch.empty(b, H, D, D, dtype=h0_dtype, device=dev) if h0_dtype is not None else None
        self.hT = torch.empty(b, H, D, D, dtype=hT_dtype, device=dev) if hT_dtype is not None else None
        self.ready = torch.cuda.Event()   # inputs landed
        self.done = torch.cuda.Event()    # compute finished
        self.drained = torch.cuda.Event()  # outputs copied back


def fwd_host(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
             cu_seqlens=None, *, device="cuda", slab_sequences: int = 1, algo: str = None):
    """Same arguments as ``fwd`` but every tensor is in HOST memory; ``out`` and ``final_state``
    are host tensors written in place.  Returns (h2d_bytes, d2h_bytes) moved.  Synchronises
    before returning (the results are in host memory)."""
    dev = torch.device(device)
    B, T, H, _ = q.shape
    A_d = A_log.to(dev, non_blocking=True)
    dt_d = dt_bias.to(dev, non_blocking=True)
    h2d = A_log.numel() * 4 + dt_bias.numel() * 4
    d2h = 0
    if cu_seqlens is not None or B <= slab_sequences:
        # one slab: ragged batches are not split
        dq, dk, dv, dg, db = (t.to(dev, non_blocking=True) for t in (q, k, v, g, beta))
        h0 = None if initial_state is None else initial_state.to(dev, non_blocking=True)
        hT = None if final_state is None else torch.empty_like(final_state, device=dev)
        cu = None if cu_seqlens is None else cu_seqlens.to(dev, non_blocking=True)
        do = torch.empty_like(dv)
        _fwd(dq, dk, dv, dg, db, scale, do, A_d, dt_d, lower_bound, h0, hT, cu, algo=algo)
        out.copy_(do, non_blocking=True)
        if hT is not None:
            final_state.copy_(hT, non_blocking=True)
        torch.cuda.synchronize(dev)
        h2d += sum(t.numel() * t.element_size() for t in (q, k, v, g, beta))
        h2d += 0 if initial_state is None else initial_state.numel() * initial_state.element_size()
        h2d += 0 if cu_seqlens is None else cu_seqlens.numel() * 8
        d2h += out.numel() * 2 + (0 if final_state is None else final_state.numel() * final_state.element_size())
        return h2d, d2h

    sb = slab_sequences
    n_slabs = (B + sb - 1) // sb
    h0_dt = None if initial_state is None else initial_state.dtype
    hT_dt = None if final_state is None else final_state.dtype
    slabs = [_Slab(sb, T, H, dev, h0_dt, hT_dt) for _ in range(min(3, n_slabs))]
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    for i in range(n_slabs):
        lo, hi = i * sb, min(B, (i + 1) * sb)
        b = hi - lo
        sl = slabs[i % len(slabs)]
        with torch.cuda.stream(s_in):
            if i >= len(slabs):
                s_in.wait_event(sl.drained)  # buffers free again
            for dst, src in ((sl.q, q), (sl.k, k), (sl.v, v), (sl.g, g), (sl.beta, beta)):
                dst[:b].copy_(src[lo:hi], non_blocking=True)
                h2d += src[lo:hi].numel() * 2
            if sl.h0 is not None:
                sl.h0[:b].copy_(initial_state[lo:hi], non_blocking=True)
                h2d += initial_state[lo:hi].numel() * initial_state.element_size()
            sl.ready.record(s_in)
        main.wait_event(sl.ready)
        _fwd(sl.q[:b], sl.k[:b], sl.v[:b], sl.g[:b], sl.beta[:b], scale, sl.out[:b], A_d, dt_d, lower_bound,
             None if sl.h0 is None else sl.h0[:b], None if sl.hT is None else sl.hT[:b], None, algo=algo)
        sl.done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(sl.done)
            out[lo:hi].copy_(sl.out[:b], non_blocking=True)
            d2h += out[lo:hi].numel() * 2
            if sl.hT is not None:
                final_state[lo:hi].copy_(sl.hT[:b], non_blocking=True)
                d2h += final_state[lo:hi].numel() * final_state.element_size()
            sl.drained.record(s_out)
    main.wait_stream(s_in)
    main.wait_stream(s_out)
    torch.cuda.synchronize(dev)
    return h2d, d2h
