"""Multi-GPU use of the KDA forward: one process per GPU.

Two ways to spread one problem over the GPUs of a box:

* **(batch, head) sharding** -- every quantity of the forward is per (batch, head), so rank
  ``r`` takes heads ``[r*H/G, (r+1)*H/G)`` (or its own batch entries) and nothing is
  exchanged.  ``head_range`` / ``forward_head_shard`` pass strided head views straight to
  the C ABI (no copy).
* **sequence split** for one long sequence -- the reference only analyses this route
  (``tools/probe_segment_affine.py:5-31,118-125`` of the reference project): a segment of
  chunks is an affine map of the state entering it, ``S_out = S_in @ M_seg + Q_seg``
  (V-first ``S`` is ``[V, K]``, ``M_seg`` is ``[K, K]``).  Rank ``j`` runs K1 on its
  contiguous segment once, then two state-only passes over the same chunk records:
  ``Q_seg`` is the final state from a zero state, ``M_seg`` the final state from the
  identity with the ``u`` term dropped.  One all-gather of ``(M_seg, Q_seg)`` (fp32,
  ``2 x 64 KiB`` per head) lets every rank fold the segments before it,
  ``S_in[j] = (((h0 M_0 + Q_0) M_1 + Q_1) ...)`` in fp32, and a last ordinary K2 pass with
  that entry state produces the rank's outputs.  Received tiles land in local memory first;
  the exchange is NCCL on GPUs and works unchanged over gloo on CPU tensors.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib, api

D = 128


# ---------------------------------------------------------------------------
# (batch, head) sharding
# ---------------------------------------------------------------------------
def head_range(H: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous head block of ``rank``; the first ``H % world`` ranks take one head more."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(H, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def forward_head_shard(q, k, v, g, beta, *, rank: int, world: int, scale=None, initial_state=None,
                       output_final_state=False, lower_bound=-5.0, A_log=None, dt_bias=None):
    """Forward of this rank's heads of a full ``[B, T, H, 128]`` problem resident on this GPU.

    Returns ``(o_local [B, T, H_local, 128], ht_local | None, (h_lo, h_hi))``.  The head
    slices are views; only the small per-head vectors are made contiguous.
    """
    B, T, H, _ = q.shape
    lo, hi = head_range(H, world, rank)
    if hi == lo:
        raise ValueError(f"rank {rank} of {world} has no head of {H}")
    sl = slice(lo, hi)
    api._validate_kda_inputs(q, k, v, g, beta, initial_state, True, True, lower_bound, A_log, dt_bias, True)
    api._require_cuda(q)
    if scale is None:
        scale = D ** -0.5
    h0 = None if initial_state is None else initial_state[:, sl].contiguous()
    db = None if dt_bias is None else dt_bias.view(H, D)[sl].contiguous().view(-1)
    o, ht = api._forward(q[:, :, sl], k[:, :, sl], v[:, :, sl], g[:, :, sl], beta[:, :, sl], scale, h0,
                         output_final_state, True, True, True, lower_bound, A_log[sl].contiguous(), db, True)
    return o, ht, (lo, hi)


# ---------------------------------------------------------------------------
# sequence split
# ---------------------------------------------------------------------------
def compose_entry_states(M: Sequence[torch.Tensor], Q: Sequence[torch.Tensor],
                         h0: Optional[torch.Tensor]) -> list[torch.Tensor]:
    """Entry state of every segment and the state after the last one.

    ``M[j]``, ``Q[j]``: ``[B, H, 128, 128]`` fp32 transforms of segment ``j``
    (``S_out = S_in @ M + Q``).  Returns ``G + 1`` tensors: ``S_in[0..G-1]`` and the final state.
    Plain fp32 matmuls (TF32 off): the fold is 128^3 per head and segment, off the hot path.
    """
    S = torch.zeros_like(Q[0]) if h0 is None else h0.to(torch.float32)
    out = [S]
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for Mj, Qj in zip(M, Q):
            S = torch.matmul(S, Mj) + Qj
            out.append(S)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return out


def exchange_segment_transforms(M_local: torch.Tensor, Q_local: torch.Tensor, group=None):
    """All-gather of the per-rank ``(M_seg, Q_seg)``; returns two lists of ``world`` tensors."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    packed = torch.stack([M_local, Q_local]).contiguous()
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    return [t[0] for t in gathered], [t[1] for t in gathered]


class _Segment:
    """K1 records of one contiguous token segment plus what is needed to re-run K2 on them."""

    def __init__(self, q, k, v, g, beta, scale, lower_bound, A_log, dt_bias):
        api._validate_kda_inputs(q, k, v, g, beta, None, True, True, lower_bound, A_log, dt_bias, True,
                                 require_contiguous=False)
        api._require_cuda(q)
        self.B, self.T, self.H, _ = q.shape
        if self.T % api.BT:
            raise ValueError("a sequence segment must be a whole number of 16-token chunks, got T=%d" % self.T)
        self.dev = q.device
        self.lib = _lib.load()
        self.ws = torch.empty(api.workspace_bytes(self.B, self.T, self.H), dtype=torch.uint8, device=self.dev)
        self.o = torch.empty((self.B, self.T, self.H, D), dtype=torch.bfloat16, device=self.dev)
        self.ht = torch.empty((self.B, self.H, D, D), dtype=torch.float32, device=self.dev)
        self.keep = (q, k, v, g, beta, A_log, dt_bias)   # the argument block holds raw pointers
        self.args = api.make_args(q, k, v, g, beta, scale=scale, lower_bound=lower_bound, A_log=A_log,
                                  dt_bias=dt_bias, h0=None, o=self.o, ht=self.ht, workspace=self.ws, flags=7)
        self.stream = api._stream_handle()
        with torch.cuda.device(self.dev):
            api._check(self.lib.kda_fwd_k1(ctypes.byref(self.args), self.stream))

    def _with_state(self, h0, ht):
        self.args.h0 = None if h0 is None else ctypes.c_void_p(h0.data_ptr())
        self.args.ht = ctypes.c_void_p(ht.data_ptr())

    def transforms(self):
        """(M_seg, Q_seg): two state-only passes over the records.  They are independent (same records,
        different entry state), and one pass leaves most of the GPU idle (a chain per head), so the second
        runs beside the first on a side stream."""
        eye = torch.eye(D, device=self.dev, dtype=torch.float32).expand(self.B, self.H, D, D).contiguous()
        M = torch.empty_like(eye)
        Q = torch.empty_like(eye)
        cur = torch.cuda.current_stream(self.dev)
        side = torch.cuda.Stream(device=self.dev)
        args_m = _lib.KdaFwdArgs.from_buffer_copy(self.args)
        args_m.h0 = ctypes.c_void_p(eye.data_ptr())
        args_m.ht = ctypes.c_void_p(M.data_ptr())
        with torch.cuda.device(self.dev):
            side.wait_stream(cur)                      # K1's records (and eye) are ready
            api._check(self.lib.kda_fwd_k2_state(ctypes.byref(args_m), 1, ctypes.c_void_p(side.cuda_stream)))
            self._with_state(None, Q)
            api._check(self.lib.kda_fwd_k2_state(ctypes.byref(self.args), 0, ctypes.c_void_p(cur.cuda_stream)))
            cur.wait_stream(side)
        self._eye = eye   # stays alive until the launches that read it have been ordered
        return M, Q

    def outputs(self, S_in):
        """Ordinary K2 pass from the true entry state: (o, state after the segment)."""
        S_in = None if S_in is None else S_in.contiguous()
        with torch.cuda.device(self.dev):
            self._with_state(S_in, self.ht)
            api._check(self.lib.kda_fwd_k2(ctypes.byref(self.args), self.stream))
        self._s_in = S_in
        return self.o, self.ht


def forward_seq_parallel(q, k, v, g, beta, *, scale=None, initial_state=None, lower_bound=-5.0,
                         A_log=None, dt_bias=None, group=None):
    """This rank's contiguous token segment of one long sequence (segments in rank order).

    ``q, k, v, g, beta`` hold the local ``T / world`` tokens (a multiple of 16);
    ``initial_state`` is the state before the FIRST segment (same tensor on every rank).
    Returns ``(o_local, final_state)``; ``final_state`` is the state after the LAST segment on
    every rank.  In-kernel gate, l2-norm and beta sigmoid, V-first state.
    """
    import torch.distributed as dist

    if scale is None:
        scale = D ** -0.5
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    seg = _Segment(q, k, v, g, beta, scale, lower_bound, A_log, dt_bias)
    if world == 1:
        o, ht = seg.outputs(initial_state)
        return o, ht.clone()
    M, Q = seg.transforms()
    Ms, Qs = exchange_segment_transforms(M, Q, group)
    states = compose_entry_states(Ms, Qs, initial_state)
    o, _ = seg.outputs(states[rank] if (rank > 0 or initial_state is not None) else None)
    return o, states[world]


def forward_seq_split_local(q, k, v, g, beta, n_segments: int, *, scale=None, initial_state=None,
                            lower_bound=-5.0, A_log=None, dt_bias=None):
    """The same three-pass schedule on ONE GPU, segments standing in for ranks (no
    communication): used to check the split against the one-pass forward."""
    if scale is None:
        scale = D ** -0.5
    B, T, H, _ = q.shape
    if T % (n_segments * api.BT):
        raise ValueError("T must split into n_segments multiples of 16")
    L = T // n_segments
    segs = [_Segment(q[:, j * L:(j + 1) * L], k[:, j * L:(j + 1) * L], v[:, j * L:(j + 1) * L],
                     g[:, j * L:(j + 1) * L], beta[:, j * L:(j + 1) * L], scale, lower_bound, A_log, dt_bias)
            for j in range(n_segments)]
    MQ = [s.transforms() for s in segs]
    states = compose_entry_states([m for m, _ in MQ], [q_ for _, q_ in MQ], initial_state)
    outs = [s.outputs(states[j] if (j > 0 or initial_state is not None) else None)[0] for j, s in enumerate(segs)]
    return torch.cat(outs, dim=1), states[n_segments]
