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
  identity with the ``u`` term dropped (one launch computes both).  The fold
  ``S_in[j] = (((h0 M_0 + Q_0) M_1 + Q_1) ...)`` is a hand-written fp32 kernel
  (``kda_state_fold``).  Two exchange patterns: **all-to-all** (default when the chains divide
  over the ranks) -- rank ``r`` folds chains ``[r*hp, (r+1)*hp)`` of ALL segments and sends
  every segment its entry states back, ``2 x 64 KiB`` per chain and hop instead of every
  rank receiving every transform; **all-gather** -- every rank receives all transforms and
  folds the segments before its own.  A last ordinary K2 pass from the entry state produces
  the rank's outputs.  Received tiles land in local memory first; the exchange is NCCL on
  GPUs and works unchanged over gloo on CPU tensors (with a caller-supplied fold).
  ``SeqParallelPlan`` allocates every buffer, stream and argument block once.
"""
from __future__ import annotations

import ctypes
import os
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
    """Entry state of every segment and the state after the last one, by plain torch matmuls.

    ``M[j]``, ``Q[j]``: ``[..., 128, 128]`` fp32 transforms of segment ``j``
    (``S_out = S_in @ M + Q``).  Returns ``G + 1`` tensors.  This is the host-side statement of
    what ``kda_state_fold`` computes on the GPU; the GPU paths below use the kernel, this
    function serves CPU tensors (the gloo tests) and cross-checks.
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


def _walk_cuda(mq, h0, n_seg, *, use_q=True, s_in=None, final_out=None, status=None):
    """``kda_state_fold_ex`` on tensors.  ``mq``: fp32 ``[segments, chains, 2, 128, 128]`` view (any segment /
    chain strides, dense 128 x 128 blocks, Q behind M); ``h0`` / ``final_out``: ``[chains, 128, 128]`` views
    (any chain stride) or None; ``s_in``: contiguous ``[n_seg + 1, chains, 128, 128]`` or None."""
    if not mq.is_cuda:
        raise RuntimeError("the fold runs the CUDA kernel kda_state_fold; there is no CPU path")
    chains = mq.shape[1]
    for t, name in ((mq, "mq"), (h0, "h0"), (final_out, "final_out")):
        if t is not None and (t.dtype != torch.float32 or t.stride()[-2:] != (D, 1)):
            raise ValueError(f"{name} must be fp32 with dense 128 x 128 blocks")
    if mq.ndim != 5 or mq.shape[2:] != (2, D, D) or mq.stride(2) != D * D:
        raise ValueError("mq must be [segments, chains, 2, 128, 128] with Q directly behind M")
    f = _lib.KdaFoldArgs()
    f.mq = mq.data_ptr()
    f.seg_stride, f.chain_stride = (mq.stride(0) if mq.shape[0] > 1 else 2 * D * D), (mq.stride(1) if chains > 1 else 2 * D * D)
    if h0 is not None:
        f.h0, f.h0_stride = h0.data_ptr(), (h0.stride(0) if chains > 1 else D * D)
    if s_in is not None:
        if tuple(s_in.shape) != (n_seg + 1, chains, D, D) or not s_in.is_contiguous() or s_in.dtype != torch.float32:
            raise ValueError("s_in must be a contiguous fp32 [n_seg + 1, chains, 128, 128] tensor")
        f.s_in = s_in.data_ptr()
    if final_out is not None:
        f.final_out, f.final_stride = final_out.data_ptr(), (final_out.stride(0) if chains > 1 else D * D)
    f.n_chains, f.n_seg, f.use_q = chains, n_seg, int(bool(use_q))
    if status is not None:
        f.status = status.data_ptr()
    with torch.cuda.device(mq.device):
        api._check(_lib.load().kda_state_fold_ex(ctypes.byref(f), api._stream_handle()))


def _walk_torch(mq, h0, n_seg, *, use_q=True, s_in=None, final_out=None, status=None):
    """The same contract in plain torch (CPU tensors: the gloo tests)."""
    chains = mq.shape[1]
    S = torch.zeros(chains, D, D, dtype=torch.float32, device=mq.device) if h0 is None else h0.clone().float()
    for j in range(n_seg):
        if s_in is not None:
            s_in[j].copy_(S)
        S = torch.matmul(S, mq[j, :, 0])
        if use_q:
            S = S + mq[j, :, 1]
    if s_in is not None:
        s_in[n_seg].copy_(S)
    if final_out is not None:
        final_out.copy_(S)


def fold_states(mq: torch.Tensor, h0: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                n_seg: Optional[int] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The fold kernel on a CUDA tensor ``mq [n_seg_total, n_chains, 2, 128, 128]`` (fp32; ``M`` then
    ``Q`` per chain, any segment / chain strides): returns ``s_in [n_seg + 1, n_chains, 128, 128]`` --
    the entry state of segments ``0..n_seg-1`` and the state after segment ``n_seg - 1``
    (``n_seg`` defaults to all segments of ``mq``).  ``status``: a workspace (or any int32 device
    tensor) whose first word receives a code if a bounded wait inside the kernel gives up."""
    segs, chains = mq.shape[:2]
    n_seg = segs if n_seg is None else n_seg
    if not 0 <= n_seg <= segs:
        raise ValueError(f"n_seg={n_seg} outside 0..{segs}")
    if out is None:
        out = torch.empty((n_seg + 1, chains, D, D), dtype=torch.float32, device=mq.device)
    if h0 is not None:
        h0 = h0.reshape(chains, D, D)
    _walk_cuda(mq, h0, n_seg, s_in=out, status=status)
    return out


def exchange_mode(chains: int, world: int, requested: str = "auto") -> str:
    """``"a2a"`` (all-to-all, chains divided over the ranks) or ``"gather"``."""
    if requested not in ("auto", "a2a", "gather"):
        raise ValueError("exchange must be 'auto', 'a2a' or 'gather'")
    if requested == "a2a" and chains % world:
        raise ValueError(f"the all-to-all exchange needs the {chains} chains to divide over {world} ranks")
    if requested == "auto":
        return "a2a" if chains % world == 0 else "gather"
    return requested


def exchange_and_fold(mq_local: torch.Tensor, h0: Optional[torch.Tensor], rank: int, world: int, *, group=None,
                      mode: str = "a2a", sub: int = 1, two_level: Optional[bool] = None, walk=None,
                      bufs: Optional[dict] = None, want_final: bool = False, status: Optional[torch.Tensor] = None,
                      mark=None, pushed: bool = False, defer_wait: bool = False):
    """From this rank's transforms to the entry states of its segment(s).

    ``mq_local``: ``[sub * chains, 2, 128, 128]`` -- ``sub`` consecutive sub-segments of this rank
    (sub-segment major), ``chains`` (batch, head) chains each.  Returns ``(s_entry, final | None)``:
    ``s_entry [sub, chains, 128, 128]`` are the entry states of this rank's sub-segments and
    ``final [chains, 128, 128]`` the state after the last segment of the last rank, on every rank
    when ``want_final`` (one more small all-gather in all-to-all mode).

    Two levels when ``sub > 1``: the rank first composes the transforms of its own sub-segments into
    one transform of its whole segment (two walks: the transition matrices, the offsets), only
    those are exchanged and folded, and a last local walk from the returned entry state gives the
    entry states of the rank's sub-segments -- the exchange and the cross-rank fold stay as small as
    without sub-segments, at the price of three more small launches.  ``two_level=None`` takes it
    when there are more than eight segments in all (measured: two ranks x two sub-segments 72 us
    flat against 119 us in two levels; at 32 segments the flat all-gather alone moves 64 MB per
    rank); the flat form all-gathers every sub-segment's transform and needs ``mode="gather"``.  ``bufs``: optional dict the function keeps its buffers in, so a plan
    allocates them once.  ``walk``: the fold routine (default: the CUDA kernel; the CPU tests pass
    the torch statement).
    """
    import torch.distributed as dist

    walk = _walk_cuda if walk is None else walk
    bufs = {} if bufs is None else bufs
    if mq_local.shape[0] % sub:
        raise ValueError("mq_local does not hold a whole number of sub-segments")
    chains = mq_local.shape[0] // sub
    kw = dict(dtype=torch.float32, device=mq_local.device)
    h0c = None if h0 is None else h0.reshape(chains, D, D)

    def buf(name, shape):
        t = bufs.get(name)
        if t is None or tuple(t.shape) != tuple(shape):
            t = bufs[name] = torch.empty(shape, **kw)
        return t

    mq5 = mq_local.contiguous().view(sub, chains, 2, D, D)
    if two_level is None:
        two_level = world * sub > 8 or mode != "gather"
    if sub > 1 and not two_level:
        if mode != "gather":
            raise ValueError("the flat exchange of several segments per rank needs the all-gather")
        segs = world * sub
        allmq = buf("gathered", (segs, chains, 2, D, D))      # segment = rank * sub + sub-segment
        dist.all_gather_into_tensor(allmq.view(segs * chains, 2, D, D), mq5.view(sub * chains, 2, D, D), group=group)
        n_seg = segs if want_final else rank * sub + sub - 1
        s_in = buf("s_in", (n_seg + 1, chains, D, D))
        walk(allmq, h0c, n_seg, s_in=s_in, status=status)
        return s_in[rank * sub:rank * sub + sub], (s_in[segs] if want_final else None)
    if sub > 1:   # this rank's whole segment as one transform
        rank_mq = buf("rank_mq", (chains, 2, D, D))
        walk(mq5[1:], mq5[0, :, 0], sub - 1, use_q=False, final_out=rank_mq[:, 0], status=status)
        walk(mq5[1:], mq5[0, :, 1], sub - 1, use_q=True, final_out=rank_mq[:, 1], status=status)
    else:
        rank_mq = mq5[0]

    final = None
    if mode == "gather":
        allmq = buf("gathered", (world, chains, 2, D, D))
        dist.all_gather_into_tensor(allmq.view(world * chains, 2, D, D), rank_mq, group=group)
        n_seg = world if want_final else rank
        s_in = buf("s_in", (n_seg + 1, chains, D, D))
        walk(allmq, h0c, n_seg, s_in=s_in, status=status)
        entry = s_in[rank]
        final = s_in[world] if want_final else None
    else:
        hp = chains // world
        h0_own = None if h0c is None else h0c[rank * hp:(rank + 1) * hp]
        peer = bufs.get("peer")
        if peer is not None:                                   # stores and flags over peer memory, three launches
            entry, last = peer.run(None if pushed else rank_mq.contiguous(), h0_own, status, want_final, mark=mark,
                                   pushed=pushed, defer_wait=defer_wait and sub == 1)
        else:
            recv = buf("recv_mq", (world, hp, 2, D, D))        # [segment][my chains]
            dist.all_to_all_single(recv, rank_mq.view(world, hp, 2, D, D), group=group)
            s_in = buf("s_in", (world + 1, hp, D, D))
            walk(recv, h0_own, world, s_in=s_in, status=status)
            ent = buf("entry", (world, hp, D, D))              # [owner of the chains][chains] = all chains in order
            dist.all_to_all_single(ent, s_in[:world], group=group)
            entry = ent.view(chains, D, D)
            last = s_in[world].contiguous() if want_final else None
        if want_final:
            final = buf("final", (world, hp, D, D))
            dist.all_gather_into_tensor(final.view(chains, D, D), last, group=group)
            final = final.view(chains, D, D)
    if sub == 1:
        return entry.view(1, chains, D, D), final
    sub_entry = buf("sub_entry", (sub, chains, D, D))          # entry states of this rank's sub-segments
    walk(mq5, entry, sub - 1, s_in=sub_entry, status=status)
    return sub_entry, final


class _PeerExchange:
    """The all-to-all exchange of a sequence split over peer memory: one process per GPU of ONE box.

    Every rank owns one block -- a receive buffer for the transforms ``[world, hp, 2, 128, 128]`` (slot =
    source rank), a buffer for the entry states of its own segment ``[world, hp, 128, 128]`` (slot =
    the rank that owns and folds those chains) and two rows of int32 flags -- and maps the blocks of
    all other ranks into its address space (CUDA IPC: ``kda_ipc_export`` / ``kda_ipc_open``, opened with
    the importing GPU current; a block stays mapped in the peers until they exit, so a plan's block is
    never returned to the driver while peers may still hold the mapping -- it goes back to torch's
    caching allocator, which keeps the allocation).  A run is
    three launches: ``kda_peer_push`` stores this rank's transforms into the owners' receive
    buffers and raises their flags; ``kda_state_fold_peer`` waits for the flags of all sources, walks
    this rank's chains and stores the state before segment j straight into rank j's entry buffer,
    then raises the entry flags; ``kda_flag_wait`` holds the stream until every owner's entry states
    have arrived.  Flags carry the run number, so nothing is reset between runs; every wait is
    bounded and reports status code 7.  Buffers are reused safely: a rank starts run e + 1 only after
    every owner has signalled the end of its walk of run e, and an owner starts its walk of run
    e + 1 only after every rank has finished reading the entry states of run e.

    ``_PeerExchange.create`` returns None (on every rank alike) when any rank could not set it up;
    the caller then uses the NCCL collectives.
    """

    FLAG_WORDS = 64       # int32: [0, world) transforms from rank j; [world, 2 world) entry states from owner j; [32, 64) self-check

    def __init__(self):
        self.epoch = 0
        self.pending = None     # (flags, n, epoch) of entry states whose arrival nothing has waited for yet

    @classmethod
    def create(cls, chains: int, world: int, rank: int, group, device):
        import torch.distributed as dist

        self = cls()
        lib = _lib.load()
        ok, info = 1, None
        try:
            if chains % world or world > _lib.MAX_PEERS or 2 * world > 32:
                raise ValueError("chain count or world size outside the peer exchange's range")
            self.world, self.rank, self.hp, self.dev = world, rank, chains // world, device
            n_recv, n_ent = chains * 2 * D * D, chains * D * D
            self.block = torch.zeros(n_recv + n_ent + cls.FLAG_WORDS, dtype=torch.float32, device=device)
            self.recv = self.block[:n_recv].view(world, self.hp, 2, D, D)
            self.ent = self.block[n_recv:n_recv + n_ent].view(world, self.hp, D, D)
            self.flag_off = n_recv + n_ent                      # in 4-byte words from the start of the block
            self.flags = self.block[self.flag_off:].view(torch.int32)
            self.counters = torch.zeros(world + 1, dtype=torch.int32, device=device)
            self.final = torch.empty((self.hp, D, D), dtype=torch.float32, device=device)
            torch.cuda.synchronize(device)
            hbuf, off = ctypes.create_string_buffer(64), ctypes.c_int64(0)
            with torch.cuda.device(device):
                api._check(lib.kda_ipc_export(self.block.data_ptr(), hbuf, ctypes.byref(off)))
            info = (bytes(hbuf.raw), int(off.value), int(device.index))
        except Exception:  # noqa: BLE001 - any failure here means: use the collectives instead
            ok = 0
        infos = [None] * world
        dist.all_gather_object(infos, (ok, info), group=group)
        if all(i is not None and i[0] == 1 for i in infos):
            try:
                self.peer_ptr = []
                self._opened = []
                self._group = group
                with torch.cuda.device(device):      # the importing GPU must be current when a handle is opened
                    for r, (_, (handle, off, owner_dev)) in enumerate(infos):
                        if r == rank:
                            self.peer_ptr.append(self.block.data_ptr())
                            continue
                        api._check(lib.kda_peer_enable(owner_dev))
                        ptr = ctypes.c_void_p(0)
                        api._check(lib.kda_ipc_open(handle, off, ctypes.byref(ptr)))
                        self._opened.append(handle)
                        self.peer_ptr.append(int(ptr.value))
                self._build_args()
            except Exception:  # noqa: BLE001
                ok = 0
        else:
            ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
        if int(agreed.item()) == 0:
            return None
        # a dry run through the real kernels: every rank sends a pattern to every rank
        try:
            good = self._self_check()
        except Exception:  # noqa: BLE001
            good = 0
        agreed = torch.tensor([good], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
        return self if int(agreed.item()) == 1 else None

    def close(self):
        """Collective: every rank unmaps the other ranks' blocks; afterwards the blocks may be freed.  Without it
        the mappings live until the processes exit, and a block must not be returned to the driver
        (``torch.cuda.empty_cache()``) while a peer still maps it."""
        import torch.distributed as dist

        if getattr(self, "_opened", None) is None:
            return
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self._group)                     # nobody stores into a block any more
        lib = _lib.load()
        with torch.cuda.device(self.dev):
            for handle in self._opened:
                lib.kda_ipc_close(handle)
        self._opened = None
        dist.barrier(group=self._group)                     # every mapping is gone: the owners may free

    def _build_args(self):
        world, rank, hp = self.world, self.rank, self.hp
        flag_addr = [ptr + 4 * self.flag_off for ptr in self.peer_ptr]          # start of rank r's flag words
        push = _lib.KdaPeerPushArgs()
        for d in range(world):
            push.dst[d] = self.peer_ptr[d]                                       # rank d's receive buffer is the start of its block
            push.flag[d] = flag_addr[d] + 4 * rank
        push.counter = self.counters.data_ptr()
        push.slice_floats = hp * 2 * D * D
        push.dst_offset_floats = rank * hp * 2 * D * D
        push.world = world
        self._push = push
        f = _lib.KdaFoldArgs()
        f.mq = self.recv.data_ptr()
        f.seg_stride, f.chain_stride = hp * 2 * D * D, 2 * D * D
        f.n_chains, f.n_seg, f.use_q = hp, world, 1
        self._fold = f
        pa = _lib.KdaFoldPeerArgs()
        pa.wait_flags, pa.n_wait = flag_addr[rank], world
        ent_off = 4 * (world * hp * 2 * D * D)                                   # bytes from the start of a block to its entry buffer
        for j in range(world):
            pa.s_in_seg[j] = self.peer_ptr[j] + ent_off + 4 * rank * hp * D * D
            pa.signal[j] = flag_addr[j] + 4 * (world + rank)
        pa.n_signal = world
        pa.counter = self.counters.data_ptr() + 4 * world
        self._peer = pa
        self._wait_flags = flag_addr[rank] + 4 * world

    def _self_check(self) -> int:
        lib = _lib.load()
        world, rank = self.world, self.rank
        self.epoch += 1
        src = (torch.arange(world, device=self.dev, dtype=torch.float32).view(world, 1) + 1.0 + 100.0 * rank).repeat(1, 4).contiguous()
        a = _lib.KdaPeerPushArgs.from_buffer_copy(self._push)
        check_off = 4 * (self.flag_off + 32)                                     # the self-check words behind the flags
        for d in range(world):
            a.dst[d] = self.peer_ptr[d] + check_off
        a.src, a.slice_floats, a.dst_offset_floats, a.epoch = src.data_ptr(), 4, 4 * rank, self.epoch
        if world * 4 > 32:
            return 0
        with torch.cuda.device(self.dev):
            stream = api._stream_handle()
            api._check(lib.kda_peer_push(ctypes.byref(a), stream))
            api._check(lib.kda_flag_wait(self._wait_flags - 4 * world, world, self.epoch, None, stream))
            torch.cuda.synchronize(self.dev)
        got = self.block[self.flag_off + 32:self.flag_off + 32 + 4 * world].view(world, 4)
        want = (100.0 * torch.arange(world, device=self.dev, dtype=torch.float32).view(world, 1) + rank + 1.0).expand(world, 4)
        return int(bool(torch.equal(got, want)))

    def begin(self):
        """Starts a run whose push is done by the transform-pair pass itself (``kda_fwd_k2_state_push``): returns the
        push block with the new run number; :meth:`run` must follow with ``pushed=True``."""
        self.epoch += 1
        self._push.src, self._push.epoch = None, self.epoch
        return self._push

    def run(self, rank_mq: Optional[torch.Tensor], h0: Optional[torch.Tensor], status: Optional[torch.Tensor], want_final: bool,
            mark=None, pushed: bool = False, defer_wait: bool = False):
        """``rank_mq``: this rank's transforms ``[chains, 2, 128, 128]`` (contiguous); ``h0``: the state before the
        first segment of this rank's OWN chains ``[hp, 128, 128]`` or None.  Returns the entry states of this
        rank's segment for all chains ``[chains, 128, 128]`` (the plan's buffer) and, with ``want_final``, the
        state after the last segment of the own chains ``[hp, 128, 128]``."""
        lib = _lib.load()
        push, f, pa = self._push, self._fold, self._peer
        if not pushed:
            if not rank_mq.is_contiguous() or rank_mq.dtype != torch.float32:
                raise ValueError("rank_mq must be a contiguous fp32 tensor")
            self.epoch += 1
            push.src, push.epoch = rank_mq.data_ptr(), self.epoch
        if h0 is not None:
            if h0.dtype != torch.float32 or h0.stride()[-2:] != (D, 1):
                raise ValueError("h0 must be fp32 with dense 128 x 128 blocks")
            f.h0, f.h0_stride = h0.data_ptr(), (h0.stride(0) if h0.shape[0] > 1 else D * D)
        else:
            f.h0, f.h0_stride = None, 0
        st_ptr = None if status is None else status.data_ptr()
        f.status = st_ptr
        pa.epoch = self.epoch
        pa.s_in_seg[self.world] = self.final.data_ptr() if want_final else None
        with torch.cuda.device(self.dev):
            stream = api._stream_handle()
            if not pushed:
                api._check(lib.kda_peer_push(ctypes.byref(push), stream))
            if mark is not None:
                mark("exchange_push")
            api._check(lib.kda_state_fold_peer(ctypes.byref(f), ctypes.byref(pa), stream))
            if mark is not None:
                mark("exchange_walk")
            if defer_wait:      # the consumer of the entry states waits itself (kda_fwd_k2_after_flags)
                self.pending = (self._wait_flags, self.world, self.epoch)
            else:
                self.pending = None
                api._check(lib.kda_flag_wait(self._wait_flags, self.world, self.epoch, st_ptr, stream))
        return self.ent.view(self.world * self.hp, D, D), (self.final if want_final else None)


def _sub_segments(x: torch.Tensor, sub: int) -> torch.Tensor:
    """``[1, L, ...]`` -> ``[sub, L / sub, ...]`` as a view (consecutive token blocks as batch entries)."""
    return x[0].unflatten(0, (sub, x.shape[1] // sub))


class _Segment:
    """One contiguous token segment: fixed buffers and argument blocks for K1, the transform pass
    (both transforms in one launch) and the ordinary K2 pass."""

    def __init__(self, q, k, v, g, beta, scale, lower_bound, A_log, dt_bias, mq_out=None):
        api._validate_kda_inputs(q, k, v, g, beta, None, True, True, lower_bound, A_log, dt_bias, True,
                                 require_contiguous=False)
        api._require_cuda(q)
        self.B, self.T, self.H, _ = q.shape
        if self.T % api.BT:
            raise ValueError("a sequence segment must be a whole number of 16-token chunks, got T=%d" % self.T)
        self.dev = q.device
        self.chains = self.B * self.H
        self.lib = _lib.load()
        kw = dict(dtype=torch.float32, device=self.dev)
        self.ws = torch.empty(api.workspace_bytes(self.B, self.T, self.H), dtype=torch.uint8, device=self.dev)
        self.o = torch.empty((self.B, self.T, self.H, D), dtype=torch.bfloat16, device=self.dev)
        self.ht = torch.empty((self.B, self.H, D, D), **kw)
        self.mq = torch.empty((self.chains, 2, D, D), **kw) if mq_out is None else mq_out
        if tuple(self.mq.shape) != (self.chains, 2, D, D) or not self.mq.is_contiguous():
            raise ValueError("mq_out must be a contiguous [B*H, 2, 128, 128] fp32 tensor")
        self.keep = (q, k, v, g, beta, A_log, dt_bias)   # the argument blocks hold raw pointers
        self.args = api.make_args(q, k, v, g, beta, scale=scale, lower_bound=lower_bound, A_log=A_log,
                                  dt_bias=dt_bias, h0=None, o=self.o, ht=self.ht, workspace=self.ws, flags=7)
        self.args_mq = _lib.KdaFwdArgs.from_buffer_copy(self.args)
        self.args_mq.h0 = None
        self.args_mq.ht = ctypes.c_void_p(self.mq.data_ptr())
        self._s_in = None

    def k1(self, stream=None):
        with torch.cuda.device(self.dev):
            api._check(self.lib.kda_fwd_k1(ctypes.byref(self.args), api._stream_handle() if stream is None else stream))

    def transforms(self, stream=None):
        """(M_seg, Q_seg) of every chain into ``self.mq``: one state-only launch over 2 x chains."""
        with torch.cuda.device(self.dev):
            api._check(self.lib.kda_fwd_k2_state(ctypes.byref(self.args_mq), 2,
                                                 api._stream_handle() if stream is None else stream))
        return self.mq

    def transforms_push(self, push, stream=None) -> int:
        """The transform pass with its tiles stored straight into the owners' receive buffers
        (``kda_fwd_k2_state_push``); returns the library's code (``ERR_UNSUPPORTED``: no such kernel for this
        problem, nothing was launched)."""
        with torch.cuda.device(self.dev):
            return self.lib.kda_fwd_k2_state_push(ctypes.byref(self.args_mq), ctypes.byref(push),
                                                  api._stream_handle() if stream is None else stream)

    def outputs(self, S_in, stream=None, after_flags=None):
        """Ordinary K2 pass from the true entry state: (o, state after the segment).  ``after_flags = (flags, n,
        epoch)``: the entry state is being stored by other GPUs and the kernel waits for those flags itself
        (``kda_fwd_k2_after_flags``); returns ``(None, None)`` when the library has no such kernel for this
        problem (nothing was launched)."""
        if S_in is not None and not (S_in.is_contiguous() and S_in.dtype == torch.float32):
            if after_flags is not None:
                raise ValueError("an entry state that is still arriving cannot be copied")
            S_in = S_in.contiguous().float()
        self._s_in = S_in   # keep the entry state alive until the launch has been ordered
        self.args.h0 = None if S_in is None else ctypes.c_void_p(S_in.data_ptr())
        with torch.cuda.device(self.dev):
            st = api._stream_handle() if stream is None else stream
            if after_flags is not None:
                rc = self.lib.kda_fwd_k2_after_flags(ctypes.byref(self.args), after_flags[0], after_flags[1], after_flags[2], st)
                if rc == _lib.ERR_UNSUPPORTED:
                    return None, None
                api._check(rc)
            else:
                api._check(self.lib.kda_fwd_k2(ctypes.byref(self.args), st))
        return self.o, self.ht


class SeqParallelPlan:
    """This rank's contiguous token segment of one long sequence, everything allocated once.

    ``q, k, v, g, beta`` hold the local ``T / world`` tokens (a multiple of 16; views are fine) and are
    re-read by every :meth:`run`; ``initial_state`` is the state before the FIRST segment (same
    tensor on every rank).  :meth:`run` launches K1, the transform pass, the exchange + fold and the
    final K2 on the current stream and returns ``(o_local, final_state)``: the state after the LAST
    segment on the last rank (from its own K2 pass), on every rank with ``final_state_on_all_ranks``,
    else ``None``.  In-kernel gate, l2-norm and beta sigmoid, V-first state.

    ``segments_per_rank``: a K2 pass is one serial chain per (batch, head), so a rank with few heads
    leaves most of its GPU idle; cutting the rank's tokens into 2 or 4 consecutive sub-segments
    (handled as batch entries of the same launches, no copy) runs that many chains side by side
    for the same total work.  ``peer_exchange``: ``"auto"`` (default; the environment variable
    ``KDA_B200_PEER_EXCHANGE=0`` turns it off), ``True`` (fail if it cannot be set up) or ``False``: the
    all-to-all exchange as stores and flags over peer memory instead of two NCCL collectives.
    ``segments_per_rank="auto"`` takes the largest of 4, 2 that keeps the chains of a pass at
    64 or fewer and the sub-segments at 2,048 tokens or more, else 1 (measured per rank on B200, 16
    heads x 16,384 tokens: K1 + transform pass + K2 = 1,060 us with one, 766 us with two, 605 us with
    four sub-segments).  The exchange stays that of one segment per rank: the rank composes its
    sub-segments' transforms into one before the exchange and walks them again after it.  Batch 1 only.
    """

    def __init__(self, q, k, v, g, beta, *, scale=None, initial_state=None, lower_bound=-5.0, A_log=None,
                 dt_bias=None, group=None, exchange="auto", final_state_on_all_ranks=False, segments_per_rank="auto",
                 peer_exchange="auto"):
        import torch.distributed as dist

        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        B, L, H = q.shape[0], q.shape[1], v.shape[2]
        sub = 1
        if segments_per_rank == "auto":
            if B == 1 and self.world > 1 and q.is_cuda:
                for cand in (4, 2):
                    if cand * H <= 64 and L % (cand * api.BT) == 0 and L // cand >= 2048:
                        sub = cand
                        break
        else:
            sub = int(segments_per_rank)
            if sub < 1 or (sub > 1 and (B != 1 or L % (sub * api.BT))):
                raise ValueError("segments_per_rank needs batch 1 and a token count that splits into multiples of 16")
        self.sub = sub
        if sub > 1:
            q, k, v, g, beta = (_sub_segments(x, sub) for x in (q, k, v, g, beta))
        self.seg = _Segment(q, k, v, g, beta, D ** -0.5 if scale is None else scale, lower_bound, A_log, dt_bias)
        self.chains = B * H
        self.h0 = None if initial_state is None else initial_state.contiguous().float()
        if exchange == "auto" and sub > 1 and self.world * sub <= 8:
            exchange = "gather"   # few segments: one all-gather of every sub-segment's transform, one flat walk
        self.mode = exchange_mode(self.chains, self.world, exchange)
        self.want_final = bool(final_state_on_all_ranks)
        self.bufs: dict = {}
        self.out_shape = (B, L, H, D)
        # The all-to-all runs over peer memory when the ranks can map each other's buffers (one box);
        # every rank takes the same decision (the set-up is collective), else the NCCL collectives.
        self.exchange_kind = "nccl"
        self._fused_push = os.environ.get("KDA_B200_FUSED_PUSH", "1") != "0"
        self._k2_waits = self._fused_push
        want_peer = peer_exchange is True or (peer_exchange == "auto" and os.environ.get("KDA_B200_PEER_EXCHANGE", "1") != "0")
        if self.world > 1 and self.mode == "a2a" and want_peer and q.is_cuda:
            peer = _PeerExchange.create(self.chains, self.world, self.rank, group, q.device)
            if peer is not None:
                self.bufs["peer"] = peer
                self.exchange_kind = "peer"
            elif peer_exchange is True:
                raise RuntimeError("the ranks could not map each other's memory: no peer exchange")

    def close(self):
        """Collective (call it on every rank, or on none): releases the peer mappings of the exchange, after
        which the plan's buffers may be freed and the plan must not run again."""
        peer = self.bufs.pop("peer", None)
        if peer is not None:
            peer.close()

    def run(self, timeline: Optional[list] = None):
        """One forward.  ``timeline``: a list that receives ``(phase, torch.cuda.Event)`` pairs
        recorded on the current stream after K1, the transform pass, the exchange + fold and K2
        (for per-phase timing)."""
        def mark(name):
            if timeline is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                timeline.append((name, ev))

        seg = self.seg
        mark("start")
        seg.k1()
        mark("k1")
        if self.world == 1:
            o, ht = seg.outputs(self.h0)
            mark("k2")
            return o, ht
        # One segment per rank over peer memory: the transform pass stores its tiles straight into the owners'
        # receive buffers (no copy kernel), where the library has a kernel for that (the 8-row pair form).
        peer = self.bufs.get("peer")
        pushed = False
        if peer is not None and self.sub == 1 and self._fused_push:
            rc = seg.transforms_push(peer.begin())
            if rc == _lib.ERR_UNSUPPORTED:          # the same answer on every rank: same shapes
                self._fused_push = False
                peer.epoch -= 1
            else:
                api._check(rc)
                pushed = True
        mq = seg.mq if pushed else seg.transforms()
        mark("transforms")
        entry, final = exchange_and_fold(mq, self.h0, self.rank, self.world, group=self.group, mode=self.mode,
                                         sub=self.sub, bufs=self.bufs, want_final=self.want_final, status=seg.ws,
                                         mark=mark if timeline is not None else None, pushed=pushed,
                                         defer_wait=self._k2_waits)
        mark("exchange_fold")
        pending = peer.pending if peer is not None else None
        if pending is not None:
            # the final pass waits for the entry states itself, behind its first record loads
            peer.pending = None
            o, ht = seg.outputs(entry.reshape(seg.B, seg.H, D, D), after_flags=pending)
            if o is None:                            # no kernel of that kind for this problem: wait, then the plain pass
                self._k2_waits = False
                with torch.cuda.device(seg.dev):
                    api._check(seg.lib.kda_flag_wait(pending[0], pending[1], pending[2], seg.ws.data_ptr(), api._stream_handle()))
                o, ht = seg.outputs(entry.reshape(seg.B, seg.H, D, D))
        else:
            o, ht = seg.outputs(entry.reshape(seg.B, seg.H, D, D))
        mark("k2")
        o = o.view(self.out_shape)
        if self.want_final:
            return o, final.view(self.out_shape[0], seg.H, D, D)
        return o, (ht[seg.B - self.out_shape[0]:] if self.rank == self.world - 1 else None)


def forward_seq_parallel(q, k, v, g, beta, *, scale=None, initial_state=None, lower_bound=-5.0,
                         A_log=None, dt_bias=None, group=None, exchange="auto"):
    """One-shot form of :class:`SeqParallelPlan`: returns ``(o_local, final_state)`` with the state
    after the LAST segment on every rank."""
    plan = SeqParallelPlan(q, k, v, g, beta, scale=scale, initial_state=initial_state, lower_bound=lower_bound,
                           A_log=A_log, dt_bias=dt_bias, group=group, exchange=exchange,
                           final_state_on_all_ranks=True)
    o, ht = plan.run()
    return o, ht.clone()


def forward_seq_split_local(q, k, v, g, beta, n_segments: int, *, scale=None, initial_state=None,
                            lower_bound=-5.0, A_log=None, dt_bias=None):
    """The same schedule on ONE GPU, segments standing in for ranks (no communication): K1 and
    the transform pass per segment, one fold over all segments, K2 per segment.  Used to check the
    split against the one-pass forward."""
    if scale is None:
        scale = D ** -0.5
    B, T, H, _ = q.shape
    if T % (n_segments * api.BT):
        raise ValueError("T must split into n_segments multiples of 16")
    L = T // n_segments
    mq = torch.empty((n_segments, B * H, 2, D, D), dtype=torch.float32, device=q.device)
    segs = [_Segment(q[:, j * L:(j + 1) * L], k[:, j * L:(j + 1) * L], v[:, j * L:(j + 1) * L],
                     g[:, j * L:(j + 1) * L], beta[:, j * L:(j + 1) * L], scale, lower_bound, A_log, dt_bias,
                     mq_out=mq[j])
            for j in range(n_segments)]
    for s_ in segs:
        s_.k1()
        s_.transforms()
    h0 = None if initial_state is None else initial_state.contiguous().float()
    states = fold_states(mq, h0)
    outs = [s_.outputs(states[j].view(B, H, D, D))[0] for j, s_ in enumerate(segs)]
    return torch.cat(outs, dim=1), states[n_segments].view(B, H, D, D).clone()
