"""Host side of the B200 KDA forward: the reference's Python forward API over the C ABI.

Two public signatures are kept so that callers of the reference can switch without
edits:

* ``kda_bt16_fwd`` / ``kda_bt16_debug`` -- names, argument order, defaults, return
  values and error behaviour of ``src/kda_bt16/kernels.py:752-850`` in the reference
  project (validation rules and messages follow ``_validate_kda_inputs``, ``:609-749``).
* ``kda_bt16_fwd_ascendc`` / ``get_last_profile`` -- the keyword interface of
  ``python/kda_ascendc_v1/api.py:759-804`` (``bias`` is ``[H, 128]`` there).

Everything numeric happens in ``libkda_b200.so`` (two CUDA kernels, see
``include/kda_b200.h``).  This module validates, allocates outputs and the K1->K2
workspace with ``torch.empty``, fills a ``KdaFwdArgs`` and launches on the current
CUDA stream without synchronising.  Inputs that are not CUDA tensors are refused:
there is no CPU path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib
from ._lib import KdaFwdArgs

BT = 16
HEAD_DIM = 128
REC_BYTES = 26112
WS_HEADER_BYTES = 256

_WORKSPACE_CACHE: dict[tuple, torch.Tensor] = {}
_LAST_PROFILE: dict[str, object] = {}
RECURRENT_MAX_TOKENS = 4   # kda_recurrent_fwd hands longer calls to the chunk kernels
_LAUNCH_COUNTS = {"kda_k1": 0, "kda_k2": 0, "kda_recurrent": 0}


# ---------------------------------------------------------------------------
# validation (same checks, order and messages as the reference's shared validator)
# ---------------------------------------------------------------------------
def _validate_kda_inputs(q, k, v, g, beta, initial_state, use_gate_in_kernel, safe_gate, lower_bound,
                         A_log, dt_bias, state_v_first, require_contiguous=True, n_states=None):
    for name, x, nd, lay in (("q", q, 4, "[B, T, H, D]"), ("k", k, 4, "[B, T, H, D]"),
                             ("v", v, 4, "[B, T, HV, V]"), ("g", g, 4, "[B, T, HV, D]"),
                             ("beta", beta, 3, "[B, T, HV]")):
        if x.ndim != nd:
            raise ValueError(f"{name} must be {nd}D {lay}, got {x.ndim}D with shape {tuple(x.shape)}")
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[-1]
    if min(B, T, H, K) <= 0:
        raise ValueError(f"q dimensions must be positive, got B={B}, T={T}, H={H}, K={K}")
    if HV <= 0 or V <= 0:
        raise ValueError(f"v dimensions must be positive, got HV={HV}, V={V}")

    if require_contiguous:
        if not q.is_contiguous():
            raise ValueError("q must be contiguous (kernel assumes stride [H*K, K, 1])")
        for name, x in (("k", k), ("v", v), ("g", g), ("beta", beta)):
            if not x.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
    else:
        for name, x in (("q", q), ("k", k), ("v", v), ("g", g)):
            if x.stride(-1) != 1:
                raise ValueError(f"{name} must be contiguous in its last dimension")

    for name, x in (("q", q), ("k", k), ("v", v)):
        if x.dtype != torch.bfloat16:
            raise TypeError(f"{name} must be bfloat16, got {x.dtype}")
    # the reference demands fp32 for the raw gate; bf16 is accepted as well here because
    # bf16 -> fp32 is exact and the kernel converts on load
    if g.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"g must be float32 (or bfloat16) when use_gate_in_kernel={use_gate_in_kernel}, got {g.dtype}")
    if beta.dtype != torch.float32:
        raise TypeError(f"beta must be float32, got {beta.dtype}")

    if k.shape != q.shape:
        raise ValueError(f"k.shape {tuple(k.shape)} must match q.shape {tuple(q.shape)}")
    if tuple(v.shape) != (B, T, HV, V):
        raise ValueError(f"v.shape {tuple(v.shape)} must be [B={B}, T={T}, HV={HV}, V={V}]")
    if tuple(g.shape) != (B, T, HV, K):
        raise ValueError(f"g.shape {tuple(g.shape)} must be [B={B}, T={T}, HV={HV}, K={K}]")
    if tuple(beta.shape) != (B, T, HV):
        raise ValueError(f"beta.shape {tuple(beta.shape)} must be [B={B}, T={T}, HV={HV}]")
    if not all(x.device == q.device for x in (k, v, g, beta)):
        raise ValueError(f"All tensors must be on same device as q ({q.device})")

    if initial_state is not None:
        if not initial_state.is_contiguous():
            raise ValueError("initial_state must be contiguous")
        if initial_state.dtype != torch.float32:
            raise TypeError(f"initial_state must be float32, got {initial_state.dtype}")
        if initial_state.device != q.device:
            raise ValueError(f"initial_state device {initial_state.device} must match q ({q.device})")
        ns = B if n_states is None else n_states   # packed sequences carry one state per sequence
        expected = (ns, HV, V, K) if state_v_first else (ns, HV, K, V)
        if tuple(initial_state.shape) != expected:
            raise ValueError(f"initial_state.shape {tuple(initial_state.shape)} must be {expected} "
                             f"(state_v_first={state_v_first})")
    if A_log is not None:
        if not A_log.is_contiguous():
            raise ValueError("A_log must be contiguous")
        if A_log.dtype != torch.float32:
            raise TypeError(f"A_log must be float32, got {A_log.dtype}")
        if A_log.device != q.device:
            raise ValueError("A_log device must match q")
        if tuple(A_log.shape) != (HV,):
            raise ValueError(f"A_log.shape {tuple(A_log.shape)} must be (HV={HV},)")
    if dt_bias is not None:
        if not dt_bias.is_contiguous():
            raise ValueError("dt_bias must be contiguous")
        if dt_bias.dtype != torch.float32:
            raise TypeError(f"dt_bias must be float32, got {dt_bias.dtype}")
        if dt_bias.device != q.device:
            raise ValueError("dt_bias device must match q")
        if tuple(dt_bias.shape) != (HV * K,):
            raise ValueError(f"dt_bias.shape {tuple(dt_bias.shape)} must be (HV*K={HV * K},)")

    if K != HEAD_DIM or V != HEAD_DIM:
        raise ValueError(f"prototype targets K=V=128, got K={K}, V={V}")
    # the reference rejects HV != H outright (src/kda_bt16/kernels.py:729-730); grouped value heads
    # (HV a multiple of H, value head h reading q/k head h // (HV // H)) are served here
    if HV % H != 0:
        raise ValueError(f"prototype targets MHA (HV == H) or grouped value heads (HV a multiple of H), "
                         f"got HV={HV}, H={H}")
    if use_gate_in_kernel:
        if not safe_gate:
            raise ValueError("use_gate_in_kernel requires safe_gate=True")
        if lower_bound is None:
            raise ValueError("use_gate_in_kernel requires lower_bound")
        if not (-11.0 < lower_bound < 0.0):
            raise ValueError("lower_bound must be in range (-11, 0) to prevent fp32 exp2 overflow "
                             f"(BT=16 can amplify exponent by ~8x), got {lower_bound}")
        if A_log is None:
            raise ValueError("use_gate_in_kernel requires A_log")
    return B, T, H, K, HV, V


def _require_cuda(q: torch.Tensor) -> None:
    if q.device.type != "cuda":
        raise RuntimeError("kda_ascendc_b200 runs on CUDA (sm_100a) tensors only; got device %s "
                           "(there is no CPU fallback)" % q.device)


# ---------------------------------------------------------------------------
# launch plumbing
# ---------------------------------------------------------------------------
def workspace_bytes(B: int, T: int, H: int) -> int:
    return int(_lib.load().kda_fwd_workspace_bytes(B, T, H))


def _strides3(x: torch.Tensor):
    return (ctypes.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))


def _ptr(x: Optional[torch.Tensor]):
    return None if x is None else ctypes.c_void_p(x.data_ptr())


def make_args(q, k, v, g, beta, *, scale, lower_bound, A_log, dt_bias, h0, o, ht, workspace,
              flags, g_out=None, ainv_out=None, k2_vsplit=0, k2_variant=0) -> KdaFwdArgs:
    """Fill the C argument block from (possibly strided) tensors; keeps no references."""
    B, T, Hq, _ = q.shape
    H = v.shape[2]          # heads of v, g, beta, o, states; q and k may have fewer (grouped value heads)
    a = KdaFwdArgs()
    a.q, a.k, a.v, a.g, a.beta = _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta)
    a.A_log, a.dt_bias, a.h0 = _ptr(A_log), _ptr(dt_bias), _ptr(h0)
    a.o, a.ht, a.workspace = _ptr(o), _ptr(ht), _ptr(workspace)
    a.g_out, a.ainv_out = _ptr(g_out), _ptr(ainv_out)
    a.B, a.T, a.H = B, T, H
    a.Hq = 0 if Hq == H else Hq
    a.g_dtype = _lib.KDA_G_BF16 if g.dtype == torch.bfloat16 else _lib.KDA_G_FP32
    a.q_stride, a.k_stride, a.v_stride, a.g_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(g)
    a.o_stride = _strides3(o) if o is not None else (ctypes.c_int64 * 3)(0, 0, 0)
    a.beta_stride = (ctypes.c_int64 * 3)(beta.stride(0), beta.stride(1), beta.stride(2))
    a.scale = float(scale)
    a.lower_bound = float(lower_bound if lower_bound is not None else -5.0)
    a.flags = int(flags)
    a.k2_vsplit = int(k2_vsplit)
    a.k2_variant = int(k2_variant)
    return a


def _check(rc: int) -> None:
    if rc != 0:
        msg = _lib.last_error()
        if rc == -1:
            raise ValueError(msg)
        raise RuntimeError(msg)


def _stream_handle() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check_device_status(workspace: torch.Tensor) -> int:
    """Synchronising read of the workspace status word; raises if a bounded wait gave up."""
    st = ctypes.c_int32(0)
    rc = _lib.load().kda_fwd_status(_ptr(workspace), _stream_handle(), ctypes.byref(st))
    _check(rc)
    return st.value


K2_FORMS = {1: "n8", 3: "m16", 4: "tc", 5: "la"}


def k2_choice(B: int, T: int, H: int, *, state_only: bool = False, n_seqs: int = 0, n_chunks: int = 0,
              sm_count: int = 0) -> tuple[str, int]:
    """(organisation, CTAs per chain) of K2 for a problem, as the library's automatic choice
    resolves it: "n8" / "m16" (``mma.sync``, 8 / 16 state rows per warp) or "tc" (tcgen05, the
    state in tensor memory).  Host logic only; ``sm_count=0`` takes the current device's."""
    a = _lib.KdaFwdArgs()
    a.B, a.T, a.H, a.n_seqs, a.n_chunks = B, T, H, n_seqs, n_chunks
    var, vs = ctypes.c_int32(0), ctypes.c_int32(0)
    _check(_lib.load().kda_fwd_k2_choice(ctypes.byref(a), int(state_only), sm_count, ctypes.byref(var), ctypes.byref(vs)))
    return K2_FORMS[var.value], vs.value


def _get_workspace(device, B, T, H, reuse: bool) -> torch.Tensor:
    nbytes = workspace_bytes(B, T, H)
    if reuse:
        key = (device, B, T, H)
        ws = _WORKSPACE_CACHE.get(key)
        if ws is None:
            ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
            _WORKSPACE_CACHE[key] = ws
        return ws
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def _varlen_tables(cu_seqlens, T: int, H: int, device):
    """(n_seqs, n_chunks, chunk_table, seq_table) for packed sequences; tables on ``device``.

    ``cu_seqlens``: 1-D integer tensor (any device) or sequence, ``[0, ..., T]``, non-decreasing,
    no empty sequence.  The tables are built on the host by the library's own helper (one
    device-to-host read if ``cu_seqlens`` lives on the GPU) and copied over.
    """
    cu = torch.as_tensor(cu_seqlens).detach().to("cpu", torch.int32).contiguous()
    if cu.ndim != 1 or cu.numel() < 2:
        raise ValueError("cu_seqlens must be 1-D with at least two entries")
    if int(cu[-1]) != T:
        raise ValueError(f"cu_seqlens must end at the number of packed tokens T={T}, got {int(cu[-1])}")
    n_seqs = cu.numel() - 1
    lib = _lib.load()
    i32p = ctypes.POINTER(ctypes.c_int32)
    cu_p = ctypes.cast(cu.data_ptr(), i32p)
    n_chunks = lib.kda_varlen_fill_tables(cu_p, n_seqs, H, None, None)
    _check(min(n_chunks, 0))
    host = torch.empty((n_chunks + n_seqs, 4), dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
        else torch.empty((n_chunks + n_seqs, 4), dtype=torch.int32)
    rc = lib.kda_varlen_fill_tables(cu_p, n_seqs, H, ctypes.cast(host.data_ptr(), i32p),
                                    ctypes.cast(host[n_chunks:].data_ptr(), i32p))
    _check(min(rc, 0))
    dev_tab = host.to(device, non_blocking=True)
    return n_seqs, n_chunks, dev_tab[:n_chunks], dev_tab[n_chunks:], host


def _flags(use_gate, use_l2, use_beta_sigmoid) -> int:
    return ((_lib.FLAG_GATE if use_gate else 0) | (_lib.FLAG_L2NORM if use_l2 else 0) |
            (_lib.FLAG_BETA_SIGMOID if use_beta_sigmoid else 0))


def _forward(q, k, v, g, beta, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
             use_gate_in_kernel, use_beta_sigmoid_in_kernel, lower_bound, A_log, dt_bias, state_v_first,
             return_intermediates=False, reuse_workspace=False, k2_vsplit=0, k2_variant=0, workspace=None,
             cu_seqlens=None):
    """Allocate, launch K1 + K2 on the current stream, return (o, ht[, intermediates])."""
    lib = _lib.load()
    B, T, _, K = q.shape
    H = v.shape[2]
    dev = q.device
    h0 = initial_state   # either layout is read and written in place by the chunk kernels
    o = torch.empty((B, T, H, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    n_states, ws_tokens, tables = B, T, None
    if cu_seqlens is not None:
        tables = _varlen_tables(cu_seqlens, T, H, dev)
        n_states, ws_tokens = tables[0], BT * tables[1]
    ht = torch.empty((n_states, H, HEAD_DIM, HEAD_DIM), dtype=torch.float32, device=dev) if output_final_state else None
    ws = workspace if workspace is not None else _get_workspace(dev, B, ws_tokens, H, reuse_workspace)
    g_out = ainv = None
    if return_intermediates:
        g_out = torch.empty((B, T, H, HEAD_DIM), dtype=torch.float32, device=dev)
        ainv = torch.empty((B, T, H, BT), dtype=torch.float32, device=dev)
    args = make_args(q, k, v, g, beta, scale=scale, lower_bound=lower_bound, A_log=A_log, dt_bias=dt_bias,
                     h0=h0, o=o, ht=ht, workspace=ws, g_out=g_out, ainv_out=ainv, k2_vsplit=k2_vsplit,
                     k2_variant=k2_variant,
                     flags=_flags(use_gate_in_kernel, use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel) |
                     (0 if state_v_first else _lib.FLAG_STATE_K_FIRST))
    if tables is not None:
        args.n_seqs, args.n_chunks = tables[0], tables[1]
        args.chunk_table, args.seq_table = _ptr(tables[2]), _ptr(tables[3])
    stream = _stream_handle()
    profile = os.environ.get("KDA_PROFILE", "0") == "1"
    with torch.cuda.device(dev):
        if profile:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            _check(lib.kda_fwd_k1(ctypes.byref(args), stream))
            ev[1].record()
            _check(lib.kda_fwd_k2(ctypes.byref(args), stream))
            ev[2].record()
            ev[2].synchronize()
            _LAST_PROFILE.clear()
            _LAST_PROFILE.update(k1_ms=ev[0].elapsed_time(ev[1]), k2_ms=ev[1].elapsed_time(ev[2]),
                                 shape=(B, T, H), workspace_bytes=ws.numel())
        else:
            _check(lib.kda_fwd(ctypes.byref(args), stream))
    _LAUNCH_COUNTS["kda_k1"] += 1
    _LAUNCH_COUNTS["kda_k2"] += 1
    if return_intermediates:
        from .layout import unpack_records
        inter = unpack_records(ws, B, T, H)
        inter["g"] = g_out
        inter["A_inv"] = ainv
        return o, ht, inter
    return o, ht


def kda_recurrent_fwd(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=True,
                      lower_bound=-5.0, A_log=None, dt_bias=None, inplace_state=False, state_v_first=True):
    """Token-by-token KDA recurrence for decode steps and short sequences.

    Same tensors as :func:`kda_bt16_fwd` with the in-kernel gate, l2-norm and beta sigmoid
    (``g`` raw, ``beta`` logits, ``A_log`` required), any ``T >= 1`` (calls of more than
    ``RECURRENT_MAX_TOKENS`` tokens run on the chunk kernels, which are faster from there on), fp32
    state ``[B, H, V, K]`` or, with ``state_v_first=False``, ``[B, H, K, V]`` (read and written in
    that layout by the kernels, no transpose).  Returns ``(o, state)``; with
    ``inplace_state=True`` the new state overwrites ``initial_state`` (which is returned).
    The reference has no decode function; the arithmetic is the token recurrence its tests use
    as the gold (``fused_recurrent_kda``, ``tests/test_kda_bt16.py:26-39`` of the reference) with
    the chunk path's bf16 rounding of the normalised q and k, so that a prefill by
    :func:`kda_bt16_fwd` followed by steps of this function continues the same sequence.
    """
    _validate_kda_inputs(q, k, v, g, beta, initial_state, True, True, lower_bound, A_log, dt_bias, state_v_first,
                         require_contiguous=False)
    _require_cuda(q)
    if inplace_state and initial_state is None:
        raise ValueError("inplace_state=True needs an initial_state to update")
    if initial_state is not None and not initial_state.is_contiguous():
        raise ValueError("initial_state must be contiguous")
    B, T, _, K = q.shape
    H = v.shape[2]
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    o = torch.empty((B, T, H, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    if inplace_state:
        ht = initial_state
    else:
        ht = torch.empty((B, H, HEAD_DIM, HEAD_DIM), dtype=torch.float32, device=dev) if output_final_state else None
    # Beyond RECURRENT_MAX_TOKENS tokens per call the chunk kernels are faster (measured on B200, B64 H32:
    # 4 tokens 88 us token by token against 104 us as one chunk, 8 tokens 151 us against 105 us, 16 tokens
    # 279 us against 107 us); each K2 CTA reads its rows of the state before it writes them, so the in-place
    # update carries over.
    chunked = T > RECURRENT_MAX_TOKENS
    ws = _get_workspace(dev, B, T, H, True) if chunked else None
    args = make_args(q, k, v, g, beta, scale=scale, lower_bound=lower_bound, A_log=A_log, dt_bias=dt_bias,
                     h0=initial_state, o=o, ht=ht, workspace=ws,
                     flags=_flags(True, True, True) | (0 if state_v_first else _lib.FLAG_STATE_K_FIRST))
    lib = _lib.load()
    with torch.cuda.device(dev):
        _check((lib.kda_fwd if chunked else lib.kda_recurrent_fwd)(ctypes.byref(args), _stream_handle()))
    _LAUNCH_COUNTS["kda_recurrent"] += 1
    return o, ht


class ForwardPlan:
    """The chunk forward on fixed buffers without per-call host work: validation, outputs, scratch
    and the argument block are made once, :meth:`run` is one C call (K1 + K2 on the current stream).

    For loops that refill the same input tensors (serving with static shapes, benchmarks).  ``o`` and
    ``final_state`` belong to the plan and are overwritten by every run.  In-kernel gate, l2-norm and
    beta sigmoid, V-first state; ``cu_seqlens`` as in :func:`kda_bt16_fwd`.
    """

    def __init__(self, q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=True,
                 lower_bound=-5.0, A_log=None, dt_bias=None, cu_seqlens=None):
        n_states = None if cu_seqlens is None else len(cu_seqlens) - 1
        if cu_seqlens is not None and q.ndim == 4 and q.shape[0] != 1:
            raise ValueError(f"cu_seqlens needs a packed batch of size 1, got B={q.shape[0]}")
        _validate_kda_inputs(q, k, v, g, beta, initial_state, True, True, lower_bound, A_log, dt_bias, True,
                             n_states=n_states)
        _require_cuda(q)
        B, T, _, K = q.shape
        H = v.shape[2]
        self.device = q.device
        tables = None if cu_seqlens is None else _varlen_tables(cu_seqlens, T, H, q.device)
        ns = B if tables is None else tables[0]
        self.o = torch.empty((B, T, H, HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        self.final_state = (torch.empty((ns, H, HEAD_DIM, HEAD_DIM), dtype=torch.float32, device=q.device)
                            if output_final_state else None)
        self._ws = torch.empty(workspace_bytes(B, T if tables is None else BT * tables[1], H), dtype=torch.uint8,
                               device=q.device)
        self._keep = (q, k, v, g, beta, A_log, dt_bias, initial_state, tables)   # the argument block holds raw pointers
        self._args = make_args(q, k, v, g, beta, scale=K ** -0.5 if scale is None else scale, lower_bound=lower_bound,
                               A_log=A_log, dt_bias=dt_bias, h0=initial_state, o=self.o, ht=self.final_state,
                               workspace=self._ws, flags=_flags(True, True, True))
        if tables is not None:
            self._args.n_seqs, self._args.n_chunks = tables[0], tables[1]
            self._args.chunk_table, self._args.seq_table = _ptr(tables[2]), _ptr(tables[3])
        self._ref = ctypes.byref(self._args)
        self._fn = _lib.load().kda_fwd

    def run(self, stream: Optional[int] = None):
        """One forward over the current contents of the input buffers; returns ``(o, final_state)``."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _call_on_device(self.device, self._fn, self._ref, ctypes.c_void_p(stream))
        if rc != 0:
            _check(rc)
        _LAUNCH_COUNTS["kda_k1"] += 1
        _LAUNCH_COUNTS["kda_k2"] += 1
        return self.o, self.final_state


def _call_on_device(device, fn, *args):
    """Call a C entry point with ``device`` current.  The library sizes grids, caches kernel
    attributes and resolves tensor maps for the CURRENT device, so a process that drives several
    GPUs must not run a plan built for one of them while another is current."""
    if torch.cuda.current_device() == device.index:
        return fn(*args)
    with torch.cuda.device(device):
        return fn(*args)


class RecurrentPlan:
    """Decode loop without per-step host work: fixed input buffers, in-place state, one C call per step.

    A serving loop writes each new token's ``q, k, v, g, beta`` into the SAME tensors and calls
    :meth:`step`; validation, output allocation and the argument block are done once here.  ``o``
    is reused by every step (copy it if it must outlive the next one); ``state`` is updated in
    place (``[B, H, V, K]``, or ``[B, H, K, V]`` with ``state_v_first=False``).  Same arithmetic and
    checks as :func:`kda_recurrent_fwd`.
    """

    def __init__(self, q, k, v, g, beta, state, *, scale=None, lower_bound=-5.0, A_log=None, dt_bias=None,
                 state_v_first=True):
        _validate_kda_inputs(q, k, v, g, beta, state, True, True, lower_bound, A_log, dt_bias, state_v_first,
                             require_contiguous=False)
        _require_cuda(q)
        if state is None:
            raise ValueError("RecurrentPlan needs the state tensor it updates in place")
        B, T, _, K = q.shape
        self.device = q.device
        self.o = torch.empty((B, T, v.shape[2], HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        self.state = state
        self._keep = (q, k, v, g, beta, A_log, dt_bias)   # the argument block holds raw pointers
        self._args = make_args(q, k, v, g, beta, scale=K ** -0.5 if scale is None else scale, lower_bound=lower_bound,
                               A_log=A_log, dt_bias=dt_bias, h0=state, o=self.o, ht=state, workspace=None,
                               flags=_flags(True, True, True) | (0 if state_v_first else _lib.FLAG_STATE_K_FIRST))
        self._ref = ctypes.byref(self._args)
        self._fn = _lib.load().kda_recurrent_fwd

    def step(self, stream: Optional[int] = None):
        """Apply the tokens currently in the input buffers; returns ``o`` (the plan's own tensor).
        ``stream``: raw CUDA stream handle; default = the current torch stream of the plan's device."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _call_on_device(self.device, self._fn, self._ref, ctypes.c_void_p(stream))
        if rc != 0:
            _check(rc)
        _LAUNCH_COUNTS["kda_recurrent"] += 1
        return self.o


# ---------------------------------------------------------------------------
# public API, reference signature 1: src/kda_bt16/kernels.py:752-850
# ---------------------------------------------------------------------------
def kda_bt16_fwd(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                 use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
                 safe_gate=True, lower_bound=-5.0, A_log=None, dt_bias=None, state_v_first=True,
                 use_fused_kernel=False, reuse_workspace=False, cu_seqlens=None):
    """KDA forward, chunk size 16.

    q/k: ``[B, T, H, 128]`` bf16; v: ``[B, T, H, 128]`` bf16; g: raw gate ``[B, T, H, 128]``
    (fp32, or bf16) when ``use_gate_in_kernel`` else the chunk-local log2 cumsum; beta:
    ``[B, T, H]`` fp32 (logits when ``use_beta_sigmoid_in_kernel``); initial_state: fp32
    ``[B, H, V, K]`` (or ``[B, H, K, V]`` with ``state_v_first=False``).  Returns ``(o, ht)``
    with ``o`` bf16 ``[B, T, H, 128]`` and ``ht`` the fp32 final state or ``None``.

    ``use_fused_kernel`` is accepted for signature compatibility: the reference's
    single-kernel variant computes the same function, and this build has one device path.
    ``reuse_workspace`` caches only the internal scratch per shape (never the outputs).

    ``cu_seqlens`` (not in the reference, which lists variable-length input as future work,
    ``README.md:509``; the convention is that of ``chunk_kda`` in flash-linear-attention): packed
    sequences in one ``[1, T, H, 128]`` batch, ``cu_seqlens = [0, ..., T]``; every sequence is
    chunked from its own first token, ``initial_state`` / the returned state are
    ``[n_seqs, H, 128, 128]``.
    """
    n_states = None
    if cu_seqlens is not None:
        if q.ndim == 4 and q.shape[0] != 1:
            raise ValueError(f"cu_seqlens needs a packed batch of size 1, got B={q.shape[0]}")
        n_states = len(cu_seqlens) - 1
    _validate_kda_inputs(q, k, v, g, beta, initial_state, use_gate_in_kernel, safe_gate, lower_bound,
                         A_log, dt_bias, state_v_first, n_states=n_states)
    _require_cuda(q)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _forward(q, k, v, g, beta, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
                    use_gate_in_kernel, use_beta_sigmoid_in_kernel, lower_bound, A_log, dt_bias, state_v_first,
                    reuse_workspace=reuse_workspace, cu_seqlens=cu_seqlens)


def kda_bt16_debug(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                   use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
                   safe_gate=True, lower_bound=-5.0, A_log=None, dt_bias=None, state_v_first=True):
    """Like :func:`kda_bt16_fwd`, and also returns the per-chunk intermediates
    ``{Aqk, A_inv, w, u, g}`` in the public ``[B, T, H, *]`` layout (plus ``qg``, ``kg``,
    ``dec``, which this build hands from K1 to K2) for stage-wise validation."""
    _validate_kda_inputs(q, k, v, g, beta, initial_state, use_gate_in_kernel, safe_gate, lower_bound,
                         A_log, dt_bias, state_v_first)
    _require_cuda(q)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _forward(q, k, v, g, beta, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
                    use_gate_in_kernel, use_beta_sigmoid_in_kernel, lower_bound, A_log, dt_bias, state_v_first,
                    return_intermediates=True)


# ---------------------------------------------------------------------------
# public API, reference signature 2: python/kda_ascendc_v1/api.py:759-804
# ---------------------------------------------------------------------------
PERSISTENT_LOOP = "persistent_loop"
CHUNK = BT


def _check_inputs_ascendc(q, k, v, g, beta, A_log, bias, initial_state):
    """Input rules of the reference's second API (python/kda_ascendc_v1/api.py:724-744)."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("q/k/v must be BF16")
    if q.ndim != 4 or tuple(q.shape) != tuple(k.shape) or tuple(q.shape) != tuple(v.shape):
        raise ValueError("q/k/v must have identical [B,T,H,128] shape")
    b, t, h, d = q.shape
    if d != HEAD_DIM or t < CHUNK or t % CHUNK:
        raise ValueError("support is T>=%d, T%%%d==0, D=128" % (CHUNK, CHUNK))
    if g.shape != q.shape or g.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("g must be FP32 [B,T,H,128]")
    if tuple(beta.shape) != (b, t, h) or beta.dtype != torch.float32:
        raise ValueError("beta must be FP32 [B,T,H]")
    if A_log is None or tuple(A_log.shape) != (h,) or A_log.dtype != torch.float32:
        raise ValueError("A_log must be FP32 [H]")
    if bias is not None and (tuple(bias.shape) != (h, HEAD_DIM) or bias.dtype != torch.float32):
        raise ValueError("bias must be FP32 [H,128]")
    if initial_state is not None and (tuple(initial_state.shape) != (b, h, HEAD_DIM, HEAD_DIM)
                                      or initial_state.dtype != torch.float32):
        raise ValueError("initial_state must be FP32 [B,H,128,128]")
    return b, t, h


def kda_bt16_fwd_ascendc(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                         A_log=None, bias=None, lower_bound=-5.0, return_intermediates=False, k2_mode=None):
    """Keyword interface of the reference's second backend.  Gate, l2-norm and beta sigmoid
    are always applied in-kernel; ``bias`` is ``[H, 128]``; the state is V-first
    ``[B, H, 128, 128]``.  Only ``k2_mode`` ``None`` / ``"persistent_loop"`` exists."""
    if k2_mode not in (None, PERSISTENT_LOOP):
        raise ValueError("unsupported k2_mode %r (choose from %s)" % (k2_mode, PERSISTENT_LOOP))
    _check_inputs_ascendc(q, k, v, g, beta, A_log, bias, initial_state)
    _require_cuda(q)
    if scale is None:
        scale = HEAD_DIM ** -0.5
    dt_bias = None if bias is None else bias.contiguous().reshape(-1)
    res = _forward(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), beta.contiguous(), scale,
                   None if initial_state is None else initial_state.contiguous(), output_final_state,
                   True, True, True, lower_bound, A_log.contiguous(), dt_bias, True,
                   return_intermediates=return_intermediates)
    if return_intermediates:
        return res[0], res[1], res[2]
    return res


def get_last_profile() -> dict:
    """Stage timings of the last call made with ``KDA_PROFILE=1`` plus launch counters."""
    prof = dict(_LAST_PROFILE)
    prof["launch_counts"] = dict(_LAUNCH_COUNTS)
    prof["launch_total"] = sum(_LAUNCH_COUNTS.values())
    prof["library"] = _lib.load().kda_version().decode()
    return prof
