"""CPU oracle for the KDA chunked forward at chunk size 16.  TEST INFRASTRUCTURE ONLY.

This file is the checker, never the product: only the test-suite, the smoke
entry and the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may
import it.  The shipped forward lives in ``kda_ascendc_b200`` and runs on the
GPU through the C-ABI library; it never calls anything in here.

What is restated (reference project paths, ``file:line``):

* ``chunk_reference``  -- the reference's own torch chunk implementation,
  ``tests/test_torch_reference.py:23-213`` (``torch_reference_kda_bt16``):
  l2-norm with eps 1e-6 and a cast of the normalised q/k back to the input
  dtype (``:77-81``), beta sigmoid (``:84``), the gate
  ``lower_bound * sigmoid(exp(A_log) * (g + dt_bias)) * RCP_LN2`` followed by a
  cumsum that restarts every 16 tokens (``:86-106``), mid-row re-centred Grams
  (``:142-156``), the unit-lower solve carried in float64 (``:158-166``), w/u
  (``:168-173``) and the state recurrence / output for both state layouts
  (``:175-211``).  ``loop_heads=True`` walks (chunk, batch, head) one tile at a
  time exactly like the reference does (that is what its CPU cost is made of);
  ``loop_heads=False`` evaluates all (batch, head) tiles of a chunk in one
  batched call and is ~10x faster, for the larger parity cases.
* ``recurrent_gold``   -- the token-by-token delta rule the reference tests use
  as mathematical gold (FLA ``fused_recurrent_kda``, a third-party dependency
  that the reference does not vendor or pin: ``pyproject.toml:31``,
  ``tests/test_kda_bt16.py:26-39``).  Its published recurrence is restated in
  float64: ``S <- S*diag(exp(gate_t)); v' = beta_t (v_t - S k_t);
  S <- S + v' (x) k_t; o_t = scale * S q_t``.
* ``make_inputs``      -- seeded synthetic tensors with the shapes and value
  distributions of the reference benchmark (``benchmarks/bench_bt16.py:26-35``)
  and of its small-magnitude device tests
  (``tests/test_chunk_shape_matrix.py:53-63``).

Pinning: ``tests/golden/`` holds input seeds and outputs produced by importing
the reference's ``torch_reference_kda_bt16`` itself (script committed beside
the fixtures); ``tests/test_oracle.py`` checks this restatement against them.
"""
from __future__ import annotations

import math

import torch

BT = 16
D = 128
EPS = 1e-6
RCP_LN2 = 1.44269504089  # the literal used by tests/test_torch_reference.py:87


# --------------------------------------------------------------------------
# shared front end: normalisation, beta, gate, chunk-local cumsum
# --------------------------------------------------------------------------
def _l2norm(x: torch.Tensor, keep_dtype: bool) -> torch.Tensor:
    xf = x.float()
    y = xf / torch.sqrt((xf * xf).sum(-1, keepdim=True) + EPS)
    return y.to(x.dtype) if keep_dtype else y


def gate_log2(g, A_log, dt_bias, lower_bound, dtype=torch.float32):
    """Per-token log2-domain gate (before the cumsum), shape [B,T,H,D]."""
    B, T, H, Dk = g.shape
    x = g.to(dtype)
    if A_log is not None:
        if dt_bias is not None:
            x = x + dt_bias.to(dtype).view(H, Dk)[None, None]
        x = torch.exp(A_log.to(dtype))[None, None, :, None] * x
    return lower_bound * torch.sigmoid(x) * RCP_LN2


def chunk_cumsum(gate: torch.Tensor) -> torch.Tensor:
    """Cumsum over T restarting at every multiple of 16."""
    out = torch.empty_like(gate)
    T = gate.shape[1]
    for s in range(0, T, BT):
        out[:, s:s + BT] = torch.cumsum(gate[:, s:s + BT], dim=1)
    return out


def _unit_lower_inverse(L: torch.Tensor) -> torch.Tensor:
    """(I + L)^-1 for strictly-lower L [..., n, n], row forward substitution in float64."""
    n = L.shape[-1]
    L64 = L.double()
    X = torch.eye(n, dtype=torch.float64).expand(L.shape).clone()
    for i in range(1, n):
        # row i of the inverse: e_i - sum_{j<i} L[i,j] * X[j,:]
        X[..., i, :] = X[..., i, :] - (L64[..., i, :i, None] * X[..., :i, :]).sum(-2)
    return X.float()


def _unit_lower_inverse_rowwise(L: torch.Tensor) -> torch.Tensor:
    """Same inverse, scalar (i, j) double loop -- the reference's operation order."""
    n = L.shape[-1]
    L64 = L.double()
    X = torch.eye(n, dtype=torch.float64)
    for i in range(1, n):
        for j in range(i):
            X[i, :] -= L64[i, j] * X[j, :]
    return X.float()


def chunk_terms(qn, kn, vc, gc, bc, scale, rowwise_solve=False):
    """State-independent per-chunk quantities.

    qn, kn, vc, gc: [..., n, 128] fp32 (n <= 16 valid rows); bc: [..., n].
    Returns dict(w, u, qg, kg, Aqk, dec, Ainv) -- the K1 stage of the reference
    pipeline in oracle precision (fp32, fp64 solve).
    """
    n = qn.shape[-2]
    mid = min(BT // 2, n - 1)
    gm = gc - gc[..., mid:mid + 1, :]
    e_pos, e_neg = torch.exp2(gm), torch.exp2(-gm)
    kneg_t = (kn * e_neg).transpose(-1, -2)
    Aqk = torch.tril(torch.matmul(qn * e_pos, kneg_t) * scale)
    Akk = torch.tril(torch.matmul(kn * e_pos, kneg_t) * bc[..., :, None], diagonal=-1)
    Ainv = _unit_lower_inverse_rowwise(Akk) if rowwise_solve else _unit_lower_inverse(Akk)
    w = torch.matmul(Ainv, kn * bc[..., :, None] * torch.exp2(gc))
    u = torch.matmul(Ainv, vc * bc[..., :, None])
    g_last = gc[..., n - 1, :]
    kg = kn * torch.exp2(g_last[..., None, :] - gc)
    qg = qn * torch.exp2(gc)
    return dict(w=w, u=u, qg=qg, kg=kg, Aqk=Aqk, dec=torch.exp2(g_last), Ainv=Ainv, Akk=Akk)


def chunk_state_step(h, t, scale):
    """One chunk of the recurrence on a V-first state h [..., V, K]; returns (o, h_next)."""
    ht = h.transpose(-1, -2)
    v_new = t["u"] - torch.matmul(t["w"], ht)
    o = torch.matmul(t["qg"], ht) * scale + torch.matmul(t["Aqk"], v_new)
    h = h * t["dec"][..., None, :]
    h = h + torch.matmul(v_new.transpose(-1, -2), t["kg"])
    return o, h


def chunk_reference(q, k, v, g, beta, scale=None, lower_bound=-5.0, A_log=None, dt_bias=None,
                    initial_state=None, state_v_first=True, loop_heads=False,
                    return_intermediates=False):
    """Chunked (BT=16) KDA forward in oracle precision.

    q, k, v: [B,T,H,128] (any float dtype; normalised q/k are cast back to it);
    g: raw gate [B,T,H,128]; beta: logits [B,T,H]; A_log [H]; dt_bias [H*128];
    initial_state: fp32 [B,H,V,K] (V-first) or [B,H,K,V].
    Returns (o [B,T,H,128] in q.dtype, final_state fp32) (+ dict of per-chunk
    intermediates in chunk-major order when return_intermediates).
    """
    B, T, H, Dk = q.shape
    if scale is None:
        scale = Dk ** -0.5
    qn = _l2norm(q, keep_dtype=True).float()
    kn = _l2norm(k, keep_dtype=True).float()
    bs = torch.sigmoid(beta.float())
    gc = chunk_cumsum(gate_log2(g.float(), A_log, dt_bias, lower_bound))
    vf = v.float()

    if initial_state is None:
        h = torch.zeros(B, H, Dk, Dk, dtype=torch.float32)
    else:
        h = initial_state.float().clone()
        if not state_v_first:
            h = h.transpose(-1, -2).contiguous()
    o = torch.zeros(B, T, H, Dk, dtype=q.dtype)
    inter = [] if return_intermediates else None

    for s in range(0, T, BT):
        e = min(s + BT, T)
        if loop_heads:
            for b in range(B):
                for hh in range(H):
                    t = chunk_terms(qn[b, s:e, hh], kn[b, s:e, hh], vf[b, s:e, hh], gc[b, s:e, hh],
                                    bs[b, s:e, hh], scale, rowwise_solve=True)
                    oc, hn = chunk_state_step(h[b, hh], t, scale)
                    o[b, s:e, hh] = oc.to(q.dtype)
                    h[b, hh] = hn
        else:
            sl = lambda x: x[:, s:e].transpose(1, 2)  # [B,H,n,D]
            t = chunk_terms(sl(qn), sl(kn), sl(vf), sl(gc), bs[:, s:e].transpose(1, 2), scale)
            oc, h = chunk_state_step(h, t, scale)
            o[:, s:e] = oc.transpose(1, 2).to(q.dtype)
            if inter is not None:
                inter.append(t)
    if not state_v_first:
        h = h.transpose(-1, -2).contiguous()
    if return_intermediates:
        return o, h, dict(g=gc, chunks=inter)
    return o, h


def recurrent_gold(q, k, v, g, beta, scale=None, lower_bound=-5.0, A_log=None, dt_bias=None,
                   initial_state=None):
    """float64 token-by-token delta rule; V-first state.  q/k are NOT re-rounded."""
    B, T, H, Dk = q.shape
    if scale is None:
        scale = Dk ** -0.5
    f64 = torch.float64
    qd, kd = q.double(), k.double()
    qn = qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + EPS)
    kn = kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + EPS)
    bs = torch.sigmoid(beta.double())
    gate = gate_log2(g, A_log, dt_bias, lower_bound, dtype=f64)  # log2 domain
    decay = torch.exp2(gate)  # == exp(natural-log gate) up to the RCP_LN2 literal
    vd = v.double()
    S = torch.zeros(B, H, Dk, Dk, dtype=f64) if initial_state is None else initial_state.double().clone()
    o = torch.empty(B, T, H, Dk, dtype=f64)
    for t in range(T):
        S = S * decay[:, t, :, None, :]
        pred = torch.einsum("bhvk,bhk->bhv", S, kn[:, t])
        vp = bs[:, t, :, None] * (vd[:, t] - pred)
        S = S + vp[..., :, None] * kn[:, t, :, None, :]
        o[:, t] = scale * torch.einsum("bhvk,bhk->bhv", S, qn[:, t])
    return o, S


# --------------------------------------------------------------------------
# seeded synthetic inputs
# --------------------------------------------------------------------------
def make_inputs(B, T, H, seed0=42, regime="baseline", h0_std=None, g_dtype=torch.bfloat16,
                head_offset=0, t_offset=0, t_total=None):
    """Seeded CPU tensors; one generator per (global) head so that any head shard
    or sequence segment of a larger problem sees the values the whole problem has.

    regime "baseline": q,k,v,g_raw ~ N(0,1) bf16; beta logits ~ N(0,1);
        A_log = log U(1,16); dt_bias ~ U(-0.1,0.1); lower_bound -5.
    regime "long_memory": small-magnitude inputs with slow decay
        (q,k ~ 0.2 N, v ~ 0.1 N, g ~ 0.1 N, A_log in [-1,0.2], bias ~ 0.03 N,
        lower_bound -1) so that the state carries across many chunks.
    regime "carry": almost no decay (gate input ~ N(-6, 0.3), A_log ~ 0, lower_bound -1):
        what a segment leaves in the state is still there many segments later, so a wrong
        state hand-over between segments cannot hide.
    h0_std: None -> no initial state; 0.0 -> zeros; else N(0, h0_std).
    t_offset/t_total: generate tokens [t_offset, t_offset+T) of a T=t_total sequence.
    Returns a dict with q,k,v,g,beta,A_log,dt_bias,initial_state,scale,lower_bound.
    """
    t_total = T if t_total is None else t_total
    q = torch.empty(B, T, H, D, dtype=torch.bfloat16)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    g = torch.empty(B, T, H, D, dtype=g_dtype)
    beta = torch.empty(B, T, H, dtype=torch.float32)
    A_log = torch.empty(H, dtype=torch.float32)
    dt_bias = torch.empty(H * D, dtype=torch.float32)
    h0 = None if h0_std is None else torch.zeros(B, H, D, D, dtype=torch.float32)
    sl = slice(t_offset, t_offset + T)
    for hh in range(H):
        gen = torch.Generator().manual_seed(seed0 + head_offset + hh)
        r = lambda *s: torch.randn(*s, generator=gen)
        u01 = lambda *s: torch.rand(*s, generator=gen)
        if regime == "baseline":
            a = torch.log(1.0 + 15.0 * u01(1))
            bias = (u01(D) * 0.2 - 0.1)
            sq, sv, sg = 1.0, 1.0, 1.0
        elif regime == "long_memory":
            a = -1.0 + 1.2 * u01(1)
            bias = 0.03 * r(D)
            sq, sv, sg = 0.2, 0.1, 0.1
        elif regime == "carry":
            a = 0.2 * u01(1) - 0.1
            bias = 0.03 * r(D) - 6.0        # gate ~ -0.004 log2 units per token: the state survives
            sq, sv, sg = 1.0, 1.0, 0.3      # thousands of tokens unless the delta rule overwrites it
        else:
            raise ValueError(regime)
        A_log[hh] = a
        dt_bias[hh * D:(hh + 1) * D] = bias
        q[:, :, hh] = (sq * r(B, t_total, D))[:, sl].to(torch.bfloat16)
        k[:, :, hh] = (sq * r(B, t_total, D))[:, sl].to(torch.bfloat16)
        v[:, :, hh] = (sv * r(B, t_total, D))[:, sl].to(torch.bfloat16)
        g[:, :, hh] = (sg * r(B, t_total, D))[:, sl].to(g_dtype)
        beta[:, :, hh] = r(B, t_total)[:, sl]
        if h0 is not None and h0_std > 0:
            h0[:, hh] = h0_std * r(B, D, D)
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias, initial_state=h0,
                scale=D ** -0.5, lower_bound=-5.0 if regime == "baseline" else -1.0)


def run_chunk_reference(inp, **kw):
    return chunk_reference(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=inp["scale"],
                           lower_bound=inp["lower_bound"], A_log=inp["A_log"], dt_bias=inp["dt_bias"],
                           initial_state=inp["initial_state"], **kw)


def run_chunk_reference_varlen(inp, cu_seqlens, **kw):
    """Packed variable-length input ([1, T, H, 128], cu_seqlens = [0, ..., T]): the chunk forward of
    every sequence on its own (chunked from its own first token), outputs re-packed; the initial
    state, if any, is [n_seqs, H, 128, 128].  Returns (o [1, T, H, 128], ht [n_seqs, H, 128, 128])."""
    cu = [int(x) for x in cu_seqlens]
    outs, states = [], []
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        h0 = None if inp["initial_state"] is None else inp["initial_state"][i:i + 1]
        o, ht = chunk_reference(inp["q"][:, a:b], inp["k"][:, a:b], inp["v"][:, a:b], inp["g"][:, a:b],
                                inp["beta"][:, a:b], scale=inp["scale"], lower_bound=inp["lower_bound"],
                                A_log=inp["A_log"], dt_bias=inp["dt_bias"], initial_state=h0, **kw)
        outs.append(o)
        states.append(ht)
    return torch.cat(outs, dim=1), torch.cat(states, dim=0)


def run_recurrent_gold(inp):
    return recurrent_gold(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=inp["scale"],
                          lower_bound=inp["lower_bound"], A_log=inp["A_log"], dt_bias=inp["dt_bias"],
                          initial_state=inp["initial_state"])
