"""Chunk-major layouts.

``pack_tokens`` / ``unpack_tokens`` keep the helper names and meaning of the reference
(``python/kda_ascendc_v1/layout.py:17-32``): the leading index of a packed tensor is
``c = (b * H + h) * NT + chunk``.  ``unpack_records`` decodes the K1 -> K2 workspace of
this build (record layout: ``csrc/kda_common.cuh``) back into plain tensors in the
public ``[B, T, H, *]`` layout for stage-wise checks.
"""
from __future__ import annotations

import torch

CHUNK = 16
D = 128
REC_BYTES = 26112
WS_HEADER_BYTES = 256
REC_W, REC_QG, REC_KGH, REC_KGL, REC_AQK, REC_AQL, REC_DEC, REC_U = 0, 4096, 8192, 12288, 16384, 16896, 17408, 17920


def pack_tokens(x: torch.Tensor, chunk: int = CHUNK) -> torch.Tensor:
    """``[B, T, H, D]`` -> ``[B*H*(T//chunk), chunk, D]`` (contiguous)."""
    if x.dim() != 4:
        raise ValueError("pack_tokens expects a 4-D [B, T, H, D] tensor")
    b, t, h, d = x.shape
    if t % chunk:
        raise ValueError(f"T={t} is not a multiple of chunk={chunk}")
    return x.view(b, t // chunk, chunk, h, d).permute(0, 3, 1, 2, 4).reshape(-1, chunk, d).contiguous()


def unpack_tokens(x: torch.Tensor, b: int, t: int, h: int, chunk: int = CHUNK) -> torch.Tensor:
    """Inverse of :func:`pack_tokens`."""
    d = x.shape[-1]
    return x.view(b, h, t // chunk, chunk, d).permute(0, 2, 3, 1, 4).reshape(b, t, h, d).contiguous()


def _swizzle_index(device) -> torch.Tensor:
    """Position (in bf16 elements) of element (r, c) inside a swizzled [16][128] tile."""
    r = torch.arange(CHUNK, device=device)[:, None]
    c = torch.arange(D, device=device)[None, :]
    return (r * D + ((((c >> 3) ^ (r & 7)) << 3) | (c & 7))).reshape(-1)


def _u_index(device) -> torch.Tensor:
    """Position (in fp32 elements) of u[tok][v] inside the fragment-ordered u block."""
    tok = torch.arange(CHUNK, device=device)[:, None]
    v = torch.arange(D, device=device)[None, :]
    tile, vr = v // 8, v % 8
    lane = (tok % 8) * 4 + vr // 2
    e = (tok // 8) * 2 + vr % 2
    return ((tile * 32 + lane) * 4 + e).reshape(-1)


def unpack_records(workspace: torch.Tensor, B: int, T: int, H: int) -> dict:
    """Decode the chunk records of a finished K1 pass.

    Returns ``w, qg`` (bf16), ``kg, u`` (fp32; kg = hi + lo), ``Aqk`` (fp32 = hi + lo, ``[B,T,H,16]``)
    in the public token layout (rows past ``T`` dropped) and ``dec`` fp32 ``[B,H,NT,128]``.
    """
    nt = (T + CHUNK - 1) // CHUNK
    c = B * H * nt
    rec = workspace[WS_HEADER_BYTES:WS_HEADER_BYTES + c * REC_BYTES].view(c, REC_BYTES)
    dev = workspace.device
    sw = _swizzle_index(dev)

    def tile(off):
        t = rec[:, off:off + 4096].contiguous().view(torch.bfloat16)  # [c, 2048]
        return t[:, sw].view(c, CHUNK, D)

    def to_public(x):  # [c, 16, n] -> [B, T, H, n]
        n = x.shape[-1]
        y = x.view(B, H, nt, CHUNK, n).permute(0, 2, 3, 1, 4).reshape(B, nt * CHUNK, H, n)
        return y[:, :T].contiguous()

    uT = rec[:, REC_U:REC_U + 8192].contiguous().view(torch.float32)[:, _u_index(dev)].view(c, CHUNK, D)
    aqk = (rec[:, REC_AQK:REC_AQK + 512].contiguous().view(torch.bfloat16).float() +
           rec[:, REC_AQL:REC_AQL + 512].contiguous().view(torch.bfloat16).float()).view(c, CHUNK, CHUNK)
    dec = rec[:, REC_DEC:REC_DEC + 512].contiguous().view(torch.float32).view(B, H, nt, D)
    return dict(w=to_public(tile(REC_W)), qg=to_public(tile(REC_QG)),
                kg=to_public(tile(REC_KGH).float() + tile(REC_KGL).float()),
                u=to_public(uT), Aqk=to_public(aqk), dec=dec)
