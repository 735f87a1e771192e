"""Stability gate at production sizes: many consecutive forwards on the same buffers must be
bit-identical (the reference's gate: 30 calls at [1, 8192, 96], tests/test_stability_gate.py:80-101
of the reference).  A persistent kernel that reuses shared-memory stages across iterations shows a
missing release/acquire as run-to-run drift long before it shows as a wrong answer, so the repeat
count matters more than the tolerance; every K2 organisation is covered (8-row at H = 32,
tensor-memory at H = 96, tensor-memory plus a tail wave in an mma.sync form at 320 chains)."""
import ctypes

import pytest
import torch

import kda_ascendc_b200 as K
from kda_ascendc_b200 import _lib, api

pytestmark = pytest.mark.gpu
D = 128
REPEATS = 30


def _inputs(dev, B, T, H, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    return dict(q=rn(B, T, H, D).bfloat16(), k=rn(B, T, H, D).bfloat16(), v=rn(B, T, H, D).bfloat16(),
                g=rn(B, T, H, D).bfloat16(), beta=rn(B, T, H),
                A_log=torch.log(1.0 + 15.0 * torch.rand(H, device=dev, generator=g)),
                dt_bias=torch.rand(H * D, device=dev, generator=g) * 0.2 - 0.1, h0=rn(B, H, D, D) * 0.02)


@pytest.mark.parametrize("B,T,H,form", [(1, 8192, 32, "n8"), (1, 8192, 96, "tc"), (10, 1024, 32, "tc")])
def test_thirty_consecutive_forwards_are_bit_identical(cuda_device, B, T, H, form):
    assert api.k2_choice(B, T, H)[0] == form
    d = _inputs(cuda_device, B, T, H, seed=300 + H + B)
    lib = _lib.load()
    ws = torch.empty(K.workspace_bytes(B, T, H), dtype=torch.uint8, device=cuda_device)
    o = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=cuda_device)
    ht = torch.empty(B, H, D, D, dtype=torch.float32, device=cuda_device)
    args = api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=D ** -0.5, lower_bound=-5.0,
                         A_log=d["A_log"], dt_bias=d["dt_bias"], h0=d["h0"], o=o, ht=ht, workspace=ws, flags=7)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    first = None
    for i in range(REPEATS):
        if i % 7 == 3:      # stale outputs and records must never survive a call
            o.fill_(float("nan"))
            ht.fill_(float("nan"))
            ws[256:].fill_(0xFF)
        assert lib.kda_fwd(ctypes.byref(args), stream) == 0, _lib.last_error()
        if first is None:
            first = (o.clone(), ht.clone())
            assert torch.isfinite(first[0].float()).all() and torch.isfinite(first[1]).all()
        else:
            assert torch.equal(o, first[0]) and torch.equal(ht, first[1]), "call %d differs from call 0" % i
    assert api.check_device_status(ws) == 0
