"""The look-ahead form of K2 (k2_variant 5) against the CPU oracle and the float64 recurrence.

That form takes the products of chunk n+1 from the decayed state of step n plus a 16x16 cross-Gram
correction, so its rounding differs from the plain forms: it is held to the same bounds as they are
(1e-3 / 2e-3 on the benchmark distribution, "no worse than the oracle against the gold", the
reference's relative bound where states are O(1)), on the regimes in which a wrong hand-over of the
state or of the cross term cannot hide: almost no decay ("carry"), long memory, a saturated gate
(lower_bound -8 / -10), odd chunk counts and a partial last chunk.  It is never chosen
automatically; these tests select it explicitly.
"""
import ctypes

import pytest
import torch

import kda_ascendc_b200 as K
from conftest import golden_cases, load_golden, to_device
from kda_ascendc_b200 import _lib, api
from oracle import kda_oracle as O

pytestmark = pytest.mark.gpu
LA = 5


def _fwd(d, variant=LA, vsplit=0, v_first=True):
    return api._forward(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["initial_state"], True,
                        True, True, True, d["lower_bound"], d["A_log"], d["dt_bias"], v_first,
                        k2_vsplit=vsplit, k2_variant=variant)


def _bf16_ulp(x: float) -> float:
    import math
    return 2.0 ** (math.floor(math.log2(max(x, 1e-30))) - 7)


@pytest.mark.parametrize("name", golden_cases())
def test_lookahead_matches_reference_golden(cuda_device, name):
    c = load_golden(name)           # includes the saturated-gate cases (lower_bound -8, -10) and both state layouts
    d = to_device(c, cuda_device)
    o, ht = _fwd(d, v_first=c["state_v_first"])
    assert torch.isfinite(o.float()).all() and torch.isfinite(ht).all()
    assert (o.float().cpu() - c["o"].float()).abs().max().item() <= 1e-3
    assert (ht.cpu() - c["ht"]).abs().max().item() <= 2e-3


@pytest.mark.parametrize("B,T,H,h0", [(1, 5, 1, None), (1, 16, 1, None), (1, 17, 1, 0.02), (1, 33, 2, 0.02),
                                      (1, 48, 3, 0.02), (2, 1037, 4, 0.02), (2, 1024, 4, 0.0)])
def test_lookahead_parity_with_oracle_and_gold(cuda_device, B, T, H, h0):
    inp = O.make_inputs(B, T, H, seed0=42, h0_std=h0)
    o_r, h_r = O.run_chunk_reference(inp)
    o_g, h_g = O.run_recurrent_gold(inp)
    o, ht = _fwd(to_device(inp, cuda_device))
    o, ht = o.cpu(), ht.cpu()
    assert (o.float() - o_r.float()).abs().max().item() <= 1e-3
    assert (ht - h_r).abs().max().item() <= 2e-3
    eo_new, eo_ref = (o.double() - o_g).abs(), (o_r.double() - o_g).abs()
    eh_new, eh_ref = (ht.double() - h_g).abs(), (h_r.double() - h_g).abs()
    assert eo_new.max().item() <= eo_ref.max().item() + _bf16_ulp(o_r.float().abs().max().item())
    assert eo_new.pow(2).mean().sqrt().item() <= 1.05 * eo_ref.pow(2).mean().sqrt().item() + 1e-9
    assert eh_new.max().item() <= 1.05 * eh_ref.max().item() + 1e-6
    assert eh_new.pow(2).mean().sqrt().item() <= 1.02 * eh_ref.pow(2).mean().sqrt().item() + 1e-9


@pytest.mark.parametrize("regime,B,T,H,h0", [("carry", 1, 512, 2, 0.5), ("carry", 1, 33, 2, 0.5),
                                             ("carry", 2, 1000, 3, 0.1), ("long_memory", 1, 48, 3, 0.1),
                                             ("long_memory", 2, 512, 2, 0.01)])
def test_lookahead_where_the_state_persists(cuda_device, regime, B, T, H, h0):
    inp = O.make_inputs(B, T, H, seed0=7, regime=regime, h0_std=h0)
    o_r, h_r = O.run_chunk_reference(inp)
    d = to_device(inp, cuda_device)
    o, ht = _fwd(d)
    omax, hmax = o_r.float().abs().max().item(), h_r.abs().max().item()
    assert (o.float().cpu() - o_r.float()).abs().max().item() < 2e-2 * omax
    assert (ht.cpu() - h_r).abs().max().item() < 2e-2 * hmax
    # and close to the plain 8-row form on the same records (only the look-ahead's rounding differs)
    o1, h1 = _fwd(d, variant=1)
    assert (o.float() - o1.float()).abs().max().item() < 1e-2 * omax
    assert (ht - h1).abs().max().item() < 5e-3 * hmax


def test_lookahead_slicings_agree_and_state_only_pass(cuda_device):
    """How the rows are spread over warps and CTAs must not change a bit; the state-only pass
    returns the state of the full pass."""
    inp = O.make_inputs(1, 208, 3, seed0=6, regime="carry", h0_std=0.5)       # 13 chunks: an odd count
    d = to_device(inp, cuda_device)
    outs = [_fwd(d, vsplit=vs) for vs in (4, 8, 16)]
    for o, ht in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(ht, outs[0][1])
    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(K.workspace_bytes(1, 208, 3), dtype=torch.uint8, device=cuda_device)
    o = torch.empty(1, 208, 3, 128, dtype=torch.bfloat16, device=cuda_device)
    ht = torch.empty(1, 3, 128, 128, device=cuda_device)
    a = api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"], lower_bound=d["lower_bound"],
                      A_log=d["A_log"], dt_bias=d["dt_bias"], h0=d["initial_state"], o=o, ht=ht, workspace=ws,
                      flags=7, k2_variant=LA)
    assert lib.kda_fwd_k1(ctypes.byref(a), st) == 0, _lib.last_error()
    assert lib.kda_fwd_k2_state(ctypes.byref(a), 0, st) == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.equal(ht, outs[0][1])
    assert api.check_device_status(ws) == 0
