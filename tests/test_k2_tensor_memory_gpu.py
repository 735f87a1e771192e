"""The tensor-memory (tcgen05) organisation of K2 against the oracle and against the mma.sync
organisations.  Same tolerances as the default path: o 1e-3, state 2e-3 on benchmark-distributed
inputs; the reference's relative 2e-2 bound where states are O(1)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kda_oracle as O  # noqa: E402


def _run(inp, variant, cu=None):
    from kda_ascendc_b200 import api
    dev = torch.device("cuda", 0)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    o, ht = api._forward(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["initial_state"], True, True, True, True,
                         d["lower_bound"], d["A_log"], d["dt_bias"], True, k2_variant=variant, cu_seqlens=cu)
    torch.cuda.synchronize()
    return o.float().cpu(), ht.cpu()


@pytest.mark.parametrize("B,T,H,h0_std", [(1, 16, 1, None), (2, 1000, 4, 0.02), (1, 333, 3, 0.0), (5, 64, 40, 0.02)])
def test_tensor_memory_k2_matches_oracle(B, T, H, h0_std):
    inp = O.make_inputs(B, T, H, seed0=17, h0_std=h0_std)
    o, ht = _run(inp, 4)
    o_r, ht_r = O.run_chunk_reference(inp)
    assert (o - o_r.float()).abs().max().item() <= 1e-3
    assert (ht - ht_r).abs().max().item() <= 2e-3
    o1, ht1 = _run(inp, 1)
    assert (o - o1).abs().max().item() <= 2.5e-4       # one bf16 step of |o| <= 0.06
    assert (ht - ht1).abs().max().item() <= 2e-5


@pytest.mark.parametrize("regime,h0_std", [("carry", 0.5), ("long_memory", 0.3)])
def test_tensor_memory_k2_carries_the_state(regime, h0_std):
    inp = O.make_inputs(2, 512, 3, seed0=23, regime=regime, h0_std=h0_std)
    o, ht = _run(inp, 4)
    o_r, ht_r = O.run_chunk_reference(inp)
    assert (o - o_r.float()).abs().max().item() <= 2e-2 * o_r.float().abs().max().item()
    assert (ht - ht_r).abs().max().item() <= 2e-2 * ht_r.abs().max().item()
    o1, ht1 = _run(inp, 3)
    assert (ht - ht1).abs().max().item() <= 1e-3 * ht_r.abs().max().item()


def test_tensor_memory_k2_packed_sequences():
    lengths = [40, 1, 17, 160, 31]
    T = sum(lengths)
    inp = O.make_inputs(1, T, 3, seed0=29, h0_std=None)
    g = torch.Generator().manual_seed(5)
    inp["initial_state"] = torch.randn(len(lengths), 3, 128, 128, generator=g) * 0.05
    cu = [0]
    for L in lengths:
        cu.append(cu[-1] + L)
    o, ht = _run(inp, 4, cu=cu)
    o_r, ht_r = O.run_chunk_reference_varlen(inp, cu)
    assert (o - o_r.float()).abs().max().item() <= 1e-3
    assert (ht - ht_r).abs().max().item() <= 2e-3


def test_tail_wave_runs_in_an_mma_sync_form():
    """320 chains on 148 SMs: 296 fill one wave of the tensor-memory form, the other 24 follow in
    the 8-row mma.sync form (a second K2 launch on the chains' sub-range).  Both halves against the oracle."""
    from kda_ascendc_b200 import _lib
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    B, T, H = 10, 72, 32
    inp = O.make_inputs(B, T, H, seed0=31, h0_std=0.02)
    o, ht = _run(inp, 0)
    launches = _lib.load().kda_last_launch_count()
    tail = (B * H) % (2 * sms)
    if B * H > 2 * sms and 0 < tail * 2 <= sms:
        assert launches == 3     # K1, K2 on tcgen05 for the full waves, K2 on mma.sync for the tail
    o_r, ht_r = O.run_chunk_reference(inp)
    assert (o - o_r.float()).abs().max().item() <= 1e-3
    assert (ht - ht_r).abs().max().item() <= 2e-3
    o3, ht3 = _run(inp, 3)
    assert (o - o3).abs().max().item() <= 2.5e-4
    assert (ht - ht3).abs().max().item() <= 2e-5
    # the tail chains are the last ones: bit-identical to the form that ran them (8-row up to SMs/4 chains)
    first_tail = B * H - tail
    if B * H > 2 * sms and 0 < tail * 2 <= sms:
        ref = _run(inp, 1)[1] if tail * 4 <= sms else ht3
        assert torch.equal(ht.reshape(B * H, 128, 128)[first_tail:], ref.reshape(B * H, 128, 128)[first_tail:])


def test_tail_wave_with_packed_sequences():
    """20 packed sequences x 16 heads = 320 chains: the automatic choice (tensor memory + tail in the
    16-row form) against the 16-row form alone."""
    lengths = [64 + 7 * i for i in range(20)]
    T, H = sum(lengths), 16
    inp = O.make_inputs(1, T, H, seed0=37, h0_std=None)
    g = torch.Generator().manual_seed(7)
    inp["initial_state"] = torch.randn(len(lengths), H, 128, 128, generator=g) * 0.05
    cu = [0]
    for L in lengths:
        cu.append(cu[-1] + L)
    o, ht = _run(inp, 0, cu=cu)
    o3, ht3 = _run(inp, 3, cu=cu)
    assert (o - o3).abs().max().item() <= 2.5e-4
    assert (ht - ht3).abs().max().item() <= 2e-5
    o_r, ht_r = O.run_chunk_reference_varlen(inp, cu)
    assert (o - o_r.float()).abs().max().item() <= 1e-3
    assert (ht - ht_r).abs().max().item() <= 2e-3
