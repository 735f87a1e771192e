"""CPU checks of the oracle itself: it must reproduce what the reference produced."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import kda_oracle as O


@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("loop_heads", [False, True])
def test_oracle_reproduces_reference_golden(name, loop_heads):
    c = load_golden(name)
    o, ht = O.chunk_reference(c["q"], c["k"], c["v"], c["g"], c["beta"], scale=c["scale"],
                              lower_bound=c["lower_bound"], A_log=c["A_log"], dt_bias=c["dt_bias"],
                              initial_state=c["initial_state"], state_v_first=c["state_v_first"],
                              loop_heads=loop_heads)
    assert o.dtype == torch.bfloat16 and ht.dtype == torch.float32
    # same algorithm, same precision: identical up to fp32 summation order inside matmul
    assert (o.float() - c["o"].float()).abs().max().item() <= 2.0 ** -9 * c["o"].float().abs().max().item()
    assert (o != c["o"]).float().mean().item() < 1e-3          # essentially every bf16 output bit-equal
    assert (ht - c["ht"]).abs().max().item() <= 1e-6


def test_batched_and_looped_oracle_agree():
    inp = O.make_inputs(2, 80, 3, seed0=5, h0_std=0.02)
    o1, h1 = O.run_chunk_reference(inp, loop_heads=True)
    o2, h2 = O.run_chunk_reference(inp, loop_heads=False)
    assert (o1.float() - o2.float()).abs().max().item() <= 2.5e-4
    assert (h1 - h2).abs().max().item() <= 1e-6


@pytest.mark.parametrize("regime,h0", [("baseline", 0.02), ("long_memory", 0.5)])
def test_chunk_oracle_agrees_with_recurrent_gold(regime, h0):
    """The chunked form and the float64 token recurrence are the same function; what is
    left is the bf16 rounding of the normalised q/k inside the chunk oracle."""
    inp = O.make_inputs(1, 80, 2, seed0=11, regime=regime, h0_std=h0)
    o, ht = O.run_chunk_reference(inp)
    og, hg = O.run_recurrent_gold(inp)
    assert (o.double() - og).abs().max().item() < 2e-3 * max(1.0, og.abs().max().item() / 0.1)
    assert (ht.double() - hg).abs().max().item() < 5e-3 * max(1.0, hg.abs().max().item())
    # a transposed state, a wrong decay axis or a dropped term would be O(signal)
    assert (o.double() - og).abs().max().item() < 0.05 * og.abs().max().item()
    assert (ht.double() - hg).abs().max().item() < 0.05 * hg.abs().max().item()


def test_segment_chaining_is_exact_in_the_oracle():
    """final_state -> initial_state chaining at a chunk boundary reproduces the long run."""
    inp = O.make_inputs(1, 96, 2, seed0=3, regime="long_memory", h0_std=0.1)
    o, ht = O.run_chunk_reference(inp)
    cut = 48
    a = {k: (v[:, :cut] if torch.is_tensor(v) and v.ndim >= 3 and v.shape[1] == 96 else v) for k, v in inp.items()}
    b = {k: (v[:, cut:] if torch.is_tensor(v) and v.ndim >= 3 and v.shape[1] == 96 else v) for k, v in inp.items()}
    o1, h1 = O.run_chunk_reference(a)
    b["initial_state"] = h1
    o2, h2 = O.run_chunk_reference(b)
    assert torch.equal(torch.cat([o1, o2], 1), o)
    assert torch.equal(h2, ht)


def test_make_inputs_is_shard_invariant():
    full = O.make_inputs(1, 64, 4, seed0=42, h0_std=0.02)
    part = O.make_inputs(1, 64, 2, seed0=42, h0_std=0.02, head_offset=2)
    for key in ("q", "k", "v", "g", "beta", "initial_state"):
        ax = 2 if key != "initial_state" else 1
        assert torch.equal(full[key].narrow(ax, 2, 2), part[key]), key
    assert torch.equal(full["A_log"][2:], part["A_log"])
    seg = O.make_inputs(1, 32, 4, seed0=42, t_offset=32, t_total=64)
    assert torch.equal(full["q"][:, 32:], seg["q"]) and torch.equal(full["beta"][:, 32:], seg["beta"])
