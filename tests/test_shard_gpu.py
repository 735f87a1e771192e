"""GPU checks of the multi-GPU drivers on one device: head shards and the sequence split
(segments standing in for ranks) against the one-pass forward and the CPU oracle."""
import pytest
import torch

import kda_ascendc_b200 as K
from conftest import to_device
from kda_ascendc_b200 import shard
from oracle import kda_oracle as O

pytestmark = pytest.mark.gpu


def _one_pass(d):
    return K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"],
                          initial_state=d["initial_state"], output_final_state=True,
                          use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                          lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])


def test_head_shards_reassemble_the_full_result(cuda_device):
    inp = O.make_inputs(2, 96, 6, seed0=31, h0_std=0.02)
    d = to_device(inp, cuda_device)
    o_full, h_full = _one_pass(d)
    world = 4
    for r in range(world):
        o, ht, (lo, hi) = shard.forward_head_shard(d["q"], d["k"], d["v"], d["g"], d["beta"], rank=r, world=world,
                                                   scale=d["scale"], initial_state=d["initial_state"],
                                                   output_final_state=True, lower_bound=d["lower_bound"],
                                                   A_log=d["A_log"], dt_bias=d["dt_bias"])
        assert torch.equal(o, o_full[:, :, lo:hi]) and torch.equal(ht, h_full[:, lo:hi])


@pytest.mark.parametrize("regime,T,nseg", [("carry", 512, 4), ("carry", 2048, 8), ("baseline", 1024, 8),
                                           ("long_memory", 256, 2)])
def test_sequence_split_matches_one_pass_and_oracle(cuda_device, regime, T, nseg):
    """K1 once per segment, two state-only passes, fold, K2: same outputs as the one-pass
    forward up to the bf16 rounding of the state inside the transition pass."""
    inp = O.make_inputs(1, T, 2, seed0=13, regime=regime, h0_std=0.1)
    d = to_device(inp, cuda_device)
    o1, h1 = _one_pass(d)
    o2, h2 = shard.forward_seq_split_local(d["q"], d["k"], d["v"], d["g"], d["beta"], nseg, scale=d["scale"],
                                           initial_state=d["initial_state"], lower_bound=d["lower_bound"],
                                           A_log=d["A_log"], dt_bias=d["dt_bias"])
    o_r, h_r = O.run_chunk_reference(inp)
    omax, hmax = o_r.float().abs().max().item(), h_r.abs().max().item()
    # against the oracle: the reference's relative bound, 2e-2 of absmax
    assert (o2.float().cpu() - o_r.float()).abs().max().item() < 2e-2 * omax
    assert (h2.cpu() - h_r).abs().max().item() < 2e-2 * hmax
    # against the one-pass kernels: only the segment hand-over differs
    assert (o2.float() - o1.float()).abs().max().item() < 1e-2 * omax
    assert (h2 - h1).abs().max().item() < 1e-2 * hmax
    if regime == "carry":
        # the hand-over matters in this regime: dropping it is visibly wrong
        o_bad = torch.cat([_one_pass(dict(d, initial_state=None if j else d["initial_state"],
                                          **{n: d[n][:, j * (T // nseg):(j + 1) * (T // nseg)].contiguous()
                                             for n in ("q", "k", "v", "g", "beta")}))[0] for j in range(nseg)], 1)
        assert (o_bad.float() - o1.float()).abs().max().item() > 0.1 * omax
