"""The benchmark configurations of the reference at their full sizes.  The CPU oracle cannot walk them whole in
reasonable time, so each is checked through properties that do not depend on size
(determinism, state chaining at a chunk boundary, head shards, the sequence split) plus the
oracle on a slice of heads / tokens that it finishes in seconds.  Inputs follow the benchmark
distributions, generated on the device."""
import pytest
import torch

import kda_ascendc_b200 as K
from kda_ascendc_b200 import shard
from oracle import kda_oracle as O

pytestmark = pytest.mark.gpu
D = 128


def _inputs(dev, B, T, H, seed, h0_std):
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    return dict(q=rn(B, T, H, D).bfloat16(), k=rn(B, T, H, D).bfloat16(), v=rn(B, T, H, D).bfloat16(),
                g=rn(B, T, H, D).bfloat16(), beta=rn(B, T, H),
                A_log=torch.log(1.0 + 15.0 * torch.rand(H, device=dev, generator=g)),
                dt_bias=torch.rand(H * D, device=dev, generator=g) * 0.2 - 0.1,
                initial_state=None if h0_std is None else rn(B, H, D, D) * h0_std,
                scale=D ** -0.5, lower_bound=-5.0)


def _fwd(d, **over):
    x = dict(d, **over)
    return K.kda_bt16_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=x["scale"],
                          initial_state=x["initial_state"], output_final_state=True,
                          use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                          lower_bound=x["lower_bound"], A_log=x["A_log"], dt_bias=x["dt_bias"])


def _oracle_on_heads(d, heads, t_len):
    """Oracle on tokens [0, t_len) of a few heads (every head is independent)."""
    hs = torch.tensor(heads, device=d["q"].device)
    sub = dict(q=d["q"][:, :t_len].index_select(2, hs).cpu(), k=d["k"][:, :t_len].index_select(2, hs).cpu(),
               v=d["v"][:, :t_len].index_select(2, hs).cpu(), g=d["g"][:, :t_len].index_select(2, hs).cpu(),
               beta=d["beta"][:, :t_len].index_select(2, hs).cpu(), A_log=d["A_log"][hs].cpu(),
               dt_bias=d["dt_bias"].view(-1, D)[hs].reshape(-1).cpu(),
               initial_state=None if d["initial_state"] is None else d["initial_state"].index_select(1, hs).cpu(),
               scale=d["scale"], lower_bound=d["lower_bound"])
    return O.run_chunk_reference(sub)


def _check_properties(d, heads, t_oracle):
    B, T, H, _ = d["q"].shape
    o, ht = _fwd(d)
    assert torch.isfinite(o.float()).all() and torch.isfinite(ht).all()
    o2, ht2 = _fwd(d)
    assert torch.equal(o, o2) and torch.equal(ht, ht2)                      # deterministic
    cut = (T // 2 // 16) * 16                                               # chaining at a chunk boundary
    first = {n: d[n][:, :cut].contiguous() for n in ("q", "k", "v", "g", "beta")}
    second = {n: d[n][:, cut:].contiguous() for n in ("q", "k", "v", "g", "beta")}
    o_a, h_a = _fwd(d, **first)
    o_b, h_b = _fwd(d, **second, initial_state=h_a)
    assert torch.equal(torch.cat([o_a, o_b], 1), o) and torch.equal(h_b, ht)
    for r in (0, 3):                                                        # two of four head shards
        o_s, h_s, (lo, hi) = shard.forward_head_shard(d["q"], d["k"], d["v"], d["g"], d["beta"], rank=r, world=4,
                                                      scale=d["scale"], initial_state=d["initial_state"],
                                                      output_final_state=True, lower_bound=d["lower_bound"],
                                                      A_log=d["A_log"], dt_bias=d["dt_bias"])
        # bit-equal when the shard runs the same K2 organisation as the whole problem (it is chosen
        # from the number of heads); otherwise only the fp32 summation order of one product differs
        if not (torch.equal(o_s, o[:, :, lo:hi]) and torch.equal(h_s, ht[:, lo:hi])):
            assert (o_s.float() - o[:, :, lo:hi].float()).abs().max().item() <= 5e-3 * o.float().abs().max().item()
            assert (h_s - ht[:, lo:hi]).abs().max().item() <= 1e-4
    o_r, h_r = _oracle_on_heads(d, heads, t_oracle)                         # oracle on a slice
    hs = torch.tensor(heads, device=o.device)
    assert (o[:, :t_oracle].index_select(2, hs).float().cpu() - o_r.float()).abs().max().item() <= 1e-3
    if t_oracle == T:
        assert (ht.index_select(1, hs).cpu() - h_r).abs().max().item() <= 2e-3
    return o, ht


def test_config1_b2_t4096_h8_whole_oracle(cuda_device):
    d = _inputs(cuda_device, 2, 4096, 8, seed=101, h0_std=0.02)
    _check_properties(d, list(range(8)), 4096)                              # the oracle walks all of it


def test_config2_b1_t8192_h32(cuda_device):
    d = _inputs(cuda_device, 1, 8192, 32, seed=102, h0_std=0.02)
    _check_properties(d, [0, 17, 31], 8192)


def test_config3_b1_t8192_h96(cuda_device):
    d = _inputs(cuda_device, 1, 8192, 96, seed=103, h0_std=0.02)
    _check_properties(d, [5, 95], 8192)


def test_config4_b1_t131072_h16_sequence_split(cuda_device):
    d = _inputs(cuda_device, 1, 131072, 16, seed=104, h0_std=0.02)
    o, ht = _check_properties(d, [0, 15], 4096)
    o8, h8 = shard.forward_seq_split_local(d["q"], d["k"], d["v"], d["g"], d["beta"], 8, scale=d["scale"],
                                           initial_state=d["initial_state"], lower_bound=d["lower_bound"],
                                           A_log=d["A_log"], dt_bias=d["dt_bias"])
    # the split against the one-pass kernels: on this distribution the absolute bounds of the
    # one-pass path hold for the split as well
    assert (o8.float() - o.float()).abs().max().item() <= 1e-3
    assert (h8 - ht).abs().max().item() <= 2e-3
    # ... and against the ORACLE on two heads across the first segment boundary (token 16384)
    heads, t_or = [0, 15], 16384 + 1024
    o_r, _ = _oracle_on_heads(d, heads, t_or)
    hs = torch.tensor(heads, device=o8.device)
    assert (o8[:, :t_or].index_select(2, hs).float().cpu() - o_r.float()).abs().max().item() <= 1e-3


def test_many_chains_b8_t2048_h32_tensor_memory_k2(cuda_device):
    """256 (batch, head) chains: more chains than SMs, so K2 runs in its tcgen05 form (two CTAs per
    SM).  Same size-independent properties; the oracle walks four heads of one batch entry."""
    d = _inputs(cuda_device, 8, 2048, 32, seed=105, h0_std=0.02)
    o, ht = _check_properties(d, [0, 9, 22, 31], 512)
    # the 16-row mma.sync organisation on the same records agrees to rounding
    from kda_ascendc_b200 import api
    o_m, ht_m = api._forward(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["initial_state"], True, True, True,
                             True, d["lower_bound"], d["A_log"], d["dt_bias"], True, k2_variant=3)
    assert (o.float() - o_m.float()).abs().max().item() <= 5e-3 * o.float().abs().max().item()
    assert (ht - ht_m).abs().max().item() <= 1e-4
