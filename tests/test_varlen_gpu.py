"""Packed variable-length sequences (cu_seqlens) against the oracle run per sequence and against
this build's own fixed-length calls (a chunk's valid rows never read the rows past its sequence's
end: within one bf16 step of o and 2e-5 on the state, since the packed batch may run another K2
organisation; bit-equal for a single packed sequence).  Tolerances as for the fixed-length path: o 1e-3, state 2e-3 (benchmark
distribution)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kda_oracle as O  # noqa: E402

FLAGS = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
             output_final_state=True)


def _setup(lengths, H, seed, h0_std):
    T = sum(lengths)
    inp = O.make_inputs(1, T, H, seed0=seed, h0_std=None)
    n = len(lengths)
    if h0_std is not None:
        g = torch.Generator().manual_seed(seed + 99)
        inp["initial_state"] = torch.randn(n, H, 128, 128, generator=g) * h0_std
    cu = [0]
    for L in lengths:
        cu.append(cu[-1] + L)
    dev = torch.device("cuda", 0)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    kw = dict(scale=d["scale"], lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])
    return inp, d, cu, kw


@pytest.mark.parametrize("lengths,H,h0_std", [([1, 15, 16, 17, 100, 33], 3, 0.02), ([40] * 20 + [7], 2, None),
                                              ([256, 1000, 16], 4, 0.05)])
def test_varlen_matches_oracle_and_fixed_length_calls(lengths, H, h0_std):
    import kda_ascendc_b200 as K
    inp, d, cu, kw = _setup(lengths, H, 21, h0_std)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=d["q"].device)
    o, ht = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                           cu_seqlens=cu_t, **FLAGS, **kw)
    torch.cuda.synchronize()
    assert tuple(ht.shape) == (len(lengths), H, 128, 128)
    o_r, ht_r = O.run_chunk_reference_varlen(inp, cu)
    assert (o.float().cpu() - o_r.float()).abs().max().item() <= 1e-3
    assert (ht.cpu() - ht_r).abs().max().item() <= 2e-3
    # the same sequences one by one through the fixed-length path
    for i in range(len(lengths)):
        a, b = cu[i], cu[i + 1]
        h0 = None if d["initial_state"] is None else d["initial_state"][i:i + 1]
        o_i, ht_i = K.kda_bt16_fwd(*(d[n][:, a:b].contiguous() for n in ("q", "k", "v", "g", "beta")),
                                   initial_state=h0, **FLAGS, **kw)
        assert (o[:, a:b].float() - o_i.float()).abs().max().item() <= 2.5e-4, i   # one bf16 step of |o| <= 0.06
        assert (ht[i:i + 1] - ht_i).abs().max().item() <= 2e-5, i


def test_varlen_single_sequence_equals_fixed_length():
    import kda_ascendc_b200 as K
    inp, d, cu, kw = _setup([333], 4, 4, 0.1)
    o1, h1 = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **FLAGS, **kw)
    o2, h2 = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                            cu_seqlens=[0, 333], **FLAGS, **kw)
    assert torch.equal(o1, o2) and torch.equal(h1, h2)


def test_varlen_argument_errors():
    import kda_ascendc_b200 as K
    inp, d, cu, kw = _setup([20, 30], 2, 1, None)
    call = lambda c, **extra: K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], cu_seqlens=c, **FLAGS, **kw, **extra)
    with pytest.raises(ValueError):
        call([0, 20, 49])            # does not end at T
    with pytest.raises(ValueError):
        call([0, 20, 20, 50])        # empty sequence
    with pytest.raises(ValueError):
        call([0, 50], initial_state=torch.zeros(2, 2, 128, 128, device=d["q"].device))   # one state per sequence
    q2 = torch.cat([d["q"], d["q"]])
    with pytest.raises(ValueError):
        K.kda_bt16_fwd(q2, q2, q2, torch.cat([d["g"], d["g"]]), torch.cat([d["beta"], d["beta"]]), cu_seqlens=[0, 50],
                       **FLAGS, **kw)
