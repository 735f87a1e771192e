"""Grouped value heads (HV a multiple of H): value head h reads q/k head h // (HV // H).  Checked
against the same kernels fed with q, k repeated per group (bit-identical) and against the oracle
on those expanded inputs (o 1e-3, state 2e-3)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kda_oracle as O  # noqa: E402

FLAGS = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
             output_final_state=True)


@pytest.mark.parametrize("B,T,H,G", [(2, 100, 2, 3), (1, 64, 1, 4)])
def test_grouped_value_heads(B, T, H, G):
    import kda_ascendc_b200 as K
    HV = H * G
    inp = O.make_inputs(B, T, HV, seed0=13, h0_std=0.05)
    # q, k of the grouped problem: the first head of every group
    inp_q = inp["q"][:, :, ::G].contiguous()
    inp_k = inp["k"][:, :, ::G].contiguous()
    full = dict(inp, q=inp_q.repeat_interleave(G, dim=2), k=inp_k.repeat_interleave(G, dim=2))
    dev = torch.device("cuda", 0)
    d = {k_: (v_.to(dev) if torch.is_tensor(v_) else v_) for k_, v_ in full.items()}
    kw = dict(scale=d["scale"], lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])
    qg, kg = inp_q.to(dev), inp_k.to(dev)
    o_g, h_g = K.kda_bt16_fwd(qg, kg, d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **FLAGS, **kw)
    o_f, h_f = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **FLAGS, **kw)
    assert tuple(o_g.shape) == (B, T, HV, 128) and tuple(h_g.shape) == (B, HV, 128, 128)
    assert torch.equal(o_g, o_f) and torch.equal(h_g, h_f)
    o_r, h_r = O.run_chunk_reference(full)
    assert (o_g.float().cpu() - o_r.float()).abs().max().item() <= 1e-3
    assert (h_g.cpu() - h_r).abs().max().item() <= 2e-3
    # the recurrent step
    o_rg, s_rg = K.kda_recurrent_fwd(qg[:, :6], kg[:, :6], d["v"][:, :6], d["g"][:, :6], d["beta"][:, :6],
                                     initial_state=d["initial_state"], **kw)
    o_rf, s_rf = K.kda_recurrent_fwd(d["q"][:, :6], d["k"][:, :6], d["v"][:, :6], d["g"][:, :6], d["beta"][:, :6],
                                     initial_state=d["initial_state"], **kw)
    assert torch.equal(o_rg, o_rf) and torch.equal(s_rg, s_rf)


def test_head_counts_that_do_not_divide_are_rejected():
    import kda_ascendc_b200 as K
    dev = torch.device("cuda", 0)
    q = torch.randn(1, 16, 2, 128, device=dev).bfloat16()
    v = torch.randn(1, 16, 3, 128, device=dev).bfloat16()
    with pytest.raises(ValueError, match="multiple of H"):
        K.kda_bt16_fwd(q, q, v, v.float(), torch.randn(1, 16, 3, device=dev), A_log=torch.zeros(3, device=dev), **FLAGS)
