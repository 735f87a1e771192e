"""Token recurrence (decode / short sequences) against the oracle and against the chunk kernels.

Tolerances: outputs of benchmark-distributed inputs are O(0.06), bf16 output -> 1e-3 max-abs as
for the chunk path; states 2e-3.  The float64 token recurrence of the oracle is the gold; the
chunk forward of this build is the consistency partner (a prefill followed by decode steps must
continue the sequence the chunk forward would have produced in one go).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kda_oracle as O  # noqa: E402


def _dev(inp):
    dev = torch.device("cuda", 0)
    return {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}


def _kw(d):
    return dict(scale=d["scale"], lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])


@pytest.mark.parametrize("B,T,H,h0_std,g_dtype", [(2, 1, 4, 0.5, torch.bfloat16), (1, 7, 3, None, torch.float32),
                                                   (3, 33, 5, 0.02, torch.bfloat16), (40, 2, 32, 0.3, torch.bfloat16)])
def test_recurrent_matches_gold_and_chunk_oracle(B, T, H, h0_std, g_dtype):
    import kda_ascendc_b200 as K
    inp = O.make_inputs(B, T, H, seed0=11, h0_std=h0_std, g_dtype=g_dtype)
    d = _dev(inp)
    o, ht = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **_kw(d))
    torch.cuda.synchronize()
    o_g, ht_g = O.run_recurrent_gold(inp)
    o_c, ht_c = O.run_chunk_reference(inp)
    o, ht = o.float().cpu(), ht.cpu()
    scale_o = max(1.0, o_g.abs().max().item() / 0.06)
    scale_h = max(1.0, ht_g.abs().max().item())
    assert (o - o_g.float()).abs().max().item() <= 1e-3 * scale_o
    assert (ht - ht_g.float()).abs().max().item() <= 2e-3 * scale_h
    assert (o - o_c.float()).abs().max().item() <= 1e-3 * scale_o
    assert (ht - ht_c).abs().max().item() <= 2e-3 * scale_h


def test_prefill_then_decode_continues_the_sequence():
    import kda_ascendc_b200 as K
    B, T, H, n_dec = 2, 200, 4, 9           # prefill ends inside a chunk (200 = 12 * 16 + 8)
    inp = O.make_inputs(B, T + n_dec, H, seed0=5, regime="carry", h0_std=0.3)
    d = _dev(inp)
    flags = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                 output_final_state=True)
    o_full, ht_full = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                                     **flags, **_kw(d))
    sl = lambda x, a, b: x[:, a:b]
    o_pre, state = K.kda_bt16_fwd(*(sl(d[n], 0, T).contiguous() for n in ("q", "k", "v", "g", "beta")),
                                  initial_state=d["initial_state"], **flags, **_kw(d))
    outs = []
    for t in range(T, T + n_dec):            # one token per call, state updated in place
        o_t, state = K.kda_recurrent_fwd(*(sl(d[n], t, t + 1) for n in ("q", "k", "v", "g", "beta")),
                                         initial_state=state, inplace_state=True, **_kw(d))
        outs.append(o_t)
    torch.cuda.synchronize()
    o_dec = torch.cat(outs, dim=1).float()
    ref = o_full[:, T:].float()
    tol_o = 2e-2 * ref.abs().max().item()    # the reference's relative bound for O(1) states
    assert (o_dec - ref).abs().max().item() <= tol_o
    assert (o_pre.float() - o_full[:, :T].float()).abs().max().item() <= tol_o
    assert (state - ht_full).abs().max().item() <= 2e-2 * ht_full.abs().max().item()
    # and against the float64 gold over the whole sequence
    o_g, ht_g = O.run_recurrent_gold(inp)
    assert (o_dec.cpu() - o_g[:, T:].float()).abs().max().item() <= 2e-2 * o_g.abs().max().item()
    assert (state.cpu() - ht_g.float()).abs().max().item() <= 2e-2 * ht_g.abs().max().item()


def test_recurrent_inplace_and_strided_views():
    import kda_ascendc_b200 as K
    B, T, H = 2, 3, 6
    inp = O.make_inputs(B, T, H, seed0=3, h0_std=0.2)
    d = _dev(inp)
    o_ref, ht_ref = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **_kw(d))
    # in place
    st = d["initial_state"].clone()
    o_ip, st2 = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=st, inplace_state=True, **_kw(d))
    assert st2.data_ptr() == st.data_ptr()
    assert torch.equal(o_ip, o_ref) and torch.equal(st, ht_ref)
    # head-sliced views of a larger problem (strides passed through, no copy)
    hs = slice(2, 5)
    o_v, ht_v = K.kda_recurrent_fwd(d["q"][:, :, hs], d["k"][:, :, hs], d["v"][:, :, hs], d["g"][:, :, hs], d["beta"][:, :, hs],
                                    initial_state=d["initial_state"][:, hs].contiguous(), scale=d["scale"],
                                    lower_bound=d["lower_bound"], A_log=d["A_log"][hs].contiguous(),
                                    dt_bias=d["dt_bias"].view(H, 128)[hs].contiguous().view(-1))
    assert torch.equal(o_v, o_ref[:, :, hs]) and torch.equal(ht_v, ht_ref[:, hs])
    # zero state when none is given
    o_z, _ = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=None, **_kw(d))
    o_z2, _ = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=torch.zeros_like(d["initial_state"]), **_kw(d))
    assert torch.equal(o_z, o_z2)


def test_recurrent_argument_errors():
    import kda_ascendc_b200 as K
    inp = O.make_inputs(1, 1, 2, seed0=1, h0_std=0.1)
    d = _dev(inp)
    with pytest.raises(ValueError):
        K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=None, inplace_state=True, **_kw(d))
    with pytest.raises((ValueError, TypeError)):
        K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"], A_log=None, dt_bias=d["dt_bias"])


@pytest.mark.parametrize("B,T,H", [(1, 3, 2), (5, 2, 8), (40, 1, 32), (2, 40, 3)])
def test_recurrent_k_first_state_is_read_and_written_natively(B, T, H):
    """state_v_first=False: the kernel moves the [B,H,K,V] state itself.  Bit-equal to the V-first run on
    the transposed state, for every rows-per-warp choice (2 / 4 / 8, picked from B*H), for the in-place
    update, for the plan, and for calls long enough to run on the chunk kernels (T = 40)."""
    import kda_ascendc_b200 as K
    inp = O.make_inputs(B, T, H, seed0=13, h0_std=0.3)
    d = _dev(inp)
    args = [d[n] for n in ("q", "k", "v", "g", "beta")]
    o_v, h_v = K.kda_recurrent_fwd(*args, initial_state=d["initial_state"], **_kw(d))
    h0_k = d["initial_state"].transpose(-1, -2).contiguous()
    o_k, h_k = K.kda_recurrent_fwd(*args, initial_state=h0_k, state_v_first=False, **_kw(d))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    # many heads and a short call: the kernel with the lanes along v (its fp32 sums run in another order)
    own_kernel = B * H * 4 >= 2 * sms and T <= K.api.RECURRENT_MAX_TOKENS

    def same(o_a, h_a, o_b, h_b):
        if not own_kernel:
            return torch.equal(o_a, o_b) and torch.equal(h_a, h_b)
        return ((o_a.float() - o_b.float()).abs().max().item() <= 2.0 ** -8 * max(o_b.float().abs().max().item(), 1e-3)
                and (h_a - h_b).abs().max().item() <= 1e-5 * max(1.0, h_b.abs().max().item()))

    assert same(o_k, h_k, o_v, h_v.transpose(-1, -2))
    # no initial state, and the in-place update
    o_v0, h_v0 = K.kda_recurrent_fwd(*args, initial_state=None, **_kw(d))
    o_k0, h_k0 = K.kda_recurrent_fwd(*args, initial_state=None, state_v_first=False, **_kw(d))
    assert same(o_k0, h_k0, o_v0, h_v0.transpose(-1, -2))
    st = h0_k.clone()
    o_i, h_i = K.kda_recurrent_fwd(*args, initial_state=st, inplace_state=True, state_v_first=False, **_kw(d))
    assert h_i is st and torch.equal(o_i, o_k) and torch.equal(st, h_k)
    if T <= K.api.RECURRENT_MAX_TOKENS:
        st2 = h0_k.clone()
        plan = K.RecurrentPlan(*args, st2, state_v_first=False, **_kw(d))
        assert torch.equal(plan.step(), o_k) and torch.equal(st2, h_k)


@pytest.mark.parametrize("B,T,H,g_dtype", [(40, 2, 32, torch.bfloat16), (20, 4, 16, torch.float32)])
def test_recurrent_k_first_kernel_matches_gold(B, T, H, g_dtype):
    """The K-first kernel (lanes along v, chosen from B*H*4 >= 2 SMs) against the float64 recurrence and the
    chunk oracle, at the bounds of the V-first kernel."""
    import kda_ascendc_b200 as K
    inp = O.make_inputs(B, T, H, seed0=17, h0_std=0.3, g_dtype=g_dtype)
    d = _dev(inp)
    o, ht = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                initial_state=d["initial_state"].transpose(-1, -2).contiguous(), state_v_first=False, **_kw(d))
    torch.cuda.synchronize()
    o_g, ht_g = O.run_recurrent_gold(inp)
    o_c, ht_c = O.run_chunk_reference(inp)
    o, ht = o.float().cpu(), ht.transpose(-1, -2).cpu()
    scale_o = max(1.0, o_g.abs().max().item() / 0.06)
    scale_h = max(1.0, ht_g.abs().max().item())
    assert (o - o_g.float()).abs().max().item() <= 1e-3 * scale_o
    assert (ht - ht_g.float()).abs().max().item() <= 2e-3 * scale_h
    assert (o - o_c.float()).abs().max().item() <= 1e-3 * scale_o
    assert (ht - ht_c).abs().max().item() <= 2e-3 * scale_h


def test_recurrent_plan_matches_stepwise_calls():
    import kda_ascendc_b200 as K
    B, H, n_tok = 3, 4, 6
    inp = O.make_inputs(B, n_tok, H, seed0=8, h0_std=0.2)
    d = _dev(inp)
    # reference: one call per token
    state = d["initial_state"].clone()
    outs = []
    for t in range(n_tok):
        o_t, state = K.kda_recurrent_fwd(*(d[n][:, t:t + 1] for n in ("q", "k", "v", "g", "beta")), initial_state=state,
                                         inplace_state=True, **_kw(d))
        outs.append(o_t.clone())
    # plan: fixed one-token buffers refilled in place
    buf = {n: d[n][:, :1].clone() for n in ("q", "k", "v", "g", "beta")}
    st2 = d["initial_state"].clone()
    plan = K.RecurrentPlan(buf["q"], buf["k"], buf["v"], buf["g"], buf["beta"], st2, **_kw(d))
    for t in range(n_tok):
        for n in buf:
            buf[n].copy_(d[n][:, t:t + 1])
        o_t = plan.step()
        assert torch.equal(o_t, outs[t])
    assert torch.equal(st2, state) and plan.state is st2


def test_long_calls_run_on_the_chunk_kernels_and_keep_the_in_place_contract():
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import api
    B, T, H = 2, api.RECURRENT_MAX_TOKENS + 12, 5
    inp = O.make_inputs(B, T, H, seed0=14, h0_std=0.2)
    d = _dev(inp)
    o_ref, ht_ref = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"], **_kw(d))
    st = d["initial_state"].clone()
    o_ip, st2 = K.kda_recurrent_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=st, inplace_state=True, **_kw(d))
    assert st2.data_ptr() == st.data_ptr() and torch.equal(o_ip, o_ref) and torch.equal(st, ht_ref)
    o_g, ht_g = O.run_recurrent_gold(inp)
    assert (o_ref.float().cpu() - o_g.float()).abs().max().item() <= 1e-3 * max(1.0, o_g.abs().max().item() / 0.06)
    assert (ht_ref.cpu() - ht_g.float()).abs().max().item() <= 2e-3 * max(1.0, ht_g.abs().max().item())
