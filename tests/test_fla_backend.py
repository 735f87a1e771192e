"""The FLA-convention adapter: verifier verdicts (CPU), results and registry dispatch (GPU)."""
import pytest
import torch

from kda_ascendc_b200 import fla_backend as FB

D = 128


def _cpu_inputs(H=2, T=32, dtype=torch.bfloat16):
    q = torch.randn(1, T, H, D).to(dtype)
    return q, q.clone(), q.clone(), torch.randn(1, T, H, D), torch.randn(1, T, H)


def test_verifier_reasons_on_cpu():
    q, k, v, g, beta = _cpu_inputs()
    full = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                A_log=torch.zeros(2))
    ok, why = FB.supports(q, k, v, g, beta, **full)
    assert not ok and "CUDA" in why                      # CPU tensors: no fallback
    with pytest.raises(NotImplementedError, match="kda_b200"):
        FB.chunk_kda(q, k, v, g, beta, **full)
    with pytest.raises(NotImplementedError):
        FB.fused_recurrent_kda(q, k, v, g, beta, **{k_: v_ for k_, v_ in full.items() if k_ != "safe_gate"})


@pytest.mark.gpu
def test_verifier_reasons_on_gpu():
    dev = torch.device("cuda", 0)
    q, k, v, g, beta = (t.to(dev) for t in _cpu_inputs())
    full = dict(use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, safe_gate=True, lower_bound=-5.0,
                A_log=torch.zeros(2, device=dev))
    assert FB.supports(q, k, v, g, beta, **full) == (True, None)
    for change, word in ((dict(use_gate_in_kernel=False), "fused"), (dict(safe_gate=False), "safe_gate"),
                         (dict(lower_bound=None), "lower_bound"), (dict(A_log=None), "A_log"),
                         (dict(return_intermediate_states=True), "intermediate")):
        ok, why = FB.supports(q, k, v, g, beta, **{**full, **change})
        assert not ok and word in why
    ok, why = FB.supports(q.float(), k, v, g, beta, **full)
    assert not ok and "bf16" in why
    ok, why = FB.supports(q[..., :64], k[..., :64], v, g, beta, **full)
    assert not ok and "128" in why
    ok, why = FB.supports(q, k, v.requires_grad_(True), g, beta, **full)
    assert not ok and "forward only" in why


@pytest.mark.gpu
def test_adapter_matches_native_calls_and_state_layouts():
    import kda_ascendc_b200 as K
    from oracle import kda_oracle as O
    inp = O.make_inputs(2, 100, 3, seed0=9, h0_std=0.1)
    dev = torch.device("cuda", 0)
    d = {k_: (v_.to(dev) if torch.is_tensor(v_) else v_) for k_, v_ in inp.items()}
    fla_kw = dict(scale=d["scale"], use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                  use_beta_sigmoid_in_kernel=True, safe_gate=True, lower_bound=d["lower_bound"], A_log=d["A_log"],
                  dt_bias=d["dt_bias"].view(3, D), output_final_state=True)
    with torch.inference_mode():
        o_n, h_n = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"],
                                  initial_state=d["initial_state"], output_final_state=True,
                                  use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                                  lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])
        o_v, h_v = FB.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                                transpose_state_layout=True, **fla_kw)
        o_k, h_k = FB.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"],
                                initial_state=d["initial_state"].transpose(-1, -2).contiguous(), **fla_kw)
        assert torch.equal(o_v, o_n) and torch.equal(h_v, h_n)
        assert torch.equal(o_k, o_n) and torch.equal(h_k, h_n.transpose(-1, -2))
        # recurrent adapter
        kw_r = {k_: v_ for k_, v_ in fla_kw.items() if k_ != "safe_gate"}
        o_r, h_r = FB.fused_recurrent_kda(d["q"][:, :5], d["k"][:, :5], d["v"][:, :5], d["g"][:, :5], d["beta"][:, :5],
                                          initial_state=d["initial_state"], transpose_state_layout=True, **kw_r)
        o_r2, h_r2 = K.kda_recurrent_fwd(d["q"][:, :5], d["k"][:, :5], d["v"][:, :5], d["g"][:, :5], d["beta"][:, :5],
                                         scale=d["scale"], initial_state=d["initial_state"], lower_bound=d["lower_bound"],
                                         A_log=d["A_log"], dt_bias=d["dt_bias"])
        assert torch.equal(o_r, o_r2) and torch.equal(h_r, h_r2)
        # FLA's default (K-first) layout on the recurrent adapter: moved by the kernel, no transpose
        o_rk, h_rk = FB.fused_recurrent_kda(d["q"][:, :5], d["k"][:, :5], d["v"][:, :5], d["g"][:, :5], d["beta"][:, :5],
                                            initial_state=d["initial_state"].transpose(-1, -2).contiguous(), **kw_r)
        assert torch.equal(o_rk, o_r2) and torch.equal(h_rk, h_r2.transpose(-1, -2))


@pytest.mark.gpu
def test_registered_backend_is_dispatched_by_fla():
    """After register(), FLA's own chunk_kda must hand an accepted call to this build: the result is
    then bit-identical to a direct call (FLA's Triton kernels would differ in the last bits)."""
    pytest.importorskip("fla")
    try:
        from fla.ops.kda import chunk_kda as fla_chunk_kda
        from fla.ops.kda.backends import kda_registry  # noqa: F401
    except Exception as e:  # noqa: BLE001
        pytest.skip("this FLA release has no backend registry: %r" % (e,))
    import kda_ascendc_b200 as K
    from oracle import kda_oracle as O
    assert FB.register()
    inp = O.make_inputs(1, 64, 2, seed0=2, h0_std=0.1)
    dev = torch.device("cuda", 0)
    d = {k_: (v_.to(dev) if torch.is_tensor(v_) else v_) for k_, v_ in inp.items()}
    with torch.inference_mode():
        o_f, h_f = fla_chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"],
                                 initial_state=d["initial_state"], output_final_state=True,
                                 use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                                 safe_gate=True, lower_bound=d["lower_bound"], transpose_state_layout=True,
                                 A_log=d["A_log"], dt_bias=d["dt_bias"])
        o_n, h_n = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"],
                                  initial_state=d["initial_state"], output_final_state=True,
                                  use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                                  lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])
    assert torch.equal(o_f, o_n) and torch.equal(h_f, h_n)
