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
    if regime == "baseline":
        # benchmark distribution: the absolute bounds of the one-pass path, against the oracle
        assert (o2.float().cpu() - o_r.float()).abs().max().item() <= 1e-3
        assert (h2.cpu() - h_r).abs().max().item() <= 2e-3
    else:
        # O(1) states that persist: the reference's relative bound, 2e-2 of absmax, against the oracle
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


@pytest.mark.parametrize("chains,n_seg", [(1, 1), (3, 5), (8, 8)])
def test_fold_kernel_against_float64(cuda_device, chains, n_seg):
    """kda_state_fold (fp32 FMAs) against the same walk in float64, on strided and dense layouts."""
    g = torch.Generator(device=cuda_device).manual_seed(chains * 10 + n_seg)
    big = torch.randn(n_seg + 1, chains + 2, 2, 128, 128, device=cuda_device, generator=g) * 0.09
    mq = big[:n_seg, 1:chains + 1]                                   # a strided view: the fold reads it in place
    h0 = torch.randn(chains, 128, 128, device=cuda_device, generator=g)
    out = shard.fold_states(mq, h0)
    S = h0.double()
    for j in range(n_seg):
        assert (out[j].double() - S).abs().max().item() <= 2e-5 * max(1.0, S.abs().max().item())
        S = S @ mq[j, :, 0].double() + mq[j, :, 1].double()
    assert (out[n_seg].double() - S).abs().max().item() <= 2e-5 * max(1.0, S.abs().max().item())
    # zero entry state, fewer segments than the buffer holds
    out0 = shard.fold_states(mq, None, n_seg=max(0, n_seg - 1))
    assert out0.shape[0] == max(0, n_seg - 1) + 1 and not out0[0].any()


def test_transform_pair_pass_matches_the_two_single_passes(cuda_device):
    """kda_fwd_k2_state(zero_u = 2) returns [chains][2][128][128] = (M, Q) of the two single passes."""
    import ctypes
    from kda_ascendc_b200 import _lib, api
    inp = O.make_inputs(2, 96, 3, seed0=17, regime="carry", h0_std=0.1)
    d = to_device(inp, cuda_device)
    B, T, H = 2, 96, 3
    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(K.workspace_bytes(B, T, H), dtype=torch.uint8, device=cuda_device)
    o = torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=cuda_device)
    eye = torch.eye(128, device=cuda_device).expand(B, H, 128, 128).contiguous()
    M, Q = torch.empty_like(eye), torch.empty_like(eye)
    mq = torch.empty(B * H, 2, 128, 128, device=cuda_device)

    def args(h0, ht):
        return api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"], lower_bound=d["lower_bound"],
                             A_log=d["A_log"], dt_bias=d["dt_bias"], h0=h0, o=o, ht=ht, workspace=ws, flags=7)
    a = args(eye, M)
    assert lib.kda_fwd_k1(ctypes.byref(a), st) == 0, _lib.last_error()
    assert lib.kda_fwd_k2_state(ctypes.byref(a), 1, st) == 0, _lib.last_error()
    a = args(None, Q)
    assert lib.kda_fwd_k2_state(ctypes.byref(a), 0, st) == 0, _lib.last_error()
    a = args(None, mq)
    assert lib.kda_fwd_k2_state(ctypes.byref(a), 2, st) == 0, _lib.last_error()
    torch.cuda.synchronize()
    # the pair launch may run another organisation of K2 (twice the chains): fp32 summation order only
    assert (mq[:, 0].view(B, H, 128, 128) - M).abs().max().item() <= 1e-5
    assert (mq[:, 1].view(B, H, 128, 128) - Q).abs().max().item() <= 1e-4 * max(1.0, Q.abs().max().item())
    assert lib.kda_fwd_k2_state(ctypes.byref(a), 3, st) == -1 and "zero_u" in _lib.last_error()


def test_two_level_fold_equals_the_flat_walk(cuda_device):
    """Composing the transforms of a rank's sub-segments first (transition matrices with use_q = 0,
    offsets with use_q = 1, written straight into an (M, Q) buffer through final_out) and walking the
    composed transforms gives the states of the flat walk over all sub-segments."""
    g = torch.Generator(device=cuda_device).manual_seed(5)
    ranks, sub, chains = 3, 4, 2
    mq = torch.randn(ranks * sub, chains, 2, 128, 128, device=cuda_device, generator=g) * 0.09
    h0 = torch.randn(chains, 128, 128, device=cuda_device, generator=g)
    flat = shard.fold_states(mq, h0)                                  # [ranks * sub + 1, chains, 128, 128]
    rank_mq = torch.full((ranks, chains, 2, 128, 128), float("nan"), device=cuda_device)
    for r in range(ranks):
        m5 = mq[r * sub:(r + 1) * sub]
        shard._walk_cuda(m5[1:], m5[0, :, 0], sub - 1, use_q=False, final_out=rank_mq[r, :, 0])
        shard._walk_cuda(m5[1:], m5[0, :, 1], sub - 1, use_q=True, final_out=rank_mq[r, :, 1])
    top = shard.fold_states(rank_mq, h0)                              # entry state of every rank
    for r in range(ranks + 1):
        ref = flat[r * sub]
        assert (top[r] - ref).abs().max().item() <= 5e-5 * max(1.0, ref.abs().max().item()), r
    for r in range(ranks):                                            # the local walk from the rank's entry state
        loc = torch.empty(sub, chains, 128, 128, device=cuda_device)
        shard._walk_cuda(mq[r * sub:(r + 1) * sub], top[r], sub - 1, s_in=loc)
        ref = flat[r * sub:(r + 1) * sub]
        assert (loc - ref).abs().max().item() <= 5e-5 * max(1.0, ref.abs().max().item()), r
