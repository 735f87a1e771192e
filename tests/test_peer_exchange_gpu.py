"""The peer-memory exchange of the sequence split on ONE GPU.

Two "ranks" share the device: both blocks are ordinary allocations of this process, so the peer
pointers are plain local pointers and no IPC is involved.  Kernels that wait on flags are only launched
after the kernels that raise those flags (one stream: pushes of both ranks, then both walks, then
both flag waits), so nothing ever spins on a kernel that has not run.  The second test lets a flag wait
run out on purpose -- a bounded wait on a word nothing writes, one second, status code 7, no fault --
and checks that the context stays usable.
"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

D = 128


def _rank_objects(world, hp, dev):
    """One _PeerExchange per emulated rank, all blocks on `dev`, wired to each other by hand."""
    from kda_ascendc_b200 import shard

    chains = world * hp
    n_recv, n_ent = chains * 2 * D * D, chains * D * D
    ranks = []
    for r in range(world):
        pe = shard._PeerExchange()
        pe.world, pe.rank, pe.hp, pe.dev = world, r, hp, dev
        pe.block = torch.zeros(n_recv + n_ent + shard._PeerExchange.FLAG_WORDS, dtype=torch.float32, device=dev)
        pe.recv = pe.block[:n_recv].view(world, hp, 2, D, D)
        pe.ent = pe.block[n_recv:n_recv + n_ent].view(world, hp, D, D)
        pe.flag_off = n_recv + n_ent
        pe.flags = pe.block[pe.flag_off:].view(torch.int32)
        pe.counters = torch.zeros(world + 1, dtype=torch.int32, device=dev)
        pe.final = torch.empty((hp, D, D), dtype=torch.float32, device=dev)
        ranks.append(pe)
    for pe in ranks:
        pe.peer_ptr = [q.block.data_ptr() for q in ranks]
        pe._build_args()
    return ranks


def test_push_walk_and_flags_between_two_emulated_ranks(cuda_device):
    from kda_ascendc_b200 import _lib, api, shard

    lib = _lib.load()
    dev = cuda_device
    world, hp = 2, 3
    chains = world * hp
    g = torch.Generator(device=dev).manual_seed(5)
    # transforms of a contraction-like walk: M near 0.9 I, Q of order 0.1, one set per (segment, chain)
    mq = torch.empty(world, chains, 2, D, D, device=dev)
    mq[:, :, 0] = 0.9 * torch.eye(D, device=dev) + 0.01 * torch.randn(world, chains, D, D, device=dev, generator=g)
    mq[:, :, 1] = 0.1 * torch.randn(world, chains, D, D, device=dev, generator=g)
    h0 = 0.2 * torch.randn(chains, D, D, device=dev, generator=g)
    want = shard.fold_states(mq, h0)                      # [world + 1, chains, 128, 128], the plain walk
    ranks = _rank_objects(world, hp, dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    stream = api._stream_handle()
    for epoch in (1, 2, 3):                               # buffers and flags are reused: run it three times
        for pe in ranks:                                  # every rank stores its transforms into the owners' buffers
            pe._push.src, pe._push.epoch = mq[pe.rank].data_ptr(), epoch
            assert lib.kda_peer_push(ctypes.byref(pe._push), stream) == 0, _lib.last_error()
        for pe in ranks:                                  # every owner walks its chains and stores the entry states
            own = h0[pe.rank * hp:(pe.rank + 1) * hp]
            pe._fold.h0, pe._fold.h0_stride, pe._fold.status = own.data_ptr(), D * D, status.data_ptr()
            pe._peer.epoch = epoch
            pe._peer.s_in_seg[world] = pe.final.data_ptr()
            assert lib.kda_state_fold_peer(ctypes.byref(pe._fold), ctypes.byref(pe._peer), stream) == 0, _lib.last_error()
        for pe in ranks:
            assert lib.kda_flag_wait(pe._wait_flags, world, epoch, status.data_ptr(), stream) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert int(status[0].item()) == 0
        for pe in ranks:
            assert torch.equal(pe.recv, mq[:, pe.rank * hp:(pe.rank + 1) * hp])               # what the all-to-all would deliver
            assert torch.equal(pe.ent.view(chains, D, D), want[pe.rank])                      # entry states of segment `rank`
            assert torch.equal(pe.final, want[world, pe.rank * hp:(pe.rank + 1) * hp])        # after the last segment
            assert pe.flags[:2 * world].tolist() == [epoch] * (2 * world)
            assert pe.counters.tolist() == [0] * (world + 1)                                  # left zeroed for the next run


def test_transform_pass_that_pushes_its_own_tiles(cuda_device):
    """kda_fwd_k2_state_push: the transform-pair pass stores (M, Q) straight into the owners' receive buffers
    and raises their flags -- the same bits as the plain pass followed by kda_peer_push."""
    from kda_ascendc_b200 import _lib, api, shard
    from oracle import kda_oracle as O

    dev = cuda_device
    world, hp, L = 2, 2, 64
    H = world * hp
    inp = O.make_inputs(1, world * L, H, seed0=4, regime="carry", h0_std=0.1)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    ranks = _rank_objects(world, hp, dev)
    segs = []
    for r in range(world):
        sl = slice(r * L, (r + 1) * L)
        seg = shard._Segment(d["q"][:, sl], d["k"][:, sl], d["v"][:, sl], d["g"][:, sl], d["beta"][:, sl], d["scale"],
                             d["lower_bound"], d["A_log"], d["dt_bias"])
        seg.k1()
        segs.append(seg)
    for epoch in (1, 2):
        for pe, seg in zip(ranks, segs):
            pe.recv.fill_(float("nan"))
        for pe, seg in zip(ranks, segs):
            push = pe.begin()
            assert push.epoch == epoch
            assert seg.transforms_push(push) == 0, _lib.last_error()
        torch.cuda.synchronize()
        for r, seg in enumerate(segs):
            mq = seg.transforms().clone()                   # the plain pass: [chains, 2, 128, 128]
            torch.cuda.synchronize()
            for dst, pe in enumerate(ranks):
                assert torch.equal(pe.recv[r], mq[dst * hp:(dst + 1) * hp])
        for pe in ranks:
            assert pe.flags[:world].tolist() == [epoch] * world and pe.counters.tolist() == [0] * (world + 1)
            assert api.check_device_status(segs[0].ws) == 0


@pytest.mark.parametrize("H,T", [(4, 256), (40, 64)])
def test_final_pass_that_waits_for_its_entry_state(cuda_device, H, T):
    """kda_fwd_k2_after_flags (the 8-row form for 4 chains, the 16-row form for 40): with the flags already raised
    the pass equals the plain one bit for bit; with flags nothing raises it gives up after the wait limit with
    status code 7 and the context stays usable."""
    from kda_ascendc_b200 import api, shard
    from oracle import kda_oracle as O

    dev = cuda_device
    inp = O.make_inputs(1, T, H, seed0=6, regime="carry", h0_std=0.3)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    seg = shard._Segment(d["q"], d["k"], d["v"], d["g"], d["beta"], d["scale"], d["lower_bound"], d["A_log"], d["dt_bias"])
    seg.k1()
    S = d["initial_state"].contiguous()
    o_p, h_p = (x.clone() for x in seg.outputs(S))
    flags = torch.full((4,), 3, dtype=torch.int32, device=dev)
    o_w, h_w = seg.outputs(S, after_flags=(flags.data_ptr(), 4, 3))
    assert o_w is not None, "the library should have a waiting kernel for this shape"
    torch.cuda.synchronize()
    assert torch.equal(o_w, o_p) and torch.equal(h_w, h_p) and api.check_device_status(seg.ws) == 0
    t0 = time.perf_counter()
    seg.outputs(S, after_flags=(flags.data_ptr(), 4, 4))          # epoch 4 never comes
    torch.cuda.synchronize()
    assert 0.5 < time.perf_counter() - t0 < 20.0
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        api.check_device_status(seg.ws)
    seg.ws[:4].zero_()
    o_a, h_a = seg.outputs(S)
    torch.cuda.synchronize()
    assert torch.equal(o_a, o_p) and torch.equal(h_a, h_p)


def test_a_flag_that_never_comes_ends_in_a_status_code(cuda_device):
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import _lib, api
    from oracle import kda_oracle as O

    lib = _lib.load()
    dev = cuda_device
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    stream = api._stream_handle()
    t0 = time.perf_counter()
    assert lib.kda_flag_wait(flags.data_ptr(), 2, 1, ws.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert 0.5 < time.perf_counter() - t0 < 10.0          # the limit is one second; the kernel came back by itself
    assert int(ws[:4].view(torch.int32).item()) == 7
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        api.check_device_status(ws)
    # a walk whose sources never signal: gives up before it reads or writes anything
    ranks = _rank_objects(2, 1, dev)
    pe = ranks[0]
    ws.zero_()
    pe.ent.fill_(-3.0)
    pe._fold.status = ws.data_ptr()
    pe._peer.epoch = 1
    assert lib.kda_state_fold_peer(ctypes.byref(pe._fold), ctypes.byref(pe._peer), stream) == 0
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 7
    assert bool((pe.ent == -3.0).all()) and pe.flags[:4].tolist() == [0, 0, 0, 0]
    # the context is intact: an ordinary forward still runs and is correct
    inp = O.make_inputs(1, 64, 2, seed0=3, h0_std=0.1)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    o, ht = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"], initial_state=d["initial_state"],
                           output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                           use_beta_sigmoid_in_kernel=True, lower_bound=d["lower_bound"], A_log=d["A_log"],
                           dt_bias=d["dt_bias"])
    o_r, ht_r = O.run_chunk_reference(inp)
    assert (o.float().cpu() - o_r.float()).abs().max().item() <= 1e-3
    assert (ht.cpu() - ht_r).abs().max().item() <= 2e-3
