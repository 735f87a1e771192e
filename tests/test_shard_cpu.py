"""CPU checks of the multi-GPU host logic: head ranges, the segment fold, and both exchange
patterns (all-to-all, all-gather) of a sequence split run as two gloo ranks (the per-segment
transforms come from the CPU oracle and the fold is the torch statement here; on GPUs the kernels
produce both)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kda_ascendc_b200 import shard
from oracle import kda_oracle as O

D = 128


def test_head_range_partitions_heads():
    for H, G in ((32, 8), (96, 8), (5, 4), (3, 8)):
        covered = []
        for r in range(G):
            lo, hi = shard.head_range(H, G, r)
            covered += list(range(lo, hi))
        assert covered == list(range(H))
    assert shard.head_range(32, 8, 3) == (12, 16)
    with pytest.raises(ValueError):
        shard.head_range(8, 4, 4)


def _segment_transforms(inp, lo, hi):
    """(M_seg, Q_seg) of tokens [lo, hi) from the oracle: Q from a zero state; M from the
    identity with v = 0 (then u = 0)."""
    seg = {k: (v[:, lo:hi] if torch.is_tensor(v) and v.ndim >= 3 and v.shape[1] == inp["q"].shape[1] else v)
           for k, v in inp.items()}
    B, _, H, _ = seg["q"].shape
    seg["initial_state"] = None
    _, Qs = O.run_chunk_reference(seg)
    segM = dict(seg, v=torch.zeros_like(seg["v"]),
                initial_state=torch.eye(D).expand(B, H, D, D).contiguous())
    _, Ms = O.run_chunk_reference(segM)
    return seg, Ms, Qs


def test_compose_entry_states_matches_one_pass():
    inp = O.make_inputs(1, 96, 2, seed0=5, regime="carry", h0_std=0.1)
    o_full, h_full = O.run_chunk_reference(inp)
    cuts = [0, 32, 64, 96]
    parts = [_segment_transforms(inp, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
    states = shard.compose_entry_states([p[1] for p in parts], [p[2] for p in parts], inp["initial_state"])
    assert (states[-1] - h_full).abs().max().item() < 2e-5 * max(1.0, h_full.abs().max().item())
    outs = []
    for (seg, _, _), S in zip(parts, states[:-1]):
        seg = dict(seg, initial_state=S)
        outs.append(O.run_chunk_reference(seg)[0])
    o_cat = torch.cat(outs, 1)
    assert (o_cat.float() - o_full.float()).abs().max().item() <= 2.0 ** -8 * o_full.float().abs().max().item()
    # a wrong fold (segments swapped) is far off: the check has teeth
    bad = shard.compose_entry_states([parts[1][1], parts[0][1], parts[2][1]],
                                     [parts[1][2], parts[0][2], parts[2][2]], inp["initial_state"])
    assert (bad[-1] - h_full).abs().max().item() > 1e-3 * h_full.abs().max().item()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret, T=64, H=2, cases=(("a2a", 1, None), ("gather", 1, None), ("a2a", 2, None),
                                                         ("gather", 2, None))):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        inp = O.make_inputs(1, T, H, seed0=9, regime="carry", h0_std=0.1)
        L = T // world
        o_full, h_full = O.run_chunk_reference(inp)
        res = {}
        for mode, sub, two_level in cases:
            Ls = L // sub
            parts = [_segment_transforms(inp, rank * L + s * Ls, rank * L + (s + 1) * Ls) for s in range(sub)]
            # [sub * chains, 2, 128, 128], sub-segment major
            mq = torch.cat([torch.stack([M[0], Q[0]], dim=1) for _, M, Q in parts]).contiguous()
            entry, final = shard.exchange_and_fold(mq, inp["initial_state"], rank, world, mode=mode, sub=sub,
                                                   two_level=two_level, walk=shard._walk_torch, want_final=True)
            assert tuple(entry.shape) == (sub, H, D, D)
            outs = [O.run_chunk_reference(dict(seg, initial_state=entry[s].reshape(1, H, D, D)))[0]
                    for s, (seg, _, _) in enumerate(parts)]
            o_loc = torch.cat(outs, 1)
            eo = (o_loc.float() - o_full[:, rank * L:(rank + 1) * L].float()).abs().max().item()
            eh = (final.view(1, H, D, D) - h_full).abs().max().item()
            res[(mode, sub, two_level)] = (eo, eh)
        # without the final state only the entry states come back (same exchange, same walk: same bits)
        mode, sub, two_level = cases[-1]
        entry2, none = shard.exchange_and_fold(mq, inp["initial_state"], rank, world, mode=mode, sub=sub,
                                               two_level=two_level, walk=shard._walk_torch)
        assert none is None and torch.equal(entry2, entry)
        ret[rank] = (res, o_full.float().abs().max().item(), h_full.abs().max().item())
    finally:
        dist.destroy_process_group()


def test_sequence_split_over_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == [0, 1]
    for r in range(world):
        res, omax, hmax = ret[r]
        for key, (eo, eh) in res.items():
            assert eo <= 2.0 ** -8 * omax, (r, key, eo)
            assert eh <= 2e-5 * max(1.0, hmax), (r, key, eh)


def test_sequence_split_over_four_gloo_ranks_two_levels():
    """Four ranks, four chains: the all-to-all with one chain per rank, and with two sub-segments per
    rank the flat all-gather (eight segments), the two-level all-gather and the two-level all-to-all."""
    world = 4
    mgr = mp.Manager()
    ret = mgr.dict()
    cases = (("a2a", 1, None), ("gather", 2, None), ("gather", 2, True), ("a2a", 2, None))
    mp.spawn(_rank_main, args=(world, _free_port(), ret, 128, 4, cases), nprocs=world, join=True)
    assert sorted(ret.keys()) == list(range(world))
    for r in range(world):
        res, omax, hmax = ret[r]
        assert len(res) == len(cases)
        for key, (eo, eh) in res.items():
            assert eo <= 2.0 ** -8 * omax, (r, key, eo)
            assert eh <= 2e-5 * max(1.0, hmax), (r, key, eh)


@pytest.mark.parametrize("world,hp", [(2, 3), (4, 8), (8, 4), (8, 2)])
def test_peer_exchange_argument_blocks(world, hp):
    """The pointer arithmetic of the peer exchange for up to eight ranks, on CPU tensors (nothing is launched):
    every rank's push targets slot [rank] of each owner's receive buffer and flag row, its walk writes slot
    [rank] of each segment owner's entry buffer and entry-flag row, all inside the owners' blocks."""
    chains = world * hp
    n_recv, n_ent = chains * 2 * D * D, chains * D * D
    ranks = []
    for r in range(world):
        pe = shard._PeerExchange()
        pe.world, pe.rank, pe.hp, pe.dev = world, r, hp, torch.device("cpu")
        pe.block = torch.zeros(n_recv + n_ent + shard._PeerExchange.FLAG_WORDS, dtype=torch.float32)
        pe.recv = pe.block[:n_recv].view(world, hp, 2, D, D)
        pe.ent = pe.block[n_recv:n_recv + n_ent].view(world, hp, D, D)
        pe.flag_off = n_recv + n_ent
        pe.flags = pe.block[pe.flag_off:].view(torch.int32)
        pe.counters = torch.zeros(world + 1, dtype=torch.int32)
        pe.final = torch.empty((hp, D, D), dtype=torch.float32)
        ranks.append(pe)
    for pe in ranks:
        pe.peer_ptr = [q.block.data_ptr() for q in ranks]
        pe._build_args()
    assert 2 * world <= 32 and 32 + 4 * world <= shard._PeerExchange.FLAG_WORDS      # flag rows and self-check words fit
    for pe in ranks:
        r = pe.rank
        assert pe._push.world == world and pe._push.slice_floats == hp * 2 * D * D
        assert pe._push.dst_offset_floats == r * hp * 2 * D * D
        assert pe._fold.mq == pe.recv.data_ptr() and pe._fold.n_chains == hp and pe._fold.n_seg == world
        assert pe._peer.wait_flags == pe.flags.data_ptr() and pe._peer.n_wait == world and pe._peer.n_signal == world
        assert pe._wait_flags == pe.flags[world:].data_ptr()
        for d, q in enumerate(ranks):
            assert pe._push.dst[d] == q.recv.data_ptr()
            assert pe._push.dst[d] + 4 * pe._push.dst_offset_floats == q.recv[r].data_ptr()       # slot [source rank]
            assert pe._push.flag[d] == q.flags[r:].data_ptr()
            assert pe._peer.s_in_seg[d] == q.ent[r].data_ptr()                                   # slot [owner of the chains]
            assert pe._peer.signal[d] == q.flags[world + r:].data_ptr()
        assert pe._peer.s_in_seg[world] is None


def test_exchange_mode_choice():
    assert shard.exchange_mode(32, 8) == "a2a" and shard.exchange_mode(16, 8) == "a2a"
    assert shard.exchange_mode(5, 4) == "gather" and shard.exchange_mode(32, 8, "gather") == "gather"
    with pytest.raises(ValueError):
        shard.exchange_mode(5, 4, "a2a")
    with pytest.raises(RuntimeError):
        shard.fold_states(torch.zeros(1, 1, 2, D, D), None)       # the fold is a CUDA kernel: no CPU path
