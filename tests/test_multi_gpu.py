"""Two real ranks over NCCL (skipped on a single-GPU box): the sequence split and the
head shards, one process per GPU, against the one-pass forward computed on rank 0."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist

    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import shard
    from oracle import kda_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        T = 1024
        inp = O.make_inputs(1, T, 4, seed0=21, regime="carry", h0_std=0.1)
        d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
        kw = dict(scale=d["scale"], lower_bound=d["lower_bound"], A_log=d["A_log"], dt_bias=d["dt_bias"])
        o1, h1 = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["initial_state"],
                                output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                use_beta_sigmoid_in_kernel=True, **kw)
        # sequence split: rank r owns tokens [r*T/world, (r+1)*T/world)
        L = T // world
        sl = slice(rank * L, (rank + 1) * L)
        o2, h2 = shard.forward_seq_parallel(d["q"][:, sl], d["k"][:, sl], d["v"][:, sl], d["g"][:, sl],
                                            d["beta"][:, sl], initial_state=d["initial_state"], **kw)
        omax, hmax = o1.float().abs().max().item(), h1.abs().max().item()
        e_seq_o = (o2.float() - o1[:, sl].float()).abs().max().item() / omax
        e_seq_h = (h2 - h1).abs().max().item() / hmax
        # head shards: rank r owns a contiguous block of heads, nothing is exchanged
        o3, h3, (lo, hi) = shard.forward_head_shard(d["q"], d["k"], d["v"], d["g"], d["beta"], rank=rank, world=world,
                                                    initial_state=d["initial_state"], output_final_state=True, **kw)
        same = bool(torch.equal(o3, o1[:, :, lo:hi]) and torch.equal(h3, h1[:, lo:hi]))
        torch.cuda.synchronize()
        ret[rank] = (e_seq_o, e_seq_h, same)
    finally:
        dist.destroy_process_group()


def test_two_ranks_sequence_split_and_head_shards():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        e_o, e_h, same = ret[r]
        assert e_o < 1e-2 and e_h < 1e-2, (r, e_o, e_h)
        assert same, r
