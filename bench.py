"""Benchmark of the KDA chunked forward (BT=16) -- one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]

A step is one whole forward (K1 + K2) over one batch of seeded synthetic inputs of the
headline workload: B=1, T=8192, H=32, K=V=128, bf16 (q, k, v, g_raw ~ N(0,1) bf16, beta
logits ~ N(0,1), A_log = log U(1,16), dt_bias ~ U(-0.1,0.1), lower_bound -5, initial
state ~ N(0, 0.02)).

N = 1: `value` = tokens/s of that forward with inputs resident in HBM.
N > 1 (one process per GPU under torchrun): STRONG scaling -- the same single sequence is
spread over the N GPUs, two ways, both timed (max over ranks, device events):
  * head shard: rank r runs heads [r*H/N, (r+1)*H/N), nothing is exchanged;
  * sequence split: rank r runs tokens [r*T/N, (r+1)*T/N): K1, one transform pass, an
    all-to-all + fp32 fold + all-to-all of the segment transforms, K2 from the entry state.
`value` = 8192 tokens / the faster of the two, `strong` holds both with the per-phase timeline
of the split, `replicas` the weak figure (one whole sequence per GPU, no exchange) and
`seq_parallel` the long-context configuration (B=1 T=131072 H=16 split over the N ranks: time,
speed-up over one GPU, and the largest deviation of any rank's slice from the one-GPU run).

Other keys: `e2e` -- tokens/s through the public Python API with pinned host buffers, H2D and
D2H copies inside the timed region; `roofline` -- the dominant kernel against the measured HBM
copy bandwidth; `kernels` -- both kernels; `parity` -- the timed outputs of one head against the
CPU oracle, computed after the timed region (out of bound or non-finite => exit code 1);
`cpu_baseline` -- the CPU port of the reference's torch chunk forward over the whole workload on
all host cores; `clocks` -- nvidia-smi samples taken during the timed region.

`--impl reference` times the CPU port of the reference's torch forward
(oracle/kda_oracle.py, looped exactly like the reference) on the host cores: every step is the
WHOLE workload, one process per core over the heads, and prints the same line with
"impl": "reference".

`--impl reference_gpu` (an extra, not part of the two-arm contract) times the reference's
own Triton kernels on this GPU when the reference package has been installed under
baseline/_ref (git-ignored); without it the line says "unavailable".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

B, T, H, D = 1, 8192, 32, 128
BT = 16
METRIC = "KDA fwd tokens/s at B1 T8192 H32 K=V=128 bf16"
K2_VARIANT = 0               # 0 = the library's automatic choice (always, except in --kernels-only captures)
# long-context configuration of the sequence split
SP_T, SP_H = 131072, 16
# parity bounds of the forward against the reference's torch chunk implementation
O_TOL, HT_TOL = 1e-3, 2e-3
# algorithmic bytes / flops per (token, head) of the two-kernel contract of the reference
K1_BYTES_PER_TH = 2084.0     # reads q,k,v,g bf16 + beta; writes w,u bf16, g fp32, Aqk bf16
K2_BYTES_PER_TH = 1856.0     # reads w,u,q,k,g,Aqk,g_last; writes o
K1_FLOPS_PER_CHUNK = 262144.0
K2_FLOPS_PER_CHUNK = 1638400.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of each kernel on the headline shape, from
# an ncu capture (profiles/kda_k1_k2_B1_T8192_H32.md, which names the commit it was taken at).  It is
# reported only for that shape and only while the record layout it was captured with is current.
NCU_TRAFFIC = dict(shape=(1, 8192, 32), record_bytes=26112, source="profiles/kda_k1_k2_B1_T8192_H32.md",
                   bytes={"kda_k1": 642.14e6, "kda_k2": 489.44e6})


def merge_exchange_marks(names, values):
    """The peer exchange marks the end of its push and of its walk inside the `exchange_fold` phase of a plan's
    timeline: fold the three intervals back into one phase (so that the timeline reads the same for both
    transports) and return the parts separately (ms; None for the NCCL exchange)."""
    if "exchange_push" not in names:
        return list(names), list(values), None
    parts = dict(zip(names, values))
    total = parts["exchange_push"] + parts["exchange_walk"] + parts["exchange_fold"]
    out_n = [n for n in names if n not in ("exchange_push", "exchange_walk")]
    out_v = [total if n == "exchange_fold" else parts[n] for n in out_n]
    return out_n, out_v, dict(push=parts["exchange_push"] * 1e3, walk_incl_waiting_for_peers=parts["exchange_walk"] * 1e3,
                              entry_states_arrive=parts["exchange_fold"] * 1e3)


def workload_text(n_gpus):
    if n_gpus == 1:
        return "KDA fwd B=1 T=8192 H=32 K=V=128 BT=16 bf16 (headline benchmark shape) on one GPU"
    return ("KDA fwd B=1 T=8192 H=32 K=V=128 BT=16 bf16 (headline benchmark shape): ONE sequence strong-scaled "
            "over %d GPUs" % n_gpus)


def make_config(n_gpus):
    """The `config` object of both arms (the reference arm times the same problem)."""
    return dict(workload=workload_text(n_gpus), global_batch=B, seq_len=T, heads=H,
                l2="inputs + K1->K2 records of one step = 0.7 GB, larger than the 126 MB L2: no flush needed")


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


# ----------------------------------------------------------------------------
# CPU port timing (cpu_baseline leg and the reference arm)
# ----------------------------------------------------------------------------
_CPU_INPUTS = {}


def _cpu_head(args):
    """One head of the workload, all T tokens, through the looped CPU port (inputs are generated
    once per worker process and kept; only the forward is timed)."""
    head, t_len, seed = args
    import torch as _t
    _t.set_num_threads(1)
    from oracle import kda_oracle as O
    key = (head, t_len, seed)
    if key not in _CPU_INPUTS:
        _CPU_INPUTS[key] = O.make_inputs(1, t_len, 1, seed0=seed, head_offset=head, h0_std=0.02)
    t0 = time.perf_counter()
    O.run_chunk_reference(_CPU_INPUTS[key], loop_heads=True)
    return time.perf_counter() - t0


def cpu_forward_steps(steps, warmup):
    """`warmup + steps` passes of the WHOLE workload (all H heads x T tokens = 16,384 chunk tiles) over
    the host cores, one process per core, one head per task.  Returns (mean seconds per step, workers)."""
    import multiprocessing as mp
    ncpu = os.cpu_count() or 1
    workers = max(1, min(ncpu, H))
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(workers) as pool:
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            pool.map(_cpu_head, [(h, T, 42) for h in range(H)], chunksize=1)
            dt = time.perf_counter() - t0
            if it >= warmup:
                times.append(dt)
    return statistics.mean(times), workers


def cpu_baseline_sample():
    """One warm-up and one timed pass of the whole workload on all host cores."""
    step_s, workers = cpu_forward_steps(1, 1)
    return dict(value=B * T / step_s, unit="tokens/s", cores=workers, kind="port",
                sample="the whole workload (%d heads x %d tokens = %d chunk tiles) per step, looped torch port of the "
                       "reference's chunk forward, one process per core, %.1f s per step, nothing extrapolated"
                       % (H, T, H * (T // BT), step_s))


def run_reference_arm(steps, warmup, n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step_s, workers = cpu_forward_steps(steps, warmup)
    value = B * T / step_s
    sample = ("every step is the whole workload (%d heads x %d tokens = %d chunk tiles), looped torch port of the "
              "reference's chunk forward, %d processes (one per core, one head per task); nothing extrapolated"
              % (H, T, H * (T // BT), workers))
    line = dict(impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=n_gpus, steps=steps,
                warmup=warmup, ms_per_step=step_s * 1e3, higher_is_better=True,
                scaling="weak" if n_gpus == 1 else "strong", vs_baseline=None,
                dtype="bf16", data="synthetic", config=make_config(n_gpus), device="host CPU",
                host_cores=os.cpu_count(), arithmetic="fp32 with bf16-rounded q/k (the reference's torch chunk forward)",
                cpu_baseline=dict(value=value, unit="tokens/s", cores=workers, kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def _latency_stats(samples_ms):
    """min / median / p20 / p80 of single-forward latencies (K1 + K2 of one step, synchronised
    per step), the figures the reference's own benchmarks report."""
    xs = sorted(samples_ms)
    pick = lambda f: xs[min(len(xs) - 1, int(f * len(xs)))]
    return dict(min=xs[0], median=statistics.median(xs), p20=pick(0.2), p80=pick(0.8), samples=len(xs))


def decode_leg(device, hbm_gbs):
    """The token recurrence (decode) on B=64 sequences x 32 heads, one token per call through the C
    ABI, device-timed; three state sets (268 MB) are rotated so that no call finds its state in L2.
    An extra figure beside the headline: the step is bound by the 128 KiB of state it moves per head."""
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import _lib, api
    lib = _lib.load()
    Bd, Td = 64, 1
    g = torch.Generator(device=device).manual_seed(7)
    rn = lambda *s: torch.randn(*s, device=device, generator=g)
    q, k, v, gr = (rn(Bd, Td, H, D).bfloat16() for _ in range(4))
    beta = rn(Bd, Td, H)
    A_log = torch.log(1.0 + 15.0 * torch.rand(H, device=device, generator=g))
    dtb = torch.rand(H * D, device=device, generator=g) * 0.2 - 0.1
    states = [rn(Bd, H, D, D) * 0.1 for _ in range(3)]
    o = torch.empty(Bd, Td, H, D, dtype=torch.bfloat16, device=device)
    argl = [api.make_args(q, k, v, gr, beta, scale=D ** -0.5, lower_bound=-5.0, A_log=A_log, dt_bias=dtb, h0=s_, o=o,
                          ht=s_, workspace=None, flags=7) for s_ in states]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    n = 30
    for i in range(3):
        assert lib.kda_recurrent_fwd(ctypes.byref(argl[i % 3]), stream) == 0, _lib.last_error()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        assert lib.kda_recurrent_fwd(ctypes.byref(argl[i % 3]), stream) == 0, _lib.last_error()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / n * 1e3
    nbytes = Bd * H * 2 * D * D * 4 + Bd * Td * H * (4 * D * 2 + 4 + D * 2)
    gbs = nbytes / (us * 1e-6) / 1e9
    return dict(workload="token recurrence B=64 T=1 H=32 (decode step, in-place state)", us_per_step=us,
                tokens_per_s=Bd * Td / (us * 1e-6), bytes_per_step=nbytes, achieved_GBps=gbs, hbm_frac=gbs / hbm_gbs)


def make_device_inputs(seed: int, device, Bx=None, Tx=None, Hx=None):
    """Seeded inputs of a workload (default: the headline one), generated on the device."""
    Bx, Tx, Hx = B if Bx is None else Bx, T if Tx is None else Tx, H if Hx is None else Hx
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=device, generator=g)
    d = dict(q=rn(Bx, Tx, Hx, D).bfloat16(), k=rn(Bx, Tx, Hx, D).bfloat16(), v=rn(Bx, Tx, Hx, D).bfloat16(),
             g=rn(Bx, Tx, Hx, D).bfloat16(), beta=rn(Bx, Tx, Hx),
             A_log=torch.log(1.0 + 15.0 * torch.rand(Hx, device=device, generator=g)),
             dt_bias=torch.rand(Hx * D, device=device, generator=g) * 0.2 - 0.1,
             h0=rn(Bx, Hx, D, D) * 0.02)
    return d


def oracle_head(d, head):
    """The CPU oracle (the reference's torch chunk forward, restated) on ONE head of device inputs `d`,
    all tokens: returns (o [B, T, 1, 128] bf16, ht [B, 1, 128, 128]) on the CPU."""
    from oracle import kda_oracle as O
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    sub = dict(q=d["q"][:, :, head:head + 1].cpu(), k=d["k"][:, :, head:head + 1].cpu(),
               v=d["v"][:, :, head:head + 1].cpu(), g=d["g"][:, :, head:head + 1].cpu(),
               beta=d["beta"][:, :, head:head + 1].cpu(), A_log=d["A_log"][head:head + 1].cpu(),
               dt_bias=d["dt_bias"].view(-1, D)[head:head + 1].reshape(-1).cpu(),
               initial_state=d["h0"][:, head:head + 1].cpu(), scale=D ** -0.5, lower_bound=-5.0)
    return O.run_chunk_reference(sub)


def parity_record(err_o, err_ht, finite, what):
    ok = bool(finite) and err_o <= O_TOL and (err_ht is None or err_ht <= HT_TOL)
    return dict(ok=ok, o_max_abs=err_o, ht_max_abs=err_ht, o_bound=O_TOL, ht_bound=HT_TOL, finite=bool(finite),
                checked=what, oracle="oracle/kda_oracle.py (restates tests/test_torch_reference.py:23-213 of the reference)")


def _view_args(api, d, sl_h, o, ht, ws, h0):
    """Argument block over a head slice of full [B, T, H, 128] inputs (strided views, no copy)."""
    return api.make_args(d["q"][:, :, sl_h], d["k"][:, :, sl_h], d["v"][:, :, sl_h], d["g"][:, :, sl_h],
                         d["beta"][:, :, sl_h], scale=D ** -0.5, lower_bound=-5.0, A_log=d["A_log"][sl_h].contiguous(),
                         dt_bias=d["dt_bias"].view(-1, D)[sl_h].contiguous().view(-1), h0=h0, o=o, ht=ht,
                         workspace=ws, flags=7)


def run_gpu_arm(steps, warmup, n_gpus, kernels_only=False):
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import _lib, api, shard

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.load()
    hbm_gbs, tc_tflops, peak_kind = load_peaks()
    warmup = max(warmup, 3)
    scale = D ** -0.5
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n_steps):
        """`warmup` untimed calls, then `n_steps` calls between a barrier + synchronize on both sides."""
        for _ in range(warmup):
            fn()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n_steps):
            fn()
        t1.record()
        barrier()
        return t0.elapsed_time(t1)

    def max_over_ranks(values):
        if dist is None:
            return [float(x) for x in values]
        t = torch.tensor(list(values), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    # the same single sequence on every rank (strong scaling splits it; N = 1 runs it whole)
    d = make_device_inputs(42, dev)
    ws = torch.empty(K.workspace_bytes(B, T, H), dtype=torch.uint8, device=dev)
    o = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=dev)
    ht = torch.empty(B, H, D, D, dtype=torch.float32, device=dev)
    args = api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale, lower_bound=-5.0,
                         A_log=d["A_log"], dt_bias=d["dt_bias"], h0=d["h0"], o=o, ht=ht, workspace=ws, flags=7,
                         k2_variant=K2_VARIANT)

    def fwd_whole():
        rc = lib.kda_fwd(ctypes.byref(args), stream)
        if rc != 0:
            raise RuntimeError(_lib.last_error())

    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- one whole sequence per GPU, inputs resident in HBM: `value` at N = 1, `replicas` at N > 1 ----
    ms_whole = timed(fwd_whole, steps)
    launches = steps * lib.kda_last_launch_count()

    # ---- per-kernel durations of the whole-sequence forward (events on the launching stream) ----
    # The pairs are queued back to back and read after one synchronise: with the stream never empty the
    # interval between two events is the kernel's device time, not the host's launch path (tensor-map
    # encoding and the launch itself, about 6 us, would otherwise sit inside K1's interval).
    k1_ms, k2_ms = [], []
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    assert lib.kda_fwd(ctypes.byref(args), stream) == 0, _lib.last_error()   # keeps the GPU busy while the first pair is queued
    for e in ev:
        e[0].record()
        assert lib.kda_fwd_k1(ctypes.byref(args), stream) == 0, _lib.last_error()
        e[1].record()
        assert lib.kda_fwd_k2(ctypes.byref(args), stream) == 0, _lib.last_error()
        e[2].record()
    torch.cuda.synchronize()
    for e in ev:
        k1_ms.append(e[0].elapsed_time(e[1]))
        k2_ms.append(e[1].elapsed_time(e[2]))
    status = api.check_device_status(ws)
    assert status == 0, "device status %d" % status
    finite = bool(torch.isfinite(o.float()).all()) and bool(torch.isfinite(ht).all())

    if kernels_only:
        if rank == 0:
            print(json.dumps(dict(kernels_only=True, ms_per_step=ms_whole / steps, k1_us=statistics.mean(k1_ms) * 1e3,
                                  k2_us=statistics.mean(k2_ms) * 1e3)), flush=True)
            if sampler is not None:
                sampler.stop()
        if dist is not None:
            dist.destroy_process_group()
        return
    o_whole, ht_whole = o.clone(), ht.clone()      # the timed outputs, for the parity check below

    # ---- strong scaling of the one sequence over the ranks (N > 1) ----
    strong = None
    if world > 1:
        lo, hi = shard.head_range(H, world, rank)
        hl = hi - lo
        ws_h = torch.empty(K.workspace_bytes(B, T, hl), dtype=torch.uint8, device=dev)
        o_h = torch.empty(B, T, hl, D, dtype=torch.bfloat16, device=dev)
        ht_h = torch.empty(B, hl, D, D, dtype=torch.float32, device=dev)
        args_h = _view_args(api, d, slice(lo, hi), o_h, ht_h, ws_h, d["h0"][:, lo:hi].contiguous())

        def fwd_heads():
            rc = lib.kda_fwd(ctypes.byref(args_h), stream)
            if rc != 0:
                raise RuntimeError(_lib.last_error())

        ms_heads = timed(fwd_heads, steps)
        launches_heads = steps * lib.kda_last_launch_count()
        hk1, hk2 = [], []
        evh = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(min(steps, 10))]
        fwd_heads()                       # keeps the GPU busy while the first pair is queued (as above)
        for e in evh:
            e[0].record()
            assert lib.kda_fwd_k1(ctypes.byref(args_h), stream) == 0, _lib.last_error()
            e[1].record()
            assert lib.kda_fwd_k2(ctypes.byref(args_h), stream) == 0, _lib.last_error()
            e[2].record()
        torch.cuda.synchronize()
        for e in evh:
            hk1.append(e[0].elapsed_time(e[1]))
            hk2.append(e[1].elapsed_time(e[2]))

        L = T // world
        tsl = slice(rank * L, (rank + 1) * L)
        plan = shard.SeqParallelPlan(d["q"][:, tsl], d["k"][:, tsl], d["v"][:, tsl], d["g"][:, tsl], d["beta"][:, tsl],
                                     scale=scale, initial_state=d["h0"], lower_bound=-5.0, A_log=d["A_log"],
                                     dt_bias=d["dt_bias"])
        ms_seq = timed(plan.run, steps)
        # per-phase timeline: steps queued back to back behind one barrier (as in the timed region: a step
        # started from a barrier would show the ranks' barrier-exit skew inside its exchange phase)
        phases = {}
        tls = [[] for _ in range(min(steps, 10))]
        barrier()
        plan.run()
        for tl in tls:
            o_s, ht_s = plan.run(timeline=tl)
        torch.cuda.synchronize()
        for tl in tls:
            for (n0, e0_), (n1, e1_) in zip(tl[:-1], tl[1:]):
                phases.setdefault(n1, []).append(e0_.elapsed_time(e1_))
        ph_names = list(phases)
        ph_max = max_over_ranks([statistics.mean(phases[n]) for n in ph_names])
        ph_names, ph_max, exchange_parts = merge_exchange_marks(ph_names, ph_max)
        # what the two splits return against the whole-sequence forward of this very run
        e_h_o = (o_h.float() - o_whole[:, :, lo:hi].float()).abs().max().item()
        e_h_s = (ht_h - ht_whole[:, lo:hi]).abs().max().item()
        e_s_o = (o_s.float() - o_whole[:, tsl].float()).abs().max().item()
        e_s_s = (ht_s - ht_whole).abs().max().item() if ht_s is not None else 0.0
        ms_heads, ms_seq, e_h_o, e_h_s, e_s_o, e_s_s, hk1m, hk2m = max_over_ranks(
            [ms_heads, ms_seq, e_h_o, e_h_s, e_s_o, e_s_s, statistics.mean(hk1), statistics.mean(hk2)])
        best = "head_shard" if ms_heads <= ms_seq else "seq_split"
        strong = dict(
            problem="one B=1 T=8192 H=32 sequence over %d GPUs" % world, chosen=best,
            head_shard=dict(ms_per_step=ms_heads / steps, tokens_per_s=B * T * steps / (ms_heads * 1e-3),
                            heads_per_gpu=hl, k1_us=hk1m * 1e3, k2_us=hk2m * 1e3, collectives=0,
                            max_abs_vs_one_gpu=dict(o=e_h_o, ht=e_h_s)),
            seq_split=dict(ms_per_step=ms_seq / steps, tokens_per_s=B * T * steps / (ms_seq * 1e-3),
                           tokens_per_gpu=L, exchange=plan.mode, exchange_transport=plan.exchange_kind,
                           timeline_us={n: v * 1e3 for n, v in zip(ph_names, ph_max)}, exchange_parts_us=exchange_parts,
                           sub_segments_per_rank=plan.sub,
                           collectives="2 all-to-all (NCCL) per forward" if plan.mode == "a2a" else "1 all-gather (NCCL) per forward",
                           max_abs_vs_one_gpu=dict(o=e_s_o, ht=e_s_s)),
            limiter="K2 is one serial chain of T/16 chunk steps per head: fewer heads per GPU shorten K1 only, "
                    "fewer tokens per GPU shorten every kernel but add the transform pass and the exchange")
        ms_strong = min(ms_heads, ms_seq)
        launches_strong = launches_heads if best == "head_shard" else steps * 4
        plan.close()
        del plan

    # ---- long-context sequence split (B=1 T=131072 H=16) over the ranks ----
    seq_parallel = None
    if world > 1:
        dl = make_device_inputs(43, dev, 1, SP_T, SP_H)

        def one_gpu():
            return K.kda_bt16_fwd(dl["q"], dl["k"], dl["v"], dl["g"], dl["beta"], scale=scale, initial_state=dl["h0"],
                                  output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                  use_beta_sigmoid_in_kernel=True, lower_bound=-5.0, A_log=dl["A_log"],
                                  dt_bias=dl["dt_bias"], reuse_workspace=True)
        o1, h1 = one_gpu()
        t_one = timed(one_gpu, 3) / 3
        Ll = SP_T // world
        tsl = slice(rank * Ll, (rank + 1) * Ll)
        plan = shard.SeqParallelPlan(dl["q"][:, tsl], dl["k"][:, tsl], dl["v"][:, tsl], dl["g"][:, tsl], dl["beta"][:, tsl],
                                     scale=scale, initial_state=dl["h0"], lower_bound=-5.0, A_log=dl["A_log"],
                                     dt_bias=dl["dt_bias"])
        ms_sp = timed(plan.run, steps) / steps
        tls = [[] for _ in range(5)]           # back-to-back steps behind one barrier, as above
        barrier()
        plan.run()
        for tl in tls:
            o2, h2 = plan.run(timeline=tl)
        torch.cuda.synchronize()
        ph = [(n1, statistics.mean(tl[i][1].elapsed_time(tl[i + 1][1]) for tl in tls))
              for i, (n1, _) in enumerate(tls[0][1:])]
        e_o = (o2.float() - o1[:, tsl].float()).abs().max().item()
        e_h = (h2 - h1).abs().max().item() if h2 is not None else 0.0
        res = max_over_ranks([ms_sp, t_one, e_o, e_h] + [v for _, v in ph])
        sp_names, sp_vals, sp_parts = merge_exchange_marks([n for n, _ in ph], res[4:])
        seq_parallel = dict(workload="KDA fwd B=1 T=%d H=%d, %d contiguous segments of %d tokens" % (SP_T, SP_H, world, Ll),
                            ms=res[0], tokens_per_s=SP_T / (res[0] * 1e-3), one_gpu_ms=res[1],
                            speedup_over_one_gpu=res[1] / res[0], exchange=plan.mode, exchange_transport=plan.exchange_kind, sub_segments_per_rank=plan.sub,
                            timeline_us={n: v * 1e3 for n, v in zip(sp_names, sp_vals)}, exchange_parts_us=sp_parts,
                            max_abs_vs_one_gpu=dict(o=res[2], ht=res[3]), o_bound=O_TOL, ht_bound=HT_TOL)
        plan.close()
        del plan, dl, o1, h1, o2, h2
        torch.cuda.empty_cache()

    # ---- e2e: public API, pinned host buffers, copies in the timed region ----
    # N = 1: the whole sequence.  N > 1: this rank's head shard of the one sequence (contiguous host
    # copies of its heads), so that the N ranks together move and compute the problem once.
    if world > 1:
        lo, hi = shard.head_range(H, world, rank)
        dloc = dict(q=d["q"][:, :, lo:hi], k=d["k"][:, :, lo:hi], v=d["v"][:, :, lo:hi], g=d["g"][:, :, lo:hi],
                    beta=d["beta"][:, :, lo:hi], A_log=d["A_log"][lo:hi], dt_bias=d["dt_bias"].view(-1, D)[lo:hi].reshape(-1),
                    h0=d["h0"][:, lo:hi])
    else:
        dloc = d
    host = {k: v.contiguous().cpu().pin_memory() for k, v in dloc.items()}
    o_host = torch.empty((B, T, host["q"].shape[2], D), dtype=torch.bfloat16).pin_memory()
    ht_host = torch.empty((B, host["q"].shape[2], D, D), dtype=torch.float32).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = o_host.numel() * o_host.element_size() + ht_host.numel() * ht_host.element_size()

    # Two steps are in flight: while step i computes, step i+1's inputs cross PCIe and step
    # i-1's outputs go back (three streams, two device-side input slots).  Every step still
    # copies all of its inputs from pinned host memory and all of its results back.
    cur = torch.cuda.current_stream()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    slots = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]
    ev_ready = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(count):
        for st_ in (s_in, s_cmp, s_out):
            st_.wait_stream(cur)
        for i in range(count):
            sl = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_free[sl])
                for k_, v_ in host.items():
                    slots[sl][k_].copy_(v_, non_blocking=True)
                ev_ready[sl].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_ready[sl])
                x = slots[sl]
                oo, hh = K.kda_bt16_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=scale,
                                        initial_state=x["h0"], output_final_state=True,
                                        use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                                        use_beta_sigmoid_in_kernel=True, lower_bound=-5.0, A_log=x["A_log"],
                                        dt_bias=x["dt_bias"], reuse_workspace=True)
                ev_free[sl].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[sl])
                if i >= 2:
                    s_out.wait_event(ev_out[sl])
                o_host.copy_(oo, non_blocking=True)
                ht_host.copy_(hh, non_blocking=True)
                oo.record_stream(s_out)
                hh.record_stream(s_out)
                ev_out[sl].record(s_out)
        for st_ in (s_in, s_cmp, s_out):
            cur.wait_stream(st_)

    e2e_steps(warmup)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_steps(steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else None

    # ---- parity of the timed outputs: one head against the CPU oracle, after the timed region ----
    p_head = 17 % H
    if world == 1 or p_head % world == rank:        # one rank walks the oracle (about two seconds of CPU)
        o_r, h_r = oracle_head(d, p_head)
        err_o = (o_whole[:, :, p_head:p_head + 1].float().cpu() - o_r.float()).abs().max().item()
        err_h = (ht_whole[:, p_head:p_head + 1].cpu() - h_r).abs().max().item()
    else:
        err_o = err_h = 0.0

    # ---- reduce over ranks: max device time ----
    ms_whole, e2e_ms, k1_avg, k2_avg, err_o, err_h, not_finite = max_over_ranks(
        [ms_whole, e2e_ms, statistics.mean(k1_ms), statistics.mean(k2_ms), err_o, err_h, 0.0 if finite else 1.0])

    rc = 0
    if rank == 0:
        th = B * T * H              # (token, head) units one launch processes
        chunks = B * H * (T // BT)
        kern = {}
        for name, t_ms, bytes_th, flops_chunk in (("kda_k1", k1_avg, K1_BYTES_PER_TH, K1_FLOPS_PER_CHUNK),
                                                  ("kda_k2", k2_avg, K2_BYTES_PER_TH, K2_FLOPS_PER_CHUNK)):
            gbs = bytes_th * th / (t_ms * 1e-3) / 1e9
            tf = flops_chunk * chunks / (t_ms * 1e-3) / 1e12
            kern[name] = dict(us=t_ms * 1e3, algorithmic_GBps=gbs, hbm_frac=gbs / hbm_gbs, TFLOPs=tf,
                              tensor_frac=tf / tc_tflops)
        dom = "kda_k2" if k2_avg >= k1_avg else "kda_k1"
        traffic = None
        if NCU_TRAFFIC["shape"] == (B, T, H) and NCU_TRAFFIC["record_bytes"] * chunks + 256 == K.workspace_bytes(B, T, H):
            traffic = NCU_TRAFFIC["bytes"].get(dom)
        roofline = dict(kernel=dom, bound="hbm", achieved=kern[dom]["algorithmic_GBps"], peak=hbm_gbs, unit="GB/s",
                        frac=kern[dom]["hbm_frac"], traffic=traffic,
                        traffic_unit="bytes per launch, from an earlier ncu capture of this shape (%s); null when the "
                                     "shape or the record layout differs" % NCU_TRAFFIC["source"],
                        algorithmic_bytes=(K2_BYTES_PER_TH if dom == "kda_k2" else K1_BYTES_PER_TH) * th,
                        measured_on="whole-sequence forward on one GPU (every rank runs it; max over ranks)",
                        peak_kind=peak_kind,
                        tensor_frac=kern[dom]["tensor_frac"], us_per_chunk_step=(k2_avg * 1e3) / (T // BT))
        parity = parity_record(err_o, err_h, not_finite == 0.0,
                               "head %d of the timed whole-sequence forward, all %d tokens, o and final state" % (p_head, T))
        if strong is not None:
            worst_o = max(strong["head_shard"]["max_abs_vs_one_gpu"]["o"], strong["seq_split"]["max_abs_vs_one_gpu"]["o"],
                          seq_parallel["max_abs_vs_one_gpu"]["o"])
            worst_h = max(strong["head_shard"]["max_abs_vs_one_gpu"]["ht"], strong["seq_split"]["max_abs_vs_one_gpu"]["ht"],
                          seq_parallel["max_abs_vs_one_gpu"]["ht"])
            parity["splits_vs_one_gpu"] = dict(o_max_abs=worst_o, ht_max_abs=worst_h)
            parity["ok"] = parity["ok"] and worst_o <= O_TOL and worst_h <= HT_TOL
        whole_tps = B * T * steps / (ms_whole * 1e-3)
        if world == 1:
            value, ms_step, scaling, n_launch = whole_tps, ms_whole / steps, "weak", launches
        else:
            value, ms_step, scaling, n_launch = B * T * steps / (ms_strong * 1e-3), ms_strong / steps, "strong", launches_strong
        line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world,
                    steps=steps, warmup=warmup, ms_per_step=ms_step, higher_is_better=True,
                    scaling=scaling, vs_baseline=None, dtype="bf16", data="synthetic",
                    config=make_config(world),
                    e2e=dict(value=B * T * steps / (e2e_ms * 1e-3), unit="tokens/s",
                             h2d_bytes_per_step=h2d * world, d2h_bytes_per_step=d2h * world, ms_per_step=e2e_ms / steps,
                             api="kda_ascendc_b200.kda_bt16_fwd", pipelining="2 steps in flight over 3 streams",
                             split="whole sequence" if world == 1 else "head shard: %d heads per GPU, host buffers per rank" % (H // world)),
                    gpu_launches=n_launch, roofline=roofline, kernels=kern, clocks=clocks, parity=parity,
                    latency_ms=_latency_stats([a_ + b_ for a_, b_ in zip(k1_ms, k2_ms)]))
        if world > 1:
            line["strong"] = strong
            line["seq_parallel"] = seq_parallel
            line["replicas"] = dict(value=world * whole_tps, unit="tokens/s", ms_per_step=ms_whole / steps,
                                    note="one whole sequence per GPU, no data-path collective (weak scaling)")
        else:
            line["decode"] = decode_leg(dev, hbm_gbs)
            line["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(line), flush=True)
        if not parity["ok"]:
            sys.stderr.write("bench: parity check failed: %r\n" % (parity,))
            rc = 1
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rc:
        sys.exit(rc)


def run_reference_gpu_arm(steps, warmup, n_gpus):
    """The reference's Triton `kda_bt16_fwd` (unmodified, from baseline/_ref) on cuda:0, same
    workload and metric; its in-kernel gate wants an fp32 g, so g is converted once, outside
    the timed region."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_dir = ROOT / "baseline" / "_ref"
    try:
        sys.path.insert(0, str(ref_dir))
        from kda_bt16 import kda_bt16_fwd as ref_fwd
    except Exception as e:  # noqa: BLE001
        print(json.dumps(dict(impl="reference_gpu", unavailable="reference package not importable from baseline/_ref: %r" % (e,))))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    d = make_device_inputs(42, dev)
    gf = d["g"].float()

    def fwd():
        return ref_fwd(d["q"], d["k"], d["v"], gf, d["beta"], scale=D ** -0.5, initial_state=d["h0"],
                       output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                       use_beta_sigmoid_in_kernel=True, safe_gate=True, lower_bound=-5.0, A_log=d["A_log"],
                       dt_bias=d["dt_bias"], state_v_first=True)

    for _ in range(max(warmup, 3)):
        fwd()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fwd()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    print(json.dumps(dict(impl="reference_gpu", metric=METRIC, value=B * T / (ms * 1e-3), unit="tokens/s", n_gpus=1,
                          steps=steps, warmup=max(warmup, 3), ms_per_step=ms, higher_is_better=True, dtype="bf16",
                          data="synthetic", config=dict(make_config(1), kernels="reference Triton K1+K2, g fp32"))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the e2e and CPU-baseline legs (short run for profiler captures)")
    ap.add_argument("--shape", default=None,
                    help="B,T,H of another workload for --kernels-only runs (profiler captures of other regimes); "
                         "the default and every reported line use the headline shape")
    ap.add_argument("--k2-variant", type=int, default=0,
                    help="K2 organisation for --kernels-only runs (profiler captures of a form the automatic "
                         "choice does not take, e.g. 5 = look-ahead); every reported line uses the automatic choice")
    a = ap.parse_args()
    if a.k2_variant and not a.kernels_only:
        ap.error("--k2-variant goes with --kernels-only")
    global K2_VARIANT
    K2_VARIANT = a.k2_variant
    if a.shape is not None:
        if not a.kernels_only:
            ap.error("--shape goes with --kernels-only")
        global B, T, H
        B, T, H = (int(x) for x in a.shape.split(","))
    if a.impl == "reference":
        run_reference_arm(a.steps, a.warmup, a.gpus)
    elif a.impl == "reference_gpu":
        run_reference_gpu_arm(a.steps, a.warmup, a.gpus)
    else:
        run_gpu_arm(a.steps, a.warmup, a.gpus, a.kernels_only)


if __name__ == "__main__":
    main()
