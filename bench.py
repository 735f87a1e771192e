"""Benchmark of the KDA chunked forward (BT=16) -- one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]

A step is one whole forward (K1 + K2) over one batch of seeded synthetic inputs of the
headline workload: B=1, T=8192, H=32, K=V=128, bf16 (q, k, v, g_raw ~ N(0,1) bf16, beta
logits ~ N(0,1), A_log = log U(1,16), dt_bias ~ U(-0.1,0.1), lower_bound -5, initial
state ~ N(0, 0.02)).  With N > 1 (one process per GPU under torchrun) every rank runs
that workload on its own sequence -- work is sharded by (batch, head) with no
communication, so the scaling is weak and `value` is the tokens of all ranks over the
max-over-ranks device time.

Keys: `value` -- tokens/s with inputs resident in HBM (CUDA events around K steps);
`e2e` -- tokens/s through the public Python API with pinned host buffers, H2D and D2H
copies inside the timed region; `roofline` -- the dominant kernel against the measured
HBM copy bandwidth; `kernels` -- both kernels; `cpu_baseline` -- the CPU port of the
reference's torch chunk forward on a bounded sample; `clocks` -- nvidia-smi samples
taken during the timed region.

`--impl reference` times the CPU port of the reference's torch forward
(oracle/kda_oracle.py, looped exactly like the reference) on the host cores, one
process per core over (head, token-slice) units, and prints the same line with
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
WORKLOAD = "KDA fwd B=1 T=8192 H=32 K=V=128 BT=16 bf16 (headline benchmark shape) per GPU"
METRIC = "KDA fwd tokens/s at B1 T8192 H32 K=V=128 bf16"
# algorithmic bytes / flops per (token, head) of the two-kernel contract of the reference
K1_BYTES_PER_TH = 2084.0     # reads q,k,v,g bf16 + beta; writes w,u bf16, g fp32, Aqk bf16
K2_BYTES_PER_TH = 1856.0     # reads w,u,q,k,g,Aqk,g_last; writes o
K1_FLOPS_PER_CHUNK = 262144.0
K2_FLOPS_PER_CHUNK = 1638400.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch on this workload, from the ncu
# capture summarised in profiles/kda_k1_k2_B1_T8192_H32.md (bytes per launch)
NCU_TRAFFIC_BYTES = {"kda_k1": 641.80e6, "kda_k2": 488.68e6}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


# ----------------------------------------------------------------------------
# CPU port timing (cpu_baseline leg and the reference arm)
# ----------------------------------------------------------------------------
def _cpu_unit(args):
    """One (head, token-slice) unit of the workload through the looped CPU port."""
    head, t_len, seed = args
    import torch as _t
    _t.set_num_threads(1)
    from oracle import kda_oracle as O
    inp = O.make_inputs(1, t_len, 1, seed0=seed, head_offset=head, h0_std=0.02)
    t0 = time.perf_counter()
    O.run_chunk_reference(inp, loop_heads=True)
    return time.perf_counter() - t0


def cpu_baseline_sample(heads=16, t_len=8192):
    """Single-thread timing of `heads` heads x `t_len` tokens of the workload."""
    torch.set_num_threads(1)
    secs = sum(_cpu_unit((h, t_len, 42)) for h in range(heads))
    units_full = H * (T // BT)
    units = heads * (t_len // BT)
    full_secs = secs * units_full / units
    return dict(value=B * T / full_secs, unit="tokens/s", cores=1, kind="port",
                sample="%d heads x %d tokens of the workload (%d of %d chunk tiles), looped torch port, "
                       "1 thread, %.1f s, extrapolated linearly" % (heads, t_len, units, units_full, secs))


def run_reference_arm(steps, warmup, n_gpus):
    import multiprocessing as mp
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ncpu = os.cpu_count() or 1
    workers = max(1, min(ncpu, 64))
    t_len = 512
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(workers) as pool:
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            pool.map(_cpu_unit, [(w % H, t_len, 42) for w in range(workers)], chunksize=1)
            dt = time.perf_counter() - t0
            if it >= warmup:
                times.append(dt)
    step_s = statistics.mean(times)
    units_per_step = workers * (t_len // BT)
    units_full = B * H * (T // BT) * n_gpus
    full_secs = step_s * units_full / units_per_step
    value = n_gpus * B * T / full_secs
    sample = ("each step: %d processes x (1 head x %d tokens) = %d of %d chunk tiles of the workload, "
              "looped torch port, extrapolated linearly" % (workers, t_len, units_per_step, units_full))
    line = dict(impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=n_gpus, steps=steps,
                warmup=warmup, ms_per_step=step_s * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="fp32 (bf16 q/k rounding)", data="synthetic",
                config=dict(workload=WORKLOAD, device="host CPU", host_cores=ncpu),
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


def make_device_inputs(rank: int, device):
    """Seeded inputs of the workload, generated on the device (per-rank seed)."""
    g = torch.Generator(device=device).manual_seed(42 + 1000 * rank)
    rn = lambda *s: torch.randn(*s, device=device, generator=g)
    d = dict(q=rn(B, T, H, D).bfloat16(), k=rn(B, T, H, D).bfloat16(), v=rn(B, T, H, D).bfloat16(),
             g=rn(B, T, H, D).bfloat16(), beta=rn(B, T, H),
             A_log=torch.log(1.0 + 15.0 * torch.rand(H, device=device, generator=g)),
             dt_bias=torch.rand(H * D, device=device, generator=g) * 0.2 - 0.1,
             h0=rn(B, H, D, D) * 0.02)
    return d


def run_gpu_arm(steps, warmup, n_gpus, kernels_only=False):
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import _lib, api

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

    d = make_device_inputs(rank, dev)
    scale = D ** -0.5
    ws = torch.empty(K.workspace_bytes(B, T, H), dtype=torch.uint8, device=dev)
    o = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=dev)
    ht = torch.empty(B, H, D, D, dtype=torch.float32, device=dev)
    args = api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale, lower_bound=-5.0,
                         A_log=d["A_log"], dt_bias=d["dt_bias"], h0=d["h0"], o=o, ht=ht, workspace=ws, flags=7)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def fwd():
        rc = lib.kda_fwd(ctypes.byref(args), stream)
        if rc != 0:
            raise RuntimeError(_lib.last_error())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: inputs resident in HBM ------------------------------------
    for _ in range(max(warmup, 3)):
        fwd()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fwd()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = steps * lib.kda_last_launch_count()

    # ---- per-kernel durations (same inputs, events on the launching stream) ----
    k1_ms, k2_ms = [], []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for _ in range(steps):
        ev[0].record()
        assert lib.kda_fwd_k1(ctypes.byref(args), stream) == 0, _lib.last_error()
        ev[1].record()
        assert lib.kda_fwd_k2(ctypes.byref(args), stream) == 0, _lib.last_error()
        ev[2].record()
        torch.cuda.synchronize()
        k1_ms.append(ev[0].elapsed_time(ev[1]))
        k2_ms.append(ev[1].elapsed_time(ev[2]))
    status = api.check_device_status(ws)
    assert status == 0, "device status %d" % status
    assert bool(torch.isfinite(o.float()).all()) and bool(torch.isfinite(ht).all()), "non-finite output"

    # ---- e2e: public API, pinned host buffers, copies in the timed region ----
    if kernels_only:
        if rank == 0:
            print(json.dumps(dict(kernels_only=True, ms_per_step=ms / steps, k1_us=statistics.mean(k1_ms) * 1e3,
                                  k2_us=statistics.mean(k2_ms) * 1e3)), flush=True)
            if sampler is not None:
                sampler.stop()
        return
    host = {k: v.cpu().pin_memory() for k, v in d.items()}
    o_host = torch.empty(o.shape, dtype=o.dtype).pin_memory()
    ht_host = torch.empty(ht.shape, dtype=ht.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = o_host.numel() * o_host.element_size() + ht_host.numel() * ht_host.element_size()

    # Two steps are in flight: while step i computes, step i+1's inputs cross PCIe and step
    # i-1's outputs go back (three streams, two device-side input slots).  Every step still
    # copies all of its inputs from pinned host memory and all of its results back.
    cur = torch.cuda.current_stream()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    slots = [{k: torch.empty_like(v) for k, v in d.items()} for _ in range(2)]
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

    e2e_steps(max(warmup, 3))
    barrier()
    e0.record()
    e2e_steps(steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else None

    # ---- reduce over ranks: max device time -------------------------------
    if dist is not None:
        t = torch.tensor([ms, e2e_ms, statistics.mean(k1_ms), statistics.mean(k2_ms)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, k1_avg, k2_avg = (float(x) for x in t.tolist())
    else:
        k1_avg, k2_avg = statistics.mean(k1_ms), statistics.mean(k2_ms)

    if rank == 0:
        tokens_per_step = world * B * T
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
        traffic = NCU_TRAFFIC_BYTES.get(dom)
        roofline = dict(kernel=dom, bound="hbm", achieved=kern[dom]["algorithmic_GBps"], peak=hbm_gbs, unit="GB/s",
                        frac=kern[dom]["hbm_frac"], traffic=traffic, traffic_unit="bytes per launch (ncu)",
                        algorithmic_bytes=(K2_BYTES_PER_TH if dom == "kda_k2" else K1_BYTES_PER_TH) * th,
                        peak_kind=peak_kind,
                        tensor_frac=kern[dom]["tensor_frac"], us_per_chunk_step=(k2_avg * 1e3) / (T // BT))
        line = dict(metric=METRIC, value=tokens_per_step * steps / (ms * 1e-3), unit="tokens/s", n_gpus=world,
                    steps=steps, warmup=max(warmup, 3), ms_per_step=ms / steps, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                    config=dict(workload=WORKLOAD, sharding="one sequence per GPU, no communication",
                                l2="inputs + K1->K2 records = 0.7 GB per step, larger than the 126 MB L2",
                                global_batch=world * B, seq_len=T, heads=H),
                    e2e=dict(value=tokens_per_step * steps / (e2e_ms * 1e-3), unit="tokens/s",
                             h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=e2e_ms / steps,
                             api="kda_ascendc_b200.kda_bt16_fwd", pipelining="2 steps in flight over 3 streams"),
                    gpu_launches=launches, roofline=roofline, kernels=kern, clocks=clocks,
                    latency_ms=_latency_stats([a_ + b_ for a_, b_ in zip(k1_ms, k2_ms)]))
        if world == 1:
            line["decode"] = decode_leg(dev, hbm_gbs)
            line["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


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
    d = make_device_inputs(0, dev)
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
                          data="synthetic", config=dict(workload=WORKLOAD, kernels="reference Triton K1+K2, g fp32"))))


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
    a = ap.parse_args()
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
