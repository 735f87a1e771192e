"""A bounded device-side wait that runs out: status word, host error, usable context afterwards.

Nothing here faults or hangs the GPU: the self-test kernel waits (with the library's own bounded
wait, limit one second) on a barrier nobody arrives on, records a status code and returns."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_times_out_and_reports_through_the_status_word():
    import kda_ascendc_b200 as K
    from kda_ascendc_b200 import _lib, api
    from oracle import kda_oracle as O

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    assert lib.kda_selftest_bounded_wait(ctypes.c_void_p(ws.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.5 < waited < 10.0, waited                      # the limit is one second; the kernel came back by itself
    assert int(ws[:4].view(torch.int32).item()) == 100      # the status code the kernel left
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        api.check_device_status(ws)
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
