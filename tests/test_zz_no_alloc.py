"""The allocation-free entry point, kda_fwd_static_scratch, against kda_fwd.

Some callers of this library cannot get device memory at the time of the call (an inference
server whose own pool already owns the GPU's free memory, a plugin without an allocator hook),
so they cannot provide the K1 -> K2 workspace kda_fwd asks for.  kda_fwd_static_scratch takes that
scratch from a fixed 32 MiB array inside the library.  This file checks, through the C ABI, that
it gives exactly what kda_fwd gives -- twice in a row, the second time on a smaller problem so
that records of the first call are still lying in the shared array -- that it refuses problems
that do not fit, and that no torch allocation happens during the calls.  It is named so that
pytest collects it after every other test file.
"""
import ctypes

import pytest
import torch

import kda_ascendc_b200 as K
from conftest import to_device
from kda_ascendc_b200 import _lib, api
from oracle import kda_oracle as O

pytestmark = pytest.mark.gpu


def _args(d, o, ht, ws):
    return api.make_args(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=d["scale"], lower_bound=d["lower_bound"],
                         A_log=d["A_log"], dt_bias=d["dt_bias"], h0=d["initial_state"], o=o, ht=ht, workspace=ws,
                         flags=7)


def _both_ways(lib, d, stream):
    B, T, H, _ = d["q"].shape
    dev = d["q"].device
    ws = torch.empty(K.workspace_bytes(B, T, H), dtype=torch.uint8, device=dev)
    o_ref = torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=dev)
    h_ref = torch.empty(B, H, 128, 128, dtype=torch.float32, device=dev)
    o_new = torch.full_like(o_ref, float("nan"))
    h_new = torch.full_like(h_ref, float("nan"))
    a_ref = _args(d, o_ref, h_ref, ws)
    assert lib.kda_fwd(ctypes.byref(a_ref), stream) == 0, _lib.last_error()
    a_new = _args(d, o_new, h_new, None)            # no workspace from the caller
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    rc = lib.kda_fwd_static_scratch(ctypes.byref(a_new), stream)
    assert rc == 0, _lib.last_error()
    assert torch.cuda.memory_allocated(dev) == before
    torch.cuda.synchronize()
    return (o_ref, h_ref), (o_new, h_new)


def test_static_scratch_matches_kda_fwd_on_two_calls_in_a_row(cuda_device):
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    first = to_device(O.make_inputs(1, 1040, 4, seed0=51, h0_std=0.02), cuda_device)       # 260 chunks, 6.8 MB
    second = to_device(O.make_inputs(2, 100, 2, seed0=52, regime="carry", h0_std=0.1), cuda_device)   # 28 chunks
    for d in (first, second):
        assert K.workspace_bytes(*d["q"].shape[:3]) <= _lib.STATIC_SCRATCH_BYTES
        (o_ref, h_ref), (o_new, h_new) = _both_ways(lib, d, stream)
        # same kernels on the same inputs: the tolerance of the parity tests is met with zero error
        assert torch.equal(o_new, o_ref)
        assert torch.equal(h_new, h_ref)
        # no bounded device-side wait gave up: the status word inside the library's array is clear
        status = ctypes.c_int32(-1)
        assert lib.kda_fwd_static_scratch_status(stream, ctypes.byref(status)) == 0, _lib.last_error()
        assert status.value == 0
    # and the result is right, not just equal
    inp = O.make_inputs(2, 100, 2, seed0=52, regime="carry", h0_std=0.1)
    o_r, h_r = O.run_chunk_reference(inp)
    assert (o_new.float().cpu() - o_r.float()).abs().max().item() < 2e-2 * o_r.float().abs().max().item()
    assert (h_new.cpu() - h_r).abs().max().item() <= 2e-3


def test_static_scratch_refuses_what_does_not_fit(cuda_device):
    lib = _lib.load()
    a = _lib.KdaFwdArgs()
    a.B, a.T, a.H = 1, 8192, 32                     # 408 MiB of records: far beyond the array
    assert K.workspace_bytes(1, 8192, 32) > _lib.STATIC_SCRATCH_BYTES
    assert lib.kda_fwd_static_scratch(ctypes.byref(a), None) == -1
    msg = _lib.last_error()
    assert "kda_fwd_static_scratch" in msg and "33554432" in msg and "use kda_fwd" in msg
    assert lib.kda_fwd_static_scratch(None, None) == -1
