"""Cross-check against the reference's own Triton kernels run on the same GPU.

The reference package is installed (unmodified) under ``baseline/_ref`` by
``pip install --no-deps --target baseline/_ref <reference checkout>``; that folder is not
part of the history, so the test skips where it is absent.  The Triton path rounds u, v_new
and kg to bf16 (``src/kda_bt16/kernels.py:171-180,265-268,287`` of the reference), which puts
its final state ~3e-3 from the torch chunk forward; the bound on the state is therefore the
reference's own test tolerance (``tests/test_kda_bt16.py`` uses 5e-3 / 2e-2), while this
build has to sit closer to the oracle than the Triton path does.
"""
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _ref_fwd():
    if not (REF / "kda_bt16").is_dir():
        pytest.skip("reference package not installed under baseline/_ref")
    sys.path.insert(0, str(REF))
    try:
        from kda_bt16 import kda_bt16_fwd
    except Exception as e:  # noqa: BLE001
        pytest.skip("reference package not importable: %r" % (e,))
    return kda_bt16_fwd


@pytest.mark.parametrize("B,T,H", [(2, 1024, 4), (1, 1000, 3)])
def test_against_reference_triton_kernels(B, T, H):
    ref_fwd = _ref_fwd()
    import kda_ascendc_b200 as K
    from oracle import kda_oracle as O

    inp = O.make_inputs(B, T, H, seed0=42, h0_std=0.02)
    dev = torch.device("cuda", 0)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in inp.items()}
    kw = dict(scale=128 ** -0.5, initial_state=d["initial_state"], output_final_state=True, use_qk_l2norm_in_kernel=True,
              use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, safe_gate=True, lower_bound=-5.0,
              A_log=d["A_log"], dt_bias=d["dt_bias"], state_v_first=True)
    o_r, ht_r = ref_fwd(d["q"], d["k"], d["v"], d["g"].float(), d["beta"], **kw)
    o_m, ht_m = K.kda_bt16_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], **kw)
    torch.cuda.synchronize()
    assert torch.isfinite(o_r.float()).all() and torch.isfinite(o_m.float()).all()
    assert (o_r.float() - o_m.float()).abs().max().item() <= 1e-3
    assert (ht_r - ht_m).abs().max().item() <= 5e-3
    o_o, ht_o = O.run_chunk_reference(inp)
    err_m = (ht_m.cpu() - ht_o).abs().max().item()
    err_r = (ht_r.cpu() - ht_o).abs().max().item()
    assert err_m <= 2e-3 and err_m <= err_r
    assert (o_m.float().cpu() - o_o.float()).abs().max().item() <= (o_r.float().cpu() - o_o.float()).abs().max().item() + 1e-6
