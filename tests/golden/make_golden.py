"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own torch chunk forward, ``torch_reference_kda_bt16``
(``tests/test_torch_reference.py:23-213`` of the reference project), feeds it inputs
built with the recipes of the reference's tests (seeds and generators cited per case
below) and stores inputs and outputs as ``<case>.pt``.  The fixtures pin the CPU oracle
of this repository (``tests/test_oracle.py``) and are a second target for the GPU
parity tests.  q, k, v are rounded to bf16 before the call, which is how the kernels
receive them (the reference's tests do the same cast for the device path).
"""
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
D = 128


def _randn_inputs(seed, B, T, H, with_state=False, a_log="randn", bias="randn"):
    # recipe of tests/test_torch_reference.py:234-243 and :407-419
    torch.manual_seed(seed)
    q = torch.randn(B, T, H, D)
    k = torch.randn(B, T, H, D)
    v = torch.randn(B, T, H, D)
    g = torch.randn(B, T, H, D)
    beta = torch.randn(B, T, H)
    A_log = torch.randn(H) if a_log == "randn" else torch.zeros(H)
    dt_bias = torch.randn(H * D) * 0.1 if bias == "randn" else None
    h0 = torch.randn(B, H, D, D) if with_state else None
    return dict(q=q.bfloat16(), k=k.bfloat16(), v=v.bfloat16(), g=g, beta=beta, A_log=A_log, dt_bias=dt_bias,
                initial_state=h0, scale=D ** -0.5, lower_bound=-5.0, state_v_first=True)


def cases():
    out = {}
    for T, H in ((16, 1), (17, 1), (32, 2), (33, 2)):       # tests/test_torch_reference.py:216-221
        out[f"ref_T{T}_H{H}"] = _randn_inputs(42, 1, T, H)
    for T in (16, 17):                                       # :390-476, both state layouts
        for vfirst in (True, False):
            c = _randn_inputs(456 + T, 1, T, 1, with_state=True)
            c["state_v_first"] = vfirst
            out[f"state_T{T}_{'vfirst' if vfirst else 'kfirst'}"] = c
    out["simple_gate"] = _randn_inputs(123, 1, 32, 2, a_log="zeros", bias=None)   # :293-351
    for lb in (-8.0, -10.0):                                 # tests/test_kda_bt16.py:128-171 (T shortened)
        c = _randn_inputs(42, 1, 48, 2, a_log="zeros", bias=None)
        c["g"] = torch.full_like(c["g"], 20.0)
        c["dt_bias"] = torch.zeros(2 * D)
        c["scale"] = 0.1
        c["lower_bound"] = lb
        out[f"saturated_lb{int(-lb)}"] = c
    # small-magnitude, long-memory inputs of tests/test_chunk_shape_matrix.py:53-63
    torch.manual_seed(240920 + 1000 * 1 + 10 * 2 + 2)
    b, t, h = 1, 32, 2
    out["small_magnitude"] = dict(
        q=(torch.randn(b, t, h, D) * 0.2).bfloat16(), k=(torch.randn(b, t, h, D) * 0.2).bfloat16(),
        v=(torch.randn(b, t, h, D) * 0.1).bfloat16(), g=torch.randn(b, t, h, D) * 0.1, beta=torch.randn(b, t, h),
        A_log=torch.linspace(-1.0, 0.2, h), dt_bias=(torch.randn(h, D) * 0.03).reshape(-1),
        initial_state=torch.randn(b, h, D, D) * 0.01, scale=D ** -0.5, lower_bound=-1.0, state_v_first=True)
    return out


def main(ref_root: str):
    sys.path[:0] = [str(Path(ref_root) / "src"), str(Path(ref_root) / "tests")]
    from test_torch_reference import torch_reference_kda_bt16
    for name, c in cases().items():
        o, ht = torch_reference_kda_bt16(c["q"], c["k"], c["v"], c["g"], c["beta"], c["scale"],
                                         lower_bound=c["lower_bound"], A_log=c["A_log"], dt_bias=c["dt_bias"],
                                         initial_state=c["initial_state"], state_v_first=c["state_v_first"])
        c = dict(c, o=o, ht=ht)
        torch.save(c, HERE / f"{name}.pt")
        print(name, tuple(o.shape), float(o.float().abs().max()), float(ht.abs().max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
