"""Caller-side hook: this build behind the `chunk_kda` / `fused_recurrent_kda` call convention of
flash-linear-attention (FLA), the library the reference measures itself against and names as the
place a drop-in would plug into (README.md:510 of the reference: "wrapping as a FLA backend for
drop-in chunk_kda use"; the constraints of a comparable inference backend are listed in its
docs/KDA_ANALYSIS.md:215-229).

Two layers:

* ``chunk_kda`` / ``fused_recurrent_kda`` here take FLA's keyword set and run the B200 kernels.
  They serve exactly one configuration -- inference (no autograd), bf16, K = V = 128, HV a multiple of H,
  gate + l2-norm (+ beta sigmoid) fused in the kernel, ``safe_gate`` with a ``lower_bound`` -- and
  raise ``NotImplementedError`` with the reason for anything else.  There is no fallback.
* ``register()`` adds a backend object to FLA's per-operation registry when FLA is importable, so
  that ``fla.ops.kda.chunk_kda`` itself dispatches here for calls the verifier accepts and keeps
  its own kernels for the rest.  Off unless called; ``FLA_KDA_B200=0`` disables it afterwards.

FLA keeps the state K-first (``[N, H, K, V]``) unless ``transpose_state_layout`` (older releases:
``state_v_first``) is set.  The chunk kernels and the token recurrence read and write either layout
in place (the reference transposes on the host, src/kda_bt16/kernels.py:497-510).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import api

BACKEND_NAME = "kda_b200"


def _v_first(kwargs: dict, transpose_state_layout) -> bool:
    if transpose_state_layout is not None:
        return bool(transpose_state_layout)
    return bool(kwargs.get("state_v_first", False))


def supports(q, k, v, g, beta, *, use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
             use_beta_sigmoid_in_kernel=False, safe_gate=False, lower_bound=None, A_log=None,
             return_intermediate_states=False, cp_context=None, **_unused) -> tuple[bool, Optional[str]]:
    """(ok, reason): whether the B200 kernels serve this call."""
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta)):
        return False, "forward only: call under torch.no_grad() / inference_mode()"
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16):
        return False, "q, k, v must be bf16 CUDA tensors"
    if q.ndim != 4 or q.shape[-1] != 128 or v.shape[-1] != 128:
        return False, "K = V = 128 only"
    if v.shape[2] % q.shape[2] != 0:
        return False, "the value heads must be a multiple of the q/k heads"
    if not (use_qk_l2norm_in_kernel and use_gate_in_kernel):
        return False, "the l2-norm and the gate must be fused in the kernel"
    if not (safe_gate and lower_bound is not None and -11.0 < lower_bound < 0.0):
        return False, "safe_gate=True with lower_bound in (-11, 0) is required"
    if A_log is None:
        return False, "A_log is required"
    if return_intermediate_states or cp_context is not None:
        return False, "intermediate states and context parallelism are not supported"
    return True, None


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              cu_seqlens=None, cu_seqlens_cpu=None, safe_gate=False, lower_bound=None, disable_recompute=False,
              return_intermediate_states=False, cp_context=None, transpose_state_layout=None, **kwargs):
    """FLA's ``chunk_kda`` keyword set on the B200 kernels (chunk size 16 inside; the result does
    not depend on the chunk size).  ``A_log`` / ``dt_bias`` come as keywords, as in FLA."""
    A_log, dt_bias = kwargs.get("A_log"), kwargs.get("dt_bias")
    ok, why = supports(q, k, v, g, beta, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                       use_gate_in_kernel=use_gate_in_kernel, use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel,
                       safe_gate=safe_gate, lower_bound=lower_bound, A_log=A_log,
                       return_intermediate_states=return_intermediate_states, cp_context=cp_context)
    if not ok:
        raise NotImplementedError(f"{BACKEND_NAME}: {why}")
    if dt_bias is not None:
        dt_bias = dt_bias.reshape(-1)
    cu = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens
    return api.kda_bt16_fwd(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), beta.float().contiguous(),
                            scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                            use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                            use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel, safe_gate=True,
                            lower_bound=lower_bound, A_log=A_log, dt_bias=dt_bias,
                            state_v_first=_v_first(kwargs, transpose_state_layout), cu_seqlens=cu)


def fused_recurrent_kda(q, k, v, g, beta, A_log=None, dt_bias=None, scale=None, initial_state=None,
                        output_final_state=False, use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                        use_beta_sigmoid_in_kernel=False, lower_bound=None, cu_seqlens=None,
                        transpose_state_layout=None, **kwargs):
    """FLA's ``fused_recurrent_kda`` keyword set on the token-recurrence kernel (decode)."""
    ok, why = supports(q, k, v, g, beta, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                       use_gate_in_kernel=use_gate_in_kernel, use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel,
                       safe_gate=True, lower_bound=lower_bound, A_log=A_log)
    if ok and not use_beta_sigmoid_in_kernel:
        ok, why = False, "the recurrent step applies the beta sigmoid in the kernel"
    if ok and cu_seqlens is not None:
        ok, why = False, "the recurrent step takes a fixed-length batch"
    if not ok:
        raise NotImplementedError(f"{BACKEND_NAME}: {why}")
    return api.kda_recurrent_fwd(q, k, v, g, beta.float(), scale=scale, initial_state=initial_state,
                                 output_final_state=output_final_state, lower_bound=lower_bound, A_log=A_log,
                                 dt_bias=None if dt_bias is None else dt_bias.reshape(-1),
                                 state_v_first=_v_first(kwargs, transpose_state_layout))


def register() -> bool:
    """Add this build to FLA's ``kda`` backend registry; False when FLA (or its registry) is absent."""
    try:
        from fla.ops.backends import BaseBackend
        from fla.ops.kda.backends import kda_registry
    except Exception:  # noqa: BLE001 - FLA not installed, or a release without the registry
        return False

    class B200KDABackend(BaseBackend):
        backend_type = BACKEND_NAME
        package_name = None
        env_var = "FLA_KDA_B200"
        default_enable = True
        priority = 2

        def chunk_kda_verifier(self, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                               use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                               use_beta_sigmoid_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None,
                               safe_gate=False, lower_bound=None, disable_recompute=False,
                               return_intermediate_states=False, cp_context=None, transpose_state_layout=False,
                               **kwargs):
            return supports(q, k, v, g, beta, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                            use_gate_in_kernel=use_gate_in_kernel,
                            use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel, safe_gate=safe_gate,
                            lower_bound=lower_bound, A_log=kwargs.get("A_log"),
                            return_intermediate_states=return_intermediate_states, cp_context=cp_context)

        def chunk_kda(self, *args, **kwargs):
            return chunk_kda(*args, **kwargs)

    kda_registry.register(B200KDABackend())
    return True
