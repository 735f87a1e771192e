"""B200-native KDA (Kimi Delta Attention) chunked forward, chunk size 16, K = V = 128.

Drop-in for the forward path of the reference project: ``kda_bt16_fwd`` /
``kda_bt16_debug`` (its Triton package) and ``kda_bt16_fwd_ascendc`` (its second
backend).  The device code is hand-written sm_100a CUDA (K1, three organisations of K2, a
token-recurrence step) behind a C ABI
(``include/kda_b200.h``); there is no other backend and no CPU fallback.
"""
from .api import (CHUNK, PERSISTENT_LOOP, ForwardPlan, RecurrentPlan, get_last_profile, kda_bt16_debug, kda_bt16_fwd,
                  kda_bt16_fwd_ascendc, kda_recurrent_fwd, workspace_bytes)
from .layout import pack_tokens, unpack_tokens

__all__ = [
    "CHUNK", "PERSISTENT_LOOP", "ForwardPlan", "RecurrentPlan", "get_last_profile", "kda_bt16_debug", "kda_bt16_fwd",
    "kda_bt16_fwd_ascendc", "kda_recurrent_fwd", "pack_tokens", "unpack_tokens", "workspace_bytes",
]
__version__ = "0.1.0"
