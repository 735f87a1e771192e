"""CPU checks of the host layer: validation rules, the C-ABI library, layouts."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import kda_ascendc_b200 as K
from kda_ascendc_b200 import _lib, api, layout

ROOT = Path(__file__).resolve().parents[1]
D = 128


def _mk(B=1, T=32, H=2):
    q = torch.randn(B, T, H, D).bfloat16()
    k = torch.randn(B, T, H, D).bfloat16()
    v = torch.randn(B, T, H, D).bfloat16()
    g = torch.randn(B, T, H, D)
    beta = torch.randn(B, T, H)
    return q, k, v, g, beta


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "kda_b200.h").read_text()
    declared = set(re.findall(r"\b(kda_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/kda_b200.h but not exported"
    assert set(_lib.EXPORTS) <= declared


def test_peer_structs_and_argument_checks():
    """The peer-exchange entry points: ctypes mirrors (sizes pinned by static_asserts in the library) and
    the host-side argument checks (nothing is launched)."""
    assert ctypes.sizeof(_lib.KdaPeerPushArgs) == 296 and _lib.KdaPeerPushArgs.epoch.offset == 292
    assert ctypes.sizeof(_lib.KdaFoldPeerArgs) == 296 and _lib.KdaFoldPeerArgs.counter.offset == 288
    lib = _lib.load()
    a = _lib.KdaPeerPushArgs()
    assert lib.kda_peer_push(None, None) == -1
    a.world, a.epoch = 17, 1
    assert lib.kda_peer_push(ctypes.byref(a), None) == -1 and "ranks" in _lib.last_error()
    a.world, a.epoch = 2, 0
    assert lib.kda_peer_push(ctypes.byref(a), None) == -1
    a.epoch, a.src, a.counter, a.slice_floats = 1, 1024, 2048, 6
    assert lib.kda_peer_push(ctypes.byref(a), None) == -1 and "16-byte" in _lib.last_error()
    a.slice_floats = 8
    assert lib.kda_peer_push(ctypes.byref(a), None) == -1 and "dst[0]" in _lib.last_error()
    assert lib.kda_flag_wait(None, 1, 1, None, None) == -1
    assert lib.kda_flag_wait(4096, 33, 1, None, None) == -1 and lib.kda_flag_wait(4096, 1, 0, None, None) == -1
    f, pa = _lib.KdaFoldArgs(), _lib.KdaFoldPeerArgs()
    f.mq, f.n_chains, f.n_seg, f.seg_stride, f.chain_stride, f.use_q = 4096, 1, 2, 32768, 32768, 1
    assert lib.kda_state_fold_peer(ctypes.byref(f), None, None) == -1
    pa.n_wait, pa.epoch = 2, 1
    assert lib.kda_state_fold_peer(ctypes.byref(f), ctypes.byref(pa), None) == -1 and "wait_flags" in _lib.last_error()
    pa.wait_flags, pa.n_signal, pa.counter = 4096, 1, 4096
    assert lib.kda_state_fold_peer(ctypes.byref(f), ctypes.byref(pa), None) == -1 and "signal[0]" in _lib.last_error()
    f.n_seg = 17
    assert lib.kda_state_fold_peer(ctypes.byref(f), ctypes.byref(pa), None) == -1 and "16 segments" in _lib.last_error()


def test_struct_layout_matches_header():
    # 13 pointers, 4 int32, 6 x 3 int64, 2 floats, uint32, 3 int32, 2 pointers, int32 + padding
    assert ctypes.sizeof(_lib.KdaFwdArgs) == 13 * 8 + 4 * 4 + 18 * 8 + 6 * 4 + 2 * 8 + 8
    assert _lib.KdaFwdArgs.chunk_table.offset == 13 * 8 + 16 + 18 * 8 + 24
    assert _lib.KdaFwdArgs.Hq.offset == ctypes.sizeof(_lib.KdaFwdArgs) - 4
    assert _lib.KdaFwdArgs.q_stride.offset == 13 * 8 + 16
    assert _lib.KdaFwdArgs.scale.offset == 13 * 8 + 16 + 18 * 8


def test_workspace_bytes_and_version():
    assert K.workspace_bytes(1, 8192, 32) == 256 + 32 * 512 * 26112
    assert K.workspace_bytes(2, 17, 3) == 256 + 2 * 3 * 2 * 26112
    assert b"sm_100a" in _lib.load().kda_version()


def test_c_abi_rejects_bad_arguments_without_a_gpu():
    lib = _lib.load()
    a = _lib.KdaFwdArgs()
    assert lib.kda_fwd(ctypes.byref(a), None) == -1
    assert "positive" in _lib.last_error()
    a.B, a.T, a.H = 1, 16, 1
    assert lib.kda_fwd(ctypes.byref(a), None) == -1
    assert "workspace" in _lib.last_error()
    assert lib.kda_fwd(None, None) == -1


def test_reference_validation_messages():
    q, k, v, g, beta = _mk()
    with pytest.raises(ValueError, match="q must be contiguous"):
        K.kda_bt16_fwd(q.transpose(1, 2), k, v, g, beta, scale=0.0883)
    with pytest.raises(TypeError, match="k must be bfloat16"):
        K.kda_bt16_fwd(q, k.float(), v, g, beta, scale=0.0883)
    v64 = torch.randn(1, 32, 2, 64).bfloat16()
    with pytest.raises(ValueError, match="prototype targets K=V=128"):
        K.kda_bt16_fwd(q, k, v64, g, beta, scale=0.0883)
    with pytest.raises(ValueError, match="beta must be 3D"):
        K.kda_bt16_fwd(q, k, v, g, beta[..., None], scale=0.1)
    with pytest.raises(TypeError, match="beta must be float32"):
        K.kda_bt16_fwd(q, k, v, g, beta.double(), scale=0.1)
    with pytest.raises(ValueError, match="requires A_log"):
        K.kda_bt16_fwd(q, k, v, g, beta, use_gate_in_kernel=True)
    with pytest.raises(ValueError, match=r"range \(-11, 0\)"):
        K.kda_bt16_fwd(q, k, v, g, beta, use_gate_in_kernel=True, A_log=torch.zeros(2), lower_bound=-12.0)
    with pytest.raises(ValueError, match="initial_state.shape"):
        K.kda_bt16_fwd(q, k, v, g, beta, initial_state=torch.zeros(1, 2, 128, 64))
    with pytest.raises(TypeError, match="initial_state must be float32"):
        K.kda_bt16_fwd(q, k, v, g, beta, initial_state=torch.zeros(1, 2, 128, 128, dtype=torch.float64))
    with pytest.raises(ValueError, match=r"dt_bias.shape"):
        K.kda_bt16_fwd(q, k, v, g, beta, use_gate_in_kernel=True, A_log=torch.zeros(2), dt_bias=torch.zeros(2, 128))


def test_no_cpu_fallback():
    q, k, v, g, beta = _mk()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        K.kda_bt16_fwd(q, k, v, g, beta, use_gate_in_kernel=True, use_qk_l2norm_in_kernel=True,
                       use_beta_sigmoid_in_kernel=True, A_log=torch.zeros(2))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        K.kda_bt16_fwd_ascendc(q, k, v, g, beta, A_log=torch.zeros(2))


def test_second_api_input_rules():
    q, k, v, g, beta = _mk(T=24)
    with pytest.raises(ValueError, match="T>=16"):
        K.kda_bt16_fwd_ascendc(q, k, v, g, beta, A_log=torch.zeros(2))
    q, k, v, g, beta = _mk()
    with pytest.raises(ValueError, match="bias must be FP32"):
        K.kda_bt16_fwd_ascendc(q, k, v, g, beta, A_log=torch.zeros(2), bias=torch.zeros(2 * 128))
    with pytest.raises(ValueError, match="unsupported k2_mode"):
        K.kda_bt16_fwd_ascendc(q, k, v, g, beta, A_log=torch.zeros(2), k2_mode="d12")


def test_pack_unpack_tokens_roundtrip():
    x = torch.randn(2, 48, 3, D)
    p = K.pack_tokens(x)
    assert p.shape == (2 * 3 * 3, 16, D)
    # chunk-major order: c = (b*H + h)*NT + n
    assert torch.equal(p[(1 * 3 + 2) * 3 + 1], x[1, 16:32, 2])
    assert torch.equal(K.unpack_tokens(p, 2, 48, 3), x)
    with pytest.raises(ValueError):
        K.pack_tokens(torch.randn(1, 17, 1, D))


def test_record_index_maps_are_permutations():
    sw = layout._swizzle_index("cpu")
    assert sorted(sw.tolist()) == list(range(16 * 128))
    ui = layout._u_index("cpu")
    assert sorted(ui.tolist()) == list(range(16 * 128))
    # ldmatrix reads 8 rows at one 16-byte column unit: all eight must hit different units
    units = sw.view(16, 128)[:8, 0] % 128 // 8
    assert len(set(units.tolist())) == 8


def test_varlen_tables_host_helper():
    """kda_varlen_fill_tables is host code: chunk and sequence tables from cu_seqlens."""
    import ctypes
    lib = _lib.load()
    cu = (ctypes.c_int32 * 4)(0, 17, 33, 34)
    n = lib.kda_varlen_fill_tables(cu, 3, 2, None, None)
    assert n == 2 + 1 + 1
    ct = (ctypes.c_int32 * (4 * n))()
    st = (ctypes.c_int32 * 12)()
    assert lib.kda_varlen_fill_tables(cu, 3, 2, ct, st) == n
    # chunk: first token, valid tokens, first record, chunks of its sequence (H = 2 records per chunk)
    assert list(ct) == [0, 16, 0, 2, 16, 1, 1, 2, 17, 16, 4, 1, 33, 1, 6, 1]
    # sequence: first token, chunks, first record, length
    assert list(st) == [0, 2, 0, 17, 17, 1, 4, 16, 33, 1, 6, 1]
    bad = (ctypes.c_int32 * 3)(0, 5, 5)
    assert lib.kda_varlen_fill_tables(bad, 2, 2, None, None) == -1
    assert "empty" in _lib.last_error()


def test_k2_choice_table():
    """Which organisation of K2 the library picks (host logic only; 148 SMs given explicitly)."""
    lib = _lib.load()

    def choice(B, T, H, state_only=0, variant=0, vsplit=0, n_seqs=0, n_chunks=0):
        a = _lib.KdaFwdArgs()
        a.B, a.T, a.H, a.k2_variant, a.k2_vsplit, a.n_seqs, a.n_chunks = B, T, H, variant, vsplit, n_seqs, n_chunks
        var, vs = ctypes.c_int32(-1), ctypes.c_int32(-1)
        assert lib.kda_fwd_k2_choice(ctypes.byref(a), state_only, 148, ctypes.byref(var), ctypes.byref(vs)) == 0
        return var.value, vs.value

    N8, M16, TC = 1, 3, 4
    assert choice(1, 8192, 32) == (N8, 4)            # the headline shape: 32 chains, one warp per SM sub-partition
    assert choice(1, 8192, 4) == (N8, 16)            # a handful of chains: sixteen CTAs per chain
    assert choice(1, 8192, 16) == (N8, 8)
    assert choice(1, 8192, 64) == (M16, 2)           # more than 37 chains, at most half as many as SMs
    assert choice(1, 8192, 74) == (M16, 2) and choice(1, 8192, 75) == (TC, 1)
    assert choice(1, 8192, 96) == (TC, 1)            # two CTAs per chain no longer fit one per SM
    assert choice(1, 256, 96) == (M16, 2)            # ... but only for long chains
    assert choice(2, 4096, 16) == (N8, 4)
    assert choice(1, 4096, 37) == (N8, 4) and choice(1, 4096, 38) == (M16, 2)
    assert choice(8, 2048, 32) == (TC, 1)            # more chains than SMs, long enough chains
    assert choice(8, 48, 32) == (M16, 2)             # three chunks per chain: set-up not amortised
    assert choice(8, 64, 32) == (TC, 1)
    assert choice(8, 2048, 32, state_only=1) == (M16, 2)   # no state-only form in tensor memory
    assert choice(8, 2048, 32, vsplit=2) == (M16, 2)       # an explicit split keeps the mma.sync forms
    assert choice(8, 2048, 32, variant=M16) == (M16, 2)
    assert choice(1, 8192, 32, variant=TC) == (TC, 1)
    # packed sequences: chains = sequences x heads, steps = the mean chunk count
    assert choice(1, 4096, 32, n_seqs=8, n_chunks=8 * 32) == (TC, 1)
    assert choice(1, 4096, 32, n_seqs=8, n_chunks=8 * 2) == (M16, 2)
    assert choice(1, 4096, 32, n_seqs=2, n_chunks=256) == (M16, 2)
    a = _lib.KdaFwdArgs()
    a.B, a.T, a.H, a.k2_variant = 1, 16, 1, 9
    var, vs = ctypes.c_int32(), ctypes.c_int32()
    assert lib.kda_fwd_k2_choice(ctypes.byref(a), 0, 148, ctypes.byref(var), ctypes.byref(vs)) != 0
    assert "k2_variant" in _lib.last_error()


def test_static_scratch_argument_checks_are_host_only():
    """kda_fwd_static_scratch sizes its request in 64 bits and refuses before touching CUDA."""
    lib = _lib.load()
    a = _lib.KdaFwdArgs()
    a.B, a.T, a.H = 1, 16, 1
    a.n_seqs, a.n_chunks = 1, 2 ** 27            # 16 * n_chunks would wrap a 32-bit T
    assert lib.kda_fwd_static_scratch(ctypes.byref(a), None) == -1
    assert "records" in _lib.last_error() and "use kda_fwd" in _lib.last_error()
    a.n_chunks = 0
    assert lib.kda_fwd_static_scratch(ctypes.byref(a), None) == -1
    assert "n_chunks" in _lib.last_error()
    a.n_seqs, a.B, a.T, a.H = 0, 2 ** 30, 2 ** 30, 2 ** 30
    assert lib.kda_fwd_static_scratch(ctypes.byref(a), None) == -1
    assert "use kda_fwd" in _lib.last_error()
    a.n_seqs = -1
    assert lib.kda_fwd_static_scratch(ctypes.byref(a), None) == -1
    assert lib.kda_fwd_static_scratch_status(None, None) == -1
    assert "status_out" in _lib.last_error()


def test_expanded_views_are_refused():
    """A zero stride on a dimension larger than one (q.expand(B, ...)) must not be read as dense."""
    lib = _lib.load()
    a = _lib.KdaFwdArgs()
    a.B, a.T, a.H, a.g_dtype = 2, 16, 1, _lib.KDA_G_BF16
    fake = ctypes.c_void_p(256 * 4096)            # never dereferenced: the checks are host-only
    a.q = a.k = a.v = a.g = a.beta = a.workspace = fake
    for f in ("q_stride", "k_stride", "v_stride", "g_stride"):
        getattr(a, f)[0], getattr(a, f)[1], getattr(a, f)[2] = 16 * 128, 128, 128
    a.q_stride[0] = 0                              # batch-expanded q
    assert lib.kda_fwd_k1(ctypes.byref(a), None) == -1
    assert "expanded" in _lib.last_error() and "q has" in _lib.last_error()
