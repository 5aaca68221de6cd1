"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header declares,
and its host-side logic (list length, workspace sizes, argument validation) behaves."""
import ctypes as C
import os
import re

import pytest

from oracle import socket_oracle as orc
from socket_b200 import _lib
from socket_b200.config import PRESETS, SocketConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "socket_b200.h")).read()
    return sorted(set(re.findall(r"SK_API[^;(]*?\b(sk_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = _declared()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names
    assert lib.sk_abi_version() == 1


def test_params_struct_matches_header_fields():
    text = open(os.path.join(ROOT, "include", "socket_b200.h")).read()
    body = text[text.index("typedef struct sk_decode_params"):text.index("} sk_decode_params;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for name in decl.split(","):
            fields.append(re.findall(r"(\w+)\s*$", name.strip())[0])
    assert fields == [f[0] for f in _lib.DecodeParams._fields_]


@pytest.mark.parametrize("T,sink,window,M", [(4096, 16, 64, 256), (32768, 64, 128, 1024),
                                             (17, 20, 5, 32), (64, 0, 0, 8), (1, 0, 0, 0),
                                             (100, 2, 4, 40), (10, 4, 8, 3), (131072, 64, 256, 2048)])
def test_list_len_matches_reference_rule(T, sink, window, M):
    lib = _lib.lib()
    expect = orc.base_indices(T, sink, window).shape[0] + min(M, T)
    assert lib.sk_list_len(T, sink, window, M) == expect
    cfg = SocketConfig(context=T, sink=sink, window=window, topk=M)
    assert cfg.ktot == expect


def test_algorithmic_bytes_of_presets():
    assert PRESETS["c2"].algorithmic_bytes() == 8388608 + 19922944
    assert PRESETS["c3"].algorithmic_bytes() == 134217728 + 155189248
    assert PRESETS["c3"].shard_kv_heads(8).algorithmic_bytes() == 36175872
    assert PRESETS["c1"].algorithmic_bytes() == 1048576 + 11010048


def test_argument_errors_are_reported_without_a_gpu():
    lib = _lib.lib()
    rc = lib.sk_score(None, None, None, None, 1, 32, 8, 32, 256, 128, None, 128, None, 128, None, None)
    assert rc == -1 and b"null pointer" in lib.sk_last_error()
    rc = lib.sk_score(None, None, None, None, 1, 30, 8, 32, 256, 128, None, 128, None, 128, None, None)
    assert rc == -1 and b"multiple" in lib.sk_last_error()
    rc = lib.sk_hash_keys(1, 0, 128, 1, 0, 4, 128, 32, 9, 1, 1, 32, None)
    assert rc == -1 and b"does not fit" in lib.sk_last_error()
    rc = lib.sk_select_list(1, 100, None, 4, 100, None, 10, 2, 2, 0, 1, 5, 1, None, None)
    assert rc == -1 and b"list_row_stride" in lib.sk_last_error()
    assert lib.sk_status_string(-4) == b"workspace too small"
    with pytest.raises(_lib.SocketError):
        _lib.check(rc, "sk_select_list")


def test_workspace_queries():
    lib = _lib.lib()
    a = lib.sk_sparse_decode_workspace_bytes(1, 32, 128, 1216)
    b = lib.sk_sparse_decode_workspace_bytes(4, 32, 128, 2368)
    assert a > 0 and b > 0 and a % 256 == 0 and b % 256 == 0
    s = lib.sk_decode_step_workspace_bytes(1, 32, 8, 128, 32, 256, 33792, 1024, 64, 128)
    assert s >= a + 32 * 33792 * 4 + 32 * 32 * 256 * 4
    assert lib.sk_lut_head_tile(4) == 4 and lib.sk_lut_head_tile(8) == 4
    assert lib.sk_lut_head_tile(2) == 2 and lib.sk_lut_head_tile(1) == 1 and lib.sk_lut_head_tile(3) == 1


def test_operators_refuse_cpu_tensors():
    import torch
    from socket_b200 import ops
    from socket_b200.kernels.sparse import build_sparse_list_decode, sparse_attention_fwd
    q = torch.zeros(1, 4, 128)
    with pytest.raises(AssertionError):
        sparse_attention_fwd(q, torch.zeros(1, 1, 8, 128), torch.zeros(1, 1, 8, 128),
                             torch.zeros(1, 4, 2, dtype=torch.int32), torch.zeros(1, 4, dtype=torch.int32))
    with pytest.raises(AssertionError):
        build_sparse_list_decode(torch.zeros(1, 4, 32, 256), torch.zeros(1, 4, 32, 8, dtype=torch.int16),
                                 torch.zeros(1, 4, 8, dtype=torch.float16),
                                 torch.ones(1, 4, 8, dtype=torch.bool), 1, 1, 2)
    with pytest.raises(RuntimeError):
        ops.hash_keys(torch.zeros(4, 128), torch.zeros(32, 8, 128))
    with pytest.raises(RuntimeError, match="must be CUDA"):
        ops.soft_hash_collision(torch.zeros(1, 1, 1, 2, 4), torch.zeros(1, 1, 2, 3, dtype=torch.int16),
                                torch.ones(1, 1, 1, 3, dtype=torch.bool), torch.zeros(1, 1, 1, 3))


def _step_params(**over):
    """A parameter block that passes every host check up to the launch (fake, aligned addresses;
    nothing is ever dereferenced on the host)."""
    p = _lib.DecodeParams()
    a = 1 << 20
    for name in ("q", "k_new", "v_new", "input_pos", "planes", "protos_T", "k_cache", "v_cache", "codes",
                 "v_norm", "prefill_len", "out", "workspace", "status"):
        setattr(p, name, a)
        a += 1 << 20
    p.temperature = 1.0
    p.q_dtype = p.kv_dtype = p.plane_dtype = _lib.SK_BF16
    p.B, p.H, p.Hkv, p.D, p.L, p.P, p.R = 1, 32, 8, 128, 32, 8, 256
    p.Tcap = p.T_max = 8192
    p.M, p.sink, p.window, p.select_path = 256, 16, 64, 0
    p.workspace_bytes = 1 << 40
    for k, v in over.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("field", ["q", "k_new", "v_new", "k_cache", "v_cache", "codes", "out", "planes"])
def test_decode_step_rejects_misaligned_pointers_on_the_host(field):
    lib = _lib.lib()
    p = _step_params()
    setattr(p, field, getattr(p, field) + 2)          # element-aligned only, like an odd storage offset
    rc = lib.sk_decode_step(C.byref(p), None)
    assert rc == -3, lib.sk_last_error()
    assert field.encode() in lib.sk_last_error() and b"aligned" in lib.sk_last_error()
    p = _step_params()
    p.v_norm += 1
    assert lib.sk_decode_step(C.byref(p), None) == -3 and b"v_norm" in lib.sk_last_error()


def test_decode_step_refuses_unsupported_shapes_before_touching_the_cache():
    lib = _lib.lib()
    # refused on the host before the first launch, so the append of the new token is never enqueued
    rc = lib.sk_decode_step(C.byref(_step_params(D=64)), None)
    assert rc == -2 and b"head_dim" in lib.sk_last_error()
    rc = lib.sk_decode_step(C.byref(_step_params(q_dtype=_lib.SK_BF16, kv_dtype=_lib.SK_F32)), None)
    assert rc == -2 and b"dtype pair" in lib.sk_last_error()
    rc = lib.sk_decode_step(C.byref(_step_params(L=24)), None)
    assert rc == -2 and b"scorer" in lib.sk_last_error()
    rc = lib.sk_decode_step(C.byref(_step_params(L=64)), None)      # 64 tables x 4 heads: table too large
    assert rc == -2 and b"scorer" in lib.sk_last_error()
    rc = lib.sk_decode_step(C.byref(_step_params(P=9, R=512)), None)
    assert rc == -1 and b"uint8" in lib.sk_last_error()


def test_budget_given_as_an_int_or_as_a_fraction():
    """`heavy_const`: an int is the budget, a float that fraction of the cached keys
    (pipeline/train_quest/modeling/modeling_llama.py:645-648, 806-808), clamped to [0, keys]."""
    from socket_b200.attention import SocketAttention
    a = SocketAttention(8, 2, 128, heavy_const=0.1, device="cpu")
    assert [a.effective_size(n) for n in (0, 9, 10, 1000, 4097)] == [0, 0, 1, 100, 409]
    b = SocketAttention(8, 2, 128, heavy_const=1024, device="cpu")
    assert [b.effective_size(n) for n in (10, 1024, 5000)] == [10, 1024, 1024]
    c = SocketAttention(8, 2, 128, heavy_const=1.5, device="cpu")
    assert c.effective_size(100) == 100
