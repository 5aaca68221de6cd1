"""The allocation-free sparse decode entry point (`sk_sparse_decode_static`) against the regular
one (`sk_sparse_decode`), both called through the C-ABI.

Some users of this library cannot allocate device memory when they call it — a server whose
memory pool already owns the whole GPU, a plug-in that is handed tensors and a stream but no
allocator — so this variant keeps its scratch inside the library.  The file name sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

from socket_b200 import _lib
from socket_b200._lib import check, dtype_code, lib, ptr, stream_ptr
from socket_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
OUT_ATOL = 2e-2          # bf16 attention-output tolerance used throughout the GPU tests


def _decode_both(q, k, v, lst, ln, T):
    B, H, D = q.shape
    Hkv = k.shape[1]
    Kmax = lst.shape[2]
    l = lib()
    need = int(l.sk_sparse_decode_workspace_bytes(B, H, D, Kmax))
    ws = torch.zeros(need, dtype=torch.uint8, device=q.device)
    ref = torch.empty_like(q)
    common = (ptr(q), dtype_code(q), ptr(k), ptr(v), dtype_code(k), k.stride(0), k.stride(1), k.stride(2),
              ptr(lst), Kmax, ptr(ln), Kmax)
    check(l.sk_sparse_decode(*common, ptr(ref), B, H, Hkv, D, T, None, ptr(ws), ws.numel(), None,
                             stream_ptr(q.device)), "sk_sparse_decode")
    got = torch.empty_like(q)
    check(l.sk_sparse_decode_static(*common, ptr(got), B, H, Hkv, D, T, None, None, stream_ptr(q.device)),
          "sk_sparse_decode_static")
    torch.cuda.synchronize()
    return ref, got


def test_static_scratch_decode_matches_regular_entry_point_twice():
    g = torch.Generator().manual_seed(0)
    for call, (B, H, Hkv, T, K) in enumerate([(2, 8, 2, 3000, 300), (1, 32, 8, 9000, 1216)]):
        inp = make_decode_inputs(B, H, Hkv, T, seed=40 + call, dtype=torch.bfloat16)
        q, k, v = inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV)
        lst = torch.randint(0, T, (B, H, K), generator=g, dtype=torch.int32)
        lst[:, :, 5] = -1                                   # a masked entry
        ln = torch.full((B, H), K, dtype=torch.int32)
        ln[0, 1] = K // 3                                   # a shorter row
        ref, got = _decode_both(q, k, v, lst.to(DEV), ln.to(DEV), T)
        assert torch.isfinite(got.float()).all()
        assert (got.float() - ref.float()).abs().max() <= OUT_ATOL
        # same kernel, same split of the list: the two results are in fact identical
        assert torch.equal(got, ref)


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_scratch_call_allocates_nothing_and_works_on_a_side_stream():
    """Free device memory (cudaMemGetInfo) is the same before and after the calls, also on a
    stream that is not the default one; the first call on the device, which resolves the buffer's
    address, is made beforehand."""
    B, H, Hkv, T, K = 2, 8, 2, 4000, 500
    inp = make_decode_inputs(B, H, Hkv, T, seed=77, dtype=torch.bfloat16)
    q, k, v = inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV)
    g = torch.Generator().manual_seed(1)
    lst = torch.randint(0, T, (B, H, K), generator=g, dtype=torch.int32).to(DEV)
    ln = torch.full((B, H), K, dtype=torch.int32, device=DEV)
    ref, got0 = _decode_both(q, k, v, lst, ln, T)            # warm: address resolved, kernels loaded
    got = torch.empty_like(q)
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream())
    l = lib()
    args = (ptr(q), dtype_code(q), ptr(k), ptr(v), dtype_code(k), k.stride(0), k.stride(1), k.stride(2),
            ptr(lst), K, ptr(ln), K, ptr(got), B, H, Hkv, 128, T, None, None)
    before = _free_bytes()
    for _ in range(3):
        check(l.sk_sparse_decode_static(*args, side.cuda_stream), "sk_sparse_decode_static")
    side.synchronize()
    assert _free_bytes() == before
    assert torch.equal(got, ref)


def test_static_scratch_large_then_small_call_back_to_back():
    """A large shape followed at once by a small one on the same stream: the second call starts
    from whatever the first left in the shared buffer and must still match."""
    g = torch.Generator().manual_seed(2)
    cases = []
    for call, (B, H, Hkv, T, K) in enumerate([(2, 32, 8, 6000, 1500), (1, 4, 1, 700, 40)]):
        inp = make_decode_inputs(B, H, Hkv, T, seed=50 + call, dtype=torch.bfloat16)
        lst = torch.randint(0, T, (B, H, K), generator=g, dtype=torch.int32).to(DEV)
        ln = torch.full((B, H), K, dtype=torch.int32, device=DEV)
        cases.append((inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), lst, ln, T))
    refs = [_decode_both(*c)[0] for c in cases]
    l = lib()
    outs = []
    for q, k, v, lst, ln, T in cases:                          # no synchronisation in between
        B, H, D = q.shape
        K = lst.shape[2]
        got = torch.empty_like(q)
        check(l.sk_sparse_decode_static(ptr(q), dtype_code(q), ptr(k), ptr(v), dtype_code(k), k.stride(0),
                                        k.stride(1), k.stride(2), ptr(lst), K, ptr(ln), K, ptr(got), B, H,
                                        k.shape[1], D, T, None, None, stream_ptr(q.device)),
              "sk_sparse_decode_static")
        outs.append(got)
    torch.cuda.synchronize()
    for got, ref in zip(outs, refs):
        assert torch.equal(got, ref)


def test_static_scratch_rejects_oversized_requests():
    l = lib()
    B, H, D, K = 64, 64, 128, 20000
    assert l.sk_sparse_decode_workspace_bytes(B, H, D, K) > _lib.SK_SPARSE_DECODE_STATIC_BYTES
    x = torch.zeros(16, device=DEV)
    rc = l.sk_sparse_decode_static(ptr(x), 1, ptr(x), ptr(x), 1, 1024, 1024, 128, ptr(x), K, ptr(x), K, ptr(x),
                                   B, H, 8, D, 100, None, None, stream_ptr(x.device))
    assert rc == -4
    msg = l.sk_last_error().decode()
    assert "built-in buffer" in msg and "sk_sparse_decode" in msg
