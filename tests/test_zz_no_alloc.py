"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers cannot allocate device memory when they need attention: a host thread that lives
inside another framework's memory pool, a serving loop that forbids allocations after start-up,
or a C / ctypes caller with raw device pointers and no allocator to lend a workspace.  For them
the library exports `fc_decode_attention_noalloc`, whose split-KV scratch is a static device
array inside the shared object.  This test loads the shared object with ctypes, calls the symbol
twice in a row on different inputs and compares each result with the regular entry point at the
same split count.  It is collected last so that a run that stops at the first failure has already
run every other test.
"""
import ctypes
import glob
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from fastcache_b200.ops.loader import ext
    ext()                                                  # resolves torch's libraries first
    path = glob.glob(os.path.join(ROOT, "fastcache_b200", "_C*.so"))[0]
    lib = ctypes.CDLL(path)
    fn = lib.fc_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 8 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p,
                                                                 ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _case(seed, B, Hq, Hkv, D, bs, lens):
    g = torch.Generator().manual_seed(seed)
    nb_per = [-(-n // bs) for n in lens]
    nb = sum(nb_per) + 2
    kc = torch.randn(nb, Hkv, bs, D, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(nb, Hkv, bs, D, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(nb, generator=g).tolist()
    bt = torch.zeros(B, max(nb_per), dtype=torch.int32)
    k = 0
    for i, n in enumerate(nb_per):
        bt[i, :n] = torch.tensor(perm[k:k + n], dtype=torch.int32)
        k += n
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16).cuda()
    cl = torch.tensor(lens, dtype=torch.int32).cuda()
    return q, kc, vc, bt.cuda(), cl


def _call(fn, q, kc, vc, bt, cl, splits):
    B, Hq, D = q.shape
    out = torch.empty_like(q)
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), cl.data_ptr(), out.data_ptr(), B, Hq,
            kc.shape[1], D, kc.shape[2], bt.shape[1], kc.shape[0], splits, float(D) ** -0.5, None, stream, err, 256)
    return rc, out, err.value.decode()


def test_noalloc_entry_matches_regular_entry_twice():
    from fastcache_b200.ops.loader import ext
    fn = _lib()
    for seed, (B, Hq, Hkv, D, bs, lens, splits) in enumerate([
            (3, 8, 2, 128, 16, [700, 33, 257], 4), (2, 4, 4, 64, 32, [1000, 90], 3)]):
        q, kc, vc, bt, cl = _case(seed, B, Hq, Hkv, D, bs, lens)
        before = torch.cuda.memory_allocated()
        rc, out, msg = _call(fn, q, kc, vc, bt, cl, splits)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # only the caller's `out` tensor was allocated (by the test itself)
        assert torch.cuda.memory_allocated() - before <= out.numel() * 2 + 512
        want = ext().decode_attention(q, kc, vc, bt, cl, float(D) ** -0.5, splits, 0)
        torch.cuda.synchronize()
        assert (out.float() - want.float()).abs().max().item() < 2e-2
        # and against the plain fp32 PyTorch statement of the op
        from fastcache_b200.ops import reference as ref
        oracle = ref.decode_attention(q.float().cpu(), kc.float().cpu(), vc.float().cpu(), bt.cpu(), cl.cpu(),
                                      float(D) ** -0.5)
        assert (out.float().cpu() - oracle.float()).abs().max().item() < 2e-2


def test_noalloc_entry_rejects_oversized_requests():
    fn = _lib()
    q, kc, vc, bt, cl = _case(0, 2, 4, 4, 64, 32, [40, 50])
    big_q = torch.empty(4096, 32, 128, dtype=torch.bfloat16, device="cuda")      # 4096*32*32*128 floats needed
    big_bt = torch.zeros(4096, 1, dtype=torch.int32, device="cuda")
    big_cl = torch.zeros(4096, dtype=torch.int32, device="cuda")
    kc128 = torch.zeros(4, 32, 32, 128, dtype=torch.bfloat16, device="cuda")
    rc, _, msg = _call(fn, big_q, kc128, kc128, big_bt, big_cl, 32)
    assert rc == 2 and "static scratch" in msg
    rc, _, msg = _call(fn, q, kc, vc, bt, cl, 0)
    assert rc == 1
    odd = torch.zeros(4, 4, 12, 64, dtype=torch.bfloat16, device="cuda")         # block size 12: not a multiple of 8
    rc, _, msg = _call(fn, q, odd, odd, bt, cl, 2)
    assert rc == 1 and "multiple of 8" in msg
