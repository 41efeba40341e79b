"""The allocation-free attention entry point, called through its exported C symbol.

For users who cannot allocate device memory around a call (a host with a fixed memory budget, a
callback in which allocation is forbidden, a process whose pool already owns the device), the
library exports ``llmie_paged_attention_noalloc``: it keeps the split-KV scratch in a fixed array
inside the library. This test calls it twice in a row, with different inputs, and compares each
result with the ordinary entry point given caller-allocated scratch; it also checks that a call
beyond the array's size is refused. Collected last on purpose, so that a run that stops at the
first failure has run everything else before.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(dtype, seed, lens, nq=14, nkv=2, d=64, ps=16):
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    max_blocks = max(-(-L // ps) for L in lens)
    pages = sum(-(-L // ps) for L in lens) + 1
    perm = (torch.randperm(pages - 1, generator=g) + 1).tolist()
    table = torch.zeros(R, max_blocks, dtype=torch.int32)
    for r, L in enumerate(lens):
        for i in range(-(-L // ps)):
            table[r, i] = perm.pop()
    kp = torch.randn(pages, nkv, ps, d, generator=g).to(dtype).cuda()
    vp = torch.randn(pages, nkv, ps, d, generator=g).to(dtype).cuda()
    qkv = torch.randn(R, (nq + 2 * nkv) * d, generator=g).to(dtype).cuda()
    tseq = torch.arange(R, dtype=torch.int32).cuda()
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32).cuda()
    return qkv, kp, vp, table.cuda(), tseq, pos, nq, nkv, d, ps


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_ordinary_one(dtype):
    from llm_infrence_engine_b200.csrc.build import load_library

    lib = load_library()
    fn = lib.llmie_paged_attention_noalloc
    fn.restype = ctypes.c_int
    lib.llmie_noalloc_error_string.restype = ctypes.c_char_p
    ordinary = lib.llmie_paged_attention_bf16 if dtype == torch.bfloat16 else lib.llmie_paged_attention_f32
    ordinary.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = 1 if dtype == torch.bfloat16 else 0

    for seed, lens, splits in ((1, [700, 130, 1025], 4), (2, [90, 2000], 7)):  # two calls in a row share the array
        qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps = _case(dtype, seed, lens)
        N = qkv.shape[0]
        scale = ctypes.c_float(1.0 / math.sqrt(d))
        want = torch.full((N, nq * d), float("nan"), dtype=dtype, device="cuda")
        scratch = torch.empty(N * nq * splits * (d + 2), dtype=torch.float32, device="cuda")
        rc = ordinary(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(want),
                      _ptr(scratch), N, nq, nkv, d, ps, scale, 0, splits, stream)
        assert rc == 0
        got = torch.full((N, nq * d), float("nan"), dtype=dtype, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(got), N, nq, nkv,
                d, ps, scale, 0, splits, code, stream)
        assert rc == 0, lib.llmie_noalloc_error_string(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        tol = 3e-6 if dtype == torch.float32 else 1e-2
        err = (got.float() - want.float()).abs().max().item()
        assert err <= tol * max(1.0, want.float().abs().max().item()), err
        assert not torch.isnan(got.float()).any()

    # beyond the fixed array: refused with a clear message, nothing launched
    qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps = _case(dtype, 3, [64] * 700)
    out = torch.zeros((700, nq * d), dtype=dtype, device="cuda")
    rc = fn(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(out), 700, nq, nkv, d, ps,
            ctypes.c_float(0.125), 0, 4, code, stream)
    assert rc == 100002
    assert b"fewer splits" in lib.llmie_noalloc_error_string(rc)
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0
