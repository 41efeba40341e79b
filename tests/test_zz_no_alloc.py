"""The allocation-free attention entry point, called through its exported C symbol.

For users who cannot allocate device memory around a call (a host with a fixed memory budget, a
callback in which allocation is forbidden, a process whose pool already owns the device), the
library exports ``llmie_paged_attention_noalloc``: it keeps the split-KV scratch in a fixed array
inside the library. This test calls it twice in a row, with different inputs, and compares each
result with the ordinary entry point given caller-allocated scratch and with a plain torch statement
of the attention (one far key made to stand out, a sliding window, a request so short that its last
slices are empty); the driver's count of free device memory must not move across a call. It also
checks that a call beyond the array's size is refused. Collected last on purpose, so that a run that stops at the
first failure has run everything else before.
"""
import ctypes
import gc
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(dtype, seed, lens, nq=14, nkv=2, d=64, ps=16, spike=False):
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
    qkv = torch.randn(R, (nq + 2 * nkv) * d, generator=g).to(dtype)
    if spike:   # key 1 of the last request gets a score far above the rest: losing it would show
        page, off = int(table[R - 1, 1 // ps]), 1 % ps
        qv = qkv[R - 1, :d].float()
        kp[page, 0, off] = (qv / qv.norm() * 6).to(dtype)
        vp[page, 0, off] = 10.0
    qkv = qkv.cuda()
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

    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from torch_kernels import TorchKernels

    # two calls in a row share the array; the second has a window and a request of 3 tokens whose later slices are empty
    for seed, lens, splits, window in ((1, [700, 130, 1025], 4, 0), (2, [90, 2000, 3], 7, 600)):
        qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps = _case(dtype, seed, lens, spike=True)
        N = qkv.shape[0]
        scale = ctypes.c_float(1.0 / math.sqrt(d))
        want = torch.full((N, nq * d), float("nan"), dtype=dtype, device="cuda")
        scratch = torch.empty(N * nq * splits * (d + 2), dtype=torch.float32, device="cuda")
        rc = ordinary(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(want),
                      _ptr(scratch), N, nq, nkv, d, ps, scale, window, splits, 0, stream)
        assert rc == 0
        got = torch.full((N, nq * d), float("nan"), dtype=dtype, device="cuda")
        plain = TorchKernels().paged_attention(qkv.cpu(), kp.cpu(), vp.cpu(), table.cpu(), tseq.cpu(), pos.cpu(), nq, nkv, d, ps,
                                               1.0 / math.sqrt(d), window, max(lens))
        gc.collect()   # (tensors of earlier tests that only a collection frees must not go while the call is measured)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]   # the driver's own count: it would see an allocation by the library itself
        rc = fn(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(got), N, nq, nkv,
                d, ps, scale, window, splits, code, stream)
        assert rc == 0, lib.llmie_noalloc_error_string(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if seed == 2:   # (the first call on a device may make the runtime load the kernels' code; the second call must not move it)
            assert torch.cuda.mem_get_info()[0] == free_before
        tol = 3e-6 if dtype == torch.float32 else 1e-2
        err = (got.float() - want.float()).abs().max().item()
        assert err <= tol * max(1.0, want.float().abs().max().item()), err
        assert not torch.isnan(got.float()).any()
        err = (got.float().cpu() - plain.float()).abs().max().item()
        assert err <= tol * max(1.0, plain.float().abs().max().item()), f"against the plain statement: {err}"

    # beyond the fixed array: refused with a clear message, nothing launched
    qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps = _case(dtype, 3, [64] * 700)
    out = torch.zeros((700, nq * d), dtype=dtype, device="cuda")
    rc = fn(_ptr(qkv), qkv.shape[1], _ptr(kp), _ptr(vp), _ptr(table), table.shape[1], _ptr(tseq), _ptr(pos), _ptr(out), 700, nq, nkv, d, ps,
            ctypes.c_float(0.125), 0, 4, code, stream)   # (scale, window, splits, dtype)
    assert rc == 100002
    assert b"fewer splits" in lib.llmie_noalloc_error_string(rc)
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0
