"""Each CUDA kernel alone against its plain torch statement (tests/torch_kernels.py), in float32 and
bfloat16, at sizes other than the engine's: odd widths, head sizes in steps of 16 (and 8), any
number of heads and groups, page edges, windows, several key slices."""
import math

import pytest
import torch

from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from llm_infrence_engine_b200.csrc import get_kernels

    return get_kernels()


REF = TorchKernels()


def tol(dtype, f32=2e-6, bf16=1e-2):
    return f32 if dtype == torch.float32 else bf16


def close(a, b, t):
    a, b = a.float().cpu(), b.float().cpu()
    scale = max(1.0, b.abs().max().item())
    err = (a - b).abs().max().item()
    assert err <= t * scale, f"max |difference| {err:.3g} > {t * scale:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,N", [(50, 24, 7), (1000, 1030, 3)])
def test_embed(K, dtype, V, H, N):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (N,), generator=g).int()
    got = K.embed(ids.cuda(), table.cuda())
    assert torch.equal(got.cpu(), REF.embed(ids, table))


@pytest.mark.parametrize("half,theta", [(8, 1e4), (24, 1e6), (64, 5e5)])
def test_rope_tables(K, half, theta):
    pos = torch.tensor([0, 1, 2, 17, 255, 256, 4095, 8191, 100000], dtype=torch.int32)
    inv = 1.0 / (theta ** (torch.arange(0, 2 * half, 2).float() / (2 * half)))
    c, s = K.rope_tables(pos.cuda(), inv.cuda())
    rc, rs = REF.rope_tables(pos, inv)
    close(c, rc, 2e-6)  # the float32 angle is rounded before cos/sin on both sides
    close(s, rs, 2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H,eps", [(5, 64, 1e-6), (3, 200, 1e-5), (2, 4100, 3e-6), (9, 896, 1e-6),
                                     (70, 896, 1e-6), (40, 1536, 1e-5), (200, 1536, 1e-5), (100, 72, 1e-5), (64, 4104, 1e-6)])
def test_add_rmsnorm(K, dtype, N, H, eps):
    g = torch.Generator().manual_seed(1)
    res = torch.randn(N, H, generator=g) * 3
    delta = (torch.randn(N, H, generator=g)).to(dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    for d in (delta, None):
        r_gpu, r_ref = res.clone().cuda(), res.clone()
        got = K.add_rmsnorm(r_gpu, None if d is None else d.cuda(), w.cuda(), eps, dtype)
        want = REF.add_rmsnorm(r_ref, d, w, eps, dtype)
        close(got, want, tol(dtype, 2e-6, 8e-3))
        assert torch.equal(r_gpu.cpu(), r_ref)  # the residual sum is exact 32-bit addition on both sides
    rows = torch.tensor([N - 1, 0, N // 2], dtype=torch.int32) if N < 32 else torch.randperm(N, generator=g)[:N - 1].int()
    r_gpu = res.clone().cuda()
    got = K.rmsnorm_rows(r_gpu, delta.cuda(), w.cuda(), eps, rows.cuda(), dtype)
    close(got, REF.rmsnorm_rows(res, delta, w, eps, rows, dtype), tol(dtype, 2e-6, 8e-3))
    assert torch.equal(r_gpu.cpu(), res)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 131, 80), (70, 65, 200), (8, 320, 96), (130, 64, 17)])
def test_linear(K, dtype, M, N, K_):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(M, K_, generator=g).to(dtype)
    w = torch.randn(N, K_, generator=g).to(dtype)
    want = x.double() @ w.double().T
    got = K.linear(x.cuda(), w.cuda())
    close(got, want, tol(dtype, 2e-6, 8e-3))
    got32 = K.linear(x.cuda(), w.cuda(), out_dtype=torch.float32)
    close(got32, want, 2e-6)
    # a row's result does not depend on the rows beside it
    if M > 1:
        alone = K.linear(x[M - 1:].contiguous().cuda(), w.cuda(), out_dtype=torch.float32)
        assert torch.equal(alone[0], got32[M - 1])


def test_linear_float32_is_true_32bit(K):
    """Inputs that a reduced-precision matrix mode (TF32, bfloat16) would round: 1 + 2^-12 squared."""
    x = torch.full((4, 64), 1 + 2.0 ** -12)
    w = torch.full((5, 64), 1 + 2.0 ** -12)
    got = K.linear(x.cuda(), w.cuda()).cpu()
    want = (x.double() @ w.double().T)
    assert (got.double() - want).abs().max() < 1e-4  # TF32 would be off by 64 * 2^-11 = 0.03


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N", [11, 200])   # (many tokens in bfloat16 take a kernel of their own with wider accesses)
@pytest.mark.parametrize("nq,nkv,d,ps,bias", [(4, 2, 16, 16, True), (3, 1, 32, 8, True), (6, 3, 48, 16, False), (14, 2, 64, 16, True),
                                              (12, 2, 128, 16, True), (5, 1, 24, 16, True)])
def test_rope_kv_write(K, dtype, N, nq, nkv, d, ps, bias):
    g = torch.Generator().manual_seed(3)
    pages = -(-N // ps) + 8
    qkv = torch.randn(N, (nq + 2 * nkv) * d, generator=g).to(dtype)
    b = torch.randn((nq + 2 * nkv) * d, generator=g) if bias else None
    pos = torch.randint(0, 500, (N,), generator=g).int()
    inv = 1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))
    cos, sin = REF.rope_tables(pos, inv)
    slots = torch.randperm(pages * ps, generator=g)[:N].int()
    kp, vp = torch.zeros(pages, nkv, ps, d, dtype=dtype), torch.zeros(pages, nkv, ps, d, dtype=dtype)
    q_ref, kp_ref, vp_ref = qkv.clone(), kp.clone(), vp.clone()
    REF.rope_kv_write(q_ref, b, cos, sin, slots, kp_ref, vp_ref, nq, nkv, d, ps, True)
    q_gpu, kp_gpu, vp_gpu = qkv.clone().cuda(), kp.cuda(), vp.cuda()
    out = K.rope_kv_write(q_gpu, None if b is None else b.cuda(), cos.cuda(), sin.cuda(), slots.cuda(), kp_gpu, vp_gpu, nq, nkv, d, ps, True)
    assert out.data_ptr() == q_gpu.data_ptr()   # same types: in place
    close(q_gpu, q_ref, tol(dtype, 1e-6, 8e-3))
    close(kp_gpu, kp_ref, tol(dtype, 1e-6, 8e-3))
    close(vp_gpu, vp_ref, tol(dtype, 1e-6, 8e-3))
    # slots that were not written stay untouched
    untouched = torch.ones(pages * ps, dtype=torch.bool)
    untouched[slots.long()] = False
    assert kp_gpu.cpu().permute(0, 2, 1, 3).reshape(pages * ps, -1)[untouched].abs().sum() == 0


@pytest.mark.parametrize("N,H,nq,nkv,ps,bias,write", [
    (2048, 896, 14, 2, 16, True, True),     # the bench's prompt
    (129, 96, 6, 2, 16, True, True),        # one row more than a tile; an inner size that is no multiple of 64
    (300, 200, 3, 1, 8, False, True),       # 5 heads: the last tile holds one head only
    (513, 1536, 12, 2, 32, True, False),    # no cache write (a layer that reads another layer's cache)
    (200, 72, 1, 1, 16, True, True),        # three heads in one block of columns; two inner blocks, the second ragged
])
def test_qkv_rope_tcgen05(K, monkeypatch, N, H, nq, nkv, ps, bias, write):
    """The q/k/v product of prompt portions with bias, rotation and cache write in its epilogue (tcgen05, head size 64)
    against product, rotation and cache write one after the other in 32-bit. Some tokens have no slot (negative)."""
    monkeypatch.setattr(K, "tc_qkv_min_rows", 129)   # (serving takes this kernel for long portions only)
    d = 64
    g = torch.Generator().manual_seed(13)
    x = torch.randn(N, H, generator=g).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, H, generator=g) / math.sqrt(H)).to(torch.bfloat16)
    b = torch.randn((nq + 2 * nkv) * d, generator=g) if bias else None
    pos = torch.randint(0, 3000, (N,), generator=g).int()
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))
    cos, sin = REF.rope_tables(pos, inv)
    pages = -(-N // ps) + 2
    slots = torch.randperm(pages * ps, generator=g)[:N].int()
    slots[::7] = -1
    kp, vp = torch.zeros(pages, nkv, ps, d, dtype=torch.bfloat16), torch.zeros(pages, nkv, ps, d, dtype=torch.bfloat16)
    want = (x.float() @ w.float().T)
    kp_ref, vp_ref = kp.float(), vp.float()
    keep = slots >= 0
    REF.rope_kv_write(want, b, cos, sin, slots.clamp(min=0), kp_ref, vp_ref, nq, nkv, d, ps, False)
    if write:
        page, off = (slots[keep] // ps).long(), (slots[keep] % ps).long()
        kp_ref[page, :, off] = want.view(N, -1, d)[keep][:, nq:nq + nkv]
        vp_ref[page, :, off] = want.view(N, -1, d)[keep][:, nq + nkv:]
    before = K.launches
    kp_gpu, vp_gpu = kp.cuda(), vp.cuda()
    for _ in range(2):
        got = K.qkv_rope(x.cuda(), w.cuda(), None if b is None else b.cuda(), cos.cuda(), sin.cuda(), slots.cuda(), kp_gpu, vp_gpu,
                         nq, nkv, d, ps, write)
        K.check_device_errors()
        close(got, want, 8e-3)
        close(kp_gpu, kp_ref, 8e-3)
        close(vp_gpu, vp_ref, 8e-3)
    assert K.launches - before == 2   # one kernel per call


def _attention_case(dtype, nq, nkv, d, ps, lens, qlens, window, seed, spike=False):
    """Requests with ``lens`` cached+new tokens, the last ``qlens`` of each being this step's tokens,
    pages handed out in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    max_blocks = max(-(-L // ps) for L in lens) + 1
    pages = sum(-(-L // ps) for L in lens) + 3
    perm = (torch.randperm(pages - 1, generator=g) + 1).tolist()
    table = torch.zeros(R, max_blocks, dtype=torch.int32)
    kp = torch.randn(pages, nkv, ps, d, generator=g).to(dtype)   # stale values everywhere, also beyond the lengths
    vp = torch.randn(pages, nkv, ps, d, generator=g).to(dtype)
    for r, L in enumerate(lens):
        for i in range(-(-L // ps)):
            table[r, i] = perm.pop()
    token_seq, positions = [], []
    for r, (L, ql) in enumerate(zip(lens, qlens)):
        token_seq += [r] * ql
        positions += list(range(L - ql, L))
    N = len(token_seq)
    qkv = torch.randn(N, (nq + 2 * nkv) * d, generator=g).to(dtype)
    if spike:  # one far key gets a score that stands out: a kernel that skips or misplaces it shows
        r = 0
        far = 1 if lens[0] > 1 else 0
        page, off = int(table[r, far // ps]), far % ps
        qv = qkv[0, :d].float()
        kp[page, 0, off] = (qv / qv.norm() * 6).to(dtype)
        vp[page, 0, off] = 10.0
    return qkv, kp, vp, table, torch.tensor(token_seq, dtype=torch.int32), torch.tensor(positions, dtype=torch.int32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,ps,lens,qlens,window,splits", [
    (4, 2, 16, 16, [1, 15, 16, 17, 33], [1, 1, 16, 2, 33], 0, None),
    (3, 1, 32, 8, [40, 9, 64], [1, 9, 5], 0, 1),
    (6, 3, 48, 16, [70, 31], [70, 1], 24, None),
    (14, 2, 64, 16, [300, 700, 5], [1, 1, 5], 0, 3),
    (14, 2, 64, 16, [900], [900], 0, None),
    (8, 8, 80, 32, [65, 130], [2, 1], 50, 2),
    (16, 1, 128, 64, [257], [3], 0, 4),
    (2, 2, 256, 16, [48], [48], 0, None),
])
def test_paged_attention(K, dtype, nq, nkv, d, ps, lens, qlens, window, splits):
    for spike in (False, True):
        qkv, kp, vp, table, tseq, pos = _attention_case(dtype, nq, nkv, d, ps, lens, qlens, window, 4, spike)
        scale = 1.0 / math.sqrt(d)
        want = REF.paged_attention(qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps, scale, window, max(lens))
        got = K.paged_attention(qkv.cuda(), kp.cuda(), vp.cuda(), table.cuda(), tseq.cuda(), pos.cuda(), nq, nkv, d, ps, scale,
                                window, max(lens), num_splits=splits)
        close(got, want, tol(dtype, 3e-6, 1e-2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(K, dtype):
    g = torch.Generator().manual_seed(5)
    for rows, width in ((7, 203), (3, 1028), (2, 8), (5, 4864), (40, 200)):  # odd widths take the scalar kernel; 1028 is 4 beyond a block of threads
        gu = (torch.randn(rows, 2 * width, generator=g) * 4).to(dtype)
        close(K.silu_mul(gu.cuda()), REF.silu_mul(gu), tol(dtype, 1e-6, 8e-3))


@pytest.mark.parametrize("M,H,I", [
    (2048, 896, 4864),     # the bench's prompt: 16 x 38 tiles on a persistent grid
    (129, 96, 200),        # one row more than a tile; inner size and width ragged
    (300, 200, 328),
    (513, 1536, 8960),     # the 1.5B model's widths
    (1000, 72, 64),        # fewer output columns than a tile is wide
    (385, 128, 136),       # four tiles of rows, the last of one row: its partner in the pair has nothing to store
    (512, 64, 4736),       # 4 x 37 tiles of 128 columns are exactly one round of 148 blocks: the widest tile is chosen
    (512, 64, 3552),       # ... and here tiles of 96 columns are
])
@pytest.mark.parametrize("form", ["one block per tile", "pairs of blocks on tiles of 256 rows", "pairs of blocks that share weights by multicast"])
def test_gate_up_act_tcgen05(K, monkeypatch, form, M, H, I):
    """The gate/up product of prompt portions with silu(gate) * up as its epilogue (one tcgen05 kernel, the float32 sums stay
    in tensor memory) against product and activation one after the other in 32-bit; all three forms of the kernel."""
    if (form.endswith("multicast") and K._gate_up_cluster is None) or (form.startswith("pairs of blocks on") and K._gate_up_pair is None):
        pytest.skip("the library was built without this optional kernel")
    monkeypatch.setattr(K, "use_cluster_gate_up", form.endswith("multicast"))
    monkeypatch.setattr(K, "use_pair_gate_up", form.startswith("pairs of blocks on"))
    monkeypatch.setattr(K, "pair_gate_up_min_rows", 129)
    g = torch.Generator().manual_seed(60)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, H, generator=g) / math.sqrt(H) * 2).to(torch.bfloat16)
    gu = x.float() @ w.float().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    before = K.launches
    for _ in range(2):
        got = K.gate_up_act(x.cuda(), w.cuda())
        K.check_device_errors()
        assert got.dtype == torch.bfloat16 and tuple(got.shape) == (M, I)
        close(got, want, 8e-3)
    assert K.launches - before == 2   # one kernel per call
    small = K.gate_up_act(x[:5].contiguous().cuda(), w.cuda())   # a decode-sized batch: product into float32 sums, then the activation kernel
    close(small, want[:5], 8e-3)
    assert K._acc.abs().sum().item() == 0


@pytest.mark.parametrize("V", [17, 320, 151936])
def test_argmax(K, V):
    g = torch.Generator().manual_seed(6)
    logits = torch.randn(5, V, generator=g)
    logits[1, V // 2] = logits[1, V - 1] = 50.0  # a tie: the lower index wins
    logits[2, 0] = 60.0
    logits[3, V - 1] = 60.0
    got = K.argmax(logits.cuda()).cpu()
    assert got.tolist() == logits.argmax(-1).tolist()
    assert got[1] == V // 2


@pytest.mark.parametrize("single_block", [False, True])
@pytest.mark.parametrize("V", [131, 320, 5000, 20001, 40000, 151936])   # a cluster of 1, 1, 1, 2, 4 and 8 blocks per row
def test_sample(K, monkeypatch, V, single_block):
    """Both sampling kernels (a cluster of blocks per row with the row in shared memory; one block per row) draw the token the
    plain sampler draws, for every combination of temperature, top-k and top-p and for draws at both ends of the range."""
    from plain_qwen2 import plain_draw, plain_logits_to_probs

    monkeypatch.setattr(K, "sample_single_block", single_block)

    g = torch.Generator().manual_seed(7)
    rows = []
    for temp, k, p in [(0.8, 0, 1.0), (1.3, 20, 1.0), (0.7, 0, 0.9), (1.0, 50, 0.5), (0.0, 0, 1.0), (0.5, 1, 1.0), (2.0, 7, 0.3)]:
        for u in (0.0, 0.123, 0.5, 0.77, 0.999999):
            rows.append((temp, k, p, u))
    M = len(rows)
    logits = torch.randn(M, V, generator=g) * 3
    got = K.sample(logits.cuda(), torch.tensor([r[0] for r in rows]).cuda(), torch.tensor([r[1] for r in rows], dtype=torch.int32).cuda(),
                   torch.tensor([r[2] for r in rows]).cuda(), torch.tensor([r[3] for r in rows]).cuda()).cpu().tolist()
    for i, (temp, k, p, u) in enumerate(rows):
        want = plain_draw(logits[i], temp, k, p, u)
        if got[i] != want:  # only a draw that lands on the edge between two tokens may differ, and then by one kept token
            probs = plain_logits_to_probs(logits[i], temp, k, p).double()
            cdf = probs.cumsum(-1)
            edge = min(abs(float(cdf[got[i]]) - u * float(cdf[-1])), abs(float(cdf[want]) - u * float(cdf[-1])))
            assert probs[got[i]] > 0 and edge < 1e-6, (i, rows[i], got[i], want)


@pytest.mark.parametrize("single_block", [False, True])
def test_sample_frequencies(K, monkeypatch, single_block):
    """Empirical frequencies follow the distribution (the reference's test draws 4,000 times, tests/test_sampler.py:6-44)."""
    monkeypatch.setattr(K, "sample_single_block", single_block)
    from plain_qwen2 import plain_logits_to_probs
    from llm_infrence_engine_b200.sampling import uniform_from

    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -3.0])
    M = 4000
    u = torch.tensor([uniform_from(11, c) for c in range(M)])
    got = K.sample(logits.repeat(M, 1).cuda(), torch.full((M,), 0.9).cuda(), torch.zeros(M, dtype=torch.int32).cuda(),
                   torch.ones(M).cuda(), u.cuda()).cpu()
    freq = torch.bincount(got.long(), minlength=6).double() / M
    assert (freq - plain_logits_to_probs(logits, 0.9).double()).abs().max() < 0.03


class _Batch:
    """What the tensor-core attention needs to know of a step: rows per request, on host and device."""

    def __init__(self, qlens):
        self.seq_lens = list(qlens)
        self.max_seq_len = max(qlens)
        starts = [0]
        for n in qlens:
            starts.append(starts[-1] + n)
        self.seq_starts_dev = torch.tensor(starts, dtype=torch.int32).cuda()
        self._tables = {}


@pytest.mark.parametrize("nq,nkv,d,ps,lens,qlens,window,splits", [
    (14, 2, 64, 16, [300, 700, 5, 64, 65], [1, 1, 1, 1, 1], 0, None),      # decode, 7 heads per group
    (14, 2, 64, 16, [8200, 100], [1, 1], 0, 5),                              # decode, long context, slices merged in the kernel
    (12, 2, 128, 16, [513, 31], [1, 1], 0, 3),                               # head size 128, 6 per group
    (16, 1, 64, 32, [257, 1], [1, 1], 0, 2),                                 # 16 heads on one key/value head; a request of one token
    (4, 4, 64, 8, [90], [1], 40, None),                                      # window, no grouping
    (14, 2, 64, 16, [300, 77, 500], [300, 1, 37], 0, None),                  # prefill rows with a decode token and a late portion between
    (14, 2, 64, 16, [1000], [1000], 0, None),                                # a long prompt whole
    (14, 2, 64, 16, [2100], [16], 0, 4),                                     # a short portion far into a long request, sliced
    (12, 2, 128, 16, [150, 64], [150, 2], 0, None),
    (6, 3, 64, 16, [200, 130], [200, 5], 48, None),                          # window in prefill
    (8, 8, 128, 64, [129], [129], 0, 2),
    (28, 4, 128, 16, [70], [70], 0, None),
])
def test_paged_attention_tensor_cores(K, nq, nkv, d, ps, lens, qlens, window, splits):
    for spike in (False, True):
        qkv, kp, vp, table, tseq, pos = _attention_case(torch.bfloat16, nq, nkv, d, ps, lens, qlens, window, 11, spike)
        scale = 1.0 / math.sqrt(d)
        want = REF.paged_attention(qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps, scale, window, max(lens))
        before = K.launches
        got = K.paged_attention(qkv.cuda(), kp.cuda(), vp.cuda(), table.cuda(), tseq.cuda(), pos.cuda(), nq, nkv, d, ps, scale,
                                window, max(lens), batch=_Batch(qlens), num_splits=splits)
        close(got, want, 1e-2)
        # twice in a row: the slice counters must be back at zero
        got = K.paged_attention(qkv.cuda(), kp.cuda(), vp.cuda(), table.cuda(), tseq.cuda(), pos.cuda(), nq, nkv, d, ps, scale,
                                window, max(lens), batch=_Batch(qlens), num_splits=splits)
        close(got, want, 1e-2)


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("nq,nkv,d,ps,lens,splits", [
    (14, 2, 64, 16, [8192] * 8, None),            # the headline decode step: the planner's own choice (9 slices on 148 SMs)
    (14, 2, 64, 16, [8192] * 7 + [40], 9),        # one request far shorter than the others: its later slices are empty
    (14, 2, 64, 16, [5000, 3000, 17], 13),        # more slices than the merge loads in one group of 12
    (14, 2, 64, 16, [8200, 100], 33),
    (14, 2, 64, 16, [8200, 1], 64),               # the most slices the kernel takes; a request of one token
    (14, 2, 64, 16, [8192] * 8, 4),               # few enough to merge as a cluster when that is on
    (12, 2, 128, 16, [8192] * 4, None),           # head size 128: chunks of 16 keys, more slices
    (12, 2, 128, 16, [4100, 900], 13),
    (28, 4, 128, 32, [6000, 64], 8),
    (16, 1, 64, 64, [3000, 3000, 2000], 25),      # 16 heads on one key/value head, pages of 64
    (14, 2, 64, 16, [300 + 7 * i for i in range(100)], None),   # more blocks than multiprocessors, no slices: blocks of four warps, two per SM
    (12, 2, 128, 16, [90 + 11 * i for i in range(80)], 1),
])
def test_decode_attention_with_many_key_slices(K, monkeypatch, cluster, nq, nkv, d, ps, lens, splits):
    """Decoded tokens at long contexts: the keys of a token are cut into slices that run as blocks of their own and are
    merged either as a thread-block cluster through shared memory (few slices) or through scratch memory, a counter and
    the last block to finish (many slices; what serving at a long context runs). Twice in a row: the counters must be
    back at zero. With a far key that must not be lost."""
    monkeypatch.setattr(K, "cluster_merge", cluster)
    qlens = [1] * len(lens)
    for spike in (False, True):
        qkv, kp, vp, table, tseq, pos = _attention_case(torch.bfloat16, nq, nkv, d, ps, lens, qlens, 0, 17, spike)
        scale = 1.0 / math.sqrt(d)
        want = REF.paged_attention(qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps, scale, 0, max(lens))
        dev = [t.cuda() for t in (qkv, kp, vp, table, tseq, pos)]
        for _ in range(2):
            got = K.paged_attention(*dev, nq, nkv, d, ps, scale, 0, max(lens), batch=_Batch(qlens), num_splits=splits)
            close(got, want, 1e-2)
    assert K._attn_counters is None or K._attn_counters.abs().sum().item() == 0


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("nq,nkv,d,ps,H,lens,window,bias,write", [
    (14, 2, 64, 16, 896, [300, 700, 5, 64, 65, 1, 33, 32], 0, True, True),   # page edges, a request of one token, chunk edges
    (14, 2, 64, 16, 896, [8192] * 8, 0, True, True),                          # the headline decode step
    (14, 2, 64, 16, 896, [4000, 17, 2100], 0, True, True),                    # several slices, one request far shorter
    (12, 2, 128, 16, 1536, [513, 31, 1000, 2049], 0, True, True),             # heads of 128
    (4, 4, 64, 8, 200, [90, 33, 41], 40, False, True),                        # a window, no bias, no grouping, pages of 8
    (6, 3, 64, 32, 96, [70, 200], 0, True, False),                            # keys and values are in the cache already
    (16, 2, 128, 64, 256, [130, 64], 0, True, True),                          # 8 heads per key/value head, pages of 64
])
def test_qkv_attention_of_a_decode_step(K, monkeypatch, cluster, nq, nkv, d, ps, H, lens, window, bias, write):
    """Decode steps: the q/k/v product leaves float32 sums, and the attention kernel itself adds the bias, rotates and writes
    the token's key and value into the cache, against product, rotation kernel and attention one after the other in plain
    torch. The tokens' own cache slots (and everything behind them) hold NaN beforehand: nothing stale may be read."""
    monkeypatch.setattr(K, "cluster_merge", cluster)
    monkeypatch.setattr(K, "fuse_decode_rope_head_dims", (64, 128))   # serving fuses heads of 64 only (measured); the kernel takes both
    g = torch.Generator().manual_seed(50)
    B = len(lens)
    qlens = [1] * B
    _, kp, vp, table, tseq, pos = _attention_case(torch.bfloat16, nq, nkv, d, ps, lens, qlens, window, 51)
    width = (nq + 2 * nkv) * d
    x = torch.randn(B, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(width, H, generator=g) / math.sqrt(H)).to(torch.bfloat16)
    b = torch.randn(width, generator=g) if bias else None
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))
    cos, sin = REF.rope_tables(pos, inv)
    slots = torch.tensor([int(table[r, (L - 1) // ps]) * ps + (L - 1) % ps for r, L in enumerate(lens)], dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    kp_ref, vp_ref = kp.float(), vp.float()
    want = REF.qkv_attention(x.float(), w.float(), b, cos, sin, slots, kp_ref, vp_ref, table, tseq, pos, nq, nkv, d, ps, scale, window,
                             max(lens), write_kv=True)   # the plain side always writes: with write off, the engine's cache holds them already
    kp_in, vp_in = (kp_ref.to(torch.bfloat16), vp_ref.to(torch.bfloat16)) if not write else (kp.clone(), vp.clone())
    if write:   # never written: the token's own slot and the rest of its page
        for r, L in enumerate(lens):
            page = int(table[r, (L - 1) // ps])
            kp_in[page, :, (L - 1) % ps:] = float("nan")
            vp_in[page, :, (L - 1) % ps:] = float("nan")
    kp_gpu, vp_gpu = kp_in.cuda(), vp_in.cuda()
    dev = [t.cuda() for t in (x, w, cos, sin, slots, table, tseq, pos)]
    for _ in range(2):
        before = K.launches
        got = K.qkv_attention(dev[0], dev[1], None if b is None else b.cuda(), dev[2], dev[3], dev[4], kp_gpu, vp_gpu, dev[5], dev[6], dev[7],
                              nq, nkv, d, ps, scale, window, max(lens), batch=_Batch(qlens), write_kv=write)
        K.check_device_errors()
        assert K.launches - before == 2 and K._dirty_qkv is not None     # the product and the attention, nothing else
        assert not torch.isnan(got).any()
        close(got, want, 1e-2)
        own_k = torch.stack([kp_gpu[int(s) // ps, :, int(s) % ps] for s in slots]).float().cpu()
        own_v = torch.stack([vp_gpu[int(s) // ps, :, int(s) % ps] for s in slots]).float().cpu()
        close(own_k, torch.stack([kp_ref[int(s) // ps, :, int(s) % ps] for s in slots]), 1e-2)
        close(own_v, torch.stack([vp_ref[int(s) // ps, :, int(s) % ps] for s in slots]), 1e-2)
        # the sums wait to be cleared by the next kernel that can do it on its way
        K.silu_mul(torch.randn(B, 64, device="cuda").to(torch.bfloat16))
        assert K._dirty_qkv is None and K._acc_qkv.abs().sum().item() == 0
    assert K._attn_counters is None or K._attn_counters.abs().sum().item() == 0


@pytest.mark.parametrize("nq,nkv,d,ps,lens,qlens,window", [
    (14, 2, 64, 16, [2048], [2048], 0),                       # the bench's prompt: 18 tokens x 7 heads per tile
    (14, 2, 64, 16, [3000], [40], 0),                         # a short portion far into a long request: few tiles, their keys in slices
    (4, 1, 64, 16, [1500, 700], [100, 5], 0),                 # slices, and a tile whose later slices are empty
    (14, 2, 64, 16, [300, 77, 500], [300, 1, 37], 0),        # a decode token and a late portion beside a prompt
    (8, 8, 64, 8, [700, 130], [700, 2], 0),                   # no grouping: 128 tokens per tile; pages of 8
    (16, 1, 64, 32, [257, 90], [257, 64], 0),                 # 16 heads on one key/value head
    (6, 3, 64, 64, [200, 1000], [200, 520], 48),              # window; a page is a whole chunk
    (12, 4, 64, 128, [640], [400], 0),                        # pages larger than a chunk
    (5, 5, 64, 16, [333], [333], 100),                        # window longer than a chunk
    (3, 1, 64, 16, [4500], [4500], 0),
    (12, 2, 128, 16, [2048], [2048], 0),                      # heads of 128: two blocks of 64 dims per operand, one block per SM
    (28, 4, 128, 16, [1500, 700], [100, 5], 0),               # 7 heads per group, slices, empty later slices
    (4, 1, 128, 16, [3000], [40], 0),                         # few tiles far into a long request: many slices
    (8, 8, 128, 8, [700, 130], [700, 2], 0),                  # pages of 8: all 32 lanes of the producer issue a box
    (12, 4, 128, 128, [640], [400], 0),                       # pages larger than a chunk
    (6, 3, 128, 64, [200, 1000], [200, 520], 48),             # window
    (12, 2, 128, 16, [300, 77, 500], [300, 1, 37], 0),
])
def test_paged_attention_tcgen05(K, monkeypatch, nq, nkv, d, ps, lens, qlens, window):
    """Prompt portions of head size 64 or 128 through tcgen05 and tensor memory. Every slot of the cache that no visible key
    occupies holds NaN (free pages, the null page, the rest of each request's last page): nothing of it may reach a result."""
    taken = []
    inner = K._attention_tc
    monkeypatch.setattr(K, "_attention_tc", lambda *a: (taken.append(inner(*a)), taken[-1])[1])
    for spike in (False, True):
        qkv, kp, vp, table, tseq, pos = _attention_case(torch.bfloat16, nq, nkv, d, ps, lens, qlens, window, 21, spike)
        used = torch.zeros(kp.shape[0], ps, dtype=torch.bool)
        for r, L in enumerate(lens):
            for i in range(L):
                used[int(table[r, i // ps]), i % ps] = True
        kp_nan, vp_nan = kp.clone(), vp.clone()
        kp_nan.permute(0, 2, 1, 3)[~used] = float("nan")
        vp_nan.permute(0, 2, 1, 3)[~used] = float("nan")
        scale = 1.0 / math.sqrt(d)
        want = REF.paged_attention(qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps, scale, window, max(lens))
        for _ in range(2):
            got = K.paged_attention(qkv.cuda(), kp_nan.cuda(), vp_nan.cuda(), table.cuda(), tseq.cuda(), pos.cuda(), nq, nkv, d, ps,
                                    scale, window, max(lens), batch=_Batch(qlens))
            K.check_device_errors()
            assert not torch.isnan(got).any()
            close(got, want, 1e-2)
    assert len(taken) == 4 and all(t is not None for t in taken)
    assert K._attn_counters is None or K._attn_counters.abs().sum().item() == 0  # the slice counters are back at zero


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("lens,qlens,splits", [([1500], [1500], None), ([1500, 900], [300, 64], None), ([1300], [40], 5)])
def test_paged_attention_tcgen05_when_the_maximum_keeps_growing(K, d, lens, qlens, splits):
    """The tcgen05 kernel takes P relative to a reference that follows a row's running maximum only when it lags by more
    than 2^8, and then scales the row's outputs down in tensor memory. Here the scores of the even heads climb along the
    sequence (by about 55 powers of two over 1,500 keys, so a row is rescaled every few chunks), those of the odd heads
    fall (never rescaled), and both kinds sit in the same warp."""
    nq, nkv, ps = 14, 2, 16
    qkv, kp, vp, table, tseq, pos = _attention_case(torch.bfloat16, nq, nkv, d, ps, lens, qlens, 0, 31)
    g = torch.Generator().manual_seed(32)
    u = torch.randn(d, generator=g)
    u /= u.norm()
    for r, L in enumerate(lens):
        for t in range(L):
            page, off = int(table[r, t // ps]), t % ps
            kp[page, :, off] = (kp[page, :, off].float() + u * (t / 40)).to(torch.bfloat16)
    q = qkv[:, :nq * d].view(-1, nq, d)
    sign = torch.tensor([8.0 if h % 2 == 0 else -8.0 for h in range(nq)]).view(1, nq, 1)
    q.copy_((q.float() + sign * u).to(torch.bfloat16))
    scale = 1.0 / math.sqrt(d)
    want = REF.paged_attention(qkv, kp, vp, table, tseq, pos, nq, nkv, d, ps, scale, 0, max(lens))
    for _ in range(2):
        got = K.paged_attention(qkv.cuda(), kp.cuda(), vp.cuda(), table.cuda(), tseq.cuda(), pos.cuda(), nq, nkv, d, ps, scale, 0,
                                max(lens), batch=_Batch(qlens), num_splits=splits)
        K.check_device_errors()
        close(got, want, 1e-2)


@pytest.mark.parametrize("M,N,K_,splits,accumulate", [
    (1, 128, 64, 1, False),
    (8, 1152, 896, 1, False),
    (8, 9728, 896, 3, True),         # 5 k-blocks per block: one more than the ring has stages
    (8, 1152, 896, 5, True),         # 3 k-blocks per block, the last block 2
    (33, 640, 960, 2, True),         # 8 k-blocks per block, two rounds of the ring
    (8, 896, 4864, 19, True),        # many blocks add into the same rows
    (64, 896, 896, 14, True),
    (40, 200, 72, 2, True),          # ragged: N and K are no multiples of the tile
    (17, 3000, 896, 1, False),
    (100, 384, 256, None, True),     # more rows than one token tile
    (5, 151936, 896, 1, False),      # the output head
])
def test_linear_tc(K, M, N, K_, splits, accumulate):
    g = torch.Generator().manual_seed(8)
    x = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) * 0.1).to(torch.bfloat16)
    base = torch.randn(M, N, generator=g)
    want = x.double() @ w.double().T + (base.double() if accumulate else 0)
    for _ in range(2):
        out = base.clone().cuda() if accumulate else None
        got = K.linear_tc(x.cuda(), w.cuda(), out=out, accumulate=accumulate, k_splits=splits)
        K.check_device_errors()
        close(got, want, 2e-5)


def test_linear_tc_into_a_strided_view(K):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(6, 128, generator=g).to(torch.bfloat16)
    w = torch.randn(130, 128, generator=g).to(torch.bfloat16)
    big = torch.zeros(6, 300, device="cuda")
    K.linear_tc(x.cuda(), w.cuda(), out=big[:, 20:150], accumulate=True, k_splits=2)
    K.check_device_errors()
    close(big[:, 20:150], x.double() @ w.double().T, 2e-5)
    assert big[:, :20].abs().sum() == 0 and big[:, 150:].abs().sum() == 0


def test_transient_products_are_consumed_and_cleared(K):
    """Small bfloat16 batches: the q/k/v and gate/up products are float32 sums of split-K blocks in the library's
    accumulation buffer; the kernels that read them leave the buffer zero for the next product."""
    g = torch.Generator().manual_seed(12)
    nq, nkv, d, ps, N, H, I = 14, 2, 64, 16, 8, 896, 4864
    x = torch.randn(N, H, generator=g).to(torch.bfloat16)
    wqkv = (torch.randn((nq + 2 * nkv) * d, H, generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn((nq + 2 * nkv) * d, generator=g)
    pos = torch.arange(100, 100 + N, dtype=torch.int32)
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))
    cos, sin = REF.rope_tables(pos, inv)
    slots = torch.arange(N, dtype=torch.int32) + 16
    kp, vp = torch.zeros(4, nkv, ps, d, dtype=torch.bfloat16), torch.zeros(4, nkv, ps, d, dtype=torch.bfloat16)
    ref_q = (x.float() @ wqkv.float().T)
    kp_ref, vp_ref = kp.clone().float(), vp.clone().float()
    REF.rope_kv_write(ref_q, bias, cos, sin, slots, kp_ref, vp_ref, nq, nkv, d, ps, True)
    for _ in range(2):
        acc = K.linear(x.cuda(), wqkv.cuda(), transient=True)
        assert acc.dtype == torch.float32 and K._is_transient(acc)
        kp_gpu, vp_gpu = kp.cuda(), vp.cuda()
        out = K.rope_kv_write(acc, bias.cuda(), cos.cuda(), sin.cuda(), slots.cuda(), kp_gpu, vp_gpu, nq, nkv, d, ps, True,
                              out_dtype=torch.bfloat16)
        assert out.dtype == torch.bfloat16 and K._acc.abs().sum().item() == 0
        close(out, ref_q, 8e-3)
        close(kp_gpu, kp_ref, 8e-3)
        close(vp_gpu, vp_ref, 8e-3)
    wgu = (torch.randn(2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    gu = K.linear(x.cuda(), wgu.cuda(), transient=True)
    assert K._is_transient(gu)
    a = K.silu_mul(gu, out_dtype=torch.bfloat16)
    assert K._acc.abs().sum().item() == 0
    close(a, REF.silu_mul(x.float() @ wgu.float().T), 8e-3)
    res = torch.randn(N, H, generator=g)
    wd = (torch.randn(H, I, generator=g) * 0.02).to(torch.bfloat16)
    r = res.clone().cuda()
    assert K.linear(a, wd.cuda(), add_to=r) is None
    close(r, res.double() + a.double().cpu() @ wd.double().T, 2e-5)
    K.check_device_errors()
