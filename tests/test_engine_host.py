"""The host side of the engine on the CPU: step building, block tables, pages that are used again,
scheduler and entry point, with the kernels replaced by their plain torch statements
(tests/torch_kernels.py). What the CUDA kernels compute is checked by the gpu tests."""
import pytest
import torch

from helpers import cut, make_model_folder, random_prompt
from plain_qwen2 import plain_forward, plain_generate, plain_load
from tiny_configs import CONFIGS, PAGE_SIZES
from torch_kernels import TorchKernels

from llm_infrence_engine_b200.engine import Engine, Request, TraceReplayer

TOL = 2e-5


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {n: make_model_folder(tmp, n) for n in CONFIGS}


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_cuts_match_plain(folders, name):
    cfg, w = plain_load(folders[name])
    vocab = cfg["vocab_size"]
    prompts = {"a": random_prompt(vocab, 70, 1), "b": random_prompt(vocab, 45, 2), "c": random_prompt(vocab, 33, 3)}
    want = {k: plain_forward(cfg, w, p) for k, p in prompts.items()}
    rp = TraceReplayer(str(folders[name]), "float32", 192, device="cpu", kernels=TorchKernels(), block_size=PAGE_SIZES[name])
    # whole
    for k, p in prompts.items():
        got = rp.step({"step": 0, "entries": [{"id": k, "tokens": p, "want": list(range(len(p)))}], "end": [k]})
        assert (got - want[k]).abs().max() < TOL
        rp.cache.check_invariants()
    # portions of changing size, two requests interleaved, a third joining on pages given back
    live = {"a": cut(70, [16, 5, 2, 9]), "b": cut(45, [2, 7, 30])}
    step = 0
    got = {k: [] for k in prompts}
    while live:
        entries = []
        for k in list(live):
            lo, hi = live[k].pop(0)
            entries.append({"id": k, "tokens": prompts[k][lo:hi], "want": list(range(hi - lo))})
        end = [k for k in live if not live[k]]
        out = rp.step({"step": step, "entries": entries, "end": end})
        o = 0
        for e in entries:
            n = len(e["tokens"])
            got[e["id"]].append(out[o:o + n]); o += n
        for k in end:
            del live[k]
            if k == "b":
                live["c"] = cut(33, [1, 1, 31])
        rp.cache.check_invariants()
        step += 1
    for k in prompts:
        assert (torch.cat(got[k]) - want[k]).abs().max() < TOL, k
    assert all(p.num_free == p.capacity for p in rp.cache.pools)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_engine_greedy_matches_plain(folders, name):
    cfg, w = plain_load(folders[name])
    vocab = cfg["vocab_size"]
    prompts = [random_prompt(vocab, n, 10 + n) for n in (1, 7, 19, 33)]
    eng = Engine(str(folders[name]), dtype="float32", device="cpu", kernels=TorchKernels(), block_size=PAGE_SIZES[name],
                 num_blocks=14, max_seqs=3, max_len=64, max_num_batched_tokens=24)
    reqs = [eng.add_request(Request(p, max_new_tokens=8)) for p in prompts]
    while eng.has_work():
        eng.step()
        eng.cache.check_invariants()
    for r, p in zip(reqs, prompts):
        assert r.output_ids == plain_generate(cfg, w, p, 8), (name, len(p))
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)
    assert eng.cache.num_free_slots() == 3


def test_engine_sampled_matches_plain(folders):
    cfg, w = plain_load(folders["B"])
    prompts = [random_prompt(320, n, 20 + n) for n in (3, 12, 40)]
    eng = Engine(str(folders["B"]), dtype="float32", device="cpu", kernels=TorchKernels(), block_size=8,
                 num_blocks=40, max_seqs=4, max_len=128, max_num_batched_tokens=16)
    res = eng.generate(prompts, max_new_tokens=6, temperature=0.8, top_k=50, top_p=0.95, seed=7)
    for i, (r, p) in enumerate(zip(res, prompts)):
        assert r.token_ids == plain_generate(cfg, w, p, 6, temperature=0.8, top_k=50, top_p=0.95, seed=7 + i)


def test_prefix_cache_gives_the_same_tokens_and_computes_less(folders):
    """Requests that share leading tokens, with and without the prefix cache: same output, fewer prompt tokens computed;
    also through preemption (a preempted request finds its own pages again) and with pages evicted under pressure."""
    cfg, w = plain_load(folders["B"])
    stem = random_prompt(320, 37, 5)
    prompts = [stem + random_prompt(320, n, 60 + n) for n in (3, 9, 1, 14)] + [random_prompt(320, 21, 77), stem[:20]]
    out = {}
    for on in (False, True):
        eng = Engine(str(folders["B"]), dtype="float32", device="cpu", kernels=TorchKernels(), block_size=8, num_blocks=16,
                     max_seqs=3, max_len=96, max_num_batched_tokens=32, prefix_cache=on)
        reqs = [eng.add_request(Request(p, max_new_tokens=10)) for p in prompts]
        while eng.has_work():
            eng.step()
            eng.cache.check_invariants()
        out[on] = ([r.output_ids for r in reqs], eng.stats())
        assert all(pool.num_free == pool.capacity for pool in eng.cache.pools) and eng.cache.num_free_slots() == 3
    assert out[True][0] == out[False][0] == [plain_generate(cfg, w, p, 10) for p in prompts]
    off, on = out[False][1], out[True][1]
    assert not off["prefix_cache"] and off["prefix_tokens_hit"] == 0
    assert on["prefix_cache"] and on["prefix_tokens_hit"] >= 3 * 32
    assert on["prefill_tokens_computed"] < off["prefill_tokens_computed"]
    assert on["preemptions"] + off["preemptions"] > 0  # the pool is small enough that both runs had to preempt


def test_graph_buckets_and_warmup_without_graphs(folders):
    """Padded batch sizes of the decode graphs: 1, 2, 4, 8, 16, then in steps of half a power of two, the largest batch last;
    an engine without graphs has nothing to warm up."""
    from llm_infrence_engine_b200.engine.graphs import bucket_sizes

    assert bucket_sizes(1) == [1]
    assert bucket_sizes(6) == [1, 2, 4, 6]
    assert bucket_sizes(64) == [1, 2, 4, 8, 16, 24, 32, 48, 64]
    assert bucket_sizes(40) == [1, 2, 4, 8, 16, 24, 32, 40]
    assert bucket_sizes(100) == [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 100]
    for m in range(1, 200):
        b = bucket_sizes(m)
        assert b[-1] == m and b == sorted(set(b))
    folder = folders["A"][0] if isinstance(folders["A"], tuple) else folders["A"]
    eng = Engine(str(folder), kernels=TorchKernels(), device="cpu", dtype="float32", block_size=PAGE_SIZES["A"], num_blocks=20,
                 max_seqs=3, max_len=64)
    assert eng.warmup() == [] and eng.warmup([1, 2]) == []


def test_a_step_that_raises_loses_nothing(folders):
    """An exception in the middle of the step function (a simulated allocation failure inside the third layer call of one
    step) reaches the caller of ``Engine.step``; the engine is still usable: the caller cancels one request, the others go
    on and produce exactly the plain tokens, and in the end every page and slot is back. (The reference's analogue is its
    server's crash test, tests/test_server.py:173-189: it fails the requests and flips health; this engine can go on.)"""
    cfg, w = plain_load(folders["B"])
    prompts = [random_prompt(320, n, 30 + n) for n in (9, 21, 5)]

    class Failing(TorchKernels):
        def __init__(self):
            super().__init__()
            self.calls, self.fail_at = 0, None

        def paged_attention(self, *a, **kw):
            self.calls += 1
            if self.calls == self.fail_at:
                raise MemoryError("simulated: out of memory inside the step")
            return super().paged_attention(*a, **kw)

    K = Failing()
    eng = Engine(str(folders["B"]), dtype="float32", device="cpu", kernels=K, block_size=8, num_blocks=20, max_seqs=3,
                 max_len=64, max_num_batched_tokens=16)
    reqs = [eng.add_request(Request(p, max_new_tokens=10)) for p in prompts]
    for _ in range(4):
        eng.step()
    before = [list(r.output_ids) for r in reqs]
    computed = [r.num_computed for r in reqs]
    K.fail_at = K.calls + 2   # the second layer of the next step: the first layer's keys are already written
    with pytest.raises(MemoryError):
        eng.step()
    assert [list(r.output_ids) for r in reqs] == before and [r.num_computed for r in reqs] == computed
    eng.cache.check_invariants()
    eng.cancel(reqs[1])
    while eng.has_work():
        eng.step()
        eng.cache.check_invariants()
    assert reqs[1].finish_reason == "abort" and reqs[1].output_ids == before[1]
    for i in (0, 2):
        assert reqs[i].output_ids == plain_generate(cfg, w, prompts[i], 10) and reqs[i].finish_reason == "length"
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools) and eng.cache.num_free_slots() == 3
