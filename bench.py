"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen2.5-0.5B (24 layers, hidden 896, 14 query / 2 key-value
heads of 64, intermediate 4864, vocabulary 151936, tied head) with random weights in bfloat16, a
batch of 8 requests and a context of 8192 tokens. A "step" is one decode step of the whole batch.

``value``     decoded tokens per second of the step function alone: W warm-up steps, then K steps
              between two CUDA events on the launching stream with a synchronize on both sides.
              The requests' cache pages hold synthetic keys and values (a step's cost does not
              depend on them); weights plus cache are far larger than L2, so nothing is flushed.
``e2e``       the same through ``Engine.step()``: requests are added as token lists on the host,
              their prompts are prefilled by the engine, and every timed step copies its inputs
              from pinned host memory and reads sampled tokens back (the engine runs pipelined: a
              step is launched before the tokens of the step before it have been read).
``prefill``   one prompt of 2,048 tokens in one step (device time between two events, median of five runs after three
              warm-up runs; a step shape that recurs is replayed from a CUDA graph, as in serving);
              ``frac`` = flops / time / bfloat16 peak.
``roofline``  bytes a decode step must read (every weight once + the live requests' cache) / its time.
``points``    decode tokens per second at batch 1 and 64, same method as ``value``.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else 6.65 TB/s and 1.59 PFLOP/s.
More than one GPU is outside this engine: ``--gpus N`` with N > 1 prints one line and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 151936, "hidden_size": 896,
    "intermediate_size": 4864, "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "use_sliding_window": False, "hidden_act": "silu",
}
CONTEXT = 8192
PREFILL_TOKENS = 2048
BLOCK = 16

# Other layer sizes of the same architecture (``--shape``): what changes against MODEL, and the context length they are quoted at.
SHAPES = {
    "0.5b": ("Qwen2.5-0.5B shape", {}, 8192),
    "1.5b": ("Qwen2.5-1.5B shape", {"hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 28, "num_attention_heads": 12,
                                    "num_key_value_heads": 2}, 8192),
    "7b": ("Qwen2.5-7B shape", {"vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
                                "num_attention_heads": 28, "num_key_value_heads": 4, "tie_word_embeddings": False}, 16384),
}


def peaks() -> dict:
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            if d.get("hbm_gbs"):
                out["hbm_gbs"] = float(d["hbm_gbs"])
            if d.get("bf16_tflops"):
                out["bf16_tflops"] = float(d["bf16_tflops"])
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            out["source"] = "measured"
        except (ValueError, OSError):
            pass
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of GPU 0 every 100 ms while running."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons}


def flops_prefill(T: int) -> float:
    m = MODEL
    d = m["hidden_size"] // m["num_attention_heads"]
    per_layer = (m["hidden_size"] * (m["num_attention_heads"] + 2 * m["num_key_value_heads"]) * d
                 + m["num_attention_heads"] * d * m["hidden_size"] + 3 * m["hidden_size"] * m["intermediate_size"])
    linear = 2.0 * T * per_layer * m["num_hidden_layers"]
    attn = m["num_hidden_layers"] * 4.0 * m["num_attention_heads"] * d * (T * (T + 1) / 2)
    head = 2.0 * m["hidden_size"] * m["vocab_size"]
    return linear + attn + head


REF_DIR = ROOT / "baseline" / "_ref"


def _reference_model(folder: Path, torch):
    """The reference's own model from a model folder, built the way its loader does (src/miniserve/loader.py:36-48:
    ``ModelConfig.from_json``, ``Qwen2`` on the meta device, ``load_state_dict(assign=True)``, the tie re-established), without the
    tokenizer and the download that ``load_model`` adds."""
    from miniserve.model import ModelConfig, Qwen2
    from safetensors.torch import load_file

    cfg = ModelConfig.from_json(folder / "config.json")
    with torch.device("meta"):
        model = Qwen2(cfg)
    state = {}
    for f in sorted(folder.glob("*.safetensors")):
        state.update(load_file(f))
    model.load_state_dict(state, strict=False, assign=True)
    if cfg.tie_word_embeddings:
        model.lm_head.weight = model.model.embed_tokens.weight
    return model.to(device="cuda:0", dtype=torch.bfloat16).eval()


def _reference_decode(model, torch, kind: str, batch: int, steps: int, warmup: int) -> dict:
    """``steps`` decode steps of ``batch`` requests whose contexts reach CONTEXT, through the reference's public calls
    (``add_request`` / ``step``, src/miniserve/engine.py:143-205, paged_engine.py:57-66). ``kind``: "graphs" is its
    ``Engine(cuda_graphs=True)`` on the slot cache (its fastest decode, docs/RESULTS.md:38-40), "paged" its ``PagedEngine``."""
    from miniserve.engine import Engine, Request
    from miniserve.paged_engine import PagedEngine

    total = steps + warmup + 8
    prompt_len = CONTEXT - total
    max_len = CONTEXT + 8
    if kind == "graphs":
        eng = Engine(model, max_slots=batch, max_len=max_len, policy="continuous", max_prefills_per_step=batch, cuda_graphs=True)
    else:
        per_seq = -(-max_len // BLOCK)
        eng = PagedEngine(model, num_blocks=batch * (per_seq + 1) + 1, block_size=BLOCK, max_seqs=batch, max_len=max_len,
                          enable_prefix_cache=False, max_prefills_per_step=batch)
    g = torch.Generator().manual_seed(9)
    reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=g).tolist(), max_new_tokens=total))
            for _ in range(batch)]
    t0 = time.perf_counter()
    eng.step()  # admits and prefills every request (one forward each), no decode yet
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    assert len(eng.running) == batch, f"the reference admitted {len(eng.running)} of {batch} requests"
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    before = sum(len(r.output_ids) for r in reqs)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        eng.step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    made = sum(len(r.output_ids) for r in reqs) - before
    ms = start.elapsed_time(stop) / steps
    del eng
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": made / (ms * steps) * 1e3, "e2e_tok_s": made / wall, "e2e_ms": wall / steps * 1e3,
            "prefill_s": round(prefill_s, 2), "made": made}


def _reference_prefill(model, torch, reps: int = 5) -> dict:
    from miniserve.paged_engine import PagedEngine
    from miniserve.engine import Request

    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, MODEL["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    eng = PagedEngine(model, num_blocks=PREFILL_TOKENS // BLOCK + 4, block_size=BLOCK, max_seqs=1, max_len=PREFILL_TOKENS + 1,
                      enable_prefix_cache=False)
    times = []
    for i in range(reps + 3):
        eng.add_request(Request(prompt, max_new_tokens=1))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        eng.step()  # prefill of the whole prompt and its first token; the request ends with it
        stop.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(stop))
    return {"ms": sorted(times)[len(times) // 2]}


def reference_arm(a) -> int:
    """The reference itself, unmodified, for the same metric: its model class and its engines from ``baseline/_ref`` (a copy
    of its pure-Python package ``src/miniserve``: what installing its wheel puts into a target folder; building that
    wheel needs the backend ``hatchling``, which the offline wheelhouse lacks). Nothing of this repository's engine, model or
    kernels is on this path; only the writer of the random-weights folder is shared, so that both arms load the same file."""
    if not (REF_DIR / "miniserve" / "paged_engine.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/miniserve (the unmodified copy of the reference's package) is not there"}))
        return 0
    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU only"}))
        return 0
    sys.path.insert(0, str(REF_DIR))
    import torch

    from llm_infrence_engine_b200.weights import write_random_model  # the folder writer only

    steps, warmup = a.steps, max(a.warmup, 3)
    pk = peaks()
    sampler = ClockSampler()
    try:
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(dict(MODEL), Path(tmp) / "model", seed=0, store_dtype="bfloat16")
            model = _reference_model(folder, torch)
        sampler.start()
        runs = {}
        for kind in ("graphs", "paged"):
            try:
                runs[kind] = _reference_decode(model, torch, kind, a.batch, steps, warmup)
            except Exception as e:  # one of its two engines failing leaves the other
                runs[kind] = {"error": f"{type(e).__name__}: {e}"[:300]}
        clocks = sampler.stop()
        ok = {k: v for k, v in runs.items() if "error" not in v}
        if not ok:
            print(json.dumps({"impl": "reference", "unavailable": "both of the reference's engines failed: " + json.dumps(runs)}))
            return 0
        best = max(ok, key=lambda k: ok[k]["tok_s"])
        main_pt = ok[best]
        points = {}
        for name, b, n in (("decode_b1", 1, min(steps, 64)), ("decode_b64", 64, min(steps, 16))):
            try:
                points[name] = round(_reference_decode(model, torch, "paged" if b > 8 else best, b, n, 3)["tok_s"], 1)
            except Exception as e:
                points[name] = None
                points[name + "_error"] = f"{type(e).__name__}: {e}"[:200]
        try:
            pre = _reference_prefill(model, torch)
        except Exception as e:
            pre = None
            points["prefill_error"] = f"{type(e).__name__}: {e}"[:200]
    finally:
        if sampler.proc is not None and sampler.proc.poll() is None:
            sampler.stop()
    fl = flops_prefill(PREFILL_TOKENS)
    cache_bytes = a.batch * CONTEXT * MODEL["num_hidden_layers"] * 2 * MODEL["num_key_value_heads"] * 64 * 2
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    achieved = (weight_bytes + cache_bytes) / (main_pt["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} (Qwen2.5-0.5B shape, bf16, random weights)",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0), uniform random token ids; contexts filled by the reference's own prefill",
        "impl": "reference",
        "config": {"model": "Qwen2.5-0.5B shape", "layers": MODEL["num_hidden_layers"], "layers_of_model": MODEL["num_hidden_layers"],
                   "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"],
                   "head_dim": 64, "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"], "tied": True,
                   "global_batch": a.batch, "seq_len": CONTEXT, "block_size": BLOCK, "parallelism": "single GPU",
                   "cuda_graphs": best == "graphs", "engine": "Engine(cuda_graphs=True), slot cache" if best == "graphs" else "PagedEngine",
                   "l2": "inputs larger than L2 (weights + cache per step >> 126 MB), no flush", "peaks": pk["source"]},
        "clocks": clocks,
        "gpu_launches": 0,
        "engines": {k: ({"tok_s": round(v["tok_s"], 1), "ms_per_step": round(v["ms"], 3), "prefill_s": v["prefill_s"]} if "error" not in v else v)
                    for k, v in runs.items()},
        "prefill": None if pre is None else {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                             "ms": round(pre["ms"], 3), "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "e2e": {"value": round(main_pt["e2e_tok_s"], 2), "unit": "tokens/s", "h2d_bytes_per_step": 16 * a.batch, "d2h_bytes_per_step": 8 * a.batch,
                "ms_per_step": round(main_pt["e2e_ms"], 3), "prefill_s": main_pt["prefill_s"]},
    }
    print(json.dumps(line))
    return 0


def check_decode_step(runner, entries, graph_logits, graph_tokens, torch) -> dict:
    """Outside the timed region: is what the captured step computes right?

    (a) The attention of this very shape (these block tables, contexts and pools, the planner's own number of key slices
    and way of merging them) against another kernel altogether: the generic one (one thread per key, 32-bit arithmetic,
    slices at fixed places), on random queries. Bound: 1e-2 of the largest output, the bound of the kernels' own tests.
    (b) The whole step again eagerly, kernel by kernel, and with the generic attention. The logits of two runs of the
    same bfloat16 step are not bit-equal: split-K partial sums meet by atomic additions in whatever order they arrive, the
    last bits of a sum decide how some activations round to bfloat16, and a deep model with random weights carries such
    a flip through to the logits (two replays of one graph were measured 1e-2 of the logits' scale apart at 24 layers, 1e-3
    at 2, and exactly equal with split-K off). So (b) is a coarse bound, 4e-2 of the scale, and the graph's tokens must be
    the eager argmax wherever the two best logits are clearly apart."""
    K = runner.K
    ctx, rows = runner.make_context(entries)
    eager = runner.forward(ctx, rows).float()
    slices = int(K.last_attention_plan[0])
    mixer = runner.spec.layers[runner.spec.schedule[0].layer].mixer
    bind = runner.bindings[runner.spec.schedule[0].cache]
    g = torch.Generator(device="cuda").manual_seed(3)
    width = (mixer.num_heads + 2 * mixer.num_kv_heads) * mixer.head_dim
    qkv = torch.randn((ctx.num_tokens, width), generator=g, device="cuda").to(torch.bfloat16)
    args = (qkv, bind.k, bind.v, ctx.block_tables[bind.group], ctx.token_seq, ctx.positions, mixer.num_heads, mixer.num_kv_heads,
            mixer.head_dim, ctx.page_size, mixer.scale, mixer.window or 0, ctx.max_context)
    fast = K.paged_attention(*args, batch=ctx).float()
    plain = K.paged_attention(*args).float()   # without the step's description the generic kernel runs
    d_attn = float((fast - plain).abs().max()) / max(float(plain.abs().max()), 1e-30)
    ctx._tables.clear()
    was = K.use_mma_attention
    K.use_mma_attention = False
    try:
        generic = runner.forward(ctx, rows).float()
    finally:
        K.use_mma_attention = was
    scale = max(1.0, float(eager.abs().max()))
    d_eager = float((graph_logits - eager).abs().max()) / scale
    d_generic = float((graph_logits - generic).abs().max()) / scale
    top2 = eager.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4 * float((graph_logits - eager).abs().max())
    same = graph_tokens.long() == eager.argmax(-1)
    ok = bool(d_attn <= 1e-2 and d_eager <= 4e-2 and d_generic <= 4e-2 and bool((same | ~clear).all())
              and bool(torch.isfinite(graph_logits).all()))
    return {"checked": ok, "attention_vs_generic_kernel": round(d_attn, 5), "graph_vs_eager": round(d_eager, 5),
            "vs_generic_attention": round(d_generic, 5), "tokens_equal": int(same.sum()), "rows": int(same.numel()),
            "attention_slices": slices}


def decode_point(folder: Path, batch: int, steps: int, warmup: int, torch, graphs: bool = True, sampler=None) -> dict:
    """Device time of ``steps`` decode steps of ``batch`` requests at CONTEXT tokens: the step function
    (replayed from its CUDA graph unless ``graphs`` is off) plus the argmax over its logits."""
    from llm_infrence_engine_b200.config import EngineConfig
    from llm_infrence_engine_b200.engine import StepEntry, build_runner

    per_seq = -(-(CONTEXT + 8) // BLOCK)
    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=batch * per_seq + 1, max_seqs=batch, max_len=CONTEXT + 8,
                       max_num_batched_tokens=max(batch, 16), cuda_graphs=graphs)
    spec, cache, runner = build_runner(folder, cfg)
    K = runner.K
    for b in runner.bindings:
        b.k.normal_(0, 0.5)
        b.v.normal_(0, 0.5)
    entries = []
    for i in range(batch):
        cache.admit(i)
        cache.reserve(i, 0, CONTEXT)
        entries.append(StepEntry(i, [(17 * i + 3) % MODEL["vocab_size"]], CONTEXT - 1, (0,)))
    check = None
    if graphs:
        runner.step(entries)  # captures the graph for this batch size and leaves the step's inputs in its static buffer
        cap = runner.graphs.captured[batch]
        per_step = cap.launches  # the captured step ends with the argmax over its logits
        check = check_decode_step(runner, entries, cap.logits[:batch].clone(), cap.tokens[:batch].clone(), torch)

        def one():
            cap.graph.replay()
            return cap.tokens
    else:
        ctx, rows = runner.make_context(entries)
        n0 = K.launches

        def one():
            ctx._tables.clear()
            return K.argmax(runner.forward(ctx, rows))

        one()
        per_step = K.launches - n0

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
        for _ in range(min(steps, 200)):  # bring the clocks up before the samples count
            one()
        torch.cuda.synchronize()
        sampler.rows.clear()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    if sampler is not None:
        sampler.clocks = sampler.stop()
    K.check_device_errors()  # a kernel that gave up on a bounded wait would have left invalid logits behind
    out = {"ms": ms, "tok_s": batch / ms * 1e3, "launches": per_step * steps, "check": check,
           "bytes": runner.weight_bytes_per_step() + batch * CONTEXT * runner.kv_bytes_per_token}
    del runner, spec, cache
    torch.cuda.empty_cache()
    return out


def prefill_point(folder: Path, torch, reps: int = 5, graphs: bool = True) -> dict:
    from llm_infrence_engine_b200.config import EngineConfig
    from llm_infrence_engine_b200.engine import StepEntry, build_runner

    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=PREFILL_TOKENS // BLOCK + 2, max_seqs=1,
                       max_len=PREFILL_TOKENS, max_num_batched_tokens=PREFILL_TOKENS, cuda_graphs=graphs)
    spec, cache, runner = build_runner(folder, cfg)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, MODEL["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(reps + 3):  # the first three runs are warm-up: with graphs the step's shape is captured at its third coming
        cache.admit("p")
        cache.reserve("p", 0, PREFILL_TOKENS)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, 0, (PREFILL_TOKENS - 1,))])
        stop.record()
        torch.cuda.synchronize()
        cache.free("p")
        if i >= 3:
            times.append(start.elapsed_time(stop))
    ms = sorted(times)[len(times) // 2]
    del runner, spec, cache
    torch.cuda.empty_cache()
    return {"ms": ms}


def e2e_point(folder: Path, batch: int, steps: int, warmup: int, torch, graphs: bool = True) -> dict:
    """``Engine.step()`` in a loop: host token lists in, sampled tokens out, after the engine prefilled the prompts itself."""
    from llm_infrence_engine_b200.engine import Engine, Request

    total = steps + warmup + 96  # nobody finishes before the timed steps, even the request that was admitted first
    prompt_len = CONTEXT - total
    per_seq = -(-(CONTEXT + 8) // BLOCK)
    eng = Engine(str(folder), dtype="bfloat16", block_size=BLOCK, num_blocks=batch * per_seq + 1, max_seqs=batch,
                 max_len=CONTEXT + 8, max_num_batched_tokens=2048, cuda_graphs=graphs, pipeline=True)
    g = torch.Generator().manual_seed(9)
    reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=g).tolist(), max_new_tokens=total))
            for _ in range(batch)]
    t0 = time.perf_counter()
    while any(r.num_computed < prompt_len for r in reqs) or any(len(r.output_ids) < 1 for r in reqs):
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    before = sum(len(r.output_ids) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(r.output_ids) for r in reqs) - before
    h2d = eng.runner.last_h2d_bytes
    return {"value": made / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
            "ms_per_step": dt / steps * 1e3, "prefill_s": round(prefill_s, 2)}


def serving_point(folder: Path, torch, n_requests: int, seed: int, budget: int, passes: int = 2) -> dict:
    """Continuous batching of ``n_requests`` requests that all arrive at once: prompt lengths uniform in [128, 2048], output
    lengths uniform in [64, 512] (seeded), through ``Engine`` with graphs captured up front (``warmup()``), the pipelined
    engine and a token budget per step. The workload is run ``passes`` times on fresh engines; the last pass counts (the
    first also pays for loading the CUDA library and the first captures). The reference's counterpart is its burst benchmark
    (benchmarks/bench_batching.py: every request at once, throughput = generated tokens / wall time)."""
    import random

    from llm_infrence_engine_b200.engine import Engine, Request

    rng = random.Random(seed)
    spec = [(rng.randint(128, 2048), rng.randint(64, 512)) for _ in range(n_requests)]
    max_len = 2048 + 512 + 16
    out = None
    for _ in range(passes):
        eng = Engine(str(folder), dtype="bfloat16", block_size=BLOCK, max_seqs=n_requests, max_len=max_len,
                     num_blocks=n_requests * (-(-max_len // BLOCK)) + 1, max_num_batched_tokens=budget, cuda_graphs=True, pipeline=True)
        t0 = time.perf_counter()
        eng.warmup()
        torch.cuda.synchronize()
        warm_s = time.perf_counter() - t0
        g = torch.Generator().manual_seed(seed + 1)
        reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (p,), generator=g).tolist(), max_new_tokens=o, ignore_eos=True))
                for p, o in spec]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.run_until_idle()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        made = sum(len(r.output_ids) for r in reqs)
        prompt = sum(p for p, _ in spec)
        dec = [s for s in eng.steps if s.num_prefill_tokens == 0 and s.decode_batch]
        mix = [s for s in eng.steps if s.num_prefill_tokens > 0]
        ttft = sorted((r.first_token_time - r.arrival_time) for r in reqs if r.first_token_time is not None)
        out = {"output_tok_s": round(made / dt, 1), "total_tok_s": round((made + prompt) / dt, 1), "wall_s": round(dt, 3),
               "requests": n_requests, "prompt_tokens": prompt, "output_tokens": made, "steps": len(eng.steps),
               "decode_only_steps": len(dec), "decode_only_ms": round(1e3 * sum(s.duration for s in dec) / max(1, len(dec)), 3),
               "mean_decode_batch": round(sum(s.decode_batch for s in dec) / max(1, len(dec)), 1),
               "steps_with_prompt_tokens": len(mix), "prompt_step_ms": round(1e3 * sum(s.duration for s in mix) / max(1, len(mix)), 3),
               "ttft_mean_s": round(sum(ttft) / max(1, len(ttft)), 3), "ttft_p95_s": round(ttft[int(0.95 * (len(ttft) - 1))], 3) if ttft else None,
               "preemptions": eng.stats()["preemptions"], "graph_warmup_s": round(warm_s, 2), "token_budget": budget}
        assert all(len(r.output_ids) == o for r, (_, o) in zip(reqs, spec))
        del eng
        torch.cuda.empty_cache()
    return out


def main() -> int:
    global CONTEXT, PREFILL_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="0.5b", choices=sorted(SHAPES), help="layer sizes (the default is the one the headline is quoted on)")
    ap.add_argument("--context", type=int, default=0, help="context length of the decode steps (default: the shape's own)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step from the host instead of replaying a CUDA graph")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"], help="measure one part only (for profiling); the JSON line then lacks the rest")
    ap.add_argument("--workload", default="steps", choices=["steps", "serving"],
                    help="serving: continuous batching of --requests requests (prompts U[128,2048], outputs U[64,512]) through Engine")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--token-budget", type=int, default=2048, help="serving: tokens per step (max_num_batched_tokens)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    PREFILL_TOKENS = a.prefill_tokens
    shape_name, changes, shape_context = SHAPES[a.shape]
    MODEL.update(changes)
    CONTEXT = a.context or shape_context
    a.layers = a.layers or MODEL["num_hidden_layers"]
    a.warmup = max(a.warmup, 3)
    graphs = not a.no_graphs

    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    model = dict(MODEL)
    model["num_hidden_layers"] = a.layers
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(model, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
        sampler = ClockSampler()
        if a.workload == "serving":
            sampler.start()
            res = serving_point(folder, torch, a.requests, 0, a.token_budget)
            print(json.dumps({"metric": f"output tok/s, continuous batching of {a.requests} requests ({shape_name}, bf16, random weights)",
                              "value": res["output_tok_s"], "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16",
                              "config": {"model": shape_name, "layers": a.layers, "layers_of_model": MODEL["num_hidden_layers"],
                                         "prompts": "U[128,2048]", "outputs": "U[64,512]", "seed": 0, "block_size": BLOCK},
                              "clocks": sampler.stop(), "serving": res}))
            return 0
        if a.only == "prefill":  # for profiling the prompt step alone: no decode step runs before it
            pre = prefill_point(folder, torch, graphs=graphs)
            fl = flops_prefill(PREFILL_TOKENS) * a.layers / MODEL["num_hidden_layers"]
            print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                          "ms": round(pre["ms"], 3),
                                          "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
                              "layers": a.layers, "cuda_graphs": graphs}))
            return 0
        main_pt = decode_point(folder, a.batch, a.steps, a.warmup, torch, graphs, sampler)
        clocks = sampler.clocks
        b1 = decode_point(folder, 1, min(a.steps, 256), a.warmup, torch, graphs) if a.only == "all" else None
        b64 = decode_point(folder, 64, min(a.steps, 128), a.warmup, torch, graphs) if a.only == "all" else None
        pre = prefill_point(folder, torch, graphs=graphs) if a.only == "all" else None
        e2e = None if (a.skip_e2e or a.only != "all") else e2e_point(folder, a.batch, min(a.steps, 512), a.warmup, torch, graphs)

    fl = flops_prefill(PREFILL_TOKENS) * a.layers / MODEL["num_hidden_layers"]
    achieved = main_pt["bytes"] / (main_pt["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} ({shape_name}, bf16, random weights)",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
        "impl": "ours",
        "config": {"model": shape_name, "layers": a.layers, "layers_of_model": MODEL["num_hidden_layers"],
                   "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"],
                   "head_dim": MODEL["hidden_size"] // MODEL["num_attention_heads"], "intermediate": MODEL["intermediate_size"],
                   "vocab": MODEL["vocab_size"], "tied": MODEL["tie_word_embeddings"], "global_batch": a.batch, "seq_len": CONTEXT, "block_size": BLOCK, "parallelism": "single GPU",
                   "cuda_graphs": graphs, "l2": "inputs larger than L2 (weights + cache per step >> 126 MB), no flush", "peaks": pk["source"]},
        "clocks": clocks,
        "gpu_launches": main_pt["launches"],
        "prefill": None if pre is None else {
            "value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
            "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": None if b1 is None else {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1)},
        "checked": {"decode_b%d" % a.batch: main_pt["check"], **({} if b1 is None else {"decode_b1": b1["check"], "decode_b64": b64["check"]})},
    }
    if e2e is not None:
        line["e2e"] = {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
