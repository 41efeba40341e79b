"""Command line: ``python -m llm_infrence_engine_b200``.

The reference's only command line starts its HTTP server (src/miniserve/server.py:435-448); servers
are outside this engine, so the same option names drive an offline run instead: ``--model``,
``--dtype``, ``--device``, ``--max-len``, ``--max-seqs``, ``--num-blocks`` and ``--cuda-graphs`` mean
what they mean there, and the sampling options carry the names of the reference's request fields
(``max_new_tokens``, ``temperature``, ``top_k``, ``top_p``, ``seed``; src/miniserve/engine.py:34-40).
Prompts are token ids (the engine holds no tokenizer): ``--prompt-ids "1 2 3" --prompt-ids "4 5"``
or one prompt per line in ``--prompt-file``. ``--random-weights CONFIG.json`` first writes a model
folder with seeded random weights to ``--model``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m llm_infrence_engine_b200", description="Generate tokens with a Qwen2 model folder on one GPU.")
    ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-len", type=int, default=1024)
    ap.add_argument("--max-seqs", type=int, default=32, help="concurrent sequences")
    ap.add_argument("--num-blocks", type=int, default=None, help="pool size in pages (default: max_seqs * max_len / block_size)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--cuda-graphs", action="store_true", help="replay decode-only steps (and prompt steps of a recurring shape) from CUDA graphs")
    ap.add_argument("--warmup", action="store_true", help="with --cuda-graphs: capture the decode graphs of all batch sizes before the first request")
    ap.add_argument("--prefix-cache", action="store_true", help="requests take over cached pages that hold their leading tokens")
    ap.add_argument("--pipeline", action="store_true", help="launch a step before the tokens of the step before it have been read back")
    ap.add_argument("--prompt-ids", action="append", default=[], help="one prompt as space- or comma-separated token ids; repeatable")
    ap.add_argument("--prompt-file", help="file with one prompt of token ids per line")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None, help="sampling seed (prompt i draws with seed + i)")
    ap.add_argument("--eos-ids", default="", help="token ids that end a request")
    ap.add_argument("--random-weights", metavar="CONFIG_JSON", help="write --model from this config.json and --weights-seed first")
    ap.add_argument("--weights-seed", type=int, default=0)
    a = ap.parse_args(argv)

    def ids(text: str):
        return [int(t) for t in text.replace(",", " ").split()]

    if a.random_weights:
        from .weights import write_random_model

        write_random_model(json.loads(Path(a.random_weights).read_text()), a.model, a.weights_seed,
                           "bfloat16" if a.dtype == "bfloat16" else "float32")
    prompts = [ids(p) for p in a.prompt_ids]
    if a.prompt_file:
        prompts += [ids(line) for line in Path(a.prompt_file).read_text().splitlines() if line.strip()]
    if not prompts:
        if a.random_weights:
            print(f"wrote {a.model}")
            return 0
        ap.error("no prompt: give --prompt-ids or --prompt-file")

    from .engine import Engine

    eng = Engine(a.model, dtype=a.dtype, device=a.device, max_len=a.max_len, max_seqs=a.max_seqs, num_blocks=a.num_blocks,
                 block_size=a.block_size, max_num_batched_tokens=a.max_batched_tokens, cuda_graphs=a.cuda_graphs, pipeline=a.pipeline, prefix_cache=a.prefix_cache)
    if a.warmup:
        eng.warmup()
    results = eng.generate(prompts, a.max_new_tokens, ids(a.eos_ids), a.temperature, a.top_k, a.top_p, a.seed)
    for r in results:
        print(json.dumps({"prompt_len": r.prompt_len, "token_ids": r.token_ids, "finish_reason": r.finish_reason,
                          "ttft_s": round(r.ttft, 6), "decode_tok_s": round(r.decode_tps, 1)}))
    print(json.dumps({"stats": eng.stats()}), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
