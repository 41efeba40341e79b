"""Compare the plain implementation (tests/plain_qwen2.py) ONCE with the reference's own model code
on the CPU, and store the reference's small outputs next to this script.

Run from the repository root with the reference project's ``src`` folder given:

    python tests/golden/make_golden.py /path/to/reference/src

It writes tiny random models A and B (tests/tiny_configs.py) into a temporary folder, loads them
into the reference's ``Qwen2`` (``ModelConfig.from_json`` + ``load_state_dict``), runs the
reference's full-sequence forward, its ``generate()`` and its ``logits_to_probs``, checks that the
plain implementation agrees (max |difference| <= 1e-5 on logits, equal greedy tokens, 1e-6 on
probabilities) and stores the reference's outputs in ``golden_A.pt`` / ``golden_B.pt``.
``tests/test_plain.py`` compares the plain implementation with these files on every run, so the
reference does not have to be present then.
"""
import json
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

from plain_qwen2 import plain_forward, plain_generate, plain_load, plain_logits_to_probs  # noqa: E402
from tiny_configs import CONFIGS, SEEDS  # noqa: E402

PROMPT_LENS = {"A": [1, 7, 19, 33], "B": [3, 12, 40, 64, 97]}


def prompts_for(name: str, vocab: int):
    g = torch.Generator().manual_seed(100 + SEEDS[name])
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in PROMPT_LENS[name]]


def main(ref_src: str) -> None:
    sys.path.insert(0, ref_src)
    from miniserve.generate import generate  # the reference's own code
    from miniserve.model import ModelConfig, Qwen2
    from miniserve.sampler import logits_to_probs
    from safetensors.torch import load_file

    from llm_infrence_engine_b200.weights import write_random_model

    for name in ("A", "B"):
        cfg = CONFIGS[name]
        with tempfile.TemporaryDirectory() as d:
            write_random_model(cfg, d, SEEDS[name], "float32")
            rcfg = ModelConfig.from_json(Path(d) / "config.json")
            with torch.device("meta"):
                model = Qwen2(rcfg)
            model.load_state_dict(load_file(str(Path(d) / "model.safetensors")), strict=False, assign=True)
            if rcfg.tie_word_embeddings:
                model.lm_head.weight = model.model.embed_tokens.weight
            model = model.eval()
            pcfg, w = plain_load(d)
            out = {"prompts": prompts_for(name, cfg["vocab_size"]), "logits": [], "greedy": [], "probs": []}
            worst = 0.0
            for p in out["prompts"]:
                with torch.inference_mode():
                    ref = model(torch.tensor([p]))[0].float()
                mine = plain_forward(pcfg, w, p)
                worst = max(worst, (ref - mine).abs().max().item())
                assert torch.equal(ref.argmax(-1), mine.argmax(-1))
                out["logits"].append(ref.clone())
                toks = generate(model, p, 16).token_ids
                assert toks == plain_generate(pcfg, w, p, 16), "greedy tokens differ"
                out["greedy"].append(toks)
                pr = logits_to_probs(ref[-1], 0.8, 20, 0.9)
                assert (pr - plain_logits_to_probs(mine[-1], 0.8, 20, 0.9)).abs().max().item() < 1e-6
                out["probs"].append(pr.clone())
            assert worst <= 1e-5, worst
            torch.save(out, HERE / f"golden_{name}.pt")
            print(f"tiny {name}: plain vs reference max |dlogits| = {worst:.3g}; greedy tokens and probabilities agree; "
                  f"wrote golden_{name}.pt")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py REFERENCE_SRC_FOLDER")
    main(sys.argv[1])
