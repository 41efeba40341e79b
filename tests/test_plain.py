"""The plain implementation against the outputs of the reference's own model code (tests/golden/)."""
from pathlib import Path

import pytest
import torch

from helpers import make_model_folder
from plain_qwen2 import (plain_draw, plain_forward, plain_generate, plain_load, plain_logits_to_probs, plain_rmsnorm,
                         plain_rope_tables, plain_uniform)

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_outputs(tmp_path, name):
    gold = torch.load(GOLDEN / f"golden_{name}.pt")
    cfg, w = plain_load(make_model_folder(tmp_path, name))
    for p, logits, greedy, probs in zip(gold["prompts"], gold["logits"], gold["greedy"], gold["probs"]):
        mine = plain_forward(cfg, w, p)
        assert (mine - logits).abs().max() <= 1e-5
        assert plain_generate(cfg, w, p, 16) == greedy
        assert (plain_logits_to_probs(mine[-1], 0.8, 20, 0.9) - probs).abs().max() < 1e-6


def test_window_changes_only_what_it_should(tmp_path):
    cfg, w = plain_load(make_model_folder(tmp_path, "C"))
    p = list(range(5, 65))
    full = dict(cfg, use_sliding_window=False)
    a, b = plain_forward(cfg, w, p), plain_forward(full, w, p)
    assert torch.equal(a[:24], b[:24])          # inside the window nothing differs
    assert not torch.allclose(a[30:], b[30:])   # beyond it the upper layers see fewer keys


def test_parts():
    x = torch.randn(3, 8)
    y = plain_rmsnorm(x, torch.ones(8), 1e-6)
    assert torch.allclose(y.pow(2).mean(-1), torch.ones(3), atol=1e-4)
    cos, sin = plain_rope_tables(torch.arange(4), 8, 10000.0, torch.float32)
    assert cos.shape == (4, 8) and torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))
    assert torch.allclose(cos[:, :4], cos[:, 4:])


def test_sampling_rules():
    logits = torch.tensor([1.0, 3.0, 2.0, 0.0, -1.0])
    assert plain_draw(logits, 0.0, 0, 1.0, 0.9) == 1
    pr = plain_logits_to_probs(logits, 1.0, top_k=2)
    assert pr[0] == 0 and pr[3] == 0 and abs(float(pr.sum()) - 1) < 1e-6
    pr = plain_logits_to_probs(logits, 1.0, top_p=0.5)
    assert (pr > 0).sum() == 1 and pr[1] == 1.0     # the first token alone already holds more than half
    us = [plain_uniform(3, c) for c in range(2000)]
    assert 0 <= min(us) and max(us) < 1 and abs(sum(us) / len(us) - 0.5) < 0.03
    assert plain_uniform(3, 5) == plain_uniform(3, 5) != plain_uniform(4, 5)
    from llm_infrence_engine_b200.sampling import uniform_from
    assert all(uniform_from(s, c) == plain_uniform(s, c) for s in (0, 7, 2**40) for c in (0, 1, 99))
