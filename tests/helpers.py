"""Shared by the tests: tiny model folders in temporary places, prompts, and replay cuts."""
from __future__ import annotations

import random
from pathlib import Path

import torch

from tiny_configs import CONFIGS, SEEDS


def make_model_folder(tmp: Path, name: str, store_dtype: str = "float32") -> Path:
    from llm_infrence_engine_b200.weights import write_random_model

    return write_random_model(CONFIGS[name], Path(tmp) / f"tiny_{name}_{store_dtype}", SEEDS[name], store_dtype)


def random_prompt(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def cut(n: int, sizes) -> list:
    """Cut ``n`` tokens into portions whose sizes cycle through ``sizes``; the rest goes to the last one."""
    out, i, k = [], 0, 0
    while i < n:
        s = min(sizes[k % len(sizes)], n - i)
        out.append((i, i + s))
        i += s
        k += 1
    return out
