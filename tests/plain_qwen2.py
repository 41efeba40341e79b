"""Plain, slow implementation of the dense Qwen2 decoder, written from the reference's formulas.

Whole sequences, no cache, one function per part, torch on the CPU. It shares no code with the
package under test: it reads ``config.json`` as a plain dict and the weights by their checkpoint
names. Every function cites the lines of the reference (paths inside the reference project) whose
arithmetic it restates.

``tests/golden/make_golden.py`` compares this file once with the reference's own model code on the
CPU and stores the small outputs; ``tests/test_plain.py`` checks them on every run.

Two things here have no counterpart in the reference and rest on the formulas alone: the sliding
window of ``plain_attention`` (``window``), and the counter-based random numbers of
``plain_uniform`` that the sampler draws with.

``store`` (default: nothing) is applied wherever the engine under test keeps an activation in its
compute dtype: the normed rows, the rotated queries and keys, the values, the softmax weights, the
attention's output, the gated activation, and the two results that are added to the residual stream
(which itself, like the logits, stays 32-bit). With ``store=bf16_store`` the plain model shows how much
bfloat16 storage alone moves the logits of a given model, which is what the bfloat16 tests measure
the engine against.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ----------------------------------------------------------------------------- configuration
def plain_config(cfg: dict) -> dict:
    """The constants the formulas need, with the reference's defaults (src/miniserve/model.py:42-58)."""
    rope = cfg.get("rope_theta")
    if rope is None:
        rope = cfg.get("rope_parameters", {}).get("rope_theta", 10000.0)  # model.py:45-47
    heads = cfg["num_attention_heads"]
    out = {
        "vocab": cfg["vocab_size"],
        "hidden": cfg["hidden_size"],
        "inter": cfg["intermediate_size"],
        "layers": cfg["num_hidden_layers"],
        "heads": heads,
        "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg.get("head_dim") or cfg["hidden_size"] // heads,  # model.py:38-40 derives it
        "eps": cfg["rms_norm_eps"],
        "theta": float(rope),
        "tied": cfg.get("tie_word_embeddings", False),  # model.py:57
        "window": [None] * cfg["num_hidden_layers"],
    }
    if cfg.get("use_sliding_window", False):  # not read by the reference; layers from max_window_layers on are windowed
        first = cfg.get("max_window_layers", 0)
        out["window"] = [cfg["sliding_window"] if i >= first else None for i in range(out["layers"])]
    return out


def plain_load(folder: str | Path, dtype: torch.dtype = torch.float32) -> tuple[dict, dict]:
    """config.json as a dict and every tensor of model.safetensors by name (src/miniserve/loader.py:36-43)."""
    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for f in sorted(folder.glob("*.safetensors")):
        weights.update(load_file(str(f)))
    return cfg, {k: v.to(dtype) for k, v in weights.items()}


# ----------------------------------------------------------------------------- parts
def keep(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16_store(x: torch.Tensor) -> torch.Tensor:
    """What a value becomes when it is written as bfloat16 and read again."""
    return x.to(torch.bfloat16).to(x.dtype)


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, store=keep) -> torch.Tensor:
    """model.py:69-73: reduce in 32-bit, cast back, then multiply by the weight."""
    dtype = x.dtype
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return store(weight * store(h.to(dtype)))


def plain_rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """model.py:83-88: positions [T] -> cos, sin [T, head_dim]; angles in 32-bit, tables cast to ``dtype``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    freqs = positions.float()[:, None] * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def plain_apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """model.py:91-98: x [heads, T, d]; pairs are (j, j + d/2)."""
    x1, x2 = x.chunk(2, dim=-1)
    rot = torch.cat((-x2, x1), dim=-1)
    return x * cos + rot * sin


def plain_attention(x, w: dict, prefix: str, c: dict, cos, sin, window=None, store=keep) -> torch.Tensor:
    """model.py:121-152 for one sequence x [T, hidden], no cache: causal softmax(q k^T / sqrt(d)) v.

    ``window`` (not in the reference): position i sees keys j with i - window < j <= i.
    """
    T = x.shape[0]
    d, nq, nkv = c["head_dim"], c["heads"], c["kv_heads"]

    def lin(name, bias=True):
        y = x @ w[f"{prefix}.{name}.weight"].T
        b = w.get(f"{prefix}.{name}.bias")
        return y + b if (bias and b is not None) else y

    q = lin("q_proj").view(T, nq, d).transpose(0, 1)  # model.py:123
    k = lin("k_proj").view(T, nkv, d).transpose(0, 1)  # model.py:124
    v = lin("v_proj").view(T, nkv, d).transpose(0, 1)  # model.py:125
    q = store(plain_apply_rope(q, cos, sin))  # model.py:127
    k = store(plain_apply_rope(k, cos, sin))  # model.py:128
    v = store(v)
    rep = nq // nkv
    k = k.repeat_interleave(rep, dim=0)  # model.py:137-139: query head h reads kv head h // rep
    v = v.repeat_interleave(rep, dim=0)
    scores = (q.float() @ k.float().transpose(1, 2)) * (1.0 / math.sqrt(d))  # SDPA default scale, model.py:143
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    allowed = j <= i  # is_causal=True, model.py:143
    if window is not None:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed, float("-inf"))
    p = store(torch.softmax(scores, dim=-1))
    out = store((p @ v.float()).to(x.dtype))
    out = out.transpose(0, 1).reshape(T, nq * d)  # model.py:151
    return store(out @ w[f"{prefix}.o_proj.weight"].T)  # model.py:152, no bias


def plain_mlp(x, w: dict, prefix: str, store=keep) -> torch.Tensor:
    """model.py:164-165: down(silu(gate(x)) * up(x)), no biases."""
    g = x @ w[f"{prefix}.gate_proj.weight"].T
    u = x @ w[f"{prefix}.up_proj.weight"].T
    return store(store(torch.nn.functional.silu(g) * u) @ w[f"{prefix}.down_proj.weight"].T)


def plain_block(x, w: dict, i: int, c: dict, cos, sin, store=keep) -> torch.Tensor:
    """model.py:184-185: pre-norm residual, twice."""
    p = f"model.layers.{i}"
    h = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], c["eps"], store)
    x = x + plain_attention(h, w, f"{p}.self_attn", c, cos, sin, c["window"][i], store)
    h = plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], c["eps"], store)
    return x + plain_mlp(h, w, f"{p}.mlp", store)


def plain_forward(cfg: dict, w: dict, token_ids, layer_order=None, store=keep) -> torch.Tensor:
    """model.py:222-237 for one sequence: logits [T, vocab] in 32-bit for every position.

    ``layer_order`` (not in the reference) runs the layers in another order than 0..L-1.
    """
    c = plain_config(cfg)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]  # model.py:229
    cos, sin = plain_rope_tables(torch.arange(len(ids)), c["head_dim"], c["theta"], x.dtype)  # model.py:228-230
    for i in (range(c["layers"]) if layer_order is None else layer_order):  # model.py:231-232
        x = plain_block(x, w, i, c, cos, sin, store)
    x = plain_rmsnorm(x, w["model.norm.weight"], c["eps"], store)  # model.py:237
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]  # model.py:204-206
    return (x @ head.T).float()


# ----------------------------------------------------------------------------- sampling
def plain_logits_to_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """src/miniserve/sampler.py:12-41: the distribution a token is drawn from; logits [vocab]."""
    if temperature <= 0.0:  # sampler.py:23-24
        return torch.zeros_like(logits, dtype=torch.float32).scatter_(-1, logits.argmax(-1, keepdim=True), 1.0)
    logits = logits.float() / temperature  # sampler.py:26
    if top_k > 0:  # sampler.py:28-30: ties with the k-th largest are kept
        kth = torch.topk(logits, min(top_k, logits.shape[-1])).values[..., -1, None]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:  # sampler.py:32-39: drop a token once the mass before it reaches top_p
        sl, si = torch.sort(logits, descending=True, dim=-1)
        probs = sl.softmax(-1)
        before = probs.cumsum(-1) - probs
        sl = sl.masked_fill(before >= top_p, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, si, sl)
    return logits.softmax(-1)  # sampler.py:41


def plain_uniform(seed: int, counter: int) -> float:
    """A number in [0, 1) from (seed, counter): two rounds of the splitmix64 finaliser, top 24 bits.

    The reference draws with torch.multinomial and a torch.Generator (sampler.py:54-55); a generator's
    stream cannot be reproduced inside a kernel, so the engine and this file use this counter-based
    rule instead and the drawn tokens are compared with ``plain_sample``, the probabilities with the
    reference.
    """
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & mask
    for _ in range(2):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def plain_draw(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """sampler.py:44-55 with the draw by inverse CDF in index order: the first token whose running mass exceeds u."""
    if temperature <= 0.0:  # sampler.py:52-53
        return int(logits.argmax(-1))
    probs = plain_logits_to_probs(logits, temperature, top_k, top_p).double()
    cdf = probs.cumsum(-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64), right=True))
    keep = torch.nonzero(probs > 0).flatten()
    return min(max(idx, int(keep[0])), int(keep[-1]))


def plain_sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, counter: int) -> int:
    return plain_draw(logits, temperature, top_k, top_p, plain_uniform(seed, counter))


# ----------------------------------------------------------------------------- generation
def plain_generate(cfg: dict, w: dict, prompt, max_new_tokens: int, eos_ids=(), temperature=0.0, top_k=0, top_p=1.0,
                   seed: int = 0) -> list[int]:
    """src/miniserve/generate.py:45-82 with use_cache=False: the whole sequence again for every token."""
    ids = list(prompt)
    out: list[int] = []
    for step in range(max_new_tokens):
        logits = plain_forward(cfg, w, ids)[-1]
        tok = plain_sample(logits, temperature, top_k, top_p, seed, step)
        if tok in eos_ids:  # generate.py:72-73: the stop token is not returned
            break
        out.append(tok)
        ids.append(tok)
    return out
