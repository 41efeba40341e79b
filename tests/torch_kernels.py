"""Plain torch statements of what each kernel of the package computes, with the kernels' own signatures.

Two uses. (1) Each function is the reference that the GPU test of the kernel of the same name is
compared with, at sizes other than the engine's. (2) As a stand-in for the kernel library they
let the host side of the engine (step building, block tables, scheduler, replay) run on the CPU in
the tests; the package itself has no such path and refuses to run without its CUDA library.

Everything is computed in float32 whatever the storage dtype, rounding only where the kernels store.
"""
from __future__ import annotations

import math

import torch


class TorchKernels:
    name = "torch-reference"

    def __init__(self):
        self.launches = 0

    def embed(self, token_ids, table):
        return table[token_ids.long()].float()

    def feed_tokens(self, token_ids, source_rows, previous_tokens):
        take = source_rows >= 0
        token_ids[take] = previous_tokens[source_rows[take].long()]

    def zero_fresh_state(self, state, seq_slots, seq_starts, positions):
        fresh = positions[seq_starts[: seq_slots.shape[0]].long()] == 0
        state[seq_slots[fresh].long()] = 0

    def rope_tables(self, positions, inv_freq):
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        return ang.cos(), ang.sin()

    def add_rmsnorm(self, residual, delta, weight, eps, out_dtype):
        if delta is not None:
            residual += delta.float()
        h = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
        return (weight.float() * h.to(out_dtype).float()).to(out_dtype)

    def rmsnorm_rows(self, residual, delta, weight, eps, rows, out_dtype):
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
        h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return (weight.float() * h.to(out_dtype).float()).to(out_dtype)

    def linear(self, x, w, out_dtype=None, add_to=None, transient=False):
        y = x.float() @ w.float().T
        if add_to is not None:
            add_to += y
            return None
        return y.to(out_dtype or x.dtype)

    def qkv_rope(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                 write_kv=True, out_dtype=None):
        qkv = self.linear(x, w, out_dtype=out_dtype)
        return self.rope_kv_write(qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                                  write_kv, out_dtype)

    def qkv_attention(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, block_table, token_seq, positions, num_heads,
                      num_kv_heads, head_dim, page_size, scale, window, max_context, batch=None, write_kv=True, out_dtype=None):
        qkv = self.qkv_rope(x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size, write_kv,
                            out_dtype)
        return self.paged_attention(qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim, page_size,
                                    scale, window, max_context, batch=batch)

    def rope_kv_write(self, qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim,
                      page_size, write_kv=True, out_dtype=None):
        N = qkv.shape[0]
        d, half = head_dim, head_dim // 2
        x = qkv.float()
        if bias is not None:
            x = x + bias.float()
        x = x.view(N, num_heads + 2 * num_kv_heads, d)
        rot = x[:, :num_heads + num_kv_heads]
        x1, x2 = rot[..., :half], rot[..., half:]
        c, s = cos[:, None, :], sin[:, None, :]
        rotated = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
        out = torch.cat((rotated, x[:, num_heads + num_kv_heads:]), dim=1)
        qkv.copy_(out.reshape(N, -1).to(qkv.dtype))
        if write_kv:
            page = (slot_mapping // page_size).long()
            off = (slot_mapping % page_size).long()
            k = qkv.view(N, -1, d)[:, num_heads:num_heads + num_kv_heads]
            v = qkv.view(N, -1, d)[:, num_heads + num_kv_heads:]
            k_pool[page, :, off] = k
            v_pool[page, :, off] = v
        return qkv

    def paged_attention(self, qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim,
                        page_size, scale, window, max_context, batch=None, num_splits=None):
        N = qkv.shape[0]
        d = head_dim
        rep = num_heads // num_kv_heads
        q = qkv.view(N, -1, d)[:, :num_heads].float()
        out = torch.zeros(N, num_heads, d)
        for t in range(N):
            p = int(positions[t])
            lo = 0 if not window else max(0, p - window + 1)
            keys = torch.arange(lo, p + 1)
            pages = block_table[int(token_seq[t])][(keys // page_size)].long()
            offs = (keys % page_size).long()
            k = k_pool[pages, :, offs].float()  # [S, kvh, d]
            v = v_pool[pages, :, offs].float()
            for h in range(num_heads):
                s = (k[:, h // rep] @ q[t, h]) * scale
                pr = torch.softmax(s, dim=0)
                out[t, h] = pr @ v[:, h // rep]
        return out.reshape(N, num_heads * d).to(qkv.dtype)

    def gate_up_act(self, x, w_gate_up, out_dtype=None):
        return self.silu_mul(self.linear(x, w_gate_up, out_dtype=torch.float32)).to(out_dtype or x.dtype)

    def silu_mul(self, gu, out_dtype=None):
        i = gu.shape[1] // 2
        g, u = gu[:, :i].float(), gu[:, i:].float()
        return (g * torch.sigmoid(g) * u).to(gu.dtype)

    def argmax(self, logits):
        return logits.argmax(-1).to(torch.int32)

    def sample(self, logits, temperature, top_k, top_p, uniform):
        from plain_qwen2 import plain_draw

        out = [plain_draw(logits[i].float(), float(temperature[i]), int(top_k[i]), float(top_p[i]), float(uniform[i]))
               for i in range(logits.shape[0])]
        return torch.tensor(out, dtype=torch.int32)
