"""Dense fp32 Llama decoding on the CPU: the checker for the engine's greedy tokens.

Follows the reference's block (deserve_worker/model/llama.py:53-88): x +
attention(attention_norm(x)), then h + ffn(ffn_norm(h)); RMSNorm of
layer/norm.py:18-19; SwiGLU of layer/linear.py:115-118; attention math of
layer/attention.py:237-266 with rotary positions offsets[i] + j; greedy argmax of
layer_storage.py:250. K/V are kept as plain per-request lists (no pages)."""
from __future__ import annotations

import torch

from . import kv_math


def _norm(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


class DenseLlama:
    def __init__(self, args, layers: list[dict], tok_embeddings, norm, output):
        """Weights are taken (as fp32 CPU copies) from the stages under test."""
        f = lambda t: t.detach().float().cpu()
        self.a = args
        self.layers = [{k: f(v) for k, v in w.items()} for w in layers]
        self.emb, self.norm, self.out = f(tok_embeddings), f(norm), f(output)
        self.kv: dict[str, list] = {}

    def step(self, task_id: str, tokens: torch.Tensor) -> int:
        """Feed `tokens` (a prompt chunk or one decode token) of one request; returns the greedy next token."""
        a, hd = self.a, self.a.dim // self.a.n_heads
        cache = self.kv.setdefault(task_id, [[None, None] for _ in self.layers])
        start = 0 if cache[0][0] is None else cache[0][0].shape[0]
        pos = torch.arange(start, start + len(tokens))
        x = self.emb[tokens.long()]
        nq, nkv = a.n_heads * hd, a.n_kv_heads * hd
        for w, c in zip(self.layers, cache):
            qkv = _norm(x, w["attn_norm"], a.norm_eps) @ w["wqkv"].t()
            q = kv_math.apply_rope(qkv[:, :nq].reshape(-1, a.n_heads, hd), pos, a.rope_theta)
            k = kv_math.apply_rope(qkv[:, nq : nq + nkv].reshape(-1, a.n_kv_heads, hd), pos, a.rope_theta)
            v = qkv[:, nq + nkv :].reshape(-1, a.n_kv_heads, hd)
            c[0] = k if c[0] is None else torch.cat([c[0], k])
            c[1] = v if c[1] is None else torch.cat([c[1], v])
            attn = kv_math.dense_attention(q, c[0], c[1], causal_tail=True)
            h = x + attn.reshape(-1, nq) @ w["wo"].t()
            gu = _norm(h, w["ffn_norm"], a.norm_eps) @ w["w13"].t()
            x = h + (torch.nn.functional.silu(gu[:, : a.ffn_dim]) * gu[:, a.ffn_dim :]) @ w["w2"].t()
        logits = _norm(x[-1], self.norm, a.norm_eps) @ self.out.t()
        self.last_logits = logits
        return int(torch.argmax(logits))
