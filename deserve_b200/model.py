"""A random-init Llama stage that drives the KV path the way the reference's
layers do (deserve_worker/model/llama.py:53-88, model/layer/attention.py:126-193,
layer/norm.py:21-34, layer/linear.py:115-123, looped by
LayerStorage.forward, deserve_worker/layer_storage.py:182-197).

It plays the role of the reference's LayerStorage for the engine classes: it has
`forward(h, ctx)`, `need_sample`, `need_tokenize`, `model_args` and a greedy
`sample`. Dense projections are torch matmuls (cuBLAS); RoPE, append and paged
attention are this package's kernels. Weights are N(0, 0.02) from a per-layer
seed, so any split of the layers over stages sees the same model.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops
from .context import FlashDecodeCtx, FlashForwardCtx, FlashPrefillCtx
from .task import TaskData


@dataclass
class ModelArgs:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    vocab_size: int = 128256
    ffn_dim: int = 14336
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    page_size: int = 16

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


llama_3_8b_args = ModelArgs()
llama_3_70b_args = ModelArgs(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_dim=28672)


def init_weight(shape, seed: int, device, dtype, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    if torch.device(device).type == "cpu" or shape[0] * shape[1] <= (1 << 22):
        return (torch.randn(shape, generator=g) * std).to(dtype).to(device)
    # large matrices: drawn on the device, row block by row block, from seeds derived from `seed`
    out = torch.empty(shape, dtype=dtype, device=device)
    gd = torch.Generator(device=device)
    rows = max(1, (1 << 24) // shape[1])
    for i, r0 in enumerate(range(0, shape[0], rows)):
        gd.manual_seed(seed * 1000003 + i)
        blk = out[r0 : r0 + rows]
        blk.copy_((torch.randn(blk.shape, generator=gd, device=device) * std).to(dtype))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return ops.rmsnorm(x, weight, eps)


class LlamaStage:
    """Layers [layer_begin, layer_end) of the model; the first stage also embeds
    tokens, the last one also applies the final norm and the output projection."""

    def __init__(self, args: ModelArgs, layer_begin: int, layer_end: int, device, dtype, seed: int = 0,
                 first: bool | None = None, last: bool | None = None, split_head: bool = False):
        """split_head: the output projection is cut in two halves of the vocabulary. The LAST stage
        applies the final norm, computes the logits of the lower half and their row maxima, and hands
        on the normed rows together with (max, argmax) of its half (`pack_partial`); the FIRST stage
        computes the upper half, combines the two (`finish_head`) and embeds the tokens for the next
        step. In a pipeline whose stages hold equal numbers of layers this halves the extra work of
        the stage that owns the head (it reads 1 GB of output weights per microbatch step instead of
        2 GB) at the price of a 2 MiB instead of a 512-byte message on the link back to the first
        stage. The reference keeps the whole head on the last worker (layer_storage.py:219-253)."""
        self.model_args = args
        self.layer_begin, self.layer_end = layer_begin, layer_end
        self.need_tokenize = layer_begin == 0 if first is None else first
        is_last = layer_end == args.n_layers if last is None else last
        self.split_head = split_head
        self.head_lo = split_head and is_last          # this stage computes the lower half of the head
        self.need_sample = is_last and not split_head  # with a split head nobody samples inside forward()
        self.vocab_lo = (args.vocab_size // 2 + 7) // 8 * 8
        self.main_device, self.dtype = torch.device(device), dtype
        a, hd = args, args.head_dim
        qkv_rows = (a.n_heads + 2 * a.n_kv_heads) * hd
        self.layers = []
        for l in range(layer_begin, layer_end):
            s = seed * 7919 + l * 16
            self.layers.append({
                "wqkv": init_weight((qkv_rows, a.dim), s + 1, device, dtype),
                "wo": init_weight((a.dim, a.n_heads * hd), s + 2, device, dtype),
                "w13": init_weight((2 * a.ffn_dim, a.dim), s + 3, device, dtype),
                "w2": init_weight((a.dim, a.ffn_dim), s + 4, device, dtype),
                "attn_norm": torch.ones(a.dim, dtype=dtype, device=device),
                "ffn_norm": torch.ones(a.dim, dtype=dtype, device=device),
            })
        if self.need_tokenize:
            self.tok_embeddings = init_weight((a.vocab_size, a.dim), seed * 7919 + 900001, device, dtype)
        if self.need_sample:
            self.norm = torch.ones(a.dim, dtype=dtype, device=device)
            self.output = init_weight((a.vocab_size, a.dim), seed * 7919 + 900002, device, dtype)
        if self.head_lo:
            self.norm = torch.ones(a.dim, dtype=dtype, device=device)
            self.output_lo = init_weight((self.vocab_lo, a.dim), seed * 7919 + 900003, device, dtype)
        if split_head and self.need_tokenize:
            self.output_hi = init_weight((a.vocab_size - self.vocab_lo, a.dim), seed * 7919 + 900004, device, dtype)

    # ---- the output head in two halves --------------------------------------------------------
    def _half_argmax(self, hn: torch.Tensor, w: torch.Tensor):
        logits = torch.mm(hn, w.t())
        idx = ops.greedy_sample(logits)
        return logits.gather(1, idx.long().unsqueeze(1)).squeeze(1).float(), idx

    def pack_partial(self, hn: torch.Tensor) -> torch.Tensor:
        """Last stage: normed rows [n, dim] + (max, argmax) over the lower half of the vocabulary, as ONE
        uint8 message: n*dim elements, then n float32 maxima, then n int32 indices."""
        mx, idx = self._half_argmax(hn, self.output_lo)
        return torch.cat([hn.reshape(-1).view(torch.uint8), mx.view(torch.uint8), idx.view(torch.uint8)])

    def partial_rows(self, packed: torch.Tensor) -> int:
        return packed.numel() // (self.model_args.dim * packed.new_empty(0, dtype=self.dtype).element_size() + 8)

    @torch.inference_mode()
    def finish_head(self, packed: torch.Tensor) -> torch.Tensor:
        """First stage: the upper half of the head on the rows of a pack_partial message, combined with
        the lower half's (max, argmax): int32 greedy tokens [n], the lowest index among equal maxima
        (the lower half wins a tie), exactly what an argmax over the whole vocabulary gives."""
        n, dim = self.partial_rows(packed), self.model_args.dim
        nb = n * dim * packed.new_empty(0, dtype=self.dtype).element_size()
        hn = packed[:nb].view(self.dtype).view(n, dim)
        mx_lo = packed[nb : nb + 4 * n].view(torch.float32)
        idx_lo = packed[nb + 4 * n : nb + 8 * n].view(torch.int32)
        mx_hi, idx_hi = self._half_argmax(hn, self.output_hi)
        return torch.where(mx_hi > mx_lo, idx_hi + self.vocab_lo, idx_lo).to(torch.int32)

    @property
    def full_output(self) -> torch.Tensor:
        """The whole output projection [vocab, dim] of a stage that holds both halves (checks only)."""
        return self.output if not self.split_head else torch.cat([self.output_lo, self.output_hi])

    # ---- one transformer block --------------------------------------------------------------
    def _block(self, w: dict, x: torch.Tensor, ctx: FlashForwardCtx) -> torch.Tensor:
        """Nine launches plus the attention kernels: norm, fused q|k|v projection, rotary +
        append, attention, output projection with the residual in its epilogue (addmm), norm,
        fused gate|up projection, SwiGLU middle, down projection with the residual (addmm)."""
        a, hd = self.model_args, self.model_args.head_dim
        qkv = torch.mm(rmsnorm(x, w["attn_norm"], a.norm_eps), w["wqkv"].t())
        nq, nkv = a.n_heads * hd, a.n_kv_heads * hd
        q = qkv[:, :nq].unflatten(1, (a.n_heads, hd))
        k = qkv[:, nq : nq + nkv].unflatten(1, (a.n_kv_heads, hd))
        v = qkv[:, nq + nkv :].unflatten(1, (a.n_kv_heads, hd))
        pages = ctx.page_pool.get_layered_pages(ctx.layer_id)
        ops.rope_append_paged_kv_cache(q, k, v, ctx.indptr, ctx.offsets, pages, ctx.kv_page_indices,
                                       ctx.kv_page_indptr, ctx.kv_last_page_lens, a.rope_theta)
        if isinstance(ctx, FlashDecodeCtx):
            attn = ctx.decode_wrapper.forward(q, pages)
        else:
            assert isinstance(ctx, FlashPrefillCtx)
            attn = ctx.prefill_wrapper.forward(q, pages, causal=True)
        h = torch.addmm(x, attn.view(-1, nq), w["wo"].t())
        gu = torch.mm(rmsnorm(h, w["ffn_norm"], a.norm_eps), w["w13"].t())
        return torch.addmm(h, ops.silu_mul(gu), w["w2"].t())

    @torch.inference_mode()
    def forward(self, h: torch.Tensor, ctx: FlashForwardCtx) -> torch.Tensor:
        """h: token ids [nnz] on the first stage, activations [nnz, dim] otherwise.
        Returns activations, or on the last stage the logits of every request's
        last row [bsz, vocab]."""
        if self.need_tokenize:
            h = self.tok_embeddings[h.long()]
        for w in self.layers:
            h = self._block(w, h, ctx)
            ctx.layer_id += 1
        if self.need_sample or self.head_lo:
            if h.shape[0] != ctx.bsz:  # prompt chunks: only every request's last row is sampled
                h = h[(ctx.indptr[1:] - 1).long()]
            hn = rmsnorm(h, self.norm, self.model_args.norm_eps)
            h = self.pack_partial(hn) if self.head_lo else torch.mm(hn, self.output.t())
        return h

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, task_datas: list[TaskData], ignore_eos: bool):
        """Greedy next token of every request that finished its prompt (one batched
        argmax and one device->host copy instead of the reference's per-task
        argmax + cat, layer_storage.py:219-253). Returns (tokens [bsz] int32 on the
        device, mask of requests that produced a token, ids done)."""
        tokens = ops.greedy_sample(logits)
        produced, done = [], []
        for t in task_datas:
            fin = t.finished_prefill()
            produced.append(fin)
            if fin:
                t.sampling_params.max_new_tokens -= 1
                if t.sampling_params.max_new_tokens <= 0 or t.start_pos >= t.sampling_params.max_seq_len:
                    done.append(t.task_id)
        return tokens, produced, done
