"""A Llama-3.1-architecture decoder with HashAttention on every layer, tensor-parallel over the GPUs of
one node: the host model of the full-model configuration (32 layers, hidden 4096, 32 query / 8 kv
heads of 128, SwiGLU FFN 14336, vocabulary 128256, RoPE theta 500000, random bf16 weights).

Parallel layout, as the reference's gpt-fast host shards it (efficiency/tp.py:48-98): the q / k / v
projections and w1 / w3 are split by columns (a rank owns whole heads: ``Hq / N`` query heads and
``Hkv / N`` kv-heads), wo and w2 by rows, and the partial results of wo and w2 are summed over the
ranks with an all-reduce after attention and after the MLP (efficiency/tp.py:104-134); embedding and
output head are replicated. One process per GPU; the all-reduce is the NCCL collective of
``torch.distributed`` (gloo in the CPU test) - a plain library call, the hot path stays inside a rank.

Attention: the prompt is prefilled with dense causal attention (``scaled_dot_product_attention``, a
library call), its keys / values go into this rank's paged cache and the key hashes are built once
(``ha_hash_prefill``); every decode step is one ``ha_decode_step`` per layer on the rank's
``Hkv / N`` kv-heads. A kv-head's keys, hash codes, hash MLPs and query heads live on one rank, so the
sparse-decode path itself needs no communication (SparseDecodeContext per layer).

Weights are drawn per block of 1/8 of every sharded dimension from seeds that depend on (layer,
matrix, block) only, so every rank count holds the same model.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .cache import PagedHashKVCache
from .ops import Budget, SparseDecodeContext, rope_split
from .synthetic import make_usa

BLOCKS = 8  # the finest partition of a sharded dimension (one kv-head's worth of every matrix)


@dataclass
class LlamaTPConfig:
    n_layers: int = 32
    dim: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 14336
    vocab_size: int = 128256
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    init_budget: int = 128
    heavy_budget: float = 1.0 / 32
    recent_budget: int = 128
    max_seq_len: int = 32768 + 256


def block_range(world: int, rank: int) -> range:
    """The 1/8 blocks of every sharded dimension that ``rank`` of ``world`` owns (contiguous, rank order)."""
    if BLOCKS % world != 0 or not 0 <= rank < world:
        raise ValueError(f"{BLOCKS} blocks cannot be dealt to rank {rank} of {world}")
    per = BLOCKS // world
    return range(rank * per, (rank + 1) * per)


def _seed(*key) -> int:
    """A seed that depends on the key alone (not on the process, as Python's hash of a string would)."""
    return zlib.crc32(repr(key).encode()) & 0x7FFFFFFF


def _draw(shape, seed: int, device, dtype, std: float = 0.02) -> torch.Tensor:
    """N(0, std) values from the generator of the tensor's own device (billions of values are drawn where they
    live; CPU and GPU generators give different, equally seeded, streams)."""
    device = torch.device(device)
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device) * std).to(dtype)


def sharded_weight(name: str, layer: int, rows: int, cols: int, split: str, blocks, device, seed: int,
                   dtype=torch.bfloat16) -> torch.Tensor:
    """Rows x cols matrix ([out, in], as nn.Linear stores it) restricted to ``blocks`` of its output rows
    (``split == 'col'``: column-parallel in the usual naming, the outputs are divided) or of its input columns
    (``split == 'row'``). Block j is drawn from a seed of (seed, layer, name, j) alone."""
    parts = []
    for j in blocks:
        s = _seed(seed, layer, name, j)
        if split == "col":
            parts.append(_draw((rows // BLOCKS, cols), s, device, dtype))
        else:
            parts.append(_draw((rows, cols // BLOCKS), s, device, dtype))
    return torch.cat(parts, dim=0 if split == "col" else 1).contiguous()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [..., T, H, D] rotated (rotate-half convention) for positions pos [T] (or broadcastable)."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=x.device) / d))
    ang = pos.to(torch.float32)[..., None] * inv  # [T, D/2]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[..., None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[..., None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., d // 2:], xf[..., : d // 2]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


class Layer:
    def __init__(self, cfg: LlamaTPConfig, idx: int, blocks, device, seed: int, dtype):
        kv_rows = cfg.n_kv_heads * cfg.head_dim
        mk = lambda name, r, c, split: sharded_weight(name, idx, r, c, split, blocks, device, seed, dtype)  # noqa: E731
        # one fused projection per rank: [local q heads | local k heads | local v heads] x dim
        self.wqkv = torch.cat([mk("wq", cfg.n_heads * cfg.head_dim, cfg.dim, "col"), mk("wk", kv_rows, cfg.dim, "col"),
                               mk("wv", kv_rows, cfg.dim, "col")], dim=0).contiguous()
        self.wo = mk("wo", cfg.dim, cfg.n_heads * cfg.head_dim, "row")
        self.w13 = torch.cat([mk("w1", cfg.ffn_dim, cfg.dim, "col"), mk("w3", cfg.ffn_dim, cfg.dim, "col")], dim=0).contiguous()
        self.w2 = mk("w2", cfg.dim, cfg.ffn_dim, "row")
        self.norm1 = torch.ones(cfg.dim, dtype=dtype, device=device)
        self.norm2 = torch.ones(cfg.dim, dtype=dtype, device=device)


class TPLlama:
    """One rank's share of the model. ``attention``: 'cuda' (the library's decode step on a paged cache) or a
    callable ``f(layer, q [B,Hq_l,D], k_all [B,Hkv_l,S,D], v_all) -> [B,Hq_l,D]`` used by CPU tests, in which
    case the keys / values are kept as plain tensors."""

    def __init__(self, cfg: LlamaTPConfig, world: int, rank: int, device, batch: int, seed: int = 0, group=None,
                 attention="cuda", dtype=torch.bfloat16):
        self.cfg, self.world, self.rank, self.device, self.group, self.batch = cfg, world, rank, torch.device(device), group, batch
        blocks = block_range(world, rank)
        self.hq = cfg.n_heads // world
        self.hkv = cfg.n_kv_heads // world
        self.layers = [Layer(cfg, i, blocks, self.device, seed, dtype) for i in range(cfg.n_layers)]
        self.embed = _draw((cfg.vocab_size, cfg.dim), _seed(seed, "embed"), self.device, dtype)
        self.head = _draw((cfg.vocab_size, cfg.dim), _seed(seed, "head"), self.device, dtype)
        self.final_norm = torch.ones(cfg.dim, dtype=dtype, device=self.device)
        self.attention = attention
        self.pos = torch.zeros(batch, dtype=torch.int64, device=self.device)  # position of the next token per sequence
        if attention == "cuda":
            budget = Budget(cfg.init_budget, cfg.heavy_budget, cfg.recent_budget)
            h0 = rank * self.hq
            self.ctxs = []
            self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)  # one copy for all layers
            for i in range(cfg.n_layers):
                cache = PagedHashKVCache(batch, self.hkv, cfg.max_seq_len, self.device)
                cache.seq_lens = self.seq_lens
                packed = make_usa(cfg.n_heads, cfg.head_dim, seed=seed * 1000 + i, bf16=True).packed(self.device)
                self.ctxs.append(SparseDecodeContext(cache, budget, packed.slice_heads(h0, h0 + self.hq)))
        else:
            self.kv = [None] * cfg.n_layers  # (k [B,Hkv_l,S,D], v)

    # -- collectives ---------------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of the row-parallel partial results over the ranks (efficiency/tp.py:114-115, 133-134)."""
        if self.world > 1:
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    # -- blocks ----------------------------------------------------------------------------------
    def _qkv(self, layer: Layer, h: torch.Tensor):
        cfg = self.cfg
        qkv = F.linear(h, layer.wqkv)
        q, k, v = qkv.split([self.hq * cfg.head_dim, self.hkv * cfg.head_dim, self.hkv * cfg.head_dim], dim=-1)
        return (q.reshape(*h.shape[:-1], self.hq, cfg.head_dim), k.reshape(*h.shape[:-1], self.hkv, cfg.head_dim),
                v.reshape(*h.shape[:-1], self.hkv, cfg.head_dim))

    def _mlp(self, layer: Layer, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        for s in range(0, x.shape[0], 8192):  # by blocks of tokens: the 14336-wide intermediate stays small
            h = rms_norm(x[s:s + 8192], layer.norm2, self.cfg.norm_eps)
            a, b = F.linear(h, layer.w13).chunk(2, dim=-1)
            out[s:s + 8192] = F.linear(F.silu(a) * b, layer.w2)
        return self.all_reduce(out)

    # -- prefill: one sequence at a time, dense causal attention -----------------------------------
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] -> next-token ids [B] (greedy). Fills the caches and builds the key hashes."""
        cfg = self.cfg
        B, S = tokens.shape
        nxt = torch.empty(B, dtype=torch.int64, device=self.device)
        pos = torch.arange(S, device=self.device)
        for b in range(B):
            x = self.embed[tokens[b]]
            for i, layer in enumerate(self.layers):
                h = rms_norm(x, layer.norm1, cfg.norm_eps)
                q, k, v = self._qkv(layer, h)               # [S, heads, D]
                q, k = rope(q, pos, cfg.rope_theta), rope(k, pos, cfg.rope_theta)
                qh, kh, vh = q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1)  # [heads, S, D]
                att = F.scaled_dot_product_attention(qh[None], kh[None], vh[None], is_causal=True, enable_gqa=True)[0]
                if self.attention == "cuda":
                    self.ctxs[i].cache.write_kv(b, kh, vh)  # (stored as bf16)
                else:
                    if self.kv[i] is None:
                        self.kv[i] = (torch.zeros(B, self.hkv, S, cfg.head_dim, dtype=kh.dtype, device=self.device),
                                      torch.zeros(B, self.hkv, S, cfg.head_dim, dtype=kh.dtype, device=self.device))
                    self.kv[i][0][b], self.kv[i][1][b] = kh, vh
                o = F.linear(att.transpose(0, 1).reshape(S, self.hq * cfg.head_dim), layer.wo)
                x = x + self.all_reduce(o)
                x = x + self._mlp(layer, x)
            last = rms_norm(x[-1:], self.final_norm, cfg.norm_eps)
            nxt[b] = F.linear(last, self.head).float().argmax(-1)[0]
        if self.attention == "cuda":
            for ctx in self.ctxs:
                ctx.hash_prefill()
        self.pos.fill_(S)
        return nxt

    # -- one greedy decode step for the whole batch ------------------------------------------------
    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, out_tokens: torch.Tensor) -> None:
        """tokens [B] -> out_tokens [B] (written in place: the call is CUDA-graph capturable; positions and
        sequence lengths advance on the device)."""
        cfg = self.cfg
        x = self.embed[tokens]                                           # [B, dim]
        if self.attention == "cuda":
            self.seq_lens += 1  # the token being decoded counts (every layer's cache shares this tensor)
        for i, layer in enumerate(self.layers):
            h = rms_norm(x, layer.norm1, cfg.norm_eps)
            if self.attention == "cuda":
                # projection, then one kernel that splits q | k | v and rotates q and k, then the decode step
                q, k, v = rope_split(F.linear(h, layer.wqkv), self.pos, self.hq, self.hkv, cfg.rope_theta)
                att = self.ctxs[i].decode_step(q, k, v).to(x.dtype)
            else:
                q, k, v = self._qkv(layer, h)                            # [B, heads, D]
                q = rope(q[:, None], self.pos[:, None], cfg.rope_theta)[:, 0]
                k = rope(k[:, None], self.pos[:, None], cfg.rope_theta)[:, 0]
                kc = torch.cat([self.kv[i][0], k[:, :, None]], dim=2)
                vc = torch.cat([self.kv[i][1], v[:, :, None]], dim=2)
                self.kv[i] = (kc, vc)
                att = self.attention(i, q, kc, vc).to(x.dtype)
            o = F.linear(att.reshape(x.shape[0], self.hq * cfg.head_dim), layer.wo)
            x = x + self.all_reduce(o)
            x = x + self._mlp(layer, x)
        logits = F.linear(rms_norm(x, self.final_norm, cfg.norm_eps), self.head)
        out_tokens.copy_(logits.float().argmax(-1))
        self.pos += 1

    def check_status(self) -> None:
        if self.attention == "cuda":
            for ctx in self.ctxs:
                ctx.check_status()


def tokens_for(cfg: LlamaTPConfig, batch: int, length: int, seed: int = 1004) -> torch.Tensor:
    """Uniform random token ids [batch, length] from a fixed seed (the same on every rank)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (batch, length), generator=g)
