"""Seeded synthetic inputs for the decode path: hash weights, post-RoPE q / k / v with a few
outlier key channels, ragged lengths, shuffled page tables and planted near-duplicate keys.

The reference publishes no dataset for this path, so benchmarks and parity tests run on these
tensors. Everything is drawn from CPU generators with fixed seeds, so the same call gives the
same tensors on every machine with the same torch build.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch

from .usa import USA

ROPE_THETA = 500000.0
OUTLIER_CHANNELS = (3, 40, 77, 101)
OUTLIER_SCALE = 8.0


def make_usa(num_heads: int = 32, head_dim: int = 128, seed: int = 0, bf16: bool = True, num_layers: int = 3) -> USA:
    """Hash weights with torch's default Linear init under ``torch.manual_seed(seed)``: the values
    the reference's ``load_usa(config, None)`` holds under the same seed
    (hashattention/hashattention_llama.py:633-646). ``bf16=True`` rounds them once to bf16."""
    state = torch.random.get_rng_state()
    try:
        torch.manual_seed(seed)
        usa = USA(num_heads, head_dim, {"lth_int_dim": 128, "lth_final_dim": 32, "lth_thold": 0,
                                        "lth_num_layers": num_layers})
    finally:
        torch.random.set_rng_state(state)
    return usa.bfloat16() if bf16 else usa


def rope_tables(positions: torch.Tensor, dim: int = 128, theta: float = ROPE_THETA):
    """cos / sin tables [len, dim] in the rotate-half convention (frequencies theta^(-2i/dim),
    repeated for both halves)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., len, dim] * cos + rotate_half(x) * sin."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


@dataclass
class DecodeInputs:
    """One decode step's tensors for a batch of sequences (all CPU, fp32 values; when ``bf16`` is
    set every value is exactly representable in bf16)."""

    q: torch.Tensor                 # [B, Hq, D]   query of the token being decoded (position S_b - 1)
    k: list[torch.Tensor]           # B x [Hkv, S_b, D]   all keys incl. the new token's (last row)
    v: list[torch.Tensor]           # B x [Hkv, S_b, D]
    seq_lens: list[int]
    bf16: bool
    planted: list[torch.Tensor] = field(default_factory=list)  # B x [n] planted key positions

    @property
    def batch(self) -> int:
        return len(self.seq_lens)

    def digest(self) -> str:
        """SHA-256 over the first sequence's q, k, v bytes (recorded in result files)."""
        h = hashlib.sha256()
        for t in (self.q[0], self.k[0], self.v[0]):
            h.update(t.contiguous().numpy().tobytes())
        return h.hexdigest()


def _round(x: torch.Tensor, bf16: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32) if bf16 else x


def _plant(q: torch.Tensor, k: torch.Tensor, S: int, init: int, recent: int, frac: float, group: int,
           gen: torch.Generator) -> torch.Tensor:
    """Overwrites round(frac*S) candidate keys of every kv-head j with vectors of the key's own
    norm and cosine 0.9 to query head j*group."""
    lo, hi = min(init, S), max(min(init, S), S - recent)
    n = min(int(round(frac * S)), hi - lo)
    pos = lo + torch.randperm(hi - lo, generator=gen)[:n]
    for j in range(k.shape[0]):
        qh = q[j * group] / q[j * group].norm()
        u = torch.randn(n, q.shape[-1], generator=gen)
        u = u - (u @ qh)[:, None] * qh[None, :]
        u = u / u.norm(dim=-1, keepdim=True)
        norms = k[j, pos].norm(dim=-1, keepdim=True)
        k[j, pos] = norms * (0.9 * qh[None, :] + (0.19 ** 0.5) * u)
    return pos


def make_decode_inputs(config_index: int, seq_lens, num_q_heads: int = 32, num_kv_heads: int = 8,
                       head_dim: int = 128, bf16: bool = True, ragged: bool | None = None,
                       plant_frac: float = 0.0, init_budget: int = 128, recent_budget: int = 128) -> DecodeInputs:
    """q, k, v ~ N(0,1); key channels 3, 40, 77, 101 scaled x8 before RoPE; RoPE with theta 5e5,
    key positions 0..S-1 and query position S-1; optional rounding to bf16 after RoPE.

    A uniform batch draws q[B,Hq,1,D], k[B,Hkv,S,D], v[B,Hkv,S,D] in this order from
    ``Generator().manual_seed(1000 + config_index)``; a ragged batch draws each sequence b
    from seed ``1000 + config_index + 1000 * (b + 1)``.
    """
    seq_lens = [int(s) for s in seq_lens]
    B = len(seq_lens)
    if ragged is None:
        ragged = len(set(seq_lens)) > 1
    group = num_q_heads // num_kv_heads
    qs, ks, vs, planted = [], [], [], []
    if not ragged:
        S = seq_lens[0]
        g = torch.Generator().manual_seed(1000 + config_index)
        q_raw = torch.randn(B, num_q_heads, 1, head_dim, generator=g)
        k_raw = torch.randn(B, num_kv_heads, S, head_dim, generator=g)
        v_raw = torch.randn(B, num_kv_heads, S, head_dim, generator=g)
        per_seq = [(q_raw[b], k_raw[b], v_raw[b], g) for b in range(B)]
    else:
        per_seq = []
        for b, S in enumerate(seq_lens):
            g = torch.Generator().manual_seed(1000 + config_index + 1000 * (b + 1))
            q_raw = torch.randn(num_q_heads, 1, head_dim, generator=g)
            k_raw = torch.randn(num_kv_heads, S, head_dim, generator=g)
            v_raw = torch.randn(num_kv_heads, S, head_dim, generator=g)
            per_seq.append((q_raw, k_raw, v_raw, g))
    for b, (q_raw, k_raw, v_raw, g) in enumerate(per_seq):
        S = seq_lens[b]
        k_raw[..., list(OUTLIER_CHANNELS)] *= OUTLIER_SCALE
        cos, sin = rope_tables(torch.arange(S))
        k = apply_rope(k_raw, cos, sin)
        q = apply_rope(q_raw, cos[S - 1:S], sin[S - 1:S])[:, 0, :]
        if plant_frac > 0.0:
            planted.append(_plant(q, k, S, init_budget, recent_budget, plant_frac, group, g))
        qs.append(_round(q, bf16))
        ks.append(_round(k, bf16).contiguous())
        vs.append(_round(v_raw, bf16).contiguous())
    return DecodeInputs(torch.stack(qs), ks, vs, seq_lens, bf16, planted)


def ragged_lengths(config_index: int, batch: int, low: int, high: int) -> list[int]:
    """Per-sequence context lengths uniform in [low, high] from seed 1000 + config_index."""
    g = torch.Generator().manual_seed(1000 + config_index)
    return torch.randint(low, high + 1, (batch,), generator=g).tolist()


def fill_cache_on_device(cache, seq_lens, seed: int, kv_head0: int = 0) -> None:
    """Fills a paged cache directly on its device with keys / values of the same distribution as
    :func:`make_decode_inputs` (N(0,1), outlier channels x8, RoPE, bf16), drawn from device
    generators. For benchmarks, where the tensors are too large to draw on the host; parity tests
    use the host generators above.

    Every kv-head has its own generator, seeded by ``(seed, global head index)``: the cache's head
    ``j`` holds global head ``kv_head0 + j``, so a GPU that owns a slice of the kv-heads gets exactly
    the rows the unsharded cache holds for those heads."""
    dev = cache.device
    gens = [torch.Generator(device=dev).manual_seed(seed * 64 + kv_head0 + j) for j in range(cache.num_kv_heads)]
    inv_freq = 1.0 / (ROPE_THETA ** (torch.arange(0, 128, 2, dtype=torch.float32, device=dev) / 128))
    for b, S in enumerate(int(s) for s in seq_lens):
        for start in range(0, S, 32768):
            n = min(32768, S - start)
            k = torch.stack([torch.randn(n, 128, generator=g, device=dev) for g in gens])
            v = torch.stack([torch.randn(n, 128, generator=g, device=dev) for g in gens])
            k[..., list(OUTLIER_CHANNELS)] *= OUTLIER_SCALE
            freqs = torch.arange(start, start + n, device=dev, dtype=torch.float32)[:, None] * inv_freq[None, :]
            emb = torch.cat([freqs, freqs], dim=-1)
            k = apply_rope(k, emb.cos(), emb.sin())
            cache.write_kv(b, k, v, start=start)


def algorithmic_bytes(seq_lens, num_q_heads: int, num_kv_heads: int, init_budget: int, recent_budget: int,
                      heavy_budget: float, head_dim: int = 128) -> dict:
    """Bytes one decode step of one layer must move: the u32 key codes of every token and query
    head, a bf16 K row and V row per attended token (sink / recent rows once per kv-head, heavy
    rows once per query head) and q / out."""
    hash_b = kv_b = 0
    for S in (int(s) for s in seq_lens):
        hb = int(heavy_budget) if heavy_budget > 1.0 else int(S * heavy_budget)
        edge = min(S, init_budget + recent_budget)
        heavy = min(hb, max(0, S - init_budget - recent_budget))
        hash_b += 4 * num_q_heads * S
        kv_b += 2 * head_dim * 2 * (num_kv_heads * edge + num_q_heads * heavy)
    qo_b = len(seq_lens) * num_q_heads * head_dim * 2 * 2
    return {"hash": hash_b, "kv": kv_b, "qo": qo_b, "total": hash_b + kv_b + qo_b}
