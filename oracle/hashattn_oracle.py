"""CPU oracle for the HashAttention sparse-decode path. TEST INFRASTRUCTURE, NOT PRODUCT CODE:
only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import it.

A restatement in plain torch-CPU ops of what the reference computes on this path, each
function citing the lines of hashattention/hashattention_llama.py it follows. The reference
itself is Python and cannot travel with the repository, so it was imported once where it is
available and its outputs were stored under tests/golden/ (script: tests/golden/make_golden.py);
tests/test_oracle_golden.py pins this restatement against those stored outputs.
Parity status: PINNED by reference-generated fixtures.

Two deliberate statements about ties and zeros, both inside what the reference leaves open:
  * the reference sorts with torch's default (unstable) sort (:430); the oracle, like the
    fixtures, uses a stable sort, i.e. ties at the budget threshold go to the lowest index;
  * the reference's sign() maps an exact 0.0 pre-activation to 0 (:55,:171-173); the packed
    code has no third state and stores bit 0 for it (as efficiency/kernels/torchatt.py:35,
    relu(sign(x)), does).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

BAND = 1e-5  # |pre-activation| below which a hash bit is excluded from bit-exact comparison


# ------------------------------------------------------------------------------------------
# hash encoder
# ------------------------------------------------------------------------------------------
def mlp_preact(nets, x: torch.Tensor) -> torch.Tensor:
    """Per-head MLP pre-activations. ``nets[h]`` is ``[(W0,b0),(W1,b1),(W2,b2)]`` (fp32, Linear
    layout [out,in]); ``x`` is ``[B, H, s, D]``; returns ``[B, H, s, 32]`` fp32.

    Follows the per-head loop of USA.forward / k_embedding / q_embedding
    (hashattention_llama.py:159-169, 204-226): Linear, SiLU, Linear, SiLU, Linear (:100-111).
    """
    outs = []
    for h, layers in enumerate(nets):
        y = x[:, h].to(torch.float32)
        if layers[0][0].shape[1] == y.shape[-1] + 1:
            y = ip_to_cs(y)  # the LSH baseline (lth_num_layers == 0, :130-139): Linear(129, 32) over the lifted vector
        for i, (w, b) in enumerate(layers):
            y = F.linear(y, w, b)
            if i + 1 < len(layers):
                y = F.silu(y)
        outs.append(y)
    return torch.stack(outs, dim=1)


def ip_to_cs(x: torch.Tensor) -> torch.Tensor:
    """IpToCS.forward (hashattention_llama.py:75-84): ``x [..., D] -> [..., D + 1]`` with the extra coordinate
    sqrt(relu(M^2 - |x|^2)), M = 1e-3 + the largest norm among ALL vectors passed (batch and positions)."""
    norm = x.norm(dim=-1).unsqueeze(-1)
    M = norm.max().item() + 1e-3
    return torch.cat([x, torch.sqrt(F.relu(M ** 2 - norm ** 2))], dim=-1)


def nets_from_usa(usa, side: str):
    """Extracts ``[(W,b)...]`` per head, up-cast to fp32, from a module with the reference's
    attribute layout (``learning_to_hash_transformation_{k,q}[h]``: a Sequential of 3, 2 or 1 Linear layers
    with SiLU between them; :99-127)."""
    mods = getattr(usa, f"learning_to_hash_transformation_{side}")
    return [[(layer.weight.detach().to(torch.float32), layer.bias.detach().to(torch.float32))
             for layer in m if hasattr(layer, "weight")] for m in mods]


def pack_codes(preact: torch.Tensor) -> torch.Tensor:
    """``[..., 32]`` pre-activations -> int64 codes in 0..2^32-1; bit i = (x_i > 0), LSB = output 0
    (efficiency/kernels/torchatt.py:35-36 with power = 2**arange(32), :159)."""
    bits = (preact > 0).to(torch.int64)
    weights = (2 ** torch.arange(preact.shape[-1], dtype=torch.int64))
    return (bits * weights).sum(dim=-1)


def band_mask(preact: torch.Tensor, band: float = BAND) -> torch.Tensor:
    """int64 mask per code with bit i set where |x_i| >= band, i.e. where the bit must match."""
    keep = (preact.abs() >= band).to(torch.int64)
    weights = (2 ** torch.arange(preact.shape[-1], dtype=torch.int64))
    return (keep * weights).sum(dim=-1)


def span_scores(q_pre: torch.Tensor, k_pre: torch.Tensor) -> torch.Tensor:
    """sign(q) . sign(k): ``[B,H,1,32] x [B,H,S,32] -> [B,H,S]`` (hashattention_llama.py:171-187)."""
    return torch.einsum("bhqd,bhsd->bhqs", torch.sign(q_pre), torch.sign(k_pre))[:, :, 0, :]


def hamming_scores(q_codes: torch.Tensor, k_codes: torch.Tensor) -> torch.Tensor:
    """popcount(~(q ^ k)) over 32 bits: ``[B,H] x [B,H,S] -> [B,H,S]`` int64
    (efficiency/kernels/torchatt.py:38-42). Equals (span + 32) / 2 when no pre-activation is 0."""
    x = (~(q_codes[..., None] ^ k_codes)) & 0xFFFFFFFF
    cnt = torch.zeros_like(x)
    for i in range(32):
        cnt += (x >> i) & 1
    return cnt


# ------------------------------------------------------------------------------------------
# budget selection
# ------------------------------------------------------------------------------------------
def heavy_tokens(seq_len: int, heavy_budget: float) -> int:
    """hashattention_llama.py:431-434."""
    return int(heavy_budget) if heavy_budget > 1.0 else int(seq_len * heavy_budget)


def select_mask(span: torch.Tensor, init_budget: int, recent_budget: int, heavy_budget: float,
                stable: bool = True, eval_mode: str = "simple", retrieve_depth: int = -1,
                bit_step: float = 1.0) -> torch.Tensor:
    """compute_mask_multi for q_len == 1 (hashattention_llama.py:423-443).

    ``span`` is ``[B, H, S]`` (any monotone score: the +-1 dot product or the Hamming count).
    ``eval_mode == 'simple'`` keeps the ``hb`` best candidates (:436-438); any other mode keeps
    every candidate scoring at least ``max(best - bit_step * retrieve_depth, hb-th best)``
    (:439-443), where ``bit_step`` is what one mismatching bit costs in the units of ``span``
    (2 for the reference's +-1 dot product, 1 for the Hamming count). Returns the bool keep-mask
    ``[B, H, S]``. In the non-simple mode ``hb == 0`` keeps no candidate (the reference raises there).
    """
    B, H, S = span.shape
    idx = torch.arange(S)
    cand = idx <= S - 1 - recent_budget          # tril(ones(1,k), diagonal=k-q-recent), q = 1   (:423)
    cand[:init_budget] = False                   # (:424)
    span = span.to(torch.float32).masked_fill(~cand, torch.finfo(torch.float32).min)   # (:426)
    mask = (~cand)[None, None, :].expand(B, H, S).clone()    # all-true causal row times ~cand   (:427-428)
    values, indices = span.sort(dim=-1, descending=True, stable=stable)                 # (:430)
    hb = heavy_tokens(S, heavy_budget)
    if eval_mode == "simple":
        mask.scatter_(2, indices[:, :, :hb], True)                                      # (:437-438)
        return mask
    if hb < 1:
        return mask
    hb = min(hb, S)  # (the reference raises for hb > S; here the smallest value stands in)
    depth_thold = values[:, :, :1] - bit_step * retrieve_depth                           # (:440)
    num_thold = values[:, :, hb - 1:hb]                                                 # (:441)
    thold = torch.maximum(depth_thold, num_thold)                                       # (:442)
    mask |= (span >= thold) & cand[None, None, :]                                       # (:443) masked entries never count
    return mask


def selected_sets(mask: torch.Tensor):
    """``[B,H,S]`` mask -> nested list of ascending index tensors."""
    return [[mask[b, h].nonzero()[:, 0] for h in range(mask.shape[1])] for b in range(mask.shape[0])]


def heavy_sets(mask: torch.Tensor, init_budget: int, recent_budget: int):
    """The selected indices that are neither sink nor recent tokens (what ha_score_select emits)."""
    S = mask.shape[-1]
    lo = min(init_budget, S)
    hi = max(lo, S - recent_budget)
    out = []
    for b in range(mask.shape[0]):
        row = []
        for h in range(mask.shape[1]):
            idx = mask[b, h].nonzero()[:, 0]
            row.append(idx[(idx >= lo) & (idx < hi)])
        out.append(row)
    return out


# ------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------
def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """hashattention_llama.py:578-623 for q_len == 1 in fp32: repeat_kv, QK^T/sqrt(d), fill of the
    unselected positions with finfo.min, fp32 softmax, .V.
    ``q [B,Hq,D]``, ``k,v [B,Hkv,S,D]``, ``mask [B,Hq,S]`` -> ``[B,Hq,D]`` fp32."""
    B, Hq, D = q.shape
    group = Hq // k.shape[1]
    kk = k.to(torch.float32).repeat_interleave(group, dim=1)      # repeat_kv (:578-579)
    vv = v.to(torch.float32).repeat_interleave(group, dim=1)
    w = torch.einsum("bhd,bhsd->bhs", q.to(torch.float32), kk) / math.sqrt(D)   # (:585)
    w = w.masked_fill(~mask, torch.finfo(torch.float32).min)                     # (:606)
    w = torch.softmax(w, dim=-1, dtype=torch.float32)                            # (:613)
    return torch.einsum("bhs,bhsd->bhd", w, vv)                                  # (:615)


# ------------------------------------------------------------------------------------------
# multi-token decode (2 <= q_len <= 128 query tokens in one call)
# ------------------------------------------------------------------------------------------
def select_mask_rows(span: torch.Tensor, init_budget: int, recent_budget: int, heavy_budget: float,
                     stable: bool = True, eval_mode: str = "simple", retrieve_depth: int = -1,
                     bit_step: float = 1.0) -> torch.Tensor:
    """compute_mask_multi for ``q`` query tokens against ``k`` keys (hashattention_llama.py:423-443):
    ``span [B,H,q,k]`` -> keep-mask ``[B,H,q,k]``. Query ``i`` sits at key position ``k - q + i``; its
    candidates are the keys ``init <= j <= k - q + i - recent`` (:423-424), the budget is
    ``int(k * heavy_budget)`` for every row (:431-434). As in the reference, surplus budget of a row
    (``hb`` > its candidates) falls on masked positions in index order, which can include positions
    after the query; the causal attention mask removes those again (masked_attention_rows)."""
    B, H, q, k = span.shape
    cand = torch.tril(torch.ones(q, k), diagonal=k - q - recent_budget).bool()            # (:423)
    cand[:, :init_budget] = False                                                         # (:424)
    span = span.to(torch.float32).masked_fill(~cand, torch.finfo(torch.float32).min)      # (:426)
    causal = torch.tril(torch.ones(q, k), diagonal=k - q).bool()                          # (:427)
    mask = (causal & ~cand)[None, None].expand(B, H, q, k).clone()                        # (:428)
    values, indices = span.sort(dim=-1, descending=True, stable=stable)                   # (:430)
    hb = heavy_tokens(k, heavy_budget)
    if eval_mode == "simple":
        mask.scatter_(3, indices[..., :hb], True)                                         # (:437-438)
        return mask
    if hb < 1:
        return mask
    hb = min(hb, k)
    thold = torch.maximum(values[..., :1] - bit_step * retrieve_depth, values[..., hb - 1:hb])   # (:440-442)
    mask |= (span >= thold) & cand[None, None]                                            # (:443)
    return mask


def masked_attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """hashattention_llama.py:578-623 for q_len > 1 in fp32 with the causal attention mask a decoder
    passes (:593-598): ``q [B,Hq,q,D]``, ``k,v [B,Hkv,S,D]``, ``mask [B,Hq,q,S]`` -> ``[B,Hq,q,D]``."""
    B, Hq, ql, D = q.shape
    S = k.shape[2]
    group = Hq // k.shape[1]
    kk = k.to(torch.float32).repeat_interleave(group, dim=1)
    vv = v.to(torch.float32).repeat_interleave(group, dim=1)
    w = torch.einsum("bhqd,bhsd->bhqs", q.to(torch.float32), kk) / math.sqrt(D)           # (:585)
    causal = torch.tril(torch.ones(ql, S), diagonal=S - ql).bool()
    w = w + torch.zeros(ql, S).masked_fill(~causal, torch.finfo(torch.float32).min)       # (:593-598)
    w = w.masked_fill(~mask, torch.finfo(torch.float32).min)                              # (:606)
    w = torch.softmax(w, dim=-1, dtype=torch.float32)                                     # (:613)
    return torch.einsum("bhqs,bhsd->bhqd", w, vv)                                         # (:615)


def decode_chunk(usa, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, init_budget: int, recent_budget: int,
                 heavy_budget: float, eval_mode: str = "simple", retrieve_depth: int = -1) -> torch.Tensor:
    """decode_step for ``q_len`` query tokens: ``q [B,Hq,q_len,D]``, ``k,v [B,Hkv,S,D]`` with the chunk's
    tokens last -> ``[B,Hq,q_len,D]`` (hashattention_llama.py:529-623 with a causal attention mask)."""
    group = q.shape[1] // k.shape[1]
    k_rep = k.to(torch.float32).repeat_interleave(group, dim=1)
    k_pre = mlp_preact(nets_from_usa(usa, "k"), k_rep)
    q_pre = mlp_preact(nets_from_usa(usa, "q"), q)
    span = torch.einsum("bhqd,bhsd->bhqs", torch.sign(q_pre), torch.sign(k_pre))          # (:171-187)
    mask = select_mask_rows(span, init_budget, recent_budget, heavy_budget, eval_mode=eval_mode,
                            retrieve_depth=retrieve_depth, bit_step=2.0)
    return masked_attention_rows(q, k, v, mask)


def cached_span(usa, q: torch.Tensor, k_new: torch.Tensor, past_signs: torch.Tensor, group: int) -> torch.Tensor:
    """The reference's cached-signature branch of compute_mask_multi (hashattention_llama.py:409-420),
    which it keeps disabled (:407-408): q_embedding of the query (:411), k_embedding of only the keys
    that are not cached yet (:412), concatenation with the stored signs (:413-414), one baddbmm (:415-420).
    ``q [B,Hq,D]``, ``k_new [B,Hkv,n,D]`` (the keys beyond the cached ones), ``past_signs [B,Hq,S-n,32]``
    (+-1) -> span ``[B,Hq,S]``."""
    q_sign = torch.sign(mlp_preact(nets_from_usa(usa, "q"), q[:, :, None, :]))                   # (:216-226)
    k_rep = k_new.to(torch.float32).repeat_interleave(group, dim=1)
    k_sign = torch.sign(mlp_preact(nets_from_usa(usa, "k"), k_rep))                              # (:204-214)
    total = torch.cat([past_signs, k_sign], dim=-2)                                              # (:413)
    B, H, S, W = total.shape
    span = torch.baddbmm(torch.empty(B * H, 1, S), q_sign.reshape(B * H, 1, W),
                         total.reshape(B * H, S, W).transpose(1, 2), beta=0, alpha=1.0)          # (:415-420)
    return span.reshape(B, H, S)


# ------------------------------------------------------------------------------------------
# the whole step, structured like the reference (re-hashes every key, full sort, dense softmax)
# ------------------------------------------------------------------------------------------
def decode_step(usa, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, init_budget: int,
                recent_budget: int, heavy_budget: float, return_parts: bool = False,
                eval_mode: str = "simple", retrieve_depth: int = -1):
    """One layer's decode attention for one uniform batch, with the cost structure of the
    reference's forward (hashattention_llama.py:578-623 + compute_mask_multi :401-446):
    every key is hashed again with the 32 key MLPs, scores are sorted in full, attention is
    dense over S with a mask. This is the function timed as the CPU baseline.

    ``q [B,Hq,D]``, ``k,v [B,Hkv,S,D]`` (post-RoPE, the new token's row last).
    """
    group = q.shape[1] // k.shape[1]
    k_rep = k.to(torch.float32).repeat_interleave(group, dim=1)                  # (:578)
    k_pre = mlp_preact(nets_from_usa(usa, "k"), k_rep)                           # (:168)
    q_pre = mlp_preact(nets_from_usa(usa, "q"), q[:, :, None, :])                # (:169)
    span = span_scores(q_pre, k_pre)                                             # (:171-187)
    mask = select_mask(span, init_budget, recent_budget, heavy_budget, eval_mode=eval_mode,
                       retrieve_depth=retrieve_depth, bit_step=2.0)              # (:423-443)
    out = masked_attention(q, k, v, mask)                                        # (:585-615)
    if return_parts:
        return out, dict(q_pre=q_pre[:, :, 0, :], k_pre=k_pre, span=span, mask=mask)
    return out
