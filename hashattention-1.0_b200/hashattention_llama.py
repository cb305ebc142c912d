"""The reference's user-facing API for Llama models, backed by the sm_100a kernels:
``load_usa``, ``convert_usa``, ``reset_usa`` and the attention module
``LlamaAttention_heavy_hitter`` (hashattention/hashattention_llama.py:229-680 of the reference).

    from hashattention_b200.hashattention_llama import convert_usa, load_usa
    config.lth_init_dim = 128; config.lth_final_dim = 32; config.lth_thold = 0; config.lth_num_layers = 3
    config.init_budget = 128; config.heavy_budget = 0.25; config.recent_budget = 128
    config.usa_eval_mode = "simple"; config.usa_retrieve_depth = -1
    usa_modules = load_usa(config, patch_path)
    model = convert_usa(model, config, usa_modules, collect_stats=False, train_usa=False)

What runs where
  * q_len == 1 (decode): q/k/v projections, RoPE and o_proj stay torch ops; the hash encode of
    the new query and key, the cache append, Hamming scoring, budget selection and the sparse
    attention are one call into the CUDA library (the registered operator torch.ops.hashattn.decode_step).
  * q_len > 128 (prefill): the original attention forward runs, as in the reference (:529-550);
    afterwards the layer's keys / values are copied into this module's paged cache and the key
    hashes are built once by the CUDA library. (The reference keeps no key hashes and re-encodes
    every cached key on every decode step, :405-408.)
  * Both ``usa_eval_mode`` settings are implemented: 'simple' (the ``hb`` best candidates) and the
    depth rule of every other mode string (:439-443).
  * 2 <= q_len <= 128 (chunked / speculative decode, :529): the same library path with one row per
    (sequence, new token); needs ``recent_budget >= q_len - 1``.
  * Training (``train_usa``) and statistics (``collect_stats``) are not implemented and raise
    ``NotImplementedError``.
  * Padded batches: the paged cache stores whole sequences from token 0, so an ``attention_mask`` that
    hides keys (left- or right-padding of a batch of prompts) is refused with ``NotImplementedError``
    at prefill instead of silently attending the pad tokens (the reference adds the mask to the
    attention weights, :593-603). Decode one sequence, or equal-length prompts, per batch.

Memory: this module keeps its own paged copy of the layer's K / V (bf16, 512 B per token and kv-head) next to
the caller's cache object, sized for the prompt plus ``config.usa_decode_headroom`` new tokens (default 4096)
and never beyond ``config.usa_max_seq_len`` (default ``max_position_embeddings``). The number of cached tokens
is tracked on the host; a step that would not fit raises ``ValueError`` before anything is launched.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn

from .cache import PAGE, PagedHashKVCache
from .ops import Budget, ChunkRows, SparseDecodeContext
from .torch_ops import decode_step_op
from .usa import USA

__all__ = ["USA", "LlamaAttention_heavy_hitter", "load_usa", "convert_usa", "reset_usa", "set_eval_usa_mode",
           "set_train_usa_mode", "print_stats"]


def _rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _apply_rotary(q, k, cos, sin):
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return q * cos + _rotate_half(q) * sin, k * cos + _rotate_half(k) * sin


def _layer_kv(cache, layer_idx):
    """Keys / values ``[B, Hkv, S, D]`` of one layer from a transformers cache object, old
    (``key_cache`` lists, as the reference uses at :329-330) or new (``layers[i].keys``) style."""
    if hasattr(cache, "key_cache"):
        return cache.key_cache[layer_idx], cache.value_cache[layer_idx]
    layer = cache.layers[layer_idx]
    return layer.keys, layer.values


class LlamaAttention_heavy_hitter(nn.Module):
    """Attention layer with HashAttention sparse decode; constructor and attributes as the
    reference's class of the same name (hashattention/hashattention_llama.py:229-292)."""

    def __init__(self, config, layer_idx: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = getattr(config, "head_dim", None) or self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.max_position_embeddings = config.max_position_embeddings
        if self.head_dim * self.num_heads != self.hidden_size:
            raise ValueError(
                f"hidden_size must be divisible by num_heads (got `hidden_size`: {self.hidden_size}"
                f" and `num_heads`: {self.num_heads})."
            )
        if self.head_dim != 128 or self.num_key_value_groups != 4:
            raise NotImplementedError("the sm_100a kernels implement head_dim 128 with 4 query heads per kv head")
        bias = getattr(config, "attention_bias", False)
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=bias)

        self.init_budget = config.init_budget
        self.heavy_budget = config.heavy_budget
        self.recent_budget = config.recent_budget
        self.usa_retrieve_depth = getattr(config, "usa_retrieve_depth", -1)
        self.usa_eval_mode = config.usa_eval_mode
        self.usa_module: Optional[USA] = None
        self.usa_module_dtype = None
        self.collect_stats = False
        self.train_usa = False
        self.flash_forward = None  # the replaced module's forward, used for prefill
        # longest sequence the paged cache may be sized for; set config.usa_max_seq_len to change it
        self.max_seq_len = int(getattr(config, "usa_max_seq_len", self.max_position_embeddings))
        # tokens of room the cache gets beyond the prompt it was created for
        self.decode_headroom = int(getattr(config, "usa_decode_headroom", 4096))
        self._ctx: Optional[SparseDecodeContext] = None
        self._cached_tokens = 0  # host-side copy of the cache's sequence length (all sequences advance together)
        self._steps_since_status_check = 0

    def __repr__(self):
        return (f"{super().__repr__()}\nSparsification Setting(topk:{self.heavy_budget}  edge:{self.init_budget, self.recent_budget} \n"
                f" eval_mode:{self.usa_eval_mode} stats:{self.collect_stats}\n Istraining:{self.train_usa} )")

    # the reference's per-sequence state is `past_key_signatures` (:275, :298-301); here it is the
    # hash pages of the paged cache
    def _reset_state(self):
        if self._ctx is not None:
            self._ctx.check_status()  # a problem a kernel reported since the last check surfaces here at the latest
            self._ctx.cache.reset()
        self._cached_tokens = 0

    def _context(self, batch: int, device, need_tokens: int = 0) -> SparseDecodeContext:
        """The decode context for ``batch`` sequences; (re)built when the batch, the device or the room
        needed (``need_tokens``, at prefill) changes."""
        ctx = self._ctx
        if ctx is None or ctx.batch != batch or ctx.device != device or need_tokens > ctx.cache.max_pages * PAGE:
            if self.usa_module is None:
                raise RuntimeError("no usa_module attached: build the model with convert_usa")
            capacity = min(self.max_seq_len, max(need_tokens, 1) + self.decode_headroom) if need_tokens else self.max_seq_len
            cache = PagedHashKVCache(batch, self.num_key_value_heads, capacity, device)
            budget = Budget(self.init_budget, self.heavy_budget, self.recent_budget,
                            "simple" if self.usa_eval_mode == "simple" else "depth", int(self.usa_retrieve_depth))
            self._ctx = ctx = SparseDecodeContext(cache, budget, self.usa_module.packed(device))
            ctx.row_contexts = {}  # q_len -> context over ChunkRows of this cache; dies with the context
            self._cached_tokens = 0
        return ctx

    def _rows_context(self, ctx: SparseDecodeContext, q_len: int) -> SparseDecodeContext:
        """The context of a multi-token step of ``q_len`` tokens per sequence: rows over the same cache."""
        if q_len not in ctx.row_contexts:
            ctx.row_contexts[q_len] = SparseDecodeContext(ChunkRows(ctx.cache, q_len), ctx.budget, ctx.weights)
        return ctx.row_contexts[q_len]

    @staticmethod
    def _hides_keys(attention_mask) -> bool:
        """Whether the mask hides a key from the last query (padding), in the forms a decoder passes:
        [B, S] of 0 / 1, or [B, 1, q, S] either boolean (True = visible) or additive (0 = visible)."""
        if attention_mask is None:
            return False
        if attention_mask.dim() == 2:
            return bool((attention_mask == 0).any())
        last = attention_mask[..., -1, :]
        return bool((~last).any()) if last.dtype == torch.bool else bool((last != 0).any())

    def _prefill(self, hidden_states, past, kwargs, new_style):
        if self.flash_forward is None:
            raise RuntimeError("prefill needs the original attention forward (set by convert_usa)")
        if hidden_states.shape[0] > 1 and self._hides_keys(kwargs.get("attention_mask")):
            raise NotImplementedError(
                "padded batches are not supported: the paged cache stores whole sequences, so pad tokens would be "
                "attended (the reference masks them, hashattention_llama.py:593-603); use equal-length prompts")
        out = self.flash_forward(hidden_states=hidden_states, **kwargs)
        if past is not None:
            k, v = _layer_kv(past, self.layer_idx)  # post-RoPE keys, all tokens so far
            if k.shape[2] > self.max_seq_len:
                raise ValueError(f"sequence of {k.shape[2]} tokens exceeds usa_max_seq_len={self.max_seq_len}")
            ctx = self._context(k.shape[0], k.device, need_tokens=k.shape[2])
            for b in range(k.shape[0]):
                ctx.cache.write_kv(b, k[b], v[b])
            ctx.hash_prefill()
            self._cached_tokens = k.shape[2]
        return out

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.LongTensor] = None, past_key_value=None,
                output_attentions: bool = False, use_cache: bool = False,
                cache_position: Optional[torch.LongTensor] = None,
                position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, **kwargs):
        """Signature of the reference's forward (:514-525). Newer transformers pass the cache as
        ``past_key_values`` and expect ``(attn_output, attn_weights)``; that convention is
        detected and answered in kind, otherwise the reference's 3-tuple is returned."""
        new_style = "past_key_values" in kwargs
        past = kwargs.pop("past_key_values") if new_style else past_key_value
        bsz, q_len, _ = hidden_states.size()
        if self.train_usa or self.collect_stats:
            raise NotImplementedError("hash training and statistics collection are not implemented")
        if q_len > 128:
            fwd = dict(attention_mask=attention_mask, position_ids=position_ids, output_attentions=output_attentions,
                       use_cache=use_cache, cache_position=cache_position, position_embeddings=position_embeddings,
                       **kwargs)
            fwd["past_key_values" if new_style else "past_key_value"] = past
            return self._prefill(hidden_states, past, fwd, new_style)
        if q_len > 1 and self.recent_budget < q_len - 1:
            raise NotImplementedError("multi-token decode needs recent_budget >= q_len - 1")
        if position_embeddings is None:
            raise ValueError("position_embeddings=(cos, sin) is required")

        q = self.q_proj(hidden_states).view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = _apply_rotary(q, k, cos, sin)
        if past is not None:  # keeps the caller's cache object consistent (sequence length bookkeeping)
            past.update(k, v, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})

        ctx = self._context(bsz, hidden_states.device)
        room = ctx.cache.max_pages * PAGE
        if self._cached_tokens + q_len > room:  # (the kernels would report it and write nothing)
            raise ValueError(f"the sequence would grow to {self._cached_tokens + q_len} tokens, the cache holds {room}: "
                             f"raise config.usa_decode_headroom (now {self.decode_headroom}) or config.usa_max_seq_len")
        self._cached_tokens += q_len
        self._steps_since_status_check += 1
        if self._steps_since_status_check >= 256:  # an occasional look at the device status word (synchronises)
            self._steps_since_status_check = 0
            ctx.check_status()
        if q_len == 1:
            ctx.cache.seq_lens += 1
            out = torch.zeros(bsz, self.num_heads, self.head_dim, dtype=torch.bfloat16, device=hidden_states.device)
            decode_step_op(ctx, q[:, :, 0].to(torch.bfloat16).contiguous(), k[:, :, 0].to(torch.bfloat16).contiguous(),
                           v[:, :, 0].to(torch.bfloat16).contiguous(), out=out)
        else:
            # 2 <= q_len <= 128 (:529): one row per (sequence, new token), each a single-token problem on
            # the keys up to its own with the budget of the whole length (:423-434)
            rctx = self._rows_context(ctx, q_len)
            rctx.cache.advance()

            def rows(t):  # [B, heads, q_len, D] -> [B * q_len, heads, D]
                return t.transpose(1, 2).reshape(bsz * q_len, t.shape[1], self.head_dim).to(torch.bfloat16).contiguous()

            out = rctx.decode_step_rows(rows(q), rows(k), rows(v))
        attn_output = self.o_proj(out.reshape(bsz, q_len, self.hidden_size).to(hidden_states.dtype))
        if new_style:
            return attn_output, None
        return attn_output, None, past


def load_usa(config, path, device="cuda"):
    """One hash-encoder module per layer, optionally loaded from a state dict saved by the
    reference (hashattention/hashattention_llama.py:633-646); ends on ``device`` ("cuda" there)."""
    cfg = {"lth_int_dim": config.lth_init_dim, "lth_final_dim": config.lth_final_dim,
           "lth_thold": config.lth_thold, "lth_num_layers": config.lth_num_layers}
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    mods = nn.ModuleList([USA(config.num_attention_heads, head_dim, cfg) for _ in range(config.num_hidden_layers)])
    if path is not None:
        mods.load_state_dict(torch.load(path))
    return mods.to(device)


def _llama_attention_class():
    from transformers.models.llama.modeling_llama import LlamaAttention
    return LlamaAttention


def _convert(model, config, usa_modules, collect_stats, train_usa, attention_cls, heavy_cls):
    """convert_usa for one host model family: ``attention_cls`` modules become ``heavy_cls``."""
    if collect_stats or train_usa:
        raise NotImplementedError("collect_stats / train_usa are not implemented")
    for name, module in reversed(list(model._modules.items())):
        if len(list(module.children())) > 0:
            model._modules[name] = _convert(module, config, usa_modules, collect_stats, train_usa, attention_cls,
                                            heavy_cls)
        if isinstance(module, attention_cls):
            device = next(module.parameters()).device
            new_module = heavy_cls(config, module.layer_idx).bfloat16().to(device)
            new_module.load_state_dict(module.state_dict())
            new_module.usa_module = usa_modules[module.layer_idx]
            new_module.usa_module_dtype = usa_modules[module.layer_idx].learning_to_hash_transformation_k[0][-1].weight.dtype
            new_module.flash_forward = module.forward
            new_module.collect_stats = collect_stats
            new_module.train_usa = train_usa
            model._modules[name] = new_module
    return model


def convert_usa(model, config, usa_modules, collect_stats, train_usa):
    """Swaps every ``LlamaAttention`` of ``model`` for ``LlamaAttention_heavy_hitter`` (bf16, same
    device, same projection weights), attaches that layer's hash module and keeps the replaced
    module's forward for prefill (hashattention/hashattention_llama.py:650-667)."""
    return _convert(model, config, usa_modules, collect_stats, train_usa, _llama_attention_class(),
                    LlamaAttention_heavy_hitter)


def reset_usa(model):
    """Forgets the cached sequences of every converted layer; call between prompts
    (hashattention/hashattention_llama.py:670-680)."""
    for name, module in reversed(list(model._modules.items())):
        if len(list(module.children())) > 0:
            model._modules[name] = reset_usa(module)
        if isinstance(module, LlamaAttention_heavy_hitter):
            module._reset_state()
    return model


def set_eval_usa_mode(model):
    """Counterpart of the reference's switch out of hash training (:700-710); training is not
    implemented here, so this only clears the flag."""
    for name, module in reversed(list(model._modules.items())):
        if len(list(module.children())) > 0:
            model._modules[name] = set_eval_usa_mode(module)
        if isinstance(module, LlamaAttention_heavy_hitter):
            module.train_usa = False
    return model


def set_train_usa_mode(model, loss_func=None, optimizer=None):
    """The reference's switch into hash training (:683-697). Training the hash functions is outside this
    library (it evaluates trained ones), so this refuses instead of silently decoding untrained."""
    raise NotImplementedError("hash training (train_usa) is not implemented: train with the reference, load with load_usa")


def print_stats(model):
    """The reference prints the overlap statistics it collected during prefill (:713-726). Statistics are not
    collected inside forward here; diagnostics/recall.py computes the same statistic on demand."""
    raise NotImplementedError("collect_stats is not implemented: see diagnostics/recall.py for the overlap statistic")

