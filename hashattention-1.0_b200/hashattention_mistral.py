"""Mistral host of the same attention layer: the reference keeps a second copy of its module for
``MistralAttention`` (hashattention/hashattention_mistral.py:582-596, same ``load_usa`` /
``convert_usa`` / ``reset_usa`` API); here it is the Llama module under the Mistral name - the
decode path (projections, RoPE, GQA with 4 query heads per kv-head, head_dim 128) is identical
and never looks at the host model's class. As in the reference, the sparse decode path ignores
``sliding_window``.
"""
from __future__ import annotations

from .hashattention_llama import (LlamaAttention_heavy_hitter, _convert, load_usa, reset_usa,  # noqa: F401
                                  set_eval_usa_mode)
from .usa import USA  # noqa: F401

__all__ = ["USA", "MistralAttention_heavy_hitter", "load_usa", "convert_usa", "reset_usa", "set_eval_usa_mode"]


class MistralAttention_heavy_hitter(LlamaAttention_heavy_hitter):
    """``MistralAttention`` with HashAttention sparse decode (hashattention/hashattention_mistral.py:170-240)."""


def convert_usa(model, config, usa_modules, collect_stats, train_usa):
    """Swaps every ``MistralAttention`` of ``model`` for ``MistralAttention_heavy_hitter``
    (hashattention/hashattention_mistral.py:582-596)."""
    from transformers.models.mistral.modeling_mistral import MistralAttention

    return _convert(model, config, usa_modules, collect_stats, train_usa, MistralAttention,
                    MistralAttention_heavy_hitter)
