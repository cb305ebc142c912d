"""Generates the golden fixtures in this directory by running the REFERENCE implementation.

Needs a checkout of the reference project (environment variable HASHATTN_REFERENCE points at
its root) and runs on CPU:

    HASHATTN_REFERENCE=<reference checkout> python tests/golden/make_golden.py [case_a|edge|config0|depth|rows ...]

For every case it imports hashattention/hashattention_llama.py unmodified, builds the
reference's USA module and LlamaAttention_heavy_hitter, and records
  * the key / query hash pre-activation signs as packed codes plus a "must match" mask
    (bits whose |pre-activation| >= 1e-5) from the reference's own MLP modules,
  * span scores from USA.forward(hard=True)                       (:151-200),
  * the keep-mask from compute_mask_multi                          (:401-446),
  * the attention output of LlamaAttention_heavy_hitter.forward    (:514-631), decode branch.
Small cases also store their inputs (bf16 bit patterns); the config-0 case stores the seeds
and a SHA-256 of the inputs.

Shims (the reference file is not edited): rope_theta set on the config (transformers >= 5 no
longer defines it), a list cache exposing .key_cache/.value_cache/.update, q/k/v/o projections
replaced by modules that return the prepared post-RoPE tensors, cos=1/sin=0 position
embeddings, and torch.Tensor.sort made stable while the reference runs, so ties at the budget
threshold go to the lowest index.
"""
from __future__ import annotations

import contextlib
import hashlib
import os
import sys

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("HASHATTN_REFERENCE")
if not REF or not os.path.isdir(REF):
    sys.exit("set HASHATTN_REFERENCE to the root of a checkout of the reference project")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
from hashattention_b200 import synthetic  # noqa: E402

import hashattention.hashattention_llama as H  # noqa: E402  (the reference)
from transformers import LlamaConfig  # noqa: E402

BAND = 1e-5
_sort = torch.Tensor.sort


@contextlib.contextmanager
def stable_sort():
    torch.Tensor.sort = lambda self, *a, **k: _sort(self, *a, **{**k, "stable": k.get("stable", True)})
    try:
        yield
    finally:
        torch.Tensor.sort = _sort


class Const(nn.Module):
    def __init__(self, value):
        super().__init__()
        self.value = value

    def forward(self, _x):
        return self.value


class ListCache:
    def __init__(self, k, v):
        self.key_cache, self.value_cache = [k], [v]

    def update(self, k, v, layer_idx, cache_kwargs=None):
        self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], k], dim=-2)
        self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], v], dim=-2)
        return self.key_cache[layer_idx], self.value_cache[layer_idx]


def reference_modules(Hq, Hkv, init, recent, heavy, seed=0, bf16_weights=True, eval_mode="simple", depth=-1, layers=3):
    cfg = LlamaConfig(hidden_size=Hq * 128, num_attention_heads=Hq, num_key_value_heads=Hkv, num_hidden_layers=1,
                      intermediate_size=256, vocab_size=128, max_position_embeddings=131072,
                      rope_parameters={"rope_theta": 500000.0, "rope_type": "default"})
    cfg.rope_theta = 500000.0
    for k, v in dict(lth_init_dim=128, lth_final_dim=32, lth_thold=0, lth_num_layers=layers, init_budget=init,
                     heavy_budget=heavy, recent_budget=recent, usa_eval_mode=eval_mode, usa_retrieve_depth=depth).items():
        setattr(cfg, k, v)
    torch.manual_seed(seed)
    usa = H.USA(Hq, 128, {"lth_int_dim": 128, "lth_final_dim": 32, "lth_thold": 0, "lth_num_layers": layers})
    mine = synthetic.make_usa(Hq, 128, seed=seed, bf16=False, num_layers=layers)
    for (n1, p1), (n2, p2) in zip(usa.state_dict().items(), mine.state_dict().items()):
        assert n1 == n2 and torch.equal(p1, p2), f"USA mirror differs from the reference at {n1}"
    if bf16_weights:
        usa = usa.bfloat16().float()
    att = H.LlamaAttention_heavy_hitter(cfg, 0)
    att.usa_module, att.usa_module_dtype, att.offloading_length = usa, torch.float32, 10 ** 12
    return cfg, usa, att


def run_reference(att, usa, q, k, v):
    """q [B,Hq,128], k/v [B,Hkv,S,128] (post-RoPE, new token last) -> dict of reference outputs."""
    B, Hq, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    group = Hq // Hkv
    with torch.no_grad(), stable_sort():
        k_rep = H.repeat_kv(k, group)
        q4 = q[:, :, None, :]
        k_pre = torch.stack([usa.learning_to_hash_transformation_k[i](k_rep[:, i]) for i in range(Hq)], dim=1)
        q_pre = torch.stack([usa.learning_to_hash_transformation_q[i](q4[:, i]) for i in range(Hq)], dim=1)[:, :, 0]
        span, _ = usa(k_rep, q4, hard=True)
        mask = att.compute_mask_multi(k_rep.clone(), q4)
        att.q_proj = Const(q.reshape(B, 1, Hq * D))
        att.k_proj = Const(k[:, :, -1].reshape(B, 1, Hkv * D))
        att.v_proj = Const(v[:, :, -1].reshape(B, 1, Hkv * D))
        att.o_proj = nn.Identity()
        cache = ListCache(k[:, :, :-1].clone(), v[:, :, :-1].clone())
        pos = (torch.ones(B, 1, D), torch.zeros(B, 1, D))
        out, _, _ = att(torch.zeros(B, 1, Hq * D), past_key_value=cache, position_embeddings=pos)
    return dict(k_pre=k_pre, q_pre=q_pre, span=span[:, :, 0], mask=mask[:, :, 0], out=out.reshape(B, Hq, D))


def run_reference_rows(att, usa, q, k, v):
    """Multi-token decode through the reference: q [B,Hq,ql,128] (the last ql tokens' queries), k/v
    [B,Hkv,S,128] with the ql new tokens last. The decoder's causal attention mask is passed as a
    transformers model would (:593-598)."""
    B, Hq, ql, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    group = Hq // Hkv
    with torch.no_grad(), stable_sort():
        k_rep = H.repeat_kv(k, group)
        span, _ = usa(k_rep, q, hard=True)
        mask = att.compute_mask_multi(k_rep.clone(), q)
        att.q_proj = Const(q.transpose(1, 2).reshape(B, ql, Hq * D))
        att.k_proj = Const(k[:, :, -ql:].transpose(1, 2).reshape(B, ql, Hkv * D))
        att.v_proj = Const(v[:, :, -ql:].transpose(1, 2).reshape(B, ql, Hkv * D))
        att.o_proj = nn.Identity()
        cache = ListCache(k[:, :, :-ql].clone(), v[:, :, :-ql].clone())
        pos = (torch.ones(B, ql, D), torch.zeros(B, ql, D))
        causal = torch.tril(torch.ones(ql, S), diagonal=S - ql).bool()
        amask = torch.zeros(ql, S).masked_fill(~causal, torch.finfo(torch.float32).min)[None, None].expand(B, 1, ql, S)
        out, _, _ = att(torch.zeros(B, ql, Hq * D), attention_mask=amask, past_key_value=cache, position_embeddings=pos)
    return dict(span=span, mask=mask, out=out.reshape(B, ql, Hq, D).transpose(1, 2))


def pack(pre):
    w = 2 ** torch.arange(32, dtype=torch.int64)
    return ((pre > 0).to(torch.int64) * w).sum(-1)


def must(pre):
    w = 2 ** torch.arange(32, dtype=torch.int64)
    return ((pre.abs() >= BAND).to(torch.int64) * w).sum(-1)


def u32(x):
    return x.numpy().astype(np.uint32)


def bf16_bits(x):
    return x.to(torch.bfloat16).view(torch.int16).numpy()


def outputs_to_arrays(r, prefix=""):
    span = r["span"]
    assert float((span - span.round()).abs().max()) == 0.0
    return {
        prefix + "k_codes": u32(pack(r["k_pre"])), prefix + "k_must": u32(must(r["k_pre"])),
        prefix + "q_codes": u32(pack(r["q_pre"])), prefix + "q_must": u32(must(r["q_pre"])),
        prefix + "span": span.to(torch.int8).numpy(),
        prefix + "mask": np.packbits(r["mask"].numpy(), axis=-1),
        prefix + "out": r["out"].numpy().astype(np.float32),
        prefix + "n_zero_preact": np.int64(int((r["k_pre"] == 0).sum() + (r["q_pre"] == 0).sum())),
    }


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().numpy().tobytes())
    return h.hexdigest()


def case_a():
    Hq, Hkv, S, init, recent, heavy = 8, 2, 520, 16, 16, 1.0 / 8
    inp = synthetic.make_decode_inputs(90, [S, S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy)
    arrays = outputs_to_arrays(run_reference(att, usa, q, k, v))
    arrays.update(q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                  meta=np.array([Hq, Hkv, S, init, recent], dtype=np.int64), heavy=np.float64(heavy))
    np.savez_compressed(os.path.join(HERE, "case_a.npz"), **arrays)


EDGE_SUBCASES = [
    # name, S, init, recent, heavy
    ("short", 100, 128, 128, 1.0 / 32),     # S < init + recent: no candidates, everything kept
    ("one_cand", 257, 128, 128, 1.0 / 32),  # exactly one candidate, budget 8 > candidates
    ("p255", 255, 16, 16, 1.0 / 8),         # page boundary - 1
    ("p256", 256, 16, 16, 1.0 / 8),         # exactly one page
    ("p257", 257, 16, 16, 1.0 / 8),         # page boundary + 1
    ("abs48", 300, 4, 8, 48.0),             # heavy_budget > 1.0: absolute token count
    ("all", 300, 0, 0, 1.0),                # heavy_budget == 1.0: fraction, selects every token
    ("zero_heavy", 300, 8, 8, 0.0),         # no heavy tokens at all
]


def edge():
    Hq, Hkv, S = 4, 1, 300
    inp = synthetic.make_decode_inputs(91, [S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    arrays = dict(q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), meta=np.array([Hq, Hkv, S], dtype=np.int64),
                  names=np.array([c[0] for c in EDGE_SUBCASES]),
                  params=np.array([[c[1], c[2], c[3]] for c in EDGE_SUBCASES], dtype=np.int64),
                  heavy=np.array([c[4] for c in EDGE_SUBCASES], dtype=np.float64))
    for name, s, init, recent, heavy in EDGE_SUBCASES:
        _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy)
        arrays.update(outputs_to_arrays(run_reference(att, usa, q, k[:, :, :s].contiguous(), v[:, :, :s].contiguous()),
                                        prefix=name + "/"))
    np.savez_compressed(os.path.join(HERE, "edge.npz"), **arrays)


def config0():
    """BASELINE config 0: B=1, 32 q / 8 kv heads, S=4096, init 128 / recent 128 / heavy 1/32;
    fp32 arithmetic on bf16-representable inputs and weights."""
    Hq, Hkv, S, init, recent, heavy = 32, 8, 4096, 128, 128, 1.0 / 32
    inp = synthetic.make_decode_inputs(0, [S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy)
    arrays = outputs_to_arrays(run_reference(att, usa, q, k, v))
    arrays.update(meta=np.array([Hq, Hkv, S, init, recent], dtype=np.int64), heavy=np.float64(heavy),
                  input_sha256=np.array(digest(q, k, v)), weight_sha256=np.array(
                      digest(*[p.float() for p in synthetic.make_usa(Hq, 128, 0, True).state_dict().values()])))
    np.savez_compressed(os.path.join(HERE, "config0.npz"), **arrays)


DEPTH_SUBCASES = [
    # name, heavy, usa_retrieve_depth   (usa_eval_mode = "depth": the non-'simple' branch, :439-443)
    ("d0", 1.0 / 8, 0),        # only the tokens tied at the best score
    ("d2", 1.0 / 8, 2),
    ("d6", 1.0 / 8, 6),        # the rank threshold wins: every token tied with the hb-th best is kept
    ("neg", 1.0 / 8, -1),      # threshold above the best score: no heavy token
    ("big_hb", 1.0, 3),        # hb beyond the candidates: the depth rule alone decides
    ("abs5", 5.0, 4),          # absolute budget of 5 tokens
]


def depth():
    """The inputs of case_a under the depth rule; codes and spans are those of case_a.npz."""
    Hq, Hkv, S, init, recent = 8, 2, 520, 16, 16
    inp = synthetic.make_decode_inputs(90, [S, S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    arrays = dict(meta=np.array([Hq, Hkv, S, init, recent], dtype=np.int64),
                  names=np.array([c[0] for c in DEPTH_SUBCASES]),
                  heavy=np.array([c[1] for c in DEPTH_SUBCASES], dtype=np.float64),
                  depth=np.array([c[2] for c in DEPTH_SUBCASES], dtype=np.int64))
    for name, heavy, d in DEPTH_SUBCASES:
        _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy, eval_mode="depth", depth=d)
        r = run_reference(att, usa, q, k, v)
        arrays[name + "/mask"] = np.packbits(r["mask"].numpy(), axis=-1)
        arrays[name + "/out"] = r["out"].numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "depth.npz"), **arrays)


ROWS_SUBCASES = [
    # name, S (after the chunk), q_len, init, recent, heavy, eval_mode, depth
    ("q5", 520, 5, 16, 16, 1.0 / 8, "simple", -1),
    ("q16_page", 260, 16, 8, 16, 1.0 / 8, "simple", -1),    # the chunk crosses the page boundary at 256
    ("q3_short", 40, 3, 16, 16, 1.0 / 8, "simple", -1),     # rows without any candidate, budget surplus
    ("q4_depth", 520, 4, 16, 16, 1.0 / 8, "depth", 3),
]


def rows():
    """Multi-token decode (2 <= q_len <= 128): queries of the last q_len tokens of case_a-like inputs."""
    Hq, Hkv = 8, 2
    arrays = dict(names=np.array([c[0] for c in ROWS_SUBCASES]),
                  params=np.array([[c[1], c[2], c[3], c[4], c[7]] for c in ROWS_SUBCASES], dtype=np.int64),
                  heavy=np.array([c[5] for c in ROWS_SUBCASES], dtype=np.float64),
                  modes=np.array([c[6] for c in ROWS_SUBCASES]), meta=np.array([Hq, Hkv], dtype=np.int64))
    inp = synthetic.make_decode_inputs(92, [520, 520], Hq, Hkv, bf16=True)
    k_all, v_all = torch.stack(inp.k), torch.stack(inp.v)   # every subcase uses the first S tokens of these
    arrays.update(k=bf16_bits(k_all), v=bf16_bits(v_all))
    for name, S, ql, init, recent, heavy, mode, d in ROWS_SUBCASES:
        k, v = k_all[:, :, :S].contiguous(), v_all[:, :, :S].contiguous()
        gen = torch.Generator().manual_seed(920 + ql)
        q = torch.randn(2, Hq, ql, 128, generator=gen).to(torch.bfloat16).to(torch.float32)
        _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy, eval_mode=mode, depth=d)
        r = run_reference_rows(att, usa, q, k, v)
        span = r["span"]
        assert float((span - span.round()).abs().max()) == 0.0
        arrays.update({name + "/q": bf16_bits(q), name + "/span": span.to(torch.int8).numpy(),
                       name + "/mask": np.packbits(r["mask"].numpy(), axis=-1),
                       name + "/out": r["out"].numpy().astype(np.float32)})
    np.savez_compressed(os.path.join(HERE, "rows.npz"), **arrays)


def layers():
    """The 2-layer and 1-layer hash functions (lth_num_layers 2 and 1, :112-127) on the inputs of edge.npz
    (S = 300, 4 query heads, 1 kv head; the inputs are stored there)."""
    Hq, Hkv, S, init, recent, heavy = 4, 1, 300, 16, 16, 1.0 / 8
    inp = synthetic.make_decode_inputs(91, [S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    arrays = dict(meta=np.array([Hq, Hkv, S, init, recent], dtype=np.int64), heavy=np.float64(heavy),
                  input_sha256=np.array(digest(q, k, v)))
    for n in (1, 2):
        _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy, layers=n)
        arrays.update(outputs_to_arrays(run_reference(att, usa, q, k, v), prefix=f"l{n}/"))
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **arrays)


def lsh():
    """The LSH baseline (lth_num_layers 0, :75-84 and :130-139): two sequences of 300 tokens, 4 query heads, 1 kv head.
    The norm bound of IpToCS is taken over both sequences; sequence 1's keys are scaled by 1.5 so that it is theirs."""
    Hq, Hkv, S, init, recent, heavy = 4, 1, 300, 16, 16, 1.0 / 8
    inp = synthetic.make_decode_inputs(191, [S, S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    k[1] = (k[1] * 1.5).bfloat16().float()
    _, usa, att = reference_modules(Hq, Hkv, init, recent, heavy, layers=0)
    arrays = dict(meta=np.array([Hq, Hkv, S, init, recent], dtype=np.int64), heavy=np.float64(heavy),
                  q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v))
    arrays.update(outputs_to_arrays(run_reference(att, usa, q, k, v), prefix=""))
    np.savez_compressed(os.path.join(HERE, "lsh.npz"), **arrays)


if __name__ == "__main__":
    which = sys.argv[1:] or ["case_a", "edge", "config0", "depth", "rows", "layers", "lsh"]
    for name in which:
        {"case_a": case_a, "edge": edge, "config0": config0, "depth": depth, "rows": rows, "layers": layers,
         "lsh": lsh}[name]()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
