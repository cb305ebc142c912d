"""Shared helpers of the test-suite: golden fixture loading and oracle-side conveniences."""
from __future__ import annotations

import os

import numpy as np
import torch

from oracle import hashattn_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the bf16 attention kernel against the fp32 reference
ATT_MAX_ABS = 2e-2
ATT_REL_L2 = 1e-2


def from_bf16_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16).to(torch.float32)


def codes64(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int64))


class GoldenCase:
    """One reference run: inputs (if stored), budgets and the reference's outputs."""

    def __init__(self, z, prefix: str, q, k, v, init: int, recent: int, heavy: float):
        self.q, self.k, self.v = q, k, v  # [B,Hq,D], [B,Hkv,S,D] fp32 (bf16-representable) or None
        self.init, self.recent, self.heavy = int(init), int(recent), float(heavy)
        self.k_codes = codes64(z[prefix + "k_codes"])  # [B,Hq,S]
        self.k_must = codes64(z[prefix + "k_must"])
        self.q_codes = codes64(z[prefix + "q_codes"])  # [B,Hq]
        self.q_must = codes64(z[prefix + "q_must"])
        self.span = torch.from_numpy(z[prefix + "span"].astype(np.int64))  # [B,Hq,S]
        S = self.span.shape[-1]
        self.S = S
        self.mask = torch.from_numpy(np.unpackbits(z[prefix + "mask"], axis=-1)[..., :S].astype(bool))
        self.out = torch.from_numpy(z[prefix + "out"])  # [B,Hq,D] fp32
        self.n_zero = int(z[prefix + "n_zero_preact"])

    @property
    def scores(self) -> torch.Tensor:
        return (self.span + 32) // 2


def load_case_a() -> GoldenCase:
    z = np.load(os.path.join(GOLDEN, "case_a.npz"))
    Hq, Hkv, S, init, recent = (int(x) for x in z["meta"])
    return GoldenCase(z, "", from_bf16_bits(z["q"]), from_bf16_bits(z["k"]), from_bf16_bits(z["v"]), init, recent,
                      float(z["heavy"]))


def load_lsh() -> GoldenCase:
    """The LSH baseline (lth_num_layers = 0) recorded from the reference: two sequences that share one norm bound."""
    z = np.load(os.path.join(GOLDEN, "lsh.npz"))
    Hq, Hkv, S, init, recent = (int(x) for x in z["meta"])
    return GoldenCase(z, "", from_bf16_bits(z["q"]), from_bf16_bits(z["k"]), from_bf16_bits(z["v"]), init, recent,
                      float(z["heavy"]))


class DepthCase:
    """case_a's inputs under the depth rule (usa_eval_mode != 'simple'): budget, depth, the
    reference's keep-mask and attention output."""

    def __init__(self, base: GoldenCase, heavy: float, depth: int, mask, out):
        self.base, self.heavy, self.depth, self.mask, self.out = base, float(heavy), int(depth), mask, out


def load_depth() -> dict[str, DepthCase]:
    base = load_case_a()
    z = np.load(os.path.join(GOLDEN, "depth.npz"))
    assert [int(x) for x in z["meta"]][2:] == [base.S, base.init, base.recent]
    out = {}
    for name, heavy, depth in zip(z["names"], z["heavy"], z["depth"]):
        mask = torch.from_numpy(np.unpackbits(z[f"{name}/mask"], axis=-1)[..., :base.S].astype(bool))
        out[str(name)] = DepthCase(base, heavy, depth, mask, torch.from_numpy(z[f"{name}/out"]))
    return out


class RowsCase:
    """Multi-token decode recorded from the reference: q [B,Hq,ql,D], k/v [B,Hkv,S,D] (the chunk's
    tokens last), span / mask [B,Hq,ql,S], out [B,Hq,ql,D]."""

    def __init__(self, z, name, S, ql, init, recent, depth, heavy, mode):
        self.S, self.ql, self.init, self.recent, self.depth = int(S), int(ql), int(init), int(recent), int(depth)
        self.heavy, self.mode = float(heavy), str(mode)
        self.q = from_bf16_bits(z[f"{name}/q"])
        self.k = from_bf16_bits(z["k"])[:, :, :self.S].contiguous()
        self.v = from_bf16_bits(z["v"])[:, :, :self.S].contiguous()
        self.span = torch.from_numpy(z[f"{name}/span"].astype(np.int64))
        self.mask = torch.from_numpy(np.unpackbits(z[f"{name}/mask"], axis=-1)[..., :self.S].astype(bool))
        self.out = torch.from_numpy(z[f"{name}/out"])

    @property
    def causal(self) -> torch.Tensor:
        return torch.tril(torch.ones(self.ql, self.S), diagonal=self.S - self.ql).bool()


def load_rows() -> dict[str, RowsCase]:
    z = np.load(os.path.join(GOLDEN, "rows.npz"))
    return {str(n): RowsCase(z, str(n), *p, h, m) for n, p, h, m in zip(z["names"], z["params"], z["heavy"], z["modes"])}


def load_edge() -> dict[str, GoldenCase]:
    z = np.load(os.path.join(GOLDEN, "edge.npz"))
    q, k, v = from_bf16_bits(z["q"]), from_bf16_bits(z["k"]), from_bf16_bits(z["v"])
    out = {}
    for name, (s, init, recent), heavy in zip(z["names"], z["params"], z["heavy"]):
        s = int(s)
        out[str(name)] = GoldenCase(z, f"{name}/", q, k[:, :, :s].contiguous(), v[:, :, :s].contiguous(), init,
                                    recent, heavy)
    return out


def load_layers() -> dict[int, GoldenCase]:
    """The 1- and 2-layer hash functions on the inputs stored in edge.npz."""
    z = np.load(os.path.join(GOLDEN, "layers.npz"))
    e = np.load(os.path.join(GOLDEN, "edge.npz"))
    Hq, Hkv, S, init, recent = (int(x) for x in z["meta"])
    q, k, v = from_bf16_bits(e["q"]), from_bf16_bits(e["k"]), from_bf16_bits(e["v"])
    assert k.shape[2] == S and q.shape[1] == Hq
    return {n: GoldenCase(z, f"l{n}/", q, k, v, init, recent, float(z["heavy"])) for n in (1, 2)}


def load_config0(synthetic):
    """Returns (case, inputs_match): inputs are regenerated from the seed and compared with the
    recorded SHA-256; inputs_match is False if this machine's generator gives other bits."""
    import hashlib

    z = np.load(os.path.join(GOLDEN, "config0.npz"))
    Hq, Hkv, S, init, recent = (int(x) for x in z["meta"])
    inp = synthetic.make_decode_inputs(0, [S], Hq, Hkv, bf16=True)
    q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
    h = hashlib.sha256()
    for t in (q, k, v):
        h.update(t.contiguous().numpy().tobytes())
    return GoldenCase(z, "", q, k, v, init, recent, float(z["heavy"])), h.hexdigest() == str(z["input_sha256"])


def oracle_preacts(usa, q, k):
    """Oracle pre-activations of query [B,Hq,32] and keys [B,Hq,S,32] for q [B,Hq,D], k [B,Hkv,S,D]."""
    group = q.shape[1] // k.shape[1]
    k_pre = orc.mlp_preact(orc.nets_from_usa(usa, "k"), k.repeat_interleave(group, dim=1))
    q_pre = orc.mlp_preact(orc.nets_from_usa(usa, "q"), q[:, :, None, :])[:, :, 0]
    return q_pre, k_pre


def codes_match(got: torch.Tensor, want: torch.Tensor, must: torch.Tensor) -> bool:
    return bool((((got ^ want) & must) == 0).all())


def att_close(got: torch.Tensor, want: torch.Tensor):
    """(ok, max_abs, rel_l2) under the tolerances of the bf16 kernel vs the fp32 reference."""
    got, want = got.float(), want.float()
    max_abs = float((got - want).abs().max())
    rel = float((got - want).norm() / want.norm().clamp_min(1e-30))
    return max_abs <= ATT_MAX_ABS and rel <= ATT_REL_L2, max_abs, rel
