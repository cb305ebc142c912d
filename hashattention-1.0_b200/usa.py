"""Host-side mirror of the reference's hash encoder module ``USA``.

The module owns the per-query-head hash MLP parameters under the reference's attribute names,
so a state dict saved by the reference (keys
``learning_to_hash_transformation_{k,q}.{head}.{0,2,4}.{weight,bias}``;
hashattention/hashattention_llama.py:99-111) loads unchanged, and a module built here under
``torch.manual_seed(s)`` holds the same values as the reference's built under the same seed
(same sub-module construction order: all key nets, then all query nets).

All arithmetic runs in the CUDA library; this class only stores parameters and repacks them
into the flat buffers the kernels read (:meth:`packed`).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from . import _lib

HIDDEN = 128
CODE_BITS = 32
MLP_ELEMS = 128 * 128 + 128 * 128 + 32 * 128
MLP_BIAS = 128 + 128 + 32

DEFAULT_USA_CFG = {"lth_int_dim": 128, "lth_final_dim": 32, "lth_thold": 0, "lth_num_layers": 3}


@dataclass
class PackedHashWeights:
    """Flat device buffers in the layout include/hashattn.h documents."""

    wq: torch.Tensor  # [Hq, 36864] bf16 or f32
    bq: torch.Tensor  # [Hq, 288] f32
    wk: torch.Tensor
    bk: torch.Tensor
    dtype_code: int
    num_layers: int = 3   # Linear layers of the hash function; unused slots of the layout hold zeros; 0: the LSH baseline

    @property
    def lsh(self) -> bool:
        return self.num_layers == 0

    def c_struct(self, lsh_state: torch.Tensor | None = None) -> _lib.HaHashWeights:
        """``lsh_state``: the cache's LSH state (see include/hashattn.h), required in LSH mode."""
        if self.lsh and lsh_state is None:
            raise ValueError("the LSH baseline needs the cache's state buffer")
        return _lib.HaHashWeights(self.wq.data_ptr(), self.bq.data_ptr(), self.wk.data_ptr(),
                                  self.bk.data_ptr(), self.dtype_code,
                                  _lib.HA_HASH_LSH if self.lsh else self.num_layers,
                                  lsh_state.data_ptr() if lsh_state is not None else None)

    def slice_heads(self, h0: int, h1: int) -> "PackedHashWeights":
        """The weights of query heads [h0, h1): what one GPU of a kv-head partition holds."""
        return PackedHashWeights(self.wq[h0:h1].contiguous(), self.bq[h0:h1].contiguous(),
                                 self.wk[h0:h1].contiguous(), self.bk[h0:h1].contiguous(), self.dtype_code,
                                 self.num_layers)


def _mlp(head_dim: int, int_dim: int, final_dim: int, num_layers: int = 3) -> nn.Sequential:
    """The hash function of one head with the reference's module structure for 3, 2 or 1 layers
    (hashattention/hashattention_llama.py:99-127)."""
    if num_layers == 3:
        return nn.Sequential(nn.Linear(head_dim, int_dim), nn.SiLU(), nn.Linear(int_dim, int_dim), nn.SiLU(),
                             nn.Linear(int_dim, final_dim))
    if num_layers == 2:
        return nn.Sequential(nn.Linear(head_dim, int_dim), nn.SiLU(), nn.Linear(int_dim, final_dim))
    return nn.Sequential(nn.Linear(head_dim, final_dim))


class IpToCS(nn.Module):
    """Placeholder with the reference's name and position (hashattention/hashattention_llama.py:75-84) so that the
    Linear(129, 32) behind it keeps its state-dict key ``...{head}.1.{weight,bias}``; the lifting itself
    (x -> [x, sqrt(relu(M^2 - |x|^2))]) runs in the CUDA kernels."""

    def forward(self, x):
        raise RuntimeError("evaluated by the CUDA library")


class USA(nn.Module):
    """Parameter container with the reference's constructor signature
    (hashattention/hashattention_llama.py:87-139).

    Only the configurations the kernels implement are accepted: 3, 2 or 1 layers or the LSH baseline
    (``lth_num_layers=0``, :130-139: one shared Linear(129, 32) per head with normal weights), hidden width 128,
    32 output bits, head_dim 128. Other ``lth_*`` settings raise ``NotImplementedError``.
    """

    def __init__(self, num_heads: int, head_dim: int, usa_params: dict = DEFAULT_USA_CFG):
        super().__init__()
        self.head_dim = head_dim
        self.num_heads = num_heads
        self.int_dim = usa_params["lth_int_dim"]
        self.lth_final_dim = usa_params["lth_final_dim"]
        self.lth_thold = usa_params["lth_thold"]
        self.num_layers = usa_params.get("lth_num_layers", 3)
        if self.num_layers not in (0, 1, 2, 3) or (self.int_dim, self.lth_final_dim, head_dim) != (HIDDEN, CODE_BITS, 128):
            raise NotImplementedError(
                "the sm_100a kernels implement lth_num_layers=0..3, lth_init_dim=128, lth_final_dim=32, "
                f"head_dim=128; got layers={self.num_layers}, int_dim={self.int_dim}, "
                f"final_dim={self.lth_final_dim}, head_dim={head_dim}"
            )
        if self.num_layers == 0:
            # the reference's structure and initialisation order (:130-139): one list under three names
            self.learning_to_hash_transformation = nn.ModuleList(
                [nn.Sequential(IpToCS(), nn.Linear(head_dim + 1, self.lth_final_dim)) for _ in range(num_heads)])
            self.learning_to_hash_transformation_k = self.learning_to_hash_transformation
            self.learning_to_hash_transformation_q = self.learning_to_hash_transformation
            for i in range(num_heads):
                nn.init.normal_(self.learning_to_hash_transformation[i][1].weight)
        else:
            self.learning_to_hash_transformation_k = nn.ModuleList(
                [_mlp(head_dim, self.int_dim, self.lth_final_dim, self.num_layers) for _ in range(num_heads)])
            self.learning_to_hash_transformation_q = nn.ModuleList(
                [_mlp(head_dim, self.int_dim, self.lth_final_dim, self.num_layers) for _ in range(num_heads)])
        self._packed: PackedHashWeights | None = None
        # a state dict loaded through this module or any parent invalidates the packed copy
        self.register_load_state_dict_post_hook(lambda module, _incompatible: setattr(module, "_packed", None))

    # -- packing ---------------------------------------------------------------------------
    def _pack_side(self, nets: nn.ModuleList, dtype: torch.dtype, device) -> tuple[torch.Tensor, torch.Tensor]:
        # the kernels' layout always has the three slots [W0 | W1 | W2]: a 2-layer function fills W0 and W2,
        # a 1-layer function W2 only; the rest stays zero
        def slots(net):
            lin = [m for m in net if isinstance(m, nn.Linear)]
            z = lambda *shape: torch.zeros(*shape, dtype=lin[0].weight.dtype, device=lin[0].weight.device)  # noqa: E731
            if self.num_layers == 0:
                # Linear(129, 32): columns 0..127 in the W2 slot, column 128 in b0[0..31], the bias in b2
                w129, b = lin[0].weight, lin[0].bias
                b0 = z(HIDDEN)
                b0[:CODE_BITS] = w129[:, self.head_dim]
                return (torch.cat([z(HIDDEN, self.head_dim).reshape(-1), z(HIDDEN, HIDDEN).reshape(-1),
                                   w129[:, :self.head_dim].reshape(-1)]), torch.cat([b0, z(HIDDEN), b]))
            first = lin[0] if len(lin) >= 2 else None
            second = lin[1] if len(lin) == 3 else None
            last = lin[-1]
            ws = [first.weight if first is not None else z(HIDDEN, self.head_dim),
                  second.weight if second is not None else z(HIDDEN, HIDDEN), last.weight]
            bs = [first.bias if first is not None else z(HIDDEN), second.bias if second is not None else z(HIDDEN),
                  last.bias]
            return torch.cat([w.reshape(-1) for w in ws]), torch.cat(bs)

        packed = [slots(net) for net in nets]
        w = torch.stack([p[0] for p in packed])
        b = torch.stack([p[1] for p in packed])
        return (w.detach().to(device=device, dtype=dtype).contiguous(),
                b.detach().to(device=device, dtype=torch.float32).contiguous())

    def packed(self, device=None, refresh: bool = False) -> PackedHashWeights:
        """Kernel-side copy of the parameters. bf16 parameters stay bf16 (the kernels up-cast
        them exactly); anything else is kept as fp32."""
        first_linear = next(m for m in self.learning_to_hash_transformation_k[0] if isinstance(m, nn.Linear))
        device = torch.device(device) if device is not None else first_linear.weight.device
        if self._packed is not None and not refresh and self._packed.wq.device == device:
            return self._packed
        pdtype = first_linear.weight.dtype
        if pdtype == torch.bfloat16:
            wdtype, code = torch.bfloat16, _lib.HA_WEIGHTS_BF16
        else:
            wdtype, code = torch.float32, _lib.HA_WEIGHTS_F32
        wq, bq = self._pack_side(self.learning_to_hash_transformation_q, wdtype, device)
        wk, bk = self._pack_side(self.learning_to_hash_transformation_k, wdtype, device)
        self._packed = PackedHashWeights(wq, bq, wk, bk, code, self.num_layers)
        return self._packed

    def _apply(self, fn, *args, **kwargs):  # .cuda() / .bfloat16() / .to() invalidate the packed copy
        self._packed = None
        return super()._apply(fn, *args, **kwargs)

    def forward(self, K, Q, hard=False):
        raise RuntimeError(
            "USA.forward is not evaluated in torch here: the hash codes are produced by the CUDA "
            "kernels (ops.hash_decode / ops.hash_prefill) and scored by ops.score_select"
        )
