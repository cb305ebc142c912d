"""Paged K / V / key-hash cache of one attention layer on one GPU.

Layout (include/hashattn.h): K and V pools ``[num_pages, Hkv, 256, 128]`` bf16, hash pool
``[num_pages, Hkv, 256, 4]`` int32 (bit pattern of the u32 codes), ``page_table[B, max_pages]``
and ``seq_lens[B]`` int32. The hash pool is the realisation of the reference's per-layer
``past_key_signatures`` state (hashattention/hashattention_llama.py:275, 409-414), which the
reference keeps disabled and recomputes on every step.
"""
from __future__ import annotations

import torch

PAGE = 256
HEAD_DIM = 128
GROUP = 4


class PagedHashKVCache:
    def __init__(self, batch: int, num_kv_heads: int, max_seq_len: int, device, num_pages: int | None = None,
                 shuffle_seed: int | None = None):
        """Reserves pages for ``batch`` sequences of up to ``max_seq_len`` tokens each.

        ``shuffle_seed`` assigns physical pages by a seeded permutation (pages of one sequence
        are then scattered through the pool); otherwise pages are assigned in order.
        """
        self.device = torch.device(device)
        self.batch = batch
        self.num_kv_heads = num_kv_heads
        self.max_pages = (max_seq_len + PAGE - 1) // PAGE
        need = batch * self.max_pages
        self.num_pages = need if num_pages is None else num_pages
        if self.num_pages < need:
            raise ValueError(f"num_pages={self.num_pages} cannot hold {batch} sequences of {self.max_pages} pages")
        if shuffle_seed is None:
            perm = torch.arange(self.num_pages)
        else:
            perm = torch.randperm(self.num_pages, generator=torch.Generator().manual_seed(shuffle_seed))
        self.page_table = perm[:need].reshape(batch, self.max_pages).to(torch.int32).to(self.device)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)
        shape = (self.num_pages, num_kv_heads, PAGE, HEAD_DIM)
        self.k_pages = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.v_pages = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.hash_pages = torch.zeros((self.num_pages, num_kv_heads, PAGE, GROUP), dtype=torch.int32,
                                      device=self.device)

    def reset(self) -> None:
        """Forgets every sequence (the counterpart of the reference's ``_reset_state``,
        hashattention/hashattention_llama.py:298-301). Page contents need no clearing."""
        self.seq_lens.zero_()

    def _slots(self, b: int, start: int, n: int):
        tok = torch.arange(start, start + n, device=self.device)
        pages = self.page_table[b, (tok // PAGE).long()].long()
        return pages, (tok % PAGE).long()

    def write_kv(self, b: int, k: torch.Tensor, v: torch.Tensor, start: int = 0) -> None:
        """Copies dense ``[Hkv, n, 128]`` keys / values of sequence ``b`` into its pages at token
        offset ``start`` and sets ``seq_lens[b] = start + n`` (prefill-side plumbing; the decode
        step appends through the kernel)."""
        n = k.shape[1]
        if start + n > self.max_pages * PAGE:
            raise ValueError("sequence does not fit its page table row")
        pages, slots = self._slots(b, start, n)
        self.k_pages[pages, :, slots, :] = k.to(self.device, torch.bfloat16).transpose(0, 1)
        self.v_pages[pages, :, slots, :] = v.to(self.device, torch.bfloat16).transpose(0, 1)
        self.seq_lens[b] = start + n

    def write_codes(self, b: int, codes: torch.Tensor, start: int = 0) -> None:
        """Stores externally computed key codes ``[Hq, n]`` (values 0..2^32-1 as int64)."""
        n = codes.shape[1]
        pages, slots = self._slots(b, start, n)
        c = codes.to(self.device).reshape(self.num_kv_heads, GROUP, n).permute(2, 0, 1)  # [n, Hkv, 4]
        c = torch.where(c >= 2 ** 31, c - 2 ** 32, c).to(torch.int32)
        self.hash_pages[pages, :, slots, :] = c

    def read_codes(self, b: int, n: int | None = None) -> torch.Tensor:
        """Key codes of sequence ``b`` as ``[Hq, n]`` int64 in 0..2^32-1."""
        n = int(self.seq_lens[b]) if n is None else n
        pages, slots = self._slots(b, 0, n)
        c = self.hash_pages[pages, :, slots, :].to(torch.int64) & 0xFFFFFFFF  # [n, Hkv, 4]
        return c.permute(1, 2, 0).reshape(self.num_kv_heads * GROUP, n)

    def read_kv(self, b: int, n: int | None = None):
        n = int(self.seq_lens[b]) if n is None else n
        pages, slots = self._slots(b, 0, n)
        return (self.k_pages[pages, :, slots, :].transpose(0, 1).contiguous(),
                self.v_pages[pages, :, slots, :].transpose(0, 1).contiguous())
