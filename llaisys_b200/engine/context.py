"""The device-side description of one step that every part reads."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.kv import KVView, PagedCache


class StepContext:
    """One step over a batch of sequences, packed without padding: sequence after sequence.

    Device tensors (int32), all views of one buffer that a single copy fills:
      tokens [T]; tok_seq [T] (index of the token's sequence in the batch); tok_pos [T]
      (absolute position); seq_start [B + 1] (first packed token of each sequence);
      seq_len_before [B] (tokens cached before this step); seq_slot [B]; out_rows [n_out]
      (packed indices whose logits are wanted); one page table [B, width] per cache group.
    err [1] is the engine's error word: kernels that meet an invalid token id or position set it.

    Host facts: n_tokens, n_seqs, max_new, max_position, is_decode (every sequence brings
    exactly one token), slots, n_new, lens_before.

    A context is a shape (B, T, n_out, table widths) plus its current contents; `load` refills
    the same device buffer, which is what lets a captured CUDA graph be replayed on new steps.
    """

    def __init__(self, cache: PagedCache, device, n_seqs: int, n_tokens: int, n_out: int,
                 widths: Sequence[int], err: torch.Tensor, sm_count: int = 148):
        self.cache, self.device = cache, torch.device(device)
        self.n_seqs, self.n_tokens, self.n_out = n_seqs, n_tokens, n_out
        self.widths = tuple(widths)
        self.err, self.sm_count = err, sm_count
        B, T = n_seqs, n_tokens
        sizes = [T, T, T, B + 1, B, B, n_out] + [B * w for w in self.widths]
        self._offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        self.meta = torch.empty(int(self._offs[-1]), dtype=torch.int32, device=self.device)
        cut = [self.meta[self._offs[i]:self._offs[i + 1]] for i in range(len(sizes))]
        (self.tokens, self.tok_seq, self.tok_pos, self.seq_start, self.seq_len_before, self.seq_slot,
         self.out_rows) = cut[:7]
        self._tables: Dict[int, torch.Tensor] = {g: cut[7 + g].view(B, w) for g, w in enumerate(self.widths)}
        self.slots: List[int] = []
        self.n_new: List[int] = []
        self.lens_before: List[int] = []
        self.max_new, self.max_position, self.is_decode = 1, 0, True

    @staticmethod
    def shape_of(cache: PagedCache, slots, n_new, out_rows, bucket: bool) -> Tuple[int, int, int, Tuple[int, ...]]:
        """(B, T, n_out, widths) of a step; with `bucket` the table widths are rounded up to a
        power of two so that steps of a growing sequence keep the same shape for a while."""
        widths = []
        for g in range(len(cache.group_keys)):
            w = cache.table_width(g, slots)
            if bucket:
                w = 1 << (w - 1).bit_length()
            widths.append(w)
        return len(slots), int(sum(n_new)), len(out_rows), tuple(widths)

    def host_meta(self, slots, n_new, tokens, out_rows) -> np.ndarray:
        cache = self.cache
        B, T = len(slots), int(sum(n_new))
        assert (B, T, len(out_rows)) == (self.n_seqs, self.n_tokens, self.n_out)
        lens = np.asarray([cache.length(s) for s in slots], dtype=np.int32)
        starts = np.zeros(B + 1, dtype=np.int32)
        starts[1:] = np.cumsum(n_new)
        tok_seq = np.repeat(np.arange(B, dtype=np.int32), n_new)
        tok_pos = np.arange(T, dtype=np.int32) - starts[tok_seq] + lens[tok_seq]
        parts = [np.asarray(tokens, dtype=np.int32), tok_seq, tok_pos.astype(np.int32), starts, lens,
                 np.asarray(slots, dtype=np.int32), np.asarray(out_rows, dtype=np.int32)]
        parts += [cache.page_table(g, slots, w).reshape(-1) for g, w in enumerate(self.widths)]
        self.slots, self.n_new, self.lens_before = list(slots), list(n_new), lens.tolist()
        self.max_new = int(max(n_new))
        self.is_decode = all(n == 1 for n in n_new)
        self.max_position = int((lens + np.asarray(n_new, dtype=np.int32)).max()) - 1
        return np.concatenate(parts)

    def load(self, slots, n_new, tokens, out_rows, staging: Optional[torch.Tensor] = None) -> None:
        """Fills the device buffer for a step of this context's shape.  `staging` is a pinned
        host tensor at least as long as the buffer; without it a fresh pinned tensor is made."""
        meta = self.host_meta(slots, n_new, tokens, out_rows)
        n = meta.size
        if staging is None:
            staging = torch.empty(n, dtype=torch.int32).pin_memory() if self.device.type == "cuda" \
                else torch.empty(n, dtype=torch.int32)
        staging[:n].numpy()[:] = meta
        self.meta.copy_(staging[:n], non_blocking=True)
        self._staging = staging

    def kv(self, call: int) -> KVView:
        return self.cache.view(call, self._tables)

    def state(self, call: int) -> torch.Tensor:
        """float32 [n_slots, state_size] of this call; row seq_slot[b] belongs to sequence b."""
        return self.cache.state[call]
