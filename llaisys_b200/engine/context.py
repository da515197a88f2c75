"""The device-side description of one step that every part reads."""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from ..cache.kv import KVView, PagedCache


class StepContext:
    """One step over a batch of sequences, packed without padding: sequence after sequence.

    Device tensors (int32): tokens [T]; tok_seq [T] (index of the token's sequence in the
    batch); tok_pos [T] (absolute position); seq_start [B + 1] (first packed token of each
    sequence); seq_len_before [B] (tokens cached before this step); seq_slot [B]; out_rows
    (packed indices whose logits are wanted); err [1] (set by kernels that meet an invalid
    token id or position).  Host facts: n_tokens, n_seqs, max_new, max_position, is_decode
    (every sequence brings exactly one token), slots, n_new, lens_before.
    """

    def __init__(self, cache: PagedCache, slots: List[int], n_new: List[int], tokens: List[int],
                 out_rows: List[int], device, sm_count: int = 148):
        self.cache = cache
        self.slots, self.n_new = list(slots), list(n_new)
        self.lens_before = [cache.length(s) for s in slots]
        B, T = len(slots), int(sum(n_new))
        self.n_seqs, self.n_tokens = B, T
        self.max_new = max(n_new)
        self.is_decode = all(n == 1 for n in n_new)
        self.max_position = max(l + n for l, n in zip(self.lens_before, n_new)) - 1
        self.sm_count = sm_count
        starts = np.zeros(B + 1, dtype=np.int32)
        starts[1:] = np.cumsum(n_new)
        tok_seq = np.repeat(np.arange(B, dtype=np.int32), n_new)
        tok_pos = (np.arange(T, dtype=np.int32) - starts[tok_seq] + np.asarray(self.lens_before, dtype=np.int32)[tok_seq])
        groups = range(len(cache.group_keys))
        tables = [cache.page_table(g, slots) for g in groups]
        parts = [np.asarray(tokens, dtype=np.int32), tok_seq, tok_pos.astype(np.int32), starts,
                 np.asarray(self.lens_before, dtype=np.int32), np.asarray(slots, dtype=np.int32),
                 np.asarray(out_rows, dtype=np.int32), np.zeros(1, dtype=np.int32)] + [t.reshape(-1) for t in tables]
        sizes = [p.size for p in parts]
        host = torch.from_numpy(np.concatenate(parts)).pin_memory() if torch.device(device).type == "cuda" \
            else torch.from_numpy(np.concatenate(parts))
        dev = host.to(device, non_blocking=True)
        self._host_meta = host          # kept until the copy has run
        offs = np.concatenate([[0], np.cumsum(sizes)])
        cut = [dev[offs[i]:offs[i + 1]] for i in range(len(parts))]
        (self.tokens, self.tok_seq, self.tok_pos, self.seq_start, self.seq_len_before,
         self.seq_slot, self.out_rows, self.err) = cut[:8]
        self._tables: Dict[int, torch.Tensor] = {g: cut[8 + g].view(B, tables[g].shape[1]) for g in groups}

    def kv(self, call: int) -> KVView:
        return self.cache.view(call, self._tables)

    def state(self, call: int) -> torch.Tensor:
        """float32 [n_slots, state_size] of this call; row seq_slot[b] belongs to sequence b."""
        return self.cache.state[call]

    def decode_splits(self, n_kv_heads: int) -> int:
        """Slices of the key range in decode attention: enough blocks to fill the device, at
        most one slice per page of the longest sequence."""
        pages = self.max_position // 64 + 1
        want = -(-2 * self.sm_count // max(1, self.n_seqs * n_kv_heads))
        return max(1, min(want, pages, 64))
