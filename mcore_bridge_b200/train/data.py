"""Synthetic token streams for benchmarks and tests: packed sequences with random segment lengths.

Batches are produced on the host in pinned memory (when CUDA is present) — the trainer copies them to the
device every step, like a real input pipeline would.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional

import torch


def packed_segments(total: int, lo: int, hi: int, gen: torch.Generator, multiple: int = 1) -> List[int]:
    """Segment lengths uniform in ``[lo, hi]`` concatenated until ``total`` tokens are filled (the last one is cut)."""
    out, used = [], 0
    while used < total:
        n = int(torch.randint(lo, hi + 1, (1,), generator=gen).item())
        n = max(multiple, n // multiple * multiple)
        n = min(n, total - used)
        out.append(n)
        used += n
    return out


class SyntheticPackedDataset:
    """Yields micro-batches ``{input_ids, labels, position_ids, loss_mask, cu_seqlens, max_seqlen}``.

    One micro-batch is one packed row of ``seq_len`` tokens (``micro_batch_size`` rows are concatenated into
    a single token stream, boundaries land in ``cu_seqlens``).  Token ids are uniform in ``[0, vocab)``.
    """

    def __init__(self, vocab_size: int, seq_len: int, micro_batch_size: int = 1, seed: int = 1234,
                 packed: bool = True, seg_lo: int = 256, seg_hi: int = 4096, segment_multiple: int = 1,
                 pin: Optional[bool] = None):
        self.vocab_size, self.seq_len, self.mbs = vocab_size, seq_len, micro_batch_size
        self.packed, self.seg_hi = packed, min(seg_hi, seq_len)
        self.seg_lo = min(seg_lo, self.seg_hi)         # sequences shorter than the smallest segment: one segment
        self.segment_multiple = segment_multiple
        self.gen = torch.Generator().manual_seed(seed)
        self.pin = torch.cuda.is_available() if pin is None else pin

    def _pin(self, t: torch.Tensor) -> torch.Tensor:
        return t.pin_memory() if self.pin else t

    def next_microbatch(self) -> Dict[str, torch.Tensor]:
        T = self.seq_len * self.mbs
        ids = torch.randint(0, self.vocab_size, (1, T + 1), generator=self.gen, dtype=torch.int64)
        segs: List[int] = []
        for _ in range(self.mbs):
            if self.packed:
                segs += packed_segments(self.seq_len, self.seg_lo, self.seg_hi, self.gen, self.segment_multiple)
            else:
                segs.append(self.seq_len)
        cu = torch.zeros(len(segs) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(segs, dtype=torch.int32).cumsum(0)
        pos = torch.cat([torch.arange(n, dtype=torch.int64) for n in segs]).unsqueeze(0)
        labels = ids[:, 1:].clone()
        mask = torch.ones(1, T, dtype=torch.float32)
        last = (cu[1:] - 1).long()
        mask[0, last] = 0.0          # the last token of a segment has no target inside the segment
        return {
            'input_ids': self._pin(ids[:, :-1].contiguous()),
            'labels': self._pin(labels),
            'position_ids': self._pin(pos),
            'loss_mask': self._pin(mask),
            'cu_seqlens': self._pin(cu),
            'max_seqlen': int(max(segs)),
        }

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        while True:
            yield self.next_microbatch()
