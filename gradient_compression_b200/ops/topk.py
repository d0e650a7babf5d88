"""Batched exact Top-K selection by magnitude over many segments of one flat buffer (``csrc/gc_topk.cu``).

``TopKSelector(segments, device)`` holds the segment table and scratch state; ``select(g, e)`` returns the
(global int32 index, value) lists of all segments back to back (segment i's entries start at
``offsets[i]``), after folding the error memory ``e`` into the selection and updating it in place:
``e <- g + e`` with the selected entries zeroed (reference: reducer.py:1161-1189).
On CPU the same contract is met with ``torch.topk`` per segment.
"""
from __future__ import annotations

import torch

from . import _native as nat


class TopKSelector:
    def __init__(self, segments, device):
        """segments: list of (start, length, k) in elements of the flat buffer."""
        self.device = torch.device(device)
        self.segments = [(int(s), int(l), int(min(k, l))) for s, l, k in segments]
        self.offsets, off = [], 0
        for _, _, k in self.segments:
            self.offsets.append(off)
            off += k
        self.total = off
        if self.device.type == "cuda":
            chunk = nat.cuda().gc_cuda_topk_chunk()
            rows, chunks = [], 0
            for (s, l, k), o in zip(self.segments, self.offsets):
                rows.append([s, l, k, o, chunks, 0])
                chunks += (l + chunk - 1) // chunk
            self.total_chunks = chunks
            self.table = torch.tensor(rows, dtype=torch.int64, device=self.device)
            self.state = torch.zeros(nat.cuda().gc_cuda_topk_state_bytes(len(rows)), dtype=torch.uint8, device=self.device)

    def select(self, g, e=None, out_idx=None, out_val=None):
        g = g.contiguous().view(-1)
        if out_idx is None:
            out_idx = torch.empty(self.total, dtype=torch.int32, device=g.device)
        if out_val is None:
            out_val = torch.empty(self.total, dtype=torch.float32, device=g.device)
        if g.is_cuda:
            with torch.cuda.device(g.device):
                nat.check(nat.cuda().gc_cuda_topk_select(g.data_ptr(), nat.ptr(e), self.table.data_ptr(), len(self.segments),
                                                         self.total_chunks, self.state.data_ptr(), out_idx.data_ptr(),
                                                         out_val.data_ptr(), nat.stream_ptr()), "topk_select")
                nat.count_launch(6)
            return out_idx, out_val
        a = g if e is None else e.add_(g)
        for (s, l, k), o in zip(self.segments, self.offsets):
            seg = a[s:s + l]
            pos = torch.topk(seg.abs(), k, sorted=False)[1]
            out_idx[o:o + k] = (pos + s).to(torch.int32)
            out_val[o:o + k] = seg[pos]
        if e is not None:
            e[out_idx.long()] = 0.0
        return out_idx, out_val
