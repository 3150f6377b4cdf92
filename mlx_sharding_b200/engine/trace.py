"""Trace replay: feed given token ids through a model step by step and collect logits (no sampling).

A *trace* is a sequence of steps; each step brings, for some requests, their next tokens (a prompt portion or a single token) and
says at which of them the logits are wanted.  All entries of a step run as ONE ragged batch through the stage executor the
generation engine uses (``parallel/pipeline.py::StageExecutor``: the model's step function, its paged pools and state slots, its
kernels); pages and state slots come from the engine's ``SequenceTable`` and go back when a request ends, so a pool sized for the
live requests only is re-used over the trace.  ``bin/trace_run`` is the command-line front end.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..ops.meta import BatchMeta
from .kv_cache import PageAllocator, SequenceTable, SlotAllocator


class TraceSession:
    def __init__(self, stage, max_live_tokens: int, max_live_requests: int = 4):
        """``stage``: a ``StageExecutor`` whose cache has at least ``pages_needed(...)`` pages and ``max_live_requests + 1`` slots."""
        self.stage = stage
        self.page_size = stage.kv.page_size
        slots = getattr(stage.kv, "num_slots", 0)
        self.table = SequenceTable(PageAllocator(stage.kv.num_pages), self.page_size, SlotAllocator(slots) if slots else None)
        self.ids: Dict[str, int] = {}
        self._next = 0

    @staticmethod
    def pages_needed(max_live_tokens: int, page_size: int) -> int:
        return (max_live_tokens + page_size - 1) // page_size + 1          # + the null page

    @torch.inference_mode()
    def step(self, entries: Sequence[dict]) -> torch.Tensor:
        """``entries``: ``[{"id": str, "tokens": [...], "want": [...]}]``.  Returns the fp32 logits ``[wanted, vocab]`` (host)."""
        entries = [e for e in entries if len(e["tokens"])]
        if not entries:
            return torch.empty(0, 0)
        t = self.table
        sids, q_lens, ctx0, toks, rows, base = [], [], [], [], [], 0
        for e in entries:
            if e["id"] not in self.ids:
                self.ids[e["id"]] = self._next
                t.add(self._next)
                self._next += 1
            sid = self.ids[e["id"]]
            t.reserve(sid, len(e["tokens"]))
            sids.append(sid)
            q_lens.append(len(e["tokens"]))
            ctx0.append(t.length[sid])
            toks.extend(int(x) for x in e["tokens"])
            rows.extend(base + int(wi) for wi in e.get("want", []))
            base += len(e["tokens"])
        dev = self.stage.device
        meta = BatchMeta.build(q_lens, ctx0, [t.pages[s] for s in sids], self.page_size, device=dev, state_slots=t.state_slots(sids))
        logits = self.stage.forward(torch.tensor(toks, dtype=torch.int64, device=dev), meta, all_logits=True)
        for s, n in zip(sids, q_lens):
            t.advance(s, n)
        if not rows:
            return torch.empty(0, logits.shape[1])
        return logits.index_select(0, torch.tensor(rows, dtype=torch.int64, device=dev)).float().cpu()

    def end(self, request_ids: Sequence[str]):
        for rid in request_ids:
            sid = self.ids.pop(rid, None)
            if sid is not None:
                self.table.release(sid)


def run_trace(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stream_in, stream_out, device=None, backend=None,
              page_size: int = 64, max_requests: int = 4):
    """Replay JSON steps from ``stream_in`` (one object per line: ``step``, ``entries``, ``end``); writes ``<step>.f32`` files of
    little-endian fp32 logits into ``out_dir`` and a ``done <step>`` line per step to ``stream_out``."""
    import json
    import os

    import numpy as np

    from ..parallel.pipeline import StageExecutor
    from ..utils.loader import load_model

    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = load_model(model_dir, dtype=tdt, device=device, backend=backend)
    if not hasattr(model, "cache_layout"):
        raise SystemExit("trace replay drives models with per-layer cache layouts")
    # each live request rounds up to whole pages: the pool holds ``max_tokens`` token rows (a multiple of the page size) + the null page
    stage = StageExecutor(model, TraceSession.pages_needed(max_tokens, page_size), page_size, num_state_slots=max_requests + 1)
    sess = TraceSession(stage, max_tokens, max_requests)
    os.makedirs(out_dir, exist_ok=True)
    for line in stream_in:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        logits = sess.step(st.get("entries", []))
        if logits.numel():
            np.ascontiguousarray(logits.numpy().astype("<f4")).tofile(os.path.join(out_dir, f"{int(st['step'])}.f32"))
        sess.end(st.get("end", []))
        stream_out.write(f"done {int(st['step'])}\n")
        stream_out.flush()
