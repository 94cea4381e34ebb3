"""Trace replay: feeds given token ids through a model step by step and writes the logits of the places asked for.
Nothing is sampled.  It drives the same engine, page table and carried state that ``Stage.generate`` drives, through
``forward_ragged`` (the scheduler step over requests of unequal length), so a trace exercises exactly the serving path.

Protocol (one JSON object per input line):
  {"step": n, "entries": [{"id": str, "tokens": [int...], "want": [index into tokens...]}...], "end": [id...]}
For a step in which something is wanted, ``<out>/<n>.f32`` receives the logits [wanted, vocab] as little-endian
fp32 in the order of the entries and of ``want``; after every step ``done <n>`` is printed and flushed."""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, List, Optional

import torch

from .._lib import AsdError
from ..models import registry

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
EXIT_UNSUPPORTED_DTYPE = 3


class TraceSession:
    """Requests by name -> (slot, length); slots and pages come from the engine's page table and go back at 'end'."""

    def __init__(self, engine, dynamic: bool):
        self.engine, self.dynamic = engine, dynamic
        self.live: Dict[str, List[int]] = {}            # id -> [slot, length]
        self._free = list(range(engine.max_seqs - 1, -1, -1)) if not dynamic else None

    def _open(self) -> int:
        if self.dynamic:
            return self.engine.open_sequence()
        if not self._free:
            raise AsdError("no free sequence slot")
        return self._free.pop()

    def _close(self, slot: int) -> None:
        if self.dynamic:
            self.engine.close_sequence(slot)
        else:
            self._free.append(slot)

    def step(self, entries: List[dict], end: List[str]) -> Optional[torch.Tensor]:
        items = []
        for e in entries:
            st = self.live.get(e["id"])
            if st is None:
                st = self.live[e["id"]] = [self._open(), 0]
            toks = [int(t) for t in e["tokens"]]
            if self.dynamic:
                self.engine.reserve(st[0], st[1] + len(toks))
            elif st[1] + len(toks) > self.engine.max_seq_len:
                raise AsdError(f"request {e['id']} outgrows max_seq_len {self.engine.max_seq_len}")
            items.append((st[0], st[1], toks, [int(i) for i in e.get("want", [])]))
            st[1] += len(toks)
        logits = self.engine.forward_ragged([it for it in items if it[2]]) if any(it[2] for it in items) else None
        for name in end:
            st = self.live.pop(name, None)
            if st is not None:
                self._close(st[0])
        return logits


def build_engine(model_dir: str, dtype: str, max_tokens: int, device="cuda"):
    """engine for a checkpoint directory, sized for ``max_tokens`` live tokens"""
    from ..models.qwen2 import load_safetensors_dir
    fam, cfg = registry.read_config(model_dir)
    if dtype not in fam.dtypes:
        return fam, None
    Engine = fam.engine()
    max_tokens = max(int(max_tokens), 1)
    if fam.name in ("mezilix", "rivetar", "mavipel", "lukopel"):
        page = 16
        pages = (max_tokens + page - 1) // page + 8          # every live request may leave a last page part empty
        eng = Engine(cfg, max_seqs=8, max_seq_len=max_tokens, max_tokens=min(1024, max_tokens), page_size=page,
                     device=device, dtype=DTYPES[dtype], num_pages=pages, dynamic_pages=True)
    else:
        eng = Engine(cfg, max_seqs=1, max_seq_len=max_tokens, max_tokens=256, device=device)
    eng.load_weights(load_safetensors_dir(model_dir))
    return fam, eng


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stdin=None, stdout=None) -> int:
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    fam, eng = build_engine(model_dir, dtype, max_tokens)
    if eng is None:
        sys.stderr.write(f"the {fam.name} engine does not run in {dtype}\n")
        return EXIT_UNSUPPORTED_DTYPE
    sess = TraceSession(eng, dynamic=getattr(eng.pages, "dynamic", False))
    os.makedirs(out_dir, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        logits = sess.step(req.get("entries", []), req.get("end", []))
        if logits is not None:
            data = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(out_dir, f".{req['step']}.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(out_dir, f"{req['step']}.f32"))
        else:
            torch.cuda.synchronize()
        stdout.write(f"done {req['step']}\n")
        stdout.flush()
    return 0
