"""Replay of given token ids through the engine (the library side of ``bin/trace_run``).

It keeps only the map from a request's id to its cache slot; every token goes through
``Engine.step``.
"""
from __future__ import annotations

import numpy as np

from ..core import RuntimeFault
from .model import Model
from .step import Engine, StepEntry


class Replayer:
    def __init__(self, model_folder: str, dtype: str, max_tokens: int, device: str = "cuda:0", model=None):
        self.model = model if model is not None else Model.load(model_folder, dtype=dtype, device=device)
        self.engine = Engine(self.model, max_tokens)
        self.slots: dict[str, int] = {}

    def run_step(self, record: dict):
        """Runs one step record; returns the wanted logits as a float32 array [wanted, vocab], or
        None if nothing was wanted."""
        entries = []
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid not in self.slots:
                self.slots[rid] = self.engine.open_slot()
            entries.append(StepEntry(self.slots[rid], list(item["tokens"]), list(item.get("want", []))))
        logits = self.engine.step(entries) if entries else None
        for rid in record.get("end", []):
            rid = str(rid)
            if rid not in self.slots:
                raise RuntimeFault(f"step {record.get('step')}: request {rid!r} ends but was never seen")
            self.engine.close_slot(self.slots.pop(rid))
        self.engine.check_errors()
        if logits is None:
            return None
        return logits.float().cpu().numpy().astype(np.float32)
