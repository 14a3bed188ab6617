"""Trace replay on top of the step function.

A trace step names requests by id, gives each its next tokens and the places whose
logits are wanted, and lists the requests that end after the step.  `Replayer` keeps the
id -> slot map, acquires a slot when an id first appears, and releases it when the id
ends; everything else is `Engine.step`.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .step import Engine, StepEntry, StepError


class Replayer:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.slots: Dict[str, int] = {}

    def run_step(self, record: dict) -> Optional[torch.Tensor]:
        """Run one trace step; return the wanted logits [n, vocab] (float32) or None."""
        entries = record.get("entries", [])
        if not entries:
            raise StepError(f"step {record.get('step')}: no entries")
        ids = [str(e["id"]) for e in entries]
        if len(set(ids)) != len(ids):
            raise StepError(f"step {record.get('step')}: a request appears twice")
        new = [i for i in ids if i not in self.slots]
        if new:
            for i, slot in zip(new, self.engine.acquire(len(new))):
                self.slots[i] = slot
        step_entries = [StepEntry(self.slots[i], list(e["tokens"]), list(e.get("want", [])))
                        for i, e in zip(ids, entries)]
        try:
            logits = self.engine.step(step_entries)
        finally:
            for ended in record.get("end", []):
                slot = self.slots.pop(str(ended), None)
                if slot is not None:
                    self.engine.release(slot)
        return logits
