"""The plain implementation behind the engine's stepping interface, for the tests.

`PlainStepper` has `alloc_slot`, `free_slot` and `step(entries)` like `LanguageModel`, but no cache and no batch: it
keeps every live sequence's tokens and, for each entry of a step, runs the whole sequence so far through
`plain_qwen3.forward` and returns the rows asked for.  So a schedule of steps can be replayed on the CPU and compared
with the engine step by step: the first step that differs is named, not only the first (request, position).
Upstream has no CPU path for the dense model (its only CPU code is a mixture-of-experts kernel,
src/src-cpu/fp8_expert_cpu.cpp), so this is the reference model with the engine's interface."""
from __future__ import annotations

import numpy as np
import torch

import plain_qwen3 as plain


class _NothingToCheck:
    def check(self) -> None:
        pass


class PlainStepper:
    def __init__(self, model_dir, dtype=torch.float32, max_slots: int = 1 << 20):
        self.cfg, self.weights = plain.read_model_dir(model_dir)
        self.dtype = dtype
        self.max_slots = max_slots
        self.tokens: dict[int, list[int]] = {}
        self._free: list[int] = []
        self._next = 0
        self.engine = _NothingToCheck()

    def alloc_slot(self) -> int:
        if self._free:
            s = self._free.pop()
        else:
            if self._next >= self.max_slots:
                raise RuntimeError("no free slot")
            s, self._next = self._next, self._next + 1
        self.tokens[s] = []
        return s

    def free_slot(self, slot: int) -> None:
        del self.tokens[slot]                       # KeyError on a slot that is not live: freed twice, or never given
        self._free.append(slot)

    def length(self, slot: int) -> int:
        return len(self.tokens[slot])

    def step(self, entries):
        """entries: objects with .slot, .tokens, .want (or tuples of the three).  float32 logits [n_wanted, vocab]
        in the order of the entries and of each entry's `want`, or None when nothing is wanted."""
        rows = []
        for e in entries:
            slot, toks, want = (e.slot, e.tokens, e.want) if hasattr(e, "slot") else e
            past = len(self.tokens[slot])
            self.tokens[slot].extend(int(t) for t in toks)
            if len(want):
                logits = plain.forward(self.cfg, self.weights, self.tokens[slot], self.dtype).to(torch.float32)
                rows += [logits[past + w] for w in want]
        return torch.stack(rows) if rows else None


def first_step_that_differs(engine_model, stepper: PlainStepper, steps, tol: float):
    """Replay `steps` on both, step by step; returns (step number, relative error) of the first step whose logits
    differ by more than `tol` of the step's largest plain logit, or None."""
    from garlic_inference_b200 import StepEntry
    slots_a, slots_b = {}, {}
    for rec in steps:
        ea, eb = [], []
        for e in rec["entries"]:
            if e["id"] not in slots_a:
                slots_a[e["id"]], slots_b[e["id"]] = engine_model.alloc_slot(), stepper.alloc_slot()
            ea.append(StepEntry(slots_a[e["id"]], e["tokens"], e["want"]))
            eb.append((slots_b[e["id"]], e["tokens"], e["want"]))
        got, want = engine_model.step(ea), stepper.step(eb)
        assert (got is None) == (want is None), f"step {rec['step']}: one side returned logits, the other none"
        if got is not None:
            g, w = got.float().cpu().numpy(), want.numpy()
            assert g.shape == w.shape, f"step {rec['step']}: {g.shape} against {w.shape}"
            err = float(np.abs(g - w).max() / np.abs(w).max())
            if not np.isfinite(g).all() or err > tol:
                return rec["step"], err
        for rid in rec["end"]:
            engine_model.free_slot(slots_a.pop(rid))
            stepper.free_slot(slots_b.pop(rid))
    engine_model.engine.check()
    return None
