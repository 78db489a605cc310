"""The step function: one forward pass over a batch of sequences with unequal
numbers of new tokens, from the cache, returning logits at the wanted places.

A step brings, for each sequence, its next tokens (a whole prompt, a chunk of
one, or a single token).  All tokens of the step run as one batch of rows:
products over all rows at once, attention per token over its own sequence's
cache.  Only the wanted rows go through the final norm and the head.

Upstream's forward is rectangular (one length for the whole batch), takes the
positions from the caller, computes logits at every position and has the
batch size baked into its cache (src/models/qwen3/qwen3.cpp:255-307,
src/src-cuda/kvcache.cu:61-84).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import PagedCache
from ..parts import StepContext, StepShape
from .model import DecoderModel


class StepError(ValueError):
    """A step that cannot run as described (bad token id, bad `want` index, empty entry)."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)    # indices into `tokens` whose logits are asked for


class _Staging:
    """One pinned host buffer and one device buffer for the step's int32 arrays, reused across steps."""

    def __init__(self, device: torch.device):
        self.device = device
        self.capacity = 0
        self.host = self.dev = None
        self.event: Optional[torch.cuda.Event] = None
        self.bytes_uploaded = 0

    def upload(self, arrays: list[np.ndarray]) -> list[torch.Tensor]:
        """Copy the int32 arrays to the device in one transfer; each starts on a 16-byte boundary."""
        offsets, total = [], 0
        for a in arrays:
            offsets.append(total)
            total += -(-a.size // 4) * 4
        if total > self.capacity:
            self.capacity = max(1024, 2 * total)
            self.host = torch.empty(self.capacity, dtype=torch.int32)
            if self.device.type == "cuda":
                self.host = self.host.pin_memory()
            self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)
            self.event = None
        if self.event is not None:
            self.event.synchronize()                 # the last copy out of the pinned buffer is done
        out = []
        host_np = self.host.numpy()
        for a, off in zip(arrays, offsets):
            host_np[off:off + a.size] = a
            out.append(self.dev[off:off + a.size])
        self.dev[:total].copy_(self.host[:total], non_blocking=True)
        self.bytes_uploaded += 4 * total
        if self.device.type == "cuda":
            self.event = torch.cuda.Event()
            self.event.record()
        return out


class Engine:
    """A model, its cache, and the step function over them."""

    def __init__(self, model: DecoderModel, max_tokens: int, page_size: int = 64,
                 max_slots: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.rt = model.rt
        self.cache = PagedCache(model.cache_requirements(), max_tokens=max_tokens,
                                max_positions=model.max_positions, dtype=model.rt.dtype,
                                device=model.rt.device, page_size=page_size, max_slots=max_slots)
        self._staging = _Staging(model.rt.device)
        if model.rt.device.type == "cuda":
            # library products accumulate in float32 all the way, and the float32 engine never uses them
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
            torch.backends.cuda.matmul.allow_tf32 = False
        # decode steps are replayed from CUDA graphs when every part allows it
        self.graphs = None
        if use_graphs and model.rt.device.type == "cuda" and model.graph_safe:
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(model, self.cache)

    # ---- slots ---------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # ---- the step --------------------------------------------------------------------
    def describe(self, entries: Sequence[StepEntry]):
        """Host arrays of a step: (tokens, tok_pos, tok_slot, want_rows) and the per-sequence lists."""
        vocab = self.model.vocab_size
        toks, pos, slot, want_rows = [], [], [], []
        starts, lens, past = [], [], []
        row = 0
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"the entry of slot {e.slot} brings no tokens")
            t = np.asarray(e.tokens, dtype=np.int64)
            if t.min() < 0 or t.max() >= vocab:
                bad = int(t[(t < 0) | (t >= vocab)][0])
                raise StepError(f"token id {bad} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"want index {w} is outside the entry's {n} tokens")
                want_rows.append(row + w)
            p0 = self.cache.length(e.slot)
            toks.append(t.astype(np.int32))
            pos.append(np.arange(p0, p0 + n, dtype=np.int32))
            slot.append(np.full(n, e.slot, dtype=np.int32))
            starts.append(row), lens.append(n), past.append(p0)
            row += n
        cat = (lambda xs: np.concatenate(xs) if xs else np.zeros(0, dtype=np.int32))
        return (cat(toks), cat(pos), cat(slot), np.asarray(want_rows, dtype=np.int32)), (starts, lens, past)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens; returns float32 logits [n_wanted, vocab] on the device in the order
        of the entries and of each entry's `want`, or None when nothing is wanted."""
        entries = list(entries)
        if not entries:
            return None
        if self.graphs is not None and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries):
            # the common decode step (one token each, each wanted), without per-entry array work
            logits = self._decode_fast(entries)
            if logits is not None:
                return logits
        (toks, pos, slot, want_rows), (starts, lens, past) = self.describe(entries)
        slots = [e.slot for e in entries]
        self.cache.prepare(slots, lens)                  # raises before anything is launched
        if self.graphs is not None and all(n == 1 for n in lens):
            logits = self.graphs.run(slots, past, toks, None)
            if logits is not None:
                self.cache.commit(slots, lens)
                if want_rows.size == 0:
                    return None
                if want_rows.size == len(slots):         # one token each and each wanted: rows as they are
                    return logits
                return logits[torch.from_numpy(want_rows.astype(np.int64)).to(logits.device)]
        shape = StepShape(slots, starts, lens, past, all(n == 1 for n in lens))
        extra = self.model.step_arrays(shape, self.cache)          # what the parts want on the device besides
        uploaded = self._staging.upload([*(a.reshape(-1) for a in extra.values()), toks, pos, slot, want_rows])
        n_extra = len(extra)
        d_toks, d_pos, d_slot, d_want = uploaded[n_extra:]
        ctx = StepContext(
            n_tokens=int(toks.size), tokens=d_toks, tok_pos=d_pos, tok_slot=d_slot,
            arrays={name: dev.view(a.shape) for (name, a), dev in zip(extra.items(), uploaded[:n_extra])},
            seq_slots=slots, seq_starts=starts, seq_lens=lens, seq_past=past, all_single=shape.all_single,
            max_kv_len=max(p + n for p, n in zip(past, lens)),
            status=self.cache.status)
        logits = self.model.forward(ctx, self.cache, d_want if want_rows.size else None)
        self.cache.commit(slots, lens)
        return logits

    def _decode_fast(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        toks = [int(e.tokens[0]) for e in entries]
        if min(toks) < 0 or max(toks) >= self.model.vocab_size:
            bad = next(t for t in toks if t < 0 or t >= self.model.vocab_size)
            raise StepError(f"token id {bad} is outside the vocabulary of {self.model.vocab_size}")
        if any(e.want[0] != 0 for e in entries):
            raise StepError("want index outside the entry's 1 tokens")
        slots = [e.slot for e in entries]
        lens = [1] * len(slots)
        self.cache.prepare(slots, lens)
        past = [self.cache.length(s) for s in slots]
        logits = self.graphs.run(slots, past, np.asarray(toks, dtype=np.int32), None)
        if logits is not None:
            self.cache.commit(slots, lens)
        return logits

    def step_decode_device(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One decode step whose tokens are already on the device (int32 [len(slots)], for instance
        the sampler's output): one token per listed slot, logits [len(slots), vocab] for all of them.
        Nothing comes back to the host, so steps can be queued without waiting for each other.  The
        ids are not checked against the vocabulary on the host; the embedding kernel writes zeros for
        an id outside it."""
        slots = list(slots)
        n = len(slots)
        if tokens.dtype != torch.int32 or tokens.numel() != n or not tokens.is_contiguous():
            raise StepError(f"tokens must be a dense int32 tensor with one id per slot ({n})")
        lens = [1] * n
        self.cache.prepare(slots, lens)
        past = [self.cache.length(s) for s in slots]
        if self.graphs is not None:
            logits = self.graphs.run(slots, past, None, tokens)
            if logits is not None:
                self.cache.commit(slots, lens)
                return logits
        d_pos, d_slot, d_want = self._staging.upload([np.asarray(past, dtype=np.int32),
                                                      np.asarray(slots, dtype=np.int32),
                                                      np.arange(n, dtype=np.int32)])
        ctx = StepContext(n_tokens=n, tokens=tokens, tok_pos=d_pos, tok_slot=d_slot, seq_slots=slots,
                          seq_starts=list(range(n)), seq_lens=lens, seq_past=past, all_single=True,
                          max_kv_len=max(past) + 1, status=self.cache.status)
        logits = self.model.forward(ctx, self.cache, d_want)
        self.cache.commit(slots, lens)
        return logits

    @property
    def bytes_uploaded(self) -> int:
        """Bytes of step descriptions (ids, positions, slots) copied to the device so far."""
        return self._staging.bytes_uploaded + (self.graphs.bytes_uploaded if self.graphs else 0)

    def check(self) -> None:
        """Raise if a kernel of an earlier step met an index outside the cache, or gave up a wait
        (synchronises)."""
        self.cache.check_status()
        if self.rt.device.type == "cuda":
            from ..ops import kernels
            kernels.check_bounded_waits(self.rt.device)
