"""Interfaces of the parts a layer is put together from, and their registry.

A part is a class registered under a `kind` name.  A configuration names
parts by kind with their sizes and constants as parameters (`PartSpec`); the
model builder looks the class up here, asks it which tensors it wants
(`wanted`), and constructs it with the loaded tensors.  No part knows which
architecture it serves, and a new part needs no change in this package:
register the class and name its kind in a plan.

    class Part                   step_arrays(shape, cache) -> {name: function making an int32 array}
    class Mixer(Part)            cache_requirement() -> KVRequirement | StateRequirement | None
                                 step(x, ctx, cache, position, writes_cache) -> y        [n, hidden]
    class FeedForward(Part)      step(x, ctx) -> y                                        [n, hidden]
    class Norm(Part)             add_norm(delta, residual, ...) -> normed                 [n, size]
    class PositionEncoding(Part) rotary_tables() / on_embedding(residual, ctx)
    class Block(Part)            step(delta, residual, ctx, cache, writes_cache) -> delta
    class Embedding(Part)        step(ctx) -> residual (float32)
    class Head(Part)             step(normed_rows) -> logits (float32)

What a part may read of the batch.  Always, on the device: `ctx.tok_pos` and `ctx.tok_slot` (the
position and the cache slot of every row; padding rows carry slot -1), the cache's tensors, and
whatever the part asked for through `step_arrays` (`ctx.arrays[name]`).  On the host, unless the step
is being recorded (`ctx.captured`): the per-sequence lists `seq_slots / seq_starts / seq_lens /
seq_past`.  A decode step (`ctx.all_single`: one row per sequence) may be recorded into a CUDA graph
and replayed for other sequences, so a part that declares `graph_safe = True` must run such a step
from the device tensors alone.  A mixer with state of its own does that with
`cache.state[ctx.tok_slot.long()]`: row i of the step belongs to slot `tok_slot[i]`, and slot -1
addresses the state region's last row, a spare that no sequence owns, so padding rows read and write
nothing that counts.  Steps that bring several tokens of a sequence are never recorded; there the part
may walk the host lists.

The hidden state between blocks is a pair: the float32 residual stream
`residual` [n, hidden] and a pending `delta` in the activation type that has
not been added yet (None after the embedding).  The next norm adds it in
float32 while it normalises, which saves a pass over the stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..weights.loader import TensorWant

_PARTS: dict[str, type] = {}


def register_part(kind: str, cls: type) -> None:
    """Make `cls` buildable under the name `kind` (replacing an earlier class of that name)."""
    if not (isinstance(cls, type) and issubclass(cls, Part)):
        raise TypeError(f"part {kind!r}: {cls!r} is not a Part class")
    _PARTS[kind] = cls


def part_class(kind: str) -> type:
    try:
        return _PARTS[kind]
    except KeyError:
        raise KeyError(f"unknown part kind {kind!r}; registered: {', '.join(sorted(_PARTS))}") from None


def known_parts() -> list[str]:
    return sorted(_PARTS)


@dataclass
class Runtime:
    """Where and in which precision a model runs."""
    dtype: torch.dtype                  # activation and cache type: bfloat16 or float32
    device: torch.device


@dataclass
class StepShape:
    """The host-side description of a step, before anything is on the device: one entry per sequence."""
    seq_slots: list                     # slot of each sequence
    seq_starts: list                    # first row of each sequence; a sequence's rows are contiguous
    seq_lens: list                      # new tokens of each sequence
    seq_past: list                      # positions already in the cache
    all_single: bool                    # every sequence brings exactly one token


@dataclass
class StepContext:
    """One step's batch as the parts see it.  All tensors are on the device, int32."""
    n_tokens: int                       # rows run in this step (padding rows included)
    tokens: torch.Tensor                # [n_tokens] token ids
    tok_pos: torch.Tensor               # [n_tokens] absolute position of each token in its sequence
    tok_slot: torch.Tensor              # [n_tokens] cache slot of each token, -1 for padding
    # host-side description, for parts that have to walk sequences (ragged prefill of a stateful mixer)
    seq_slots: list = field(default_factory=list)      # slot of each sequence
    seq_starts: list = field(default_factory=list)     # first row of each sequence; rows are contiguous
    seq_lens: list = field(default_factory=list)       # new tokens of each sequence
    seq_past: list = field(default_factory=list)       # positions already in the cache
    all_single: bool = False            # every sequence brings exactly one token (a decode step)
    max_kv_len: int = 0                 # longest sequence after this step (an upper bound is allowed)
    # int32 device tensors that parts asked for through `step_arrays`, by name (uploaded with the step's
    # other arrays in one copy); empty in decode steps
    arrays: dict = field(default_factory=dict)
    status: Optional[torch.Tensor] = None   # int32[1] error flag shared with the cache
    captured: bool = False              # the step is being recorded into a CUDA graph: the host-side
                                        # lists above are empty, everything must come from the tensors


class Part:
    kind: str = ""
    # True if `step` reads the batch only through the context's device tensors and the cache's
    # tensors, so that a recorded decode step can be replayed for other sequences.  A part that
    # walks `seq_slots` / `seq_lens` on the host leaves this False and the engine launches it
    # step by step.
    graph_safe: bool = False

    @classmethod
    def wanted(cls, params: dict) -> dict[str, TensorWant]:
        """Local tensor names this part loads, with shapes, given its parameters."""
        return {}

    def __init__(self, params: dict, load: Callable, rt: Runtime):
        """`load(local_name, out=None)` returns the device tensor (or copies it into `out`)."""
        self.params = dict(params)
        self.rt = rt

    def step_arrays(self, shape: StepShape, cache) -> dict:
        """Small int32 arrays this part wants on the device for the step that `shape` describes, as
        {name: zero-argument function returning a numpy array}.  The engine makes each name once per step
        (parts of one kind ask for the same names), copies them with the step's other arrays and hands
        them over as `ctx.arrays[name]`, each starting on a 16-byte boundary.  `cache` is the part's view of
        the cache.  Not called for recorded decode steps."""
        return {}


class Mixer(Part):
    def cache_requirement(self):
        return None

    def step(self, x, ctx: StepContext, cache, position, writes_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def step(self, x, ctx: StepContext):
        raise NotImplementedError


class Norm(Part):
    def add_norm(self, delta, residual, rows=None, write_residual=True):
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_tables(self):
        """(cos, sin, rotary_dim) float32 tables [max_positions, rotary_dim/2], or None."""
        return None

    def on_embedding(self, residual, ctx: StepContext) -> None:
        """Hook for encodings that act on the embedded tokens (learned absolute positions)."""


class Block(Part):
    def cache_requirement(self):
        return None

    def step_arrays(self, shape: StepShape, cache) -> dict:
        """The arrays of the block's parts (see `Part.step_arrays`)."""
        return {}

    def step(self, delta, residual, ctx: StepContext, cache, writes_cache: bool = True):
        raise NotImplementedError


class Embedding(Part):
    def step(self, ctx: StepContext):
        raise NotImplementedError


class Head(Part):
    def step(self, normed):
        raise NotImplementedError
