"""A decoder built from a `ModelPlan`: embedding, blocks run in the order the
schedule lists, final norm, head.

Upstream's model class owns its tensors by field and runs its layers in a
fixed loop (src/models/qwen3/qwen3.h:77-93, qwen3.cpp:292-303).  Here the
model is data: which parts, with which sizes, in which order, reading which
cache entry.  `wanted_tensors(plan)` lists every checkpoint tensor the plan
needs with its shape, which is also what random initialisation writes.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.base import ModelPlan, PartSpec
from ..parts import Runtime, StepContext, part_class
from ..weights.loader import TensorWant, WeightError, device_dtype


def _part_wants(spec: PartSpec) -> dict[str, TensorWant]:
    cls = part_class(spec.kind)
    local = cls.wanted(spec.params)
    missing = [n for n in local if n not in spec.weights]
    if missing:
        raise WeightError(f"part '{spec.kind}' wants tensors {missing} that its plan entry does not name")
    return {spec.weights[n]: w for n, w in local.items()}


def plan_part_specs(plan: ModelPlan) -> list[PartSpec]:
    specs = [plan.embedding, *plan.positions.values()]
    for layer in plan.layers:
        specs += [layer.mixer, layer.feed_forward, *layer.norms.values()]
    return specs + [plan.final_norm, plan.head]


def wanted_tensors(plan: ModelPlan) -> dict[str, TensorWant]:
    """Checkpoint name -> shape and role, for every tensor the plan's parts load."""
    out: dict[str, TensorWant] = {}
    for spec in plan_part_specs(plan):
        for name, want in _part_wants(spec).items():
            if name in out and tuple(out[name].shape) != tuple(want.shape):
                raise WeightError(f"tensor '{name}' is wanted with shapes {list(out[name].shape)} and "
                                  f"{list(want.shape)} by two parts")
            out.setdefault(name, want)
    return out


class _PartLoader:
    """What a part's constructor calls to get its tensors onto the device."""

    def __init__(self, spec: PartSpec, source, rt: Runtime, shared: dict):
        self.spec, self.source, self.rt, self.shared = spec, source, rt, shared

    def dtype(self, *locals_: str) -> torch.dtype:
        """The type in which the named tensor is kept on the device; for several names (tensors packed into
        one) the widest of theirs, so that a tensor stored in 32 bits is never narrowed by its neighbours."""
        kept = [device_dtype(self.source.stored_dtype(self.spec.weights[n]), self.rt.dtype) for n in locals_]
        return torch.float32 if torch.float32 in kept else kept[0]

    def __call__(self, local: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        name = self.spec.weights[local]
        if out is not None:
            out.copy_(self.source.tensor(name))
            return out
        if name not in self.shared:                 # a tensor named by two parts is loaded once
            self.shared[name] = self.source.tensor(name).to(device=self.rt.device, dtype=self.dtype(local)).contiguous()
        return self.shared[name]


class DecoderModel:
    def __init__(self, plan: ModelPlan, source, rt: Runtime):
        self.plan, self.rt = plan, rt
        shared: dict[str, torch.Tensor] = {}

        def make(spec: PartSpec):
            return part_class(spec.kind)(spec.params, _PartLoader(spec, source, rt, shared), rt)

        self.embedding = make(plan.embedding)
        self.positions = {name: make(spec) for name, spec in plan.positions.items()}
        self.blocks = []
        for i, layer in enumerate(plan.layers):
            if layer.position is not None and layer.position not in self.positions:
                raise KeyError(f"layer {i} names position encoding {layer.position!r}; the plan has "
                               f"{sorted(self.positions)}")
            block_cls = part_class(layer.block)
            self.blocks.append(block_cls(make(layer.mixer), make(layer.feed_forward),
                                         {n: make(s) for n, s in layer.norms.items()},
                                         self.positions.get(layer.position), rt))
        self.final_norm = make(plan.final_norm)
        self.head = make(plan.head)
        self.schedule = tuple(plan.schedule)
        for e in self.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise IndexError(f"the schedule names layer {e.layer}; the plan has {len(self.blocks)}")
        self.vocab_size, self.hidden_size, self.max_positions = plan.vocab_size, plan.hidden_size, plan.max_positions

    @property
    def graph_safe(self) -> bool:
        """True if every part allows a decode step to be recorded into a CUDA graph."""
        return all(p.graph_safe for p in (self.embedding, *self.positions.values(), *self.blocks,
                                          self.final_norm, self.head))

    def cache_requirements(self) -> list:
        """What each cache entry has to hold; entries shared by several runs must agree."""
        reqs: list = [None] * self.plan.n_cache_entries()
        written = [False] * len(reqs)
        for e in self.schedule:
            req = self.blocks[e.layer].cache_requirement()
            if reqs[e.cache] is not None and reqs[e.cache] != req:
                raise ValueError(f"cache entry {e.cache} is used by layers with different needs: "
                                 f"{reqs[e.cache]} and {req}")
            if not e.writes_cache and not written[e.cache]:
                raise ValueError(f"the schedule reads cache entry {e.cache} before any layer wrote it")
            reqs[e.cache] = req
            written[e.cache] = written[e.cache] or e.writes_cache
        return reqs

    def step_arrays(self, shape, cache) -> dict:
        """The int32 arrays the scheduled layers' parts want on the device for this step, each name made once
        ({name: numpy array}); the engine copies them with the step's own arrays."""
        out: dict = {}
        for e in self.schedule:
            for name, make in self.blocks[e.layer].step_arrays(shape, cache.view(e.cache)).items():
                if name not in out:
                    out[name] = make()
        return out

    def forward(self, ctx: StepContext, cache, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled layer; float32 logits [n_wanted, vocab] at
        `want_rows` (int32 row indices), or None when nothing is wanted."""
        residual = self.embedding.step(ctx)
        for pos in self.positions.values():
            pos.on_embedding(residual, ctx)
        delta = None
        for e in self.schedule:
            delta = self.blocks[e.layer].step(delta, residual, ctx, cache.view(e.cache), e.writes_cache)
        if want_rows is None or want_rows.numel() == 0:
            return None
        normed = self.final_norm.add_norm(delta, residual, rows=want_rows)
        return self.head.step(normed)

    def weight_bytes(self) -> int:
        """Bytes of all distinct weight tensors on the device."""
        seen, total = set(), 0
        for obj in self._all_parts():
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_floating_point() and v.data_ptr() not in seen and v.numel():
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    def _all_parts(self):
        yield self.embedding
        yield from self.positions.values()
        for b in self.blocks:
            yield from (b.mixer, b.feed_forward, *[v for v in vars(b).values() if hasattr(v, "add_norm")])
        yield self.final_norm
        yield self.head
