"""The Python entry point: a model folder in, a model that steps and generates out.

Names follow upstream's (`AutoConfig::from_pretrained`, `AutoModel::from_pretrained(dir, device)`,
src/models/model.h:6-12); what upstream's `main` does around the model
(inference.cpp:53-168: caches, the loop, the argmax) is `LanguageModel.generate`.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Sequence

import torch

from ..config import load_config
from ..parts import Runtime
from ..sampling import Sampler, SamplingParams
from ..weights import Checkpoint, RandomSource
from .generate import GenerationLoop, GenParams
from .model import DecoderModel, wanted_tensors
from .step import Engine, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def engine_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', not {dtype!r}") from None


def _device(device) -> torch.device:
    if isinstance(device, int):
        return torch.device("cuda", device)
    return torch.device(device)


class AutoConfig:
    @staticmethod
    def from_pretrained(model_dir):
        """The typed configuration of the folder, its class chosen by config.json's `architectures[0]`."""
        return load_config(model_dir)


class LanguageModel:
    """A model on the GPU with its cache: `step` for given tokens, `generate` for sampled ones."""

    def __init__(self, config, model: DecoderModel, max_tokens: int, page_size: int = 64,
                 default_stop_ids: Sequence[int] = (), use_graphs: bool = True, max_slots: Optional[int] = None):
        self.config = config
        self.model = model
        self.engine = Engine(model, max_tokens=max_tokens, page_size=page_size, use_graphs=use_graphs,
                             max_slots=max_slots)
        self.sampler = Sampler(model.rt.device)
        self.default_stop_ids = tuple(default_stop_ids)
        self.last_stats = None
        self.run_ahead = True          # generate() launches each decode step before it has read the last one's tokens

    # ---- construction ----------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir, device=0, dtype="bfloat16", max_tokens: int = 8192,
                        page_size: int = 64, use_graphs: bool = True, max_slots: Optional[int] = None) -> "LanguageModel":
        """`max_tokens` sizes the cache (tokens that live requests hold, each request's count in units of 64);
        `max_slots` is the most requests that can be live at once (default: one per 64 tokens of the cache)."""
        from ..ops import require_gpu
        dev = _device(device)
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        require_gpu()
        config = load_config(model_dir)
        plan = config.plan()
        ckpt = Checkpoint(model_dir)
        ckpt.check(wanted_tensors(plan))
        model = DecoderModel(plan, ckpt, Runtime(engine_dtype(dtype), dev))
        stop = ()
        gen_cfg = Path(model_dir) / "generation_config.json"
        if gen_cfg.is_file():
            eos = json.loads(gen_cfg.read_text()).get("eos_token_id")
            stop = tuple(eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        return cls(config, model, max_tokens, page_size, stop, use_graphs, max_slots)

    @classmethod
    def from_random(cls, config, seed: int = 0, device=0, dtype="bfloat16", max_tokens: int = 8192,
                    page_size: int = 64, std: float = 0.02, norm_std: float = 0.0,
                    use_graphs: bool = True, max_slots: Optional[int] = None) -> "LanguageModel":
        """Random weights made on the device (bfloat16 storage), nothing written to disk."""
        from ..ops import require_gpu
        dev = _device(device)
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        require_gpu()
        plan = config.plan()
        source = RandomSource(wanted_tensors(plan), seed=seed, std=std, norm_std=norm_std,
                              dtype=torch.bfloat16, device=dev)
        return cls(config, DecoderModel(plan, source, Runtime(engine_dtype(dtype), dev)), max_tokens, page_size,
                   use_graphs=use_graphs, max_slots=max_slots)

    # ---- stepping ----------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def step(self, entries: Sequence) -> Optional[torch.Tensor]:
        """entries: StepEntry or (slot, tokens, want) tuples.  float32 logits [n_wanted, vocab] on the device."""
        return self.engine.step([e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries])

    # ---- generation ----------------------------------------------------------------------
    def _pick(self, logits, request_ids, token_indices, params: GenParams) -> list[int]:
        toks = self.sampler.sample(logits, SamplingParams(params.temperature, params.seed), request_ids,
                                   token_indices)
        return toks.tolist()                        # device -> host: the step's only synchronisation

    def _pick_on_device(self, logits, request_ids, token_indices, params: GenParams) -> "_Picked":
        toks = self.sampler.sample(logits, SamplingParams(params.temperature, params.seed), request_ids,
                                   token_indices)
        if not hasattr(self, "_pinned"):            # two pinned buffers, used in turn: a copy per step in flight
            n = self.engine.cache.max_slots
            self._pinned, self._pinned_turn = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)], 0
        self._pinned_turn ^= 1
        return _Picked(toks, self._pinned[self._pinned_turn])

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128, temperature: float = 0.0,
                 seed: int = 0, stop_token_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None) -> list[list[int]]:
        """New token ids for each prompt (lists of ids).  Prompts run in batches that start together."""
        params = GenParams(max_new_tokens=max_new_tokens, temperature=temperature, seed=seed,
                           stop_token_ids=self.default_stop_ids if stop_token_ids is None else tuple(stop_token_ids))
        cache = self.engine.cache
        ahead = self.engine.rt.device.type == "cuda" and self.run_ahead
        loop = GenerationLoop(self.engine, self._pick, capacity_tokens=cache.max_tokens,
                              max_positions=self.model.max_positions,
                              max_batch=min(max_batch or cache.max_slots, cache.max_slots),
                              device_picker=self._pick_on_device if ahead else None)
        out = loop.run(prompts, params)
        self.last_stats = loop.stats
        self.engine.check()
        return out


class _Picked:
    """The tokens chosen in one step, on the device, with their copy to the host under way."""

    def __init__(self, tokens: torch.Tensor, pinned: Optional[torch.Tensor], host_rows=None, parent=None):
        self.tokens, self._pinned, self._rows, self._parent = tokens, pinned, host_rows, parent
        self._event = None

    def start_copy(self) -> None:
        n = self.tokens.numel()
        self._pinned[:n].copy_(self.tokens, non_blocking=True)
        self._event = torch.cuda.Event()
        self._event.record()

    def to_host(self) -> list:
        if self._parent is not None:
            all_rows = self._parent.to_host()
            return [all_rows[r] for r in self._rows]
        if not hasattr(self, "_list"):
            self._event.synchronize()
            self._list = self._pinned[:self.tokens.numel()].tolist()
        return self._list

    def select(self, rows) -> torch.Tensor:
        """The device tokens of the listed rows."""
        idx = torch.tensor(list(rows), dtype=torch.int64, device=self.tokens.device)
        return self.tokens.index_select(0, idx).contiguous()

    def narrowed(self, rows) -> "_Picked":
        """These rows only (the others belonged to requests that have ended since)."""
        return _Picked(self.select(rows), None, host_rows=list(rows), parent=self)


class AutoModel:
    @staticmethod
    def from_pretrained(model_dir, device=0, **kwargs) -> LanguageModel:
        """The model of the folder on GPU `device`, its class chosen by config.json."""
        return LanguageModel.from_pretrained(model_dir, device=device, **kwargs)

    @staticmethod
    def from_random(config, seed: int = 0, device=0, **kwargs) -> LanguageModel:
        """A model of the configuration's sizes with random weights made on GPU `device`."""
        return LanguageModel.from_random(config, seed=seed, device=device, **kwargs)
