"""Typed configuration of the Qwen3 dense decoder (`Qwen3ForCausalLM`).

Keys are those of the architecture's own config.json.  Upstream reads ten of
them, all required and with no check (src/models/qwen3/qwen3.cpp:24-40); it
ignores `tie_word_embeddings` (the head is always the embedding table,
qwen3.cpp:58) and every sliding-window key.  Here `tie_word_embeddings` and
the window keys are honoured, `head_dim` may be absent (hidden // heads), and
options whose arithmetic this library does not have are refused by name.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

from .base import (ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry,
                   optional, require)

ARCHITECTURE = "Qwen3ForCausalLM"


@dataclass
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    # sliding window: layer i uses a window of `sliding_window` keys when
    # `layer_types[i] == "sliding_attention"`, or, without `layer_types`, when
    # `use_sliding_window` and i >= `max_window_layers`.
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None
    layer_types: Optional[list] = None
    architectures: list = field(default_factory=lambda: [ARCHITECTURE])

    def __post_init__(self):
        if self.head_dim is None:
            if self.num_attention_heads <= 0 or self.hidden_size % self.num_attention_heads:
                raise ConfigError("config: 'head_dim' is absent and hidden_size is not a "
                                  "multiple of num_attention_heads")
            self.head_dim = self.hidden_size // self.num_attention_heads
        self.validate()

    # ---- reading and writing -------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, where: str = "config.json") -> "Qwen3Config":
        refuse = []
        if optional(cfg, "hidden_act", str, "silu", where) != "silu":
            refuse.append(f"hidden_act={cfg['hidden_act']!r} (only 'silu' is computed)")
        if optional(cfg, "attention_bias", bool, False, where):
            refuse.append("attention_bias=true (projections have no bias here)")
        if cfg.get("rope_scaling") is not None:
            refuse.append("rope_scaling (only unscaled rotary positions are computed)")
        if optional(cfg, "attention_dropout", float, 0.0, where) != 0.0:
            refuse.append("attention_dropout != 0")
        if refuse:
            raise ConfigError(f"{where}: not supported: " + "; ".join(refuse))
        return cls(
            hidden_size=require(cfg, "hidden_size", int, where),
            num_hidden_layers=require(cfg, "num_hidden_layers", int, where),
            num_attention_heads=require(cfg, "num_attention_heads", int, where),
            num_key_value_heads=require(cfg, "num_key_value_heads", int, where),
            intermediate_size=require(cfg, "intermediate_size", int, where),
            vocab_size=require(cfg, "vocab_size", int, where),
            max_position_embeddings=require(cfg, "max_position_embeddings", int, where),
            head_dim=optional(cfg, "head_dim", int, None, where),
            rms_norm_eps=optional(cfg, "rms_norm_eps", float, 1e-6, where),
            rope_theta=optional(cfg, "rope_theta", float, 1e6, where),
            tie_word_embeddings=optional(cfg, "tie_word_embeddings", bool, False, where),
            sliding_window=optional(cfg, "sliding_window", int, None, where),
            use_sliding_window=optional(cfg, "use_sliding_window", bool, False, where),
            max_window_layers=optional(cfg, "max_window_layers", int, None, where),
            layer_types=optional(cfg, "layer_types", list, None, where),
            architectures=list(cfg.get("architectures") or [ARCHITECTURE]),
        )

    @classmethod
    def from_json_file(cls, path) -> "Qwen3Config":
        path = Path(path)
        try:
            cfg = json.loads(path.read_text())
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
        return cls.from_dict(cfg, str(path))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["rope_scaling"] = None
        d["model_type"] = "qwen3"
        d["torch_dtype"] = "bfloat16"
        return d

    # ---- checks ----------------------------------------------------------------
    def validate(self) -> None:
        bad = []
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "intermediate_size", "vocab_size",
                     "max_position_embeddings", "head_dim"):
            if getattr(self, name) <= 0:
                bad.append(f"{name} must be positive, found {getattr(self, name)}")
        if not bad and self.num_attention_heads % self.num_key_value_heads:
            bad.append(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                       f"num_key_value_heads ({self.num_key_value_heads})")
        if not bad and self.head_dim % 2:
            bad.append(f"head_dim ({self.head_dim}) must be even for rotary positions")
        if not (self.rms_norm_eps > 0):
            bad.append(f"rms_norm_eps must be positive, found {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            bad.append(f"rope_theta must be positive, found {self.rope_theta}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            bad.append(f"sliding_window must be positive, found {self.sliding_window}")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                bad.append(f"layer_types has {len(self.layer_types)} entries for "
                           f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    bad.append(f"layer_types entry {t!r} is neither 'full_attention' nor "
                               "'sliding_attention'")
                    break
            if "sliding_attention" in self.layer_types and self.sliding_window is None:
                bad.append("layer_types names 'sliding_attention' but sliding_window is absent")
        if bad:
            raise ConfigError("config: " + "; ".join(bad))

    # ---- derived -----------------------------------------------------------------
    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_windows(self) -> list:
        """Window of each layer in keys, None = all earlier keys."""
        n = self.num_hidden_layers
        if self.layer_types is not None:
            return [self.sliding_window if t == "sliding_attention" else None
                    for t in self.layer_types]
        if self.use_sliding_window and self.sliding_window is not None:
            first = n if self.max_window_layers is None else self.max_window_layers
            return [self.sliding_window if i >= first else None for i in range(n)]
        return [None] * n

    def plan(self) -> ModelPlan:
        """The decoder as parts: per layer an RMSNorm, grouped-query attention
        with per-head q/k RMSNorm before the rotation, another RMSNorm and a
        SwiGLU feed-forward, in the pre-norm residual arrangement
        (src/models/qwen3/qwen3.cpp:205-253); each layer runs once, in order,
        on a cache entry of its own."""
        eps = self.rms_norm_eps
        layers = []
        for i, window in enumerate(self.layer_windows()):
            p = f"model.layers.{i}."
            mixer = PartSpec(
                "gqa_attention",
                dict(hidden_size=self.hidden_size, n_heads=self.num_attention_heads,
                     n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                     qk_norm=True, qk_norm_eps=eps, window=window,
                     softmax_scale=self.head_dim ** -0.5),
                dict(q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
                     v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight",
                     q_norm=p + "self_attn.q_norm.weight", k_norm=p + "self_attn.k_norm.weight"))
            ffn = PartSpec(
                "swiglu_mlp",
                dict(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size),
                dict(gate_proj=p + "mlp.gate_proj.weight", up_proj=p + "mlp.up_proj.weight",
                     down_proj=p + "mlp.down_proj.weight"))
            norms = {
                "input": PartSpec("rms_norm", dict(size=self.hidden_size, eps=eps),
                                  dict(weight=p + "input_layernorm.weight")),
                "post_mixer": PartSpec("rms_norm", dict(size=self.hidden_size, eps=eps),
                                       dict(weight=p + "post_attention_layernorm.weight")),
            }
            layers.append(LayerSpec("pre_norm_residual", mixer, ffn, norms, position="rotary"))
        head_weights = ({"weight": "model.embed_tokens.weight"} if self.tie_word_embeddings
                        else {"weight": "lm_head.weight"})
        return ModelPlan(
            architecture=ARCHITECTURE,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding",
                               dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size),
                               dict(weight="model.embed_tokens.weight")),
            positions={"rotary": PartSpec(
                "rotary", dict(head_dim=self.head_dim, rotary_dim=self.head_dim,
                               theta=self.rope_theta, max_positions=self.max_position_embeddings))},
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rms_norm", dict(size=self.hidden_size, eps=eps),
                                dict(weight="model.norm.weight")),
            head=PartSpec("linear_head",
                          dict(hidden_size=self.hidden_size, vocab_size=self.vocab_size),
                          head_weights),
        )
