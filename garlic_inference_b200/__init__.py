"""garlic_inference_b200: a small Qwen3-dense inference library for one B200.

    from garlic_inference_b200 import AutoModel
    model = AutoModel.from_pretrained("/path/to/model", device=0, dtype="bfloat16")
    new_ids = model.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)

Sub-packages: `config` (typed configuration, registry), `weights`
(safetensors, random weights), `parts` (mixer, feed-forward, norm, position
encoding, block), `cache`, `engine` (model, step function, generation loop,
entry point), `sampling`, `ops` and `csrc` (the CUDA kernels).
"""
from .config import ConfigError, Qwen3Config, load_config, register_architecture
from .engine import AutoConfig, AutoModel, GenParams, LanguageModel, StepEntry
from .parts import register_part
from .weights import WeightError, write_random_model

__all__ = ["AutoConfig", "AutoModel", "LanguageModel", "GenParams", "StepEntry", "Qwen3Config",
           "ConfigError", "WeightError", "load_config", "register_architecture", "register_part",
           "write_random_model"]
