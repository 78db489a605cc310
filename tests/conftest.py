import sys
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
for p in (str(HERE), str(HERE.parent)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu); everything else runs on the CPU")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Folders with config.json and model.safetensors for the tiny configurations, made once, in a
    temporary place."""
    import tiny
    made = {}

    def get(name: str) -> Path:
        if name not in made:
            made[name] = tiny.write_model(name, tmp_path_factory.mktemp(f"tiny_{name}"))
        return made[name]

    return get


@pytest.fixture(scope="session")
def gpu_models(model_dirs):
    """LanguageModel per (configuration, dtype), loaded once per session."""
    made = {}

    def get(name: str, dtype: str, max_tokens: int = 4096, page_size: int = 16):
        key = (name, dtype, max_tokens, page_size)
        if key not in made:
            from garlic_inference_b200 import AutoModel
            made[key] = AutoModel.from_pretrained(model_dirs(name), device=0, dtype=dtype,
                                                  max_tokens=max_tokens, page_size=page_size)
        return made[key]

    return get
