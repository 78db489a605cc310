"""Plain, slow restatement of the Qwen3 dense decoder, used only by the tests.

Whole sequences, no cache, one function for each part, torch on the CPU.  It
shares no code with the package under test: it has its own reader for
config.json and for safetensors files and its own arithmetic.

It rests on the formulas of NikolayBlagoev/garlic-inference (each function
cites the file and lines it restates).  That project's model code is C++/CUDA
with no CPU path for the dense model, so it cannot run on the CPU.  It was
compiled unmodified for a B200 with a small driver and run there on two tiny
tied random models in bfloat16 (batch 2, prompts of 40 tokens, 8 decode steps);
its logits are kept under tests/golden with the script that made them, and
tests/test_reference_golden.py compares this file with them at every position:
worst difference 3.4e-3 and 7.0e-3 of the largest logit (bfloat16 rounding),
against 2e-1 to 1.3 for a wrong key/value head mapping or rotation.

Two things are stated here that the upstream files leave to a library:
  * grouped-query attention: query head h reads key/value head h // (n_q // n_kv)
    (confirmed by the comparison above);
  * a sliding window of w keys: query at position i sees keys j with
    i - w < j <= i (upstream has no window; w = None means every earlier key).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------
# files
# --------------------------------------------------------------------------
_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, a JSON header, then raw tensors
    (src/models/loader.h:30-54).  Everything floating is returned as float32."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        arr = np.frombuffer(raw[base + lo:base + hi], dtype=np_dtype).reshape(info["shape"])
        if info["dtype"] == "BF16":
            t = torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy())
        elif info["dtype"] in ("F32", "F16"):
            t = torch.from_numpy(arr.astype(np.float32))
        else:
            t = torch.from_numpy(arr.copy())
        out[name] = t
    return out


def read_model_dir(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


def layer_windows(cfg: dict) -> list:
    """Window of each layer (None = all keys) from the architecture's own keys:
    `layer_types` when present, else `use_sliding_window`, `sliding_window`
    and `max_window_layers` (layers from that index on use the window)."""
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is not None:
        return [w if t == "sliding_attention" else None for t in types]
    if cfg.get("use_sliding_window", False) and w is not None:
        first = cfg.get("max_window_layers", n)
        return [w if i >= first else None for i in range(n)]
    return [None] * n


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t, :] = table[id[t], :], no scaling (src/src-cuda/embedding.cu:29-53,
    src/models/qwen3/qwen3.cpp:263-265)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight is used
    as it is (src/src-cuda/norm.cu:17-48)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> torch.Tensor:
    """inv_freq[i] = theta^(-2i/d) for i < d/2; angle = pos * inv_freq[i]
    (src/src-cuda/rope.cu:3-16, 41-66).  Angles are made in float64 and then
    rounded, so that large positions do not lose their low bits."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = theta ** (-2.0 * i / head_dim)
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    return ang.to(dtype)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half on the whole head, scaling 1.0 (src/src-cuda/rope.cu:109-131):
    y[i] = x[i] cos - x[i+d/2] sin ; y[i+d/2] = x[i+d/2] cos + x[i] sin.
    x is [S, heads, d]."""
    d = x.shape[-1]
    ang = rope_angles(positions, d, theta, torch.float64)
    cos = ang.cos().to(x.dtype)[:, None, :]
    sin = ang.sin().to(x.dtype)[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention_scores(q, k, v, window=None) -> torch.Tensor:
    """softmax(q k^T / sqrt(d) + causal mask) v, one sequence, every key in view
    (src/src-cuda/attention/fattn.cu:74-86: scale 1/sqrt(head_dim), causal).
    q [S, n_q, d]; k, v [S, n_kv, d]; returns [S, n_q, d]."""
    S, n_q, d = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    out = torch.empty_like(q)
    pos = torch.arange(S)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > (pos[:, None] - window)
    for h in range(n_q):
        kh, vh = k[:, h // g, :], v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) / math.sqrt(d)
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ vh
    return out


def attention_block(x, w, prefix, cfg, positions, window=None) -> torch.Tensor:
    """q/k/v projections without bias, per-head RMSNorm of q and k before the
    rotation, attention, output projection (src/models/qwen3/qwen3.cpp:140-179).
    x [S, H]."""
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    S = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(S, n_q, d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(S, n_kv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(S, n_kv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    q = apply_rope(q, positions, theta)
    k = apply_rope(k, positions, theta)
    o = attention_scores(q, k, v, window).reshape(S, n_q * d)
    return o @ w[prefix + "o_proj.weight"].T


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + exp(-z)) (src/src-cuda/activations/activations.cuh:4-6)."""
    return z / (1.0 + torch.exp(-z))


def swiglu_mlp(x, w, prefix) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), no biases (src/models/qwen3/qwen3.cpp:186-203)."""
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    return (silu(gate) * up) @ w[prefix + "down_proj.weight"].T


def decoder_layer(h, w, i, cfg, positions, window=None) -> torch.Tensor:
    """r = h; x = norm(h); r = attn(x) + r; x = norm(r); h = mlp(x) + r
    (src/models/qwen3/qwen3.cpp:225-248)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    r = h
    x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    r = attention_block(x, w, p + "self_attn.", cfg, positions, window) + r
    x = rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    return swiglu_mlp(x, w, p + "mlp.") + r


def output_head(h, w, cfg) -> torch.Tensor:
    """Final RMSNorm, then logits against the head matrix
    (src/models/qwen3/qwen3.cpp:299-303).  Upstream always uses the embedding
    table as the head (qwen3.cpp:58); here `tie_word_embeddings` decides."""
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------
def forward(cfg: dict, weights: dict[str, torch.Tensor], ids, dtype=torch.float32) -> torch.Tensor:
    """Logits [S, V] at every position of one whole sequence
    (src/models/qwen3/qwen3.cpp:255-307)."""
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    h = embed(ids, w["model.embed_tokens.weight"])
    for i, window in enumerate(layer_windows(cfg)):
        h = decoder_layer(h, w, i, cfg, positions, window)
    return output_head(h, w, cfg)


def greedy(cfg, weights, prompt, n_new, stop_ids=(), dtype=torch.float32) -> list[int]:
    """Greedy continuation, the whole sequence run again for each new token
    (inference.cpp:137-168 without its cache); ties go to the lowest id."""
    ids = list(prompt)
    new = []
    for _ in range(n_new):
        logits = forward(cfg, weights, ids, dtype)[-1]
        tok = int(torch.argmax(logits))  # torch returns the first maximum
        new.append(tok)
        ids.append(tok)
        if tok in stop_ids:
            break
    return new
