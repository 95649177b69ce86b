"""Writes a small synthetic model bundle in the reference's on-disk format (tools/prepare.py:47-52,56-92,109-114):
raw little-endian `<name>.bin` files and a `manifest.json` with shape, dtype and sha256 per tensor.  Test code only."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

from oracle import oracle


def write_bundle(path: Path, *, layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=640, context=64,
                 seed=0) -> dict:
    rng = np.random.default_rng(seed)
    path.mkdir(parents=True, exist_ok=True)
    tensors = {}

    def emit(name, a, dtype):
        a = np.ascontiguousarray(a, dtype=dtype)
        raw = a.tobytes()
        (path / f"{name}.bin").write_bytes(raw)
        tensors[name] = dict(shape=list(a.shape), dtype=dtype, sha256=hashlib.sha256(raw).hexdigest())

    def bf16_bits(shape, scale=1.0):
        return oracle.bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))

    def gain(n):
        return oracle.bf16((1 + 0.1 * rng.standard_normal(n)).astype(np.float32))

    emit("embedding", bf16_bits((vocab, hidden)), "<u2")
    emit("head", bf16_bits((vocab, hidden), 0.05), "<u2")
    emit("final_gain", gain(hidden), "<f4")
    widths = {"q": (q_heads * 128, hidden), "k": (kv_heads * 128, hidden), "v": (kv_heads * 128, hidden),
              "o": (hidden, q_heads * 128), "gate": (intermediate, hidden), "up": (intermediate, hidden),
              "down": (hidden, intermediate)}
    for l in range(layers):
        for short, n in [("norm1", hidden), ("norm2", hidden), ("qnorm", 128), ("knorm", 128)]:
            emit(f"layer.{l}.{short}", gain(n), "<f4")
        for short, (n, k) in widths.items():
            w = (rng.standard_normal((n, k)) * (1.0 / np.sqrt(k))).astype(np.float32)
            q, s = oracle.weight_quantize(w)  # tools/prepare.py:79-81
            emit(f"layer.{l}.{short}.w", q, "|i1")
            emit(f"layer.{l}.{short}.scale", s, "<f4")
    freq = 1.0 / (1e6 ** (np.arange(0, 128, 2, dtype=np.float32) / np.float32(128)))
    angles = np.arange(context, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]
    emit("rope", np.concatenate([np.cos(angles), np.sin(angles)], 1).astype(np.float32), "<f4")
    config = dict(hidden_size=hidden, intermediate_size=intermediate, num_hidden_layers=layers, num_attention_heads=q_heads,
                  num_key_value_heads=kv_heads, head_dim=128, vocab_size=vocab, rms_norm_eps=1e-6, rope_theta=1000000,
                  rope_scaling=None, attention_bias=False, use_sliding_window=False, tie_word_embeddings=False, hidden_act="silu")
    manifest = dict(format_version=1, profile="synthetic-test", model_revision="none", max_context=context, config=config,
                    tensors=tensors)
    (path / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    return manifest
