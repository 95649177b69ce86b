"""Reader for the reference's on-disk model bundle: `manifest.json` plus one raw little-endian `<name>.bin` per tensor.

Format as written by crates/inferrous-qwen3/tools/prepare.py:47-52,56-92,109-114 and read by `Model::load`
(src/model.rs:46-165):
    embedding, head              <u2  [vocab, hidden]         bf16 bit patterns
    final_gain                   <f4  [hidden]
    layer.L.{norm1,norm2}        <f4  [hidden]
    layer.L.{qnorm,knorm}        <f4  [128]
    layer.L.{q,k,v,o,gate,up,down}.w      |i1  [N, K]         per-output-channel symmetric int8
    layer.L.{q,k,v,o,gate,up,down}.scale  <f4  [N]
    rope                         <f4  [context, 128]          64 cosines then 64 sines per position
Every tensor's shape, dtype and sha256 are checked against the manifest, as the reference does.  Unlike the reference's
loader, which accepts the Qwen3-8B dimensions only, the dimensions are taken from the manifest's `config` (head width
128 and the operator set are still required), so that small bundles can be used in tests.

What this loader does beyond copying: Q, K, V (and gate, up) are concatenated along the output dimension and the gains
of the hidden-width norms are converted to the activation dtype (they are bf16 values in the checkpoint).  The head stays
bf16, as the reference runs it (`head="bf16"`, the default); `head="w8a8"` instead quantizes it per output channel with
the formula the bundle's other matrices were quantized with (tools/prepare.py:79-81) -- the benchmark's W8A8 lm_head,
whose logits differ from the reference's.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import torch

from .qwen3 import Layer, Qwen3Config, Qwen3Weights

FORMAT_VERSION = 1
_DTYPES = {"|i1": np.int8, "<u2": np.uint16, "<f4": np.float32}


class BundleError(ValueError):
    pass


def config_from_manifest(manifest: dict) -> Qwen3Config:
    c = manifest["config"]
    if c.get("head_dim") != 128:
        raise BundleError("unsupported head_dim (the kernels are written for 128)")
    if not (c.get("rms_norm_eps") == 1e-6 and c.get("rope_scaling") is None and c.get("attention_bias") is False
            and c.get("tie_word_embeddings") is False and c.get("hidden_act") == "silu"):
        raise BundleError("unsupported model operators")  # the checks of src/model.rs:65-77
    return Qwen3Config(layers=c["num_hidden_layers"], hidden=c["hidden_size"], q_heads=c["num_attention_heads"],
                       kv_heads=c["num_key_value_heads"], intermediate=c["intermediate_size"], vocab=c["vocab_size"],
                       context=manifest["max_context"], rope_theta=float(c["rope_theta"]))


class Bundle:
    def __init__(self, path, verify_hashes: bool = True):
        self.path = Path(path)
        self.manifest = json.loads((self.path / "manifest.json").read_text())
        if self.manifest.get("format_version") != FORMAT_VERSION:
            raise BundleError("unsupported bundle format version")
        self.config = config_from_manifest(self.manifest)
        self.verify_hashes = verify_hashes

    def tensor(self, name: str, dtype: str, shape) -> np.ndarray:
        meta = self.manifest["tensors"].get(name)
        if meta is None:
            raise BundleError(f"missing {name}")
        if meta["dtype"] != dtype or list(meta["shape"]) != list(shape):
            raise BundleError(f"{name}: wrong type or shape")
        raw = (self.path / f"{name}.bin").read_bytes()
        if len(raw) != int(np.prod(shape)) * np.dtype(_DTYPES[dtype]).itemsize:
            raise BundleError(f"{name}: size mismatch")
        if self.verify_hashes and hashlib.sha256(raw).hexdigest() != meta["sha256"]:
            raise BundleError(f"{name}: hash mismatch")
        a = np.frombuffer(raw, dtype=_DTYPES[dtype]).reshape(shape)
        if dtype == "<f4" and not np.isfinite(a).all():
            raise BundleError(f"{name}: nonfinite float")
        return a

    def weight(self, name: str, n: int, k: int):
        """An int8 matrix and its per-channel scales as Model::load admits them (src/model.rs:143-145): symmetric
        quantization never produces the code -128, and a scale must be positive."""
        w = self.tensor(f"{name}.w", "|i1", (n, k))
        if (w == -128).any():
            raise BundleError(f"{name}.w: invalid quantized weight")
        scale = self.tensor(f"{name}.scale", "<f4", (n,))
        if not (scale > 0).all():
            raise BundleError(f"{name}.scale: invalid weight scale")
        return w, scale


def quantize_rows(w: torch.Tensor):
    """Per-output-channel symmetric int8 (tools/prepare.py:79-81): scale = max(|row|, 1e-8) / 127, q = rne(w / scale)."""
    w = w.float()
    scale = w.abs().amax(1, keepdim=True).clamp(min=1e-8) / 127.0
    q = torch.round(w / scale).clamp(-127, 127).to(torch.int8)
    return q, scale.flatten().contiguous()


def load_bundle(path, device="cuda", verify_hashes: bool = True, head: str = "bf16") -> Qwen3Weights:
    if head not in ("bf16", "w8a8", "both"):
        raise ValueError("head must be 'bf16', 'w8a8' or 'both'")
    b = Bundle(path, verify_hashes)
    c = b.config
    act = torch.bfloat16

    def dev(a, dtype=None):
        t = torch.from_numpy(np.array(a)).to(device)  # np.array: a writable copy of the read-only file view
        return t if dtype is None else t.to(dtype)

    def bf16(a):
        return torch.from_numpy(np.array(a).view(np.int16)).to(device).view(torch.bfloat16)

    shapes = {"q": (c.q_width, c.hidden), "k": (c.kv_heads * 128, c.hidden), "v": (c.kv_heads * 128, c.hidden),
              "o": (c.hidden, c.q_width), "gate": (c.intermediate, c.hidden), "up": (c.intermediate, c.hidden),
              "down": (c.hidden, c.intermediate)}

    def matrix(layer, names):
        pairs = [b.weight(f"layer.{layer}.{n}", *shapes[n]) for n in names]
        return torch.cat([dev(w) for w, _ in pairs]).contiguous(), torch.cat([dev(s) for _, s in pairs]).contiguous()

    layers = []
    for l in range(c.layers):
        gain = lambda n, width: b.tensor(f"layer.{l}.{n}", "<f4", (width,))
        qkv, qkv_s = matrix(l, ["q", "k", "v"])
        o, o_s = matrix(l, ["o"])
        gate_up, gate_up_s = matrix(l, ["gate", "up"])
        down, down_s = matrix(l, ["down"])
        layers.append(Layer(c, dev(gain("norm1", c.hidden), act), qkv, qkv_s, dev(gain("qnorm", 128)), dev(gain("knorm", 128)),
                            o, o_s, dev(gain("norm2", c.hidden), act), gate_up, gate_up_s, down, down_s))
    embedding = bf16(b.tensor("embedding", "<u2", (c.vocab, c.hidden)))
    head_bits = bf16(b.tensor("head", "<u2", (c.vocab, c.hidden)))
    head_q, head_s = quantize_rows(head_bits) if head in ("w8a8", "both") else (None, None)
    weights = Qwen3Weights(c, embedding, layers, dev(b.tensor("final_gain", "<f4", (c.hidden,)), act), head_q, head_s, device,
                           head_bf16=head_bits.contiguous() if head in ("bf16", "both") else None)
    weights.rope = dev(b.tensor("rope", "<f4", (c.context, 128)))  # the bundle's table, not a recomputed one
    return weights
