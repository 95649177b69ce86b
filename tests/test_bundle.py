"""The on-disk bundle reader (inferrous_b200/bundle.py; format of the reference's tools/prepare.py and src/model.rs):
CPU checks of the format handling, and on a GPU a generation from a bundle through the Python and the C++ hosts."""
import json
import subprocess

import numpy as np
import pytest

from tests.bundle_writer import write_bundle


def test_bundle_tensors_round_trip_and_are_verified(tmp_path):
    from inferrous_b200.bundle import Bundle, BundleError

    manifest = write_bundle(tmp_path / "b", seed=3)
    b = Bundle(tmp_path / "b")
    assert (b.config.layers, b.config.hidden, b.config.q_heads, b.config.kv_heads) == (2, 256, 4, 2)
    assert (b.config.intermediate, b.config.vocab, b.config.context) == (512, 640, 64)
    w = b.tensor("layer.1.down.w", "|i1", (256, 512))
    assert w.dtype == np.int8 and np.abs(w).max() == 127
    assert b.tensor("rope", "<f4", (64, 128))[0, :64].tolist() == [1.0] * 64  # cos(0)
    with pytest.raises(BundleError, match="wrong type or shape"):
        b.tensor("layer.1.down.w", "|i1", (512, 256))
    with pytest.raises(BundleError, match="missing"):
        b.tensor("layer.2.down.w", "|i1", (256, 512))
    # a flipped byte is caught by the digest
    p = tmp_path / "b" / "final_gain.bin"
    raw = bytearray(p.read_bytes())
    raw[5] ^= 1
    p.write_bytes(bytes(raw))
    with pytest.raises(BundleError, match="hash mismatch"):
        b.tensor("final_gain", "<f4", (256,))
    assert Bundle(tmp_path / "b", verify_hashes=False).tensor("final_gain", "<f4", (256,)).shape == (256,)
    # unsupported operators and versions are refused like src/model.rs:50-77
    for key, value in [("hidden_act", "gelu"), ("head_dim", 64), ("tie_word_embeddings", True)]:
        bad = json.loads(json.dumps(manifest))
        bad["config"][key] = value
        (tmp_path / "b" / "manifest.json").write_text(json.dumps(bad))
        with pytest.raises(BundleError):
            Bundle(tmp_path / "b")
    bad = json.loads(json.dumps(manifest))
    bad["format_version"] = 2
    (tmp_path / "b" / "manifest.json").write_text(json.dumps(bad))
    with pytest.raises(BundleError, match="version"):
        Bundle(tmp_path / "b")


def test_invalid_weights_are_refused_at_load(tmp_path):
    """Model::load rejects the code -128 and non-positive scales (src/model.rs:143-145); so do both readers here."""
    import hashlib

    from inferrous_b200.bundle import Bundle, BundleError

    manifest = write_bundle(tmp_path / "b", seed=5)
    root = tmp_path / "b"

    def rewrite(name, mutate):
        path = root / f"{name}.bin"
        original = path.read_bytes()
        raw = bytearray(original)
        mutate(raw)
        path.write_bytes(bytes(raw))
        m = json.loads(json.dumps(manifest))
        m["tensors"][name]["sha256"] = hashlib.sha256(bytes(raw)).hexdigest()  # the digest is right: the VALUE is refused
        (root / "manifest.json").write_text(json.dumps(m))
        return path, original

    b = Bundle(root)
    assert b.weight("layer.0.o", 256, 512)[0].shape == (256, 512)
    path, original = rewrite("layer.0.o.w", lambda raw: raw.__setitem__(7, 0x80))
    with pytest.raises(BundleError, match="invalid quantized weight"):
        Bundle(root).weight("layer.0.o", 256, 512)
    path.write_bytes(original)
    for bits in (0.0, -1.0):
        path, original = rewrite("layer.1.gate.scale", lambda raw: raw.__setitem__(slice(8, 12), np.float32(bits).tobytes()))
        with pytest.raises(BundleError, match="invalid weight scale"):
            Bundle(root).weight("layer.1.gate", 512, 256)
        path.write_bytes(original)
    (root / "manifest.json").write_text(json.dumps(manifest))
    assert Bundle(root).weight("layer.1.gate", 512, 256)[1].min() > 0


def test_cpp_generation_program_compiles():
    from tests.cpp.build import build

    assert build("generate").exists()


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len,steps,shape", [
    (5, 8, dict()),
    (130, 6, dict(layers=2, hidden=512, q_heads=4, kv_heads=1, intermediate=1024, vocab=1024, context=192)),
])
def test_generation_from_a_bundle_python_cpp_and_cpu_agree(tmp_path, prompt_len, steps, shape):
    """The same bundle through three hosts: inferrous_b200.qwen3 (bf16 activations, concatenated gate|up, CUDA graph),
    the C++ harness (f32 carrier, separate gate and up, graph and eager) and the CPU restatement."""
    from inferrous_b200.bundle import load_bundle
    from inferrous_b200.qwen3 import Qwen3Runner
    from tests.cpp.build import build
    from tests.qwen3_oracle import OracleModel, export

    import os

    write_bundle(tmp_path / "b", seed=11, **shape)
    rng = np.random.default_rng(1)
    for head in ("bf16", "w8a8"):  # the reference's head (the default of both hosts) and the W8A8 head
        weights = load_bundle(tmp_path / "b", head=head)
        prompt = [int(t) for t in rng.integers(0, weights.config.vocab, prompt_len)]
        tokens, _ = Qwen3Runner(weights).generate(prompt, steps)
        # graph and eager; the decode step as one resident kernel (f32 carrier) and as one launch per operator
        for use_graph, resident in ((1, 1), (0, 1), (1, 0)):
            r = subprocess.run([str(build("generate")), str(tmp_path / "b"), str(steps), str(use_graph), *map(str, prompt)],
                               capture_output=True, text=True, timeout=600,
                               env=dict(os.environ, W8A8_HEAD=head, W8A8_RESIDENT_DECODE=str(resident)))
            assert r.returncode == 0, r.stdout + r.stderr
            assert [int(t) for t in r.stdout.split("tokens:")[1].split("\n")[0].split()] == tokens
            assert f"resident decode: {resident}" in r.stdout
        if prompt_len <= 16:
            assert OracleModel(export(weights)).generate(prompt, steps) == tokens


@pytest.mark.gpu
def test_generation_from_a_bundle_with_the_reference_head(tmp_path):
    """A bundle loads with its bf16 head by default, as the reference runs it (src/gpu.rs:801-811): tokens equal the CPU
    restatement's (bf16 head in the reference's summation order), fused selection equals stored logits + selection, and
    the W8A8 head remains available as an option."""
    from inferrous_b200.bundle import load_bundle
    from inferrous_b200.qwen3 import Qwen3Runner
    from tests.qwen3_oracle import OracleModel, export

    write_bundle(tmp_path / "b", seed=13)
    weights = load_bundle(tmp_path / "b")
    assert weights.head is None and weights.head_bf16 is not None
    prompt = [5, 17, 600, 3]
    tokens, _ = Qwen3Runner(weights).generate(prompt, 8)
    assert OracleModel(export(weights)).generate(prompt, 8) == tokens
    assert Qwen3Runner(weights, unfused=True).generate(prompt, 8)[0] == tokens
    assert Qwen3Runner(weights).generate(prompt, 8, use_graph=False)[0] == tokens
    both = load_bundle(tmp_path / "b", head="both")
    assert both.head is not None and Qwen3Runner(both).generate(prompt, 8)[0] == tokens  # the bf16 head wins when both exist
    with pytest.raises(ValueError):
        load_bundle(tmp_path / "b", head="fp8")
