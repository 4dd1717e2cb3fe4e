#!/usr/bin/env python3
"""Generate the committed golden packages under tests/golden/packages/.

Runs the reference's own Python compiler (imported read-only from the
reference checkout given by --reference) on seeded synthetic source
checkpoints.  The only stage that cannot run without a graphics toolchain is
the GLSL -> SPIR-V step; it is replaced by a stub that writes a 5-word SPIR-V
header per shader (the CUDA backend never reads shader files, but they are
listed in the manifest's artifact_integrity table, so they stay in the
package).  Everything else - transpile, lowering, tensor repacking, manifest,
integrity, validation - is the reference's code, so these packages pin the
mounter against real compiler output.

Usage:  python tests/golden/make_packages.py --reference /path/to/reference
"""

from __future__ import annotations

import argparse
import json
import shutil
import struct
import sys
import tempfile
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from llmoop_b200.synth import ModelSpec, write_source_checkpoint  # noqa: E402

SPIRV_STUB = struct.pack("<5I", 0x07230203, 0x00010600, 0, 1, 0)

BF16_FEATURES = ("shader_bfloat16_type",)
FP8_FEATURES = (
    "shader_bfloat16_type",
    "shader_float8",
    "shader_mixed_float_dot_product_float8_acc_float32",
)

SPECS = [
    # BASELINE config 1: tiny Llama-style decoder + one MTP layer, BF16 storage.
    (ModelSpec(name="cfg1_bf16_mtp", hidden=64, layers=2, q_heads=4, kv_heads=2, head_dim=16, ffn=128,
               vocab=256, quant="bf16", std=0.02, seed=0), BF16_FEATURES),
    # Same shape class as config 2 (INT4 g128 + bf16 lm_head + MTP), scaled down; larger std so that
    # greedy decisions are well separated.
    (ModelSpec(name="tiny_int4_mtp", hidden=128, layers=2, q_heads=4, kv_heads=2, head_dim=32, ffn=256,
               vocab=256, quant="int4", std=0.08, seed=1), BF16_FEATURES),
    # Tiny vocabulary so that a random MTP head is accepted often (exercises partial acceptance).
    (ModelSpec(name="tiny_int4_mtp_v16", hidden=128, layers=1, q_heads=4, kv_heads=2, head_dim=32, ffn=128,
               vocab=16, quant="int4", std=0.08, seed=2), BF16_FEATURES),
    (ModelSpec(name="tiny_fp8_mtp", hidden=128, layers=2, q_heads=4, kv_heads=2, head_dim=32, ffn=256,
               vocab=256, quant="fp8", std=0.08, seed=3), FP8_FEATURES),
    (ModelSpec(name="tiny_moe_fp8_mtp", hidden=128, layers=2, q_heads=4, kv_heads=2, head_dim=32, ffn=128,
               vocab=256, quant="fp8", std=0.08, seed=4, experts=8, experts_per_token=2, moe_ffn=128,
               qk_norm=True), FP8_FEATURES),
]


def install_spirv_stub():
    import nerve.model_package_manifest as manifest_module

    def stub(shader_dir, *, progress=None, cancel_requested=None):
        for source in sorted(Path(shader_dir).glob("*.comp")):
            source.with_suffix(".spv").write_bytes(SPIRV_STUB)
            source.unlink()

    manifest_module.compile_shader_artifacts = stub
    try:
        import nerve.model_package as package_module

        if hasattr(package_module, "compile_shader_artifacts"):
            package_module.compile_shader_artifacts = stub
    except ImportError:
        pass


def compile_one(reference: Path, spec: ModelSpec, features, destination: Path) -> None:
    from nerve.compiler_target import CompilerTarget
    from nerve.model_compiler import compile_model

    with tempfile.TemporaryDirectory(prefix="golden-src-") as temporary:
        source = Path(temporary) / "source"
        write_source_checkpoint(spec, source)
        shutil.rmtree(destination, ignore_errors=True)
        compile_model(
            source,
            compiled_model_dir=destination,
            shader_source_dir=reference / "runtime-rs" / "shaders",
            target=CompilerTarget.for_features(features),
        )
    (destination / "synthetic_spec.json").write_text(json.dumps(spec.to_json(), indent=2) + "\n")


def compile_reference_fixture(reference: Path, destination: Path) -> None:
    """The reference's own tiny test model (scripts/generate_tiny_test_model.py:28-99: 1 layer, hidden 16, 2 q /
    1 kv heads, head 8, FFN 32, vocab 32, BF16 values ((i mod 29) - 14) / 29, tied lm_head, no MTP), rebuilt from
    the formula so that the result can be compared with the package checked into the reference."""
    import numpy as np

    from llmoop_b200.safetensors_io import f32_to_bf16_bits, write_safetensors
    from nerve.compiler_target import CompilerTarget
    from nerve.model_compiler import compile_model

    def tensor(shape, offset):
        count = int(np.prod(shape))
        values = np.arange(offset, offset + count, dtype=np.float32)
        values = ((np.remainder(values, 29) - 14) / np.float32(29)).astype(np.float32)
        return ("BF16", shape, f32_to_bf16_bits(values).reshape(shape))

    ones = lambda n: ("BF16", (n,), f32_to_bf16_bits(np.ones(n, dtype=np.float32)))
    tensors = {
        "model.embed_tokens.weight": tensor((32, 16), 0), "model.norm.weight": ones(16),
        "model.layers.0.input_layernorm.weight": ones(16), "model.layers.0.post_attention_layernorm.weight": ones(16),
        "model.layers.0.self_attn.q_proj.weight": tensor((16, 16), 512), "model.layers.0.self_attn.k_proj.weight": tensor((8, 16), 768),
        "model.layers.0.self_attn.v_proj.weight": tensor((8, 16), 896), "model.layers.0.self_attn.o_proj.weight": tensor((16, 16), 1024),
        "model.layers.0.mlp.gate_proj.weight": tensor((32, 16), 1280), "model.layers.0.mlp.up_proj.weight": tensor((32, 16), 1792),
        "model.layers.0.mlp.down_proj.weight": tensor((16, 32), 2304),
    }
    config = {
        "architectures": ["TinyTestForCausalLM"], "model_type": "tiny_test", "dtype": "bfloat16", "torch_dtype": "bfloat16",
        "hidden_size": 16, "intermediate_size": 32, "num_hidden_layers": 1, "num_attention_heads": 2, "num_key_value_heads": 1,
        "head_dim": 8, "max_position_embeddings": 64, "rms_norm_eps": 1e-5, "rope_theta": 10_000.0, "hidden_act": "silu",
        "vocab_size": 32, "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0, "layer_types": ["full_attention"],
    }
    with tempfile.TemporaryDirectory(prefix="golden-src-") as temporary:
        source = Path(temporary) / "source"
        source.mkdir()
        (source / "config.json").write_text(json.dumps(config, indent=2) + "\n")
        (source / "generation_config.json").write_text(json.dumps({"do_sample": False, "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0}, indent=2) + "\n")
        write_safetensors(source / "model.safetensors", tensors, metadata={"format": "pt"})
        vocabulary = {"[PAD]": 0, "[BOS]": 1, "[EOS]": 2, "[UNK]": 3, **{f"token_{index:02d}": index for index in range(4, 32)}}
        (source / "tokenizer.json").write_text(json.dumps({
            "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
            "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
            "model": {"type": "WordLevel", "vocab": vocabulary, "unk_token": "[UNK]"}}))
        (source / "tokenizer_config.json").write_text(json.dumps({"bos_token": "[BOS]", "eos_token": "[EOS]", "pad_token": "[PAD]", "unk_token": "[UNK]"}, indent=2) + "\n")
        shutil.rmtree(destination, ignore_errors=True)
        compile_model(source, compiled_model_dir=destination, shader_source_dir=reference / "runtime-rs" / "shaders",
                      target=CompilerTarget.for_features(BF16_FEATURES))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--out", type=Path, default=REPO / "tests" / "golden" / "packages")
    parser.add_argument("--only", default=None)
    args = parser.parse_args()
    sys.path.insert(0, str(args.reference))
    install_spirv_stub()
    args.out.mkdir(parents=True, exist_ok=True)
    for spec, features in SPECS:
        if args.only and spec.name != args.only:
            continue
        compile_one(args.reference, spec, features, args.out / spec.name)
        print("compiled", spec.name)
    if not args.only or args.only == "reference_tiny_model":
        compile_reference_fixture(args.reference, args.out / "reference_tiny_model")
        print("compiled reference_tiny_model")


if __name__ == "__main__":
    main()
