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


if __name__ == "__main__":
    main()
