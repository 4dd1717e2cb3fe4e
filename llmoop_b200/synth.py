"""Seeded synthetic source checkpoints in the layouts the NERVE compiler accepts.

The shapes and distributions stand in for public checkpoints (there is no
network): weights N(0, std) from `numpy.random.default_rng(seed)`, norm weights
1, BF16 storage; optional compressed-tensors INT4 (symmetric, group 128 along
K, bf16 scales; reference: nerve/model_transpiler_quantization.py:349-418) or
FP8 e4m3 with 128x128 block scales stored as `<name>_scale_inv` in BF16
(reference: nerve/model_transpiler_quantization.py:465-504).  MTP tensors live
under the `mtp.` prefix (reference: nerve/model_transpiler_types.py:257-274).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path

import numpy as np

from .safetensors_io import (
    bf16_bits_to_f32,
    f32_to_bf16_bits,
    f32_to_e4m3_bits,
    E4M3_TO_F32,
    write_safetensors,
)


@dataclass
class ModelSpec:
    name: str
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    max_positions: int = 256
    rope_theta: float = 10000.0
    eps: float = 1e-5
    quant: str = "bf16"  # bf16 | int4 | fp8
    mtp: bool = True
    tied: bool = False
    std: float = 0.02
    experts: int = 0
    experts_per_token: int = 0
    moe_ffn: int = 0
    qk_norm: bool = False
    seed: int = 0
    eos_token_id: int = 2

    def to_json(self) -> dict:
        return asdict(self)


def quantize_int4_group(weight_f32: np.ndarray, group: int = 128):
    """Returns (packed int32 [N, K/8], scale bf16 bits [N, K/group]).

    scale = bf16(absmax/7); q = clamp(rint(w/scale), -8, 7) + 8; nibble j of a
    word is column 8*w + j (low nibble first)."""
    n, k = weight_f32.shape
    assert k % group == 0 and k % 8 == 0
    grouped = weight_f32.reshape(n, k // group, group)
    absmax = np.abs(grouped).max(axis=2)
    scale_bits = f32_to_bf16_bits(np.maximum(absmax / 7.0, 1e-8).astype(np.float32))
    scale = bf16_bits_to_f32(scale_bits)
    q = np.clip(np.rint(grouped / scale[:, :, None]), -8, 7).astype(np.int32) + 8
    q = q.reshape(n, k // 8, 8).astype(np.uint32)
    packed = np.zeros((n, k // 8), dtype=np.uint32)
    for j in range(8):
        packed |= q[:, :, j] << np.uint32(4 * j)
    return packed.view(np.int32), scale_bits


def quantize_fp8_block(weight_f32: np.ndarray, block: int = 128):
    """Returns (e4m3 bits [N, K], scale_inv bf16 bits [ceil(N/block), K/block])."""
    n, k = weight_f32.shape
    assert k % block == 0
    rows = (n + block - 1) // block
    padded = np.zeros((rows * block, k), dtype=np.float32)
    padded[:n] = weight_f32
    tiles = padded.reshape(rows, block, k // block, block)
    absmax = np.abs(tiles).max(axis=(1, 3))
    scale_bits = f32_to_bf16_bits(np.maximum(absmax / 448.0, 1e-12).astype(np.float32))
    scale = bf16_bits_to_f32(scale_bits)
    q = f32_to_e4m3_bits((tiles / scale[:, None, :, None]).astype(np.float32))
    q = q.reshape(rows * block, k)[:n]
    return np.ascontiguousarray(q), scale_bits


def _normal(rng, shape, std):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def build_checkpoint(spec: ModelSpec):
    """Returns (config dict, tensors dict name -> (dtype, shape, array))."""
    rng = np.random.default_rng(spec.seed)
    tensors: dict = {}

    def put_bf16(name, values):
        tensors[name] = ("BF16", values.shape, f32_to_bf16_bits(values).reshape(values.shape))

    def put_linear(name, n, k, quantize=True):
        w = _normal(rng, (n, k), spec.std)
        if quantize and spec.quant == "int4":
            packed, scale = quantize_int4_group(w)
            tensors[name + ".weight_packed"] = ("I32", packed.shape, packed)
            tensors[name + ".weight_scale"] = ("BF16", scale.shape, scale)
            tensors[name + ".weight_shape"] = ("I64", (2,), np.array([n, k], dtype=np.int64))
        elif quantize and spec.quant == "fp8":
            q, scale = quantize_fp8_block(w)
            tensors[name + ".weight"] = ("F8_E4M3", q.shape, q)
            tensors[name + ".weight_scale_inv"] = ("BF16", scale.shape, scale)
        else:
            put_bf16(name + ".weight", w)

    def put_layer(prefix):
        h = spec.hidden
        put_bf16(prefix + ".input_layernorm.weight", np.ones(h, dtype=np.float32))
        put_bf16(prefix + ".post_attention_layernorm.weight", np.ones(h, dtype=np.float32))
        put_linear(prefix + ".self_attn.q_proj", spec.q_heads * spec.head_dim, h)
        put_linear(prefix + ".self_attn.k_proj", spec.kv_heads * spec.head_dim, h)
        put_linear(prefix + ".self_attn.v_proj", spec.kv_heads * spec.head_dim, h)
        put_linear(prefix + ".self_attn.o_proj", h, spec.q_heads * spec.head_dim)
        if spec.qk_norm:
            put_bf16(prefix + ".self_attn.q_norm.weight", np.ones(spec.head_dim, dtype=np.float32))
            put_bf16(prefix + ".self_attn.k_norm.weight", np.ones(spec.head_dim, dtype=np.float32))
        if spec.experts:
            put_bf16(prefix + ".mlp.gate.weight", _normal(rng, (spec.experts, h), spec.std))
            for e in range(spec.experts):
                put_linear(f"{prefix}.mlp.experts.{e}.gate_proj", spec.moe_ffn, h)
                put_linear(f"{prefix}.mlp.experts.{e}.up_proj", spec.moe_ffn, h)
                put_linear(f"{prefix}.mlp.experts.{e}.down_proj", h, spec.moe_ffn)
        else:
            put_linear(prefix + ".mlp.gate_proj", spec.ffn, h)
            put_linear(prefix + ".mlp.up_proj", spec.ffn, h)
            put_linear(prefix + ".mlp.down_proj", h, spec.ffn)

    put_bf16("model.embed_tokens.weight", _normal(rng, (spec.vocab, spec.hidden), spec.std))
    put_bf16("model.norm.weight", np.ones(spec.hidden, dtype=np.float32))
    if not spec.tied:
        put_bf16("lm_head.weight", _normal(rng, (spec.vocab, spec.hidden), spec.std))
    for layer in range(spec.layers):
        put_layer(f"model.layers.{layer}")
    if spec.mtp:
        put_bf16("mtp.fc.weight", _normal(rng, (spec.hidden, 2 * spec.hidden), spec.std))
        put_bf16("mtp.pre_fc_norm_embedding.weight", np.ones(spec.hidden, dtype=np.float32))
        put_bf16("mtp.pre_fc_norm_hidden.weight", np.ones(spec.hidden, dtype=np.float32))
        put_bf16("mtp.norm.weight", np.ones(spec.hidden, dtype=np.float32))
        put_layer("mtp.layers.0")

    config = {
        "architectures": ["SyntheticForCausalLM"],
        "model_type": "synthetic_" + spec.quant,
        "dtype": "bfloat16",
        "torch_dtype": "bfloat16",
        "hidden_size": spec.hidden,
        "intermediate_size": spec.ffn,
        "num_hidden_layers": spec.layers,
        "num_attention_heads": spec.q_heads,
        "num_key_value_heads": spec.kv_heads,
        "head_dim": spec.head_dim,
        "max_position_embeddings": spec.max_positions,
        "rms_norm_eps": spec.eps,
        "rope_theta": spec.rope_theta,
        "hidden_act": "silu",
        "vocab_size": spec.vocab,
        "bos_token_id": 1,
        "eos_token_id": spec.eos_token_id,
        "pad_token_id": 0,
        "tie_word_embeddings": bool(spec.tied),
    }
    if spec.experts:
        config.update(
            num_experts=spec.experts,
            num_experts_per_tok=spec.experts_per_token,
            moe_intermediate_size=spec.moe_ffn,
            norm_topk_prob=True,
        )
    if spec.quant == "int4":
        config["quantization_config"] = {
            "quant_method": "compressed-tensors",
            "format": "pack-quantized",
            "config_groups": {
                "group_0": {
                    "targets": ["Linear"],
                    "format": "pack-quantized",
                    "weights": {
                        "num_bits": 4,
                        "group_size": 128,
                        "symmetric": True,
                        "strategy": "group",
                        "type": "int",
                    },
                }
            },
        }
    elif spec.quant == "fp8":
        config["quantization_config"] = {
            "quant_method": "fp8",
            "fmt": "e4m3",
            "activation_scheme": "dynamic",
            "weight_block_size": [128, 128],
        }
    return config, tensors


def write_source_checkpoint(spec: ModelSpec, directory) -> None:
    """Writes config.json, generation_config.json, model.safetensors and a
    WordLevel tokenizer (same shape as the reference's tiny-model script,
    scripts/generate_tiny_test_model.py:102-123)."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    config, tensors = build_checkpoint(spec)
    (directory / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    (directory / "generation_config.json").write_text(
        json.dumps({"do_sample": False, "bos_token_id": 1, "eos_token_id": spec.eos_token_id, "pad_token_id": 0}, indent=2)
        + "\n"
    )
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt"})
    vocabulary = {"[PAD]": 0, "[BOS]": 1, "[EOS]": 2, "[UNK]": 3}
    vocabulary.update({f"token_{index:06d}": index for index in range(4, spec.vocab)})
    tokenizer = {
        "version": "1.0",
        "truncation": None,
        "padding": None,
        "added_tokens": [],
        "normalizer": None,
        "pre_tokenizer": {"type": "Whitespace"},
        "post_processor": None,
        "decoder": None,
        "model": {"type": "WordLevel", "vocab": vocabulary, "unk_token": "[UNK]"},
    }
    (directory / "tokenizer.json").write_text(json.dumps(tokenizer))
    (directory / "tokenizer_config.json").write_text(
        json.dumps({"bos_token": "[BOS]", "eos_token": "[EOS]", "pad_token": "[PAD]", "unk_token": "[UNK]"}, indent=2)
        + "\n"
    )


def iter_checkpoint_torch(spec: ModelSpec, device="cuda"):
    """Large-model variant of build_checkpoint: tensors are drawn and quantised with torch on `device` (seeded
    torch.Generator) and yielded one at a time as (name, dtype, shape, numpy array), so an 8B-parameter package
    streams to disk without ever being resident in host memory.  Same distributions and formats as the numpy
    builder; the random stream differs (torch Philox instead of numpy PCG64)."""
    import torch

    if spec.experts or spec.quant not in ("bf16", "int4"):
        raise ValueError("iter_checkpoint_torch covers dense BF16 and INT4 decoders")
    generator = torch.Generator(device=device)
    generator.manual_seed(spec.seed)

    def bf16_bits(values):
        bits = values.contiguous().view(torch.int32)
        lsb = (bits >> 16) & 1
        return (((bits + 0x7FFF + lsb) >> 16) & 0xFFFF).to(torch.int32)

    def to_u16(values_bits):
        return values_bits.to(torch.int16).cpu().numpy().view(np.uint16)

    def normal(shape):
        return torch.randn(shape, generator=generator, device=device, dtype=torch.float32) * spec.std

    def ones(name, width):
        return name, "BF16", (width,), f32_to_bf16_bits(np.ones(width, dtype=np.float32))

    def linear(name, n, k, quantize=True):
        w = normal((n, k))
        if quantize and spec.quant == "int4":
            grouped = w.view(n, k // 128, 128)
            absmax = grouped.abs().amax(dim=2)
            scale_bits = bf16_bits(torch.clamp(absmax / 7.0, min=1e-8))
            scale = (scale_bits << 16).view(torch.float32)
            q = torch.clamp(torch.round(grouped / scale[:, :, None]), -8, 7).to(torch.int32) + 8
            q = q.view(n, k // 8, 8)
            packed = torch.zeros((n, k // 8), dtype=torch.int32, device=device)
            for j in range(8):
                packed |= q[:, :, j] << (4 * j)
            yield name + ".weight_packed", "I32", (n, k // 8), packed.cpu().numpy()
            yield name + ".weight_scale", "BF16", (n, k // 128), to_u16(scale_bits)
        else:
            yield name + ".weight", "BF16", (n, k), to_u16(bf16_bits(w))

    def layer(prefix):
        h = spec.hidden
        yield ones(prefix + ".input_layernorm.weight", h)
        yield ones(prefix + ".post_attention_layernorm.weight", h)
        yield from linear(prefix + ".self_attn.q_proj", spec.q_heads * spec.head_dim, h)
        yield from linear(prefix + ".self_attn.k_proj", spec.kv_heads * spec.head_dim, h)
        yield from linear(prefix + ".self_attn.v_proj", spec.kv_heads * spec.head_dim, h)
        yield from linear(prefix + ".self_attn.o_proj", h, spec.q_heads * spec.head_dim)
        yield from linear(prefix + ".mlp.gate_proj", spec.ffn, h)
        yield from linear(prefix + ".mlp.up_proj", spec.ffn, h)
        yield from linear(prefix + ".mlp.down_proj", h, spec.ffn)

    yield from linear("model.embed_tokens", spec.vocab, spec.hidden, quantize=False)
    yield ones("model.norm.weight", spec.hidden)
    if not spec.tied:
        yield from linear("lm_head", spec.vocab, spec.hidden, quantize=False)
    for index in range(spec.layers):
        yield from layer(f"model.layers.{index}")
    if spec.mtp:
        yield from linear("mtp.fc", spec.hidden, 2 * spec.hidden, quantize=False)
        yield ones("mtp.pre_fc_norm_embedding.weight", spec.hidden)
        yield ones("mtp.pre_fc_norm_hidden.weight", spec.hidden)
        yield ones("mtp.norm.weight", spec.hidden)
        yield from layer("mtp.layers.0")


LLAMA3_8B_INT4 = dict(hidden=4096, layers=32, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                      rope_theta=500000.0, quant="int4", std=0.02, max_positions=34816)
