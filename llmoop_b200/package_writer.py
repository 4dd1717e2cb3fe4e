"""Native writer for compiled packages of Llama-style decoders (+ one MTP
layer; dense BF16 / INT4 / FP8, or FP8 with sparse experts and per-head q/k
norms) in the schema the reference compiler emits
(nerve.vulkan_resident_model_package.v3 / nerve.tensor_index.v1 /
nerve.stream_circuit.v1), without importing the reference.

Scope: the fields the runtime contract needs - circuit graph with fused
`nodes` and `semantic_execution_nodes`, params refs, `component_executions`
kernel lists (op, node_id, source_node_ids), transducer and sampler specs,
`speculative_decoders`, tensor index with per-tensor SHA-256, weights as one
safetensors file per tensor named tensor_<blake2s-8(name)>.safetensors, and
the artifact_integrity table over every JSON artifact written.  Shader
artifacts are not produced (a CUDA backend has no use for SPIR-V), so the
kernels carry no shader_path.  tests/test_package_writer.py checks the output
field by field against packages compiled by the reference compiler from the
same synthetic checkpoints.

Kernel lists follow nerve/circuit_optimizer.py: BF16 weights fuse q/k/v into
parallel_linear_3way, o/down into linear_residual and gate/up/SiLU/multiply
into parallel_linear_silu_multiply; INT4 weights stay as separate linear,
residual_add and silu_multiply kernels.  FP8 (e4m3, block-scaled) weights fuse
like BF16 ones where the branches' scale grids imply the same block shape
(nerve/model_package_tensors.py:618-660, 1278-1323) - else q stays a linear of
its own and k/v become parallel_linear_2way - and every consumer of an
activation reads it through one quantize_fp8_e4m3 node per (signal, width)
(nerve/circuit_optimizer.py:150-250).  Sparse-expert layers keep the router
as a BF16 linear, route with moe_topk and run sparse_moe_gate_up /
sparse_moe_down / moe_reduce on expert tensors packed [expert, row, column]
(nerve/model_transpiler_quantization.py:22-250); per-head q/k norms fuse with
the rotary embedding into parallel_head_norm_rope_2way.
"""

from __future__ import annotations

import hashlib
import json
import math
import re
from pathlib import Path

import numpy as np

from .safetensors_io import DTYPE_BYTES, write_safetensors
from .synth import ModelSpec, build_checkpoint


def _tensor_file(name: str) -> str:
    return "weights/tensor_" + hashlib.blake2s(name.encode("utf-8"), digest_size=8).hexdigest() + ".safetensors"


def _dump(path: Path, value) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(value, indent=2) + "\n")


def _attention_attrs(spec: ModelSpec) -> dict:
    return {
        "query_heads": spec.q_heads, "key_value_heads": spec.kv_heads, "head_width": spec.head_dim,
        "query_groups_per_kv_head": spec.q_heads // spec.kv_heads,
    }


def _layer_circuit(spec: ModelSpec, component_id: str, prefix: str, layer_index, quant: str):
    """Returns (component dict, execution dict) of one full-attention layer."""
    h, ffn = spec.hidden, spec.ffn
    att = _attention_attrs(spec)
    norm_attrs = {"eps": spec.eps, "weight_offset": 0.0}
    rope = {"position_source": "stream_tick", "theta": float(spec.rope_theta), "rope_type": "default", "scaling": None,
            "interleaved": False, "rotary_width": spec.head_dim, **att}
    refs = {
        "operator_norm": {"tensor": f"{prefix}.input_layernorm.weight", "role": "operator_normalization_weight"},
        "ffn_norm": {"tensor": f"{prefix}.post_attention_layernorm.weight", "role": "feed_forward_normalization_weight"},
    }
    if quant == "fp8":
        return _fp8_layer_circuit(spec, component_id, prefix, layer_index)
    suffix = ".weight_packed" if quant == "int4" else ".weight"
    for ref, tensor, role in (
        ("ffn_gate", "mlp.gate_proj", "feed_forward_swiglu_gate_projection"),
        ("ffn_down", "mlp.down_proj", "feed_forward_down_projection"),
        ("ffn_up", "mlp.up_proj", "feed_forward_up_projection"),
        ("q_projection", "self_attn.q_proj", "attention_query_projection"),
        ("k_projection", "self_attn.k_proj", "attention_key_projection"),
        ("v_projection", "self_attn.v_proj", "attention_value_projection"),
        ("attention_out_projection", "self_attn.o_proj", "attention_output_projection"),
    ):
        refs[ref] = {"tensor": f"{prefix}.{tensor}{suffix}", "role": role}
    if quant == "int4":
        for ref, tensor, role in (
            ("ffn_gate", "mlp.gate_proj", "feed_forward_swiglu_gate_projection"),
            ("ffn_down", "mlp.down_proj", "feed_forward_down_projection"),
            ("ffn_up", "mlp.up_proj", "feed_forward_up_projection"),
            ("q_projection", "self_attn.q_proj", "attention_query_projection"),
            ("k_projection", "self_attn.k_proj", "attention_key_projection"),
            ("v_projection", "self_attn.v_proj", "attention_value_projection"),
            ("attention_out_projection", "self_attn.o_proj", "attention_output_projection"),
        ):
            refs[ref + "_scales"] = {"tensor": f"{prefix}.{tensor}.weight_scale", "role": role + "_group_scales"}

    def linear_params(ref):
        return [ref, ref + "_scales"] if quant == "int4" else [ref]

    semantic = [
        {"id": "operator_norm", "op": "rms_norm", "inputs": ["input_frame"], "outputs": ["operator_norm_out"],
         "params": ["operator_norm"], "attrs": dict(norm_attrs)},
        {"id": "q_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["q_projected"],
         "params": linear_params("q_projection")},
        {"id": "k_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["k_projected"],
         "params": linear_params("k_projection")},
        {"id": "v_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["v_projected"],
         "params": linear_params("v_projection")},
        {"id": "q_rope", "op": "rotary_position_embedding", "inputs": ["q_projected"], "outputs": ["q_positioned"],
         "attrs": {**rope, "head_count": spec.q_heads}},
        {"id": "k_rope", "op": "rotary_position_embedding", "inputs": ["k_projected"], "outputs": ["k_positioned"],
         "attrs": {**rope, "head_count": spec.kv_heads}},
        {"id": "kv_memory_append", "op": "append_state_update", "inputs": ["k_positioned", "v_projected", "kv_memory"],
         "outputs": ["k_memory", "v_memory"], "state_reads": ["kv_memory"], "state_writes": ["kv_memory"],
         "attrs": {"growth": "per_activation", **att}},
        {"id": "attention_read", "op": "scaled_dot_product_attention", "inputs": ["q_positioned", "k_memory", "v_memory"],
         "outputs": ["attention_out"], "params": [],
         "attrs": {"causal": True, "scale": spec.head_dim ** -0.5, "window_size": None, "attention_sinks": False, **att}},
        {"id": "attention_out_projection", "op": "linear", "inputs": ["attention_out"], "outputs": ["operator_out"],
         "params": linear_params("attention_out_projection")},
        {"id": "operator_residual", "op": "residual_add", "inputs": ["input_frame", "operator_out"],
         "outputs": ["operator_residual_out"]},
        {"id": "ffn_norm", "op": "rms_norm", "inputs": ["operator_residual_out"], "outputs": ["ffn_norm_out"],
         "params": ["ffn_norm"], "attrs": dict(norm_attrs)},
        {"id": "ffn_gate_projection", "op": "linear", "inputs": ["ffn_norm_out"], "outputs": ["ffn_gate"],
         "params": linear_params("ffn_gate")},
        {"id": "ffn_up_projection", "op": "linear", "inputs": ["ffn_norm_out"], "outputs": ["ffn_up"],
         "params": linear_params("ffn_up")},
        {"id": "ffn_gate_activation", "op": "silu", "inputs": ["ffn_gate"], "outputs": ["ffn_gate_activated"],
         "attrs": {"element_count": ffn}},
        {"id": "ffn_gate_multiply", "op": "multiply", "inputs": ["ffn_gate_activated", "ffn_up"], "outputs": ["ffn_hidden"]},
        {"id": "ffn_down_projection", "op": "linear", "inputs": ["ffn_hidden"], "outputs": ["ffn_out"],
         "params": linear_params("ffn_down")},
        {"id": "ffn_residual", "op": "residual_add", "inputs": ["operator_residual_out", "ffn_out"], "outputs": ["output_frame"]},
    ]
    by_id = {node["id"]: node for node in semantic}
    eb = {"output_element_bytes": [2]}
    attention_node = {
        "id": "kv_memory_append__attention_read", "op": "append_scaled_dot_product_attention",
        "inputs": ["q_positioned", "k_positioned", "v_projected", "kv_memory"], "outputs": ["attention_out"], "params": [],
        "state_reads": ["kv_memory"], "state_writes": ["kv_memory"],
        "attrs": {"compiled_from": ["kv_memory_append", "attention_read"], "append": by_id["kv_memory_append"]["attrs"],
                  "attention": by_id["attention_read"]["attrs"], "current_kv_source": "direct_bf16_input", **eb},
    }

    def plain(node_id):
        node = dict(by_id[node_id])
        node["attrs"] = {**node.get("attrs", {}), **eb}
        return node

    if quant == "int4":
        fused = [
            plain("operator_norm"), plain("q_projection"), plain("k_projection"), plain("v_projection"), plain("q_rope"),
            plain("k_rope"), attention_node, plain("attention_out_projection"), plain("operator_residual"), plain("ffn_norm"),
            plain("ffn_gate_projection"), plain("ffn_up_projection"),
            {"id": "ffn_gate_activation__ffn_gate_multiply", "op": "silu_multiply", "inputs": ["ffn_gate", "ffn_up"],
             "outputs": ["ffn_hidden"],
             "attrs": {"compiled_from": ["ffn_gate_activation", "ffn_gate_multiply"], "intermediate_rounding": "BF16",
                       "element_count": ffn, **eb}},
            plain("ffn_down_projection"), plain("ffn_residual"),
        ]
        kernels = [
            ("rms_norm", "operator_norm", ["operator_norm"]), ("linear", "q_projection", ["q_projection"]),
            ("linear", "k_projection", ["k_projection"]), ("linear", "v_projection", ["v_projection"]),
            ("rotary_position_embedding", "q_rope", ["q_rope"]), ("rotary_position_embedding", "k_rope", ["k_rope"]),
            ("append_scaled_dot_product_attention", "kv_memory_append__attention_read", ["kv_memory_append", "attention_read"]),
            ("linear", "attention_out_projection", ["attention_out_projection"]),
            ("residual_add", "operator_residual", ["operator_residual"]), ("rms_norm", "ffn_norm", ["ffn_norm"]),
            ("linear", "ffn_gate_projection", ["ffn_gate_projection"]), ("linear", "ffn_up_projection", ["ffn_up_projection"]),
            ("silu_multiply", "ffn_gate_activation__ffn_gate_multiply", ["ffn_gate_activation", "ffn_gate_multiply"]),
            ("linear", "ffn_down_projection", ["ffn_down_projection"]), ("residual_add", "ffn_residual", ["ffn_residual"]),
        ]
    else:
        fused = [
            plain("operator_norm"),
            {"id": "q_projection__k_projection__v_projection", "op": "parallel_linear_3way", "inputs": ["operator_norm_out"],
             "outputs": ["q_projected", "k_projected", "v_projected"], "params": ["q_projection", "k_projection", "v_projection"],
             "attrs": {"compiled_from": ["q_projection", "k_projection", "v_projection"], "branch_count": 3,
                       "output_element_bytes": [2, 2, 2]}},
            plain("q_rope"), plain("k_rope"), attention_node,
            {"id": "attention_out_projection__operator_residual", "op": "linear_residual", "inputs": ["attention_out", "input_frame"],
             "outputs": ["operator_residual_out"], "params": ["attention_out_projection"],
             "attrs": {"compiled_from": ["attention_out_projection", "operator_residual"], "intermediate_rounding": "BF16", **eb}},
            plain("ffn_norm"),
            {"id": "ffn_gate_projection__ffn_up_projection__ffn_gate_activation__ffn_gate_multiply",
             "op": "parallel_linear_silu_multiply", "inputs": ["ffn_norm_out"], "outputs": ["ffn_hidden"],
             "params": ["ffn_gate", "ffn_up"],
             "attrs": {"compiled_from": ["ffn_gate_projection", "ffn_up_projection", "ffn_gate_activation", "ffn_gate_multiply"],
                       "branch_count": 2, "intermediate_rounding": "BF16", "element_count": ffn, **eb}},
            {"id": "ffn_down_projection__ffn_residual", "op": "linear_residual", "inputs": ["ffn_hidden", "operator_residual_out"],
             "outputs": ["output_frame"], "params": ["ffn_down"],
             "attrs": {"compiled_from": ["ffn_down_projection", "ffn_residual"], "intermediate_rounding": "BF16", **eb}},
        ]
        kernels = [
            ("rms_norm", "operator_norm", ["operator_norm"]),
            ("parallel_linear_3way", "q_projection__k_projection__v_projection", ["q_projection", "k_projection", "v_projection"]),
            ("rotary_position_embedding", "q_rope", ["q_rope"]), ("rotary_position_embedding", "k_rope", ["k_rope"]),
            ("append_scaled_dot_product_attention", "kv_memory_append__attention_read", ["kv_memory_append", "attention_read"]),
            ("linear_residual", "attention_out_projection__operator_residual", ["attention_out_projection", "operator_residual"]),
            ("rms_norm", "ffn_norm", ["ffn_norm"]),
            ("parallel_linear_silu_multiply", "ffn_gate_projection__ffn_up_projection__ffn_gate_activation__ffn_gate_multiply",
             ["ffn_gate_projection", "ffn_up_projection", "ffn_gate_activation", "ffn_gate_multiply"]),
            ("linear_residual", "ffn_down_projection__ffn_residual", ["ffn_down_projection", "ffn_residual"]),
        ]

    return _layer_component(spec, component_id, layer_index, refs, semantic, fused, kernels)


def _layer_component(spec: ModelSpec, component_id: str, layer_index, refs, semantic, fused, kernels,
                     layout: str = "gqa_attention_layer_params_v1_dense_swiglu"):
    h = spec.hidden
    state_port = {
        "id": "kv_memory", "type": "append_only_attention_memory", "query_heads": spec.q_heads,
        "key_shape_per_token": [spec.kv_heads, spec.head_dim], "value_shape_per_token": [spec.kv_heads, spec.head_dim],
        "dtype": "BF16", "growth": "per_activation", "max_dynamic_activations": None,
        "sharing": "per_stream_per_node_instance", "owner": "stream", "layout": "append_only_kv",
        "source_layout": "batch_kvheads_seq_headdim",
    }
    circuit_id = f"{component_id}_gqa_attention_circuit_v1"
    params = {"schema": "nerve.circuit_params.v1", "circuit": circuit_id, "layout": layout, "storage": "source_tensor_refs", "refs": refs}
    circuit = {
        "schema": "nerve.stream_circuit.v1", "id": circuit_id,
        "source": {"component_id": component_id, "source_layer_index": layer_index, "source_operator_type": "full_attention"},
        "runtime_role": "signal_processor", "behavioral_role": "source_reference_circuit",
        "implementation": "reference_gqa_attention_layer_circuit_v1",
        "boundary": {"inputs": [{"id": "input_frame", "signal": "frame", "shape": [h], "component_port": "input"}],
                     "outputs": [{"id": "output_frame", "signal": "frame", "shape": [h], "source": "output_frame",
                                  "component_port": "output"}], "controls": []},
        "state_ports": [state_port],
        "parameters": {"layout": params["layout"], "storage": params["storage"], "refs": refs},
        "semantic_execution_nodes": semantic, "nodes": fused,
    }
    component = {
        "component_id": component_id, "operator_type": "full_attention", "runtime_role": "signal_processor",
        "implementation": "reference_gqa_attention_layer_circuit_v1", "behavioral_role": "source_reference_circuit",
        "circuit": circuit, "params": params,
        "state": {"schema": "nerve.circuit_state.v1", "circuit": circuit_id, "state_ports": [state_port]},
    }
    execution = {
        "component_id": component_id, "operator_type": "full_attention",
        "implementation": "reference_gqa_attention_layer_circuit_v1",
        "kernels": [{"execution_index": index, "node_id": node_id, "op": op, "source_node_ids": sources,
                     "execution_domain": "decode"} for index, (op, node_id, sources) in enumerate(kernels)],
    }
    return component, execution


FP8_CONTRACT = "bf16_blockwise_fp8_e4m3_f32_scale.v1"


def _fp8_block_shape(rows: int, columns: int, block: int = 128):
    """The block shape the reference infers from a weight's scale grid (nerve/model_package_tensors.py:1302-1303);
    the grid itself is ceil(dim / 128) per side (synth.quantize_fp8_block)."""
    grid = (-(-rows // block), -(-columns // block))
    return (-(-rows // grid[0]), -(-columns // grid[1]))


def _fp8_layer_circuit(spec: ModelSpec, component_id: str, prefix: str, layer_index):
    """One full-attention layer with e4m3 block-scaled linears, as the reference compiler lowers it."""
    h, ffn = spec.hidden, spec.ffn
    q_width, kv_width = spec.q_heads * spec.head_dim, spec.kv_heads * spec.head_dim
    att = _attention_attrs(spec)
    norm_attrs = {"eps": spec.eps, "weight_offset": 0.0}
    rope = {"position_source": "stream_tick", "theta": float(spec.rope_theta), "rope_type": "default", "scaling": None,
            "interleaved": False, "rotary_width": spec.head_dim, **att}
    linears = (
        ("ffn_gate", "mlp.gate_proj", "feed_forward_swiglu_gate_projection"),
        ("ffn_down", "mlp.down_proj", "feed_forward_down_projection"),
        ("ffn_up", "mlp.up_proj", "feed_forward_up_projection"),
        ("q_projection", "self_attn.q_proj", "attention_query_projection"),
        ("k_projection", "self_attn.k_proj", "attention_key_projection"),
        ("v_projection", "self_attn.v_proj", "attention_value_projection"),
        ("attention_out_projection", "self_attn.o_proj", "attention_output_projection"),
    )
    refs = {
        "operator_norm": {"tensor": f"{prefix}.input_layernorm.weight", "role": "operator_normalization_weight"},
        "ffn_norm": {"tensor": f"{prefix}.post_attention_layernorm.weight", "role": "feed_forward_normalization_weight"},
    }
    moe = bool(spec.experts)
    if moe:
        linears = tuple(entry for entry in linears if not entry[0].startswith("ffn_"))
        refs["moe_input"] = {"tensor": f"{prefix}.mlp.experts.gate_up_proj", "role": "mixture_of_experts_gate_up_weights"}
        refs["moe_output"] = {"tensor": f"{prefix}.mlp.experts.down_proj", "role": "mixture_of_experts_down_weights"}
        refs["moe_router"] = {"tensor": f"{prefix}.mlp.gate.weight", "role": "mixture_of_experts_router_projection"}
    for ref, tensor, role in linears:
        refs[ref] = {"tensor": f"{prefix}.{tensor}.weight", "role": role}
    if spec.qk_norm:
        refs["q_norm"] = {"tensor": f"{prefix}.self_attn.q_norm.weight", "role": "attention_query_head_normalization"}
        refs["k_norm"] = {"tensor": f"{prefix}.self_attn.k_norm.weight", "role": "attention_key_head_normalization"}
    if moe:
        refs["moe_input_scale_inv"] = {"tensor": f"{prefix}.mlp.experts.gate_up_proj_scale_inv",
                                       "role": "mixture_of_experts_gate_up_weights_block_scale_inverse"}
        refs["moe_output_scale_inv"] = {"tensor": f"{prefix}.mlp.experts.down_proj_scale_inv",
                                        "role": "mixture_of_experts_down_weights_block_scale_inverse"}
    for ref, tensor, role in linears:
        refs[ref + "_scale_inv"] = {"tensor": f"{prefix}.{tensor}.weight_scale_inv", "role": role + "_block_scale_inverse"}

    def pair(ref):
        return [ref, ref + "_scale_inv"]

    semantic = [
        {"id": "operator_norm", "op": "rms_norm", "inputs": ["input_frame"], "outputs": ["operator_norm_out"],
         "params": ["operator_norm"], "attrs": dict(norm_attrs)},
        {"id": "q_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["q_projected"], "params": pair("q_projection")},
        {"id": "k_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["k_projected"], "params": pair("k_projection")},
        {"id": "v_projection", "op": "linear", "inputs": ["operator_norm_out"], "outputs": ["v_projected"], "params": pair("v_projection")},
    ]
    if spec.qk_norm:
        semantic += [
            {"id": "q_head_norm", "op": "rms_norm_per_head", "inputs": ["q_projected"], "outputs": ["q_normed"], "params": ["q_norm"],
             "attrs": {**norm_attrs, **att, "head_count": spec.q_heads}},
            {"id": "k_head_norm", "op": "rms_norm_per_head", "inputs": ["k_projected"], "outputs": ["k_normed"], "params": ["k_norm"],
             "attrs": {**norm_attrs, **att, "head_count": spec.kv_heads}},
        ]
    semantic += [
        {"id": "q_rope", "op": "rotary_position_embedding", "inputs": ["q_normed" if spec.qk_norm else "q_projected"], "outputs": ["q_positioned"],
         "attrs": {**rope, "head_count": spec.q_heads}},
        {"id": "k_rope", "op": "rotary_position_embedding", "inputs": ["k_normed" if spec.qk_norm else "k_projected"], "outputs": ["k_positioned"],
         "attrs": {**rope, "head_count": spec.kv_heads}},
        {"id": "kv_memory_append", "op": "append_state_update", "inputs": ["k_positioned", "v_projected", "kv_memory"],
         "outputs": ["k_memory", "v_memory"], "state_reads": ["kv_memory"], "state_writes": ["kv_memory"],
         "attrs": {"growth": "per_activation", **att}},
        {"id": "attention_read", "op": "scaled_dot_product_attention", "inputs": ["q_positioned", "k_memory", "v_memory"],
         "outputs": ["attention_out"], "params": [],
         "attrs": {"causal": True, "scale": spec.head_dim ** -0.5, "window_size": None, "attention_sinks": False, **att}},
        {"id": "attention_out_projection", "op": "linear", "inputs": ["attention_out"], "outputs": ["operator_out"],
         "params": pair("attention_out_projection")},
        {"id": "operator_residual", "op": "residual_add", "inputs": ["input_frame", "operator_out"], "outputs": ["operator_residual_out"]},
        {"id": "ffn_norm", "op": "rms_norm", "inputs": ["operator_residual_out"], "outputs": ["ffn_norm_out"],
         "params": ["ffn_norm"], "attrs": dict(norm_attrs)},
    ]
    if moe:
        expert_attrs = {"hidden_size": h, "intermediate_size": spec.moe_ffn, "num_experts": spec.experts, "experts_per_token": spec.experts_per_token}
        semantic += [
            {"id": "moe_router_projection", "op": "linear", "inputs": ["ffn_norm_out"], "outputs": ["moe_router_logits"], "params": ["moe_router"]},
            {"id": "moe_topk", "op": "moe_topk", "inputs": ["moe_router_logits"], "outputs": ["moe_routes"], "params": [],
             "attrs": {"num_experts": spec.experts, "experts_per_token": spec.experts_per_token, "activation": "softmax",
                       "normalize_selected": True, "logit_softcap": 0.0, "selection_bias": False}},
            {"id": "sparse_moe_gate_up", "op": "sparse_moe_gate_up", "inputs": ["ffn_norm_out", "moe_routes"],
             "outputs": ["moe_expert_intermediates"], "params": pair("moe_input"), "attrs": dict(expert_attrs)},
            {"id": "sparse_moe_down", "op": "sparse_moe_down", "inputs": ["moe_expert_intermediates", "moe_routes"],
             "outputs": ["moe_expert_outputs"], "params": pair("moe_output"), "attrs": dict(expert_attrs)},
            {"id": "moe_reduce", "op": "moe_reduce", "inputs": ["moe_expert_outputs"], "outputs": ["ffn_out"],
             "attrs": {"hidden_size": h, "experts_per_token": spec.experts_per_token, "routed_scaling_factor": 1.0}},
        ]
    else:
        semantic += [
            {"id": "ffn_gate_projection", "op": "linear", "inputs": ["ffn_norm_out"], "outputs": ["ffn_gate"], "params": pair("ffn_gate")},
            {"id": "ffn_up_projection", "op": "linear", "inputs": ["ffn_norm_out"], "outputs": ["ffn_up"], "params": pair("ffn_up")},
            {"id": "ffn_gate_activation", "op": "silu", "inputs": ["ffn_gate"], "outputs": ["ffn_gate_activated"], "attrs": {"element_count": ffn}},
            {"id": "ffn_gate_multiply", "op": "multiply", "inputs": ["ffn_gate_activated", "ffn_up"], "outputs": ["ffn_hidden"]},
            {"id": "ffn_down_projection", "op": "linear", "inputs": ["ffn_hidden"], "outputs": ["ffn_out"], "params": pair("ffn_down")},
        ]
    semantic.append({"id": "ffn_residual", "op": "residual_add", "inputs": ["operator_residual_out", "ffn_out"], "outputs": ["output_frame"]})
    by_id = {node["id"]: node for node in semantic}
    eb = {"output_element_bytes": [2]}

    def plain(node_id):
        node = dict(by_id[node_id])
        node["attrs"] = {**node.get("attrs", {}), **eb}
        return node

    # q/k/v: the widest group of consecutive projections whose block shapes agree (three, else two, else one)
    projections = [("q_projection", q_width), ("k_projection", kv_width), ("v_projection", kv_width)]
    groups, index = [], 0
    while index < len(projections):
        for count in (3, 2, 1):
            group = projections[index:index + count]
            if len(group) == count and len({_fp8_block_shape(width, h) for _, width in group}) == 1:
                break
        groups.append([name for name, _ in group])
        index += len(group)
    projection_nodes = []
    for group in groups:
        if len(group) == 1:
            node = plain(group[0])
        else:
            node = {"id": "__".join(group), "op": f"parallel_linear_{len(group)}way", "inputs": ["operator_norm_out"],
                    "outputs": [by_id[name]["outputs"][0] for name in group], "params": [p for name in group for p in pair(name)],
                    "attrs": {"compiled_from": list(group), "branch_count": len(group), "branch_parameter_counts": [2] * len(group),
                              "output_element_bytes": [2] * len(group)}}
        projection_nodes.append((node, group))

    fused, kernels = [], []

    def emit(node, sources):
        fused.append(node)
        kernels.append((node["op"], node["id"], list(sources)))

    def emit_prequantized(consumers, signal, width):
        """One quantize node for all `consumers` [(node, semantic source ids)] of `signal`, then the consumers."""
        first = consumers[0][0]["id"]
        helper, quantized, scale = f"{first}__quantize_input", f"{first}__input_fp8_e4m3", f"{first}__input_scale_f32"
        sources = [source for _, ids in consumers for source in ids]
        emit({"id": helper, "op": "quantize_fp8_e4m3", "inputs": [signal], "outputs": [quantized, scale],
              "attrs": {"physical_representation_contract": FP8_CONTRACT, "consumer_node_ids": [node["id"] for node, _ in consumers],
                        "semantic_source_node_ids": sources, "element_count": width, "block_columns": 128,
                        "output_element_bytes": [1, 4]}}, sources)
        for node, ids in consumers:
            logical = list(node["inputs"])
            node["inputs"] = [quantized, scale, *logical[1:]]
            node["attrs"] = {**node["attrs"], "physical_input_contract": FP8_CONTRACT, "physical_input_provider_id": helper,
                             "physical_logical_inputs": logical}
            emit(node, ids)

    emit(plain("operator_norm"), ["operator_norm"])
    emit_prequantized(projection_nodes, "operator_norm_out", h)
    if spec.qk_norm:
        branch_ids = ["q_head_norm", "q_rope", "k_head_norm", "k_rope"]
        emit({"id": "__".join(branch_ids), "op": "parallel_head_norm_rope_2way", "inputs": ["q_projected", "k_projected"],
              "outputs": ["q_positioned", "k_positioned"], "params": ["q_norm", "k_norm"],
              "attrs": {"compiled_from": branch_ids,
                        "branches": [{"norm": dict(by_id["q_head_norm"]["attrs"]), "rope": dict(by_id["q_rope"]["attrs"])},
                                     {"norm": dict(by_id["k_head_norm"]["attrs"]), "rope": dict(by_id["k_rope"]["attrs"])}],
                        "intermediate_rounding": "BF16", "output_element_bytes": [2, 2]}}, branch_ids)
    else:
        emit(plain("q_rope"), ["q_rope"])
        emit(plain("k_rope"), ["k_rope"])
    emit({"id": "kv_memory_append__attention_read", "op": "append_scaled_dot_product_attention",
          "inputs": ["q_positioned", "k_positioned", "v_projected", "kv_memory"], "outputs": ["attention_out"], "params": [],
          "state_reads": ["kv_memory"], "state_writes": ["kv_memory"],
          "attrs": {"compiled_from": ["kv_memory_append", "attention_read"], "append": by_id["kv_memory_append"]["attrs"],
                    "attention": by_id["attention_read"]["attrs"], "current_kv_source": "direct_bf16_input", **eb}},
         ["kv_memory_append", "attention_read"])
    out_sources = ["attention_out_projection", "operator_residual"]
    emit_prequantized([({"id": "__".join(out_sources), "op": "linear_residual", "inputs": ["attention_out", "input_frame"],
                         "outputs": ["operator_residual_out"], "params": pair("attention_out_projection"),
                         "attrs": {"compiled_from": out_sources, "intermediate_rounding": "BF16", **eb}}, out_sources)], "attention_out", q_width)
    emit(plain("ffn_norm"), ["ffn_norm"])
    if moe:
        # the router is a BF16 linear and the expert kernels quantise their own input: no quantize nodes here
        for node_id in ("moe_router_projection", "moe_topk", "sparse_moe_gate_up", "sparse_moe_down", "moe_reduce", "ffn_residual"):
            emit(plain(node_id), [node_id])
        return _layer_component(spec, component_id, layer_index, refs, semantic, fused, kernels, layout="gqa_attention_layer_params_v1_sparse_moe")
    gate_sources = ["ffn_gate_projection", "ffn_up_projection", "ffn_gate_activation", "ffn_gate_multiply"]
    emit_prequantized([({"id": "__".join(gate_sources), "op": "parallel_linear_silu_multiply", "inputs": ["ffn_norm_out"],
                         "outputs": ["ffn_hidden"], "params": pair("ffn_gate") + pair("ffn_up"),
                         "attrs": {"compiled_from": gate_sources, "branch_count": 2, "intermediate_rounding": "BF16",
                                   "element_count": ffn, **eb}}, gate_sources)], "ffn_norm_out", h)
    down_sources = ["ffn_down_projection", "ffn_residual"]
    emit_prequantized([({"id": "__".join(down_sources), "op": "linear_residual", "inputs": ["ffn_hidden", "operator_residual_out"],
                         "outputs": ["output_frame"], "params": pair("ffn_down"),
                         "attrs": {"compiled_from": down_sources, "intermediate_rounding": "BF16", **eb}}, down_sources)], "ffn_hidden", ffn)
    return _layer_component(spec, component_id, layer_index, refs, semantic, fused, kernels)


def _adapter_circuit(spec: ModelSpec, decoder_id: str):
    h = spec.hidden
    component_id = f"{decoder_id}_input_adapter"
    refs = {
        "embedding_norm": {"tensor": "mtp.pre_fc_norm_embedding.weight", "role": f"{component_id}.embedding_norm"},
        "hidden_norm": {"tensor": "mtp.pre_fc_norm_hidden.weight", "role": f"{component_id}.hidden_norm"},
        "input_projection": {"tensor": "mtp.fc.weight", "role": f"{component_id}.input_projection"},
    }
    eb = {"output_element_bytes": [2]}
    common = {"state_reads": [], "state_writes": []}
    nodes = [
        {"id": "embedding_norm", "op": "rms_norm", "inputs": ["token_embedding"], "outputs": ["normalized_embedding"],
         "params": ["embedding_norm"], **common, "attrs": {"eps": spec.eps, "weight_offset": 0.0, **eb}},
        {"id": "hidden_norm", "op": "rms_norm", "inputs": ["target_hidden"], "outputs": ["normalized_hidden"],
         "params": ["hidden_norm"], **common, "attrs": {"eps": spec.eps, "weight_offset": 0.0, **eb}},
        {"id": "embedding_hidden_concat", "op": "concatenate", "inputs": ["normalized_embedding", "normalized_hidden"],
         "outputs": ["combined_frame"], "params": [], **common, "attrs": {"axis": "channel", "part_widths": [h, h], **eb}},
        {"id": "input_projection", "op": "linear", "inputs": ["combined_frame"], "outputs": ["output_frame"],
         "params": ["input_projection"], **common, "attrs": dict(eb)},
    ]
    circuit_id = f"{component_id}_circuit_v1"
    params = {"schema": "nerve.circuit_params.v1", "circuit": circuit_id, "layout": "source_tensor_refs",
              "storage": "safetensors", "refs": refs}
    circuit = {
        "schema": "nerve.stream_circuit.v1", "id": circuit_id,
        "source": {"component_id": component_id, "source_layer_index": None, "source_operator_type": "draft_input_adapter"},
        "runtime_role": "draft_input_adapter", "behavioral_role": "stream_generation_circuit",
        "implementation": "compiled_normalized_embedding_hidden_projection_v1",
        "boundary": {"inputs": [{"id": "token_embedding", "signal": "frame", "shape": [h], "component_port": "token_embedding"},
                                {"id": "target_hidden", "signal": "frame", "shape": [h], "component_port": "target_hidden"}],
                     "outputs": [{"id": "output_frame", "signal": "frame", "shape": [h], "component_port": "output_frame",
                                  "source": "output_frame"}], "controls": []},
        "state_ports": [], "parameters": {"layout": "source_tensor_refs", "storage": "safetensors", "refs": refs},
        "nodes": nodes,
    }
    component = {
        "component_id": component_id, "operator_type": "draft_input_adapter", "runtime_role": "draft_input_adapter",
        "implementation": "compiled_normalized_embedding_hidden_projection_v1", "behavioral_role": "stream_generation_circuit",
        "circuit": circuit, "params": params,
        "state": {"schema": "nerve.circuit_state.v1", "circuit": circuit_id, "state_ports": []},
    }
    kernels = [("rms_norm", "embedding_norm"), ("rms_norm", "hidden_norm"), ("concatenate", "embedding_hidden_concat"),
               ("linear", "input_projection")]
    execution = {
        "component_id": component_id, "operator_type": "draft_input_adapter",
        "implementation": "compiled_normalized_embedding_hidden_projection_v1",
        "kernels": [{"execution_index": index, "node_id": node_id, "op": op, "source_node_ids": [node_id],
                     "execution_domain": "decode"} for index, (op, node_id) in enumerate(kernels)],
    }
    return component, execution


def _draft_output_component(spec: ModelSpec, decoder_id: str, projection_tensor: str):
    component_id = f"{decoder_id}_output_transducer"
    circuit_id = f"{component_id}_circuit_v1"
    refs = {"norm": {"tensor": "mtp.norm.weight", "role": f"{component_id}.norm"},
            "projection": {"tensor": projection_tensor, "role": f"{component_id}.projection"}}
    nodes = [
        {"id": "output_norm", "op": "rms_norm", "inputs": ["input_frame"], "outputs": ["output_hidden"], "params": ["norm"],
         "state_reads": [], "state_writes": [], "attrs": {"eps": spec.eps, "weight_offset": 0.0, "output_element_bytes": [2]}},
        {"id": "output_projection", "op": "linear_projection", "inputs": ["output_hidden"], "outputs": ["output_logits"],
         "params": ["projection"], "state_reads": [], "state_writes": [],
         "attrs": {"scale": 1.0, "soft_cap": None, "output_element_bytes": [2]}},
    ]
    return {
        "component_id": component_id, "operator_type": "draft_output_transducer", "runtime_role": "draft_output_transducer",
        "implementation": "compiled_draft_output_transducer_v1", "behavioral_role": "stream_generation_circuit",
        "circuit": {"schema": "nerve.stream_circuit.v1", "id": circuit_id, "boundary": {
            "inputs": [{"id": "input_frame", "signal": "frame", "shape": [spec.hidden], "component_port": "input_frame"}],
            "outputs": [{"id": "output_hidden", "signal": "frame", "shape": [spec.hidden], "component_port": "output_hidden",
                         "source": "output_hidden"},
                        {"id": "output_logits", "signal": "logits", "shape": [spec.vocab], "component_port": "output_logits",
                         "source": "output_logits"}],
            "controls": []}, "state_ports": [],
            "parameters": {"layout": "source_tensor_refs", "storage": "safetensors", "refs": refs}, "nodes": nodes},
        "params": {"schema": "nerve.circuit_params.v1", "circuit": circuit_id, "layout": "source_tensor_refs",
                   "storage": "safetensors", "refs": refs},
        "state": {"schema": "nerve.circuit_state.v1", "circuit": circuit_id, "state_ports": []},
    }


def build_manifest(spec: ModelSpec) -> dict:
    if spec.quant not in ("bf16", "int4", "fp8") or ((spec.experts or spec.qk_norm) and spec.quant != "fp8"):
        raise ValueError("the native writer covers dense BF16 / INT4 / FP8 decoders and FP8 decoders with sparse experts or per-head q/k norms")
    projection_tensor = "model.embed_tokens.weight" if spec.tied else "lm_head.weight"
    components, executions, edges = [], [], []
    previous = ("input_transducer", "output_frame")
    for layer in range(spec.layers):
        component_id = f"layer_{layer:02d}"
        component, execution = _layer_circuit(spec, component_id, f"model.layers.{layer}", layer, spec.quant)
        components.append(component)
        executions.append(execution)
        edges.append({"id": f"edge_{len(edges):04d}", "connection": {"kind": "forward"},
                      "source": {"component_id": previous[0], "port_id": previous[1]},
                      "destination": {"component_id": component_id, "port_id": "input_frame"}})
        previous = (component_id, "output_frame")
    edges.append({"id": f"edge_{len(edges):04d}", "connection": {"kind": "forward"},
                  "source": {"component_id": previous[0], "port_id": previous[1]},
                  "destination": {"component_id": "output_transducer", "port_id": "input_frame"}})
    edges.append({"id": f"edge_{len(edges):04d}", "connection": {"kind": "forward"},
                  "source": {"component_id": "output_transducer", "port_id": "logits"},
                  "destination": {"component_id": "sampler", "port_id": "logits"}})
    dimensions = {
        "hidden_size": spec.hidden, "intermediate_sizes": [spec.moe_ffn if spec.experts else spec.ffn] * spec.layers, "num_hidden_layers": spec.layers,
        "num_attention_heads": spec.q_heads, "num_key_value_heads": spec.kv_heads, "head_width": spec.head_dim,
        "rotary_width": spec.head_dim, "attention_window_size": None, "conv_l_cache": 0, "vocab_size": spec.vocab,
        "max_position_embeddings": spec.max_positions, "num_experts": spec.experts or None, "experts_per_token": spec.experts_per_token or None,
        "attention_layer_shapes": [
            {"layer": layer, "query_heads": spec.q_heads, "key_value_heads": spec.kv_heads, "head_width": spec.head_dim,
             "rotary_width": spec.head_dim, "rope_theta": float(spec.rope_theta), "rope_type": "default",
             "shared_kv_source_layer": None} for layer in range(spec.layers)],
    }
    manifest = {
        "schema": "nerve.vulkan_resident_model_package.v3",
        "package_id": f"model_{spec.name}_cuda_resident",
        "compiler_fingerprint": "llmoop_b200.package_writer.v1",
        "circuit_graph": {
            "topology": "explicit_graph", "edges": edges,
            "boundary": {
                "external_inputs": [{"id": "user_input", "endpoint": {"component_id": "input_transducer", "port_id": "input_token"}},
                                    {"id": "random_seed", "endpoint": {"component_id": "sampler", "port_id": "random_seed"}}],
                "public_outputs": [{"id": "model_output", "endpoint": {"component_id": "sampler", "port_id": "sampled_token"}}]},
            "architecture": {"family": "decoder_only_transformer", "model_type": "synthetic_" + spec.quant,
                             "architectures": ["SyntheticForCausalLM"], "dtype": "bfloat16"},
            "dimensions": dimensions,
            "input_transducer": {"id": "token_embedding", "type": "embedding_lookup", "output": "stream_frame",
                                 "attrs": {"scale": 1.0}, "params": {"weight": {"tensor": "model.embed_tokens.weight"}}},
            "output_transducer": {"components": [
                {"id": "output_norm", "type": "rms_norm", "attrs": {"eps": spec.eps, "weight_offset": 0.0},
                 "params": {"weight": {"tensor": "model.norm.weight"}}},
                {"id": "output_projection", "type": "linear_projection", "attrs": {"scale": 1.0, "soft_cap": None},
                 "params": {"weight": {"tensor": projection_tensor}}}]},
            "components": components,
        },
        "tensor_index_path": "tensors.json",
        "config_path": "config.json",
        "activation_element_bytes": 2,
        "max_context_activations": spec.max_positions,
        "input_transducer": {"spec": {
            "transducer_id": "input_transducer.token_embedding", "parameter_tensor": "model.embed_tokens.weight",
            "parameter_dtype": "BF16", "parameter_shape": [spec.vocab, spec.hidden],
            "parameter_byte_capacity": spec.vocab * spec.hidden * 2, "output_signal_id": "input_frame",
            "output_frame_byte_capacity": spec.hidden * 2, "output_frame_word_count": spec.hidden // 2}},
        "output_transducer": {"spec": {
            "transducer_id": "output_transducer", "input_signal_id": "output_frame",
            "node_ids": ["output_norm", "output_projection"], "norm_parameter_tensor": "model.norm.weight",
            "norm_parameter_dtype": "BF16", "norm_parameter_shape": [spec.hidden],
            "projection_parameter_tensor": projection_tensor, "projection_parameter_dtype": "BF16",
            "projection_parameter_shape": [spec.vocab, spec.hidden], "projection_scale_parameter_tensor": None,
            "logits_byte_capacity": spec.vocab * 4}},
        "sampler": {"spec": {"sampler_id": "greedy_sampler", "method": "greedy", "temperature": 1.0, "top_k": 1, "top_p": 1.0,
                             "min_p": 0.0, "presence_penalty": 0.0, "repetition_penalty": 1.0, "runtime_parameterized": False}},
        "component_executions": executions,
        "speculative_decoders": [],
    }
    if spec.mtp:
        decoder_id = "draft_00"
        adapter_component, adapter_execution = _adapter_circuit(spec, decoder_id)
        layer_id = f"{decoder_id}_layer_00"
        layer_component, layer_execution = _layer_circuit(spec, layer_id, "mtp.layers.0", 0, spec.quant)
        manifest["speculative_decoders"].append({
            "id": decoder_id, "type": "multi_token_prediction", "source_prefix": "mtp",
            "circuit_graph": {
                "topology": "explicit_graph",
                "edges": [
                    {"id": f"{decoder_id}_edge_0000", "connection": {"kind": "forward"},
                     "source": {"component_id": adapter_component["component_id"], "port_id": "output_frame"},
                     "destination": {"component_id": layer_id, "port_id": "input_frame"}},
                    {"id": f"{decoder_id}_edge_0001", "connection": {"kind": "forward"},
                     "source": {"component_id": layer_id, "port_id": "output_frame"},
                     "destination": {"component_id": f"{decoder_id}_output_transducer", "port_id": "input_frame"}}],
                "components": [adapter_component, layer_component, _draft_output_component(spec, decoder_id, projection_tensor)],
            },
            "input_adapter": {"component_id": adapter_component["component_id"], "token_embedding_signal_id": "token_embedding",
                              "target_hidden_signal_id": "target_hidden", "output_signal_id": "output_frame",
                              "input_frame_byte_capacity": spec.hidden * 2, "target_hidden_byte_capacity": spec.hidden * 2,
                              "output_frame_byte_capacity": spec.hidden * 2},
            "output_transducer": {
                "component_id": f"{decoder_id}_output_transducer", "input_signal_id": "output_frame",
                "hidden_signal_id": "output_hidden", "logits_signal_id": "output_logits",
                "norm_parameter_tensor": "mtp.norm.weight", "norm_parameter_dtype": "BF16",
                "projection_parameter_tensor": projection_tensor, "projection_parameter_dtype": "BF16",
                "vocabulary_size": spec.vocab, "hidden_size": spec.hidden,
                "norm_shader_path": f"shaders/rms_norm_bf16_h{spec.hidden}_eps{format(spec.eps, '.9g')}_offset0.spv"},
            "component_executions": [adapter_execution, layer_execution],
            "state_contract": {"ownership": "per_stream_per_node_instance", "draft_updates": "tentative",
                               "acceptance": "commit_accepted_prefix", "rejection": "restore_last_committed_state"},
            "verification_contract": {"target_execution": "multi_token", "state_updates": "transactional",
                                      "acceptance": "longest_matching_prefix"},
        })
    return manifest


def runtime_config(spec: ModelSpec) -> dict:
    return {
        "schema": "nerve.runtime_model_config.v1", "bos_token_id": 1, "eos_token_id": spec.eos_token_id, "pad_token_id": 0,
        "numerics": {"rms_norm_eps": spec.eps, "rope_theta": float(spec.rope_theta), "rope_interleaved": False,
                     "rms_norm_weight_offset": 0.0, "embedding_scale": 1.0, "residual_scale": 1.0,
                     "attention_scale": spec.head_dim ** -0.5, "logits_scale": 1.0, "logits_soft_cap": None},
    }


_EXPERT_TENSOR = re.compile(r"^(.*\.mlp\.experts)\.(\d+)\.(gate|up|down)_proj\.(weight|weight_scale_inv)$")


def _pack_expert_tensors(tensors):
    """Separately stored experts become the packed [expert, row, column] tensors every sparse MoE component reads
    (nerve/model_transpiler_quantization.py:22-250): `experts.gate_up_proj` = per expert the gate rows, then the up
    rows; `experts.down_proj` = the down matrices stacked; their block scales packed the same way."""
    parts, order = {}, []
    for name, dtype, shape, data in tensors:
        match = _EXPERT_TENSOR.match(name)
        if match is None:
            yield name, dtype, shape, data
            continue
        base, expert, projection, kind = match.group(1), int(match.group(2)), match.group(3), match.group(4)
        if base not in parts:
            parts[base] = {}
            order.append(base)
        raw = data if isinstance(data, (bytes, bytearray, memoryview)) else np.ascontiguousarray(data).tobytes()
        parts[base][(expert, projection, kind)] = (dtype, [int(d) for d in shape], bytes(raw))
    for base in order:
        group = parts[base]
        experts = sorted({expert for expert, _, _ in group})
        if experts != list(range(len(experts))):
            raise ValueError(f"{base}: expert indices are not contiguous")
        for kind, suffix in (("weight", ""), ("weight_scale_inv", "_scale_inv")):
            gate_dtype, gate_shape, _ = group[(0, "gate", kind)]
            down_dtype, down_shape, _ = group[(0, "down", kind)]
            for expert in experts:
                if group[(expert, "gate", kind)][1] != gate_shape or group[(expert, "up", kind)][1] != gate_shape or group[(expert, "down", kind)][1] != down_shape:
                    raise ValueError(f"{base}: expert {expert} has other projection shapes than expert 0")
            yield (f"{base}.gate_up_proj{suffix}", gate_dtype, [len(experts), 2 * gate_shape[0], gate_shape[1]],
                   b"".join(group[(expert, projection, kind)][2] for expert in experts for projection in ("gate", "up")))
            yield (f"{base}.down_proj{suffix}", down_dtype, [len(experts), down_shape[0], down_shape[1]],
                   b"".join(group[(expert, "down", kind)][2] for expert in experts))


def write_package(spec: ModelSpec, directory, tensors=None, hash_tensors: bool = True) -> Path:
    """Writes a complete package directory.  `tensors` is an iterable of (name, dtype, shape, array-or-bytes);
    default = the seeded numpy checkpoint of llmoop_b200.synth.build_checkpoint(spec)."""
    directory = Path(directory)
    (directory / "weights").mkdir(parents=True, exist_ok=True)
    if tensors is None:
        _, built = build_checkpoint(spec)
        tensors = ((name, dtype, shape, data) for name, (dtype, shape, data) in built.items())
    if spec.experts:
        tensors = _pack_expert_tensors(tensors)
    index = {}
    for name, dtype, shape, data in tensors:
        if name.endswith(".weight_shape"):
            continue  # the compiler folds weight_shape into logical_shape
        raw = data if isinstance(data, (bytes, bytearray, memoryview)) else np.ascontiguousarray(data)
        relative = _tensor_file(name)
        write_safetensors(directory / relative, {name: (dtype, shape, raw)}, metadata={"format": "nerve", "layout": "row_major"})
        count = int(np.prod(shape)) if len(shape) else 1
        byte_count = count * DTYPE_BYTES[dtype]
        entry = {"dtype": dtype, "shape": [int(d) for d in shape], "data_offsets": [0, byte_count], "parameter_count": count,
                 "byte_count": byte_count, "source_file": relative, "layout": "row_major"}
        if hash_tensors:
            view = raw if isinstance(raw, (bytes, bytearray, memoryview)) else raw.view(np.uint8).reshape(-1)
            entry["data_sha256"] = hashlib.sha256(view).hexdigest()
        if name.endswith(".weight_packed"):
            base = name[: -len(".weight_packed")]
            entry["logical_shape"] = [int(shape[0]), int(shape[1]) * 8]
            entry["quantization"] = {"format": "compressed_tensors_pack_quantized", "bits": 4, "group_size": 128,
                                     "symmetric": True, "signed_offset": 8, "scales": base + ".weight_scale"}
        index[name] = entry
    _dump(directory / "tensors.json", {
        "schema": "nerve.tensor_index.v1", "source": {"packaged": True, "compiled": True, "weights_dir": "weights"},
        "totals": {"tensor_count": len(index), "parameter_count": sum(e["parameter_count"] for e in index.values()),
                   "byte_count": sum(e["byte_count"] for e in index.values())},
        "tensors": index})
    _dump(directory / "config.json", runtime_config(spec))
    manifest = build_manifest(spec)
    lowered = directory / "lowered"
    for component in manifest["circuit_graph"]["components"]:
        _dump(lowered / component["component_id"] / "circuit.json", component["circuit"])
        _dump(lowered / component["component_id"] / "params.json", component["params"])
        _dump(lowered / component["component_id"] / "state.json", component["state"])
    for decoder in manifest["speculative_decoders"]:
        for component in decoder["circuit_graph"]["components"]:
            base = lowered / "drafts" / decoder["id"] / component["component_id"]
            _dump(base / "circuit.json", component["circuit"])
            _dump(base / "params.json", component["params"])
            _dump(base / "state.json", component["state"])
    files = {}
    for path in sorted(directory.rglob("*.json")):
        relative = path.relative_to(directory).as_posix()
        if relative in ("vulkan_resident_package.json", "synthetic_spec.json"):
            continue
        blob = path.read_bytes()
        files[relative] = {"byte_count": len(blob), "sha256": hashlib.sha256(blob).hexdigest()}
    manifest["artifact_integrity"] = {"schema": "nerve.package_artifact_integrity.v1", "algorithm": "sha256", "files": files}
    _dump(directory / "vulkan_resident_package.json", manifest)
    _dump(directory / "synthetic_spec.json", spec.to_json())
    return directory
