"""The native package writer must agree, field by field, with what the reference compiler emitted for the same
synthetic checkpoint (golden packages), on every field the runtime contract reads."""

import json

import pytest

from conftest import GOLDEN


def _load(path):
    return json.loads((path / "vulkan_resident_package.json").read_text())


def _strip(node):
    node = dict(node)
    node.setdefault("params", [])
    for key in ("state_reads", "state_writes"):
        node.setdefault(key, [])
    return node


def _components(manifest):
    out = {c["component_id"]: c for c in manifest["circuit_graph"]["components"]}
    for decoder in manifest["speculative_decoders"]:
        out.update({c["component_id"]: c for c in decoder["circuit_graph"]["components"]})
    return out


def _executions(manifest):
    out = {e["component_id"]: e for e in manifest["component_executions"]}
    for decoder in manifest["speculative_decoders"]:
        out.update({e["component_id"]: e for e in decoder["component_executions"]})
    return out


@pytest.mark.parametrize("name", ["cfg1_bf16_mtp", "tiny_int4_mtp", "tiny_int4_mtp_v16", "tiny_fp8_mtp", "tiny_moe_fp8_mtp"])
def test_native_writer_matches_reference_compiler(name, tmp_path):
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec

    spec = ModelSpec(**json.loads((GOLDEN / name / "synthetic_spec.json").read_text()))
    write_package(spec, tmp_path / name)
    ours, theirs = _load(tmp_path / name), _load(GOLDEN / name)

    assert ours["schema"] == theirs["schema"]
    for key in ("tensor_index_path", "config_path", "activation_element_bytes", "max_context_activations"):
        assert ours[key] == theirs[key], key
    assert ours["circuit_graph"]["dimensions"] == theirs["circuit_graph"]["dimensions"]
    assert ours["circuit_graph"]["input_transducer"] == theirs["circuit_graph"]["input_transducer"]
    assert ours["circuit_graph"]["output_transducer"] == theirs["circuit_graph"]["output_transducer"]
    for key, value in ours["input_transducer"]["spec"].items():
        assert theirs["input_transducer"]["spec"][key] == value, key
    for key, value in ours["output_transducer"]["spec"].items():
        assert theirs["output_transducer"]["spec"][key] == value, key
    for key, value in ours["sampler"]["spec"].items():
        assert theirs["sampler"]["spec"][key] == value, key

    our_components, their_components = _components(ours), _components(theirs)
    for component_id, component in our_components.items():
        reference = their_components[component_id]
        assert component["params"]["refs"] == reference["params"]["refs"], component_id
        assert component["circuit"]["boundary"] == reference["circuit"]["boundary"], component_id
        assert component["circuit"]["state_ports"] == reference["circuit"]["state_ports"], component_id
        assert [_strip(n) for n in component["circuit"]["nodes"]] == [_strip(n) for n in reference["circuit"]["nodes"]], component_id
        if "semantic_execution_nodes" in component["circuit"]:
            assert ([_strip(n) for n in component["circuit"]["semantic_execution_nodes"]]
                    == [_strip(n) for n in reference["circuit"]["semantic_execution_nodes"]]), component_id
    our_exec, their_exec = _executions(ours), _executions(theirs)
    assert list(our_exec) == list(their_exec)
    for component_id, execution in our_exec.items():
        mine = [(k["op"], k["node_id"], k["source_node_ids"]) for k in execution["kernels"]]
        want = [(k["op"], k["node_id"], k["source_node_ids"]) for k in their_exec[component_id]["kernels"]]
        assert mine == want, component_id
    our_decoder, their_decoder = ours["speculative_decoders"][0], theirs["speculative_decoders"][0]
    for key in ("id", "type", "source_prefix", "input_adapter", "state_contract", "verification_contract"):
        assert our_decoder[key] == their_decoder[key], key
    for key, value in our_decoder["output_transducer"].items():
        assert their_decoder["output_transducer"][key] == value, key

    our_index = json.loads((tmp_path / name / "tensors.json").read_text())["tensors"]
    their_index = json.loads((GOLDEN / name / "tensors.json").read_text())["tensors"]
    assert set(our_index) == set(their_index)
    for tensor, entry in our_index.items():
        assert entry == their_index[tensor], tensor  # dtype, shape, offsets, file name, sha256, quantization


def test_native_package_passes_the_mounter_validation(tmp_path):
    import llmoop_b200 as nb
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec

    spec = ModelSpec(name="writer_check", hidden=128, layers=3, q_heads=4, kv_heads=1, head_dim=32, ffn=384, vocab=64,
                     quant="int4", seed=11)
    write_package(spec, tmp_path / "pkg")
    ops, tensors = nb.validate_package(tmp_path / "pkg", 2)
    assert ops == 3 * 15 + 4 + 15
    assert tensors == 2 + 1 + 3 * 16 + 4 + 16  # embed+lm_head, norm, layers, mtp head, mtp layer


def test_native_fp8_package_fuses_projections_by_block_shape_and_passes_the_mounter_validation(tmp_path):
    """q/k/v whose scale grids imply one block shape become parallel_linear_3way behind one quantize node
    (nerve/model_package_tensors.py:618-660); narrower k/v leave q a linear of its own, as in the golden package."""
    import llmoop_b200 as nb
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec

    spec = ModelSpec(name="writer_fp8_check", hidden=256, layers=2, q_heads=8, kv_heads=4, head_dim=32, ffn=512, vocab=64,
                     quant="fp8", seed=12)
    write_package(spec, tmp_path / "pkg")
    manifest = _load(tmp_path / "pkg")
    ops = [kernel["op"] for kernel in manifest["component_executions"][0]["kernels"]]
    assert ops == ["rms_norm", "quantize_fp8_e4m3", "parallel_linear_3way", "rotary_position_embedding", "rotary_position_embedding",
                   "append_scaled_dot_product_attention", "quantize_fp8_e4m3", "linear_residual", "rms_norm", "quantize_fp8_e4m3",
                   "parallel_linear_silu_multiply", "quantize_fp8_e4m3", "linear_residual"]
    fused = manifest["circuit_graph"]["components"][0]["circuit"]["nodes"][2]
    assert fused["attrs"]["branch_parameter_counts"] == [2, 2, 2] and len(fused["params"]) == 6
    op_count, tensor_count = nb.validate_package(tmp_path / "pkg", 2)
    assert op_count == 2 * 13 + 4 + 13
    assert tensor_count == 2 + 1 + 2 * 16 + 4 + 16


def test_native_moe_package_passes_the_mounter_validation(tmp_path):
    import llmoop_b200 as nb
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec

    spec = ModelSpec(name="writer_moe_check", hidden=256, layers=2, q_heads=8, kv_heads=4, head_dim=32, ffn=256, vocab=64,
                     quant="fp8", seed=13, experts=4, experts_per_token=2, moe_ffn=128, qk_norm=True)
    write_package(spec, tmp_path / "pkg")
    manifest = _load(tmp_path / "pkg")
    ops = [kernel["op"] for kernel in manifest["component_executions"][0]["kernels"]]
    assert ops == ["rms_norm", "quantize_fp8_e4m3", "parallel_linear_3way", "parallel_head_norm_rope_2way",
                   "append_scaled_dot_product_attention", "quantize_fp8_e4m3", "linear_residual", "rms_norm", "linear", "moe_topk",
                   "sparse_moe_gate_up", "sparse_moe_down", "moe_reduce", "residual_add"]
    index = json.loads((tmp_path / "pkg" / "tensors.json").read_text())["tensors"]
    assert index["model.layers.0.mlp.experts.gate_up_proj"]["shape"] == [4, 256, 256]
    assert index["model.layers.0.mlp.experts.down_proj_scale_inv"]["shape"] == [4, 2, 1]
    assert not any(".experts.0." in name for name in index)
    op_count, tensor_count = nb.validate_package(tmp_path / "pkg", 2)
    assert op_count == 2 * 14 + 4 + 14
