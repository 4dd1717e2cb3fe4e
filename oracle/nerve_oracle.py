"""CPU oracle for the MTP speculative decode path of a compiled NERVE package.

TEST INFRASTRUCTURE ONLY.  Only tests/, __graft_entry__.smoke() and bench.py's
CPU-baseline / reference legs may import this module; the product
(llmoop_b200) never does.

Parity status: "parity unpinned" for layer numerics, logits and token
sequences - the reference ships no golden data for them and its Vulkan path
cannot run here.  The oracle is a restatement of the reference's shader
arithmetic (oracle/nerve_oracle_ops.c, each function citing its shader) driven
op-by-op by the package's own kernel lists, plus the host-side cycle semantics
of
  runtime-rs/src/vulkan_stream_circuit/placed_stream_processor/feedback_generation.rs:66-194
  runtime-rs/src/vulkan_stream_circuit/resident_package_slices/speculative_decoder_processor.rs:206-488
  runtime-rs/src/vulkan_stream_circuit/placed_stream_processor/temporal_prompt.rs:298-478
  runtime-rs/src/vulkan_stream_circuit/placed_prompt_event.rs:167-291
  runtime-rs/src/vulkan_stream_circuit/speculative_decode.rs:54-105
What the reference's tests do pin (acceptance rule, sampler records, hash,
control/page-table bytes, number formats) is checked in tests/test_oracle_pins.py.
"""

from __future__ import annotations

import ctypes
import json
import os
import struct
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libnerve_oracle.so"

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> Path:
    source = HERE / "nerve_oracle_ops.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < source.stat().st_mtime:
        subprocess.check_call(["make", "-s", "-C", str(HERE), "libnerve_oracle.so"])
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.orc_bf16_to_f32.restype = ctypes.c_float
        _lib.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.orc_f32_to_bf16.restype = ctypes.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.orc_e4m3_to_f32.restype = ctypes.c_float
        _lib.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        _lib.orc_f32_to_e4m3.restype = ctypes.c_uint8
        _lib.orc_f32_to_e4m3.argtypes = [ctypes.c_float]
        _lib.orc_top2_gap.restype = ctypes.c_float
        _lib.orc_greedy.restype = ctypes.c_uint32
        _lib.orc_hash_u32.restype = ctypes.c_uint32
        _lib.orc_hash_u32.argtypes = [ctypes.c_uint32]
        _lib.orc_sample_top_k_top_p.restype = ctypes.c_uint32
        _lib.orc_sample_top_k_top_p.argtypes = [_f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                                ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, _u32p]
    return _lib


def _p(array, kind):
    return array.ctypes.data_as(kind)


def shader_float(value: float) -> np.float32:
    """Shader constants travel through the shader file name formatted with
    format(x, ".9g") and are parsed back to f32
    (nerve/model_package_shader_selection.py:1272-1273)."""
    return np.float32(float(format(float(value), ".9g")))


def attention_tile_tokens(head_width: int) -> int:
    """nerve/model_package_shader_selection.py:1245-1263."""
    padded = ((head_width + 63) // 64) * 64
    physical = 1024 // padded
    budget = (32 * 1024) // 4
    fixed = 2 * head_width + 4
    per_tile = head_width + ((head_width + 31) // 32) + 3
    batches = max(1, min(7, (budget - fixed) // (physical * per_tile)))
    return physical * batches


# --------------------------------------------------------------------------- package


_CARRIER = {"BF16": np.uint16, "F8_E4M3": np.uint8, "I32": np.uint32, "F32": np.float32, "I64": np.int64}


class OraclePackage:
    """Reads a compiled package directory straight from its JSON + safetensors
    files (independent of the product's mounter)."""

    def __init__(self, directory):
        self.dir = Path(directory)
        self.manifest = json.loads((self.dir / "vulkan_resident_package.json").read_text())
        index = json.loads((self.dir / self.manifest["tensor_index_path"]).read_text())
        self.tensor_index = index["tensors"]
        self._cache: dict = {}
        dims = self.manifest["circuit_graph"]["dimensions"]
        self.hidden = dims["hidden_size"]
        self.vocab = dims["vocab_size"]
        self.components = {}
        for component in self.manifest["circuit_graph"]["components"]:
            self.components[component["component_id"]] = component
        self.layers = list(self.manifest["component_executions"])
        self.draft = None
        decoders = self.manifest.get("speculative_decoders") or []
        if decoders:
            decoder = decoders[0]
            for component in decoder["circuit_graph"]["components"]:
                self.components[component["component_id"]] = component
            self.draft = decoder
        self.embedding_scale = shader_float(self.manifest["circuit_graph"]["input_transducer"]["attrs"]["scale"])
        out = self.manifest["output_transducer"]["spec"]
        self.out_norm_tensor = out["norm_parameter_tensor"]
        self.out_proj_tensor = out["projection_parameter_tensor"]
        norm_component = self.manifest["circuit_graph"]["output_transducer"]["components"][0]
        self.out_eps = shader_float(norm_component["attrs"]["eps"])
        self.out_offset = shader_float(norm_component["attrs"]["weight_offset"])
        self.logits_scale = np.float32(1.0)
        for component in self.manifest["circuit_graph"]["output_transducer"]["components"]:
            if "scale" in component.get("attrs", {}):
                self.logits_scale = shader_float(component["attrs"]["scale"])
        self.embed_tensor = self.manifest["input_transducer"]["spec"]["parameter_tensor"]

    def tensor(self, name):
        if name not in self._cache:
            entry = self.tensor_index[name]
            path = self.dir / entry["source_file"]
            with open(path, "rb") as handle:
                (header_len,) = struct.unpack("<Q", handle.read(8))
                handle.seek(8 + header_len + entry["data_offsets"][0])
                raw = handle.read(entry["data_offsets"][1] - entry["data_offsets"][0])
            array = np.frombuffer(raw, dtype=np.uint8).view(_CARRIER[entry["dtype"]]).reshape(entry["shape"]).copy()
            self._cache[name] = array
        return self._cache[name]

    def nodes(self, component_id):
        """The un-fused semantic nodes that kernels name in `source_node_ids`."""
        circuit = self.components[component_id]["circuit"]
        return {node["id"]: node for node in circuit.get("semantic_execution_nodes") or circuit["nodes"]}

    def refs(self, component_id):
        return self.components[component_id]["params"]["refs"]


# --------------------------------------------------------------------------- ops


def rms_norm(x, w, eps, offset):
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    lib().orc_rms_norm(_p(x, _u16p), _p(w, _u16p), _p(y, _u16p), x.shape[0], x.shape[1],
                       ctypes.c_float(eps), ctypes.c_float(offset))
    return y


def quantize_fp8(x, block=128):
    x = np.ascontiguousarray(x)
    q = np.empty(x.shape, dtype=np.uint8)
    scales = np.empty((x.shape[0], x.shape[1] // block), dtype=np.float32)
    lib().orc_quantize_fp8(_p(x, _u16p), _p(q, _u8p), _p(scales, _f32p), x.shape[0], x.shape[1], block)
    return q, scales


class OracleStream:
    """Per-stream transient state: KV rings for every target and draft layer,
    the pending target hidden, and the tick counter."""

    def __init__(self, package: OraclePackage, capacity: int):
        self.pkg = package
        self.capacity = capacity
        self.kv = {}
        self.pending_hidden = np.zeros((1, package.hidden), dtype=np.uint16)
        self.next_tick = 0

    def kv_state(self, component_id, kv_heads, head_width):
        if component_id not in self.kv:
            self.kv[component_id] = np.zeros((self.capacity, 2 * kv_heads * head_width), dtype=np.uint16)
        return self.kv[component_id]

    def fork(self):
        other = OracleStream(self.pkg, self.capacity)
        other.kv = {key: value.copy() for key, value in self.kv.items()}
        other.pending_hidden = self.pending_hidden.copy()
        other.next_tick = self.next_tick
        return other


class Oracle:
    def __init__(self, package: OraclePackage):
        self.pkg = package
        self.trace = None  # optional dict collecting per-op outputs

    # -- linear dispatch on the tensor's storage ------------------------------------------
    def _linear(self, x, tensor_name, residual=None):
        pkg = self.pkg
        entry = pkg.tensor_index[tensor_name]
        lanes = x.shape[0]
        x = np.ascontiguousarray(x)
        if entry["dtype"] == "BF16":
            w = pkg.tensor(tensor_name)
            n, k = w.shape
            y = np.empty((lanes, n), dtype=np.uint16)
            if residual is None:
                lib().orc_linear_bf16(_p(x, _u16p), _p(w, _u16p), _p(y, _u16p), lanes, n, k)
            else:
                residual = np.ascontiguousarray(residual)
                lib().orc_linear_residual_bf16(_p(x, _u16p), _p(w, _u16p), _p(residual, _u16p), _p(y, _u16p), lanes, n, k)
            return y
        if entry["dtype"] == "I32":
            quant = entry["quantization"]
            assert quant["format"] == "compressed_tensors_pack_quantized" and quant["bits"] == 4
            qw = pkg.tensor(tensor_name)
            scales = pkg.tensor(quant["scales"])
            n, k = entry["logical_shape"]
            y = np.empty((lanes, n), dtype=np.uint16)
            lib().orc_linear_int4_ct(_p(x, _u16p), _p(qw, _u32p), _p(scales, _u16p), _p(y, _u16p), lanes, n, k,
                                     quant["group_size"])
            if residual is not None:  # never fused for INT4 in real packages; kept for completeness
                out = np.empty_like(y)
                lib().orc_add_bf16(_p(np.ascontiguousarray(residual), _u16p), _p(y, _u16p), _p(out, _u16p), y.size)
                y = out
            return y
        if entry["dtype"] == "F8_E4M3":
            w = pkg.tensor(tensor_name)
            wscale = pkg.tensor(tensor_name + "_scale_inv")
            n, k = w.shape
            xq, xs = quantize_fp8(x)
            y = np.empty((lanes, n), dtype=np.uint16)
            res_ptr = _p(np.ascontiguousarray(residual), _u16p) if residual is not None else None
            lib().orc_linear_fp8(_p(xq, _u8p), _p(xs, _f32p), _p(w, _u8p), _p(wscale, _u16p), res_ptr, _p(y, _u16p),
                                 lanes, n, k, 128, 128)
            return y
        raise NotImplementedError(entry["dtype"])

    def _linear_silu_multiply(self, x, gate_name, up_name):
        pkg = self.pkg
        entry = pkg.tensor_index[gate_name]
        lanes = x.shape[0]
        x = np.ascontiguousarray(x)
        wg, wu = pkg.tensor(gate_name), pkg.tensor(up_name)
        n, k = wg.shape
        y = np.empty((lanes, n), dtype=np.uint16)
        if entry["dtype"] == "BF16":
            lib().orc_linear_silu_multiply_bf16(_p(x, _u16p), _p(wg, _u16p), _p(wu, _u16p), _p(y, _u16p), lanes, n, k)
        elif entry["dtype"] == "F8_E4M3":
            xq, xs = quantize_fp8(x)
            sg, su = pkg.tensor(gate_name + "_scale_inv"), pkg.tensor(up_name + "_scale_inv")
            lib().orc_linear_silu_multiply_fp8(_p(xq, _u8p), _p(xs, _f32p), _p(wg, _u8p), _p(sg, _u16p), _p(wu, _u8p),
                                               _p(su, _u16p), _p(y, _u16p), lanes, n, k, 128, 128)
        else:
            raise NotImplementedError(entry["dtype"])
        return y

    # -- one component (layer / adapter) over M lanes ------------------------------------------
    def run_component(self, execution, stream: OracleStream, inputs: dict, ticks: np.ndarray):
        pkg = self.pkg
        component_id = execution["component_id"]
        nodes = pkg.nodes(component_id)
        refs = pkg.refs(component_id)
        sig = dict(inputs)
        lanes = len(ticks)
        positions = (ticks & 0xFFFFFFFF).astype(np.uint32)

        def tensor_of(param):
            return refs[param]["tensor"]

        for kernel in execution["kernels"]:
            op = kernel["op"]
            src = [nodes[node_id] for node_id in kernel["source_node_ids"]]
            if op == "rms_norm":
                node = src[0]
                sig[node["outputs"][0]] = rms_norm(sig[node["inputs"][0]], pkg.tensor(tensor_of(node["params"][0])),
                                                   shader_float(node["attrs"]["eps"]),
                                                   shader_float(node["attrs"]["weight_offset"]))
            elif op == "quantize_fp8_e4m3":
                pass  # consumers quantise on the fly: identical arithmetic (quantize_fp8_e4m3.comp.template:41-60)
            elif op == "linear" or op.startswith("parallel_linear_") and op.endswith("way"):
                for node in src:
                    sig[node["outputs"][0]] = self._linear(sig[node["inputs"][0]], tensor_of(node["params"][0]))
            elif op == "linear_residual":
                linear, residual = src[0], src[1]
                res_input = [name for name in residual["inputs"] if name != linear["outputs"][0]][0]
                sig[residual["outputs"][0]] = self._linear(sig[linear["inputs"][0]], tensor_of(linear["params"][0]),
                                                           residual=sig[res_input])
            elif op == "parallel_linear_silu_multiply":
                linears = [node for node in src if node["op"] == "linear"]
                silu = [node for node in src if node["op"] == "silu"][0]
                multiply = [node for node in src if node["op"] == "multiply"][0]
                gate = [node for node in linears if node["outputs"][0] == silu["inputs"][0]][0]
                up = [node for node in linears if node is not gate][0]
                sig[multiply["outputs"][0]] = self._linear_silu_multiply(
                    sig[gate["inputs"][0]], tensor_of(gate["params"][0]), tensor_of(up["params"][0]))
            elif op == "rotary_position_embedding":
                node = src[0]
                attrs = node["attrs"]
                assert attrs["rope_type"] == "default" and attrs["scaling"] is None
                x = np.ascontiguousarray(sig[node["inputs"][0]])
                y = np.empty_like(x)
                lib().orc_rotary(_p(x, _u16p), _p(y, _u16p), _p(positions, _u32p), lanes, attrs["head_count"],
                                 attrs["head_width"], attrs["rotary_width"], int(attrs["interleaved"]),
                                 ctypes.c_float(shader_float(attrs["theta"])))
                sig[node["outputs"][0]] = y
            elif op == "parallel_head_norm_rope_2way":
                for norm, rope in ((src[0], src[1]), (src[2], src[3])):
                    attrs = rope["attrs"]
                    x = np.ascontiguousarray(sig[norm["inputs"][0]])
                    y = np.empty_like(x)
                    lib().orc_head_norm_rope(
                        _p(x, _u16p), _p(pkg.tensor(tensor_of(norm["params"][0])), _u16p), _p(y, _u16p),
                        _p(positions, _u32p), lanes, attrs["head_count"], attrs["head_width"], attrs["rotary_width"],
                        int(attrs["interleaved"]), ctypes.c_float(shader_float(attrs["theta"])),
                        ctypes.c_float(shader_float(norm["attrs"]["eps"])),
                        ctypes.c_float(shader_float(norm["attrs"]["weight_offset"])))
                    sig[rope["outputs"][0]] = y
            elif op == "append_scaled_dot_product_attention":
                append, read = src[0], src[1]
                attrs = read["attrs"]
                assert attrs["window_size"] is None and not attrs["attention_sinks"]
                qh, kvh, hd = attrs["query_heads"], attrs["key_value_heads"], attrs["head_width"]
                q = np.ascontiguousarray(sig[read["inputs"][0]])
                k = np.ascontiguousarray(sig[append["inputs"][0]])
                v = np.ascontiguousarray(sig[append["inputs"][1]])
                state = stream.kv_state(component_id, kvh, hd)
                out = np.empty((lanes, qh * hd), dtype=np.uint16)
                scale = shader_float(attrs["scale"])
                tile = attention_tile_tokens(hd)
                for lane in range(lanes):  # lanes in order: lane i sees what lanes < i appended
                    lib().orc_append_attention(
                        _p(q[lane], _u16p), _p(k[lane], _u16p), _p(v[lane], _u16p), _p(state, _u16p),
                        _p(out[lane], _u16p), ctypes.c_uint32(int(positions[lane])), ctypes.c_uint32(stream.capacity),
                        qh, kvh, hd, ctypes.c_float(scale), tile)
                sig[read["outputs"][0]] = out
            elif op == "residual_add":
                node = src[0]
                a = np.ascontiguousarray(sig[node["inputs"][0]])
                b = np.ascontiguousarray(sig[node["inputs"][1]])
                y = np.empty_like(a)
                lib().orc_add_bf16(_p(a, _u16p), _p(b, _u16p), _p(y, _u16p), a.size)
                sig[node["outputs"][0]] = y
            elif op == "silu_multiply":
                silu, multiply = src[0], src[1]
                gate = np.ascontiguousarray(sig[silu["inputs"][0]])
                up_name = [name for name in multiply["inputs"] if name != silu["outputs"][0]][0]
                up = np.ascontiguousarray(sig[up_name])
                y = np.empty_like(gate)
                lib().orc_silu_multiply(_p(gate, _u16p), _p(up, _u16p), _p(y, _u16p), gate.size)
                sig[multiply["outputs"][0]] = y
            elif op == "concatenate":
                node = src[0]
                sig[node["outputs"][0]] = np.concatenate([sig[name] for name in node["inputs"]], axis=1)
            elif op == "moe_topk":
                node = src[0]
                attrs = node["attrs"]
                assert attrs["activation"] == "softmax" and attrs["normalize_selected"] and not attrs["selection_bias"]
                logits = np.ascontiguousarray(sig[node["inputs"][0]])
                routes = np.empty((lanes, attrs["experts_per_token"]), dtype=np.uint32)
                lib().orc_moe_topk(_p(logits, _u16p), _p(routes, _u32p), lanes, attrs["num_experts"],
                                   attrs["experts_per_token"])
                sig[node["outputs"][0]] = routes
            elif op == "sparse_moe_gate_up":
                self._moe_gate_up = src[0]  # executed together with down + reduce below
            elif op == "sparse_moe_down":
                self._moe_down = src[0]
            elif op == "moe_reduce":
                node = src[0]
                gate_up, down = self._moe_gate_up, self._moe_down
                attrs = gate_up["attrs"]
                hidden = np.ascontiguousarray(sig[gate_up["inputs"][0]])
                routes = np.ascontiguousarray(sig[gate_up["inputs"][1]])
                wgu = pkg.tensor(tensor_of(gate_up["params"][0]))
                sgu = pkg.tensor(tensor_of(gate_up["params"][1]))
                wd = pkg.tensor(tensor_of(down["params"][0]))
                sd = pkg.tensor(tensor_of(down["params"][1]))
                assert pkg.tensor_index[tensor_of(gate_up["params"][0])]["dtype"] == "F8_E4M3"
                y = np.empty((lanes, attrs["hidden_size"]), dtype=np.uint16)
                lib().orc_moe_experts_fp8(
                    _p(hidden, _u16p), _p(routes, _u32p), _p(wgu, _u8p), _p(sgu, _u16p), _p(wd, _u8p), _p(sd, _u16p),
                    _p(y, _u16p), lanes, attrs["hidden_size"], attrs["intermediate_size"], attrs["num_experts"],
                    attrs["experts_per_token"], ctypes.c_float(shader_float(node["attrs"]["routed_scaling_factor"])))
                sig[node["outputs"][0]] = y
            else:
                raise NotImplementedError(f"oracle has no restatement for op {op!r}")
            if self.trace is not None:
                self.trace.setdefault(component_id, []).append((op, kernel["node_id"], {
                    name: value.copy() for name, value in sig.items()}))
        return sig

    # -- transducers ---------------------------------------------------------------------------
    def embed(self, tokens):
        pkg = self.pkg
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        table = pkg.tensor(pkg.embed_tensor)
        y = np.zeros((len(tokens), pkg.hidden), dtype=np.uint16)
        lib().orc_embedding(_p(table, _u16p), _p(tokens, _u32p), _p(y, _u16p), len(tokens), pkg.hidden, pkg.vocab,
                            ctypes.c_float(pkg.embedding_scale))
        return y

    def project(self, normalized):
        pkg = self.pkg
        w = pkg.tensor(pkg.out_proj_tensor)
        normalized = np.ascontiguousarray(normalized)
        logits = np.empty((normalized.shape[0], pkg.vocab), dtype=np.float32)
        lib().orc_output_projection(_p(normalized, _u16p), _p(w, _u16p), _p(logits, _f32p), normalized.shape[0],
                                    pkg.vocab, pkg.hidden, ctypes.c_float(pkg.logits_scale))
        return logits

    @staticmethod
    def greedy(logits):
        tokens = np.empty(logits.shape[0], dtype=np.uint32)
        for lane in range(logits.shape[0]):
            row = np.ascontiguousarray(logits[lane])
            tokens[lane] = lib().orc_greedy(_p(row, _f32p), row.shape[0], None)
        return tokens

    # sampler.rs:748-873: `sampler` = None (greedy) or dict(top_k, temperature, top_p, min_p, seed); draft and
    # target draw with the same hash(seed ^ tick) at the same tick
    sampler = None

    def sample(self, logits, first_tick):
        """One token per logits row; row i belongs to stream tick first_tick + i."""
        if self.sampler is None:
            return self.greedy(logits)
        cfg = self.sampler
        tokens = np.empty(logits.shape[0], dtype=np.uint32)
        for lane in range(logits.shape[0]):
            row = np.ascontiguousarray(logits[lane], dtype=np.float32)
            tick = int(first_tick) + lane
            tokens[lane] = lib().orc_sample_top_k_top_p(_p(row, _f32p), row.shape[0], int(cfg["top_k"]), float(cfg["temperature"]),
                                                        float(cfg["top_p"]), float(cfg["min_p"]), int(cfg["seed"]) & 0xffffffff,
                                                        tick & 0xffffffff, (tick >> 32) & 0xffffffff, None)
        return tokens

    @staticmethod
    def top2_gap(logits_row):
        row = np.ascontiguousarray(logits_row, dtype=np.float32)
        return float(lib().orc_top2_gap(_p(row, _f32p), row.shape[0]))

    # -- target model over M lanes (verify candidates or a prefill chunk) -----------------------
    def target_forward(self, stream, tokens, start_tick, want_logits=True):
        pkg = self.pkg
        ticks = np.arange(start_tick, start_tick + len(tokens), dtype=np.uint64)
        frame = self.embed(tokens)
        for execution in pkg.layers:
            sig = self.run_component(execution, stream, {"input_frame": frame}, ticks)
            frame = sig["output_frame"]
        normalized = rms_norm(frame, pkg.tensor(pkg.out_norm_tensor), pkg.out_eps, pkg.out_offset)
        logits = self.project(normalized) if want_logits else None
        return normalized, logits

    # -- MTP draft head -------------------------------------------------------------------------
    def draft_forward(self, stream, tokens, hidden, start_tick, want_logits):
        """adapter -> draft layer(s) -> (mtp.norm -> lm_head).  `hidden` is [M][H]."""
        pkg = self.pkg
        decoder = pkg.draft
        ticks = np.arange(start_tick, start_tick + len(tokens), dtype=np.uint64)
        adapter_id = decoder["input_adapter"]["component_id"]
        frame = None
        for execution in decoder["component_executions"]:
            if execution["component_id"] == adapter_id:
                sig = self.run_component(execution, stream, {
                    decoder["input_adapter"]["token_embedding_signal_id"]: self.embed(tokens),
                    decoder["input_adapter"]["target_hidden_signal_id"]: hidden,
                }, ticks)
                frame = sig[decoder["input_adapter"]["output_signal_id"]]
            else:
                sig = self.run_component(execution, stream, {"input_frame": frame}, ticks)
                frame = sig["output_frame"]
        if not want_logits:
            return None, None
        out = decoder["output_transducer"]
        norm_attrs = self._draft_norm_attrs()
        normalized = rms_norm(frame, pkg.tensor(out["norm_parameter_tensor"]), norm_attrs[0], norm_attrs[1])
        w = pkg.tensor(out["projection_parameter_tensor"])
        logits = np.empty((len(tokens), pkg.vocab), dtype=np.float32)
        lib().orc_output_projection(_p(normalized, _u16p), _p(w, _u16p), _p(logits, _f32p), len(tokens), pkg.vocab,
                                    pkg.hidden, ctypes.c_float(pkg.logits_scale))
        return normalized, logits

    def _draft_norm_attrs(self):
        """eps/offset of the draft output norm come from its shader name
        (rms_norm_bf16_h<H>_eps<e>_offset<o>)."""
        name = self.pkg.draft["output_transducer"]["norm_shader_path"]
        eps = float(name.split("_eps")[1].split("_offset")[0])
        offset = float(name.split("_offset")[1].rsplit(".spv", 1)[0])
        return np.float32(eps), np.float32(offset)

    # -- prefill (temporal_prompt.rs:298-478) -----------------------------------------------------
    def prefill(self, stream, tokens, sample_last=True, chunk=64):
        """Processes prompt tokens at ticks next_tick...; with an MTP decoder the
        draft gets one state step per prompt token, pairing token[i] with the
        target hidden of tick i-1.  Returns the first sampled token (or None)."""
        tokens = np.asarray(tokens, dtype=np.uint32)
        sampled = None
        last_logits = None
        for offset in range(0, len(tokens), chunk):
            piece = tokens[offset:offset + chunk]
            start = stream.next_tick
            is_last = offset + chunk >= len(tokens)
            normalized, logits = self.target_forward(stream, piece, start, want_logits=False)
            if self.pkg.draft is not None:
                hidden = np.concatenate([stream.pending_hidden, normalized[:-1]], axis=0)
                self.draft_forward(stream, piece, hidden, start, want_logits=False)
                stream.pending_hidden = normalized[-1:].copy()
            if is_last and sample_last:
                last_logits = self.project(normalized[-1:])
                sampled = int(self.sample(last_logits, start + len(piece) - 1)[0])
            stream.next_tick += len(piece)
        return sampled, last_logits

    # -- single (non-speculative) tick: placed_prompt_stream.rs:353-420 ------------------------------
    def single_tick(self, stream, token, emit):
        tick = stream.next_tick
        normalized, logits = self.target_forward(stream, [token], tick, want_logits=emit)
        if self.pkg.draft is not None:
            self.draft_forward(stream, [token], stream.pending_hidden, tick, want_logits=False)
            stream.pending_hidden = normalized.copy()
        stream.next_tick += 1
        return (int(self.sample(logits, tick)[0]), logits) if emit else (None, None)

    # -- stream state a cycle changes besides the (positional, overwritable) KV slots ------------------------
    @staticmethod
    def checkpoint(stream):
        return stream.next_tick, None if stream.pending_hidden is None else stream.pending_hidden.copy()

    @staticmethod
    def restore(stream, saved):
        stream.next_tick, stream.pending_hidden = saved[0], None if saved[1] is None else saved[1].copy()

    # -- one speculative cycle: feedback_generation.rs:66-194 ---------------------------------------------
    def speculative_cycle(self, stream, initial_token, draft_count, stop_tokens=(), forced_drafts=None, forced_targets=None):
        """forced_drafts / forced_targets replace the sampled draft / target tokens (the sampled ones are kept in
        `sampled_draft_token_ids` / `sampled_target_token_ids`): teacher forcing, and following another
        implementation's run through a near-tie."""
        start = stream.next_tick
        drafts = []
        token, hidden = initial_token, stream.pending_hidden
        draft_logits, sampled_drafts = [], []
        for j in range(draft_count):
            normalized, logits = self.draft_forward(stream, [token], hidden, start + j, want_logits=True)
            token = int(self.sample(logits, start + j)[0])
            sampled_drafts.append(token)
            draft_logits.append(logits[0])
            if forced_drafts is not None:
                token = int(forced_drafts[j])
            drafts.append(token)
            hidden = normalized
        inputs = [initial_token] + drafts
        normalized, logits = self.target_forward(stream, inputs, start, want_logits=True)
        sampled_targets = [int(t) for t in self.sample(logits, start)]
        targets = list(sampled_targets)
        if forced_targets is not None:
            for position, forced in enumerate(forced_targets):
                if position < len(targets):
                    targets[position] = int(forced)
        accepted, committed, emitted = verify_prefix(drafts, targets, stop_tokens)
        # draft catch-up: state steps for the committed inputs with hidden = pending / target frame i-1
        hidden = np.concatenate([stream.pending_hidden, normalized[:committed - 1]], axis=0)
        self.draft_forward(stream, inputs[:committed], hidden, start, want_logits=False)
        stream.pending_hidden = normalized[committed - 1:committed].copy()
        stream.next_tick += len(emitted)
        return {
            "draft_token_ids": drafts, "target_token_ids": targets, "accepted": accepted, "committed": committed,
            "emitted": emitted, "target_logits": logits, "draft_logits": draft_logits, "start_tick": start,
            "sampled_draft_token_ids": sampled_drafts, "sampled_target_token_ids": sampled_targets,
        }

    # -- a whole input event: placed_prompt_event.rs:167-291 + placed_prompt_stream.rs:570-645 ------------
    def generate(self, stream, prompt, max_new_tokens, k, stop_tokens=(), teacher=None, collect_logits=False):
        """Returns dict(tokens, cycles, ticks).  `teacher`: optional callable(list_of_generated) -> list of
        forced draft tokens (teacher-forced full acceptance harness mode)."""
        stop = set(int(t) for t in stop_tokens)
        generated, cycles, logits_log = [], [], []
        remaining = max_new_tokens
        if remaining == 0:
            self.prefill(stream, prompt, sample_last=False)
            return {"tokens": [], "cycles": [], "logits": []}
        token, logits = self.prefill(stream, prompt, sample_last=True)
        generated.append(token)
        if collect_logits:
            logits_log.append(logits[0])
        remaining -= 1
        closes = token in stop or remaining == 0
        if token in stop:
            remaining = 0
        while not closes:
            if k > 0 and self.pkg.draft is not None and remaining >= 2:
                count = min(k, remaining - 1)
                forced = teacher(generated, count) if teacher is not None else None
                cycle = self.speculative_cycle(stream, token, count, stop, forced_drafts=forced)
                cycles.append(cycle)
                for position, emitted in enumerate(cycle["emitted"]):
                    generated.append(emitted)
                    if collect_logits:
                        logits_log.append(cycle["target_logits"][position])
                    remaining -= 1
                    if emitted in stop:
                        remaining = 0
                token = generated[-1]
                closes = token in stop or remaining == 0
            else:
                token, logits = self.single_tick(stream, token, emit=True)
                generated.append(token)
                if collect_logits:
                    logits_log.append(logits[0])
                remaining -= 1
                if token in stop:
                    remaining = 0
                closes = token in stop or remaining == 0
        self.single_tick(stream, token, emit=False)  # closing feedback tick: P + N ticks in total
        return {"tokens": generated, "cycles": cycles, "logits": logits_log}


def verify_prefix(drafts, targets, stop_tokens=()):
    """speculative_decode.rs:54-105 through the C restatement."""
    drafts_a = np.asarray(drafts, dtype=np.uint32)
    targets_a = np.asarray(targets, dtype=np.uint32)
    stop_a = np.asarray(sorted(stop_tokens), dtype=np.uint32)
    out = np.zeros(2, dtype=np.uint32)
    emitted = np.zeros(len(drafts) + 2, dtype=np.uint32)
    count = ctypes.c_int(0)
    status = lib().orc_verify_prefix(_p(drafts_a, _u32p), len(drafts_a), _p(targets_a, _u32p), len(targets_a),
                                     _p(stop_a, _u32p), len(stop_a), _p(out, _u32p), _p(emitted, _u32p),
                                     ctypes.byref(count))
    if status != 0:
        raise ValueError(
            f"speculative verification has {len(drafts)} draft tokens but {len(targets)} target predictions; "
            f"expected {len(drafts) + 1}")
    return int(out[0]), int(out[1]), [int(t) for t in emitted[:count.value]]
