#include "package.hpp"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <sys/stat.h>

#include "sha256.hpp"

namespace nerve {

namespace {

[[noreturn]] void fail(const std::string &message) { throw std::runtime_error(message); }

bool is_directory(const std::string &path) {
    struct stat info;
    return stat(path.c_str(), &info) == 0 && S_ISDIR(info.st_mode);
}

uint64_t file_size(const std::string &path) {
    struct stat info;
    if (stat(path.c_str(), &info) != 0) fail("package file is missing: " + path);
    return static_cast<uint64_t>(info.st_size);
}

std::string hash_file(const std::string &path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) fail("cannot open " + path);
    Sha256 hash;
    std::vector<char> buffer(1 << 20);
    while (in) {
        in.read(buffer.data(), static_cast<std::streamsize>(buffer.size()));
        if (in.gcount() > 0) hash.update(buffer.data(), static_cast<size_t>(in.gcount()));
    }
    return hash.hex();
}

std::vector<std::string> string_list(const Json &value) {
    std::vector<std::string> out;
    if (value.is_array())
        for (const Json &item : value.items()) out.push_back(item.as_string());
    return out;
}

const Json *find_by(const Json &array, const char *key, const std::string &value) {
    if (!array.is_array()) return nullptr;
    for (const Json &item : array.items())
        if (item[key].is_string() && item[key].as_string() == value) return &item;
    return nullptr;
}

RopeAttrs rope_attrs(const Json &attrs) {
    if (attrs["rope_type"].is_string() && attrs["rope_type"].as_string() != "default")
        fail("unsupported rope_type " + attrs["rope_type"].as_string());
    if (!attrs["scaling"].is_null()) fail("rope scaling is not supported by the CUDA backend");
    RopeAttrs rope;
    rope.heads = static_cast<int>(attrs.at("head_count").as_int());
    rope.head_width = static_cast<int>(attrs.at("head_width").as_int());
    rope.rotary_width = static_cast<int>(attrs.at("rotary_width").as_int());
    rope.interleaved = attrs["interleaved"].is_bool() && attrs["interleaved"].as_bool();
    rope.theta = shader_float(attrs.at("theta").as_double());
    return rope;
}

}  // namespace

float shader_float(double value) {
    char text[64];
    std::snprintf(text, sizeof(text), "%.9g", value);
    return std::strtof(text, nullptr);
}

std::string read_file(const std::string &path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) fail("cannot open " + path);
    std::ostringstream out;
    out << in.rdbuf();
    return out.str();
}

std::shared_ptr<HostPackage> HostPackage::open(const std::string &path, VerifyLevel verify) {
    auto package = std::shared_ptr<HostPackage>(new HostPackage());
    package->load(path, verify);
    return package;
}

const TensorInfo &HostPackage::tensor(const std::string &name) const {
    auto found = tensors_.find(name);
    if (found == tensors_.end()) fail("package tensor index has no tensor \"" + name + "\"");
    return found->second;
}

namespace {
// Bytes per element of the safetensors dtypes a package can hold (0: unknown to this backend, checked where used).
uint64_t dtype_bytes(const std::string &dtype) {
    if (dtype == "BF16" || dtype == "F16" || dtype == "I16" || dtype == "U16") return 2;
    if (dtype == "F32" || dtype == "I32" || dtype == "U32") return 4;
    if (dtype == "F8_E4M3" || dtype == "F8_E5M2" || dtype == "I8" || dtype == "U8" || dtype == "BOOL") return 1;
    if (dtype == "F64" || dtype == "I64" || dtype == "U64") return 8;
    return 0;
}
}  // namespace

// Fails unless `name` holds exactly `elements` values of `dtype`.
void HostPackage::require_elements(const std::string &name, const std::string &dtype, uint64_t elements, const std::string &what) const {
    const TensorInfo &info = tensor(name);
    if (info.dtype != dtype) fail(what + " " + name + " must be " + dtype + " (it is " + info.dtype + ")");
    if (info.byte_count() != elements * dtype_bytes(dtype))
        fail(what + " " + name + ": " + std::to_string(info.byte_count()) + " bytes where the plan's dimensions need " +
             std::to_string(elements * dtype_bytes(dtype)));
}

void HostPackage::load(const std::string &path, VerifyLevel verify) {
    std::string manifest_path = path;
    if (is_directory(path)) manifest_path = path + "/vulkan_resident_package.json";
    size_t slash = manifest_path.find_last_of('/');
    dir_ = slash == std::string::npos ? "." : manifest_path.substr(0, slash);
    manifest_ = Json::parse(read_file(manifest_path));
    const std::string schema = manifest_["schema"].is_string() ? manifest_["schema"].as_string() : "";
    if (schema != "nerve.vulkan_resident_model_package.v3")
        fail("unsupported package schema \"" + schema + "\" (expected nerve.vulkan_resident_model_package.v3)");

    verify_artifacts(verify);

    const std::string index_path = dir_ + "/" + manifest_.at("tensor_index_path").as_string();
    Json index = Json::parse(read_file(index_path));
    if (!index["schema"].is_string() || index["schema"].as_string() != "nerve.tensor_index.v1")
        fail("unsupported tensor index schema in " + index_path);
    for (const auto &member : index.at("tensors").members()) {
        const Json &entry = member.second;
        TensorInfo info;
        info.name = member.first;
        info.dtype = entry.at("dtype").as_string();
        for (const Json &dim : entry.at("shape").items()) info.shape.push_back(dim.as_int());
        if (entry["logical_shape"].is_array())
            for (const Json &dim : entry["logical_shape"].items()) info.logical_shape.push_back(dim.as_int());
        else
            info.logical_shape = info.shape;
        info.source_file = entry.at("source_file").as_string();
        info.begin = static_cast<uint64_t>(entry.at("data_offsets")[0].as_int());
        info.end = static_cast<uint64_t>(entry.at("data_offsets")[1].as_int());
        if (info.end < info.begin) fail("tensor " + info.name + ": data_offsets end before they begin");
        if (entry["byte_count"].is_number() && static_cast<uint64_t>(entry["byte_count"].as_int()) != info.end - info.begin)
            fail("tensor " + info.name + ": byte_count disagrees with data_offsets");
        // the kernels take their extents from the shapes: the bytes on disk must cover them exactly
        // (the reference refuses such a tensor too: vulkan_distributed/planning.rs:582, "byte count does not match ... shape")
        if (const uint64_t element = dtype_bytes(info.dtype)) {
            uint64_t elements = 1;
            for (int64_t dim : info.shape) {
                if (dim < 0) fail("tensor " + info.name + ": negative dimension");
                elements *= static_cast<uint64_t>(dim);
            }
            if (elements * element != info.end - info.begin)
                fail("tensor " + info.name + ": byte count " + std::to_string(info.end - info.begin) + " does not match shape x " + info.dtype + " = " +
                     std::to_string(elements * element));
        }
        info.sha256 = entry["data_sha256"].is_string() ? entry["data_sha256"].as_string() : "";
        if (entry["layout"].is_string() && entry["layout"].as_string() != "row_major")
            fail("tensor " + info.name + ": unsupported layout " + entry["layout"].as_string());
        const Json &quant = entry["quantization"];
        if (quant.is_object()) {
            info.quantized = true;
            const std::string format = quant.at("format").as_string();
            if (format != "compressed_tensors_pack_quantized")
                fail("tensor " + info.name + ": unsupported quantization format " + format);
            info.bits = static_cast<int>(quant.at("bits").as_int());
            info.group_size = static_cast<int>(quant.at("group_size").as_int());
            info.signed_offset = static_cast<int>(quant["signed_offset"].is_number() ? quant["signed_offset"].as_int() : 0);
            info.scales = quant.at("scales").as_string();
            if (info.bits != 4 || info.signed_offset != 8 || !(quant["symmetric"].is_bool() && quant["symmetric"].as_bool()))
                fail("tensor " + info.name + ": only symmetric 4-bit pack-quantized weights with offset 8 are supported");
        }
        tensors_.emplace(info.name, std::move(info));
    }
    build_plan();
}

void HostPackage::verify_artifacts(VerifyLevel verify) {
    if (verify == VerifyLevel::None) return;
    const Json &integrity = manifest_["artifact_integrity"];
    if (!integrity.is_object()) fail("package manifest has no artifact_integrity table");
    if (integrity["algorithm"].is_string() && integrity["algorithm"].as_string() != "sha256")
        fail("unsupported artifact_integrity algorithm");
    for (const auto &member : integrity.at("files").members()) {
        const std::string &relative = member.first;
        // Level Used: every JSON artifact the mounter reads; level All: every listed file.
        bool used = relative == manifest_["tensor_index_path"].as_string() || relative == "config.json" ||
                    relative.rfind("lowered/", 0) == 0;
        if (verify == VerifyLevel::Used && !used) continue;
        const std::string full = dir_ + "/" + relative;
        uint64_t expected_bytes = static_cast<uint64_t>(member.second.at("byte_count").as_int());
        if (file_size(full) != expected_bytes)
            fail("package artifact " + relative + " has " + std::to_string(file_size(full)) + " bytes; manifest records " +
                 std::to_string(expected_bytes));
        if (hash_file(full) != member.second.at("sha256").as_string())
            fail("package artifact " + relative + " failed its sha256 check");
        verified_files_++;
    }
}

void HostPackage::read_tensor_range(const std::string &name, uint64_t byte_begin, uint64_t byte_count, void *out) const {
    const TensorInfo &info = tensor(name);
    if (byte_begin + byte_count > info.byte_count()) fail("tensor " + name + ": byte range outside the tensor");
    const std::string path = dir_ + "/" + info.source_file;
    auto base = data_base_.find(info.source_file);
    std::FILE *file = std::fopen(path.c_str(), "rb");
    if (!file) fail("cannot open weights file " + path);
    uint64_t data_base;
    if (base == data_base_.end()) {
        uint8_t header[8];
        if (std::fread(header, 1, 8, file) != 8) {
            std::fclose(file);
            fail("weights file " + path + " is truncated");
        }
        uint64_t header_len = 0;
        for (int i = 7; i >= 0; i--) header_len = (header_len << 8) | header[i];
        data_base = 8 + header_len;
        data_base_[info.source_file] = data_base;
    } else {
        data_base = base->second;
    }
    if (fseeko(file, static_cast<off_t>(data_base + info.begin + byte_begin), SEEK_SET) != 0 ||
        std::fread(out, 1, byte_count, file) != byte_count) {
        std::fclose(file);
        fail("weights file " + path + " is truncated (tensor " + name + ")");
    }
    std::fclose(file);
}

std::vector<uint8_t> HostPackage::read_tensor(const std::string &name, bool verify) const {
    const TensorInfo &info = tensor(name);
    std::vector<uint8_t> data(info.byte_count());
    read_tensor_range(name, 0, info.byte_count(), data.data());
    if (verify && !info.sha256.empty() && Sha256::of(data.data(), data.size()) != info.sha256)
        fail("tensor " + name + " failed its sha256 check");
    return data;
}

WeightRef HostPackage::weight_ref(const Json &refs, const std::string &param) const {
    const Json &ref = refs[param];
    if (!ref.is_object()) fail("circuit params have no ref \"" + param + "\"");
    WeightRef out;
    out.tensor = ref.at("tensor").as_string();
    const TensorInfo &info = tensor(out.tensor);
    if (info.logical_shape.size() < 2) fail("linear weight " + out.tensor + " is not a matrix");
    out.n = info.logical_shape[info.logical_shape.size() - 2];
    out.k = info.logical_shape[info.logical_shape.size() - 1];
    if (info.dtype == "BF16") {
        out.storage = TensorStorage::BF16;
        if (out.n <= 0 || out.k <= 0) fail("linear weight " + out.tensor + ": empty matrix");
        require_elements(out.tensor, "BF16", static_cast<uint64_t>(out.n) * out.k, "linear weight");
    } else if (info.dtype == "I32" && info.quantized) {
        out.storage = TensorStorage::INT4_CT;
        out.scale = info.scales;
        out.group = info.group_size;
        const TensorInfo &scale = tensor(out.scale);
        if (scale.dtype != "BF16") fail("INT4 scales " + out.scale + " must be BF16");
        if (out.n <= 0 || out.k <= 0 || out.group <= 0) fail("INT4 weight " + out.tensor + ": empty matrix or group");
        if (out.k % out.group != 0 || out.k % 8 != 0) fail("INT4 weight " + out.tensor + ": K is not a multiple of the group size");
        if (info.byte_count() != static_cast<uint64_t>(out.n) * out.k / 2)
            fail("INT4 weight " + out.tensor + ": " + std::to_string(info.byte_count()) + " packed bytes where its logical shape needs " +
                 std::to_string(static_cast<uint64_t>(out.n) * out.k / 2));
        require_elements(out.scale, "BF16", static_cast<uint64_t>(out.n) * (out.k / out.group), "INT4 scales");
    } else if (info.dtype == "F8_E4M3") {
        out.storage = TensorStorage::FP8_BLOCK;
        out.scale = out.tensor + "_scale_inv";
        if (!has_tensor(out.scale)) {
            // expert tensors: "<name>_scale_inv" without the ".weight" suffix already matches
            fail("FP8 weight " + out.tensor + " has no " + out.scale);
        }
        if (tensor(out.scale).dtype != "BF16") fail("FP8 block scales " + out.scale + " must be BF16");
        out.group = 128;
        if (out.n <= 0 || out.k <= 0) fail("FP8 weight " + out.tensor + ": empty matrix");
        if (out.k % 128 != 0) fail("FP8 weight " + out.tensor + ": K is not a multiple of 128");
        // stacked expert tensors carry their expert count in front of [n][k]
        uint64_t stack = 1;
        for (size_t d = 0; d + 2 < info.logical_shape.size(); d++) stack *= static_cast<uint64_t>(info.logical_shape[d]);
        if (info.byte_count() != stack * static_cast<uint64_t>(out.n) * out.k)
            fail("FP8 weight " + out.tensor + ": " + std::to_string(info.byte_count()) + " bytes where its shape needs " +
                 std::to_string(stack * static_cast<uint64_t>(out.n) * out.k));
        require_elements(out.scale, "BF16", stack * static_cast<uint64_t>((out.n + 127) / 128) * (out.k / 128), "FP8 block scales");
    } else {
        fail("unsupported weight dtype " + info.dtype + " for " + out.tensor);
    }
    return out;
}

ComponentPlan HostPackage::build_component(const Json &execution, const Json &component) {
    ComponentPlan plan;
    plan.id = execution.at("component_id").as_string();
    plan.operator_type = execution["operator_type"].is_string() ? execution["operator_type"].as_string() : "";
    const Json &circuit = component.at("circuit");
    const Json &refs = component.at("params").at("refs");
    for (const Json &input : circuit.at("boundary").at("inputs").items()) {
        const std::string id = input.at("id").as_string();
        plan.boundary_inputs.push_back(id);
        plan.signals[id] = SignalInfo{input.at("shape")[0].as_int(), 2};
    }
    plan.boundary_output = circuit.at("boundary").at("outputs")[0].at("id").as_string();

    auto width_of = [&](const std::string &name) -> int64_t {
        auto found = plan.signals.find(name);
        if (found == plan.signals.end()) fail("component " + plan.id + ": signal " + name + " is read before it is produced");
        return found->second.width;
    };

    for (const Json &kernel : execution.at("kernels").items()) {
        const std::string op = kernel.at("op").as_string();
        const std::string node_id = kernel.at("node_id").as_string();
        const Json *node_ptr = find_by(circuit.at("nodes"), "id", node_id);
        if (!node_ptr) fail("component " + plan.id + ": kernel node " + node_id + " is not in the circuit");
        const Json &node = *node_ptr;
        const Json &attrs = node["attrs"];
        OpSpec spec;
        spec.op_name = op;
        spec.node_id = node_id;
        spec.inputs = string_list(node["inputs"]);
        spec.outputs = string_list(node["outputs"]);
        std::vector<std::string> params = string_list(node["params"]);
        spec.prequantized_input = attrs["physical_input_contract"].is_string();
        auto declare = [&](size_t index, int64_t width, int bytes = 2) {
            plan.signals[spec.outputs.at(index)] = SignalInfo{width, bytes};
        };

        if (op == "rms_norm") {
            spec.kind = OpKind::RmsNorm;
            spec.norm_weights.push_back(refs[params.at(0)].at("tensor").as_string());
            spec.eps = shader_float(attrs.at("eps").as_double());
            spec.weight_offset = shader_float(attrs.at("weight_offset").as_double());
            require_elements(spec.norm_weights.back(), "BF16", static_cast<uint64_t>(width_of(spec.inputs.at(0))), "norm weight");
            declare(0, width_of(spec.inputs.at(0)));
        } else if (op == "linear" || op == "parallel_linear_2way" || op == "parallel_linear_3way") {
            spec.kind = OpKind::Linear;
            // params: one entry per branch for BF16/INT4, (weight, scale_inv) pairs for FP8
            std::vector<std::string> weight_params;
            if (attrs["branch_parameter_counts"].is_array()) {
                size_t cursor = 0;
                for (const Json &count : attrs["branch_parameter_counts"].items()) {
                    weight_params.push_back(params.at(cursor));
                    cursor += static_cast<size_t>(count.as_int());
                }
            } else if (spec.outputs.size() == 1) {
                weight_params.push_back(params.at(0));
            } else {
                weight_params = params;
            }
            if (weight_params.size() != spec.outputs.size()) fail("component " + plan.id + ": " + node_id + " branch count mismatch");
            for (size_t branch = 0; branch < weight_params.size(); branch++) {
                spec.weights.push_back(weight_ref(refs, weight_params[branch]));
                declare(branch, spec.weights.back().n);
            }
        } else if (op == "linear_residual") {
            spec.kind = OpKind::LinearResidual;
            spec.weights.push_back(weight_ref(refs, params.at(0)));
            spec.residual_input = spec.inputs.back();
            // BF16 rounds the product before adding (linear_residual_bf16.comp.template:47-53);
            // FP8 adds in f32 and rounds once (nerve/model_package_shader_templates.py:746-783).
            spec.residual_rounds_product = spec.weights[0].storage != TensorStorage::FP8_BLOCK;
            declare(0, spec.weights[0].n);
        } else if (op == "parallel_linear_silu_multiply") {
            spec.kind = OpKind::LinearSiluMultiply;
            if (attrs["branch_parameter_counts"].is_array()) {
                size_t cursor = 0;
                for (const Json &count : attrs["branch_parameter_counts"].items()) {
                    spec.weights.push_back(weight_ref(refs, params.at(cursor)));
                    cursor += static_cast<size_t>(count.as_int());
                }
            } else if (params.size() == 2) {
                spec.weights.push_back(weight_ref(refs, params[0]));
                spec.weights.push_back(weight_ref(refs, params[1]));
            } else if (params.size() == 4) {
                spec.weights.push_back(weight_ref(refs, params[0]));
                spec.weights.push_back(weight_ref(refs, params[2]));
            } else {
                fail("component " + plan.id + ": unexpected parameter list on " + node_id);
            }
            declare(0, spec.weights[0].n);
        } else if (op == "quantize_fp8_e4m3") {
            spec.kind = OpKind::QuantizeFp8;
            int64_t width = width_of(spec.inputs.at(0));
            int64_t block = attrs.at("block_columns").as_int();
            if (block != 128 || width % 128 != 0) fail("quantize_fp8_e4m3 expects 128-column blocks");
            declare(0, width, 1);
            declare(1, width / block, 4);
        } else if (op == "rotary_position_embedding") {
            spec.kind = OpKind::Rope;
            spec.rope.push_back(rope_attrs(attrs));
            declare(0, width_of(spec.inputs.at(0)));
        } else if (op == "parallel_head_norm_rope_2way") {
            spec.kind = OpKind::HeadNormRope;
            size_t branch = 0;
            for (const Json &entry : attrs.at("branches").items()) {
                spec.rope.push_back(rope_attrs(entry.at("rope")));
                spec.eps = shader_float(entry.at("norm").at("eps").as_double());
                spec.weight_offset = shader_float(entry.at("norm").at("weight_offset").as_double());
                spec.norm_weights.push_back(refs[params.at(branch)].at("tensor").as_string());
                declare(branch, width_of(spec.inputs.at(branch)));
                branch++;
            }
        } else if (op == "append_scaled_dot_product_attention") {
            spec.kind = OpKind::AppendAttention;
            const Json &attention = attrs.at("attention");
            if (!attention["window_size"].is_null()) fail("sliding-window attention is not supported by the CUDA backend");
            if (attention["attention_sinks"].is_bool() && attention["attention_sinks"].as_bool())
                fail("attention sinks are not supported by the CUDA backend");
            spec.q_heads = static_cast<int>(attention.at("query_heads").as_int());
            spec.kv_heads = static_cast<int>(attention.at("key_value_heads").as_int());
            spec.head_width = static_cast<int>(attention.at("head_width").as_int());
            spec.attention_scale = shader_float(attention.at("scale").as_double());
            plan.has_kv = true;
            plan.kv_heads = spec.kv_heads;
            plan.head_width = spec.head_width;
            plan.q_heads = spec.q_heads;
            declare(0, static_cast<int64_t>(spec.q_heads) * spec.head_width);
        } else if (op == "residual_add") {
            spec.kind = OpKind::ResidualAdd;
            declare(0, width_of(spec.inputs.at(0)));
        } else if (op == "silu_multiply") {
            spec.kind = OpKind::SiluMultiply;
            declare(0, width_of(spec.inputs.at(0)));
        } else if (op == "concatenate") {
            spec.kind = OpKind::Concat;
            int64_t width = 0;
            for (const std::string &input : spec.inputs) width += width_of(input);
            declare(0, width);
        } else if (op == "moe_topk") {
            spec.kind = OpKind::MoeTopk;
            spec.experts = static_cast<int>(attrs.at("num_experts").as_int());
            spec.top_k = static_cast<int>(attrs.at("experts_per_token").as_int());
            if (attrs.at("activation").as_string() != "softmax" || !attrs.at("normalize_selected").as_bool() ||
                attrs.at("selection_bias").as_bool() || attrs.at("logit_softcap").as_double() != 0.0)
                fail("only softmax-over-selected MoE routing is supported by the CUDA backend");
            declare(0, spec.top_k, 4);
        } else if (op == "sparse_moe_gate_up" || op == "sparse_moe_down") {
            spec.kind = op == "sparse_moe_gate_up" ? OpKind::MoeGateUp : OpKind::MoeDown;
            spec.experts = static_cast<int>(attrs.at("num_experts").as_int());
            spec.top_k = static_cast<int>(attrs.at("experts_per_token").as_int());
            spec.moe_hidden = static_cast<int>(attrs.at("hidden_size").as_int());
            spec.moe_inter = static_cast<int>(attrs.at("intermediate_size").as_int());
            spec.weights.push_back(weight_ref(refs, params.at(0)));
            declare(0, static_cast<int64_t>(spec.top_k) * (spec.kind == OpKind::MoeGateUp ? spec.moe_inter : spec.moe_hidden));
        } else if (op == "moe_reduce") {
            spec.kind = OpKind::MoeReduce;
            spec.top_k = static_cast<int>(attrs.at("experts_per_token").as_int());
            spec.moe_hidden = static_cast<int>(attrs.at("hidden_size").as_int());
            spec.routed_scale = shader_float(attrs.at("routed_scaling_factor").as_double());
            declare(0, spec.moe_hidden);
        } else {
            fail("component " + plan.id + ": the CUDA backend has no kernel for op \"" + op + "\"");
        }
        plan.ops.push_back(std::move(spec));
    }
    if (!plan.signals.count(plan.boundary_output))
        fail("component " + plan.id + ": no kernel produces the boundary output " + plan.boundary_output);
    return plan;
}

void HostPackage::build_plan() {
    const Json &graph = manifest_.at("circuit_graph");
    const Json &dims = graph.at("dimensions");
    plan_.hidden = dims.at("hidden_size").as_int();
    plan_.vocab = dims.at("vocab_size").as_int();
    plan_.max_context = manifest_["max_context_activations"].is_number() ? manifest_["max_context_activations"].as_int() : 0;
    plan_.embedding_tensor = manifest_.at("input_transducer").at("spec").at("parameter_tensor").as_string();
    plan_.embedding_scale = shader_float(graph.at("input_transducer")["attrs"]["scale"].is_number()
                                             ? graph.at("input_transducer")["attrs"]["scale"].as_double()
                                             : 1.0);
    if (plan_.hidden <= 0 || plan_.vocab <= 0) fail("hidden_size and vocab_size must be positive");
    require_elements(plan_.embedding_tensor, "BF16", static_cast<uint64_t>(plan_.vocab) * plan_.hidden, "embedding table");

    const Json &out_spec = manifest_.at("output_transducer").at("spec");
    plan_.output.norm_tensor = out_spec.at("norm_parameter_tensor").as_string();
    plan_.output.projection_tensor = out_spec.at("projection_parameter_tensor").as_string();
    require_elements(plan_.output.projection_tensor, "BF16", static_cast<uint64_t>(plan_.vocab) * plan_.hidden, "output projection");
    require_elements(plan_.output.norm_tensor, "BF16", static_cast<uint64_t>(plan_.hidden), "output norm");
    for (const Json &component : graph.at("output_transducer").at("components").items()) {
        const std::string type = component.at("type").as_string();
        if (type == "rms_norm") {
            plan_.output.eps = shader_float(component.at("attrs").at("eps").as_double());
            plan_.output.weight_offset = shader_float(component.at("attrs").at("weight_offset").as_double());
        } else if (type == "linear_projection") {
            plan_.output.logits_scale = shader_float(component.at("attrs").at("scale").as_double());
            if (!component.at("attrs")["soft_cap"].is_null()) fail("logit soft-cap is not supported by the CUDA backend");
        }
    }

    const Json &sampler = manifest_["sampler"]["spec"];
    if (sampler.is_object()) {
        plan_.sampler_method = sampler["method"].is_string() ? sampler["method"].as_string() : "greedy";
        plan_.temperature = static_cast<float>(sampler["temperature"].is_number() ? sampler["temperature"].as_double() : 1.0);
        plan_.top_k = static_cast<int>(sampler["top_k"].is_number() ? sampler["top_k"].as_int() : 1);
        plan_.top_p = static_cast<float>(sampler["top_p"].is_number() ? sampler["top_p"].as_double() : 1.0);
        plan_.min_p = static_cast<float>(sampler["min_p"].is_number() ? sampler["min_p"].as_double() : 0.0);
    }

    for (const Json &execution : manifest_.at("component_executions").items()) {
        const std::string id = execution.at("component_id").as_string();
        const Json *component = find_by(graph.at("components"), "component_id", id);
        if (!component) fail("component_executions names unknown component " + id);
        plan_.layers.push_back(build_component(execution, *component));
    }

    const Json &decoders = manifest_["speculative_decoders"];
    if (decoders.is_array() && decoders.size() > 0) {
        const Json &decoder = decoders[0];
        if (decoder.at("type").as_string() != "multi_token_prediction")
            fail("unsupported speculative decoder type " + decoder.at("type").as_string());
        const Json &verification = decoder.at("verification_contract");
        if (verification.at("acceptance").as_string() != "longest_matching_prefix")
            fail("unsupported speculative acceptance rule " + verification.at("acceptance").as_string());
        plan_.has_draft = true;
        plan_.draft_id = decoder.at("id").as_string();
        const Json &adapter = decoder.at("input_adapter");
        const std::string adapter_id = adapter.at("component_id").as_string();
        plan_.adapter_token_signal = adapter.at("token_embedding_signal_id").as_string();
        plan_.adapter_hidden_signal = adapter.at("target_hidden_signal_id").as_string();
        plan_.adapter_output_signal = adapter.at("output_signal_id").as_string();
        const Json &components = decoder.at("circuit_graph").at("components");
        for (const Json &execution : decoder.at("component_executions").items()) {
            const std::string id = execution.at("component_id").as_string();
            const Json *component = find_by(components, "component_id", id);
            if (!component) fail("draft component_executions names unknown component " + id);
            if (id == adapter_id) plan_.draft_adapter = build_component(execution, *component);
            else plan_.draft_layers.push_back(build_component(execution, *component));
        }
        const Json &out = decoder.at("output_transducer");
        plan_.draft_output.norm_tensor = out.at("norm_parameter_tensor").as_string();
        plan_.draft_output.projection_tensor = out.at("projection_parameter_tensor").as_string();
        require_elements(plan_.draft_output.projection_tensor, "BF16", static_cast<uint64_t>(plan_.vocab) * plan_.hidden, "draft output projection");
        require_elements(plan_.draft_output.norm_tensor, "BF16", static_cast<uint64_t>(plan_.hidden), "draft output norm");
        const Json *out_component = find_by(components, "component_id", out.at("component_id").as_string());
        if (!out_component) fail("draft output transducer component is missing");
        for (const Json &node : out_component->at("circuit").at("nodes").items()) {
            if (node.at("op").as_string() == "rms_norm") {
                plan_.draft_output.eps = shader_float(node.at("attrs").at("eps").as_double());
                plan_.draft_output.weight_offset = shader_float(node.at("attrs").at("weight_offset").as_double());
            } else if (node.at("op").as_string() == "linear_projection") {
                plan_.draft_output.logits_scale = shader_float(node.at("attrs").at("scale").as_double());
            }
        }
    }

    const std::string config_path = dir_ + "/" + (manifest_["config_path"].is_string() ? manifest_["config_path"].as_string() : "config.json");
    Json config = Json::parse(read_file(config_path));
    const Json &eos = config["eos_token_id"];
    if (eos.is_number()) plan_.eos_token_ids.push_back(static_cast<uint32_t>(eos.as_int()));
    else if (eos.is_array())
        for (const Json &item : eos.items()) plan_.eos_token_ids.push_back(static_cast<uint32_t>(item.as_int()));
}

}  // namespace nerve
