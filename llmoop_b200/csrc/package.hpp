// Host-side view of a compiled NERVE package (manifest schema
// nerve.vulkan_resident_model_package.v3, tensor index nerve.tensor_index.v1):
// parsing, integrity verification, tensor byte-range reads, and the execution
// plan the CUDA backend runs.
//
// Replaces, for the CUDA backend, the reference's mount path
//   runtime-rs/src/vulkan_stream_circuit/placed_model_package_loader.rs:79-404
//   runtime-rs/src/package/specs.rs:1-256 (manifest schema)
//   runtime-rs/src/tensor_storage.rs:21-136 (tensor byte ranges + SHA-256)
//   runtime-rs/src/vulkan_stream_circuit/resident_package_slices/speculative_decoder_package.rs:25-122
// The backend ignores `shader_path`s and dispatches on `kernels[].op` plus the
// fused circuit node of the same id (inputs, outputs, params, attrs).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "json.hpp"

namespace nerve {

enum class TensorStorage { BF16, INT4_CT, FP8_BLOCK, F32, OTHER };

struct TensorInfo {
    std::string name;
    std::string dtype;                 // BF16, I32, F8_E4M3, ...
    std::vector<int64_t> shape;        // physical shape
    std::vector<int64_t> logical_shape;  // [N, K] for packed tensors, else = shape
    std::string source_file;           // relative to the package directory
    uint64_t begin = 0, end = 0;       // data_offsets inside the safetensors data section
    std::string sha256;                // of the raw data bytes
    // quantisation (INT4 compressed-tensors pack-quantized)
    bool quantized = false;
    int bits = 0, group_size = 0, signed_offset = 0;
    std::string scales;
    uint64_t byte_count() const { return end - begin; }
};

enum class OpKind {
    RmsNorm,
    Linear,             // 1..3 branches sharing one input (linear / parallel_linear_{2,3}way)
    LinearResidual,
    LinearSiluMultiply,  // parallel_linear_silu_multiply (gate, up)
    QuantizeFp8,
    Rope,
    HeadNormRope,       // parallel_head_norm_rope_2way
    AppendAttention,
    ResidualAdd,
    SiluMultiply,
    Concat,
    MoeTopk,
    MoeGateUp,
    MoeDown,
    MoeReduce,
};

struct WeightRef {
    std::string tensor;       // weight tensor name
    std::string scale;        // INT4 scales / FP8 scale_inv tensor name (empty for BF16)
    TensorStorage storage = TensorStorage::BF16;
    int64_t n = 0, k = 0;     // logical [out, in]
    int group = 0;            // INT4 group size along K, FP8 block columns
    // tensor-parallel shard held by this process (n, k above are the shard's; the full tensor is full_n x full_k)
    int64_t full_n = 0, full_k = 0, row_begin = 0, col_begin = 0;
};

struct RopeAttrs {
    int heads = 0, head_width = 0, rotary_width = 0;
    bool interleaved = false;
    float theta = 10000.0f;
};

struct OpSpec {
    OpKind kind;
    std::string op_name;   // the manifest's op string
    std::string node_id;
    std::vector<std::string> inputs, outputs;
    std::vector<WeightRef> weights;       // Linear branches in output order; norm weights
    std::vector<std::string> norm_weights;  // RmsNorm / HeadNormRope weight tensors
    float eps = 0.0f, weight_offset = 0.0f;
    std::vector<RopeAttrs> rope;          // 1 (Rope) or 2 (HeadNormRope) branches
    int q_heads = 0, kv_heads = 0, head_width = 0;
    float attention_scale = 0.0f;
    int experts = 0, top_k = 0, moe_hidden = 0, moe_inter = 0;
    float routed_scale = 1.0f;
    bool residual_rounds_product = false;  // BF16 linear_residual rounds the product before the add
    std::string residual_input;
    bool prequantized_input = false;       // FP8 linears fed by a QuantizeFp8 op
    bool tp_partial = false;               // row-parallel linear: the output is a partial sum to all-reduce over the TP group
};

struct SignalInfo {
    int64_t width = 0;     // elements per lane
    int element_bytes = 2;
};

struct ComponentPlan {
    std::string id;
    std::string operator_type;
    std::vector<OpSpec> ops;
    std::map<std::string, SignalInfo> signals;
    std::vector<std::string> boundary_inputs;
    std::string boundary_output;
    // attention state declared by the component (at most one KV memory per layer)
    bool has_kv = false;
    int kv_heads = 0, head_width = 0, q_heads = 0;
};

struct TransducerPlan {
    std::string norm_tensor, projection_tensor;
    float eps = 1e-5f, weight_offset = 0.0f, logits_scale = 1.0f;
};

struct ModelPlan {
    int64_t hidden = 0, vocab = 0;
    int64_t max_context = 0;
    std::string embedding_tensor;
    float embedding_scale = 1.0f;
    std::vector<ComponentPlan> layers;
    TransducerPlan output;
    // sampler spec (package default; streams may override)
    std::string sampler_method = "greedy";
    float temperature = 1.0f, top_p = 1.0f, min_p = 0.0f;
    int top_k = 1;
    // speculative decoder (first entry of speculative_decoders[])
    bool has_draft = false;
    std::string draft_id;
    ComponentPlan draft_adapter;
    std::string adapter_token_signal, adapter_hidden_signal, adapter_output_signal;
    std::vector<ComponentPlan> draft_layers;
    TransducerPlan draft_output;
    std::vector<uint32_t> eos_token_ids;
};

enum class VerifyLevel { None = 0, Used = 1, All = 2 };

class HostPackage {
public:
    // Throws std::runtime_error with a message naming the offending file/field.
    static std::shared_ptr<HostPackage> open(const std::string &manifest_path_or_dir, VerifyLevel verify);

    const std::string &directory() const { return dir_; }
    const Json &manifest() const { return manifest_; }
    const ModelPlan &plan() const { return plan_; }
    const TensorInfo &tensor(const std::string &name) const;
    bool has_tensor(const std::string &name) const { return tensors_.count(name) != 0; }
    const std::map<std::string, TensorInfo> &tensors() const { return tensors_; }

    // Reads rows [row_begin, row_end) of a row-major tensor whose first dimension
    // is rows (byte-range read; the rest of the file is never touched).  With
    // verify, a full-tensor read checks data_sha256.
    std::vector<uint8_t> read_tensor(const std::string &name, bool verify) const;
    void read_tensor_range(const std::string &name, uint64_t byte_begin, uint64_t byte_count, void *out) const;

    // Number of files whose hash was checked at open().
    size_t verified_file_count() const { return verified_files_; }

private:
    void load(const std::string &path, VerifyLevel verify);
    void verify_artifacts(VerifyLevel verify);
    void build_plan();
    ComponentPlan build_component(const Json &execution, const Json &component);
    WeightRef weight_ref(const Json &refs, const std::string &param) const;
    void require_elements(const std::string &name, const std::string &dtype, uint64_t elements, const std::string &what) const;

    std::string dir_;
    Json manifest_;
    std::map<std::string, TensorInfo> tensors_;
    mutable std::map<std::string, uint64_t> data_base_;  // file -> 8 + header length
    ModelPlan plan_;
    size_t verified_files_ = 0;
};

// format(x, ".9g") parsed back to f32: the route every shader constant takes
// (nerve/model_package_shader_selection.py:1272-1273).
float shader_float(double value);

std::string read_file(const std::string &path);

}  // namespace nerve
