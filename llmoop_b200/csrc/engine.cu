#include "engine.hpp"
#include "state_abi.hpp"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace nerve {

namespace {

[[noreturn]] void fail(const std::string &message) { throw std::runtime_error(message); }

void cuda_check(cudaError_t status, const char *what) {
    if (status != cudaSuccess) fail(std::string(what) + ": " + cudaGetErrorString(status));
}

DeviceBuffer device_alloc(size_t bytes, bool zero = true) {
    DeviceBuffer buffer;
    buffer.bytes = bytes ? bytes : 16;
    cuda_check(cudaMalloc(&buffer.ptr, buffer.bytes), "cudaMalloc");
    if (zero) cuda_check(cudaMemset(buffer.ptr, 0, buffer.bytes), "cudaMemset");
    return buffer;
}

uint64_t now_ns() {
    return static_cast<uint64_t>(
        std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

uint32_t float_bits(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    return bits;
}

uint16_t host_f32_to_bf16(float value) {
    uint32_t bits = float_bits(value);
    uint32_t lsb = (bits >> 16) & 1u;
    return static_cast<uint16_t>((bits + 0x7fffu + lsb) >> 16);
}

void collect_component_tensors(const ComponentPlan &plan, std::set<std::string> &names) {
    for (const OpSpec &op : plan.ops) {
        for (const WeightRef &weight : op.weights) {
            names.insert(weight.tensor);
            if (!weight.scale.empty()) names.insert(weight.scale);
        }
        for (const std::string &name : op.norm_weights) names.insert(name);
    }
}

}  // namespace

// ---- tensor parallelism (vulkan_distributed/planning.rs:180-528 is the reference's only sharding; here the
// Megatron split of a dense layer: q/k/v and gate/up by output rows (whole heads), o and down by input columns
// (whole groups of 128), one all-reduce of f32 partial sums after o and after down; norms, embedding and the
// output projection are replicated).
void shard_linear_rows(WeightRef &w, int rank, int size, int64_t unit, const std::string &what) {
    w.full_n = w.n;
    w.full_k = w.k;
    try {
        tp_shard_range(w.full_n, unit, rank, size, w.row_begin, w.n);
    } catch (const std::exception &error) {
        fail("tensor-parallel mount: rows of the " + what + ": " + error.what());
    }
}
void shard_linear_columns(WeightRef &w, int rank, int size, const std::string &what) {
    w.full_n = w.n;
    w.full_k = w.k;
    try {
        tp_shard_range(w.full_k, 128, rank, size, w.col_begin, w.k);
    } catch (const std::exception &error) {
        fail("tensor-parallel mount: columns of the " + what + ": " + error.what());
    }
}

void shard_component(ComponentPlan &layer, int rank, int size) {
    static const OpKind expected[15] = {OpKind::RmsNorm, OpKind::Linear, OpKind::Linear, OpKind::Linear, OpKind::Rope, OpKind::Rope,
                                        OpKind::AppendAttention, OpKind::Linear, OpKind::ResidualAdd, OpKind::RmsNorm, OpKind::Linear,
                                        OpKind::Linear, OpKind::SiluMultiply, OpKind::Linear, OpKind::ResidualAdd};
    if (layer.ops.size() != 15) fail("tensor-parallel mount: component " + layer.id + " is not a dense layer of 15 kernels");
    for (int i = 0; i < 15; i++)
        if (layer.ops[i].kind != expected[i] || (layer.ops[i].kind == OpKind::Linear && layer.ops[i].weights.size() != 1))
            fail("tensor-parallel mount: component " + layer.id + " is not a dense layer of 15 kernels");
    for (int i : {1, 2, 3, 7, 10, 11, 13}) {
        TensorStorage storage = layer.ops[i].weights[0].storage;
        if (storage != TensorStorage::INT4_CT && storage != TensorStorage::BF16)
            fail("tensor-parallel mount: only INT4 and BF16 linears are sharded");
    }
    OpSpec &q = layer.ops[1], &k = layer.ops[2], &v = layer.ops[3], &rope_q = layer.ops[4], &rope_k = layer.ops[5], &attention = layer.ops[6],
           &o = layer.ops[7], &gate = layer.ops[10], &up = layer.ops[11], &silu = layer.ops[12], &down = layer.ops[13];
    const int head = attention.head_width;
    if (attention.q_heads % size != 0 || attention.kv_heads % size != 0)
        fail("tensor-parallel mount: " + std::to_string(attention.q_heads) + " query / " + std::to_string(attention.kv_heads) +
             " key-value heads do not divide over " + std::to_string(size) + " ranks");
    shard_linear_rows(q.weights[0], rank, size, head, "q projection");
    shard_linear_rows(k.weights[0], rank, size, head, "k projection");
    shard_linear_rows(v.weights[0], rank, size, head, "v projection");
    shard_linear_columns(o.weights[0], rank, size, "o projection");
    shard_linear_rows(gate.weights[0], rank, size, 16, "gate projection");
    shard_linear_rows(up.weights[0], rank, size, 16, "up projection");
    shard_linear_columns(down.weights[0], rank, size, "down projection");
    o.tp_partial = true;
    down.tp_partial = true;
    attention.q_heads /= size;
    attention.kv_heads /= size;
    for (OpSpec *rope : {&rope_q, &rope_k})
        for (RopeAttrs &attrs : rope->rope) attrs.heads /= size;
    layer.q_heads = attention.q_heads;
    layer.kv_heads = attention.kv_heads;
    auto set_width = [&](const std::string &signal, int64_t width) { layer.signals[signal].width = width; };
    set_width(q.outputs[0], q.weights[0].n);
    set_width(k.outputs[0], k.weights[0].n);
    set_width(v.outputs[0], v.weights[0].n);
    set_width(rope_q.outputs[0], q.weights[0].n);
    set_width(rope_k.outputs[0], k.weights[0].n);
    set_width(attention.outputs[0], q.weights[0].n);
    set_width(gate.outputs[0], gate.weights[0].n);
    set_width(up.outputs[0], up.weights[0].n);
    set_width(silu.outputs[0], gate.weights[0].n);
}

ModelPlan shard_plan(const ModelPlan &full, int rank, int size) {
    ModelPlan plan = full;
    if (size <= 1) return plan;
    if (rank < 0 || rank >= size) fail("tensor-parallel rank " + std::to_string(rank) + " outside 0.." + std::to_string(size - 1));
    for (ComponentPlan &layer : plan.layers) shard_component(layer, rank, size);
    for (ComponentPlan &layer : plan.draft_layers) shard_component(layer, rank, size);
    return plan;
}

// Rows [row_begin, row_begin + n) and columns [col_begin, col_begin + k) of a row-major [full_n][full_k] weight whose
// rows take `row_bytes` bytes; `per_column_num / per_column_den` bytes per column (INT4: 1/2, bf16: 2, a group
// scale: 2/128).
std::vector<uint8_t> slice_tensor(const std::vector<uint8_t> &data, const WeightRef &w, int64_t num, int64_t den) {
    if (w.full_n == 0) return data;
    const size_t full_row = static_cast<size_t>(w.full_k) * num / den, row = static_cast<size_t>(w.k) * num / den,
                 offset = static_cast<size_t>(w.col_begin) * num / den;
    if (data.size() != full_row * static_cast<size_t>(w.full_n)) fail("tensor-parallel mount: tensor " + w.tensor + " has an unexpected size");
    std::vector<uint8_t> out(row * static_cast<size_t>(w.n));
    for (int64_t r = 0; r < w.n; r++)
        std::memcpy(out.data() + static_cast<size_t>(r) * row, data.data() + static_cast<size_t>(w.row_begin + r) * full_row + offset, row);
    return out;
}

// ============================================================================ MountedModel

std::shared_ptr<MountedModel> MountedModel::mount(const std::string &path, const MountOptions &options) {
    if (options.page_tokens <= 0 || options.capacity_tokens <= 0 || options.max_streams <= 0 || options.max_lanes <= 0)
        fail("mount options must be positive");
    int device_count = 0;
    cuda_check(cudaGetDeviceCount(&device_count), "cudaGetDeviceCount");
    if (options.device < 0 || options.device >= device_count)
        fail("CUDA device " + std::to_string(options.device) + " is not present (" + std::to_string(device_count) + " visible)");
    cuda_check(cudaSetDevice(options.device), "cudaSetDevice");

    auto model = std::shared_ptr<MountedModel>(new MountedModel());
    model->options_ = options;
    VerifyLevel level = options.verify_level >= 2 ? VerifyLevel::All : (options.verify_level == 1 ? VerifyLevel::Used : VerifyLevel::None);
    model->package_ = HostPackage::open(path, level);
    model->plan_ = shard_plan(model->package_->plan(), options.tp_rank, options.tp_size);
    const ModelPlan &plan = model->plan_;
    if (plan.max_context > 0 && options.capacity_tokens > plan.max_context)
        fail("requested context " + std::to_string(options.capacity_tokens) + " exceeds the package's max_context_activations " +
             std::to_string(plan.max_context));

    model->upload_tensors();

    // paged KV pools: one per attention layer (target layers, then draft layers), all sharing one block table
    model->pages_per_stream_ = (options.capacity_tokens + options.page_tokens - 1) / options.page_tokens;
    model->physical_pages_ = model->pages_per_stream_ * options.max_streams + options.extra_pages;
    auto add_pool = [&](const ComponentPlan &component) {
        if (!component.has_kv) return;
        size_t page_bytes = static_cast<size_t>(2) * component.kv_heads * options.page_tokens * component.head_width * 2;
        model->kv_page_bytes_.push_back(page_bytes);
        model->kv_shapes_.emplace_back(component.kv_heads, component.head_width);
        model->kv_pools_.push_back(device_alloc(page_bytes * model->physical_pages_));
    };
    for (const ComponentPlan &layer : plan.layers) {
        add_pool(layer);
        if (layer.has_kv) model->kv_bytes_per_token_ += static_cast<uint64_t>(2) * layer.kv_heads * layer.head_width * 2;
    }
    for (const ComponentPlan &layer : plan.draft_layers) add_pool(layer);
    model->block_table_ = device_alloc(sizeof(int32_t) * options.max_streams * model->pages_per_stream_);
    model->build_rope_tables();
    cuda_check(cudaDeviceGetAttribute(&model->sm_count_, cudaDevAttrMultiProcessorCount, options.device), "cudaDeviceGetAttribute");
    // the output projection tables, once more in the order the streaming kernel reads them
    for (const std::string &name : {plan.output.projection_tensor, plan.has_draft ? plan.draft_output.projection_tensor : std::string()}) {
        if (name.empty() || model->projection_tables_.count(name) || !output_projection_supported(1, static_cast<int>(plan.hidden))) continue;
        DeviceBuffer table = device_alloc(projection_table_bytes(static_cast<int>(plan.vocab), static_cast<int>(plan.hidden)), false);
        cuda_check(launch_projection_table(static_cast<const uint16_t *>(model->tensor(name)), table.ptr, static_cast<int>(plan.vocab),
                                           static_cast<int>(plan.hidden), nullptr),
                   "output projection table copy");
        model->projection_tables_.emplace(name, table);
    }
    // ... and the bf16 linears of the draft adapter (one launch per draft step each, a single lane wide)
    if (plan.has_draft) {
        for (const OpSpec &op : plan.draft_adapter.ops) {
            if (op.kind != OpKind::Linear) continue;
            for (const WeightRef &w : op.weights) {
                if (w.storage != TensorStorage::BF16 || w.n < 256 || model->projection_tables_.count(w.tensor) ||
                    !output_projection_supported(1, static_cast<int>(w.k)))
                    continue;
                DeviceBuffer table = device_alloc(projection_table_bytes(static_cast<int>(w.n), static_cast<int>(w.k)), false);
                cuda_check(launch_projection_table(static_cast<const uint16_t *>(model->tensor(w.tensor)), table.ptr, static_cast<int>(w.n),
                                                   static_cast<int>(w.k), nullptr),
                           "linear table copy");
                model->projection_tables_.emplace(w.tensor, table);
            }
        }
    }
    cuda_check(cudaDeviceSynchronize(), "output projection table copies");
    {
        int target_kv_layers = 0;
        for (const ComponentPlan &layer : plan.layers) target_kv_layers += layer.has_kv ? 1 : 0;
        model->build_stack(plan.layers, 0, model->target_stack_);
        if (plan.has_draft) model->build_stack(plan.draft_layers, target_kv_layers, model->draft_stack_);
    }
    return model;
}

MountedModel::~MountedModel() {
    for (auto &entry : tensors_) cudaFree(entry.second.ptr);
    for (auto &pool : kv_pools_) cudaFree(pool.ptr);
    for (auto &entry : rope_tables_) cudaFree(entry.second.ptr);
    for (auto &entry : projection_tables_) cudaFree(entry.second.ptr);
    for (StackPlan *stack : {&target_stack_, &draft_stack_}) {
        for (DeviceBuffer &buffer : stack->storage) cudaFree(buffer.ptr);
        cudaFree(stack->device_layers.ptr);
    }
    cudaFree(block_table_.ptr);
}

const void *MountedModel::tensor(const std::string &name) const {
    auto found = tensors_.find(name);
    if (found == tensors_.end()) fail("tensor " + name + " is not resident on the device");
    return found->second.ptr;
}

void MountedModel::upload_tensors() {
    const ModelPlan &plan = plan_;
    // which linears hold only a tensor-parallel shard of their weight (and scales)
    std::map<std::string, std::pair<WeightRef, std::pair<int64_t, int64_t>>> shards;  // tensor -> (ref, bytes per column as a fraction)
    auto note = [&](const ComponentPlan &component) {
        for (const OpSpec &op : component.ops)
            for (const WeightRef &w : op.weights)
                if (w.full_n != 0) {
                    if (w.storage == TensorStorage::INT4_CT) {
                        shards[w.tensor] = {w, {1, 2}};
                        shards[w.scale] = {w, {2, 128}};
                    } else {
                        shards[w.tensor] = {w, {2, 1}};
                    }
                }
    };
    for (const ComponentPlan &layer : plan.layers) note(layer);
    for (const ComponentPlan &layer : plan.draft_layers) note(layer);
    std::set<std::string> target, draft, shared;
    for (const ComponentPlan &layer : plan.layers) collect_component_tensors(layer, target);
    target.insert(plan.output.norm_tensor);
    target.insert(plan.output.projection_tensor);
    shared.insert(plan.embedding_tensor);
    if (plan.has_draft) {
        collect_component_tensors(plan.draft_adapter, draft);
        for (const ComponentPlan &layer : plan.draft_layers) collect_component_tensors(layer, draft);
        draft.insert(plan.draft_output.norm_tensor);
        draft.insert(plan.draft_output.projection_tensor);
    }
    std::set<std::string> all = target;
    all.insert(draft.begin(), draft.end());
    all.insert(shared.begin(), shared.end());
    const bool verify = options_.verify_level >= 1;
    for (const std::string &name : all) {
        std::vector<uint8_t> data = package_->read_tensor(name, verify);
        auto shard = shards.find(name);
        if (shard != shards.end()) data = slice_tensor(data, shard->second.first, shard->second.second.first, shard->second.second.second);
        DeviceBuffer buffer = device_alloc(data.size(), false);
        cuda_check(cudaMemcpy(buffer.ptr, data.data(), data.size(), cudaMemcpyHostToDevice), "weight upload");
        tensors_[name] = buffer;
        weight_bytes_ += data.size();
    }
    for (const std::string &name : target) target_step_bytes_ += tensors_.at(name).bytes;
    for (const std::string &name : draft) draft_step_bytes_ += tensors_.at(name).bytes;
}

void MountedModel::build_rope_tables() {
    const ModelPlan &plan = plan_;
    rope_positions_ = static_cast<uint32_t>(std::max<int64_t>(plan.max_context, options_.capacity_tokens)) + 64;
    auto add = [&](const ComponentPlan &component) {
        for (const OpSpec &op : component.ops)
            for (const RopeAttrs &rope : op.rope) {
                auto key = std::make_pair(float_bits(rope.theta), rope.rotary_width);
                if (rope_tables_.count(key)) continue;
                // Same f32 sequence as rotary_bf16.comp.template:67-109: inv_freq = pow(theta, -2 f / rotary),
                // angle = float(position) * inv_freq, cos and sin each rounded to bf16.
                int half = rope.rotary_width / 2;
                std::vector<uint32_t> table(static_cast<size_t>(rope_positions_) * half);
                for (uint32_t position = 0; position < rope_positions_; position++)
                    for (int f = 0; f < half; f++) {
                        float inv_freq = powf(rope.theta, -2.0f * static_cast<float>(f) / static_cast<float>(rope.rotary_width));
                        float angle = static_cast<float>(position) * inv_freq;
                        uint32_t cosine = host_f32_to_bf16(cosf(angle) * 1.0f), sine = host_f32_to_bf16(sinf(angle) * 1.0f);
                        table[static_cast<size_t>(position) * half + f] = (sine << 16) | cosine;
                    }
                DeviceBuffer buffer = device_alloc(table.size() * sizeof(uint32_t), false);
                cuda_check(cudaMemcpy(buffer.ptr, table.data(), table.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "rope table upload");
                rope_tables_[key] = buffer;
            }
    };
    for (const ComponentPlan &layer : plan.layers) add(layer);
    for (const ComponentPlan &layer : plan.draft_layers) add(layer);
}

// Recognises the kernel list of a dense Llama-style layer whose seven linears are INT4 g128
// (rms_norm, q, k, v, rope q, rope k, append attention, o, residual, rms_norm, gate, up, silu*up, down, residual)
// and makes the tile-major weight copies the persistent decode kernel streams.
void MountedModel::build_stack(const std::vector<ComponentPlan> &layers, int first_kv_index, StackPlan &out) {
    out = StackPlan{};
    auto refuse = [&](const std::string &why) {
        out.reason = why;
        if (getenv("NERVE_B200_VERBOSE")) fprintf(stderr, "nerve_b200: decode stack kernel not used: %s\n", why.c_str());
    };
    if (layers.empty()) return refuse("no layers");
    auto int4 = [](const OpSpec &op) {
        return op.kind == OpKind::Linear && op.weights.size() == 1 && op.weights[0].storage == TensorStorage::INT4_CT &&
               op.weights[0].group == 128;
    };
    static const OpKind expected[15] = {OpKind::RmsNorm, OpKind::Linear, OpKind::Linear, OpKind::Linear, OpKind::Rope, OpKind::Rope,
                                        OpKind::AppendAttention, OpKind::Linear, OpKind::ResidualAdd, OpKind::RmsNorm, OpKind::Linear,
                                        OpKind::Linear, OpKind::SiluMultiply, OpKind::Linear, OpKind::ResidualAdd};
    StackShape shape{};
    int kv_index = first_kv_index;
    std::vector<StackLayer> built;
    std::vector<DeviceBuffer> storage;
    uint64_t bytes = 0;
    auto drop = [&]() {
        for (DeviceBuffer &buffer : storage) cudaFree(buffer.ptr);
    };
    for (size_t index = 0; index < layers.size(); index++) {
        const ComponentPlan &layer = layers[index];
        if (layer.ops.size() != 15 || !layer.has_kv || layer.boundary_inputs.size() != 1) return drop(), refuse("layer is not the dense 15-kernel form");
        for (int i = 0; i < 15; i++)
            if (layer.ops[i].kind != expected[i]) return drop(), refuse("layer kernel " + std::to_string(i) + " differs from the dense form");
        const OpSpec &norm1 = layer.ops[0], &q = layer.ops[1], &k = layer.ops[2], &v = layer.ops[3], &rope_q = layer.ops[4], &rope_k = layer.ops[5],
                     &attention = layer.ops[6], &o = layer.ops[7], &add1 = layer.ops[8], &norm2 = layer.ops[9], &gate = layer.ops[10],
                     &up = layer.ops[11], &silu = layer.ops[12], &down = layer.ops[13], &add2 = layer.ops[14];
        for (const OpSpec *linear : {&q, &k, &v, &o, &gate, &up, &down})
            if (!int4(*linear)) return drop(), refuse("a linear of the layer is not INT4 g128");
        const std::string &input = layer.boundary_inputs[0];
        auto is_pair = [](const OpSpec &add, const std::string &a, const std::string &b) {
            return add.inputs.size() == 2 && ((add.inputs[0] == a && add.inputs[1] == b) || (add.inputs[0] == b && add.inputs[1] == a));
        };
        bool wired = norm1.inputs[0] == input && q.inputs[0] == norm1.outputs[0] && k.inputs[0] == norm1.outputs[0] &&
                     v.inputs[0] == norm1.outputs[0] && rope_q.inputs[0] == q.outputs[0] && rope_k.inputs[0] == k.outputs[0] &&
                     attention.inputs.size() >= 3 && attention.inputs[0] == rope_q.outputs[0] && attention.inputs[1] == rope_k.outputs[0] &&
                     attention.inputs[2] == v.outputs[0] && o.inputs[0] == attention.outputs[0] && is_pair(add1, o.outputs[0], input) &&
                     norm2.inputs[0] == add1.outputs[0] && gate.inputs[0] == norm2.outputs[0] && up.inputs[0] == norm2.outputs[0] &&
                     silu.inputs.size() == 2 && silu.inputs[0] == gate.outputs[0] && silu.inputs[1] == up.outputs[0] &&
                     down.inputs[0] == silu.outputs[0] && is_pair(add2, down.outputs[0], add1.outputs[0]) &&
                     add2.outputs[0] == layer.boundary_output;
        if (!wired) return drop(), refuse("layer wiring differs from the dense form");
        if (rope_q.rope.size() != 1 || rope_k.rope.size() != 1) return drop(), refuse("rotary attributes missing");
        const RopeAttrs &rq = rope_q.rope[0], &rk = rope_k.rope[0];
        StackShape here{};
        here.hidden = static_cast<int>(q.weights[0].k);
        here.q_heads = attention.q_heads;
        here.kv_heads = attention.kv_heads;
        here.head_width = attention.head_width;
        here.ffn = static_cast<int>(gate.weights[0].n);
        here.eps = norm1.eps;
        here.norm_offset = norm1.weight_offset;
        here.attention_scale = attention.attention_scale;
        bool dims = rq.head_width == here.head_width && rk.head_width == here.head_width && rq.rotary_width == here.head_width &&
                    rk.rotary_width == here.head_width && !rq.interleaved && !rk.interleaved && float_bits(rq.theta) == float_bits(rk.theta) &&
                    rq.heads == here.q_heads && rk.heads == here.kv_heads && q.weights[0].n == int64_t(here.q_heads) * here.head_width &&
                    k.weights[0].n == int64_t(here.kv_heads) * here.head_width && v.weights[0].n == k.weights[0].n &&
                    k.weights[0].k == here.hidden && v.weights[0].k == here.hidden && o.weights[0].k == q.weights[0].n &&
                    o.weights[0].n == here.hidden && gate.weights[0].k == here.hidden && up.weights[0].k == here.hidden &&
                    up.weights[0].n == here.ffn && down.weights[0].k == here.ffn && down.weights[0].n == here.hidden &&
                    float_bits(norm2.eps) == float_bits(norm1.eps) && float_bits(norm2.weight_offset) == float_bits(norm1.weight_offset) &&
                    here.head_width % 16 == 0 && here.hidden % 128 == 0 && here.ffn % 128 == 0 && (here.q_heads * here.head_width) % 128 == 0 &&
                    layer.kv_heads == here.kv_heads && layer.head_width == here.head_width;
        if (!dims) return drop(), refuse("layer dimensions or rotary form are outside the decode stack kernel");
        here.rope_table = rope_table(rq.theta, rq.rotary_width);
        here.rope_positions = rope_positions_;
        here.grid = sm_count_;
        if (index == 0) shape = here;
        else if (std::memcmp(&shape, &here, sizeof(StackShape)) != 0) return drop(), refuse("layers differ in shape");
        size_t unused = 0;
        if (!decode_stack_supported(shape, 1, &unused)) return drop(), refuse("no decode stack kernel instance for this head shape");

        auto streamed = [&](std::initializer_list<const OpSpec *> sources, bool pair, bool rope_first_two) {
            RelayoutSegment segments[3];
            int count = 0, rows = 0;
            const int kk = static_cast<int>((*sources.begin())->weights[0].k);
            for (const OpSpec *source : sources) {
                const WeightRef &w = source->weights[0];
                segments[count].qweight = static_cast<const uint32_t *>(tensor(w.tensor));
                segments[count].scales = static_cast<const uint16_t *>(tensor(w.scale));
                segments[count].rows = static_cast<int>(w.n);
                segments[count].rope_head_width = (rope_first_two && count < 2) ? here.head_width : 0;
                if (!pair || count == 0) rows += static_cast<int>(w.n);
                count++;
            }
            DeviceBuffer stream = device_alloc(std::max<size_t>(16, int4_cta_stream_bytes(rows, kk, pair, here.grid)), false);
            storage.push_back(stream);
            cuda_check(launch_int4_cta_streams(segments, count, pair, kk, here.grid, static_cast<uint8_t *>(stream.ptr), nullptr), "per-CTA INT4 stream copy");
            bytes += stream.bytes;
            return static_cast<const uint8_t *>(stream.ptr);
        };
        StackLayer spec{};
        spec.qkv = streamed({&q, &k, &v}, false, true);
        spec.o = streamed({&o}, false, false);
        spec.gate_up = streamed({&gate, &up}, true, false);
        spec.down = streamed({&down}, false, false);
        spec.input_norm = static_cast<const uint16_t *>(tensor(norm1.norm_weights[0]));
        spec.post_norm = static_cast<const uint16_t *>(tensor(norm2.norm_weights[0]));
        spec.kv = kv_layer(kv_index++);
        bytes += 2 * static_cast<uint64_t>(here.hidden) * 2;
        built.push_back(spec);
    }
    cuda_check(cudaDeviceSynchronize(), "per-CTA INT4 stream copies");
    out.available = true;
    out.shape = shape;
    out.layers = built;
    out.storage = storage;
    out.weight_bytes = bytes;
    out.device_layers = device_alloc(built.size() * sizeof(StackLayer), false);
    cuda_check(cudaMemcpy(out.device_layers.ptr, built.data(), built.size() * sizeof(StackLayer), cudaMemcpyHostToDevice), "stack layer table upload");
}

const uint32_t *MountedModel::rope_table(float theta, int rotary) const {
    auto found = rope_tables_.find(std::make_pair(float_bits(theta), rotary));
    if (found == rope_tables_.end()) fail("no RoPE table for this theta/rotary width");
    return static_cast<const uint32_t *>(found->second.ptr);
}

KvLayer MountedModel::kv_layer(int index) const {
    KvLayer layer;
    layer.pool = static_cast<uint16_t *>(kv_pools_.at(index).ptr);
    layer.block_table = static_cast<const int32_t *>(block_table_.ptr);
    layer.pages_per_slot = pages_per_stream_;
    layer.page_tokens = options_.page_tokens;
    layer.kv_heads = kv_shapes_[index].first;
    layer.head_width = kv_shapes_[index].second;
    layer.capacity = capacity();
    return layer;
}

// ============================================================================ Engine

namespace {
constexpr int MAX_STOP_TOKENS = 8;
}

// ---- NCCL through its C ABI, loaded at run time (ncclUniqueId is 128 bytes; ncclFloat32 = 7, ncclSum = 0)
namespace {
struct NcclApi {
    int (*get_unique_id)(void *id);
    int (*comm_init_rank)(void **comm, int size, const void *id_by_value_128, int rank);
    int (*all_reduce)(const void *send, void *recv, size_t count, int datatype, int op, void *comm, cudaStream_t stream);
    int (*comm_destroy)(void *comm);
    const char *(*get_error_string)(int result);
};
struct NcclId {
    char bytes[128];
};
void *open_nccl(const std::string &library, NcclApi &api) {
    void *handle = dlopen(library.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (handle == nullptr) fail("cannot load NCCL from " + library + ": " + dlerror());
    auto need = [&](const char *name) {
        void *symbol = dlsym(handle, name);
        if (symbol == nullptr) fail(std::string("NCCL library lacks ") + name);
        return symbol;
    };
    api.get_unique_id = reinterpret_cast<int (*)(void *)>(need("ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<int (*)(void **, int, const void *, int)>(need("ncclCommInitRank"));
    api.all_reduce = reinterpret_cast<int (*)(const void *, void *, size_t, int, int, void *, cudaStream_t)>(need("ncclAllReduce"));
    api.comm_destroy = reinterpret_cast<int (*)(void *)>(need("ncclCommDestroy"));
    api.get_error_string = reinterpret_cast<const char *(*)(int)>(need("ncclGetErrorString"));
    return handle;
}
NcclApi g_nccl{};
}  // namespace

Engine::Engine(std::shared_ptr<MountedModel> model) : model_(std::move(model)) {
    const MountOptions &options = model_->options();
    const ModelPlan &plan = model_->plan();
    cuda_check(cudaSetDevice(options.device), "cudaSetDevice");
    cuda_check(cudaStreamCreateWithFlags(&cuda_stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaEventCreate(&event_a_), "cudaEventCreate");
    cuda_check(cudaEventCreate(&event_b_), "cudaEventCreate");
    cuda_check(cudaEventCreate(&event_begin_), "cudaEventCreate");
    cuda_check(cudaEventCreate(&run_begin_), "cudaEventCreate");
    cuda_check(cudaEventCreate(&run_end_), "cudaEventCreate");
    cuda_check(cudaEventCreate(&event_end_), "cudaEventCreate");
    const size_t lanes = options.max_lanes;
    const size_t frame = static_cast<size_t>(plan.hidden) * 2;

    auto declare = [&](const ComponentPlan &component) {
        for (const auto &entry : component.signals) {
            size_t bytes = lanes * entry.second.width * entry.second.element_bytes;
            auto found = signals_.find(entry.first);
            if (found == signals_.end()) signals_[entry.first] = DeviceBuffer{nullptr, bytes};
            else found->second.bytes = std::max(found->second.bytes, bytes);
        }
    };
    for (const ComponentPlan &layer : plan.layers) declare(layer);
    if (plan.has_draft) {
        declare(plan.draft_adapter);
        for (const ComponentPlan &layer : plan.draft_layers) declare(layer);
    }
    for (auto &entry : signals_) entry.second = device_alloc(entry.second.bytes);

    frame_a_ = device_alloc(lanes * frame);
    frame_b_ = device_alloc(lanes * frame);
    embedding_out_ = device_alloc(lanes * frame);
    normalized_ = device_alloc(lanes * frame);
    draft_normalized_ = device_alloc(lanes * frame);
    draft_hidden_in_ = device_alloc(lanes * frame);
    logits_ = device_alloc(lanes * static_cast<size_t>(plan.vocab) * sizeof(float));
    records_ = device_alloc(lanes * 4 * sizeof(uint32_t));
    argmax_scratch_ = device_alloc(argmax_scratch_bytes(options.max_lanes));
    sampler_table_ = device_alloc(static_cast<size_t>(options.max_streams) * sizeof(SamplerParams));
    lane_tokens_ = device_alloc(lanes * sizeof(uint32_t));
    lane_positions_ = device_alloc(lanes * sizeof(uint32_t));
    lane_slots_ = device_alloc(lanes * sizeof(int32_t));
    pending_hidden_ = device_alloc(static_cast<size_t>(options.max_streams) * frame);
    pending_backup_ = device_alloc(static_cast<size_t>(options.max_streams) * frame);

    split_tokens_ = 64;
    max_splits_ = static_cast<int>((model_->capacity() + split_tokens_ - 1) / split_tokens_);
    int max_q_heads = 1, max_head_width = 1;
    auto scan = [&](const ComponentPlan &component) {
        if (component.has_kv) {
            max_q_heads = std::max(max_q_heads, component.q_heads);
            max_head_width = std::max(max_head_width, component.head_width);
        }
    };
    for (const ComponentPlan &layer : plan.layers) scan(layer);
    for (const ComponentPlan &layer : plan.draft_layers) scan(layer);
    // Scratch of the split attention.  The persistent kernel (at most eight lanes) takes 64-token splits over the
    // whole ring.  The kernel-per-operator path takes splits of a length fixed per engine - 64 tokens where the
    // partials of the largest batch over the whole ring fit 1 GB, else the next multiple of 64 that makes them fit
    // (a prefill chunk of 2048 lanes over a 32K ring: 1152 tokens), walked tile by tile inside the kernel - so the
    // arithmetic of a lane never depends on which batch it runs in.
    max_q_heads_ = max_q_heads;
    const size_t partial_bytes = static_cast<size_t>(max_head_width + 2) * sizeof(float);
    const size_t budget = (size_t(1) << 30) / partial_bytes;
    const size_t all = static_cast<size_t>(options.max_lanes) * max_q_heads * max_splits_;
    const int factor = static_cast<int>(std::max<size_t>(1, (all + budget - 1) / budget));
    op_split_tokens_ = split_tokens_ * factor;
    const size_t op_splits = (model_->capacity() + op_split_tokens_ - 1) / op_split_tokens_;
    // (the persistent kernel merges rows of more than 32 splits in two levels: one more partial per 32 splits)
    const size_t small_batches = static_cast<size_t>(std::min(options.max_lanes, 8)) * max_q_heads * (max_splits_ + (max_splits_ + 31) / 32);
    attention_scratch_ = device_alloc(std::max(small_batches, static_cast<size_t>(options.max_lanes) * max_q_heads * op_splits) * partial_bytes);

    // cycle arrays: verify tokens, forced drafts, stop tokens/counts, accept rows, per-step draft tokens, slots
    cycle_state_ = device_alloc(lanes * 64 * sizeof(uint32_t) + static_cast<size_t>(options.max_streams) * (MAX_STOP_TOKENS + 64) * sizeof(uint32_t) * 4);

    staging_bytes_ = std::max<size_t>(size_t(1) << 20, lanes * 1024 + static_cast<size_t>(options.max_streams) * model_->pages_per_stream() * 8);
    cuda_check(cudaMallocHost(&staging_, staging_bytes_), "cudaMallocHost");
    cuda_check(cudaMallocHost(&host_records_, lanes * 64 * sizeof(uint32_t)), "cudaMallocHost");

    kernel_error_ = device_alloc(sizeof(int));
    if (options.tp_size > 1) tp_partial_ = device_alloc(lanes * static_cast<size_t>(plan.hidden) * sizeof(float));
    {
        size_t q_width = 0, ffn = 0;
        for (const StackPlan *stack : {&model_->target_stack(), &model_->draft_stack()})
            if (stack->available) {
                q_width = std::max<size_t>(q_width, static_cast<size_t>(stack->shape.q_heads) * stack->shape.head_width);
                ffn = std::max<size_t>(ffn, stack->shape.ffn);
            }
        if (q_width != 0) {
            stack_q_ = device_alloc(8 * q_width * 2);
            stack_attention_out_ = device_alloc(8 * q_width * 2);
            stack_activation_ = device_alloc(8 * ffn * 2);
            stack_barrier_ = device_alloc(STACK_BARRIER_WORDS * sizeof(unsigned int));
            stack_timing_ = device_alloc(std::max<size_t>(1, plan.layers.size()) * 32 * sizeof(unsigned long long));
        }
    }

    for (int slot = options.max_streams - 1; slot >= 0; slot--) free_slots_.push_back(slot);
    for (int page = model_->physical_pages() - 1; page >= 0; page--) free_pages_.push_back(page);
    page_refcount_.assign(model_->physical_pages(), 0);
    block_table_host_.assign(static_cast<size_t>(options.max_streams) * model_->pages_per_stream(), 0);
}

Engine::~Engine() {
    cudaStreamSynchronize(cuda_stream_);
    if (nccl_comm_ != nullptr) g_nccl.comm_destroy(nccl_comm_);
    for (void *mapping : tp_peer_mappings_) cudaIpcCloseMemHandle(mapping);
    for (auto &entry : signals_) cudaFree(entry.second.ptr);
    for (DeviceBuffer *buffer : {&frame_a_, &frame_b_, &embedding_out_, &normalized_, &draft_normalized_, &draft_hidden_in_, &logits_,
                                 &records_, &argmax_scratch_, &sampler_scratch_, &sampler_table_, &lane_tokens_, &lane_positions_, &lane_slots_, &pending_hidden_, &pending_backup_, &attention_scratch_,
                                 &cycle_state_, &kernel_error_, &tp_partial_, &tp_exchange_, &tp_description_, &stack_q_, &stack_attention_out_, &stack_activation_, &stack_barrier_, &stack_timing_, &prefix_pending_})
        cudaFree(buffer->ptr);
    cudaFreeHost(staging_);
    cudaFreeHost(host_records_);
    for (cudaEvent_t event : profile_events_) cudaEventDestroy(event);
    for (auto &entry : graphs_)
        if (entry.second.exec) cudaGraphExecDestroy(entry.second.exec);
    cudaEventDestroy(event_a_);
    cudaEventDestroy(event_b_);
    cudaEventDestroy(event_begin_);
    cudaEventDestroy(run_begin_);
    cudaEventDestroy(run_end_);
    cudaEventDestroy(event_end_);
    cudaStreamDestroy(cuda_stream_);
}

void Engine::tensor_parallel_unique_id(const std::string &library, uint8_t *out_128_bytes) {
    NcclApi api{};
    open_nccl(library, api);  // stays loaded: the communicator is made from the same library
    NcclId id{};
    int result = api.get_unique_id(&id);
    if (result != 0) fail(std::string("ncclGetUniqueId: ") + api.get_error_string(result));
    std::memcpy(out_128_bytes, id.bytes, 128);
}

void Engine::init_tensor_parallel(const std::string &library, int rank, int size, const uint8_t *unique_id_128_bytes) {
    const MountOptions &options = model_->options();
    if (size != options.tp_size || rank != options.tp_rank)
        fail("tensor-parallel group (" + std::to_string(rank) + " of " + std::to_string(size) + ") differs from the mounted shard (" +
             std::to_string(options.tp_rank) + " of " + std::to_string(options.tp_size) + ")");
    if (size <= 1) return;
    if (nccl_comm_ != nullptr) fail("tensor parallelism is already initialised");
    cuda_check(cudaSetDevice(options.device), "cudaSetDevice");
    nccl_library_ = open_nccl(library, g_nccl);
    NcclId id{};
    std::memcpy(id.bytes, unique_id_128_bytes, 128);
    // ncclCommInitRank takes the id by value: a 128-byte struct is passed in memory, which is how this call passes it
    using InitByValue = int (*)(void **, int, NcclId, int);
    int result = reinterpret_cast<InitByValue>(g_nccl.comm_init_rank)(&nccl_comm_, size, id, rank);
    if (result != 0) fail(std::string("ncclCommInitRank: ") + g_nccl.get_error_string(result));
}

namespace {
size_t tp_exchange_bytes(size_t hidden) { return stack_tp_exchange_floats(static_cast<int>(hidden)) * sizeof(float); }
}  // namespace

void Engine::tp_exchange_handle(uint8_t *out_64_bytes) {
    const MountOptions &options = model_->options();
    if (options.tp_size <= 1) fail("this package was not mounted as a tensor-parallel shard");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "inter-process memory handles are 64 bytes");
    cuda_check(cudaSetDevice(options.device), "cudaSetDevice");
    if (!tp_exchange_.ptr) tp_exchange_ = device_alloc(tp_exchange_bytes(model_->plan().hidden) + STACK_TP_CONTROL_BYTES);  // zeroed
    cudaIpcMemHandle_t handle;
    cuda_check(cudaIpcGetMemHandle(&handle, tp_exchange_.ptr), "cudaIpcGetMemHandle");
    std::memcpy(out_64_bytes, &handle, sizeof(handle));
}

void Engine::tp_connect(const uint8_t *handles_64_bytes_each, int count) {
    const MountOptions &options = model_->options();
    if (count != options.tp_size || count > STACK_TP_MAX_RANKS) fail("tp_connect needs one handle per rank of the mounted group (at most 8)");
    if (!tp_exchange_.ptr) fail("call tp_exchange_handle before tp_connect");
    if (tp_connected_) fail("the tensor-parallel exchange is already connected");
    cuda_check(cudaSetDevice(options.device), "cudaSetDevice");
    const size_t floats = stack_tp_exchange_floats(static_cast<int>(model_->plan().hidden));
    StackTp description;
    description.rank = options.tp_rank;
    description.size = options.tp_size;
    for (int r = 0; r < count; r++) {
        void *base = tp_exchange_.ptr;
        if (r != options.tp_rank) {
            cudaIpcMemHandle_t handle;
            std::memcpy(&handle, handles_64_bytes_each + static_cast<size_t>(r) * 64, sizeof(handle));
            cuda_check(cudaIpcOpenMemHandle(&base, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle (is peer access between the GPUs available?)");
            tp_peer_mappings_.push_back(base);
        }
        description.exchange[r] = static_cast<float *>(base);
        description.counter[r] = reinterpret_cast<unsigned long long *>(static_cast<float *>(base) + floats);
    }
    tp_description_ = device_alloc(sizeof(StackTp));
    cuda_check(cudaMemcpy(tp_description_.ptr, &description, sizeof(description), cudaMemcpyHostToDevice), "exchange description upload");
    tp_connected_ = true;
}

void Engine::tp_all_reduce(float *values, size_t count) {
    if (nccl_comm_ == nullptr) fail("this package was mounted as a tensor-parallel shard: call init_tensor_parallel before running");
    int result = g_nccl.all_reduce(values, values, count, 7 /* ncclFloat32 */, 0 /* ncclSum */, nccl_comm_, cuda_stream_);
    if (result != 0) fail(std::string("ncclAllReduce: ") + g_nccl.get_error_string(result));
    counters_.kernel_launches++;
}

void Engine::check(cudaError_t status, const char *what) {
    counters_.kernel_launches++;
    cuda_check(status, what);
}

Engine::Stream &Engine::stream(int64_t id) {
    auto found = streams_.find(id);
    if (found == streams_.end()) fail("unknown stream " + std::to_string(id));
    return found->second;
}
const Engine::Stream &Engine::stream(int64_t id) const {
    auto found = streams_.find(id);
    if (found == streams_.end()) fail("unknown stream " + std::to_string(id));
    return found->second;
}

uint64_t Engine::stream_tick(int64_t id) const { return stream(id).next_tick; }

void Engine::add_stream(int64_t id, uint32_t seed, int speculative_draft_tokens, const SamplerConfig &sampler) {
    register_stream(id, seed, speculative_draft_tokens, sampler);
    scheduler_.add_stream(scheduler_id(id));
}

void Engine::rejoin_scheduler(int64_t id) {
    const std::string name = scheduler_id(id);
    carried_activations_.erase(std::remove_if(carried_activations_.begin(), carried_activations_.end(),
                                              [&](const runtime::Activation &activation) { return activation.stream_id == name; }),
                               carried_activations_.end());
    scheduler_.interrupt_stream(name, "the stream's events were dropped");  // also forgets activations in flight
    scheduler_.remove_stream(name);
    scheduler_.add_stream(name);
}

void Engine::register_stream(int64_t id, uint32_t seed, int speculative_draft_tokens, const SamplerConfig &sampler) {
    if (streams_.count(id)) fail("stream " + std::to_string(id) + " already exists");
    if (free_slots_.empty()) fail("no free stream slot (max_streams = " + std::to_string(model_->options().max_streams) + ")");
    if (sampler.method != 0 && sampler.method != 1) fail("sampler method must be 0 (greedy) or 1 (temperature_top_k_top_p)");
    if (sampler.method == 1) {
        if (!(sampler.temperature > 0.0f)) fail("sampler temperature must be positive");
        if (sampler.top_k < 1 || sampler.top_k > SAMPLER_MAX_TOP_K)
            fail("sampler top_k must be between 1 and " + std::to_string(SAMPLER_MAX_TOP_K));
        if (!(sampler.top_p > 0.0f) || sampler.top_p > 1.0f || sampler.min_p < 0.0f || sampler.min_p > 1.0f)
            fail("sampler top_p must be in (0, 1] and min_p in [0, 1]");
    }
    if (speculative_draft_tokens < 0) fail("speculative_draft_tokens must be >= 0");
    if (speculative_draft_tokens > 0 && !model_->plan().has_draft)
        fail("resident model package has no mounted speculative decoder");
    Stream s;
    s.id = id;
    s.slot = free_slots_.back();
    free_slots_.pop_back();
    s.seed = seed;
    s.k = speculative_draft_tokens;
    s.sampler = sampler;
    {
        SamplerParams params{};
        params.method = static_cast<uint32_t>(sampler.method);
        params.top_k = static_cast<uint32_t>(sampler.method == 1 ? sampler.top_k : 1);
        params.seed = seed;
        params.temperature = sampler.temperature;
        params.top_p = sampler.top_p;
        params.min_p = sampler.min_p;
        upload(static_cast<uint8_t *>(sampler_table_.ptr) + static_cast<size_t>(s.slot) * sizeof(SamplerParams), &params, sizeof(params),
               "sampler parameters upload");
        if (sampler.method != 0) {
            stochastic_streams_++;
            if (sampler_scratch_.ptr == nullptr) sampler_scratch_ = device_alloc(sampler_scratch_bytes(model_->options().max_lanes), false);
        }
    }
    s.pages.assign(model_->pages_per_stream(), -1);
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    cuda_check(cudaMemsetAsync(static_cast<uint8_t *>(pending_hidden_.ptr) + s.slot * frame, 0, frame, cuda_stream_), "pending reset");
    streams_.emplace(id, std::move(s));
}

void Engine::release_pages(Stream &s) {
    for (int32_t &page : s.pages) {
        if (page >= 0 && --page_refcount_[page] == 0) free_pages_.push_back(page);
        page = -1;
    }
    s.block_table_dirty = true;
}

// Output projection + sampler of `lanes` normalised rows (output transducer: tied_output_projection_batch_bf16.comp.template:52-142,
// then the sampler dispatch).  A tensor-parallel group with the peer exchange connected and only greedy streams
// splits the vocabulary: every rank projects its own slice of the (replicated) table, takes the slice's arg-max and
// the ranks vote (launch_tensor_parallel_argmax) - V / T rows of the table per rank instead of V.
void Engine::project_and_sample(const uint16_t *normalized, const std::string &projection_tensor, float scale, int lanes, const int32_t *slots,
                                const uint32_t *ticks, const char *what) {
    const ModelPlan &plan = model_->plan();
    const int vocab = static_cast<int>(plan.vocab), hidden = static_cast<int>(plan.hidden);
    const uint16_t *table = static_cast<const uint16_t *>(model_->tensor(projection_tensor));
    const void *streamed = lanes <= 8 && streaming_projection_ ? model_->projection_table(projection_tensor) : nullptr;
    const int size = model_->options().tp_size, rank = model_->options().tp_rank;
    // rows [first, first + count) into logits [lanes][count]
    auto project = [&](int first, int count, const char *label) {
        if (streamed != nullptr && first % 16 == 0) {
            check(launch_output_projection(normalized, streamed, first, static_cast<float *>(logits_.ptr), lanes, count, hidden, scale, model_->sm_count(),
                                           static_cast<int *>(kernel_error_.ptr), cuda_stream_),
                  label);
        } else {
            check(launch_linear_bf16(normalized, table + static_cast<size_t>(first) * hidden, logits_.ptr, nullptr, lanes, count, hidden, EPILOGUE_F32_SCALED, scale,
                                     cuda_stream_, static_cast<int *>(kernel_error_.ptr)),
                  label);
        }
    };
    if (size > 1 && tp_connected_ && vocabulary_parallel_ && stochastic_streams_ == 0 && !full_logits_ && lanes <= STACK_TP_VOTE_LANES) {
        const int per_rank = ((vocab + size - 1) / size + 15) / 16 * 16, first = std::min(vocab, rank * per_rank);
        const int count = std::max(0, std::min(vocab, first + per_rank) - first);
        project(first, count, "output projection (vocabulary slice)");
        check(launch_argmax(static_cast<const float *>(logits_.ptr), static_cast<uint32_t *>(records_.ptr), lanes, count, argmax_scratch_.ptr, cuda_stream_), what);
        counters_.kernel_launches++;
        check(launch_tensor_parallel_argmax(static_cast<const uint32_t *>(records_.ptr), static_cast<uint32_t>(first), static_cast<uint32_t *>(records_.ptr), lanes,
                                            static_cast<const StackTp *>(tp_description_.ptr), static_cast<int *>(kernel_error_.ptr), cuda_stream_),
              "arg-max vote");
        return;
    }
    project(0, vocab, "output projection");
    sample_lanes(static_cast<const float *>(logits_.ptr), static_cast<uint32_t *>(records_.ptr), lanes, slots, ticks, what);
}

void Engine::sample_lanes(const float *logits, uint32_t *records, int lanes, const int32_t *slots, const uint32_t *ticks, const char *what) {
    const int vocab = static_cast<int>(model_->plan().vocab);
    if (stochastic_streams_ == 0) {
        check(launch_argmax(logits, records, lanes, vocab, argmax_scratch_.ptr, cuda_stream_), what);
        counters_.kernel_launches++;
        return;
    }
    check(launch_sample(logits, records, lanes, vocab, static_cast<const SamplerParams *>(sampler_table_.ptr), slots, ticks,
                        sampler_scratch_.ptr, cuda_stream_),
          what);
    counters_.kernel_launches++;
}

void Engine::remove_stream(int64_t id) {
    Stream &s = stream(id);
    release_pages(s);
    if (s.sampler.method != 0) stochastic_streams_--;
    free_slots_.push_back(s.slot);
    latest_checkpoint_by_stream_.erase(id);
    streams_.erase(id);
    rejoin_scheduler(id);
    scheduler_.remove_stream(scheduler_id(id));
}

void Engine::reset_stream(int64_t id) {
    Stream &s = stream(id);
    release_pages(s);
    s.next_tick = 0;
    s.history.clear();
    latest_checkpoint_by_stream_.erase(id);  // the retained state itself stays until it is the least recently used
    s.queue.clear();
    s.active.reset();
    s.detached = false;
    rejoin_scheduler(id);
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    cuda_check(cudaMemsetAsync(static_cast<uint8_t *>(pending_hidden_.ptr) + s.slot * frame, 0, frame, cuda_stream_), "pending reset");
}

void Engine::interrupt_stream(int64_t id) {
    Stream &s = stream(id);
    s.queue.clear();
    s.active.reset();
    s.detached = false;
    rejoin_scheduler(id);  // interrupt (stream_runtime.rs:770-817), then a fresh entry: the scheduler keeps an interrupted stream closed to new events, the engine's streams take them
}

// stop_stream_after_current (placed_prompt_engine.rs:307-331, placed_prompt_event.rs:320-341): the active event
// emits nothing more; the token it emitted last is still fed back (the closing tick), so the state stays complete.
// Queued events are dropped (stream_runtime.rs:819-831).
void Engine::stop_stream_after_current(int64_t id) {
    Stream &s = stream(id);
    if (!s.active) return;
    s.queue.clear();
    s.active->remaining = 0;
    if (s.active->has_feedback) s.active->feedback_closes = true;
    // the scheduler drops the stream's queued events and its view of the current one; what is left of the event -
    // the closing tick - runs as a control step at the start of the next run
    scheduler_.close_stream_after_current(scheduler_id(id));
    rejoin_scheduler(id);
    s.detached = true;
}

Engine::StreamSnapshot Engine::stream_snapshot(int64_t id) const {
    const Stream &s = stream(id);
    StreamSnapshot snapshot;
    snapshot.pending_input_event_count = s.queue.size() + (s.active ? 1 : 0);
    snapshot.next_stream_tick = s.next_tick;
    snapshot.completed_prompt_event_count = s.completed_events;
    snapshot.idle = !s.active && s.queue.empty();
    snapshot.context_window_activations = model_->capacity();
    snapshot.speculative_draft_tokens = s.k;
    size_t pages = 0;
    for (int32_t page : s.pages) pages += page >= 0 ? 1 : 0;
    snapshot.mapped_state_pages = pages;
    return snapshot;
}

void Engine::scheduler_stream_counts(int64_t id, uint64_t out_counts[6]) const {
    stream(id);  // unknown stream: the engine's error
    const std::string name = scheduler_id(id);
    for (const runtime::StreamSnapshot &snapshot : scheduler_.snapshot().streams) {
        if (snapshot.stream_id != name) continue;
        out_counts[0] = snapshot.scheduled_activation_count;
        out_counts[1] = snapshot.completed_input_event_count;
        out_counts[2] = snapshot.generated_token_count;
        out_counts[3] = snapshot.in_flight_activation_count;
        out_counts[4] = snapshot.queued_input_event_count;
        out_counts[5] = snapshot.current_input_event_id.has_value() ? 1 : 0;
        return;
    }
    fail("stream " + name + " is unknown to the scheduler");
}

Engine::EngineSnapshot Engine::snapshot() const {
    EngineSnapshot snapshot;
    snapshot.stream_count = streams_.size();
    for (const auto &entry : streams_) snapshot.active_stream_count += (entry.second.active || !entry.second.queue.empty()) ? 1 : 0;
    snapshot.idle = snapshot.active_stream_count == 0;
    return snapshot;
}

void Engine::fork_stream(int64_t source, int64_t destination, uint32_t seed) {
    Stream &src = stream(source);
    if (src.active) fail("cannot fork stream " + std::to_string(source) + " while an input event is active");
    register_stream(destination, seed, src.k, src.sampler);
    scheduler_.fork_stream_transient_state(scheduler_id(source), scheduler_id(destination), "default");
    Stream &dst = stream(destination);
    dst.next_tick = src.next_tick;
    dst.history = src.history;
    // Every mapped page is shared by reference count, no copies (stream_state.rs:474-496); the first write of
    // either stream to a shared page replaces it with a private copy (ensure_pages, copy-on-write).
    for (size_t page = 0; page < src.pages.size(); page++) {
        int32_t physical = src.pages[page];
        if (physical < 0) continue;
        dst.pages[page] = physical;
        page_refcount_[physical]++;
    }
    dst.block_table_dirty = true;
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    cuda_check(cudaMemcpyAsync(static_cast<uint8_t *>(pending_hidden_.ptr) + dst.slot * frame,
                               static_cast<uint8_t *>(pending_hidden_.ptr) + src.slot * frame, frame, cudaMemcpyDeviceToDevice, cuda_stream_),
               "fork pending hidden");
}

// ---------------------------------------------------------------------------- prefix-state cache

namespace {
const char *const PREFIX_EXECUTION_CLASS = "default";
const runtime::StateKey PREFIX_STATE_KEY{"kv", "pages"};
}  // namespace

// What shaped the state besides the tokens (placed_prompt_engine.rs:1463-1480): the sampler and the draft count.
std::string Engine::prefix_modifier_bytes(const Stream &s) const {
    char text[192];
    std::snprintf(text, sizeof(text), "nerve.prefix_state_runtime_modifiers.v1;method=%d;temperature=%.9g;top_k=%d;top_p=%.9g;min_p=%.9g;drafts=%d",
                  s.sampler.method, s.sampler.temperature, s.sampler.top_k, s.sampler.top_p, s.sampler.min_p, s.k);
    return text;
}

void Engine::release_checkpoint(PrefixCheckpoint &checkpoint) {
    for (int32_t page : checkpoint.pages)
        if (page >= 0 && --page_refcount_[page] == 0) free_pages_.push_back(page);
    checkpoint.pages.clear();
    if (checkpoint.pending_slot >= 0) free_pending_slots_.push_back(checkpoint.pending_slot);
    checkpoint.pending_slot = -1;
}

void Engine::set_prefix_cache_capacity(size_t entries) {
    if (entries > 4096) fail("prefix cache capacity must be at most 4096 entries");
    for (auto &removed : prefix_index_.set_capacity(0)) release_checkpoint(removed.second);
    latest_checkpoint_by_stream_.clear();
    cuda_check(cudaStreamSynchronize(cuda_stream_), "prefix cache synchronize");
    cudaFree(prefix_pending_.ptr);
    prefix_pending_ = DeviceBuffer{};
    free_pending_slots_.clear();
    if (entries == 0) return;
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    prefix_pending_ = device_alloc((entries + 1) * frame);  // one frame more: an entry is filed before the oldest one leaves
    for (size_t slot = 0; slot <= entries; slot++) free_pending_slots_.push_back(static_cast<int>(slot));
    prefix_index_.set_capacity(entries);
}

Engine::PrefixCacheStats Engine::prefix_cache_stats() const {
    PrefixCacheStats stats = prefix_stats_;
    stats.resident_entry_count = prefix_index_.entries().size();
    const uint64_t page_bytes = model_->kv_bytes_per_token() * static_cast<uint64_t>(model_->options().page_tokens);
    for (const auto &item : prefix_index_.entries())
        stats.resident_byte_count += item.second.payload.pages.size() * page_bytes + static_cast<uint64_t>(model_->plan().hidden) * 2;
    return stats;
}

// The tick at which the prompt being prefilled gets its checkpoint: the last page boundary of the prompt (fewer
// than a page of prompt tokens remain there, capture_aligned_prefix_checkpoint, placed_prompt_engine.rs:964-1005),
// provided the stream's tokens are known from tick 0 and the ring has not wrapped.  0 = no checkpoint.
uint64_t Engine::prefix_checkpoint_tick(const Stream &s) const {
    if (!prefix_cache_on() || !s.active || s.history.size() != s.next_tick) return 0;
    const uint64_t page = static_cast<uint64_t>(model_->options().page_tokens);
    const uint64_t prompt_end = s.next_tick + (s.active->input.token_ids.size() - s.active->next_external);
    const uint64_t boundary = prompt_end / page * page;
    return boundary <= model_->capacity() ? boundary : 0;
}

void Engine::capture_prefix_checkpoint(Stream &s) {
    const size_t page_tokens = static_cast<size_t>(model_->options().page_tokens);
    const size_t page_count = static_cast<size_t>(s.next_tick) / page_tokens;
    if (page_count == 0 || s.history.size() != s.next_tick || free_pending_slots_.empty()) return;
    PrefixCheckpoint checkpoint;
    for (size_t page = 0; page < page_count; page++) {
        if (s.pages[page] < 0) return;  // not all of the prefix is resident
        checkpoint.pages.push_back(s.pages[page]);
    }
    const runtime::PrefixStateCacheKey key = runtime::PrefixStateCacheKey::from_token_prefix(PREFIX_EXECUTION_CLASS, model_->package().directory(), s.history,
                                                                                             prefix_modifier_bytes(s), {PREFIX_STATE_KEY});
    for (int32_t page : checkpoint.pages) page_refcount_[page]++;
    checkpoint.pending_slot = free_pending_slots_.back();
    free_pending_slots_.pop_back();
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    cuda_check(cudaMemcpyAsync(static_cast<uint8_t *>(prefix_pending_.ptr) + checkpoint.pending_slot * frame,
                               static_cast<uint8_t *>(pending_hidden_.ptr) + s.slot * frame, frame, cudaMemcpyDeviceToDevice, cuda_stream_),
               "prefix checkpoint pending hidden");
    auto inserted = prefix_index_.insert(key, std::move(checkpoint));
    prefix_stats_.insertion_count++;
    if (inserted.replaced) release_checkpoint(*inserted.replaced);
    std::set<runtime::PrefixStateCacheKey> gone;
    for (auto &removed : inserted.evicted) {
        release_checkpoint(removed.second);
        gone.insert(removed.first);
        prefix_stats_.eviction_count++;
    }
    // a stream keeps one checkpoint, its latest (placed_prompt_engine.rs:1046-1057)
    auto previous = latest_checkpoint_by_stream_.find(s.id);
    if (previous != latest_checkpoint_by_stream_.end() && previous->second != key && !gone.count(previous->second)) {
        if (auto removed = prefix_index_.evict(previous->second)) {
            release_checkpoint(*removed);
            prefix_stats_.eviction_count++;
        }
    }
    for (auto it = latest_checkpoint_by_stream_.begin(); it != latest_checkpoint_by_stream_.end();)
        it = gone.count(it->second) ? latest_checkpoint_by_stream_.erase(it) : std::next(it);
    latest_checkpoint_by_stream_.insert_or_assign(s.id, key);
}

// Only a fresh, idle stream takes a retained prefix, and the prompt's last token is always prefilled (it produces
// the first output): placed_prompt_engine.rs:198-253.
size_t Engine::restore_longest_prefix(Stream &s, const std::vector<uint32_t> &token_ids) {
    if (!prefix_cache_on() || s.next_tick != 0 || s.active || !s.queue.empty() || !s.history.empty() || token_ids.size() <= 1) return 0;
    for (int32_t page : s.pages)
        if (page >= 0) return 0;
    const std::vector<uint32_t> restorable(token_ids.begin(), token_ids.end() - 1);
    const std::optional<runtime::PrefixStateCacheKey> key =
        prefix_index_.longest_matching_key(PREFIX_EXECUTION_CLASS, model_->package().directory(), restorable, prefix_modifier_bytes(s), {PREFIX_STATE_KEY});
    if (!key) {
        prefix_stats_.miss_count++;
        return 0;
    }
    const PrefixCheckpoint &checkpoint = *prefix_index_.use(*key);
    for (size_t page = 0; page < checkpoint.pages.size(); page++) {
        s.pages[page] = checkpoint.pages[page];
        page_refcount_[checkpoint.pages[page]]++;
    }
    s.block_table_dirty = true;
    const size_t frame = static_cast<size_t>(model_->plan().hidden) * 2;
    cuda_check(cudaMemcpyAsync(static_cast<uint8_t *>(pending_hidden_.ptr) + s.slot * frame,
                               static_cast<uint8_t *>(prefix_pending_.ptr) + checkpoint.pending_slot * frame, frame, cudaMemcpyDeviceToDevice, cuda_stream_),
               "prefix restore pending hidden");
    s.next_tick = key->token_count;
    s.history = key->token_ids;
    prefix_stats_.hit_count++;
    prefix_stats_.reused_token_count += key->token_count;
    prefix_stats_.saved_prefill_token_count += key->token_count;
    return key->token_count;
}

void Engine::enqueue(int64_t id, const InputEvent &event) {
    Stream &s = stream(id);
    if (event.token_ids.empty()) fail("input event has no tokens");
    if (event.stop_token_ids.size() > MAX_STOP_TOKENS) fail("at most 8 stop tokens are supported per event");
    for (uint32_t token : event.token_ids)
        if (token >= static_cast<uint32_t>(model_->plan().vocab)) fail("input token id is outside the vocabulary");
    InputEvent accepted = event;
    const size_t reused = restore_longest_prefix(s, event.token_ids);
    if (reused > 0) accepted.token_ids.erase(accepted.token_ids.begin(), accepted.token_ids.begin() + static_cast<std::ptrdiff_t>(reused));
    runtime::InputEvent scheduled;
    scheduled.id = accepted.id.empty() ? std::string("event") : accepted.id;
    scheduled.token_ids = accepted.token_ids;
    scheduled.max_public_tokens = accepted.max_public_tokens;
    try {
        scheduler_.enqueue_input_event(scheduler_id(id), scheduled);
    } catch (...) {
        if (reused > 0) {  // the event was not taken: the stream is fresh again
            release_pages(s);
            s.next_tick = 0;
            s.history.clear();
            prefix_stats_.hit_count--;
            prefix_stats_.reused_token_count -= reused;
            prefix_stats_.saved_prefill_token_count -= reused;
        }
        throw;
    }
    s.queue.push_back(std::move(accepted));
}

void Engine::set_teacher_tokens(int64_t id, const std::vector<uint32_t> &tokens) { stream(id).teacher = tokens; }

void Engine::activate_next_event(Stream &s) {
    if (s.active || s.queue.empty()) return;
    auto active = std::make_unique<ActiveEvent>();
    active->input = std::move(s.queue.front());
    s.queue.pop_front();
    active->remaining = active->input.max_public_tokens;
    s.active = std::move(active);
}

void Engine::ensure_pages(Stream &s, uint64_t last_tick) {
    // every logical page touched by ticks <= last_tick must be mapped (ring: page index modulo pages per stream);
    // a page shared with another stream is replaced by a private copy before it is written (copy-on-write)
    const int page_tokens = model_->options().page_tokens;
    const int pages = static_cast<int>(s.pages.size());
    if (last_tick >= model_->rope_positions()) fail("stream tick exceeds the mounted position range");
    uint64_t first_tick = s.next_tick;
    for (uint64_t page_index = first_tick / page_tokens; page_index <= last_tick / page_tokens; page_index++) {
        int logical = static_cast<int>(page_index % pages);
        int32_t physical = s.pages[logical];
        if (physical >= 0 && page_refcount_[physical] == 1) continue;
        if (free_pages_.empty()) fail("KV page pool exhausted");
        int32_t fresh = free_pages_.back();
        free_pages_.pop_back();
        page_refcount_[fresh] = 1;
        if (physical >= 0) {  // shared page: copy, then drop the shared reference
            for (int layer = 0; layer < model_->kv_layer_count(); layer++) {
                size_t bytes = model_->page_bytes(layer);
                uint8_t *pool = reinterpret_cast<uint8_t *>(model_->kv_layer(layer).pool);
                cuda_check(cudaMemcpyAsync(pool + fresh * bytes, pool + physical * bytes, bytes, cudaMemcpyDeviceToDevice, cuda_stream_),
                           "copy-on-write page copy");
            }
            page_refcount_[physical]--;
        }
        s.pages[logical] = fresh;
        s.block_table_dirty = true;
    }
}

void Engine::sync_block_tables() {
    const int pages = model_->pages_per_stream();
    for (auto &entry : streams_) {
        Stream &s = entry.second;
        if (!s.block_table_dirty) continue;
        int32_t *row = block_table_host_.data() + static_cast<size_t>(s.slot) * pages;
        for (int page = 0; page < pages; page++) row[page] = s.pages[page] >= 0 ? s.pages[page] : 0;
        upload(model_->block_table_device() + static_cast<size_t>(s.slot) * pages, row, sizeof(int32_t) * pages, "block table upload");
        s.block_table_dirty = false;
    }
}

void *Engine::signal_buffer(const std::string &name) {
    auto found = signals_.find(name);
    if (found == signals_.end()) fail("no workspace for signal " + name);
    return found->second.ptr;
}

// ---------------------------------------------------------------------------- executor

void Engine::run_component(const ComponentPlan &plan, int kv_index, int lanes, const std::map<std::string, void *> &bound,
                           void *output) {
    cudaStream_t st = cuda_stream_;
    auto ptr = [&](const std::string &name) -> void * {
        auto found = bound.find(name);
        if (found != bound.end()) return found->second;
        if (name == plan.boundary_output) return output;
        return signal_buffer(name);
    };
    auto u16 = [&](const std::string &name) { return static_cast<uint16_t *>(ptr(name)); };
    auto width = [&](const std::string &name) { return static_cast<int>(plan.signals.at(name).width); };
    auto weight = [&](const std::string &name) { return model_->tensor(name); };
    const LaneTable lane_table = current_lanes_;

    auto consumers = [&](const std::string &signal, size_t after) {
        int count = 0;
        for (size_t i = after; i < plan.ops.size(); i++)
            for (const std::string &input : plan.ops[i].inputs) count += input == signal;
        if (signal == plan.boundary_output) count += 1;
        return count;
    };
    auto is_int4_single = [&](const OpSpec &op) {
        return op.kind == OpKind::Linear && op.weights.size() == 1 && op.weights[0].storage == TensorStorage::INT4_CT &&
               op.weights[0].group == 128;
    };

    for (size_t index = 0; index < plan.ops.size(); index++) {
        const OpSpec &op = plan.ops[index];
        switch (op.kind) {
        case OpKind::RmsNorm:
            check(launch_rms_norm(u16(op.inputs[0]), static_cast<const uint16_t *>(weight(op.norm_weights[0])), u16(op.outputs[0]), lanes,
                                  width(op.inputs[0]), op.eps, op.weight_offset, st),
                  "rms_norm");
            break;
        case OpKind::Linear: {
            if (op.tp_partial) {
                // row-parallel linear: f32 partial sums of this rank's columns -> all-reduce -> the linear's bf16 rounding
                // (and, when a residual_add of its output follows, that add with its second rounding)
                const WeightRef &w = op.weights[0];
                float *partial = static_cast<float *>(tp_partial_.ptr);
                if (w.storage == TensorStorage::INT4_CT) {
                    profile_begin(static_cast<uint64_t>(w.n) * (w.k / 2 + w.k / 64));
                    check(launch_linear_int4(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(w.tensor)),
                                             static_cast<const uint16_t *>(weight(w.scale)), reinterpret_cast<uint16_t *>(partial), nullptr, lanes,
                                             static_cast<int>(w.n), static_cast<int>(w.k), w.group, EPILOGUE_F32_SCALED, st, static_cast<int *>(kernel_error_.ptr)),
                          "linear_int4 (row-parallel)");
                    profile_end();
                } else {
                    check(launch_linear_bf16(u16(op.inputs[0]), static_cast<const uint16_t *>(weight(w.tensor)), partial, nullptr, lanes,
                                             static_cast<int>(w.n), static_cast<int>(w.k), EPILOGUE_F32_SCALED, 1.0f, st, static_cast<int *>(kernel_error_.ptr)),
                          "linear_bf16 (row-parallel)");
                }
                tp_all_reduce(partial, static_cast<size_t>(lanes) * w.n);
                const bool fold = index + 1 < plan.ops.size() && plan.ops[index + 1].kind == OpKind::ResidualAdd &&
                                  consumers(op.outputs[0], index + 2) == 0 &&
                                  (plan.ops[index + 1].inputs[0] == op.outputs[0] || plan.ops[index + 1].inputs[1] == op.outputs[0]);
                if (fold) {
                    const OpSpec &add = plan.ops[index + 1];
                    const std::string &residual = add.inputs[0] == op.outputs[0] ? add.inputs[1] : add.inputs[0];
                    check(launch_round_add(partial, u16(residual), u16(add.outputs[0]), static_cast<size_t>(lanes) * w.n, st), "round + residual");
                    index += 1;
                } else {
                    check(launch_round_add(partial, nullptr, u16(op.outputs[0]), static_cast<size_t>(lanes) * w.n, st), "round");
                }
                break;
            }
            if (is_int4_single(op)) {
                // gate/up + SiLU*up in one launch (batches below the GEMM threshold; wide batches run the three operators
                // as the package lists them, the two projections as tensor-core GEMMs)
                if (!linear_int4_gemm_supported(lanes, static_cast<int>(op.weights[0].n), static_cast<int>(op.weights[0].k)) &&
                    index + 2 < plan.ops.size() && is_int4_single(plan.ops[index + 1]) && plan.ops[index + 2].kind == OpKind::SiluMultiply &&
                    plan.ops[index + 1].inputs[0] == op.inputs[0] && plan.ops[index + 2].inputs[0] == op.outputs[0] &&
                    plan.ops[index + 2].inputs[1] == plan.ops[index + 1].outputs[0] && op.weights[0].n == plan.ops[index + 1].weights[0].n &&
                    consumers(op.outputs[0], index + 3) == 0 && consumers(plan.ops[index + 1].outputs[0], index + 3) == 0) {
                    const OpSpec &up = plan.ops[index + 1];
                    profile_begin(2 * static_cast<uint64_t>(op.weights[0].n) * (op.weights[0].k / 2 + op.weights[0].k / 64));
                    check(launch_linear_int4_silu_pair(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(op.weights[0].tensor)),
                                                       static_cast<const uint16_t *>(weight(op.weights[0].scale)),
                                                       static_cast<const uint32_t *>(weight(up.weights[0].tensor)),
                                                       static_cast<const uint16_t *>(weight(up.weights[0].scale)),
                                                       u16(plan.ops[index + 2].outputs[0]), lanes, static_cast<int>(op.weights[0].n),
                                                       static_cast<int>(op.weights[0].k), st),
                          "linear_int4 gate/up");
                    profile_end();
                    index += 2;
                    break;
                }
                // consecutive INT4 linears that share their input (q, k, v) in one launch
                size_t last = index;
                while (last + 1 < plan.ops.size() && last - index < 2 && is_int4_single(plan.ops[last + 1]) &&
                       plan.ops[last + 1].inputs[0] == op.inputs[0] && plan.ops[last + 1].weights[0].k == op.weights[0].k)
                    last++;
                // a lone INT4 linear followed by the residual add of its output: fold the add into the epilogue
                if (last == index && index + 1 < plan.ops.size() && plan.ops[index + 1].kind == OpKind::ResidualAdd &&
                    consumers(op.outputs[0], index + 2) == 0 &&
                    (plan.ops[index + 1].inputs[0] == op.outputs[0] || plan.ops[index + 1].inputs[1] == op.outputs[0])) {
                    const OpSpec &add = plan.ops[index + 1];
                    const std::string &residual = add.inputs[0] == op.outputs[0] ? add.inputs[1] : add.inputs[0];
                    profile_begin(static_cast<uint64_t>(op.weights[0].n) * (op.weights[0].k / 2 + op.weights[0].k / 64));
                    check(launch_linear_int4(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(op.weights[0].tensor)),
                                             static_cast<const uint16_t *>(weight(op.weights[0].scale)), u16(add.outputs[0]), u16(residual),
                                             lanes, static_cast<int>(op.weights[0].n), static_cast<int>(op.weights[0].k), 128,
                                             EPILOGUE_RESIDUAL_ROUNDED, st, static_cast<int *>(kernel_error_.ptr)),
                          "linear_int4 + residual");
                    profile_end();
                    index += 1;
                    break;
                }
                const uint32_t *qweights[3];
                const uint16_t *scales[3];
                uint16_t *outputs[3];
                int ns[3];
                int branches = 0;
                uint64_t branch_bytes = 0;
                for (size_t i = index; i <= last; i++, branches++) {
                    branch_bytes += static_cast<uint64_t>(plan.ops[i].weights[0].n) * (plan.ops[i].weights[0].k / 2 + plan.ops[i].weights[0].k / 64);
                    qweights[branches] = static_cast<const uint32_t *>(weight(plan.ops[i].weights[0].tensor));
                    scales[branches] = static_cast<const uint16_t *>(weight(plan.ops[i].weights[0].scale));
                    outputs[branches] = u16(plan.ops[i].outputs[0]);
                    ns[branches] = static_cast<int>(plan.ops[i].weights[0].n);
                }
                profile_begin(branch_bytes);
                check(launch_linear_int4_multi(u16(op.inputs[0]), branches, qweights, scales, outputs, ns, nullptr, lanes,
                                               static_cast<int>(op.weights[0].k), EPILOGUE_BF16, st, static_cast<int *>(kernel_error_.ptr)),
                      "linear_int4");
                profile_end();
                index = last;
                break;
            }
            for (size_t branch = 0; branch < op.weights.size(); branch++) {
                const WeightRef &w = op.weights[branch];
                if (w.storage == TensorStorage::BF16) {
                    const void *streamed = lanes <= 8 && streaming_projection_ ? model_->projection_table(w.tensor) : nullptr;
                    if (streamed != nullptr) {
                        check(launch_output_projection(u16(op.inputs[0]), streamed, 0, nullptr, lanes, static_cast<int>(w.n), static_cast<int>(w.k), 1.0f,
                                                       model_->sm_count(), static_cast<int *>(kernel_error_.ptr), st, u16(op.outputs[branch])),
                              "linear_bf16 (streamed)");
                    } else {
                        check(launch_linear_bf16(u16(op.inputs[0]), static_cast<const uint16_t *>(weight(w.tensor)), ptr(op.outputs[branch]), nullptr,
                                                 lanes, static_cast<int>(w.n), static_cast<int>(w.k), EPILOGUE_BF16, 1.0f, st, static_cast<int *>(kernel_error_.ptr)),
                              "linear_bf16");
                    }
                } else if (w.storage == TensorStorage::INT4_CT) {
                    check(launch_linear_int4(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(w.tensor)),
                                             static_cast<const uint16_t *>(weight(w.scale)), u16(op.outputs[branch]), nullptr, lanes,
                                             static_cast<int>(w.n), static_cast<int>(w.k), w.group, EPILOGUE_BF16, st, static_cast<int *>(kernel_error_.ptr)),
                          "linear_int4");
                } else if (w.storage == TensorStorage::FP8_BLOCK) {
                    if (!op.prequantized_input) fail("FP8 linear " + op.node_id + " without a prequantised input is not mounted");
                    check(launch_linear_fp8(static_cast<const uint8_t *>(ptr(op.inputs[0])), static_cast<const float *>(ptr(op.inputs[1])),
                                            static_cast<const uint8_t *>(weight(w.tensor)), static_cast<const uint16_t *>(weight(w.scale)),
                                            u16(op.outputs[branch]), nullptr, lanes, static_cast<int>(w.n), static_cast<int>(w.k),
                                            EPILOGUE_BF16, st),
                          "linear_fp8");
                }
            }
            break;
        }
        case OpKind::LinearResidual: {
            const WeightRef &w = op.weights[0];
            if (w.storage == TensorStorage::BF16) {
                check(launch_linear_bf16(u16(op.inputs[0]), static_cast<const uint16_t *>(weight(w.tensor)), ptr(op.outputs[0]),
                                         u16(op.residual_input), lanes, static_cast<int>(w.n), static_cast<int>(w.k),
                                         EPILOGUE_RESIDUAL_ROUNDED, 1.0f, st, static_cast<int *>(kernel_error_.ptr)),
                      "linear_residual_bf16");
            } else if (w.storage == TensorStorage::FP8_BLOCK) {
                check(launch_linear_fp8(static_cast<const uint8_t *>(ptr(op.inputs[0])), static_cast<const float *>(ptr(op.inputs[1])),
                                        static_cast<const uint8_t *>(weight(w.tensor)), static_cast<const uint16_t *>(weight(w.scale)),
                                        u16(op.outputs[0]), u16(op.residual_input), lanes, static_cast<int>(w.n), static_cast<int>(w.k),
                                        EPILOGUE_RESIDUAL_F32, st),
                      "linear_residual_fp8");
            } else {
                check(launch_linear_int4(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(w.tensor)),
                                         static_cast<const uint16_t *>(weight(w.scale)), u16(op.outputs[0]), u16(op.residual_input), lanes,
                                         static_cast<int>(w.n), static_cast<int>(w.k), w.group, EPILOGUE_RESIDUAL_ROUNDED, st, static_cast<int *>(kernel_error_.ptr)),
                      "linear_residual_int4");
            }
            break;
        }
        case OpKind::LinearSiluMultiply: {
            const WeightRef &gate = op.weights[0], &up = op.weights[1];
            if (gate.storage == TensorStorage::BF16) {
                check(launch_linear_silu_multiply_bf16(u16(op.inputs[0]), static_cast<const uint16_t *>(weight(gate.tensor)),
                                                       static_cast<const uint16_t *>(weight(up.tensor)), u16(op.outputs[0]), lanes,
                                                       static_cast<int>(gate.n), static_cast<int>(gate.k), st),
                      "linear_silu_multiply_bf16");
            } else if (gate.storage == TensorStorage::FP8_BLOCK) {
                check(launch_linear_silu_multiply_fp8(static_cast<const uint8_t *>(ptr(op.inputs[0])), static_cast<const float *>(ptr(op.inputs[1])),
                                                      static_cast<const uint8_t *>(weight(gate.tensor)),
                                                      static_cast<const uint16_t *>(weight(gate.scale)),
                                                      static_cast<const uint8_t *>(weight(up.tensor)),
                                                      static_cast<const uint16_t *>(weight(up.scale)), u16(op.outputs[0]), lanes,
                                                      static_cast<int>(gate.n), static_cast<int>(gate.k), st),
                      "linear_silu_multiply_fp8");
            } else {
                check(launch_linear_int4_silu_pair(u16(op.inputs[0]), static_cast<const uint32_t *>(weight(gate.tensor)),
                                                   static_cast<const uint16_t *>(weight(gate.scale)),
                                                   static_cast<const uint32_t *>(weight(up.tensor)),
                                                   static_cast<const uint16_t *>(weight(up.scale)), u16(op.outputs[0]), lanes,
                                                   static_cast<int>(gate.n), static_cast<int>(gate.k), st),
                      "linear_silu_multiply_int4");
            }
            break;
        }
        case OpKind::QuantizeFp8:
            check(launch_quantize_fp8(u16(op.inputs[0]), static_cast<uint8_t *>(ptr(op.outputs[0])), static_cast<float *>(ptr(op.outputs[1])),
                                      lanes, width(op.inputs[0]), st),
                  "quantize_fp8");
            break;
        case OpKind::Rope: {
            const RopeAttrs &rope = op.rope[0];
            check(launch_rope(u16(op.inputs[0]), u16(op.outputs[0]), model_->rope_table(rope.theta, rope.rotary_width), model_->rope_positions(),
                              lane_table.position, lanes, rope.heads, rope.head_width, rope.rotary_width, rope.interleaved, nullptr, 0.0f, 0.0f,
                              st),
                  "rope");
            break;
        }
        case OpKind::HeadNormRope:
            for (size_t branch = 0; branch < op.rope.size(); branch++) {
                const RopeAttrs &rope = op.rope[branch];
                check(launch_rope(u16(op.inputs[branch]), u16(op.outputs[branch]), model_->rope_table(rope.theta, rope.rotary_width),
                                  model_->rope_positions(), lane_table.position, lanes, rope.heads, rope.head_width, rope.rotary_width,
                                  rope.interleaved, static_cast<const uint16_t *>(weight(op.norm_weights[branch])), op.eps, op.weight_offset,
                                  st),
                      "head_norm_rope");
            }
            break;
        case OpKind::AppendAttention: {
            if (kv_index < 0) fail("attention op in a component without KV state");
            KvLayer kv = model_->kv_layer(kv_index);
            check(launch_kv_append(u16(op.inputs[1]), u16(op.inputs[2]), kv, lane_table, lanes, st), "kv_append");
            check(launch_attention(u16(op.inputs[0]), u16(op.outputs[0]), kv, lane_table, lanes, current_width_, op.q_heads, op.attention_scale, op_split_tokens_,
                                   current_op_splits_, static_cast<float *>(attention_scratch_.ptr), st),
                  "attention");
            counters_.kernel_launches++;
            break;
        }
        case OpKind::ResidualAdd:
            check(launch_add(u16(op.inputs[0]), u16(op.inputs[1]), u16(op.outputs[0]), static_cast<size_t>(lanes) * width(op.inputs[0]), st),
                  "residual_add");
            break;
        case OpKind::SiluMultiply:
            check(launch_silu_multiply(u16(op.inputs[0]), u16(op.inputs[1]), u16(op.outputs[0]),
                                       static_cast<size_t>(lanes) * width(op.inputs[0]), st),
                  "silu_multiply");
            break;
        case OpKind::Concat:
            if (op.inputs.size() != 2) fail("concatenate with other than two inputs is not mounted");
            check(launch_concat(u16(op.inputs[0]), u16(op.inputs[1]), u16(op.outputs[0]), lanes, width(op.inputs[0]), width(op.inputs[1]), st),
                  "concatenate");
            break;
        case OpKind::MoeTopk:
            check(launch_moe_topk(u16(op.inputs[0]), static_cast<uint32_t *>(ptr(op.outputs[0])), lanes, op.experts, op.top_k, st), "moe_topk");
            break;
        case OpKind::MoeGateUp: {
            const WeightRef &w = op.weights[0];
            if (w.storage != TensorStorage::FP8_BLOCK) fail("only FP8 expert weights are mounted");
            check(launch_moe_gate_up_fp8(u16(op.inputs[0]), static_cast<const uint32_t *>(ptr(op.inputs[1])),
                                         static_cast<const uint8_t *>(weight(w.tensor)), static_cast<const uint16_t *>(weight(w.scale)),
                                         u16(op.outputs[0]), lanes, op.moe_hidden, op.moe_inter, op.experts, op.top_k, 0, op.experts, st),
                  "sparse_moe_gate_up");
            break;
        }
        case OpKind::MoeDown: {
            const WeightRef &w = op.weights[0];
            if (w.storage != TensorStorage::FP8_BLOCK) fail("only FP8 expert weights are mounted");
            check(launch_moe_down_fp8(u16(op.inputs[0]), static_cast<const uint32_t *>(ptr(op.inputs[1])),
                                      static_cast<const uint8_t *>(weight(w.tensor)), static_cast<const uint16_t *>(weight(w.scale)),
                                      u16(op.outputs[0]), lanes, op.moe_hidden, op.moe_inter, op.experts, op.top_k, 0, op.experts, st),
                  "sparse_moe_down");
            break;
        }
        case OpKind::MoeReduce:
            check(launch_moe_reduce(u16(op.inputs[0]), u16(op.outputs[0]), lanes, op.moe_hidden, op.top_k, op.routed_scale, st), "moe_reduce");
            break;
        }
    }
}

void Engine::upload(void *device_destination, const void *host_source, size_t bytes, const char *what) {
    size_t aligned = (bytes + 15) & ~size_t(15);
    if (staging_used_ + aligned > staging_bytes_) {
        // arena full: drain the stream so that earlier regions may be reused
        synchronize("staging drain");
    }
    if (aligned > staging_bytes_) fail("upload larger than the pinned staging arena");
    uint8_t *region = staging_ + staging_used_;
    staging_used_ += aligned;
    std::memcpy(region, host_source, bytes);
    cuda_check(cudaMemcpyAsync(device_destination, region, bytes, cudaMemcpyHostToDevice, cuda_stream_), what);
    counters_.h2d_bytes += bytes;
}

void Engine::synchronize(const char *what) {
    cuda_check(cudaStreamSynchronize(cuda_stream_), what);
    counters_.host_syncs++;
    staging_used_ = 0;
    for (size_t i = 0; i + 1 < profile_used_; i += 2) {
        float ms = 0.0f;
        cuda_check(cudaEventElapsedTime(&ms, profile_events_[i], profile_events_[i + 1]), "profile event elapsed");
        profile_ms_ += ms;
    }
    profile_used_ = 0;
}

void Engine::profile_begin(uint64_t bytes) {
    if (!profile_) return;
    if (profile_used_ + 2 > profile_events_.size()) {
        for (int i = 0; i < 2; i++) {
            cudaEvent_t event;
            cuda_check(cudaEventCreate(&event), "cudaEventCreate");
            profile_events_.push_back(event);
        }
    }
    cuda_check(cudaEventRecord(profile_events_[profile_used_], cuda_stream_), "profile event record");
    profile_bytes_ += bytes;
    profile_launches_++;
}

void Engine::profile_end() {
    if (!profile_) return;
    cuda_check(cudaEventRecord(profile_events_[profile_used_ + 1], cuda_stream_), "profile event record");
    profile_used_ += 2;
}

void Engine::upload_lanes(const std::vector<uint32_t> &positions, const std::vector<int32_t> &slots) {
    upload(lane_positions_.ptr, positions.data(), positions.size() * sizeof(uint32_t), "lane positions upload");
    upload(lane_slots_.ptr, slots.data(), slots.size() * sizeof(int32_t), "lane slots upload");
    current_lanes_ = LaneTable{static_cast<const uint32_t *>(lane_positions_.ptr), static_cast<const int32_t *>(lane_slots_.ptr)};
    uint32_t newest = 0;
    for (uint32_t position : positions) newest = std::max(newest, position);
    plan_splits(static_cast<int>(positions.size()), newest);
}

void Engine::upload_tokens(const uint32_t *tokens, int count) {
    upload(lane_tokens_.ptr, tokens, static_cast<size_t>(count) * sizeof(uint32_t), "lane tokens upload");
    current_tokens_ = static_cast<const uint32_t *>(lane_tokens_.ptr);
}

// Attention launches cover ceil(context / split) splits, rounded up to a power of two so that a handful of graph
// shapes serves a growing context: splits of 64 tokens in the persistent kernel, of the engine's fixed length on the
// kernel-per-operator path.  Returns a word for graph keys.
int Engine::plan_splits(int lanes, uint64_t newest_tick) {
    (void)lanes;
    const uint64_t tokens = std::min<uint64_t>(newest_tick + 1, model_->capacity());
    auto bucket = [&](int split_tokens) {
        const int needed = std::max(1, static_cast<int>((tokens + split_tokens - 1) / split_tokens));
        const int most = std::max(1, static_cast<int>((model_->capacity() + split_tokens - 1) / split_tokens));
        int count = 1;
        while (count < needed) count <<= 1;
        return std::min(count, most);
    };
    current_splits_ = bucket(split_tokens_);
    current_op_splits_ = bucket(op_split_tokens_);
    return current_splits_ | (current_op_splits_ << 16);
}

// Runs `body` (stream-ordered launches only: no uploads, read-backs or synchronisation) directly the first time a
// key is seen, then captures it into a CUDA graph and replays the graph from the third call on.
void Engine::run_phase(const std::vector<int> &key, const std::function<void()> &body) {
    // Tensor-parallel engines replay graphs only for phases that contain no NCCL call: every forward of the phase
    // runs in the persistent kernel (at most 8 lanes), whose exchange goes over peer memory.  A launch with the
    // barrier test hook armed is never captured (the hook is a kernel argument).
    bool direct = !use_graphs_ || profile_ || inject_barrier_timeouts_ > 0;
    if (model_->options().tp_size > 1) {
        const bool stacks = model_->target_stack().available && (!model_->plan().has_draft || model_->draft_stack().available);
        const bool small = key.size() >= 3 && key[1] * (key[2] + 1) <= 8;
        if (!(tp_connected_ && stack_enabled_ && stacks && small)) direct = true;
    }
    if (direct) {
        body();
        return;
    }
    GraphEntry &entry = graphs_[key];
    if (entry.exec == nullptr) {
        if (entry.warm++ == 0) {
            body();
            return;
        }
        uint64_t before = counters_.kernel_launches;
        cudaGraph_t graph = nullptr;
        cuda_check(cudaStreamBeginCapture(cuda_stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        try {
            body();
        } catch (...) {
            cudaStreamEndCapture(cuda_stream_, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        cuda_check(cudaStreamEndCapture(cuda_stream_, &graph), "cudaStreamEndCapture");
        entry.kernel_nodes = counters_.kernel_launches - before;
        counters_.kernel_launches = before;
        cuda_check(cudaGraphInstantiate(&entry.exec, graph, 0), "cudaGraphInstantiate");
        cudaGraphDestroy(graph);
    }
    cuda_check(cudaGraphLaunch(entry.exec, cuda_stream_), "cudaGraphLaunch");
    counters_.graph_launches++;
    counters_.kernel_launches += entry.kernel_nodes;
}

// Runs a whole layer stack over `hidden` ([lanes][hidden], in place) with the persistent decode kernel when the
// stack and the batch qualify; false = the caller runs the layers kernel by kernel.
bool Engine::run_stack(const StackPlan &stack, int lanes, void *hidden) {
    const int tp_size = model_->options().tp_size;
    if (tp_size > 1 && !tp_connected_) return false;  // without the peer exchange the shards meet in NCCL all-reduces, kernel by kernel
    if (!stack_enabled_ || !stack.available || lanes < 1 || lanes > 8 || current_width_ <= 0 || lanes % current_width_ != 0) return false;
    size_t smem = 0;
    if (!decode_stack_supported(stack.shape, lanes, &smem) || current_splits_ > 1024) return false;  // two merge levels of 32 splits
    StackBuffers buffers{};
    buffers.hidden = static_cast<uint16_t *>(hidden);
    buffers.q = static_cast<uint16_t *>(stack_q_.ptr);
    buffers.attention_scratch = static_cast<float *>(attention_scratch_.ptr);
    buffers.attention_out = static_cast<uint16_t *>(stack_attention_out_.ptr);
    buffers.activation = static_cast<uint16_t *>(stack_activation_.ptr);
    buffers.barrier = static_cast<unsigned int *>(stack_barrier_.ptr);
    buffers.error_flag = static_cast<int *>(kernel_error_.ptr);
    buffers.timing = (profile_ && &stack == &model_->target_stack()) ? static_cast<unsigned long long *>(stack_timing_.ptr) : nullptr;
    buffers.barrier_handicap = 0;
    if (inject_barrier_timeouts_ > 0) {
        inject_barrier_timeouts_--;
        buffers.barrier_handicap = 1u << 20;
    }
    profile_begin(stack.weight_bytes);
    check(launch_decode_stack(static_cast<const StackLayer *>(stack.device_layers.ptr), static_cast<int>(stack.layers.size()), stack.shape,
                              buffers, current_lanes_, lanes, current_width_, split_tokens_, current_splits_, cuda_stream_,
                              static_cast<const StackTp *>(tp_description_.ptr), tp_size),
          "decode stack");
    profile_end();
    return true;
}

std::vector<unsigned long long> Engine::decode_stack_timing() {
    std::vector<unsigned long long> stamps;
    if (!stack_timing_.ptr || !model_->target_stack().available) return stamps;
    stamps.resize(model_->target_stack().layers.size() * 32);
    cuda_check(cudaStreamSynchronize(cuda_stream_), "stream synchronize");
    cuda_check(cudaMemcpy(stamps.data(), stack_timing_.ptr, stamps.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost), "timing readback");
    return stamps;
}

void Engine::target_forward(int lanes, bool want_logits) {
    const ModelPlan &plan = model_->plan();
    check(launch_embedding(static_cast<const uint16_t *>(model_->tensor(plan.embedding_tensor)), current_tokens_,
                           static_cast<uint16_t *>(frame_a_.ptr), lanes, static_cast<int>(plan.hidden), static_cast<int>(plan.vocab),
                           plan.embedding_scale, cuda_stream_),
          "embedding");
    void *input = frame_a_.ptr, *output = frame_b_.ptr;
    if (!run_stack(model_->target_stack(), lanes, input)) {
        int kv_index = 0;
        for (const ComponentPlan &layer : plan.layers) {
            std::map<std::string, void *> bound{{layer.boundary_inputs.at(0), input}};
            run_component(layer, layer.has_kv ? kv_index : -1, lanes, bound, output);
            if (layer.has_kv) kv_index++;
            std::swap(input, output);
        }
    }
    check(launch_rms_norm(static_cast<const uint16_t *>(input), static_cast<const uint16_t *>(model_->tensor(plan.output.norm_tensor)),
                          static_cast<uint16_t *>(normalized_.ptr), lanes, static_cast<int>(plan.hidden), plan.output.eps,
                          plan.output.weight_offset, cuda_stream_),
          "output norm");
    if (want_logits) {
        project_and_sample(static_cast<const uint16_t *>(normalized_.ptr), plan.output.projection_tensor, plan.output.logits_scale, lanes,
                           current_lanes_.slot, current_lanes_.position, "sampler");
    }
}

void Engine::draft_forward(int lanes, const uint16_t *hidden_in, bool want_logits) {
    const ModelPlan &plan = model_->plan();
    check(launch_embedding(static_cast<const uint16_t *>(model_->tensor(plan.embedding_tensor)), current_tokens_,
                           static_cast<uint16_t *>(embedding_out_.ptr), lanes, static_cast<int>(plan.hidden), static_cast<int>(plan.vocab),
                           plan.embedding_scale, cuda_stream_),
          "draft embedding");
    std::map<std::string, void *> adapter_bound{{plan.adapter_token_signal, embedding_out_.ptr},
                                                {plan.adapter_hidden_signal, const_cast<uint16_t *>(hidden_in)}};
    run_component(plan.draft_adapter, -1, lanes, adapter_bound, frame_a_.ptr);
    void *input = frame_a_.ptr, *output = frame_b_.ptr;
    if (!run_stack(model_->draft_stack(), lanes, input)) {
        int kv_index = 0;
        for (const ComponentPlan &layer : plan.layers) kv_index += layer.has_kv ? 1 : 0;
        for (const ComponentPlan &layer : plan.draft_layers) {
            std::map<std::string, void *> bound{{layer.boundary_inputs.at(0), input}};
            run_component(layer, layer.has_kv ? kv_index : -1, lanes, bound, output);
            if (layer.has_kv) kv_index++;
            std::swap(input, output);
        }
    }
    if (!want_logits) return;
    check(launch_rms_norm(static_cast<const uint16_t *>(input), static_cast<const uint16_t *>(model_->tensor(plan.draft_output.norm_tensor)),
                          static_cast<uint16_t *>(draft_normalized_.ptr), lanes, static_cast<int>(plan.hidden), plan.draft_output.eps,
                          plan.draft_output.weight_offset, cuda_stream_),
          "draft output norm");
    project_and_sample(static_cast<const uint16_t *>(draft_normalized_.ptr), plan.draft_output.projection_tensor, plan.draft_output.logits_scale, lanes,
                       current_lanes_.slot, current_lanes_.position, "draft sampler");
}

// ---------------------------------------------------------------------------- prefill (temporal_prompt.rs:298-478)

void Engine::run_prefill_chunk(Stream &s, const uint32_t *tokens, int count, bool sample_last, uint32_t *sampled) {
    const ModelPlan &plan = model_->plan();
    ensure_pages(s, s.next_tick + count - 1);
    sync_block_tables();
    std::vector<uint32_t> positions(count);
    std::vector<int32_t> slots(count, s.slot);
    for (int i = 0; i < count; i++) positions[i] = static_cast<uint32_t>(s.next_tick + i);
    upload_lanes(positions, slots);
    upload_tokens(tokens, count);
    current_width_ = count;
    target_forward(count, false);
    const size_t frame = static_cast<size_t>(plan.hidden) * 2;
    uint8_t *pending = static_cast<uint8_t *>(pending_hidden_.ptr) + s.slot * frame;
    if (plan.has_draft) {
        // draft state steps for every prompt token: token i pairs with the target hidden of tick i-1
        // (verification.rs:10-34): lane 0 takes the pending hidden, lane i the normalised frame i-1.
        check(launch_shift_hidden(static_cast<const uint16_t *>(pending_hidden_.ptr), static_cast<const int32_t *>(lane_slots_.ptr),
                                  static_cast<const uint16_t *>(normalized_.ptr), static_cast<uint16_t *>(draft_hidden_in_.ptr), 1, count,
                                  static_cast<int>(plan.hidden), cuda_stream_),
              "prefill draft hidden");
        draft_forward(count, static_cast<const uint16_t *>(draft_hidden_in_.ptr), false);
        cuda_check(cudaMemcpyAsync(pending, static_cast<uint8_t *>(normalized_.ptr) + static_cast<size_t>(count - 1) * frame, frame,
                                   cudaMemcpyDeviceToDevice, cuda_stream_),
                   "commit target hidden");
    }
    if (sample_last) {
        project_and_sample(static_cast<const uint16_t *>(normalized_.ptr) + static_cast<size_t>(count - 1) * plan.hidden, plan.output.projection_tensor,
                           plan.output.logits_scale, 1, current_lanes_.slot + (count - 1), current_lanes_.position + (count - 1), "prefill sampler");
        cuda_check(cudaMemcpyAsync(host_records_, records_.ptr, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, cuda_stream_), "record readback");
        synchronize("prefill synchronize");
        counters_.d2h_bytes += 16;
        *sampled = host_records_[0];
    }
    s.next_tick += count;
}

void Engine::emit(Stream &s, uint32_t token, uint64_t tick, const std::function<void(const OutputEvent &)> &on_output, RunReport &report) {
    ActiveEvent &event = *s.active;
    OutputEvent output{s.id, token, tick, event.generated.size()};
    event.generated.push_back(token);
    event.remaining -= 1;
    bool closes;
    if (std::find(event.input.stop_token_ids.begin(), event.input.stop_token_ids.end(), token) != event.input.stop_token_ids.end()) {
        event.remaining = 0;
        closes = true;
    } else {
        closes = event.remaining == 0;
    }
    event.has_feedback = true;
    event.feedback_token = token;
    event.feedback_closes = closes;
    report.generated_tokens++;
    if (on_output) on_output(output);
}

// ---------------------------------------------------------------------------- kernel errors
// A kernel whose bounded wait expired sets the error word and finishes on garbage.  The word travels back with every
// batch's read-back; when it is set nothing of the batch is emitted or committed - stream ticks are untouched, the
// pending hidden states are put back as they were (the KV slots the batch wrote are rewritten when the ticks are
// replayed) - and the call fails, as the reference restores the state of a failed cycle
// (placed_stream_processor/feedback_generation.rs:188-192).

void Engine::backup_pending() {
    cuda_check(cudaMemcpyAsync(pending_backup_.ptr, pending_hidden_.ptr, pending_hidden_.bytes, cudaMemcpyDeviceToDevice, cuda_stream_), "pending hidden backup");
}

void Engine::check_kernel_status(const uint32_t *status_word) {
    if (*status_word == 0) return;
    const int code = static_cast<int>(*status_word);
    cuda_check(cudaMemsetAsync(kernel_error_.ptr, 0, sizeof(int), cuda_stream_), "kernel status reset");
    if (stack_barrier_.ptr) cuda_check(cudaMemsetAsync(stack_barrier_.ptr, 0, stack_barrier_.bytes, cuda_stream_), "barrier reset");
    cuda_check(cudaMemcpyAsync(pending_hidden_.ptr, pending_backup_.ptr, pending_hidden_.bytes, cudaMemcpyDeviceToDevice, cuda_stream_), "pending hidden restore");
    synchronize("restore synchronize");
    if (model_->options().tp_size > 1) failed_ = true;  // the peers' exchange counters have moved on without this rank
    fail(code == 2 ? "the decode stack kernel gave up waiting at a grid barrier (or for a tensor-parallel peer); the batch was discarded and the streams are as before it"
                   : "a kernel gave up waiting on its copy pipeline; the batch was discarded and the streams are as before it");
}

// ---------------------------------------------------------------------------- single ticks (placed_prompt_stream.rs:353-420)

void Engine::run_single_ticks(std::vector<Stream *> &batch, const std::function<void(const OutputEvent &)> &on_output, RunReport &report) {
    const ModelPlan &plan = model_->plan();
    const int lanes = static_cast<int>(batch.size());
    std::vector<uint32_t> positions(lanes);
    std::vector<int32_t> slots(lanes);
    std::vector<uint32_t> tokens(lanes);
    bool any_emit = false;
    for (int i = 0; i < lanes; i++) {
        Stream &s = *batch[i];
        ensure_pages(s, s.next_tick);
        positions[i] = static_cast<uint32_t>(s.next_tick);
        slots[i] = s.slot;
        tokens[i] = s.active->feedback_token;
        any_emit |= !s.active->feedback_closes && s.active->remaining > 0;
    }
    sync_block_tables();
    upload_lanes(positions, slots);
    upload_tokens(tokens.data(), lanes);
    current_width_ = 1;
    if (plan.has_draft) backup_pending();
    target_forward(lanes, any_emit);
    if (plan.has_draft) {
        check(launch_gather_rows(static_cast<const uint16_t *>(pending_hidden_.ptr), static_cast<const int32_t *>(lane_slots_.ptr),
                                 static_cast<uint16_t *>(draft_hidden_in_.ptr), lanes, static_cast<int>(plan.hidden), cuda_stream_),
              "gather pending hidden");
        draft_forward(lanes, static_cast<const uint16_t *>(draft_hidden_in_.ptr), false);
        const size_t frame = static_cast<size_t>(plan.hidden) * 2;
        for (int i = 0; i < lanes; i++)
            cuda_check(cudaMemcpyAsync(static_cast<uint8_t *>(pending_hidden_.ptr) + batch[i]->slot * frame,
                                       static_cast<uint8_t *>(normalized_.ptr) + i * frame, frame, cudaMemcpyDeviceToDevice, cuda_stream_),
                       "commit target hidden");
    }
    if (any_emit) {
        cuda_check(cudaMemcpyAsync(host_records_, records_.ptr, lanes * 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, cuda_stream_),
                   "record readback");
        counters_.d2h_bytes += lanes * 16;
    }
    uint32_t *status_word = host_records_ + static_cast<size_t>(lanes) * 4;
    cuda_check(cudaMemcpyAsync(status_word, kernel_error_.ptr, sizeof(int), cudaMemcpyDeviceToHost, cuda_stream_), "kernel status readback");
    counters_.d2h_bytes += 4;
    synchronize("tick synchronize");
    check_kernel_status(status_word);
    for (int i = 0; i < lanes; i++) {
        Stream &s = *batch[i];
        ActiveEvent &event = *s.active;
        uint64_t tick = s.next_tick;
        if (prefix_cache_on() && s.history.size() == s.next_tick) s.history.push_back(tokens[i]);
        s.next_tick += 1;
        bool was_closing = event.feedback_closes;
        bool should_emit = !was_closing && event.remaining > 0;
        event.has_feedback = false;
        if (should_emit) emit(s, host_records_[i * 4], tick, on_output, report);
        if (was_closing || !event.has_feedback) {
            s.active.reset();
            s.completed_events++;
        }
    }
}

// ---------------------------------------------------------------------------- speculative cycles (feedback_generation.rs:66-194)

void Engine::run_speculative_cycles(std::vector<Stream *> &batch, int drafts, const std::function<void(const OutputEvent &)> &on_output,
                                    RunReport &report) {
    const ModelPlan &plan = model_->plan();
    const int streams = static_cast<int>(batch.size());
    const int width = drafts + 1;
    const int lanes = streams * width;
    if (lanes > model_->options().max_lanes) fail("verify batch exceeds max_lanes");

    // device cycle arrays carved out of cycle_state_; everything up to `accept_rows` is uploaded in one copy
    uint32_t *base = static_cast<uint32_t *>(cycle_state_.ptr);
    uint32_t *verify_tokens = base;                              // [streams][width]
    uint32_t *forced = verify_tokens + lanes;                    // [streams][drafts]
    uint32_t *stop_tokens = forced + lanes;                      // [streams][MAX_STOP]
    int32_t *stop_counts = reinterpret_cast<int32_t *>(stop_tokens + streams * MAX_STOP_TOKENS);  // [streams]
    int32_t *stream_slots = stop_counts + streams;               // [streams]
    uint32_t *draft_positions = reinterpret_cast<uint32_t *>(stream_slots + streams);  // [drafts][streams]
    uint32_t *verify_positions = draft_positions + drafts * streams;                   // [lanes]
    int32_t *verify_slots = reinterpret_cast<int32_t *>(verify_positions + lanes);     // [lanes]
    uint32_t *draft_tokens = reinterpret_cast<uint32_t *>(verify_slots + lanes);       // [streams]
    const size_t upload_words = static_cast<size_t>(lanes) * 4 + streams * MAX_STOP_TOKENS + 3 * streams + drafts * streams;
    uint32_t *accept_rows = base + upload_words;                 // [streams][4 + 2*width]

    std::vector<uint32_t> staging(upload_words, 0);
    uint32_t *s_forced = staging.data() + lanes, *s_stop = s_forced + lanes, *s_counts = s_stop + streams * MAX_STOP_TOKENS;
    uint32_t *s_slots = s_counts + streams, *s_dpos = s_slots + streams, *s_vpos = s_dpos + drafts * streams;
    uint32_t *s_vslots = s_vpos + lanes, *s_dtokens = s_vslots + lanes;
    uint64_t newest_tick = 0;
    for (int s = 0; s < streams; s++) {
        Stream &st = *batch[s];
        ensure_pages(st, st.next_tick + drafts);
        newest_tick = std::max<uint64_t>(newest_tick, st.next_tick + drafts);
        staging[static_cast<size_t>(s) * width] = st.active->feedback_token;
        s_dtokens[s] = st.active->feedback_token;
        for (int j = 0; j < drafts; j++) {
            size_t output_index = st.active->generated.size() + j;
            s_forced[static_cast<size_t>(s) * drafts + j] = output_index < st.teacher.size() ? st.teacher[output_index] : 0xffffffffu;
            s_dpos[static_cast<size_t>(j) * streams + s] = static_cast<uint32_t>(st.next_tick + j);
        }
        const auto &stops = st.active->input.stop_token_ids;
        for (size_t t = 0; t < stops.size(); t++) s_stop[s * MAX_STOP_TOKENS + t] = stops[t];
        s_counts[s] = static_cast<uint32_t>(stops.size());
        s_slots[s] = static_cast<uint32_t>(st.slot);
        for (int i = 0; i < width; i++) {
            s_vpos[s * width + i] = static_cast<uint32_t>(st.next_tick + i);
            s_vslots[s * width + i] = static_cast<uint32_t>(st.slot);
        }
    }
    sync_block_tables();
    upload(base, staging.data(), upload_words * sizeof(uint32_t), "cycle state upload");
    const int splits = plan_splits(streams * (drafts + 1), newest_tick);

    backup_pending();
    cuda_check(cudaEventRecord(event_begin_, cuda_stream_), "event record");
    // ---- draft loop: `drafts` serial steps over `streams` lanes
    run_phase({0, streams, drafts, splits, stochastic_streams_ != 0 ? 1 : 0, stack_enabled_ ? 1 : 0}, [&] {
        for (int j = 0; j < drafts; j++) {
            current_lanes_ = LaneTable{draft_positions + static_cast<size_t>(j) * streams, stream_slots};
            current_tokens_ = draft_tokens;
            current_width_ = 1;
            if (j == 0) {
                check(launch_gather_rows(static_cast<const uint16_t *>(pending_hidden_.ptr), stream_slots,
                                         static_cast<uint16_t *>(draft_hidden_in_.ptr), streams, static_cast<int>(plan.hidden), cuda_stream_),
                      "gather pending hidden");
                draft_forward(streams, static_cast<const uint16_t *>(draft_hidden_in_.ptr), true);
            } else {
                draft_forward(streams, static_cast<const uint16_t *>(draft_normalized_.ptr), true);
            }
            check(launch_draft_select(static_cast<const uint32_t *>(records_.ptr), forced, j, streams, drafts, draft_tokens, verify_tokens,
                                      cuda_stream_),
                  "draft select");
        }
    });
    cuda_check(cudaEventRecord(event_a_, cuda_stream_), "event record");

    // ---- verify: all candidates of all streams in one batch of lanes
    run_phase({1, streams, drafts, splits, stochastic_streams_ != 0 ? 1 : 0, stack_enabled_ ? 1 : 0}, [&] {
        current_lanes_ = LaneTable{verify_positions, verify_slots};
        current_tokens_ = verify_tokens;
        current_width_ = width;
        target_forward(lanes, true);
    });
    cuda_check(cudaEventRecord(event_b_, cuda_stream_), "event record");

    // ---- accept on the device, then the draft catch-up over the same lanes: state steps for the verify inputs
    // with the target's hidden states.  Lanes beyond the committed prefix write slots that the next cycle
    // overwrites before reading (like the draft loop's own tentative writes in the reference).
    const size_t row_words = 4 + 2 * width;
    run_phase({2, streams, drafts, splits, stochastic_streams_ != 0 ? 1 : 0, stack_enabled_ ? 1 : 0}, [&] {
        current_lanes_ = LaneTable{verify_positions, verify_slots};
        current_tokens_ = verify_tokens;
        current_width_ = width;
        check(launch_shift_hidden(static_cast<const uint16_t *>(pending_hidden_.ptr), stream_slots, static_cast<const uint16_t *>(normalized_.ptr),
                                  static_cast<uint16_t *>(draft_hidden_in_.ptr), streams, width, static_cast<int>(plan.hidden), cuda_stream_),
              "catch-up hidden");
        check(launch_accept(verify_tokens, static_cast<const uint32_t *>(records_.ptr), stop_tokens, stop_counts, MAX_STOP_TOKENS, streams, drafts,
                            accept_rows, static_cast<const uint16_t *>(normalized_.ptr), static_cast<uint16_t *>(pending_hidden_.ptr), stream_slots,
                            static_cast<int>(plan.hidden), cuda_stream_),
              "accept");
        draft_forward(lanes, static_cast<const uint16_t *>(draft_hidden_in_.ptr), false);
    });
    cuda_check(cudaEventRecord(event_end_, cuda_stream_), "event record");
    cuda_check(cudaMemcpyAsync(host_records_, accept_rows, streams * row_words * sizeof(uint32_t), cudaMemcpyDeviceToHost, cuda_stream_),
               "accept readback");
    uint32_t *status_word = host_records_ + static_cast<size_t>(streams) * row_words;
    cuda_check(cudaMemcpyAsync(status_word, kernel_error_.ptr, sizeof(int), cudaMemcpyDeviceToHost, cuda_stream_), "kernel status readback");
    counters_.d2h_bytes += streams * row_words * 4 + 4;
    synchronize("cycle synchronize");
    check_kernel_status(status_word);  // nothing of a failed cycle is emitted
    float verify_ms = 0.0f, draft_ms = 0.0f, catch_up_ms = 0.0f;
    cuda_check(cudaEventElapsedTime(&verify_ms, event_a_, event_b_), "event elapsed");
    cuda_check(cudaEventElapsedTime(&draft_ms, event_begin_, event_a_), "event elapsed");
    cuda_check(cudaEventElapsedTime(&catch_up_ms, event_b_, event_end_), "event elapsed");
    report.verify_ms_sum += verify_ms;
    report.verify_steps++;
    uint64_t kv_bytes = 0;
    for (int s = 0; s < streams; s++) kv_bytes += model_->kv_bytes_per_token() * std::min<uint64_t>(batch[s]->next_tick + width, model_->capacity());
    report.verify_bytes += model_->target_step_weight_bytes() + kv_bytes;

    for (int s = 0; s < streams; s++) {
        Stream &st = *batch[s];
        const uint32_t *row = host_records_ + s * row_words;
        uint32_t accepted = row[0], committed = row[1], count = row[2];
        report.speculative.cycle_count++;
        report.speculative.proposed_draft_token_count += drafts;
        report.speculative.accepted_draft_token_count += accepted;
        report.speculative.emitted_token_count += count;
        if (log_cycles_) {
            CycleRecord record;
            record.stream_id = st.id;
            record.start_tick = st.next_tick;
            record.accepted = accepted;
            record.committed = committed;
            record.emitted_token_ids.assign(row + 4, row + 4 + count);
            record.target_token_ids.assign(row + 4 + width, row + 4 + 2 * width);
            cycle_log_.push_back(std::move(record));
        }
        st.active->has_feedback = false;
        const uint32_t fed_back = st.active->feedback_token;  // the input of the cycle's first tick; every later tick takes the token before it
        for (uint32_t i = 0; i < count; i++) {
            uint64_t tick = st.next_tick;
            if (prefix_cache_on() && st.history.size() == st.next_tick) st.history.push_back(i == 0 ? fed_back : row[4 + i - 1]);
            st.next_tick += 1;
            emit(st, row[4 + i], tick, on_output, report);
        }
    }
    report.speculative.target_verification_time_ns += static_cast<uint64_t>(verify_ms * 1e6);
    report.speculative.draft_time_ns += static_cast<uint64_t>(draft_ms * 1e6);            // feedback_generation.rs:100-131
    report.speculative.draft_catch_up_time_ns += static_cast<uint64_t>(catch_up_ms * 1e6);  // feedback_generation.rs:160-174 (acceptance included)
}

// ---------------------------------------------------------------------------- run loop

RunReport Engine::run_until_idle(const std::function<void(const OutputEvent &)> &on_output) { return run(0, on_output); }

RunReport Engine::run(uint64_t max_batches, const std::function<void(const OutputEvent &)> &on_output) {
    if (failed_) fail("this tensor-parallel rank gave up waiting for its peers in an earlier run: the group's engines must be created anew");
    RunReport report;
    counters_ = ExecCounters{};
    profile_ms_ = 0.0;
    profile_bytes_ = profile_launches_ = 0;
    cuda_check(cudaEventRecord(run_begin_, cuda_stream_), "event record");
    // One scheduled activation in execution: the stream, where it stood, and what it has emitted so far.
    struct Work {
        runtime::Activation activation;
        Stream *stream;
        uint64_t start_tick;
        size_t emitted_before;
        std::vector<uint32_t> generated;
    };
    auto note_generated = [](Work &work) {
        if (work.stream->active == nullptr) return;
        const std::vector<uint32_t> &all = work.stream->active->generated;
        work.generated.assign(all.begin() + static_cast<std::ptrdiff_t>(std::min(work.emitted_before, all.size())), all.end());
    };
    auto run_ticks_in_batches = [&](std::vector<Stream *> &streams) {
        const size_t per_batch = model_->options().max_lanes;
        for (size_t offset = 0; offset < streams.size(); offset += per_batch) {
            std::vector<Stream *> batch(streams.begin() + offset, streams.begin() + std::min(streams.size(), offset + per_batch));
            run_single_ticks(batch, on_output, report);
            report.batch_count++;
            report.activation_count += batch.size();
            report.max_batch_width = std::max<uint64_t>(report.max_batch_width, batch.size());
        }
    };
    while (true) {
        if (max_batches && report.batch_count >= max_batches) {
            report.idle = false;
            break;
        }
        // 0. control steps: events that were stopped from outside still feed their last token back (the closing
        // tick, placed_prompt_event.rs:320-341); the scheduler no longer tracks them
        {
            std::vector<Stream *> closing;
            for (auto &entry : streams_) {
                Stream &s = entry.second;
                if (!s.detached) continue;
                s.detached = false;
                if (!s.active) continue;
                if (s.active->has_feedback) {
                    closing.push_back(&s);
                } else {
                    s.active.reset();
                    s.completed_events++;
                }
            }
            if (!closing.empty()) {
                uint64_t start = now_ns();
                run_ticks_in_batches(closing);
                report.decode_ns += now_ns() - start;
            }
        }
        // 1. the scheduler's step: at most one activation per stream - a prefill chunk or a decode window
        size_t widest_window = 1;
        for (auto &entry : streams_) widest_window = std::max<size_t>(widest_window, static_cast<size_t>(entry.second.k) + 1);
        const size_t chunk_budget = static_cast<size_t>(std::max(1, std::min(prefill_chunk_, model_->options().max_lanes)));
        const runtime::SchedulerBudget budget =
            runtime::SchedulerBudget(std::max<size_t>(1, streams_.size()), chunk_budget, std::numeric_limits<size_t>::max())
                .with_max_decode_tokens_per_activation(widest_window);
        std::vector<runtime::Activation> scheduled;
        if (!carried_activations_.empty()) {
            scheduled.swap(carried_activations_);  // the activations of a batch that failed: the same work again
        } else {
            scheduled = scheduler_.schedule_step(budget).activations;
        }
        if (scheduled.empty()) break;
        std::vector<Work> works;
        works.reserve(scheduled.size());
        for (runtime::Activation &activation : scheduled) {
            Stream &s = stream(std::stoll(activation.stream_id));
            activate_next_event(s);
            if (!s.active) fail("scheduler activation for stream " + activation.stream_id + " without an input event");
            works.push_back(Work{std::move(activation), &s, s.next_tick, s.active->generated.size(), {}});
        }
        try {
        // 2. prefill chunks, one stream at a time
        for (Work &work : works) {
            if (work.activation.kind != runtime::ActivationKind::PrefillChunk) continue;
            Stream &s = *work.stream;
            ActiveEvent &event = *s.active;
            if (event.next_external != work.activation.token_offset || event.input.token_ids.size() < work.activation.token_offset + work.activation.token_ids.size())
                fail("scheduler and engine disagree about the prompt position of stream " + work.activation.stream_id);
            uint64_t start = now_ns();
            size_t left = work.activation.token_ids.size();
            const bool ends_prompt = work.activation.remaining_prompt_token_count == 0;
            while (left > 0) {
                int count = static_cast<int>(left);
                // A batch appends the K/V of all its lanes before any lane attends.  Once the KV ring wraps, a later
                // lane's slot is the one an earlier lane's window still ends in, and the reference runs the lanes one
                // after the other (append_gqa_attention_bf16.comp.template:189-215 per tick).  So a chunk stops at the
                // wrap, and beyond it every tick is a batch of its own.
                const uint64_t ring = model_->capacity();
                if (s.next_tick + static_cast<uint64_t>(count) > ring) count = s.next_tick < ring ? static_cast<int>(ring - s.next_tick) : 1;
                // with the prefix cache on, a chunk also stops at the prompt's last page boundary: the state there is retained
                const uint64_t checkpoint_tick = prefix_checkpoint_tick(s);
                if (checkpoint_tick > s.next_tick && checkpoint_tick < s.next_tick + static_cast<uint64_t>(count)) count = static_cast<int>(checkpoint_tick - s.next_tick);
                const bool last = ends_prompt && static_cast<size_t>(count) == left;
                const bool sample = last && event.remaining > 0;
                uint32_t sampled = 0;
                const uint64_t tick_of_last = s.next_tick + count - 1;
                run_prefill_chunk(s, event.input.token_ids.data() + event.next_external, count, sample, &sampled);
                if (prefix_cache_on() && s.history.size() + static_cast<size_t>(count) == s.next_tick) {
                    s.history.insert(s.history.end(), event.input.token_ids.begin() + static_cast<std::ptrdiff_t>(event.next_external),
                                     event.input.token_ids.begin() + static_cast<std::ptrdiff_t>(event.next_external + count));
                    if (checkpoint_tick != 0 && s.next_tick == checkpoint_tick) capture_prefix_checkpoint(s);
                }
                event.next_external += count;
                left -= static_cast<size_t>(count);
                report.prefill_tokens += count;
                if (sample) emit(s, sampled, tick_of_last, on_output, report);
                else if (last) {
                    synchronize("prefill synchronize");
                    note_generated(work);
                    s.active.reset();  // no public outputs requested: the event ends with the prompt
                    s.completed_events++;
                }
            }
            report.activation_count++;
            report.prefill_ns += now_ns() - start;
        }
        // 3. decode windows: grouped into speculative cycles of equal draft count and single ticks
        std::map<int, std::vector<Stream *>> speculative;
        std::vector<Stream *> single;
        for (Work &work : works) {
            if (work.activation.kind != runtime::ActivationKind::DecodeFeedback) continue;
            Stream &s = *work.stream;
            ActiveEvent &event = *s.active;
            if (!event.has_feedback) fail("scheduler decode window for stream " + work.activation.stream_id + " without a token to feed back");
            const size_t window = std::min<size_t>(work.activation.max_tokens, event.remaining);
            // no speculation across or beyond the wrap of the KV ring (see the prefill chunks above): the rejected
            // lanes of a cycle would also overwrite slots that are still inside the window
            const bool ring_wraps = s.next_tick + static_cast<uint64_t>(s.k) + 1 > model_->capacity();
            if (s.k > 0 && model_->plan().has_draft && !event.feedback_closes && window >= 2 && !ring_wraps) {
                int drafts = static_cast<int>(std::min<size_t>(s.k, window - 1));
                speculative[drafts].push_back(&s);
            } else {
                single.push_back(&s);
            }
        }
        uint64_t start = now_ns();
        for (auto &group : speculative) {
            // split groups that would exceed the lane budget
            size_t per_batch = std::max<size_t>(1, model_->options().max_lanes / (group.first + 1));
            for (size_t offset = 0; offset < group.second.size(); offset += per_batch) {
                std::vector<Stream *> batch(group.second.begin() + offset,
                                            group.second.begin() + std::min(group.second.size(), offset + per_batch));
                run_speculative_cycles(batch, group.first, on_output, report);
                report.batch_count++;
                report.activation_count += batch.size();
                report.max_batch_width = std::max<uint64_t>(report.max_batch_width, batch.size());
            }
        }
        if (!single.empty()) run_ticks_in_batches(single);
        // 4. what the activations emitted; then the closing tick of every event that has emitted its last token (the
        // scheduler reserves one state activation beyond the window for it, stream_runtime.rs:1262-1290)
        std::vector<Stream *> closing;
        for (Work &work : works) {
            note_generated(work);
            Stream &s = *work.stream;
            if (s.active && s.active->has_feedback && s.active->feedback_closes) closing.push_back(&s);
        }
        if (!closing.empty()) run_ticks_in_batches(closing);
        report.decode_ns += now_ns() - start;
        // 5. outcomes: generated tokens, whether the event goes on, and the ticks the stream advanced by
        for (Work &work : works) {
            Stream &s = *work.stream;
            runtime::ActivationOutcome outcome;
            outcome.generated_token_ids = work.generated;
            outcome.continue_generation = s.active != nullptr;
            outcome.processed_state_activation_count = static_cast<size_t>(s.next_tick - work.start_tick);
            scheduler_.complete_activation(work.activation.id, outcome);
        }
        } catch (...) {
            // A batch failed and was discarded: its streams stand where they stood.  Activations that did run are
            // completed (an event that still owes its closing tick gets it as a control step of the next run), the
            // others are carried into the next run, which repeats them before it asks the scheduler for more.
            for (Work &work : works) {
                Stream &s = *work.stream;
                note_generated(work);
                const bool ran = s.next_tick != work.start_tick || !work.generated.empty() || s.active == nullptr;
                if (!ran) {
                    carried_activations_.push_back(work.activation);
                    continue;
                }
                runtime::ActivationOutcome outcome;
                outcome.generated_token_ids = work.generated;
                const bool owes_closing_tick = s.active && s.active->has_feedback && s.active->feedback_closes;
                outcome.continue_generation = s.active != nullptr && !owes_closing_tick;
                outcome.processed_state_activation_count = static_cast<size_t>(s.next_tick - work.start_tick);
                if (owes_closing_tick) s.detached = true;
                try {
                    scheduler_.complete_activation(work.activation.id, outcome);
                } catch (...) {
                }
            }
            throw;
        }
    }
    cuda_check(cudaEventRecord(run_end_, cuda_stream_), "event record");
    cuda_check(cudaMemcpyAsync(host_records_, kernel_error_.ptr, sizeof(int), cudaMemcpyDeviceToHost, cuda_stream_), "kernel status readback");
    synchronize("run synchronize");
    check_kernel_status(host_records_);  // batches that read nothing back (prompt chunks without a sampled token)
    float device_ms = 0.0f;
    cuda_check(cudaEventElapsedTime(&device_ms, run_begin_, run_end_), "event elapsed");
    report.device_ms = device_ms;
    report.int4_ms = profile_ms_;
    report.int4_bytes = profile_bytes_;
    report.int4_launches = profile_launches_;
    report.counters = counters_;
    return report;
}

void Engine::debug_target_logits(int64_t id, const std::vector<uint32_t> &tokens, float *logits_out, uint16_t *hidden_out) {
    Stream &s = stream(id);
    const ModelPlan &plan = model_->plan();
    const int lanes = static_cast<int>(tokens.size());
    if (lanes <= 0 || lanes > model_->options().max_lanes) fail("debug_target_logits: lane count outside [1, max_lanes]");
    ensure_pages(s, s.next_tick + lanes - 1);
    sync_block_tables();
    std::vector<uint32_t> positions(lanes);
    std::vector<int32_t> slots(lanes, s.slot);
    for (int i = 0; i < lanes; i++) positions[i] = static_cast<uint32_t>(s.next_tick + i);
    upload_lanes(positions, slots);
    upload_tokens(tokens.data(), lanes);
    current_width_ = lanes;
    full_logits_ = true;  // the whole vocabulary on every rank, whatever the sampling path would project
    try {
        target_forward(lanes, true);
    } catch (...) {
        full_logits_ = false;
        throw;
    }
    full_logits_ = false;
    synchronize("debug synchronize");
    if (logits_out)
        cuda_check(cudaMemcpy(logits_out, logits_.ptr, static_cast<size_t>(lanes) * plan.vocab * sizeof(float), cudaMemcpyDeviceToHost), "logits readback");
    if (hidden_out)
        cuda_check(cudaMemcpy(hidden_out, normalized_.ptr, static_cast<size_t>(lanes) * plan.hidden * 2, cudaMemcpyDeviceToHost), "hidden readback");
}

}  // namespace nerve
