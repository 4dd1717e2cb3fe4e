// extern "C" surface declared in include/nerve_b200.h: exception -> status + thread-local message.
#include <cstring>
#include <exception>
#include <string>

#include "../../include/nerve_b200.h"
#include "engine.hpp"
#include "state_abi.hpp"
#include "stream_runtime.hpp"

using namespace nerve;

struct nerve_b200_package {
    std::shared_ptr<MountedModel> model;
    int references = 1;
};

struct nerve_b200_engine {
    nerve_b200_package *package;
    std::unique_ptr<Engine> engine;
};

struct nerve_b200_scheduler {
    nerve::runtime::StreamScheduler scheduler;
    nerve::runtime::SchedulerStep step;  // the last schedule_step, read back by index
};

namespace {

thread_local std::string last_error;

template <typename Body>
int32_t guarded(Body body) {
    try {
        body();
        return NERVE_B200_OK;
    } catch (const std::exception &error) {
        last_error = error.what();
    } catch (...) {
        last_error = "unknown failure";
    }
    return NERVE_B200_ERROR;
}

void require(bool condition, const char *message) {
    if (!condition) throw std::runtime_error(message);
}

int32_t cuda_status(cudaError_t status, const char *what) {
    if (status == cudaSuccess) return NERVE_B200_OK;
    last_error = std::string(what) + ": " + cudaGetErrorString(status);
    return NERVE_B200_ERROR;
}

void copy_text(char (&out)[64], const std::string &text) {
    const size_t count = text.size() < 63 ? text.size() : 63;
    std::memcpy(out, text.data(), count);
    out[count] = 0;
}

void fill_snapshot(nerve_b200_stream_snapshot *out, const nerve::runtime::StreamSnapshot &snapshot) {
    if (out == nullptr) return;
    out->status = static_cast<int32_t>(snapshot.status);
    out->queued_input_event_count = snapshot.queued_input_event_count;
    out->in_flight_activation_count = snapshot.in_flight_activation_count;
    out->completed_input_event_count = snapshot.completed_input_event_count;
    out->scheduled_activation_count = snapshot.scheduled_activation_count;
    out->generated_token_count = snapshot.generated_token_count;
    out->transient_state_entry_count = snapshot.transient_state_entry_count;
    out->transient_state_block_count = snapshot.transient_state_block_count;
    out->transient_state_logical_activation_count = snapshot.transient_state_logical_activation_count;
    copy_text(out->current_input_event_id, snapshot.current_input_event_id.value_or(""));
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

const char *nerve_b200_last_error(void) { return last_error.c_str(); }
int32_t nerve_b200_abi_version(void) { return 1; }

int32_t nerve_b200_package_mount(const char *path, const nerve_b200_mount_options *options, nerve_b200_package **out_package) {
    return guarded([&] {
        require(path && options && out_package, "nerve_b200_package_mount: null argument");
        MountOptions mount;
        mount.device = options->device;
        mount.capacity_tokens = options->capacity_tokens;
        mount.page_tokens = options->page_tokens;
        mount.max_streams = options->max_streams;
        mount.max_lanes = options->max_lanes;
        mount.verify_level = options->verify_level;
        mount.tp_rank = options->tp_rank;
        mount.tp_size = options->tp_size > 0 ? options->tp_size : 1;
        mount.extra_pages = options->extra_pages;
        require(mount.tp_rank >= 0 && mount.tp_rank < mount.tp_size, "tp_rank must be in [0, tp_size)");
        auto package = new nerve_b200_package();
        try {
            package->model = MountedModel::mount(path, mount);
        } catch (...) {
            delete package;
            throw;
        }
        *out_package = package;
    });
}

int32_t nerve_b200_package_unmount(nerve_b200_package *package) {
    return guarded([&] {
        require(package != nullptr, "nerve_b200_package_unmount: null package");
        if (--package->references == 0) delete package;
    });
}

int32_t nerve_b200_package_describe(const nerve_b200_package *package, nerve_b200_package_info *out) {
    return guarded([&] {
        require(package && out, "nerve_b200_package_describe: null argument");
        const MountedModel &model = *package->model;
        const ModelPlan &plan = model.plan();
        std::memset(out, 0, sizeof(*out));
        out->hidden_size = plan.hidden;
        out->vocab_size = plan.vocab;
        out->layer_count = static_cast<int64_t>(plan.layers.size());
        out->max_context = plan.max_context;
        out->has_speculative_decoder = plan.has_draft ? 1 : 0;
        out->kv_layer_count = model.kv_layer_count();
        out->weight_bytes = model.weight_bytes();
        out->verify_step_weight_bytes = model.target_step_weight_bytes();
        out->draft_step_weight_bytes = model.draft_step_weight_bytes();
        out->kv_bytes_per_token = model.kv_bytes_per_token();
        out->pages_per_stream = model.pages_per_stream();
        out->physical_pages = model.physical_pages();
        out->page_tokens = model.options().page_tokens;
        out->eos_token_id = plan.eos_token_ids.empty() ? 0xffffffffu : plan.eos_token_ids[0];
        out->target_decode_stack = model.target_stack().available ? 1 : 0;
        out->draft_decode_stack = model.draft_stack().available ? 1 : 0;
        out->target_stack_weight_bytes = model.target_stack().weight_bytes;
    });
}

int32_t nerve_b200_package_validate(const char *path, int32_t verify_level, int64_t *out_op_count, int64_t *out_tensor_count) {
    return guarded([&] {
        require(path != nullptr, "nerve_b200_package_validate: null path");
        VerifyLevel level = verify_level >= 2 ? VerifyLevel::All : (verify_level == 1 ? VerifyLevel::Used : VerifyLevel::None);
        auto package = HostPackage::open(path, level);
        if (verify_level >= 1)
            for (const auto &entry : package->tensors())
                if (entry.second.dtype != "I64") (void)package->read_tensor(entry.first, true);
        int64_t ops = 0;
        const ModelPlan &plan = package->plan();
        for (const ComponentPlan &layer : plan.layers) ops += static_cast<int64_t>(layer.ops.size());
        ops += static_cast<int64_t>(plan.draft_adapter.ops.size());
        for (const ComponentPlan &layer : plan.draft_layers) ops += static_cast<int64_t>(layer.ops.size());
        if (out_op_count) *out_op_count = ops;
        if (out_tensor_count) *out_tensor_count = static_cast<int64_t>(package->tensors().size());
    });
}

int32_t nerve_b200_engine_create(nerve_b200_package *package, nerve_b200_engine **out_engine) {
    return guarded([&] {
        require(package && out_engine, "nerve_b200_engine_create: null argument");
        auto engine = new nerve_b200_engine();
        try {
            engine->engine = std::make_unique<Engine>(package->model);
        } catch (...) {
            delete engine;
            throw;
        }
        engine->package = package;
        package->references++;
        *out_engine = engine;
    });
}

int32_t nerve_b200_engine_destroy(nerve_b200_engine *engine) {
    return guarded([&] {
        require(engine != nullptr, "nerve_b200_engine_destroy: null engine");
        nerve_b200_package *package = engine->package;
        engine->engine.reset();
        delete engine;
        if (--package->references == 0) delete package;
    });
}

int32_t nerve_b200_engine_add_stream(nerve_b200_engine *engine, int64_t stream_id, uint32_t seed, int32_t drafts,
                                     const nerve_b200_sampler_config *sampler) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        SamplerConfig config;
        if (sampler) {
            config.method = sampler->method;
            config.temperature = sampler->temperature;
            config.top_p = sampler->top_p;
            config.min_p = sampler->min_p;
            config.top_k = sampler->top_k;
        }
        engine->engine->add_stream(stream_id, seed, drafts, config);
    });
}

int32_t nerve_b200_engine_fork_stream(nerve_b200_engine *engine, int64_t source, int64_t destination, uint32_t seed) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->fork_stream(source, destination, seed);
    });
}

int32_t nerve_b200_engine_reset_stream(nerve_b200_engine *engine, int64_t stream_id) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->reset_stream(stream_id);
    });
}

int32_t nerve_b200_engine_remove_stream(nerve_b200_engine *engine, int64_t stream_id) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->remove_stream(stream_id);
    });
}

int32_t nerve_b200_engine_interrupt_stream(nerve_b200_engine *engine, int64_t stream_id) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->interrupt_stream(stream_id);
    });
}

int32_t nerve_b200_engine_enqueue(nerve_b200_engine *engine, int64_t stream_id, const char *event_id, const uint32_t *token_ids,
                                  size_t token_count, size_t max_public_tokens, const uint32_t *stop_token_ids, size_t stop_token_count) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        require(token_ids != nullptr || token_count == 0, "null token_ids");
        InputEvent event;
        event.id = event_id ? event_id : "";
        event.token_ids.assign(token_ids, token_ids + token_count);
        event.max_public_tokens = max_public_tokens;
        if (stop_token_count) event.stop_token_ids.assign(stop_token_ids, stop_token_ids + stop_token_count);
        engine->engine->enqueue(stream_id, event);
    });
}

int32_t nerve_b200_engine_run_until_idle(nerve_b200_engine *engine, nerve_b200_output_callback on_output, void *user,
                                         nerve_b200_run_report *out) {
    return nerve_b200_engine_run(engine, 0, on_output, user, out);
}

int32_t nerve_b200_tp_shard_range(int64_t total, int64_t unit, int32_t rank, int32_t size, int64_t *out_begin, int64_t *out_count) {
    return guarded([&] {
        require(out_begin && out_count, "null output");
        tp_shard_range(total, unit, rank, size, *out_begin, *out_count);
    });
}

int32_t nerve_b200_tp_unique_id(const char *nccl_library_path, uint8_t *out_128_bytes) {
    return guarded([&] {
        require(nccl_library_path && out_128_bytes, "null argument");
        Engine::tensor_parallel_unique_id(nccl_library_path, out_128_bytes);
    });
}

int32_t nerve_b200_engine_init_tp(nerve_b200_engine *engine, const char *nccl_library_path, int32_t rank, int32_t size,
                                  const uint8_t *unique_id_128_bytes) {
    return guarded([&] {
        require(engine && nccl_library_path && unique_id_128_bytes, "null argument");
        engine->engine->init_tensor_parallel(nccl_library_path, rank, size, unique_id_128_bytes);
    });
}

int32_t nerve_b200_engine_stop_after_current(nerve_b200_engine *engine, int64_t stream_id) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->stop_stream_after_current(stream_id);
    });
}

int32_t nerve_b200_engine_stream_snapshot_of(nerve_b200_engine *engine, int64_t stream_id, nerve_b200_engine_stream_snapshot *out) {
    return guarded([&] {
        require(engine != nullptr && out != nullptr, "null argument");
        const Engine::StreamSnapshot snapshot = engine->engine->stream_snapshot(stream_id);
        out->pending_input_event_count = snapshot.pending_input_event_count;
        out->next_stream_tick = snapshot.next_stream_tick;
        out->completed_prompt_event_count = snapshot.completed_prompt_event_count;
        out->context_window_activations = snapshot.context_window_activations;
        out->mapped_state_pages = snapshot.mapped_state_pages;
        out->speculative_draft_tokens = snapshot.speculative_draft_tokens;
        out->idle = snapshot.idle ? 1 : 0;
    });
}

int32_t nerve_b200_engine_scheduler_stream_counts(nerve_b200_engine *engine, int64_t stream_id, uint64_t out_counts[6]) {
    return guarded([&] {
        require(engine != nullptr && out_counts != nullptr, "null argument");
        engine->engine->scheduler_stream_counts(stream_id, out_counts);
    });
}

int32_t nerve_b200_engine_set_prefix_cache_capacity(nerve_b200_engine *engine, uint64_t entries) {
    return guarded([&] {
        require(engine != nullptr, "null argument");
        engine->engine->set_prefix_cache_capacity(static_cast<size_t>(entries));
    });
}

int32_t nerve_b200_engine_prefix_cache_stats(nerve_b200_engine *engine, uint64_t out_stats[8]) {
    return guarded([&] {
        require(engine != nullptr && out_stats != nullptr, "null argument");
        const Engine::PrefixCacheStats stats = engine->engine->prefix_cache_stats();
        const uint64_t values[8] = {stats.hit_count,          stats.miss_count,
                                    stats.insertion_count,    stats.eviction_count,
                                    stats.reused_token_count, stats.saved_prefill_token_count,
                                    stats.resident_entry_count, stats.resident_byte_count};
        for (int i = 0; i < 8; i++) out_stats[i] = values[i];
    });
}

int32_t nerve_b200_engine_snapshot(nerve_b200_engine *engine, nerve_b200_engine_snapshot_counts *out) {
    return guarded([&] {
        require(engine != nullptr && out != nullptr, "null argument");
        const Engine::EngineSnapshot snapshot = engine->engine->snapshot();
        out->stream_count = snapshot.stream_count;
        out->active_stream_count = snapshot.active_stream_count;
        out->idle = snapshot.idle ? 1 : 0;
    });
}

int32_t nerve_b200_engine_tp_exchange_handle(nerve_b200_engine *engine, uint8_t *out_64_bytes) {
    return guarded([&] {
        require(engine && out_64_bytes, "null argument");
        engine->engine->tp_exchange_handle(out_64_bytes);
    });
}

int32_t nerve_b200_engine_tp_connect(nerve_b200_engine *engine, const uint8_t *handles_64_bytes_each, int32_t count) {
    return guarded([&] {
        require(engine && handles_64_bytes_each, "null argument");
        engine->engine->tp_connect(handles_64_bytes_each, count);
    });
}

int32_t nerve_b200_engine_set_decode_stack(nerve_b200_engine *engine, int32_t enabled) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->set_decode_stack(enabled != 0);
    });
}

int32_t nerve_b200_engine_decode_stack_timing(nerve_b200_engine *engine, uint64_t *out_stamps, size_t max_stamps, size_t *out_count) {
    return guarded([&] {
        require(engine && out_count, "null argument");
        std::vector<unsigned long long> stamps = engine->engine->decode_stack_timing();
        *out_count = stamps.size();
        for (size_t i = 0; i < stamps.size() && i < max_stamps && out_stamps; i++) out_stamps[i] = stamps[i];
    });
}

int32_t nerve_b200_engine_set_profiling(nerve_b200_engine *engine, int32_t enabled) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->set_profiling(enabled != 0);
    });
}

int32_t nerve_b200_engine_inject_barrier_timeouts(nerve_b200_engine *engine, int32_t launches) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        require(launches >= 0, "launches must not be negative");
        engine->engine->inject_barrier_timeouts(launches);
    });
}

int32_t nerve_b200_engine_run(nerve_b200_engine *engine, uint64_t max_batches, nerve_b200_output_callback on_output, void *user,
                              nerve_b200_run_report *out) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        RunReport report = engine->engine->run(max_batches, [&](const OutputEvent &event) {
            if (on_output) on_output(user, event.stream_id, event.token_id, event.source_stream_tick, event.output_index);
        });
        if (out) {
            std::memset(out, 0, sizeof(*out));
            out->prefill_ns = report.prefill_ns;
            out->decode_ns = report.decode_ns;
            out->prefill_tokens = report.prefill_tokens;
            out->generated_tokens = report.generated_tokens;
            out->activation_count = report.activation_count;
            out->batch_count = report.batch_count;
            out->max_batch_width = report.max_batch_width;
            out->cycle_count = report.speculative.cycle_count;
            out->proposed_draft_token_count = report.speculative.proposed_draft_token_count;
            out->accepted_draft_token_count = report.speculative.accepted_draft_token_count;
            out->emitted_token_count = report.speculative.emitted_token_count;
            out->draft_time_ns = report.speculative.draft_time_ns;
            out->target_verification_time_ns = report.speculative.target_verification_time_ns;
            out->draft_catch_up_time_ns = report.speculative.draft_catch_up_time_ns;
            out->kernel_launches = report.counters.kernel_launches;
            out->graph_launches = report.counters.graph_launches;
            out->h2d_bytes = report.counters.h2d_bytes;
            out->d2h_bytes = report.counters.d2h_bytes;
            out->host_syncs = report.counters.host_syncs;
            out->verify_ms_sum = report.verify_ms_sum;
            out->verify_steps = report.verify_steps;
            out->verify_bytes = report.verify_bytes;
            out->device_ms = report.device_ms;
            out->int4_ms = report.int4_ms;
            out->int4_bytes = report.int4_bytes;
            out->int4_launches = report.int4_launches;
            out->idle = report.idle ? 1 : 0;
        }
    });
}

int32_t nerve_b200_engine_stream_tick(const nerve_b200_engine *engine, int64_t stream_id, uint64_t *out_tick) {
    return guarded([&] {
        require(engine && out_tick, "null argument");
        *out_tick = engine->engine->stream_tick(stream_id);
    });
}

int32_t nerve_b200_engine_set_teacher_tokens(nerve_b200_engine *engine, int64_t stream_id, const uint32_t *tokens, size_t count) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->set_teacher_tokens(stream_id, std::vector<uint32_t>(tokens, tokens + count));
    });
}

int32_t nerve_b200_engine_set_prefill_chunk(nerve_b200_engine *engine, int32_t tokens) {
    return guarded([&] {
        require(engine != nullptr && tokens > 0, "prefill chunk must be positive");
        engine->engine->set_prefill_chunk(tokens);
    });
}

int32_t nerve_b200_engine_set_cycle_logging(nerve_b200_engine *engine, int32_t enabled) {
    return guarded([&] {
        require(engine != nullptr, "null engine");
        engine->engine->set_cycle_logging(enabled != 0);
    });
}

int32_t nerve_b200_engine_cycle_log(const nerve_b200_engine *engine, uint64_t *out_rows, size_t max_rows, size_t *out_count) {
    return guarded([&] {
        require(engine && out_count, "null argument");
        const auto &log = engine->engine->cycle_log();
        *out_count = log.size();
        for (size_t i = 0; i < log.size() && i < max_rows; i++) {
            uint64_t *row = out_rows + i * 22;
            std::memset(row, 0, 22 * sizeof(uint64_t));
            row[0] = static_cast<uint64_t>(log[i].stream_id);
            row[1] = log[i].start_tick;
            row[2] = log[i].accepted;
            row[3] = log[i].committed;
            row[4] = log[i].emitted_token_ids.size();
            row[5] = log[i].target_token_ids.size();
            for (size_t j = 0; j < log[i].emitted_token_ids.size() && j < 8; j++) row[6 + j] = log[i].emitted_token_ids[j];
            for (size_t j = 0; j < log[i].target_token_ids.size() && j < 8; j++) row[14 + j] = log[i].target_token_ids[j];
        }
    });
}

int32_t nerve_b200_debug_target_logits(nerve_b200_engine *engine, int64_t stream_id, const uint32_t *tokens, size_t count,
                                       float *out_logits, uint16_t *out_hidden) {
    return guarded([&] {
        require(engine && tokens, "null argument");
        engine->engine->debug_target_logits(stream_id, std::vector<uint32_t>(tokens, tokens + count), out_logits, out_hidden);
    });
}

// ---- operator-level entry points

int32_t nerve_b200_op_linear_int4(const void *x, const void *qweight, const void *scales, void *y, const void *residual, int32_t lanes,
                                  int32_t n, int32_t k, int32_t group, void *stream) {
    return cuda_status(launch_linear_int4(static_cast<const uint16_t *>(x), static_cast<const uint32_t *>(qweight),
                                          static_cast<const uint16_t *>(scales), static_cast<uint16_t *>(y),
                                          static_cast<const uint16_t *>(residual), lanes, n, k, group,
                                          residual ? EPILOGUE_RESIDUAL_ROUNDED : EPILOGUE_BF16, static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_linear_int4");
}

int32_t nerve_b200_op_linear_int4_silu_pair(const void *x, const void *gate_q, const void *gate_s, const void *up_q, const void *up_s,
                                            void *y, int32_t lanes, int32_t n, int32_t k, void *stream) {
    return cuda_status(launch_linear_int4_silu_pair(static_cast<const uint16_t *>(x), static_cast<const uint32_t *>(gate_q),
                                                    static_cast<const uint16_t *>(gate_s), static_cast<const uint32_t *>(up_q),
                                                    static_cast<const uint16_t *>(up_s), static_cast<uint16_t *>(y), lanes, n, k,
                                                    static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_linear_int4_silu_pair");
}

int32_t nerve_b200_op_linear_bf16(const void *x, const void *w, void *y, const void *residual, int32_t lanes, int32_t n, int32_t k,
                                  int32_t to_f32, float scale, void *stream) {
    int epilogue = to_f32 ? EPILOGUE_F32_SCALED : (residual ? EPILOGUE_RESIDUAL_ROUNDED : EPILOGUE_BF16);
    return cuda_status(launch_linear_bf16(static_cast<const uint16_t *>(x), static_cast<const uint16_t *>(w), y,
                                          static_cast<const uint16_t *>(residual), lanes, n, k, epilogue, scale,
                                          static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_linear_bf16");
}

int32_t nerve_b200_op_rms_norm(const void *x, const void *weight, void *y, int32_t lanes, int32_t width, float eps, float weight_offset,
                               void *stream) {
    return cuda_status(launch_rms_norm(static_cast<const uint16_t *>(x), static_cast<const uint16_t *>(weight), static_cast<uint16_t *>(y),
                                       lanes, width, eps, weight_offset, static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_rms_norm");
}

int32_t nerve_b200_op_linear_fp8(const void *x, const void *w, const void *wscale, void *y, const void *residual, void *xq_scratch,
                                 void *xscale_scratch, int32_t lanes, int32_t n, int32_t k, void *stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t status = cuda_status(launch_quantize_fp8(static_cast<const uint16_t *>(x), static_cast<uint8_t *>(xq_scratch),
                                                     static_cast<float *>(xscale_scratch), lanes, k, st),
                                 "nerve_b200_op_linear_fp8 (quantize)");
    if (status != NERVE_B200_OK) return status;
    return cuda_status(launch_linear_fp8(static_cast<const uint8_t *>(xq_scratch), static_cast<const float *>(xscale_scratch),
                                         static_cast<const uint8_t *>(w), static_cast<const uint16_t *>(wscale), static_cast<uint16_t *>(y),
                                         static_cast<const uint16_t *>(residual), lanes, n, k,
                                         residual ? EPILOGUE_RESIDUAL_F32 : EPILOGUE_BF16, st),
                       "nerve_b200_op_linear_fp8");
}

int32_t nerve_b200_op_greedy(const void *logits, void *records, void *scratch, int32_t lanes, int32_t vocab, void *stream) {
    if (scratch == nullptr) {
        last_error = "nerve_b200_op_greedy: scratch must hold nerve_b200_op_greedy_scratch_bytes(lanes) device bytes";
        return NERVE_B200_ERROR;
    }
    return cuda_status(launch_argmax(static_cast<const float *>(logits), static_cast<uint32_t *>(records), lanes, vocab, scratch,
                                     static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_greedy");
}

uint64_t nerve_b200_op_greedy_scratch_bytes(int32_t lanes) { return argmax_scratch_bytes(lanes); }

int32_t nerve_b200_op_sample_top_k_top_p(const void *logits, void *records, void *scratch, int32_t lanes, int32_t vocab, int32_t top_k,
                                         float temperature, float top_p, float min_p, uint32_t seed, const uint32_t *ticks_device,
                                         void *params_device, void *stream) {
    return guarded([&] {
        require(logits && records && scratch && params_device, "nerve_b200_op_sample_top_k_top_p: null pointer");
        require(top_k >= 1 && top_k <= SAMPLER_MAX_TOP_K, "top_k must be between 1 and 64");
        require(temperature > 0.0f && top_p > 0.0f && top_p <= 1.0f && min_p >= 0.0f && min_p <= 1.0f, "sampler parameters out of range");
        SamplerParams params{};
        params.method = 1;
        params.top_k = static_cast<uint32_t>(top_k);
        params.seed = seed;
        params.temperature = temperature;
        params.top_p = top_p;
        params.min_p = min_p;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        cudaError_t status = cudaMemcpyAsync(params_device, &params, sizeof(params), cudaMemcpyHostToDevice, st);
        if (status == cudaSuccess)
            status = launch_sample(static_cast<const float *>(logits), static_cast<uint32_t *>(records), lanes, vocab,
                                   static_cast<const SamplerParams *>(params_device), nullptr, ticks_device, scratch, st);
        if (status != cudaSuccess) throw std::runtime_error(std::string("nerve_b200_op_sample_top_k_top_p: ") + cudaGetErrorString(status));
    });
}

uint64_t nerve_b200_op_sample_scratch_bytes(int32_t lanes) { return sampler_scratch_bytes(lanes); }

int32_t nerve_b200_op_greedy_static(const void *logits, void *records, int32_t lanes, int32_t vocab, void *stream) {
    if (lanes < 0 || vocab <= 0 || logits == nullptr || records == nullptr) {
        last_error = "nerve_b200_op_greedy_static: null pointer or non-positive size";
        return NERVE_B200_ERROR;
    }
    if (lanes > argmax_static_max_lanes()) {
        last_error = "nerve_b200_op_greedy_static: " + std::to_string(lanes) + " lanes exceed the built-in scratch of " +
                     std::to_string(argmax_static_max_lanes()) + " lanes; use nerve_b200_op_greedy with a caller-provided scratch buffer";
        return NERVE_B200_ERROR;
    }
    return cuda_status(launch_argmax_static(static_cast<const float *>(logits), static_cast<uint32_t *>(records), lanes, vocab,
                                            static_cast<cudaStream_t>(stream)),
                       "nerve_b200_op_greedy_static");
}

int32_t nerve_b200_stream_control_bytes(uint32_t token_id, uint64_t stream_tick, uint32_t control_flags, uint32_t capacity,
                                        uint8_t *out_20_bytes) {
    return guarded([&] {
        require(out_20_bytes != nullptr, "null output");
        stream_control_bytes(token_id, stream_tick, control_flags, capacity, out_20_bytes);
    });
}

int32_t nerve_b200_state_page_table_bytes(int64_t static_bytes, int64_t bytes_per_activation, int64_t max_dynamic_activations,
                                          int64_t capacity_activations, const uint32_t *logical_to_physical, size_t mapping_count,
                                          uint8_t *out_bytes, size_t out_capacity, int64_t *out_layout) {
    return guarded([&] {
        StateLayout layout = state_layout(static_bytes, bytes_per_activation, max_dynamic_activations, capacity_activations);
        std::vector<uint32_t> mapping;
        if (logical_to_physical && mapping_count) mapping.assign(logical_to_physical, logical_to_physical + mapping_count);
        std::vector<uint8_t> bytes = state_page_table_bytes(layout, mapping);
        if (out_layout) {
            const int64_t values[7] = {layout.block_activation_capacity, layout.page_count, layout.page_bytes, layout.page_table_bytes,
                                       layout.static_offset, layout.dynamic_offset, layout.byte_capacity};
            std::memcpy(out_layout, values, sizeof(values));
        }
        if (out_bytes) {
            require(out_capacity >= bytes.size(), "output buffer is smaller than the page table");
            std::memcpy(out_bytes, bytes.data(), bytes.size());
        }
    });
}

int32_t nerve_b200_verify_prefix(const uint32_t *draft, size_t draft_count, const uint32_t *target, size_t target_count,
                                 const uint32_t *stop, size_t stop_count, uint32_t *out_counts, uint32_t *out_emitted,
                                 size_t *out_emitted_count) {
    return guarded([&] {
        require(out_counts && out_emitted && out_emitted_count, "null output");
        if (target_count != draft_count + 1)
            throw std::runtime_error("speculative verification has " + std::to_string(draft_count) + " draft tokens but " +
                                     std::to_string(target_count) + " target predictions; expected " + std::to_string(draft_count + 1));
        size_t accepted = 0;
        while (accepted < draft_count && draft[accepted] == target[accepted]) accepted++;
        size_t committed = accepted + 1, count = 0;
        for (size_t i = 0; i < accepted; i++) out_emitted[count++] = draft[i];
        out_emitted[count++] = target[accepted];
        for (size_t i = 0; i < count; i++) {
            bool is_stop = false;
            for (size_t s = 0; s < stop_count; s++) is_stop |= stop[s] == out_emitted[i];
            if (is_stop) {
                if (accepted > i + 1) accepted = i + 1;
                committed = i + 1;
                count = i + 1;
                break;
            }
        }
        out_counts[0] = static_cast<uint32_t>(accepted);
        out_counts[1] = static_cast<uint32_t>(committed);
        *out_emitted_count = count;
    });
}

// ---- stream scheduler (host only) ----------------------------------------------------------------------------

int32_t nerve_b200_scheduler_create(nerve_b200_scheduler **out) {
    return guarded([&] {
        require(out != nullptr, "out must not be NULL");
        *out = new nerve_b200_scheduler();
    });
}

int32_t nerve_b200_scheduler_destroy(nerve_b200_scheduler *scheduler) {
    return guarded([&] { delete scheduler; });
}

int32_t nerve_b200_scheduler_add_stream(nerve_b200_scheduler *scheduler, const char *stream_id, const char *execution_class_id,
                                        const nerve_b200_state_declaration *declarations, size_t declaration_count,
                                        nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr, "scheduler and stream_id must not be NULL");
        require(declaration_count == 0 || declarations != nullptr, "declarations must not be NULL");
        nerve::runtime::StreamScheduler::Declarations list;
        for (size_t i = 0; i < declaration_count; i++) {
            const nerve_b200_state_declaration &d = declarations[i];
            require(d.node_instance_id != nullptr && d.state_id != nullptr, "state key strings must not be NULL");
            nerve::runtime::BlockShape shape = d.retention == 1 ? nerve::runtime::BlockShape::mutable_singleton(d.bytes_per_activation)
                                                                : nerve::runtime::BlockShape::append(d.bytes_per_activation, d.activation_capacity);
            require(d.retention == 0 || d.retention == 1, "retention must be 0 (append) or 1 (mutable singleton)");
            if (d.maximum_activation_count != 0) shape = shape.with_maximum_activation_count(d.maximum_activation_count);
            list.emplace_back(nerve::runtime::StateKey{d.node_instance_id, d.state_id}, shape);
        }
        fill_snapshot(out, scheduler->scheduler.add_stream(stream_id, execution_class_id ? execution_class_id : "default", list));
    });
}

int32_t nerve_b200_scheduler_fork_stream(nerve_b200_scheduler *scheduler, const char *source_stream_id, const char *target_stream_id,
                                         const char *execution_class_id, nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && source_stream_id != nullptr && target_stream_id != nullptr && execution_class_id != nullptr,
                "scheduler and ids must not be NULL");
        fill_snapshot(out, scheduler->scheduler.fork_stream_transient_state(source_stream_id, target_stream_id, execution_class_id));
    });
}

int32_t nerve_b200_scheduler_enqueue(nerve_b200_scheduler *scheduler, const char *stream_id, const char *event_id,
                                     const uint32_t *token_ids, size_t token_count, uint64_t max_public_tokens,
                                     nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr && event_id != nullptr, "scheduler and ids must not be NULL");
        require(token_count == 0 || token_ids != nullptr, "token_ids must not be NULL");
        nerve::runtime::InputEvent event;
        event.id = event_id;
        event.token_ids.assign(token_ids, token_ids + token_count);
        event.max_public_tokens = max_public_tokens;
        fill_snapshot(out, scheduler->scheduler.enqueue_input_event(stream_id, event));
    });
}

int32_t nerve_b200_scheduler_interrupt(nerve_b200_scheduler *scheduler, const char *stream_id, const char *reason,
                                       nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr && reason != nullptr, "scheduler, stream_id and reason must not be NULL");
        fill_snapshot(out, scheduler->scheduler.interrupt_stream(stream_id, reason));
    });
}

int32_t nerve_b200_scheduler_reset_stream_state(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr, "scheduler and stream_id must not be NULL");
        fill_snapshot(out, scheduler->scheduler.reset_stream_transient_state(stream_id));
    });
}

int32_t nerve_b200_scheduler_remove_stream(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr, "scheduler and stream_id must not be NULL");
        fill_snapshot(out, scheduler->scheduler.remove_stream(stream_id));
    });
}

int32_t nerve_b200_scheduler_close_after_current(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr, "scheduler and stream_id must not be NULL");
        fill_snapshot(out, scheduler->scheduler.close_stream_after_current(stream_id));
    });
}

int32_t nerve_b200_scheduler_schedule_step(nerve_b200_scheduler *scheduler, const nerve_b200_scheduler_budget *budget,
                                           size_t *out_activation_count, int32_t *out_flags) {
    return guarded([&] {
        require(scheduler != nullptr && budget != nullptr, "scheduler and budget must not be NULL");
        nerve::runtime::SchedulerBudget limits(budget->max_activations, budget->max_prefill_tokens_per_activation, budget->max_work_units);
        limits.max_decode_tokens_per_activation = budget->max_decode_tokens_per_activation;
        scheduler->step = scheduler->scheduler.schedule_step(limits);
        if (out_activation_count) *out_activation_count = scheduler->step.activations.size();
        if (out_flags)
            *out_flags = (scheduler->step.exhausted_activation_budget ? 1 : 0) | (scheduler->step.exhausted_work_budget ? 2 : 0) |
                         (scheduler->step.idle ? 4 : 0);
    });
}

int32_t nerve_b200_scheduler_step_activation(nerve_b200_scheduler *scheduler, size_t index, nerve_b200_activation *out,
                                             uint32_t *out_token_ids, size_t max_token_ids) {
    return guarded([&] {
        require(scheduler != nullptr && out != nullptr, "scheduler and out must not be NULL");
        require(index < scheduler->step.activations.size(), "activation index is outside the last step");
        const nerve::runtime::Activation &activation = scheduler->step.activations[index];
        out->id = activation.id;
        out->kind = static_cast<int32_t>(activation.kind);
        out->token_offset = activation.token_offset;
        out->token_count = activation.token_ids.size();
        out->remaining_prompt_token_count = activation.remaining_prompt_token_count;
        out->feedback_depth = activation.feedback_depth;
        out->max_tokens = activation.max_tokens;
        out->max_state_activation_count = activation.max_state_activation_count;
        out->reservation_count = activation.state_reservations.size();
        copy_text(out->stream_id, activation.stream_id);
        copy_text(out->execution_class_id, activation.execution_class_id);
        copy_text(out->input_event_id, activation.input_event_id);
        if (out_token_ids != nullptr) {
            require(max_token_ids >= activation.token_ids.size(), "out_token_ids is too small for the chunk");
            std::memcpy(out_token_ids, activation.token_ids.data(), activation.token_ids.size() * sizeof(uint32_t));
        }
    });
}

int32_t nerve_b200_scheduler_step_reservation(nerve_b200_scheduler *scheduler, size_t activation_index, size_t reservation_index,
                                              char *out_node_instance_id, char *out_state_id, nerve_b200_state_slot *out_slots,
                                              size_t max_slots, size_t *out_slot_count) {
    return guarded([&] {
        require(scheduler != nullptr, "scheduler must not be NULL");
        require(activation_index < scheduler->step.activations.size(), "activation index is outside the last step");
        const nerve::runtime::Activation &activation = scheduler->step.activations[activation_index];
        require(reservation_index < activation.state_reservations.size(), "reservation index is outside the activation");
        const nerve::runtime::StateReservation &reservation = activation.state_reservations[reservation_index];
        char text[64];
        if (out_node_instance_id) {
            copy_text(text, reservation.key.node_instance_id);
            std::memcpy(out_node_instance_id, text, 64);
        }
        if (out_state_id) {
            copy_text(text, reservation.key.state_id);
            std::memcpy(out_state_id, text, 64);
        }
        if (out_slot_count) *out_slot_count = reservation.slots.size();
        if (out_slots != nullptr) {
            require(max_slots >= reservation.slots.size(), "out_slots is too small for the reservation");
            for (size_t i = 0; i < reservation.slots.size(); i++) {
                const nerve::runtime::StateSlot &slot = reservation.slots[i];
                out_slots[i].logical_activation_index = slot.logical_activation_index;
                out_slots[i].block_id = slot.block_id;
                out_slots[i].block_activation_offset = slot.block_activation_offset;
                out_slots[i].block_activation_capacity = slot.block_activation_capacity;
                out_slots[i].allocated_block = slot.allocated_block ? 1 : 0;
                out_slots[i].copy_from_block_id = slot.copy_from_block_id ? static_cast<int64_t>(*slot.copy_from_block_id) : -1;
            }
        }
    });
}

int32_t nerve_b200_scheduler_complete(nerve_b200_scheduler *scheduler, uint64_t activation_id, const uint32_t *generated_token_ids,
                                      size_t generated_count, int32_t continue_generation, int64_t processed_state_activation_count,
                                      nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr, "scheduler must not be NULL");
        require(generated_count == 0 || generated_token_ids != nullptr, "generated_token_ids must not be NULL");
        nerve::runtime::ActivationOutcome outcome;
        outcome.generated_token_ids.assign(generated_token_ids, generated_token_ids + generated_count);
        outcome.continue_generation = continue_generation != 0;
        if (processed_state_activation_count >= 0) outcome.processed_state_activation_count = static_cast<size_t>(processed_state_activation_count);
        fill_snapshot(out, scheduler->scheduler.complete_activation(activation_id, outcome));
    });
}

int32_t nerve_b200_scheduler_snapshot(nerve_b200_scheduler *scheduler, nerve_b200_scheduler_counts *out) {
    return guarded([&] {
        require(scheduler != nullptr && out != nullptr, "scheduler and out must not be NULL");
        const nerve::runtime::SchedulerSnapshot snapshot = scheduler->scheduler.snapshot();
        out->stream_count = snapshot.stream_count;
        out->active_stream_count = snapshot.active_stream_count;
        out->in_flight_activation_count = snapshot.in_flight_activation_count;
        out->allocated_block_count = snapshot.transient_state_arena.allocated_block_count;
        out->free_block_count = snapshot.transient_state_arena.free_block_count;
        out->live_block_count = snapshot.transient_state_arena.live_block_count;
    });
}

int32_t nerve_b200_scheduler_set_prefix_state_cache_capacity(nerve_b200_scheduler *scheduler, uint64_t capacity_entries, uint64_t *out_evicted) {
    return guarded([&] {
        require(scheduler != nullptr, "scheduler must not be NULL");
        const size_t evicted = scheduler->scheduler.set_prefix_state_cache_capacity(static_cast<size_t>(capacity_entries)).size();
        if (out_evicted != nullptr) *out_evicted = evicted;
    });
}

int32_t nerve_b200_scheduler_cache_stream_prefix_state_for_tokens(nerve_b200_scheduler *scheduler, const char *stream_id, const char *runtime_graph_id,
                                                                  const uint32_t *token_ids, size_t token_count,
                                                                  const uint8_t *runtime_modifier_bytes, size_t runtime_modifier_count,
                                                                  int32_t *out_flags, uint64_t *out_evicted) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr && runtime_graph_id != nullptr, "scheduler and ids must not be NULL");
        require((token_count == 0 || token_ids != nullptr) && (runtime_modifier_count == 0 || runtime_modifier_bytes != nullptr), "NULL array with a non-zero count");
        std::vector<nerve::runtime::StateKey> keys;
        for (const nerve::runtime::EntrySnapshot &entry : scheduler->scheduler.stream_transient_state_snapshot(stream_id).entries) keys.push_back(entry.key);
        const std::string execution_class = [&] {
            for (const nerve::runtime::StreamSnapshot &stream : scheduler->scheduler.snapshot().streams)
                if (stream.stream_id == stream_id) return stream.execution_class_id;
            throw std::runtime_error(std::string("unknown stream \"") + stream_id + "\"");
        }();
        const nerve::runtime::PrefixStateCacheKey key = nerve::runtime::PrefixStateCacheKey::from_token_prefix(
            execution_class, runtime_graph_id, std::vector<uint32_t>(token_ids, token_ids + token_count),
            std::string(reinterpret_cast<const char *>(runtime_modifier_bytes), runtime_modifier_count), std::move(keys));
        const nerve::runtime::PrefixStateCacheInsert inserted = scheduler->scheduler.cache_stream_prefix_state(stream_id, key);
        if (out_flags != nullptr) *out_flags = inserted.replaced_existing ? 1 : 0;
        if (out_evicted != nullptr) *out_evicted = inserted.evicted_keys.size();
    });
}

int32_t nerve_b200_scheduler_restore_longest_stream_prefix_state(nerve_b200_scheduler *scheduler, const char *target_stream_id,
                                                                 const char *runtime_graph_id, const uint32_t *token_ids, size_t token_count,
                                                                 const uint8_t *runtime_modifier_bytes, size_t runtime_modifier_count,
                                                                 uint64_t *out_restored_token_count) {
    return guarded([&] {
        require(scheduler != nullptr && target_stream_id != nullptr && runtime_graph_id != nullptr && out_restored_token_count != nullptr,
                "scheduler, ids and out must not be NULL");
        require((token_count == 0 || token_ids != nullptr) && (runtime_modifier_count == 0 || runtime_modifier_bytes != nullptr), "NULL array with a non-zero count");
        std::vector<nerve::runtime::StateKey> keys;
        for (const nerve::runtime::EntrySnapshot &entry : scheduler->scheduler.stream_transient_state_snapshot(target_stream_id).entries) keys.push_back(entry.key);
        const std::optional<nerve::runtime::PrefixStateCacheKey> key = scheduler->scheduler.restore_longest_stream_prefix_state(
            target_stream_id, runtime_graph_id, std::vector<uint32_t>(token_ids, token_ids + token_count),
            std::string(reinterpret_cast<const char *>(runtime_modifier_bytes), runtime_modifier_count), std::move(keys));
        *out_restored_token_count = key ? key->token_count : 0;
    });
}

int32_t nerve_b200_scheduler_prefix_state_cache_counts(nerve_b200_scheduler *scheduler, uint64_t out_counts[3]) {
    return guarded([&] {
        require(scheduler != nullptr && out_counts != nullptr, "scheduler and out must not be NULL");
        const nerve::runtime::PrefixStateCacheSnapshot snapshot = scheduler->scheduler.prefix_state_cache_snapshot();
        out_counts[0] = snapshot.capacity_entries;
        out_counts[1] = snapshot.entry_count;
        out_counts[2] = snapshot.eviction_count;
    });
}

int32_t nerve_b200_scheduler_stream_snapshot(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out) {
    return guarded([&] {
        require(scheduler != nullptr && stream_id != nullptr && out != nullptr, "scheduler, stream_id and out must not be NULL");
        const nerve::runtime::SchedulerSnapshot snapshot = scheduler->scheduler.snapshot();
        for (const nerve::runtime::StreamSnapshot &stream : snapshot.streams)
            if (stream.stream_id == stream_id) {
                fill_snapshot(out, stream);
                return;
            }
        throw std::runtime_error(std::string("unknown stream \"") + stream_id + "\"");
    });
}

}  // extern "C"
#pragma GCC visibility pop
