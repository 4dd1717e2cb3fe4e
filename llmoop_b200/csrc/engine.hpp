// CUDA backend for the MTP speculative decode step of a compiled NERVE package:
// device-resident package (weights, paged KV pools, RoPE tables), the executor
// that runs a component's kernel list over a batch of lanes, and the engine that
// owns streams and drives prefill / draft / verify / accept / catch-up.
//
// Reference behaviour this replaces (paths inside the reference project):
//   mount      runtime-rs/src/vulkan_stream_circuit/placed_model_package_loader.rs:79-404,431-833
//   engine     runtime-rs/src/vulkan_stream_circuit/placed_prompt_engine.rs:48-589
//   stream     runtime-rs/src/vulkan_stream_circuit/placed_prompt_stream.rs:144-193,353-645
//   events     runtime-rs/src/vulkan_stream_circuit/placed_prompt_event.rs:167-298
//   cycle      runtime-rs/src/vulkan_stream_circuit/placed_stream_processor/feedback_generation.rs:66-194
//   draft      runtime-rs/src/vulkan_stream_circuit/resident_package_slices/speculative_decoder_processor.rs:206-488
//   prefill    runtime-rs/src/vulkan_stream_circuit/placed_stream_processor/temporal_prompt.rs:298-478
//   verify     runtime-rs/src/vulkan_stream_circuit/placed_stream_processor/temporal_prompt.rs:480-657
//   acceptance runtime-rs/src/vulkan_stream_circuit/speculative_decode.rs:54-105
// Handles are thread-compatible, not thread-safe (the reference engine is
// single-threaded); callbacks run on the calling thread.
#pragma once

#include <cuda_runtime.h>

#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "kernels.cuh"
#include "package.hpp"
#include "stream_runtime.hpp"

namespace nerve {

struct MountOptions {
    int device = 0;
    int capacity_tokens = 1024;  // per-stream context ring (rounded up to whole pages)
    int page_tokens = 16;
    int max_streams = 8;
    int max_lanes = 64;          // largest batch of lanes in one launch (prefill chunk / verify batch)
    int verify_level = 1;        // 0 none, 1 JSON artifacts + tensor hashes, 2 every listed file
    int tp_rank = 0, tp_size = 1;
    int extra_pages = 0;         // physical pages beyond max_streams * pages_per_stream (fork / COW headroom)
};

struct DeviceBuffer {
    void *ptr = nullptr;
    size_t bytes = 0;
};

// Tile-major INT4 copies and per-layer descriptors of a layer stack the persistent decode kernel can run
// (kernels_stack.cu); `available` is false when the stack does not have the dense INT4 Llama layer shape.
struct StackPlan {
    bool available = false;
    std::string reason;                 // why not, for diagnostics
    StackShape shape{};
    std::vector<StackLayer> layers;     // host copy of the device array
    DeviceBuffer device_layers;
    std::vector<DeviceBuffer> storage;  // tile-major weights and scales
    uint64_t weight_bytes = 0;          // bytes one pass over the stack streams
};

struct ExecCounters {
    uint64_t kernel_launches = 0;
    uint64_t graph_launches = 0;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;
    uint64_t host_syncs = 0;
};

class MountedModel {
public:
    static std::shared_ptr<MountedModel> mount(const std::string &path, const MountOptions &options);
    ~MountedModel();

    const ModelPlan &plan() const { return plan_; }  // the package's plan, cut down to this process's tensor-parallel shard
    const HostPackage &package() const { return *package_; }
    const MountOptions &options() const { return options_; }
    const void *tensor(const std::string &name) const;
    uint64_t weight_bytes() const { return weight_bytes_; }

    int pages_per_stream() const { return pages_per_stream_; }
    int physical_pages() const { return physical_pages_; }
    uint32_t capacity() const { return static_cast<uint32_t>(pages_per_stream_) * options_.page_tokens; }
    int kv_layer_count() const { return static_cast<int>(kv_pools_.size()); }
    KvLayer kv_layer(int index) const;
    size_t page_bytes(int index) const { return kv_page_bytes_[index]; }
    int32_t *block_table_device() const { return static_cast<int32_t *>(block_table_.ptr); }
    const uint32_t *rope_table(float theta, int rotary) const;
    uint32_t rope_positions() const { return rope_positions_; }

    // algorithmic bytes one verify step reads: every mounted weight byte of the target once
    // (packed weights + scales + norms) + lm_head, excluding the embedding table and the draft head.
    uint64_t target_step_weight_bytes() const { return target_step_bytes_; }
    uint64_t draft_step_weight_bytes() const { return draft_step_bytes_; }
    uint64_t kv_bytes_per_token() const { return kv_bytes_per_token_; }
    const StackPlan &target_stack() const { return target_stack_; }
    const StackPlan &draft_stack() const { return draft_stack_; }
    // The output projection tables in the streaming kernel's order (by tensor name), or nullptr.
    const void *projection_table(const std::string &name) const {
        auto found = projection_tables_.find(name);
        return found == projection_tables_.end() ? nullptr : found->second.ptr;
    }
    int sm_count() const { return sm_count_; }

private:
    MountedModel() = default;
    void upload_tensors();
    void build_rope_tables();
    void build_stack(const std::vector<ComponentPlan> &layers, int first_kv_index, StackPlan &out);

    std::shared_ptr<HostPackage> package_;
    ModelPlan plan_;
    MountOptions options_;
    std::map<std::string, DeviceBuffer> tensors_;
    uint64_t weight_bytes_ = 0, target_step_bytes_ = 0, draft_step_bytes_ = 0, kv_bytes_per_token_ = 0;
    std::vector<DeviceBuffer> kv_pools_;
    std::vector<size_t> kv_page_bytes_;
    std::vector<std::pair<int, int>> kv_shapes_;  // (kv_heads, head_width) per kv layer
    DeviceBuffer block_table_;
    int pages_per_stream_ = 0, physical_pages_ = 0;
    std::map<std::pair<uint32_t, int>, DeviceBuffer> rope_tables_;  // (theta bits, rotary) -> table
    uint32_t rope_positions_ = 0;
    int sm_count_ = 0;  // CTAs of the persistent kernels (one per SM of the mount device)
    StackPlan target_stack_, draft_stack_;
    std::map<std::string, DeviceBuffer> projection_tables_;
};

struct SamplerConfig {
    int method = 0;  // 0 greedy
    float temperature = 1.0f, top_p = 1.0f, min_p = 0.0f;
    int top_k = 1;
};

struct InputEvent {
    std::string id;
    std::vector<uint32_t> token_ids;
    size_t max_public_tokens = 0;
    std::vector<uint32_t> stop_token_ids;
};

struct OutputEvent {
    int64_t stream_id;
    uint32_t token_id;
    uint64_t source_stream_tick;
    size_t output_index;
};

struct SpeculativeStats {  // speculative_decode.rs:21-52
    uint64_t cycle_count = 0, proposed_draft_token_count = 0, accepted_draft_token_count = 0, emitted_token_count = 0;
    uint64_t draft_time_ns = 0, target_verification_time_ns = 0, draft_catch_up_time_ns = 0;
};

struct RunReport {
    uint64_t prefill_ns = 0, decode_ns = 0;
    uint64_t prefill_tokens = 0, generated_tokens = 0;
    uint64_t activation_count = 0, batch_count = 0, max_batch_width = 0;
    SpeculativeStats speculative;
    ExecCounters counters;
    double verify_ms_sum = 0.0;  // device time of verify steps (CUDA events)
    uint64_t verify_steps = 0;
    uint64_t verify_bytes = 0;   // algorithmic bytes of all verify steps
    double device_ms = 0.0;      // CUDA-event time from the first to the last launch of this run
    double int4_ms = 0.0;        // with profiling on: summed device time of the INT4 linear launches
    uint64_t int4_bytes = 0, int4_launches = 0;
    bool idle = true;            // false when the run stopped at max_batches with work left
};

struct CycleRecord {  // one speculative cycle of one stream, for parity tests
    int64_t stream_id;
    uint64_t start_tick;
    std::vector<uint32_t> draft_token_ids, target_token_ids, emitted_token_ids;
    uint32_t accepted = 0, committed = 0;
};

class Engine {
public:
    explicit Engine(std::shared_ptr<MountedModel> model);
    ~Engine();

    void add_stream(int64_t id, uint32_t seed, int speculative_draft_tokens, const SamplerConfig &sampler);
    void fork_stream(int64_t source, int64_t destination, uint32_t seed);
    void reset_stream(int64_t id);
    void remove_stream(int64_t id);
    void enqueue(int64_t id, const InputEvent &event);
    void interrupt_stream(int64_t id);
    // Teacher-forced harness mode: output index i of the stream's next event is forced to tokens[i] as the
    // draft proposal, so every draft is accepted when tokens are the target's own greedy continuation.
    void set_teacher_tokens(int64_t id, const std::vector<uint32_t> &tokens);
    RunReport run_until_idle(const std::function<void(const OutputEvent &)> &on_output);
    // Bounded form (run_until_idle_bounded, placed_prompt_engine.rs:420-589): stops after `max_batches` decode
    // batches (speculative cycles or single-tick batches); 0 = unbounded.
    RunReport run(uint64_t max_batches, const std::function<void(const OutputEvent &)> &on_output);
    void set_profiling(bool enabled) { profile_ = enabled; }
    // Tensor parallelism: every rank of the group runs the same streams in lock step on its shard of the weights and
    // meets the others in one NCCL all-reduce of f32 partial sums after each o and down projection.  `library` is the
    // path of libnccl.so.2 (loaded at run time, the engine does not link it); `unique_id` the 128 bytes rank 0 got
    // from tensor_parallel_unique_id and passed to the other ranks.
    static void tensor_parallel_unique_id(const std::string &library, uint8_t *out_128_bytes);
    void init_tensor_parallel(const std::string &library, int rank, int size, const uint8_t *unique_id_128_bytes);
    // Exchange inside the persistent decode kernel (no NCCL on that path): every rank allocates an exchange buffer
    // and hands out its 64-byte inter-process memory handle (tp_exchange_handle); once it has everybody's handles
    // (rank order, its own included) tp_connect maps the peers' buffers and the decode stack kernel then adds the
    // partial sums of the o and down projections up over peer memory.  Without it tensor-parallel batches run kernel
    // by kernel with NCCL all-reduces.
    void tp_exchange_handle(uint8_t *out_64_bytes);
    void tp_connect(const uint8_t *handles_64_bytes_each, int count);

    uint64_t stream_tick(int64_t id) const;
    void stop_stream_after_current(int64_t id);
    // placed_prompt_engine.rs:1238-1258, 1388-1400 (the fields that exist on one device)
    struct StreamSnapshot {
        uint64_t pending_input_event_count = 0, next_stream_tick = 0, completed_prompt_event_count = 0, context_window_activations = 0,
                 mapped_state_pages = 0;
        int speculative_draft_tokens = 0;
        bool idle = true;
    };
    struct EngineSnapshot {
        uint64_t stream_count = 0, active_stream_count = 0;
        bool idle = true;
    };
    StreamSnapshot stream_snapshot(int64_t id) const;
    EngineSnapshot snapshot() const;
    void scheduler_stream_counts(int64_t id, uint64_t out_counts[6]) const;
    // Prefix-state cache (stream_prefix_cache.rs:104-312, placed_prefix_state_cache.rs:50-365,
    // placed_prompt_engine.rs:190-280, 964-1060).  While a prompt is prefilled, the stream's state at the last
    // page boundary of the prompt is retained under the tokens that produced it; an input event for a fresh stream
    // that begins with a retained prefix starts from that state and prefills only the rest.  Retaining copies no KV:
    // the entry holds references to the stream's (full, never rewritten) pages, as a fork does, plus a copy of the
    // draft head's pending hidden state.  Off (capacity 0) unless set; setting a capacity drops what is retained.
    struct PrefixCacheStats {
        uint64_t hit_count = 0, miss_count = 0, insertion_count = 0, eviction_count = 0, reused_token_count = 0, saved_prefill_token_count = 0,
                 resident_entry_count = 0, resident_byte_count = 0;
    };
    void set_prefix_cache_capacity(size_t entries);
    PrefixCacheStats prefix_cache_stats() const;
    const std::vector<CycleRecord> &cycle_log() const { return cycle_log_; }
    // Test hook: the next `launches` launches of the persistent decode kernel wait (briefly) at their first grid barrier for
    // an arrival count the grid cannot reach, give up and report it - a failure made without faulting anything.
    void inject_barrier_timeouts(int launches) { inject_barrier_timeouts_ = launches; }
    void set_cycle_logging(bool enabled) {  // switching it on starts a new log
        log_cycles_ = enabled;
        if (enabled) cycle_log_.clear();
    }
    void set_use_graphs(bool enabled) { use_graphs_ = enabled; }
    // The persistent decode stack kernel serves batches of at most 8 lanes of dense INT4 stacks; off = the
    // kernel-per-operator path for everything.
    void set_decode_stack(bool enabled) { stack_enabled_ = enabled; }
    // Profiling aid: nanosecond stamps CTA 0 took at the phase boundaries of the target stack's last launch
    // ([layers][32]: layer start, then after each staging step, matrix or attention step and grid barrier, in
    // program order).  Empty when the stack kernel is not in use.
    std::vector<unsigned long long> decode_stack_timing();
    void set_prefill_chunk(int tokens) { prefill_chunk_ = tokens; }

    // Test hook: run the target over `tokens` at consecutive ticks starting at the stream's next tick WITHOUT
    // advancing it (state slots are overwritten later, as after a rejected speculation); copies f32 logits out.
    void debug_target_logits(int64_t id, const std::vector<uint32_t> &tokens, float *logits_out, uint16_t *hidden_out);

    MountedModel &model() { return *model_; }

private:
    struct ActiveEvent {
        InputEvent input;
        size_t next_external = 0;
        bool has_feedback = false;
        uint32_t feedback_token = 0;
        bool feedback_closes = false;
        size_t remaining = 0;
        std::vector<uint32_t> generated;
    };
    struct Stream {
        int64_t id = 0;
        int slot = -1;
        uint32_t seed = 0;
        int k = 0;
        SamplerConfig sampler;
        uint64_t next_tick = 0;
        std::deque<InputEvent> queue;
        std::unique_ptr<ActiveEvent> active;
        std::vector<int32_t> pages;  // logical page -> physical page (-1 = unmapped)
        std::vector<uint32_t> teacher;
        std::vector<uint32_t> history;  // the token fed at every tick so far (kept while the prefix cache is on)
        bool block_table_dirty = true;
        uint64_t completed_events = 0;
        bool detached = false;  // the active event was stopped from outside: the scheduler no longer tracks it
    };

    Stream &stream(int64_t id);
    const Stream &stream(int64_t id) const;
    void activate_next_event(Stream &s);
    void register_stream(int64_t id, uint32_t seed, int speculative_draft_tokens, const SamplerConfig &sampler);
    void rejoin_scheduler(int64_t id);  // a fresh scheduler entry for the stream (its events were dropped)
    static std::string scheduler_id(int64_t id) { return std::to_string(id); }
    // Admission: which stream runs what next (events -> prefill chunks -> decode windows, running before waiting,
    // one activation per stream and step) is decided by the scheduler unit that restates stream_runtime.rs; the
    // engine executes the activations and reports their outcomes (placed_prompt_engine.rs:455-520).
    runtime::StreamScheduler scheduler_;
    std::vector<runtime::Activation> carried_activations_;  // scheduled, but their batch failed: executed first by the next run
    // prefix-state cache: the index decides what stays (least recently used goes first), the payload is the page list
    struct PrefixCheckpoint {
        std::vector<int32_t> pages;  // physical pages of ticks [0, token_count), one reference held on each
        int pending_slot = -1;       // frame of prefix_pending_ with the draft head's pending hidden state
    };
    runtime::PrefixCacheIndex<PrefixCheckpoint> prefix_index_{0};
    std::map<int64_t, runtime::PrefixStateCacheKey> latest_checkpoint_by_stream_;
    DeviceBuffer prefix_pending_;  // [capacity + 1][hidden]
    std::vector<int> free_pending_slots_;
    PrefixCacheStats prefix_stats_;
    bool prefix_cache_on() const { return prefix_index_.capacity_entries() > 0; }
    std::string prefix_modifier_bytes(const Stream &s) const;
    uint64_t prefix_checkpoint_tick(const Stream &s) const;  // where the active event's prompt gets its checkpoint (0 = nowhere)
    void capture_prefix_checkpoint(Stream &s);
    size_t restore_longest_prefix(Stream &s, const std::vector<uint32_t> &token_ids);  // tokens reused
    void release_checkpoint(PrefixCheckpoint &checkpoint);
    void ensure_pages(Stream &s, uint64_t last_tick);
    void release_pages(Stream &s);
    void sync_block_tables();
    void emit(Stream &s, uint32_t token, uint64_t tick, const std::function<void(const OutputEvent &)> &on_output,
              RunReport &report);

    // device work
    struct LaneBatch {
        int lanes = 0;
    };
    void upload(void *device_destination, const void *host_source, size_t bytes, const char *what);
    void synchronize(const char *what);
    void upload_lanes(const std::vector<uint32_t> &positions, const std::vector<int32_t> &slots);
    void upload_tokens(const uint32_t *tokens, int count);
    void run_component(const ComponentPlan &plan, int kv_index, int lanes,
                       const std::map<std::string, void *> &bound, void *output);
    // embedding -> layers -> final norm (-> logits -> argmax records)
    void target_forward(int lanes, bool want_logits);
    void draft_forward(int lanes, const uint16_t *hidden_in, bool want_logits);
    void run_prefill_chunk(Stream &s, const uint32_t *tokens, int count, bool sample_last, uint32_t *sampled);
    void run_single_ticks(std::vector<Stream *> &batch, const std::function<void(const OutputEvent &)> &on_output,
                          RunReport &report);
    void run_speculative_cycles(std::vector<Stream *> &batch, int draft_count,
                                const std::function<void(const OutputEvent &)> &on_output, RunReport &report);
    void check(cudaError_t status, const char *what);
    void *signal_buffer(const std::string &name);

    std::shared_ptr<MountedModel> model_;
    std::map<int64_t, Stream> streams_;
    std::vector<int> free_slots_;
    std::vector<int32_t> free_pages_;
    std::vector<int32_t> page_refcount_;
    std::vector<int32_t> block_table_host_;
    cudaStream_t cuda_stream_ = nullptr;
    cudaEvent_t event_a_ = nullptr, event_b_ = nullptr, event_begin_ = nullptr, event_end_ = nullptr, run_begin_ = nullptr, run_end_ = nullptr;

    // workspaces
    std::map<std::string, DeviceBuffer> signals_;
    DeviceBuffer frame_a_, frame_b_;        // residual stream ping-pong [max_lanes][hidden]
    DeviceBuffer embedding_out_;            // [max_lanes][hidden]
    DeviceBuffer normalized_;               // target final-norm output [max_lanes][hidden]
    DeviceBuffer draft_normalized_;         // draft final-norm output [max_lanes][hidden]
    DeviceBuffer draft_hidden_in_;          // [max_lanes][hidden]
    DeviceBuffer logits_;                   // f32 [max_lanes][vocab]
    DeviceBuffer records_;                  // u32 [max_lanes][4]
    DeviceBuffer argmax_scratch_;
    DeviceBuffer sampler_scratch_, sampler_table_;   // stochastic sampler: candidate lists, per-slot parameters
    int stochastic_streams_ = 0;                     // streams whose sampler is not greedy
    // arg-max for all-greedy engines, else the seeded sampler (greedy lanes take its first entry)
    void sample_lanes(const float *logits, uint32_t *records, int lanes, const int32_t *slots, const uint32_t *ticks, const char *what);
    DeviceBuffer lane_tokens_, lane_positions_, lane_slots_;
    DeviceBuffer pending_hidden_;           // [max_streams][hidden]
    DeviceBuffer pending_backup_;           // the same rows as they were before the batch in flight (restored when a kernel reports an error)
    DeviceBuffer attention_scratch_;
    DeviceBuffer kernel_error_;             // device word set by pipelined kernels whose bounded waits expired
    DeviceBuffer tp_partial_;               // f32 [max_lanes][hidden] partial sums of row-parallel linears
    void *nccl_library_ = nullptr, *nccl_comm_ = nullptr;
    DeviceBuffer tp_exchange_;              // this rank's exchange buffer + arrival counter + consumed-arrivals word
    DeviceBuffer tp_description_;           // StackTp in device memory
    std::vector<void *> tp_peer_mappings_;  // opened peer handles
    bool tp_connected_ = false;
    void tp_all_reduce(float *values, size_t count);
    // persistent decode stack workspaces ([8 lanes][width]) and its two barrier words
    DeviceBuffer stack_q_, stack_attention_out_, stack_activation_, stack_barrier_, stack_timing_;
    bool stack_enabled_ = true;
    bool run_stack(const StackPlan &stack, int lanes, void *hidden);
    void project_and_sample(const uint16_t *normalized, const std::string &projection_tensor, float scale, int lanes, const int32_t *slots,
                            const uint32_t *ticks, const char *what);
    void backup_pending();
    void check_kernel_status(const uint32_t *status_word);  // throws (after restoring the pending hidden states) when a kernel reported an error
    DeviceBuffer cycle_state_;              // device-side per-batch cycle arrays (see engine.cu)
    // Pinned staging arena for host->device uploads: every upload between two host synchronisations gets its
    // own region (an asynchronous copy reads the pinned source when it executes, not when it is enqueued).
    uint8_t *staging_ = nullptr;
    size_t staging_bytes_ = 0, staging_used_ = 0;
    uint32_t *host_records_ = nullptr;      // pinned readback area
    int split_tokens_ = 256, max_splits_ = 1;
    int prefill_chunk_ = 64;
    bool use_graphs_ = true, log_cycles_ = false;
    bool streaming_projection_ = true;      // output projections of at most 8 lanes run the streaming kernel on the mount-time table copy
    bool vocabulary_parallel_ = true;       // tensor-parallel greedy sampling splits the vocabulary over the ranks
    bool full_logits_ = false;              // debug_target_logits wants every rank to project the whole vocabulary
    bool failed_ = false;                   // a tensor-parallel rank whose kernel gave up is out of step with its peers for good
    int inject_barrier_timeouts_ = 0;       // test hook: this many decode stack launches wait for arrivals that cannot come
    std::vector<CycleRecord> cycle_log_;
    ExecCounters counters_;
    // per-launch CUDA events around the INT4 linears (profiling mode only)
    bool profile_ = false;
    std::vector<cudaEvent_t> profile_events_;
    size_t profile_used_ = 0;
    double profile_ms_ = 0.0;
    uint64_t profile_bytes_ = 0, profile_launches_ = 0;
    void profile_begin(uint64_t bytes);
    void profile_end();
    // lane table and token ids the forward passes read (device pointers; fixed per phase so that a phase can be
    // replayed as a CUDA graph while the host only rewrites the arrays' contents)
    LaneTable current_lanes_{nullptr, nullptr};
    const uint32_t *current_tokens_ = nullptr;
    int current_width_ = 1;                 // lanes per stream of the current batch (stream-major lane order)
    int current_splits_ = 1;                // attention split count (stride of the scratch partials) of this launch
    int op_split_tokens_ = 64;              // tokens per split on the kernel-per-operator path: fixed per engine, so that a lane's
                                            // arithmetic does not depend on the batch it runs in
    int current_op_splits_ = 1;             // split count of this launch on that path
    int max_q_heads_ = 1;
    struct GraphEntry {
        cudaGraphExec_t exec = nullptr;
        uint64_t kernel_nodes = 0;
        int warm = 0;
    };
    std::map<std::vector<int>, GraphEntry> graphs_;
    void run_phase(const std::vector<int> &key, const std::function<void()> &body);
    int plan_splits(int lanes, uint64_t newest_tick);  // sets the split length and count of the next launches, returns a graph-key word
};

}  // namespace nerve
