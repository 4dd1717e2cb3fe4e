/*
 * nerve_b200 - C ABI of the B200 (sm_100a) backend for the MTP speculative
 * decode path of compiled NERVE packages.
 *
 * The reference project has no FFI or plugin boundary for this path (its only
 * backend is in-process Vulkan); the entry points below are what a binding for
 * it would need.  Each one names the reference interface it stands in for, by
 * file:line inside the reference project.
 *
 * Conventions (mirroring the reference's `Result<_, *Error(String)>`): every
 * function returns 0 on success and a non-zero status otherwise, never aborts;
 * nerve_b200_last_error() returns the message of the calling thread's most
 * recent failure.  Handles are opaque, thread-compatible but not thread-safe
 * (the reference engine is single-threaded: runtime-rs/src/vulkan_stream_circuit/
 * placed_prompt_stream.rs:9); callbacks run on the calling thread.  All pointers
 * are plain host pointers unless a parameter says "device".
 */
#ifndef NERVE_B200_H
#define NERVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NERVE_B200_OK 0
#define NERVE_B200_ERROR 1

typedef struct nerve_b200_package nerve_b200_package;
typedef struct nerve_b200_engine nerve_b200_engine;

const char *nerve_b200_last_error(void);
/* ABI version of this header (bumped on incompatible changes). */
int32_t nerve_b200_abi_version(void);

/* ---- package mount ---------------------------------------------------------
 * Replaces VulkanResidentInProcessPlacedModelPackage::from_runtime_model_for_bound_devices
 * (runtime-rs/src/vulkan_stream_circuit/placed_model_package_loader.rs:54-77,79-404):
 * parses vulkan_resident_package.json (schema v3), checks artifact_integrity and
 * per-tensor SHA-256 (runtime-rs/src/tensor_storage.rs:66-136), uploads weights to
 * device buffers, allocates the paged KV pools and per-stream state.
 */
typedef struct nerve_b200_mount_options {
    int32_t device;           /* CUDA device ordinal */
    int32_t capacity_tokens;  /* per-stream context (the CLI's --context-size) */
    int32_t page_tokens;      /* KV page size in tokens (the reference uses min(capacity, 64)) */
    int32_t max_streams;
    int32_t max_lanes;        /* largest lane batch per launch: prefill chunk / streams * (k+1) */
    int32_t verify_level;     /* 0 none, 1 JSON artifacts + tensor hashes, 2 every listed artifact */
    int32_t tp_rank, tp_size; /* tensor-parallel shard of this process */
    int32_t extra_pages;      /* physical KV pages beyond max_streams * pages per stream */
} nerve_b200_mount_options;

int32_t nerve_b200_package_mount(const char *manifest_path_or_dir, const nerve_b200_mount_options *options,
                                 nerve_b200_package **out_package);
/* Packages are reference counted (Arc in the reference, placed_prompt_stream.rs:60-68); engines hold a reference. */
int32_t nerve_b200_package_unmount(nerve_b200_package *package);

typedef struct nerve_b200_package_info {
    int64_t hidden_size, vocab_size, layer_count, max_context;
    int32_t has_speculative_decoder;
    int32_t kv_layer_count;
    uint64_t weight_bytes;              /* device-resident weight bytes */
    uint64_t verify_step_weight_bytes;  /* target weight bytes one verify step streams (incl. lm_head) */
    uint64_t draft_step_weight_bytes;   /* draft head weight bytes one draft step streams (incl. lm_head) */
    uint64_t kv_bytes_per_token;        /* target KV bytes per context token */
    int32_t pages_per_stream, physical_pages, page_tokens;
    uint32_t eos_token_id;              /* first EOS id of config.json, 0xffffffff if none */
    int32_t target_decode_stack;        /* 1 when the target layers run as one persistent kernel for batches <= 8 lanes */
    int32_t draft_decode_stack;         /* same for the speculative decoder's layers */
    uint64_t target_stack_weight_bytes; /* bytes one pass of that kernel streams (tile-major INT4 + scales + norms) */
} nerve_b200_package_info;
int32_t nerve_b200_package_describe(const nerve_b200_package *package, nerve_b200_package_info *out_info);

/* Host-only manifest check (no GPU needed): parse + integrity verification + execution-plan build.
 * Counterpart of the mount-time validation in runtime-rs/src/package/mount.rs and
 * resident_package_execution_contract.rs. */
int32_t nerve_b200_package_validate(const char *manifest_path_or_dir, int32_t verify_level, int64_t *out_op_count,
                                    int64_t *out_tensor_count);

/* ---- engine ------------------------------------------------------------------
 * Replaces VulkanResidentInProcessPlacedPromptEngine
 * (runtime-rs/src/vulkan_stream_circuit/placed_prompt_engine.rs:48-589).
 */
int32_t nerve_b200_engine_create(nerve_b200_package *package, nerve_b200_engine **out_engine);
int32_t nerve_b200_engine_destroy(nerve_b200_engine *engine);

typedef struct nerve_b200_sampler_config {
    int32_t method; /* 0 = greedy, 1 = temperature_top_k_top_p (seeded; top_k 1..64, temperature > 0) */
    float temperature, top_p, min_p;
    int32_t top_k;
} nerve_b200_sampler_config;

/* add_stream (placed_prompt_engine.rs:48-78) with the stream constructor's arguments
 * (placed_prompt_stream.rs:48-72): seed, speculative_draft_tokens, sampler config (NULL = package default). */
int32_t nerve_b200_engine_add_stream(nerve_b200_engine *engine, int64_t stream_id, uint32_t seed,
                                     int32_t speculative_draft_tokens, const nerve_b200_sampler_config *sampler);
/* fork_stream (placed_prompt_engine.rs:80-140): the new stream shares the source's state pages copy-on-write. */
int32_t nerve_b200_engine_fork_stream(nerve_b200_engine *engine, int64_t source_stream_id, int64_t new_stream_id,
                                      uint32_t seed);
int32_t nerve_b200_engine_reset_stream(nerve_b200_engine *engine, int64_t stream_id);
int32_t nerve_b200_engine_remove_stream(nerve_b200_engine *engine, int64_t stream_id);
int32_t nerve_b200_engine_interrupt_stream(nerve_b200_engine *engine, int64_t stream_id);
/* stop_stream_after_current (placed_prompt_engine.rs:307-331): the active event emits no more tokens, its last token is
 * still fed back as the closing tick; queued events are dropped.  No effect on an idle stream. */
int32_t nerve_b200_engine_stop_after_current(nerve_b200_engine *engine, int64_t stream_id);
/* snapshot (placed_prompt_engine.rs:1238-1258, 1388-1400). */
typedef struct {
    uint64_t pending_input_event_count, next_stream_tick, completed_prompt_event_count, context_window_activations,
        mapped_state_pages;
    int32_t speculative_draft_tokens, idle;
} nerve_b200_engine_stream_snapshot;
typedef struct {
    uint64_t stream_count, active_stream_count;
    int32_t idle;
} nerve_b200_engine_snapshot_counts;
int32_t nerve_b200_engine_stream_snapshot_of(nerve_b200_engine *engine, int64_t stream_id, nerve_b200_engine_stream_snapshot *out);
int32_t nerve_b200_engine_snapshot(nerve_b200_engine *engine, nerve_b200_engine_snapshot_counts *out);
/* The runtime scheduler's view of one of the engine's streams (RuntimeStreamSnapshot, stream_runtime.rs:258-300; the
 * engine owns a scheduler as placed_prompt_engine.rs:455-520 does and runs what it schedules): out_counts[0] =
 * scheduled activations, [1] = completed input events, [2] = generated tokens, [3] = activations in flight,
 * [4] = queued input events, [5] = 1 while an input event is current.  Counts restart when the stream's events are
 * dropped (reset, interrupt, stop after current). */
int32_t nerve_b200_engine_scheduler_stream_counts(nerve_b200_engine *engine, int64_t stream_id, uint64_t out_counts[6]);

/* Prefix-state cache (stream_prefix_cache.rs:104-312; placed_prefix_state_cache.rs:50-365; the engine's use of both,
 * placed_prompt_engine.rs:190-280 and 964-1060).  With a capacity of N > 0 entries, a prompt's prefill stops once at
 * the prompt's last KV page boundary and retains the stream's state there under the tokens that produced it (one
 * checkpoint per stream, the latest; least recently used entries leave first); nerve_b200_engine_enqueue on a fresh
 * stream (tick 0, nothing queued) whose tokens - all but the last - begin with a retained prefix starts the stream at
 * that state and prefills only the rest.  The sampler settings and the draft count of the stream are part of the key.
 * Retaining copies no KV: the entry holds references to the stream's pages (copy-on-write, as after a fork) and one
 * hidden-state frame.  Capacity 0 (the default) switches the cache off; every call drops what was retained.  The
 * reference keeps the cache always on with streams + 1 entries; here it is the caller's choice because a prefill
 * cut at the boundary runs other batch shapes, so the low bits of the logits may differ from an uncut prefill.
 * out_stats (VulkanResidentPlacedPrefixStateCacheStats, placed_prefix_state_cache.rs:38-48): [0] hit_count,
 * [1] miss_count, [2] insertion_count, [3] eviction_count, [4] reused_token_count, [5] saved_prefill_token_count,
 * [6] resident_entry_count, [7] resident_byte_count (KV bytes the entries keep alive, shared pages counted per entry). */
int32_t nerve_b200_engine_set_prefix_cache_capacity(nerve_b200_engine *engine, uint64_t entries);
int32_t nerve_b200_engine_prefix_cache_stats(nerve_b200_engine *engine, uint64_t out_stats[8]);

/* enqueue_input_event (placed_prompt_engine.rs:256-331): VulkanResidentTokenInputEvent
 * {id, token_ids, max_public_tokens, stop_token_ids}. */
int32_t nerve_b200_engine_enqueue(nerve_b200_engine *engine, int64_t stream_id, const char *event_id,
                                  const uint32_t *token_ids, size_t token_count, size_t max_public_tokens,
                                  const uint32_t *stop_token_ids, size_t stop_token_count);

/* VulkanResidentTokenOutputEvent {token_id, source_stream_tick, output_index}. */
typedef void (*nerve_b200_output_callback)(void *user, int64_t stream_id, uint32_t token_id,
                                           uint64_t source_stream_tick, uint64_t output_index);

/* Field names follow RuntimePromptTimingReport / VulkanSpeculativeDecodeStats
 * (runtime-rs/src/bin/nerve_runtime/placed_chat.rs:98-121, speculative_decode.rs:21-52). */
typedef struct nerve_b200_run_report {
    uint64_t prefill_ns, decode_ns;
    uint64_t prefill_tokens, generated_tokens;
    uint64_t activation_count, batch_count, max_batch_width;
    uint64_t cycle_count, proposed_draft_token_count, accepted_draft_token_count, emitted_token_count;
    uint64_t draft_time_ns, target_verification_time_ns, draft_catch_up_time_ns;
    uint64_t kernel_launches, graph_launches, h2d_bytes, d2h_bytes, host_syncs;
    double verify_ms_sum;    /* device time of all verify steps (CUDA events) */
    uint64_t verify_steps;
    uint64_t verify_bytes;   /* algorithmic bytes of all verify steps (weights once + attended KV) */
    double device_ms;        /* CUDA-event time from the first to the last launch of the run */
    double int4_ms;          /* profiling mode: summed device time of the INT4 linear launches */
    uint64_t int4_bytes, int4_launches;
    int32_t idle;            /* 0 when a bounded run stopped with work left */
} nerve_b200_run_report;

/* run_until_idle_bounded_with_output (placed_prompt_engine.rs:420-589). */
int32_t nerve_b200_engine_run_until_idle(nerve_b200_engine *engine, nerve_b200_output_callback on_output, void *user,
                                         nerve_b200_run_report *out_report);

/* Bounded form: stops after max_batches decode batches (speculative cycles / single-tick batches); 0 = unbounded. */
int32_t nerve_b200_engine_run(nerve_b200_engine *engine, uint64_t max_batches, nerve_b200_output_callback on_output,
                              void *user, nerve_b200_run_report *out_report);

int32_t nerve_b200_engine_stream_tick(const nerve_b200_engine *engine, int64_t stream_id, uint64_t *out_tick);

/* ---- harness / test hooks (no reference counterpart) ---------------------------- */
/* Teacher-forced full-acceptance mode: draft proposal for output index i is forced to tokens[i]. */
int32_t nerve_b200_engine_set_teacher_tokens(nerve_b200_engine *engine, int64_t stream_id, const uint32_t *tokens,
                                             size_t count);
int32_t nerve_b200_engine_set_prefill_chunk(nerve_b200_engine *engine, int32_t tokens);
/* Keeps one record per speculative cycle (nerve_b200_engine_cycle_log); switching it on starts a new log. */
int32_t nerve_b200_engine_set_cycle_logging(nerve_b200_engine *engine, int32_t enabled);
/* Failure injection without a fault: the next `launches` launches of the persistent decode kernel wait at their first
 * grid barrier for arrivals that cannot come; the bounded wait gives up after a few milliseconds, the kernel reports
 * it and the run call fails with the streams as they were before the batch (nothing emitted, ticks unchanged; the
 * reference restores a failed cycle the same way, placed_stream_processor/feedback_generation.rs:188-192).  The
 * engine stays usable. */
int32_t nerve_b200_engine_inject_barrier_timeouts(nerve_b200_engine *engine, int32_t launches);
/* Records CUDA events around every INT4 linear launch (adds launch overhead; for roofline measurement only). */
int32_t nerve_b200_engine_set_profiling(nerve_b200_engine *engine, int32_t enabled);
/* Tensor parallelism (the reference's sharding plan: vulkan_distributed/planning.rs:180-528).  A package mounted
 * with tp_size > 1 holds rank tp_rank's shard of every dense layer: q/k/v and gate/up by output rows (whole
 * heads), o and down by input columns (whole groups of 128); norms, embedding and output projection are
 * replicated.  Every rank runs the same streams with the same calls; after each o and down projection the ranks'
 * f32 partial sums meet in one NCCL all-reduce, then the bf16 rounding and the residual add follow.
 * nerve_b200_tp_unique_id: rank 0 obtains the 128-byte NCCL id and hands it to the other ranks (any transport);
 * nerve_b200_engine_init_tp: every rank joins the group before its first run.  nccl_library_path: libnccl.so.2,
 * loaded at run time (the library does not link NCCL). */
int32_t nerve_b200_tp_unique_id(const char *nccl_library_path, uint8_t *out_128_bytes);
/* The shard rule of the mount (pure host function): rank's [begin, begin + count) of `total` rows or columns kept
 * in whole units (head width for q/k/v rows, 16 for gate/up rows, 128 for o/down columns); an error when total is
 * not a multiple of unit x size. */
int32_t nerve_b200_tp_shard_range(int64_t total, int64_t unit, int32_t rank, int32_t size, int64_t *out_begin, int64_t *out_count);
int32_t nerve_b200_engine_init_tp(nerve_b200_engine *engine, const char *nccl_library_path, int32_t rank, int32_t size,
                                  const uint8_t *unique_id_128_bytes);
/* Exchange inside the persistent decode kernel (no reference counterpart; the reference shards through shared host
 * memory, vulkan_distributed/planning.rs:180-528).  Every rank calls ..._tp_exchange_handle (allocates its exchange
 * buffer, returns the 64-byte inter-process memory handle), the handles travel to every rank by any transport, and
 * ..._tp_connect(handles of ranks 0..size-1, in rank order, own included) maps the peers' buffers over NVLink.  From
 * then on batches of at most 8 lanes run the persistent kernel on every rank: the o and down projections leave their
 * f32 partial sums in the rank's own buffer, all CTAs of all ranks meet at a two-level barrier (local arrivals, one system-scope
 * store per peer) with bounded waits, and each rank reads everybody's partials with plain peer loads and adds them up in rank order.  Larger batches keep
 * the NCCL path of nerve_b200_engine_init_tp, which is still required.  The ranks must issue the same calls in the
 * same order; a rank that stays away ends the others' launches with the barrier-timeout error, after which the
 * engines of the group have to be created anew. */
int32_t nerve_b200_engine_tp_exchange_handle(nerve_b200_engine *engine, uint8_t *out_64_bytes);
int32_t nerve_b200_engine_tp_connect(nerve_b200_engine *engine, const uint8_t *handles_64_bytes_each, int32_t count);
/* Batches of at most 8 lanes of a dense INT4 g128 layer stack (the verify batch, draft and single-tick steps) run
 * as one persistent kernel per stack; 0 selects the kernel-per-operator path for them as well.  Default on; the
 * library reads no environment switch for it.  No counterpart in the reference: its Vulkan
 * runtime always records one dispatch per kernel (placed_stream_processor/temporal_prompt.rs:480-657). */
int32_t nerve_b200_engine_set_decode_stack(nerve_b200_engine *engine, int32_t enabled);
/* Profiling aid (no reference counterpart): with profiling on, CTA 0 of the persistent kernel stamps the GPU's
 * nanosecond timer at each layer's start and after each staging step, matrix or attention step and grid barrier
 * of the layer, in program order; this copies the stamps of the last target-stack launch, [layers][32].
 * Row 0 also carries the kernel's entry (index 16) and the end of its last layer (index 30).
 * *out_count = stamps available. */
int32_t nerve_b200_engine_decode_stack_timing(nerve_b200_engine *engine, uint64_t *out_stamps, size_t max_stamps, size_t *out_count);
/* Cycle log rows: {stream_id, start_tick, accepted, committed, emitted_count, width, emitted[8], targets[8]} as u64. */
int32_t nerve_b200_engine_cycle_log(const nerve_b200_engine *engine, uint64_t *out_rows, size_t max_rows,
                                    size_t *out_count);
/* Target forward over `count` tokens at the stream's next ticks without advancing it; f32 logits [count][vocab]
 * and bf16 final-norm hidden [count][hidden] (either may be NULL). */
int32_t nerve_b200_debug_target_logits(nerve_b200_engine *engine, int64_t stream_id, const uint32_t *tokens,
                                       size_t count, float *out_logits, uint16_t *out_hidden);

/* ---- operator-level entry points (device pointers; bf16 activations [lanes][width]) -----------
 * One per shader family on the path; `stream` is a cudaStream_t passed as void* (NULL = default stream).
 */
/* linear_int4_ct.comp.template:80-150 (+ residual add of add_bf16.comp.template when residual != NULL). */
int32_t nerve_b200_op_linear_int4(const void *x_device, const void *qweight_device, const void *scales_device,
                                  void *y_device, const void *residual_device, int32_t lanes, int32_t n, int32_t k,
                                  int32_t group, void *stream);
/* gate/up pair + silu_multiply_bf16.comp.template:30-52 in one launch: y = bf16(silu_bf16(bf16(x.Wg)) * bf16(x.Wu)). */
int32_t nerve_b200_op_linear_int4_silu_pair(const void *x_device, const void *gate_qweight_device,
                                            const void *gate_scales_device, const void *up_qweight_device,
                                            const void *up_scales_device, void *y_device, int32_t lanes, int32_t n,
                                            int32_t k, void *stream);
/* linear_bf16.comp.template:38-95; to_f32 != 0 gives tied_output_projection_bf16.comp.template:33-91 (f32 * scale). */
int32_t nerve_b200_op_linear_bf16(const void *x_device, const void *w_device, void *y_device,
                                  const void *residual_device, int32_t lanes, int32_t n, int32_t k, int32_t to_f32,
                                  float scale, void *stream);
/* rms_norm_bf16.comp.template:49-72 */
int32_t nerve_b200_op_rms_norm(const void *x_device, const void *weight_device, void *y_device, int32_t lanes,
                               int32_t width, float eps, float weight_offset, void *stream);
/* quantize_fp8_e4m3.comp.template:41-60 + linear_prequant_fp8_e4m3.comp.template:69-120 */
int32_t nerve_b200_op_linear_fp8(const void *x_device, const void *w_device, const void *wscale_device,
                                 void *y_device, const void *residual_device, void *xq_scratch_device,
                                 void *xscale_scratch_device, int32_t lanes, int32_t n, int32_t k, void *stream);
/* greedy_sampler_f32.comp.template:52-109: records u32[lanes][4] = {token, logit bits, 0, 0}.  Two-stage
 * reduction: scratch_device must hold nerve_b200_op_greedy_scratch_bytes(lanes) bytes. */
int32_t nerve_b200_op_greedy(const void *logits_device, void *records_device, void *scratch_device, int32_t lanes,
                             int32_t vocab, void *stream);
uint64_t nerve_b200_op_greedy_scratch_bytes(int32_t lanes);
/* Seeded temperature / top-k / top-p / min-p sampler (sampler.rs:748-873;
 * temperature_top_k_candidates_f32.comp.template:48-127 + temperature_top_k_top_p_sampler_f32.comp.template:56-216):
 * exact top-k (ties -> lower id, NaNs skipped), weights exp(l/T - max/T), min-p cut, top-p nucleus, uniform
 * u = (hash_u32(seed ^ tick) >> 8) * 2^-24 with the shader's hash, first index whose cumulative weight exceeds
 * u * nucleus weight.  records u32[lanes][4] = {token, logit bits, 1, 0}; lane l draws for stream tick
 * ticks_device[l] (0 when NULL).  scratch_device: nerve_b200_op_sample_scratch_bytes(lanes) bytes;
 * params_device: 32 bytes the call fills with the parameters.  top_k <= 64. */
int32_t nerve_b200_op_sample_top_k_top_p(const void *logits_device, void *records_device, void *scratch_device, int32_t lanes,
                                         int32_t vocab, int32_t top_k, float temperature, float top_p, float min_p, uint32_t seed,
                                         const uint32_t *ticks_device, void *params_device, void *stream);
uint64_t nerve_b200_op_sample_scratch_bytes(int32_t lanes);
/* The same arg-max for callers that must not allocate device memory and have none to lend: the partial winners
 * of the two-stage reduction live in a 32 KB device array built into the library, so neither this call nor the
 * caller ever allocates or frees anything.  No counterpart in the reference (its sampler dispatch always binds a
 * buffer the runtime allocated at mount).
 * Who needs it: a sampler thread inside a serving process whose device memory was carved up once at start-up
 * (a later cudaMalloc may fail under fragmentation, and it synchronises the whole device, stalling every other
 * stream's decode step).
 * Limits and rules:
 *  - at most 64 lanes per call; more is rejected with an error naming the limit (use nerve_b200_op_greedy);
 *  - the first call on each device looks up the array's device address (with that device current) and caches
 *    it: make that first call during set-up, before any stream capture is begun;
 *  - the array is shared by every caller in the process and keeps the last call's partials.  A call overwrites
 *    every slot it later reads, so nothing has to be cleared, but two calls that overlap in time on one device
 *    (two streams, two threads) race: issue them on one stream or order them yourself. */
int32_t nerve_b200_op_greedy_static(const void *logits_device, void *records_device, int32_t lanes, int32_t vocab,
                                    void *stream);
/* Kernel-ABI byte layouts of the reference (pure host functions): the 20-byte stream-control record
 * (stream_control_bytes.rs:8-18) and the transient-state header + page table
 * (transient_state_buffer_layout.rs:24-154; out_layout = {block capacity, page count, page bytes, page-table
 * bytes, static offset, dynamic offset, byte capacity}; logical_to_physical NULL = identity). */
int32_t nerve_b200_stream_control_bytes(uint32_t token_id, uint64_t stream_tick, uint32_t control_flags,
                                        uint32_t capacity, uint8_t *out_20_bytes);
int32_t nerve_b200_state_page_table_bytes(int64_t static_bytes, int64_t bytes_per_activation,
                                          int64_t max_dynamic_activations, int64_t capacity_activations,
                                          const uint32_t *logical_to_physical, size_t mapping_count,
                                          uint8_t *out_bytes, size_t out_capacity, int64_t *out_layout);
/* speculative_decode.rs:54-105 on host arrays (pure function, no GPU): out = {accepted, committed}. */
int32_t nerve_b200_verify_prefix(const uint32_t *draft, size_t draft_count, const uint32_t *target,
                                 size_t target_count, const uint32_t *stop, size_t stop_count, uint32_t *out_counts,
                                 uint32_t *out_emitted, size_t *out_emitted_count);


/* ---- stream scheduler and transient-state arena (host only, no GPU) -------------------------------------------
 * The reference's RuntimeStreamScheduler (stream_runtime.rs:426-1433) over its TransientStateArena / Table
 * (stream_state.rs:122-633), without the prefix-state cache: input events are cut into prefill chunks that end at
 * state-page boundaries and into decode feedback windows; each activation reserves its state slots (KV pages)
 * ahead of execution and gives back the ones it did not use when it completes; interrupt, close-after-current,
 * reset, remove and fork follow the reference.  Strings written into the structs below are NUL-terminated and cut
 * at 63 bytes. */
typedef struct nerve_b200_scheduler nerve_b200_scheduler;
typedef struct {
    const char *node_instance_id, *state_id;
    uint64_t bytes_per_activation, activation_capacity;
    uint64_t maximum_activation_count; /* 0 = unbounded; else the state is a ring of that many activations */
    int32_t retention;                 /* 0 = append, 1 = mutable singleton (activation_capacity is ignored) */
} nerve_b200_state_declaration;
typedef struct {
    uint64_t max_activations, max_prefill_tokens_per_activation, max_decode_tokens_per_activation, max_work_units;
} nerve_b200_scheduler_budget;
typedef struct {
    int32_t status; /* 0 idle, 1 active, 2 interrupted, 3 closing (stream_runtime.rs:15-21) */
    uint64_t queued_input_event_count, in_flight_activation_count, completed_input_event_count, scheduled_activation_count,
        generated_token_count, transient_state_entry_count, transient_state_block_count, transient_state_logical_activation_count;
    char current_input_event_id[64]; /* empty = none */
} nerve_b200_stream_snapshot;
typedef struct {
    uint64_t stream_count, active_stream_count, in_flight_activation_count, allocated_block_count, free_block_count, live_block_count;
} nerve_b200_scheduler_counts;
typedef struct {
    uint64_t id;
    int32_t kind; /* 0 = prefill chunk, 1 = decode feedback (stream_runtime.rs:44-55) */
    uint64_t token_offset, token_count, remaining_prompt_token_count; /* prefill chunk */
    uint64_t feedback_depth, max_tokens;                              /* decode feedback */
    uint64_t max_state_activation_count, reservation_count;
    char stream_id[64], execution_class_id[64], input_event_id[64];
} nerve_b200_activation;
typedef struct {
    uint64_t logical_activation_index, block_id, block_activation_offset, block_activation_capacity;
    int32_t allocated_block;
    int64_t copy_from_block_id; /* -1 = none; else copy that block into block_id before the write */
} nerve_b200_state_slot;

int32_t nerve_b200_scheduler_create(nerve_b200_scheduler **out);
int32_t nerve_b200_scheduler_destroy(nerve_b200_scheduler *scheduler);
/* add_stream_with_state_declarations_and_execution_class (stream_runtime.rs:482-515); execution_class_id NULL = "default". */
int32_t nerve_b200_scheduler_add_stream(nerve_b200_scheduler *scheduler, const char *stream_id, const char *execution_class_id,
                                        const nerve_b200_state_declaration *declarations, size_t declaration_count,
                                        nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_fork_stream(nerve_b200_scheduler *scheduler, const char *source_stream_id, const char *target_stream_id,
                                         const char *execution_class_id, nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_enqueue(nerve_b200_scheduler *scheduler, const char *stream_id, const char *event_id,
                                     const uint32_t *token_ids, size_t token_count, uint64_t max_public_tokens,
                                     nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_interrupt(nerve_b200_scheduler *scheduler, const char *stream_id, const char *reason,
                                       nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_reset_stream_state(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_remove_stream(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_close_after_current(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out);
/* schedule_step (stream_runtime.rs:833-889).  The step stays inside the scheduler until the next schedule call;
 * out_flags: bit 0 activation budget exhausted, bit 1 work budget exhausted, bit 2 idle. */
int32_t nerve_b200_scheduler_schedule_step(nerve_b200_scheduler *scheduler, const nerve_b200_scheduler_budget *budget,
                                           size_t *out_activation_count, int32_t *out_flags);
/* Activation `index` of the last step; its prefill tokens go to out_token_ids (may be NULL). */
int32_t nerve_b200_scheduler_step_activation(nerve_b200_scheduler *scheduler, size_t index, nerve_b200_activation *out,
                                             uint32_t *out_token_ids, size_t max_token_ids);
/* State reservation `reservation_index` of that activation: the state's key (two 64-byte buffers) and its slots. */
int32_t nerve_b200_scheduler_step_reservation(nerve_b200_scheduler *scheduler, size_t activation_index, size_t reservation_index,
                                              char *out_node_instance_id, char *out_state_id, nerve_b200_state_slot *out_slots,
                                              size_t max_slots, size_t *out_slot_count);
/* complete_activation (stream_runtime.rs:1032-1175).  processed_state_activation_count -1 = the activation's work units. */
int32_t nerve_b200_scheduler_complete(nerve_b200_scheduler *scheduler, uint64_t activation_id, const uint32_t *generated_token_ids,
                                      size_t generated_count, int32_t continue_generation, int64_t processed_state_activation_count,
                                      nerve_b200_stream_snapshot *out);
int32_t nerve_b200_scheduler_snapshot(nerve_b200_scheduler *scheduler, nerve_b200_scheduler_counts *out);
int32_t nerve_b200_scheduler_stream_snapshot(nerve_b200_scheduler *scheduler, const char *stream_id, nerve_b200_stream_snapshot *out);

/* The scheduler's prefix-state cache (stream_runtime.rs:541-559, 616-705; stream_prefix_cache.rs:104-312).  A new
 * scheduler has capacity 0 (RuntimeStreamScheduler::default); set_prefix_state_cache_capacity evicts down to the new
 * capacity and reports how many entries left.  cache_stream_prefix_state_for_tokens retains a fork of the stream's
 * state table under (the stream's execution class, runtime_graph_id, token_ids, the hash of runtime_modifier_bytes,
 * all of the stream's state keys): the append states must stand exactly at token_count activations, on a block
 * boundary.  out_flags bit 0 = an entry of the same key was replaced; out_evicted = entries evicted to make room.
 * restore_longest_stream_prefix_state shares the blocks of the longest retained prefix of token_ids into the target
 * stream's (empty) states - the key set is the target's declared states - and writes its token count, 0 when nothing
 * matches.  prefix_state_cache_counts: [0] capacity_entries, [1] entry_count, [2] eviction_count. */
int32_t nerve_b200_scheduler_set_prefix_state_cache_capacity(nerve_b200_scheduler *scheduler, uint64_t capacity_entries, uint64_t *out_evicted);
int32_t nerve_b200_scheduler_cache_stream_prefix_state_for_tokens(nerve_b200_scheduler *scheduler, const char *stream_id, const char *runtime_graph_id,
                                                                  const uint32_t *token_ids, size_t token_count,
                                                                  const uint8_t *runtime_modifier_bytes, size_t runtime_modifier_count,
                                                                  int32_t *out_flags, uint64_t *out_evicted);
int32_t nerve_b200_scheduler_restore_longest_stream_prefix_state(nerve_b200_scheduler *scheduler, const char *target_stream_id,
                                                                 const char *runtime_graph_id, const uint32_t *token_ids, size_t token_count,
                                                                 const uint8_t *runtime_modifier_bytes, size_t runtime_modifier_count,
                                                                 uint64_t *out_restored_token_count);
int32_t nerve_b200_scheduler_prefix_state_cache_counts(nerve_b200_scheduler *scheduler, uint64_t out_counts[3]);

#ifdef __cplusplus
}
#endif

#endif /* NERVE_B200_H */
