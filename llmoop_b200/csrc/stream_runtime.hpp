// Host-side stream scheduler and transient-state arena of the runtime: which stream runs next, in what chunk, and
// which state pages (KV blocks) it may write.  Restates, in C++, the semantics of the reference's
//   runtime-rs/src/stream_state.rs:5-747    (block arena with reference counts, per-stream state tables, append /
//                                            rollback / fork / share, ring-bounded states, mutable singletons)
//   runtime-rs/src/stream_runtime.rs:15-1433 (input events, prefill chunks cut at page boundaries, decode feedback
//                                            windows, reservations of state slots ahead of execution, rollback of
//                                            the slots an activation did not use, interrupt / close / remove / fork,
//                                            grouping of compatible activations into batches)
// without the prefix-state cache (stream_runtime.rs:541-705).  Pure host code, no CUDA: errors are exceptions of
// type RuntimeError, the C ABI turns them into a status and a message.
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace nerve {
namespace runtime {

struct RuntimeError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

using BlockId = uint64_t;

struct StateKey {
    std::string node_instance_id, state_id;
    bool operator<(const StateKey &other) const;
    bool operator==(const StateKey &other) const;
    bool operator!=(const StateKey &other) const { return !(*this == other); }
};

enum class Retention { Append = 0, MutableSingleton = 1 };

// stream_state.rs:23-86
struct BlockShape {
    size_t bytes_per_activation = 0, activation_capacity = 0;
    std::optional<size_t> maximum_activation_count;  // ring bound: logical index % maximum is the resident index
    Retention retention = Retention::Append;

    static BlockShape append(size_t bytes_per_activation, size_t activation_capacity);
    BlockShape with_maximum_activation_count(size_t maximum) const;
    static BlockShape mutable_singleton(size_t byte_capacity);
    size_t byte_capacity() const;
    bool operator<(const BlockShape &other) const;
    bool operator==(const BlockShape &other) const;
    bool operator!=(const BlockShape &other) const { return !(*this == other); }
};

// stream_state.rs:88-97: one activation's place in a block; copy_from = the shared block whose contents must be
// copied into a freshly allocated replacement before the write (copy on write).
struct StateSlot {
    StateKey key;
    size_t logical_activation_index = 0;
    BlockId block_id = 0;
    size_t block_activation_offset = 0, block_activation_capacity = 0;
    bool allocated_block = false;
    std::optional<BlockId> copy_from_block_id;
    bool operator==(const StateSlot &other) const;
};

struct BlockSnapshot {
    BlockId block_id;
    BlockShape shape;
    size_t ref_count, byte_capacity;
    bool operator==(const BlockSnapshot &other) const;
};
struct ArenaSnapshot {
    size_t allocated_block_count = 0, free_block_count = 0, live_block_count = 0;
    std::vector<BlockSnapshot> blocks;  // by block id
    bool operator==(const ArenaSnapshot &other) const;
};

// stream_state.rs:122-239
class StateArena {
  public:
    BlockId allocate_block(const BlockShape &shape);  // reuses the most recently freed block of the same shape
    void retain_block(BlockId block);
    void release_block(BlockId block);
    size_t ref_count(BlockId block) const;
    ArenaSnapshot snapshot() const;

  private:
    struct Block {
        BlockShape shape;
        size_t ref_count;
    };
    Block &block(BlockId id);
    const Block &block(BlockId id) const;
    BlockId next_block_id_ = 0;
    std::map<BlockId, Block> blocks_;
    std::map<BlockShape, std::vector<BlockId>> free_blocks_;
};

struct EntrySnapshot {
    StateKey key;
    BlockShape shape;
    size_t logical_activation_count;
    std::vector<BlockId> block_ids;
    bool operator==(const EntrySnapshot &other) const;
};
struct TableSnapshot {
    std::string stream_id;
    size_t entry_count = 0, logical_activation_count = 0, block_count = 0;
    std::vector<EntrySnapshot> entries;  // by key
    bool operator==(const TableSnapshot &other) const;
};

// stream_state.rs:265-633
class StateTable {
  public:
    explicit StateTable(std::string stream_id);
    const std::string &stream_id() const { return stream_id_; }
    void declare_state(const StateKey &key, const BlockShape &shape);
    std::vector<StateSlot> append_activations(StateArena &arena, const StateKey &key, size_t activation_count);
    // `slots` must be the latest contiguous reservation of the state (checked); pages left empty are released.
    void rollback_slots(StateArena &arena, const StateKey &key, const StateSlot *slots, size_t count);
    void reset_state(StateArena &arena, const StateKey &key);
    void reset_all(StateArena &arena);
    StateTable fork(StateArena &arena, std::string new_stream_id) const;
    void share_states_from(StateArena &arena, const StateTable &source, const std::vector<StateKey> &keys);
    TableSnapshot snapshot() const;
    std::vector<StateKey> state_keys() const;
    // Activations until the append states of this stream reach their next common page boundary, if that is
    // within maximum_distance (stream_state.rs:578-611).
    std::optional<size_t> next_append_block_boundary_distance(size_t maximum_distance) const;

  private:
    struct Entry {
        BlockShape shape;
        size_t logical_activation_count = 0;
        std::vector<BlockId> block_ids;
    };
    Entry &entry(const StateKey &key);
    const Entry &entry(const StateKey &key) const;
    std::string stream_id_;
    std::map<StateKey, Entry> entries_;
};

// ---------------------------------------------------------------------------------------------- scheduler

enum class StreamStatus { Idle = 0, Active = 1, Interrupted = 2, Closing = 3 };

struct InputEvent {
    std::string id;
    std::vector<uint32_t> token_ids;
    size_t max_public_tokens = 0;
};

enum class ActivationKind { PrefillChunk = 0, DecodeFeedback = 1 };

struct StateReservation {
    StateKey key;
    std::vector<StateSlot> slots;
};

// stream_runtime.rs:44-81
struct Activation {
    uint64_t id = 0;
    std::string stream_id, execution_class_id, input_event_id;
    ActivationKind kind = ActivationKind::PrefillChunk;
    // PrefillChunk
    size_t token_offset = 0;
    std::vector<uint32_t> token_ids;
    size_t remaining_prompt_token_count = 0;
    // DecodeFeedback
    size_t feedback_depth = 0, max_tokens = 0;
    size_t max_state_activation_count = 0;
    std::vector<StateReservation> state_reservations;
    size_t work_units() const { return kind == ActivationKind::PrefillChunk ? token_ids.size() : max_tokens; }
};

// stream_runtime.rs:83-118
struct ActivationOutcome {
    std::vector<uint32_t> generated_token_ids;
    bool continue_generation = true;
    std::optional<size_t> processed_state_activation_count;
    static ActivationOutcome prefill_complete() { return {}; }
    static ActivationOutcome generated(std::vector<uint32_t> tokens, bool continue_generation) {
        ActivationOutcome outcome;
        outcome.generated_token_ids = std::move(tokens);
        outcome.continue_generation = continue_generation;
        return outcome;
    }
    ActivationOutcome with_processed_state_activations(size_t count) const {
        ActivationOutcome outcome = *this;
        outcome.processed_state_activation_count = count;
        return outcome;
    }
};

// stream_runtime.rs:120-146
struct SchedulerBudget {
    size_t max_activations = 0, max_prefill_tokens_per_activation = 0, max_decode_tokens_per_activation = 1, max_work_units = 0;
    SchedulerBudget() = default;
    SchedulerBudget(size_t activations, size_t prefill_tokens, size_t work_units)
        : max_activations(activations), max_prefill_tokens_per_activation(prefill_tokens), max_work_units(work_units) {}
    SchedulerBudget with_max_decode_tokens_per_activation(size_t tokens) const {
        SchedulerBudget budget = *this;
        budget.max_decode_tokens_per_activation = tokens;
        return budget;
    }
};

struct SchedulerStep {
    std::vector<Activation> activations;
    bool exhausted_activation_budget = false, exhausted_work_budget = false, idle = false;
};

// Activations of one batch share the execution class, the kind and its width (stream_runtime.rs:156-183).
struct BatchKind {
    ActivationKind kind;
    std::string execution_class_id;
    size_t width;  // prefill: token count; decode: max_tokens
    bool operator==(const BatchKind &other) const {
        return kind == other.kind && execution_class_id == other.execution_class_id && width == other.width;
    }
};
struct ActivationBatch {
    BatchKind kind;
    std::vector<Activation> activations;
};
struct SchedulerBatchStep {
    std::vector<ActivationBatch> batches;
    bool exhausted_activation_budget = false, exhausted_work_budget = false, idle = false;
};

struct StreamSnapshot {
    std::string stream_id, execution_class_id;
    StreamStatus status = StreamStatus::Idle;
    size_t queued_input_event_count = 0;
    std::optional<std::string> current_input_event_id;
    size_t in_flight_activation_count = 0, completed_input_event_count = 0, scheduled_activation_count = 0, generated_token_count = 0;
    size_t transient_state_entry_count = 0, transient_state_block_count = 0, transient_state_logical_activation_count = 0;
};
struct SchedulerSnapshot {
    size_t stream_count = 0, active_stream_count = 0, in_flight_activation_count = 0;
    ArenaSnapshot transient_state_arena;
    std::vector<StreamSnapshot> streams;  // by stream id
};

enum class RunStop { Idle = 0, StepBudget = 1 };
struct CompletedActivation {
    Activation activation;
    ActivationOutcome outcome;
};
struct BatchActivationOutcome {
    uint64_t activation_id;
    ActivationOutcome outcome;
};
struct SchedulerRun {
    RunStop stop_condition = RunStop::Idle;
    size_t max_steps = 0, scheduled_steps = 0;
    std::vector<CompletedActivation> completed_activations;
    SchedulerSnapshot final_snapshot;
};

// stream_runtime.rs:426-1433
class StreamScheduler {
  public:
    using Declarations = std::vector<std::pair<StateKey, BlockShape>>;
    StreamSnapshot add_stream(const std::string &stream_id, const std::string &execution_class_id = "default",
                              const Declarations &state_declarations = {});
    StreamSnapshot declare_stream_state(const std::string &stream_id, const StateKey &key, const BlockShape &shape);
    ArenaSnapshot transient_state_arena_snapshot() const { return arena_.snapshot(); }
    TableSnapshot stream_transient_state_snapshot(const std::string &stream_id) const;
    StreamSnapshot fork_stream_transient_state(const std::string &source_stream_id, const std::string &target_stream_id,
                                               const std::string &execution_class_id);
    StreamSnapshot share_stream_state(const std::string &target_stream_id, const std::string &source_stream_id, const StateKey &key);
    StreamSnapshot enqueue_input_event(const std::string &stream_id, const InputEvent &event);
    StreamSnapshot interrupt_stream(const std::string &stream_id, const std::string &reason);
    StreamSnapshot reset_stream_transient_state(const std::string &stream_id);
    StreamSnapshot remove_stream(const std::string &stream_id);
    StreamSnapshot close_stream_after_current(const std::string &stream_id);
    SchedulerStep schedule_step(const SchedulerBudget &budget);
    SchedulerBatchStep schedule_batch_step(const SchedulerBudget &budget);
    StreamSnapshot complete_activation(uint64_t activation_id, const ActivationOutcome &outcome);
    SchedulerRun run_until_idle_with(const SchedulerBudget &budget, size_t max_steps,
                                     const std::function<ActivationOutcome(const Activation &)> &execute);
    SchedulerRun run_batches_until_idle_with(const SchedulerBudget &budget, size_t max_steps,
                                             const std::function<std::vector<BatchActivationOutcome>(const ActivationBatch &)> &execute);
    SchedulerSnapshot snapshot() const;

  private:
    struct CurrentEvent {
        InputEvent event;
        size_t next_prompt_token_index = 0, generated_token_count = 0, next_feedback_depth = 0;
        bool prompt_done() const { return next_prompt_token_index >= event.token_ids.size(); }
        bool generation_done() const { return generated_token_count >= event.max_public_tokens; }
    };
    struct Stream {
        std::string stream_id, execution_class_id;
        StreamStatus status = StreamStatus::Idle;
        bool closing_after_current = false;
        std::deque<InputEvent> queued_input_events;
        std::optional<CurrentEvent> current_event;
        std::vector<uint64_t> in_flight_activation_ids;
        size_t completed_input_event_count = 0, scheduled_activation_count = 0, generated_token_count = 0;
        StateTable table;
        Stream(std::string id, std::string execution_class, StateTable state_table);
        bool has_in_flight_work() const { return !in_flight_activation_ids.empty(); }
        bool has_schedulable_running_work() const { return current_event.has_value() && !has_in_flight_work(); }
        bool has_schedulable_waiting_work() const;
        bool has_pending_work() const { return current_event.has_value() || !queued_input_events.empty() || has_in_flight_work(); }
        void refresh_status();
        StreamSnapshot snapshot() const;
    };
    Stream &stream(const std::string &stream_id);
    const Stream &stream(const std::string &stream_id) const;
    std::optional<Activation> prepare_activation(const std::string &stream_id, size_t max_prefill_tokens, size_t max_decode_tokens);
    void rollback_unused_activation_state(const Activation &activation, size_t processed_state_activation_count);
    std::optional<std::string> next_schedulable_stream_id();
    void refresh_active_queue();
    void activate_stream(const std::string &stream_id);
    size_t active_stream_count() const;

    std::map<std::string, Stream> streams_;
    std::deque<std::string> active_queue_;
    std::map<uint64_t, Activation> in_flight_;
    StateArena arena_;
    uint64_t next_activation_id_ = 0;
};

std::vector<ActivationBatch> group_compatible_stream_activations(std::vector<Activation> activations);

}  // namespace runtime
}  // namespace nerve
