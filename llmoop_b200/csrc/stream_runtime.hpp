// Host-side stream scheduler and transient-state arena of the runtime: which stream runs next, in what chunk, and
// which state pages (KV blocks) it may write.  Restates, in C++, the semantics of the reference's
//   runtime-rs/src/stream_state.rs:5-747    (block arena with reference counts, per-stream state tables, append /
//                                            rollback / fork / share, ring-bounded states, mutable singletons)
//   runtime-rs/src/stream_runtime.rs:15-1433 (input events, prefill chunks cut at page boundaries, decode feedback
//                                            windows, reservations of state slots ahead of execution, rollback of
//                                            the slots an activation did not use, interrupt / close / remove / fork,
//                                            grouping of compatible activations into batches; the scheduler's
//                                            hooks of the prefix-state cache, :541-705)
//   runtime-rs/src/stream_prefix_cache.rs:1-379 (prefix-state cache: states retained under the token prefix that
//                                            produced them, least-recently-used eviction, longest-prefix lookup)
// Pure host code, no CUDA: errors are exceptions of type RuntimeError, the C ABI turns them into a status and a
// message.
#pragma once

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
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

// ---------------------------------------------------------------------------------------------- prefix cache

// FNV-1a over a domain string, the length and the little-endian contents (stream_prefix_cache.rs:330-353).
uint64_t stable_token_prefix_hash(const uint32_t *token_ids, size_t count);
uint64_t stable_runtime_modifier_hash(const uint8_t *bytes, size_t count);

// What a retained state is filed under: who may use it (execution class, runtime graph, the hash of the runtime
// modifiers - sampler, draft count - that shaped it), the tokens that produced it, and the states it holds
// (stream_prefix_cache.rs:12-71).  Ordered field by field, which is also the order of the snapshots.
struct PrefixStateCacheKey {
    std::string execution_class_id, runtime_graph_id;
    size_t token_count = 0;
    std::vector<uint32_t> token_ids;
    uint64_t token_hash = 0, runtime_modifier_hash = 0;
    std::vector<StateKey> state_keys;  // sorted, without duplicates

    static PrefixStateCacheKey from_token_prefix(const std::string &execution_class_id, const std::string &runtime_graph_id,
                                                 const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                 std::vector<StateKey> state_keys);
    bool operator<(const PrefixStateCacheKey &other) const;
    bool operator==(const PrefixStateCacheKey &other) const;
    bool operator!=(const PrefixStateCacheKey &other) const { return !(*this == other); }
};

// The filing system itself, for any payload: entries under their keys with the time and the number of their uses,
// a capacity in entries, eviction of the least recently used entry (ties: the less used one), and the lookup of the
// longest filed prefix of a token sequence.  Whoever owns the payloads releases what a call hands back.
// (stream_prefix_cache.rs:104-312, without the state tables.)  The lookup walks the entries - a handful, one per
// stream - and compares tokens, instead of hashing every prefix length of the query as the reference does: a
// 32 768-token prompt would cost 5 * 10^8 hash steps there.
template <class Payload>
class PrefixCacheIndex {
  public:
    struct Entry {
        Payload payload;
        uint64_t last_used_tick = 0;
        size_t use_count = 0;
    };
    using Removed = std::vector<std::pair<PrefixStateCacheKey, Payload>>;

    explicit PrefixCacheIndex(size_t capacity_entries = 0) : capacity_entries_(capacity_entries) {}
    size_t capacity_entries() const { return capacity_entries_; }
    size_t eviction_count() const { return eviction_count_; }
    const std::map<PrefixStateCacheKey, Entry> &entries() const { return entries_; }

    Removed set_capacity(size_t capacity_entries) {
        capacity_entries_ = capacity_entries;
        return evict_until_within_capacity();
    }
    std::optional<Payload> evict(const PrefixStateCacheKey &key) {
        auto found = entries_.find(key);
        if (found == entries_.end()) return std::nullopt;
        Payload payload = std::move(found->second.payload);
        entries_.erase(found);
        eviction_count_++;
        return payload;
    }
    // Files the payload (an entry of the same key is handed back as `replaced`), then evicts down to the capacity.
    struct Inserted {
        std::optional<Payload> replaced;
        Removed evicted;
    };
    Inserted insert(const PrefixStateCacheKey &key, Payload payload) {
        Inserted result;
        auto found = entries_.find(key);
        if (found != entries_.end()) {
            result.replaced = std::move(found->second.payload);
            entries_.erase(found);
        }
        entries_.emplace(key, Entry{std::move(payload), next_tick(), 0});
        result.evicted = evict_until_within_capacity();
        return result;
    }
    // The payload under `key`, counted as a use; nullptr when nothing is filed there.
    Payload *use(const PrefixStateCacheKey &key) {
        const uint64_t tick = next_tick();
        auto found = entries_.find(key);
        if (found == entries_.end()) return nullptr;
        found->second.last_used_tick = tick;
        found->second.use_count++;
        return &found->second.payload;
    }
    std::optional<PrefixStateCacheKey> longest_matching_key(const std::string &execution_class_id, const std::string &runtime_graph_id,
                                                            const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                            std::vector<StateKey> state_keys) const;
    std::string next_cached_stream_id() { return "prefix_cache_" + std::to_string(next_cached_stream_id_++); }

  private:
    uint64_t next_tick() { return next_tick_++; }
    Removed evict_until_within_capacity() {
        Removed removed;
        while (entries_.size() > capacity_entries_) {
            auto oldest = entries_.begin();
            for (auto it = entries_.begin(); it != entries_.end(); ++it)
                if (std::make_pair(it->second.last_used_tick, it->second.use_count) < std::make_pair(oldest->second.last_used_tick, oldest->second.use_count))
                    oldest = it;
            removed.emplace_back(oldest->first, std::move(oldest->second.payload));
            entries_.erase(oldest);
            eviction_count_++;
        }
        return removed;
    }
    size_t capacity_entries_;
    std::map<PrefixStateCacheKey, Entry> entries_;
    uint64_t next_tick_ = 0, next_cached_stream_id_ = 0;
    size_t eviction_count_ = 0;
};

void check_prefix_lookup_ids(const std::string &execution_class_id, const std::string &runtime_graph_id);
std::vector<StateKey> normalized_state_keys(std::vector<StateKey> state_keys);

template <class Payload>
std::optional<PrefixStateCacheKey> PrefixCacheIndex<Payload>::longest_matching_key(const std::string &execution_class_id, const std::string &runtime_graph_id,
                                                                                   const std::vector<uint32_t> &token_ids,
                                                                                   const std::string &runtime_modifier_bytes,
                                                                                   std::vector<StateKey> state_keys) const {
    check_prefix_lookup_ids(execution_class_id, runtime_graph_id);
    if (token_ids.empty()) return std::nullopt;
    state_keys = normalized_state_keys(std::move(state_keys));
    if (state_keys.empty()) throw RuntimeError("prefix cache state key set must not be empty");
    const uint64_t modifier_hash =
        stable_runtime_modifier_hash(reinterpret_cast<const uint8_t *>(runtime_modifier_bytes.data()), runtime_modifier_bytes.size());
    const PrefixStateCacheKey *best = nullptr;
    for (const auto &item : entries_) {
        const PrefixStateCacheKey &key = item.first;
        if (key.execution_class_id != execution_class_id || key.runtime_graph_id != runtime_graph_id || key.runtime_modifier_hash != modifier_hash ||
            key.state_keys != state_keys || key.token_count > token_ids.size() || (best != nullptr && key.token_count <= best->token_count))
            continue;
        if (std::equal(key.token_ids.begin(), key.token_ids.end(), token_ids.begin())) best = &key;
    }
    return best != nullptr ? std::optional<PrefixStateCacheKey>(*best) : std::nullopt;
}

struct PrefixStateCacheEntrySnapshot {
    PrefixStateCacheKey key;
    std::string cached_stream_id;
    size_t block_count = 0, logical_activation_count = 0;
    uint64_t last_used_tick = 0;
    size_t use_count = 0;
};
struct PrefixStateCacheSnapshot {
    size_t capacity_entries = 0, entry_count = 0, eviction_count = 0;
    std::vector<PrefixStateCacheEntrySnapshot> entries;  // by key
};
struct PrefixStateCacheInsert {
    bool replaced_existing = false;
    std::vector<PrefixStateCacheKey> evicted_keys;
};

// The cache of state tables (stream_prefix_cache.rs:104-312): an entry is a fork of the source stream's table, so
// its blocks stay alive in the arena after the source has moved on or gone; restoring shares them into a fresh table.
class PrefixStateCache {
  public:
    explicit PrefixStateCache(size_t capacity_entries = 0) : index_(capacity_entries) {}
    size_t capacity_entries() const { return index_.capacity_entries(); }
    std::vector<PrefixStateCacheKey> set_capacity(StateArena &arena, size_t capacity_entries);
    bool evict(StateArena &arena, const PrefixStateCacheKey &key);
    // The source's append states must stand exactly at the key's token count, on a block boundary; its mutable
    // states must be initialised (stream_prefix_cache.rs:354-403).  With capacity 0 nothing is retained.
    PrefixStateCacheInsert insert(StateArena &arena, const PrefixStateCacheKey &key, const StateTable &source);
    bool restore_into(StateArena &arena, const PrefixStateCacheKey &key, StateTable &target);
    std::optional<PrefixStateCacheKey> longest_matching_key(const std::string &execution_class_id, const std::string &runtime_graph_id,
                                                            const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                            std::vector<StateKey> state_keys) const {
        return index_.longest_matching_key(execution_class_id, runtime_graph_id, token_ids, runtime_modifier_bytes, std::move(state_keys));
    }
    PrefixStateCacheSnapshot snapshot() const;

  private:
    struct Retained {
        std::string cached_stream_id;
        StateTable table;
    };
    std::vector<PrefixStateCacheKey> release(StateArena &arena, PrefixCacheIndex<Retained>::Removed removed);
    PrefixCacheIndex<Retained> index_;
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
    explicit StreamScheduler(size_t prefix_state_cache_capacity = 0) : prefix_cache_(prefix_state_cache_capacity) {}
    // prefix-state cache (stream_runtime.rs:541-559, 616-705)
    PrefixStateCacheSnapshot prefix_state_cache_snapshot() const { return prefix_cache_.snapshot(); }
    std::vector<PrefixStateCacheKey> set_prefix_state_cache_capacity(size_t capacity_entries) { return prefix_cache_.set_capacity(arena_, capacity_entries); }
    bool evict_prefix_state(const PrefixStateCacheKey &key) { return prefix_cache_.evict(arena_, key); }
    PrefixStateCacheInsert cache_stream_prefix_state(const std::string &stream_id, const PrefixStateCacheKey &key);
    PrefixStateCacheKey cache_stream_prefix_state_for_tokens(const std::string &stream_id, const std::string &runtime_graph_id,
                                                             const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                             std::vector<StateKey> state_keys);
    bool restore_stream_prefix_state(const std::string &target_stream_id, const PrefixStateCacheKey &key);
    std::optional<PrefixStateCacheKey> restore_longest_stream_prefix_state(const std::string &target_stream_id, const std::string &runtime_graph_id,
                                                                           const std::vector<uint32_t> &token_ids,
                                                                           const std::string &runtime_modifier_bytes, std::vector<StateKey> state_keys);
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
    PrefixStateCache prefix_cache_;
    uint64_t next_activation_id_ = 0;
};

std::vector<ActivationBatch> group_compatible_stream_activations(std::vector<Activation> activations);

}  // namespace runtime
}  // namespace nerve
