// Stream scheduler and transient-state arena (see stream_runtime.hpp for the reference files this restates).
#include "stream_runtime.hpp"

#include <algorithm>
#include <limits>
#include <set>
#include <tuple>

namespace nerve {
namespace runtime {

namespace {

[[noreturn]] void fail(const std::string &message) { throw RuntimeError(message); }

std::string quoted(const std::string &text) { return "\"" + text + "\""; }

std::string key_name(const StateKey &key) { return key.node_instance_id + "." + key.state_id; }

size_t checked_add(size_t left, size_t right, const char *what) {
    if (left > std::numeric_limits<size_t>::max() - right) fail(std::string(what) + " overflow");
    return left + right;
}

std::vector<BlockId> unique_block_ids(const std::vector<BlockId> &ids) {
    std::set<BlockId> unique(ids.begin(), ids.end());
    return std::vector<BlockId>(unique.begin(), unique.end());
}

size_t greatest_common_divisor(size_t left, size_t right) {
    while (right != 0) {
        const size_t remainder = left % right;
        left = right;
        right = remainder;
    }
    return left;
}

size_t least_common_multiple(size_t left, size_t right) {
    const size_t divisor = greatest_common_divisor(left, right);
    const size_t reduced = divisor == 0 ? 0 : left / divisor;
    if (divisor == 0 || (right != 0 && reduced > std::numeric_limits<size_t>::max() / right)) fail("transient state block alignment overflow");
    return reduced * right;
}

size_t resident_index(const BlockShape &shape, size_t logical_index) {
    return shape.maximum_activation_count ? logical_index % *shape.maximum_activation_count : logical_index;
}

}  // namespace

// ---------------------------------------------------------------------------------------------- keys and shapes

bool StateKey::operator<(const StateKey &other) const {
    return std::tie(node_instance_id, state_id) < std::tie(other.node_instance_id, other.state_id);
}
bool StateKey::operator==(const StateKey &other) const { return node_instance_id == other.node_instance_id && state_id == other.state_id; }

BlockShape BlockShape::append(size_t bytes_per_activation, size_t activation_capacity) {
    if (bytes_per_activation == 0) fail("transient state block bytes_per_activation must be positive");
    if (activation_capacity == 0) fail("transient state block activation_capacity must be positive");
    BlockShape shape;
    shape.bytes_per_activation = bytes_per_activation;
    shape.activation_capacity = activation_capacity;
    return shape;
}

BlockShape BlockShape::with_maximum_activation_count(size_t maximum) const {
    if (maximum == 0) fail("transient state maximum activation count must be positive");
    BlockShape shape = *this;
    shape.maximum_activation_count = maximum;
    return shape;
}

BlockShape BlockShape::mutable_singleton(size_t byte_capacity) {
    BlockShape shape = append(byte_capacity, 1);
    shape.retention = Retention::MutableSingleton;
    return shape;
}

size_t BlockShape::byte_capacity() const {
    if (activation_capacity != 0 && bytes_per_activation > std::numeric_limits<size_t>::max() / activation_capacity)
        fail("transient state block byte capacity overflow");
    return bytes_per_activation * activation_capacity;
}

bool BlockShape::operator<(const BlockShape &other) const {
    return std::make_tuple(bytes_per_activation, activation_capacity, maximum_activation_count, static_cast<int>(retention)) <
           std::make_tuple(other.bytes_per_activation, other.activation_capacity, other.maximum_activation_count, static_cast<int>(other.retention));
}
bool BlockShape::operator==(const BlockShape &other) const {
    return bytes_per_activation == other.bytes_per_activation && activation_capacity == other.activation_capacity &&
           maximum_activation_count == other.maximum_activation_count && retention == other.retention;
}

bool StateSlot::operator==(const StateSlot &other) const {
    return key == other.key && logical_activation_index == other.logical_activation_index && block_id == other.block_id &&
           block_activation_offset == other.block_activation_offset && block_activation_capacity == other.block_activation_capacity &&
           allocated_block == other.allocated_block && copy_from_block_id == other.copy_from_block_id;
}
bool BlockSnapshot::operator==(const BlockSnapshot &other) const {
    return block_id == other.block_id && shape == other.shape && ref_count == other.ref_count && byte_capacity == other.byte_capacity;
}
bool ArenaSnapshot::operator==(const ArenaSnapshot &other) const {
    return allocated_block_count == other.allocated_block_count && free_block_count == other.free_block_count &&
           live_block_count == other.live_block_count && blocks == other.blocks;
}
bool EntrySnapshot::operator==(const EntrySnapshot &other) const {
    return key == other.key && shape == other.shape && logical_activation_count == other.logical_activation_count && block_ids == other.block_ids;
}
bool TableSnapshot::operator==(const TableSnapshot &other) const {
    return stream_id == other.stream_id && entry_count == other.entry_count && logical_activation_count == other.logical_activation_count &&
           block_count == other.block_count && entries == other.entries;
}

// ---------------------------------------------------------------------------------------------- arena

StateArena::Block &StateArena::block(BlockId id) {
    auto found = blocks_.find(id);
    if (found == blocks_.end()) fail("unknown transient state block " + std::to_string(id));
    return found->second;
}
const StateArena::Block &StateArena::block(BlockId id) const {
    auto found = blocks_.find(id);
    if (found == blocks_.end()) fail("unknown transient state block " + std::to_string(id));
    return found->second;
}

BlockId StateArena::allocate_block(const BlockShape &shape) {
    shape.byte_capacity();
    auto free_for_shape = free_blocks_.find(shape);
    if (free_for_shape != free_blocks_.end() && !free_for_shape->second.empty()) {
        const BlockId id = free_for_shape->second.back();
        free_for_shape->second.pop_back();
        if (free_for_shape->second.empty()) free_blocks_.erase(free_for_shape);
        block(id).ref_count = 1;
        return id;
    }
    const BlockId id = next_block_id_;
    if (next_block_id_ == std::numeric_limits<BlockId>::max()) fail("transient state block id overflow");
    next_block_id_++;
    blocks_.emplace(id, Block{shape, 1});
    return id;
}

void StateArena::retain_block(BlockId id) {
    Block &target = block(id);
    target.ref_count = checked_add(target.ref_count, 1, "transient state block refcount");
}

void StateArena::release_block(BlockId id) {
    Block &target = block(id);
    if (target.ref_count == 0) fail("transient state block " + std::to_string(id) + " is already free");
    if (--target.ref_count == 0) free_blocks_[target.shape].push_back(id);
}

size_t StateArena::ref_count(BlockId id) const { return block(id).ref_count; }

ArenaSnapshot StateArena::snapshot() const {
    ArenaSnapshot snapshot;
    snapshot.allocated_block_count = blocks_.size();
    for (const auto &item : blocks_) {
        snapshot.blocks.push_back(BlockSnapshot{item.first, item.second.shape, item.second.ref_count, item.second.shape.byte_capacity()});
        if (item.second.ref_count == 0) snapshot.free_block_count++;
        else snapshot.live_block_count++;
    }
    return snapshot;
}

// ---------------------------------------------------------------------------------------------- state table

StateTable::StateTable(std::string stream_id) : stream_id_(std::move(stream_id)) {
    if (stream_id_.empty()) fail("transient state table stream id must not be empty");
}

StateTable::Entry &StateTable::entry(const StateKey &key) {
    auto found = entries_.find(key);
    if (found == entries_.end()) fail("stream " + quoted(stream_id_) + " has no transient state " + key_name(key));
    return found->second;
}
const StateTable::Entry &StateTable::entry(const StateKey &key) const {
    auto found = entries_.find(key);
    if (found == entries_.end()) fail("stream " + quoted(stream_id_) + " has no transient state " + key_name(key));
    return found->second;
}

void StateTable::declare_state(const StateKey &key, const BlockShape &shape) {
    if (key.node_instance_id.empty() || key.state_id.empty()) fail("transient state key node_instance_id and state_id must not be empty");
    auto found = entries_.find(key);
    if (found != entries_.end()) {
        if (found->second.shape != shape) fail("transient state " + key_name(key) + " was already declared with a different block shape");
        return;
    }
    Entry fresh;
    fresh.shape = shape;
    entries_.emplace(key, std::move(fresh));
}

std::vector<StateSlot> StateTable::append_activations(StateArena &arena, const StateKey &key, size_t activation_count) {
    std::vector<StateSlot> slots;
    if (activation_count == 0) return slots;
    Entry &target = entry(key);
    if (target.shape.retention == Retention::MutableSingleton) {
        // one block rewritten in place; a forked (shared) block is replaced by a private copy first (stream_state.rs:635-669)
        StateSlot slot;
        slot.key = key;
        slot.block_activation_capacity = 1;
        if (target.block_ids.empty()) {
            slot.block_id = arena.allocate_block(target.shape);
            target.block_ids.push_back(slot.block_id);
            target.logical_activation_count = 1;
            slot.allocated_block = true;
        } else if (arena.ref_count(target.block_ids[0]) > 1) {
            const BlockId shared = target.block_ids[0];
            slot.block_id = arena.allocate_block(target.shape);
            arena.release_block(shared);
            target.block_ids[0] = slot.block_id;
            slot.allocated_block = true;
            slot.copy_from_block_id = shared;
        } else {
            slot.block_id = target.block_ids[0];
        }
        slots.push_back(std::move(slot));
        return slots;
    }
    slots.reserve(activation_count);
    for (size_t n = 0; n < activation_count; n++) {
        const size_t resident = resident_index(target.shape, target.logical_activation_count);
        const size_t page = resident / target.shape.activation_capacity;
        StateSlot slot;
        slot.key = key;
        slot.logical_activation_index = target.logical_activation_count;
        slot.block_activation_offset = resident % target.shape.activation_capacity;
        slot.block_activation_capacity = target.shape.activation_capacity;
        if (page == target.block_ids.size()) {
            target.block_ids.push_back(arena.allocate_block(target.shape));
            slot.allocated_block = true;
        } else if (arena.ref_count(target.block_ids[page]) > 1) {
            const BlockId shared = target.block_ids[page];
            const BlockId replacement = arena.allocate_block(target.shape);
            arena.release_block(shared);
            target.block_ids[page] = replacement;
            slot.allocated_block = true;
            slot.copy_from_block_id = shared;
        }
        slot.block_id = target.block_ids[page];
        slots.push_back(std::move(slot));
        target.logical_activation_count = checked_add(target.logical_activation_count, 1, "transient state logical activation count");
    }
    return slots;
}

void StateTable::rollback_slots(StateArena &arena, const StateKey &key, const StateSlot *slots, size_t count) {
    if (count == 0) return;
    Entry &target = entry(key);
    if (target.shape.retention == Retention::MutableSingleton) {
        // stream_state.rs:671-700
        if (count != 1 || slots[0].key != key) fail("mutable singleton rollback for " + key_name(key) + " requires its one reservation slot");
        const StateSlot &slot = slots[0];
        if (target.block_ids.empty() || target.block_ids[0] != slot.block_id)
            fail("mutable singleton rollback for " + key_name(key) + " no longer owns block " + std::to_string(slot.block_id));
        if (slot.copy_from_block_id) {
            arena.retain_block(*slot.copy_from_block_id);
            arena.release_block(slot.block_id);
            target.block_ids[0] = *slot.copy_from_block_id;
        } else if (slot.allocated_block) {
            arena.release_block(slot.block_id);
            target.block_ids.clear();
            target.logical_activation_count = 0;
        }
        return;
    }
    for (size_t n = count; n-- > 0;) {
        const StateSlot &slot = slots[n];
        if (target.logical_activation_count == 0) fail("cannot roll back empty transient state " + key_name(key));
        const size_t expected = target.logical_activation_count - 1;
        if (slot.key != key || slot.logical_activation_index != expected)
            fail("transient state rollback for " + key_name(key) + " is not the latest contiguous reservation");
        const size_t page = resident_index(target.shape, slot.logical_activation_index) / target.shape.activation_capacity;
        if (page >= target.block_ids.size() || target.block_ids[page] != slot.block_id)
            fail("transient state rollback for " + key_name(key) + " no longer owns block " + std::to_string(slot.block_id));
        if (slot.copy_from_block_id) {  // undo the copy on write: the shared block comes back
            arena.retain_block(*slot.copy_from_block_id);
            arena.release_block(slot.block_id);
            target.block_ids[page] = *slot.copy_from_block_id;
        }
        target.logical_activation_count = expected;
    }
    size_t retained = target.logical_activation_count;
    if (target.shape.maximum_activation_count) retained = std::min(retained, *target.shape.maximum_activation_count);
    const size_t retained_pages = (retained + target.shape.activation_capacity - 1) / target.shape.activation_capacity;
    while (target.block_ids.size() > retained_pages) {
        arena.release_block(target.block_ids.back());
        target.block_ids.pop_back();
    }
}

void StateTable::reset_state(StateArena &arena, const StateKey &key) {
    Entry &target = entry(key);
    for (BlockId id : unique_block_ids(target.block_ids)) arena.release_block(id);
    target.block_ids.clear();
    target.logical_activation_count = 0;
}

void StateTable::reset_all(StateArena &arena) {
    std::vector<BlockId> all;
    for (const auto &item : entries_) all.insert(all.end(), item.second.block_ids.begin(), item.second.block_ids.end());
    for (BlockId id : unique_block_ids(all)) arena.release_block(id);
    for (auto &item : entries_) {
        item.second.block_ids.clear();
        item.second.logical_activation_count = 0;
    }
}

StateTable StateTable::fork(StateArena &arena, std::string new_stream_id) const {
    if (new_stream_id.empty()) fail("forked transient state table stream id must not be empty");
    std::vector<BlockId> all;
    for (const auto &item : entries_) all.insert(all.end(), item.second.block_ids.begin(), item.second.block_ids.end());
    for (BlockId id : unique_block_ids(all)) arena.retain_block(id);
    StateTable forked(std::move(new_stream_id));
    forked.entries_ = entries_;
    return forked;
}

void StateTable::share_states_from(StateArena &arena, const StateTable &source, const std::vector<StateKey> &keys) {
    // everything is checked before a single block is retained (stream_state.rs:507-548)
    std::vector<std::pair<StateKey, Entry>> shares;
    for (const StateKey &key : keys) {
        const Entry &source_entry = source.entry(key);
        auto existing = entries_.find(key);
        if (existing != entries_.end()) {
            if (existing->second.shape != source_entry.shape)
                fail("cannot share transient state " + key_name(key) + " into a table with a different shape");
            if (!existing->second.block_ids.empty() || existing->second.logical_activation_count != 0)
                fail("cannot replace non-empty transient state " + key_name(key) + " with shared blocks");
        }
        shares.emplace_back(key, source_entry);
    }
    std::vector<BlockId> all;
    for (const auto &share : shares) all.insert(all.end(), share.second.block_ids.begin(), share.second.block_ids.end());
    for (BlockId id : unique_block_ids(all)) arena.retain_block(id);
    for (auto &share : shares) entries_[share.first] = std::move(share.second);
}

TableSnapshot StateTable::snapshot() const {
    TableSnapshot snapshot;
    snapshot.stream_id = stream_id_;
    snapshot.entry_count = entries_.size();
    for (const auto &item : entries_) {
        snapshot.entries.push_back(EntrySnapshot{item.first, item.second.shape, item.second.logical_activation_count, item.second.block_ids});
        snapshot.logical_activation_count += item.second.logical_activation_count;
        snapshot.block_count += item.second.block_ids.size();
    }
    return snapshot;
}

std::vector<StateKey> StateTable::state_keys() const {
    std::vector<StateKey> keys;
    for (const auto &item : entries_) keys.push_back(item.first);
    return keys;
}

std::optional<size_t> StateTable::next_append_block_boundary_distance(size_t maximum_distance) const {
    if (maximum_distance == 0) return std::nullopt;
    const Entry *first = nullptr;
    size_t alignment = 1;
    for (const auto &item : entries_) {
        if (item.second.shape.retention != Retention::Append) continue;
        if (first == nullptr) first = &item.second;
        else if (item.second.logical_activation_count != first->logical_activation_count)
            fail("append-state activation depths diverged within one stream");
        alignment = least_common_multiple(alignment, item.second.shape.activation_capacity);
    }
    if (first == nullptr) return std::nullopt;
    const size_t remainder = first->logical_activation_count % alignment;
    const size_t distance = remainder == 0 ? alignment : alignment - remainder;
    if (distance <= maximum_distance) return distance;
    return std::nullopt;
}

// ---------------------------------------------------------------------------------------------- prefix cache

namespace {

constexpr uint64_t FNV64_OFFSET = 0xcbf29ce484222325ull, FNV64_PRIME = 0x100000001b3ull;

uint64_t fnv_bytes(uint64_t hash, const uint8_t *bytes, size_t count) {
    for (size_t i = 0; i < count; i++) hash = (hash ^ bytes[i]) * FNV64_PRIME;
    return hash;
}
uint64_t fnv_text(uint64_t hash, const char *text) { return fnv_bytes(hash, reinterpret_cast<const uint8_t *>(text), std::char_traits<char>::length(text)); }
uint64_t fnv_u64(uint64_t hash, uint64_t value) {
    uint8_t bytes[8];
    for (int i = 0; i < 8; i++) bytes[i] = static_cast<uint8_t>(value >> (8 * i));
    return fnv_bytes(hash, bytes, 8);
}

}  // namespace

uint64_t stable_token_prefix_hash(const uint32_t *token_ids, size_t count) {
    uint64_t hash = fnv_u64(fnv_text(FNV64_OFFSET, "nerve:token-prefix:v1"), count);
    for (size_t i = 0; i < count; i++) {
        const uint32_t token = token_ids[i];
        const uint8_t bytes[4] = {static_cast<uint8_t>(token), static_cast<uint8_t>(token >> 8), static_cast<uint8_t>(token >> 16), static_cast<uint8_t>(token >> 24)};
        hash = fnv_bytes(hash, bytes, 4);
    }
    return hash;
}

uint64_t stable_runtime_modifier_hash(const uint8_t *bytes, size_t count) {
    return fnv_bytes(fnv_u64(fnv_text(FNV64_OFFSET, "nerve:runtime-modifiers:v1"), count), bytes, count);
}

void check_prefix_lookup_ids(const std::string &execution_class_id, const std::string &runtime_graph_id) {
    if (execution_class_id.empty()) fail("prefix cache execution class id must not be empty");
    if (runtime_graph_id.empty()) fail("prefix cache runtime graph id must not be empty");
}

std::vector<StateKey> normalized_state_keys(std::vector<StateKey> state_keys) {
    std::sort(state_keys.begin(), state_keys.end());
    state_keys.erase(std::unique(state_keys.begin(), state_keys.end()), state_keys.end());
    return state_keys;
}

PrefixStateCacheKey PrefixStateCacheKey::from_token_prefix(const std::string &execution_class_id, const std::string &runtime_graph_id,
                                                           const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                           std::vector<StateKey> state_keys) {
    check_prefix_lookup_ids(execution_class_id, runtime_graph_id);
    if (token_ids.empty()) fail("prefix cache token prefix must not be empty");
    PrefixStateCacheKey key;
    key.state_keys = normalized_state_keys(std::move(state_keys));
    if (key.state_keys.empty()) fail("prefix cache state key set must not be empty");
    key.execution_class_id = execution_class_id;
    key.runtime_graph_id = runtime_graph_id;
    key.token_count = token_ids.size();
    key.token_ids = token_ids;
    key.token_hash = stable_token_prefix_hash(token_ids.data(), token_ids.size());
    key.runtime_modifier_hash = stable_runtime_modifier_hash(reinterpret_cast<const uint8_t *>(runtime_modifier_bytes.data()), runtime_modifier_bytes.size());
    return key;
}

bool PrefixStateCacheKey::operator<(const PrefixStateCacheKey &other) const {
    return std::tie(execution_class_id, runtime_graph_id, token_count, token_ids, token_hash, runtime_modifier_hash, state_keys) <
           std::tie(other.execution_class_id, other.runtime_graph_id, other.token_count, other.token_ids, other.token_hash, other.runtime_modifier_hash,
                    other.state_keys);
}
bool PrefixStateCacheKey::operator==(const PrefixStateCacheKey &other) const { return !(*this < other) && !(other < *this); }

std::vector<PrefixStateCacheKey> PrefixStateCache::release(StateArena &arena, PrefixCacheIndex<Retained>::Removed removed) {
    std::vector<PrefixStateCacheKey> keys;
    for (auto &item : removed) {
        item.second.table.reset_all(arena);
        keys.push_back(std::move(item.first));
    }
    return keys;
}

std::vector<PrefixStateCacheKey> PrefixStateCache::set_capacity(StateArena &arena, size_t capacity_entries) {
    return release(arena, index_.set_capacity(capacity_entries));
}

bool PrefixStateCache::evict(StateArena &arena, const PrefixStateCacheKey &key) {
    std::optional<Retained> removed = index_.evict(key);
    if (!removed) return false;
    removed->table.reset_all(arena);
    return true;
}

PrefixStateCacheInsert PrefixStateCache::insert(StateArena &arena, const PrefixStateCacheKey &key, const StateTable &source) {
    PrefixStateCacheInsert result;
    if (index_.capacity_entries() == 0) return result;
    const TableSnapshot state = source.snapshot();
    for (const StateKey &state_key : key.state_keys) {
        const auto entry = std::find_if(state.entries.begin(), state.entries.end(), [&](const EntrySnapshot &e) { return e.key == state_key; });
        if (entry == state.entries.end()) fail("prefix cache source stream " + quoted(state.stream_id) + " has no state " + key_name(state_key));
        if (entry->shape.retention == Retention::Append) {
            if (entry->logical_activation_count != key.token_count)
                fail("prefix cache key for " + std::to_string(key.token_count) + " tokens does not match source state " + key_name(state_key) + " with " +
                     std::to_string(entry->logical_activation_count) + " activations");
            if (entry->logical_activation_count % entry->shape.activation_capacity != 0)
                fail("prefix cache source state " + key_name(state_key) + " has " + std::to_string(entry->logical_activation_count) +
                     " activations, which is not aligned to block capacity " + std::to_string(entry->shape.activation_capacity));
        } else if (entry->logical_activation_count != 1 || entry->block_ids.size() != 1) {
            fail("prefix cache source mutable state " + key_name(state_key) + " is not initialized");
        }
    }
    std::string cached_stream_id = index_.next_cached_stream_id();
    StateTable retained = source.fork(arena, cached_stream_id);
    auto inserted = index_.insert(key, Retained{std::move(cached_stream_id), std::move(retained)});
    if (inserted.replaced) {
        inserted.replaced->table.reset_all(arena);
        result.replaced_existing = true;
    }
    result.evicted_keys = release(arena, std::move(inserted.evicted));
    return result;
}

bool PrefixStateCache::restore_into(StateArena &arena, const PrefixStateCacheKey &key, StateTable &target) {
    Retained *retained = index_.use(key);
    if (retained == nullptr) return false;
    target.share_states_from(arena, retained->table, key.state_keys);
    return true;
}

PrefixStateCacheSnapshot PrefixStateCache::snapshot() const {
    PrefixStateCacheSnapshot snapshot;
    snapshot.capacity_entries = index_.capacity_entries();
    snapshot.entry_count = index_.entries().size();
    snapshot.eviction_count = index_.eviction_count();
    for (const auto &item : index_.entries()) {
        const TableSnapshot state = item.second.payload.table.snapshot();
        snapshot.entries.push_back(PrefixStateCacheEntrySnapshot{item.first, item.second.payload.cached_stream_id, state.block_count, state.logical_activation_count,
                                                                 item.second.last_used_tick, item.second.use_count});
    }
    return snapshot;
}

// ---------------------------------------------------------------------------------------------- scheduler

StreamScheduler::Stream::Stream(std::string id, std::string execution_class, StateTable state_table)
    : stream_id(std::move(id)), execution_class_id(std::move(execution_class)), table(std::move(state_table)) {
    if (stream_id.empty()) fail("stream id must not be empty");
    if (execution_class_id.empty()) fail("stream execution class id must not be empty");
    if (table.stream_id() != stream_id)
        fail("transient state table stream id " + quoted(table.stream_id()) + " does not match runtime stream id " + quoted(stream_id));
}

bool StreamScheduler::Stream::has_schedulable_waiting_work() const {
    return !current_event.has_value() && !queued_input_events.empty() && !has_in_flight_work() && status != StreamStatus::Closing &&
           status != StreamStatus::Interrupted;
}

void StreamScheduler::Stream::refresh_status() {
    if (status == StreamStatus::Interrupted) return;  // sticky: only a new stream state clears it
    if (closing_after_current) status = StreamStatus::Closing;
    else if (has_pending_work()) status = StreamStatus::Active;
    else status = StreamStatus::Idle;
}

StreamSnapshot StreamScheduler::Stream::snapshot() const {
    const TableSnapshot state = table.snapshot();
    StreamSnapshot snapshot;
    snapshot.stream_id = stream_id;
    snapshot.execution_class_id = execution_class_id;
    snapshot.status = status;
    snapshot.queued_input_event_count = queued_input_events.size();
    if (current_event) snapshot.current_input_event_id = current_event->event.id;
    snapshot.in_flight_activation_count = in_flight_activation_ids.size();
    snapshot.completed_input_event_count = completed_input_event_count;
    snapshot.scheduled_activation_count = scheduled_activation_count;
    snapshot.generated_token_count = generated_token_count;
    snapshot.transient_state_entry_count = state.entry_count;
    snapshot.transient_state_block_count = state.block_count;
    snapshot.transient_state_logical_activation_count = state.logical_activation_count;
    return snapshot;
}

StreamScheduler::Stream &StreamScheduler::stream(const std::string &stream_id) {
    auto found = streams_.find(stream_id);
    if (found == streams_.end()) fail("unknown stream " + quoted(stream_id));
    return found->second;
}
const StreamScheduler::Stream &StreamScheduler::stream(const std::string &stream_id) const {
    auto found = streams_.find(stream_id);
    if (found == streams_.end()) fail("unknown stream " + quoted(stream_id));
    return found->second;
}

StreamSnapshot StreamScheduler::add_stream(const std::string &stream_id, const std::string &execution_class_id,
                                           const Declarations &state_declarations) {
    if (stream_id.empty()) fail("stream id must not be empty");
    if (execution_class_id.empty()) fail("stream execution class id must not be empty");
    if (streams_.count(stream_id)) fail("stream " + quoted(stream_id) + " already exists");
    Stream fresh(stream_id, execution_class_id, StateTable(stream_id));
    for (const auto &declaration : state_declarations) fresh.table.declare_state(declaration.first, declaration.second);
    const StreamSnapshot snapshot = fresh.snapshot();  // the stream is registered only when every declaration was accepted
    streams_.emplace(stream_id, std::move(fresh));
    return snapshot;
}

StreamSnapshot StreamScheduler::declare_stream_state(const std::string &stream_id, const StateKey &key, const BlockShape &shape) {
    Stream &target = stream(stream_id);
    target.table.declare_state(key, shape);
    return target.snapshot();
}

TableSnapshot StreamScheduler::stream_transient_state_snapshot(const std::string &stream_id) const { return stream(stream_id).table.snapshot(); }

StreamSnapshot StreamScheduler::fork_stream_transient_state(const std::string &source_stream_id, const std::string &target_stream_id,
                                                            const std::string &execution_class_id) {
    // all checks come before any block is retained (stream_runtime.rs:563-597)
    if (target_stream_id.empty()) fail("forked stream id must not be empty");
    if (execution_class_id.empty()) fail("forked stream execution class id must not be empty");
    if (streams_.count(target_stream_id)) fail("stream " + quoted(target_stream_id) + " already exists");
    const Stream &source = stream(source_stream_id);
    Stream forked(target_stream_id, execution_class_id, source.table.fork(arena_, target_stream_id));
    const StreamSnapshot snapshot = forked.snapshot();
    streams_.emplace(target_stream_id, std::move(forked));
    return snapshot;
}

StreamSnapshot StreamScheduler::share_stream_state(const std::string &target_stream_id, const std::string &source_stream_id, const StateKey &key) {
    const StateTable source_table = stream(source_stream_id).table;
    Stream &target = stream(target_stream_id);
    target.table.share_states_from(arena_, source_table, {key});
    return target.snapshot();
}

PrefixStateCacheInsert StreamScheduler::cache_stream_prefix_state(const std::string &stream_id, const PrefixStateCacheKey &key) {
    const Stream &source = stream(stream_id);
    if (source.execution_class_id != key.execution_class_id)
        fail("cannot cache stream " + quoted(stream_id) + " with execution class " + quoted(source.execution_class_id) + " under prefix key execution class " +
             quoted(key.execution_class_id));
    return prefix_cache_.insert(arena_, key, source.table);
}

PrefixStateCacheKey StreamScheduler::cache_stream_prefix_state_for_tokens(const std::string &stream_id, const std::string &runtime_graph_id,
                                                                          const std::vector<uint32_t> &token_ids, const std::string &runtime_modifier_bytes,
                                                                          std::vector<StateKey> state_keys) {
    PrefixStateCacheKey key =
        PrefixStateCacheKey::from_token_prefix(stream(stream_id).execution_class_id, runtime_graph_id, token_ids, runtime_modifier_bytes, std::move(state_keys));
    cache_stream_prefix_state(stream_id, key);
    return key;
}

bool StreamScheduler::restore_stream_prefix_state(const std::string &target_stream_id, const PrefixStateCacheKey &key) {
    Stream &target = stream(target_stream_id);
    if (target.execution_class_id != key.execution_class_id)
        fail("cannot restore prefix key execution class " + quoted(key.execution_class_id) + " into stream " + quoted(target_stream_id) +
             " with execution class " + quoted(target.execution_class_id));
    return prefix_cache_.restore_into(arena_, key, target.table);
}

std::optional<PrefixStateCacheKey> StreamScheduler::restore_longest_stream_prefix_state(const std::string &target_stream_id, const std::string &runtime_graph_id,
                                                                                        const std::vector<uint32_t> &token_ids,
                                                                                        const std::string &runtime_modifier_bytes,
                                                                                        std::vector<StateKey> state_keys) {
    std::optional<PrefixStateCacheKey> key =
        prefix_cache_.longest_matching_key(stream(target_stream_id).execution_class_id, runtime_graph_id, token_ids, runtime_modifier_bytes, std::move(state_keys));
    if (key) restore_stream_prefix_state(target_stream_id, *key);
    return key;
}

StreamSnapshot StreamScheduler::enqueue_input_event(const std::string &stream_id, const InputEvent &event) {
    if (event.id.empty()) fail("input event id must not be empty");
    if (event.token_ids.empty()) fail("input event " + event.id + " has no tokens");
    Stream &target = stream(stream_id);
    if (target.status == StreamStatus::Closing) fail("stream " + quoted(stream_id) + " is closing");
    if (target.status == StreamStatus::Interrupted) fail("stream " + quoted(stream_id) + " is interrupted");
    target.queued_input_events.push_back(event);
    target.refresh_status();
    const StreamSnapshot snapshot = target.snapshot();
    activate_stream(stream_id);
    return snapshot;
}

StreamSnapshot StreamScheduler::interrupt_stream(const std::string &stream_id, const std::string &reason) {
    if (reason.empty()) fail("interrupt reason must not be empty");
    Stream &target = stream(stream_id);
    target.queued_input_events.clear();
    target.current_event.reset();
    std::vector<Activation> in_flight;
    for (uint64_t id : target.in_flight_activation_ids) {
        auto found = in_flight_.find(id);
        if (found != in_flight_.end()) in_flight.push_back(found->second);
    }
    for (const Activation &activation : in_flight) rollback_unused_activation_state(activation, 0);  // nothing of them counts as executed
    for (const Activation &activation : in_flight) in_flight_.erase(activation.id);
    target.in_flight_activation_ids.clear();
    target.status = StreamStatus::Interrupted;
    active_queue_.erase(std::remove(active_queue_.begin(), active_queue_.end(), stream_id), active_queue_.end());
    return target.snapshot();
}

StreamSnapshot StreamScheduler::reset_stream_transient_state(const std::string &stream_id) {
    Stream &target = stream(stream_id);
    if (target.has_in_flight_work()) fail("cannot reset transient state for stream " + quoted(stream_id) + " while activations are in flight");
    target.table.reset_all(arena_);
    return target.snapshot();
}

StreamSnapshot StreamScheduler::remove_stream(const std::string &stream_id) {
    Stream &target = stream(stream_id);
    if (target.has_in_flight_work()) fail("cannot remove stream " + quoted(stream_id) + " while activations are in flight");
    target.table.reset_all(arena_);
    const StreamSnapshot snapshot = target.snapshot();
    streams_.erase(stream_id);
    active_queue_.erase(std::remove(active_queue_.begin(), active_queue_.end(), stream_id), active_queue_.end());
    return snapshot;
}

StreamSnapshot StreamScheduler::close_stream_after_current(const std::string &stream_id) {
    Stream &target = stream(stream_id);
    target.closing_after_current = true;
    target.queued_input_events.clear();
    target.refresh_status();
    if (target.has_pending_work()) activate_stream(stream_id);
    return target.snapshot();
}

SchedulerStep StreamScheduler::schedule_step(const SchedulerBudget &budget) {
    SchedulerStep step;
    if (budget.max_activations == 0 || budget.max_work_units == 0) {
        step.exhausted_activation_budget = budget.max_activations == 0;
        step.exhausted_work_budget = budget.max_work_units == 0;
        step.idle = active_stream_count() == 0;
        return step;
    }
    if (budget.max_prefill_tokens_per_activation == 0) fail("max_prefill_tokens_per_activation must be positive");
    if (budget.max_decode_tokens_per_activation == 0) fail("max_decode_tokens_per_activation must be positive");
    refresh_active_queue();
    size_t consumed = 0;
    while (step.activations.size() < budget.max_activations && consumed < budget.max_work_units) {
        const std::optional<std::string> next = next_schedulable_stream_id();
        if (!next) break;
        const size_t remaining = budget.max_work_units - consumed;
        std::optional<Activation> activation = prepare_activation(*next, std::min(budget.max_prefill_tokens_per_activation, remaining),
                                                                  std::min(budget.max_decode_tokens_per_activation, remaining));
        if (!activation) continue;
        const size_t units = activation->work_units();
        consumed = consumed > std::numeric_limits<size_t>::max() - units ? std::numeric_limits<size_t>::max() : consumed + units;
        step.activations.push_back(std::move(*activation));
    }
    step.exhausted_activation_budget = step.activations.size() == budget.max_activations;
    step.exhausted_work_budget = consumed == budget.max_work_units;
    step.idle = active_stream_count() == 0 && step.activations.empty();
    return step;
}

std::vector<ActivationBatch> group_compatible_stream_activations(std::vector<Activation> activations) {
    std::vector<ActivationBatch> batches;
    for (Activation &activation : activations) {
        const BatchKind kind{activation.kind, activation.execution_class_id, activation.work_units()};
        auto found = std::find_if(batches.begin(), batches.end(), [&](const ActivationBatch &batch) { return batch.kind == kind; });
        if (found == batches.end()) {
            batches.push_back(ActivationBatch{kind, {}});
            found = batches.end() - 1;
        }
        found->activations.push_back(std::move(activation));
    }
    return batches;
}

SchedulerBatchStep StreamScheduler::schedule_batch_step(const SchedulerBudget &budget) {
    SchedulerStep step = schedule_step(budget);
    SchedulerBatchStep batched;
    batched.batches = group_compatible_stream_activations(std::move(step.activations));
    batched.exhausted_activation_budget = step.exhausted_activation_budget;
    batched.exhausted_work_budget = step.exhausted_work_budget;
    batched.idle = step.idle;
    return batched;
}

void StreamScheduler::rollback_unused_activation_state(const Activation &activation, size_t processed_state_activation_count) {
    Stream &target = stream(activation.stream_id);
    for (const StateReservation &reservation : activation.state_reservations) {
        const size_t committed = std::min(processed_state_activation_count, reservation.slots.size());
        target.table.rollback_slots(arena_, reservation.key, reservation.slots.data() + committed, reservation.slots.size() - committed);
    }
}

StreamSnapshot StreamScheduler::complete_activation(uint64_t activation_id, const ActivationOutcome &outcome) {
    auto in_flight = in_flight_.find(activation_id);
    if (in_flight == in_flight_.end()) fail("unknown in-flight activation " + std::to_string(activation_id));
    const Activation activation = in_flight->second;
    const size_t processed = outcome.processed_state_activation_count.value_or(activation.work_units());
    if (processed > activation.max_state_activation_count)
        fail("activation " + std::to_string(activation_id) + " processed " + std::to_string(processed) +
             " state activations, exceeding its reservation of " + std::to_string(activation.max_state_activation_count));
    rollback_unused_activation_state(activation, processed);
    in_flight_.erase(activation_id);
    Stream &target = stream(activation.stream_id);
    auto &ids = target.in_flight_activation_ids;
    ids.erase(std::remove(ids.begin(), ids.end(), activation_id), ids.end());
    if (!target.current_event)
        fail("stream " + quoted(activation.stream_id) + " has no current event for activation " + std::to_string(activation_id));
    CurrentEvent &current = *target.current_event;
    const size_t generated = outcome.generated_token_ids.size();
    const char *label = activation.kind == ActivationKind::PrefillChunk ? "prefill" : "decode";

    if (activation.kind == ActivationKind::PrefillChunk) {
        current.next_prompt_token_index = checked_add(current.next_prompt_token_index, activation.token_ids.size(), "prompt token index");
        if (generated != 0 && !current.prompt_done())
            fail("prefill activation " + std::to_string(activation_id) + " emitted public tokens before the prompt was complete");
    } else {
        if (generated == 0) fail("decode activation " + std::to_string(activation_id) + " completed without generated tokens");
        if (generated > activation.max_tokens)
            fail("decode activation " + std::to_string(activation_id) + " generated " + std::to_string(generated) +
                 " tokens, exceeding its window of " + std::to_string(activation.max_tokens));
    }
    if (generated != 0) {
        const size_t event_total = checked_add(current.generated_token_count, generated, "generated token count");
        if (event_total > current.event.max_public_tokens)
            fail(std::string(label) + " activation " + std::to_string(activation_id) + " exceeded input event public output budget");
        const size_t depth = checked_add(current.next_feedback_depth, generated, "feedback depth");
        target.generated_token_count = checked_add(target.generated_token_count, generated, "total generated token count");
        current.generated_token_count = event_total;
        current.next_feedback_depth = depth;
    }
    if (!outcome.continue_generation) current.generated_token_count = current.event.max_public_tokens;  // the event's budget counts as spent

    if (current.prompt_done() && current.generation_done()) {
        target.current_event.reset();
        target.completed_input_event_count++;
        if (target.closing_after_current) {
            target.closing_after_current = false;
            target.status = StreamStatus::Idle;
        }
    }
    target.refresh_status();
    const StreamSnapshot snapshot = target.snapshot();
    if (target.has_schedulable_running_work() || target.has_schedulable_waiting_work()) activate_stream(activation.stream_id);
    return snapshot;
}

std::optional<Activation> StreamScheduler::prepare_activation(const std::string &stream_id, size_t max_prefill_tokens, size_t max_decode_tokens) {
    // the id is taken even if the stream turns out to have nothing to run (stream_runtime.rs:1221-1225)
    const uint64_t activation_id = next_activation_id_;
    if (next_activation_id_ == std::numeric_limits<uint64_t>::max()) fail("activation id overflow");
    next_activation_id_++;

    Stream &target = stream(stream_id);
    if (target.has_in_flight_work()) return std::nullopt;
    if (!target.current_event) {
        if (target.queued_input_events.empty()) {
            target.refresh_status();
            return std::nullopt;
        }
        CurrentEvent fresh;
        fresh.event = std::move(target.queued_input_events.front());
        target.queued_input_events.pop_front();
        target.current_event = std::move(fresh);
    }
    const CurrentEvent &current = *target.current_event;
    Activation activation;
    activation.id = activation_id;
    activation.stream_id = stream_id;
    activation.execution_class_id = target.execution_class_id;
    activation.input_event_id = current.event.id;
    bool can_close_feedback_loop = true;
    if (!current.prompt_done()) {
        const size_t offset = current.next_prompt_token_index;
        const size_t remaining = current.event.token_ids.size() - offset;
        const size_t maximum_chunk = std::min(max_prefill_tokens, remaining);
        // a chunk ends at the next page boundary of the stream's append states when that is nearer
        const size_t chunk = target.table.next_append_block_boundary_distance(maximum_chunk).value_or(maximum_chunk);
        activation.kind = ActivationKind::PrefillChunk;
        activation.token_offset = offset;
        activation.token_ids.assign(current.event.token_ids.begin() + offset, current.event.token_ids.begin() + offset + chunk);
        activation.remaining_prompt_token_count = remaining - chunk;
        // the chunk that ends the prompt may also run the first feedback tick
        can_close_feedback_loop = offset + chunk == current.event.token_ids.size() && current.generated_token_count < current.event.max_public_tokens;
    } else if (!current.generation_done()) {
        activation.kind = ActivationKind::DecodeFeedback;
        activation.feedback_depth = current.next_feedback_depth;
        activation.max_tokens = std::min(max_decode_tokens, current.event.max_public_tokens - current.generated_token_count);
    } else {
        return std::nullopt;
    }
    activation.max_state_activation_count = checked_add(activation.work_units(), can_close_feedback_loop ? 1 : 0, "activation state reservation width");
    const std::vector<StateKey> keys = target.table.state_keys();
    if (!keys.empty() && activation.max_state_activation_count != 0)
        for (const StateKey &key : keys)
            activation.state_reservations.push_back(StateReservation{key, target.table.append_activations(arena_, key, activation.max_state_activation_count)});
    target.in_flight_activation_ids.push_back(activation_id);
    target.scheduled_activation_count++;
    target.refresh_status();
    in_flight_.emplace(activation_id, activation);
    return activation;
}

std::optional<std::string> StreamScheduler::next_schedulable_stream_id() {
    refresh_active_queue();
    // streams in the middle of an event come before streams whose next event has not started
    for (int pass = 0; pass < 2; pass++)
        for (auto position = active_queue_.begin(); position != active_queue_.end(); ++position) {
            auto found = streams_.find(*position);
            if (found == streams_.end()) continue;
            const bool eligible = pass == 0 ? found->second.has_schedulable_running_work() : found->second.has_schedulable_waiting_work();
            if (eligible) {
                std::string id = *position;
                active_queue_.erase(position);
                return id;
            }
        }
    return std::nullopt;
}

void StreamScheduler::refresh_active_queue() {
    std::vector<std::string> active;
    for (auto &item : streams_) {
        item.second.refresh_status();
        if (item.second.has_schedulable_running_work() || item.second.has_schedulable_waiting_work()) active.push_back(item.first);
    }
    active_queue_.erase(std::remove_if(active_queue_.begin(), active_queue_.end(),
                                       [&](const std::string &id) { return std::find(active.begin(), active.end(), id) == active.end(); }),
                        active_queue_.end());
    for (const std::string &id : active) activate_stream(id);
}

void StreamScheduler::activate_stream(const std::string &stream_id) {
    if (std::find(active_queue_.begin(), active_queue_.end(), stream_id) == active_queue_.end()) active_queue_.push_back(stream_id);
}

size_t StreamScheduler::active_stream_count() const {
    size_t count = 0;
    for (const auto &item : streams_) count += item.second.status == StreamStatus::Active ? 1 : 0;
    return count;
}

SchedulerSnapshot StreamScheduler::snapshot() const {
    SchedulerSnapshot snapshot;
    snapshot.stream_count = streams_.size();
    snapshot.active_stream_count = active_stream_count();
    snapshot.in_flight_activation_count = in_flight_.size();
    snapshot.transient_state_arena = arena_.snapshot();
    for (const auto &item : streams_) snapshot.streams.push_back(item.second.snapshot());
    return snapshot;
}

SchedulerRun StreamScheduler::run_until_idle_with(const SchedulerBudget &budget, size_t max_steps,
                                                  const std::function<ActivationOutcome(const Activation &)> &execute) {
    SchedulerRun run;
    run.max_steps = max_steps;
    while (run.scheduled_steps < max_steps) {
        SchedulerStep step = schedule_step(budget);
        if (step.activations.empty() && step.idle) {
            run.stop_condition = RunStop::Idle;
            run.final_snapshot = snapshot();
            return run;
        }
        if (step.activations.empty()) break;
        run.scheduled_steps++;
        for (Activation &activation : step.activations) {
            ActivationOutcome outcome = execute(activation);
            complete_activation(activation.id, outcome);
            run.completed_activations.push_back(CompletedActivation{std::move(activation), std::move(outcome)});
        }
    }
    run.final_snapshot = snapshot();
    run.stop_condition = run.final_snapshot.active_stream_count == 0 && run.final_snapshot.in_flight_activation_count == 0 ? RunStop::Idle : RunStop::StepBudget;
    return run;
}

SchedulerRun StreamScheduler::run_batches_until_idle_with(const SchedulerBudget &budget, size_t max_steps,
                                                          const std::function<std::vector<BatchActivationOutcome>(const ActivationBatch &)> &execute) {
    SchedulerRun run;
    run.max_steps = max_steps;
    while (run.scheduled_steps < max_steps) {
        SchedulerBatchStep step = schedule_batch_step(budget);
        if (step.batches.empty() && step.idle) {
            run.stop_condition = RunStop::Idle;
            run.final_snapshot = snapshot();
            return run;
        }
        if (step.batches.empty()) break;
        run.scheduled_steps++;
        for (ActivationBatch &batch : step.batches) {
            std::vector<BatchActivationOutcome> outcomes = execute(batch);
            for (Activation &activation : batch.activations) {
                auto found = std::find_if(outcomes.begin(), outcomes.end(),
                                          [&](const BatchActivationOutcome &candidate) { return candidate.activation_id == activation.id; });
                if (found == outcomes.end()) fail("batch executor did not return an outcome for activation " + std::to_string(activation.id));
                ActivationOutcome outcome = std::move(found->outcome);
                outcomes.erase(found);
                complete_activation(activation.id, outcome);
                run.completed_activations.push_back(CompletedActivation{std::move(activation), std::move(outcome)});
            }
            if (!outcomes.empty()) fail("batch executor returned outcomes for unknown activations");
        }
    }
    run.final_snapshot = snapshot();
    run.stop_condition = run.final_snapshot.active_stream_count == 0 && run.final_snapshot.in_flight_activation_count == 0 ? RunStop::Idle : RunStop::StepBudget;
    return run;
}

}  // namespace runtime
}  // namespace nerve
