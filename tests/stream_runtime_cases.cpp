// Behavioural cases for llmoop_b200/csrc/stream_runtime.cpp, one per scenario the reference's own unit tests pin:
//   runtime-rs/src/stream_state.rs:761-985           (arena and state tables)
//   runtime-rs/src/stream_runtime_tests.rs:16-1337   (scheduler, its prefix-cache hooks :518-769 included)
//   runtime-rs/src/stream_prefix_cache.rs:406-583     (prefix-state cache)
// Same inputs, same expected values, written against the C++ API.  Usage: stream_runtime_cases [case name]; prints
// "ok <name>" or "FAIL <name>: <what>" per case and exits with the number of failures.
#include <cstdio>
#include <cstring>
#include <functional>
#include <set>
#include <string>
#include <vector>

#include "../llmoop_b200/csrc/stream_runtime.hpp"

using namespace nerve::runtime;

namespace {

struct CaseFailure {
    std::string what;
};

#define CHECK(condition)                                                                             \
    do {                                                                                             \
        if (!(condition)) throw CaseFailure{std::string(#condition) + " (line " + std::to_string(__LINE__) + ")"}; \
    } while (0)

template <typename F>
std::string error_of(F &&call) {
    try {
        call();
    } catch (const RuntimeError &error) {
        return error.what();
    }
    throw CaseFailure{"expected an error"};
}

BlockShape shape4() { return BlockShape::append(16, 4); }
StateKey kv_key() { return StateKey{"layer_00", "kv"}; }

// scheduler helpers (stream_runtime_tests.rs:4-14)
SchedulerBudget budget(size_t max_activations) { return SchedulerBudget(max_activations, 2, 16); }
StateKey state_key() { return StateKey{"layer_00", "kv_memory"}; }
BlockShape state_shape() { return BlockShape::append(16, 2); }
InputEvent event(const std::string &id, std::vector<uint32_t> tokens, size_t max_public) { return InputEvent{id, std::move(tokens), max_public}; }
Activation first_activation(StreamScheduler &scheduler, const SchedulerBudget &b) {
    SchedulerStep step = scheduler.schedule_step(b);
    CHECK(!step.activations.empty());
    return step.activations[0];
}
bool is_prefill(const Activation &a, size_t offset, std::vector<uint32_t> tokens, size_t remaining) {
    return a.kind == ActivationKind::PrefillChunk && a.token_offset == offset && a.token_ids == tokens && a.remaining_prompt_token_count == remaining;
}
bool is_decode(const Activation &a, size_t depth, size_t max_tokens) {
    return a.kind == ActivationKind::DecodeFeedback && a.feedback_depth == depth && a.max_tokens == max_tokens;
}

struct Case {
    const char *name;
    std::function<void()> run;
};

std::vector<Case> cases() {
    std::vector<Case> all;

    // ------------------------------------------------------------------ arena and tables (stream_state.rs:761-985)
    all.push_back({"state_appends_slots_across_fixed_size_blocks", [] {
        StateArena arena;
        StateTable table("stream_a");
        table.declare_state(kv_key(), shape4());
        auto slots = table.append_activations(arena, kv_key(), 6);
        CHECK(slots.size() == 6);
        CHECK(slots[0].logical_activation_index == 0 && slots[0].block_activation_offset == 0);
        CHECK(slots[3].block_activation_offset == 3);
        CHECK(slots[3].block_id != slots[4].block_id);
        CHECK(slots[4].block_activation_offset == 0);
        CHECK(table.snapshot().block_count == 2);
        CHECK(arena.snapshot().live_block_count == 2);
    }});
    all.push_back({"state_reset_releases_and_reuses_matching_blocks", [] {
        StateArena arena;
        StateTable first("stream_a");
        first.declare_state(kv_key(), shape4());
        std::set<BlockId> allocated, reused;
        for (const auto &slot : first.append_activations(arena, kv_key(), 5)) allocated.insert(slot.block_id);
        first.reset_state(arena, kv_key());
        CHECK(arena.snapshot().free_block_count == 2);
        StateTable second("stream_b");
        second.declare_state(kv_key(), shape4());
        for (const auto &slot : second.append_activations(arena, kv_key(), 5)) reused.insert(slot.block_id);
        CHECK(allocated == reused);
        CHECK(arena.snapshot().allocated_block_count == 2 && arena.snapshot().live_block_count == 2);
    }});
    all.push_back({"state_fork_shares_blocks_until_each_table_resets", [] {
        StateArena arena;
        StateTable parent("parent");
        parent.declare_state(kv_key(), shape4());
        const BlockId block = parent.append_activations(arena, kv_key(), 3)[0].block_id;
        StateTable child = parent.fork(arena, "child");
        CHECK(arena.ref_count(block) == 2);
        parent.reset_all(arena);
        CHECK(arena.ref_count(block) == 1 && arena.snapshot().free_block_count == 0);
        child.reset_all(arena);
        CHECK(arena.ref_count(block) == 0 && arena.snapshot().free_block_count == 1);
    }});
    all.push_back({"state_fork_copies_a_shared_partial_append_block_before_writing", [] {
        StateArena arena;
        StateTable parent("parent");
        parent.declare_state(kv_key(), shape4());
        const BlockId shared = parent.append_activations(arena, kv_key(), 3)[0].block_id;
        StateTable child = parent.fork(arena, "child");
        const StateSlot slot = child.append_activations(arena, kv_key(), 1)[0];
        CHECK(slot.block_id != shared);
        CHECK(slot.copy_from_block_id && *slot.copy_from_block_id == shared);
        CHECK(slot.block_activation_offset == 3);
        CHECK(parent.snapshot().entries[0].block_ids == std::vector<BlockId>{shared});
        CHECK(arena.ref_count(shared) == 1 && arena.ref_count(slot.block_id) == 1);
    }});
    all.push_back({"bounded_append_state_reuses_its_physical_block_after_wrapping", [] {
        StateArena arena;
        StateTable table("stream");
        table.declare_state(kv_key(), shape4().with_maximum_activation_count(4));
        const BlockId first = table.append_activations(arena, kv_key(), 4)[0].block_id;
        auto wrapped = table.append_activations(arena, kv_key(), 1);
        CHECK(wrapped[0].logical_activation_index == 4 && wrapped[0].block_activation_offset == 0);
        CHECK(wrapped[0].block_id == first && !wrapped[0].copy_from_block_id);
        CHECK(table.snapshot().block_count == 1);
        CHECK(arena.snapshot().allocated_block_count == 1 && arena.snapshot().live_block_count == 1);
    }});
    all.push_back({"bounded_append_state_copies_a_shared_page_before_wrapped_write", [] {
        StateArena arena;
        StateTable parent("parent");
        parent.declare_state(kv_key(), shape4().with_maximum_activation_count(4));
        const BlockId shared = parent.append_activations(arena, kv_key(), 4)[0].block_id;
        StateTable child = parent.fork(arena, "child");
        const StateSlot wrapped = child.append_activations(arena, kv_key(), 1)[0];
        CHECK(wrapped.logical_activation_index == 4 && wrapped.block_activation_offset == 0);
        CHECK(wrapped.block_id != shared);
        CHECK(wrapped.copy_from_block_id && *wrapped.copy_from_block_id == shared);
        CHECK(parent.snapshot().entries[0].block_ids == std::vector<BlockId>{shared});
        CHECK(arena.ref_count(shared) == 1 && arena.ref_count(wrapped.block_id) == 1);
    }});
    all.push_back({"rollback_releases_unused_pages_but_keeps_committed_slots", [] {
        StateArena arena;
        StateTable table("stream");
        table.declare_state(kv_key(), shape4());
        auto slots = table.append_activations(arena, kv_key(), 6);
        table.rollback_slots(arena, kv_key(), slots.data() + 3, 3);
        const TableSnapshot state = table.snapshot();
        CHECK(state.logical_activation_count == 3 && state.block_count == 1);
        CHECK(state.entries[0].block_ids == std::vector<BlockId>{slots[0].block_id});
        CHECK(arena.snapshot().live_block_count == 1 && arena.snapshot().free_block_count == 1);
    }});
    all.push_back({"rollback_restores_a_shared_block_replaced_by_copy_on_write", [] {
        StateArena arena;
        StateTable parent("parent");
        parent.declare_state(kv_key(), shape4());
        const BlockId shared = parent.append_activations(arena, kv_key(), 3)[0].block_id;
        StateTable child = parent.fork(arena, "child");
        auto slot = child.append_activations(arena, kv_key(), 1);
        child.rollback_slots(arena, kv_key(), slot.data(), slot.size());
        CHECK(child.snapshot().logical_activation_count == 3);
        CHECK(child.snapshot().entries[0].block_ids == std::vector<BlockId>{shared});
        CHECK(arena.ref_count(shared) == 2);
        CHECK(arena.snapshot().live_block_count == 1 && arena.snapshot().free_block_count == 1);
    }});
    all.push_back({"rollback_rejects_a_reservation_that_is_not_the_latest", [] {
        StateArena arena;
        StateTable table("stream");
        table.declare_state(kv_key(), shape4());
        auto slots = table.append_activations(arena, kv_key(), 4);
        const std::string error = error_of([&] { table.rollback_slots(arena, kv_key(), slots.data(), 2); });
        CHECK(error.find("not the latest contiguous reservation") != std::string::npos);
    }});
    all.push_back({"rollback_releases_a_new_mutable_singleton_reservation", [] {
        StateArena arena;
        StateTable table("stream");
        table.declare_state(kv_key(), BlockShape::mutable_singleton(128));
        auto slot = table.append_activations(arena, kv_key(), 64);
        table.rollback_slots(arena, kv_key(), slot.data(), slot.size());
        CHECK(table.snapshot().logical_activation_count == 0 && table.snapshot().block_count == 0);
        CHECK(arena.snapshot().live_block_count == 0 && arena.snapshot().free_block_count == 1);
    }});
    all.push_back({"mutable_singleton_state_reuses_one_block_and_copies_on_forked_write", [] {
        StateArena arena;
        StateTable parent("parent");
        parent.declare_state(kv_key(), BlockShape::mutable_singleton(128));
        auto first = parent.append_activations(arena, kv_key(), 64);
        CHECK(first.size() == 1);
        const BlockId shared = first[0].block_id;
        CHECK(parent.snapshot().logical_activation_count == 1);
        StateTable child = parent.fork(arena, "child");
        const StateSlot child_slot = child.append_activations(arena, kv_key(), 64)[0];
        CHECK(child_slot.block_id != shared);
        CHECK(child_slot.copy_from_block_id && *child_slot.copy_from_block_id == shared);
        CHECK(child.snapshot().logical_activation_count == 1);
        auto next = child.append_activations(arena, kv_key(), 64);
        CHECK(next.size() == 1 && next[0].block_id == child_slot.block_id && !next[0].copy_from_block_id);
    }});
    all.push_back({"state_can_share_one_component_state_between_streams", [] {
        StateArena arena;
        StateTable source("source");
        const StateKey kv{"layer_02", "kv_memory"}, conv{"layer_02", "conv_state"};
        source.declare_state(kv, shape4());
        source.declare_state(conv, BlockShape::append(8, 2));
        const BlockId kv_block = source.append_activations(arena, kv, 1)[0].block_id;
        const BlockId conv_block = source.append_activations(arena, conv, 1)[0].block_id;
        StateTable target("target");
        target.share_states_from(arena, source, {kv});
        CHECK(target.snapshot().entry_count == 1);
        CHECK(arena.ref_count(kv_block) == 2 && arena.ref_count(conv_block) == 1);
    }});
    all.push_back({"shape_and_table_reject_empty_or_zero_arguments", [] {
        CHECK(error_of([] { BlockShape::append(0, 4); }).find("bytes_per_activation") != std::string::npos);
        CHECK(error_of([] { BlockShape::append(16, 0); }).find("activation_capacity") != std::string::npos);
        CHECK(error_of([] { shape4().with_maximum_activation_count(0); }).find("maximum activation count") != std::string::npos);
        CHECK(error_of([] { StateTable table(""); }).find("must not be empty") != std::string::npos);
        StateTable table("s");
        table.declare_state(kv_key(), shape4());
        table.declare_state(kv_key(), shape4());  // the same shape again is accepted
        CHECK(error_of([&] { table.declare_state(kv_key(), BlockShape::append(16, 8)); }).find("different block shape") != std::string::npos);
        StateArena arena;
        CHECK(error_of([&] { table.append_activations(arena, StateKey{"x", "y"}, 1); }).find("has no transient state") != std::string::npos);
        CHECK(table.append_activations(arena, kv_key(), 0).empty());
    }});
    all.push_back({"boundary_distance_is_the_common_page_boundary_of_append_states", [] {
        StateArena arena;
        StateTable table("s");
        CHECK(!table.next_append_block_boundary_distance(8));
        table.declare_state(StateKey{"a", "kv"}, BlockShape::append(16, 4));
        table.declare_state(StateKey{"b", "kv"}, BlockShape::append(16, 6));
        table.declare_state(StateKey{"c", "scratch"}, BlockShape::mutable_singleton(64));
        CHECK(!table.next_append_block_boundary_distance(0));
        CHECK(*table.next_append_block_boundary_distance(64) == 12);  // lcm(4, 6), from depth 0
        CHECK(!table.next_append_block_boundary_distance(11));
        table.append_activations(arena, StateKey{"a", "kv"}, 5);
        CHECK(error_of([&] { table.next_append_block_boundary_distance(64); }).find("diverged") != std::string::npos);
        table.append_activations(arena, StateKey{"b", "kv"}, 5);
        CHECK(*table.next_append_block_boundary_distance(64) == 7);
    }});

    // ------------------------------------------------------------------ scheduler (stream_runtime_tests.rs)
    all.push_back({"scheduler_adds_stream_with_declared_transient_state_atomically", [] {
        StreamScheduler scheduler;
        const StreamSnapshot snapshot = scheduler.add_stream("stream_a", "default", {{state_key(), state_shape()}});
        CHECK(snapshot.transient_state_entry_count == 1);
        CHECK(scheduler.stream_transient_state_snapshot("stream_a").entries[0].key == state_key());
        // a bad declaration leaves no stream behind
        CHECK(error_of([&] { scheduler.add_stream("stream_b", "default", {{StateKey{"", "kv"}, state_shape()}}); }).find("must not be empty") != std::string::npos);
        CHECK(scheduler.snapshot().stream_count == 1);
        CHECK(error_of([&] { scheduler.add_stream("stream_a"); }).find("already exists") != std::string::npos);
    }});
    all.push_back({"scheduler_chunks_prefill_before_decode_feedback", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2, 3}, 2));
        const Activation first = first_activation(scheduler, budget(1));
        CHECK(is_prefill(first, 0, {1, 2}, 1));
        scheduler.complete_activation(first.id, ActivationOutcome::prefill_complete());
        const Activation second = first_activation(scheduler, budget(1));
        CHECK(is_prefill(second, 2, {3}, 0));
        scheduler.complete_activation(second.id, ActivationOutcome::prefill_complete());
        CHECK(is_decode(first_activation(scheduler, budget(1)), 0, 1));
    }});
    all.push_back({"scheduler_prioritizes_running_streams_before_new_waiting_events", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.add_stream("stream_b");
        scheduler.enqueue_input_event("stream_a", event("event_a", {10}, 1));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        scheduler.enqueue_input_event("stream_b", event("event_b", {20}, 1));
        const Activation next = first_activation(scheduler, budget(1));
        CHECK(next.stream_id == "stream_a" && next.kind == ActivationKind::DecodeFeedback);
    }});
    all.push_back({"scheduler_prefill_chunk_lands_on_the_next_state_page_boundary", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a", "default", {{state_key(), BlockShape::append(16, 4)}});
        scheduler.enqueue_input_event("stream_a", event("first", {1, 2, 3}, 0));
        const Activation first = first_activation(scheduler, SchedulerBudget(1, 64, 64));
        scheduler.complete_activation(first.id, ActivationOutcome::prefill_complete());
        scheduler.enqueue_input_event("stream_a", event("second", {4, 5}, 0));
        const Activation boundary = first_activation(scheduler, SchedulerBudget(1, 64, 64));
        CHECK(is_prefill(boundary, 0, {4}, 1));
        CHECK(boundary.state_reservations[0].slots.size() == 1);
        CHECK(boundary.state_reservations[0].slots[0].block_activation_offset == 3);
    }});
    all.push_back({"scheduler_completes_stream_without_destroying_it", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 1));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const Activation decode = first_activation(scheduler, budget(1));
        const StreamSnapshot done = scheduler.complete_activation(decode.id, ActivationOutcome::generated({42}, true));
        CHECK(done.status == StreamStatus::Idle && done.completed_input_event_count == 1);
        CHECK(scheduler.snapshot().stream_count == 1 && scheduler.snapshot().active_stream_count == 0);
    }});
    all.push_back({"scheduler_interrupt_clears_work_and_keeps_stream_registered", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2}, 8));
        CHECK(scheduler.schedule_step(budget(1)).activations.size() == 1);
        const StreamSnapshot interrupted = scheduler.interrupt_stream("stream_a", "user requested stop");
        CHECK(interrupted.status == StreamStatus::Interrupted && interrupted.in_flight_activation_count == 0);
        CHECK(scheduler.snapshot().stream_count == 1 && scheduler.snapshot().in_flight_activation_count == 0);
        CHECK(error_of([&] { scheduler.enqueue_input_event("stream_a", event("event_1", {1}, 1)); }).find("is interrupted") != std::string::npos);
        CHECK(error_of([&] { scheduler.interrupt_stream("stream_a", ""); }).find("reason must not be empty") != std::string::npos);
    }});
    all.push_back({"scheduler_reserves_transient_state_slots_for_prefill_and_decode", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.declare_stream_state("stream_a", state_key(), state_shape());
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2, 3}, 1));
        const Activation first = first_activation(scheduler, budget(1));
        CHECK(first.work_units() == 2 && first.state_reservations.size() == 1 && first.state_reservations[0].slots.size() == 2);
        CHECK(first.state_reservations[0].slots[0].block_activation_offset == 0 && first.state_reservations[0].slots[1].block_activation_offset == 1);
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 1);
        scheduler.complete_activation(first.id, ActivationOutcome::prefill_complete());
        const Activation second = first_activation(scheduler, budget(1));  // the last chunk also reserves the first feedback tick
        CHECK(second.work_units() == 1 && second.state_reservations[0].slots.size() == 2);
        CHECK(second.state_reservations[0].slots[0].block_activation_offset == 0);
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 2);
        scheduler.complete_activation(second.id, ActivationOutcome::prefill_complete());
        const Activation decode = first_activation(scheduler, budget(1));
        CHECK(decode.kind == ActivationKind::DecodeFeedback && decode.state_reservations[0].slots.size() == 2);
        CHECK(decode.state_reservations[0].slots[0].block_activation_offset == 1);
    }});
    all.push_back({"scheduler_interrupt_rolls_back_unexecuted_reservations_and_preserves_committed_state", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.declare_stream_state("stream_a", state_key(), state_shape());
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const SchedulerStep scheduled = scheduler.schedule_step(SchedulerBudget(1, 2, 16).with_max_decode_tokens_per_activation(4));
        CHECK(scheduled.activations[0].state_reservations[0].slots.size() == 5);
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 4);
        const StreamSnapshot interrupted = scheduler.interrupt_stream("stream_a", "cancel");
        CHECK(interrupted.transient_state_block_count == 1 && interrupted.transient_state_logical_activation_count == 2);
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 1);
        scheduler.reset_stream_transient_state("stream_a");
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 0);
        CHECK(scheduler.snapshot().transient_state_arena.free_block_count == 4);
    }});
    all.push_back({"scheduler_stream_removal_reclaims_all_transient_blocks", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a", "default", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 0));
        const Activation activation = first_activation(scheduler, budget(1));
        CHECK(error_of([&] { scheduler.remove_stream("stream_a"); }).find("while activations are in flight") != std::string::npos);
        scheduler.complete_activation(activation.id, ActivationOutcome::generated({}, false));
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 1);
        scheduler.remove_stream("stream_a");
        CHECK(scheduler.snapshot().stream_count == 0);
        CHECK(scheduler.snapshot().transient_state_arena.live_block_count == 0 && scheduler.snapshot().transient_state_arena.free_block_count == 1);
    }});
    all.push_back({"scheduler_forks_stream_transient_state_without_copying_blocks", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("source", "default", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("source", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const StreamSnapshot forked = scheduler.fork_stream_transient_state("source", "child", "same_package");
        CHECK(forked.stream_id == "child" && forked.execution_class_id == "same_package" && forked.status == StreamStatus::Idle);
        CHECK(forked.queued_input_event_count == 0 && !forked.current_input_event_id);
        CHECK(forked.transient_state_entry_count == 1 && forked.transient_state_block_count == 1 && forked.transient_state_logical_activation_count == 2);
        const ArenaSnapshot arena = scheduler.transient_state_arena_snapshot();
        CHECK(arena.live_block_count == 1 && arena.blocks[0].ref_count == 2);
        scheduler.interrupt_stream("source", "discard source");
        const TableSnapshot child_state = scheduler.stream_transient_state_snapshot("child");
        CHECK(child_state.block_count == 1 && child_state.logical_activation_count == 2);
        const ArenaSnapshot after = scheduler.transient_state_arena_snapshot();
        CHECK(after.live_block_count == 1 && after.free_block_count == 1 && after.blocks[0].ref_count == 2);
    }});
    all.push_back({"scheduler_rejects_invalid_fork_before_retaining_blocks", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("source", "default", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("source", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const ArenaSnapshot before = scheduler.transient_state_arena_snapshot();
        const std::string error = error_of([&] { scheduler.fork_stream_transient_state("source", "child", ""); });
        CHECK(error.find("forked stream execution class id must not be empty") != std::string::npos);
        CHECK(scheduler.transient_state_arena_snapshot() == before);
        CHECK(scheduler.snapshot().stream_count == 1);
    }});
    all.push_back({"scheduler_shares_single_component_state_between_streams", [] {
        const StateKey kv = state_key(), conv{"layer_00", "conv_state"};
        StreamScheduler scheduler;
        scheduler.add_stream("source", "default", {{kv, state_shape()}, {conv, state_shape()}});
        scheduler.add_stream("target", "default", {{kv, state_shape()}});
        scheduler.enqueue_input_event("source", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const StreamSnapshot shared = scheduler.share_stream_state("target", "source", kv);
        CHECK(shared.stream_id == "target" && shared.status == StreamStatus::Idle);
        CHECK(shared.transient_state_entry_count == 1 && shared.transient_state_block_count == 1 && shared.transient_state_logical_activation_count == 2);
        const TableSnapshot source_state = scheduler.stream_transient_state_snapshot("source");
        const TableSnapshot target_state = scheduler.stream_transient_state_snapshot("target");
        std::vector<BlockId> source_kv, source_conv;
        for (const auto &entry : source_state.entries) (entry.key == kv ? source_kv : source_conv) = entry.block_ids;
        CHECK(target_state.entries[0].block_ids == source_kv && target_state.entries[0].block_ids != source_conv);
        const ArenaSnapshot arena = scheduler.transient_state_arena_snapshot();
        CHECK(arena.live_block_count == 2);
        for (const auto &block : arena.blocks) {
            if (block.block_id == source_kv[0]) CHECK(block.ref_count == 2);
            if (block.block_id == source_conv[0]) CHECK(block.ref_count == 1);
        }
    }});
    all.push_back({"scheduler_run_drives_executor_until_stream_is_idle", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2, 3}, 2));
        uint32_t next_token = 200;
        const SchedulerRun run = scheduler.run_until_idle_with(budget(1), 16, [&](const Activation &activation) {
            if (activation.kind == ActivationKind::PrefillChunk) return ActivationOutcome::prefill_complete();
            return ActivationOutcome::generated({next_token++}, true);
        });
        CHECK(run.stop_condition == RunStop::Idle && run.completed_activations.size() == 4);
        CHECK(run.final_snapshot.active_stream_count == 0);
        CHECK(run.final_snapshot.streams[0].completed_input_event_count == 1 && run.final_snapshot.streams[0].generated_token_count == 2);
        size_t prefills = 0;
        for (const auto &completed : run.completed_activations) prefills += completed.activation.kind == ActivationKind::PrefillChunk ? 1 : 0;
        CHECK(prefills == 2);
    }});
    all.push_back({"scheduler_batch_step_groups_compatible_decode_windows_across_streams", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.add_stream("stream_b");
        scheduler.declare_stream_state("stream_a", state_key(), state_shape());
        scheduler.declare_stream_state("stream_b", state_key(), state_shape());
        scheduler.enqueue_input_event("stream_a", event("event_a", {10}, 4));
        scheduler.enqueue_input_event("stream_b", event("event_b", {20}, 4));
        const SchedulerBatchStep prefill = scheduler.schedule_batch_step(budget(2));
        CHECK(prefill.batches.size() == 1);
        CHECK((prefill.batches[0].kind == BatchKind{ActivationKind::PrefillChunk, "default", 1}));
        for (const Activation &activation : prefill.batches[0].activations) scheduler.complete_activation(activation.id, ActivationOutcome::prefill_complete());
        const SchedulerBatchStep decode = scheduler.schedule_batch_step(SchedulerBudget(2, 2, 16).with_max_decode_tokens_per_activation(4));
        CHECK(decode.batches.size() == 1);
        CHECK((decode.batches[0].kind == BatchKind{ActivationKind::DecodeFeedback, "default", 4}));
        CHECK(decode.batches[0].activations.size() == 2);
        CHECK(decode.batches[0].activations[0].stream_id == "stream_a" && decode.batches[0].activations[1].stream_id == "stream_b");
        CHECK(decode.batches[0].activations[0].state_reservations[0].slots[0].block_id != decode.batches[0].activations[1].state_reservations[0].slots[0].block_id);
    }});
    all.push_back({"scheduler_batch_step_keeps_incompatible_prefill_shapes_separate", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.add_stream("stream_b");
        scheduler.enqueue_input_event("stream_a", event("event_a", {1, 2}, 1));
        scheduler.enqueue_input_event("stream_b", event("event_b", {3}, 1));
        const SchedulerBatchStep step = scheduler.schedule_batch_step(budget(2));
        CHECK(step.batches.size() == 2);
        CHECK((step.batches[0].kind == BatchKind{ActivationKind::PrefillChunk, "default", 2}));
        CHECK((step.batches[1].kind == BatchKind{ActivationKind::PrefillChunk, "default", 1}));
        CHECK(step.batches[0].activations.size() == 1 && step.batches[1].activations.size() == 1);
    }});
    all.push_back({"scheduler_batch_step_keeps_different_execution_classes_separate", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a", "package_a");
        scheduler.add_stream("stream_b", "package_b");
        scheduler.enqueue_input_event("stream_a", event("event_a", {1}, 1));
        scheduler.enqueue_input_event("stream_b", event("event_b", {2}, 1));
        const SchedulerBatchStep step = scheduler.schedule_batch_step(budget(2));
        CHECK(step.batches.size() == 2);
        CHECK((step.batches[0].kind == BatchKind{ActivationKind::PrefillChunk, "package_a", 1}));
        CHECK((step.batches[1].kind == BatchKind{ActivationKind::PrefillChunk, "package_b", 1}));
    }});
    all.push_back({"scheduler_batch_step_admits_waiting_prefill_alongside_running_prefill_when_capacity_exists", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("long_stream");
        scheduler.add_stream("new_stream");
        scheduler.enqueue_input_event("long_stream", event("long_event", {1, 2, 3, 4, 5}, 1));
        const SchedulerBatchStep first = scheduler.schedule_batch_step(budget(1));
        CHECK(first.batches.size() == 1 && is_prefill(first.batches[0].activations[0], 0, {1, 2}, 3));
        scheduler.complete_activation(first.batches[0].activations[0].id, ActivationOutcome::prefill_complete());
        scheduler.enqueue_input_event("new_stream", event("new_event", {9, 10}, 1));
        const SchedulerBatchStep next = scheduler.schedule_batch_step(budget(2));
        CHECK(next.batches.size() == 1);
        CHECK((next.batches[0].kind == BatchKind{ActivationKind::PrefillChunk, "default", 2}));
        const auto &scheduled = next.batches[0].activations;
        CHECK(scheduled.size() == 2);
        CHECK(scheduled[0].stream_id == "long_stream" && is_prefill(scheduled[0], 2, {3, 4}, 1) && scheduled[0].state_reservations.empty());
        CHECK(scheduled[1].stream_id == "new_stream" && is_prefill(scheduled[1], 0, {9, 10}, 0) && scheduled[1].state_reservations.empty());
    }});
    all.push_back({"scheduler_batch_run_requires_exact_outcomes_for_every_activation", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.add_stream("stream_b");
        scheduler.enqueue_input_event("stream_a", event("event_a", {1}, 1));
        scheduler.enqueue_input_event("stream_b", event("event_b", {2}, 1));
        const std::string error = error_of([&] {
            scheduler.run_batches_until_idle_with(budget(2), 1, [](const ActivationBatch &batch) {
                return std::vector<BatchActivationOutcome>{{batch.activations[0].id, ActivationOutcome::prefill_complete()}};
            });
        });
        CHECK(error.find("batch executor did not return an outcome for activation") != std::string::npos);
    }});
    all.push_back({"scheduler_batch_run_drives_multiple_streams_until_idle", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.add_stream("stream_b");
        scheduler.enqueue_input_event("stream_a", event("event_a", {1}, 2));
        scheduler.enqueue_input_event("stream_b", event("event_b", {2}, 2));
        const SchedulerRun run = scheduler.run_batches_until_idle_with(
            SchedulerBudget(2, 2, 16).with_max_decode_tokens_per_activation(2), 8, [](const ActivationBatch &batch) {
                std::vector<BatchActivationOutcome> outcomes;
                for (const Activation &activation : batch.activations) {
                    if (activation.kind == ActivationKind::PrefillChunk) outcomes.push_back({activation.id, ActivationOutcome::prefill_complete()});
                    else outcomes.push_back({activation.id, ActivationOutcome::generated({static_cast<uint32_t>(activation.id), static_cast<uint32_t>(activation.id) + 100}, false)});
                }
                return outcomes;
            });
        CHECK(run.stop_condition == RunStop::Idle && run.final_snapshot.active_stream_count == 0 && run.completed_activations.size() == 4);
        size_t generated = 0;
        for (const auto &stream : run.final_snapshot.streams) {
            CHECK(stream.completed_input_event_count == 1);
            generated += stream.generated_token_count;
        }
        CHECK(generated == 4);
    }});
    all.push_back({"scheduler_decode_activation_can_cover_a_feedback_window", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 5));
        const SchedulerBudget windowed = SchedulerBudget(1, 2, 16).with_max_decode_tokens_per_activation(4);
        const Activation prefill = first_activation(scheduler, windowed);
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const Activation decode = first_activation(scheduler, windowed);
        CHECK(is_decode(decode, 0, 4));
        const StreamSnapshot done = scheduler.complete_activation(decode.id, ActivationOutcome::generated({10, 11, 12, 13}, true));
        CHECK(done.generated_token_count == 4 && done.status == StreamStatus::Active);
        CHECK(is_decode(first_activation(scheduler, windowed), 4, 1));
    }});
    all.push_back({"scheduler_commits_only_the_feedback_ticks_that_actually_executed", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a", "default", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 5));
        const SchedulerBudget windowed = SchedulerBudget(1, 2, 16).with_max_decode_tokens_per_activation(4);
        const Activation prefill = first_activation(scheduler, windowed);
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const Activation decode = first_activation(scheduler, windowed);
        CHECK(scheduler.stream_transient_state_snapshot("stream_a").logical_activation_count == 6);
        scheduler.complete_activation(decode.id, ActivationOutcome::generated({10, 11}, false).with_processed_state_activations(2));
        const TableSnapshot state = scheduler.stream_transient_state_snapshot("stream_a");
        CHECK(state.logical_activation_count == 3 && state.block_count == 2);
        const ArenaSnapshot arena = scheduler.transient_state_arena_snapshot();
        CHECK(arena.live_block_count == 2 && arena.free_block_count == 1);
    }});
    all.push_back({"scheduler_rejects_a_processed_tick_count_larger_than_the_reservation", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a", "default", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 5));
        const Activation prefill = first_activation(scheduler, budget(1));
        const TableSnapshot reserved = scheduler.stream_transient_state_snapshot("stream_a");
        const std::string error = error_of([&] { scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete().with_processed_state_activations(3)); });
        CHECK(error.find("exceeding its reservation") != std::string::npos);
        CHECK(scheduler.stream_transient_state_snapshot("stream_a") == reserved);
        CHECK(scheduler.snapshot().in_flight_activation_count == 1);
    }});
    all.push_back({"scheduler_prefill_completion_can_emit_initial_feedback_token", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2}, 3));
        const Activation prefill = first_activation(scheduler, SchedulerBudget(1, 8, 8));
        CHECK(is_prefill(prefill, 0, {1, 2}, 0));
        const StreamSnapshot active = scheduler.complete_activation(prefill.id, ActivationOutcome::generated({99}, true));
        CHECK(active.generated_token_count == 1);
        CHECK(is_decode(first_activation(scheduler, SchedulerBudget(1, 8, 8).with_max_decode_tokens_per_activation(8)), 1, 2));
    }});
    all.push_back({"scheduler_run_preserves_in_flight_work_when_step_budget_expires", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 1));
        const SchedulerRun run = scheduler.run_until_idle_with(budget(1), 1, [](const Activation &activation) {
            return activation.kind == ActivationKind::PrefillChunk ? ActivationOutcome::prefill_complete() : ActivationOutcome::generated({42}, true);
        });
        CHECK(run.stop_condition == RunStop::StepBudget && run.completed_activations.size() == 1);
        CHECK(run.final_snapshot.active_stream_count == 1 && run.final_snapshot.streams[0].completed_input_event_count == 0);
    }});
    all.push_back({"scheduler_budget_and_outcome_rules", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        CHECK(error_of([&] { scheduler.enqueue_input_event("stream_a", event("", {1}, 1)); }).find("event id must not be empty") != std::string::npos);
        CHECK(error_of([&] { scheduler.enqueue_input_event("stream_a", event("e", {}, 1)); }).find("has no tokens") != std::string::npos);
        scheduler.enqueue_input_event("stream_a", event("event_0", {1, 2, 3}, 2));
        const SchedulerStep none = scheduler.schedule_step(SchedulerBudget(0, 2, 16));
        CHECK(none.activations.empty() && none.exhausted_activation_budget && !none.exhausted_work_budget && !none.idle);
        CHECK(error_of([&] { scheduler.schedule_step(SchedulerBudget(1, 0, 16)); }).find("max_prefill_tokens_per_activation") != std::string::npos);
        // the work budget caps the chunk: 1 unit left -> 1 token
        const Activation one = first_activation(scheduler, SchedulerBudget(4, 8, 1));
        CHECK(is_prefill(one, 0, {1}, 2));
        // a prefill chunk that does not end the prompt may not emit tokens
        CHECK(error_of([&] { scheduler.complete_activation(one.id, ActivationOutcome::generated({7}, true)); }).find("before the prompt was complete") != std::string::npos);
        CHECK(error_of([&] { scheduler.complete_activation(12345, ActivationOutcome::prefill_complete()); }).find("unknown in-flight activation") != std::string::npos);
    }});
    all.push_back({"scheduler_close_after_current_finishes_the_event_and_drops_the_queue", [] {
        StreamScheduler scheduler;
        scheduler.add_stream("stream_a");
        scheduler.enqueue_input_event("stream_a", event("event_0", {1}, 1));
        scheduler.enqueue_input_event("stream_a", event("event_1", {2}, 1));
        const Activation prefill = first_activation(scheduler, budget(1));
        const StreamSnapshot closing = scheduler.close_stream_after_current("stream_a");
        CHECK(closing.status == StreamStatus::Closing && closing.queued_input_event_count == 0);
        CHECK(error_of([&] { scheduler.enqueue_input_event("stream_a", event("event_2", {3}, 1)); }).find("is closing") != std::string::npos);
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        const Activation decode = first_activation(scheduler, budget(1));
        const StreamSnapshot done = scheduler.complete_activation(decode.id, ActivationOutcome::generated({5}, true));
        CHECK(done.status == StreamStatus::Idle && done.completed_input_event_count == 1);
        scheduler.enqueue_input_event("stream_a", event("event_3", {4}, 1));  // open again once the event is over
    }});

    // ------------------------------------------------------------------ prefix-state cache (stream_prefix_cache.rs:406-583)
    auto layer_key = [](const char *state_id) { return StateKey{"layer_00", state_id}; };
    auto cache_key = [](std::vector<uint32_t> tokens, std::vector<StateKey> state_keys) {
        return PrefixStateCacheKey::from_token_prefix("package_a", "graph_a", tokens, "reasoning=true", std::move(state_keys));
    };
    all.push_back({"prefix_cache_key_normalizes_state_keys_and_hashes_prefix_contents", [=] {
        const PrefixStateCacheKey left = cache_key({1, 2, 3}, {layer_key("v"), layer_key("k"), layer_key("k")});
        const PrefixStateCacheKey right = cache_key({1, 2, 3}, {layer_key("k"), layer_key("v")});
        const PrefixStateCacheKey different_tokens = cache_key({1, 2, 4}, {layer_key("k"), layer_key("v")});
        CHECK(left == right);
        CHECK(left.token_hash != different_tokens.token_hash);
        CHECK(left.state_keys == (std::vector<StateKey>{layer_key("k"), layer_key("v")}));
        // FNV-1a, 64 bit, of "nerve:token-prefix:v1" | u64 count | u32 tokens, all little-endian: worked by hand for
        // the empty sequence from the published offset and prime
        uint64_t expected = 0xcbf29ce484222325ull;
        for (const char *c = "nerve:token-prefix:v1"; *c; c++) expected = (expected ^ static_cast<uint8_t>(*c)) * 0x100000001b3ull;
        for (int i = 0; i < 8; i++) expected = (expected ^ 0u) * 0x100000001b3ull;
        CHECK(stable_token_prefix_hash(nullptr, 0) == expected);
        CHECK(error_of([&] { cache_key({}, {layer_key("k")}); }).find("token prefix must not be empty") != std::string::npos);
        CHECK(error_of([&] { cache_key({1}, {}); }).find("state key set must not be empty") != std::string::npos);
    }});
    all.push_back({"prefix_cache_eviction_releases_retained_state_blocks", [=] {
        StateArena arena;
        StateTable first("source_a"), second("source_b");
        const BlockShape shape = BlockShape::append(16, 2);
        first.declare_state(layer_key("kv"), shape);
        second.declare_state(layer_key("kv"), shape);
        first.append_activations(arena, layer_key("kv"), 2);
        second.append_activations(arena, layer_key("kv"), 2);
        const BlockId first_block = first.snapshot().entries[0].block_ids[0], second_block = second.snapshot().entries[0].block_ids[0];
        PrefixStateCache cache(1);
        cache.insert(arena, cache_key({1, 2}, {layer_key("kv")}), first);
        CHECK(arena.ref_count(first_block) == 2);
        const PrefixStateCacheInsert inserted = cache.insert(arena, cache_key({3, 4}, {layer_key("kv")}), second);
        CHECK(inserted.evicted_keys.size() == 1 && inserted.evicted_keys[0] == cache_key({1, 2}, {layer_key("kv")}) && !inserted.replaced_existing);
        CHECK(cache.snapshot().entry_count == 1 && cache.snapshot().eviction_count == 1);
        CHECK(arena.ref_count(first_block) == 1);
        CHECK(arena.ref_count(second_block) == 2);
    }});
    all.push_back({"prefix_cache_rejects_non_block_aligned_state", [=] {
        StateArena arena;
        StateTable source("source");
        source.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        source.append_activations(arena, layer_key("kv"), 1);
        PrefixStateCache cache(1);
        const std::string error = error_of([&] { cache.insert(arena, cache_key({1}, {layer_key("kv")}), source); });
        CHECK(error.find("is not aligned to block capacity") != std::string::npos);
        CHECK(cache.snapshot().entry_count == 0);
        CHECK(arena.snapshot().blocks[0].ref_count == 1);
    }});
    all.push_back({"prefix_cache_accepts_initialized_mutable_state_alongside_aligned_append_state", [=] {
        StateArena arena;
        StateTable source("source");
        source.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        source.declare_state(layer_key("recurrent"), BlockShape::mutable_singleton(64));
        source.append_activations(arena, layer_key("kv"), 2);
        source.append_activations(arena, layer_key("recurrent"), 2);
        PrefixStateCache cache(1);
        cache.insert(arena, cache_key({1, 2}, {layer_key("kv"), layer_key("recurrent")}), source);
        CHECK(cache.snapshot().entry_count == 1);
        CHECK(cache.snapshot().entries[0].block_count == 2);
        CHECK(cache.snapshot().entries[0].cached_stream_id == "prefix_cache_0");
    }});
    all.push_back({"prefix_cache_rejects_key_that_does_not_match_source_state_depth", [=] {
        StateArena arena;
        StateTable source("source");
        source.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        source.append_activations(arena, layer_key("kv"), 2);
        PrefixStateCache cache(1);
        const std::string error = error_of([&] { cache.insert(arena, cache_key({1, 2, 3, 4}, {layer_key("kv")}), source); });
        CHECK(error.find("does not match source state") != std::string::npos);
        CHECK(cache.snapshot().entry_count == 0);
        CHECK(arena.snapshot().blocks[0].ref_count == 1);
    }});
    all.push_back({"prefix_cache_finds_longest_compatible_token_prefix", [=] {
        StateArena arena;
        StateTable short_source("short_source"), long_source("long_source");
        short_source.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        long_source.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        short_source.append_activations(arena, layer_key("kv"), 2);
        long_source.append_activations(arena, layer_key("kv"), 4);
        PrefixStateCache cache(4);
        cache.insert(arena, cache_key({1, 2}, {layer_key("kv")}), short_source);
        cache.insert(arena, cache_key({1, 2, 3, 4}, {layer_key("kv")}), long_source);
        const auto matched = cache.longest_matching_key("package_a", "graph_a", {1, 2, 3, 4, 5, 6}, "reasoning=true", {layer_key("kv")});
        CHECK(matched.has_value() && matched->token_count == 4);
        const uint32_t four[4] = {1, 2, 3, 4};
        CHECK(matched->token_hash == stable_token_prefix_hash(four, 4));
        CHECK(!cache.longest_matching_key("package_a", "graph_a", {1, 2, 3, 4, 5, 6}, "reasoning=false", {layer_key("kv")}).has_value());
        // a sequence that parts from the long entry after two tokens falls back to the short one; other packages and
        // graphs see nothing
        const auto shorter = cache.longest_matching_key("package_a", "graph_a", {1, 2, 9, 4}, "reasoning=true", {layer_key("kv")});
        CHECK(shorter.has_value() && shorter->token_count == 2);
        CHECK(!cache.longest_matching_key("package_b", "graph_a", {1, 2, 3, 4}, "reasoning=true", {layer_key("kv")}).has_value());
        CHECK(!cache.longest_matching_key("package_a", "graph_b", {1, 2, 3, 4}, "reasoning=true", {layer_key("kv")}).has_value());
        CHECK(!cache.longest_matching_key("package_a", "graph_a", {}, "reasoning=true", {layer_key("kv")}).has_value());
    }});
    all.push_back({"prefix_cache_evicts_the_least_recently_used_entry_and_keeps_nothing_at_capacity_zero", [=] {
        StateArena arena;
        StateTable a("a"), b("b"), c("c"), target("target");
        for (StateTable *table : {&a, &b, &c}) {
            table->declare_state(layer_key("kv"), BlockShape::append(16, 2));
            table->append_activations(arena, layer_key("kv"), 2);
        }
        target.declare_state(layer_key("kv"), BlockShape::append(16, 2));
        PrefixStateCache cache(2);
        cache.insert(arena, cache_key({1, 2}, {layer_key("kv")}), a);
        cache.insert(arena, cache_key({3, 4}, {layer_key("kv")}), b);
        CHECK(cache.restore_into(arena, cache_key({1, 2}, {layer_key("kv")}), target));  // a is now the more recently used one
        CHECK(target.snapshot().logical_activation_count == 2);
        const PrefixStateCacheInsert inserted = cache.insert(arena, cache_key({5, 6}, {layer_key("kv")}), c);
        CHECK(inserted.evicted_keys.size() == 1 && inserted.evicted_keys[0] == cache_key({3, 4}, {layer_key("kv")}));
        CHECK(!cache.restore_into(arena, cache_key({3, 4}, {layer_key("kv")}), target));
        const std::vector<PrefixStateCacheKey> dropped = cache.set_capacity(arena, 0);
        CHECK(dropped.size() == 2 && cache.snapshot().entry_count == 0 && cache.snapshot().eviction_count == 3);
        CHECK(!cache.insert(arena, cache_key({1, 2}, {layer_key("kv")}), a).replaced_existing && cache.snapshot().entry_count == 0);
    }});

    // ------------------------------------------------------------------ scheduler hooks (stream_runtime_tests.rs:518-769)
    all.push_back({"scheduler_prefix_cache_restores_state_after_source_reset", [] {
        const PrefixStateCacheKey prefix_key = PrefixStateCacheKey::from_token_prefix("package_a", "graph_a", {1, 2}, "reasoning=true", {state_key()});
        StreamScheduler scheduler(2);
        scheduler.add_stream("source", "package_a", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("source", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        scheduler.cache_stream_prefix_state("source", prefix_key);
        const BlockId cached_block = scheduler.stream_transient_state_snapshot("source").entries[0].block_ids[0];
        auto ref_count = [&](BlockId id) {
            for (const BlockSnapshot &block : scheduler.transient_state_arena_snapshot().blocks)
                if (block.block_id == id) return block.ref_count;
            throw CaseFailure{"block not in the arena"};
        };
        CHECK(ref_count(cached_block) == 2);
        scheduler.interrupt_stream("source", "drop source");
        scheduler.reset_stream_transient_state("source");
        scheduler.add_stream("target", "package_a", {{state_key(), state_shape()}});
        CHECK(scheduler.restore_stream_prefix_state("target", prefix_key));
        CHECK(scheduler.stream_transient_state_snapshot("target").entries[0].block_ids == std::vector<BlockId>{cached_block});
        const PrefixStateCacheSnapshot cache = scheduler.prefix_state_cache_snapshot();
        CHECK(cache.entry_count == 1 && cache.entries[0].use_count == 1);
        CHECK(ref_count(cached_block) == 2);
    }});
    all.push_back({"scheduler_prefix_cache_rejects_execution_class_mismatch_without_mutation", [] {
        const PrefixStateCacheKey prefix_key = PrefixStateCacheKey::from_token_prefix("package_a", "graph_a", {1, 2}, "reasoning=true", {state_key()});
        StreamScheduler scheduler(2);
        scheduler.add_stream("source", "package_a", {{state_key(), state_shape()}});
        scheduler.add_stream("target", "package_b", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("source", event("event_0", {1, 2}, 8));
        const Activation prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        scheduler.cache_stream_prefix_state("source", prefix_key);
        const TableSnapshot before_target = scheduler.stream_transient_state_snapshot("target");
        const std::string error = error_of([&] { scheduler.restore_stream_prefix_state("target", prefix_key); });
        CHECK(error.find("cannot restore prefix key execution class") != std::string::npos);
        CHECK(scheduler.stream_transient_state_snapshot("target") == before_target);
        CHECK(scheduler.prefix_state_cache_snapshot().entries[0].use_count == 0);
        CHECK(error_of([&] { scheduler.cache_stream_prefix_state("target", prefix_key); }).find("under prefix key execution class") != std::string::npos);
    }});
    all.push_back({"scheduler_restores_longest_matching_prefix_state", [] {
        StreamScheduler scheduler(4);
        scheduler.add_stream("short_source", "package_a", {{state_key(), state_shape()}});
        scheduler.add_stream("long_source", "package_a", {{state_key(), state_shape()}});
        scheduler.enqueue_input_event("short_source", event("short_event", {1, 2}, 0));
        const Activation short_prefill = first_activation(scheduler, budget(1));
        scheduler.complete_activation(short_prefill.id, ActivationOutcome::prefill_complete());
        scheduler.enqueue_input_event("long_source", event("long_event", {1, 2, 3, 4}, 0));
        for (int i = 0; i < 2; i++) {
            const Activation prefill = first_activation(scheduler, budget(1));
            scheduler.complete_activation(prefill.id, ActivationOutcome::prefill_complete());
        }
        const PrefixStateCacheKey short_key = scheduler.cache_stream_prefix_state_for_tokens("short_source", "graph_a", {1, 2}, "reasoning=true", {state_key()});
        const PrefixStateCacheKey long_key = scheduler.cache_stream_prefix_state_for_tokens("long_source", "graph_a", {1, 2, 3, 4}, "reasoning=true", {state_key()});
        scheduler.add_stream("target", "package_a", {{state_key(), state_shape()}});
        const auto matched = scheduler.restore_longest_stream_prefix_state("target", "graph_a", {1, 2, 3, 4, 5}, "reasoning=true", {state_key()});
        CHECK(matched.has_value() && *matched == long_key && *matched != short_key);
        CHECK(scheduler.stream_transient_state_snapshot("target").logical_activation_count == 4);
        for (const PrefixStateCacheEntrySnapshot &entry : scheduler.prefix_state_cache_snapshot().entries)
            CHECK(entry.use_count == (entry.key == long_key ? 1u : 0u));
    }});
    return all;
}

}  // namespace

int main(int argc, char **argv) {
    int failures = 0, ran = 0;
    for (const Case &one : cases()) {
        if (argc > 1 && std::strcmp(argv[1], "--list") == 0) {
            std::printf("%s\n", one.name);
            continue;
        }
        if (argc > 1 && std::strcmp(argv[1], one.name) != 0) continue;
        ran++;
        try {
            one.run();
            std::printf("ok %s\n", one.name);
        } catch (const CaseFailure &failure) {
            failures++;
            std::printf("FAIL %s: %s\n", one.name, failure.what.c_str());
        } catch (const std::exception &error) {
            failures++;
            std::printf("FAIL %s: unexpected error: %s\n", one.name, error.what());
        }
    }
    if (argc > 1 && std::strcmp(argv[1], "--list") != 0 && ran == 0) {
        std::printf("FAIL %s: no such case\n", argv[1]);
        return 1;
    }
    return failures;
}
