"""ctypes mirror of the stream scheduler entry points of libnerve_b200.so (host only, no GPU needed): the
reference's RuntimeStreamScheduler (runtime-rs/src/stream_runtime.rs:426-1433) over its transient-state arena
(runtime-rs/src/stream_state.rs:122-633).  Names and argument meaning follow the reference's methods."""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

from .runtime import NerveError, library

STATUS = ("idle", "active", "interrupted", "closing")


class _Declaration(ctypes.Structure):
    _fields_ = [("node_instance_id", ctypes.c_char_p), ("state_id", ctypes.c_char_p), ("bytes_per_activation", ctypes.c_uint64),
                ("activation_capacity", ctypes.c_uint64), ("maximum_activation_count", ctypes.c_uint64), ("retention", ctypes.c_int32)]


class _Budget(ctypes.Structure):
    _fields_ = [("max_activations", ctypes.c_uint64), ("max_prefill_tokens_per_activation", ctypes.c_uint64),
                ("max_decode_tokens_per_activation", ctypes.c_uint64), ("max_work_units", ctypes.c_uint64)]


class _StreamSnapshot(ctypes.Structure):
    _fields_ = [("status", ctypes.c_int32), ("queued_input_event_count", ctypes.c_uint64), ("in_flight_activation_count", ctypes.c_uint64),
                ("completed_input_event_count", ctypes.c_uint64), ("scheduled_activation_count", ctypes.c_uint64),
                ("generated_token_count", ctypes.c_uint64), ("transient_state_entry_count", ctypes.c_uint64),
                ("transient_state_block_count", ctypes.c_uint64), ("transient_state_logical_activation_count", ctypes.c_uint64),
                ("current_input_event_id", ctypes.c_char * 64)]


class _Counts(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint64) for name in ("stream_count", "active_stream_count", "in_flight_activation_count",
                                                     "allocated_block_count", "free_block_count", "live_block_count")]


class _Activation(ctypes.Structure):
    _fields_ = [("id", ctypes.c_uint64), ("kind", ctypes.c_int32), ("token_offset", ctypes.c_uint64), ("token_count", ctypes.c_uint64),
                ("remaining_prompt_token_count", ctypes.c_uint64), ("feedback_depth", ctypes.c_uint64), ("max_tokens", ctypes.c_uint64),
                ("max_state_activation_count", ctypes.c_uint64), ("reservation_count", ctypes.c_uint64),
                ("stream_id", ctypes.c_char * 64), ("execution_class_id", ctypes.c_char * 64), ("input_event_id", ctypes.c_char * 64)]


class _Slot(ctypes.Structure):
    _fields_ = [("logical_activation_index", ctypes.c_uint64), ("block_id", ctypes.c_uint64), ("block_activation_offset", ctypes.c_uint64),
                ("block_activation_capacity", ctypes.c_uint64), ("allocated_block", ctypes.c_int32), ("copy_from_block_id", ctypes.c_int64)]


@dataclass
class StateDeclaration:
    node_instance_id: str
    state_id: str
    bytes_per_activation: int
    activation_capacity: int = 1
    maximum_activation_count: int = 0  # 0 = unbounded
    mutable_singleton: bool = False


@dataclass
class Budget:
    max_activations: int
    max_prefill_tokens_per_activation: int
    max_work_units: int
    max_decode_tokens_per_activation: int = 1


@dataclass
class Activation:
    id: int
    kind: str  # "prefill_chunk" | "decode_feedback"
    stream_id: str
    execution_class_id: str
    input_event_id: str
    token_offset: int
    token_ids: list
    remaining_prompt_token_count: int
    feedback_depth: int
    max_tokens: int
    max_state_activation_count: int
    state_reservations: list = field(default_factory=list)  # [{"key": (node, state), "slots": [dict, ...]}]

    @property
    def work_units(self) -> int:
        return len(self.token_ids) if self.kind == "prefill_chunk" else self.max_tokens


def _check(status: int) -> None:
    if status != 0:
        raise NerveError(library().nerve_b200_last_error().decode())


def _snapshot(raw: _StreamSnapshot) -> dict:
    out = {name: getattr(raw, name) for name, _ in _StreamSnapshot._fields_ if name not in ("status", "current_input_event_id")}
    out["status"] = STATUS[raw.status]
    out["current_input_event_id"] = raw.current_input_event_id.decode() or None
    return out


class Scheduler:
    def __init__(self):
        self._lib = library()
        self._handle = ctypes.c_void_p()
        _check(self._lib.nerve_b200_scheduler_create(ctypes.byref(self._handle)))

    def close(self) -> None:
        if self._handle:
            self._lib.nerve_b200_scheduler_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream_call(self, function, *arguments) -> dict:
        raw = _StreamSnapshot()
        _check(function(self._handle, *arguments, ctypes.byref(raw)))
        return _snapshot(raw)

    def add_stream(self, stream_id: str, execution_class_id: str = "default", state_declarations=()) -> dict:
        declarations = (_Declaration * max(1, len(state_declarations)))()
        for index, one in enumerate(state_declarations):
            declarations[index] = _Declaration(one.node_instance_id.encode(), one.state_id.encode(), one.bytes_per_activation,
                                               one.activation_capacity, one.maximum_activation_count, 1 if one.mutable_singleton else 0)
        return self._stream_call(self._lib.nerve_b200_scheduler_add_stream, stream_id.encode(), execution_class_id.encode(), declarations,
                                 ctypes.c_size_t(len(state_declarations)))

    def fork_stream_transient_state(self, source_stream_id: str, target_stream_id: str, execution_class_id: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_fork_stream, source_stream_id.encode(), target_stream_id.encode(),
                                 execution_class_id.encode())

    def enqueue_input_event(self, stream_id: str, event_id: str, token_ids, max_public_tokens: int) -> dict:
        tokens = (ctypes.c_uint32 * max(1, len(token_ids)))(*token_ids)
        return self._stream_call(self._lib.nerve_b200_scheduler_enqueue, stream_id.encode(), event_id.encode(), tokens,
                                 ctypes.c_size_t(len(token_ids)), ctypes.c_uint64(max_public_tokens))

    def interrupt_stream(self, stream_id: str, reason: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_interrupt, stream_id.encode(), reason.encode())

    def reset_stream_transient_state(self, stream_id: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_reset_stream_state, stream_id.encode())

    def remove_stream(self, stream_id: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_remove_stream, stream_id.encode())

    def close_stream_after_current(self, stream_id: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_close_after_current, stream_id.encode())

    def stream_snapshot(self, stream_id: str) -> dict:
        return self._stream_call(self._lib.nerve_b200_scheduler_stream_snapshot, stream_id.encode())

    # prefix-state cache (stream_runtime.rs:541-559, 616-705)
    def set_prefix_state_cache_capacity(self, capacity_entries: int) -> int:
        """Returns how many entries were evicted to get down to the new capacity."""
        evicted = ctypes.c_uint64()
        _check(self._lib.nerve_b200_scheduler_set_prefix_state_cache_capacity(self._handle, ctypes.c_uint64(capacity_entries), ctypes.byref(evicted)))
        return evicted.value

    def cache_stream_prefix_state_for_tokens(self, stream_id: str, runtime_graph_id: str, token_ids, runtime_modifier_bytes: bytes = b"") -> dict:
        tokens = (ctypes.c_uint32 * max(1, len(token_ids)))(*[int(t) for t in token_ids])
        modifiers = (ctypes.c_uint8 * max(1, len(runtime_modifier_bytes)))(*runtime_modifier_bytes)
        flags, evicted = ctypes.c_int32(), ctypes.c_uint64()
        _check(self._lib.nerve_b200_scheduler_cache_stream_prefix_state_for_tokens(
            self._handle, stream_id.encode(), runtime_graph_id.encode(), tokens, ctypes.c_size_t(len(token_ids)), modifiers,
            ctypes.c_size_t(len(runtime_modifier_bytes)), ctypes.byref(flags), ctypes.byref(evicted)))
        return {"replaced_existing": bool(flags.value & 1), "evicted_count": evicted.value}

    def restore_longest_stream_prefix_state(self, target_stream_id: str, runtime_graph_id: str, token_ids, runtime_modifier_bytes: bytes = b"") -> int:
        """Token count of the retained prefix whose state the target stream now shares; 0 when none matches."""
        tokens = (ctypes.c_uint32 * max(1, len(token_ids)))(*[int(t) for t in token_ids])
        modifiers = (ctypes.c_uint8 * max(1, len(runtime_modifier_bytes)))(*runtime_modifier_bytes)
        restored = ctypes.c_uint64()
        _check(self._lib.nerve_b200_scheduler_restore_longest_stream_prefix_state(
            self._handle, target_stream_id.encode(), runtime_graph_id.encode(), tokens, ctypes.c_size_t(len(token_ids)), modifiers,
            ctypes.c_size_t(len(runtime_modifier_bytes)), ctypes.byref(restored)))
        return restored.value

    def prefix_state_cache_counts(self) -> dict:
        counts = (ctypes.c_uint64 * 3)()
        _check(self._lib.nerve_b200_scheduler_prefix_state_cache_counts(self._handle, counts))
        return {"capacity_entries": counts[0], "entry_count": counts[1], "eviction_count": counts[2]}

    def snapshot(self) -> dict:
        raw = _Counts()
        _check(self._lib.nerve_b200_scheduler_snapshot(self._handle, ctypes.byref(raw)))
        return {name: getattr(raw, name) for name, _ in _Counts._fields_}

    def schedule_step(self, budget: Budget) -> dict:
        raw_budget = _Budget(budget.max_activations, budget.max_prefill_tokens_per_activation, budget.max_decode_tokens_per_activation,
                             budget.max_work_units)
        count, flags = ctypes.c_size_t(), ctypes.c_int32()
        _check(self._lib.nerve_b200_scheduler_schedule_step(self._handle, ctypes.byref(raw_budget), ctypes.byref(count), ctypes.byref(flags)))
        activations = [self._activation(index) for index in range(count.value)]
        return {"activations": activations, "exhausted_activation_budget": bool(flags.value & 1),
                "exhausted_work_budget": bool(flags.value & 2), "idle": bool(flags.value & 4)}

    def _activation(self, index: int) -> Activation:
        raw = _Activation()
        _check(self._lib.nerve_b200_scheduler_step_activation(self._handle, ctypes.c_size_t(index), ctypes.byref(raw), None, ctypes.c_size_t(0)))
        tokens = (ctypes.c_uint32 * max(1, raw.token_count))()
        _check(self._lib.nerve_b200_scheduler_step_activation(self._handle, ctypes.c_size_t(index), ctypes.byref(raw), tokens,
                                                             ctypes.c_size_t(raw.token_count)))
        reservations = []
        for reservation in range(raw.reservation_count):
            node, state = ctypes.create_string_buffer(64), ctypes.create_string_buffer(64)
            slots = (_Slot * max(1, raw.max_state_activation_count))()
            slot_count = ctypes.c_size_t()
            _check(self._lib.nerve_b200_scheduler_step_reservation(self._handle, ctypes.c_size_t(index), ctypes.c_size_t(reservation), node, state,
                                                                  slots, ctypes.c_size_t(len(slots)), ctypes.byref(slot_count)))
            reservations.append({"key": (node.value.decode(), state.value.decode()),
                                 "slots": [{"logical_activation_index": s.logical_activation_index, "block_id": s.block_id,
                                            "block_activation_offset": s.block_activation_offset,
                                            "block_activation_capacity": s.block_activation_capacity, "allocated_block": bool(s.allocated_block),
                                            "copy_from_block_id": None if s.copy_from_block_id < 0 else s.copy_from_block_id}
                                           for s in slots[: slot_count.value]]})
        return Activation(raw.id, "prefill_chunk" if raw.kind == 0 else "decode_feedback", raw.stream_id.decode(),
                          raw.execution_class_id.decode(), raw.input_event_id.decode(), raw.token_offset, list(tokens[: raw.token_count]),
                          raw.remaining_prompt_token_count, raw.feedback_depth, raw.max_tokens, raw.max_state_activation_count, reservations)

    def complete_activation(self, activation_id: int, generated_token_ids=(), continue_generation: bool = True,
                            processed_state_activation_count: int | None = None) -> dict:
        tokens = (ctypes.c_uint32 * max(1, len(generated_token_ids)))(*generated_token_ids)
        processed = -1 if processed_state_activation_count is None else processed_state_activation_count
        return self._stream_call(self._lib.nerve_b200_scheduler_complete, ctypes.c_uint64(activation_id), tokens,
                                 ctypes.c_size_t(len(generated_token_ids)), ctypes.c_int32(1 if continue_generation else 0), ctypes.c_int64(processed))
