"""ctypes mirror of include/nerve_b200.h.

Names follow the reference engine's API (add_stream, fork_stream,
enqueue_input_event, run_until_idle ...: runtime-rs/src/vulkan_stream_circuit/
placed_prompt_engine.rs:48-589) so that tests read like the reference's own.
Every failure raises NerveError with the library's message; a missing library
is an error, never a fallback.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libnerve_b200.so"


class NerveError(RuntimeError):
    pass


class _MountOptions(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        "device", "capacity_tokens", "page_tokens", "max_streams", "max_lanes", "verify_level", "tp_rank", "tp_size",
        "extra_pages")]


class _PackageInfo(ctypes.Structure):
    _fields_ = [
        ("hidden_size", ctypes.c_int64), ("vocab_size", ctypes.c_int64), ("layer_count", ctypes.c_int64),
        ("max_context", ctypes.c_int64), ("has_speculative_decoder", ctypes.c_int32), ("kv_layer_count", ctypes.c_int32),
        ("weight_bytes", ctypes.c_uint64), ("verify_step_weight_bytes", ctypes.c_uint64),
        ("draft_step_weight_bytes", ctypes.c_uint64), ("kv_bytes_per_token", ctypes.c_uint64),
        ("pages_per_stream", ctypes.c_int32), ("physical_pages", ctypes.c_int32), ("page_tokens", ctypes.c_int32),
        ("eos_token_id", ctypes.c_uint32), ("target_decode_stack", ctypes.c_int32), ("draft_decode_stack", ctypes.c_int32),
        ("target_stack_weight_bytes", ctypes.c_uint64),
    ]


class _SamplerConfig(ctypes.Structure):
    _fields_ = [("method", ctypes.c_int32), ("temperature", ctypes.c_float), ("top_p", ctypes.c_float),
                ("min_p", ctypes.c_float), ("top_k", ctypes.c_int32)]


_REPORT_U64 = (
    "prefill_ns", "decode_ns", "prefill_tokens", "generated_tokens", "activation_count", "batch_count",
    "max_batch_width", "cycle_count", "proposed_draft_token_count", "accepted_draft_token_count",
    "emitted_token_count", "draft_time_ns", "target_verification_time_ns", "draft_catch_up_time_ns",
    "kernel_launches", "graph_launches", "h2d_bytes", "d2h_bytes", "host_syncs")


class _EngineStreamSnapshot(ctypes.Structure):
    _fields_ = [("pending_input_event_count", ctypes.c_uint64), ("next_stream_tick", ctypes.c_uint64),
                ("completed_prompt_event_count", ctypes.c_uint64), ("context_window_activations", ctypes.c_uint64),
                ("mapped_state_pages", ctypes.c_uint64), ("speculative_draft_tokens", ctypes.c_int32), ("idle", ctypes.c_int32)]


class _EngineSnapshotCounts(ctypes.Structure):
    _fields_ = [("stream_count", ctypes.c_uint64), ("active_stream_count", ctypes.c_uint64), ("idle", ctypes.c_int32)]


class _RunReport(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint64) for name in _REPORT_U64] + [
        ("verify_ms_sum", ctypes.c_double), ("verify_steps", ctypes.c_uint64), ("verify_bytes", ctypes.c_uint64),
        ("device_ms", ctypes.c_double), ("int4_ms", ctypes.c_double), ("int4_bytes", ctypes.c_uint64),
        ("int4_launches", ctypes.c_uint64), ("idle", ctypes.c_int32)]


_OUTPUT_CALLBACK = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64)

EXPORTED_SYMBOLS = (
    "nerve_b200_last_error", "nerve_b200_abi_version", "nerve_b200_package_mount", "nerve_b200_package_unmount",
    "nerve_b200_package_describe", "nerve_b200_package_validate", "nerve_b200_engine_create",
    "nerve_b200_engine_destroy", "nerve_b200_engine_add_stream", "nerve_b200_engine_fork_stream",
    "nerve_b200_engine_reset_stream", "nerve_b200_engine_remove_stream", "nerve_b200_engine_interrupt_stream",
    "nerve_b200_engine_enqueue", "nerve_b200_engine_run_until_idle", "nerve_b200_engine_run",
    "nerve_b200_engine_set_profiling", "nerve_b200_engine_inject_barrier_timeouts", "nerve_b200_tp_unique_id", "nerve_b200_tp_shard_range", "nerve_b200_engine_stop_after_current", "nerve_b200_engine_stream_snapshot_of", "nerve_b200_engine_snapshot", "nerve_b200_engine_scheduler_stream_counts", "nerve_b200_engine_set_prefix_cache_capacity", "nerve_b200_engine_prefix_cache_stats", "nerve_b200_engine_init_tp", "nerve_b200_engine_tp_exchange_handle", "nerve_b200_engine_tp_connect", "nerve_b200_engine_set_decode_stack", "nerve_b200_engine_decode_stack_timing", "nerve_b200_engine_stream_tick",
    "nerve_b200_engine_set_teacher_tokens", "nerve_b200_engine_set_prefill_chunk",
    "nerve_b200_engine_set_cycle_logging", "nerve_b200_engine_cycle_log", "nerve_b200_debug_target_logits",
    "nerve_b200_op_linear_int4", "nerve_b200_op_linear_int4_silu_pair",
    "nerve_b200_op_linear_bf16", "nerve_b200_op_rms_norm", "nerve_b200_op_linear_fp8",
    "nerve_b200_op_greedy", "nerve_b200_op_greedy_scratch_bytes", "nerve_b200_op_greedy_static", "nerve_b200_op_sample_top_k_top_p", "nerve_b200_op_sample_scratch_bytes", "nerve_b200_verify_prefix",
    "nerve_b200_stream_control_bytes", "nerve_b200_state_page_table_bytes",
    "nerve_b200_scheduler_create", "nerve_b200_scheduler_destroy", "nerve_b200_scheduler_add_stream",
    "nerve_b200_scheduler_fork_stream", "nerve_b200_scheduler_enqueue", "nerve_b200_scheduler_interrupt",
    "nerve_b200_scheduler_reset_stream_state", "nerve_b200_scheduler_remove_stream",
    "nerve_b200_scheduler_close_after_current", "nerve_b200_scheduler_schedule_step",
    "nerve_b200_scheduler_step_activation", "nerve_b200_scheduler_step_reservation", "nerve_b200_scheduler_complete",
    "nerve_b200_scheduler_snapshot", "nerve_b200_scheduler_stream_snapshot",
    "nerve_b200_scheduler_set_prefix_state_cache_capacity", "nerve_b200_scheduler_cache_stream_prefix_state_for_tokens",
    "nerve_b200_scheduler_restore_longest_stream_prefix_state", "nerve_b200_scheduler_prefix_state_cache_counts",
)

_library = None


def library() -> ctypes.CDLL:
    """Loads libnerve_b200.so (built in-tree by llmoop_b200.build); raises if it is absent."""
    global _library
    if _library is None:
        if not LIB_PATH.exists():
            raise NerveError(f"{LIB_PATH} is missing: run `python -m llmoop_b200.build` (there is no CPU fallback)")
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.nerve_b200_last_error.restype = ctypes.c_char_p
        for name in EXPORTED_SYMBOLS:
            if name != "nerve_b200_last_error":
                getattr(lib, name).restype = ctypes.c_int32
        lib.nerve_b200_op_greedy_scratch_bytes.restype = ctypes.c_uint64
        lib.nerve_b200_op_sample_scratch_bytes.restype = ctypes.c_uint64
        _library = lib
    return _library


def _check(status: int) -> None:
    if status != 0:
        raise NerveError(library().nerve_b200_last_error().decode("utf-8", "replace"))


def validate_package(path, verify_level: int = 2):
    """Host-only parse + integrity check + plan build.  Returns (op_count, tensor_count)."""
    ops, tensors = ctypes.c_int64(0), ctypes.c_int64(0)
    _check(library().nerve_b200_package_validate(str(path).encode(), verify_level, ctypes.byref(ops), ctypes.byref(tensors)))
    return ops.value, tensors.value


def verify_prefix(draft, target, stop=()):
    """speculative_decode.rs:54-105 -> (accepted, committed, emitted)."""
    draft_a = (ctypes.c_uint32 * max(1, len(draft)))(*draft)
    target_a = (ctypes.c_uint32 * max(1, len(target)))(*target)
    stop_a = (ctypes.c_uint32 * max(1, len(stop)))(*stop)
    counts = (ctypes.c_uint32 * 2)()
    emitted = (ctypes.c_uint32 * (len(draft) + 2))()
    count = ctypes.c_size_t(0)
    _check(library().nerve_b200_verify_prefix(draft_a, ctypes.c_size_t(len(draft)), target_a, ctypes.c_size_t(len(target)),
                                              stop_a, ctypes.c_size_t(len(stop)), counts, emitted, ctypes.byref(count)))
    return counts[0], counts[1], list(emitted[:count.value])


@dataclass
class RunReport:
    values: dict

    def __getattr__(self, name):
        try:
            return self.values[name]
        except KeyError as error:
            raise AttributeError(name) from error


class Package:
    """A compiled package resident on one GPU."""

    def __init__(self, path, *, device=0, capacity_tokens=1024, page_tokens=16, max_streams=8, max_lanes=64,
                 verify_level=1, tp_rank=0, tp_size=1, extra_pages=0):
        options = _MountOptions(device, capacity_tokens, page_tokens, max_streams, max_lanes, verify_level, tp_rank,
                                tp_size, extra_pages)
        self._handle = ctypes.c_void_p()
        _check(library().nerve_b200_package_mount(str(path).encode(), ctypes.byref(options), ctypes.byref(self._handle)))
        info = _PackageInfo()
        _check(library().nerve_b200_package_describe(self._handle, ctypes.byref(info)))
        self.info = {name: getattr(info, name) for name, _ in _PackageInfo._fields_}

    def unmount(self):
        if self._handle:
            _check(library().nerve_b200_package_unmount(self._handle))
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.unmount()
        except Exception:
            pass


def nccl_library_path() -> str:
    """libnccl.so.2 as shipped with torch's CUDA wheels, or the system's."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is not None and spec.submodule_search_locations:
        for base in spec.submodule_search_locations:
            candidate = Path(base) / "lib" / "libnccl.so.2"
            if candidate.exists():
                return str(candidate)
    return "libnccl.so.2"


def tp_shard_range(total: int, unit: int, rank: int, size: int):
    """(begin, count) of rank's tensor-parallel shard; raises NerveError when total is not a multiple of unit x size."""
    begin, count = ctypes.c_int64(0), ctypes.c_int64(0)
    _check(library().nerve_b200_tp_shard_range(ctypes.c_int64(total), ctypes.c_int64(unit), rank, size, ctypes.byref(begin), ctypes.byref(count)))
    return begin.value, count.value


def tensor_parallel_unique_id() -> bytes:
    """The 128-byte NCCL id rank 0 creates and passes to the other ranks."""
    buffer = (ctypes.c_uint8 * 128)()
    _check(library().nerve_b200_tp_unique_id(nccl_library_path().encode(), buffer))
    return bytes(buffer)


class Engine:
    def __init__(self, package: Package):
        self.package = package
        self._handle = ctypes.c_void_p()
        _check(library().nerve_b200_engine_create(package._handle, ctypes.byref(self._handle)))

    def close(self):
        if self._handle:
            _check(library().nerve_b200_engine_destroy(self._handle))
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add_stream(self, stream_id: int, *, seed: int = 0, speculative_draft_tokens: int = 0, sampler=None):
        config = None
        if sampler is not None:
            config = ctypes.byref(_SamplerConfig(sampler.get("method", 0), sampler.get("temperature", 1.0),
                                                 sampler.get("top_p", 1.0), sampler.get("min_p", 0.0), sampler.get("top_k", 1)))
        _check(library().nerve_b200_engine_add_stream(self._handle, ctypes.c_int64(stream_id), ctypes.c_uint32(seed),
                                                      speculative_draft_tokens, config))

    def fork_stream(self, source: int, destination: int, *, seed: int = 0):
        _check(library().nerve_b200_engine_fork_stream(self._handle, ctypes.c_int64(source), ctypes.c_int64(destination),
                                                       ctypes.c_uint32(seed)))

    def reset_stream_transient_state(self, stream_id: int):
        _check(library().nerve_b200_engine_reset_stream(self._handle, ctypes.c_int64(stream_id)))

    def remove_stream(self, stream_id: int):
        _check(library().nerve_b200_engine_remove_stream(self._handle, ctypes.c_int64(stream_id)))

    def interrupt_stream(self, stream_id: int):
        _check(library().nerve_b200_engine_interrupt_stream(self._handle, ctypes.c_int64(stream_id)))

    def stop_stream_after_current(self, stream_id: int):
        _check(library().nerve_b200_engine_stop_after_current(self._handle, ctypes.c_int64(stream_id)))

    def stream_snapshot(self, stream_id: int) -> dict:
        raw = _EngineStreamSnapshot()
        _check(library().nerve_b200_engine_stream_snapshot_of(self._handle, ctypes.c_int64(stream_id), ctypes.byref(raw)))
        out = {name: getattr(raw, name) for name, _ in _EngineStreamSnapshot._fields_}
        out["idle"] = bool(out["idle"])
        return out

    def scheduler_stream_counts(self, stream_id: int) -> dict:
        """The runtime scheduler's counters for one stream (see nerve_b200_engine_scheduler_stream_counts)."""
        counts = (ctypes.c_uint64 * 6)()
        _check(library().nerve_b200_engine_scheduler_stream_counts(self._handle, ctypes.c_int64(stream_id), counts))
        names = ("scheduled_activation_count", "completed_input_event_count", "generated_token_count", "in_flight_activation_count",
                 "queued_input_event_count", "has_current_input_event")
        return {name: int(value) for name, value in zip(names, counts)}

    def set_prefix_cache_capacity(self, entries: int) -> None:
        """Retain up to `entries` prompt prefixes (0 = off, the default); see nerve_b200_engine_set_prefix_cache_capacity."""
        _check(library().nerve_b200_engine_set_prefix_cache_capacity(self._handle, ctypes.c_uint64(entries)))

    def prefix_cache_stats(self) -> dict:
        stats = (ctypes.c_uint64 * 8)()
        _check(library().nerve_b200_engine_prefix_cache_stats(self._handle, stats))
        names = ("hit_count", "miss_count", "insertion_count", "eviction_count", "reused_token_count", "saved_prefill_token_count",
                 "resident_entry_count", "resident_byte_count")
        return {name: int(value) for name, value in zip(names, stats)}

    def snapshot(self) -> dict:
        raw = _EngineSnapshotCounts()
        _check(library().nerve_b200_engine_snapshot(self._handle, ctypes.byref(raw)))
        return {"stream_count": raw.stream_count, "active_stream_count": raw.active_stream_count, "idle": bool(raw.idle)}

    def enqueue_input_event(self, stream_id: int, token_ids, max_public_tokens: int, stop_token_ids=(), event_id="event"):
        tokens = (ctypes.c_uint32 * max(1, len(token_ids)))(*[int(t) for t in token_ids])
        stops = (ctypes.c_uint32 * max(1, len(stop_token_ids)))(*[int(t) for t in stop_token_ids])
        _check(library().nerve_b200_engine_enqueue(self._handle, ctypes.c_int64(stream_id), event_id.encode(), tokens,
                                                   ctypes.c_size_t(len(token_ids)), ctypes.c_size_t(max_public_tokens), stops,
                                                   ctypes.c_size_t(len(stop_token_ids))))

    def run_until_idle(self, on_output=None):
        """Returns (outputs, report): outputs is a list of (stream_id, token_id, source_stream_tick, output_index)."""
        return self.run(0, on_output)

    def init_tensor_parallel(self, rank: int, size: int, unique_id: bytes):
        buffer = (ctypes.c_uint8 * 128).from_buffer_copy(unique_id)
        _check(library().nerve_b200_engine_init_tp(self._handle, nccl_library_path().encode(), rank, size, buffer))

    def tp_exchange_handle(self) -> bytes:
        """This rank's 64-byte inter-process handle of its exchange buffer (see nerve_b200_engine_tp_connect)."""
        buffer = (ctypes.c_uint8 * 64)()
        _check(library().nerve_b200_engine_tp_exchange_handle(self._handle, buffer))
        return bytes(buffer)

    def tp_connect(self, handles) -> None:
        """handles: every rank's tp_exchange_handle() in rank order (own included)."""
        joined = b"".join(handles)
        buffer = (ctypes.c_uint8 * len(joined)).from_buffer_copy(joined)
        _check(library().nerve_b200_engine_tp_connect(self._handle, buffer, len(handles)))

    def set_decode_stack(self, enabled: bool):
        _check(library().nerve_b200_engine_set_decode_stack(self._handle, int(enabled)))

    def decode_stack_timing(self):
        """[layers][32] nanosecond stamps of the last profiled target-stack launch (see the header)."""
        import numpy as np

        count = ctypes.c_size_t(0)
        _check(library().nerve_b200_engine_decode_stack_timing(self._handle, None, ctypes.c_size_t(0), ctypes.byref(count)))
        stamps = (ctypes.c_uint64 * max(1, count.value))()
        _check(library().nerve_b200_engine_decode_stack_timing(self._handle, stamps, ctypes.c_size_t(count.value), ctypes.byref(count)))
        return np.array(stamps[:count.value], dtype=np.uint64).reshape(-1, 32)

    def set_profiling(self, enabled: bool):
        _check(library().nerve_b200_engine_set_profiling(self._handle, int(enabled)))

    def inject_barrier_timeouts(self, launches: int):
        """Test hook: the next `launches` persistent-kernel launches give up at their first grid barrier."""
        _check(library().nerve_b200_engine_inject_barrier_timeouts(self._handle, int(launches)))

    def run(self, max_batches: int = 0, on_output=None):
        """Bounded run: stops after `max_batches` decode batches (0 = until idle)."""
        outputs = []

        def trampoline(_user, stream_id, token_id, tick, index):
            outputs.append((stream_id, token_id, tick, index))
            if on_output is not None:
                on_output(stream_id, token_id, tick, index)

        callback = _OUTPUT_CALLBACK(trampoline)
        report = _RunReport()
        _check(library().nerve_b200_engine_run(self._handle, ctypes.c_uint64(max_batches), callback, None, ctypes.byref(report)))
        values = {name: getattr(report, name) for name, _ in _RunReport._fields_}
        return outputs, RunReport(values)

    def submit_input_event_until_idle(self, stream_id: int, token_ids, max_public_tokens: int, stop_token_ids=()):
        self.enqueue_input_event(stream_id, token_ids, max_public_tokens, stop_token_ids)
        outputs, report = self.run_until_idle()
        return [token for sid, token, _, _ in outputs if sid == stream_id], report

    def stream_tick(self, stream_id: int) -> int:
        tick = ctypes.c_uint64(0)
        _check(library().nerve_b200_engine_stream_tick(self._handle, ctypes.c_int64(stream_id), ctypes.byref(tick)))
        return tick.value

    def set_teacher_tokens(self, stream_id: int, tokens):
        array = (ctypes.c_uint32 * max(1, len(tokens)))(*[int(t) for t in tokens])
        _check(library().nerve_b200_engine_set_teacher_tokens(self._handle, ctypes.c_int64(stream_id), array,
                                                              ctypes.c_size_t(len(tokens))))

    def set_prefill_chunk(self, tokens: int):
        _check(library().nerve_b200_engine_set_prefill_chunk(self._handle, tokens))

    def set_cycle_logging(self, enabled: bool):
        _check(library().nerve_b200_engine_set_cycle_logging(self._handle, int(enabled)))

    def cycle_log(self):
        count = ctypes.c_size_t(0)
        _check(library().nerve_b200_engine_cycle_log(self._handle, None, ctypes.c_size_t(0), ctypes.byref(count)))
        rows = (ctypes.c_uint64 * (22 * max(1, count.value)))()
        _check(library().nerve_b200_engine_cycle_log(self._handle, rows, ctypes.c_size_t(count.value), ctypes.byref(count)))
        out = []
        for i in range(count.value):
            row = rows[i * 22:(i + 1) * 22]
            out.append({
                "stream_id": row[0], "start_tick": row[1], "accepted": row[2], "committed": row[3],
                "emitted": list(row[6:6 + row[4]]), "target_token_ids": list(row[14:14 + row[5]]),
            })
        return out

    def debug_target_logits(self, stream_id: int, tokens):
        import numpy as np

        info = self.package.info
        array = (ctypes.c_uint32 * len(tokens))(*[int(t) for t in tokens])
        logits = np.empty((len(tokens), info["vocab_size"]), dtype=np.float32)
        hidden = np.empty((len(tokens), info["hidden_size"]), dtype=np.uint16)
        _check(library().nerve_b200_debug_target_logits(
            self._handle, ctypes.c_int64(stream_id), array, ctypes.c_size_t(len(tokens)),
            logits.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), hidden.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))))
        return logits, hidden
