"""Scheduler and transient-state arena (host code, no GPU).

1. tests/stream_runtime_cases.cpp holds one case per scenario that the reference's own unit tests pin
   (runtime-rs/src/stream_state.rs:761-985, runtime-rs/src/stream_runtime_tests.rs); it is compiled here with g++
   against llmoop_b200/csrc/stream_runtime.cpp and every case is run.
2. The same unit through the C ABI of libnerve_b200.so (ctypes): a stream with a KV state is driven through
   prefill chunks, a speculative decode window that commits fewer ticks than it reserved, a fork and an interrupt.
"""

import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def cases_binary(tmp_path_factory):
    out = tmp_path_factory.mktemp("stream_runtime") / "stream_runtime_cases"
    command = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", str(ROOT / "tests" / "stream_runtime_cases.cpp"),
               str(ROOT / "llmoop_b200" / "csrc" / "stream_runtime.cpp"), "-o", str(out)]
    result = subprocess.run(command, capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    return out


def test_reference_pinned_cases_all_pass(cases_binary):
    names = subprocess.run([str(cases_binary), "--list"], capture_output=True, text=True, check=True).stdout.split()
    assert len(names) >= 50
    result = subprocess.run([str(cases_binary)], capture_output=True, text=True)
    lines = result.stdout.strip().splitlines()
    failed = [line for line in lines if not line.startswith("ok ")]
    assert result.returncode == 0 and not failed, "\n".join(failed)
    assert [line[3:] for line in lines] == names


def test_cases_are_clean_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The scheduler, the arena and the prefix cache are plain host code: every case again in a build instrumented
    by ASan and UBSan (leaks, out-of-bounds and use-after-free accesses, signed overflow, misaligned or null
    dereferences abort the run)."""
    out = tmp_path / "stream_runtime_cases_sanitized"
    command = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
               str(ROOT / "tests" / "stream_runtime_cases.cpp"), str(ROOT / "llmoop_b200" / "csrc" / "stream_runtime.cpp"), "-o", str(out)]
    built = subprocess.run(command, capture_output=True, text=True)
    if built.returncode != 0 and "sanitize" in built.stderr and ("cannot find" in built.stderr or "unrecognized" in built.stderr):
        pytest.skip("the sanitizer runtimes are not installed")
    assert built.returncode == 0, built.stdout + built.stderr
    result = subprocess.run([str(out)], capture_output=True, text=True)
    failed = [line for line in result.stdout.strip().splitlines() if not line.startswith("ok ")]
    assert result.returncode == 0 and not failed and not result.stderr.strip(), "\n".join(failed) + result.stderr[-2000:]


def test_unknown_case_name_is_an_error(cases_binary):
    result = subprocess.run([str(cases_binary), "no_such_case"], capture_output=True, text=True)
    assert result.returncode != 0


def test_scheduler_through_the_c_abi():
    from llmoop_b200.runtime import NerveError
    from llmoop_b200.scheduler import Budget, Scheduler, StateDeclaration

    scheduler = Scheduler()
    kv = StateDeclaration("layer_00", "kv_memory", bytes_per_activation=4096, activation_capacity=16)
    added = scheduler.add_stream("stream_a", "package_x", [kv])
    assert added["status"] == "idle" and added["transient_state_entry_count"] == 1
    with pytest.raises(NerveError, match="already exists"):
        scheduler.add_stream("stream_a")

    prompt = list(range(100, 140))  # 40 tokens: chunks end at the 16-token page boundaries, 16 + 16 + 8
    scheduler.enqueue_input_event("stream_a", "event_0", prompt, max_public_tokens=12)
    budget = Budget(max_activations=4, max_prefill_tokens_per_activation=64, max_work_units=256, max_decode_tokens_per_activation=4)
    chunks = []
    while True:
        step = scheduler.schedule_step(budget)
        activation = step["activations"][0]
        if activation.kind != "prefill_chunk":
            break
        chunks.append((activation.token_offset, len(activation.token_ids), activation.remaining_prompt_token_count))
        assert activation.token_ids == prompt[activation.token_offset : activation.token_offset + len(activation.token_ids)]
        assert activation.execution_class_id == "package_x" and activation.input_event_id == "event_0"
        slots = activation.state_reservations[0]["slots"]
        assert activation.state_reservations[0]["key"] == ("layer_00", "kv_memory")
        # the chunk that ends the prompt also reserves the first feedback tick
        assert len(slots) == len(activation.token_ids) + (1 if activation.remaining_prompt_token_count == 0 else 0)
        assert [slot["logical_activation_index"] for slot in slots] == list(range(activation.token_offset, activation.token_offset + len(slots)))
        scheduler.complete_activation(activation.id)
    assert chunks == [(0, 16, 24), (16, 16, 8), (32, 8, 0)]

    # a speculative window of 4 that commits only 2 ticks: the other reserved slots are given back
    assert activation.kind == "decode_feedback" and activation.feedback_depth == 0 and activation.max_tokens == 4
    assert len(activation.state_reservations[0]["slots"]) == 5
    assert scheduler.stream_snapshot("stream_a")["transient_state_logical_activation_count"] == 45
    done = scheduler.complete_activation(activation.id, [7, 8], True, processed_state_activation_count=2)
    assert done["generated_token_count"] == 2 and done["transient_state_logical_activation_count"] == 42
    with pytest.raises(NerveError, match="unknown in-flight activation"):
        scheduler.complete_activation(activation.id, [1])

    forked = scheduler.fork_stream_transient_state("stream_a", "stream_b", "package_x")
    assert forked["transient_state_block_count"] == 3 and forked["status"] == "idle"
    counts = scheduler.snapshot()
    assert counts["stream_count"] == 2 and counts["live_block_count"] == 3  # shared, not copied

    # whoever writes the shared, partly filled page first gets a private copy of it; the other then owns the original
    scheduler.enqueue_input_event("stream_b", "event_b", [1, 2], 0)
    step = scheduler.schedule_step(budget)
    by_stream = {a.stream_id: a for a in step["activations"]}
    assert set(by_stream) == {"stream_a", "stream_b"}
    assert [a.stream_id for a in step["activations"]] == ["stream_a", "stream_b"]  # the stream in the middle of an event goes first
    first_a = by_stream["stream_a"].state_reservations[0]["slots"][0]
    first_b = by_stream["stream_b"].state_reservations[0]["slots"][0]
    assert first_a["block_activation_offset"] == first_b["block_activation_offset"] == 42 % 16
    assert first_a["allocated_block"] and first_a["copy_from_block_id"] == first_b["block_id"]
    assert not first_b["allocated_block"] and first_b["copy_from_block_id"] is None

    interrupted = scheduler.interrupt_stream("stream_b", "cancel")
    assert interrupted["status"] == "interrupted" and interrupted["transient_state_logical_activation_count"] == 42
    assert interrupted["in_flight_activation_count"] == 0
    with pytest.raises(NerveError, match="while activations are in flight"):
        scheduler.remove_stream("stream_a")
    scheduler.complete_activation(by_stream["stream_a"].id, [9], False)
    assert scheduler.stream_snapshot("stream_a")["status"] == "idle"
    scheduler.remove_stream("stream_a")
    scheduler.remove_stream("stream_b")
    counts = scheduler.snapshot()
    assert counts["stream_count"] == 0 and counts["live_block_count"] == 0 and counts["free_block_count"] == counts["allocated_block_count"]
    scheduler.close()


def test_prefix_state_cache_through_the_c_abi():
    """The scenario of stream_runtime_tests.rs:665-769 (two sources, the longer retained prefix wins), extended by
    the capacity rule, through the C ABI."""
    from llmoop_b200.runtime import NerveError
    from llmoop_b200.scheduler import Budget, Scheduler, StateDeclaration

    scheduler = Scheduler()
    kv = StateDeclaration("layer_00", "kv_memory", bytes_per_activation=16, activation_capacity=2)
    budget = Budget(max_activations=1, max_prefill_tokens_per_activation=2, max_work_units=16)

    def prefill(stream_id, tokens):
        scheduler.add_stream(stream_id, "package_a", [kv])
        scheduler.enqueue_input_event(stream_id, "event", tokens, max_public_tokens=0)
        while scheduler.stream_snapshot(stream_id)["status"] != "idle":
            scheduler.complete_activation(scheduler.schedule_step(budget)["activations"][0].id)

    assert scheduler.prefix_state_cache_counts() == {"capacity_entries": 0, "entry_count": 0, "eviction_count": 0}
    prefill("short_source", [1, 2])
    # capacity 0 retains nothing (stream_prefix_cache.rs:155-160)
    scheduler.cache_stream_prefix_state_for_tokens("short_source", "graph_a", [1, 2], b"reasoning=true")
    assert scheduler.prefix_state_cache_counts()["entry_count"] == 0
    assert scheduler.set_prefix_state_cache_capacity(2) == 0

    prefill("long_source", [1, 2, 3, 4])
    assert scheduler.cache_stream_prefix_state_for_tokens("short_source", "graph_a", [1, 2], b"reasoning=true") == {"replaced_existing": False, "evicted_count": 0}
    assert scheduler.cache_stream_prefix_state_for_tokens("long_source", "graph_a", [1, 2, 3, 4], b"reasoning=true")["evicted_count"] == 0
    assert scheduler.cache_stream_prefix_state_for_tokens("long_source", "graph_a", [1, 2, 3, 4], b"reasoning=true")["replaced_existing"]
    with pytest.raises(NerveError, match="does not match source state"):
        scheduler.cache_stream_prefix_state_for_tokens("long_source", "graph_a", [1, 2], b"reasoning=true")
    live_before = scheduler.snapshot()["live_block_count"]

    scheduler.add_stream("target", "package_a", [kv])
    assert scheduler.restore_longest_stream_prefix_state("target", "graph_a", [1, 2, 3, 4, 5], b"reasoning=false") == 0
    assert scheduler.restore_longest_stream_prefix_state("target", "graph_b", [1, 2, 3, 4, 5], b"reasoning=true") == 0
    assert scheduler.restore_longest_stream_prefix_state("target", "graph_a", [1, 2, 3, 4, 5], b"reasoning=true") == 4
    restored = scheduler.stream_snapshot("target")
    assert restored["transient_state_logical_activation_count"] == 4 and restored["transient_state_block_count"] == 2
    assert scheduler.snapshot()["live_block_count"] == live_before  # shared, not copied
    with pytest.raises(NerveError, match="cannot replace non-empty transient state"):
        scheduler.restore_longest_stream_prefix_state("target", "graph_a", [1, 2, 9], b"reasoning=true")

    # the sources go; what the cache retains stays alive until the capacity drops
    for stream_id in ("short_source", "long_source"):
        scheduler.remove_stream(stream_id)
    assert scheduler.snapshot()["live_block_count"] == live_before
    assert scheduler.set_prefix_state_cache_capacity(0) == 2
    assert scheduler.prefix_state_cache_counts() == {"capacity_entries": 0, "entry_count": 0, "eviction_count": 2}
    assert scheduler.snapshot()["live_block_count"] == 2  # the target's two blocks
