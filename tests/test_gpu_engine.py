"""Parity of the CUDA engine (through the C ABI) against the CPU oracle on the
golden packages: greedy token ids, per-cycle acceptance counts and logits.

Tolerances (stated by the task's north star): token ids and acceptance counts
exact, a divergence being allowed only where the oracle's top-2 logit gap is
below 1e-3; logits max-abs <= 2e-2 and mean-abs <= 2e-3.
"""

import numpy as np
import pytest

from conftest import GOLDEN, PACKAGES

pytestmark = pytest.mark.gpu

GAP_RULE = 1e-3
LOGITS_MAX_ABS = 2e-2
LOGITS_MEAN_ABS = 2e-3


def _oracle(name):
    from oracle.nerve_oracle import Oracle, OraclePackage

    package = OraclePackage(GOLDEN / name)
    return package, Oracle(package)


def _prompt(vocab, count, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=count)]


def _assert_tokens_match(got, expected, oracle_logits, oracle):
    """Exact match, except that the sequences may part at a position where the oracle's top-2 gap < 1e-3
    (after which they are different continuations and cannot be compared)."""
    for index, (a, b) in enumerate(zip(got, expected)):
        if a != b:
            gap = oracle.top2_gap(oracle_logits[index])
            assert gap < GAP_RULE, f"token {index}: cuda {a} != oracle {b} with top-2 gap {gap}"
            return index
    assert len(got) == len(expected)
    return None


@pytest.mark.parametrize("name", PACKAGES)
@pytest.mark.parametrize("drafts", [0, 1, 3])
def test_greedy_generation_matches_oracle(name, drafts):
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    opkg, oracle = _oracle(name)
    prompt = _prompt(opkg.vocab, 16)
    ostream = OracleStream(opkg, 128)
    expected = oracle.generate(ostream, prompt, 32, drafts, collect_logits=True)

    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=64, verify_level=2)
    engine = nb.Engine(package)
    engine.set_cycle_logging(True)
    engine.add_stream(7, seed=0, speculative_draft_tokens=drafts)
    tokens, report = engine.submit_input_event_until_idle(7, prompt, 32)
    diverged = _assert_tokens_match(tokens, expected["tokens"], expected["logits"], oracle)
    if diverged is None:
        assert engine.stream_tick(7) == ostream.next_tick == len(prompt) + 32  # P + N ticks
        cycles = engine.cycle_log()
        assert [c["accepted"] for c in cycles] == [c["accepted"] for c in expected["cycles"]]
        assert [c["committed"] for c in cycles] == [c["committed"] for c in expected["cycles"]]
        assert [c["emitted"] for c in cycles] == [c["emitted"] for c in expected["cycles"]]
        assert report.generated_tokens == 32
        if drafts:
            assert report.cycle_count == len(expected["cycles"])
            assert report.kernel_launches > 0
    engine.close()
    package.unmount()


@pytest.mark.parametrize("name", PACKAGES)
@pytest.mark.parametrize("count", [24, 7])
def test_target_logits_within_tolerance(name, count):
    """24 lanes run kernel by kernel; 7 lanes go through the persistent decode stack kernel where the package's
    layers have its form (the INT4 packages)."""
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    opkg, oracle = _oracle(name)
    tokens = _prompt(opkg.vocab, count, seed=5)
    ostream = OracleStream(opkg, 128)
    _, expected = oracle.target_forward(ostream, tokens, 0, want_logits=True)

    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=1, max_lanes=32)
    engine = nb.Engine(package)
    engine.add_stream(1)
    logits, hidden = engine.debug_target_logits(1, tokens)
    difference = np.abs(logits - expected)
    assert difference.max() <= LOGITS_MAX_ABS, difference.max()
    assert difference.mean() <= LOGITS_MEAN_ABS, difference.mean()
    engine.close()
    package.unmount()


@pytest.mark.parametrize("name", ["tiny_int4_mtp_v16", "tiny_int4_mtp"])
def test_teacher_forced_full_acceptance(name):
    """Feeding the target's own greedy continuation as the draft proposal makes every cycle accept all drafts
    and must not change the emitted tokens."""
    import llmoop_b200 as nb

    opkg, oracle = _oracle(name)
    prompt = _prompt(opkg.vocab, 12, seed=3)
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=64)
    engine = nb.Engine(package)
    engine.add_stream(1, speculative_draft_tokens=0)
    plain, _ = engine.submit_input_event_until_idle(1, prompt, 24)
    engine.add_stream(2, speculative_draft_tokens=3)
    engine.set_teacher_tokens(2, plain)
    engine.set_cycle_logging(True)
    forced, report = engine.submit_input_event_until_idle(2, prompt, 24)
    assert forced == plain
    cycles = engine.cycle_log()
    assert cycles and all(c["accepted"] == len(c["emitted"]) - 1 for c in cycles)
    assert report.accepted_draft_token_count == report.proposed_draft_token_count
    engine.close()
    package.unmount()


def test_stop_token_truncates_and_closes():
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    name = "tiny_int4_mtp_v16"
    opkg, oracle = _oracle(name)
    prompt = _prompt(opkg.vocab, 10, seed=9)
    free_run = oracle.generate(OracleStream(opkg, 128), prompt, 20, 0)["tokens"]
    stop = free_run[5]
    ostream = OracleStream(opkg, 128)
    expected = oracle.generate(ostream, prompt, 20, 3, stop_tokens=[stop])
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=1, max_lanes=32)
    engine = nb.Engine(package)
    engine.add_stream(1, speculative_draft_tokens=3)
    tokens, _ = engine.submit_input_event_until_idle(1, prompt, 20, [stop])
    assert tokens == expected["tokens"]
    assert tokens[-1] == stop and stop not in tokens[:-1]
    assert engine.stream_tick(1) == ostream.next_tick
    engine.close()
    package.unmount()


@pytest.mark.parametrize("streams,decode_stack", [(4, False), (2, True), (2, False)])
def test_multi_stream_batched_verify_matches_single_stream_runs(streams, decode_stack):
    """Several streams decoding together (one batched verify per cycle) must emit what each emits alone.
    Batches of more than 8 lanes run kernel by kernel and smaller ones in the persistent stack kernel, whose
    sums are ordered differently, so each case keeps its batches on one side of that line: 4 streams x 3 lanes
    with the stack kernel off, 2 streams x 3 lanes with it on (and off)."""
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, _ = _oracle(name)
    prompts = [_prompt(opkg.vocab, 5 + i, seed=20 + i) for i in range(streams)]
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=5, max_lanes=64)
    assert package.info["target_decode_stack"] == 1 and package.info["draft_decode_stack"] == 1
    engine = nb.Engine(package)
    engine.set_decode_stack(decode_stack)
    alone = []
    for i, prompt in enumerate(prompts):
        engine.add_stream(100 + i, speculative_draft_tokens=2)
        tokens, _ = engine.submit_input_event_until_idle(100 + i, prompt, 16)
        alone.append(tokens)
        engine.remove_stream(100 + i)
    for i, prompt in enumerate(prompts):
        engine.add_stream(i, speculative_draft_tokens=2)
        engine.enqueue_input_event(i, prompt, 16)
    outputs, report = engine.run_until_idle()
    together = [[t for sid, t, _, _ in outputs if sid == i] for i in range(streams)]
    assert together == alone
    assert report.max_batch_width == streams
    engine.close()
    package.unmount()


def test_fork_shares_prefix_and_diverges_copy_on_write():
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, _ = _oracle(name)
    prefix = _prompt(opkg.vocab, 21, seed=31)  # ends inside a page: the tail page must be copied on write
    tail_a, tail_b = _prompt(opkg.vocab, 5, seed=32), _prompt(opkg.vocab, 7, seed=33)
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=4, max_lanes=64, extra_pages=8)
    engine = nb.Engine(package)
    # references: each branch from scratch
    expected = []
    for i, tail in enumerate((tail_a, tail_b)):
        engine.add_stream(50 + i, speculative_draft_tokens=2)
        tokens, _ = engine.submit_input_event_until_idle(50 + i, prefix + tail, 12)
        expected.append(tokens)
        engine.remove_stream(50 + i)
    # shared prefix, then fork
    engine.add_stream(1, speculative_draft_tokens=2)
    engine.submit_input_event_until_idle(1, prefix, 0)
    engine.fork_stream(1, 2)
    assert engine.stream_tick(2) == engine.stream_tick(1) == len(prefix)
    engine.enqueue_input_event(1, tail_a, 12)
    engine.enqueue_input_event(2, tail_b, 12)
    outputs, _ = engine.run_until_idle()
    got = [[t for sid, t, _, _ in outputs if sid == s] for s in (1, 2)]
    assert got == expected
    engine.close()
    package.unmount()


def test_mount_errors_are_reported_not_fatal(tmp_path):
    import shutil

    import llmoop_b200 as nb

    broken = tmp_path / "broken"
    shutil.copytree(GOLDEN / "tiny_int4_mtp_v16", broken)
    weights = sorted((broken / "weights").glob("*.safetensors"))[0]
    data = bytearray(weights.read_bytes())
    data[-1] ^= 0xFF
    weights.write_bytes(bytes(data))
    with pytest.raises(nb.NerveError, match="sha256"):
        nb.Package(broken, capacity_tokens=64)
    with pytest.raises(nb.NerveError):
        nb.Package(GOLDEN / "tiny_int4_mtp_v16", capacity_tokens=100000)  # beyond max_context_activations


def test_reference_tiny_model_greedy_decode_matches_oracle():
    """The reference's own test fixture (1 layer, hidden 16, head 8, tied lm_head, no MTP decoder)."""
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    name = "reference_tiny_model"
    opkg, oracle = _oracle(name)
    prompt = _prompt(opkg.vocab, 9, seed=4)
    ostream = OracleStream(opkg, 64)
    expected = oracle.generate(ostream, prompt, 20, 0, collect_logits=True)
    package = nb.Package(GOLDEN / name, capacity_tokens=64, page_tokens=16, max_streams=1, max_lanes=16, verify_level=2)
    assert package.info["has_speculative_decoder"] == 0
    engine = nb.Engine(package)
    with pytest.raises(nb.NerveError, match="no mounted speculative decoder"):
        engine.add_stream(9, speculative_draft_tokens=2)
    engine.add_stream(1)
    tokens, _ = engine.submit_input_event_until_idle(1, prompt, 20)
    _assert_tokens_match(tokens, expected["tokens"], expected["logits"], oracle)
    engine.close()
    package.unmount()


@pytest.mark.parametrize("name", ["tiny_int4_mtp", "cfg1_bf16_mtp"])
@pytest.mark.parametrize("drafts", [0, 3])
def test_seeded_sampling_matches_oracle(name, drafts):
    """temperature_top_k_top_p streams: the draft and the target draw with hash(seed ^ tick) at the same tick, so
    speculation stays token-match acceptance (speculative_decode.rs:54-87); tokens and acceptance counts must equal
    the oracle's with the same sampler and seed."""
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    opkg, oracle = _oracle(name)
    sampler = {"method": 1, "top_k": 8, "temperature": 0.9, "top_p": 0.95, "min_p": 0.01}
    seed = 0x5EED1234
    oracle.sampler = dict(sampler, seed=seed)
    prompt = _prompt(opkg.vocab, 12, seed=9)
    ostream = OracleStream(opkg, 128)
    expected = oracle.generate(ostream, prompt, 24, drafts, collect_logits=True)

    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=64)
    engine = nb.Engine(package)
    # A drawn token follows the logits to the last bit (a 1e-2 change of one logit moves a nucleus boundary), so this
    # comparison runs the kernel-per-operator path, which reproduces the oracle's logits exactly on these packages;
    # the persistent stack kernel's sums differ in the last bit now and then and are covered by the test below.
    engine.set_decode_stack(False)
    engine.set_cycle_logging(True)
    engine.add_stream(3, seed=seed, speculative_draft_tokens=drafts, sampler=sampler)
    tokens, report = engine.submit_input_event_until_idle(3, prompt, 24)
    assert len(set(tokens)) > 3  # it does sample: a greedy run of these tiny models repeats itself
    diverged = _assert_tokens_match(tokens, expected["tokens"], expected["logits"], oracle)
    if diverged is None and drafts:
        cycles = engine.cycle_log()
        assert [c["accepted"] for c in cycles] == [c["accepted"] for c in expected["cycles"]]
        assert [c["emitted"] for c in cycles] == [c["emitted"] for c in expected["cycles"]]
    engine.close()
    package.unmount()


@pytest.mark.parametrize("decode_stack", [True, False])
def test_seeded_sampling_is_independent_of_speculation(decode_stack):
    """With a seeded sampler the stream's tokens are a function of (logits, seed, tick) only: drafting k tokens
    ahead and verifying them in one batch must emit exactly what one-token-at-a-time decoding emits, on either
    execution path (here also through the persistent stack kernel: 1-lane ticks against 4-lane verify batches)."""
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, _ = _oracle(name)
    sampler = {"method": 1, "top_k": 8, "temperature": 0.9, "top_p": 0.95, "min_p": 0.01}
    prompt = _prompt(opkg.vocab, 7, seed=13)
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=3, max_lanes=64)
    engine = nb.Engine(package)
    engine.set_decode_stack(decode_stack)
    runs = []
    for stream_id, drafts in ((1, 0), (2, 3), (3, 1)):
        engine.add_stream(stream_id, seed=77, speculative_draft_tokens=drafts, sampler=sampler)
        tokens, report = engine.submit_input_event_until_idle(stream_id, prompt, 28)
        runs.append(tokens)
    assert runs[0] == runs[1] == runs[2]
    assert len(set(runs[0])) > 3
    engine.close()
    package.unmount()


@pytest.mark.parametrize("drafts", [0, 3])
def test_consecutive_events_reset_and_interrupt(drafts):
    """Stream life cycle (placed_prompt_engine.rs:48-589 as used by the chat front end): a second input event
    continues the first one's context; after reset_stream the same events give the same tokens again (state pages
    and the draft's state start over); an interrupted stream drops its queued work and runs again afterwards."""
    import llmoop_b200 as nb
    from oracle.nerve_oracle import OracleStream

    name = "tiny_int4_mtp"
    opkg, oracle = _oracle(name)
    first, second = _prompt(opkg.vocab, 13, seed=41), _prompt(opkg.vocab, 6, seed=42)
    ostream = OracleStream(opkg, 128)
    expected_first = oracle.generate(ostream, first, 9, drafts)["tokens"]
    expected_second = oracle.generate(ostream, second, 11, drafts)["tokens"]

    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=32)
    engine = nb.Engine(package)
    engine.add_stream(7, speculative_draft_tokens=drafts)
    for _ in range(2):
        got_first, _ = engine.submit_input_event_until_idle(7, first, 9)
        ticks_after_first = engine.stream_tick(7)
        got_second, _ = engine.submit_input_event_until_idle(7, second, 11)
        assert got_first == expected_first and got_second == expected_second
        assert ticks_after_first == len(first) + 9 and engine.stream_tick(7) == ticks_after_first + len(second) + 11
        engine.reset_stream_transient_state(7)
        assert engine.stream_tick(7) == 0

    engine.enqueue_input_event(7, first, 9)
    engine.interrupt_stream(7)
    outputs, _ = engine.run_until_idle()
    assert outputs == []
    engine.reset_stream_transient_state(7)
    again, _ = engine.submit_input_event_until_idle(7, first, 9)
    assert again == expected_first
    engine.close()
    package.unmount()


def test_ragged_streams_with_different_draft_counts_budgets_and_stops():
    """Streams that differ in prompt length, draft count (0, 1, 3), output budget (down to one token) and stop
    tokens share an engine: each must emit what it emits alone (the kernel-per-operator path keeps the sums of
    every batch composition identical)."""
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, oracle = _oracle(name)
    cases = [  # prompt length, drafts, budget
        (1, 3, 1), (9, 0, 14), (17, 1, 9), (4, 3, 20), (33, 3, 2),
    ]
    prompts = [_prompt(opkg.vocab, length, seed=60 + i) for i, (length, _, _) in enumerate(cases)]
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=6, max_lanes=64)
    engine = nb.Engine(package)
    engine.set_decode_stack(False)
    alone, stops = [], []
    for i, ((_, drafts, budget), prompt) in enumerate(zip(cases, prompts)):
        engine.add_stream(100 + i, speculative_draft_tokens=drafts)
        tokens, _ = engine.submit_input_event_until_idle(100 + i, prompt, budget)
        engine.remove_stream(100 + i)
        assert 1 <= len(tokens) <= budget
        # the longest run also gets a stop token taken from the middle of its own output
        stop = [tokens[len(tokens) // 2]] if budget == 20 else []
        if stop:
            engine.add_stream(200 + i, speculative_draft_tokens=drafts)
            tokens, _ = engine.submit_input_event_until_idle(200 + i, prompt, budget, stop_token_ids=stop)
            engine.remove_stream(200 + i)
            assert tokens[-1] == stop[0] and stop[0] not in tokens[:-1]
        alone.append(tokens)
        stops.append(stop)
    for i, ((_, drafts, budget), prompt) in enumerate(zip(cases, prompts)):
        engine.add_stream(i, speculative_draft_tokens=drafts)
        engine.enqueue_input_event(i, prompt, budget, stop_token_ids=stops[i])
    outputs, _ = engine.run_until_idle()
    together = [[t for sid, t, _, _ in outputs if sid == i] for i in range(len(cases))]
    assert together == alone
    # and the oracle agrees on the plain greedy case
    from oracle.nerve_oracle import OracleStream

    assert oracle.generate(OracleStream(opkg, 128), prompts[1], 14, 0)["tokens"] == alone[1]
    engine.close()
    package.unmount()


@pytest.mark.parametrize("drafts", [0, 3])
def test_stop_after_current_and_snapshots(drafts):
    """stop_stream_after_current (placed_prompt_engine.rs:307-331): the active event emits nothing more, its last token
    is still fed back (the stream's tick count stays prompt + emitted), queued events are dropped and the stream can
    be used again; snapshots report queue depth, ticks, finished events and mapped pages."""
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, _ = _oracle(name)
    prompt, later = _prompt(opkg.vocab, 10, seed=71), _prompt(opkg.vocab, 4, seed=72)
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=32)
    engine = nb.Engine(package)
    engine.add_stream(3, speculative_draft_tokens=drafts)
    full, _ = engine.submit_input_event_until_idle(3, prompt, 20)
    engine.reset_stream_transient_state(3)
    assert engine.snapshot() == {"stream_count": 1, "active_stream_count": 0, "idle": True}

    engine.enqueue_input_event(3, prompt, 20)
    engine.enqueue_input_event(3, later, 5)
    before = engine.stream_snapshot(3)
    assert before["pending_input_event_count"] == 2 and not before["idle"] and before["next_stream_tick"] == 0
    assert engine.snapshot()["active_stream_count"] == 1
    first, _ = engine.run(1)   # prompt chunk and the first decode batch
    got = [token for sid, token, _, _ in first if sid == 3]
    assert 1 <= len(got) < 20 and got == full[: len(got)]
    engine.stop_stream_after_current(3)
    rest, _ = engine.run_until_idle()
    assert [t for sid, t, _, _ in rest if sid == 3] == []          # nothing more is emitted, the queued event is gone
    after = engine.stream_snapshot(3)
    assert after["idle"] and after["pending_input_event_count"] == 0 and after["completed_prompt_event_count"] == 2
    assert after["next_stream_tick"] == len(prompt) + len(got)      # the last token was fed back: P + N ticks
    assert after["mapped_state_pages"] == (after["next_stream_tick"] + 15) // 16
    assert after["speculative_draft_tokens"] == drafts and after["context_window_activations"] == 128
    # the state is complete: continuing from here equals continuing an uninterrupted run of the same length
    engine.add_stream(4, speculative_draft_tokens=drafts)
    engine.submit_input_event_until_idle(4, prompt, len(got))
    expected, _ = engine.submit_input_event_until_idle(4, later, 6)
    continued, _ = engine.submit_input_event_until_idle(3, later, 6)
    assert continued == expected
    engine.stop_stream_after_current(3)                             # idle stream: no effect
    assert engine.stream_snapshot(3)["idle"]
    engine.close()
    package.unmount()


def test_engine_runs_what_the_scheduler_schedules():
    """The engine owns a runtime scheduler (placed_prompt_engine.rs:455-520) and executes its activations: prompt
    chunks of the configured length, then decode windows of k + 1 tokens; every outcome is reported back, so the
    scheduler's counters follow the event exactly, also across a fork and a dropped event."""
    import llmoop_b200 as nb

    name = "tiny_int4_mtp"
    opkg, _ = _oracle(name)
    prompt = _prompt(opkg.vocab, 40, seed=91)
    package = nb.Package(GOLDEN / name, capacity_tokens=128, page_tokens=16, max_streams=3, max_lanes=32)
    engine = nb.Engine(package)
    engine.set_prefill_chunk(16)
    engine.add_stream(1, speculative_draft_tokens=3)
    engine.enqueue_input_event(1, prompt, 9)
    queued = engine.scheduler_stream_counts(1)
    assert queued["queued_input_event_count"] == 1 and queued["scheduled_activation_count"] == 0
    outputs, report = engine.run_until_idle()
    assert len(outputs) == 9
    counts = engine.scheduler_stream_counts(1)
    # 40 prompt tokens in chunks of 16 -> 3 prefill activations (the last one samples the first token), then decode
    # windows until the 9 tokens are out: one activation per speculative cycle
    assert counts["completed_input_event_count"] == 1 and counts["generated_token_count"] == 9
    assert counts["in_flight_activation_count"] == 0 and counts["has_current_input_event"] == 0 and counts["queued_input_event_count"] == 0
    # (8 tokens after the first: between two full windows of four and eight windows of one accepted token)
    assert 3 + 2 <= counts["scheduled_activation_count"] <= 3 + 8
    assert counts["scheduled_activation_count"] >= 3 + report.cycle_count  # + single ticks when one token is left
    assert engine.stream_tick(1) == 40 + 9
    # a fork starts with its own (empty) scheduler entry and takes events of its own
    engine.fork_stream(1, 2)
    assert engine.scheduler_stream_counts(2)["scheduled_activation_count"] == 0
    engine.enqueue_input_event(2, prompt[:3], 2)
    engine.enqueue_input_event(1, prompt[:5], 4)
    engine.interrupt_stream(1)                       # the event is dropped before it ran
    outputs, _ = engine.run_until_idle()
    assert [sid for sid, _, _, _ in outputs] == [2, 2]
    assert engine.scheduler_stream_counts(1)["queued_input_event_count"] == 0
    assert engine.scheduler_stream_counts(2)["generated_token_count"] == 2
    engine.close()
    package.unmount()
