"""A kernel-side failure made without a fault: the persistent decode kernel is told to wait at its first grid barrier
for arrivals that cannot come; its bounded wait gives up, the kernel reports it, and the engine must discard the
batch - no token emitted, stream ticks unchanged, pending hidden states restored - fail the call, and stay usable:
the same event run again afterwards equals the oracle's.  (Reference: a failed speculative cycle restores the state
snapshot, placed_stream_processor/feedback_generation.rs:188-192.)"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def package_dir(tmp_path_factory):
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec

    spec = ModelSpec(name="failure_injection", hidden=512, layers=3, q_heads=8, kv_heads=2, head_dim=64, ffn=1408, vocab=1024,
                     max_positions=512, quant="int4", std=0.01, seed=7)
    directory = tmp_path_factory.mktemp("packages") / spec.name
    write_package(spec, directory)
    return directory, spec


@pytest.mark.parametrize("drafts", [3, 0], ids=["speculative_cycle", "single_tick"])
def test_barrier_timeout_discards_the_batch_and_the_engine_recovers(package_dir, drafts):
    import llmoop_b200 as nb
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream
    from oracle.parity import follow_generation

    directory, spec = package_dir
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, spec.vocab, size=6)]
    package = nb.Package(directory, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=64, verify_level=0)
    assert package.info["target_decode_stack"] == 1
    engine = nb.Engine(package)
    engine.set_decode_stack(True)
    engine.set_cycle_logging(True)
    engine.add_stream(3, speculative_draft_tokens=drafts)
    engine.enqueue_input_event(3, prompt, 16)
    first, _ = engine.run(2)                       # the prompt and two decode batches
    emitted_before = len(first)
    tick_before = engine.stream_tick(3)
    assert emitted_before >= 2

    engine.inject_barrier_timeouts(1)
    seen = []
    with pytest.raises(nb.NerveError, match="gave up waiting at a grid barrier"):
        engine.run(1, on_output=lambda *event: seen.append(event))
    assert seen == []                               # nothing of the failed batch was emitted
    assert engine.stream_tick(3) == tick_before     # ... nor committed

    rest, report = engine.run_until_idle()          # the same batch again, and the rest of the event
    tokens = [token for _, token, _, _ in first] + [token for _, token, _, _ in rest]
    assert len(tokens) == 16
    opkg = OraclePackage(directory)
    outcome = follow_generation(Oracle(opkg), OracleStream(opkg, 128), prompt, tokens, engine.cycle_log(), drafts)
    assert outcome["tokens_compared"] == 16 and not outcome["violations"] and outcome["accepted_equal"], outcome
    engine.close()
    package.unmount()
