"""The long-context configuration: one 8B INT4 stream with a 32768-token prompt, prefilled in 2048-token chunks into
paged bf16 KV (16-token pages); a prefix fork at 16384 tokens creates a second stream that shares those pages; both
streams then decode greedily with MTP k = 3 in one batch (ragged contexts of 32K and 16K tokens, eight verify lanes,
every rejected draft rolled back in place).

No CPU oracle finishes this size, so the full-size test checks properties that hold at any size:
  * the fork decodes exactly what a stream that was given the same 16385 tokens without any fork decodes;
  * the forked-from stream, decoding next to the fork, emits exactly what a stream that prefilled the whole prompt
    alone and decodes WITHOUT speculation emits (fork isolation: copy on write; rollback: a rejected draft leaves no
    trace in the KV ring; batching: a lane's result does not depend on its neighbours);
  * the fork maps the prefix pages of its source instead of new ones.
The same scenario scaled down to the tiny INT4 package is followed by the oracle token by token, with the 1e-3 rule.
Synthetic data: seeded N(0, 0.02) weights, prompt uniform over the vocabulary.
"""

import sys
import time
from pathlib import Path

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _scenario(engine, prompt, fork_at, drafts, decode_tokens):
    """Stream 1 takes prompt[:fork_at], is forked into stream 2, takes the rest of the prompt; then both decode.
    Returns (tokens of 1, tokens of 2, mapped pages of 1 and 2 right after the fork)."""
    engine.add_stream(1, speculative_draft_tokens=drafts)
    engine.submit_input_event_until_idle(1, prompt[:fork_at], 0)
    engine.fork_stream(1, 2)
    assert engine.stream_tick(1) == engine.stream_tick(2) == fork_at
    mapped = (engine.stream_snapshot(1)["mapped_state_pages"], engine.stream_snapshot(2)["mapped_state_pages"])
    engine.submit_input_event_until_idle(1, prompt[fork_at:-1], 0)
    engine.enqueue_input_event(1, prompt[-1:], decode_tokens)
    engine.enqueue_input_event(2, prompt[fork_at:fork_at + 1], decode_tokens)
    outputs, _ = engine.run_until_idle()
    return [t for sid, t, _, _ in outputs if sid == 1], [t for sid, t, _, _ in outputs if sid == 2], mapped


def test_config_long_context_prefix_fork_properties():
    import llmoop_b200 as nb

    sys.path.insert(0, str(ROOT))
    import bench

    spec = bench.bench_spec()
    directory = bench.ensure_package(spec, "cuda:0")
    prompt_tokens, fork_at, drafts, decode_tokens, compared = 32768, 16384, 3, 512, 128
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, spec.vocab, size=prompt_tokens)]
    package = nb.Package(directory, capacity_tokens=prompt_tokens + 1024, page_tokens=16, max_streams=2, max_lanes=2048, verify_level=0)
    engine = nb.Engine(package)
    engine.set_decode_stack(True)
    engine.set_prefill_chunk(2048)

    started = time.perf_counter()
    tokens_a, tokens_b, mapped = _scenario(engine, prompt, fork_at, drafts, decode_tokens)
    elapsed = time.perf_counter() - started
    print("32768-token prompt, fork at 16384, 2 x %d tokens with k = %d: %.1f s in all" % (decode_tokens, drafts, elapsed))
    assert len(tokens_a) == decode_tokens and len(tokens_b) == decode_tokens
    assert mapped[0] == mapped[1] == fork_at // 16  # the fork maps its source's pages
    assert engine.stream_tick(1) == prompt_tokens + decode_tokens and engine.stream_tick(2) == fork_at + 1 + decode_tokens

    # the fork against a stream that never was one
    engine.remove_stream(2)
    engine.add_stream(3, speculative_draft_tokens=drafts)
    engine.submit_input_event_until_idle(3, prompt[:fork_at], 0)
    tokens_c, _ = engine.submit_input_event_until_idle(3, prompt[fork_at:fork_at + 1], compared)
    assert tokens_c == tokens_b[:compared]

    # the long stream against one that ran alone and without speculation
    engine.remove_stream(1)
    engine.remove_stream(3)
    engine.add_stream(4, speculative_draft_tokens=0)
    engine.submit_input_event_until_idle(4, prompt[:-1], 0)
    tokens_d, _ = engine.submit_input_event_until_idle(4, prompt[-1:], compared)
    assert tokens_d == tokens_a[:compared]
    engine.close()
    package.unmount()


def test_scaled_down_prefix_fork_follows_the_oracle():
    import llmoop_b200 as nb
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream
    from oracle.parity import follow_generation, summary

    name, prompt_tokens, fork_at, drafts, decode_tokens = "tiny_int4_mtp", 96, 48, 3, 24
    opkg = OraclePackage(GOLDEN / name)
    oracle = Oracle(opkg)
    prompt = [int(t) for t in np.random.default_rng(11).integers(0, opkg.vocab, size=prompt_tokens)]
    package = nb.Package(GOLDEN / name, capacity_tokens=256, page_tokens=16, max_streams=2, max_lanes=64)
    engine = nb.Engine(package)
    engine.set_prefill_chunk(32)
    engine.set_cycle_logging(True)
    tokens_a, tokens_b, mapped = _scenario(engine, prompt, fork_at, drafts, decode_tokens)
    cycles = engine.cycle_log()
    assert mapped[0] == mapped[1] == fork_at // 16
    for stream_id, tokens, seen in ((1, tokens_a, prompt), (2, tokens_b, prompt[:fork_at + 1])):
        mine = [c for c in cycles if c["stream_id"] == stream_id]
        outcome = follow_generation(oracle, OracleStream(opkg, 256), seen, tokens, mine, drafts, prefill_chunk=32)
        print("stream", stream_id, summary(outcome), outcome["divergences"])
        assert outcome["tokens_compared"] == len(tokens) == decode_tokens and not outcome["violations"], outcome["violations"]
        assert outcome["accepted_equal"], outcome["divergences"]
    engine.close()
    package.unmount()
