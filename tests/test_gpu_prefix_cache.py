"""Prefix-state cache of the engine (reference: stream_prefix_cache.rs:104-312, placed_prefix_state_cache.rs:50-365,
placed_prompt_engine.rs:190-280 and 964-1060): a prompt's state at its last page boundary is retained under the
tokens that produced it, and a fresh stream whose prompt begins with those tokens starts from it.

The oracle knows nothing of the cache, so a stream that started from a retained prefix must emit what the oracle
emits for the whole prompt: token ids exact, a divergence allowed only where the oracle's top-2 gap is below 1e-3.
The bookkeeping (hits, misses, reused tokens, prefilled tokens, ticks) is exact.
"""

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

GAP_RULE = 1e-3
NAME = "tiny_int4_mtp"
PAGE = 16


def _tokens(vocab, count, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=count)]


def _expected(opkg, oracle, prompt, count, drafts):
    from oracle.nerve_oracle import OracleStream

    return oracle.generate(OracleStream(opkg, 128), prompt, count, drafts, collect_logits=True)


def _assert_follows_oracle(got, expected, oracle):
    for index, (a, b) in enumerate(zip(got, expected["tokens"])):
        if a != b:
            gap = oracle.top2_gap(expected["logits"][index])
            assert gap < GAP_RULE, f"token {index}: cuda {a} != oracle {b} with top-2 gap {gap}"
            return
    assert len(got) == len(expected["tokens"])


def test_prefix_cache_restores_the_longest_retained_prefix():
    import llmoop_b200 as nb
    from oracle.nerve_oracle import Oracle, OraclePackage

    opkg = OraclePackage(GOLDEN / NAME)
    oracle = Oracle(opkg)
    shared = _tokens(opkg.vocab, 37, 41)
    prompt_a = shared + _tokens(opkg.vocab, 3, 42)  # 40 tokens: retained at tick 32
    prompt_b = shared + _tokens(opkg.vocab, 9, 43)  # 46 tokens, the first 37 as in prompt_a: starts at tick 32
    prompt_c = _tokens(opkg.vocab, 30, 44)          # nothing in common: a miss, retained at tick 16

    package = nb.Package(GOLDEN / NAME, capacity_tokens=128, page_tokens=PAGE, max_streams=4, max_lanes=64, extra_pages=16)
    engine = nb.Engine(package)
    assert engine.prefix_cache_stats()["resident_entry_count"] == 0

    # off by default: nothing is retained, nothing is looked up
    engine.add_stream(9, speculative_draft_tokens=2)
    plain, report = engine.submit_input_event_until_idle(9, prompt_a, 12)
    assert report.prefill_tokens == len(prompt_a)
    assert engine.prefix_cache_stats() == dict.fromkeys(engine.prefix_cache_stats(), 0)
    engine.remove_stream(9)
    _assert_follows_oracle(plain, _expected(opkg, oracle, prompt_a, 12, 2), oracle)

    engine.set_prefix_cache_capacity(4)
    engine.add_stream(1, speculative_draft_tokens=2)
    tokens_a, report = engine.submit_input_event_until_idle(1, prompt_a, 12)
    _assert_follows_oracle(tokens_a, _expected(opkg, oracle, prompt_a, 12, 2), oracle)
    assert report.prefill_tokens == len(prompt_a) and engine.stream_tick(1) == len(prompt_a) + 12
    stats = engine.prefix_cache_stats()
    assert (stats["miss_count"], stats["hit_count"], stats["insertion_count"], stats["resident_entry_count"]) == (1, 0, 1, 1)
    assert stats["resident_byte_count"] > 0
    engine.remove_stream(1)  # the retained pages outlive the stream that wrote them

    engine.add_stream(2, speculative_draft_tokens=2)
    tokens_b, report = engine.submit_input_event_until_idle(2, prompt_b, 12)
    _assert_follows_oracle(tokens_b, _expected(opkg, oracle, prompt_b, 12, 2), oracle)
    assert report.prefill_tokens == len(prompt_b) - 2 * PAGE  # the first two pages came from the cache
    assert engine.stream_tick(2) == len(prompt_b) + 12
    stats = engine.prefix_cache_stats()
    assert (stats["miss_count"], stats["hit_count"], stats["reused_token_count"], stats["saved_prefill_token_count"]) == (1, 1, 2 * PAGE, 2 * PAGE)
    assert stats["insertion_count"] == 1  # prompt_b's last page boundary is the one it started from

    engine.add_stream(3, speculative_draft_tokens=2)
    tokens_c, report = engine.submit_input_event_until_idle(3, prompt_c, 12)
    _assert_follows_oracle(tokens_c, _expected(opkg, oracle, prompt_c, 12, 2), oracle)
    assert report.prefill_tokens == len(prompt_c)
    stats = engine.prefix_cache_stats()
    assert (stats["miss_count"], stats["hit_count"], stats["insertion_count"], stats["resident_entry_count"]) == (2, 1, 2, 2)

    # another draft count is another runtime modifier: the retained state is not offered
    engine.add_stream(4, speculative_draft_tokens=0)
    tokens_d, report = engine.submit_input_event_until_idle(4, prompt_b, 6)
    _assert_follows_oracle(tokens_d, _expected(opkg, oracle, prompt_b, 6, 0), oracle)
    assert report.prefill_tokens == len(prompt_b)
    stats = engine.prefix_cache_stats()
    assert (stats["miss_count"], stats["hit_count"], stats["insertion_count"], stats["resident_entry_count"]) == (3, 1, 3, 3)

    # a second stream on the same retained prefix while the first one still holds it: both go on, copy-on-write
    engine.reset_stream_transient_state(3)
    tokens_e, report = engine.submit_input_event_until_idle(3, prompt_b, 12)
    assert tokens_e == tokens_b and report.prefill_tokens == len(prompt_b) - 2 * PAGE
    assert engine.prefix_cache_stats()["hit_count"] == 2

    engine.set_prefix_cache_capacity(0)
    stats = engine.prefix_cache_stats()
    assert stats["resident_entry_count"] == 0 and stats["resident_byte_count"] == 0
    # the streams that started from the dropped entries keep their pages
    more, _ = engine.submit_input_event_until_idle(2, _tokens(opkg.vocab, 3, 45), 4)
    assert len(more) == 4
    engine.close()
    package.unmount()
