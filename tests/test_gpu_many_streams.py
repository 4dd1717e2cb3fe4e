"""The many-stream shape of the batched verify at full layer width: 32 concurrent streams with prompt lengths uniform
in [128, 2048], each generating 128 tokens with MTP k = 4, so that every cycle verifies M = 32 x 5 = 160 candidate
lanes in one batch (the shape BASELINE's 70B configuration names; run here on the 8B INT4 package, whose layers are
the widest the test boxes mount without a 37 GB download-sized synthetic checkpoint).  Batches of this width run
kernel by kernel: the `tcgen05` INT4 GEMM for the linears, the tiled split-K attention with ragged contexts, the
device-side acceptance for 32 streams at once.

No CPU oracle finishes this size; the test checks properties that hold at any size:
  * every stream emits its 128 tokens and ends at prompt + 128 ticks, all 32 streams share every verify batch;
  * the run is deterministic: the same events on fresh streams emit the same tokens;
  * teacher-forced full acceptance: with each stream's own natural tokens forced as its drafts, every draft is
    accepted and the emitted tokens are the natural ones again - the verify lanes of accepted drafts reproduce what
    one-token-at-a-time decoding computed (acceptance, in-place KV commit and catch-up at M = 160).  The comparison
    stops k + 1 tokens before the events' ends, where the two runs' last windows shrink differently and batches of
    fewer than 64 lanes take another kernel.
Synthetic data: seeded N(0, 0.02) weights, prompts uniform over the vocabulary.
"""

import sys
import time
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
STREAMS, DRAFTS, TOKENS = 32, 4, 128


def _run(engine, prompts, teacher=None):
    for i, prompt in enumerate(prompts):
        engine.add_stream(i, speculative_draft_tokens=DRAFTS)
        engine.set_teacher_tokens(i, teacher[i] if teacher else [])
        engine.enqueue_input_event(i, prompt, TOKENS)
    started = time.perf_counter()
    outputs, report = engine.run_until_idle()
    seconds = time.perf_counter() - started
    tokens = [[t for sid, t, _, _ in outputs if sid == i] for i in range(len(prompts))]
    ticks = [engine.stream_tick(i) for i in range(len(prompts))]
    for i in range(len(prompts)):
        engine.remove_stream(i)
    return tokens, ticks, report, seconds


def test_thirty_two_streams_verify_160_lanes_per_cycle():
    import llmoop_b200 as nb

    sys.path.insert(0, str(ROOT))
    import bench

    spec = bench.bench_spec()
    directory = bench.ensure_package(spec, "cuda:0")
    rng = np.random.default_rng(9)
    lengths = [int(n) for n in rng.integers(128, 2049, size=STREAMS)]
    prompts = [[int(t) for t in rng.integers(0, spec.vocab, size=n)] for n in lengths]
    package = nb.Package(directory, capacity_tokens=2048 + TOKENS + 64, page_tokens=16, max_streams=STREAMS, max_lanes=2048, verify_level=0)
    engine = nb.Engine(package)
    engine.set_prefill_chunk(2048)

    natural, ticks, report, seconds = _run(engine, prompts)
    assert all(len(tokens) == TOKENS for tokens in natural)
    assert ticks == [n + TOKENS for n in lengths]
    assert report.max_batch_width == STREAMS
    print("%d streams, k = %d, %d lanes per verify: natural %.0f tokens/s in all (%.1f s, %d cycles)"
          % (STREAMS, DRAFTS, STREAMS * (DRAFTS + 1), STREAMS * TOKENS / seconds, seconds, report.cycle_count))

    again, _, _, _ = _run(engine, prompts)
    assert again == natural

    forced, ticks, report, seconds = _run(engine, prompts, teacher=natural)
    # Compared while both runs verify 160 lanes per cycle: with fewer than k + 1 tokens left the windows shrink, the
    # batches fall below 64 lanes and another kernel (another order of f32 additions) computes the last tokens.
    same_regime = TOKENS - 2 * (DRAFTS + 1)
    mismatches = [(i, next(j for j in range(same_regime) if forced[i][j] != natural[i][j]))
                  for i in range(STREAMS) if forced[i][:same_regime] != natural[i][:same_regime]]
    assert not mismatches, mismatches
    assert all(len(tokens) == TOKENS for tokens in forced)
    assert ticks == [n + TOKENS for n in lengths]
    assert report.accepted_draft_token_count >= 0.9 * report.proposed_draft_token_count > 0
    print("teacher-forced full acceptance: %.0f tokens/s in all (%.1f s, %d cycles)" % (STREAMS * TOKENS / seconds, seconds, report.cycle_count))
    engine.close()
    package.unmount()
