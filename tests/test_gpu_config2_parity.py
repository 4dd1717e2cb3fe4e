"""BASELINE config 2 end to end: the Llama-3-8B-shaped INT4 g128 + MTP package (32 layers, hidden 4096, vocab 128256,
synthetic N(0, 0.02) weights) mounted on the GPU and compared with the CPU oracle on the same package - target
logits of a 4-lane verify batch, then tokens and per-cycle acceptance of a short speculative event followed by
oracle/parity.py.  The oracle needs about 1.2 s per cycle here, so the event is short (16-token prompt).

What can be asserted here: 32 layers of random (untrained) weights amplify a single bf16 rounding of the hidden
state, so any two f32 summation orders of this model - the oracle, the kernel-per-operator path, the persistent
kernel - differ mutually by a few 1e-2 in a logit (logits reach +-6), far above the north star's absolute bars,
which the smaller packages of the other tests meet.  The test therefore checks that the persistent kernel is as close
to the oracle as the kernel-per-operator path is (the one whose operators are bit-checked against the oracle one by
one), that per-cycle acceptance bookkeeping follows the oracle after every divergence, and that a token divergence
only happens at a near-tie on the scale of the logit differences actually measured (gap < 2 x the largest one)."""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def config2_package():
    sys.path.insert(0, str(ROOT))
    import bench

    spec = bench.bench_spec()
    directory = bench.ensure_package(spec, "cuda:0")
    return directory, spec


def test_config2_logits_and_short_event_follow_the_oracle(config2_package):
    import llmoop_b200 as nb
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream
    from oracle.parity import follow_generation, summary

    directory, spec = config2_package
    try:
        import ctypes

        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(os.cpu_count() or 1)
    except OSError:
        pass
    opkg = OraclePackage(directory)
    oracle = Oracle(opkg)
    rng = np.random.default_rng(0)
    prompt = [int(t) for t in rng.integers(0, spec.vocab, size=16)]
    probe = [int(t) for t in rng.integers(0, spec.vocab, size=4)]

    package = nb.Package(directory, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=32, verify_level=0)
    assert package.info["target_decode_stack"] == 1
    engine = nb.Engine(package)
    engine.set_decode_stack(True)
    engine.add_stream(1, speculative_draft_tokens=3)
    engine.submit_input_event_until_idle(1, prompt, 0)
    logits, _ = engine.debug_target_logits(1, probe)
    engine.set_decode_stack(False)
    plain, _ = engine.debug_target_logits(1, probe)
    engine.set_decode_stack(True)

    ostream = OracleStream(opkg, 128)
    oracle.target_forward(ostream, prompt, 0, want_logits=False)
    _, expected = oracle.target_forward(ostream, probe, len(prompt), want_logits=True)
    scale = float(np.abs(expected).max())
    stack_difference, plain_difference = np.abs(logits - expected), np.abs(plain - expected)
    print(f"config 2 logits vs oracle: largest |logit| {scale:.2f}; stack kernel max {stack_difference.max():.3e} mean {stack_difference.mean():.3e}; "
          f"kernel per operator max {plain_difference.max():.3e} mean {plain_difference.mean():.3e}")
    mutual = np.abs(logits - plain)
    print(f"config 2 logits, persistent kernel vs kernel per operator: max {mutual.max():.3e} mean {mutual.mean():.3e}")
    assert stack_difference.mean() <= 1.25 * plain_difference.mean() + 1e-4
    assert stack_difference.max() <= 1.5 * plain_difference.max() + 1e-3

    engine.reset_stream_transient_state(1)
    engine.set_cycle_logging(True)
    tokens, report = engine.submit_input_event_until_idle(1, prompt, 12)
    cycles = engine.cycle_log()
    outcome = follow_generation(oracle, OracleStream(opkg, 128), prompt, tokens, cycles, 3, prefill_chunk=16)
    print("config 2 short event:", summary(outcome), outcome["divergences"])
    assert outcome["tokens_compared"] == len(tokens) == 12 and outcome["accepted_equal"]
    # a divergence is a near-tie on the scale of this model's measured logit differences
    assert all(entry["gap"] < 2.0 * float(stack_difference.max()) for entry in outcome["divergences"]), outcome["divergences"]
    engine.close()
    package.unmount()
