"""oracle/parity.py on the CPU: the oracle following its own run reports no divergence; following a run with one
token changed reports exactly that divergence (a violation, since the oracle's logits are no near-tie there) and
still compares every later cycle."""

from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden" / "packages"


def _run(drafts):
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream

    package = OraclePackage(GOLDEN / "tiny_int4_mtp_v16")
    oracle = Oracle(package)
    prompt = [int(t) for t in np.random.default_rng(1).integers(0, 16, size=9)]
    expected = oracle.generate(OracleStream(package, 128), prompt, 14, drafts)
    cycles = [{"accepted": c["accepted"], "committed": c["committed"], "emitted": c["emitted"], "target_token_ids": c["target_token_ids"]}
              for c in expected["cycles"]]
    return package, oracle, prompt, expected["tokens"], cycles


@pytest.mark.parametrize("drafts", [0, 3])
def test_following_its_own_run_finds_no_divergence(drafts):
    from oracle.nerve_oracle import OracleStream
    from oracle.parity import follow_generation, summary

    package, oracle, prompt, tokens, cycles = _run(drafts)
    report = follow_generation(oracle, OracleStream(package, 128), prompt, tokens, cycles, drafts)
    assert report["tokens_equal"] and report["accepted_equal"] and not report["divergences"]
    assert report["tokens_compared"] == len(tokens) and report["cycles_compared"] == len(cycles)
    assert summary(report)["violations"] == 0


def test_a_changed_target_token_is_reported_and_the_comparison_goes_on():
    from oracle.nerve_oracle import OracleStream
    from oracle.parity import follow_generation

    package, oracle, prompt, tokens, cycles = _run(3)
    # pretend the other implementation chose another target token in the second cycle
    changed = cycles[1]
    wrong = (changed["target_token_ids"][0] + 1) % package.vocab
    changed["target_token_ids"] = [wrong] + list(changed["target_token_ids"][1:])
    changed["accepted"], changed["committed"], changed["emitted"] = 0, 1, [wrong]
    consumed = 1 + len(cycles[0]["emitted"])
    tokens = tokens[:consumed] + [wrong, 1, 2]  # two more tokens, decoded tick by tick, keep the changed cycle a cycle
    cycles = cycles[:2]
    report = follow_generation(oracle, OracleStream(package, 128), prompt, tokens, cycles, 3)
    assert report["divergences"] and report["divergences"][0]["kind"] in ("target", "draft")
    assert report["divergences"][0]["position"] == consumed and report["violations"]
    assert report["cycles_compared"] == 2 and report["tokens_compared"] == len(tokens)
