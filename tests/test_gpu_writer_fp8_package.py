"""A dense FP8 (e4m3, block-scaled) package from the native writer whose q/k/v projections share one block shape, so
that they fuse into `parallel_linear_3way` behind one `quantize_fp8_e4m3` node - the form a model of config 3's
width takes (the reference compiler's golden FP8 package is too narrow for it: its q stays a linear of its own).
The engine's greedy generation with MTP drafts must follow the CPU oracle: token ids exact, a divergence allowed
only where the oracle's top-2 logit gap is below 1e-3; acceptance counts exact while the sequences agree.
Synthetic data: seeded N(0, 0.08) weights quantised per 128 x 128 block, prompt uniform over the vocabulary."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GAP_RULE = 1e-3


@pytest.mark.parametrize("drafts", [0, 2])
def test_fp8_three_way_projection_package_follows_the_oracle(tmp_path, drafts):
    import llmoop_b200 as nb
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream

    spec = ModelSpec(name="writer_fp8_3way", hidden=256, layers=2, q_heads=8, kv_heads=4, head_dim=32, ffn=512, vocab=256,
                     quant="fp8", std=0.08, seed=21)
    directory = write_package(spec, tmp_path / spec.name)
    opkg = OraclePackage(directory)
    oracle = Oracle(opkg)
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, spec.vocab, size=16)]
    expected = oracle.generate(OracleStream(opkg, 128), prompt, 24, drafts, collect_logits=True)

    package = nb.Package(directory, capacity_tokens=128, page_tokens=16, max_streams=2, max_lanes=64, verify_level=2)
    engine = nb.Engine(package)
    engine.set_cycle_logging(True)
    engine.add_stream(1, seed=0, speculative_draft_tokens=drafts)
    tokens, report = engine.submit_input_event_until_idle(1, prompt, 24)
    diverged = None
    for index, (a, b) in enumerate(zip(tokens, expected["tokens"])):
        if a != b:
            gap = oracle.top2_gap(expected["logits"][index])
            assert gap < GAP_RULE, f"token {index}: cuda {a} != oracle {b} with top-2 gap {gap}"
            diverged = index
            break
    if diverged is None:
        assert tokens == expected["tokens"] and engine.stream_tick(1) == len(prompt) + 24
        cycles = engine.cycle_log()
        assert [c["accepted"] for c in cycles] == [c["accepted"] for c in expected["cycles"]]
        assert [c["emitted"] for c in cycles] == [c["emitted"] for c in expected["cycles"]]
    assert report.generated_tokens == 24
    engine.close()
    package.unmount()
