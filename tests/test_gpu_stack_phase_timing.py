"""The persistent decode kernel on a small package of 8B-class layer width (hidden 4096, 32 q / 8 kv heads of 128,
FFN 14336, four layers, small vocabulary: about 1 GB on the device), with CTA 0's step stamps read back.

This is the small case the profiles of the kernel are taken on (`python -m pytest tests/test_gpu_stack_phase_timing.py
-q -s` runs a handful of launches of a few hundred microseconds each) and it prints the per-step table of a verify
launch.  As a test it checks that the stamps are complete and ordered, that the four matrix steps stream their
weights at a sane rate, and that speculative cycles on this package still follow the oracle (the widest layer shape
any parity test runs end to end besides the full configuration)."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LAYERS, DRAFTS, PROMPT = 4, 3, 512


@pytest.fixture(scope="module")
def wide_package(tmp_path_factory):
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec, iter_checkpoint_torch

    spec = ModelSpec(name="stack_timing_4l", hidden=4096, layers=LAYERS, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=4096,
                     max_positions=2048, quant="int4", std=0.01, seed=3, rope_theta=500000.0)
    directory = tmp_path_factory.mktemp("packages") / spec.name
    write_package(spec, directory, tensors=iter_checkpoint_torch(spec, "cuda:0"), hash_tensors=False)
    return directory, spec


def phase_table(stamps):
    """Mean microseconds per layer of every step of the launch (the first layer also pays the launch ramp)."""
    layers = stamps[1:].astype(np.float64) if len(stamps) > 1 else stamps.astype(np.float64)
    table = {}
    for step, label in enumerate(["qkv", "o", "gate_up", "down"]):
        begin, staged, done, met = (layers[:, 4 * step + i] for i in range(4))
        table[label] = {"stage": float(np.mean(staged - begin) / 1e3), "blocks": float(np.mean(layers[:, 26 + step] - staged) / 1e3),
                        "epilogue": float(np.mean(done - layers[:, 26 + step]) / 1e3), "barrier": float(np.mean(met - done) / 1e3)}
    table["attention"] = {"items": float(np.mean(layers[:, 17] - layers[:, 3]) / 1e3), "merge_and_barrier": float(np.mean(layers[:, 18] - layers[:, 17]) / 1e3)}
    table["layer"] = float(np.mean(layers[:, 15] - layers[:, 0]) / 1e3)
    return table


def test_step_stamps_of_a_verify_launch_and_parity_on_the_wide_package(wide_package):
    import llmoop_b200 as nb
    from oracle.nerve_oracle import Oracle, OraclePackage, OracleStream
    from oracle.parity import follow_generation, summary

    directory, spec = wide_package
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, spec.vocab, size=PROMPT)]
    package = nb.Package(directory, capacity_tokens=PROMPT + 512, page_tokens=16, max_streams=1, max_lanes=PROMPT, verify_level=0)
    assert package.info["target_decode_stack"] == 1
    engine = nb.Engine(package)
    engine.set_decode_stack(True)
    engine.set_prefill_chunk(PROMPT)
    engine.add_stream(0, seed=0, speculative_draft_tokens=DRAFTS)
    engine.enqueue_input_event(0, prompt, 64)
    engine.set_profiling(True)  # plain launches with device timing around every stack launch; CTA 0 stamps its steps
    _, report = engine.run(4)
    stamps = engine.decode_stack_timing()
    engine.set_profiling(False)
    assert stamps.shape == (LAYERS, 32)
    table = phase_table(stamps)
    weight_bytes = package.info["target_stack_weight_bytes"] / LAYERS
    print("decode_stack_kernel, verify launch of %d lanes, microseconds per layer:" % (DRAFTS + 1))
    for label, row in table.items():
        print("  ", label, row if not isinstance(row, dict) else {k: round(v, 2) for k, v in row.items()})
    print("   layer weights %.1f MB -> %.0f GB/s per layer" % (weight_bytes / 1e6, weight_bytes / table["layer"] / 1e3))
    # complete and ordered stamps of every layer behind the first
    order = [0, 1, 26, 2, 3, 17, 18, 4, 5, 27, 6, 7, 8, 9, 28, 10, 11, 12, 13, 29, 14]
    for layer in range(1, LAYERS):
        values = [int(stamps[layer, index]) for index in order]
        assert all(v > 0 for v in values) and values == sorted(values), (layer, values)
    assert 10.0 < table["layer"] < 400.0  # a layer of 112 MB: 17 us at the HBM rate, far below a kernel-per-operator layer
    assert report.int4_launches > 0

    # the same engine, a short event from a 16-token prompt against the oracle
    engine.reset_stream_transient_state(0)
    engine.set_cycle_logging(True)
    short = prompt[32:48]  # a prompt whose closest calls stay clear of the 1e-3 rule (random weights: near-uniform logits)
    tokens, _ = engine.submit_input_event_until_idle(0, short, 10)
    opkg = OraclePackage(directory)
    outcome = follow_generation(Oracle(opkg), OracleStream(opkg, 128), short, tokens, engine.cycle_log(), DRAFTS, prefill_chunk=16)
    print("parity on the wide package:", summary(outcome), outcome["divergences"])
    assert outcome["tokens_compared"] == len(tokens) == 10 and outcome["accepted_equal"] and not outcome["violations"], outcome["divergences"]
    engine.close()
    package.unmount()
