"""Pins the CPU oracle - and the product's host-side pure functions - against every known-answer vector the
reference's own tests hold for this path.  (The reference has no golden logits or token sequences; those stay
"parity unpinned" and are covered by oracle-vs-CUDA parity tests instead.)

Sources, by path inside the reference project:
  runtime-rs/src/vulkan_stream_circuit/tests/package_batch.rs:296-335            acceptance rule
  runtime-rs/src/vulkan_stream_circuit/tests/component_transducer_sampler_tests.rs:317-406  greedy sampler
  runtime-rs/src/vulkan_stream_circuit/tests/kernel_abi.rs:111-155               stream-control bytes
  runtime-rs/src/vulkan_stream_circuit/transient_state_buffer_layout.rs:231-268  state header / page table
  tests/test_model_package_tensor_layout.py (bf16 / e4m3 conversions, checked against ml_dtypes when present)
  runtime-rs/test-fixtures/tiny_model (generator formula of scripts/generate_tiny_test_model.py:28-34)
"""

import ctypes
import struct

import numpy as np
import pytest

from oracle import nerve_oracle as orc


# ---- acceptance rule --------------------------------------------------------------------------------------

def _both_verify(draft, target, stop=()):
    import llmoop_b200 as nb

    a = orc.verify_prefix(draft, target, stop)
    b = nb.verify_prefix(draft, target, stop)
    assert a == (b[0], b[1], b[2])
    return a


def test_speculative_verification_commits_through_the_first_mismatch():
    assert _both_verify([11, 12, 13], [11, 99, 88, 77]) == (1, 2, [11, 99])


def test_speculative_verification_emits_the_bonus_token_when_all_drafts_match():
    assert _both_verify([11, 12], [11, 12, 13]) == (2, 3, [11, 12, 13])


def test_speculative_verification_rejects_incomplete_target_results():
    import llmoop_b200 as nb

    with pytest.raises(ValueError, match="2 draft tokens but 2 target predictions; expected 3"):
        orc.verify_prefix([11, 12], [11, 12])
    with pytest.raises(nb.NerveError, match="2 draft tokens but 2 target predictions; expected 3"):
        nb.verify_prefix([11, 12], [11, 12])


def test_speculative_verification_stops_at_the_first_emitted_stop_token():
    assert _both_verify([11, 12], [11, 12, 99], stop=[11]) == (1, 1, [11])


def test_stop_on_the_bonus_token_keeps_all_drafts():
    assert _both_verify([5, 6], [5, 6, 2], stop=[2]) == (2, 3, [5, 6, 2])


# ---- greedy sampler ---------------------------------------------------------------------------------------

def test_greedy_sampler_selects_largest_logit_and_advances_the_tick():
    logits = np.zeros(65536, dtype=np.float32)
    logits[7] = 3.5
    logits[1024] = 9.25
    record = np.zeros(4, dtype=np.uint32)
    token = orc.lib().orc_greedy(orc._p(logits, orc._f32p), logits.size, orc._p(record, orc._u32p))
    assert token == 1024
    assert record.tobytes() == bytes([0x00, 0x04, 0x00, 0x00, 0x00, 0x00, 0x14, 0x41, 0, 0, 0, 0, 0, 0, 0, 0])
    control = np.frombuffer(bytearray(20), dtype=np.uint32).copy()
    raw = (ctypes.c_uint8 * 20)()
    orc.lib().orc_stream_control_bytes(ctypes.c_uint32(0), ctypes.c_uint64(0x0000_0007_FFFF_FFFF), ctypes.c_uint32(0),
                                       ctypes.c_uint32(8), raw)
    control = np.frombuffer(bytes(raw), dtype=np.uint32).copy()
    orc.lib().orc_sampler_advance_control(orc._p(control, orc._u32p), ctypes.c_uint32(token))
    assert control[0] == 1024 and control[1] == 0 and control[2] == 8  # carry 0x7_ffff_ffff -> 0x8_0000_0000


def test_greedy_ties_resolve_to_the_lowest_token_id():
    logits = np.full(100, -1.0, dtype=np.float32)
    logits[[40, 17, 99]] = 2.0
    assert orc.lib().orc_greedy(orc._p(logits, orc._f32p), 100, None) == 17


# ---- control / state byte layouts ---------------------------------------------------------------------------

def test_stream_control_buffer_bytes_follow_kernel_abi_order():
    import llmoop_b200 as nb

    for make in ("oracle", "product"):
        raw = (ctypes.c_uint8 * 20)()
        if make == "oracle":
            orc.lib().orc_stream_control_bytes(ctypes.c_uint32(11), ctypes.c_uint64(42), ctypes.c_uint32(7), ctypes.c_uint32(4), raw)
        else:
            assert nb.library().nerve_b200_stream_control_bytes(ctypes.c_uint32(11), ctypes.c_uint64(42), ctypes.c_uint32(7),
                                                               ctypes.c_uint32(4), raw) == 0
        data = bytes(raw)
        assert data[0:4] == struct.pack("<I", 11)
        assert data[4:12] == struct.pack("<Q", 42)
        assert data[12:16] == struct.pack("<I", 7)
        assert data[16:20] == struct.pack("<I", 4)


def _layouts(static_bytes, per_activation, capacity):
    import llmoop_b200 as nb

    out = []
    table = (ctypes.c_uint8 * 4096)()
    layout = (ctypes.c_int64 * 7)()
    size = orc.lib().orc_state_page_table(ctypes.c_int64(static_bytes), ctypes.c_int64(per_activation), ctypes.c_int64(0),
                                          ctypes.c_int64(capacity), table, ctypes.c_int64(4096), layout)
    out.append((list(layout), bytes(table)[:layout[3]]))
    assert size == layout[3]
    table2 = (ctypes.c_uint8 * 4096)()
    layout2 = (ctypes.c_int64 * 7)()
    assert nb.library().nerve_b200_state_page_table_bytes(ctypes.c_int64(static_bytes), ctypes.c_int64(per_activation), ctypes.c_int64(0),
                                                          ctypes.c_int64(capacity), None, ctypes.c_size_t(0), table2,
                                                          ctypes.c_size_t(4096), layout2) == 0
    out.append((list(layout2), bytes(table2)[:layout2[3]]))
    assert out[0] == out[1]
    return out[0]


def test_dynamic_state_layout_separates_device_page_table_from_physical_pages():
    (block, pages, page_bytes, table_bytes, static_offset, dynamic_offset, total), table = _layouts(0, 16, 130)
    assert block == 64 and pages == 3 and page_bytes == 1024
    assert dynamic_offset == table_bytes
    assert total == dynamic_offset + 3 * 1024
    assert struct.unpack_from("<I", table, 0)[0] == 0x4E525653
    assert struct.unpack_from("<I", table, 36)[0] == 0
    assert struct.unpack_from("<I", table, 44)[0] == 2


def test_fixed_state_layout_uses_the_same_abi_without_dynamic_pages():
    (block, pages, page_bytes, table_bytes, static_offset, dynamic_offset, total), _ = _layouts(3072, 0, 65536)
    assert pages == 0
    assert static_offset == table_bytes
    assert dynamic_offset == total == static_offset + 3072


# ---- number formats ----------------------------------------------------------------------------------------------

def test_bf16_rounding_is_nearest_even_on_the_bit_pattern():
    from llmoop_b200.safetensors_io import f32_to_bf16_bits

    values = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40, 0.0, -0.0], dtype=np.float32)
    ours = [orc.lib().orc_f32_to_bf16(ctypes.c_float(float(v))) for v in values]
    assert ours == list(f32_to_bf16_bits(values))
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(0)
    sample = rng.standard_normal(4096).astype(np.float32)
    want = sample.astype(ml_dtypes.bfloat16).view(np.uint16)
    assert np.array_equal(f32_to_bf16_bits(sample), want)
    assert [orc.lib().orc_f32_to_bf16(ctypes.c_float(float(v))) for v in sample[:512]] == list(want[:512])


def test_e4m3_conversions_match_ml_dtypes():
    from llmoop_b200.safetensors_io import E4M3_TO_F32, f32_to_e4m3_bits

    ml_dtypes = pytest.importorskip("ml_dtypes")
    codes = np.arange(256, dtype=np.uint8)
    want = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    ours = np.array([orc.lib().orc_e4m3_to_f32(ctypes.c_uint8(int(c))) for c in codes], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(ours[finite], want[finite]) and np.array_equal(E4M3_TO_F32[finite], want[finite])
    rng = np.random.default_rng(1)
    sample = np.concatenate([rng.uniform(-448, 448, 4000), rng.standard_normal(2000) * 0.01, [0.0, 448.0, -448.0, 2 ** -9, 2 ** -10]]).astype(np.float32)
    expected = sample.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(f32_to_e4m3_bits(sample), expected)
    got = np.array([orc.lib().orc_f32_to_e4m3(ctypes.c_float(float(v))) for v in sample], dtype=np.uint8)
    assert np.array_equal(got, expected)


def test_shader_float_round_trips_through_nine_significant_digits():
    assert orc.shader_float(0.3535533905932738) == np.float32(0.353553391)
    assert orc.shader_float(1e-5) == np.float32(1e-05)
    assert orc.attention_tile_tokens(8) == 112 and orc.attention_tile_tokens(128) == 56


# ---- seeded top-k / top-p sampler ---------------------------------------------------------------------------
def test_seeded_sampler_matches_the_reference_known_answer():
    """component_transducer_sampler_tests.rs:409-533: vocabulary 64, logits -100 except tokens 7, 8, 19, 51 at 2.0,
    temperature 1, top_k 4, top_p 1, min_p 0, seed 0x5eed1234; at stream tick t the sampler must pick
    TOP_TOKENS[((hash(seed ^ t) >> 8) * 4) >> 24] with logit bits of 2.0 and record flags 1, and all four tokens
    must appear over ticks 0..15."""
    top_tokens = [7, 8, 19, 51]
    logits = np.full(64, -100.0, dtype=np.float32)
    logits[top_tokens] = 2.0
    seen = set()
    for tick in range(16):
        bits = orc.lib().orc_hash_u32(ctypes.c_uint32(0x5EED1234 ^ tick))
        expected = top_tokens[((bits >> 8) * 4) >> 24]
        record = np.zeros(4, dtype=np.uint32)
        token = orc.lib().orc_sample_top_k_top_p(orc._p(logits, orc._f32p), 64, 4, 1.0, 1.0, 0.0, 0x5EED1234, tick, 0,
                                                 orc._p(record, orc._u32p))
        assert token == expected
        assert list(record) == [expected, int(np.float32(2.0).view(np.uint32)), 1, 0]
        seen.add(token)
    assert seen == set(top_tokens)


def test_sampler_hash_is_the_shader_hash():
    """temperature_top_k_top_p_sampler_f32.comp.template:56-63, evaluated by hand for two inputs."""
    def reference(value):
        value ^= value >> 16
        value = (value * 0x7FEB352D) & 0xFFFFFFFF
        value ^= value >> 15
        value = (value * 0x846CA68B) & 0xFFFFFFFF
        value ^= value >> 16
        return value

    for value in (0, 1, 0x5EED1234, 0xFFFFFFFF, 123456789):
        assert orc.lib().orc_hash_u32(ctypes.c_uint32(value)) == reference(value)


def test_sampler_min_p_top_p_and_nan_rules():
    """min-p cuts entries below top + T*log(min_p); top-p keeps the shortest prefix reaching p of the weight; NaN
    logits never enter the list; ties go to the lower token id."""
    logits = np.array([1.0, np.nan, 3.0, 3.0, 0.5, -2.0, 2.9, np.nan], dtype=np.float32)
    picks = set()
    for tick in range(64):
        picks.add(int(orc.lib().orc_sample_top_k_top_p(orc._p(logits, orc._f32p), 8, 8, 1.0, 1.0, 0.0, 7, tick, 0, None)))
    assert picks <= {0, 2, 3, 4, 5, 6} and {2, 3, 6} <= picks          # NaN tokens 1 and 7 never drawn
    # min_p 0.5: only logits >= 3 + log(0.5) = 2.307 survive -> tokens 2, 3, 6
    picks = {int(orc.lib().orc_sample_top_k_top_p(orc._p(logits, orc._f32p), 8, 8, 1.0, 1.0, 0.5, 7, tick, 0, None)) for tick in range(64)}
    assert picks == {2, 3, 6}
    # top_p tiny: the nucleus is the first entry alone, and the tie between tokens 2 and 3 goes to token 2
    picks = {int(orc.lib().orc_sample_top_k_top_p(orc._p(logits, orc._f32p), 8, 8, 1.0, 0.01, 0.0, 7, tick, 0, None)) for tick in range(64)}
    assert picks == {2}
