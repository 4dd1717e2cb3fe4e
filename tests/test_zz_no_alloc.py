"""nerve_b200_op_greedy_static: the greedy arg-max whose reduction scratch is a device array built into the
library (no allocation by the call or the caller).  Called through the C ABI and compared with
nerve_b200_op_greedy (caller-provided scratch) on two calls in a row - the second with other logits and another
lane count, so that it runs over the partials the first left behind.  This file sorts last on purpose: it must
pass alone and after every other GPU test has used the library.
"""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def _records(torch, lib, logits, lanes, vocab, static):
    records = torch.full((lanes, 4), 0xFFFF, dtype=torch.int32, device="cuda")
    if static:
        status = lib.nerve_b200_op_greedy_static(_ptr(logits), _ptr(records), lanes, vocab, None)
    else:
        scratch = torch.zeros(int(lib.nerve_b200_op_greedy_scratch_bytes(lanes)), dtype=torch.uint8, device="cuda")
        status = lib.nerve_b200_op_greedy(_ptr(logits), _ptr(records), _ptr(scratch), lanes, vocab, None)
    assert status == 0, lib.nerve_b200_last_error()
    torch.cuda.synchronize()
    return records.cpu().numpy().view(np.uint32)


def test_static_scratch_greedy_matches_scratch_variant_twice_in_a_row():
    import torch

    import llmoop_b200 as nb

    lib = nb.library()
    generator = torch.Generator(device="cuda").manual_seed(123)
    cases = [(5, 128256), (64, 4099)]  # the second call: other lane count (the maximum), odd vocabulary
    for lanes, vocab in cases:
        logits = torch.randn(lanes, vocab, device="cuda", generator=generator, dtype=torch.float32)
        logits[0, 17] = logits[0, 4001] = 50.0  # a tie: the lower id wins
        expected = _records(torch, lib, logits, lanes, vocab, static=False)
        got = _records(torch, lib, logits, lanes, vocab, static=True)
        assert np.array_equal(got, expected)
        assert got[0, 0] == 17
        reference = torch.argmax(logits, dim=1).cpu().numpy()
        assert np.array_equal(got[1:, 0], reference[1:].astype(np.uint32))


def test_static_scratch_greedy_rejects_more_lanes_than_its_array_holds():
    import torch

    import llmoop_b200 as nb

    lib = nb.library()
    logits = torch.zeros(65, 32, device="cuda", dtype=torch.float32)
    records = torch.zeros(65, 4, dtype=torch.int32, device="cuda")
    status = lib.nerve_b200_op_greedy_static(_ptr(logits), _ptr(records), 65, 32, None)
    assert status != 0
    message = lib.nerve_b200_last_error().decode()
    assert "64 lanes" in message and "nerve_b200_op_greedy" in message
