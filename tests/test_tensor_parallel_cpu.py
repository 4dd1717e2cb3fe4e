"""The tensor-parallel shard plan on CPU, two `gloo` ranks: each rank cuts its shard of an INT4 g128 layer's
weights with the mount's own range rule (nerve_b200_tp_shard_range through the C ABI), evaluates it with numpy,
and the ranks meet in one all-reduce per row-parallel linear - exactly the data flow of the sharded engine
(q/k/v and gate/up by rows, o and down by columns, f32 partial sums summed, then one bf16 rounding).  The result
must equal the unsharded layer's to f32 summation-order accuracy.
"""

import os
import socket

import numpy as np
import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dequant(packed, scales):
    from llmoop_b200.safetensors_io import bf16_bits_to_f32

    words = packed.view(np.uint32)
    nibbles = np.stack([(words >> (4 * i)) & 15 for i in range(8)], axis=-1).reshape(words.shape[0], -1).astype(np.float32) - 8.0
    return nibbles * np.repeat(bf16_bits_to_f32(scales), 128, axis=1)


def _worker(rank, size, port, out):
    import torch
    import torch.distributed as dist

    import llmoop_b200 as nb
    from llmoop_b200.safetensors_io import bf16_bits_to_f32, f32_to_bf16_bits
    from llmoop_b200.synth import quantize_int4_group

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    rng = np.random.default_rng(5)  # the same "checkpoint" on every rank
    hidden, heads, head, ffn, lanes = 512, 4, 128, 1024, 3
    weights = {}
    for name, (n, k) in {"qkv": (heads * head, hidden), "o": (hidden, heads * head), "gate": (ffn, hidden), "down": (hidden, ffn)}.items():
        weights[name] = quantize_int4_group(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
    x = bf16_bits_to_f32(f32_to_bf16_bits(rng.standard_normal((lanes, hidden), dtype=np.float32)))

    def bf16(a):
        return bf16_bits_to_f32(f32_to_bf16_bits(a.astype(np.float32)))

    def full_layer():
        q = bf16(x @ _dequant(*weights["qkv"]).T)
        h = bf16(bf16(q @ _dequant(*weights["o"]).T) + x)
        g = bf16(h @ _dequant(*weights["gate"]).T)
        return bf16(bf16(g @ _dequant(*weights["down"]).T) + h)

    def rows(name, unit):
        packed, scales = weights[name]
        begin, count = nb.tp_shard_range(packed.shape[0], unit, rank, size)
        return packed[begin:begin + count], scales[begin:begin + count], begin, count

    def columns(name):
        packed, scales = weights[name]
        begin, count = nb.tp_shard_range(packed.shape[1] * 8, 128, rank, size)
        return packed[:, begin // 8:(begin + count) // 8], scales[:, begin // 128:(begin + count) // 128], begin, count

    def all_reduce(partial):
        tensor = torch.from_numpy(np.ascontiguousarray(partial, dtype=np.float32))
        dist.all_reduce(tensor)
        return tensor.numpy()

    qp, qs, q_begin, q_count = rows("qkv", head)
    q_local = bf16(x @ _dequant(qp, qs).T)                                  # column-parallel: this rank's heads
    op, osc, o_begin, o_count = columns("o")
    assert (o_begin, o_count) == (q_begin, q_count)                        # o's input columns are exactly those heads
    h = bf16(bf16(all_reduce(q_local @ _dequant(op, osc).T)) + x)           # row-parallel + all-reduce + rounding + residual
    gp, gs, g_begin, g_count = rows("gate", 16)
    g_local = bf16(h @ _dequant(gp, gs).T)
    dp, ds, d_begin, d_count = columns("down")
    assert (d_begin, d_count) == (g_begin, g_count)
    y = bf16(bf16(all_reduce(g_local @ _dequant(dp, ds).T)) + h)
    expected = full_layer()
    gathered = [None] * size
    dist.all_gather_object(gathered, y.tobytes())
    if rank == 0:
        assert all(blob == gathered[0] for blob in gathered)               # every rank holds the same result
        difference = np.abs(y - expected)
        out.put((float(difference.max()), float((difference != 0).mean()), float(np.abs(expected).max())))
    dist.destroy_process_group()


def test_two_rank_shard_plan_reproduces_the_unsharded_layer():
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    out = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_worker, args=(rank, 2, port, out)) for rank in range(2)]
    for process in processes:
        process.start()
    try:
        for process in processes:
            process.join(timeout=240)
            assert process.exitcode == 0
    finally:
        for process in processes:
            if process.is_alive():
                process.kill()
    worst, changed, scale = out.get(timeout=10)
    # partial sums are added in another order: an output may move by one bf16 ulp, never more
    assert worst <= scale * 2.0 ** -7, (worst, scale)
    assert changed < 0.05


def test_shard_range_rule():
    import llmoop_b200 as nb

    assert nb.tp_shard_range(4096, 128, 0, 2) == (0, 2048)
    assert nb.tp_shard_range(4096, 128, 1, 2) == (2048, 2048)
    assert nb.tp_shard_range(14336, 128, 7, 8) == (12544, 1792)
    assert nb.tp_shard_range(1024, 128, 3, 8) == (384, 128)
    with pytest.raises(nb.NerveError):
        nb.tp_shard_range(4096, 128, 0, 3)       # 4096 columns do not split into three shards of whole groups
    with pytest.raises(nb.NerveError):
        nb.tp_shard_range(128, 128, 0, 2)        # one group cannot be halved
    with pytest.raises(nb.NerveError):
        nb.tp_shard_range(1024, 128, 2, 2)       # rank outside the group
