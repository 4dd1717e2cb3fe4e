"""Per-phase timing of the persistent decode stack kernel on a small package of 8B-class layer width:

    python -m llmoop_b200.stackbench --layers 4 --drafts 3 --cycles 3

Writes a synthetic INT4 g128 + MTP package (hidden 4096, 32 q / 8 kv heads of 128, FFN 14336, small vocabulary,
`--layers` layers; about 0.25 GB per layer on the device) under --directory once, prefills a 512-token prompt and
runs `--cycles` speculative cycles with per-launch profiling on.  CTA 0 of the kernel stamps the GPU's nanosecond
timer at every phase boundary; the printed JSON line gives the mean microseconds per layer of each phase of the
last target-stack launch (`--drafts 0` makes that a 1-lane single tick, otherwise a `drafts + 1`-lane verify
batch).  The working set is small enough for `ncu --set full -k regex:decode_stack_kernel`.

Under `python -m torch.distributed.run --nproc-per-node N -m llmoop_b200.stackbench ...` the N ranks mount their
tensor-parallel shards, connect the exchange over peer memory and run the same stream; rank 0 prints its stamps
(the o and down barriers then contain the exchange).
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import numpy as np


def main():
    import llmoop_b200 as nb
    from llmoop_b200.package_writer import write_package
    from llmoop_b200.synth import ModelSpec, iter_checkpoint_torch

    parser = argparse.ArgumentParser()
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--drafts", type=int, default=3)
    parser.add_argument("--cycles", type=int, default=3)
    parser.add_argument("--prompt", type=int, default=512)
    parser.add_argument("--directory", default="/tmp/nerve_b200_stackbench")
    args = parser.parse_args()

    spec = ModelSpec(name=f"stackbench_{args.layers}l", hidden=4096, layers=args.layers, q_heads=32, kv_heads=8, head_dim=128,
                     ffn=14336, vocab=4096, max_positions=2048, quant="int4", std=0.02, seed=3, rope_theta=500000.0)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    device = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(device)
        dist.init_process_group("nccl", device_id=torch.device("cuda", device))
    directory = Path(args.directory) / spec.name
    if rank == 0 and not (directory / "vulkan_resident_package.json").exists():
        write_package(spec, directory, tensors=iter_checkpoint_torch(spec, f"cuda:{device}"), hash_tensors=False)
    if world > 1:
        dist.barrier()
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, spec.vocab, size=args.prompt)]
    package = nb.Package(directory, device=device, capacity_tokens=args.prompt + 512, page_tokens=16, max_streams=1, max_lanes=args.prompt,
                         verify_level=0, tp_rank=rank, tp_size=world)
    if not package.info["target_decode_stack"]:
        raise SystemExit("the decode stack kernel is not available for this package")
    engine = nb.Engine(package)
    if world > 1:
        unique_id = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            unique_id.copy_(torch.frombuffer(bytearray(nb.tensor_parallel_unique_id()), dtype=torch.uint8))
        dist.broadcast(unique_id, src=0)
        engine.init_tensor_parallel(rank, world, bytes(unique_id.cpu().numpy().tobytes()))
        mine = torch.frombuffer(bytearray(engine.tp_exchange_handle()), dtype=torch.uint8).cuda()
        handles = [torch.zeros(64, dtype=torch.uint8, device="cuda") for _ in range(world)]
        dist.all_gather(handles, mine)
        engine.tp_connect([bytes(handle.cpu().numpy().tobytes()) for handle in handles])
    engine.set_decode_stack(True)
    engine.set_prefill_chunk(args.prompt)
    engine.add_stream(0, seed=0, speculative_draft_tokens=args.drafts)
    engine.enqueue_input_event(0, prompt, 16 * (args.drafts + 1) * args.cycles)
    engine.set_profiling(True)  # plain launches (no graph replay), device timing around every stack launch
    _, report = engine.run(args.cycles)
    stamps = engine.decode_stack_timing().astype(np.float64)
    layers = stamps[1:] if len(stamps) > 1 else stamps  # the first layer also pays the launch ramp
    phases = {}
    for step, label in enumerate(["qkv", "o", "gate_up", "down"]):
        s0, s1, s2, s3 = (layers[:, 4 * step + i] for i in range(4))
        phases[label] = {"stage_us": float(np.mean(s1 - s0) / 1e3), "tiles_us": float(np.mean(s2 - s1) / 1e3),
                         "steps_us": float(np.mean(layers[:, 26 + step] - s1) / 1e3),
                         "barrier_us": float(np.mean(s3 - s2) / 1e3)}
    phases["attention"] = {"teams_us": float(np.mean(layers[:, 17] - layers[:, 3]) / 1e3),
                           "barrier_us": float(np.mean(layers[:, 18] - layers[:, 17]) / 1e3),
                           "merge_us": float(np.mean(layers[:, 19] - layers[:, 18]) / 1e3),
                           "barrier2_us": float(np.mean(layers[:, 4] - layers[:, 19]) / 1e3)}
    phases["attention_item"] = {f"t{i}_us": float(np.mean(layers[:, 20 + i] - layers[:, 3]) / 1e3) for i in range(6)}
    layer_us = float(np.mean(layers[:, 15] - layers[:, 0]) / 1e3)
    weight_bytes = package.info["target_stack_weight_bytes"] / max(1, args.layers)
    if rank == 0:
        print(json.dumps({"lanes": args.drafts + 1 if args.drafts else 1, "layers": args.layers, "tensor_parallel": world, "layer_us": layer_us,
                          "layer_weight_bytes": weight_bytes, "layer_gbs": weight_bytes / layer_us / 1e3, "phases": phases,
                          "stack_launches": report.int4_launches, "stack_ms_per_launch": report.int4_ms / max(1, report.int4_launches)}))
    if world > 1:
        dist.barrier()
    engine.close()
    package.unmount()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
