"""Operator micro-benchmark through the C ABI: times one weight-streaming linear on rotating weight copies
(the working set is kept larger than the 126 MB L2) with CUDA events on the launching stream.

    python -m llmoop_b200.opbench --op int4 --n 28672 --k 4096 --lanes 4

Prints one JSON line with the achieved algorithmic GB/s.  Small enough to run under `ncu --set full`.
"""

from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np


def main():
    import torch

    import llmoop_b200 as nb

    parser = argparse.ArgumentParser()
    parser.add_argument("--op", default="int4", choices=["int4", "int4pair", "bf16"])
    parser.add_argument("--n", type=int, default=28672)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--lanes", type=int, default=4)
    parser.add_argument("--iters", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--working-set-mb", type=int, default=512)
    parser.add_argument("--register-kernel", action="store_true", help="use the register-prefetch INT4 kernel")
    args = parser.parse_args()

    lib = nb.library()
    if args.register_kernel:
        lib.nerve_b200_set_int4_kernel(0)
    n, k, lanes = args.n, args.k, args.lanes
    if args.op in ("int4", "int4pair"):
        weight_bytes = n * k // 2
        scale_bytes = n * (k // 128) * 2
    else:
        weight_bytes = n * k * 2
        scale_bytes = 0
    copies = max(2, (args.working_set_mb << 20) // weight_bytes + 1)
    generator = torch.Generator(device="cuda").manual_seed(0)
    weights = [torch.randint(0, 2 ** 31 - 1, (weight_bytes // 4,), dtype=torch.int32, device="cuda", generator=generator)
               for _ in range(copies)]
    if args.op == "bf16":
        weights = [(torch.randn(n * k, device="cuda", generator=generator) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    scales = [(torch.rand(max(1, scale_bytes // 2), device="cuda", generator=generator) * 0.01).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(lanes * k, device="cuda", generator=generator).to(torch.bfloat16)
    y = torch.zeros(lanes * n, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream()
    handle = ctypes.c_void_p(stream.cuda_stream)

    def launch(index):
        w, s = weights[index % copies], scales[index % copies]
        if args.op == "int4pair":
            w2, s2 = weights[(index + 1) % copies], scales[(index + 1) % copies]
            status = lib.nerve_b200_op_linear_int4_silu_pair(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(s.data_ptr()),
                                                             ctypes.c_void_p(w2.data_ptr()), ctypes.c_void_p(s2.data_ptr()),
                                                             ctypes.c_void_p(y.data_ptr()), lanes, n, k, handle)
        elif args.op == "int4":
            status = lib.nerve_b200_op_linear_int4(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(s.data_ptr()),
                                                   ctypes.c_void_p(y.data_ptr()), None, lanes, n, k, 128, handle)
        else:
            status = lib.nerve_b200_op_linear_bf16(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                                   None, lanes, n, k, 0, ctypes.c_float(1.0), handle)
        if status != 0:
            raise RuntimeError(lib.nerve_b200_last_error().decode())

    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    for i in range(args.iters):
        launch(args.warmup + i)
    end.record(stream)
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / args.iters
    algorithmic = (weight_bytes + scale_bytes) * (2 if args.op == "int4pair" else 1)
    print(json.dumps({"op": args.op, "n": n, "k": k, "lanes": lanes, "us_per_launch": ms * 1e3,
                      "algorithmic_bytes": algorithmic, "gbs": algorithmic / (ms * 1e-3) / 1e9, "weight_copies": copies}))


if __name__ == "__main__":
    main()
