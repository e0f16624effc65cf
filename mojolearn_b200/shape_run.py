"""Run and time one identical-mode product on the current CUDA device.

    python -m mojolearn_b200.shape_run M N K [--op NT] [--wkind f32|bf16|int8] [--plan -1] [--groups 0]
                                             [--reps 5] [--warmup 2] [--buffers 1]

Operands are seeded N(0, 1) (weights N(0, 0.02) for the low-bit kinds), created
on the device; `--buffers B` rotates B distinct weight buffers so that a small
weight matrix is not served from L2. Prints one JSON line with the CUDA-event
time per launch, TFLOP/s and algorithmic GB/s. It is also the command the
profiler summaries under profiles/ were captured with.
"""
import argparse
import json

import torch

from . import linalg, torch_ops

OPS = {"NN": linalg.OP_NN, "NT": linalg.OP_NT, "TN": linalg.OP_TN}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--op", default="NT", choices=sorted(OPS))
    ap.add_argument("--wkind", default="f32", choices=["f32", "bf16", "int8", "int8s", "int8i32", "int15i64"],
                    help="int8i32 / int15i64: the integer product profiles (both operands codes with row exponents, op NT)")
    ap.add_argument("--plan", type=int, default=-1)
    ap.add_argument("--groups", type=int, default=0)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--buffers", type=int, default=1)
    ap.add_argument("--graph", action="store_true", help="replay the launches from one CUDA graph (no host launch cost)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    m, n, k, op = args.m, args.n, args.k, OPS[args.op]
    if args.wkind in ("int8i32", "int15i64"):
        return int8_product(args, dev, g)
    a = torch.randn((k, m) if op == linalg.OP_TN else (m, k), generator=g, device=dev)
    wshape = (n, k) if op == linalg.OP_NT else (k, n)
    ws, scale, wkind, wbytes = [], None, linalg.W_F32, 4
    for _ in range(args.buffers):
        if args.wkind == "f32":
            ws.append(torch.randn(wshape, generator=g, device=dev))
        elif args.wkind == "bf16":
            ws.append(torch_ops.to_bf16(torch.randn(wshape, generator=g, device=dev) * 0.02))
            wkind, wbytes = linalg.W_BF16, 2
        else:
            ws.append(torch.randint(-127, 128, wshape, generator=g, device=dev, dtype=torch.int8))
            wbytes = 1
            if args.wkind == "int8":
                wkind, scale = linalg.W_INT8_EXP, torch.randint(-10, -5, (n,), generator=g, device=dev, dtype=torch.int32)
            else:
                wkind, scale = linalg.W_INT8_SCALE, torch.rand((n,), generator=g, device=dev) * 0.019 + 0.001
    c = torch.empty((m, n), device=dev)

    def run(i):
        torch_ops.product(a, ws[i % len(ws)], scale, wkind, op, out=c, plan=args.plan, group_leaves=args.groups)

    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run(0)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.reps):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    else:
        e0.record()
        for i in range(args.reps):
            run(i)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.reps
    nbytes = m * k * 4 + n * k * wbytes + (n * 4 if scale is not None else 0) + m * n * 4
    print(json.dumps({"m": m, "n": n, "k": k, "op": args.op, "wkind": args.wkind, "plan": args.plan, "groups": args.groups, "graph": bool(args.graph),
                      "ms": ms, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12, "algorithmic_gbs": nbytes / (ms * 1e-3) / 1e9}))


def int8_product(args, dev, g):
    m, n, k = args.m, args.n, args.k
    qa = torch.randint(-127, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
    ea = torch.randint(-10, -5, (m,), generator=g, device=dev, dtype=torch.int32)
    qbs = [torch.randint(-127, 128, (n, k), generator=g, device=dev, dtype=torch.int8) for _ in range(args.buffers)]
    eb = torch.randint(-10, -5, (n,), generator=g, device=dev, dtype=torch.int32)
    if args.wkind == "int15i64":  # the low planes hold [0, 127]
        al = torch.randint(0, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
        bl = torch.randint(0, 128, (n, k), generator=g, device=dev, dtype=torch.int8)

        def run(i):
            torch_ops.matmul_int15(qa, al, ea, qbs[i % len(qbs)], bl, eb)
    else:
        def run(i):
            torch_ops.matmul_int8(qa, ea, qbs[i % len(qbs)], eb)
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.reps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.reps
    print(json.dumps({"m": m, "n": n, "k": k, "op": "NT", "wkind": args.wkind, "ms": ms, "tops": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
                      "algorithmic_gbs": (m * k + n * k + 4 * m * n) / (ms * 1e-3) / 1e9}))


if __name__ == "__main__":
    main()
