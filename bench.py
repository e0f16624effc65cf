"""Benchmark of the identical-mode matrix product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A STEP is one pass of the product over the FP32 GEMM shape sweep of the
baseline's second configuration: (M, N, K) in {(4096, 4096, 4096),
(8192, 8192, 1024), (128, 11008, 4096), (2048, 50304, 768), (1000, 1000, 1000)},
operands i.i.d. N(0, 1) float32 from seed 0, linear-layer orientation
C = A . W^T. The metric is whole-job GFLOP/s with 2*M*N*K flops per product.

  value   operands resident in HBM, CUDA-event timed on the launching stream.
  e2e     the same sweep through the public host-buffer call
          (mojolearn_b200.linalg.matmul) from pinned host memory, uploads and
          downloads inside the timed region.
  roofline        the tiled GEMM kernel against the FP32 fused-multiply-add peak
                  (an in-run probe; the contract's one-rounding-per-step chain
                  cannot run on tensor cores).
  roofline_decode the row-streaming decode kernel (INT8 weights [11008, 4096],
                  one activation row) against the measured HBM copy bandwidth.
  cpu_baseline    the reference's CPU algorithm (AVX2 restatement, all host
                  threads) on a bounded sample of the same sweep.

With --impl reference the CPU algorithm itself is the timed arm. Under torchrun
(N > 1) every rank runs the sweep on its own shard of a batch N times larger
(rows of A are independent), there is no data-path collective, and the value
is the total work over the slowest rank's time.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SWEEP = [(4096, 4096, 4096), (8192, 8192, 1024), (128, 11008, 4096), (2048, 50304, 768), (1000, 1000, 1000)]
DECODE_N, DECODE_K = 11008, 4096
CONFIG1 = (1024, 1024, 1024)
# DRAM bytes of one launch from the committed ncu captures (profiles/): the bench cannot read counters itself
DECODE_INT8_M1_DRAM_BYTES = 45202944  # profiles/decode_pair_kernel_int8_m1_11008x4096.md
PACKED_4096_DRAM_BYTES = 1060e6 + 940.4e6  # dram__bytes_read + dram__bytes_write of one 4096-cubed launch (profiles/gemm_packed_kernel_4096cubed.md)


def sweep_flops(shapes):
    return sum(2.0 * m * n * k for m, n, k in shapes)


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([v.strip() for v in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, power) if p > 250.0] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample_shapes(target_seconds, gflops_guess):
    """A bounded sample of the sweep for the CPU arm: every shape keeps its n and k
    (k is what the leaf rule and the fold read) and takes the first rows of A."""
    budget = target_seconds * gflops_guess * 1e9
    per_row = sum(2.0 * n * k for _, n, k in SWEEP)
    rows = max(8, int(budget / per_row))
    return [(min(m, rows), n, k) for m, n, k in SWEEP]


def run_cpu(shapes, steps, warmup, threads):
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    ops = []
    for m, n, k in shapes:
        ops.append((rng.standard_normal((m, k), dtype=np.float32), rng.standard_normal((n, k), dtype=np.float32)))
    for _ in range(warmup):
        for a, w in ops[2:3]:
            oracle.gemm_rows(a[:8], w, oracle.OP_NT, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        for a, w in ops:
            oracle.gemm_rows(a, w, oracle.OP_NT, threads=threads)
    dt = time.perf_counter() - t0
    return sweep_flops(shapes) * steps / dt / 1e9, dt


def serve_oracle_row0(serve_bench, kept, sargs, gpu_hash):
    """Sequence 0 of the serving run through the CPU oracle: one teacher-forced forward over its prompt and its
    generated ids, whose last position holds the logits the run ended on. Checker only, never timed as product."""
    import hashlib
    import oracle
    cfg, row = kept["cfg"], kept["row0_ids"]
    w = serve_bench.build_weights(cfg, sargs.format)  # the run's own weights again (fixed device generator)

    def host(layer):
        if getattr(layer, "scale", None) is None:
            return layer.w.cpu().numpy()
        return oracle.dequantize_int8(layer.w.cpu().numpy(), layer.scale.cpu().numpy())

    def slots(i):
        p = "model.layers.%d." % i
        names = dict(q="self_attn.q_proj", k="self_attn.k_proj", v="self_attn.v_proj", o="self_attn.o_proj",
                     gate="mlp.gate_proj", up="mlp.up_proj", down="mlp.down_proj")
        out = {slot: host(w[p + name + ".weight"]) for slot, name in names.items()}
        out["norm1"] = w[p + "input_layernorm.weight"].cpu().numpy()
        out["norm2"] = w[p + "post_attention_layernorm.weight"].cpu().numpy()
        return out

    t0 = time.perf_counter()
    want = oracle.teacher_forced_logits(cfg, row, len(row) - 1, slots, w["model.embed_tokens.weight"].cpu().numpy(), None,
                                        w["model.norm.weight"].cpu().numpy(), None, host(w["lm_head.weight"]))
    digest = hashlib.sha256(want[0].tobytes()).hexdigest()[:16]
    return {"logits_sha256": digest, "equal": digest == gpu_hash, "positions": int(len(row)), "cpu_seconds": time.perf_counter() - t0,
            "what": "sequence 0 (prompt + generated ids) through the CPU oracle, logits after the last token"}


def reference_arm(args, rank, world):
    """The reference's CPU implementation of the path (its AVX2 host product,
    restated; the reference itself is Mojo and cannot be built here), all host
    threads, on a bounded sample of the sweep."""
    if rank != 0:
        return
    threads = host_threads()
    shapes = cpu_sample_shapes(min(4.0, 60.0 / max(args.steps, 1)), 25.0 * threads)  # the whole run stays near a minute
    gflops, dt = run_cpu(shapes, args.steps, min(args.warmup, 1), threads)
    sample = "first rows of A per sweep shape, n and k exact: " + ", ".join("%dx%dx%d" % s for s in shapes)
    line = {"impl": "reference", "metric": "identical_fp32_gemm_gflops", "value": gflops, "unit": "GFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "fp32_gemm_shape_sweep (baseline config 2), CPU arm on a bounded sample", "op": "NT",
                       "shapes": [list(s) for s in shapes]},
            "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-serve", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from mojolearn_b200 import _native, linalg, torch_ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _native.lib()
    args.warmup = max(args.warmup, 3)

    # ---- operands resident in HBM (1.5 GB per pass: far beyond the 126 MB L2) ----
    gen = torch.Generator(device=dev).manual_seed(rank)
    ops = []
    for m, n, k in SWEEP:
        a = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32)
        w = torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32)
        c = torch.empty((m, n), device=dev, dtype=torch.float32)
        ops.append((a, w, c))

    def one_pass():
        for a, w, c in ops:
            torch_ops.matmul(a, w, transpose_b=True, out=c)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        one_pass()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = lib.b200i_launch_count()
    lib.b200i_kernel_timing(1)  # event pairs around every product's main kernel, on the launching stream
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    shape_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(SWEEP) + 1)] for _ in range(args.steps)]
    barrier()
    ev[0].record()
    for s in range(args.steps):
        shape_ev[s][0].record()
        for i, (a, w, c) in enumerate(ops):
            torch_ops.matmul(a, w, transpose_b=True, out=c)
            shape_ev[s][i + 1].record()
    ev[1].record()
    barrier()
    elapsed_ms = ev[0].elapsed_time(ev[1])
    launches = lib.b200i_launch_count() - launches0
    kernel_ms, kernel_calls = ctypes.c_double(0.0), ctypes.c_int64(0)
    lib.b200i_kernel_timing_read(ctypes.byref(kernel_ms), ctypes.byref(kernel_calls))
    lib.b200i_kernel_timing(0)
    clocks = sampler.stop() if rank == 0 else None
    per_shape_ms = [statistics.mean(shape_ev[s][i].elapsed_time(shape_ev[s][i + 1]) for s in range(args.steps))
                    for i in range(len(SWEEP))]
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    flops_step = sweep_flops(SWEEP) * world
    value = flops_step * args.steps / (elapsed_ms * 1e-3) / 1e9

    # ---- FP32 peak probe (scalar and packed fused multiply-add) ----
    scratch = torch.zeros(4, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    peaks = {}
    for packed in (0, 1):
        blocks, iters = sms * 8, 20000
        for _ in range(2):
            _native.call("b200i_ffma_probe", local_rank, None, ctypes.c_void_p(scratch.data_ptr()), blocks, iters, packed)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.default_stream(dev))
        for _ in range(3):
            _native.call("b200i_ffma_probe", local_rank, None, ctypes.c_void_p(scratch.data_ptr()), blocks, iters, packed)
        e1.record(torch.cuda.default_stream(dev))
        torch.cuda.synchronize(dev)
        fl = 3.0 * blocks * 256 * 16 * iters * 2 * (2 if packed else 1)
        peaks["packed" if packed else "scalar"] = fl / (e0.elapsed_time(e1) * 1e-3) / 1e12
    fp32_peak = max(peaks.values())

    # the dominant kernel: each product's main kernel (gemm_packed_kernel on all five shapes), timed by the
    # library's own event pairs: operand packing and the group fold are outside these pairs and inside `value`
    tile_flops = sweep_flops(SWEEP) * (kernel_calls.value / float(len(SWEEP)))  # the pairs recorded (the library keeps 4096)
    tile_ms = float(kernel_ms.value)
    tile_tflops = tile_flops / (tile_ms * 1e-3) / 1e12 if tile_ms > 0 else 0.0
    sm_max = (clocks or {}).get("sm_max_mhz") or 1965.0
    roofline = {"bound": "fp32_ffma", "kernel": "gemm_packed_kernel (128x128 tiles, bulk-copy ring)", "achieved": tile_tflops,
                "peak": fp32_peak, "unit": "TFLOP/s", "frac": tile_tflops / fp32_peak if fp32_peak else None,
                "kernel_launches_timed": int(kernel_calls.value),
                "kernel_ms_per_step": tile_ms / max(kernel_calls.value / float(len(SWEEP)), 1.0),
                "peak_source": "in-run fused-multiply-add probe (max of scalar %.1f and packed f32x2 %.1f TFLOP/s); nominal %d SMs x 128 lanes x 2 x %.0f MHz = %.1f"
                % (peaks["scalar"], peaks["packed"], sms, sm_max, sms * 128 * 2 * sm_max * 1e6 / 1e12),
                "launch_ms": {"%dx%dx%d" % SWEEP[i]: per_shape_ms[i] for i in range(len(SWEEP))},
                "per_shape": {"%dx%dx%d" % SWEEP[i]: {"ms": per_shape_ms[i], "tflops": 2.0 * SWEEP[i][0] * SWEEP[i][1] * SWEEP[i][2] / (per_shape_ms[i] * 1e-3) / 1e12,
                                                       "frac_fp32": 2.0 * SWEEP[i][0] * SWEEP[i][1] * SWEEP[i][2] / (per_shape_ms[i] * 1e-3) / 1e12 / fp32_peak}
                              for i in range(len(SWEEP))},
                "algorithmic_bytes_per_step": int(sum(4 * (m * k + n * k + m * n) for m, n, k in SWEEP)),
                # DRAM bytes cannot be read inside the bench: the committed ncu capture of the 4096-cubed launch is scaled to the
                # sweep by multiply-adds (the panels and the fold traffic both grow with m * n * k / tile)
                "traffic": (PACKED_4096_DRAM_BYTES * sweep_flops(SWEEP) / (2.0 * 4096 ** 3)) if PACKED_4096_DRAM_BYTES else None,
                "traffic_source": "profiles/gemm_packed_kernel_4096cubed.md (one 4096-cubed launch), scaled to a step by multiply-adds"}

    # ---- configuration 1: M = N = K = 1024, U(-1, 1) from seed 0, row-major C = A . B, timed on its own ----
    g1 = torch.Generator(device=dev).manual_seed(0)
    a1 = torch.rand((CONFIG1[0], CONFIG1[2]), generator=g1, device=dev) * 2.0 - 1.0
    b1 = torch.rand((CONFIG1[2], CONFIG1[1]), generator=g1, device=dev) * 2.0 - 1.0
    c1 = torch.empty((CONFIG1[0], CONFIG1[1]), device=dev)
    flush = torch.empty((160 << 20,), dtype=torch.uint8, device=dev)  # larger than L2: written between timed launches
    for _ in range(3):
        torch_ops.matmul(a1, b1, out=c1)
    c1_ms = []
    for _ in range(10):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch_ops.matmul(a1, b1, out=c1)
        e1.record()
        torch.cuda.synchronize(dev)
        c1_ms.append(e0.elapsed_time(e1))
    c1_us = statistics.median(c1_ms) * 1e3
    config1 = {"shape": list(CONFIG1), "op": "NN", "operands": "U(-1, 1) float32, torch generator seed 0", "us": c1_us,
               "tflops": 2.0 * CONFIG1[0] * CONFIG1[1] * CONFIG1[2] / (c1_us * 1e-6) / 1e12,
               "frac_fp32": 2.0 * CONFIG1[0] * CONFIG1[1] * CONFIG1[2] / (c1_us * 1e-6) / 1e12 / fp32_peak,
               "l2": "a 160 MB buffer is written between timed launches", "launches_timed": 10}
    del a1, b1, c1

    # ---- the int8 x int8 -> int32 product profile (tensor cores): 4096 cubed, timed on its own like configuration 1 ----
    gi = torch.Generator(device=dev).manual_seed(3)
    qa8 = torch.randint(-127, 128, (4096, 4096), generator=gi, device=dev, dtype=torch.int8)
    qb8 = torch.randint(-127, 128, (4096, 4096), generator=gi, device=dev, dtype=torch.int8)
    ea8 = torch.randint(-10, -5, (4096,), generator=gi, device=dev, dtype=torch.int32)
    eb8 = torch.randint(-10, -5, (4096,), generator=gi, device=dev, dtype=torch.int32)
    for _ in range(3):
        torch_ops.matmul_int8(qa8, ea8, qb8, eb8)
    i8_ms = []
    for _ in range(10):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch_ops.matmul_int8(qa8, ea8, qb8, eb8)
        e1.record()
        torch.cuda.synchronize(dev)
        i8_ms.append(e0.elapsed_time(e1))
    i8_us = statistics.median(i8_ms) * 1e3
    i8_tops = 2.0 * 4096 ** 3 / (i8_us * 1e-6) / 1e12
    int8_product = {"kernel": "gemm_int8_tma_kernel (tensor-map copies, tcgen05.mma kind::i8, two int32 accumulators in tensor memory)", "shape": [4096, 4096, 4096],
                    "us": i8_us, "tops": i8_tops, "bound": "tensor", "peak": 4500.0, "unit": "TOP/s", "frac": i8_tops / 4500.0,
                    "peak_source": "nominal dense int8 rate of the part (twice the nominal bf16 rate; no measured int8 figure exists)",
                    "l2": "a 160 MB buffer is written between timed launches", "launches_timed": 10,
                    "note": "no baseline configuration uses this product profile; it is the one place of the path where an MMA is contract-legal"}
    # the fifteen-bit profile on the same shape: four int8 plane products per cell (2 * m * n * k counted once)
    al8 = torch.randint(0, 128, (4096, 4096), generator=gi, device=dev, dtype=torch.int8)
    bl8 = torch.randint(0, 128, (4096, 4096), generator=gi, device=dev, dtype=torch.int8)
    for _ in range(3):
        torch_ops.matmul_int15(qa8, al8, ea8, qb8, bl8, eb8)
    i15_ms = []
    for _ in range(10):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch_ops.matmul_int15(qa8, al8, ea8, qb8, bl8, eb8)
        e1.record()
        torch.cuda.synchronize(dev)
        i15_ms.append(e0.elapsed_time(e1))
    i15_us = statistics.median(i15_ms) * 1e3
    int8_product["int15i64"] = {"kernel": "gemm_int15_tma_kernel (two int8 planes per operand, three int32 accumulators, recombined in int64)",
                                "shape": [4096, 4096, 4096], "us": i15_us, "tops": 2.0 * 4096 ** 3 / (i15_us * 1e-6) / 1e12,
                                "mma_tops": 4 * 2.0 * 4096 ** 3 / (i15_us * 1e-6) / 1e12, "frac_mma": 4 * 2.0 * 4096 ** 3 / (i15_us * 1e-6) / 1e12 / 4500.0}
    del flush, qa8, qb8, ea8, eb8, al8, bl8

    # ---- decode kernel against HBM: weights [11008, 4096] in three storage kinds, one activation row ----
    peaks_file = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm_peak, hbm_src = 6650.0, "fallback"
    if os.path.exists(peaks_file):
        try:
            hbm_peak, hbm_src = float(json.load(open(peaks_file))["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    from mojolearn_b200.linalg import OP_NT, W_BF16, W_F32, W_INT8_EXP, W_INT8_SCALE
    g2 = torch.Generator(device=dev).manual_seed(100 + rank)
    we = torch.randint(-10, -5, (DECODE_N,), generator=g2, device=dev, dtype=torch.int32)
    ws = torch.rand((DECODE_N,), generator=g2, device=dev) * 0.019 + 0.001  # per-row float32 scales U(0.001, 0.02)
    decode = {}
    for kind_name, wkind, wbytes, nbuf, rows in (("int8", W_INT8_EXP, 1, 6, (1, 8, 32, 128)), ("int8_f32scale", W_INT8_SCALE, 1, 6, (1, 8, 32, 128)),
                                                 ("bf16", W_BF16, 2, 4, (1, 8, 32, 128)), ("f32", W_F32, 4, 3, (1, 8))):
        # nbuf weight buffers rotate through, so no launch finds its weights in the 126 MB L2
        if wbytes == 1:
            wq = [torch.randint(-127, 128, (DECODE_N, DECODE_K), generator=g2, device=dev, dtype=torch.int8) for _ in range(nbuf)]
        elif wkind == W_BF16:
            wq = [torch_ops.to_bf16(torch.randn((DECODE_N, DECODE_K), generator=g2, device=dev) * 0.02) for _ in range(nbuf)]
        else:
            wq = [torch.randn((DECODE_N, DECODE_K), generator=g2, device=dev) * 0.02 for _ in range(nbuf)]
        scale = we if wkind == W_INT8_EXP else (ws if wkind == W_INT8_SCALE else None)
        for mrows in rows:
            x = torch.randn((mrows, DECODE_K), generator=g2, device=dev)
            y = torch.empty((mrows, DECODE_N), device=dev)
            reps = 4
            for i in range(nbuf):
                torch_ops.product(x, wq[i], scale, wkind, OP_NT, out=y)
            torch.cuda.synchronize(dev)
            # the launches are replayed from one CUDA graph, so the host's launch cost is not in the number
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps):
                    for i in range(nbuf):
                        torch_ops.product(x, wq[i], scale, wkind, OP_NT, out=y)
            graph.replay()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            us = e0.elapsed_time(e1) * 1e3 / (reps * nbuf)
            nbytes = mrows * DECODE_K * 4 + DECODE_N * DECODE_K * wbytes + (DECODE_N * 4 if scale is not None else 0) + mrows * DECODE_N * 4
            flops = 2.0 * mrows * DECODE_N * DECODE_K
            # the floor of one launch: the slower of its bytes at the measured HBM rate and its flops at the FP32 peak
            floor_us = max(nbytes / (hbm_peak * 1e9), flops / (fp32_peak * 1e12)) * 1e6
            decode[(kind_name, mrows)] = {"us": us, "gbs": nbytes / (us * 1e-6) / 1e9, "bytes": nbytes, "frac_hbm": nbytes / (us * 1e-6) / 1e9 / hbm_peak,
                                          "tflops": flops / (us * 1e-6) / 1e12, "frac_fp32": flops / (us * 1e-6) / 1e12 / fp32_peak,
                                          "floor_us": floor_us, "frac_of_floor": floor_us / us,
                                          "bound": "hbm" if nbytes / (hbm_peak * 1e9) >= flops / (fp32_peak * 1e12) else "fp32"}
            del graph
        del wq
    d1 = decode[("int8", 1)]
    roofline_decode = {"bound": "hbm", "kernel": "decode_pair_kernel<int8,1>", "achieved": d1["gbs"], "peak": hbm_peak, "unit": "GB/s",
                       "frac": d1["gbs"] / hbm_peak, "peak_source": hbm_src + " HBM copy bandwidth", "us_per_launch": d1["us"],
                       "algorithmic_bytes": d1["bytes"], "traffic": DECODE_INT8_M1_DRAM_BYTES,
                       "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, profiles/decode_pair_kernel_int8_m1_11008x4096.md",
                       "timing": "CUDA events around one graph replay of 24 launches",
                       "workload": "W[11008, 4096] (baseline configuration 3), rows M in {1, 8, 32, 128}: int8 + int32 row exponents, "
                                   "int8 + float32 row scales U(0.001, 0.02), bf16; float32 at 1 and 8 rows",
                       "all": {"%s_m%d" % k: v for k, v in decode.items()}}
    nbuf = 6

    # ---- end to end: host buffers through linalg.matmul, pinned memory ----
    e2e = None
    if not args.skip_e2e:
        host = []
        for (m, n, k), (a, w, c) in zip(SWEEP, ops):
            ha = torch.empty((m, k), dtype=torch.float32).pin_memory()
            hw = torch.empty((n, k), dtype=torch.float32).pin_memory()
            hc = torch.empty((m, n), dtype=torch.float32).pin_memory()
            ha.copy_(a)
            hw.copy_(w)
            host.append((ha.numpy(), hw.numpy(), hc.numpy()))
        e2e_steps = max(1, min(args.steps, 3))
        for ha, hw, hc in host:
            linalg.matmul(ha, hw, transpose_b=True, out=hc)
        barrier()
        t0 = time.perf_counter()
        e2e_shape_s = [0.0] * len(host)
        for _ in range(e2e_steps):
            for i, (ha, hw, hc) in enumerate(host):
                t1 = time.perf_counter()
                linalg.matmul(ha, hw, transpose_b=True, out=hc)  # returns with the result in host memory
                e2e_shape_s[i] += time.perf_counter() - t1
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        e2e = {"value": flops_step * e2e_steps / dt / 1e9, "unit": "GFLOP/s",
               "h2d_bytes_per_step": int(sum(4 * (m * k + n * k) for m, n, k in SWEEP)),
               "d2h_bytes_per_step": int(sum(4 * m * n for m, n, k in SWEEP)), "steps": e2e_steps,
               "ms_per_shape": {"%dx%dx%d" % SWEEP[i]: 1e3 * e2e_shape_s[i] / e2e_steps for i in range(len(SWEEP))},
               "api": "mojolearn_b200.linalg.matmul(a, w, transpose_b=True, out=...) on pinned host arrays"}
        del host

    # ---- CPU baseline on rank 0 at N = 1 ----
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        threads = host_threads()
        shapes = cpu_sample_shapes(4.0, 25.0 * threads)
        _, probe_dt = run_cpu(shapes, 1, 1, threads)
        passes = max(1, min(20, int(12.0 / max(probe_dt, 0.05))))  # about 12 s of CPU work
        gflops, dt = run_cpu(shapes, passes, 0, threads)
        cpu = {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "seconds": dt,
               "sample": "%d passes over the first rows of A per sweep shape, n and k exact: " % passes
                         + ", ".join("%dx%dx%d" % s for s in shapes)}

    # ---- decoder serving, baseline configuration 5 (INT8 weights), sharded by output columns when N > 1 ----
    serve = None
    if not args.skip_serve:
        import argparse as _ap
        from mojolearn_b200 import serve_bench
        # all 256 greedy steps are run; the last 64 are the timed ones (the caches are then at 1216 .. 1279 positions)
        sargs = _ap.Namespace(layers=24, d_model=2048, heads=16, mlp=8192, vocab=50304, batch=32, prompt=1024, decode=256,
                              timed_steps=64, format="int8", no_graph=False)
        del ops
        torch.cuda.empty_cache()
        kept = {}
        serve, _ = serve_bench.run(sargs, keep=kept)
        if rank == 0 and world == 1 and not args.skip_cpu:
            serve["oracle_row0"] = serve_oracle_row0(serve_bench, kept, sargs, serve["row0_logits_sha256"])
        if world > 1:
            # the single-GPU figure of the same run, on rank 0 alone while the others wait: the sharded tokens/s over
            # N times this one is the scaling efficiency, and the hashes say the sharded logits are the same words
            solo = None
            torch.cuda.empty_cache()
            if rank == 0:
                solo, _ = serve_bench.run(sargs, solo=True)
            dist.barrier()
            if rank == 0:
                serve["scaling"] = {"1": {"tokens_per_s": solo["value"], "ms_per_decode_step": solo["ms_per_decode_step"],
                                          "prefill_ms": solo["prefill_ms"]},
                                    str(world): {"tokens_per_s": serve["value"], "ms_per_decode_step": serve["ms_per_decode_step"],
                                                 "prefill_ms": serve["prefill_ms"],
                                                 "decode_efficiency": serve["value"] / (world * solo["value"]),
                                                 "prefill_efficiency": solo["prefill_ms"] / (world * serve["prefill_ms"])},
                                    "kind": "strong (the batch of 32 is fixed)",
                                    "bit_identical_to_1gpu": solo["ids_sha256"] == serve["ids_sha256"] and solo["logits_sha256"] == serve["logits_sha256"]}

    if rank == 0:
        line = {"metric": "identical_fp32_gemm_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "fp32_gemm_shape_sweep (baseline config 2)", "op": "NT (C = A . W^T)",
                           "shapes": [list(s) for s in SWEEP], "operands": "N(0,1) float32, torch generator seed = rank",
                           "l2": "inputs larger than L2: one pass reads 1.5 GB of operands",
                           "bit_exact": "every product is the oracle's bits (tests/test_gpu_gemm.py)"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "roofline_decode": roofline_decode, "cpu_baseline": cpu, "config1": config1, "int8_product": int8_product,
                "decode": {"metric": "int8w_matvec_rows_per_s", "value": 1e6 / d1["us"], "unit": "rows/s",
                           "weights": "int8 [11008, 4096] + int32 row exponents", "rotating_weight_buffers": nbuf},
                "serve": serve}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
