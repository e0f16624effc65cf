"""Decoder serving benchmark: INT8-weight decode tokens/s (baseline configuration 5).

    python -m mojolearn_b200.serve_bench [--layers 24] [--d-model 2048] [--heads 16] [--mlp 8192] [--vocab 50304]
                                         [--batch 32] [--prompt 1024] [--decode 256] [--timed-steps 32] [--format int8]
    torchrun --nproc-per-node N -m mojolearn_b200.serve_bench ...   (output-column sharded, NCCL all-gather)

Random-init weights N(0, 0.02) quantised per row to int8 codes with power-of-two
exponents, uniform random token ids, prefill on the prompt, then greedy decode
steps timed with CUDA events (max over ranks). Prints one JSON line on rank 0,
with a hash of the generated ids and of the last logits so runs at different N
can be compared word for word.
"""
import argparse
import hashlib
import json
import os

import numpy as np
import torch

from . import _native, _prof
from .models import CausalLM, CausalLMConfig


def build_weights(cfg, fmt, seed=0):
    """Random-init weights built and quantised on the device (nothing crosses the host)."""
    from . import torch_ops
    from .linalg import W_BF16, W_INT8_EXP
    from .transformer import Linear
    g = torch.Generator(device="cuda").manual_seed(seed)

    def mat(*shape):
        return torch.randn(shape, generator=g, device="cuda") * 0.02

    def proj(*shape):
        a = mat(*shape)
        if fmt == "int8":
            codes, exps = torch_ops.quantize_int8(a)
            return Linear.from_device(codes, exps, W_INT8_EXP)
        if fmt == "bfloat16":
            return Linear.from_device(torch_ops.to_bf16(a), None, W_BF16)
        return Linear.from_device(a)

    dm, hd, nh, nkv, it = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate
    ones = torch.ones(dm, device="cuda")
    w = {"model.embed_tokens.weight": mat(cfg.vocab, dm), "model.norm.weight": ones, "lm_head.weight": proj(cfg.vocab, dm)}
    for i in range(cfg.n_layers):
        p = "model.layers.%d." % i
        w[p + "input_layernorm.weight"] = ones
        w[p + "post_attention_layernorm.weight"] = ones
        w[p + "self_attn.q_proj.weight"] = proj(nh * hd, dm)
        w[p + "self_attn.k_proj.weight"] = proj(nkv * hd, dm)
        w[p + "self_attn.v_proj.weight"] = proj(nkv * hd, dm)
        w[p + "self_attn.o_proj.weight"] = proj(dm, nh * hd)
        w[p + "mlp.gate_proj.weight"] = proj(it, dm)
        w[p + "mlp.up_proj.weight"] = proj(it, dm)
        w[p + "mlp.down_proj.weight"] = proj(dm, it)
    return w


def build_ids(cfg, batch, prompt, device=None):
    """The benchmark's prompt: uniform random token ids from a fixed device generator."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    gen = torch.Generator(device=dev).manual_seed(1)
    return torch.randint(0, cfg.vocab, (batch, prompt), generator=gen, device=dev, dtype=torch.int32)


def run(args, solo=False, keep=None):
    """One serving run. `solo`: ignore the process group and run the whole model on this rank's GPU alone (the
    single-GPU figure a sharded run is compared with). `keep`: a dict that receives what a checker needs to replay
    sequence 0 elsewhere (its prompt + generated ids, the plan)."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if solo:
        rank, world = 0, 1
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    cfg = CausalLMConfig(vocab=args.vocab, d_model=args.d_model, n_layers=args.layers, n_heads=args.heads,
                         intermediate=args.mlp, max_positions=8192)
    emulate = int(getattr(args, "emulate_world", 0) or 0) if world == 1 else 0
    lm = CausalLM(cfg, build_weights(cfg, args.format), device=dev, group=group, emulate_world=emulate,
                  prefill_by_batch=os.environ.get("MOJOLEARN_B200_PREFILL", "batch") != "columns")
    ids = build_ids(cfg, args.batch, args.prompt, dev)
    # warm-up, untimed: a short prompt and three steps load every kernel, open the collectives' connections and
    # the peer exchange, and capture a decode graph once
    lm.generate(ids[:, :min(16, args.prompt)].contiguous(), 3, graph=not args.no_graph)
    torch.cuda.synchronize(dev)
    state = lm.allocate_state(args.batch, args.prompt + args.decode)
    launches0 = _native.lib().b200i_launch_count()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    torch.cuda.synchronize(dev)
    e[0].record()
    logits = lm.forward_device(ids, state, last_only=True)
    e[1].record()
    steps, timed, toks = args.decode, min(args.timed_steps, args.decode), []
    session = lm.decode_session(state, logits, graph=not args.no_graph)
    for step in range(steps):
        if step == steps - timed:
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize(dev)
            if getattr(args, "breakdown", False):
                _prof.enable(True)
            e[2].record()
        toks.append(session.next_ids().clone())
        logits = session.step()
    e[3].record()
    torch.cuda.synchronize(dev)
    breakdown = None
    if getattr(args, "breakdown", False):
        breakdown = {k: {"us_per_step": v["us"] / timed, "spans_per_step": v["spans"] / timed} for k, v in sorted(_prof.report().items())}
        _prof.enable(False)
    t = torch.tensor([e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3])], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    prefill_ms, decode_ms = float(t[0]), float(t[1])
    lm.check_ids()
    seq = torch.cat(toks, dim=1).cpu().numpy()
    out = {"metric": "int8w_decode_tokens_per_s", "value": args.batch * timed / (decode_ms * 1e-3), "unit": "tokens/s",
           "n_gpus": world, "ms_per_decode_step": decode_ms / timed, "prefill_ms": prefill_ms,
           "prefill_tokens_per_s": args.batch * args.prompt / (prefill_ms * 1e-3), "timed_steps": timed,
           "config": {"layers": args.layers, "d_model": args.d_model, "heads": args.heads, "mlp": args.mlp, "vocab": args.vocab,
                      "batch": args.batch, "prompt": args.prompt, "decode": args.decode, "weights": args.format,
                      "decode_step": "launch by launch" if args.no_graph else "CUDA graph replay",
                      "sharding": ("output columns over %d ranks" % world if world > 1 else
                                   ("rank 0's share of %d ranks on one GPU, loopback gathers: TIMING ONLY, not the model's outputs" % emulate
                                    if emulate else "none")),
                      "gathers": ("peer stores" if lm.exchange is not None else "NCCL all-gather") if world > 1 else "none",
                      "prefill": ("cut by sequences, KV re-cut by one all-to-all" if lm.prefill_by_batch else "cut by output columns") if world > 1 else "one GPU"},
           "ids_sha256": hashlib.sha256(seq.tobytes()).hexdigest()[:16],
           "logits_sha256": hashlib.sha256(logits.cpu().numpy().tobytes()).hexdigest()[:16],
           # sequence 0 alone: the logits after its last generated token
           "row0_logits_sha256": hashlib.sha256(logits[0].cpu().numpy().tobytes()).hexdigest()[:16],
           # the library counts a captured launch once, at capture, when nothing runs; replays are counted here
           "gpu_launches": int(_native.lib().b200i_launch_count() - launches0 + (session.replays - 1) * session.graph_launches
                               if session.replays else _native.lib().b200i_launch_count() - launches0)}
    if breakdown is not None:
        out["breakdown_rank0"] = breakdown
    if keep is not None:
        import numpy as np
        keep["cfg"] = cfg
        keep["row0_ids"] = np.concatenate([ids[0].cpu().numpy().reshape(-1), seq[0].reshape(-1)]).astype(np.int32)
    return out, rank


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--mlp", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--timed-steps", type=int, default=32)
    ap.add_argument("--format", default="int8", choices=["int8", "bfloat16", "float32"])
    ap.add_argument("--no-graph", action="store_true", help="launch every decode step kernel by kernel")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="one process, one GPU: time rank 0's share of a model cut over this many ranks (loopback gathers)")
    ap.add_argument("--breakdown", action="store_true",
                    help="with --no-graph: CUDA event pairs around each class of work of the timed steps (rank 0's are printed)")
    args = ap.parse_args()
    out, rank = run(args)
    if rank == 0:
        print(json.dumps(out))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
