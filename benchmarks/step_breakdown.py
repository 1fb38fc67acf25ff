"""Where one engine step goes: per-kernel-class device time of a decode or prefill step.

The forward of one step is captured in a CUDA graph while every native launch is recorded (entry point and
arguments). The whole graph is then replayed and timed with CUDA events, and so is one graph per launch class
(entry point + its integer arguments, which separates the four GEMM shapes of a layer) holding only that class's
launches in their original order. Because a class graph replays the launches of all layers back to back, each
layer reading its own weights and cache, its time per launch includes the launch-to-launch cost inside a graph and
sees a cold L2, like the real step. The sum over classes against the time of the full graph shows what the
dependency chain itself costs.

  python benchmarks/step_breakdown.py --phase decode --batch 64 --ctx 2176                  (one GPU, TP1 shapes)
  python benchmarks/step_breakdown.py --phase decode --emulate-tp 8                          (one GPU, the shapes
        of one rank of an 8-way tensor-parallel job, no communication)
  torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/step_breakdown.py --phase decode   (real TP ranks;
        communication kernels appear as classes of their own, every rank replays the same graphs in the same order)

``--phase both`` times a decode and a prefill step of the same model; ``--variants`` repeats the measurement under
several settings of the environment switches (read per call by the communication layer) without starting over.

Prints one JSON line per table (rank 0); ``bench.py --breakdown`` calls the same function.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from collections import OrderedDict

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _class_key(name, args):
    ints = []
    for a in args:
        if isinstance(a, bool):
            continue
        if isinstance(a, int) and 0 <= a < (1 << 20):
            ints.append(a)
    return name.replace("ksana_", "") + "(" + ",".join(str(i) for i in ints[:10]) + ")"


def _time_graph(torch, graph, reps, sync_all=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    if sync_all is not None:
        sync_all()
    times = []
    for _ in range(reps):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
    return statistics.median(times)


def build_step(torch, model, phase, batch, ctx, q_len, block_tokens):
    """A synthetic step: ``batch`` sequences with ``ctx`` tokens of context each; decode = one new token per
    sequence, prefill = ``q_len`` new tokens per sequence (context = those tokens). Blocks are laid out
    sequence by sequence."""
    from ksanallm_b200.models.common import StepInput
    from ksanallm_b200.ops import dispatch as ops
    dev = model.device
    kv = ctx if phase == "decode" else q_len
    bps = (kv + block_tokens - 1) // block_tokens
    table = torch.arange(batch * bps, dtype=torch.int32, device=dev).view(batch, bps)
    kv_lens = torch.full((batch,), kv, dtype=torch.int32, device=dev)
    if phase == "decode":
        T = batch
        pos = torch.full((T,), kv - 1, dtype=torch.int32, device=dev)
        cu_q = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        step_kw = dict(num_multi=0, num_single=batch, num_tokens=T, num_multi_tokens=0, max_q_len=1)
    else:
        T = batch * q_len
        pos = torch.arange(q_len, dtype=torch.int32, device=dev).repeat(batch)
        cu_q = (torch.arange(batch + 1, dtype=torch.int32, device=dev) * q_len).to(torch.int32)
        step_kw = dict(num_multi=batch, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=q_len)
    seq = torch.arange(T, device=dev) // (1 if phase == "decode" else q_len)
    slots = (table[seq.long(), (pos // block_tokens).long()] * block_tokens + pos % block_tokens).to(torch.int32)
    ids = torch.randint(0, model.cfg.vocab_size, (T,), dtype=torch.int32, device=dev)
    rows = None if phase == "decode" else (cu_q[1:] - 1).to(torch.int32)
    step = StepInput(ids, pos, slots, cu_q, kv_lens, table, logits_rows=rows, **step_kw)
    step.max_kv_len = kv
    if phase == "decode":
        step.decode_splits = ops.decode_splits(batch, model.Hkv, kv)
    return step, batch * bps


def run_breakdown(model, phase="decode", batch=64, ctx=2176, q_len=2048, reps=10, block_tokens=16, sync_all=None,
                  classes=True):
    """``classes=False`` times the whole step only: needed when a kernel of one class waits for a flag that a kernel of
    another class raises (a graph of one class alone would wait until its limit)."""
    import torch
    from ksanallm_b200.ops import native
    step, nblocks = build_step(torch, model, phase, batch, ctx, q_len, block_tokens)
    if model.kv_cache is None or model.kv_cache.shape[0] < nblocks:
        model.allocate_kv_cache(nblocks, block_tokens)
    with torch.inference_mode():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            model.forward(step)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        calls = []
        full = torch.cuda.CUDAGraph()
        with native.recording(calls):
            with torch.cuda.graph(full):
                keep = model.forward(step)
        t_full = _time_graph(torch, full, reps, sync_all)
        groups = OrderedDict()
        for name, fn, args in calls:
            groups.setdefault(_class_key(name, args), []).append((fn, args))
        rows = []
        for key, lst in (groups.items() if classes else ()):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st = torch.cuda.current_stream().cuda_stream
                for fn, args in lst:
                    fn(*args[:-1], st)                   # the stream is every entry point's last argument
            t = _time_graph(torch, g, reps, sync_all)
            rows.append({"class": key, "launches": len(lst), "us_total": round(t, 1), "us_each": round(t / len(lst), 2)})
            del g
        native.check_err_flag(model.device)
    s = sum(r["us_total"] for r in rows)
    return {"phase": phase, "batch": batch, "ctx": ctx if phase == "decode" else q_len, "native_launches": len(calls),
            "full_graph_us": round(t_full, 1), "sum_of_classes_us": round(s, 1), "classes": rows, "_keep": keep is not None}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--phase", default="decode", choices=["decode", "prefill", "both"])
    ap.add_argument("--batch", type=int, default=64, help="sequences of the decode step")
    ap.add_argument("--prefill-batch", type=int, default=None, help="sequences of the prefill step (default: --batch)")
    ap.add_argument("--variants", default="", help="settings to time one after the other in this process, e.g. "
                    "'base:;nopush:KSANA_PUSH=0;sig:KSANA_PUSH=1,KSANA_PUSH_SIGNAL=1' (name:VAR=value,...)")
    ap.add_argument("--ctx", type=int, default=2176)
    ap.add_argument("--q-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--emulate-tp", type=int, default=1, help="one GPU: the weight shapes of one rank of this many")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--scale-mode", default="ue8m0", choices=["ue8m0", "fp32"])
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from ksanallm_b200.config import ModelConfig
    from ksanallm_b200.llm import init_distributed
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.ops import reference as ref
    from ksanallm_b200.parallel.comm import TPComm

    rank, world, dev_group, ctl_group, _ = init_distributed("cuda", 1)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    e = args.emulate_tp if world == 1 else 1
    mc = ModelConfig(model_type="llama", hidden_size=8192, num_layers=args.layers, num_heads=64 // e,
                     num_kv_heads=max(1, 8 // e), head_dim=128, intermediate_size=28672 // e,
                     vocab_size=128256 // e, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192,
                     max_token_len=8192, eos_token_ids=[1])
    ref.WEIGHT_SCALE_POW2 = args.scale_mode != "fp32"
    phases = ["decode", "prefill"] if args.phase == "both" else [args.phase]
    pbatch = args.prefill_batch if args.prefill_batch is not None else args.batch
    tokens = max(args.batch if "decode" in phases else 0, pbatch * args.q_len if "prefill" in phases else 0)
    comm = TPComm(dev_group, rank, world, args.comm, dev, max_tokens=max(tokens, 64), hidden=mc.hidden_size) if world > 1 else None
    model = build_model(mc, RandomSource(seed=0, on_device=True), rank, world, comm, dev, torch.bfloat16, "fp8_block",
                        max_positions=max(args.ctx, args.q_len) + 64)

    def sync_all():
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    variants = []
    for item in (args.variants.split(";") if args.variants else [":"]):
        name, _, sets = item.partition(":")
        variants.append((name or "default", dict(kv.split("=", 1) for kv in sets.split(",") if kv)))
    base_env = {k: os.environ.get(k) for _, env in variants for k in env}
    # phase by phase (a prefill step leaves the GPU at the power cap, which would slow the decode step timed after it)
    for phase in phases:
        for name, env in variants:
            for k, v in base_env.items():          # every variant starts from the environment the process was given
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
            os.environ.update(env)
            from ksanallm_b200.utils.clocks import ClockSampler
            sampler = ClockSampler(local, enabled=rank == 0)       # clock record of this table's measurements
            sampler.start()
            res = run_breakdown(model, phase, args.batch if phase == "decode" else pbatch, args.ctx, args.q_len, args.reps,
                                sync_all=sync_all, classes=os.environ.get("KSANA_PUSH_SIGNAL", "0") != "1")
            res.update(world=world, emulate_tp=e, comm=args.comm if world > 1 else None, variant=name, env=env,
                       clocks=sampler.stop() if rank == 0 else None)
            if rank == 0:
                print(json.dumps(res))
                print("== %s / %s %s" % (name, phase, env), file=sys.stderr)
                print("%-58s %6s %10s %8s" % ("class", "n", "us total", "us each"), file=sys.stderr)
                for r in res["classes"]:
                    print("%-58s %6d %10.1f %8.2f" % (r["class"][:58], r["launches"], r["us_total"], r["us_each"]), file=sys.stderr)
                print("full graph %.1f us; sum of classes %.1f us; %d launches; clocks %s" %
                      (res["full_graph_us"], res["sum_of_classes_us"], res["native_launches"], res["clocks"]), file=sys.stderr)
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
