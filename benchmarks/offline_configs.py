"""Offline runs of the named benchmark configurations through the public ``LLM.generate`` API (synthetic prompts,
random-init weights of the named architecture), one JSON line per run.

  b  Llama-3-8B architecture, bf16, 500 requests with log-normal input / output lengths (continuous batching under
     a mixed-length load)
  d  Qwen2-72B architecture (QKV bias), block-scaled FP8 weights so that it fits one GPU, N requests that share a
     2048-token prefix followed by a private 128-token suffix, prefix caching on or off (--no-prefix-cache)
  e  DeepSeek-V3 architecture cut down to fit one GPU (--layers, --experts): latent attention + grouped FP8 experts

  python benchmarks/offline_configs.py --config b
  python -m torch.distributed.run --nproc-per-node 8 benchmarks/offline_configs.py --config d --requests 1024

Timing: one warm-up pass over a tenth of the requests, then the whole request set between synchronisations, CUDA
events on the compute stream, max over ranks. Reported: output tok/s, total (input + output) tok/s, requests/s,
and for d the prefix-cache hit tokens.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_config(name: str, args):
    from ksanallm_b200.config import ModelConfig
    if name == "b":
        return ModelConfig(model_type="llama", hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128,
                           intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                           max_position_embeddings=8192, max_token_len=8192, eos_token_ids=[128001])
    if name == "d":
        return ModelConfig(model_type="qwen", hidden_size=8192, num_layers=args.layers or 80, num_heads=64, num_kv_heads=8,
                           head_dim=128, intermediate_size=29568, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1000000.0,
                           max_position_embeddings=32768, max_token_len=8192, qkv_bias=True, eos_token_ids=[151643])
    if name == "e":
        return ModelConfig(model_type="deepseek_v3", hidden_size=7168, num_layers=args.layers or 6, num_heads=128,
                           num_kv_heads=128, head_dim=192, intermediate_size=18432, vocab_size=129280, rms_norm_eps=1e-6,
                           rope_theta=10000.0, rope_neox=False, max_position_embeddings=4096, max_token_len=4096,
                           num_experts=args.experts or 32, num_experts_per_tok=8, moe_intermediate_size=2048,
                           shared_expert_intermediate_size=2048, num_shared_experts=1, moe_scoring="sigmoid",
                           routed_scaling_factor=2.5, n_group=8, topk_group=4, first_k_dense_replace=1, q_lora_rank=1536,
                           kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, eos_token_ids=[1])
    raise SystemExit(f"unknown config {name}")


def make_requests(name: str, args, vocab: int):
    """List of (prompt token ids, max_new_tokens)."""
    import numpy as np
    rng = np.random.default_rng(args.seed)
    n = args.requests
    if name == "b":
        ins = np.clip(np.round(rng.lognormal(math.log(args.input_len), 0.6, n)), 8, 4096).astype(int)
        outs = np.clip(np.round(rng.lognormal(math.log(args.output_len), 0.5, n)), 4, 1024).astype(int)
        return [(rng.integers(3, vocab, int(i)).tolist(), int(o)) for i, o in zip(ins, outs)]
    if name == "d":
        prefix = rng.integers(3, vocab, 2048).tolist()
        return [(prefix + rng.integers(3, vocab, 128).tolist(), args.output_len) for _ in range(n)]
    return [(rng.integers(3, vocab, args.input_len).tolist(), args.output_len) for _ in range(n)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["b", "d", "e"])
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--input-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--max-batch", type=int, default=256)
    ap.add_argument("--no-prefix-cache", action="store_true")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--weights", default="", choices=["", "auto", "fp8_block", "nvfp4", "w4a16"],
                    help="weight format (default: bf16 for config b, fp8_block for d and e)")
    args = ap.parse_args()
    defaults = {"b": (500, 512, 128), "d": (256, 2176, 64), "e": (64, 1024, 64)}[args.config]
    args.requests = args.requests or defaults[0]
    args.input_len = args.input_len or defaults[1]
    args.output_len = args.output_len or defaults[2]

    import torch
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.ops import native
    from ksanallm_b200.utils import native_engine as ne

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    mc = model_config(args.config, args)
    on_gpu = torch.cuda.is_available()
    if not on_gpu:
        # no GPU: the same request mix through a toy-sized model on the CPU (a functional check of this script)
        mc.hidden_size, mc.num_layers, mc.num_heads, mc.num_kv_heads, mc.head_dim = 64, 2, 4, 2, 16
        mc.intermediate_size, mc.vocab_size = 128, 512
        if args.config == "e":
            mc.num_kv_heads, mc.head_dim = 4, 24
            mc.q_lora_rank, mc.kv_lora_rank, mc.qk_nope_head_dim, mc.qk_rope_head_dim, mc.v_head_dim = 32, 32, 16, 8, 16
            mc.num_experts, mc.num_experts_per_tok, mc.n_group, mc.topk_group = 8, 2, 4, 2
            mc.moe_intermediate_size = mc.shared_expert_intermediate_size = 32
    reqs = make_requests(args.config, args, mc.vocab_size)
    longest = max(len(p) + o for p, o in reqs)
    ec = EngineConfig()
    ec.global_.comm_backend = args.comm
    ec.global_.enable_cuda_graph = True
    ec.batch_scheduler.max_batch_size = args.max_batch
    ec.batch_scheduler.max_token_len = longest + 16
    ec.batch_scheduler.max_step_tokens = 16384
    ec.batch_scheduler.max_waiting_queue_len = max(4096, 2 * len(reqs))
    ec.batch_scheduler.preempt_mode = 1
    ec.batch_scheduler.enable_auto_prefix_cache = args.config == "d" and not args.no_prefix_cache
    ec.block_manager.block_token_num = 16
    ec.block_manager.reserved_device_memory_ratio = 0.08
    ec.quantization.weight_quant_method = args.weights or ("auto" if (args.config == "b" or not on_gpu) else "fp8_block")
    if not on_gpu:
        ec.block_manager.device_blocks_num = 4096
    llm = LLM(ec, mc, weights="random", device="cuda" if on_gpu else "cpu", dtype=torch.bfloat16 if on_gpu else torch.float32,
              max_positions=longest + 64)
    dev = llm.device

    def run(subset):
        handles = []
        if rank == 0:
            for p, o in subset:
                s = ne.SamplingConfig()
                s.max_new_tokens, s.ignore_eos, s.topk = o, True, 1
                handles.append(llm.engine.add_request(p, s))
            debug = on_gpu and os.environ.get("KSANA_CHECK_INPUTS", "0") not in ("", "0")
            while not all(h.done.is_set() for h in handles):
                if not llm.engine.step() and llm.engine.scheduler.idle():
                    break
                if debug:                       # debug runs: surface a kernel's index-guard report at the step it happened
                    native.check_err_flag(dev)
            if world > 1:
                import numpy as np
                from ksanallm_b200.parallel.control import broadcast_plan
                broadcast_plan(llm.engine.control_group, np.zeros(0, dtype=np.int32))
        else:
            llm.follow()
        return handles

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    run(reqs[: max(2, len(reqs) // 10)])
    barrier()
    stats0 = llm.engine.scheduler.stats() if rank == 0 else {}
    import time
    if on_gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    handles = run(reqs)
    if on_gpu:
        e1.record()
    barrier()
    ms = e0.elapsed_time(e1) if on_gpu else (time.perf_counter() - t0) * 1000.0
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    if on_gpu:
        native.check_err_flag(dev)
    if rank == 0:
        n_out = sum(len(h.outputs[0].tokens) for h in handles)
        n_in = sum(len(p) for p, _ in reqs)
        ok = sum(1 for h in handles if h.status_code == 0)
        stats1 = llm.engine.scheduler.stats()
        res = {"config": args.config, "model": f"{mc.model_type} {mc.hidden_size}x{mc.num_layers}", "n_gpus": world,
               "requests": len(reqs), "finished_ok": ok, "input_tokens": n_in, "output_tokens": n_out, "seconds": ms / 1000.0,
               "output_tok_s": n_out / (ms / 1000.0), "total_tok_s": (n_in + n_out) / (ms / 1000.0),
               "requests_s": len(reqs) / (ms / 1000.0), "engine_steps": llm.engine.steps,
               "prefix_hit_tokens": int(stats1.get("prefix_hit_tokens", 0)) - int(stats0.get("prefix_hit_tokens", 0)),
               "weights": ec.quantization.weight_quant_method, "data": "synthetic", "graph_replays":
               getattr(llm.engine.runner, "graph_replays", 0)}
        print(json.dumps(res))
    sys.stdout.flush()
    llm.shutdown()             # the worker ranks have left ``follow`` with the end-of-batch signal: nobody to release
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
