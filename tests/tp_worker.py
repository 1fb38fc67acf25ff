"""Worker of the multi-GPU tests (launched by torchrun, one rank per GPU): runs a small Llama with tensor
parallelism through the fused peer-memory path and through the NCCL path and writes the logits of rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.config import EngineConfig, ModelConfig  # noqa: E402
from ksanallm_b200.llm import LLM  # noqa: E402
from ksanallm_b200.models.weights import RandomSource  # noqa: E402
from ksanallm_b200.ops import native  # noqa: E402
from ksanallm_b200.utils import native_engine as ne  # noqa: E402


def main():
    out_path, backend, quant = sys.argv[1], sys.argv[2], sys.argv[3]
    graphs = (sys.argv[4] == "graphs") if len(sys.argv) > 4 else backend == "fused"
    arch = sys.argv[5] if len(sys.argv) > 5 else "llama"          # llama | moe (experts sliced) | moe_ep (whole experts)
    log_dir = os.environ.get("KSANA_TP_LOG_DIR")
    rank_env = os.environ.get("RANK", "0")
    log = open(os.path.join(log_dir, f"tp_model_{backend}_{quant}_{int(graphs)}_{sys.argv[5] if len(sys.argv) > 5 else 'llama'}_rank{rank_env}.log"), "w") if log_dir else None

    def say(*a):
        if log:
            log.write(" ".join(str(x) for x in a) + "\n")
            log.flush()

    mc = ModelConfig(model_type="llama", hidden_size=1024, num_layers=3, num_heads=8, num_kv_heads=4, head_dim=128,
                     intermediate_size=2048, vocab_size=32000, rms_norm_eps=1e-5, max_position_embeddings=512,
                     max_token_len=512)
    if arch.startswith("moe"):
        mc.model_type, mc.num_experts, mc.num_experts_per_tok, mc.moe_intermediate_size = "mixtral", 8, 2, 512
    ec = EngineConfig()
    if arch == "moe_ep":
        ec.global_.expert_para_size = int(os.environ.get("WORLD_SIZE", "1"))
    ec.global_.comm_backend = backend
    ec.global_.enable_cuda_graph = graphs
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 300
    ec.batch_scheduler.max_step_tokens = 512
    ec.block_manager.device_blocks_num = 128
    ec.quantization.weight_quant_method = quant
    say("building")
    llm = LLM(ec, mc, weights=RandomSource(seed=11, std=0.05), device="cuda")
    if arch.startswith("moe"):
        # decisive routing: with near-tied router logits, rounding differences between layouts flip expert choices
        # and the comparison would measure routing luck instead of the kernels
        for lw in llm.model.layers:
            if lw.moe is not None:
                lw.moe.router.mul_(16.0)
    say("llm ready")
    inner = llm.engine.runner.execute

    def traced(plan, extra=None, patch=None):
        say("execute: seqs", len(plan.seq_ids), "tokens", plan.num_tokens, "multi", plan.num_multi)
        out = inner(plan, extra, patch)
        say("launched")
        return out

    llm.engine.runner.execute = traced
    first, last = {}, {}

    def hook(plan, lg):
        for i, sid in enumerate(plan.sample_seq_ids.tolist()):
            row = lg[i].float().cpu().clone()
            first.setdefault(sid, row)
            last[sid] = row

    if os.environ.get("KSANA_TP_TEST_NOHOOK") != "1":     # without the hook nothing reads whole logits rows: the ranks
        llm.engine.step_hook = hook                        # then exchange per-shard sampling candidates only
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (70, 5, 33, 128)]
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 5, True
    if os.environ.get("KSANA_TP_SAMPLING") == "topk":
        s.topk, s.topp, s.temperature, s.seed, s.logprobs_num, s.max_new_tokens = 20, 0.9, 0.8, 1234, 3, 12
    reqs = llm.generate(prompts if llm.rank == 0 else [], s)
    say("generate returned")
    torch.cuda.synchronize()
    say("synchronised")
    native.check_err_flag(llm.device)
    if llm.rank == 0:
        order = sorted(first)
        zero = torch.zeros(1, 1)
        torch.save({"tokens": [r.outputs[0].tokens for r in reqs],
                    "logprobs": [r.outputs[0].logprobs for r in reqs],
                    "first": torch.stack([first[k] for k in order]) if first else zero,
                    "last": torch.stack([last[k] for k in order]) if last else zero,
                    "graph_replays": getattr(llm.engine.runner, "graph_replays", 0)}, out_path)
    import torch.distributed as dist
    llm.shutdown()
    say("shut down")
    if dist.is_initialized():
        dist.barrier()
        say("barrier passed")
    if log:
        log.close()
    sys.stdout.flush()
    os._exit(0)      # skip communicator teardown: nothing is in flight and the results are on disk


if __name__ == "__main__":
    main()
