"""Worker of the attention-data-parallel tests (launched by torchrun): a small MoE model with a shared expert,
sequences spread over the ranks, routed experts spread over the same ranks. argv: out_path device"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.config import EngineConfig, ModelConfig  # noqa: E402
from ksanallm_b200.llm import LLM  # noqa: E402
from ksanallm_b200.models.weights import RandomSource  # noqa: E402
from ksanallm_b200.utils import native_engine as ne  # noqa: E402


def model_cfg(device):
    big = device == "cuda"
    return ModelConfig(model_type="qwen2_moe", hidden_size=512 if big else 64, num_layers=3, num_heads=4, num_kv_heads=2,
                       head_dim=128 if big else 16, intermediate_size=1024 if big else 128, vocab_size=2000 if big else 300,
                       rms_norm_eps=1e-5, max_position_embeddings=512, max_token_len=512, eos_token_ids=[2],
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256 if big else 64,
                       shared_expert_intermediate_size=256 if big else 64, shared_expert_gate=True, norm_topk_prob=False,
                       qkv_bias=True)


def prompts_for(vocab):
    g = torch.Generator().manual_seed(0)
    return [torch.randint(3, vocab, (n,), generator=g).tolist() for n in (40, 5, 33, 70, 9)]


def engine_cfg():
    ec = EngineConfig()
    ec.global_.comm_backend = "nccl"
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 300
    ec.batch_scheduler.max_step_tokens = 512
    ec.block_manager.device_blocks_num = int(os.environ.get("KSANA_TEST_DP_BLOCKS", "128"))
    ec.batch_scheduler.max_token_len = min(300, ec.block_manager.device_blocks_num * 16)
    if os.environ.get("KSANA_TEST_DP_HOST_BLOCKS"):
        ec.block_manager.host_blocks_num = int(os.environ["KSANA_TEST_DP_HOST_BLOCKS"])
        ec.batch_scheduler.preempt_mode = 0
    return ec


def main():
    out_path, device = sys.argv[1], sys.argv[2]
    mc = model_cfg(device)
    ec = engine_cfg()
    if len(sys.argv) > 3:
        ec.global_.comm_backend = sys.argv[3]          # fused: dispatch / combine over peer memory
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ec.global_.attn_data_para_size = world
    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    llm = LLM(ec, mc, weights=RandomSource(seed=11, std=0.2 if device == "cpu" else 0.05), device=device, dtype=dtype)
    first = {}

    def hook(plan, lg):
        for i, sid in enumerate(plan.sample_seq_ids.tolist()):
            first.setdefault(sid, lg[i].float().cpu().clone())

    llm.engine.step_hook = hook
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = int(os.environ.get("KSANA_TEST_DP_NEW", "5")), True
    if os.environ.get("KSANA_TEST_DP_N"):
        # sampled siblings: every request forks into n sequences that share their prompt blocks (copy-on-write)
        s.num_return_sequences, s.topk, s.temperature, s.seed = int(os.environ["KSANA_TEST_DP_N"]), 20, 1.0, 1234
    reqs = llm.generate(prompts_for(mc.vocab_size) if llm.rank == 0 else [], s)
    if llm.rank == 0:
        order = sorted(first)
        moe = llm.model.layers[0].moe
        # a request with per-row extras is answered with a status at admission: nothing is scheduled for it
        refused = (llm.engine.add_request([5, 6, 7], s, request_target={"transformer": {"token_reduce_mode": "GATHER_ALL"}})
                   if llm.model.dp is not None else None)
        torch.save({"tokens": [r.outputs[0].tokens for r in reqs], "all_tokens": [[o.tokens for o in r.outputs] for r in reqs], "first": torch.stack([first[k] for k in order]),
                    "experts": (moe.expert_lo, moe.expert_hi), "gathered_bytes": llm.model.dp.gathered_bytes if llm.model.dp else 0,
                    "dispatched_rows": llm.model.dp.dispatched_rows if llm.model.dp else 0,
                    "peer_memory": bool(llm.model.dp is not None and llm.model.dp.symm is not None),
                    "stats": dict(llm.engine.scheduler.stats()) if llm.engine.scheduler else {},
                    "refused": (refused.status_code, refused.done.is_set()) if llm.model.dp is not None else None},
                   out_path)
    import torch.distributed as dist
    llm.shutdown()
    if dist.is_initialized():
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
