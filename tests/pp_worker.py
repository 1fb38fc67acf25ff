"""Worker of the pipeline-parallel tests (launched by torchrun): a small Llama split into pipeline stages
(optionally with tensor parallelism inside a stage) through the public LLM API; rank 0 writes tokens and logits.
argv: out_path device pp micro_batches"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.config import EngineConfig, ModelConfig  # noqa: E402
from ksanallm_b200.llm import LLM  # noqa: E402
from ksanallm_b200.models.weights import RandomSource  # noqa: E402
from ksanallm_b200.utils import native_engine as ne  # noqa: E402


def model_cfg(device):
    if device == "cuda":
        return ModelConfig(model_type="llama", hidden_size=1024, num_layers=4, num_heads=8, num_kv_heads=4, head_dim=128,
                           intermediate_size=2048, vocab_size=32000, rms_norm_eps=1e-5, max_position_embeddings=512,
                           max_token_len=512)
    return ModelConfig(model_type="llama", hidden_size=64, num_layers=5, num_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=300, rms_norm_eps=1e-5, max_position_embeddings=512,
                       max_token_len=512, eos_token_ids=[2])


def prompts_for(vocab):
    g = torch.Generator().manual_seed(0)
    return [torch.randint(3, vocab, (n,), generator=g).tolist() for n in (70, 5, 33, 128)]


TARGETS = {"transformer": {"slice_pos": [[0, 3]], "token_reduce_mode": "GATHER_ALL"},
           "layernorm": {"slice_pos": [[2, 2]], "token_reduce_mode": "GATHER_ALL"},
           "logits": {"slice_pos": [[0, 10]], "token_reduce_mode": "GATHER_TOKEN_ID"}}


def refit_for(mc):
    """Embeddings spliced over prompt positions 1..2 and 7 (what a vision plug-in hands to the engine)."""
    g = torch.Generator().manual_seed(5)
    return [1, 7], [torch.randn(2, mc.hidden_size, generator=g), torch.randn(mc.hidden_size, generator=g)]


def run_targets(llm):
    """Two prefill-only requests with request targets (hidden states, normed states, next-token probabilities) in one
    batch, through the engine of every rank; rank 0 returns their responses."""
    import copy
    import numpy as np
    from ksanallm_b200.parallel.control import broadcast_plan
    if llm.rank != 0:
        llm.follow()
        return None
    s = ne.SamplingConfig()
    s.max_new_tokens = 1
    prompts = prompts_for(llm.engine.model_cfg.vocab_size)[2:]
    reqs = [llm.engine.add_request(p, s, request_target=copy.deepcopy(TARGETS)) for p in prompts]
    reqs.append(llm.engine.add_request(prompts[0], s, request_target=copy.deepcopy(TARGETS), refit=refit_for(llm.engine.model_cfg)))
    while not all(r.done.is_set() for r in reqs):
        if not llm.engine.step() and llm.engine.scheduler.idle():
            break
    if llm.world > 1:
        broadcast_plan(llm.engine.control_group, np.zeros(0, dtype=np.int32))
    return [{k: v.clone() for k, v in r.response.items()} for r in reqs]


def main():
    out_path, device, pp, mb = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
    mc = model_cfg(device)
    ec = EngineConfig()
    ec.global_.pipeline_para_size = pp
    ec.global_.pipeline_micro_batches = mb
    ec.global_.comm_backend = "nccl"
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 300
    ec.batch_scheduler.max_step_tokens = 512
    ec.block_manager.device_blocks_num = 128
    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    llm = LLM(ec, mc, weights=RandomSource(seed=11, std=0.2 if device == "cpu" else 0.05), device=device, dtype=dtype)
    first = {}

    def hook(plan, lg):
        for i, sid in enumerate(plan.sample_seq_ids.tolist()):
            first.setdefault(sid, lg[i].float().cpu().clone())

    llm.engine.step_hook = hook
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 5, True
    reqs = llm.generate(prompts_for(mc.vocab_size) if llm.rank == 0 else [], s)
    targets = run_targets(llm) if os.environ.get("PP_TARGETS") else None
    if llm.rank == 0:
        order = sorted(first)
        torch.save({"tokens": [r.outputs[0].tokens for r in reqs], "first": torch.stack([first[k] for k in order]),
                    "targets": targets,
                    "layers": (llm.model.layer_lo, llm.model.layer_hi),
                    "sent_bytes": llm.engine.runner.pipeline.sent_bytes if llm.engine.runner.pipeline else 0}, out_path)
    import torch.distributed as dist
    llm.shutdown()
    if dist.is_initialized():
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
