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
    if llm.rank == 0:
        order = sorted(first)
        torch.save({"tokens": [r.outputs[0].tokens for r in reqs], "first": torch.stack([first[k] for k in order]),
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
