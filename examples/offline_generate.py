"""Offline generation with random weights (no checkpoint needed): a small Llama-style model on one GPU or CPU."""
import torch

from ksanallm_b200.config import EngineConfig, ModelConfig
from ksanallm_b200.llm import LLM
from ksanallm_b200.utils import native_engine as ne

mc = ModelConfig(model_type="llama", hidden_size=1024, num_layers=4, num_heads=8, num_kv_heads=2, head_dim=128,
                 intermediate_size=2816, vocab_size=32000, max_position_embeddings=2048, max_token_len=2048)
ec = EngineConfig()
ec.batch_scheduler.max_batch_size = 16
ec.block_manager.device_blocks_num = 512
ec.global_.enable_cuda_graph = torch.cuda.is_available()
llm = LLM(ec, mc, weights="random")
s = ne.SamplingConfig()
s.max_new_tokens, s.ignore_eos, s.topk, s.temperature = 16, True, 20, 0.8
for r in llm.generate([[1, 2, 3, 4, 5], [9, 8, 7]], s):
    print(r.prompt, "->", r.outputs[0].tokens)
