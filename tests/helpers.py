"""Shared test helpers: a byte-level tokenizer and tiny model builders."""
import torch

from ksanallm_b200.config import EngineConfig, ModelConfig
from ksanallm_b200.models.weights import RandomSource, build_model
from ksanallm_b200.runtime.engine import LLMEngine
from ksanallm_b200.utils import native_engine as ne


class ByteTokenizer:
    """One token per UTF-8 byte (ids 3..258); 0 pad, 1 bos, 2 eos."""
    eos_token_id = 2
    bos_token_id = 1

    def encode(self, text, add_special_tokens=True):
        ids = [b + 3 for b in text.encode("utf-8")]
        return ([self.bos_token_id] if add_special_tokens else []) + ids

    def decode(self, ids, skip_special_tokens=True):
        bs = bytes([i - 3 for i in ids if 3 <= i < 259])
        return bs.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True):
        text = "".join(f"<{m['role']}>{m['content']}" for m in messages) + ("<assistant>" if add_generation_prompt else "")
        return self.encode(text) if tokenize else text


def tiny_model_cfg(vocab=300, **kw):
    c = ModelConfig(model_type="llama", hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                    intermediate_size=128, vocab_size=vocab, rms_norm_eps=1e-5, max_position_embeddings=512,
                    max_token_len=512, eos_token_ids=[2])
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def tiny_engine(cfg=None, seed=0, num_blocks=128, host_blocks=32, tokenizer=None, std=0.2, **sched):
    cfg = cfg or tiny_model_cfg()
    model = build_model(cfg, RandomSource(seed=seed, std=std), device="cpu", dtype=torch.float32)
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 16
    ec.batch_scheduler.max_token_len = 256
    for k, v in sched.items():
        setattr(ec.batch_scheduler, k, v)
    return LLMEngine(model, cfg, ec, num_blocks=num_blocks, num_host_blocks=host_blocks, tokenizer=tokenizer)


def sampling(**kw):
    s = ne.SamplingConfig()
    for k, v in kw.items():
        setattr(s, k, v)
    return s
