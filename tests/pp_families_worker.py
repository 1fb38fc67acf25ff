"""Worker of the pipeline-parallel family test (torchrun on CPU ranks, gloo): every family's tiny Hugging Face model
split into pipeline stages through the public LLM API; rank 0 compares the greedy continuation of two prompts with
Hugging Face's own greedy generation. argv: out_path pp family[,family...]"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from ksanallm_b200.config import EngineConfig, model_config_from_hf  # noqa: E402
from ksanallm_b200.llm import LLM  # noqa: E402
from ksanallm_b200.models.weights import DictSource  # noqa: E402
from ksanallm_b200.utils import native_engine as ne  # noqa: E402
from test_hf_parity_cpu import _init  # noqa: E402
from tp_families_worker import family  # noqa: E402


def main():
    out_path, pp, names = sys.argv[1], int(sys.argv[2]), sys.argv[3].split(",")
    results = {}
    for name in names:
        hf, c, _ = family(name)
        hf = _init(hf, std=0.2).eval()
        cfg = model_config_from_hf(c.to_dict())
        cfg.max_token_len = 128
        cfg.eos_token_ids = []
        ec = EngineConfig()
        ec.global_.pipeline_para_size = pp
        ec.global_.comm_backend = "nccl"
        ec.batch_scheduler.max_batch_size = 4
        ec.batch_scheduler.max_token_len = 128
        ec.batch_scheduler.max_step_tokens = 256
        ec.block_manager.device_blocks_num = 64
        sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
        llm = LLM(ec, cfg, weights=DictSource(sd, cfg.model_type), device="cpu", dtype=torch.float32)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(3, 203, (n,), generator=g).tolist() for n in (19, 7)]
        s = ne.SamplingConfig()
        s.max_new_tokens, s.ignore_eos, s.topk = 6, True, 1
        reqs = llm.generate(prompts if llm.rank == 0 else [], s)
        if llm.rank == 0:
            got = [list(r.outputs[0].tokens) for r in reqs]
            want = []
            with torch.no_grad():
                for p in prompts:
                    out = hf.generate(torch.tensor([p]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)
                    want.append(out[0, len(p):].tolist())
            results[name] = {"got": got, "want": want, "layers": [llm.model.layer_lo, llm.model.layer_hi], "ok": got == want}
        llm.shutdown()
    import torch.distributed as dist
    if llm.rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)
    if dist.is_initialized():
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
