"""Worker of the service-lifetime test: two CPU ranks (gloo) of one engine; rank 1 leaves between two steps and rank 0
has to notice through the control channel, answer its requests with an error status and end its service.
argv: out_path. Environment: RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT."""
import json
import os
import sys
import threading

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.config import EngineConfig, ModelConfig  # noqa: E402
from ksanallm_b200.llm import LLM  # noqa: E402
from ksanallm_b200.models.weights import RandomSource  # noqa: E402
from ksanallm_b200.parallel import coordinator  # noqa: E402
from ksanallm_b200.utils import native_engine as ne  # noqa: E402


def main():
    out_path = sys.argv[1]
    rank = int(os.environ["RANK"])
    mc = ModelConfig(model_type="llama", hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                     intermediate_size=128, vocab_size=300, rms_norm_eps=1e-5, max_position_embeddings=256,
                     max_token_len=256, eos_token_ids=[2])
    ec = EngineConfig()
    ec.global_.comm_backend = "nccl"
    ec.batch_scheduler.max_batch_size = 4
    ec.batch_scheduler.max_token_len = 200
    ec.block_manager.device_blocks_num = 64
    llm = LLM(ec, mc, weights=RandomSource(seed=3, std=0.2), device="cpu", dtype=torch.float32)
    if rank == 1:
        # follow a few steps, then leave between two steps: nothing of this rank is in flight when it goes
        inner = llm.engine.run_with_extras
        seen = {"n": 0}

        def counted(plan, extra, patch=None):
            out = inner(plan, extra, patch)
            seen["n"] += 1
            if seen["n"] == 4:
                os._exit(0)
            return out

        llm.engine.run_with_extras = counted
        llm.follow()
        os._exit(0)
    reqs = []

    def stop_hook(reason):
        with open(out_path, "w") as f:
            json.dump({"reason": reason, "fatal": llm.engine.fatal,
                       "statuses": [(r.status_code, r.done.is_set(), len(r.outputs[0].tokens)) for r in reqs]}, f)

    coordinator.register_stop_hook(stop_hook)
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 100, True
    reqs.extend(llm.engine.add_request(list(range(5, 15)), s) for _ in range(2))
    # generate on a helper thread: the main thread of a real server is free too; the lost rank leaves this thread in a
    # collective that cannot complete, and the liveness monitor ends the process
    t = threading.Thread(target=lambda: llm.generate([list(range(20, 30))], s), daemon=True)
    t.start()
    t.join(60)
    import time
    time.sleep(5)          # (over gloo the broken collective raises in the helper thread; the monitor acts within 0.1 s)
    with open(out_path, "w") as f:
        json.dump({"reason": "no failure was detected"}, f)
    os._exit(5)


if __name__ == "__main__":
    main()
