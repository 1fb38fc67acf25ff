"""Offline / embedded entry point: builds the model, the KV cache and the engine from a serving
YAML (or explicit configs) and exposes ``generate``. One process per GPU; with ``WORLD_SIZE`` > 1
(torchrun) the ranks form ``pipeline_para_size`` stages of tensor-parallel groups, rank 0 schedules and
the others follow the broadcast step plans (the reference runs one thread per GPU inside one process instead:
src/ksana_llm/runtime/worker.cpp:43-54).
"""
from __future__ import annotations

import os
from typing import List, Optional

import numpy as np
import torch

from .config import EngineConfig, ModelConfig, check_tp, load_kv_scales, load_model_config, load_yaml_config
from .models.weights import CheckpointSource, RandomSource, build_model
from .parallel.comm import TPComm
from .runtime.engine import LLMEngine
from .utils import native_engine as ne


def _dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init_distributed(device_type: str, pp: int = 1):
    """Process groups of the job: a device group (NCCL / gloo) for this rank's tensor-parallel collectives and a
    CPU gloo group over all ranks for step-plan broadcast. With ``pp`` pipeline stages the ranks
    ``[s*tp, (s+1)*tp)`` form stage ``s`` and get a tensor-parallel group of their own; hidden states travel
    between stages point to point over the world group. Rendezvous uses MASTER_ADDR / MASTER_PORT (127.0.0.1 on
    one node). Returns (rank, world, tensor-parallel group, control group, world device group)."""
    import torch.distributed as dist
    rank, world, local = _dist_env()
    if world == 1:
        return 0, 1, None, None, None
    # MASTER_HOST is the reference's spelling of the rendezvous address (src/ksana_llm/utils/environment.cpp reads it
    # with MASTER_PORT / WORLD_SIZE / NODE_RANK): accepted where MASTER_ADDR is not given
    os.environ.setdefault("MASTER_ADDR", os.environ.get("MASTER_HOST") or "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if not dist.is_initialized():
        backend = "nccl" if device_type == "cuda" else "gloo"
        if device_type == "cuda":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
    world_group = dist.group.WORLD
    dev_group = world_group
    if pp > 1:
        if world % pp:
            raise ValueError(f"world size {world} is not a multiple of pipeline_para_size {pp}")
        tp = world // pp
        for stage in range(pp):                  # every rank creates every group (collective call)
            g = dist.new_group(ranks=list(range(stage * tp, (stage + 1) * tp)))
            if rank // tp == stage:
                dev_group = g
    ctl_group = dist.new_group(backend="gloo") if device_type == "cuda" else world_group
    return rank, world, dev_group, ctl_group, world_group


def kv_dtype_from(cfg: EngineConfig, default):
    k = cfg.quantization.kv_cache_dtype
    if k == "fp8_e4m3":
        return torch.float8_e4m3fn
    if k == "fp8_e5m2":
        return torch.float8_e4m3fn   # stored as e4m3 (the tensor-core friendly 8-bit format on sm_100a)
    return default


def auto_num_blocks(cfg: EngineConfig, block_bytes: int, device) -> int:
    """Device blocks from free memory: (free - reserved share) / block bytes, or the explicit ratio
    (src/ksana_llm/block_manager/block_manager.cpp:102-163)."""
    bm = cfg.block_manager
    if bm.device_blocks_num > 0:
        return bm.device_blocks_num
    if torch.device(device).type != "cuda":
        return 256
    free, total = torch.cuda.mem_get_info(device)
    if bm.block_device_memory_ratio >= 0:
        budget = int(total * bm.block_device_memory_ratio)
    else:
        budget = free - int(total * bm.reserved_device_memory_ratio)
    return max(int(budget // block_bytes), 0)


def auto_host_blocks(cfg: EngineConfig, num_device_blocks: int, block_bytes: int) -> int:
    bm = cfg.block_manager
    if bm.host_blocks_num > 0:
        return bm.host_blocks_num
    if cfg.batch_scheduler.preempt_mode != 0:
        return 0
    try:
        import psutil
        host_free = psutil.virtual_memory().available
    except Exception:  # noqa: BLE001
        host_free = 8 << 30
    return int(min(num_device_blocks * bm.block_host_memory_factor, 0.8 * host_free / block_bytes))


class LLM:
    def __init__(self, engine_cfg: Optional[EngineConfig] = None, model_cfg: Optional[ModelConfig] = None,
                 config_file: Optional[str] = None, weights="checkpoint", device: Optional[str] = None,
                 dtype=None, tokenizer=None, seed: int = 0, max_positions: Optional[int] = None):
        if config_file is not None:
            engine_cfg = load_yaml_config(config_file)
        self.engine_cfg = engine_cfg or EngineConfig()
        if model_cfg is None:
            model_cfg = load_model_config(self.engine_cfg.model_dir)
        self.model_cfg = model_cfg
        dev_type = "cuda" if (device is None and torch.cuda.is_available()) or (device and "cuda" in str(device)) else "cpu"
        pp = max(1, self.engine_cfg.global_.pipeline_para_size) if _dist_env()[1] > 1 else 1
        self.rank, self.world, dev_group, ctl_group, world_group = init_distributed(dev_type, pp)
        local = _dist_env()[2]
        self.device = torch.device("cuda", local) if dev_type == "cuda" else torch.device("cpu")
        if dtype is None:
            # the kernels compute in bf16 (fp16 checkpoints are converted on load); on the CPU path a float32 checkpoint
            # keeps its precision
            dtype = torch.float32 if (dev_type == "cpu" and getattr(model_cfg, "dtype", "") == "float32") else torch.bfloat16
        if dev_type == "cuda":
            torch.cuda.set_device(self.device)
        tp = self.world // pp
        adp = max(1, self.engine_cfg.global_.attn_data_para_size) if self.world > 1 else 1
        if adp > 1:
            # attention data parallel over all ranks, routed experts spread over the same ranks
            if adp != self.world or pp != 1:
                raise ValueError(f"attn_data_para_size {adp} must equal the world size {self.world} (no pipeline stages)")
            if not model_cfg.is_moe:
                raise ValueError("attn_data_para_size > 1 needs a mixture-of-experts model (dense models: run replicas)")
            tp = 1
            model_cfg.ep_layout_override = (self.rank, self.world)
        self.adp_size = adp
        self.pp_size, self.tp_size = pp, tp
        self.pp_rank, self.tp_rank = (self.rank // tp, self.rank % tp) if adp == 1 else (0, 0)
        check_tp(model_cfg, tp)
        ep = self.engine_cfg.global_.expert_para_size if adp == 1 else 1
        if ep not in (1, tp):
            raise ValueError(f"expert_para_size {ep} must be 1 or equal to the tensor-parallel size {tp}")
        model_cfg.expert_para_size = ep
        # the peer-memory kernels address ranks of the world group: with several stages the tensor-parallel
        # groups are sub-groups and use the library collectives
        backend = self.engine_cfg.global_.comm_backend if (dev_type == "cuda" and pp == 1) else "nccl"
        self.comm = TPComm(dev_group, self.tp_rank, tp, backend, self.device,
                           max_tokens=self.engine_cfg.batch_scheduler.max_step_tokens,
                           hidden=model_cfg.hidden_size) if tp > 1 else None
        quant = self.engine_cfg.quantization.weight_quant_method
        quant = {"auto": None, "fp8_e4m3": "fp8_block", "fp8_block": "fp8_block", "nvfp4": "nvfp4", "w4a16": "w4a16",
                 "gptq": "w4a16", "awq": "w4a16"}[quant]
        if model_cfg.fp8_checkpoint and quant is None:
            quant = "fp8_block"
        if model_cfg.quant_method in ("gptq", "awq") and quant is None:
            quant = "w4a16"                  # 4-bit checkpoints stay 4-bit unless another format is asked for
        if quant == "w4a16" and model_cfg.quant_group_size > 0:
            quant = f"w4a16:{model_cfg.quant_group_size}"
        from .ops import reference as _ref
        _ref.WEIGHT_SCALE_POW2 = self.engine_cfg.quantization.fp8_scale_mode != "fp32"
        if weights == "random":
            source = RandomSource(seed=seed, on_device=dev_type == "cuda" and model_cfg.hidden_size >= 2048)
        elif weights == "checkpoint":
            import glob as _glob
            ggufs = sorted(_glob.glob(os.path.join(self.engine_cfg.model_dir, "*.gguf")))
            if ggufs and not _glob.glob(os.path.join(self.engine_cfg.model_dir, "*.safetensors")):
                from .models.gguf import GGUFSource
                source = GGUFSource(ggufs[0])
            else:
                source = CheckpointSource(self.engine_cfg.model_dir, model_cfg.model_type, model_cfg.hf_model_type)
        else:
            source = weights
        kv_path = os.path.join(self.engine_cfg.model_dir or ".", "kv_cache_scales.json")
        if self.engine_cfg.quantization.kv_cache_dtype != "auto" and os.path.exists(kv_path):
            model_cfg.kv_scales = load_kv_scales(kv_path, model_cfg.num_layers)
        mp = max_positions or min(model_cfg.max_token_len, max(self.engine_cfg.batch_scheduler.max_token_len, 16))
        layer_range = None
        if pp > 1:
            from .parallel.pipeline import stage_layers
            layer_range = stage_layers(model_cfg.num_layers, pp, self.pp_rank)
        self.model = build_model(model_cfg, source, self.tp_rank, tp, self.comm, self.device, dtype, quant,
                                 layer_range=layer_range, max_positions=mp)
        if self.engine_cfg.global_.embed_tokens_use_cpu and self.model.embed is not None and not model_cfg.tie_word_embeddings:
            host = self.model.embed.to("cpu")
            self.model.embed = host.pin_memory() if dev_type == "cuda" else host
        if adp > 1:
            from .parallel.data_parallel import AttentionDP
            symm = None
            if dev_type == "cuda" and self.engine_cfg.global_.comm_backend == "fused":
                from .parallel.symm import SymmetricComm
                # room for every rank's padded rows: the longest per-rank row count times the ranks (bounded)
                cap = self.engine_cfg.batch_scheduler.max_step_tokens * min(self.world, 4)
                symm = SymmetricComm(dev_group, self.rank, self.world, self.device, cap, model_cfg.hidden_size)
            self.model.dp = AttentionDP(self.rank, self.world, dev_group, symm)
        kv_dtype = kv_dtype_from(self.engine_cfg, dtype)
        bt = self.engine_cfg.block_manager.block_token_num
        probe = self.model.allocate_kv_cache(1, bt, kv_dtype)
        block_bytes = probe[0].numel() * probe.element_size()
        self.model.kv_cache = None
        nblocks = auto_num_blocks(self.engine_cfg, block_bytes, self.device)
        nhost = auto_host_blocks(self.engine_cfg, nblocks, block_bytes)
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([nblocks, nhost], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=ctl_group)
            nblocks, nhost = int(t[0]), int(t[1])
        pipeline = None
        if pp > 1:
            from .parallel.pipeline import PipelineRunner
            pipeline = PipelineRunner(self.model, self.pp_rank, pp, self.tp_rank, tp, world_group,
                                      micro_batches=self.engine_cfg.global_.pipeline_micro_batches)
        self.engine = LLMEngine(self.model, model_cfg, self.engine_cfg, nblocks, nhost, tokenizer, kv_dtype,
                                self.rank, self.world, ctl_group, pipeline=pipeline)
        # liveness of the other ranks: a lost peer ends this rank's service instead of leaving it in a collective
        from .parallel.coordinator import DistributedCoordinator, register_stop_hook
        self.coordinator = DistributedCoordinator.from_env(self.rank, self.world)
        if self.coordinator is not None:
            self.coordinator.start()
            register_stop_hook(self.engine.on_service_stop)
        self.tokenizer = tokenizer
        from .utils import logger
        logger.info(f"engine ready: model {model_cfg.model_type} ({model_cfg.num_layers} layers, hidden "
                    f"{model_cfg.hidden_size}), rank {self.rank}/{self.world} tp {tp} pp {pp} attention-dp {adp}, "
                    f"{nblocks} device KV blocks of {bt} tokens, {nhost} host blocks, weights {quant or 'dense'}")
        self.warmup()

    def warmup(self):
        """One short request through the whole engine before serving (kernel modules loaded, workspaces and the
        first decode graph created, collectives' first-call set-up done), as the reference does at start-up unless
        ``DISABLE_WARMUP`` is set (src/ksana_llm/service/inference_engine.cpp:218-247). Collective: every rank of the
        engine runs it from its constructor."""
        if os.environ.get("DISABLE_WARMUP", "").lower() in ("1", "true", "yes", "on"):
            return
        from .utils import logger
        limit = min(self.model_cfg.max_token_len or 64, self.engine_cfg.batch_scheduler.max_token_len)
        if limit < 4:
            return
        s = ne.SamplingConfig()
        s.max_new_tokens, s.ignore_eos = 2, True
        tok = min(1, self.model_cfg.vocab_size - 1)
        import time
        t0 = time.time()
        reqs = self.generate([[tok] * min(8, limit - 2)] if self.rank == 0 else [], s)
        if self.rank == 0:
            ok = bool(reqs) and reqs[0].status_code == 0
            logger.info(f"warm-up request {'finished' if ok else 'FAILED'} in {(time.time() - t0) * 1000.0:.0f} ms")
            if not ok:
                raise RuntimeError(f"warm-up request failed: {reqs[0].status_message if reqs else 'no result'}")

    # ------------------------------------------------------------------ API
    def generate(self, prompt_token_ids: List[List[int]], sampling=None, timeout: Optional[float] = None):
        """Blocking batch generation. On ranks other than 0 this serves steps until rank 0 is done."""
        if self.rank != 0:
            self.follow()
            return []
        reqs = self.engine.generate(prompt_token_ids, sampling, timeout)
        if self.world > 1:
            from .parallel.control import broadcast_plan
            broadcast_plan(self.engine.control_group, np.zeros(0, dtype=np.int32))   # end of this batch
        return reqs

    def follow(self):
        """Worker ranks: execute broadcast step plans until the end-of-batch (empty image) or stop (None) signal."""
        from .parallel.control import broadcast_plan, unpack_extras
        while True:
            img, blob = broadcast_plan(self.engine.control_group, None, with_extras=True)
            if img is None:
                return False
            if img.size == 0:
                return True
            n_aux = int(img[-1])                         # the image ends with the pipelined-step data and its length
            aux = img[img.size - 1 - n_aux:img.size - 1] if n_aux > 0 else None
            plan = ne.StepPlan.unpack(img[:img.size - 1 - n_aux])
            self.engine.follow_step(plan, unpack_extras(blob), aux)

    def shutdown(self, stop_followers: bool = False):
        """Stops the engine loop. ``stop_followers`` additionally releases worker ranks blocked in ``follow``."""
        self.engine.runner.release_graphs()
        if getattr(self, "coordinator", None) is not None:
            self.coordinator.close()
        if self.rank == 0:
            self.engine.stop()
            if stop_followers and self.world > 1:
                from .parallel.control import broadcast_plan
                broadcast_plan(self.engine.control_group, None)
