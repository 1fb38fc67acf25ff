"""Configuration: the serving YAML (same schema and defaults as the reference) and the model
hyper-parameters read from a Hugging Face ``config.json`` / ``generation_config.json``.

Reference behaviour: src/ksana_llm/utils/environment.cpp:275-438 (YAML), :527-620 (model config),
:121-192 (max length / rope scaling), :194-227 (EOS ids), :229-273 (KV scale files), :640-675
(block sizes); defaults from src/ksana_llm/utils/environment.h:139-260 and examples/ksana_llm.yaml.
Unknown keys are accepted with a warning. New keys: ``expert_para_size``, ``attn_data_para_size``,
``quant_method: fp8_block|nvfp4``, ``comm_backend: fused|nccl``.
"""
from __future__ import annotations

import json
import logging
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

import yaml

log = logging.getLogger("ksana_llm")


@dataclass
class GlobalConfig:
    tensor_para_size: int = 1
    pipeline_para_size: int = 1
    pipeline_micro_batches: int = 2      # micro-batches of one step in flight across the pipeline stages
    expert_para_size: int = 1
    attn_data_para_size: int = 1
    enable_lora_adapter: bool = False
    embed_tokens_use_cpu: bool = False
    enable_cuda_graph: bool = False
    is_version_report: bool = True
    comm_backend: str = "fused"          # fused | nccl


@dataclass
class BatchSchedulerConfig:
    schedule_strategy: int = 0
    waiting_timeout_in_ms: int = 600000
    max_waiting_queue_len: int = 256
    max_token_len: int = 2048
    max_step_tokens: int = 4096
    max_batch_size: int = 8
    swapout_block_threshold: float = 1.0
    swapin_block_threshold: float = 2.0
    launch_block_threshold: float = 2.0
    preempt_mode: int = 0
    split_fuse_token_num: int = 0
    swap_threadpool_size: int = 2
    min_flexible_cache_num: int = 0
    enable_auto_prefix_cache: bool = False


@dataclass
class BlockManagerConfig:
    block_token_num: int = 16
    reserved_device_memory_ratio: float = 0.05
    lora_deivce_memory_ratio: float = 0.0     # (sic) key spelling of the reference YAML
    block_device_memory_ratio: float = -1.0
    lora_host_memory_factor: float = 10.0
    block_host_memory_factor: float = 10.0
    # optional explicit block counts (tests, CPU runs)
    device_blocks_num: int = 0
    host_blocks_num: int = 0


@dataclass
class QuantConfig:
    gptq_backend: str = "cutlass"
    kv_cache_dtype: str = "auto"              # auto | fp8_e5m2 | fp8_e4m3
    weight_quant_method: str = "auto"         # auto | fp8_e4m3 | fp8_block | nvfp4 | w4a16 (gptq / awq select w4a16)
    # scales of weights quantised at load time: "ue8m0" = powers of two (applied by the tensor cores through the
    # block-scaled MMA), "fp32" = amax / 448 exactly (served by the register-promotion GEMM)
    fp8_scale_mode: str = "ue8m0"


@dataclass
class ProfilerConfig:
    trace_export_url: str = ""
    metrics_export_url: str = ""
    export_interval_millis: int = 60000
    export_timeout_millis: int = 1000
    attributes: Dict[str, str] = field(default_factory=dict)


@dataclass
class PluginModelConfig:
    enable_tensorrt: bool = True
    plugin_thread_pool_size: int = 1


@dataclass
class EngineConfig:
    global_: GlobalConfig = field(default_factory=GlobalConfig)
    batch_scheduler: BatchSchedulerConfig = field(default_factory=BatchSchedulerConfig)
    block_manager: BlockManagerConfig = field(default_factory=BlockManagerConfig)
    quantization: QuantConfig = field(default_factory=QuantConfig)
    profiler: ProfilerConfig = field(default_factory=ProfilerConfig)
    plugin_model: PluginModelConfig = field(default_factory=PluginModelConfig)
    endpoint_type: str = "python"
    model_dir: str = ""
    tokenizer_dir: str = ""
    lora_models: List[Dict[str, Any]] = field(default_factory=list)
    # pipeline (multi-node) settings come from the process environment
    master_host: str = ""
    master_port: int = 0
    world_size: int = 1
    node_rank: int = 0


def _fill(dc, section: Optional[dict], where: str):
    if not section:
        return
    names = {f.name for f in fields(dc)}
    for k, v in section.items():
        if k in names:
            cur = getattr(dc, k)
            try:
                if isinstance(cur, bool):
                    v = bool(v)
                elif isinstance(cur, int) and not isinstance(v, bool):
                    v = int(v)
                elif isinstance(cur, float):
                    v = float(v)
            except (TypeError, ValueError):
                raise ValueError(f"bad value for {where}.{k}: {v!r}")
            setattr(dc, k, v)
        elif isinstance(v, dict):
            continue
        else:
            log.warning("unknown config key %s.%s ignored", where, k)


def load_yaml_config(path_or_dict) -> EngineConfig:
    """Parse the serving YAML (a path, a YAML string's dict, or an already-loaded dict)."""
    if isinstance(path_or_dict, dict):
        doc = path_or_dict
        base_dir = os.getcwd()
    else:
        with open(path_or_dict, "r", encoding="utf-8") as f:
            doc = yaml.safe_load(f) or {}
        base_dir = os.path.dirname(os.path.abspath(path_or_dict))
    cfg = EngineConfig()
    setting = doc.get("setting", {}) or {}
    _fill(cfg.global_, setting.get("global"), "setting.global")
    _fill(cfg.batch_scheduler, setting.get("batch_scheduler"), "setting.batch_scheduler")
    _fill(cfg.block_manager, setting.get("block_manager"), "setting.block_manager")
    q = setting.get("quantization_config", {}) or {}
    cfg.quantization.gptq_backend = str(q.get("gptq_backend", cfg.quantization.gptq_backend))
    cfg.quantization.kv_cache_dtype = str((q.get("kv_cache") or {}).get("dtype", "auto"))
    cfg.quantization.weight_quant_method = str((q.get("weight") or {}).get("quant_method", "auto"))
    cfg.quantization.fp8_scale_mode = str((q.get("weight") or {}).get("scale_mode", cfg.quantization.fp8_scale_mode))
    if cfg.quantization.fp8_scale_mode not in ("ue8m0", "fp32"):
        raise ValueError(f"unsupported weight.scale_mode {cfg.quantization.fp8_scale_mode}")
    if cfg.quantization.kv_cache_dtype not in ("auto", "fp8_e5m2", "fp8_e4m3"):
        raise ValueError(f"unsupported kv_cache.dtype {cfg.quantization.kv_cache_dtype}")
    if cfg.quantization.weight_quant_method not in ("auto", "fp8_e4m3", "fp8_block", "nvfp4", "w4a16", "gptq", "awq"):
        raise ValueError(f"unsupported weight.quant_method {cfg.quantization.weight_quant_method}")
    prof = setting.get("profiler", {}) or {}
    for k in ("trace_export_url", "metrics_export_url"):
        if k in prof:
            setattr(cfg.profiler, k, str(prof[k]))
    for k in ("export_interval_millis", "export_timeout_millis"):
        if k in prof:
            setattr(cfg.profiler, k, int(prof[k]))
    cfg.profiler.attributes = {str(k): str(v) for k, v in (prof.get("attributes") or {}).items()}
    cfg.endpoint_type = str(setting.get("endpoint_type", "python"))
    spec = doc.get("model_spec", {}) or {}
    base = spec.get("base_model", {}) or {}
    model_dir = str(base.get("model_dir", ""))
    if model_dir and not os.path.isabs(model_dir):
        model_dir = os.path.normpath(os.path.join(base_dir, model_dir))
    cfg.model_dir = model_dir
    cfg.tokenizer_dir = str(base.get("tokenizer_dir", "")) or model_dir
    _fill(cfg.plugin_model, spec.get("plugin_model"), "model_spec.plugin_model")
    cfg.lora_models = list(spec.get("lora_models") or [])
    # prefix caching is implied by the flexible cache, as in the reference
    if cfg.batch_scheduler.min_flexible_cache_num > 0:
        cfg.batch_scheduler.enable_auto_prefix_cache = True
    if cfg.global_.pipeline_para_size < 1 or cfg.global_.tensor_para_size < 1:
        raise ValueError("tensor_para_size and pipeline_para_size must be >= 1")
    if cfg.batch_scheduler.preempt_mode not in (0, 1):
        raise ValueError("preempt_mode must be 0 (SWAP) or 1 (RECOMPUTE)")
    # multi-node pipeline environment (src/ksana_llm/service/inference_server.cpp:43-67)
    cfg.master_host = os.environ.get("MASTER_HOST", "")
    cfg.master_port = int(os.environ.get("MASTER_PORT", "0") or 0)
    cfg.world_size = int(os.environ.get("WORLD_SIZE_NODES", os.environ.get("KSANA_WORLD_SIZE", "1")) or 1)
    cfg.node_rank = int(os.environ.get("NODE_RANK", "0") or 0)
    return cfg


# --------------------------------------------------------------------------------- model config
@dataclass
class ModelConfig:
    model_type: str = "llama"
    hf_model_type: str = ""        # model_type as config.json spells it (names the optional weight map file)
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    rotary_dim: int = 0                   # 0 -> head_dim
    rope_neox: bool = True
    max_position_embeddings: int = 2048
    max_token_len: int = 2048             # after rope-scaling extension
    tie_word_embeddings: bool = False
    qkv_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    activation: str = "silu"
    gated_mlp: bool = True
    norm_type: str = "rmsnorm"            # rmsnorm | layernorm
    post_norm: bool = False               # GPT-1 / fairseq style
    position_embedding: str = "rope"      # rope | alibi | learned | sinusoidal | mrope
    mrope_section: Optional[List[int]] = None
    emb_scale: float = 1.0
    lm_head_norm: bool = False            # Baichuan2 normalised lm_head
    eos_token_ids: List[int] = field(default_factory=list)
    pad_token_id: int = 0
    dtype: str = "bfloat16"
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    num_shared_experts: int = 0
    norm_topk_prob: bool = True
    moe_scoring: str = "softmax"          # softmax | sigmoid
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    shared_expert_gate: bool = False
    expert_para_size: int = 1             # > 1: whole experts per rank of the tensor-parallel group (set by the engine)
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # quantisation found in the checkpoint
    quant_method: str = ""                # "", fp8, gptq, awq
    quant_bits: int = 0
    quant_group_size: int = 0
    quant_desc_act: bool = False
    fp8_checkpoint: bool = False
    weight_block_size: Optional[List[int]] = None
    is_visual: bool = False
    kv_scales: Optional[List[List[float]]] = None     # per layer (k_scale, v_scale)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0


_ARCH_ALIASES = {
    "llama": "llama", "mistral": "llama", "qwen2": "qwen", "qwen": "qwen", "qwen2_vl": "qwen2_vl", "baichuan": "baichuan",
    "chatglm": "chatglm", "glm": "chatglm", "gpt2": "gpt", "openai-gpt": "gpt", "fairseq-transformer": "gpt", "mixtral": "mixtral",
    "qwen2_moe": "qwen2_moe", "deepseek_v3": "deepseek_v3", "deepseek_v2": "deepseek_v3", "internlm2": "llama",
    "yi": "llama",
}


def parse_model_max_length(hf: dict, max_pos: int) -> int:
    """Extend the position range by the rope-scaling factor the way the reference does
    (environment.cpp:121-192): su/longrope use original_max*factor when given, llama3/yarn/linear/dynamic
    multiply max_position_embeddings."""
    rs = hf.get("rope_scaling") or {}
    if not rs:
        return max_pos
    kind = rs.get("rope_type", rs.get("type", "default"))
    factor = float(rs.get("factor", 1.0))
    if kind in ("su", "longrope"):
        return int(hf.get("max_position_embeddings", max_pos))
    if kind in ("yarn",):
        orig = int(rs.get("original_max_position_embeddings", max_pos))
        return int(orig * factor)
    if kind in ("llama3",):
        return max_pos           # HF already lists the extended length
    if kind in ("linear", "dynamic"):
        return int(max_pos * factor)
    return max_pos


def resolve_architecture(model_type: str, model_dir: Optional[str] = None) -> str:
    """Model family that serves a config.json ``model_type``: a known name, else a family whose name the type
    contains (case-insensitive, e.g. "codellama" -> llama), else Llama when a weight map
    ``<model_type>_weight_map.json`` exists for it (next to the checkpoint or in the package: a Llama-shaped model
    whose tensors only carry other names), else an error (src/ksana_llm/runtime/model_instance.cpp:42-86)."""
    if model_type in _ARCH_ALIASES:
        return _ARCH_ALIASES[model_type]
    low = model_type.lower()
    for part, arch in (("llama", "llama"), ("qwen2_moe", "qwen2_moe"), ("qwen2_vl", "qwen2_vl"), ("qwen", "qwen"),
                       ("baichuan", "baichuan"), ("chatglm", "chatglm"), ("gpt", "gpt"), ("fairseq-transformer", "gpt"),
                       ("mixtral", "mixtral"), ("deepseek", "deepseek_v3")):
        if part in low:
            return arch
    if find_weight_map(low, model_dir) or find_weight_map(model_type, model_dir):
        return "llama"
    raise ValueError(f"Model type {model_type} is not supported (no <model_type>_weight_map.json found for it either).")


def find_weight_map(model_type: str, model_dir: Optional[str] = None) -> Optional[str]:
    """Path of ``<model_type>_weight_map.json``: the checkpoint directory first, then the package's weight_map folder
    (src/ksana_llm/utils/optional_file.h:23-61)."""
    name = f"{model_type}_weight_map.json"
    for folder in ([model_dir] if model_dir else []) + [os.path.join(os.path.dirname(os.path.abspath(__file__)), "weight_map")]:
        path = os.path.join(folder, name)
        if os.path.exists(path):
            return path
    return None


def model_config_from_hf(hf: dict, generation: Optional[dict] = None, model_dir: Optional[str] = None) -> ModelConfig:
    tc = hf.get("text_config")
    if isinstance(tc, dict):
        # multimodal config.json files of newer exports keep the language model's fields under text_config
        merged = dict(tc)
        merged.update({k: v for k, v in hf.items() if k not in ("text_config",) and (v is not None or k not in merged)})
        merged["model_type"] = hf.get("model_type", tc.get("model_type", "llama"))
        for k in ("tie_word_embeddings",):
            if hf.get(k) is None and tc.get(k) is not None:
                merged[k] = tc[k]
        hf = merged
    rp = hf.get("rope_parameters")
    if isinstance(rp, dict):
        # newer config.json files keep rope_theta and the scaling description together under rope_parameters
        hf = dict(hf)
        if rp.get("rope_theta") is not None and hf.get("rope_theta") is None:
            hf["rope_theta"] = rp["rope_theta"]
        if hf.get("rope_scaling") is None and rp.get("rope_type", rp.get("type", "default")) != "default":
            hf["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
        elif hf.get("rope_scaling") is None and rp.get("mrope_section"):
            hf["rope_scaling"] = {"mrope_section": rp["mrope_section"]}
    mt = hf.get("model_type", "llama")
    arch = resolve_architecture(mt, model_dir)
    c = ModelConfig(model_type=arch, hf_model_type=mt)
    if arch == "gpt":
        c.hidden_size = hf.get("n_embd", hf.get("hidden_size", hf.get("decoder_embed_dim", 768)))
        c.num_layers = hf.get("n_layer", hf.get("num_hidden_layers", hf.get("decoder_layers", 12)))
        c.num_heads = hf.get("n_head", hf.get("num_attention_heads", hf.get("decoder_attention_heads", 12)))
        c.num_kv_heads = c.num_heads
        c.intermediate_size = hf.get("n_inner") or hf.get("decoder_ffn_embed_dim") or 4 * c.hidden_size
        c.vocab_size = hf.get("vocab_size", 50257)
        c.max_position_embeddings = hf.get("n_positions", hf.get("max_position_embeddings", hf.get("max_target_positions", 1024)))
        c.rms_norm_eps = hf.get("layer_norm_epsilon", 1e-5)
        c.norm_type, c.gated_mlp = "layernorm", False
        c.activation = {"gelu_new": "gelu", "gelu": "gelu", "relu": "relu"}.get(hf.get("activation_function", hf.get("afn", "gelu")), "gelu")
        c.qkv_bias = c.o_bias = c.mlp_bias = True
        c.position_embedding = "sinusoidal" if mt == "fairseq-transformer" else "learned"
        c.post_norm = mt in ("openai-gpt", "fairseq-transformer") and not hf.get("decoder_normalize_before", False)
        c.tie_word_embeddings = hf.get("tie_word_embeddings", True)
        if mt == "fairseq-transformer" and not hf.get("no_scale_embedding", False):
            c.emb_scale = float(c.hidden_size) ** 0.5
    else:
        c.hidden_size = hf.get("hidden_size", 4096)
        c.num_layers = hf.get("num_hidden_layers", hf.get("num_layers", 32))
        c.num_heads = hf.get("num_attention_heads", 32)
        c.num_kv_heads = hf.get("num_key_value_heads", hf.get("multi_query_group_num", c.num_heads)) or c.num_heads
        c.intermediate_size = hf.get("intermediate_size", hf.get("ffn_hidden_size", 11008))
        c.vocab_size = hf.get("vocab_size", hf.get("padded_vocab_size", 32000))
        c.max_position_embeddings = hf.get("max_position_embeddings", hf.get("seq_length", 2048))
        c.rms_norm_eps = hf.get("rms_norm_eps", hf.get("layernorm_epsilon", 1e-6))
        c.rope_theta = float(hf.get("rope_theta", hf.get("rotary_emb_base", 10000.0)))
        c.tie_word_embeddings = bool(hf.get("tie_word_embeddings", False))
        c.activation = {"silu": "silu", "swiglu": "silu", "gelu": "gelu", "relu": "relu"}.get(hf.get("hidden_act", "silu"), "silu")
    c.head_dim = hf.get("head_dim") or hf.get("kv_channels") or c.hidden_size // c.num_heads
    c.rope_scaling = hf.get("rope_scaling")
    c.max_token_len = parse_model_max_length(hf, c.max_position_embeddings)
    if arch == "qwen" or arch == "qwen2_vl" or arch == "qwen2_moe":
        c.qkv_bias = True
    if mt == "qwen":
        # first-generation Qwen: config.json counts gate and up together (w1 and w2 are intermediate_size / 2 wide each)
        c.intermediate_size //= 2
        c.rms_norm_eps = hf.get("layer_norm_epsilon", c.rms_norm_eps)
    if arch == "qwen2_vl":
        c.position_embedding, c.is_visual = "mrope", True
        c.mrope_section = list((hf.get("rope_scaling") or {}).get("mrope_section", [16, 24, 24]))
        c.rope_scaling = None
    if arch == "baichuan":
        # 13B-class checkpoints (hidden != 4096) use ALiBi; Baichuan2 normalises lm_head rows
        if c.hidden_size != 4096:
            c.position_embedding = "alibi"
        c.lm_head_norm = hf.get("vocab_size", 0) == 125696
    if arch == "chatglm":
        # ChatGLM2/3 (THUDM config names) and GLM-4 in the Hugging Face layout (model_type "glm"): rotary pairs are
        # interleaved and cover only part of the head, QKV carries a bias, gate and up are one fused matrix
        c.rope_neox = False
        prf = hf.get("partial_rotary_factor", (hf.get("rope_parameters") or {}).get("partial_rotary_factor", 0.5))
        c.rotary_dim = int(c.head_dim * float(prf))
        c.qkv_bias = bool(hf.get("attention_bias", hf.get("add_qkv_bias", True)))
        if mt == "glm":
            c.num_kv_heads = hf.get("num_key_value_heads", c.num_heads) or c.num_heads
        else:
            c.num_kv_heads = hf.get("multi_query_group_num", c.num_kv_heads) if hf.get("multi_query_attention", True) else c.num_heads
    if arch in ("mixtral", "qwen2_moe", "deepseek_v3"):
        c.num_experts = hf.get("num_local_experts", hf.get("num_experts", hf.get("n_routed_experts", 8)))
        c.num_experts_per_tok = hf.get("num_experts_per_tok", 2)
        c.moe_intermediate_size = hf.get("moe_intermediate_size", c.intermediate_size)
        c.norm_topk_prob = bool(hf.get("norm_topk_prob", arch != "qwen2_moe"))
    if arch == "qwen2_moe":
        c.shared_expert_intermediate_size = hf.get("shared_expert_intermediate_size", 0)
        c.shared_expert_gate = True
    if arch == "deepseek_v3":
        c.num_shared_experts = hf.get("n_shared_experts", 1)
        c.shared_expert_intermediate_size = c.moe_intermediate_size * c.num_shared_experts
        c.moe_scoring = hf.get("scoring_func", "sigmoid")
        c.routed_scaling_factor = float(hf.get("routed_scaling_factor", 2.5))
        c.n_group, c.topk_group = hf.get("n_group", 8), hf.get("topk_group", 4)
        c.first_k_dense_replace = hf.get("first_k_dense_replace", 3)
        c.moe_layer_freq = hf.get("moe_layer_freq", 1)
        c.q_lora_rank = hf.get("q_lora_rank") or 0
        c.kv_lora_rank = hf.get("kv_lora_rank", 512)
        c.qk_nope_head_dim = hf.get("qk_nope_head_dim", 128)
        c.qk_rope_head_dim = hf.get("qk_rope_head_dim", 64)
        c.v_head_dim = hf.get("v_head_dim", 128)
        c.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        c.rope_neox = False
    q = hf.get("quantization_config") or {}
    if q:
        c.quant_method = str(q.get("quant_method", ""))
        c.quant_bits = int(q.get("bits", 0) or 0)
        c.quant_group_size = int(q.get("group_size", 0) or 0)
        c.quant_desc_act = bool(q.get("desc_act", False))
        if c.quant_method == "fp8":
            c.fp8_checkpoint = True
            c.weight_block_size = q.get("weight_block_size")
    td = hf.get("torch_dtype") or hf.get("dtype") or "bfloat16"          # newer exports write "dtype"
    c.dtype = {"float16": "float16", "bfloat16": "bfloat16", "float32": "float32"}.get(str(td).replace("torch.", ""), "bfloat16")
    eos = (generation or {}).get("eos_token_id", hf.get("eos_token_id"))
    if eos is not None:
        c.eos_token_ids = [int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])]
    pad = hf.get("pad_token_id")
    c.pad_token_id = int(pad) if pad is not None else (1 if mt == "fairseq-transformer" else 0)   # fairseq dictionaries put <pad> at 1
    if c.num_heads % max(c.num_kv_heads, 1):
        raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
    return c


def load_model_config(model_dir: str) -> ModelConfig:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        hf = json.load(f)
    gen = None
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gpath):
        with open(gpath, "r", encoding="utf-8") as f:
            gen = json.load(f)
    return model_config_from_hf(hf, gen, model_dir)


def load_kv_scales(path: str, num_layers: int) -> List[List[float]]:
    """``kv_cache_scales.json``: {"kv_cache": {"scaling_factor": {"0": {"<layer>": scale}}}} (one scale
    used for both K and V of a layer)."""
    with open(path, "r", encoding="utf-8") as f:
        doc = json.load(f)
    table = doc["kv_cache"]["scaling_factor"]["0"]
    return [[float(table[str(i)]), float(table[str(i)])] for i in range(num_layers)]


def check_tp(model: ModelConfig, tp: int) -> None:
    if model.num_heads % tp:
        raise ValueError(f"num_heads {model.num_heads} is not divisible by tensor_para_size {tp}")
    if model.num_kv_heads % tp and tp % model.num_kv_heads:
        raise ValueError(f"num_kv_heads {model.num_kv_heads} incompatible with tensor_para_size {tp}")


def kv_block_bytes(model: ModelConfig, block_token_num: int, tp: int, pp: int, kv_dtype_bytes: int) -> int:
    """Bytes of one KV block on one rank: layers/pp x kv_heads/tp x head_dim x block_tokens x 2 (K,V)."""
    layers = (model.num_layers + pp - 1) // pp
    if model.is_mla:
        return layers * block_token_num * (model.kv_lora_rank + model.qk_rope_head_dim) * kv_dtype_bytes
    kvh = max(1, model.num_kv_heads // tp)
    return layers * kvh * model.head_dim * block_token_num * 2 * kv_dtype_bytes
