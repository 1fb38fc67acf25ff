"""Weight sources and the loader that turns canonical (Llama-style) tensor names into the packed,
tensor-parallel-sliced, optionally FP8-quantised weights the model code consumes.

Reference behaviour: src/ksana_llm/models/common/common_weight.cpp:98-724 (slicing rules: q/k/v,
gate/up, lm_head by output rows; o_proj/down by input columns; q,k,v packed into one QKV matrix;
tied embeddings), src/ksana_llm/utils/get_custom_weight_name.cpp:1-55 (regex weight maps),
src/ksana_llm/runtime/model_instance.cpp:184-230 (file priority safetensors > gguf > bin).
Weights stay in the Hugging Face [out, in] layout: that is the K-major operand the tcgen05 GEMM
wants, so no transposes are needed at load time.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import re
from typing import Callable, Dict, List, Optional

import torch

from ..config import ModelConfig
from ..ops.dispatch import LinearWeight
from ..ops import reference as ref
from .common import CommonModel, LayerWeights

WEIGHT_MAP_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "weight_map")


# ------------------------------------------------------------------------------------ sources
class RandomSource:
    """N(0, std) tensors, deterministic per tensor name. ``on_device`` draws shards directly on the
    target device (large synthetic models); otherwise full tensors are drawn on the CPU so that
    every TP degree slices the same model."""

    def __init__(self, seed: int = 0, std: float = 0.02, on_device: bool = False):
        self.seed, self.std, self.on_device = seed, std, on_device

    def has(self, name: str) -> bool:
        return True

    def _gen(self, name: str, device) -> torch.Generator:
        h = int.from_bytes(hashlib.sha256(f"{self.seed}:{name}".encode()).digest()[:8], "little") & ((1 << 62) - 1)
        g = torch.Generator(device=device)
        g.manual_seed(h)
        return g

    def get(self, name: str, shape, device="cpu", kind: str = "normal") -> torch.Tensor:
        dev = torch.device(device) if self.on_device else torch.device("cpu")
        if kind == "ones":
            return torch.ones(shape, dtype=torch.float32, device=dev)
        if kind == "zeros":
            return torch.zeros(shape, dtype=torch.float32, device=dev)
        if self.on_device and dev.type == "cuda":
            t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
            t.normal_(0.0, self.std, generator=self._gen(name, dev))
            return t
        return torch.randn(shape, generator=self._gen(name, "cpu"), dtype=torch.float32) * self.std


def _python_replacement(repl: str) -> str:
    """Replacement strings may name groups the ECMAScript way the reference's maps do (``$1``, ``$2`` ...;
    src/ksana_llm/utils/get_custom_weight_name.cpp:47 uses std::regex_replace) or the Python way (``\\1``): both are
    accepted, ``$$`` stands for a literal dollar sign."""
    out = re.sub(r"\$(\d+)", r"\\g<\1>", repl.replace("$$", "\0"))
    return out.replace("\0", "$")


def load_weight_map(model_type: str, path: Optional[str] = None, model_dir: Optional[str] = None,
                    hf_model_type: str = "") -> List[tuple]:
    """Rules of a weight map: an ordered list of (compiled pattern, replacement). ``path`` names a file outright (e.g.
    one written for the reference engine); otherwise the first of ``<hf_model_type>_weight_map.json`` (config.json's
    own spelling of the type) and ``<model_type>_weight_map.json`` (the family) that exists, looked for next to the
    checkpoint before the package's folder, so that a map shipped with a model wins
    (src/ksana_llm/utils/optional_file.h:23-61)."""
    from ..config import find_weight_map
    if path is None:
        for name in ([hf_model_type] if hf_model_type and hf_model_type != model_type else []) + [model_type]:
            path = find_weight_map(name, model_dir)
            if path:
                break
    if not path or not os.path.exists(path):
        return []
    with open(path, "r", encoding="utf-8") as f:
        return [(re.compile(k), _python_replacement(v)) for k, v in json.load(f).items()]


def apply_weight_map(name: str, rules: List[tuple]) -> str:
    for pat, repl in rules:
        new = pat.sub(repl, name)
        if new != name:
            name = new
    return name


# ------------------------------------------------------------------------------------- FP8 checkpoints
class Fp8Pair:
    """A projection weight as an FP8 checkpoint stores it: e4m3 values [N, K] and one fp32 scale per 128 x 128
    block [ceil(N/128), ceil(K/128)] (DeepSeek-V3 style ``weight_scale_inv``; a per-tensor ``weight_scale`` is
    spread over the blocks). Slicing for tensor parallelism and packing (QKV, gate|up, expert stacks) act on values
    and scales together as long as the cuts fall on block boundaries, so the checkpoint's own quantisation reaches
    the GEMMs unchanged (src/ksana_llm/models/quant/quant_weight.cpp:729-896 binds checkpoint scales per layer);
    a cut inside a block falls back to the dense fp32 values."""
    BLOCK = 128

    def __init__(self, q: torch.Tensor, s: torch.Tensor):
        self.q, self.s = q, s

    @property
    def shape(self):
        return self.q.shape

    def to(self, device=None, dtype=None, **kw):
        return Fp8Pair(self.q.to(device), self.s.to(device)) if device is not None else self

    def dense(self, dtype=torch.float32) -> torch.Tensor:
        N, K = self.q.shape
        full = self.s.float().repeat_interleave(self.BLOCK, 0)[:N].repeat_interleave(self.BLOCK, 1)[:, :K]
        return (self.q.float() * full.to(self.q.device)).to(dtype)

    def rows(self, lo: int, hi: int):
        hi = min(hi, self.q.shape[0])
        if lo % self.BLOCK or (hi % self.BLOCK and hi != self.q.shape[0]):
            return self.dense()[lo:hi]
        return Fp8Pair(self.q[lo:hi], self.s[lo // self.BLOCK:(hi + self.BLOCK - 1) // self.BLOCK])

    def cols(self, lo: int, hi: int):
        hi = min(hi, self.q.shape[1])
        if lo % self.BLOCK or (hi % self.BLOCK and hi != self.q.shape[1]):
            return self.dense()[:, lo:hi]
        return Fp8Pair(self.q[:, lo:hi], self.s[:, lo // self.BLOCK:(hi + self.BLOCK - 1) // self.BLOCK])

    def split(self, sizes, dim=0):
        assert dim == 0
        out, lo = [], 0
        for n in sizes:
            out.append(self.rows(lo, lo + n))
            lo += n
        return out

    def chunk(self, n, dim=0):
        assert dim == 0
        step = (self.q.shape[0] + n - 1) // n
        return self.split([min(step, self.q.shape[0] - i * step) for i in range(n)], 0)


def _dense(t, dtype=None):
    """Plain tensor of a weight (FP8 pairs are expanded exactly)."""
    if isinstance(t, Fp8Pair):
        return t.dense(dtype or torch.float32)
    return t


def _cat0(parts):
    """Row-wise concatenation of weights; FP8 pairs stay pairs when every part but the last ends on a block row."""
    if any(isinstance(p, Fp8Pair) for p in parts):
        if all(isinstance(p, Fp8Pair) for p in parts) and all(p.q.shape[0] % Fp8Pair.BLOCK == 0 for p in parts[:-1]):
            return Fp8Pair(torch.cat([p.q for p in parts], 0), torch.cat([p.s for p in parts], 0))
        return torch.cat([_dense(p) for p in parts], 0)
    return torch.cat(parts, 0)


class _Fp8Mixin:
    """``<layer>.weight`` stored as float8_e4m3fn with ``<layer>.weight_scale_inv`` (block scales) or a scalar
    ``<layer>.weight_scale`` is served as an Fp8Pair."""

    def _fp8_pair(self, name: str, t: torch.Tensor):
        if t.dtype != torch.float8_e4m3fn or t.dim() != 2 or not name.endswith(".weight"):
            return t
        nb, kb = (t.shape[0] + 127) // 128, (t.shape[1] + 127) // 128
        if self._has_raw(name + "_scale_inv"):
            s = self._get_raw(name + "_scale_inv").float()
            if tuple(s.shape) == (nb, kb):
                return Fp8Pair(t, s)
            return t.float() * s if s.numel() == 1 else t.float()
        if self._has_raw(name + "_scale"):
            s = self._get_raw(name + "_scale").float()
            if s.numel() == 1:
                return Fp8Pair(t, s.reshape(1, 1).expand(nb, kb).contiguous())
            if s.numel() == t.shape[0]:                       # one scale per output channel: no block form
                return t.float() * s.reshape(-1, 1)
        return t.float()



class _PackedW4Mixin:
    """``<layer>.weight`` of a GPTQ / AWQ layer (stored as qweight / qzeros / scales [/ g_idx]) is served as its exact
    dense expansion; see models/quant_w4.py."""

    def _packed(self, name: str) -> Optional[str]:
        if name.endswith(".weight"):
            base = name[: -len("weight")]
            if self._has_raw(base + "qweight") and self._has_raw(base + "scales"):
                return base
        return None

    def _dense_from_packed(self, base: str) -> torch.Tensor:
        from .quant_w4 import unpack_auto
        g_idx = self._get_raw(base + "g_idx") if self._has_raw(base + "g_idx") else None
        return unpack_auto(self._get_raw(base + "qweight"), self._get_raw(base + "qzeros"), self._get_raw(base + "scales"),
                           g_idx)


class CheckpointSource(_PackedW4Mixin, _Fp8Mixin):
    """Tensors of a Hugging Face checkpoint directory (``*.safetensors`` preferred, then ``*.bin`` /
    ``*.pt``), renamed to canonical names through the optional regex weight map."""

    def __init__(self, model_dir: str, model_type: str = "llama", hf_model_type: str = ""):
        self.rules = load_weight_map(model_type, model_dir=model_dir, hf_model_type=hf_model_type)
        self.index: Dict[str, tuple] = {}
        self._bin_cache: Dict[str, dict] = {}
        st = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        bins = sorted(glob.glob(os.path.join(model_dir, "*.bin")) + glob.glob(os.path.join(model_dir, "*.pt")))
        bins = [b for b in bins if "training_args" not in os.path.basename(b) and "optimizer" not in os.path.basename(b)]
        def add(kind, f, k):
            name = apply_weight_map(k, self.rules)
            transpose = name.endswith(".conv1d_t")        # GPT-2 style Conv1D weights are stored [in, out]
            if transpose:
                name = name[: -len(".conv1d_t")]
            self.index[name] = (kind, f, k, transpose)

        if st:
            from safetensors import safe_open
            for f in st:
                with safe_open(f, framework="pt") as sf:
                    for k in sf.keys():
                        add("st", f, k)
        elif bins:
            for f in bins:
                sd = torch.load(f, map_location="cpu", weights_only=True)
                self._bin_cache[f] = sd
                for k in sd.keys():
                    add("bin", f, k)
        else:
            raise FileNotFoundError(f"no safetensors / bin weights under {model_dir}")

    def has(self, name: str) -> bool:
        return name in self.index or self._packed(name) is not None

    def _has_raw(self, name: str) -> bool:
        return name in self.index

    def names(self):
        return list(self.index.keys())

    def get(self, name: str, shape=None, device="cpu", kind: str = "normal") -> torch.Tensor:
        if name not in self.index:
            base = self._packed(name)
            if base is not None:
                return self._dense_from_packed(base)
        return self._fp8_pair(name, self._get_raw(name))

    def _get_raw(self, name: str) -> torch.Tensor:
        kind_, f, k, transpose = self.index[name]
        if kind_ == "st":
            from safetensors import safe_open
            with safe_open(f, framework="pt") as sf:
                t = sf.get_tensor(k)
        else:
            t = self._bin_cache[f][k]
        return t.t().contiguous() if transpose else t


class DictSource(_PackedW4Mixin, _Fp8Mixin):
    def __init__(self, tensors: Dict[str, torch.Tensor], model_type: str = "llama"):
        rules = load_weight_map(model_type)
        self.t = {}
        for k, v in tensors.items():
            name = apply_weight_map(k, rules)
            if name.endswith(".conv1d_t"):
                name, v = name[: -len(".conv1d_t")], v.t().contiguous()
            self.t[name] = v

    def has(self, name):
        return name in self.t or self._packed(name) is not None

    def _has_raw(self, name):
        return name in self.t

    def _get_raw(self, name):
        return self.t[name]

    def names(self):
        return list(self.t.keys())

    def get(self, name, shape=None, device="cpu", kind="normal"):
        if name not in self.t:
            base = self._packed(name)
            if base is not None:
                return self._dense_from_packed(base)
        return self._fp8_pair(name, self.t[name])


# ------------------------------------------------------------------------------------- loader
def _rows(t, rank: int, size: int):
    n = (t.shape[0] + size - 1) // size
    if isinstance(t, Fp8Pair):
        return t.rows(rank * n, (rank + 1) * n)
    return t[rank * n:(rank + 1) * n]


def _cols(t, rank: int, size: int):
    n = (t.shape[1] + size - 1) // size
    if isinstance(t, Fp8Pair):
        return t.cols(rank * n, (rank + 1) * n)
    return t[:, rank * n:(rank + 1) * n]


def _make_linear(w, bias, device, dtype, quant: Optional[str]) -> LinearWeight:
    b = bias.to(device=device, dtype=dtype) if bias is not None else None
    if isinstance(w, Fp8Pair):
        if (quant is None or quant == "fp8_block") and w.shape[1] % 128 == 0:
            # the checkpoint's own FP8 values and block scales, bit for bit
            return LinearWeight(bias=b, wq=w.q.to(device).contiguous(), ws=w.s.float().to(device).contiguous())
        w = w.dense()
    w = w.to(device)
    if quant and quant.startswith("w4a16") and w.shape[1] % 32 == 0:
        group = int(quant.split(":")[1]) if ":" in quant else 128
        while w.shape[1] % group:
            group //= 2
        return LinearWeight(w=w.float(), bias=b).quantize_w4(max(group, 32))
    if quant == "nvfp4" and w.shape[1] % 256 == 0:
        lw = LinearWeight(w=w.float(), bias=b).quantize_nvfp4()
        return lw
    if quant in ("fp8_block", "nvfp4") and w.shape[1] % 128 == 0:
        wq, ws = ref.quant_weight_fp8_block(w)
        return LinearWeight(bias=b, wq=wq.contiguous(), ws=ws.contiguous())
    return LinearWeight(w=w.to(dtype).contiguous(), bias=b)


def build_model(cfg: ModelConfig, source, tp_rank: int = 0, tp_size: int = 1, comm=None, device="cpu",
                dtype=torch.bfloat16, quant: Optional[str] = None, layer_range=None, max_positions=None,
                model_cls=None) -> CommonModel:
    """Instantiate and fill a model. ``quant``: None | "fp8_block" (projection weights only; norms,
    embeddings, router and lm_head stay in ``dtype``)."""
    if cfg.is_mla:
        from .deepseek import build_deepseek
        return build_deepseek(cfg, source, tp_rank, tp_size, comm, device, dtype, quant, layer_range, max_positions)
    cls = model_cls or CommonModel
    m = cls(cfg, tp_rank, tp_size, comm, device, dtype, layer_range, max_positions=max_positions)
    H, D = cfg.hidden_size, cfg.head_dim
    Hq_all, Hkv_all = cfg.num_heads, cfg.num_kv_heads
    shard_on_device = isinstance(source, RandomSource) and source.on_device

    def get(name, shape, kind="normal"):
        return source.get(name, shape, device=device, kind=kind)

    def opt(name, shape, kind="zeros"):
        return get(name, shape, kind) if (source.has(name) and not isinstance(source, RandomSource)) or \
            (isinstance(source, RandomSource) and kind != "absent") else None

    ln = cfg.norm_type == "layernorm"
    if m.is_first_stage or cfg.tie_word_embeddings:
        m.embed = get("model.embed_tokens.weight", (cfg.vocab_size, H)).to(device=device, dtype=dtype)
        if cfg.position_embedding == "learned":
            m.pos_embed = get("model.embed_positions.weight", (cfg.max_position_embeddings, H)).to(device=device, dtype=dtype)
        elif cfg.position_embedding == "sinusoidal":
            m.pos_embed = _sinusoidal_table(cfg.max_position_embeddings + 2, H, cfg.pad_token_id).to(device=device, dtype=dtype)

    kv_rep = max(1, tp_size // Hkv_all)      # ranks sharing one kv head when tp > kv heads
    for li in range(m.layer_lo, m.layer_hi + 1):
        p = f"model.layers.{li}."
        if shard_on_device:
            qkv_w = get(p + f"self_attn.query_key_value.weight.tp{tp_rank}", ((m.Hq + 2 * m.Hkv) * D, H))
            qkv_b = get(p + "self_attn.query_key_value.bias", ((m.Hq + 2 * m.Hkv) * D,)) if cfg.qkv_bias else None
            o_w = get(p + f"self_attn.o_proj.weight.tp{tp_rank}", (H, m.Hq * D))
        else:
            if source.has(p + "self_attn.query_key_value.weight") and not isinstance(source, RandomSource):
                packed = get(p + "self_attn.query_key_value.weight", None)
                q_w, k_w, v_w = packed.split([Hq_all * D, Hkv_all * D, Hkv_all * D], dim=0)
                pb = get(p + "self_attn.query_key_value.bias", None) if source.has(p + "self_attn.query_key_value.bias") else None
                q_b, k_b, v_b = pb.split([Hq_all * D, Hkv_all * D, Hkv_all * D]) if pb is not None else (None, None, None)
            else:
                q_w = get(p + "self_attn.q_proj.weight", (Hq_all * D, H))
                k_w = get(p + "self_attn.k_proj.weight", (Hkv_all * D, H))
                v_w = get(p + "self_attn.v_proj.weight", (Hkv_all * D, H))
                has_b = cfg.qkv_bias and (isinstance(source, RandomSource) or source.has(p + "self_attn.q_proj.bias"))
                q_b = get(p + "self_attn.q_proj.bias", (Hq_all * D,)) if has_b else None
                k_b = get(p + "self_attn.k_proj.bias", (Hkv_all * D,)) if has_b else None
                v_b = get(p + "self_attn.v_proj.bias", (Hkv_all * D,)) if has_b else None
            kv_rank, kv_size = (tp_rank // kv_rep, tp_size // kv_rep) if tp_size > 1 else (0, 1)
            qkv_w = _cat0([_rows(q_w, tp_rank, tp_size), _rows(k_w, kv_rank, kv_size), _rows(v_w, kv_rank, kv_size)])
            qkv_b = None
            if q_b is not None:
                qkv_b = torch.cat([_rows(q_b, tp_rank, tp_size), _rows(k_b, kv_rank, kv_size), _rows(v_b, kv_rank, kv_size)], 0)
            o_w = _cols(get(p + "self_attn.o_proj.weight", (H, Hq_all * D)), tp_rank, tp_size)
        o_b = None
        if cfg.o_bias and (isinstance(source, RandomSource) or source.has(p + "self_attn.o_proj.bias")):
            o_b = get(p + "self_attn.o_proj.bias", (H,))
            if tp_rank != 0:
                o_b = torch.zeros_like(o_b)     # the bias is added once across the reduction
        lw = LayerWeights(
            input_norm=get(p + "input_layernorm.weight", (H,), "ones").to(device=device, dtype=dtype),
            input_norm_bias=get(p + "input_layernorm.bias", (H,), "zeros").to(device=device, dtype=dtype) if ln else None,
            qkv=_make_linear(qkv_w, qkv_b, device, dtype, quant),
            o_proj=_make_linear(o_w, o_b, device, dtype, quant),
            post_norm=get(p + "post_attention_layernorm.weight", (H,), "ones").to(device=device, dtype=dtype),
            post_norm_bias=get(p + "post_attention_layernorm.bias", (H,), "zeros").to(device=device, dtype=dtype) if ln else None,
        )
        is_moe_layer = cfg.is_moe and li >= cfg.first_k_dense_replace and (li % max(cfg.moe_layer_freq, 1) == 0)
        if is_moe_layer:
            from .moe import load_moe
            from .moe import ep_layout
            ep_rank, ep = ep_layout(cfg, tp_rank, tp_size)
            lw.moe = load_moe(cfg, source, p, tp_rank, tp_size, device, dtype, quant, ep_rank=ep_rank, ep_size=ep)
        else:
            inter = cfg.intermediate_size
            isz = (inter + tp_size - 1) // tp_size
            if shard_on_device:
                gu_w = get(p + f"mlp.gate_up_proj.weight.tp{tp_rank}", ((2 if cfg.gated_mlp else 1) * isz, H))
                d_w = get(p + f"mlp.down_proj.weight.tp{tp_rank}", (H, isz))
            else:
                if cfg.gated_mlp:
                    if source.has(p + "mlp.gate_up_proj.weight") and not isinstance(source, RandomSource):
                        g_w, u_w = get(p + "mlp.gate_up_proj.weight", None).chunk(2, dim=0)   # ChatGLM packs gate|up
                    else:
                        g_w = get(p + "mlp.gate_proj.weight", (inter, H))
                        u_w = get(p + "mlp.up_proj.weight", (inter, H))
                    gu_w = _cat0([_rows(g_w, tp_rank, tp_size), _rows(u_w, tp_rank, tp_size)])
                else:
                    gu_w = _rows(get(p + "mlp.up_proj.weight", (inter, H)), tp_rank, tp_size)
                d_w = _cols(get(p + "mlp.down_proj.weight", (H, inter)), tp_rank, tp_size)
            gu_b = d_b = None
            if cfg.mlp_bias:
                ub = get(p + "mlp.up_proj.bias", (inter,), "zeros")
                gu_b = _rows(ub, tp_rank, tp_size)
                d_b = get(p + "mlp.down_proj.bias", (H,), "zeros")
                if tp_rank != 0:
                    d_b = torch.zeros_like(d_b)
            lw.gate_up = _make_linear(gu_w, gu_b, device, dtype, quant)
            lw.down = _make_linear(d_w, d_b, device, dtype, quant)
        m.layers.append(lw)

    if m.is_last_stage:
        has_final = not cfg.post_norm
        if has_final:
            m.final_norm = get("model.norm.weight", (H,), "ones").to(device=device, dtype=dtype)
            m.final_norm_bias = get("model.norm.bias", (H,), "zeros").to(device=device, dtype=dtype) if ln else None
        tied = cfg.tie_word_embeddings or (not isinstance(source, RandomSource) and not source.has("lm_head.weight"))
        if tied:
            head = m.embed if m.embed is not None else get("model.embed_tokens.weight", (cfg.vocab_size, H))
        else:
            head = get("lm_head.weight", (cfg.vocab_size, H))
        head = head.float() if not head.is_cuda else head
        if cfg.lm_head_norm:
            head = torch.nn.functional.normalize(head.float(), dim=-1)
        # vocabulary shards are padded to a multiple of 8 rows for the GEMM epilogue's 16-byte stores
        vs = (cfg.vocab_size + tp_size - 1) // tp_size
        vs_pad = (vs + 7) // 8 * 8
        shard = head[tp_rank * vs:(tp_rank + 1) * vs]
        if shard.shape[0] < vs_pad:
            shard = torch.cat([shard, torch.zeros(vs_pad - shard.shape[0], H, dtype=shard.dtype, device=shard.device)], 0)
        m.lm_head = LinearWeight(w=shard.to(device=device, dtype=dtype).contiguous())
        m.vocab_shard = vs
    return m


def _sinusoidal_table(n: int, dim: int, padding_idx: int) -> torch.Tensor:
    """fairseq-style sinusoidal positions (sin | cos halves). fairseq numbers the positions of a sequence from
    ``padding_idx + 1`` on, so row p of this table (looked up with the engine's positions 0, 1, ...) holds the
    embedding of fairseq position ``p + padding_idx + 1``."""
    import math
    half = dim // 2
    emb = math.log(10000) / (half - 1)
    emb = torch.exp(torch.arange(half, dtype=torch.float32) * -emb)
    pos = torch.arange(n, dtype=torch.float32) + float(padding_idx + 1)
    emb = pos.unsqueeze(1) * emb.unsqueeze(0)
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=1)
    if dim % 2 == 1:
        emb = torch.cat([emb, torch.zeros(n, 1)], dim=1)
    return emb
