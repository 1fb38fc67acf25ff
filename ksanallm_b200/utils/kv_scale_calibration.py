"""Calibration of the per-layer KV-cache scales used with an FP8 KV cache.

The reference ships ready-made ``kv_scale_files/<model>/kv_cache_scales.json`` files for a few checkpoints
(src/ksana_llm/python/kv_scale_files/, read by src/ksana_llm/utils/environment.cpp:229-273) and has no tool to make
one. This module produces a file of the same format for any model: it runs calibration prompts through the engine
with an unquantised cache, takes the largest |K| and |V| every layer wrote, and stores ``amax / 448`` (the e4m3
range) per layer - one scale for both K and V of a layer, as the format has it.

  python -m ksanallm_b200.utils.kv_scale_calibration --config_file examples/ksana_llm.yaml \\
      --prompts prompts.txt --out kv_cache_scales.json
"""
from __future__ import annotations

import argparse
import json
from typing import Iterable, List, Sequence

import torch

E4M3_MAX = 448.0


def layer_amax(kv_cache: torch.Tensor) -> torch.Tensor:
    """[layers, 2] largest magnitudes of K and V in a paged cache [blocks, layers, 2, heads, tokens, head_dim]
    (blocks never written are zero and do not matter)."""
    return kv_cache.float().abs().amax(dim=(0, 3, 4, 5))


def calibrate_kv_scales(llm, prompts: Iterable[Sequence[int]], max_new_tokens: int = 8, batch: int = 8) -> List[float]:
    """Runs the prompts (token id lists) in batches and returns one scale per layer of this rank's model."""
    from ..utils import native_engine as ne
    cache = llm.model.kv_cache
    if cache is None or cache.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise ValueError("calibration needs an unquantised KV cache (kv_cache_dtype auto)")
    if cache.dim() != 6:
        raise ValueError("latent (MLA) caches are not FP8-quantised per layer: nothing to calibrate")
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos, s.topk = max_new_tokens, True, 1
    amax = torch.zeros(cache.shape[1], 2)
    group: List[Sequence[int]] = []

    def flush():
        nonlocal amax
        if group:
            llm.generate([list(p) for p in group], s)
            amax = torch.maximum(amax, layer_amax(llm.model.kv_cache).cpu())
            group.clear()

    for p in prompts:
        group.append(p)
        if len(group) >= batch:
            flush()
    flush()
    both = amax.amax(dim=1).clamp_min(1e-6)
    return [float(v) / E4M3_MAX for v in both]


def write_kv_scales(path: str, scales: Sequence[float], first_layer: int = 0) -> None:
    """The reference's file format: {"kv_cache": {"dtype": ..., "scaling_factor": {"0": {"<layer>": scale}}}}."""
    doc = {"model_type": "", "kv_cache": {"dtype": "float8_e4m3fn",
                                          "scaling_factor": {"0": {str(first_layer + i): float(v) for i, v in enumerate(scales)}}}}
    with open(path, "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=1)


def main(argv=None):
    ap = argparse.ArgumentParser(description="write kv_cache_scales.json for an FP8 KV cache")
    ap.add_argument("--config_file", required=True)
    ap.add_argument("--prompts", required=True, help="text file, one prompt per line")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max_new_tokens", type=int, default=8)
    ap.add_argument("--limit", type=int, default=128)
    args = ap.parse_args(argv)
    from ..serving.auto_model import AutoModel
    model = AutoModel.from_config(args.config_file)
    model.init_serving()
    tok = model.tokenizer
    with open(args.prompts, "r", encoding="utf-8") as f:
        lines = [ln.strip() for ln in f if ln.strip()][: args.limit]
    scales = calibrate_kv_scales(model.llm, (tok.encode(ln, add_special_tokens=True) for ln in lines), args.max_new_tokens)
    write_kv_scales(args.out, scales)
    print(json.dumps({"layers": len(scales), "max_scale": max(scales), "min_scale": min(scales), "out": args.out}))
    model.shutdown()


if __name__ == "__main__":
    main()
