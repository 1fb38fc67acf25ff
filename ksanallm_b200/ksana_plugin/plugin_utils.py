"""Helpers for plug-in authors, under the names plug-ins written for the reference import
(src/ksana_llm/python/ksana_plugin/plugin_utils.py:8-57): ``from plugin_utils import free_cache, ...`` works because the
plug-in host puts this folder on the import path before it loads a plug-in."""
from __future__ import annotations

import gc
import importlib.util
import os
import re

import torch


def free_cache() -> None:
    """Drops unreferenced Python objects and returns the allocator's cached device memory (after a tower was built)."""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def load_safetensors(file_path: str) -> dict:
    """All tensors of one ``.safetensors`` file as a name -> tensor dict (on the host)."""
    from safetensors import safe_open
    out = {}
    with safe_open(file_path, framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


def check_file_dir(file_path: str) -> None:
    """Creates the folder a file is about to be written into."""
    folder = os.path.dirname(file_path)
    if folder:
        os.makedirs(folder, exist_ok=True)


def get_module(module_name: str, py_path: str, class_name: str):
    """Attribute ``class_name`` of the Python file ``py_path`` loaded as module ``module_name``."""
    spec = importlib.util.spec_from_file_location(module_name, py_path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return getattr(module, class_name)


_RESERVED = re.compile(r"^(\s*reserved_device_memory_ratio:\s*)([0-9]*\.?[0-9]+(?:[eE][-+]?[0-9]+)?)(.*)$", re.MULTILINE)


def adjust_device_memory_ratio(config_file: str, reserved_device_memory_ratio: float) -> bool:
    """Raises ``reserved_device_memory_ratio`` in a YAML configuration to at least the given share (room for a vision
    tower beside the KV cache), editing the one line in place so that comments and key order survive. Returns whether
    the file changed; a file without the key, or with a larger value already, is left alone."""
    with open(config_file, "r", encoding="utf-8") as f:
        text = f.read()
    m = _RESERVED.search(text)
    if m is None or float(m.group(2)) >= reserved_device_memory_ratio:
        return False
    text = text[:m.start()] + f"{m.group(1)}{reserved_device_memory_ratio}{m.group(3)}" + text[m.end():]
    with open(config_file, "w", encoding="utf-8") as f:
        f.write(text)
    return True
