"""Plugin host: a model directory (or the working directory / an installed package) may ship a
``ksana_plugin.py`` with a ``KsanaPlugin`` class offering ``init_plugin``, ``preprocess`` and
``postprocess``. Pre-processing may rewrite the input tokens, add ``input_refit_embedding`` entries
(e.g. vision-tower outputs) and ``additional_tensors`` (e.g. multimodal rotary positions).
Behaviour follows src/ksana_llm/python/ksana_llm/ksana_plugin.py:19-190.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Optional


@dataclass
class PluginConfig:
    model_dir: str = ""
    config_file: str = ""
    plugin_name: str = ""
    enable_trt: bool = True
    thread_num: int = 1


def search_plugin_path(model_dir: str, plugin_name: str = "") -> Optional[str]:
    """Search order: model_dir, current working directory, installed ``ksana_plugin/<name>`` package dir."""
    cands = [os.path.join(model_dir, "ksana_plugin.py"), os.path.join(os.getcwd(), "ksana_plugin.py")]
    if plugin_name:
        here = os.path.dirname(os.path.abspath(__file__))
        cands.append(os.path.join(here, "..", "ksana_plugin", plugin_name, "ksana_plugin.py"))
        for p in sys.path:
            cands.append(os.path.join(p, "ksana_plugin", plugin_name, "ksana_plugin.py"))
    for c in cands:
        if c and os.path.isfile(c):
            return os.path.abspath(c)
    return None


class KsanaPlugin:
    def __init__(self, config: PluginConfig):
        self.config = config
        self._plugin = None
        self._pool = ThreadPoolExecutor(max_workers=max(1, config.thread_num))
        path = search_plugin_path(config.model_dir, config.plugin_name)
        if path is not None:
            spec = importlib.util.spec_from_file_location("ksana_plugin_user", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            cls = getattr(mod, "KsanaPlugin", None)
            if cls is not None:
                self._plugin = cls()
                if hasattr(self._plugin, "init_plugin"):
                    self._plugin.init_plugin(model_path=config.model_dir, enable_trt=config.enable_trt,
                                             preprocess=True, postprocess=True)

    @property
    def loaded(self) -> bool:
        return self._plugin is not None

    def preprocess(self, **kwargs):
        if self._plugin is None or not hasattr(self._plugin, "preprocess"):
            return None
        return self._pool.submit(self._plugin.preprocess, **kwargs).result()

    def postprocess(self, **kwargs):
        if self._plugin is None or not hasattr(self._plugin, "postprocess"):
            return None
        return self._pool.submit(self._plugin.postprocess, **kwargs).result()
