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
import threading
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Optional

from ..utils import logger


@dataclass
class PluginConfig:
    model_dir: str = ""
    config_file: str = ""
    plugin_name: str = ""
    enable_trt: bool = True
    thread_pool_size: int = 1          # plug-in calls in flight at once; above 1 the plug-in must be thread-safe


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
    """Loads the plug-in and runs its calls on a small thread pool. On a GPU every pool thread works in a CUDA stream
    of its own (and waits for it before returning), so that a vision tower neither queues behind the engine's step on
    the default stream nor holds it up."""

    def __init__(self, config: PluginConfig):
        self.config = config
        self._plugin = None
        workers = max(1, min(int(config.thread_pool_size), 32, (os.cpu_count() or 1) * 5))
        self._pool = ThreadPoolExecutor(max_workers=workers)
        self._streams = {}
        self._streams_lock = threading.Lock()
        path = search_plugin_path(config.model_dir, config.plugin_name)
        if path is None:
            return
        # plug-ins written for the reference import their helpers as top-level modules (``from plugin_utils import
        # ...``) and their own neighbours by folder name: both folders go on the import path
        helpers = os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "ksana_plugin"))
        for folder in (helpers, os.path.dirname(os.path.dirname(path))):
            if folder not in sys.path:
                sys.path.append(folder)
        try:
            spec = importlib.util.spec_from_file_location("ksana_plugin_user", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            cls = getattr(mod, "KsanaPlugin", None)
            if cls is None:
                logger.warning(f"plug-in {path} has no KsanaPlugin class; serving without it")
                return
            plugin = cls()
            if hasattr(plugin, "init_plugin"):
                plugin.init_plugin(model_path=config.model_dir, config_file=config.config_file,
                                   enable_trt=config.enable_trt, preprocess=True, postprocess=True)
            self._plugin = plugin
            logger.info(f"plug-in loaded from {path} ({workers} worker thread(s))")
        except Exception as e:  # noqa: BLE001 - a broken plug-in must not keep the text model from serving
            logger.warning(f"plug-in {path} could not be loaded ({e!r}); serving without it")

    @property
    def loaded(self) -> bool:
        return self._plugin is not None

    def _call(self, fn, kwargs):
        import torch
        if not torch.cuda.is_available():
            return fn(**kwargs)
        ident = threading.get_ident()
        with self._streams_lock:
            stream = self._streams.get(ident)
            if stream is None:
                stream = self._streams[ident] = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            out = fn(**kwargs)
        stream.synchronize()          # what the plug-in wrote (embeddings) is complete before the engine reads it
        return out

    def preprocess(self, **kwargs):
        if self._plugin is None or not hasattr(self._plugin, "preprocess"):
            return None
        return self._pool.submit(self._call, self._plugin.preprocess, kwargs).result()

    def postprocess(self, **kwargs):
        if self._plugin is None or not hasattr(self._plugin, "postprocess"):
            return None
        return self._pool.submit(self._call, self._plugin.postprocess, kwargs).result()
