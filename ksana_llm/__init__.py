"""Import-compatibility package: code written against KsanaLLM's Python package (``import ksana_llm``;
``ksana_llm.AutoModel.from_config(yaml)``, ``ksana_llm.EndpointConfig``, ``ksana_llm.PluginConfig``, as exported by
src/ksana_llm/python/ksana_llm/__init__.py in the reference) runs on this engine unchanged. Everything lives in
``ksanallm_b200``; this package only re-exports the serving surface under the old name."""
from ksanallm_b200.serving.auto_model import AutoModel
from ksanallm_b200.serving.plugin import KsanaPlugin, PluginConfig
from ksanallm_b200.serving.serving_model import EndpointConfig, ServingModel

__all__ = ["AutoModel", "EndpointConfig", "KsanaPlugin", "PluginConfig", "ServingModel"]
