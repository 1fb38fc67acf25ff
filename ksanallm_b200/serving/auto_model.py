"""``AutoModel.from_config(yaml)``: factory of the serving model (src/ksana_llm/python/ksana_llm/auto_model.py:11-30)."""
import os

from .serving_model import ServingModel


class AutoModel:
    def __init__(self):
        raise EnvironmentError("AutoModel is created with AutoModel.from_config(config_file)")

    @classmethod
    def from_config(cls, config_file, **kwargs) -> ServingModel:
        """The serving model of a YAML configuration; the file must exist and be a ``.yaml`` (checked here, before any
        weight is touched). Extra keyword arguments are accepted and ignored, as callers of the reference pass them."""
        config_file = os.fspath(config_file)
        if not os.path.exists(config_file):
            raise RuntimeError(f"The config file {config_file} does not exist.")
        if not config_file.lower().endswith((".yaml", ".yml")):
            raise RuntimeError(f"The config file {config_file} must be in YAML format.")
        return ServingModel(config_file)
