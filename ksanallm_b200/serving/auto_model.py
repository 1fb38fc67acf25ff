"""``AutoModel.from_config(yaml)``: factory of the serving model (src/ksana_llm/python/ksana_llm/auto_model.py:11-30)."""
from .serving_model import ServingModel


class AutoModel:
    def __init__(self):
        raise EnvironmentError("AutoModel is created with AutoModel.from_config(config_file)")

    @classmethod
    def from_config(cls, config_file: str) -> ServingModel:
        return ServingModel(config_file)
