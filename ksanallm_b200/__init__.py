"""ksanallm_b200: a Blackwell-native LLM inference and serving engine."""
__version__ = "0.1.0"
