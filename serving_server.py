"""``python serving_server.py --config_file X.yaml --port P``: the reference's server entry point under its own name
(src/ksana_llm/python/serving_server.py); the implementation is ``ksanallm_b200.serving.serving_server``."""
from ksanallm_b200.serving.serving_server import main

if __name__ == "__main__":
    main()
