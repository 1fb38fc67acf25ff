"""Command-line client of ``/generate`` (counterpart of src/ksana_llm/python/serving_generate_client.py in the
reference, which posts a fixed prompt with a sampling configuration to --host / --port):

  python serving_generate_client.py --port 8080 --prompt "Hello" --max_new_tokens 32 [--stream]
"""
import argparse
import json

from ksanallm_b200.serving import clients


def args_config(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--host", type=str, default="localhost", help="server host address")
    p.add_argument("--port", type=int, default=8888, help="server port")
    p.add_argument("--prompt", type=str, default="Hello, my name is")
    p.add_argument("--input_tokens", type=int, nargs="*", default=None, help="token ids instead of a text prompt")
    p.add_argument("--stream", action="store_true")
    p.add_argument("--max_new_tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--topk", type=int, default=1)
    p.add_argument("--topp", type=float, default=1.0)
    p.add_argument("--num_beams", type=int, default=1)
    p.add_argument("--num_return_sequences", type=int, default=1)
    p.add_argument("--logprobs", type=int, default=0)
    p.add_argument("--stop_strings", type=str, nargs="*", default=None)
    p.add_argument("--structured_output_regex", type=str, default=None)
    return p.parse_args(argv)


def main(argv=None):
    a = args_config(argv)
    sampling = {"temperature": a.temperature, "topk": a.topk, "topp": a.topp, "max_new_tokens": a.max_new_tokens,
                "num_beams": a.num_beams, "num_return_sequences": a.num_return_sequences, "logprobs": a.logprobs}
    if a.stop_strings:
        sampling["stop_strings"] = a.stop_strings
    extra = {"structured_output_regex": a.structured_output_regex} if a.structured_output_regex else {}
    url = f"http://{a.host}:{a.port}"
    res = clients.generate(url, prompt=None if a.input_tokens else a.prompt, input_tokens=a.input_tokens,
                           sampling_config=sampling, stream=a.stream, **extra)
    if a.stream:
        for chunk in res["chunks"]:
            print(json.dumps(chunk, ensure_ascii=False))
    else:
        print(json.dumps(res, ensure_ascii=False, indent=1))
    return res


if __name__ == "__main__":
    main()
