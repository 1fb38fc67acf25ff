"""Stand-alone server process end to end (the shape of the reference's tests/integration_test.py): a tiny Hugging
Face Llama checkpoint and tokenizer are written to disk, ``python serving_server.py --config_file X.yaml --port P`` is
started as a child process - alone, as two tensor-parallel ranks under torchrun (rank 0 serves, the others follow the
broadcast step plans) and as four ranks (more ranks than KV heads: neighbouring ranks hold copies of one KV head, and the
vocabulary does not divide by four) - and the answers of /generate (blocking and streaming) are compared token by token with Hugging
Face's own greedy generation from the same files."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import torch

transformers = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")
requests = pytest.importorskip("requests")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_model(path: str):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast
    words = ["<unk>", "<s>", "</s>"] + [f"w{i}" for i in range(60)] + ["the", "cat", "sat", "on", "mat", "hello", "world"]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")
    fast.chat_template = ("{% for m in messages %}{{ 'w1 ' if m['role'] == 'user' else 'w2 ' }}{{ m['content'] }} {% endfor %}"
                          "{% if add_generation_prompt %}w3{% endif %}")
    fast.save_pretrained(path)
    cfg = LlamaConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                      vocab_size=len(words), max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False,
                      bos_token_id=1, eos_token_id=2, torch_dtype="float32")
    torch.manual_seed(3)
    model = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.3)
    model.save_pretrained(path, safe_serialization=True)
    return model, fast


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module", params=[1, 2, 4], ids=["one-process", "two-tensor-parallel-ranks", "four-ranks-sharing-kv-heads"])
def served(request, tmp_path_factory):
    nproc = request.param
    d = tmp_path_factory.mktemp("served")
    model_dir = str(d / "model")
    os.makedirs(model_dir)
    model, tok = _write_model(model_dir)
    yaml_path = str(d / "ksana_llm.yaml")
    with open(yaml_path, "w", encoding="utf-8") as f:
        f.write(f"""setting:
  global:
    tensor_para_size: {nproc}
    enable_cuda_graph: false
    comm_backend: nccl
  batch_scheduler:
    max_batch_size: 8
    max_token_len: 96
    max_step_tokens: 256
    enable_auto_prefix_cache: true
  block_manager:
    block_token_num: 16
    device_blocks_num: 64
  endpoint_type: python
model_spec:
  base_model:
    model_dir: {model_dir}
""")
    port = _free_port()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    launcher = [sys.executable] if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
        "--master-port", str(_free_port())]
    proc = subprocess.Popen(launcher + [os.path.join(ROOT, "serving_server.py"), "--config_file", yaml_path, "--host",
                                        "127.0.0.1", "--port", str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                            env=env, start_new_session=True)
    deadline = time.time() + 120
    up = False
    while time.time() < deadline and proc.poll() is None:
        try:
            if requests.get(f"http://127.0.0.1:{port}/health", timeout=1).status_code == 200:
                up = True
                break
        except Exception:
            time.sleep(0.5)
    if not up:
        out = proc.stdout.read().decode(errors="replace")[-3000:] if proc.poll() is not None else ""
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass
        pytest.fail("server did not come up: " + out)
    yield f"http://127.0.0.1:{port}", model, tok
    try:
        os.killpg(proc.pid, signal.SIGTERM)
        proc.wait(timeout=20)
    except Exception:
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass


def _hf_greedy(model, tok, prompt, n):
    ids = tok(prompt, return_tensors="pt").input_ids
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=n, do_sample=False, eos_token_id=None, pad_token_id=0)
    return ids[0].tolist(), out[0, ids.shape[1]:].tolist()


def test_generate_matches_hugging_face_greedy(served):
    url, model, tok = served
    for prompt in ("the cat sat on the mat", "hello world w1 w2 w3 w4 w5"):
        ids, want = _hf_greedy(model, tok, prompt, 12)
        r = requests.post(url + "/generate", json={"prompt": prompt, "stream": False,
                                                   "sampling_config": {"max_new_tokens": 12, "topk": 1, "ignore_eos": True}})
        assert r.status_code == 200, r.text
        body = r.json()
        assert body["input_token_ids"] == ids
        assert body["output_token_ids"][0] == want
        assert body["texts"][0].split() == tok.decode(want).split()


def test_streaming_and_token_input(served):
    url, model, tok = served
    ids, want = _hf_greedy(model, tok, "w7 w8 w9 the cat", 8)
    r = requests.post(url + "/generate", json={"input_tokens": ids, "stream": True,
                                               "sampling_config": {"max_new_tokens": 8, "topk": 1, "ignore_eos": True}}, stream=True)
    chunks = [json.loads(c) for c in r.content.split(b"\0") if c]
    assert chunks and chunks[-1]["output_token_ids"][0] == want
    lens = [len(c["output_token_ids"][0]) for c in chunks]
    assert lens == sorted(lens) and lens[-1] == 8
    m = requests.get(url + "/metrics").text
    assert "forward_req_total_num" in m or "metric_" in m


def test_chat_messages_and_stop_strings(served):
    """OpenAI-style messages go through the tokenizer's chat template on the server; a stop string cuts the answer
    where Hugging Face's text has it."""
    url, model, tok = served
    messages = [{"role": "user", "content": "the cat sat"}, {"role": "assistant", "content": "on the mat"},
                {"role": "user", "content": "hello world"}]
    ids = tok.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
    ids = list(ids["input_ids"]) if hasattr(ids, "keys") else list(ids)
    with torch.no_grad():
        out = model.generate(torch.tensor([ids]), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0)
    want = out[0, len(ids):].tolist()
    r = requests.post(url + "/generate", json={"messages": messages, "stream": False,
                                               "sampling_config": {"max_new_tokens": 10, "topk": 1, "ignore_eos": True}})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["input_token_ids"] == ids and body["output_token_ids"][0] == want
    words = tok.decode(want, skip_special_tokens=True).split()      # the server's text leaves special tokens out
    stop = words[4]
    cut = words.index(stop)
    r = requests.post(url + "/generate", json={"messages": messages, "stream": False,
                                               "sampling_config": {"max_new_tokens": 10, "topk": 1, "ignore_eos": True,
                                                                   "stop_strings": [stop]}})
    got = r.json()["output_token_ids"][0]
    assert tok.decode(got, skip_special_tokens=True).split() == words[:cut]


def test_parallel_sampling_beams_and_logprobs(served):
    url, model, tok = served
    prompt = "the cat sat on"
    r = requests.post(url + "/generate", json={"prompt": prompt, "stream": False,
                                               "sampling_config": {"max_new_tokens": 6, "topk": 5, "temperature": 0.9,
                                                                   "num_return_sequences": 3, "ignore_eos": True, "logprobs": 2}})
    assert r.status_code == 200, r.text
    body = r.json()
    assert len(body["output_token_ids"]) == 3 and all(len(o) == 6 for o in body["output_token_ids"])
    assert len(body["logprobs"]) == 3 and all(len(lp) == 6 for lp in body["logprobs"])
    # greedy first token must be among the top-2 log-probabilities reported for step 0
    ids, want = _hf_greedy(model, tok, prompt, 1)
    top_ids = {int(t) for t, _ in body["logprobs"][0][0]}
    assert want[0] in top_ids
    r = requests.post(url + "/generate", json={"prompt": prompt, "stream": False,
                                               "sampling_config": {"max_new_tokens": 5, "num_beams": 3, "num_return_sequences": 2,
                                                                   "logprobs": 3, "ignore_eos": True}})
    assert r.status_code == 200, r.text
    beams = r.json()["output_token_ids"]
    assert len(beams) == 2 and all(len(b) == 5 for b in beams) and beams[0] != beams[1]


def test_auto_model_from_config_loads_the_tokenizer_beside_the_checkpoint(tmp_path):
    """`ksana_llm.AutoModel.from_config(yaml)` (the package API of the reference) without an explicit tokenizer: the one
    in the model directory is used, so stop strings work on a model created that way."""
    import ksana_llm
    model_dir = str(tmp_path / "model")
    os.makedirs(model_dir)
    hf, tok = _write_model(model_dir)
    yaml_path = str(tmp_path / "k.yaml")
    with open(yaml_path, "w", encoding="utf-8") as f:
        f.write(f"""setting:
  global: {{tensor_para_size: 1, enable_cuda_graph: false}}
  batch_scheduler: {{max_batch_size: 4, max_token_len: 96, max_step_tokens: 256}}
  block_manager: {{block_token_num: 16, device_blocks_num: 32}}
  endpoint_type: python
model_spec:
  base_model: {{model_dir: {model_dir}}}
""")
    sm = ksana_llm.AutoModel.from_config(yaml_path)
    sm.init_serving(device="cpu")
    try:
        assert sm.tokenizer is not None and sm.llm.engine.tokenizer is sm.tokenizer
        ids, want = _hf_greedy(hf, tok, "the cat sat on the mat", 8)
        st, out = sm.generate(inputs=ids, generation_config={"max_new_tokens": 8, "ignore_eos": True})
        assert st.OK() and out.output_tokens[0] == want
        words = tok.decode(want, skip_special_tokens=True).split()
        st, out = sm.generate(inputs=ids, generation_config={"max_new_tokens": 8, "ignore_eos": True, "stop_strings": [words[3]]})
        assert st.OK() and tok.decode(out.output_tokens[0], skip_special_tokens=True).split() == words[:words.index(words[3])]
    finally:
        sm.shutdown()


def test_forward_perplexity_matches_hugging_face(served):
    """/forward with a logits GATHER_TOKEN_ID target returns the probabilities of the prompt's own next tokens; the
    perplexity computed from them equals the one from Hugging Face's logits (the check of the reference's
    src/ksana_llm/python/tests/test_models.py)."""
    import math
    from ksanallm_b200.serving import clients
    url, model, tok = served
    prompt = "the cat sat on the mat hello world w1 w2"
    ids = tok(prompt).input_ids
    doc = clients.forward(url, [{"prompt": prompt, "request_target": [{"target_name": "logits", "token_reduce_mode": "GATHER_TOKEN_ID",
                                                                      "slice_pos": [[0, len(ids) - 2]]}]}])
    got = clients.perplexity_from_forward(doc)[0]
    with torch.no_grad():
        logp = torch.log_softmax(model(torch.tensor([ids])).logits[0].float(), -1)
    nll = -sum(float(logp[i, ids[i + 1]]) for i in range(len(ids) - 1)) / (len(ids) - 1)
    assert math.isclose(got, math.exp(nll), rel_tol=2e-3)


def test_cpp_forward_client_against_the_live_server(served):
    """The stand-alone C++ /forward client (own msgpack codec, plain sockets) posts its two-request batch - a text
    prompt and a token list, each with a logits GATHER_TOKEN_ID target - and prints the probabilities it got back."""
    import re
    from urllib.parse import urlparse
    from ksanallm_b200.build import build_client
    url, model, tok = served
    u = urlparse(url)
    exe = str(build_client())
    r = subprocess.run([exe, "-s", u.hostname, "-p", str(u.port), "-a", "forward"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    blocks = re.findall(r"input_token_ids : \[ ([\d ]+)\], target_name : logits, tensor : \n\[ ([-\d. e]+)\]", r.stdout)
    assert len(blocks) == 2, r.stdout
    second_ids = [int(x) for x in blocks[1][0].split()]
    assert second_ids == [1, 22, 13]
    # slice (-3, -2) of a three-token input = positions 0 and 1: the probabilities of tokens 22 and 13 given their prefixes
    probs = [float(x) for x in blocks[1][1].split()]
    with torch.no_grad():
        p = torch.softmax(model(torch.tensor([second_ids])).logits[0].float(), -1)
    assert len(probs) == 2 and abs(probs[0] - float(p[0, 22])) < 2e-3 and abs(probs[1] - float(p[1, 13])) < 2e-3
    assert "request duration:" in r.stdout
