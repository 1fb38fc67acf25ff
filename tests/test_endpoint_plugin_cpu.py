"""RPC endpoint plug-ins: a shared object built on the fly is found by name, started with callbacks into the
serving model, sends a request through them and can ask for a service shutdown."""
import json
import os
import subprocess

import pytest
import torch

from helpers import ByteTokenizer, tiny_model_cfg
from ksanallm_b200.utils import native_engine as ne

PLUGIN_SRC = r'''
#include <cstring>
#include <string>
extern "C" {
typedef void (*ReplyFn)(void*, const char*, unsigned long long, int);
typedef void (*HandleFn)(void*, const char*, unsigned long long, ReplyFn, void*);
struct Api { void* ctx; HandleFn generate; HandleFn forward; void (*shutdown)(void*); };
struct Endpoint { void* self; int (*start)(void*, const char*, int); int (*stop)(void*); };
static Api g_api;
static std::string g_reply;
static int g_status = -1, g_port = 0, g_stopped = 0;
static void on_reply(void*, const char* d, unsigned long long n, int status) { g_reply.assign(d, n); g_status = status; }
static int start(void*, const char* host, int port) {
  g_port = port;
  const char* body = "{\"input_tokens\": [1, 5, 6, 7], \"sampling_config\": {\"max_new_tokens\": 4, \"ignore_eos\": true}}";
  g_api.generate(g_api.ctx, body, std::strlen(body), on_reply, nullptr);   // a real plug-in would do this per RPC
  return std::strcmp(host, "127.0.0.1") == 0 ? 0 : 3;
}
static int stop(void*) { g_stopped = 1; return 0; }
static Endpoint g_ep{nullptr, start, stop};
Endpoint* CreateEchoEndpoint(const Api* api) { g_api = *api; return &g_ep; }
const char* echo_last_reply() { return g_reply.c_str(); }
int echo_last_status() { return g_status; }
int echo_stopped() { return g_stopped; }
void echo_request_shutdown() { g_api.shutdown(g_api.ctx); }
}
'''


@pytest.fixture(scope="module")
def plugin_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("plugin")
    src = d / "echo.cpp"
    src.write_text(PLUGIN_SRC)
    subprocess.run(["g++", "-shared", "-fPIC", "-O1", "-o", str(d / "libecho_endpoint.so"), str(src)], check=True)
    return str(d)


def test_loader_resolves_symbol_and_reports_errors(plugin_dir):
    p = ne.EndpointPlugin("echo", plugin_dir)
    assert p.symbol == "CreateEchoEndpoint" and p.path.endswith("libecho_endpoint.so")
    calls = []
    rc = p.start(lambda kind, body: (calls.append((kind, body)) or (200, b"ok")), None, "127.0.0.1", 9000)
    assert rc == 0 and calls and calls[0][0] == "generate" and b"input_tokens" in calls[0][1]
    assert p.stop() == 0
    with pytest.raises(RuntimeError, match="cannot load endpoint plug-in"):
        ne.EndpointPlugin("missing", plugin_dir)


def test_serving_model_starts_the_named_endpoint(plugin_dir):
    import ctypes
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.serving.serving_model import EndpointConfig, ServingModel
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.model_dir = plugin_dir
    ec.batch_scheduler.max_token_len = 64
    ec.block_manager.device_blocks_num = 64
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving(endpoint_config=EndpointConfig("echo", "127.0.0.1", 9123))
    lib = ctypes.CDLL(os.path.join(plugin_dir, "libecho_endpoint.so"))
    lib.echo_last_reply.restype = ctypes.c_char_p
    assert lib.echo_last_status() == 200
    body = json.loads(lib.echo_last_reply().decode())
    assert body["input_token_ids"] == [1, 5, 6, 7] and len(body["output_token_ids"][0]) == 4
    assert not model.wait_for_shutdown(0)
    lib.echo_request_shutdown()                      # the plug-in lost its peer: it asks the service to stop
    assert lib.echo_stopped() == 1 and model.rpc_endpoint is None
    assert model.wait_for_shutdown(0)                # what the server process of an RPC endpoint waits for
