// Stand-alone C++ client of the /forward endpoint: two requests in one msgpack batch (a text prompt and a list of token
// ids, each asking for the `logits` target gathered at chosen positions), the reply's tensors printed as numbers.
//
// Same job as the reference's example client (src/ksana_llm/cpp/serving_forward_client.cpp:1-141), without its
// third-party HTTP and msgpack libraries: the body is built and parsed with the engine's own msgpack codec
// (csrc/engine/request_packer.{h,cpp}) and sent over a plain POSIX socket as one HTTP/1.1 POST.
//
//   serving_forward_client [-s HOST] [-p PORT] [-a API]        (defaults: localhost 8888 forward)
//
// Build: python -m ksanallm_b200.build --client   (g++ -std=c++17 -DKSANA_NO_PYBIND ... -o lib/serving_forward_client)
#include <arpa/inet.h>
#include <getopt.h>
#include <netdb.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../engine/request_packer.h"

using ksana::MsgValue;

namespace {

struct Args {
  std::string host = "localhost";
  int port = 8888;
  std::string api = "forward";
};

[[noreturn]] void Usage(const char* prog) {
  std::cout << "usage: " << prog << " [-h, --help] [-s, --host HOST] [-p, --port PORT] [-a, --api API]\n";
  std::exit(1);
}

Args ParseArgs(int argc, char** argv) {
  Args a;
  const option opts[] = {{"host", required_argument, nullptr, 's'}, {"port", required_argument, nullptr, 'p'},
                         {"api", required_argument, nullptr, 'a'},  {"help", no_argument, nullptr, 'h'},
                         {nullptr, 0, nullptr, 0}};
  int c;
  while ((c = getopt_long(argc, argv, "s:p:a:h", opts, nullptr)) != -1) {
    if (c == 's') a.host = optarg;
    else if (c == 'p') a.port = std::atoi(optarg);
    else if (c == 'a') a.api = optarg;
    else Usage(argv[0]);
  }
  return a;
}

// ---- msgpack value helpers
MsgValue Str(const std::string& s) { MsgValue v; v.kind = MsgValue::STR; v.s = s; return v; }
MsgValue Int(int64_t i) { MsgValue v; v.kind = MsgValue::INT; v.i = i; return v; }
MsgValue Arr(std::vector<MsgValue> items) { MsgValue v; v.kind = MsgValue::ARRAY; v.items = std::move(items); return v; }
MsgValue Map(std::vector<std::pair<std::string, MsgValue>> kv) {
  MsgValue v;
  v.kind = MsgValue::MAP;
  for (auto& e : kv) v.fields.emplace_back(Str(e.first), std::move(e.second));
  return v;
}

MsgValue LogitsTarget(int begin, int end) {
  return Map({{"target_name", Str("logits")},
              {"slice_pos", Arr({Arr({Int(begin), Int(end)})})},      // sorted inclusive intervals; negative = from the end
              {"token_reduce_mode", Str("GATHER_TOKEN_ID")}});
}

// ---- one HTTP/1.1 POST over a blocking socket; returns the status code, the body in *body
int HttpPost(const Args& a, const std::string& payload, std::string* body) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(a.host.c_str(), std::to_string(a.port).c_str(), &hints, &res) != 0 || !res)
    throw std::runtime_error("cannot resolve " + a.host);
  int fd = -1;
  for (addrinfo* p = res; p; p = p->ai_next) {
    fd = ::socket(p->ai_family, p->ai_socktype, p->ai_protocol);
    if (fd < 0) continue;
    if (::connect(fd, p->ai_addr, p->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) throw std::runtime_error("cannot connect to " + a.host + ":" + std::to_string(a.port));
  std::string req = "POST /" + a.api + " HTTP/1.1\r\nHost: " + a.host + ":" + std::to_string(a.port) +
                    "\r\nContent-Type: application/x-msgpack\r\nContent-Length: " + std::to_string(payload.size()) +
                    "\r\nConnection: close\r\n\r\n" + payload;
  for (size_t off = 0; off < req.size();) {
    const ssize_t n = ::send(fd, req.data() + off, req.size() - off, 0);
    if (n <= 0) { ::close(fd); throw std::runtime_error("send failed"); }
    off += static_cast<size_t>(n);
  }
  std::string raw;
  char buf[65536];
  for (;;) {
    const ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
    if (n <= 0) break;                       // Connection: close -> the server ends the reply by closing
    raw.append(buf, static_cast<size_t>(n));
  }
  ::close(fd);
  const size_t hdr_end = raw.find("\r\n\r\n");
  if (hdr_end == std::string::npos || raw.compare(0, 5, "HTTP/") != 0) throw std::runtime_error("malformed HTTP reply");
  const int status = std::atoi(raw.c_str() + raw.find(' ') + 1);
  std::string head = raw.substr(0, hdr_end);
  for (auto& ch : head) ch = static_cast<char>(::tolower(ch));
  std::string rest = raw.substr(hdr_end + 4);
  if (head.find("transfer-encoding: chunked") != std::string::npos) {
    body->clear();
    for (size_t pos = 0; pos < rest.size();) {
      const size_t eol = rest.find("\r\n", pos);
      if (eol == std::string::npos) break;
      const size_t len = std::strtoul(rest.substr(pos, eol - pos).c_str(), nullptr, 16);
      if (len == 0) break;
      body->append(rest, eol + 2, len);
      pos = eol + 2 + len + 2;
    }
  } else {
    *body = std::move(rest);
  }
  return status;
}

std::string Base64Decode(const std::string& in) {
  std::string out;
  int val = 0, bits = -8;
  for (unsigned char c : in) {
    int d;
    if (c >= 'A' && c <= 'Z') d = c - 'A';
    else if (c >= 'a' && c <= 'z') d = c - 'a' + 26;
    else if (c >= '0' && c <= '9') d = c - '0' + 52;
    else if (c == '+' || c == '-') d = 62;
    else if (c == '/' || c == '_') d = 63;
    else continue;                           // padding / whitespace
    val = (val << 6) | d;
    bits += 6;
    if (bits >= 0) { out.push_back(static_cast<char>((val >> bits) & 0xff)); bits -= 8; }
  }
  return out;
}

}  // namespace

int main(int argc, char** argv) {
  const Args args = ParseArgs(argc, argv);
  try {
    const auto t0 = std::chrono::steady_clock::now();
    MsgValue batch = Map({{"requests", Arr({
        Map({{"prompt", Str("Hello, world!")}, {"request_target", Arr({LogitsTarget(0, 1)})}}),
        Map({{"input_tokens", Arr({Int(1), Int(22), Int(13)})}, {"request_target", Arr({LogitsTarget(-3, -2)})}})})}});
    std::string body;
    const int status = HttpPost(args, ksana::MsgPack(batch), &body);
    if (status != 200) {
      std::cerr << "server answered HTTP " << status << ": " << body.substr(0, 400) << std::endl;
      return 2;
    }
    const MsgValue doc = ksana::MsgUnpack(body);
    const MsgValue* responses = doc.Find("responses");
    if (!responses || responses->kind != MsgValue::ARRAY) {
      const MsgValue* msg = doc.Find("message");
      std::cerr << "no responses in the reply" << (msg ? ": " + msg->s : std::string()) << std::endl;
      return 3;
    }
    std::cout.setf(std::ios::fixed);
    std::cout.precision(5);
    for (const MsgValue& one : responses->items) {
      const MsgValue* ids = one.Find("input_token_ids");
      const MsgValue* targets = one.Find("response");
      if (!targets) continue;
      for (const MsgValue& t : targets->items) {
        const MsgValue* name = t.Find("target_name");
        const MsgValue* tensor = t.Find("tensor");
        if (!tensor) continue;
        const MsgValue* data = tensor->Find("data");
        const MsgValue* dtype = tensor->Find("dtype");
        const MsgValue* shape = tensor->Find("shape");
        if (!data || !dtype || dtype->s != "float32") {     // C++ has no half-precision primitive: the example asks for fp32
          std::cerr << "unexpected tensor dtype " << (dtype ? dtype->s : "?") << std::endl;
          continue;
        }
        // raw bytes (msgpack bin) from this engine; base64 text from servers that encode tensors that way
        const std::string bytes = data->kind == MsgValue::BIN ? data->s : Base64Decode(data->s);
        size_t count = 1;
        if (shape)
          for (const MsgValue& d : shape->items) count *= static_cast<size_t>(d.kind == MsgValue::UINT ? d.u : d.i);
        if (count * sizeof(float) != bytes.size()) { std::cerr << "tensor size does not match its shape\n"; continue; }
        std::vector<float> values(count);
        std::memcpy(values.data(), bytes.data(), bytes.size());
        std::cout << "input_token_ids : [ ";
        if (ids)
          for (const MsgValue& tok : ids->items) std::cout << (tok.kind == MsgValue::UINT ? static_cast<int64_t>(tok.u) : tok.i) << " ";
        std::cout << "], target_name : " << (name ? name->s : "?") << ", tensor : \n[ ";
        for (float v : values) std::cout << v << " ";
        std::cout << "]" << std::endl;
      }
    }
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    std::cout << "request duration: " << ms << " ms" << std::endl;
  } catch (const std::exception& e) {
    std::cerr << "error: " << e.what() << std::endl;
    return 1;
  }
  return 0;
}
