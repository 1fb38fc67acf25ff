// RPC endpoint plug-ins: a shared object `lib<name>_endpoint.so` that exports `Create<Name>Endpoint`, looked up at
// run time, as in the reference's endpoint factory (src/ksana_llm/endpoints/endpoint_factory.cpp:19-39).
// The plug-in receives a table of C callbacks into the engine (handle a serialized request, shut the service down)
// and returns an opaque endpoint with start / stop entry points, so it needs no headers of this project.
#pragma once
#include <string>

namespace ksana {

extern "C" {
// Callbacks handed to a plug-in. `handle` receives a request body (bytes) and writes the response through `reply`.
typedef void (*KsanaReplyFn)(void* reply_ctx, const char* data, unsigned long long len, int status);
typedef void (*KsanaHandleFn)(void* engine_ctx, const char* data, unsigned long long len, KsanaReplyFn reply, void* reply_ctx);
struct KsanaEndpointApi {
  void* engine_ctx;
  KsanaHandleFn handle_generate;
  KsanaHandleFn handle_forward;
  void (*shutdown_service)(void* engine_ctx);
};
struct KsanaEndpoint {
  void* self;
  int (*start)(void* self, const char* host, int port);
  int (*stop)(void* self);
};
typedef KsanaEndpoint* (*KsanaCreateEndpointFn)(const KsanaEndpointApi* api);
}

class EndpointPlugin {
 public:
  // Loads lib<name>_endpoint.so (searching `dir` first when given) and resolves Create<Name>Endpoint
  // (first letter upper-cased). Throws std::runtime_error with the loader's message on failure.
  EndpointPlugin(const std::string& name, const std::string& dir);
  ~EndpointPlugin();
  EndpointPlugin(const EndpointPlugin&) = delete;
  EndpointPlugin& operator=(const EndpointPlugin&) = delete;

  const std::string& symbol() const { return symbol_; }
  const std::string& path() const { return path_; }
  // Creates the endpoint with `api` and starts it; returns the plug-in's status code.
  int Start(const KsanaEndpointApi& api, const std::string& host, int port);
  int Stop();

 private:
  void* handle_ = nullptr;
  KsanaCreateEndpointFn create_ = nullptr;
  KsanaEndpoint* endpoint_ = nullptr;
  std::string symbol_, path_;
};

}  // namespace ksana
