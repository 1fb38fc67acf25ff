#include "endpoint_plugin.h"

#include <dlfcn.h>

#include <cctype>
#include <stdexcept>

namespace ksana {

EndpointPlugin::EndpointPlugin(const std::string& name, const std::string& dir) {
  if (name.empty()) throw std::runtime_error("endpoint plug-in name is empty");
  const std::string file = "lib" + name + "_endpoint.so";
  std::string err;
  for (const std::string& cand : {dir.empty() ? std::string() : dir + "/" + file, file}) {
    if (cand.empty()) continue;
    handle_ = dlopen(cand.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (handle_) { path_ = cand; break; }
    const char* e = dlerror();
    err = e ? e : "dlopen failed";
  }
  if (!handle_) throw std::runtime_error("cannot load endpoint plug-in " + file + ": " + err);
  symbol_ = "Create" + name + "Endpoint";
  symbol_[6] = static_cast<char>(std::toupper(static_cast<unsigned char>(symbol_[6])));
  create_ = reinterpret_cast<KsanaCreateEndpointFn>(dlsym(handle_, symbol_.c_str()));
  if (!create_) {
    dlclose(handle_);
    handle_ = nullptr;
    throw std::runtime_error("endpoint plug-in " + path_ + " does not export " + symbol_);
  }
}

EndpointPlugin::~EndpointPlugin() {
  if (endpoint_) Stop();
  if (handle_) dlclose(handle_);
}

int EndpointPlugin::Start(const KsanaEndpointApi& api, const std::string& host, int port) {
  if (!endpoint_) endpoint_ = create_(&api);
  if (!endpoint_ || !endpoint_->start) return -1;
  return endpoint_->start(endpoint_->self, host.c_str(), port);
}

int EndpointPlugin::Stop() {
  int rc = 0;
  if (endpoint_ && endpoint_->stop) rc = endpoint_->stop(endpoint_->self);
  endpoint_ = nullptr;
  return rc;
}

}  // namespace ksana
