#include "otlp_export.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>
#include <fcntl.h>

#include <cerrno>
#include <cmath>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "logger.h"

namespace ksana {
namespace {

std::string Esc(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 8);
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof(b), "\\u%04x", c); o += b; }
        else o += static_cast<char>(c);
    }
  }
  return o;
}

void Attributes(std::ostringstream& o, const std::map<std::string, std::string>& kv) {
  o << "[";
  bool first = true;
  for (const auto& a : kv) {
    o << (first ? "" : ",") << "{\"key\":\"" << Esc(a.first) << "\",\"value\":{\"stringValue\":\"" << Esc(a.second) << "\"}}";
    first = false;
  }
  o << "]";
}

std::map<std::string, std::string> WithServiceName(std::map<std::string, std::string> r) {
  if (!r.count("service.name")) r["service.name"] = "ksana_llm";
  return r;
}

// JSON has no spelling for infinities and NaN (the minimum of a metric without samples): they go out as 0
double Num(double v) { return std::isfinite(v) ? v : 0.0; }

int64_t NowNano() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

}  // namespace

OtlpUrl ParseHttpUrl(const std::string& url) {
  OtlpUrl u;
  const std::string scheme = "http://";
  if (url.compare(0, scheme.size(), scheme) != 0) return u;     // https is not spoken here
  std::string rest = url.substr(scheme.size());
  const size_t slash = rest.find('/');
  std::string hostport = slash == std::string::npos ? rest : rest.substr(0, slash);
  u.path = slash == std::string::npos ? "/" : rest.substr(slash);
  const size_t colon = hostport.rfind(':');
  if (colon != std::string::npos) {
    u.host = hostport.substr(0, colon);
    u.port = atoi(hostport.c_str() + colon + 1);
  } else {
    u.host = hostport;
  }
  u.ok = !u.host.empty() && u.port > 0 && u.port < 65536;
  return u;
}

std::string OtlpTraceRequestJson(const std::vector<OtlpSpan>& spans, const std::map<std::string, std::string>& resource) {
  std::ostringstream o;
  o << "{\"resourceSpans\":[{\"resource\":{\"attributes\":";
  Attributes(o, WithServiceName(resource));
  o << "},\"scopeSpans\":[{\"scope\":{\"name\":\"ksana_llm\"},\"spans\":[";
  bool first = true;
  for (const auto& s : spans) {
    o << (first ? "" : ",") << "{\"traceId\":\"" << s.trace_id << "\",\"spanId\":\"" << s.span_id << "\"";
    if (!s.parent_id.empty()) o << ",\"parentSpanId\":\"" << s.parent_id << "\"";
    // kind 2 = server; times are unix nanoseconds as decimal strings (64-bit integers in the JSON mapping)
    o << ",\"name\":\"" << Esc(s.name) << "\",\"kind\":2,\"startTimeUnixNano\":\"" << s.start_us * 1000
      << "\",\"endTimeUnixNano\":\"" << s.end_us * 1000 << "\",\"attributes\":";
    Attributes(o, s.attrs);
    o << ",\"status\":{}}";
    first = false;
  }
  o << "]}]}]}";
  return o.str();
}

std::string OtlpMetricsRequestJson(const std::vector<OtlpMetricPoint>& points, const std::map<std::string, std::string>& resource,
                                   int64_t start_unix_nano, int64_t now_unix_nano) {
  std::ostringstream o;
  o.precision(17);
  o << "{\"resourceMetrics\":[{\"resource\":{\"attributes\":";
  Attributes(o, WithServiceName(resource));
  o << "},\"scopeMetrics\":[{\"scope\":{\"name\":\"ksana_llm\"},\"metrics\":[";
  bool first = true;
  for (const auto& p : points) {
    o << (first ? "" : ",") << "{\"name\":\"" << Esc(p.name) << "\",";
    const std::string times = "\"startTimeUnixNano\":\"" + std::to_string(start_unix_nano) + "\",\"timeUnixNano\":\"" +
                              std::to_string(now_unix_nano) + "\"";
    if (p.counter) {
      // cumulative (2) monotonic sum since the profiler started
      o << "\"sum\":{\"dataPoints\":[{" << times << ",\"asDouble\":" << Num(p.sum)
        << "}],\"aggregationTemporality\":2,\"isMonotonic\":true}}";
    } else {
      // a histogram without buckets carries the count, sum, minimum and maximum of the samples
      o << "\"histogram\":{\"dataPoints\":[{" << times << ",\"count\":\"" << p.count << "\",\"sum\":" << Num(p.sum)
        << ",\"min\":" << Num(p.min) << ",\"max\":" << Num(p.max) << "}],\"aggregationTemporality\":2}}";
    }
    first = false;
  }
  o << "]}]}]}";
  return o.str();
}

int HttpPostJson(const OtlpUrl& url, const std::string& body, int timeout_ms) {
  if (!url.ok) return -1;
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(url.host.c_str(), std::to_string(url.port).c_str(), &hints, &res) != 0 || !res) return -1;
  int fd = -1;
  for (addrinfo* a = res; a; a = a->ai_next) {
    fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
    int rc = connect(fd, a->ai_addr, a->ai_addrlen);
    if (rc != 0 && errno == EINPROGRESS) {
      pollfd p{fd, POLLOUT, 0};
      int err = 0; socklen_t len = sizeof(err);
      if (poll(&p, 1, timeout_ms) == 1 && getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &len) == 0 && err == 0) rc = 0;
    }
    if (rc == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return -1;
  std::ostringstream req;
  req << "POST " << url.path << " HTTP/1.1\r\nHost: " << url.host << ":" << url.port
      << "\r\nContent-Type: application/json\r\nContent-Length: " << body.size() << "\r\nConnection: close\r\n\r\n" << body;
  const std::string data = req.str();
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  auto left = [&]() {
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
    return ms > 0 ? static_cast<int>(ms) : 0;
  };
  size_t off = 0;
  while (off < data.size()) {
    pollfd p{fd, POLLOUT, 0};
    if (poll(&p, 1, left()) != 1) { close(fd); return -3; }
    const ssize_t n = send(fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) continue;      // poll again, within the deadline
    if (n <= 0) { close(fd); return -2; }
    off += static_cast<size_t>(n);
  }
  std::string answer;
  char buf[512];
  while (answer.find("\r\n") == std::string::npos) {
    pollfd p{fd, POLLIN, 0};
    if (poll(&p, 1, left()) != 1) { close(fd); return -3; }
    const ssize_t n = recv(fd, buf, sizeof(buf), 0);
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) continue;
    if (n <= 0) break;
    answer.append(buf, static_cast<size_t>(n));
  }
  close(fd);
  // "HTTP/1.1 200 OK"
  if (answer.size() < 12 || answer.compare(0, 5, "HTTP/") != 0) return -3;
  return atoi(answer.c_str() + 9);
}

OtlpExporter& OtlpExporter::Instance() {
  static OtlpExporter e;
  return e;
}

void OtlpExporter::Configure(const std::map<std::string, std::string>& resource, int timeout_ms) {
  std::lock_guard<std::mutex> g(mu_);
  resource_ = resource;
  if (timeout_ms > 0) timeout_ms_ = timeout_ms;
}

void OtlpExporter::EnsureThread() {
  if (!thread_.joinable()) thread_ = std::thread([this]() { Loop(); });
}

void OtlpExporter::EnqueueSpan(const std::string& url, OtlpSpan span) {
  std::lock_guard<std::mutex> g(mu_);
  if (spans_.size() >= 8192) { ++dropped_; return; }       // the collector is away: keep memory bounded
  spans_.emplace_back(url, std::move(span));
  EnsureThread();
  if (spans_.size() >= 64) cv_.notify_all();
}

void OtlpExporter::EnqueueMetrics(const std::string& url, std::vector<OtlpMetricPoint> points, int64_t start_unix_nano) {
  std::lock_guard<std::mutex> g(mu_);
  if (jobs_.size() >= 64) { ++dropped_; return; }
  jobs_.push_back({url, OtlpMetricsRequestJson(points, resource_, start_unix_nano, NowNano())});
  EnsureThread();
  cv_.notify_all();
}

void OtlpExporter::Loop() {
  std::unique_lock<std::mutex> lk(mu_);
  while (!stop_) {
    if (spans_.empty() && jobs_.empty()) cv_.wait_for(lk, std::chrono::milliseconds(500));
    else if (spans_.size() < 64 && jobs_.empty()) cv_.wait_for(lk, std::chrono::milliseconds(500));
    if (stop_ && spans_.empty() && jobs_.empty()) break;
    // one request per target URL and batch
    std::vector<Job> out;
    while (!spans_.empty()) {
      const std::string url = spans_.front().first;
      std::vector<OtlpSpan> batch;
      for (auto it = spans_.begin(); it != spans_.end() && batch.size() < 256;) {
        if (it->first == url) { batch.push_back(std::move(it->second)); it = spans_.erase(it); }
        else ++it;
      }
      out.push_back({url, OtlpTraceRequestJson(batch, resource_)});
    }
    while (!jobs_.empty()) { out.push_back(std::move(jobs_.front())); jobs_.pop_front(); }
    const int timeout = timeout_ms_;
    busy_ = true;
    lk.unlock();
    for (const auto& j : out) {
      const int code = HttpPostJson(ParseHttpUrl(j.url), j.body, timeout);
      if (code >= 200 && code < 300) ++sent_;
      else {
        ++dropped_;
        KLLM_LOG_WARNING << "OTLP export to " << j.url << " failed (" << code << "), request dropped";
      }
    }
    lk.lock();
    busy_ = false;
    cv_.notify_all();
  }
}

void OtlpExporter::Flush(int wait_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  cv_.notify_all();
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(wait_ms);
  while ((!spans_.empty() || !jobs_.empty() || busy_) && std::chrono::steady_clock::now() < deadline) {
    cv_.notify_all();
    cv_.wait_for(lk, std::chrono::milliseconds(20));
  }
}

OtlpExporter::~OtlpExporter() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

}  // namespace ksana
