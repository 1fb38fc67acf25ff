// OTLP over HTTP with JSON bodies (the OpenTelemetry protocol's /v1/traces and /v1/metrics requests), written
// against the protocol description only: no SDK. The profiler hands finished spans and periodic metric snapshots
// to this exporter when the configured export target is an http:// URL, which is how the reference sends both to a
// collector through the opentelemetry-cpp OTLP/HTTP exporters (src/ksana_llm/profiler/profiler.cpp:45-48, 88-93).
//
// One background thread owns the socket work: spans are batched (up to 64, or every 500 ms), a metrics request is
// sent when the profiler's export timer fires. A request that cannot be delivered within the timeout is dropped
// and counted; nothing here ever blocks the serving loop.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace ksana {

struct OtlpSpan {
  std::string name, trace_id, span_id, parent_id;
  int64_t start_us = 0, end_us = 0;
  std::map<std::string, std::string> attrs;
};

struct OtlpMetricPoint {
  std::string name;
  bool counter = false;     // monotonic sum; otherwise a distribution (count / sum / min / max)
  int64_t count = 0;
  double sum = 0, min = 0, max = 0;
};

struct OtlpUrl {
  std::string host, path;
  int port = 80;
  bool ok = false;
};
OtlpUrl ParseHttpUrl(const std::string& url);

// Request bodies (exposed for tests).
std::string OtlpTraceRequestJson(const std::vector<OtlpSpan>& spans, const std::map<std::string, std::string>& resource);
std::string OtlpMetricsRequestJson(const std::vector<OtlpMetricPoint>& points, const std::map<std::string, std::string>& resource,
                                   int64_t start_unix_nano, int64_t now_unix_nano);

// POST body to url; returns the HTTP status code, or a negative value (-1 resolve / connect, -2 send, -3 timeout or
// malformed answer).
int HttpPostJson(const OtlpUrl& url, const std::string& body, int timeout_ms);

class OtlpExporter {
 public:
  static OtlpExporter& Instance();
  void Configure(const std::map<std::string, std::string>& resource, int timeout_ms);
  void EnqueueSpan(const std::string& url, OtlpSpan span);
  void EnqueueMetrics(const std::string& url, std::vector<OtlpMetricPoint> points, int64_t start_unix_nano);
  void Flush(int wait_ms);                 // wait until the queue is empty (tests, shutdown)
  int64_t sent() const { return sent_; }
  int64_t dropped() const { return dropped_; }
  ~OtlpExporter();

 private:
  OtlpExporter() = default;
  void Loop();
  void EnsureThread();
  struct Job { std::string url, body; };
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::pair<std::string, OtlpSpan>> spans_;
  std::deque<Job> jobs_;
  std::map<std::string, std::string> resource_;
  int timeout_ms_ = 1000;
  bool stop_ = false, busy_ = false;
  std::thread thread_;
  std::atomic<int64_t> sent_{0}, dropped_{0};
};

}  // namespace ksana
