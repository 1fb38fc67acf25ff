// Observability of the engine: named metrics (counters and value distributions), request spans
// with W3C `traceparent` propagation, a chrome-trace event recorder with a writer thread, and
// scoped timers.
//
// Metric names and the chrome-trace event vocabulary are those of the reference, so dashboards
// and trace viewers carry over (src/ksana_llm/profiler/profiler.h:137-165,
// src/ksana_llm/profiler/trace_event_recorder.h:18-114, src/ksana_llm/profiler/reporter.h:42-55).
// Export is text based (Prometheus exposition, JSON lines); no OpenTelemetry SDK is required.
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

namespace pybind11 { class module_; }

namespace ksana {

struct MetricValue {
  int64_t count = 0;
  double sum = 0, min = 0, max = 0, last = 0;
  bool counter = false;      // reported through ReportCounter (a monotonic sum)
};

class Profiler {
 public:
  static Profiler& Instance();
  static const std::vector<std::string>& MetricNames();

  void SetAttributes(const std::map<std::string, std::string>& attrs);
  void ReportMetric(const std::string& name, double value);     // distribution sample / gauge
  void ReportCounter(const std::string& name, int64_t delta);   // monotonic counter
  std::map<std::string, MetricValue> Snapshot();
  std::string PrometheusText();
  std::string JsonLine();
  void Reset();

  // Periodic export: JsonLine() to a file ("debug" = stdout), or an OTLP/HTTP metrics request when the target is an
  // http:// URL (see otlp_export.h); stops with StopExport / destruction.
  void StartExport(const std::string& target, int interval_ms);
  void StopExport();

  // Spans. `traceparent` (may be empty) continues a caller's trace; returns the span id.
  std::string StartSpan(const std::string& name, const std::string& traceparent);
  void EndSpan(const std::string& span_id, const std::map<std::string, std::string>& attrs);
  void SetSpanSink(const std::string& target);   // file path, "debug" (stdout), an http:// URL (OTLP/HTTP) or "" (off)
  std::vector<std::string> FinishedSpans();      // JSON objects of spans ended so far (kept in memory, bounded)

  ~Profiler();

 private:
  Profiler();
  int64_t epoch_offset_us_ = 0;      // wall clock minus the monotonic clock spans are timed with
  int64_t start_unix_nano_ = 0;
  struct Span { std::string name, trace_id, span_id, parent_id; int64_t start_us; };
  std::mutex mu_;
  std::map<std::string, MetricValue> metrics_;
  std::map<std::string, std::string> attrs_;
  std::map<std::string, Span> open_spans_;
  std::deque<std::string> finished_spans_;
  std::string span_sink_;
  std::thread export_thread_;
  std::atomic<bool> export_stop_{false};
  std::condition_variable export_cv_;
  std::mutex export_mu_;
};

// Chrome-trace ("chrome://tracing", Perfetto) recorder with a background writer.
class TraceEventRecorder {
 public:
  static TraceEventRecorder& Instance();
  static const std::vector<std::string>& EventNames();
  void Enable(const std::string& path);    // default path comes from KLLM_EVENT_RECORD_FILE
  void Disable();                          // flushes and closes the JSON array
  bool enabled() const { return enabled_.load(); }
  // ph: "B" begin, "E" end, "i" instant, "C" counter
  void Record(const std::string& name, const std::string& phase, int64_t tid, double value);
  ~TraceEventRecorder();

 private:
  TraceEventRecorder() = default;
  void WriterLoop();
  std::atomic<bool> enabled_{false};
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::string> queue_;
  std::thread writer_;
  bool stop_ = false;
  std::string path_;
};

class ScopedTimer {   // reports elapsed milliseconds as a metric sample on destruction
 public:
  explicit ScopedTimer(std::string name);
  ~ScopedTimer();

 private:
  std::string name_;
  int64_t start_us_;
};

void BindProfiler(pybind11::module_& m);

}  // namespace ksana
