#include "profiler.h"
#include "otlp_export.h"

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <random>
#include <sstream>

#include "common.h"

namespace ksana {

namespace {
std::string HexId(int bytes) {
  static thread_local std::mt19937_64 rng(std::random_device{}() ^ static_cast<uint64_t>(NowUs()));
  static const char* d = "0123456789abcdef";
  std::string s;
  for (int i = 0; i < bytes; ++i) {
    const uint64_t r = rng();
    s.push_back(d[(r >> 4) & 15]);
    s.push_back(d[r & 15]);
  }
  return s;
}
std::string JsonEscape(const std::string& in) {
  std::string o;
  for (char c : in) {
    if (c == '"' || c == '\\') { o.push_back('\\'); o.push_back(c); }
    else if (c == '\n') o += "\\n";
    else if (static_cast<unsigned char>(c) < 0x20) o += ' ';
    else o.push_back(c);
  }
  return o;
}
bool IsHttp(const std::string& target) { return target.compare(0, 7, "http://") == 0; }
void EmitLine(const std::string& target, const std::string& line) {
  if (target.empty() || IsHttp(target)) return;
  if (target == "debug") { std::cout << line << std::endl; return; }
  std::ofstream f(target, std::ios::app);
  f << line << "\n";
}
}  // namespace

Profiler::Profiler() {
  const int64_t wall_us = std::chrono::duration_cast<std::chrono::microseconds>(
      std::chrono::system_clock::now().time_since_epoch()).count();
  epoch_offset_us_ = wall_us - NowUs();
  start_unix_nano_ = wall_us * 1000;
}

Profiler& Profiler::Instance() {
  static Profiler p;
  return p;
}

const std::vector<std::string>& Profiler::MetricNames() {
  static const std::vector<std::string> names = {
      "forward_req_total_num", "forward_req_error_num", "forward_req_timeout_num", "forward_req_aborted_num",
      "forward_cost_time_ms", "prefix_cache_hit_req_num", "prefix_cache_hit_token_num", "prefix_cache_hit_block_num",
      "full_prompt_matched_req_num", "full_prompt_matched_block_num", "batch_scheduler_batch_size",
      "batch_scheduler_waiting_size", "batch_scheduler_swapped_size", "batch_scheduler_pending_swapin_size",
      "batch_scheduler_pending_swapout_size", "batch_manager_schedule_ms", "req_total_cost_in_queue_ms",
      "token_num_in_batch", "token_fill_ratio", "block_num_free", "block_num_used", "time_to_first_token_ms",
      "time_to_per_output_token_ms", "metric_input_tokens_num", "metric_output_token_num"};
  return names;
}

void Profiler::SetAttributes(const std::map<std::string, std::string>& attrs) {
  {
    std::lock_guard<std::mutex> g(mu_);
    attrs_ = attrs;
  }
  OtlpExporter::Instance().Configure(attrs, 0);
}

void Profiler::ReportMetric(const std::string& name, double value) {
  std::lock_guard<std::mutex> g(mu_);
  MetricValue& m = metrics_[name];
  if (m.count == 0) { m.min = value; m.max = value; }
  m.min = std::min(m.min, value);
  m.max = std::max(m.max, value);
  m.sum += value;
  m.last = value;
  ++m.count;
}

void Profiler::ReportCounter(const std::string& name, int64_t delta) {
  std::lock_guard<std::mutex> g(mu_);
  MetricValue& m = metrics_[name];
  m.sum += static_cast<double>(delta);
  m.last = m.sum;
  m.max = m.sum;
  m.counter = true;
  ++m.count;
}

std::map<std::string, MetricValue> Profiler::Snapshot() {
  std::lock_guard<std::mutex> g(mu_);
  return metrics_;
}

void Profiler::Reset() {
  std::lock_guard<std::mutex> g(mu_);
  metrics_.clear();
  open_spans_.clear();
  finished_spans_.clear();
}

std::string Profiler::PrometheusText() {
  std::lock_guard<std::mutex> g(mu_);
  std::ostringstream o;
  std::string labels;
  for (auto& kv : attrs_) labels += (labels.empty() ? "" : ",") + kv.first + "=\"" + JsonEscape(kv.second) + "\"";
  const std::string l = labels.empty() ? "" : "{" + labels + "}";
  for (const auto& name : MetricNames()) {
    auto it = metrics_.find(name);
    const MetricValue m = it == metrics_.end() ? MetricValue() : it->second;
    o << "# TYPE ksana_" << name << " summary\n";
    o << "ksana_" << name << "_count" << l << " " << m.count << "\n";
    o << "ksana_" << name << "_sum" << l << " " << m.sum << "\n";
    o << "ksana_" << name << "_last" << l << " " << m.last << "\n";
  }
  for (auto& kv : metrics_) {
    if (std::find(MetricNames().begin(), MetricNames().end(), kv.first) != MetricNames().end()) continue;
    o << "ksana_" << kv.first << "_count" << l << " " << kv.second.count << "\n";
    o << "ksana_" << kv.first << "_sum" << l << " " << kv.second.sum << "\n";
  }
  return o.str();
}

std::string Profiler::JsonLine() {
  std::lock_guard<std::mutex> g(mu_);
  std::ostringstream o;
  o << "{\"ts_ms\":" << NowMs() << ",\"attributes\":{";
  bool first = true;
  for (auto& kv : attrs_) { o << (first ? "" : ",") << "\"" << JsonEscape(kv.first) << "\":\"" << JsonEscape(kv.second) << "\""; first = false; }
  o << "},\"metrics\":{";
  first = true;
  for (auto& kv : metrics_) {
    o << (first ? "" : ",") << "\"" << kv.first << "\":{\"count\":" << kv.second.count << ",\"sum\":" << kv.second.sum
      << ",\"min\":" << kv.second.min << ",\"max\":" << kv.second.max << ",\"last\":" << kv.second.last << "}";
    first = false;
  }
  o << "}}";
  return o.str();
}

void Profiler::StartExport(const std::string& target, int interval_ms) {
  StopExport();
  export_stop_ = false;
  export_thread_ = std::thread([this, target, interval_ms]() {
    std::unique_lock<std::mutex> lk(export_mu_);
    while (!export_stop_) {
      export_cv_.wait_for(lk, std::chrono::milliseconds(interval_ms));
      if (export_stop_) break;
      if (IsHttp(target)) {
        std::vector<OtlpMetricPoint> points;
        for (const auto& kv : Snapshot()) {
          OtlpMetricPoint p;
          p.name = "ksana_" + kv.first;
          p.counter = kv.second.counter;
          p.count = kv.second.count; p.sum = kv.second.sum; p.min = kv.second.min; p.max = kv.second.max;
          points.push_back(std::move(p));
        }
        OtlpExporter::Instance().EnqueueMetrics(target, std::move(points), start_unix_nano_);
      } else {
        EmitLine(target, JsonLine());
      }
    }
  });
}

void Profiler::StopExport() {
  {
    std::lock_guard<std::mutex> lk(export_mu_);
    export_stop_ = true;
  }
  export_cv_.notify_all();
  if (export_thread_.joinable()) export_thread_.join();
}

Profiler::~Profiler() { StopExport(); }

std::string Profiler::StartSpan(const std::string& name, const std::string& traceparent) {
  Span s;
  s.name = name;
  s.start_us = NowUs();
  s.span_id = HexId(8);
  // traceparent: version-traceid(32 hex)-parentid(16 hex)-flags
  if (traceparent.size() >= 55 && traceparent[2] == '-' && traceparent[35] == '-') {
    s.trace_id = traceparent.substr(3, 32);
    s.parent_id = traceparent.substr(36, 16);
  } else {
    s.trace_id = HexId(16);
  }
  std::lock_guard<std::mutex> g(mu_);
  open_spans_[s.span_id] = s;
  return s.span_id;
}

void Profiler::EndSpan(const std::string& span_id, const std::map<std::string, std::string>& attrs) {
  std::string line, sink;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = open_spans_.find(span_id);
    if (it == open_spans_.end()) return;
    const Span& s = it->second;
    std::ostringstream o;
    o << "{\"name\":\"" << JsonEscape(s.name) << "\",\"trace_id\":\"" << s.trace_id << "\",\"span_id\":\"" << s.span_id
      << "\",\"parent_id\":\"" << s.parent_id << "\",\"start_us\":" << s.start_us << ",\"duration_us\":"
      << (NowUs() - s.start_us) << ",\"attributes\":{";
    bool first = true;
    for (auto& kv : attrs) { o << (first ? "" : ",") << "\"" << JsonEscape(kv.first) << "\":\"" << JsonEscape(kv.second) << "\""; first = false; }
    o << "}}";
    line = o.str();
    finished_spans_.push_back(line);
    while (finished_spans_.size() > 4096) finished_spans_.pop_front();
    sink = span_sink_;
    if (IsHttp(sink)) {
      OtlpSpan os;
      os.name = s.name; os.trace_id = s.trace_id; os.span_id = s.span_id; os.parent_id = s.parent_id;
      os.start_us = s.start_us + epoch_offset_us_;
      os.end_us = NowUs() + epoch_offset_us_;
      os.attrs = attrs;
      open_spans_.erase(it);
      OtlpExporter::Instance().EnqueueSpan(sink, std::move(os));
      return;
    }
    open_spans_.erase(it);
  }
  EmitLine(sink, line);
}

void Profiler::SetSpanSink(const std::string& target) {
  std::lock_guard<std::mutex> g(mu_);
  span_sink_ = target;
}

std::vector<std::string> Profiler::FinishedSpans() {
  std::lock_guard<std::mutex> g(mu_);
  return std::vector<std::string>(finished_spans_.begin(), finished_spans_.end());
}

// ------------------------------------------------------------------------ chrome trace
TraceEventRecorder& TraceEventRecorder::Instance() {
  static TraceEventRecorder r;
  return r;
}

const std::vector<std::string>& TraceEventRecorder::EventNames() {
  static const std::vector<std::string> names = {"SchedBegin", "DropReq", "FinishReq", "Prefill", "Decode", "SwapOut",
                                                 "SwapIn", "InputTokenNum", "ForwardTokenNum", "TokenNumPerSec",
                                                 "UsableBlockNum", "FutureBlockNum"};
  return names;
}

void TraceEventRecorder::Enable(const std::string& path_in) {
  Disable();
  std::string path = path_in;
  if (path.empty()) {
    const char* env = std::getenv("KLLM_EVENT_RECORD_FILE");
    path = env ? env : "log/ksana_event_record.json";
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    path_ = path;
    stop_ = false;
    queue_.clear();
    std::ofstream f(path_, std::ios::trunc);
    f << "[\n";
  }
  enabled_ = true;
  writer_ = std::thread(&TraceEventRecorder::WriterLoop, this);
}

void TraceEventRecorder::Disable() {
  if (!writer_.joinable()) { enabled_ = false; return; }
  enabled_ = false;
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  writer_.join();
  std::ofstream f(path_, std::ios::app);
  f << "{\"name\":\"end\",\"ph\":\"i\",\"ts\":" << NowUs() << ",\"pid\":0,\"tid\":0,\"s\":\"g\"}\n]\n";
}

void TraceEventRecorder::Record(const std::string& name, const std::string& phase, int64_t tid, double value) {
  if (!enabled_) return;
  std::ostringstream o;
  o << "{\"name\":\"" << JsonEscape(name) << "\",\"ph\":\"" << phase << "\",\"ts\":" << NowUs()
    << ",\"pid\":0,\"tid\":" << tid;
  if (phase == "C") o << ",\"args\":{\"value\":" << value << "}";
  else if (phase == "i") o << ",\"s\":\"t\",\"args\":{\"value\":" << value << "}";
  else o << ",\"args\":{\"value\":" << value << "}";
  o << "},";
  {
    std::lock_guard<std::mutex> g(mu_);
    queue_.push_back(o.str());
  }
  cv_.notify_one();
}

void TraceEventRecorder::WriterLoop() {
  std::unique_lock<std::mutex> lk(mu_);
  while (true) {
    cv_.wait_for(lk, std::chrono::milliseconds(200), [this] { return stop_ || !queue_.empty(); });
    std::deque<std::string> batch;
    batch.swap(queue_);
    const bool stop = stop_;
    lk.unlock();
    if (!batch.empty()) {
      std::ofstream f(path_, std::ios::app);
      for (auto& l : batch) f << l << "\n";
    }
    lk.lock();
    if (stop && queue_.empty()) break;
  }
}

TraceEventRecorder::~TraceEventRecorder() { Disable(); }

ScopedTimer::ScopedTimer(std::string name) : name_(std::move(name)), start_us_(NowUs()) {}
ScopedTimer::~ScopedTimer() { Profiler::Instance().ReportMetric(name_, (NowUs() - start_us_) / 1000.0); }

void BindProfiler(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("metric_names", []() { return Profiler::MetricNames(); });
  m.def("trace_event_names", []() { return TraceEventRecorder::EventNames(); });
  m.def("report_metric", [](const std::string& n, double v) { Profiler::Instance().ReportMetric(n, v); });
  m.def("report_counter", [](const std::string& n, int64_t d) { Profiler::Instance().ReportCounter(n, d); });
  m.def("metrics_snapshot", []() {
    py::dict d;
    for (auto& kv : Profiler::Instance().Snapshot()) {
      py::dict v;
      v["count"] = kv.second.count; v["sum"] = kv.second.sum; v["min"] = kv.second.min; v["max"] = kv.second.max;
      v["last"] = kv.second.last;
      d[py::str(kv.first)] = v;
    }
    return d;
  });
  m.def("metrics_prometheus", []() { return Profiler::Instance().PrometheusText(); });
  m.def("metrics_json", []() { return Profiler::Instance().JsonLine(); });
  m.def("metrics_reset", []() { Profiler::Instance().Reset(); });
  m.def("metrics_set_attributes", [](const std::map<std::string, std::string>& a) { Profiler::Instance().SetAttributes(a); });
  m.def("metrics_start_export", [](const std::string& t, int ms) { Profiler::Instance().StartExport(t, ms); });
  m.def("metrics_stop_export", []() { py::gil_scoped_release r; Profiler::Instance().StopExport(); });
  m.def("span_start", [](const std::string& n, const std::string& tp) { return Profiler::Instance().StartSpan(n, tp); });
  m.def("span_end", [](const std::string& id, const std::map<std::string, std::string>& a) { Profiler::Instance().EndSpan(id, a); },
        py::arg("span_id"), py::arg("attributes") = std::map<std::string, std::string>());
  m.def("span_set_sink", [](const std::string& t) { Profiler::Instance().SetSpanSink(t); });
  m.def("otlp_configure", [](const std::map<std::string, std::string>& resource, int timeout_ms) {
    OtlpExporter::Instance().Configure(resource, timeout_ms);
  }, py::arg("resource"), py::arg("timeout_ms") = 1000);
  m.def("otlp_flush", [](int wait_ms) { py::gil_scoped_release r; OtlpExporter::Instance().Flush(wait_ms); },
        py::arg("wait_ms") = 2000);
  m.def("otlp_stats", []() { return std::make_pair(OtlpExporter::Instance().sent(), OtlpExporter::Instance().dropped()); });
  m.def("otlp_trace_request_json", [](const std::string& name, const std::string& trace_id, const std::string& span_id,
                                      const std::string& parent_id, int64_t start_us, int64_t end_us,
                                      const std::map<std::string, std::string>& attrs,
                                      const std::map<std::string, std::string>& resource) {
    OtlpSpan s;
    s.name = name; s.trace_id = trace_id; s.span_id = span_id; s.parent_id = parent_id;
    s.start_us = start_us; s.end_us = end_us; s.attrs = attrs;
    return OtlpTraceRequestJson({s}, resource);
  });
  m.def("spans_finished", []() { return Profiler::Instance().FinishedSpans(); });
  m.def("trace_enable", [](const std::string& p) { TraceEventRecorder::Instance().Enable(p); }, py::arg("path") = "");
  m.def("trace_disable", []() { py::gil_scoped_release r; TraceEventRecorder::Instance().Disable(); });
  m.def("trace_record", [](const std::string& n, const std::string& ph, int64_t tid, double v) {
    TraceEventRecorder::Instance().Record(n, ph, tid, v);
  }, py::arg("name"), py::arg("phase"), py::arg("tid") = 0, py::arg("value") = 0.0);
}

}  // namespace ksana
