// pybind11 surface of the native host runtime (module `_ksana_engine`).
// Blocking calls release the GIL. Counterpart of the reference binding layer
// (src/ksana_llm/torch_op/serving_op.cpp:98-245), reduced to the engine-facing objects: the
// HTTP-facing Python package builds the request/response objects on top of these.
#include "endpoint_plugin.h"
#include "stop_checker.h"
#include "waiter.h"
#include "request_packer.h"
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "batch_loop.h"
#include "cache_manager.h"
#include "common.h"
#include "control_channel.h"
#include "fsm.h"
#include "logger.h"
#include "profiler.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace ksana;

namespace {

template <typename T>
py::array_t<T> ToArray(const std::vector<T>& v) {
  py::array_t<T> a(v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

py::list EventsToList(const std::vector<SeqEvent>& ev) {
  py::list out;
  for (auto& e : ev) out.append(py::make_tuple(e.seq_id, e.req_id, e.index, e.new_token, e.finished, e.code, e.message));
  return out;
}

py::dict StatsToDict(const SchedulerStats& s) {
  py::dict d;
  d["waiting"] = s.waiting; d["running"] = s.running; d["swapped"] = s.swapped;
  d["free_blocks"] = s.free_blocks; d["used_blocks"] = s.used_blocks; d["usable_blocks"] = s.usable_blocks;
  d["free_host_blocks"] = s.free_host_blocks;
  d["total_requests"] = s.total_requests; d["finished"] = s.finished; d["timeouts"] = s.timeouts;
  d["aborted"] = s.aborted; d["rejected"] = s.rejected;
  d["preempt_swap"] = s.preempt_swap; d["preempt_recompute"] = s.preempt_recompute; d["swap_in"] = s.swap_in;
  d["steps"] = s.steps; d["step_tokens"] = s.step_tokens; d["input_tokens"] = s.input_tokens;
  d["output_tokens"] = s.output_tokens;
  d["prefix_hit_requests"] = s.cache.prefix_hit_requests; d["prefix_hit_tokens"] = s.cache.prefix_hit_tokens;
  d["prefix_hit_blocks"] = s.cache.prefix_hit_blocks; d["evicted_blocks"] = s.cache.evicted_blocks;
  d["swapped_out_blocks"] = s.cache.swapped_out_blocks; d["swapped_in_blocks"] = s.cache.swapped_in_blocks;
  d["dedup_blocks"] = s.cache.dedup_blocks; d["flexible_hit_tokens"] = s.cache.flexible_hit_tokens;
  return d;
}

}  // namespace

namespace {
// Bridges a plug-in's C callbacks to Python callables: handler(kind, bytes) -> (status, bytes); shutdown().
struct PluginBridge {
  py::object handler, shutdown;
};
void BridgeHandle(void* ctx, const char* kind, const char* data, unsigned long long len, ksana::KsanaReplyFn reply,
                  void* reply_ctx) {
  auto* b = static_cast<PluginBridge*>(ctx);
  py::gil_scoped_acquire gil;
  try {
    py::object r = b->handler(py::str(kind), py::bytes(data, static_cast<size_t>(len)));
    py::tuple t = r.cast<py::tuple>();
    std::string body = t[1].cast<std::string>();
    reply(reply_ctx, body.data(), body.size(), t[0].cast<int>());
  } catch (const std::exception& e) {
    std::string msg = e.what();
    reply(reply_ctx, msg.data(), msg.size(), 500);
  }
}
void BridgeGenerate(void* ctx, const char* d, unsigned long long n, ksana::KsanaReplyFn r, void* rc) {
  BridgeHandle(ctx, "generate", d, n, r, rc);
}
void BridgeForward(void* ctx, const char* d, unsigned long long n, ksana::KsanaReplyFn r, void* rc) {
  BridgeHandle(ctx, "forward", d, n, r, rc);
}
void BridgeShutdown(void* ctx) {
  auto* b = static_cast<PluginBridge*>(ctx);
  py::gil_scoped_acquire gil;
  if (!b->shutdown.is_none()) b->shutdown();
}
struct PyEndpointPlugin {
  PyEndpointPlugin(const std::string& name, const std::string& dir) : plugin(name, dir) {}
  ksana::EndpointPlugin plugin;
  PluginBridge bridge;
};
}  // namespace

PYBIND11_MODULE(_ksana_engine, m) {
  m.doc() = "native host runtime: scheduler, KV cache manager, structured-output FSM, profiler, control plane";

  ksana::BindRequestPacker(m);
  ksana::BindStopChecker(m);

  // process-wide logger (KLLM_LOG_LEVEL / KLLM_LOG_FILE); the Python side writes through the same sink
  m.def("log_message", [](int level, const std::string& file, int line, const std::string& text) {
    ksana::Logger::Get().Write(level, file.c_str(), line, text);
  });
  m.def("log_enabled", [](int level) { return ksana::Logger::Get().Enabled(level); });
  m.def("log_level", []() { return ksana::Logger::Get().level(); });
  m.def("set_log_level", [](const std::string& name) {
    auto& lg = ksana::Logger::Get();
    lg.SetLevel(ksana::Logger::ParseLevel(name, lg.level()));
  });
  m.def("set_log_file", [](const std::string& path) { ksana::Logger::Get().SetFile(path); });
  m.def("log_file", []() { return ksana::Logger::Get().file(); });

  py::class_<PyEndpointPlugin>(m, "EndpointPlugin")
      .def(py::init<const std::string&, const std::string&>(), py::arg("name"), py::arg("search_dir") = "")
      .def_property_readonly("symbol", [](const PyEndpointPlugin& p) { return p.plugin.symbol(); })
      .def_property_readonly("path", [](const PyEndpointPlugin& p) { return p.plugin.path(); })
      .def("start", [](PyEndpointPlugin& p, py::object handler, py::object shutdown, const std::string& host, int port) {
        p.bridge.handler = handler;
        p.bridge.shutdown = shutdown;
        ksana::KsanaEndpointApi api{&p.bridge, BridgeGenerate, BridgeForward, BridgeShutdown};
        py::gil_scoped_release rel;
        return p.plugin.Start(api, host, port);
      }, py::arg("handler"), py::arg("shutdown") = py::none(), py::arg("host") = "0.0.0.0", py::arg("port") = 8080)
      .def("stop", [](PyEndpointPlugin& p) {
        py::gil_scoped_release rel;
        return p.plugin.Stop();
      });

  py::enum_<RetCode>(m, "RetCode")
      .value("RET_SUCCESS", RET_SUCCESS).value("RET_INVALID_ARGUMENT", RET_INVALID_ARGUMENT)
      .value("RET_SEGMENT_FAULT", RET_SEGMENT_FAULT).value("RET_OUT_OF_MEMORY", RET_OUT_OF_MEMORY)
      .value("RET_TERMINATED", RET_TERMINATED).value("RET_EXCEED_CAPACITY", RET_EXCEED_CAPACITY)
      .value("RET_EXCEED_LENGTH", RET_EXCEED_LENGTH).value("RET_TIMEOUT", RET_TIMEOUT)
      .value("RET_ALLOCATE_FAIL", RET_ALLOCATE_FAIL).value("RET_FREE_FAIL", RET_FREE_FAIL)
      .value("RET_UNDEFINED_REFERENCE", RET_UNDEFINED_REFERENCE).value("RET_STOP_ITERATION", RET_STOP_ITERATION)
      .value("RET_RUNTIME", RET_RUNTIME).value("RET_UNKNOWN", RET_UNKNOWN)
      .export_values();

  py::class_<SamplingConfig>(m, "SamplingConfig")
      .def(py::init<>())
      .def_readwrite("topk", &SamplingConfig::topk)
      .def_readwrite("num_beams", &SamplingConfig::num_beams)
      .def_readwrite("num_return_sequences", &SamplingConfig::num_return_sequences)
      .def_readwrite("topp", &SamplingConfig::topp)
      .def_readwrite("temperature", &SamplingConfig::temperature)
      .def_readwrite("repetition_penalty", &SamplingConfig::repetition_penalty)
      .def_readwrite("length_penalty", &SamplingConfig::length_penalty)
      .def_readwrite("no_repeat_ngram_size", &SamplingConfig::no_repeat_ngram_size)
      .def_readwrite("encoder_no_repeat_ngram_size", &SamplingConfig::encoder_no_repeat_ngram_size)
      .def_readwrite("max_new_tokens", &SamplingConfig::max_new_tokens)
      .def_readwrite("logprobs_num", &SamplingConfig::logprobs_num)
      .def_readwrite("stop_token_ids", &SamplingConfig::stop_token_ids)
      .def_readwrite("stop_strings", &SamplingConfig::stop_strings)
      .def_readwrite("ignore_eos", &SamplingConfig::ignore_eos)
      .def_readwrite("seed", &SamplingConfig::seed)
      .def("verify_args", [](SamplingConfig& c) {
        Status s = c.VerifyArgs();
        return py::make_tuple(static_cast<int>(s.code), s.message);
      });

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("schedule_strategy", &SchedulerConfig::schedule_strategy)
      .def_readwrite("dp_size", &SchedulerConfig::dp_size)
      .def_readwrite("waiting_timeout_in_ms", &SchedulerConfig::waiting_timeout_in_ms)
      .def_readwrite("max_waiting_queue_len", &SchedulerConfig::max_waiting_queue_len)
      .def_readwrite("max_step_tokens", &SchedulerConfig::max_step_tokens)
      .def_readwrite("max_batch_size", &SchedulerConfig::max_batch_size)
      .def_readwrite("max_token_len", &SchedulerConfig::max_token_len)
      .def_readwrite("swapout_block_threshold", &SchedulerConfig::swapout_block_threshold)
      .def_readwrite("swapin_block_threshold", &SchedulerConfig::swapin_block_threshold)
      .def_readwrite("launch_block_threshold", &SchedulerConfig::launch_block_threshold)
      .def_readwrite("preempt_mode", &SchedulerConfig::preempt_mode)
      .def_readwrite("split_fuse_token_num", &SchedulerConfig::split_fuse_token_num)
      .def_readwrite("min_flexible_cache_num", &SchedulerConfig::min_flexible_cache_num)
      .def_readwrite("enable_prefix_cache", &SchedulerConfig::enable_prefix_cache)
      .def_readwrite("block_token_num", &SchedulerConfig::block_token_num)
      .def_readwrite("auto_batch_wait_ms", &SchedulerConfig::auto_batch_wait_ms)
      .def_readwrite("eos_token_ids", &SchedulerConfig::eos_token_ids);

  py::class_<StepPlan>(m, "StepPlan")
      .def(py::init<>())
      .def_property_readonly("seq_ids", [](const StepPlan& p) { return ToArray(p.seq_ids); })
      .def_property_readonly("q_lens", [](const StepPlan& p) { return ToArray(p.q_lens); })
      .def_property_readonly("kv_lens", [](const StepPlan& p) { return ToArray(p.kv_lens); })
      .def_property_readonly("input_ids", [](const StepPlan& p) { return ToArray(p.input_ids); })
      .def_property_readonly("positions", [](const StepPlan& p) { return ToArray(p.positions); })
      .def_property_readonly("slots", [](const StepPlan& p) { return ToArray(p.slots); })
      .def_property_readonly("cu_q", [](const StepPlan& p) { return ToArray(p.cu_q); })
      .def_property_readonly("block_table", [](const StepPlan& p) { return ToArray(p.block_table); })
      .def_property_readonly("sample_seq_ids", [](const StepPlan& p) { return ToArray(p.sample_seq_ids); })
      .def_property_readonly("sample_rows", [](const StepPlan& p) { return ToArray(p.sample_rows); })
      .def_property_readonly("swap_out", [](const StepPlan& p) {
        std::vector<int> v; for (auto& s : p.swap_out) { v.push_back(s.device_block); v.push_back(s.host_block); }
        return ToArray(v); })
      .def_property_readonly("swap_in", [](const StepPlan& p) {
        std::vector<int> v; for (auto& s : p.swap_in) { v.push_back(s.device_block); v.push_back(s.host_block); }
        return ToArray(v); })
      .def_property_readonly("copies", [](const StepPlan& p) {
        std::vector<int> v; for (auto& c : p.copies) { v.push_back(c.src); v.push_back(c.dst); v.push_back(c.pos_delta); }
        return ToArray(v); })
      .def_property_readonly("pre_copies", [](const StepPlan& p) {
        std::vector<int> v; for (auto& c : p.pre_copies) { v.push_back(c.src); v.push_back(c.dst); v.push_back(c.pos_delta); }
        return ToArray(v); })
      .def("has_block_ops", &StepPlan::has_block_ops)
      .def_property_readonly("events", [](const StepPlan& p) { return EventsToList(p.events); })
      .def_readonly("max_blocks", &StepPlan::max_blocks)
      .def_readonly("num_multi", &StepPlan::num_multi)
      .def_readonly("num_single", &StepPlan::num_single)
      .def_readonly("num_tokens", &StepPlan::num_tokens)
      .def_readonly("num_multi_tokens", &StepPlan::num_multi_tokens)
      .def_readonly("max_q_len", &StepPlan::max_q_len)
      .def_readonly("sample_k", &StepPlan::sample_k)
      .def_readwrite("sample_full", &StepPlan::sample_full)
      .def("empty", &StepPlan::empty)
      .def("pack", [](const StepPlan& p) { return ToArray(p.Pack()); })
      .def("step_image_words", &StepPlan::StepImageWords)
      .def("write_step_image", [](const StepPlan& p, uintptr_t dst, size_t capacity_words) {
        if (capacity_words < p.StepImageWords()) throw std::runtime_error("step image does not fit its buffer");
        return p.WriteStepImage(reinterpret_cast<int32_t*>(dst));
      })
      .def("write_decode_image", [](const StepPlan& p, uintptr_t dst, size_t capacity_words, int bs, int mb) {
        if (capacity_words < static_cast<size_t>(4) * bs + static_cast<size_t>(bs) * mb)
          throw std::runtime_error("decode image does not fit its buffer");
        return p.WriteDecodeImage(reinterpret_cast<int32_t*>(dst), bs, mb);
      })
      .def_property_readonly("num_seqs", [](const StepPlan& p) { return p.seq_ids.size(); })
      .def_property_readonly("num_samples", [](const StepPlan& p) { return p.sample_rows.size(); })
      .def_property_readonly("max_kv_len", [](const StepPlan& p) {
        int m = 0; for (int v : p.kv_lens) m = std::max(m, v); return m; })
      .def_property_readonly("max_single_kv_len", [](const StepPlan& p) {
        int m = 0; for (size_t i = p.num_multi; i < p.kv_lens.size(); ++i) m = std::max(m, p.kv_lens[i]); return m; })
      .def_static("unpack", [](py::array_t<int32_t, py::array::c_style | py::array::forcecast> a) {
        StepPlan p;
        if (!StepPlan::Unpack(a.data(), static_cast<size_t>(a.size()), &p)) throw std::runtime_error("bad step plan image");
        return p;
      });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerConfig&, int, int>(), py::arg("config"), py::arg("num_device_blocks"),
           py::arg("num_host_blocks"))
      .def("add_request", [](Scheduler& s, int64_t req_id, const std::vector<int>& prompt, const SamplingConfig& cfg) {
        std::vector<int64_t> ids;
        Status st = s.AddRequest(req_id, prompt, cfg, &ids);
        return py::make_tuple(static_cast<int>(st.code), st.message, ids);
      })
      .def("abort", &Scheduler::Abort)
      .def("idle", &Scheduler::Idle)
      .def("schedule", [](Scheduler& s) {
        StepPlan p;
        {
          py::gil_scoped_release rel;
          s.Schedule(&p);
        }
        return p;
      })
      .def("post_step", [](Scheduler& s, const StepPlan& plan, const std::vector<int>& tokens,
                           const std::vector<int64_t>& parents) {
        std::vector<SampledToken> st(tokens.size());
        for (size_t i = 0; i < tokens.size(); ++i) {
          st[i].token = tokens[i];
          st[i].parent_seq = i < parents.size() ? parents[i] : -1;
        }
        std::vector<SeqEvent> ev;
        {
          py::gil_scoped_release rel;
          s.PostStep(plan, st, &ev);
        }
        return EventsToList(ev);
      }, py::arg("plan"), py::arg("tokens"), py::arg("parents") = std::vector<int64_t>())
      .def("can_pipeline", &Scheduler::CanPipeline)
      .def("advance", [](Scheduler& s, const StepPlan& plan) {
        py::gil_scoped_release rel;
        s.Advance(plan);
      })
      .def("resolve", [](Scheduler& s, const StepPlan& plan, const std::vector<int>& tokens) {
        std::vector<SeqEvent> ev;
        {
          py::gil_scoped_release rel;
          s.Resolve(plan, tokens, &ev);
        }
        return EventsToList(ev);
      })
      .def("finish_sequence", [](Scheduler& s, int64_t seq_id, int keep, int code, const std::string& msg) {
        std::vector<SeqEvent> ev;
        s.FinishSequence(seq_id, keep, code, msg, &ev);
        return EventsToList(ev);
      })
      .def("replace_generated", &Scheduler::ReplaceGenerated)
      .def("get_tokens", &Scheduler::GetTokens)
      .def("get_prompt_len", &Scheduler::GetPromptLen)
      .def("stats", [](Scheduler& s) { return StatsToDict(s.GetStats()); })
      .def("check_invariants", [](Scheduler& s) {
        std::string why;
        const bool ok = s.CheckInvariants(&why);
        return py::make_tuple(ok, why);
      });

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<int, int, int, bool>())
      .def_property_readonly("free_blocks", &CacheManager::free_blocks)
      .def_property_readonly("usable_blocks", &CacheManager::usable_blocks)
      .def_property_readonly("evictable_blocks", &CacheManager::evictable_blocks)
      .def_property_readonly("free_host_blocks", &CacheManager::free_host_blocks)
      .def("ref_count", &CacheManager::ref_count)
      .def("in_tree", &CacheManager::in_tree)
      .def("acquire_prefix", [](CacheManager& c, const std::vector<int>& tokens) {
        std::vector<int> b;
        const int n = c.AcquirePrefix(tokens, &b);
        return py::make_tuple(n, b);
      })
      .def("allocate", [](CacheManager& c, int n) {
        std::vector<int> b;
        const bool ok = c.Allocate(n, &b);
        return py::make_tuple(ok, b);
      })
      .def("release", &CacheManager::Release)
      .def("promote", [](CacheManager& c, const std::vector<int>& tokens, std::vector<int> blocks, int computed, int first) {
        const int p = c.Promote(tokens, &blocks, computed, first);
        return py::make_tuple(p, blocks);
      })
      .def("fork", [](CacheManager& c, const std::vector<int>& src, int cached) {
        std::vector<int> dst; std::vector<BlockCopy> cp;
        const bool ok = c.Fork(src, cached, &dst, &cp);
        std::vector<std::pair<int, int>> pairs;
        for (auto& x : cp) pairs.emplace_back(x.src, x.dst);
        return py::make_tuple(ok, dst, pairs);
      })
      .def("swap_out", [](CacheManager& c, std::vector<int> blocks) {
        std::vector<int> host; std::vector<SwapCopy> cp;
        const bool ok = c.SwapOut(&blocks, &host, &cp);
        std::vector<std::pair<int, int>> pairs;
        for (auto& x : cp) pairs.emplace_back(x.device_block, x.host_block);
        return py::make_tuple(ok, blocks, host, pairs);
      })
      .def("swap_in", [](CacheManager& c, std::vector<int> blocks, std::vector<int> host) {
        std::vector<SwapCopy> cp;
        const bool ok = c.SwapIn(&blocks, &host, &cp);
        std::vector<std::pair<int, int>> pairs;
        for (auto& x : cp) pairs.emplace_back(x.device_block, x.host_block);
        return py::make_tuple(ok, blocks, pairs);
      })
      .def("acquire_flexible", [](CacheManager& c, const std::vector<int>& tokens, int prefix, int min_tokens) {
        std::vector<int> b; std::vector<BlockCopy> cp;
        const int n = c.AcquireFlexible(tokens, prefix, min_tokens, &b, &cp);
        std::vector<std::tuple<int, int, int>> t;
        for (auto& x : cp) t.emplace_back(x.src, x.dst, x.pos_delta);
        return py::make_tuple(n, b, t);
      })
      .def("check_invariants", [](CacheManager& c) {
        std::string why;
        const bool ok = c.CheckInvariants(&why);
        return py::make_tuple(ok, why);
      });

  {
    // python callables for the native loop thread: entered with the interpreter lock, released with it, and an
    // exception that escapes one becomes a plain C++ exception carrying its text
    auto hold = [](py::function f) {
      return std::shared_ptr<py::function>(new py::function(std::move(f)), [](py::function* p) {
        py::gil_scoped_acquire g;
        delete p;
      });
    };
    py::class_<BatchLoop>(m, "BatchLoop")
        .def(py::init<>())
        .def("start", [hold](BatchLoop& self, py::function step, py::function idle, py::function on_error) {
          auto s = hold(std::move(step)), i = hold(std::move(idle)), e = hold(std::move(on_error));
          auto call_bool = [](const std::shared_ptr<py::function>& f) {
            py::gil_scoped_acquire g;
            try {
              return (*f)().cast<bool>();
            } catch (py::error_already_set& err) {
              const std::string msg = err.what();
              throw std::runtime_error(msg);
            }
          };
          py::gil_scoped_release rel;        // Start() may join a previous thread that needs the lock
          self.Start([s, call_bool]() { return call_bool(s); }, [i, call_bool]() { return call_bool(i); },
                     [e](const std::string& msg) {
                       py::gil_scoped_acquire g;
                       try {
                         (*e)(msg);
                       } catch (py::error_already_set& err) {
                         throw std::runtime_error(std::string(err.what()));
                       }
                     });
        }, py::arg("step"), py::arg("idle"), py::arg("on_error"))
        .def("notify", &BatchLoop::Notify)
        .def("stop", [](BatchLoop& self) { py::gil_scoped_release rel; self.Stop(); })
        .def_property_readonly("running", &BatchLoop::running)
        .def_property_readonly("steps", &BatchLoop::steps)
        .def_property_readonly("sleeps", &BatchLoop::sleeps);
  }
  {
    // same surface as threading.Event / queue.Queue (set, is_set, wait(timeout seconds) / put, get(timeout seconds)
    // raising queue.Empty), so the request objects use them in place of the interpreter's own primitives
    py::class_<Waiter>(m, "Waiter")
        .def(py::init<>())
        .def("set", &Waiter::Set)
        .def("clear", &Waiter::Clear)
        .def("is_set", &Waiter::IsSet)
        .def("wait", [](Waiter& self, py::object timeout) {
          const long long ms = timeout.is_none() ? -1 : static_cast<long long>(timeout.cast<double>() * 1000.0);
          py::gil_scoped_release rel;
          return self.Wait(ms);
        }, py::arg("timeout") = py::none());
    using Channel = StreamChannel<std::shared_ptr<py::object>>;
    py::class_<Channel>(m, "StreamChannel")
        .def(py::init<>())
        .def("put", [](Channel& self, py::object item) {
          // the handle dies with the interpreter lock held wherever the last reference goes away
          self.Put(std::shared_ptr<py::object>(new py::object(std::move(item)), [](py::object* p) {
            py::gil_scoped_acquire g;
            delete p;
          }));
        })
        .def("get", [](Channel& self, py::object timeout) -> py::object {
          const long long ms = timeout.is_none() ? -1 : static_cast<long long>(timeout.cast<double>() * 1000.0);
          std::shared_ptr<py::object> item;
          bool ok;
          {
            py::gil_scoped_release rel;
            ok = self.Get(&item, ms);
          }
          if (!ok) {
            PyErr_SetNone(py::module_::import("queue").attr("Empty").ptr());
            throw py::error_already_set();
          }
          return *item;
        }, py::arg("timeout") = py::none())
        .def("qsize", &Channel::Size)
        .def("empty", [](Channel& self) { return self.Size() == 0; });
  }
  BindFsm(m);
  BindProfiler(m);
  BindControlChannel(m);
}
