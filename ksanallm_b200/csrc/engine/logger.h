// Process-wide logger of the host runtime.
//
// Same knobs as the reference logger (src/ksana_llm/utils/logger.h:15-40): the level comes from KLLM_LOG_LEVEL
// (DEBUG / INFO / WARNING / ERROR / FATAL, default INFO), the sink from KLLM_LOG_FILE (default log/ksana_llm.log,
// opened in append mode, directories created on demand), and call sites use stream-style macros:
//
//   KLLM_LOG_INFO << "scheduled " << n << " sequences";
//
// A record is "<date time.ms> <LEVEL> <thread id> <file>:<line>] <text>". Records below the level cost one relaxed
// atomic load and build nothing. KLLM_LOG_FILE=stderr (or "-") writes to standard error instead; FATAL records also
// go to standard error. The Python side logs through the same sink (see bindings: log_message / set_log_level).
#pragma once
#include <atomic>
#include <sstream>
#include <string>

namespace ksana {

enum LogLevel : int { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARNING = 2, LOG_ERROR = 3, LOG_FATAL = 4 };

class Logger {
 public:
  static Logger& Get();
  bool Enabled(int level) const { return level >= level_.load(std::memory_order_relaxed); }
  int level() const { return level_.load(std::memory_order_relaxed); }
  void SetLevel(int level) { level_.store(level, std::memory_order_relaxed); }
  // Re-opens the sink (tests, log rotation). "" keeps the current target; "stderr" / "-" selects standard error.
  void SetFile(const std::string& path);
  std::string file() const;
  void Write(int level, const char* file, int line, const std::string& text);
  static int ParseLevel(const std::string& name, int fallback);
  static const char* LevelName(int level);

 private:
  Logger();
  std::atomic<int> level_;
  struct Sink;
  Sink* sink_;
};

// One record: collects the streamed pieces and hands them to the logger when it goes out of scope.
class LogRecord {
 public:
  LogRecord(int level, const char* file, int line) : level_(level), file_(file), line_(line) {}
  ~LogRecord() { Logger::Get().Write(level_, file_, line_, os_.str()); }
  std::ostringstream& stream() { return os_; }

 private:
  int level_;
  const char* file_;
  int line_;
  std::ostringstream os_;
};

}  // namespace ksana

#define KLLM_LOG_AT(level) \
  if (!::ksana::Logger::Get().Enabled(level)) {} else ::ksana::LogRecord(level, __FILE__, __LINE__).stream()
#define KLLM_LOG_DEBUG KLLM_LOG_AT(::ksana::LOG_DEBUG)
#define KLLM_LOG_INFO KLLM_LOG_AT(::ksana::LOG_INFO)
#define KLLM_LOG_WARNING KLLM_LOG_AT(::ksana::LOG_WARNING)
#define KLLM_LOG_ERROR KLLM_LOG_AT(::ksana::LOG_ERROR)
#define KLLM_LOG_FATAL KLLM_LOG_AT(::ksana::LOG_FATAL)
