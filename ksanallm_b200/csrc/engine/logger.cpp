#include "logger.h"

#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>

namespace ksana {

struct Logger::Sink {
  std::mutex mu;
  FILE* fp = nullptr;       // nullptr: standard error
  std::string path;
};

namespace {

void MakeParentDirs(const std::string& path) {
  for (size_t i = 1; i < path.size(); ++i) {
    if (path[i] == '/') {
      const std::string dir = path.substr(0, i);
      ::mkdir(dir.c_str(), 0755);          // an existing directory is fine
    }
  }
}

const char* Basename(const char* path) {
  const char* slash = std::strrchr(path, '/');
  return slash ? slash + 1 : path;
}

}  // namespace

int Logger::ParseLevel(const std::string& name, int fallback) {
  static const char* names[] = {"DEBUG", "INFO", "WARNING", "ERROR", "FATAL"};
  for (int i = 0; i < 5; ++i)
    if (name == names[i]) return i;
  return fallback;
}

const char* Logger::LevelName(int level) {
  static const char* names[] = {"DEBUG", "INFO", "WARNING", "ERROR", "FATAL"};
  return (level >= 0 && level < 5) ? names[level] : "?";
}

Logger::Logger() : level_(LOG_INFO), sink_(new Sink()) {
  if (const char* lv = std::getenv("KLLM_LOG_LEVEL")) level_.store(ParseLevel(lv, LOG_INFO));
  const char* f = std::getenv("KLLM_LOG_FILE");
  SetFile(f ? f : "log/ksana_llm.log");
}

Logger& Logger::Get() {
  static Logger* inst = new Logger();     // never destroyed: records may be written during process teardown
  return *inst;
}

void Logger::SetFile(const std::string& path) {
  if (path.empty()) return;
  std::lock_guard<std::mutex> g(sink_->mu);
  if (sink_->fp) { std::fclose(sink_->fp); sink_->fp = nullptr; }
  sink_->path = path;
  if (path == "stderr" || path == "-") return;
  MakeParentDirs(path);
  sink_->fp = std::fopen(path.c_str(), "a");
  if (!sink_->fp) sink_->path = "stderr";   // an unwritable target must not take the service down
}

std::string Logger::file() const {
  std::lock_guard<std::mutex> g(sink_->mu);
  return sink_->path;
}

void Logger::Write(int level, const char* file, int line, const std::string& text) {
  if (!Enabled(level)) return;
  using namespace std::chrono;
  const auto now = system_clock::now();
  const std::time_t secs = system_clock::to_time_t(now);
  const int ms = static_cast<int>(duration_cast<milliseconds>(now.time_since_epoch()).count() % 1000);
  std::tm tm_buf;
  localtime_r(&secs, &tm_buf);
  char head[96];
  const size_t n = std::strftime(head, sizeof(head), "%Y-%m-%d %H:%M:%S", &tm_buf);
  std::snprintf(head + n, sizeof(head) - n, ".%03d %-7s %ld", ms, LevelName(level), static_cast<long>(::syscall(SYS_gettid)));
  std::lock_guard<std::mutex> g(sink_->mu);
  FILE* out = sink_->fp ? sink_->fp : stderr;
  std::fprintf(out, "%s %s:%d] %s\n", head, Basename(file), line, text.c_str());
  if (level >= LOG_WARNING || !sink_->fp) std::fflush(out);
  if (level >= LOG_FATAL && sink_->fp) {
    std::fflush(out);
    std::fprintf(stderr, "%s %s:%d] %s\n", head, Basename(file), line, text.c_str());
  }
}

}  // namespace ksana
