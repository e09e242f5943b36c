// Leveled logging for the host runtime: PSB_LOG(INFO) << "restored storage " << sid;
//
// The level comes from $PSB_LOG_LEVEL (DEBUG, INFO, WARNING, ERROR, OFF; default WARNING, so a quiet process stays
// quiet) or set_log_level(); lines go to stderr as "<L> <time> <thread> <file>:<line>] message", or to a sink that
// the embedding program installs (the Python binding hands them to the `logging` module). The role of the
// reference's SLOG / BLOG / LOG macros (glog through prpc, pico-ps/common/core.h:43-222).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>

namespace psb {

enum class LogLevel : int { DEBUG = 0, INFO = 1, WARNING = 2, ERROR = 3, OFF = 4 };

namespace log_detail {
inline LogLevel parse(const char* s, LogLevel dflt) {
    if (!s || !*s) return dflt;
    switch (s[0]) {
        case 'D': case 'd': return LogLevel::DEBUG;
        case 'I': case 'i': return LogLevel::INFO;
        case 'W': case 'w': return LogLevel::WARNING;
        case 'E': case 'e': return LogLevel::ERROR;
        case 'O': case 'o': return LogLevel::OFF;
        default: return dflt;
    }
}
inline std::atomic<int>& level() {
    static std::atomic<int> l{(int)parse(std::getenv("PSB_LOG_LEVEL"), LogLevel::WARNING)};
    return l;
}
using Sink = std::function<void(LogLevel, const std::string&)>;
inline std::mutex& sink_mu() {
    static std::mutex m;
    return m;
}
inline std::shared_ptr<Sink>& sink() {
    static std::shared_ptr<Sink> s;
    return s;
}
}  // namespace log_detail

inline void set_log_level(LogLevel l) { log_detail::level() = (int)l; }
inline LogLevel log_level() { return (LogLevel)log_detail::level().load(); }
inline bool log_enabled(LogLevel l) { return (int)l >= log_detail::level().load(std::memory_order_relaxed); }
// Replaces stderr as the destination (nullptr puts stderr back). The sink may be called from any thread.
inline void set_log_sink(log_detail::Sink s) {
    std::lock_guard<std::mutex> g(log_detail::sink_mu());
    log_detail::sink() = s ? std::make_shared<log_detail::Sink>(std::move(s)) : nullptr;
}

class LogLine {
public:
    LogLine(LogLevel l, const char* file, int line) : level_(l) {
        const char* base = std::strrchr(file, '/');
        where_ = std::string(base ? base + 1 : file) + ":" + std::to_string(line);
    }
    ~LogLine() {
        std::shared_ptr<log_detail::Sink> s;
        {
            std::lock_guard<std::mutex> g(log_detail::sink_mu());
            s = log_detail::sink();
        }
        const std::string msg = where_ + "] " + os_.str();
        if (s) {
            (*s)(level_, msg);
            return;
        }
        const auto now = std::chrono::system_clock::now();
        const std::time_t t = std::chrono::system_clock::to_time_t(now);
        const int ms = (int)(std::chrono::duration_cast<std::chrono::milliseconds>(now.time_since_epoch()).count() % 1000);
        std::tm tm_buf;
        localtime_r(&t, &tm_buf);
        char stamp[32];
        std::strftime(stamp, sizeof stamp, "%m%d %H:%M:%S", &tm_buf);
        std::ostringstream tid;
        tid << std::this_thread::get_id();
        std::fprintf(stderr, "%c%s.%03d %s %s\n", "DIWE"[(int)level_], stamp, ms, tid.str().c_str(), msg.c_str());
    }
    template <class T>
    LogLine& operator<<(const T& v) {
        os_ << v;
        return *this;
    }

private:
    LogLevel level_;
    std::string where_;
    std::ostringstream os_;
};

}  // namespace psb

// The message expression is not evaluated when the level is off.
#define PSB_LOG(severity)                                      \
    if (!::psb::log_enabled(::psb::LogLevel::severity)) {      \
    } else                                                     \
        ::psb::LogLine(::psb::LogLevel::severity, __FILE__, __LINE__)
