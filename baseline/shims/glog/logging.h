// Minimal stand-in for <glog/logging.h>, enough to build the reference project when its glog
// submodule is absent: LOG(severity), VLOG(n), CHECK / CHECK_op / CHECK_NOTNULL, DCHECK_op and the
// init / shutdown entry points.  Messages go to stderr as "[I|W|E|F] file:line] text"; FATAL aborts.
#pragma once
// the real header pulls these in; sources of the reference rely on that
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <format>
#include <iomanip>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace google {
enum LogSeverity { GLOG_INFO = 0, GLOG_WARNING = 1, GLOG_ERROR = 2, GLOG_FATAL = 3 };
inline void InitGoogleLogging(const char*) {}
inline void ShutdownGoogleLogging() {}

class LogMessage {
public:
    LogMessage(const char* file, int line, int severity) : severity_(severity) {
        const char* base = file;
        for (const char* p = file; *p; ++p)
            if (*p == '/') base = p + 1;
        stream_ << "[" << "IWEF"[severity] << "] " << base << ":" << line << "] ";
    }
    ~LogMessage() noexcept(false) {
        stream_ << "\n";
        std::cerr << stream_.str();
        if (severity_ == GLOG_FATAL) {
            std::cerr.flush();
            std::abort();
        }
    }
    std::ostream& stream() { return stream_; }

private:
    std::ostringstream stream_;
    int severity_;
};

struct LogMessageVoidify {
    void operator&(std::ostream&) {}
};

inline int VerbosityFromEnv() {
    static int v = [] {
        const char* e = std::getenv("GLOG_v");
        return e ? std::atoi(e) : 0;
    }();
    return v;
}

template <typename T> T CheckNotNull(const char* file, int line, const char* names, T&& t) {
    if (t == nullptr) { LogMessage(file, line, GLOG_FATAL).stream() << names; }
    return std::forward<T>(t);
}
}  // namespace google

#define LOG(severity) ::google::LogMessage(__FILE__, __LINE__, ::google::GLOG_##severity).stream()
#define LOG_IF(severity, cond) !(cond) ? (void)0 : ::google::LogMessageVoidify() & LOG(severity)
#define VLOG(n) !(::google::VerbosityFromEnv() >= (n)) ? (void)0 : ::google::LogMessageVoidify() & LOG(INFO)
#define VLOG_IS_ON(n) (::google::VerbosityFromEnv() >= (n))

#define CHECK(cond) \
    (cond) ? (void)0 : ::google::LogMessageVoidify() & LOG(FATAL) << "Check failed: " #cond " "
#define ITB_CHECK_OP(a, b, op) \
    ((a)op(b)) ? (void)0 : ::google::LogMessageVoidify() & LOG(FATAL) << "Check failed: " #a " " #op " " #b " "
#define CHECK_EQ(a, b) ITB_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) ITB_CHECK_OP(a, b, !=)
#define CHECK_LT(a, b) ITB_CHECK_OP(a, b, <)
#define CHECK_LE(a, b) ITB_CHECK_OP(a, b, <=)
#define CHECK_GT(a, b) ITB_CHECK_OP(a, b, >)
#define CHECK_GE(a, b) ITB_CHECK_OP(a, b, >=)
#define CHECK_NOTNULL(p) ::google::CheckNotNull(__FILE__, __LINE__, "'" #p "' Must be non NULL", (p))
#define DCHECK(cond) CHECK(cond)
#define DCHECK_EQ(a, b) CHECK_EQ(a, b)
#define DCHECK_NE(a, b) CHECK_NE(a, b)
#define DCHECK_LT(a, b) CHECK_LT(a, b)
#define DCHECK_LE(a, b) CHECK_LE(a, b)
#define DCHECK_GT(a, b) CHECK_GT(a, b)
#define DCHECK_GE(a, b) CHECK_GE(a, b)
