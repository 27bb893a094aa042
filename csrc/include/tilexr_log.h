// Minimal stream-style logger: TILEXR_LOG(INFO) << "text" << value;
// Level from TILEXR_LOG_LEVEL (DEBUG/INFO/WARN/ERROR/FATAL or 0..4), default WARN.
// One line per statement, written under a mutex; ERROR and above go to stderr.
// (Reference: src/comm/tilexr_log.h:33-233; the spdlog backend is not reproduced.)
#ifndef TILEXR_LOG_H
#define TILEXR_LOG_H

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>
#include <strings.h>

namespace TileXR {

enum LogLevel { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3, LOG_FATAL = 4 };

inline int ParseLogLevel(const char *text, int fallback)
{
    if (text == nullptr || *text == '\0') return fallback;
    static const char *names[] = {"DEBUG", "INFO", "WARN", "ERROR", "FATAL"};
    for (int i = 0; i < 5; ++i) {
        if (strcasecmp(text, names[i]) == 0) return i;
    }
    if (text[0] >= '0' && text[0] <= '4' && text[1] == '\0') return text[0] - '0';
    return fallback;
}

inline int CurrentLogLevel()
{
    static int level = [] {
        const char *env = std::getenv("TILEXR_LOG_LEVEL");
        if (env == nullptr) env = std::getenv("ASDOPS_LOG_LEVEL");
        return ParseLogLevel(env, LOG_WARN);
    }();
    return level;
}

inline std::mutex &LogMutex()
{
    static std::mutex m;
    return m;
}

class LogLine {
public:
    LogLine(int level, const char *file, int line) : level_(level)
    {
        static const char *tags[] = {"DEBUG", "INFO", "WARN", "ERROR", "FATAL"};
        const char *base = std::strrchr(file, '/');
        os_ << "[TileXR " << tags[level] << " " << (base ? base + 1 : file) << ":" << line << "] ";
    }
    ~LogLine()
    {
        os_ << '\n';
        std::lock_guard<std::mutex> lock(LogMutex());
        std::fputs(os_.str().c_str(), level_ >= LOG_ERROR ? stderr : stdout);
        std::fflush(level_ >= LOG_ERROR ? stderr : stdout);
    }
    template <typename T>
    LogLine &operator<<(const T &v)
    {
        os_ << v;
        return *this;
    }

private:
    int level_;
    std::ostringstream os_;
};

struct LogVoidify {
    void operator&(const LogLine &) {}
};

} // namespace TileXR

#define TILEXR_LOG(LEVEL)                                                   \
    (TileXR::LOG_##LEVEL < TileXR::CurrentLogLevel()) ? (void)0             \
        : TileXR::LogVoidify() & TileXR::LogLine(TileXR::LOG_##LEVEL, __FILE__, __LINE__)

#endif // TILEXR_LOG_H
