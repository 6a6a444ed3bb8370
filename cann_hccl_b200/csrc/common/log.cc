#include "common/log.h"
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <sys/time.h>
#include <unistd.h>

namespace hcclb {
static std::atomic<int> g_level{-1};
static thread_local std::string t_last_error;

int log_level()
{
    int l = g_level.load(std::memory_order_relaxed);
    if (l < 0) {
        const char *e = getenv("HCCL_LOG_LEVEL");
        l = e ? atoi(e) : LOG_WARN;
        if (l < 0) l = 0;
        if (l > LOG_ERROR) l = LOG_ERROR;
        g_level.store(l);
    }
    return l;
}
void log_set_level(int lvl) { g_level.store(lvl); }
const std::string &last_error_message() { return t_last_error; }

void log_write(int lvl, const char *file, int line, const char *fmt, ...)
{
    static const char *names[] = {"DEBUG", "INFO", "WARN", "ERROR", "RUN"};
    char msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    if (lvl == LOG_ERROR) t_last_error = msg;
    const char *base = strrchr(file, '/');
    base = base ? base + 1 : file;
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    struct tm tmv;
    localtime_r(&tv.tv_sec, &tmv);
    fprintf(stderr, "[HCCL-B200][%s][%02d:%02d:%02d.%03d][pid %d][%s:%d] %s\n", names[lvl > 4 ? 4 : lvl],
            tmv.tm_hour, tmv.tm_min, tmv.tm_sec, (int)(tv.tv_usec / 1000), (int)getpid(), base, line, msg);
}
}  // namespace hcclb
