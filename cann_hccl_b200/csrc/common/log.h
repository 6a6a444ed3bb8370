// Minimal levelled logger (HCCL_LOG_LEVEL = 0 debug, 1 info, 2 warning, 3 error; default 2).
// Mirrors the role of HCCL_DEBUG/INFO/WARNING/ERROR/RUN_INFO in the reference's closed log.h.
#pragma once
#include <string>
namespace hcclb {
enum LogLevel { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3, LOG_RUN = 4 };
int log_level();
void log_set_level(int lvl);
void log_write(int lvl, const char *file, int line, const char *fmt, ...) __attribute__((format(printf, 4, 5)));
const std::string &last_error_message();  // text of the newest LOG_ERROR on this thread
}  // namespace hcclb
#define HLOG(lvl, ...)                                                        \
    do {                                                                      \
        if ((lvl) >= ::hcclb::log_level()) ::hcclb::log_write((lvl), __FILE__, __LINE__, __VA_ARGS__); \
    } while (0)
#define HLOG_DEBUG(...) HLOG(::hcclb::LOG_DEBUG, __VA_ARGS__)
#define HLOG_INFO(...) HLOG(::hcclb::LOG_INFO, __VA_ARGS__)
#define HLOG_WARN(...) HLOG(::hcclb::LOG_WARN, __VA_ARGS__)
#define HLOG_ERROR(...) HLOG(::hcclb::LOG_ERROR, __VA_ARGS__)
#define HLOG_RUN(...) HLOG(::hcclb::LOG_RUN, __VA_ARGS__)
// Return `ret` from the current function when `cond` holds, after logging.
#define CHK_RET_LOG(cond, ret, ...)      \
    do {                                 \
        if (cond) {                      \
            HLOG_ERROR(__VA_ARGS__);     \
            return (ret);                \
        }                                \
    } while (0)
#define CHK_RET(expr)                               \
    do {                                            \
        HcclResult _r = (expr);                     \
        if (_r != HCCL_SUCCESS) return _r;          \
    } while (0)
