// Log lines of the benchmark driver. The line layout
//   [HGEMM <date> <time> <pid>:<tid> <file>:<line> <function>] message
// is the reference's (src/common/logging.h:36-42); its plot tool finds the kernel name,
// TFLOPS and percentage by splitting result lines on spaces
// (tools/performance/performance.py:27-29,56-62), so the field order is kept exactly.
// Unlike the reference's static time buffer (logging.h:15-22) this formatter is re-entrant.
#pragma once

#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#define HGEMM_LOG_TAG "HGEMM"

namespace hgemm_log {

inline const char *base_name(const char *path) {
    const char *slash = strrchr(path, '/');
    return slash ? slash + 1 : path;
}

__attribute__((format(printf, 4, 5))) inline void emit(const char *file, int line, const char *func, const char *fmt,
                                                       ...) {
    char stamp[32];
    time_t now = time(nullptr);
    struct tm parts;
    localtime_r(&now, &parts);
    strftime(stamp, sizeof(stamp), "%Y-%m-%d %H:%M:%S", &parts);

    char body[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(body, sizeof(body), fmt, ap);
    va_end(ap);

    static thread_local long tid = syscall(SYS_gettid);
    fprintf(stderr, "[%s %s %d:%ld %s:%d %s] %s\n", HGEMM_LOG_TAG, stamp, static_cast<int>(getpid()), tid,
            base_name(file), line, func, body);
}

}  // namespace hgemm_log

#define HLOG(...) ::hgemm_log::emit(__FILE__, __LINE__, __FUNCTION__, __VA_ARGS__)
