// Status strings and the thread-local "last error" buffer of the C ABI.
#include "common.cuh"

#include <cstring>

namespace i8tk {
namespace {
thread_local char g_last_error[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}
}  // namespace i8tk

extern "C" const char* i8tk_status_string(int status) {
    switch (status) {
        case I8TK_OK: return "ok";
        case I8TK_ERR_INVALID_ARGUMENT: return "invalid argument";
        case I8TK_ERR_UNSUPPORTED: return "unsupported shape or option";
        case I8TK_ERR_WORKSPACE: return "workspace missing or too small";
        case I8TK_ERR_ALIGNMENT: return "misaligned pointer";
        case I8TK_ERR_CUDA: return "CUDA call failed";
        case I8TK_ERR_DEVICE_TIMEOUT: return "bounded device-side wait gave up";
        default: return "unknown status";
    }
}

extern "C" const char* i8tk_last_error(void) { return i8tk::g_last_error; }

extern "C" int i8tk_version(void) { return 100; }
