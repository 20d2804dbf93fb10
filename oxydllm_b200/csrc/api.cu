// Status strings and the per-thread error message of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "oxq_common.cuh"

namespace oxq {

static thread_local char g_last_error[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_last_error[0] = '\0'; }

} // namespace oxq

OXQ_EXPORT const char *oxq_status_string(int status)
{
    switch (status) {
    case OXQ_OK: return "ok";
    case OXQ_ERR_BAD_SHAPE: return "bad shape";
    case OXQ_ERR_BAD_ALIGN: return "bad alignment";
    case OXQ_ERR_UNSUPPORTED: return "unsupported";
    case OXQ_ERR_NULL: return "null pointer";
    case OXQ_ERR_WORKSPACE: return "workspace missing or too small";
    case OXQ_ERR_CUDA: return "cuda error";
    case OXQ_ERR_DEVICE_FLAG: return "device-side bounded wait ran out";
    default: return "unknown status";
    }
}

OXQ_EXPORT const char *oxq_last_error(void) { return oxq::g_last_error; }

OXQ_EXPORT int oxq_version(void) { return 1; }
