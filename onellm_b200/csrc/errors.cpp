// Thread-local error text behind onellm_last_error().
#include <stdarg.h>
#include <stdio.h>

#include "onellm_b200.h"

namespace onellm {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

}  // namespace onellm

extern "C" const char* onellm_last_error(void) { return onellm::g_err; }

extern "C" int onellm_abi_version(void) { return 1; }
