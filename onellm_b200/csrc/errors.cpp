// Thread-local error text behind onellm_last_error(), and the per-thread count of kernel launches.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace onellm {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// Kernel launches issued by the calling thread through this library (the model reports them:
// onellm_llama_get_state).
static thread_local long g_launches = 0;
void note_launch(int n) { g_launches += n; }
long launches_noted() { return g_launches; }

cudaError_t prefer_max_shared(const void* kernel)
{
    static std::mutex mu;
    static std::set<std::pair<const void*, int>> done;
    const auto key = std::make_pair(kernel, current_device());
    std::lock_guard<std::mutex> lock(mu);
    if (done.count(key)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) done.insert(key);
    return e;
}

}  // namespace onellm

extern "C" const char* onellm_last_error(void) { return onellm::g_err; }

extern "C" int onellm_abi_version(void) { return 1; }
