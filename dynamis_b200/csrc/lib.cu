// Library-wide pieces of the dynb C ABI: error reporting and version.
#include "common.cuh"

#include <stdio.h>
#include <string.h>

namespace dynb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* msg)
{
    strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = '\0';
}

int fail_cuda(cudaError_t e, const char* what)
{
    char buf[512];
    snprintf(buf, sizeof(buf), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    set_last_error(buf);
    return DYNB_ERR_CUDA;
}

int fail_arg(const char* what)
{
    set_last_error(what);
    return DYNB_ERR_ARG;
}

}  // namespace dynb

extern "C" const char* dynb_last_error(void) { return dynb::g_last_error; }
extern "C" int dynb_version(void) { return 1; }
