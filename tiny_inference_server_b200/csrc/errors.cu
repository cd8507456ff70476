// Last-error text of the library (per host thread) and the launch check.
#include "common.cuh"
#include "timeline.cuh"
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

static thread_local char g_err[512] = "";

void tis_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int tis_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        tis_set_error("%s: %s", what, cudaGetErrorString(e));
        return TIS_CUDA_ERROR;
    }
    return TIS_OK;
}

TIS_API const char* tis_last_error() { return g_err; }

bool tis_pdl_enabled() {
    static const bool on = [] {
        const char* v = getenv("TIS_NO_PDL");
        return !(v != nullptr && v[0] != '\0' && v[0] != '0');
    }();
    return on;
}

// Version of the launcher interface; the Python side refuses a library built from
// other sources than its own.
TIS_API int tis_abi_version() { return 4; }

#ifdef TIS_TIMELINE
static thread_local unsigned long long* g_timeline = nullptr;

// The next launch of an instrumented kernel of this library writes its stamps to `buffer`
// ([CTAs][TIS_TIMELINE_SLOTS] 64-bit words, zeroed by the caller); the launches after it write nothing.
TIS_API void tis_timeline_next(void* buffer) { g_timeline = static_cast<unsigned long long*>(buffer); }
TIS_API int tis_timeline_slots() { return TIS_TIMELINE_SLOTS; }

Timeline tis_timeline_take() {
    Timeline t{g_timeline};
    g_timeline = nullptr;
    return t;
}
#endif
