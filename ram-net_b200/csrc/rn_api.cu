// Library-wide C-ABI helpers: error text, version, cached device properties.
#include "rn_common.cuh"

#include <mutex>

static thread_local char g_rn_error[512] = {0};

void rn_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_rn_error, sizeof(g_rn_error), fmt, ap);
    va_end(ap);
}

void rn_clear_error() { g_rn_error[0] = 0; }

int rn_sm_count(int device) {
    // read-mostly cache; a race only repeats the query
    static int cached[64] = {0};
    if (device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

extern "C" int rn_int_bits(void) { return 32; }

extern "C" const char *rn_last_error(void) { return g_rn_error; }

extern "C" const char *rn_version(void) { return "ramnet_b200 sm_100a"; }

// ------------------------------------------------------------------------------------------
// optional per-kernel timing for benchmarks: CUDA events recorded around each launch of the
// calling thread's next entry-point calls, on the stream the kernels run on
// ------------------------------------------------------------------------------------------
static thread_local bool g_prof_on = false;
static thread_local int g_prof_count = 0;
static thread_local cudaEvent_t g_prof_events[16];
static thread_local int g_prof_created = 0;

void rn_prof_reset() { g_prof_count = 0; }

void rn_prof_mark(cudaStream_t stream) {
    if (!g_prof_on || g_prof_count >= 16) return;
    if (g_prof_count >= g_prof_created) {
        if (cudaEventCreate(&g_prof_events[g_prof_created]) != cudaSuccess) return;
        ++g_prof_created;
    }
    cudaEventRecord(g_prof_events[g_prof_count++], stream);
}

extern "C" int rn_prof_enable(int on) {
    g_prof_on = on != 0;
    g_prof_count = 0;
    return 0;
}

extern "C" int rn_prof_read(float *ms, int n) {
    if (g_prof_count < 2) return 0;
    if (cudaEventSynchronize(g_prof_events[g_prof_count - 1]) != cudaSuccess) return -1;
    int out = 0;
    for (int i = 1; i < g_prof_count && out < n; ++i, ++out)
        if (cudaEventElapsedTime(&ms[out], g_prof_events[i - 1], g_prof_events[i]) != cudaSuccess) return -1;
    return out;
}
