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
