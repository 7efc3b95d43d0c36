// Library-wide C-ABI helpers: error text, version, cached device properties.
#include "rn_prefill.cuh"

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

// ------------------------------------------------------------------------------------------
// device status word: how a kernel reports a failure it cannot raise itself
// ------------------------------------------------------------------------------------------
// Every wait of a kernel on an asynchronous copy is bounded.  When one runs out the kernel records a
// non-zero code here with atomicMax, finishes without touching more state and returns, so the context
// stays usable; the word is sticky until rn_device_status() clears it.  One word per GPU that loads
// the library (it lives in the module image, nothing is allocated).
static __device__ int rn_status_word_dev = 0;

int *rn_status_word(int device) {
    static std::mutex mu;
    static int *cached[64] = {nullptr};
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[device] == nullptr) {
        RnDeviceGuard guard(device);
        void *ptr = nullptr;
        if (!guard.ok || cudaGetSymbolAddress(&ptr, rn_status_word_dev) != cudaSuccess) return nullptr;
        cached[device] = static_cast<int *>(ptr);
    }
    return cached[device];
}

extern "C" int rn_device_status(int device, void *stream, int reset, int *status) {
    rn_clear_error();
    RN_REQUIRE(status != nullptr, "null pointer argument");
    int *word = rn_status_word(device);
    RN_REQUIRE(word != nullptr, "cannot locate the status word of device %d", device);
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);
    cudaStream_t s = cudaStream_t(stream);
    int host = 0;
    RN_CUDA(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, s));
    if (reset) RN_CUDA(cudaMemsetAsync(word, 0, sizeof(int), s));
    RN_CUDA(cudaStreamSynchronize(s));
    *status = host;
    return 0;
}

// Diagnostic: one CTA arms an mbarrier for MORE bytes than its single 256-byte bulk copy delivers, so the
// copy itself completes, the barrier phase never does, and the bounded wait gives up after 2^limit_log2
// clock cycles.  The kernel then reports RN_STATUS_WAIT_TIMEOUT through the status word, waits (bounded)
// until the copied bytes are visible, invalidates the barrier and returns: nothing is left in flight and
// nothing faults.  Exercises exactly the wait the product kernels use.
static __device__ __align__(16) unsigned char rn_selftest_src[256];

__global__ void rn_wait_selftest_kernel(int *status, int extra_bytes, int limit_log2) {
    __shared__ __align__(16) uint32_t dst[64];
    __shared__ __align__(8) uint64_t bar;
    const int tid = threadIdx.x;
    if (tid < 64) dst[tid] = 0xffffffffu;
    if (tid == 0) {
        rn_mbar_init(&bar, 1);
        rn_mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
        rn_fence_proxy_async();
        rn_mbar_expect_tx(&bar, 256u + uint32_t(extra_bytes));
        rn_bulk_g2s(dst, rn_selftest_src, 256u, &bar);
        if (!rn_mbar_wait_bounded(&bar, 0u, 1ll << limit_log2)) atomicMax(status, RN_STATUS_WAIT_TIMEOUT);
        // the copy is independent of the barrier's phase: let it finish before the CTA's shared memory goes away
        const long long start = clock64();
        while (*reinterpret_cast<volatile uint32_t *>(&dst[63]) != 0u && clock64() - start < (1ll << 24)) {}
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(rn_smem_u32(&bar)) : "memory");
    }
}

extern "C" int rn_selftest_wait_timeout(int extra_bytes, int limit_log2, int device, void *stream) {
    rn_clear_error();
    RN_REQUIRE(extra_bytes >= 0 && extra_bytes <= 4096 && (extra_bytes % 16) == 0, "extra_bytes must be a multiple of 16 in [0, 4096]");
    RN_REQUIRE(limit_log2 >= 10 && limit_log2 <= 24, "limit_log2 must be in [10, 24]");
    int *word = rn_status_word(device);
    RN_REQUIRE(word != nullptr, "cannot locate the status word of device %d", device);
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);
    rn_wait_selftest_kernel<<<1, 64, 0, cudaStream_t(stream)>>>(word, extra_bytes, limit_log2);
    RN_CUDA(cudaGetLastError());
    return 0;
}
