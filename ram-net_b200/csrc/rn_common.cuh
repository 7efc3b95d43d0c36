// Shared host/device helpers for the ramnet_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/ramnet_b200.h"

// ------------------------------------------------------------------------------------------
// host-side error plumbing: thread-local message + int return code
// ------------------------------------------------------------------------------------------
void rn_set_error(const char *fmt, ...);
void rn_clear_error();

#define RN_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            rn_set_error(__VA_ARGS__);   \
            return 1;                    \
        }                                \
    } while (0)

#define RN_CUDA(call)                                                                   \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) {                                                        \
            rn_set_error("%s failed: %s", #call, cudaGetErrorString(e_));               \
            return 2;                                                                   \
        }                                                                               \
    } while (0)

// Makes `device` current for the scope of one entry point and restores the previous one.
struct RnDeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit RnDeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
        cur = device;
    }
    ~RnDeviceGuard() {
        if (prev >= 0 && prev != cur) cudaSetDevice(prev);
    }
    int cur = -1;
};

int rn_sm_count(int device);

// Per-device status word (see rn_api.cu): device address, or nullptr when it cannot be found.
int *rn_status_word(int device);
constexpr int RN_STATUS_WAIT_TIMEOUT = 1;  // a bounded wait on an asynchronous copy ran out

// benchmark-only timing hooks (no-ops unless rn_prof_enable(1) was called on this thread)
void rn_prof_reset();
void rn_prof_mark(cudaStream_t stream);

// ------------------------------------------------------------------------------------------
// device helpers
// ------------------------------------------------------------------------------------------
constexpr unsigned RN_FULL = 0xffffffffu;

template <typename T> __device__ __forceinline__ float rn_to_float(T v);
template <> __device__ __forceinline__ float rn_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float rn_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float rn_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T rn_from_float(float v);
template <> __device__ __forceinline__ float rn_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half rn_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 rn_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 4 consecutive elements <-> float4; pointers must be aligned to 4 elements
template <typename T> __device__ __forceinline__ float4 rn_load4(const T *p);
template <> __device__ __forceinline__ float4 rn_load4<float>(const float *p) { return *reinterpret_cast<const float4 *>(p); }
template <> __device__ __forceinline__ float4 rn_load4<__half>(const __half *p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <> __device__ __forceinline__ float4 rn_load4<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// Four elements as loaded, not yet converted: a prefetch keeps these so that the conversion (the first use
// of the loaded registers) happens when the value is needed, not right behind the load.
template <typename T> struct RnRaw4 { uint2 v; };
template <> struct RnRaw4<float> { float4 v; };
template <typename T> __device__ __forceinline__ RnRaw4<T> rn_zero_raw4() { RnRaw4<T> r; r.v = make_uint2(0u, 0u); return r; }
template <> __device__ __forceinline__ RnRaw4<float> rn_zero_raw4<float>() { RnRaw4<float> r; r.v = make_float4(0.f, 0.f, 0.f, 0.f); return r; }
template <typename T> __device__ __forceinline__ RnRaw4<T> rn_load_raw4(const T *p) { RnRaw4<T> r; r.v = *reinterpret_cast<const uint2 *>(p); return r; }
template <> __device__ __forceinline__ RnRaw4<float> rn_load_raw4<float>(const float *p) { RnRaw4<float> r; r.v = *reinterpret_cast<const float4 *>(p); return r; }
__device__ __forceinline__ float4 rn_cvt_raw4(const RnRaw4<float> &r) { return r.v; }
__device__ __forceinline__ float4 rn_cvt_raw4(const RnRaw4<__half> &r) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 rn_cvt_raw4(const RnRaw4<__nv_bfloat16> &r) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// four floats rounded to the 16-bit type, packed as rn_load_raw4 delivers them
template <typename T> __device__ __forceinline__ RnRaw4<T> rn_pack_raw4(float4 v);
template <> __device__ __forceinline__ RnRaw4<__half> rn_pack_raw4<__half>(float4 v) {
    RnRaw4<__half> r;
    *reinterpret_cast<__half2 *>(&r.v.x) = __floats2half2_rn(v.x, v.y);
    *reinterpret_cast<__half2 *>(&r.v.y) = __floats2half2_rn(v.z, v.w);
    return r;
}
template <> __device__ __forceinline__ RnRaw4<__nv_bfloat16> rn_pack_raw4<__nv_bfloat16>(float4 v) {
    RnRaw4<__nv_bfloat16> r;
    *reinterpret_cast<__nv_bfloat162 *>(&r.v.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162 *>(&r.v.y) = __floats2bfloat162_rn(v.z, v.w);
    return r;
}
template <typename T> __device__ __forceinline__ void rn_store4(T *p, float4 v);
template <> __device__ __forceinline__ void rn_store4<float>(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
template <> __device__ __forceinline__ void rn_store4<__half>(__half *p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__half2 *>(&raw.x) = __floats2half2_rn(v.x, v.y);
    *reinterpret_cast<__half2 *>(&raw.y) = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = raw;
}
template <> __device__ __forceinline__ void rn_store4<__nv_bfloat16>(__nv_bfloat16 *p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// Monotone map float -> uint32 (larger float => larger integer); -0.0 must be canonicalised
// by the caller (x + 0.0f) so that it ties with +0.0.
__device__ __forceinline__ uint32_t rn_ord(float f) {
    uint32_t b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}
__device__ __forceinline__ float rn_unord(uint32_t o) {
    return __uint_as_float(o ^ ((o >> 31) ? 0x80000000u : 0xffffffffu));
}
// Key whose unsigned order is (score descending-is-larger, index ascending-is-larger):
// max over keys == best candidate under (score desc, index asc).
__device__ __forceinline__ uint64_t rn_key(float score, int idx) {
    return (uint64_t(rn_ord(score + 0.0f)) << 32) | uint32_t(~uint32_t(idx));
}
__device__ __forceinline__ float rn_key_score(uint64_t k) { return rn_unord(uint32_t(k >> 32)); }
__device__ __forceinline__ int rn_key_index(uint64_t k) { return int(~uint32_t(k)); }

__device__ __forceinline__ uint64_t rn_shfl_xor(uint64_t v, int m) {
    uint32_t lo = __shfl_xor_sync(RN_FULL, uint32_t(v), m);
    uint32_t hi = __shfl_xor_sync(RN_FULL, uint32_t(v >> 32), m);
    return (uint64_t(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t rn_shfl(uint64_t v, int src) {
    uint32_t lo = __shfl_sync(RN_FULL, uint32_t(v), src);
    uint32_t hi = __shfl_sync(RN_FULL, uint32_t(v >> 32), src);
    return (uint64_t(hi) << 32) | lo;
}

__device__ __forceinline__ float rn_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(RN_FULL, v, o));
    return v;
}
__device__ __forceinline__ float rn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(RN_FULL, v, o);
    return v;
}

// Descending bitonic sort of 32*KPL keys held KPL per lane; element e = lane*KPL + r.
// After the call element 0 is the largest key.
template <int KPL>
__device__ __forceinline__ void rn_bitonic_stage(uint64_t (&k)[KPL], int lane, int size, int stride) {
    // one compare-exchange stage of the classic network over N = 32*KPL elements
    if (stride >= KPL) {
        const int lstride = stride / KPL;  // partner lane distance
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            const int e = lane * KPL + r;
            const uint64_t other = rn_shfl_xor(k[r], lstride);
            const bool desc = (e & size) == 0;
            const bool lower = (e & stride) == 0;  // this element is the first of the pair
            const bool keep_max = (desc == lower);
            const uint64_t mx = k[r] > other ? k[r] : other;
            const uint64_t mn = k[r] > other ? other : k[r];
            k[r] = keep_max ? mx : mn;
        }
    } else {
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            if ((r & stride) == 0) {
                const int e = lane * KPL + r;
                const bool desc = (e & size) == 0;
                uint64_t &a = k[r];
                uint64_t &b = k[r | stride];
                const bool sw = desc ? (a < b) : (a > b);
                if (sw) { uint64_t t = a; a = b; b = t; }
            }
        }
    }
}

template <int KPL>
__device__ __forceinline__ void rn_bitonic_sort_desc(uint64_t (&k)[KPL], int lane) {
    constexpr int N = 32 * KPL;
#pragma unroll
    for (int size = 2; size <= N; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            // the final merge (size == N) sorts the whole array descending: (e & N) == 0 always
            rn_bitonic_stage<KPL>(k, lane, size, stride);
        }
    }
}

// Merge step only: `k` holds a bitonic sequence of N elements; sort it descending.
template <int KPL>
__device__ __forceinline__ void rn_bitonic_merge_desc(uint64_t (&k)[KPL], int lane) {
    constexpr int N = 32 * KPL;
#pragma unroll
    for (int stride = N >> 1; stride > 0; stride >>= 1) rn_bitonic_stage<KPL>(k, lane, N, stride);
}
