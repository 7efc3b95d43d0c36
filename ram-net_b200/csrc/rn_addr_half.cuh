// Sixteen lanes per address: the decoder of the fused decode step for U = 2, P = 64, K = 16 and
// 16-bit logits.
//
// The decode step has few rows (two per (batch, head) pair) and nothing else can start before their
// addresses are known, so what matters is the length of the dependent instruction chain of ONE row.
// Here a row is spread over the 16 lanes of a half-warp, four keys per lane, and every sort is a
// bitonic network over those 64 keys: 21 compare-exchange stages, 10 of them across lanes (one
// shuffle each), instead of thousands of dependent register-to-register instructions.  A warp
// decodes the write and the read address of one pair at the same time (lower / upper half).
//
//   per digit   64 keys (ordered 16-bit logit << 16 | 0xffff - p), sorted descending; rank g ends in lane g
//   level 2     the 50 candidates (i, j), (i+1)(j+1) <= 16, four per lane, as (ordered fp32 score, ~index)
//               keys, sorted descending; rank g ends in lane g
// Same total order (score descending, index ascending), same fp32 score x0 + x1 and the same special
// cases (inactive token, -inf entries report their rank) as rn_addr_fast.cuh.
#pragma once

#include "rn_addr_fast.cuh"

namespace rn_half {
using rn_fast::Key32;

// Keys are plain unsigned integers here (32-bit digit keys, 64-bit candidate keys = ordered score << 32 |
// ~index) and every compare-exchange is written with max / min / select, never a branch: the lanes of a
// warp take different directions in the same stage.
__device__ __forceinline__ uint32_t shfl_xor(uint32_t k, int m) { return __shfl_xor_sync(RN_FULL, k, m); }
__device__ __forceinline__ uint64_t shfl_xor(uint64_t k, int m) {
    const uint32_t hi = __shfl_xor_sync(RN_FULL, uint32_t(k >> 32), m), lo = __shfl_xor_sync(RN_FULL, uint32_t(k), m);
    return (uint64_t(hi) << 32) | lo;
}
__device__ __forceinline__ uint32_t shfl_idx(uint32_t k, int src) { return __shfl_sync(RN_FULL, k, src); }
__device__ __forceinline__ uint64_t shfl_idx(uint64_t k, int src) {
    const uint32_t hi = __shfl_sync(RN_FULL, uint32_t(k >> 32), src), lo = __shfl_sync(RN_FULL, uint32_t(k), src);
    return (uint64_t(hi) << 32) | lo;
}
// afterwards a >= b
__device__ __forceinline__ void cmpx_desc(uint32_t &a, uint32_t &b) {
    const uint32_t mx = max(a, b), mn = min(a, b);
    a = mx;
    b = mn;
}
__device__ __forceinline__ void cmpx_desc(uint64_t &a, uint64_t &b) {
    const bool lt = a < b;
    const uint64_t t = lt ? b : a;
    b = lt ? a : b;
    a = t;
}
// keep the larger (or the smaller) of this lane's key and the partner's
__device__ __forceinline__ uint32_t pick(uint32_t mine, uint32_t other, bool keep_max) {
    return keep_max ? max(mine, other) : min(mine, other);
}
__device__ __forceinline__ uint64_t pick(uint64_t mine, uint64_t other, bool keep_max) {
    return ((mine < other) == keep_max) ? other : mine;
}

// Bitonic sort, descending, of the 64 keys of a half-warp; element index = lane_in_half * 4 + slot.
// The variant whose merges start with a mirrored exchange (element i with i ^ (size - 1)): every
// compare-exchange then points the same way (the larger key to the lower index), so the only per-lane
// predicate is "this lane holds the lower element", one test per lane-distance bit for the whole sort.
// Every lane of the warp must call it (the two halves sort independently).
template <typename Key>
__device__ __forceinline__ void sort64_desc(Key (&k)[4], const int hl) {
    const bool low[4] = {(hl & 1) == 0, (hl & 2) == 0, (hl & 4) == 0, (hl & 8) == 0};
#pragma unroll
    for (int lg = 1; lg <= 6; ++lg) {  // merges of 2^lg elements
        if (lg >= 3) {
            // mirrored exchange with lane ^ (2^(lg-2) - 1), slots reversed
            const int m = (1 << (lg - 2)) - 1;
            const bool lower = low[lg - 3];  // highest bit of the lane distance
            Key o[4];
#pragma unroll
            for (int s = 0; s < 4; ++s) o[s] = shfl_xor(k[3 - s], m);
#pragma unroll
            for (int s = 0; s < 4; ++s) k[s] = pick(k[s], o[s], lower);
        } else if (lg == 2) {
            cmpx_desc(k[0], k[3]);
            cmpx_desc(k[1], k[2]);
        } else {
            cmpx_desc(k[0], k[1]);
            cmpx_desc(k[2], k[3]);
        }
#pragma unroll
        for (int jl = lg - 2; jl >= 0; --jl) {  // exchanges at distance 2^jl
            if (jl >= 2) {
                const int m = 1 << (jl - 2);
#pragma unroll
                for (int s = 0; s < 4; ++s) k[s] = pick(k[s], shfl_xor(k[s], m), low[jl - 2]);
            } else if (jl == 1) {
                cmpx_desc(k[0], k[2]);
                cmpx_desc(k[1], k[3]);
            } else {
                cmpx_desc(k[0], k[1]);
                cmpx_desc(k[2], k[3]);
            }
        }
    }
}
// the key of rank hl (element hl of the sorted sequence) -> this lane
template <typename Key>
__device__ __forceinline__ Key take_rank(const Key (&k)[4], const int lane, const int hl) {
    const int src = (lane & 16) | (hl >> 2);
    const Key t0 = shfl_idx(k[0], src), t1 = shfl_idx(k[1], src), t2 = shfl_idx(k[2], src), t3 = shfl_idx(k[3], src);
    const int s = hl & 3;
    const Key lo = (s & 1) ? t1 : t0, hi = (s & 1) ? t3 : t2;
    return (s & 2) ? hi : lo;
}
__device__ __forceinline__ float sum16(float v) {
    v += __shfl_xor_sync(RN_FULL, v, 1);
    v += __shfl_xor_sync(RN_FULL, v, 2);
    v += __shfl_xor_sync(RN_FULL, v, 4);
    v += __shfl_xor_sync(RN_FULL, v, 8);
    return v;
}

// candidate (i, j) of slot c = lane_in_half * 4 + s, row-major over i with j < 16 / (i + 1); 0xff = none
__device__ __align__(4) const unsigned char kCandidates[64] = {
    0x00, 0x01, 0x02, 0x03, 0x04, 0x05, 0x06, 0x07, 0x08, 0x09, 0x0a, 0x0b, 0x0c, 0x0d, 0x0e, 0x0f,
    0x10, 0x11, 0x12, 0x13, 0x14, 0x15, 0x16, 0x17, 0x20, 0x21, 0x22, 0x23, 0x24, 0x30, 0x31, 0x32,
    0x33, 0x40, 0x41, 0x42, 0x50, 0x51, 0x60, 0x61, 0x70, 0x71, 0x80, 0x90, 0xa0, 0xb0, 0xc0, 0xd0,
    0xe0, 0xf0, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff};
__device__ __forceinline__ uint32_t load_candidates(int hl) { return reinterpret_cast<const uint32_t *>(kCandidates)[hl]; }

// One row of 2 * 64 sixteen-bit logits, decoded by the 16 lanes of a half-warp: lane hl receives the
// entry of rank hl (content index before CAPE; a no-op entry reports its rank; weight > 0, or 0 for an
// inactive token).  cand = load_candidates(hl).  Every lane of the warp must call it.
template <typename T>
__device__ __forceinline__ void load_logits(const T *src, const int lane, uint2 (&raw)[2]) {
    raw[0] = *reinterpret_cast<const uint2 *>(src + (lane & 15) * 4);
    raw[1] = *reinterpret_cast<const uint2 *>(src + 64 + (lane & 15) * 4);
}
// logits: this lane's 4 + 4 logits of the two digits as loaded by load_logits (so that a caller can request
// them ahead of time)
template <typename T>
__device__ __forceinline__ void decode_u2p64k16(const uint2 (&logits)[2], const float rho, const int lane, const uint32_t cand,
                                                int &content, float &weight) {
    static_assert(!rn_fast::Raw<T>::wide, "16-bit logits only");
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float LN2 = 0.6931471805599453f;
    const int hl = lane & 15, base = lane & 16;
    uint32_t top[2];
    float lse_total = 0.f;
    bool inactive = false;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint2 raw = logits[u];
        const uint32_t p0 = uint32_t(hl) * 4u;
        uint32_t k[4];
        k[0] = (rn_fast::ord16_from_bf16(raw.x & 0xffffu) << 16) | (0xffffu - p0);
        k[1] = (rn_fast::ord16_from_bf16(raw.x >> 16) << 16) | (0xffffu - (p0 + 1u));
        k[2] = (rn_fast::ord16_from_bf16(raw.y & 0xffffu) << 16) | (0xffffu - (p0 + 2u));
        k[3] = (rn_fast::ord16_from_bf16(raw.y >> 16) << 16) | (0xffffu - (p0 + 3u));
        sort64_desc(k, hl);
        top[u] = take_rank(k, lane, hl);
        // the two halves of a warp may take different branches: every shuffle stays outside of them
        const float xmax = rn_fast::digit_value<T>(Key32{shfl_idx(top[u], base)});
        const bool dead = xmax == -INFINITY;
        const float off = dead ? 0.f : xmax * LOG2E;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) s += rn_fast::fast_ex2(fmaf(rn_fast::digit_value<T>(Key32{k[i]}), LOG2E, -off));
        s = sum16(s);
        if (dead) inactive = true;
        else lse_total += xmax + rn_fast::fast_lg2(s) * LN2;
    }

    uint64_t c[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t ij = (cand >> (8 * s)) & 0xffu;
        const Key32 a{shfl_idx(top[0], base | int((ij >> 4) & 15u))};
        const Key32 b{shfl_idx(top[1], base | int(ij & 15u))};
        const float score = rn_fast::digit_value<T>(a) + rn_fast::digit_value<T>(b) + 0.0f;
        const int cont = rn_fast::digit_index(a) + 64 * rn_fast::digit_index(b);
        c[s] = ij == 0xffu ? uint64_t(0) : ((uint64_t(rn_ord(score)) << 32) | uint32_t(~uint32_t(cont)));
    }
    sort64_desc(c, hl);
    const uint64_t mine = take_rank(c, lane, hl);
    float logq = rn_unord(uint32_t(mine >> 32)) - lse_total;
    const float q0 = __shfl_sync(RN_FULL, logq, base);
    const bool renorm = rho != 0.f && !inactive && q0 > -INFINITY;
    const float rs = sum16(renorm ? rn_fast::fast_ex2((logq - q0) * LOG2E) : 0.f);
    if (renorm) logq -= rho * (q0 + rn_fast::fast_lg2(rs) * LN2);
    const bool noop = inactive || logq == -INFINITY;
    content = noop ? hl : int(~uint32_t(mine));
    weight = inactive ? 0.f : rn_fast::fast_ex2(logq * LOG2E);
}

}  // namespace rn_half
