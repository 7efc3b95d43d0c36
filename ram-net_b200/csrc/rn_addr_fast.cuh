// Thread-per-row address decoder for the shapes the models use (device code shared by the address
// kernel and the fused decode-step kernel) ((U,P,K) known at compile time).
//
// One thread decodes one (batch, token, head, write|read) block of U*P logits entirely in
// registers with fully unrolled compare-exchange networks, so no shuffles and no shared memory
// are needed and a warp's 32 rows progress in lockstep without divergence:
//   per digit   Top-K of the P logits: sort blocks of K (Batcher odd-even merge sort), then fold
//               the blocks pairwise with a bitonic top-half + bitonic merge.  16-bit inputs use one
//               32-bit key per logit, (ordered bits << 16) | (0xffff - p), so a compare-exchange
//               is an integer max/min pair.
//   per level   candidates (i, j) with (i+1)(j+1) <= K between the sorted prefixes and the sorted
//               digit; row 0 and column 0 of that table are already sorted, only the remainder is
//               sorted, then the blocks are folded the same way.  Keys are (ordered fp32 score,
//               ~index) pairs compared as 64-bit integers.
// Same total order, same fp32 left-fold score and same special cases as rn_addr.cuh; the
// general warp-cooperative kernel remains the path for every other (U,P,K).
#pragma once

#include "rn_addr.cuh"

#include <type_traits>

namespace rn_fast {


__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_lg2(float x) {
    float y;
    asm("lg2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- keys ------------------------------------------------------------------------------------
struct Key32 {
    uint32_t v;
};
struct Key64 {
    uint32_t hi, lo;
};
__device__ __forceinline__ bool key_less(const Key32 &a, const Key32 &b) { return a.v < b.v; }
__device__ __forceinline__ bool key_less(const Key64 &a, const Key64 &b) {
    return a.hi < b.hi || (a.hi == b.hi && a.lo < b.lo);
}
__device__ __forceinline__ void cmpx(Key32 &a, Key32 &b) {  // afterwards a >= b
    const uint32_t mx = max(a.v, b.v), mn = min(a.v, b.v);
    a.v = mx;
    b.v = mn;
}
__device__ __forceinline__ void cmpx(Key64 &a, Key64 &b) {
    if (key_less(a, b)) {
        const Key64 t = a;
        a = b;
        b = t;
    }
}
__device__ __forceinline__ Key32 key_max(const Key32 &a, const Key32 &b) { return Key32{max(a.v, b.v)}; }
__device__ __forceinline__ Key64 key_max(const Key64 &a, const Key64 &b) { return key_less(a, b) ? b : a; }
__device__ __forceinline__ Key32 key_lowest(Key32) { return Key32{0u}; }
__device__ __forceinline__ Key64 key_lowest(Key64) { return Key64{0u, 0u}; }

// ---- networks: every index is a template constant, so key arrays stay in registers ------------
// Batcher's odd-even merge sort (descending), recursive formulation.
template <int I, int End, int Step, int R, typename Key>
__device__ __forceinline__ void oem_cmp_row(Key *k) {
    if constexpr (I + R < End) {
        cmpx(k[I], k[I + R]);
        oem_cmp_row<I + Step, End, Step, R>(k);
    }
}
template <int Lo, int N, int R, typename Key>
__device__ __forceinline__ void oem_merge(Key *k) {
    constexpr int M = R * 2;
    if constexpr (M < N) {
        oem_merge<Lo, N, M>(k);
        oem_merge<Lo + R, N, M>(k);
        oem_cmp_row<Lo + R, Lo + N, M, R>(k);
    } else {
        cmpx(k[Lo], k[Lo + R]);
    }
}
template <int Lo, int N, typename Key>
__device__ __forceinline__ void oem_sort_range(Key *k) {
    if constexpr (N > 1) {
        oem_sort_range<Lo, N / 2>(k);
        oem_sort_range<Lo + N / 2, N / 2>(k);
        oem_merge<Lo, N, 1>(k);
    }
}
template <int N, typename Key>
__device__ __forceinline__ void oem_sort_desc(Key *k) {
    oem_sort_range<0, N>(k);
}
// k[0..N) bitonic -> sorted descending
template <int I, int N, int S, typename Key>
__device__ __forceinline__ void bitonic_row(Key *k) {
    if constexpr (I < N) {
        if constexpr ((I & S) == 0) cmpx(k[I], k[I | S]);
        bitonic_row<I + 1, N, S>(k);
    }
}
template <int N, int S, typename Key>
__device__ __forceinline__ void bitonic_stage(Key *k) {
    if constexpr (S >= 1) {
        bitonic_row<0, N, S>(k);
        bitonic_stage<N, S / 2>(k);
    }
}
template <int N, typename Key>
__device__ __forceinline__ void bitonic_merge_desc(Key *k) {
    bitonic_stage<N, N / 2>(k);
}
// a[0..K) and b[0..K) sorted descending -> a = the K largest of both, sorted descending
template <int K, typename Key>
__device__ __forceinline__ void fold_topk(Key *a, const Key *b) {
#pragma unroll
    for (int i = 0; i < K; ++i) a[i] = key_max(a[i], b[K - 1 - i]);
    bitonic_merge_desc<K>(a);
}

// candidates (i, j) with i >= 1, j >= 1 and (i+1)(j+1) <= K, in row-major order
__host__ __device__ constexpr int rn_remainder_before(int K, int i) {
    int n = 0;
    for (int ii = 1; ii < i; ++ii) n += (K / (ii + 1) > 1) ? K / (ii + 1) - 1 : 0;
    return n;
}
__host__ __device__ constexpr int rn_remainder_count(int K) { return rn_remainder_before(K, K); }

template <int Lo, int Hi, typename F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (Lo < Hi) {
        f(std::integral_constant<int, Lo>{});
        static_for<Lo + 1, Hi>(f);
    }
}

// Writes candidate (I, J), (I+1)(J+1) <= K, I, J >= 1, into its slot of remainder block BID and
// recurses over the rest of the table; every index is a template constant.
template <int K, int BID, int I, int J>
struct RemFill {
    static __device__ __forceinline__ void run(Key64 (&blk)[K], const float (&beam_s)[K], const int (&beam_i)[K],
                                               const float (&dv)[K], const int (&dp)[K]) {
        if constexpr ((I + 1) * (J + 1) <= K) {
            constexpr int pos = rn_remainder_before(K, I) + (J - 1);
            if constexpr (pos / K == BID)
                blk[pos % K] = Key64{rn_ord(beam_s[I] + dv[J] + 0.0f), ~uint32_t(beam_i[I] + dp[J])};
            if constexpr (J + 1 < K) RemFill<K, BID, I, J + 1>::run(blk, beam_s, beam_i, dv, dp);
            else if constexpr (I + 1 < K) RemFill<K, BID, I + 1, 1>::run(blk, beam_s, beam_i, dv, dp);
        } else if constexpr (I + 1 < K && J > 1) {
            RemFill<K, BID, I + 1, 1>::run(blk, beam_s, beam_i, dv, dp);  // rest of row I is out of range too
        }
    }
};

template <typename T> struct Raw;  // logits as stored
template <> struct Raw<float> {
    static constexpr bool wide = true;
};
template <> struct Raw<__half> {
    static constexpr bool wide = false;
};
template <> struct Raw<__nv_bfloat16> {
    static constexpr bool wide = false;
};

__device__ __forceinline__ uint32_t ord16_from_bf16(uint32_t h) {
    if (h == 0x8000u) h = 0u;  // -0.0 ties with +0.0
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}
__device__ __forceinline__ float f32_from_ord16_bf16(uint32_t o) {
    const uint32_t h = (o & 0x8000u) ? (o & 0x7fffu) : (~o & 0xffffu);
    return __uint_as_float(h << 16);
}
__device__ __forceinline__ float f32_from_ord16_half(uint32_t o) {
    const uint32_t h = (o & 0x8000u) ? (o & 0x7fffu) : (~o & 0xffffu);
    return __half2float(__ushort_as_half((unsigned short)h));
}

template <typename T>
__device__ __forceinline__ float digit_value(const Key32 &k) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) return f32_from_ord16_bf16(k.v >> 16);
    else return f32_from_ord16_half(k.v >> 16);
}
__device__ __forceinline__ int digit_index(const Key32 &k) { return int(0xffffu - (k.v & 0xffffu)); }
template <typename T>
__device__ __forceinline__ float digit_value(const Key64 &k) { return rn_unord(k.hi); }
__device__ __forceinline__ int digit_index(const Key64 &k) { return int(~k.lo); }

// Visit the P logits of one digit as floats; q is a compile-time index after unrolling.
template <typename T, int P, typename F>
__device__ __forceinline__ void rn_for_each_logit(const T *src, F &&f) {
    if constexpr (Raw<T>::wide) {
#pragma unroll
        for (int v = 0; v < P / 4; ++v) {
            const float4 x = reinterpret_cast<const float4 *>(src)[v];
            f(4 * v, x.x); f(4 * v + 1, x.y); f(4 * v + 2, x.z); f(4 * v + 3, x.w);
        }
    } else {
#pragma unroll
        for (int v = 0; v < P / 8; ++v) {
            const uint4 raw = reinterpret_cast<const uint4 *>(src)[v];
            const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t lo = wds[c] & 0xffffu, hi = wds[c] >> 16;
                if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                    f(8 * v + 2 * c, __uint_as_float(lo << 16));
                    f(8 * v + 2 * c + 1, __uint_as_float(hi << 16));
                } else {
                    f(8 * v + 2 * c, __half2float(__ushort_as_half((unsigned short)lo)));
                    f(8 * v + 2 * c + 1, __half2float(__ushort_as_half((unsigned short)hi)));
                }
            }
        }
    }
}

template <typename T, int P>
__device__ __forceinline__ void rn_make_keys(const T *src, Key64 *dk) {
    rn_for_each_logit<T, P>(src, [&](int q, float x) { dk[q] = Key64{rn_ord(x + 0.0f), ~uint32_t(q)}; });
}
template <typename T, int P>
__device__ __forceinline__ void rn_make_keys(const T *src, Key32 *dk) {
#pragma unroll
    for (int v = 0; v < P / 8; ++v) {
        const uint4 raw = reinterpret_cast<const uint4 *>(src)[v];
        const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int q = 8 * v + 2 * c;
            dk[q] = Key32{(ord16_from_bf16(wds[c] & 0xffffu) << 16) | (0xffffu - uint32_t(q))};
            dk[q + 1] = Key32{(ord16_from_bf16(wds[c] >> 16) << 16) | (0xffffu - uint32_t(q + 1))};
        }
    }
}


// Decode one row: content indices (before CAPE; a no-op entry reports its rank) and positive
// weights (zero for an inactive token), in canonical order.
template <typename T, int U, int P, int K>
__device__ __forceinline__ void thread_decode(const T *src, const float rho, int (&content)[K], float (&weight)[K]) {
    using DKey = typename std::conditional<Raw<T>::wide, Key64, Key32>::type;
    // A digit contributes its KD = min(K, P) best logits.  With K > P the beam and the digit list are padded to K
    // entries of score -inf: a padded candidate sorts with the masked ones and, like them, ends as a no-op entry.
    constexpr int KD = K < P ? K : P;
    constexpr int NB = P / KD;                // digit blocks of KD logits
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float LN2 = 0.6931471805599453f;
    static_assert(P % KD == 0 && (K & (K - 1)) == 0 && (KD & (KD - 1)) == 0 && K >= 2, "K and min(K, P) powers of two, P a multiple of min(K, P)");

    float beam_s[K];
    int beam_i[K];
    float lse_total = 0.f;
    bool inactive = false;
    int stride = 1;

    auto digit = [&](const int u) __attribute__((always_inline)) {
        // ---- digit u: keys, log-sum-exp, sorted Top-K -------------------------------------------
        // Passes over the row's P logits (L1-resident after the first); nothing but the keys stays in registers.
        // Rolled digit loop (three or more digits): keys, then the sum of exponentials; the maximum the sum needs is
        // the value of the best key (8 % faster at U = 3, P = 32, K = 8).  Unrolled (two digits of 64 logits): a
        // maximum pass first, the keys last, which keeps the 64 keys out of the way of the exponentials (the
        // two-pass order is 2.5 % slower there).
        constexpr bool MAX_FROM_KEYS = U >= 3;
        DKey dk[P];
        float xmax = -INFINITY;
        auto sort_keys = [&]() __attribute__((always_inline)) {
            rn_make_keys<T, P>(src + u * P, dk);
            static_for<0, NB>([&](auto BI) __attribute__((always_inline)) { oem_sort_desc<KD>(dk + decltype(BI)::value * KD); });
            static_for<1, NB>([&](auto BI) __attribute__((always_inline)) { fold_topk<KD>(dk, dk + decltype(BI)::value * KD); });
        };
        if constexpr (MAX_FROM_KEYS) {
            sort_keys();
            xmax = digit_value<T>(dk[0]);
        } else {
            rn_for_each_logit<T, P>(src + u * P, [&](int, float x) { xmax = fmaxf(xmax, x); });
        }
        if (xmax == -INFINITY) {
            inactive = true;
        } else {
            float s = 0.f;
            const float off = xmax * LOG2E;
            rn_for_each_logit<T, P>(src + u * P, [&](int, float x) { s += fast_ex2(fmaf(x, LOG2E, -off)); });
            lse_total += xmax + fast_lg2(s) * LN2;
        }
        if constexpr (!MAX_FROM_KEYS) sort_keys();
        // dk[0..KD) = this digit's KD best logits, sorted descending

        if (u == 0) {
#pragma unroll
            for (int e = 0; e < K; ++e) {
                beam_s[e] = e < KD ? digit_value<T>(dk[e < KD ? e : 0]) + 0.0f : -INFINITY;
                beam_i[e] = e < KD ? digit_index(dk[e < KD ? e : 0]) : 0;
            }
        } else {
            // ---- candidates (i, j), (i+1)(j+1) <= K --------------------------------------------
            float dv[K];
            int dp[K];
#pragma unroll
            for (int e = 0; e < K; ++e) {
                dv[e] = e < KD ? digit_value<T>(dk[e < KD ? e : 0]) : -INFINITY;
                dp[e] = e < KD ? digit_index(dk[e < KD ? e : 0]) * stride : 0;
            }
            // block 0: row i = 0 (sorted);  block 1: column j = 0, i >= 1 (sorted) + one pad
            Key64 best[K], blk[K];
#pragma unroll
            for (int j = 0; j < K; ++j) best[j] = Key64{rn_ord(beam_s[0] + dv[j] + 0.0f), ~uint32_t(beam_i[0] + dp[j])};
#pragma unroll
            for (int i = 1; i < K; ++i) blk[i - 1] = Key64{rn_ord(beam_s[i] + dv[0] + 0.0f), ~uint32_t(beam_i[i] + dp[0])};
            blk[K - 1] = Key64{0u, 0u};
            fold_topk<K>(best, blk);
            // the remainder (i >= 1, j >= 1), K at a time, each block sorted then folded in.
            // Position of (i, j) in the remainder list: rows before it + (j - 1); all of it folds
            // to constants once the loops are unrolled.
            constexpr int NREM = rn_remainder_count(K);
            constexpr int NBLK = (NREM + K - 1) / K;
            static_for<0, NBLK>([&](auto BID) __attribute__((always_inline)) {
#pragma unroll
                for (int e = 0; e < K; ++e) blk[e] = Key64{0u, 0u};
                RemFill<K, decltype(BID)::value, 1, 1>::run(blk, beam_s, beam_i, dv, dp);
                oem_sort_desc<K>(blk);
                fold_topk<K>(best, blk);
            });
#pragma unroll
            for (int e = 0; e < K; ++e) {
                beam_s[e] = rn_unord(best[e].hi);
                beam_i[e] = int(~best[e].lo);
            }
        }
        stride *= P;
    };
    if constexpr (U >= 3) {
        // three or more digits: the loop stays rolled.  The straight-line sorting networks are long, and with
        // the body emitted once instruction fetch stops setting the pace (10 % faster at U = 3, P = 32, K = 8;
        // at U = 2, P = 64, K = 16 the rolled form needs more registers and is slower)
#pragma unroll 1
        for (int u = 0; u < U; ++u) digit(u);
    } else {
#pragma unroll
        for (int u = 0; u < U; ++u) digit(u);
    }

    // ---- weights and stores --------------------------------------------------------------------
    float logq[K];
#pragma unroll
    for (int e = 0; e < K; ++e) logq[e] = beam_s[e] - lse_total;
    if (rho != 0.f && !inactive && logq[0] > -INFINITY) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < K; ++e) s += fast_ex2((logq[e] - logq[0]) * LOG2E);
        const float l = logq[0] + fast_lg2(s) * LN2;
#pragma unroll
        for (int e = 0; e < K; ++e) logq[e] -= rho * l;
    }
#pragma unroll
    for (int e = 0; e < K; ++e) {
        const bool noop = inactive || logq[e] == -INFINITY;
        content[e] = noop ? e : beam_i[e];
        weight[e] = inactive ? 0.f : fast_ex2(logq[e] * LOG2E);
    }
}

// ---- four lanes per row ------------------------------------------------------------------------
// Same result as thread_decode, but the work of one row is spread over four adjacent lanes so the
// dependent instruction chain is ~5x shorter (used where few rows must finish quickly: the decode
// step).  Needs P == 4 * K: each lane sorts K logits of a digit, then two cross-lane folds
// (xor 1, xor 2) leave the digit's sorted Top-K in all four lanes; candidate blocks of a level are
// built one per lane and folded the same way.  Every lane of the warp must call it.
__device__ __forceinline__ Key32 key_shfl_xor(const Key32 &k, int m) { return Key32{__shfl_xor_sync(RN_FULL, k.v, m)}; }
__device__ __forceinline__ Key64 key_shfl_xor(const Key64 &k, int m) {
    return Key64{__shfl_xor_sync(RN_FULL, k.hi, m), __shfl_xor_sync(RN_FULL, k.lo, m)};
}
template <int K, typename Key>
__device__ __forceinline__ void fold_topk_xlane(Key *a, int m) {
    Key t[K];
#pragma unroll
    for (int i = 0; i < K; ++i) t[i] = key_max(a[i], key_shfl_xor(a[K - 1 - i], m));
#pragma unroll
    for (int i = 0; i < K; ++i) a[i] = t[i];
    bitonic_merge_desc<K>(a);
}

template <typename T, int K>
__device__ __forceinline__ void quad_make_keys(const T *src, int p0, Key64 *dk) {
    rn_for_each_logit<T, K>(src, [&](int q, float x) { dk[q] = Key64{rn_ord(x + 0.0f), ~uint32_t(p0 + q)}; });
}
template <typename T, int K>
__device__ __forceinline__ void quad_make_keys(const T *src, int p0, Key32 *dk) {
    if constexpr (K >= 8) {
#pragma unroll
        for (int v = 0; v < K / 8; ++v) {
            const uint4 raw = reinterpret_cast<const uint4 *>(src)[v];
            const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int q = 8 * v + 2 * c;
                dk[q] = Key32{(ord16_from_bf16(wds[c] & 0xffffu) << 16) | (0xffffu - uint32_t(p0 + q))};
                dk[q + 1] = Key32{(ord16_from_bf16(wds[c] >> 16) << 16) | (0xffffu - uint32_t(p0 + q + 1))};
            }
        }
    } else {
        const uint2 raw = *reinterpret_cast<const uint2 *>(src);  // K == 4 sixteen-bit logits
        const uint32_t wds[2] = {raw.x, raw.y};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            dk[2 * c] = Key32{(ord16_from_bf16(wds[c] & 0xffffu) << 16) | (0xffffu - uint32_t(p0 + 2 * c))};
            dk[2 * c + 1] = Key32{(ord16_from_bf16(wds[c] >> 16) << 16) | (0xffffu - uint32_t(p0 + 2 * c + 1))};
        }
    }
}

template <typename T, int U, int P, int K>
__device__ __forceinline__ void quad_decode(const T *src, const float rho, const int gl, int (&content)[K],
                                            float (&weight)[K]) {
    using DKey = typename std::conditional<Raw<T>::wide, Key64, Key32>::type;
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float LN2 = 0.6931471805599453f;
    static_assert(P == 4 * K && (K & (K - 1)) == 0 && K >= 4, "quad_decode needs P == 4 K");
    constexpr int NREM = rn_remainder_count(K);
    constexpr int NBLK = (NREM + K - 1) / K;
    static_assert(NBLK <= 2, "candidate blocks must fit the four lanes");

    float beam_s[K];
    int beam_i[K];
    float lse_total = 0.f;
    bool inactive = false;
    int stride = 1;

    // the digit loop stays rolled: the straight-line networks are long and this code runs on few
    // warps, so instruction fetch, not issue, would otherwise set the pace
#pragma unroll 1
    for (int u = 0; u < U; ++u) {
        const T *mine = src + u * P + gl * K;  // this lane's K logits of digit u
        DKey dk[K];
        quad_make_keys<T, K>(mine, gl * K, dk);
        oem_sort_desc<K>(dk);
#pragma unroll 1
        for (int m = 1; m <= 2; m <<= 1) fold_topk_xlane<K>(dk, m);
        // dk[0..K) = the digit's K best logits, sorted, in all four lanes
        const float xmax = digit_value<T>(dk[0]);
        if (xmax == -INFINITY) {
            inactive = true;
        } else {
            float s = 0.f;
            const float off = xmax * LOG2E;
            if constexpr (Raw<T>::wide || K >= 8) {
                rn_for_each_logit<T, K>(mine, [&](int, float x) { s += fast_ex2(fmaf(x, LOG2E, -off)); });
            } else {
#pragma unroll
                for (int q = 0; q < K; ++q) s += fast_ex2(fmaf(rn_to_float<T>(mine[q]), LOG2E, -off));
            }
            s += __shfl_xor_sync(RN_FULL, s, 1);
            s += __shfl_xor_sync(RN_FULL, s, 2);
            lse_total += xmax + fast_lg2(s) * LN2;
        }
        if (u == 0) {
#pragma unroll
            for (int e = 0; e < K; ++e) {
                beam_s[e] = digit_value<T>(dk[e]) + 0.0f;
                beam_i[e] = digit_index(dk[e]);
            }
        } else {
            float dv[K];
            int dp[K];
#pragma unroll
            for (int e = 0; e < K; ++e) {
                dv[e] = digit_value<T>(dk[e]);
                dp[e] = digit_index(dk[e]) * stride;
            }
            Key64 blk[K];
#pragma unroll
            for (int e = 0; e < K; ++e) blk[e] = Key64{0u, 0u};
            if (gl == 0) {          // row i = 0, already sorted
#pragma unroll
                for (int j = 0; j < K; ++j) blk[j] = Key64{rn_ord(beam_s[0] + dv[j] + 0.0f), ~uint32_t(beam_i[0] + dp[j])};
            } else if (gl == 1) {   // column j = 0, i >= 1, already sorted
#pragma unroll
                for (int i = 1; i < K; ++i) blk[i - 1] = Key64{rn_ord(beam_s[i] + dv[0] + 0.0f), ~uint32_t(beam_i[i] + dp[0])};
            } else if (gl == 2) {   // first block of the remainder
                RemFill<K, 0, 1, 1>::run(blk, beam_s, beam_i, dv, dp);
            } else if (NBLK > 1) {  // second block of the remainder
                RemFill<K, 1, 1, 1>::run(blk, beam_s, beam_i, dv, dp);
            }
            if (gl >= 2) oem_sort_desc<K>(blk);
#pragma unroll 1
            for (int m = 1; m <= 2; m <<= 1) fold_topk_xlane<K>(blk, m);
#pragma unroll
            for (int e = 0; e < K; ++e) {
                beam_s[e] = rn_unord(blk[e].hi);
                beam_i[e] = int(~blk[e].lo);
            }
        }
        stride *= P;
    }

    float logq[K];
#pragma unroll
    for (int e = 0; e < K; ++e) logq[e] = beam_s[e] - lse_total;
    if (rho != 0.f && !inactive && logq[0] > -INFINITY) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < K; ++e) s += fast_ex2((logq[e] - logq[0]) * LOG2E);
        const float l = logq[0] + fast_lg2(s) * LN2;
#pragma unroll
        for (int e = 0; e < K; ++e) logq[e] -= rho * l;
    }
#pragma unroll
    for (int e = 0; e < K; ++e) {
        const bool noop = inactive || logq[e] == -INFINITY;
        content[e] = noop ? e : beam_i[e];
        weight[e] = inactive ? 0.f : fast_ex2(logq[e] * LOG2E);
    }
}

}  // namespace rn_fast
