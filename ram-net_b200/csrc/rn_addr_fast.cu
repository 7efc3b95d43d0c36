// Thread-per-row address decoder for the shapes the models use ((U,P,K) known at compile time).
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
#include "rn_addr.cuh"

#include <type_traits>

namespace {

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

struct FastParams {
    const void *addr[2];
    int64_t sb, sh, st;      // element strides of batch / head / token; the U*P block is contiguous
    const int32_t *pos;
    int64_t pb, pt;
    int32_t *idx;
    float *val;
    int64_t ob, oh, ot;      // output strides; the K entries of a row are contiguous
    int B, H, T, E, A;
    float re_norm[2];
    float sign[2];
    int encode_batch;
    int nwhich;
    int64_t n_rows;          // B*T*H
};

constexpr int FAST_THREADS = 128;

template <typename T, int U, int P, int K>
__global__ void __launch_bounds__(FAST_THREADS) rn_addr_fast_kernel(const FastParams p) {
    using DKey = typename std::conditional<Raw<T>::wide, Key64, Key32>::type;
    constexpr int NB = P / K;                 // digit blocks of K logits
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr float LN2 = 0.6931471805599453f;
    static_assert(P % K == 0 && (K & (K - 1)) == 0 && K >= 2, "P must be a multiple of the power-of-two K");

    // rows of one tensor are adjacent across the CTA: item = which * n_rows + row
    const int64_t item = int64_t(blockIdx.x) * FAST_THREADS + threadIdx.x;
    if (item >= p.n_rows * p.nwhich) return;
    const int which = int(item / p.n_rows);
    const int64_t row = item - int64_t(which) * p.n_rows;
    const int h = int(row % p.H);
    const int t = int((row / p.H) % p.T);
    const int b = int(row / (int64_t(p.H) * p.T));
    const T *src = static_cast<const T *>(p.addr[which]) + b * p.sb + h * p.sh + t * p.st;

    float beam_s[K];
    int beam_i[K];
    float lse_total = 0.f;
    bool inactive = false;
    int stride = 1;

#pragma unroll
    for (int u = 0; u < U; ++u) {
        // ---- digit u: keys, log-sum-exp, sorted Top-K -------------------------------------------
        // three passes over the row's P logits (L1-resident after the first): max, sum of
        // exponentials, keys; nothing but the keys stays in registers
        DKey dk[P];
        float xmax = -INFINITY;
        rn_for_each_logit<T, P>(src + u * P, [&](int, float x) { xmax = fmaxf(xmax, x); });
        if (xmax == -INFINITY) {
            inactive = true;
        } else {
            float s = 0.f;
            const float off = xmax * LOG2E;
            rn_for_each_logit<T, P>(src + u * P, [&](int, float x) { s += fast_ex2(fmaf(x, LOG2E, -off)); });
            lse_total += xmax + fast_lg2(s) * LN2;
        }
        rn_make_keys<T, P>(src + u * P, dk);
        static_for<0, NB>([&](auto BI) __attribute__((always_inline)) { oem_sort_desc<K>(dk + decltype(BI)::value * K); });
        static_for<1, NB>([&](auto BI) __attribute__((always_inline)) { fold_topk<K>(dk, dk + decltype(BI)::value * K); });
        // dk[0..K) = this digit's K best logits, sorted descending

        if (u == 0) {
#pragma unroll
            for (int e = 0; e < K; ++e) {
                beam_s[e] = digit_value<T>(dk[e]) + 0.0f;
                beam_i[e] = digit_index(dk[e]);
            }
        } else {
            // ---- candidates (i, j), (i+1)(j+1) <= K --------------------------------------------
            float dv[K];
            int dp[K];
#pragma unroll
            for (int e = 0; e < K; ++e) {
                dv[e] = digit_value<T>(dk[e]);
                dp[e] = digit_index(dk[e]) * stride;
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
    }

    // ---- weights and stores --------------------------------------------------------------------
    float logq[K];
#pragma unroll
    for (int e = 0; e < K; ++e) logq[e] = beam_s[e] - lse_total;
    const float rho = p.re_norm[which];
    if (rho != 0.f && !inactive && logq[0] > -INFINITY) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < K; ++e) s += fast_ex2((logq[e] - logq[0]) * LOG2E);
        const float l = logq[0] + fast_lg2(s) * LN2;
#pragma unroll
        for (int e = 0; e < K; ++e) logq[e] -= rho * l;
    }
    const int shift = (h < p.E) ? rn_pos_mod(p.pos[b * p.pb + t * p.pt], p.A) : 0;
    const int offs = (p.encode_batch ? (b * p.H + h) : h) * p.A;
    const int64_t o = b * p.ob + h * p.oh + t * p.ot + (which ? K : 0);
    int out_i[K];
    float out_v[K];
#pragma unroll
    for (int e = 0; e < K; ++e) {
        const bool noop = inactive || logq[e] == -INFINITY;
        out_i[e] = offs + rn_cape(noop ? e : beam_i[e], shift, p.A);
        out_v[e] = inactive ? 0.f : p.sign[which] * fast_ex2(logq[e] * LOG2E);
    }
#pragma unroll
    for (int v = 0; v < K / 4; ++v) {
        reinterpret_cast<int4 *>(p.idx + o)[v] = make_int4(out_i[4 * v], out_i[4 * v + 1], out_i[4 * v + 2], out_i[4 * v + 3]);
        reinterpret_cast<float4 *>(p.val + o)[v] = make_float4(out_v[4 * v], out_v[4 * v + 1], out_v[4 * v + 2], out_v[4 * v + 3]);
    }
}

template <typename T, int U, int P, int K>
int launch_fast(const FastParams &p, cudaStream_t stream) {
    const int64_t items = p.n_rows * p.nwhich;
    const int64_t grid = (items + FAST_THREADS - 1) / FAST_THREADS;
    rn_addr_fast_kernel<T, U, P, K><<<unsigned(grid), FAST_THREADS, 0, stream>>>(p);
    return 0;
}

template <typename T>
int dispatch_fast(const FastParams &p, int U, int P, int K, cudaStream_t stream) {
    if (U == 2 && P == 64 && K == 16) return launch_fast<T, 2, 64, 16>(p, stream);
    if (U == 3 && P == 32 && K == 8) return launch_fast<T, 3, 32, 8>(p, stream);
    if (U == 2 && P == 16 && K == 4) return launch_fast<T, 2, 16, 4>(p, stream);
    return -1;
}

}  // namespace

// Returns 0 when a specialised kernel was launched, -1 when the shape / layout has none.
int rn_addr_fwd_fast(const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides, const int32_t *pos,
                     const int64_t *pos_strides, int32_t *idx, float *val, const int64_t *out_strides, int64_t B,
                     int64_t H, int64_t U, int64_t P, int64_t T, int64_t E, int64_t A, int64_t Kw, int64_t Kr,
                     double w_re_norm, double r_re_norm, int w_neg, int r_neg, int encode_batch, cudaStream_t stream) {
    if (r_addr != nullptr && Kw != Kr) return -1;
    const bool shape_ok = (U == 2 && P == 64 && Kw == 16) || (U == 3 && P == 32 && Kw == 8) || (U == 2 && P == 16 && Kw == 4);
    if (!shape_ok) return -1;
    const size_t esz = dtype == RN_F32 ? 4 : 2;
    // the U*P block of a row must be contiguous and 16-byte aligned; the K outputs of a row too
    if (addr_strides[3] != 1 || addr_strides[2] != P) return -1;
    if (((addr_strides[0] | addr_strides[1] | addr_strides[4]) * int64_t(esz)) % 16 != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(w_addr) | reinterpret_cast<uintptr_t>(r_addr)) & 15) return -1;
    if (out_strides[2] != 1 || ((out_strides[0] | out_strides[1] | out_strides[3]) & 3) != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(val)) & 15) return -1;
    if (B * T * H * (r_addr ? 2 : 1) >= (int64_t(1) << 31) * FAST_THREADS) return -1;

    FastParams p{};
    p.addr[0] = w_addr; p.addr[1] = r_addr;
    p.sb = addr_strides[0]; p.sh = addr_strides[1]; p.st = addr_strides[4];
    p.pos = pos; p.pb = pos_strides[0]; p.pt = pos_strides[1];
    p.idx = idx; p.val = val;
    p.ob = out_strides[0]; p.oh = out_strides[1]; p.ot = out_strides[3];
    p.B = int(B); p.H = int(H); p.T = int(T); p.E = int(E); p.A = int(A);
    p.re_norm[0] = float(w_re_norm); p.re_norm[1] = float(r_re_norm);
    p.sign[0] = w_neg ? -1.f : 1.f; p.sign[1] = r_neg ? -1.f : 1.f;
    p.encode_batch = encode_batch;
    p.nwhich = r_addr ? 2 : 1;
    p.n_rows = B * T * H;
    if (dtype == RN_F32) return dispatch_fast<float>(p, int(U), int(P), int(Kw), stream);
    if (dtype == RN_F16) return dispatch_fast<__half>(p, int(U), int(P), int(Kw), stream);
    return dispatch_fast<__nv_bfloat16>(p, int(U), int(P), int(Kw), stream);
}
