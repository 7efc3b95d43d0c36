// Warp-cooperative address decoder shared by the address kernel and the fused decode step.
//
// One warp decodes one (U, P) block of logits into the K best slot addresses under the total
// order (score descending, content index ascending), where the score of address
// (d_0 .. d_{U-1}) is the fp32 left-fold sum of the raw digit logits and digit 0 is the least
// significant digit.  The search is the exact Top-K prefix search: after each digit only the K
// best partial addresses survive.  Ranking never touches a transcendental; exp/log are used
// only for the K output weights  w_k = exp(score_k - sum_u logsumexp(x_u)).
//
// Candidate pruning: with the surviving prefixes and the new digit's logits both sorted, the
// pair (prefix rank i, digit rank j) can reach the Top-K only if (i+1)(j+1) <= K, so a level
// examines ~K ln K candidates instead of K*P.  The (i, j) list is built once per CTA.
#pragma once

#include "rn_common.cuh"

constexpr int RN_KMAX = 128;       // largest Top-K
constexpr int RN_PMAX = 128;       // largest radix
constexpr int RN_UMAX = 8;         // most digits
constexpr int RN_PAIR_CAP = 704;   // >= #{(i,j): (i+1)(j+1) <= 128}

struct RnPairTable {
    int count;
    uint16_t ij[RN_PAIR_CAP];  // (i << 8) | j
};

struct RnWarpScratch {
    float beam_s[RN_KMAX];
    int beam_i[RN_KMAX];
    float dig_s[RN_KMAX];
    int dig_p[RN_KMAX];
};

__host__ __device__ inline int rn_pair_count(int K) {
    int n = 0;
    for (int i = 1; i <= K; ++i) n += K / i;
    return n;
}

// Called by every thread of the CTA; ends with a __syncthreads().
__device__ inline void rn_build_pairs(RnPairTable *tab, int K, int *row_off /* >= K+1 ints of smem */) {
    if (threadIdx.x == 0) {
        int off = 0;
        for (int i = 0; i < K; ++i) {
            row_off[i] = off;
            off += K / (i + 1);
        }
        row_off[K] = off;
        tab->count = off;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        const int n = K / (i + 1);
        const int base = row_off[i];
        for (int j = 0; j < n; ++j) tab->ij[base + j] = uint16_t((i << 8) | j);
    }
    __syncthreads();
}

template <typename T>
struct RnDigitLoader {
    const T *base;      // points at logit (u = 0, p = 0) of this token
    int64_t su, sp;     // element strides of digit and radix axes
    __device__ __forceinline__ float operator()(int u, int p) const {
        return rn_to_float<T>(base[u * su + p * sp]);
    }
};

// Result of a decode, distributed over the warp: entry e = lane*KPL + r (valid for e < K).
template <int KPL>
struct RnDecoded {
    int idx[KPL];      // content index (before CAPE)
    float val[KPL];    // positive weight (0 for inactive tokens)
};

// KPL = ceil(K / 32), PPL = ceil(P / 32), each rounded up to a power of two (1, 2 or 4).
template <int KPL, int PPL, typename Loader>
__device__ __forceinline__ RnDecoded<KPL> rn_warp_decode(const Loader &load, int U, int P, int K, float re_norm,
                                                         RnWarpScratch *ws, const RnPairTable *tab, int lane) {
    constexpr int N = 32 * KPL;
    uint64_t best[KPL];
    float lse_total = 0.f;
    bool inactive = false;
    int n_b = 0;
    int stride = 1;

    for (int u = 0; u < U; ++u) {
        // ---- load digit u, log-sum-exp, sorted list of its best min(P, K) logits ------------
        // element p lives in lane p / PPL, register p % PPL
        uint64_t dk[PPL];
        float xmax = -INFINITY;
#pragma unroll
        for (int r = 0; r < PPL; ++r) {
            const int p = lane * PPL + r;
            float x = -INFINITY;
            dk[r] = 0;
            if (p < P) {
                x = load(u, p);
                dk[r] = rn_key(x, p);
            }
            xmax = fmaxf(xmax, x);
        }
        xmax = rn_warp_max(xmax);
        if (xmax == -INFINITY) {
            inactive = true;  // the reference zeroes every logit of such a token: all scores tie
        } else {
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < PPL; ++r) {
                const int p = lane * PPL + r;
                if (p < P) s += expf(rn_key_score(dk[r]) - xmax);
            }
            s = rn_warp_sum(s);
            lse_total += xmax + logf(s);
        }
        rn_bitonic_sort_desc<PPL>(dk, lane);
#pragma unroll
        for (int r = 0; r < PPL; ++r) {
            const int e = lane * PPL + r;
            if (e < K && e < P) {
                ws->dig_s[e] = rn_key_score(dk[r]);
                ws->dig_p[e] = rn_key_index(dk[r]);
            }
        }
        const int n_d = min(P, K);
        __syncwarp();

        if (u == 0) {
            for (int e = lane; e < n_d; e += 32) {
                ws->beam_s[e] = ws->dig_s[e];
                ws->beam_i[e] = ws->dig_p[e];
            }
            n_b = n_d;
            __syncwarp();
        } else {
            // ---- candidates (i, j) with (i+1)(j+1) <= K, i < n_b, j < n_d; keep the best K ---
            const int n_pairs = tab->count;
            int n_valid = 0;
            for (int base = 0; base < n_pairs; base += N) {
                uint64_t ck[KPL];
#pragma unroll
                for (int r = 0; r < KPL; ++r) {
                    const int c = base + lane * KPL + r;
                    uint64_t key = 0;
                    if (c < n_pairs) {
                        const int ij = tab->ij[c];
                        const int i = ij >> 8, j = ij & 0xff;
                        if (i < n_b && j < n_d) {
                            key = rn_key(ws->beam_s[i] + ws->dig_s[j], ws->beam_i[i] + stride * ws->dig_p[j]);
                            ++n_valid;
                        }
                    }
                    ck[r] = key;
                }
                rn_bitonic_sort_desc<KPL>(ck, lane);
                if (base == 0) {
#pragma unroll
                    for (int r = 0; r < KPL; ++r) best[r] = ck[r];
                } else {
                    // best[e] = max(best[e], ck[N-1-e]) is bitonic and holds the N largest
#pragma unroll
                    for (int r = 0; r < KPL; ++r) {
                        const uint64_t rev = rn_shfl(ck[KPL - 1 - r], 31 - lane);
                        best[r] = best[r] > rev ? best[r] : rev;
                    }
                    rn_bitonic_merge_desc<KPL>(best, lane);
                }
            }
            n_valid = __reduce_add_sync(RN_FULL, n_valid);
            n_b = min(K, n_valid);
            __syncwarp();
#pragma unroll
            for (int r = 0; r < KPL; ++r) {
                const int e = lane * KPL + r;
                if (e < n_b) {
                    ws->beam_s[e] = rn_key_score(best[r]);
                    ws->beam_i[e] = rn_key_index(best[r]);
                }
            }
            __syncwarp();
        }
        stride *= P;
    }

    // ---- weights --------------------------------------------------------------------------
    RnDecoded<KPL> out;
    float logq[KPL];
#pragma unroll
    for (int r = 0; r < KPL; ++r) {
        const int e = lane * KPL + r;
        const bool live = e < K;
        out.idx[r] = live ? ws->beam_i[e] : 0;
        logq[r] = live ? (ws->beam_s[e] - lse_total) : -INFINITY;
    }
    if (re_norm != 0.f && !inactive) {
        const float m = __shfl_sync(RN_FULL, logq[0], 0);  // entry 0 is the largest
        if (m > -INFINITY) {
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < KPL; ++r) s += (lane * KPL + r < K) ? expf(logq[r] - m) : 0.f;
            s = rn_warp_sum(s);
            const float l = m + logf(s);
#pragma unroll
            for (int r = 0; r < KPL; ++r) logq[r] -= re_norm * l;
        }
    }
#pragma unroll
    for (int r = 0; r < KPL; ++r) {
        const int e = lane * KPL + r;
        out.val[r] = (e < K && !inactive) ? expf(logq[r]) : 0.f;
        // inactive token: every score ties, canonical order is 0, 1, 2, ...; an entry with score
        // -inf is a zero-weight no-op and reports its rank as well
        if (inactive || logq[r] == -INFINITY) out.idx[r] = e;
    }
    __syncwarp();
    return out;
}

// Stored index for a content index: CAPE shift (content - position) mod A on the first E heads.
__device__ __forceinline__ int rn_cape(int content, int shift /* pos mod A, or 0 */, int A) {
    int a = content - shift;
    return a < 0 ? a + A : a;
}
__device__ __forceinline__ int rn_pos_mod(int pos, int A) {
    int m = pos % A;
    return m < 0 ? m + A : m;
}

// Specialised thread-per-row decoder (rn_addr_fast.cu): returns 0 when it launched a kernel for
// this shape and layout, -1 when the caller should use the general warp-cooperative kernel.
int rn_addr_fwd_fast(const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides, const int32_t *pos,
                     const int64_t *pos_strides, int32_t *idx, float *val, const int64_t *out_strides, int64_t B,
                     int64_t H, int64_t U, int64_t P, int64_t T, int64_t E, int64_t A, int64_t Kw, int64_t Kr,
                     double w_re_norm, double r_re_norm, int w_neg, int r_neg, int encode_batch, cudaStream_t stream);
int rn_addr_bwd_fast(const int32_t *idx, const float *val, const int64_t *out_strides, const float *d_val,
                     const int64_t *dval_strides, const void *w_addr, const void *r_addr, int dtype,
                     const int64_t *addr_strides, const int32_t *pos, const int64_t *pos_strides, void *d_w, void *d_r,
                     const int64_t *dgrad_strides, int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E,
                     int64_t A, int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm, int w_neg, int r_neg,
                     cudaStream_t stream);
