// Shared declarations of the prefill (T > 1) gated-sparse-update kernels.
//
// The sequence is cut into time chunks of L tokens.  Inside a chunk every live event (one write
// or one read of one slot) gets a ROUND number: the count of earlier live events of the same
// chunk on the same slot (writes of a token come before its reads).  Events of one round touch
// pairwise different slots, so a round is applied by all threads in parallel with no atomics;
// rounds are separated by CTA barriers.  Two kernels:
//
//   schedule (one CTA per (b,h), chunks in order):   rounds, the mass recurrence and the gain
//       of every write, the (mass-aware) coefficient of every read -> per-chunk event lists
//       sorted by round.  Channel independent, so done once per (b,h).
//   apply (one CTA per (b,h, channel slice)):   the slice [A][cs] of the slot state stays in
//       shared memory for the whole sequence; per chunk it stages the x tile, applies the
//       rounds (row update / row read into a per-(token,k) buffer), reduces the reads over k in a
//       fixed order and stores y.  Deterministic: no floating-point atomics anywhere.
#pragma once

#include "rn_common.cuh"
#include "rn_gsu.cuh"

constexpr int RN_GSU_THREADS = 256;
constexpr int RN_GSU_LMAX = 64;                   // longest time chunk
constexpr int RN_GSU_NE_MAX = 4096;               // most events per chunk (L * (Kw + Kr))
constexpr int RN_GSU_RMAX = 2 * RN_GSU_LMAX;      // most rounds in a chunk
constexpr int RN_GSU_OFFS = RN_GSU_RMAX + 4;      // per-chunk header: n_rounds, off[0 .. R+1]

constexpr uint32_t RN_EV_READ = 1u << 16;
constexpr uint32_t RN_EV_ZERO = 1u << 17;

struct RnGsuParams {
    // decoded addresses, logical (B,H,Kw+Kr,T)
    const int32_t *idx;
    const float *val;
    int64_t ib, ih, ik, it;
    // values / gamma / mask / output
    const void *x;
    int64_t xb, xh, xt;
    const void *gamma;
    int64_t gb, gh, gt;
    const uint8_t *mask;
    int64_t mb, mt;
    void *y;
    int64_t yb, yh, yt;
    // state (contiguous (B,H,A,C) / (B,H,A)); in == out for the in-place form
    const float *slot_in;
    float *slot_out;
    const float *mass_in;
    float *mass_out;
    int B, H, T, A, C, Kw, Kr, L, nchunks, NE;
    int mass_aware;
    float eps;
    // schedule workspace
    uint32_t *ev_slot;
    uint32_t *ev_meta;
    float *ev_coef;
    uint16_t *ev_offs;
    uint32_t *claim;  // global claim table (B*H*A) when the tables do not fit shared memory
    // apply kernel
    int cs;           // channels per CTA (multiple of 4)
    int nslices;
    int state_in_smem;
};

__host__ __device__ inline int rn_gsu_chunk_len(int Kw, int Kr) {
    int L = RN_GSU_NE_MAX / (Kw + Kr);
    return L > RN_GSU_LMAX ? RN_GSU_LMAX : (L < 1 ? 1 : L);
}
