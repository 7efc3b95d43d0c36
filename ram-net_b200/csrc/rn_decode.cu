// Fused autoregressive decode step (address decode, gated update of the Kw selected slots, weighted read of
// the Kr selected slots after the update, optional head RMSNorm + sigmoid gate).  Three kernels, picked by
// shape in rn_decode_step:
//
//   rn_decode_pair_kernel  U = 2, P = 64, K = 16, 16-bit logits, C = 128 or 256: one WARP per (batch, head)
//       pair, its two halves decode the write and the read address with sixteen lanes per address; the 16
//       write rows go global -> shared -> global by 1-D bulk async copies (mbarrier, bounded wait), the 16
//       read rows by per-lane loads in flight at the same time; a CTA's warps draw pairs from a shared counter.
//   rn_decode_fast_kernel  (U,P,K) = (2,64,16), (3,32,8), (2,16,4) with 32-bit or 16-bit logits: one CTA per
//       16 pairs, four lanes per address on warps 0-3, then warp w owns pairs 2w and 2w+1; rows as above.
//   rn_decode_kernel       any U <= 8, P <= 128, K <= 128, C <= 1024: one CTA per pair, warp 0 / 1 decode the
//       write / read address, rows updated in place (128-bit accesses when C is a multiple of 4), reads
//       gathered after a CTA barrier and reduced over K in a fixed order.
//
// A read of a slot written in the same step sees the new value.  State offsets are 64-bit: B*H*A*C may
// exceed 2^31 elements.  A bounded wait that runs out is reported through the device's status word; slot
// and mass of that pair stay as they were and its output is zero.
#include "rn_addr_fast.cuh"
#include "rn_addr_half.cuh"
#include "rn_prefill.cuh"
#include "rn_gsu.cuh"

constexpr int RN_DEC_WARPS = 4;
constexpr int RN_DEC_CMAX = 1024;

struct RnDecodeParams {
    const void *w_addr, *r_addr, *x, *gamma;
    float *slot, *mass;
    const uint8_t *mask;
    const int32_t *pos;
    void *y;
    const float *norm_weight;
    const void *gate;
    const void *scale[2];  // optional (H,U) factors of the write / read logits, in the dtype of the logits
    // element strides between batch rows of w_addr / r_addr, x, gamma and the gate logits (heads are contiguous
    // inside a batch row: the inputs may be column slices of one wider projection output)
    int64_t ld_addr[2], ld_x, ld_gamma, ld_gate;
    float norm_eps;
    int B, H, U, P, C, E, A;
    int K[2];
    float re_norm[2];
    int mass_aware;
    float eps;
    int *status;  // the device's status word (rn_status_word): set when a bounded wait runs out
};

// element offset of the (b,h) row of an input whose batch rows are `ld` apart and whose heads take `per_head` each
__device__ __forceinline__ int64_t rn_in_row(const RnDecodeParams &p, const int bh, const int64_t ld, const int per_head) {
    if (ld == int64_t(p.H) * per_head) return int64_t(bh) * per_head;  // contiguous: no division on the way to the first load
    const int b = bh / p.H, h = bh - b * p.H;
    return b * ld + int64_t(h) * per_head;
}

template <typename T, int KPL, int PPL>
__global__ void __launch_bounds__(RN_DEC_WARPS * 32) rn_decode_kernel(const RnDecodeParams p) {
    extern __shared__ float dyn[];  // xs[C] | yred[4][C]
    __shared__ RnPairTable tabs[2];
    __shared__ RnWarpScratch scratch[2];
    __shared__ int row_off[RN_KMAX + 1];
    __shared__ int sel_slot[2][RN_KMAX];
    __shared__ float sel_val[2][RN_KMAX];
    __shared__ float red[RN_DEC_WARPS][2];
    __shared__ float bcast;

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int C = p.C;
    T *y = static_cast<T *>(p.y) + int64_t(bh) * C;

    if (p.mask != nullptr && p.mask[b] == 0) {
        for (int c = tid; c < C; c += blockDim.x) y[c] = rn_from_float<T>(0.f);
        return;
    }

    float *xs = dyn;
    float *yred = dyn + C;

    rn_build_pairs(&tabs[0], p.K[0], row_off);
    if (p.K[1] != p.K[0]) rn_build_pairs(&tabs[1], p.K[1], row_off);
    const RnPairTable *tab_r = (p.K[1] != p.K[0]) ? &tabs[1] : &tabs[0];

    if (warp < 2) {
        RnDigitLoader<T> load;
        load.base = static_cast<const T *>(warp == 0 ? p.w_addr : p.r_addr) + rn_in_row(p, bh, p.ld_addr[warp == 0 ? 0 : 1], p.U * p.P);
        load.su = p.P;
        load.sp = 1;
        const int K = p.K[warp];
        const RnDecoded<KPL> d =
            rn_warp_decode<KPL, PPL>(load, p.U, p.P, K, p.re_norm[warp], &scratch[warp], warp == 0 ? &tabs[0] : tab_r, lane);
        const int shift = (h < p.E) ? rn_pos_mod(p.pos[b], p.A) : 0;
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            const int e = lane * KPL + r;
            if (e < K) {
                sel_slot[warp][e] = rn_cape(d.idx[r], shift, p.A);
                sel_val[warp][e] = d.val[r];
            }
        }
    } else {
        const T *x = static_cast<const T *>(p.x) + rn_in_row(p, bh, p.ld_x, C);
        for (int c = tid - 64; c < C; c += 64) xs[c] = rn_to_float<T>(x[c]);
    }
    for (int c = tid; c < RN_DEC_WARPS * C; c += blockDim.x) yred[c] = 0.f;
    __syncthreads();

    const float gamma = rn_to_float<T>(static_cast<const T *>(p.gamma)[rn_in_row(p, bh, p.ld_gamma, 1)]);
    float *slot = p.slot + int64_t(bh) * p.A * C;
    float *mass = p.mass + int64_t(bh) * p.A;
    const bool vec4 = (C & 3) == 0;

    // ---- write: gated update of the selected rows ---------------------------------------------
    for (int k = warp; k < p.K[0]; k += RN_DEC_WARPS) {
        const float w = sel_val[0][k];
        if (w == 0.f) continue;
        const int a = sel_slot[0][k];
        const RnGate g = rn_gate(w, gamma, mass[a], p.eps);
        float *row = slot + int64_t(a) * C;
        if (vec4) {
            for (int c = lane * 4; c < C; c += 128) {
                float4 s = *reinterpret_cast<float4 *>(row + c);
                const float4 xv = *reinterpret_cast<const float4 *>(xs + c);
                s.x = fmaf(g.gain, xv.x - s.x, s.x);
                s.y = fmaf(g.gain, xv.y - s.y, s.y);
                s.z = fmaf(g.gain, xv.z - s.z, s.z);
                s.w = fmaf(g.gain, xv.w - s.w, s.w);
                *reinterpret_cast<float4 *>(row + c) = s;
            }
        } else {
            for (int c = lane; c < C; c += 32) row[c] = fmaf(g.gain, xs[c] - row[c], row[c]);
        }
        __syncwarp();
        if (lane == 0) mass[a] = g.mass;
    }
    __syncthreads();

    // ---- read: weighted sum of the selected rows (after this step's writes) --------------------
    float sum_r = 0.f, sum_rm = 0.f;
    float *acc = yred + warp * C;
    for (int k = warp; k < p.K[1]; k += RN_DEC_WARPS) {
        const float r = sel_val[1][k];
        if (r == 0.f) continue;
        const int a = sel_slot[1][k];
        float coef = r;
        if (p.mass_aware) {
            coef = r * mass[a];
            sum_r += r;
            sum_rm += coef;
        }
        const float *row = slot + int64_t(a) * C;
        if (vec4) {
            for (int c = lane * 4; c < C; c += 128) {
                const float4 s = *reinterpret_cast<const float4 *>(row + c);
                float4 o = *reinterpret_cast<float4 *>(acc + c);
                o.x = fmaf(coef, s.x, o.x);
                o.y = fmaf(coef, s.y, o.y);
                o.z = fmaf(coef, s.z, o.z);
                o.w = fmaf(coef, s.w, o.w);
                *reinterpret_cast<float4 *>(acc + c) = o;
            }
        } else {
            for (int c = lane; c < C; c += 32) acc[c] = fmaf(coef, row[c], acc[c]);
        }
    }
    if (lane == 0) {
        red[warp][0] = sum_r;
        red[warp][1] = sum_rm;
    }
    __syncthreads();

    float scale = 1.f;
    if (p.mass_aware) {
        float sr = 0.f, srm = 0.f;
        for (int w = 0; w < RN_DEC_WARPS; ++w) {
            sr += red[w][0];
            srm += red[w][1];
        }
        scale = sr / (srm + p.eps);
    }
    const bool epilogue = p.norm_weight != nullptr || p.gate != nullptr;
    float sq = 0.f;
    for (int c = tid; c < C; c += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < RN_DEC_WARPS; ++w) v += yred[w * C + c];
        v *= scale;
        if (epilogue) {
            yred[c] = v;  // column c is owned by this thread in every pass
            sq += v * v;
        } else {
            y[c] = rn_from_float<T>(v);
        }
    }
    if (!epilogue) return;

    float inv_rms = 1.f;
    if (p.norm_weight != nullptr) {
        sq = rn_warp_sum(sq);
        __syncthreads();  // red[] is reused
        if (lane == 0) red[warp][0] = sq;
        __syncthreads();
        if (tid == 0) {
            float s = 0.f;
            for (int w = 0; w < RN_DEC_WARPS; ++w) s += red[w][0];
            bcast = rsqrtf(s / float(C) + p.norm_eps);
        }
        __syncthreads();
        inv_rms = bcast;
    }
    const T *gate = p.gate ? static_cast<const T *>(p.gate) + rn_in_row(p, bh, p.ld_gate, C) : nullptr;
    for (int c = tid; c < C; c += blockDim.x) {
        float v = yred[c];
        if (p.norm_weight != nullptr) v = v * inv_rms * p.norm_weight[c];
        if (gate != nullptr) v = v / (1.f + expf(-rn_to_float<T>(gate[c])));
        y[c] = rn_from_float<T>(v);
    }
}

// ------------------------------------------------------------------------------------------
// specialised decode step: 16 (b,h) pairs per CTA
// ------------------------------------------------------------------------------------------
// Warps 0-3 decode the 32 addresses of the CTA (16 pairs x write/read logits), four lanes per
// address, with the register-resident sorting networks of rn_addr_fast.cuh: a warp instruction
// serves 8 addresses and the dependent chain of one address is short enough to hide behind the
// row traffic of the other resident CTA.  Then warp w owns pairs 2w and 2w+1.  The K write rows of
// a pair travel by 1-D bulk async copies: global -> this warp's shared-memory buffer (one mbarrier
// per warp, bounded wait), update in shared memory, shared -> global.  Random 512-byte rows fetched
// this way reach about twice the bandwidth of per-lane loads, whose outstanding requests per SM run
// out first.  The K read rows are loaded into registers at the same time; a read row that is also a
// write row of this step is taken from the updated copy in shared memory instead.
constexpr int RN_DECF_PAIRS = 16;
constexpr int RN_DECF_THREADS = 256;

template <typename T, int U, int P, int K, int NV>
__global__ void __launch_bounds__(RN_DECF_THREADS, 2) rn_decode_fast_kernel(const RnDecodeParams p) {
    extern __shared__ __align__(128) unsigned char row_bytes_buf[];  // per warp: K rows of C floats
    __shared__ int sel_slot[RN_DECF_PAIRS][2][K];
    __shared__ float sel_val[RN_DECF_PAIRS][2][K];
    __shared__ __align__(8) uint64_t mbar[RN_DECF_THREADS / 32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int BH = p.B * p.H;
    const int bh0 = blockIdx.x * RN_DECF_PAIRS;
    const int C = p.C;
    constexpr uint32_t ROW_BYTES = NV * 512;
    float *wbuf = reinterpret_cast<float *>(row_bytes_buf) + size_t(warp) * K * (NV * 128);
    if (lane == 0) {
        rn_mbar_init(&mbar[warp], 1);
        rn_mbar_fence_init();
    }

    if (warp < 4) {
        // four lanes per address: 32 addresses (16 pairs x write/read) on warps 0-3
        const int group = tid >> 2, gl = tid & 3;
        const int pair = group & 15, which = group >> 4;
        const int bh = min(bh0 + pair, BH - 1);  // surplus groups redo the last pair and discard it
        const int b = bh / p.H, h = bh % p.H;
        const T *src = static_cast<const T *>(which ? p.r_addr : p.w_addr) + rn_in_row(p, bh, p.ld_addr[which ? 1 : 0], U * P);
        int content[K];
        float weight[K];
        rn_fast::quad_decode<T, U, P, K>(src, p.re_norm[which], gl, content, weight);
        if (gl == 0 && bh0 + pair < BH) {
            const int shift = (h < p.E) ? rn_pos_mod(p.pos[b], p.A) : 0;
#pragma unroll
            for (int e = 0; e < K; ++e) {
                sel_slot[pair][which][e] = rn_cape(content[e], shift, p.A);
                sel_val[pair][which][e] = weight[e];
            }
        }
    }
    __syncthreads();

    uint32_t phase = 0;  // parity of this warp's mbarrier
#pragma unroll 1
    for (int pp = 0; pp < 2; ++pp) {
        const int pair = warp * 2 + pp;
        const int bh = bh0 + pair;
        if (bh >= BH) break;
        const int b = bh / p.H;
        T *y = static_cast<T *>(p.y) + int64_t(bh) * C;
        if (p.mask != nullptr && p.mask[b] == 0) {
#pragma unroll
            for (int v = 0; v < NV; ++v) rn_store4<T>(y + v * 128 + lane * 4, make_float4(0.f, 0.f, 0.f, 0.f));
            continue;
        }
        float *slot = p.slot + int64_t(bh) * p.A * C;
        float *mass = p.mass + int64_t(bh) * p.A;
        const float gamma = rn_to_float<T>(static_cast<const T *>(p.gamma)[rn_in_row(p, bh, p.ld_gamma, 1)]);
        float4 xv[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) xv[v] = rn_load4<T>(static_cast<const T *>(p.x) + rn_in_row(p, bh, p.ld_x, C) + v * 128 + lane * 4);

        // ---- write rows: bulk copies into this warp's buffer -------------------------------------------
        const int a_l = lane < K ? sel_slot[pair][0][lane] : 0;
        const float w_l = lane < K ? sel_val[pair][0][lane] : 0.f;
        const bool live_w = lane < K && w_l != 0.f;
        const int nlive = __popc(__ballot_sync(RN_FULL, live_w));
        if (nlive > 0) {
            if (lane == 0) rn_mbar_expect_tx(&mbar[warp], uint32_t(nlive) * ROW_BYTES);
            __syncwarp();
            if (live_w) rn_bulk_g2s(wbuf + lane * (NV * 128), slot + int64_t(a_l) * C, ROW_BYTES, &mbar[warp]);
        }

        // ---- read rows: per-lane loads into registers, in flight together with the bulk copies -------------
        const int ar_l = lane < K ? sel_slot[pair][1][lane] : 0;
        float r_l = lane < K ? sel_val[pair][1][lane] : 0.f;
        float4 rows[K][NV];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int a = __shfl_sync(RN_FULL, ar_l, k);
#pragma unroll
            for (int v = 0; v < NV; ++v) rows[k][v] = *reinterpret_cast<const float4 *>(slot + int64_t(a) * C + v * 128 + lane * 4);
        }
        // a read row that this step also writes: index of that write row, else -1
        int alias_l = -1;
#pragma unroll
        for (int j = 0; j < K; ++j) {
            const int aw = __shfl_sync(RN_FULL, a_l, j);
            const float ww = __shfl_sync(RN_FULL, w_l, j);
            if (ww != 0.f && aw == ar_l) alias_l = j;
        }
        float gain_l = 0.f, mass_new = 0.f;
        if (live_w) {
            const RnGate g = rn_gate(w_l, gamma, mass[a_l], p.eps);
            gain_l = g.gain;
            mass_new = g.mass;
        }
        __syncwarp();

        bool landed = true;
        if (nlive > 0) {
            landed = rn_mbar_wait_bounded(&mbar[warp], phase);
            phase ^= 1u;
        }
        if (!__all_sync(RN_FULL, landed)) {
            // A bulk copy never completed: report it through the status word, leave slot AND mass of this
            // pair as they were, give the pairs this warp still owns a defined (zero) output and stop using
            // the buffer (the copy may still land).
            if (lane == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
            for (int rest = pp; rest < 2 && bh0 + warp * 2 + rest < BH; ++rest) {
                T *yr = static_cast<T *>(p.y) + int64_t(bh0 + warp * 2 + rest) * C;
#pragma unroll
                for (int v = 0; v < NV; ++v) rn_store4<T>(yr + v * 128 + lane * 4, make_float4(0.f, 0.f, 0.f, 0.f));
            }
            break;
        }
        if (live_w) mass[a_l] = mass_new;  // only once the rows are here: slot and mass move together
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const float w = __shfl_sync(RN_FULL, w_l, k);
            const float gain = __shfl_sync(RN_FULL, gain_l, k);
            if (w != 0.f) {
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    float4 *cell = reinterpret_cast<float4 *>(wbuf + k * (NV * 128) + v * 128 + lane * 4);
                    float4 s = *cell;
                    s.x = fmaf(gain, xv[v].x - s.x, s.x);
                    s.y = fmaf(gain, xv[v].y - s.y, s.y);
                    s.z = fmaf(gain, xv[v].z - s.z, s.z);
                    s.w = fmaf(gain, xv[v].w - s.w, s.w);
                    *cell = s;
                }
            }
        }
        rn_fence_proxy_async();  // the updated rows are read by the bulk copy engine next
        __syncwarp();
        if (live_w) rn_bulk_s2g(slot + int64_t(a_l) * C, wbuf + lane * (NV * 128), ROW_BYTES);
        rn_bulk_commit();

        // ---- reads (after the writes of this step) ---------------------------------------------------
        float4 acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        float scale = 1.f;
        {
            if (p.mass_aware) {
                const float rm = (lane < K && r_l != 0.f) ? r_l * mass[ar_l] : 0.f;
                const float sr = rn_warp_sum(lane < K ? r_l : 0.f), srm = rn_warp_sum(rm);
                scale = sr / (srm + p.eps);
                r_l = rm;
            }
#pragma unroll
            for (int k = K - 1; k >= 0; --k) {
                const float coef = __shfl_sync(RN_FULL, r_l, k);
                const int al = __shfl_sync(RN_FULL, alias_l, k);
                if (coef != 0.f) {
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        float4 s = rows[k][v];
                        if (al >= 0) s = *reinterpret_cast<const float4 *>(wbuf + al * (NV * 128) + v * 128 + lane * 4);
                        acc[v].x = fmaf(coef, s.x, acc[v].x);
                        acc[v].y = fmaf(coef, s.y, acc[v].y);
                        acc[v].z = fmaf(coef, s.z, acc[v].z);
                        acc[v].w = fmaf(coef, s.w, acc[v].w);
                    }
                }
            }
        }
        rn_bulk_wait_read();  // the buffer is free again once the outgoing copies have read it
        __syncwarp();
        float sq = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            acc[v].x *= scale; acc[v].y *= scale; acc[v].z *= scale; acc[v].w *= scale;
            sq += acc[v].x * acc[v].x + acc[v].y * acc[v].y + acc[v].z * acc[v].z + acc[v].w * acc[v].w;
        }
        if (p.norm_weight != nullptr) {
            const float inv_rms = rsqrtf(rn_warp_sum(sq) / float(C) + p.norm_eps);
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const float4 nw = *reinterpret_cast<const float4 *>(p.norm_weight + v * 128 + lane * 4);
                acc[v].x *= inv_rms * nw.x; acc[v].y *= inv_rms * nw.y; acc[v].z *= inv_rms * nw.z; acc[v].w *= inv_rms * nw.w;
            }
        }
        if (p.gate != nullptr) {
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const float4 gl = rn_load4<T>(static_cast<const T *>(p.gate) + rn_in_row(p, bh, p.ld_gate, C) + v * 128 + lane * 4);
                acc[v].x /= 1.f + expf(-gl.x); acc[v].y /= 1.f + expf(-gl.y);
                acc[v].z /= 1.f + expf(-gl.z); acc[v].w /= 1.f + expf(-gl.w);
            }
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) rn_store4<T>(y + v * 128 + lane * 4, acc[v]);
    }
}

// ------------------------------------------------------------------------------------------
// decode step, one warp per (b,h) pair: U = 2, P = 64, K = 16, 16-bit logits
// ------------------------------------------------------------------------------------------
// The two halves of a warp decode the write and the read address of the pair with the
// sixteen-lanes-per-row decoder (rn_addr_half.cuh; a dependent chain of ~2 us instead of ~14 us),
// then the same warp moves the rows, all by 1-D bulk async copies through its shared-memory buffer: the 16
// write rows (global -> shared, update, shared -> global), then, into the same buffer, the 16 read rows; a read
// row that is also written in this step is taken from the updated copy before the buffer is reused.  Warps are independent (no CTA barrier), so the address
// decode of some pairs overlaps the row traffic of others; a CTA's warps walk the pairs with a
// grid-wide stride.
// Warps per CTA: with C = 128 a warp needs 8 KB of shared memory (its 16 write rows) and the kernel fits 72 registers
// (the read rows stream through registers four at a time), so two CTAs of 14 warps are resident per SM: 28 warps,
// one for each of the 27.7 (b,h) pairs an SM gets at batch 256 x 16 heads, and no pair waits for a second round.
template <int NV> struct RnDecPair { static constexpr int THREADS = NV == 1 ? 448 : 256; };

template <typename T, int NV, bool EXTRA>
__device__ __forceinline__ uint32_t rn_decode_pair_task(const RnDecodeParams &p, const int bh, const int lane, const int hl,
                                                        const int which, const uint32_t cand, const uint2 (&logits)[2],
                                                        float *wbuf, uint64_t *bar, uint32_t phase);

// EXTRA: logit scales and / or strided batch rows (the plain instance carries none of that)
template <typename T, int NV, bool EXTRA>
__global__ void __launch_bounds__(RnDecPair<NV>::THREADS, 2) rn_decode_pair_kernel(const RnDecodeParams p) {
    constexpr int U = 2, P = 64, K = 16;
    constexpr int RN_DECP_THREADS = RnDecPair<NV>::THREADS;
    extern __shared__ __align__(128) unsigned char row_bytes_buf[];  // per warp: K rows of C floats
    __shared__ __align__(8) uint64_t mbar[RN_DECP_THREADS / 32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, hl = lane & 15;
    const int BH = p.B * p.H;
    constexpr int C = NV * 128;
    constexpr uint32_t ROW_BYTES = C * 4;
    float *wbuf = reinterpret_cast<float *>(row_bytes_buf) + size_t(warp) * K * C;
    if (lane == 0) {
        rn_mbar_init(&mbar[warp], 1);
        rn_mbar_fence_init();
    }
    __syncwarp();
    const uint32_t cand = rn_half::load_candidates(hl);
    const int which = lane >> 4;  // lower half: write address, upper half: read address
    uint32_t phase = 0;           // parity of this warp's mbarrier

    // This CTA's share of the pairs (equal shares, so every SM gets the same work); its warps take them
    // one by one from a counter in shared memory, whichever warp is free.
    __shared__ int next_task;
    const int first = int(int64_t(BH) * blockIdx.x / gridDim.x), last = int(int64_t(BH) * (blockIdx.x + 1) / gridDim.x);
    if (tid == 0) next_task = first + RN_DECP_THREADS / 32;
    __syncthreads();

    const T *logit_base = static_cast<const T *>(which ? p.r_addr : p.w_addr);
    uint2 logits[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
    if (first + warp < last) rn_half::load_logits<T>(logit_base + (EXTRA ? rn_in_row(p, first + warp, p.ld_addr[which], U * P) : int64_t(first + warp) * (U * P)), lane, logits);
#pragma unroll 1
    for (int bh = first + warp; bh < last;) {
        int following = 0;
        if (lane == 0) following = atomicAdd(&next_task, 1);
        following = __shfl_sync(RN_FULL, following, 0);
        // the logits of the following pair are requested now and used after this pair is done
        uint2 logits_next[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
        if (following < last) rn_half::load_logits<T>(logit_base + (EXTRA ? rn_in_row(p, following, p.ld_addr[which], U * P) : int64_t(following) * (U * P)), lane, logits_next);
        phase = rn_decode_pair_task<T, NV, EXTRA>(p, bh, lane, hl, which, cand, logits, wbuf, &mbar[warp], phase);
        if (phase & 2u) {  // a bulk copy never completed: the pair this warp had already drawn gets a zero output
            if (following < last) {
                T *yr = static_cast<T *>(p.y) + int64_t(following) * (NV * 128);
#pragma unroll
                for (int v = 0; v < NV; ++v) rn_store4<T>(yr + v * 128 + lane * 4, make_float4(0.f, 0.f, 0.f, 0.f));
            }
            break;
        }
        bh = following;
        logits[0] = logits_next[0];
        logits[1] = logits_next[1];
    }
}

// One (b,h) pair on one warp; phase bit 0 = parity of the warp's mbarrier, bit 1 = failure (returned).
template <typename T, int NV, bool EXTRA>
__device__ __forceinline__ uint32_t rn_decode_pair_task(const RnDecodeParams &p, const int bh, const int lane, const int hl,
                                                        const int which, const uint32_t cand, const uint2 (&logits)[2],
                                                        float *wbuf, uint64_t *bar, uint32_t phase) {
    constexpr int U = 2, P = 64, K = 16;
    constexpr int C = NV * 128;
    constexpr uint32_t ROW_BYTES = C * 4;
    {
        const int b = bh / p.H, h = bh % p.H;
        T *y = static_cast<T *>(p.y) + int64_t(bh) * C;
        if (p.mask != nullptr && p.mask[b] == 0) {
#pragma unroll
            for (int v = 0; v < NV; ++v) rn_store4<T>(y + v * 128 + lane * 4, make_float4(0.f, 0.f, 0.f, 0.f));
            return phase;
        }
        float *slot = p.slot + int64_t(bh) * p.A * C;
        float *mass = p.mass + int64_t(bh) * p.A;

        // inputs that do not depend on the addresses are requested first
        const float gamma = rn_to_float<T>(static_cast<const T *>(p.gamma)[(EXTRA ? rn_in_row(p, bh, p.ld_gamma, 1) : int64_t(bh) * (1))]);
        const int shift = (h < p.E) ? rn_pos_mod(p.pos[b], p.A) : 0;
        RnRaw4<T> xraw[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) xraw[v] = rn_load_raw4<T>(static_cast<const T *>(p.x) + (EXTRA ? rn_in_row(p, bh, p.ld_x, C) : int64_t(bh) * (C)) + v * 128 + lane * 4);

        // ---- both addresses of the pair --------------------------------------------------------------
        int content;
        float weight;
        uint2 scaled[2] = {logits[0], logits[1]};
        if (EXTRA && p.scale[which] != nullptr) {
            // the layer's learned scale over the temperature, one factor per (head, digit): the product is rounded
            // to the dtype of the logits, as the separate elementwise multiply of the layer code rounds it
            const T *sc = static_cast<const T *>(p.scale[which]) + h * U;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float f = rn_to_float<T>(sc[u]);
                const float4 v = rn_cvt_raw4(RnRaw4<T>{scaled[u]});
                scaled[u] = rn_pack_raw4<T>(make_float4(v.x * f, v.y * f, v.z * f, v.w * f)).v;
            }
        }
        rn_half::decode_u2p64k16<T>(scaled, p.re_norm[which], lane, cand, content, weight);
        const int my_slot = rn_cape(content, shift, p.A);
        // lanes 0-15: entry `lane` of the write address; their read entry comes from the upper half
        const int a_l = my_slot;
        const float w_l = lane < K ? weight : 0.f;
        const int ar_l = __shfl_down_sync(RN_FULL, my_slot, 16);
        float r_l = __shfl_down_sync(RN_FULL, weight, 16);
        if (lane >= K) r_l = 0.f;

        // ---- the rows, in two stages through this warp's buffer: the 16 write rows, then the 16 read rows ----
        // One loop body for both stages on purpose: it holds the only wait of the task (two separate bounded waits
        // in one task make ptxas 12.9 fail to allocate registers).
        const bool live_w = lane < K && w_l != 0.f;
        const float mass_l = live_w ? mass[a_l] : 0.f;  // requested before the row traffic
        // a read row that this step also writes: index of that write row, else -1.  All 32 lanes hold a slot
        // (lower half write, upper half read): one match finds the equal ones.
        const unsigned live_mask = __ballot_sync(RN_FULL, live_w);
        const unsigned same = __match_any_sync(RN_FULL, my_slot) & live_mask;  // live write lanes with this lane's slot
        const int alias_up = same ? __ffs(same) - 1 : -1;
        const int alias_l = __shfl_down_sync(RN_FULL, alias_up, 16);
        float gain_l = 0.f, mass_new = 0.f;
        if (live_w) {
            const RnGate g = rn_gate(w_l, gamma, mass_l, p.eps);
            gain_l = g.gain;
            mass_new = g.mass;
        }
        float4 xv[NV], acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            xv[v] = rn_cvt_raw4(xraw[v]);
            acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float scale = 1.f;
        bool want = live_w;        // this lane fetches a row in the current stage ...
        int row = a_l;             // ... this one
        float coef_l = gain_l;     // and lane k < 16 holds the coefficient of row k (gain, then read weight)
#pragma unroll 1
        for (int stage = 0; stage < 2; ++stage) {
            const unsigned rows = __ballot_sync(RN_FULL, want);
            bool landed = true;
            if (rows != 0u) {
                if (lane == 0) rn_mbar_expect_tx(bar, uint32_t(__popc(rows)) * ROW_BYTES);
                __syncwarp();
                if (want) rn_bulk_g2s(wbuf + lane * C, slot + int64_t(row) * C, ROW_BYTES, bar);
                landed = rn_mbar_wait_bounded(bar, phase & 1u);
                phase ^= 1u;
            }
            if (!__all_sync(RN_FULL, landed)) {
                // A bulk copy never completed: report it through the status word and give the pair a defined (zero)
                // output.  In the first stage slot AND mass of the pair stay as they were; in the second the state
                // is already updated and only the output is lost.  The buffer is not used again (the copy may
                // still land).
                if (lane == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
#pragma unroll
                for (int v = 0; v < NV; ++v) rn_store4<T>(y + v * 128 + lane * 4, make_float4(0.f, 0.f, 0.f, 0.f));
                return phase | 2u;
            }
            if (stage == 0) {
                if (live_w) mass[a_l] = mass_new;  // only once the rows are here: slot and mass move together
                // four rows at a time: their loads are issued before the first store (the compiler cannot reorder
                // them itself, loads and stores go to the same buffer)
#pragma unroll
                for (int k0 = 0; k0 < K; k0 += 4) {
                    float4 cur[4][NV];
                    float gain[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        gain[i] = __shfl_sync(RN_FULL, coef_l, k0 + i);
#pragma unroll
                        for (int v = 0; v < NV; ++v) cur[i][v] = *reinterpret_cast<const float4 *>(wbuf + (k0 + i) * C + v * 128 + lane * 4);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (!(rows & (1u << (k0 + i)))) continue;  // not loaded: the buffer holds stale rows there
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            float4 s = cur[i][v];
                            s.x = fmaf(gain[i], xv[v].x - s.x, s.x);
                            s.y = fmaf(gain[i], xv[v].y - s.y, s.y);
                            s.z = fmaf(gain[i], xv[v].z - s.z, s.z);
                            s.w = fmaf(gain[i], xv[v].w - s.w, s.w);
                            *reinterpret_cast<float4 *>(wbuf + (k0 + i) * C + v * 128 + lane * 4) = s;
                        }
                    }
                }
                rn_fence_proxy_async();  // the updated rows are read by the bulk copy engine next
                __syncwarp();
                if (live_w) rn_bulk_s2g(slot + int64_t(a_l) * C, wbuf + lane * C, ROW_BYTES);
                rn_bulk_commit();

                // reads come after the writes of this step
                if (p.mass_aware) {
                    const float rm = (lane < K && r_l != 0.f) ? r_l * mass[ar_l] : 0.f;
                    const float sr = rn_warp_sum(lane < K ? r_l : 0.f), srm = rn_warp_sum(rm);
                    scale = sr / (srm + p.eps);
                    r_l = rm;
                }
                // read rows that this step also wrote: from the updated copies in the buffer (rare: ~6 % of the pairs)
                const bool live_r = lane < K && r_l != 0.f;
                if (__any_sync(RN_FULL, live_r && alias_l >= 0)) {
#pragma unroll 1
                    for (int k = 0; k < K; ++k) {
                        const float coef = __shfl_sync(RN_FULL, r_l, k);
                        const int al = __shfl_sync(RN_FULL, alias_l, k);
                        if (coef != 0.f && al >= 0) {
#pragma unroll
                            for (int v = 0; v < NV; ++v) {
                                const float4 s = *reinterpret_cast<const float4 *>(wbuf + al * C + v * 128 + lane * 4);
                                acc[v].x = fmaf(coef, s.x, acc[v].x);
                                acc[v].y = fmaf(coef, s.y, acc[v].y);
                                acc[v].z = fmaf(coef, s.z, acc[v].z);
                                acc[v].w = fmaf(coef, s.w, acc[v].w);
                            }
                        }
                    }
                }
                // the other read rows come by bulk copies too (a 512-byte bulk copy moves random rows at about twice
                // the rate of per-lane loads), into the same buffer, once the outgoing copies have read it
                rn_bulk_wait_read();
                __syncwarp();
                want = live_r && alias_l < 0;
                row = ar_l;
                coef_l = r_l;
            } else {
#pragma unroll
                for (int k0 = 0; k0 < K; k0 += 4) {
                    float4 cur[4][NV];
                    float coef[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        coef[i] = __shfl_sync(RN_FULL, coef_l, k0 + i);
#pragma unroll
                        for (int v = 0; v < NV; ++v) cur[i][v] = *reinterpret_cast<const float4 *>(wbuf + (k0 + i) * C + v * 128 + lane * 4);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (!(rows & (1u << (k0 + i)))) continue;  // not fetched: the buffer holds other rows there
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            acc[v].x = fmaf(coef[i], cur[i][v].x, acc[v].x);
                            acc[v].y = fmaf(coef[i], cur[i][v].y, acc[v].y);
                            acc[v].z = fmaf(coef[i], cur[i][v].z, acc[v].z);
                            acc[v].w = fmaf(coef[i], cur[i][v].w, acc[v].w);
                        }
                    }
                }
            }
        }
        float sq = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            acc[v].x *= scale; acc[v].y *= scale; acc[v].z *= scale; acc[v].w *= scale;
            sq += acc[v].x * acc[v].x + acc[v].y * acc[v].y + acc[v].z * acc[v].z + acc[v].w * acc[v].w;
        }
        if (p.norm_weight != nullptr) {
            const float inv_rms = rsqrtf(rn_warp_sum(sq) / float(C) + p.norm_eps);
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const float4 nw = *reinterpret_cast<const float4 *>(p.norm_weight + v * 128 + lane * 4);
                acc[v].x *= inv_rms * nw.x; acc[v].y *= inv_rms * nw.y; acc[v].z *= inv_rms * nw.z; acc[v].w *= inv_rms * nw.w;
            }
        }
        if (p.gate != nullptr) {
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const float4 gl = rn_load4<T>(static_cast<const T *>(p.gate) + (EXTRA ? rn_in_row(p, bh, p.ld_gate, C) : int64_t(bh) * (C)) + v * 128 + lane * 4);
                acc[v].x /= 1.f + expf(-gl.x); acc[v].y /= 1.f + expf(-gl.y);
                acc[v].z /= 1.f + expf(-gl.z); acc[v].w /= 1.f + expf(-gl.w);
            }
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) rn_store4<T>(y + v * 128 + lane * 4, acc[v]);
        __syncwarp();  // every lane is done with the buffer before the next pair's copies are requested
    }
    return phase;
}

// 0 = launched, -1 = not this kernel's shape
template <typename T>
static int rn_launch_decode_pair(const RnDecodeParams &p, int device, cudaStream_t stream) {
    if constexpr (rn_fast::Raw<T>::wide) {
        return -1;
    } else {
        if (!(p.U == 2 && p.P == 64 && p.K[0] == 16 && p.K[1] == 16)) return -1;
        if (p.C != 128 && p.C != 256) return -1;
        const int threads = p.C == 128 ? RnDecPair<1>::THREADS : RnDecPair<2>::THREADS;
        const bool extra = p.scale[0] != nullptr || p.ld_addr[0] != int64_t(p.H) * p.U * p.P || p.ld_addr[1] != int64_t(p.H) * p.U * p.P ||
                           p.ld_x != int64_t(p.H) * p.C || p.ld_gamma != p.H || (p.gate != nullptr && p.ld_gate != int64_t(p.H) * p.C);
        const int wpc = threads / 32;
        // CTAs: enough for one warp per pair, but at least one per SM while there are pairs to hand out (a small
        // batch is spread over all SMs instead of filling a few), at most the two resident CTAs per SM
        const int sms = rn_sm_count(device), pairs = p.B * p.H;
        int grid = (pairs + wpc - 1) / wpc;
        if (grid < sms) grid = pairs < sms ? pairs : sms;
        if (grid > 2 * sms) grid = 2 * sms;
        if (p.C == 128) {
            constexpr int smem = (RnDecPair<1>::THREADS / 32) * 16 * 128 * 4;
            if (extra) {
                if (cudaFuncSetAttribute(rn_decode_pair_kernel<T, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -1;
                rn_decode_pair_kernel<T, 1, true><<<grid, threads, smem, stream>>>(p);
            } else {
                if (cudaFuncSetAttribute(rn_decode_pair_kernel<T, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -1;
                rn_decode_pair_kernel<T, 1, false><<<grid, threads, smem, stream>>>(p);
            }
        } else {
            constexpr int smem = (RnDecPair<2>::THREADS / 32) * 16 * 256 * 4;
            if (extra) {
                if (cudaFuncSetAttribute(rn_decode_pair_kernel<T, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -1;
                rn_decode_pair_kernel<T, 2, true><<<grid, threads, smem, stream>>>(p);
            } else {
                if (cudaFuncSetAttribute(rn_decode_pair_kernel<T, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -1;
                rn_decode_pair_kernel<T, 2, false><<<grid, threads, smem, stream>>>(p);
            }
        }
        return 0;
    }
}

template <typename T, int U, int P, int K>
static int rn_launch_decode_fast_c(const RnDecodeParams &p, cudaStream_t stream) {
    const int grid = (p.B * p.H + RN_DECF_PAIRS - 1) / RN_DECF_PAIRS;
    // dynamic shared memory: one buffer of K rows per warp
    if (p.C == 128) {
        constexpr int smem = (RN_DECF_THREADS / 32) * K * 128 * 4;
        if (cudaFuncSetAttribute(rn_decode_fast_kernel<T, U, P, K, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return -1;
        rn_decode_fast_kernel<T, U, P, K, 1><<<grid, RN_DECF_THREADS, smem, stream>>>(p);
    } else if (p.C == 256) {
        constexpr int smem = (RN_DECF_THREADS / 32) * K * 256 * 4;
        if (cudaFuncSetAttribute(rn_decode_fast_kernel<T, U, P, K, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return -1;
        rn_decode_fast_kernel<T, U, P, K, 2><<<grid, RN_DECF_THREADS, smem, stream>>>(p);
    } else {
        return -1;
    }
    return 0;
}

// 0 = launched, -1 = no specialised kernel for this shape
template <typename T>
static int rn_launch_decode_fast(const RnDecodeParams &p, int device, cudaStream_t stream) {
    if (p.K[0] != p.K[1]) return -1;
    const size_t esz = sizeof(T);
    const uintptr_t io = reinterpret_cast<uintptr_t>(p.w_addr) | reinterpret_cast<uintptr_t>(p.r_addr) |
                         reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y) |
                         reinterpret_cast<uintptr_t>(p.gate) | reinterpret_cast<uintptr_t>(p.norm_weight);
    if ((io & 15) != 0 || (size_t(p.U) * p.P * esz) % 16 != 0) return -1;
    if (((p.ld_addr[0] | p.ld_addr[1] | p.ld_x | p.ld_gate) * int64_t(esz)) % 16 != 0) return -1;
    if (rn_launch_decode_pair<T>(p, device, stream) == 0) return 0;
    if (p.U == 2 && p.P == 64 && p.K[0] == 16) return rn_launch_decode_fast_c<T, 2, 64, 16>(p, stream);
    if (p.U == 3 && p.P == 32 && p.K[0] == 8) return rn_launch_decode_fast_c<T, 3, 32, 8>(p, stream);
    if (p.U == 2 && p.P == 16 && p.K[0] == 4) return rn_launch_decode_fast_c<T, 2, 16, 4>(p, stream);
    return -1;
}

static int rn_per_lane_dec(int64_t n) { return n <= 32 ? 1 : (n <= 64 ? 2 : 4); }

template <typename T>
static int rn_launch_decode(const RnDecodeParams &p, int kpl, int ppl, int grid, size_t smem, cudaStream_t stream) {
#define RN_CASE(KP, PP)                                                                       \
    if (kpl == KP && ppl == PP) {                                                             \
        rn_decode_kernel<T, KP, PP><<<grid, RN_DEC_WARPS * 32, smem, stream>>>(p);            \
        return 0;                                                                             \
    }
    RN_CASE(1, 1) RN_CASE(1, 2) RN_CASE(1, 4) RN_CASE(2, 1) RN_CASE(2, 2) RN_CASE(2, 4) RN_CASE(4, 1) RN_CASE(4, 2)
    RN_CASE(4, 4)
#undef RN_CASE
    rn_set_error("no decode kernel for K-per-lane=%d, P-per-lane=%d", kpl, ppl);
    return 1;
}

extern "C" int rn_decode_step_scaled(const void *w_addr, const void *r_addr, const void *x, const void *gamma, int dtype,
                                     float *slot, float *mass, const uint8_t *mask, const int32_t *pos, void *y,
                                     const float *norm_weight, const void *gate_logits, double norm_eps,
                                     const void *w_scale, const void *r_scale, const int64_t *batch_strides, int64_t B,
                                     int64_t H, int64_t U, int64_t P, int64_t C, int64_t E, int64_t Kw, int64_t Kr,
                                     double w_re_norm, double r_re_norm, int mass_aware, double eps, int device, void *stream);

// 1 when rn_decode_step_scaled() takes logit scales for this shape (the one-warp-per-pair kernel does), else 0
extern "C" int rn_decode_scales_supported(int dtype, int64_t U, int64_t P, int64_t C, int64_t Kw, int64_t Kr) {
    return (dtype == RN_F16 || dtype == RN_BF16) && U == 2 && P == 64 && Kw == 16 && Kr == 16 && (C == 128 || C == 256);
}

extern "C" int rn_decode_step(const void *w_addr, const void *r_addr, const void *x, const void *gamma, int dtype,
                              float *slot, float *mass, const uint8_t *mask, const int32_t *pos, void *y,
                              const float *norm_weight, const void *gate_logits, double norm_eps, int64_t B, int64_t H,
                              int64_t U, int64_t P, int64_t C, int64_t E, int64_t Kw, int64_t Kr, double w_re_norm,
                              double r_re_norm, int mass_aware, double eps, int device, void *stream) {
    return rn_decode_step_scaled(w_addr, r_addr, x, gamma, dtype, slot, mass, mask, pos, y, norm_weight, gate_logits, norm_eps,
                                 nullptr, nullptr, nullptr, B, H, U, P, C, E, Kw, Kr, w_re_norm, r_re_norm, mass_aware, eps, device,
                                 stream);
}

extern "C" int rn_decode_step_scaled(const void *w_addr, const void *r_addr, const void *x, const void *gamma, int dtype,
                                     float *slot, float *mass, const uint8_t *mask, const int32_t *pos, void *y,
                                     const float *norm_weight, const void *gate_logits, double norm_eps,
                                     const void *w_scale, const void *r_scale, const int64_t *batch_strides, int64_t B,
                                     int64_t H, int64_t U, int64_t P, int64_t C, int64_t E, int64_t Kw, int64_t Kr,
                                     double w_re_norm, double r_re_norm, int mass_aware, double eps, int device, void *stream) {
    rn_clear_error();
    RN_REQUIRE((w_scale == nullptr) == (r_scale == nullptr), "give both logit scales or none");
    RN_REQUIRE(w_scale == nullptr || rn_decode_scales_supported(dtype, U, P, C, Kw, Kr),
               "logit scales are taken for 16-bit logits with U=2, P=64, K=16, C in {128, 256} only");
    RN_REQUIRE(w_addr && r_addr && x && gamma && slot && mass && pos && y, "null pointer argument");
    RN_REQUIRE(B > 0 && H > 0 && U > 0 && P > 0 && C > 0, "decode dims must be positive");
    RN_REQUIRE(U <= RN_UMAX, "Expect U <= %d but got %lld", RN_UMAX, (long long)U);
    RN_REQUIRE(P <= RN_PMAX, "Expect P <= %d but got %lld", RN_PMAX, (long long)P);
    RN_REQUIRE(C <= RN_DEC_CMAX, "Expect C <= %d but got %lld", RN_DEC_CMAX, (long long)C);
    int64_t A = 1;
    for (int64_t u = 0; u < U; ++u) {
        A *= P;
        RN_REQUIRE(A < (int64_t(1) << 30), "Address space overflow: P^U must stay below 2^30");
    }
    RN_REQUIRE(Kw > 0 && Kw <= RN_KMAX && Kw <= A, "Expect 0 < w_top_k <= min(%d, A) but got %lld", RN_KMAX, (long long)Kw);
    RN_REQUIRE(Kr > 0 && Kr <= RN_KMAX && Kr <= A, "Expect 0 < r_top_k <= min(%d, A) but got %lld", RN_KMAX, (long long)Kr);
    RN_REQUIRE(E >= 0 && E <= H, "Expect embed_num in [0, H]");
    RN_REQUIRE(w_re_norm >= 0.0 && w_re_norm <= 1.0, "w_re_norm must be in [0, 1].");
    RN_REQUIRE(r_re_norm >= 0.0 && r_re_norm <= 1.0, "r_re_norm must be in [0, 1].");
    RN_REQUIRE(dtype == RN_F32 || dtype == RN_F16 || dtype == RN_BF16, "unsupported dtype code %d", dtype);
    RN_REQUIRE(B * H < (int64_t(1) << 31), "B*H too large");
    RN_REQUIRE((reinterpret_cast<uintptr_t>(slot) & 15) == 0, "slot must be 16-byte aligned");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);

    RnDecodeParams p{};
    p.w_addr = w_addr; p.r_addr = r_addr; p.x = x; p.gamma = gamma;
    p.slot = slot; p.mass = mass; p.mask = mask; p.pos = pos; p.y = y;
    p.norm_weight = norm_weight; p.gate = gate_logits; p.norm_eps = float(norm_eps);
    p.scale[0] = w_scale; p.scale[1] = r_scale;
    p.ld_addr[0] = batch_strides ? batch_strides[0] : H * U * P;
    p.ld_addr[1] = batch_strides ? batch_strides[1] : H * U * P;
    p.ld_x = batch_strides ? batch_strides[2] : H * C;
    p.ld_gamma = batch_strides ? batch_strides[3] : H;
    p.ld_gate = batch_strides ? batch_strides[4] : H * C;
    RN_REQUIRE(p.ld_addr[0] >= H * U * P && p.ld_addr[1] >= H * U * P && p.ld_x >= H * C && p.ld_gamma >= H && p.ld_gate >= H * C,
               "a batch stride is smaller than a batch row");
    p.B = int(B); p.H = int(H); p.U = int(U); p.P = int(P); p.C = int(C); p.E = int(E); p.A = int(A);
    p.K[0] = int(Kw); p.K[1] = int(Kr);
    p.re_norm[0] = float(w_re_norm); p.re_norm[1] = float(r_re_norm);
    p.mass_aware = mass_aware; p.eps = float(eps);
    p.status = rn_status_word(device);
    RN_REQUIRE(p.status != nullptr, "cannot locate the status word of device %d", device);

    const int kpl = rn_per_lane_dec(Kw > Kr ? Kw : Kr), ppl = rn_per_lane_dec(P);
    const size_t smem = size_t(C) * (1 + RN_DEC_WARPS) * sizeof(float);
    const int grid = int(B * H);
    int rc;
    rn_prof_reset();
    rn_prof_mark(cudaStream_t(stream));
    rc = dtype == RN_F32 ? rn_launch_decode_fast<float>(p, device, cudaStream_t(stream))
         : dtype == RN_F16 ? rn_launch_decode_fast<__half>(p, device, cudaStream_t(stream))
                           : rn_launch_decode_fast<__nv_bfloat16>(p, device, cudaStream_t(stream));
    if (rc == 0) {
        RN_CUDA(cudaGetLastError());
        rn_prof_mark(cudaStream_t(stream));
        return 0;
    }
    if (dtype == RN_F32) rc = rn_launch_decode<float>(p, kpl, ppl, grid, smem, cudaStream_t(stream));
    else if (dtype == RN_F16) rc = rn_launch_decode<__half>(p, kpl, ppl, grid, smem, cudaStream_t(stream));
    else rc = rn_launch_decode<__nv_bfloat16>(p, kpl, ppl, grid, smem, cudaStream_t(stream));
    if (rc) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(cudaStream_t(stream));
    return 0;
}
