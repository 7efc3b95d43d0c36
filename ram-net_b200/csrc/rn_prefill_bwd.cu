// Prefill backward: gradients of the gated sparse update / read w.r.t. the event weights, x,
// gamma and the initial state.  Replaces ramnet_ops::topk_segment_backward
// (packages/ramnet-ops/csrc/ram_attn_ops.cpp:267-310, kernels
//  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-416 (replay) and :418-606 (reverse)).
//
// Same time-chunk / round structure as the forward pass (rn_prefill.cuh); the chunk records are
// rebuilt by the schedule kernel (which also stores the mass each write found), then
//   replay   (one CTA per (b,h,channel slice), chunks forward):  re-runs the state, stores
//            delta = x - slot_before of every write and accumulates d_r = <slot_at_read, d_y>;
//   reverse  (same mapping, chunks and rounds backward):  carries d_slot in shared memory;
//            read:  d_slot[a] += r d_y;   write:  d_gain = <d_slot[a], delta>,
//            d_x += gain d_slot[a],  d_slot[a] *= 1 - gain;
//   scalar   (one CTA per (b,h), chunks and rounds backward):  the mass chain: d_w, d_gamma, d_mass.
// The workspaces of the sweeps are laid out per channel slice, so that a CTA streams through memory of its own:
// delta as [bh][slice][t][k][channels of the slice] and the partial dot products of a slice (d_r from the replay,
// d_gain from the reverse sweep) as [bh][slice][t][k]; a reduce kernel adds the slices (fixed order, no atomics).
#include "rn_prefill.cuh"

struct RnGsuBwdParams {
    RnGsuParams f;            // forward description (idx/val, x, gamma, mask, records, ...)
    const void *dy;           // (B,H,T,C) upstream gradient of y, dtype of x
    int64_t dyb, dyh, dyt;
    float *delta;             // workspace [(bh*nslices + slice)*T + t][Kw][cs]
    float *part;              // workspace [(bh*nslices + slice)*T + t][Kw + Kr]: d_gain (k < Kw) and d_r partial sums
    float *dgain;             // workspace [(bh*T + t)*Kw + k], written by the reduce kernel
    float *dval;              // output (B,H,Kw+Kr,T) via strides, zeroed by the caller
    int64_t vb, vh, vk, vt;
    void *dx;                 // output (B,H,T,C), dtype of x
    int64_t dxb, dxh, dxt;
    float *dgamma;            // output (B,H,T) contiguous fp32
    const float *dslot_post;  // (B,H,A,C)
    float *dslot_out;
    const float *dmass_post;  // (B,H,A)
    float *dmass_out;
    float *dmass_ws;          // global d_mass table when it does not fit shared memory (aliases dmass_out)
};

__device__ __forceinline__ float rn_group_sum(float v, int G, unsigned mask) {
    for (int off = 1; off < G; off <<= 1) v += __shfl_xor_sync(mask, v, off);
    return v;
}

// ------------------------------------------------------------------------------------------
// replay / reverse kernels: same organisation as rn_gsu_apply_fast_kernel
// ------------------------------------------------------------------------------------------
// One 1024-thread CTA per (b,h, channel slice); the slice of the slot state (replay) or of its gradient
// (reverse) stays in shared memory; the {coef, link} pairs and the chain heads of a chunk arrive by a
// 1-D bulk async copy one chunk ahead (one polling thread).  An event that is the first (replay) / the
// last (reverse) of its slot in the chunk is handled token-major, two events in flight per thread; the
// other events of a slot form a chain that one thread group walks with the row in registers, forwards
// in time in the replay and against it in the reverse sweep.
//   replay   write: delta = x - slot is stored for the reverse sweep, slot += gain * delta
//            read:  this slice's part of d_r = <slot, d_y>
//   reverse  read:  d_slot += r * d_y
//            write: this slice's part of d_gain = <d_slot, delta>, d_x += gain * d_slot, d_slot *= 1 - gain
// Every (token, k) of a chunk gets its partial dot product from exactly one thread (zero for a no-op event), so the
// partial sums need no clearing.
// MODEL: the instance for Kw = Kr = 16 with 64-token chunks (see rn_gsu_apply_fast_kernel)
template <typename T, int CS, int EV, bool REVERSE, bool MODEL = false>
__global__ void __launch_bounds__(RN_APPLY_THREADS, 1) rn_gsu_bwd_sweep_kernel(const RnGsuBwdParams bp, const int tpt_log2_) {
    constexpr int G = CS / 4;
    const RnGsuParams &p = bp.f;
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t mbar[2];

    const int slice = blockIdx.x % p.nslices;
    const int bh = blockIdx.x / p.nslices;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, lane = tid & 31;
    const int C = p.C, A = p.A;
    const int Kw = MODEL ? 16 : p.Kw, KT = MODEL ? 32 : p.Kw + p.Kr, L = MODEL ? 64 : p.L, NEp = MODEL ? 2048 : p.NEp;
    const int tpt_log2 = MODEL ? 4 : tpt_log2_;
    const int c0 = slice * CS;
    const int cvalid = min(CS, C - c0);
    const uint32_t rec_copy = uint32_t(size_t(NEp) * 9 + 16);  // {coef, link}[NEp], heads[8 + NEp/2]
    const uint32_t kt_magic = 0xffffffffu / uint32_t(KT) + 1u;  // e / KT == __umulhi(e, kt_magic) for e < 4096

    const int TPT = 1 << tpt_log2;
    const int KL = TPT / G;
    const int tok = tid >> tpt_log2;
    const int w = tid & (TPT - 1);
    const int sub = w % G, q = w / G;
    const bool chan_ok = MODEL || sub * 4 < cvalid;  // MODEL: C is a multiple of the slice width
    // is this thread's j-th event a write?  MODEL: 8 k-lanes per token, so events 0, 1 are writes and 2, 3 reads
    auto wr_of = [&](int j) { return MODEL ? (j < 2) : (q + j * KL < Kw); };
    const unsigned gmask = (G >= 32 ? 0xffffffffu : ((1u << G) - 1u)) << (lane & ~(G - 1));  // the lanes of one event

    // dynamic smem: rec[2][rec_stride] | S[A*CS] | xt[L*CS] (replay) | dyt[L*CS] | per-(token,k) rows handed from the chains
    // to the token's owners: dxlate[L*Kw*CS] (reverse: d_x parts of chain writes) or [L*Kr*CS] (replay: slot rows at chain reads)
    const size_t rec_stride = (size_t(rec_copy) + 127) / 128 * 128;
    unsigned char *rec0 = dyn;
    float *S = reinterpret_cast<float *>(dyn + 2 * rec_stride);  // slot slice (replay) or d_slot slice (reverse)
    float *xt = S + size_t(A) * CS;
    float *dyt = xt + size_t(L) * CS;
    float *dxlate = dyt + size_t(L) * CS;

    if (tid == 0) {
        rn_mbar_init(&mbar[0], 1);
        rn_mbar_init(&mbar[1], 1);
        rn_mbar_fence_init();
    }
    __syncthreads();
    // forward sweeps read the pairs / heads built for time order, the reverse sweep their mirror image
    const unsigned char *records = p.records + int64_t(bh) * p.nchunks * p.rec_bytes + RN_GSU_HDR_BYTES +
                                   size_t(NEp) * (REVERSE ? 17 : 8) + (REVERSE ? 16 : 0);
    const int first = REVERSE ? p.nchunks - 1 : 0;
    const int step = REVERSE ? -1 : 1;
    auto fetch = [&](int it, int chunk) {  // one thread; the target buffer was last read before a CTA barrier
        uint64_t *bar = &mbar[it & 1];
        rn_mbar_expect_tx(bar, rec_copy);
        rn_bulk_g2s(rec0 + (it & 1) * rec_stride, records + int64_t(chunk) * p.rec_bytes, rec_copy, bar);
    };
    auto landed = [&](int it) { return rn_mbar_wait_bounded(&mbar[it & 1], uint32_t(it >> 1) & 1u); };
    bool failed = false;
    if (tid == 0) fetch(0, first);
    {
        const float *src = (REVERSE ? bp.dslot_post : p.slot_in) + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * G; i += RN_APPLY_THREADS) {
            const int a = i / G, sg = i - a * G;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sg * 4 < cvalid) v = *reinterpret_cast<const float4 *>(src + int64_t(a) * C + sg * 4);
            *reinterpret_cast<float4 *>(S + rn_row_of_slot(uint32_t(a), A, p.row_shift) * CS + sg * 4) = v;
        }
    }
    const T *x = static_cast<const T *>(p.x) + b * p.xb + h * p.xh + c0 + sub * 4;
    const T *dy = static_cast<const T *>(bp.dy) + b * bp.dyb + h * bp.dyh + c0 + sub * 4;
    T *dx = static_cast<T *>(bp.dx) + b * bp.dxb + h * bp.dxh + c0 + sub * 4;

    auto load_row = [&](const T *base, int64_t tstride, int chunk) {  // raw bits, converted one chunk later
        const int t = chunk * L + tok;
        RnRaw4<T> v = rn_zero_raw4<T>();
        if (chunk >= 0 && chunk < p.nchunks && tok < L && t < p.T && chan_ok) v = rn_load_raw4<T>(base + int64_t(t) * tstride);
        return v;
    };
    RnRaw4<T> xnext = rn_zero_raw4<T>();
    if (!REVERSE) xnext = load_row(x, p.xt, first);
    RnRaw4<T> dynext = load_row(dy, bp.dyt, first);
    if (tid == 0 && !landed(0)) failed = true;
    if (__syncthreads_or(failed)) {
        if (tid == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
        return;
    }

    for (int it = 0; it < p.nchunks; ++it) {
        const int chunk = first + it * step;
        const int t0 = chunk * L;
        const bool tok_ok = tok < min(L, p.T - t0);
        const bool more = it + 1 < p.nchunks;
        const float4 xv = rn_cvt_raw4(xnext), dyv = rn_cvt_raw4(dynext);
        if (tid == 0 && more) fetch(it + 1, chunk + step);
        if (!REVERSE) xnext = load_row(x, p.xt, more ? chunk + step : -1);
        dynext = load_row(dy, bp.dyt, more ? chunk + step : -1);
        const unsigned char *rec = rec0 + (it & 1) * rec_stride;
        const uint2 *e_pair = reinterpret_cast<const uint2 *>(rec);
        const uint16_t *heads = reinterpret_cast<const uint16_t *>(rec + size_t(NEp) * 8);
        // this slice's rows of the workspaces: write event (t, k) at (t*Kw + k)*CS in delta, event (t, k) at t*KT + k in part
        float *dchunk = bp.delta + ((int64_t(bh) * p.nslices + slice) * p.T + t0) * Kw * CS;
        float *dtok = dchunk + int64_t(tok) * Kw * CS + sub * 4;
        float *pchunk = bp.part + ((int64_t(bh) * p.nslices + slice) * p.T + t0) * KT;
        if (REVERSE && more && tid == 32) {
            // the deltas of the chunk after this one: one contiguous piece of this slice's workspace
            const int tn = (chunk + step) * L;
            rn_bulk_prefetch_l2(bp.delta + ((int64_t(bh) * p.nslices + slice) * p.T + tn) * Kw * CS,
                                uint32_t(min(L, p.T - tn) * Kw * CS * 4));
        }

        if (q == 0 && tok < L) {
            if (!REVERSE) *reinterpret_cast<float4 *>(xt + tok * CS + sub * 4) = xv;
            *reinterpret_cast<float4 *>(dyt + tok * CS + sub * 4) = dyv;
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);  // reverse: d_x of this token
        uint32_t late = 0;                             // this thread's events that a chain handles (reverse: writes, replay: reads)
        float late_cf[EV];                             // reverse: their coefficients (the record buffer may be refilled by then)
#pragma unroll
        for (int j = 0; j < EV; ++j) late_cf[j] = 0.f;

        // ---- token-major events: records, then rows (and deltas), then arithmetic, then stores --------------
        constexpr int NB = EV < 2 ? EV : 2;
#pragma unroll
        for (int jb = 0; jb < EV; jb += NB) {
            uint2 pr[NB];
            float4 row[NB], dl[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int k = q + (jb + i) * KL;
                pr[i] = make_uint2(0u, RN_LINK_DEAD);
                if (tok_ok && (MODEL || k < KT)) pr[i] = e_pair[tok * KT + k];
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int k = q + (jb + i) * KL;
                const uint32_t kind = (pr[i].y >> RN_LINK_KIND_SHIFT) & 7u;  // bit 2: dead
                dl[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (kind < RN_KIND_HEAD) {
                    row[i] = *reinterpret_cast<const float4 *>(S + (pr[i].y & 0xffffu) * CS + sub * 4);
                    if (REVERSE && wr_of(jb + i) && chan_ok) dl[i] = *reinterpret_cast<const float4 *>(dtok + k * CS);
                } else if (kind <= RN_KIND_LATER) {
                    if (wr_of(jb + i) == REVERSE) {  // reverse: writes, replay: reads that a chain handles
                        late |= 1u << (jb + i);
                        late_cf[jb + i] = __uint_as_float(pr[i].x);
                    }
                } else if (tok_ok && (MODEL || k < KT) && sub == 0 && wr_of(jb + i) == REVERSE) {
                    pchunk[tok * KT + k] = 0.f;  // a no-op event
                }
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                if (((pr[i].y >> RN_LINK_KIND_SHIFT) & 7u) >= RN_KIND_HEAD) continue;
                const int k = q + (jb + i) * KL;
                const float cf = __uint_as_float(pr[i].x);
                float *dst = S + (pr[i].y & 0xffffu) * CS + sub * 4;
                float4 s = row[i];
                if (!REVERSE) {
                    if (wr_of(jb + i)) {
                        const float4 d = make_float4(xv.x - s.x, xv.y - s.y, xv.z - s.z, xv.w - s.w);
                        if (chan_ok) *reinterpret_cast<float4 *>(dtok + k * CS) = d;
                        s.x = fmaf(cf, d.x, s.x);
                        s.y = fmaf(cf, d.y, s.y);
                        s.z = fmaf(cf, d.z, s.z);
                        s.w = fmaf(cf, d.w, s.w);
                        *reinterpret_cast<float4 *>(dst) = s;
                    } else {
                        float dot = s.x * dyv.x + s.y * dyv.y + s.z * dyv.z + s.w * dyv.w;
                        dot = rn_group_sum(dot, G, gmask);
                        if (sub == 0) pchunk[tok * KT + k] = dot;
                    }
                } else {
                    if (!wr_of(jb + i)) {
                        s.x = fmaf(cf, dyv.x, s.x);
                        s.y = fmaf(cf, dyv.y, s.y);
                        s.z = fmaf(cf, dyv.z, s.z);
                        s.w = fmaf(cf, dyv.w, s.w);
                    } else {
                        float dot = s.x * dl[i].x + s.y * dl[i].y + s.z * dl[i].z + s.w * dl[i].w;
                        dot = rn_group_sum(dot, G, gmask);
                        if (sub == 0) pchunk[tok * KT + k] = dot;
                        acc.x = fmaf(cf, s.x, acc.x);
                        acc.y = fmaf(cf, s.y, acc.y);
                        acc.z = fmaf(cf, s.z, acc.z);
                        acc.w = fmaf(cf, s.w, acc.w);
                        const float keep = 1.f - cf;
                        s.x *= keep; s.y *= keep; s.z *= keep; s.w *= keep;
                    }
                    *reinterpret_cast<float4 *>(dst) = s;
                }
            }
        }
        __syncthreads();

        // ---- the chains of this chunk, dealt to the thread groups ----------------------------------------
        {
            const int n_heads = heads[0];
            const int csub = tid % G;
            const bool cok = csub * 4 < cvalid;
            for (int i = tid / G; i < n_heads; i += RN_APPLY_THREADS / G) {
                int e = heads[8 + i];
                uint2 pr = e_pair[e];
                float *row = S + (pr.y & 0xffffu) * CS + csub * 4;
                float4 s = *reinterpret_cast<float4 *>(row);
                for (int guard = 0; guard < RN_GSU_NE_MAX; ++guard) {
                    // the following event's record is requested before this one is applied
                    const bool more_ev = (pr.y & RN_LINK_NEXT) != 0;
                    const int en = int((pr.y >> 16) & 0xfffu);
                    uint2 pr_n = make_uint2(0u, 0u);
                    if (more_ev) pr_n = e_pair[en];
                    const int ct = int(__umulhi(uint32_t(e), kt_magic)), ck = e - ct * KT;
                    const float cf = __uint_as_float(pr.x);
                    const bool wr = ck < Kw;
                    if (!REVERSE) {
                        if (wr) {
                            const float4 xr = *reinterpret_cast<const float4 *>(xt + ct * CS + csub * 4);
                            const float4 d = make_float4(xr.x - s.x, xr.y - s.y, xr.z - s.z, xr.w - s.w);
                            if (cok) *reinterpret_cast<float4 *>(dchunk + (ct * Kw + ck) * CS + csub * 4) = d;
                            s.x = fmaf(cf, d.x, s.x);
                            s.y = fmaf(cf, d.y, s.y);
                            s.z = fmaf(cf, d.z, s.z);
                            s.w = fmaf(cf, d.w, s.w);
                        }
                        // a read hands the row as it is now to the token's owners, who take the dot product with d_y
                        // after the chains (all threads at once, instead of one by one on the chain)
                        if (!wr) *reinterpret_cast<float4 *>(dxlate + (ct * (KT - Kw) + (ck - Kw)) * CS + csub * 4) = s;
                    } else {
                        const float4 dyr = *reinterpret_cast<const float4 *>(dyt + ct * CS + csub * 4);
                        if (wr) {
                            // a write hands d_slot as it is now to the token's owners: they take the dot product with
                            // the write's delta and the d_x part after the chains, all threads at once
                            *reinterpret_cast<float4 *>(dxlate + (ct * Kw + ck) * CS + csub * 4) = s;
                            const float keep = 1.f - cf;
                            s.x *= keep; s.y *= keep; s.z *= keep; s.w *= keep;
                        } else {
                            s.x = fmaf(cf, dyr.x, s.x);
                            s.y = fmaf(cf, dyr.y, s.y);
                            s.z = fmaf(cf, dyr.z, s.z);
                            s.w = fmaf(cf, dyr.w, s.w);
                        }
                    }
                    if (!more_ev) break;
                    e = en;
                    pr = pr_n;
                }
                *reinterpret_cast<float4 *>(row) = s;
            }
        }
        // the next record (requested at the top of this step) has to be there for the next step
        if (tid == 0 && more && !landed(it + 1)) failed = true;
        if (__syncthreads_or(failed)) {
            if (tid == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
            return;
        }

        if (!REVERSE) {
            // ---- d_r of the reads that a chain handled: <row at the read, d_y>, this slice's part -----------------
#pragma unroll
            for (int j = 0; j < EV; ++j) {
                if (!(late & (1u << j))) continue;
                const int k = q + j * KL;
                const float4 v = *reinterpret_cast<const float4 *>(dxlate + (tok * (KT - Kw) + (k - Kw)) * CS + sub * 4);
                const float4 dyr = *reinterpret_cast<const float4 *>(dyt + tok * CS + sub * 4);
                float dot = v.x * dyr.x + v.y * dyr.y + v.z * dyr.z + v.w * dyr.w;
                dot = rn_group_sum(dot, G, gmask);
                if (sub == 0) pchunk[tok * KT + k] = dot;
            }
            // a token's threads share a warp: none of them goes on to overwrite the token's d_y row for the next chunk
            // while another one still reads it here
            __syncwarp();
        }
        if (REVERSE) {
            // ---- d_x: the writes that a chain handled, then combine the k-lanes ----------------------------------
#pragma unroll
            for (int j = 0; j < EV; ++j) {
                if (!(late & (1u << j))) continue;
                const int k = q + j * KL;
                const float4 v = *reinterpret_cast<const float4 *>(dxlate + (tok * Kw + k) * CS + sub * 4);  // d_slot at the write
                const float cf = late_cf[j];
                float4 dl = make_float4(0.f, 0.f, 0.f, 0.f);
                if (chan_ok) dl = *reinterpret_cast<const float4 *>(dtok + k * CS);
                float dot = v.x * dl.x + v.y * dl.y + v.z * dl.z + v.w * dl.w;
                dot = rn_group_sum(dot, G, gmask);
                if (sub == 0) pchunk[tok * KT + k] = dot;
                acc.x = fmaf(cf, v.x, acc.x);
                acc.y = fmaf(cf, v.y, acc.y);
                acc.z = fmaf(cf, v.z, acc.z);
                acc.w = fmaf(cf, v.w, acc.w);
            }
            for (int off = G; off < TPT; off <<= 1) {
                acc.x += __shfl_xor_sync(RN_FULL, acc.x, off);
                acc.y += __shfl_xor_sync(RN_FULL, acc.y, off);
                acc.z += __shfl_xor_sync(RN_FULL, acc.z, off);
                acc.w += __shfl_xor_sync(RN_FULL, acc.w, off);
            }
            if (q == 0 && tok_ok && chan_ok) rn_store4<T>(dx + int64_t(t0 + tok) * bp.dxt, acc);
        }
    }

    if (REVERSE) {
        __syncthreads();
        float *dst = bp.dslot_out + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * G; i += RN_APPLY_THREADS) {
            const int a = i / G, sg = i - a * G;
            if (sg * 4 < cvalid)
                *reinterpret_cast<float4 *>(dst + int64_t(a) * C + sg * 4) = *reinterpret_cast<const float4 *>(S + rn_row_of_slot(uint32_t(a), A, p.row_shift) * CS + sg * 4);
        }
    }
}

// ------------------------------------------------------------------------------------------
// reduce kernel: adds the channel slices' partial dot products, slice 0 first
// ------------------------------------------------------------------------------------------
// One CTA per (b,h) and 32 tokens.  d_gain of the writes goes to the compact table the scalar kernel reads, d_r of
// the reads to the caller's gradient tensor, through a shared-memory transpose because that tensor runs along time.
constexpr int RN_RED_TOKENS = 32;
constexpr int RN_RED_THREADS = 256;
__global__ void __launch_bounds__(RN_RED_THREADS) rn_gsu_bwd_reduce_kernel(const RnGsuBwdParams bp) {
    const RnGsuParams &p = bp.f;
    extern __shared__ float red_tile[];  // [Kr][RN_RED_TOKENS + 1]
    const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int t0 = blockIdx.x * RN_RED_TOKENS;
    const int nt = min(RN_RED_TOKENS, p.T - t0);
    const int Kw = p.Kw, Kr = p.Kr, KT = Kw + Kr;
    const int64_t slice_stride = int64_t(p.T) * KT;
    const float *src = bp.part + (int64_t(bh) * p.nslices * p.T + t0) * KT;
    auto put = [&](const int i, const float sum) {
        const int t = i / KT, k = i - t * KT;
        if (k < Kw) bp.dgain[(int64_t(bh) * p.T + t0 + t) * Kw + k] = sum;
        else red_tile[(k - Kw) * (RN_RED_TOKENS + 1) + t] = sum;
    };
    if (((slice_stride | (int64_t(t0) * KT) | (int64_t(nt) * KT)) & 3) == 0) {
        // four entries per thread and slice: sixteen-byte loads, all slices of an entry requested before the sum
        for (int i = threadIdx.x * 4; i < nt * KT; i += RN_RED_THREADS * 4) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int sl = 0; sl < p.nslices; ++sl) {
                const float4 v = *reinterpret_cast<const float4 *>(src + sl * slice_stride + i);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            put(i, sum.x); put(i + 1, sum.y); put(i + 2, sum.z); put(i + 3, sum.w);
        }
    } else {
        for (int i = threadIdx.x; i < nt * KT; i += RN_RED_THREADS) {
            float sum = 0.f;
#pragma unroll 8
            for (int sl = 0; sl < p.nslices; ++sl) sum += src[sl * slice_stride + i];
            put(i, sum);
        }
    }
    __syncthreads();
    float *dst = bp.dval + b * bp.vb + h * bp.vh + int64_t(t0) * bp.vt;
    for (int i = threadIdx.x; i < Kr * RN_RED_TOKENS; i += RN_RED_THREADS) {
        const int k = i / RN_RED_TOKENS, t = i - k * RN_RED_TOKENS;
        if (t < nt) dst[int64_t(Kw + k) * bp.vk + int64_t(t) * bp.vt] = red_tile[k * (RN_RED_TOKENS + 1) + t];
    }
}

// ------------------------------------------------------------------------------------------
// scalar reverse kernel: the mass chain
// ------------------------------------------------------------------------------------------
struct RnGateBwd {
    float d_w, d_gamma, d_prev_mass;
};
// Adjoint of rn_gate(): given d(loss)/d(gain) and d(loss)/d(new mass).
__device__ __forceinline__ RnGateBwd rn_gate_bwd(float d_gain, float d_mass, float w, float gamma, float prev_mass, float eps) {
    const float e = expf(-fabsf(gamma));
    const float cw = 1.f - w;
    const float inv_den = 1.f / (gamma >= 0.f ? (w + e * cw) : (cw + e * w));
    const float alpha = (gamma >= 0.f ? cw * e : cw) * inv_den;
    const float inv_new = 1.f / (fmaf(alpha, prev_mass, w) + eps);
    const float d_mass_total = d_mass - d_gain * w * inv_new * inv_new;  // via gain = w / (mass' + eps)
    const float d_alpha = prev_mass * d_mass_total;
    RnGateBwd o;
    o.d_w = inv_new * d_gain + (-e * inv_den * inv_den) * d_alpha + d_mass_total;
    o.d_gamma = -alpha * (1.f - alpha) * d_alpha;
    o.d_prev_mass = alpha * d_mass_total;
    return o;
}

template <typename T, bool SMEM_TABLE, int EPT, bool MASS_AWARE>
__global__ void __launch_bounds__(RN_SCHED_THREADS_MAX) rn_gsu_scalar_bwd_kernel(const RnGsuBwdParams bp) {
    const RnGsuParams &p = bp.f;
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float gam[RN_GSU_LMAX];
    __shared__ float tok_scale[RN_GSU_LMAX], tok_dr[RN_GSU_LMAX], tok_du[RN_GSU_LMAX];

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, NT = blockDim.x;  // the thread count and events per thread of the schedule kernel
    const int A = p.A, Kw = p.Kw, Kr = p.Kr, KT = p.Kw + p.Kr, NEp = p.NEp;
    const bool pow2 = (A & (A - 1)) == 0;

    // dynamic smem: [d_mass A] (SMEM_TABLE) | dg_term[L*Kw] | (mass-aware) rd_u, rd_r, rd_dot [L*Kr] each
    float *dmass = SMEM_TABLE ? reinterpret_cast<float *>(dyn) : bp.dmass_ws + int64_t(bh) * A;
    float *dg_term = reinterpret_cast<float *>(dyn + (SMEM_TABLE ? size_t(A) * 4 : 0));
    float *rd_u = dg_term + size_t(p.L) * Kw;
    float *rd_r = rd_u + size_t(p.L) * Kr;
    float *rd_dot = rd_r + size_t(p.L) * Kr;
    const float *src = bp.dmass_post + int64_t(bh) * A;
    for (int a = tid; a < A; a += NT)
        if (SMEM_TABLE || src != dmass) dmass[a] = src[a];

    int ev_t[EPT], ev_k[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = j * NT + tid;
        ev_t[j] = e / KT;
        ev_k[j] = e - ev_t[j] * KT;
    }
    const T *gamma = static_cast<const T *>(p.gamma) + b * p.gb + h * p.gh;
    const int64_t ibase = b * p.ib + h * p.ih;
    __syncthreads();

    // What a chunk needs from global memory is requested one chunk ahead, so that the loads are in flight during
    // the rounds of the chunk before: per event its record word, address, weight, the mass it saw and d_gain
    // (a write) or <slot, d_y> (a read of the mass-aware variant); per token gamma; the number of rounds.
    struct Ev {
        uint32_t meta;
        int raw;
        float w, m, g;
    };
    auto request = [&](const int chunk, Ev (&ev)[EPT], float &gam_r, int &rounds) {
        const int t0 = chunk * p.L;
        const int Lc = chunk >= 0 ? min(p.L, p.T - t0) : 0;
        const unsigned char *rec = p.records + (int64_t(bh) * p.nchunks + max(chunk, 0)) * p.rec_bytes;
        const uint32_t *e_meta = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES);
        rounds = chunk >= 0 ? int(*reinterpret_cast<const uint32_t *>(rec)) : 0;
        gam_r = tid < Lc ? rn_to_float<T>(gamma[(t0 + tid) * p.gt]) : 0.f;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            ev[j] = Ev{RN_EV_DEAD, 0, 0.f, 0.f, 0.f};
            const int e = j * NT + tid;
            const bool is_write = ev_k[j] < Kw;
            if (ev_t[j] < Lc && e < NEp && (is_write || MASS_AWARE)) {
                ev[j].meta = e_meta[ev_t[j] * KT + ev_k[j]];
                const int64_t o = ibase + int64_t(ev_k[j]) * p.ik + int64_t(t0 + ev_t[j]) * p.it;
                ev[j].raw = p.idx[o];
                ev[j].w = p.val[o];
                if (is_write) {
                    const int64_t wi = (int64_t(bh) * p.T + t0 + ev_t[j]) * Kw + ev_k[j];
                    ev[j].m = p.prev_mass[wi];
                    ev[j].g = bp.dgain[wi];
                } else {
                    ev[j].m = p.read_mass[(int64_t(bh) * p.T + t0 + ev_t[j]) * Kr + (ev_k[j] - Kw)];
                    ev[j].g = bp.dval[b * bp.vb + h * bp.vh + int64_t(ev_k[j]) * bp.vk + int64_t(t0 + ev_t[j]) * bp.vt];
                }
            }
        }
    };
    Ev ev_next[EPT];
    float gam_next;
    int rounds_next;
    request(p.nchunks - 1, ev_next, gam_next, rounds_next);

    for (int chunk = p.nchunks - 1; chunk >= 0; --chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);
        const int R = rounds_next;
        Ev cur[EPT];
#pragma unroll
        for (int j = 0; j < EPT; ++j) cur[j] = ev_next[j];
        if (tid < Lc) gam[tid] = gam_next;
        request(chunk - 1, ev_next, gam_next, rounds_next);
        for (int i = tid; i < Lc * Kw; i += NT) dg_term[i] = 0.f;
        if (MASS_AWARE)
            for (int i = tid; i < Lc * Kr; i += NT) rd_u[i] = rd_r[i] = rd_dot[i] = 0.f;
        __syncthreads();

        // this thread's live events: round, slot, weight, mass seen, d_gain (writes) / <slot, d_y> (reads)
        int er[EPT];
        uint32_t ea[EPT];
        float ew[EPT], em[EPT], eg[EPT];
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            er[j] = -1;
            ea[j] = 0;
            ew[j] = em[j] = eg[j] = 0.f;
            if (!(cur[j].meta & RN_EV_DEAD)) {
                er[j] = rn_ev_round(cur[j].meta);
                ea[j] = pow2 ? uint32_t(cur[j].raw & (A - 1)) : uint32_t(cur[j].raw % A);
                ew[j] = fabsf(cur[j].w);
                em[j] = cur[j].m;
                eg[j] = cur[j].g;
                if (ev_k[j] >= Kw) {
                    const int kr = ev_k[j] - Kw;
                    rd_u[ev_t[j] * Kr + kr] = ew[j] * em[j];
                    rd_r[ev_t[j] * Kr + kr] = ew[j];
                    rd_dot[ev_t[j] * Kr + kr] = eg[j];
                }
            }
        }
        __syncthreads();
        if (MASS_AWARE) {
            // y = scale * sum_k u_k slot_k,  u = r m,  scale = sum r / (sum u + eps)
            if (tid < Lc) {
                float U = 0.f, Rs = 0.f, ds = 0.f;
                for (int k = 0; k < Kr; ++k) {
                    U += rd_u[tid * Kr + k];
                    Rs += rd_r[tid * Kr + k];
                    ds += rd_u[tid * Kr + k] * rd_dot[tid * Kr + k];  // d(loss)/d(scale) = <d_y, sum_k u_k slot_k>
                }
                const float inv = 1.f / (U + p.eps);
                tok_scale[tid] = Rs * inv;
                tok_dr[tid] = ds * inv;                 // d(loss)/d(sum r)
                tok_du[tid] = -ds * Rs * inv * inv;     // d(loss)/d(sum u)
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (er[j] < 0 || ev_k[j] < Kw) continue;
                const float d_u = tok_scale[ev_t[j]] * eg[j] + tok_du[ev_t[j]];
                bp.dval[b * bp.vb + h * bp.vh + int64_t(ev_k[j]) * bp.vk + int64_t(t0 + ev_t[j]) * bp.vt] =
                    d_u * em[j] + tok_dr[ev_t[j]];
                eg[j] = d_u * ew[j];  // flows into the mass the read saw
            }
        }
        for (int r = R - 1; r >= 0; --r) {
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (er[j] != r) continue;
                if (ev_k[j] < Kw) {
                    const RnGateBwd g = rn_gate_bwd(eg[j], dmass[ea[j]], ew[j], gam[ev_t[j]], em[j], p.eps);
                    dmass[ea[j]] = g.d_prev_mass;
                    dg_term[ev_t[j] * Kw + ev_k[j]] = g.d_gamma;
                    bp.dval[b * bp.vb + h * bp.vh + int64_t(ev_k[j]) * bp.vk + int64_t(t0 + ev_t[j]) * bp.vt] = g.d_w;
                } else {
                    dmass[ea[j]] += eg[j];
                }
            }
            __syncthreads();
        }
        if (tid < Lc) {
            float s = 0.f;
            for (int k = 0; k < Kw; ++k) s += dg_term[tid * Kw + k];
            bp.dgamma[(int64_t(bh)) * p.T + t0 + tid] = s;
        }
        __syncthreads();
    }
    if (SMEM_TABLE) {
        float *dst = bp.dmass_out + int64_t(bh) * A;
        for (int a = tid; a < A; a += NT) dst[a] = dmass[a];
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct RnBwdLayout {
    size_t off_fwd, off_prev_mass, off_read_mass, off_dgain, off_part, off_delta, total;
};

static void rn_bwd_layout(const RnGsuPlan &pl, int64_t B, int64_t H, int64_t T, int64_t C, int64_t Kw, int64_t Kr,
                          RnBwdLayout *lo) {
    size_t off = 0;
    lo->off_fwd = off;
    off = rn_align(off + pl.total, 256);
    lo->off_prev_mass = off;
    off = rn_align(off + size_t(B * H * T * Kw) * 4, 256);
    lo->off_read_mass = off;
    off = rn_align(off + size_t(B * H * T * Kr) * 4, 256);
    lo->off_dgain = off;
    off = rn_align(off + size_t(B * H * T * Kw) * 4, 256);
    lo->off_part = off;
    off = rn_align(off + size_t(B * H * T * (Kw + Kr)) * size_t(pl.nslices) * 4, 256);
    lo->off_delta = off;
    off = rn_align(off + size_t(B * H * T * Kw) * size_t(pl.nslices) * size_t(pl.cs) * 4, 256);
    lo->total = off;
}

extern "C" int64_t rn_gsu_bwd_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr,
                                              int device) {
    rn_clear_error();
    RnGsuPlan pl;
    if (rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl, 1)) return -1;
    RnBwdLayout lo;
    rn_bwd_layout(pl, B, H, T, C, Kw, Kr, &lo);
    return int64_t(lo.total);
}

template <typename T, bool REVERSE>
static int rn_launch_sweep(const RnGsuBwdParams &bp, const RnGsuPlan &pl, cudaStream_t stream) {
    const int grid = bp.f.B * bp.f.H * pl.nslices;
    // records double buffered, state slice, x / d_y rows of the chunk, per-(token,k) d_x buffer of the reverse chains
    const size_t smem = 2 * rn_align(size_t(pl.NEp) * 9 + 16, 128) +
                        (size_t(bp.f.A) * pl.cs + 2 * size_t(pl.L) * pl.cs + size_t(pl.L) * (REVERSE ? bp.f.Kw : bp.f.Kr) * pl.cs) * 4;
    if (smem > 227 * 1024) {
        rn_set_error("backward sweep needs %zu bytes of shared memory", smem);
        return 1;
    }
    if (pl.cs == 8 && pl.ev == 4 && bp.f.Kw == 16 && bp.f.Kr == 16 && pl.L == 64 && pl.NEp == 2048 && pl.tpt_log2 == 4 && bp.f.C % 8 == 0) {
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_bwd_sweep_kernel<T, 8, 4, REVERSE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(smem)));
        rn_gsu_bwd_sweep_kernel<T, 8, 4, REVERSE, true><<<grid, RN_APPLY_THREADS, smem, stream>>>(bp, pl.tpt_log2);
        return 0;
    }
#define RN_CASE(CSV, EVV)                                                                                            \
    if (pl.cs == CSV && pl.ev == EVV) {                                                                               \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_bwd_sweep_kernel<T, CSV, EVV, REVERSE>,                                  \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));                       \
        rn_gsu_bwd_sweep_kernel<T, CSV, EVV, REVERSE><<<grid, RN_APPLY_THREADS, smem, stream>>>(bp, pl.tpt_log2);    \
        return 0;                                                                                                    \
    }
#define RN_CASES(CSV) RN_CASE(CSV, 1) RN_CASE(CSV, 2) RN_CASE(CSV, 4) RN_CASE(CSV, 8) RN_CASE(CSV, 16)
    RN_CASES(4) RN_CASES(8) RN_CASES(16) RN_CASES(32)
#undef RN_CASES
#undef RN_CASE
    rn_set_error("no backward kernel for %d channels per CTA, %d events per thread", pl.cs, pl.ev);
    return 1;
}

template <typename T, bool SMEM, bool MA>
static int rn_launch_scalar_bwd(const RnGsuBwdParams &bp, const RnGsuPlan &pl, size_t smem, cudaStream_t stream) {
    const int bh = bp.f.B * bp.f.H;
#define RN_CASE(E)                                                                                                   \
    if (pl.sched_ept == E) {                                                                                         \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_scalar_bwd_kernel<T, SMEM, E, MA>,                                       \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));                       \
        rn_gsu_scalar_bwd_kernel<T, SMEM, E, MA><<<bh, pl.sched_threads, smem, stream>>>(bp);                        \
        return 0;                                                                                                    \
    }
    RN_CASE(2) RN_CASE(4)
#undef RN_CASE
    rn_set_error("no scalar backward kernel for %d events per thread", pl.sched_ept);
    return 1;
}

template <typename T>
static int rn_run_bwd(const RnGsuBwdParams &bp, const RnGsuPlan &pl, int dtype, cudaStream_t stream) {
    rn_prof_reset();
    rn_prof_mark(stream);
    if (int rc = rn_gsu_launch_schedule(bp.f, pl, dtype, stream)) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    if (int rc = rn_launch_sweep<T, false>(bp, pl, stream)) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    if (int rc = rn_launch_sweep<T, true>(bp, pl, stream)) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    {
        const dim3 grid(unsigned((bp.f.T + RN_RED_TOKENS - 1) / RN_RED_TOKENS), unsigned(bp.f.B * bp.f.H));
        rn_gsu_bwd_reduce_kernel<<<grid, RN_RED_THREADS, size_t(bp.f.Kr) * (RN_RED_TOKENS + 1) * 4, stream>>>(bp);
        RN_CUDA(cudaGetLastError());
    }
    const size_t ev_smem = size_t(pl.L) * (bp.f.Kw + 3 * bp.f.Kr) * 4;
    const bool smem_table = size_t(bp.f.A) * 4 + ev_smem <= 200 * 1024;
    const size_t smem = (smem_table ? size_t(bp.f.A) * 4 : 0) + ev_smem;
    int rc;
    if (bp.f.mass_aware)
        rc = smem_table ? rn_launch_scalar_bwd<T, true, true>(bp, pl, smem, stream)
                        : rn_launch_scalar_bwd<T, false, true>(bp, pl, smem, stream);
    else
        rc = smem_table ? rn_launch_scalar_bwd<T, true, false>(bp, pl, smem, stream)
                        : rn_launch_scalar_bwd<T, false, false>(bp, pl, smem, stream);
    if (rc) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    return 0;
}

extern "C" int rn_gsu_bwd(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
                          const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
                          const uint8_t *mask, const int64_t *mask_strides, const float *slot_in, const float *mass_in,
                          const void *d_y, const int64_t *dy_strides, const float *d_slot_post, const float *d_mass_post,
                          float *d_val, const int64_t *dval_strides, void *d_x, const int64_t *dx_strides, float *d_gamma,
                          float *d_slot, float *d_mass, void *workspace, int64_t workspace_bytes, int64_t B, int64_t H,
                          int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int mass_aware, double eps, int device,
                          void *stream_) {
    rn_clear_error();
    RN_REQUIRE(idx && val && idx_strides && x && x_strides && gamma && gamma_strides && slot_in && mass_in && d_y &&
                   dy_strides && d_slot_post && d_mass_post && d_val && dval_strides && d_x && dx_strides && d_gamma &&
                   d_slot && d_mass && workspace,
               "null pointer argument");
    RN_REQUIRE(dtype == RN_F32 || dtype == RN_F16 || dtype == RN_BF16, "unsupported dtype code %d", dtype);
    RN_REQUIRE(x_strides[3] == 1 && dy_strides[3] == 1 && dx_strides[3] == 1, "Tensor x / d_y / d_x last dim must be contiguous");
    RnGsuPlan pl;
    if (int rc = rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl, 1)) return rc;
    RN_REQUIRE(pl.fast, "the backward pass needs C %% 4 == 0, A <= 65536 and a channel slice of the state that fits shared "
                        "memory (A=%lld, C=%lld)", (long long)A, (long long)C);
    const size_t esz = dtype == RN_F32 ? 4 : 2;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(d_y) | reinterpret_cast<uintptr_t>(d_x);
    RN_REQUIRE((ptrs & (4 * esz - 1)) == 0 &&
                   ((x_strides[0] | x_strides[1] | x_strides[2] | dy_strides[0] | dy_strides[1] | dy_strides[2] |
                     dx_strides[0] | dx_strides[1] | dx_strides[2]) & 3) == 0,
               "x, d_y and d_x must be aligned to 4 elements (pointer and strides)");
    RnBwdLayout lo;
    rn_bwd_layout(pl, B, H, T, C, Kw, Kr, &lo);
    RN_REQUIRE(workspace_bytes >= int64_t(lo.total), "workspace too small: %lld < %lld bytes", (long long)workspace_bytes,
               (long long)lo.total);
    RN_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);
    cudaStream_t stream = cudaStream_t(stream_);
    unsigned char *ws = static_cast<unsigned char *>(workspace);

    RnGsuBwdParams bp{};
    RnGsuParams &p = bp.f;
    p.idx = idx; p.val = val;
    p.ib = idx_strides[0]; p.ih = idx_strides[1]; p.ik = idx_strides[2]; p.it = idx_strides[3];
    p.x = x; p.xb = x_strides[0]; p.xh = x_strides[1]; p.xt = x_strides[2];
    p.gamma = gamma; p.gb = gamma_strides[0]; p.gh = gamma_strides[1]; p.gt = gamma_strides[2];
    p.mask = mask;
    if (mask) { p.mb = mask_strides[0]; p.mt = mask_strides[1]; }
    p.slot_in = slot_in; p.mass_in = mass_in;
    p.B = int(B); p.H = int(H); p.T = int(T); p.A = int(A); p.C = int(C); p.Kw = int(Kw); p.Kr = int(Kr);
    p.L = pl.L; p.nchunks = pl.nchunks; p.NE = pl.NE; p.NEp = pl.NEp;
    p.row_shift = rn_row_shift(A);
    p.mass_aware = mass_aware; p.eps = float(eps);
    unsigned char *fws = ws + lo.off_fwd;
    p.status = rn_status_word(device);
    RN_REQUIRE(p.status != nullptr, "cannot locate the status word of device %d", device);
    p.records = fws + pl.off_records;
    p.rec_bytes = pl.rec_bytes;
    p.wide = pl.wide;
    p.claim = reinterpret_cast<uint32_t *>(fws + pl.off_claim);
    p.cs = pl.cs; p.nslices = pl.nslices; p.state_in_smem = pl.state_in_smem;
    p.reverse = 1;
    p.prev_mass = reinterpret_cast<float *>(ws + lo.off_prev_mass);
    p.read_mass = mass_aware ? reinterpret_cast<float *>(ws + lo.off_read_mass) : nullptr;
    // the schedule kernel writes the final mass somewhere: d_mass doubles as that scratch before
    // the scalar kernel overwrites it with the gradient
    p.mass_out = d_mass;

    bp.dy = d_y; bp.dyb = dy_strides[0]; bp.dyh = dy_strides[1]; bp.dyt = dy_strides[2];
    bp.delta = reinterpret_cast<float *>(ws + lo.off_delta);
    bp.dgain = reinterpret_cast<float *>(ws + lo.off_dgain);
    bp.part = reinterpret_cast<float *>(ws + lo.off_part);
    bp.dval = d_val; bp.vb = dval_strides[0]; bp.vh = dval_strides[1]; bp.vk = dval_strides[2]; bp.vt = dval_strides[3];
    bp.dx = d_x; bp.dxb = dx_strides[0]; bp.dxh = dx_strides[1]; bp.dxt = dx_strides[2];
    bp.dgamma = d_gamma;
    bp.dslot_post = d_slot_post; bp.dslot_out = d_slot;
    bp.dmass_post = d_mass_post; bp.dmass_out = d_mass; bp.dmass_ws = d_mass;

    RN_REQUIRE(pl.smem_tables, "the backward pass needs the per-head mass table to fit shared memory (A=%lld)", (long long)A);

    if (dtype == RN_F32) return rn_run_bwd<float>(bp, pl, dtype, stream);
    if (dtype == RN_F16) return rn_run_bwd<__half>(bp, pl, dtype, stream);
    return rn_run_bwd<__nv_bfloat16>(bp, pl, dtype, stream);
}
