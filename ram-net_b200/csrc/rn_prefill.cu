// Prefill forward: schedule + apply kernels (see rn_prefill.cuh) and the C-ABI entry points.
// Replaces gather_segment + ramnet_ops::topk_segment_forward / topk_segment_forward_
// (packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py:72-141,
//  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-416): no global sort, no
// per-event atomics into y, y written once in the I/O dtype.
#include "rn_prefill.cuh"

// ------------------------------------------------------------------------------------------
// schedule kernel: EPT events per thread live in registers across all phases of a chunk
// ------------------------------------------------------------------------------------------
template <typename T, bool SMEM_TABLES, int EPT>
__global__ void __launch_bounds__(RN_SCHED_THREADS_MAX) rn_gsu_schedule_kernel(const RnGsuParams p) {
    const int NT = blockDim.x;  // threads of this CTA: EPT * NT >= events per chunk
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float tok_scale[RN_GSU_LMAX];
    __shared__ int n_heads, n_rheads;

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int A = p.A, KT = p.Kw + p.Kr, NEp = p.NEp;
    const bool pow2 = (A & (A - 1)) == 0;

    // dynamic smem: [mass A][claim A][nxt NEp][prv NEp][last A][clen A] (SMEM_TABLES) | ev_v[NE] ev_c[NE] (mass-aware only)
    unsigned char *cur = dyn;
    float *mass;
    uint32_t *claim;
    // successor / predecessor of every event on its slot; latest event of every slot; its events after the first
    uint16_t *nxt = nullptr, *prv = nullptr, *last = nullptr, *clen = nullptr;
    if (SMEM_TABLES) {
        mass = reinterpret_cast<float *>(cur);
        cur += size_t(A) * 4;
        claim = reinterpret_cast<uint32_t *>(cur);
        cur += size_t(A) * 4;
        nxt = reinterpret_cast<uint16_t *>(cur);
        cur += size_t(NEp) * 2;
        prv = reinterpret_cast<uint16_t *>(cur);
        cur += size_t(NEp) * 2;
        last = reinterpret_cast<uint16_t *>(cur);
        cur += (size_t(A) * 2 + 15) / 16 * 16;
        clen = reinterpret_cast<uint16_t *>(cur);
        cur += (size_t(A) * 2 + 15) / 16 * 16;
    } else {
        mass = p.mass_out + int64_t(bh) * A;
        claim = p.claim + int64_t(bh) * A;
    }
    float *ev_v = reinterpret_cast<float *>(cur);
    float *ev_c = ev_v + p.NE;

    const float *mass_in = p.mass_in + int64_t(bh) * A;
    for (int a = tid; a < A; a += NT) {
        if (SMEM_TABLES || mass_in != mass) mass[a] = mass_in[a];
        claim[a] = 0xffffffffu;
    }

    // event e = j * 256 + tid  ->  (token in chunk, k); fixed for the whole kernel
    int ev_t[EPT], ev_k[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = j * NT + tid;
        ev_t[j] = e / KT;
        ev_k[j] = e - ev_t[j] * KT;
    }

    const T *gamma = static_cast<const T *>(p.gamma) + b * p.gb + h * p.gh;
    const int64_t ibase = b * p.ib + h * p.ih;

    // software pipeline: what the next chunk needs from global memory is requested while this one is resolved and
    // waits in registers: per event the raw idx / val and its token's gamma and mask byte (a warp's events share
    // few tokens, so these are broadcast loads)
    int nraw[EPT];
    float nval[EPT], ngam[EPT];
    bool nlive[EPT];
    auto prefetch = [&](int chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            nraw[j] = 0;
            nval[j] = 0.f;
            ngam[j] = 0.f;
            nlive[j] = false;
            if (chunk < p.nchunks && ev_t[j] < Lc) {
                const int64_t o = ibase + int64_t(ev_k[j]) * p.ik + int64_t(t0 + ev_t[j]) * p.it;
                nraw[j] = p.idx[o];
                nval[j] = p.val[o];
                ngam[j] = rn_to_float<T>(gamma[(t0 + ev_t[j]) * p.gt]);
                nlive[j] = p.mask ? p.mask[b * p.mb + (t0 + ev_t[j]) * p.mt] != 0 : true;
            }
        }
    };
    prefetch(0);
    __syncthreads();

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);

        // ---- this thread's events ---------------------------------------------------------------
        uint32_t ea[EPT];
        float ev[EPT], ec[EPT], em[EPT];  // slot, weight, coefficient, mass before the write
        float alpha[EPT], mnew[EPT];      // writes: forgetting factor (needs no mass: computed up front), mass after
        int er[EPT];          // round, or -1 dead (zero weight / masked token), -3 out of range
        uint32_t pend = 0;
        if (tid == 0) {
            n_heads = 0;
            n_rheads = 0;
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            er[j] = -3;
            ec[j] = 0.f;
            em[j] = 0.f;
            ea[j] = pow2 ? uint32_t(nraw[j] & (A - 1)) : uint32_t(nraw[j] % A);
            ev[j] = fabsf(nval[j]);
            mnew[j] = 0.f;
            // outside the rounds on purpose: there the lanes of a warp win at different times, and everything
            // inside is paid once per round by the whole warp
            alpha[j] = ev_k[j] < p.Kw ? rn_alpha(ev[j], ngam[j]) : 0.f;
            if (ev_t[j] < Lc) {
                const bool live = nlive[j] && ev[j] != 0.f;
                er[j] = live ? 0 : -1;
                if (live) pend |= 1u << j;
            }
            if (SMEM_TABLES && j * NT + tid < NEp) {
                nxt[j * NT + tid] = 0xffffu;
                prv[j * NT + tid] = 0xffffu;
            }
        }
        prefetch(chunk + 1);

        // ---- rounds: the earliest pending event of each slot wins, is processed and retires ----
        int R = 0;
        for (;;) {
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (pend & (1u << j)) atomicMin(&claim[ea[j]], uint32_t(j * NT + tid));
            __syncthreads();
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (!(pend & (1u << j))) continue;
                if (claim[ea[j]] == uint32_t(j * NT + tid)) {
                    if (ev_k[j] < p.Kw) {
                        em[j] = mass[ea[j]];
                        mnew[j] = fmaf(alpha[j], em[j], ev[j]);  // rn_gate(): mass' = alpha * mass + w
                        mass[ea[j]] = mnew[j];
                    } else {
                        em[j] = mass[ea[j]];
                        ec[j] = p.mass_aware ? ev[j] * em[j] : ev[j];
                    }
                    if (SMEM_TABLES) {  // link the slot's events in time order (one winner per slot and round)
                        if (R > 0) {
                            nxt[last[ea[j]]] = uint16_t(j * NT + tid);
                            prv[j * NT + tid] = last[ea[j]];
                        }
                        last[ea[j]] = uint16_t(j * NT + tid);
                        clen[ea[j]] = uint16_t(R);  // ends as the round of the slot's last event
                    }
                    er[j] = R;
                    claim[ea[j]] = 0xffffffffu;
                    pend &= ~(1u << j);
                }
            }
            ++R;
            if (!__syncthreads_or(pend != 0)) break;
        }
        // the gains of the writes, rn_gate(): gain = w / (mass' + eps)
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (er[j] >= 0 && ev_k[j] < p.Kw) ec[j] = ev[j] / (mnew[j] + p.eps);

        // ---- mass-aware reads: y_t = sum_k (r m slot) * sum r / (sum r m + eps) -------------------
        if (p.mass_aware) {
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (ev_t[j] < Lc) {
                    const int e = ev_t[j] * KT + ev_k[j];
                    ev_v[e] = er[j] >= 0 ? ev[j] : 0.f;
                    ev_c[e] = er[j] >= 0 ? ec[j] : 0.f;
                }
            }
            __syncthreads();
            if (tid < Lc) {
                float sr = 0.f, srm = 0.f;
                for (int k = p.Kw; k < KT; ++k) {
                    sr += ev_v[tid * KT + k];
                    srm += ev_c[tid * KT + k];
                }
                tok_scale[tid] = sr / (srm + p.eps);
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (ev_t[j] < Lc && ev_k[j] >= p.Kw && er[j] >= 0) ec[j] *= tok_scale[ev_t[j]];
        }

        // ---- the chunk record, in event order (coalesced) ------------------------------------------
        unsigned char *rec = p.records + (int64_t(bh) * p.nchunks + chunk) * p.rec_bytes;
        uint32_t *o_meta = reinterpret_cast<uint32_t *>(rec + RN_GSU_HDR_BYTES);
        float *o_coef = reinterpret_cast<float *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 4);
        uint2 *o_pair = reinterpret_cast<uint2 *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 8);
        uint16_t *o_heads = reinterpret_cast<uint16_t *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 16);
        uint32_t *o_slot = reinterpret_cast<uint32_t *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 17 + 16);
        if (tid == 0) reinterpret_cast<uint32_t *>(rec)[0] = uint32_t(R);
        // chain heads (the events that retired in the second claim round, er == 1) in any order: warp-aggregated append
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const bool emit = er[j] == 1;
            const unsigned act = __ballot_sync(RN_FULL, emit);
            if (act != 0u) {
                const int lane = tid & 31, leader = __ffs(act) - 1;
                int base = 0;
                if (lane == leader) base = atomicAdd(&n_heads, __popc(act));
                base = __shfl_sync(RN_FULL, base, leader);
                if (emit) o_heads[8 + base + __popc(act & ((1u << lane) - 1u))] = uint16_t(j * NT + tid);
            }
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int e = j * NT + tid;
            if (e < NEp) {
                const bool dead = er[j] < 0;
                o_meta[e] = rn_ev_pack(ea[j], dead ? 0 : er[j], dead);
                o_coef[e] = dead ? 0.f : ec[j];
                uint32_t link = RN_LINK_DEAD;
                if (!dead) {
                    const uint32_t kind = er[j] == 0 ? RN_KIND_FIRST : (er[j] == 1 ? RN_KIND_HEAD : RN_KIND_LATER);
                    link = (rn_row_of_slot(ea[j], A, p.row_shift) & 0xffffu) | (kind << RN_LINK_KIND_SHIFT);
                    const uint32_t nx = SMEM_TABLES ? nxt[e] : 0xffffu;
                    if (nx != 0xffffu) link |= RN_LINK_NEXT | (nx << 16);
                }
                o_pair[e] = make_uint2(__float_as_uint(dead ? 0.f : ec[j]), link);
                if (p.wide) o_slot[e] = ea[j];
            }
        }
        // ---- the mirror image for a sweep against time --------------------------------------------------
        if (SMEM_TABLES && p.reverse) {
            uint2 *o_rpair = reinterpret_cast<uint2 *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 17 + 16);
            uint16_t *o_rheads = reinterpret_cast<uint16_t *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 25 + 16);
            int back[EPT];  // events of the slot after this one
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                back[j] = er[j] >= 0 ? int(clen[ea[j]]) - er[j] : -1;
                const bool emit = back[j] == 1;
                const unsigned act = __ballot_sync(RN_FULL, emit);
                if (act != 0u) {
                    const int lane = tid & 31, leader = __ffs(act) - 1;
                    int base = 0;
                    if (lane == leader) base = atomicAdd(&n_rheads, __popc(act));
                    base = __shfl_sync(RN_FULL, base, leader);
                    if (emit) o_rheads[8 + base + __popc(act & ((1u << lane) - 1u))] = uint16_t(j * NT + tid);
                }
            }
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int e = j * NT + tid;
                if (e < NEp) {
                    uint32_t link = RN_LINK_DEAD;
                    if (er[j] >= 0) {
                        const uint32_t kind = back[j] == 0 ? RN_KIND_FIRST : (back[j] == 1 ? RN_KIND_HEAD : RN_KIND_LATER);
                        link = (rn_row_of_slot(ea[j], A, p.row_shift) & 0xffffu) | (kind << RN_LINK_KIND_SHIFT);
                        const uint32_t pv = prv[e];
                        if (pv != 0xffffu) link |= RN_LINK_NEXT | (pv << 16);
                    }
                    o_rpair[e] = make_uint2(__float_as_uint(er[j] >= 0 ? ec[j] : 0.f), link);
                }
            }
        }
        __syncthreads();  // n_heads / n_rheads are complete
        if (tid == 0) {
            o_heads[0] = uint16_t(n_heads);
            if (SMEM_TABLES && p.reverse)
                reinterpret_cast<uint16_t *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 25 + 16)[0] = uint16_t(n_rheads);
        }
        if (p.prev_mass != nullptr) {
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (er[j] >= 0 && ev_k[j] < p.Kw)
                    p.prev_mass[(int64_t(bh) * p.T + t0 + ev_t[j]) * p.Kw + ev_k[j]] = em[j];
        }
        if (p.read_mass != nullptr) {
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (er[j] >= 0 && ev_k[j] >= p.Kw)
                    p.read_mass[(int64_t(bh) * p.T + t0 + ev_t[j]) * p.Kr + (ev_k[j] - p.Kw)] = em[j];
        }
        __syncthreads();  // gam / tok_live of the next chunk are complete; ev_v / ev_c may be reused
    }

    if (SMEM_TABLES) {
        float *mass_out = p.mass_out + int64_t(bh) * A;
        for (int a = tid; a < A; a += NT) mass_out[a] = mass[a];
    }
}

// ------------------------------------------------------------------------------------------
// generic apply kernel: any C, state in shared or global memory, records read from global.
// Each round scans the whole record; reads go through a per-(token,k) buffer.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(RN_GSU_THREADS) rn_gsu_apply_kernel(const RnGsuParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];

    const int slice = blockIdx.x % p.nslices;
    const int bh = blockIdx.x / p.nslices;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int cs = p.cs, G = cs >> 2, C = p.C, A = p.A;
    const int c0 = slice * cs;
    const int cvalid = min(cs, C - c0);
    const int Kw = p.Kw, Kr = p.Kr, KT = Kw + Kr;

    // dynamic smem: [S A*cs] (state_in_smem) | xt[L*cs] | yk[L*Kr*cs]
    float *cur = reinterpret_cast<float *>(dyn);
    float *S;
    int64_t srow;  // row stride of S in floats
    if (p.state_in_smem) {
        S = cur;
        cur += size_t(A) * cs;
        srow = cs;
        const float *src = p.slot_in + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * cs; i += RN_GSU_THREADS) {
            const int a = i / cs, c = i - a * cs;
            S[i] = c < cvalid ? src[int64_t(a) * C + c] : 0.f;
        }
    } else {
        S = p.slot_out + int64_t(bh) * A * C + c0;  // holds the initial state already
        srow = C;
    }
    float *xt = cur;
    cur += size_t(p.L) * cs;
    float *yk = cur;
    const bool vec = p.state_in_smem || (C & 3) == 0;

    const T *x = static_cast<const T *>(p.x) + b * p.xb + h * p.xh + c0;
    T *y = static_cast<T *>(p.y) + b * p.yb + h * p.yh + c0;

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);
        const int ne = Lc * KT;
        const unsigned char *rec = p.records + (int64_t(bh) * p.nchunks + chunk) * p.rec_bytes;
        const uint32_t *e_meta = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES);
        const float *e_coef = reinterpret_cast<const float *>(rec + RN_GSU_HDR_BYTES + size_t(p.NEp) * 4);
        const uint32_t *e_slot = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES + size_t(p.NEp) * 17 + 16);
        const int R = int(*reinterpret_cast<const uint32_t *>(rec));

        for (int i = tid; i < Lc * cs; i += RN_GSU_THREADS) {
            const int t = i / cs, c = i - t * cs;
            xt[i] = c < cvalid ? rn_to_float<T>(x[int64_t(t0 + t) * p.xt + c]) : 0.f;
        }
        __syncthreads();

        for (int r = 0; r < R; ++r) {
            for (int i = tid; i < ne * G; i += RN_GSU_THREADS) {
                const int ev = i / G, sub = i - ev * G;
                if (sub * 4 >= cvalid) continue;  // channel group beyond C in the last slice: nothing to touch
                const uint32_t meta = e_meta[ev];
                const int t = ev / KT, k = ev - t * KT;
                const bool dead = (meta & RN_EV_DEAD) != 0;
                if (dead ? (r != 0 || k < Kw) : rn_ev_round(meta) != r) continue;
                float *dst = yk + (t * Kr + (k - Kw)) * cs + sub * 4;
                if (dead) {  // a no-op read contributes zero
                    dst[0] = dst[1] = dst[2] = dst[3] = 0.f;
                    continue;
                }
                const uint32_t a = p.wide ? e_slot[ev] : (meta & 0xffffu);
                const float coef = e_coef[ev];
                float *row = S + int64_t(a) * srow + sub * 4;
                if (vec) {
                    float4 s = *reinterpret_cast<float4 *>(row);
                    if (k >= Kw) {
                        s.x *= coef; s.y *= coef; s.z *= coef; s.w *= coef;
                        *reinterpret_cast<float4 *>(dst) = s;
                    } else {
                        const float4 xv = *reinterpret_cast<const float4 *>(xt + t * cs + sub * 4);
                        s.x = fmaf(coef, xv.x - s.x, s.x);
                        s.y = fmaf(coef, xv.y - s.y, s.y);
                        s.z = fmaf(coef, xv.z - s.z, s.z);
                        s.w = fmaf(coef, xv.w - s.w, s.w);
                        *reinterpret_cast<float4 *>(row) = s;
                    }
                } else {
                    const int nc = min(4, cvalid - sub * 4);
                    for (int j = 0; j < nc; ++j) {
                        if (k >= Kw) dst[j] = coef * row[j];
                        else row[j] = fmaf(coef, xt[t * cs + sub * 4 + j] - row[j], row[j]);
                    }
                }
            }
            __syncthreads();
        }

        // ---- y[t] = sum_k yk[t][k], fixed order ------------------------------------------------
        for (int i = tid; i < Lc * G; i += RN_GSU_THREADS) {
            const int t = i / G, sub = i - t * G;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const float *src = yk + t * Kr * cs + sub * 4;
            for (int k = 0; k < Kr; ++k) {
                const float4 v = *reinterpret_cast<const float4 *>(src + k * cs);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            T *dst = y + int64_t(t0 + t) * p.yt + sub * 4;
            const int nc = cvalid - sub * 4;
            if (nc > 0) dst[0] = rn_from_float<T>(acc.x);
            if (nc > 1) dst[1] = rn_from_float<T>(acc.y);
            if (nc > 2) dst[2] = rn_from_float<T>(acc.z);
            if (nc > 3) dst[3] = rn_from_float<T>(acc.w);
        }
        __syncthreads();
    }

    if (p.state_in_smem) {
        float *dst = p.slot_out + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * cs; i += RN_GSU_THREADS) {
            const int a = i / cs, c = i - a * cs;
            if (c < cvalid) dst[int64_t(a) * C + c] = S[i];
        }
    }
}

// ------------------------------------------------------------------------------------------
// fast apply kernel: C % 4 == 0, A <= 65536; slice state + streamed chunk records in shared memory.
//
// The first event of every slot in a chunk (~80 % of the events) is applied token-major: the CTA's
// threads are split into one group per token; thread (q, sub) of a group owns the events k = q,
// q + KL, ... of that token for the 4 channels sub*4 .. sub*4+3, with x[t] in registers and the
// token's output accumulating in registers.  First events touch pairwise different slots, so a
// thread requests the records and then the rows of all its events before it uses any of them.
// The later events of a slot form a chain (link words of the record); the chains of a chunk are
// dealt evenly to the thread groups from the record's head list, a group walks its chain with the
// row in registers, and the reads of a chain go through a per-(token,k) buffer to the token's
// owners.  Two CTA barriers per chunk; the records are double buffered by 1-D bulk copies and only
// one thread polls the copy's mbarrier.
// ------------------------------------------------------------------------------------------
// MODEL: the instance for Kw = Kr = 16 with 64-token chunks (2048 events, 16 threads per token): these are then
// compile-time constants, so the index arithmetic of the event loops folds into shifts.
template <typename T, int CS, int EV, bool MODEL = false>
__global__ void __launch_bounds__(RN_APPLY_THREADS, 1) rn_gsu_apply_fast_kernel(const RnGsuParams p, const int tpt_log2_) {
    constexpr int G = CS / 4;  // threads per event (one float4 of channels each)
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t mbar[2];

    const int slice = blockIdx.x % p.nslices;
    const int bh = blockIdx.x / p.nslices;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int C = p.C, A = p.A;
    const int Kw = MODEL ? 16 : p.Kw, Kr = MODEL ? 16 : p.Kr, KT = MODEL ? 32 : p.Kw + p.Kr, L = MODEL ? 64 : p.L;
    const int NEp = MODEL ? 2048 : p.NEp;
    const int tpt_log2 = MODEL ? 4 : tpt_log2_;
    const int c0 = slice * CS;
    const int cvalid = min(CS, C - c0);  // multiple of 4
    const uint32_t rec_copy = uint32_t(size_t(NEp) * 9 + 16);  // {coef, link}[NEp], heads[8 + NEp/2]
    const uint32_t kt_magic = 0xffffffffu / uint32_t(KT) + 1u;  // e / KT == __umulhi(e, kt_magic) for e < 4096

    // thread -> (token of the chunk, k-lane, channel group)
    const int TPT = 1 << tpt_log2;          // threads per token (8, 16 or 32: a group never leaves its warp)
    const int KL = TPT / G;                 // k-lanes per token
    const int tok = tid >> tpt_log2;        // tokens >= L (surplus threads) take no token-major work
    const int w = tid & (TPT - 1);
    const int sub = w % G, q = w / G;
    const bool chan_ok = MODEL || sub * 4 < cvalid;  // MODEL: C is a multiple of the slice width
    // is this thread's j-th event a write?  MODEL: 8 k-lanes per token, so events 0, 1 are writes and 2, 3 reads
    auto wr_of = [&](int j) { return MODEL ? (j < 2) : (q + j * KL < Kw); };

    // dynamic smem: rec[2][rec_stride] | S[A*CS] | xt[L*CS] | ylate[L*Kr*CS]
    const size_t rec_stride = (size_t(rec_copy) + 127) / 128 * 128;
    unsigned char *rec0 = dyn;
    float *S = reinterpret_cast<float *>(dyn + 2 * rec_stride);
    float *xt = S + size_t(A) * CS;
    float *ylate = xt + size_t(L) * CS;

    if (tid == 0) {
        rn_mbar_init(&mbar[0], 1);
        rn_mbar_init(&mbar[1], 1);
        rn_mbar_fence_init();
    }
    __syncthreads();
    // the part of a chunk record this kernel reads: the {coef, link} pairs and the head list, contiguous
    const unsigned char *records = p.records + int64_t(bh) * p.nchunks * p.rec_bytes + RN_GSU_HDR_BYTES + size_t(NEp) * 8;
    auto fetch = [&](int chunk) {  // one thread; the target buffer was last read before a CTA barrier
        uint64_t *bar = &mbar[chunk & 1];
        rn_mbar_expect_tx(bar, rec_copy);
        rn_bulk_g2s(rec0 + (chunk & 1) * rec_stride, records + int64_t(chunk) * p.rec_bytes, rec_copy, bar);
    };
    auto landed = [&](int chunk) {  // one thread: bounded wait for the copy of a chunk's record
        return rn_mbar_wait_bounded(&mbar[chunk & 1], uint32_t(chunk >> 1) & 1u);
    };
    bool failed = false;
    if (tid == 0) fetch(0);

    // state slice -> shared memory
    {
        const float *src = p.slot_in + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * G; i += RN_APPLY_THREADS) {
            const int a = i / G, sg = i - a * G;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sg * 4 < cvalid) v = *reinterpret_cast<const float4 *>(src + int64_t(a) * C + sg * 4);
            *reinterpret_cast<float4 *>(S + rn_row_of_slot(uint32_t(a), A, p.row_shift) * CS + sg * 4) = v;
        }
    }
    const T *x = static_cast<const T *>(p.x) + b * p.xb + h * p.xh + c0 + sub * 4;
    T *y = static_cast<T *>(p.y) + b * p.yb + h * p.yh + c0 + sub * 4;

    auto load_x = [&](int chunk) {  // raw bits: converted one chunk later, when the load has long landed
        const int t = chunk * L + tok;
        RnRaw4<T> v = rn_zero_raw4<T>();
        if (chunk < p.nchunks && tok < L && t < p.T && chan_ok) v = rn_load_raw4<T>(x + int64_t(t) * p.xt);
        return v;
    };

    RnRaw4<T> xnext = load_x(0);
    if (tid == 0 && !landed(0)) failed = true;
    if (__syncthreads_or(failed)) {  // state and barriers are set up, the first record has landed
        if (tid == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
        return;
    }

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * L;
        const bool tok_ok = tok < min(L, p.T - t0);
        const bool has_next = chunk + 1 < p.nchunks;
        const float4 xv = rn_cvt_raw4(xnext);
        if (tid == 0 && has_next) fetch(chunk + 1);
        xnext = load_x(chunk + 1);
        const unsigned char *rec = rec0 + (chunk & 1) * rec_stride;
        const uint2 *e_pair = reinterpret_cast<const uint2 *>(rec);
        const uint16_t *heads = reinterpret_cast<const uint16_t *>(rec + size_t(NEp) * 8);

        // ---- first events, token-major: records, then rows, then arithmetic, then stores ------------------
        if (q == 0 && tok < L) *reinterpret_cast<float4 *>(xt + tok * CS + sub * 4) = xv;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t late = 0;  // this thread's reads that a chain delivers
        constexpr int NB = EV < 2 ? EV : 2;  // events in flight per thread
#pragma unroll
        for (int jb = 0; jb < EV; jb += NB) {
            uint2 pr[NB];
            float4 row[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int k = q + (jb + i) * KL;
                pr[i] = make_uint2(0u, RN_LINK_DEAD);
                if (tok_ok && (MODEL || k < KT)) pr[i] = e_pair[tok * KT + k];
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const uint32_t kind = (pr[i].y >> RN_LINK_KIND_SHIFT) & 7u;  // bit 2: dead
                if (kind < RN_KIND_HEAD) {
                    row[i] = *reinterpret_cast<const float4 *>(S + (pr[i].y & 0xffffu) * CS + sub * 4);
                } else if (kind <= RN_KIND_LATER && !wr_of(jb + i)) {
                    late |= 1u << (jb + i);
                }
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                if (((pr[i].y >> RN_LINK_KIND_SHIFT) & 7u) >= RN_KIND_HEAD) continue;
                const float cf = __uint_as_float(pr[i].x);
                if (wr_of(jb + i)) {
                    float4 s = row[i];
                    s.x = fmaf(cf, xv.x - s.x, s.x);
                    s.y = fmaf(cf, xv.y - s.y, s.y);
                    s.z = fmaf(cf, xv.z - s.z, s.z);
                    s.w = fmaf(cf, xv.w - s.w, s.w);
                    *reinterpret_cast<float4 *>(S + (pr[i].y & 0xffffu) * CS + sub * 4) = s;
                } else {
                    acc.x = fmaf(cf, row[i].x, acc.x);
                    acc.y = fmaf(cf, row[i].y, acc.y);
                    acc.z = fmaf(cf, row[i].z, acc.z);
                    acc.w = fmaf(cf, row[i].w, acc.w);
                }
            }
        }
        __syncthreads();

        // ---- the chains of this chunk, dealt to the thread groups ----------------------------------------
        {
            const int n_heads = heads[0];
            const int csub = tid % G;
            for (int i = tid / G; i < n_heads; i += RN_APPLY_THREADS / G) {
                int e = heads[8 + i];
                uint2 pr = e_pair[e];
                float *row = S + (pr.y & 0xffffu) * CS + csub * 4;
                float4 s = *reinterpret_cast<float4 *>(row);
                bool dirty = false;
                for (int guard = 0; guard < RN_GSU_NE_MAX; ++guard) {
                    // the following event's record is requested before this one is applied
                    const bool more = (pr.y & RN_LINK_NEXT) != 0;
                    const int en = int((pr.y >> 16) & 0xfffu);
                    uint2 pr_n = make_uint2(0u, 0u);
                    if (more) pr_n = e_pair[en];
                    const float cf = __uint_as_float(pr.x);
                    const int ct = int(__umulhi(uint32_t(e), kt_magic)), ck = e - ct * KT;
                    // one instruction stream for writes and reads: the lanes of a warp hold both kinds
                    const bool wr = ck < Kw;
                    const float4 xr = *reinterpret_cast<const float4 *>(xt + ct * CS + csub * 4);
                    if (!wr)
                        *reinterpret_cast<float4 *>(ylate + (ct * Kr + (ck - Kw)) * CS + csub * 4) =
                            make_float4(cf * s.x, cf * s.y, cf * s.z, cf * s.w);
                    const float g = wr ? cf : 0.f;  // a read leaves the row as it is
                    s.x = fmaf(g, xr.x - s.x, s.x);
                    s.y = fmaf(g, xr.y - s.y, s.y);
                    s.z = fmaf(g, xr.z - s.z, s.z);
                    s.w = fmaf(g, xr.w - s.w, s.w);
                    dirty |= wr;
                    if (!more) break;
                    e = en;
                    pr = pr_n;
                }
                if (dirty) *reinterpret_cast<float4 *>(row) = s;
            }
        }
        // the next record (requested at the top of this step) has to be there for the next step
        if (tid == 0 && has_next && !landed(chunk + 1)) failed = true;
        if (__syncthreads_or(failed)) {
            if (tid == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
            return;
        }

        // ---- reads delivered by the chains, then combine the k-lanes ----------------------------------------
#pragma unroll
        for (int j = 0; j < EV; ++j) {
            if (!(late & (1u << j))) continue;
            const int k = q + j * KL;
            const float4 v = *reinterpret_cast<const float4 *>(ylate + (tok * Kr + (k - Kw)) * CS + sub * 4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (KL >= 4) {
            // transposing butterfly over the k-lanes: after two exchange levels lane (q & 3) holds one channel
            const bool b0 = (q & 1) != 0, b1 = (q & 2) != 0;
            float k0 = b0 ? acc.z : acc.x, k1 = b0 ? acc.w : acc.y;
            const float s0 = b0 ? acc.x : acc.z, s1 = b0 ? acc.y : acc.w;
            k0 += __shfl_xor_sync(RN_FULL, s0, G);
            k1 += __shfl_xor_sync(RN_FULL, s1, G);
            float r = b1 ? k1 : k0;
            r += __shfl_xor_sync(RN_FULL, b1 ? k0 : k1, 2 * G);
            for (int off = 4 * G; off < TPT; off <<= 1) r += __shfl_xor_sync(RN_FULL, r, off);
            if (q < 4 && tok_ok && chan_ok) y[int64_t(t0 + tok) * p.yt + (b0 ? 2 : 0) + (b1 ? 1 : 0)] = rn_from_float<T>(r);
        } else {
            for (int off = G; off < TPT; off <<= 1) {
                acc.x += __shfl_xor_sync(RN_FULL, acc.x, off);
                acc.y += __shfl_xor_sync(RN_FULL, acc.y, off);
                acc.z += __shfl_xor_sync(RN_FULL, acc.z, off);
                acc.w += __shfl_xor_sync(RN_FULL, acc.w, off);
            }
            if (q == 0 && tok_ok && chan_ok) rn_store4<T>(y + int64_t(t0 + tok) * p.yt, acc);
        }
    }

    __syncthreads();
    float *dst = p.slot_out + int64_t(bh) * A * C + c0;
    for (int i = tid; i < A * G; i += RN_APPLY_THREADS) {
        const int a = i / G, sg = i - a * G;
        if (sg * 4 < cvalid)
            *reinterpret_cast<float4 *>(dst + int64_t(a) * C + sg * 4) = *reinterpret_cast<const float4 *>(S + rn_row_of_slot(uint32_t(a), A, p.row_shift) * CS + sg * 4);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
constexpr size_t RN_SMEM_BUDGET = 225 * 1024;

static size_t rn_fast_smem(int64_t A, int cs, int NEp, int L, int64_t Kr) {
    const size_t rec_stride = rn_align(size_t(NEp) * 9 + 16, 128);  // {coef, link}[], heads[]; double buffered
    return 2 * rec_stride + (size_t(A) * cs + size_t(L) * cs + size_t(L) * Kr * cs) * 4;
}

// fast kernel geometry: threads / next_pow2(L) tokens; events per thread (power of two) or 0 if > 16
static int rn_fast_geometry(int threads, int L, int KT, int cs, int *tpt_log2) {
    int lp = 1;
    while (lp < L) lp <<= 1;
    int tpt = threads / lp, lg = 0;
    if (tpt > 32) tpt = 32;  // a token's group stays inside one warp; surplus threads idle
    while ((1 << lg) < tpt) ++lg;
    *tpt_log2 = lg;
    const int G = cs / 4;
    if (tpt > 32 || tpt < G) return 0;
    const int KL = tpt / G;
    const int ev = (KT + KL - 1) / KL;
    if (ev > 16) return 0;
    return ev <= 1 ? 1 : (ev <= 2 ? 2 : (ev <= 4 ? 4 : (ev <= 8 ? 8 : 16)));
}

int rn_gsu_plan(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int device,
                       RnGsuPlan *pl, int reverse) {
    RN_REQUIRE(B > 0 && H > 0 && T > 0 && A > 0 && C > 0, "prefill dims must be positive");
    RN_REQUIRE(Kw > 0 && Kw <= 128 && Kr > 0 && Kr <= 128, "Expect 0 < top_k <= 128 (got %lld, %lld)", (long long)Kw,
               (long long)Kr);
    RN_REQUIRE(A < (int64_t(1) << 30), "Address space overflow: A must stay below 2^30");
    RN_REQUIRE(B * H < (int64_t(1) << 24), "B*H too large");
    pl->L = rn_gsu_chunk_len(int(Kw), int(Kr));
    pl->nchunks = int((T + pl->L - 1) / pl->L);
    pl->NE = pl->L * int(Kw + Kr);
    pl->NEp = int(rn_align(pl->NE, 16));
    int ept = (pl->NE + RN_GSU_THREADS - 1) / RN_GSU_THREADS;
    pl->ept = ept <= 1 ? 1 : (ept <= 2 ? 2 : (ept <= 4 ? 4 : (ept <= 8 ? 8 : 16)));
    // schedule kernel: two events per thread (four when a chunk has more than 2048 events)
    pl->sched_ept = pl->NE > 2 * RN_SCHED_THREADS_MAX ? 4 : 2;
    pl->sched_threads = int(rn_align((pl->NE + pl->sched_ept - 1) / pl->sched_ept, 32));
    const size_t ev_bytes = size_t(pl->NE) * 8 + 16;  // mass-aware per-event scratch
    // mass + claim tables, the successor / predecessor links of a chunk's events, the latest event and the
    // number of later events of every slot
    const size_t table_bytes = size_t(A) * 8 + size_t(pl->NEp) * 4 + 2 * rn_align(size_t(A) * 2, 16);
    pl->smem_tables = (table_bytes + ev_bytes) <= RN_SMEM_BUDGET;
    pl->sched_smem = rn_align((pl->smem_tables ? table_bytes : 0) + ev_bytes, 16);
    pl->wide = A > 65536;
    pl->reverse = reverse && !pl->wide;
    pl->rec_bytes = int64_t(rn_align(RN_GSU_HDR_BYTES + size_t(pl->NEp) * (pl->wide ? 21 : (pl->reverse ? 26 : 17)) + 32, 128));

    // apply kernel: channels per CTA.  Largest slice that still gives two CTAs per SM of work,
    // else the smallest one (most parallelism).
    const int sms = rn_sm_count(device);
    // the fast kernels walk the per-slot event chains, which only the shared-memory schedule builds
    const bool fast_ok = !pl->wide && (C % 4) == 0 && pl->smem_tables;
    int best = 0;
    for (int cs = 4; cs <= (fast_ok ? 32 : 128); cs *= 2) {
        int lg = 0;
        if (fast_ok && (rn_fast_geometry(RN_APPLY_THREADS, pl->L, int(Kw + Kr), cs, &lg) == 0 ||
                        rn_fast_geometry(RN_SWEEP_THREADS, pl->L, int(Kw + Kr), cs, &lg) == 0))
            break;
        const size_t need = fast_ok ? rn_fast_smem(A, cs, pl->NEp, pl->L, Kr)
                                    : (size_t(A) * cs + size_t(pl->L) * cs + size_t(pl->L) * Kr * cs) * 4;
        if (need > RN_SMEM_BUDGET) break;
        const int64_t ncta = B * H * ((C + cs - 1) / cs);
        if (best == 0 || ncta >= 2 * int64_t(sms)) best = cs;
        if (cs >= C) break;
    }
    if (best) {
        pl->cs = best;
        pl->state_in_smem = 1;
        pl->fast = fast_ok;
        pl->apply_smem = fast_ok ? rn_fast_smem(A, best, pl->NEp, pl->L, Kr)
                                 : (size_t(A) * best + size_t(pl->L) * best + size_t(pl->L) * Kr * best) * 4;
        if (fast_ok) {
            pl->ev = rn_fast_geometry(RN_APPLY_THREADS, pl->L, int(Kw + Kr), best, &pl->tpt_log2);
            pl->evb = rn_fast_geometry(RN_SWEEP_THREADS, pl->L, int(Kw + Kr), best, &pl->tptb_log2);
        }
    } else {
        // slot state stays in global memory; keep the per-CTA read buffer small
        int cs = 4;
        while (cs * 2 <= 32 && cs * 2 <= C && (size_t(pl->L) * (Kr + 1) * cs * 2) * 4 <= 96 * 1024) cs *= 2;
        pl->cs = cs;
        pl->state_in_smem = 0;
        pl->fast = 0;
        pl->apply_smem = (size_t(pl->L) * cs + size_t(pl->L) * Kr * cs) * 4;
    }
    pl->nslices = int((C + pl->cs - 1) / pl->cs);

    const size_t n = size_t(B * H) * pl->nchunks;
    size_t off = 256;  // status word
    pl->off_records = off;
    off = rn_align(off + n * size_t(pl->rec_bytes), 256);
    pl->off_claim = off;
    if (!pl->smem_tables) off = rn_align(off + size_t(B * H) * A * 4, 256);
    pl->total = off;
    return 0;
}

extern "C" int64_t rn_gsu_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr,
                                          int device) {
    rn_clear_error();
    RnGsuPlan pl;
    if (rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return -1;
    return int64_t(pl.total);
}

// Which kernels a prefill call of this shape runs, for tests and benchmarks that must prove they exercise the
// same template instances: out[0] = 1 fast apply kernel / 0 general, out[1] = channels per CTA, out[2] = events
// per thread (forward), out[3] = channel slices, out[4] = chunk length, out[5] = state slice in shared memory,
// out[6] = events per thread (backward sweeps), out[7] = schedule tables in shared memory.
extern "C" int rn_gsu_plan_info(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int reverse,
                                int device, int32_t *out, int n) {
    rn_clear_error();
    RN_REQUIRE(out != nullptr && n >= 8, "out must hold at least 8 integers");
    RnGsuPlan pl{};
    if (int rc = rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl, reverse)) return rc;
    out[0] = pl.fast; out[1] = pl.cs; out[2] = pl.ev; out[3] = pl.nslices; out[4] = pl.L; out[5] = pl.state_in_smem;
    out[6] = pl.evb; out[7] = pl.smem_tables;
    return 0;
}

extern "C" int64_t rn_gsu_fwd_workspace_bytes(int dtype, int rows_aligned, int64_t B, int64_t H, int64_t T, int64_t A,
                                              int64_t C, int64_t Kw, int64_t Kr, int device) {
    rn_clear_error();
    RnGsuPlan pl;
    if (rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return -1;
    if (rows_aligned) {
        alignas(16) static const char probe[16] = {0};
        const int64_t ok_strides[4] = {8, 8, 8, 1};
        RnDeviceGuard guard(device);
        if (guard.ok && rn_gsu_owner_eligible(dtype, A, C, Kw, Kr, probe, ok_strides, probe, ok_strides) &&
            rn_gsu_owner_clusters(dtype, device) > 0)
            return 0;
    }
    return int64_t(pl.total);
}

// Which forward path rn_gsu_fwd takes for a shape: 0 general apply kernel, 1 channel-slice kernels with per-slot chains,
// 2 slot-owner cluster kernel.  rows_aligned: x / y rows start on 16-byte boundaries.
extern "C" int rn_gsu_fwd_path(int dtype, int rows_aligned, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw,
                               int64_t Kr, int device) {
    rn_clear_error();
    RnGsuPlan pl;
    if (rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return -1;
    if (rn_gsu_fwd_workspace_bytes(dtype, rows_aligned, B, H, T, A, C, Kw, Kr, device) == 0) return 2;
    return (pl.fast && rows_aligned) ? 1 : 0;
}

template <typename T, bool SMEM>
static int rn_launch_schedule(const RnGsuParams &p, const RnGsuPlan &pl, cudaStream_t stream) {
    const int bh = p.B * p.H;
#define RN_CASE(E)                                                                                              \
    if (pl.sched_ept == E) {                                                                                    \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_schedule_kernel<T, SMEM, E>,                                        \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(pl.sched_smem)));         \
        rn_gsu_schedule_kernel<T, SMEM, E><<<bh, pl.sched_threads, pl.sched_smem, stream>>>(p);                 \
        return 0;                                                                                               \
    }
    RN_CASE(2) RN_CASE(4)
#undef RN_CASE
    rn_set_error("no schedule kernel for %d events per thread", pl.sched_ept);
    return 1;
}

template <typename T>
static int rn_launch_apply_fast(const RnGsuParams &p, const RnGsuPlan &pl, cudaStream_t stream) {
    const int grid = p.B * p.H * pl.nslices;
    if (pl.cs == 8 && pl.ev == 4 && p.Kw == 16 && p.Kr == 16 && pl.L == 64 && pl.NEp == 2048 && pl.tpt_log2 == 4 && p.C % 8 == 0) {
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_apply_fast_kernel<T, 8, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(pl.apply_smem)));
        rn_gsu_apply_fast_kernel<T, 8, 4, true><<<grid, RN_APPLY_THREADS, pl.apply_smem, stream>>>(p, pl.tpt_log2);
        return 0;
    }
#define RN_CASE(CSV, EVV)                                                                                       \
    if (pl.cs == CSV && pl.ev == EVV) {                                                                         \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_apply_fast_kernel<T, CSV, EVV>,                                     \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(pl.apply_smem)));         \
        rn_gsu_apply_fast_kernel<T, CSV, EVV><<<grid, RN_APPLY_THREADS, pl.apply_smem, stream>>>(p, pl.tpt_log2); \
        return 0;                                                                                               \
    }
#define RN_CASES(CSV) RN_CASE(CSV, 1) RN_CASE(CSV, 2) RN_CASE(CSV, 4) RN_CASE(CSV, 8) RN_CASE(CSV, 16)
    RN_CASES(4) RN_CASES(8) RN_CASES(16) RN_CASES(32)
#undef RN_CASES
#undef RN_CASE
    rn_set_error("no fast apply kernel for %d channels per CTA, %d events per thread", pl.cs, pl.ev);
    return 1;
}

int rn_gsu_launch_schedule(const RnGsuParams &p, const RnGsuPlan &pl, int dtype, cudaStream_t stream) {
    if (dtype == RN_F32)
        return pl.smem_tables ? rn_launch_schedule<float, true>(p, pl, stream) : rn_launch_schedule<float, false>(p, pl, stream);
    if (dtype == RN_F16)
        return pl.smem_tables ? rn_launch_schedule<__half, true>(p, pl, stream) : rn_launch_schedule<__half, false>(p, pl, stream);
    return pl.smem_tables ? rn_launch_schedule<__nv_bfloat16, true>(p, pl, stream)
                          : rn_launch_schedule<__nv_bfloat16, false>(p, pl, stream);
}

template <typename T>
static int rn_launch_gsu(const RnGsuParams &p, const RnGsuPlan &pl, bool fast, cudaStream_t stream) {
    rn_prof_reset();
    rn_prof_mark(stream);
    if (int rc = pl.smem_tables ? rn_launch_schedule<T, true>(p, pl, stream) : rn_launch_schedule<T, false>(p, pl, stream))
        return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    if (fast) {
        if (int rc = rn_launch_apply_fast<T>(p, pl, stream)) return rc;
    } else {
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(pl.apply_smem)));
        rn_gsu_apply_kernel<T><<<p.B * p.H * pl.nslices, RN_GSU_THREADS, pl.apply_smem, stream>>>(p);
    }
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    return 0;
}

extern "C" int rn_gsu_fwd(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
                          const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
                          const uint8_t *mask, const int64_t *mask_strides, const float *slot_in, const float *mass_in,
                          float *slot_out, float *mass_out, void *y, const int64_t *y_strides, void *workspace,
                          int64_t workspace_bytes, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw,
                          int64_t Kr, int mass_aware, double eps, int device, void *stream_) {
    rn_clear_error();
    RN_REQUIRE(idx && val && idx_strides && x && x_strides && gamma && gamma_strides && slot_in && mass_in && slot_out &&
                   mass_out && y && y_strides,
               "null pointer argument");
    RN_REQUIRE(dtype == RN_F32 || dtype == RN_F16 || dtype == RN_BF16, "unsupported dtype code %d", dtype);
    RN_REQUIRE(x_strides[3] == 1 && y_strides[3] == 1, "Tensor x / y last dim must be contiguous");
    RN_REQUIRE(mask == nullptr || mask_strides != nullptr, "mask needs strides");
    RnGsuPlan pl;
    if (int rc = rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return rc;
    RN_REQUIRE((reinterpret_cast<uintptr_t>(slot_in) & 15) == 0 && (reinterpret_cast<uintptr_t>(slot_out) & 15) == 0,
               "slot state must be 16-byte aligned");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);
    cudaStream_t stream = cudaStream_t(stream_);

    // model shapes: the slot-owner kernel (one cluster per (b,h)), which needs no schedule and no workspace
    if (rn_gsu_owner_eligible(dtype, A, C, Kw, Kr, x, x_strides, y, y_strides)) {
        RnGsuParams q{};
        q.idx = idx; q.val = val;
        q.ib = idx_strides[0]; q.ih = idx_strides[1]; q.ik = idx_strides[2]; q.it = idx_strides[3];
        q.x = x; q.xb = x_strides[0]; q.xh = x_strides[1]; q.xt = x_strides[2];
        q.gamma = gamma; q.gb = gamma_strides[0]; q.gh = gamma_strides[1]; q.gt = gamma_strides[2];
        q.mask = mask;
        if (mask) { q.mb = mask_strides[0]; q.mt = mask_strides[1]; }
        q.y = y; q.yb = y_strides[0]; q.yh = y_strides[1]; q.yt = y_strides[2];
        q.slot_in = slot_in; q.slot_out = slot_out; q.mass_in = mass_in; q.mass_out = mass_out;
        q.B = int(B); q.H = int(H); q.T = int(T); q.A = int(A); q.C = int(C); q.Kw = int(Kw); q.Kr = int(Kr);
        q.mass_aware = mass_aware; q.eps = float(eps);
        q.status = rn_status_word(device);
        RN_REQUIRE(q.status != nullptr, "cannot locate the status word of device %d", device);
        rn_prof_reset();
        rn_prof_mark(stream);
        const int rc = rn_gsu_owner_launch(q, dtype, device, stream);
        if (rc == 0) {
            RN_CUDA(cudaGetLastError());
            rn_prof_mark(stream);
            return 0;
        }
        if (rc > 0) return rc;
        // rc < 0: this device cannot keep a 16-CTA cluster of that size resident; use the channel-slice kernels
    }
    RN_REQUIRE(workspace != nullptr && workspace_bytes >= int64_t(pl.total), "workspace too small: %lld < %lld bytes",
               (long long)workspace_bytes, (long long)pl.total);
    RN_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");

    RnGsuParams p{};
    p.idx = idx; p.val = val;
    p.ib = idx_strides[0]; p.ih = idx_strides[1]; p.ik = idx_strides[2]; p.it = idx_strides[3];
    p.x = x; p.xb = x_strides[0]; p.xh = x_strides[1]; p.xt = x_strides[2];
    p.gamma = gamma; p.gb = gamma_strides[0]; p.gh = gamma_strides[1]; p.gt = gamma_strides[2];
    p.mask = mask;
    if (mask) { p.mb = mask_strides[0]; p.mt = mask_strides[1]; }
    p.y = y; p.yb = y_strides[0]; p.yh = y_strides[1]; p.yt = y_strides[2];
    p.slot_in = slot_in; p.slot_out = slot_out; p.mass_in = mass_in; p.mass_out = mass_out;
    p.B = int(B); p.H = int(H); p.T = int(T); p.A = int(A); p.C = int(C); p.Kw = int(Kw); p.Kr = int(Kr);
    p.L = pl.L; p.nchunks = pl.nchunks; p.NE = pl.NE; p.NEp = pl.NEp;
    p.row_shift = rn_row_shift(A);
    p.mass_aware = mass_aware; p.eps = float(eps);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    p.status = rn_status_word(device);
    RN_REQUIRE(p.status != nullptr, "cannot locate the status word of device %d", device);
    p.records = ws + pl.off_records;
    p.rec_bytes = pl.rec_bytes;
    p.wide = pl.wide;
    p.claim = reinterpret_cast<uint32_t *>(ws + pl.off_claim);
    p.cs = pl.cs; p.nslices = pl.nslices; p.state_in_smem = pl.state_in_smem;

    // the fast apply kernel moves x / y in 4-element vectors
    const size_t esz = dtype == RN_F32 ? 4 : 2;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & (4 * esz - 1)) == 0 &&
                         ((x_strides[0] | x_strides[1] | x_strides[2] | y_strides[0] | y_strides[1] | y_strides[2]) & 3) == 0;
    const bool fast = pl.fast && aligned;

    if (!pl.state_in_smem && slot_in != slot_out)
        RN_CUDA(cudaMemcpyAsync(slot_out, slot_in, size_t(B * H * A * C) * 4, cudaMemcpyDeviceToDevice, stream));
    if (!pl.smem_tables && mass_in != mass_out)
        RN_CUDA(cudaMemcpyAsync(mass_out, mass_in, size_t(B * H * A) * 4, cudaMemcpyDeviceToDevice, stream));

    if (dtype == RN_F32) return rn_launch_gsu<float>(p, pl, fast, stream);
    if (dtype == RN_F16) return rn_launch_gsu<__half>(p, pl, fast, stream);
    return rn_launch_gsu<__nv_bfloat16>(p, pl, fast, stream);
}

// ------------------------------------------------------------------------------------------
// rn_gsu_fwd_static: the same prefill update for callers that must not allocate
// ------------------------------------------------------------------------------------------
// Some hosts of this library cannot hand over a workspace: code running inside a region where
// device allocation is forbidden or would deadlock (an allocator callback, a real-time serving
// loop that pre-sized its pools, a plugin whose host owns all device memory and exposes no
// allocator).  For them the event schedule that rn_gsu_fwd keeps in a caller workspace lives in
// one fixed array inside the library image instead.  The array is part of the module, so every
// GPU that loads the library keeps RN_STATIC_SCRATCH_BYTES of device memory until the process
// exits; that is why the limit is small.
constexpr size_t RN_STATIC_SCRATCH_BYTES = size_t(32) << 20;  // 32 MiB
static __device__ __align__(256) unsigned char rn_static_scratch[RN_STATIC_SCRATCH_BYTES];

#include <mutex>

// In host code `rn_static_scratch` is only a handle for the runtime, not a device address; the
// address the kernels need comes from cudaGetSymbolAddress, asked once per device with that
// device current.
static int rn_static_scratch_ptr(int device, void **out) {
    static std::mutex mu;
    static void *cached[64] = {nullptr};
    RN_REQUIRE(device >= 0 && device < 64, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[device] == nullptr) {
        void *ptr = nullptr;
        RN_CUDA(cudaGetSymbolAddress(&ptr, rn_static_scratch));
        RN_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address");
        cached[device] = ptr;
    }
    *out = cached[device];
    return 0;
}

extern "C" int64_t rn_gsu_static_scratch_bytes(void) { return int64_t(RN_STATIC_SCRATCH_BYTES); }

extern "C" int rn_gsu_fwd_static(const int32_t *idx, const float *val, const int64_t *idx_strides, const void *x,
                                 const int64_t *x_strides, const void *gamma, const int64_t *gamma_strides, int dtype,
                                 const uint8_t *mask, const int64_t *mask_strides, const float *slot_in,
                                 const float *mass_in, float *slot_out, float *mass_out, void *y,
                                 const int64_t *y_strides, int64_t B, int64_t H, int64_t T, int64_t A, int64_t C,
                                 int64_t Kw, int64_t Kr, int mass_aware, double eps, int device, void *stream) {
    rn_clear_error();
    RnGsuPlan pl;
    if (int rc = rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return rc;
    RN_REQUIRE(pl.total <= RN_STATIC_SCRATCH_BYTES,
               "rn_gsu_fwd_static: this shape needs %lld bytes of schedule scratch but the built-in array holds %lld; "
               "split the sequence into shorter calls (state carries over) or use rn_gsu_fwd with a workspace",
               (long long)pl.total, (long long)RN_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    {
        RnDeviceGuard guard(device);
        RN_REQUIRE(guard.ok, "cannot make device %d current", device);
        if (int rc = rn_static_scratch_ptr(device, &scratch)) return rc;
    }
    return rn_gsu_fwd(idx, val, idx_strides, x, x_strides, gamma, gamma_strides, dtype, mask, mask_strides, slot_in,
                      mass_in, slot_out, mass_out, y, y_strides, scratch, int64_t(RN_STATIC_SCRATCH_BYTES), B, H, T, A, C,
                      Kw, Kr, mass_aware, eps, device, stream);
}
