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
__global__ void __launch_bounds__(RN_GSU_THREADS) rn_gsu_schedule_kernel(const RnGsuParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int hist[RN_GSU_RMAX + 2];
    __shared__ int cursor[RN_GSU_RMAX + 2];
    __shared__ float gam[RN_GSU_LMAX];
    __shared__ float tok_scale[RN_GSU_LMAX];
    __shared__ unsigned char tok_live[RN_GSU_LMAX];

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, lane = tid & 31;
    const int A = p.A, KT = p.Kw + p.Kr, NEp = p.NEp;
    const bool pow2 = (A & (A - 1)) == 0;

    // dynamic smem: [mass A][claim A] (SMEM_TABLES) | ev_v[NE] ev_c[NE] (mass-aware only)
    unsigned char *cur = dyn;
    float *mass;
    uint32_t *claim;
    if (SMEM_TABLES) {
        mass = reinterpret_cast<float *>(cur);
        cur += size_t(A) * 4;
        claim = reinterpret_cast<uint32_t *>(cur);
        cur += size_t(A) * 4;
    } else {
        mass = p.mass_out + int64_t(bh) * A;
        claim = p.claim + int64_t(bh) * A;
    }
    float *ev_v = reinterpret_cast<float *>(cur);
    float *ev_c = ev_v + p.NE;

    if (bh == 0 && tid == 0) *p.status = 0;
    const float *mass_in = p.mass_in + int64_t(bh) * A;
    for (int a = tid; a < A; a += RN_GSU_THREADS) {
        if (SMEM_TABLES || mass_in != mass) mass[a] = mass_in[a];
        claim[a] = 0xffffffffu;
    }

    // event e = j * 256 + tid  ->  (token in chunk, k); fixed for the whole kernel
    int ev_t[EPT], ev_k[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = j * RN_GSU_THREADS + tid;
        ev_t[j] = e / KT;
        ev_k[j] = e - ev_t[j] * KT;
    }
    __syncthreads();

    const T *gamma = static_cast<const T *>(p.gamma) + b * p.gb + h * p.gh;
    const int64_t ibase = b * p.ib + h * p.ih;

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);

        if (tid < Lc) {
            gam[tid] = rn_to_float<T>(gamma[(t0 + tid) * p.gt]);
            tok_live[tid] = p.mask ? p.mask[b * p.mb + (t0 + tid) * p.mt] : 1;
        }
        // ---- stage this thread's events -------------------------------------------------------
        uint32_t ea[EPT];
        float ev[EPT], ec[EPT];
        int er[EPT];          // round, or -1 dead write, -2 dead read, -3 out of range
        uint32_t pend = 0;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            er[j] = -3;
            ea[j] = 0;
            ev[j] = 0.f;
            ec[j] = 0.f;
            if (ev_t[j] < Lc) {
                const int64_t o = ibase + int64_t(ev_k[j]) * p.ik + int64_t(t0 + ev_t[j]) * p.it;
                const int raw = p.idx[o];
                ea[j] = pow2 ? uint32_t(raw & (A - 1)) : uint32_t(raw % A);
                ev[j] = fabsf(p.val[o]);
            }
        }
        __syncthreads();  // gam / tok_live visible
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            if (ev_t[j] < Lc) {
                const bool live = tok_live[ev_t[j]] && ev[j] != 0.f;
                er[j] = live ? 0 : (ev_k[j] < p.Kw ? -1 : -2);
                if (live) pend |= 1u << j;
            }
        }

        // ---- rounds: the earliest pending event of each slot wins, is processed and retires ----
        int R = 0;
        for (;;) {
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (pend & (1u << j)) atomicMin(&claim[ea[j]], uint32_t(j * RN_GSU_THREADS + tid));
            __syncthreads();
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (!(pend & (1u << j))) continue;
                if (claim[ea[j]] == uint32_t(j * RN_GSU_THREADS + tid)) {
                    if (ev_k[j] < p.Kw) {
                        const RnGate g = rn_gate(ev[j], gam[ev_t[j]], mass[ea[j]], p.eps);
                        mass[ea[j]] = g.mass;
                        ec[j] = g.gain;
                    } else {
                        ec[j] = p.mass_aware ? ev[j] * mass[ea[j]] : ev[j];
                    }
                    er[j] = R;
                    claim[ea[j]] = 0xffffffffu;
                    pend &= ~(1u << j);
                }
            }
            ++R;
            if (!__syncthreads_or(pend != 0)) break;
        }

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

        // ---- counting sort by round (dead reads ride in round 0 with the zero flag) ---------------
        for (int r = tid; r < R + 2; r += RN_GSU_THREADS) hist[r] = 0;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const bool emit = er[j] >= 0 || er[j] == -2;
            const int list = er[j] >= 0 ? er[j] : 0;
            const unsigned act = __ballot_sync(RN_FULL, emit);
            if (emit) {
                const unsigned grp = __match_any_sync(act, list);
                if (lane == __ffs(grp) - 1) atomicAdd(&hist[list + 1], __popc(grp));
            }
        }
        __syncthreads();
        if (tid == 0) {
            int acc = 0;
            for (int r = 0; r <= R; ++r) {
                acc += hist[r];
                hist[r] = acc;  // first entry of round r; hist[R] = entry count
                cursor[r] = acc;
            }
        }
        __syncthreads();
        unsigned char *rec = p.records + (int64_t(bh) * p.nchunks + chunk) * p.rec_bytes;
        uint16_t *o_hdr = reinterpret_cast<uint16_t *>(rec);
        uint32_t *o_meta = reinterpret_cast<uint32_t *>(rec + RN_GSU_HDR_BYTES);
        float *o_coef = reinterpret_cast<float *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 4);
        uint32_t *o_slot = reinterpret_cast<uint32_t *>(rec + RN_GSU_HDR_BYTES + size_t(NEp) * 8);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const bool emit = er[j] >= 0 || er[j] == -2;
            const int list = er[j] >= 0 ? er[j] : 0;
            const unsigned act = __ballot_sync(RN_FULL, emit);
            if (emit) {
                const unsigned grp = __match_any_sync(act, list);
                const int leader = __ffs(grp) - 1;
                int base = 0;
                if (lane == leader) base = atomicAdd(&cursor[list], __popc(grp));
                base = __shfl_sync(grp, base, leader);
                const int pos = base + __popc(grp & ((1u << lane) - 1u));
                const bool read = ev_k[j] >= p.Kw;
                o_meta[pos] = rn_ev_pack(ea[j], ev_t[j], read ? ev_k[j] - p.Kw : ev_k[j], read, er[j] < 0);
                o_coef[pos] = er[j] >= 0 ? ec[j] : 0.f;
                if (p.wide) o_slot[pos] = ea[j];
            }
        }
        if (tid == 0) o_hdr[0] = uint16_t(R);
        for (int r = tid; r <= R; r += RN_GSU_THREADS) o_hdr[1 + r] = uint16_t(hist[r]);
        __syncthreads();
    }

    if (SMEM_TABLES) {
        float *mass_out = p.mass_out + int64_t(bh) * A;
        for (int a = tid; a < A; a += RN_GSU_THREADS) mass_out[a] = mass[a];
    }
}

// ------------------------------------------------------------------------------------------
// generic apply kernel: any C, state in shared or global memory, records read from global
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(RN_GSU_THREADS) rn_gsu_apply_kernel(const RnGsuParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int offs[RN_GSU_HDR];

    const int slice = blockIdx.x % p.nslices;
    const int bh = blockIdx.x / p.nslices;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int cs = p.cs, G = cs >> 2, C = p.C, A = p.A;
    const int c0 = slice * cs;
    const int cvalid = min(cs, C - c0);
    const int Kr = p.Kr;

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
        const unsigned char *rec = p.records + (int64_t(bh) * p.nchunks + chunk) * p.rec_bytes;
        const uint16_t *e_hdr = reinterpret_cast<const uint16_t *>(rec);
        const uint32_t *e_meta = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES);
        const float *e_coef = reinterpret_cast<const float *>(rec + RN_GSU_HDR_BYTES + size_t(p.NEp) * 4);
        const uint32_t *e_slot = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES + size_t(p.NEp) * 8);

        const int R = e_hdr[0];
        for (int i = tid; i <= R; i += RN_GSU_THREADS) offs[i] = e_hdr[1 + i];
        for (int i = tid; i < Lc * cs; i += RN_GSU_THREADS) {
            const int t = i / cs, c = i - t * cs;
            xt[i] = c < cvalid ? rn_to_float<T>(x[int64_t(t0 + t) * p.xt + c]) : 0.f;
        }
        __syncthreads();

        for (int r = 0; r < R; ++r) {
            const int beg = offs[r], end = offs[r + 1];
            for (int i = beg * G + tid; i < end * G; i += RN_GSU_THREADS) {
                const int ev = i / G, sub = i - ev * G;
                const uint32_t meta = e_meta[ev];
                const uint32_t a = p.wide ? e_slot[ev] : (meta & 0xffffu);
                const float coef = e_coef[ev];
                const int t = rn_ev_t(meta), k = rn_ev_k(meta);
                float *row = S + int64_t(a) * srow + sub * 4;
                float *dst = yk + (t * Kr + k) * cs + sub * 4;
                if (meta & RN_EV_ZERO) {
                    dst[0] = dst[1] = dst[2] = dst[3] = 0.f;
                } else if (vec) {
                    float4 s = *reinterpret_cast<float4 *>(row);
                    if (meta & RN_EV_READ) {
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
                        if (meta & RN_EV_READ) dst[j] = coef * row[j];
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
// fast apply kernel: C % 4 == 0, A <= 65536, slice state + streamed chunk records in shared memory
// ------------------------------------------------------------------------------------------
constexpr int RN_APPLY_THREADS = 512;

template <int CS>
__device__ __forceinline__ void rn_apply_entry(const uint32_t meta, const float coef, float *__restrict__ S,
                                               const float *__restrict__ xt, float *__restrict__ yk, const int Kr,
                                               const int sub) {
    // one thread handles CPT = min(CS, 8) channels of one event, starting at channel sub * CPT
    constexpr int CPT = CS >= 8 ? 8 : 4;
    const int t = rn_ev_t(meta), k = rn_ev_k(meta);
    float *dst = yk + (t * Kr + k) * CS + sub * CPT;
    if (meta & RN_EV_ZERO) {
#pragma unroll
        for (int v = 0; v < CPT / 4; ++v) reinterpret_cast<float4 *>(dst)[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    float *row = S + (meta & 0xffffu) * CS + sub * CPT;
    if (meta & RN_EV_READ) {
#pragma unroll
        for (int v = 0; v < CPT / 4; ++v) {
            float4 s = reinterpret_cast<const float4 *>(row)[v];
            s.x *= coef; s.y *= coef; s.z *= coef; s.w *= coef;
            reinterpret_cast<float4 *>(dst)[v] = s;
        }
    } else {
        const float *xr = xt + t * CS + sub * CPT;
#pragma unroll
        for (int v = 0; v < CPT / 4; ++v) {
            float4 s = reinterpret_cast<const float4 *>(row)[v];
            const float4 xv = reinterpret_cast<const float4 *>(xr)[v];
            s.x = fmaf(coef, xv.x - s.x, s.x);
            s.y = fmaf(coef, xv.y - s.y, s.y);
            s.z = fmaf(coef, xv.z - s.z, s.z);
            s.w = fmaf(coef, xv.w - s.w, s.w);
            reinterpret_cast<float4 *>(row)[v] = s;
        }
    }
}

template <typename T, int CS>
__global__ void __launch_bounds__(RN_APPLY_THREADS, 1) rn_gsu_apply_fast_kernel(const RnGsuParams p) {
    constexpr int CPT = CS >= 8 ? 8 : 4;   // channels per thread per event
    constexpr int G = CS / CPT;            // threads per event
    constexpr int G4 = CS / 4;             // float4 groups per row
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t mbar[2];

    const int slice = blockIdx.x % p.nslices;
    const int bh = blockIdx.x / p.nslices;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = p.C, A = p.A, Kr = p.Kr, L = p.L;
    const int c0 = slice * CS;
    const int cvalid = min(CS, C - c0);  // multiple of 4
    const uint32_t rec_copy = uint32_t(RN_GSU_HDR_BYTES + size_t(p.NEp) * 8);  // header + meta + coef

    // dynamic smem: rec[2][rec_copy] | S[A*CS] | yk[L*Kr*CS] | xt[2][L*CS]
    const size_t rec_stride = (size_t(rec_copy) + 127) / 128 * 128;
    unsigned char *rec0 = dyn;
    float *S = reinterpret_cast<float *>(dyn + 2 * rec_stride);
    float *yk = S + size_t(A) * CS;
    float *xt0 = yk + size_t(L) * Kr * CS;

    if (tid == 0) {
        rn_mbar_init(&mbar[0], 1);
        rn_mbar_init(&mbar[1], 1);
        rn_mbar_fence_init();
    }
    __syncthreads();
    const unsigned char *records = p.records + int64_t(bh) * p.nchunks * p.rec_bytes;
    if (tid == 0) {
        rn_mbar_expect_tx(&mbar[0], rec_copy);
        rn_bulk_g2s(rec0, records, rec_copy, &mbar[0]);
    }

    // state slice -> shared memory
    {
        const float *src = p.slot_in + int64_t(bh) * A * C + c0;
        for (int i = tid; i < A * G4; i += RN_APPLY_THREADS) {
            const int a = i / G4, sub = i - a * G4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sub * 4 < cvalid) v = *reinterpret_cast<const float4 *>(src + int64_t(a) * C + sub * 4);
            *reinterpret_cast<float4 *>(S + a * CS + sub * 4) = v;
        }
    }
    const T *x = static_cast<const T *>(p.x) + b * p.xb + h * p.xh + c0;
    T *y = static_cast<T *>(p.y) + b * p.yb + h * p.yh + c0;

    // x tile of chunk 0 (threads cover (t, 4-channel group) pairs; L*G4 <= 64*32 = 2048 -> up to 4 per thread)
    constexpr int XPT = (RN_GSU_LMAX * G4 + RN_APPLY_THREADS - 1) / RN_APPLY_THREADS;
    float4 xreg[XPT];
    auto load_x = [&](int chunk) {
        const int t0 = chunk * L;
        const int Lc = min(L, p.T - t0);
#pragma unroll
        for (int q = 0; q < XPT; ++q) {
            const int i = q * RN_APPLY_THREADS + tid;
            const int t = i / G4, sub = i - t * G4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < Lc && sub * 4 < cvalid) {
                v = rn_load4<T>(x + int64_t(t0 + t) * p.xt + sub * 4);
            }
            xreg[q] = v;
        }
    };
    auto store_x = [&](float *xt) {
#pragma unroll
        for (int q = 0; q < XPT; ++q) {
            const int i = q * RN_APPLY_THREADS + tid;
            if (i < L * G4) *reinterpret_cast<float4 *>(xt + i * 4) = xreg[q];
        }
    };
    load_x(0);
    store_x(xt0);
    __syncthreads();

    bool failed = false;
    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int buf = chunk & 1;
        const int t0 = chunk * L;
        const int Lc = min(L, p.T - t0);
        const bool more = chunk + 1 < p.nchunks;
        // prefetch the next chunk: its record by bulk copy, its x tile into registers
        if (more) {
            if (tid == 0) {
                rn_fence_proxy_async();
                rn_mbar_expect_tx(&mbar[buf ^ 1], rec_copy);
                rn_bulk_g2s(rec0 + (buf ^ 1) * rec_stride, records + int64_t(chunk + 1) * p.rec_bytes, rec_copy,
                            &mbar[buf ^ 1]);
            }
            load_x(chunk + 1);
        }
        if (!rn_mbar_wait_bounded(&mbar[buf], (chunk >> 1) & 1)) failed = true;
        if (__syncthreads_or(failed)) {
            // a bulk copy never completed: record it, give the copy in flight a last bounded chance
            // to land (it targets this CTA's shared memory), and leave without touching the outputs
            if (tid == 0) atomicExch(p.status, 1);
            if (more) rn_mbar_wait_bounded(&mbar[buf ^ 1], ((chunk + 1) >> 1) & 1);
            return;
        }

        const unsigned char *rec = rec0 + buf * rec_stride;
        const uint16_t *hdr = reinterpret_cast<const uint16_t *>(rec);
        const uint32_t *e_meta = reinterpret_cast<const uint32_t *>(rec + RN_GSU_HDR_BYTES);
        const float *e_coef = reinterpret_cast<const float *>(rec + RN_GSU_HDR_BYTES + size_t(p.NEp) * 4);
        const float *xt = xt0 + buf * (L * CS);
        const int R = hdr[0];

        // rounds 0 and 1 on the whole CTA, the sparse later rounds on warp 0 alone
        const int wide_rounds = min(R, 2);
        for (int r = 0; r < wide_rounds; ++r) {
            const int beg = hdr[1 + r], end = hdr[2 + r];
            for (int i = beg * G + tid; i < end * G; i += RN_APPLY_THREADS) {
                const int ev = i / G, sub = i - ev * G;
                rn_apply_entry<CS>(e_meta[ev], e_coef[ev], S, xt, yk, Kr, sub);
            }
            __syncthreads();
        }
        if (R > 2) {
            if (warp == 0) {
                for (int r = 2; r < R; ++r) {
                    const int beg = hdr[1 + r], end = hdr[2 + r];
                    for (int i = beg * G + lane; i < end * G; i += 32) {
                        const int ev = i / G, sub = i - ev * G;
                        rn_apply_entry<CS>(e_meta[ev], e_coef[ev], S, xt, yk, Kr, sub);
                    }
                    __syncwarp();
                }
            }
            __syncthreads();
        }

        // ---- y[t] = sum_k yk[t][k], fixed order ------------------------------------------------
        for (int i = tid; i < Lc * G4; i += RN_APPLY_THREADS) {
            const int t = i / G4, sub = i - t * G4;
            if (sub * 4 >= cvalid) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const float *src = yk + t * Kr * CS + sub * 4;
#pragma unroll 4
            for (int k = 0; k < Kr; ++k) {
                const float4 v = *reinterpret_cast<const float4 *>(src + k * CS);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            rn_store4<T>(y + int64_t(t0 + t) * p.yt + sub * 4, acc);
        }
        if (more) store_x(xt0 + (buf ^ 1) * (L * CS));
        __syncthreads();
    }

    float *dst = p.slot_out + int64_t(bh) * A * C + c0;
    for (int i = tid; i < A * G4; i += RN_APPLY_THREADS) {
        const int a = i / G4, sub = i - a * G4;
        if (sub * 4 < cvalid)
            *reinterpret_cast<float4 *>(dst + int64_t(a) * C + sub * 4) = *reinterpret_cast<const float4 *>(S + a * CS + sub * 4);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
constexpr size_t RN_SMEM_BUDGET = 225 * 1024;

struct RnGsuPlan {
    int L, nchunks, NE, NEp, ept;
    int smem_tables;       // schedule kernel keeps mass + claim tables in shared memory
    size_t sched_smem;
    int wide;              // A > 65536: records carry a separate slot array
    int64_t rec_bytes;
    int fast;              // fast apply kernel (C % 4 == 0, narrow records, state in shared memory)
    int cs, nslices, state_in_smem;
    size_t apply_smem;
    // workspace layout (byte offsets)
    size_t off_records, off_claim, total;
};

static size_t rn_align(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t rn_fast_smem(int64_t A, int cs, int L, int64_t Kr, int NEp) {
    const size_t rec_stride = rn_align(RN_GSU_HDR_BYTES + size_t(NEp) * 8, 128);
    return 2 * rec_stride + (size_t(A) * cs + size_t(L) * Kr * cs + 2 * size_t(L) * cs) * 4;
}

static int rn_gsu_plan(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int device,
                       RnGsuPlan *pl) {
    RN_REQUIRE(B > 0 && H > 0 && T > 0 && A > 0 && C > 0, "prefill dims must be positive");
    RN_REQUIRE(Kw > 0 && Kw <= 128 && Kr > 0 && Kr <= 128, "Expect 0 < top_k <= 128 (got %lld, %lld)", (long long)Kw,
               (long long)Kr);
    RN_REQUIRE(A < (int64_t(1) << 30), "Address space overflow: A must stay below 2^30");
    RN_REQUIRE(B * H < (int64_t(1) << 24), "B*H too large");
    pl->L = rn_gsu_chunk_len(int(Kw), int(Kr));
    pl->nchunks = int((T + pl->L - 1) / pl->L);
    pl->NE = pl->L * int(Kw + Kr);
    pl->NEp = int(rn_align(pl->NE, 4));
    int ept = (pl->NE + RN_GSU_THREADS - 1) / RN_GSU_THREADS;
    pl->ept = ept <= 1 ? 1 : (ept <= 2 ? 2 : (ept <= 4 ? 4 : (ept <= 8 ? 8 : 16)));
    const size_t ev_bytes = size_t(pl->NE) * 8 + 16;
    pl->smem_tables = (size_t(A) * 8 + ev_bytes) <= RN_SMEM_BUDGET;
    pl->sched_smem = rn_align((pl->smem_tables ? size_t(A) * 8 : 0) + ev_bytes, 16);
    pl->wide = A > 65536;
    pl->rec_bytes = int64_t(rn_align(RN_GSU_HDR_BYTES + size_t(pl->NEp) * (pl->wide ? 12 : 8), 128));

    // apply kernel: channels per CTA.  Largest slice that still gives two CTAs per SM of work,
    // else the smallest one (most parallelism).
    const int sms = rn_sm_count(device);
    const bool fast_ok = !pl->wide && (C % 4) == 0;
    int best = 0;
    for (int cs = 4; cs <= (fast_ok ? 32 : 128); cs *= 2) {
        const size_t need = fast_ok ? rn_fast_smem(A, cs, pl->L, Kr, pl->NEp)
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
        pl->apply_smem = fast_ok ? rn_fast_smem(A, best, pl->L, Kr, pl->NEp)
                                 : (size_t(A) * best + size_t(pl->L) * best + size_t(pl->L) * Kr * best) * 4;
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

template <typename T, bool SMEM>
static int rn_launch_schedule(const RnGsuParams &p, const RnGsuPlan &pl, cudaStream_t stream) {
    const int bh = p.B * p.H;
#define RN_CASE(E)                                                                                              \
    if (pl.ept == E) {                                                                                          \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_schedule_kernel<T, SMEM, E>,                                        \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(pl.sched_smem)));         \
        rn_gsu_schedule_kernel<T, SMEM, E><<<bh, RN_GSU_THREADS, pl.sched_smem, stream>>>(p);                   \
        return 0;                                                                                               \
    }
    RN_CASE(1) RN_CASE(2) RN_CASE(4) RN_CASE(8) RN_CASE(16)
#undef RN_CASE
    rn_set_error("no schedule kernel for %d events per thread", pl.ept);
    return 1;
}

template <typename T>
static int rn_launch_apply_fast(const RnGsuParams &p, const RnGsuPlan &pl, cudaStream_t stream) {
    const int grid = p.B * p.H * pl.nslices;
#define RN_CASE(CSV)                                                                                            \
    if (pl.cs == CSV) {                                                                                         \
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_apply_fast_kernel<T, CSV>,                                          \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(pl.apply_smem)));         \
        rn_gsu_apply_fast_kernel<T, CSV><<<grid, RN_APPLY_THREADS, pl.apply_smem, stream>>>(p);                 \
        return 0;                                                                                               \
    }
    RN_CASE(4) RN_CASE(8) RN_CASE(16) RN_CASE(32)
#undef RN_CASE
    rn_set_error("no fast apply kernel for %d channels per CTA", pl.cs);
    return 1;
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
                   mass_out && y && y_strides && workspace,
               "null pointer argument");
    RN_REQUIRE(dtype == RN_F32 || dtype == RN_F16 || dtype == RN_BF16, "unsupported dtype code %d", dtype);
    RN_REQUIRE(x_strides[3] == 1 && y_strides[3] == 1, "Tensor x / y last dim must be contiguous");
    RN_REQUIRE(mask == nullptr || mask_strides != nullptr, "mask needs strides");
    RnGsuPlan pl;
    if (int rc = rn_gsu_plan(B, H, T, A, C, Kw, Kr, device, &pl)) return rc;
    RN_REQUIRE(workspace_bytes >= int64_t(pl.total), "workspace too small: %lld < %lld bytes", (long long)workspace_bytes,
               (long long)pl.total);
    RN_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
    RN_REQUIRE((reinterpret_cast<uintptr_t>(slot_in) & 15) == 0 && (reinterpret_cast<uintptr_t>(slot_out) & 15) == 0,
               "slot state must be 16-byte aligned");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);
    cudaStream_t stream = cudaStream_t(stream_);

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
    p.mass_aware = mass_aware; p.eps = float(eps);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    p.status = reinterpret_cast<int *>(ws);
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
