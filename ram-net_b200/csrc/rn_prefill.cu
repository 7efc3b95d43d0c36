// Prefill forward: schedule + apply kernels (see rn_prefill.cuh) and the C-ABI entry points.
// Replaces gather_segment + ramnet_ops::topk_segment_forward / topk_segment_forward_
// (packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py:72-141,
//  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-416): no global sort, no
// per-event atomics into y, y written once in the I/O dtype.
#include "rn_prefill.cuh"

// ------------------------------------------------------------------------------------------
// schedule kernel
// ------------------------------------------------------------------------------------------
template <typename T, bool SMEM_TABLES>
__global__ void __launch_bounds__(RN_GSU_THREADS) rn_gsu_schedule_kernel(const RnGsuParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int hist[RN_GSU_RMAX + 3];
    __shared__ int cursor[RN_GSU_RMAX + 3];
    __shared__ float gam[RN_GSU_LMAX];
    __shared__ float tok_scale[RN_GSU_LMAX];
    __shared__ unsigned char tok_live[RN_GSU_LMAX];

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int A = p.A, KT = p.Kw + p.Kr, NE = p.NE;

    // dynamic smem: [mass A][claim A] (SMEM_TABLES) | ev_a[NE] | ev_v[NE] | ev_c[NE] | ev_rank[NE]
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
    uint32_t *ev_a = reinterpret_cast<uint32_t *>(cur);
    cur += size_t(NE) * 4;
    float *ev_v = reinterpret_cast<float *>(cur);
    cur += size_t(NE) * 4;
    float *ev_c = reinterpret_cast<float *>(cur);
    cur += size_t(NE) * 4;
    unsigned char *ev_rank = cur;

    const float *mass_in = p.mass_in + int64_t(bh) * A;
    for (int a = tid; a < A; a += RN_GSU_THREADS) {
        if (SMEM_TABLES || mass_in != mass) mass[a] = mass_in[a];
        claim[a] = 0xffffffffu;
    }
    __syncthreads();

    const T *gamma = static_cast<const T *>(p.gamma) + b * p.gb + h * p.gh;
    const int64_t ibase = b * p.ib + h * p.ih;

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);
        const int ne = Lc * KT;

        // ---- stage the chunk's events ---------------------------------------------------------
        for (int t = tid; t < Lc; t += RN_GSU_THREADS) {
            gam[t] = rn_to_float<T>(gamma[(t0 + t) * p.gt]);
            tok_live[t] = p.mask ? p.mask[b * p.mb + (t0 + t) * p.mt] : 1;
        }
        __syncthreads();
        for (int e = tid; e < ne; e += RN_GSU_THREADS) {
            const int t = e / KT, k = e - t * KT;
            const int64_t o = ibase + int64_t(k) * p.ik + int64_t(t0 + t) * p.it;
            const float v = fabsf(p.val[o]);
            const bool live = tok_live[t] && v != 0.f;
            ev_a[e] = uint32_t(p.idx[o] % A);
            ev_v[e] = v;
            ev_c[e] = 0.f;
            ev_rank[e] = live ? 0xff : 0xfe;
        }
        __syncthreads();

        // ---- rounds: the earliest pending event of each slot wins, is processed and retires ----
        int round = 0;
        for (;;) {
            for (int e = tid; e < ne; e += RN_GSU_THREADS)
                if (ev_rank[e] == 0xff) atomicMin(&claim[ev_a[e]], uint32_t(e));
            __syncthreads();
            int pending = 0;
            for (int e = tid; e < ne; e += RN_GSU_THREADS) {
                if (ev_rank[e] != 0xff) continue;
                const uint32_t a = ev_a[e];
                if (claim[a] == uint32_t(e)) {
                    const int t = e / KT, k = e - t * KT;
                    if (k < p.Kw) {
                        const RnGate g = rn_gate(ev_v[e], gam[t], mass[a], p.eps);
                        mass[a] = g.mass;
                        ev_c[e] = g.gain;
                    } else {
                        ev_c[e] = p.mass_aware ? ev_v[e] * mass[a] : ev_v[e];
                    }
                    ev_rank[e] = (unsigned char)round;
                    claim[a] = 0xffffffffu;
                } else {
                    pending = 1;
                }
            }
            ++round;
            if (!__syncthreads_or(pending)) break;
        }
        const int R = round;  // rounds used: 1 .. 2*L

        // ---- mass-aware reads: y_t = sum_k (r m slot) * sum r / (sum r m + eps) -------------------
        if (p.mass_aware) {
            for (int t = tid; t < Lc; t += RN_GSU_THREADS) {
                float sr = 0.f, srm = 0.f;
                for (int k = p.Kw; k < KT; ++k) {
                    const int e = t * KT + k;
                    if (ev_rank[e] < 0xfe) {
                        sr += ev_v[e];
                        srm += ev_c[e];
                    }
                }
                tok_scale[t] = sr / (srm + p.eps);
            }
            __syncthreads();
            for (int e = tid; e < ne; e += RN_GSU_THREADS) {
                const int t = e / KT, k = e - t * KT;
                if (k >= p.Kw && ev_rank[e] < 0xfe) ev_c[e] *= tok_scale[t];
            }
        }

        // ---- counting sort by round; dead reads go to one extra list (y contribution 0) ----------
        for (int r = tid; r < R + 3; r += RN_GSU_THREADS) hist[r] = 0;
        __syncthreads();
        for (int e = tid; e < ne; e += RN_GSU_THREADS) {
            const int k = e % KT;
            const int r = ev_rank[e];
            if (r < 0xfe) atomicAdd(&hist[r + 1], 1);
            else if (k >= p.Kw) atomicAdd(&hist[R + 1], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int acc = 0;
            for (int r = 0; r <= R + 1; ++r) {
                acc += hist[r];
                hist[r] = acc;      // hist[r] = start offset of list r (list R = dead reads)
                cursor[r] = acc;
            }
        }
        __syncthreads();
        const int64_t cbase = (int64_t(bh) * p.nchunks + chunk);
        uint32_t *o_slot = p.ev_slot + cbase * NE;
        uint32_t *o_meta = p.ev_meta + cbase * NE;
        float *o_coef = p.ev_coef + cbase * NE;
        uint16_t *o_offs = p.ev_offs + cbase * RN_GSU_OFFS;
        for (int e = tid; e < ne; e += RN_GSU_THREADS) {
            const int t = e / KT, k = e - t * KT;
            const int r = ev_rank[e];
            int list;
            uint32_t meta;
            if (r < 0xfe) {
                list = r;
                meta = uint32_t(t) | (uint32_t(k < p.Kw ? k : k - p.Kw) << 8) | (k < p.Kw ? 0u : RN_EV_READ);
            } else if (k >= p.Kw) {
                list = R;
                meta = uint32_t(t) | (uint32_t(k - p.Kw) << 8) | RN_EV_READ | RN_EV_ZERO;
            } else {
                continue;
            }
            const int pos = atomicAdd(&cursor[list], 1);
            o_slot[pos] = ev_a[e];
            o_meta[pos] = meta;
            o_coef[pos] = ev_c[e];
        }
        if (tid == 0) o_offs[0] = uint16_t(R);
        for (int r = tid; r <= R + 1; r += RN_GSU_THREADS) o_offs[1 + r] = uint16_t(hist[r]);
        __syncthreads();
    }

    if (SMEM_TABLES) {
        float *mass_out = p.mass_out + int64_t(bh) * A;
        for (int a = tid; a < A; a += RN_GSU_THREADS) mass_out[a] = mass[a];
    }
}

// ------------------------------------------------------------------------------------------
// apply kernel
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(RN_GSU_THREADS) rn_gsu_apply_kernel(const RnGsuParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int offs[RN_GSU_OFFS];

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
        if ((C & 3) == 0) {
            for (int i = tid; i < A * G; i += RN_GSU_THREADS) {
                const int a = i / G, sub = i - a * G;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (sub * 4 < cvalid) v = *reinterpret_cast<const float4 *>(src + int64_t(a) * C + sub * 4);
                *reinterpret_cast<float4 *>(S + a * cs + sub * 4) = v;
            }
        } else {
            for (int i = tid; i < A * cs; i += RN_GSU_THREADS) {
                const int a = i / cs, c = i - a * cs;
                S[i] = c < cvalid ? src[int64_t(a) * C + c] : 0.f;
            }
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
    const int NE = p.NE;

    for (int chunk = 0; chunk < p.nchunks; ++chunk) {
        const int t0 = chunk * p.L;
        const int Lc = min(p.L, p.T - t0);
        const int64_t cbase = (int64_t(bh) * p.nchunks + chunk);
        const uint32_t *e_slot = p.ev_slot + cbase * NE;
        const uint32_t *e_meta = p.ev_meta + cbase * NE;
        const float *e_coef = p.ev_coef + cbase * NE;
        const uint16_t *e_offs = p.ev_offs + cbase * RN_GSU_OFFS;

        const int R = e_offs[0];
        for (int i = tid; i <= R + 1; i += RN_GSU_THREADS) offs[i] = e_offs[1 + i];
        for (int i = tid; i < Lc * cs; i += RN_GSU_THREADS) {
            const int t = i / cs, c = i - t * cs;
            xt[i] = c < cvalid ? rn_to_float<T>(x[int64_t(t0 + t) * p.xt + c]) : 0.f;
        }
        __syncthreads();

        for (int r = 0; r < R; ++r) {
            const int beg = offs[r], end = offs[r + 1];
            for (int i = beg * G + tid; i < end * G; i += RN_GSU_THREADS) {
                const int ev = i / G, sub = i - ev * G;
                const uint32_t a = e_slot[ev];
                const uint32_t meta = e_meta[ev];
                const float coef = e_coef[ev];
                const int t = meta & 0xff, k = (meta >> 8) & 0xff;
                float *row = S + int64_t(a) * srow + sub * 4;
                if (vec) {
                    float4 s = *reinterpret_cast<float4 *>(row);
                    if (meta & RN_EV_READ) {
                        s.x *= coef; s.y *= coef; s.z *= coef; s.w *= coef;
                        *reinterpret_cast<float4 *>(yk + (t * Kr + k) * cs + sub * 4) = s;
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
                        if (meta & RN_EV_READ) {
                            yk[(t * Kr + k) * cs + sub * 4 + j] = coef * row[j];
                        } else {
                            row[j] = fmaf(coef, xt[t * cs + sub * 4 + j] - row[j], row[j]);
                        }
                    }
                }
            }
            __syncthreads();
        }
        {   // dead reads contribute zero
            const int beg = offs[R], end = offs[R + 1];
            for (int i = beg * G + tid; i < end * G; i += RN_GSU_THREADS) {
                const int ev = i / G, sub = i - ev * G;
                const uint32_t meta = e_meta[ev];
                const int t = meta & 0xff, k = (meta >> 8) & 0xff;
                *reinterpret_cast<float4 *>(yk + (t * Kr + k) * cs + sub * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        __syncthreads();

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
        if ((C & 3) == 0) {
            for (int i = tid; i < A * G; i += RN_GSU_THREADS) {
                const int a = i / G, sub = i - a * G;
                if (sub * 4 < cvalid)
                    *reinterpret_cast<float4 *>(dst + int64_t(a) * C + sub * 4) =
                        *reinterpret_cast<const float4 *>(S + a * cs + sub * 4);
            }
        } else {
            for (int i = tid; i < A * cs; i += RN_GSU_THREADS) {
                const int a = i / cs, c = i - a * cs;
                if (c < cvalid) dst[int64_t(a) * C + c] = S[i];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
constexpr size_t RN_SMEM_BUDGET = 220 * 1024;

struct RnGsuPlan {
    int L, nchunks, NE;
    int smem_tables;       // schedule kernel keeps mass + claim tables in shared memory
    size_t sched_smem;
    int cs, nslices, state_in_smem;
    size_t apply_smem;
    // workspace layout (byte offsets)
    size_t off_slot, off_meta, off_coef, off_offs, off_claim, total;
};

static size_t rn_align(size_t v, size_t a) { return (v + a - 1) / a * a; }

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
    const size_t ev_bytes = size_t(pl->NE) * 13 + 16;
    pl->smem_tables = (size_t(A) * 8 + ev_bytes) <= RN_SMEM_BUDGET;
    pl->sched_smem = rn_align((pl->smem_tables ? size_t(A) * 8 : 0) + ev_bytes, 16);

    // apply kernel: channels per CTA
    const int sms = rn_sm_count(device);
    int best = 0;
    for (int cs = 4; cs <= 128; cs *= 2) {
        const size_t need = (size_t(A) * cs + size_t(pl->L) * cs + size_t(pl->L) * Kr * cs) * 4;
        if (need > RN_SMEM_BUDGET) break;
        const int64_t ncta = B * H * ((C + cs - 1) / cs);
        if (best == 0 || ncta >= 2 * int64_t(sms)) best = cs;
        if (cs >= C) break;
    }
    if (best) {
        pl->cs = best;
        pl->state_in_smem = 1;
        pl->apply_smem = (size_t(A) * best + size_t(pl->L) * best + size_t(pl->L) * Kr * best) * 4;
    } else {
        // slot state stays in global memory; keep the per-CTA read buffer small
        int cs = 4;
        while (cs * 2 <= 32 && cs * 2 <= C && (size_t(pl->L) * (Kr + 1) * cs * 2) * 4 <= 96 * 1024) cs *= 2;
        pl->cs = cs;
        pl->state_in_smem = 0;
        pl->apply_smem = (size_t(pl->L) * cs + size_t(pl->L) * Kr * cs) * 4;
    }
    pl->nslices = int((C + pl->cs - 1) / pl->cs);

    const size_t n = size_t(B * H) * pl->nchunks;
    size_t off = 0;
    pl->off_slot = off; off = rn_align(off + n * pl->NE * 4, 256);
    pl->off_meta = off; off = rn_align(off + n * pl->NE * 4, 256);
    pl->off_coef = off; off = rn_align(off + n * pl->NE * 4, 256);
    pl->off_offs = off; off = rn_align(off + n * RN_GSU_OFFS * 2, 256);
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

template <typename T>
static int rn_launch_gsu(const RnGsuParams &p, const RnGsuPlan &pl, cudaStream_t stream) {
    const int bh = p.B * p.H;
    rn_prof_reset();
    rn_prof_mark(stream);
    if (pl.smem_tables) {
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_schedule_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(pl.sched_smem)));
        rn_gsu_schedule_kernel<T, true><<<bh, RN_GSU_THREADS, pl.sched_smem, stream>>>(p);
    } else {
        RN_CUDA(cudaFuncSetAttribute(rn_gsu_schedule_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(pl.sched_smem)));
        rn_gsu_schedule_kernel<T, false><<<bh, RN_GSU_THREADS, pl.sched_smem, stream>>>(p);
    }
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(stream);
    RN_CUDA(cudaFuncSetAttribute(rn_gsu_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(pl.apply_smem)));
    rn_gsu_apply_kernel<T><<<bh * pl.nslices, RN_GSU_THREADS, pl.apply_smem, stream>>>(p);
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
    p.L = pl.L; p.nchunks = pl.nchunks; p.NE = pl.NE;
    p.mass_aware = mass_aware; p.eps = float(eps);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    p.ev_slot = reinterpret_cast<uint32_t *>(ws + pl.off_slot);
    p.ev_meta = reinterpret_cast<uint32_t *>(ws + pl.off_meta);
    p.ev_coef = reinterpret_cast<float *>(ws + pl.off_coef);
    p.ev_offs = reinterpret_cast<uint16_t *>(ws + pl.off_offs);
    p.claim = reinterpret_cast<uint32_t *>(ws + pl.off_claim);
    p.cs = pl.cs; p.nslices = pl.nslices; p.state_in_smem = pl.state_in_smem;

    if (!pl.state_in_smem && slot_in != slot_out)
        RN_CUDA(cudaMemcpyAsync(slot_out, slot_in, size_t(B * H * A * C) * 4, cudaMemcpyDeviceToDevice, stream));
    if (!pl.smem_tables && mass_in != mass_out)
        RN_CUDA(cudaMemcpyAsync(mass_out, mass_in, size_t(B * H * A) * 4, cudaMemcpyDeviceToDevice, stream));

    if (dtype == RN_F32) return rn_launch_gsu<float>(p, pl, stream);
    if (dtype == RN_F16) return rn_launch_gsu<__half>(p, pl, stream);
    return rn_launch_gsu<__nv_bfloat16>(p, pl, stream);
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
