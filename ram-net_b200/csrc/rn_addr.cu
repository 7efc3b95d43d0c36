// Address decode kernels (forward and backward) and their C-ABI entry points.
//
// Forward: one warp per (batch, token, head, write|read) block of U*P logits; see rn_addr.cuh.
// The kernel reads the logits through element strides, so the caller's native (B,T,H,U,P)
// tensor is consumed in place (U*P contiguous logits per warp) without the transposed copy
// the reference makes (packages/ramnet-ops/csrc/ram_attn_ops.cpp:162,168), and write and read
// logits are decoded by the same launch.
#include "rn_addr.cuh"

struct RnAddrFwdParams {
    const void *addr[2];
    int64_t sb, sh, su, sp, st;
    const int32_t *pos;
    int64_t pb, pt;
    int32_t *idx;
    float *val;
    int64_t ob, oh, ok, ot;
    int B, H, U, P, T, E, A;
    int K[2];
    float re_norm[2];
    float sign[2];
    int encode_batch;
    int nwhich;
    int64_t n_items;
};

constexpr int RN_ADDR_WARPS = 4;

template <typename T, int KPL, int PPL>
__global__ void __launch_bounds__(RN_ADDR_WARPS * 32) rn_addr_fwd_kernel(const RnAddrFwdParams p) {
    __shared__ RnPairTable tabs[2];
    __shared__ RnWarpScratch scratch[RN_ADDR_WARPS];
    __shared__ int row_off[RN_KMAX + 1];

    rn_build_pairs(&tabs[0], p.K[0], row_off);
    if (p.nwhich > 1) rn_build_pairs(&tabs[1], p.K[1], row_off);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    RnWarpScratch *ws = &scratch[warp];

    for (int64_t item = int64_t(blockIdx.x) * RN_ADDR_WARPS + warp; item < p.n_items;
         item += int64_t(gridDim.x) * RN_ADDR_WARPS) {
        const int which = int(item % p.nwhich);
        const int64_t row = item / p.nwhich;
        const int h = int(row % p.H);
        const int t = int((row / p.H) % p.T);
        const int b = int(row / (int64_t(p.H) * p.T));

        RnDigitLoader<T> load;
        load.base = static_cast<const T *>(p.addr[which]) + b * p.sb + h * p.sh + t * p.st;
        load.su = p.su;
        load.sp = p.sp;
        const int K = p.K[which];
        const RnDecoded<KPL> d = rn_warp_decode<KPL, PPL>(load, p.U, p.P, K, p.re_norm[which], ws, &tabs[which], lane);

        const int shift = (h < p.E) ? rn_pos_mod(p.pos[b * p.pb + t * p.pt], p.A) : 0;
        const int offs = (p.encode_batch ? (b * p.H + h) : h) * p.A;
        const int koff = which ? p.K[0] : 0;
        const int64_t obase = b * p.ob + h * p.oh + t * p.ot;
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            const int e = lane * KPL + r;
            if (e < K) {
                const int64_t o = obase + int64_t(koff + e) * p.ok;
                p.idx[o] = offs + rn_cape(d.idx[r], shift, p.A);
                p.val[o] = p.sign[which] * d.val[r];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------
struct RnAddrBwdParams {
    const int32_t *idx;
    const float *val;
    int64_t ob, oh, ok, ot;
    const float *d_val;
    int64_t gb, gh, gk, gt;
    const void *addr[2];
    int64_t sb, sh, su, sp, st;
    const int32_t *pos;
    int64_t pb, pt;
    void *d_addr[2];
    int64_t db, dh, du, dp, dt;
    int B, H, U, P, T, E, A;
    int K[2];
    float re_norm[2];
    float sign[2];
    int nwhich;
    int64_t n_items;
};

struct RnBwdScratch {
    int content[RN_KMAX];
    float d[RN_KMAX];
};

// d logit[u][p] = sum_{k : digit_u(content_k) = p} D'_k  -  softmax_u[p] * (1 - rho) * sum_k D_k
// with D_k = d_val_k * w_k and D'_k = D_k - rho * (w_k / sum w) * sum D   (w = positive weight).
template <typename T, int PPL>
__global__ void __launch_bounds__(RN_ADDR_WARPS * 32) rn_addr_bwd_kernel(const RnAddrBwdParams p) {
    __shared__ RnBwdScratch scratch[RN_ADDR_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    RnBwdScratch *ws = &scratch[warp];

    for (int64_t item = int64_t(blockIdx.x) * RN_ADDR_WARPS + warp; item < p.n_items;
         item += int64_t(gridDim.x) * RN_ADDR_WARPS) {
        const int which = int(item % p.nwhich);
        const int64_t row = item / p.nwhich;
        const int h = int(row % p.H);
        const int t = int((row / p.H) % p.T);
        const int b = int(row / (int64_t(p.H) * p.T));
        const int K = p.K[which];
        const int koff = which ? p.K[0] : 0;
        const float rho = p.re_norm[which];
        const int shift = (h < p.E) ? rn_pos_mod(p.pos[b * p.pb + t * p.pt], p.A) : 0;

        float dsum = 0.f, wsum = 0.f;
        for (int k = lane; k < K; k += 32) {
            const int64_t o = b * p.ob + h * p.oh + int64_t(koff + k) * p.ok + t * p.ot;
            const int64_t g = b * p.gb + h * p.gh + int64_t(koff + k) * p.gk + t * p.gt;
            const float w = p.sign[which] * p.val[o];
            const float dk = p.d_val[g] * w;
            int local = p.idx[o] % p.A;
            local += shift;
            ws->content[k] = local >= p.A ? local - p.A : local;
            ws->d[k] = dk;
            dsum += dk;
            wsum += w;
        }
        dsum = rn_warp_sum(dsum);
        wsum = rn_warp_sum(wsum);
        __syncwarp();
        if (rho != 0.f && wsum > 0.f) {
            for (int k = lane; k < K; k += 32) {
                const int64_t o = b * p.ob + h * p.oh + int64_t(koff + k) * p.ok + t * p.ot;
                const float w = p.sign[which] * p.val[o];
                ws->d[k] -= rho * (w / wsum) * dsum;
            }
            __syncwarp();
        }
        const float tail = (1.f - rho) * dsum;

        const T *src = static_cast<const T *>(p.addr[which]) + b * p.sb + h * p.sh + t * p.st;
        T *dst = static_cast<T *>(p.d_addr[which]) + b * p.db + h * p.dh + t * p.dt;

        // a token with an all -inf digit carries zero weights and zero gradients
        bool inactive = false;
        for (int u = 0; u < p.U; ++u) {
            float m = -INFINITY;
#pragma unroll
            for (int r = 0; r < PPL; ++r) {
                const int pp = lane * PPL + r;
                if (pp < p.P) m = fmaxf(m, rn_to_float<T>(src[u * p.su + pp * p.sp]));
            }
            m = rn_warp_max(m);
            inactive |= (m == -INFINITY);
        }

        int stride = 1;
        for (int u = 0; u < p.U; ++u) {
            float xv[PPL];
            float m = -INFINITY;
#pragma unroll
            for (int r = 0; r < PPL; ++r) {
                const int pp = lane * PPL + r;
                xv[r] = (pp < p.P) ? rn_to_float<T>(src[u * p.su + pp * p.sp]) : -INFINITY;
                m = fmaxf(m, xv[r]);
            }
            m = rn_warp_max(m);
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < PPL; ++r) s += (lane * PPL + r < p.P && !inactive) ? expf(xv[r] - m) : 0.f;
            s = rn_warp_sum(s);
            float acc[PPL];
#pragma unroll
            for (int r = 0; r < PPL; ++r) acc[r] = 0.f;
            for (int k = 0; k < K; ++k) {
                const int digit = (ws->content[k] / stride) % p.P;
                const float dk = ws->d[k];
#pragma unroll
                for (int r = 0; r < PPL; ++r) acc[r] += (digit == lane * PPL + r) ? dk : 0.f;
            }
#pragma unroll
            for (int r = 0; r < PPL; ++r) {
                const int pp = lane * PPL + r;
                if (pp < p.P) {
                    float g = 0.f;
                    if (!inactive) g = acc[r] - (expf(xv[r] - m) / s) * tail;
                    dst[u * p.du + pp * p.dp] = rn_from_float<T>(g);
                }
            }
            stride *= p.P;
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int rn_pow_fits(int64_t P, int64_t U, int64_t *A_out) {
    int64_t A = 1;
    for (int64_t u = 0; u < U; ++u) {
        A *= P;
        if (A >= (int64_t(1) << 30)) return 0;
    }
    *A_out = A;
    return 1;
}

static int rn_per_lane(int64_t n) { return n <= 32 ? 1 : (n <= 64 ? 2 : 4); }

static int rn_check_addr_dims(int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E, int64_t Kw,
                              int64_t Kr, double w_re_norm, double r_re_norm, int dtype, int64_t *A) {
    RN_REQUIRE(B > 0 && H > 0 && U > 0 && P > 0 && T > 0, "address dims must be positive (B=%lld H=%lld U=%lld P=%lld T=%lld)",
               (long long)B, (long long)H, (long long)U, (long long)P, (long long)T);
    RN_REQUIRE(U <= RN_UMAX, "Expect U <= %d but got %lld", RN_UMAX, (long long)U);
    RN_REQUIRE(P <= RN_PMAX, "Expect P <= %d but got %lld", RN_PMAX, (long long)P);
    RN_REQUIRE(rn_pow_fits(P, U, A), "Address space overflow: P^U must stay below 2^30 (P=%lld U=%lld)", (long long)P,
               (long long)U);
    RN_REQUIRE(Kw > 0 && Kw <= RN_KMAX && Kw <= *A, "Expect 0 < w_top_k <= min(%d, A=%lld) but got %lld", RN_KMAX,
               (long long)*A, (long long)Kw);
    RN_REQUIRE(Kr >= 0 && Kr <= RN_KMAX && Kr <= *A, "Expect 0 <= r_top_k <= min(%d, A=%lld) but got %lld", RN_KMAX,
               (long long)*A, (long long)Kr);
    RN_REQUIRE(E >= 0 && E <= H, "Expect embed_num in [0, H=%lld] but got %lld", (long long)H, (long long)E);
    RN_REQUIRE(w_re_norm >= 0.0 && w_re_norm <= 1.0 && r_re_norm >= 0.0 && r_re_norm <= 1.0,
               "top_k_re_norm must be in [0, 1].");
    RN_REQUIRE(dtype == RN_F32 || dtype == RN_F16 || dtype == RN_BF16, "unsupported dtype code %d", dtype);
    RN_REQUIRE(B * H * *A < (int64_t(1) << 31), "slot index overflow: B*H*A = %lld does not fit int32",
               (long long)(B * H * *A));
    return 0;
}

template <typename T>
static int rn_launch_addr_fwd(const RnAddrFwdParams &p, int kpl, int ppl, int grid, cudaStream_t stream) {
#define RN_CASE(KP, PP)                                                                              \
    if (kpl == KP && ppl == PP) {                                                                    \
        rn_addr_fwd_kernel<T, KP, PP><<<grid, RN_ADDR_WARPS * 32, 0, stream>>>(p);                   \
        return 0;                                                                                    \
    }
    RN_CASE(1, 1) RN_CASE(1, 2) RN_CASE(1, 4) RN_CASE(2, 1) RN_CASE(2, 2) RN_CASE(2, 4) RN_CASE(4, 1) RN_CASE(4, 2)
    RN_CASE(4, 4)
#undef RN_CASE
    rn_set_error("no address kernel for K-per-lane=%d, P-per-lane=%d", kpl, ppl);
    return 1;
}

extern "C" int rn_addr_fwd(const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides,
                           const int32_t *pos, const int64_t *pos_strides, int32_t *idx, float *val,
                           const int64_t *out_strides, int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E,
                           int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm, int w_neg, int r_neg,
                           int encode_batch, int device, void *stream) {
    rn_clear_error();
    int64_t A = 0;
    if (int rc = rn_check_addr_dims(B, H, U, P, T, E, Kw, Kr, w_re_norm, r_re_norm, dtype, &A)) return rc;
    RN_REQUIRE(w_addr && pos && idx && val && addr_strides && pos_strides && out_strides, "null pointer argument");
    RN_REQUIRE((r_addr != nullptr) == (Kr > 0), "r_addr must be given exactly when r_top_k > 0");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);

    rn_prof_reset();
    rn_prof_mark(cudaStream_t(stream));
    if (rn_addr_fwd_fast(w_addr, r_addr, dtype, addr_strides, pos, pos_strides, idx, val, out_strides, B, H, U, P, T, E, A,
                         Kw, Kr, w_re_norm, r_re_norm, w_neg, r_neg, encode_batch, cudaStream_t(stream)) == 0) {
        RN_CUDA(cudaGetLastError());
        rn_prof_mark(cudaStream_t(stream));
        return 0;
    }

    RnAddrFwdParams p{};
    p.addr[0] = w_addr;
    p.addr[1] = r_addr;
    p.sb = addr_strides[0]; p.sh = addr_strides[1]; p.su = addr_strides[2]; p.sp = addr_strides[3]; p.st = addr_strides[4];
    p.pos = pos; p.pb = pos_strides[0]; p.pt = pos_strides[1];
    p.idx = idx; p.val = val;
    p.ob = out_strides[0]; p.oh = out_strides[1]; p.ok = out_strides[2]; p.ot = out_strides[3];
    p.B = int(B); p.H = int(H); p.U = int(U); p.P = int(P); p.T = int(T); p.E = int(E); p.A = int(A);
    p.K[0] = int(Kw); p.K[1] = int(Kr);
    p.re_norm[0] = float(w_re_norm); p.re_norm[1] = float(r_re_norm);
    p.sign[0] = w_neg ? -1.f : 1.f; p.sign[1] = r_neg ? -1.f : 1.f;
    p.encode_batch = encode_batch;
    p.nwhich = r_addr ? 2 : 1;
    p.n_items = B * T * H * p.nwhich;

    const int kpl = rn_per_lane(Kw > Kr ? Kw : Kr), ppl = rn_per_lane(P);
    const int64_t want = (p.n_items + RN_ADDR_WARPS - 1) / RN_ADDR_WARPS;
    const int64_t cap = int64_t(rn_sm_count(device)) * 16;
    const int grid = int(want < cap ? want : cap);
    int rc;
    rn_prof_reset();
    rn_prof_mark(cudaStream_t(stream));
    if (dtype == RN_F32) rc = rn_launch_addr_fwd<float>(p, kpl, ppl, grid, cudaStream_t(stream));
    else if (dtype == RN_F16) rc = rn_launch_addr_fwd<__half>(p, kpl, ppl, grid, cudaStream_t(stream));
    else rc = rn_launch_addr_fwd<__nv_bfloat16>(p, kpl, ppl, grid, cudaStream_t(stream));
    if (rc) return rc;
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(cudaStream_t(stream));
    return 0;
}

template <typename T>
static int rn_launch_addr_bwd(const RnAddrBwdParams &p, int ppl, int grid, cudaStream_t stream) {
    if (ppl == 1) rn_addr_bwd_kernel<T, 1><<<grid, RN_ADDR_WARPS * 32, 0, stream>>>(p);
    else if (ppl == 2) rn_addr_bwd_kernel<T, 2><<<grid, RN_ADDR_WARPS * 32, 0, stream>>>(p);
    else rn_addr_bwd_kernel<T, 4><<<grid, RN_ADDR_WARPS * 32, 0, stream>>>(p);
    return 0;
}

extern "C" int rn_addr_bwd(const int32_t *idx, const float *val, const int64_t *out_strides, const float *d_val,
                           const int64_t *dval_strides, const void *w_addr, const void *r_addr, int dtype,
                           const int64_t *addr_strides, const int32_t *pos, const int64_t *pos_strides, void *d_w,
                           void *d_r, const int64_t *dgrad_strides, int64_t B, int64_t H, int64_t U, int64_t P,
                           int64_t T, int64_t E, int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm, int w_neg,
                           int r_neg, int device, void *stream) {
    rn_clear_error();
    int64_t A = 0;
    if (int rc = rn_check_addr_dims(B, H, U, P, T, E, Kw, Kr, w_re_norm, r_re_norm, dtype, &A)) return rc;
    RN_REQUIRE(idx && val && d_val && w_addr && pos && d_w && out_strides && dval_strides && addr_strides &&
                   pos_strides && dgrad_strides,
               "null pointer argument");
    RN_REQUIRE((r_addr != nullptr) == (Kr > 0) && (d_r != nullptr) == (Kr > 0),
               "r_addr and d_r must be given exactly when r_top_k > 0");
    RnDeviceGuard guard(device);
    RN_REQUIRE(guard.ok, "cannot make device %d current", device);

    rn_prof_reset();
    rn_prof_mark(cudaStream_t(stream));
    if (rn_addr_bwd_fast(idx, val, out_strides, d_val, dval_strides, w_addr, r_addr, dtype, addr_strides, pos, pos_strides,
                         d_w, d_r, dgrad_strides, B, H, U, P, T, E, A, Kw, Kr, w_re_norm, r_re_norm, w_neg, r_neg,
                         cudaStream_t(stream)) == 0) {
        RN_CUDA(cudaGetLastError());
        rn_prof_mark(cudaStream_t(stream));
        return 0;
    }

    RnAddrBwdParams p{};
    p.idx = idx; p.val = val;
    p.ob = out_strides[0]; p.oh = out_strides[1]; p.ok = out_strides[2]; p.ot = out_strides[3];
    p.d_val = d_val;
    p.gb = dval_strides[0]; p.gh = dval_strides[1]; p.gk = dval_strides[2]; p.gt = dval_strides[3];
    p.addr[0] = w_addr; p.addr[1] = r_addr;
    p.sb = addr_strides[0]; p.sh = addr_strides[1]; p.su = addr_strides[2]; p.sp = addr_strides[3]; p.st = addr_strides[4];
    p.pos = pos; p.pb = pos_strides[0]; p.pt = pos_strides[1];
    p.d_addr[0] = d_w; p.d_addr[1] = d_r;
    p.db = dgrad_strides[0]; p.dh = dgrad_strides[1]; p.du = dgrad_strides[2]; p.dp = dgrad_strides[3]; p.dt = dgrad_strides[4];
    p.B = int(B); p.H = int(H); p.U = int(U); p.P = int(P); p.T = int(T); p.E = int(E); p.A = int(A);
    p.K[0] = int(Kw); p.K[1] = int(Kr);
    p.re_norm[0] = float(w_re_norm); p.re_norm[1] = float(r_re_norm);
    p.sign[0] = w_neg ? -1.f : 1.f; p.sign[1] = r_neg ? -1.f : 1.f;
    p.nwhich = r_addr ? 2 : 1;
    p.n_items = B * T * H * p.nwhich;

    const int ppl = rn_per_lane(P);
    const int64_t want = (p.n_items + RN_ADDR_WARPS - 1) / RN_ADDR_WARPS;
    const int64_t cap = int64_t(rn_sm_count(device)) * 16;
    const int grid = int(want < cap ? want : cap);
    if (dtype == RN_F32) rn_launch_addr_bwd<float>(p, ppl, grid, cudaStream_t(stream));
    else if (dtype == RN_F16) rn_launch_addr_bwd<__half>(p, ppl, grid, cudaStream_t(stream));
    else rn_launch_addr_bwd<__nv_bfloat16>(p, ppl, grid, cudaStream_t(stream));
    RN_CUDA(cudaGetLastError());
    rn_prof_mark(cudaStream_t(stream));
    return 0;
}
