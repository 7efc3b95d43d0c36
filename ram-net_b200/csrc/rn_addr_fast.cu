// Address kernel built on the thread-per-row decoder (rn_addr_fast.cuh): one thread per
// (batch, token, head, write|read) row, 16-byte vector loads of the contiguous U*P block and
// 16-byte vector stores of the K indices / weights.
#include "rn_addr_fast.cuh"

namespace {
using namespace rn_fast;

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
    // rows of one tensor are adjacent across the CTA: item = which * n_rows + row
    const int64_t item = int64_t(blockIdx.x) * FAST_THREADS + threadIdx.x;
    if (item >= p.n_rows * p.nwhich) return;
    const int which = int(item / p.n_rows);
    const int64_t row = item - int64_t(which) * p.n_rows;
    const int h = int(row % p.H);
    const int t = int((row / p.H) % p.T);
    const int b = int(row / (int64_t(p.H) * p.T));
    const T *src = static_cast<const T *>(p.addr[which]) + b * p.sb + h * p.sh + t * p.st;

    int content[K];
    float weight[K];
    thread_decode<T, U, P, K>(src, p.re_norm[which], content, weight);
    const int shift = (h < p.E) ? rn_pos_mod(p.pos[b * p.pb + t * p.pt], p.A) : 0;
    const int offs = (p.encode_batch ? (b * p.H + h) : h) * p.A;
    const int64_t o = b * p.ob + h * p.oh + t * p.ot + (which ? K : 0);
    int out_i[K];
    float out_v[K];
#pragma unroll
    for (int e = 0; e < K; ++e) {
        out_i[e] = offs + rn_cape(content[e], shift, p.A);
        out_v[e] = p.sign[which] * weight[e];
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
    if (U == 5 && P == 8 && K == 8) return launch_fast<T, 5, 8, 8>(p, stream);  // 32768 slots at the reference's radix limit
    if (U == 4 && P == 8 && K == 16) return launch_fast<T, 4, 8, 16>(p, stream);  // 4096 slots, K above the radix
    return -1;
}


// ------------------------------------------------------------------------------------------
// address backward, specialised: P/8 lanes per row (each lane owns 8 consecutive logits of every digit:
// one 16-byte load / store per digit for 16-bit types), K / (P/8) Top-K entries per lane.  The K entries
// are scattered into a per-row accumulator in shared memory (U*P floats) by digit, then every lane
// reads back its own 8 positions per digit:
//   d logit[u][p] = sum_{k : digit_u(content_k) = p} D'_k  -  softmax_u[p] * (1 - rho) * sum_k D_k
// with D_k = d_val_k * w_k and D'_k = D_k - rho * (w_k / sum w) * sum D.
// ------------------------------------------------------------------------------------------
struct FastBwdParams {
    const int32_t *idx;
    const float *val;
    int64_t ob, oh, ot;      // strides of idx / val; the Kw + Kr entries of a row are contiguous
    const float *d_val;
    int64_t gb, gh, gt;
    const void *addr[2];
    int64_t sb, sh, st;
    void *d_addr[2];
    int64_t db, dh, dt;
    const int32_t *pos;
    int64_t pb, pt;
    int B, H, T, E, A;
    float re_norm[2];
    float sign[2];
    int nwhich;
    int64_t n_rows;          // B*T*H
};

template <typename T> struct Vec8;   // eight consecutive elements
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float *p, float (&x)[8]) {
        const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&x)[8]) {
        reinterpret_cast<float4 *>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
        reinterpret_cast<float4 *>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
};
template <> struct Vec8<__half> {
    static __device__ __forceinline__ void load(const __half *p, float (&x)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            x[2 * i] = f.x; x[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__half *p, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<__half2 *>(&w[i]) = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&x)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
            x[2 * i] = f.x; x[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<__nv_bfloat162 *>(&w[i]) = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <typename T, int U, int P, int K>
__global__ void __launch_bounds__(FAST_THREADS) rn_addr_bwd_fast_kernel(const FastBwdParams p) {
    constexpr int LPR = P / 8;              // lanes per row
    constexpr int RPC = FAST_THREADS / LPR; // rows per CTA
    constexpr int EPL = K / LPR;            // Top-K entries per lane
    constexpr int ROW = U * P + (LPR <= 2 ? 4 : 0);  // accumulator stride: short rows are staggered over the banks
    static_assert(K % LPR == 0 && EPL % 2 == 0, "an even number of Top-K entries per lane");
    __shared__ __align__(16) float accum[RPC][ROW];

    const int tid = threadIdx.x, lr = tid % LPR, rc = tid / LPR;
    const int64_t item = int64_t(blockIdx.x) * RPC + rc;  // rows of one tensor are adjacent: item = which * n_rows + row
    const bool valid = item < p.n_rows * p.nwhich;
    const int64_t it = valid ? item : 0;                   // surplus rows recompute row 0 and store nothing
    const int which = int(it / p.n_rows);
    const int64_t row = it - int64_t(which) * p.n_rows;
    const int h = int(row % p.H);
    const int t = int((row / p.H) % p.T);
    const int b = int(row / (int64_t(p.H) * p.T));
    const float rho = p.re_norm[which];
    const int shift = (h < p.E) ? rn_pos_mod(p.pos[b * p.pb + t * p.pt], p.A) : 0;
    // the lanes of a row are LPR consecutive lanes of one warp
    const unsigned gmask = (LPR >= 32 ? 0xffffffffu : ((1u << LPR) - 1u)) << ((tid & 31) & ~(LPR - 1));

    // ---- this lane's entries -----------------------------------------------------------------------
    const int64_t o = b * p.ob + h * p.oh + t * p.ot + (which ? K : 0) + EPL * lr;
    const int64_t g = b * p.gb + h * p.gh + t * p.gt + (which ? K : 0) + EPL * lr;
    int ce[EPL];
    float we[EPL], de[EPL];
    float dsum = 0.f, wsum = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; e += 2) {
        const int2 ix = *reinterpret_cast<const int2 *>(p.idx + o + e);
        const float2 wv = *reinterpret_cast<const float2 *>(p.val + o + e);
        const float2 dv = *reinterpret_cast<const float2 *>(p.d_val + g + e);
        we[e] = p.sign[which] * wv.x;
        we[e + 1] = p.sign[which] * wv.y;
        de[e] = dv.x * we[e];
        de[e + 1] = dv.y * we[e + 1];
        int c0 = ix.x % p.A + shift, c1 = ix.y % p.A + shift;
        ce[e] = c0 >= p.A ? c0 - p.A : c0;
        ce[e + 1] = c1 >= p.A ? c1 - p.A : c1;
        dsum += de[e] + de[e + 1];
        wsum += we[e] + we[e + 1];
    }
#pragma unroll
    for (int off = 1; off < LPR; off <<= 1) {
        dsum += __shfl_xor_sync(gmask, dsum, off);
        wsum += __shfl_xor_sync(gmask, wsum, off);
    }
    if (rho != 0.f && wsum > 0.f) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) de[e] -= rho * (we[e] / wsum) * dsum;
    }
    const float tail = (1.f - rho) * dsum;

    // ---- softmax of every digit: this lane's 8 logits ------------------------------------------------
    const T *src = static_cast<const T *>(p.addr[which]) + b * p.sb + h * p.sh + t * p.st + lr * 8;
    float sm[U][8];
    bool inactive = false;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        Vec8<T>::load(src + u * P, sm[u]);
        float m = sm[u][0];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, sm[u][i]);
#pragma unroll
        for (int off = 1; off < LPR; off <<= 1) m = fmaxf(m, __shfl_xor_sync(gmask, m, off));
        inactive |= (m == -INFINITY);
        float ssum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sm[u][i] = (m == -INFINITY) ? 0.f : expf(sm[u][i] - m);
            ssum += sm[u][i];
        }
#pragma unroll
        for (int off = 1; off < LPR; off <<= 1) ssum += __shfl_xor_sync(gmask, ssum, off);
        const float scale = ssum > 0.f ? tail / ssum : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sm[u][i] *= scale;  // softmax * (1 - rho) * sum D
    }

    // ---- scatter the entries by digit, read back this lane's positions -------------------------------
    float *acc = accum[rc];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        *reinterpret_cast<float4 *>(acc + u * P + lr * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(acc + u * P + lr * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncwarp(gmask);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        int a = ce[e];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            atomicAdd(acc + u * P + a % P, de[e]);
            a /= P;
        }
    }
    __syncwarp(gmask);
    if (!valid) return;
    T *dst = static_cast<T *>(p.d_addr[which]) + b * p.db + h * p.dh + t * p.dt + lr * 8;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const float4 g0 = *reinterpret_cast<const float4 *>(acc + u * P + lr * 8);
        const float4 g1 = *reinterpret_cast<const float4 *>(acc + u * P + lr * 8 + 4);
        float out[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = inactive ? 0.f : out[i] - sm[u][i];
        Vec8<T>::store(dst + u * P, out);
    }
}

template <typename T, int U, int P, int K>
int launch_bwd_fast(const FastBwdParams &p, cudaStream_t stream) {
    constexpr int RPC = FAST_THREADS / (P / 8);
    const int64_t items = p.n_rows * p.nwhich;
    const int64_t grid = (items + RPC - 1) / RPC;
    rn_addr_bwd_fast_kernel<T, U, P, K><<<unsigned(grid), FAST_THREADS, 0, stream>>>(p);
    return 0;
}

template <typename T>
int dispatch_bwd_fast(const FastBwdParams &p, int U, int P, int K, cudaStream_t stream) {
    if (U == 2 && P == 64 && K == 16) return launch_bwd_fast<T, 2, 64, 16>(p, stream);
    if (U == 3 && P == 32 && K == 8) return launch_bwd_fast<T, 3, 32, 8>(p, stream);
    if (U == 2 && P == 16 && K == 4) return launch_bwd_fast<T, 2, 16, 4>(p, stream);
    if (U == 5 && P == 8 && K == 8) return launch_bwd_fast<T, 5, 8, 8>(p, stream);
    if (U == 4 && P == 8 && K == 16) return launch_bwd_fast<T, 4, 8, 16>(p, stream);
    return -1;
}

}  // namespace

// Returns 0 when a specialised kernel was launched, -1 when the shape / layout has none.
int rn_addr_fwd_fast(const void *w_addr, const void *r_addr, int dtype, const int64_t *addr_strides, const int32_t *pos,
                     const int64_t *pos_strides, int32_t *idx, float *val, const int64_t *out_strides, int64_t B,
                     int64_t H, int64_t U, int64_t P, int64_t T, int64_t E, int64_t A, int64_t Kw, int64_t Kr,
                     double w_re_norm, double r_re_norm, int w_neg, int r_neg, int encode_batch, cudaStream_t stream) {
    if (r_addr != nullptr && Kw != Kr) return -1;
    const bool shape_ok = (U == 2 && P == 64 && Kw == 16) || (U == 3 && P == 32 && Kw == 8) || (U == 2 && P == 16 && Kw == 4) ||
                          (U == 5 && P == 8 && Kw == 8) || (U == 4 && P == 8 && Kw == 16);
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

// Backward of the address decode for the same shapes and layouts; 0 = launched, -1 = use the general kernel.
int rn_addr_bwd_fast(const int32_t *idx, const float *val, const int64_t *out_strides, const float *d_val,
                     const int64_t *dval_strides, const void *w_addr, const void *r_addr, int dtype,
                     const int64_t *addr_strides, const int32_t *pos, const int64_t *pos_strides, void *d_w, void *d_r,
                     const int64_t *dgrad_strides, int64_t B, int64_t H, int64_t U, int64_t P, int64_t T, int64_t E,
                     int64_t A, int64_t Kw, int64_t Kr, double w_re_norm, double r_re_norm, int w_neg, int r_neg,
                     cudaStream_t stream) {
    if (r_addr != nullptr && Kw != Kr) return -1;
    const bool shape_ok = (U == 2 && P == 64 && Kw == 16) || (U == 3 && P == 32 && Kw == 8) || (U == 2 && P == 16 && Kw == 4) ||
                          (U == 5 && P == 8 && Kw == 8) || (U == 4 && P == 8 && Kw == 16);
    if (!shape_ok) return -1;
    const size_t esz = dtype == RN_F32 ? 4 : 2;
    // logits and their gradients: the U*P block of a row contiguous, rows 16-byte aligned (32 for fp32 pairs of float4)
    if (addr_strides[3] != 1 || addr_strides[2] != P || dgrad_strides[3] != 1 || dgrad_strides[2] != P) return -1;
    if (((addr_strides[0] | addr_strides[1] | addr_strides[4] | dgrad_strides[0] | dgrad_strides[1] | dgrad_strides[4]) *
         int64_t(esz)) % 16 != 0)
        return -1;
    if ((reinterpret_cast<uintptr_t>(w_addr) | reinterpret_cast<uintptr_t>(r_addr) | reinterpret_cast<uintptr_t>(d_w) |
         reinterpret_cast<uintptr_t>(d_r)) & 15)
        return -1;
    // the entries of a row contiguous, pairs 8-byte aligned
    if (out_strides[2] != 1 || dval_strides[2] != 1) return -1;
    if (((out_strides[0] | out_strides[1] | out_strides[3] | dval_strides[0] | dval_strides[1] | dval_strides[3]) & 1) != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(val) | reinterpret_cast<uintptr_t>(d_val)) & 7) return -1;
    if (B * T * H * (r_addr ? 2 : 1) >= (int64_t(1) << 31)) return -1;

    FastBwdParams p{};
    p.idx = idx; p.val = val;
    p.ob = out_strides[0]; p.oh = out_strides[1]; p.ot = out_strides[3];
    p.d_val = d_val;
    p.gb = dval_strides[0]; p.gh = dval_strides[1]; p.gt = dval_strides[3];
    p.addr[0] = w_addr; p.addr[1] = r_addr;
    p.sb = addr_strides[0]; p.sh = addr_strides[1]; p.st = addr_strides[4];
    p.d_addr[0] = d_w; p.d_addr[1] = d_r;
    p.db = dgrad_strides[0]; p.dh = dgrad_strides[1]; p.dt = dgrad_strides[4];
    p.pos = pos; p.pb = pos_strides[0]; p.pt = pos_strides[1];
    p.B = int(B); p.H = int(H); p.T = int(T); p.E = int(E); p.A = int(A);
    p.re_norm[0] = float(w_re_norm); p.re_norm[1] = float(r_re_norm);
    p.sign[0] = w_neg ? -1.f : 1.f; p.sign[1] = r_neg ? -1.f : 1.f;
    p.nwhich = r_addr ? 2 : 1;
    p.n_rows = B * T * H;
    if (dtype == RN_F32) return dispatch_bwd_fast<float>(p, int(U), int(P), int(Kw), stream);
    if (dtype == RN_F16) return dispatch_bwd_fast<__half>(p, int(U), int(P), int(Kw), stream);
    return dispatch_bwd_fast<__nv_bfloat16>(p, int(U), int(P), int(Kw), stream);
}
