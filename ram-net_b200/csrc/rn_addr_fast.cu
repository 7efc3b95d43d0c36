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
