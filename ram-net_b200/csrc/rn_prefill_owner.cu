// Prefill forward, slot-owner form: one thread-block CLUSTER of 16 CTAs per (batch, head).
//
// Replaces gather_segment + ramnet_ops::topk_segment_forward / topk_segment_forward_
// (packages/ramnet-ops/src/ramnet_ops/impl/cuda_impl.py:72-141,
//  packages/ramnet-ops/csrc/ram_attn_segment_parallel.cu:241-416) for the model shapes
// (C = 128, A <= 4096, 16-bit values): every event is decoded ONCE and moves a whole 512-byte row.
//
// Ownership.  Slot a = 16 * row + lo belongs to CTA (lo ^ row ^ (row >> 4) ^ (row >> 8)) & 15 of the
// cluster and, inside it, to worker warp row & 15.  The CTA keeps its A / 16 rows (all 128 channels,
// fp32) and their mass in shared memory for the whole sequence: 128 KB of state per CTA, 2 MB per
// cluster.  One warp owns a row for good, so the events of a slot are applied in time order without
// any lock, and a row access is one conflict-free 16-byte access per lane.
//
// Time is cut into chunks of 64 tokens.  Per chunk, three stages run one behind the other:
//   D  distribute (4 extra warps per CTA): CTA s reads idx / val of tokens 4s .. 4s+3 of the chunk
//      (one warp per token, one lane per Top-K entry), counting-sorts the <= 128 live events by
//      (owner CTA, owner warp) and pushes them through distributed shared memory into the owners'
//      queues, with a table (start, count) per owner warp.  No global sort, no event workspace.
//   E  events (16 worker warps): a warp gathers its events of the chunk (time order), resolves the
//      scalar mass recurrence and the gains / read coefficients for them, then applies them two at
//      a time: write  row += gain * (x_t - row);  read  push coef * row into the buffer of the CTA
//      that owns the token (again through distributed shared memory).
//   R  reduce: CTA s sums the K read rows of its 4 tokens in fixed order and stores y once, in the
//      I/O dtype.  Deterministic: no floating-point atomics anywhere.
// x arrives by 1-D bulk async copies (TMA, mbarrier completion, bounded wait) one chunk ahead.
// Two hardware cluster barriers per chunk; the second one is split (arrive after R, wait before the
// next chunk's first push).  No multicast copies and no peer-GPU memory.
//
// Measured on B200 (B8 T16384 H16 U2 P64 K16 C128, bf16): 27.0 ms, against 11.9 ms for the schedule +
// channel-slice kernels, so this kernel is opt-in (rn_gsu_owner_enable).  Why: only 7 such clusters are
// resident (112 of 148 SMs); a coalesced 512-byte row pushed through distributed shared memory moves at
// 16 B/clk per SM (3.5 TB/s over the GPU, an eighth of local shared memory), which alone bounds the 17 GB
// of read rows at 4.9 ms; the scattered 2/4-byte pushes of D cost ~10,000 cycles per chunk and are the
// critical path; a cluster barrier costs ~480 cycles; and with 20 warps per SM every stage is a chain of
// dependent shared-memory round trips (gather + scalar part ~2,500 cycles, vector part ~2,500, reduce ~850
// per chunk, cycle counters of CTA 0).
#include "rn_prefill.cuh"

constexpr int RN_OWN_NC = 16;                         // CTAs per cluster
constexpr int RN_OWN_NW = 16;                         // worker warps per CTA
constexpr int RN_OWN_ND = 4;                          // distributor warps per CTA = tokens per source CTA
constexpr int RN_OWN_THREADS = (RN_OWN_NW + RN_OWN_ND) * 32;
constexpr int RN_OWN_L = RN_OWN_NC * RN_OWN_ND;       // 64 tokens per chunk
constexpr int RN_OWN_QCAP = RN_OWN_ND * 32;           // most events one source sends to one owner CTA
constexpr int RN_OWN_C = 128;
constexpr int RN_OWN_ROWS = 256;                      // most rows per CTA (A <= 4096)
constexpr int RN_OWN_KR = 16;                         // most read entries per token

// shared-memory layout (bytes)
constexpr int OWN_S = 0;                                                  // float S[ROWS][128]
constexpr int OWN_MASS = OWN_S + RN_OWN_ROWS * RN_OWN_C * 4;              // float mass[ROWS]
constexpr int OWN_QVAL = OWN_MASS + RN_OWN_ROWS * 4;                      // float qval[2][NC][QCAP]
constexpr int OWN_QMETA = OWN_QVAL + 2 * RN_OWN_NC * RN_OWN_QCAP * 4;     // u16 qmeta[2][NC][QCAP]
constexpr int OWN_QTAB = OWN_QMETA + 2 * RN_OWN_NC * RN_OWN_QCAP * 2;     // u16 qtab[2][NC][NW]: start << 8 | count
constexpr int OWN_QGAM = OWN_QTAB + 2 * RN_OWN_NC * RN_OWN_NW * 2;        // float qgam[2][NC][ND]
constexpr int OWN_YBUF = OWN_QGAM + 2 * RN_OWN_NC * RN_OWN_ND * 4;        // float ybuf[ND][KR][128]
constexpr int OWN_YSCAL = OWN_YBUF + RN_OWN_ND * RN_OWN_KR * RN_OWN_C * 4;  // float yscal[ND][KR]
constexpr int OWN_XS = OWN_YSCAL + RN_OWN_ND * RN_OWN_KR * 4;             // 16-bit xs[2][L][128]
constexpr int OWN_CNT = OWN_XS + 2 * RN_OWN_L * RN_OWN_C * 2;             // u8 cnt[2][ND][256]
constexpr int OWN_START = OWN_CNT + 2 * RN_OWN_ND * 256;                  // u8 start[256]
constexpr int OWN_WSRC = OWN_START + 256;                                 // u32 wsrc[NW][16]
constexpr int OWN_MISC = OWN_WSRC + RN_OWN_NW * 16 * 4;                   // rvalid[2][ND] u32 | sumr[2][ND] f32 | fail u32 | mbar[2] u64
constexpr int OWN_SMEM = OWN_MISC + 128;
static_assert(OWN_SMEM <= 227 * 1024, "owner kernel shared memory");
static_assert(OWN_XS % 128 == 0 && OWN_YBUF % 16 == 0 && (OWN_MISC + 80) % 8 == 0, "alignment");

struct RnOwnParams {
    const int32_t *idx;
    const float *val;
    int64_t ib, ih, ik, it;
    const void *x;
    int64_t xb, xh, xt;
    const void *gamma;
    int64_t gb, gh, gt;
    const uint8_t *mask;
    int64_t mb, mt;
    void *y;
    int64_t yb, yh, yt;
    const float *slot_in;
    float *slot_out;
    const float *mass_in;
    float *mass_out;
    int B, H, T, A, Kw, Kr, nchunks, rows;
    int mass_aware;
    float eps;
    int *status;
    long long *prof;  // optional: 8 cycle counters of cluster 0 / CTA 0 (benchmark aid), else nullptr
};

// ---- cluster primitives ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t rn_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t rn_mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void rn_st_cluster_v4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void rn_st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void rn_st_cluster_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void rn_st_cluster_u16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u16 [%0], %1;" ::"r"(addr), "h"(uint16_t(v)) : "memory");
}
__device__ __forceinline__ void rn_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void rn_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ void rn_dist_sync() { asm volatile("bar.sync 1, %0;" ::"n"(RN_OWN_ND * 32) : "memory"); }

// slot of row `row` in CTA `rank`, and the inverse maps
__device__ __forceinline__ uint32_t rn_own_fold(uint32_t row) { return (row ^ (row >> 4) ^ (row >> 8)) & 15u; }
__device__ __forceinline__ uint32_t rn_own_slot(uint32_t row, uint32_t rank) { return (row << 4) | (rank ^ rn_own_fold(row)); }

template <typename T> __device__ __forceinline__ float4 rn_cvt16x4(uint2 raw);
template <> __device__ __forceinline__ float4 rn_cvt16x4<__nv_bfloat16>(uint2 raw) {
    // bf16 -> fp32 is a shift
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                       __uint_as_float(raw.y & 0xffff0000u));
}
template <> __device__ __forceinline__ float4 rn_cvt16x4<__half>(uint2 raw) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T>
__global__ void __launch_bounds__(RN_OWN_THREADS, 1) rn_gsu_owner_kernel(const RnOwnParams p) {
    static_assert(sizeof(T) == 2, "the owner kernel stages 16-bit values");
    extern __shared__ __align__(128) unsigned char sm[];
    float *S = reinterpret_cast<float *>(sm + OWN_S);
    float *massS = reinterpret_cast<float *>(sm + OWN_MASS);
    float *qval = reinterpret_cast<float *>(sm + OWN_QVAL);
    uint16_t *qmeta = reinterpret_cast<uint16_t *>(sm + OWN_QMETA);
    uint16_t *qtab = reinterpret_cast<uint16_t *>(sm + OWN_QTAB);
    float *qgam = reinterpret_cast<float *>(sm + OWN_QGAM);
    float *ybuf = reinterpret_cast<float *>(sm + OWN_YBUF);
    float *yscal = reinterpret_cast<float *>(sm + OWN_YSCAL);
    T *xs = reinterpret_cast<T *>(sm + OWN_XS);
    uint8_t *cntT = sm + OWN_CNT;
    uint8_t *startT = sm + OWN_START;
    uint32_t *wsrc = reinterpret_cast<uint32_t *>(sm + OWN_WSRC);
    uint32_t *rvalid = reinterpret_cast<uint32_t *>(sm + OWN_MISC);
    float *sumr = reinterpret_cast<float *>(sm + OWN_MISC + 32);
    volatile uint32_t *fail = reinterpret_cast<volatile uint32_t *>(sm + OWN_MISC + 64);
    uint64_t *mbar = reinterpret_cast<uint64_t *>(sm + OWN_MISC + 80);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = rn_cluster_rank();
    const int bh = blockIdx.x / RN_OWN_NC;
    const int b = bh / p.H, h = bh % p.H;
    const int A = p.A, rows = p.rows, Kw = p.Kw, Kr = p.Kr, KT = p.Kw + p.Kr, T_ = p.T;
    const bool worker = warp < RN_OWN_NW;
    const int dw = warp - RN_OWN_NW;  // distributor index = token of this CTA's group (distributor warps only)
    const unsigned lt = (1u << lane) - 1u;

    // ---- set-up: this CTA's rows and their mass --------------------------------------------------
    {
        const float *src = p.slot_in + int64_t(bh) * A * RN_OWN_C;
        for (int r = warp; r < rows; r += RN_OWN_THREADS / 32)
            *reinterpret_cast<float4 *>(S + r * RN_OWN_C + lane * 4) =
                *reinterpret_cast<const float4 *>(src + int64_t(rn_own_slot(r, crank)) * RN_OWN_C + lane * 4);
        const float *msrc = p.mass_in + int64_t(bh) * A;
        for (int r = tid; r < rows; r += RN_OWN_THREADS) massS[r] = msrc[rn_own_slot(r, crank)];
        for (int i = tid; i < 2 * RN_OWN_ND * 256 / 4; i += RN_OWN_THREADS) reinterpret_cast<uint32_t *>(cntT)[i] = 0u;
        if (tid == 0) {
            *fail = 0u;
            rn_mbar_init(&mbar[0], 1);
            rn_mbar_init(&mbar[1], 1);
            rn_mbar_fence_init();
        }
    }
    __syncthreads();
    rn_cluster_arrive();  // every CTA of the cluster is set up before anything is pushed into it
    rn_cluster_wait();

    const T *xg = static_cast<const T *>(p.x) + b * p.xb + h * p.xh;
    T *yg = static_cast<T *>(p.y) + b * p.yb + h * p.yh;
    const int64_t ibase = b * p.ib + h * p.ih;
    const bool pow2 = (A & (A - 1)) == 0;

    // ---- distributor state: this warp's token of a chunk, loaded one iteration before it is used -------
    int d_idx = 0;
    float d_val = 0.f, d_gam = 0.f;
    bool d_tok = false;
    auto prefetch_d = [&](int chunk) {
        d_idx = 0;
        d_val = 0.f;
        d_gam = 0.f;
        d_tok = false;
        const int t = chunk * RN_OWN_L + int(crank) * RN_OWN_ND + dw;
        if (chunk < p.nchunks && t < T_) {
            d_tok = p.mask ? p.mask[b * p.mb + t * p.mt] != 0 : true;
            d_gam = rn_to_float<T>(static_cast<const T *>(p.gamma)[b * p.gb + h * p.gh + t * p.gt]);
            if (lane < KT) {
                const int64_t o = ibase + int64_t(lane) * p.ik + int64_t(t) * p.it;
                d_idx = p.idx[o];
                d_val = p.val[o];
            }
        }
    };
    // x rows of a chunk -> xs[chunk & 1] by bulk copies (one distributor warp)
    auto fetch_x = [&](int chunk) {
        if (chunk >= p.nchunks) return;
        const int t0 = chunk * RN_OWN_L;
        const int Lc = min(RN_OWN_L, T_ - t0);
        uint64_t *bar = &mbar[chunk & 1];
        if (lane == 0) rn_mbar_expect_tx(bar, uint32_t(Lc) * RN_OWN_C * 2u);
        __syncwarp();
        for (int r = lane; r < Lc; r += 32)
            rn_bulk_g2s(xs + ((chunk & 1) * RN_OWN_L + r) * RN_OWN_C, xg + int64_t(t0 + r) * p.xt, RN_OWN_C * 2u, bar);
    };
    // D: sort this CTA's events of `chunk` by (owner CTA, owner warp) and push them to the owners
    auto distribute = [&](int chunk) {
        const int buf = chunk & 1;
        uint8_t *cnt = cntT + buf * (RN_OWN_ND * 256);
        const uint32_t a = pow2 ? uint32_t(d_idx) & uint32_t(A - 1) : uint32_t(d_idx % A);
        const float w = fabsf(d_val);
        const bool live = d_tok && lane < KT && w != 0.f;
        const uint32_t row = a >> 4;
        const uint32_t dest = ((a & 15u) ^ rn_own_fold(row)) & 15u, tw = row & 15u, key = dest * 16u + tw;
        const unsigned peers = __match_any_sync(RN_FULL, live ? key : 256u + uint32_t(lane));
        const int rank = __popc(peers & lt);
        if (live && rank == 0) cnt[dw * 256 + key] = uint8_t(__popc(peers));
        const bool live_r = live && lane >= Kw;
        const unsigned rv = __ballot_sync(RN_FULL, live_r) >> Kw;
        const float sr = rn_warp_sum(live_r ? w : 0.f);
        if (lane == 0) {
            rvalid[buf * RN_OWN_ND + dw] = rv;
            sumr[buf * RN_OWN_ND + dw] = sr;
        }
        // the counters of the other parity are cleared for the chunk after this one
        reinterpret_cast<uint2 *>(cntT + (buf ^ 1) * (RN_OWN_ND * 256))[dw * 32 + lane] = make_uint2(0u, 0u);
        rn_dist_sync();
        {
            // thread j of the 128 owns keys 2j, 2j+1 (same owner CTA, neighbouring owner warps)
            const int j = dw * 32 + lane, k0 = 2 * j;
            uint32_t c0 = 0, c1 = 0;
#pragma unroll
            for (int q = 0; q < RN_OWN_ND; ++q) {
                const uint32_t two = *reinterpret_cast<const uint16_t *>(cnt + q * 256 + k0);
                c0 += two & 0xffu;
                c1 += two >> 8;
            }
            const uint32_t pair = c0 + c1;
            uint32_t incl = pair;  // inclusive scan inside the 8 threads of one owner CTA
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) {
                const uint32_t v = __shfl_up_sync(RN_FULL, incl, off, 8);
                if ((lane & 7) >= off) incl += v;
            }
            const uint32_t s0 = incl - pair, s1 = s0 + c0;
            *reinterpret_cast<uint16_t *>(startT + k0) = uint16_t(s0 | (s1 << 8));
            const uint32_t packed = ((s0 << 8) | c0) | (((s1 << 8) | c1) << 16);
            const uint32_t local = rn_smem_u32(qtab + (buf * RN_OWN_NC + int(crank)) * RN_OWN_NW + (k0 & 15));
            rn_st_cluster_u32(rn_mapa(local, uint32_t(k0 >> 4)), packed);
        }
        rn_dist_sync();
        if (live) {
            uint32_t pos = startT[key] + uint32_t(rank);
            for (int q = 0; q < dw; ++q) pos += cnt[q * 256 + key];
            const uint32_t meta = row | (uint32_t(dw) << 9) | (uint32_t(lane) << 11);
            const int slot = (buf * RN_OWN_NC + int(crank)) * RN_OWN_QCAP + int(pos);
            rn_st_cluster_u16(rn_mapa(rn_smem_u32(qmeta + slot), dest), meta);
            rn_st_cluster_f32(rn_mapa(rn_smem_u32(qval + slot), dest), w);
        }
        if (lane < RN_OWN_NC)
            rn_st_cluster_f32(rn_mapa(rn_smem_u32(qgam + (buf * RN_OWN_NC + int(crank)) * RN_OWN_ND + dw), uint32_t(lane)), d_gam);
    };

    // one event on its row (already loaded into `r`)
    auto apply_event = [&](uint32_t meta, float coef, int src, int xbuf, float4 r, float4 *rp) {
        const int tl = int((meta >> 9) & 3u), k = int(meta >> 11);
        if (k < Kw) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(xs + ((xbuf * RN_OWN_L) + src * RN_OWN_ND + tl) * RN_OWN_C + lane * 4);
            const float4 xv = rn_cvt16x4<T>(raw);
            r.x = fmaf(coef, xv.x - r.x, r.x);
            r.y = fmaf(coef, xv.y - r.y, r.y);
            r.z = fmaf(coef, xv.z - r.z, r.z);
            r.w = fmaf(coef, xv.w - r.w, r.w);
            *rp = r;
        } else {
            r.x *= coef; r.y *= coef; r.z *= coef; r.w *= coef;
            const int e = tl * RN_OWN_KR + (k - Kw);
            rn_st_cluster_v4(rn_mapa(rn_smem_u32(ybuf + e * RN_OWN_C + lane * 4), uint32_t(src)), r);
            if (p.mass_aware && lane == 0) rn_st_cluster_f32(rn_mapa(rn_smem_u32(yscal + e), uint32_t(src)), coef);
        }
    };

    // ---- prologue: chunk 0 is distributed before the loop ------------------------------------------------
    if (!worker) {
        prefetch_d(0);
        if (dw == 0) fetch_x(0);
        distribute(0);
        prefetch_d(1);
    }
    rn_cluster_arrive();
    rn_cluster_wait();

    const bool profiled = p.prof != nullptr && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == RN_OWN_NW);
    long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long tmark = profiled ? clock64() : 0;
    auto lap = [&](int slot) {
        if (profiled) {
            const long long now = clock64();
            pc[slot] += now - tmark;
            tmark = now;
        }
    };
    for (int i = 0; i < p.nchunks; ++i) {
        const int buf = i & 1;
        bool bad = false;
        if (!worker) {
            if (dw == 0) fetch_x(i + 1);
            if (i + 1 < p.nchunks) distribute(i + 1);
            prefetch_d(i + 2);
            lap(6);
            if (i > 0) rn_cluster_wait();  // second barrier of the previous chunk
            lap(7);
        } else {
            // ---- x of this chunk has to be here -----------------------------------------------------------
            {
                int ok = 1;
                if (lane == 0) ok = rn_mbar_wait_bounded(&mbar[buf], uint32_t(i >> 1) & 1u) ? 1 : 0;
                ok = __shfl_sync(RN_FULL, ok, 0);
                if (!ok) {
                    bad = true;
                    if (lane == 0) atomicMax(p.status, RN_STATUS_WAIT_TIMEOUT);
                    if (lane < RN_OWN_NC) rn_st_cluster_u32(rn_mapa(rn_smem_u32(const_cast<uint32_t *>(fail)), uint32_t(lane)), 1u);
                    // the copy may still be on its way: give it one more bounded chance before shared memory is given up
                    if (lane == 0) rn_mbar_wait_bounded(&mbar[buf], uint32_t(i >> 1) & 1u, 1ll << 28);
                }
            }
            lap(0);
            // ---- this warp's events of the chunk, in time order -------------------------------------------
            const uint16_t *tab = qtab + buf * RN_OWN_NC * RN_OWN_NW;
            const uint16_t *qm = qmeta + buf * RN_OWN_NC * RN_OWN_QCAP;
            const float *qv = qval + buf * RN_OWN_NC * RN_OWN_QCAP;
            const float *gam = qgam + buf * RN_OWN_NC * RN_OWN_ND;
            uint32_t my_cnt = 0, my_start = 0;
            if (lane < RN_OWN_NC) {
                const uint32_t tv = tab[lane * RN_OWN_NW + warp];
                my_cnt = tv & 0xffu;
                my_start = tv >> 8;
            }
            uint32_t incl = my_cnt;
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) {
                const uint32_t v = __shfl_up_sync(RN_FULL, incl, off);
                if (lane >= off) incl += v;
            }
            const uint32_t n_ev = __shfl_sync(RN_FULL, incl, RN_OWN_NC - 1);
            if (bad) {
                if (i > 0) rn_cluster_wait();
            } else if (n_ev <= 32u) {
                // lane j takes event j of the concatenated list: sources with events announce (source, first
                // event number, queue position) in the order of their first event
                const uint32_t excl = incl - my_cnt;
                const unsigned nonempty = __ballot_sync(RN_FULL, my_cnt != 0u);
                const unsigned firsts = __reduce_or_sync(RN_FULL, (my_cnt != 0u && excl < 32u) ? (1u << excl) : 0u);
                if (my_cnt != 0u) wsrc[warp * 16 + __popc(nonempty & lt)] = uint32_t(lane) | (excl << 8) | (my_start << 16);
                __syncwarp();
                const bool have = uint32_t(lane) < n_ev;
                uint32_t meta = 0, src = 0;
                float wv = 0.f, coef = 0.f;
                if (have) {
                    const uint32_t ws = wsrc[warp * 16 + __popc(firsts & ((2u << lane) - 1u)) - 1];
                    src = ws & 0xffu;
                    const uint32_t pos = (ws >> 16) + uint32_t(lane) - ((ws >> 8) & 0xffu);
                    meta = qm[src * RN_OWN_QCAP + pos];
                    wv = qv[src * RN_OWN_QCAP + pos];
                }
                // scalar part: the mass recurrence of every row (events of one row in lane order = time order)
                const uint32_t row = meta & 0x1ffu;
                const bool wr = int(meta >> 11) < Kw;
                const unsigned peers = __match_any_sync(RN_FULL, have ? row : 512u + uint32_t(lane));
                const int rank = __popc(peers & lt);
                const int depth = int(__reduce_max_sync(RN_FULL, have ? uint32_t(__popc(peers)) : 0u));
                const float alpha = (have && wr) ? rn_alpha(wv, gam[src * RN_OWN_ND + ((meta >> 9) & 3u)]) : 0.f;
                float m_seen = 0.f;  // write: mass after the update; read: mass at the read
                for (int r = 0; r < depth; ++r) {
                    if (have && rank == r) {
                        m_seen = massS[row];
                        if (wr) {
                            m_seen = fmaf(alpha, m_seen, wv);
                            massS[row] = m_seen;
                        }
                    }
                    __syncwarp();
                }
                if (have) coef = wr ? wv / (m_seen + p.eps) : (p.mass_aware ? wv * m_seen : wv);
                lap(1);
                if (i > 0) rn_cluster_wait();  // second barrier of the previous chunk: the read buffers are free
                lap(2);
                // vector part: two events at a time when they are on different rows
                unsigned todo = __ballot_sync(RN_FULL, have);
                while (todo != 0u) {
                    const int j0 = __ffs(todo) - 1;
                    todo &= todo - 1u;
                    const uint32_t m0 = __shfl_sync(RN_FULL, meta, j0);
                    const float c0 = __shfl_sync(RN_FULL, coef, j0);
                    const int s0 = int(__shfl_sync(RN_FULL, src, j0));
                    float4 *rp0 = reinterpret_cast<float4 *>(S + (m0 & 0x1ffu) * RN_OWN_C) + lane;
                    bool two = todo != 0u;
                    const int j1 = two ? __ffs(todo) - 1 : j0;
                    const uint32_t m1 = __shfl_sync(RN_FULL, meta, j1);
                    const float c1 = __shfl_sync(RN_FULL, coef, j1);
                    const int s1 = int(__shfl_sync(RN_FULL, src, j1));
                    two = two && ((m1 ^ m0) & 0x1ffu) != 0u;
                    float4 *rp1 = reinterpret_cast<float4 *>(S + (m1 & 0x1ffu) * RN_OWN_C) + lane;
                    const float4 r0 = *rp0;
                    if (two) {
                        todo &= todo - 1u;
                        const float4 r1 = *rp1;
                        apply_event(m0, c0, s0, buf, r0, rp0);
                        apply_event(m1, c1, s1, buf, r1, rp1);
                    } else {
                        apply_event(m0, c0, s0, buf, r0, rp0);
                    }
                }
            } else {
                // more than 32 events for this warp in one chunk (rare): one by one, straight from the queues
                if (i > 0) rn_cluster_wait();
                for (int s = 0; s < RN_OWN_NC; ++s) {
                    const uint32_t tv = tab[s * RN_OWN_NW + warp];
                    const uint32_t cnt = tv & 0xffu, start = tv >> 8;
                    for (uint32_t e = 0; e < cnt; ++e) {
                        const uint32_t meta = qm[s * RN_OWN_QCAP + start + e];
                        const float wv = qv[s * RN_OWN_QCAP + start + e];
                        const uint32_t row = meta & 0x1ffu;
                        const bool wr = int(meta >> 11) < Kw;
                        float m = massS[row];
                        float coef;
                        __syncwarp();
                        if (wr) {
                            m = fmaf(rn_alpha(wv, gam[s * RN_OWN_ND + ((meta >> 9) & 3u)]), m, wv);
                            if (lane == 0) massS[row] = m;
                            coef = wv / (m + p.eps);
                        } else {
                            coef = p.mass_aware ? wv * m : wv;
                        }
                        __syncwarp();
                        float4 *rp = reinterpret_cast<float4 *>(S + row * RN_OWN_C) + lane;
                        apply_event(meta, coef, s, buf, *rp, rp);
                    }
                }
            }
        }
        if (worker) lap(3);
        // ---- first barrier: the pushes of this chunk's events and of the next chunk's distribution are visible
        rn_cluster_arrive();
        rn_cluster_wait();
        if (worker) lap(4);
        if (*fail != 0u) return;  // some CTA of the cluster lost a copy; reported through the status word

        // ---- R: y of this CTA's tokens ------------------------------------------------------------------
        if (worker) {
            const int tl = warp >> 2, c = (warp & 3) * 32 + lane;
            const int t = i * RN_OWN_L + int(crank) * RN_OWN_ND + tl;
            if (t < T_) {
                const uint32_t rv = rvalid[buf * RN_OWN_ND + tl];
                float scale = 1.f;
                if (p.mass_aware) {
                    float srm = 0.f;
                    for (int k = 0; k < Kr; ++k)
                        if ((rv >> k) & 1u) srm += yscal[tl * RN_OWN_KR + k];
                    scale = sumr[buf * RN_OWN_ND + tl] / (srm + p.eps);
                }
                float acc = 0.f;
                const float *yb = ybuf + tl * RN_OWN_KR * RN_OWN_C + c;
#pragma unroll 4
                for (int k = 0; k < Kr; ++k)
                    if ((rv >> k) & 1u) acc += yb[k * RN_OWN_C];
                yg[int64_t(t) * p.yt + c] = rn_from_float<T>(acc * scale);
            }
        }
        if (worker) lap(5);
        rn_cluster_arrive();  // second barrier (waited for before the next chunk's first push)
    }
    if (p.nchunks > 0) rn_cluster_wait();
    if (profiled) {
        if (warp == 0) for (int q = 0; q < 6; ++q) p.prof[q] = pc[q];
        else { p.prof[6] = pc[6]; p.prof[7] = pc[7]; }
    }

    // ---- state back to global memory ---------------------------------------------------------------------
    {
        float *dst = p.slot_out + int64_t(bh) * A * RN_OWN_C;
        for (int r = warp; r < rows; r += RN_OWN_THREADS / 32)
            *reinterpret_cast<float4 *>(dst + int64_t(rn_own_slot(r, crank)) * RN_OWN_C + lane * 4) =
                *reinterpret_cast<const float4 *>(S + r * RN_OWN_C + lane * 4);
        float *mdst = p.mass_out + int64_t(bh) * A;
        for (int r = tid; r < rows; r += RN_OWN_THREADS) mdst[rn_own_slot(r, crank)] = massS[r];
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <typename T>
static int rn_owner_prepare(int device, int *clusters) {
    // once per device and dtype: opt in to the shared-memory size and the 16-CTA cluster, and ask how many
    // such clusters the device keeps resident (0 = this device cannot run the kernel)
    static int cached[64] = {0};  // 0 unknown, -1 unusable, else clusters + 1
    if (device < 0 || device >= 64) return 1;
    if (cached[device] == 0) {
        int n = 0;
        bool ok = cudaFuncSetAttribute(rn_gsu_owner_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, OWN_SMEM) == cudaSuccess &&
                  cudaFuncSetAttribute(rn_gsu_owner_kernel<T>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        if (ok) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(RN_OWN_NC);
            cfg.blockDim = dim3(RN_OWN_THREADS);
            cfg.dynamicSmemBytes = OWN_SMEM;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = RN_OWN_NC;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            ok = cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void *>(rn_gsu_owner_kernel<T>), &cfg) == cudaSuccess && n > 0;
        }
        if (!ok) cudaGetLastError();  // clear: the caller falls back to the channel-slice kernels
        cached[device] = ok ? n + 1 : -1;
    }
    *clusters = cached[device] > 0 ? cached[device] - 1 : 0;
    return cached[device] > 0 ? 0 : 1;
}

// Shapes the slot-owner kernel takes: C = 128, A a multiple of 16 up to 4096, Kr <= 16, Kw + Kr <= 32, 16-bit
// values whose rows can be bulk-copied (16-byte aligned).  The kernel is OFF unless rn_gsu_owner_enable(1) was
// called (or RN_PREFILL_OWNER=1 is set in the environment): measured on B200 it is slower than the channel-slice
// kernels (see the header of this file), so it is kept as a tested alternative, not as the default.
static int g_owner_enabled = -1;  // -1: take the environment variable
extern "C" int rn_gsu_owner_enable(int on) {
    const int before = g_owner_enabled;
    g_owner_enabled = on ? 1 : 0;
    return before;
}

bool rn_gsu_owner_eligible(int dtype, int64_t A, int64_t C, int64_t Kw, int64_t Kr, const void *x, const int64_t *x_strides,
                           const void *y, const int64_t *y_strides) {
    if (g_owner_enabled < 0) {
        const char *e = getenv("RN_PREFILL_OWNER");
        g_owner_enabled = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    if (!g_owner_enabled) return false;
    if (dtype != RN_F16 && dtype != RN_BF16) return false;
    if (C != RN_OWN_C || A < 16 || A > 16 * RN_OWN_ROWS || (A % 16) != 0) return false;
    if (Kw < 1 || Kr < 1 || Kr > RN_OWN_KR || Kw + Kr > 32) return false;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((x_strides[0] | x_strides[1] | x_strides[2]) & 7) != 0 || x_strides[3] != 1) return false;
    if ((reinterpret_cast<uintptr_t>(y) & 1) != 0 || y_strides[3] != 1) return false;
    return true;
}

// Benchmark aid: device buffer of 8 cycle counters filled by CTA 0 of the next launches (worker warp 0: wait for x,
// gather + scalar part, wait for the read buffers, vector part, first barrier, reduce; distributor warp: distribute,
// its wait).  NULL switches it off.
static long long *g_owner_prof = nullptr;
extern "C" int rn_gsu_owner_profile(long long *device_counters) {
    g_owner_prof = device_counters;
    return 0;
}

// 0 = launched, -1 = this device cannot run the kernel (nothing launched, no error set), > 0 error
int rn_gsu_owner_launch(const RnGsuParams &g, int dtype, int device, cudaStream_t stream) {
    RnOwnParams p{};
    p.idx = g.idx; p.val = g.val; p.ib = g.ib; p.ih = g.ih; p.ik = g.ik; p.it = g.it;
    p.x = g.x; p.xb = g.xb; p.xh = g.xh; p.xt = g.xt;
    p.gamma = g.gamma; p.gb = g.gb; p.gh = g.gh; p.gt = g.gt;
    p.mask = g.mask; p.mb = g.mb; p.mt = g.mt;
    p.y = g.y; p.yb = g.yb; p.yh = g.yh; p.yt = g.yt;
    p.slot_in = g.slot_in; p.slot_out = g.slot_out; p.mass_in = g.mass_in; p.mass_out = g.mass_out;
    p.B = g.B; p.H = g.H; p.T = g.T; p.A = g.A; p.Kw = g.Kw; p.Kr = g.Kr;
    p.nchunks = (g.T + RN_OWN_L - 1) / RN_OWN_L;
    p.rows = g.A / RN_OWN_NC;
    p.mass_aware = g.mass_aware; p.eps = g.eps; p.status = g.status;
    p.prof = g_owner_prof;

    int clusters = 0;
    const int rc = dtype == RN_F16 ? rn_owner_prepare<__half>(device, &clusters) : rn_owner_prepare<__nv_bfloat16>(device, &clusters);
    if (rc != 0) return -1;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(g.B) * unsigned(g.H) * RN_OWN_NC);
    cfg.blockDim = dim3(RN_OWN_THREADS);
    cfg.dynamicSmemBytes = OWN_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = RN_OWN_NC;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (dtype == RN_F16) RN_CUDA(cudaLaunchKernelEx(&cfg, rn_gsu_owner_kernel<__half>, p));
    else RN_CUDA(cudaLaunchKernelEx(&cfg, rn_gsu_owner_kernel<__nv_bfloat16>, p));
    return 0;
}

int rn_gsu_owner_clusters(int dtype, int device) {
    int clusters = 0;
    const int rc = dtype == RN_F16 ? rn_owner_prepare<__half>(device, &clusters) : rn_owner_prepare<__nv_bfloat16>(device, &clusters);
    return rc == 0 ? clusters : 0;
}
