// Shared declarations of the prefill (T > 1) gated-sparse-update kernels.
//
// The sequence is cut into time chunks of L tokens.  Inside a chunk every live event (one write
// or one read of one slot) gets a ROUND number: the count of earlier live events of the same
// chunk on the same slot (writes of a token come before its reads).  Events of one round touch
// pairwise different slots, so a round is applied by all threads in parallel with no atomics;
// rounds are separated by barriers.  Two kernels:
//
//   schedule (one CTA per (b,h), chunks in order):   rounds, the mass recurrence and the gain
//       of every write, the (mass-aware) coefficient of every read -> one record per chunk with
//       the events sorted by round.  Channel independent, so done once per (b,h).
//   apply (one CTA per (b,h, channel slice)):   the slice [A][cs] of the slot state stays in
//       shared memory for the whole sequence; the chunk records are streamed into shared memory
//       with 1-D bulk async copies (TMA, mbarrier completion) one chunk ahead; per chunk the
//       rounds are applied (row update / row read into a per-(token,k) buffer), the reads are
//       reduced over k in a fixed order and y is stored.  Deterministic: no floating-point
//       atomics anywhere.
//
// Chunk record (global workspace, 16-byte aligned, fixed size per call); entry e = t * (Kw+Kr) + k
// keeps the order of the decoded addresses, so the record is written and read coalesced:
//   header (16 bytes): u32 R (rounds of this chunk)
//   u32 meta[NEp]:  bits 0-15 slot (narrow format, A <= 65536), 16-23 round, 24 dead (no-op event:
//                   zero weight or masked token)
//   f32 coef[NEp]:  gain of a write / weight of a read (mass-aware scaling folded in)
//   {f32 coef, u32 link}[NEp]:  the same coefficient next to the event's link word: bits 0-15 row of the
//                   slot in the shared-memory slice (rn_row_of_slot),
//                   16-27 the following live event of the chunk on the same slot, 28-29 kind (0 first
//                   event of its slot in the chunk, 2 second event = head of the slot's chain,
//                   3 later), 30 dead, 31 has a
//                   following event (successors are built only when the schedule tables are in shared
//                   memory)
//   u16 heads[8 + NEp/2]:  heads[0] = number of chains, heads[8..] their head events in any order
//   u32 slot[NEp]:  only in the wide format (A > 65536)
// Records built for a backward pass (narrow format only) continue with the mirror image for the sweep
// that runs against time:
//   {f32 coef, u32 link}[NEp]:  link with the PRECEDING event of the slot instead of the following one and
//                   kind 0 = last event of its slot in the chunk, 2 = second to last (head of the backward
//                   chain), 3 = earlier
//   u16 heads[8 + NEp/2]:  the backward chain heads
// The first events (~80 % of a chunk) are applied token-major (dense).  The later events of a slot
// form a chain (head, then link by link); the fast apply kernel walks a chain with the slot row in
// registers.  The backward sweeps and the general apply kernel go round by round over meta[]
// instead.
#pragma once

#include "rn_common.cuh"
#include "rn_gsu.cuh"

constexpr int RN_GSU_THREADS = 256;               // generic apply kernel, scalar backward kernel
constexpr int RN_SCHED_THREADS_MAX = 1024;        // schedule kernel: 2 events per thread when possible
constexpr int RN_GSU_LMAX = 64;                   // longest time chunk
constexpr int RN_GSU_NE_MAX = 4096;               // most events per chunk (L * (Kw + Kr))
constexpr int RN_GSU_RMAX = 2 * RN_GSU_LMAX;      // most rounds in a chunk
constexpr int RN_GSU_HDR_BYTES = 16;

constexpr uint32_t RN_EV_DEAD = 1u << 24;
constexpr uint32_t RN_LINK_DEAD = 1u << 30, RN_LINK_NEXT = 1u << 31;
constexpr int RN_LINK_KIND_SHIFT = 28;
constexpr uint32_t RN_KIND_FIRST = 0, RN_KIND_HEAD = 2, RN_KIND_LATER = 3;

// Row of slot a inside a CTA's shared-memory state slice.  The Top-K addresses of a token are combinations
// of a few best digits, so the rows that a quarter-warp touches in one access (consecutive entries of a
// token) collide on the shared-memory bank groups more often than random rows would when rows are stored
// in slot order.  XOR-ing the low three bits with the low bits of the upper half of the address (the next
// digit for U = 2) sends combinations of the same few digits to different bank groups; measured on the
// config-3 shape this beats both slot order and a hash of all address bits.  A bijection on every aligned
// group of 8 slots (shift >= 3); the link words of a record carry this row, not the slot.
__host__ __device__ inline uint32_t rn_row_of_slot(uint32_t a, int A, int shift) {
    return (A & 7) ? a : a ^ ((a >> shift) & 7u);
}
__host__ __device__ inline int rn_row_shift(int64_t A) {
    int bits = 0;
    while ((int64_t(1) << (bits + 1)) <= A) ++bits;  // floor(log2(A))
    const int s = bits / 2;
    return s < 3 ? 3 : s;
}

__host__ __device__ inline uint32_t rn_ev_pack(uint32_t slot16, int round, bool dead) {
    return (slot16 & 0xffffu) | (uint32_t(round & 0xff) << 16) | (dead ? RN_EV_DEAD : 0u);
}
__host__ __device__ inline int rn_ev_round(uint32_t m) { return int((m >> 16) & 0xffu); }

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
    int B, H, T, A, C, Kw, Kr, L, nchunks, NE, NEp;
    int mass_aware;
    float eps;
    // schedule workspace
    int *status;              // the device's status word (rn_status_word): set when a bounded wait runs out
    unsigned char *records;   // nchunks * B * H records of rec_bytes each
    int64_t rec_bytes;
    int wide;                 // records carry the separate u32 slot array
    uint32_t *claim;          // global claim table (B*H*A) when the tables do not fit shared memory
    float *prev_mass;         // optional: mass of the slot before each write, [(bh*T + t)*Kw + k] (backward)
    float *read_mass;         // optional: mass of the slot at each read, [(bh*T + t)*Kr + k] (mass-aware backward)
    int reverse;              // also emit the backward pairs / heads of every chunk
    int row_shift;            // rn_row_of_slot
    // apply kernel
    int cs;                   // channels per CTA (multiple of 4)
    int nslices;
    int state_in_smem;
};

__host__ __device__ inline int rn_gsu_chunk_len(int Kw, int Kr) {
    int L = RN_GSU_NE_MAX / (Kw + Kr);
    return L > RN_GSU_LMAX ? RN_GSU_LMAX : (L < 1 ? 1 : L);
}

// ---- launch plan shared by the forward and backward entry points ---------------------------------
constexpr int RN_APPLY_THREADS = 1024;  // forward apply kernel
constexpr int RN_SWEEP_THREADS = 512;   // backward replay / reverse kernels

struct RnGsuPlan {
    int L, nchunks, NE, NEp, ept;  // ept: events per thread with RN_GSU_THREADS threads
    int sched_threads, sched_ept;  // schedule kernel launch geometry
    int smem_tables;       // schedule kernel keeps mass + claim tables in shared memory
    size_t sched_smem;
    int wide;              // A > 65536: records carry a separate slot array
    int64_t rec_bytes;
    int reverse;           // records carry the backward links
    int fast;              // fast apply kernel (C % 4 == 0, narrow records, state in shared memory)
    int tpt_log2, ev;      // fast apply kernel: threads per token, events per thread
    int tptb_log2, evb;    // backward sweep kernels (RN_SWEEP_THREADS threads)
    int cs, nslices, state_in_smem;
    size_t apply_smem;
    // workspace layout (byte offsets)
    size_t off_records, off_claim, total;
};

// reverse: the records also carry the backward links (see above); used by the backward entry points
int rn_gsu_plan(int64_t B, int64_t H, int64_t T, int64_t A, int64_t C, int64_t Kw, int64_t Kr, int device, RnGsuPlan *pl,
                int reverse = 0);
int rn_gsu_launch_schedule(const RnGsuParams &p, const RnGsuPlan &pl, int dtype, cudaStream_t stream);
inline size_t rn_align(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- slot-owner forward kernel (rn_prefill_owner.cu): one 16-CTA cluster per (b,h), no schedule workspace ----
bool rn_gsu_owner_eligible(int dtype, int64_t A, int64_t C, int64_t Kw, int64_t Kr, const void *x, const int64_t *x_strides,
                           const void *y, const int64_t *y_strides);
// 0 = launched, -1 = this device cannot keep such a cluster resident (nothing launched), > 0 error (message set)
int rn_gsu_owner_launch(const RnGsuParams &p, int dtype, int device, cudaStream_t stream);
// resident 16-CTA clusters of the kernel on this device (0 = cannot run)
int rn_gsu_owner_clusters(int dtype, int device);

// ---- mbarrier / bulk-copy (TMA 1-D) primitives -----------------------------------------------
__device__ __forceinline__ uint32_t rn_smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void rn_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rn_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void rn_mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void rn_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void rn_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rn_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rn_mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(rn_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` clock cycles (default 2^31, about a second) and reports failure.
__device__ __forceinline__ bool rn_mbar_wait_bounded(uint64_t *bar, uint32_t parity, long long limit = (1ll << 31)) {
    if (rn_mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!rn_mbar_try_wait(bar, parity)) {
        if (clock64() - start > limit) return false;
    }
    return true;
}
// asks the L2 for a contiguous piece of global memory (16-byte aligned, a multiple of 16 bytes) ahead of its use
__device__ __forceinline__ void rn_bulk_prefetch_l2(const void *gptr, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gptr), "r"(bytes) : "memory");
}
// shared -> global bulk copy (one bulk group per commit); wait_read returns once the copies of this thread's
// groups have read their shared-memory source
__device__ __forceinline__ void rn_bulk_s2g(void *dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(rn_smem_u32(src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void rn_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void rn_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void rn_bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     rn_smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(rn_smem_u32(bar))
                 : "memory");
}
