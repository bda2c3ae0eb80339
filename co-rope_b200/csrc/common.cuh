// Shared device/host helpers for the corope_b200 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/corope_b200.h"

namespace corope {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// element type helpers
// ---------------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kDtype = COROPE_DTYPE_F32;
    __device__ static float to_f32(float x) { return x; }
    __device__ static float from_f32(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kDtype = COROPE_DTYPE_BF16;
    __device__ static float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
    static constexpr int kDtype = COROPE_DTYPE_F16;
    __device__ static float to_f32(__half x) { return __half2float(x); }
    __device__ static __half from_f32(float x) { return __float2half_rn(x); }
};

__host__ __device__ inline size_t dtype_bytes(int dtype) { return dtype == COROPE_DTYPE_F32 ? 4 : 2; }

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Strides of a [B, H, N, D] tensor in elements; the head-dim stride is always 1.  Tensor-core paths also need every
// stride to be a multiple of 8 elements (16 bytes, the TMA granularity) -- the entry points check that.
struct Strides {
    int64_t b, h, n;
};
__host__ __device__ inline Strides contiguous_strides(int H, int N, int D) {
    Strides st;
    st.n = D;
    st.h = (int64_t)N * D;
    st.b = (int64_t)H * N * D;
    return st;
}
// rows evenly spaced over heads and batch entries: a 2-D [B H N, D] view with row stride st.n exists
__host__ __device__ inline bool rows_collapse(const Strides& st, int H, int N) { return st.h == (int64_t)N * st.n && st.b == (int64_t)H * st.h; }
// element offset of row n of head-slice bh (= b * H + h) of a tensor with H heads
__host__ __device__ inline int64_t row_offset(const Strides& st, int H, int bh, int n) {
    return (int64_t)(bh / H) * st.b + (int64_t)(bh % H) * st.h + (int64_t)n * st.n;
}

// Addressing of flat row index `row` (= (b * H + h) * N + n) of a strided [B, H, N, D] tensor in the elementwise kernels.  The
// host decides once whether the rows are evenly spaced (every contiguous tensor): then the offset is one multiply; the general
// form costs two integer divisions per thread, which these memory-bound kernels (a few 16-byte accesses per thread) would feel.
struct RowAddr {
    Strides st;
    int H, N;
    int flat;
};
inline RowAddr row_addr(const Strides& st, int H, int N) {
    RowAddr a;
    a.st = st; a.H = H; a.N = N;
    a.flat = rows_collapse(st, H, N) ? 1 : 0;
    return a;
}
__host__ __device__ inline int64_t flat_row_offset(const RowAddr& a, size_t row) {
    if (a.flat) return (int64_t)row * a.st.n;
    const unsigned r = (unsigned)row, bh = r / (unsigned)a.N;   // row counts stay below 2^31 (checked at the entry points)
    return row_offset(a.st, a.H, (int)bh, (int)(r - bh * (unsigned)a.N));
}

// Launch parameters common to the fused-RoPE kernels.
struct RopeParams {
    const void* q;
    const void* k;
    const void* v;
    const void* o;      // forward output (read by backward)
    const void* d_o;
    void* out_o;        // forward: o
    void* dq;
    void* dk;
    void* dv;
    float* lse2;        // [B,H,N] log2-domain LSE
    float* delta;       // [B,H,N] rowsum(O * dO)
    float* dq_acc;      // [B,H,N,D] fp32 accumulator of rotated-frame dQ (tensor-core backward)
    const float* cos;
    const float* sin;
    int64_t table_stride;
    const uint32_t* packed_tab;  // [N, D/2] (cos, sin) pairs in 16-bit fixed point, built per call in the workspace
    int B, H, N, D;     // H = number of query heads
    int Hkv;            // number of K / V heads (H % Hkv == 0; query head h reads KV head h / (H / Hkv)); equals H for the fused-RoPE ops
    int no_rope;        // 1 = plain attention: no rotation anywhere (cos / sin are null, the packed table holds the identity)
    int causal;
    float sm_scale;
    int* status;
    int* sched_counter; // zeroed word in the workspace: next work item / unit of the persistent tensor-core kernels
    int head_chunk;     // heads per chunk of the persistent kernels' work order (set by their launchers)
    const void* k_rot;  // forward: [B,H,N,D] fp16, K already rotated by the pre-pass; null = the kernel rotates K tiles itself
    const void* q_rot;  // backward: [B,H,N,D] fp16, Q rotated and scaled by the pre-pass; null = the kernel rotates Q tiles itself
    Strides sq, sk, sv, so, sdo, sdq, sdk, sdv;   // strides of q, k, v, o (forward output or backward input), dO, dq, dk, dv
    int flat_q, flat_k, flat_v, flat_do;          // tensor-core kernels: which of their TMA maps are 2-D (set by the launchers)
    int dq_acc_zeroed;  // backward: the pre-pass has already cleared dq_acc (otherwise the launcher of the main kernel does)
};

struct GqaParams {
    const void* q;
    const void* k;
    const void* v;
    const void* o;
    const void* d_o;
    void* out_o;
    void* dq;
    void* dk;
    void* dv;
    float* lse2;     // [B,Hq,N]
    float* a_diag;   // [B,Hkv,N]
    float* delta;    // [B,Hq,N]
    float* dk_acc;   // [B,Hkv,N,D] fp32
    float* dv_acc;   // [B,Hkv,N,D] fp32
    uint32_t* k_pairs;  // tensor-core forward: [B,Hkv,N,D/2] fp16 (k1, k2) pairs in MMA operand order (workspace)
    __half* v_half;     // tensor-core forward: [B,Hkv,N,D] fp16 copy of V (workspace)
    int use_mma;        // backward: 1 = tensor-core main kernel (k_pairs / v_half are set), 0 = general kernel
    int B, Hq, Hkv, G, N, D;
    float sm_scale;
    float theta;
    int* status;
    Strides sq, sk, sv, so, sdo, sdq, sdk, sdv;   // strides of q, k, v, o (forward output or backward input), dO, dq, dk, dv
};

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// mbarrier / TMA / tcgen05 wrappers (inline PTX).  Every wait is bounded.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival per warp: every lane has finished (and fenced) its part, lane 0 arrives.  Barriers signalled this
// way are initialised with the number of warps, which keeps 128 threads from serialising on one shared word.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false (after recording `id` in *status) when the limit is hit; callers
// then leave their loops and fall through to the common exit path.  try_wait itself blocks for
// a hardware-defined slice, so the limit corresponds to well over a second.
constexpr uint32_t kWaitLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, int* status, int id, volatile int* abort_flag,
                                                  uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, COROPE_DEV_WAIT_EXPIRED | id);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int id, volatile int* abort_flag) {
    return mbar_wait_limited(bar, parity, status, id, abort_flag, kWaitLimit);
}

// Non-blocking probe of a phase, and a bounded spin on it.  try_wait parks the thread and wakes it some hundreds of
// cycles after the phase completes; the MMA issuer sits on the critical path of every step, so it spins instead
// (one warp; it backs off to try_wait after a while so that a long wait does not burn issue slots).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_spin_warp(uint64_t* bar, uint32_t parity, int* status, int id, volatile int* abort_flag) {
    bool done = false;
    for (int it = 0; it < 4096 && !done; ++it) done = mbar_test_wait(bar, parity);
    if (!done) done = mbar_wait(bar, parity, status, id, abort_flag);
    return __all_sync(0xffffffffu, done);
}

// Same, for roles in which all 32 lanes wait: the outcome is made warp-uniform so that the lanes leave together.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int id, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, status, id, abort_flag));
}

// 2-D tiled TMA load into shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// 4-D tiled TMA load (coordinates: head-dim column, row, head, batch) into shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int x, int n, int h, int b, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(n), "r"(h), "r"(b)
        : "memory");
}
// Row loads of a [B, H, N, D] tensor through either kind of map: `flat` = the tensor's rows are evenly spaced over heads and
// batch entries as well (stride_h = N stride_n, stride_b = H stride_h; every contiguous tensor), so a 2-D map [B H N, D]
// addresses it and one coordinate replaces three; otherwise the 4-D map.  (The 2-D form measured 2 - 10 % faster in the
// backward's Q / dO ring, so it stays the path for the common layout.)
__device__ __forceinline__ void tma_load_rows(void* smem_dst, const CUtensorMap* map, bool flat, int x, int n, int h, int b, int H, int N,
                                              uint64_t* bar) {
    if (flat)
        tma_load_2d(smem_dst, map, x, (b * H + h) * N + n, bar);
    else
        tma_load_4d(smem_dst, map, x, n, h, b, bar);
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Bulk reduce-add of a dense shared-memory tile into a 2-D tiled global tensor (element type and the add come from the
// tensor map / the instruction: fp32 add).  Completion is tracked with bulk async-groups of the issuing thread.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// --- tensor memory ---
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// MMA completion -> mbarrier arrive (implies fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor for kind::f16: fp32 accumulator, A/B formats 0 = f16, 1 = bf16,
// a_mn / b_mn = 1 when the operand's M/N extent (not K) is the contiguous one in memory.
__host__ __device__ constexpr uint32_t make_idesc(int a_fmt, int b_fmt, int a_mn, int b_mn, int M, int N) {
    return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// lbo / sbo are byte offsets (multiples of 16).
__device__ __forceinline__ uint64_t make_sdesc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Split form of the same descriptor for the MMA issue loops: a single thread issues every MMA, so the per-MMA
// instruction count is on the critical path (a freshly built 64-bit descriptor per MMA costs ~190 cycles of
// dependent integer work, three times the 64 cycles a 128x128x16 MMA takes to execute).  The high word depends
// only on SBO; the low word is (address >> 4) | (LBO >> 4) << 16, so stepping the start address is one 32-bit add.
__device__ __forceinline__ uint32_t sdesc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t sdesc_hi(uint32_t sbo_bytes) { return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29); }

__device__ __forceinline__ void umma_ss2(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_ts2(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

// TMEM <-> registers: 32 lanes x 32-bit, N consecutive columns per thread.
#define COROPE_TMEM_LD32(taddr, r)                                                                                                  \
    asm volatile(                                                                                                                   \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22," \
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"                                                                              \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),   \
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),      \
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),      \
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                                        \
        : "r"(taddr))

#define COROPE_TMEM_ST32(taddr, r)                                                                                                  \
    asm volatile(                                                                                                                   \
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21," \
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),                                                               \
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),   \
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),     \
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),     \
        "r"(r[31])                                                                                                                  \
        : "memory")

#define COROPE_TMEM_ST16(taddr, r)                                                                                              \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), \
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),       \
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])                                             \
                 : "memory")

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// Elects one lane of a fully converged warp.  The MMA issuer runs its whole loop warp-uniformly (all 32 lanes wait
// on the barriers and compute the descriptors) and only the issue itself is predicated on the elected lane: the
// same loop inside an `if (lane == 0)` branch issued one MMA every ~210 cycles instead of every 64 (measured).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\telect.sync rx|px, 0xffffffff;\n\tselp.u32 %0, 1, 0, px;\n\t}" : "=r"(pred));
    return pred != 0;
}

// register re-allocation between warpgroups (all four warps of a warpgroup must execute the same one)
template <int N> __device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Packed pairs of fp32 in one 64-bit register: add / mul / fma on both lanes with one instruction (one issue slot for
// two results; the pipe runs them at half the warp rate of the scalar forms, so the gain is in issue slots).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// volatile variant: keeps its program order relative to the TMEM loads / stores, which bounds how far the compiler
// can hoist the exponentials of later chunks (and with them the register pressure of the softmax loop)
__device__ __forceinline__ float fast_exp2_ordered(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// two floats -> packed fp16 pair, values beyond the fp16 range saturate to +-65504 instead of becoming inf
__device__ __forceinline__ uint32_t pack_half2_sat(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float2 unpack_half2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
}
__device__ __forceinline__ float2 unpack_bf162(uint32_t u) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(h);
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// (cos, sin) in [-1, 1] as two 16-bit offset-binary fixed-point numbers u = round((x + 1) * 2^15), clamped to
// 65535 (so +1.0 decodes to 1 - 2^-15; 0 and -1 are exact).  Decoding costs one byte-permute and one FMA per
// value and no conversion instruction: float(0x4B000000 | u) = 2^23 + u exactly.
__device__ __forceinline__ uint32_t pack_unorm_pair(float c, float s) {
    float uc = fminf(fmaxf(rintf((c + 1.f) * 32768.f), 0.f), 65535.f);
    float us = fminf(fmaxf(rintf((s + 1.f) * 32768.f), 0.f), 65535.f);
    return (uint32_t)uc | ((uint32_t)us << 16);
}
__device__ __forceinline__ float2 unpack_unorm_pair(uint32_t u) {
    float lo = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7410));  // bytes: u.b0, u.b1, 0x00, 0x4B
    float hi = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7432));  // bytes: u.b2, u.b3, 0x00, 0x4B
    return make_float2(fmaf(lo, 1.f / 32768.f, -257.f), fmaf(hi, 1.f / 32768.f, -257.f));
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) { return unpack_bf162(u); }
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) { return unpack_half2(u); }
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) { return pack_bf162(a, b); }
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) { return pack_half2(a, b); }

// In-place half-layout rotation of a ROWS x 128 tile held as two 128-byte-swizzled ROWS x 64 boxes
// (columns [0,64) and [64,128)).  Element (r, c) of a box sits at r*128 + ((c/8) ^ (r%8))*16 + (c%8)*2, so the
// pair (d, d+64) has the same offset in the two boxes.  8 consecutive threads cover one 128-byte row; 128 threads.
// The result is written as fp16 whatever the input type T.  The packed (cos, sin) rows of the tile (16-bit fixed
// point, see unpack_unorm_pair) are fetched into registers by load_table_regs, which does not depend on the tile
// having landed: callers issue it before waiting for the TMA so that the L2 latency is hidden.
template <int ROWS>
struct TabRegs {
    uint4 t[ROWS / 16 * 2];
};

template <int ROWS>
__device__ __forceinline__ void load_table_regs(TabRegs<ROWS>& tr, const uint32_t* __restrict__ tab, int tid) {
#pragma unroll
    for (int it = 0; it < ROWS / 16; ++it) {
        const int row = it * 16 + (tid >> 3);
        const int c = (tid & 7) ^ (row & 7);
        const uint4* tp = reinterpret_cast<const uint4*>(tab + row * 64 + c * 8);
        tr.t[2 * it] = __ldg(tp);
        tr.t[2 * it + 1] = __ldg(tp + 1);
    }
}

// Rotation of 8 (x1, x2) pairs held as two 16-byte vectors of T (x1: columns d..d+7, x2: columns d+64..d+71) by the 8
// packed table entries t0, t1; k1 / k0 are the table's decode constants with the output scale folded in.  The result
// is fp16 whatever T.  x1' = x1 c - x2 s,  x2' = x2 c + x1 s  (the reference's rotation, fused_rope_attn.py:96-99).
template <typename T>
__device__ __forceinline__ void rotate_vec8(uint4& x1, uint4& x2, const uint4& t0, const uint4& t1, float k1, float k0) {
    uint32_t a[4] = {x1.x, x1.y, x1.z, x1.w};
    uint32_t b[4] = {x2.x, x2.y, x2.z, x2.w};
    const uint32_t cs[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = unpack2<T>(a[i]), fb = unpack2<T>(b[i]);
        const float c0 = fmaf(__uint_as_float(__byte_perm(cs[2 * i], 0x4B000000u, 0x7410)), k1, k0);
        const float s0 = fmaf(__uint_as_float(__byte_perm(cs[2 * i], 0x4B000000u, 0x7432)), k1, k0);
        const float c1 = fmaf(__uint_as_float(__byte_perm(cs[2 * i + 1], 0x4B000000u, 0x7410)), k1, k0);
        const float s1 = fmaf(__uint_as_float(__byte_perm(cs[2 * i + 1], 0x4B000000u, 0x7432)), k1, k0);
        a[i] = pack_half2_sat(fmaf(fa.x, c0, -fb.x * s0), fmaf(fa.y, c1, -fb.y * s1));
        b[i] = pack_half2_sat(fmaf(fb.x, c0, fa.x * s0), fmaf(fb.y, c1, fa.y * s1));
    }
    x1 = make_uint4(a[0], a[1], a[2], a[3]);
    x2 = make_uint4(b[0], b[1], b[2], b[3]);
}

template <typename T, int ROWS, int BOX_BYTES = ROWS * 128, int BATCH = 4>
__device__ __forceinline__ void rotate_tile_regs(uint8_t* tile, const TabRegs<ROWS>& tr, int tid, float scale) {
    constexpr int kBoxBytes = BOX_BYTES;   // distance between the [0,64) and [64,128) column boxes (ROWS may be part of a taller tile)
    constexpr int kIters = ROWS / 16;
    constexpr int kBatch = BATCH;                                    // rows in flight per thread: loads first, then math, then stores
    const float k1 = scale * (1.f / 32768.f), k0 = -257.f * scale;   // decode constants with the scale folded in
    uint8_t* base = tile + (tid >> 3) * 128 + (tid & 7) * 16;
#pragma unroll
    for (int h = 0; h < kIters; h += kBatch) {
        uint4 x1[kBatch], x2[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            x1[u] = *reinterpret_cast<const uint4*>(base + (h + u) * 2048);
            x2[u] = *reinterpret_cast<const uint4*>(base + kBoxBytes + (h + u) * 2048);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            rotate_vec8<T>(x1[u], x2[u], tr.t[2 * (h + u)], tr.t[2 * (h + u) + 1], k1, k0);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            *reinterpret_cast<uint4*>(base + (h + u) * 2048) = x1[u];
            *reinterpret_cast<uint4*>(base + kBoxBytes + (h + u) * 2048) = x2[u];
        }
    }
}

#endif  // __CUDACC__

// Same for a 2-D row-major fp32 tensor without swizzle (box_cols * 4 bytes a multiple of 16, box_cols <= 256): used for
// bulk reduce-add stores of dense shared-memory tiles.
inline int encode_tensor_map_2d_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !sym) return COROPE_ERR_NO_DEVICE;
        fn = (EncodeFn)sym;
    }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 4};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : COROPE_ERR_TENSOR_MAP;
}

// Every kernel launch of the library bumps this counter (read through corope_launch_count()).
void count_launch(int n = 1);
// Diagnostics kept by abi.cu (see include/corope_b200_debug.h): which kernel family an op took last, and the policy in force.
void note_kernel_family(int op, int family);
int kernel_policy();

// ---------------------------------------------------------------------------------------------
// host launchers implemented by the kernel translation units (return cudaError_t as int)
// ---------------------------------------------------------------------------------------------
int launch_rope_fwd_general(const RopeParams& p, int dtype, cudaStream_t s);
int launch_rope_bwd_general(const RopeParams& p, int dtype, cudaStream_t s);
int launch_rope_delta(const RopeParams& p, int dtype, cudaStream_t s);
// tensor-core backward, D = 128, 16-bit: delta, the rotated fp16 copy of Q (scaled by sm_scale * log2e) into p.q_rot and a
// zeroed p.dq_acc in one launch; sets nothing in p
int launch_rope_bwd_prepass(const RopeParams& p, int dtype, cudaStream_t s);
// cos == nullptr packs the identity rotation (plain attention)
int launch_pack_tables(const float* cos, const float* sin, int64_t stride, uint32_t* packed, int N, int half_d, cudaStream_t s, int half_src = -1);
// cos / sin tables [N, half_d] fp32 for positions 0 .. N-1 from per-pair frequencies: angle = float(n) * inv_freq[d]
int launch_synth_tables(const float* inv_freq, float* cos_out, float* sin_out, int N, int half_d, cudaStream_t s);
// x / out: [B, H, N, 64] with strides st (the padded side is contiguous [B*H*N, 128])
int launch_unpad_d64(const void* xp, void* out, const Strides& st, int B, int H, int N, int rope_layout, int dtype, cudaStream_t s);
// one tensor of a batched pad / un-pad launch: the caller's [B, H, N, 64] tensor with its strides and its padded copy
struct PadSpec {
    const void* tensor;   // written by an un-pad
    void* padded;
    Strides strides;
    int H;
    int rope_layout;
};
int launch_pad_d64_many(int n, const PadSpec* specs, int B, int N, bool unpad, int dtype, cudaStream_t s);
int launch_rope_prerotate(const void* x, const Strides& st, void* out_f16, const uint32_t* packed, int B, int H, int N, float scale,
                          int dtype, cudaStream_t s);   // H = heads of x; out is contiguous [B*H*N, 128]
bool rope_fwd_tc_supported(int B, int H, int N, int D, int dtype, int causal);
int launch_rope_fwd_tc(const RopeParams& p, int dtype, cudaStream_t s);
bool rope_bwd_tc_supported(int B, int H, int N, int D, int dtype, int causal);
int launch_rope_bwd_tc(const RopeParams& p, int dtype, cudaStream_t s);
bool gqa_fwd_mma_supported(int N, int D, int dtype);
int launch_gqa_bwd_mma(const GqaParams& p, int dtype, cudaStream_t s);
int launch_gqa_fwd_mma(const GqaParams& p, int dtype, cudaStream_t s);
int launch_gqa_fwd_general(const GqaParams& p, int dtype, cudaStream_t s);
int launch_gqa_bwd_general(const GqaParams& p, int dtype, cudaStream_t s);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
// Encodes a 2-D row-major [rows, cols] tensor of 16-bit elements with a [box_rows, box_cols] box and
// 128-byte swizzle (box_cols * 2 bytes must be 128).  Returns 0 on success.
inline int encode_tensor_map_2d_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                                      uint32_t box_cols, int dtype, uint64_t row_stride_elems = 0) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !sym) return COROPE_ERR_NO_DEVICE;
        fn = (EncodeFn)sym;
    }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {(row_stride_elems ? row_stride_elems : cols) * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = dtype == COROPE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : COROPE_ERR_TENSOR_MAP;
}

// The same for a [B, H, N, D] tensor of 16-bit elements with arbitrary batch / head / row strides (multiples of 8 elements):
// a 4-D map with dimensions (D, N, H, B) and a [box_rows, box_cols] box inside one head.  Rows beyond N read as zeros.
inline int encode_tensor_map_4d_sw128(CUtensorMap* out, const void* base, uint64_t B, uint64_t H, uint64_t N, uint64_t D, const Strides& st,
                                      uint32_t box_rows, uint32_t box_cols, int dtype) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !sym) return COROPE_ERR_NO_DEVICE;
        fn = (EncodeFn)sym;
    }
    cuuint64_t gdim[4] = {D, N, H, B};
    // a dimension of extent 1 is never stepped over, but its stride still has to be a valid one
    cuuint64_t gstride[3] = {(cuuint64_t)st.n * 2, (cuuint64_t)(H > 1 ? st.h : st.n * (int64_t)N) * 2, (cuuint64_t)(B > 1 ? st.b : st.n * (int64_t)N) * 2};
    cuuint32_t box[4] = {box_cols, box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMapDataType dt = dtype == COROPE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(out, dt, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : COROPE_ERR_TENSOR_MAP;
}

// 2-D map when the rows collapse, else 4-D; `flat` tells the kernel which coordinates to use
inline int encode_rows_map(CUtensorMap* out, bool* flat, const void* base, int B, int H, int N, int D, const Strides& st, uint32_t box_rows,
                           uint32_t box_cols, int dtype) {
    *flat = rows_collapse(st, H, N);
    if (*flat) return encode_tensor_map_2d_sw128(out, base, (uint64_t)B * H * N, D, box_rows, box_cols, dtype, (uint64_t)st.n);
    return encode_tensor_map_4d_sw128(out, base, B, H, N, D, st, box_rows, box_cols, dtype);
}

}  // namespace corope
