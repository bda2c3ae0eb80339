// Fused-RoPE flash-attention backward (causal or full) for sm_100a: TMA -> shared memory -> in-place rotation of K
// (once) and of every Q tile -> five tcgen05 MMAs per (K block, Q tile) pair with TMEM accumulators.
// 16-bit inputs, D = 128, N % 128 == 0.
//
// Work unit = one K/V block of 128 keys of one (batch, head): the CTA sweeps the query tiles (64 rows each) at or
// below the block's diagonal.  CTAs are persistent (one per SM) and take units from a global counter, the first unit
// of CTA c being c; every role walks the same unit sequence and keeps a running step count, from which ring stages
// and mbarrier parities follow, so the rings run on across units: Q / dO tiles of the next unit are requested while
// the last steps of the current one compute, its K / V block as soon as the last MMA of the current one has completed,
// and that block lands and is rotated while the softmax groups write dV / dK of the current one.
// Per step, with everything transposed so that thread = key row:
//     S^T  = K~ Q~^T                      [128 keys x 64 queries]   (Q~ carries sm_scale*log2e)
//     dP^T = V dO^T                       [128 x 64]
//     P^T  = exp2(S^T - lse2_i),  dS^T = P^T o (dP^T - delta_i)     (CUDA cores)
//     dV  += P^T  dO                      [128 keys x 128]  accumulated in TMEM over the sweep
//     dK~ += dS^T Q~                      [128 keys x 128]  accumulated in TMEM over the sweep
//     dQ~^T = K~^T dS^T                   [128 (head dim) x 64 queries]  -> added to a global fp32 accumulator
// i.e. five tile products per pair (the reference's Triton kernel spends seven, fused_rope_attn.py:341-470).
// dS^T is written to shared memory (fp16, 128-byte swizzle) as the MN-major B operand of dQ~^T and to TMEM (behind P^T, over
// S^T columns its group has already read) as the A operand of dK~ -- the TMEM copy takes 16 KiB per step off the
// shared-memory port, which bounds the step (0.933 -> 0.917 ms at Llama-7B-4K); K~, Q~ and dO serve two MMAs each from one buffer.
//
// Warp roles (768 threads = 6 warpgroups, registers re-divided with setmaxnreg): warp 0 TMA producer; warp 1 MMA
// issuer + TMEM owner (warps 2-3 spare); warps 4-11 two rotation groups (half of the K block once, half of every Q
// tile); warps 12-15 / 16-19 two softmax groups, each taking 32 of the 64 query columns of every step; warps 20-23
// drain dQ~^T from TMEM and add it to the fp32 accumulator with reductions.  After the sweep the softmax groups write
// dV and dK (inverse rotation and the ln2 factor applied in registers).
// TMEM columns: S^T/P^T/dS^T buffers [0,64) [64,128) (P^T of queries 0-31 in columns 0-15 and their dS^T in 16-31, of queries 32-63 in columns 32-47 / 48-63); dP^T/dQ~^T buffers [128,192) [192,256); dV [256,384); dK~ [384,512).
// A separate small kernel turns the fp32 dQ~ accumulator into dQ (inverse rotation, * sm_scale).
//
// Replaces _attn_bwd / _attn_bwd_dkdv / _attn_bwd_dq of the reference (fused-rope/fused_rope_attn.py:341-649).
#include "common.cuh"

namespace corope {
namespace {

constexpr int kD = 128;
constexpr int kBK = 128;                 // keys per CTA
constexpr int kBQ = 64;                  // query rows per step
constexpr int kStages = 3;               // Q / dO ring.  With 2 stages the sweep is latency-bound on this ring (1.56 ms against 1.08 ms
                                         // with 3); a 4th stage gave nothing, so its 32 KiB stage the dQ~ tile for the bulk reduce instead
constexpr int kKVBytes = kBK * kD * 2;   // 32 KiB
constexpr int kKVBox = kKVBytes / 2;
constexpr int kQBytes = kBQ * kD * 2;    // 16 KiB
constexpr int kQBox = kQBytes / 2;
constexpr int kDsBytes = kBK * kBQ * 2;  // 16 KiB
constexpr int kDqBytes = kBQ * kD * 4;   // 32 KiB: dQ~ tile [64 queries][128] fp32, dense, staged for the bulk reduce-add
constexpr int kThreads = 768;             // six warpgroups: control (TMA, MMA, 2 spare) | rotation (2) | softmax A | softmax B | dQ drain
constexpr int kMmaWarp = 1;
constexpr int kRotWarp0 = 4, kSmxWarp0 = 12, kDrainWarp0 = 20;
// setmaxnreg only moves registers inside the CTA's own launch allocation (768 threads x 80): what the softmax groups
// gain must be released by the others first, or their setmaxnreg.inc waits forever.  128 * (48 + 2 * 72 + 2 * 104 + 80) = 768 * 80.
constexpr int kLaunchRegs = 80;
constexpr int kRegsCtl = 48, kRegsRot = 72, kRegsSmx = 104, kRegsDrain = 80;
static_assert(128 * (kRegsCtl + 2 * kRegsRot + 2 * kRegsSmx + kRegsDrain) <= kThreads * kLaunchRegs, "register budget");
constexpr int kHeadChunk = 4;
constexpr int kUnitSlots = 4;
constexpr int kUnitReaders = 1 + 8 + 8 + 4;   // MMA warp, rotation warps, softmax warps, drain warps: one arrival each

enum Bar {
    K_FULL = 0, V_FULL, K_ROT,
    QDO_FULL,                            // + stage
    Q_ROT = QDO_FULL + kStages,
    QDO_EMPTY = Q_ROT + kStages,
    ST_FULL = QDO_EMPTY + kStages,       // + buffer
    P_READY = ST_FULL + 2,
    DQ_FULL = P_READY + 2,
    DQ_EMPTY = DQ_FULL + 2,
    ACC_FULL = DQ_EMPTY + 2,
    DQ_DONE,                             // + buffer: dQ~^T of the step is in TMEM
    UNIT_FULL = DQ_DONE + 2,             // + slot: a unit index has been published in the unit ring
    UNIT_EMPTY = UNIT_FULL + kUnitSlots, // + slot: every role has read it
    NUM_BARS = UNIT_EMPTY + kUnitSlots
};

// Unit order: heads in chunks of kHeadChunk (the CTAs at work at one time then share few heads, so their Q / dO tiles
// and above all the fp32 dQ accumulator rows stay in L2); within a chunk low key blocks first, since they sweep the
// most query tiles.
struct Unit {
    int jb, bh;
};
__device__ __forceinline__ Unit unit_of(int w, int n_kb, int BH, int head_chunk) {
    const int chunk_units = head_chunk * n_kb;
    const int chunk = w / chunk_units, within = w % chunk_units;
    const int heads_here = min(head_chunk, BH - chunk * head_chunk);
    Unit u;
    u.jb = within / heads_here;
    u.bh = chunk * head_chunk + within % heads_here;
    return u;
}
// Heads per chunk: 4 for N >= 4096 (their Q / dO tiles stay in L2), proportionally more for shorter heads so that a chunk
// holds several units per SM (list-scheduling simulation of the Llama-70B-1K shape: 12 % over the ideal makespan with chunks
// of 4 heads, 4 % with 32).
inline int head_chunk_for(int N) { return N >= 4096 ? kHeadChunk : kHeadChunk * 2 * (4096 / (N < 128 ? 128 : N)); }

// Consumer side of the unit ring: the n-th unit of this CTA, or -1 when there is none left (or a wait gave up).
// Called by all 32 lanes of a warp; one arrival per warp.
__device__ __forceinline__ int fetch_unit(uint64_t* bars, volatile int* unit_ring, int n, int lane, int* status, volatile int* abort_flag) {
    const int slot = n % kUnitSlots;
    if (!mbar_wait_warp(&bars[UNIT_FULL + slot], (n / kUnitSlots) & 1, status, UNIT_FULL, abort_flag)) return -1;
    const int w = unit_ring[slot];
    mbar_arrive_warp(&bars[UNIT_EMPTY + slot], lane);
    return w;
}

constexpr size_t kSmemData = 2 * kKVBytes + kStages * 2 * kQBytes + 2 * kDsBytes + kDqBytes + kStages * 2 * kBQ * sizeof(float);
constexpr size_t kSmemSlack = 512;       // room to round the dynamic shared memory base up to 1024 bytes (checked at run time)
constexpr size_t kSmemBytes = kSmemData + NUM_BARS * 8 + 64 + kSmemSlack;
static_assert(kSmemBytes <= 232448, "shared memory budget");

constexpr uint32_t TS0 = 0, TD0 = 128, TDV = 256, TDK = 384;

// kPlain: one query head per K / V head and every tensor's rows evenly spaced (all contiguous MHA calls): the group and
// layout arithmetic folds away at compile time (it measured 1 - 2 % of the kernel when left to run-time flags).
template <typename T, bool kPlain>
__global__ void __launch_bounds__(kThreads, 1)
rope_bwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                      const __grid_constant__ CUtensorMap mapDQ, RopeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = sm;
    uint8_t* sV = sK + kKVBytes;
    uint8_t* sQ = sV + kKVBytes;                       // [stage] Q tile
    uint8_t* sDO = sQ + kStages * kQBytes;             // [stage] dO tile
    uint8_t* sDS = sDO + kStages * kQBytes;            // [2] dS^T
    float* sDQ = reinterpret_cast<float*>(sDS + 2 * kDsBytes);  // dQ~ staging tile
    float* sLD = sDQ + kDqBytes / 4;                            // [stage][lse 64 | delta 64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sLD + kStages * 2 * kBQ);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* unit_ring = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [kUnitSlots]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = p.N;
    const int G = kPlain ? 1 : p.H / p.Hkv;   // query heads per K / V head (1 for the fused-RoPE ops)
    const bool flat_q = kPlain || p.flat_q, flat_do = kPlain || p.flat_do, flat_k = kPlain || p.flat_k, flat_v = kPlain || p.flat_v;
    const int BH = p.B * p.Hkv;           // units are taken per K / V head; a unit sweeps the query tiles of all G heads of its group
    const int n_kb = N / kBK;
    const int n_units = BH * n_kb;
    const bool causal = p.causal != 0;
    // per unit (jb, bh): first query row visited q_first = causal ? jb * kBK : 0 (causal: the block's own diagonal),
    // spg = (N - q_first) / kBQ steps per query head (even) and n_steps = G * spg, so the two-buffer indices of a unit's
    // first step are always 0.  Step s works on query head bh * G + s / spg, rows q_first + (s % spg) * kBQ .. + kBQ - 1.
    // (no division when every K / V head has a single query head: then s < spg)
    auto step_head = [&](int spg, int s) { return G == 1 ? 0 : s / spg; };
    auto step_q0 = [&](int q_first, int spg, int s) { return q_first + (G == 1 ? s : s % spg) * kBQ; };
    auto step_row = [&](int bh, int q_first, int spg, int s) { return (bh * G + step_head(spg, s)) * N + step_q0(q_first, spg, s); };

    if (reinterpret_cast<uintptr_t>(sm) - reinterpret_cast<uintptr_t>(smem_raw) > kSmemSlack) {   // base less aligned than assumed
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, COROPE_DEV_WAIT_EXPIRED | 0xfff);
        return;
    }
    // A non-zero status word means an earlier CTA (of this or a previous launch) gave up on a wait: do not pile up
    // more timeouts behind it.  The word stays set until the host reads and clears it.
    if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(&bars[K_FULL], 1);
        mbar_init(&bars[V_FULL], 1);
        mbar_init(&bars[K_ROT], 8);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars[QDO_FULL + s], 1);
            mbar_init(&bars[Q_ROT + s], 8);
            mbar_init(&bars[QDO_EMPTY + s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars[ST_FULL + b], 1);
            mbar_init(&bars[P_READY + b], 8);
            mbar_init(&bars[DQ_FULL + b], 1);
            mbar_init(&bars[DQ_EMPTY + b], 4);
            mbar_init(&bars[DQ_DONE + b], 1);
        }
        mbar_init(&bars[ACC_FULL], 1);
        for (int i = 0; i < kUnitSlots; ++i) {
            mbar_init(&bars[UNIT_FULL + i], 1);
            mbar_init(&bars[UNIT_EMPTY + i], kUnitReaders);
        }
        fence_mbar_init();
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
        tma_prefetch_desc(&mapDO);
        tma_prefetch_desc(&mapDQ);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // setmaxnreg sits inside each role's branch: placed before the dispatch, the merge point would force the
    // smallest count on all the code that follows
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        reg_dealloc<kRegsCtl>();
        if (lane == 0) {
            int g = 0;                   // steps before this unit
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int slot = n % kUnitSlots;
                if (n >= kUnitSlots && !(ok = mbar_wait(&bars[UNIT_EMPTY + slot], ((n / kUnitSlots) - 1) & 1, p.status, UNIT_EMPTY, abort_flag))) break;
                int w = n == 0 ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(p.sched_counter, 1);
                if (w >= n_units) w = -1;
                unit_ring[slot] = w;
                mbar_arrive(&bars[UNIT_FULL + slot]);
                if (w < 0) break;
                const Unit un = unit_of(w, n_kb, BH, p.head_chunk);
                const int q_first = causal ? un.jb * kBK : 0;
                const int spg = (N - q_first) / kBQ, n_steps = G * spg;
                auto load_step = [&](int s) -> bool {
                    const int gs = g + s, st = gs % kStages;
                    if (gs >= kStages && !mbar_wait(&bars[QDO_EMPTY + st], ((gs / kStages) - 1) & 1, p.status, QDO_EMPTY, abort_flag)) return false;
                    const int qr = step_row(un.bh, q_first, spg, s);   // flat row of the contiguous side inputs (LSE, delta)
                    mbar_arrive_expect_tx(&bars[QDO_FULL + st], 2 * kQBytes + 2 * kBQ * (uint32_t)sizeof(float));
                    if (flat_q) {
                        tma_load_2d(sQ + st * kQBytes, &mapQ, 0, qr, &bars[QDO_FULL + st]);
                        tma_load_2d(sQ + st * kQBytes + kQBox, &mapQ, 64, qr, &bars[QDO_FULL + st]);
                    }
                    if (flat_do) {
                        tma_load_2d(sDO + st * kQBytes, &mapDO, 0, qr, &bars[QDO_FULL + st]);
                        tma_load_2d(sDO + st * kQBytes + kQBox, &mapDO, 64, qr, &bars[QDO_FULL + st]);
                    }
                    if (!flat_q || !flat_do) {   // 4-D maps: (row, head, batch) coordinates
                        const int qhead = un.bh * G + step_head(spg, s), q0 = step_q0(q_first, spg, s);
                        const int qb = qhead / p.H, qh = qhead % p.H;
                        if (!flat_q) {
                            tma_load_4d(sQ + st * kQBytes, &mapQ, 0, q0, qh, qb, &bars[QDO_FULL + st]);
                            tma_load_4d(sQ + st * kQBytes + kQBox, &mapQ, 64, q0, qh, qb, &bars[QDO_FULL + st]);
                        }
                        if (!flat_do) {
                            tma_load_4d(sDO + st * kQBytes, &mapDO, 0, q0, qh, qb, &bars[QDO_FULL + st]);
                            tma_load_4d(sDO + st * kQBytes + kQBox, &mapDO, 64, q0, qh, qb, &bars[QDO_FULL + st]);
                        }
                    }
                    bulk_load_1d(sLD + st * 2 * kBQ, p.lse2 + qr, kBQ * sizeof(float), &bars[QDO_FULL + st]);
                    bulk_load_1d(sLD + st * 2 * kBQ + kBQ, p.delta + qr, kBQ * sizeof(float), &bars[QDO_FULL + st]);
                    return true;
                };
                // the first two Q / dO tiles only need ring stages, which the last steps of the previous unit free: ask
                // for them before waiting for that unit's last MMA (n_steps >= 2)
                if (!(ok = load_step(0) && load_step(1))) break;
                // K and V are read by MMAs up to the previous unit's last step
                if (n > 0 && !(ok = mbar_wait(&bars[ACC_FULL], (n - 1) & 1, p.status, ACC_FULL, abort_flag))) break;
                const int kr = un.jb * kBK, kb = un.bh / p.Hkv, kh = un.bh % p.Hkv;
                mbar_arrive_expect_tx(&bars[K_FULL], kKVBytes);
                tma_load_rows(sK, &mapK, flat_k, 0, kr, kh, kb, p.Hkv, N, &bars[K_FULL]);
                tma_load_rows(sK + kKVBox, &mapK, flat_k, 64, kr, kh, kb, p.Hkv, N, &bars[K_FULL]);
                mbar_arrive_expect_tx(&bars[V_FULL], kKVBytes);
                tma_load_rows(sV, &mapV, flat_v, 0, kr, kh, kb, p.Hkv, N, &bars[V_FULL]);
                tma_load_rows(sV + kKVBox, &mapV, flat_v, 64, kr, kh, kb, p.Hkv, N, &bars[V_FULL]);
                for (int s = 2; ok && s < n_steps; ++s) ok = load_step(s);
                g += n_steps;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        reg_dealloc<kRegsCtl>();
        {
            const bool leader = elect_one();
            constexpr int kTFmt = Elem<T>::kDtype == COROPE_DTYPE_BF16 ? 1 : 0;
            const uint32_t id_st = make_idesc(0, 0, 0, 0, kBK, kBQ);             // S^T : fp16 x fp16, both K-major
            const uint32_t id_dp = make_idesc(kTFmt, kTFmt, 0, 0, kBK, kBQ);     // dP^T: T x T, both K-major
            const uint32_t id_dv = make_idesc(kTFmt, kTFmt, 0, 1, kBK, kD);      // dV  : P^T (TMEM) x dO (MN-major)
            const uint32_t id_dk = make_idesc(0, 0, 0, 1, kBK, kD);              // dK~ : dS^T (K-major) x Q~ (MN-major)
            const uint32_t id_dq = make_idesc(0, 0, 1, 1, kD, kBQ);              // dQ~^T: K~ (MN-major) x dS^T (MN-major)
            constexpr uint32_t kHi = sdesc_hi(1024);
            // The buffers follow one another in shared memory (K | V | Q ring | dO ring | dS^T x 2) and the address field of
            // a descriptor (address >> 4, 14 bits) cannot wrap below 256 KiB, so every descriptor is the one of K plus a
            // constant: one live register instead of eight in this 48-register warp.
            const uint32_t k_lo = sdesc_lo(smem_u32(sK), 0);
            constexpr uint32_t kLboQ = (uint32_t)(kQBox >> 4) << 16, kLboKV = (uint32_t)(kKVBox >> 4) << 16;   // leading-dimension byte offset of the MN-major views
            const uint32_t v_lo = k_lo + (kKVBytes >> 4), q_lo = k_lo + (2 * kKVBytes >> 4), do_lo = q_lo + (kStages * kQBytes >> 4);
            const uint32_t ds_lo = do_lo + (kStages * kQBytes >> 4);
            const uint32_t do_mn = do_lo + kLboQ, q_mn = q_lo + kLboQ, k_mn = k_lo + kLboKV;
            auto issue_st = [&](int st, int b) {      // S^T = K~ Q~^T
                const uint32_t qb = q_lo + st * (kQBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t offA = ((kk >> 2) * kKVBox + (kk & 3) * 32) >> 4, offB = ((kk >> 2) * kQBox + (kk & 3) * 32) >> 4;
                    if (leader) umma_ss2(tmem + TS0 + b * 64, k_lo + offA, kHi, qb + offB, kHi, id_st, kk > 0);
                }
            };
            auto issue_dp = [&](int st, int b) {      // dP^T = V dO^T
                const uint32_t dob = do_lo + st * (kQBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t offA = ((kk >> 2) * kKVBox + (kk & 3) * 32) >> 4, offB = ((kk >> 2) * kQBox + (kk & 3) * 32) >> 4;
                    if (leader) umma_ss2(tmem + TD0 + b * 64, v_lo + offA, kHi, dob + offB, kHi, id_dp, kk > 0);
                }
            };
            auto issue_dq = [&](int b) {              // dQ~^T = K~^T dS^T : K = 128 keys
                const uint32_t dsb = ds_lo + b * (kDsBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    if (leader) umma_ss2(tmem + TD0 + b * 64, k_mn + kk * (2048 >> 4), kHi, dsb + kk * (2048 >> 4), kHi, id_dq, kk > 0);
            };
            auto issue_dvdk = [&](int st, int b, bool acc) {
                const uint32_t dob = do_mn + st * (kQBytes >> 4), qb = q_mn + st * (kQBytes >> 4), dsb = ds_lo + b * (kDsBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kBQ / 16; ++kk)   // dV += P^T dO : K = 64 queries
                    if (leader) umma_ts2(tmem + TDV, tmem + TS0 + b * 64 + (kk >> 1) * 32 + (kk & 1) * 8, dob + kk * (2048 >> 4), kHi, id_dv, (acc || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < kBQ / 16; ++kk)   // dK~ += dS^T Q~ : A = dS^T from TMEM (columns 16-31 / 48-63 of the S^T buffer)
                    if (leader) umma_ts2(tmem + TDK, tmem + TS0 + b * 64 + (kk >> 1) * 32 + 16 + (kk & 1) * 8, qb + kk * (2048 >> 4), kHi, id_dk, (acc || kk > 0) ? 1u : 0u);
            };
            // Q tiles that arrive rotated (pre-pass) are ready as they land; otherwise the rotation groups pass them on
            const int q_bar = p.q_rot != nullptr ? QDO_FULL : Q_ROT;
            int g = 0;                   // steps before this unit
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int w = fetch_unit(bars, unit_ring, n, lane, p.status, abort_flag);
                if (w < 0) break;
                const Unit un = unit_of(w, n_kb, BH, p.head_chunk);
                const int n_steps = G * ((N - (causal ? un.jb * kBK : 0)) / kBQ);
                {
                    const int st0 = g % kStages, b0 = g & 1;
                    ok = mbar_wait_warp(&bars[K_ROT], n & 1, p.status, K_ROT, abort_flag) && mbar_wait_warp(&bars[V_FULL], n & 1, p.status, V_FULL, abort_flag) &&
                         mbar_wait_warp(&bars[q_bar + st0], (g / kStages) & 1, p.status, Q_ROT, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_st(st0, b0);
                    // the dQ~^T of two steps ago (previous unit) has left this buffer
                    if (g >= 2 && !(ok = mbar_wait_warp(&bars[DQ_EMPTY + b0], ((g >> 1) - 1) & 1, p.status, DQ_EMPTY, abort_flag))) break;
                    tc_fence_after();
                    issue_dp(st0, b0);
                    if (leader) umma_commit(&bars[ST_FULL + b0]);
                }
                for (int s = 0; s < n_steps; ++s) {
                    const int gs = g + s, b = gs & 1;
                    if (s + 1 < n_steps) {
                        const int g1 = gs + 1, st1 = g1 % kStages, b1 = g1 & 1;
                        if (!(ok = mbar_wait_warp(&bars[q_bar + st1], (g1 / kStages) & 1, p.status, Q_ROT, abort_flag))) break;
                        tc_fence_after();
                        issue_st(st1, b1);       // S^T first: it does not need the dQ~^T buffer, so it runs while that drains
                        if (g1 >= 2 && !(ok = mbar_wait_warp(&bars[DQ_EMPTY + b1], ((g1 >> 1) - 1) & 1, p.status, DQ_EMPTY, abort_flag))) break;
                        tc_fence_after();
                        issue_dp(st1, b1);
                        if (leader) umma_commit(&bars[ST_FULL + b1]);
                    }
                    if (!(ok = mbar_wait_warp(&bars[P_READY + b], (gs >> 1) & 1, p.status, P_READY, abort_flag))) break;
                    tc_fence_after();
                    issue_dq(b);                           // first, so that its drain starts as early as possible
                    if (leader) umma_commit(&bars[DQ_DONE + b]);
                    // step 0 overwrites dV / dK~: the softmax groups have read the previous unit's out of TMEM before
                    // they arrive on P_READY for this step
                    issue_dvdk(gs % kStages, b, s > 0);
                    if (leader) umma_commit(&bars[DQ_FULL + b]);      // everything that reads dS^T / P^T of this buffer is done
                    if (leader) umma_commit(&bars[QDO_EMPTY + gs % kStages]);
                }
                if (!ok) break;
                if (leader) umma_commit(&bars[ACC_FULL]);
                g += n_steps;
            }
        }
        __syncwarp();
    } else if (warp < kRotWarp0) {
        reg_dealloc<kRegsCtl>();   // spare warps of the control group
    } else if (warp < kSmxWarp0) {
        // ------------------------------------------------------------------ rotation groups
        // Two groups of 128 threads: group r rotates rows [64 r, 64 r + 64) of the K block once, then rows
        // [32 r, 32 r + 32) of every Q tile.
        reg_dealloc<kRegsRot>();
        const int rg = (warp - kRotWarp0) >> 2;
        const int tid = (threadIdx.x - kRotWarp0 * 32) & 127;
        constexpr int kQHalf = kBQ / 2;
        const bool q_pre = p.q_rot != nullptr;   // Q tiles arrive rotated and scaled (pre-pass): nothing to do per step
        int g = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
            const int w = fetch_unit(bars, unit_ring, n, lane, p.status, abort_flag);
            if (w < 0) break;
            const Unit un = unit_of(w, n_kb, BH, p.head_chunk);
            const int q_first = causal ? un.jb * kBK : 0;
            const int spg = (N - q_first) / kBQ, n_steps = G * spg;
            {
                TabRegs<kBQ> trk;
                load_table_regs<kBQ>(trk, p.packed_tab + (size_t)(un.jb * kBK + rg * kBQ) * (kD / 2), tid);
                if (!(ok = mbar_wait_warp(&bars[K_FULL], n & 1, p.status, K_FULL, abort_flag))) break;
                rotate_tile_regs<T, kBQ, kKVBox, 2>(sK + rg * kBQ * 128, trk, tid, 1.0f);
                fence_proxy_async();
                mbar_arrive_warp(&bars[K_ROT], lane);
            }
            if (q_pre) continue;
            TabRegs<kQHalf> tr;
            load_table_regs<kQHalf>(tr, p.packed_tab + (size_t)(q_first + rg * kQHalf) * (kD / 2), tid);
            for (int s = 0; s < n_steps; ++s) {
                const int gs = g + s, st = gs % kStages;
                if (!(ok = mbar_wait_warp(&bars[QDO_FULL + st], (gs / kStages) & 1, p.status, QDO_FULL, abort_flag))) break;
                rotate_tile_regs<T, kQHalf, kQBox, 2>(sQ + st * kQBytes + rg * kQHalf * 128, tr, tid, p.sm_scale * kLog2e);
                fence_proxy_async();
                mbar_arrive_warp(&bars[Q_ROT + st], lane);
                if (s + 1 < n_steps) load_table_regs<kQHalf>(tr, p.packed_tab + (size_t)(step_q0(q_first, spg, s + 1) + rg * kQHalf) * (kD / 2), tid);
            }
            g += n_steps;
        }
    } else if (warp < kDrainWarp0) {
        // ------------------------------------------------------------------ softmax groups (each takes half the query columns of every step)
        reg_alloc<kRegsSmx>();
        const int wg = (warp - kSmxWarp0) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                 // key row within the block
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        int g = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
        const int w = fetch_unit(bars, unit_ring, n, lane, p.status, abort_flag);
        if (w < 0) break;
        const Unit un = unit_of(w, n_kb, BH, p.head_chunk);
        const int jb = un.jb;
        const int q_first = causal ? jb * kBK : 0;
        const int spg = (N - q_first) / kBQ, n_steps = G * spg;
        const int key = jb * kBK + row;
        for (int s = 0; s < n_steps; ++s) {
            const int gs = g + s, u = gs >> 1, st = gs % kStages, b = gs & 1;
            const uint32_t tS = tmem + lane_base + TS0 + b * 64;
            const uint32_t tD = tmem + lane_base + TD0 + b * 64;
            uint8_t* ds_row = sDS + b * kDsBytes + row * 128;
            if (!(ok = mbar_wait_warp(&bars[ST_FULL + b], u & 1, p.status, ST_FULL + b, abort_flag))) break;
            if (!(ok = mbar_wait_warp(&bars[QDO_FULL + st], (gs / kStages) & 1, p.status, QDO_FULL, abort_flag))) break;
            if (u > 0 && !(ok = mbar_wait_warp(&bars[DQ_FULL + b], (u - 1) & 1, p.status, DQ_FULL + b, abort_flag))) break;
            tc_fence_after();
            const float* lse = sLD + st * 2 * kBQ;
            const float* dlt = lse + kBQ;
            const int q0 = step_q0(q_first, spg, s);
            const bool diag = causal && q0 < jb * kBK + kBK;   // some keys of this block lie above the diagonal for these queries
            {
                const int c = wg;   // this group's 32 query columns
                uint32_t rs[32], rd[32];
                COROPE_TMEM_LD32(tS + c * 32, rs);
                COROPE_TMEM_LD32(tD + c * 32, rd);
                tmem_wait_ld();
                uint32_t pp[16], dd[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int c0 = c * 32 + 2 * i;
                    const float2 l2 = *reinterpret_cast<const float2*>(lse + c0);
                    const float2 d2 = *reinterpret_cast<const float2*>(dlt + c0);
                    float p0 = fast_exp2(__uint_as_float(rs[2 * i]) - l2.x);
                    float p1 = fast_exp2(__uint_as_float(rs[2 * i + 1]) - l2.y);
                    if (diag && key > q0 + c0) p0 = 0.f;
                    if (diag && key > q0 + c0 + 1) p1 = 0.f;
                    const float s0 = p0 * (__uint_as_float(rd[2 * i]) - d2.x);
                    const float s1 = p1 * (__uint_as_float(rd[2 * i + 1]) - d2.y);
                    pp[i] = pack2<T>(p0, p1);
                    dd[i] = pack_half2_sat(s0, s1);
                }
                COROPE_TMEM_ST16(tS + c * 32, pp);   // each group writes P^T over the start of its own 32 S^T columns: the other group's S^T may still be unread
                COROPE_TMEM_ST16(tS + c * 32 + 16, dd);   // dS^T behind it, as the A operand of dK~ (TMEM, not shared memory: 16 KiB less through the port per step)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int chunk = (c * 4 + w) ^ (row & 7);
                    *reinterpret_cast<uint4*>(ds_row + chunk * 16) = make_uint4(dd[4 * w], dd[4 * w + 1], dd[4 * w + 2], dd[4 * w + 3]);
                }
            }
            tmem_wait_st();
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive_warp(&bars[P_READY + b], lane);
        }
        // epilogue: group 0 writes dV, group 1 writes dK (inverse rotation, * ln2 because Q~ carried log2e)
        if (ok) ok = mbar_wait_warp(&bars[ACC_FULL], n & 1, p.status, ACC_FULL, abort_flag);
        if (ok) {
            tc_fence_after();
            if (wg == 0) {
                T* dst = reinterpret_cast<T*>(p.dv) + (kPlain ? ((int64_t)un.bh * N + key) * p.sdv.n : row_offset(p.sdv, p.Hkv, un.bh, key));
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    COROPE_TMEM_LD32(tmem + lane_base + TDV + c * 32, r);
                    tmem_wait_ld();
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) d4[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                }
            } else {
                T* dst = reinterpret_cast<T*>(p.dk) + (kPlain ? ((int64_t)un.bh * N + key) * p.sdk.n : row_offset(p.sdk, p.Hkv, un.bh, key));
                const uint32_t* tab = p.packed_tab + (size_t)key * (kD / 2);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r1[32], r2[32];
                    COROPE_TMEM_LD32(tmem + lane_base + TDK + c * 32, r1);
                    COROPE_TMEM_LD32(tmem + lane_base + TDK + 64 + c * 32, r2);
                    tmem_wait_ld();
                    uint32_t o1[16], o2[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint2 tt = __ldg(reinterpret_cast<const uint2*>(tab + c * 32 + 2 * i));
                        const float2 cs0 = unpack_unorm_pair(tt.x), cs1 = unpack_unorm_pair(tt.y);
                        const float a0 = __uint_as_float(r1[2 * i]), a1 = __uint_as_float(r1[2 * i + 1]);
                        const float b0 = __uint_as_float(r2[2 * i]), b1 = __uint_as_float(r2[2 * i + 1]);
                        o1[i] = pack2<T>((a0 * cs0.x + b0 * cs0.y) * kLn2, (a1 * cs1.x + b1 * cs1.y) * kLn2);
                        o2[i] = pack2<T>((b0 * cs0.x - a0 * cs0.y) * kLn2, (b1 * cs1.x - a1 * cs1.y) * kLn2);
                    }
                    uint4* d1 = reinterpret_cast<uint4*>(dst + c * 32);
                    uint4* d2 = reinterpret_cast<uint4*>(dst + 64 + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        d1[i] = make_uint4(o1[4 * i], o1[4 * i + 1], o1[4 * i + 2], o1[4 * i + 3]);
                        d2[i] = make_uint4(o2[4 * i], o2[4 * i + 1], o2[4 * i + 2], o2[4 * i + 3]);
                    }
                }
            }
        }
        tc_fence_before();   // the TMEM reads above are ordered before this warp's next P_READY arrival, on which the next unit's first dV / dK~ MMA waits
        g += n_steps;
        }
    } else {
        // ------------------------------------------------------------------ dQ~^T drain: TMEM -> global fp32 reductions
        // stays at the launch count when kRegsDrain equals it; any other share has to be taken or released here, because the
        // register budget above counts on it and setmaxnreg.inc in another group waits without a time limit
        if constexpr (kRegsDrain < kLaunchRegs) reg_dealloc<kRegsDrain>();
        if constexpr (kRegsDrain > kLaunchRegs) reg_alloc<kRegsDrain>();
        const int quad = warp & 3;
        const int dcol = quad * 32 + lane;                // head-dim index held by this thread (TMEM lane)
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        int g = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
        const int w = fetch_unit(bars, unit_ring, n, lane, p.status, abort_flag);
        if (w < 0) break;
        const Unit un = unit_of(w, n_kb, BH, p.head_chunk);
        const int q_first = causal ? un.jb * kBK : 0;
        const int spg = (N - q_first) / kBQ, n_steps = G * spg;
        for (int s = 0; s < n_steps; ++s) {
            const int gs = g + s, b = gs & 1;
            if (!(ok = mbar_wait_warp(&bars[DQ_DONE + b], (gs >> 1) & 1, p.status, DQ_DONE + b, abort_flag))) break;
            tc_fence_after();
            uint32_t r0[32], r1[32];
            COROPE_TMEM_LD32(tmem + lane_base + TD0 + b * 64, r0);
            COROPE_TMEM_LD32(tmem + lane_base + TD0 + b * 64 + 32, r1);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive_warp(&bars[DQ_EMPTY + b], lane);
            // stage the tile as [query][head dim] (lanes = consecutive head-dim indices: conflict-free), then one thread
            // adds it to the fp32 accumulator with a single bulk reduce.  (256 warp-wide red.global.add.f32 per step straight
            // from the registers, one 128-byte line each, skip the staging tile but measured 8 % slower: 0.992 against 0.917 ms)
            if (threadIdx.x == kDrainWarp0 * 32) bulk_wait_group_read0();   // the previous reduce has finished reading the tile
            named_bar_sync(1, 128);
            float* tile = sDQ + dcol;
#pragma unroll
            for (int i = 0; i < 32; ++i) tile[i * kD] = __uint_as_float(r0[i]);
#pragma unroll
            for (int i = 0; i < 32; ++i) tile[(32 + i) * kD] = __uint_as_float(r1[i]);
            fence_proxy_async();
            named_bar_sync(1, 128);
            if (threadIdx.x == kDrainWarp0 * 32) {
                tma_reduce_add_2d(&mapDQ, 0, step_row(un.bh, q_first, spg, s), sDQ);
                bulk_commit_group();
            }
        }
        g += n_steps;
        }
        if (threadIdx.x == kDrainWarp0 * 32) bulk_wait_group0();   // all reduces have landed before the CTA exits
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// dQ = inverse_rotate(dQ~ accumulator) * sm_scale; one thread per (row, 4 consecutive d < 64): 16-byte loads of the
// accumulator halves and of the packed (cos, sin) table the main kernel used (the caller's own tables may be narrower than
// 64 columns when a D = 64 problem runs zero-padded; the packed table then holds the identity in columns 32..63), 8-byte stores
template <typename T>
__global__ void rope_bwd_dq_finalize_kernel(const float* __restrict__ acc, T* __restrict__ dq, const uint32_t* __restrict__ packed,
                                            size_t rows, int N, float scale, Strides sdq, int H, int flat) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * 16) return;
    const size_t row = idx >> 4;
    const int d = (int)(idx & 15) * 4;
    const int pos = (int)((unsigned)row % (unsigned)N);
    const float4 a1 = *reinterpret_cast<const float4*>(acc + row * kD + d);
    const float4 a2 = *reinterpret_cast<const float4*>(acc + row * kD + d + 64);
    const uint4 t4 = __ldg(reinterpret_cast<const uint4*>(packed + (size_t)pos * (kD / 2) + d));
    const float2 cs[4] = {unpack_unorm_pair(t4.x), unpack_unorm_pair(t4.y), unpack_unorm_pair(t4.z), unpack_unorm_pair(t4.w)};
    const float x1[4] = {a1.x, a1.y, a1.z, a1.w}, x2[4] = {a2.x, a2.y, a2.z, a2.w};
    uint2 o1, o2;
    o1.x = pack2<T>((x1[0] * cs[0].x + x2[0] * cs[0].y) * scale, (x1[1] * cs[1].x + x2[1] * cs[1].y) * scale);
    o1.y = pack2<T>((x1[2] * cs[2].x + x2[2] * cs[2].y) * scale, (x1[3] * cs[3].x + x2[3] * cs[3].y) * scale);
    o2.x = pack2<T>((x2[0] * cs[0].x - x1[0] * cs[0].y) * scale, (x2[1] * cs[1].x - x1[1] * cs[1].y) * scale);
    o2.y = pack2<T>((x2[2] * cs[2].x - x1[2] * cs[2].y) * scale, (x2[3] * cs[3].x - x1[3] * cs[3].y) * scale);
    T* out = dq + (flat ? (int64_t)row * sdq.n : row_offset(sdq, H, (int)((unsigned)row / (unsigned)N), pos));
    *reinterpret_cast<uint2*>(out + d) = o1;
    *reinterpret_cast<uint2*>(out + d + 64) = o2;
}

template <typename T>
int launch_t(const RopeParams& p, int dtype, cudaStream_t s) {
    CUtensorMap mq, mk, mv, mdo, mdq;
    const uint64_t rows = (uint64_t)p.B * p.H * p.N;
    // maps over the caller's tensors with their own strides (2-D when the rows collapse, else 4-D: head dim, row, head, batch);
    // the pre-rotated Q copy is contiguous
    RopeParams pp = p;
    bool fq, fdo, fk, fv;
    if (int e = p.q_rot ? encode_rows_map(&mq, &fq, p.q_rot, p.B, p.H, p.N, kD, contiguous_strides(p.H, p.N, kD), kBQ, 64, COROPE_DTYPE_F16)
                        : encode_rows_map(&mq, &fq, p.q, p.B, p.H, p.N, kD, p.sq, kBQ, 64, dtype))
        return e;
    if (int e = encode_rows_map(&mdo, &fdo, p.d_o, p.B, p.H, p.N, kD, p.sdo, kBQ, 64, dtype)) return e;
    if (int e = encode_rows_map(&mk, &fk, p.k, p.B, p.Hkv, p.N, kD, p.sk, kBK, 64, dtype)) return e;
    if (int e = encode_rows_map(&mv, &fv, p.v, p.B, p.Hkv, p.N, kD, p.sv, kBK, 64, dtype)) return e;
    pp.flat_q = fq; pp.flat_do = fdo; pp.flat_k = fk; pp.flat_v = fv;
    pp.head_chunk = head_chunk_for(p.N);
    if (int e = encode_tensor_map_2d_f32(&mdq, p.dq_acc, rows, kD, kBQ, kD)) return e;
    cudaError_t e = p.dq_acc_zeroed ? cudaSuccess : cudaMemsetAsync(p.dq_acc, 0, rows * kD * sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
    const bool plain = p.H == p.Hkv && fq && fdo && fk && fv && rows_collapse(p.sdk, p.Hkv, p.N) && rows_collapse(p.sdv, p.Hkv, p.N);
    auto kern = plain ? rope_bwd_sm100_kernel<T, true> : rope_bwd_sm100_kernel<T, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const unsigned units = (unsigned)((p.N / kBK) * p.B * p.Hkv);
    const unsigned grid = units < (unsigned)sms ? units : (unsigned)sms;   // persistent: one CTA per SM
    kern<<<grid, kThreads, kSmemBytes, s>>>(mq, mk, mv, mdo, mdq, pp); count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    const size_t n = rows * 16;
    rope_bwd_dq_finalize_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(p.dq_acc, reinterpret_cast<T*>(p.dq), p.packed_tab, rows, p.N,
                                                                              p.sm_scale, p.sdq, p.H, rows_collapse(p.sdq, p.H, p.N) ? 1 : 0); count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

bool rope_bwd_tc_supported(int B, int H, int N, int D, int dtype, int causal) {
    (void)B; (void)H;
    (void)causal;
    return D == kD && (dtype == COROPE_DTYPE_BF16 || dtype == COROPE_DTYPE_F16) && N % kBK == 0;
}

int launch_rope_bwd_tc(const RopeParams& p, int dtype, cudaStream_t s) {
    if (dtype == COROPE_DTYPE_BF16) return launch_t<__nv_bfloat16>(p, dtype, s);
    return launch_t<__half>(p, dtype, s);
}

}  // namespace corope
