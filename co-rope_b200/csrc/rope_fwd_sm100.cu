// Fused-RoPE flash-attention forward (causal or full) for sm_100a: TMA -> shared memory -> in-place rotation ->
// tcgen05 MMAs with TMEM accumulators -> online softmax in registers.  16-bit inputs, D = 128.
//
// A work item is 256 consecutive query rows (two 128-row tiles, "Q0" and "Q1") of one (batch, head) with the K/V
// tiles 0 .. 2t+1 they can see.  CTAs are persistent (one per SM) and take items from a global counter, heaviest
// first.  Warp roles (896 threads = 7 warpgroups; registers are re-divided between the groups with setmaxnreg):
//   warp 0        TMA producer: fetches work items, loads Q per item and the K ring (3 stages)
//   warp 1        TMA producer: the V ring (2 stages)
//   warp 2        MMA issuer (warp-uniform loop, issue predicated on one elected lane) and TMEM owner;  warp 3 idle
//   warps 4-11    two rotation groups: group r rotates rows [64r, 64r+64) of Q0/Q1 (scaled by sm_scale*log2e, once
//                 per item) and of every K tile as it lands, in place in shared memory, as fp16
//   warps 12-19   two softmax groups of Q0, each taking 64 of the 128 key columns: thread = row; half an S row from
//                 TMEM into registers, half-row max exchanged with the partner group, exp2, row sum, P written back
//                 over S in TMEM, lazy rescale of its 64 O columns in TMEM, final normalise + store
//   warps 20-27   the same for Q1
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i (16-bit) is written over S_i: keys 0-63 in
// columns 0-31, keys 64-127 in columns 64-95 (each softmax group writes only over columns it has already read).
// MMA order per K tile j:  PV0(j) QK0(j+1) | PV1(j) QK1(j+1)  so that one group's softmax overlaps the
// other group's MMAs.
// K tiles come in one of two ways.  By default a pre-pass (rope_prerotate_d128_kernel) has written a rotated fp16 copy
// of K to the workspace and the K ring loads that copy: every K tile is consumed by up to N/256 work items, and rotating
// it in shared memory for each of them cost 14 % of the kernel (issue slots and shared-memory port time that the softmax
// and the MMA operand fetch need), more than the copy's extra HBM traffic.  With p.k_rot == nullptr (kernel policy 2 of
// the diagnostics header, and the entry point that takes no workspace) the rotation groups rotate every K tile in shared
// memory as it lands and nothing rotated is ever written to HBM.  Q is always rotated in shared memory, once per item.
//
// Replaces _attn_fwd / _attn_fwd_inner of the reference (fused-rope/fused_rope_attn.py:47-138, 219-320):
// rotation formula :96-99 / :286-287, exp2-domain softmax :103-114, M = m + log2(l) :316.
#include "common.cuh"

namespace corope {
namespace {

constexpr int kD = 128;
constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kTileBytes = kBM * kD * 2;   // 32 KiB: two 128 x 64 boxes
constexpr int kBoxBytes = kTileBytes / 2;
constexpr int kThreads = 896;          // seven warpgroups: control (TMA K, TMA V, MMA, spare) | rotation (2) | softmax of Q0 (2) | of Q1 (2)
constexpr int kMmaWarp = 2;
constexpr int kRotWarp0 = 4;
constexpr int kSmxWarp0 = 12;
// setmaxnreg only moves registers inside the CTA's own launch allocation (512 threads x 128): the sum must not exceed it
constexpr int kLaunchRegs = 72;        // 65536 / 896 rounded down to a multiple of 8
// 128 * (40 + 2 * 56 + 4 * 88) = 64512 = 896 * 72.  While the rotation groups rotated every K tile in the loop they needed
// the room (40 / 72 / 80 measured 0.437 ms against 0.456 ms at the Llama-7B-4K shape); with K arriving rotated they only
// rotate Q once per item and the registers serve the softmax groups better: 0.387 against 0.401 ms.
constexpr int kRegsCtl = 40, kRegsRot = 56, kRegsSmx = 88;
static_assert(128 * (kRegsCtl + 2 * kRegsRot + 4 * kRegsSmx) <= kThreads * kLaunchRegs, "register budget");
constexpr int kHeadChunk = 8;   // heads per chunk of the work order for N >= 4096 (more for shorter heads, see head_chunk_for)
constexpr int kItemSlots = 4;
constexpr int kItemReaders = 1 + 1 + 8 + 16;   // V producer, MMA warp, rotation warps, softmax warps: one arrival each

enum Bar {
    Q_FULL = 0,                        // +i
    Q_ROT = 2,                         // +i
    K_FULL = 4,                        // +stage
    K_ROT = K_FULL + kKStages,
    K_EMPTY = K_ROT + kKStages,
    V_FULL = K_EMPTY + kKStages,
    V_EMPTY = V_FULL + kVStages,
    S_FULL = V_EMPTY + kVStages,       // +i
    P_FULL = S_FULL + 2,
    O_FULL = P_FULL + 2,
    Q_EMPTY = O_FULL + 2,              // +i: the item's last Q_i K^T has completed, the Q_i buffer may be reloaded
    O_FREE = Q_EMPTY + 2,              // +i: the item's output has been read out of TMEM, O_i may be overwritten
    ITEM_FULL = O_FREE + 2,            // +slot: a work item index has been published in the item ring
    ITEM_EMPTY = ITEM_FULL + kItemSlots,   // +slot: every role has read it
    NUM_BARS = ITEM_EMPTY + kItemSlots
};

constexpr size_t kSmemTiles = (size_t)(2 + kKStages + kVStages) * kTileBytes;
constexpr size_t kXchBytes = 2 * 2 * kBM * sizeof(float);         // half-row maxima / sums exchanged between the two groups of a Q tile
constexpr size_t kSmemSlack = 512;     // room to round the dynamic shared memory base up to 1024 bytes (checked at run time)
constexpr size_t kSmemBytes = kSmemTiles + kXchBytes + NUM_BARS * 8 + 64 + kSmemSlack;
static_assert(kSmemBytes <= 232448, "shared memory budget");  // + alignment slack (tmem slot, abort flag and the item ring live in the 64)

// Work items (one = 256 query rows of one head) in the order CTAs take them: heads in chunks of kHeadChunk so that
// the items in flight at one time share few heads (their K/V stay in L2), heaviest query blocks first inside a chunk.
struct WorkItem {
    int t, bh;
};
__device__ __forceinline__ WorkItem work_item(int w, int n_qt, int BH, int head_chunk) {
    const int chunk_items = head_chunk * n_qt;
    const int chunk = w / chunk_items, within = w % chunk_items;
    const int heads_here = min(head_chunk, BH - chunk * head_chunk);
    WorkItem it;
    it.t = n_qt - 1 - within / heads_here;
    it.bh = chunk * head_chunk + within % heads_here;
    return it;
}
// Heads per chunk: a chunk's K and V should stay in L2 while its items are in flight, and a chunk should hold a few items per
// SM, or the light tail of one chunk and the heavy head of the next leave SMs idle (a list-scheduling simulation of the
// Llama-70B-1K shape: 22 % over the ideal makespan with chunks of 8 heads, 8 % with 64).  8 heads of 4096 rows are 16 MB of
// K + V; shorter heads get proportionally more heads per chunk.
inline int head_chunk_for(int N) { return N >= 4096 ? kHeadChunk : kHeadChunk * (4096 / (N < 128 ? 128 : N)); }

// Consumer side of the item ring: the n-th item of this CTA, or -1 when there is none left (or a wait gave up).
// Warp roles call it with all 32 lanes (one arrival per warp); the V producer calls it from its single thread.
__device__ __forceinline__ int fetch_item(uint64_t* bars, volatile int* item_ring, int n, int lane, bool whole_warp, int* status,
                                          volatile int* abort_flag) {
    const int slot = n % kItemSlots;
    const uint32_t parity = (n / kItemSlots) & 1;
    int w = -1;
    if (whole_warp) {
        if (!mbar_wait_warp(&bars[ITEM_FULL + slot], parity, status, ITEM_FULL, abort_flag)) return -1;
        w = item_ring[slot];
        mbar_arrive_warp(&bars[ITEM_EMPTY + slot], lane);
    } else {
        if (!mbar_wait(&bars[ITEM_FULL + slot], parity, status, ITEM_FULL, abort_flag)) return -1;
        w = item_ring[slot];
        mbar_arrive(&bars[ITEM_EMPTY + slot]);
    }
    return w;
}

// kPlain: one query head per K / V head and every tensor's rows evenly spaced (all contiguous MHA calls): the group and
// layout arithmetic folds away at compile time (it measured 1 - 2 % of the kernel when left to run-time flags).
template <typename T, bool kPlain>
__global__ void __launch_bounds__(kThreads, 1)
rope_fwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, RopeParams p) {
    // P is written in the inputs' own 16-bit format so that V can be used as it lands (tcgen05.mma wants both operands in
    // one format).  For bf16 the row sums are taken from the rounded P, which keeps the normalised weights consistent:
    // measured max-abs error of O at the Llama-7B-4K shape is unchanged (0.0080, rounding of the bf16 output itself 0.0077).
    constexpr bool kPBf16 = Elem<T>::kDtype == COROPE_DTYPE_BF16;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = sm;
    uint8_t* sK = sQ + 2 * kTileBytes;
    uint8_t* sV = sK + kKStages * kTileBytes;
    float* xch = reinterpret_cast<float*>(sV + kVStages * kTileBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xch) + kXchBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* item_ring = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [kItemSlots]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = p.N;
    const int BH = p.B * p.H;
    const int G = kPlain ? 1 : p.H / p.Hkv;   // query heads per K / V head (1 for the fused-RoPE ops); query head bh reads KV head bh / G
    const bool flat_q = kPlain || p.flat_q, flat_k = kPlain || p.flat_k, flat_v = kPlain || p.flat_v;
    // N is a multiple of 128: when it is not a multiple of 256 the last item of a head has only Q0; its Q1 tile (and, causal,
    // the K tile behind the diagonal) lies beyond the head -- TMA fetches the next head's rows there (2-D maps) or zeros (4-D
    // maps and behind the tensor); the results are finite and are not stored
    const int n_qt = (N + 2 * kBM - 1) / (2 * kBM);
    const int n_items = n_qt * BH;
    // K tiles an item sees: up to its diagonal (causal: Q0 one tile less than Q1), or all of them
    const bool causal = p.causal != 0;
    const int nk_all = N / kBN;   // full attention: every tile that lies inside the head
    // Persistent CTAs with a dynamic schedule: the first item of CTA c is c, further ones come from a global counter
    // (heavy items first, so the greedy order balances to a few percent; a static round-robin was 19 % off).  The K
    // producer fetches an item, publishes it in a small shared-memory ring and every other role reads it from there.
    // Every role walks the same item sequence and keeps running counters (K tiles, V tiles, S tiles per group, items) from which ring stages and mbarrier parities follow, so the
    // pipeline runs across item boundaries: the next item's Q and K tiles are loaded and rotated while the current
    // item's last tiles are still in the MMAs and its output is being written.

    if (reinterpret_cast<uintptr_t>(sm) - reinterpret_cast<uintptr_t>(smem_raw) > kSmemSlack) {   // base less aligned than assumed
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, COROPE_DEV_WAIT_EXPIRED | 0xfff);
        return;
    }
    // A non-zero status word means an earlier CTA (of this or a previous launch) gave up on a wait: do not pile up
    // more timeouts behind it.  The word stays set until the host reads and clears it.
    if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars[Q_FULL + i], 1);
            mbar_init(&bars[Q_ROT + i], 8);
            mbar_init(&bars[Q_EMPTY + i], 1);
            mbar_init(&bars[S_FULL + i], 1);
            mbar_init(&bars[P_FULL + i], 8);
            mbar_init(&bars[O_FULL + i], 1);
            mbar_init(&bars[O_FREE + i], 8);
        }
        for (int i = 0; i < kItemSlots; ++i) {
            mbar_init(&bars[ITEM_FULL + i], 1);
            mbar_init(&bars[ITEM_EMPTY + i], kItemReaders);
        }
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(&bars[K_FULL + s], 1);
            mbar_init(&bars[K_ROT + s], 8);
            mbar_init(&bars[K_EMPTY + s], 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(&bars[V_FULL + s], 1);
            mbar_init(&bars[V_EMPTY + s], 1);
        }
        fence_mbar_init();
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < kRotWarp0) {
        // producers and the MMA issuer need few registers: hand the rest to the softmax groups
        reg_dealloc<kRegsCtl>();
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer: Q per item, and the K ring
            if (lane == 0) {
                int gk = 0;
                bool ok = true;
                for (int n = 0; ok; ++n) {
                    const int slot = n % kItemSlots;
                    if (n >= kItemSlots && !(ok = mbar_wait(&bars[ITEM_EMPTY + slot], ((n / kItemSlots) - 1) & 1, p.status, ITEM_EMPTY, abort_flag))) break;
                    int w = n == 0 ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(p.sched_counter, 1);
                    if (w >= n_items) w = -1;
                    item_ring[slot] = w;
                    mbar_arrive(&bars[ITEM_FULL + slot]);
                    if (w < 0) break;
                    const WorkItem wi = work_item(w, n_qt, BH, p.head_chunk);
                    const int nk = causal ? 2 * wi.t + 2 : nk_all;
                    const int qb = wi.bh / p.H, qh = wi.bh % p.H;                       // batch and head coordinates of the 4-D maps
                    const int kb = (wi.bh / G) / p.Hkv, kh = (wi.bh / G) % p.Hkv;
                    for (int i = 0; i < 2; ++i) {
                        if (n > 0 && !(ok = mbar_wait(&bars[Q_EMPTY + i], (n - 1) & 1, p.status, Q_EMPTY, abort_flag))) break;
                        const int r = wi.t * 2 * kBM + i * kBM;   // rows at or beyond N (a head's last, half-empty item) read as zeros
                        mbar_arrive_expect_tx(&bars[Q_FULL + i], kTileBytes);
                        tma_load_rows(sQ + i * kTileBytes, &mapQ, flat_q, 0, r, qh, qb, p.H, N, &bars[Q_FULL + i]);
                        tma_load_rows(sQ + i * kTileBytes + kBoxBytes, &mapQ, flat_q, 64, r, qh, qb, p.H, N, &bars[Q_FULL + i]);
                    }
                    for (int j = 0; ok && j < nk; ++j, ++gk) {
                        const int r = j * kBN;
                        const int ks = gk % kKStages;
                        if (gk >= kKStages && !(ok = mbar_wait(&bars[K_EMPTY + ks], ((gk / kKStages) - 1) & 1, p.status, K_EMPTY, abort_flag))) break;
                        mbar_arrive_expect_tx(&bars[K_FULL + ks], kTileBytes);
                        tma_load_rows(sK + ks * kTileBytes, &mapK, flat_k, 0, r, kh, kb, p.Hkv, N, &bars[K_FULL + ks]);
                        tma_load_rows(sK + ks * kTileBytes + kBoxBytes, &mapK, flat_k, 64, r, kh, kb, p.Hkv, N, &bars[K_FULL + ks]);
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // -------------------------------------------------------------- TMA producer: the V ring
            if (lane == 0) {
                int gv = 0;
                bool ok = true;
                for (int n = 0; ok; ++n) {
                    const int w = fetch_item(bars, item_ring, n, lane, false, p.status, abort_flag);
                    if (w < 0) break;
                    const WorkItem wi = work_item(w, n_qt, BH, p.head_chunk);
                    const int nk = causal ? 2 * wi.t + 2 : nk_all;
                    const int kb = (wi.bh / G) / p.Hkv, kh = (wi.bh / G) % p.Hkv;
                    for (int j = 0; j < nk; ++j, ++gv) {
                        const int r = j * kBN;
                        const int vs = gv % kVStages;
                        if (gv >= kVStages && !(ok = mbar_wait(&bars[V_EMPTY + vs], ((gv / kVStages) - 1) & 1, p.status, V_EMPTY, abort_flag))) break;
                        mbar_arrive_expect_tx(&bars[V_FULL + vs], kTileBytes);
                        tma_load_rows(sV + vs * kTileBytes, &mapV, flat_v, 0, r, kh, kb, p.Hkv, N, &bars[V_FULL + vs]);
                        tma_load_rows(sV + vs * kTileBytes + kBoxBytes, &mapV, flat_v, 64, r, kh, kb, p.Hkv, N, &bars[V_FULL + vs]);
                    }
                }
            }
            __syncwarp();
        } else if (warp == kMmaWarp) {
            // -------------------------------------------------------------- MMA issuer
            const bool leader = elect_one();
            constexpr int kVFmt = Elem<T>::kDtype == COROPE_DTYPE_F16 ? 0 : 1;
            const uint32_t idesc_qk = make_idesc(0, 0, 0, 0, kBM, kBN);
            const uint32_t idesc_pv = make_idesc(kVFmt, kVFmt, 0, 1, kBM, kD);
            constexpr uint32_t kHi = sdesc_hi(1024);
            const uint32_t q_lo = sdesc_lo(smem_u32(sQ), 0), k_lo = sdesc_lo(smem_u32(sK), 0), v_lo = sdesc_lo(smem_u32(sV), kBoxBytes);
            auto issue_qk = [&](int i, int ks) {
                const uint32_t a0 = q_lo + i * (kTileBytes >> 4), b0 = k_lo + ks * (kTileBytes >> 4), d = tmem + i * 128;
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4;
                    if (leader) umma_ss2(d, a0 + off, kHi, b0 + off, kHi, idesc_qk, kk > 0);
                }
            };
            auto issue_pv = [&](int i, int vs, bool acc) {
                const uint32_t b0 = v_lo + vs * (kTileBytes >> 4), d = tmem + 256 + i * 128, a = tmem + i * 128;
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk)
                    if (leader) umma_ts2(d, a + (kk >> 2) * 64 + (kk & 3) * 8, b0 + kk * (2048 >> 4), kHi, idesc_pv, (acc || kk > 0) ? 1u : 0u);
            };
            // "K ready": straight from the TMA barrier when the pre-pass has rotated K, else from the rotation groups
            const int kReadyBar = p.k_rot != nullptr ? K_FULL : K_ROT;
            constexpr int kVReadyBar = V_FULL;
            int gk = 0, gv = 0, s0 = 0, s1 = 0;   // K tiles, V tiles, S tiles of group 0 / 1 so far
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int w = fetch_item(bars, item_ring, n, lane, true, p.status, abort_flag);
                if (w < 0) break;
                const WorkItem wi = work_item(w, n_qt, BH, p.head_chunk);
                const int nk = causal ? 2 * wi.t + 2 : nk_all, nk0 = causal ? nk - 1 : nk;
                // One loop body for the whole item, the first tile included (j = -1 only issues the two Q K^T of tile 0): the
                // instructions that issue the MMAs then exist once (1 % faster than a peeled first tile at the Llama-7B-4K shape).
                for (int j = -1; j < nk; ++j) {
                    const bool have_next = j + 1 < nk;
                    const int ks1 = gk % kKStages;
                    const int vs = gv % kVStages;
                    if (j >= 0) {
                        if (!(ok = mbar_wait_warp(&bars[kVReadyBar + vs], (gv / kVStages) & 1, p.status, V_FULL, abort_flag))) break;
                        if (j < nk0) {
                            if (!(ok = mbar_wait_warp(&bars[P_FULL + 0], s0 & 1, p.status, P_FULL, abort_flag))) break;
                            if (j == 0 && n > 0 && !(ok = mbar_wait_warp(&bars[O_FREE + 0], (n - 1) & 1, p.status, O_FREE, abort_flag))) break;
                            tc_fence_after();
                            issue_pv(0, vs, j > 0);
                            if (leader) umma_commit(&bars[O_FULL + 0]);
                            ++s0;
                        }
                    } else {
                        if (!(ok = mbar_wait_warp(&bars[Q_ROT + 0], n & 1, p.status, Q_ROT, abort_flag))) break;
                    }
                    if (have_next) {
                        if (!(ok = mbar_wait_warp(&bars[kReadyBar + ks1], (gk / kKStages) & 1, p.status, K_ROT, abort_flag))) break;
                        tc_fence_after();
                        if (j + 1 < nk0) {
                            issue_qk(0, ks1);
                            if (leader) umma_commit(&bars[S_FULL + 0]);
                            if (j + 2 == nk0 && leader) umma_commit(&bars[Q_EMPTY + 0]);   // last use of Q0 in this item
                        }
                    }
                    if (j >= 0) {
                        if (!(ok = mbar_wait_warp(&bars[P_FULL + 1], s1 & 1, p.status, P_FULL + 1, abort_flag))) break;
                        if (j == 0 && n > 0 && !(ok = mbar_wait_warp(&bars[O_FREE + 1], (n - 1) & 1, p.status, O_FREE + 1, abort_flag))) break;
                        tc_fence_after();
                        issue_pv(1, vs, j > 0);
                        if (leader) umma_commit(&bars[O_FULL + 1]);
                        if (leader) umma_commit(&bars[V_EMPTY + vs]);
                        ++s1;
                        ++gv;
                    } else {
                        if (!(ok = mbar_wait_warp(&bars[Q_ROT + 1], n & 1, p.status, Q_ROT + 1, abort_flag))) break;
                        tc_fence_after();
                    }
                    if (have_next) {
                        issue_qk(1, ks1);
                        if (leader) umma_commit(&bars[S_FULL + 1]);
                        if (leader) umma_commit(&bars[K_EMPTY + ks1]);
                        if (j + 2 == nk && leader) umma_commit(&bars[Q_EMPTY + 1]);       // last use of Q1 in this item
                        ++gk;
                    }
                }
            }
            __syncwarp();
        }
    } else if (warp < kSmxWarp0) {
        // ------------------------------------------------------------------ rotation groups
        // Two groups of 128 threads; group r rotates rows [64 r, 64 r + 64) of every tile (Q0, Q1 once per item, every
        // K tile).  With kRegsRot equal to the launch count they keep what they have; a smaller kRegsRot has to be released
        // here, or the softmax groups' setmaxnreg.inc (which has no time limit) waits for registers that never come.
        if constexpr (kRegsRot < kLaunchRegs) reg_dealloc<kRegsRot>();
        const int rg = (warp - kRotWarp0) >> 2;
        const int tid = (threadIdx.x - kRotWarp0 * 32) & 127;
        constexpr int kHalfRows = kBM / 2;
        bool ok = true;
        TabRegs<kHalfRows> tr;
        int gk = 0;
        for (int n = 0; ok; ++n) {
            const int w = fetch_item(bars, item_ring, n, lane, true, p.status, abort_flag);
            if (w < 0) break;
            const WorkItem wi = work_item(w, n_qt, BH, p.head_chunk);
            const int nk = causal ? 2 * wi.t + 2 : nk_all;
            for (int i = 0; i < 2 && ok; ++i) {
                load_table_regs<kHalfRows>(tr, p.packed_tab + (size_t)(wi.t * 2 * kBM + i * kBM + rg * kHalfRows) * (kD / 2), tid);
                if (!(ok = mbar_wait_warp(&bars[Q_FULL + i], n & 1, p.status, Q_FULL, abort_flag))) break;
                rotate_tile_regs<T, kHalfRows, kBoxBytes, 1>(sQ + i * kTileBytes + rg * kHalfRows * 128, tr, tid, p.sm_scale * kLog2e);
                fence_proxy_async();
                mbar_arrive_warp(&bars[Q_ROT + i], lane);
            }
            if (!ok) break;
            // K tiles: only when no pre-pass has rotated them; otherwise the MMA warp takes them straight from the TMA barriers
            if (p.k_rot != nullptr) continue;
            load_table_regs<kHalfRows>(tr, p.packed_tab + (size_t)(rg * kHalfRows) * (kD / 2), tid);
            for (int j = 0; j < nk; ++j, ++gk) {
                const int ks = gk % kKStages;
                if (!(ok = mbar_wait_warp(&bars[K_FULL + ks], (gk / kKStages) & 1, p.status, K_FULL, abort_flag))) break;
                rotate_tile_regs<T, kHalfRows, kBoxBytes, 1>(sK + ks * kTileBytes + rg * kHalfRows * 128, tr, tid, 1.0f);
                fence_proxy_async();
                mbar_arrive_warp(&bars[K_ROT + ks], lane);
                if (j + 1 < nk) load_table_regs<kHalfRows>(tr, p.packed_tab + (size_t)((j + 1) * kBN + rg * kHalfRows) * (kD / 2), tid);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax groups
        reg_alloc<kRegsSmx>();
        // Two warpgroups per Q tile, each taking 64 of the 128 key columns of every S tile: the per-tile chain
        // S ready -> exponentials -> P ready is what bounds the loop (one warp needs 8 cycles of the XU pipe per
        // exp2 instruction), and halving the columns per thread halves it.  The two threads that share a row
        // exchange their half-row maxima through shared memory (named barrier of their two warps) so that both use
        // the same reference max; row sums stay partial until the end of the item.
        const int wsm = warp - kSmxWarp0;
        const int wg = wsm >> 3;            // Q tile
        const int half = (wsm >> 2) & 1;    // which 64 key columns (and, for O, which 64 head-dim columns)
        const int quad = warp & 3;          // the TMEM lane quadrant a warp may touch is warp_id % 4
        const int row = quad * 32 + lane;
        const int pair_bar = 1 + wg * 4 + quad;   // named barrier of the two warps that hold the same 32 rows
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const uint32_t tS = tmem + lane_base + wg * 128 + half * 64;          // this group's 64 S columns; its P goes over their start
        const uint32_t tO = tmem + lane_base + 256 + wg * 128 + half * 64;    // this group's 64 O columns
        float* xmine = xch + (wg * 2 + half) * kBM + row;
        const float* xother = xch + (wg * 2 + (half ^ 1)) * kBM + row;
        int gs = 0;   // S tiles of this Q tile so far (across items): parity of S_FULL / O_FULL and of the exchange slots
        bool ok = true;
        for (int n = 0; ok; ++n) {
            const int w = fetch_item(bars, item_ring, n, lane, true, p.status, abort_flag);
            if (w < 0) break;
            const WorkItem wi = work_item(w, n_qt, BH, p.head_chunk);
            const int nk_i = causal ? 2 * wi.t + 1 + wg : nk_all;
            float m = -INFINITY, l = 0.f;
            for (int j = 0; j < nk_i; ++j, ++gs) {
                if (!(ok = mbar_wait_warp(&bars[S_FULL + wg], gs & 1, p.status, S_FULL + wg, abort_flag))) break;
                tc_fence_after();
                const bool diag = causal && (j == nk_i - 1);
                uint32_t s0[32], s1[32];
                COROPE_TMEM_LD32(tS, s0);
                COROPE_TMEM_LD32(tS + 32, s1);
                tmem_wait_ld();
                if (diag) {   // causal mask on the diagonal tile: key column > query row
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (half * 64 + i > row) s0[i] = 0xff800000u;
                        if (half * 64 + 32 + i > row) s1[i] = 0xff800000u;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    mx0 = fmax3(mx0, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
                    mx1 = fmax3(mx1, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
                }
                const float mx_half = fmaxf(mx0, mx1);
                *xmine = mx_half;
                named_bar_sync(pair_bar, 64);
                const float m_new = fmaxf(m, fmaxf(mx_half, *xother));
                named_bar_sync(pair_bar, 64);   // both have read before either writes its slot again
                const bool need = m_new > m + 8.f;   // lazy rescale: tolerate P up to 2^8 before moving the reference max
                const float m_old = m;
                m = need ? m_new : m;
                // two elements per instruction for the subtraction of the reference max and for the row sum
                const uint64_t neg_m = f2_pack(-m, -m);
                uint64_t la = 0, lb = 0;   // two packed accumulators (bit pattern 0 = +0.0f twice)
#define COROPE_EXP_CHUNK(sx, cidx)                                                           \
                {                                                                            \
                    uint32_t pk[16];                                                         \
                    _Pragma("unroll") for (int i = 0; i < 16; ++i) {                         \
                        float d0, d1;                                                        \
                        f2_unpack(f2_add(f2_pack_bits(sx[2 * i], sx[2 * i + 1]), neg_m), d0, d1); \
                        const float p0 = fast_exp2(d0), p1 = fast_exp2(d1);                  \
                        uint64_t pr;                                                         \
                        if (kPBf16) {   /* row sums from the rounded P, for both formats */   \
                            pk[i] = pack_bf162(p0, p1);                                      \
                            pr = f2_pack_bits(pk[i] << 16, pk[i] & 0xffff0000u);             \
                        } else {                                                             \
                            pk[i] = pack_half2(p0, p1);                                      \
                            const float2 rr = unpack_half2(pk[i]);                           \
                            pr = f2_pack(rr.x, rr.y);                                        \
                        }                                                                    \
                        if (i & 1) lb = f2_add(lb, pr); else la = f2_add(la, pr);            \
                    }                                                                        \
                    COROPE_TMEM_ST16(tS + (cidx) * 16, pk);                                  \
                }
                COROPE_EXP_CHUNK(s0, 0)
                COROPE_EXP_CHUNK(s1, 1)
#undef COROPE_EXP_CHUNK
                float l0, l1;
                f2_unpack(f2_add(la, lb), l0, l1);
                // The rescale of O (this group's 64 columns) comes after P is written so that S is no longer live.
                if (j > 0 && __any_sync(0xffffffffu, need)) {
                    if (!(ok = mbar_wait_warp(&bars[O_FULL + wg], (gs - 1) & 1, p.status, O_FULL + wg, abort_flag))) break;
                    tc_fence_after();
                    const float alpha = fast_exp2(m_old - m);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t r[32];
                        COROPE_TMEM_LD32(tO + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        COROPE_TMEM_ST32(tO + c * 32, r);
                    }
                    l *= alpha;
                }
                l += l0 + l1;
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive_warp(&bars[P_FULL + wg], lane);
            }
            if (!ok) break;
            // output of this item: total row sum from the two halves, wait for the last P V, normalise, store this
            // group's 64 head-dim columns; then hand O back to the MMA issuer
            *xmine = l;
            named_bar_sync(pair_bar, 64);
            const float l_tot = l + *xother;
            named_bar_sync(pair_bar, 64);   // both have read before either writes this slot again
            if (!(ok = mbar_wait_warp(&bars[O_FULL + wg], (gs - 1) & 1, p.status, O_FULL + wg, abort_flag))) break;
            tc_fence_after();
            const float inv = 1.f / l_tot;
            const bool in_head = (2 * wi.t + wg) * kBM < N;   // false for the Q1 tile of a head's last, half-empty item
            const size_t grow = (size_t)wi.bh * N + (size_t)(2 * wi.t + wg) * kBM + row;   // row of the (contiguous) LSE
            T* orow = reinterpret_cast<T*>(p.out_o) + half * 64 +
                      (kPlain ? (int64_t)grow * p.so.n : row_offset(p.so, p.H, wi.bh, (2 * wi.t + wg) * kBM + row));
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                COROPE_TMEM_LD32(tO + c * 32, r);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
                if (in_head) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                }
            }
            tc_fence_before();
            mbar_arrive_warp(&bars[O_FREE + wg], lane);
            if (half == 0 && in_head) p.lse2[grow] = m + log2f(l_tot);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <typename T>
int launch_t(const RopeParams& p, int dtype, cudaStream_t s) {
    CUtensorMap mq, mk, mv;
    // maps over the caller's q / k / v with their own strides (2-D when the rows collapse, else 4-D: head dim, row, head, batch);
    // the pre-rotated K copy is contiguous
    RopeParams pp = p;
    bool fq, fk, fv;
    if (int e = encode_rows_map(&mq, &fq, p.q, p.B, p.H, p.N, kD, p.sq, kBM, 64, dtype)) return e;
    if (int e = p.k_rot ? encode_rows_map(&mk, &fk, p.k_rot, p.B, p.Hkv, p.N, kD, contiguous_strides(p.Hkv, p.N, kD), kBN, 64, COROPE_DTYPE_F16)
                        : encode_rows_map(&mk, &fk, p.k, p.B, p.Hkv, p.N, kD, p.sk, kBN, 64, dtype))
        return e;
    if (int e = encode_rows_map(&mv, &fv, p.v, p.B, p.Hkv, p.N, kD, p.sv, kBN, 64, dtype)) return e;
    pp.flat_q = fq; pp.flat_k = fk; pp.flat_v = fv;
    pp.head_chunk = head_chunk_for(p.N);
    const bool plain = p.H == p.Hkv && fq && fk && fv && rows_collapse(p.so, p.H, p.N);
    auto kern = plain ? rope_fwd_sm100_kernel<T, true> : rope_fwd_sm100_kernel<T, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    const unsigned items = (unsigned)(((p.N + 2 * kBM - 1) / (2 * kBM)) * p.B * p.H);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const unsigned grid = items < (unsigned)sms ? items : (unsigned)sms;   // persistent: one CTA per SM
    kern<<<grid, kThreads, kSmemBytes, s>>>(mq, mk, mv, pp); count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

bool rope_fwd_tc_supported(int B, int H, int N, int D, int dtype, int causal) {
    (void)B; (void)H;
    (void)causal;
    return D == kD && (dtype == COROPE_DTYPE_BF16 || dtype == COROPE_DTYPE_F16) && N % kBM == 0;
}

int launch_rope_fwd_tc(const RopeParams& p, int dtype, cudaStream_t s) {
    if (dtype == COROPE_DTYPE_BF16) return launch_t<__nv_bfloat16>(p, dtype, s);
    return launch_t<__half>(p, dtype, s);
}

}  // namespace corope
