// Fused-RoPE causal flash-attention forward for sm_100a: TMA -> shared memory -> in-place rotation ->
// tcgen05 MMAs with TMEM accumulators -> online softmax in registers.  16-bit inputs, D = 128.
//
// One CTA owns 256 consecutive query rows (two 128-row tiles, "Q0" and "Q1") of one (batch, head)
// and sweeps the K/V tiles 0 .. 2t+1 they can see.  Warp roles (448 threads):
//   warp 0        TMA producer: Q tiles once, then the K ring and the V ring
//   warp 1        MMA issuer (one elected lane) and TMEM owner
//   warps 2-5     rotation group: rotates Q0/Q1 once (scaled by sm_scale*log2e) and every K tile as it
//                 lands, in place in shared memory, as fp16; converts bf16 V tiles to fp16 in place
//   warps 6-9     softmax group of Q0: thread = row; S from TMEM, running max / sum, P (fp16) written
//                 back over S in TMEM, lazy rescale of O in TMEM, final normalise + store
//   warps 10-13   softmax group of Q1
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i aliases the first 64 columns of S_i.
// MMA order per K tile j:  PV0(j) QK0(j+1) | PV1(j) QK1(j+1)  so that one group's softmax overlaps the
// other group's MMAs.  The rotated Q / K never leave shared memory.
//
// Replaces _attn_fwd / _attn_fwd_inner of the reference (fused-rope/fused_rope_attn.py:47-138, 219-320):
// rotation formula :96-99 / :286-287, exp2-domain softmax :103-114, M = m + log2(l) :316.
#include "common.cuh"

namespace corope {
namespace {

constexpr int kD = 128;
constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kKStages = 2;
constexpr int kVStages = 2;
constexpr int kTileBytes = kBM * kD * 2;   // 32 KiB: two 128 x 64 boxes
constexpr int kBoxBytes = kTileBytes / 2;
constexpr int kThreads = 448;
constexpr int kRotWarp0 = 2;
constexpr int kSmxWarp0 = 6;

enum Bar {
    Q_FULL = 0,                        // +i
    Q_ROT = 2,                         // +i
    K_FULL = 4,                        // +stage
    K_ROT = K_FULL + kKStages,
    K_EMPTY = K_ROT + kKStages,
    V_FULL = K_EMPTY + kKStages,
    V_READY = V_FULL + kVStages,
    V_EMPTY = V_READY + kVStages,
    S_FULL = V_EMPTY + kVStages,       // +i
    P_FULL = S_FULL + 2,
    O_FULL = P_FULL + 2,
    NUM_BARS = O_FULL + 2
};

constexpr size_t kSmemTiles = (size_t)(2 + kKStages + kVStages) * kTileBytes;
constexpr size_t kSmemBytes = kSmemTiles + NUM_BARS * 8 + 64 + 1024;  // + alignment slack

// bf16 -> fp16 in place over a whole tile (layout-agnostic).  Values beyond the fp16 range saturate.
__device__ __forceinline__ void convert_tile_bf16_to_f16(uint8_t* tile, int tid) {
#pragma unroll 4
    for (int it = 0; it < kTileBytes / (16 * 128); ++it) {
        uint4* p = reinterpret_cast<uint4*>(tile) + it * 128 + tid;
        uint4 x = *p;
        uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = unpack_bf162(w[i]);
            f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
            f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
            w[i] = pack_half2(f.x, f.y);
        }
        *p = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
rope_fwd_sm100_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, RopeParams p) {
    constexpr bool kConvertV = (Elem<T>::kDtype == COROPE_DTYPE_BF16);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = sm;
    uint8_t* sK = sQ + 2 * kTileBytes;
    uint8_t* sV = sK + kKStages * kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kVStages * kTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = p.N;
    const int BH = p.B * p.H;
    const int n_qt = N / (2 * kBM);
    const int t = n_qt - 1 - (int)(blockIdx.x / BH);   // heaviest (latest) query blocks first
    const int bh = (int)(blockIdx.x % BH);
    const int row_base = bh * N;                        // row in the [B*H*N, D] view
    const int nk = 2 * t + 2;                           // K tiles seen by Q1; Q0 sees nk - 1
    const int nk0 = nk - 1;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars[Q_FULL + i], 1);
            mbar_init(&bars[Q_ROT + i], 128);
            mbar_init(&bars[S_FULL + i], 1);
            mbar_init(&bars[P_FULL + i], 128);
            mbar_init(&bars[O_FULL + i], 1);
        }
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(&bars[K_FULL + s], 1);
            mbar_init(&bars[K_ROT + s], 128);
            mbar_init(&bars[K_EMPTY + s], 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(&bars[V_FULL + s], 1);
            mbar_init(&bars[V_READY + s], 128);
            mbar_init(&bars[V_EMPTY + s], 1);
        }
        fence_mbar_init();
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
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

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int i = 0; i < 2; ++i) {
                const int r = row_base + t * 2 * kBM + i * kBM;
                mbar_arrive_expect_tx(&bars[Q_FULL + i], kTileBytes);
                tma_load_2d(sQ + i * kTileBytes, &mapQ, 0, r, &bars[Q_FULL + i]);
                tma_load_2d(sQ + i * kTileBytes + kBoxBytes, &mapQ, 64, r, &bars[Q_FULL + i]);
            }
            for (int j = 0; j < nk; ++j) {
                const int r = row_base + j * kBN;
                const int ks = j % kKStages, vs = j % kVStages;
                if (j >= kKStages && !mbar_wait(&bars[K_EMPTY + ks], ((j / kKStages) - 1) & 1, p.status, K_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&bars[K_FULL + ks], kTileBytes);
                tma_load_2d(sK + ks * kTileBytes, &mapK, 0, r, &bars[K_FULL + ks]);
                tma_load_2d(sK + ks * kTileBytes + kBoxBytes, &mapK, 64, r, &bars[K_FULL + ks]);
                if (j >= kVStages && !mbar_wait(&bars[V_EMPTY + vs], ((j / kVStages) - 1) & 1, p.status, V_EMPTY, abort_flag)) break;
                mbar_arrive_expect_tx(&bars[V_FULL + vs], kTileBytes);
                tma_load_2d(sV + vs * kTileBytes, &mapV, 0, r, &bars[V_FULL + vs]);
                tma_load_2d(sV + vs * kTileBytes + kBoxBytes, &mapV, 64, r, &bars[V_FULL + vs]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr int kVFmt = (kConvertV || Elem<T>::kDtype == COROPE_DTYPE_F16) ? 0 : 1;
            const uint32_t idesc_qk = make_idesc(0, 0, 0, 0, kBM, kBN);
            const uint32_t idesc_pv = make_idesc(kVFmt, kVFmt, 0, 1, kBM, kD);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            auto issue_qk = [&](int i, int ks) {
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
                    umma_ss(tmem + i * 128, make_sdesc_sw128(q_addr + i * kTileBytes + off, 0, 1024),
                            make_sdesc_sw128(k_addr + ks * kTileBytes + off, 0, 1024), idesc_qk, kk > 0);
                }
            };
            auto issue_pv = [&](int i, int vs, bool acc) {
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk)
                    umma_ts(tmem + 256 + i * 128, tmem + i * 128 + kk * 8, make_sdesc_sw128(v_addr + vs * kTileBytes + kk * 2048, kBoxBytes, 1024),
                            idesc_pv, (acc || kk > 0) ? 1u : 0u);
            };
            bool ok = mbar_wait(&bars[Q_ROT + 0], 0, p.status, Q_ROT, abort_flag) && mbar_wait(&bars[K_ROT + 0], 0, p.status, K_ROT, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
                umma_commit(&bars[S_FULL + 0]);
                ok = mbar_wait(&bars[Q_ROT + 1], 0, p.status, Q_ROT + 1, abort_flag);
            }
            if (ok) {
                tc_fence_after();
                issue_qk(1, 0);
                umma_commit(&bars[S_FULL + 1]);
                umma_commit(&bars[K_EMPTY + 0]);
            }
            for (int j = 0; ok && j < nk; ++j) {
                const int vs = j % kVStages;
                const int ks1 = (j + 1) % kKStages;
                const bool have_next = j + 1 < nk;
                if (!mbar_wait(&bars[V_READY + vs], (j / kVStages) & 1, p.status, V_READY, abort_flag)) break;
                if (j < nk0) {
                    if (!mbar_wait(&bars[P_FULL + 0], j & 1, p.status, P_FULL, abort_flag)) break;
                    tc_fence_after();
                    issue_pv(0, vs, j > 0);
                    umma_commit(&bars[O_FULL + 0]);
                }
                if (have_next) {
                    if (!mbar_wait(&bars[K_ROT + ks1], ((j + 1) / kKStages) & 1, p.status, K_ROT, abort_flag)) break;
                    tc_fence_after();
                    if (j + 1 < nk0) {
                        issue_qk(0, ks1);
                        umma_commit(&bars[S_FULL + 0]);
                    }
                }
                if (!mbar_wait(&bars[P_FULL + 1], j & 1, p.status, P_FULL + 1, abort_flag)) break;
                tc_fence_after();
                issue_pv(1, vs, j > 0);
                umma_commit(&bars[O_FULL + 1]);
                umma_commit(&bars[V_EMPTY + vs]);
                if (have_next) {
                    issue_qk(1, ks1);
                    umma_commit(&bars[S_FULL + 1]);
                    umma_commit(&bars[K_EMPTY + ks1]);
                }
            }
        }
        __syncwarp();
    } else if (warp < kSmxWarp0) {
        // ------------------------------------------------------------------ rotation group
        const int tid = threadIdx.x - kRotWarp0 * 32;
        bool ok = true;
        for (int i = 0; i < 2 && ok; ++i) {
            ok = mbar_wait(&bars[Q_FULL + i], 0, p.status, Q_FULL, abort_flag);
            if (!ok) break;
            rotate_tile_inplace<T, kBM>(sQ + i * kTileBytes, p.packed_tab + (size_t)(t * 2 * kBM + i * kBM) * (kD / 2), tid, p.sm_scale * kLog2e);
            fence_proxy_async();
            mbar_arrive(&bars[Q_ROT + i]);
        }
        for (int j = 0; ok && j < nk; ++j) {
            const int ks = j % kKStages, vs = j % kVStages;
            if (!mbar_wait(&bars[K_FULL + ks], (j / kKStages) & 1, p.status, K_FULL, abort_flag)) break;
            rotate_tile_inplace<T, kBM>(sK + ks * kTileBytes, p.packed_tab + (size_t)(j * kBN) * (kD / 2), tid, 1.0f);
            fence_proxy_async();
            mbar_arrive(&bars[K_ROT + ks]);
            if (!mbar_wait(&bars[V_FULL + vs], (j / kVStages) & 1, p.status, V_FULL, abort_flag)) break;
            if (kConvertV) {
                convert_tile_bf16_to_f16(sV + vs * kTileBytes, tid);
                fence_proxy_async();
            }
            mbar_arrive(&bars[V_READY + vs]);
        }
    } else {
        // ------------------------------------------------------------------ softmax groups
        const int wg = (warp - kSmxWarp0) >> 2;
        const int quad = warp & 3;  // the TMEM lane quadrant a warp may touch is warp_id % 4
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const uint32_t tS = tmem + lane_base + wg * 128;
        const uint32_t tO = tmem + lane_base + 256 + wg * 128;
        const int nk_i = nk0 + wg;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nk_i; ++j) {
            if (!(ok = mbar_wait(&bars[S_FULL + wg], j & 1, p.status, S_FULL + wg, abort_flag))) break;
            tc_fence_after();
            const bool diag = (j == nk_i - 1);
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                COROPE_TMEM_LD32(tS + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(r[i]);
                    if (diag && (c * 32 + i > row)) s = -INFINITY;
                    mx = fmaxf(mx, s);
                }
            }
            const float m_new = fmaxf(m, mx);
            const bool need = m_new > m + 8.f;   // lazy rescale: tolerate P up to 2^8 before moving the reference max
            const float m_use = need ? m_new : m;
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                if (!(ok = mbar_wait(&bars[O_FULL + wg], (j - 1) & 1, p.status, O_FULL + wg, abort_flag))) break;
                tc_fence_after();
                const float alpha = fast_exp2(m - m_use);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    COROPE_TMEM_LD32(tO + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    COROPE_TMEM_ST32(tO + c * 32, r);
                }
                l *= alpha;
            }
            m = m_use;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                COROPE_TMEM_LD32(tS + c * 32, r);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
                    float p0 = fast_exp2(s0 - m), p1 = fast_exp2(s1 - m);
                    if (diag && (c * 32 + 2 * i > row)) p0 = 0.f;
                    if (diag && (c * 32 + 2 * i + 1 > row)) p1 = 0.f;
                    l += p0 + p1;
                    pk[i] = pack_half2(p0, p1);
                }
                COROPE_TMEM_ST16(tS + c * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[P_FULL + wg]);
        }
        if (ok) ok = mbar_wait(&bars[O_FULL + wg], (nk_i - 1) & 1, p.status, O_FULL + wg, abort_flag);
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l;
            const size_t grow = (size_t)row_base + (size_t)(2 * t + wg) * kBM + row;
            T* orow = reinterpret_cast<T*>(p.out_o) + grow * kD;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                COROPE_TMEM_LD32(tO + c * 32, r);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
                uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
            p.lse2[grow] = m + log2f(l);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <typename T>
int launch_t(const RopeParams& p, int dtype, cudaStream_t s) {
    CUtensorMap mq, mk, mv;
    const uint64_t rows = (uint64_t)p.B * p.H * p.N;
    if (int e = encode_tensor_map_2d_sw128(&mq, p.q, rows, kD, kBM, 64, dtype)) return e;
    if (int e = encode_tensor_map_2d_sw128(&mk, p.k, rows, kD, kBN, 64, dtype)) return e;
    if (int e = encode_tensor_map_2d_sw128(&mv, p.v, rows, kD, kBN, 64, dtype)) return e;
    auto kern = rope_fwd_sm100_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    const unsigned grid = (unsigned)((p.N / (2 * kBM)) * p.B * p.H);
    kern<<<grid, kThreads, kSmemBytes, s>>>(mq, mk, mv, p); count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

bool rope_fwd_tc_supported(int B, int H, int N, int D, int dtype, int causal) {
    (void)B; (void)H;
    return causal && D == kD && (dtype == COROPE_DTYPE_BF16 || dtype == COROPE_DTYPE_F16) && N % (2 * kBM) == 0;
}

int launch_rope_fwd_tc(const RopeParams& p, int dtype, cudaStream_t s) {
    if (dtype == COROPE_DTYPE_BF16) return launch_t<__nv_bfloat16>(p, dtype, s);
    return launch_t<__half>(p, dtype, s);
}

}  // namespace corope
