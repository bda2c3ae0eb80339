// Co-RoPE GQA attention forward for 16-bit inputs at D = 128: the per-(i, j, d) rotation of the key stays on the
// CUDA cores (it cannot be factored: the phase Delta_ij * w_d depends on query, key and frequency), every dot
// product over d moves to the tensor cores (mma.sync m16n8k16, fp16 operands, fp32 accumulators).
//
// Definition (corope-exp/corope_attn_gqa_pytorch.py:56-124), one KV head and its G query heads, leader = first head:
//     z_ik = sigmoid(s * qL_i . k_k)    Delta_ij = sum_{k=j+1..i} z_ik
//     S_hij = s * sum_p ( q1_hip K'1_ijp + q2_hip K'2_ijp ),  K'1 = k1 cos + k2 sin,  K'2 = k2 cos - k1 sin,  angle = Delta_ij w_p
// One CTA = 8 consecutive query rows of one (batch, KV head), one warp per row; keys in tiles of 64, swept downward
// from the diagonal so that Delta is a running suffix sum (as in the general kernel).  Per tile:
//   1. leader scores of the CTA's 8 rows against the 64 keys: warp w takes keys 8w..8w+7 (8 MMAs, rows of the A
//      operand = the 8 query rows), sigmoid, causal mask -> z in shared memory;
//   2. each warp turns its row of z into Delta (suffix sums inside the tile + carry from the tiles above);
//   3. for every block of 8 keys: lane (key = lane/4, c = lane%4) rotates the 16 (k1, k2) pairs p = c mod 4 of its key
//      by Delta_ij w_p -- these are exactly the B-operand registers of 8 MMAs whose A operand holds the G heads of
//      the row (rows >= G are zero) -> S[h][key];
//   4. online softmax per head (log2 domain), P as fp16 A operand, V through ldmatrix.trans, O in registers.
// The K dimension of the score MMAs is ordered (pair, component): index 2p is the first half of pair p, 2p+1 the
// second; Q and K use the same order, so dot products are unchanged.  Shared-memory rows of K / leader Q are stored
// permuted so that a lane's 16 pairs are four 16-byte loads without bank conflicts (see perm_slot).
#include "corope_mma.cuh"

namespace corope {
namespace {

using namespace gqa_mma;

constexpr int kKTileBytes = kKT * kKRow * 4;
constexpr int kVTileBytes = kKT * kVRowBytes;
constexpr int kAqBytes = kThreads * 16 * 4;   // the query operand of every lane (16 registers' worth), re-read per key block
constexpr size_t kSmemBytes = 2 * (kKTileBytes + kVTileBytes) + kRows * kPairs * 4 + 2 * kRows * kKT * 4 + 4 * kWStride * 4 + kAqBytes;

template <typename T, int G, bool DIRECT>
__global__ void __launch_bounds__(kThreads, 2) corope_fwd_mma_kernel(GqaParams p) {
    extern __shared__ __align__(16) uint8_t smem_dyn[];
    uint8_t* ks_base = smem_dyn;                                        // 2 x K tile, (k1, k2) fp16 pairs, permuted rows
    uint8_t* vs_base = ks_base + 2 * kKTileBytes;                       // 2 x V tile, fp16 row-major
    uint32_t* qls = reinterpret_cast<uint32_t*>(vs_base + 2 * kVTileBytes);   // leader rows of the CTA's queries, permuted like K
    float* zs = reinterpret_cast<float*>(qls + kRows * kPairs);
    float* dl = zs + kRows * kKT;
    float* ws = dl + kRows * kKT;   // inverse frequencies, permuted like K: the 16 of lane c are contiguous (stride kWStride)
    // query operands (A fragments of head lane/4 for the 16 pairs of lane%4): chunk s of lane l at [warp][s][l], so that a
    // warp's 16-byte loads are contiguous

    const int N = p.N;
    const int bg = blockIdx.y;
    const int b = bg / p.Hkv, g = bg % p.Hkv;
    const int i0 = (gridDim.x - 1 - blockIdx.x) * kRows;   // heavy (late) rows first
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = lane >> 2, c = lane & 3;
    const int i = i0 + warp;
    uint4* aqs = reinterpret_cast<uint4*>(ws + 4 * kWStride) + warp * 128;
    const size_t q_head0 = (size_t)b * p.Hq + (size_t)g * G;
    const uint32_t* Kp = p.k_pairs + (size_t)bg * N * kPairs;
    const __half* Vh = p.v_half + (size_t)bg * N * kD;
    // asynchronous copy of one tile into buffer `buf`: 64 keys x (16 chunks of K pairs + 16 chunks of V), 8 chunks per thread
    auto load_tile = [&](int j0, int buf) {
        uint8_t* kd = ks_base + buf * kKTileBytes;
        uint8_t* vd = vs_base + buf * kVTileBytes;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * kThreads, r = idx >> 4, ch = idx & 15;
            cp_async16(kd + r * (kKRow * 4) + ch * 16, Kp + (size_t)(j0 + r) * kPairs + ch * 4);
            cp_async16(vd + r * kVRowBytes + ch * 16, Vh + (size_t)(j0 + r) * kD + ch * 8);
        }
        cp_async_commit();
    };
    const T* QL = reinterpret_cast<const T*>(p.q) + q_head0 * N * kD;

    for (int idx = tid; idx < kRows * kPairs; idx += kThreads) {
        const int r = idx >> 6, pp = idx & 63;
        const T* row = QL + (size_t)(i0 + r) * kD;
        qls[r * kPairs + perm_slot(pp)] = to_half2<T>(row[pp], row[pp + kPairs]);
    }
    for (int d = tid; d < kPairs; d += kThreads) {
        const int cc = (d & 7) & 3, s = d >> 4, e = ((d >> 3) & 1) * 2 + ((d & 7) >> 2);
        ws[cc * kWStride + s * 4 + e] = 1.0f / powf(p.theta, (float)(2 * d) / (float)kD);
    }
    __syncthreads();

    // per-lane constants: the 16 pairs of this lane (p = c mod 4), their frequencies, and the query operand of head h
    {
        uint32_t aq[16];
        const T* qrow = reinterpret_cast<const T*>(p.q) + ((q_head0 + (h < G ? h : 0)) * N + i) * kD;
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int pp = lane_pair(c, s, e);
                aq[s * 4 + e] = (h < G) ? to_half2<T>(qrow[pp], qrow[pp + kPairs]) : 0u;
            }
#pragma unroll
        for (int s = 0; s < 4; ++s) aqs[s * 32 + lane] = make_uint4(aq[s * 4], aq[s * 4 + 1], aq[s * 4 + 2], aq[s * 4 + 3]);
        __syncwarp();
    }

    float m = -INFINITY, l = 0.f;   // of head h (the 4 lanes of a head agree on m; l is a per-lane partial sum)
    float o[16][2];
#pragma unroll
    for (int db = 0; db < 16; ++db) o[db][0] = o[db][1] = 0.f;
    float carry = 0.f;              // sum of z_ik over the keys of the tiles already swept
    const float sc2 = p.sm_scale * kLog2e;

    const int j_first = ((i0 + kRows - 1) / kKT) * kKT;
    load_tile(j_first, 0);
    int buf = 0;
    for (int j0 = j_first; j0 >= 0; j0 -= kKT, buf ^= 1) {
        cp_async_wait_all();
        __syncthreads();   // this tile has landed for every thread, and every warp is done with the previous tile
        if (j0 >= kKT) load_tile(j0 - kKT, buf ^ 1);
        const uint32_t* ks = reinterpret_cast<const uint32_t*>(ks_base + buf * kKTileBytes);
        const uint8_t* vs = vs_base + buf * kVTileBytes;

        // 1. leader gates: rows of A = the CTA's 8 query rows, warp w takes keys 8w .. 8w+7 (B = raw K pairs)
        {
            const uint4* kp = reinterpret_cast<const uint4*>(ks + (warp * 8 + h) * kKRow) + c;
            const uint4* qp = reinterpret_cast<const uint4*>(qls + h * kPairs) + c;
            float z0 = 0.f, z1 = 0.f;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 kv = kp[4 * s], qv = qp[4 * s];
                mma16816(z0, z1, qv.x, qv.y, kv.x, kv.y, z0, z1);
                mma16816(z0, z1, qv.z, qv.w, kv.z, kv.w, z0, z1);
            }
            // result: row h (query i0 + h), keys j0 + 8 warp + 2c, + 1
            const int key = j0 + warp * 8 + 2 * c;
            const int qi = i0 + h;
            zs[h * kKT + warp * 8 + 2 * c] = key <= qi ? 1.f / (1.f + __expf(-z0 * p.sm_scale)) : 0.f;
            zs[h * kKT + warp * 8 + 2 * c + 1] = key + 1 <= qi ? 1.f / (1.f + __expf(-z1 * p.sm_scale)) : 0.f;
        }
        __syncthreads();
        // 2. Delta of this warp's row: Delta_j = carry + sum of z over the keys of the tile above j
        {
            const float za = zs[warp * kKT + 2 * lane], zb = zs[warp * kKT + 2 * lane + 1];
            float suf = za + zb;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float t = __shfl_down_sync(0xffffffffu, suf, off);
                if (lane + off < 32) suf += t;
            }
            const float above = carry + suf - (za + zb);   // keys beyond this lane's pair
            dl[warp * kKT + 2 * lane + 1] = above;
            dl[warp * kKT + 2 * lane] = above + zb;
            carry += __shfl_sync(0xffffffffu, suf, 0);
        }
        __syncwarp();

        // 3. scores of the G heads for this row, 8 keys at a time
        float sc[8][2];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            sc[nb][0] = sc[nb][1] = -INFINITY;
            if (j0 + nb * 8 > i) continue;   // every key of the block is above the diagonal (warp-uniform)
            const float delta = dl[warp * kKT + nb * 8 + h];
            const uint4* kp = reinterpret_cast<const uint4*>(ks + (nb * 8 + h) * kKRow) + c;
            float s0 = 0.f, s1 = 0.f, t0 = 0.f, t1 = 0.f;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 kv = kp[4 * s];
                const float4 wv = *reinterpret_cast<const float4*>(ws + c * kWStride + s * 4);
                const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
                const float wq[4] = {wv.x, wv.y, wv.z, wv.w};
                uint32_t bf[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float sn, cs;
                    sincos_fast<DIRECT>(delta * wq[e], &sn, &cs);
                    // (K'1, K'2) = (k1, k2) (c, c) + (k2, k1) (s, -s) in packed fp16 arithmetic
                    const __half2 kk = *reinterpret_cast<const __half2*>(&kw[e]);
                    const uint32_t sw = __byte_perm(kw[e], 0, 0x1032);
                    const __half2 ksw = *reinterpret_cast<const __half2*>(&sw);
                    const __half2 r = __hfma2(kk, __floats2half2_rn(cs, cs), __hmul2(ksw, __floats2half2_rn(sn, -sn)));
                    bf[e] = *reinterpret_cast<const uint32_t*>(&r);
                }
                const uint4 av = aqs[s * 32 + lane];
                mma16816(s0, s1, av.x, av.y, bf[0], bf[1], s0, s1);
                mma16816(t0, t1, av.z, av.w, bf[2], bf[3], t0, t1);   // two accumulator chains
            }
            const int key = j0 + nb * 8 + 2 * c;
            sc[nb][0] = key <= i ? (s0 + t0) * sc2 : -INFINITY;
            sc[nb][1] = key + 1 <= i ? (s1 + t1) * sc2 : -INFINITY;
        }

        // 4. online softmax of head h (lanes 4h .. 4h+3 hold its 64 scores), then O += P V
        float mx = m;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) mx = fmax3(mx, sc[nb][0], sc[nb][1]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float alpha = fast_exp2(m - mx);   // the first tile holds the diagonal, so mx is finite
        m = mx;
        float psum = 0.f;
        uint32_t pa[8];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            const float p0 = fast_exp2(sc[nb][0] - mx), p1 = fast_exp2(sc[nb][1] - mx);
            pa[nb] = pack_half2(p0, p1);
            const float2 pr = unpack_half2(pa[nb]);   // row sums from the rounded P
            psum += pr.x + pr.y;
        }
        l = l * alpha + psum;
#pragma unroll
        for (int db = 0; db < 16; ++db) {
            o[db][0] *= alpha;
            o[db][1] *= alpha;
        }
        const int n_kc = min(4, (i - j0) / 16 + 1);   // 16-key chunks that hold visible keys (warp-uniform)
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
            if (kc >= n_kc) break;
            const uint8_t* vrow = vs + (kc * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kVRowBytes + (lane >> 4) * 16;
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4_trans(r0, r1, r2, r3, vrow + dp * 32);
                mma16816(o[2 * dp][0], o[2 * dp][1], pa[2 * kc], pa[2 * kc + 1], r0, r1, o[2 * dp][0], o[2 * dp][1]);
                mma16816(o[2 * dp + 1][0], o[2 * dp + 1][1], pa[2 * kc], pa[2 * kc + 1], r2, r3, o[2 * dp + 1][0], o[2 * dp + 1][1]);
            }
        }
    }

    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (h < G) {
        const float inv = 1.f / l;
        T* O = reinterpret_cast<T*>(p.out_o) + ((q_head0 + h) * N + i) * kD;
#pragma unroll
        for (int db = 0; db < 16; ++db)
            *reinterpret_cast<uint32_t*>(O + db * 8 + 2 * c) = pack2<T>(o[db][0] * inv, o[db][1] * inv);
        if (c == 0) p.lse2[(q_head0 + h) * N + i] = m + log2f(l);
    }
    if (lane == 0) p.a_diag[(size_t)bg * N + i] = carry;
}

template <typename T, int G>
int launch_g(const GqaParams& p, cudaStream_t s) {
    dim3 grid(p.N / kRows, p.B * p.Hkv);
    const size_t rows = (size_t)p.B * p.Hkv * p.N;
    gqa_pack_kv_kernel<T><<<(unsigned)((rows * 16 + 255) / 256), 256, 0, s>>>((const T*)p.k, (const T*)p.v, p.k_pairs, p.v_half, rows);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    // phases up to a few thousand radians (N <= 8192) go to the hardware sin / cos directly
    if (p.N <= 8192) {
        auto kern = corope_fwd_mma_kernel<T, G, true>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)) != cudaSuccess) return (int)e;
        kern<<<grid, kThreads, kSmemBytes, s>>>(p);
    } else {
        auto kern = corope_fwd_mma_kernel<T, G, false>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)) != cudaSuccess) return (int)e;
        kern<<<grid, kThreads, kSmemBytes, s>>>(p);
    }
    count_launch();
    return (int)cudaGetLastError();
}

template <typename T>
int dispatch(const GqaParams& p, cudaStream_t s) {
    switch (p.G) {
        case 1: return launch_g<T, 1>(p, s);
        case 2: return launch_g<T, 2>(p, s);
        case 3: return launch_g<T, 3>(p, s);
        case 4: return launch_g<T, 4>(p, s);
        case 5: return launch_g<T, 5>(p, s);
        case 6: return launch_g<T, 6>(p, s);
        case 7: return launch_g<T, 7>(p, s);
        case 8: return launch_g<T, 8>(p, s);
        default: return COROPE_ERR_BAD_GROUP;
    }
}

}  // namespace

bool gqa_fwd_mma_supported(int N, int D, int dtype) {
    return D == kD && N % kKT == 0 && (dtype == COROPE_DTYPE_BF16 || dtype == COROPE_DTYPE_F16);
}

int launch_gqa_fwd_mma(const GqaParams& p, int dtype, cudaStream_t s) {
    if (dtype == COROPE_DTYPE_BF16) return dispatch<__nv_bfloat16>(p, s);
    return dispatch<__half>(p, s);
}

}  // namespace corope
