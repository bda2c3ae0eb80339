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
//   3. for every block of 16 keys the scores come out transposed, S^T = K' Q^T: the keys are the 16 rows of the A operand
//      (all in use) and the G heads the columns; lane (r = lane/4, c = lane%4) rotates the 16 (k1, k2) pairs p = c mod 4 of
//      keys r and r + 8 by Delta_ij w_p, and the rotated pairs are the A-operand registers as they stand;
//   4. online softmax per head (log2 domain); O^T += V^T P^T with V through ldmatrix.trans (A) and P transposed in
//      registers (movmatrix) as B; O^T [d][head] stays in registers.
// (With the heads as the rows of A, as a first version had them, half of every operand quad was zero padding that had to be
// rebuilt in registers per MMA: 19.9 instead of 14.7 instructions per (query, key, pair) and twice the MMAs.)
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
    const T* QL = reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.Hq, (int)q_head0, 0);   // leader head of the group

    for (int idx = tid; idx < kRows * kPairs; idx += kThreads) {
        const int r = idx >> 6, pp = idx & 63;
        const T* row = QL + (int64_t)(i0 + r) * p.sq.n;
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
        const T* qrow = reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.Hq, (int)q_head0 + (h < G ? h : 0), i);
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

    // From here on the MMAs are "transposed": keys are the M rows (16 per MMA, all used), the group's heads the 8 N columns.
    // A lane (r = lane / 4, c = lane % 4) owns keys r and r + 8 of a 16-key block on the A side and heads 2c, 2c + 1 on the
    // result side; the query operand above (head r, pairs of class c) is the B operand as it stands.
    const int r = h;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // heads 2c, 2c + 1 (l: partial sums over this lane's keys)
    float o[8][4];   // O^T: [db] rows d = 16 db + r (+ 8 for entries 2, 3), columns heads 2c, 2c + 1
#pragma unroll
    for (int db = 0; db < 8; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
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

        // 3. S^T of the row: 16 keys x 8 heads per block; the lane rotates the 16 pairs of its two keys, which are the A
        //    operand registers as they stand (a0 / a2: key r, a1 / a3: key r + 8)
        float sc[4][4];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            sc[kb][0] = sc[kb][1] = sc[kb][2] = sc[kb][3] = -INFINITY;
            if (j0 + kb * 16 > i) continue;   // every key of the block is above the diagonal (warp-uniform)
            const float dA = dl[warp * kKT + kb * 16 + r], dB = dl[warp * kKT + kb * 16 + r + 8];
            const uint4* kpA = reinterpret_cast<const uint4*>(ks + (kb * 16 + r) * kKRow) + c;
            const uint4* kpB = reinterpret_cast<const uint4*>(ks + (kb * 16 + r + 8) * kKRow) + c;
            float accE[4] = {0.f, 0.f, 0.f, 0.f}, accO[4] = {0.f, 0.f, 0.f, 0.f};   // two accumulator chains
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 kva = kpA[4 * s], kvb = kpB[4 * s];
                const float4 wv = *reinterpret_cast<const float4*>(ws + c * kWStride + s * 4);
                const float wq[4] = {wv.x, wv.y, wv.z, wv.w};
                const uint32_t kwa[4] = {kva.x, kva.y, kva.z, kva.w}, kwb[4] = {kvb.x, kvb.y, kvb.z, kvb.w};
                uint32_t ra[4], rb[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    ra[e] = rotate_pair<DIRECT>(kwa[e], dA * wq[e]);
                    rb[e] = rotate_pair<DIRECT>(kwb[e], dB * wq[e]);
                }
                const uint32_t a_even[4] = {ra[0], rb[0], ra[1], rb[1]}, a_odd[4] = {ra[2], rb[2], ra[3], rb[3]};
                const uint4 av = aqs[s * 32 + lane];   // the query operand (re-read per block: registers are short)
                mma16816_full(accE, a_even, av.x, av.y);
                mma16816_full(accO, a_odd, av.z, av.w);
            }
            const int keyA = j0 + kb * 16 + r;
            if (keyA <= i) sc[kb][0] = (accE[0] + accO[0]) * sc2, sc[kb][1] = (accE[1] + accO[1]) * sc2;
            if (keyA + 8 <= i) sc[kb][2] = (accE[2] + accO[2]) * sc2, sc[kb][3] = (accE[3] + accO[3]) * sc2;
        }

        // 4. online softmax of heads 2c, 2c + 1 (their 64 scores sit in the 8 lanes of class c), then O^T += V^T P^T
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            mx0 = fmax3(mx0, sc[kb][0], sc[kb][2]);
            mx1 = fmax3(mx1, sc[kb][1], sc[kb][3]);
        }
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float alpha0 = fast_exp2(m0 - mx0), alpha1 = fast_exp2(m1 - mx1);   // the first tile holds the diagonal: mx is finite
        m0 = mx0, m1 = mx1;
#pragma unroll
        for (int db = 0; db < 8; ++db) {
            o[db][0] *= alpha0, o[db][1] *= alpha1;
            o[db][2] *= alpha0, o[db][3] *= alpha1;
        }
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            if (j0 + kb * 16 > i) continue;   // nothing visible in this block (warp-uniform)
            const uint32_t pa = pack_half2(fast_exp2(sc[kb][0] - mx0), fast_exp2(sc[kb][1] - mx1));   // key r
            const uint32_t pb = pack_half2(fast_exp2(sc[kb][2] - mx0), fast_exp2(sc[kb][3] - mx1));   // key r + 8
            const float2 fa = unpack_half2(pa), fb = unpack_half2(pb);   // row sums from the rounded P
            ps0 += fa.x + fb.x;
            ps1 += fa.y + fb.y;
            // P^T as B operand: (keys 2c, 2c + 1 | head r) is the transpose of what the lane holds (key r | heads 2c, 2c + 1)
            const uint32_t b0 = movmatrix_trans(pa), b1 = movmatrix_trans(pb);
            // V^T as A operand: four transposed 8x8 blocks (d 0-7 | 8-15) x (keys 0-7 | 8-15) of the block's V rows
            const uint8_t* vrow = vs + (kb * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * kVRowBytes + ((lane >> 3) & 1) * 16;
#pragma unroll
            for (int db = 0; db < 8; ++db) {
                uint32_t a[4];
                ldmatrix_x4_trans(a[0], a[1], a[2], a[3], vrow + db * 32);
                mma16816_full(o[db], a, b0, b1);
            }
        }
        l0 = l0 * alpha0 + ps0;
        l1 = l1 * alpha1 + ps1;
    }

#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int head = 2 * c + x;
        if (head >= G) continue;
        const float inv = 1.f / (x ? l1 : l0);
        T* O = reinterpret_cast<T*>(p.out_o) + row_offset(p.so, p.Hq, (int)q_head0 + head, i);
#pragma unroll
        for (int db = 0; db < 8; ++db) {
            O[db * 16 + r] = Elem<T>::from_f32(o[db][x] * inv);
            O[db * 16 + r + 8] = Elem<T>::from_f32(o[db][2 + x] * inv);
        }
        if (r == 0) p.lse2[(q_head0 + head) * N + i] = (x ? m1 : m0) + log2f(x ? l1 : l0);
    }
    if (lane == 0) p.a_diag[(size_t)bg * N + i] = carry;
}

template <typename T, int G>
int launch_g(const GqaParams& p, cudaStream_t s) {
    dim3 grid(p.N / kRows, p.B * p.Hkv);
    const size_t rows = (size_t)p.B * p.Hkv * p.N;
    gqa_pack_kv_kernel<T><<<(unsigned)((rows * 16 + 255) / 256), 256, 0, s>>>((const T*)p.k, (const T*)p.v, p.k_pairs, p.v_half, rows,
                                                                                  row_addr(p.sk, p.Hkv, p.N), row_addr(p.sv, p.Hkv, p.N));
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
