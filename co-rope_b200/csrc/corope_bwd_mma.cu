// Co-RoPE GQA attention backward for 16-bit inputs at D = 128, tensor-core version: as in the forward, the only work
// left on the CUDA cores is what depends on query, key and frequency together (the rotation by Delta_ij w_p and its
// inverse); every contraction is an mma.sync m16n8k16 (fp16 operands, fp32 accumulators).
//
// Math (corope-exp/corope_attn_gqa_pytorch.py:182-298), one KV head, its G query heads h, leader = first head, s = sm_scale:
//     z_ik = sigmoid(s qL_i.k_k)   Delta_ij = a_ii - sum_{k<=j} z_ik   K'_ij = R(Delta_ij w) k_j   S_hij = s q_hi.K'_ij
//     P = exp(S - lse)   g_hij = s P_hij (dO_hi.V_j - delta_hi)
//     dV_j   += sum_{i,h} P_hij dO_hi
//     dq_hi  += sum_j g_hij K'_ij                                   (per pair p: components 1 and 2)
//     u_ij    = sum_h g_hij q_hi        dk_j += R(-Delta_ij w) u_ij
//     gD_ij   = - sum_h g_hij sum_p w_p (q2 K'1 - q1 K'2)           (mileage gradient)
//     gz_ik   = sum_{j<k} gD_ij   graw_ik = gz_ik z_ik (1 - z_ik) s    dqL_i += sum_k graw_ik k_k    dk_k += sum_i graw_ik qL_i
// One CTA = 8 consecutive query rows of one (batch, KV head), one warp per row, key tiles of 64 swept upward (gz is a
// prefix sum in j).  Per block of 8 keys a warp runs, with lane = (key or head: lane / 4, c = lane % 4):
//   K' for the lane's 16 pairs (B operand)            -> S (A = q pairs) and the mileage term (A = w (q2, -q1))
//   dO.V (A = dO of the row, B = V via ldmatrix)      -> P, g, gD (summed over heads with shuffles, kept per key)
//   u = g^T q (A = g transposed with movmatrix)       -> inverse rotation on the CUDA cores, added to a shared dK tile
//   dq += g K'^T (B = movmatrix of the K' registers): accumulators in registers for the whole row
// Once per tile: each warp turns its row of gD into gz (prefix over the keys) and graw; then, summed over the CTA's rows
// by the tensor cores, dV (K dimension = (row, head)), the leader terms dk += graw^T qL and dqL += graw k (K dimension
// = row / key); dV and the shared dK tile go to the fp32 global accumulators with vector reductions.
#include "corope_mma.cuh"

namespace corope {
namespace {

using namespace gqa_mma;

constexpr int kKTileBytes = kKT * kKRow * 4;
constexpr int kVTileBytes = kKT * kVRowBytes;
constexpr int kTabBytes = kThreads * 16 * 4;    // one per-lane operand table: 16 registers' worth for each of the 256 threads
constexpr int kPsRowBytes = 144;                // P rows (64 keys fp16) + 16 bytes of padding
constexpr int kDkStride = 132;                  // words per row of the shared dK tile (128 + 4: conflict-free reductions)
// The shared dK tile is summed in 32-bit fixed point (2^-14 units): integer shared-memory atomics are single
// instructions, fp32 ones are compare-and-swap loops, and the sum no longer depends on the order of the warps.  The
// rounding error of one contribution, 3e-5, is far below the 16-bit output resolution.
// Fast form: x * 2^14 + 1.5 * 2^23 holds round(x * 2^14) in its low mantissa bits -- valid for |x| < 256 only.  Per block
// of 8 keys a warp therefore bounds its contributions (|x| <= sqrt(2) G max|g| max|q_row|, one vote instruction) and takes
// the range-safe form when the bound is not below 256: a real float -> int conversion of x clamped to +-4096 (the tile sum
// of 9 such terms still fits 32 bits).  A contribution that had to be clamped is reported in the status word
// (COROPE_DEV_RANGE): the result is then inaccurate, never wrapped around.
constexpr float kDkScale = 16384.f, kDkMagic = 12582912.f, kDkFastLimit = 250.f, kDkClamp = 4096.f;
__device__ __forceinline__ void dk_add(int* slot, float x) {
    atomicAdd(slot, __float_as_int(fmaf(x, kDkScale, kDkMagic)) - 0x4B400000);
}
__device__ __forceinline__ void dk_add_safe(int* slot, float x, bool& clamped) {
    const float xc = fminf(fmaxf(x, -kDkClamp), kDkClamp);
    clamped |= xc != x;
    atomicAdd(slot, __float2int_rn(xc * kDkScale));
}
constexpr int kGrRowBytes = 144;                // rows of the leader-term operand graw (64 keys fp16 + padding)
constexpr size_t kSmemBytes = 2 * (kKTileBytes + kVTileBytes) + kRows * kPairs * 4 + 2 * kRows * kKT * 4 + 4 * kWStride * 4 + 4 * kTabBytes +
                              64 * kPsRowBytes + 64 * kVRowBytes + kKT * kDkStride * 4 + kRows * kKT * 4 + 16 * kGrRowBytes + 16 * kVRowBytes;
static_assert(kSmemBytes <= 232448 - 1024, "shared memory budget");

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void red_add_v2(float* gptr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(gptr), "f"(a), "f"(b) : "memory");
}

template <typename T, int G, bool DIRECT>
__global__ void __launch_bounds__(kThreads, 1) corope_bwd_mma_kernel(GqaParams p) {
    constexpr int kKG = 8 * G;                        // (row, head) pairs of the CTA: K dimension of the dV product
    constexpr int kKSteps = (kKG + 15) / 16;
    extern __shared__ __align__(16) uint8_t smem_dyn[];
    uint8_t* ks_base = smem_dyn;
    uint8_t* vs_base = ks_base + 2 * kKTileBytes;
    uint32_t* qls = reinterpret_cast<uint32_t*>(vs_base + 2 * kVTileBytes);   // leader rows, permuted like K
    float* zs = reinterpret_cast<float*>(qls + kRows * kPairs);
    float* dl = zs + kRows * kKT;
    float* ws = dl + kRows * kKT;
    uint4* tab = reinterpret_cast<uint4*>(ws + 4 * kWStride);                  // 4 tables x [warp][chunk s][lane]
    uint8_t* ps = reinterpret_cast<uint8_t*>(tab) + 4 * kTabBytes;             // P of the tile: [(row, head)][key] fp16
    uint8_t* dos = ps + 64 * kPsRowBytes;                                      // dO of the CTA's rows: [(row, head)][d] fp16
    int* dk_t = reinterpret_cast<int*>(dos + 64 * kVRowBytes);                 // [key][d] fixed point, reduced into by all warps
    float* gds = reinterpret_cast<float*>(dk_t + kKT * kDkStride);             // gD of the tile: [row][key]
    uint8_t* grs = reinterpret_cast<uint8_t*>(gds + kRows * kKT);              // graw of the tile: [16 rows (8 used)][key] fp16
    uint8_t* qlr = grs + 16 * kGrRowBytes;                                     // leader rows, natural order: [16 rows (8 used)][d] fp16

    const int N = p.N;
    const int bg = blockIdx.y;
    const int b = bg / p.Hkv, g = bg % p.Hkv;
    const int i0 = (gridDim.x - 1 - blockIdx.x) * kRows;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = lane >> 2, c = lane & 3;
    const int i = i0 + warp;
    const size_t q_head0 = (size_t)b * p.Hq + (size_t)g * G;
    const uint32_t* Kp = p.k_pairs + (size_t)bg * N * kPairs;
    const __half* Vh = p.v_half + (size_t)bg * N * kD;
    const T* Q = reinterpret_cast<const T*>(p.q);
    const T* DO = reinterpret_cast<const T*>(p.d_o);
    float* dk_acc = p.dk_acc + (size_t)bg * N * kD;
    float* dv_acc = p.dv_acc + (size_t)bg * N * kD;
    uint4* aqs = tab + warp * 128;             // (q1, q2) pairs of head h for the lane's 16 pairs: A operand of S
    uint4* aws = aqs + kThreads * 4;           // w (q2, -q1): A operand of the mileage term
    uint4* ados = aws + kThreads * 4;          // dO of head h, all d: A operand of dO.V
    uint4* bqs = ados + kThreads * 4;          // q of heads 2c, 2c+1 at the pair component lane/4 selects: B operand of u = g^T q

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
    load_tile(0, 0);

    // ---- per-CTA and per-lane constants
    for (int idx = tid; idx < kRows * kPairs; idx += kThreads) {
        const int r = idx >> 6, pp = idx & 63;
        const T* row = Q + row_offset(p.sq, p.Hq, (int)q_head0, i0 + r);
        qls[r * kPairs + perm_slot(pp)] = to_half2<T>(row[pp], row[pp + kPairs]);
    }
    for (int d = tid; d < kPairs; d += kThreads) {
        const int cc = (d & 7) & 3, s = d >> 4, e = ((d >> 3) & 1) * 2 + ((d & 7) >> 2);
        ws[cc * kWStride + s * 4 + e] = 1.0f / powf(p.theta, (float)(2 * d) / (float)kD);
    }
    for (int idx = tid; idx < 64 * (kPsRowBytes / 4); idx += kThreads) reinterpret_cast<uint32_t*>(ps)[idx] = 0u;
    for (int idx = tid; idx < 64 * 64; idx += kThreads) {   // dO rows of the CTA as fp16, rows beyond 8 G stay zero
        const int r = idx >> 6, d2 = idx & 63;
        uint32_t val = 0u;
        if (r < kKG) {
            const T* row = DO + row_offset(p.sdo, p.Hq, (int)q_head0 + r % G, i0 + r / G);
            val = to_half2<T>(row[2 * d2], row[2 * d2 + 1]);
        }
        *reinterpret_cast<uint32_t*>(dos + r * kVRowBytes + d2 * 4) = val;
    }
    for (int idx = tid; idx < kKT * kDkStride; idx += kThreads) dk_t[idx] = 0;
    for (int idx = tid; idx < 16 * (kGrRowBytes / 4); idx += kThreads) reinterpret_cast<uint32_t*>(grs)[idx] = 0u;
    for (int idx = tid; idx < 16 * 64; idx += kThreads) {
        const int r = idx >> 6, d2 = idx & 63;
        uint32_t val = 0u;
        if (r < kRows) {
            const T* row = Q + row_offset(p.sq, p.Hq, (int)q_head0, i0 + r);
            val = to_half2<T>(row[2 * d2], row[2 * d2 + 1]);
        }
        *reinterpret_cast<uint32_t*>(qlr + r * kVRowBytes + d2 * 4) = val;
    }
    __syncthreads();
    {
        const bool valid = h < G;
        const T* qrow = Q + row_offset(p.sq, p.Hq, (int)q_head0 + (valid ? h : 0), i);
        const T* dorow = DO + row_offset(p.sdo, p.Hq, (int)q_head0 + (valid ? h : 0), i);
        const int ha = 2 * c, hb = 2 * c + 1;   // the two heads of the lane's B-operand entries
        const T* qa = Q + row_offset(p.sq, p.Hq, (int)q_head0 + (ha < G ? ha : 0), i);
        const T* qb = Q + row_offset(p.sq, p.Hq, (int)q_head0 + (hb < G ? hb : 0), i);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            uint32_t a[4], aw[4], ad[4], bq[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int pp = lane_pair(c, s, e);
                const float w = ws[c * kWStride + s * 4 + e];
                const float q1 = Elem<T>::to_f32(qrow[pp]), q2 = Elem<T>::to_f32(qrow[pp + kPairs]);
                a[e] = valid ? pack_half2(q1, q2) : 0u;
                aw[e] = valid ? pack_half2(w * q2, -w * q1) : 0u;
                // dO operand: k-step t = 2 s + e / 2, register e % 2 (0: d = 16 t + 2c, +1;  1: d = 16 t + 8 + 2c, +1)
                const int d0 = 16 * (2 * s + (e >> 1)) + 8 * (e & 1) + 2 * c;
                ad[e] = valid ? to_half2<T>(dorow[d0], dorow[d0 + 1]) : 0u;
                // B operand of u-MMA x = 4 s + e = 2 t + u: column n = lane / 4 is pair 8 t + n / 2 + 4 u, component n % 2
                const int t = 2 * s + (e >> 1), u = e & 1;
                const int col = 8 * t + (h >> 1) + 4 * u + kPairs * (h & 1);
                bq[e] = pack_half2(ha < G ? Elem<T>::to_f32(qa[col]) : 0.f, hb < G ? Elem<T>::to_f32(qb[col]) : 0.f);
            }
            aqs[s * 32 + lane] = make_uint4(a[0], a[1], a[2], a[3]);
            aws[s * 32 + lane] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
            ados[s * 32 + lane] = make_uint4(ad[0], ad[1], ad[2], ad[3]);
            bqs[s * 32 + lane] = make_uint4(bq[0], bq[1], bq[2], bq[3]);
        }
        __syncwarp();
    }
    uint32_t aq[16], aw[16];   // A operands of S and of the mileage term stay in registers for the whole row
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint4 a = aqs[s * 32 + lane], w4 = aws[s * 32 + lane];
        aq[4 * s] = a.x; aq[4 * s + 1] = a.y; aq[4 * s + 2] = a.z; aq[4 * s + 3] = a.w;
        aw[4 * s] = w4.x; aw[4 * s + 1] = w4.y; aw[4 * s + 2] = w4.z; aw[4 * s + 3] = w4.w;
    }
    const bool valid = h < G;
    // largest |g| for which every dK contribution of a block stays inside the fast fixed-point form (see dk_add)
    float g_fast_limit;
    {
        float qmax = 0.f;
#pragma unroll
        for (int x = 0; x < 16; ++x) {
            const float2 f = unpack_half2(aq[x]);
            qmax = fmaxf(qmax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) qmax = fmaxf(qmax, __shfl_xor_sync(0xffffffffu, qmax, off));
        g_fast_limit = kDkFastLimit / (1.4143f * (float)G * fmaxf(qmax, 1e-20f));
    }
    bool range_clamped = false;
    const float lse = valid ? p.lse2[(q_head0 + h) * N + i] : 0.f;
    const float dlt = valid ? p.delta[(q_head0 + h) * N + i] : 0.f;
    const float a_ii = p.a_diag[(size_t)bg * N + i];
    const float sc2 = p.sm_scale * kLog2e;
    float dq[16][2];
#pragma unroll
    for (int x = 0; x < 16; ++x) dq[x][0] = dq[x][1] = 0.f;
    float carry_a = 0.f, carry_g = 0.f;
    float dql[2][4];   // leader-term dq of the CTA's 8 rows, operand-order columns 16 warp .. 16 warp + 15 (summed into dq at the end)
#pragma unroll
    for (int n = 0; n < 2; ++n) dql[n][0] = dql[n][1] = dql[n][2] = dql[n][3] = 0.f;

    const int j_last = ((i0 + kRows - 1) / kKT) * kKT;
    int buf = 0;
    for (int j0 = 0; j0 <= j_last; j0 += kKT, buf ^= 1) {
        cp_async_wait_all();
        __syncthreads();   // tile landed; the previous tile's dV / dK flush is complete
        if (j0 + kKT <= j_last) load_tile(j0 + kKT, buf ^ 1);
        const uint32_t* ks = reinterpret_cast<const uint32_t*>(ks_base + buf * kKTileBytes);
        const uint8_t* vs = vs_base + buf * kVTileBytes;

        // 1. leader gates (rows of A = the CTA's 8 query rows; warp w takes keys 8w .. 8w+7)
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
            const int key = j0 + warp * 8 + 2 * c;
            const int qi = i0 + h;
            zs[h * kKT + warp * 8 + 2 * c] = key <= qi ? 1.f / (1.f + __expf(-z0 * p.sm_scale)) : 0.f;
            zs[h * kKT + warp * 8 + 2 * c + 1] = key + 1 <= qi ? 1.f / (1.f + __expf(-z1 * p.sm_scale)) : 0.f;
        }
        __syncthreads();
        // 2. Delta_ij = a_ii - sum_{k <= j} z_ik
        {
            const float za = zs[warp * kKT + 2 * lane], zb = zs[warp * kKT + 2 * lane + 1];
            float pre = za + zb;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, pre, off);
                if (lane >= off) pre += t;
            }
            dl[warp * kKT + 2 * lane] = a_ii - (carry_a + pre - zb);
            dl[warp * kKT + 2 * lane + 1] = a_ii - (carry_a + pre);
            carry_a += __shfl_sync(0xffffffffu, pre, 31);
        }
        __syncwarp();

        // 3. blocks of 8 keys
#pragma unroll 1
        for (int nb = 0; nb < 8; ++nb) {
            uint32_t* ps_out = reinterpret_cast<uint32_t*>(ps + (warp * G + h) * kPsRowBytes + (nb * 8 + 2 * c) * 2);
            float* gd_out = gds + warp * kKT + nb * 8 + 2 * c;
            if (j0 + nb * 8 > i) {   // every key of the block is above the diagonal (warp-uniform)
                if (valid) *ps_out = 0u;
                if (h == 0) gd_out[0] = gd_out[1] = 0.f;
                continue;
            }
            const float delta = dl[warp * kKT + nb * 8 + h];
            const uint4* kp = reinterpret_cast<const uint4*>(ks + (nb * 8 + h) * kKRow) + c;
            uint32_t kpr[16], csr[16];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 kv = kp[4 * s];
                const float4 wv = *reinterpret_cast<const float4*>(ws + c * kWStride + s * 4);
                const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
                const float wq[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float sn, cs;
                    sincos_fast<DIRECT>(delta * wq[e], &sn, &cs);
                    const __half2 kk = *reinterpret_cast<const __half2*>(&kw[e]);
                    const uint32_t sw = __byte_perm(kw[e], 0, 0x1032);
                    const __half2 ksw = *reinterpret_cast<const __half2*>(&sw);
                    const __half2 r = __hfma2(kk, __floats2half2_rn(cs, cs), __hmul2(ksw, __floats2half2_rn(sn, -sn)));
                    kpr[s * 4 + e] = *reinterpret_cast<const uint32_t*>(&r);
                    csr[s * 4 + e] = pack_half2(cs, sn);
                }
            }
            // S, the mileage term and dO.V
            float s0 = 0.f, s1 = 0.f, t0 = 0.f, t1 = 0.f, m0 = 0.f, m1 = 0.f, n0 = 0.f, n1 = 0.f, dp0 = 0.f, dp1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 ad = ados[s * 32 + lane];
                mma16816(s0, s1, aq[4 * s], aq[4 * s + 1], kpr[4 * s], kpr[4 * s + 1], s0, s1);
                mma16816(t0, t1, aq[4 * s + 2], aq[4 * s + 3], kpr[4 * s + 2], kpr[4 * s + 3], t0, t1);
                mma16816(m0, m1, aw[4 * s], aw[4 * s + 1], kpr[4 * s], kpr[4 * s + 1], m0, m1);
                mma16816(n0, n1, aw[4 * s + 2], aw[4 * s + 3], kpr[4 * s + 2], kpr[4 * s + 3], n0, n1);
                uint32_t r0, r1, r2, r3;   // V[key][d]: k-steps 2s and 2s+1 (16 d each)
                ldmatrix_x4(r0, r1, r2, r3, vs + (nb * 8 + (lane & 7)) * kVRowBytes + s * 64 + (lane >> 3) * 16);
                mma16816(dp0, dp1, ad.x, ad.y, r0, r1, dp0, dp1);
                mma16816(e0, e1, ad.z, ad.w, r2, r3, e0, e1);
            }
            // P, g, gD (rows = heads, columns = keys 2c, 2c+1 of the block)
            const int key = j0 + nb * 8 + 2 * c;
            const bool vis0 = valid && key <= i, vis1 = valid && key + 1 <= i;
            const float p0 = vis0 ? fast_exp2((s0 + t0) * sc2 - lse) : 0.f;
            const float p1 = vis1 ? fast_exp2((s1 + t1) * sc2 - lse) : 0.f;
            const float g0 = p0 * (dp0 + e0 - dlt) * p.sm_scale, g1 = p1 * (dp1 + e1 - dlt) * p.sm_scale;
            if (valid) *ps_out = pack_half2(p0, p1);
            const uint32_t gp = pack_half2_sat(g0, g1);
            const float g_abs = fmaxf(fabsf(g0), fabsf(g1));
            const bool big = __any_sync(0xffffffffu, g_abs > g_fast_limit);   // warp-uniform: some contribution may leave the fast range
            float gd0 = -g0 * (m0 + n0), gd1 = -g1 * (m1 + n1);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {   // sum over the heads
                gd0 += __shfl_xor_sync(0xffffffffu, gd0, off);
                gd1 += __shfl_xor_sync(0xffffffffu, gd1, off);
            }
            if (h == 0) {   // the mileage-gradient chain (prefix over the keys, leader terms) runs once per tile, below
                gd_out[0] = gd0;
                gd_out[1] = gd1;
            }

            // u = g^T q per pair, inverse rotation, into the shared dK tile
            const uint32_t gT = movmatrix_trans(gp);
            int* dkrow = dk_t + (nb * 8 + h) * kDkStride;
            if (!big) {
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint4 bv = bqs[s * 32 + lane];
                    const uint32_t bq[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float u1 = 0.f, u2 = 0.f;
                        mma16816(u1, u2, gT, 0u, bq[e], 0u, 0.f, 0.f);
                        const float2 cs = unpack_half2(csr[s * 4 + e]);
                        const int pp = lane_pair(c, s, e);
                        dk_add(dkrow + pp, fmaf(u1, cs.x, -u2 * cs.y));
                        dk_add(dkrow + pp + kPairs, fmaf(u2, cs.x, u1 * cs.y));
                    }
                }
            } else {
                range_clamped |= g_abs > 65504.f;   // g itself no longer fits the fp16 operand (it was saturated above)
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint4 bv = bqs[s * 32 + lane];
                    const uint32_t bq[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float u1 = 0.f, u2 = 0.f;
                        mma16816(u1, u2, gT, 0u, bq[e], 0u, 0.f, 0.f);
                        const float2 cs = unpack_half2(csr[s * 4 + e]);
                        const int pp = lane_pair(c, s, e);
                        dk_add_safe(dkrow + pp, fmaf(u1, cs.x, -u2 * cs.y), range_clamped);
                        dk_add_safe(dkrow + pp + kPairs, fmaf(u2, cs.x, u1 * cs.y), range_clamped);
                    }
                }
            }
            // dq += g K'^T
#pragma unroll
            for (int x = 0; x < 16; ++x) mma16816(dq[x][0], dq[x][1], gp, 0u, movmatrix_trans(kpr[x]), 0u, dq[x][0], dq[x][1]);
        }
        // mileage-gradient chain of this row: gz_k = sum of gD over the keys before k, graw = gz z (1 - z) s
        {
            __syncwarp();
            const float ga = gds[warp * kKT + 2 * lane], gb = gds[warp * kKT + 2 * lane + 1];
            float pre = ga + gb;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, pre, off);
                if (lane >= off) pre += t;
            }
            const float gz0 = carry_g + pre - (ga + gb), gz1 = gz0 + ga;
            carry_g += __shfl_sync(0xffffffffu, pre, 31);
            const float z0 = zs[warp * kKT + 2 * lane], z1 = zs[warp * kKT + 2 * lane + 1];
            const int key = j0 + 2 * lane;
            const float gr0 = key <= i ? gz0 * z0 * (1.f - z0) * p.sm_scale : 0.f;
            const float gr1 = key + 1 <= i ? gz1 * z1 * (1.f - z1) * p.sm_scale : 0.f;
            range_clamped |= fmaxf(fabsf(gr0), fabsf(gr1)) > 65504.f;
            *reinterpret_cast<uint32_t*>(grs + warp * kGrRowBytes + lane * 4) = pack_half2_sat(gr0, gr1);
        }
        __syncthreads();

        // 4. dV of the tile: [key][d] = sum over (row, head) of P^T dO; warp w takes keys 16 (w / 2) .. +15 and d 64 (w % 2) .. +63
        {
            const int mb = warp >> 1, nh = warp & 1;
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < kKSteps; ++kk) {
                uint32_t a[4];
                ldmatrix_x4_trans(a[0], a[1], a[2], a[3],
                                  ps + (kk * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * kPsRowBytes + (mb * 16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4_trans(r0, r1, r2, r3,
                                      dos + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kVRowBytes + (nh * 64 + np * 16 + (lane >> 4) * 8) * 2);
                    mma16816_full(acc[2 * np], a, r0, r1);
                    mma16816_full(acc[2 * np + 1], a, r2, r3);
                }
            }
            const int i_last = i0 + kRows - 1;
            const int ka = j0 + mb * 16 + h, kb = ka + 8;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const int d = nh * 64 + n * 8 + 2 * c;
                if (ka <= i_last) red_add_v2(dv_acc + (size_t)ka * kD + d, acc[n][0], acc[n][1]);
                if (kb <= i_last) red_add_v2(dv_acc + (size_t)kb * kD + d, acc[n][2], acc[n][3]);
            }
            // leader terms of the tile, summed over the CTA's rows by MMAs (K dimension = row):
            //   dk[key][d] += sum_i graw_ik qL_i[d]   -- the same (keys, d) block of the output as above
            {
                float acc2[8][4];
#pragma unroll
                for (int n = 0; n < 8; ++n) acc2[n][0] = acc2[n][1] = acc2[n][2] = acc2[n][3] = 0.f;
                uint32_t a[4];
                ldmatrix_x4_trans(a[0], a[1], a[2], a[3], grs + ((lane & 7) + ((lane >> 4) & 1) * 8) * kGrRowBytes + (mb * 16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4_trans(r0, r1, r2, r3, qlr + ((lane & 7) + ((lane >> 3) & 1) * 8) * kVRowBytes + (nh * 64 + np * 16 + (lane >> 4) * 8) * 2);
                    mma16816_full(acc2[2 * np], a, r0, r1);
                    mma16816_full(acc2[2 * np + 1], a, r2, r3);
                }
                int* ra = dk_t + (mb * 16 + h) * kDkStride + nh * 64 + 2 * c;   // into the shared dK tile (flushed below)
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    dk_add_safe(ra + n * 8, acc2[n][0], range_clamped);   // once per tile: the range-safe form costs nothing here
                    dk_add_safe(ra + n * 8 + 1, acc2[n][1], range_clamped);
                    dk_add_safe(ra + 8 * kDkStride + n * 8, acc2[n][2], range_clamped);
                    dk_add_safe(ra + 8 * kDkStride + n * 8 + 1, acc2[n][3], range_clamped);
                }
            }
            //   dqL_i += sum_k graw_ik k_k   -- warp w takes the operand-order columns 16 w .. 16 w + 15 of k
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t a[4], r0, r1, r2, r3;
                ldmatrix_x4(a[0], a[1], a[2], a[3], grs + ((lane & 7) + ((lane >> 3) & 1) * 8) * kGrRowBytes + (kk * 16 + (lane >> 4) * 8) * 2);
                ldmatrix_x4_trans(r0, r1, r2, r3, reinterpret_cast<const uint8_t*>(ks) + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * (kKRow * 4) +
                                                      (warp * 16 + (lane >> 4) * 8) * 2);
                mma16816_full(dql[0], a, r0, r1);
                mma16816_full(dql[1], a, r2, r3);
            }
            // the shared dK tile goes to the global accumulator and is cleared for the next tile
            __syncthreads();
            for (int idx = tid; idx < kKT * 64; idx += kThreads) {
                const int r = idx >> 6, d2 = (idx & 63) * 2;
                int* src = dk_t + r * kDkStride + d2;
                if (j0 + r <= i_last) red_add_v2(dk_acc + (size_t)(j0 + r) * kD + d2, (float)src[0] * (1.f / kDkScale), (float)src[1] * (1.f / kDkScale));
                src[0] = 0;
                src[1] = 0;
            }
        }
    }

    // leader-term dq: from the per-warp column blocks to the lanes that hold the leader head (h == 0) of each row
    __syncthreads();
    {
        float* xs = reinterpret_cast<float*>(dk_t);   // [row][operand-order column], the dK tile is no longer needed
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            xs[h * kD + warp * 16 + n * 8 + 2 * c] = dql[n][0];
            xs[h * kD + warp * 16 + n * 8 + 2 * c + 1] = dql[n][1];
        }
        __syncthreads();
        if (h == 0) {
#pragma unroll
            for (int s = 0; s < 4; ++s)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int slot = perm_slot(lane_pair(c, s, e));
                    dq[s * 4 + e][0] += xs[warp * kD + 2 * slot];
                    dq[s * 4 + e][1] += xs[warp * kD + 2 * slot + 1];
                }
        }
    }
    if (__any_sync(0xffffffffu, range_clamped) && lane == 0 && p.status) atomicCAS(p.status, 0, COROPE_DEV_RANGE);
    if (valid) {
        T* DQ = reinterpret_cast<T*>(p.dq) + row_offset(p.sdq, p.Hq, (int)q_head0 + h, i);
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int pp = lane_pair(c, s, e);
                DQ[pp] = Elem<T>::from_f32(dq[s * 4 + e][0]);
                DQ[pp + kPairs] = Elem<T>::from_f32(dq[s * 4 + e][1]);
            }
    }
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
    if (p.N <= 8192) {
        auto kern = corope_bwd_mma_kernel<T, G, true>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)) != cudaSuccess) return (int)e;
        kern<<<grid, kThreads, kSmemBytes, s>>>(p);
    } else {
        auto kern = corope_bwd_mma_kernel<T, G, false>;
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

// The main backward kernel only (delta, the zeroing of the fp32 dK / dV accumulators and their conversion are the caller's).
int launch_gqa_bwd_mma(const GqaParams& p, int dtype, cudaStream_t s) {
    if (dtype == COROPE_DTYPE_BF16) return dispatch<__nv_bfloat16>(p, s);
    return dispatch<__half>(p, s);
}

}  // namespace corope
