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
// prefix sum in j).  The per-row products are transposed: the 16 keys of a block are the rows of the A operand (all in use),
// the group's heads the 8 columns; lane (r = lane / 4, c = lane % 4) owns keys r, r + 8 on the operand side and heads 2c,
// 2c + 1 on the result side.  Per block of 16 keys a warp runs
//   K' for the 16 pairs of its two keys (A operand)     -> S^T (B = q pairs of head r) and the mileage term (B = w (q2, -q1))
//   (dO.V)^T (A = V via ldmatrix, B = dO of head r)     -> P, g, gD (summed over heads with shuffles, kept per key)
//   u = g^T q, one m16n8k8 per pair slot (K = 8 heads; g's result registers are its A operand as they stand)
//                                                       -> inverse rotation on the CUDA cores, added to a shared dK tile
//   dq^T += K'^T g^T (A = movmatrix of the K' registers, B = movmatrix of g): accumulators in registers for the whole row
// (A first version had the heads as the rows of A: half of every operand quad was zero padding rebuilt in registers per MMA
// and the MMA count was 2.3 times higher: 52 instead of 37 instructions per (query, key, pair).)
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
// Fast form: a float in [512, 1024) has a last-place unit of 2^-14, so 768 + x, for |x| < 256, holds round(x 2^14) in its
// low mantissa bits: its bit pattern is kDkBias + round(x 2^14).  The 768 is the addend of the inverse rotation's last
// multiply-add, the raw bit pattern goes to the atomic, and the bias is taken off when the tile is flushed: every (row, 16-key
// block) that is not skipped adds exactly once to each of the block's slots, so a slot holds count x kDkBias too much.
// Per block a warp bounds its contributions (|x| <= sqrt(2) G max|g| max|q_row|, one vote instruction) and takes the
// range-safe form when the bound is not below 256: a real float -> int conversion of x clamped to +-4096 (the tile sum
// of 9 such terms still fits 32 bits), plus the bias.  A contribution that had to be clamped is reported in the status word
// (COROPE_DEV_RANGE): the result is then inaccurate, never wrapped around.
constexpr float kDkScale = 16384.f, kDkMagic = 768.f, kDkFastLimit = 250.f, kDkClamp = 4096.f;
constexpr int kDkBias = 0x44400000;   // bit pattern of 768.f
// x_plus_magic = kDkMagic + x, computed by the caller's last multiply-add
__device__ __forceinline__ void dk_add_biased(int* slot, float x_plus_magic) { atomicAdd(slot, __float_as_int(x_plus_magic)); }
__device__ __forceinline__ void dk_add_safe(int* slot, float x, bool& clamped, int bias = 0) {
    const float xc = fminf(fmaxf(x, -kDkClamp), kDkClamp);
    clamped |= xc != x;
    atomicAdd(slot, __float2int_rn(xc * kDkScale) + bias);
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
__device__ __forceinline__ void red_add_v4(float* gptr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gptr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
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
    // From here on the per-row MMAs are "transposed": the 16 keys of a block are the rows of the A operand (all in use), the
    // group's heads the 8 columns.  Lane (r = lane / 4, c = lane % 4): keys r and r + 8 on the operand side, heads 2c and
    // 2c + 1 on the result side.  The per-head operands above (head = lane / 4) are the B operands as they stand.
    const int r = h;
    float lse[2], dlt[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const bool ok = 2 * c + x < G;
        lse[x] = ok ? p.lse2[(q_head0 + 2 * c + x) * N + i] : 0.f;
        dlt[x] = ok ? p.delta[(q_head0 + 2 * c + x) * N + i] : 0.f;
    }
    const float a_ii = p.a_diag[(size_t)bg * N + i];
    const float sc2 = p.sm_scale * kLog2e;
    // dq^T: [xb] rows = (pair class r / 2, component r % 2) of slots 2 xb (entries 0, 1) and 2 xb + 1 (entries 2, 3),
    // columns = heads 2c, 2c + 1
    float dq[8][4];
#pragma unroll
    for (int x = 0; x < 8; ++x) dq[x][0] = dq[x][1] = dq[x][2] = dq[x][3] = 0.f;
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

        // 3. blocks of 16 keys
#pragma unroll 1
        for (int kb = 0; kb < 4; ++kb) {
            // P^T of the row for the dV product: [(row, head)][key]; the lane writes head r, keys 2c, 2c + 1 (and + 8)
            uint32_t* ps_out = reinterpret_cast<uint32_t*>(ps + (warp * G + r) * kPsRowBytes + (kb * 16 + 2 * c) * 2);
            float* gd_out = gds + warp * kKT + kb * 16 + r;
            if (j0 + kb * 16 > i) {   // every key of the block is above the diagonal (warp-uniform)
                if (r < G) ps_out[0] = 0u, ps_out[4] = 0u;
                if (c == 0) gd_out[0] = gd_out[8] = 0.f;
                continue;
            }
            const float dA = dl[warp * kKT + kb * 16 + r], dB = dl[warp * kKT + kb * 16 + r + 8];
            const uint4* kpA = reinterpret_cast<const uint4*>(ks + (kb * 16 + r) * kKRow) + c;
            const uint4* kpB = reinterpret_cast<const uint4*>(ks + (kb * 16 + r + 8) * kKRow) + c;
            uint32_t kprA[16], kprB[16], csrA[16], csrB[16];   // rotated pairs (A-operand registers) and packed (cos, sin)
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 kva = kpA[4 * s], kvb = kpB[4 * s];
                const float4 wv = *reinterpret_cast<const float4*>(ws + c * kWStride + s * 4);
                const uint32_t kwa[4] = {kva.x, kva.y, kva.z, kva.w}, kwb[4] = {kvb.x, kvb.y, kvb.z, kvb.w};
                const float wq[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    kprA[s * 4 + e] = rotate_pair<DIRECT>(kwa[e], dA * wq[e], &csrA[s * 4 + e]);
                    kprB[s * 4 + e] = rotate_pair<DIRECT>(kwb[e], dB * wq[e], &csrB[s * 4 + e]);
                }
            }
            // S^T, the mileage term and (dO.V)^T: rows = keys r (entries 0, 1) and r + 8 (entries 2, 3), columns = heads 2c, 2c + 1
            float sE[4] = {0.f, 0.f, 0.f, 0.f}, sO[4] = {0.f, 0.f, 0.f, 0.f}, mE[4] = {0.f, 0.f, 0.f, 0.f}, mO[4] = {0.f, 0.f, 0.f, 0.f};
            float pE[4] = {0.f, 0.f, 0.f, 0.f}, pO[4] = {0.f, 0.f, 0.f, 0.f};
            const uint8_t* vrow = vs + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kVRowBytes + ((lane >> 4) & 1) * 16;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t a_even[4] = {kprA[4 * s], kprB[4 * s], kprA[4 * s + 1], kprB[4 * s + 1]};
                const uint32_t a_odd[4] = {kprA[4 * s + 2], kprB[4 * s + 2], kprA[4 * s + 3], kprB[4 * s + 3]};
                mma16816_full(sE, a_even, aq[4 * s], aq[4 * s + 1]);
                mma16816_full(sO, a_odd, aq[4 * s + 2], aq[4 * s + 3]);
                mma16816_full(mE, a_even, aw[4 * s], aw[4 * s + 1]);
                mma16816_full(mO, a_odd, aw[4 * s + 2], aw[4 * s + 3]);
                const uint4 ad = ados[s * 32 + lane];
                uint32_t v[4];   // V[key][d] of the block, d = 32 s .. 32 s + 15, then + 16
                ldmatrix_x4(v[0], v[1], v[2], v[3], vrow + s * 64);
                mma16816_full(pE, v, ad.x, ad.y);
                ldmatrix_x4(v[0], v[1], v[2], v[3], vrow + s * 64 + 32);
                mma16816_full(pO, v, ad.z, ad.w);
            }
            // P, g, gD
            const int keyA = j0 + kb * 16 + r;
            float pv[4], gv[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const bool vis = 2 * c + (x & 1) < G && keyA + (x >> 1) * 8 <= i;
                pv[x] = vis ? fast_exp2((sE[x] + sO[x]) * sc2 - lse[x & 1]) : 0.f;
                gv[x] = pv[x] * (pE[x] + pO[x] - dlt[x & 1]) * p.sm_scale;
            }
            // transposed copies: (head r | keys 2c, 2c + 1) of the first and second 8 keys
            const uint32_t paT = movmatrix_trans(pack_half2(pv[0], pv[1])), pbT = movmatrix_trans(pack_half2(pv[2], pv[3]));
            if (r < G) ps_out[0] = paT, ps_out[4] = pbT;
            const uint32_t ga = pack_half2_sat(gv[0], gv[1]), gb = pack_half2_sat(gv[2], gv[3]);
            const float g_abs = fmaxf(fmaxf(fabsf(gv[0]), fabsf(gv[1])), fmaxf(fabsf(gv[2]), fabsf(gv[3])));
            const bool big = __any_sync(0xffffffffu, g_abs > g_fast_limit);   // warp-uniform: some contribution may leave the fast range
            float gdA = -(gv[0] * (mE[0] + mO[0]) + gv[1] * (mE[1] + mO[1]));
            float gdB = -(gv[2] * (mE[2] + mO[2]) + gv[3] * (mE[3] + mO[3]));
#pragma unroll
            for (int off = 1; off < 4; off <<= 1) {   // sum over the heads
                gdA += __shfl_xor_sync(0xffffffffu, gdA, off);
                gdB += __shfl_xor_sync(0xffffffffu, gdB, off);
            }
            if (c == 0) {   // the mileage-gradient chain (prefix over the keys, leader terms) runs once per tile, below
                gd_out[0] = gdA;
                gd_out[8] = gdB;
            }

            // u = g^T q per pair (one m16n8k8 per pair slot: K dimension = the 8 heads), inverse rotation, into the shared dK tile
            int* dkA = dk_t + (kb * 16 + r) * kDkStride;
            int* dkB = dkA + 8 * kDkStride;
            if (!big) {
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint4 bv = bqs[s * 32 + lane];
                    const uint32_t bq[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float u[4];
                        mma1688(u, ga, gb, bq[e]);
                        const float2 ca = unpack_half2(csrA[s * 4 + e]), cb = unpack_half2(csrB[s * 4 + e]);
                        const int pp = lane_pair(c, s, e);
                        dk_add_biased(dkA + pp, fmaf(u[0], ca.x, fmaf(-u[1], ca.y, kDkMagic)));
                        dk_add_biased(dkA + pp + kPairs, fmaf(u[1], ca.x, fmaf(u[0], ca.y, kDkMagic)));
                        dk_add_biased(dkB + pp, fmaf(u[2], cb.x, fmaf(-u[3], cb.y, kDkMagic)));
                        dk_add_biased(dkB + pp + kPairs, fmaf(u[3], cb.x, fmaf(u[2], cb.y, kDkMagic)));
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
                        float u[4];
                        mma1688(u, ga, gb, bq[e]);
                        const float2 ca = unpack_half2(csrA[s * 4 + e]), cb = unpack_half2(csrB[s * 4 + e]);
                        const int pp = lane_pair(c, s, e);
                        dk_add_safe(dkA + pp, fmaf(u[0], ca.x, -u[1] * ca.y), range_clamped, kDkBias);
                        dk_add_safe(dkA + pp + kPairs, fmaf(u[1], ca.x, u[0] * ca.y), range_clamped, kDkBias);
                        dk_add_safe(dkB + pp, fmaf(u[2], cb.x, -u[3] * cb.y), range_clamped, kDkBias);
                        dk_add_safe(dkB + pp + kPairs, fmaf(u[3], cb.x, u[2] * cb.y), range_clamped, kDkBias);
                    }
                }
            }
            // dq^T += K'^T g^T: A = the rotated pairs transposed in registers (rows = (pair class, component) of two slots,
            // K dimension = the 16 keys), B = g transposed (keys | head r)
            const uint32_t gaT = movmatrix_trans(ga), gbT = movmatrix_trans(gb);
#pragma unroll
            for (int xb = 0; xb < 8; ++xb) {
                const uint32_t a[4] = {movmatrix_trans(kprA[2 * xb]), movmatrix_trans(kprA[2 * xb + 1]), movmatrix_trans(kprB[2 * xb]),
                                       movmatrix_trans(kprB[2 * xb + 1])};
                mma16816_full(dq[xb], a, gaT, gbT);
            }
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
            // 16-byte reductions: the lanes c and c ^ 1 hold neighbouring column pairs of both rows; the even one takes row ka of
            // both, the odd one row kb
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const bool odd = c & 1;
                const float s0 = odd ? acc[n][0] : acc[n][2], s1 = odd ? acc[n][1] : acc[n][3];   // what the partner needs
                const float r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
                const int d = nh * 64 + n * 8 + 2 * (c & 2);
                if (!odd) {
                    if (ka <= i_last) red_add_v4(dv_acc + (size_t)ka * kD + d, acc[n][0], acc[n][1], r0, r1);
                } else {
                    if (kb <= i_last) red_add_v4(dv_acc + (size_t)kb * kD + d, r0, r1, acc[n][2], acc[n][3]);
                }
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
            for (int idx = tid; idx < kKT * 32; idx += kThreads) {
                const int r = idx >> 5, d4 = (idx & 31) * 4;
                int* src = dk_t + r * kDkStride + d4;
                // rows of the CTA that did not skip this key's 16-key block: each left one bias in every slot of the block
                const int cnt = min(kRows, max(0, i_last + 1 - (j0 + (r & ~15))));
                const unsigned bias = (unsigned)cnt * (unsigned)kDkBias;   // modulo 2^32, like the sums themselves
                const int4 v = *reinterpret_cast<const int4*>(src);
                if (j0 + r <= i_last)
                    red_add_v4(dk_acc + (size_t)(j0 + r) * kD + d4, (float)(int)((unsigned)v.x - bias) * (1.f / kDkScale),
                               (float)(int)((unsigned)v.y - bias) * (1.f / kDkScale), (float)(int)((unsigned)v.z - bias) * (1.f / kDkScale),
                               (float)(int)((unsigned)v.w - bias) * (1.f / kDkScale));
                *reinterpret_cast<int4*>(src) = make_int4(0, 0, 0, 0);
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
        if (c == 0) {   // the lanes that hold head 0 (entries 0 and 2 of every dq^T block)
#pragma unroll
            for (int xb = 0; xb < 8; ++xb)
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    const int x = 2 * xb + y;
                    const int slot = perm_slot(lane_pair(r >> 1, x >> 2, x & 3));
                    dq[xb][2 * y] += xs[warp * kD + 2 * slot + (r & 1)];
                }
        }
    }
    if (__any_sync(0xffffffffu, range_clamped) && lane == 0 && p.status) atomicCAS(p.status, 0, COROPE_DEV_RANGE);
#pragma unroll
    for (int x2 = 0; x2 < 2; ++x2) {
        if (2 * c + x2 >= G) continue;
        T* DQ = reinterpret_cast<T*>(p.dq) + row_offset(p.sdq, p.Hq, (int)q_head0 + 2 * c + x2, i) + (r & 1) * kPairs;
#pragma unroll
        for (int xb = 0; xb < 8; ++xb)
#pragma unroll
            for (int y = 0; y < 2; ++y) {
                const int x = 2 * xb + y;
                DQ[lane_pair(r >> 1, x >> 2, x & 3)] = Elem<T>::from_f32(dq[xb][2 * y + x2]);
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
