// Co-RoPE GQA attention, general kernels: exact per-(i, j, d) phases, fp32 arithmetic on the CUDA cores.
//
// Definition (corope-exp/corope_attn_gqa_pytorch.py:56-124), for one KV head and its G query heads, leader =
// first head of the group:
//     z_ik = sigmoid(s * qL_i . k_k)      a_ij = sum_{k<=j} z_ik      Delta_ij = a_ii - a_ij
//     S_hij = s * sum_d [ (q1 k1 + q2 k2) cos(Delta w_d) - (q2 k1 - q1 k2) sin(Delta w_d) ],  w_d = theta^(-2d/D)
// which is  S_hij = s * sum_d ( q1_hid K'1_ijd + q2_hid K'2_ijd )  with the head-independent rotated key
//     K'1 = k1 cos + k2 sin,   K'2 = k2 cos - k1 sin.
// cos/sin and K' are computed once per (i, j, d) and shared by the G heads of the group.
//
// Tiling: one CTA = 8 consecutive query rows of one (batch, KV head), one warp per row, all G heads of the
// group; K/V stream through shared memory in tiles of 32 keys; lane = key for the score phase, lane = head-dim
// column for the accumulation phase.  The forward sweeps key tiles downward from the diagonal, so
// Delta_ij = sum_{k=j+1..i} z_ik is a running suffix sum and no mileage pre-pass is needed; a_ii falls out at
// the end and is saved for the backward, which sweeps upward (its mileage gradient is a prefix sum in j).
//
// Backward (corope_attn_gqa_pytorch.py:182-298), with g = dS * s and dS = P (dP - delta):
//     dq1_h += g K'1, dq2_h += g K'2;   dk1_j += (sum_h g q1) cos - (sum_h g q2) sin,  dk2_j += (sum_h g q2) cos + (sum_h g q1) sin
//     gD_ij = - sum_h g_hij * sum_d w_d ( q1 (k1 sin - k2 cos) + q2 (k2 sin + k1 cos) )
//     gz_ik = sum_{j<k} gD_ij (k <= i),  graw = gz z (1 - z) s,  dqL_i += graw k,  dk_k += graw qL_i
// dK / dV partial sums of a CTA's 8 rows are combined in shared memory and added to fp32 global accumulators.
#include "common.cuh"

namespace corope {
namespace {

constexpr int kWarps = 8;      // query rows per CTA
constexpr int kTile = 32;      // keys per step
constexpr int kThreads = kWarps * 32;
constexpr int kPad = 4;        // row padding (floats) of the per-lane K / V tiles: rows stay 16-byte aligned and 16-byte loads of 8
                               // consecutive lanes fall into distinct bank groups

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// inclusive prefix sum over lanes (lane 0 first)
__device__ __forceinline__ float warp_prefix_incl(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}
// inclusive suffix sum over lanes (lane 31 first)
__device__ __forceinline__ float warp_suffix_incl(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float t = __shfl_down_sync(0xffffffffu, v, o);
        if (lane + o < 32) v += t;
    }
    return v;
}

template <bool ACCURATE>
__device__ __forceinline__ void sincos_phase(float x, float* s, float* c, bool direct) {
    if (ACCURATE) {
        sincosf(x, s, c);
    } else if (direct) {
        // phases up to a few thousand radians (N <= 8192): the hardware approximations alone; their internal range
        // reduction in fp32 costs ~1e-4 rad there, far inside the 16-bit tolerance
        __sincosf(x, s, c);
    } else {
        // 16-bit inputs: two-constant reduction to [-pi, pi] then the fast hardware approximations
        float kf = rintf(x * 0.15915494309189535f);
        float r = fmaf(kf, -6.28318548202514648f, x);
        r = fmaf(kf, 1.7484555e-7f, r);
        __sincosf(r, s, c);
    }
}

template <typename T, int D>
__device__ __forceinline__ void stage_plain(float* dst, int ld, const T* X, int64_t xs, int r0, int rows, int N) {   // xs: row stride of X
    for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
        int r = idx / D, d = idx % D;
        int pos = r0 + r;
        dst[r * ld + d] = pos < N ? Elem<T>::to_f32(X[(int64_t)pos * xs + d]) : 0.f;
    }
}

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
template <typename T, int D, int G, bool ACCURATE>
__global__ void __launch_bounds__(kThreads) corope_fwd_general_kernel(GqaParams p) {
    constexpr int H2 = D / 2;
    constexpr int NC = D / 32;
    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                         // [G][8][D]
    float* k_s = q_s + G * kWarps * D;         // [32][D+1]
    float* v_s = k_s + kTile * (D + kPad);        // [32][D]
    float* w_s = v_s + kTile * D;              // [H2] inverse frequencies

    const int N = p.N;
    const int bg = blockIdx.y;                 // b * Hkv + g
    const int b = bg / p.Hkv, g = bg % p.Hkv;
    const int i0 = (gridDim.x - 1 - blockIdx.x) * kWarps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = i0 + warp;
    const size_t q_head0 = ((size_t)b * p.Hq + (size_t)g * G);
    const T* K = reinterpret_cast<const T*>(p.k) + row_offset(p.sk, p.Hkv, bg, 0);
    const T* V = reinterpret_cast<const T*>(p.v) + row_offset(p.sv, p.Hkv, bg, 0);

    for (int h = 0; h < G; ++h)
        stage_plain<T, D>(q_s + h * kWarps * D, D, reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.Hq, (int)q_head0 + h, 0), p.sq.n, i0, kWarps, N);
    for (int d = threadIdx.x; d < H2; d += kThreads) w_s[d] = 1.0f / powf(p.theta, (float)(2 * d) / (float)D);

    float m[G], l[G], acc[G][NC];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[h][c] = 0.f;
    }
    float carry = 0.f;  // sum of z_ik over keys already swept (k > current tile), for this warp's row
    const float sc2 = p.sm_scale * kLog2e;
    const bool direct = p.N <= 8192;
    const int i_last = min(N - 1, i0 + kWarps - 1);
    for (int j0 = (i_last / kTile) * kTile; j0 >= 0; j0 -= kTile) {
        __syncthreads();
        stage_plain<T, D>(k_s, D + kPad, K, p.sk.n, j0, kTile, N);
        stage_plain<T, D>(v_s, D, V, p.sv.n, j0, kTile, N);
        __syncthreads();
        if (i >= N) continue;
        const int j = j0 + lane;
        const bool vis = (j <= i);  // implies j < N
        const float* kr = k_s + lane * (D + kPad);
        const float* qL = q_s + warp * D;
        // leader score -> z   (16-byte shared-memory loads throughout: the loop is load-issue bound otherwise)
        float dot = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            const float4 a = *reinterpret_cast<const float4*>(qL + d);
            const float4 b = *reinterpret_cast<const float4*>(kr + d);
            dot = fmaf(a.x, b.x, dot);
            dot = fmaf(a.y, b.y, dot);
            dot = fmaf(a.z, b.z, dot);
            dot = fmaf(a.w, b.w, dot);
        }
        float z = vis ? 1.f / (1.f + __expf(-dot * p.sm_scale)) : 0.f;
        // Delta_ij = sum_{k=j+1..i} z_ik = carry + (suffix over lanes above this one)
        float suf = warp_suffix_incl(z, lane);
        float delta = carry + suf - z;
        carry += __shfl_sync(0xffffffffu, suf, 0);
        // scores of the G heads
        float s[G];
#pragma unroll
        for (int h = 0; h < G; ++h) s[h] = 0.f;
#pragma unroll 1
        for (int d = 0; d < H2; d += 4) {
            const float4 w4 = *reinterpret_cast<const float4*>(w_s + d);
            const float4 k1v = *reinterpret_cast<const float4*>(kr + d);
            const float4 k2v = *reinterpret_cast<const float4*>(kr + d + H2);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
            const float k1a[4] = {k1v.x, k1v.y, k1v.z, k1v.w}, k2a[4] = {k2v.x, k2v.y, k2v.z, k2v.w};
            float r1[4], r2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sn, cs;
                sincos_phase<ACCURATE>(delta * wv[e], &sn, &cs, direct);
                r1[e] = fmaf(k1a[e], cs, k2a[e] * sn);
                r2[e] = fmaf(k2a[e], cs, -k1a[e] * sn);
            }
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float* qh = q_s + (h * kWarps + warp) * D;
                const float4 q1v = *reinterpret_cast<const float4*>(qh + d);
                const float4 q2v = *reinterpret_cast<const float4*>(qh + d + H2);
                float acc = s[h];
                acc = fmaf(q1v.x, r1[0], acc); acc = fmaf(q2v.x, r2[0], acc);
                acc = fmaf(q1v.y, r1[1], acc); acc = fmaf(q2v.y, r2[1], acc);
                acc = fmaf(q1v.z, r1[2], acc); acc = fmaf(q2v.z, r2[2], acc);
                acc = fmaf(q1v.w, r1[3], acc); acc = fmaf(q2v.w, r2[3], acc);
                s[h] = acc;
            }
        }
        // online softmax per head (log2 domain), then P V with lane = column
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float sv = vis ? s[h] * sc2 : -INFINITY;
            float mx = fmaxf(m[h], warp_max(sv));
            float alpha = exp2f(m[h] - mx);   // first tile holds the diagonal, so mx is finite
            float pv = vis ? exp2f(sv - mx) : 0.f;
            l[h] = l[h] * alpha + warp_sum(pv);
            m[h] = mx;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[h][c] *= alpha;
            s[h] = pv;
        }
#pragma unroll 4
        for (int jj = 0; jj < kTile; ++jj) {
            float vv[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) vv[c] = v_s[jj * D + lane + 32 * c];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float pj = __shfl_sync(0xffffffffu, s[h], jj);
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[h][c] = fmaf(pj, vv[c], acc[h][c]);
            }
        }
    }
    if (i < N) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            T* O = reinterpret_cast<T*>(p.out_o) + row_offset(p.so, p.Hq, (int)q_head0 + h, i);
            float inv = 1.f / l[h];
#pragma unroll
            for (int c = 0; c < NC; ++c) O[lane + 32 * c] = Elem<T>::from_f32(acc[h][c] * inv);
            if (lane == 0) p.lse2[(q_head0 + h) * N + i] = m[h] + log2f(l[h]);
        }
        if (lane == 0) p.a_diag[(size_t)bg * N + i] = carry;
    }
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gqa_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, size_t rows, int D, RowAddr ao,
                                 RowAddr ado) {
    size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float s = 0.f;
    const T* orow = o + flat_row_offset(ao, row);
    const T* drow = d_o + flat_row_offset(ado, row);
    for (int d = lane; d < D; d += 32) s += Elem<T>::to_f32(orow[d]) * Elem<T>::to_f32(drow[d]);
    s = warp_sum(s);
    if (lane == 0) delta[row] = s;
}

template <typename T>
__global__ void gqa_finalize_kernel(const float* __restrict__ acc, T* __restrict__ out, size_t n, int D, RowAddr aout) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // over the contiguous fp32 accumulator [rows, D]
    if (i < n) out[flat_row_offset(aout, i / (size_t)D) + (int)(i % (size_t)D)] = Elem<T>::from_f32(acc[i]);
}

template <typename T, int D, int G, bool ACCURATE>
__global__ void __launch_bounds__(kThreads) corope_bwd_general_kernel(GqaParams p) {
    constexpr int H2 = D / 2;
    constexpr int NC = D / 32;                    // head-dim columns per lane
    constexpr int NPI = (H2 + 31) / 32;           // (d, d + D/2) pairs per lane
    constexpr int kXch = (2 * G + 2) * kTile;     // floats exchanged per warp between the two phases
    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                            // [G][8][D]
    float* do_s = q_s + G * kWarps * D;           // [G][8][D]
    float* k_s = do_s + G * kWarps * D;           // [32][D+1]
    float* v_s = k_s + kTile * (D + kPad);           // [32][D+1]
    float* dk_t = v_s + kTile * (D + kPad);          // [32][D] tile accumulators shared by the CTA's 8 rows
    float* dv_t = dk_t + kTile * D;               // [32][D]
    float* w_s = dv_t + kTile * D;                // [H2]
    float* xch = w_s + H2;                        // [8][kXch]

    const int N = p.N;
    const int bg = blockIdx.y;
    const int b = bg / p.Hkv, g = bg % p.Hkv;
    const int i0 = (gridDim.x - 1 - blockIdx.x) * kWarps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = i0 + warp;
    const size_t q_head0 = ((size_t)b * p.Hq + (size_t)g * G);
    const T* K = reinterpret_cast<const T*>(p.k) + row_offset(p.sk, p.Hkv, bg, 0);
    const T* V = reinterpret_cast<const T*>(p.v) + row_offset(p.sv, p.Hkv, bg, 0);
    float* dk_acc = p.dk_acc + (size_t)bg * N * D;
    float* dv_acc = p.dv_acc + (size_t)bg * N * D;
    float* xg = xch + warp * kXch;                // g[G][32]
    float* xp = xg + G * kTile;                   // P[G][32]
    float* xd = xp + G * kTile;                   // Delta[32]
    float* xr = xd + kTile;                       // graw[32]

    for (int h = 0; h < G; ++h) {
        stage_plain<T, D>(q_s + h * kWarps * D, D, reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.Hq, (int)q_head0 + h, 0), p.sq.n, i0, kWarps, N);
        stage_plain<T, D>(do_s + h * kWarps * D, D, reinterpret_cast<const T*>(p.d_o) + row_offset(p.sdo, p.Hq, (int)q_head0 + h, 0), p.sdo.n, i0, kWarps, N);
    }
    for (int d = threadIdx.x; d < H2; d += kThreads) w_s[d] = 1.0f / powf(p.theta, (float)(2 * d) / (float)D);
    for (int idx = threadIdx.x; idx < kTile * D; idx += kThreads) dk_t[idx] = dv_t[idx] = 0.f;

    float lse[G], dl[G], dq1[G][NPI], dq2[G][NPI];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        lse[h] = i < N ? p.lse2[(q_head0 + h) * N + i] : 0.f;
        dl[h] = i < N ? p.delta[(q_head0 + h) * N + i] : 0.f;
#pragma unroll
        for (int pi = 0; pi < NPI; ++pi) dq1[h][pi] = dq2[h][pi] = 0.f;
    }
    const float a_ii = i < N ? p.a_diag[(size_t)bg * N + i] : 0.f;
    float carry_a = 0.f, carry_g = 0.f;
    const float sc2 = p.sm_scale * kLog2e;
    const bool direct = p.N <= 8192;
    const int i_last = min(N - 1, i0 + kWarps - 1);
    for (int j0 = 0; j0 <= i_last; j0 += kTile) {
        __syncthreads();   // previous tile's flush done, accumulators are zero
        stage_plain<T, D>(k_s, D + kPad, K, p.sk.n, j0, kTile, N);
        stage_plain<T, D>(v_s, D + kPad, V, p.sv.n, j0, kTile, N);
        __syncthreads();
        if (i < N && j0 <= i) {
            // ---------------- phase A: lane = key
            const int j = j0 + lane;
            const bool vis = (j <= i);
            const float* kr = k_s + lane * (D + kPad);
            const float* vr = v_s + lane * (D + kPad);
            const float* qL = q_s + warp * D;
            float dot = 0.f;
#pragma unroll 4
            for (int d = 0; d < D; d += 4) {
                const float4 a = *reinterpret_cast<const float4*>(qL + d);
                const float4 b = *reinterpret_cast<const float4*>(kr + d);
                dot = fmaf(a.x, b.x, dot);
                dot = fmaf(a.y, b.y, dot);
                dot = fmaf(a.z, b.z, dot);
                dot = fmaf(a.w, b.w, dot);
            }
            const float z = vis ? 1.f / (1.f + __expf(-dot * p.sm_scale)) : 0.f;
            const float pre = warp_prefix_incl(z, lane);
            const float delta = a_ii - (carry_a + pre);
            carry_a += __shfl_sync(0xffffffffu, pre, 31);
            float s[G], tq[G], dp[G];
#pragma unroll
            for (int h = 0; h < G; ++h) s[h] = tq[h] = dp[h] = 0.f;
#pragma unroll 1
            for (int d = 0; d < H2; d += 4) {
                const float4 w4 = *reinterpret_cast<const float4*>(w_s + d);
                const float4 k1v = *reinterpret_cast<const float4*>(kr + d);
                const float4 k2v = *reinterpret_cast<const float4*>(kr + d + H2);
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
                const float k1a[4] = {k1v.x, k1v.y, k1v.z, k1v.w}, k2a[4] = {k2v.x, k2v.y, k2v.z, k2v.w};
                float r1[4], r2[4], wr1[4], wr2[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float sn, cs;
                    sincos_phase<ACCURATE>(delta * wv[e], &sn, &cs, direct);
                    r1[e] = fmaf(k1a[e], cs, k2a[e] * sn);
                    r2[e] = fmaf(k2a[e], cs, -k1a[e] * sn);
                    wr1[e] = wv[e] * r1[e];
                    wr2[e] = wv[e] * r2[e];
                }
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float* qh = q_s + (h * kWarps + warp) * D;
                    const float4 q1v = *reinterpret_cast<const float4*>(qh + d);
                    const float4 q2v = *reinterpret_cast<const float4*>(qh + d + H2);
                    const float q1a[4] = {q1v.x, q1v.y, q1v.z, q1v.w}, q2a[4] = {q2v.x, q2v.y, q2v.z, q2v.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[h] = fmaf(q1a[e], r1[e], s[h]);
                        s[h] = fmaf(q2a[e], r2[e], s[h]);
                        tq[h] = fmaf(q2a[e], wr1[e], tq[h]);
                        tq[h] = fmaf(-q1a[e], wr2[e], tq[h]);
                    }
                }
            }
#pragma unroll 2
            for (int d = 0; d < D; d += 4) {
                const float4 vv = *reinterpret_cast<const float4*>(vr + d);
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float4 g4 = *reinterpret_cast<const float4*>(do_s + (h * kWarps + warp) * D + d);
                    dp[h] = fmaf(g4.x, vv.x, dp[h]);
                    dp[h] = fmaf(g4.y, vv.y, dp[h]);
                    dp[h] = fmaf(g4.z, vv.z, dp[h]);
                    dp[h] = fmaf(g4.w, vv.w, dp[h]);
                }
            }
            float gD = 0.f;
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float pv = vis ? exp2f(s[h] * sc2 - lse[h]) : 0.f;
                float gT = pv * (dp[h] - dl[h]) * p.sm_scale;
                gD = fmaf(-gT, tq[h], gD);
                xg[h * kTile + lane] = gT;
                xp[h * kTile + lane] = pv;
            }
            const float gpre = warp_prefix_incl(gD, lane);
            const float gz = carry_g + gpre - gD;
            carry_g += __shfl_sync(0xffffffffu, gpre, 31);
            xd[lane] = delta;
            xr[lane] = vis ? gz * z * (1.f - z) * p.sm_scale : 0.f;
            __syncwarp();
            // ---------------- phase B: lane = head-dim pair / column
            const int jj_end = min(kTile, i - j0 + 1);
            for (int jj = 0; jj < jj_end; ++jj) {
                const float dlt = xd[jj], graw = xr[jj];
#pragma unroll
                for (int pi = 0; pi < NPI; ++pi) {
                    const int pd = lane + 32 * pi;
                    if (pd < H2) {
                        float sn, cs;
                        sincos_phase<ACCURATE>(dlt * w_s[pd], &sn, &cs, direct);
                        float k1 = k_s[jj * (D + kPad) + pd], k2 = k_s[jj * (D + kPad) + pd + H2];
                        float r1 = fmaf(k1, cs, k2 * sn);
                        float r2 = fmaf(k2, cs, -k1 * sn);
                        float a1 = 0.f, a2 = 0.f;
#pragma unroll
                        for (int h = 0; h < G; ++h) {
                            float gT = xg[h * kTile + jj];
                            dq1[h][pi] = fmaf(gT, r1, dq1[h][pi]);
                            dq2[h][pi] = fmaf(gT, r2, dq2[h][pi]);
                            a1 = fmaf(gT, q_s[(h * kWarps + warp) * D + pd], a1);
                            a2 = fmaf(gT, q_s[(h * kWarps + warp) * D + pd + H2], a2);
                        }
                        dq1[0][pi] = fmaf(graw, k1, dq1[0][pi]);
                        dq2[0][pi] = fmaf(graw, k2, dq2[0][pi]);
                        float dk1 = a1 * cs - a2 * sn + graw * qL[pd];
                        float dk2 = a2 * cs + a1 * sn + graw * qL[pd + H2];
                        atomicAdd(&dk_t[jj * D + pd], dk1);
                        atomicAdd(&dk_t[jj * D + pd + H2], dk2);
                    }
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int col = lane + 32 * c;
                    float a = 0.f;
#pragma unroll
                    for (int h = 0; h < G; ++h) a = fmaf(xp[h * kTile + jj], do_s[(h * kWarps + warp) * D + col], a);
                    atomicAdd(&dv_t[jj * D + col], a);
                }
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < kTile * D; idx += kThreads) {
            int r = idx / D;
            if (j0 + r < N && j0 + r <= i_last) {
                atomicAdd(&dk_acc[(size_t)(j0 + r) * D + (idx % D)], dk_t[idx]);
                atomicAdd(&dv_acc[(size_t)(j0 + r) * D + (idx % D)], dv_t[idx]);
            }
            dk_t[idx] = 0.f;
            dv_t[idx] = 0.f;
        }
    }
    if (i < N) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            T* DQ = reinterpret_cast<T*>(p.dq) + row_offset(p.sdq, p.Hq, (int)q_head0 + h, i);
#pragma unroll
            for (int pi = 0; pi < NPI; ++pi) {
                const int pd = lane + 32 * pi;
                if (pd < H2) {
                    DQ[pd] = Elem<T>::from_f32(dq1[h][pi]);
                    DQ[pd + H2] = Elem<T>::from_f32(dq2[h][pi]);
                }
            }
        }
    }
}

template <typename T, int D, int G>
int launch_fwd_g(const GqaParams& p, cudaStream_t s) {
    constexpr bool kAcc = (Elem<T>::kDtype == COROPE_DTYPE_F32);
    size_t smem = sizeof(float) * ((size_t)G * kWarps * D + kTile * (D + kPad) + kTile * D + D / 2);
    auto kern = corope_fwd_general_kernel<T, D, G, kAcc>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((p.N + kWarps - 1) / kWarps, p.B * p.Hkv);
    kern<<<grid, kThreads, smem, s>>>(p); count_launch();
    return (int)cudaGetLastError();
}

template <typename T, int D, int G>
int launch_bwd_g(const GqaParams& p, cudaStream_t s) {
    constexpr bool kAcc = (Elem<T>::kDtype == COROPE_DTYPE_F32);
    size_t smem = sizeof(float) * ((size_t)2 * G * kWarps * D + 2 * kTile * (D + kPad) + 2 * kTile * D + D / 2 + (size_t)kWarps * (2 * G + 2) * kTile);
    auto kern = corope_bwd_general_kernel<T, D, G, kAcc>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((p.N + kWarps - 1) / kWarps, p.B * p.Hkv);
    kern<<<grid, kThreads, smem, s>>>(p); count_launch();
    return (int)cudaGetLastError();
}

template <typename T, int D>
int dispatch_g(const GqaParams& p, cudaStream_t s, bool bwd) {
    switch (p.G) {
        case 1: return bwd ? launch_bwd_g<T, D, 1>(p, s) : launch_fwd_g<T, D, 1>(p, s);
        case 2: return bwd ? launch_bwd_g<T, D, 2>(p, s) : launch_fwd_g<T, D, 2>(p, s);
        case 4: return bwd ? launch_bwd_g<T, D, 4>(p, s) : launch_fwd_g<T, D, 4>(p, s);
        case 8: return bwd ? launch_bwd_g<T, D, 8>(p, s) : launch_fwd_g<T, D, 8>(p, s);
        case 3: return bwd ? launch_bwd_g<T, D, 3>(p, s) : launch_fwd_g<T, D, 3>(p, s);
        case 5: return bwd ? launch_bwd_g<T, D, 5>(p, s) : launch_fwd_g<T, D, 5>(p, s);
        case 6: return bwd ? launch_bwd_g<T, D, 6>(p, s) : launch_fwd_g<T, D, 6>(p, s);
        case 7: return bwd ? launch_bwd_g<T, D, 7>(p, s) : launch_fwd_g<T, D, 7>(p, s);
        default: return COROPE_ERR_BAD_GROUP;
    }
}

template <typename T>
int dispatch_gd(const GqaParams& p, cudaStream_t s, bool bwd) {
    switch (p.D) {
        case 32: return dispatch_g<T, 32>(p, s, bwd);
        case 64: return dispatch_g<T, 64>(p, s, bwd);
        case 128: return dispatch_g<T, 128>(p, s, bwd);
        default: return COROPE_ERR_BAD_HEAD_DIM;
    }
}

template <typename T>
int bwd_all(const GqaParams& p, cudaStream_t s) {
    const size_t rows = (size_t)p.B * p.Hq * p.N;
    const size_t kv_elems = (size_t)p.B * p.Hkv * p.N * p.D;
    gqa_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const T*)p.o, (const T*)p.d_o, p.delta, rows, p.D, row_addr(p.so, p.Hq, p.N),
                                                                           row_addr(p.sdo, p.Hq, p.N)); count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if ((e = cudaMemsetAsync(p.dk_acc, 0, kv_elems * sizeof(float), s)) != cudaSuccess) return (int)e;
    if ((e = cudaMemsetAsync(p.dv_acc, 0, kv_elems * sizeof(float), s)) != cudaSuccess) return (int)e;
    if (int r = p.use_mma ? launch_gqa_bwd_mma(p, Elem<T>::kDtype, s) : dispatch_gd<T>(p, s, true)) return r;
    gqa_finalize_kernel<T><<<(unsigned)((kv_elems + 255) / 256), 256, 0, s>>>(p.dk_acc, (T*)p.dk, kv_elems, p.D, row_addr(p.sdk, p.Hkv, p.N)); count_launch();
    gqa_finalize_kernel<T><<<(unsigned)((kv_elems + 255) / 256), 256, 0, s>>>(p.dv_acc, (T*)p.dv, kv_elems, p.D, row_addr(p.sdv, p.Hkv, p.N)); count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

int launch_gqa_fwd_general(const GqaParams& p, int dtype, cudaStream_t s) {
    switch (dtype) {
        case COROPE_DTYPE_F32: return dispatch_gd<float>(p, s, false);
        case COROPE_DTYPE_BF16: return dispatch_gd<__nv_bfloat16>(p, s, false);
        case COROPE_DTYPE_F16: return dispatch_gd<__half>(p, s, false);
        default: return COROPE_ERR_BAD_DTYPE;
    }
}

int launch_gqa_bwd_general(const GqaParams& p, int dtype, cudaStream_t s) {
    switch (dtype) {
        case COROPE_DTYPE_F32: return bwd_all<float>(p, s);
        case COROPE_DTYPE_BF16: return bwd_all<__nv_bfloat16>(p, s);
        case COROPE_DTYPE_F16: return bwd_all<__half>(p, s);
        default: return COROPE_ERR_BAD_DTYPE;
    }
}

}  // namespace corope
