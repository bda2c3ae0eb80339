// General fused-RoPE attention kernels: fp32 arithmetic on the CUDA cores, any N, causal or not,
// D in {32, 64, 128}, inputs fp32 / bf16 / fp16.  This is the accuracy path (fp32 inputs must match
// the fp32 reference to 1e-4, which rules out 16-bit tensor-core operands) and the path for shapes the
// tensor-core kernels do not take.  Q and every K tile are rotated while being staged into shared
// memory; rotated values never go back to HBM.
//
// Tiling: one CTA = 32 rows (queries for fwd / dQ, keys for dK / dV), 4 warps x 8 rows; the other
// operand streams through shared memory in tiles of 32.  Within a warp, lane = column of the
// 32 x 32 score tile for the dot products, and lane = head-dim column (lane + 32 c) for the
// accumulators.
//
// Math follows fused-rope/rope_attn_pytorch.py:108-155 (forward) and :187-222 (backward); the exp2-domain
// softmax and the log2-domain LSE follow fused-rope/fused_rope_attn.py:103-114, 316.
#include "common.cuh"

namespace corope {
namespace {

constexpr int kRows = 32;     // rows per CTA
constexpr int kTile = 32;     // streamed rows per step
constexpr int kThreads = 128;
constexpr int kRowsPerWarp = 8;

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

// Stage `kTile` rows [r0, r0+32) of X[N][D] into dst[32][LD] as fp32, rotated by the half-layout RoPE
// and multiplied by `scale`.  Rows >= N become zeros.
template <typename T, int D, int LD, bool ROTATE>
__device__ __forceinline__ void stage_rows(float* dst, const T* X, int64_t xs, int r0, int N, const float* cosT, const float* sinT, int64_t ts,
                                           float scale) {   // xs: row stride of X in elements
    constexpr int H2 = D / 2;
    for (int idx = threadIdx.x; idx < kTile * H2; idx += kThreads) {
        int r = idx / H2, d = idx % H2;
        int pos = r0 + r;
        float y1 = 0.f, y2 = 0.f;
        if (pos < N) {
            float x1 = Elem<T>::to_f32(X[(int64_t)pos * xs + d]);
            float x2 = Elem<T>::to_f32(X[(int64_t)pos * xs + d + H2]);
            if (ROTATE && cosT != nullptr) {   // null tables: plain attention, no rotation
                float c = cosT[pos * ts + d], s = sinT[pos * ts + d];
                y1 = (x1 * c - x2 * s) * scale;
                y2 = (x2 * c + x1 * s) * scale;
            } else {
                y1 = x1 * scale;
                y2 = x2 * scale;
            }
        }
        dst[r * LD + d] = y1;
        dst[r * LD + d + H2] = y2;
    }
}

// 8 x 32 tile of dot products: out[r] = sum_d A[(row0 + r)][d] * Bp[lane][d]; A rows broadcast (stride D),
// B rows per lane (stride D + 1, conflict-free).
template <int D>
__device__ __forceinline__ void dot_rows(float (&out)[kRowsPerWarp], const float* A, int row0, const float* Bp, int lane) {
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) out[r] = 0.f;
    const float* b = Bp + lane * (D + 1);
#pragma unroll 4
    for (int d = 0; d < D; d += 4) {
        float b0 = b[d], b1 = b[d + 1], b2 = b[d + 2], b3 = b[d + 3];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            float4 a = *reinterpret_cast<const float4*>(A + (row0 + r) * D + d);
            out[r] = fmaf(a.x, b0, out[r]);
            out[r] = fmaf(a.y, b1, out[r]);
            out[r] = fmaf(a.z, b2, out[r]);
            out[r] = fmaf(a.w, b3, out[r]);
        }
    }
}

// acc[r][c] += sum_j w[r] (held by lane j) * Bp[j][lane + 32 c]
template <int D, int LD>
__device__ __forceinline__ void accumulate_cols(float (&acc)[kRowsPerWarp][(D + 31) / 32], const float (&w)[kRowsPerWarp], const float* Bp,
                                                int lane) {
    constexpr int NC = D / 32;
#pragma unroll 4
    for (int j = 0; j < kTile; ++j) {
        float bv[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) bv[c] = Bp[j * LD + lane + 32 * c];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            float wj = __shfl_sync(0xffffffffu, w[r], j);
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[r][c] = fmaf(wj, bv[c], acc[r][c]);
        }
    }
}

// Inverse rotation of a row held as columns (lane + 32 c), then * scale, stored as T.
template <typename T, int D>
__device__ __forceinline__ void store_inverse_rotated(T* dst_row, const float (&a)[(D + 31) / 32], int pos, const float* cosT,
                                                      const float* sinT, int64_t ts, float scale, int lane, bool rotate) {
    constexpr int NC = D / 32;
    constexpr int H2 = D / 2;
    if (D == 32) {
        float other = __shfl_xor_sync(0xffffffffu, a[0], 16);
        int d = lane & 15;
        float c = rotate ? cosT[pos * ts + d] : 1.f, s = rotate ? sinT[pos * ts + d] : 0.f;
        float g = lane < 16 ? (a[0] * c + other * s) : (a[0] * c - other * s);
        dst_row[lane] = Elem<T>::from_f32(g * scale);
    } else {
#pragma unroll
        for (int c2 = 0; c2 < NC / 2; ++c2) {
            int d = lane + 32 * c2;
            float c = rotate ? cosT[pos * ts + d] : 1.f, s = rotate ? sinT[pos * ts + d] : 0.f;
            float a1 = a[c2], a2 = a[c2 + NC / 2];
            dst_row[d] = Elem<T>::from_f32((a1 * c + a2 * s) * scale);
            dst_row[d + H2] = Elem<T>::from_f32((a2 * c - a1 * s) * scale);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) rope_fwd_general_kernel(RopeParams p) {
    constexpr int NC = D / 32;
    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                       // [32][D]     rotated * sm_scale * log2e
    float* k_s = q_s + kRows * D;            // [32][D+1]   rotated
    float* v_s = k_s + kTile * (D + 1);      // [32][D]

    const int N = p.N;
    const int bh = blockIdx.y;
    const int m0 = (gridDim.x - 1 - blockIdx.x) * kRows;  // longest causal rows first
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = bh / (p.H / p.Hkv);   // [B, H] flattened -> [B, Hkv] flattened: the heads of a group are adjacent
    const T* Q = reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.H, bh, 0);
    const T* K = reinterpret_cast<const T*>(p.k) + row_offset(p.sk, p.Hkv, kvh, 0);
    const T* V = reinterpret_cast<const T*>(p.v) + row_offset(p.sv, p.Hkv, kvh, 0);
    T* O = reinterpret_cast<T*>(p.out_o) + row_offset(p.so, p.H, bh, 0);

    stage_rows<T, D, D, true>(q_s, Q, p.sq.n, m0, N, p.cos, p.sin, p.table_stride, p.sm_scale * kLog2e);

    float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][NC];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
    }
    const int row0 = warp * kRowsPerWarp;
    const int n_end = p.causal ? min(N, m0 + kRows) : N;
    for (int j0 = 0; j0 < n_end; j0 += kTile) {
        __syncthreads();
        stage_rows<T, D, D + 1, true>(k_s, K, p.sk.n, j0, N, p.cos, p.sin, p.table_stride, 1.f);
        stage_rows<T, D, D, false>(v_s, V, p.sv.n, j0, N, nullptr, nullptr, 0, 1.f);
        __syncthreads();
        float s[kRowsPerWarp];
        dot_rows<D>(s, q_s, row0, k_s, lane);
        const int j = j0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int i = m0 + row0 + r;
            bool ok = (j < N) && (!p.causal || j <= i);
            float sv = ok ? s[r] : -INFINITY;
            float mx = fmaxf(m[r], warp_max(sv));
            float alpha = (mx == -INFINITY) ? 1.f : exp2f(m[r] - mx);
            float pv = (mx == -INFINITY || !ok) ? 0.f : exp2f(sv - mx);
            l[r] = l[r] * alpha + warp_sum(pv);
            m[r] = mx;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[r][c] *= alpha;
            s[r] = pv;
        }
        accumulate_cols<D, D>(acc, s, v_s, lane);
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = m0 + row0 + r;
        if (i >= N) continue;
        float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) O[(int64_t)i * p.so.n + lane + 32 * c] = Elem<T>::from_f32(acc[r][c] * inv);
        if (lane == 0) p.lse2[(size_t)bh * N + i] = m[r] + log2f(l[r]);
    }
}

// ------------------------------------------------------------------------------------------------
// delta = rowsum(O * dO)   (fused_rope_attn.py:324-337)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, size_t rows, int D, RowAddr ao,
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

// Same for 16-bit elements and D = 128: 16 threads per row, 16 bytes of O and of dO per thread.
template <typename T>
__global__ void rope_delta_d128_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, size_t rows, RowAddr ao,
                                       RowAddr ado) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t row = t >> 4;
    const int part = (int)(t & 15);
    float s = 0.f;
    if (row < rows) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + flat_row_offset(ao, row)) + part);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(d_o + flat_row_offset(ado, row)) + part);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = unpack2<T>(aw[i]), fb = unpack2<T>(bw[i]);
            s = fmaf(fa.x, fb.x, s);
            s = fmaf(fa.y, fb.y, s);
        }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (part == 0 && row < rows) delta[row] = s;
}

// ------------------------------------------------------------------------------------------------
// backward, dQ: one CTA per 32 query rows, streams K/V tiles
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) rope_bwd_dq_general_kernel(RopeParams p) {
    constexpr int NC = D / 32;
    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                        // [32][D]   rotated * sm_scale * log2e
    float* do_s = q_s + kRows * D;            // [32][D]
    float* k_s = do_s + kRows * D;            // [32][D+1] rotated
    float* v_s = k_s + kTile * (D + 1);       // [32][D+1]

    const int N = p.N;
    const int bh = blockIdx.y;
    const int m0 = (gridDim.x - 1 - blockIdx.x) * kRows;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = bh / (p.H / p.Hkv);
    const T* Q = reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.H, bh, 0);
    const T* K = reinterpret_cast<const T*>(p.k) + row_offset(p.sk, p.Hkv, kvh, 0);
    const T* V = reinterpret_cast<const T*>(p.v) + row_offset(p.sv, p.Hkv, kvh, 0);
    const T* DO = reinterpret_cast<const T*>(p.d_o) + row_offset(p.sdo, p.H, bh, 0);
    T* DQ = reinterpret_cast<T*>(p.dq) + row_offset(p.sdq, p.H, bh, 0);

    stage_rows<T, D, D, true>(q_s, Q, p.sq.n, m0, N, p.cos, p.sin, p.table_stride, p.sm_scale * kLog2e);
    stage_rows<T, D, D, false>(do_s, DO, p.sdo.n, m0, N, nullptr, nullptr, 0, 1.f);

    const int row0 = warp * kRowsPerWarp;
    float lse[kRowsPerWarp], dl[kRowsPerWarp], acc[kRowsPerWarp][NC];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = m0 + row0 + r;
        lse[r] = i < N ? p.lse2[(size_t)bh * N + i] : 0.f;
        dl[r] = i < N ? p.delta[(size_t)bh * N + i] : 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
    }
    const int n_end = p.causal ? min(N, m0 + kRows) : N;
    for (int j0 = 0; j0 < n_end; j0 += kTile) {
        __syncthreads();
        stage_rows<T, D, D + 1, true>(k_s, K, p.sk.n, j0, N, p.cos, p.sin, p.table_stride, 1.f);
        stage_rows<T, D, D + 1, false>(v_s, V, p.sv.n, j0, N, nullptr, nullptr, 0, 1.f);
        __syncthreads();
        float s[kRowsPerWarp], dp[kRowsPerWarp];
        dot_rows<D>(s, q_s, row0, k_s, lane);
        dot_rows<D>(dp, do_s, row0, v_s, lane);
        const int j = j0 + lane;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int i = m0 + row0 + r;
            bool ok = (j < N) && (i < N) && (!p.causal || j <= i);
            float pv = ok ? exp2f(s[r] - lse[r]) : 0.f;
            s[r] = pv * (dp[r] - dl[r]);
        }
        accumulate_cols<D, D + 1>(acc, s, k_s, lane);
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = m0 + row0 + r;
        if (i >= N) continue;  // warp-uniform: i does not depend on the lane
        store_inverse_rotated<T, D>(DQ + (int64_t)i * p.sdq.n, acc[r], i, p.cos, p.sin, p.table_stride, p.sm_scale, lane, p.cos != nullptr);
    }
}

// ------------------------------------------------------------------------------------------------
// backward, dK / dV: one CTA per 32 keys, streams Q / dO tiles
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) rope_bwd_dkdv_general_kernel(RopeParams p) {
    constexpr int NC = D / 32;
    extern __shared__ __align__(16) float smem[];
    float* k_s = smem;                        // [32][D]   rotated
    float* v_s = k_s + kRows * D;             // [32][D]
    float* q_s = v_s + kRows * D;             // [32][D+1] rotated * sm_scale * log2e
    float* do_s = q_s + kTile * (D + 1);      // [32][D+1]
    float* lse_s = do_s + kTile * (D + 1);    // [32]
    float* dl_s = lse_s + kTile;              // [32]

    const int N = p.N;
    const int kvh = blockIdx.y;         // KV head (over batch x Hkv); its G query heads are kvh * G .. kvh * G + G - 1
    const int G = p.H / p.Hkv;
    const int n0 = blockIdx.x * kRows;  // causal: low key blocks are the long ones and come first
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* K = reinterpret_cast<const T*>(p.k) + row_offset(p.sk, p.Hkv, kvh, 0);
    const T* V = reinterpret_cast<const T*>(p.v) + row_offset(p.sv, p.Hkv, kvh, 0);
    T* DK = reinterpret_cast<T*>(p.dk) + row_offset(p.sdk, p.Hkv, kvh, 0);
    T* DV = reinterpret_cast<T*>(p.dv) + row_offset(p.sdv, p.Hkv, kvh, 0);

    stage_rows<T, D, D, true>(k_s, K, p.sk.n, n0, N, p.cos, p.sin, p.table_stride, 1.f);
    stage_rows<T, D, D, false>(v_s, V, p.sv.n, n0, N, nullptr, nullptr, 0, 1.f);

    const int row0 = warp * kRowsPerWarp;
    float dk[kRowsPerWarp][NC], dv[kRowsPerWarp][NC];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c) dk[r][c] = dv[r][c] = 0.f;

    const int i_begin = p.causal ? n0 : 0;
    for (int g = 0; g < G; ++g) {   // dK / dV are summed over the group's query heads
    const int bh = kvh * G + g;
    const T* Q = reinterpret_cast<const T*>(p.q) + row_offset(p.sq, p.H, bh, 0);
    const T* DO = reinterpret_cast<const T*>(p.d_o) + row_offset(p.sdo, p.H, bh, 0);
    for (int i0 = i_begin; i0 < N; i0 += kTile) {
        __syncthreads();
        stage_rows<T, D, D + 1, true>(q_s, Q, p.sq.n, i0, N, p.cos, p.sin, p.table_stride, p.sm_scale * kLog2e);
        stage_rows<T, D, D + 1, false>(do_s, DO, p.sdo.n, i0, N, nullptr, nullptr, 0, 1.f);
        if (threadIdx.x < kTile) {
            int i = i0 + threadIdx.x;
            lse_s[threadIdx.x] = i < N ? p.lse2[(size_t)bh * N + i] : 0.f;
            dl_s[threadIdx.x] = i < N ? p.delta[(size_t)bh * N + i] : 0.f;
        }
        __syncthreads();
        float s[kRowsPerWarp], dp[kRowsPerWarp];
        dot_rows<D>(s, k_s, row0, q_s, lane);
        dot_rows<D>(dp, v_s, row0, do_s, lane);
        const int i = i0 + lane;
        const float lse = lse_s[lane], dl = dl_s[lane];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int j = n0 + row0 + r;
            bool ok = (j < N) && (i < N) && (!p.causal || j <= i);
            float pv = ok ? exp2f(s[r] - lse) : 0.f;
            s[r] = pv;
            dp[r] = pv * (dp[r] - dl);
        }
        accumulate_cols<D, D + 1>(dv, s, do_s, lane);
        accumulate_cols<D, D + 1>(dk, dp, q_s, lane);
    }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int j = n0 + row0 + r;
        if (j >= N) continue;
#pragma unroll
        for (int c = 0; c < NC; ++c) DV[(int64_t)j * p.sdv.n + lane + 32 * c] = Elem<T>::from_f32(dv[r][c]);
        // q_s carried sm_scale * log2e, so dk holds dK~ * log2e: undo with ln2
        store_inverse_rotated<T, D>(DK + (int64_t)j * p.sdk.n, dk[r], j, p.cos, p.sin, p.table_stride, kLn2, lane, p.cos != nullptr);
    }
}

// cos/sin fp32 tables -> compact [N][D/2] table of (cos, sin) pairs in 16-bit offset-binary fixed point
// (see pack_unorm_pair): half the bytes of the fp32 tables with an absolute error of 1.5e-5.
// half_src < half_d: the caller's tables have half_src columns; the pairs beyond them get the identity rotation (used when
// a D = 64 problem is run zero-padded on the D = 128 kernels).
__global__ void pack_tables_kernel(const float* __restrict__ cosT, const float* __restrict__ sinT, int64_t ts, uint32_t* __restrict__ out,
                                   int N, int half_d, int half_src) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx == 0) out[(size_t)N * half_d] = 0u;   // the word after the table: work counter of the persistent forward kernel
    if (idx >= (size_t)N * half_d) return;
    int n = (int)(idx / half_d), d = (int)(idx % half_d);
    out[idx] = (cosT != nullptr && d < half_src) ? pack_unorm_pair(cosT[n * ts + d], sinT[n * ts + d]) : pack_unorm_pair(1.f, 0.f);
}

// cos / sin tables for positions 0 .. N-1 from the per-pair frequencies, as precompute_freqs_cis forms them
// (fused-rope/rope_attn_pytorch.py:33-47): angle = float(position) * inv_freq[d] in fp32, then cos / sin of it.
__global__ void synth_tables_kernel(const float* __restrict__ inv_freq, float* __restrict__ cosT, float* __restrict__ sinT, int N, int half_d) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)N * half_d) return;
    const int n = (int)(idx / half_d), d = (int)(idx % half_d);
    const float ang = __fmul_rn((float)n, inv_freq[d]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    cosT[idx] = cs;
    sinT[idx] = sn;
}

// D = 64 <-> D = 128 with zero padding, 16-byte chunks.  "rope" layout keeps the half-layout pairs together for the
// D = 128 kernels: first half of the row (32 columns) to columns 0..31, second half to columns 64..95; "plain" layout
// puts the 64 columns first.  Everything else is zero, so dot products and rotations are unchanged.
template <typename T>
__global__ void __launch_bounds__(256) unpad_d64_kernel(const T* __restrict__ xp, T* __restrict__ out, size_t rows, int rope_layout, RowAddr ax) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // rows * 8 output chunks
    if (idx >= rows * 8) return;
    const size_t r = idx >> 3;
    const int c = (int)(idx & 7);
    const int src = rope_layout ? (c < 4 ? c : c + 4) : c;
    *reinterpret_cast<uint4*>(out + flat_row_offset(ax, r) + c * 8) = *reinterpret_cast<const uint4*>(xp + r * 128 + src * 8);
}

// Up to four tensors per launch (blockIdx.y picks the tensor): the D = 64 problems that take this path are small, and their
// time is made of launches.
struct PadJob {
    const void* src;
    void* dst;
    size_t rows;
    int rope_layout;
    RowAddr addr;
};
struct PadJobs {
    PadJob j[4];
};
template <typename T>
__global__ void __launch_bounds__(256) pad_d64_many_kernel(PadJobs jobs) {
    const PadJob& jb = jobs.j[blockIdx.y];
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // rows * 16 output chunks
    if (idx >= jb.rows * 16) return;
    const size_t r = idx >> 4;
    const int c = (int)(idx & 15);
    int src = -1;
    if (jb.rope_layout) {
        if (c < 4) src = c;
        else if (c >= 8 && c < 12) src = c - 4;
    } else if (c < 8) {
        src = c;
    }
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (src >= 0) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(jb.src) + flat_row_offset(jb.addr, r) + src * 8);
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(jb.dst) + r * 128 + c * 8) = v;
}
template <typename T>
__global__ void __launch_bounds__(256) unpad_d64_many_kernel(PadJobs jobs) {
    const PadJob& jb = jobs.j[blockIdx.y];   // src = padded copy, dst = the caller's tensor
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // rows * 8 output chunks
    if (idx >= jb.rows * 8) return;
    const size_t r = idx >> 3;
    const int c = (int)(idx & 7);
    const int src = jb.rope_layout ? (c < 4 ? c : c + 4) : c;
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(jb.dst) + flat_row_offset(jb.addr, r) + c * 8) =
        *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(jb.src) + r * 128 + src * 8);
}

// Rotation as a pass of its own, for the tensor-core kernels at D = 128: out[r, :] = rot(x[r, :]) * scale as fp16, with the
// same packed table and the same arithmetic as the in-kernel rotation (rotate_vec8), so both give identical bits.  The
// forward uses it for K (every K tile is consumed by up to N/256 work items; rotating it once here instead of once per
// consumer removes the rotation from the forward's inner loop), the backward for Q (consumed by every key block below
// its diagonal).  One thread = 8 pairs of one row: two 16-byte loads, 32 bytes of table, two 16-byte stores.
template <typename T>
__global__ void __launch_bounds__(256) rope_prerotate_d128_kernel(const T* __restrict__ x, __half* __restrict__ out,
                                                                   const uint32_t* __restrict__ tab, size_t rows, int N, float scale, RowAddr ax) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * 8) return;
    const size_t row = idx >> 3;
    const int c = (int)(idx & 7) * 8;
    const int n = (int)(row % (size_t)N);
    const uint4* src = reinterpret_cast<const uint4*>(x + flat_row_offset(ax, row) + c);
    uint4 x1 = __ldg(src), x2 = __ldg(src + 8);
    const uint4* tp = reinterpret_cast<const uint4*>(tab + (size_t)n * 64 + c);
    const uint4 t0 = __ldg(tp), t1 = __ldg(tp + 1);
    rotate_vec8<T>(x1, x2, t0, t1, scale * (1.f / 32768.f), -257.f * scale);
    uint4* dst = reinterpret_cast<uint4*>(out + row * 128 + c);
    dst[0] = x1;
    dst[8] = x2;
}

// Everything the tensor-core backward needs before its main kernel, in one pass over the rows (16 threads per row):
// delta = rowsum(O * dO), the rotated and scaled fp16 copy of Q (threads 0-7 of a row: 8 pairs each, same arithmetic as
// rope_prerotate_d128_kernel) and a zeroed row of the fp32 dQ accumulator (32 bytes per thread).  One launch instead of
// a memset and two kernels; all three parts are bound by the same HBM traffic.
template <typename T>
__global__ void __launch_bounds__(256) rope_bwd_prepass_d128_kernel(const T* __restrict__ q, const T* __restrict__ o, const T* __restrict__ d_o,
                                                                     const uint32_t* __restrict__ tab, __half* __restrict__ q_rot,
                                                                     float* __restrict__ delta, float* __restrict__ dq_acc, size_t rows, int N,
                                                                     float scale, RowAddr aq, RowAddr ao, RowAddr ado) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t row = t >> 4;
    const int part = (int)(t & 15);
    const bool live = row < rows;
    float s = 0.f;
    if (live) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + flat_row_offset(ao, row)) + part);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(d_o + flat_row_offset(ado, row)) + part);
        if (part < 8) {
            const int c = part * 8;
            const int n = (int)(row % (size_t)N);
            const uint4* src = reinterpret_cast<const uint4*>(q + flat_row_offset(aq, row) + c);
            uint4 x1 = __ldg(src), x2 = __ldg(src + 8);
            const uint4* tp = reinterpret_cast<const uint4*>(tab + (size_t)n * 64 + c);
            const uint4 t0 = __ldg(tp), t1 = __ldg(tp + 1);
            rotate_vec8<T>(x1, x2, t0, t1, scale * (1.f / 32768.f), -257.f * scale);
            uint4* dst = reinterpret_cast<uint4*>(q_rot + row * 128 + c);
            dst[0] = x1;
            dst[8] = x2;
        }
        uint4* z = reinterpret_cast<uint4*>(dq_acc + row * 128) + part * 2;
        z[0] = make_uint4(0u, 0u, 0u, 0u);
        z[1] = make_uint4(0u, 0u, 0u, 0u);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = unpack2<T>(aw[i]), fb = unpack2<T>(bw[i]);
            s = fmaf(fa.x, fb.x, s);
            s = fmaf(fa.y, fb.y, s);
        }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (part == 0 && live) delta[row] = s;
}

template <typename T, int D>
int launch_fwd_t(const RopeParams& p, cudaStream_t s) {
    size_t smem = sizeof(float) * (kRows * D + kTile * (D + 1) + kTile * D);
    auto kern = rope_fwd_general_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((p.N + kRows - 1) / kRows, p.B * p.H);
    kern<<<grid, kThreads, smem, s>>>(p); count_launch();
    return (int)cudaGetLastError();
}

template <typename T, int D>
int launch_bwd_t(const RopeParams& p, cudaStream_t s) {
    dim3 grid((p.N + kRows - 1) / kRows, p.B * p.H);
    {
        size_t smem = sizeof(float) * (2 * kRows * D + 2 * kTile * (D + 1));
        auto kern = rope_bwd_dq_general_kernel<T, D>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, kThreads, smem, s>>>(p); count_launch();
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    {
        size_t smem = sizeof(float) * (2 * kRows * D + 2 * kTile * (D + 1) + 2 * kTile);
        auto kern = rope_bwd_dkdv_general_kernel<T, D>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        dim3 grid_kv((p.N + kRows - 1) / kRows, p.B * p.Hkv);   // one CTA per 32 keys of a KV head; it sums over the group's query heads
        kern<<<grid_kv, kThreads, smem, s>>>(p); count_launch();
        return (int)cudaGetLastError();
    }
}

template <typename T>
int dispatch_d(const RopeParams& p, cudaStream_t s, bool bwd) {
    switch (p.D) {
        case 32: return bwd ? launch_bwd_t<T, 32>(p, s) : launch_fwd_t<T, 32>(p, s);
        case 64: return bwd ? launch_bwd_t<T, 64>(p, s) : launch_fwd_t<T, 64>(p, s);
        case 128: return bwd ? launch_bwd_t<T, 128>(p, s) : launch_fwd_t<T, 128>(p, s);
        default: return COROPE_ERR_BAD_HEAD_DIM;
    }
}

}  // namespace

int launch_rope_fwd_general(const RopeParams& p, int dtype, cudaStream_t s) {
    switch (dtype) {
        case COROPE_DTYPE_F32: return dispatch_d<float>(p, s, false);
        case COROPE_DTYPE_BF16: return dispatch_d<__nv_bfloat16>(p, s, false);
        case COROPE_DTYPE_F16: return dispatch_d<__half>(p, s, false);
        default: return COROPE_ERR_BAD_DTYPE;
    }
}

int launch_rope_bwd_general(const RopeParams& p, int dtype, cudaStream_t s) {
    switch (dtype) {
        case COROPE_DTYPE_F32: return dispatch_d<float>(p, s, true);
        case COROPE_DTYPE_BF16: return dispatch_d<__nv_bfloat16>(p, s, true);
        case COROPE_DTYPE_F16: return dispatch_d<__half>(p, s, true);
        default: return COROPE_ERR_BAD_DTYPE;
    }
}

int launch_rope_delta(const RopeParams& p, int dtype, cudaStream_t s) {
    size_t rows = (size_t)p.B * p.H * p.N;
    // the 16-bytes-per-thread form needs 16-byte aligned rows; row strides that are not multiples of 8 elements take the scalar form
    auto aligned = [](const void* ptr, const Strides& st) {
        return ((uintptr_t)ptr % 16) == 0 && st.b % 8 == 0 && st.h % 8 == 0 && st.n % 8 == 0;
    };
    if (p.D == 128 && dtype != COROPE_DTYPE_F32 && aligned(p.o, p.so) && aligned(p.d_o, p.sdo)) {
        const unsigned blocks = (unsigned)((rows * 16 + 255) / 256);
        if (dtype == COROPE_DTYPE_BF16)
            rope_delta_d128_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)p.o, (const __nv_bfloat16*)p.d_o, p.delta, rows, row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N));
        else
            rope_delta_d128_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)p.o, (const __half*)p.d_o, p.delta, rows, row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N));
        count_launch();
        return (int)cudaGetLastError();
    }
    const int warps = 8;
    unsigned blocks = (unsigned)((rows + warps - 1) / warps);
    switch (dtype) {
        case COROPE_DTYPE_F32:
            rope_delta_kernel<float><<<blocks, warps * 32, 0, s>>>((const float*)p.o, (const float*)p.d_o, p.delta, rows, p.D, row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N)); count_launch();
            break;
        case COROPE_DTYPE_BF16:
            rope_delta_kernel<__nv_bfloat16>
                <<<blocks, warps * 32, 0, s>>>((const __nv_bfloat16*)p.o, (const __nv_bfloat16*)p.d_o, p.delta, rows, p.D, row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N)); count_launch();
            break;
        case COROPE_DTYPE_F16:
            rope_delta_kernel<__half><<<blocks, warps * 32, 0, s>>>((const __half*)p.o, (const __half*)p.d_o, p.delta, rows, p.D, row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N)); count_launch();
            break;
        default: return COROPE_ERR_BAD_DTYPE;
    }
    return (int)cudaGetLastError();
}

int launch_rope_prerotate(const void* x, const Strides& st, void* out_f16, const uint32_t* packed, int B, int H, int N, float scale, int dtype,
                          cudaStream_t s) {
    const size_t rows = (size_t)B * H * N;
    const unsigned grid = (unsigned)((rows * 8 + 255) / 256);
    if (dtype == COROPE_DTYPE_BF16)
        rope_prerotate_d128_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (__half*)out_f16, packed, rows, N, scale, row_addr(st, H, N));
    else
        rope_prerotate_d128_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, (__half*)out_f16, packed, rows, N, scale, row_addr(st, H, N));
    count_launch();
    return (int)cudaGetLastError();
}

int launch_rope_bwd_prepass(const RopeParams& p, int dtype, cudaStream_t s) {
    const size_t rows = (size_t)p.B * p.H * p.N;
    const unsigned grid = (unsigned)((rows * 16 + 255) / 256);
    const float scale = p.sm_scale * kLog2e;
    if (dtype == COROPE_DTYPE_BF16)
        rope_bwd_prepass_d128_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)p.q, (const __nv_bfloat16*)p.o, (const __nv_bfloat16*)p.d_o,
                                                                        p.packed_tab, (__half*)const_cast<void*>(p.q_rot), p.delta, p.dq_acc, rows, p.N, scale, row_addr(p.sq, p.H, p.N), row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N));
    else
        rope_bwd_prepass_d128_kernel<__half><<<grid, 256, 0, s>>>((const __half*)p.q, (const __half*)p.o, (const __half*)p.d_o, p.packed_tab,
                                                                 (__half*)const_cast<void*>(p.q_rot), p.delta, p.dq_acc, rows, p.N, scale, row_addr(p.sq, p.H, p.N), row_addr(p.so, p.H, p.N), row_addr(p.sdo, p.H, p.N));
    count_launch();
    return (int)cudaGetLastError();
}

int launch_pack_tables(const float* cos, const float* sin, int64_t stride, uint32_t* packed, int N, int half_d, cudaStream_t s, int half_src) {
    size_t n = (size_t)N * half_d;
    pack_tables_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(cos, sin, stride, packed, N, half_d, half_src < 0 ? half_d : half_src);
    count_launch();
    return (int)cudaGetLastError();
}

int launch_synth_tables(const float* inv_freq, float* cos_out, float* sin_out, int N, int half_d, cudaStream_t s) {
    size_t n = (size_t)N * half_d;
    synth_tables_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(inv_freq, cos_out, sin_out, N, half_d);
    count_launch();
    return (int)cudaGetLastError();
}

// n <= 4 tensors [B, H_i, N, 64] <-> their zero-padded [B, H_i, N, 128] copies in one launch (unpad: the other direction)
int launch_pad_d64_many(int n, const PadSpec* specs, int B, int N, bool unpad, int dtype, cudaStream_t s) {
    PadJobs jobs{};
    size_t max_rows = 0;
    for (int i = 0; i < n; ++i) {
        const size_t rows = (size_t)B * specs[i].H * N;
        jobs.j[i].src = unpad ? specs[i].padded : specs[i].tensor;
        jobs.j[i].dst = unpad ? const_cast<void*>(specs[i].tensor) : specs[i].padded;
        jobs.j[i].rows = rows;
        jobs.j[i].rope_layout = specs[i].rope_layout;
        jobs.j[i].addr = row_addr(specs[i].strides, specs[i].H, N);
        max_rows = rows > max_rows ? rows : max_rows;
    }
    const dim3 grid((unsigned)((max_rows * (unpad ? 8 : 16) + 255) / 256), (unsigned)n);
    if (dtype == COROPE_DTYPE_BF16) {
        if (unpad) unpad_d64_many_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(jobs);
        else pad_d64_many_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(jobs);
    } else {
        if (unpad) unpad_d64_many_kernel<__half><<<grid, 256, 0, s>>>(jobs);
        else pad_d64_many_kernel<__half><<<grid, 256, 0, s>>>(jobs);
    }
    count_launch();
    return (int)cudaGetLastError();
}

int launch_unpad_d64(const void* xp, void* out, const Strides& st, int B, int H, int N, int rope_layout, int dtype, cudaStream_t s) {
    const size_t rows = (size_t)B * H * N;
    const unsigned grid = (unsigned)((rows * 8 + 255) / 256);
    if (dtype == COROPE_DTYPE_BF16)
        unpad_d64_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)xp, (__nv_bfloat16*)out, rows, rope_layout, row_addr(st, H, N));
    else
        unpad_d64_kernel<__half><<<grid, 256, 0, s>>>((const __half*)xp, (__half*)out, rows, rope_layout, row_addr(st, H, N));
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace corope
