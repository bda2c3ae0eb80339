// Helpers shared by the tensor-core (mma.sync) Co-RoPE GQA kernels: operand layouts, MMA / ldmatrix / cp.async wrappers
// and the pre-pass that writes the fp16 operand copies of K and V.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace corope {
namespace gqa_mma {

constexpr int kRows = 8;            // query rows (= warps) per CTA
constexpr int kThreads = kRows * 32;
constexpr int kKT = 64;             // keys per tile
constexpr int kD = 128;
constexpr int kPairs = kD / 2;
constexpr int kKRow = 80;           // u32 per K row: 64 pairs + 16 of padding (rows of a quarter-warp land in distinct bank groups)
constexpr int kWStride = 20;        // floats between the frequency blocks of the 4 lane classes (16 + 4: distinct banks)
constexpr int kVRowBytes = 272;     // bytes per V row: 128 halves + 16 bytes of padding (conflict-free ldmatrix)

// Position (u32 index within a row) of pair p.  MMA k-step t = p / 8 covers pairs 8t..8t+7; lane c = (p % 8) % 4 holds
// pair 8t + c in b0 / a0 and pair 8t + c + 4 in b1 / a2.  The 16 pairs of lane c are stored as four 16-byte chunks
// (chunk index 4s + c for s = t / 2), each holding (t = 2s: b0, b1; t = 2s + 1: b0, b1).
__device__ __forceinline__ int perm_slot(int p) {
    const int t = p >> 3, r = p & 7, c = r & 3, u = r >> 2, s = t >> 1, tt = t & 1;
    return ((4 * s + c) << 2) + tt * 2 + u;
}
// the pair held in slot (s, e) of lane c: e = 0..3 as stored in the 16-byte chunk
__device__ __forceinline__ int lane_pair(int c, int s, int e) { return 8 * (2 * s + (e >> 1)) + c + 4 * (e & 1); }

__device__ __forceinline__ void mma16816(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1, float c0, float c1) {
    float x2, x3;   // rows 8..15 of the A operand are zero: their results are discarded
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d0), "=f"(d1), "=f"(x2), "=f"(x3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(0.f), "f"(0.f));
    (void)x2;
    (void)x3;
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(smem_u32(smem_row)));
}

template <bool DIRECT>
__device__ __forceinline__ void sincos_fast(float x, float* s, float* c) {
    if (DIRECT) {
        // phases up to a few thousand radians (N <= 8192): the hardware approximations alone
        __sincosf(x, s, c);
    } else {
        // two-constant reduction to [-pi, pi], then the hardware approximations
        float kf = rintf(x * 0.15915494309189535f);
        float r = fmaf(kf, -6.28318548202514648f, x);
        r = fmaf(kf, 1.7484555e-7f, r);
        __sincosf(r, s, c);
    }
}

// m16n8k16 with all four A registers, both B registers and all four accumulators in use
__device__ __forceinline__ void mma16816_full(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// transpose of an 8x8 matrix of 16-bit values held one register per lane (row = lane / 4, columns 2 (lane % 4), +1)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// One (k1, k2) pair of a key as packed fp16, rotated by `angle`: (K'1, K'2) = (k1 cos + k2 sin, k2 cos - k1 sin), in packed
// fp16 arithmetic: k1 (c, -s) + k2 (s, c), the broadcasts of k1 / k2 being operand selectors of the packed instructions.
template <bool DIRECT>
__device__ __forceinline__ uint32_t rotate_pair(uint32_t kpair, float angle) {
    float sn, cs;
    sincos_fast<DIRECT>(angle, &sn, &cs);
    const __half2 kk = *reinterpret_cast<const __half2*>(&kpair);
    const __half2 rr = __hfma2(__low2half2(kk), __floats2half2_rn(cs, -sn), __hmul2(__high2half2(kk), __floats2half2_rn(sn, cs)));
    return *reinterpret_cast<const uint32_t*>(&rr);
}

// the same, and the packed (cos, sin) of the angle for the inverse rotation of the backward
template <bool DIRECT>
__device__ __forceinline__ uint32_t rotate_pair(uint32_t kpair, float angle, uint32_t* cos_sin) {
    float sn, cs;
    sincos_fast<DIRECT>(angle, &sn, &cs);
    const __half2 kk = *reinterpret_cast<const __half2*>(&kpair);
    const __half2 rr = __hfma2(__low2half2(kk), __floats2half2_rn(cs, -sn), __hmul2(__high2half2(kk), __floats2half2_rn(sn, cs)));
    *cos_sin = pack_half2(cs, sn);
    return *reinterpret_cast<const uint32_t*>(&rr);
}
// m16n8k8: 16 rows x 8 columns from a K dimension of 8, fresh accumulators
__device__ __forceinline__ void mma1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.f));
}

template <typename T>
__device__ __forceinline__ uint32_t to_half2(T a, T b) {
    return pack_half2(Elem<T>::to_f32(a), Elem<T>::to_f32(b));
}

// Pre-pass: K -> fp16 (k1, k2) pairs in the permuted row order (64 u32 per key), V -> fp16 row-major.  The main kernel
// then brings tiles in with 16-byte asynchronous copies, two tiles in flight, instead of converting and scattering
// every tile once per 8 query rows.
template <typename T>
__global__ void __launch_bounds__(256) gqa_pack_kv_kernel(const T* __restrict__ K, const T* __restrict__ V, uint32_t* __restrict__ kp,
                                                          __half* __restrict__ vh, size_t rows, RowAddr ak, RowAddr av) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // rows * 16: 8 K chunks + 8 V double-chunks
    if (idx >= rows * 16) return;
    const size_t r = idx >> 4;
    const int ch = (int)(idx & 15);
    if (ch < 8) {
        const T* src = K + flat_row_offset(ak, r) + ch * 8;
        const uint4 x1 = *reinterpret_cast<const uint4*>(src);
        const uint4 x2 = *reinterpret_cast<const uint4*>(src + kPairs);
        const uint32_t a[4] = {x1.x, x1.y, x1.z, x1.w}, bb[4] = {x2.x, x2.y, x2.z, x2.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f1 = unpack2<T>(a[e]), f2 = unpack2<T>(bb[e]);
            kp[r * kPairs + perm_slot(ch * 8 + 2 * e)] = pack_half2_sat(f1.x, f2.x);
            kp[r * kPairs + perm_slot(ch * 8 + 2 * e + 1)] = pack_half2_sat(f1.y, f2.y);
        }
    } else {
        const int c2 = ch - 8;   // 16 elements of V
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint4 x = *reinterpret_cast<const uint4*>(V + flat_row_offset(av, r) + c2 * 16 + u * 8);
            if (Elem<T>::kDtype == COROPE_DTYPE_BF16) {
                uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf162(w4[e]);
                    w4[e] = pack_half2_sat(f.x, f.y);
                }
                x = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
            *reinterpret_cast<uint4*>(vh + r * kD + c2 * 16 + u * 8) = x;
        }
    }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }


}  // namespace gqa_mma
}  // namespace corope
