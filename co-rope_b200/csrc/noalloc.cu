// corope_rope_attn_fwd_noalloc: the fused-RoPE attention forward for callers that cannot provide scratch
// memory.  The tensor-core forward needs one piece of scratch, the packed (cos, sin) table built by
// pack_tables_kernel; here it lives in a fixed array inside the library image instead of a caller workspace.
#include <mutex>

#include "common.cuh"

namespace corope {
namespace {

// Scratch: packed (cos, sin) table, one 32-bit entry per (position, d < D/2).  2 MiB per GPU that loads the
// library, held until the process exits.  Enough for N * D/2 <= 524288, i.e. N <= 8192 at D = 128.
constexpr size_t kNoAllocMaxEntries = (size_t)8192 * 64;
static __device__ __align__(256) uint32_t g_noalloc_table[kNoAllocMaxEntries + 64];   // + the forward kernel's work counter behind the table

// In host code `g_noalloc_table` is only a handle for the runtime, not an address a kernel can use; the device
// address is looked up once per device (with that device current) and cached here.
constexpr int kMaxDevices = 64;
uint32_t* g_table_addr[kMaxDevices] = {};
std::mutex g_table_mutex;

int scratch_on_current_device(uint32_t** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return COROPE_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_table_mutex);
    if (g_table_addr[dev] == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_noalloc_table);
        if (e != cudaSuccess) return (int)e;
        if (addr == nullptr) return COROPE_ERR_NO_DEVICE;
        g_table_addr[dev] = static_cast<uint32_t*>(addr);
    }
    *out = g_table_addr[dev];
    return COROPE_OK;
}

}  // namespace
}  // namespace corope

using namespace corope;

extern "C" int corope_rope_attn_fwd_noalloc(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                                            int64_t table_row_stride, void* o, float* lse2, int B, int H, int N, int D, int dtype,
                                            int causal, float sm_scale, int* status_word, void* stream) {
    if (!q || !k || !v || !cos || !sin || !o || !lse2) return COROPE_ERR_NULL_POINTER;
    if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return COROPE_ERR_BAD_SHAPE;
    if (D != 32 && D != 64 && D != 128) return COROPE_ERR_BAD_HEAD_DIM;
    if (dtype != COROPE_DTYPE_F32 && dtype != COROPE_DTYPE_BF16 && dtype != COROPE_DTYPE_F16) return COROPE_ERR_BAD_DTYPE;
    if ((size_t)B * H > 65535u * 32u) return COROPE_ERR_TOO_LARGE;
    if ((size_t)N * (size_t)(D / 2) > kNoAllocMaxEntries) return COROPE_ERR_TOO_LARGE;  // table would not fit the fixed array

    cudaStream_t s = (cudaStream_t)stream;
    RopeParams p{};
    p.q = q; p.k = k; p.v = v; p.out_o = o; p.lse2 = lse2;
    p.cos = cos; p.sin = sin; p.table_stride = table_row_stride;
    p.B = B; p.H = H; p.Hkv = H; p.N = N; p.D = D; p.causal = causal ? 1 : 0; p.sm_scale = sm_scale; p.status = status_word;
    p.sq = p.sk = p.sv = p.so = contiguous_strides(H, N, D);
    // the kernel-selection policy of the diagnostics header applies here too: 1 = general kernels; 0 and 2 both mean the
    // tensor-core kernel with its in-kernel K rotation (this entry point has no room for a rotated copy)
    if (kernel_policy() != 1 && rope_fwd_tc_supported(B, H, N, D, dtype, causal)) {
        uint32_t* table = nullptr;
        if (int e = scratch_on_current_device(&table)) return e;
        // the table is rebuilt in full for rows [0, N) on every call, so stale contents of an earlier call are never read
        if (int e = launch_pack_tables(cos, sin, table_row_stride, table, N, D / 2, s)) return e;
        p.packed_tab = table;
        p.sched_counter = reinterpret_cast<int*>(table + (size_t)N * (D / 2));
        note_kernel_family(COROPE_OP_ROPE_FWD, 1);
        return launch_rope_fwd_tc(p, dtype, s);
    }
    note_kernel_family(COROPE_OP_ROPE_FWD, 0);
    return launch_rope_fwd_general(p, dtype, s);  // the general kernels use no scratch at all
}
