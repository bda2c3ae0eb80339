// extern "C" entry points of libcorope_b200.so: argument validation, workspace carving, kernel selection.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace corope {
namespace {

std::atomic<int> g_policy{0};
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_last_family[4] = {{0}, {0}, {0}, {0}};

constexpr size_t kAlign = 256;

bool head_dim_ok(int D) { return D == 32 || D == 64 || D == 128; }

struct RopeWorkspace {
    size_t packed_tab, synth_cos, synth_sin, rot, delta, dq_acc, pad[5], total;
};

// 16-bit problems with D = 64 and N % 128 == 0 run zero-padded to D = 128 on the tensor-core kernels (half of the MMA work
// is on zeros, which still is an order of magnitude faster than the CUDA-core kernels); the workspace then also holds the
// padded copies.
bool rope_d64_padded(int N, int D, int dtype) { return D == 64 && dtype != COROPE_DTYPE_F32 && N % 128 == 0; }

// Hq query heads, Hkv K / V heads (equal for the fused-RoPE ops).  `synth`: room for fp32 cos / sin tables [N, D/2] that the
// entry points taking frequencies instead of tables fill in.
RopeWorkspace rope_workspace_layout(bool bwd, int B, int Hq, int Hkv, int N, int D, int dtype, bool synth) {
    RopeWorkspace w{};
    const bool padded = rope_d64_padded(N, D, dtype);
    const int Dk = padded ? 128 : D;                 // head dimension the kernels see
    const bool tc = dtype != COROPE_DTYPE_F32 && Dk == 128;
    const size_t q_elems = (size_t)B * Hq * N * Dk, kv_elems = (size_t)B * Hkv * N * Dk;
    size_t off = 0;
    w.packed_tab = off;
    off += align_up((size_t)N * (Dk / 2) * sizeof(uint32_t) + 64, kAlign);   // + the work counter behind the table
    if (synth) {
        w.synth_cos = off;
        off += align_up((size_t)N * (D / 2) * sizeof(float), kAlign);
        w.synth_sin = off;
        off += align_up((size_t)N * (D / 2) * sizeof(float), kAlign);
    }
    w.rot = off;   // tensor-core kernels: fp16 copy of the rotated K (forward) / rotated and scaled Q (backward)
    if (tc) off += align_up((bwd ? q_elems : kv_elems) * 2, kAlign);
    if (bwd) {
        w.delta = off;
        off += align_up((size_t)B * Hq * N * sizeof(float), kAlign);
        w.dq_acc = off;
        if (tc) off += align_up(q_elems * sizeof(float), kAlign);
    }
    if (padded) {
        // forward: q, v, o (k before its rotation shares o's buffer: needs the larger of the two); backward: k, v, dO / dq,
        // dk (q before its rotation shares dk's buffer), dv
        const size_t fwd_sizes[3] = {q_elems, kv_elems, q_elems};
        const size_t bwd_sizes[5] = {kv_elems, kv_elems, q_elems, q_elems, kv_elems};
        for (int i = 0; i < (bwd ? 5 : 3); ++i) {
            w.pad[i] = off;
            off += align_up((bwd ? bwd_sizes[i] : fwd_sizes[i]) * 2, kAlign);
        }
    }
    w.total = off < kAlign ? kAlign : off;
    return w;
}

struct GqaWorkspace {
    size_t delta, dk_acc, dv_acc, k_pairs, v_half, total;
};

GqaWorkspace gqa_workspace_layout(bool bwd, int B, int Hq, int Hkv, int N, int D, int dtype) {
    GqaWorkspace w{};
    size_t off = 0;
    if (gqa_fwd_mma_supported(N, D, dtype)) {   // fp16 operand copies of K (pair order) and V for the tensor-core kernels
        w.k_pairs = off;
        off += align_up((size_t)B * Hkv * N * D * 2, kAlign);
        w.v_half = off;
        off += align_up((size_t)B * Hkv * N * D * 2, kAlign);
    }
    if (bwd) {
        w.delta = off;
        off += align_up((size_t)B * Hq * N * sizeof(float), kAlign);
        w.dk_acc = off;
        off += align_up((size_t)B * Hkv * N * D * sizeof(float), kAlign);
        w.dv_acc = off;
        off += align_up((size_t)B * Hkv * N * D * sizeof(float), kAlign);
    }
    w.total = off < kAlign ? kAlign : off;
    return w;
}

int check_common(int B, int H, int N, int D, int dtype) {
    if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return COROPE_ERR_BAD_SHAPE;
    if (!head_dim_ok(D)) return COROPE_ERR_BAD_HEAD_DIM;
    if (dtype != COROPE_DTYPE_F32 && dtype != COROPE_DTYPE_BF16 && dtype != COROPE_DTYPE_F16) return COROPE_ERR_BAD_DTYPE;
    if ((size_t)B * H > 65535u * 32u) return COROPE_ERR_TOO_LARGE;
    if ((size_t)B * H * N >= (1ull << 31)) return COROPE_ERR_TOO_LARGE;   // row indices are 32-bit in the kernels
    return COROPE_OK;
}

int check_workspace(const void* ws, size_t have, size_t need) {
    if (!ws || have < need || ((uintptr_t)ws % kAlign) != 0) return COROPE_ERR_WORKSPACE;
    return COROPE_OK;
}

}  // namespace

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n); }
void note_kernel_family(int op, int family) {
    if (op >= 0 && op < 4) g_last_family[op] = family;
}
int kernel_policy() { return g_policy.load(); }

}  // namespace corope

using namespace corope;

extern "C" {

int corope_abi_version(void) { return 1; }

// ---- host mirror of the status word -----------------------------------------------------------------------------------
// A side stream per device copies the word to a pinned host location whenever the caller's stream reaches the point of the
// call; the caller's stream is not delayed (it only records an event) and the host never synchronises.
namespace {
struct MirrorState {
    cudaStream_t side = nullptr;
    cudaEvent_t reached = nullptr;
};
MirrorState g_mirror[64];
std::mutex g_mirror_mutex;
int mirror_state(MirrorState** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return COROPE_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_mirror_mutex);
    MirrorState& m = g_mirror[dev];
    if (!m.side) {
        if ((e = cudaStreamCreateWithFlags(&m.side, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if ((e = cudaEventCreateWithFlags(&m.reached, cudaEventDisableTiming)) != cudaSuccess) return (int)e;
    }
    *out = &m;
    return COROPE_OK;
}
}  // namespace

int corope_status_mirror_refresh(const int* status_word, int* host_mirror, void* stream) {
    if (!status_word || !host_mirror) return COROPE_ERR_NULL_POINTER;
    MirrorState* m = nullptr;
    if (int e = mirror_state(&m)) return e;
    cudaError_t e = cudaEventRecord(m->reached, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(m->side, m->reached, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_mirror, status_word, sizeof(int), cudaMemcpyDeviceToHost, m->side);
    return (int)e;
}

int corope_status_mirror_clear(int* status_word, int* host_mirror, void* stream) {
    if (!status_word || !host_mirror) return COROPE_ERR_NULL_POINTER;
    MirrorState* m = nullptr;
    if (int e = mirror_state(&m)) return e;
    cudaError_t e = cudaStreamSynchronize(m->side);   // no copy of the old value may land after the mirror is reset
    if (e == cudaSuccess) e = cudaMemsetAsync(status_word, 0, sizeof(int), (cudaStream_t)stream);
    *host_mirror = 0;
    return (int)e;
}

const char* corope_status_string(int status) {
    switch (status) {
        case COROPE_OK: return "ok";
        case COROPE_ERR_NULL_POINTER: return "null pointer argument";
        case COROPE_ERR_BAD_SHAPE: return "non-positive tensor extent";
        case COROPE_ERR_BAD_HEAD_DIM: return "unsupported head dimension (supported: 32, 64, 128)";
        case COROPE_ERR_BAD_DTYPE: return "unsupported element type";
        case COROPE_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case COROPE_ERR_BAD_GROUP: return "query heads must be a multiple of KV heads with group size <= 8";
        case COROPE_ERR_SEQ_NOT_128: return "sequence length must be a multiple of 128";
        case COROPE_ERR_TENSOR_MAP: return "TMA tensor map could not be encoded";
        case COROPE_ERR_NO_DEVICE: return "no usable CUDA device or driver entry point";
        case COROPE_ERR_TOO_LARGE: return "size beyond the supported maximum";
        case COROPE_ERR_BAD_STRIDE: return "row stride smaller than the head dimension, or a negative stride";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

size_t corope_workspace_bytes(int op, int B, int Hq, int Hkv, int N, int D, int dtype) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || D <= 0) return 0;
    switch (op) {
        case COROPE_OP_ROPE_FWD: return rope_workspace_layout(false, B, Hq, Hq, N, D, dtype, false).total;
        case COROPE_OP_ROPE_BWD: return rope_workspace_layout(true, B, Hq, Hq, N, D, dtype, false).total;
        case COROPE_OP_ROPE_FWD_FREQS: return rope_workspace_layout(false, B, Hq, Hq, N, D, dtype, true).total;
        case COROPE_OP_ROPE_BWD_FREQS: return rope_workspace_layout(true, B, Hq, Hq, N, D, dtype, true).total;
        case COROPE_OP_FLASH_FWD: return Hq % Hkv ? 0 : rope_workspace_layout(false, B, Hq, Hkv, N, D, dtype, false).total;
        case COROPE_OP_FLASH_BWD: return Hq % Hkv ? 0 : rope_workspace_layout(true, B, Hq, Hkv, N, D, dtype, false).total;
        case COROPE_OP_GQA_FWD: return gqa_workspace_layout(false, B, Hq, Hkv, N, D, dtype).total;
        case COROPE_OP_GQA_BWD: return gqa_workspace_layout(true, B, Hq, Hkv, N, D, dtype).total;
        default: return 0;
    }
}

uint64_t corope_launch_count(void) { return (uint64_t)g_launches.load(); }

int corope_set_kernel_policy(int policy) { return g_policy.exchange(policy); }

int corope_last_kernel_family(int op) { return (op >= 0 && op < 4) ? g_last_family[op].load() : -1; }

}  // extern "C"

namespace {

// Where the rotation comes from: caller tables (cos / sin + row stride), per-pair frequencies (tables are synthesized into
// the workspace first), or nothing at all (plain attention).
struct Rotation {
    const float* cos = nullptr;
    const float* sin = nullptr;
    int64_t stride = 0;
    const float* inv_freq = nullptr;
    bool none = false;
};

// Fills the kernels' stride fields from the ABI struct (null = contiguous [B, H, N, D]).
void set_strides(RopeParams& p, const corope_strides_t* st, int Hq, int Hkv, int N, int D) {
    auto conv = [](const int64_t (&a)[3]) {
        Strides r;
        r.b = a[0]; r.h = a[1]; r.n = a[2];
        return r;
    };
    const Strides cq = contiguous_strides(Hq, N, D), ckv = contiguous_strides(Hkv, N, D);
    p.sq = st ? conv(st->q) : cq;
    p.sk = st ? conv(st->k) : ckv;
    p.sv = st ? conv(st->v) : ckv;
    p.so = st ? conv(st->o) : cq;
    p.sdo = st ? conv(st->d_o) : cq;
    p.sdq = st ? conv(st->dq) : cq;
    p.sdk = st ? conv(st->dk) : ckv;
    p.sdv = st ? conv(st->dv) : ckv;
}
void set_gqa_strides(GqaParams& p, const corope_strides_t* st) {
    auto conv = [](const int64_t (&a)[3]) {
        Strides r;
        r.b = a[0]; r.h = a[1]; r.n = a[2];
        return r;
    };
    const Strides cq = contiguous_strides(p.Hq, p.N, p.D), ckv = contiguous_strides(p.Hkv, p.N, p.D);
    p.sq = st ? conv(st->q) : cq;
    p.sk = st ? conv(st->k) : ckv;
    p.sv = st ? conv(st->v) : ckv;
    p.so = st ? conv(st->o) : cq;
    p.sdo = st ? conv(st->d_o) : cq;
    p.sdq = st ? conv(st->dq) : cq;
    p.sdk = st ? conv(st->dk) : ckv;
    p.sdv = st ? conv(st->dv) : ckv;
}
// The tensor-core paths move rows with TMA and 16-byte vector accesses: base pointers and all strides must be multiples of 16 bytes.
bool vec_ok(const void* ptr, const Strides& st) {
    return ((uintptr_t)ptr % 16) == 0 && st.b % 8 == 0 && st.h % 8 == 0 && st.n % 8 == 0 && st.n > 0;
}
bool strides_positive(const Strides& st, int D) { return st.n >= D && st.b >= 0 && st.h >= 0; }

// ops whose kernel family is recorded: the fused-RoPE pair also stands for its variants
constexpr int kFamFwd = COROPE_OP_ROPE_FWD, kFamBwd = COROPE_OP_ROPE_BWD;

int rope_fwd_impl(const void* q, const void* k, const void* v, Rotation rot, void* o, float* lse2, int B, int Hq, int Hkv, int N, int D,
                  int dtype, int causal, float sm_scale, void* workspace, size_t workspace_bytes, int* status_word, void* stream,
                  const corope_strides_t* strides = nullptr) {
    if (!q || !k || !v || !o || !lse2) return COROPE_ERR_NULL_POINTER;
    if (!rot.none && !rot.inv_freq && (!rot.cos || !rot.sin)) return COROPE_ERR_NULL_POINTER;
    if (int e = check_common(B, Hq, N, D, dtype)) return e;
    if (Hkv <= 0 || Hq % Hkv != 0) return COROPE_ERR_BAD_GROUP;
    RopeWorkspace w = rope_workspace_layout(false, B, Hq, Hkv, N, D, dtype, rot.inv_freq != nullptr);
    if (int e = check_workspace(workspace, workspace_bytes, w.total)) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (rot.inv_freq) {
        float* c = reinterpret_cast<float*>((char*)workspace + w.synth_cos);
        float* sn = reinterpret_cast<float*>((char*)workspace + w.synth_sin);
        if (int e = launch_synth_tables(rot.inv_freq, c, sn, N, D / 2, s)) return e;
        rot.cos = c; rot.sin = sn; rot.stride = D / 2;
    }
    RopeParams p{};
    p.q = q; p.k = k; p.v = v; p.out_o = o; p.lse2 = lse2;
    p.cos = rot.none ? nullptr : rot.cos; p.sin = rot.none ? nullptr : rot.sin; p.table_stride = rot.stride;
    p.B = B; p.H = Hq; p.Hkv = Hkv; p.no_rope = rot.none ? 1 : 0;
    p.N = N; p.D = D; p.causal = causal ? 1 : 0; p.sm_scale = sm_scale; p.status = status_word;
    set_strides(p, strides, Hq, Hkv, N, D);
    if (!strides_positive(p.sq, D) || !strides_positive(p.sk, D) || !strides_positive(p.sv, D) || !strides_positive(p.so, D)) return COROPE_ERR_BAD_STRIDE;
    // rows are moved with TMA / 16-byte vectors on the tensor-core paths; otherwise the CUDA-core kernels take over
    const bool vec = vec_ok(q, p.sq) && vec_ok(k, p.sk) && vec_ok(v, p.sv) && vec_ok(o, p.so);
    const int policy = vec ? g_policy.load() : 1;
    if (policy == 0 && rope_d64_padded(N, D, dtype)) {
        // D = 64: zero-padded copies of q, k, v in the layout that keeps the rotation pairs together, the D = 128 kernels, o back
        uint32_t* tab = reinterpret_cast<uint32_t*>((char*)workspace + w.packed_tab);
        void* k_rot = (char*)workspace + w.rot;
        void* qp = (char*)workspace + w.pad[0];
        void* vp = (char*)workspace + w.pad[1];
        void* op = (char*)workspace + w.pad[2];   // first the padded k (until it is rotated), then the padded output
        if (int e = launch_pack_tables(p.cos, p.sin, p.table_stride, tab, N, 64, s, 32)) return e;
        const PadSpec in3[3] = {{q, qp, p.sq, Hq, 1}, {k, op, p.sk, Hkv, 1}, {v, vp, p.sv, Hkv, 0}};
        if (int e = launch_pad_d64_many(3, in3, B, N, false, dtype, s)) return e;
        if (int e = launch_rope_prerotate(op, contiguous_strides(Hkv, N, 128), k_rot, tab, B, Hkv, N, 1.0f, dtype, s)) return e;
        const Strides so_caller = p.so;
        p.q = qp; p.k = op; p.v = vp; p.out_o = op; p.D = 128;
        set_strides(p, nullptr, Hq, Hkv, N, 128);   // the padded copies are contiguous
        p.packed_tab = tab;
        p.sched_counter = reinterpret_cast<int*>(tab + (size_t)N * 64);
        p.k_rot = k_rot;
        g_last_family[kFamFwd] = 1;
        if (int e = launch_rope_fwd_tc(p, dtype, s)) return e;
        return launch_unpad_d64(op, o, so_caller, B, Hq, N, 0, dtype, s);
    }
    if (policy != 1 && rope_fwd_tc_supported(B, Hq, N, D, dtype, causal)) {
        uint32_t* tab = reinterpret_cast<uint32_t*>((char*)workspace + w.packed_tab);
        if (int e = launch_pack_tables(p.cos, p.sin, p.table_stride, tab, N, D / 2, s)) return e;
        p.packed_tab = tab;
        p.sched_counter = reinterpret_cast<int*>(tab + (size_t)N * (D / 2));
        // policy 2: every K tile is rotated in shared memory by the main kernel, nothing rotated is written to HBM (for plain
        // attention the "rotation" by the identity table is what brings K to fp16, the format Q is written in)
        if (policy == 0) {
            void* k_rot = (char*)workspace + w.rot;
            if (int e = launch_rope_prerotate(k, p.sk, k_rot, tab, B, Hkv, N, 1.0f, dtype, s)) return e;
            p.k_rot = k_rot;
        }
        g_last_family[kFamFwd] = 1;
        return launch_rope_fwd_tc(p, dtype, s);
    }
    g_last_family[kFamFwd] = 0;
    return launch_rope_fwd_general(p, dtype, s);
}

int rope_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2, Rotation rot, void* dq,
                  void* dk, void* dv, int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale, void* workspace,
                  size_t workspace_bytes, int* status_word, void* stream, const corope_strides_t* strides = nullptr) {
    if (!q || !k || !v || !o || !d_o || !lse2 || !dq || !dk || !dv) return COROPE_ERR_NULL_POINTER;
    if (!rot.none && !rot.inv_freq && (!rot.cos || !rot.sin)) return COROPE_ERR_NULL_POINTER;
    if (int e = check_common(B, Hq, N, D, dtype)) return e;
    if (Hkv <= 0 || Hq % Hkv != 0) return COROPE_ERR_BAD_GROUP;
    RopeWorkspace w = rope_workspace_layout(true, B, Hq, Hkv, N, D, dtype, rot.inv_freq != nullptr);
    if (int e = check_workspace(workspace, workspace_bytes, w.total)) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (rot.inv_freq) {
        float* c = reinterpret_cast<float*>((char*)workspace + w.synth_cos);
        float* sn = reinterpret_cast<float*>((char*)workspace + w.synth_sin);
        if (int e = launch_synth_tables(rot.inv_freq, c, sn, N, D / 2, s)) return e;
        rot.cos = c; rot.sin = sn; rot.stride = D / 2;
    }
    RopeParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.d_o = d_o; p.dq = dq; p.dk = dk; p.dv = dv;
    p.lse2 = const_cast<float*>(lse2);
    p.delta = reinterpret_cast<float*>((char*)workspace + w.delta);
    p.cos = rot.none ? nullptr : rot.cos; p.sin = rot.none ? nullptr : rot.sin; p.table_stride = rot.stride;
    p.B = B; p.H = Hq; p.Hkv = Hkv; p.no_rope = rot.none ? 1 : 0;
    p.N = N; p.D = D; p.causal = causal ? 1 : 0; p.sm_scale = sm_scale; p.status = status_word;
    set_strides(p, strides, Hq, Hkv, N, D);
    for (const Strides* st : {&p.sq, &p.sk, &p.sv, &p.so, &p.sdo, &p.sdq, &p.sdk, &p.sdv})
        if (!strides_positive(*st, D)) return COROPE_ERR_BAD_STRIDE;
    const bool vec = vec_ok(q, p.sq) && vec_ok(k, p.sk) && vec_ok(v, p.sv) && vec_ok(o, p.so) && vec_ok(d_o, p.sdo) && vec_ok(dq, p.sdq) &&
                     vec_ok(dk, p.sdk) && vec_ok(dv, p.sdv);
    const int policy = vec ? g_policy.load() : 1;
    const bool tc_direct = policy != 1 && !(policy == 0 && rope_d64_padded(N, D, dtype)) && rope_bwd_tc_supported(B, Hq, N, D, dtype, causal);
    if (!(tc_direct && policy == 0))   // the tensor-core path at D = 128 computes delta in its fused pre-pass
        if (int e = launch_rope_delta(p, dtype, s)) return e;
    if (policy == 0 && rope_d64_padded(N, D, dtype)) {
        uint32_t* tab = reinterpret_cast<uint32_t*>((char*)workspace + w.packed_tab);
        void* q_rot = (char*)workspace + w.rot;
        void* kp = (char*)workspace + w.pad[0];
        void* vp = (char*)workspace + w.pad[1];
        void* dop = (char*)workspace + w.pad[2];   // padded dO; after the main kernel the padded dq (the finalize kernel writes it)
        void* dkp = (char*)workspace + w.pad[3];   // first the padded q (until it is rotated), then the padded dk
        void* dvp = (char*)workspace + w.pad[4];
        if (int e = launch_pack_tables(p.cos, p.sin, p.table_stride, tab, N, 64, s, 32)) return e;
        const PadSpec in4[4] = {{q, dkp, p.sq, Hq, 1}, {k, kp, p.sk, Hkv, 1}, {v, vp, p.sv, Hkv, 0}, {d_o, dop, p.sdo, Hq, 0}};
        if (int e = launch_pad_d64_many(4, in4, B, N, false, dtype, s)) return e;
        if (int e = launch_rope_prerotate(dkp, contiguous_strides(Hq, N, 128), q_rot, tab, B, Hq, N, sm_scale * kLog2e, dtype, s)) return e;
        const Strides sdq_caller = p.sdq, sdk_caller = p.sdk, sdv_caller = p.sdv;
        p.q = dkp; p.k = kp; p.v = vp; p.d_o = dop; p.dq = dop; p.dk = dkp; p.dv = dvp; p.D = 128;
        set_strides(p, nullptr, Hq, Hkv, N, 128);   // the padded copies are contiguous
        p.packed_tab = tab;
        p.sched_counter = reinterpret_cast<int*>(tab + (size_t)N * 64);   // zeroed by the table pack
        p.dq_acc = reinterpret_cast<float*>((char*)workspace + w.dq_acc);
        p.q_rot = q_rot;
        g_last_family[kFamBwd] = 1;
        if (int e = launch_rope_bwd_tc(p, dtype, s)) return e;
        const PadSpec out3[3] = {{dq, dop, sdq_caller, Hq, 1}, {dk, dkp, sdk_caller, Hkv, 1}, {dv, dvp, sdv_caller, Hkv, 0}};
        return launch_pad_d64_many(3, out3, B, N, true, dtype, s);
    }
    if (tc_direct) {
        uint32_t* tab = reinterpret_cast<uint32_t*>((char*)workspace + w.packed_tab);
        if (int e = launch_pack_tables(p.cos, p.sin, p.table_stride, tab, N, D / 2, s)) return e;
        p.packed_tab = tab;
        p.sched_counter = reinterpret_cast<int*>(tab + (size_t)N * (D / 2));   // zeroed by the table pack
        p.dq_acc = reinterpret_cast<float*>((char*)workspace + w.dq_acc);
        if (policy == 0) {   // policy 2: every Q tile is rotated in shared memory by the main kernel, nothing rotated is written to HBM
            p.q_rot = (char*)workspace + w.rot;
            if (int e = launch_rope_bwd_prepass(p, dtype, s)) return e;   // delta, rotated Q, cleared dQ accumulator
            p.dq_acc_zeroed = 1;
        }
        g_last_family[kFamBwd] = 1;
        return launch_rope_bwd_tc(p, dtype, s);
    }
    g_last_family[kFamBwd] = 0;
    return launch_rope_bwd_general(p, dtype, s);
}

Rotation from_tables(const float* cos, const float* sin, int64_t stride) {
    Rotation r;
    r.cos = cos; r.sin = sin; r.stride = stride;
    return r;
}
Rotation from_freqs(const float* inv_freq) {
    Rotation r;
    r.inv_freq = inv_freq;
    return r;
}
Rotation no_rotation() {
    Rotation r;
    r.none = true;
    return r;
}

}  // namespace

extern "C" {

int corope_rope_attn_fwd(const void* q, const void* k, const void* v, const float* cos, const float* sin, int64_t table_row_stride, void* o,
                         float* lse2, int B, int H, int N, int D, int dtype, int causal, float sm_scale, void* workspace,
                         size_t workspace_bytes, int* status_word, void* stream) {
    return rope_fwd_impl(q, k, v, from_tables(cos, sin, table_row_stride), o, lse2, B, H, H, N, D, dtype, causal, sm_scale, workspace,
                         workspace_bytes, status_word, stream);
}

int corope_rope_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2, const float* cos,
                         const float* sin, int64_t table_row_stride, void* dq, void* dk, void* dv, int B, int H, int N, int D, int dtype,
                         int causal, float sm_scale, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
    return rope_bwd_impl(q, k, v, o, d_o, lse2, from_tables(cos, sin, table_row_stride), dq, dk, dv, B, H, H, N, D, dtype, causal, sm_scale,
                         workspace, workspace_bytes, status_word, stream);
}

int corope_rope_attn_fwd_strided(const void* q, const void* k, const void* v, const float* cos, const float* sin, int64_t table_row_stride,
                                 void* o, float* lse2, int B, int H, int N, int D, int dtype, int causal, float sm_scale, void* workspace,
                                 size_t workspace_bytes, int* status_word, void* stream, const corope_strides_t* strides) {
    return rope_fwd_impl(q, k, v, from_tables(cos, sin, table_row_stride), o, lse2, B, H, H, N, D, dtype, causal, sm_scale, workspace,
                         workspace_bytes, status_word, stream, strides);
}

int corope_rope_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                                 const float* cos, const float* sin, int64_t table_row_stride, void* dq, void* dk, void* dv, int B, int H,
                                 int N, int D, int dtype, int causal, float sm_scale, void* workspace, size_t workspace_bytes,
                                 int* status_word, void* stream, const corope_strides_t* strides) {
    return rope_bwd_impl(q, k, v, o, d_o, lse2, from_tables(cos, sin, table_row_stride), dq, dk, dv, B, H, H, N, D, dtype, causal, sm_scale,
                         workspace, workspace_bytes, status_word, stream, strides);
}

int corope_flash_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse2, int B, int Hq, int Hkv, int N, int D,
                                  int dtype, int causal, float sm_scale, void* workspace, size_t workspace_bytes, int* status_word,
                                  void* stream, const corope_strides_t* strides) {
    return rope_fwd_impl(q, k, v, no_rotation(), o, lse2, B, Hq, Hkv, N, D, dtype, causal, sm_scale, workspace, workspace_bytes, status_word,
                         stream, strides);
}

int corope_flash_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2, void* dq,
                                  void* dk, void* dv, int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale,
                                  void* workspace, size_t workspace_bytes, int* status_word, void* stream,
                                  const corope_strides_t* strides) {
    return rope_bwd_impl(q, k, v, o, d_o, lse2, no_rotation(), dq, dk, dv, B, Hq, Hkv, N, D, dtype, causal, sm_scale, workspace,
                         workspace_bytes, status_word, stream, strides);
}

int corope_rope_attn_fwd_freqs(const void* q, const void* k, const void* v, const float* inv_freq, void* o, float* lse2, int B, int H, int N,
                               int D, int dtype, int causal, float sm_scale, void* workspace, size_t workspace_bytes, int* status_word,
                               void* stream) {
    if (!inv_freq) return COROPE_ERR_NULL_POINTER;
    return rope_fwd_impl(q, k, v, from_freqs(inv_freq), o, lse2, B, H, H, N, D, dtype, causal, sm_scale, workspace, workspace_bytes,
                         status_word, stream);
}

int corope_rope_attn_bwd_freqs(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                               const float* inv_freq, void* dq, void* dk, void* dv, int B, int H, int N, int D, int dtype, int causal,
                               float sm_scale, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
    if (!inv_freq) return COROPE_ERR_NULL_POINTER;
    return rope_bwd_impl(q, k, v, o, d_o, lse2, from_freqs(inv_freq), dq, dk, dv, B, H, H, N, D, dtype, causal, sm_scale, workspace,
                         workspace_bytes, status_word, stream);
}

int corope_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse2, int B, int Hq, int Hkv, int N, int D, int dtype,
                          int causal, float sm_scale, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
    return rope_fwd_impl(q, k, v, no_rotation(), o, lse2, B, Hq, Hkv, N, D, dtype, causal, sm_scale, workspace, workspace_bytes, status_word,
                         stream);
}

int corope_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2, void* dq, void* dk,
                          void* dv, int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale, void* workspace,
                          size_t workspace_bytes, int* status_word, void* stream) {
    return rope_bwd_impl(q, k, v, o, d_o, lse2, no_rotation(), dq, dk, dv, B, Hq, Hkv, N, D, dtype, causal, sm_scale, workspace,
                         workspace_bytes, status_word, stream);
}

static int check_gqa(int B, int Hq, int Hkv, int N, int D, int dtype) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || D <= 0) return COROPE_ERR_BAD_SHAPE;
    if (Hq % Hkv != 0 || Hq / Hkv > 8) return COROPE_ERR_BAD_GROUP;
    return check_common(B, Hq, N, D, dtype);
}

int corope_gqa_fwd(const void* q, const void* k, const void* v, void* o, float* lse2, float* a_diag, int B, int Hq, int Hkv, int N, int D,
                   int dtype, float sm_scale, float theta, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
    return corope_gqa_fwd_strided(q, k, v, o, lse2, a_diag, B, Hq, Hkv, N, D, dtype, sm_scale, theta, workspace, workspace_bytes, status_word,
                                  stream, nullptr);
}

int corope_gqa_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse2, float* a_diag, int B, int Hq, int Hkv, int N,
                           int D, int dtype, float sm_scale, float theta, void* workspace, size_t workspace_bytes, int* status_word,
                           void* stream, const corope_strides_t* strides) {
    if (!q || !k || !v || !o || !lse2 || !a_diag) return COROPE_ERR_NULL_POINTER;
    if (int e = check_gqa(B, Hq, Hkv, N, D, dtype)) return e;
    GqaWorkspace w = gqa_workspace_layout(false, B, Hq, Hkv, N, D, dtype);
    if (int e = check_workspace(workspace, workspace_bytes, w.total)) return e;
    GqaParams p{};
    p.q = q; p.k = k; p.v = v; p.out_o = o; p.lse2 = lse2; p.a_diag = a_diag;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.N = N; p.D = D; p.sm_scale = sm_scale; p.theta = theta; p.status = status_word;
    set_gqa_strides(p, strides);
    if (!strides_positive(p.sq, D) || !strides_positive(p.sk, D) || !strides_positive(p.sv, D) || !strides_positive(p.so, D)) return COROPE_ERR_BAD_STRIDE;
    // the tensor-core kernels read K and V in 16-byte vectors and store O in element pairs
    if (g_policy.load() == 0 && gqa_fwd_mma_supported(N, D, dtype) && vec_ok(q, p.sq) && vec_ok(k, p.sk) && vec_ok(v, p.sv) && vec_ok(o, p.so)) {
        p.k_pairs = reinterpret_cast<uint32_t*>((char*)workspace + w.k_pairs);
        p.v_half = reinterpret_cast<__half*>((char*)workspace + w.v_half);
        g_last_family[COROPE_OP_GQA_FWD] = 1;
        return launch_gqa_fwd_mma(p, dtype, (cudaStream_t)stream);
    }
    g_last_family[COROPE_OP_GQA_FWD] = 0;
    return launch_gqa_fwd_general(p, dtype, (cudaStream_t)stream);
}

int corope_gqa_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2, const float* a_diag,
                   void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int N, int D, int dtype, float sm_scale, float theta,
                   void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
    return corope_gqa_bwd_strided(q, k, v, o, d_o, lse2, a_diag, dq, dk, dv, B, Hq, Hkv, N, D, dtype, sm_scale, theta, workspace,
                                  workspace_bytes, status_word, stream, nullptr);
}

int corope_gqa_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                           const float* a_diag, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int N, int D, int dtype,
                           float sm_scale, float theta, void* workspace, size_t workspace_bytes, int* status_word, void* stream,
                           const corope_strides_t* strides) {
    if (!q || !k || !v || !o || !d_o || !lse2 || !a_diag || !dq || !dk || !dv) return COROPE_ERR_NULL_POINTER;
    if (int e = check_gqa(B, Hq, Hkv, N, D, dtype)) return e;
    GqaWorkspace w = gqa_workspace_layout(true, B, Hq, Hkv, N, D, dtype);
    if (int e = check_workspace(workspace, workspace_bytes, w.total)) return e;
    GqaParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.d_o = d_o; p.dq = dq; p.dk = dk; p.dv = dv;
    p.lse2 = const_cast<float*>(lse2); p.a_diag = const_cast<float*>(a_diag);
    p.delta = reinterpret_cast<float*>((char*)workspace + w.delta);
    p.dk_acc = reinterpret_cast<float*>((char*)workspace + w.dk_acc);
    p.dv_acc = reinterpret_cast<float*>((char*)workspace + w.dv_acc);
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.N = N; p.D = D; p.sm_scale = sm_scale; p.theta = theta; p.status = status_word;
    set_gqa_strides(p, strides);
    for (const Strides* st : {&p.sq, &p.sk, &p.sv, &p.so, &p.sdo, &p.sdq, &p.sdk, &p.sdv})
        if (!strides_positive(*st, D)) return COROPE_ERR_BAD_STRIDE;
    const bool vec = vec_ok(q, p.sq) && vec_ok(k, p.sk) && vec_ok(v, p.sv) && vec_ok(o, p.so) && vec_ok(d_o, p.sdo) && vec_ok(dq, p.sdq) &&
                     vec_ok(dk, p.sdk) && vec_ok(dv, p.sdv);
    if (g_policy.load() == 0 && gqa_fwd_mma_supported(N, D, dtype) && vec) {
        p.k_pairs = reinterpret_cast<uint32_t*>((char*)workspace + w.k_pairs);
        p.v_half = reinterpret_cast<__half*>((char*)workspace + w.v_half);
        p.use_mma = 1;
    }
    g_last_family[COROPE_OP_GQA_BWD] = p.use_mma;
    return launch_gqa_bwd_general(p, dtype, (cudaStream_t)stream);
}

}  // extern "C"
