/*
 * corope_b200 -- C ABI of the B200 (sm_100a) fused-RoPE attention and Co-RoPE GQA attention kernels.
 *
 * Plain pointers and sizes only; no C++ or torch types cross this boundary.  All tensor
 * pointers are DEVICE pointers.  q/k/v/o/dO/dq/dk/dv are row-major contiguous [B, H, N, D]
 * in the element type named by `dtype` (the *_strided entry points take other layouts).  Every call enqueues work on `stream` (a
 * cudaStream_t passed as void*) and returns without synchronising.
 *
 * Return value: 0 = OK, < 0 = argument error found on the host (nothing was launched),
 * > 0 = a cudaError_t from a launch.  Kernels never trap: a device-side bounded wait that
 * expires writes a non-zero code into `*status_word` (device memory, may be NULL) and the
 * kernel exits cleanly.  While the word is non-zero, later tensor-core launches that are given the
 * same word return without computing (their outputs are then undefined): read and clear it on the
 * host after synchronising.  The Python modules of this package do that for the caller: every call
 * first looks at a pinned host mirror of the word that the previous call's stream refreshed, and
 * raises (and clears the word) if it was set.
 *
 * Supported value range of 16-bit inputs: the tensor-core kernels feed fp16 operands to the MMAs
 * (rotated Q / K, dS) with saturating conversions, so results are exact in kind for |q|, |k| up to
 * a few hundred and for gradient magnitudes |dO| up to about 2^10; beyond that single products may
 * clamp to +-65504 and results lose accuracy without becoming inf / NaN.  fp32 inputs have no such
 * limit (fp32 arithmetic throughout).
 *
 * Each entry point names the interface of the reference (Superposition09m/Co-RoPE) it stands in for.
 */
#ifndef COROPE_B200_H_
#define COROPE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of q/k/v/o and gradients */
#define COROPE_DTYPE_F32 0
#define COROPE_DTYPE_BF16 1
#define COROPE_DTYPE_F16 2

/* `op` values for corope_workspace_bytes */
#define COROPE_OP_ROPE_FWD 0
#define COROPE_OP_ROPE_BWD 1
#define COROPE_OP_GQA_FWD 2
#define COROPE_OP_GQA_BWD 3
#define COROPE_OP_ROPE_FWD_FREQS 4   /* corope_rope_attn_fwd_freqs: as ROPE_FWD plus room for the synthesized tables */
#define COROPE_OP_ROPE_BWD_FREQS 5
#define COROPE_OP_FLASH_FWD 6        /* corope_flash_attn_fwd (Hq query heads, Hkv K / V heads) */
#define COROPE_OP_FLASH_BWD 7

/* host-side argument errors */
#define COROPE_OK 0
#define COROPE_ERR_NULL_POINTER (-1)
#define COROPE_ERR_BAD_SHAPE (-2)      /* non-positive extent */
#define COROPE_ERR_BAD_HEAD_DIM (-3)   /* D outside the supported set (fused_rope_attn.py:661 asserts the same way) */
#define COROPE_ERR_BAD_DTYPE (-4)
#define COROPE_ERR_WORKSPACE (-5)      /* workspace missing, too small or misaligned (needs 256-byte alignment) */
#define COROPE_ERR_BAD_GROUP (-6)      /* Hq % Hkv != 0 or group size > 8 (flash_attn_co_rope_gqa_triton.py:421-425) */
#define COROPE_ERR_SEQ_NOT_128 (-7)    /* backward needs N % 128 == 0 (fused_rope_attn.py:750) -- only when strict_n is set */
#define COROPE_ERR_TENSOR_MAP (-8)     /* TMA descriptor could not be encoded */
#define COROPE_ERR_NO_DEVICE (-9)      /* no sm_100 device / driver entry point */
#define COROPE_ERR_TOO_LARGE (-10)     /* size beyond what the entry point supports */
#define COROPE_ERR_BAD_STRIDE (-11)    /* row stride below D, or a negative stride */

/* device-side status codes written to *status_word */
#define COROPE_DEV_OK 0
#define COROPE_DEV_WAIT_EXPIRED 0x1000 /* | barrier id: a bounded mbarrier wait ran out */
#define COROPE_DEV_RANGE 0x2000        /* a gradient term left the range of the 16-bit Co-RoPE backward and was clamped */

int corope_abi_version(void);

/*
 * Host mirror of a status word, for callers that want to learn of a device-side error without ever synchronising:
 * `_refresh` makes a side stream of the library copy *status_word to *host_mirror (pinned host memory) once `stream` has
 * executed everything enqueued so far -- `stream` itself only records an event -- so that reading *host_mirror on the host
 * before a later call shows whether an earlier call failed.  `_clear` resets both (it waits for the side stream first).
 * No counterpart in the reference, whose kernels report nothing.
 */
int corope_status_mirror_refresh(const int* status_word, int* host_mirror, void* stream);
int corope_status_mirror_clear(int* status_word, int* host_mirror, void* stream);
const char* corope_status_string(int status);

/* Bytes of caller-provided scratch (device memory, 256-byte aligned) an op needs.  Contents
 * need not be initialised by the caller.  For MHA pass Hkv == Hq.  For 16-bit inputs at D = 128 the
 * fused-RoPE ops keep a rotated fp16 copy of K (forward) or Q (backward) there, so the size grows
 * with B*H*N*D (forward: 2 bytes per element of k; backward: 6 bytes per element of q).  16-bit
 * inputs at D = 64 with N % 128 == 0 are run zero-padded to D = 128 and also keep their padded copies
 * there (forward: 16 bytes per element of q; backward: 32).  Always ask this function. */
size_t corope_workspace_bytes(int op, int B, int Hq, int Hkv, int N, int D, int dtype);

/*
 * Fused RoPE attention forward.  Replaces the launch in _attention.forward
 * (fused-rope/fused_rope_attn.py:655-722, kernels _attn_fwd / _attn_fwd_inner :47-320).
 *   cos, sin : fp32 tables, row n at cos + n*table_row_stride, only columns [0, D/2) are read
 *              (fused_rope_attn.py:88-93, 279-284) -- both [N, D] "cat" and [N, D/2] tables work.
 *   o        : [B,H,N,D] output in `dtype`.
 *   lse2     : [B,H,N] fp32, log2-domain log-sum-exp of the scaled scores (the reference's M, :316).
 */
int corope_rope_attn_fwd(const void* q, const void* k, const void* v,
                         const float* cos, const float* sin, int64_t table_row_stride,
                         void* o, float* lse2,
                         int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                         void* workspace, size_t workspace_bytes,
                         int* status_word, void* stream);

/*
 * Fused RoPE attention forward that allocates nothing and takes no workspace.  It has no counterpart in the
 * reference.  It exists for callers that may not allocate device memory at the point of the call and have no
 * spare buffer to lend: code running under a framework that hands out a fixed, fully planned memory arena,
 * inference servers with a hard memory budget, or a call site where an allocation would synchronise the device.
 * Same arguments and results as corope_rope_attn_fwd minus the workspace.  The one piece of scratch the forward
 * uses (the packed cos/sin table) lives in a 2 MiB array inside the library image, per GPU, until the process
 * exits.  Limit: N * (D/2) <= 524288 (N <= 8192 at D = 128); larger sizes return COROPE_ERR_TOO_LARGE.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  All calls on a device share the array: two calls
 * whose kernels can overlap on the GPU (different streams, no ordering between them) race on it; calls ordered
 * on one stream are safe, and nothing left by an earlier call is ever read.  Calls no cudaMalloc/cudaFree.
 */
int corope_rope_attn_fwd_noalloc(const void* q, const void* k, const void* v,
                                 const float* cos, const float* sin, int64_t table_row_stride,
                                 void* o, float* lse2,
                                 int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                                 int* status_word, void* stream);

/*
 * Fused RoPE attention backward.  Replaces _attention.backward
 * (fused-rope/fused_rope_attn.py:725-777: the K pre-scale :746-748, _attn_bwd_preprocess :324-337,
 * _attn_bwd :474-649).  o and lse2 are the forward's outputs; dq/dk/dv are written in `dtype`.
 */
int corope_rope_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                         const float* lse2,
                         const float* cos, const float* sin, int64_t table_row_stride,
                         void* dq, void* dk, void* dv,
                         int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                         void* workspace, size_t workspace_bytes,
                         int* status_word, void* stream);

/*
 * Strides, in elements, of the eight [B, H, N, D] tensors an op can touch: {batch, head, row} each; the head-dim stride is
 * always 1.  The reference hands all four strides of q / k / v / o to its kernels (fused-rope/fused_rope_attn.py:709-710,
 * flash_attn_v2_triton.py:601-603), so views such as a [B, N, H, D] buffer transposed to [B, H, N, D] need no copy there;
 * the *_strided entry points below take them here.  Fields an op does not use (d_o, dq, dk, dv in a forward) are ignored.
 * The tensor-core kernels need every used stride and base pointer to be a multiple of 16 bytes (8 elements for 16-bit
 * types); other strides run on the CUDA-core kernels.  lse2 (and the tables) stay contiguous.  A NULL `strides` means
 * contiguous tensors, i.e. the plain entry point.
 */
typedef struct corope_strides_t {
    int64_t q[3], k[3], v[3], o[3], d_o[3], dq[3], dk[3], dv[3];
} corope_strides_t;

int corope_rope_attn_fwd_strided(const void* q, const void* k, const void* v,
                                 const float* cos, const float* sin, int64_t table_row_stride,
                                 void* o, float* lse2,
                                 int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                                 void* workspace, size_t workspace_bytes,
                                 int* status_word, void* stream, const corope_strides_t* strides);
int corope_rope_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse2,
                                 const float* cos, const float* sin, int64_t table_row_stride,
                                 void* dq, void* dk, void* dv,
                                 int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                                 void* workspace, size_t workspace_bytes,
                                 int* status_word, void* stream, const corope_strides_t* strides);

/*
 * Fused RoPE attention with the cos / sin tables synthesized on the device instead of read from the caller: the angle
 * of position n and pair d is float(n) * inv_freq[d] in fp32, exactly how precompute_freqs_cis forms it
 * (fused-rope/rope_attn_pytorch.py:29-47: inv_freq[d] = 1 / theta^(2d/D), positions 0 .. N-1), followed by cosf / sinf.
 * For callers whose tables are that function's output, this removes the tables from the interface and from HBM
 * traffic; corope_rope_attn_fwd / _bwd with explicit tables remain the general case (arbitrary positions, scaled
 * or interpolated frequencies).   inv_freq : D/2 floats in device memory.  Workspace: COROPE_OP_ROPE_FWD_FREQS /
 * COROPE_OP_ROPE_BWD_FREQS.  Everything else as corope_rope_attn_fwd / corope_rope_attn_bwd.
 */
int corope_rope_attn_fwd_freqs(const void* q, const void* k, const void* v, const float* inv_freq,
                               void* o, float* lse2,
                               int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                               void* workspace, size_t workspace_bytes,
                               int* status_word, void* stream);
int corope_rope_attn_bwd_freqs(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                               const float* lse2, const float* inv_freq,
                               void* dq, void* dk, void* dv,
                               int B, int H, int N, int D, int dtype, int causal, float sm_scale,
                               void* workspace, size_t workspace_bytes,
                               int* status_word, void* stream);

/*
 * Plain flash attention (no RoPE) with grouped K / V heads.  Replaces _attention.forward / .backward of the reference's
 * un-fused kernel (fused-rope/flash_attn_v2_triton.py:513-631; head mapping off_h_kv = off_h_q // GROUP_SIZE :194-196);
 * the math is that of assets/flashattn-gqa/attn_gqa_pytorch.py:17-190.
 *   q, o, d_o, dq : [B,Hq,N,D];  k, v, dk, dv : [B,Hkv,N,D];  Hq % Hkv == 0 (any group size);  lse2 : [B,Hq,N].
 * dk / dv are summed over each group (the reference's backward takes Hq == Hkv only, :560; this one takes both).
 * Same kernels as the fused-RoPE ops with the rotation switched off.  Workspace: COROPE_OP_FLASH_FWD / COROPE_OP_FLASH_BWD.
 */
int corope_flash_attn_fwd(const void* q, const void* k, const void* v,
                          void* o, float* lse2,
                          int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale,
                          void* workspace, size_t workspace_bytes,
                          int* status_word, void* stream);
int corope_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse2,
                          void* dq, void* dk, void* dv,
                          int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale,
                          void* workspace, size_t workspace_bytes,
                          int* status_word, void* stream);

int corope_flash_attn_fwd_strided(const void* q, const void* k, const void* v,
                                  void* o, float* lse2,
                                  int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale,
                                  void* workspace, size_t workspace_bytes,
                                  int* status_word, void* stream, const corope_strides_t* strides);
int corope_flash_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                  const float* lse2,
                                  void* dq, void* dk, void* dv,
                                  int B, int Hq, int Hkv, int N, int D, int dtype, int causal, float sm_scale,
                                  void* workspace, size_t workspace_bytes,
                                  int* status_word, void* stream, const corope_strides_t* strides);

/*
 * Co-RoPE GQA attention forward (causal only).  Replaces the launch in _attention.forward
 * (corope-exp/flash_attn_co_rope_gqa_triton.py:406-456, kernel _corope_fwd_backbone :47-400);
 * the math is that of corope-exp/corope_attn_gqa_pytorch.py:56-124.
 *   q, o   : [B,Hq,N,D];  k, v : [B,Hkv,N,D];  Hq % Hkv == 0, Hq/Hkv <= 8.
 *   lse2   : [B,Hq,N] fp32 (log2 domain);  a_diag : [B,Hkv,N] fp32, the leader mileage a_ii.
 * For 16-bit inputs at D = 128 and N % 64 == 0 the workspace holds fp16 operand copies of K and V
 * (4 bytes per element of k); otherwise the forward needs none (corope_workspace_bytes returns the 256-byte minimum).
 */
int corope_gqa_fwd(const void* q, const void* k, const void* v,
                   void* o, float* lse2, float* a_diag,
                   int B, int Hq, int Hkv, int N, int D, int dtype, float sm_scale, float theta,
                   void* workspace, size_t workspace_bytes,
                   int* status_word, void* stream);

/* corope_gqa_fwd with every tensor's own {batch, head, row} strides (the q, k, v, o fields of `strides`, in elements; NULL =
 * contiguous).  Replaces the stride arguments of the reference's kernel launch (flash_attn_co_rope_gqa_triton.py:439-442).
 * The tensor-core kernels run when all pointers and strides are multiples of 16 bytes, the CUDA-core kernels otherwise. */
int corope_gqa_fwd_strided(const void* q, const void* k, const void* v,
                           void* o, float* lse2, float* a_diag,
                           int B, int Hq, int Hkv, int N, int D, int dtype, float sm_scale, float theta,
                           void* workspace, size_t workspace_bytes,
                           int* status_word, void* stream, const corope_strides_t* strides);

/*
 * Co-RoPE GQA attention backward.  Replaces _attention.backward
 * (corope-exp/flash_attn_co_rope_gqa_triton.py:459-577, dense PyTorch there); the math is that of
 * corope-exp/corope_attn_gqa_pytorch.py:138-300.  dk/dv are [B,Hkv,N,D] (summed over the group).
 */
int corope_gqa_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                   const float* lse2, const float* a_diag,
                   void* dq, void* dk, void* dv,
                   int B, int Hq, int Hkv, int N, int D, int dtype, float sm_scale, float theta,
                   void* workspace, size_t workspace_bytes,
                   int* status_word, void* stream);

/* corope_gqa_bwd with every tensor's own strides (all eight fields of `strides`; NULL = contiguous). */
int corope_gqa_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                           const float* lse2, const float* a_diag,
                           void* dq, void* dk, void* dv,
                           int B, int Hq, int Hkv, int N, int D, int dtype, float sm_scale, float theta,
                           void* workspace, size_t workspace_bytes,
                           int* status_word, void* stream, const corope_strides_t* strides);

#ifdef __cplusplus
}
#endif
#endif /* COROPE_B200_H_ */
