/*
 * msda_b200.h - C ABI of the sm_100a multi-scale deformable attention kernels.
 *
 * Plain pointers and sizes only; no torch types cross this boundary.  The library
 * (libmsda_b200.so) is what an operator registry binds in place of the reference's
 * native entry points.  Each function below names the reference interface it replaces
 * (paths relative to the reference project).
 *
 * Conventions
 *   - All pointers are DEVICE pointers on `device`, 16-byte aligned, contiguous row-major:
 *       value / grad_value   (B, S, G, D)          element type `dtype`
 *       spatial_shapes       (L, 2) int64 rows (height, width)
 *       level_start_index    (L)    int64 exclusive prefix sum of height*width
 *       loc / grad_loc       (B, Q, G, L, K, 2)    float32, (x, y) normalised to [0, 1]
 *       attn / grad_attn     (B, Q, G, L*K)        element type `dtype`
 *       out / grad_out       (B, Q, G*D)           element type `dtype`
 *   - The level tables are read on the device; no call synchronises with the host.  A level
 *     whose table entry does not lie inside the value tensor (non-positive height or width,
 *     negative start, start + height*width > S) is treated as empty: its points contribute
 *     nothing and receive zero gradients; no address outside the tensors is formed.
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = default
 *     stream) and the call returns immediately.  Inputs are borrowed, outputs are
 *     caller-allocated; nothing is allocated or freed here.
 *   - Return value: MSDA_B200_OK or a negative status; the message of the last failure
 *     on the calling thread is available from msda_b200_last_error().  No exception or
 *     longjmp ever crosses the boundary.
 *   - Thread safety: no mutable global state; concurrent calls from several host
 *     threads (for example the autograd thread) are allowed.
 *   - Supported: dtype f32 / f16 / bf16 (and f64, see the enum); D a multiple of 4 (f32) or
 *     8 (f16, bf16);
 *     1 <= L <= 16; any K >= 1; S*G*D < 2^31 per sample.  B == 0 or Q == 0 is a
 *     successful no-op (backward still clears grad_value).
 */
#ifndef MSDA_B200_H_
#define MSDA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSDA_B200_ABI_VERSION 5

/*
 * MSDA_B200_F64: value, attn, out AND loc / grad_loc are double (pass the double pointers
 * through the `float *` parameters).  Meant for numerical differentiation
 * (torch.autograd.gradcheck), as in the reference (msda_launch.cuh:54-61); simple kernels, any
 * D >= 1, no scratch, not available through the *_offsets entry points.
 */
enum msda_b200_dtype { MSDA_B200_F32 = 0, MSDA_B200_F16 = 1, MSDA_B200_BF16 = 2, MSDA_B200_F64 = 3 };

enum msda_b200_status {
    MSDA_B200_OK = 0,
    MSDA_B200_INVALID_ARGUMENT = -1, /* null / misaligned pointer, negative size, bad enum */
    MSDA_B200_UNSUPPORTED = -2,      /* shape outside the envelope listed above */
    MSDA_B200_CUDA_ERROR = -3        /* the CUDA runtime reported an error (message has it) */
};

/* Version of this ABI; bumped on any signature change. */
int msda_b200_abi_version(void);

/* Message of the last failing call on this thread ("" if none). Never NULL. */
const char *msda_b200_last_error(void);

/*
 * Forward: out[b,q,g,:] = sum_{l,k} a[b,q,g,l,k] * bilinear(value level l, loc[b,q,g,l,k]).
 * apply_softmax != 0 normalises attn over its L*K entries inside the kernel first.
 *
 * Replaces: boxed op `<prefix>_forward` / `<prefix>_softmax_forward`
 *   sources/deformops/backends/cuda/include/msda_boxed.cuh:14-28
 *   sources/deformops/backends/cuda/include/msda_launch.cuh:63-138 (forward_cuda)
 *   schema sources/deformops/backends/cuda/_schema.py:18-23
 * Differences: the output is caller-allocated and need not be zeroed (every element is
 * written); there is no batch chunking (chunk_step has no effect on results).
 */
int msda_b200_forward(const void *value, const int64_t *spatial_shapes,
                      const int64_t *level_start_index, const float *loc, const void *attn,
                      void *out, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
                      int64_t K, int dtype, int apply_softmax, int device, void *stream);

/*
 * Backward: given grad_out, produces grad_value (scatter with packed 16-byte reductions),
 * grad_loc (float32) and grad_attn (`dtype`; gradient w.r.t. the raw logits when
 * apply_softmax != 0).  grad_loc and grad_attn are written in full (skipped points get
 * exact zeros).  If zero_grad_value != 0 the call first clears grad_value on `stream`;
 * pass 0 to accumulate into a buffer the caller prepared (scratch must then be NULL).
 *
 * scratch (16-bit dtypes only): summing n contributions per element in f16/bf16 loses about
 * sqrt(n) ulps (2^-9 each for bf16), and a coarse pyramid level receives hundreds.  When
 * `scratch` is not NULL it must hold msda_b200_backward_scratch_bytes(...) bytes.  The call
 * then multiplies every contribution by one power of two, chosen on the device from the
 * largest |grad_out| and |attn| element so that no sum can leave the float16 range, adds it
 * in float16 (11 significant bits, packed 16-byte reductions) into an image of grad_value
 * held in the scratch (a level that receives more than 256 additions per element is given
 * several accumulators there), and a last pass unscales the sums into grad_value in `dtype`.  Such
 * a call enqueues a 256-byte memset and three kernels; for large shapes the second and third are
 * launched as programmatic dependents of the one before (they become resident while it drains
 * and wait for its completion on the device), which CUDA-graph capture records as well.  With
 * scratch == NULL every contribution is added straight into grad_value in `dtype` (least
 * accurate for bf16).  Ignored for float32.  `scratch_adds` is accepted for callers written
 * against ABI version 4 and has no effect.
 *
 * Replaces: boxed op `<prefix>_backward` / `<prefix>_softmax_backward`
 *   sources/deformops/backends/cuda/include/msda_boxed.cuh:32-53
 *   sources/deformops/backends/cuda/include/msda_launch.cuh:141-275 (backward_cuda)
 *   schema sources/deformops/backends/cuda/_schema.py:24-29
 * Differences: gradients and scratch are caller-allocated; grad_attn is produced directly
 * in `dtype`; accuracy comes from scaled float16 accumulation (2 bytes per element) instead
 * of a float32 copy of the whole tensor (msda_launch.cuh:188-197, 263-273 upcast, clear and
 * cast back 4 bytes per element).
 */
int msda_b200_backward(const void *value, const int64_t *spatial_shapes,
                       const int64_t *level_start_index, const float *loc, const void *attn,
                       const void *grad_out, void *grad_value, float *grad_loc, void *grad_attn,
                       void *scratch, int64_t scratch_bytes, int64_t scratch_adds, int64_t B,
                       int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                       int apply_softmax, int zero_grad_value, int device, void *stream);

/*
 * Bytes of scratch msda_b200_backward can use for a shape, for the 16-bit dtypes: a 256-byte
 * header, one float16 image of grad_value (B*S*G*D*2) and, per sample, room for the extra
 * accumulators of coarse levels (at most L * K*Q*G*D / 64 float16, a few per cent of the
 * image when Q is about S).  0 for float32.
 * Replaces: the `new_zeros` float32 grad_value of msda_launch.cuh:188-197.
 */
int64_t msda_b200_backward_scratch_bytes(int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q,
                                         int64_t L, int64_t K, int dtype);

/*
 * Forward / backward with the caller's location arithmetic fused in.  Instead of a location
 * tensor the call takes what a deformable-attention layer predicts and where it anchors it:
 *   offsets           (B, Q, G, L, K, 2)  float32 or `dtype` (offsets_dtype says which)
 *   reference_points  (B, Q, L, ref_coords) float32, 16-byte aligned;
 *                     ref_coords = 2: (x, y) normalised;  4: a box (cx, cy, w, h)
 * and samples at, in float32,
 *   ref_coords = 2:  reference.xy + offset / (W_l, H_l)
 *   ref_coords = 4:  reference.xy + offset / K * reference.wh * 0.5
 * so the location tensor (the largest operand of the op) is never written or read.
 * grad_offsets has the shape and element type of offsets and is written in full.  No gradient
 * is produced for reference_points; for ref_coords = 2 it is the sum of
 * grad_offsets * (W_l, H_l) over heads and points, which a caller can form from grad_offsets.
 * Everything else (value, attn, scratch, status codes, stream and device) is as in
 * msda_b200_forward / msda_b200_backward.
 * Replaces: the elementwise location passes the reference's layers run in torch before the
 * op and autograd runs after it (sources/deformops/nn/msda.py:222-239,
 * sources/deformops/integrations/transformers.py:185-218) together with
 * msda_launch.cuh:63-138 / :141-275.
 */
int msda_b200_forward_offsets(const void *value, const int64_t *spatial_shapes,
                              const int64_t *level_start_index, const float *reference_points,
                              int ref_coords, const void *offsets, int offsets_dtype,
                              const void *attn, void *out, int64_t B, int64_t S, int64_t G,
                              int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                              int apply_softmax, int device, void *stream);

int msda_b200_backward_offsets(const void *value, const int64_t *spatial_shapes,
                               const int64_t *level_start_index, const float *reference_points,
                               int ref_coords, const void *offsets, int offsets_dtype,
                               const void *attn, const void *grad_out, void *grad_value,
                               void *grad_offsets, void *grad_attn, void *scratch,
                               int64_t scratch_bytes, int64_t scratch_adds, int64_t B, int64_t S,
                               int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                               int apply_softmax, int zero_grad_value, int device, void *stream);

/*
 * Backward for callers that cannot allocate device memory (a runtime that handed all of it
 * out at start-up and forbids cudaMalloc afterwards, a plugin running inside someone else's
 * step, a C program without a caching allocator).  Same results as msda_b200_backward with a
 * scratch buffer, but the scratch is a fixed 32 MiB array inside the library: a GPU that
 * uses this entry point holds it until the process exits.
 *   - A shape whose msda_b200_backward_scratch_bytes(...) exceed 32 MiB (about 14 million
 *     grad_value elements for a three-level pyramid with Q = S; 16-bit dtypes) returns
 *     MSDA_B200_UNSUPPORTED.
 *   - No cudaMalloc / cudaFree / allocating library call is made.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress); make
 *     that first call outside any stream capture.
 *   - Every call reuses the one array, which still holds the previous call's sums; each call
 *     clears what it adds into.  Calls that overlap on the GPU race: serialise them.
 *   - grad_value is always cleared (there is no accumulate mode here).
 * This entry point has no counterpart in the reference.
 */
int msda_b200_backward_static_scratch(const void *value, const int64_t *spatial_shapes,
                                      const int64_t *level_start_index, const float *loc,
                                      const void *attn, const void *grad_out, void *grad_value,
                                      float *grad_loc, void *grad_attn, int64_t scratch_adds,
                                      int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q,
                                      int64_t L, int64_t K, int dtype, int apply_softmax,
                                      int device, void *stream);

/*
 * Launch geometry the library plans for a shape, for harnesses that count launches or size
 * grids: `grid` = CTAs needed to give every group of (query, head) pairs one warp pass,
 * threads per CTA and dynamic shared memory of the forward (*_fwd) and backward (*_bwd)
 * kernels.  Pure function of its arguments and independent of the device; at launch time the
 * forward caps its grid at the number of CTAs the device holds at once (persistent CTAs) and
 * the backward lets a CTA make two adjacent passes when that still leaves several waves.
 * Replaces: forward_thread_layout / backward_thread_layout
 *   sources/deformops/core/tuning.py:55-133, include/msda_launch.cuh:26-52
 */
int msda_b200_launch_geometry(int64_t B, int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K,
                              int dtype, int apply_softmax, int64_t *grid, int *threads,
                              int64_t *smem_fwd, int64_t *smem_bwd);

#ifdef __cplusplus
}
#endif

#endif /* MSDA_B200_H_ */
