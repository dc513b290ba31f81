// C ABI of the library (declared in include/msda_b200.h): argument checks, launch
// geometry and error reporting.  Takes over the role of the reference's host entry
// sources/deformops/backends/cuda/include/msda_launch.cuh:63-275 without any torch type.
#include <cstdarg>
#include <cstdio>

#include "../../include/msda_b200.h"
#include "msda_common.cuh"

namespace {

thread_local char g_error[512] = "";

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int element_size(int dtype) {
    return dtype == MSDA_B200_F64 ? 8 : dtype == MSDA_B200_F32 ? 4 : 2;
}

constexpr size_t kSmemBudget = 96 * 1024;   // per CTA, so that at least two CTAs share an SM

// Shape checks shared by forward, backward and the geometry query; fills the launch plan.
int plan(msda_b200::Params &p, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
         int64_t K, int dtype, bool softmax) {
    if (dtype != MSDA_B200_F32 && dtype != MSDA_B200_F16 && dtype != MSDA_B200_BF16 &&
        dtype != MSDA_B200_F64)
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "dtype %d is not f32(0), f16(1), bf16(2) or f64(3)", dtype);
    if (B < 0 || S < 0 || Q < 0 || G <= 0 || D <= 0 || L <= 0 || K <= 0)
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "sizes must satisfy B,S,Q >= 0 and G,D,L,K > 0 (got B=%lld S=%lld G=%lld "
                    "D=%lld Q=%lld L=%lld K=%lld)",
                    (long long)B, (long long)S, (long long)G, (long long)D, (long long)Q,
                    (long long)L, (long long)K);
    const int vec = dtype == MSDA_B200_F64 ? 1 : 16 / element_size(dtype);
    if (D % vec != 0)
        return fail(MSDA_B200_UNSUPPORTED,
                    "head dimension D=%lld must be a multiple of %d for this dtype (16-byte "
                    "channel vectors)",
                    (long long)D, vec);
    if (L > msda_b200::kMaxLevels)
        return fail(MSDA_B200_UNSUPPORTED, "L=%lld levels exceed the supported %d", (long long)L,
                    msda_b200::kMaxLevels);
    if (S * G * D >= (int64_t)1 << 31 || L * K >= (int64_t)1 << 15)
        return fail(MSDA_B200_UNSUPPORTED,
                    "S*G*D = %lld must stay below 2^31 (32-bit offsets inside a sample) and "
                    "L*K below 2^15",
                    (long long)(S * G * D));

    p.B = B;
    p.S = S;
    p.Q = Q;
    p.G = (int)G;
    p.D = (int)D;
    p.L = (int)L;
    p.K = (int)K;
    if (dtype == MSDA_B200_F64) {
        // the float64 kernels (msda_f64.cu) run a warp per (query, head) pair, no staging
        p.lph_log2 = 5;
        p.point_chunk = (int)(L * K);
        p.threads = 256;
        p.num_groups = B * Q * G;
        const int64_t grid = (p.num_groups + 7) / 8;
        p.grid = (unsigned)(grid > 148 * 64 ? 148 * 64 : grid);
        return MSDA_B200_OK;
    }
    const int lanes = (int)(D / vec);
    int lg = 0;
    while ((1 << lg) < lanes && lg < 5) ++lg;
    p.lph_log2 = lg;
    const int ppw = 32 >> lg;
    const int P = (int)(L * K);
    p.point_chunk = P < msda_b200::kDescPerWarp / ppw ? P : msda_b200::kDescPerWarp / ppw;
    if (MSDA_POINT_CHUNK_CAP > 0 && p.point_chunk > MSDA_POINT_CHUNK_CAP && lanes <= 32)
        p.point_chunk = MSDA_POINT_CHUNK_CAP;
    if (lanes > 32 && P > p.point_chunk)
        return fail(MSDA_B200_UNSUPPORTED,
                    "D=%lld needs several channel passes and L*K=%d several point chunks; "
                    "only one of the two is supported",
                    (long long)D, P);

    // CTA size: 8 warps unless the per-warp gradient staging of the backward is too large
    p.threads = 256;
    while (p.threads > 32 && (msda_b200::backward_smem_bytes(p, softmax) > kSmemBudget ||
                              msda_b200::forward_smem_bytes(p, softmax) > kSmemBudget))
        p.threads >>= 1;
    if (msda_b200::backward_smem_bytes(p, softmax) > 200 * 1024)
        return fail(MSDA_B200_UNSUPPORTED, "L*K = %d is too large for the shared-memory staging", P);
    const int nwarps = p.threads / 32;
    p.num_groups = (B * Q * G + ppw - 1) / ppw;
    const int64_t grid = (p.num_groups + nwarps - 1) / nwarps;
    p.grid = (unsigned)(grid > 0x7fffffff ? 0x7fffffff : grid);   // kernels are grid-stride
    return MSDA_B200_OK;
}

// Makes `device` current for the duration of a call and restores the previous one.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device) {
        if (device < 0) return;
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            switched = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

int cuda_fail(cudaError_t e, const char *what) {
    return fail(MSDA_B200_CUDA_ERROR, "%s: %s (%s)", what, cudaGetErrorName(e),
                cudaGetErrorString(e));
}

// Where the sample locations come from: a location tensor, or predicted offsets plus
// reference points (the kernels then do the layer's location arithmetic themselves).
struct Points {
    const void *data;        // locations (float32) or offsets
    void *grad;              // gradient of `data`, same layout and element type (backward)
    const float *ref;        // reference points, or null when `data` holds locations
    int ref_coords;
    int offsets16;
};

int check_points(const Points &pts, int offsets_dtype, int dtype, const char *who) {
    if (pts.ref_coords != 2 && pts.ref_coords != 4)
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "%s: reference points carry %d coordinates; 2 (x, y) or 4 (cx, cy, w, h) "
                    "are supported", who, pts.ref_coords);
    if (dtype == MSDA_B200_F64)
        return fail(MSDA_B200_UNSUPPORTED,
                    "%s: float64 values take locations (msda_b200_forward / _backward)", who);
    if (offsets_dtype != MSDA_B200_F32 && offsets_dtype != dtype)
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "%s: offsets must be float32 or the value dtype (got %d for value dtype %d)",
                    who, offsets_dtype, dtype);
    return MSDA_B200_OK;
}

int forward_impl(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                 const Points &pts, const void *attn, void *out, int64_t B, int64_t S, int64_t G,
                 int64_t D, int64_t Q, int64_t L, int64_t K, int dtype, int apply_softmax,
                 int device, void *stream);
int backward_impl(const void *value, const int64_t *spatial_shapes,
                  const int64_t *level_start_index, const Points &pts, const void *attn,
                  const void *grad_out, void *grad_value, void *grad_attn, void *scratch,
                  int64_t scratch_bytes, int64_t scratch_adds, int64_t B, int64_t S, int64_t G,
                  int64_t D, int64_t Q, int64_t L, int64_t K, int dtype, int apply_softmax,
                  int zero_grad_value, int device, void *stream);

}  // namespace

namespace msda_b200 {
int set_last_error(int status, const char *message) { return fail(status, "%s", message); }
}  // namespace msda_b200

extern "C" {

int msda_b200_abi_version(void) { return MSDA_B200_ABI_VERSION; }

const char *msda_b200_last_error(void) { return g_error; }

int64_t msda_b200_backward_scratch_bytes(int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q,
                                         int64_t L, int64_t K, int dtype) {
    if (dtype != MSDA_B200_F16 && dtype != MSDA_B200_BF16) return 0;
    if (B <= 0 || S <= 0 || G <= 0 || D <= 0 || Q <= 0 || L <= 0 || K <= 0) return 0;
    return msda_b200::kScratchHeaderBytes +
           2 * B * (S * G * D + msda_b200::extra_elems_per_sample(Q, G, D, L, K));
}

int msda_b200_launch_geometry(int64_t B, int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K,
                              int dtype, int apply_softmax, int64_t *grid, int *threads,
                              int64_t *smem_fwd, int64_t *smem_bwd) {
    msda_b200::Params p{};
    const int st = plan(p, B, 1, G, D, Q, L, K, dtype, apply_softmax != 0);
    if (st != MSDA_B200_OK) return st;
    if (grid) *grid = p.grid;
    if (threads) *threads = p.threads;
    const bool f64 = dtype == MSDA_B200_F64;   // those kernels use no dynamic shared memory
    if (smem_fwd) *smem_fwd = f64 ? 0 : (int64_t)msda_b200::forward_smem_bytes(p, apply_softmax != 0);
    if (smem_bwd) *smem_bwd = f64 ? 0 : (int64_t)msda_b200::backward_smem_bytes(p, apply_softmax != 0);
    return MSDA_B200_OK;
}

int msda_b200_forward(const void *value, const int64_t *spatial_shapes,
                      const int64_t *level_start_index, const float *loc, const void *attn,
                      void *out, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
                      int64_t K, int dtype, int apply_softmax, int device, void *stream) {
    const Points pts{loc, nullptr, nullptr, 0, 0};
    return forward_impl(value, spatial_shapes, level_start_index, pts, attn, out, B, S, G, D, Q, L,
                        K, dtype, apply_softmax, device, stream);
}

int msda_b200_forward_offsets(const void *value, const int64_t *spatial_shapes,
                              const int64_t *level_start_index, const float *reference_points,
                              int ref_coords, const void *offsets, int offsets_dtype,
                              const void *attn, void *out, int64_t B, int64_t S, int64_t G,
                              int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                              int apply_softmax, int device, void *stream) {
    const Points pts{offsets, nullptr, reference_points, ref_coords,
                     offsets_dtype != MSDA_B200_F32};
    const int st = check_points(pts, offsets_dtype, dtype, "forward_offsets");
    if (st != MSDA_B200_OK) return st;
    if (B > 0 && Q > 0 && (!reference_points || !aligned16(reference_points)))
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "forward_offsets: reference_points is null or not 16-byte aligned");
    return forward_impl(value, spatial_shapes, level_start_index, pts, attn, out, B, S, G, D, Q, L,
                        K, dtype, apply_softmax, device, stream);
}

int msda_b200_backward(const void *value, const int64_t *spatial_shapes,
                       const int64_t *level_start_index, const float *loc, const void *attn,
                       const void *grad_out, void *grad_value, float *grad_loc, void *grad_attn,
                       void *scratch, int64_t scratch_bytes, int64_t scratch_adds, int64_t B,
                       int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                       int apply_softmax, int zero_grad_value, int device, void *stream) {
    const Points pts{loc, grad_loc, nullptr, 0, 0};
    return backward_impl(value, spatial_shapes, level_start_index, pts, attn, grad_out, grad_value,
                         grad_attn, scratch, scratch_bytes, scratch_adds, B, S, G, D, Q, L, K,
                         dtype, apply_softmax, zero_grad_value, device, stream);
}

int msda_b200_backward_offsets(const void *value, const int64_t *spatial_shapes,
                               const int64_t *level_start_index, const float *reference_points,
                               int ref_coords, const void *offsets, int offsets_dtype,
                               const void *attn, const void *grad_out, void *grad_value,
                               void *grad_offsets, void *grad_attn, void *scratch,
                               int64_t scratch_bytes, int64_t scratch_adds, int64_t B, int64_t S,
                               int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K, int dtype,
                               int apply_softmax, int zero_grad_value, int device, void *stream) {
    const Points pts{offsets, grad_offsets, reference_points, ref_coords,
                     offsets_dtype != MSDA_B200_F32};
    const int st = check_points(pts, offsets_dtype, dtype, "backward_offsets");
    if (st != MSDA_B200_OK) return st;
    if (B > 0 && Q > 0 && (!reference_points || !aligned16(reference_points)))
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "backward_offsets: reference_points is null or not 16-byte aligned");
    return backward_impl(value, spatial_shapes, level_start_index, pts, attn, grad_out, grad_value,
                         grad_attn, scratch, scratch_bytes, scratch_adds, B, S, G, D, Q, L, K,
                         dtype, apply_softmax, zero_grad_value, device, stream);
}

}  // extern "C"

namespace {

int forward_impl(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                 const Points &pts, const void *attn, void *out, int64_t B, int64_t S, int64_t G,
                 int64_t D, int64_t Q, int64_t L, int64_t K, int dtype, int apply_softmax,
                 int device, void *stream) {
    const void *loc = pts.data;
    msda_b200::Params p{};
    const int st = plan(p, B, S, G, D, Q, L, K, dtype, apply_softmax != 0);
    if (st != MSDA_B200_OK) return st;
    if (B == 0 || Q == 0) return MSDA_B200_OK;
    if (S == 0) {
        // nothing to sample from: every point falls outside, the output is zero
        if (!out) return fail(MSDA_B200_INVALID_ARGUMENT, "forward: null pointer argument");
        DeviceGuard guard(device);
        if (guard.err != cudaSuccess) return cuda_fail(guard.err, "forward: selecting the device");
        const cudaError_t e =
            cudaMemsetAsync(out, 0, (size_t)(B * Q * G * D) * element_size(dtype),
                            static_cast<cudaStream_t>(stream));
        return e == cudaSuccess ? MSDA_B200_OK : cuda_fail(e, "forward: clearing the output");
    }
    if (!value || !spatial_shapes || !level_start_index || !loc || !attn || !out)
        return fail(MSDA_B200_INVALID_ARGUMENT, "forward: null pointer argument");
    if (!aligned16(value) || !aligned16(loc) || !aligned16(attn) || !aligned16(out))
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "forward: value, loc, attn and out must be 16-byte aligned");
    p.value = value;
    p.spatial_shapes = spatial_shapes;
    p.level_start_index = level_start_index;
    p.loc = static_cast<const float *>(loc);
    p.ref = pts.ref;
    p.ref_coords = pts.ref_coords;
    p.offsets16 = pts.offsets16;
    p.attn = attn;
    p.out = out;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "forward: selecting the device");
    const cudaError_t e =
        dtype == MSDA_B200_F64
            ? msda_b200::launch_forward_f64(p, apply_softmax != 0, static_cast<cudaStream_t>(stream))
            : msda_b200::launch_forward(p, dtype, apply_softmax != 0,
                                        static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "forward: kernel launch");
    return MSDA_B200_OK;
}

int backward_impl(const void *value, const int64_t *spatial_shapes,
                  const int64_t *level_start_index, const Points &pts, const void *attn,
                  const void *grad_out, void *grad_value, void *grad_attn, void *scratch,
                  int64_t scratch_bytes, int64_t scratch_adds, int64_t B, int64_t S, int64_t G,
                  int64_t D, int64_t Q, int64_t L, int64_t K, int dtype, int apply_softmax,
                  int zero_grad_value, int device, void *stream) {
    const void *loc = pts.data;
    void *grad_loc = pts.grad;
    msda_b200::Params p{};
    const int st = plan(p, B, S, G, D, Q, L, K, dtype, apply_softmax != 0);
    if (st != MSDA_B200_OK) return st;
    if (B == 0) return MSDA_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (S == 0) {
        // an empty value tensor: no point samples anything, all gradients are zero
        if (Q == 0) return MSDA_B200_OK;
        if (!pts.grad || !grad_attn)
            return fail(MSDA_B200_INVALID_ARGUMENT, "backward: null pointer argument");
        DeviceGuard guard(device);
        if (guard.err != cudaSuccess) return cuda_fail(guard.err, "backward: selecting the device");
        const size_t points = (size_t)(B * Q * G) * (size_t)(L * K);
        const size_t loc_elem =
            pts.ref != nullptr && pts.offsets16 ? 2 : (dtype == MSDA_B200_F64 ? 8 : 4);
        cudaError_t e = cudaMemsetAsync(pts.grad, 0, points * 2 * loc_elem, s);
        if (e == cudaSuccess) e = cudaMemsetAsync(grad_attn, 0, points * element_size(dtype), s);
        return e == cudaSuccess ? MSDA_B200_OK : cuda_fail(e, "backward: clearing the gradients");
    }
    const bool use_scratch = scratch != nullptr &&
                             (dtype == MSDA_B200_F16 || dtype == MSDA_B200_BF16) && S > 0 && Q > 0;
    if (use_scratch) {
        if (!zero_grad_value)
            return fail(MSDA_B200_INVALID_ARGUMENT,
                        "backward: accumulating into a caller-prepared grad_value "
                        "(zero_grad_value = 0) cannot be combined with a scratch buffer");
        // (offsets into a sample's block of extra accumulators are 32-bit)
        if (msda_b200::extra_elems_per_sample(Q, G, D, L, K) >= ((int64_t)1 << 32))
            return fail(MSDA_B200_UNSUPPORTED,
                        "backward: Q*G*D*L*K = %lld is too large for the scratch layout (pass "
                        "scratch = NULL, or split the queries)",
                        (long long)(Q * G * D * L * K));
        const int64_t need = msda_b200_backward_scratch_bytes(B, S, G, D, Q, L, K, dtype);
        if (scratch_bytes < need)
            return fail(MSDA_B200_INVALID_ARGUMENT,
                        "backward: scratch holds %lld bytes, %lld are needed",
                        (long long)scratch_bytes, (long long)need);
        if (!aligned16(scratch))
            return fail(MSDA_B200_INVALID_ARGUMENT, "backward: scratch must be 16-byte aligned");
    }
    if ((S > 0 && !grad_value) || !aligned16(grad_value))
        return fail(MSDA_B200_INVALID_ARGUMENT, "backward: grad_value is null or misaligned");
    if (Q > 0) {
        if (!value || !spatial_shapes || !level_start_index || !loc || !attn || !grad_out ||
            !grad_loc || !grad_attn)
            return fail(MSDA_B200_INVALID_ARGUMENT, "backward: null pointer argument");
        if (!aligned16(value) || !aligned16(loc) || !aligned16(attn) || !aligned16(grad_out) ||
            !aligned16(grad_loc) || !aligned16(grad_attn))
            return fail(MSDA_B200_INVALID_ARGUMENT, "backward: all tensors must be 16-byte aligned");
    }
    p.value = value;
    p.spatial_shapes = spatial_shapes;
    p.level_start_index = level_start_index;
    p.loc = static_cast<const float *>(loc);
    p.ref = pts.ref;
    p.ref_coords = pts.ref_coords;
    p.offsets16 = pts.offsets16;
    p.attn = attn;
    p.grad_out = grad_out;
    p.grad_value = grad_value;
    p.grad_loc = static_cast<float *>(grad_loc);
    p.grad_attn = grad_attn;
    p.scratch = use_scratch ? scratch : nullptr;
    (void)scratch_adds;   // kept in the signature for callers written against ABI 4; has no effect

    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "backward: selecting the device");
    cudaError_t e;
    if (use_scratch) {
        e = msda_b200::launch_prepare_grad_value(p, dtype, apply_softmax != 0, s);
        if (e != cudaSuccess) return cuda_fail(e, "backward: clearing grad_value / scratch");
    } else if (zero_grad_value && S > 0) {
        e = cudaMemsetAsync(grad_value, 0, (size_t)(B * S * G * D) * element_size(dtype), s);
        if (e != cudaSuccess) return cuda_fail(e, "backward: clearing grad_value");
    }
    if (Q == 0) return MSDA_B200_OK;
    if (dtype == MSDA_B200_F64)
        e = msda_b200::launch_backward_f64(p, apply_softmax != 0, s);
    else
        e = msda_b200::launch_backward(p, dtype, apply_softmax != 0, s);
    if (e != cudaSuccess) return cuda_fail(e, "backward: kernel launch");
    if (use_scratch) {
        e = msda_b200::launch_finalize_grad_value(p, dtype, apply_softmax != 0, s);
        if (e != cudaSuccess) return cuda_fail(e, "backward: converting the scratch image");
    }
    return MSDA_B200_OK;
}

}  // namespace
