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

int element_size(int dtype) { return dtype == MSDA_B200_F32 ? 4 : 2; }

// Shape checks shared by forward, backward and the geometry query; fills the launch plan.
int plan(msda_b200::Params &p, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
         int64_t K, int dtype, bool softmax, bool backward) {
    if (dtype != MSDA_B200_F32 && dtype != MSDA_B200_F16 && dtype != MSDA_B200_BF16)
        return fail(MSDA_B200_INVALID_ARGUMENT, "dtype %d is not f32(0), f16(1) or bf16(2)", dtype);
    if (B < 0 || S < 0 || Q < 0 || G <= 0 || D <= 0 || L <= 0 || K <= 0)
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "sizes must satisfy B,S,Q >= 0 and G,D,L,K > 0 (got B=%lld S=%lld G=%lld "
                    "D=%lld Q=%lld L=%lld K=%lld)",
                    (long long)B, (long long)S, (long long)G, (long long)D, (long long)Q,
                    (long long)L, (long long)K);
    const int vec = 16 / element_size(dtype);
    if (D % vec != 0)
        return fail(MSDA_B200_UNSUPPORTED,
                    "head dimension D=%lld must be a multiple of %d for this dtype (16-byte "
                    "channel vectors)",
                    (long long)D, vec);
    if (L > msda_b200::kMaxLevels)
        return fail(MSDA_B200_UNSUPPORTED, "L=%lld levels exceed the supported %d", (long long)L,
                    msda_b200::kMaxLevels);
    if (S >= (int64_t)1 << 31 || G * D >= (int64_t)1 << 24 || L * K >= (int64_t)1 << 16)
        return fail(MSDA_B200_UNSUPPORTED, "S, G*D or L*K too large for 32-bit tile indexing");

    p.B = B;
    p.S = S;
    p.Q = Q;
    p.G = (int)G;
    p.D = (int)D;
    p.L = (int)L;
    p.K = (int)K;
    int lanes = (int)(D / vec), lg = 0;
    while ((1 << lg) < lanes && lg < 5) ++lg;
    p.lph_log2 = lg;

    // queries per CTA tile: a multiple of 8 keeps every tile's loc/attn slice 16-byte
    // aligned; prefer the largest tile that still lets four CTAs share an SM
    const int64_t per_query = G * L * K * (int64_t)sizeof(float) * ((backward && softmax) ? 4 : 3);
    int tq = 0;
    for (int cand : {32, 24, 16, 8})
        if (cand * per_query <= 56 * 1024) {
            tq = cand;
            break;
        }
    if (tq == 0) {
        if (8 * per_query > 200 * 1024)
            return fail(MSDA_B200_UNSUPPORTED,
                        "G*L*K = %lld does not fit a shared-memory tile of 8 queries",
                        (long long)(G * L * K));
        tq = 8;
    }
    p.tile_queries = tq;
    p.num_tiles = (B * Q + tq - 1) / tq;
    if (p.num_tiles >= (int64_t)1 << 31)
        return fail(MSDA_B200_UNSUPPORTED, "B*Q = %lld needs too many CTAs", (long long)(B * Q));
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

}  // namespace

extern "C" {

int msda_b200_abi_version(void) { return MSDA_B200_ABI_VERSION; }

const char *msda_b200_last_error(void) { return g_error; }

int msda_b200_launch_geometry(int64_t B, int64_t G, int64_t D, int64_t Q, int64_t L, int64_t K,
                              int dtype, int apply_softmax, int64_t *grid, int *tile_queries,
                              int64_t *smem_fwd, int64_t *smem_bwd) {
    msda_b200::Params pf{}, pb{};
    int st = plan(pf, B, 1, G, D, Q, L, K, dtype, apply_softmax != 0, false);
    if (st != MSDA_B200_OK) return st;
    st = plan(pb, B, 1, G, D, Q, L, K, dtype, apply_softmax != 0, true);
    if (st != MSDA_B200_OK) return st;
    if (grid) *grid = pf.num_tiles;
    if (tile_queries) *tile_queries = pf.tile_queries;
    if (smem_fwd) *smem_fwd = (int64_t)msda_b200::forward_smem_bytes(pf);
    if (smem_bwd) *smem_bwd = (int64_t)msda_b200::backward_smem_bytes(pb, apply_softmax != 0);
    return MSDA_B200_OK;
}

int msda_b200_forward(const void *value, const int64_t *spatial_shapes,
                      const int64_t *level_start_index, const float *loc, const void *attn,
                      void *out, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
                      int64_t K, int dtype, int apply_softmax, int device, void *stream) {
    msda_b200::Params p{};
    const int st = plan(p, B, S, G, D, Q, L, K, dtype, apply_softmax != 0, false);
    if (st != MSDA_B200_OK) return st;
    if (B == 0 || Q == 0) return MSDA_B200_OK;
    if (!value || !spatial_shapes || !level_start_index || !loc || !attn || !out)
        return fail(MSDA_B200_INVALID_ARGUMENT, "forward: null pointer argument");
    if (!aligned16(value) || !aligned16(loc) || !aligned16(attn) || !aligned16(out))
        return fail(MSDA_B200_INVALID_ARGUMENT,
                    "forward: value, loc, attn and out must be 16-byte aligned");
    p.value = value;
    p.spatial_shapes = spatial_shapes;
    p.level_start_index = level_start_index;
    p.loc = loc;
    p.attn = attn;
    p.out = out;
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "forward: selecting the device");
    const cudaError_t e =
        msda_b200::launch_forward(p, dtype, apply_softmax != 0, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "forward: kernel launch");
    return MSDA_B200_OK;
}

int msda_b200_backward(const void *value, const int64_t *spatial_shapes,
                       const int64_t *level_start_index, const float *loc, const void *attn,
                       const void *grad_out, void *grad_value, float *grad_loc, void *grad_attn,
                       int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q, int64_t L,
                       int64_t K, int dtype, int apply_softmax, int zero_grad_value, int device,
                       void *stream) {
    msda_b200::Params p{};
    const int st = plan(p, B, S, G, D, Q, L, K, dtype, apply_softmax != 0, true);
    if (st != MSDA_B200_OK) return st;
    if (B == 0) return MSDA_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "backward: selecting the device");
    if (zero_grad_value && S > 0) {
        if (!grad_value) return fail(MSDA_B200_INVALID_ARGUMENT, "backward: grad_value is null");
        const cudaError_t e = cudaMemsetAsync(
            grad_value, 0, (size_t)(B * S * G * D) * element_size(dtype), s);
        if (e != cudaSuccess) return cuda_fail(e, "backward: clearing grad_value");
    }
    if (Q == 0) return MSDA_B200_OK;
    if (!value || !spatial_shapes || !level_start_index || !loc || !attn || !grad_out ||
        !grad_value || !grad_loc || !grad_attn)
        return fail(MSDA_B200_INVALID_ARGUMENT, "backward: null pointer argument");
    if (!aligned16(value) || !aligned16(loc) || !aligned16(attn) || !aligned16(grad_out) ||
        !aligned16(grad_value) || !aligned16(grad_loc) || !aligned16(grad_attn))
        return fail(MSDA_B200_INVALID_ARGUMENT, "backward: all tensors must be 16-byte aligned");
    p.value = value;
    p.spatial_shapes = spatial_shapes;
    p.level_start_index = level_start_index;
    p.loc = loc;
    p.attn = attn;
    p.grad_out = grad_out;
    p.grad_value = grad_value;
    p.grad_loc = grad_loc;
    p.grad_attn = grad_attn;
    const cudaError_t e = msda_b200::launch_backward(p, dtype, apply_softmax != 0, s);
    if (e != cudaSuccess) return cuda_fail(e, "backward: kernel launch");
    return MSDA_B200_OK;
}

}  // extern "C"
