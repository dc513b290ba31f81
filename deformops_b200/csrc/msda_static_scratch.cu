// msda_b200_backward_static_scratch: the backward pass for callers that cannot allocate.
//
// Some hosts of this library have no allocator to offer at the moment they call it: an
// inference or training runtime that carved up all device memory at start-up and forbids
// cudaMalloc afterwards (the call synchronises the whole device and can fail late), a plugin
// that runs inside somebody else's step where any allocator call is off limits, or a plain C
// caller with no caching allocator at hand.  For a 16-bit backward they still need the
// scratch image in which grad_value is accumulated accurately (scaled float16).  This entry
// point brings its own: a fixed array that lives in the library's device image.
//
//  * The array is `kStaticScratchFloats` floats (32 MiB).  Every GPU on which this entry
//    point is used holds those 32 MiB from then until the process exits.
//  * The backward wants msda_b200_backward_scratch_bytes(...) of scratch: 2 bytes per grad_value
//    element, a 256-byte header and a few per cent for the replicas of coarse levels.  Shapes
//    that need more than the 32 MiB (about 14 million grad_value elements for a three-level
//    pyramid with Q = S) are refused with MSDA_B200_UNSUPPORTED; use msda_b200_backward with a
//    caller-owned scratch for those.
//  * Nothing is allocated or freed, here or further down: no cudaMalloc, no cudaFree, no
//    library routine that allocates.  Inputs and outputs are still the caller's buffers.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, once per device, with that device current) and remembers it.
//    Make that first call outside any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left in it.  The
//    rows a call adds into are cleared by its own prepare kernel first, so stale contents
//    never leak into a result - but two calls whose kernels overlap on the GPU (different
//    streams, or different host threads on the same device) race on it.  Serialise them.
//  * Arguments are validated before the array is looked up, so a call that is refused for its
//    shape or dtype never makes a device hold the 32 MiB.
#include <cstdio>
#include <mutex>

#include "../../include/msda_b200.h"
#include "msda_common.cuh"

namespace {

constexpr int64_t kStaticScratchFloats = 8ll * 1024 * 1024;   // 32 MiB
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime, not a device address: handing it
// to a kernel would make the kernel use host memory (or fault).  The address kernels may use
// comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

std::mutex g_setup_mutex;
float *g_scratch_address[kMaxDevices] = {};   // per device, filled on first use

// Device address of the array on `device`, looked up once with that device current.
cudaError_t scratch_address(int device, float **out) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        int previous = -1;
        cudaError_t e = cudaGetDevice(&previous);
        if (e != cudaSuccess) return e;
        if (previous != device && (e = cudaSetDevice(device)) != cudaSuccess) return e;
        float *address = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&address), g_static_scratch);
        if (previous != device) cudaSetDevice(previous);
        if (e != cudaSuccess) return e;
        g_scratch_address[device] = address;
    }
    *out = g_scratch_address[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int msda_b200_backward_static_scratch(
    const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
    const float *loc, const void *attn, const void *grad_out, void *grad_value, float *grad_loc,
    void *grad_attn, int64_t scratch_adds, int64_t B, int64_t S, int64_t G, int64_t D, int64_t Q,
    int64_t L, int64_t K, int dtype, int apply_softmax, int device, void *stream) {
    char message[256];
    // shape / dtype checks first (they set the error message themselves)
    const int valid = msda_b200_launch_geometry(B, G, D, Q, L, K, dtype, apply_softmax, nullptr,
                                                nullptr, nullptr, nullptr);
    if (valid != MSDA_B200_OK) return valid;
    const int64_t need = msda_b200_backward_scratch_bytes(B, S, G, D, Q, L, K, dtype);
    if (need > kStaticScratchFloats * (int64_t)sizeof(float)) {
        snprintf(message, sizeof(message),
                 "backward_static_scratch: B*S*G*D = %lld elements need %lld bytes of scratch and exceed the "
                 "built-in scratch of 32 MiB; call msda_b200_backward with a scratch buffer of "
                 "your own",
                 (long long)(B * S * G * D), (long long)need);
        return msda_b200::set_last_error(MSDA_B200_UNSUPPORTED, message);
    }
    float *scratch = nullptr;
    if (need > 0) {
        int dev = device;
        if (dev < 0) {
            const cudaError_t e = cudaGetDevice(&dev);
            if (e != cudaSuccess) {
                snprintf(message, sizeof(message), "backward_static_scratch: cudaGetDevice: %s",
                         cudaGetErrorString(e));
                return msda_b200::set_last_error(MSDA_B200_CUDA_ERROR, message);
            }
        }
        if (dev >= kMaxDevices)
            return msda_b200::set_last_error(MSDA_B200_UNSUPPORTED,
                                             "backward_static_scratch: device index above 63");
        const cudaError_t e = scratch_address(dev, &scratch);
        if (e != cudaSuccess) {
            snprintf(message, sizeof(message),
                     "backward_static_scratch: cudaGetSymbolAddress on device %d: %s (%s)", dev,
                     cudaGetErrorName(e), cudaGetErrorString(e));
            return msda_b200::set_last_error(MSDA_B200_CUDA_ERROR, message);
        }
    }
    // same code path as the caller-scratch entry point from here on; it clears the header and
    // the image this call accumulates into before adding anything
    return msda_b200_backward(value, spatial_shapes, level_start_index, loc, attn, grad_out,
                              grad_value, grad_loc, grad_attn, scratch,
                              scratch ? kStaticScratchFloats * (int64_t)sizeof(float) : 0,
                              scratch_adds, B, S, G, D, Q, L, K, dtype, apply_softmax,
                              /*zero_grad_value=*/1, device, stream);
}
