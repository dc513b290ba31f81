// float64 kernels: value, locations, weights and all gradients in double precision.
//
// The reference's CUDA operator accepts float64 values with float64 locations
// (sources/deformops/backends/cuda/include/msda_launch.cuh:54-61, :185-187) so that
// torch.autograd.gradcheck can differentiate it numerically.  That is this file's only job:
// the kernels are written for exactness and simplicity, not for throughput.  One warp owns a
// (query, head) pair; lanes stride over the D channels; every quantity is a double; the
// reductions into grad_value are native double atomics; grad_loc and grad_attn have exactly one
// writer per element.  Semantics are those of the 16/32-bit kernels: pixel = loc * size - 0.5,
// a point is skipped unless -1 <= pixel < size on both axes, corners outside the level
// contribute zero, the softmax denominator includes skipped points.
#include "msda_common.cuh"

namespace msda_b200 {

namespace {

constexpr int kThreadsF64 = 256;

struct Levels64 {
    int H[kMaxLevels], W[kMaxLevels], start[kMaxLevels];
};

// a level that does not lie inside the value tensor becomes an empty level (all points skipped)
__device__ __forceinline__ void load_levels(Levels64 &t, const Params &p) {
    if (threadIdx.x < p.L) {
        const int64_t h = p.spatial_shapes[2 * threadIdx.x];
        const int64_t w = p.spatial_shapes[2 * threadIdx.x + 1];
        const int64_t first = p.level_start_index[threadIdx.x];
        const bool fits = h > 0 && w > 0 && first >= 0 && h <= p.S && w <= p.S &&
                          h * w <= p.S && first <= p.S - h * w;
        t.H[threadIdx.x] = fits ? (int)h : 0;
        t.W[threadIdx.x] = fits ? (int)w : 0;
        t.start[threadIdx.x] = fits ? (int)first : 0;
    }
    __syncthreads();
}

struct Point64 {
    bool inside;
    bool ok[4];          // corner (r0,c0), (r0,c0+1), (r0+1,c0), (r0+1,c0+1) lies inside the level
    int64_t off[4];      // element offset of each corner's channel 0 inside the sample
    double fr, fc;
};

__device__ __forceinline__ Point64 locate64(double x, double y, int H, int W, int start, int GD) {
    Point64 g;
    const double px = x * (double)W - 0.5, py = y * (double)H - 0.5;
    g.inside = (py >= -1.0) && (px >= -1.0) && (py < (double)H) && (px < (double)W) && H > 0;
    const double sx = g.inside ? px : 0.0, sy = g.inside ? py : 0.0;
    const double r0f = floor(sy), c0f = floor(sx);
    const int r0 = (int)r0f, c0 = (int)c0f;
    g.fr = sy - r0f;
    g.fc = sx - c0f;
    const bool r_ok[2] = {r0 >= 0, r0 + 1 < H}, c_ok[2] = {c0 >= 0, c0 + 1 < W};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        g.ok[i] = g.inside && r_ok[i >> 1] && c_ok[i & 1];
        g.off[i] = ((int64_t)start + (int64_t)(r0 + (i >> 1)) * W + (c0 + (i & 1))) * GD;
    }
    return g;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// (max, 1 / sum exp(logit - max)) of a pair's P logits, computed by every lane alike
__device__ __forceinline__ void softmax_stats64(const double *logits, int P, double &m, double &inv) {
    m = -INFINITY;
    for (int i = 0; i < P; ++i) m = fmax(m, logits[i]);
    double s = 0.0;
    for (int i = 0; i < P; ++i) s += exp(logits[i] - m);
    inv = 1.0 / s;
}

template <bool SOFTMAX>
__global__ void __launch_bounds__(kThreadsF64) forward_f64_kernel(const Params p) {
    __shared__ Levels64 lt;
    load_levels(lt, p);
    const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int G = p.G, D = p.D, K = p.K, P = p.L * p.K, GD = p.G * p.D;
    const double *value = static_cast<const double *>(p.value);
    const double *attn = static_cast<const double *>(p.attn);
    const double *loc = reinterpret_cast<const double *>(p.loc);
    double *out = static_cast<double *>(p.out);
    const int64_t pairs = p.B * p.Q * G;
    for (int64_t pair = (int64_t)blockIdx.x * nwarps + (threadIdx.x >> 5); pair < pairs;
         pair += (int64_t)gridDim.x * nwarps) {
        const int64_t bq = pair / G;
        const int g = (int)(pair - bq * G);
        const double *vb = value + ((bq / p.Q) * p.S * G + g) * (int64_t)D;
        double m = 0.0, inv = 1.0;
        if (SOFTMAX) softmax_stats64(attn + pair * P, P, m, inv);
        for (int d0 = 0; d0 < D; d0 += 32) {
            const int d = d0 + lane;
            double acc = 0.0;
            for (int pt = 0; pt < P; ++pt) {
                const int l = pt / K;
                const int64_t e = pair * P + pt;
                double a = attn[e];
                if (SOFTMAX) a = exp(a - m) * inv;
                const Point64 geo =
                    locate64(loc[2 * e], loc[2 * e + 1], lt.H[l], lt.W[l], lt.start[l], GD);
                if (!geo.inside || d >= D) continue;
                const double w[4] = {(1.0 - geo.fr) * (1.0 - geo.fc), (1.0 - geo.fr) * geo.fc,
                                     geo.fr * (1.0 - geo.fc), geo.fr * geo.fc};
                double s = 0.0;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (geo.ok[c]) s += w[c] * vb[geo.off[c] + d];
                acc += a * s;
            }
            if (d < D) out[pair * D + d] = acc;
        }
    }
}

template <bool SOFTMAX>
__global__ void __launch_bounds__(kThreadsF64) backward_f64_kernel(const Params p) {
    __shared__ Levels64 lt;
    load_levels(lt, p);
    const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int G = p.G, D = p.D, K = p.K, P = p.L * p.K, GD = p.G * p.D;
    const double *value = static_cast<const double *>(p.value);
    const double *attn = static_cast<const double *>(p.attn);
    const double *loc = reinterpret_cast<const double *>(p.loc);
    const double *grad_out = static_cast<const double *>(p.grad_out);
    double *grad_value = static_cast<double *>(p.grad_value);
    double *grad_loc = reinterpret_cast<double *>(p.grad_loc);
    double *grad_attn = static_cast<double *>(p.grad_attn);
    const int64_t pairs = p.B * p.Q * G;
    for (int64_t pair = (int64_t)blockIdx.x * nwarps + (threadIdx.x >> 5); pair < pairs;
         pair += (int64_t)gridDim.x * nwarps) {
        const int64_t bq = pair / G;
        const int g = (int)(pair - bq * G);
        const int64_t sample = ((bq / p.Q) * p.S * G + g) * (int64_t)D;
        const double *go = grad_out + pair * D;
        double m = 0.0, inv = 1.0;
        if (SOFTMAX) softmax_stats64(attn + pair * P, P, m, inv);
        double inner = 0.0;      // softmax: sum_j p_j * dL/dp_j (the same in every lane)
        for (int pt = 0; pt < P; ++pt) {
            const int l = pt / K;
            const int64_t e = pair * P + pt;
            double a = attn[e];
            if (SOFTMAX) a = exp(a - m) * inv;
            const Point64 geo =
                locate64(loc[2 * e], loc[2 * e + 1], lt.H[l], lt.W[l], lt.start[l], GD);
            double dot_a = 0.0, dot_x = 0.0, dot_y = 0.0;
            if (geo.inside) {
                const double w[4] = {(1.0 - geo.fr) * (1.0 - geo.fc), (1.0 - geo.fr) * geo.fc,
                                     geo.fr * (1.0 - geo.fc), geo.fr * geo.fc};
                for (int d = lane; d < D; d += 32) {
                    const double gd = go[d];
                    double v[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        v[c] = geo.ok[c] ? value[sample + geo.off[c] + d] : 0.0;
                        if (geo.ok[c]) atomicAdd(grad_value + sample + geo.off[c] + d, gd * a * w[c]);
                    }
                    dot_a += gd * (w[0] * v[0] + w[1] * v[1] + w[2] * v[2] + w[3] * v[3]);
                    dot_x += gd * ((1.0 - geo.fr) * (v[1] - v[0]) + geo.fr * (v[3] - v[2]));
                    dot_y += gd * ((1.0 - geo.fc) * (v[2] - v[0]) + geo.fc * (v[3] - v[1]));
                }
            }
            dot_a = warp_sum(dot_a);
            dot_x = warp_sum(dot_x);
            dot_y = warp_sum(dot_y);
            inner += a * dot_a;
            if (lane == 0) {
                // a skipped point gets exact zeros whatever its weight holds
                grad_loc[2 * e] = geo.inside ? (double)lt.W[l] * a * dot_x : 0.0;
                grad_loc[2 * e + 1] = geo.inside ? (double)lt.H[l] * a * dot_y : 0.0;
                grad_attn[e] = dot_a;        // softmax: dL/dp for now, finished below
            }
        }
        if (SOFTMAX) {
            __syncwarp();
            for (int pt = lane; pt < P; pt += 32) {
                const int64_t e = pair * P + pt;
                const double prob = exp(attn[e] - m) * inv;
                grad_attn[e] = prob * (grad_attn[e] - inner);
            }
        }
    }
}

unsigned grid_for(const Params &p) {
    const int64_t pairs = p.B * p.Q * p.G;
    const int64_t blocks = (pairs + kThreadsF64 / 32 - 1) / (kThreadsF64 / 32);
    return (unsigned)(blocks > 148 * 64 ? 148 * 64 : (blocks > 0 ? blocks : 1));
}

}  // namespace

cudaError_t launch_forward_f64(const Params &p, bool softmax, cudaStream_t stream) {
    if (softmax)
        forward_f64_kernel<true><<<grid_for(p), kThreadsF64, 0, stream>>>(p);
    else
        forward_f64_kernel<false><<<grid_for(p), kThreadsF64, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_backward_f64(const Params &p, bool softmax, cudaStream_t stream) {
    if (softmax)
        backward_f64_kernel<true><<<grid_for(p), kThreadsF64, 0, stream>>>(p);
    else
        backward_f64_kernel<false><<<grid_for(p), kThreadsF64, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace msda_b200
