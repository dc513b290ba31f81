// Backward kernel: scatters grad_value and reduces grad_loc / grad_attn with no
// intermediate sampling buffer in global memory.
//
// Replaces the reference's backward path
//   sources/deformops/backends/cuda/include/msda_backward.cuh:14-240 (kernel)
//   sources/deformops/backends/cuda/include/interpolate.cuh:78-218   (scatter + gradients)
//   sources/deformops/backends/cuda/include/utils.cuh:172-220         (softmax Jacobian, reductions)
// with a design of its own:
//  * the tile's locations and weights are staged in shared memory once (coalesced,
//    streaming); the same shared tile later carries grad_loc / grad_attn, which leave
//    the CTA as coalesced 16-byte streaming stores;
//  * every lane owns 16 bytes of channels, reloads the four corners with one 16-byte
//    load each, and issues ONE 16-byte packed reduction per corner
//    (red.global.add.noftz.v4.bf16x2 / .v4.f16x2 / .v4.f32) into grad_value - lanes of
//    a warp instruction always target distinct (pixel, head, channel-group) addresses;
//  * the three per-point scalars (d/dx, d/dy, d/da) come from four corner dot products
//    and are reduced over the LPH lanes of a slot with xor shuffles;
//  * softmax weights are normalised in shared memory and the softmax Jacobian is applied
//    as p_i * (g_i - sum_j p_j g_j), one thread per (query, head) pair.
#include "msda_common.cuh"

namespace msda_b200 {

namespace {

template <typename T, int KT, bool SOFTMAX>
__global__ void __launch_bounds__(kThreads, 3) backward_kernel(const Params p) {
    using VT = VecTraits<T>;
    constexpr int V = VT::kVec;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ LevelTable lt;

    const int G = p.G, D = p.D, L = p.L;
    const int K = KT > 0 ? KT : p.K;
    const int P = L * K;
    const int TQ = p.tile_queries;
    float *sLoc = reinterpret_cast<float *>(smem_raw);   // in: loc, out: grad_loc   [pair][P][2]
    float *sAttn = sLoc + (size_t)TQ * G * P * 2;         // weights / probabilities [pair][P]
    // gradient w.r.t. the (normalised) weights; aliases sAttn when there is no softmax
    float *sGrad = SOFTMAX ? sAttn + (size_t)TQ * G * P : sAttn;

    load_level_table(lt, p);

    const int64_t total_q = p.B * p.Q;
    const int64_t bq0 = (int64_t)blockIdx.x * TQ;
    const int nq = (int)min((int64_t)TQ, total_q - bq0);
    const int npairs = nq * G;

    stage_f32(sLoc, p.loc + bq0 * G * P * 2, npairs * P * 2);
    stage_as_f32<T>(sAttn, reinterpret_cast<const T *>(p.attn) + bq0 * G * P, npairs * P);
    __syncthreads();

    if constexpr (SOFTMAX) {
        for (int pair = threadIdx.x; pair < npairs; pair += kThreads) {
            float *a = sAttn + pair * P;
            float m = -INFINITY;
            for (int i = 0; i < P; ++i) m = fmaxf(m, a[i]);
            float sum = 0.f;
            for (int i = 0; i < P; ++i) {
                const float e = expf(a[i] - m);
                a[i] = e;
                sum += e;
            }
            const float inv = 1.f / sum;
            for (int i = 0; i < P; ++i) a[i] *= inv;
        }
        __syncthreads();
    }

    const int lph = 1 << p.lph_log2;
    const int slot = threadIdx.x >> p.lph_log2;
    const int sub = threadIdx.x & (lph - 1);
    const int nslots = kThreads >> p.lph_log2;
    const int GD = G * D;
    const T *value = reinterpret_cast<const T *>(p.value);
    const T *grad_out = reinterpret_cast<const T *>(p.grad_out);
    T *grad_value = reinterpret_cast<T *>(p.grad_value);
    const int ch0 = sub * V;

    // warp-uniform trip count: every lane takes part in the shuffles of every iteration
    for (int base = 0; base < npairs; base += nslots) {
        const bool live = base + slot < npairs;
        const int pair = live ? base + slot : npairs - 1;
        const int64_t bq = bq0 + pair / G;
        const int g = pair % G;
        const int64_t b = bq / p.Q;
        float2 *pl = reinterpret_cast<float2 *>(sLoc) + pair * P;
        const float *pa = sAttn + pair * P;
        float *pg = sGrad + pair * P;
        const int64_t sample_base = (b * p.S * G + g) * (int64_t)D;
        const T *go_row = grad_out + (bq * G + g) * (int64_t)D;

        float2 go0[V / 2];  // this lane's first (usually only) channel vector of grad_out
        {
            float f[V];
#pragma unroll
            for (int i = 0; i < V; ++i) f[i] = 0.f;
            if (live && ch0 < D) VT::unpack(ld_stream16(go_row + ch0), f);
#pragma unroll
            for (int i = 0; i < V / 2; ++i) go0[i] = make_float2(f[2 * i], f[2 * i + 1]);
        }

        auto point = [&](int l, int H, int W, int pt) {
            const float2 xy = pl[pt];
            const float a = pa[pt];
            const Corners c = locate(xy.x, xy.y, H, W);
            const int64_t level_base = sample_base + (int64_t)lt.start[l] * GD;
            float dot[4] = {0.f, 0.f, 0.f, 0.f};
            for (int ch = ch0; ch < D; ch += lph * V) {
                float2 go[V / 2];
                if (ch == ch0) {
#pragma unroll
                    for (int i = 0; i < V / 2; ++i) go[i] = go0[i];
                } else {
                    float f[V];
                    VT::unpack(ld_stream16(go_row + ch), f);
#pragma unroll
                    for (int i = 0; i < V / 2; ++i) go[i] = make_float2(f[2 * i], f[2 * i + 1]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (c.ok[j] && live) {
                        const int64_t idx = level_base + (int64_t)c.off[j] * GD + ch;
                        float f[V];
                        VT::unpack(ldg16(value + idx), f);
                        float2 d2 = make_float2(0.f, 0.f);
                        const float s = a * c.w[j];
                        const float2 s2 = make_float2(s, s);
                        float gv[V];
#pragma unroll
                        for (int i = 0; i < V / 2; ++i) {
                            ffma2(d2, make_float2(f[2 * i], f[2 * i + 1]), go[i]);
                            const float2 t = fmul2(go[i], s2);
                            gv[2 * i] = t.x;
                            gv[2 * i + 1] = t.y;
                        }
                        dot[j] += d2.x + d2.y;
                        VT::red_add(grad_value + idx, gv);
                    }
                }
            }
            // d/dx, d/dy inside the cell [floor, floor+1), d/da = sampled value . grad_out
            float gx = (1.f - c.fr) * (dot[1] - dot[0]) + c.fr * (dot[3] - dot[2]);
            float gy = (1.f - c.fc) * (dot[2] - dot[0]) + c.fc * (dot[3] - dot[1]);
            float ga = c.w[0] * dot[0] + c.w[1] * dot[1] + c.w[2] * dot[2] + c.w[3] * dot[3];
            for (int o = lph >> 1; o > 0; o >>= 1) {
                gx += __shfl_xor_sync(0xffffffffu, gx, o);
                gy += __shfl_xor_sync(0xffffffffu, gy, o);
                ga += __shfl_xor_sync(0xffffffffu, ga, o);
            }
            if (sub == 0 && live) {
                // skipped points get exact zeros, whatever their weight holds
                pl[pt] = c.inside ? make_float2((float)W * a * gx, (float)H * a * gy)
                                  : make_float2(0.f, 0.f);
                pg[pt] = c.inside ? ga : 0.f;
            }
        };

        for (int l = 0; l < L; ++l) {
            const int H = lt.H[l], W = lt.W[l];
            if constexpr (KT > 0) {
#pragma unroll
                for (int k = 0; k < KT; ++k) point(l, H, W, l * KT + k);
            } else {
                for (int k = 0; k < K; ++k) point(l, H, W, l * K + k);
            }
        }
    }
    __syncthreads();

    if constexpr (SOFTMAX) {
        for (int pair = threadIdx.x; pair < npairs; pair += kThreads) {
            const float *pr = sAttn + pair * P;
            float *g = sGrad + pair * P;
            float inner = 0.f;
            for (int i = 0; i < P; ++i) inner += pr[i] * g[i];
            for (int i = 0; i < P; ++i) g[i] = pr[i] * (g[i] - inner);
        }
        __syncthreads();
    }

    // coalesced write-out of the tile's grad_loc (float32) and grad_attn (T)
    {
        const int n = npairs * P * 2;
        float *dst = p.grad_loc + bq0 * G * P * 2;
        const int n4 = n >> 2;
        for (int i = threadIdx.x; i < n4; i += kThreads)
            st_stream16(reinterpret_cast<uint4 *>(dst) + i, reinterpret_cast<const uint4 *>(sLoc)[i]);
        for (int i = (n4 << 2) + threadIdx.x; i < n; i += kThreads) dst[i] = sLoc[i];
    }
    {
        const int n = npairs * P;
        T *dst = reinterpret_cast<T *>(p.grad_attn) + bq0 * G * P;
        const int nv = n / V;
        for (int i = threadIdx.x; i < nv; i += kThreads) {
            float f[V];
#pragma unroll
            for (int j = 0; j < V; ++j) f[j] = sGrad[i * V + j];
            st_stream16(reinterpret_cast<uint4 *>(dst) + i, VT::pack(f));
        }
        for (int i = nv * V + threadIdx.x; i < n; i += kThreads) dst[i] = VT::from_float(sGrad[i]);
    }
}

template <typename T, bool SOFTMAX>
cudaError_t launch_typed(const Params &p, cudaStream_t stream) {
    const size_t smem = backward_smem_bytes(p, SOFTMAX);
    auto go = [&](auto kernel) -> cudaError_t {
        if (smem > 48 * 1024) {  // opt in to large dynamic shared memory only when needed
            cudaError_t e = cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        kernel<<<(unsigned)p.num_tiles, kThreads, smem, stream>>>(p);
        return cudaGetLastError();
    };
    switch (p.K) {
        case 4: return go(backward_kernel<T, 4, SOFTMAX>);
        case 8: return go(backward_kernel<T, 8, SOFTMAX>);
        default: return go(backward_kernel<T, 0, SOFTMAX>);
    }
}

}  // namespace

size_t backward_smem_bytes(const Params &p, bool softmax) {
    return (size_t)p.tile_queries * p.G * p.L * p.K * (softmax ? 4 : 3) * sizeof(float);
}

cudaError_t launch_backward(const Params &p, int dtype, bool softmax, cudaStream_t stream) {
    switch (dtype) {
        case 0:
            return softmax ? launch_typed<float, true>(p, stream)
                           : launch_typed<float, false>(p, stream);
        case 1:
            return softmax ? launch_typed<__half, true>(p, stream)
                           : launch_typed<__half, false>(p, stream);
        case 2:
            return softmax ? launch_typed<__nv_bfloat16, true>(p, stream)
                           : launch_typed<__nv_bfloat16, false>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda_b200
