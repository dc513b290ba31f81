// Forward kernel: out[b,q,g,:] = sum_{l,k} a[l,k] * bilinear(value_l, loc[l,k]).
//
// Replaces the reference's forward path
//   sources/deformops/backends/cuda/include/msda_forward.cuh:13-123 (kernel)
//   sources/deformops/backends/cuda/include/interpolate.cuh:14-72   (bilinear gather)
// with a design of its own: one CTA stages the sampling locations and weights of a tile
// of queries in shared memory with coalesced 16-byte streaming loads (each is read from
// HBM exactly once), then every slot of LPH lanes walks the points of one (query, head)
// pair and gathers the four bilinear corners with one 16-byte load per lane along the
// head dimension, accumulating in float32 with packed f32x2 FMAs.
#include "msda_common.cuh"

namespace msda_b200 {

namespace {

template <typename T, int KT, bool SOFTMAX>
__global__ void __launch_bounds__(kThreads, 4) forward_kernel(const Params p) {
    using VT = VecTraits<T>;
    constexpr int V = VT::kVec;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ LevelTable lt;

    const int G = p.G, D = p.D, L = p.L;
    const int K = KT > 0 ? KT : p.K;
    const int P = L * K;
    const int TQ = p.tile_queries;
    float *sLoc = reinterpret_cast<float *>(smem_raw);   // [pair][P][2]
    float *sAttn = sLoc + (size_t)TQ * G * P * 2;         // [pair][P]

    load_level_table(lt, p);

    const int64_t total_q = p.B * p.Q;
    const int64_t bq0 = (int64_t)blockIdx.x * TQ;
    const int nq = (int)min((int64_t)TQ, total_q - bq0);
    const int npairs = nq * G;

    stage_f32(sLoc, p.loc + bq0 * G * P * 2, npairs * P * 2);
    stage_as_f32<T>(sAttn, reinterpret_cast<const T *>(p.attn) + bq0 * G * P, npairs * P);
    __syncthreads();

    if constexpr (SOFTMAX) {
        // normalise each pair's L*K logits in place; skipped points stay in the denominator
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
    T *out = reinterpret_cast<T *>(p.out);

    for (int pair = slot; pair < npairs; pair += nslots) {
        const int64_t bq = bq0 + pair / G;
        const int g = pair % G;
        const int64_t b = bq / p.Q;
        const float2 *pl = reinterpret_cast<const float2 *>(sLoc) + pair * P;
        const float *pa = sAttn + pair * P;
        for (int ch = sub * V; ch < D; ch += lph * V) {
            float2 acc[V / 2];
#pragma unroll
            for (int i = 0; i < V / 2; ++i) acc[i] = make_float2(0.f, 0.f);
            const T *vb = value + (b * p.S * G + g) * (int64_t)D + ch;
            auto sample_point = [&](const T *vl, int H, int W, int pt) {
                const float2 xy = pl[pt];
                const float a = pa[pt];
                const Corners c = locate(xy.x, xy.y, H, W);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (c.ok[j]) {
                        float f[V];
                        VT::unpack(ldg16(vl + (int64_t)c.off[j] * GD), f);
                        const float wa = a * c.w[j];
                        const float2 wa2 = make_float2(wa, wa);
#pragma unroll
                        for (int i = 0; i < V / 2; ++i)
                            ffma2(acc[i], make_float2(f[2 * i], f[2 * i + 1]), wa2);
                    }
                }
            };
            for (int l = 0; l < L; ++l) {
                const int H = lt.H[l], W = lt.W[l];
                const T *vl = vb + (int64_t)lt.start[l] * GD;
                if constexpr (KT > 0) {
#pragma unroll
                    for (int k = 0; k < KT; ++k) sample_point(vl, H, W, l * KT + k);
                } else {
                    for (int k = 0; k < K; ++k) sample_point(vl, H, W, l * K + k);
                }
            }
            float r[V];
#pragma unroll
            for (int i = 0; i < V / 2; ++i) {
                r[2 * i] = acc[i].x;
                r[2 * i + 1] = acc[i].y;
            }
            st_stream16(out + (bq * G + g) * (int64_t)D + ch, VT::pack(r));
        }
    }
}

template <typename T, bool SOFTMAX>
cudaError_t launch_typed(const Params &p, cudaStream_t stream) {
    const size_t smem = forward_smem_bytes(p);
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
        case 4: return go(forward_kernel<T, 4, SOFTMAX>);
        case 8: return go(forward_kernel<T, 8, SOFTMAX>);
        default: return go(forward_kernel<T, 0, SOFTMAX>);
    }
}

}  // namespace

size_t forward_smem_bytes(const Params &p) {
    return (size_t)p.tile_queries * p.G * p.L * p.K * 3 * sizeof(float);
}

cudaError_t launch_forward(const Params &p, int dtype, bool softmax, cudaStream_t stream) {
    switch (dtype) {
        case 0:
            return softmax ? launch_typed<float, true>(p, stream) : launch_typed<float, false>(p, stream);
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
