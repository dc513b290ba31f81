// Backward kernels: scatter grad_value and reduce grad_loc / grad_attn with no
// intermediate sampling buffer in global memory.
//
// Replaces the reference's backward path
//   sources/deformops/backends/cuda/include/msda_backward.cuh:14-240 (kernel)
//   sources/deformops/backends/cuda/include/interpolate.cuh:78-218   (scatter + gradients)
//   sources/deformops/backends/cuda/include/utils.cuh:172-220         (softmax Jacobian, reductions)
//   sources/deformops/backends/cuda/include/msda_launch.cuh:188-197,252-273 (scratch, cast-back)
// with a design of its own.  A warp owns a group of 32/LPH (query, head) pairs:
//  * pre-pass as in the forward kernel: one lane per point builds a 32-byte descriptor
//    (corner offset, row stride, flags, weight a, fractions, a*W, a*H) in shared memory;
//  * every lane owns 16 bytes of channels, reloads the four corners (predicated 16-byte
//    loads), forms four corner dot products with grad_out and issues ONE 16-byte packed
//    reduction per corner into grad_value (red.global.add.noftz.v4.bf16x2 / .v4.f16x2 /
//    .v4.f32); lanes of one warp instruction always target distinct addresses;
//  * d/dx, d/dy, d/da follow from the four dots and are reduced over the slot's lanes with
//    xor shuffles; they are staged in shared memory and leave the warp as contiguous
//    streaming stores (grad_loc float32, grad_attn in T);
//  * softmax: weights are normalised in the pre-pass and the Jacobian is applied as
//    p_i * (g_i - sum_j p_j g_j) before the store.
//
// Accuracy of 16-bit grad_value.  A coarse pyramid level receives hundreds of additions per
// element; summing those in bf16 loses about sqrt(n) * 2^-9 of the result.  With a scratch
// buffer the contributions are therefore scaled by a power of two and added in float16 into an
// image held in the scratch (see "Scaled float16 accumulation" in msda_common.cuh); a level
// that receives more than 256 additions per element gets extra replicas of itself there.
// prepare_kernel clears what is added into and finds the magnitudes the scale is derived from,
// finalize_kernel sums the replicas, unscales and writes grad_value in its own type.
#include <type_traits>

#include "msda_common.cuh"

// What bounds this kernel on B200 is not arithmetic and not DRAM but each SM's request path to
// L2, which the gather's L1 misses share with the reductions: a kernel that issues nothing but
// this kernel's reductions takes 0.40 ms at the headline shape, one that gathers every row and
// then adds into it 0.46 ms (csrc/floors/bench_floors.cu), this one 0.47 ms.
//
// tuning knobs (compile-time): points in flight together and CTAs per SM the registers allow.
// Measured on B200 at the headline shape (backward call, ms, with an earlier accumulation scheme
// whose extra passes cost 0.04 ms more than today's; the order is what matters): unroll 2 / 4
// CTAs 0.583, 3 / 4 0.585, 1 / 4 0.593, 1 / 3 0.604, 2 / 3 0.605, 4 / 4 0.680, 1 / 5 0.815.
//
// The two sweep kernels around the backward kernel (prepare, finalize): CTAs of the grid per SM,
// vectors a finalize thread has in flight, and the residency the register allocation is held
// to.  Measured on B200 at the headline shape (backward call, ms): prepare's grid and finalize's
// vectors are flat (8..32 CTAs per SM, 2..8 vectors); registers are not - prepare left alone
// takes 87 registers and costs 0.014 ms more than at 56, held to 32 it gains another 0.002;
// finalize held to 64 registers gains 0.004 over 72 (0.5250 -> 0.5192 together) - and finalize
// wants exactly the CTAs that fit at once: one wave of four per SM 0.5138, three 0.5169, sixteen
// (two waves, each thread paying its set-up for a quarter of the vectors) 0.5181.
#ifndef MSDA_PREP_CTAS_PER_SM
#define MSDA_PREP_CTAS_PER_SM 16
#endif
#ifndef MSDA_FIN_CTAS_PER_SM
#define MSDA_FIN_CTAS_PER_SM 4
#endif
#ifndef MSDA_FIN_VECS
#define MSDA_FIN_VECS 4
#endif
#ifndef MSDA_FIN_MIN_CTAS
#define MSDA_FIN_MIN_CTAS 4
#endif
#ifndef MSDA_PREP_MIN_CTAS
#define MSDA_PREP_MIN_CTAS 8
#endif
#ifndef MSDA_BWD_UNROLL
#define MSDA_BWD_UNROLL 2
#endif
#ifndef MSDA_BWD_MIN_CTAS
#define MSDA_BWD_MIN_CTAS 4
#endif

namespace msda_b200 {

namespace {

// SCALED: grad_value contributions go, times 2^e, into the float16 image of the scratch
template <typename T, bool SOFTMAX, bool SCALED>
__global__ void __launch_bounds__(256, MSDA_BWD_MIN_CTAS) backward_kernel(const Params p) {
    using VT = VecTraits<T>;
    constexpr int V = VT::kVec;
    constexpr int NV2 = V / 2;
    constexpr int kUnroll = MSDA_BWD_UNROLL;
    extern __shared__ uint4 smem[];
    __shared__ LevelTable lt;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int lph = 1 << p.lph_log2;
    const int ppw = 32 >> p.lph_log2;
    const int PC = p.point_chunk;
    const int DS = 2 * PC + 1;                 // uint4 stride between slots (odd: no bank conflicts)
    const int G = p.G, D = p.D, K = p.K;
    const int P = p.L * K;
    const int GD = G * D;
    const float inv_K = 1.f / (float)K;
    const float inv_P = 1.f / (float)P;

    // per-warp shared memory: descriptors, then staged gradients of the whole group
    uint4 *desc = smem + (size_t)warp * desc_warp_vec(ppw, PC);
    const int stage_floats = backward_stage_floats(ppw, P, SOFTMAX);
    float *stage = reinterpret_cast<float *>(smem + (size_t)nwarps * desc_warp_vec(ppw, PC)) +
                   (size_t)warp * stage_floats;
    float2 *s_stats = reinterpret_cast<float2 *>(stage);         // [32] softmax (max, 1/sum)
    float2 *s_gloc = s_stats + 32;                               // [ppw*P] (dx, dy)
    float *s_gatt = stage + 64 + ppw * P * 2;                    // [ppw*P] d/d(weight)
    float *s_prob = s_gatt + ppw * P;                            // [ppw*P] softmax only

    load_level_table(lt, p);
    __syncthreads();
    // everything above reads the caller's tables only; the scratch header and image below are
    // written by the kernel before this one
    grid_dependency_wait();
    grid_launch_dependents();
    float scale = 1.f;
    if constexpr (SCALED) {
        scale = ldexpf(1.f, grad_scale_exponent<T>(reinterpret_cast<const unsigned *>(p.scratch),
                                                   p.Q, K, SOFTMAX));
        if (threadIdx.x == 0) plan_replicas(lt, p);
        __syncthreads();
    }

    const int64_t total_pairs = p.B * p.Q * G;
    const int slot = lane >> p.lph_log2;
    const int sub = lane & (lph - 1);
    const T *value = reinterpret_cast<const T *>(p.value);
    const T *attn = reinterpret_cast<const T *>(p.attn);
    const T *grad_out = reinterpret_cast<const T *>(p.grad_out);
    // where the packed reductions go: grad_value itself, or the float16 image in the scratch
    using RT = typename std::conditional<SCALED, __half, T>::type;
    RT *red_base = SCALED ? reinterpret_cast<RT *>(reinterpret_cast<char *>(p.scratch) +
                                                   kScratchHeaderBytes)
                          : reinterpret_cast<RT *>(p.grad_value);
    RT *extras = red_base + p.B * p.S * (int64_t)GD;     // SCALED only: replicas of coarse levels
    const int64_t extra_sample = extra_elems_per_sample(p.Q, G, D, p.L, K);

    // A CTA walks `passes` ADJACENT sets of nwarps groups; the grid covers every group.  (A
    // grid-stride loop here cost registers the kernel does not have: 0.617 ms per call with it
    // against 0.583 ms in this form.  The register allocation at 64 registers is sensitive to
    // the shape of this loop: check `-Xptxas -v` for spills after touching it.)
    const int passes = p.passes > 1 ? p.passes : 1;
    for (int pass = 0; pass < passes; ++pass) {
        const int64_t group = ((int64_t)blockIdx.x * passes + pass) * nwarps + warp;
        if (group >= p.num_groups) break;
        const int64_t pair0 = group * ppw;
        const int nlive = (int)min((int64_t)ppw, total_pairs - pair0);
        if constexpr (SOFTMAX) {
            if (lane < nlive) s_stats[lane] = softmax_stats(attn + (pair0 + lane) * P, P);
            __syncwarp();
        }
        const bool live = slot < nlive;
        const int64_t my_pair = pair0 + (live ? slot : 0);
        const int64_t bq = my_pair / G;
        const int g = (int)(my_pair - bq * G);
        const int64_t b = bq / p.Q;
        const int64_t sample = (b * p.S * G + g) * (int64_t)D;

        for (int c0 = 0; c0 < P; c0 += PC) {
            const int pc = min(PC, P - c0);
            const float inv_pc = 1.f / (float)pc;
            // ---- pre-pass ----------------------------------------------------------------
            for (int it = lane; it < ppw * pc; it += 32) {
                const int sl = (int)(((float)it + 0.5f) * inv_pc);   // it / pc
                const int j = it - sl * pc;
                const int pt = c0 + j;
                uint4 A = make_uint4(0u, 0u, 0u, 0u), Fr = make_uint4(0u, 0u, 0u, 0u);
                if (sl < nlive) {
                    const int64_t e = (pair0 + sl) * P + pt;
                    const int l = (int)(((float)pt + 0.5f) * inv_K);  // pt / K
                    float2 dpix;
                    const float2 xy = sample_location<T>(p, e, pair0 + sl, l, (float)lt.W[l],
                                                         (float)lt.H[l], dpix);
                    float a = VT::to_float(attn[e]);
                    if constexpr (SOFTMAX) {
                        const float2 st = s_stats[sl];
                        a = expf(a - st.x) * st.y;
                        s_prob[sl * P + pt] = a;
                    }
                    const PointGeom geo = locate(xy.x, xy.y, lt.H[l], lt.W[l], lt.start[l], GD);
                    // a skipped point contributes exact zeros whatever its weight holds
                    const float au = (geo.flags & kInside) ? a : 0.f;
                    unsigned flags = geo.flags | ((unsigned)l << kLevelShift);
                    unsigned red_off = (unsigned)geo.off00;         // the image: same place as value
                    if constexpr (SCALED) {
                        if (lt.rep[l] > 1) {
                            // spread the additions of a coarse level over its accumulators
                            const unsigned r = (unsigned)((pair0 + sl) / G + pt) % (unsigned)lt.rep[l];
                            if (r > 0) {
                                red_off = lt.rep_base[l] + (r - 1) * lt.level_elems[l] +
                                          (unsigned)((geo.r0 * lt.W[l] + geo.c0) * GD);
                                flags |= kUseExtra;
                            }
                        }
                    }
                    // .w: the weight as the grad_value scatter uses it (times 2^e when scaled)
                    A = make_uint4((unsigned)geo.off00, red_off, flags, __float_as_uint(au * scale));
                    Fr = make_uint4(__float_as_uint(geo.fr), __float_as_uint(geo.fc),
                                    __float_as_uint(au * dpix.x), __float_as_uint(au * dpix.y));
                }
                desc[sl * DS + 2 * j] = A;
                desc[sl * DS + 2 * j + 1] = Fr;
            }
            __syncwarp();
            // ---- gather, scatter, reduce -------------------------------------------------
            const uint4 *dp = desc + slot * DS;
            // the trip count is the same for every lane (the shuffles below are warp-wide);
            // a lane whose channels lie beyond D only contributes zeros
            for (int cb = 0; cb < D; cb += lph * V) {
                const int ch = cb + sub * V;
                const bool first_ch = cb == 0;
                const bool on_lane = live && ch < D;
                float2 go[NV2];
                VT::unpack(on_lane ? ld_stream16(grad_out + my_pair * D + ch)
                                   : make_uint4(0, 0, 0, 0), go);
                const T *vc = value + sample + ch;
                RT *gc = red_base + sample + ch;
                RT *xc = extras + b * extra_sample + g * D + ch;
#pragma unroll kUnroll
                for (int j = 0; j < pc; ++j) {
                    const uint4 A = dp[2 * j];
                    const uint4 Fr = dp[2 * j + 1];
                    const unsigned flags_all = A.z;
                    const unsigned flags = on_lane ? flags_all : 0u;
                    const float a = __uint_as_float(A.w);
                    const float fr = __uint_as_float(Fr.x), fc = __uint_as_float(Fr.y);
                    const float wr0 = 1.f - fr, wc0 = 1.f - fc;
                    const float w[4] = {wr0 * wc0, wr0 * fc, fr * wc0, fr * fc};
                    const int rs = lt.rowstride[flags_all >> kLevelShift];
                    const int o00 = (int)A.x, o10 = o00 + rs;
                    const int off[4] = {o00, o00 + GD, o10, o10 + GD};
                    // where the reductions go (32-bit unsigned offsets, wrapping like the
                    // corner arithmetic): the image, or this point's replica in the extras
                    const unsigned q00 = A.y, q10 = q00 + (unsigned)rs;
                    const unsigned roff[4] = {q00, q00 + (unsigned)GD, q10, q10 + (unsigned)GD};
                    RT *rbase = (flags_all & kUseExtra) ? xc : gc;
                    uint4 raw[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) raw[c] = ldg16_if(vc + off[c], flags & (1u << c));
                    float dot[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float2 f[NV2];
                        VT::unpack(raw[c], f);
                        float2 d2 = make_float2(0.f, 0.f);
                        const float s = a * w[c];
                        const float2 s2 = make_float2(s, s);
                        float2 gv[NV2];
#pragma unroll
                        for (int i = 0; i < NV2; ++i) {
                            ffma2(d2, f[i], go[i]);
                            gv[i] = fmul2(go[i], s2);
                        }
                        dot[c] = d2.x + d2.y;
                        red_if<RT>(rbase + roff[c], gv, flags & (1u << c));
                    }
                    // derivative inside the cell [floor, floor+1); d/da = sample . grad_out
                    float gx = wr0 * (dot[1] - dot[0]) + fr * (dot[3] - dot[2]);
                    float gy = wc0 * (dot[2] - dot[0]) + fc * (dot[3] - dot[1]);
                    float ga = w[0] * dot[0] + w[1] * dot[1] + w[2] * dot[2] + w[3] * dot[3];
                    for (int o = lph >> 1; o > 0; o >>= 1) {
                        gx += __shfl_xor_sync(0xffffffffu, gx, o);
                        gy += __shfl_xor_sync(0xffffffffu, gy, o);
                        ga += __shfl_xor_sync(0xffffffffu, ga, o);
                    }
                    if (sub == 0 && live) {
                        const int idx = slot * P + c0 + j;
                        const float2 gl = make_float2(__uint_as_float(Fr.z) * gx,
                                                      __uint_as_float(Fr.w) * gy);
                        if (first_ch) {
                            s_gloc[idx] = gl;
                            s_gatt[idx] = ga;
                        } else {
                            const float2 old = s_gloc[idx];
                            s_gloc[idx] = make_float2(old.x + gl.x, old.y + gl.y);
                            s_gatt[idx] += ga;
                        }
                    }
                }
            }
            __syncwarp();
        }

        // ---- softmax Jacobian and contiguous write-out of the group's gradients -------------
        if constexpr (SOFTMAX) {
            if (lane < nlive) {
                float inner = 0.f;
                for (int i = 0; i < P; ++i) inner += s_prob[lane * P + i] * s_gatt[lane * P + i];
                s_stats[lane].x = inner;
            }
            __syncwarp();
        }
        float2 *gl_out = reinterpret_cast<float2 *>(p.grad_loc) + pair0 * P;
        T *ga_out = reinterpret_cast<T *>(p.grad_attn) + pair0 * P;
        for (int idx = lane; idx < nlive * P; idx += 32) {
            float ga = s_gatt[idx];
            if constexpr (SOFTMAX) {
                const int sl = (int)(((float)idx + 0.5f) * inv_P);
                ga = s_prob[idx] * (ga - s_stats[sl].x);
            }
            if constexpr (sizeof(T) == 2) {
                // offsets predicted in the value dtype get their gradient in that dtype
                if (p.ref != nullptr && p.offsets16)
                    reinterpret_cast<uint32_t *>(p.grad_loc)[pair0 * P + idx] = VT::pack2(s_gloc[idx]);
                else
                    st_stream_f2(gl_out + idx, s_gloc[idx]);
            } else {
                st_stream_f2(gl_out + idx, s_gloc[idx]);
            }
            ga_out[idx] = VT::from_float(ga);
        }
        __syncwarp();
    }
}

// ---- scaled float16 image: preparation and finalisation ----------------------------------------
// largest magnitude pattern among the eight 16-bit elements of a vector
__device__ __forceinline__ unsigned max_magnitude_bits(const uint4 &v) {
    const unsigned a = __vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu);
    const unsigned b = __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu);
    const unsigned m = __vmaxu2(a, b);
    return max(m & 0xffffu, m >> 16);
}

// largest magnitude pattern over vectors first, first + stride, ... of `p`: four loads in flight
__device__ __forceinline__ unsigned scan_max_magnitude(const uint4 *__restrict__ p, int64_t n,
                                                       int64_t first, int64_t stride) {
    unsigned m = 0;
    int64_t v = first;
    for (; v + 3 * stride < n; v += 4 * stride) {
        const uint4 a = p[v], b = p[v + stride], c = p[v + 2 * stride], d = p[v + 3 * stride];
        m = max(max(m, max(max_magnitude_bits(a), max_magnitude_bits(b))),
                max(max_magnitude_bits(c), max_magnitude_bits(d)));
    }
    for (; v < n; v += stride) m = max(m, max_magnitude_bits(p[v]));
    return m;
}

// Clears the float16 image the backward kernel adds into and records the largest |grad_out|
// (and, without softmax, |attn|) element in the scratch header.  The header cells were set to
// zero on the stream before this kernel.
template <bool WITH_ATTN>
__global__ void __launch_bounds__(256, MSDA_PREP_MIN_CTAS) prepare_kernel(const Params p) {
    grid_launch_dependents();   // the backward kernel may load its tables meanwhile
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned *header = reinterpret_cast<unsigned *>(p.scratch);
    uint4 *image = reinterpret_cast<uint4 *>(reinterpret_cast<char *>(p.scratch) + kScratchHeaderBytes);
    const int64_t image_vecs = p.B * p.S * (p.G * p.D / 8);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // (the extras are cleared in full: at most K*Q*G*D*L / 64 elements per sample)
    const int64_t clear_vecs = image_vecs + p.B * (extra_elems_per_sample(p.Q, p.G, p.D, p.L, p.K) / 8);
    unsigned mg = 0, ma = 0;
    const int64_t go_vecs = p.B * p.Q * (p.G * p.D / 8);
    const uint4 *go = reinterpret_cast<const uint4 *>(p.grad_out);
    mg = scan_max_magnitude(go, go_vecs, first, stride);
    if constexpr (WITH_ATTN) {
        // (B*Q*G*L*K 16-bit elements; the tail that does not fill a vector is read singly)
        const int64_t n = p.B * p.Q * p.G * p.L * p.K;
        const uint4 *at = reinterpret_cast<const uint4 *>(p.attn);
        ma = scan_max_magnitude(at, n / 8, first, stride);
        const unsigned short *tail = reinterpret_cast<const unsigned short *>(p.attn);
        for (int64_t i = (n / 8) * 8 + first; i < n; i += stride) ma = max(ma, tail[i] & 0x7fffu);
    }
    // the clearing stores come after the scan's loads were issued: they need no answer, and the
    // loads' round trips to DRAM are the longest thing this kernel waits for
    for (int64_t v = first; v < clear_vecs; v += stride) image[v] = zero;
    // one atomic per CTA and cell: the warps' maxima meet in shared memory first (every warp
    // finishes at about the same time, and same-address atomics are served one after another)
    __shared__ unsigned cta_max[2];
    if (threadIdx.x < 2) cta_max[threadIdx.x] = 0u;
    __syncthreads();
    mg = __reduce_max_sync(0xffffffffu, mg);
    if constexpr (WITH_ATTN) ma = __reduce_max_sync(0xffffffffu, ma);
    if ((threadIdx.x & 31) == 0) {
        if (mg != 0) atomicMax(&cta_max[0], mg);
        if (WITH_ATTN && ma != 0) atomicMax(&cta_max[1], ma);
    }
    __syncthreads();
    if (threadIdx.x < (WITH_ATTN ? 2 : 1) && cta_max[threadIdx.x] != 0)
        atomicMax(header + threadIdx.x, cta_max[threadIdx.x]);
}

// grad_value = (image + the replicas of the position's level) * 2^-e, rounded to T.
// Positions of levels that have replicas form a small range of every sample (the coarse levels:
// 1 024 of 21 504 positions at the headline shape); everything outside it takes the short path.
template <typename T, bool SOFTMAX>
__global__ void __launch_bounds__(256, MSDA_FIN_MIN_CTAS) finalize_kernel(const Params p) {
    using VT = VecTraits<T>;
    __shared__ LevelTable lt;
    __shared__ int extra_range[2];
    load_level_table(lt, p);
    __syncthreads();
    if (threadIdx.x == 0) {
        plan_replicas(lt, p);
        int lo = 0x7fffffff, hi = 0;
        for (int l = 0; l < p.L; ++l)
            if (lt.rep[l] > 1) {
                lo = min(lo, lt.start[l]);
                hi = max(hi, lt.start[l] + lt.H[l] * lt.W[l]);
            }
        extra_range[0] = lo;
        extra_range[1] = hi;
    }
    __syncthreads();
    grid_dependency_wait();     // the image is complete once the backward kernel has finished
    const int extra_lo = extra_range[0], extra_hi = extra_range[1];
    const bool any_extra = extra_lo < extra_hi;
    const int GD = p.G * p.D;
    const int vec_per_row = GD / 8;
    const int S = (int)p.S;
    const int64_t extra_sample = extra_elems_per_sample(p.Q, p.G, p.D, p.L, p.K);
    const float inv = ldexpf(1.f, -grad_scale_exponent<T>(reinterpret_cast<const unsigned *>(p.scratch),
                                                          p.Q, p.K, SOFTMAX));
    const float2 inv2 = make_float2(inv, inv);
    const uint4 *image = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(p.scratch) +
                                                         kScratchHeaderBytes);
    const __half *extras = reinterpret_cast<const __half *>(image) + p.B * p.S * (int64_t)GD;
    uint4 *gv = reinterpret_cast<uint4 *>(p.grad_value);
    const int64_t total = p.B * p.S * (int64_t)vec_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // where the thread's current vector lies - sample b, position s of the sample, vector col of
    // the position's row - kept up to date by additions: one division per thread, none per vector
    // (first and stride are below 2^31: the grid is capped at a few thousand CTAs of 256 threads)
    const unsigned first_row = (unsigned)first / (unsigned)vec_per_row;
    int col = (int)((unsigned)first - first_row * (unsigned)vec_per_row);
    int64_t b = first_row / (unsigned)S;
    int s = (int)(first_row - (unsigned)b * (unsigned)S);
    const unsigned step_rows_all = (unsigned)stride / (unsigned)vec_per_row;
    const int step_cols = (int)((unsigned)stride - step_rows_all * (unsigned)vec_per_row);
    const int step_samples = (int)(step_rows_all / (unsigned)S);          // whole samples per stride
    const int step_rows = (int)(step_rows_all - (unsigned)step_samples * (unsigned)S);
    constexpr int kTurn = MSDA_FIN_VECS;
    for (int64_t v0 = first; v0 < total; v0 += kTurn * stride) {
        // several vectors per turn, their image loads issued together
        uint4 raw[kTurn];
#pragma unroll
        for (int u = 0; u < kTurn; ++u)
            raw[u] = v0 + u * stride < total ? ld_stream16(image + v0 + u * stride)
                                             : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < kTurn; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= total) break;
            float2 f[4];
            VecTraits<__half>::unpack(raw[u], f);
            if (any_extra) {
                if (s >= extra_lo && s < extra_hi) {
                    const __half *sample_extras = extras + b * extra_sample + col * 8;
                    // every level whose range holds this position (one, for a well-formed table)
                    for (int l = 0; l < p.L; ++l) {
                        const int at = s - lt.start[l];
                        if (lt.rep[l] <= 1 || at < 0 || at >= lt.H[l] * lt.W[l]) continue;
                        const __half *src = sample_extras + lt.rep_base[l] + (int64_t)at * GD;
                        for (int r = 1; r < lt.rep[l]; ++r) {
                            float2 x[4];
                            VecTraits<__half>::unpack(
                                ld_stream16(src + (int64_t)(r - 1) * lt.level_elems[l]), x);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                f[i].x += x[i].x;
                                f[i].y += x[i].y;
                            }
                        }
                    }
                }
                // on to the vector one stride further
                col += step_cols;
                s += step_rows;
                b += step_samples;
                if (col >= vec_per_row) {
                    col -= vec_per_row;
                    ++s;
                }
                if (s >= S) {
                    s -= S;
                    ++b;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = fmul2(f[i], inv2);
            gv[v] = VT::pack(f);
        }
    }
}

template <typename T, bool SOFTMAX, bool SCALED>
cudaError_t launch_kernel(const Params &p, cudaStream_t stream) {
    const size_t smem = backward_smem_bytes(p, SOFTMAX);
    auto kernel = backward_kernel<T, SOFTMAX, SCALED>;
    if (smem > 48 * 1024) {  // opt in to large dynamic shared memory only when needed
        cudaError_t e =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    // Two adjacent passes per CTA once that still leaves every SM several waves of CTAs
    // (the per-CTA prologue is paid half as often; worth about 0.2 % at the headline shape).
    Params q = p;
    int device = 0, sms = 0, per_sm = 0;
    q.passes = 1;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, p.threads, smem) ==
            cudaSuccess &&
        sms > 0 && per_sm > 0 && p.grid >= 8u * (unsigned)(sms * per_sm))
        q.passes = 2;
    const int64_t per_cta = (int64_t)(p.threads / 32) * q.passes;   // groups one CTA covers
    const int64_t ctas = (p.num_groups + per_cta - 1) / per_cta;
    if (ctas > 0x7fffffffll) return cudaErrorInvalidConfiguration;   // > 10^11 pairs
    q.grid = (unsigned)ctas;
    if constexpr (SCALED) return launch_after_predecessor(kernel, q.grid, q.threads, smem, stream, q);
    kernel<<<q.grid, q.threads, smem, stream>>>(q);
    return cudaGetLastError();
}

template <typename T, bool SOFTMAX>
cudaError_t launch_typed(const Params &p, cudaStream_t stream) {
    if constexpr (sizeof(T) == 2) {
        if (p.scratch != nullptr) return launch_kernel<T, SOFTMAX, true>(p, stream);
    }
    return launch_kernel<T, SOFTMAX, false>(p, stream);
}

unsigned sweep_grid(const Params &p, int vec, int ctas_per_sm) {
    const int64_t total = p.B * p.S * (p.G * p.D / vec);
    const int64_t blocks = (total + 256 * 4 - 1) / (256 * 4);   // ~4 vectors per thread
    const int64_t cap = 148 * (int64_t)ctas_per_sm;
    return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

size_t backward_smem_bytes(const Params &p, bool softmax) {
    const size_t nwarps = p.threads / 32;
    const size_t stage_floats = backward_stage_floats(32 >> p.lph_log2, p.L * p.K, softmax);
    return nwarps * (desc_warp_vec(32 >> p.lph_log2, p.point_chunk) * 16 + stage_floats * sizeof(float));
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

cudaError_t launch_prepare_grad_value(const Params &p, int dtype, bool softmax, cudaStream_t stream) {
    if (dtype != 1 && dtype != 2) return cudaErrorInvalidValue;
    cudaError_t e = cudaMemsetAsync(p.scratch, 0, kScratchHeaderBytes, stream);
    if (e != cudaSuccess) return e;
    if (softmax)
        prepare_kernel<false><<<sweep_grid(p, 8, MSDA_PREP_CTAS_PER_SM), 256, 0, stream>>>(p);
    else
        prepare_kernel<true><<<sweep_grid(p, 8, MSDA_PREP_CTAS_PER_SM), 256, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_finalize_grad_value(const Params &p, int dtype, bool softmax, cudaStream_t stream) {
    const unsigned grid = sweep_grid(p, 8, MSDA_FIN_CTAS_PER_SM);
    if (dtype == 1)
        return softmax ? launch_after_predecessor(finalize_kernel<__half, true>, grid, 256, 0, stream, p)
                       : launch_after_predecessor(finalize_kernel<__half, false>, grid, 256, 0, stream, p);
    if (dtype == 2)
        return softmax
                   ? launch_after_predecessor(finalize_kernel<__nv_bfloat16, true>, grid, 256, 0, stream, p)
                   : launch_after_predecessor(finalize_kernel<__nv_bfloat16, false>, grid, 256, 0, stream, p);
    return cudaErrorInvalidValue;
}

}  // namespace msda_b200
