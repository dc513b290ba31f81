// Backward kernel for self-attention over the pyramid ("encoder" calls: Q == S, query i is
// pixel i of the flattened levels).  Same mathematics and same outputs as backward_kernel in
// msda_backward.cu; what changes is who works on what, so that most of the grad_value
// reductions happen on chip instead of in the L2 reduction units, which bound that kernel
// (81 G 64-byte reduction segments per second on B200: 408 us for the 33 M corner segments of
// the headline shape).
//
//  * Work item = (sample, region, head).  The unit square is cut into regions of about 16x16
//    pixels of the finest level; an item owns the queries of EVERY level whose pixel falls
//    into the region (256 + 64 + 16 for a three-level pyramid) for ONE head.  Their samples
//    land in the same neighbourhood of each level.
//  * For every level but the finest, the item keeps a window of that neighbourhood (region
//    plus a margin of 0.1 in normalised coordinates) in shared memory as int32 fixed-point
//    accumulators.  Corner contributions inside the window are added with native
//    red.shared.add.s32 (one lane per channel, rotated per slot: conflict free, one warp
//    instruction per clock; float shared atomics are a CAS loop and five times slower).
//    Integer addition is associative, so this part of grad_value is bit-reproducible.
//    The fixed-point scale is chosen per item from max|grad_out| * max|weight| and the
//    number of points of the item, which bounds every accumulator below 2^30: no overflow.
//  * When the item is done its windows are converted and flushed with packed 16-byte
//    reductions, one per (pixel, 8 channels) instead of one per sample corner: about fifteen
//    times fewer.  Corners outside a window, and the whole finest level, use the global
//    reductions of the generic kernel (and its replica plan).
//  * A warp owns 32/LPH consecutive queries of the item's head; pre-pass, descriptors,
//    gather, dot products, shuffle reduction and staged write-out are those of the generic
//    kernel, processed one level (K points) at a time.
//
// If the level table does not tile the Q queries the enumeration degenerates to consecutive
// chunks of queries without windows; results do not depend on the enumeration.
#include "msda_common.cuh"

namespace msda_b200 {

namespace {

constexpr int kRegionEdge = 16;               // pixels of the largest level per region edge
constexpr int kWindowInts = 28 * 1024;        // 112 KB of int32 window accumulators per CTA
constexpr float kWindowMargin = 0.1f;         // window margin in normalised coordinates
constexpr int kRegionThreads = 512;

enum : unsigned { kWinShift = 16 };           // flags bits 16..19: corner lies inside the window

struct RegionPlan {                           // same for every item of a launch
    int RX, RY;                               // regions along x / y
    int enum_levels;                          // levels used to enumerate queries (1 if degenerate)
    int eH[kMaxLevels], eW[kMaxLevels], ebase[kMaxLevels];   // enumeration table
    int wh[kMaxLevels], ww[kMaxLevels];       // window size per level (0: the level has none)
    int woff[kMaxLevels];                     // first int of the level's window
    int margin_y[kMaxLevels], margin_x[kMaxLevels];
};

struct ItemGeom {                             // per work item
    int qy0[kMaxLevels], qx0[kMaxLevels], qw[kMaxLevels];
    int qprefix[kMaxLevels + 1];              // queries of the item before level l
    int wy0[kMaxLevels], wx0[kMaxLevels];     // window origin in the level
    float scale, inv_scale;
    int use_windows;
};

__device__ inline void make_region_plan(RegionPlan &rp, const LevelTable &lt, const Params &p) {
    const int window_budget = p.region_window_ints;
    long long total = 0;
    int maxH = 1, maxW = 1;
    for (int l = 0; l < p.L; ++l) {
        total += (long long)lt.H[l] * lt.W[l];
        maxH = max(maxH, lt.H[l]);
        maxW = max(maxW, lt.W[l]);
    }
    const bool tiled = total == p.Q;
    if (tiled) {
        rp.enum_levels = p.L;
        int base = 0;
        for (int l = 0; l < p.L; ++l) {
            rp.eH[l] = lt.H[l];
            rp.eW[l] = lt.W[l];
            rp.ebase[l] = base;
            base += lt.H[l] * lt.W[l];
        }
        rp.RX = (maxW + kRegionEdge - 1) / kRegionEdge;
        rp.RY = (maxH + kRegionEdge - 1) / kRegionEdge;
    } else {   // enumerate the queries as one row, in chunks; no spatial meaning, no windows
        rp.enum_levels = 1;
        rp.eH[0] = 1;
        rp.eW[0] = (int)p.Q;
        rp.ebase[0] = 0;
        rp.RX = (int)((p.Q + 335) / 336);
        rp.RY = 1;
    }
    // windows: coarsest levels first, as long as they fit
    int used = 0;
    for (int l = 0; l < p.L; ++l) rp.wh[l] = rp.ww[l] = 0;
    if (!tiled) return;
    bool taken[kMaxLevels] = {};
    for (int n = 0; n < p.L; ++n) {
        int best = -1;
        for (int l = 0; l < p.L; ++l)
            if (!taken[l] && (best < 0 || lt.H[l] * lt.W[l] < lt.H[best] * lt.W[best])) best = l;
        taken[best] = true;
        const int my = (int)ceilf(kWindowMargin * lt.H[best]) + 1;
        const int mx = (int)ceilf(kWindowMargin * lt.W[best]) + 1;
        const int wh = min(lt.H[best], (lt.H[best] + rp.RY - 1) / rp.RY + 1 + 2 * my);
        const int ww = min(lt.W[best], (lt.W[best] + rp.RX - 1) / rp.RX + 1 + 2 * mx);
        const int ints = wh * ww * p.D;
        if (used + ints > window_budget) break;
        rp.wh[best] = wh;
        rp.ww[best] = ww;
        rp.woff[best] = used;
        rp.margin_y[best] = my;
        rp.margin_x[best] = mx;
        used += ints;
    }
}

// queries and windows of region (ry, rx)
__device__ inline void make_item_geom(ItemGeom &ig, const RegionPlan &rp, const LevelTable &lt,
                                      const Params &p, int ry, int rx) {
    int count = 0;
    for (int l = 0; l < rp.enum_levels; ++l) {
        const int y0 = (int)((long long)ry * rp.eH[l] / rp.RY);
        const int y1 = (int)((long long)(ry + 1) * rp.eH[l] / rp.RY);
        const int x0 = (int)((long long)rx * rp.eW[l] / rp.RX);
        const int x1 = (int)((long long)(rx + 1) * rp.eW[l] / rp.RX);
        ig.qy0[l] = y0;
        ig.qx0[l] = x0;
        ig.qw[l] = x1 - x0;
        ig.qprefix[l] = count;
        count += (y1 - y0) * (x1 - x0);
    }
    ig.qprefix[rp.enum_levels] = count;
    for (int l = 0; l < p.L; ++l) {
        if (rp.ww[l] == 0) continue;
        const int y0 = (int)((long long)ry * lt.H[l] / rp.RY) - rp.margin_y[l];
        const int x0 = (int)((long long)rx * lt.W[l] / rp.RX) - rp.margin_x[l];
        ig.wy0[l] = min(max(y0, 0), lt.H[l] - rp.wh[l]);
        ig.wx0[l] = min(max(x0, 0), lt.W[l] - rp.ww[l]);
    }
}

// i-th query of the item -> query index in [0, Q)
__device__ __forceinline__ int item_query(const ItemGeom &ig, const RegionPlan &rp, int i) {
    int l = 0;
    while (l + 1 < rp.enum_levels && i >= ig.qprefix[l + 1]) ++l;
    const int rel = i - ig.qprefix[l];
    const int iy = rel / ig.qw[l];
    return rp.ebase[l] + (ig.qy0[l] + iy) * rp.eW[l] + ig.qx0[l] + (rel - iy * ig.qw[l]);
}

// Rotates an array left by `r` positions (r < V) with log2(V) select stages, so that no
// register array is ever indexed dynamically.
template <int V>
__device__ __forceinline__ void rotate_left(float (&x)[V], int r) {
#pragma unroll
    for (int step = 1; step < V; step <<= 1) {
        float y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = x[(i + step) & (V - 1)];
        const bool take = (r & step) != 0;
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = take ? y[i] : x[i];
    }
}

// V integer reductions into a window pixel.  `gr` holds the lane's grad_out channels already
// rotated by its slot and `rot_bytes[i]` the matching byte offsets, so that at step i the lanes
// of a warp add channel (i + slot) mod V: 32 different banks, one instruction per clock.
template <int V>
__device__ __forceinline__ void window_add(const int *win_pixel, const float (&gr)[V],
                                           const unsigned (&rot_bytes)[V], float sv, bool pred) {
    const unsigned base = (unsigned)__cvta_generic_to_shared(win_pixel);
#pragma unroll
    for (int i = 0; i < V; ++i) {
        asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t"
                     "@q red.shared.add.s32 [%0], %1;\n\t}" ::"r"(base + rot_bytes[i]),
                     "r"(__float2int_rn(gr[i] * sv)), "r"((unsigned)pred));
    }
}

template <typename T, bool SOFTMAX>
__global__ void __launch_bounds__(kRegionThreads) backward_region_kernel(const Params p) {
    using VT = VecTraits<T>;
    constexpr int V = VT::kVec;
    constexpr int NV2 = V / 2;
    extern __shared__ uint4 smem[];
    __shared__ LevelTable lt;
    __shared__ RegionPlan rp;
    __shared__ ItemGeom ig;
    __shared__ float s_amax[2][kRegionThreads / 32];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int lph = 1 << p.lph_log2;
    const int ppw = 32 >> p.lph_log2;
    const int G = p.G, D = p.D, K = p.K;
    const int P = p.L * K;
    const int GD = G * D;
    const int DS = 3 * K + 1 + (K & 1);             // uint4 stride between slots (odd)
    const float inv_K = 1.f / (float)K;
    const float inv_P = 1.f / (float)P;

    // shared memory: windows | per-warp descriptors | per-warp staging
    int *windows = reinterpret_cast<int *>(smem);
    uint4 *desc = smem + p.region_window_ints / 4 + (size_t)warp * (ppw * DS);
    const int stage_floats = backward_stage_floats(ppw, P, SOFTMAX) + 32;
    float *stage = reinterpret_cast<float *>(smem + p.region_window_ints / 4 + (size_t)nwarps * (ppw * DS)) +
                   (size_t)warp * stage_floats;
    float2 *s_stats = reinterpret_cast<float2 *>(stage);          // [32]
    float2 *s_gloc = s_stats + 32;                                // [ppw*P]
    float *s_gatt = stage + 64 + ppw * P * 2;                     // [ppw*P]
    float *s_prob = s_gatt + ppw * P;                             // [ppw*P] softmax only
    int *s_q = reinterpret_cast<int *>(stage + stage_floats - 32);   // [32] query of each slot

    load_level_table(lt, p);
    __syncthreads();
    if (threadIdx.x == 0) {
        plan_replicas(lt, p);
        make_region_plan(rp, lt, p);
    }
    __syncthreads();

    const int slot = lane >> p.lph_log2;
    const int sub = lane & (lph - 1);
    const int ch = sub * V;
    const bool lane_has_channels = ch < D;
    unsigned rot_bytes[V];                     // byte offset of channel (i + slot) mod V
#pragma unroll
    for (int i = 0; i < V; ++i) rot_bytes[i] = 4u * (unsigned)((i + slot) & (V - 1));
    const T *value = reinterpret_cast<const T *>(p.value);
    const T *attn = reinterpret_cast<const T *>(p.attn);
    const T *grad_out = reinterpret_cast<const T *>(p.grad_out);
    const float2 *loc2 = reinterpret_cast<const float2 *>(p.loc);
    T *grad_value = reinterpret_cast<T *>(p.grad_value);
    T *scratch = reinterpret_cast<T *>(p.scratch);
    int window_ints = 0;
    for (int l = 0; l < p.L; ++l) window_ints = max(window_ints, rp.ww[l] ? rp.woff[l] + rp.wh[l] * rp.ww[l] * D : 0);

    const int64_t regions = (int64_t)rp.RX * rp.RY;
    const int64_t items = p.B * regions * G;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        // item -> (sample, region, head); the head varies slowest so that CTAs running at the
        // same time read neighbouring regions of the same head
        const int g = (int)(item / (p.B * regions));
        const int64_t rem = item - (int64_t)g * (p.B * regions);
        const int64_t b = rem / regions;
        const int region = (int)(rem - b * regions);
        __syncthreads();                                   // previous item fully flushed
        if (threadIdx.x == 0) make_item_geom(ig, rp, lt, p, region / rp.RX, region % rp.RX);
        for (int i = threadIdx.x; i < window_ints / 4; i += blockDim.x)
            reinterpret_cast<uint4 *>(windows)[i] = make_uint4(0u, 0u, 0u, 0u);
        __syncthreads();
        const int nq = ig.qprefix[rp.enum_levels];
        if (nq == 0) continue;

        // ---- fixed-point scale: bound on |grad_out| * |weight| over the item ----------------
        if (window_ints > 0) {
            float mg = 0.f, ma = SOFTMAX ? 1.f : 0.f;
            bool finite = true;
            const int vec_per_row = D / V;
            for (int i = threadIdx.x; i < nq * vec_per_row; i += blockDim.x) {
                const int qi = i / vec_per_row;
                const int64_t pair = (b * p.Q + item_query(ig, rp, qi)) * G + g;
                float2 f[NV2];
                VT::unpack(ldg16(grad_out + pair * D + (i - qi * vec_per_row) * V), f);
#pragma unroll
                for (int k = 0; k < NV2; ++k) mg = fmaxf(mg, fmaxf(fabsf(f[k].x), fabsf(f[k].y)));
            }
            if (!SOFTMAX) {
                for (int i = threadIdx.x; i < nq * P; i += blockDim.x) {
                    const int qi = (int)(((float)i + 0.5f) * inv_P);
                    const int64_t pair = (b * p.Q + item_query(ig, rp, qi)) * G + g;
                    ma = fmaxf(ma, fabsf(VT::to_float(attn[pair * P + (i - qi * P)])));
                }
            }
            finite = (mg <= 3.0e38f) && (ma <= 3.0e38f);      // false for inf and NaN
            for (int o = 16; o > 0; o >>= 1) {
                mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
                ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
            }
            const bool all_finite = __all_sync(0xffffffffu, finite);
            if (lane == 0) {
                s_amax[0][warp] = all_finite ? mg : INFINITY;
                s_amax[1][warp] = ma;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                float tg = 0.f, ta = 0.f;
                for (int w = 0; w < nwarps; ++w) {
                    tg = fmaxf(tg, s_amax[0][w]);
                    ta = fmaxf(ta, s_amax[1][w]);
                }
                const float bound = tg * ta * (float)(nq * K);   // |sum| of any accumulator
                if (bound > 0.f && bound <= 3.0e38f) {
                    int e;
                    frexpf(bound, &e);                             // bound < 2^e
                    ig.scale = ldexpf(1.f, 30 - e);
                    ig.inv_scale = ldexpf(1.f, e - 30);
                    ig.use_windows = 1;
                } else {
                    ig.scale = ig.inv_scale = 0.f;
                    ig.use_windows = 0;                            // zeros or non-finite: global path
                }
            }
            __syncthreads();
        } else if (threadIdx.x == 0) {
            ig.use_windows = 0;
        }
        __syncthreads();
        const bool use_windows = ig.use_windows != 0;
        const float scale = ig.scale;

        // ---- groups of ppw queries -----------------------------------------------------------
        const int ngroups = (nq + ppw - 1) / ppw;
        for (int grp = warp; grp < ngroups; grp += nwarps) {
            const int i0 = grp * ppw;
            const int nlive = min(ppw, nq - i0);
            if (lane < ppw) s_q[lane] = lane < nlive ? item_query(ig, rp, i0 + lane) : -1;
            __syncwarp();
            const bool live = slot < nlive;
            const int my_q = live ? s_q[slot] : s_q[0];
            const int64_t my_pair = (b * p.Q + my_q) * G + g;
            if constexpr (SOFTMAX) {
                if (lane < nlive)
                    s_stats[lane] = softmax_stats(attn + ((b * p.Q + s_q[lane]) * G + g) * P, P);
                __syncwarp();
            }
            const bool on_lane = live && lane_has_channels;
            float2 go[NV2];
            VT::unpack(on_lane ? ld_stream16(grad_out + my_pair * D + ch) : make_uint4(0, 0, 0, 0), go);
            float gr[V];                       // the same channels, rotated by the slot
#pragma unroll
            for (int i = 0; i < NV2; ++i) {
                gr[2 * i] = go[i].x;
                gr[2 * i + 1] = go[i].y;
            }
            rotate_left<V>(gr, slot & (V - 1));
            const int64_t sample = (b * p.S * G + g) * (int64_t)D;
            const T *vc = value + sample + ch;
            T *gc = grad_value + sample + ch;
            T *sc = scratch + b * (int64_t)lt.scratch_sample_elems + g * D + ch;

            for (int l = 0; l < p.L; ++l) {
                const bool windowed = use_windows && rp.ww[l] > 0;
                // ---- pre-pass: the K points of level l for every slot -----------------------
                for (int it = lane; it < ppw * K; it += 32) {
                    const int sl = (int)(((float)it + 0.5f) * inv_K);
                    const int k = it - sl * K;
                    const int pt = l * K + k;
                    uint4 A = make_uint4(0u, 0u, 0u, 0u), Fr = A, Wn = A;
                    if (sl < nlive) {
                        const int q = s_q[sl];
                        const int64_t e = ((b * p.Q + q) * G + g) * P + pt;
                        const float2 xy = ld_stream_f2(loc2 + e);
                        float a = VT::to_float(attn[e]);
                        if constexpr (SOFTMAX) {
                            const float2 st = s_stats[sl];
                            a = expf(a - st.x) * st.y;
                            s_prob[sl * P + pt] = a;
                        }
                        const PointGeom geo = locate(xy.x, xy.y, lt.H[l], lt.W[l], lt.start[l], GD);
                        const float au = (geo.flags & kInside) ? a : 0.f;
                        unsigned flags = geo.flags | ((unsigned)l << kLevelShift);
                        unsigned red_off = (unsigned)geo.off00;
                        if (lt.rep[l] > 0) {
                            const unsigned r = (unsigned)(q + pt) % (unsigned)lt.rep[l];
                            red_off = lt.rep_base[l] + r * lt.level_elems[l] +
                                      (unsigned)((geo.r0 * lt.W[l] + geo.c0) * GD);
                            flags |= kUseScratch;
                        }
                        int win_off = 0;
                        if (windowed) {
                            const int wr = geo.r0 - ig.wy0[l], wc = geo.c0 - ig.wx0[l];
                            const bool r_in0 = wr >= 0 && wr < rp.wh[l], r_in1 = wr + 1 >= 0 && wr + 1 < rp.wh[l];
                            const bool c_in0 = wc >= 0 && wc < rp.ww[l], c_in1 = wc + 1 >= 0 && wc + 1 < rp.ww[l];
                            unsigned w = (r_in0 && c_in0 ? 1u : 0u) | (r_in0 && c_in1 ? 2u : 0u) |
                                         (r_in1 && c_in0 ? 4u : 0u) | (r_in1 && c_in1 ? 8u : 0u);
                            w &= geo.flags & 15u;                     // only corners inside the level
                            flags |= w << kWinShift;
                            win_off = rp.woff[l] + (wr * rp.ww[l] + wc) * D;
                        }
                        A = make_uint4((unsigned)geo.off00, red_off, flags, __float_as_uint(au));
                        Fr = make_uint4(__float_as_uint(geo.fr), __float_as_uint(geo.fc),
                                        __float_as_uint(au * geo.Wf), __float_as_uint(au * geo.Hf));
                        Wn = make_uint4((unsigned)win_off, (unsigned)(rp.ww[l] * D), 0u, 0u);
                    }
                    desc[sl * DS + 3 * k] = A;
                    desc[sl * DS + 3 * k + 1] = Fr;
                    desc[sl * DS + 3 * k + 2] = Wn;
                }
                __syncwarp();
                // ---- gather, scatter, reduce --------------------------------------------------
                const uint4 *dp = desc + slot * DS;
                const int rs = lt.rowstride[l];
#pragma unroll 2
                for (int k = 0; k < K; ++k) {
                    const uint4 A = dp[3 * k];
                    const uint4 Fr = dp[3 * k + 1];
                    const unsigned flags_all = A.z;
                    const unsigned flags = on_lane ? flags_all : 0u;
                    const float a = __uint_as_float(A.w);
                    const float fr = __uint_as_float(Fr.x), fc = __uint_as_float(Fr.y);
                    const float wr0 = 1.f - fr, wc0 = 1.f - fc;
                    const float w[4] = {wr0 * wc0, wr0 * fc, fr * wc0, fr * fc};
                    const int o00 = (int)A.x, o10 = o00 + rs;
                    const int off[4] = {o00, o00 + GD, o10, o10 + GD};
                    const unsigned q00 = A.y, q10 = q00 + (unsigned)rs;
                    const unsigned roff[4] = {q00, q00 + (unsigned)GD, q10, q10 + (unsigned)GD};
                    T *rbase = (flags_all & kUseScratch) ? sc : gc;
                    int woff[4] = {0, 0, 0, 0};
                    unsigned wbits = 0;
                    if (windowed) {
                        const uint4 Wn = dp[3 * k + 2];
                        const int w00 = (int)Wn.x + ch, w10 = w00 + (int)Wn.y;
                        woff[0] = w00;
                        woff[1] = w00 + D;
                        woff[2] = w10;
                        woff[3] = w10 + D;
                        wbits = (flags >> kWinShift) & 15u;
                    }
                    uint4 raw[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) raw[c] = ldg16_if(vc + off[c], flags & (1u << c));
                    // corners that are inside the level but outside the window go to global memory
                    const unsigned gbits = flags & 15u & ~wbits;
                    const bool any_global = __any_sync(0xffffffffu, gbits != 0u);
                    float dot[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float2 f[NV2];
                        VT::unpack(raw[c], f);
                        float2 d2 = make_float2(0.f, 0.f);
                        const float s = a * w[c];
#pragma unroll
                        for (int i = 0; i < NV2; ++i) ffma2(d2, f[i], go[i]);
                        dot[c] = d2.x + d2.y;
                        if (windowed)
                            window_add<V>(windows + woff[c], gr, rot_bytes, s * scale, wbits & (1u << c));
                        if (any_global) {
                            const float2 s2 = make_float2(s, s);
                            float2 gv[NV2];
#pragma unroll
                            for (int i = 0; i < NV2; ++i) gv[i] = fmul2(go[i], s2);
                            red_if<T>(rbase + roff[c], gv, gbits & (1u << c));
                        }
                    }
                    float gx = wr0 * (dot[1] - dot[0]) + fr * (dot[3] - dot[2]);
                    float gy = wc0 * (dot[2] - dot[0]) + fc * (dot[3] - dot[1]);
                    float ga = w[0] * dot[0] + w[1] * dot[1] + w[2] * dot[2] + w[3] * dot[3];
                    for (int o = lph >> 1; o > 0; o >>= 1) {
                        gx += __shfl_xor_sync(0xffffffffu, gx, o);
                        gy += __shfl_xor_sync(0xffffffffu, gy, o);
                        ga += __shfl_xor_sync(0xffffffffu, ga, o);
                    }
                    if (sub == 0 && live) {
                        const int idx = slot * P + l * K + k;
                        s_gloc[idx] = make_float2(__uint_as_float(Fr.z) * gx, __uint_as_float(Fr.w) * gy);
                        s_gatt[idx] = ga;
                    }
                }
                __syncwarp();
            }

            // ---- softmax Jacobian and write-out of the group's location / weight gradients ---
            if constexpr (SOFTMAX) {
                if (lane < nlive) {
                    float inner = 0.f;
                    for (int i = 0; i < P; ++i) inner += s_prob[lane * P + i] * s_gatt[lane * P + i];
                    s_stats[lane].x = inner;
                }
                __syncwarp();
            }
            for (int idx = lane; idx < nlive * P; idx += 32) {
                const int sl = (int)(((float)idx + 0.5f) * inv_P);
                const int64_t e = ((b * p.Q + s_q[sl]) * G + g) * P + (idx - sl * P);
                float ga = s_gatt[idx];
                if constexpr (SOFTMAX) ga = s_prob[idx] * (ga - s_stats[sl].x);
                st_stream_f2(reinterpret_cast<float2 *>(p.grad_loc) + e, s_gloc[idx]);
                reinterpret_cast<T *>(p.grad_attn)[e] = VT::from_float(ga);
            }
            __syncwarp();
        }

        // ---- flush the windows: one packed reduction per touched (pixel, channel vector) -----
        __syncthreads();
        if (use_windows) {
            const float inv_scale = ig.inv_scale;
            const int vec_per_pix = D / V;
            for (int l = 0; l < p.L; ++l) {
                if (rp.ww[l] == 0) continue;
                const int nvec = rp.wh[l] * rp.ww[l] * vec_per_pix;
                const int *win = windows + rp.woff[l];
                const unsigned rep = (unsigned)lt.rep[l];
                T *base = rep ? scratch + b * (int64_t)lt.scratch_sample_elems + lt.rep_base[l] +
                                    (int64_t)((unsigned)item % rep) * lt.level_elems[l]
                              : grad_value + (b * p.S + lt.start[l]) * (int64_t)GD;
                for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
                    const int pix = v / vec_per_pix;
                    const int cv = v - pix * vec_per_pix;
                    const int *src = win + pix * D + cv * V;
                    int any = 0;
                    float2 f[NV2];
#pragma unroll
                    for (int i = 0; i < NV2; ++i) {
                        const int x = src[2 * i], y = src[2 * i + 1];
                        any |= x | y;
                        f[i] = make_float2((float)x * inv_scale, (float)y * inv_scale);
                    }
                    if (any == 0) continue;
                    const int wy = pix / rp.ww[l];
                    const int gy_ = ig.wy0[l] + wy, gx_ = ig.wx0[l] + (pix - wy * rp.ww[l]);
                    VT::red_add(base + (int64_t)(gy_ * lt.W[l] + gx_) * GD + g * D + cv * V, f);
                }
            }
        }
    }
}

}  // namespace

size_t backward_region_smem_bytes(const Params &p, bool softmax, int threads, int window_ints) {
    const size_t nwarps = threads / 32;
    const size_t ppw = 32 >> p.lph_log2;
    const size_t DS = 3 * p.K + 1 + (p.K & 1);
    const size_t stage_floats = backward_stage_floats((int)ppw, p.L * p.K, softmax) + 32;
    return (size_t)window_ints * 4 + nwarps * (ppw * DS * 16 + stage_floats * sizeof(float));
}

// The region kernel takes encoder-shaped calls whose per-warp state fits: one channel vector
// per lane (D*e <= 512 bytes) and one level's points per descriptor chunk.
bool backward_region_eligible(const Params &p, int dtype, bool softmax) {
    const int vec = dtype == 0 ? 4 : 8;
    const int ppw = 32 >> p.lph_log2;
    if (p.ref != nullptr) return false;                     // reads locations, not offsets
    if (p.Q != p.S || p.Q >= (1ll << 31) || p.D > 32 * vec || p.D % vec != 0) return false;
    if ((1 << p.lph_log2) * vec != p.D) return false;      // every lane of a slot carries channels
    if (ppw * p.K > 128 || p.D * 4 > kWindowInts) return false;
    return backward_region_smem_bytes(p, softmax, kRegionThreads, kWindowInts) <= 220 * 1024;
}

template <typename T, bool SOFTMAX>
static cudaError_t launch_region_typed(const Params &p, bool windows, cudaStream_t stream) {
    Params q = p;
    q.threads = windows ? kRegionThreads : 256;
    q.region_window_ints = windows ? kWindowInts : 0;
    const size_t smem = backward_region_smem_bytes(p, SOFTMAX, q.threads, q.region_window_ints);
    auto kernel = backward_region_kernel<T, SOFTMAX>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // persistent CTAs walk the work items: one per SM with windows, three without
    q.grid = (unsigned)(windows ? sms : 3 * sms);
    const size_t value_bytes = (size_t)(p.B * p.S) * p.G * p.D * sizeof(T);
    return launch_with_value_window(kernel, q, value_bytes, smem, stream);
}

cudaError_t launch_backward_region(const Params &p, int dtype, bool softmax, bool windows,
                                   cudaStream_t stream) {
    switch (dtype) {
        case 0:
            return softmax ? launch_region_typed<float, true>(p, windows, stream)
                           : launch_region_typed<float, false>(p, windows, stream);
        case 1:
            return softmax ? launch_region_typed<__half, true>(p, windows, stream)
                           : launch_region_typed<__half, false>(p, windows, stream);
        case 2:
            return softmax ? launch_region_typed<__nv_bfloat16, true>(p, windows, stream)
                           : launch_region_typed<__nv_bfloat16, false>(p, windows, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace msda_b200
