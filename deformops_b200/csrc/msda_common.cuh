// Shared device helpers for the sm_100a multi-scale deformable attention kernels.
//
// Layouts (all contiguous, row-major):
//   value / grad_value   (B, S, G, D)            element type T (f32, f16, bf16)
//   spatial_shapes       (L, 2) int64, rows (H, W)      level_start_index (L) int64
//   loc / grad_loc       (B, Q, G, L, K, 2) float32, (x, y) = (width, height) axis
//   attn / grad_attn     (B, Q, G, L*K)         element type T
//   out / grad_out       (B, Q, G*D)            element type T
//
// Vocabulary
//   pair    one (batch*query, head) row: P = L*K sample points, D channels.
//   slot    the LPH lanes of a warp that own a pair; each lane owns one 16-byte vector of
//           channels (8 for 16-bit types, 4 for float).  A bf16 head of 32 channels is a
//           4-lane slot, so a warp covers the 8 heads of one query.
//   group   the 32/LPH pairs a warp processes together.
//   point descriptor   32 bytes in shared memory per (pair, point): element offset of the
//           top-left corner, row stride, validity flags and the interpolation weights.
//           Descriptors are computed once per point by one lane (a warp-wide pre-pass over
//           coalesced loc/attn loads) and then broadcast to the slot's lanes, so the
//           gather loop itself is loads, unpacks and FMAs only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace msda_b200 {

constexpr int kMaxLevels = 16;           // level table kept in shared memory
constexpr int kScratchHeaderBytes = 256;  // backward scratch: header (magnitude cells), then the image
constexpr int kDescPerWarp = 128;        // descriptors (32 B each) a warp holds at a time
// tuning knob (compile-time): most descriptors per pair a warp holds at a time; 0 = no cap
#ifndef MSDA_POINT_CHUNK_CAP
#define MSDA_POINT_CHUNK_CAP 0
#endif
// uint4 words of descriptor storage per warp: a row of 2 * point_chunk words per slot, padded by
// one word so that the 8 (or fewer) slots of a warp read their 16-byte descriptor halves from
// distinct banks.  Sized to what the call needs: shared memory a CTA does not take stays L1,
// and L1 hits are what the gather lacks.
__host__ __device__ inline int desc_warp_vec(int pairs_per_warp, int point_chunk) {
    return pairs_per_warp * (2 * point_chunk + 1);
}

struct Params {
    const void *value;
    const int64_t *spatial_shapes;
    const int64_t *level_start_index;
    const float *loc;
    const void *attn;
    void *out;              // forward only
    const void *grad_out;   // backward only
    void *grad_value;       // backward only
    float *grad_loc;        // backward only
    void *grad_attn;        // backward only
    void *scratch;          // backward only, 16-bit dtypes: header + scaled f16 image of grad_value, or null
    int64_t B, S, Q;
    int G, D, L, K;
    int lph_log2;           // log2(lanes per slot)
    int threads;            // threads per CTA (multiple of 32)
    int point_chunk;        // descriptors per pair held in shared memory at a time
    int64_t num_groups;     // ceil(B*Q*G / pairs per warp)
    unsigned grid;
    int passes;             // backward: adjacent sets of groups one CTA walks (0 or 1: one)
    // Fused location arithmetic.  When `ref` is set, `loc` / `grad_loc` hold the predicted
    // offsets (B,Q,G,L,K,2) and their gradient, and a point samples at
    //   ref_coords == 2:  ref.xy + offset / (W_l, H_l)
    //   ref_coords == 4:  ref.xy + offset / K * ref.wh * 0.5      (ref = cx, cy, w, h)
    const float *ref;       // (B,Q,L,ref_coords) float32, or null: `loc` holds locations
    int ref_coords;
    int offsets16;          // offsets and their gradient are stored in the 16-bit value dtype
};

// ---------------------------------------------------------------------------------
// 16-byte channel vectors, handled as float2 pairs for the packed f32x2 pipe
// ---------------------------------------------------------------------------------
template <typename T> struct VecTraits;

template <> struct VecTraits<float> {
    static constexpr int kVec = 4;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float2 (&f)[2]) {
        f[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
        f[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
    }
    __device__ static __forceinline__ uint4 pack(const float2 (&f)[2]) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y),
                          __float_as_uint(f[1].x), __float_as_uint(f[1].y));
    }
    __device__ static __forceinline__ float to_float(float v) { return v; }
    __device__ static __forceinline__ float from_float(float v) { return v; }
    // 16-byte reduction into global memory, no return value.  Reductions carry no "memory"
    // clobber: their targets are never read by the kernels, so gather loads of later
    // points may be scheduled above them.
    __device__ static __forceinline__ void red_add(void *addr, const float2 (&f)[2]) {
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr),
                     "f"(f[0].x), "f"(f[0].y), "f"(f[1].x), "f"(f[1].y));
    }
};

template <> struct VecTraits<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float2 (&f)[4]) {
        // bf16 -> f32 is a 16-bit shift: low half by shl, high half by mask
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
    __device__ static __forceinline__ float2 unpack2(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    __device__ static __forceinline__ uint32_t pack2(float2 v) {
        uint32_t r;  // cvt packs {upper, lower} with round-to-nearest-even
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(v.y), "f"(v.x));
        return r;
    }
    __device__ static __forceinline__ uint4 pack(const float2 (&f)[4]) {
        return make_uint4(pack2(f[0]), pack2(f[1]), pack2(f[2]), pack2(f[3]));
    }
    __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_float(float v) {
        return __float2bfloat16_rn(v);
    }
    // one 16-byte packed reduction (eight bf16 adds) instead of four bf16x2 atomics
    __device__ static __forceinline__ void red_add(void *addr, const float2 (&f)[4]) {
        const uint4 p = pack(f);
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                         addr),
                     "r"(p.x), "r"(p.y), "r"(p.z), "r"(p.w));
    }
};

template <> struct VecTraits<__half> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float2 (&f)[4]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    }
    __device__ static __forceinline__ float2 unpack2(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    }
    __device__ static __forceinline__ uint32_t pack2(float2 v) {
        const __half2 h = __float22half2_rn(v);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    __device__ static __forceinline__ uint4 pack(const float2 (&f)[4]) {
        return make_uint4(pack2(f[0]), pack2(f[1]), pack2(f[2]), pack2(f[3]));
    }
    __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
    __device__ static __forceinline__ void red_add(void *addr, const float2 (&f)[4]) {
        const uint4 p = pack(f);
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                         addr),
                     "r"(p.x), "r"(p.y), "r"(p.z), "r"(p.w));
    }
};

// predicated packed reductions: one instruction, no branch
template <typename T>
__device__ __forceinline__ void red_if(T *addr, const float2 (&g)[VecTraits<T>::kVec / 2], bool pred);

template <>
__device__ __forceinline__ void red_if<float>(float *addr, const float2 (&g)[2], bool pred) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %5, 0;\n\t"
                 "@q red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n\t}" ::"l"(addr),
                 "f"(g[0].x), "f"(g[0].y), "f"(g[1].x), "f"(g[1].y), "r"((unsigned)pred));
}
template <>
__device__ __forceinline__ void red_if<__nv_bfloat16>(__nv_bfloat16 *addr, const float2 (&g)[4],
                                                      bool pred) {
    const uint4 v = VecTraits<__nv_bfloat16>::pack(g);
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %5, 0;\n\t"
                 "@q red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};\n\t}" ::"l"(
                     addr),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"((unsigned)pred));
}
template <>
__device__ __forceinline__ void red_if<__half>(__half *addr, const float2 (&g)[4], bool pred) {
    const uint4 v = VecTraits<__half>::pack(g);
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %5, 0;\n\t"
                 "@q red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};\n\t}" ::"l"(
                     addr),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"((unsigned)pred));
}

// packed two-wide float32 arithmetic (sm_100): one issue slot for two lanes of work
__device__ __forceinline__ void ffma2(float2 &acc, const float2 a, const float2 b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;"
        : "+l"(reinterpret_cast<unsigned long long &>(acc))
        : "l"(reinterpret_cast<const unsigned long long &>(a)),
          "l"(reinterpret_cast<const unsigned long long &>(b)));
}
__device__ __forceinline__ float2 fmul2(const float2 a, const float2 b) {
    float2 r;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long &>(r))
        : "l"(reinterpret_cast<const unsigned long long &>(a)),
          "l"(reinterpret_cast<const unsigned long long &>(b)));
    return r;
}

// read-only 16-byte gather load
__device__ __forceinline__ uint4 ldg16(const void *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}

// load instruction of the backward's corner gather (a tuning knob: cache operators and
// eviction hints can be swapped in at compile time)
#ifndef MSDA_BWD_GATHER_LD
#define MSDA_BWD_GATHER_LD "ld.global.nc.v4.u32"
#endif

// Read-only 16-byte gather load, predicated: returns zeros and touches no memory when
// `pred` is false.  Not volatile, so the compiler may batch the loads of several points.
__device__ __forceinline__ uint4 ldg16_if(const void *p, bool pred) {
    uint4 r;
    asm("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %5, 0;\n\tmov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\t"
        "mov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t@q " MSDA_BWD_GATHER_LD " {%0, %1, %2, %3}, [%4];\n\t}"
        : "=&r"(r.x), "=&r"(r.y), "=&r"(r.z), "=&r"(r.w)
        : "l"(p), "r"((unsigned)pred));
    return r;
}

// streaming loads/stores for operands touched exactly once (loc, attn, out, grads): keeps
// them from displacing the value tensor in L1/L2
__device__ __forceinline__ float2 ld_stream_f2(const float2 *p) {
    float2 r;
    asm volatile("ld.global.cs.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "l"(p));
    return r;
}
// Programmatic dependent launch.  A kernel launched with launch_after_predecessor() may become
// resident while the kernel before it in the stream is still draining; it must pass
// grid_dependency_wait() before it touches anything that kernel writes (the wait returns once
// the predecessor has completed and its writes are visible).  grid_launch_dependents() lets the
// next such kernel in: it takes effect once every CTA of this grid has issued it or exited.
// In a kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launching with the attribute costs the host a few microseconds more than an ordinary launch
// (measured: a Deformable-DETR decoder layer's backward call, which is bound by the host's launch
// rate, went from 0.052 to 0.065 ms with it, the headline shape from 0.530 to 0.525 ms), so it
// is used only for calls whose kernels run long enough to hide that.
inline bool worth_dependent_launch(const Params &p) {
    return p.B * p.Q * p.G * (int64_t)(p.L * p.K) >= ((int64_t)1 << 21);
}

template <typename Kernel>
inline cudaError_t launch_after_predecessor(Kernel kernel, unsigned grid, unsigned threads, size_t smem,
                                            cudaStream_t stream, const Params &p) {
    if (!worth_dependent_launch(p)) {
        kernel<<<grid, threads, smem, stream>>>(p);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 r;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_stream16(void *p, const uint4 &v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w));
}
__device__ __forceinline__ void st_stream_f2(float2 *p, float2 v) {
    asm volatile("st.global.cs.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v.x), "f"(v.y));
}

// ---------------------------------------------------------------------------------
// Scaled float16 accumulation of a 16-bit grad_value
// ---------------------------------------------------------------------------------
// With a scratch buffer the 16-bit backward does not add into grad_value itself.  Every
// contribution is multiplied by one power of two, 2^e, rounded to float16 and added (packed
// red.global.add.f16x2) into a float16 image of grad_value that lives in the scratch; a last
// pass multiplies by 2^-e and writes grad_value in its own type.  float16 keeps 11 significant
// bits per addition where bfloat16 keeps 8, and the scale puts the sums where float16 can hold
// them: e is chosen from the largest |grad_out| and |attn| element of the call (found on the
// device, no host read) so that even Q*K contributions of the largest possible magnitude -
// the most one element can receive - stay below the float16 maximum.
//
// A float16 sum of n terms still loses about sqrt(n) * 2^-12 of its value, and the coarsest
// level of a pyramid can receive more than a thousand additions per element.  A level whose
// elements receive n = 4*K*Q / (H*W) > kAddsPerAccumulator additions on average is therefore
// given R = ceil(n / kAddsPerAccumulator) accumulators per element: the image itself plus R-1
// replicas of the level in a per-sample block of "extras"; a point adds into replica
// (query + point) mod R and the last pass sums them in float32.  Such levels are small by
// construction: all extras of a sample take at most L * K*Q*G*D / 64 elements.
//
// Scratch layout: kScratchHeaderBytes of header, then the image, B*S*G*D float16, then B blocks
// of extra_elems_per_sample() float16.  Header cell 0 / 1: the 15 magnitude bits of the largest
// |grad_out| / |attn| element (16-bit patterns order like their magnitudes; a NaN sorts above
// everything and switches the scaling off).
constexpr int kAddsPerAccumulator = 256;
constexpr int kMaxReplicas = 64;

__host__ __device__ inline int64_t extra_elems_per_sample(int64_t Q, int64_t G, int64_t D,
                                                         int64_t L, int64_t K) {
    return L * ((((K * Q * G * D + 63) / 64) + 7) & ~(int64_t)7);   // whole 16-byte vectors
}
template <typename T>
__device__ __forceinline__ float magnitude_from_bits(unsigned bits);
template <>
__device__ __forceinline__ float magnitude_from_bits<__nv_bfloat16>(unsigned bits) {
    return __uint_as_float(bits << 16);
}
template <>
__device__ __forceinline__ float magnitude_from_bits<__half>(unsigned bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}

template <typename T>
__device__ __forceinline__ int grad_scale_exponent(const unsigned *header, int64_t Q, int K,
                                                   bool softmax) {
    const float mg = magnitude_from_bits<T>(header[0]);
    const float ma = softmax ? 1.f : magnitude_from_bits<T>(header[1]);   // probabilities are <= 1
    const float bound = mg * ma * (float)Q * (float)K;
    if (!(bound > 0.f) || !(bound < INFINITY)) return 0;   // all zero, or inf / NaN in the inputs
    const int e = 14 - ilogbf(bound);                      // bound * 2^e in [2^14, 2^15)
    return e < -100 ? -100 : (e > 100 ? 100 : e);
}

// ---------------------------------------------------------------------------------
// Level table -> shared memory (read from device memory: no host synchronisation)
// ---------------------------------------------------------------------------------
struct LevelTable {
    int H[kMaxLevels];
    int W[kMaxLevels];
    int start[kMaxLevels];          // first position of the level on the S axis
    int rowstride[kMaxLevels];      // elements between image rows: W * G * D
    // scaled float16 backward: accumulators per element of the level (1 = the image only) and
    // where the level's additional replicas start in a sample's block of extras
    int rep[kMaxLevels];
    unsigned rep_base[kMaxLevels];
    unsigned level_elems[kMaxLevels];   // H * W * G * D
};

// Accumulators per level for the scaled float16 backward (see above); every kernel of a call
// derives the same plan from the same level table.  (R-1) * H*W*G*D <= K*Q*G*D / 64 per level,
// so the extras always fit the block extra_elems_per_sample() reserves.
__device__ inline void plan_replicas(LevelTable &t, const Params &p) {
    const long long n4 = 4ll * p.K * p.Q;
    unsigned base = 0;
    for (int l = 0; l < p.L; ++l) {
        const long long hw = (long long)t.H[l] * t.W[l];
        long long r = hw > 0 ? (n4 + kAddsPerAccumulator * hw - 1) / (kAddsPerAccumulator * hw) : 1;
        r = r < 1 ? 1 : (r > kMaxReplicas ? kMaxReplicas : r);
        t.rep[l] = (int)r;
        t.rep_base[l] = base;
        base += (unsigned)(r - 1) * t.level_elems[l];
    }
}

// Loads the level table from device memory.  A level that does not lie inside the value tensor
// (non-positive size, negative start, or start + H*W beyond S) becomes an empty level at
// position 0: every point on it is skipped, so a malformed table produces zeros for that level
// instead of an access outside `value` / `grad_value`.
__device__ __forceinline__ void load_level_table(LevelTable &t, const Params &p) {
    if (threadIdx.x < p.L) {
        const int64_t h = p.spatial_shapes[2 * threadIdx.x];
        const int64_t w = p.spatial_shapes[2 * threadIdx.x + 1];
        const int64_t first = p.level_start_index[threadIdx.x];
        const bool fits = h > 0 && w > 0 && first >= 0 && h <= p.S && w <= p.S &&
                          h * w <= p.S && first <= p.S - h * w;
        const int H = fits ? (int)h : 0, W = fits ? (int)w : 0;
        t.H[threadIdx.x] = H;
        t.W[threadIdx.x] = W;
        t.start[threadIdx.x] = fits ? (int)first : 0;
        t.rowstride[threadIdx.x] = W * p.G * p.D;
        t.level_elems[threadIdx.x] = (unsigned)H * (unsigned)W * (unsigned)(p.G * p.D);
    }
}

// ---------------------------------------------------------------------------------
// Point geometry -> descriptor
// ---------------------------------------------------------------------------------
enum : unsigned {
    kCorner00 = 1u, kCorner01 = 2u, kCorner10 = 4u, kCorner11 = 8u,  // corner inside the level
    kInside = 16u,       // point passes -1 <= pixel < size on both axes (NaN / inf fail)
    kUseExtra = 32u,     // backward: this point adds into a replica in the extras, not the image
    kLevelShift = 8,     // bits 8.. of the flags word carry the level index (backward)
};

struct PointGeom {
    int off00;       // element offset of corner (r0, c0) from the sample's first element
    int rowstride;   // elements between image rows of this level: W * G * D
    unsigned flags;
    int r0, c0;      // integer pixel of corner (r0, c0); -1 is possible on either axis
    float fr, fc;    // fractional parts along height / width
    float Hf, Wf;
};

// pixel = loc * size - 0.5 in float32; corners outside the level are flagged off, never
// clamped; a point outside [-1, size) on either axis is skipped altogether.
__device__ __forceinline__ PointGeom locate(float x, float y, int H, int W, int start, int GD) {
    PointGeom g;
    g.Hf = (float)H;
    g.Wf = (float)W;
    const float px = fmaf(x, g.Wf, -0.5f);
    const float py = fmaf(y, g.Hf, -0.5f);
    // (an empty level, H == 0, skips everything: see load_level_table)
    const bool inside = (py >= -1.f) && (px >= -1.f) && (py < g.Hf) && (px < g.Wf) && H > 0;
    // keep the arithmetic finite for skipped points (their loads are predicated off)
    const float sx = inside ? px : 0.f;
    const float sy = inside ? py : 0.f;
    const float r0f = floorf(sy), c0f = floorf(sx);
    const int r0 = (int)r0f, c0 = (int)c0f;
    g.fr = sy - r0f;
    g.fc = sx - c0f;
    const bool r_ok0 = inside && r0 >= 0, r_ok1 = inside && r0 + 1 < H;
    const bool c_ok0 = c0 >= 0, c_ok1 = c0 + 1 < W;
    g.flags = (r_ok0 && c_ok0 ? kCorner00 : 0u) | (r_ok0 && c_ok1 ? kCorner01 : 0u) |
              (r_ok1 && c_ok0 ? kCorner10 : 0u) | (r_ok1 && c_ok1 ? kCorner11 : 0u) |
              (inside ? kInside : 0u);
    g.r0 = r0;
    g.c0 = c0;
    g.off00 = (start + r0 * W + c0) * GD;
    g.rowstride = W * GD;
    return g;
}

// Sample location of element `e` = (pair, point) of level `l`, and in `dpix` the derivative of
// the pixel coordinate with respect to what the caller differentiates: the location itself
// (W, H), or the predicted offset when the call carries reference points.  The offset
// arithmetic follows the torch expressions of the layers it replaces, in float32:
// `ref + offset / (W, H)` and `ref.xy + offset / K * ref.wh * 0.5`.
template <typename T>
__device__ __forceinline__ float2 sample_location(const Params &p, int64_t e, int64_t pair, int l,
                                                  float Wf, float Hf, float2 &dpix) {
    const float2 *loc2 = reinterpret_cast<const float2 *>(p.loc);
    if (p.ref == nullptr) {
        dpix = make_float2(Wf, Hf);
        return ld_stream_f2(loc2 + e);
    }
    float2 off;
    if constexpr (sizeof(T) == 2) {
        if (p.offsets16)
            off = VecTraits<T>::unpack2(__ldg(reinterpret_cast<const uint32_t *>(p.loc) + e));
        else
            off = ld_stream_f2(loc2 + e);
    } else {
        off = ld_stream_f2(loc2 + e);
    }
    const int64_t bq = pair / p.G;
    if (p.ref_coords == 2) {
        const float2 r = __ldg(reinterpret_cast<const float2 *>(p.ref) + bq * p.L + l);
        dpix = make_float2(1.f, 1.f);
        return make_float2(r.x + off.x / Wf, r.y + off.y / Hf);
    }
    const float4 r = __ldg(reinterpret_cast<const float4 *>(p.ref) + bq * p.L + l);
    const float Kf = (float)p.K;
    // d(location)/d(offset) = wh * 0.5 / K, evaluated as the forward expression at offset 1
    dpix = make_float2(Wf * (1.f / Kf * r.z * 0.5f), Hf * (1.f / Kf * r.w * 0.5f));
    return make_float2(r.x + off.x / Kf * r.z * 0.5f, r.y + off.y / Kf * r.w * 0.5f);
}

// softmax statistics of one pair's P logits: (max, 1 / sum of exp(logit - max))
template <typename T>
__device__ __forceinline__ float2 softmax_stats(const T *logits, int P) {
    float m = -INFINITY;
    for (int i = 0; i < P; ++i) m = fmaxf(m, VecTraits<T>::to_float(logits[i]));
    float sum = 0.f;
    for (int i = 0; i < P; ++i) sum += expf(VecTraits<T>::to_float(logits[i]) - m);
    return make_float2(m, 1.f / sum);
}

// floats of per-warp staging in the backward kernel: softmax stats (32 float2), then per
// (pair, point) a float2 location gradient, a weight gradient and (softmax) a probability;
// a multiple of 4 so every warp's region stays 16-byte aligned
__host__ __device__ inline int backward_stage_floats(int pairs_per_warp, int P, bool softmax) {
    const int n = 64 + pairs_per_warp * P * (softmax ? 4 : 3);
    return (n + 3) & ~3;
}

// launchers implemented in msda_forward.cu / msda_backward.cu; dtype: 0 f32, 1 f16, 2 bf16
cudaError_t launch_forward(const Params &p, int dtype, bool softmax, cudaStream_t stream);
cudaError_t launch_backward(const Params &p, int dtype, bool softmax, cudaStream_t stream);
cudaError_t launch_prepare_grad_value(const Params &p, int dtype, bool softmax, cudaStream_t stream);
cudaError_t launch_finalize_grad_value(const Params &p, int dtype, bool softmax, cudaStream_t stream);
// float64 kernels (msda_f64.cu): loc / grad_loc point at doubles
cudaError_t launch_forward_f64(const Params &p, bool softmax, cudaStream_t stream);
cudaError_t launch_backward_f64(const Params &p, bool softmax, cudaStream_t stream);
size_t forward_smem_bytes(const Params &p, bool softmax);
size_t backward_smem_bytes(const Params &p, bool softmax);
// records `message` as the calling thread's last error (what msda_b200_last_error returns)
// and hands `status` back; defined in msda_abi.cu next to the buffer it writes
int set_last_error(int status, const char *message);

}  // namespace msda_b200
