// Shared device helpers for the sm_100a multi-scale deformable attention kernels.
//
// Layouts (all contiguous, row-major):
//   value / grad_value   (B, S, G, D)            element type T (f32, f16, bf16)
//   spatial_shapes       (L, 2) int64, rows (H, W)      level_start_index (L) int64
//   loc / grad_loc       (B, Q, G, L, K, 2) float32, (x, y) = (width, height) axis
//   attn / grad_attn     (B, Q, G, L*K)         element type T
//   out / grad_out       (B, Q, G*D)            element type T
//
// A "pair" is one (batch*query, head) row: L*K sample points, D channels.  A "slot"
// is the group of LPH lanes that owns a pair; every lane owns one 16-byte vector of
// channels (8 for 16-bit types, 4 for float), so a bf16 head of 32 channels is a
// 4-lane slot and a warp covers 8 whole heads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace msda_b200 {

constexpr int kMaxLevels = 16;      // level table kept in shared memory
constexpr int kThreads = 256;       // threads per CTA for both kernels

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
    int64_t B, S, Q;
    int G, D, L, K;
    int lph_log2;           // log2(lanes per head slot)
    int tile_queries;       // queries staged per CTA tile
    int64_t num_tiles;
};

// ---------------------------------------------------------------------------------
// 16-byte channel vectors
// ---------------------------------------------------------------------------------
template <typename T> struct VecTraits;

template <> struct VecTraits<float> {
    static constexpr int kVec = 4;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float (&f)[4]) {
        f[0] = __uint_as_float(raw.x);
        f[1] = __uint_as_float(raw.y);
        f[2] = __uint_as_float(raw.z);
        f[3] = __uint_as_float(raw.w);
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    __device__ static __forceinline__ float to_float(float v) { return v; }
    __device__ static __forceinline__ float from_float(float v) { return v; }
    // 16-byte reduction into global memory: four float adds, no return value.  No "memory"
    // clobber on the reductions and streaming stores: their targets are never read by the
    // kernels, so gather loads of later points may be scheduled above them.
    __device__ static __forceinline__ void red_add(void *addr, const float (&f)[4]) {
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr),
                     "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]));
    }
};

template <> struct VecTraits<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float (&f)[8]) {
        // bf16 -> f32 is a 16-bit shift: low half by shl, high half by mask
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        uint32_t r;  // cvt packs {hi, lo} with round-to-nearest-even
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
        return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]),
                          pack2(f[6], f[7]));
    }
    __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_float(float v) {
        return __float2bfloat16_rn(v);
    }
    // one 16-byte packed reduction (eight bf16 adds) instead of four bf16x2 atomics
    __device__ static __forceinline__ void red_add(void *addr, const float (&f)[8]) {
        const uint4 p = pack(f);
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                         addr),
                     "r"(p.x), "r"(p.y), "r"(p.z), "r"(p.w));
    }
};

template <> struct VecTraits<__half> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ void unpack(const uint4 &raw, float (&f)[8]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
        return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]),
                          pack2(f[6], f[7]));
    }
    __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
    __device__ static __forceinline__ void red_add(void *addr, const float (&f)[8]) {
        const uint4 p = pack(f);
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(
                         addr),
                     "r"(p.x), "r"(p.y), "r"(p.z), "r"(p.w));
    }
};

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

// read-only 16-byte gather load (value is never written by these kernels)
__device__ __forceinline__ uint4 ldg16(const void *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}

// streaming 16-byte load/store for operands touched exactly once (loc, attn, out, grads):
// keeps them from displacing the value tensor in L1/L2
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

// Copy n floats global -> shared with 16-byte streaming loads (src 16-byte aligned).
__device__ __forceinline__ void stage_f32(float *dst, const float *src, int n) {
    const int n4 = n >> 2;
    for (int i = threadIdx.x; i < n4; i += kThreads)
        reinterpret_cast<uint4 *>(dst)[i] = ld_stream16(reinterpret_cast<const uint4 *>(src) + i);
    for (int i = (n4 << 2) + threadIdx.x; i < n; i += kThreads) dst[i] = src[i];
}

// Copy n elements of T global -> shared as float (src 16-byte aligned).
template <typename T>
__device__ __forceinline__ void stage_as_f32(float *dst, const T *src, int n) {
    using VT = VecTraits<T>;
    constexpr int V = VT::kVec;
    const int nv = n / V;
    for (int i = threadIdx.x; i < nv; i += kThreads) {
        float f[V];
        VT::unpack(ld_stream16(reinterpret_cast<const uint4 *>(src) + i), f);
#pragma unroll
        for (int j = 0; j < V; ++j) dst[i * V + j] = f[j];
    }
    for (int i = nv * V + threadIdx.x; i < n; i += kThreads) dst[i] = VT::to_float(src[i]);
}

// ---------------------------------------------------------------------------------
// One sample point: pixel mapping, skip test, corner offsets and weights
// ---------------------------------------------------------------------------------
struct Corners {
    float w[4];     // bilinear weights, order (r0,c0) (r0,c0+1) (r0+1,c0) (r0+1,c0+1)
    int off[4];     // pixel index r*W + c inside the level (valid corners only)
    bool ok[4];     // corner lies inside the level
    float fr, fc;   // fractional parts along height / width
    bool inside;    // point passes -1 <= pix < size on both axes (NaN/inf fail)
};

__device__ __forceinline__ Corners locate(float x, float y, int H, int W) {
    Corners c;
    const float Hf = (float)H, Wf = (float)W;
    // pixel = loc * size - 0.5, always in float32
    const float px = fmaf(x, Wf, -0.5f);
    const float py = fmaf(y, Hf, -0.5f);
    c.inside = (py >= -1.f) && (px >= -1.f) && (py < Hf) && (px < Wf);
    // keep the arithmetic finite for skipped points (their loads are predicated off)
    const float sx = c.inside ? px : 0.f;
    const float sy = c.inside ? py : 0.f;
    const float r0f = floorf(sy), c0f = floorf(sx);
    const int r0 = (int)r0f, c0 = (int)c0f;
    c.fr = sy - r0f;
    c.fc = sx - c0f;
    const bool r_ok0 = c.inside && r0 >= 0, r_ok1 = c.inside && r0 + 1 < H;
    const bool c_ok0 = c0 >= 0, c_ok1 = c0 + 1 < W;
    const float wr0 = 1.f - c.fr, wc0 = 1.f - c.fc;
    c.w[0] = wr0 * wc0;
    c.w[1] = wr0 * c.fc;
    c.w[2] = c.fr * wc0;
    c.w[3] = c.fr * c.fc;
    c.ok[0] = r_ok0 && c_ok0;
    c.ok[1] = r_ok0 && c_ok1;
    c.ok[2] = r_ok1 && c_ok0;
    c.ok[3] = r_ok1 && c_ok1;
    const int o = r0 * W + c0;
    c.off[0] = o;
    c.off[1] = o + 1;
    c.off[2] = o + W;
    c.off[3] = o + W + 1;
    return c;
}

// Level table -> shared memory (read from device memory: no host synchronisation)
struct LevelTable {
    int H[kMaxLevels];
    int W[kMaxLevels];
    int start[kMaxLevels];   // first position of the level on the S axis (< 2^31)
};

__device__ __forceinline__ void load_level_table(LevelTable &t, const Params &p) {
    if (threadIdx.x < p.L) {
        t.H[threadIdx.x] = (int)p.spatial_shapes[2 * threadIdx.x];
        t.W[threadIdx.x] = (int)p.spatial_shapes[2 * threadIdx.x + 1];
        t.start[threadIdx.x] = (int)p.level_start_index[threadIdx.x];
    }
}

// launchers implemented in msda_forward.cu / msda_backward.cu; dtype: 0 f32, 1 f16, 2 bf16
cudaError_t launch_forward(const Params &p, int dtype, bool softmax, cudaStream_t stream);
cudaError_t launch_backward(const Params &p, int dtype, bool softmax, cudaStream_t stream);
size_t forward_smem_bytes(const Params &p);
size_t backward_smem_bytes(const Params &p, bool softmax);

}  // namespace msda_b200
