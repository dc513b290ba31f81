// Hardware floors of the deformable-attention kernels, measured by kernels that do nothing else.
//
// Built into its own library (libmsda_b200_floors.so) and loaded by bench.py only; the operator
// library does not contain or call any of this.  Each kernel takes the addresses it touches
// from a table the caller computes from a real workload (one 64-byte row of 32 16-bit channels
// per bilinear corner), so the access pattern is the operator's, minus every other instruction:
//
//   floors_red_rows     one packed 16-byte reduction per lane into `dst`; four lanes cover a row
//                       (what the backward's grad_value scatter costs on its way to L2)
//   floors_red_rows_on  the same from a given number of SMs only (one CTA of 32 warps each):
//                       shows whether the limit sits in the SMs or behind them
//   floors_bulk_red_rows  the same additions sent by the copy engine instead of the load/store
//                       unit: the warp stages its rows in shared memory and one lane per piece
//                       of 1, 2 or 4 adjacent rows issues cp.reduce.async.bulk (shows whether
//                       the other way out of the SM is any wider)
//   floors_gather_rows  one 16-byte read-only load per lane; four lanes cover a row
//                       (what the forward's and backward's corner gather costs in L1 / L2)
//   floors_gather_red_rows  both: every lane loads its 16 bytes of a row of `src` and adds 16
//                       bytes into the same row of `dst`, eight rows in flight per lane, the
//                       rows dealt to CTAs and warps as the backward kernel deals its queries, with
//                       as much idle shared memory per CTA as the caller says (the backward
//                       kernel's, so that L1 keeps the capacity it has there) - the backward
//                       kernel minus its arithmetic, descriptors and gradient write-out
//   floors_mma          back-to-back mma.sync m16n8k16 bf16 instructions, eight independent
//                       accumulator sets per warp (legacy tensor-core issue rate of one SM)
//   floors_smem_rmw     16-byte load / packed add / store on warp-private shared memory rows
//
// All return a CUDA error code; timing is done by the caller with events on `stream`.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 256;

// mode: 0 bf16x2, 1 f16x2
template <int MODE, int THREADS>
__global__ void __launch_bounds__(THREADS) red_rows_kernel(uint16_t *dst, const uint32_t *row_off,
                                                         int64_t rows) {
    const int sub = threadIdx.x & 3;
    const int64_t stride = (int64_t)gridDim.x * (THREADS / 4);
    const uint32_t one = MODE == 0 ? 0x3c003c00u : 0x14001400u;   // small finite addends
    for (int64_t r = (int64_t)blockIdx.x * (THREADS / 4) + (threadIdx.x >> 2); r < rows; r += stride) {
        uint16_t *a = dst + row_off[r] + sub * 8;
        if (MODE == 0)
            asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %1, %1, %1};" ::"l"(a),
                         "r"(one));
        else
            asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %1, %1, %1};" ::"l"(a),
                         "r"(one));
    }
}

// RPP adjacent 64-byte rows per bulk reduction; a warp turn stages eight rows (512 bytes) in one
// of NS ring slots and 8 / RPP lanes send them.  The waits are the bulk-group waits of the
// issuing lanes on their own groups: they end when the engine has read the slot.
template <int RPP>
__global__ void __launch_bounds__(kThreads) bulk_red_rows_kernel(uint16_t *dst, const uint32_t *row_off,
                                                               int64_t rows) {
    constexpr int NS = 4;
    constexpr int OPS = 8 / RPP;
    constexpr int PIECE = RPP * 64;
    __shared__ __align__(128) unsigned char stage[kThreads / 32][NS][512];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t turns = rows / 8;
    const int64_t stride = (int64_t)gridDim.x * (kThreads / 32);
    const uint4 addend = make_uint4(0x14001400u, 0x14001400u, 0x14001400u, 0x14001400u);
    int slot = 0;
    for (int64_t t = (int64_t)blockIdx.x * (kThreads / 32) + w; t < turns; t += stride) {
        if (lane < OPS) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(NS - 1) : "memory");
        __syncwarp();
        *reinterpret_cast<uint4 *>(&stage[w][slot][lane * 16]) = addend;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane < OPS) {
            // the piece that holds this lane's first row, at a multiple of the piece size
            const uint32_t first = row_off[t * 8 + lane * RPP] / (32u * RPP) * (32u * RPP);
            const uint32_t src = (uint32_t)__cvta_generic_to_shared(&stage[w][slot][lane * PIECE]);
            asm volatile(
                "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(
                    dst + first),
                "r"(src), "n"(PIECE)
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        slot = (slot + 1) % NS;
    }
    if (lane < OPS) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads) gather_rows_kernel(const uint16_t *src,
                                                             const uint32_t *row_off, int64_t rows,
                                                             uint32_t *sink) {
    const int sub = threadIdx.x & 3;
    const int64_t stride = (int64_t)gridDim.x * (kThreads / 4);
    uint32_t acc = 0;
    for (int64_t r = (int64_t)blockIdx.x * (kThreads / 4) + (threadIdx.x >> 2); r < rows; r += stride) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src + row_off[r] + sub * 8));
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9e3779b9u) *sink = acc;   // keeps the loads alive; practically never taken
}

// The rows are walked the way the backward kernel walks its queries: the table is cut into
// blocks of `block_rows` consecutive rows (about one query's: its points, corners and heads), a
// CTA takes sixteen consecutive blocks, warp w of it blocks w and 8 + w, eight rows per
// instruction and eight instructions (two points' corners) in flight.
__global__ void __launch_bounds__(kThreads, 4) gather_red_rows_kernel(const uint16_t *src, uint16_t *dst,
                                                                    const uint32_t *row_off, int64_t rows,
                                                                    int block_rows) {
    constexpr int kInFlight = 8;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, sub = lane & 3, slot = lane >> 2;
    for (int pass = 0; pass < 2; ++pass) {
        const int64_t base = ((int64_t)blockIdx.x * 16 + pass * 8 + w) * block_rows;
        for (int i = 0; i < block_rows; i += 8 * kInFlight) {
            uint32_t off[kInFlight];
            uint4 v[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int64_t r = base + i + u * 8 + slot;
                off[u] = (i + u * 8 < block_rows && r < rows) ? row_off[r] : 0xffffffffu;
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (off[u] != 0xffffffffu)
                    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                                 : "l"(src + off[u] + sub * 8));
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (off[u] == 0xffffffffu) continue;
                // an addend that depends on what was loaded, and stays small whatever that was
                const uint32_t a = ((v[u].x ^ v[u].y ^ v[u].z ^ v[u].w) & 0x03ff03ffu) | 0x10001000u;
                asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %1, %1, %1};" ::"l"(
                                 dst + off[u] + sub * 8),
                             "r"(a)
                             : "memory");
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads) mma_kernel(int iters, float *sink) {
    float c[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
    uint32_t a0 = threadIdx.x, a1 = a0 * 3u, a2 = a0 * 5u, a3 = a0 * 7u, b0 = a0 * 11u, b1 = a0 * 13u;
    a0 &= 0x3f803f80u; a1 &= 0x3f803f80u; a2 &= 0x3f803f80u; a3 &= 0x3f803f80u;
    b0 &= 0x3f803f80u; b1 &= 0x3f803f80u;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, "
                "{%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                : "+f"(c[i][0]), "+f"(c[i][1]), "+f"(c[i][2]), "+f"(c[i][3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += c[i][0] + c[i][1] + c[i][2] + c[i][3];
    if (s == 12345.678f) *sink = s;
}

// every warp owns `rows_per_warp` 64-byte rows of shared memory; each 4-lane slot updates a
// pseudo-random row of its warp: 16-byte load, four packed half2 fused multiply-adds, 16-byte
// store (the cost of accumulating one corner's grad_value contribution on chip)
__global__ void __launch_bounds__(kThreads) smem_rmw_kernel(int iters, int rows_per_warp, uint32_t *sink) {
    extern __shared__ uint4 rows[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 3, slot = lane >> 2;
    uint4 *mine = rows + (size_t)warp * rows_per_warp * 4;
    for (int i = lane; i < rows_per_warp * 4; i += 32) mine[i] = make_uint4(0, 0, 0, 0);
    __syncwarp();
    uint32_t r = (blockIdx.x * kThreads + threadIdx.x) / 4 * 2654435761u + 12345u;
    const uint32_t m = 0x3c003c00u, w = 0x14001400u;
    for (int it = 0; it < iters; ++it) {
        r = r * 1664525u + 1013904223u;
        // slots of one warp instruction take distinct rows: row index = 8 * k + slot
        const int row = (int)(((r >> 8) % (uint32_t)(rows_per_warp / 8)) * 8 + slot);
        uint4 v = mine[row * 4 + sub];
        asm("fma.rn.f16x2 %0, %1, %2, %0;" : "+r"(v.x) : "r"(m), "r"(w));
        asm("fma.rn.f16x2 %0, %1, %2, %0;" : "+r"(v.y) : "r"(m), "r"(w));
        asm("fma.rn.f16x2 %0, %1, %2, %0;" : "+r"(v.z) : "r"(m), "r"(w));
        asm("fma.rn.f16x2 %0, %1, %2, %0;" : "+r"(v.w) : "r"(m), "r"(w));
        mine[row * 4 + sub] = v;
        __syncwarp();
    }
    const uint4 v = mine[lane];
    if ((v.x ^ v.y) == 0x9e3779b9u) *sink = v.x;
}

int grid_for(int ctas_per_sm) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms * ctas_per_sm;
}

}  // namespace

extern "C" {

// rows: number of 64-byte rows; row_off[i]: offset of row i in 16-bit elements from dst/src
int floors_red_rows(void *dst, const uint32_t *row_off, int64_t rows, int f16, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (f16)
        red_rows_kernel<1, kThreads><<<grid_for(8), kThreads, 0, s>>>(static_cast<uint16_t *>(dst), row_off, rows);
    else
        red_rows_kernel<0, kThreads><<<grid_for(8), kThreads, 0, s>>>(static_cast<uint16_t *>(dst), row_off, rows);
    return (int)cudaGetLastError();
}

// the float16 reductions again, issued by `sms` CTAs of 1024 threads: one CTA fills an SM, so
// only that many SMs take part
int floors_red_rows_on(void *dst, const uint32_t *row_off, int64_t rows, int sms, void *stream) {
    if (sms < 1) return (int)cudaErrorInvalidValue;
    red_rows_kernel<1, 1024><<<sms, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t *>(dst), row_off, rows);
    return (int)cudaGetLastError();
}

// rows_per_piece 1, 2 or 4; `dst` must hold a multiple of four rows and every row_off a multiple
// of 32 (a 64-byte row), which the caller's table of bilinear corner rows does
int floors_bulk_red_rows(void *dst, const uint32_t *row_off, int64_t rows, int rows_per_piece,
                         void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint16_t *d = static_cast<uint16_t *>(dst);
    if ((reinterpret_cast<uintptr_t>(dst) & 255) != 0) return (int)cudaErrorInvalidValue;
    switch (rows_per_piece) {
        case 1: bulk_red_rows_kernel<1><<<grid_for(4), kThreads, 0, s>>>(d, row_off, rows); break;
        case 2: bulk_red_rows_kernel<2><<<grid_for(4), kThreads, 0, s>>>(d, row_off, rows); break;
        case 4: bulk_red_rows_kernel<4><<<grid_for(4), kThreads, 0, s>>>(d, row_off, rows); break;
        default: return (int)cudaErrorInvalidValue;
    }
    return (int)cudaGetLastError();
}

int floors_gather_rows(const void *src, const uint32_t *row_off, int64_t rows, void *sink,
                       void *stream) {
    gather_rows_kernel<<<grid_for(8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(src), row_off, rows, static_cast<uint32_t *>(sink));
    return (int)cudaGetLastError();
}

// idle_smem_bytes: dynamic shared memory each CTA holds without using it; block_rows: rows of
// one block of the table (a multiple of 8; about the rows of one query), sixteen blocks per CTA
int floors_gather_red_rows(const void *src, void *dst, const uint32_t *row_off, int64_t rows,
                           int block_rows, int idle_smem_bytes, void *stream) {
    if (idle_smem_bytes < 0 || idle_smem_bytes > 48 * 1024 || block_rows < 8 || block_rows % 8 != 0)
        return (int)cudaErrorInvalidValue;
    const int64_t per_cta = 16ll * block_rows;
    const int64_t ctas = (rows + per_cta - 1) / per_cta;
    if (ctas < 1 || ctas > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    gather_red_rows_kernel<<<(unsigned)ctas, kThreads, (size_t)idle_smem_bytes,
                             static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(src), static_cast<uint16_t *>(dst), row_off, rows, block_rows);
    return (int)cudaGetLastError();
}

// launches sms * 4 CTAs of 8 warps; every warp issues iters * 8 instructions
int floors_mma(int iters, void *sink, int64_t *instructions, void *stream) {
    const int grid = grid_for(4);
    mma_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(iters, static_cast<float *>(sink));
    if (instructions) *instructions = (int64_t)grid * (kThreads / 32) * iters * 8;
    return (int)cudaGetLastError();
}

// launches sms * 4 CTAs of 8 warps; every warp performs iters row updates per 4-lane slot
int floors_smem_rmw(int iters, int rows_per_warp, void *sink, int64_t *row_updates, void *stream) {
    const int grid = grid_for(4);
    const size_t smem = (size_t)(kThreads / 32) * rows_per_warp * 64;
    if (rows_per_warp < 8 || rows_per_warp % 8 != 0 || smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    smem_rmw_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        iters, rows_per_warp, static_cast<uint32_t *>(sink));
    if (row_updates) *row_updates = (int64_t)grid * (kThreads / 4) * iters;
    return (int)cudaGetLastError();
}

}  // extern "C"
