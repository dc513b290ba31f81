// Native registration of the private operators with the torch dispatcher, for processes that
// run exported programs (AOTInductor packages, TorchScript-free C++ runtimes) without Python.
//
// The Python package registers the same operators itself (deformops_b200/ops.py: schemas,
// CUDA implementations over ctypes, fake kernels, autograd) and never loads this library.  A
// process that has no Python side loads libmsda_b200_torch.so instead
// (torch.ops.load_library / dlopen): the static initialisers below define the schemas and
// attach CUDA implementations that allocate the outputs and call the C ABI of libmsda_b200.so
// on the caller's current stream.  Inference and explicit backward calls only: the autograd
// formula lives in Python.  Do not load both into one process (the schemas would be defined
// twice).
//
// Plays the role of the reference's static registration
//   sources/deformops/backends/cuda/msda_fp32acc.cu:20-25 (STABLE_TORCH_LIBRARY_IMPL)
//   sources/deformops/backends/cuda/include/msda_boxed.cuh:14-53
// with the same operator schemas (sources/deformops/backends/cuda/_schema.py:18-29).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <tuple>

#include "../../include/msda_b200.h"

namespace {

int dtype_code(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return MSDA_B200_F32;
        case at::kHalf: return MSDA_B200_F16;
        case at::kBFloat16: return MSDA_B200_BF16;
        case at::kDouble: return MSDA_B200_F64;
        default: TORCH_CHECK(false, "deformops_b200: unsupported value dtype ", t);
    }
}

struct Dims {
    int64_t B, S, G, D, Q, L, K;
};

Dims check(const at::Tensor &value, const at::Tensor &shapes, const at::Tensor &starts,
           const at::Tensor &loc, const at::Tensor &attn, int64_t K) {
    TORCH_CHECK(value.is_cuda(), "deformops_b200 kernels run on CUDA tensors only");
    TORCH_CHECK(value.dim() == 4 && loc.dim() == 6 && shapes.dim() == 2 && starts.dim() == 1,
                "deformops_b200: value (B,S,G,D), loc (B,Q,G,L,K,2), shapes (L,2), starts (L)");
    const bool f64 = value.scalar_type() == at::kDouble;
    TORCH_CHECK(loc.scalar_type() == (f64 ? at::kDouble : at::kFloat),
                "deformops_b200: sampling locations must be float32 (float64 with float64 values)");
    TORCH_CHECK(attn.scalar_type() == value.scalar_type(),
                "deformops_b200: attention weights must have the value dtype");
    TORCH_CHECK(shapes.scalar_type() == at::kLong && starts.scalar_type() == at::kLong,
                "deformops_b200: spatial_shapes and level_start_index must be int64");
    for (const at::Tensor *t : {&value, &shapes, &starts, &loc, &attn}) {
        TORCH_CHECK(t->is_contiguous(), "deformops_b200: operands must be contiguous");
        TORCH_CHECK(t->device() == value.device(), "deformops_b200: operands on different devices");
    }
    TORCH_CHECK(loc.size(4) == K, "deformops_b200: K does not match the locations");
    return {value.size(0), value.size(1), value.size(2), value.size(3),
            loc.size(1),   loc.size(3),   loc.size(4)};
}

// The C ABI wants 16-byte aligned operands.  Torch's allocations are, a view at an odd storage
// offset is not: such an operand is copied (what the Python side does as well).
at::Tensor aligned(const at::Tensor &t) {
    return reinterpret_cast<uintptr_t>(t.const_data_ptr()) % 16 == 0 ? t : t.clone();
}

void raise(int status, const char *what) {
    TORCH_CHECK(status == MSDA_B200_OK, what, " failed with status ", status, ": ",
                msda_b200_last_error());
}

template <bool SOFTMAX>
at::Tensor forward(const at::Tensor &value_in, const at::Tensor &shapes, const at::Tensor &starts,
                   const at::Tensor &loc_in, const at::Tensor &attn_in, int64_t /*chunk_step*/,
                   int64_t K, int64_t /*channels_per_thread*/, int64_t /*threads_per_block*/) {
    const Dims d = check(value_in, shapes, starts, loc_in, attn_in, K);
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = aligned(value_in), loc = aligned(loc_in), attn = aligned(attn_in);
    at::Tensor out = at::empty({d.B, d.Q, d.G * d.D}, value.options());
    if (d.B == 0 || d.Q == 0) return out;
    const int st = msda_b200_forward(
        value.const_data_ptr(), shapes.const_data_ptr<int64_t>(), starts.const_data_ptr<int64_t>(),
        static_cast<const float *>(loc.const_data_ptr()), attn.const_data_ptr(),
        out.mutable_data_ptr(), d.B, d.S, d.G, d.D, d.Q, d.L, d.K, dtype_code(value.scalar_type()),
        SOFTMAX, value.device().index(), c10::cuda::getCurrentCUDAStream().stream());
    raise(st, "msda_b200_forward");
    return out;
}

template <bool SOFTMAX>
std::tuple<at::Tensor, at::Tensor, at::Tensor> backward(
    const at::Tensor &value_in, const at::Tensor &shapes, const at::Tensor &starts,
    const at::Tensor &loc_in, const at::Tensor &attn_in, const at::Tensor &grad_output_in,
    int64_t /*chunk_step*/, int64_t K, int64_t /*channels_per_thread*/,
    int64_t /*threads_per_block*/) {
    const Dims d = check(value_in, shapes, starts, loc_in, attn_in, K);
    TORCH_CHECK(grad_output_in.scalar_type() == value_in.scalar_type() && grad_output_in.is_contiguous(),
                "deformops_b200: grad_output must be contiguous and have the value dtype");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = aligned(value_in), loc = aligned(loc_in), attn = aligned(attn_in),
                     grad_output = aligned(grad_output_in);
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_loc = at::empty_like(loc);
    at::Tensor grad_attn = at::empty_like(attn);
    if (d.B == 0) return {grad_value, grad_loc, grad_attn};
    const int code = dtype_code(value.scalar_type());
    // scratch of a 16-bit backward (scaled float16 image), from torch's caching allocator
    const int64_t nbytes = d.Q > 0 ? msda_b200_backward_scratch_bytes(d.B, d.S, d.G, d.D, d.Q, d.L, d.K, code) : 0;
    at::Tensor scratch;
    if (nbytes > 0) scratch = at::empty({nbytes}, value.options().dtype(at::kByte));
    const int st = msda_b200_backward(
        value.const_data_ptr(), shapes.const_data_ptr<int64_t>(), starts.const_data_ptr<int64_t>(),
        static_cast<const float *>(loc.const_data_ptr()), attn.const_data_ptr(),
        grad_output.const_data_ptr(), grad_value.mutable_data_ptr(),
        static_cast<float *>(grad_loc.mutable_data_ptr()), grad_attn.mutable_data_ptr(),
        nbytes > 0 ? scratch.mutable_data_ptr() : nullptr, nbytes, 0, d.B, d.S, d.G, d.D, d.Q, d.L,
        d.K, code, SOFTMAX, 1, value.device().index(),
        c10::cuda::getCurrentCUDAStream().stream());
    raise(st, "msda_b200_backward");
    return {grad_value, grad_loc, grad_attn};
}

// ---- fused location arithmetic: reference points + predicted offsets instead of locations ----
Dims check_offsets(const at::Tensor &value, const at::Tensor &shapes, const at::Tensor &starts,
                   const at::Tensor &ref, const at::Tensor &offsets, const at::Tensor &attn) {
    TORCH_CHECK(value.is_cuda(), "deformops_b200 kernels run on CUDA tensors only");
    TORCH_CHECK(value.dim() == 4 && offsets.dim() == 6 && offsets.size(5) == 2 && shapes.dim() == 2 &&
                    starts.dim() == 1,
                "deformops_b200: value (B,S,G,D), offsets (B,Q,G,L,K,2), shapes (L,2), starts (L)");
    TORCH_CHECK(value.scalar_type() != at::kDouble,
                "deformops_b200: float64 values take locations, not offsets");
    TORCH_CHECK(offsets.scalar_type() == at::kFloat || offsets.scalar_type() == value.scalar_type(),
                "deformops_b200: offsets must be float32 or the value dtype");
    TORCH_CHECK(attn.scalar_type() == value.scalar_type(),
                "deformops_b200: attention weights must have the value dtype");
    TORCH_CHECK(shapes.scalar_type() == at::kLong && starts.scalar_type() == at::kLong,
                "deformops_b200: spatial_shapes and level_start_index must be int64");
    TORCH_CHECK(ref.scalar_type() == at::kFloat, "deformops_b200: reference points must be float32");
    for (const at::Tensor *t : {&value, &shapes, &starts, &ref, &offsets, &attn}) {
        TORCH_CHECK(t->is_contiguous(), "deformops_b200: operands must be contiguous");
        TORCH_CHECK(t->device() == value.device(), "deformops_b200: operands on different devices");
    }
    const Dims d{value.size(0), value.size(1), value.size(2), value.size(3),
                 offsets.size(1), offsets.size(3), offsets.size(4)};
    TORCH_CHECK(ref.dim() == 4 && ref.size(0) == d.B && ref.size(1) == d.Q && ref.size(2) == d.L &&
                    (ref.size(3) == 2 || ref.size(3) == 4),
                "deformops_b200: reference points must be (B, Q, L, 2 or 4)");
    return d;
}

at::Tensor offsets_forward(const at::Tensor &value_in, const at::Tensor &shapes, const at::Tensor &starts,
                           const at::Tensor &ref_in, const at::Tensor &offsets_in,
                           const at::Tensor &attn_in, bool softmax) {
    const Dims d = check_offsets(value_in, shapes, starts, ref_in, offsets_in, attn_in);
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = aligned(value_in), ref = aligned(ref_in), offsets = aligned(offsets_in),
                     attn = aligned(attn_in);
    at::Tensor out = at::empty({d.B, d.Q, d.G * d.D}, value.options());
    if (d.B == 0 || d.Q == 0) return out;
    const int st = msda_b200_forward_offsets(
        value.const_data_ptr(), shapes.const_data_ptr<int64_t>(), starts.const_data_ptr<int64_t>(),
        ref.const_data_ptr<float>(), (int)ref.size(3), offsets.const_data_ptr(),
        dtype_code(offsets.scalar_type()), attn.const_data_ptr(), out.mutable_data_ptr(), d.B, d.S, d.G,
        d.D, d.Q, d.L, d.K, dtype_code(value.scalar_type()), softmax, value.device().index(),
        c10::cuda::getCurrentCUDAStream().stream());
    raise(st, "msda_b200_forward_offsets");
    return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> offsets_backward(
    const at::Tensor &value_in, const at::Tensor &shapes, const at::Tensor &starts,
    const at::Tensor &ref_in, const at::Tensor &offsets_in, const at::Tensor &attn_in,
    const at::Tensor &grad_output_in, bool softmax) {
    const Dims d = check_offsets(value_in, shapes, starts, ref_in, offsets_in, attn_in);
    TORCH_CHECK(grad_output_in.scalar_type() == value_in.scalar_type() && grad_output_in.is_contiguous(),
                "deformops_b200: grad_output must be contiguous and have the value dtype");
    const c10::cuda::CUDAGuard guard(value_in.device());
    const at::Tensor value = aligned(value_in), ref = aligned(ref_in), offsets = aligned(offsets_in),
                     attn = aligned(attn_in), grad_output = aligned(grad_output_in);
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_offsets = at::empty_like(offsets);
    at::Tensor grad_attn = at::empty_like(attn);
    if (d.B == 0) return {grad_value, grad_offsets, grad_attn};
    const int code = dtype_code(value.scalar_type());
    const int64_t nbytes = d.Q > 0 ? msda_b200_backward_scratch_bytes(d.B, d.S, d.G, d.D, d.Q, d.L, d.K, code) : 0;
    at::Tensor scratch;
    if (nbytes > 0) scratch = at::empty({nbytes}, value.options().dtype(at::kByte));
    const int st = msda_b200_backward_offsets(
        value.const_data_ptr(), shapes.const_data_ptr<int64_t>(), starts.const_data_ptr<int64_t>(),
        ref.const_data_ptr<float>(), (int)ref.size(3), offsets.const_data_ptr(),
        dtype_code(offsets.scalar_type()), attn.const_data_ptr(), grad_output.const_data_ptr(),
        grad_value.mutable_data_ptr(), grad_offsets.mutable_data_ptr(), grad_attn.mutable_data_ptr(),
        nbytes > 0 ? scratch.mutable_data_ptr() : nullptr, nbytes, 0, d.B, d.S, d.G, d.D, d.Q, d.L, d.K,
        code, softmax, 1, value.device().index(), c10::cuda::getCurrentCUDAStream().stream());
    raise(st, "msda_b200_backward_offsets");
    return {grad_value, grad_offsets, grad_attn};
}

constexpr const char *kForwardArgs =
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
    "int chunk_step, int K, int channels_per_thread, int threads_per_block) -> Tensor";
constexpr const char *kBackwardArgs =
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
    "Tensor grad_output, int chunk_step, int K, int channels_per_thread, "
    "int threads_per_block) -> (Tensor, Tensor, Tensor)";

}  // namespace

TORCH_LIBRARY_FRAGMENT(deformops_b200, m) {
    m.def((std::string("msda_forward") + kForwardArgs).c_str());
    m.def((std::string("msda_softmax_forward") + kForwardArgs).c_str());
    m.def((std::string("msda_backward") + kBackwardArgs).c_str());
    m.def((std::string("msda_softmax_backward") + kBackwardArgs).c_str());
    // what the default layer (fused location arithmetic) and the Hugging Face replacements call
    m.def("msda_offsets_forward(Tensor value, Tensor spatial_shapes, Tensor level_start_index, "
          "Tensor reference_points, Tensor offsets, Tensor attn, bool softmax) -> Tensor");
    m.def("msda_offsets_backward(Tensor value, Tensor spatial_shapes, Tensor level_start_index, "
          "Tensor reference_points, Tensor offsets, Tensor attn, Tensor grad_output, bool softmax) "
          "-> (Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(deformops_b200, CUDA, m) {
    m.impl("msda_forward", &forward<false>);
    m.impl("msda_softmax_forward", &forward<true>);
    m.impl("msda_backward", &backward<false>);
    m.impl("msda_softmax_backward", &backward<true>);
    m.impl("msda_offsets_forward", &offsets_forward);
    m.impl("msda_offsets_backward", &offsets_backward);
}
