// Host side of the two hottest wrappers in C++: a Python call of the fused RMSNorm+quant or
// SwiGLU+quant wrapper costs about 20 us when the output tensors are allocated from Python
// (three torch.empty calls, a ctypes marshal), more than the 12 us the kernel takes at the small
// benchmark shapes.  The same steps from C++ -- allocate through ATen, take the current stream,
// call the C ABI of include/linghe_b200.h -- cost a few microseconds.  Nothing here computes:
// this is the argument handling of linghe_b200/utils/norm.py and utils/silu.py, restated, in
// front of the same two entry points, with the same return contract as the upstream wrappers
// (linghe/utils/norm.py:343-502, linghe/utils/silu.py:279-335).
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstdint>
#include <optional>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "linghe_b200.h"

namespace {

using OptT = std::optional<at::Tensor>;

[[noreturn]] void raise_assert(const std::string& msg) {
    PyErr_SetString(PyExc_AssertionError, msg.c_str());
    throw py::error_already_set();
}

int dtype_code(const at::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kBFloat16: return LH_BF16;
        case at::kHalf: return LH_F16;
        case at::kFloat: return LH_F32;
        default: raise_assert("unsupported dtype");
    }
}

// argument errors are AssertionError (the upstream wrappers use bare asserts), CUDA errors RuntimeError
void check_rc(int rc, const char* name) {
    if (rc == LH_OK) return;
    const std::string msg = lh_last_error();
    if (rc == LH_ERR_ARG) raise_assert(msg);
    throw std::runtime_error(std::string("linghe_b200 ") + name + ": CUDA error " + std::to_string(rc) + ": " + msg);
}

void check_device(const at::Tensor& x) {
    if (!x.is_cuda()) throw std::runtime_error("linghe_b200 runs on CUDA tensors only (no CPU fallback)");
    static bool checked[64] = {};
    const int idx = x.get_device();
    if (idx >= 0 && idx < 64 && !checked[idx]) {
        if (lh_device_check(idx) != LH_OK) throw std::runtime_error(std::string("linghe_b200: ") + lh_last_error());
        checked[idx] = true;
    }
}

void* ptr(const OptT& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// (out, scale, rms, transpose_output, transpose_scale); entries a mode does not produce and the
// caller did not pass are None, except the transposed pair, which upstream always allocates
std::tuple<OptT, OptT, at::Tensor, at::Tensor, at::Tensor> rms_norm_and_block_quant_forward(
    const at::Tensor& x, const at::Tensor& weight, double eps, OptT out, OptT scale, OptT rms, bool round_scale,
    int64_t output_mode) {
    if (!x.is_contiguous() || !weight.is_contiguous()) raise_assert("x and weight must be contiguous");
    if (x.dim() != 2) raise_assert("x must be 2-D");
    const int64_t M = x.size(0), n = x.size(1);
    if (n > 8192) raise_assert("n <= 8192");
    if (output_mode < 0 || output_mode > 2) raise_assert("output_mode in (0, 1, 2)");
    if (output_mode == 0 && rms.has_value()) raise_assert("rms must be None in output_mode 0");
    if (output_mode == 1 && !rms.has_value()) raise_assert("rms is required in output_mode 1");
    check_device(x);
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    const auto fp8 = x.options().dtype(at::kFloat8_e4m3fn);
    const auto f32 = x.options().dtype(at::kFloat);
    if (output_mode != 1) {
        if (!out.has_value()) out = at::empty({M, n}, fp8);
        if (!scale.has_value()) scale = at::empty({n / 128, M}, f32);
    }
    at::Tensor tq, ts;
    if (output_mode != 0) {
        tq = at::empty({n, M}, fp8);
        ts = at::empty({(M + 127) / 128, n}, f32);
    }
    if (output_mode != 1) rms = at::empty({M}, f32);
    const int rc = lh_rmsnorm_blockquant_fwd(x.data_ptr(), weight.data_ptr(), dtype_code(x), M, n, float(eps),
                                             output_mode != 1 ? ptr(out) : nullptr,
                                             output_mode != 1 ? static_cast<float*>(ptr(scale)) : nullptr,
                                             static_cast<float*>(ptr(rms)), tq.defined() ? tq.data_ptr() : nullptr,
                                             ts.defined() ? static_cast<float*>(ts.data_ptr()) : nullptr, round_scale ? 1 : 0,
                                             int(output_mode), c10::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "lh_rmsnorm_blockquant_fwd");
    if (!tq.defined()) {   // not written in mode 0: allocated behind the launch, where it delays nothing
        tq = at::empty({n, M}, fp8);
        ts = at::empty({(M + 127) / 128, n}, f32);
    }
    return {out, scale, *rms, tq, ts};
}

// (out, scale, transpose_output, transpose_scale)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> silu_and_block_quant_forward(const at::Tensor& x, OptT out,
                                                                                        OptT scale, bool round_scale,
                                                                                        int64_t output_mode) {
    if (!x.is_contiguous()) raise_assert("x must be contiguous");
    if (x.dim() != 2) raise_assert("x must be 2-D");
    const int64_t M = x.size(0), n = x.size(1) / 2;
    // upstream tiles the width by 128 columns, by 64 when only the transposed pair is written
    if (n % (output_mode == 1 ? 64 : 128) != 0) raise_assert("n % 128 == 0 (n % 64 == 0 in output_mode 1)");
    check_device(x);
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    const auto fp8 = x.options().dtype(at::kFloat8_e4m3fn);
    const auto f32 = x.options().dtype(at::kFloat);
    if (!out.has_value()) out = at::empty({M, n}, fp8);
    if (!scale.has_value()) scale = at::empty({n / 128, M}, f32);
    at::Tensor tq, ts;
    if (output_mode != 0) {
        tq = at::empty({n, M}, fp8);
        ts = at::empty({(M + 127) / 128, n}, f32);
    }
    const int rc = lh_silu_blockquant_fwd(x.data_ptr(), dtype_code(x), M, n, out->data_ptr(),
                                          static_cast<float*>(scale->data_ptr()), tq.defined() ? tq.data_ptr() : nullptr,
                                          ts.defined() ? static_cast<float*>(ts.data_ptr()) : nullptr, round_scale ? 1 : 0,
                                          int(output_mode), c10::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "lh_silu_blockquant_fwd");
    if (!tq.defined()) {
        tq = at::empty({n, M}, fp8);
        ts = at::empty({(M + 127) / 128, n}, f32);
    }
    return {*out, *scale, tq, ts};
}

// Several uninitialised tensors on the device of `ref` from one call: specs = [(shape, code), ...]
// with code 0 e4m3, 1 float32, 2 bfloat16, 3 float16, 4 uint8, 5 int32, 6 int64.  One
// Python -> C++ transition instead of one per torch.empty.
std::vector<at::Tensor> empty_many(const at::Tensor& ref, const std::vector<std::pair<std::vector<int64_t>, int>>& specs) {
    static const at::ScalarType kinds[] = {at::kFloat8_e4m3fn, at::kFloat, at::kBFloat16, at::kHalf, at::kByte, at::kInt, at::kLong};
    if (!ref.is_cuda()) throw std::runtime_error("linghe_b200 runs on CUDA tensors only (no CPU fallback)");
    std::vector<at::Tensor> out;
    out.reserve(specs.size());
    const c10::cuda::OptionalCUDAGuard guard(ref.device());
    for (const auto& sp : specs) {
        if (sp.second < 0 || sp.second > 6) raise_assert("empty_many: unknown dtype code");
        out.push_back(at::empty(sp.first, ref.options().dtype(kinds[sp.second])));
    }
    return out;
}

uintptr_t current_stream(int device) { return reinterpret_cast<uintptr_t>(c10::cuda::getCurrentCUDAStream(device).stream()); }

}  // namespace

PYBIND11_MODULE(_lh_host, m) {
    m.doc() = "C++ argument handling for the hottest linghe_b200 wrappers (allocation + C-ABI call)";
    m.def("empty_many", &empty_many);
    m.def("current_stream", &current_stream);
#include "lh_host_bindings.inc"
    m.def("rms_norm_and_block_quant_forward", &rms_norm_and_block_quant_forward);
    m.def("silu_and_block_quant_forward", &silu_and_block_quant_forward);
}
