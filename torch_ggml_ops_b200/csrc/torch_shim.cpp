// libtorch stable-ABI registration of the six torch_ggml_ops operators over the C ABI of
// libtgo_mmq.so.  This file holds no kernel and no arithmetic: it validates tensors the way the
// reference's native layer does (reference: csrc/mmq_hip.cu:325-519, 587-631, 680-736: same
// conditions, same fail-fast policy, error texts carrying the same key phrases), allocates the
// outputs and the per-call workspace with new_empty on the input's device, looks up the current
// stream and calls the matching tgo_* entry point.
//
// Schemas are those of the reference (csrc/mmq_hip.cu:1197-1215), byte for byte.
#include <Python.h>

#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/ops.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>
#include <torch/headeronly/macros/Macros.h>

#include <array>
#include <cstdint>
#include <limits>
#include <tuple>
#include <vector>

#include "../../include/tgo_mmq.h"

namespace {

using torch::headeronly::IntHeaderOnlyArrayRef;
using torch::headeronly::ScalarType;
using torch::stable::Tensor;

constexpr int64_t kSuperBlock = 256;
constexpr int64_t kIntMax = std::numeric_limits<int>::max();

int64_t block_bytes_or_throw(int64_t quant_type) {
    const int64_t bytes =
        quant_type >= 0 && quant_type <= kIntMax ? tgo_block_bytes(static_cast<int>(quant_type)) : -1;
    STD_TORCH_CHECK(bytes > 0, "unsupported quant_type: ", quant_type);
    return bytes;
}

void check_call(int rc, const char* what) {
    STD_TORCH_CHECK(rc == TGO_OK, what, " failed: ", tgo_last_error());
}

// Device residency, dtype, layout: the fail-fast part every tensor argument goes through.
void check_tensor(const Tensor& t, const char* name, ScalarType dtype, const char* dtype_name) {
    STD_TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    STD_TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", dtype_name);
    STD_TORCH_CHECK(t.is_contiguous(), name, " must be contiguous; torch_ggml_ops will not insert a hidden copy");
    STD_TORCH_CHECK(t.storage_offset() == 0, name, " must have zero storage offset");
}

void check_aligned(const Tensor& t, const char* name) {
    STD_TORCH_CHECK(reinterpret_cast<uintptr_t>(t.const_data_ptr()) % 16 == 0, name,
                    " data pointer must be 16-byte aligned");
}

void* current_stream(int32_t device_index) {
    void* stream = nullptr;
    TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(device_index, &stream));
    return stream;
}

Tensor new_bf16(const Tensor& like, const std::vector<int64_t>& sizes) {
    return torch::stable::new_empty(like, IntHeaderOnlyArrayRef(sizes.data(), sizes.size()), ScalarType::BFloat16);
}

Tensor new_bytes(const Tensor& like, int64_t bytes) {
    std::array<int64_t, 1> size{bytes};
    return torch::stable::new_empty(like, IntHeaderOnlyArrayRef(size.data(), size.size()), ScalarType::Byte);
}

// ---------------------------------------------------------------------------- dense
struct DenseShape {
    int64_t rows, red, other;  // rows, activation width, the weight's other dimension
};

// `act` is the input (forward, width = in_features) or grad_output (backward, width =
// out_features); `other_features` is the explicit integer argument of the op.
DenseShape check_dense(const Tensor& act, const char* act_name, const Tensor& packed, int64_t quant_type,
                       int64_t other_features, bool forward) {
    STD_TORCH_CHECK(act.is_cuda(), act_name, " must be a CUDA tensor");
    STD_TORCH_CHECK(packed.is_cuda(), "packed_weight must be a CUDA tensor");
    STD_TORCH_CHECK(act.get_device_index() == packed.get_device_index(), act_name,
                    " and packed_weight must be on the same device");
    check_tensor(act, act_name, ScalarType::BFloat16, "torch.bfloat16");
    check_tensor(packed, "packed_weight", ScalarType::Byte, "torch.uint8");
    STD_TORCH_CHECK(act.dim() >= 1, act_name, " must have at least one dimension");
    const int64_t width = act.size(act.dim() - 1);
    const int64_t in_features = forward ? width : other_features;
    const int64_t out_features = forward ? other_features : width;
    STD_TORCH_CHECK(in_features > 0 && in_features % kSuperBlock == 0,
                    forward ? "input width" : "in_features", " must be a positive multiple of 256; got ", in_features);
    STD_TORCH_CHECK(out_features > 0, forward ? "out_features must be positive; got "
                                              : "grad_output final dimension must be positive; got ", out_features);
    STD_TORCH_CHECK(act.numel() % width == 0, act_name, " numel is inconsistent with its final dimension");
    const int64_t rows = act.numel() / width;
    STD_TORCH_CHECK(rows > 0, "zero-row ", forward ? "inputs" : "grad_output tensors", " are not supported");
    STD_TORCH_CHECK(rows <= kIntMax, "flattened ", act_name, " row count exceeds the kernel limit");
    STD_TORCH_CHECK(in_features <= kIntMax, "in_features exceeds the kernel limit");
    STD_TORCH_CHECK(out_features <= kIntMax, "out_features exceeds the kernel limit");
    const int64_t expected = out_features * (in_features / kSuperBlock) * block_bytes_or_throw(quant_type);
    STD_TORCH_CHECK(packed.numel() == expected, "packed_weight has ", packed.numel(), " bytes, expected ", expected,
                    " for [", out_features, ", ", in_features, "] quant_type=", quant_type);
    check_aligned(act, act_name);
    check_aligned(packed, "packed_weight");
    return {rows, width, other_features};
}

Tensor mmq_op(const Tensor& input, const Tensor& packed_weight, int64_t quant_type, int64_t out_features) {
    const DenseShape s = check_dense(input, "input", packed_weight, quant_type, out_features, true);
    const int32_t device = input.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    std::vector<int64_t> sizes(input.sizes().begin(), input.sizes().end());
    sizes.back() = out_features;
    Tensor output = new_bf16(input, sizes);
    check_call(tgo_mmq_fwd(input.const_data_ptr(), packed_weight.const_data_ptr(), output.mutable_data_ptr(), s.rows,
                           out_features, s.red, static_cast<int>(quant_type), current_stream(device)),
               "mmq");
    return output;
}

Tensor mmq_grad_input_op(const Tensor& grad_output, const Tensor& packed_weight, int64_t quant_type,
                         int64_t in_features) {
    const DenseShape s = check_dense(grad_output, "grad_output", packed_weight, quant_type, in_features, false);
    const int32_t device = grad_output.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    std::vector<int64_t> sizes(grad_output.sizes().begin(), grad_output.sizes().end());
    sizes.back() = in_features;
    Tensor grad_input = new_bf16(grad_output, sizes);
    // few rows against very many out-features (an LM head): the reduction is split over the CTA
    // pairs and its fp32 partial sums need a per-call workspace, a fresh tensor like the outputs
    const int64_t ws_bytes = tgo_mmq_dx_workspace_bytes(s.rows, s.red, in_features, static_cast<int>(quant_type));
    if (ws_bytes > 0) {
        Tensor workspace = new_bytes(grad_output, ws_bytes);
        check_call(tgo_mmq_dx_ws(grad_output.const_data_ptr(), packed_weight.const_data_ptr(), grad_input.mutable_data_ptr(),
                                 s.rows, s.red, in_features, static_cast<int>(quant_type), workspace.mutable_data_ptr(),
                                 ws_bytes, current_stream(device)),
                   "mmq_grad_input");
        return grad_input;
    }
    check_call(tgo_mmq_dx(grad_output.const_data_ptr(), packed_weight.const_data_ptr(), grad_input.mutable_data_ptr(),
                          s.rows, s.red, in_features, static_cast<int>(quant_type), current_stream(device)),
               "mmq_grad_input");
    return grad_input;
}

// ---------------------------------------------------------------------------- grouped
struct GroupedShape {
    int64_t rows, in_features, out_features, experts, groups;
};

void check_routing(const Tensor& expert_indices, const Tensor& expert_offsets, int32_t device, const char* family) {
    STD_TORCH_CHECK(expert_indices.is_cuda(), "expert_indices must be a CUDA tensor");
    STD_TORCH_CHECK(expert_offsets.is_cuda(), "expert_offsets must be a CUDA tensor");
    STD_TORCH_CHECK(expert_indices.get_device_index() == device && expert_offsets.get_device_index() == device,
                    "all ", family, " tensors must be on the same device");
    check_tensor(expert_indices, "expert_indices", ScalarType::Long, "torch.int64");
    check_tensor(expert_offsets, "expert_offsets", ScalarType::Int, "torch.int32");
    STD_TORCH_CHECK(expert_indices.dim() == 1, "expert_indices must be one-dimensional");
    STD_TORCH_CHECK(expert_offsets.dim() == 1, "expert_offsets must be one-dimensional");
    STD_TORCH_CHECK(expert_indices.numel() == expert_offsets.numel(),
                    "expert_indices and expert_offsets must have equal lengths");
    STD_TORCH_CHECK(expert_indices.numel() > 0, family, " requires at least one active expert");
}

void check_grouped_weight(const Tensor& packed, const char* name, int32_t device, const char* family,
                          int64_t quant_type, int64_t in_features, int64_t out_features, int64_t experts) {
    STD_TORCH_CHECK(packed.is_cuda(), name, " must be a CUDA tensor");
    STD_TORCH_CHECK(packed.get_device_index() == device, "all ", family, " tensors must be on the same device");
    check_tensor(packed, name, ScalarType::Byte, "torch.uint8");
    STD_TORCH_CHECK(packed.dim() == 3, "grouped ", name,
                    " must have physical shape [experts, out_features, row_bytes]");
    STD_TORCH_CHECK(packed.size(0) == experts, name, " expert count does not match the first packed weight");
    const int64_t row_bytes = (in_features / kSuperBlock) * block_bytes_or_throw(quant_type);
    STD_TORCH_CHECK(packed.size(1) == out_features, name, " physical output dimension does not match out_features");
    STD_TORCH_CHECK(packed.size(2) == row_bytes, name, " has ", packed.size(2), " bytes per row, expected ", row_bytes,
                    " for in_features=", in_features, " quant_type=", quant_type);
    STD_TORCH_CHECK(packed.numel() == experts * out_features * row_bytes, name,
                    " byte count is inconsistent with its grouped physical shape");
    check_aligned(packed, name);
}

// `act` = input [rows, K] (forward) or grad_output [rows, N] (backward).
GroupedShape check_grouped(const Tensor& act, const char* act_name, const Tensor& packed, const char* packed_name,
                           const Tensor& expert_indices, const Tensor& expert_offsets, int64_t quant_type,
                           int64_t other_features, bool forward) {
    const char* family = forward ? "grouped MMQ" : "grouped MMQ backward";
    STD_TORCH_CHECK(act.is_cuda(), act_name, " must be a CUDA tensor");
    const int32_t device = act.get_device_index();
    check_tensor(act, act_name, ScalarType::BFloat16, "torch.bfloat16");
    STD_TORCH_CHECK(act.dim() == 2, "grouped MMQ ", act_name, " must have shape [rows, ",
                    forward ? "in_features]" : "out_features]");
    check_routing(expert_indices, expert_offsets, device, family);
    const int64_t rows = act.size(0);
    const int64_t in_features = forward ? act.size(1) : other_features;
    const int64_t out_features = forward ? other_features : act.size(1);
    STD_TORCH_CHECK(rows > 0, "zero-row ", forward ? "inputs" : "grad_output tensors", " are not supported");
    STD_TORCH_CHECK(in_features > 0 && in_features % kSuperBlock == 0,
                    forward ? "input width" : "in_features", " must be a positive multiple of 256; got ", in_features);
    STD_TORCH_CHECK(out_features > 0, "out_features must be positive; got ", out_features);
    STD_TORCH_CHECK(packed.dim() == 3, "grouped ", packed_name,
                    " must have physical shape [experts, out_features, row_bytes]");
    const int64_t experts = packed.size(0);
    const int64_t groups = expert_indices.numel();
    STD_TORCH_CHECK(experts > 0, packed_name, " must contain at least one expert");
    STD_TORCH_CHECK(groups <= experts, "active expert count exceeds packed expert count");
    STD_TORCH_CHECK(rows <= kIntMax && in_features <= kIntMax && out_features <= kIntMax && experts <= kIntMax,
                    "a dimension exceeds the kernel limit");
    check_grouped_weight(packed, packed_name, device, family, quant_type, in_features, out_features, experts);
    check_aligned(act, act_name);
    return {rows, in_features, out_features, experts, groups};
}

Tensor grouped_mmq_op(const Tensor& input, const Tensor& packed_weight, const Tensor& expert_indices,
                      const Tensor& expert_offsets, int64_t quant_type, int64_t out_features) {
    const GroupedShape s = check_grouped(input, "input", packed_weight, "packed_weight", expert_indices,
                                         expert_offsets, quant_type, out_features, true);
    const int32_t device = input.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    Tensor output = new_bf16(input, {s.rows, s.out_features});
    const int64_t ws_bytes = tgo_grouped_workspace_bytes(s.rows, s.groups);
    Tensor workspace = new_bytes(input, ws_bytes);
    check_call(tgo_grouped_fwd(input.const_data_ptr(), packed_weight.const_data_ptr(), nullptr,
                               output.mutable_data_ptr(), nullptr,
                               static_cast<const int64_t*>(expert_indices.const_data_ptr()),
                               static_cast<const int32_t*>(expert_offsets.const_data_ptr()), s.groups, s.experts,
                               s.rows, s.out_features, s.in_features, static_cast<int>(quant_type),
                               workspace.mutable_data_ptr(), ws_bytes, current_stream(device)),
               "grouped_mmq");
    return output;
}

std::tuple<Tensor, Tensor> grouped_mmq_pair_op(const Tensor& input, const Tensor& first_packed_weight,
                                               const Tensor& second_packed_weight, const Tensor& expert_indices,
                                               const Tensor& expert_offsets, int64_t quant_type,
                                               int64_t out_features) {
    const GroupedShape s = check_grouped(input, "input", first_packed_weight, "first_packed_weight", expert_indices,
                                         expert_offsets, quant_type, out_features, true);
    const int32_t device = input.get_device_index();
    check_grouped_weight(second_packed_weight, "second_packed_weight", device, "grouped MMQ", quant_type,
                         s.in_features, s.out_features, s.experts);
    torch::stable::accelerator::DeviceGuard guard(device);
    Tensor first = new_bf16(input, {s.rows, s.out_features});
    Tensor second = new_bf16(input, {s.rows, s.out_features});
    const int64_t ws_bytes = tgo_grouped_workspace_bytes(s.rows, s.groups);
    Tensor workspace = new_bytes(input, ws_bytes);
    check_call(tgo_grouped_fwd(input.const_data_ptr(), first_packed_weight.const_data_ptr(),
                               second_packed_weight.const_data_ptr(), first.mutable_data_ptr(),
                               second.mutable_data_ptr(),
                               static_cast<const int64_t*>(expert_indices.const_data_ptr()),
                               static_cast<const int32_t*>(expert_offsets.const_data_ptr()), s.groups, s.experts,
                               s.rows, s.out_features, s.in_features, static_cast<int>(quant_type),
                               workspace.mutable_data_ptr(), ws_bytes, current_stream(device)),
               "grouped_mmq_pair");
    return {first, second};
}

Tensor grouped_mmq_grad_input_op(const Tensor& grad_output, const Tensor& packed_weight, const Tensor& expert_indices,
                                 const Tensor& expert_offsets, int64_t quant_type, int64_t in_features) {
    const GroupedShape s = check_grouped(grad_output, "grad_output", packed_weight, "packed_weight", expert_indices,
                                         expert_offsets, quant_type, in_features, false);
    const int32_t device = grad_output.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    Tensor grad_input = new_bf16(grad_output, {s.rows, s.in_features});
    const int64_t ws_bytes = tgo_grouped_workspace_bytes(s.rows, s.groups);
    Tensor workspace = new_bytes(grad_output, ws_bytes);
    check_call(tgo_grouped_dx(grad_output.const_data_ptr(), nullptr, packed_weight.const_data_ptr(), nullptr,
                              grad_input.mutable_data_ptr(),
                              static_cast<const int64_t*>(expert_indices.const_data_ptr()),
                              static_cast<const int32_t*>(expert_offsets.const_data_ptr()), s.groups, s.experts,
                              s.rows, s.out_features, s.in_features, static_cast<int>(quant_type),
                              workspace.mutable_data_ptr(), ws_bytes, current_stream(device)),
               "grouped_mmq_grad_input");
    return grad_input;
}

Tensor grouped_mmq_pair_grad_input_op(const Tensor& first_grad_output, const Tensor& second_grad_output,
                                      const Tensor& first_packed_weight, const Tensor& second_packed_weight,
                                      const Tensor& expert_indices, const Tensor& expert_offsets, int64_t quant_type,
                                      int64_t in_features) {
    const GroupedShape s = check_grouped(first_grad_output, "first_grad_output", first_packed_weight,
                                         "first_packed_weight", expert_indices, expert_offsets, quant_type,
                                         in_features, false);
    const int32_t device = first_grad_output.get_device_index();
    STD_TORCH_CHECK(second_grad_output.is_cuda() && second_grad_output.get_device_index() == device,
                    "all grouped MMQ backward tensors must be on the same device");
    check_tensor(second_grad_output, "second_grad_output", ScalarType::BFloat16, "torch.bfloat16");
    STD_TORCH_CHECK(second_grad_output.dim() == 2 && second_grad_output.size(0) == s.rows &&
                        second_grad_output.size(1) == s.out_features,
                    "first_grad_output and second_grad_output must have the same shape");
    check_aligned(second_grad_output, "second_grad_output");
    check_grouped_weight(second_packed_weight, "second_packed_weight", device, "grouped MMQ backward", quant_type,
                         s.in_features, s.out_features, s.experts);
    torch::stable::accelerator::DeviceGuard guard(device);
    Tensor grad_input = new_bf16(first_grad_output, {s.rows, s.in_features});
    const int64_t ws_bytes = tgo_grouped_workspace_bytes(s.rows, s.groups);
    Tensor workspace = new_bytes(first_grad_output, ws_bytes);
    check_call(tgo_grouped_dx(first_grad_output.const_data_ptr(), second_grad_output.const_data_ptr(),
                              first_packed_weight.const_data_ptr(), second_packed_weight.const_data_ptr(),
                              grad_input.mutable_data_ptr(),
                              static_cast<const int64_t*>(expert_indices.const_data_ptr()),
                              static_cast<const int32_t*>(expert_offsets.const_data_ptr()), s.groups, s.experts,
                              s.rows, s.out_features, s.in_features, static_cast<int>(quant_type),
                              workspace.mutable_data_ptr(), ws_bytes, current_stream(device)),
               "grouped_mmq_pair_grad_input");
    return grad_input;
}

}  // namespace

STABLE_TORCH_LIBRARY(torch_ggml_ops, m) {
    m.def("mmq(Tensor input, Tensor packed_weight, int quant_type, int out_features) -> Tensor");
    m.def("mmq_grad_input(Tensor grad_output, Tensor packed_weight, int quant_type, int in_features) -> Tensor");
    m.def(
        "grouped_mmq(Tensor input, Tensor packed_weight, Tensor expert_indices, Tensor expert_offsets, "
        "int quant_type, int out_features) -> Tensor");
    m.def(
        "grouped_mmq_grad_input(Tensor grad_output, Tensor packed_weight, Tensor expert_indices, "
        "Tensor expert_offsets, int quant_type, int in_features) -> Tensor");
    m.def(
        "grouped_mmq_pair(Tensor input, Tensor first_packed_weight, Tensor second_packed_weight, "
        "Tensor expert_indices, Tensor expert_offsets, int quant_type, int out_features) -> (Tensor, Tensor)");
    m.def(
        "grouped_mmq_pair_grad_input(Tensor first_grad_output, Tensor second_grad_output, "
        "Tensor first_packed_weight, Tensor second_packed_weight, Tensor expert_indices, "
        "Tensor expert_offsets, int quant_type, int in_features) -> Tensor");
}

STABLE_TORCH_LIBRARY_IMPL(torch_ggml_ops, CUDA, m) {
    m.impl("mmq", TORCH_BOX(&mmq_op));
    m.impl("mmq_grad_input", TORCH_BOX(&mmq_grad_input_op));
    m.impl("grouped_mmq", TORCH_BOX(&grouped_mmq_op));
    m.impl("grouped_mmq_grad_input", TORCH_BOX(&grouped_mmq_grad_input_op));
    m.impl("grouped_mmq_pair", TORCH_BOX(&grouped_mmq_pair_op));
    m.impl("grouped_mmq_pair_grad_input", TORCH_BOX(&grouped_mmq_pair_grad_input_op));
}

// Importing the module runs the static registrars above; it exports nothing else.
extern "C" PyObject* PyInit__C(void) {
    static PyModuleDef module = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr};
    return PyModule_Create(&module);
}
