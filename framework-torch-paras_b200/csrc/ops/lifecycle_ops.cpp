// The few aten operators a tensor needs in order to exist on `paras:N`, move to and from
// the host and be viewed; plus the boxed CPU fallback for everything that is not on the
// transformer hot path.
//
// Counterpart of the lifecycle part of the reference's csrc/ops/tensor_ops.cpp
// (empty 57-69, empty_strided 78-88, view 90-101, as_strided 103-113, _copy_from 252-330,
// fill_/zero_, _local_scalar_dense 379-396, resize_/set_, boxed fallback 971-977,
// AutogradPrivateUse1 fallthrough 1027-1029).  The reference can read device memory from the
// host because it allocates unified memory; here every host read is an explicit
// device->host copy through the C ABI.
#include <ATen/InferSize.h>
#include <ATen/native/CPUFallback.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include "core/device_runtime.h"

namespace paras {
namespace {

using at::Tensor;

int copy_code(c10::ScalarType t) {
    switch (t) {
        case c10::kFloat: return PARAS_SC_F32;
        case c10::kBFloat16: return PARAS_SC_BF16;
        case c10::kHalf: return PARAS_SC_F16;
        case c10::kDouble: return PARAS_SC_F64;
        case c10::kLong: return PARAS_SC_I64;
        case c10::kInt: return PARAS_SC_I32;
        case c10::kShort: return PARAS_SC_I16;
        case c10::kChar: return PARAS_SC_I8;
        case c10::kByte: return PARAS_SC_U8;
        case c10::kBool: return PARAS_SC_BOOL;
        default: TORCH_CHECK(false, "paras: unsupported dtype ", t); return -1;
    }
}

Tensor new_tensor(c10::IntArrayRef sizes, c10::Device device, c10::ScalarType dtype) {
    TORCH_CHECK(device.type() == kDevice, "paras: expected a paras device, got ", device);
    const c10::Device dev(kDevice, device.has_index() ? device.index() : current_device().index());
    Runtime::get().check_index(int(dev.index()));
    c10::DeviceGuard guard(dev);  // the allocator reads the current device
    int64_t numel = 1;
    for (auto s : sizes) {
        TORCH_CHECK(s >= 0, "paras: negative dimension ", s);
        numel *= s;
    }
    const size_t nbytes = size_t(numel) * c10::elementSize(dtype);
    c10::Allocator* alloc = device_allocator();
    c10::Storage storage(c10::Storage::use_byte_size_t(), nbytes, alloc->allocate(nbytes), alloc,
                         /*resizable=*/true);
    auto impl = c10::make_intrusive<c10::TensorImpl>(
        std::move(storage), c10::DispatchKeySet{c10::DispatchKey::PrivateUse1},
        caffe2::TypeMeta::fromScalarType(dtype));
    impl->set_sizes_contiguous(sizes);
    return Tensor(std::move(impl));
}

Tensor empty_memory_format(c10::IntArrayRef size, std::optional<c10::ScalarType> dtype,
                           std::optional<c10::Layout> layout, std::optional<c10::Device> device,
                           std::optional<bool> /*pin_memory*/,
                           std::optional<c10::MemoryFormat> /*memory_format*/) {
    PARAS_TRACE_OP("empty.memory_format");
    TORCH_CHECK(!layout || *layout == c10::kStrided, "paras backend supports only strided layout");
    return new_tensor(size, device.value_or(current_device()), dtype.value_or(c10::kFloat));
}

Tensor empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride,
                     std::optional<c10::ScalarType> dtype, std::optional<c10::Layout> layout,
                     std::optional<c10::Device> device, std::optional<bool> /*pin_memory*/) {
    PARAS_TRACE_OP("empty_strided");
    TORCH_CHECK(!layout || *layout == c10::kStrided, "paras backend supports only strided layout");
    const auto st = dtype.value_or(c10::kFloat);
    const size_t nbytes = at::detail::computeStorageNbytes(size, stride, c10::elementSize(st));
    const int64_t elems = int64_t(nbytes / c10::elementSize(st));
    Tensor flat = new_tensor({elems}, device.value_or(current_device()), st);
    flat.unsafeGetTensorImpl()->set_sizes_and_strides(size, stride);
    return flat;
}

Tensor view(const Tensor& self, c10::IntArrayRef size) {
    PARAS_TRACE_OP("view");
    auto inferred = at::infer_size_dv(size, self.numel());
    auto stride = at::detail::computeStride(self.sizes(), self.strides(), inferred);
    TORCH_CHECK(stride.has_value(),
                "view size is not compatible with input tensor's size and stride (at least one "
                "dimension spans across two contiguous subspaces). Use .reshape(...) instead.");
    Tensor out = at::alias(self);
    out.unsafeGetTensorImpl()->set_sizes_and_strides(inferred, *stride);
    return out;
}

Tensor reshape_alias(const Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride) {
    PARAS_TRACE_OP("_reshape_alias");
    Tensor out = at::alias(self);
    out.unsafeGetTensorImpl()->set_sizes_and_strides(size, stride);
    return out;
}

Tensor as_strided(const Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride,
                  std::optional<int64_t> storage_offset) {
    PARAS_TRACE_OP("as_strided");
    Tensor out = at::alias(self);
    out.unsafeGetTensorImpl()->set_sizes_and_strides(size, stride, storage_offset);
    return out;
}

// ---- copies --------------------------------------------------------------------------
bool is_paras(const Tensor& t) { return t.device().type() == kDevice; }
bool on_gpu(const Tensor& t) { return is_paras(t) && Runtime::get().is_gpu(int(t.device().index())); }

// A host-memory `paras:0` tensor seen as an ordinary CPU tensor sharing its bytes.
Tensor host_alias(const Tensor& t) {
    return at::from_blob(t.data_ptr(), t.sizes(), t.strides(), t.options().device(c10::kCPU));
}

void device_strided_copy(const Tensor& src, const Tensor& dst) {
    Runtime& rt = Runtime::get();
    const int gpu = rt.gpu_of(dst);
    if (src.scalar_type() == dst.scalar_type() && src.is_contiguous() && dst.is_contiguous()) {
        PARAS_ABI(paras_b200_memcpy_d2d(gpu, dst.data_ptr(), src.data_ptr(), dst.nbytes(), nullptr));
        return;
    }
    TORCH_CHECK(dst.dim() <= 8, "paras copy: rank exceeds kernel limit");
    PARAS_ABI(paras_b200_strided_copy(gpu, dst.data_ptr(), copy_code(dst.scalar_type()),
                                      dst.strides().data(), src.data_ptr(),
                                      copy_code(src.scalar_type()), src.strides().data(),
                                      dst.sizes().data(), int(dst.dim()), nullptr));
}

Tensor copy_from(const Tensor& self, const Tensor& dst, bool non_blocking) {
    PARAS_TRACE_OP("_copy_from");
    TORCH_CHECK(self.numel() == dst.numel(), "paras copy: element count mismatch (",
                self.numel(), " vs ", dst.numel(), ")");
    TORCH_CHECK(self.sizes() == dst.sizes() || self.numel() == dst.numel(),
                "paras copy: shape mismatch");
    if (dst.numel() == 0) return dst;
    Runtime& rt = Runtime::get();

    // paras:0 keeps its bytes in host memory: treat it as a CPU tensor.
    if (is_paras(self) && !on_gpu(self)) {
        Tensor s = host_alias(self);
        if (on_gpu(dst)) {
            copy_from(s, dst, non_blocking);
        } else {
            Tensor d = is_paras(dst) ? host_alias(dst) : dst;
            d.copy_(s.sizes() == d.sizes() ? s : s.reshape(d.sizes()));
        }
        return dst;
    }
    if (is_paras(dst) && !on_gpu(dst)) {
        Tensor d = host_alias(dst);
        if (on_gpu(self)) copy_from(self, d, non_blocking);
        else d.copy_(self.sizes() == d.sizes() ? self : self.reshape(d.sizes()));
        return dst;
    }
    Tensor src = self.sizes() == dst.sizes() ? self : self.reshape(dst.sizes());

    if (!is_paras(src)) {
        // host -> GPU
        TORCH_CHECK(src.device().is_cpu(), "paras copy: unsupported source device ", src.device());
        const int gpu = rt.gpu_of(dst);
        Tensor staged = src;
        if (staged.scalar_type() != dst.scalar_type()) staged = staged.to(dst.scalar_type());
        staged = staged.contiguous();
        if (dst.is_contiguous()) {
            if (non_blocking) note_pinned_async_read(staged.data_ptr(), gpu);
            PARAS_ABI(paras_b200_memcpy_h2d(gpu, dst.data_ptr(), staged.data_ptr(), dst.nbytes(),
                                            nullptr, non_blocking ? 0 : 1));
        } else {
            Tensor tmp = new_tensor(dst.sizes(), dst.device(), dst.scalar_type());
            PARAS_ABI(paras_b200_memcpy_h2d(gpu, tmp.data_ptr(), staged.data_ptr(), tmp.nbytes(),
                                            nullptr, 1));
            device_strided_copy(tmp, dst);
        }
        return dst;
    }
    if (!is_paras(dst)) {
        // GPU -> host (always blocking)
        TORCH_CHECK(dst.device().is_cpu(), "paras copy: unsupported destination device ", dst.device());
        const int gpu = rt.gpu_of(src);
        Tensor dense = src;
        if (!src.is_contiguous() || src.scalar_type() != dst.scalar_type()) {
            dense = new_tensor(src.sizes(), src.device(), dst.scalar_type());
            device_strided_copy(src, dense);
        }
        if (dst.is_contiguous()) {
            PARAS_ABI(paras_b200_memcpy_d2h(gpu, dst.data_ptr(), dense.data_ptr(), dst.nbytes(), nullptr));
        } else {
            Tensor tmp = at::empty(dst.sizes(), dst.options());
            PARAS_ABI(paras_b200_memcpy_d2h(gpu, tmp.data_ptr(), dense.data_ptr(), tmp.nbytes(), nullptr));
            dst.copy_(tmp);
        }
        return dst;
    }
    // GPU -> GPU
    if (src.device() == dst.device()) {
        device_strided_copy(src, dst);
        return dst;
    }
    // Two GPUs: dense staging on each side, one peer copy over NVLink.  (The reference
    // bounces through a host tensor, csrc/ops/tensor_ops.cpp:313-322.)
    Tensor s_dense = src;
    if (!src.is_contiguous() || src.scalar_type() != dst.scalar_type()) {
        s_dense = new_tensor(src.sizes(), src.device(), dst.scalar_type());
        device_strided_copy(src, s_dense);
    }
    Tensor d_dense = dst.is_contiguous() ? dst : new_tensor(dst.sizes(), dst.device(), dst.scalar_type());
    PARAS_ABI(paras_b200_memcpy_peer(rt.gpu_of(d_dense), d_dense.data_ptr(), rt.gpu_of(s_dense),
                                     s_dense.data_ptr(), d_dense.nbytes()));
    if (!dst.is_contiguous()) device_strided_copy(d_dense, dst);
    return dst;
}

// aten::_to_copy for a paras source (`.cpu()`, `.to(dtype)`, `.to("paras:2")`).  A host
// destination is allocated page-locked (from the cached pinned allocator), so the
// device->host transfer is one direct DMA at PCIe speed instead of a staged copy into
// pageable memory.
Tensor to_copy(const Tensor& self, std::optional<c10::ScalarType> dtype,
               std::optional<c10::Layout> layout, std::optional<c10::Device> device,
               std::optional<bool> pin_memory, bool non_blocking,
               std::optional<c10::MemoryFormat> /*memory_format*/) {
    PARAS_TRACE_OP("_to_copy");
    TORCH_CHECK(!layout || *layout == c10::kStrided, "paras backend supports only strided layout");
    const c10::Device target = device.value_or(self.device());
    const c10::ScalarType st = dtype.value_or(self.scalar_type());
    Tensor dst;
    if (target.is_cpu()) {
        const bool pinned = pin_memory.value_or(on_gpu(self));
        dst = at::empty(self.sizes(), at::TensorOptions().dtype(st).device(c10::kCPU).pinned_memory(pinned));
    } else {
        dst = at::empty(self.sizes(), self.options().dtype(st).device(target));
    }
    if (is_paras(dst) || is_paras(self)) copy_from(self, dst, non_blocking);
    else dst.copy_(self, non_blocking);
    return dst;
}

Tensor copy_from_and_resize(const Tensor& self, const Tensor& dst) {
    PARAS_TRACE_OP("_copy_from_and_resize");
    if (dst.sizes() != self.sizes()) dst.resize_(self.sizes());
    return copy_from(self, dst, false);
}

Tensor& fill_scalar(Tensor& self, const c10::Scalar& value) {
    PARAS_TRACE_OP("fill_.Scalar");
    if (self.numel() == 0) return self;
    if (!on_gpu(self)) {
        host_alias(self).fill_(value);
        return self;
    }
    const int gpu = Runtime::get().gpu_of(self);
    if (self.is_contiguous()) {
        PARAS_ABI(paras_b200_fill(gpu, self.data_ptr(), copy_code(self.scalar_type()),
                                  value.toDouble(), self.numel(), nullptr));
    } else {
        Tensor dense = new_tensor(self.sizes(), self.device(), self.scalar_type());
        PARAS_ABI(paras_b200_fill(gpu, dense.data_ptr(), copy_code(self.scalar_type()),
                                  value.toDouble(), dense.numel(), nullptr));
        device_strided_copy(dense, self);
    }
    return self;
}

Tensor& zero_(Tensor& self) {
    PARAS_TRACE_OP("zero_");
    if (on_gpu(self) && self.is_contiguous() && self.numel() > 0) {
        PARAS_ABI(paras_b200_memset(Runtime::get().gpu_of(self), self.data_ptr(), 0, self.nbytes(), nullptr));
        return self;
    }
    return fill_scalar(self, 0);
}

c10::Scalar local_scalar_dense(const Tensor& self) {
    PARAS_TRACE_OP("_local_scalar_dense");
    TORCH_CHECK(self.numel() == 1, "paras: a Tensor with ", self.numel(),
                " elements cannot be converted to Scalar");
    Tensor host = at::empty({}, self.options().device(c10::kCPU));
    copy_from(self.reshape({}), host, false);
    return host.item();
}

const Tensor& resize_(const Tensor& self, c10::IntArrayRef size,
                      std::optional<c10::MemoryFormat> /*format*/) {
    PARAS_TRACE_OP("resize_");
    auto* impl = self.unsafeGetTensorImpl();
    int64_t numel = 1;
    for (auto s : size) numel *= s;
    const size_t need = size_t(impl->storage_offset() + numel) * self.element_size();
    const c10::Storage& storage = impl->storage();
    if (need > storage.nbytes()) {
        c10::DeviceGuard guard(self.device());
        c10::Allocator* alloc = device_allocator();
        c10::DataPtr fresh = alloc->allocate(need);
        if (storage.nbytes() > 0) {
            if (on_gpu(self)) {
                PARAS_ABI(paras_b200_memcpy_d2d(Runtime::get().gpu_of(self), fresh.get(),
                                                storage.data(), storage.nbytes(), nullptr));
            } else {
                std::memcpy(fresh.get(), storage.data(), storage.nbytes());
            }
        }
        storage.set_data_ptr_noswap(std::move(fresh));
        storage.set_nbytes(need);
    }
    impl->set_sizes_contiguous(size);
    return self;
}

Tensor& set_storage_offset(Tensor& self, c10::Storage source, int64_t storage_offset,
                           c10::IntArrayRef size, c10::IntArrayRef stride) {
    PARAS_TRACE_OP("set_.source_Storage_storage_offset");
    auto* impl = self.unsafeGetTensorImpl();
    impl->set_storage_keep_dtype(std::move(source));
    impl->set_storage_offset(storage_offset);
    if (stride.data() == nullptr || (stride.empty() && !size.empty())) {
        impl->set_sizes_contiguous(size);
    } else {
        impl->set_sizes_and_strides(size, stride);
    }
    return self;
}

Tensor& set_storage(Tensor& self, c10::Storage source) {
    PARAS_TRACE_OP("set_.source_Storage");
    const int64_t n = int64_t(source.nbytes() / self.element_size());
    return set_storage_offset(self, std::move(source), 0, {n}, {});
}

Tensor& set_tensor(Tensor& self, const Tensor& source) {
    PARAS_TRACE_OP("set_.source_Tensor");
    return set_storage_offset(self, source.storage(), source.storage_offset(), source.sizes(),
                              source.strides());
}

bool has_compatible_shallow_copy_type(const Tensor& self, const Tensor& from) {
    return self.device().type() == from.device().type();
}

// Everything else: run on the host and copy back, as the reference does for operators it
// has no kernel for (csrc/ops/tensor_ops.cpp:971-977).  The hot-path operators are
// registered explicitly and never come here.
void cpu_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack) {
    PARAS_INFO("falling back to CPU for %s", op.schema().operator_name().name.c_str());
    at::native::cpu_fallback(op, stack);
}

}  // namespace
}  // namespace paras

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("aten::empty.memory_format", &paras::empty_memory_format);
    m.impl("aten::empty_strided", &paras::empty_strided);
    m.impl("aten::view", &paras::view);
    m.impl("aten::_reshape_alias", &paras::reshape_alias);
    m.impl("aten::as_strided", &paras::as_strided);
    m.impl("aten::_copy_from", &paras::copy_from);
    m.impl("aten::_copy_from_and_resize", &paras::copy_from_and_resize);
    m.impl("aten::_to_copy", &paras::to_copy);
    m.impl("aten::fill_.Scalar", &paras::fill_scalar);
    m.impl("aten::zero_", &paras::zero_);
    m.impl("aten::_local_scalar_dense", &paras::local_scalar_dense);
    m.impl("aten::resize_", &paras::resize_);
    m.impl("aten::set_.source_Storage", &paras::set_storage);
    m.impl("aten::set_.source_Storage_storage_offset", &paras::set_storage_offset);
    m.impl("aten::set_.source_Tensor", &paras::set_tensor);
    m.impl("aten::_has_compatible_shallow_copy_type", &paras::has_compatible_shallow_copy_type);
}

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) {
    m.fallback(torch::CppFunction::makeFromBoxedFunction<&paras::cpu_fallback>());
}

TORCH_LIBRARY_IMPL(_, AutogradPrivateUse1, m) {
    m.fallback(torch::CppFunction::makeFallthrough());
}
