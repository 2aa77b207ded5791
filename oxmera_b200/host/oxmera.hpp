// C++ host mirror of the oxmera vocabulary and of the B200 backend.
//
// The reference's host code is Rust; where no Rust toolchain exists this header
// is the compiled-language host side above the C ABI (include/oxmera_b200.h).
// Names, argument meaning and error behaviour follow the reference crates:
//   oxmera-core     DType, Device, Shape, Strides, Layout, Error, Result,
//                   broadcast_shapes, contiguous_strides
//   oxmera-tensor   Storage, Tensor (views: reshape / permute / narrow / contiguous)
//   oxmera-ops      UnaryOps, BinaryOps, MatmulOps (+ the batched extension), ReduceOps
//   oxmera-runtime  Backend, backend_for, register_backend, Tensor::matmul
// Header only, C++17.  Link against liboxmera_b200.so to use B200Backend.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "../../include/oxmera_b200.h"

namespace oxmera {

// ---------------------------------------------------------------- core ----

// crates/oxmera-core/src/dtype.rs:9-22, plus the two 16-bit floats the backend adds.
enum class DType : int32_t { F32 = 0, F64 = 1, I32 = 2, I64 = 3, U8 = 4, Bool = 5, BF16 = 6, F16 = 7, F8E4M3 = 8, F8E5M2 = 9 };

inline size_t size_in_bytes(DType d) {
  switch (d) {
    case DType::F32: case DType::I32: return 4;
    case DType::F64: case DType::I64: return 8;
    case DType::U8: case DType::Bool: case DType::F8E4M3: case DType::F8E5M2: return 1;
    default: return 2;
  }
}
inline bool is_float(DType d) {
  return d == DType::F32 || d == DType::F64 || d == DType::BF16 || d == DType::F16 || d == DType::F8E4M3 || d == DType::F8E5M2;
}
inline const char *dtype_name(DType d) {
  static const char *n[] = {"F32", "F64", "I32", "I64", "U8", "Bool", "BF16", "F16", "F8E4M3", "F8E5M2"};
  return n[static_cast<int>(d)];
}

// crates/oxmera-core/src/device.rs:8-24: a place, not a backend.
struct Device {
  enum class Kind { Cpu, Metal, Cuda } kind = Kind::Cpu;
  size_t index = 0;
  static Device cpu() { return {Kind::Cpu, 0}; }
  static Device metal(size_t i) { return {Kind::Metal, i}; }
  static Device cuda(size_t i) { return {Kind::Cuda, i}; }
  const char *kind_name() const { return kind == Kind::Cpu ? "cpu" : kind == Kind::Metal ? "metal" : "cuda"; }
  bool operator==(const Device &o) const { return kind == o.kind && index == o.index; }
  bool operator<(const Device &o) const { return std::make_pair(static_cast<int>(kind), index) < std::make_pair(static_cast<int>(o.kind), o.index); }
  std::string debug() const {  // the spelling of Rust's {:?}
    if (kind == Kind::Cpu) return "Cpu";
    return std::string(kind == Kind::Metal ? "Metal" : "Cuda") + " { index: " + std::to_string(index) + " }";
  }
};

using Dims = std::vector<size_t>;

// crates/oxmera-core/src/shape.rs:11-35
class Shape {
 public:
  Shape() = default;
  Shape(std::initializer_list<size_t> d) : dims_(d) {}
  explicit Shape(Dims d) : dims_(std::move(d)) {}
  const Dims &dims() const { return dims_; }
  size_t ndim() const { return dims_.size(); }
  size_t numel() const {  // a scalar has one element; any zero extent empties the tensor
    size_t n = 1;
    for (size_t d : dims_) n *= d;
    return n;
  }
  bool operator==(const Shape &o) const { return dims_ == o.dims_; }
  bool operator!=(const Shape &o) const { return !(*this == o); }
  std::string debug() const {
    std::ostringstream s;
    s << "[";
    for (size_t i = 0; i < dims_.size(); ++i) s << (i ? ", " : "") << dims_[i];
    s << "]";
    return s.str();
  }
 private:
  Dims dims_;
};

// crates/oxmera-core/src/layout.rs:6-22: element strides, signed.
class Strides {
 public:
  Strides() = default;
  explicit Strides(std::vector<ptrdiff_t> v) : v_(std::move(v)) {}
  const std::vector<ptrdiff_t> &values() const { return v_; }
  bool operator==(const Strides &o) const { return v_ == o.v_; }
 private:
  std::vector<ptrdiff_t> v_;
};

// crates/oxmera-core/src/error.rs:12-102: one kind per variant, fields kept.
struct Error {
  enum class Kind {
    ShapeMismatch = 1, BroadcastIncompatible, DTypeMismatch, UnsupportedDType, DeviceMismatch,
    IndexOutOfBounds, RankMismatch, BackendUnavailable, NotImplemented,
    // BinaryOps::div: "Integer division by zero is a typed error" (crates/oxmera-ops/src/lib.rs:47-49);
    // the reference's non_exhaustive enum has no variant for it yet.
    DivisionByZero = 13
  } kind;
  Shape expected, got;        // ShapeMismatch; BroadcastIncompatible uses them as lhs, rhs; IndexOutOfBounds: got = shape
  std::vector<size_t> index;  // IndexOutOfBounds
  size_t index_rank = 0, shape_rank = 0;
  Device lhs_device, rhs_device;
  std::string op, detail;

  std::string to_string() const {
    switch (kind) {
      case Kind::ShapeMismatch:
        return !detail.empty() ? detail : "shape mismatch: expected " + expected.debug() + ", got " + got.debug() + " in " + op;
      case Kind::BroadcastIncompatible:
        return "cannot broadcast " + expected.debug() + " with " + got.debug();
      case Kind::DTypeMismatch: return !detail.empty() ? detail : "dtype mismatch in " + op;
      case Kind::UnsupportedDType: return !detail.empty() ? detail : "dtype is not supported by " + op;
      case Kind::DeviceMismatch:
        return "device mismatch: " + lhs_device.debug() + " vs " + rhs_device.debug() + " in " + op;
      case Kind::IndexOutOfBounds: return "index " + Shape(Dims(index)).debug() + " out of bounds for shape " + got.debug();
      case Kind::RankMismatch:
        return "rank mismatch: index of rank " + std::to_string(index_rank) + " against shape of rank " + std::to_string(shape_rank);
      case Kind::BackendUnavailable:
        return !detail.empty() ? detail : "no backend available for device " + lhs_device.debug();
      case Kind::DivisionByZero: return "integer division by zero in " + op;
      default: return op + " is not implemented for " + detail;
    }
  }
};

// The shape of Rust's Result<T>: a value or a typed error, never an exception.
template <class T>
class Result {
 public:
  Result(T v) : v_(std::move(v)) {}
  Result(Error e) : v_(std::move(e)) {}
  bool is_ok() const { return std::holds_alternative<T>(v_); }
  bool is_err() const { return !is_ok(); }
  T &unwrap() {
    if (is_err()) throw std::runtime_error("unwrap on Err: " + std::get<Error>(v_).to_string());
    return std::get<T>(v_);
  }
  const Error &unwrap_err() const {
    if (is_ok()) throw std::runtime_error("unwrap_err on Ok");
    return std::get<Error>(v_);
  }
 private:
  std::variant<T, Error> v_;
};

// crates/oxmera-core/src/layout.rs:58-62
inline Strides contiguous_strides(const Shape &shape) {
  std::vector<ptrdiff_t> s(shape.ndim());
  ptrdiff_t acc = 1;
  for (size_t i = shape.ndim(); i-- > 0;) {
    s[i] = acc;
    acc *= static_cast<ptrdiff_t>(shape.dims()[i] > 1 ? shape.dims()[i] : 1);
  }
  return Strides(s);
}

// crates/oxmera-core/src/shape.rs:49-58: NumPy's rule as a total function.
inline Result<Shape> broadcast_shapes(const Shape &lhs, const Shape &rhs) {
  const size_t n = std::max(lhs.ndim(), rhs.ndim());
  Dims out(n);
  for (size_t i = 0; i < n; ++i) {
    const size_t l = i < lhs.ndim() ? lhs.dims()[lhs.ndim() - 1 - i] : 1;
    const size_t r = i < rhs.ndim() ? rhs.dims()[rhs.ndim() - 1 - i] : 1;
    if (l != r && l != 1 && r != 1) {
      Error e{Error::Kind::BroadcastIncompatible};
      e.expected = lhs; e.got = rhs;
      return e;
    }
    out[n - 1 - i] = l == 1 ? r : l;
  }
  return Shape(out);
}

// crates/oxmera-core/src/layout.rs:26-56
struct Layout {
  Shape shape;
  Strides strides;
  size_t offset = 0;

  static Layout contiguous(Shape shape) {
    Strides s = contiguous_strides(shape);
    return Layout{std::move(shape), std::move(s), 0};
  }
  Result<size_t> offset_of(const std::vector<size_t> &index) const {
    if (index.size() != shape.ndim()) {
      Error e{Error::Kind::RankMismatch};
      e.index_rank = index.size(); e.shape_rank = shape.ndim();
      return e;
    }
    ptrdiff_t off = static_cast<ptrdiff_t>(offset);
    for (size_t i = 0; i < index.size(); ++i) {
      if (index[i] >= shape.dims()[i]) {
        Error e{Error::Kind::IndexOutOfBounds};
        e.index = index; e.got = shape;
        return e;
      }
      off += static_cast<ptrdiff_t>(index[i]) * strides.values()[i];
    }
    return static_cast<size_t>(off);
  }
  bool is_contiguous() const {  // a scalar and any empty tensor count as contiguous
    if (shape.numel() == 0) return true;
    ptrdiff_t acc = 1;
    for (size_t i = shape.ndim(); i-- > 0;) {
      if (shape.dims()[i] != 1 && strides.values()[i] != acc) return false;
      acc *= static_cast<ptrdiff_t>(shape.dims()[i]);
    }
    return true;
  }
  // lowest and highest storage element the layout touches
  std::pair<ptrdiff_t, ptrdiff_t> extent() const {
    ptrdiff_t lo = static_cast<ptrdiff_t>(offset), hi = lo;
    for (size_t i = 0; i < shape.ndim(); ++i) {
      if (shape.dims()[i] == 0) continue;
      const ptrdiff_t span = static_cast<ptrdiff_t>(shape.dims()[i] - 1) * strides.values()[i];
      (span > 0 ? hi : lo) += span;
    }
    return {lo, hi};
  }
};

// -------------------------------------------------------------- tensor ----

// crates/oxmera-tensor/src/storage.rs:12-67 with the device variant added:
// host bytes for Device::Cpu, or a device pointer released through `release`.
class Storage {
 public:
  static std::shared_ptr<Storage> cpu_from_bytes(std::vector<uint8_t> bytes, DType dtype) {
    auto s = std::shared_ptr<Storage>(new Storage());
    s->host_ = std::move(bytes); s->dtype_ = dtype; s->device_ = Device::cpu();
    s->numel_ = s->host_.size() / size_in_bytes(dtype);
    return s;
  }
  static std::shared_ptr<Storage> cpu_zeros(size_t numel, DType dtype) {
    return cpu_from_bytes(std::vector<uint8_t>(numel * size_in_bytes(dtype), 0), dtype);
  }
  static std::shared_ptr<Storage> device(void *ptr, size_t numel, DType dtype, Device dev, std::function<void(void *)> release) {
    auto s = std::shared_ptr<Storage>(new Storage());
    s->dev_ptr_ = ptr; s->numel_ = numel; s->dtype_ = dtype; s->device_ = dev; s->release_ = std::move(release);
    return s;
  }
  ~Storage() {
    if (dev_ptr_ && release_) release_(dev_ptr_);
  }
  DType dtype() const { return dtype_; }
  Device device() const { return device_; }
  size_t numel() const { return numel_; }
  // The raw bytes when the storage is on the CPU; nullptr otherwise.
  const uint8_t *cpu_bytes() const { return device_.kind == Device::Kind::Cpu ? host_.data() : nullptr; }
  uint8_t *cpu_bytes_mut() { return device_.kind == Device::Kind::Cpu ? host_.data() : nullptr; }
  void *device_ptr() const { return dev_ptr_; }
 private:
  Storage() = default;
  std::vector<uint8_t> host_;
  void *dev_ptr_ = nullptr;
  size_t numel_ = 0;
  DType dtype_ = DType::F32;
  Device device_;
  std::function<void(void *)> release_;
};

class Backend;
inline Result<std::shared_ptr<Backend>> backend_for(Device device);

// crates/oxmera-tensor/src/tensor.rs:15-100
class Tensor {
 public:
  static Result<Tensor> from_storage(std::shared_ptr<Storage> storage, Layout layout) {
    if (layout.shape.numel() > 0) {
      auto [lo, hi] = layout.extent();
      if (lo < 0 || hi >= static_cast<ptrdiff_t>(storage->numel())) {
        Error e{Error::Kind::IndexOutOfBounds};
        e.index = {static_cast<size_t>(hi)}; e.got = Shape{storage->numel()};
        return e;
      }
    }
    return Tensor(std::move(storage), std::move(layout));
  }
  static Result<Tensor> from_vec_f32(const std::vector<float> &data, Shape shape) {
    if (data.size() != shape.numel()) {
      Error e{Error::Kind::ShapeMismatch};
      e.expected = shape; e.got = Shape{data.size()}; e.op = "from_vec_f32";
      return e;
    }
    std::vector<uint8_t> bytes(data.size() * 4);
    if (!data.empty()) std::memcpy(bytes.data(), data.data(), bytes.size());
    return Tensor(Storage::cpu_from_bytes(std::move(bytes), DType::F32), Layout::contiguous(std::move(shape)));
  }
  const Shape &shape() const { return layout_.shape; }
  const Layout &layout() const { return layout_; }
  DType dtype() const { return storage_->dtype(); }
  Device device() const { return storage_->device(); }
  const std::shared_ptr<Storage> &storage() const { return storage_; }

  Result<Tensor> reshape(Shape shape) const {
    if (shape.numel() != layout_.shape.numel()) {
      Error e{Error::Kind::ShapeMismatch};
      e.expected = layout_.shape; e.got = shape; e.op = "reshape";
      return e;
    }
    if (!layout_.is_contiguous()) {
      Error e{Error::Kind::NotImplemented};
      e.op = "reshape"; e.detail = "a non-contiguous view (it would copy; call contiguous() first)";
      return e;
    }
    Layout l{shape, contiguous_strides(shape), layout_.offset};
    return Tensor(storage_, std::move(l));
  }
  Result<Tensor> permute(const std::vector<size_t> &perm) const {
    const size_t n = layout_.shape.ndim();
    std::vector<bool> seen(n, false);
    bool ok = perm.size() == n;
    for (size_t i = 0; ok && i < n; ++i) {
      ok = perm[i] < n && !seen[perm[i]];
      if (ok) seen[perm[i]] = true;
    }
    if (!ok) {
      Error e{Error::Kind::ShapeMismatch};
      e.expected = layout_.shape; e.got = Shape(Dims(perm.begin(), perm.end())); e.op = "permute";
      return e;
    }
    Dims d(n);
    std::vector<ptrdiff_t> s(n);
    for (size_t i = 0; i < n; ++i) {
      d[i] = layout_.shape.dims()[perm[i]];
      s[i] = layout_.strides.values()[perm[i]];
    }
    return Tensor(storage_, Layout{Shape(d), Strides(s), layout_.offset});
  }
  Result<Tensor> narrow(size_t dim, size_t start, size_t len) const {
    if (dim >= layout_.shape.ndim() || start + len > layout_.shape.dims()[dim]) {
      Error e{Error::Kind::IndexOutOfBounds};
      e.index = {dim, start, len}; e.got = layout_.shape;
      return e;
    }
    Dims d = layout_.shape.dims();
    d[dim] = len;
    const ptrdiff_t off = static_cast<ptrdiff_t>(layout_.offset) + static_cast<ptrdiff_t>(start) * layout_.strides.values()[dim];
    return Tensor(storage_, Layout{Shape(d), layout_.strides, static_cast<size_t>(off)});
  }
  // Logical order in fresh storage on the same device; shares storage when already contiguous.
  Result<Tensor> contiguous() const;
  // One element, for tests.  CPU float storage only (tensor.rs:92-100).
  Result<float> get_f32(const std::vector<size_t> &index) const {
    auto off = layout_.offset_of(index);
    if (off.is_err()) return off.unwrap_err();
    const uint8_t *bytes = storage_->cpu_bytes();
    if (!bytes || dtype() != DType::F32) {
      Error e{Error::Kind::UnsupportedDType};
      e.op = "get_f32"; e.detail = "get_f32 reads f32 CPU storage only; copy device tensors to the host first";
      return e;
    }
    float v;
    std::memcpy(&v, bytes + off.unwrap() * 4, 4);
    return v;
  }
  // TensorOps (crates/oxmera-runtime/src/lib.rs:57-72): resolve the backend from the device and dispatch.
  Result<Tensor> matmul(const Tensor &rhs) const;
  Result<Tensor> batched_matmul(const Tensor &rhs) const;
  Result<Tensor> add(const Tensor &rhs) const;
  Result<Tensor> sub(const Tensor &rhs) const;
  Result<Tensor> mul(const Tensor &rhs) const;
  Result<Tensor> div(const Tensor &rhs) const;
  Result<Tensor> neg() const;
  Result<Tensor> sum(const std::vector<size_t> &axes) const;

 private:
  Tensor(std::shared_ptr<Storage> s, Layout l) : storage_(std::move(s)), layout_(std::move(l)) {}
  std::shared_ptr<Storage> storage_;
  Layout layout_;
};

// ----------------------------------------------------------------- ops ----

// crates/oxmera-ops/src/lib.rs:53-59, with the batched extension.
class MatmulOps {
 public:
  virtual ~MatmulOps() = default;
  virtual Result<Tensor> matmul(const Tensor &lhs, const Tensor &rhs) = 0;
  virtual Result<Tensor> batched_matmul(const Tensor &lhs, const Tensor &rhs) {
    (void)lhs; (void)rhs;
    Error e{Error::Kind::NotImplemented};
    e.op = "batched_matmul"; e.detail = "this backend";
    return e;
  }
};

namespace detail {
template <typename... A>
inline Result<Tensor> not_implemented(const char *op, const A &...) {
  Error e{Error::Kind::NotImplemented};
  e.op = op; e.detail = "this backend";
  return e;
}
}  // namespace detail

// crates/oxmera-ops/src/lib.rs:27-37: exp and ln are for float dtypes only.
class UnaryOps {
 public:
  virtual ~UnaryOps() = default;
  virtual Result<Tensor> neg(const Tensor &a) { return detail::not_implemented("neg", a); }
  virtual Result<Tensor> exp(const Tensor &a) { return detail::not_implemented("exp", a); }
  virtual Result<Tensor> ln(const Tensor &a) { return detail::not_implemented("ln", a); }
  virtual Result<Tensor> abs(const Tensor &a) { return detail::not_implemented("abs", a); }
};

// crates/oxmera-ops/src/lib.rs:39-50: operands broadcast by NumPy's rule.
class BinaryOps {
 public:
  virtual ~BinaryOps() = default;
  virtual Result<Tensor> add(const Tensor &l, const Tensor &r) { return detail::not_implemented("add", l, r); }
  virtual Result<Tensor> sub(const Tensor &l, const Tensor &r) { return detail::not_implemented("sub", l, r); }
  virtual Result<Tensor> mul(const Tensor &l, const Tensor &r) { return detail::not_implemented("mul", l, r); }
  virtual Result<Tensor> div(const Tensor &l, const Tensor &r) { return detail::not_implemented("div", l, r); }
};

// crates/oxmera-ops/src/lib.rs:61-69: the reduced axes leave the shape; no axes means all axes.
class ReduceOps {
 public:
  virtual ~ReduceOps() = default;
  virtual Result<Tensor> sum(const Tensor &a, const std::vector<size_t> &axes) { return detail::not_implemented("sum", a, axes); }
  virtual Result<Tensor> max(const Tensor &a, const std::vector<size_t> &axes) { return detail::not_implemented("max", a, axes); }
};

// ------------------------------------------------------------- runtime ----

// crates/oxmera-runtime/src/lib.rs:29-34: a backend is all four op families on one device.
class Backend : public UnaryOps, public BinaryOps, public MatmulOps, public ReduceOps {
 public:
  virtual Device device() const = 0;
  virtual const char *name() const = 0;
  virtual Result<Tensor> contiguous(const Tensor &t) {
    (void)t;
    Error e{Error::Kind::NotImplemented};
    e.op = "contiguous"; e.detail = "this backend";
    return e;
  }
};

namespace detail {
inline std::map<Device, std::shared_ptr<Backend>> &registry() {
  static std::map<Device, std::shared_ptr<Backend>> r;
  return r;
}
inline std::mutex &registry_mu() {
  static std::mutex m;
  return m;
}
}  // namespace detail

// Register a backend for its device, replacing any previous registration (lib.rs:46-53).
inline void register_backend(std::shared_ptr<Backend> backend) {
  std::lock_guard<std::mutex> lock(detail::registry_mu());
  detail::registry()[backend->device()] = std::move(backend);
}
inline void unregister_all() {
  std::lock_guard<std::mutex> lock(detail::registry_mu());
  detail::registry().clear();
}
// The backend serving `device`; an unregistered device is BackendUnavailable, never a crash (lib.rs:36-44).
inline Result<std::shared_ptr<Backend>> backend_for(Device device) {
  std::lock_guard<std::mutex> lock(detail::registry_mu());
  auto it = detail::registry().find(device);
  if (it == detail::registry().end()) {
    Error e{Error::Kind::BackendUnavailable};
    e.lhs_device = device;
    return e;
  }
  return it->second;
}

inline Result<Tensor> Tensor::matmul(const Tensor &rhs) const {
  auto b = backend_for(device());
  if (b.is_err()) return b.unwrap_err();
  return b.unwrap()->matmul(*this, rhs);
}
inline Result<Tensor> Tensor::batched_matmul(const Tensor &rhs) const {
  auto b = backend_for(device());
  if (b.is_err()) return b.unwrap_err();
  return b.unwrap()->batched_matmul(*this, rhs);
}
#define OXMERA_TENSOR_BINARY(NAME)                           \
  inline Result<Tensor> Tensor::NAME(const Tensor &rhs) const { \
    auto b = backend_for(device());                            \
    if (b.is_err()) return b.unwrap_err();                     \
    return b.unwrap()->NAME(*this, rhs);                       \
  }
OXMERA_TENSOR_BINARY(add)
OXMERA_TENSOR_BINARY(sub)
OXMERA_TENSOR_BINARY(mul)
OXMERA_TENSOR_BINARY(div)
#undef OXMERA_TENSOR_BINARY
inline Result<Tensor> Tensor::neg() const {
  auto b = backend_for(device());
  if (b.is_err()) return b.unwrap_err();
  return b.unwrap()->neg(*this);
}
inline Result<Tensor> Tensor::sum(const std::vector<size_t> &axes) const {
  auto b = backend_for(device());
  if (b.is_err()) return b.unwrap_err();
  return b.unwrap()->sum(*this, axes);
}
inline Result<Tensor> Tensor::contiguous() const {
  if (layout_.is_contiguous()) return *this;
  if (const uint8_t *src = storage_->cpu_bytes()) {
    const size_t esz = size_in_bytes(dtype()), n = layout_.shape.numel();
    std::vector<uint8_t> out(n * esz);
    std::vector<size_t> idx(layout_.shape.ndim(), 0);
    for (size_t i = 0; i < n; ++i) {
      ptrdiff_t off = static_cast<ptrdiff_t>(layout_.offset);
      for (size_t d = 0; d < idx.size(); ++d) off += static_cast<ptrdiff_t>(idx[d]) * layout_.strides.values()[d];
      std::memcpy(out.data() + i * esz, src + off * esz, esz);
      for (size_t d = idx.size(); d-- > 0;) {
        if (++idx[d] < layout_.shape.dims()[d]) break;
        idx[d] = 0;
      }
    }
    return Tensor(Storage::cpu_from_bytes(std::move(out), dtype()), Layout::contiguous(layout_.shape));
  }
  auto b = backend_for(device());
  if (b.is_err()) return b.unwrap_err();
  return b.unwrap()->contiguous(*this);
}

// ------------------------------------------------------------ B200 backend ----

// Device::Cuda{index} served by liboxmera_b200.so.  Stateless apart from the
// context handle; safe to share between threads (the library serialises
// launches per context), as `Backend: Send + Sync` requires.
class B200Backend : public Backend {
 public:
  static Result<std::shared_ptr<B200Backend>> create(size_t index) {
    oxm_ctx *ctx = nullptr;
    const int st = oxm_ctx_create(static_cast<int>(index), &ctx);
    if (st != OXM_OK) return from_status(st, "ctx_create", Device::cuda(index), Device::cuda(index));
    return std::shared_ptr<B200Backend>(new B200Backend(ctx, index));
  }
  ~B200Backend() override { oxm_ctx_destroy(ctx_); }
  Device device() const override { return Device::cuda(index_); }
  const char *name() const override { return oxm_backend_name(); }

  Result<Tensor> matmul(const Tensor &lhs, const Tensor &rhs) override { return run(lhs, rhs, false); }
  Result<Tensor> batched_matmul(const Tensor &lhs, const Tensor &rhs) override { return run(lhs, rhs, true); }

  Result<Tensor> neg(const Tensor &a) override { return unary(OXM_NEG, "neg", a); }
  Result<Tensor> exp(const Tensor &a) override { return unary(OXM_EXP, "exp", a); }
  Result<Tensor> ln(const Tensor &a) override { return unary(OXM_LN, "ln", a); }
  Result<Tensor> abs(const Tensor &a) override { return unary(OXM_ABS, "abs", a); }
  Result<Tensor> add(const Tensor &l, const Tensor &r) override { return binary(OXM_ADD, "add", l, r); }
  Result<Tensor> sub(const Tensor &l, const Tensor &r) override { return binary(OXM_SUB, "sub", l, r); }
  Result<Tensor> mul(const Tensor &l, const Tensor &r) override { return binary(OXM_MUL, "mul", l, r); }
  Result<Tensor> div(const Tensor &l, const Tensor &r) override { return binary(OXM_DIV, "div", l, r); }
  Result<Tensor> sum(const Tensor &a, const std::vector<size_t> &axes) override { return reduce(OXM_SUM, "sum", a, axes); }
  Result<Tensor> max(const Tensor &a, const std::vector<size_t> &axes) override { return reduce(OXM_MAX, "max", a, axes); }

  // The fused form of a linear layer's product (no counterpart in the reference's traits):
  // out = act(lhs . rhs + bias), or out += lhs . rhs when `accumulate_into` is given.
  Result<Tensor> matmul_fused(const Tensor &lhs, const Tensor &rhs, const Tensor *bias, int activation,
                              const Tensor *accumulate_into = nullptr) {
    for (const Tensor *t : {&lhs, &rhs}) {
      if (!(t->device() == device())) {
        Error e{Error::Kind::DeviceMismatch};
        e.lhs_device = t->device(); e.rhs_device = device(); e.op = "matmul_fused";
        return e;
      }
    }
    if (lhs.shape().ndim() != 2 || rhs.shape().ndim() != 2) {
      Error e{Error::Kind::NotImplemented};
      e.op = "matmul_fused"; e.detail = "operands of rank other than 2";
      return e;
    }
    Result<Tensor> out = accumulate_into ? Result<Tensor>(*accumulate_into)
                                         : empty(Shape{lhs.shape().dims()[0], rhs.shape().dims()[1]}, lhs.dtype());
    if (out.is_err()) return out;
    oxm_view a = view(lhs), b = view(rhs), o = view(out.unwrap()), bv{};
    oxm_epilogue ep{};
    if (bias) { bv = view(*bias); ep.bias = &bv; }
    ep.activation = activation;
    ep.accumulate = accumulate_into ? 1 : 0;
    const int st = oxm_matmul_fused(ctx_, &a, &b, &o, &ep);
    if (st != OXM_OK) {
      Error e = from_status(st, "matmul_fused", lhs.device(), rhs.device());
      e.expected = lhs.shape(); e.got = rhs.shape();
      return e;
    }
    return out;
  }

  // The block-scaled fp8 product (MXFP8; no counterpart in the reference's traits): fp8 operands,
  // one E8M0 exponent (a U8) per 32 contraction elements of every row of lhs ([M, K/32]) and
  // column of rhs ([K/32, N]).
  Result<Tensor> matmul_mx(const Tensor &lhs, const Tensor &lhs_scale, const Tensor &rhs, const Tensor &rhs_scale, DType out_dtype) {
    for (const Tensor *t : {&lhs, &lhs_scale, &rhs, &rhs_scale}) {
      if (!(t->device() == device())) {
        Error e{Error::Kind::DeviceMismatch};
        e.lhs_device = t->device(); e.rhs_device = device(); e.op = "matmul_mx";
        return e;
      }
    }
    if (lhs.shape().ndim() != 2 || rhs.shape().ndim() != 2) {
      Error e{Error::Kind::NotImplemented};
      e.op = "matmul_mx"; e.detail = "operands of rank other than 2";
      return e;
    }
    Result<Tensor> out = empty(Shape{lhs.shape().dims()[0], rhs.shape().dims()[1]}, out_dtype);
    if (out.is_err()) return out;
    oxm_view a = view(lhs), sa = view(lhs_scale), b = view(rhs), sb = view(rhs_scale), o = view(out.unwrap());
    const int st = oxm_matmul_mx(ctx_, &a, &sa, &b, &sb, &o);
    if (st != OXM_OK) {
      Error e = from_status(st, "matmul_mx", lhs.device(), rhs.device());
      e.expected = lhs.shape(); e.got = rhs.shape();
      return e;
    }
    return out;
  }

  Result<Tensor> contiguous(const Tensor &t) override {
    auto out = empty(t.shape(), t.dtype());
    if (out.is_err()) return out;
    oxm_view s = view(t), d = view(out.unwrap());
    const int st = oxm_contiguous(ctx_, &s, &d);
    if (st != OXM_OK) return from_status(st, "contiguous", t.device(), device());
    return out;
  }

  // A fresh contiguous device tensor holding `count` elements copied from host memory.
  Result<Tensor> from_host(const void *data, Shape shape, DType dtype) {
    auto t = empty(shape, dtype);
    if (t.is_err()) return t;
    const size_t bytes = shape.numel() * size_in_bytes(dtype);
    const int st = oxm_h2d(ctx_, t.unwrap().storage()->device_ptr(), data, bytes);
    if (st != OXM_OK) return from_status(st, "from_host", device(), device());
    return t;
  }
  Result<Tensor> from_vec_f32(const std::vector<float> &data, Shape shape) {
    if (data.size() != shape.numel()) {
      Error e{Error::Kind::ShapeMismatch};
      e.expected = shape; e.got = Shape{data.size()}; e.op = "from_vec_f32";
      return e;
    }
    return from_host(data.data(), std::move(shape), DType::F32);
  }
  // The view's elements in logical order as a CPU tensor.
  Result<Tensor> to_host(const Tensor &t) {
    auto c = t.contiguous();
    if (c.is_err()) return c;
    const Tensor &ct = c.unwrap();
    const size_t esz = size_in_bytes(ct.dtype());
    std::vector<uint8_t> bytes(ct.shape().numel() * esz);
    const uint8_t *src = static_cast<const uint8_t *>(ct.storage()->device_ptr()) + ct.layout().offset * esz;
    const int st = bytes.empty() ? oxm_sync(ctx_) : oxm_d2h(ctx_, bytes.data(), src, bytes.size());
    if (st != OXM_OK) return from_status(st, "to_host", device(), device());
    return Tensor::from_storage(Storage::cpu_from_bytes(std::move(bytes), ct.dtype()), Layout::contiguous(ct.shape()));
  }
  Result<Tensor> empty(const Shape &shape, DType dtype) {
    void *ptr = nullptr;
    const int st = oxm_alloc(ctx_, shape.numel() * size_in_bytes(dtype), &ptr);
    if (st != OXM_OK) return from_status(st, "alloc", device(), device());
    oxm_ctx *ctx = ctx_;
    auto storage = Storage::device(ptr, shape.numel(), dtype, device(), [ctx](void *p) { oxm_free(ctx, p); });
    return Tensor::from_storage(std::move(storage), Layout::contiguous(shape));
  }
  oxm_ctx *raw() const { return ctx_; }

 private:
  B200Backend(oxm_ctx *ctx, size_t index) : ctx_(ctx), index_(index) {}

  static oxm_view view(const Tensor &t) {
    oxm_view v{};
    v.dtype = static_cast<int32_t>(t.dtype());
    v.ndim = static_cast<int32_t>(t.shape().ndim());
    for (size_t i = 0; i < t.shape().ndim() && i < OXM_MAX_DIMS; ++i) {
      v.shape[i] = static_cast<int64_t>(t.shape().dims()[i]);
      v.strides[i] = static_cast<int64_t>(t.layout().strides.values()[i]);
    }
    v.offset = static_cast<int64_t>(t.layout().offset);
    v.base = t.storage()->device_ptr();
    v.device = static_cast<int32_t>(t.device().index);
    return v;
  }

  // Status code -> the Error variant with the same number (error.rs:12-102);
  // backend conditions fold into NotImplemented{op, detail}.
  static Error from_status(int st, const char *op, Device lhs, Device rhs) {
    Error e{Error::Kind::NotImplemented};
    if ((st >= 1 && st <= 9) || st == OXM_DIVIDE_BY_ZERO) e.kind = static_cast<Error::Kind>(st);
    e.op = op;
    e.detail = oxm_last_error();
    e.lhs_device = lhs; e.rhs_device = rhs;
    return e;
  }

  Result<Tensor> unary(int code, const char *op, const Tensor &a) {
    if (!(a.device() == device())) {
      Error e{Error::Kind::DeviceMismatch};
      e.lhs_device = a.device(); e.rhs_device = device(); e.op = op;
      return e;
    }
    auto out = empty(a.shape(), a.dtype());
    if (out.is_err()) return out;
    oxm_view v = view(a), o = view(out.unwrap());
    const int st = oxm_unary(ctx_, code, &v, &o);
    if (st != OXM_OK) return from_status(st, op, a.device(), device());
    return out;
  }

  Result<Tensor> binary(int code, const char *op, const Tensor &l, const Tensor &r) {
    for (const Tensor *t : {&l, &r}) {
      if (!(t->device() == device())) {
        Error e{Error::Kind::DeviceMismatch};
        e.lhs_device = t->device(); e.rhs_device = device(); e.op = op;
        return e;
      }
    }
    auto shape = broadcast_shapes(l.shape(), r.shape());
    if (shape.is_err()) return shape.unwrap_err();
    auto out = empty(shape.unwrap(), l.dtype());
    if (out.is_err()) return out;
    oxm_view a = view(l), b = view(r), o = view(out.unwrap());
    const int st = oxm_binary(ctx_, code, &a, &b, &o);
    if (st != OXM_OK) {
      Error e = from_status(st, op, l.device(), r.device());
      e.expected = l.shape(); e.got = r.shape();
      return e;
    }
    return out;
  }

  Result<Tensor> reduce(int code, const char *op, const Tensor &a, const std::vector<size_t> &axes) {
    if (!(a.device() == device())) {
      Error e{Error::Kind::DeviceMismatch};
      e.lhs_device = a.device(); e.rhs_device = device(); e.op = op;
      return e;
    }
    const size_t nd = a.shape().ndim();
    std::vector<bool> gone(nd, axes.empty());
    std::vector<int32_t> ax;
    for (size_t x : axes) {
      if (x >= nd || gone[x]) {
        Error e{Error::Kind::IndexOutOfBounds};
        e.index = {x}; e.got = a.shape();
        return e;
      }
      gone[x] = true;
      ax.push_back(static_cast<int32_t>(x));
    }
    Dims kept;
    for (size_t d = 0; d < nd; ++d)
      if (!gone[d]) kept.push_back(a.shape().dims()[d]);
    auto out = empty(Shape(kept), a.dtype());
    if (out.is_err()) return out;
    oxm_view v = view(a), o = view(out.unwrap());
    const int st = oxm_reduce(ctx_, code, &v, ax.empty() ? nullptr : ax.data(), static_cast<int>(ax.size()), &o);
    if (st != OXM_OK) return from_status(st, op, a.device(), device());
    return out;
  }

  Result<Tensor> run(const Tensor &lhs, const Tensor &rhs, bool batched) {
    const char *op = batched ? "batched_matmul" : "matmul";
    for (const Tensor *t : {&lhs, &rhs}) {
      if (!(t->device() == device())) {
        Error e{Error::Kind::DeviceMismatch};
        e.lhs_device = t->device(); e.rhs_device = device(); e.op = op;
        return e;
      }
    }
    // Enough of the output shape to allocate; the library owns validation.
    Shape oshape{1, 1};
    const size_t an = lhs.shape().ndim(), bn = rhs.shape().ndim();
    if (an >= 2 && bn >= 2 && (batched || (an == 2 && bn == 2))) {
      auto lead = broadcast_shapes(Shape(Dims(lhs.shape().dims().begin(), lhs.shape().dims().end() - 2)),
                                   Shape(Dims(rhs.shape().dims().begin(), rhs.shape().dims().end() - 2)));
      if (lead.is_err()) {
        Error e = lead.unwrap_err();
        e.expected = lhs.shape(); e.got = rhs.shape();
        return e;
      }
      Dims d = lead.unwrap().dims();
      d.push_back(lhs.shape().dims()[an - 2]);
      d.push_back(rhs.shape().dims()[bn - 1]);
      oshape = Shape(d);
    }
    auto out = empty(oshape, lhs.dtype());
    if (out.is_err()) return out;
    oxm_view a = view(lhs), b = view(rhs), o = view(out.unwrap());
    const int st = batched ? oxm_batched_matmul(ctx_, &a, &b, &o) : oxm_matmul(ctx_, &a, &b, &o);
    if (st != OXM_OK) {
      Error e = from_status(st, op, lhs.device(), rhs.device());
      e.expected = lhs.shape(); e.got = rhs.shape();
      return e;
    }
    return out;
  }

  oxm_ctx *ctx_;
  size_t index_;
};

}  // namespace oxmera
