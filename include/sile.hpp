// C++ mirror of sile's host-side launch surface over libsile_cuda (include/sile_cuda.h).
//
// The reference is a Rust crate; without a Rust toolchain its host layer is restated here in
// C++ with the same names, argument meaning and error behaviour, so a program (or test) reads
// like the reference's own:
//
//   reference (crates/sile/examples/matmul.rs:20-41)          here
//   let device = Device::default()?;                          auto device = sile::Device::default_device();
//   let stream = device.create_stream()?;                     auto stream = device.create_stream();
//   let a = Tensor::random([m, k], &device)?;                 auto a = sile::Tensor::random({m, k}, device);
//   matmul::<BM,BN,BK>(&a, &b, &mut c)                        sile::matmul<BM, BN, BK>(a, b, c)
//       .grid((gx, gy, 1)).apply(&stream)?;                       .grid({gx, gy, 1}).apply(stream);
//   let host = c.to_vec(&stream)?;                            auto host = c.to_vec(stream);
//
// Types mirrored: Device / Stream (crates/sile-core/src/device.rs:16-49, stream.rs:4-19), Error
// (error.rs:2-13), Tensor (crates/sile/src/tensor.rs:27-88), LaunchConfig / KernelArg
// (crates/sile-core/src/kernel.rs:4-14), KernelLauncher (crates/sile/src/kernel_launcher.rs:15-74).
// The kernels are the reference's example kernels (crates/sile/examples/*.rs), recognised by
// name instead of being compiled from a proc-macro body.
//
// Differences, all forced by the backend: the only executable device is Cuda (Cpu / Metal / Wgpu
// devices can be constructed, as in the reference, and fail at apply() with UnsupportedBackend,
// exactly as the reference's Cuda device does today, kernel_launcher.rs:69-71); Result<T> becomes
// a thrown sile::Error.
//
// Beyond the reference: a Tensor made for a Cuda device LIVES on that device (the reference's is
// a host Vec<f32> that every GPU backend uploads per launch, tensor.rs:5-9,
// metal/mod.rs:117-125) and a Cuda Stream is a real stream.  from_vec / zeros / ones / random
// upload once, apply() launches asynchronously on the stream with device pointers
// (sile_cuda_launch), and to_vec(stream) synchronises the stream and downloads.  A chain such as
// gemm -> matvec -> relu (examples/mlp.rs) therefore moves no data between its kernels.
#ifndef SILE_HPP
#define SILE_HPP

#include <algorithm>
#include <array>
#include <cstdint>
#include <cstdlib>
#include <initializer_list>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "sile_cuda.h"

namespace sile {

// crates/sile-core/src/error.rs:2-13
class Error : public std::runtime_error {
 public:
  enum class Kind { InvalidDevice, UnsupportedBackend, Compile, Io, Shape };
  Error(Kind kind, const std::string& what) : std::runtime_error(prefix(kind) + what), kind_(kind) {}
  Kind kind() const { return kind_; }

 private:
  static std::string prefix(Kind k) {
    switch (k) {
      case Kind::InvalidDevice: return "invalid SILE_DEVICE value: ";
      case Kind::UnsupportedBackend: return "backend not implemented: ";
      case Kind::Compile: return "compile failed: ";
      case Kind::Io: return "io error: ";
      default: return "shape mismatch: ";
    }
  }
  Kind kind_;
};

class Stream;

// crates/sile-core/src/device.rs:16-49
class Device {
 public:
  enum class Kind { Cpu, Metal, Cuda, Wgpu };
  static Device cpu() { return Device(Kind::Cpu); }
  static Device metal() { return Device(Kind::Metal); }
  static Device cuda(int index = 0) { return Device(Kind::Cuda, index); }
  static Device wgpu() { return Device(Kind::Wgpu); }
  // Device::default(): SILE_DEVICE selects the backend; unset means Cpu in the reference.
  static Device default_device() {
    const char* e = std::getenv("SILE_DEVICE");
    if (!e) return cpu();
    const std::string v(e);
    if (v == "C" || v == "CPU") return cpu();
    if (v == "METAL") return metal();
    if (v == "CUDA") return cuda();
    if (v == "WGPU") return wgpu();
    throw Error(Error::Kind::InvalidDevice, v);
  }
  Stream create_stream() const;
  Kind kind() const { return kind_; }
  int index() const { return index_; }
  bool operator==(const Device& o) const { return kind_ == o.kind_ && index_ == o.index_; }

 private:
  explicit Device(Kind k, int index = 0) : kind_(k), index_(index) {}
  Kind kind_;
  int index_;
};

// crates/sile-core/src/stream.rs:4-19.  synchronize() is a no-op in the reference; here a Cuda
// stream is a real one: launches are queued on it and synchronize() waits for them and reports a
// device-side time-out recorded meanwhile.
class Stream {
 public:
  const Device& device() const { return device_; }
  void* handle() const { return handle_.get(); }  // cudaStream_t for a Cuda device, else null
  void synchronize() const {
    if (device_.kind() != Device::Kind::Cuda) return;
    const int rc = sile_cuda_synchronize(handle());
    if (rc != SILE_OK) throw Error(Error::Kind::Io, sile_cuda_last_error());
  }

 private:
  friend class Device;
  explicit Stream(Device d) : device_(std::move(d)) {
    if (device_.kind() != Device::Kind::Cuda) return;
    if (sile_cuda_set_device(device_.index()) != SILE_OK) throw Error(Error::Kind::InvalidDevice, sile_cuda_last_error());
    void* st = nullptr;
    if (sile_cuda_stream_create(&st) != SILE_OK) throw Error(Error::Kind::Io, sile_cuda_last_error());
    handle_ = std::shared_ptr<void>(st, [](void* p) { sile_cuda_stream_destroy(p); });
  }
  Device device_;
  std::shared_ptr<void> handle_;
};
inline Stream Device::create_stream() const { return Stream(*this); }

// crates/sile/src/tensor.rs:5-88: f32 data with a shape and the device it was made for.  On a Cuda
// device the data is a device buffer (shared by copies of the Tensor, freed with the last one);
// on the other devices it is the reference's host vector.
class Tensor {
 public:
  using Shape = std::vector<int64_t>;
  static Tensor zeros(Shape shape, const Device& d) { return filled(std::move(shape), 0.0f, d); }
  static Tensor ones(Shape shape, const Device& d) { return filled(std::move(shape), 1.0f, d); }
  static Tensor random(Shape shape, const Device& d) {  // uniform [0, 1), unseeded, as tensor.rs:39-50
    std::vector<float> host(count(shape));
    std::mt19937 rng(std::random_device{}());
    std::uniform_real_distribution<float> u(0.0f, 1.0f);
    for (float& x : host) x = u(rng);
    return Tensor(std::move(host), std::move(shape), d);
  }
  static Tensor from_vec(std::vector<float> data, Shape shape, const Device& d) {
    const size_t len = count(shape);
    if (data.size() != len)
      throw Error(Error::Kind::Shape, "expected " + std::to_string(len) + " elements, got " + std::to_string(data.size()));
    return Tensor(std::move(data), std::move(shape), d);
  }
  const Shape& shape() const { return shape_; }
  size_t len() const { return len_; }
  // The pointer a kernel argument carries (tensor.rs:64-81): device memory on a Cuda device.
  const float* as_ptr() const { return dev_ ? static_cast<const float*>(dev_.get()) : host_.data(); }
  float* as_mut_ptr() { return dev_ ? static_cast<float*>(dev_.get()) : host_.data(); }
  // tensor.rs:83-85.  On a Cuda device: waits for the work queued on `stream`, then downloads.
  std::vector<float> to_vec(const Stream& stream) const {
    if (!dev_) return host_;
    std::vector<float> out(len_);
    const void* st = stream.device() == device_ ? stream.handle() : nullptr;
    if (sile_cuda_set_device(device_.index()) != SILE_OK) throw Error(Error::Kind::InvalidDevice, sile_cuda_last_error());
    if (sile_cuda_memcpy_d2h(out.data(), dev_.get(), len_ * sizeof(float), const_cast<void*>(st)) != SILE_OK)
      throw Error(Error::Kind::Io, sile_cuda_last_error());
    return out;
  }
  const Device& device() const { return device_; }
  bool on_device() const { return static_cast<bool>(dev_); }

 private:
  Tensor(std::vector<float> data, Shape shape, Device d) : shape_(std::move(shape)), device_(std::move(d)), len_(data.size()) {
    if (device_.kind() != Device::Kind::Cuda) {
      host_ = std::move(data);
      return;
    }
    if (sile_cuda_set_device(device_.index()) != SILE_OK) throw Error(Error::Kind::InvalidDevice, sile_cuda_last_error());
    void* p = nullptr;
    if (sile_cuda_malloc(&p, std::max<size_t>(len_, 1) * sizeof(float)) != SILE_OK) throw Error(Error::Kind::Io, sile_cuda_last_error());
    dev_ = std::shared_ptr<void>(p, [](void* q) { sile_cuda_free(q); });
    if (sile_cuda_memcpy_h2d(p, data.data(), len_ * sizeof(float), nullptr) != SILE_OK) throw Error(Error::Kind::Io, sile_cuda_last_error());
  }
  static size_t count(const Shape& s) {
    size_t n = 1;
    for (int64_t v : s) n *= static_cast<size_t>(v);
    return n;
  }
  static Tensor filled(Shape shape, float v, const Device& d) {
    const size_t n = count(shape);
    return Tensor(std::vector<float>(n, v), std::move(shape), d);
  }
  std::vector<float> host_;
  std::shared_ptr<void> dev_;
  Shape shape_;
  Device device_;
  size_t len_ = 0;
};

// crates/sile-core/src/kernel.rs:4-14
struct LaunchConfig {
  std::array<uint32_t, 3> grid{1, 1, 1};
};
struct KernelArg {
  float* mut_ptr;
  const std::vector<int64_t>* shape;
};

// crates/sile/src/kernel_launcher.rs:15-74: kernel + args + grid; apply() dispatches on the
// stream's device.  Only the Cuda arm exists here.
class KernelLauncher {
 public:
  KernelLauncher(SileKernelDesc desc, std::vector<KernelArg> args) : desc_(desc), args_(std::move(args)) {}
  KernelLauncher& grid(std::array<uint32_t, 3> g) {
    launch_.grid = g;
    return *this;
  }
  void apply(const Stream& stream) {
    switch (stream.device().kind()) {
      case Device::Kind::Cuda: break;
      default: throw Error(Error::Kind::UnsupportedBackend, "backend not implemented");
    }
    int rc = sile_cuda_set_device(stream.device().index());
    if (rc != SILE_OK) throw Error(Error::Kind::InvalidDevice, sile_cuda_last_error());
    std::vector<void*> buffers;
    std::vector<int64_t> shapes;  // concatenation of every argument's shape (cpu/mod.rs:104-107)
    for (const KernelArg& a : args_) {
      buffers.push_back(a.mut_ptr);
      shapes.insert(shapes.end(), a.shape->begin(), a.shape->end());
    }
    // Arguments are device buffers of tensors made for a Cuda device; the launch is queued on the
    // stream and errors of the kernel itself surface at Stream::synchronize / Tensor::to_vec.
    rc = sile_cuda_launch(&desc_, buffers.data(), shapes.data(), static_cast<int64_t>(shapes.size()), launch_.grid.data(), stream.handle());
    if (rc == SILE_OK) return;
    const std::string msg = sile_cuda_last_error();
    switch (rc) {
      case SILE_ERR_INVALID: throw Error(Error::Kind::Shape, msg);
      case SILE_ERR_UNSUPPORTED: throw Error(Error::Kind::UnsupportedBackend, msg);
      case SILE_ERR_NO_DEVICE: throw Error(Error::Kind::InvalidDevice, msg);
      default: throw Error(Error::Kind::Io, msg);
    }
  }

 private:
  SileKernelDesc desc_;
  std::vector<KernelArg> args_;
  LaunchConfig launch_;
};

namespace detail {
inline SileKernelDesc f32_desc(int op, std::initializer_list<int64_t> consts) {
  SileKernelDesc d{};
  d.struct_size = sizeof(SileKernelDesc);
  d.op = op;
  d.in_dtype = SILE_DTYPE_F32;
  d.out_dtype = SILE_DTYPE_F32;
  d.b_layout = SILE_LAYOUT_ROW_MAJOR;
  d.scale = 1.0f;
  int i = 0;
  for (int64_t c : consts) d.consts[i++] = c;
  return d;
}
inline KernelArg arg(const Tensor& t) { return KernelArg{const_cast<float*>(t.as_ptr()), &t.shape()}; }
inline KernelArg arg(Tensor& t) { return KernelArg{t.as_mut_ptr(), &t.shape()}; }
}  // namespace detail

// The reference's example kernels, const generics as template arguments.
// matmul / gemm: crates/sile/examples/matmul.rs:3-18, mlp.rs:6-22
template <int64_t BM, int64_t BN, int64_t BK>
KernelLauncher matmul(const Tensor& a, const Tensor& b, Tensor& c) {
  return KernelLauncher(detail::f32_desc(SILE_OP_MATMUL, {BM, BN, BK}), {detail::arg(a), detail::arg(b), detail::arg(c)});
}
template <int64_t BM, int64_t BN, int64_t BK>
KernelLauncher gemm(const Tensor& a, const Tensor& b, Tensor& c) {
  return matmul<BM, BN, BK>(a, b, c);
}
// vec_add: crates/sile/examples/vec_add.rs:3-10 (tile of 4 elements)
inline KernelLauncher vec_add(const Tensor& a, const Tensor& b, Tensor& c) {
  return KernelLauncher(detail::f32_desc(SILE_OP_VEC_ADD, {4}), {detail::arg(a), detail::arg(b), detail::arg(c)});
}
// relu: crates/sile/examples/mlp.rs:51-55
template <int64_t D>
KernelLauncher relu(Tensor& x) {
  return KernelLauncher(detail::f32_desc(SILE_OP_RELU, {D}), {detail::arg(x)});
}
// softmax: crates/sile/examples/softmax.rs:3-16
template <int64_t BM, int64_t BN>
KernelLauncher softmax(const Tensor& x, Tensor& y) {
  return KernelLauncher(detail::f32_desc(SILE_OP_SOFTMAX, {BM, BN}), {detail::arg(x), detail::arg(y)});
}
// parallel_reduce: crates/sile/examples/parallel_reduce.rs:3-9
template <int64_t TILE>
KernelLauncher parallel_reduce(const Tensor& a, Tensor& out) {
  return KernelLauncher(detail::f32_desc(SILE_OP_PARALLEL_REDUCE, {TILE}), {detail::arg(a), detail::arg(out)});
}
// matvec: crates/sile/examples/mlp.rs:28-46
template <int64_t BM, int64_t BK>
KernelLauncher matvec(const Tensor& x, const Tensor& y, Tensor& z) {
  return KernelLauncher(detail::f32_desc(SILE_OP_MATVEC, {BM, BK}), {detail::arg(x), detail::arg(y), detail::arg(z)});
}

}  // namespace sile

#endif  // SILE_HPP
