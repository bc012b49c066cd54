// The reference's own integration tests and examples, replayed through the C++ mirror of its
// host API (include/sile.hpp).  Each case names the reference test it follows.
//   reference_tests            all cases (needs an sm_100 GPU)
//   reference_tests --host     only the cases that never reach the device
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "sile.hpp"

using sile::Device;
using sile::Error;
using sile::Tensor;

static int failures = 0;
#define CHECK(cond, ...)                         \
  do {                                           \
    if (!(cond)) {                               \
      std::printf("  FAILED %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                  \
      std::printf("\n");                         \
      ++failures;                                \
      return;                                    \
    }                                            \
  } while (0)

// crates/sile/tests/backend_matmul.rs:21-72
static void cuda_backend_executes_matmul_through_tile_pipeline() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  constexpr int64_t BM = 2, BN = 2, BK = 2;
  Tensor a = Tensor::from_vec({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16}, {4, 4}, device);
  Tensor b = Tensor::from_vec({1, 0, 2, 1, 0, 1, 3, 2, 1, 0, 4, 3, 0, 1, 5, 4}, {4, 4}, device);
  Tensor c = Tensor::zeros({4, 4}, device);
  sile::matmul<BM, BN, BK>(a, b, c).grid({4, 1, 1}).apply(stream);
  const std::vector<float> actual = c.to_vec(stream);
  const float expected[16] = {4, 6, 40, 30, 12, 14, 96, 70, 20, 22, 152, 110, 28, 30, 208, 150};
  for (int i = 0; i < 16; ++i) CHECK(std::fabs(actual[i] - expected[i]) < 1e-4f, "mismatch at %d: got %f, expected %f", i, actual[i], expected[i]);
}

// crates/sile/tests/backend_vec_add.rs:11-25
static void cuda_backend_executes_vec_add() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  Tensor a = Tensor::from_vec(std::vector<float>(16, 1.0f), {16}, device);
  Tensor b = Tensor::from_vec(std::vector<float>(16, 2.0f), {16}, device);
  Tensor c = Tensor::zeros({16}, device);
  sile::vec_add(a, b, c).grid({4, 1, 1}).apply(stream);
  for (float v : c.to_vec(stream)) CHECK(v == 3.0f, "got %f", v);
}

// crates/sile/tests/llvm_ir_cpu_runtime.rs:105-141
static void cuda_backend_executes_relu_max_tile() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  Tensor x = Tensor::from_vec({-3.0f, -1.0f, 0.0f, 2.5f, 4.0f, -7.0f, 8.0f, -0.5f}, {8}, device);
  sile::relu<8>(x).grid({1, 1, 1}).apply(stream);
  const float expected[8] = {0, 0, 0, 2.5f, 4.0f, 0, 8.0f, 0};
  const auto got = x.to_vec(stream);
  for (int i = 0; i < 8; ++i) CHECK(got[i] == expected[i], "relu[%d] = %f", i, got[i]);
}

// crates/sile/tests/backend_softmax.rs:17-38
static void cuda_backend_executes_softmax_rows_that_sum_to_one() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  std::vector<float> data(32);
  for (int i = 0; i < 32; ++i) data[i] = static_cast<float>(i);
  Tensor x = Tensor::from_vec(data, {4, 8}, device);
  Tensor y = Tensor::zeros({4, 8}, device);
  sile::softmax<2, 8>(x, y).grid({2, 1, 1}).apply(stream);
  const auto out = y.to_vec(stream);
  for (int r = 0; r < 4; ++r) {
    float sum = 0;
    for (int c = 0; c < 8; ++c) sum += out[r * 8 + c];
    CHECK(std::fabs(sum - 1.0f) < 1e-4f, "softmax row sum = %f, expected 1.0", sum);
  }
}

// crates/sile/tests/backend_parallel_reduce.rs:11-29
static void cuda_backend_executes_parallel_reduce_with_atomic_add() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  constexpr int64_t TILE = 1000, LEN = 100000;
  Tensor a = Tensor::from_vec(std::vector<float>(LEN, 1.0f), {LEN}, device);
  Tensor out = Tensor::zeros({1}, device);
  sile::parallel_reduce<TILE>(a, out).grid({static_cast<uint32_t>(LEN / TILE), 1, 1}).apply(stream);
  const float result = out.to_vec(stream)[0];
  CHECK(std::fabs(result - static_cast<float>(LEN)) < 1e-4f, "got %f", result);
}

// crates/sile/examples/matmul.rs:20-58: 128 x 128 x 64, tiles 32 x 16 x 8, host check 1e-2
static void example_matmul() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  constexpr int64_t m = 128, n = 128, k = 64, BM = 32, BN = 16, BK = 8;
  Tensor a = Tensor::random({m, k}, device), b = Tensor::random({k, n}, device);
  Tensor c = Tensor::zeros({m, n}, device);
  sile::matmul<BM, BN, BK>(a, b, c).grid({static_cast<uint32_t>(m / BM), static_cast<uint32_t>(n / BN), 1}).apply(stream);
  const auto ah = a.to_vec(stream), bh = b.to_vec(stream), ch = c.to_vec(stream);
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0;
      for (int64_t kk = 0; kk < k; ++kk) sum += ah[i * k + kk] * bh[kk * n + j];
      CHECK(std::fabs(ch[i * n + j] - sum) < 1e-2f, "c[%lld,%lld] = %f, host %f", (long long)i, (long long)j, ch[i * n + j], sum);
    }
}

// crates/sile/examples/mlp.rs:60-153: gemm -> matvec -> relu, tolerance 1e-3
static void example_mlp() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  constexpr int64_t dim = 64;
  Tensor w0 = Tensor::random({dim, dim}, device), w1 = Tensor::random({dim}, device), x = Tensor::random({dim, dim}, device);
  Tensor out0 = Tensor::zeros({dim, dim}, device);
  sile::gemm<32, 32, 8>(x, w0, out0).grid({2, 2, 1}).apply(stream);
  Tensor out1 = Tensor::zeros({dim}, device);
  sile::matvec<32, 8>(out0, w1, out1).grid({2, 1, 1}).apply(stream);
  sile::relu<64>(out1).grid({1, 1, 1}).apply(stream);
  const auto xh = x.to_vec(stream), w0h = w0.to_vec(stream), w1h = w1.to_vec(stream), got = out1.to_vec(stream);
  for (int64_t i = 0; i < dim; ++i) {
    float acc = 0;
    for (int64_t j = 0; j < dim; ++j) {
      float s = 0;
      for (int64_t kk = 0; kk < dim; ++kk) s += xh[i * dim + kk] * w0h[kk * dim + j];
      acc += s * w1h[j];
    }
    if (acc < 0) acc = 0;
    CHECK(std::fabs(got[i] - acc) < 1e-3f * std::fmax(1.0f, std::fabs(acc)), "mlp[%lld] = %f, host %f", (long long)i, got[i], acc);
  }
}

// crates/sile-core/tests/device_selection.rs and crates/sile/tests/device_selection.rs
static void device_selection_follows_sile_device() {
  unsetenv("SILE_DEVICE");
  CHECK(Device::default_device() == Device::cpu(), "unset SILE_DEVICE must select the cpu device");
  setenv("SILE_DEVICE", "CUDA", 1);
  CHECK(Device::default_device() == Device::cuda(), "SILE_DEVICE=CUDA");
  setenv("SILE_DEVICE", "METAL", 1);
  CHECK(Device::default_device() == Device::metal(), "SILE_DEVICE=METAL");
  setenv("SILE_DEVICE", "bogus", 1);
  bool threw = false;
  try {
    Device::default_device();
  } catch (const Error& e) {
    threw = e.kind() == Error::Kind::InvalidDevice && std::string(e.what()) == "invalid SILE_DEVICE value: bogus";
  }
  unsetenv("SILE_DEVICE");
  CHECK(threw, "an unknown SILE_DEVICE value must raise InvalidDevice");
}

// crates/sile/src/kernel_launcher.rs:55-72: a device without a backend fails at apply()
static void devices_without_a_backend_report_unsupported_backend() {
  for (Device device : {Device::cpu(), Device::metal(), Device::wgpu()}) {
    auto stream = device.create_stream();
    Tensor a = Tensor::ones({16}, device), b = Tensor::ones({16}, device), c = Tensor::zeros({16}, device);
    bool threw = false;
    try {
      sile::vec_add(a, b, c).grid({4, 1, 1}).apply(stream);
    } catch (const Error& e) {
      threw = e.kind() == Error::Kind::UnsupportedBackend && std::string(e.what()) == "backend not implemented: backend not implemented";
    }
    CHECK(threw, "apply() on a device without a backend must raise UnsupportedBackend");
    CHECK(c.to_vec(stream)[0] == 0.0f, "output must be untouched");
  }
}

// crates/sile/src/tensor.rs:52-66
static void from_vec_checks_the_element_count() {
  bool threw = false;
  try {
    Tensor::from_vec({1, 2, 3}, {2, 2}, Device::cuda());
  } catch (const Error& e) {
    threw = e.kind() == Error::Kind::Shape && std::string(e.what()) == "shape mismatch: expected 4 elements, got 3";
  }
  CHECK(threw, "from_vec with the wrong element count must raise Shape");
}

int main(int argc, char** argv) {
  const bool host_only = argc > 1 && !std::strcmp(argv[1], "--host");
  struct Case { const char* name; std::function<void()> fn; bool needs_gpu; };
  const std::vector<Case> cases = {
      {"device_selection_follows_sile_device", device_selection_follows_sile_device, false},
      {"devices_without_a_backend_report_unsupported_backend", devices_without_a_backend_report_unsupported_backend, false},
      {"from_vec_checks_the_element_count", from_vec_checks_the_element_count, false},
      {"cuda_backend_executes_matmul_through_tile_pipeline", cuda_backend_executes_matmul_through_tile_pipeline, true},
      {"cuda_backend_executes_vec_add", cuda_backend_executes_vec_add, true},
      {"cuda_backend_executes_relu_max_tile", cuda_backend_executes_relu_max_tile, true},
      {"cuda_backend_executes_softmax_rows_that_sum_to_one", cuda_backend_executes_softmax_rows_that_sum_to_one, true},
      {"cuda_backend_executes_parallel_reduce_with_atomic_add", cuda_backend_executes_parallel_reduce_with_atomic_add, true},
      {"example_matmul", example_matmul, true},
      {"example_mlp", example_mlp, true},
  };
  int ran = 0;
  for (const Case& c : cases) {
    if (host_only && c.needs_gpu) continue;
    const int before = failures;
    try {
      c.fn();
    } catch (const std::exception& e) {
      std::printf("  EXCEPTION in %s: %s\n", c.name, e.what());
      ++failures;
    }
    std::printf("%s %s\n", failures == before ? "ok  " : "FAIL", c.name);
    ++ran;
  }
  std::printf("%d cases, %d failures\n", ran, failures);
  return failures ? 1 : 0;
}
