// The reference's exercise specs, restated against the C++ host mirror
// (oxmera_b200/host/oxmera.hpp).  Each test names the spec it follows.
//
//   spec_tests cpu   A1 / A2 / A3 / A5 hand cases, dispatch, and the A4 matmul
//                    spec through a CpuBackend that wraps the CPU oracle
//   spec_tests gpu   the A4 matmul spec through B200Backend on cuda:0
//
// The CpuBackend below exists only in this test: the oracle is test
// infrastructure and the shipped host mirror has no CPU compute path.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>

#include "../../oracle/oxm_oracle.h"
#include "../../oxmera_b200/host/oxmera.hpp"

using namespace oxmera;

static int g_failed = 0, g_checks = 0;
#define CHECK(cond)                                                                  \
  do {                                                                               \
    ++g_checks;                                                                      \
    if (!(cond)) {                                                                   \
      ++g_failed;                                                                    \
      std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond);                    \
    }                                                                                \
  } while (0)

// ---- test-only CPU backend: oxmera-cpu's matmul as the oracle restates it ----
class CpuBackend : public Backend {
 public:
  Device device() const override { return Device::cpu(); }
  const char *name() const override { return "cpu-reference"; }  // crates/oxmera-cpu/src/lib.rs:95-97
  Result<Tensor> matmul(const Tensor &lhs, const Tensor &rhs) override { return run(lhs, rhs, false); }
  Result<Tensor> batched_matmul(const Tensor &lhs, const Tensor &rhs) override { return run(lhs, rhs, true); }

 private:
  static orc_view view(const Tensor &t) {
    orc_view v{};
    v.dtype = static_cast<int32_t>(t.dtype());
    v.ndim = static_cast<int32_t>(t.shape().ndim());
    for (size_t i = 0; i < t.shape().ndim(); ++i) {
      v.shape[i] = static_cast<int64_t>(t.shape().dims()[i]);
      v.strides[i] = static_cast<int64_t>(t.layout().strides.values()[i]);
    }
    v.offset = static_cast<int64_t>(t.layout().offset);
    v.base = const_cast<uint8_t *>(t.storage()->cpu_bytes());
    return v;
  }
  Result<Tensor> run(const Tensor &lhs, const Tensor &rhs, bool batched) {
    orc_view a = view(lhs), b = view(rhs);
    int st = orc_check_matmul(&a, &b, nullptr, batched ? 1 : 0);
    if (st != ORC_OK) {
      Error e{static_cast<Error::Kind>(st)};
      e.expected = lhs.shape(); e.got = rhs.shape(); e.op = "matmul";
      return e;
    }
    const size_t an = lhs.shape().ndim(), bn = rhs.shape().ndim();
    auto lead = broadcast_shapes(Shape(Dims(lhs.shape().dims().begin(), lhs.shape().dims().end() - 2)),
                                 Shape(Dims(rhs.shape().dims().begin(), rhs.shape().dims().end() - 2)));
    Dims d = lead.unwrap().dims();
    d.push_back(lhs.shape().dims()[an - 2]);
    d.push_back(rhs.shape().dims()[bn - 1]);
    Shape os(d);
    auto out = Tensor::from_storage(Storage::cpu_zeros(os.numel(), lhs.dtype()), Layout::contiguous(os));
    orc_view o = view(out.unwrap());
    o.base = out.unwrap().storage()->cpu_bytes_mut();
    st = batched ? orc_batched_matmul(&a, &b, &o, ORC_ACC_NATIVE, 1) : orc_matmul(&a, &b, &o, ORC_ACC_NATIVE, 1);
    if (st != ORC_OK) {
      Error e{static_cast<Error::Kind>(st)};
      e.op = "matmul";
      return e;
    }
    return out;
  }
};

static Tensor t(const std::vector<float> &data, Shape shape) { return Tensor::from_vec_f32(data, std::move(shape)).unwrap(); }

// ---- A1: exercises/a1-shape-and-strides/tests/spec.rs ----
static void a1_shape_and_strides() {
  CHECK(size_in_bytes(DType::F32) == 4 && size_in_bytes(DType::F64) == 8 && size_in_bytes(DType::I32) == 4);
  CHECK(size_in_bytes(DType::I64) == 8 && size_in_bytes(DType::U8) == 1 && size_in_bytes(DType::Bool) == 1);
  CHECK(size_in_bytes(DType::BF16) == 2 && size_in_bytes(DType::F16) == 2);
  CHECK(is_float(DType::F32) && is_float(DType::F64) && !is_float(DType::I32) && !is_float(DType::I64));
  CHECK(!is_float(DType::U8) && !is_float(DType::Bool));
  CHECK(Shape{}.numel() == 1);
  CHECK((Shape{0}).numel() == 0 && (Shape{2, 3}).numel() == 6 && (Shape{2, 0, 3}).numel() == 0 && (Shape{1, 1, 1}).numel() == 1);
  CHECK(contiguous_strides(Shape{}).values().empty());
  CHECK((contiguous_strides(Shape{4}).values() == std::vector<ptrdiff_t>{1}));
  CHECK((contiguous_strides(Shape{2, 3}).values() == std::vector<ptrdiff_t>{3, 1}));
  CHECK((contiguous_strides(Shape{2, 1, 3}).values() == std::vector<ptrdiff_t>{3, 3, 1}));
  CHECK((contiguous_strides(Shape{4, 2, 3}).values() == std::vector<ptrdiff_t>{6, 3, 1}));
  Layout l = Layout::contiguous(Shape{2, 3});
  CHECK(l.offset_of({0, 0}).unwrap() == 0 && l.offset_of({0, 2}).unwrap() == 2);
  CHECK(l.offset_of({1, 0}).unwrap() == 3 && l.offset_of({1, 2}).unwrap() == 5);
  CHECK(Layout::contiguous(Shape{}).offset_of({}).unwrap() == 0);
  CHECK(l.offset_of({0}).unwrap_err().kind == Error::Kind::RankMismatch);
  CHECK(l.offset_of({0, 0, 0}).unwrap_err().kind == Error::Kind::RankMismatch);
  CHECK(l.offset_of({2, 0}).unwrap_err().kind == Error::Kind::IndexOutOfBounds);
  CHECK(l.offset_of({0, 3}).unwrap_err().kind == Error::Kind::IndexOutOfBounds);
  CHECK(l.is_contiguous() && Layout::contiguous(Shape{}).is_contiguous() && Layout::contiguous(Shape{0, 3}).is_contiguous());
  Layout transposed{Shape{2, 3}, Strides({1, 2}), 0};
  CHECK(!transposed.is_contiguous());
}

// ---- A2: exercises/a2-broadcasting/tests/spec.rs ----
static void a2_broadcasting() {
  struct C { Dims l, r, e; };
  const std::vector<C> ok = {{{2, 3}, {3}, {2, 3}}, {{3}, {2, 3}, {2, 3}}, {{2, 1}, {1, 3}, {2, 3}}, {{}, {2, 3}, {2, 3}},
                             {{2, 3}, {}, {2, 3}}, {{}, {}, {}}, {{4, 1, 5}, {3, 1}, {4, 3, 5}}, {{1}, {1}, {1}},
                             {{5}, {1}, {5}}, {{0}, {1}, {0}}, {{2, 0}, {1, 1}, {2, 0}}};
  for (const auto &c : ok) {
    auto r = broadcast_shapes(Shape(c.l), Shape(c.r));
    CHECK(r.is_ok() && r.unwrap() == Shape(c.e));
    auto rr = broadcast_shapes(Shape(c.r), Shape(c.l));  // commutative
    CHECK(rr.is_ok() && rr.unwrap() == Shape(c.e));
  }
  const std::vector<std::pair<Dims, Dims>> bad = {{{2}, {3}}, {{2, 3}, {2, 4}}, {{4, 3}, {2, 1, 2}}, {{0}, {2}}};
  for (const auto &c : bad) {
    auto r = broadcast_shapes(Shape(c.first), Shape(c.second));
    CHECK(r.is_err() && r.unwrap_err().kind == Error::Kind::BroadcastIncompatible);
    CHECK(r.unwrap_err().expected == Shape(c.first) && r.unwrap_err().got == Shape(c.second));  // operands verbatim
  }
}

// ---- A3: exercises/a3-strided-views/tests/spec.rs ----
static void a3_strided_views() {
  Tensor x = t({1, 2, 3, 4, 5, 6}, Shape{2, 3});
  Tensor tt = x.permute({1, 0}).unwrap();
  CHECK(tt.shape() == (Shape{3, 2}));
  CHECK(tt.get_f32({0, 0}).unwrap() == 1.0f && tt.get_f32({0, 1}).unwrap() == 4.0f);
  CHECK(tt.get_f32({1, 0}).unwrap() == 2.0f && tt.get_f32({2, 1}).unwrap() == 6.0f);
  CHECK(tt.storage() == x.storage());
  Tensor n = x.narrow(1, 1, 2).unwrap();
  CHECK(n.shape() == (Shape{2, 2}) && n.storage() == x.storage());
  CHECK(n.get_f32({0, 0}).unwrap() == 2.0f && n.get_f32({0, 1}).unwrap() == 3.0f);
  CHECK(n.get_f32({1, 0}).unwrap() == 5.0f && n.get_f32({1, 1}).unwrap() == 6.0f);
  Tensor r = x.reshape(Shape{3, 2}).unwrap();
  CHECK(r.get_f32({0, 1}).unwrap() == 2.0f && r.get_f32({1, 0}).unwrap() == 3.0f && r.get_f32({2, 1}).unwrap() == 6.0f);
  CHECK(r.storage() == x.storage());
  CHECK(!tt.layout().is_contiguous());
  Tensor c = tt.contiguous().unwrap();
  CHECK(c.layout().is_contiguous() && c.storage() != tt.storage());
  for (size_t i = 0; i < 3; ++i)
    for (size_t j = 0; j < 2; ++j) CHECK(c.get_f32({i, j}).unwrap() == tt.get_f32({i, j}).unwrap());
  CHECK(x.contiguous().unwrap().storage() == x.storage());
  CHECK(x.permute({0, 0}).is_err() && x.permute({0}).is_err());
  CHECK(x.narrow(1, 2, 2).is_err() && x.narrow(2, 0, 1).is_err());
  CHECK(x.reshape(Shape{4, 2}).unwrap_err().kind == Error::Kind::ShapeMismatch);
  CHECK(Tensor::from_vec_f32(std::vector<float>(5, 1.0f), Shape{2, 3}).unwrap_err().kind == Error::Kind::ShapeMismatch);
}

// ---- A5: exercises/a5-error-taxonomy/tests/spec.rs ----
static void a5_error_taxonomy() {
  CHECK(std::string(Device::cpu().kind_name()) == "cpu");
  CHECK(std::string(Device::metal(0).kind_name()) == "metal");
  CHECK(std::string(Device::cuda(1).kind_name()) == "cuda");
  auto e = broadcast_shapes(Shape{2}, Shape{3}).unwrap_err();
  CHECK(e.to_string().find('2') != std::string::npos && e.to_string().find('3') != std::string::npos);
  Layout l = Layout::contiguous(Shape{2, 3});
  auto r = l.offset_of({0}).unwrap_err();
  CHECK(r.index_rank == 1 && r.shape_rank == 2);
  auto o = l.offset_of({0, 3}).unwrap_err();
  CHECK((o.index == std::vector<size_t>{0, 3}) && o.got == (Shape{2, 3}));
  CHECK(o.to_string().find("[0, 3]") != std::string::npos);
  Error sm{Error::Kind::ShapeMismatch};
  sm.expected = Shape{2, 2}; sm.got = Shape{2, 3}; sm.op = "matmul";
  CHECK(sm.to_string().find("matmul") != std::string::npos);
  Error dm{Error::Kind::DeviceMismatch};
  dm.lhs_device = Device::cpu(); dm.rhs_device = Device::metal(0); dm.op = "add";
  const std::string msg = dm.to_string();
  CHECK(msg.find("add") != std::string::npos && msg.find("Cpu") != std::string::npos && msg.find("Metal") != std::string::npos);
}

// ---- dispatch: crates/oxmera-runtime/tests/harness.rs:9-17 ----
static void runtime_dispatch() {
  unregister_all();
  auto r = backend_for(Device::cuda(0));
  CHECK(r.is_err() && r.unwrap_err().kind == Error::Kind::BackendUnavailable);
  auto cpu = std::make_shared<CpuBackend>();
  register_backend(cpu);
  CHECK(backend_for(Device::cpu()).unwrap().get() == cpu.get());
  auto cpu2 = std::make_shared<CpuBackend>();
  register_backend(cpu2);  // replaces the previous registration
  CHECK(backend_for(Device::cpu()).unwrap().get() == cpu2.get());
  // the umbrella harness: an operation through the tensor surface
  CHECK(t({1, 2, 3, 4}, Shape{2, 2}).matmul(t({5, 6, 7, 8}, Shape{2, 2})).unwrap().get_f32({1, 1}).unwrap() == 50.0f);
}

// ---- A4: exercises/a4-reference-matmul/tests/spec.rs, against any backend ----
struct Harness {
  Backend *be;
  std::function<Tensor(const std::vector<float> &, Shape)> make;  // a tensor on the backend's device
  std::function<Tensor(const Tensor &)> host;                     // back to CPU storage for get_f32
};

static void expect_tensor(const Harness &h, Result<Tensor> got, const std::vector<float> &exp, Shape shape) {
  CHECK(got.is_ok());
  if (got.is_err()) { std::printf("   error: %s\n", got.unwrap_err().to_string().c_str()); return; }
  CHECK(got.unwrap().shape() == shape);
  CHECK(got.unwrap().layout().is_contiguous());  // a fresh contiguous tensor (ops/lib.rs:16-17)
  Tensor c = h.host(got.unwrap());
  std::vector<size_t> ix(shape.ndim(), 0);
  for (size_t n = 0; n < shape.numel(); ++n) {  // row-major walk of any rank
    CHECK(c.get_f32(ix).unwrap() == exp[n]);
    for (size_t d = shape.ndim(); d-- > 0;) {
      if (++ix[d] < shape.dims()[d]) break;
      ix[d] = 0;
    }
  }
}

static void a4_reference_matmul(const Harness &h) {
  // hand_computed_2x2 (spec.rs:31-38)
  expect_tensor(h, h.be->matmul(h.make({1, 2, 3, 4}, Shape{2, 2}), h.make({5, 6, 7, 8}, Shape{2, 2})), {19, 22, 43, 50}, Shape{2, 2});
  // hand_computed_rectangular (:40-50)
  expect_tensor(h, h.be->matmul(h.make({1, 2, 3, 4, 5, 6}, Shape{2, 3}), h.make({1, 10, 100}, Shape{3, 1})), {321, 654}, Shape{2, 1});
  // identity_leaves_a_matrix_alone (:52-58)
  expect_tensor(h, h.be->matmul(h.make({1.5f, -2.0f, 0.25f, 4.0f}, Shape{2, 2}), h.make({1, 0, 0, 1}, Shape{2, 2})),
                {1.5f, -2.0f, 0.25f, 4.0f}, Shape{2, 2});
  // zero_annihilates (:60-66)
  expect_tensor(h, h.be->matmul(h.make({3, -1, 2, 7, 0.5f, -4}, Shape{2, 3}), h.make(std::vector<float>(6, 0.0f), Shape{3, 2})),
                {0, 0, 0, 0}, Shape{2, 2});
  // inner_dimension_mismatch_is_a_typed_error (:68-76)
  auto bad = h.be->matmul(h.make(std::vector<float>(6, 1.0f), Shape{2, 3}), h.make(std::vector<float>(8, 1.0f), Shape{4, 2}));
  CHECK(bad.is_err() && bad.unwrap_err().kind == Error::Kind::ShapeMismatch);
  CHECK(bad.is_err() && bad.unwrap_err().to_string().find("matmul") != std::string::npos);
  // non_rank_2_operands_are_refused (:78-83)
  CHECK(h.be->matmul(h.make(std::vector<float>(6, 1.0f), Shape{6}), h.make(std::vector<float>(6, 1.0f), Shape{6})).is_err());
  // matmul_works_on_a_transposed_view (:85-94)
  Tensor bt = h.make({5, 7, 6, 8}, Shape{2, 2}).permute({1, 0}).unwrap();
  expect_tensor(h, h.be->matmul(h.make({1, 2, 3, 4}, Shape{2, 2}), bt), {19, 22, 43, 50}, Shape{2, 2});
  // transpose_law and columns_are_independent (:96-130), seeded draws from (-8, 8)
  std::mt19937 rng(4);
  std::uniform_real_distribution<float> dist(-8.0f, 8.0f);
  auto draw = [&](size_t n) { std::vector<float> v(n); for (auto &x : v) x = dist(rng); return v; };
  auto close = [](float x, float y) { return std::fabs(x - y) <= 1e-4f * (1.0f + std::fmax(std::fabs(x), std::fabs(y))); };
  for (int rep = 0; rep < 16; ++rep) {
    Tensor a = h.make(draw(6), Shape{2, 3}), b = h.make(draw(6), Shape{3, 2});
    Tensor ab_t = h.host(h.be->matmul(a, b).unwrap().permute({1, 0}).unwrap());
    Tensor bt_at = h.host(h.be->matmul(b.permute({1, 0}).unwrap(), a.permute({1, 0}).unwrap()).unwrap());
    for (size_t i = 0; i < 2; ++i)
      for (size_t j = 0; j < 2; ++j) CHECK(close(ab_t.get_f32({i, j}).unwrap(), bt_at.get_f32({i, j}).unwrap()));
    Tensor a3 = h.make(draw(9), Shape{3, 3});
    Tensor full = h.host(h.be->matmul(a3, b).unwrap());
    for (size_t j = 0; j < 2; ++j) {
      Tensor col = h.host(h.be->matmul(a3, b.narrow(1, j, 1).unwrap()).unwrap());
      for (size_t i = 0; i < 3; ++i) CHECK(close(full.get_f32({i, j}).unwrap(), col.get_f32({i, 0}).unwrap()));
    }
  }
  // the batched extension: [2,1,2,2] x [1,3,2,2] broadcasts to [2,3,2,2]
  Tensor ba = h.make({1, 2, 3, 4, 0, 1, 1, 0}, Shape{2, 1, 2, 2});
  Tensor bb = h.make({1, 0, 0, 1, 2, 0, 0, 2, 0, 1, 1, 0}, Shape{1, 3, 2, 2});
  auto bo = h.be->batched_matmul(ba, bb);
  CHECK(bo.is_ok() && bo.unwrap().shape() == (Shape{2, 3, 2, 2}));
  if (bo.is_ok()) {
    Tensor o = h.host(bo.unwrap());
    const float exp[2][3][4] = {{{1, 2, 3, 4}, {2, 4, 6, 8}, {2, 1, 4, 3}}, {{0, 1, 1, 0}, {0, 2, 2, 0}, {1, 0, 0, 1}}};
    for (size_t i = 0; i < 2; ++i)
      for (size_t j = 0; j < 3; ++j)
        for (size_t r = 0; r < 2; ++r)
          for (size_t c = 0; c < 2; ++c) CHECK(o.get_f32({i, j, r, c}).unwrap() == exp[i][j][r * 2 + c]);
  }
  CHECK(h.be->batched_matmul(h.make(std::vector<float>(24, 1.0f), Shape{2, 4, 3}), h.make(std::vector<float>(45, 1.0f), Shape{3, 3, 5}))
            .unwrap_err().kind == Error::Kind::BroadcastIncompatible);
}

int main(int argc, char **argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  if (mode == "cpu") {
    a1_shape_and_strides();
    a2_broadcasting();
    a3_strided_views();
    a5_error_taxonomy();
    runtime_dispatch();
    CpuBackend cpu;
    Harness h{&cpu, [](const std::vector<float> &d, Shape s) { return t(d, std::move(s)); }, [](const Tensor &x) { return x; }};
    a4_reference_matmul(h);
    // a device with no GPU behind it: a typed error, never a crash
    auto none = B200Backend::create(63);
    CHECK(none.is_err() && none.unwrap_err().kind == Error::Kind::BackendUnavailable);
  } else {
    auto made = B200Backend::create(0);
    if (made.is_err()) {
      std::printf("FAIL no B200 backend: %s\n", made.unwrap_err().to_string().c_str());
      return 2;
    }
    std::shared_ptr<B200Backend> gpu = made.unwrap();
    register_backend(gpu);
    CHECK(std::string(gpu->name()) == "b200-tcgen05" && gpu->device() == Device::cuda(0));
    Harness h{gpu.get(),
              [&](const std::vector<float> &d, Shape s) { return gpu->from_vec_f32(d, std::move(s)).unwrap(); },
              [&](const Tensor &x) { return gpu->to_host(x).unwrap(); }};
    for (int kernel = 0; kernel <= 2; ++kernel) {  // auto, FFMA, tensor cores
      oxm_set_option(gpu->raw(), "kernel", kernel);
      a4_reference_matmul(h);
    }
    oxm_set_option(gpu->raw(), "kernel", 0);
    // TensorOps dispatch on a device tensor; operands on different devices refuse
    Tensor a = gpu->from_vec_f32({1, 2, 3, 4}, Shape{2, 2}).unwrap(), b = gpu->from_vec_f32({5, 6, 7, 8}, Shape{2, 2}).unwrap();
    CHECK(gpu->to_host(a.matmul(b).unwrap()).unwrap().get_f32({0, 1}).unwrap() == 22.0f);
    CHECK(gpu->matmul(a, t({5, 6, 7, 8}, Shape{2, 2})).unwrap_err().kind == Error::Kind::DeviceMismatch);
    // the other op families of the Backend trait (ops/lib.rs:27-69), through the tensor surface
    Tensor row = gpu->from_vec_f32({10, 20}, Shape{2}).unwrap();
    expect_tensor(h, a.add(row), {11, 22, 13, 24}, Shape{2, 2});            // NumPy broadcast of a row
    expect_tensor(h, a.sub(b), {-4, -4, -4, -4}, Shape{2, 2});
    expect_tensor(h, a.mul(b.permute({1, 0}).unwrap()), {5, 14, 18, 32}, Shape{2, 2});  // a transposed view
    expect_tensor(h, b.div(a), {5, 3, 7.0f / 3.0f, 2}, Shape{2, 2});
    expect_tensor(h, a.neg(), {-1, -2, -3, -4}, Shape{2, 2});
    expect_tensor(h, gpu->abs(a.neg().unwrap()), {1, 2, 3, 4}, Shape{2, 2});
    expect_tensor(h, a.sum({}), {10}, Shape{});
    expect_tensor(h, a.sum({0}), {4, 6}, Shape{2});
    expect_tensor(h, gpu->max(a, {1}), {2, 4}, Shape{2});
    CHECK(a.sum({2}).unwrap_err().kind == Error::Kind::IndexOutOfBounds);
    CHECK(a.add(gpu->from_vec_f32({1, 2, 3}, Shape{3}).unwrap()).unwrap_err().kind == Error::Kind::BroadcastIncompatible);
    // fused linear-layer forms: relu(a.b + bias), then an accumulation on top of it
    Tensor bias = gpu->from_vec_f32({-30, 0}, Shape{2}).unwrap();
    auto fused = gpu->matmul_fused(a, b, &bias, OXM_ACT_RELU);
    expect_tensor(h, fused, {0, 22, 13, 50}, Shape{2, 2});
    Tensor acc = fused.unwrap();
    expect_tensor(h, gpu->matmul_fused(a, b, nullptr, OXM_ACT_NONE, &acc), {19, 44, 56, 100}, Shape{2, 2});
    // the block-scaled fp8 product: ones (e4m3 0x38) times ones over K = 64, row 1 of A scaled by 2
    // in its second block, column 2 of B by 1/2 in its first; B is the transposed view of an [N, K] tensor
    {
      const size_t M = 2, N = 3, K = 64;
      std::vector<uint8_t> ones_a(M * K, 0x38), ones_b(N * K, 0x38), sa = {127, 127, 127, 128}, sbt = {127, 127, 127, 127, 126, 127};
      Tensor ma = gpu->from_host(ones_a.data(), Shape{M, K}, DType::F8E4M3).unwrap();
      Tensor mbt = gpu->from_host(ones_b.data(), Shape{N, K}, DType::F8E4M3).unwrap();
      Tensor msa = gpu->from_host(sa.data(), Shape{M, K / 32}, DType::U8).unwrap();
      Tensor msbt = gpu->from_host(sbt.data(), Shape{N, K / 32}, DType::U8).unwrap();
      auto prod = gpu->matmul_mx(ma, msa, mbt.permute({1, 0}).unwrap(), msbt.permute({1, 0}).unwrap(), DType::F32);
      expect_tensor(h, prod, {64, 64, 48, 96, 96, 80}, Shape{M, N});
      CHECK(gpu->matmul_mx(a, msa, b, msbt, DType::F32).unwrap_err().kind == Error::Kind::UnsupportedDType);
    }
    unregister_all();
  }
  std::printf("%s: %d checks, %d failed\n", mode.c_str(), g_checks, g_failed);
  return g_failed ? 1 : 0;
}
