// Host-side checks of the C++ mirror: every case here must be decided before any device work, so
// the program runs without a GPU.  Prints one "ok <name>" line per case and exits 0, or the first
// mismatch and exits 1.
#include <cstdio>
#include <cstring>
#include <string>

#include "candle_b200.hpp"

using namespace candle_b200;

static int failures = 0;
template <typename F>
static void expect_error(const char* name, const std::string& want_substr, F&& f) {
  try {
    f();
    std::printf("FAIL %s: no error\n", name);
    ++failures;
  } catch (const Error& e) {
    if (std::string(e.what()).find(want_substr) == std::string::npos) {
      std::printf("FAIL %s: got '%s', want '%s'\n", name, e.what(), want_substr.c_str());
      ++failures;
    } else {
      std::printf("ok %s\n", name);
    }
  }
}

int main() {
  void* fake = reinterpret_cast<void*>(0x1000);  // 16-byte aligned, never dereferenced on the host
  Tensor x{fake, {4, 8}, DType::F32, true}, a{fake, {8}, DType::F32, true}, y{fake, {4, 8}, DType::F32, true};
  Tensor a7{fake, {7}, DType::F32, true}, a2d{fake, {1, 8}, DType::F32, true}, ah{fake, {8}, DType::F16, true};
  Tensor xs{fake, {4, 8}, DType::F32, false}, xi{fake, {4, 8}, DType::U32, true};
  expect_error("rms_norm shape", "shape mismatch in rms-norm [4, 8] [7]", [&] { ops::rms_norm(x, a7, 1e-5f, y, nullptr); });
  expect_error("rms_norm alpha rank", "unexpected rank, expected: 1, got: 2 ([1, 8])", [&] { ops::rms_norm(x, a2d, 1e-5f, y, nullptr); });
  expect_error("rms_norm dtype mix", "unsupported dtype for rmsnorm F32", [&] { ops::rms_norm(x, ah, 1e-5f, y, nullptr); });
  expect_error("rms_norm int dtype", "unsupported dtype for rmsnorm U32", [&] { ops::rms_norm(xi, a, 1e-5f, y, nullptr); });
  expect_error("rms_norm contiguous", "input has to be contiguous", [&] { ops::rms_norm(xs, a, 1e-5f, y, nullptr); });
  Tensor r3{fake, {4, 3}, DType::F32, true};
  expect_error("rms_norm residual shape", "shape mismatch in binary op add, lhs: [4, 8], rhs: [4, 3]",
               [&] { ops::rms_norm(x, a, 1e-5f, y, nullptr, &r3); });
  expect_error("layer_norm shape", "shape mismatch in layer-norm src: [4, 8] alpha: [8] beta: [7]",
               [&] { ops::layer_norm(x, a, a7, 1e-5f, y, nullptr); });
  Tensor anc{fake, {8}, DType::F32, false};
  expect_error("layer_norm beta contiguous", "beta has to be contiguous", [&] { ops::layer_norm(x, a, anc, 1e-5f, y, nullptr); });
  Tensor t{fake, {10, 4}, DType::F32, true}, ids{fake, {3}, DType::I64, true}, ids2{fake, {2, 2}, DType::I64, true};
  Tensor idf{fake, {3}, DType::F32, true}, out{fake, {3, 4}, DType::F32, true}, tnc{fake, {10, 4}, DType::F32, false};
  expect_error("index_select ids rank", "unexpected number of dims: expected 1, got 2, shape [2, 2]",
               [&] { index_select(t, ids2, 0, out, nullptr, nullptr); });
  expect_error("index_select ids dtype", "for index-select ids (expected U8, U32 or I64)",
               [&] { index_select(t, idf, 0, out, nullptr, nullptr); });
  expect_error("index_select contiguous", "index-select requires contiguous tensors",
               [&] { index_select(tnc, ids, 0, out, nullptr, nullptr); });
  expect_error("index_select dim", "dim out of range in index-select: 2 for shape [10, 4]",
               [&] { index_select(t, ids, 2, out, nullptr, nullptr); });
  if (index_select_shape(t, ids, 1) != Shape{10, 3} || index_select_shape(t, ids, -2) != Shape{3, 4}) {
    std::printf("FAIL index_select_shape\n");
    ++failures;
  } else {
    std::printf("ok index_select_shape\n");
  }
  Embedding emb(t, 4);
  Tensor idm{fake, {2, 3}, DType::U32, true};
  if (emb.forward_shape(idm) != Shape{2, 3, 4} || emb.hidden_size() != 4) {
    std::printf("FAIL embedding shape\n");
    ++failures;
  } else {
    std::printf("ok embedding shape\n");
  }
  Tensor bad_out{fake, {2, 3, 5}, DType::F32, true};
  expect_error("embedding out shape", "the destination must be a contiguous F32 tensor of shape [2, 3, 4]",
               [&] { emb.forward(idm, bad_out, nullptr, nullptr); });
  QTensor q{fake, CB200_QTYPE_Q8_0, {100, 64}};
  Tensor qo{fake, {3, 64}, DType::BF16, true};
  expect_error("qembedding shard", "vocab shard [10, 60) does not match the table's 100 rows",
               [&] { q.embedding(ids, qo, nullptr, nullptr, 10, 60, 200); });
  QTensor q33{fake, CB200_QTYPE_Q8_0, {100, 33}};
  Tensor qo33{fake, {3, 33}, DType::BF16, true};
  expect_error("qembedding hidden", "not divisible by 32", [&] { q33.embedding(ids, qo33, nullptr, nullptr); });  // from the C ABI
  // zero rows: nothing to launch, accepted without a device
  Tensor x0{fake, {0, 8}, DType::F32, true}, y0{fake, {0, 8}, DType::F32, true};
  ops::rms_norm(x0, a, 1e-5f, y0, nullptr);
  std::printf("ok zero rows\n");
  // modules: candle's dispatch (layer_norm.rs:108-136, 186-194) decided on the host
  LayerNorm ln = LayerNorm::create(a, a, 1e-5), ln_nb = LayerNorm::new_no_bias(a, 1e-5);
  RmsNorm rn(a, 1e-5);
  ln.forward(x0, y0, nullptr);      // fused op, zero rows: nothing launched
  ln_nb.forward(x0, y0, nullptr);   // composite chain, zero rows
  rn.forward(x0, y0, nullptr);
  rn.forward_diff(x0, y0, nullptr);
  std::printf("ok module zero rows\n");
  expect_error("LayerNorm fused weight shape", "shape mismatch in layer-norm src: [4, 8] alpha: [7] beta: [7]",
               [&] { LayerNorm::create(a7, a7, 1e-5).forward(x, y, nullptr); });
  expect_error("LayerNorm slow weight shape", "shape mismatch in broadcast_mul, lhs: [4, 8], rhs: [7]",
               [&] { LayerNorm::new_no_bias(a7, 1e-5).forward(x, y, nullptr); });
  expect_error("LayerNorm slow weight dtype", "dtype mismatch in mul, lhs: F32, rhs: F16",
               [&] { LayerNorm::rms_norm(ah, 1e-5).forward(x, y, nullptr); });
  expect_error("RmsNorm strided input", "input has to be contiguous", [&] { rn.forward(xs, y, nullptr); });
  if (ln.bias() == nullptr || ln_nb.bias() != nullptr || rn.into_inner().bias() != nullptr) {
    std::printf("FAIL module accessors\n");
    ++failures;
  } else {
    std::printf("ok module accessors\n");
  }
  cb200_status st{};
  st.code = 1;
  st.index = 12;
  st.size = 10;
  if (status_error(st) != "index-select invalid index 12 with dim size 10" || !status_error(cb200_status{}).empty()) {
    std::printf("FAIL status_error\n");
    ++failures;
  } else {
    std::printf("ok status_error\n");
  }
  return failures ? 1 : 0;
}
