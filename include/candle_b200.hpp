/*
 * C++ host mirror of candle's operator interface for the norm + embedding path, over the C ABI of
 * candle_b200.h.  candle's own host side is Rust (candle-nn/src/ops.rs, embedding.rs, layer_norm.rs,
 * candle-core/src/tensor.rs); this header gives a C++ caller the same entry points with the same
 * names, argument meaning, checks and error strings:
 *
 *   ops::rms_norm(xs, alpha, eps)            candle_nn::ops::rms_norm        ops.rs:641-652, 536-543
 *   ops::layer_norm(xs, alpha, beta, eps)    candle_nn::ops::layer_norm      ops.rs:896-909, 770-781
 *   ops::rms_norm_slow / layer_norm_slow     candle_nn::ops::*_slow          ops.rs:628-639, 876-894
 *   LayerNorm / RmsNorm {..}.forward(xs)     candle_nn::{LayerNorm,RmsNorm}  layer_norm.rs:63-194
 *   index_select(t, ids, dim)                Tensor::index_select            tensor.rs:1568-1589
 *   Embedding{table, hidden}.forward(ids)    candle_nn::Embedding::forward   embedding.rs:28-37
 *   QTensor::embedding / embedding_rms_norm  (new: lookups out of GGML blocks)
 *
 * A Tensor here is a non-owning view of caller-allocated device memory (pointer, dims, dtype) --
 * the library never allocates -- and every function takes the destination view and a stream.
 * Header-only, C++17, needs no CUDA headers: a stream is passed as the opaque pointer the C ABI takes.
 * Failures throw candle_b200::Error with candle's message; a bad id is reported through the caller's
 * device status record, to be read after the stream is synchronised (status_error turns a record
 * copied to the host into the InvalidIndex message of candle's CPU backend).
 */
#ifndef CANDLE_B200_HPP_
#define CANDLE_B200_HPP_

#include <cstdint>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "candle_b200.h"

namespace candle_b200 {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

enum class DType { F32 = CB200_DTYPE_F32, F16 = CB200_DTYPE_F16, BF16 = CB200_DTYPE_BF16, U8 = 100, U32 = 101, I64 = 102 };

inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "F32";
    case DType::F16: return "F16";
    case DType::BF16: return "BF16";
    case DType::U8: return "U8";
    case DType::U32: return "U32";
    default: return "I64";
  }
}
inline int elem_size(DType d) {
  switch (d) {
    case DType::F32: case DType::U32: return 4;
    case DType::F16: case DType::BF16: return 2;
    case DType::U8: return 1;
    default: return 8;
  }
}
inline bool is_float(DType d) { return d == DType::F32 || d == DType::F16 || d == DType::BF16; }

using Shape = std::vector<int64_t>;
inline std::string dims_string(const Shape& s) {
  std::ostringstream o;
  o << "[";
  for (size_t i = 0; i < s.size(); ++i) o << (i ? ", " : "") << s[i];
  o << "]";
  return o.str();
}
inline int64_t elem_count(const Shape& s) {
  return std::accumulate(s.begin(), s.end(), int64_t{1}, [](int64_t a, int64_t b) { return a * b; });
}

/* Non-owning view of a device tensor.  `contiguous` is what Layout::is_contiguous would say. */
struct Tensor {
  void* data = nullptr;
  Shape dims;
  DType dtype = DType::F32;
  bool contiguous = true;
  int64_t elem_count() const { return candle_b200::elem_count(dims); }
  size_t rank() const { return dims.size(); }
};

namespace detail {
inline void check_rc(int rc) {
  if (rc != CB200_OK) throw Error(cb200_last_error());
}
inline int id_code(DType d) {
  switch (d) {
    case DType::U8: return CB200_ID_U8;
    case DType::U32: return CB200_ID_U32;
    case DType::I64: return CB200_ID_I64;
    default: throw Error(std::string("unsupported dtype ") + dtype_name(d) + " for index-select ids (expected U8, U32 or I64)");
  }
}
inline void check_out(const Tensor& out, const Shape& want, DType dtype, const char* op) {
  if (out.data == nullptr || out.dims != want || out.dtype != dtype || !out.contiguous)
    throw Error(std::string(op) + ": the destination must be a contiguous " + dtype_name(dtype) + " tensor of shape " +
                dims_string(want) + ", got " + dims_string(out.dims));
}
inline void norm_checks(const Tensor& xs, const Tensor* params[], const char* names[], int n_params,
                        const Tensor* residual) {
  if (!is_float(xs.dtype)) throw Error(std::string("unsupported dtype for rmsnorm ") + dtype_name(xs.dtype));
  for (int i = 0; i < n_params; ++i)
    if (params[i]->dtype != xs.dtype) throw Error(std::string("unsupported dtype for rmsnorm ") + dtype_name(xs.dtype));
  if (!xs.contiguous) throw Error("input has to be contiguous");  // ops.rs:537
  for (int i = 0; i < n_params; ++i)
    if (!params[i]->contiguous) throw Error(std::string(names[i]) + " has to be contiguous");  // ops.rs:541
  if (residual != nullptr) {
    if (residual->dims != xs.dims || residual->dtype != xs.dtype)
      throw Error("shape mismatch in binary op add, lhs: " + dims_string(xs.dims) + ", rhs: " + dims_string(residual->dims));
    if (!residual->contiguous) throw Error("input has to be contiguous");
  }
}
}  // namespace detail

namespace ops {

/* candle_nn::ops::rms_norm(xs, alpha, eps); with `residual` the norm of xs + residual (the sum itself
 * goes to `sum_out` when given).  The result is written to `out`. */
inline void rms_norm(const Tensor& xs, const Tensor& alpha, float eps, Tensor& out, cb200_stream_t stream,
                     const Tensor* residual = nullptr, Tensor* sum_out = nullptr, int flags = 0) {
  if (xs.rank() == 0) throw Error("unexpected rank, expected: at least 1, got: 0");
  if (alpha.rank() != 1)
    throw Error("unexpected rank, expected: 1, got: " + std::to_string(alpha.rank()) + " (" + dims_string(alpha.dims) + ")");
  if (xs.dims.back() != alpha.dims[0])
    throw Error("shape mismatch in rms-norm " + dims_string(xs.dims) + " " + dims_string(alpha.dims));  // ops.rs:645-649
  const Tensor* params[] = {&alpha};
  const char* names[] = {"alpha"};
  detail::norm_checks(xs, params, names, 1, residual);
  detail::check_out(out, xs.dims, xs.dtype, "rms-norm");
  if (sum_out != nullptr) detail::check_out(*sum_out, xs.dims, xs.dtype, "rms-norm");
  const int64_t cols = xs.dims.back();
  const int64_t rows = cols ? xs.elem_count() / cols : 0;
  detail::check_rc(cb200_rms_norm(xs.data, residual ? residual->data : nullptr, alpha.data, out.data,
                                  sum_out ? sum_out->data : nullptr, rows, static_cast<int32_t>(cols), eps,
                                  static_cast<int>(xs.dtype), flags, stream));
}

/* candle_nn::ops::layer_norm(xs, alpha, beta, eps), optional residual as above. */
inline void layer_norm(const Tensor& xs, const Tensor& alpha, const Tensor& beta, float eps, Tensor& out,
                       cb200_stream_t stream, const Tensor* residual = nullptr, Tensor* sum_out = nullptr,
                       int flags = 0) {
  if (xs.rank() == 0) throw Error("unexpected rank, expected: at least 1, got: 0");
  if (alpha.rank() != 1 || beta.rank() != 1) {
    const Tensor& bad = alpha.rank() != 1 ? alpha : beta;
    throw Error("unexpected rank, expected: 1, got: " + std::to_string(bad.rank()) + " (" + dims_string(bad.dims) + ")");
  }
  if (xs.dims.back() != alpha.dims[0] || xs.dims.back() != beta.dims[0])
    throw Error("shape mismatch in layer-norm src: " + dims_string(xs.dims) + " alpha: " + dims_string(alpha.dims) +
                " beta: " + dims_string(beta.dims));  // ops.rs:901-906
  const Tensor* params[] = {&alpha, &beta};
  const char* names[] = {"alpha", "beta"};
  detail::norm_checks(xs, params, names, 2, residual);
  detail::check_out(out, xs.dims, xs.dtype, "layer-norm");
  if (sum_out != nullptr) detail::check_out(*sum_out, xs.dims, xs.dtype, "layer-norm");
  const int64_t cols = xs.dims.back();
  const int64_t rows = cols ? xs.elem_count() / cols : 0;
  detail::check_rc(cb200_layer_norm(xs.data, residual ? residual->data : nullptr, alpha.data, beta.data, out.data,
                                    sum_out ? sum_out->data : nullptr, rows, static_cast<int32_t>(cols), eps,
                                    static_cast<int>(xs.dtype), flags, stream));
}

/* the composite norm behind rms_norm_slow, layer_norm_slow and the modules' slow branch */
inline void norm_slow_chain(const Tensor& xs, const Tensor& weight, const Tensor* bias, float eps, bool remove_mean,
                      Tensor& out, cb200_stream_t stream) {
  if (xs.rank() == 0) throw Error("unexpected rank, expected: at least 1, got: 0");
  if (!is_float(xs.dtype)) throw Error(std::string("unsupported dtype for rmsnorm ") + dtype_name(xs.dtype));
  /* candle's chain starts with to_dtype, which copies a strided input; a view here has no strides,
   * so the caller makes that copy */
  if (!xs.contiguous) throw Error("input has to be contiguous");
  const int64_t cols = xs.dims.back();
  const Tensor* params[] = {&weight, bias};
  for (const Tensor* p : params) {
    if (p == nullptr) continue;
    if (p->dtype != xs.dtype)
      throw Error(std::string("dtype mismatch in mul, lhs: ") + dtype_name(xs.dtype) + ", rhs: " + dtype_name(p->dtype));
    if (p->rank() != 1 || p->dims[0] != cols || !p->contiguous)
      throw Error("shape mismatch in broadcast_mul, lhs: " + dims_string(xs.dims) + ", rhs: " + dims_string(p->dims));
  }
  detail::check_out(out, xs.dims, xs.dtype, "layer-norm");
  const int64_t rows = cols ? xs.elem_count() / cols : 0;
  detail::check_rc(cb200_layer_norm_slow(xs.data, weight.data, bias ? bias->data : nullptr, out.data, rows,
                                         static_cast<int32_t>(cols), eps, static_cast<int>(xs.dtype),
                                         remove_mean ? 1 : 0, stream));
}

/* candle_nn::ops::rms_norm_slow (ops.rs:628-639): f32 inside, one rounding, weight applied in T. */
inline void rms_norm_slow(const Tensor& xs, const Tensor& alpha, float eps, Tensor& out, cb200_stream_t stream) {
  norm_slow_chain(xs, alpha, nullptr, eps, false, out, stream);
}
/* candle_nn::ops::layer_norm_slow (ops.rs:876-894). */
inline void layer_norm_slow(const Tensor& xs, const Tensor& alpha, const Tensor& beta, float eps, Tensor& out,
                            cb200_stream_t stream) {
  norm_slow_chain(xs, alpha, &beta, eps, true, out, stream);
}

}  // namespace ops

/* candle_nn::LayerNorm (layer_norm.rs:63-136): the fused op iff the input is contiguous, the mean is
 * removed and there is a bias; the composite chain otherwise. */
class LayerNorm {
 public:
  static LayerNorm create(Tensor weight, Tensor bias, double eps) { return LayerNorm(std::move(weight), std::move(bias), true, true, eps); }
  static LayerNorm new_no_bias(Tensor weight, double eps) { return LayerNorm(std::move(weight), Tensor{}, false, true, eps); }
  static LayerNorm rms_norm(Tensor weight, double eps) { return LayerNorm(std::move(weight), Tensor{}, false, false, eps); }
  const Tensor& weight() const { return weight_; }
  const Tensor* bias() const { return has_bias_ ? &bias_ : nullptr; }
  double eps() const { return eps_; }
  void forward(const Tensor& x, Tensor& out, cb200_stream_t stream) const {
    if (x.contiguous && remove_mean_ && has_bias_) {
      ops::layer_norm(x, weight_, bias_, static_cast<float>(eps_), out, stream);
      return;
    }
    ops::norm_slow_chain(x, weight_, bias(), static_cast<float>(eps_), remove_mean_, out, stream);
  }

 private:
  LayerNorm(Tensor w, Tensor b, bool has_bias, bool remove_mean, double eps)
      : weight_(std::move(w)), bias_(std::move(b)), has_bias_(has_bias), remove_mean_(remove_mean), eps_(eps) {}
  Tensor weight_, bias_;
  bool has_bias_, remove_mean_;
  double eps_;
};

/* candle_nn::RmsNorm (layer_norm.rs:167-194): the fused op on contiguous input, else the inner
 * LayerNorm's composite chain; forward_diff always takes the latter. */
class RmsNorm {
 public:
  RmsNorm(Tensor weight, double eps) : inner_(LayerNorm::rms_norm(std::move(weight), eps)) {}
  const LayerNorm& into_inner() const { return inner_; }
  void forward_diff(const Tensor& xs, Tensor& out, cb200_stream_t stream) const { inner_.forward(xs, out, stream); }
  void forward(const Tensor& xs, Tensor& out, cb200_stream_t stream) const {
    if (xs.contiguous)
      ops::rms_norm(xs, inner_.weight(), static_cast<float>(inner_.eps()), out, stream);
    else
      inner_.forward(xs, out, stream);
  }

 private:
  LayerNorm inner_;
};

/* Shape of t.index_select(ids, dim); throws what Tensor::index_select would for bad arguments. */
inline Shape index_select_shape(const Tensor& t, const Tensor& ids, int64_t dim) {
  if (!t.contiguous) throw Error("index-select requires contiguous tensors");
  if (ids.rank() != 1)
    throw Error("unexpected number of dims: expected 1, got " + std::to_string(ids.rank()) + ", shape " + dims_string(ids.dims));
  detail::id_code(ids.dtype);
  const int64_t d = dim >= 0 ? dim : dim + static_cast<int64_t>(t.rank());
  if (d < 0 || d >= static_cast<int64_t>(t.rank()))
    throw Error("dim out of range in index-select: " + std::to_string(dim) + " for shape " + dims_string(t.dims));
  Shape s = t.dims;
  s[d] = ids.dims[0];
  return s;
}

/* Tensor::index_select(ids, dim) into `out`; ids beyond the dimension are recorded in `status`. */
inline void index_select(const Tensor& t, const Tensor& ids, int64_t dim, Tensor& out, cb200_status* status,
                         cb200_stream_t stream) {
  const Shape want = index_select_shape(t, ids, dim);
  if (!ids.contiguous) throw Error("index-select ids must be contiguous on the device");
  detail::check_out(out, want, t.dtype, "index-select");
  const int64_t d = dim >= 0 ? dim : dim + static_cast<int64_t>(t.rank());
  int64_t left = 1, right = 1;
  for (int64_t i = 0; i < d; ++i) left *= t.dims[i];
  for (size_t i = d + 1; i < t.rank(); ++i) right *= t.dims[i];
  detail::check_rc(cb200_index_select(t.data, ids.data, out.data, left, t.dims[d], right, ids.dims[0],
                                      elem_size(t.dtype), detail::id_code(ids.dtype), status, stream));
}

/* The message candle's CPU backend raises for a record that was copied back to the host
 * (cpu_backend/mod.rs:539-546, worded as candle-core/src/error.rs:129), or an empty string when the
 * record is clean. */
inline std::string status_error(const cb200_status& st, const char* op = "index-select") {
  if (st.code == 1)
    return std::string(op) + " invalid index " + std::to_string(st.index) + " with dim size " + std::to_string(st.size);
  if (st.code == 2) return std::string("device-side wait timed out at row ") + std::to_string(st.position) + " in " + op;
  return "";
}

/* candle_nn::Embedding (embedding.rs:11-37). */
class Embedding {
 public:
  Embedding(Tensor embeddings, int64_t hidden_size) : embeddings_(std::move(embeddings)), hidden_size_(hidden_size) {}
  const Tensor& embeddings() const { return embeddings_; }
  int64_t hidden_size() const { return hidden_size_; }
  /* dims of forward(indexes): indexes.dims ++ [hidden_size] */
  Shape forward_shape(const Tensor& indexes) const {
    Shape s = indexes.dims;
    s.push_back(hidden_size_);
    return s;
  }
  void forward(const Tensor& indexes, Tensor& out, cb200_status* status, cb200_stream_t stream) const {
    if (embeddings_.rank() != 2)
      throw Error("unexpected rank, expected: 2, got: " + std::to_string(embeddings_.rank()) + " (" + dims_string(embeddings_.dims) + ")");
    if (!indexes.contiguous) throw Error("index-select ids must be contiguous on the device");
    detail::check_out(out, forward_shape(indexes), embeddings_.dtype, "embedding");
    Tensor flat = indexes;  // flatten_all
    flat.dims = {indexes.elem_count()};
    Tensor out2 = out;
    out2.dims = {flat.dims[0], embeddings_.dims[1]};
    index_select(embeddings_, flat, 0, out2, status, stream);
  }

 private:
  Tensor embeddings_;
  int64_t hidden_size_;
};

/* Raw GGML blocks + logical shape on the device (candle-core/src/quantized/mod.rs:35-38). */
struct QTensor {
  const void* data = nullptr;
  int ggml_dtype = CB200_QTYPE_Q8_0;  // ggml type id
  Shape dims;

  /* rows `ids` of a [vocab, hidden] table, decoded to out.dtype */
  void embedding(const Tensor& ids, Tensor& out, cb200_status* status, cb200_stream_t stream,
                 int64_t vocab_begin = 0, int64_t vocab_end = -1, int64_t vocab = -1) const {
    const auto [total, begin, end] = range(vocab_begin, vocab_end, vocab);
    Shape want = ids.dims;
    want.push_back(dims[1]);
    detail::check_out(out, want, out.dtype, "qembedding");
    detail::check_rc(cb200_qembedding(data, ggml_dtype, ids.data, out.data, total, static_cast<int32_t>(dims[1]),
                                      ids.elem_count(), static_cast<int>(out.dtype), detail::id_code(ids.dtype), begin,
                                      end, status, stream));
  }
  /* the same followed by rms_norm(., alpha, eps), one launch where the fused kernel applies */
  void embedding_rms_norm(const Tensor& ids, const Tensor& alpha, float eps, Tensor& out, cb200_status* status,
                          cb200_stream_t stream, Tensor* gathered = nullptr, int64_t vocab_begin = 0,
                          int64_t vocab_end = -1, int64_t vocab = -1, int flags = 0) const {
    const auto [total, begin, end] = range(vocab_begin, vocab_end, vocab);
    Shape want = ids.dims;
    want.push_back(dims[1]);
    if (alpha.rank() != 1 || alpha.dims[0] != dims[1] || !alpha.contiguous)
      throw Error("shape mismatch in rms-norm " + dims_string(want) + " " + dims_string(alpha.dims));
    detail::check_out(out, want, alpha.dtype, "qembedding-rms-norm");
    if (gathered != nullptr) detail::check_out(*gathered, want, alpha.dtype, "qembedding-rms-norm");
    detail::check_rc(cb200_qembedding_rms_norm(data, ggml_dtype, ids.data, alpha.data, out.data,
                                               gathered ? gathered->data : nullptr, total,
                                               static_cast<int32_t>(dims[1]), ids.elem_count(), eps,
                                               static_cast<int>(alpha.dtype), detail::id_code(ids.dtype), begin, end,
                                               flags, status, stream));
  }

 private:
  struct Range {
    int64_t total, begin, end;
  };
  Range range(int64_t vocab_begin, int64_t vocab_end, int64_t vocab) const {
    if (dims.size() != 2) throw Error("qembedding expects a rank-2 QTensor");
    const int64_t end = vocab_end < 0 ? vocab_begin + dims[0] : vocab_end;
    if (end - vocab_begin != dims[0])
      throw Error("vocab shard [" + std::to_string(vocab_begin) + ", " + std::to_string(end) + ") does not match the table's " +
                  std::to_string(dims[0]) + " rows");
    return {vocab < 0 ? end : vocab, vocab_begin, end};
  }
};

}  // namespace candle_b200

#endif /* CANDLE_B200_HPP_ */
