// The C++ mirror on a GPU: reads raw inputs written by the test, runs rms_norm (+ residual) and
// Embedding::forward through candle_b200.hpp, writes the raw outputs back.  Usage:
//   host_mirror_gpu <dir> <rows> <cols> <vocab> <n_ids>
// Files in <dir>: x.bf16 res.bf16 alpha.bf16 table.f32 ids.u32  ->  y.bf16 h.bf16 emb.f32 status.bin
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "candle_b200.hpp"

using namespace candle_b200;

static std::vector<char> slurp(const std::string& p) {
  FILE* f = std::fopen(p.c_str(), "rb");
  if (!f) { std::perror(p.c_str()); std::exit(2); }
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> b(n);
  if (std::fread(b.data(), 1, n, f) != static_cast<size_t>(n)) std::exit(2);
  std::fclose(f);
  return b;
}
static void dump(const std::string& p, const void* d, size_t n) {
  FILE* f = std::fopen(p.c_str(), "wb");
  if (!f || std::fwrite(d, 1, n, f) != n) std::exit(2);
  std::fclose(f);
}
static void* to_device(const std::vector<char>& b) {
  void* d = nullptr;
  if (cudaMalloc(&d, b.size() ? b.size() : 16) != cudaSuccess) std::exit(3);
  cudaMemcpy(d, b.data(), b.size(), cudaMemcpyHostToDevice);
  return d;
}
static void from_device(const std::string& p, const void* d, size_t n) {
  std::vector<char> b(n);
  cudaMemcpy(b.data(), d, n, cudaMemcpyDeviceToHost);
  dump(p, b.data(), n);
}

int main(int argc, char** argv) {
  if (argc != 6) return 2;
  const std::string dir = argv[1];
  const int64_t rows = std::atoll(argv[2]), cols = std::atoll(argv[3]), vocab = std::atoll(argv[4]), n_ids = std::atoll(argv[5]);
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  try {
    Tensor x{to_device(slurp(dir + "/x.bf16")), {rows, cols}, DType::BF16, true};
    Tensor r{to_device(slurp(dir + "/res.bf16")), {rows, cols}, DType::BF16, true};
    Tensor a{to_device(slurp(dir + "/alpha.bf16")), {cols}, DType::BF16, true};
    Tensor y{nullptr, {rows, cols}, DType::BF16, true}, h{nullptr, {rows, cols}, DType::BF16, true};
    cudaMalloc(&y.data, rows * cols * 2);
    cudaMalloc(&h.data, rows * cols * 2);
    ops::rms_norm(x, a, 1e-5f, y, stream, &r, &h);

    Embedding emb(Tensor{to_device(slurp(dir + "/table.f32")), {vocab, cols}, DType::F32, true}, cols);
    Tensor ids{to_device(slurp(dir + "/ids.u32")), {2, n_ids / 2}, DType::U32, true};
    Tensor e{nullptr, emb.forward_shape(ids), DType::F32, true};
    cudaMalloc(&e.data, n_ids * cols * 4);
    cudaMemset(e.data, 0, n_ids * cols * 4);
    cb200_status* st = nullptr;
    cudaMalloc(&st, sizeof(cb200_status));
    cudaMemset(st, 0, sizeof(cb200_status));
    emb.forward(ids, e, st, stream);
    if (cudaStreamSynchronize(stream) != cudaSuccess) return 4;
    from_device(dir + "/y.bf16", y.data, rows * cols * 2);
    from_device(dir + "/h.bf16", h.data, rows * cols * 2);
    from_device(dir + "/emb.f32", e.data, n_ids * cols * 4);
    cb200_status host_st;
    cudaMemcpy(&host_st, st, sizeof(host_st), cudaMemcpyDeviceToHost);
    dump(dir + "/status.bin", &host_st, sizeof(host_st));
    std::printf("%s\n", status_error(host_st).c_str());
  } catch (const Error& e) {
    std::printf("error: %s\n", e.what());
    return 1;
  }
  return 0;
}
