// Row gathers: index_select / Embedding::forward on dense tables and row lookups out of
// Q4_0 / Q8_0 tables with on-the-fly decode.
//
// Dense rows are moved by the bulk-copy engine only: global -> shared -> global, no registers
// involved.  A CTA is one warp whose lane 0 keeps a ring of row buffers in flight; all other
// resources of the SM stay free, and a few CTAs per SM are enough to cover HBM latency because
// each holds tens of KB in flight.  Short or unaligned rows take a plain vector-copy kernel.
#include "launch.h"
#include "qblocks.cuh"

namespace cb200 {

// ---------------------------------------------------------------------------------------------
// Dense gather through shared memory with bulk copies
// ---------------------------------------------------------------------------------------------
constexpr int kGatherStages = 4;
constexpr int kGatherChunk = 16 * 1024;  // bytes per ring slot

__global__ void __launch_bounds__(32) gather_rows_bulk_kernel(const GatherArgs a, int chunks_per_row) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);  // [kGatherStages]
  unsigned char* ring = smem_raw + 128;
  if (threadIdx.x != 0) return;  // one issuing thread; the copy engine does the work

  for (int s = 0; s < kGatherStages; ++s) mbar_init(&bars[s], 1);
  mbar_init_fence();

  const int64_t rows = a.left * a.n_ids;
  const int64_t n_items = rows * chunks_per_row;
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t n_my = first < n_items ? (n_items - first + step - 1) / step : 0;

  uint32_t size[kGatherStages];      // bytes loaded into the slot (0: skipped item)
  unsigned char* dst[kGatherStages]; // where the slot goes
  uint32_t phase = 0;                // one parity bit per slot
  uint32_t pending = 0;              // slots with a load in flight

  auto issue_load = [&](int64_t j) {
    const int s = static_cast<int>(j % kGatherStages);
    const int64_t item = first + j * step;
    const int64_t row = item / chunks_per_row;
    const int64_t c = item - row * chunks_per_row;
    const int64_t l = row / a.n_ids, i = row - l * a.n_ids;
    const uint64_t id = read_id(a.ids, a.id_dtype, i);
    if (id >= static_cast<uint64_t>(a.src_dim)) {
      report_status(a.status, CB200_STATUS_INVALID_INDEX, i, static_cast<int64_t>(id), a.src_dim);
      size[s] = 0;
      return;
    }
    const int64_t off = c * kGatherChunk;
    const int64_t left_bytes = a.row_bytes - off;
    const uint32_t bytes = static_cast<uint32_t>(left_bytes < kGatherChunk ? left_bytes : kGatherChunk);
    const unsigned char* src = a.src + (l * a.src_dim + static_cast<int64_t>(id)) * a.row_bytes + off;
    size[s] = bytes;
    dst[s] = a.out + row * a.row_bytes + off;
    mbar_expect_tx(&bars[s], bytes + a.wt.extra_tx);
    bulk_g2s(ring + static_cast<size_t>(s) * kGatherChunk, src, bytes, &bars[s]);
    pending |= 1u << s;
  };

  for (int64_t j = 0; j < n_my && j < kGatherStages; ++j) issue_load(j);
  bool timed_out = false;
  for (int64_t j = 0; j < n_my; ++j) {
    const int s = static_cast<int>(j % kGatherStages);
    if (size[s] != 0) {
      if (!mbar_wait(&bars[s], (phase >> s) & 1u, a.wt.spins)) {
        report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, first + j * step, 0, a.src_dim);
        timed_out = true;
        break;
      }
      phase ^= 1u << s;
      pending &= ~(1u << s);
      fence_proxy_async_smem();
      bulk_s2g(dst[s], ring + static_cast<size_t>(s) * kGatherChunk, size[s]);
    }
    bulk_commit();
    // refill the slot of the previous item once its store has finished reading shared memory
    if (j >= 1 && j - 1 + kGatherStages < n_my) {
      bulk_wait_read<1>();
      issue_load(j - 1 + kGatherStages);
    }
  }
  bulk_wait_all<0>();
  if (timed_out) {
    // bounded second chance for loads still in flight, so none lands after the CTA retires
    for (int s = 0; s < kGatherStages; ++s)
      if (pending & (1u << s)) mbar_wait(&bars[s], (phase >> s) & 1u, a.wt.spins);
    drain_pause();
  }
}

// ---------------------------------------------------------------------------------------------
// Dense gather with plain W-byte accesses: one warp per output row
// ---------------------------------------------------------------------------------------------
template <typename W>
__global__ void __launch_bounds__(256) gather_rows_vec_kernel(const GatherArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t rows = a.left * a.n_ids;
  const int64_t units = a.row_bytes / static_cast<int64_t>(sizeof(W));
  for (int64_t row = warp; row < rows; row += n_warps) {
    const int64_t l = row / a.n_ids, i = row - l * a.n_ids;
    const uint64_t id = read_id(a.ids, a.id_dtype, i);
    if (id >= static_cast<uint64_t>(a.src_dim)) {
      if (lane == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, i, static_cast<int64_t>(id), a.src_dim);
      continue;
    }
    const W* src = reinterpret_cast<const W*>(a.src + (l * a.src_dim + static_cast<int64_t>(id)) * a.row_bytes);
    W* dst = reinterpret_cast<W*>(a.out + row * a.row_bytes);
    for (int64_t u = lane; u < units; u += 32) dst[u] = src[u];
  }
}

static int64_t common_alignment(const GatherArgs& a) {
  uint64_t bits = reinterpret_cast<uint64_t>(a.src) | reinterpret_cast<uint64_t>(a.out) |
                  static_cast<uint64_t>(a.row_bytes);
  for (int64_t w = 16; w > 1; w >>= 1)
    if ((bits & static_cast<uint64_t>(w - 1)) == 0) return w;
  return 1;
}

cudaError_t launch_gather_rows(const GatherArgs& a_in, cudaStream_t stream) {
  GatherArgs a = a_in;
  a.wt = wait_tuning();
  const int64_t rows = a.left * a.n_ids;
  if (rows == 0 || a.row_bytes == 0) return cudaSuccess;
  const int64_t align = common_alignment(a);
  if (align == 16 && a.row_bytes >= 1024) {
    const int64_t chunks = (a.row_bytes + kGatherChunk - 1) / kGatherChunk;
    const size_t smem = 128 + static_cast<size_t>(kGatherStages) * kGatherChunk;
    cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(gather_rows_bulk_kernel), 32, smem, -1, nullptr);
    if (e != cudaSuccess) return e;
    int64_t grid = static_cast<int64_t>(sm_count()) * 3;  // 3 x 64 KB rings per SM
    if (grid > rows * chunks) grid = rows * chunks;
    gather_rows_bulk_kernel<<<static_cast<unsigned>(grid), 32, smem, stream>>>(a, static_cast<int>(chunks));
    return cudaGetLastError();
  }
  int64_t warps = rows;
  const int64_t max_warps = static_cast<int64_t>(sm_count()) * 8 * 8;
  if (warps > max_warps) warps = max_warps;
  const unsigned grid = static_cast<unsigned>((warps + 7) / 8);
  switch (align) {
    case 16:
      gather_rows_vec_kernel<uint4><<<grid, 256, 0, stream>>>(a);
      break;
    case 8:
      gather_rows_vec_kernel<uint2><<<grid, 256, 0, stream>>>(a);
      break;
    case 4:
      gather_rows_vec_kernel<uint32_t><<<grid, 256, 0, stream>>>(a);
      break;
    case 2:
      gather_rows_vec_kernel<uint16_t><<<grid, 256, 0, stream>>>(a);
      break;
    default:
      gather_rows_vec_kernel<uint8_t><<<grid, 256, 0, stream>>>(a);
      break;
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Quantised row lookup: bulk-stage the row of blocks, decode from shared memory, store T
// ---------------------------------------------------------------------------------------------
constexpr int kQGatherStages = 2;
constexpr int kQGatherThreads = 256;

// `wide`: the f32 destination is 32-byte aligned, so a lane's eight values go out in one 256-bit store
template <int DT>
__device__ __forceinline__ void store_decoded(void* out_row, int v, const float (&f)[8], bool wide) {
  if constexpr (DT == kDtF32) {
    uint4* o = static_cast<uint4*>(out_row) + 2 * v;
    stg_stream_pair(o, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])),
                    make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])),
                    wide);
  } else {
    stg_stream(static_cast<uint4*>(out_row) + v, make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]),
                                                            pack2<DT>(f[4], f[5]), pack2<DT>(f[6], f[7])));
  }
}

template <int QT, int DT>
__global__ void __launch_bounds__(kQGatherThreads) qgather_kernel(const QGatherArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tx = threadIdx.x;
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kQGatherStages * stage_bytes);
  const int V = a.n / 8;
  const size_t out_row_bytes = static_cast<size_t>(a.n) * Elem<DT>::kBytes;
  // (f32 rows are multiples of 128 bytes: a 32-byte aligned base makes every lane's 32 bytes aligned)
  const bool wide = (reinterpret_cast<uintptr_t>(a.out) & 31u) == 0;

  if (tx == 0) {
    for (int s = 0; s < kQGatherStages; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  auto classify = [&](int64_t row, uint64_t& id) -> int {  // 0 decode, 1 masked (zero bits), 2 bad id
    id = read_id(a.ids, a.id_dtype, row);
    if (id >= static_cast<uint64_t>(a.vocab)) return 2;
    if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) return 1;
    return 0;
  };
  auto issue = [&](int64_t row, int stage) {
    uint64_t id;
    if (classify(row, id) != 0) return;
    const unsigned char* src = a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes);
    mbar_expect_tx(&bars[stage], static_cast<uint32_t>(a.row_bytes) + a.wt.extra_tx);
    bulk_g2s(smem_raw + stage * stage_bytes, src, static_cast<uint32_t>(a.row_bytes), &bars[stage]);
  };

  const int64_t first = blockIdx.x, step = gridDim.x;
  if (a.bulk && tx == 0 && first < a.rows) issue(first, 0);
  uint32_t phase = 0;
  int it = 0;
  for (int64_t row = first; row < a.rows; row += step, ++it) {
    const int stage = it % kQGatherStages;
    unsigned char* buf = smem_raw + stage * stage_bytes;
    uint64_t id;
    const int kind = classify(row, id);
    const bool has_next = row + step < a.rows;
    if (a.bulk && tx == 0 && has_next) issue(row + step, (it + 1) % kQGatherStages);
    if (kind == 0) {
      if (a.bulk) {
        const bool ok = mbar_wait(&bars[stage], (phase >> stage) & 1u, a.wt.spins);
        phase ^= 1u << stage;
        if (!__syncthreads_and(ok ? 1 : 0)) {
          if (tx == 0) {
            report_status(a.status, CB200_STATUS_WAIT_TIMEOUT, row, static_cast<int64_t>(id), a.vocab);
            // bounded second chance for this row's copy and for the prefetch of the next one
            mbar_wait(&bars[stage], ((phase >> stage) & 1u) ^ 1u, a.wt.spins);
            uint64_t nid;
            if (has_next && classify(row + step, nid) == 0) {
              const int ns = (it + 1) % kQGatherStages;
              mbar_wait(&bars[ns], (phase >> ns) & 1u, a.wt.spins);
            }
            drain_pause();
          }
          return;
        }
      } else {
        const uint16_t* src =
            reinterpret_cast<const uint16_t*>(a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes));
        uint16_t* dst = reinterpret_cast<uint16_t*>(buf);
        for (int i = tx; i < a.row_bytes / 2; i += kQGatherThreads) dst[i] = src[i];
        __syncthreads();
      }
    }
    unsigned char* out_row = static_cast<unsigned char*>(a.out) + static_cast<size_t>(row) * out_row_bytes;
    if (kind == 0) {
      for (int v = tx; v < V; v += kQGatherThreads) {
        float f[8];
        decode8<QT, true>(buf, v, f);  // the staged row starts on a 16-byte boundary
        store_decoded<DT>(out_row, v, f, wide);
      }
    } else if (kind == 1) {
      const int n_vec = static_cast<int>(out_row_bytes / 16);
      for (int v = tx; v < n_vec; v += kQGatherThreads)
        stg_stream(reinterpret_cast<uint4*>(out_row) + v, masked_row_vec());
    } else if (tx == 0) {
      report_status(a.status, CB200_STATUS_INVALID_INDEX, row, static_cast<int64_t>(id), a.vocab);
    }
    __syncthreads();  // `buf` may now be refilled
  }
}

template <int QT, int DT>
static cudaError_t launch_qgather_t(const QGatherArgs& a_in, cudaStream_t stream) {
  QGatherArgs a = a_in;
  a.wt = wait_tuning();
  const int stage_bytes = (a.row_bytes + 15) & ~15;
  const size_t smem = static_cast<size_t>(kQGatherStages) * stage_bytes + kQGatherStages * 8;
  auto kern = qgather_kernel<QT, DT>;
  cudaError_t e = kernel_launch_config(reinterpret_cast<const void*>(kern), kQGatherThreads, smem, -1, nullptr);
  if (e != cudaSuccess) return e;
  int64_t grid = static_cast<int64_t>(sm_count()) * 8;
  if (grid > a.rows) grid = a.rows;
  kern<<<static_cast<unsigned>(grid), kQGatherThreads, smem, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_qgather(int qtype, int out_dtype, const QGatherArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
#define CB200_QG(QT)                                               \
  switch (out_dtype) {                                             \
    case kDtF32:                                                   \
      return launch_qgather_t<QT, kDtF32>(a, stream);              \
    case kDtF16:                                                   \
      return launch_qgather_t<QT, kDtF16>(a, stream);              \
    default:                                                       \
      return launch_qgather_t<QT, kDtBF16>(a, stream);             \
  }
  if (qtype == CB200_QTYPE_Q8_0) {
    CB200_QG(CB200_QTYPE_Q8_0)
  }
  if (qtype == CB200_QTYPE_Q4_1) {
    CB200_QG(CB200_QTYPE_Q4_1)
  }
  if (qtype == CB200_QTYPE_Q5_0) {
    CB200_QG(CB200_QTYPE_Q5_0)
  }
  if (qtype == CB200_QTYPE_Q5_1) {
    CB200_QG(CB200_QTYPE_Q5_1)
  }
  if (qtype == CB200_QTYPE_Q2K) {
    CB200_QG(CB200_QTYPE_Q2K)
  }
  if (qtype == CB200_QTYPE_Q3K) {
    CB200_QG(CB200_QTYPE_Q3K)
  }
  if (qtype == CB200_QTYPE_Q4K) {
    CB200_QG(CB200_QTYPE_Q4K)
  }
  if (qtype == CB200_QTYPE_Q5K) {
    CB200_QG(CB200_QTYPE_Q5K)
  }
  if (qtype == CB200_QTYPE_Q6K) {
    CB200_QG(CB200_QTYPE_Q6K)
  }
  if (qtype == CB200_QTYPE_Q8K) {
    CB200_QG(CB200_QTYPE_Q8K)
  }
  CB200_QG(CB200_QTYPE_Q4_0)
#undef CB200_QG
}

// ---------------------------------------------------------------------------------------------
// Routing of raw block rows for a vocabulary-sharded table whose consumers are row-sharded: the
// rank that owns id[i] copies the QUANTISED row (a few KB instead of the decoded 2 * hidden bytes) into
// the staging buffer of the rank whose block of token rows contains i, at row i - row_bounds[r].
// One warp per token row, plain 16-byte loads and stores (peer memory is only ever stored to).
// ---------------------------------------------------------------------------------------------
struct QRouteArgs {
  const unsigned char* qtable;  // rows [vocab_begin, vocab_end)
  const void* ids;
  int id_dtype;
  int64_t vocab, vocab_begin, vocab_end;
  cb200_status* status;
  int64_t rows;
  int row_bytes;
  int n_dsts;
  unsigned char* dsts[8];
  int64_t row_bounds[9];
};

template <typename W>
__global__ void __launch_bounds__(256) qroute_rows_kernel(const QRouteArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int units = a.row_bytes / static_cast<int>(sizeof(W));
  constexpr int K = 8;  // units per lane in flight
  for (int64_t i = warp; i < a.rows; i += n_warps) {
    const uint64_t id = read_id(a.ids, a.id_dtype, i);
    if (id >= static_cast<uint64_t>(a.vocab)) {
      if (lane == 0) report_status(a.status, CB200_STATUS_INVALID_INDEX, i, static_cast<int64_t>(id), a.vocab);
      continue;
    }
    if (id < static_cast<uint64_t>(a.vocab_begin) || id >= static_cast<uint64_t>(a.vocab_end)) continue;  // another rank's
    int r = 0;
#pragma unroll
    for (int d = 1; d < 8; ++d)
      if (d < a.n_dsts && i >= a.row_bounds[d]) r = d;
    const W* src = reinterpret_cast<const W*>(a.qtable + (id - a.vocab_begin) * static_cast<uint64_t>(a.row_bytes));
    W* dst = reinterpret_cast<W*>(a.dsts[r] + (i - a.row_bounds[r]) * static_cast<int64_t>(a.row_bytes));
    for (int u0 = 0; u0 < units; u0 += 32 * K) {
      W v[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int u = u0 + 32 * k + lane;
        if (u < units) v[k] = src[u];
      }
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int u = u0 + 32 * k + lane;
        if (u < units) dst[u] = v[k];
      }
    }
  }
}

cudaError_t launch_qroute_rows(const unsigned char* qtable, const void* ids, int id_dtype, int64_t vocab,
                               int64_t vocab_begin, int64_t vocab_end, cb200_status* status, int64_t rows, int row_bytes,
                               void* const* dsts, int n_dsts, const int64_t* row_bounds, cudaStream_t stream) {
  if (rows == 0 || row_bytes == 0) return cudaSuccess;
  QRouteArgs a{};
  a.qtable = qtable;
  a.ids = ids;
  a.id_dtype = id_dtype;
  a.vocab = vocab;
  a.vocab_begin = vocab_begin;
  a.vocab_end = vocab_end;
  a.status = status;
  a.rows = rows;
  a.row_bytes = row_bytes;
  a.n_dsts = n_dsts;
  bool vec = (reinterpret_cast<uintptr_t>(qtable) & 15u) == 0 && row_bytes % 16 == 0;
  for (int d = 0; d < n_dsts; ++d) {
    a.dsts[d] = static_cast<unsigned char*>(dsts[d]);
    a.row_bounds[d] = row_bounds[d];
    vec = vec && (reinterpret_cast<uintptr_t>(dsts[d]) & 15u) == 0;
  }
  a.row_bounds[n_dsts] = row_bounds[n_dsts];
  int64_t grid = (rows + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  if (vec)
    qroute_rows_kernel<uint4><<<static_cast<unsigned>(grid), 256, 0, stream>>>(a);
  else
    qroute_rows_kernel<uint16_t><<<static_cast<unsigned>(grid), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Whole-buffer decode (QTensor::dequantize): 8 elements per thread straight from global memory
// ---------------------------------------------------------------------------------------------
template <int QT, int DT>
__global__ void __launch_bounds__(256) dequantize_flat_kernel(const unsigned char* __restrict__ blocks,
                                                              void* __restrict__ out, int64_t n_vec, int aligned16) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const bool wide = (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
    constexpr int kVecs = qblock_elems(QT) / 8;  // 8-element groups per block
    const unsigned char* blk = blocks + (v / kVecs) * QBlock<QT>::kBytes;
    float f[8];
    if (aligned16)  // (uniform: a property of the `blocks` pointer)
      decode8<QT, true>(blk, static_cast<int>(v % kVecs), f);
    else
      decode8<QT, false>(blk, static_cast<int>(v % kVecs), f);
    // element offset 8v: express as a row of one vector
    unsigned char* o = static_cast<unsigned char*>(out) + static_cast<size_t>(v) * 8 * Elem<DT>::kBytes;
    store_decoded<DT>(o, 0, f, wide);
  }
}

cudaError_t launch_dequantize_flat(int qtype, int out_dtype, const void* blocks, void* out, int64_t n_vec,
                                   cudaStream_t stream) {
  if (n_vec == 0) return cudaSuccess;
  int64_t grid = (n_vec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (grid > cap) grid = cap;
  const unsigned char* b = static_cast<const unsigned char*>(blocks);
  const int aligned16 = (reinterpret_cast<uintptr_t>(blocks) & 15u) == 0;
#define CB200_DQ(QT)                                                                            \
  switch (out_dtype) {                                                                          \
    case kDtF32:                                                                                \
      dequantize_flat_kernel<QT, kDtF32><<<static_cast<unsigned>(grid), 256, 0, stream>>>(b, out, n_vec, aligned16);  \
      break;                                                                                    \
    case kDtF16:                                                                                \
      dequantize_flat_kernel<QT, kDtF16><<<static_cast<unsigned>(grid), 256, 0, stream>>>(b, out, n_vec, aligned16);  \
      break;                                                                                    \
    default:                                                                                    \
      dequantize_flat_kernel<QT, kDtBF16><<<static_cast<unsigned>(grid), 256, 0, stream>>>(b, out, n_vec, aligned16); \
      break;                                                                                    \
  }
  if (qtype == CB200_QTYPE_Q8_0) {
    CB200_DQ(CB200_QTYPE_Q8_0)
  } else if (qtype == CB200_QTYPE_Q4_1) {
    CB200_DQ(CB200_QTYPE_Q4_1)
  } else if (qtype == CB200_QTYPE_Q5_0) {
    CB200_DQ(CB200_QTYPE_Q5_0)
  } else if (qtype == CB200_QTYPE_Q5_1) {
    CB200_DQ(CB200_QTYPE_Q5_1)
  } else if (qtype == CB200_QTYPE_Q2K) {
    CB200_DQ(CB200_QTYPE_Q2K)
  } else if (qtype == CB200_QTYPE_Q3K) {
    CB200_DQ(CB200_QTYPE_Q3K)
  } else if (qtype == CB200_QTYPE_Q4K) {
    CB200_DQ(CB200_QTYPE_Q4K)
  } else if (qtype == CB200_QTYPE_Q5K) {
    CB200_DQ(CB200_QTYPE_Q5K)
  } else if (qtype == CB200_QTYPE_Q6K) {
    CB200_DQ(CB200_QTYPE_Q6K)
  } else if (qtype == CB200_QTYPE_Q8K) {
    CB200_DQ(CB200_QTYPE_Q8K)
  } else {
    CB200_DQ(CB200_QTYPE_Q4_0)
  }
#undef CB200_DQ
  return cudaGetLastError();
}

}  // namespace cb200
