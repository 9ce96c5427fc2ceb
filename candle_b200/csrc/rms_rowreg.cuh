// Register-resident RMS norm for 16-bit element types (bf16 / f16).
//
// One row is spread over `tpr` threads (a warp up to 512 threads), each holding up to VPT 16-byte
// vectors of the row in registers, so the row is read from HBM exactly once.
//
// Bit-exactness with candle's CPU path (candle-nn/src/ops.rs:484-495) needs the row's sum of
// squares in strictly sequential f32 order, which a parallel reduction cannot give directly.
// But the CPU path rounds m = sqrt(sum/n + eps) to the 16-bit type before using it, so all that
// matters is T(m).  The kernel therefore
//   1. reduces sum(p_j) and W = sum(p_j * (n - j)) in tree order (p_j = h_j^2 is exact in f32
//      for 16-bit h_j),
//   2. bounds the sequential result rigorously: with u = 2^-24, |seq - exact| <= u(1+g) * W
//      (each of the n-1 additions errs by at most u times its partial sum, and the partial sums
//      add up to at most W) and |tree - exact| <= 128u * exact,
//   3. evaluates candle's f32 pipeline (all of it monotone) at both ends of the interval; if
//      T(m) agrees at both ends it IS the sequential answer,
//   4. otherwise (a few percent of rows at 8192 columns) parks the row in shared memory and replays
//      it exactly (replay_sum_sq below).
// Arithmetic in T uses the packed two-element instructions (add/mul .rn .bf16x2/.f16x2): the
// kernel is otherwise bound by instruction issue rather than by HBM.
// The division x / m rounded to bf16 is evaluated as bf16(x * (1/m)): a quotient of two 8-bit
// significands is never closer than 2^-17 (relative) to a bf16 rounding boundary, far more than
// the 2^-22 error of the reciprocal product, so both round identically.  f16 has no such margin
// and uses the correctly rounded division.
#pragma once

#include "common.cuh"

namespace cb200 {

struct RmsRowRegArgs {
  const uint4* x;      // [rows, V] vectors, or the dense table [vocab, V] when ids != nullptr
  const uint4* res;    // optional residual [rows, V]
  const uint4* alpha;  // [V]
  uint4* y;            // [rows, V]
  uint4* sum_out;      // optional: h = x + res (or the gathered rows)
  const void* ids;     // optional row ids into x
  int id_dtype;
  int64_t vocab;
  cb200_status* status;
  int64_t rows;
  int V;  // 16-byte vectors per row = cols / 8
  int n;  // cols
  float eps;
  int flags;
};

// Arguments of the kernel whose rows come out of a Q4_0 / Q8_0 table.
struct QRmsArgs {
  const unsigned char* qtable;  // rows [vocab_begin, vocab_end) of the table
  const void* ids;
  const uint4* alpha;
  uint4* y;
  uint4* gathered;  // optional decoded rows
  int id_dtype;
  int64_t vocab, vocab_begin, vocab_end;
  cb200_status* status;
  int64_t rows;
  int V, n;
  int row_bytes;  // bytes of one quantised row
  int bulk;       // 1: rows are 16-byte multiples and the table is 16-byte aligned
  float eps;
  int flags;
  // Owner-writes-to-all mode for a vocabulary-sharded table: rows whose id lies outside
  // [vocab_begin, vocab_end) are skipped instead of written as zero bits, and every finished row also
  // goes to `n_more` further buffers of the same shape (peers' memory mapped into this process).
  // owned_only == 2 (row-owner mode): a finished row goes to exactly one buffer, that of the rank
  // whose block of token rows contains it: destination r (y for r == 0, y_more[r - 1] otherwise)
  // holds rows [row_bounds[r], row_bounds[r + 1]) as a [rows_r, V] tensor of its own.
  int owned_only;
  int n_more;
  int wide;  // filled by the launcher: every destination is 32-byte aligned
  uint4* y_more[7];
  int64_t row_bounds[9];
  WaitTuning wt;  // filled by the launcher
};

// Shared-memory layout of one CTA of the row-register kernels (per row slot `ty`).
struct RowRegSmem {
  float* red;    // [48]: warp partials of sum (0..15), of the weighted sum (16..31), of a minimum (32..47)
  float* pub;    // [4]: the resolved T(m), published by warp 0 of the row
  int4* chunks;  // [tpr] replay: {A, B - A, L, -}: while the sum's bit pattern stays in the
                 // binade that starts at L, a chunk adds A to an even and B to an odd one
  int4* segs;    // [tpr] replay: the same for runs of chunks, {A, B - A, L, first | count << 16}
                 // (one more array of [tpr] follows segs: the second parts of runs that cross a binade)
  uint4* rows;   // [V]: h, parked for the replay
  __device__ RowRegSmem(unsigned char* base, int rpc, int tpr, int V, int ty) {
    unsigned char* mine = base + static_cast<size_t>(ty) * slot_bytes(tpr);
    chunks = reinterpret_cast<int4*>(mine);
    segs = chunks + tpr;
    red = reinterpret_cast<float*>(mine + static_cast<size_t>(tpr) * 48);
    pub = red + 48;
    rows = reinterpret_cast<uint4*>(base + static_cast<size_t>(rpc) * slot_bytes(tpr)) + static_cast<size_t>(ty) * V;
  }
  // (48 bytes per thread; every byte of shared memory is taken from L1, where the data of loads in flight lands)
  __host__ __device__ static size_t slot_bytes(int tpr) { return static_cast<size_t>(tpr) * 48 + 52 * sizeof(float); }
  __host__ __device__ static size_t bytes(int rpc, int tpr, int V, bool with_rows) {
    return static_cast<size_t>(rpc) * slot_bytes(tpr) + (with_rows ? static_cast<size_t>(rpc) * V * 16 : 0);
  }
};

// Packed two-element arithmetic in T with one IEEE rounding per lane -- exactly what crate `half`
// yields for `a + b` / `a * b` on T (operate in f32, round back): the exact sum or product of two
// 16-bit values fits the f32 significand's 2p+2 bits, so rounding it once to T is the same thing.
template <int DT>
__device__ __forceinline__ uint32_t add2_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (DT == kDtBF16)
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
template <int DT>
__device__ __forceinline__ uint32_t mul2_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (DT == kDtBF16)
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ void row_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// h = T(x + res) for one vector.
template <int DT>
__device__ __forceinline__ uint4 add_round_vec(const uint4& a, const uint4& b) {
  return make_uint4(add2_rn<DT>(a.x, b.x), add2_rn<DT>(a.y, b.y), add2_rn<DT>(a.z, b.z), add2_rn<DT>(a.w, b.w));
}

// Adds one vector's squares to the tree-order sums.  `vec_index` is the vector's position in the
// row; all eight elements are weighted with n - 8*vec_index, an upper bound of their own n - j.
// h*h is exact in f32 for 16-bit h, so the fused multiply-add rounds exactly like add(s, h*h).
template <int DT>
__device__ __forceinline__ void accumulate_vec(const uint4& h, int vec_index, int n, float& lsum, float& lw) {
  const uint32_t w[4] = {h.x, h.y, h.z, h.w};
  float vs = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = unpack2<DT>(w[i]);
    vs = fmaf(f.x, f.x, vs);
    vs = fmaf(f.y, f.y, vs);
  }
  lsum += vs;
  lw = fmaf(vs, static_cast<float>(n - 8 * vec_index), lw);
}

// Sequential sum of squares over vectors [v0, v1) of a row in shared memory, continuing from s:
// candle's order and roundings (candle-nn/src/ops.rs:484-490).
// A row of 16-bit elements as seen by the replay: vector v = elements [8v, 8v+8).  ParkedRow reads
// h parked in shared memory; the quantised kernels pass an accessor that decodes on the fly.
struct ParkedRow {
  const uint4* p;
  __device__ __forceinline__ uint4 vec(int v) const { return p[v]; }
};

template <int DT, typename Row>
__device__ __forceinline__ float sequential_sum_sq(const Row& row, int v0, int v1, float s) {
#pragma unroll 2
  for (int v = v0; v < v1; ++v) {
    uint4 q = row.vec(v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = unpack2<DT>(w[i]);
      s = __fadd_rn(s, __fmul_rn(f.x, f.x));
      s = __fadd_rn(s, __fmul_rn(f.y, f.y));
    }
  }
  return s;
}

// Exact sequential-order sum of squares of the row parked in sm.rows, computed cooperatively by
// the tpr threads of the row (all must call; the result is valid in thread 0 of the row).
//
// A chain s <- fl(s + p) with p >= 0 cannot be split naively, but while s stays inside one
// binade [2^e, 2^(e+1)) it is integer arithmetic on the significand S: fl(S + P) = S + round(P)
// where the tie rule only looks at the parity of S.  So the effect of a run of additions on ANY
// start value of that binade is "S + A if S is even, S + B if S is odd", and A, B can be measured
// by running the run twice, from an even and from an odd reference value of the same binade.
// Every thread measures (A, B) for its own contiguous chunk, using the approximate prefix sum to
// pick the binade -- and, where that prefix says the sum leaves the binade inside the chunk, cuts
// the chunk there: (A, B) up to the crossing element, the element itself, (A, B) after it in the
// next binade.  Thread 0 then walks the chunks with exact integer updates (the crossing element
// with a real addition), checking that the true value really is in the assumed binade before and
// after each part (the sum is monotone, so that covers the whole part) and falling back to plain
// sequential addition for the chunk otherwise.  The checks make the result exact whatever the
// quality of the guesses.
template <int DT, typename Row>
__device__ __noinline__ float replay_sum_sq(const Row rows, int4* chunks, int4* segs, float* red, int V,
                                            int bar_id) {
  const int tx = threadIdx.x, tpr = blockDim.x;
  const int lane = tx & 31, warp = tx >> 5, wpr = tpr >> 5;
  const int vpc = (V + tpr - 1) / tpr;  // vectors per chunk
  const int v0 = min(V, tx * vpc), v1 = min(V, v0 + vpc);

  float sig = 0.0f;
  for (int v = v0; v < v1; ++v) {
    uint4 q = rows.vec(v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = unpack2<DT>(w[i]);
      sig = fmaf(f.x, f.x, sig);
      sig = fmaf(f.y, f.y, sig);
    }
  }
  // approximate exclusive prefix of the chunk sums
  float incl = sig;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += t;
  }
  if (wpr > 1) {
    if (lane == 31) red[warp] = incl;
    row_barrier(bar_id, tpr);
    float base = 0.0f;
    for (int i = 0; i < warp; ++i) base += red[i];
    incl += base;
  }
  const float prefix = incl - sig;

  // Measure the chunk from an even and an odd reference value next to the approximate prefix.  The
  // approximate running sum `t` also tells where the sum leaves the binade: the chunk is then cut at
  // that element -- {A, B} before it, the element itself (added for real by the walk), {A, B} after it
  // in the next binade.  A second crossing in one chunk leaves the chunk to the sequential fallback.
  int4* segs2 = segs + tpr;
  uint32_t base = __float_as_uint(prefix) & ~1u;
  int e = static_cast<int>(base >> 23);
  const bool ok = (v0 < v1) && (prefix > 0.0f) && (e >= 67) && (e <= 187);  // 2^-60 .. 2^60
  float s0 = __uint_as_float(base), s1 = __uint_as_float(base + 1u);
  float t = prefix, pcross = 0.0f;
  uint32_t A1 = 0u, BA1 = 0u, lo1 = 0xFFFFFFFFu, A2 = 0u, BA2 = 0u, lo2 = 0xFFFFFFFFu;
  int ncross = 0;
  {
    // second pair of references: they start, in the next binade, at the crossing element
    float s0b = 0.0f, s1b = 0.0f;
    uint32_t base2 = 0u;
    uint32_t texp = __float_as_uint(t) >> 23;
    for (int k = 0; k < vpc; ++k) {  // every thread of the warp makes vpc trips: the vote below is warp-wide
      const int v = v0 + k;
      const uint4 q = v < v1 ? rows.vec(v) : make_uint4(0, 0, 0, 0);  // (past the row: zeros change nothing)
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      float p[8];
      float vs = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = unpack2<DT>(w[i]);
        p[2 * i] = __fmul_rn(f.x, f.x);  // exact
        p[2 * i + 1] = __fmul_rn(f.y, f.y);
        vs += p[2 * i] + p[2 * i + 1];
      }
      const float t8 = t + vs;
      const bool calm = ok && ncross == 0 && (__float_as_uint(t8) >> 23) == texp;
      if (__all_sync(0xFFFFFFFFu, calm || !ok)) {
        // no lane of the warp sees a crossing in these eight elements (the sum never decreases: equal
        // ends mean none inside): the plain pair of chains
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          s0 = __fadd_rn(s0, p[i]);
          s1 = __fadd_rn(s1, p[i]);
        }
        t = t8;
      } else {
        // branch-free form: an element goes to the first pair of references before the crossing, to
        // the second pair after it, and is kept aside if it is the crossing element itself
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float tn = t + p[i];
          const uint32_t nexp = __float_as_uint(tn) >> 23;
          const bool changed = nexp != texp;
          const bool first = changed && ncross == 0;
          const float a1 = (ncross == 0 && !changed) ? p[i] : 0.0f;
          const float a2 = (ncross == 1 && !changed) ? p[i] : 0.0f;
          s0 = __fadd_rn(s0, a1);
          s1 = __fadd_rn(s1, a1);
          s0b = __fadd_rn(s0b, a2);
          s1b = __fadd_rn(s1b, a2);
          if (first) {
            pcross = p[i];
            base2 = __float_as_uint(tn) & ~1u;
            s0b = __uint_as_float(base2);
            s1b = __uint_as_float(base2 + 1u);
          }
          ncross += changed ? 1 : 0;
          t = tn;
          texp = nexp;
        }
      }
    }
    if (ok) {
      const bool in1 = static_cast<int>(__float_as_uint(s1) >> 23) == e;  // the references stayed in the binade
      A1 = __float_as_uint(s0) - base;
      BA1 = (__float_as_uint(s1) - (base + 1u)) - A1;
      lo1 = in1 ? (static_cast<uint32_t>(e) << 23) : 0xFFFFFFFFu;
      if (ncross == 1) {
        const int e2 = static_cast<int>(base2 >> 23);
        const bool in2 = static_cast<int>(__float_as_uint(s1b) >> 23) == e2 && e2 <= 187;
        A2 = __float_as_uint(s0b) - base2;
        BA2 = (__float_as_uint(s1b) - (base2 + 1u)) - A2;
        lo2 = in2 ? (static_cast<uint32_t>(e2) << 23) : 0xFFFFFFFFu;
      }
    }
  }
  if (ncross >= 2) lo1 = 0xFFFFFFFFu;
  // chunk record: {A, B - A, first bit pattern of the binade, -}; an unusable chunk gets a binade
  // start no running sum can reach, so the range check of the walk rejects it.  Only chunks that stay
  // in one binade take part in the composition below.
  const bool whole = lo1 != 0xFFFFFFFFu && ncross == 0;
  uint32_t inc_even = A1, inc_odd = A1 + BA1;
  const uint32_t lo = whole ? lo1 : 0xFFFFFFFFu;
  chunks[tx] = make_int4(static_cast<int>(A1), static_cast<int>(BA1), static_cast<int>(ncross == 0 ? lo1 : 0xFFFFFFFFu), 0);

  // Runs of consecutive chunks of one warp that share a binade compose into one record: for an
  // even start the run adds A1 + (A1 odd ? B2 : A2), for an odd start B1 + (B1 odd ? A2 : B2).
  // A suffix scan restricted to the run leaves the whole run's record in its first lane.
  const uint32_t key = whole ? lo : (0xFFFFFF00u | static_cast<uint32_t>(lane));  // the others stay alone
  const uint32_t prev_key = __shfl_up_sync(0xFFFFFFFFu, key, 1);
  const bool head = (lane == 0) || (key != prev_key);
  const uint32_t heads = __ballot_sync(0xFFFFFFFFu, head);
  const int sid = __popc(heads & (0xFFFFFFFFu >> (31 - lane)));  // 1-based run number inside the warp
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t nA = __shfl_down_sync(0xFFFFFFFFu, inc_even, d);
    const uint32_t nB = __shfl_down_sync(0xFFFFFFFFu, inc_odd, d);
    const int nsid = __shfl_down_sync(0xFFFFFFFFu, sid, d);
    if (lane + d < 32 && nsid == sid) {
      const uint32_t a2 = (inc_even & 1u) ? nB : nA;
      const uint32_t b2 = (inc_odd & 1u) ? nA : nB;
      inc_even += a2;
      inc_odd += b2;
    }
  }
  const int n_runs = __popc(heads);
  int run_base = 0;
  if (wpr > 1) {
    if (lane == 0) red[16 + warp] = __int_as_float(n_runs);
    row_barrier(bar_id, tpr);
    for (int i = 0; i < warp; ++i) run_base += __float_as_int(red[16 + i]);
  }
  if (head) {
    // length of the run: distance to the next head of the warp
    const uint32_t later = heads & ~(0xFFFFFFFFu >> (31 - lane));
    const int len = (later ? __ffs(later) - 1 : 32) - lane;
    if (ncross == 1) {
      // a chunk that crosses is a run of its own, and the run record carries both of its parts
      segs[run_base + sid - 1] = make_int4(static_cast<int>(A1), static_cast<int>(BA1), static_cast<int>(lo1),
                                           tx | (1 << 16) | (1 << 30));
      segs2[run_base + sid - 1] =
          make_int4(static_cast<int>(A2), static_cast<int>(BA2), static_cast<int>(lo2), __float_as_int(pcross));
    } else {
      segs[run_base + sid - 1] = make_int4(static_cast<int>(inc_even), static_cast<int>(inc_odd - inc_even),
                                           static_cast<int>(lo), tx | (len << 16));
    }
  }
  int total_runs = n_runs;
  if (wpr > 1) {
    row_barrier(bar_id, tpr);
    total_runs = 0;
    for (int i = 0; i < wpr; ++i) total_runs += __float_as_int(red[16 + i]);
  } else {
    __syncwarp();
  }

  float result = 0.0f;
  if (tx == 0) {
    uint32_t S = 0u;  // bits of the running sum (+0.0f)
    // One chunk: S stays in the chunk's binade before and after (the sum never decreases, so in
    // between as well) -> exact integer update; otherwise add the chunk's elements one by one.
    auto chunk_step = [&](int c) {
      const int4 k = chunks[c];
      const uint32_t lo_c = static_cast<uint32_t>(k.z);
      const uint32_t S2 = S + static_cast<uint32_t>(k.x) + (S & 1u) * static_cast<uint32_t>(k.y);
      if (lo_c != 0xFFFFFFFFu && S >= lo_c && (S2 - lo_c) < 0x800000u) {
        S = S2;
        return;
      }
      // (a chunk that crosses a binade has its two parts in its run record only: if that did not apply,
      // the prediction was off and the chunk is added element by element)
      const int c0 = min(V, c * vpc), c1 = min(V, c0 + vpc);
      S = __float_as_uint(sequential_sum_sq<DT, Row>(rows, c0, c1, __uint_as_float(S)));
    };
    int4 cur = segs[0], cur2 = segs2[0];
    for (int r = 0; r < total_runs; ++r) {
      const int rn = min(r + 1, total_runs - 1);
      const int4 nxt = segs[rn], nxt2 = segs2[rn];  // off the dependency chain (segs2 is read even where unused)
      const bool cross = (cur.w >> 30) & 1;
      const uint32_t lo_r = static_cast<uint32_t>(cur.z);
      const uint32_t S2 = S + static_cast<uint32_t>(cur.x) + (S & 1u) * static_cast<uint32_t>(cur.y);
      bool ok = lo_r != 0xFFFFFFFFu && S >= lo_r && (S2 - lo_r) < 0x800000u;
      uint32_t Sn = S2;
      if (cross) {
        // the crossing element for real, then the second part in the next binade
        const uint32_t lo_2 = static_cast<uint32_t>(cur2.z);
        const uint32_t S3 = __float_as_uint(__fadd_rn(__uint_as_float(S2), __int_as_float(cur2.w)));
        Sn = S3 + static_cast<uint32_t>(cur2.x) + (S3 & 1u) * static_cast<uint32_t>(cur2.y);
        ok = ok && lo_2 != 0xFFFFFFFFu && S3 >= lo_2 && (Sn - lo_2) < 0x800000u;
      }
      if (ok) {
        S = Sn;
      } else {
        // the run as a whole does not apply: take its chunks one at a time
        const int first = cur.w & 0xFFFF, count = (cur.w >> 16) & 0x3FFF;
        for (int c = first; c < first + count; ++c) chunk_step(c);
      }
      cur = nxt;
      cur2 = nxt2;
    }
    result = __uint_as_float(S);
  }
  return result;
}

// Decides T(m) from the tree-order sums (s, w); returns false if only a sequential replay can.
// Must be called by a full warp with the same (s, w) in every lane: even lanes evaluate the lower
// end of the interval and odd lanes the upper end, side by side, and swap results.
template <int DT>
__device__ __forceinline__ bool decide_m(float s, float w, float nf, float eps, float& m) {
  constexpr float kU = 5.9604644775390625e-8f;  // 2^-24
  // |seq - tree| <= 1.01*u*W + 160*u*s covers both bounds, the f32 rounding of w and of this
  // expression itself.
  const float err = 1.01f * kU * w + 160.0f * kU * s;
  const bool upper = threadIdx.x & 1;
  const float mine = round_to<DT>(rms_from_sum(upper ? s + err : s - err, nf, eps));
  const float other = __shfl_xor_sync(0xFFFFFFFFu, mine, 1);
  m = upper ? other : mine;  // T(m) at the lower end, in every lane
  // Squares below 2^-149 are not exact in f32; that can only matter when the whole row is that
  // small AND eps is too: let the replay, which rounds like the CPU, handle it.
  const bool tiny = (s < 7.8886091e-31f) && (eps < 1e-18f) && (s != 0.0f || w != 0.0f);
  return (mine == other) && !tiny;  // false as well when anything is NaN
}

// Step 1 of resolving T(m) for the row whose per-thread partial sums are (lsum, lw): the tpr
// threads of row slot threadIdx.y reduce them (named barrier id 1 + threadIdx.y for rows wider
// than a warp) and warp 0 of the row decides.  Returns T(m) if `need_replay` comes back false;
// otherwise only replay_row can tell.  `lmin` is a per-thread value whose minimum over the row
// is returned in `row_min` when that pointer is given.
// ONE_BARRIER (rows of up to four warps): after the exchange of the warp partials every warp adds them
// up and decides for itself -- same inputs, same operations, same answer -- instead of waiting for
// warp 0 to publish.  The warps then leave at different times, so the caller must synchronise the
// row's warps again before anything overwrites sm.red: before the next row, and before replay_row.
template <int DT, bool ONE_BARRIER = false>
__device__ __forceinline__ float decide_row(float lsum, float lw, int n, float eps, int flags, RowRegSmem& sm,
                                            bool& need_replay, float lmin = 0.0f, float* row_min = nullptr) {
  const int tx = threadIdx.x, tpr = blockDim.x;
  const int lane = tx & 31, warp = tx >> 5, wpr = tpr >> 5;
  const float nf = static_cast<float>(n);
  const bool fast = flags & CB200_FLAG_FAST_SUM;
  const bool force = flags & CB200_FLAG_FORCE_REPLAY;
  const int bar_id = 1 + threadIdx.y;

  float s = warp_sum(lsum), w = warp_sum(lw);
  float m = 0.0f;
  if (row_min != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmin = fminf(lmin, __shfl_xor_sync(0xFFFFFFFFu, lmin, o));
  }
  if (wpr == 1) {
    if (row_min != nullptr) *row_min = lmin;
    if (fast) {
      need_replay = false;
      return round_to<DT>(rms_from_sum(s, nf, eps));
    }
    need_replay = !decide_m<DT>(s, w, nf, eps, m) || force;  // warp-uniform
    return m;
  }
  if (lane == 0) {
    sm.red[warp] = s;
    sm.red[16 + warp] = w;
    if (row_min != nullptr) sm.red[32 + warp] = lmin;
  }
  row_barrier(bar_id, tpr);
  if (ONE_BARRIER && wpr <= 4) {
    s = sm.red[0];
    w = sm.red[16];
    float mn = row_min != nullptr ? sm.red[32] : 0.0f;
    for (int i = 1; i < wpr; ++i) {
      s += sm.red[i];
      w += sm.red[16 + i];
      if (row_min != nullptr) mn = fminf(mn, sm.red[32 + i]);
    }
    if (row_min != nullptr) *row_min = mn;
    if (fast) {
      need_replay = false;
      return round_to<DT>(rms_from_sum(s, nf, eps));
    }
    need_replay = !decide_m<DT>(s, w, nf, eps, m) || force;
    return m;
  }
  if (warp == 0) {
    s = warp_sum(lane < wpr ? sm.red[lane] : 0.0f);
    bool need = false;
    if (fast) {
      m = round_to<DT>(rms_from_sum(s, nf, eps));
    } else {
      w = warp_sum(lane < wpr ? sm.red[16 + lane] : 0.0f);
      need = !decide_m<DT>(s, w, nf, eps, m) || force;
    }
    float mn = 0.0f;
    if (row_min != nullptr) {
      mn = lane < wpr ? sm.red[32 + lane] : 3.0e38f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
    }
    if (lane == 0) *reinterpret_cast<float4*>(sm.pub) = make_float4(m, need ? 1.0f : 0.0f, 0.0f, mn);
  }
  row_barrier(bar_id, tpr);
  const float4 pub = *reinterpret_cast<const float4*>(sm.pub);
  need_replay = pub.y != 0.0f;  // row-uniform
  if (row_min != nullptr) *row_min = pub.w;
  return pub.x;
}

// Step 2, for the few rows that need it: T(m) from the exact sequential-order sum of the row as
// `row` presents it.  All tpr threads of the row call it; whatever `row` reads must be complete
// and visible to them (the caller synchronises after parking).
template <int DT, typename Row>
__device__ __forceinline__ float replay_row(const Row& row, int V, int n, float eps, RowRegSmem& sm) {
  const int tx = threadIdx.x, tpr = blockDim.x, wpr = tpr >> 5;
  const int bar_id = 1 + threadIdx.y;
  const float nf = static_cast<float>(n);
  const float total = replay_sum_sq<DT, Row>(row, sm.chunks, sm.segs, sm.red, V, bar_id);
  if (wpr == 1) return __shfl_sync(0xFFFFFFFFu, round_to<DT>(rms_from_sum(total, nf, eps)), 0);
  if (tx == 0) sm.pub[2] = round_to<DT>(rms_from_sum(total, nf, eps));
  row_barrier(bar_id, tpr);
  return sm.pub[2];
}

// Both steps for a row held in registers (register k = vector k*tpr + tx): on a replay h is parked
// in `park`, and re-read from it afterwards so that nothing has to stay in registers across the
// out-of-line replay; `replayed` tells the caller to refresh its own long-lived registers too.
template <int DT, int VPT>
__device__ __forceinline__ float resolve_row_m(uint4 (&h)[VPT], float lsum, float lw, int V, int n, float eps,
                                               int flags, RowRegSmem& sm, uint4* park, bool& replayed) {
  const int tx = threadIdx.x, tpr = blockDim.x, wpr = tpr >> 5;
  bool need;
  float m = decide_row<DT>(lsum, lw, n, eps, flags, sm, need);
  replayed = false;
  if (need) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int v = k * tpr + tx;
      if (v < V) park[v] = h[k];
    }
    if (wpr > 1)
      row_barrier(1 + threadIdx.y, tpr);
    else
      __syncwarp();
    m = replay_row<DT, ParkedRow>(ParkedRow{park}, V, n, eps, sm);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int v = k * tpr + tx;
      h[k] = v < V ? park[v] : make_uint4(0, 0, 0, 0);
    }
    replayed = true;
  }
  return m;
}

// Squares of one vector added to the tree-order sums; `weight` = n - 8 * (vector index).
template <int DT>
__device__ __forceinline__ void accumulate_vec_w(const uint4& h, float weight, float& lsum, float& lw) {
  const uint32_t w[4] = {h.x, h.y, h.z, h.w};
  float vs = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = unpack2<DT>(w[i]);
    vs = fmaf(f.x, f.x, vs);
    vs = fmaf(f.y, f.y, vs);
  }
  lsum += vs;
  lw = fmaf(vs, weight, lw);
}

// x / m correctly rounded to f32 in three instructions, for finite x and 2^-60 <= m <= 2^60 with
// r = RN(1 / m) (Markstein: q = RN(x r) is within an ulp, q m - x is exact in an FMA, one correction
// step lands on the rounded quotient; checked against the division for every pair of f16 values).
// The sign of a zero result is not defined by this sequence: callers take it from x.
__device__ __forceinline__ float quotient_by_reciprocal(float x, float m, float r) {
  const float q = __fmul_rn(x, r);
  const float t = __fmaf_rn(q, m, -x);
  return __fmaf_rn(-t, r, q);
}

// T(h / m) for the two f16 values of `w` (f32 quotient, then one rounding to f16, as crate `half`
// divides), sign bits taken from `w`: every quotient has the sign of its numerator, zeros included.
template <int DT>
__device__ __forceinline__ uint32_t quotient2_f16(uint32_t w, float m, float r) {
  const float2 hf = unpack2<DT>(w);
  const uint32_t q = pack2<DT>(quotient_by_reciprocal(hf.x, m, r), quotient_by_reciprocal(hf.y, m, r));
  return (q & 0x7FFF7FFFu) | (w & 0x80008000u);
}

// y = T(T(h / m) * alpha) for one vector; r = 1/m when fast_div (2^-60 <= m <= 2^60: bf16 multiplies by
// r, f16 uses the three-instruction quotient; a row with an infinity or a NaN has no such m).
// GUARD = false is for callers that know no element of the row is tiny and non-zero.
template <int DT, bool GUARD = true>
__device__ __forceinline__ uint4 rms_output_vec(const uint4& h, const uint4& alpha, float m, float r, bool fast_div) {
  const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
  const uint32_t aw[4] = {alpha.x, alpha.y, alpha.z, alpha.w};
  if (DT != kDtBF16 && fast_div)
    return make_uint4(mul2_rn<DT>(quotient2_f16<DT>(hw[0], m, r), aw[0]), mul2_rn<DT>(quotient2_f16<DT>(hw[1], m, r), aw[1]),
                      mul2_rn<DT>(quotient2_f16<DT>(hw[2], m, r), aw[2]), mul2_rn<DT>(quotient2_f16<DT>(hw[3], m, r), aw[3]));
  float q[8];
  if (fast_div) {
    float amin = 3.0e38f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 hf = unpack2<DT>(hw[i]);
      q[2 * i] = __fmul_rn(hf.x, r);
      q[2 * i + 1] = __fmul_rn(hf.y, r);
      if (GUARD) amin = fminf(amin, fminf(fabsf(q[2 * i]), fabsf(q[2 * i + 1])));
    }
    // below 2^-100 the bf16 result may be subnormal, where the margin argument does not hold:
    // recompute such elements with the exact quotient.  A vector with an exact zero also lands
    // here, but costs only the comparisons.
    if (GUARD && amin < 7.8886091e-31f) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 hf = unpack2<DT>(hw[i]);
        // exact zeros are already right; only tiny non-zero products need the division
        if (fabsf(q[2 * i]) < 7.8886091e-31f && q[2 * i] != 0.0f) q[2 * i] = __fdiv_rn(hf.x, m);
        if (fabsf(q[2 * i + 1]) < 7.8886091e-31f && q[2 * i + 1] != 0.0f) q[2 * i + 1] = __fdiv_rn(hf.y, m);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 hf = unpack2<DT>(hw[i]);
      q[2 * i] = __fdiv_rn(hf.x, m);
      q[2 * i + 1] = __fdiv_rn(hf.y, m);
    }
  }
  return make_uint4(mul2_rn<DT>(pack2<DT>(q[0], q[1]), aw[0]), mul2_rn<DT>(pack2<DT>(q[2], q[3]), aw[1]),
                    mul2_rn<DT>(pack2<DT>(q[4], q[5]), aw[2]), mul2_rn<DT>(pack2<DT>(q[6], q[7]), aw[3]));
}

// The common case of rms_output_vec only, for callers that have established it holds for the whole
// row: 2^-60 <= m <= 2^60 and, for bf16, no tiny non-zero element (quotient = product with r = 1/m;
// f16: the three-instruction quotient).  Kept apart so that hot loops carry nothing else.
template <int DT>
__device__ __forceinline__ uint4 rms_output_plain(const uint4& h, const uint4& alpha, float m, float r) {
  const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
  const uint32_t aw[4] = {alpha.x, alpha.y, alpha.z, alpha.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t q;
    if (DT == kDtBF16) {
      const float2 hf = unpack2<DT>(hw[i]);
      q = pack2<DT>(__fmul_rn(hf.x, r), __fmul_rn(hf.y, r));
    } else {
      q = quotient2_f16<DT>(hw[i], m, r);
    }
    o[i] = mul2_rn<DT>(q, aw[i]);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// The guarded form out of line, for rare rows: one copy of the code however often it is called.
template <int DT>
__device__ __noinline__ uint4 rms_output_rare(uint4 h, uint4 alpha, float m, float r, bool fast_div) {
  return rms_output_vec<DT, true>(h, alpha, m, r, fast_div);
}

// Same as rms_output_vec for a vector whose elements are already widened to f32 (hf).
template <int DT, bool GUARD>
__device__ __forceinline__ uint4 rms_output_floats(const float (&hf)[8], const uint4& alpha, float m, float r,
                                                   bool fast_div) {
  const uint32_t aw[4] = {alpha.x, alpha.y, alpha.z, alpha.w};
  float q[8];
  if (DT != kDtBF16 && fast_div) {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = copysignf(quotient_by_reciprocal(hf[i], m, r), hf[i]);
  } else if (fast_div) {
    float amin = 3.0e38f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q[i] = __fmul_rn(hf[i], r);
      if (GUARD) amin = fminf(amin, fabsf(q[i]));
    }
    if (GUARD && amin < 7.8886091e-31f) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (fabsf(q[i]) < 7.8886091e-31f && q[i] != 0.0f) q[i] = __fdiv_rn(hf[i], m);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(hf[i], m);
  }
  return make_uint4(mul2_rn<DT>(pack2<DT>(q[0], q[1]), aw[0]), mul2_rn<DT>(pack2<DT>(q[2], q[3]), aw[1]),
                    mul2_rn<DT>(pack2<DT>(q[4], q[5]), aw[2]), mul2_rn<DT>(pack2<DT>(q[6], q[7]), aw[3]));
}

// Widens a packed vector to f32 and adds its squares to the tree-order sums.
template <int DT>
__device__ __forceinline__ void widen_accumulate(const uint4& h, float weight, float (&hf)[8], float& lsum, float& lw) {
  const uint32_t w[4] = {h.x, h.y, h.z, h.w};
  float vs = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = unpack2<DT>(w[i]);
    hf[2 * i] = f.x;
    hf[2 * i + 1] = f.y;
    vs = fmaf(f.x, f.x, vs);
    vs = fmaf(f.y, f.y, vs);
  }
  lsum += vs;
  lw = fmaf(vs, weight, lw);
}

}  // namespace cb200
