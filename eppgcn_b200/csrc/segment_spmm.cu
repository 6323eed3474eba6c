// Edge-chunked neighbour aggregation for sm_100a, driven by a plan that is
// prepared once per edge list (forward: the CSR of the graph; backward: the
// compacted execution path).
//
// Work unit.  The edge list is cut into chunks of 64 consecutive edges,
// whatever rows they belong to.  A sub-warp of LPR lanes owns one chunk, a
// warp owns 32/LPR consecutive chunks ("a set").  Every sub-warp therefore has
// the same number of edges, every load slot is used, and a chunk costs
// eight rounds of eight independent 16-byte row loads per lane -- the group kernel
// (spmm.cu) pays one round per tail batch of every short group instead.
//
// Row boundaries come from the plan: one 64-bit word per chunk with a bit at
// every edge that starts a row, and the rank (index among the non-empty rows)
// of the row the chunk begins in.  While a lane adds up its columns it closes
// a row whenever it meets a start bit.  Rows that lie inside a chunk are
// stored plainly as they are closed.  The open ends of a chunk -- the piece of
// a row that began in an earlier chunk, and the last row, which may go on in
// the next chunk -- are passed from sub-warp to sub-warp with shuffles after
// the edge loop, so a row that stays inside one set is still stored exactly
// once, without atomics.  Only a row that crosses a set boundary is
// accumulated with vector atomics; the plan lists those rows (and the rows
// without edges), and a small kernel zeroes them first.  The result matrix is
// therefore written once, not zero-filled and written again.
//
// Source rows.  The kernel reads rows that already carry their source-side
// factor (the update step, or the backward's packing step, folds it in), 16
// bytes per lane; a row of up to 16 / 32 / 64 / 128 columns is covered by 4 /
// 8 / 16 / 32 lanes, wider rows take one launch per 128 columns.
#include <mutex>
#include <new>

#include "rowio.cuh"

struct eppgcn_segment_plan {
  // device arrays inside the caller's buffer
  unsigned long long *mask;   // [num_chunks] bit i: edge 64*k+i starts a row
  int *first_rank;            // [num_chunks] rank of the row that holds edge 64*k
  int *rows;                  // [num_ranks]  rank -> row id
  int *zero_rows;             // [num_zero]   rows the zeroing kernel clears
  int *counters;              // [0] num_ranks, [1] num_zero
  int *tile_sums;             // scan scratch
  int *row_flags;             // [num_rows] scratch of the id-list builder
  // host copies
  long long num_edges;
  int num_rows, num_chunks, groups, num_ranks, num_zero, identity, zero_all;
};

namespace epp {
namespace {

constexpr int kChunk = 64;            // edges per sub-warp chunk
constexpr int kPlanTile = 1024;       // chunks per block in the rank scan
#ifndef EPP_SEG_THREADS
#define EPP_SEG_THREADS 256
#endif
#ifndef EPP_SEG_MINB
#define EPP_SEG_MINB 3
#endif
constexpr int kSegThreads = EPP_SEG_THREADS;
constexpr int kSegMinBlocks = EPP_SEG_MINB;

struct SegArgs {
  float *out;
  long long out_ld;
  const float *src;               // rows of src_ld floats, 16-byte aligned, pre-scaled by the source factor
  long long src_ld;
  const int *col;                 // source row per edge, 16-byte aligned
  const unsigned long long *mask;
  const int *first_rank;
  const int *rows;                // NULL: rank == row
  const float *row_scale;         // destination-side factor per row id, or NULL
  long long num_edges;
  int num_chunks;
  int dim;                        // columns handled by this launch
  int ovec;
};

// Eight column ids of one chunk starting at p (16-byte aligned); `left` edges
// of the chunk remain, ids beyond them are not read.
__device__ __forceinline__ void load_ids(const int *p, int left, int (&c)[8]) {
  if (left >= 8) {
    const int4 a = __ldg(reinterpret_cast<const int4 *>(p));
    const int4 b = __ldg(reinterpret_cast<const int4 *>(p) + 1);
    c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) c[u] = u < left ? __ldg(p + u) : 0;
  }
}

__device__ __forceinline__ void add4(float (&acc)[4], const float4 &v) {
  acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
}

// Row id and destination-side factor of the row with rank `rank`.
__device__ __forceinline__ void row_of_rank(const SegArgs &a, int rank, int &row, float &scale) {
  row = a.rows ? __ldg(a.rows + rank) : rank;
  scale = a.row_scale ? __ldg(a.row_scale + row) : 1.f;
}

// The lane's four columns of a row sum, times `scale`, to `dst` (n <= 4 of
// them exist): a plain store, or an atomic add for a piece of a row that other
// warps add to as well.
template <int OV>
__device__ __forceinline__ void put4(float *dst, const float (&acc)[4], float scale, int n, bool atomic) {
  const float val[4] = {acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale};
  if (atomic) add_row<4>(dst, val, n, OV);
  else store_row<4>(dst, val, n, OV);
}

// The 64 (or, at the end of the list, fewer) edges of one chunk.  `bits` holds
// the row starts of the chunk without bit 0 (a start at the first edge closes
// nothing).  On return `acc` is the sum of the chunk's last piece, `head` the
// sum of the piece in front of the chunk's first start when the chunk began
// inside a row (`nseen` == 0 on entry), `cur` the rank of the last piece's row
// and `nseen` the number of starts met, the one at edge 0 included.
//
// A batch is eight edges.  Where a batch holds row starts, the per-edge step is
// branch-free: the running sum is parked in the lane's shared-memory slots
// (`stage`, slot i at stage[i * kSegThreads]) under a predicate and the sum
// restarts from the edge's row.  The parked sums are written out afterwards in
// a loop whose trip count is the same for the whole warp, so rows that close
// at different edges in different sub-warps are stored by the same
// instructions.  The row ids and factors of the rows that close in a batch are
// asked for together with the batch's source rows.
template <int LPR, int OV>
__device__ __forceinline__ void run_chunk(const SegArgs &a, const int *cp, int len, int trips,
                                          unsigned long long bits, bool has_cols, const char *glane,
                                          unsigned ld_bytes, float *out_lane, int n, int sub, int sl,
                                          unsigned sub_mask, float4 *stage, float (&acc)[4], float (&head)[4],
                                          int &cur, int &nseen) {
  constexpr int U = 8;                             // edges per batch: U row loads in flight per lane
  int c[U];
  load_ids(cp, len, c);
#pragma unroll 1
  for (int b = 0; b < trips; b += U) {
    float4 v[U];
    const int left = len - b;
    // Nothing is consumed in this loop, so U loads are in flight.  Ids past the end of the list are
    // 0 (row 0 is read and not added); lanes without columns read column 0 and never store.
#pragma unroll
    for (int u = 0; u < U; ++u)
      v[u] = __ldg(reinterpret_cast<const float4 *>(
          glane + static_cast<unsigned long long>(static_cast<unsigned>(c[u])) * ld_bytes));
    if (b + U < kChunk) load_ids(cp + b + U, left - U, c);      // ids of the next batch, behind the gathers
#ifdef EPP_SEG_NOCLOSE
    const unsigned bb = 0u;                        // timing experiment: rows are never closed inside a chunk
#else
    const unsigned bb = static_cast<unsigned>(bits >> b) & ((1u << U) - 1u);
#endif
    // One decision for the whole warp: the branch below holds warp-wide votes and shuffles.
    if (!__any_sync(kFull, bb != 0u || left < U)) {
#pragma unroll
      for (int u = 0; u < U; ++u) add4(acc, v[u]);
    } else {
      // The rows that close in this batch have ranks cur, cur+1, ...: lane j of the sub-warp asks
      // for the row id and factor of the j-th one (and of the (j+LPR)-th when a batch can close more
      // rows than the sub-warp has lanes).
      const int ncl = __popc(bb);
      int rw0 = 0, rw1 = 0;
      float sc0 = 1.f, sc1 = 1.f;
      if (sl < ncl) row_of_rank(a, cur + sl, rw0, sc0);
      if (LPR < U && sl + LPR < ncl) row_of_rank(a, cur + sl + LPR, rw1, sc1);
      if (left < U) {                              // end of the list: edges that do not exist add nothing
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (u >= left) v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      int cnt = 0;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const bool p = ((bb >> u) & 1u) != 0u;     // edge b+u starts a row: park the running sum, restart
        if (p) stage[cnt * kSegThreads] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        cnt += p ? 1 : 0;
        acc[0] = (p ? 0.f : acc[0]) + v[u].x;
        acc[1] = (p ? 0.f : acc[1]) + v[u].y;
        acc[2] = (p ? 0.f : acc[2]) + v[u].z;
        acc[3] = (p ? 0.f : acc[3]) + v[u].w;
      }
      const int most = __reduce_max_sync(kFull, ncl);
#pragma unroll 1
      for (int i = 0; i < most; ++i) {
        if (i < ncl) {
          const float4 s4 = stage[i * kSegThreads];
          const int from = (sub * LPR) + (i & (LPR - 1));
          const bool second = LPR < U && i >= LPR;
          const int row = __shfl_sync(sub_mask, second ? rw1 : rw0, from);
          const float scale = __shfl_sync(sub_mask, second ? sc1 : sc0, from);
          const float piece[4] = {s4.x, s4.y, s4.z, s4.w};
          if (i == 0 && nseen == 0) {              // the piece in front of the chunk's first start
#pragma unroll
            for (int q = 0; q < 4; ++q) head[q] = piece[q];
          } else if (has_cols) {
            put4<OV>(out_lane + static_cast<long long>(row) * a.out_ld, piece, scale, n, false);
          }
        }
      }
      cur += ncl;
      nseen += ncl;
    }
  }
}

template <int LPR, int OV>
__global__ void __launch_bounds__(kSegThreads, kSegMinBlocks) segment_spmm_kernel(const SegArgs a) {
  constexpr int G = kWarp / LPR;               // chunks per set
  __shared__ float4 s_stage[8 * kSegThreads];  // eight parked row sums per lane, slot-major
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const int fcol = sl * 4;
  const bool has_cols = fcol < a.dim;
  const int n = min(4, a.dim - fcol);          // columns of this lane that exist
  const unsigned sub_mask = (LPR == 32 ? kFull : ((1u << LPR) - 1u)) << (sub * LPR);
  float4 *stage = s_stage + threadIdx.x;
  const char *glane = reinterpret_cast<const char *>(a.src + (has_cols ? fcol : 0));
  const unsigned ld_bytes = static_cast<unsigned>(a.src_ld) * 4u;
  float *const out_lane = a.out + fcol;

  const int wpb = blockDim.x >> 5;
  const long long stride = static_cast<long long>(gridDim.x) * wpb;
  const long long nsets = (static_cast<long long>(a.num_chunks) + G - 1) / G;
  long long set = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5);
  if (set >= nsets) return;

  unsigned long long m_next = 0;
  int r_next = 0;
  {
    const long long k0 = set * G + sub;
    if (k0 < a.num_chunks) { m_next = __ldg(a.mask + k0); r_next = __ldg(a.first_rank + k0); }
  }
  for (; set < nsets; set += stride) {
    const long long k = set * G + sub;
    const unsigned long long m = m_next;
    int cur = r_next;
    {                                          // descriptors of this warp's next set
      const long long kn = (set + stride) * G + sub;
      m_next = 0; r_next = 0;
      if (kn < a.num_chunks) { m_next = __ldg(a.mask + kn); r_next = __ldg(a.first_rank + kn); }
    }
    const long long kq = (set + 1) * G;        // first chunk of the following set
    const bool next_starts = kq >= a.num_chunks || (__ldg(a.mask + kq) & 1ull) != 0ull;
    const bool valid = k < a.num_chunks;
    const long long e0 = k * kChunk;
    const int len = valid ? static_cast<int>(min(static_cast<long long>(kChunk), a.num_edges - e0)) : 0;
    const bool open_head = valid && (m & 1ull) == 0ull;           // the chunk begins inside a row
    int head_row = 0;
    float head_scale = 1.f;
    if (open_head) row_of_rank(a, cur, head_row, head_scale);     // needed after the edge loop; asked for now

    float acc[4] = {0.f, 0.f, 0.f, 0.f}, head[4] = {0.f, 0.f, 0.f, 0.f};
    int nseen = static_cast<int>(m & 1ull);
    const int trips = (set + 1) * G * kChunk <= a.num_edges ? kChunk : __reduce_max_sync(kFull, len);
    run_chunk<LPR, OV>(a, a.col + e0, len, trips, m & ~1ull, has_cols, glane, ld_bytes, out_lane, n, sub, sl,
                       sub_mask, stage, acc, head, cur, nseen);

    // -- open ends: hand the last piece of every chunk to the sub-warp on its right ------------------
    // `acc` is the carry this sub-warp sends on, with the row it belongs to and that row's factor;
    // carry_ext: the piece began before this set.
    const bool has_start = nseen > 0;
    int carry_row = head_row;
    float carry_scale = head_scale;
    if (has_start && len > 0) row_of_rank(a, cur, carry_row, carry_scale);
    bool carry_ext = !has_start;               // a chunk without a start passes on what it received (none yet)
    bool carry_valid = len > 0;
    if (sub == 0 && has_start && open_head && has_cols)
      put4<OV>(out_lane + static_cast<long long>(head_row) * a.out_ld, head, head_scale, n, true);
#pragma unroll 1
    for (int j = 1; j < G; ++j) {
      float inc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) inc[i] = __shfl_up_sync(kFull, acc[i], LPR);
      const int inc_row = __shfl_up_sync(kFull, carry_row, LPR);
      const float inc_scale = __shfl_up_sync(kFull, carry_scale, LPR);
      const int inc_flags = __shfl_up_sync(kFull, (carry_ext ? 1 : 0) | (carry_valid ? 2 : 0), LPR);
      const bool inc_ext = (inc_flags & 1) != 0, inc_valid = (inc_flags & 2) != 0;
      if (sub == j) {
        if (len == 0) {                        // past the end of the list: pass the carry through
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] = inc[i];
          carry_row = inc_row; carry_scale = inc_scale; carry_ext = inc_ext; carry_valid = inc_valid;
        } else if (has_start) {
          // either the row that ends in this chunk (earlier pieces + head), or, when the chunk begins
          // with a start, the row that ended exactly at the chunk boundary
          if (open_head) {
#pragma unroll
            for (int i = 0; i < 4; ++i) inc[i] = head[i] + (inc_valid ? inc[i] : 0.f);
          }
          const int row = open_head ? head_row : inc_row;
          const float scale = open_head ? head_scale : inc_scale;
          const bool atomic = open_head ? (inc_ext || !inc_valid) : inc_ext;
          if ((open_head || inc_valid) && has_cols)
            put4<OV>(out_lane + static_cast<long long>(row) * a.out_ld, inc, scale, n, atomic);
        } else {                               // the whole chunk lies inside one row
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += inc_valid ? inc[i] : 0.f;
          if (inc_valid) { carry_row = inc_row; carry_scale = inc_scale; }
          carry_ext = inc_valid ? inc_ext : true;
        }
      }
    }
    if (sub == G - 1 && carry_valid && has_cols)
      put4<OV>(out_lane + static_cast<long long>(carry_row) * a.out_ld, acc, carry_scale, n,
               carry_ext || !next_starts);
  }
}

// Clears the rows the plan lists (rows without edges and rows that are
// accumulated with atomics), W floats per store.
template <int W>
__global__ void __launch_bounds__(256) zero_listed_rows_kernel(float *out, long long out_ld, int dim,
                                                               const int *__restrict__ rows, int count) {
  const int per_row = (dim + W - 1) / W;
  const long long total = static_cast<long long>(count) * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % per_row) * W;
    float *p = out + static_cast<long long>(__ldg(rows + i / per_row)) * out_ld + c;
    if constexpr (W == 4) *reinterpret_cast<float4 *>(p) = make_float4(0.f, 0.f, 0.f, 0.f);
    else if constexpr (W == 2) *reinterpret_cast<float2 *>(p) = make_float2(0.f, 0.f);
    else *p = 0.f;
  }
}

// ---------------------------------------------------------------------------
// Plan preparation (one-time per edge list)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void append_row(int *list, int *counter, int row) { list[atomicAdd(counter, 1)] = row; }

// CSR input: one thread per row sets the row's start bit and lists the row for
// zeroing when it has no edges or crosses a set boundary (set_edges edges).
__global__ void __launch_bounds__(256) plan_mark_csr_kernel(const int *__restrict__ row_ptr, int num_rows,
                                                            int set_edges, unsigned long long *mask,
                                                            int *zero_rows, int *counters) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= num_rows) return;
  const int beg = __ldg(row_ptr + r), end = __ldg(row_ptr + r + 1);
  if (end > beg) {
    atomicOr(mask + (beg >> 6), 1ull << (beg & 63));
    if (beg / set_edges != (end - 1) / set_edges) append_row(zero_rows, counters + 1, r);
  } else {
    append_row(zero_rows, counters + 1, r);
  }
}

// Row-id-per-edge input (the compacted path, sorted by row): one thread per
// edge; a warp writes one 32-bit half of a mask word.  row_flags: bit 0 the
// row has edges, bit 1 it crosses a set boundary.
__global__ void __launch_bounds__(256) plan_mark_ids_kernel(const int *__restrict__ ids, long long num_edges,
                                                            int set_edges, unsigned *mask32, int *row_flags) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  bool start = false;
  if (e < num_edges) {
    const int r = __ldg(ids + e);
    const int prev = e > 0 ? __ldg(ids + e - 1) : -1;
    start = e == 0 || prev != r;
    if (start) atomicOr(row_flags + r, 1);
    else if (e % set_edges == 0) atomicOr(row_flags + r, 2);
  }
  const unsigned b = __ballot_sync(kFull, start);
  if ((threadIdx.x & 31) == 0 && e < ((num_edges + 63) / 64) * 64) mask32[e >> 5] = b;
}

__global__ void __launch_bounds__(256) plan_zero_list_kernel(const int *__restrict__ row_flags, int num_rows,
                                                             int *zero_rows, int *counters) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= num_rows) return;
  const int f = row_flags[r];
  if (!(f & 1) || (f & 2)) append_row(zero_rows, counters + 1, r);
}

// Rank scan, pass 1: row starts per tile of kPlanTile chunks.
__global__ void __launch_bounds__(kPlanTile) plan_tile_counts_kernel(const unsigned long long *__restrict__ mask,
                                                                     int num_chunks, int *tile_sums) {
  __shared__ int s_w[32];
  const int k = blockIdx.x * kPlanTile + threadIdx.x;
  int c = k < num_chunks ? __popcll(mask[k]) : 0;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) c += __shfl_xor_sync(kFull, c, off);
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    int t = s_w[threadIdx.x];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) t += __shfl_xor_sync(kFull, t, off);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = t;
  }
}

// Pass 2: exclusive scan of the tile sums by one block.
__global__ void __launch_bounds__(1024) plan_scan_tiles_kernel(int *tile_sums, int num_tiles) {
  __shared__ int s_w[33];
  __shared__ int s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < num_tiles; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < num_tiles ? tile_sums[i] : 0;
    int s = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(kFull, s, off);
      if (lane >= off) s += t;
    }
    if (lane == 31) s_w[warp] = s;
    __syncthreads();
    if (warp == 0) {
      const int w = s_w[lane];
      int ws = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(kFull, ws, off);
        if (lane >= off) ws += t;
      }
      s_w[lane] = ws - w;
      if (lane == 31) s_w[32] = ws;
    }
    __syncthreads();
    if (i < num_tiles) tile_sums[i] = s_carry + s_w[warp] + s - v;
    __syncthreads();
    if (threadIdx.x == 0) s_carry += s_w[32];
    __syncthreads();
  }
}

// Pass 3: rank of the row each chunk begins in; the last chunk stores the
// number of non-empty rows.
__global__ void __launch_bounds__(kPlanTile) plan_ranks_kernel(const unsigned long long *__restrict__ mask,
                                                               int num_chunks, const int *__restrict__ tile_sums,
                                                               int *first_rank, int *counters) {
  __shared__ int s_w[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k = blockIdx.x * kPlanTile + threadIdx.x;
  const unsigned long long m = k < num_chunks ? mask[k] : 0ull;
  const int c = __popcll(m);
  int s = c;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(kFull, s, off);
    if (lane >= off) s += t;
  }
  if (lane == 31) s_w[warp] = s;
  __syncthreads();
  if (warp == 0) {
    const int w = s_w[lane];
    int ws = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(kFull, ws, off);
      if (lane >= off) ws += t;
    }
    s_w[lane] = ws - w;
  }
  __syncthreads();
  const int ex = tile_sums[blockIdx.x] + s_w[warp] + s - c;      // starts before this chunk
  if (k < num_chunks) {
    first_rank[k] = ex + static_cast<int>(m & 1ull) - 1;
    if (k == num_chunks - 1) counters[0] = ex + c;
  }
}

__device__ __forceinline__ int rank_of_start(const unsigned long long *mask, const int *first_rank, long long e) {
  const long long k = e >> 6;
  const unsigned long long m = mask[k];
  const int before = first_rank[k] + 1 - static_cast<int>(m & 1ull);
  return before + __popcll(m & ((1ull << (e & 63)) - 1ull));
}

__global__ void __launch_bounds__(256) plan_rows_csr_kernel(const int *__restrict__ row_ptr, int num_rows,
                                                            const unsigned long long *__restrict__ mask,
                                                            const int *__restrict__ first_rank, int *rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= num_rows) return;
  const int beg = __ldg(row_ptr + r), end = __ldg(row_ptr + r + 1);
  if (end > beg) rows[rank_of_start(mask, first_rank, beg)] = r;
}

__global__ void __launch_bounds__(256) plan_rows_ids_kernel(const int *__restrict__ ids, long long num_edges,
                                                            const unsigned long long *__restrict__ mask,
                                                            const int *__restrict__ first_rank, int *rows) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= num_edges) return;
  if ((mask[e >> 6] >> (e & 63)) & 1ull) rows[rank_of_start(mask, first_rank, e)] = __ldg(ids + e);
}

int lanes_for_dim(int dim) {            // lanes per row: four columns per lane, at most 128 columns per launch
  if (dim <= 16) return 4;
  if (dim <= 32) return 8;
  if (dim <= 64) return 16;
  return 32;
}

size_t round256(size_t b) { return (b + 255) / 256 * 256; }

struct PlanLayout {
  size_t mask, first_rank, rows, zero_rows, row_flags, tile_sums, total;
};
PlanLayout plan_layout(long long num_edges, int num_rows) {
  const size_t chunks = static_cast<size_t>((num_edges + kChunk - 1) / kChunk);
  const size_t tiles = (chunks + kPlanTile - 1) / kPlanTile + 1;
  PlanLayout l{};
  size_t off = 256;                                     // counters
  l.mask = off;       off += round256(8 * (chunks + 1));
  l.first_rank = off; off += round256(4 * (chunks + 1));
  l.rows = off;       off += round256(4 * (static_cast<size_t>(num_rows) + 1));
  l.zero_rows = off;  off += round256(4 * (static_cast<size_t>(num_rows) + 1));
  l.row_flags = off;  off += round256(4 * (static_cast<size_t>(num_rows) + 1));
  l.tile_sums = off;  off += round256(4 * tiles);
  l.total = off;
  return l;
}

}  // namespace
}  // namespace epp

using namespace epp;

namespace {

int plan_alloc(eppgcn_segment_plan **plan, void *dev_buf, size_t dev_bytes, long long num_edges, int num_rows,
               int dim) {
  const PlanLayout l = plan_layout(num_edges, num_rows);
  if (dev_bytes < l.total) {
    set_error("plan buffer too small: %zu bytes given, %zu needed", dev_bytes, l.total);
    return EPP_ERR_BAD_ARG;
  }
  eppgcn_segment_plan *p = new (std::nothrow) eppgcn_segment_plan();
  if (!p) {
    set_error("out of host memory");
    return EPP_ERR_BAD_ARG;
  }
  char *base = static_cast<char *>(dev_buf);
  p->counters = reinterpret_cast<int *>(base);
  p->mask = reinterpret_cast<unsigned long long *>(base + l.mask);
  p->first_rank = reinterpret_cast<int *>(base + l.first_rank);
  p->rows = reinterpret_cast<int *>(base + l.rows);
  p->zero_rows = reinterpret_cast<int *>(base + l.zero_rows);
  p->row_flags = reinterpret_cast<int *>(base + l.row_flags);
  p->tile_sums = reinterpret_cast<int *>(base + l.tile_sums);
  p->num_edges = num_edges;
  p->num_rows = num_rows;
  p->num_chunks = static_cast<int>((num_edges + kChunk - 1) / kChunk);
  p->groups = kWarp / lanes_for_dim(dim > 128 ? 128 : dim);
  p->num_ranks = p->num_zero = p->identity = p->zero_all = 0;
  *plan = p;
  return EPP_OK;
}

// Scan of the start bits and read-back of the two counts (synchronises `s`).
int plan_finish(eppgcn_segment_plan *p, bool from_csr, cudaStream_t s) {
  const int tiles = (p->num_chunks + kPlanTile - 1) / kPlanTile;
  if (p->num_chunks > 0) {
    plan_tile_counts_kernel<<<tiles, kPlanTile, 0, s>>>(p->mask, p->num_chunks, p->tile_sums);
    EPP_CHECK_LAUNCH("plan_tile_counts_kernel");
    plan_scan_tiles_kernel<<<1, 1024, 0, s>>>(p->tile_sums, tiles);
    EPP_CHECK_LAUNCH("plan_scan_tiles_kernel");
    plan_ranks_kernel<<<tiles, kPlanTile, 0, s>>>(p->mask, p->num_chunks, p->tile_sums, p->first_rank, p->counters);
    EPP_CHECK_LAUNCH("plan_ranks_kernel");
  }
  (void)from_csr;
  return EPP_OK;
}

int plan_read_counts(eppgcn_segment_plan *p, bool from_csr, cudaStream_t s) {
  int host[2] = {0, 0};
  EPP_CUDA_TRY(cudaMemcpyAsync(host, p->counters, sizeof(host), cudaMemcpyDeviceToHost, s));
  EPP_CUDA_TRY(cudaStreamSynchronize(s));
  p->num_ranks = host[0];
  p->num_zero = host[1];
  p->identity = from_csr && p->num_ranks == p->num_rows;
  p->zero_all = p->num_zero > p->num_rows / 2;     // mostly empty result: one memset beats a long list
  return EPP_OK;
}

template <int LPR, int OV>
int launch_segments(const SegArgs &a, cudaStream_t s) {
  constexpr int G = kWarp / LPR;
  int num_sms = 0;
  if (const int rc = device_sm_count(&num_sms); rc != EPP_OK) return rc;
  const long long nsets = ceil_div_ll(a.num_chunks, G);
  long long blocks = ceil_div_ll(nsets, kSegThreads / kWarp);
  const long long cap = static_cast<long long>(num_sms) * kSegMinBlocks;
  if (blocks > cap) blocks = cap;
  segment_spmm_kernel<LPR, OV><<<static_cast<unsigned>(blocks), kSegThreads, 0, s>>>(a);
  EPP_CHECK_LAUNCH("segment_spmm_kernel");
  return EPP_OK;
}

template <int LPR>
int launch_by_store(const SegArgs &a, cudaStream_t s) {
  if (a.ovec == 4) return launch_segments<LPR, 4>(a, s);
  if (a.ovec == 2) return launch_segments<LPR, 2>(a, s);
  return launch_segments<LPR, 1>(a, s);
}

// The plan fixes the lanes per row: its list of cleared rows belongs to that set size.
int launch_by_width(const SegArgs &a, int lanes, cudaStream_t s) {
  if (lanes == 4) return launch_by_store<4>(a, s);
  if (lanes == 8) return launch_by_store<8>(a, s);
  if (lanes == 16) return launch_by_store<16>(a, s);
  return launch_by_store<32>(a, s);
}

}  // namespace

EPP_EXPORT size_t eppgcn_segment_plan_bytes(long long num_edges, int num_rows) {
  if (num_edges < 0 || num_rows < 0) return 0;
  return plan_layout(num_edges, num_rows).total;
}

EPP_EXPORT int eppgcn_segment_plan_from_csr(eppgcn_segment_plan **plan, void *dev_buf, size_t dev_bytes,
                                            const int *row_ptr, int num_rows, long long num_edges, int dim,
                                            void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan && dev_buf && num_rows >= 0 && num_edges >= 0 && dim >= 1, "bad argument");
  EPP_REQUIRE(num_edges < (1LL << 31), "edge count exceeds int32");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(dev_buf) % 256 == 0, "plan buffer must be 256-byte aligned");
  EPP_REQUIRE(num_rows == 0 || row_ptr, "null pointer");
  if (const int rc = plan_alloc(plan, dev_buf, dev_bytes, num_edges, num_rows, dim); rc != EPP_OK) return rc;
  eppgcn_segment_plan *p = *plan;
  const PlanLayout l = plan_layout(num_edges, num_rows);
  EPP_CUDA_TRY(cudaMemsetAsync(dev_buf, 0, l.first_rank, s));            // counters and start bits
  if (num_rows > 0) {
    const int blocks = static_cast<int>(ceil_div_ll(num_rows, 256));
    plan_mark_csr_kernel<<<blocks, 256, 0, s>>>(row_ptr, num_rows, p->groups * kChunk, p->mask, p->zero_rows,
                                                 p->counters);
    EPP_CHECK_LAUNCH("plan_mark_csr_kernel");
    if (const int rc = plan_finish(p, true, s); rc != EPP_OK) return rc;
    if (p->num_chunks > 0) {
      plan_rows_csr_kernel<<<blocks, 256, 0, s>>>(row_ptr, num_rows, p->mask, p->first_rank, p->rows);
      EPP_CHECK_LAUNCH("plan_rows_csr_kernel");
    }
  }
  return plan_read_counts(p, true, s);
}

EPP_EXPORT int eppgcn_segment_plan_from_ids(eppgcn_segment_plan **plan, void *dev_buf, size_t dev_bytes,
                                            const int *ids, long long num_edges, int num_rows, int dim,
                                            void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan && dev_buf && num_rows >= 0 && num_edges >= 0 && dim >= 1, "bad argument");
  EPP_REQUIRE(num_edges < (1LL << 31), "edge count exceeds int32");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(dev_buf) % 256 == 0, "plan buffer must be 256-byte aligned");
  EPP_REQUIRE(num_edges == 0 || ids, "null pointer");
  if (const int rc = plan_alloc(plan, dev_buf, dev_bytes, num_edges, num_rows, dim); rc != EPP_OK) return rc;
  eppgcn_segment_plan *p = *plan;
  const PlanLayout l = plan_layout(num_edges, num_rows);
  EPP_CUDA_TRY(cudaMemsetAsync(dev_buf, 0, l.first_rank, s));
  EPP_CUDA_TRY(cudaMemsetAsync(p->row_flags, 0, sizeof(int) * (static_cast<size_t>(num_rows) + 1), s));
  if (num_edges > 0) {
    const long long covered = static_cast<long long>(p->num_chunks) * kChunk;
    const unsigned blocks = static_cast<unsigned>(ceil_div_ll(covered, 256));
    plan_mark_ids_kernel<<<blocks, 256, 0, s>>>(ids, num_edges, p->groups * kChunk,
                                                 reinterpret_cast<unsigned *>(p->mask), p->row_flags);
    EPP_CHECK_LAUNCH("plan_mark_ids_kernel");
    if (const int rc = plan_finish(p, false, s); rc != EPP_OK) return rc;
    plan_rows_ids_kernel<<<blocks, 256, 0, s>>>(ids, num_edges, p->mask, p->first_rank, p->rows);
    EPP_CHECK_LAUNCH("plan_rows_ids_kernel");
  }
  if (num_rows > 0) {
    plan_zero_list_kernel<<<static_cast<unsigned>(ceil_div_ll(num_rows, 256)), 256, 0, s>>>(p->row_flags, num_rows,
                                                                                             p->zero_rows, p->counters);
    EPP_CHECK_LAUNCH("plan_zero_list_kernel");
  }
  return plan_read_counts(p, false, s);
}

EPP_EXPORT void eppgcn_segment_plan_destroy(eppgcn_segment_plan *plan) { delete plan; }

EPP_EXPORT int eppgcn_segment_plan_info(const eppgcn_segment_plan *plan, long long *out8) {
  EPP_REQUIRE(plan && out8, "null pointer");
  out8[0] = plan->num_edges; out8[1] = plan->num_rows; out8[2] = plan->num_chunks; out8[3] = plan->groups;
  out8[4] = plan->num_ranks; out8[5] = plan->num_zero; out8[6] = plan->identity; out8[7] = plan->zero_all;
  return EPP_OK;
}

EPP_EXPORT int eppgcn_spmm_segments(float *out, long long out_ld, const float *src, long long src_ld,
                                    const int *col_idx, const eppgcn_segment_plan *plan, const float *row_scale,
                                    int dim, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan, "null plan");
  EPP_REQUIRE(dim >= 1, "dim < 1");
  EPP_REQUIRE(out_ld == 0 || out_ld >= dim, "out_ld must be 0 or >= dim");
  const int n = plan->num_rows;
  if (n == 0) return EPP_OK;
  EPP_REQUIRE(out, "null pointer");
  if (out_ld == 0) out_ld = dim;
  EPP_REQUIRE(kWarp / lanes_for_dim(dim > 128 ? 128 : dim) == plan->groups,
              "the plan was prepared for another row width class (<= 16, <= 32, <= 64, wider)");
  int ovec = 1;
  if (out_ld % 4 == 0 && aligned(out, 16)) ovec = 4;
  else if (out_ld % 2 == 0 && aligned(out, 8)) ovec = 2;
  // rows without edges and rows that are summed with atomics start from zero
  if (plan->zero_all) {
    if (out_ld == dim) EPP_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(n) * dim, s));
    else if (const int rc = zero_column_block(out, out_ld, dim, n, s); rc != EPP_OK) return rc;
  } else if (plan->num_zero > 0) {
    const int w = (ovec == 4 && dim % 4 == 0) ? 4 : (ovec >= 2 && dim % 2 == 0) ? 2 : 1;
    const long long total = static_cast<long long>(plan->num_zero) * ((dim + w - 1) / w);
    long long blocks = ceil_div_ll(total, 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    const unsigned g = static_cast<unsigned>(blocks);
    if (w == 4) zero_listed_rows_kernel<4><<<g, 256, 0, s>>>(out, out_ld, dim, plan->zero_rows, plan->num_zero);
    else if (w == 2) zero_listed_rows_kernel<2><<<g, 256, 0, s>>>(out, out_ld, dim, plan->zero_rows, plan->num_zero);
    else zero_listed_rows_kernel<1><<<g, 256, 0, s>>>(out, out_ld, dim, plan->zero_rows, plan->num_zero);
    EPP_CHECK_LAUNCH("zero_listed_rows_kernel");
  }
  if (plan->num_edges == 0) return EPP_OK;
  EPP_REQUIRE(src && col_idx, "null pointer");
  EPP_REQUIRE(src_ld % 4 == 0 && src_ld >= (dim + 3) / 4 * 4 && src_ld <= 0x3fffffffLL && aligned(src, 16),
              "source rows must be 16-byte aligned and padded to a multiple of 4 floats");
  EPP_REQUIRE(aligned(col_idx, 16), "col_idx must be 16-byte aligned");
  for (int col0 = 0; col0 < dim; col0 += 128) {          // one launch unless the row is wider than 128
    SegArgs a{};
    a.out = out + col0; a.out_ld = out_ld; a.src = src + col0; a.src_ld = src_ld; a.col = col_idx;
    a.mask = plan->mask; a.first_rank = plan->first_rank; a.rows = plan->identity ? nullptr : plan->rows;
    a.row_scale = row_scale; a.num_edges = plan->num_edges; a.num_chunks = plan->num_chunks;
    a.dim = dim - col0 < 128 ? dim - col0 : 128; a.ovec = ovec;
    const int lanes = kWarp / plan->groups;
    const int rc = launch_by_width(a, lanes, s);
    if (rc != EPP_OK) return rc;
  }
  return EPP_OK;
}
