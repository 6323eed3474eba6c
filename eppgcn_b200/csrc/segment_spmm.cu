// Edge-chunked neighbour aggregation for sm_100a, driven by a plan that is
// prepared once per edge list (forward: the CSR of the graph; backward: the
// compacted execution path).
//
// Work unit.  The edge list is cut into chunks of 64 consecutive edges,
// whatever rows they belong to.  A sub-warp of LPR lanes owns one chunk, a
// warp owns 32/LPR consecutive chunks ("a set").  Every sub-warp therefore has
// the same number of edges, every load slot is used, and a chunk costs
// 64/U rounds of U independent 16-byte row loads per lane -- the group kernel
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
// bytes per lane and tile.  Optionally the first `hub_rows` rows of the source
// matrix are copied into shared memory when a block starts and served from
// there: with a producer that places the most referenced rows first, the share
// of gathers that leave the SM shrinks by the hubs' share of the edges.
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
#ifndef EPP_HUB_THREADS
#define EPP_HUB_THREADS 768
#endif
constexpr int kSegThreads = EPP_SEG_THREADS;
constexpr int kSegMinBlocks = EPP_SEG_MINB;
constexpr int kHubThreads = EPP_HUB_THREADS;
constexpr int kMaxHubBytes = 200 * 1024;

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
  int hub_rows;
};

// U column ids of one chunk starting at p (16-byte aligned when FULL).
template <int U, bool FULL>
__device__ __forceinline__ void load_ids(const int *p, int left, int (&c)[U]) {
  if constexpr (FULL && U == 8) {
    const int4 a = __ldg(reinterpret_cast<const int4 *>(p));
    const int4 b = __ldg(reinterpret_cast<const int4 *>(p) + 1);
    c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
  } else if constexpr (FULL && U == 4) {
    const int4 a = __ldg(reinterpret_cast<const int4 *>(p));
    c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w;
  } else if constexpr (FULL && U == 2) {
    const int2 a = __ldg(reinterpret_cast<const int2 *>(p));
    c[0] = a.x; c[1] = a.y;
  } else {
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = (FULL || u < left) ? __ldg(p + u) : 0;
  }
}

// Issues the row loads of one batch; nothing is consumed here, so all
// U*T 16-byte loads of the lane are in flight together.
template <int LPR, int T, int U, bool FULL, bool HUB>
__device__ __forceinline__ void gather_rows(const int (&c)[U], int left, unsigned tiles, const char *glane,
                                            unsigned ld_bytes, const float *hlane, int hub_ld, int hub_rows,
                                            float4 (&v)[U][T]) {
  constexpr unsigned kTileBytes = 16u * LPR;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (FULL || u < left) {
      const unsigned cu = static_cast<unsigned>(c[u]);
      if (HUB && cu < static_cast<unsigned>(hub_rows)) {
        const float *p = hlane + cu * hub_ld;
#pragma unroll
        for (int k = 0; k < T; ++k)
          v[u][k] = ((tiles >> k) & 1u) ? *reinterpret_cast<const float4 *>(p + k * 4 * LPR)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        const char *p = glane + static_cast<unsigned long long>(cu) * ld_bytes;
#pragma unroll
        for (int k = 0; k < T; ++k)
          v[u][k] = ((tiles >> k) & 1u) ? __ldg(reinterpret_cast<const float4 *>(p + k * kTileBytes))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
#pragma unroll
      for (int k = 0; k < T; ++k) v[u][k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

template <int T>
__device__ __forceinline__ void add4(float (&acc)[T][4], const float4 (&v)[T]) {
#pragma unroll
  for (int k = 0; k < T; ++k) {
    acc[k][0] += v[k].x; acc[k][1] += v[k].y; acc[k][2] += v[k].z; acc[k][3] += v[k].w;
  }
}

// Writes one finished (or partial, when `atomic`) row sum: the lane's tiles,
// times the destination-side factor of the row.
template <int LPR, int T>
__device__ __forceinline__ void flush_row(const SegArgs &a, int rank, const float (&acc)[T][4], bool atomic,
                                          int fcol, unsigned tiles) {
  if (!tiles) return;
  const int row = a.rows ? __ldg(a.rows + rank) : rank;
  const float s = a.row_scale ? __ldg(a.row_scale + row) : 1.f;
  float *dst = a.out + static_cast<long long>(row) * a.out_ld + fcol;
#pragma unroll
  for (int k = 0; k < T; ++k) {
    if ((tiles >> k) & 1u) {
      const int n = min(4, a.dim - (fcol + k * 4 * LPR));
      const float val[4] = {acc[k][0] * s, acc[k][1] * s, acc[k][2] * s, acc[k][3] * s};
      if (atomic) add_row<4>(dst + k * 4 * LPR, val, n, a.ovec);
      else store_row<4>(dst + k * 4 * LPR, val, n, a.ovec);
    }
  }
}

// The 64 (or, in the last set of the list, fewer) edges of one chunk.  `bits`
// holds the row starts of the chunk without bit 0 (a start at the first edge
// closes nothing).  On return `acc` is the sum of the chunk's last row piece,
// `head` the sum of the piece before the first start (only meaningful when the
// chunk began inside a row), `cur` the rank of the last piece's row and
// `nseen` the number of starts met, the one at edge 0 included.
template <int LPR, int T, int U, bool FULL, bool HUB>
__device__ __forceinline__ void run_chunk(const SegArgs &a, const int *cp, int len, int maxlen,
                                          unsigned long long bits, unsigned tiles, const char *glane,
                                          unsigned ld_bytes, const float *hlane, int fcol,
                                          float (&acc)[T][4], float (&head)[T][4], int &cur, int &nseen) {
  int c[U], cn[U];
  load_ids<U, FULL>(cp, len, c);
#pragma unroll
  for (int u = 0; u < U; ++u) cn[u] = c[u];
  const int trips = FULL ? kChunk : maxlen;
#pragma unroll 1
  for (int b = 0; b < trips; b += U) {
    float4 v[U][T];
    const int left = len - b;
    gather_rows<LPR, T, U, FULL, HUB>(c, left, tiles, glane, ld_bytes, hlane, static_cast<int>(a.src_ld),
                                      a.hub_rows, v);
    if (b + U < kChunk) load_ids<U, FULL>(cp + b + U, left - U, cn);   // ids of the next batch, behind the gathers
    const unsigned bb = static_cast<unsigned>(bits >> b) & ((1u << U) - 1u);
    if (bb == 0u) {
#pragma unroll
      for (int u = 0; u < U; ++u) add4<T>(acc, v[u]);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if ((bb >> u) & 1u) {                      // edge b+u starts a row: close the running piece
          if (nseen == 0) {
#pragma unroll
            for (int k = 0; k < T; ++k)
#pragma unroll
              for (int i = 0; i < 4; ++i) head[k][i] = acc[k][i];
          } else {
            flush_row<LPR, T>(a, cur, acc, false, fcol, tiles);
          }
#pragma unroll
          for (int k = 0; k < T; ++k)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[k][i] = 0.f;
          ++cur;
          ++nseen;
        }
        add4<T>(acc, v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = cn[u];
  }
}

template <int LPR, int T, bool HUB>
__global__ void __launch_bounds__(HUB ? kHubThreads : kSegThreads, HUB ? 1 : kSegMinBlocks)
segment_spmm_kernel(const SegArgs a) {
  constexpr int G = kWarp / LPR;               // chunks per set
  constexpr int U = T >= 8 ? 1 : 8 / T;        // edges per batch: U*T row loads in flight per lane
  extern __shared__ __align__(16) float s_hub[];
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const int fcol = sl * 4;
  unsigned tiles = 0;
#pragma unroll
  for (int k = 0; k < T; ++k)
    if (fcol + k * 4 * LPR < a.dim) tiles |= 1u << k;

  if (HUB) {                                   // the hub rows, once per block
    const int n4 = static_cast<int>(a.hub_rows * a.src_ld / 4);
    const float4 *g4 = reinterpret_cast<const float4 *>(a.src);
    float4 *s4 = reinterpret_cast<float4 *>(s_hub);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) s4[i] = __ldg(g4 + i);
    __syncthreads();
  }
  const char *glane = reinterpret_cast<const char *>(a.src + fcol);
  const float *hlane = s_hub + fcol;
  const unsigned ld_bytes = static_cast<unsigned>(a.src_ld) * 4u;

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
    const bool full = (set + 1) * G * kChunk <= a.num_edges;      // warp-uniform
    const bool open_head = valid && (m & 1ull) == 0ull;           // the chunk begins inside a row
    const int head_rank = cur;

    float acc[T][4], head[T][4];
#pragma unroll
    for (int k2 = 0; k2 < T; ++k2)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[k2][i] = 0.f; head[k2][i] = 0.f; }
    int nseen = static_cast<int>(m & 1ull);
    const unsigned long long bits = m & ~1ull;
    const int *cp = a.col + e0;
    if (full) {
      run_chunk<LPR, T, U, true, HUB>(a, cp, kChunk, kChunk, bits, tiles, glane, ld_bytes, hlane, fcol,
                                      acc, head, cur, nseen);
    } else {
      const int maxlen = __reduce_max_sync(kFull, len);
      run_chunk<LPR, T, U, false, HUB>(a, cp, len, maxlen, bits, tiles, glane, ld_bytes, hlane, fcol,
                                       acc, head, cur, nseen);
    }

    // -- open ends: hand the last piece of every chunk to the sub-warp on its right ------------------
    const bool has_start = nseen > 0;
    // `acc` now is the carry this sub-warp sends on; carry_ext: the piece began before this set
    int carry_rank = cur;
    bool carry_ext = !has_start;               // a chunk without a start passes on what it received (none yet)
    bool carry_valid = len > 0;
    if (sub == 0 && has_start && open_head) flush_row<LPR, T>(a, head_rank, head, true, fcol, tiles);
#pragma unroll
    for (int j = 1; j < G; ++j) {
      float inc[T][4];
#pragma unroll
      for (int k2 = 0; k2 < T; ++k2)
#pragma unroll
        for (int i = 0; i < 4; ++i) inc[k2][i] = __shfl_up_sync(kFull, acc[k2][i], LPR);
      const int inc_rank = __shfl_up_sync(kFull, carry_rank, LPR);
      const int inc_flags = __shfl_up_sync(kFull, (carry_ext ? 1 : 0) | (carry_valid ? 2 : 0), LPR);
      const bool inc_ext = (inc_flags & 1) != 0, inc_valid = (inc_flags & 2) != 0;
      if (sub == j) {
        if (len == 0) {                        // past the end of the list: pass the carry through
#pragma unroll
          for (int k2 = 0; k2 < T; ++k2)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[k2][i] = inc[k2][i];
          carry_rank = inc_rank; carry_ext = inc_ext; carry_valid = inc_valid;
        } else if (has_start) {
          if (open_head) {                     // the row that ends in this chunk: earlier pieces + head
#pragma unroll
            for (int k2 = 0; k2 < T; ++k2)
#pragma unroll
              for (int i = 0; i < 4; ++i) head[k2][i] += inc_valid ? inc[k2][i] : 0.f;
            flush_row<LPR, T>(a, head_rank, head, inc_ext || !inc_valid, fcol, tiles);
          } else if (inc_valid) {              // the row ended exactly at the chunk boundary
            flush_row<LPR, T>(a, inc_rank, inc, inc_ext, fcol, tiles);
          }
        } else {                               // the whole chunk lies inside one row
#pragma unroll
          for (int k2 = 0; k2 < T; ++k2)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[k2][i] += inc_valid ? inc[k2][i] : 0.f;
          carry_rank = inc_valid ? inc_rank : head_rank;
          carry_ext = inc_valid ? inc_ext : true;
        }
      }
    }
    if (sub == G - 1 && carry_valid) flush_row<LPR, T>(a, carry_rank, acc, carry_ext || !next_starts, fcol, tiles);
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

int lanes_for_dim(int dim) {            // lanes per row of the kernel shape that serves `dim` columns
  if (dim <= 32) return 4;
  if (dim <= 64) return 8;
  return 16;
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

template <int LPR, int T, bool HUB>
int launch_segments(const SegArgs &a, int hub_bytes, cudaStream_t s) {
  constexpr int G = kWarp / LPR;
  static SmemOptIn memo;
  int num_sms = 0;
  if (const int rc = device_sm_count(&num_sms); rc != EPP_OK) return rc;
  const int threads = HUB ? kHubThreads : kSegThreads;
  const int per_sm = HUB ? 1 : kSegMinBlocks;
  if (HUB)
    if (const int rc = smem_opt_in(memo, reinterpret_cast<const void *>(segment_spmm_kernel<LPR, T, HUB>), hub_bytes);
        rc != EPP_OK)
      return rc;
  const long long nsets = ceil_div_ll(a.num_chunks, G);
  long long blocks = ceil_div_ll(nsets, threads / kWarp);
  const long long cap = static_cast<long long>(num_sms) * per_sm;
  if (blocks > cap) blocks = cap;
  segment_spmm_kernel<LPR, T, HUB><<<static_cast<unsigned>(blocks), threads, HUB ? hub_bytes : 0, s>>>(a);
  EPP_CHECK_LAUNCH("segment_spmm_kernel");
  return EPP_OK;
}

// The plan fixes the lanes per row (its list of cleared rows belongs to that
// set size); the columns of this launch pick the tiles per lane.
template <bool HUB>
int launch_by_width(const SegArgs &a, int lanes, int hub_bytes, cudaStream_t s) {
  if (lanes == 4) return a.dim <= 16 ? launch_segments<4, 1, HUB>(a, hub_bytes, s) : launch_segments<4, 2, HUB>(a, hub_bytes, s);
  if (lanes == 8) return a.dim <= 32 ? launch_segments<8, 1, HUB>(a, hub_bytes, s) : launch_segments<8, 2, HUB>(a, hub_bytes, s);
  return a.dim <= 64 ? launch_segments<16, 1, HUB>(a, hub_bytes, s) : launch_segments<16, 2, HUB>(a, hub_bytes, s);
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
                                    int dim, int hub_rows, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan, "null plan");
  EPP_REQUIRE(dim >= 1 && hub_rows >= 0, "dim < 1 or negative hub_rows");
  EPP_REQUIRE(out_ld == 0 || out_ld >= dim, "out_ld must be 0 or >= dim");
  const int n = plan->num_rows;
  if (n == 0) return EPP_OK;
  EPP_REQUIRE(out, "null pointer");
  if (out_ld == 0) out_ld = dim;
  EPP_REQUIRE(kWarp / lanes_for_dim(dim > 128 ? 128 : dim) == plan->groups,
              "the plan was prepared for another row width class (<= 32, <= 64, wider)");
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
  const long long hub_bytes = static_cast<long long>(hub_rows) * src_ld * 4;
  EPP_REQUIRE(hub_bytes <= kMaxHubBytes, "hub rows exceed the shared memory of an SM");
  for (int col0 = 0; col0 < dim; col0 += 128) {          // one launch unless the row is wider than 128
    SegArgs a{};
    a.out = out + col0; a.out_ld = out_ld; a.src = src + col0; a.src_ld = src_ld; a.col = col_idx;
    a.mask = plan->mask; a.first_rank = plan->first_rank; a.rows = plan->identity ? nullptr : plan->rows;
    a.row_scale = row_scale; a.num_edges = plan->num_edges; a.num_chunks = plan->num_chunks;
    a.dim = dim - col0 < 128 ? dim - col0 : 128; a.ovec = ovec; a.hub_rows = hub_rows;
    const int lanes = kWarp / plan->groups;
    const int rc = (hub_rows > 0 && dim <= 128) ? launch_by_width<true>(a, lanes, static_cast<int>(hub_bytes), s)
                                                : launch_by_width<false>(a, lanes, 0, s);
    if (rc != EPP_OK) return rc;
  }
  return EPP_OK;
}
