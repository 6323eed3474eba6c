// Neighbour aggregation over width-classed row tiles for sm_100a, driven by a
// plan that is prepared once per edge list (forward: the CSR of the graph;
// backward: the compacted execution path).
//
// Layout.  The plan owns a re-ordered, padded copy of the edge list's source
// ids.  Rows are sorted into classes by their number of edges: 1, 2, 3-4, and
// then every multiple of eight up to 64; a row of a class is padded with -1
// ids to the class width W.  A row with more than 64 edges is cut into pieces
// of 64 (class 64) plus a remainder piece in the class of its length; its
// pieces are added to the result with vector atomics, and such rows (a few
// thousand hubs of a power-law graph) are cleared by a small kernel first,
// together with the rows that have no edge at all.  Every other row is summed
// by one group of lanes and stored exactly once: the result matrix is not
// zero-filled and written again.
//
// Work unit.  A "sub-warp" of L = ceil(columns / 4) lanes (four columns per
// lane: 4 lanes for 16 columns, 6 for 22, 16 for 64 ...) owns one row of the
// current class, a warp owns floor(32 / L) consecutive rows of that class ("a tile"),
// and tiles are dealt to the persistent warps in descending class order.  All
// sub-warps of a warp therefore run the same number of batches of eight
// independent 16-byte row loads, close their rows at the same instruction, and
// no lane ever waits for a neighbour's longer row -- the cost the group kernel
// (spmm.cu) pays for groups of mixed length.  In the three narrow classes a
// sub-warp packs 8, 4 or 2 rows into one batch.
//
// Source rows already carry their source-side factor (the update step, or the
// backward's packing step, folds it in); the destination-side factor is
// applied when a row is written.
#include <algorithm>
#include <new>
#include <vector>

#include "rowio.cuh"

namespace epp {
namespace {

constexpr int kMaxClasses = 12;
constexpr int kPieceEdges = 64;                 // widest class; hub rows are cut into pieces of this size
constexpr unsigned kAtomicBit = 0x80000000u;    // in a rank's row id: the piece is added atomically
#ifndef EPP_TILE_THREADS
#define EPP_TILE_THREADS 256
#endif
#ifndef EPP_TILE_MINB
#define EPP_TILE_MINB 3
#endif
// Rank count of a class is a multiple of this (times 8 in the narrow classes, where a sub-warp
// takes up to 8 rows): divisible by every rows-per-tile value floor(32 / L), L = 1..32.
constexpr int kRankPad = 480;
constexpr int kTileThreads = EPP_TILE_THREADS;
constexpr int kTileMinBlocks = EPP_TILE_MINB;

// Classes in processing order (widest first).  Class k covers ranks
// [rank_off[k], rank_off[k+1]) and slots [slot_off[k], slot_off[k+1]); a rank
// owns width[k] consecutive slots.  tile_begin[k], the index of the class's
// first tile, depends on the rows per tile and is filled in per launch; the
// rank counts are padded so that every tile shape divides them.
struct ClassTable {
  int count;
  int width[kMaxClasses];
  int tile_begin[kMaxClasses + 1];
  int rank_off[kMaxClasses + 1];
  long long slot_off[kMaxClasses + 1];
};

}  // namespace
}  // namespace epp

struct eppgcn_tile_plan {
  // device arrays inside the caller's buffer
  int *slots;       // [num_slots] source row per padded edge slot, -1 = padding
  int *row_of;      // [num_ranks] row id (| kAtomicBit for a piece of a hub row), -1 = padding rank
  int *seg_start;   // [num_ranks] build-time: first edge of the rank in the caller's edge list
  int *seg_len;     // [num_ranks] build-time: number of edges of the rank
  int *zero_rows;   // [num_zero]  rows cleared before every aggregation
  unsigned char *used;  // [num_sources] 1 where an edge of the list names the source row
  int *active_rows; // [nonempty_rows] the rows that have edges, ascending
  // host side
  epp::ClassTable table;
  long long num_edges, num_slots;
  int num_rows, num_sources, num_ranks, num_zero, zero_all, nonempty_rows, hub_rows;
};

namespace epp {
namespace {

struct TileArgs {
  float *out;
  long long out_ld;
  const float *src;               // rows of src_ld floats, 16-byte aligned, pre-scaled by the source factor
  long long src_ld;
  const int *slots;
  const int *row_of;
  const float *row_scale;         // destination-side factor per row id, or NULL
  int num_tiles;
  int dim;                        // columns handled by this launch
  int lanes;                      // lanes per row, ceil(dim / 4)
  int num_rows, num_sources;      // limits of the ids (looked at by the bounds-checking build only)
  int accumulate;                 // 1: every row is added to what `out` holds (red.global.add) instead of stored
  ClassTable t;
};

// Bounds-checking build (-DEPP_DEBUG_BOUNDS), the stand-in for a memory checker: every source id and
// every row id is compared with its limit before it is used; an offender is not dereferenced, the
// first one is recorded here ({code, value, limit, tile}; code 1 = source id, 2 = row id) and the
// kernel carries on.  eppgcn_debug_status returns the record.
#ifdef EPP_DEBUG_BOUNDS
__device__ int g_debug_record[4];
__device__ __forceinline__ void debug_report(int code, int value, int limit, int tile) {
  if (atomicCAS(&g_debug_record[0], 0, code) == 0) {
    g_debug_record[1] = value; g_debug_record[2] = limit; g_debug_record[3] = tile;
  }
}
#endif

__device__ __forceinline__ void load8(const int *p, int (&c)[8]) {
  const int4 a = __ldg(reinterpret_cast<const int4 *>(p));
  const int4 b = __ldg(reinterpret_cast<const int4 *>(p) + 1);
  c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
}

__device__ __forceinline__ void add4(float (&acc)[4], const float4 &v) {
  acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
}

// The lane's four columns of a row sum, times the row's destination-side
// factor: a plain store, or an atomic add for a piece of a hub row.
template <int OV>
__device__ __forceinline__ void put_row(const TileArgs &a, float *out_lane, int rid, const float (&acc)[4], int n,
                                        bool has_cols) {
  if (rid == -1 || !has_cols) return;
  const int row = static_cast<int>(static_cast<unsigned>(rid) & ~kAtomicBit);
#ifdef EPP_DEBUG_BOUNDS
  if (row >= a.num_rows) {
    debug_report(2, row, a.num_rows, -1);
    return;
  }
#endif
  const float s = a.row_scale ? __ldg(a.row_scale + row) : 1.f;
  const float val[4] = {acc[0] * s, acc[1] * s, acc[2] * s, acc[3] * s};
  float *dst = out_lane + static_cast<long long>(row) * a.out_ld;
  if (rid < 0 || a.accumulate) add_row<4>(dst, val, n, OV);
  else store_row<4>(dst, val, n, OV);
}

// Position of a tile: its class, and the first rank and slot of this
// sub-warp's share of it.  `k` only moves forward (a warp's tiles ascend).
struct TilePos {
  int width;
  int rank;
  long long slot;
};
__device__ __forceinline__ TilePos locate(const ClassTable &t, int G, int tile, int sub, int &k) {
  while (k + 1 < t.count && tile >= t.tile_begin[k + 1]) ++k;
  const int w = t.width[k];
  const int per_sub = w >= 8 ? 1 : 8 / w;                    // rows of one sub-warp in this tile
  const int first = ((tile - t.tile_begin[k]) * G + sub) * per_sub;
  TilePos p;
  p.width = w;
  p.rank = t.rank_off[k] + first;
  p.slot = t.slot_off[k] + static_cast<long long>(first) * w;
  return p;
}

template <int OV>
__global__ void __launch_bounds__(kTileThreads, kTileMinBlocks) tiled_spmm_kernel(const TileArgs a) {
  const int G = kWarp / a.lanes;               // rows (of the wide classes) per tile
  const int lane = threadIdx.x & 31;
  // lanes beyond the last whole sub-warp (32 is not a multiple of 6, say) shadow the last row and never store
  const bool spare = lane >= G * a.lanes;
  const int sub = spare ? G - 1 : lane / a.lanes;
  const int fcol = spare ? 0 : (lane % a.lanes) * 4;
  const bool has_cols = !spare && fcol < a.dim;
  const int n = min(4, a.dim - fcol);          // columns of this lane that exist
  // lanes without columns read column 0 and never store
  const char *glane = reinterpret_cast<const char *>(a.src + (has_cols ? fcol : 0));
  const unsigned ld_bytes = static_cast<unsigned>(a.src_ld) * 4u;
  float *const out_lane = a.out + fcol;

  const int wpb = blockDim.x >> 5;
  const int stride = gridDim.x * wpb;
  int tile = blockIdx.x * wpb + (threadIdx.x >> 5);
  if (tile >= a.num_tiles) return;

  int k = 0;
  TilePos pos = locate(a.t, G, tile, sub, k);
  int c[8];
  load8(a.slots + pos.slot, c);
  int rid_wide = pos.width >= 8 ? __ldg(a.row_of + pos.rank) : -1;
  for (; tile < a.num_tiles; tile += stride) {
    // the position of this warp's next tile, its first eight ids and its row id are fetched behind
    // this tile's row loads
    const int next = tile + stride;
    TilePos npos = pos;
    int kn = k;
    if (next < a.num_tiles) npos = locate(a.t, G, next, sub, kn);
    int cn[8];
    int rid_next = -1;
    float4 v[8];
    auto gather = [&]() {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#ifdef EPP_DEBUG_BOUNDS
        if (c[u] >= a.num_sources) {
          debug_report(1, c[u], a.num_sources, tile);
          c[u] = -1;                               // treated as padding: neither loaded nor added
        }
#endif
        if (c[u] >= 0)
          v[u] = __ldg(reinterpret_cast<const float4 *>(
              glane + static_cast<unsigned long long>(static_cast<unsigned>(c[u])) * ld_bytes));
      }
    };
    auto prefetch_next = [&]() {
      if (next < a.num_tiles) {
        load8(a.slots + npos.slot, cn);
        if (npos.width >= 8) rid_next = __ldg(a.row_of + npos.rank);
      }
    };
    if (pos.width >= 8) {
      // one row per sub-warp, width/8 batches; the row's factor is asked for before the first batch
      int rid = rid_wide;
      const int row = static_cast<int>(static_cast<unsigned>(rid) & ~kAtomicBit);
#ifdef EPP_DEBUG_BOUNDS
      if (rid != -1 && row >= a.num_rows) {
        debug_report(2, row, a.num_rows, tile);
        rid = -1;
      }
#endif
      const float scale = (rid != -1 && a.row_scale) ? __ldg(a.row_scale + row) : 1.f;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const int *cp = a.slots + pos.slot;
#pragma unroll 1
      for (int b = 0; b < pos.width; b += 8) {
        gather();
        if (b + 8 < pos.width) load8(cp + b + 8, cn);
        else prefetch_next();
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (c[u] >= 0) add4(acc, v[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u) c[u] = cn[u];
      }
      if (rid != -1 && has_cols) {
        const float val[4] = {acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale};
        float *dst = out_lane + static_cast<long long>(row) * a.out_ld;
        if (rid < 0 || a.accumulate) add_row<4>(dst, val, n, OV);
        else store_row<4>(dst, val, n, OV);
      }
    } else {
      // narrow classes: 8 / 4 / 2 rows of 1 / 2 / 4 slots in one batch; a row's id and factor are
      // fetched when it is written (these classes hold a few per cent of the edges)
      gather();
      prefetch_next();
      const int *rid = a.row_of + pos.rank;
      if (pos.width == 1) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          if (c[r] >= 0) add4(acc, v[r]);
          put_row<OV>(a, out_lane, __ldg(rid + r), acc, n, has_cols);
        }
      } else if (pos.width == 2) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (c[2 * r + j] >= 0) add4(acc, v[2 * r + j]);
          put_row<OV>(a, out_lane, __ldg(rid + r), acc, n, has_cols);
        }
      } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c[4 * r + j] >= 0) add4(acc, v[4 * r + j]);
          put_row<OV>(a, out_lane, __ldg(rid + r), acc, n, has_cols);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) c[u] = cn[u];
    }
    pos = npos;
    k = kn;
    rid_wide = rid_next;
  }
}

// Clears the rows the plan lists (rows without edges and hub rows), W floats per store.
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

// Plan preparation: fills the padded slot array of one class from the caller's
// edge list; one thread per slot.
__global__ void __launch_bounds__(256) fill_slots_kernel(const int *__restrict__ col, const int *__restrict__ seg_start,
                                                         const int *__restrict__ seg_len, int *slots,
                                                         long long slot_off, int rank_off, int width,
                                                         long long count, unsigned char *used, int num_sources) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int rank = rank_off + static_cast<int>(i / width);
  const int j = static_cast<int>(i % width);
  const int len = __ldg(seg_len + rank);
  const int c = j < len ? __ldg(col + __ldg(seg_start + rank) + j) : -1;
  slots[slot_off + i] = c;
  if (c >= 0 && c < num_sources) used[c] = 1;
}

// dst[r][0..dim) = scale[r] * x[r][0..dim) for the rows an edge list names
// (`used`, or every row when NULL); one thread per four columns.  SV: widest
// aligned load from x (4, 2 or 1 floats).
template <int SV>
__global__ void __launch_bounds__(256) pack_scaled_rows_kernel(float *dst, long long dst_ld, const float *__restrict__ x,
                                                               long long ldx, const float *__restrict__ scale,
                                                               const unsigned char *__restrict__ used,
                                                               int num_rows, int dim) {
  const int per_row = (dim + 3) / 4;
  const long long total = static_cast<long long>(num_rows) * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / per_row);
    const int c0 = static_cast<int>(i % per_row) * 4;
    if (used && !used[r]) continue;
    const float s = scale ? __ldg(scale + r) : 1.f;
    const float *p = x + static_cast<long long>(r) * ldx + c0;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const int n = min(4, dim - c0);
    if (SV == 4 && n == 4) {
      const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if (SV >= 2 && n >= 2) {
      const float2 t = __ldg(reinterpret_cast<const float2 *>(p));
      v[0] = t.x; v[1] = t.y;
      if (n == 4) {
        const float2 u = __ldg(reinterpret_cast<const float2 *>(p) + 1);
        v[2] = u.x; v[3] = u.y;
      } else if (n == 3) {
        v[2] = __ldg(p + 2);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q < n) v[q] = __ldg(p + q);
    }
    *reinterpret_cast<float4 *>(dst + static_cast<long long>(r) * dst_ld + c0) =
        make_float4(v[0] * s, v[1] * s, v[2] * s, v[3] * s);
  }
}

int lanes_for_dim(int dim) {            // lanes per row: four columns per lane, at most 128 columns per launch
  const int l = (dim + 3) / 4;
  return l > 32 ? 32 : l;
}

// Class of a row (or of the remainder piece of a hub row) with `len` edges, as
// an index into the processing order: 0 = width 64 ... 7 = width 8, 8 = width
// 4 (3-4 edges), 9 = width 2, 10 = width 1.
constexpr int kNumClasses = 11;
inline int class_width(int k) { return k <= 7 ? 64 - 8 * k : (k == 8 ? 4 : (k == 9 ? 2 : 1)); }
inline int class_of(int len) {
  if (len >= 5) return 7 - (len - 1) / 8 + 0 * len;   // 5..8 -> 7, 9..16 -> 6, ... 57..64 -> 0
  return len >= 3 ? 8 : (len == 2 ? 9 : 10);
}

size_t round256(size_t b) { return (b + 255) / 256 * 256; }

// Upper bounds that depend only on the sizes the caller knows beforehand.
struct PlanBounds {
  size_t slots, ranks;
};
PlanBounds plan_bounds(long long num_edges, int num_rows) {
  const size_t rows_with_edges = static_cast<size_t>(std::min<long long>(num_rows, num_edges));
  PlanBounds b;
  // a rank is padded by at most 7 slots; every class ends with at most one tile of padding ranks
  b.ranks = rows_with_edges + static_cast<size_t>(num_edges / kPieceEdges) + kNumClasses * 8 * kRankPad + 64;
  b.slots = static_cast<size_t>(num_edges) + 7 * (rows_with_edges + static_cast<size_t>(num_edges / kPieceEdges)) +
            static_cast<size_t>(kRankPad) * (64 + 56 + 48 + 40 + 32 + 24 + 16 + 8 + 8 * (4 + 2 + 1)) + 64;
  return b;
}
struct PlanLayout {
  size_t slots, row_of, seg_start, seg_len, zero_rows, used, active_rows, total;
};
PlanLayout plan_layout(long long num_edges, int num_rows, int num_sources) {
  const PlanBounds b = plan_bounds(num_edges, num_rows);
  PlanLayout l{};
  size_t off = 0;
  l.slots = off;     off += round256(4 * b.slots);
  l.row_of = off;    off += round256(4 * b.ranks);
  l.seg_start = off; off += round256(4 * b.ranks);
  l.seg_len = off;   off += round256(4 * b.ranks);
  l.zero_rows = off; off += round256(4 * (static_cast<size_t>(num_rows) + 1));
  l.used = off;      off += round256(static_cast<size_t>(num_sources) + 1);
  l.active_rows = off; off += round256(4 * (static_cast<size_t>(num_rows) + 1));
  l.total = off;
  return l;
}

struct Segment {
  int row, start, len;
};

// Builds the plan from the rows that have edges, in the order they appear in
// the edge list.  Host work is linear in the number of rows; the padded slot
// array is filled on the device.
int build_plan(eppgcn_tile_plan **out_plan, void *dev_buf, size_t dev_bytes, const std::vector<Segment> &segs,
               const int *col_dev, long long num_edges, int num_rows, int num_sources, cudaStream_t s) {
  const PlanLayout l = plan_layout(num_edges, num_rows, num_sources);
  if (dev_bytes < l.total) {
    set_error("plan buffer too small: %zu bytes given, %zu needed", dev_bytes, l.total);
    return EPP_ERR_BAD_ARG;
  }
  eppgcn_tile_plan *p = new (std::nothrow) eppgcn_tile_plan();
  if (!p) {
    set_error("out of host memory");
    return EPP_ERR_BAD_ARG;
  }
  char *base = static_cast<char *>(dev_buf);
  p->slots = reinterpret_cast<int *>(base + l.slots);
  p->row_of = reinterpret_cast<int *>(base + l.row_of);
  p->seg_start = reinterpret_cast<int *>(base + l.seg_start);
  p->seg_len = reinterpret_cast<int *>(base + l.seg_len);
  p->zero_rows = reinterpret_cast<int *>(base + l.zero_rows);
  p->used = reinterpret_cast<unsigned char *>(base + l.used);
  p->active_rows = reinterpret_cast<int *>(base + l.active_rows);
  p->num_edges = num_edges;
  p->num_rows = num_rows;
  p->num_sources = num_sources;

  // ranks per class: hub rows contribute their 64-edge pieces to class 0 and their remainder to its own class
  long long count[kNumClasses] = {0};
  for (const Segment &g : segs) {
    if (g.len > kPieceEdges) {
      count[0] += g.len / kPieceEdges;
      if (g.len % kPieceEdges) ++count[class_of(g.len % kPieceEdges)];
    } else {
      ++count[class_of(g.len)];
    }
  }
  ClassTable &t = p->table;
  t.count = 0;
  long long rank_off = 0, slot_off = 0;
  int slot_of_class[kNumClasses];
  long long next_rank[kNumClasses];
  for (int k = 0; k < kNumClasses; ++k) {
    slot_of_class[k] = -1;
    if (!count[k]) continue;
    const int w = class_width(k);
    const long long pad = w >= 8 ? kRankPad : 8 * kRankPad;            // every tile shape divides it
    const long long ranks = (count[k] + pad - 1) / pad * pad;
    const int idx = t.count++;
    slot_of_class[k] = idx;
    t.width[idx] = w;
    t.tile_begin[idx] = 0;
    t.rank_off[idx] = static_cast<int>(rank_off);
    t.slot_off[idx] = slot_off;
    next_rank[k] = rank_off;
    rank_off += ranks;
    slot_off += ranks * w;
  }
  for (int i = t.count; i <= kMaxClasses; ++i) {
    t.tile_begin[i] = 0;
    t.rank_off[i] = static_cast<int>(rank_off);
    t.slot_off[i] = slot_off;
    if (i < kMaxClasses) t.width[i] = 1;
  }
  const PlanBounds bound = plan_bounds(num_edges, num_rows);
  if (static_cast<size_t>(rank_off) > bound.ranks || static_cast<size_t>(slot_off) > bound.slots ||
      rank_off >= (1LL << 31)) {
    delete p;
    set_error("plan exceeds its size bound (%lld ranks, %lld slots)", rank_off, slot_off);
    return EPP_ERR_TOO_LARGE;
  }
  p->num_ranks = static_cast<int>(rank_off);
  p->num_slots = slot_off;

  std::vector<int> row_of(static_cast<size_t>(rank_off), -1), seg_start(static_cast<size_t>(rank_off), 0),
      seg_len(static_cast<size_t>(rank_off), 0);
  std::vector<char> has_edges(static_cast<size_t>(num_rows), 0);
  std::vector<int> zero_rows;
  int hubs = 0;
  auto place = [&](int k, int row_id, int start, int len) {
    const long long r = next_rank[k]++;
    row_of[r] = row_id;
    seg_start[r] = start;
    seg_len[r] = len;
  };
  for (const Segment &g : segs) {
    has_edges[g.row] = 1;
    if (g.len > kPieceEdges) {
      ++hubs;
      zero_rows.push_back(g.row);
      const int flagged = static_cast<int>(static_cast<unsigned>(g.row) | kAtomicBit);
      int done = 0;
      for (; done + kPieceEdges <= g.len; done += kPieceEdges) place(0, flagged, g.start + done, kPieceEdges);
      if (done < g.len) place(class_of(g.len - done), flagged, g.start + done, g.len - done);
    } else {
      place(class_of(g.len), g.row, g.start, g.len);
    }
  }
  for (int r = 0; r < num_rows; ++r)
    if (!has_edges[r]) zero_rows.push_back(r);
  p->nonempty_rows = static_cast<int>(segs.size());
  p->hub_rows = hubs;
  p->num_zero = static_cast<int>(zero_rows.size());
  p->zero_all = p->num_zero > num_rows / 2;      // mostly empty result: one memset beats a long list

  const size_t rb = sizeof(int) * static_cast<size_t>(rank_off);
  if (rb) {
    EPP_CUDA_TRY(cudaMemcpyAsync(p->row_of, row_of.data(), rb, cudaMemcpyHostToDevice, s));
    EPP_CUDA_TRY(cudaMemcpyAsync(p->seg_start, seg_start.data(), rb, cudaMemcpyHostToDevice, s));
    EPP_CUDA_TRY(cudaMemcpyAsync(p->seg_len, seg_len.data(), rb, cudaMemcpyHostToDevice, s));
  }
  if (!zero_rows.empty())
    EPP_CUDA_TRY(cudaMemcpyAsync(p->zero_rows, zero_rows.data(), sizeof(int) * zero_rows.size(),
                                 cudaMemcpyHostToDevice, s));
  std::vector<int> active;
  active.reserve(segs.size());
  for (int r = 0; r < num_rows; ++r)
    if (has_edges[r]) active.push_back(r);
  if (!active.empty())
    EPP_CUDA_TRY(cudaMemcpyAsync(p->active_rows, active.data(), sizeof(int) * active.size(), cudaMemcpyHostToDevice, s));
  EPP_CUDA_TRY(cudaMemsetAsync(p->used, 0, static_cast<size_t>(num_sources) + 1, s));
  for (int i = 0; i < t.count; ++i) {
    const long long slots = t.slot_off[i + 1] - t.slot_off[i];
    if (slots <= 0) continue;
    fill_slots_kernel<<<static_cast<unsigned>(ceil_div_ll(slots, 256)), 256, 0, s>>>(
        col_dev, p->seg_start, p->seg_len, p->slots, t.slot_off[i], t.rank_off[i], t.width[i], slots, p->used,
        num_sources);
    EPP_CHECK_LAUNCH("fill_slots_kernel");
  }
  EPP_CUDA_TRY(cudaStreamSynchronize(s));         // the host vectors above must outlive the copies
  *out_plan = p;
  return EPP_OK;
}

template <int OV>
int launch_tiles(TileArgs &a, cudaStream_t s) {
  int num_sms = 0;
  if (const int rc = device_sm_count(&num_sms); rc != EPP_OK) return rc;
  // tiles of this launch's shape: floor(32 / lanes) rows per tile (times 8, 4, 2 in the narrow classes)
  const int G = kWarp / a.lanes;
  long long tiles = 0;
  for (int k = 0; k < a.t.count; ++k) {
    const int w = a.t.width[k];
    a.t.tile_begin[k] = static_cast<int>(tiles);
    tiles += (a.t.rank_off[k + 1] - a.t.rank_off[k]) / (G * (w >= 8 ? 1 : 8 / w));
  }
  for (int k = a.t.count; k <= kMaxClasses; ++k) a.t.tile_begin[k] = static_cast<int>(tiles);
  a.num_tiles = static_cast<int>(tiles);
  long long blocks = ceil_div_ll(tiles, kTileThreads / kWarp);
  const long long cap = static_cast<long long>(num_sms) * kTileMinBlocks;
  if (blocks > cap) blocks = cap;
  tiled_spmm_kernel<OV><<<static_cast<unsigned>(blocks), kTileThreads, 0, s>>>(a);
  EPP_CHECK_LAUNCH("tiled_spmm_kernel");
  return EPP_OK;
}

}  // namespace
}  // namespace epp

using namespace epp;

EPP_EXPORT size_t eppgcn_tile_plan_bytes(long long num_edges, int num_rows, int num_sources) {
  if (num_edges < 0 || num_rows < 0 || num_sources < 0) return 0;
  return plan_layout(num_edges, num_rows, num_sources).total;
}

EPP_EXPORT int eppgcn_tile_plan_from_csr(eppgcn_tile_plan **plan, void *dev_buf, size_t dev_bytes,
                                         const int *row_ptr, const int *col_idx, int num_rows, long long num_edges,
                                         int num_sources, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan && dev_buf && num_rows >= 0 && num_edges >= 0 && num_sources >= 0, "bad argument");
  EPP_REQUIRE(num_edges < (1LL << 31), "edge count exceeds int32");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(dev_buf) % 256 == 0, "plan buffer must be 256-byte aligned");
  EPP_REQUIRE(num_rows == 0 || row_ptr, "null pointer");
  EPP_REQUIRE(num_edges == 0 || col_idx, "null pointer");
  std::vector<int> ptr(static_cast<size_t>(num_rows) + 1, 0);
  if (num_rows > 0) {
    EPP_CUDA_TRY(cudaMemcpyAsync(ptr.data(), row_ptr, sizeof(int) * ptr.size(), cudaMemcpyDeviceToHost, s));
    EPP_CUDA_TRY(cudaStreamSynchronize(s));
  }
  std::vector<Segment> segs;
  segs.reserve(static_cast<size_t>(num_rows));
  for (int r = 0; r < num_rows; ++r) {
    const int beg = ptr[r], end = ptr[r + 1];
    EPP_REQUIRE(beg >= 0 && end >= beg && end <= num_edges, "row_ptr is not a non-decreasing offset array");
    if (end > beg) segs.push_back({r, beg, end - beg});
  }
  return build_plan(plan, dev_buf, dev_bytes, segs, col_idx, num_edges, num_rows, num_sources, s);
}

EPP_EXPORT int eppgcn_tile_plan_from_ids(eppgcn_tile_plan **plan, void *dev_buf, size_t dev_bytes,
                                         const int *ids, const int *col_idx, long long num_edges, int num_rows,
                                         int num_sources, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan && dev_buf && num_rows >= 0 && num_edges >= 0 && num_sources >= 0, "bad argument");
  EPP_REQUIRE(num_edges < (1LL << 31), "edge count exceeds int32");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(dev_buf) % 256 == 0, "plan buffer must be 256-byte aligned");
  EPP_REQUIRE(num_edges == 0 || (ids && col_idx), "null pointer");
  std::vector<int> host(static_cast<size_t>(num_edges));
  if (num_edges > 0) {
    EPP_CUDA_TRY(cudaMemcpyAsync(host.data(), ids, sizeof(int) * host.size(), cudaMemcpyDeviceToHost, s));
    EPP_CUDA_TRY(cudaStreamSynchronize(s));
  }
  std::vector<Segment> segs;
  std::vector<char> seen(static_cast<size_t>(num_rows), 0);
  for (long long e = 0; e < num_edges;) {
    const int r = host[e];
    EPP_REQUIRE(r >= 0 && r < num_rows, "row id out of range");
    EPP_REQUIRE(!seen[r], "the edges of a row must be consecutive");
    seen[r] = 1;
    long long f = e + 1;
    while (f < num_edges && host[f] == r) ++f;
    segs.push_back({r, static_cast<int>(e), static_cast<int>(f - e)});
    e = f;
  }
  return build_plan(plan, dev_buf, dev_bytes, segs, col_idx, num_edges, num_rows, num_sources, s);
}

EPP_EXPORT int eppgcn_pack_scaled_rows(float *dst, long long dst_ld, const float *x, long long ldx,
                                       const float *scale, const eppgcn_tile_plan *plan, int num_rows, int dim,
                                       void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(num_rows >= 0 && dim >= 1, "negative size or dim < 1");
  if (num_rows == 0) return EPP_OK;
  EPP_REQUIRE(dst && x, "null pointer");
  EPP_REQUIRE(dst_ld % 4 == 0 && dst_ld >= (dim + 3) / 4 * 4 && aligned(dst, 16),
              "destination rows must be 16-byte aligned and padded to a multiple of 4 floats");
  EPP_REQUIRE(ldx >= dim, "ldx must be >= dim");
  EPP_REQUIRE(!plan || plan->num_sources >= num_rows, "the plan names fewer source rows than num_rows");
  const long long total = static_cast<long long>(num_rows) * ((dim + 3) / 4);
  long long blocks = ceil_div_ll(total, 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  const unsigned g = static_cast<unsigned>(blocks);
  const unsigned char *used = plan ? plan->used : nullptr;
  if (ldx % 4 == 0 && aligned(x, 16))
    pack_scaled_rows_kernel<4><<<g, 256, 0, s>>>(dst, dst_ld, x, ldx, scale, used, num_rows, dim);
  else if (ldx % 2 == 0 && aligned(x, 8))
    pack_scaled_rows_kernel<2><<<g, 256, 0, s>>>(dst, dst_ld, x, ldx, scale, used, num_rows, dim);
  else
    pack_scaled_rows_kernel<1><<<g, 256, 0, s>>>(dst, dst_ld, x, ldx, scale, used, num_rows, dim);
  EPP_CHECK_LAUNCH("pack_scaled_rows_kernel");
  return EPP_OK;
}

EPP_EXPORT void eppgcn_tile_plan_destroy(eppgcn_tile_plan *plan) { delete plan; }

EPP_EXPORT int eppgcn_tile_plan_info(const eppgcn_tile_plan *plan, long long *out8) {
  EPP_REQUIRE(plan && out8, "null pointer");
  out8[0] = plan->num_edges; out8[1] = plan->num_rows; out8[2] = plan->num_slots; out8[3] = plan->num_ranks;
  out8[4] = plan->nonempty_rows; out8[5] = plan->num_zero; out8[6] = plan->hub_rows; out8[7] = plan->zero_all;
  return EPP_OK;
}

EPP_EXPORT int eppgcn_tile_plan_active_rows(const eppgcn_tile_plan *plan, const int **rows_dev, int *count) {
  EPP_REQUIRE(plan && rows_dev && count, "null pointer");
  *rows_dev = plan->active_rows;
  *count = plan->nonempty_rows;
  return EPP_OK;
}

// The tile launches of one aggregation (one unless the row is wider than 128 columns).
static int run_tiles(float *out, long long out_ld, const float *src, long long src_ld, const eppgcn_tile_plan *plan,
                     const float *row_scale, int dim, int ovec, int accumulate, cudaStream_t s) {
  if (plan->num_ranks == 0) return EPP_OK;
  EPP_REQUIRE(src, "null pointer");
  EPP_REQUIRE(src_ld % 4 == 0 && src_ld >= (dim + 3) / 4 * 4 && src_ld <= 0x3fffffffLL && aligned(src, 16),
              "source rows must be 16-byte aligned and padded to a multiple of 4 floats");
  for (int col0 = 0; col0 < dim; col0 += 128) {
    TileArgs a{};
    a.out = out + col0; a.out_ld = out_ld; a.src = src + col0; a.src_ld = src_ld;
    a.slots = plan->slots; a.row_of = plan->row_of; a.row_scale = row_scale;
    a.dim = dim - col0 < 128 ? dim - col0 : 128; a.lanes = lanes_for_dim(a.dim); a.t = plan->table;
    a.num_rows = plan->num_rows; a.num_sources = plan->num_sources;
    a.accumulate = accumulate;
    const int rc = ovec == 4 ? launch_tiles<4>(a, s) : ovec == 2 ? launch_tiles<2>(a, s) : launch_tiles<1>(a, s);
    if (rc != EPP_OK) return rc;
  }
  return EPP_OK;
}

EPP_EXPORT int eppgcn_spmm_tiles(float *out, long long out_ld, const float *src, long long src_ld,
                                 const eppgcn_tile_plan *plan, const float *row_scale, int dim, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan, "null plan");
  EPP_REQUIRE(dim >= 1, "dim < 1");
  EPP_REQUIRE(out_ld == 0 || out_ld >= dim, "out_ld must be 0 or >= dim");
  const int n = plan->num_rows;
  if (n == 0) return EPP_OK;
  EPP_REQUIRE(out, "null pointer");
  if (out_ld == 0) out_ld = dim;
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
  return run_tiles(out, out_ld, src, src_ld, plan, row_scale, dim, ovec, 0, s);
}

EPP_EXPORT int eppgcn_spmm_tiles_add(float *out, long long out_ld, const float *src, long long src_ld,
                                     const eppgcn_tile_plan *plan, const float *row_scale, int dim, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(plan, "null plan");
  EPP_REQUIRE(dim >= 1, "dim < 1");
  EPP_REQUIRE(out_ld == 0 || out_ld >= dim, "out_ld must be 0 or >= dim");
  if (plan->num_rows == 0) return EPP_OK;
  EPP_REQUIRE(out, "null pointer");
  if (out_ld == 0) out_ld = dim;
  int ovec = 1;
  if (out_ld % 4 == 0 && aligned(out, 16)) ovec = 4;
  else if (out_ld % 2 == 0 && aligned(out, 8)) ovec = 2;
  return run_tiles(out, out_ld, src, src_ld, plan, row_scale, dim, ovec, 1, s);
}

EPP_EXPORT int eppgcn_debug_status(int *out4, int reset) {
  EPP_REQUIRE(out4, "null pointer");
#ifdef EPP_DEBUG_BOUNDS
  EPP_CUDA_TRY(cudaDeviceSynchronize());
  EPP_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_debug_record, sizeof(int) * 4));
  if (reset) {
    const int zero[4] = {0, 0, 0, 0};
    EPP_CUDA_TRY(cudaMemcpyToSymbol(g_debug_record, zero, sizeof(zero)));
  }
#else
  (void)reset;
  out4[0] = -1; out4[1] = out4[2] = out4[3] = 0;      // not a bounds-checking build
#endif
  return EPP_OK;
}
