// One-time execution-path preparation for sm_100a: path marking, stable
// compaction of the marked edges and splitting of the active rows into parts.
//
// The two scans (compaction ranks, part offsets) are single-pass chained scans:
// a tile takes its id from an atomic ticket (so every predecessor of a waiting
// tile has already started), publishes its aggregate in a 64-bit descriptor and
// looks back over its predecessors' descriptors.  Every wait is bounded; when
// the bound is hit the kernel records EPP_ERR_SCAN_TIMEOUT, releases its
// successors and returns.  A three-kernel mode (counts, scan, scatter) that
// never waits is kept as the fallback and as a cross-check.
#include "common.cuh"

namespace epp {
namespace {

constexpr int kScanThreads = 512;
constexpr int kScanWarps = kScanThreads / kWarp;
constexpr int kCompactItems = 8;                                  // per thread
constexpr int kCompactTile = kScanThreads * kCompactItems;        // 4096 edges
constexpr int kSplitItems = 4;
constexpr int kSplitTile = kScanThreads * kSplitItems;            // 2048 vertices
constexpr int kMaxPolls = 1 << 21;                                // bounded look-back wait

enum ScanMode { kLookback = 0, kCountOnly = 1, kGivenOffsets = 2 };

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Exclusive prefix (fields a, b) of tile `tile`; called by all lanes of one warp.
// Publishes the tile's aggregate first and its inclusive prefix afterwards.
__device__ void chained_lookback(unsigned long long *desc, ScanHeader *hdr, int tile,
                                 unsigned agg_a, unsigned agg_b, unsigned &ex_a, unsigned &ex_b) {
  const int lane = threadIdx.x & 31;
  volatile unsigned long long *vdesc = desc;
  volatile int *verr = &hdr->error;
  if (tile == 0) {
    if (lane == 0) vdesc[0] = tile_pack(kTilePrefix, agg_a, agg_b);
    ex_a = ex_b = 0;
    return;
  }
  if (lane == 0) vdesc[tile] = tile_pack(kTileAggregate, agg_a, agg_b);
  unsigned long long sum = 0;   // packed fields, state bits stay zero
  int window_top = tile - 1;
  bool failed = false;
  while (true) {
    const int p = window_top - lane;
    unsigned long long w = tile_pack(kTilePrefix, 0, 0);   // lanes before tile 0 end the search
    if (p >= 0) {
      int polls = 0;
      w = vdesc[p];
      while (tile_state(w) == kTileEmpty) {
        if (++polls > kMaxPolls || *verr != EPP_OK) { failed = true; break; }
        if (polls > 16) __nanosleep(polls > 1024 ? 256 : 32);
        w = vdesc[p];
      }
    }
    if (__any_sync(kFull, failed)) break;
    const unsigned done = __ballot_sync(kFull, tile_state(w) == kTilePrefix);
    // lanes up to and including the nearest predecessor that holds a full prefix
    const unsigned take = done ? ((2u << (__ffs(done) - 1)) - 1u) : kFull;
    unsigned long long v = ((take >> lane) & 1u) ? (w & 0x3fffffffffffffffull) : 0ull;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(kFull, v, off);
    sum += v;
    if (done) break;
    window_top -= kWarp;
  }
  if (__any_sync(kFull, failed)) {
    if (lane == 0) {
      atomicExch(&hdr->error, EPP_ERR_SCAN_TIMEOUT);
      vdesc[tile] = tile_pack(kTilePrefix, 0, 0);   // let successors go; the result is void
    }
    ex_a = ex_b = 0;
    return;
  }
  ex_a = tile_a(sum);
  ex_b = tile_b(sum);
  if (lane == 0) vdesc[tile] = tile_pack(kTilePrefix, ex_a + agg_a, ex_b + agg_b);
}

// Block-wide exclusive scan of one (a, b) pair per thread over kScanThreads
// threads; returns the thread's exclusive prefix and the block totals.
__device__ __forceinline__ void block_scan_pair(unsigned a, unsigned b, unsigned &ex_a, unsigned &ex_b,
                                                unsigned &tot_a, unsigned &tot_b,
                                                unsigned (*s_warp)[2]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned ia = a, ib = b;
#pragma unroll
  for (int off = 1; off < kWarp; off <<= 1) {
    const unsigned ta = __shfl_up_sync(kFull, ia, off), tb = __shfl_up_sync(kFull, ib, off);
    if (lane >= off) { ia += ta; ib += tb; }
  }
  if (lane == kWarp - 1) { s_warp[warp][0] = ia; s_warp[warp][1] = ib; }
  __syncthreads();
  if (warp == 0) {
    unsigned wa = lane < kScanWarps ? s_warp[lane][0] : 0, wb = lane < kScanWarps ? s_warp[lane][1] : 0;
    unsigned sa = wa, sb = wb;
#pragma unroll
    for (int off = 1; off < kWarp; off <<= 1) {
      const unsigned ta = __shfl_up_sync(kFull, sa, off), tb = __shfl_up_sync(kFull, sb, off);
      if (lane >= off) { sa += ta; sb += tb; }
    }
    if (lane < kScanWarps) { s_warp[lane][0] = sa - wa; s_warp[lane][1] = sb - wb; }
    if (lane == kWarp - 1) { s_warp[kScanWarps][0] = sa; s_warp[kScanWarps][1] = sb; }
  }
  __syncthreads();
  ex_a = s_warp[warp][0] + ia - a;
  ex_b = s_warp[warp][1] + ib - b;
  tot_a = s_warp[kScanWarps][0];
  tot_b = s_warp[kScanWarps][1];
}

// ---------------------------------------------------------------------------
// path marking
// ---------------------------------------------------------------------------
constexpr int kMaskLanes = 8;   // lanes per group

__global__ void __launch_bounds__(256) mask_forward_kernel(
    const int *__restrict__ ids, const int *__restrict__ part_ptr, const int *__restrict__ edge_list,
    const unsigned char *__restrict__ src_mask, unsigned char *ngh_mask,
    int *__restrict__ back_edge_mask, int *__restrict__ node_degs,
    int num_parts, bool is_last, int row_offset) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long g = t / kMaskLanes;
  const int sl = threadIdx.x % kMaskLanes;
  int count = 0, r = 0;
  bool mark = false, any_edge = false;
  if (g < num_parts) {
    r = __ldg(ids + g);
    const int beg = __ldg(part_ptr + g), end = __ldg(part_ptr + g + 1);
    any_edge = end > beg;
    mark = !is_last && any_edge && src_mask[r + row_offset] != 0;
    for (int e = beg + sl; e < end; e += kMaskLanes) {
      const int c = __ldg(edge_list + e);
      if (mark) ngh_mask[c] = 1;
      if (src_mask[c] != 0) {
        back_edge_mask[e] = r;
        ++count;
      }
    }
  }
#pragma unroll
  for (int off = kMaskLanes / 2; off >= 1; off >>= 1) count += __shfl_xor_sync(kFull, count, off);
  if (sl == 0 && g < num_parts) {
    if (count) atomicAdd(node_degs + r, count);
    if (mark) ngh_mask[r + row_offset] = 1;
  }
}

// ---------------------------------------------------------------------------
// stable compaction of (edge_mask, col) pairs with edge_mask != -1
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kScanThreads) compact_mask_kernel(
    const int *__restrict__ mask, const int *__restrict__ col, int *__restrict__ out_id,
    int *__restrict__ out_edge, int length, int num_tiles, ScanHeader *hdr,
    unsigned long long *desc, int *valid_len_dev) {
  __shared__ unsigned s_warp[kScanWarps + 1][2];
  __shared__ unsigned s_base;
  __shared__ int s_tile;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int tile = blockIdx.x;
  if (MODE == kLookback) {
    if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(&hdr->ticket, 1u));
    __syncthreads();
    tile = s_tile;
  }
  const long long base = static_cast<long long>(tile) * kCompactTile + warp * (kWarp * kCompactItems);
  int m[kCompactItems];
  unsigned ballots[kCompactItems];
  unsigned count = 0;
#pragma unroll
  for (int k = 0; k < kCompactItems; ++k) {
    const long long idx = base + k * kWarp + lane;
    m[k] = idx < length ? __ldg(mask + idx) : -1;
    ballots[k] = __ballot_sync(kFull, m[k] != -1);
    count += __popc(ballots[k]);
  }
  // warp totals -> exclusive warp offsets (count is warp-uniform)
  if (lane == 0) s_warp[warp][0] = count;
  __syncthreads();
  if (warp == 0) {
    const unsigned w = lane < kScanWarps ? s_warp[lane][0] : 0;
    unsigned s = w;
#pragma unroll
    for (int off = 1; off < kWarp; off <<= 1) {
      const unsigned t = __shfl_up_sync(kFull, s, off);
      if (lane >= off) s += t;
    }
    const unsigned total = __shfl_sync(kFull, s, kWarp - 1);
    if (lane < kScanWarps) s_warp[lane][0] = s - w;
    unsigned ex = 0, unused = 0;
    if (MODE == kLookback) {
      chained_lookback(desc, hdr, tile, total, 0u, ex, unused);
    } else if (MODE == kCountOnly) {
      if (lane == 0) desc[tile] = tile_pack(0, total, 0);
    } else {
      ex = tile_a(desc[tile]);
    }
    if (lane == 0) {
      s_base = ex;
      if (MODE != kCountOnly && tile == num_tiles - 1) *valid_len_dev = static_cast<int>(ex + total);
    }
  }
  if (MODE == kCountOnly) return;
  __syncthreads();
  unsigned offset = s_base + s_warp[warp][0];
  const unsigned lt = lanemask_lt();
#pragma unroll
  for (int k = 0; k < kCompactItems; ++k) {
    if (m[k] != -1) {
      const long long idx = base + k * kWarp + lane;
      const unsigned dst = offset + __popc(ballots[k] & lt);
      out_id[dst] = m[k];
      out_edge[dst] = __ldg(col + idx);
    }
    offset += __popc(ballots[k]);
  }
}

// Exclusive scan of packed tile totals by one block (fallback mode).
__global__ void __launch_bounds__(1024) scan_tiles_kernel(unsigned long long *desc, int num_tiles) {
  __shared__ unsigned long long s_warp[33];
  __shared__ unsigned long long s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < num_tiles; base += 1024) {
    const int i = base + threadIdx.x;
    const unsigned long long v = i < num_tiles ? desc[i] : 0ull;
    unsigned long long s = v;
#pragma unroll
    for (int off = 1; off < kWarp; off <<= 1) {
      const unsigned long long t = __shfl_up_sync(kFull, s, off);
      if (lane >= off) s += t;
    }
    if (lane == 31) s_warp[warp] = s;
    __syncthreads();
    if (warp == 0) {
      const unsigned long long w = s_warp[lane];
      unsigned long long ws = w;
#pragma unroll
      for (int off = 1; off < kWarp; off <<= 1) {
        const unsigned long long t = __shfl_up_sync(kFull, ws, off);
        if (lane >= off) ws += t;
      }
      s_warp[lane] = ws - w;
      if (lane == 31) s_warp[32] = ws;
    }
    __syncthreads();
    if (i < num_tiles) desc[i] = s_carry + s_warp[warp] + s - v;
    __syncthreads();
    if (threadIdx.x == 0) s_carry += s_warp[32];
    __syncthreads();
  }
}

// Zero-fills [ *count_dev + skip, length ) of up to two arrays.
__global__ void zero_tail_kernel(int *a, int *b, const int *count_dev, int skip, long long length) {
  const long long start = static_cast<long long>(*count_dev) + skip;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = start + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < length; i += stride) {
    a[i] = 0;
    if (b) b[i] = 0;
  }
}

__global__ void publish_status_kernel(const ScanHeader *hdr, int *status_dev) { *status_dev = hdr->error; }

// Self-test of the bounded wait: makes the first ticket 1, so tile 0 -- whose
// descriptor the look-back of tile 1 needs -- never exists.
__global__ void skip_first_ticket_kernel(ScanHeader *hdr) { hdr->ticket = 1u; }

// ---------------------------------------------------------------------------
// splitting active rows into parts
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kScanThreads) split_parts_kernel(
    const int *__restrict__ node_deg, int num_nodes, int part_size, int *__restrict__ part_pointer,
    int out_len, int num_tiles, ScanHeader *hdr, unsigned long long *desc, int *num_parts_dev,
    int *__restrict__ part2node = nullptr, int part2node_len = 0) {
  __shared__ unsigned s_warp[kScanWarps + 1][2];
  __shared__ unsigned s_cpre[kSplitTile + 1];
  __shared__ unsigned s_epre[kSplitTile];
  __shared__ unsigned s_base[2];
  __shared__ int s_tile;
  int tile = blockIdx.x;
  if (MODE == kLookback) {
    if (threadIdx.x == 0) s_tile = static_cast<int>(atomicAdd(&hdr->ticket, 1u));
    __syncthreads();
    tile = s_tile;
  }
  const long long v0 = static_cast<long long>(tile) * kSplitTile + threadIdx.x * kSplitItems;
  unsigned cnt[kSplitItems], deg[kSplitItems];
  unsigned tc = 0, td = 0;
#pragma unroll
  for (int i = 0; i < kSplitItems; ++i) {
    const long long v = v0 + i;
    const int d = v < num_nodes ? __ldg(node_deg + v) : 0;
    deg[i] = d > 0 ? static_cast<unsigned>(d) : 0u;
    cnt[i] = d > 0 ? static_cast<unsigned>((d - 1) / part_size + 1) : 0u;
    tc += cnt[i];
    td += deg[i];
  }
  unsigned ec, ed, tot_c, tot_d;
  block_scan_pair(tc, td, ec, ed, tot_c, tot_d, s_warp);
  if (MODE != kCountOnly) {
#pragma unroll
    for (int i = 0; i < kSplitItems; ++i) {
      s_cpre[threadIdx.x * kSplitItems + i] = ec;
      s_epre[threadIdx.x * kSplitItems + i] = ed;
      ec += cnt[i];
      ed += deg[i];
    }
    if (threadIdx.x == 0) s_cpre[kSplitTile] = tot_c;
  }
  if (threadIdx.x < kWarp) {
    unsigned ex_c = 0, ex_d = 0;
    if (MODE == kLookback) {
      chained_lookback(desc, hdr, tile, tot_c, tot_d, ex_c, ex_d);
    } else if (MODE == kCountOnly) {
      if (threadIdx.x == 0) desc[tile] = tile_pack(0, tot_c, tot_d);
    } else {
      ex_c = tile_a(desc[tile]);
      ex_d = tile_b(desc[tile]);
    }
    if (threadIdx.x == 0) { s_base[0] = ex_c; s_base[1] = ex_d; }
  }
  if (MODE == kCountOnly) return;
  __syncthreads();
  const unsigned pc = s_base[0], pe = s_base[1];
  // One thread per output slot: find the owning vertex in the tile by binary
  // search over the exclusive part counts (vertices without parts are skipped
  // because they share their successor's prefix).
  for (unsigned j = threadIdx.x; j < tot_c; j += kScanThreads) {
    int lo = 0, hi = kSplitTile;          // largest v with s_cpre[v] <= j
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_cpre[mid] <= j) lo = mid; else hi = mid;
    }
    const unsigned k = j - s_cpre[lo];
    const long long slot = static_cast<long long>(pc) + j;
    if (slot < out_len) part_pointer[slot] = static_cast<int>(pe + s_epre[lo] + k * static_cast<unsigned>(part_size));
    if (part2node && slot < part2node_len) part2node[slot] = tile * kSplitTile + lo;     // the part's vertex
  }
  if (tile == num_tiles - 1 && threadIdx.x == 0) {
    const long long slot = static_cast<long long>(pc) + tot_c;
    if (slot < out_len) part_pointer[slot] = static_cast<int>(pe + tot_d);
    *num_parts_dev = static_cast<int>(pc + tot_c);
  }
}

// Row lengths of a CSR, the input of the part splitting when it builds the forward groups.
__global__ void __launch_bounds__(256) row_lengths_kernel(const int *__restrict__ row_ptr, int num_nodes, int *deg) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v < num_nodes) deg[v] = __ldg(row_ptr + v + 1) - __ldg(row_ptr + v);
}

__global__ void __launch_bounds__(256) count_nonzero_kernel(const int *__restrict__ v, long long length, int *count_dev) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  int c = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < length; i += stride)
    c += __ldg(v + i) != 0;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) c += __shfl_xor_sync(kFull, c, off);
  __shared__ int s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 8; ++i) t += s[i];
    if (t) atomicAdd(count_dev, t);
  }
}

inline int tail_grid(long long length) {
  long long b = ceil_div_ll(length, 256);
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 8 ? 148 * 8 : b));
}

}  // namespace
}  // namespace epp

using namespace epp;

EPP_EXPORT int eppgcn_mask_forward(const int *ids, const int *part_ptr, const int *edge_list,
                                   const unsigned char *src_mask, unsigned char *ngh_mask,
                                   int *back_edge_mask, int *node_degs,
                                   int num_parts, int is_last, int row_offset,
                                   int blockx, int blocky, void *stream) {
  (void)blockx; (void)blocky;
  EPP_REQUIRE(num_parts >= 0 && row_offset >= 0, "negative size");
  if (num_parts == 0) return EPP_OK;
  EPP_REQUIRE(ids && part_ptr && edge_list && src_mask && back_edge_mask && node_degs, "null pointer");
  EPP_REQUIRE(is_last || ngh_mask, "ngh_mask is required before the last step");
  const long long threads = static_cast<long long>(num_parts) * kMaskLanes;
  const long long blocks = ceil_div_ll(threads, 256);
  mask_forward_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, part_ptr, edge_list, src_mask, ngh_mask, back_edge_mask, node_degs, num_parts, is_last != 0,
      row_offset);
  EPP_CHECK_LAUNCH("mask_forward_kernel");
  return EPP_OK;
}

static size_t scan_scratch_bytes(long long tiles) {
  return sizeof(ScanHeader) + sizeof(unsigned long long) * static_cast<size_t>(tiles < 1 ? 1 : tiles);
}

EPP_EXPORT size_t eppgcn_compact_scratch_bytes(int length) {
  return scan_scratch_bytes(ceil_div_ll(length < 0 ? 0 : length, kCompactTile));
}

EPP_EXPORT size_t eppgcn_split_scratch_bytes(int num_nodes) {
  return scan_scratch_bytes(ceil_div_ll(num_nodes < 0 ? 0 : num_nodes, kSplitTile));
}

EPP_EXPORT int eppgcn_compact_mask(const int *edge_mask, const int *col_idx, int *out_id, int *out_edge,
                                   int length, void *scratch, size_t scratch_bytes,
                                   int *valid_len_dev, int *status_dev, int mode, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(length >= 0, "negative length");
  EPP_REQUIRE(valid_len_dev && status_dev, "null result pointer");
  EPP_REQUIRE(mode >= 0 && mode <= 2, "mode must be 0, 1 or 2");
  EPP_REQUIRE(mode != 2 || length > kCompactTile, "the wait self-test needs more than one tile of input");
  EPP_CUDA_TRY(cudaMemsetAsync(valid_len_dev, 0, sizeof(int), s));
  EPP_CUDA_TRY(cudaMemsetAsync(status_dev, 0, sizeof(int), s));
  if (length == 0) return EPP_OK;
  EPP_REQUIRE(edge_mask && col_idx && out_id && out_edge && scratch, "null pointer");
  EPP_REQUIRE(scratch_bytes >= eppgcn_compact_scratch_bytes(length), "scratch too small");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(scratch) % 8 == 0, "scratch must be 8-byte aligned");
  const int tiles = static_cast<int>(ceil_div_ll(length, kCompactTile));
  ScanHeader *hdr = static_cast<ScanHeader *>(scratch);
  unsigned long long *desc = reinterpret_cast<unsigned long long *>(hdr + 1);
  EPP_CUDA_TRY(cudaMemsetAsync(scratch, 0, scan_scratch_bytes(tiles), s));
  if (mode == 0) {
    compact_mask_kernel<kLookback><<<tiles, kScanThreads, 0, s>>>(edge_mask, col_idx, out_id, out_edge, length,
                                                                  tiles, hdr, desc, valid_len_dev);
    EPP_CHECK_LAUNCH("compact_mask_kernel<lookback>");
  } else if (mode == 2) {
    // tile ids 1 .. tiles-1 are handed out; tile 1 looks back at a descriptor nobody writes, its
    // bounded wait runs out, the error word is set and every other tile leaves as soon as it sees it
    skip_first_ticket_kernel<<<1, 1, 0, s>>>(hdr);
    EPP_CHECK_LAUNCH("skip_first_ticket_kernel");
    compact_mask_kernel<kLookback><<<tiles - 1, kScanThreads, 0, s>>>(edge_mask, col_idx, out_id, out_edge, length,
                                                                      tiles, hdr, desc, valid_len_dev);
    EPP_CHECK_LAUNCH("compact_mask_kernel<lookback, wait self-test>");
  } else {
    compact_mask_kernel<kCountOnly><<<tiles, kScanThreads, 0, s>>>(edge_mask, col_idx, out_id, out_edge, length,
                                                                   tiles, hdr, desc, valid_len_dev);
    EPP_CHECK_LAUNCH("compact_mask_kernel<count>");
    scan_tiles_kernel<<<1, 1024, 0, s>>>(desc, tiles);
    EPP_CHECK_LAUNCH("scan_tiles_kernel");
    compact_mask_kernel<kGivenOffsets><<<tiles, kScanThreads, 0, s>>>(edge_mask, col_idx, out_id, out_edge,
                                                                      length, tiles, hdr, desc, valid_len_dev);
    EPP_CHECK_LAUNCH("compact_mask_kernel<scatter>");
  }
  zero_tail_kernel<<<tail_grid(length), 256, 0, s>>>(out_id, out_edge, valid_len_dev, 0, length);
  EPP_CHECK_LAUNCH("zero_tail_kernel");
  publish_status_kernel<<<1, 1, 0, s>>>(hdr, status_dev);
  EPP_CHECK_LAUNCH("publish_status_kernel");
  return EPP_OK;
}

// ---------------------------------------------------------------------------
// Compaction without any allocation by anyone.
//
// Some hosts cannot give this library scratch memory at call time: a process
// that handed the whole device to its own pool at start-up and runs without
// headroom, a latency-critical thread that must never hit the device-wide
// synchronisation cudaMalloc/cudaFree imply, or an embedding application that
// forbids device allocation after initialisation.  For them the tile
// descriptors of the single-pass scan live in this fixed array instead of a
// caller-supplied buffer.  It is part of the library image: every GPU that
// loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------
constexpr int kStaticCompactMaxLength = 1 << 26;   // 67,108,864 edges
constexpr size_t kStaticCompactBytes =
    sizeof(epp::ScanHeader) + sizeof(unsigned long long) * (kStaticCompactMaxLength / epp::kCompactTile);   // 131,328 B
static __device__ __align__(256) unsigned char g_static_compact_scratch[kStaticCompactBytes];

// In host code `g_static_compact_scratch` is only a handle for the runtime, not
// a device address; the address is looked up once per device, with that device
// current, and cached.
static int static_compact_scratch_address(void **ptr) {
  constexpr int kMaxDevices = 64;
  static void *cached[kMaxDevices] = {nullptr};
  int dev = 0;
  EPP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device ordinal %d is beyond the %d devices this entry point tracks", dev, kMaxDevices);
    return EPP_ERR_TOO_LARGE;
  }
  if (!cached[dev]) {
    void *p = nullptr;
    EPP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_compact_scratch));
    if (!p || reinterpret_cast<uintptr_t>(p) % 256 != 0) {
      set_error("static scratch symbol resolved to an unusable address");
      return EPP_ERR_CUDA;
    }
    cached[dev] = p;
  }
  *ptr = cached[dev];
  return EPP_OK;
}

EPP_EXPORT int eppgcn_compact_mask_static(const int *edge_mask, const int *col_idx, int *out_id, int *out_edge,
                                          int length, int *valid_len_dev, int *status_dev, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(length >= 0, "negative length");
  EPP_REQUIRE(valid_len_dev && status_dev, "null result pointer");
  if (length > kStaticCompactMaxLength) {
    set_error("eppgcn_compact_mask_static handles at most %d edges per call, got %d; "
              "use eppgcn_compact_mask with caller-provided scratch", kStaticCompactMaxLength, length);
    return EPP_ERR_TOO_LARGE;
  }
  void *scratch = nullptr;
  const int rc = static_compact_scratch_address(&scratch);
  if (rc != EPP_OK) return rc;
  EPP_CUDA_TRY(cudaMemsetAsync(valid_len_dev, 0, sizeof(int), s));
  EPP_CUDA_TRY(cudaMemsetAsync(status_dev, 0, sizeof(int), s));
  if (length == 0) return EPP_OK;
  EPP_REQUIRE(edge_mask && col_idx && out_id && out_edge, "null pointer");
  const int tiles = static_cast<int>(ceil_div_ll(length, kCompactTile));
  ScanHeader *hdr = static_cast<ScanHeader *>(scratch);
  unsigned long long *desc = reinterpret_cast<unsigned long long *>(hdr + 1);
  // The array keeps the previous call's ticket, error word and descriptors:
  // everything this call will read has to start from zero again.
  EPP_CUDA_TRY(cudaMemsetAsync(scratch, 0, scan_scratch_bytes(tiles), s));
  compact_mask_kernel<kLookback><<<tiles, kScanThreads, 0, s>>>(edge_mask, col_idx, out_id, out_edge, length,
                                                                tiles, hdr, desc, valid_len_dev);
  EPP_CHECK_LAUNCH("compact_mask_kernel<lookback, static scratch>");
  zero_tail_kernel<<<tail_grid(length), 256, 0, s>>>(out_id, out_edge, valid_len_dev, 0, length);
  EPP_CHECK_LAUNCH("zero_tail_kernel");
  publish_status_kernel<<<1, 1, 0, s>>>(hdr, status_dev);
  EPP_CHECK_LAUNCH("publish_status_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_split_parts(const int *node_deg, int num_nodes, int part_size, int *part_pointer,
                                  int out_len, void *scratch, size_t scratch_bytes, int *num_parts_dev,
                                  int *status_dev, int mode, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(num_nodes >= 0 && out_len >= 0, "negative size");
  EPP_REQUIRE(part_size >= 1, "back part size must be >= 1");
  EPP_REQUIRE(num_parts_dev && status_dev, "null result pointer");
  EPP_REQUIRE(mode == 0 || mode == 1, "mode must be 0 or 1");
  EPP_CUDA_TRY(cudaMemsetAsync(num_parts_dev, 0, sizeof(int), s));
  EPP_CUDA_TRY(cudaMemsetAsync(status_dev, 0, sizeof(int), s));
  EPP_REQUIRE(out_len == 0 || part_pointer, "null pointer");
  if (num_nodes == 0) {
    if (out_len) EPP_CUDA_TRY(cudaMemsetAsync(part_pointer, 0, sizeof(int) * static_cast<size_t>(out_len), s));
    return EPP_OK;
  }
  EPP_REQUIRE(node_deg && scratch, "null pointer");
  EPP_REQUIRE(scratch_bytes >= eppgcn_split_scratch_bytes(num_nodes), "scratch too small");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(scratch) % 8 == 0, "scratch must be 8-byte aligned");
  const int tiles = static_cast<int>(ceil_div_ll(num_nodes, kSplitTile));
  ScanHeader *hdr = static_cast<ScanHeader *>(scratch);
  unsigned long long *desc = reinterpret_cast<unsigned long long *>(hdr + 1);
  EPP_CUDA_TRY(cudaMemsetAsync(scratch, 0, scan_scratch_bytes(tiles), s));
  if (mode == 0) {
    split_parts_kernel<kLookback><<<tiles, kScanThreads, 0, s>>>(node_deg, num_nodes, part_size, part_pointer,
                                                                 out_len, tiles, hdr, desc, num_parts_dev);
    EPP_CHECK_LAUNCH("split_parts_kernel<lookback>");
  } else {
    split_parts_kernel<kCountOnly><<<tiles, kScanThreads, 0, s>>>(node_deg, num_nodes, part_size, part_pointer,
                                                                  out_len, tiles, hdr, desc, num_parts_dev);
    EPP_CHECK_LAUNCH("split_parts_kernel<count>");
    scan_tiles_kernel<<<1, 1024, 0, s>>>(desc, tiles);
    EPP_CHECK_LAUNCH("scan_tiles_kernel");
    split_parts_kernel<kGivenOffsets><<<tiles, kScanThreads, 0, s>>>(node_deg, num_nodes, part_size,
                                                                     part_pointer, out_len, tiles, hdr, desc,
                                                                     num_parts_dev);
    EPP_CHECK_LAUNCH("split_parts_kernel<scatter>");
  }
  if (out_len) {
    zero_tail_kernel<<<tail_grid(out_len), 256, 0, s>>>(part_pointer, nullptr, num_parts_dev, 1, out_len);
    EPP_CHECK_LAUNCH("zero_tail_kernel");
  }
  publish_status_kernel<<<1, 1, 0, s>>>(hdr, status_dev);
  EPP_CHECK_LAUNCH("publish_status_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_count_nonzero(const int *values, int length, int *count_dev, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(length >= 0 && count_dev, "bad argument");
  EPP_CUDA_TRY(cudaMemsetAsync(count_dev, 0, sizeof(int), s));
  if (length == 0) return EPP_OK;
  EPP_REQUIRE(values, "null pointer");
  count_nonzero_kernel<<<tail_grid(length), 256, 0, s>>>(values, length, count_dev);
  EPP_CHECK_LAUNCH("count_nonzero_kernel");
  return EPP_OK;
}

// ---------------------------------------------------------------------------
// Neighbour groups on the device.  build_part (EPPGCN.cpp:186-227) and the
// part splitting compute the same thing from different inputs: a vertex with d
// edges yields ceil(d / part_size) consecutive pieces of its edge range.  With
// the row lengths of the CSR as "node degrees", the splitting kernel's part
// pointers are the group pointers (edge offsets equal CSR offsets), and the
// vertex it finds for every slot is part2Node.
// ---------------------------------------------------------------------------
EPP_EXPORT size_t eppgcn_build_part_scratch_bytes(int num_nodes) {
  const size_t n = num_nodes < 0 ? 0 : static_cast<size_t>(num_nodes);
  return (eppgcn_split_scratch_bytes(num_nodes) + 255) / 256 * 256 + sizeof(int) * (n + 1);
}

EPP_EXPORT int eppgcn_build_part(const int *row_ptr, int num_nodes, int part_size, int *part_ptr, int part_ptr_len,
                                 int *part2node, int part2node_len, void *scratch, size_t scratch_bytes,
                                 int *num_parts_dev, int *status_dev, int mode, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_REQUIRE(num_nodes >= 0 && part_ptr_len >= 0 && part2node_len >= 0, "negative size");
  EPP_REQUIRE(part_size >= 1, "part size must be >= 1");
  EPP_REQUIRE(num_parts_dev && status_dev, "null result pointer");
  EPP_REQUIRE(mode == 0 || mode == 1, "mode must be 0 or 1");
  EPP_CUDA_TRY(cudaMemsetAsync(num_parts_dev, 0, sizeof(int), s));
  EPP_CUDA_TRY(cudaMemsetAsync(status_dev, 0, sizeof(int), s));
  EPP_REQUIRE(part_ptr_len == 0 || part_ptr, "null pointer");
  EPP_REQUIRE(part2node_len == 0 || part2node, "null pointer");
  if (num_nodes == 0) {
    if (part_ptr_len) EPP_CUDA_TRY(cudaMemsetAsync(part_ptr, 0, sizeof(int) * static_cast<size_t>(part_ptr_len), s));
    return EPP_OK;
  }
  EPP_REQUIRE(row_ptr && scratch, "null pointer");
  EPP_REQUIRE(scratch_bytes >= eppgcn_build_part_scratch_bytes(num_nodes), "scratch too small");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(scratch) % 8 == 0, "scratch must be 8-byte aligned");
  const size_t scan_bytes = (eppgcn_split_scratch_bytes(num_nodes) + 255) / 256 * 256;
  int *deg = reinterpret_cast<int *>(static_cast<char *>(scratch) + scan_bytes);
  row_lengths_kernel<<<static_cast<unsigned>(ceil_div_ll(num_nodes, 256)), 256, 0, s>>>(row_ptr, num_nodes, deg);
  EPP_CHECK_LAUNCH("row_lengths_kernel");
  const int tiles = static_cast<int>(ceil_div_ll(num_nodes, kSplitTile));
  ScanHeader *hdr = static_cast<ScanHeader *>(scratch);
  unsigned long long *desc = reinterpret_cast<unsigned long long *>(hdr + 1);
  EPP_CUDA_TRY(cudaMemsetAsync(scratch, 0, scan_scratch_bytes(tiles), s));
  if (mode == 0) {
    split_parts_kernel<kLookback><<<tiles, kScanThreads, 0, s>>>(deg, num_nodes, part_size, part_ptr, part_ptr_len,
                                                                 tiles, hdr, desc, num_parts_dev, part2node,
                                                                 part2node_len);
    EPP_CHECK_LAUNCH("split_parts_kernel<lookback, groups>");
  } else {
    split_parts_kernel<kCountOnly><<<tiles, kScanThreads, 0, s>>>(deg, num_nodes, part_size, part_ptr, part_ptr_len,
                                                                  tiles, hdr, desc, num_parts_dev);
    EPP_CHECK_LAUNCH("split_parts_kernel<count>");
    scan_tiles_kernel<<<1, 1024, 0, s>>>(desc, tiles);
    EPP_CHECK_LAUNCH("scan_tiles_kernel");
    split_parts_kernel<kGivenOffsets><<<tiles, kScanThreads, 0, s>>>(deg, num_nodes, part_size, part_ptr,
                                                                     part_ptr_len, tiles, hdr, desc, num_parts_dev,
                                                                     part2node, part2node_len);
    EPP_CHECK_LAUNCH("split_parts_kernel<scatter, groups>");
  }
  publish_status_kernel<<<1, 1, 0, s>>>(hdr, status_dev);
  EPP_CHECK_LAUNCH("publish_status_kernel");
  return EPP_OK;
}
