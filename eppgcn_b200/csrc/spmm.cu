// Neighbour-group aggregation kernels for sm_100a: the forward SpMM over the
// build_part groups and the backward SpMM over the compacted execution path.
//
// Both directions run one persistent kernel template.
//
// Mapping.  A "sub-warp" of LPR lanes owns one group (at most part_size
// consecutive edges of one row) at a time; a lane owns T tiles of VEC
// consecutive feature columns (tile k starts at column (k*LPR + lane)*VEC), so
// one warp-level load instruction fetches VEC*LPR*4 contiguous bytes of
// 32/LPR different neighbour rows.  Narrow rows (16 or 22 floats) use 4 lanes
// per row, i.e. 8 rows per warp instruction; wide rows keep 4 lanes and add
// tiles, so the per-edge index work is amortised over more bytes.
//
// Staging.  A warp walks over "sets" of 32/LPR consecutive groups.  The column
// ids of a set are one contiguous slice of the edge array; the warp copies that
// slice into its private shared-memory slab with cp.async while it is still
// busy with the previous set (two slabs per warp), and the group descriptors of
// the set after that are already on their way in registers.  Inside a set the
// only exposed memory latency is the gather itself: a lane keeps up to eight
// 16-byte row loads in flight and reads the column id as a shared-memory
// broadcast.  The source-side degree is either a sub-warp-uniform cached load
// (HASW) or absent: when the producer of the feature rows has already
// multiplied them by the degree (deg_col == NULL), an edge costs one id and
// one row and nothing else.
//
// Reduction.  After the edge loop the sub-warps of a warp that worked on the
// same row are combined with a segmented shuffle reduction, and only the head
// of each run touches memory: a plain vector store when the run covers the
// whole row, a vector atomic add otherwise (a row split across warps).
#include <mutex>

#include "rowio.cuh"

namespace epp {
namespace {

template <int VEC>
__device__ __forceinline__ void load_vec(const float *p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (VEC == 2) {
    float2 t = __ldg(reinterpret_cast<const float2 *>(p));
    v[0] = t.x; v[1] = t.y;
  } else {
    v[0] = __ldg(p);
  }
}

struct GroupArgs {
  float *out;              // [num_rows][dim], rows out_ld floats apart
  long long out_ld;
  const float *feat;       // rows of stride ld
  long long ld;
  const int *part_ptr;     // [num_parts+1]
  const int *row_of;       // forward: part2node[num_parts]; backward: ids[] per compacted edge
  const int *col;          // column id per edge
  const float *deg_row;
  const float *deg_col;
  int num_parts;
  int dim;
  int ovec;                // widest aligned access into `out`: 4, 2 or 1 floats
  int bwd;                 // 0: groups over a CSR (part2node), 1: parts over the compacted edge list (ids)
};

__device__ __forceinline__ void cp_async_4(int *smem_dst, const int *gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_16(int *smem_dst, const int *gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct SetMeta {
  int beg, end, row;   // this sub-warp's group: edge range and destination row (-1: nothing to do)
  int lo, hi;          // row of the group before / after this one (-1 at either end of the list)
};

// bwd = 0: groups (part_ptr, part2node) from build_part.  A row's groups are
//              consecutive, so a run of groups covers its whole row exactly when
//              the groups on either side belong to other rows.
// bwd = 1: parts over the compacted edge list; the row of a part is
//              ids[part_ptr[p]], and the rows on either side are the ids of the
//              edge before the part and of the edge after it.
__device__ __forceinline__ SetMeta load_set_meta(const GroupArgs &a, int g, int total_edges) {
  SetMeta m{0, 0, -1, -1, -1};
  if (g < a.num_parts) {
    m.beg = __ldg(a.part_ptr + g);
    m.end = __ldg(a.part_ptr + g + 1);
    if (a.bwd) {
      if (m.end > m.beg) {
        m.row = __ldg(a.row_of + m.beg);
        m.lo = m.beg > 0 ? __ldg(a.row_of + m.beg - 1) : -1;
        m.hi = m.end < total_edges ? __ldg(a.row_of + m.end) : -1;
      }
    } else {
      m.row = __ldg(a.row_of + g);
      m.lo = g > 0 ? __ldg(a.row_of + g - 1) : -1;
      m.hi = g + 1 < a.num_parts ? __ldg(a.row_of + g + 1) : -1;
    }
    if (m.end <= m.beg) { m.end = m.beg; m.row = -1; }
  }
  return m;
}

// N edges of one group: all loads are issued before the first use.  `cs` points
// at the group's column ids (shared-memory slab, or global memory when the set
// did not fit its slab).  FULL: every sub-warp of the warp has all N edges, so
// no edge bound is tested.  `tiles` is the lane's bit mask of tiles that hold
// feature columns (only looked at when a lane owns more than one tile).
template <int VEC, int T, int N, bool FULL, bool HASW>
__device__ __forceinline__ void gather_batch(const int *cs, int i0, int len, unsigned tiles, const char *fbytes,
                                             unsigned ld_bytes, unsigned tile_bytes, const float *deg_col,
                                             float (&acc)[T][VEC]) {
  int c[N];
  float w[N];
  float v[N][T][VEC];
#pragma unroll
  for (int u = 0; u < N; ++u) c[u] = (FULL || i0 + u < len) ? cs[i0 + u] : -1;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    if (FULL || c[u] >= 0) {
      w[u] = HASW ? __ldg(deg_col + c[u]) : 1.f;
      const char *rowp = fbytes + static_cast<unsigned long long>(static_cast<unsigned>(c[u])) * ld_bytes;
#pragma unroll
      for (int k = 0; k < T; ++k) {
        if (T == 1 || ((tiles >> k) & 1u)) {
          load_vec<VEC>(reinterpret_cast<const float *>(rowp + k * tile_bytes), v[u][k]);
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) v[u][k][i] = 0.f;
        }
      }
    } else {
      w[u] = 0.f;
#pragma unroll
      for (int k = 0; k < T; ++k)
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[u][k][i] = 0.f;
    }
  }
#pragma unroll
  for (int u = 0; u < N; ++u)
#pragma unroll
    for (int k = 0; k < T; ++k)
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        acc[k][i] = HASW ? fmaf(w[u], v[u][k][i], acc[k][i]) : acc[k][i] + v[u][k][i];   // rows beyond len are zero
}

// One launch covers feature columns [0, min(dim_left, VEC*LPR*T)) of the
// pointers it is given; wider rows are handled by the host with further
// launches on shifted pointers.
template <int VEC, int LPR, int T, bool HASW>
__global__ void __launch_bounds__(256, (T <= 4 ? 3 : 2))
staged_spmm_kernel(const GroupArgs a, const int cols, const int slab, const int col_aligned) {
  constexpr int G = kWarp / LPR;               // groups per set
  constexpr int U = T >= 8 ? 1 : 8 / T;        // edges per batch: U*T row loads in flight per lane
  extern __shared__ __align__(16) int s_cols[];
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const int wib = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  int *const slab0 = s_cols + (wib * 2) * slab;   // this warp's two slabs: slab0 + cur * slab
  const int nsets = (a.num_parts + G - 1) / G;
  const int stride = gridDim.x * wpb;
  int set = blockIdx.x * wpb + wib;
  if (set >= nsets) return;
  const int total_edges = __ldg(a.part_ptr + a.num_parts);
  const unsigned ld_bytes = static_cast<unsigned>(a.ld) * 4u;
  constexpr unsigned tile_bytes = VEC * LPR * 4u;

  // Column ownership of this lane: the same for every set.
  const int fcol = sl * VEC;
  unsigned tiles = 0;
#pragma unroll
  for (int k = 0; k < T; ++k)
    if (fcol + k * VEC * LPR < cols) tiles |= 1u << k;
  const char *fbytes = reinterpret_cast<const char *>(a.feat + fcol);

  // Starts the copy of one set's column ids; returns the first edge held by the
  // slab, or -1 when the slice cannot be staged (too long for the slab, or its
  // last 16-byte chunk would reach past the edge array); such a set reads its
  // column ids from global memory.
  auto stage = [&](const SetMeta &m, int *dst) -> int {
    const int send = __reduce_max_sync(kFull, m.end);
    const int sbeg = __shfl_sync(kFull, m.beg, 0);
    if (col_aligned) {
      const int abase = sbeg & ~3;
      const int count = (send - abase + 3) & ~3;
      if (send <= sbeg || count > slab || abase + count > total_edges) return -1;
      for (int j = lane * 4; j < count; j += kWarp * 4) cp_async_16(dst + j, a.col + abase + j);
      return abase;
    }
    const int count = send - sbeg;
    if (count <= 0 || count > slab) return -1;
    for (int j = lane; j < count; j += kWarp) cp_async_4(dst + j, a.col + sbeg + j);
    return sbeg;
  };

  SetMeta m0 = load_set_meta(a, set * G + sub, total_edges);
  SetMeta m1 = load_set_meta(a, set + stride < nsets ? (set + stride) * G + sub : a.num_parts, total_edges);
  int base0 = stage(m0, slab0);
  cp_async_commit();
  float wr0 = m0.row >= 0 ? __ldg(a.deg_row + m0.row) : 0.f;
  int cur = 0;

  for (; set < nsets; set += stride) {
    const int set2 = set + 2 * stride;
    const SetMeta m2 = load_set_meta(a, set2 < nsets ? set2 * G + sub : a.num_parts, total_edges);
    const int base1 = stage(m1, slab0 + (cur ^ 1) * slab);
    cp_async_commit();
    const float wr1 = m1.row >= 0 ? __ldg(a.deg_row + m1.row) : 0.f;
    cp_async_wait<1>();
    __syncwarp();

    const int len = (tiles && m0.row >= 0) ? m0.end - m0.beg : 0;   // lanes without columns gather nothing
    const int maxlen = __reduce_max_sync(kFull, len);
    const int minlen = __reduce_min_sync(kFull, len);
    const int *cs = base0 >= 0 ? slab0 + cur * slab + (m0.beg - base0) : a.col + m0.beg;

    float acc[T][VEC];
#pragma unroll
    for (int k = 0; k < T; ++k)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[k][i] = 0.f;

    int i0 = 0;
#pragma unroll 1
    for (; i0 + U <= minlen; i0 += U)
      gather_batch<VEC, T, U, true, HASW>(cs, i0, len, tiles, fbytes, ld_bytes, tile_bytes, a.deg_col, acc);
#pragma unroll 1
    for (; i0 + U <= maxlen; i0 += U)
      gather_batch<VEC, T, U, false, HASW>(cs, i0, len, tiles, fbytes, ld_bytes, tile_bytes, a.deg_col, acc);
    // warp-uniform tail: 4 + 2 + 1 covers any remainder below 8
    if (U > 4 && maxlen - i0 >= 4) {
      gather_batch<VEC, T, 4, false, HASW>(cs, i0, len, tiles, fbytes, ld_bytes, tile_bytes, a.deg_col, acc);
      i0 += 4;
    }
    if (U > 2 && maxlen - i0 >= 2) {
      gather_batch<VEC, T, 2, false, HASW>(cs, i0, len, tiles, fbytes, ld_bytes, tile_bytes, a.deg_col, acc);
      i0 += 2;
    }
    if (U > 1 && maxlen - i0 >= 1)
      gather_batch<VEC, T, 1, false, HASW>(cs, i0, len, tiles, fbytes, ld_bytes, tile_bytes, a.deg_col, acc);
#pragma unroll
    for (int k = 0; k < T; ++k)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[k][i] *= wr0;

    // Sub-warps with the same row are neighbours (lo of one is the row of the
    // one before); when no two neighbours agree there is nothing to combine.
    const bool cont = sub > 0 && m0.row >= 0 && m0.lo == m0.row;
    int rhi = m0.hi;
    if (__any_sync(kFull, cont)) {
#pragma unroll
      for (int off = LPR; off < kWarp; off <<= 1) {
        const int orow = __shfl_down_sync(kFull, m0.row, off);
        const int ohi = __shfl_down_sync(kFull, rhi, off);
        const bool take = lane + off < kWarp && m0.row >= 0 && orow == m0.row;
#pragma unroll
        for (int k = 0; k < T; ++k)
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float o = __shfl_down_sync(kFull, acc[k][i], off);
            if (take) acc[k][i] += o;
          }
        if (take) rhi = ohi;
      }
    }
    if (m0.row >= 0 && !cont && tiles) {
      const bool whole = m0.lo != m0.row && rhi != m0.row;
      float *dst = a.out + static_cast<long long>(m0.row) * a.out_ld + fcol;
#pragma unroll
      for (int k = 0; k < T; ++k) {
        if ((tiles >> k) & 1u) {
          const int n = min(VEC, cols - (fcol + k * VEC * LPR));
          if (whole) store_row<VEC>(dst + k * VEC * LPR, acc[k], n, a.ovec);
          else add_row<VEC>(dst + k * VEC * LPR, acc[k], n, a.ovec);
        }
      }
    }
    __syncwarp();   // everyone is done with the current slab before the next iteration refills it
    m0 = m1; m1 = m2; base0 = base1; wr0 = wr1; cur ^= 1;
  }
  cp_async_wait<0>();
}

// Launch geometry of one kernel instantiation, remembered per device: the
// shared-memory opt-in is a per-device attribute and the occupancy answer
// belongs to the device that gave it.
struct LaunchInfo {
  int blocks_per_sm = 0;
  int smem = -1;
  int num_sms = 0;
};
constexpr int kMaxDevices = 64;

template <int VEC, int LPR, int T, bool HASW>
int launch_staged(const GroupArgs &a0, int part_size, cudaStream_t s) {
  constexpr int G = kWarp / LPR;
  constexpr int SPAN = VEC * LPR * T;           // feature columns per launch
  const int ps = part_size >= 1 ? part_size : 32;
  const long long want = static_cast<long long>(G) * ps + 8;
  const int slab = static_cast<int>(want > 1024 ? 1024 : (want + 3) / 4 * 4);
  const int smem = slab * 2 * 8 * static_cast<int>(sizeof(int));
  static LaunchInfo per_device[kMaxDevices];   // per instantiation and device
  static std::mutex mu;
  int dev = 0;
  EPP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device ordinal %d is beyond the %d devices this library tracks", dev, kMaxDevices);
    return EPP_ERR_TOO_LARGE;
  }
  LaunchInfo info;
  {
    std::lock_guard<std::mutex> lock(mu);
    LaunchInfo &slot = per_device[dev];
    if (slot.smem != smem) {             // first launch on this device, or another slab size
      EPP_CUDA_TRY(cudaDeviceGetAttribute(&slot.num_sms, cudaDevAttrMultiProcessorCount, dev));
      if (smem > 48 * 1024)
        EPP_CUDA_TRY(cudaFuncSetAttribute(staged_spmm_kernel<VEC, LPR, T, HASW>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      EPP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&slot.blocks_per_sm,
                                                                 staged_spmm_kernel<VEC, LPR, T, HASW>, 256, smem));
      if (slot.blocks_per_sm < 1) slot.blocks_per_sm = 1;
      slot.smem = smem;
    }
    info = slot;
  }
  const long long nsets = ceil_div_ll(a0.num_parts, G);
  long long blocks = ceil_div_ll(nsets, 8);
  const long long cap = static_cast<long long>(info.num_sms) * info.blocks_per_sm;
  if (blocks > cap) blocks = cap;
  const int col_aligned = aligned(a0.col, 16) ? 1 : 0;
  for (int col0 = 0; col0 < a0.dim; col0 += SPAN) {     // one launch unless the row is wider than SPAN
    GroupArgs a = a0;
    a.feat = a0.feat + col0;
    a.out = a0.out + col0;
    const int cols = a0.dim - col0 < SPAN ? a0.dim - col0 : SPAN;
    staged_spmm_kernel<VEC, LPR, T, HASW><<<static_cast<unsigned>(blocks), 256, smem, s>>>(a, cols, slab, col_aligned);
    EPP_CHECK_LAUNCH("staged_spmm_kernel");
  }
  return EPP_OK;
}

// Lanes per row and tiles per lane for a row of `lanes_needed` VEC-wide pieces.
template <int VEC, bool HASW>
int launch_shape(const GroupArgs &a, int lanes_needed, int part_size, cudaStream_t s) {
  if (lanes_needed <= 1) return launch_staged<VEC, 1, 1, HASW>(a, part_size, s);
  if (lanes_needed <= 2) return launch_staged<VEC, 2, 1, HASW>(a, part_size, s);
  if (lanes_needed <= 4) return launch_staged<VEC, 4, 1, HASW>(a, part_size, s);
  if (lanes_needed <= 8) return launch_staged<VEC, 4, 2, HASW>(a, part_size, s);
  if (lanes_needed <= 12) return launch_staged<VEC, 4, 3, HASW>(a, part_size, s);
  if (lanes_needed <= 16) return launch_staged<VEC, 4, 4, HASW>(a, part_size, s);
  if (lanes_needed <= 32) return launch_staged<VEC, 4, 8, HASW>(a, part_size, s);
  if (lanes_needed <= 64) return launch_staged<VEC, 8, 8, HASW>(a, part_size, s);
  if (lanes_needed <= 128) return launch_staged<VEC, 16, 8, HASW>(a, part_size, s);
  return launch_staged<VEC, 32, 8, HASW>(a, part_size, s);   // wider rows take several passes
}

// Zeroes columns 0 .. dim-1 of rows that are out_ld floats apart, W floats per store.
template <int W>
__global__ void __launch_bounds__(256) zero_column_block_kernel(float *out, long long out_ld, int dim, long long num_rows) {
  const int per_row = dim / W;
  const long long total = num_rows * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float *p = out + (i / per_row) * out_ld + (i % per_row) * W;
    if constexpr (W == 4) *reinterpret_cast<float4 *>(p) = make_float4(0.f, 0.f, 0.f, 0.f);
    else if constexpr (W == 2) *reinterpret_cast<float2 *>(p) = make_float2(0.f, 0.f);
    else *p = 0.f;
  }
}

}  // namespace

int zero_column_block(float *out, long long out_ld, int dim, long long num_rows, cudaStream_t s) {
  int w = 1;
  if (dim % 4 == 0 && out_ld % 4 == 0 && aligned(out, 16)) w = 4;
  else if (dim % 2 == 0 && out_ld % 2 == 0 && aligned(out, 8)) w = 2;
  const long long total = num_rows * (dim / w);
  long long blocks = ceil_div_ll(total, 256 * 4);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  if (w == 4) zero_column_block_kernel<4><<<static_cast<unsigned>(blocks), 256, 0, s>>>(out, out_ld, dim, num_rows);
  else if (w == 2) zero_column_block_kernel<2><<<static_cast<unsigned>(blocks), 256, 0, s>>>(out, out_ld, dim, num_rows);
  else zero_column_block_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(out, out_ld, dim, num_rows);
  EPP_CHECK_LAUNCH("zero_column_block_kernel");
  return EPP_OK;
}

namespace {

template <bool HASW>
int launch_group_spmm(GroupArgs a, int num_rows, int part_size, cudaStream_t s) {
  // Dense result: rows that no group touches, and rows that are accumulated
  // with atomics, start from zero.
  if (a.out_ld == a.dim)
    EPP_CUDA_TRY(cudaMemsetAsync(a.out, 0, sizeof(float) * static_cast<size_t>(num_rows) * a.dim, s));
  else if (const int rc = zero_column_block(a.out, a.out_ld, a.dim, num_rows, s); rc != EPP_OK)
    return rc;
  if (a.num_parts == 0) return EPP_OK;
  if (a.ld > 0x3fffffffLL) {
    set_error("row stride too large");
    return EPP_ERR_TOO_LARGE;
  }
  // Widest gather: the lane's VEC floats must be aligned and inside the row stride.
  int vec = 1;
  if (a.ld % 4 == 0 && aligned(a.feat, 16) && a.ld >= ((a.dim + 3) / 4) * 4) vec = 4;
  else if (a.ld % 2 == 0 && aligned(a.feat, 8) && a.ld >= ((a.dim + 1) / 2) * 2) vec = 2;
  a.ovec = 1;
  if (a.out_ld % 4 == 0 && aligned(a.out, 16)) a.ovec = 4;
  else if (a.out_ld % 2 == 0 && aligned(a.out, 8)) a.ovec = 2;
  const int lanes_needed = (a.dim + vec - 1) / vec;
  switch (vec) {
    case 4:  return launch_shape<4, HASW>(a, lanes_needed, part_size, s);
    case 2:  return launch_shape<2, HASW>(a, lanes_needed, part_size, s);
    default: return launch_shape<1, HASW>(a, lanes_needed, part_size, s);
  }
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_spmm_forward(float *out, long long out_ld, const float *feat, long long feat_ld,
                                   const int *row_ptr, const int *col_idx,
                                   const float *deg_row, const float *deg_col,
                                   const int *part_ptr, const int *part2node,
                                   int num_nodes, int dim, int num_parts,
                                   int part_size, int dim_worker, int warp_per_block,
                                   void *stream) {
  (void)dim_worker; (void)warp_per_block;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(feat_ld >= dim, "feat_ld must be >= dim");
  EPP_REQUIRE(out_ld == 0 || out_ld >= dim, "out_ld must be 0 or >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(out && feat && row_ptr && deg_row, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (col_idx && part_ptr && part2node), "null pointer");
  epp::GroupArgs a{};
  a.out = out; a.out_ld = out_ld ? out_ld : dim; a.feat = feat; a.ld = feat_ld;
  a.part_ptr = part_ptr; a.row_of = part2node; a.col = col_idx;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim; a.bwd = 0;
  return deg_col ? epp::launch_group_spmm<true>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream))
                 : epp::launch_group_spmm<false>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream));
}

EPP_EXPORT int eppgcn_spmm_backward_compacted(float *d_in, long long d_in_ld, const float *d_out, long long d_out_ld,
                                              const int *ids, const int *part_ptr, const int *edge_list,
                                              const float *deg_row, const float *deg_col,
                                              int num_nodes, int dim, int num_parts,
                                              int part_size, int blockx, int blocky,
                                              void *stream) {
  (void)blockx; (void)blocky;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(d_out_ld >= dim, "d_out_ld must be >= dim");
  EPP_REQUIRE(d_in_ld == 0 || d_in_ld >= dim, "d_in_ld must be 0 or >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(d_in && d_out && deg_row, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (ids && part_ptr && edge_list), "null pointer");
  epp::GroupArgs a{};
  a.out = d_in; a.out_ld = d_in_ld ? d_in_ld : dim; a.feat = d_out; a.ld = d_out_ld;
  a.part_ptr = part_ptr; a.row_of = ids; a.col = edge_list;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim; a.bwd = 1;
  return deg_col ? epp::launch_group_spmm<true>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream))
                 : epp::launch_group_spmm<false>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream));
}
