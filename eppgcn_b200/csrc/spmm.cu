// Neighbour-group aggregation kernels for sm_100a: the forward SpMM over the
// build_part groups and the backward SpMM over the compacted execution path.
//
// Both directions run one kernel template.  A "sub-warp" of LPR lanes owns one
// group (at most part_size consecutive edges of one row); each lane owns VEC
// consecutive feature columns, so a neighbour row is fetched with one 4/8/16
// byte load per lane and one warp-level load instruction gathers 32/LPR
// different neighbour rows.  Column ids and the edge weight deg[r]*deg[c] are
// loaded once per edge by one lane and broadcast with shuffles.  After the
// edge loop the sub-warps of a warp that worked on the same row are combined
// with a segmented shuffle reduction, and only the head of each run touches
// memory: a plain vector store when the run covers the whole row, a vector
// atomic add otherwise (a row split across warps).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace epp {
namespace {

inline bool aligned(const void *p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

template <int VEC> struct VecT;
template <> struct VecT<4> { using type = float4; };
template <> struct VecT<2> { using type = float2; };
template <> struct VecT<1> { using type = float; };

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

// Writes n (<= VEC) floats starting at p with the widest store `ovec` allows.
template <int VEC>
__device__ __forceinline__ void store_row(float *p, const float (&v)[VEC], int n, int ovec) {
  if (VEC == 4 && ovec == 4 && n == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if (VEC >= 2 && ovec >= 2) {
#pragma unroll
    for (int i = 0; i + 1 < VEC; i += 2)
      if (i + 1 < n) *reinterpret_cast<float2 *>(p + i) = make_float2(v[i], v[i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) p[i] = v[i];
  }
}

template <int VEC>
__device__ __forceinline__ void add_row(float *p, const float (&v)[VEC], int n, int ovec) {
  if (VEC == 4 && ovec == 4 && n == 4) {
    atomicAdd(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
  } else if (VEC >= 2 && ovec >= 2) {
#pragma unroll
    for (int i = 0; i + 1 < VEC; i += 2)
      if (i + 1 < n) atomicAdd(reinterpret_cast<float2 *>(p + i), make_float2(v[i], v[i + 1]));
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) atomicAdd(p + i, v[i]);
  }
}

struct GroupArgs {
  float *out;              // [num_rows][dim]
  const float *feat;       // rows of stride ld
  long long ld;
  const int *part_ptr;     // [num_parts+1]
  const int *row_of;       // forward: part2node[num_parts]; backward: ids[] per compacted edge
  const int *row_ptr;      // forward only
  const int *col;          // column id per edge
  const float *deg_row;
  const float *deg_col;
  int num_parts;
  int dim;
  int ovec;                // widest aligned access into `out`: 4, 2 or 1 floats
};

// BWD = false: groups (part_ptr, part2node) over a CSR (row_ptr).
// BWD = true : parts over the compacted edge list; the row of a part is
//              ids[part_ptr[p]] and the extent of a row is found by looking at
//              the ids on either side of the run.
template <int VEC, int LPR, bool BWD>
__global__ void __launch_bounds__(256) group_spmm_kernel(const GroupArgs a) {
  constexpr int G = kWarp / LPR;          // groups per warp
  constexpr int U = LPR < 8 ? LPR : 8;    // neighbour rows in flight per lane
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const long long warp = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long g = warp * G + sub;

  int beg = 0, end = 0, row = -1;
  if (g < a.num_parts) {
    beg = __ldg(a.part_ptr + g);
    end = __ldg(a.part_ptr + g + 1);
    if (end > beg) row = BWD ? __ldg(a.row_of + beg) : __ldg(a.row_of + g);
    else end = beg;
  }
  const float wr = row >= 0 ? __ldg(a.deg_row + row) : 0.f;
  int iters = (end - beg + LPR - 1) / LPR;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) iters = max(iters, __shfl_xor_sync(kFull, iters, off));

  // Run bookkeeping is the same for every column tile; computed once below.
  int run_end = end;
  bool head = false, whole = false;

  for (int tile = 0; tile < a.dim; tile += VEC * LPR) {
    const int fcol = tile + sl * VEC;
    const bool fact = fcol < a.dim;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

    for (int it = 0; it < iters; ++it) {
      const int e0 = beg + it * LPR;
      const int e = e0 + sl;
      int c = 0;
      float w = 0.f;
      if (e < end) {
        c = __ldg(a.col + e);
        w = __fmul_rn(wr, __ldg(a.deg_col + c));
      }
#pragma unroll
      for (int j0 = 0; j0 < LPR; j0 += U) {
        float v[U][VEC];
        float wj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int cj = __shfl_sync(kFull, c, j0 + u, LPR);
          wj[u] = __shfl_sync(kFull, w, j0 + u, LPR);
          if (fact && e0 + j0 + u < end) {
            load_vec<VEC>(a.feat + static_cast<long long>(cj) * a.ld + fcol, v[u]);
          } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[u][i] = 0.f;
            wj[u] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[i] = fmaf(wj[u], v[u][i], acc[i]);
      }
    }

    // Segmented reduction over the sub-warps of this warp that share a row.
    int rend = end;
#pragma unroll
    for (int off = LPR; off < kWarp; off <<= 1) {
      const int orow = __shfl_down_sync(kFull, row, off);
      const int oend = __shfl_down_sync(kFull, rend, off);
      float o[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = __shfl_down_sync(kFull, acc[i], off);
      if (lane + off < kWarp && row >= 0 && orow == row) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] += o[i];
        rend = max(rend, oend);
      }
    }
    if (tile == 0) {
      run_end = rend;
      const int prow = __shfl_up_sync(kFull, row, LPR);
      head = row >= 0 && (sub == 0 || prow != row);
      if (head) {
        if (BWD) {
          const int total = __ldg(a.part_ptr + a.num_parts);
          whole = (beg == 0 || __ldg(a.row_of + beg - 1) != row) &&
                  (run_end >= total || __ldg(a.row_of + run_end) != row);
        } else {
          whole = beg == __ldg(a.row_ptr + row) && run_end == __ldg(a.row_ptr + row + 1);
        }
      }
    }
    if (head && fact) {
      float *dst = a.out + static_cast<long long>(row) * a.dim + fcol;
      const int n = min(VEC, a.dim - fcol);
      if (whole) store_row<VEC>(dst, acc, n, a.ovec);
      else add_row<VEC>(dst, acc, n, a.ovec);
    }
  }
}

// ---------------------------------------------------------------------------
// Staged, persistent variant.
//
// A warp walks over "sets" of G = 32/LPR consecutive groups.  The column ids of
// a set are one contiguous slice of the edge array; the warp copies that slice
// into its private shared-memory slab with cp.async while it is still busy with
// the previous set (two slabs per warp), and the group descriptors of the set
// after that are already on their way in registers.  Inside a set the only
// exposed memory latency is therefore the gather itself: every lane keeps
// eight neighbour rows in flight, reads the column id as a shared-memory
// broadcast and the source-side degree as a (sub-warp uniform) cached load.
// ---------------------------------------------------------------------------
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
  int lo, hi;          // forward: row_ptr[row], row_ptr[row+1]; backward: row id of the edge before / after
};

template <bool BWD>
__device__ __forceinline__ SetMeta load_set_meta(const GroupArgs &a, long long set, long long nsets, int groups,
                                                 int sub, int total_edges) {
  SetMeta m{0, 0, -1, -1, -1};
  const long long g = set * groups + sub;
  if (set < nsets && g < a.num_parts) {
    m.beg = __ldg(a.part_ptr + g);
    m.end = __ldg(a.part_ptr + g + 1);
    if (m.end > m.beg) {
      if (BWD) {
        m.row = __ldg(a.row_of + m.beg);
        m.lo = m.beg > 0 ? __ldg(a.row_of + m.beg - 1) : -1;
        m.hi = m.end < total_edges ? __ldg(a.row_of + m.end) : -1;
      } else {
        m.row = __ldg(a.row_of + g);
        m.lo = __ldg(a.row_ptr + m.row);
        m.hi = __ldg(a.row_ptr + m.row + 1);
      }
    } else {
      m.end = m.beg;
    }
  }
  return m;
}

// N neighbour rows of one group, all loads issued before the first use.
// `cs` points at the group's column ids (shared-memory slab or global memory).
template <int VEC, int N>
__device__ __forceinline__ void gather_batch(const int *cs, int i0, int len, bool fact, const char *fbytes,
                                             unsigned ld_bytes, const float *deg_col, float (&acc)[VEC]) {
  int c[N];
  float w[N];
  float v[N][VEC];
#pragma unroll
  for (int u = 0; u < N; ++u) c[u] = (fact && i0 + u < len) ? cs[i0 + u] : -1;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    if (c[u] >= 0) {
      w[u] = __ldg(deg_col + c[u]);
      load_vec<VEC>(reinterpret_cast<const float *>(fbytes + static_cast<unsigned long long>(static_cast<unsigned>(c[u])) * ld_bytes), v[u]);
    } else {
      w[u] = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[u][i] = 0.f;
    }
  }
#pragma unroll
  for (int u = 0; u < N; ++u)
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
}

template <int VEC, int LPR, bool BWD>
__global__ void __launch_bounds__(256) staged_spmm_kernel(const GroupArgs a, const int slab, const int col_aligned) {
  constexpr int G = kWarp / LPR;
  extern __shared__ __align__(16) int s_cols[];
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int sl = lane % LPR;
  const int wib = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  int *const slab0 = s_cols + (wib * 2) * slab;   // this warp's two slabs: slab0 + cur * slab
  const long long nsets = (static_cast<long long>(a.num_parts) + G - 1) / G;
  const long long stride = static_cast<long long>(gridDim.x) * wpb;
  long long set = static_cast<long long>(blockIdx.x) * wpb + wib;
  if (set >= nsets) return;
  const int total_edges = __ldg(a.part_ptr + a.num_parts);
  const unsigned ld_bytes = static_cast<unsigned>(a.ld) * 4u;

  // Starts the copy of one set's column ids; returns the first edge held by the
  // slab, or -1 when the slice does not fit (the set then reads global memory).
  auto stage = [&](const SetMeta &m, int *dst) -> int {
    const int send = __reduce_max_sync(kFull, m.end);
    const int sbeg = __shfl_sync(kFull, m.beg, 0);
    if (send <= sbeg) return -1;
    const int abase = col_aligned ? (sbeg & ~3) : sbeg;
    const int count = send - abase;
    if (count > slab) return -1;
    if (col_aligned) {
      for (int j = lane * 4; j < count; j += kWarp * 4) {
        if (abase + j + 4 <= total_edges) {
          cp_async_16(dst + j, a.col + abase + j);
        } else {
          for (int k = 0; k < 4; ++k)
            if (abase + j + k < send) cp_async_4(dst + j + k, a.col + abase + j + k);
        }
      }
    } else {
      for (int j = lane; j < count; j += kWarp) cp_async_4(dst + j, a.col + abase + j);
    }
    return abase;
  };

  SetMeta m0 = load_set_meta<BWD>(a, set, nsets, G, sub, total_edges);
  SetMeta m1 = load_set_meta<BWD>(a, set + stride, nsets, G, sub, total_edges);
  int base0 = stage(m0, slab0);
  cp_async_commit();
  float wr0 = m0.row >= 0 ? __ldg(a.deg_row + m0.row) : 0.f;
  int cur = 0;

  for (; set < nsets; set += stride) {
    const SetMeta m2 = load_set_meta<BWD>(a, set + 2 * stride, nsets, G, sub, total_edges);
    const int base1 = stage(m1, slab0 + (cur ^ 1) * slab);
    cp_async_commit();
    const float wr1 = m1.row >= 0 ? __ldg(a.deg_row + m1.row) : 0.f;
    cp_async_wait<1>();
    __syncwarp();

    const int len = m0.end - m0.beg;
    const int maxlen = __reduce_max_sync(kFull, len);
    const int *cs = base0 >= 0 ? slab0 + cur * slab + (m0.beg - base0) : a.col + m0.beg;
    // Sub-warps with the same row are neighbours; when no two neighbours agree the
    // shuffle reduction below has nothing to combine and is skipped.
    const int prow = __shfl_up_sync(kFull, m0.row, LPR);
    const bool cont = sub > 0 && m0.row >= 0 && prow == m0.row;
    const bool any_run = __any_sync(kFull, cont);

#pragma unroll 1
    for (int tile = 0; tile < a.dim; tile += VEC * LPR) {
      const int fcol = tile + sl * VEC;
      const bool fact = fcol < a.dim && m0.row >= 0;
      const char *fbytes = reinterpret_cast<const char *>(a.feat + fcol);
      float acc[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
      int i0 = 0;
#pragma unroll 1
      for (; i0 + 8 <= maxlen; i0 += 8) gather_batch<VEC, 8>(cs, i0, len, fact, fbytes, ld_bytes, a.deg_col, acc);
      // warp-uniform tail: 4 + 2 + 1 covers any remainder below 8
      if (maxlen - i0 >= 4) { gather_batch<VEC, 4>(cs, i0, len, fact, fbytes, ld_bytes, a.deg_col, acc); i0 += 4; }
      if (maxlen - i0 >= 2) { gather_batch<VEC, 2>(cs, i0, len, fact, fbytes, ld_bytes, a.deg_col, acc); i0 += 2; }
      if (maxlen - i0 >= 1) { gather_batch<VEC, 1>(cs, i0, len, fact, fbytes, ld_bytes, a.deg_col, acc); }
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] *= wr0;

      int rend = m0.end, rhi = m0.hi;
      if (any_run) {
#pragma unroll
        for (int off = LPR; off < kWarp; off <<= 1) {
          const int orow = __shfl_down_sync(kFull, m0.row, off);
          const int oend = __shfl_down_sync(kFull, rend, off);
          const int ohi = __shfl_down_sync(kFull, rhi, off);
          float o[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) o[i] = __shfl_down_sync(kFull, acc[i], off);
          if (lane + off < kWarp && m0.row >= 0 && orow == m0.row) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] += o[i];
            rend = max(rend, oend);
            rhi = ohi;
          }
        }
      }
      if (m0.row >= 0 && !cont && fcol < a.dim) {
        const bool whole = BWD ? (m0.lo != m0.row && rhi != m0.row) : (m0.beg == m0.lo && rend == m0.hi);
        float *dst = a.out + static_cast<long long>(m0.row) * a.dim + fcol;
        const int n = min(VEC, a.dim - fcol);
        if (whole) store_row<VEC>(dst, acc, n, a.ovec);
        else add_row<VEC>(dst, acc, n, a.ovec);
      }
    }
    __syncwarp();   // everyone is done with the current slab before the next iteration refills it
    m0 = m1; m1 = m2; base0 = base1; wr0 = wr1; cur ^= 1;
  }
  cp_async_wait<0>();
}

// 0: pick automatically, 1: one launch of non-persistent warps reading global
// memory directly, 2: staged persistent kernel.  Read once from
// EPPGCN_SPMM_KERNEL ("direct" / "staged"); meant for A/B measurements.
int spmm_kernel_choice() {
  static const int choice = [] {
    const char *e = getenv("EPPGCN_SPMM_KERNEL");
    if (!e) return 0;
    if (!strcmp(e, "direct")) return 1;
    if (!strcmp(e, "staged")) return 2;
    return 0;
  }();
  return choice;
}

template <int VEC, int LPR, bool BWD>
int launch_staged(const GroupArgs &a, int part_size, cudaStream_t s) {
  constexpr int G = kWarp / LPR;
  const int ps = part_size >= 1 ? part_size : 32;
  long long want = static_cast<long long>(G) * ps + 4;
  int slab = static_cast<int>(want > 1024 ? 1024 : (want + 3) / 4 * 4);
  const int smem = slab * 2 * 8 * static_cast<int>(sizeof(int));
  static int blocks_per_sm = 0;      // per instantiation; depends only on smem through `slab`, re-queried below
  static int cached_smem = -1;
  static int num_sms = 0;
  if (cached_smem != smem) {
    int dev = 0;
    EPP_CUDA_TRY(cudaGetDevice(&dev));
    EPP_CUDA_TRY(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
    if (smem > 48 * 1024)
      EPP_CUDA_TRY(cudaFuncSetAttribute(staged_spmm_kernel<VEC, LPR, BWD>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    EPP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, staged_spmm_kernel<VEC, LPR, BWD>,
                                                               256, smem));
    if (blocks_per_sm < 1) blocks_per_sm = 1;
    cached_smem = smem;
  }
  const long long nsets = ceil_div_ll(a.num_parts, G);
  long long blocks = ceil_div_ll(nsets, 8);
  const long long cap = static_cast<long long>(num_sms) * blocks_per_sm;
  if (blocks > cap) blocks = cap;
  const int col_aligned = aligned(a.col, 16) ? 1 : 0;
  staged_spmm_kernel<VEC, LPR, BWD><<<static_cast<unsigned>(blocks), 256, smem, s>>>(a, slab, col_aligned);
  EPP_CHECK_LAUNCH("staged_spmm_kernel");
  return EPP_OK;
}

template <int VEC, bool BWD>
int launch_staged_lpr(const GroupArgs &a, int lpr, int part_size, cudaStream_t s) {
  switch (lpr) {
    case 1:  return launch_staged<VEC, 1, BWD>(a, part_size, s);
    case 2:  return launch_staged<VEC, 2, BWD>(a, part_size, s);
    case 4:  return launch_staged<VEC, 4, BWD>(a, part_size, s);
    case 8:  return launch_staged<VEC, 8, BWD>(a, part_size, s);
    case 16: return launch_staged<VEC, 16, BWD>(a, part_size, s);
    default: return launch_staged<VEC, 32, BWD>(a, part_size, s);
  }
}

template <int VEC, bool BWD>
int launch_lpr(const GroupArgs &a, int lpr, cudaStream_t s) {
  const long long groups_per_warp = kWarp / lpr;
  const long long warps = ceil_div_ll(a.num_parts, groups_per_warp);
  const long long blocks = ceil_div_ll(warps, 8);
  if (blocks > 0x7fffffffLL) {
    set_error("too many groups for one launch");
    return EPP_ERR_TOO_LARGE;
  }
  const dim3 grid(static_cast<unsigned>(blocks)), block(256);
  switch (lpr) {
    case 1:  group_spmm_kernel<VEC, 1, BWD><<<grid, block, 0, s>>>(a); break;
    case 2:  group_spmm_kernel<VEC, 2, BWD><<<grid, block, 0, s>>>(a); break;
    case 4:  group_spmm_kernel<VEC, 4, BWD><<<grid, block, 0, s>>>(a); break;
    case 8:  group_spmm_kernel<VEC, 8, BWD><<<grid, block, 0, s>>>(a); break;
    case 16: group_spmm_kernel<VEC, 16, BWD><<<grid, block, 0, s>>>(a); break;
    default: group_spmm_kernel<VEC, 32, BWD><<<grid, block, 0, s>>>(a); break;
  }
  EPP_CHECK_LAUNCH("group_spmm_kernel");
  return EPP_OK;
}

template <bool BWD>
int launch_group_spmm(GroupArgs a, int num_rows, int part_size, cudaStream_t s) {
  // Dense result: rows that no group touches, and rows that are accumulated
  // with atomics, start from zero.
  EPP_CUDA_TRY(cudaMemsetAsync(a.out, 0, sizeof(float) * static_cast<size_t>(num_rows) * a.dim, s));
  if (a.num_parts == 0) return EPP_OK;
  // Widest gather: the lane's VEC floats must be aligned and inside the row stride.
  int vec = 1;
  if (a.ld % 4 == 0 && aligned(a.feat, 16) && a.ld >= ((a.dim + 3) / 4) * 4) vec = 4;
  else if (a.ld % 2 == 0 && aligned(a.feat, 8) && a.ld >= ((a.dim + 1) / 2) * 2) vec = 2;
  a.ovec = 1;
  if (a.dim % 4 == 0 && aligned(a.out, 16)) a.ovec = 4;
  else if (a.dim % 2 == 0 && aligned(a.out, 8)) a.ovec = 2;
  const int lanes_needed = (a.dim + vec - 1) / vec;
  int lpr = 1;
  while (lpr < 32 && lpr < lanes_needed) lpr <<= 1;
  if (spmm_kernel_choice() != 1) {
    switch (vec) {
      case 4:  return launch_staged_lpr<4, BWD>(a, lpr, part_size, s);
      case 2:  return launch_staged_lpr<2, BWD>(a, lpr, part_size, s);
      default: return launch_staged_lpr<1, BWD>(a, lpr, part_size, s);
    }
  }
  switch (vec) {
    case 4:  return launch_lpr<4, BWD>(a, lpr, s);
    case 2:  return launch_lpr<2, BWD>(a, lpr, s);
    default: return launch_lpr<1, BWD>(a, lpr, s);
  }
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_spmm_forward(float *out, const float *feat, long long feat_ld,
                                   const int *row_ptr, const int *col_idx,
                                   const float *deg_row, const float *deg_col,
                                   const int *part_ptr, const int *part2node,
                                   int num_nodes, int dim, int num_parts,
                                   int part_size, int dim_worker, int warp_per_block,
                                   void *stream) {
  (void)dim_worker; (void)warp_per_block;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(feat_ld >= dim, "feat_ld must be >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(out && feat && row_ptr && deg_row && deg_col, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (col_idx && part_ptr && part2node), "null pointer");
  epp::GroupArgs a{};
  a.out = out; a.feat = feat; a.ld = feat_ld;
  a.part_ptr = part_ptr; a.row_of = part2node; a.row_ptr = row_ptr; a.col = col_idx;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim;
  return epp::launch_group_spmm<false>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream));
}

EPP_EXPORT int eppgcn_spmm_backward_compacted(float *d_in, const float *d_out, long long d_out_ld,
                                              const int *ids, const int *part_ptr, const int *edge_list,
                                              const float *deg_row, const float *deg_col,
                                              int num_nodes, int dim, int num_parts,
                                              int part_size, int blockx, int blocky,
                                              void *stream) {
  (void)blockx; (void)blocky;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(d_out_ld >= dim, "d_out_ld must be >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(d_in && d_out && deg_row && deg_col, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (ids && part_ptr && edge_list), "null pointer");
  epp::GroupArgs a{};
  a.out = d_in; a.feat = d_out; a.ld = d_out_ld;
  a.part_ptr = part_ptr; a.row_of = ids; a.row_ptr = nullptr; a.col = edge_list;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim;
  return epp::launch_group_spmm<true>(a, num_nodes, part_size, static_cast<cudaStream_t>(stream));
}
