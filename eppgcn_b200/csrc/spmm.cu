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
#include "common.cuh"

namespace epp {
namespace {

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

inline bool aligned(const void *p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

template <bool BWD>
int launch_group_spmm(GroupArgs a, int num_rows, cudaStream_t s) {
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
  (void)part_size; (void)dim_worker; (void)warp_per_block;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(feat_ld >= dim, "feat_ld must be >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(out && feat && row_ptr && deg_row && deg_col, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (col_idx && part_ptr && part2node), "null pointer");
  epp::GroupArgs a{};
  a.out = out; a.feat = feat; a.ld = feat_ld;
  a.part_ptr = part_ptr; a.row_of = part2node; a.row_ptr = row_ptr; a.col = col_idx;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim;
  return epp::launch_group_spmm<false>(a, num_nodes, static_cast<cudaStream_t>(stream));
}

EPP_EXPORT int eppgcn_spmm_backward_compacted(float *d_in, const float *d_out, long long d_out_ld,
                                              const int *ids, const int *part_ptr, const int *edge_list,
                                              const float *deg_row, const float *deg_col,
                                              int num_nodes, int dim, int num_parts,
                                              int part_size, int blockx, int blocky,
                                              void *stream) {
  (void)part_size; (void)blockx; (void)blocky;
  EPP_REQUIRE(num_nodes >= 0 && dim >= 1 && num_parts >= 0, "negative size or dim < 1");
  EPP_REQUIRE(d_out_ld >= dim, "d_out_ld must be >= dim");
  if (num_nodes == 0) return EPP_OK;
  EPP_REQUIRE(d_in && d_out && deg_row && deg_col, "null pointer");
  EPP_REQUIRE(num_parts == 0 || (ids && part_ptr && edge_list), "null pointer");
  epp::GroupArgs a{};
  a.out = d_in; a.feat = d_out; a.ld = d_out_ld;
  a.part_ptr = part_ptr; a.row_of = ids; a.row_ptr = nullptr; a.col = edge_list;
  a.deg_row = deg_row; a.deg_col = deg_col; a.num_parts = num_parts; a.dim = dim;
  return epp::launch_group_spmm<true>(a, num_nodes, static_cast<cudaStream_t>(stream));
}
