// Small dense update of the GCN layer, fused with the source-side scaling:
//
//   out[r][c] = scale[r] * sum_k X[r][k] * W[k][c]          c < dout <= 32
//
// The reference runs this as a cuBLAS SGEMM (torch::mm, EPPGCN_kernel.cu:142)
// and gathers deg[col] per edge inside the aggregation kernel.  With the factor
// folded into the rows here, the aggregation fetches one 32-byte sector less per
// edge.  The product is tall and skinny (millions of rows, 16..24 columns): it
// is bound by reading X once, so plain FP32 FMA on the CUDA cores is enough and
// keeps full fp32 accuracy.
//
// A block owns 128 rows.  X is streamed through shared memory in chunks of 32
// columns with cp.async (two buffers); the matching 32 rows of W ride along.
// A thread accumulates a 4x4 tile: four rows (32 apart) times four output columns, as packed pairs of columns.
#include "rowio.cuh"

namespace epp {
namespace {

constexpr int kRowsPerBlock = 128;
constexpr int kChunk = 32;            // columns of X per stage
constexpr int kXStride = kChunk + 4;  // floats; keeps rows 16-byte aligned and spreads banks

__device__ __forceinline__ void cp16(void *smem_dst, const void *gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp8(void *smem_dst, const void *gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}
// Four consecutive floats of a row into shared memory: one 16-byte or two 8-byte asynchronous copies
// when the row stride allows (align: 4, 2 or 1 floats), plain loads otherwise; `valid` floats exist.
__device__ __forceinline__ void stage4(float *dst, const float *src, int valid, int align) {
  if (valid >= 4 && align == 4) {
    cp16(dst, src);
  } else if (align >= 2) {
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      if (j + 2 <= valid) cp8(dst + j, src + j);
      else { dst[j] = j < valid ? src[j] : 0.f; dst[j + 1] = 0.f; }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = j < valid ? src[j] : 0.f;
  }
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Two fp32 fused multiply-adds per instruction (fma.rn.f32x2 of sm_100): a register pair holds two floats and
// each half rounds exactly like fmaf.  Both kernels below are bound by issue slots, and this halves their FMA count.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma2(f32x2 &acc, f32x2 a, f32x2 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// DP: output width rounded up to a multiple of 4 (<= 32); blockDim.x = (DP/4) * 32.
template <int DP>
__global__ void __launch_bounds__((DP / 4) * 32) update_scaled_kernel(
    float *__restrict__ out, long long ld_out, const float *__restrict__ x, long long ldx,
    const float *__restrict__ w, long long ldw, const float *__restrict__ scale, int n, int k, int dout,
    int owned_cols) {
  constexpr int TX = DP / 4;
  constexpr int THREADS = TX * 32;
  const int align_x = ldx % 4 == 0 ? 4 : (ldx % 2 == 0 ? 2 : 1);   // floats every row start is aligned to
  __shared__ __align__(16) float xs[2][kRowsPerBlock][kXStride];
  __shared__ __align__(16) float ws[2][kChunk][DP];
  const int tx = threadIdx.x % TX;        // column quad
  const int ty = threadIdx.x / TX;        // 0..31: rows ty, ty+32, ty+64, ty+96 of the block (a warp's shared loads of
                                          // consecutive rows fall into distinct banks, and its stores are contiguous)
  const long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock;
  const int chunks = (k + kChunk - 1) / kChunk;

  auto stage = [&](int chunk, int buf) {
    const int k0 = chunk * kChunk;
    // X: 128 rows x 8 pieces of 16 bytes
    for (int i = threadIdx.x; i < kRowsPerBlock * (kChunk / 4); i += THREADS) {
      const int r = i / (kChunk / 4), piece = i % (kChunk / 4);
      const long long row = row0 + r;
      const int kk = k0 + piece * 4;
      if (kk >= k) continue;                 // beyond a short last chunk: never read
      float *dst = &xs[buf][r][piece * 4];
      stage4(dst, x + row * ldx + kk, row < n ? min(4, k - kk) : 0, align_x);
    }
    // W: 32 rows x DP columns, zero beyond dout / k
    for (int i = threadIdx.x; i < kChunk * DP; i += THREADS) {
      const int kk = i / DP, c = i % DP;
      ws[buf][kk][c] = (k0 + kk < k && c < dout) ? __ldg(w + static_cast<long long>(k0 + kk) * ldw + c) : 0.f;
    }
    cp_commit();
  };

  f32x2 acc[4][2];          // 4 rows x 4 columns, two columns per register pair
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = pack2(0.f, 0.f);

  stage(0, 0);
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < chunks) {
      stage(c + 1, buf ^ 1);
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const int klim = min(kChunk, k - c * kChunk);     // a short last chunk skips its zero padding
#pragma unroll
    for (int kk = 0; kk < kChunk; kk += 4) {
      if (kk >= klim) break;
      float4 xv[4];
      ulonglong2 wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = *reinterpret_cast<const float4 *>(&xs[buf][ty + 32 * i][kk]);
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const ulonglong2 *>(&ws[buf][kk + j][tx * 4]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float xk[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 xx = pack2(xk[j], xk[j]);
          fma2(acc[i][0], xx, wv[j].x);
          fma2(acc[i][1], xx, wv[j].y);
        }
      }
    }
    __syncthreads();   // the buffer is refilled by the next iteration's stage()
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long row = row0 + ty + 32 * i;
    if (row < n) {
      const float s = scale ? __ldg(scale + row) : 1.f;
      float *dst = out + row * ld_out + tx * 4;
      float v[4];
      unpack2(acc[i][0], v[0], v[1]);
      unpack2(acc[i][1], v[2], v[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] *= s;
      if (tx * 4 + 4 <= owned_cols) {      // columns dout..owned_cols-1 receive the zeros of the padded W
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (tx * 4 + j < dout) dst[j] = v[j];
      }
      if (tx == TX - 1)      // owned padding columns beyond the last quad
        for (int c = DP; c < owned_cols; ++c) out[row * ld_out + c] = 0.f;
    }
  }
}

template <int DP>
int launch_update(float *out, long long ld_out, const float *x, long long ldx, const float *w, long long ldw,
                  const float *scale, int n, int k, int dout, int owned_cols, cudaStream_t s) {
  const long long blocks = ceil_div_ll(n, kRowsPerBlock);
  update_scaled_kernel<DP><<<static_cast<unsigned>(blocks), (DP / 4) * 32, 0, s>>>(out, ld_out, x, ldx, w, ldw, scale,
                                                                                     n, k, dout, owned_cols);
  EPP_CHECK_LAUNCH("update_scaled_kernel");
  return EPP_OK;
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_update_scaled(float *out, long long ld_out, const float *x, long long ldx, const float *w,
                                    long long ldw, const float *scale, int num_rows, int k, int dout, int pad_cols,
                                    void *stream) {
  using namespace epp;
  EPP_REQUIRE(num_rows >= 0 && k >= 1 && dout >= 1, "negative size, k < 1 or dout < 1");
  if (dout > 32) {
    set_error("eppgcn_update_scaled handles at most 32 output columns, got %d", dout);
    return EPP_ERR_TOO_LARGE;
  }
  if (num_rows == 0) return EPP_OK;
  EPP_REQUIRE(out && x && w, "null pointer");
  EPP_REQUIRE(pad_cols >= 0 && ldx >= k && ld_out >= dout + pad_cols && ldw >= dout, "row stride smaller than the row");
  const int owned = dout + pad_cols;
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0, "x must be 16-byte aligned");
  EPP_REQUIRE(ld_out % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0, "out rows must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int dp = (dout + 3) / 4 * 4;
  switch (dp) {
    case 4:  return launch_update<4>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 8:  return launch_update<8>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 12: return launch_update<12>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 16: return launch_update<16>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 20: return launch_update<20>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 24: return launch_update<24>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    case 28: return launch_update<28>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
    default: return launch_update<32>(out, ld_out, x, ldx, w, ldw, scale, num_rows, k, dout, owned, s);
  }
}

// ---------------------------------------------------------------------------
// Weight gradient of a layer:  dw[k][c] = sum_r x[r][k] * d[r][c]
// (the X^T * d' product of the backward wrapper, EPPGCN_kernel.cu:615).  A tall
// reduction with a tiny result: bound by reading the listed rows of x once.
//
// A lane owns four k-values and CT columns of dw (4 x CT accumulators, held as
// packed pairs) and adds one outer product per row; min(k/4, 32) lanes cover a
// row, so one pass of a warp's lanes takes 1..8 rows and a batch is four passes.
// Wider products are cut into units of 128 k-values x CT columns, the eight
// warps of a block being dealt over the units.  Every warp streams its batches
// (dealt round-robin over the grid) through a private ring of shared memory with cp.async (kWgDepth
// batches in flight, no block-wide barrier in the loop); row ids are fetched 32
// at a time, one set ahead.  At the end the warps of a unit add their tiles into
// shared memory one after the other (plain read-modify-write: shared-memory
// float atomics took a third of the kernel), and a block adds one value per
// element of dw with global atomics (dw is cleared first).
// ---------------------------------------------------------------------------
namespace epp {
namespace {

constexpr int kWgWarps = 8;
constexpr int kWgDepth = 3;      // batches of a warp in flight
constexpr int kWgPasses = 4;     // rows a lane takes per batch (2 passes x 4 in flight: 7 % slower for k = 128)
constexpr int kWgMaxRows = 8;    // rows of one pass at most

struct WgShape {
  int tk, q, rows, batch_rows, rowf, slot, cc, units, wpu;
};
// CT columns per lane; tk = k quads; q lanes per row; a ring slot holds `batch_rows` rows of 4q + CT floats.
__host__ __device__ inline WgShape wg_shape(int k, int dout, int ct) {
  WgShape s;
  s.tk = (k + 3) / 4;
  s.q = s.tk < 32 ? s.tk : 32;
  s.rows = 32 / s.q < kWgMaxRows ? 32 / s.q : kWgMaxRows;
  s.batch_rows = s.rows * kWgPasses;
  s.rowf = 4 * s.q + ct;
  s.slot = s.batch_rows * s.rowf;
  s.cc = ((dout + 3) / 4 * 4 + ct - 1) / ct;
  s.units = s.cc * ((s.tk + 31) / 32);
  s.wpu = kWgWarps / s.units;
  return s;
}

template <int CT>
__global__ void __launch_bounds__(kWgWarps * 32, 2) weight_grad_kernel(
    float *__restrict__ dw, const float *__restrict__ x, long long ldx, const float *__restrict__ d, long long ldd,
    const int *__restrict__ row_list, int n, int k, int dout) {
  extern __shared__ __align__(16) float wg_smem[];
  constexpr unsigned kFull = 0xffffffffu;
  const WgShape sh = wg_shape(k, dout, CT);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int unit = warp / sh.wpu, wj = warp % sh.wpu;       // this warp's unit and its place among the unit's warps
  const bool warp_on = unit < sh.units;
  const int slab = warp_on ? unit / sh.cc : 0, chunk = warp_on ? unit % sh.cc : 0;
  const int r = lane / sh.q, kq = lane % sh.q;               // this lane's row of a pass and k quad of the slab
  const bool lane_on = r < sh.rows;
  const int kquad = slab * 32 + kq;
  const int x_valid = lane_on ? max(0, min(4, k - kquad * 4)) : 0;
  const int pr = lane / (CT / 4), pc = lane % (CT / 4);      // the piece of d this lane stages: row, column quad
  const bool piece_on = pr < sh.rows;
  const int d_col = chunk * CT + pc * 4;
  const int d_valid = piece_on ? max(0, min(4, dout - d_col)) : 0;
  const int align_x = ldx % 4 == 0 ? 4 : (ldx % 2 == 0 ? 2 : 1);
  const int align_d = ldd % 4 == 0 ? 4 : (ldd % 2 == 0 ? 2 : 1);
  float *ring = wg_smem + static_cast<size_t>(warp) * kWgDepth * sh.slot;
  const int x_at = (lane_on ? r : 0) * sh.rowf + kq * 4;                 // float offsets inside a pass of a slot
  const int d_at = (piece_on ? pr : 0) * sh.rowf + 4 * sh.q + pc * 4;
  const int pass_floats = sh.rows * sh.rowf;

  // Batches are dealt round-robin over all warps of the unit in the grid, so that at any time the grid reads one
  // contiguous window of the (listed) rows: DRAM pages are used whole while they are open.
  const long long all_batches = (static_cast<long long>(n) + sh.batch_rows - 1) / sh.batch_rows;
  const long long gw = static_cast<long long>(blockIdx.x) * sh.wpu + wj, grid_warps = static_cast<long long>(gridDim.x) * sh.wpu;
  const int batches = warp_on && all_batches > gw ? static_cast<int>((all_batches - gw + grid_warps - 1) / grid_warps) : 0;

  // Row ids are fetched a whole set of batches at a time (lane l holds the id of the set's l-th row) and
  // one set ahead of their use, so that no batch waits for the load of its own ids.
  const int set_batches = 32 / sh.batch_rows, set_rows = set_batches * sh.batch_rows;
  auto load_ids = [&](int set) {
    const long long batch = gw + (static_cast<long long>(set) * set_batches + lane / sh.batch_rows) * grid_warps;
    const long long at = batch * sh.batch_rows + lane % sh.batch_rows;
    int rid = -1;
    if (lane < set_rows && at < n) rid = row_list ? __ldg(row_list + at) : static_cast<int>(at);
    return rid;
  };
  int ids_now = load_ids(0), ids_next = load_ids(1);
  int staged_set = 0, staged_in_set = 0;            // where the next batch to stage sits

  auto stage = [&](int b) {                         // called for b = 0, 1, 2, ... in turn
    float *slot = ring + (b % kWgDepth) * sh.slot;
    const int first = staged_in_set * sh.batch_rows;
#pragma unroll
    for (int u = 0; u < kWgPasses; ++u) {
      const int xr = __shfl_sync(kFull, ids_now, first + u * sh.rows + (lane_on ? r : 0));
      const int dr = __shfl_sync(kFull, ids_now, first + u * sh.rows + (piece_on ? pr : 0));
      if (lane_on)
        stage4(slot + u * pass_floats + x_at, x + static_cast<long long>(xr < 0 ? 0 : xr) * ldx + kquad * 4,
               xr < 0 ? 0 : x_valid, align_x);
      if (piece_on)
        stage4(slot + u * pass_floats + d_at, d + static_cast<long long>(dr < 0 ? 0 : dr) * ldd + d_col,
               dr < 0 ? 0 : d_valid, align_d);
    }
    if (++staged_in_set == set_batches) {
      staged_in_set = 0;
      ids_now = ids_next;
      ids_next = load_ids(++staged_set + 1);
    }
  };

  f32x2 acc[4][CT / 2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < CT / 2; ++j) acc[i][j] = pack2(0.f, 0.f);

  for (int b = 0; b < kWgDepth - 1; ++b) {
    if (b < batches) stage(b);
    cp_commit();
  }
  for (int b = 0; b < batches; ++b) {
    if (b + kWgDepth - 1 < batches) stage(b + kWgDepth - 1);
    cp_commit();
    cp_wait<kWgDepth - 1>();
    __syncwarp();
    if (lane_on) {
      const float *slot = ring + (b % kWgDepth) * sh.slot;
#pragma unroll
      for (int u = 0; u < kWgPasses; ++u) {
        const float4 xv = *reinterpret_cast<const float4 *>(slot + u * pass_floats + x_at);
        const f32x2 xk[4] = {pack2(xv.x, xv.x), pack2(xv.y, xv.y), pack2(xv.z, xv.z), pack2(xv.w, xv.w)};
        const float *dp = slot + u * pass_floats + r * sh.rowf + 4 * sh.q;
#pragma unroll
        for (int j = 0; j < CT / 4; ++j) {
          const ulonglong2 dv = *reinterpret_cast<const ulonglong2 *>(dp + 4 * j);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            fma2(acc[i][2 * j], xk[i], dv.x);
            fma2(acc[i][2 * j + 1], xk[i], dv.y);
          }
        }
      }
    }
    __syncwarp();          // the slot is staged again by the next iteration
  }
  cp_wait<0>();
  __syncthreads();         // every ring is drained: the block's tiles of dw take its place

  // tile[r][kp][dp]: one plane per row of a pass; the warps of a unit take turns, so no two lanes meet
  const int kp = sh.tk * 4, dp = (dout + 3) / 4 * 4, plane = kp * dp;
  float *tile = wg_smem;
  for (int w = 0; w < sh.wpu; ++w) {
    if (warp_on && wj == w && lane_on) {
      float *t = tile + r * plane + kquad * 4 * dp + chunk * CT;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < CT / 4; ++j) {
          if (kquad * 4 + i < kp && chunk * CT + 4 * j < dp) {
            float4 v;
            unpack2(acc[i][2 * j], v.x, v.y);
            unpack2(acc[i][2 * j + 1], v.z, v.w);
            float4 *at = reinterpret_cast<float4 *>(t + i * dp + 4 * j);
            if (w > 0) {
              const float4 o = *at;
              v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            *at = v;
          }
        }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < plane; i += blockDim.x) {
    const int kk = i / dp, c = i % dp;
    float v = 0.f;
    for (int p = 0; p < sh.rows; ++p) v += tile[p * plane + i];
    if (kk < k && c < dout && v != 0.f) atomicAdd(dw + static_cast<long long>(kk) * dout + c, v);
  }
}

template <int CT>
int launch_weight_grad(float *dw, const float *x, long long ldx, const float *d, long long ldd, const int *row_list,
                       int n, int k, int dout, cudaStream_t s) {
  const WgShape sh = wg_shape(k, dout, CT);
  const int kp = sh.tk * 4, dp = (dout + 3) / 4 * 4;
  const int ring_floats = kWgWarps * kWgDepth * sh.slot, tile_floats = sh.rows * kp * dp;
  const int smem = static_cast<int>(sizeof(float)) * (ring_floats > tile_floats ? ring_floats : tile_floats);
  static SmemOptIn memo;                         // per instantiation; remembers the opt-in per device
  if (const int rc = smem_opt_in(memo, reinterpret_cast<const void *>(weight_grad_kernel<CT>), smem); rc != EPP_OK)
    return rc;
  int sms = 148;
  if (const int rc = device_sm_count(&sms); rc != EPP_OK) return rc;
  // two resident blocks per SM
  const long long all_batches = ceil_div_ll(n, sh.batch_rows);
  long long blocks = ceil_div_ll(all_batches, sh.wpu);
  if (blocks > static_cast<long long>(sms) * 2) blocks = static_cast<long long>(sms) * 2;
  weight_grad_kernel<CT><<<static_cast<unsigned>(blocks), kWgWarps * 32, smem, s>>>(dw, x, ldx, d, ldd, row_list, n, k,
                                                                                   dout);
  EPP_CHECK_LAUNCH("weight_grad_kernel");
  return EPP_OK;
}

}  // namespace
}  // namespace epp

static int weight_grad_impl(float *dw, const float *x, long long ldx, const float *d, long long ldd,
                            const int *row_list, int num_rows, int k, int dout, void *stream) {
  using namespace epp;
  EPP_REQUIRE(num_rows >= 0 && k >= 1 && dout >= 1, "negative size, k < 1 or dout < 1");
  const int dp = (dout + 3) / 4 * 4;
  const int kp = (k + 3) / 4 * 4;
  if (dout > 32 || (kp / 4) * (dp / 4) > 256) {
    set_error("eppgcn_weight_grad handles dout <= 32 and k * dout <= 4096, got k = %d, dout = %d", k, dout);
    return EPP_ERR_TOO_LARGE;
  }
  EPP_REQUIRE(dw, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EPP_CUDA_TRY(cudaMemsetAsync(dw, 0, sizeof(float) * static_cast<size_t>(k) * dout, s));
  if (num_rows == 0) return EPP_OK;
  EPP_REQUIRE(x && d && ldx >= k && ldd >= dout, "null pointer or row stride smaller than the row");
  EPP_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(d) % 16 == 0,
              "x and d must be 16-byte aligned");
  // columns per lane: the whole padded width up to 16, half of it (rounded up to a quad) beyond
  const int ct = dp <= 16 ? dp : (dp / 2 + 3) / 4 * 4;
  switch (ct) {
    case 4:  return launch_weight_grad<4>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 8:  return launch_weight_grad<8>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 12: return launch_weight_grad<12>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    default: return launch_weight_grad<16>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
  }
}

EPP_EXPORT int eppgcn_weight_grad(float *dw, const float *x, long long ldx, const float *d, long long ldd,
                                  int num_rows, int k, int dout, void *stream) {
  return weight_grad_impl(dw, x, ldx, d, ldd, nullptr, num_rows, k, dout, stream);
}

EPP_EXPORT int eppgcn_weight_grad_rows(float *dw, const float *x, long long ldx, const float *d, long long ldd,
                                       const int *rows, int num_listed, int k, int dout, void *stream) {
  if (num_listed > 0 && !rows) {
    epp::set_error("eppgcn_weight_grad_rows: null row list");
    return EPP_ERR_BAD_ARG;
  }
  return weight_grad_impl(dw, x, ldx, d, ldd, num_listed > 0 ? rows : nullptr, num_listed, k, dout, stream);
}
