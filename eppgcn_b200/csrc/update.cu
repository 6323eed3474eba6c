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
// A thread accumulates a 4x4 tile: four rows times four output columns.
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
  const int ty = threadIdx.x / TX;        // row quad: rows ty*4 .. ty*4+3 of the block
  const long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock;
  const int chunks = (k + kChunk - 1) / kChunk;

  auto stage = [&](int chunk, int buf) {
    const int k0 = chunk * kChunk;
    // X: 128 rows x 8 pieces of 16 bytes
    for (int i = threadIdx.x; i < kRowsPerBlock * (kChunk / 4); i += THREADS) {
      const int r = i / (kChunk / 4), piece = i % (kChunk / 4);
      const long long row = row0 + r;
      const int kk = k0 + piece * 4;
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

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

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
#pragma unroll
    for (int kk = 0; kk < kChunk; kk += 4) {
      float4 xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = *reinterpret_cast<const float4 *>(&xs[buf][ty * 4 + i][kk]);
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const float4 *>(&ws[buf][kk + j][tx * 4]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float xk[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][0] = fmaf(xk[j], wv[j].x, acc[i][0]);
          acc[i][1] = fmaf(xk[j], wv[j].y, acc[i][1]);
          acc[i][2] = fmaf(xk[j], wv[j].z, acc[i][2]);
          acc[i][3] = fmaf(xk[j], wv[j].w, acc[i][3]);
        }
      }
    }
    __syncthreads();   // the buffer is refilled by the next iteration's stage()
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long row = row0 + ty * 4 + i;
    if (row < n) {
      const float s = scale ? __ldg(scale + row) : 1.f;
      float *dst = out + row * ld_out + tx * 4;
      const float v[4] = {acc[i][0] * s, acc[i][1] * s, acc[i][2] * s, acc[i][3] * s};
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
// reduction with a tiny result: bound by reading x once.  A block walks over a
// contiguous slab of rows, one stage of rows at a time through shared memory (cp.async,
// two buffers); inside a block "row groups" of (K/4)*(D/4) threads share the
// staged rows, every thread accumulating a 4x4 tile of dw for its rows; the
// tiles are added into dw with atomics at the end (dw is cleared first).  A
// stage holds as many rows as fit about 36 KB.
// ---------------------------------------------------------------------------
namespace epp {
namespace {

// rows per stage: sized by the launcher so that a stage moves about 36 KB whatever the row width

template <int DP>
__global__ void __launch_bounds__(256) weight_grad_kernel(float *__restrict__ dw, const float *__restrict__ x,
                                                          long long ldx, const float *__restrict__ d, long long ldd,
                                                          const int *__restrict__ row_list,
                                                          int n, int k, int dout, int rows_per_block,
                                                          int kWgRows) {
  extern __shared__ __align__(16) float wg_smem[];
  constexpr int TX = DP / 4;
  const int kp = (k + 3) / 4 * 4;               // staged row length of x
  const int tk = kp / 4;
  const int group_threads = tk * TX;
  const int groups = blockDim.x / group_threads;
  float *xs = wg_smem;                          // [2][kWgRows][kp]
  float *ds = wg_smem + 2 * kWgRows * kp;       // [2][kWgRows][DP]
  const int grp = threadIdx.x / group_threads;
  const int t = threadIdx.x % group_threads;
  const int ky = t / TX, tx = t % TX;           // this thread's 4 k-values and 4 columns
  const bool worker = grp < groups;
  const long long row_beg = static_cast<long long>(blockIdx.x) * rows_per_block;
  long long row_end = row_beg + rows_per_block;
  if (row_end > n) row_end = n;
  if (row_beg >= row_end) return;
  const int stages = static_cast<int>((row_end - row_beg + kWgRows - 1) / kWgRows);
  const int align_x = ldx % 4 == 0 ? 4 : (ldx % 2 == 0 ? 2 : 1);
  const int align_d = ldd % 4 == 0 ? 4 : (ldd % 2 == 0 ? 2 : 1);

  auto stage = [&](int s, int buf) {
    const long long r0 = row_beg + static_cast<long long>(s) * kWgRows;
    float *xb = xs + buf * kWgRows * kp;
    float *db = ds + buf * kWgRows * DP;
    {   // (r, piece) walk i = threadIdx.x, threadIdx.x + blockDim.x, ... without a division per element
      const int dr = blockDim.x / tk, dp = blockDim.x % tk;
      int r = threadIdx.x / tk, piece = threadIdx.x % tk;
      while (r < kWgRows) {
        const long long at = r0 + r;                 // position in the walk; the row itself may come from the list
        const long long row = (row_list && at < row_end) ? __ldg(row_list + at) : at;
        stage4(xb + r * kp + piece * 4, x + row * ldx + piece * 4, at < row_end ? min(4, k - piece * 4) : 0, align_x);
        r += dr;
        piece += dp;
        if (piece >= tk) { piece -= tk; ++r; }
      }
    }
    for (int i = threadIdx.x; i < kWgRows * TX; i += blockDim.x) {
      const int r = i / TX, piece = i % TX;
      const long long at = r0 + r;
      const long long row = (row_list && at < row_end) ? __ldg(row_list + at) : at;
      float *dst = db + r * DP + piece * 4;
      stage4(dst, d + row * ldd + piece * 4, at < row_end ? min(4, dout - piece * 4) : 0, align_d);
    }
    cp_commit();
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  stage(0, 0);
  for (int s = 0; s < stages; ++s) {
    const int buf = s & 1;
    if (s + 1 < stages) {
      stage(s + 1, buf ^ 1);
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    if (worker) {
      const float *xb = xs + buf * kWgRows * kp + ky * 4;
      const float *db = ds + buf * kWgRows * DP + tx * 4;
#pragma unroll 4
      for (int r = grp; r < kWgRows; r += groups) {
        const float4 xv = *reinterpret_cast<const float4 *>(xb + r * kp);
        const float4 dv = *reinterpret_cast<const float4 *>(db + r * DP);
        const float xk[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[i][0] = fmaf(xk[i], dv.x, acc[i][0]);
          acc[i][1] = fmaf(xk[i], dv.y, acc[i][1]);
          acc[i][2] = fmaf(xk[i], dv.z, acc[i][2]);
          acc[i][3] = fmaf(xk[i], dv.w, acc[i][3]);
        }
      }
    }
    __syncthreads();
  }
  if (worker) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kk = ky * 4 + i, c = tx * 4 + j;
        if (kk < k && c < dout && acc[i][j] != 0.f) atomicAdd(dw + static_cast<long long>(kk) * dout + c, acc[i][j]);
      }
  }
}

template <int DP>
int launch_weight_grad(float *dw, const float *x, long long ldx, const float *d, long long ldd, const int *row_list,
                       int n, int k, int dout, cudaStream_t s) {
  const int kp = (k + 3) / 4 * 4;
  int kWgRows = 36 * 1024 / ((kp + DP) * static_cast<int>(sizeof(float)));
  kWgRows = kWgRows < 32 ? 32 : (kWgRows > 512 ? 512 : kWgRows / 32 * 32);
  const int smem = 2 * kWgRows * (kp + DP) * static_cast<int>(sizeof(float));
  static SmemOptIn memo;                         // per instantiation; remembers the opt-in per device
  if (const int rc = smem_opt_in(memo, reinterpret_cast<const void *>(weight_grad_kernel<DP>), smem); rc != EPP_OK)
    return rc;
  int sms = 148;
  if (const int rc = device_sm_count(&sms); rc != EPP_OK) return rc;
  long long blocks = static_cast<long long>(sms) * 4;
  long long rows_per_block = ceil_div_ll(ceil_div_ll(n, blocks), kWgRows) * kWgRows;
  if (rows_per_block < kWgRows) rows_per_block = kWgRows;
  blocks = ceil_div_ll(n, rows_per_block);
  weight_grad_kernel<DP><<<static_cast<unsigned>(blocks), 256, smem, s>>>(dw, x, ldx, d, ldd, row_list, n, k, dout,
                                                                          static_cast<int>(rows_per_block), kWgRows);
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
  switch (dp) {
    case 4:  return launch_weight_grad<4>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 8:  return launch_weight_grad<8>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 12: return launch_weight_grad<12>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 16: return launch_weight_grad<16>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 20: return launch_weight_grad<20>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 24: return launch_weight_grad<24>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    case 28: return launch_weight_grad<28>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
    default: return launch_weight_grad<32>(dw, x, ldx, d, ldd, row_list, num_rows, k, dout, s);
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
