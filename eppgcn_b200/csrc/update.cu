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
#include "common.cuh"

namespace epp {
namespace {

constexpr int kRowsPerBlock = 128;
constexpr int kChunk = 32;            // columns of X per stage
constexpr int kXStride = kChunk + 4;  // floats; keeps rows 16-byte aligned and spreads banks

__device__ __forceinline__ void cp16(void *smem_dst, const void *gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// DP: output width rounded up to a multiple of 4 (<= 32); blockDim.x = (DP/4) * 32.
template <int DP>
__global__ void __launch_bounds__((DP / 4) * 32) update_scaled_kernel(
    float *__restrict__ out, long long ld_out, const float *__restrict__ x, long long ldx,
    const float *__restrict__ w, const float *__restrict__ scale, int n, int k, int dout) {
  constexpr int TX = DP / 4;
  constexpr int THREADS = TX * 32;
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
      if (row < n && kk + 4 <= k) {
        cp16(dst, x + row * ldx + kk);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = (row < n && kk + j < k) ? x[row * ldx + kk + j] : 0.f;
      }
    }
    // W: 32 rows x DP columns, zero beyond dout / k
    for (int i = threadIdx.x; i < kChunk * DP; i += THREADS) {
      const int kk = i / DP, c = i % DP;
      ws[buf][kk][c] = (k0 + kk < k && c < dout) ? __ldg(w + static_cast<long long>(k0 + kk) * dout + c) : 0.f;
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
      if (tx * 4 + 4 <= ld_out) {
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (tx * 4 + j < dout) dst[j] = v[j];
      }
      if (tx == TX - 1)      // padding columns beyond the last quad
        for (long long c = DP; c < ld_out; ++c) out[row * ld_out + c] = 0.f;
    }
  }
}

template <int DP>
int launch_update(float *out, long long ld_out, const float *x, long long ldx, const float *w, const float *scale,
                  int n, int k, int dout, cudaStream_t s) {
  const long long blocks = ceil_div_ll(n, kRowsPerBlock);
  update_scaled_kernel<DP><<<static_cast<unsigned>(blocks), (DP / 4) * 32, 0, s>>>(out, ld_out, x, ldx, w, scale, n,
                                                                                     k, dout);
  EPP_CHECK_LAUNCH("update_scaled_kernel");
  return EPP_OK;
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_update_scaled(float *out, long long ld_out, const float *x, long long ldx, const float *w,
                                    const float *scale, int num_rows, int k, int dout, void *stream) {
  using namespace epp;
  EPP_REQUIRE(num_rows >= 0 && k >= 1 && dout >= 1, "negative size, k < 1 or dout < 1");
  if (dout > 32) {
    set_error("eppgcn_update_scaled handles at most 32 output columns, got %d", dout);
    return EPP_ERR_TOO_LARGE;
  }
  if (num_rows == 0) return EPP_OK;
  EPP_REQUIRE(out && x && w, "null pointer");
  EPP_REQUIRE(ldx >= k && ld_out >= dout, "row stride smaller than the row");
  EPP_REQUIRE(ldx % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0, "X rows must be 16-byte aligned");
  EPP_REQUIRE(ld_out % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0, "out rows must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int dp = (dout + 3) / 4 * 4;
  switch (dp) {
    case 4:  return launch_update<4>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 8:  return launch_update<8>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 12: return launch_update<12>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 16: return launch_update<16>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 20: return launch_update<20>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 24: return launch_update<24>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    case 28: return launch_update<28>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
    default: return launch_update<32>(out, ld_out, x, ldx, w, scale, num_rows, k, dout, s);
  }
}
