// Measurement aid of bench.py, built into its own small library
// (libeppgcn_probe.so) and not part of the product's C-ABI: the bare gather of
// an aggregation.  For every entry of col_idx the fp32 row feat[col_idx[e]][0..dim)
// is loaded with 16-byte loads and discarded -- no weights, no result.  Its
// duration is the floor for any kernel that has to perform these gathers, in
// this order, on the device at hand.
#include "../rowio.cuh"

namespace epp {
void set_error(const char *, ...) {}   // this library reports through return codes only
namespace {

// Diagnostic: the bare gather of the aggregation -- every edge's source row is
// fetched (4 lanes per row, 16-byte loads, eight rows in flight per lane) and
// summed into a value nobody reads.  No weights, no output rows, column ids read
// straight from global memory.  Its time is the floor for any kernel that has
// to perform these gathers on this GPU.
template <int T>
__global__ void __launch_bounds__(256) gather_probe_kernel(const int *__restrict__ col, long long num_edges,
                                                           const float *__restrict__ feat, unsigned ld_bytes,
                                                           int dim, float *sink) {
  constexpr int CH = 64;                       // edges per 4-lane group
  const long long q = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 2;
  const int sl = threadIdx.x & 3;
  const long long beg = q * CH;
  const long long end = beg + CH < num_edges ? beg + CH : num_edges;
  constexpr int U = T >= 8 ? 1 : 8 / T;
  float acc = 0.f;
  const char *fb = reinterpret_cast<const char *>(feat + sl * 4);
  for (long long e = beg; e + U <= end; e += U) {
    int c[U];
    float4 v[U][T];
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = __ldg(col + e + u);
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < T; ++k)
        v[u][k] = (sl * 4 + k * 16 < dim)
                      ? __ldg(reinterpret_cast<const float4 *>(fb + static_cast<unsigned long long>(
                                  static_cast<unsigned>(c[u])) * ld_bytes + k * 64))
                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < T; ++k) acc += v[u][k].x + v[u][k].y + v[u][k].z + v[u][k].w;
  }
  if (acc == 1.2345e-30f) *sink = acc;         // keeps the loads alive
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_probe_gather(const int *col_idx, long long num_edges, const float *feat, long long feat_ld,
                                   int dim, float *sink, void *stream) {
  using namespace epp;
  EPP_REQUIRE(num_edges >= 0 && dim >= 1 && dim <= 128, "sizes out of range (dim 1..128)");
  EPP_REQUIRE(feat_ld % 4 == 0 && feat_ld >= (dim + 3) / 4 * 4 && feat_ld <= 0x3fffffffLL, "rows must be padded to 16 bytes");
  if (num_edges == 0) return EPP_OK;
  EPP_REQUIRE(col_idx && feat && sink && aligned(feat, 16), "null or misaligned pointer");
  const long long quads = ceil_div_ll(num_edges, 64);
  const long long blocks = ceil_div_ll(quads * 4, 256);
  if (blocks > 0x7fffffffLL) return EPP_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned ldb = static_cast<unsigned>(feat_ld) * 4u;
  const int tiles = (dim + 15) / 16;
  const unsigned grid = static_cast<unsigned>(blocks);
  if (tiles <= 1) gather_probe_kernel<1><<<grid, 256, 0, s>>>(col_idx, num_edges, feat, ldb, dim, sink);
  else if (tiles <= 2) gather_probe_kernel<2><<<grid, 256, 0, s>>>(col_idx, num_edges, feat, ldb, dim, sink);
  else if (tiles <= 4) gather_probe_kernel<4><<<grid, 256, 0, s>>>(col_idx, num_edges, feat, ldb, dim, sink);
  else gather_probe_kernel<8><<<grid, 256, 0, s>>>(col_idx, num_edges, feat, ldb, dim, sink);
  EPP_CHECK_LAUNCH("gather_probe_kernel");
  return EPP_OK;
}

