// Host side of the C-ABI: status strings, the CPU helpers of the operator API
// (group partition, part-size rules, degree histogram) and the lazily resolved
// event timers behind print_time / clear_time.
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "rowio.cuh"

namespace epp {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static std::mutex g_launch_mu;

int smem_opt_in(SmemOptIn &memo, const void *kernel, int smem) {
  if (smem <= 48 * 1024) return EPP_OK;
  int dev = 0;
  EPP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= SmemOptIn::kMaxDevices) {
    set_error("device ordinal %d is beyond the %d devices this library tracks", dev, SmemOptIn::kMaxDevices);
    return EPP_ERR_TOO_LARGE;
  }
  std::lock_guard<std::mutex> lock(g_launch_mu);
  if (memo.granted[dev] < smem) {
    EPP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    memo.granted[dev] = smem;
  }
  return EPP_OK;
}

int device_sm_count(int *num_sms) {
  int dev = 0;
  EPP_CUDA_TRY(cudaGetDevice(&dev));
  EPP_CUDA_TRY(cudaDeviceGetAttribute(num_sms, cudaDevAttrMultiProcessorCount, dev));
  return EPP_OK;
}

namespace {

struct PendingTime {
  cudaEvent_t start, stop;
  int category, layer;
  bool ended;
  int id;
};

struct Timers {
  std::mutex mu;
  bool enabled = true;
  float acc[11] = {0};                 // 0..4 categories, 5..10 per-layer backward aggregation
  std::vector<PendingTime> pending;    // looked up by id
  std::vector<cudaEvent_t> pool;
  int next_id = 0;

  cudaEvent_t get_event() {
    if (!pool.empty()) {
      cudaEvent_t e = pool.back();
      pool.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
  // Folds every finished pair into the accumulators.  `wait` blocks on pairs
  // still in flight; otherwise they stay pending.
  void resolve(bool wait) {
    std::vector<PendingTime> keep;
    for (PendingTime &p : pending) {
      if (!p.ended) { keep.push_back(p); continue; }
      cudaError_t q = wait ? cudaEventSynchronize(p.stop) : cudaEventQuery(p.stop);
      if (q == cudaErrorNotReady) { keep.push_back(p); continue; }
      float ms = 0.f;
      if (q == cudaSuccess && cudaEventElapsedTime(&ms, p.start, p.stop) == cudaSuccess) {
        acc[p.category] += ms;
        if (p.category == 2 && p.layer >= 1 && p.layer <= 6) acc[4 + p.layer] += ms;
      } else {
        (void)cudaGetLastError();
      }
      pool.push_back(p.start);
      pool.push_back(p.stop);
    }
    pending.swap(keep);
  }
};

Timers &timers() {
  static Timers t;
  return t;
}

}  // namespace
}  // namespace epp

using namespace epp;

EPP_EXPORT int eppgcn_version(void) { return 100; }

EPP_EXPORT const char *eppgcn_status_string(int status) {
  switch (status) {
    case EPP_OK: return "EPP_OK";
    case EPP_ERR_BAD_ARG: return "EPP_ERR_BAD_ARG";
    case EPP_ERR_CUDA: return "EPP_ERR_CUDA";
    case EPP_ERR_SCAN_TIMEOUT: return "EPP_ERR_SCAN_TIMEOUT";
    case EPP_ERR_TOO_LARGE: return "EPP_ERR_TOO_LARGE";
    case EPP_ERR_PEER_TIMEOUT: return "EPP_ERR_PEER_TIMEOUT";
    default: return "EPP_ERR_UNKNOWN";
  }
}

EPP_EXPORT const char *eppgcn_last_error(void) { return g_error; }

EPP_EXPORT int eppgcn_build_part_host(int part_size, const int *indptr, int num_nodes, int *part_ptr,
                                      int *part2node, long long *num_parts) {
  EPP_REQUIRE(part_size >= 1, "partSize must be >= 1");
  EPP_REQUIRE(num_nodes >= 0 && indptr && num_parts, "bad argument");
  long long total = 0;
  for (int v = 0; v < num_nodes; ++v) {
    const long long deg = static_cast<long long>(indptr[v + 1]) - indptr[v];
    EPP_REQUIRE(deg >= 0, "indptr must be non-decreasing");
    total += (deg + part_size - 1) / part_size;
  }
  *num_parts = total;
  if (!part_ptr) return EPP_OK;
  EPP_REQUIRE(part2node || total == 0, "null pointer");
  if (total >= 0x7fffffffLL) {
    set_error("group count exceeds int32");
    return EPP_ERR_TOO_LARGE;
  }
  long long g = 0;
  for (int v = 0; v < num_nodes; ++v) {
    const int beg = indptr[v], end = indptr[v + 1];
    for (long long e = beg; e < end; e += part_size) {
      part_ptr[g] = static_cast<int>(e);
      part2node[g] = v;
      ++g;
    }
  }
  part_ptr[g] = indptr[num_nodes];
  return EPP_OK;
}

EPP_EXPORT int eppgcn_map_back_part_size(int valid_node, int valid_len, int *part_size) {
  EPP_REQUIRE(part_size, "null pointer");
  EPP_REQUIRE(valid_node > 0, "no active vertex");
  const double valid_degree = 1.0 * valid_len / valid_node;
  const double beta0 = 0.65538, beta1 = 1.67431e-5, beta2 = -2.24342e-6, beta3 = 0.63641;
  *part_size = static_cast<int>(round(beta0 + beta1 * valid_node + beta2 * valid_len + beta3 * valid_degree));
  return EPP_OK;
}

EPP_EXPORT int eppgcn_bucket_back_part_size(int valid_node, int valid_len, int *part_size) {
  EPP_REQUIRE(part_size, "null pointer");
  EPP_REQUIRE(valid_node > 0, "no active vertex");
  const int d = valid_len / valid_node;
  int ps = 0;
  if (d < 4) ps = 4;
  else if (d < 16) ps = 8;
  else if (d < 64) ps = 16;
  else if (d < 256) ps = 32;
  else if (d < 512) ps = 64;
  *part_size = ps;
  return EPP_OK;
}

EPP_EXPORT int eppgcn_get_ginfo_host(const int *node_deg, int num_nodes, int valid_len, float *out10) {
  EPP_REQUIRE(num_nodes >= 0 && out10 && (node_deg || num_nodes == 0), "bad argument");
  long long h[10] = {0};
  for (int i = 0; i < num_nodes; ++i) {
    const int d = node_deg[i];
    if (d != 0) ++h[0];
    if (d >= 1 && d < 5) ++h[3];
    else if (d >= 5 && d < 10) ++h[4];
    else if (d >= 10 && d < 20) ++h[5];
    else if (d >= 20 && d < 40) ++h[6];
    else if (d >= 40 && d < 80) ++h[7];
    else if (d >= 80 && d < 160) ++h[8];
    else ++h[9];
  }
  const int valid_node = static_cast<int>(h[0]);
  // The reference divides by valid_node unguarded (EPPGCN.cpp:378-384); an
  // entry point that never takes the process down reports the empty path instead.
  EPP_REQUIRE(valid_node > 0, "no active vertex");
  out10[0] = static_cast<float>(valid_node * 1.0 / 10000);
  out10[1] = static_cast<float>(valid_len * 1.0 / 10000);
  out10[2] = static_cast<float>(1.0 * valid_len / valid_node);
  for (int i = 3; i < 10; ++i) out10[i] = static_cast<float>(static_cast<float>(h[i]) * 1.0 / valid_node);
  return EPP_OK;
}

EPP_EXPORT int eppgcn_timing_enable(int on) {
  Timers &t = timers();
  std::lock_guard<std::mutex> lock(t.mu);
  const int prev = t.enabled ? 1 : 0;
  t.enabled = on != 0;
  return prev;
}

EPP_EXPORT int eppgcn_time_begin(void *stream) {
  Timers &t = timers();
  std::lock_guard<std::mutex> lock(t.mu);
  if (!t.enabled) return -1;
  if (t.pending.size() >= 2048) t.resolve(false);
  if (t.pending.size() >= 8192) t.resolve(true);
  PendingTime p{t.get_event(), t.get_event(), 0, 0, false, t.next_id};
  t.next_id = (t.next_id + 1) & 0x3fffffff;
  if (!p.start || !p.stop || cudaEventRecord(p.start, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  t.pending.push_back(p);
  return p.id;
}

EPP_EXPORT int eppgcn_time_end(int slot, int category, int layer, void *stream) {
  if (slot < 0) return EPP_OK;
  Timers &t = timers();
  std::lock_guard<std::mutex> lock(t.mu);
  EPP_REQUIRE(category >= 0 && category <= 4, "unknown timer category");
  int i = static_cast<int>(t.pending.size()) - 1;
  while (i >= 0 && t.pending[i].id != slot) --i;
  if (i < 0 || t.pending[i].ended) return EPP_OK;
  PendingTime &p = t.pending[i];
  p.category = category;
  p.layer = layer;
  EPP_CUDA_TRY(cudaEventRecord(p.stop, static_cast<cudaStream_t>(stream)));
  p.ended = true;
  return EPP_OK;
}

EPP_EXPORT int eppgcn_time_read(float *out11) {
  EPP_REQUIRE(out11, "null pointer");
  Timers &t = timers();
  std::lock_guard<std::mutex> lock(t.mu);
  t.resolve(true);
  memcpy(out11, t.acc, sizeof(t.acc));
  return EPP_OK;
}

// Same keys and "%.6f" seconds as the reference's print_time
// (EPPGCN/GCNConv/EPPGCN_kernel.cu:96-106), which scripts grep.
EPP_EXPORT int eppgcn_print_time(void) {
  float a[11];
  const int rc = eppgcn_time_read(a);
  if (rc != EPP_OK) return rc;
  printf("for_agg_time: %.6f\n", a[0] / 1000);
  printf("back_agg_time: %.6f\n", a[2] / 1000);
  for (int i = 0; i < 6 && a[5 + i] != 0.0f; ++i) printf("l%d_back_agg_time: %.6f\n", i + 1, a[5 + i] / 1000);
  printf("mask_time: %.6f\n", a[4] / 1000);
  fflush(stdout);
  return EPP_OK;
}

// The reference's clear_time leaves mask_time alone
// (EPPGCN/GCNConv/EPPGCN_kernel.cu:108-116); so does this.
EPP_EXPORT int eppgcn_clear_time(void) {
  Timers &t = timers();
  std::lock_guard<std::mutex> lock(t.mu);
  t.resolve(true);
  const float mask = t.acc[4];
  memset(t.acc, 0, sizeof(t.acc));
  t.acc[4] = mask;
  return EPP_OK;
}
