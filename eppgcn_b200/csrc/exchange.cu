// Row exchange between the GPUs of one node for the row-partitioned
// aggregation: the rows other ranks' edges reference are gathered from this
// rank's matrix and stored straight into the readers' source buffers over
// NVLink (plain peer stores, no staging copy, no library collective), and a
// flag barrier with bounded waits orders the pushes against the readers'
// kernels.  The reference is single-GPU and has no counterpart of this file.
//
// Only plain loads and stores touch peer memory here: no bulk/TMA copies, no
// multicast.  Every wait has an iteration limit; when it runs out the kernel
// records EPP_ERR_PEER_TIMEOUT in a status word and returns.
#include "common.cuh"

namespace epp {
namespace {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void *base[kMaxPeers];            // peer r's buffer, as mapped into this process
  long long first_row[kMaxPeers];   // where this rank's rows start in peer r's buffer
  long long send_ptr[kMaxPeers + 1];// rows [send_ptr[r], send_ptr[r+1]) of the send list go to peer r
};

// One float4 per thread: send-list entry j, piece q of its row.  The walk over
// the send list starts at entry start_row and wraps around, so that the ranks
// of a group, each starting at its right-hand neighbour's rows, store into
// different peers at any one time instead of all into rank 0 first.
__global__ void __launch_bounds__(256) push_rows_kernel(const float *__restrict__ rows, long long rows_ld,
                                                        const int *__restrict__ send_idx, PeerTable t,
                                                        long long peer_ld, int pieces, int world,
                                                        long long start_row) {
  const long long num_rows = t.send_ptr[world];
  const long long total = num_rows * pieces;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long j0 = i / pieces;
    const int q = static_cast<int>(i - j0 * pieces);
    long long j = j0 + start_row;
    if (j >= num_rows) j -= num_rows;
    int r = 0;
#pragma unroll
    for (int k = 1; k < kMaxPeers; ++k) r += (k < world && j >= t.send_ptr[k]) ? 1 : 0;
    const float4 v = __ldg(reinterpret_cast<const float4 *>(rows + static_cast<long long>(__ldg(send_idx + j)) * rows_ld) + q);
    float *dst = static_cast<float *>(t.base[r]) + (t.first_row[r] + (j - t.send_ptr[r])) * peer_ld;
    reinterpret_cast<float4 *>(dst)[q] = v;
  }
}

struct FlagTable {
  unsigned *flags[kMaxPeers];       // peer r's flag array (one word per rank), as mapped into this process
};

__device__ __forceinline__ void store_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned load_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Lane r tells peer r "this rank has reached barrier `value`" and waits for
// peer r's word in this rank's own flag array.  Words only grow (modulo 2^32).
__global__ void peer_barrier_kernel(FlagTable t, int rank, int world, unsigned value, long long max_polls,
                                    int *status) {
  const int r = threadIdx.x;
  __threadfence_system();
  bool timed_out = false;
  if (r < world) {
    store_release_sys(t.flags[r] + rank, value);
    const unsigned *mine = t.flags[rank] + r;
    long long polls = 0;
    // an earlier barrier that gave up leaves its mark: announce the arrival, but do not wait again
    const bool broken = *reinterpret_cast<volatile int *>(status) != EPP_OK;
    while (!broken && static_cast<int>(load_acquire_sys(mine) - value) < 0) {
      if (++polls > max_polls) { timed_out = true; break; }
      __nanosleep(polls < 64 ? 100 : 1000);
    }
  }
  __threadfence_system();
  if (timed_out) atomicExch(status, EPP_ERR_PEER_TIMEOUT);
}

}  // namespace
}  // namespace epp

EPP_EXPORT int eppgcn_push_rows(const float *rows, long long rows_ld, const int *send_idx,
                                const long long *send_ptr, void *const *peer_base,
                                const long long *peer_first_row, long long peer_ld, int dim, int world,
                                long long start_row, void *stream) {
  EPP_REQUIRE(world >= 1 && world <= epp::kMaxPeers, "world must be 1..16");
  EPP_REQUIRE(dim >= 4 && dim % 4 == 0 && rows_ld % 4 == 0 && peer_ld % 4 == 0 && rows_ld >= dim && peer_ld >= dim,
              "rows must be whole 16-byte pieces");
  EPP_REQUIRE(send_ptr && peer_base && peer_first_row, "null pointer");
  epp::PeerTable t{};
  for (int r = 0; r <= world; ++r) {
    EPP_REQUIRE(send_ptr[r] >= 0 && (r == 0 || send_ptr[r] >= send_ptr[r - 1]), "send_ptr must be a non-decreasing prefix");
    t.send_ptr[r] = send_ptr[r];
  }
  EPP_REQUIRE(send_ptr[0] == 0, "send_ptr must start at 0");
  const long long total_rows = send_ptr[world];
  if (total_rows == 0) return EPP_OK;
  EPP_REQUIRE(start_row >= 0 && start_row < total_rows, "start_row must be an entry of the send list");
  EPP_REQUIRE(rows && send_idx, "null pointer");
  EPP_REQUIRE((reinterpret_cast<uintptr_t>(rows) % 16) == 0, "rows must be 16-byte aligned");
  for (int r = 0; r < world; ++r) {
    const bool used = send_ptr[r + 1] > send_ptr[r];
    EPP_REQUIRE(!used || (peer_base[r] && (reinterpret_cast<uintptr_t>(peer_base[r]) % 16) == 0 && peer_first_row[r] >= 0),
                "peer buffer missing or misaligned");
    t.base[r] = peer_base[r];
    t.first_row[r] = peer_first_row[r];
  }
  const int pieces = dim / 4;
  long long blocks = epp::ceil_div_ll(total_rows * pieces, 256 * 4);
  if (blocks > 148 * 8) blocks = 148 * 8;
  epp::push_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      rows, rows_ld, send_idx, t, peer_ld, pieces, world, start_row);
  EPP_CHECK_LAUNCH("push_rows_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_peer_barrier(void *const *peer_flags, int rank, int world, unsigned value,
                                   long long max_polls, int *status_dev, void *stream) {
  EPP_REQUIRE(world >= 1 && world <= epp::kMaxPeers && rank >= 0 && rank < world, "rank/world out of range");
  EPP_REQUIRE(peer_flags && status_dev && max_polls >= 1, "null pointer or max_polls < 1");
  epp::FlagTable t{};
  for (int r = 0; r < world; ++r) {
    EPP_REQUIRE(peer_flags[r] != nullptr, "null flag array");
    t.flags[r] = static_cast<unsigned *>(peer_flags[r]);
  }
  epp::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, rank, world, value, max_polls,
                                                                           status_dev);
  EPP_CHECK_LAUNCH("peer_barrier_kernel");
  return EPP_OK;
}
