// Row exchange between the GPUs of one node for the row-partitioned
// aggregation: the rows other ranks' edges reference are gathered from this
// rank's matrix and stored straight into the readers' source buffers over
// NVLink (plain peer stores, no staging copy, no library collective), and a
// flag barrier with bounded waits orders the pushes against the readers'
// kernels.  The reference is single-GPU and has no counterpart of this file.
//
// Only plain per-thread loads and stores touch peer memory here, each addressed
// to one GPU.  Every wait has an iteration limit; when it runs out the kernel
// records EPP_ERR_PEER_TIMEOUT in a status word and returns.
#include "rowio.cuh"

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

// The same push peer by peer, with a word stored into every served peer's "landed" array as soon as
// all of its rows are there, so that a reader can start on one owner's rows while the others still
// travel.  The send list is cut into chunks of kPushChunkRows rows that never straddle two peers; a
// block takes chunks c = blockIdx.x, blockIdx.x + gridDim.x, ... in the order the peers are served, and
// the block that stores a peer's last chunk signals it.
constexpr int kPushChunkRows = 512;

struct SignalTable {
  unsigned *landed[kMaxPeers];      // the word of peer r's array that this rank writes, as mapped here
  int order[kMaxPeers];             // i-th peer to be served
  int chunk_ptr[kMaxPeers + 1];     // chunks [chunk_ptr[i], chunk_ptr[i+1]) go to peer order[i]
};

__global__ void __launch_bounds__(256) push_rows_signal_kernel(const float *__restrict__ rows, long long rows_ld,
                                                               const int *__restrict__ send_idx, PeerTable t,
                                                               SignalTable g, long long peer_ld, int pieces, int world,
                                                               const unsigned *epoch, unsigned *done) {
  const unsigned value = *epoch;              // written by an earlier launch of the stream, constant during this one
  const int total_chunks = g.chunk_ptr[world];
  for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    int i = 0;
#pragma unroll
    for (int k = 1; k < kMaxPeers; ++k) i += (k < world && c >= g.chunk_ptr[k]) ? 1 : 0;
    const int r = g.order[i];
    const long long j0 = t.send_ptr[r] + static_cast<long long>(c - g.chunk_ptr[i]) * kPushChunkRows;
    const long long left = t.send_ptr[r + 1] - j0;
    const int count = static_cast<int>(left < kPushChunkRows ? left : kPushChunkRows);
    float *base = static_cast<float *>(t.base[r]) + (t.first_row[r] + (j0 - t.send_ptr[r])) * peer_ld;
    // four pieces per thread and turn: the gathers of a turn are in flight together before the first peer store
    const int total = count * pieces;
    for (int e0 = threadIdx.x; e0 < total; e0 += 4 * blockDim.x) {
      float4 v[4];
      int at[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * blockDim.x;
        at[u] = -1;
        if (e < total) {
          const int jj = e / pieces, q = e - jj * pieces;
          at[u] = jj * static_cast<int>(peer_ld) + q * 4;
          v[u] = __ldg(reinterpret_cast<const float4 *>(rows + static_cast<long long>(__ldg(send_idx + j0 + jj)) * rows_ld) + q);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (at[u] >= 0) *reinterpret_cast<float4 *>(base + at[u]) = v[u];
    }
    __threadfence_system();                   // this thread's stores have reached the peer before the block counts itself
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned chunks = static_cast<unsigned>(g.chunk_ptr[i + 1] - g.chunk_ptr[i]);
      if (atomicAdd(done + i, 1u) + 1u == chunks) {
        done[i] = 0u;                         // ready for the next launch
        store_release_sys(g.landed[r], value);
      }
    }
  }
}

__global__ void bump_kernel(unsigned *counter) { *counter += 1u; }

// Lane r waits (bounded) until word r of this rank's "landed" array has reached *epoch, for every r in
// `owners`.  A launch of its own in front of the aggregation that reads those owners' rows: the waiting
// warp occupies one block slot, so it cannot keep this GPU's own push from running, and the readers start
// with a cold L1.
__global__ void wait_landed_kernel(const unsigned *landed, unsigned owners, const unsigned *epoch, long long max_polls,
                                   int *status) {
  const int r = threadIdx.x;
  bool timed_out = false;
  if ((owners >> r) & 1u) {
    const unsigned want = *epoch;
    const bool broken = *reinterpret_cast<volatile int *>(status) != EPP_OK;
    long long polls = 0;
    while (!broken && static_cast<int>(load_acquire_sys(landed + r) - want) < 0) {
      if (++polls > max_polls) { timed_out = true; break; }
      __nanosleep(polls < 64 ? 100 : 1000);
    }
  }
  __threadfence_system();
  if (timed_out) atomicExch(status, EPP_ERR_PEER_TIMEOUT);
}

struct FlagTable {
  unsigned *flags[kMaxPeers];       // peer r's flag array (one word per rank), as mapped into this process
};

// Lane r tells peer r "this rank has reached barrier `value`" and waits for
// peer r's word in this rank's own flag array.  Words only grow (modulo 2^32).
__device__ __forceinline__ void barrier_body(const FlagTable &t, int rank, int world, unsigned value,
                                             long long max_polls, int *status) {
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

__global__ void peer_barrier_kernel(FlagTable t, int rank, int world, unsigned value, long long max_polls,
                                    int *status) {
  barrier_body(t, rank, world, value, max_polls, status);
}

// The same barrier numbered on the device: every launch takes the next number from a word of this
// rank's memory, so a captured launch can be replayed (all ranks replay the same sequence).
__global__ void peer_barrier_counted_kernel(FlagTable t, int rank, int world, unsigned *counter, long long max_polls,
                                            int *status) {
  unsigned value = 0;
  if (threadIdx.x == 0) {
    value = *counter + 1u;
    *counter = value;
  }
  value = __shfl_sync(0xffffffffu, value, 0);
  barrier_body(t, rank, world, value, max_polls, status);
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

EPP_EXPORT int eppgcn_peer_barrier_counted(void *const *peer_flags, int rank, int world, unsigned *counter_dev,
                                           long long max_polls, int *status_dev, void *stream) {
  EPP_REQUIRE(world >= 1 && world <= epp::kMaxPeers && rank >= 0 && rank < world, "rank/world out of range");
  EPP_REQUIRE(peer_flags && counter_dev && status_dev && max_polls >= 1, "null pointer or max_polls < 1");
  epp::FlagTable t{};
  for (int r = 0; r < world; ++r) {
    EPP_REQUIRE(peer_flags[r] != nullptr, "null flag array");
    t.flags[r] = static_cast<unsigned *>(peer_flags[r]);
  }
  epp::peer_barrier_counted_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, rank, world, counter_dev,
                                                                                   max_polls, status_dev);
  EPP_CHECK_LAUNCH("peer_barrier_counted_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_push_rows_signal(const float *rows, long long rows_ld, const int *send_idx,
                                       const long long *send_ptr, void *const *peer_base,
                                       const long long *peer_first_row, long long peer_ld, int dim, int world,
                                       int rank, void *const *peer_landed, const unsigned *epoch_dev,
                                       unsigned *done_dev, void *stream) {
  using namespace epp;
  EPP_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "rank/world out of range");
  EPP_REQUIRE(dim >= 4 && dim % 4 == 0 && rows_ld % 4 == 0 && peer_ld % 4 == 0 && rows_ld >= dim && peer_ld >= dim,
              "rows must be whole 16-byte pieces");
  EPP_REQUIRE(send_ptr && peer_base && peer_first_row && peer_landed && epoch_dev && done_dev, "null pointer");
  PeerTable t{};
  for (int r = 0; r <= world; ++r) {
    EPP_REQUIRE(send_ptr[r] >= 0 && (r == 0 || send_ptr[r] >= send_ptr[r - 1]), "send_ptr must be a non-decreasing prefix");
    t.send_ptr[r] = send_ptr[r];
  }
  EPP_REQUIRE(send_ptr[0] == 0, "send_ptr must start at 0");
  EPP_REQUIRE(send_ptr[rank + 1] == send_ptr[rank], "a rank sends no rows to itself");
  if (send_ptr[world] == 0) return EPP_OK;
  EPP_REQUIRE(rows && send_idx, "null pointer");
  EPP_REQUIRE((reinterpret_cast<uintptr_t>(rows) % 16) == 0, "rows must be 16-byte aligned");
  SignalTable g{};
  int chunks = 0;
  for (int i = 0; i < world; ++i) {
    // peers are served leftwards from the rank: rank-1, rank-2, ...; so every rank receives its right-hand
    // neighbour's rows first, then the next one's, and no two ranks store into the same peer at a time
    const int r = ((rank - 1 - i) % world + world) % world;
    const long long count = send_ptr[r + 1] - send_ptr[r];
    EPP_REQUIRE(count == 0 || (peer_base[r] && (reinterpret_cast<uintptr_t>(peer_base[r]) % 16) == 0 &&
                               peer_first_row[r] >= 0 && peer_landed[r]),
                "peer buffer or landed word missing or misaligned");
    t.base[r] = peer_base[r];
    t.first_row[r] = peer_first_row[r];
    g.order[i] = r;
    g.landed[r] = count ? static_cast<unsigned *>(peer_landed[r]) + rank : nullptr;
    g.chunk_ptr[i] = chunks;
    const long long c = ceil_div_ll(count, kPushChunkRows);
    EPP_REQUIRE(chunks + c < (1LL << 30), "too many rows");
    chunks += static_cast<int>(c);
  }
  g.chunk_ptr[world] = chunks;
  int sms = 148;
  if (const int rc = device_sm_count(&sms); rc != EPP_OK) return rc;
  // one block per SM at most: the push is bound by the links, and the aggregation that runs beside it keeps
  // the rest of every SM
  const int blocks = chunks < sms ? chunks : sms;
  push_rows_signal_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      rows, rows_ld, send_idx, t, g, peer_ld, dim / 4, world, epoch_dev, done_dev);
  EPP_CHECK_LAUNCH("push_rows_signal_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_bump_counter(unsigned *counter_dev, void *stream) {
  EPP_REQUIRE(counter_dev, "null pointer");
  epp::bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(counter_dev);
  EPP_CHECK_LAUNCH("bump_kernel");
  return EPP_OK;
}

EPP_EXPORT int eppgcn_wait_landed(const unsigned *landed_dev, unsigned owners, const unsigned *epoch_dev,
                                  long long max_polls, int *status_dev, void *stream) {
  EPP_REQUIRE(landed_dev && epoch_dev && status_dev && max_polls >= 1, "null pointer or max_polls < 1");
  EPP_REQUIRE((owners >> epp::kMaxPeers) == 0, "owners beyond rank 15");
  if (owners == 0) return EPP_OK;
  epp::wait_landed_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(landed_dev, owners, epoch_dev, max_polls,
                                                                          status_dev);
  EPP_CHECK_LAUNCH("wait_landed_kernel");
  return EPP_OK;
}
