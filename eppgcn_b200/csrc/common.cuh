// Shared helpers of the eppgcn_b200 C-ABI library: status plumbing, launch
// checks and the packed tile descriptor used by the single-pass scans.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/eppgcn_b200.h"

// Entry points are the only symbols the shared library exports.
#define EPP_EXPORT extern "C" __attribute__((visibility("default")))

namespace epp {

void set_error(const char *fmt, ...);

#define EPP_CUDA_TRY(expr)                                                        \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      ::epp::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                       __FILE__, __LINE__);                                       \
      return EPP_ERR_CUDA;                                                        \
    }                                                                             \
  } while (0)

#define EPP_CHECK_LAUNCH(name)                                                    \
  do {                                                                            \
    cudaError_t _e = cudaPeekAtLastError();                                       \
    if (_e != cudaSuccess) {                                                      \
      ::epp::set_error("launch of %s failed: %s", name, cudaGetErrorString(_e));  \
      (void)cudaGetLastError();                                                   \
      return EPP_ERR_CUDA;                                                        \
    }                                                                             \
  } while (0)

#define EPP_REQUIRE(cond, msg)                                                    \
  do {                                                                            \
    if (!(cond)) {                                                                \
      ::epp::set_error("%s: %s", __func__, msg);                                  \
      return EPP_ERR_BAD_ARG;                                                     \
    }                                                                             \
  } while (0)

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

__host__ __device__ inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// Flag words another GPU writes or reads: release / acquire at system scope.
__device__ __forceinline__ void store_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned load_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------------------
// Tile descriptor of the chained (decoupled look-back) scans.
// One 64-bit word per tile: bits 63..62 state, 61..31 field B, 30..0 field A.
// Both fields are partial sums of int32 totals that the host has checked to be
// below 2^31, so they never carry into each other.
// ---------------------------------------------------------------------------
constexpr unsigned long long kTileEmpty = 0ull;
constexpr unsigned long long kTileAggregate = 1ull;   // sum of this tile only
constexpr unsigned long long kTilePrefix = 2ull;      // sum of tiles 0..this

__host__ __device__ inline unsigned long long tile_pack(unsigned long long state, unsigned a, unsigned b) {
  return (state << 62) | (static_cast<unsigned long long>(b) << 31) | static_cast<unsigned long long>(a);
}
__host__ __device__ inline unsigned tile_state(unsigned long long w) { return static_cast<unsigned>(w >> 62); }
__host__ __device__ inline unsigned tile_a(unsigned long long w) { return static_cast<unsigned>(w & 0x7fffffffull); }
__host__ __device__ inline unsigned tile_b(unsigned long long w) { return static_cast<unsigned>((w >> 31) & 0x7fffffffull); }

// Layout of the scratch buffer handed to the scan entry points.
struct ScanHeader {
  unsigned int ticket;      // next tile id to hand out
  int error;                // EPP_OK or EPP_ERR_SCAN_TIMEOUT
  unsigned int pad[62];     // keeps the descriptors 256-byte aligned
};
static_assert(sizeof(ScanHeader) == 256, "ScanHeader must be 256 bytes");

}  // namespace epp
