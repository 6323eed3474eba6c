// Row-piece stores shared by the aggregation kernels: a lane owns VEC
// consecutive columns of a result row and writes the first n of them (n < VEC
// only for the lane that holds the row's last, partial piece).
#pragma once

#include "common.cuh"

namespace epp {

inline bool aligned(const void *p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

// Writes n (<= VEC) floats starting at p with the widest store `ovec` allows
// (ovec = 4, 2 or 1: p and the row stride are aligned to that many floats).
template <int VEC>
__device__ __forceinline__ void store_row(float *p, const float (&v)[VEC], int n, int ovec) {
  if (VEC == 4 && ovec == 4 && n == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if (VEC >= 2 && ovec >= 2) {
#pragma unroll
    for (int i = 0; i + 1 < VEC; i += 2)
      if (i + 1 < n) *reinterpret_cast<float2 *>(p + i) = make_float2(v[i], v[i + 1]);
#pragma unroll
    for (int i = 0; i < VEC; i += 2)
      if (i + 1 == n) p[i] = v[i];               // odd n: the last column has no partner
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
#pragma unroll
    for (int i = 0; i < VEC; i += 2)
      if (i + 1 == n) atomicAdd(p + i, v[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) atomicAdd(p + i, v[i]);
  }
}

// Zeroes columns 0 .. dim-1 of num_rows rows that are out_ld floats apart.
int zero_column_block(float *out, long long out_ld, int dim, long long num_rows, cudaStream_t s);

// Per-device memo of "this kernel may use `smem` bytes of dynamic shared
// memory": cudaFuncSetAttribute is a per-device setting, so it is repeated on
// every device a process uses; the memo only avoids repeating it per launch.
struct SmemOptIn {
  static constexpr int kMaxDevices = 64;
  int granted[kMaxDevices];
  SmemOptIn() { for (int &g : granted) g = 0; }
};
int smem_opt_in(SmemOptIn &memo, const void *kernel, int smem);
int device_sm_count(int *num_sms);

}  // namespace epp
