// Standalone global-softmax merge of a self branch with scattered remote contributions: the operator the
// reference exposes as merge_forward (src/moba_opt/ops/merge_cuda.py:32-60, ops/bindings.cpp:6-22,
// ops/merge.cu:27-288).  The prefill path does not use it (there the merge is the epilogue of the forward
// kernel); it exists for callers that hold the two branches themselves.
//   row p of the self branch (P = T*H rows) and every remote row m with mapping[m] == p are combined as
//   mx = max l, w = exp(l - mx), z = sum w, O = sum w o / z, L = mx + log z      (natural-log LSE, FP32 math)
// Two kernels: contributions are ticketed into per-row slot lists (atomic counters), then every row sorts
// its at most 32 contribution indices and reduces them in ascending order, so the result does not depend
// on the ticket order.  HBM-bound: every input byte is read once, every output byte written once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "moba_b200.h"
#include "sm100.cuh"

namespace moba {
namespace {

__global__ void __launch_bounds__(256) merge_ticket_kernel(const int64_t* __restrict__ mapping, long long M, long long P, int kmax,
                                                           int* __restrict__ counts, int* __restrict__ slots, unsigned* status) {
  const long long m = (long long)blockIdx.x * 256 + threadIdx.x;
  if (m >= M) return;
  const long long p = mapping[m];
  if (p < 0 || p >= P) { atomicOr(status, kErrBadIndex); return; }
  const int slot = atomicAdd(counts + p, 1);
  if (slot < kmax) slots[p * kmax + slot] = (int)m;
  else atomicOr(status, kErrCapacity);
}

// 16 bytes of a row as eight (bf16, half) or four (fp32) FP32 values.
template <typename T> struct Chunk;
template <> struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Chunk<__half> {
  static constexpr int N = 8;
  __device__ static void load(const __half* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static void store(__half* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Chunk<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};

// LPR lanes share a row (16 bytes of it each per pass), 32 / LPR rows per warp.  Every lane of a row's group
// sorts the row's few contribution indices itself and forms the weights, then accumulates its own columns
// in ascending index order: no cross-lane traffic, all loads 16 bytes wide.
template <typename T, int LPR>
__global__ void __launch_bounds__(256) merge_rows_kernel(const T* __restrict__ self_out, const float* __restrict__ self_lse,
                                                         const T* __restrict__ remote_out, const float* __restrict__ remote_lse,
                                                         const int* __restrict__ counts, const int* __restrict__ slots, long long P,
                                                         int D, int kmax, T* __restrict__ out, float* __restrict__ lse) {
  constexpr int N = Chunk<T>::N;
  const int lane = threadIdx.x & 31, sub = lane % LPR;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * (32 / LPR) + lane / LPR;
  if (row >= P) return;
  const int cnt = min(counts[row], kmax);
  int idx[32];
  float w[32];
  for (int i = 0; i < cnt; ++i) {  // insertion sort of the contribution indices (ascending)
    const int v = slots[row * kmax + i];
    int j = i;
    while (j > 0 && idx[j - 1] > v) { idx[j] = idx[j - 1]; --j; }
    idx[j] = v;
  }
  const float l_self = self_lse[row];
  float mx = l_self;
  for (int i = 0; i < cnt; ++i) { w[i] = remote_lse[idx[i]]; mx = fmaxf(mx, w[i]); }
  const bool empty = mx == -INFINITY;  // no branch saw a key: zero output, LSE stays -inf
  const float w_self = empty ? 0.f : expf(l_self - mx);
  float z = w_self;
  for (int i = 0; i < cnt; ++i) { w[i] = empty ? 0.f : expf(w[i] - mx); z += w[i]; }
  const float inv = z > 0.f ? 1.f / z : 0.f;
  for (int d = sub * N; d < D; d += LPR * N) {
    float acc[N], v[N];
    Chunk<T>::load(self_out + row * D + d, v);
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] = w_self * v[e];
    for (int i = 0; i < cnt; ++i) {
      Chunk<T>::load(remote_out + (long long)idx[i] * D + d, v);
#pragma unroll
      for (int e = 0; e < N; ++e) acc[e] = fmaf(w[i], v[e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] *= inv;
    Chunk<T>::store(out + row * D + d, acc);
  }
  if (sub == 0) lse[row] = empty ? -INFINITY : mx + logf(z);
}

// Fallback for head dimensions whose rows are not multiples of 16 bytes: one warp per row, scalar accesses.
template <typename T>
__global__ void __launch_bounds__(256) merge_rows_scalar_kernel(const T* __restrict__ self_out, const float* __restrict__ self_lse,
                                                                const T* __restrict__ remote_out, const float* __restrict__ remote_lse,
                                                                const int* __restrict__ counts, const int* __restrict__ slots,
                                                                long long P, int D, int kmax, T* __restrict__ out,
                                                                float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= P) return;
  const int cnt = min(counts[row], kmax);
  int idx[32];
  float w[32];
  for (int i = 0; i < cnt; ++i) {
    const int v = slots[row * kmax + i];
    int j = i;
    while (j > 0 && idx[j - 1] > v) { idx[j] = idx[j - 1]; --j; }
    idx[j] = v;
  }
  const float l_self = self_lse[row];
  float mx = l_self;
  for (int i = 0; i < cnt; ++i) { w[i] = remote_lse[idx[i]]; mx = fmaxf(mx, w[i]); }
  const bool empty = mx == -INFINITY;
  const float w_self = empty ? 0.f : expf(l_self - mx);
  float z = w_self;
  for (int i = 0; i < cnt; ++i) { w[i] = empty ? 0.f : expf(w[i] - mx); z += w[i]; }
  const float inv = z > 0.f ? 1.f / z : 0.f;
  for (int d = lane; d < D; d += 32) {
    float acc = w_self * (float)self_out[row * D + d];
    for (int i = 0; i < cnt; ++i) acc = fmaf(w[i], (float)remote_out[(long long)idx[i] * D + d], acc);
    out[row * D + d] = (T)(acc * inv);
  }
  if (lane == 0) lse[row] = empty ? -INFINITY : mx + logf(z);
}

template <typename T>
void launch_rows(const void* self_out, const float* self_lse, const void* remote_out, const float* remote_lse, const int* counts,
                 const int* slots, long long rows, int dim, int kmax, void* out, float* lse, cudaStream_t st) {
  const T* so = static_cast<const T*>(self_out);
  const T* ro = static_cast<const T*>(remote_out);
  T* o = static_cast<T*>(out);
  constexpr int N = Chunk<T>::N;
  const bool vec = dim % N == 0 && (reinterpret_cast<uintptr_t>(so) | reinterpret_cast<uintptr_t>(ro) | reinterpret_cast<uintptr_t>(o)) % 16 == 0;
  if (!vec) {
    merge_rows_scalar_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(so, self_lse, ro, remote_lse, counts, slots, rows, dim, kmax, o, lse);
    return;
  }
  const int chunks = dim / N;
  if (chunks <= 4) merge_rows_kernel<T, 4><<<(unsigned)((rows + 63) / 64), 256, 0, st>>>(so, self_lse, ro, remote_lse, counts, slots, rows, dim, kmax, o, lse);
  else if (chunks <= 8) merge_rows_kernel<T, 8><<<(unsigned)((rows + 31) / 32), 256, 0, st>>>(so, self_lse, ro, remote_lse, counts, slots, rows, dim, kmax, o, lse);
  else if (chunks <= 16) merge_rows_kernel<T, 16><<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(so, self_lse, ro, remote_lse, counts, slots, rows, dim, kmax, o, lse);
  else merge_rows_kernel<T, 32><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(so, self_lse, ro, remote_lse, counts, slots, rows, dim, kmax, o, lse);
}

inline size_t align256m(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace
}  // namespace moba

using namespace moba;

extern "C" size_t moba_merge_scratch_bytes(long long rows, int kmax) {
  if (rows < 1 || kmax < 1 || kmax > 32) return 0;
  return align256m((size_t)rows * 4) + align256m((size_t)rows * kmax * 4);
}

extern "C" int moba_merge_forward(const void* self_out, const float* self_lse, const void* remote_out, const float* remote_lse,
                                  const int64_t* mapping, long long rows, long long remote_rows, int dim, int kmax, int dtype,
                                  void* scratch, size_t scratch_bytes, void* out, float* lse, unsigned* status, void* stream) {
  if (rows < 1 || remote_rows < 0 || dim < 1 || !self_out || !self_lse || !out || !lse || !status || !scratch) return MOBA_ERR_INVALID;
  if (remote_rows > 0 && (!remote_out || !remote_lse || !mapping)) return MOBA_ERR_INVALID;
  if (kmax < 1 || kmax > 32 || dtype < 0 || dtype > 2) return MOBA_ERR_UNSUPPORTED;
  if (scratch_bytes < moba_merge_scratch_bytes(rows, kmax)) return MOBA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  int* counts = static_cast<int*>(scratch);
  int* slots = reinterpret_cast<int*>(static_cast<char*>(scratch) + align256m((size_t)rows * 4));
  if (cudaMemsetAsync(counts, 0, (size_t)rows * 4, st) != cudaSuccess) return MOBA_ERR_CUDA;
  if (remote_rows > 0)
    merge_ticket_kernel<<<(unsigned)((remote_rows + 255) / 256), 256, 0, st>>>(mapping, remote_rows, rows, kmax, counts, slots, status);
  if (dtype == 0)
    launch_rows<__nv_bfloat16>(self_out, self_lse, remote_out, remote_lse, counts, slots, rows, dim, kmax, out, lse, st);
  else if (dtype == 2)
    launch_rows<__half>(self_out, self_lse, remote_out, remote_lse, counts, slots, rows, dim, kmax, out, lse, st);
  else
    launch_rows<float>(self_out, self_lse, remote_out, remote_lse, counts, slots, rows, dim, kmax, out, lse, st);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
