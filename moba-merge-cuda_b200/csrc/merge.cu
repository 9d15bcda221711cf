// Standalone global-softmax merge of a self branch with scattered remote contributions: the operator the
// reference exposes as merge_forward (src/moba_opt/ops/merge_cuda.py:32-60, ops/bindings.cpp:6-22,
// ops/merge.cu:27-288).  The prefill path does not use it (there the merge is the epilogue of the forward
// kernel); it exists for callers that hold the two branches themselves.
//   row p of the self branch (P = T*H rows) and every remote row m with mapping[m] == p are combined as
//   mx = max l, w = exp(l - mx), z = sum w, O = sum w o / z, L = mx + log z      (natural-log LSE, FP32 math)
// Two kernels: contributions are ticketed into per-row slot lists (atomic counters), then one warp per row
// sorts its at most 32 contribution indices and reduces them in ascending order, so the result does not
// depend on the ticket order.  HBM-bound: every input byte is read once, every output byte written once.
#include <cuda_bf16.h>
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

template <typename T> __device__ __forceinline__ float load_f(const T* p);
template <> __device__ __forceinline__ float load_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void store_f(T* p, float v);
template <> __device__ __forceinline__ void store_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One warp per row.
template <typename T>
__global__ void __launch_bounds__(256) merge_rows_kernel(const T* __restrict__ self_out, const float* __restrict__ self_lse,
                                                         const T* __restrict__ remote_out, const float* __restrict__ remote_lse,
                                                         const int* __restrict__ counts, const int* __restrict__ slots, long long P,
                                                         int D, int kmax, T* __restrict__ out, float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= P) return;
  const int cnt = min(counts[row], kmax);
  // contribution indices in ascending order: rank by counting smaller ones, then hand each rank its value
  const int mine = lane < cnt ? slots[row * kmax + lane] : 0x7FFFFFFF;
  int rank = 0;
  for (int i = 0; i < cnt; ++i) rank += __shfl_sync(0xFFFFFFFFu, mine, i) < mine;
  int idx = 0x7FFFFFFF;
  for (int i = 0; i < cnt; ++i) {
    const int v = __shfl_sync(0xFFFFFFFFu, mine, i), r = __shfl_sync(0xFFFFFFFFu, rank, i);
    if (r == lane) idx = v;
  }
  const float l_self = self_lse[row];
  const float l_mine = lane < cnt ? remote_lse[idx] : -INFINITY;
  float mx = fmaxf(l_self, l_mine);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  const bool empty = mx == -INFINITY;  // no branch saw a key: zero output, LSE stays -inf
  const float w_self = empty ? 0.f : expf(l_self - mx);
  const float w_mine = (empty || lane >= cnt) ? 0.f : expf(l_mine - mx);
  float z = w_self;
  for (int i = 0; i < cnt; ++i) z += __shfl_sync(0xFFFFFFFFu, w_mine, i);  // fixed order
  const float inv = z > 0.f ? 1.f / z : 0.f;
  for (int d = lane; d < D; d += 32) {
    float acc = w_self * load_f(self_out + row * D + d);
    for (int i = 0; i < cnt; ++i) {
      const float w = __shfl_sync(0xFFFFFFFFu, w_mine, i);
      const int m = __shfl_sync(0xFFFFFFFFu, idx, i);
      acc = fmaf(w, load_f(remote_out + (long long)m * D + d), acc);
    }
    store_f(out + row * D + d, acc * inv);
  }
  if (lane == 0) lse[row] = empty ? -INFINITY : mx + logf(z);
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
  if (kmax < 1 || kmax > 32 || (dtype != 0 && dtype != 1)) return MOBA_ERR_UNSUPPORTED;
  if (scratch_bytes < moba_merge_scratch_bytes(rows, kmax)) return MOBA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  int* counts = static_cast<int*>(scratch);
  int* slots = reinterpret_cast<int*>(static_cast<char*>(scratch) + align256m((size_t)rows * 4));
  if (cudaMemsetAsync(counts, 0, (size_t)rows * 4, st) != cudaSuccess) return MOBA_ERR_CUDA;
  if (remote_rows > 0)
    merge_ticket_kernel<<<(unsigned)((remote_rows + 255) / 256), 256, 0, st>>>(mapping, remote_rows, rows, kmax, counts, slots, status);
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == 0)
    merge_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(self_out), self_lse,
                                                           static_cast<const __nv_bfloat16*>(remote_out), remote_lse, counts, slots,
                                                           rows, dim, kmax, static_cast<__nv_bfloat16*>(out), lse);
  else
    merge_rows_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(self_out), self_lse, static_cast<const float*>(remote_out),
                                                   remote_lse, counts, slots, rows, dim, kmax, static_cast<float*>(out), lse);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
