// Device self-test of the tcgen05 tile primitives in sm100.cuh: one CTA multiplies two bf16
// matrices through shared-memory operand descriptors in each operand-major combination the
// attention kernels use, and returns the fp32 accumulator read back from tensor memory.
//   mode 0:  D[128,N]  = A[128,K] * B[N,K]^T     (both operands K-major;   S = Q K^T, dP = dO V^T)
//   mode 1:  D[128,N]  = A[128,K] * B[K,N]       (A K-major, B MN-major;   O = P V,  dQ = dS K)
//   mode 2:  D[128,N]  = A[K,128]^T * B[K,N]     (both operands MN-major;  dV = P^T dO, dK = dS^T Q)
//   mode 3:  D[128,N]  = A[128,K] * B[K,N]       (A in tensor memory as packed bf16 pairs, B MN-major; O = P V)
#include "moba_b200.h"
#include "moba_b200_debug.h"
#include "sm100.cuh"

namespace moba {

__device__ __forceinline__ void load_tile_sw128(uint8_t* tile, const __nv_bfloat16* g, int rows, int cols, int ld) {
  const int upr = cols >> 3;
  for (int i = threadIdx.x; i < rows * upr; i += blockDim.x) {
    int r = i / upr, u = i - r * upr;
    cp_async16(smem_u32(tile) + sw128_offset(rows, r, u), g + (size_t)r * ld + u * 8, true);
  }
}

__global__ void __launch_bounds__(128) umma_selftest_kernel(int mode, const __nv_bfloat16* A, const __nv_bfloat16* B,
                                                            float* D, int N, int K, unsigned* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;

  // Tile geometry per mode (rows x cols of the row-major global matrices).
  const int a_rows = (mode == 2) ? K : 128, a_cols = (mode == 2) ? 128 : K;
  const int b_rows = (mode == 0) ? N : K, b_cols = (mode == 0) ? K : N;
  uint8_t* tA = smem;
  uint8_t* tB = smem + (size_t)a_rows * a_cols * 2;

  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  uint32_t ncols = 32;
  while (ncols < (uint32_t)N + (mode == 3 ? 128u : 0u)) ncols <<= 1;
  const uint32_t a_col0 = (uint32_t)N;  // mode 3: the A operand sits after the accumulator columns
  if (warp == 0) tmem_alloc(&tmem_slot, ncols);
  if (mode != 3) load_tile_sw128(tA, A, a_rows, a_cols, a_cols);
  load_tile_sw128(tB, B, b_rows, b_cols, b_cols);
  cp_async_commit();
  cp_async_wait<0>();
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (mode == 3) {  // every thread writes its row of A into tensor memory, 64 elements per store
    for (int c0 = 0; c0 < K; c0 += 64) {
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        r[j] = (c0 + 2 * j < K) ? *reinterpret_cast<const uint32_t*>(A + (size_t)threadIdx.x * K + c0 + 2 * j) : 0u;
      tmem_st32(tmem + (uint32_t(warp * 32) << 16) + a_col0 + c0 / 2, r);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
  }

  if (threadIdx.x == 0 && mode == 3) {
    const uint32_t idesc = umma_idesc_bf16(128, N, 0u, 1u);
    for (int k0 = 0; k0 < K; k0 += 16)
      umma_ts(tmem, tmem + a_col0 + k0 / 2, umma_desc_mnmajor(smem_u32(tB), b_rows, k0, 0), idesc, k0 > 0);
    umma_commit(&bar);
  } else if (threadIdx.x == 0) {
    const uint32_t idesc = umma_idesc_bf16(128, N, mode == 2 ? 1u : 0u, mode == 0 ? 0u : 1u);
    for (int k0 = 0; k0 < K; k0 += 16) {
      uint64_t ad = (mode == 2) ? umma_desc_mnmajor(smem_u32(tA), a_rows, k0, 0) : umma_desc_kmajor(smem_u32(tA), a_rows, k0);
      uint64_t bd = (mode == 0) ? umma_desc_kmajor(smem_u32(tB), b_rows, k0) : umma_desc_mnmajor(smem_u32(tB), b_rows, k0, 0);
      umma_ss(tmem, ad, bd, idesc, k0 > 0);
    }
    umma_commit(&bar);
  }
  bool ok = mbar_wait(&bar, 0, status);
  tc_fence_after_sync();
  if (ok) {
    const int row = threadIdx.x;
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + (uint32_t(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < N) D[(size_t)row * N + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, ncols);
}

// The way every kernel here gives up on a barrier: one thread waits, with the given limit, for a phase of an
// mbarrier that nothing will ever complete.  The wait must run out, set the time-out bit of the status word and let
// the kernel return normally, leaving the context usable.
__global__ void wait_selftest_kernel(long long limit_clocks, unsigned* status, int* returned) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_for(&bar, 0, status, limit_clocks);
  __syncthreads();
  if (threadIdx.x == 0 && returned) *returned = ok ? 1 : 2;
}

}  // namespace moba

extern "C" int moba_selftest_wait(long long limit_clocks, unsigned* status, int* returned, void* stream) {
  if (limit_clocks < 1 || limit_clocks > moba::kWaitLimitClocks || !status) return MOBA_ERR_INVALID;
  moba::wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_clocks, status, returned);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_selftest_umma(int mode, const void* a, const void* b, float* d, int n, int k, unsigned* status,
                                  void* stream) {
  if (mode < 0 || mode > 3 || n < 16 || n > 256 || (n % 16) || k < 16 || k > 256 || (k % 16)) return MOBA_ERR_INVALID;
  if (mode != 2 && (k % 64)) return MOBA_ERR_INVALID;
  if (mode == 3 && n > 128) return MOBA_ERR_INVALID;
  if (mode != 0 && (n % 64)) return MOBA_ERR_INVALID;
  size_t bytes = (size_t)128 * k * 2 + (size_t)n * k * 2 + 1024;
  cudaError_t e = cudaFuncSetAttribute(moba::umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  moba::umma_selftest_kernel<<<1, 128, bytes, (cudaStream_t)stream>>>(
      mode, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, d, n, k, status);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
