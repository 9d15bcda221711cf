// Shared by the two backward kernels: argument block and small device helpers.
#pragma once
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t bwd_pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
struct BwdArgs {
  PrefillView pv;
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* dout;  // [T,Hq,D] contiguous
  const float* lse;           // [T,Hq] natural log
  const float* delta;         // [T,Hq] rowsum(dO * O)
  const int* rowlist;
  const int* seg_base;
  const int* kv_order;  // [num_qtiles] key blocks by decreasing expected work
  const int* tile_base; // [n_chunks*Hkv + 1] 128-row tiles of all experts before expert e
  // Packed query tiles (warp-specialised kernel only), see bwd_pack_kernel
  const __nv_bfloat16* qpack;   // [tiles][128 x 64] swizzled shared-memory images of Q rows (from the forward)
  const __nv_bfloat16* kpack;   // [key blocks * Hkv] images of the K and V key blocks (from the forward)
  const __nv_bfloat16* vpack;
  const __nv_bfloat16* dopack;  // images of the dO rows, tile for tile like qpack
  const int* rowpack;           // [tiles][128] t*Hq+h, -1 = padding row
  const float* lsepack;         // [tiles][128] LSE * log2(e), +inf for padding rows
  const float* deltapack;       // [tiles][128] delta / sqrt(D)
  float* dq_acc;        // [T,Hq,D] fp32, zero-initialised (ordinary mode)
  unsigned long long* dq_fixed;  // [T,Hq,D] 64-bit fixed point, zero-initialised (deterministic mode), else null
  __nv_bfloat16* dk;    // [T,Hkv,D] contiguous
  __nv_bfloat16* dv;
  unsigned* status;
  float scale_log2, scale;
};

// Warp-specialised backward for head_dim <= 64 (prefill_attn_bwd_ws.cu).
// ---- small helpers shared by the warp-specialised kernels
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, unsigned* status, bool alive) {
  // every lane polls for itself: a barrier that has already completed costs one shared-memory round trip
  // instead of a poll, a warp barrier and a shuffle
  return alive ? mbar_wait(bar, parity, status) : true;
}
// One arrival per warp: every lane's earlier writes are ordered before it by __syncwarp.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool bwd_elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

cudaError_t launch_bwd_ws128(const BwdArgs& a, cudaStream_t st);  // 64 < head_dim <= 128
cudaError_t launch_bwd_ws(const BwdArgs& a, cudaStream_t st);
// Packs dO, LSE and delta of every query tile (rows as listed in a.rowpack).
cudaError_t launch_bwd_pack(const BwdArgs& a, long long tiles, void* dopack, float* lsepack, float* deltapack, cudaStream_t st);

}  // namespace moba
