// Layer glue of the full-model decode step: the few elementwise operations between the GEMMs and the attention
// of a Qwen2-architecture layer, each as one launch, so that a decode step is about a dozen launches per layer
// instead of about fifty.  No counterpart in the reference, which leaves these to the Hugging Face modules
// (examples/full_qwen2.py:76-90, 160-190 of the reference call q_proj/k_proj/v_proj, apply_rotary_pos_emb,
// the RMSNorm modules and the MLP module one after the other).  Arithmetic follows those modules step by
// step, rounding to bf16 where they do, so the fused path gives the same bits.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moba_b200.h"

namespace moba {
namespace {

__device__ __forceinline__ float bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// h_out = h_in + delta (bf16 add, skipped when delta is null); y = weight * bf16(h_out * rsqrt(mean(h_out^2) + eps)).
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ h_in, const __nv_bfloat16* __restrict__ delta,
                                                          const __nv_bfloat16* __restrict__ weight, float eps, int hidden,
                                                          __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ y) {
  __shared__ float s_part[8];
  const long long row = blockIdx.x;
  const __nv_bfloat16* hi = h_in + row * hidden;
  const __nv_bfloat16* dl = delta ? delta + row * hidden : nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += 256) {
    float v = __bfloat162float(hi[i]);
    if (dl) v = bf(v + __bfloat162float(dl[i]));
    if (h_out) h_out[row * hidden + i] = __float2bfloat16_rn(v);
    sum = fmaf(v, v, sum);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += s_part[i];
  const float r = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += 256) {
    float v = __bfloat162float(hi[i]);
    if (dl) v = bf(v + __bfloat162float(dl[i]));
    y[row * hidden + i] = __float2bfloat16_rn(__bfloat162float(weight[i]) * bf(v * r));
  }
}

// qkv [rows, (hq + 2 hk) * dim] -> q [rows, hq, dim], k [rows, hk, dim] with rotate-half rotary embedding, v copied.
__global__ void __launch_bounds__(256) rope_split_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cosv,
                                                         const __nv_bfloat16* __restrict__ sinv, int hq, int hk, int dim,
                                                         __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                                         __nv_bfloat16* __restrict__ v) {
  const long long row = blockIdx.x;
  const int heads = hq + 2 * hk, half = dim >> 1;
  const __nv_bfloat16* src = qkv + row * heads * dim;
  for (int i = threadIdx.x; i < heads * dim; i += 256) {
    const int h = i / dim, d = i - h * dim;
    const float x = __bfloat162float(src[i]);
    if (h >= hq + hk) { v[(row * hk + (h - hq - hk)) * dim + d] = src[i]; continue; }
    const float other = __bfloat162float(src[h * dim + (d < half ? d + half : d - half)]);
    const float rot = d < half ? -other : other;
    const float c = __bfloat162float(cosv[row * dim + d]), s = __bfloat162float(sinv[row * dim + d]);
    const __nv_bfloat16 out = __float2bfloat16_rn(bf(x * c) + bf(rot * s));
    if (h < hq) q[(row * hq + h) * dim + d] = out;
    else k[(row * hk + (h - hq)) * dim + d] = out;
  }
}

// gu [rows, 2 * ffn] (gate then up) -> out [rows, ffn] = bf16(silu(gate)) * up
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, int ffn, __nv_bfloat16* __restrict__ out) {
  const long long row = blockIdx.y;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= ffn) return;
  const float g = __bfloat162float(gu[row * 2 * ffn + i]), u = __bfloat162float(gu[row * 2 * ffn + ffn + i]);
  out[row * ffn + i] = __float2bfloat16_rn(bf(g / (1.f + expf(-g))) * u);
}

}  // namespace
}  // namespace moba

using namespace moba;

extern "C" int moba_add_rmsnorm(const void* h_in, const void* delta, const void* weight, float eps, long long rows, int hidden,
                                void* h_out, void* y, void* stream) {
  if (!h_in || !weight || !y || rows < 1 || hidden < 1) return MOBA_ERR_INVALID;
  add_rmsnorm_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(h_in), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight), eps,
      hidden, static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(y));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_rope_split(const void* qkv, const void* cosv, const void* sinv, long long rows, int hq, int hk, int dim, void* q,
                               void* k, void* v, void* stream) {
  if (!qkv || !cosv || !sinv || !q || !k || !v || rows < 1 || hq < 1 || hk < 1 || dim < 2 || (dim & 1)) return MOBA_ERR_INVALID;
  rope_split_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(cosv), static_cast<const __nv_bfloat16*>(sinv), hq, hk,
      dim, static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_silu_mul(const void* gate_up, long long rows, int ffn, void* out, void* stream) {
  if (!gate_up || !out || rows < 1 || ffn < 1) return MOBA_ERR_INVALID;
  silu_mul_kernel<<<dim3((unsigned)((ffn + 255) / 256), (unsigned)rows), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ffn, static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
