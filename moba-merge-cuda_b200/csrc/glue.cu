// Layer glue of the full-model decode step: the few elementwise operations between the GEMMs and the attention
// of a Qwen2-architecture layer, each as one launch, so that a decode step is about a dozen launches per layer
// instead of about fifty.  No counterpart in the reference, which leaves these to the Hugging Face modules
// (examples/full_qwen2.py:76-90, 160-190 of the reference call q_proj/k_proj/v_proj, apply_rotary_pos_emb,
// the RMSNorm modules and the MLP module one after the other).  Arithmetic follows those modules step by
// step, rounding to bf16 where they do, so the fused path gives the same bits.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"
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


// ---- the same three operations over many rows (a prefill), eight elements per thread -----------------------------
__device__ __forceinline__ void unpack8(const uint4& r, float (&f)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp per row, the row kept in registers between the sum of squares and the scaling (hidden <= 8 * 32 * 8).
__global__ void __launch_bounds__(256) add_rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ h_in, const __nv_bfloat16* __restrict__ delta,
                                                               const __nv_bfloat16* __restrict__ weight, float eps, long long rows,
                                                               int hidden, __nv_bfloat16* __restrict__ h_out,
                                                               __nv_bfloat16* __restrict__ y) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31, chunks = hidden >> 3;
  float v[8][8];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = lane + j * 32;
    if (c < chunks) {
      unpack8(*reinterpret_cast<const uint4*>(h_in + row * hidden + c * 8), v[j]);
      if (delta) {
        float d[8];
        unpack8(*reinterpret_cast<const uint4*>(delta + row * hidden + c * 8), d);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] = bf(v[j][i] + d[i]);
      }
      if (h_out) *reinterpret_cast<uint4*>(h_out + row * hidden + c * 8) = pack8(v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum = fmaf(v[j][i], v[j][i], sum);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  const float r = rsqrtf(sum / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = lane + j * 32;
    if (c < chunks) {
      float w[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(weight + c * 8), w);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = w[i] * bf(v[j][i] * r);
      *reinterpret_cast<uint4*>(y + row * hidden + c * 8) = pack8(o);
    }
  }
}

// One thread per 8 consecutive dimensions of a head; the rotation partner is the chunk half a head away.
__global__ void __launch_bounds__(256) rope_split_rows_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cosv,
                                                              const __nv_bfloat16* __restrict__ sinv, long long rows, int hq, int hk,
                                                              int dim, __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                                              __nv_bfloat16* __restrict__ v) {
  const int cpd = dim >> 3, heads = hq + 2 * hk;
  const long long item = (long long)blockIdx.x * 256 + threadIdx.x;
  if (item >= rows * heads * cpd) return;
  const int c = (int)(item % cpd);
  const int h = (int)((item / cpd) % heads);
  const long long row = item / ((long long)cpd * heads);
  const __nv_bfloat16* src = qkv + (row * heads + h) * dim;
  const uint4 own = *reinterpret_cast<const uint4*>(src + c * 8);
  if (h >= hq + hk) {
    *reinterpret_cast<uint4*>(v + (row * hk + (h - hq - hk)) * dim + c * 8) = own;
    return;
  }
  const bool low = c < (cpd >> 1);
  float x[8], other[8], cs[8], sn[8], o[8];
  unpack8(own, x);
  unpack8(*reinterpret_cast<const uint4*>(src + (low ? c + (cpd >> 1) : c - (cpd >> 1)) * 8), other);
  unpack8(*reinterpret_cast<const uint4*>(cosv + row * dim + c * 8), cs);
  unpack8(*reinterpret_cast<const uint4*>(sinv + row * dim + c * 8), sn);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = bf(x[i] * cs[i]) + bf((low ? -other[i] : other[i]) * sn[i]);
  __nv_bfloat16* dst = h < hq ? q + (row * hq + h) * dim : k + (row * hk + (h - hq)) * dim;
  *reinterpret_cast<uint4*>(dst + c * 8) = pack8(o);
}

__global__ void __launch_bounds__(256) silu_mul_rows_kernel(const __nv_bfloat16* __restrict__ gu, long long rows, int ffn,
                                                            __nv_bfloat16* __restrict__ out) {
  const int cpr = ffn >> 3;
  const long long item = (long long)blockIdx.x * 256 + threadIdx.x;
  if (item >= rows * cpr) return;
  const long long row = item / cpr;
  const int c = (int)(item - row * cpr);
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * ffn + c * 8), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * ffn + ffn + c * 8), u);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = bf(g[i] / (1.f + expf(-g[i]))) * u[i];
  *reinterpret_cast<uint4*>(out + row * ffn + c * 8) = pack8(o);
}

// ---- batch-1 linear layers of the decode step -----------------------------------------------------------------
// y = W x (+ bias) for one token: W [N, K] bf16 row-major is read once from HBM, which is all the step costs, so
// the kernel is built to have every byte of its rows in flight at once: a group of 32..256 threads owns one output
// (or one gate/up pair), each thread issues all of its 16-byte weight loads before anything else, and only then
// the CTA prepares x in shared memory - either a plain copy, or the residual add + RMSNorm that precedes the
// projection in the layer (recomputed by every CTA: 2 KB of input, cheaper than a launch of its own; CTA 0 writes
// the new residual).  FP32 accumulation, one rounding to bf16 at the end as in a bf16 GEMM.
struct LinearArgs {
  const __nv_bfloat16 *x, *h_in, *delta, *norm_w, *W, *bias;
  __nv_bfloat16 *h_out, *y;
  float eps;
  int K, N;  // N outputs; with PAIR the weight has 2 N rows (gate rows, then up rows)
};

__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
  const uint32_t wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = fmaf(__uint_as_float(wv[i] << 16), __uint_as_float(xv[i] << 16), acc);
    acc = fmaf(__uint_as_float(wv[i] & 0xFFFF0000u), __uint_as_float(xv[i] & 0xFFFF0000u), acc);
  }
  return acc;
}

template <int TPR, bool PAIR>
__global__ void __launch_bounds__(256, 4) decode_linear_kernel(LinearArgs a) {
  constexpr int CH = PAIR ? 4 : 8;     // 16-byte loads per thread and weight row
  constexpr int GROUPS = 256 / TPR;    // outputs per CTA and pass
  extern __shared__ __align__(16) uint8_t s_raw[];
  __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(s_raw);
  __shared__ float s_part[8], s_red[2][8];
  const int tid = threadIdx.x, t = tid % TPR, group = tid / TPR;
  const int chunks = a.K >> 3;
  const int stride = gridDim.x * GROUPS;
  // When the outputs outnumber the groups that can be resident, a CTA makes several passes (the same number for
  // all of its groups) and x is prepared once.
  const int passes = (a.N - blockIdx.x * GROUPS + stride - 1) / stride;
  int out = blockIdx.x * GROUPS + group;
  uint4 w0[CH], w1[PAIR ? CH : 1];
  auto load_weights = [&]() {  // every weight byte of this thread in flight
    const bool live = out < a.N;
    const uint4* r0 = reinterpret_cast<const uint4*>(a.W + (long long)(live ? out : 0) * a.K);
    const uint4* r1 = reinterpret_cast<const uint4*>(a.W + ((long long)(live ? out : 0) + a.N) * a.K);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = t + i * TPR;
      w0[i] = live && c < chunks ? __ldcs(r0 + c) : make_uint4(0u, 0u, 0u, 0u);
      if (PAIR) w1[i] = live && c < chunks ? __ldcs(r1 + c) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_weights();
  // the norm weight is a constant too: the first 1024 entries travel with the projection's weights
  float nw[4] = {0.f, 0.f, 0.f, 0.f};
  if (a.h_in) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (tid + j * 256 < a.K) nw[j] = __bfloat162float(a.norm_w[tid + j * 256]);
  }
  // Programmatic dependent launch: the weights above do not depend on the kernel before this one, so this grid
  // may start while that one still runs (and lets its own successor do the same); everything below reads what the
  // predecessor wrote, or writes what it may still read, and waits for it to have completed.
  dependents_may_start();
  wait_for_predecessor();
  // x into shared memory while the weights are on their way
  if (a.h_in) {
    float sum = 0.f;
    for (int i = tid; i < a.K; i += 256) {
      float v = __bfloat162float(a.h_in[i]);
      if (a.delta) v = bf(v + __bfloat162float(a.delta[i]));
      const __nv_bfloat16 vb = __float2bfloat16_rn(v);
      s_x[i] = vb;
      if (a.h_out && blockIdx.x == 0) a.h_out[i] = vb;
      sum = fmaf(v, v, sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if ((tid & 31) == 0) s_part[tid >> 5] = sum;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += s_part[i];
    const float r = rsqrtf(total / (float)a.K + a.eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {         // the same thread wrote s_x[i]
      const int i = tid + j * 256;
      if (i < a.K) s_x[i] = __float2bfloat16_rn(nw[j] * bf(__bfloat162float(s_x[i]) * r));
    }
    for (int i = tid + 1024; i < a.K; i += 256)
      s_x[i] = __float2bfloat16_rn(__bfloat162float(a.norm_w[i]) * bf(__bfloat162float(s_x[i]) * r));
  } else {
    for (int c = tid; c < chunks; c += 256)
      reinterpret_cast<uint4*>(s_x)[c] = __ldcg(reinterpret_cast<const uint4*>(a.x) + c);  // not the read-only path: see above
  }
  __syncthreads();
  for (int pass = 0; pass < passes; ++pass) {
    if (pass) load_weights();
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = t + i * TPR;
      if (c < chunks) {
        const uint4 xv = reinterpret_cast<const uint4*>(s_x)[c];
        acc0 = dot8(w0[i], xv, acc0);
        if (PAIR) acc1 = dot8(w1[i], xv, acc1);
      }
    }
#pragma unroll
    for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1) {
      acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, o);
      if (PAIR) acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, o);
    }
    if (TPR > 32) {
      if (pass) __syncthreads();  // the previous pass's sums have been read
      if ((tid & 31) == 0) { s_red[0][tid >> 5] = acc0; s_red[1][tid >> 5] = acc1; }
      __syncthreads();
      if (t == 0) {
        acc0 = 0.f; acc1 = 0.f;
#pragma unroll
        for (int i = 0; i < TPR / 32; ++i) { acc0 += s_red[0][group * (TPR / 32) + i]; acc1 += s_red[1][group * (TPR / 32) + i]; }
      }
    }
    if (t == 0 && out < a.N) {
      if (PAIR) {
        const float g = bf(acc0), u = bf(acc1);
        a.y[out] = __float2bfloat16_rn(bf(g / (1.f + expf(-g))) * u);
      } else {
        a.y[out] = __float2bfloat16_rn(a.bias ? acc0 + __bfloat162float(a.bias[out]) : acc0);
      }
    }
    out += stride;
  }
}

// Inputs of a decode step in one launch: the embedding row of each token and the rotary table of its position,
// cos / sin [rows, dim] = cos / sin(position * inv_freq[d mod dim/2]) * scaling computed in FP32 and rounded to bf16 -
// the arithmetic of the Hugging Face rotary module (default rope type), which takes about ten small launches.
__global__ void __launch_bounds__(256) step_inputs_kernel(const long long* tokens, const __nv_bfloat16* __restrict__ embed, int hidden,
                                                          const int* positions, const float* __restrict__ inv_freq, float scaling,
                                                          int dim, __nv_bfloat16* h, __nv_bfloat16* cosv, __nv_bfloat16* sinv) {
  const long long row = blockIdx.x;
  const long long tok = tokens[row];
  const __nv_bfloat16* src = embed + tok * hidden;
  for (int i = threadIdx.x; i < hidden; i += 256) h[row * hidden + i] = src[i];
  const float pos = (float)positions[row];
  const int half = dim >> 1;
  for (int d = threadIdx.x; d < dim; d += 256) {
    const float f = inv_freq[d < half ? d : d - half] * pos;
    cosv[row * dim + d] = __float2bfloat16_rn(cosf(f) * scaling);
    sinv[row * dim + d] = __float2bfloat16_rn(sinf(f) * scaling);
  }
}

// ---- greedy token: arg-max over one row of bf16 logits, lowest index among equal maxima ---------------------------
// kArgmaxCtas CTAs scan slices with 16-byte loads and leave one candidate each; the CTA that finishes last (atomic
// ticket, nobody waits) picks among the candidates, writes the int64 index and clears the ticket for the next launch.
constexpr int kArgmaxCtas = 148;

__device__ __forceinline__ void argmax_pick(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void __launch_bounds__(256) argmax_kernel(const __nv_bfloat16* logits, int n, float* cand_v, int* cand_i, unsigned* ticket,
                                                     long long* out) {
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  __shared__ bool s_last;
  dependents_may_start();
  wait_for_predecessor();  // the logits
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  const int chunks = n >> 3;
  for (int c = blockIdx.x * 256 + tid; c < chunks; c += gridDim.x * 256) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(logits) + c);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      argmax_pick(bv, bi, __uint_as_float(w[j] << 16), c * 8 + 2 * j);
      argmax_pick(bv, bi, __uint_as_float(w[j] & 0xFFFF0000u), c * 8 + 2 * j + 1);
    }
  }
  if (blockIdx.x == 0)
    for (int i = (chunks << 3) + tid; i < n; i += 256) argmax_pick(bv, bi, __bfloat162float(logits[i]), i);
  auto reduce = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      argmax_pick(bv, bi, ov, oi);
    }
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < 8 ? s_v[lane] : -INFINITY;
      bi = lane < 8 ? s_i[lane] : 0x7FFFFFFF;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        argmax_pick(bv, bi, ov, oi);
      }
    }
  };
  reduce();
  if (tid == 0) {
    cand_v[blockIdx.x] = bv;
    cand_i[blockIdx.x] = bi;
    __threadfence();
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  bv = -INFINITY;
  bi = 0x7FFFFFFF;
  for (int c = tid; c < (int)gridDim.x; c += 256) argmax_pick(bv, bi, __ldcg(cand_v + c), __ldcg(cand_i + c));
  __syncthreads();  // s_v / s_i of the first reduction have been read
  reduce();
  if (tid == 0) {
    *out = bi == 0x7FFFFFFF ? 0 : bi;  // a row of NaN or -inf only: index 0
    *ticket = 0u;
  }
}

}  // namespace
}  // namespace moba

using namespace moba;

extern "C" int moba_add_rmsnorm(const void* h_in, const void* delta, const void* weight, float eps, long long rows, int hidden,
                                void* h_out, void* y, void* stream) {
  if (!h_in || !weight || !y || rows < 1 || hidden < 1) return MOBA_ERR_INVALID;
  const bool aligned = !(((uintptr_t)h_in | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)h_out | (uintptr_t)y) & 15);
  if (rows >= 64 && hidden % 8 == 0 && hidden <= 2048 && aligned) {  // many rows: a warp per row, 16-byte accesses
    add_rmsnorm_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(h_in), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
        eps, rows, hidden, static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(y));
    return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
  }
  add_rmsnorm_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(h_in), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight), eps,
      hidden, static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(y));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_rope_split(const void* qkv, const void* cosv, const void* sinv, long long rows, int hq, int hk, int dim, void* q,
                               void* k, void* v, void* stream) {
  if (!qkv || !cosv || !sinv || !q || !k || !v || rows < 1 || hq < 1 || hk < 1 || dim < 2 || (dim & 1)) return MOBA_ERR_INVALID;
  if (rows >= 64 && dim % 16 == 0 &&
      !(((uintptr_t)qkv | (uintptr_t)cosv | (uintptr_t)sinv | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15)) {
    const long long items = rows * (hq + 2 * hk) * (dim / 8);
    rope_split_rows_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(cosv), static_cast<const __nv_bfloat16*>(sinv), rows,
        hq, hk, dim, static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v));
    return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
  }
  rope_split_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(cosv), static_cast<const __nv_bfloat16*>(sinv), hq, hk,
      dim, static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_silu_mul(const void* gate_up, long long rows, int ffn, void* out, void* stream) {
  if (!gate_up || !out || rows < 1 || ffn < 1) return MOBA_ERR_INVALID;
  if (rows >= 64 && ffn % 8 == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15)) {
    const long long items = rows * (ffn / 8);
    silu_mul_rows_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(gate_up), rows, ffn, static_cast<__nv_bfloat16*>(out));
    return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
  }
  silu_mul_kernel<<<dim3((unsigned)((ffn + 255) / 256), (unsigned)rows), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ffn, static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_linear(const void* x, const void* h_in, const void* delta, const void* norm_weight, float eps, void* h_out,
                                  const void* weight, const void* bias, int k, int n, int epilogue, void* y, void* stream) {
  if (!weight || !y || k < 8 || (k & 7) || n < 1 || (epilogue != 0 && epilogue != 1)) return MOBA_ERR_INVALID;
  if ((h_in == nullptr) == (x == nullptr)) return MOBA_ERR_INVALID;  // exactly one source of the input vector
  if (h_in && !norm_weight) return MOBA_ERR_INVALID;
  if (!h_in && (delta || h_out)) return MOBA_ERR_INVALID;
  // every CTA re-reads h_in and delta while the first one writes h_out: in place would hand some CTAs updated rows
  if (h_out && (h_out == h_in || h_out == delta)) return MOBA_ERR_INVALID;
  if (epilogue == 1 && bias) return MOBA_ERR_INVALID;
  if (((uintptr_t)weight | (uintptr_t)(x ? x : weight)) & 15) return MOBA_ERR_INVALID;
  const bool pair = epilogue == 1;
  const int per_thread = (pair ? 4 : 8) * 8;  // elements of a row one thread can hold
  int tpr = 32;
  while (tpr < 256 && tpr * per_thread < k) tpr *= 2;
  if (tpr * per_thread < k) return MOBA_ERR_UNSUPPORTED;
  LinearArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x); a.h_in = static_cast<const __nv_bfloat16*>(h_in);
  a.delta = static_cast<const __nv_bfloat16*>(delta); a.norm_w = static_cast<const __nv_bfloat16*>(norm_weight);
  a.W = static_cast<const __nv_bfloat16*>(weight); a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.h_out = static_cast<__nv_bfloat16*>(h_out); a.y = static_cast<__nv_bfloat16*>(y);
  a.eps = eps; a.K = k; a.N = n;
  const size_t smem = (size_t)k * 2;
  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return MOBA_ERR_CUDA;
#define MOBA_LAUNCH_LINEAR_P(T, P)                                                                                  \
  do {                                                                                                              \
    int per_sm = 0;                                                                                                 \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_linear_kernel<T, P>, 256, smem) != cudaSuccess || per_sm < 1) \
      return MOBA_ERR_CUDA;                                                                                         \
    const long long units = (n + 256 / T - 1) / (256 / T), resident = (long long)per_sm * sms;                      \
    const long long passes = units > 4 * resident ? (units + resident - 1) / resident : 1; /* a short tail is cheaper */ \
    if (launch_dependent(1u, decode_linear_kernel<T, P>, dim3((unsigned)((units + passes - 1) / passes)), dim3(256), smem, st, \
                         a) != cudaSuccess)                                                                         \
      return MOBA_ERR_CUDA;                                                                                         \
  } while (0)
#define MOBA_LAUNCH_LINEAR(T)                                                                                       \
  do {                                                                                                              \
    if (pair) MOBA_LAUNCH_LINEAR_P(T, true);                                                                        \
    else MOBA_LAUNCH_LINEAR_P(T, false);                                                                            \
  } while (0)
  if (tpr == 32) MOBA_LAUNCH_LINEAR(32);
  else if (tpr == 64) MOBA_LAUNCH_LINEAR(64);
  else if (tpr == 128) MOBA_LAUNCH_LINEAR(128);
  else MOBA_LAUNCH_LINEAR(256);
#undef MOBA_LAUNCH_LINEAR_P
#undef MOBA_LAUNCH_LINEAR
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_step_inputs(const int64_t* tokens, const void* embedding, int hidden, const int32_t* positions,
                                       const float* inv_freq, float scaling, int dim, long long rows, void* h, void* cosv, void* sinv,
                                       void* stream) {
  if (!tokens || !embedding || !positions || !inv_freq || !h || !cosv || !sinv || hidden < 1 || dim < 2 || (dim & 1) || rows < 1)
    return MOBA_ERR_INVALID;
  step_inputs_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const long long*>(tokens), static_cast<const __nv_bfloat16*>(embedding), hidden, positions, inv_freq, scaling, dim,
      static_cast<__nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(cosv), static_cast<__nv_bfloat16*>(sinv));
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" size_t moba_argmax_workspace_bytes(void) { return 256 + (size_t)kArgmaxCtas * 8; }

extern "C" int moba_argmax_bf16(const void* logits, int n, void* workspace, size_t workspace_bytes, int64_t* out, void* stream) {
  if (!logits || !workspace || !out || n < 1) return MOBA_ERR_INVALID;
  if (workspace_bytes < moba_argmax_workspace_bytes()) return MOBA_ERR_WORKSPACE;
  if (((uintptr_t)logits & 15) || ((uintptr_t)workspace & 15)) return MOBA_ERR_INVALID;
  char* p = static_cast<char*>(workspace);
  unsigned* ticket = reinterpret_cast<unsigned*>(p);
  float* cand_v = reinterpret_cast<float*>(p + 256);
  int* cand_i = reinterpret_cast<int*>(p + 256 + kArgmaxCtas * 4);
  const int chunks = n >> 3;
  const int ctas = chunks >= 256 * kArgmaxCtas ? kArgmaxCtas : (chunks + 255) / 256 > 0 ? (chunks + 255) / 256 : 1;
  if (launch_dependent(16u, argmax_kernel, dim3(ctas), dim3(256), 0, (cudaStream_t)stream, static_cast<const __nv_bfloat16*>(logits), n,
                       cand_v, cand_i, ticket, reinterpret_cast<long long*>(out)) != cudaSuccess)
    return MOBA_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
