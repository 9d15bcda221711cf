// Prefill attention backward, host entry: exact gradients of the merged (global softmax) output with the route
// held fixed, as OptMixedAttention.backward of the reference (src/moba_opt/mixed_attention.py:141-225) obtains from
// two FlashAttention backward calls on the global O and LSE.
//
// Launch sequence: dq_acc = 0, delta = rowsum(dO * O), pack dO / LSE / delta per query tile, the KV-stationary main
// kernel (prefill_attn_bwd_ws.cu for head_dim <= 64, prefill_attn_bwd_ws128.cu above that: dK and dV of a key block
// accumulate in tensor memory and are written once, dQ of every tile is added into the FP32 buffer row by row with bulk
// reductions of the copy engine), dq = dq_acc rounded to the input format.  With MOBA_BWD_DETERMINISTIC the accumulator
// is 64-bit fixed point and the reductions are integer, which makes dQ bit-repeatable like everything else (the
// reference asks FlashAttention for the same: deterministic=True in both backward calls, mixed_attention.py:185,220).
#include "prefill_bwd.cuh"

namespace moba {

// delta[row] = sum_d dO[row,d] * O[row,d].  LPR lanes share a (token, head) row, 16 bytes of it each, so
// every lane of a warp has work at any head dimension (LPR = 4, 8, 16 or 32: smallest power of two >= D/8).
template <int LPR>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                                        const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                                        long long rows, int D, bool f16) {
  constexpr int RPW = 32 / LPR;  // rows per warp
  const int lane = threadIdx.x & 31, sub = lane % LPR;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + lane / LPR;
  float s = 0.f;
  if (row < rows && sub * 8 < D) {
    const uint4 a = *reinterpret_cast<const uint4*>(out + row * D + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + row * D + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack16(aw[i], f16), y = unpack16(bw[i], f16);
      s = fmaf(x.x, y.x, s);
      s = fmaf(x.y, y.y, s);
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  if (sub == 0 && row < rows) delta[row] = s;
}

__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                             long long n8, bool f16) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(acc)[2 * i], b = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  reinterpret_cast<uint4*>(dq)[i] =
      make_uint4(pack16(a.x, a.y, f16), pack16(a.z, a.w, f16), pack16(b.x, b.y, f16), pack16(b.z, b.w, f16));
}

__global__ void __launch_bounds__(256) bwd_dq_convert_fixed_kernel(const long long* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                                   long long n8, bool f16) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float f[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const longlong2 w = reinterpret_cast<const longlong2*>(acc)[4 * i + j];
    f[2 * j] = (float)((double)w.x * (1.0 / 4294967296.0));
    f[2 * j + 1] = (float)((double)w.y * (1.0 / 4294967296.0));
  }
  reinterpret_cast<uint4*>(dq)[i] =
      make_uint4(pack16(f[0], f[1], f16), pack16(f[2], f[3], f16), pack16(f[4], f[5], f16), pack16(f[6], f[7], f16));
}

}  // namespace moba

using namespace moba;


extern "C" size_t moba_prefill_bwd_scratch_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  const size_t rows = (size_t)d->total_tokens * d->hq;
  size_t bytes = align256(rows * 4) + align256(rows * d->dim * ((d->flags & MOBA_BWD_DETERMINISTIC) ? 8 : 4));
  {
    const size_t tiles = (size_t)pack_q_tiles(*d);
    bytes += align256(tiles * kTile * pack_dpad(*d) * 2) + 2 * align256(tiles * kTile * 4);
  }
  return bytes;
}

extern "C" int moba_prefill_bwd(const moba_prefill_desc* d, const void* q, const void* k, const void* v, const void* out,
                                const float* lse, const void* dout, const void* route_state, void* scratch,
                                size_t scratch_bytes, void* dq, void* dk, void* dv, unsigned* status, void* stream) {
  int rc = validate_desc(d);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !out || !lse || !dout || !scratch || !dq || !dk || !dv || !status || !d->kv_order ||
      !route_state)
    return MOBA_ERR_INVALID;
  if (d->dim > 128) return MOBA_ERR_UNSUPPORTED;
  if (scratch_bytes < moba_prefill_bwd_scratch_bytes(d)) return MOBA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const long long rows = (long long)d->total_tokens * d->hq;
  float* delta = static_cast<float*>(scratch);
  float* dq_acc = reinterpret_cast<float*>(static_cast<char*>(scratch) + align256((size_t)rows * 4));
  const bool fixed = (d->flags & MOBA_BWD_DETERMINISTIC) != 0;
  const size_t acc_bytes = (size_t)rows * d->dim * (fixed ? 8 : 4);
  if (cudaMemsetAsync(dq_acc, 0, acc_bytes, st) != cudaSuccess) return MOBA_ERR_CUDA;
  {
    const __nv_bfloat16* o16 = static_cast<const __nv_bfloat16*>(out);
    const __nv_bfloat16* do16 = static_cast<const __nv_bfloat16*>(dout);
    const int units = d->dim / 8;
    const bool f16 = (d->flags & MOBA_INPUT_FP16) != 0;
    if (units <= 4) bwd_delta_kernel<4><<<(unsigned)((rows + 63) / 64), 256, 0, st>>>(o16, do16, delta, rows, d->dim, f16);
    else if (units <= 8) bwd_delta_kernel<8><<<(unsigned)((rows + 31) / 32), 256, 0, st>>>(o16, do16, delta, rows, d->dim, f16);
    else if (units <= 16) bwd_delta_kernel<16><<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(o16, do16, delta, rows, d->dim, f16);
    else bwd_delta_kernel<32><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(o16, do16, delta, rows, d->dim, f16);
  }
  BwdArgs a;
  a.pv = make_view(*d);
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.dout = static_cast<const __nv_bfloat16*>(dout);
  a.lse = lse;
  a.delta = delta;
  a.rowlist = a.seg_base = nullptr;
  if (d->remote_k > 0) {
    RouteState rs = carve_route_state(*d, const_cast<void*>(route_state));
    a.rowlist = rs.rowlist;
    a.seg_base = rs.seg_base;
  }
  a.kv_order = d->kv_order;
  a.tile_base = nullptr;
  if (d->remote_k > 0) a.tile_base = carve_route_state(*d, const_cast<void*>(route_state)).tile_base;
  a.qpack = a.dopack = a.kpack = a.vpack = nullptr;
  a.rowpack = nullptr;
  a.lsepack = a.deltapack = nullptr;
  a.dq_acc = dq_acc;
  a.dq_fixed = fixed ? reinterpret_cast<unsigned long long*>(dq_acc) : nullptr;
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.status = status;
  a.scale = (float)(1.0 / sqrt((double)d->dim));
  a.scale_log2 = (float)(1.4426950408889634 / sqrt((double)d->dim));
  {
    const size_t tiles = (size_t)pack_q_tiles(*d);
    char* p = reinterpret_cast<char*>(dq_acc) + align256(acc_bytes);
    void* dopack = p; p += align256(tiles * kTile * pack_dpad(*d) * 2);
    float* lsepack = reinterpret_cast<float*>(p); p += align256(tiles * kTile * 4);
    float* deltapack = reinterpret_cast<float*>(p);
    const PackState ps = carve_pack_state(*d, const_cast<void*>(route_state));
    a.qpack = ps.qpack; a.kpack = ps.kpack; a.vpack = ps.vpack; a.rowpack = ps.rowpack;
    const long long used = d->remote_k > 0 ? (long long)tiles : (long long)d->num_qtiles * d->hq;
    if (launch_bwd_pack(a, used, dopack, lsepack, deltapack, st) != cudaSuccess) return MOBA_ERR_CUDA;
    a.dopack = static_cast<const __nv_bfloat16*>(dopack);
    a.lsepack = lsepack; a.deltapack = deltapack;
  }
  prof_begin(kProfBwdMain, st);
  cudaError_t e = d->dim > 64 ? launch_bwd_ws128(a, st) : launch_bwd_ws(a, st);
  prof_end(kProfBwdMain, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  const long long n8 = rows * d->dim / 8;
  if (fixed)
    bwd_dq_convert_fixed_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const long long*>(dq_acc),
                                                                           static_cast<__nv_bfloat16*>(dq), n8, a.pv.fp16 != 0);
  else
    bwd_dq_convert_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), n8, a.pv.fp16 != 0);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
