// Prefill attention backward on tcgen05 tensor cores: exact gradients of the merged (global
// softmax) output with the route held fixed, as OptMixedAttention.backward of the reference
// (src/moba_opt/mixed_attention.py:141-225) obtains from two FlashAttention backward calls on the
// global O and LSE.
//
// KV-stationary: one CTA owns a block of 128 keys of one (chunk, kv head) and walks over every
// 128-row query tile that attends it - the causal tiles of the own chunk for each query head of
// the group, then the gathered rows of the expert list.  dK and dV of the block accumulate in
// tensor memory across the walk and are written once (no cross-CTA reduction); dQ of every tile
// is reduced into an FP32 buffer with vector atomics and converted to bf16 at the end.
//
// Per query tile:  S = Q K^T, dP = dO V^T (TMEM)  ->  P = exp2(S*c - LSE), dS = P (dP - delta) / sqrt(D)
// (registers, written as bf16 tiles)  ->  dV += P^T dO, dK += dS^T Q, dQ = dS K.
// The same swizzled shared-memory image of a tile serves as K-major and as MN-major operand, so
// no transposes are materialised.
#include "prefill_bwd.cuh"

namespace moba {

// delta[row] = sum_d dO[row,d] * O[row,d].  LPR lanes share a (token, head) row, 16 bytes of it each, so
// every lane of a warp has work at any head dimension (LPR = 4, 8, 16 or 32: smallest power of two >= D/8).
template <int LPR>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                                        const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                                        long long rows, int D) {
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
      s = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), s);
      s = fmaf(__uint_as_float(aw[i] & 0xFFFF0000u), __uint_as_float(bw[i] & 0xFFFF0000u), s);
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  if (sub == 0 && row < rows) delta[row] = s;
}

__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                             long long n8) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(acc)[2 * i], b = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  reinterpret_cast<uint4*>(dq)[i] =
      make_uint4(bwd_pack_bf16(a.x, a.y), bwd_pack_bf16(a.z, a.w), bwd_pack_bf16(b.x, b.y), bwd_pack_bf16(b.z, b.w));
}

template <int DPAD>
__global__ void __launch_bounds__(128, 1) attn_bwd_kernel(BwdArgs a) {
  constexpr int UPR = DPAD / 8;
  constexpr int TILE_BYTES = kTile * DPAD * 2;
  constexpr int PT_BYTES = kTile * kTile * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + DPAD, COL_DQ = 0;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t& bar1 = *reinterpret_cast<uint64_t*>(smem);
  uint64_t& bar2 = *reinterpret_cast<uint64_t*>(smem + 8);
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(smem + 16);
  int* s_rowth = reinterpret_cast<int*>(smem + 64);
  uint8_t* sK = smem + 1024;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sP = sdO + TILE_BYTES;
  uint8_t* sdS = sP + PT_BYTES;

  const PrefillView& pv = a.pv;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = pv.D;
  const int kblock = a.kv_order[blockIdx.x];
  const int g = blockIdx.y;
  const int c = pv.qtile_chunk[kblock];
  const int k0 = pv.qtile_tok0[kblock];
  const int chunk_begin = pv.chunk_start[c], chunk_end = pv.chunk_start[c + 1];
  const int nkeys = min(kTile, chunk_end - k0);
  const int kb = (k0 - chunk_begin) / kTile;
  const int tiles_in_chunk = (chunk_end - chunk_begin + kTile - 1) / kTile;
  const int n_self = tiles_in_chunk - kb;
  int remote_begin = 0, remote_rows = 0;
  if (pv.R > 0) {
    remote_begin = a.seg_base[c * pv.Hq + g * pv.G];
    remote_rows = a.seg_base[c * pv.Hq + (g + 1) * pv.G] - remote_begin;
  }
  const int n_remote = (remote_rows + kTile - 1) / kTile;
  const int n_iter = pv.G * n_self + n_remote;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (tid == 0) atomicOr(a.status, kErrBadIndex);
    return;
  }
  if (tid == 0) {
    mbar_init(&bar1, 1);
    mbar_init(&bar2, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, TMEM_COLS);

  // stationary K and V tiles of the key block
  {
    const __nv_bfloat16* kbase = a.k + (long long)g * pv.k_sh;
    const __nv_bfloat16* vbase = a.v + (long long)g * pv.v_sh;
    for (int i = tid; i < kTile * UPR; i += 128) {
      const int r = i / UPR, u = i - r * UPR;
      const bool ok = r < nkeys && u * 8 < D;
      cp_async16(smem_u32(sK) + sw128_offset(kTile, r, u), ok ? kbase + (long long)(k0 + r) * pv.k_st + u * 8 : kbase, ok);
      cp_async16(smem_u32(sV) + sw128_offset(kTile, r, u), ok ? vbase + (long long)(k0 + r) * pv.v_st + u * 8 : vbase, ok);
    }
    cp_async_commit();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tlane = tmem + (uint32_t(warp * 32) << 16);
  const uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
  const uint32_t idesc_kv = umma_idesc_bf16(128, DPAD, 1, 1);
  const uint32_t idesc_dq = umma_idesc_bf16(128, DPAD, 0, 1);
  uint32_t phase = 0;
  bool alive = true;

  for (int it = 0; it < n_iter; ++it) {
    // ---- rows of this query tile
    int th = -1;        // t*Hq+h of this thread's row
    bool diag = false;  // causal mask inside the tile
    if (it < pv.G * n_self) {
      const int hl = it / n_self, i = kb + (it - hl * n_self);
      const int tok = chunk_begin + i * kTile + tid;
      if (tok < chunk_end) th = tok * pv.Hq + g * pv.G + hl;
      diag = i == kb;
    } else {
      const int idx = (it - pv.G * n_self) * kTile + tid;
      if (idx < remote_rows) {
        th = a.rowlist[remote_begin + idx] / pv.R;
        if (th < 0 || th >= pv.T * pv.Hq) { atomicOr(a.status, kErrBadIndex); th = -1; }
      }
    }
    s_rowth[tid] = th;
    float lse2 = INFINITY, delta = 0.f;
    if (th >= 0) {
      lse2 = a.lse[th] * 1.4426950408889634f;
      delta = a.delta[th];
    }
    __syncthreads();  // row ids visible; previous tile's MMAs were awaited by every thread
    for (int i = tid; i < kTile * UPR; i += 128) {
      const int r = i / UPR, u = i - r * UPR;
      const int rth = s_rowth[r];
      const bool ok = rth >= 0 && u * 8 < D;
      const int t = rth / pv.Hq, h = rth - t * pv.Hq;
      cp_async16(smem_u32(sQ) + sw128_offset(kTile, r, u),
                 ok ? a.q + (long long)t * pv.q_st + (long long)h * pv.q_sh + u * 8 : a.q, ok);
      cp_async16(smem_u32(sdO) + sw128_offset(kTile, r, u), ok ? a.dout + (long long)rth * D + u * 8 : a.dout, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < DPAD; kk += 16)
        umma_ss(tmem + COL_S, umma_desc_kmajor(smem_u32(sQ), kTile, kk), umma_desc_kmajor(smem_u32(sK), kTile, kk), idesc_qk, kk > 0);
#pragma unroll
      for (int kk = 0; kk < DPAD; kk += 16)
        umma_ss(tmem + COL_DP, umma_desc_kmajor(smem_u32(sdO), kTile, kk), umma_desc_kmajor(smem_u32(sV), kTile, kk), idesc_qk, kk > 0);
      umma_commit(&bar1);
    }
    if (alive) alive = mbar_wait(&bar1, phase, a.status);
    tc_fence_after_sync();

    // ---- P and dS of this thread's row
    int klimit = nkeys;
    if (diag) klimit = min(klimit, tid + 1);
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) {
      uint32_t s[32], dp[32];
      tmem_ld32(tlane + COL_S + pc * 32, s);
      tmem_ld32(tlane + COL_DP + pc * 32, dp);
      tmem_ld_wait();
      uint32_t pp[16], ds[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = bwd_exp2(fmaf(__uint_as_float(s[i]), a.scale_log2, -lse2));
        float p1 = bwd_exp2(fmaf(__uint_as_float(s[i + 1]), a.scale_log2, -lse2));
        if (pc * 32 + i >= klimit) p0 = 0.f;
        if (pc * 32 + i + 1 >= klimit) p1 = 0.f;
        const float d0 = p0 * (__uint_as_float(dp[i]) - delta) * a.scale;
        const float d1 = p1 * (__uint_as_float(dp[i + 1]) - delta) * a.scale;
        pp[i >> 1] = bwd_pack_bf16(p0, p1);
        ds[i >> 1] = bwd_pack_bf16(d0, d1);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        *reinterpret_cast<uint4*>(sP + sw128_offset(kTile, tid, pc * 4 + u)) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
        *reinterpret_cast<uint4*>(sdS + sw128_offset(kTile, tid, pc * 4 + u)) = make_uint4(ds[4 * u], ds[4 * u + 1], ds[4 * u + 2], ds[4 * u + 3]);
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < kTile; kk += 16)  // dV += P^T dO  (contraction over the tile's query rows)
        umma_ss(tmem + COL_DV, umma_desc_mnmajor(smem_u32(sP), kTile, kk, 0), umma_desc_mnmajor(smem_u32(sdO), kTile, kk, 0),
                idesc_kv, (it > 0) || (kk > 0));
#pragma unroll
      for (int kk = 0; kk < kTile; kk += 16)  // dK += dS^T Q
        umma_ss(tmem + COL_DK, umma_desc_mnmajor(smem_u32(sdS), kTile, kk, 0), umma_desc_mnmajor(smem_u32(sQ), kTile, kk, 0),
                idesc_kv, (it > 0) || (kk > 0));
#pragma unroll
      for (int kk = 0; kk < kTile; kk += 16)  // dQ = dS K  (contraction over the block's keys)
        umma_ss(tmem + COL_DQ, umma_desc_kmajor(smem_u32(sdS), kTile, kk), umma_desc_mnmajor(smem_u32(sK), kTile, kk, 0),
                idesc_dq, kk > 0);
      umma_commit(&bar2);
    }
    if (alive) alive = mbar_wait(&bar2, phase, a.status);
    tc_fence_after_sync();
    phase ^= 1;
    {
      // every thread issues the warp-wide TMEM loads; padding rows drop their dQ row
      const bool ok = th >= 0 && alive;
      float* dst = a.dq_acc + (long long)(ok ? th : 0) * D;
#pragma unroll
      for (int pc = 0; pc < DPAD / 32; ++pc) {
        uint32_t r[32];
        tmem_ld32(tlane + COL_DQ + pc * 32, r);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            if (pc * 32 + i < D)
              red_add_v4(dst + pc * 32 + i, __uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                         __uint_as_float(r[i + 3]));
        }
      }
    }
    tc_fence_before_sync();
  }

  // ---- dK, dV of the key block: thread = key row
  __syncthreads();
  tc_fence_after_sync();
  {
    const bool ok = tid < nkeys && alive;
    __nv_bfloat16* dkrow = a.dk + ((long long)(k0 + tid) * pv.Hkv + g) * D;
    __nv_bfloat16* dvrow = a.dv + ((long long)(k0 + tid) * pv.Hkv + g) * D;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
#pragma unroll
      for (int pc = 0; pc < DPAD / 32; ++pc) {
        uint32_t r[32];
        tmem_ld32(tlane + (which == 0 ? COL_DK : COL_DV) + pc * 32, r);
        tmem_ld_wait();
        if (ok) {
          __nv_bfloat16* dst = which == 0 ? dkrow : dvrow;
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            if (pc * 32 + i < D)
              *reinterpret_cast<uint4*>(dst + pc * 32 + i) =
                  make_uint4(bwd_pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                             bwd_pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                             bwd_pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                             bwd_pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, TMEM_COLS);
}

template <int DPAD>
static cudaError_t launch_bwd(const BwdArgs& a, cudaStream_t st) {
  const size_t smem = 1024 + (size_t)kTile * DPAD * 2 * 4 + (size_t)kTile * kTile * 2 * 2;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<DPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  attn_bwd_kernel<DPAD><<<dim3(a.pv.n_qtiles, a.pv.Hkv), 128, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace moba

using namespace moba;


extern "C" size_t moba_prefill_bwd_scratch_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  const size_t rows = (size_t)d->total_tokens * d->hq;
  size_t bytes = align256(rows * 4) + align256(rows * d->dim * 4);
  if (d->dim <= 128 && !(d->flags & MOBA_BWD_SINGLE_WARPGROUP)) {
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
  if (cudaMemsetAsync(dq_acc, 0, (size_t)rows * d->dim * 4, st) != cudaSuccess) return MOBA_ERR_CUDA;
  {
    const __nv_bfloat16* o16 = static_cast<const __nv_bfloat16*>(out);
    const __nv_bfloat16* do16 = static_cast<const __nv_bfloat16*>(dout);
    const int units = d->dim / 8;
    if (units <= 4) bwd_delta_kernel<4><<<(unsigned)((rows + 63) / 64), 256, 0, st>>>(o16, do16, delta, rows, d->dim);
    else if (units <= 8) bwd_delta_kernel<8><<<(unsigned)((rows + 31) / 32), 256, 0, st>>>(o16, do16, delta, rows, d->dim);
    else if (units <= 16) bwd_delta_kernel<16><<<(unsigned)((rows + 15) / 16), 256, 0, st>>>(o16, do16, delta, rows, d->dim);
    else bwd_delta_kernel<32><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(o16, do16, delta, rows, d->dim);
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
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.status = status;
  a.scale = (float)(1.0 / sqrt((double)d->dim));
  a.scale_log2 = (float)(1.4426950408889634 / sqrt((double)d->dim));
  const bool ws = d->dim <= 128 && !(d->flags & MOBA_BWD_SINGLE_WARPGROUP);
  if (ws) {
    const size_t tiles = (size_t)pack_q_tiles(*d);
    char* p = reinterpret_cast<char*>(dq_acc) + align256((size_t)rows * d->dim * 4);
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
  cudaError_t e = ws ? (d->dim > 64 ? launch_bwd_ws128(a, st) : launch_bwd_ws(a, st))
                     : (d->dim > 64 ? launch_bwd<128>(a, st) : launch_bwd<64>(a, st));
  prof_end(kProfBwdMain, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  const long long n8 = rows * d->dim / 8;
  bwd_dq_convert_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), n8);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
