// Prefill attention forward on tcgen05 tensor cores with the LSE merge fused into the epilogue.
//
// Work decomposition (KV-stationary experts as in the reference, src/moba_opt/grouped_attention.py:76-90):
//   remote pass  one CTA per 128 gathered query rows of an expert (chunk, kv head): the rows of any
//                query head of the group that selected the chunk attend the whole chunk; the
//                normalised partial output (bf16) and its log2-sum-exp go to the fixed slot of the
//                (row, chunk) pair, so no atomics or tickets are needed and the merge order is fixed
//   self pass    one CTA per (128-token query tile, query head): causal attention inside the own
//                chunk, then the epilogue merges the row's remote partials with the global-softmax
//                rule of src/moba_opt/ops/merge.cu:113-151 and writes O (bf16) and LSE (fp32) once
//
// Per key tile (128 keys): S = Q K^T (tcgen05.mma, accumulator in TMEM) -> each thread owns one
// query row, reads it with tcgen05.ld, applies masks and the online softmax in the exp2 domain,
// writes P (bf16) into a swizzled shared-memory tile -> O' = P V (tcgen05.mma) -> O = O*alpha + O'.
// K/V tiles are double-buffered with cp.async so the next tile's loads overlap this tile's math.
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

struct FwdArgs {
  PrefillView pv;
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int* sel;
  const int* rowlist;
  const int* seg_base;
  const int* tile_base;
  const uint8_t* qpack;  // packed operand tiles, see PackState
  const uint8_t* kpack;
  const uint8_t* vpack;
  __nv_bfloat16* part_o;  // [T*Hq*R, D]
  float* part_lse;        // [T*Hq*R] log2 domain
  __nv_bfloat16* out;     // [T, Hq, D]
  float* lse;             // [T, Hq]
  unsigned* status;
  float scale_log2;
};

template <int DPAD, bool SELF>
__global__ void __launch_bounds__(128, (DPAD <= 64 ? 2 : 1)) attn_fwd_kernel(FwdArgs a) {
  constexpr int UPR = DPAD / 8;
  constexpr int TILE_BYTES = kTile * DPAD * 2;
  constexpr uint32_t TMEM_COLS = 256;
  // Dynamic shared memory only (no static), so that two CTAs of the D<=64 variant fit one SM:
  // [0,1024) control block (barriers, TMEM slot), then the 1024-aligned operand tiles.
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t& bar_s = *reinterpret_cast<uint64_t*>(smem);
  uint64_t& bar_o = *reinterpret_cast<uint64_t*>(smem + 8);
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(smem + 16);
  uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + 32);  // [2] K/V stage (and, for stage 0's first fill, Q) has landed
  uint8_t* sQ = smem + 1024;
  uint8_t* sK = sQ + TILE_BYTES;      // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;  // 2 stages
  uint8_t* sP = sV + 2 * TILE_BYTES;  // 128 x 128 bf16

  const PrefillView& pv = a.pv;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = pv.D;

  // ---- decode the work item
  int kv_head, key_begin, key_end, nrows, n_kv_tiles;
  int row_id = -1;   // SELF: t*Hq+h of this thread's row; REMOTE: slot id
  long long q_tile;  // packed query tile of this CTA
  int kblock0;       // packed key block (= 128-token tile id) holding the chunk's first keys
  int tok = 0;       // SELF: packed token of this thread's row
  if (SELF) {
    const int w = blockIdx.x;
    const int tile = pv.self_order[w / pv.Hq];
    const int h = w - (w / pv.Hq) * pv.Hq;
    const int c = pv.qtile_chunk[tile];
    const int tok0 = pv.qtile_tok0[tile];
    key_begin = pv.chunk_start[c];
    nrows = min(kTile, pv.chunk_start[c + 1] - tok0);
    key_end = tok0 + nrows;  // causal: no row of the tile sees keys past the tile's last token
    kv_head = h / pv.G;
    tok = tok0 + tid;
    if (tid < nrows) row_id = tok * pv.Hq + h;
    q_tile = (long long)tile * pv.Hq + h;
    kblock0 = tile - (tok0 - key_begin) / kTile;  // the tiles of a chunk have consecutive ids
  } else {
    const int E = pv.n_chunks * pv.Hkv;
    const int w = blockIdx.x;
    if (w >= a.tile_base[E]) return;
    int lo = 0, hi = E;  // largest e with tile_base[e] <= w
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.tile_base[mid] <= w) lo = mid; else hi = mid;
    }
    const int e = lo, i = w - a.tile_base[e];
    const int c = e / pv.Hkv;
    kv_head = e - c * pv.Hkv;
    const int start = a.seg_base[c * pv.Hq + kv_head * pv.G] + i * kTile;
    const int end = a.seg_base[c * pv.Hq + (kv_head + 1) * pv.G];
    nrows = min(kTile, end - start);
    key_begin = pv.chunk_start[c];
    key_end = pv.chunk_start[c + 1];
    if (tid < nrows) {
      row_id = a.rowlist[start + tid];
      if (row_id < 0 || row_id / pv.R >= pv.T * pv.Hq) { atomicOr(a.status, kErrBadIndex); row_id = -1; }
    }
    q_tile = (long long)pv.n_qtiles * pv.Hq + w;
    int qlo = 0, qhi = pv.n_qtiles - 1;  // first 128-token tile of chunk c (tile ids ascend with the chunk id)
    while (qlo < qhi) {
      const int mid = (qlo + qhi) >> 1;
      if (pv.qtile_chunk[mid] < c) qlo = mid + 1; else qhi = mid;
    }
    kblock0 = qlo;
  }
  n_kv_tiles = (key_end - key_begin + kTile - 1) / kTile;

  if ((smem_u32(smem) & 1023u) != 0) {  // operand tiles need 1024-byte alignment for the swizzle
    if (tid == 0) atomicOr(a.status, kErrBadIndex);
    return;
  }
  if (tid == 0) {
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, TMEM_COLS);
  __syncthreads();

  // ---- Q tile and first K/V tile: three bulk copies of packed tile images, issued by one thread
  const uint8_t* kp = a.kpack + ((size_t)kblock0 * pv.Hkv + kv_head) * TILE_BYTES;
  const uint8_t* vp = a.vpack + ((size_t)kblock0 * pv.Hkv + kv_head) * TILE_BYTES;
  const size_t kv_step = (size_t)pv.Hkv * TILE_BYTES;  // next key block of the same kv head
  if (tid == 0) {
    mbar_arrive_expect_tx(&bar_kv[0], 3 * TILE_BYTES);
    bulk_load(sQ, a.qpack + q_tile * TILE_BYTES, TILE_BYTES, &bar_kv[0]);
    bulk_load(sK, kp, TILE_BYTES, &bar_kv[0]);
    bulk_load(sV, vp, TILE_BYTES, &bar_kv[0]);
  }

  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem + (uint32_t(warp * 32) << 16);
  const uint32_t tO = tS + 128;
  const uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
  const uint32_t idesc_o = umma_idesc_bf16(128, DPAD, 0, 1);

  float o_acc[DPAD];
#pragma unroll
  for (int d = 0; d < DPAD; ++d) o_acc[d] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  uint32_t phase = 0;
  bool alive = true;

  for (int j = 0; j < n_kv_tiles; ++j) {
    const int st = j & 1;
    const int k0 = key_begin + j * kTile;
    if (tid == 0) {
      if (alive) alive = mbar_wait(&bar_kv[st], (j >> 1) & 1, a.status);
      tc_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < DPAD; kk += 16)
        umma_ss(tmem, umma_desc_kmajor(smem_u32(sQ), kTile, kk), umma_desc_kmajor(smem_u32(sK + st * TILE_BYTES), kTile, kk),
                idesc_s, kk > 0);
      umma_commit(&bar_s);
      // prefetch the next K/V tile into the other stage: its readers (S and PV of tile j-1) are done
      if (j + 1 < n_kv_tiles) {
        mbar_arrive_expect_tx(&bar_kv[st ^ 1], 2 * TILE_BYTES);
        bulk_load(sK + (st ^ 1) * TILE_BYTES, kp + (size_t)(j + 1) * kv_step, TILE_BYTES, &bar_kv[st ^ 1]);
        bulk_load(sV + (st ^ 1) * TILE_BYTES, vp + (size_t)(j + 1) * kv_step, TILE_BYTES, &bar_kv[st ^ 1]);
      }
    }
    if (alive) alive = mbar_wait(&bar_s, phase, a.status);
    tc_fence_after_sync();

    // ---- online softmax of this thread's row
    int klimit = key_end - k0;                       // keys of the tile that exist
    if (SELF) klimit = min(klimit, tok - k0 + 1);    // causal inside the own chunk
    const bool need_mask = klimit < kTile;
    float mx = -INFINITY;
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) {
      uint32_t r[32];
      tmem_ld32(tS + pc * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float s = __uint_as_float(r[i]);
        if (need_mask && pc * 32 + i >= klimit) s = -INFINITY;
        mx = fmaxf(mx, s);
      }
    }
    float m_new = fmaxf(m_run, mx * a.scale_log2);
    if (m_new == -INFINITY) m_new = 0.f;  // row with no visible key in this tile (padding rows only)
    const float alpha = fast_exp2(m_run - m_new);
    float l_tile = 0.f;
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) {
      uint32_t r[32];
      tmem_ld32(tS + pc * 32, r);
      tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), a.scale_log2, -m_new));
        float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), a.scale_log2, -m_new));
        if (need_mask) {
          if (pc * 32 + i >= klimit) p0 = 0.f;
          if (pc * 32 + i + 1 >= klimit) p1 = 0.f;
        }
        l_tile += p0 + p1;
        pk[i >> 1] = pack_bf16(p0, p1);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        *reinterpret_cast<uint4*>(sP + sw128_offset(kTile, tid, pc * 4 + u)) =
            make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
    }
    l_run = l_run * alpha + l_tile;
    m_run = m_new;

    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < kTile; kk += 16)
        umma_ss(tmem + 128, umma_desc_kmajor(smem_u32(sP), kTile, kk),
                umma_desc_mnmajor(smem_u32(sV + st * TILE_BYTES), kTile, kk, 0), idesc_o, kk > 0);
      umma_commit(&bar_o);
    }
    if (alive) alive = mbar_wait(&bar_o, phase, a.status);
    tc_fence_after_sync();
    phase ^= 1;
#pragma unroll
    for (int pc = 0; pc < DPAD / 32; ++pc) {
      uint32_t r[32];
      tmem_ld32(tO + pc * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[pc * 32 + i] = fmaf(o_acc[pc * 32 + i], alpha, __uint_as_float(r[i]));
    }
    tc_fence_before_sync();
  }

  // ---- epilogue
  if (row_id >= 0 && alive) {
    if (!SELF) {
      const float inv = 1.f / l_run;
      __nv_bfloat16* dst = a.part_o + (long long)row_id * D;
#pragma unroll
      for (int u = 0; u < UPR; ++u) {
        if (u * 8 < D)
          *reinterpret_cast<uint4*>(dst + u * 8) =
              make_uint4(pack_bf16(o_acc[u * 8] * inv, o_acc[u * 8 + 1] * inv), pack_bf16(o_acc[u * 8 + 2] * inv, o_acc[u * 8 + 3] * inv),
                         pack_bf16(o_acc[u * 8 + 4] * inv, o_acc[u * 8 + 5] * inv), pack_bf16(o_acc[u * 8 + 6] * inv, o_acc[u * 8 + 7] * inv));
      }
      a.part_lse[row_id] = m_run + log2f(l_run);
    } else {
      // global-softmax merge of the self branch with the row's remote partials (fixed slot order)
      const int R = pv.R;
      const float l2_self = m_run + log2f(l_run);
      float big = l2_self;
      const int* mysel = a.sel + (long long)row_id * R;
      int nsel = 0;
      for (int s = 0; s < R; ++s) {
        if (mysel[s] < 0) break;
        big = fmaxf(big, a.part_lse[(long long)row_id * R + s]);
        ++nsel;
      }
      const float w_self = fast_exp2(l2_self - big);
      float z = w_self;
      const float f_self = w_self / l_run;
#pragma unroll
      for (int d = 0; d < DPAD; ++d) o_acc[d] *= f_self;
      for (int s = 0; s < nsel; ++s) {
        const long long slot = (long long)row_id * R + s;
        const float w = fast_exp2(a.part_lse[slot] - big);
        z += w;
        const __nv_bfloat16* src = a.part_o + slot * D;
#pragma unroll
        for (int u = 0; u < UPR; ++u) {
          if (u * 8 < D) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src + u * 8);
            const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              o_acc[u * 8 + 2 * i] = fmaf(w, __uint_as_float(wv[i] << 16), o_acc[u * 8 + 2 * i]);
              o_acc[u * 8 + 2 * i + 1] = fmaf(w, __uint_as_float(wv[i] & 0xFFFF0000u), o_acc[u * 8 + 2 * i + 1]);
            }
          }
        }
      }
      const float inv = 1.f / z;
      __nv_bfloat16* dst = a.out + (long long)row_id * D;
#pragma unroll
      for (int u = 0; u < UPR; ++u) {
        if (u * 8 < D)
          *reinterpret_cast<uint4*>(dst + u * 8) =
              make_uint4(pack_bf16(o_acc[u * 8] * inv, o_acc[u * 8 + 1] * inv), pack_bf16(o_acc[u * 8 + 2] * inv, o_acc[u * 8 + 3] * inv),
                         pack_bf16(o_acc[u * 8 + 4] * inv, o_acc[u * 8 + 5] * inv), pack_bf16(o_acc[u * 8 + 6] * inv, o_acc[u * 8 + 7] * inv));
      }
      a.lse[row_id] = (big + log2f(z)) * 0.6931471805599453f;
    }
  }
  __syncthreads();
  if (warp == 0) tmem_free(tmem, TMEM_COLS);
}

template <int DPAD, bool SELF>
static cudaError_t launch_fwd(const FwdArgs& a, int grid, cudaStream_t st) {
  const size_t smem = 1024 + (size_t)kTile * DPAD * 2 * 5 + (size_t)kTile * kTile * 2;
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<DPAD, SELF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  attn_fwd_kernel<DPAD, SELF><<<grid, 128, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace moba

using namespace moba;

extern "C" size_t moba_prefill_fwd_scratch_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  const size_t slots = (size_t)d->total_tokens * d->hq * d->remote_k;
  return align256(slots * d->dim * 2) + align256(slots * 4) + 256;
}

extern "C" int moba_prefill_fwd(const moba_prefill_desc* d, const void* q, const void* k, const void* v,
                                const void* route_state, void* scratch, size_t scratch_bytes, void* out, float* lse,
                                unsigned* status, void* stream) {
  int rc = validate_desc(d);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !v || !out || !lse || !status || !route_state || (d->remote_k > 0 && !scratch)) return MOBA_ERR_INVALID;
  if (d->dim > 128) return MOBA_ERR_UNSUPPORTED;
  if (scratch_bytes < moba_prefill_fwd_scratch_bytes(d)) return MOBA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  FwdArgs a;
  a.pv = make_view(*d);
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.status = status;
  a.scale_log2 = (float)(1.4426950408889634 / sqrt((double)d->dim));
  a.sel = a.rowlist = a.seg_base = a.tile_base = nullptr;
  a.part_o = nullptr;
  a.part_lse = nullptr;
  const bool wide = d->dim > 64;
  cudaError_t e = launch_prefill_pack(*d, q, k, v, const_cast<void*>(route_state), status, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  {
    const PackState ps = carve_pack_state(*d, const_cast<void*>(route_state));
    a.qpack = reinterpret_cast<const uint8_t*>(ps.qpack);
    a.kpack = reinterpret_cast<const uint8_t*>(ps.kpack);
    a.vpack = reinterpret_cast<const uint8_t*>(ps.vpack);
  }
  if (d->remote_k > 0) {
    RouteState rs = carve_route_state(*d, const_cast<void*>(route_state));
    a.sel = rs.sel; a.rowlist = rs.rowlist; a.seg_base = rs.seg_base; a.tile_base = rs.tile_base;
    const size_t slots = (size_t)d->total_tokens * d->hq * d->remote_k;
    a.part_o = static_cast<__nv_bfloat16*>(scratch);
    a.part_lse = reinterpret_cast<float*>(static_cast<char*>(scratch) + align256(slots * d->dim * 2));
    // every expert has at most ceil(rows/128) tiles; the sum is bounded by slots/128 + experts
    const long long bound = (long long)(slots / kTile) + (long long)d->num_chunks * d->hkv;
    prof_begin(kProfFwdRemote, st);
    e = wide ? launch_fwd<128, false>(a, (int)bound, st) : launch_fwd<64, false>(a, (int)bound, st);
    prof_end(kProfFwdRemote, st);
    if (e != cudaSuccess) return MOBA_ERR_CUDA;
  }
  const int grid = d->num_qtiles * d->hq;
  prof_begin(kProfFwdSelf, st);
  e = wide ? launch_fwd<128, true>(a, grid, st) : launch_fwd<64, true>(a, grid, st);
  prof_end(kProfFwdSelf, st);
  return e == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
