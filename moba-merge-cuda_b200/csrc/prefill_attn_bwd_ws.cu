// Warp-specialised prefill backward for head_dim <= 64: the same mathematics and work decomposition
// as attn_bwd_kernel (one CTA owns 128 keys of one (chunk, kv head) and walks over every 128-row
// query tile that attends them), organised so that the tensor pipe, the exp/FMA pipes and the memory
// system work on different query tiles at the same time.
//   warps 0-7  compute: two threads per query row (64 of the 128 key columns each).  Per tile they read
//              S and dP from TMEM and release them at once, form P and dS in registers, drain dQ of the
//              previous tile into the FP32 accumulator, issue the cp.async copies of the Q and dO rows
//              of tile i+2 (256 threads issuing keeps enough copies in flight; two dedicated loader
//              warps could not), and store P and dS as swizzled bf16 tiles
//   warp 8     one thread issues every tcgen05.mma, polling two work streams: S/dP of tile n as soon
//              as its rows have landed and the compute warps have read tile n-1; dV/dK/dQ of tile i
//              as soon as P and dS of tile i are in shared memory
//   warp 9     resolves row ids (expert list) and gathers LSE and delta of tiles further ahead into a
//              four-slot metadata ring, with its dependent global loads software-pipelined
// TMEM columns: S 0-127, dP 128-255, dV 256-319, dK 320-383, dQ 384-447.
#include "prefill_bwd.cuh"

namespace moba {

#ifdef MOBA_BWD_TRACE
// Debug build only: per-tile clock stamps of one CTA, for finding where a tile's time goes.
__device__ long long* g_bwd_trace = nullptr;
#define WS_TRACE(role, it, slot)                                                                           \
  do {                                                                                                     \
    if (g_bwd_trace && blockIdx.x == 40 && blockIdx.y == 0 && (it) < 256)                                  \
      g_bwd_trace[((it) * 4 + (role)) * 8 + (slot)] = clock64();                                           \
  } while (0)
#else
#define WS_TRACE(role, it, slot) do {} while (0)
#endif

constexpr int kWsThreads = 320;  // 8 compute warps, 1 MMA warp, 1 metadata warp
constexpr int kWsRing = 3;       // Q/dO tiles in shared memory
constexpr int kWsMeta = 4;       // metadata slots

// One lane polls the barrier for its warp; __syncwarp orders the other lanes' later reads after
// lane 0's acquire.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, unsigned* status, bool alive) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0 && alive) ok = mbar_wait(bar, parity, status);
  __syncwarp();
  return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}
// One arrival per warp: every lane's earlier writes are ordered before it by __syncwarp.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

struct WsSmem {
  uint64_t sdp_full, sdp_free, pds_ready, kvq_done;
  uint64_t qdo_full[kWsRing], qdo_free[kWsRing];
  uint64_t meta_full[kWsMeta], meta_free[kWsMeta];
  uint32_t tmem_slot;
  uint32_t pad;
  int rowth[kWsMeta][kTile];      // t*Hq+h of every row of the tile, -1 = padding row
  float lse2[kWsMeta][kTile];     // LSE in the log2 domain (+inf for padding rows)
  float delta_s[kWsMeta][kTile];  // rowsum(dO*O) / sqrt(D)
};
static_assert(sizeof(WsSmem) <= 8192, "control block must fit its reservation");

__global__ void __launch_bounds__(kWsThreads, 1) attn_bwd_ws_kernel(BwdArgs a) {
  constexpr int DPAD = 64, UPR = 8;
  constexpr int TILE_BYTES = kTile * DPAD * 2;
  constexpr int PT_BYTES = kTile * kTile * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 320, COL_DQ = 384;
  extern __shared__ __align__(1024) uint8_t smem[];
  WsSmem& cb = *reinterpret_cast<WsSmem*>(smem);
  uint8_t* sK = smem + 8192;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;             // kWsRing tiles
  uint8_t* sdO = sQ + kWsRing * TILE_BYTES;  // kWsRing tiles
  uint8_t* sP = sdO + kWsRing * TILE_BYTES;
  uint8_t* sdS = sP + PT_BYTES;

  const PrefillView& pv = a.pv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
    mbar_init(&cb.sdp_full, 1);
    mbar_init(&cb.sdp_free, 8);
    mbar_init(&cb.pds_ready, 8);
    mbar_init(&cb.kvq_done, 1);
    for (int i = 0; i < kWsRing; ++i) { mbar_init(&cb.qdo_full[i], 256); mbar_init(&cb.qdo_free[i], 1); }
    for (int i = 0; i < kWsMeta; ++i) { mbar_init(&cb.meta_full[i], 1); mbar_init(&cb.meta_free[i], 8); }
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&cb.tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = cb.tmem_slot;
  bool alive = true;

  if (warp == 9) {
    // ================================================================== metadata
    // Row ids come from the expert list and LSE/delta are gathered by row id: two dependent global
    // loads per row, pipelined (ids two tiles ahead, LSE/delta one tile ahead of their use).
    auto resolve = [&](int j, int x) -> int {
      if (j >= n_iter) return -1;
      const int r = lane + 32 * x;
      if (j < pv.G * n_self) {
        const int hl = j / n_self, i = kb + (j - hl * n_self);
        const int tok = chunk_begin + i * kTile + r;
        return tok < chunk_end ? tok * pv.Hq + g * pv.G + hl : -1;
      }
      const int idx = (j - pv.G * n_self) * kTile + r;
      if (idx >= remote_rows) return -1;
      const int th = __ldg(a.rowlist + remote_begin + idx) / pv.R;
      if (th < 0 || th >= pv.T * pv.Hq) { atomicOr(a.status, kErrBadIndex); return -1; }
      return th;
    };
    int th_cur[4], th_nxt[4];
    float lse_cur[4], del_cur[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) { th_cur[x] = resolve(0, x); th_nxt[x] = resolve(1, x); }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      lse_cur[x] = th_cur[x] >= 0 ? __ldg(a.lse + th_cur[x]) : 0.f;
      del_cur[x] = th_cur[x] >= 0 ? __ldg(a.delta + th_cur[x]) : 0.f;
    }
    for (int j = 0; j < n_iter; ++j) {
      const int ms = j % kWsMeta;
      int th_nn[4];
      float lse_nxt[4], del_nxt[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        th_nn[x] = resolve(j + 2, x);
        lse_nxt[x] = th_nxt[x] >= 0 ? __ldg(a.lse + th_nxt[x]) : 0.f;
        del_nxt[x] = th_nxt[x] >= 0 ? __ldg(a.delta + th_nxt[x]) : 0.f;
      }
      if (j >= kWsMeta) alive = warp_wait(&cb.meta_free[ms], ((j / kWsMeta) - 1) & 1, a.status, alive);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int r = lane + 32 * x;
        cb.rowth[ms][r] = th_cur[x];
        cb.lse2[ms][r] = th_cur[x] >= 0 ? lse_cur[x] * 1.4426950408889634f : INFINITY;
        cb.delta_s[ms][r] = th_cur[x] >= 0 ? del_cur[x] * a.scale : 0.f;
      }
      warp_arrive(&cb.meta_full[ms]);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        th_cur[x] = th_nxt[x]; th_nxt[x] = th_nn[x];
        lse_cur[x] = lse_nxt[x]; del_cur[x] = del_nxt[x];
      }
    }
  } else if (warp == 8) {
    // ================================================================== MMA issue
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_kv = umma_idesc_bf16(128, DPAD, 1, 1);
      const uint32_t idesc_dq = umma_idesc_bf16(128, DPAD, 0, 1);
      // Operand descriptors are built once; inside the loop a descriptor is its base plus a constant
      // (the start-address field counts 16-byte units).
      const uint64_t k_km = umma_desc_kmajor(smem_u32(sK), kTile, 0), k_mn = umma_desc_mnmajor(smem_u32(sK), kTile, 0, 0);
      const uint64_t v_km = umma_desc_kmajor(smem_u32(sV), kTile, 0);
      const uint64_t q_km = umma_desc_kmajor(smem_u32(sQ), kTile, 0), q_mn = umma_desc_mnmajor(smem_u32(sQ), kTile, 0, 0);
      const uint64_t o_km = umma_desc_kmajor(smem_u32(sdO), kTile, 0), o_mn = umma_desc_mnmajor(smem_u32(sdO), kTile, 0, 0);
      const uint64_t p_mn = umma_desc_mnmajor(smem_u32(sP), kTile, 0, 0);
      const uint64_t s_mn = umma_desc_mnmajor(smem_u32(sdS), kTile, 0, 0), s_km = umma_desc_kmajor(smem_u32(sdS), kTile, 0);
      auto issue_sdp = [&](int j) {
        const uint64_t slot = (uint64_t)((j % kWsRing) * (TILE_BYTES >> 4));
#pragma unroll
        for (int kk = 0; kk < DPAD; kk += 16)  // K-major step: 16 elements = 32 bytes = 2 units
          umma_ss(tmem + COL_S, q_km + slot + (kk >> 3), k_km + (kk >> 3), idesc_qk, kk > 0);
#pragma unroll
        for (int kk = 0; kk < DPAD; kk += 16)
          umma_ss(tmem + COL_DP, o_km + slot + (kk >> 3), v_km + (kk >> 3), idesc_qk, kk > 0);
        umma_commit(&cb.sdp_full);
      };
      auto issue_kvq = [&](int it) {
        const uint64_t slot = (uint64_t)((it % kWsRing) * (TILE_BYTES >> 4));
        const uint32_t acc = it > 0;
#pragma unroll
        for (int kk = 0; kk < kTile; kk += 16)  // dV += P^T dO; MN-major step: 16 rows = 2048 bytes = 128 units
          umma_ss(tmem + COL_DV, p_mn + kk * 8, o_mn + slot + kk * 8, idesc_kv, acc | (kk > 0));
#pragma unroll
        for (int kk = 0; kk < kTile; kk += 16)  // dK += dS^T Q
          umma_ss(tmem + COL_DK, s_mn + kk * 8, q_mn + slot + kk * 8, idesc_kv, acc | (kk > 0));
        umma_commit(&cb.qdo_free[it % kWsRing]);  // the tile's Q and dO rows are no longer needed
#pragma unroll
        for (int kk = 0; kk < kTile; kk += 16)  // dQ = dS K; dS K-major over two 64-key panels of 16 KB
          umma_ss(tmem + COL_DQ, s_km + (kk >> 6) * (kTile * 128 >> 4) + ((kk & 63) >> 3), k_mn + kk * 8, idesc_dq, kk > 0);
        umma_commit(&cb.kvq_done);
      };
      // Two streams of work are issued as their inputs become ready, whichever comes first:
      //   S, dP of tile n    needs the tile's Q/dO in the ring and S/dP of tile n-1 read by the compute warps
      //   dV, dK, dQ of tile i needs P and dS of tile i in shared memory
      int next_sdp = 0, next_kvq = 0;
      const long long t_start = clock64();
      while (next_kvq < n_iter) {
        bool progressed = false;
        if (next_sdp < n_iter && next_sdp <= next_kvq + 1) {
          const bool loaded = !alive || mbar_test(&cb.qdo_full[next_sdp % kWsRing], (next_sdp / kWsRing) & 1);
          const bool freed = next_sdp == 0 || !alive || mbar_test(&cb.sdp_free, (next_sdp - 1) & 1);
          if (loaded && freed) {
            fence_async_smem();  // cp.async data of the ring -> visible to the tensor pipe
            tc_fence_after_sync();
            WS_TRACE(1, next_sdp, 0);
            issue_sdp(next_sdp++);
            progressed = true;
          }
        }
        if (next_kvq < next_sdp && (!alive || mbar_test(&cb.pds_ready, next_kvq & 1))) {
          tc_fence_after_sync();
          WS_TRACE(1, next_kvq, 1);
          issue_kvq(next_kvq++);
          progressed = true;
        }
        if (!progressed) {
          __nanosleep(32);
          if (alive && clock64() - t_start > 4000000000ll) {
            atomicOr(a.status, kErrBarrierTimeout);
            alive = false;
          }
        }
      }
    }
  } else {
    // ================================================================== compute (warps 0-7)
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t tlane = tmem + (uint32_t(quad * 32) << 16);
    // Copies of the Q and dO rows of tile j into ring slot j % kWsRing: thread = (unit, 4 rows), so
    // eight consecutive threads fetch one 128-byte row.  The slot's barrier gets one asynchronous
    // arrival per thread, fired by the hardware when that thread's copies have landed.
    auto issue_tile_copies = [&](int j) {
      const int ms = j % kWsMeta, b = j % kWsRing;
      alive = warp_wait(&cb.meta_full[ms], (j / kWsMeta) & 1, a.status, alive);
      const uint32_t qdst = smem_u32(sQ + b * TILE_BYTES), odst = smem_u32(sdO + b * TILE_BYTES);
      const int u = tid & 7;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int row = (tid >> 3) + 32 * x;
        const int rth = cb.rowth[ms][row];
        const bool ok = rth >= 0 && u * 8 < D;
        const int t = rth / pv.Hq, h = rth - t * pv.Hq;
        const uint32_t off = sw128_offset(kTile, row, u);
        cp_async16(qdst + off, ok ? a.q + (long long)t * pv.q_st + (long long)h * pv.q_sh + u * 8 : a.q, ok);
        cp_async16(odst + off, ok ? a.dout + (long long)rth * D + u * 8 : a.dout, ok);
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];" ::"r"(smem_u32(&cb.qdo_full[b])) : "memory");
    };
    {  // stationary K and V tiles of the key block ride along with tile 0
      const __nv_bfloat16* kbase = a.k + (long long)g * pv.k_sh;
      const __nv_bfloat16* vbase = a.v + (long long)g * pv.v_sh;
      for (int i = tid; i < kTile * UPR; i += 256) {
        const int row = i >> 3, u = i & 7;
        const bool ok = row < nkeys && u * 8 < D;
        cp_async16(smem_u32(sK) + sw128_offset(kTile, row, u), ok ? kbase + (long long)(k0 + row) * pv.k_st + u * 8 : kbase, ok);
        cp_async16(smem_u32(sV) + sw128_offset(kTile, row, u), ok ? vbase + (long long)(k0 + row) * pv.v_st + u * 8 : vbase, ok);
      }
    }
    issue_tile_copies(0);
    if (n_iter > 1) issue_tile_copies(1);

    int th_prev = -1;
    auto drain_dq = [&](int th) {  // dQ of the previous tile: this thread's 32 of the 64 columns
      uint32_t v[32];
      tmem_ld32(tlane + COL_DQ + half * 32, v);
      tmem_ld_wait();
#ifdef MOBA_BWD_NODRAIN
      if (th == -12345) {
#else
      if (th >= 0 && alive) {
#endif
        float* dst = a.dq_acc + (long long)th * D + half * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          if (half * 32 + i < D)
            red_add_v4(dst + i, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
      }
    };
    for (int it = 0; it < n_iter; ++it) {
      const int ms = it % kWsMeta;
      if (tid == 0) WS_TRACE(0, it, 0);
      // metadata of this tile was acquired when its copies were issued (two tiles ago)
      const int th = cb.rowth[ms][r];
      const float lse2 = cb.lse2[ms][r], delta_s = cb.delta_s[ms][r];
      warp_arrive(&cb.meta_free[ms]);
      const bool diag = it < pv.G * n_self && (it % n_self) == 0;
      int klimit = nkeys;
      if (diag) klimit = min(klimit, r + 1);
      klimit -= half * 64;  // relative to this thread's first column

      alive = warp_wait(&cb.sdp_full, it & 1, a.status, alive);
      if (tid == 0) WS_TRACE(0, it, 2);
      tc_fence_after_sync();
      uint32_t sv[64], dv[64];
      {
        uint32_t t0[32], t1[32];
        tmem_ld32(tlane + COL_S + half * 64, t0);
        tmem_ld32(tlane + COL_S + half * 64 + 32, t1);
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = t0[i]; sv[32 + i] = t1[i]; }
        tmem_ld32(tlane + COL_DP + half * 64, t0);
        tmem_ld32(tlane + COL_DP + half * 64 + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { dv[i] = t0[i]; dv[32 + i] = t1[i]; }
      }
      tc_fence_before_sync();
      warp_arrive(&cb.sdp_free);  // S and dP may be overwritten by the next tile's products
      if (tid == 0) WS_TRACE(0, it, 3);

      uint32_t pp[32], ds[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        float p0 = bwd_exp2(fmaf(__uint_as_float(sv[i]), a.scale_log2, -lse2));
        float p1 = bwd_exp2(fmaf(__uint_as_float(sv[i + 1]), a.scale_log2, -lse2));
        if (i >= klimit) p0 = 0.f;
        if (i + 1 >= klimit) p1 = 0.f;
        const float d0 = p0 * fmaf(__uint_as_float(dv[i]), a.scale, -delta_s);
        const float d1 = p1 * fmaf(__uint_as_float(dv[i + 1]), a.scale, -delta_s);
        pp[i >> 1] = bwd_pack_bf16(p0, p1);
        ds[i >> 1] = bwd_pack_bf16(d0, d1);
      }
      if (tid == 0) WS_TRACE(0, it, 4);
      if (it > 0) {  // previous tile's dV/dK/dQ products are complete: sP/sdS are free, dQ can be drained
        alive = warp_wait(&cb.kvq_done, (it - 1) & 1, a.status, alive);
        if (tid == 0) WS_TRACE(0, it, 5);
        tc_fence_after_sync();
        drain_dq(th_prev);
        tc_fence_before_sync();
      }
      if (tid == 0) WS_TRACE(3, it, 0);
      // ring slot (it+2) % 3 held tile it-1, whose last readers (dV, dK) finished before kvq_done(it-1)
      if (it + 2 < n_iter) issue_tile_copies(it + 2);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        *reinterpret_cast<uint4*>(sP + sw128_offset(kTile, r, half * 8 + u)) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
        *reinterpret_cast<uint4*>(sdS + sw128_offset(kTile, r, half * 8 + u)) = make_uint4(ds[4 * u], ds[4 * u + 1], ds[4 * u + 2], ds[4 * u + 3]);
      }
      if (tid == 0) WS_TRACE(0, it, 6);
      fence_async_smem();
      warp_arrive(&cb.pds_ready);
      if (tid == 0) WS_TRACE(0, it, 7);
      th_prev = th;
    }
    cp_async_wait<0>();
    if (n_iter > 0) {
      alive = warp_wait(&cb.kvq_done, (n_iter - 1) & 1, a.status, alive);
      tc_fence_after_sync();
      drain_dq(th_prev);
      // dK (warps 0-3) and dV (warps 4-7) of the key block: thread = key row
      const bool ok = r < nkeys && alive;
      __nv_bfloat16* dst = (half == 0 ? a.dk : a.dv) + ((long long)(k0 + r) * pv.Hkv + g) * D;
#pragma unroll
      for (int pc = 0; pc < 2; ++pc) {
        uint32_t v[32];
        tmem_ld32(tlane + (half == 0 ? COL_DK : COL_DV) + pc * 32, v);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            if (pc * 32 + i < D)
              *reinterpret_cast<uint4*>(dst + pc * 32 + i) =
                  make_uint4(bwd_pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                             bwd_pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                             bwd_pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                             bwd_pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, TMEM_COLS);
}

cudaError_t launch_bwd_ws(const BwdArgs& a, cudaStream_t st) {
  const size_t smem = 8192 + (size_t)kTile * 64 * 2 * (2 + 2 * kWsRing) + (size_t)kTile * kTile * 2 * 2;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  attn_bwd_ws_kernel<<<dim3(a.pv.n_qtiles, a.pv.Hkv), kWsThreads, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace moba

#ifdef MOBA_BWD_TRACE
extern "C" int moba_debug_set_bwd_trace(long long* buf) {
  return cudaMemcpyToSymbol(moba::g_bwd_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : 2;
}
#endif
