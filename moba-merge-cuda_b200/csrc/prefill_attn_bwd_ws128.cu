// Warp-specialised prefill backward for 64 < head_dim <= 128.  Same scheme as prefill_attn_bwd_ws.cu
// (one CTA owns 128 keys of one (chunk, kv head); scores transposed, keys on the tensor-memory lanes;
// P^T and dS^T are tensor-memory operands of the dV and dK products), with the geometry that fits the
// 512 tensor-memory columns at this head dimension: query tiles are taken 64 rows at a time, and dQ is
// formed transposed,
//     S^T[128 keys, 64 q] = K Q^T,  dP^T = V dO^T,  dV[128, D] += P^T dO,  dK[128, D] += dS^T Q,
//     dQ^T[D, 64 q] = K^T dS^T,
// with the head dimension on the tensor-memory lanes; the drain warps write it to shared memory as query rows
// and the copy engine adds every row to the FP32 accumulator with one bulk reduction.
// Tensor memory: S^T 0-63 and dP^T 64-127 (P^T and dS^T as packed 16-bit values over the first columns of each
// thread's own range), dV 128-255, dK 256-383, dQ^T 384-447, K 448-511 as a stationary A operand.
// Shared memory: K and V images (32 KB each), a 3-slot ring of (Q, dO) half tiles (64 rows x 128 columns
// each, 16 KB), the dS^T tile (128 key rows x 64 query columns, 16 KB), the dQ rows of a step (32 KB).
#include "prefill_bwd.cuh"

namespace moba {

namespace {

constexpr int kThreads = 512;  // 8 compute warps, MMA warp, producer warp (+2 idle), 4 dQ drain warps
constexpr int kRing = 3;       // (Q, dO) half tiles in flight; the dQ staging takes the room of a fourth
constexpr int kQRows = 64;     // query rows per step

struct Smem128 {
  uint64_t st_full, p_ready, ka_ready, dpt_full, ds_ready, dq_done, dq_free, kv_ready;
  uint64_t qdo_full[kRing], qdo_free[kRing];
  uint32_t tmem_slot;
  uint32_t pad;
  __align__(16) int rowth[kRing][kQRows];      // t*Hq+h of every query row of the step, -1 = padding row
  __align__(16) float lse2[kRing][kQRows];     // -LSE in the log2 domain (-inf for padding rows)
  __align__(16) float delta_s[kRing][kQRows];  // -rowsum(dO*O) / sqrt(D)
};
static_assert(sizeof(Smem128) <= 4096, "control block must fit its reservation");

}  // namespace

template <bool F16>
__global__ void __launch_bounds__(kThreads, 1) attn_bwd_ws128_kernel(BwdArgs a) {
  constexpr int DPAD = 128;
  constexpr int KV_BYTES = kTile * DPAD * 2;      // 32 KB: two 64-column panels of 128 rows
  constexpr int HALF_BYTES = kQRows * DPAD * 2;   // 16 KB: two 64-column panels of 64 rows
  constexpr int PANEL_BYTES = kQRows * 128;       // 8 KB
  constexpr int SLOT_BYTES = 2 * HALF_BYTES;      // Q half tile followed by dO half tile
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_ST = 0, COL_DPT = 64, COL_DV = 128, COL_DK = 256, COL_DQT = 384, COL_KA = 448;
  extern __shared__ __align__(1024) uint8_t smem[];
  Smem128& cb = *reinterpret_cast<Smem128*>(smem);
  uint8_t* sK = smem + 4096;
  uint8_t* sV = sK + KV_BYTES;
  uint8_t* sQ = sV + KV_BYTES;
  uint8_t* sdO = sQ + HALF_BYTES;
  uint8_t* sdS = sQ + kRing * SLOT_BYTES;  // dS^T: 128 key rows x 64 query columns bf16 (one panel)
  uint8_t* sStage = sdS + kTile * kQRows * 2;  // dQ of a step as 64 query rows x 128 floats (32 KB)

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
  int remote_rows = 0;
  if (pv.R > 0) remote_rows = a.seg_base[c * pv.Hq + (g + 1) * pv.G] - a.seg_base[c * pv.Hq + g * pv.G];
  const int n_remote = (remote_rows + kTile - 1) / kTile;
  const int n_tiles = pv.G * n_self + n_remote;
  const int n_iter = 2 * n_tiles;  // two 64-row steps per query tile

  if ((smem_u32(smem) & 1023u) != 0) {
    if (tid == 0) atomicOr(a.status, kErrBadIndex);
    return;
  }
  if (tid == 0) {
    mbar_init(&cb.st_full, 1);
    mbar_init(&cb.p_ready, 8);
    mbar_init(&cb.ka_ready, 8);
    mbar_init(&cb.dpt_full, 1);
    mbar_init(&cb.ds_ready, 8);
    mbar_init(&cb.dq_done, 1);
    mbar_init(&cb.dq_free, 4);
    mbar_init(&cb.kv_ready, 1);
    for (int i = 0; i < kRing; ++i) { mbar_init(&cb.qdo_full[i], 1); mbar_init(&cb.qdo_free[i], 5); }
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&cb.tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = cb.tmem_slot;
  bool alive = true;

  if (warp >= 12) {
    // ================================================================== dQ drain (warps 12-15)
    // dQ^T has the head dimension on the lanes: a warp owns 32 consecutive dimensions, every thread the
    // 64 query rows of its dimension.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    const int quad = warp & 3;
    float* rows = reinterpret_cast<float*>(sStage);                  // [64 queries][128 dimensions]
    const bool fixed = a.dq_fixed != nullptr;
    const uint32_t tlane = tmem + (uint32_t(quad * 32) << 16);
    auto drain_sync = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    for (int it = 0; it < n_iter; ++it) {
      const int slot = it % kRing;
      alive = warp_wait(&cb.qdo_full[slot], (it / kRing) & 1, a.status, alive);
      const int th0 = cb.rowth[slot][lane], th1 = cb.rowth[slot][32 + lane];
      warp_arrive(&cb.qdo_free[slot]);
      alive = warp_wait(&cb.dq_done, it & 1, a.status, alive);
      tc_fence_after_sync();
      uint32_t v0[32], v1[32];
      tmem_ld32(tlane + COL_DQT, v0);
      tmem_ld32(tlane + COL_DQT + 32, v1);
      tmem_ld_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.dq_free);
      if (!fixed) {
        // Ordinary mode: the step's dQ goes to shared memory as 64 query rows (a thread writes its dimension of every
        // row, lanes on consecutive floats), and the copy engine adds each row to its place in the FP32 accumulator:
        // one 512-byte reduction per row issued by warps 12 and 13, carried by the engine's own path to the L2 cache
        // instead of the load/store pipe.  The four warps meet twice per step: before writing (the engine has read
        // the previous step's rows) and before the rows are handed over.
        if (quad < 2) bulk_wait_group_read();
        drain_sync();
        const int dcol = quad * 32 + lane;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          rows[i * 128 + dcol] = __uint_as_float(v0[i]);
          rows[(32 + i) * 128 + dcol] = __uint_as_float(v1[i]);
        }
        fence_async_smem();
        drain_sync();
        if (quad < 2) {
          const int th = quad == 0 ? th0 : th1;
          if (th >= 0 && alive) bulk_reduce_add_f32(a.dq_acc + (long long)th * D, rows + (quad * 32 + lane) * 128, (uint32_t)D * 4u);
          bulk_commit_group();
        }
        continue;
      }
      // Deterministic mode: the same hand-over with 64-bit fixed-point values (32 fractional bits), whose integer sums
      // do not depend on the order in which the key blocks' contributions arrive.  A query row of 128 such values is
      // twice the size of a staged row, so it goes in two rounds of 64 dimensions: warps 12, 13 hold the first 64,
      // warps 14, 15 the second.
      unsigned long long* rows64 = reinterpret_cast<unsigned long long*>(sStage);   // [64 queries][64 dimensions]
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (quad < 2) bulk_wait_group_read();
        drain_sync();
        if ((quad >> 1) == r) {
          const int dl = (quad & 1) * 32 + lane;   // dimension inside the round
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            rows64[i * 64 + dl] = (unsigned long long)__float2ll_rn(__uint_as_float(v0[i]) * 4294967296.f);
            rows64[(32 + i) * 64 + dl] = (unsigned long long)__float2ll_rn(__uint_as_float(v1[i]) * 4294967296.f);
          }
          fence_async_smem();
        }
        drain_sync();
        if (quad < 2) {
          const int th = quad == 0 ? th0 : th1;
          if (th >= 0 && alive && r * 64 < D)
            bulk_reduce_add_u64(a.dq_fixed + (long long)th * D + r * 64, rows64 + (quad * 32 + lane) * 64, (uint32_t)min(64, D - r * 64) * 8u);
          bulk_commit_group();
        }
      }
    }
    bulk_wait_group();   // the engine has finished with this CTA's shared memory and its reductions are performed
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 9) {
      // ================================================================== producer
      if (lane == 0) {
        {  // stationary K and V images of the key block
          const size_t kvoff = ((size_t)kblock * pv.Hkv + g) * KV_BYTES;
          mbar_arrive_expect_tx(&cb.kv_ready, 2 * KV_BYTES);
          bulk_load(sK, reinterpret_cast<const uint8_t*>(a.kpack) + kvoff, KV_BYTES, &cb.kv_ready);
          bulk_load(sV, reinterpret_cast<const uint8_t*>(a.vpack) + kvoff, KV_BYTES, &cb.kv_ready);
        }
        const long long self_tiles = (long long)pv.n_qtiles * pv.Hq;
        const long long remote_tile0 = pv.R > 0 ? self_tiles + a.tile_base[c * pv.Hkv + g] : 0;
        for (int j = 0; j < n_iter; ++j) {
          const int b = j % kRing, jt = j >> 1, sub = j & 1;
          long long tile;
          if (jt < n_remote) {
            // the key blocks of a chunk walk the same expert list at the same time, a couple of tiles apart
            int jr = jt + (kb * 2) % n_remote;
            if (jr >= n_remote) jr -= n_remote;
            tile = remote_tile0 + jr;
          } else {
            const int s = jt - n_remote;
            const int hl = s / n_self, i = kb + (s - hl * n_self);
            tile = (long long)(kblock - kb + i) * pv.Hq + g * pv.G + hl;  // query tiles of a chunk are consecutive
          }
          if (j >= kRing && alive) alive = mbar_wait(&cb.qdo_free[b], ((j / kRing) - 1) & 1, a.status);
          mbar_arrive_expect_tx(&cb.qdo_full[b], 2 * HALF_BYTES + 3 * kQRows * 4);
          // rows [64 sub, 64 sub + 64) of both 64-column panels of the packed 128-row images
          const uint8_t* qsrc = reinterpret_cast<const uint8_t*>(a.qpack) + tile * KV_BYTES + sub * PANEL_BYTES;
          const uint8_t* osrc = reinterpret_cast<const uint8_t*>(a.dopack) + tile * KV_BYTES + sub * PANEL_BYTES;
          uint8_t* qdst = sQ + b * SLOT_BYTES;
          uint8_t* odst = sdO + b * SLOT_BYTES;
          bulk_load(qdst, qsrc, PANEL_BYTES, &cb.qdo_full[b]);
          bulk_load(qdst + PANEL_BYTES, qsrc + kTile * 128, PANEL_BYTES, &cb.qdo_full[b]);
          bulk_load(odst, osrc, PANEL_BYTES, &cb.qdo_full[b]);
          bulk_load(odst + PANEL_BYTES, osrc + kTile * 128, PANEL_BYTES, &cb.qdo_full[b]);
          const long long moff = tile * kTile + sub * kQRows;
          bulk_load(cb.rowth[b], a.rowpack + moff, kQRows * 4, &cb.qdo_full[b]);
          bulk_load(cb.lse2[b], a.lsepack + moff, kQRows * 4, &cb.qdo_full[b]);
          bulk_load(cb.delta_s[b], a.deltapack + moff, kQRows * 4, &cb.qdo_full[b]);
        }
      }
    } else if (warp == 8) {
      // ================================================================== MMA issue
      // Fixed order per step n:  dV(n) | S^T(n+1) | dK(n) | dP^T(n+1) | dQ^T(n): P^T lives in the columns of S^T, dS^T in
      // those of dP^T, and the tensor pipe runs in issue order.  K is a stationary A operand in tensor memory.
      const bool leader = bwd_elect_one();
      const uint32_t idesc_st = umma_idesc_16<F16>(128, kQRows, 0, 0);   // K-major x K-major, N = 64 queries
      const uint32_t idesc_kv = umma_idesc_16<F16>(128, DPAD, 0, 1);     // A from tensor memory, B MN-major, N = 128
      const uint32_t idesc_dq = umma_idesc_16<F16>(128, kQRows, 1, 1);   // A = K (MN-major), B = dS^T tile (MN-major)
      // Operand descriptors are built once; a descriptor is its base plus a constant (the start-address
      // field counts 16-byte units): a K-major step of 16 elements is 2 units inside a 64-column panel,
      // an MN-major step of 16 rows is 128 units.
      const uint64_t k_mn = umma_desc_mnmajor(smem_u32(sK), kTile, 0, 0);
      const uint64_t v_km = umma_desc_kmajor(smem_u32(sV), kTile, 0);
      const uint64_t q_km = umma_desc_kmajor(smem_u32(sQ), kQRows, 0), q_mn = umma_desc_mnmajor(smem_u32(sQ), kQRows, 0, 0);
      const uint64_t o_km = umma_desc_kmajor(smem_u32(sdO), kQRows, 0), o_mn = umma_desc_mnmajor(smem_u32(sdO), kQRows, 0, 0);
      const uint64_t s_mn = umma_desc_mnmajor(smem_u32(sdS), kTile, 0, 0);
      constexpr uint32_t KV_PANEL_U = (kTile * 128) >> 4, Q_PANEL_U = (kQRows * 128) >> 4;  // V is still read from shared memory
      auto slot_u = [&](int n) { return (uint64_t)((n % kRing) * (SLOT_BYTES >> 4)); };
      auto issue_st = [&](int n) {
        if (alive) alive = mbar_wait(&cb.qdo_full[n % kRing], (n / kRing) & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
          const uint64_t su = slot_u(n);
#pragma unroll
          for (int kk = 0; kk < DPAD; kk += 16)
            umma_ts(tmem + COL_ST, tmem + COL_KA + (kk >> 1), q_km + su + (kk >> 6) * Q_PANEL_U + ((kk & 63) >> 3), idesc_st, kk > 0);
          umma_commit(&cb.st_full);
        }
        __syncwarp();
      };
      auto issue_dpt = [&](int n) {
        if (leader) {
          const uint64_t su = slot_u(n);
#pragma unroll
          for (int kk = 0; kk < DPAD; kk += 16)
            umma_ss(tmem + COL_DPT, v_km + (kk >> 6) * KV_PANEL_U + ((kk & 63) >> 3), o_km + su + (kk >> 6) * Q_PANEL_U + ((kk & 63) >> 3),
                    idesc_st, kk > 0);
          umma_commit(&cb.dpt_full);
        }
        __syncwarp();
      };
      if (n_iter > 0) {
        if (alive) alive = mbar_wait(&cb.ka_ready, 0, a.status);
        issue_st(0);
        issue_dpt(0);
      }
      for (int n = 0; n < n_iter; ++n) {
        const uint32_t acc = n > 0;
        const uint64_t su = slot_u(n);
        if (alive) alive = mbar_wait(&cb.p_ready, n & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kQRows; kk += 16)  // dV += P^T dO over the 64 query rows of the step; queries 0-31 at columns 0.., 32-63 at columns 32..
            umma_ts(tmem + COL_DV, tmem + COL_ST + (kk >> 5) * 32 + ((kk & 31) >> 1), o_mn + su + kk * 8, idesc_kv, acc | (kk > 0));
        }
        __syncwarp();
        if (n + 1 < n_iter) issue_st(n + 1);
        if (alive) alive = mbar_wait(&cb.ds_ready, n & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kQRows; kk += 16)  // dK += dS^T Q; queries 0-31 at columns 64.., 32-63 at columns 96..
            umma_ts(tmem + COL_DK, tmem + COL_DPT + (kk >> 5) * 32 + ((kk & 31) >> 1), q_mn + su + kk * 8, idesc_kv, acc | (kk > 0));
          umma_commit(&cb.qdo_free[n % kRing]);  // the step's Q and dO rows are no longer needed
        }
        __syncwarp();
        if (n + 1 < n_iter) issue_dpt(n + 1);
        if (n > 0 && alive) alive = mbar_wait(&cb.dq_free, (n - 1) & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kTile; kk += 16)  // dQ^T = K^T dS^T, contraction over the 128 keys
            umma_ss(tmem + COL_DQT, k_mn + kk * 8, s_mn + kk * 8, idesc_dq, kk > 0);
          umma_commit(&cb.dq_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ================================================================== compute (warps 0-7)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;  // key row of this thread; its query columns are [32 half, 32 half + 32)
    const uint32_t tlane = tmem + (uint32_t(quad * 32) << 16);
    if (n_iter > 0) {
      // K of the key block into tensor memory as an A operand: thread = key row, one 32-bit column per pair of
      // dimensions; warps 0-3 take the first 64-column panel, warps 4-7 the second
      alive = warp_wait(&cb.kv_ready, 0, a.status, alive);
      uint32_t kv[32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 w = *reinterpret_cast<const uint4*>(sK + sw128_offset(kTile, r, half * 8 + u));
        kv[4 * u] = w.x; kv[4 * u + 1] = w.y; kv[4 * u + 2] = w.z; kv[4 * u + 3] = w.w;
      }
      tmem_st32(tlane + COL_KA + half * 32, kv);
      tmem_st_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.ka_ready);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int ms = it % kRing, jt = it >> 1, sub = it & 1;
      // queries below qmin (index inside the 128-row tile) are masked for this key
      const bool diag = jt >= n_remote && ((jt - n_remote) % n_self) == 0;
      const int qmin = r >= nkeys ? kTile : (diag ? r : 0);
      const int q0 = sub * kQRows + half * 32;  // first query of this thread's columns
      const bool unmasked = __all_sync(0xFFFFFFFFu, qmin <= q0);
      alive = warp_wait(&cb.qdo_full[ms], (it / kRing) & 1, a.status, alive);
      alive = warp_wait(&cb.st_full, it & 1, a.status, alive);
      tc_fence_after_sync();
      float p[32];
      {
        uint32_t t[32];
        tmem_ld32(tlane + COL_ST + half * 32, t);
        tmem_ld_wait();
        const float4* lse4 = reinterpret_cast<const float4*>(&cb.lse2[ms][half * 32]);
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 la = lse4[i >> 2];
          const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(t[i]), __uint_as_float(t[i + 1])), sc2, make_float2(la.x, la.y));
          const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(t[i + 2]), __uint_as_float(t[i + 3])), sc2, make_float2(la.z, la.w));
          p[i] = bwd_exp2(x0.x); p[i + 1] = bwd_exp2(x0.y); p[i + 2] = bwd_exp2(x1.x); p[i + 3] = bwd_exp2(x1.y);
        }
      }
      if (!unmasked) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (q0 + i < qmin) p[i] = 0.f;
      }
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = pack16<F16>(p[2 * i], p[2 * i + 1]);
      tmem_st16(tlane + COL_ST + half * 32, pk);  // over the first 16 of this thread's own S^T columns, which it has read
      tmem_st_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.p_ready);

      alive = warp_wait(&cb.dpt_full, it & 1, a.status, alive);
      tc_fence_after_sync();
      {
        uint32_t t[32];
        tmem_ld32(tlane + COL_DPT + half * 32, t);
        tmem_ld_wait();
        const float4* del4 = reinterpret_cast<const float4*>(&cb.delta_s[ms][half * 32]);
        const float2 sc = make_float2(a.scale, a.scale);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 dl = del4[i >> 2];
          const float2 e0 = __ffma2_rn(make_float2(__uint_as_float(t[i]), __uint_as_float(t[i + 1])), sc, make_float2(dl.x, dl.y));
          const float2 e1 = __ffma2_rn(make_float2(__uint_as_float(t[i + 2]), __uint_as_float(t[i + 3])), sc, make_float2(dl.z, dl.w));
          const float2 d0 = __fmul2_rn(make_float2(p[i], p[i + 1]), e0);
          const float2 d1 = __fmul2_rn(make_float2(p[i + 2], p[i + 3]), e1);
          pk[i >> 1] = pack16<F16>(d0.x, d0.y);
          pk[(i >> 1) + 1] = pack16<F16>(d1.x, d1.y);
        }
      }
      // dS^T: over the first 16 of this thread's own dP^T columns for the dK product, and as a tile row in
      // shared memory for the dQ^T product (whose previous run must be over)
      tmem_st16(tlane + COL_DPT + half * 32, pk);
      if (it > 0) alive = warp_wait(&cb.dq_done, (it - 1) & 1, a.status, alive);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        *reinterpret_cast<uint4*>(sdS + sw128_offset(kTile, r, half * 4 + u)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before_sync();
      warp_arrive(&cb.ds_ready);
    }
    if (n_iter > 0) {
      alive = warp_wait(&cb.dq_done, (n_iter - 1) & 1, a.status, alive);
      tc_fence_after_sync();
      // dK (warps 0-3) and dV (warps 4-7) of the key block: thread = key row
      const bool ok = r < nkeys && alive;
      __nv_bfloat16* dst = (half == 0 ? a.dk : a.dv) + ((long long)(k0 + r) * pv.Hkv + g) * D;
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        uint32_t v[32];
        tmem_ld32(tlane + (half == 0 ? COL_DK : COL_DV) + pc * 32, v);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            if (pc * 32 + i < D)
              *reinterpret_cast<uint4*>(dst + pc * 32 + i) =
                  make_uint4(pack16<F16>(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                             pack16<F16>(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                             pack16<F16>(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                             pack16<F16>(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, TMEM_COLS);
}

cudaError_t launch_bwd_ws128(const BwdArgs& a, cudaStream_t st) {
  const size_t smem = 4096 + 2 * (size_t)kTile * 128 * 2 + (size_t)kRing * 2 * kQRows * 128 * 2 + (size_t)kTile * kQRows * 2 + (size_t)kQRows * 128 * 4;
  const auto kernel = a.pv.fp16 ? attn_bwd_ws128_kernel<true> : attn_bwd_ws128_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kernel<<<dim3(a.pv.n_qtiles, a.pv.Hkv), kThreads, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace moba
