// Warp-specialised prefill backward for head_dim <= 64.  One CTA owns 128 keys of one (chunk, kv head),
// keeps K and V in shared memory and dK, dV in tensor memory for its whole life, and walks over every
// 128-row query tile that attends them.  Scores are formed transposed, keys on the tensor-memory lanes
// and queries along the columns:
//     S^T = K Q^T, dP^T = V dO^T     ->  P^T = exp2(S^T c - LSE[q]),  dS^T = P^T (dP^T - delta[q]) / sqrt(D)
//     dV += P^T dO,  dK += dS^T Q    with P^T and dS^T read by the tensor cores straight from tensor memory,
//                                    and so are K and V in the first two products
//     dQ  = dS K                     with dS^T also stored once as a shared-memory tile
// so per tile only dS crosses shared memory (the five products of a tile otherwise read every operand
// from shared memory, which is what bounded the kernel).
//   warps 0-7    compute: two threads per key row (64 of the 128 query columns each)
//   warp 8       issues every tcgen05.mma in a fixed order (whole warp walks the schedule, one lane issues)
//   warp 9       one thread asks the copy engine for the tiles: a packing pass has gathered the scattered
//                Q and dO rows, row ids, LSE and delta of every tile into contiguous, already swizzled
//                16 KB images, so a tile is five bulk copies into a four-slot ring
//   warps 12-15  dQ drain: tensor memory -> registers -> one row per thread in shared memory -> one bulk reduction
//                per row into the FP32 accumulator by the copy engine, behind the next tile's math
// Tensor memory: S^T 0-127 (P^T as packed 16-bit over the first columns of each thread's range), dP^T 128-255 (dS^T
// likewise), dV 256-319, dK 320-383, dQ 384-447, K 448-479 and V 480-511 as stationary A operands.
#include "prefill_bwd.cuh"

namespace moba {

// ---------------------------------------------------------------------------------------------
// Backward packing pass: dO rows, LSE (log2 domain) and delta / sqrt(D) of every query tile, in the
// tile order of the forward's Q pack (row ids come from its rowpack), as contiguous swizzled images.
struct PackArgs {
  BwdArgs a;
  __nv_bfloat16* dopack;
  float* lsepack;
  float* deltapack;
  int dpad;  // 64 or 128 columns per packed row
};

__global__ void __launch_bounds__(128) bwd_pack_kernel(PackArgs pa) {
  __shared__ int s_th[kTile];
  const BwdArgs& a = pa.a;
  const PrefillView& pv = a.pv;
  const int tid = threadIdx.x;
  const long long tile = blockIdx.x;
  const long long n_self = (long long)pv.n_qtiles * pv.Hq;
  if (tile >= n_self && (pv.R == 0 || tile - n_self >= a.tile_base[pv.n_chunks * pv.Hkv])) return;
  const int th = a.rowpack[tile * kTile + tid];
  s_th[tid] = th;
  pa.lsepack[tile * kTile + tid] = th >= 0 ? -a.lse[th] * 1.4426950408889634f : -INFINITY;
  pa.deltapack[tile * kTile + tid] = th >= 0 ? -a.delta[th] * a.scale : 0.f;
  __syncthreads();
  const int upr = pa.dpad >> 3;
  uint8_t* odst = reinterpret_cast<uint8_t*>(pa.dopack) + tile * ((size_t)kTile * pa.dpad * 2);
  for (int i = tid; i < kTile * upr; i += 128) {
    const int row = i / upr, u = i - row * upr;
    const int rth = s_th[row];
    uint4 ov = make_uint4(0, 0, 0, 0);
    if (rth >= 0 && u * 8 < pv.D) ov = *reinterpret_cast<const uint4*>(a.dout + (long long)rth * pv.D + u * 8);
    *reinterpret_cast<uint4*>(odst + sw128_offset(kTile, row, u)) = ov;
  }
}

cudaError_t launch_bwd_pack(const BwdArgs& a, long long tiles, void* dopack, float* lsepack, float* deltapack, cudaStream_t st) {
  PackArgs pa;
  pa.a = a;
  pa.dopack = static_cast<__nv_bfloat16*>(dopack);
  pa.lsepack = lsepack;
  pa.deltapack = deltapack;
  pa.dpad = a.pv.D <= 64 ? 64 : 128;
  bwd_pack_kernel<<<(unsigned)tiles, 128, 0, st>>>(pa);
  return cudaGetLastError();
}

constexpr int kWsThreads = 512;  // 8 compute warps, MMA warp, producer warp (+2 idle), 4 dQ drain warps
constexpr int kWsRing = 4;       // Q/dO tiles in shared memory
constexpr int kStageRow = 272;   // bytes per staged dQ row: 64 floats + 16, so that eight lanes' 16-byte stores hit 32 banks

struct WsSmem {
  uint64_t st_full;    // S^T of the tile is in tensor memory (tcgen05.commit)
  uint64_t p_ready;    // P^T of the tile is in tensor memory, over the S^T columns its threads have read (8 warps)
  uint64_t ka_ready;   // K and V of the key block are in tensor memory as A operands (8 warps)
  uint64_t dpt_full;   // dP^T of the tile is in tensor memory
  uint64_t ds_ready;   // dS^T of the tile is in tensor memory and in shared memory (8 warps)
  uint64_t dq_done;    // dQ (and everything issued before it) of the tile is done
  uint64_t dq_free;    // the drain warps hold the tile's dQ in registers (4 warps)
  uint64_t kv_ready;
  uint64_t qdo_full[kWsRing];  // tile (Q, dO, row metadata) landed in the slot
  uint64_t qdo_free[kWsRing];  // dK of the tile is done and the drain warps have its row ids (1 + 4)
  uint32_t tmem_slot;
  uint32_t pad;
  __align__(16) int rowth[kWsRing][kTile];      // t*Hq+h of every row of the tile, -1 = padding row
  __align__(16) float lse2[kWsRing][kTile];     // -LSE in the log2 domain (-inf for padding rows)
  __align__(16) float delta_s[kWsRing][kTile];  // -rowsum(dO*O) / sqrt(D)
};
static_assert(sizeof(WsSmem) <= 8192, "control block must fit its reservation");

template <bool F16>
__global__ void __launch_bounds__(kWsThreads, 1) attn_bwd_ws_kernel(BwdArgs a) {
  constexpr int DPAD = 64;
  constexpr int TILE_BYTES = kTile * DPAD * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 320, COL_DQ = 384, COL_KA = 448, COL_VA = 480;
  extern __shared__ __align__(1024) uint8_t smem[];
  WsSmem& cb = *reinterpret_cast<WsSmem*>(smem);
  uint8_t* sK = smem + 8192;
  uint8_t* sV = sK + TILE_BYTES;
  // dQ staging of the drain warps.  It starts on the V image, which is dead once V sits in tensor memory (long before
  // the first dQ exists): 128 rows of kStageRow bytes for the copy-engine reductions.
  uint8_t* sStage = sV;
  constexpr int SLOT_BYTES = 2 * TILE_BYTES;  // ring slot: Q tile followed by dO tile
  uint8_t* sQ = sStage + kTile * kStageRow;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sdS = sQ + kWsRing * SLOT_BYTES;  // dS^T: 128 key rows x 128 query columns, bf16, two 64-column panels

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
    mbar_init(&cb.st_full, 1);
    mbar_init(&cb.p_ready, 8);
    mbar_init(&cb.ka_ready, 8);
    mbar_init(&cb.dpt_full, 1);
    mbar_init(&cb.ds_ready, 8);
    mbar_init(&cb.dq_done, 1);
    mbar_init(&cb.dq_free, 4);
    mbar_init(&cb.kv_ready, 1);
    for (int i = 0; i < kWsRing; ++i) { mbar_init(&cb.qdo_full[i], 1); mbar_init(&cb.qdo_free[i], 5); }
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
    // A warp takes the 32 rows of its tensor-memory lanes: dQ of the finished tile goes to registers at
    // once (the accumulator is then free for the next tile) and from there into the FP32 accumulator, in the
    // background of the next tile's math.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    const int quad = warp & 3;
    const uint32_t tlane = tmem + (uint32_t(quad * 32) << 16);
    const bool fixed = a.dq_fixed != nullptr;
    uint8_t* myrow = sStage + (quad * 32 + lane) * kStageRow;       // this thread's row
    for (int it = 0; it < n_iter; ++it) {
      const int slot = it % kWsRing;
      alive = warp_wait(&cb.qdo_full[slot], (it / kWsRing) & 1, a.status, alive);
      const int th = cb.rowth[slot][quad * 32 + lane];
      warp_arrive(&cb.qdo_free[slot]);
      alive = warp_wait(&cb.dq_done, it & 1, a.status, alive);
      tc_fence_after_sync();
      uint32_t v0[32], v1[32];
      tmem_ld32(tlane + COL_DQ, v0);
      tmem_ld32(tlane + COL_DQ + 32, v1);
      tmem_ld_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.dq_free);
      if (!fixed) {
        // Ordinary mode: the thread writes its row (one query, D floats) to shared memory and asks the copy engine to
        // add it to the row's place in the FP32 accumulator - one reduction of whole lines per row, carried by the
        // engine's own path to the L2 cache, so that neither the reductions nor a transposition pass through the
        // load/store pipe the compute warps need.  A thread only ever touches its own row, so it only has to wait
        // for its own previous reduction to have read the row before overwriting it.
        bulk_wait_group_read();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          *reinterpret_cast<uint4*>(myrow + u * 16) = make_uint4(v0[4 * u], v0[4 * u + 1], v0[4 * u + 2], v0[4 * u + 3]);
          *reinterpret_cast<uint4*>(myrow + 128 + u * 16) = make_uint4(v1[4 * u], v1[4 * u + 1], v1[4 * u + 2], v1[4 * u + 3]);
        }
        fence_async_smem();
        if (th >= 0 && alive) bulk_reduce_add_f32(a.dq_acc + (long long)th * D, myrow, (uint32_t)D * 4u);
        bulk_commit_group();
        continue;
      }
      // Deterministic mode: the same hand-over with 64-bit fixed-point values (32 fractional bits), whose integer sums
      // do not depend on the order in which the key blocks' contributions arrive; a row of 64 such values is twice the
      // size of the staging row, so it goes in two rounds of 32 dimensions.
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        bulk_wait_group_read();
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float x0 = __uint_as_float(p == 0 ? v0[2 * u] : v1[2 * u]), x1 = __uint_as_float(p == 0 ? v0[2 * u + 1] : v1[2 * u + 1]);
          *reinterpret_cast<longlong2*>(myrow + u * 16) = make_longlong2(__float2ll_rn(x0 * 4294967296.f), __float2ll_rn(x1 * 4294967296.f));
        }
        fence_async_smem();
        if (th >= 0 && alive && p * 32 < D)
          bulk_reduce_add_u64(a.dq_fixed + (long long)th * D + p * 32, myrow, (uint32_t)min(32, D - p * 32) * 8u);
        bulk_commit_group();
      }
    }
    bulk_wait_group();   // the engine has finished with this CTA's shared memory and its reductions are performed
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 9) {
      // ================================================================== producer
      // One thread asks the copy engine for the packed tiles: 16 KB of Q, 16 KB of dO and three 512-byte
      // metadata rows per tile, all contiguous in global memory, completion counted on the slot's barrier.
      if (lane == 0) {
        {  // stationary K and V images of the key block
          const size_t kvoff = ((size_t)kblock * pv.Hkv + g) * TILE_BYTES;
          mbar_arrive_expect_tx(&cb.kv_ready, 2 * TILE_BYTES);
          bulk_load(sK, reinterpret_cast<const uint8_t*>(a.kpack) + kvoff, TILE_BYTES, &cb.kv_ready);
          bulk_load(sV, reinterpret_cast<const uint8_t*>(a.vpack) + kvoff, TILE_BYTES, &cb.kv_ready);
        }
        const long long self_tiles = (long long)pv.n_qtiles * pv.Hq;
        const long long remote_tile0 = pv.R > 0 ? self_tiles + a.tile_base[c * pv.Hkv + g] : 0;
        for (int j = 0; j < n_iter; ++j) {
          const int b = j % kWsRing;
          long long tile;
          if (j < n_remote) {
            // The key blocks of a chunk walk the same expert list at the same time, each a couple of tiles
            // apart: a tile fetched by one of them is still in the L2 cache for the others, the dQ rows
            // they all add into stay there too, and no two of them add into the same rows at once.
            int jr = j + (kb * 2) % n_remote;
            if (jr >= n_remote) jr -= n_remote;
            tile = remote_tile0 + jr;
          } else {
            const int s = j - n_remote;
            const int hl = s / n_self, i = kb + (s - hl * n_self);
            tile = (long long)(kblock - kb + i) * pv.Hq + g * pv.G + hl;  // query tiles of a chunk are consecutive
          }
          if (j >= kWsRing && alive) alive = mbar_wait(&cb.qdo_free[b], ((j / kWsRing) - 1) & 1, a.status);
          mbar_arrive_expect_tx(&cb.qdo_full[b], 2 * TILE_BYTES + 3 * kTile * 4);
          bulk_load(sQ + b * SLOT_BYTES, reinterpret_cast<const uint8_t*>(a.qpack) + tile * TILE_BYTES, TILE_BYTES, &cb.qdo_full[b]);
          bulk_load(sdO + b * SLOT_BYTES, reinterpret_cast<const uint8_t*>(a.dopack) + tile * TILE_BYTES, TILE_BYTES, &cb.qdo_full[b]);
          bulk_load(cb.rowth[b], a.rowpack + tile * kTile, kTile * 4, &cb.qdo_full[b]);
          bulk_load(cb.lse2[b], a.lsepack + tile * kTile, kTile * 4, &cb.qdo_full[b]);
          bulk_load(cb.delta_s[b], a.deltapack + tile * kTile, kTile * 4, &cb.qdo_full[b]);
        }
      }
    } else if (warp == 8) {
      // ================================================================== MMA issue
      // Fixed order per tile n:  dV(n) | S^T(n+1) | dK(n) | dP^T(n+1) | dQ(n).  P^T lives in the columns of S^T and
      // dS^T in those of dP^T, so S^T of the next tile follows dV of this one and dP^T of the next tile follows dK of
      // this one in the (in-order) tensor pipe; every other awaited event depends only on instructions issued earlier
      // and has most of a tile of slack.  K and V, which never change, are A operands in tensor memory.
      const bool leader = bwd_elect_one();
      const uint32_t idesc_st = umma_idesc_16<F16>(128, 128, 0, 0);
      const uint32_t idesc_kv = umma_idesc_16<F16>(128, DPAD, 0, 1);   // A from tensor memory, B MN-major
      const uint32_t idesc_dq = umma_idesc_16<F16>(128, DPAD, 1, 1);   // A = dS^T tile (MN-major), B = K (MN-major)
      // Operand descriptors are built once; a descriptor is its base plus a constant (the start-address
      // field counts 16-byte units).
      const uint64_t k_mn = umma_desc_mnmajor(smem_u32(sK), kTile, 0, 0);
      const uint64_t q_km = umma_desc_kmajor(smem_u32(sQ), kTile, 0), q_mn = umma_desc_mnmajor(smem_u32(sQ), kTile, 0, 0);
      const uint64_t o_km = umma_desc_kmajor(smem_u32(sdO), kTile, 0), o_mn = umma_desc_mnmajor(smem_u32(sdO), kTile, 0, 0);
      const uint64_t s_mn = umma_desc_mnmajor(smem_u32(sdS), kTile, 0, 0);
      auto slot_u = [&](int n) { return (uint64_t)((n % kWsRing) * (SLOT_BYTES >> 4)); };
      auto issue_st = [&](int n) {
        if (alive) alive = mbar_wait(&cb.qdo_full[n % kWsRing], (n / kWsRing) & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
          const uint64_t su = slot_u(n);
#pragma unroll
          for (int kk = 0; kk < DPAD; kk += 16)  // K-major step: 16 elements = 32 bytes = 2 units
            umma_ts(tmem + COL_ST, tmem + COL_KA + (kk >> 1), q_km + su + (kk >> 3), idesc_st, kk > 0);
          umma_commit(&cb.st_full);
        }
        __syncwarp();
      };
      auto issue_dpt = [&](int n) {
        if (leader) {
          const uint64_t su = slot_u(n);
#pragma unroll
          for (int kk = 0; kk < DPAD; kk += 16)
            umma_ts(tmem + COL_DPT, tmem + COL_VA + (kk >> 1), o_km + su + (kk >> 3), idesc_st, kk > 0);
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
        const uint64_t su = slot_u(n);
        const uint32_t acc = n > 0;
        if (alive) alive = mbar_wait(&cb.p_ready, n & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kTile; kk += 16)  // dV += P^T dO; queries 0-63 at columns 0.., 64-127 at columns 64..; B MN-major step: 16 rows = 128 units
            umma_ts(tmem + COL_DV, tmem + COL_ST + (kk >> 6) * 64 + ((kk & 63) >> 1), o_mn + su + kk * 8, idesc_kv, acc | (kk > 0));
        }
        __syncwarp();
        if (n + 1 < n_iter) issue_st(n + 1);
        if (alive) alive = mbar_wait(&cb.ds_ready, n & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kTile; kk += 16)  // dK += dS^T Q; queries 0-63 at columns 128.., 64-127 at columns 192..
            umma_ts(tmem + COL_DK, tmem + COL_DPT + (kk >> 6) * 64 + ((kk & 63) >> 1), q_mn + su + kk * 8, idesc_kv, acc | (kk > 0));
          umma_commit(&cb.qdo_free[n % kWsRing]);  // the tile's Q and dO rows are no longer needed
        }
        __syncwarp();
        if (n + 1 < n_iter) issue_dpt(n + 1);
        if (n > 0 && alive) alive = mbar_wait(&cb.dq_free, (n - 1) & 1, a.status);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kTile; kk += 16)  // dQ = dS K; both MN-major: 16 key rows = 2048 bytes = 128 units
            umma_ss(tmem + COL_DQ, s_mn + kk * 8, k_mn + kk * 8, idesc_dq, kk > 0);
          umma_commit(&cb.dq_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ================================================================== compute (warps 0-7)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;  // key row of this thread
    const uint32_t tlane = tmem + (uint32_t(quad * 32) << 16);
    if (n_iter > 0) {
      // K (warps 0-3) and V (warps 4-7) of the key block into tensor memory as A operands: thread = key row, one
      // 32-bit column per pair of dimensions
      alive = warp_wait(&cb.kv_ready, 0, a.status, alive);
      const uint8_t* src = half == 0 ? sK : sV;
      uint32_t kv[32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 w = *reinterpret_cast<const uint4*>(src + sw128_offset(kTile, r, u));
        kv[4 * u] = w.x; kv[4 * u + 1] = w.y; kv[4 * u + 2] = w.z; kv[4 * u + 3] = w.w;
      }
      tmem_st32(tlane + (half == 0 ? COL_KA : COL_VA), kv);
      tmem_st_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.ka_ready);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int ms = it % kWsRing;
      // queries below qmin are masked for this key: all of them for a key that does not exist, the
      // earlier ones on the causal diagonal (tile of the key block itself)
      const bool diag = it >= n_remote && ((it - n_remote) % n_self) == 0;
      const int qmin = r >= nkeys ? kTile : (diag ? r : 0);
      const bool unmasked = __all_sync(0xFFFFFFFFu, qmin <= half * 64);
      alive = warp_wait(&cb.qdo_full[ms], (it / kWsRing) & 1, a.status, alive);  // the tile's metadata is in the slot
      alive = warp_wait(&cb.st_full, it & 1, a.status, alive);
      tc_fence_after_sync();
      float p[64];
      {
        uint32_t t0[32], t1[32];
        tmem_ld32(tlane + COL_ST + half * 64, t0);
        tmem_ld32(tlane + COL_ST + half * 64 + 32, t1);
        tmem_ld_wait();
        const float4* lse4 = reinterpret_cast<const float4*>(&cb.lse2[ms][half * 64]);
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {  // two elements per instruction for the scale-and-shift
          const float4 la = lse4[i >> 2], lb = lse4[8 + (i >> 2)];
          const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(t0[i]), __uint_as_float(t0[i + 1])), sc2, make_float2(la.x, la.y));
          const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(t0[i + 2]), __uint_as_float(t0[i + 3])), sc2, make_float2(la.z, la.w));
          const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(t1[i]), __uint_as_float(t1[i + 1])), sc2, make_float2(lb.x, lb.y));
          const float2 x3 = __ffma2_rn(make_float2(__uint_as_float(t1[i + 2]), __uint_as_float(t1[i + 3])), sc2, make_float2(lb.z, lb.w));
          p[i] = bwd_exp2(x0.x); p[i + 1] = bwd_exp2(x0.y); p[i + 2] = bwd_exp2(x1.x); p[i + 3] = bwd_exp2(x1.y);
          p[32 + i] = bwd_exp2(x2.x); p[32 + i + 1] = bwd_exp2(x2.y); p[32 + i + 2] = bwd_exp2(x3.x); p[32 + i + 3] = bwd_exp2(x3.y);
        }
      }
      if (!unmasked) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (half * 64 + i < qmin) p[i] = 0.f;
      }
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) pk[i] = pack16<F16>(p[2 * i], p[2 * i + 1]);
      tmem_st32(tlane + COL_ST + half * 64, pk);  // over the first 32 of this thread's own S^T columns, which it has read
      tmem_st_wait();
      tc_fence_before_sync();
      warp_arrive(&cb.p_ready);

      alive = warp_wait(&cb.dpt_full, it & 1, a.status, alive);
      tc_fence_after_sync();
      const float4* del4 = reinterpret_cast<const float4*>(&cb.delta_s[ms][half * 64]);
#pragma unroll
      for (int pc = 0; pc < 2; ++pc) {
        uint32_t t[32];
        tmem_ld32(tlane + COL_DPT + half * 64 + pc * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 dl = del4[pc * 8 + (i >> 2)];
          const float2 sc = make_float2(a.scale, a.scale);
          const float2 e0 = __ffma2_rn(make_float2(__uint_as_float(t[i]), __uint_as_float(t[i + 1])), sc, make_float2(dl.x, dl.y));
          const float2 e1 = __ffma2_rn(make_float2(__uint_as_float(t[i + 2]), __uint_as_float(t[i + 3])), sc, make_float2(dl.z, dl.w));
          const float2 d0 = __fmul2_rn(make_float2(p[pc * 32 + i], p[pc * 32 + i + 1]), e0);
          const float2 d1 = __fmul2_rn(make_float2(p[pc * 32 + i + 2], p[pc * 32 + i + 3]), e1);
          pk[pc * 16 + (i >> 1)] = pack16<F16>(d0.x, d0.y);
          pk[pc * 16 + (i >> 1) + 1] = pack16<F16>(d1.x, d1.y);
        }
      }
      // dS^T: over the first 32 of this thread's own dP^T columns for the dK product, and as a tile row
      // in shared memory for the dQ product (whose previous run must be over)
      tmem_st32(tlane + COL_DPT + half * 64, pk);
      if (it > 0) alive = warp_wait(&cb.dq_done, (it - 1) & 1, a.status, alive);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        *reinterpret_cast<uint4*>(sdS + sw128_offset(kTile, r, half * 8 + u)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
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
      for (int pc = 0; pc < 2; ++pc) {
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

cudaError_t launch_bwd_ws(const BwdArgs& a, cudaStream_t st) {
  const size_t smem = 8192 + (size_t)kTile * 64 * 2 * (1 + 2 * kWsRing) + (size_t)kTile * kStageRow + (size_t)kTile * kTile * 2;
  const auto kernel = a.pv.fp16 ? attn_bwd_ws_kernel<true> : attn_bwd_ws_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kernel<<<dim3(a.pv.n_qtiles, a.pv.Hkv), kWsThreads, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace moba
