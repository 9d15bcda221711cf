// Prefill attention forward on tcgen05 tensor cores with the LSE merge fused into the epilogue.
//
// Work decomposition (KV-stationary experts as in the reference, src/moba_opt/grouped_attention.py:76-90):
//   remote pass  a work item is a pair of 128-row tiles of one expert (chunk, kv head): the gathered rows
//                of any query head of the group that selected the chunk attend the whole chunk; the
//                normalised partial output (bf16) and its log2-sum-exp go to the fixed slot of the
//                (row, chunk) pair, so no atomics or tickets are needed and the merge order is fixed
//   self pass    a work item is a pair of consecutive 128-token query tiles of a chunk for one query
//                head: causal attention inside the own chunk, then the epilogue merges the row's remote
//                partials with the global-softmax rule of src/moba_opt/ops/merge.cu:113-151 and writes
//                O (bf16) and LSE (fp32) once
//
// One persistent CTA per SM walks its share of the items.  Inside a CTA the two tiles of an item are
// two "lanes" that share one stream of K/V tiles and are served by specialised warps:
//   warps 0-3   softmax of lane 0 (a thread owns a query row)      warp 8   issues every tcgen05.mma
//   warps 4-7   softmax of lane 1                                   warp 9   issues the bulk copies
// Per key tile and lane: S = Q K^T (accumulator in TMEM) -> the row is read with tcgen05.ld, masked,
// exponentiated in the exp2 domain against a running maximum that is only raised when it grew by more
// than 2^8 (the rescale of O in TMEM is then done by the row's own thread), P is written back into
// tensor memory over S as packed bf16 -> O += P V with P read from TMEM.  While one lane does its
// softmax the tensor pipe works for the other, and the copy engine runs K/V tiles ahead of both.
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// One in eight of the exponentials of a tile is computed on the FMA pipe instead of the exp2 unit, which two softmax
// warps per scheduler keep busy most of the time: iterations i (step 2) of the exponential loops with
// (i & MASK) == MASK use the polynomial.  Measured on the 4 x 32768-token configuration: remote pass 2.655 ms without,
// 2.554 ms with MASK 14 (one in eight), 2.547 with 6 (one in four, but the self pass 2 % slower), 2.699 with 2 (half).
#ifndef MOBA_FWD_POLY_MASK
#define MOBA_FWD_POLY_MASK 14
#endif
// 2^x for a pair of values, x in (-inf, 2^21], without the exp2 unit: x is clamped to -126, rounded to the nearest
// integer j with the magic-number add (j sits in the low mantissa bits of t), 2^f for f = x - j in [-0.5, 0.5] comes
// from a cubic (relative error 7.5e-5) and j is added to the exponent field.  Three packed adds, three packed
// multiply-adds, two maxima, two shifts and two integer adds for two results.
__device__ __forceinline__ float2 poly_exp2x2(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));
  const float2 jf = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(jf, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(f, make_float2(0.0551716611f, 0.0551716611f), make_float2(0.242611125f, 0.242611125f));
  p = __ffma2_rn(p, f, make_float2(0.693260968f, 0.693260968f));
  p = __ffma2_rn(p, f, make_float2(0.999928057f, 0.999928057f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

struct FwdArgs {
  PrefillView pv;
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

// One work item as every role sees it.
struct FwdItem {
  long long q_tile[2];  // packed query tile of each lane
  int n[2];             // key tiles the lane walks (0 = lane idle)
  int rows[2];          // valid rows of the lane's tile
  int first[2];         // SELF: first packed token of the tile; REMOTE: first rowlist entry of the tile
  int kblock0;          // packed key block holding the chunk's first keys
  int key_begin, key_end;
  int g, h;             // kv head; SELF: query head
};

template <bool SELF>
__device__ __forceinline__ bool fwd_decode_item(const FwdArgs& a, long long idx, FwdItem& it) {
  const PrefillView& pv = a.pv;
  if (SELF) {
    if (idx >= (long long)pv.n_self_pairs * pv.Hq) return false;
    const int pair = (int)(idx / pv.Hq);
    it.h = (int)(idx - (long long)pair * pv.Hq);
    it.g = it.h / pv.G;
    const int t0 = pv.self_pairs[pair];
    const int c = pv.qtile_chunk[t0];
    const int tok0 = pv.qtile_tok0[t0];
    it.key_begin = pv.chunk_start[c];
    it.key_end = pv.chunk_start[c + 1];
    const int i0 = (tok0 - it.key_begin) / kTile;
    it.kblock0 = t0 - i0;  // the tiles of a chunk have consecutive ids
    it.first[0] = tok0;
    it.first[1] = tok0 + kTile;
    it.rows[0] = min(kTile, it.key_end - tok0);
    it.rows[1] = max(0, min(kTile, it.key_end - tok0 - kTile));
    it.n[0] = i0 + 1;
    it.n[1] = it.rows[1] > 0 ? i0 + 2 : 0;
    it.q_tile[0] = (long long)t0 * pv.Hq + it.h;
    it.q_tile[1] = (long long)(t0 + 1) * pv.Hq + it.h;
    return true;
  } else {
    const int E = pv.n_chunks * pv.Hkv;
    const long long w = idx * 2;
    if (w >= a.tile_base[E]) return false;
    int lo = 0, hi = E;  // largest e with tile_base[e] <= w
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.tile_base[mid] <= w) lo = mid; else hi = mid;
    }
    const int e = lo, i = (int)(w - a.tile_base[e]);
    const int c = e / pv.Hkv;
    it.g = e - c * pv.Hkv;
    it.h = 0;
    const int start = a.seg_base[c * pv.Hq + it.g * pv.G] + i * kTile;
    const int end = a.seg_base[c * pv.Hq + (it.g + 1) * pv.G];
    it.key_begin = pv.chunk_start[c];
    it.key_end = pv.chunk_start[c + 1];
    const int nt = (it.key_end - it.key_begin + kTile - 1) / kTile;
    it.first[0] = start;
    it.first[1] = start + kTile;
    it.rows[0] = max(0, min(kTile, end - start));
    it.rows[1] = max(0, min(kTile, end - start - kTile));
    it.n[0] = it.rows[0] > 0 ? nt : 0;
    it.n[1] = it.rows[1] > 0 ? nt : 0;
    it.q_tile[0] = (long long)pv.n_qtiles * pv.Hq + w;
    it.q_tile[1] = it.q_tile[0] + 1;
    int qlo = 0, qhi = pv.n_qtiles - 1;  // first 128-token tile of chunk c (tile ids ascend with the chunk id)
    while (qlo < qhi) {
      const int mid = (qlo + qhi) >> 1;
      if (pv.qtile_chunk[mid] < c) qlo = mid + 1; else qhi = mid;
    }
    it.kblock0 = qlo;
    return true;
  }
}

// k-th item of this CTA: rounds alternate direction so that the sorted (heaviest first) item list is
// dealt out evenly.
__device__ __forceinline__ long long fwd_item_index(int k) {
  const long long G = gridDim.x;
  return (long long)k * G + ((k & 1) ? (G - 1 - blockIdx.x) : blockIdx.x);
}

constexpr int kFwdThreads = 384;  // warps 10 and 11 only complete the third warpgroup (register hand-over works per warpgroup)

template <int DPAD>
struct FwdCfg {
  static constexpr int TILE_BYTES = kTile * DPAD * 2;
  static constexpr int QBUFS = DPAD <= 64 ? 2 : 1;   // query tile buffers per lane
  static constexpr int STAGES = DPAD <= 64 ? 4 : 2;  // K/V ring depth (a stage = K tile + V tile)
  static constexpr int SMEM = 1024 + 2 * QBUFS * TILE_BYTES + STAGES * 2 * TILE_BYTES;
  static constexpr uint32_t TMEM_COLS = 512;
  // Tensor memory: S0 0-127, S1 128-255, O0/O1 from 256.  With D <= 64 P has columns of its own (384-511),
  // so the next S of a lane can be computed while its softmax still runs; with D = 128 all 512 columns are
  // taken and P overlays the first 64 columns of S.
  static constexpr bool OVERLAY = DPAD > 64;
  static constexpr uint32_t COL_S = 0;    // + lane * 128
  static constexpr uint32_t COL_O = 256;  // + lane * DPAD
  static constexpr uint32_t COL_P = OVERLAY ? 0 : 384;
  static constexpr uint32_t P_STRIDE = OVERLAY ? 128 : 64;
};

struct FwdSmem {
  uint64_t q_full[2][2], q_free[2][2];  // [lane][buffer]
  uint64_t s_full[2], s_free[2], p_ready[2], o_full[2], o_free[2];
  uint64_t kv_full[4], kv_free[4];
  uint32_t tmem_slot;
};
static_assert(sizeof(FwdSmem) <= 1024, "control block must fit its reservation");

template <int DPAD, bool SELF, bool F16>
__global__ void __launch_bounds__(kFwdThreads, 1) attn_fwd_kernel(FwdArgs a) {
  using Cfg = FwdCfg<DPAD>;
  constexpr int TILE_BYTES = Cfg::TILE_BYTES, QBUFS = Cfg::QBUFS, STAGES = Cfg::STAGES;
  constexpr int UPR = DPAD / 8;
  extern __shared__ __align__(1024) uint8_t smem[];
  FwdSmem& cb = *reinterpret_cast<FwdSmem*>(smem);
  uint8_t* sQ = smem + 1024;                      // [lane][buffer]
  uint8_t* sKV = sQ + 2 * QBUFS * TILE_BYTES;     // [stage]{K, V}

  const PrefillView& pv = a.pv;
  const int tid = threadIdx.x, warp = tid >> 5, lane_id = tid & 31;
  const int D = pv.D;

  if ((smem_u32(smem) & 1023u) != 0) {  // operand tiles need 1024-byte alignment for the swizzle
    if (tid == 0) atomicOr(a.status, kErrBadIndex);
    return;
  }
  if (tid == 0) {
    for (int l = 0; l < 2; ++l) {
      for (int b = 0; b < 2; ++b) { mbar_init(&cb.q_full[l][b], 1); mbar_init(&cb.q_free[l][b], 1); }
      mbar_init(&cb.s_full[l], 1);
      mbar_init(&cb.s_free[l], 4);
      mbar_init(&cb.p_ready[l], 4);
      mbar_init(&cb.o_full[l], 1);
      mbar_init(&cb.o_free[l], 4);
    }
    for (int s = 0; s < 4; ++s) { mbar_init(&cb.kv_full[s], 1); mbar_init(&cb.kv_free[s], 1); }
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&cb.tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = cb.tmem_slot;
  bool alive = true;

  // The softmax warpgroups keep a whole row of S in registers; the third warpgroup gives them its share.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  if (warp == 9) {
    // ================================================================== producer (one thread)
    if (lane_id == 0) {
      int use[2] = {0, 0};  // items each lane took part in so far
      int kvt = 0;          // K/V tiles fetched so far
      FwdItem it;
      for (int k = 0; fwd_decode_item<SELF>(a, fwd_item_index(k), it); ++k) {
#pragma unroll
        for (int l = 0; l < 2; ++l) {
          if (it.n[l] == 0) continue;
          const int u = use[l]++, b = u % QBUFS;
          if (u >= QBUFS && alive) alive = mbar_wait(&cb.q_free[l][b], ((u / QBUFS) - 1) & 1, a.status);
          mbar_arrive_expect_tx(&cb.q_full[l][b], TILE_BYTES);
          bulk_load(sQ + (l * QBUFS + b) * TILE_BYTES, a.qpack + it.q_tile[l] * TILE_BYTES, TILE_BYTES, &cb.q_full[l][b]);
        }
        const int n = max(it.n[0], it.n[1]);
        const size_t kv_step = (size_t)pv.Hkv * TILE_BYTES;  // next key block of the same kv head
        const size_t kv0 = ((size_t)it.kblock0 * pv.Hkv + it.g) * TILE_BYTES;
        for (int j = 0; j < n; ++j, ++kvt) {
          const int s = kvt % STAGES;
          if (kvt >= STAGES && alive) alive = mbar_wait(&cb.kv_free[s], ((kvt / STAGES) - 1) & 1, a.status);
          mbar_arrive_expect_tx(&cb.kv_full[s], 2 * TILE_BYTES);
          bulk_load(sKV + s * 2 * TILE_BYTES, a.kpack + kv0 + j * kv_step, TILE_BYTES, &cb.kv_full[s]);
          bulk_load(sKV + s * 2 * TILE_BYTES + TILE_BYTES, a.vpack + kv0 + j * kv_step, TILE_BYTES, &cb.kv_full[s]);
        }
      }
      // no copy may be in flight when the CTA exits: the last stages are consumed by the MMA warp in
      // normal operation; after a timeout wait for them here
      if (!alive)
        for (int s = 0; s < STAGES && s < kvt; ++s) mbar_wait(&cb.kv_full[(kvt - 1 - s) % STAGES], (((kvt - 1 - s) / STAGES)) & 1, nullptr);
    }
  } else if (warp == 8) {
    // ================================================================== MMA issue
    // The whole warp walks the schedule (warp-uniform control flow and operands); one elected lane
    // issues.  The order is fixed: per key tile, lane 0 then lane 1, each "next S" and "P V".  Every
    // awaited event depends only on instructions issued earlier in this order, and each has about a
    // tile of slack, so waiting in a fixed order costs nothing.
    const bool leader = elect_one_sync();
    const uint32_t idesc_s = umma_idesc_16<F16>(128, 128, 0, 0);
    const uint32_t idesc_o = umma_idesc_16<F16>(128, DPAD, 0, 1);
    // Operand descriptors are built once; a descriptor is its base plus a constant (the start-address
    // field counts 16-byte units).
    const uint64_t qd0 = umma_desc_kmajor(smem_u32(sQ), kTile, 0);
    const uint64_t kd0 = umma_desc_kmajor(smem_u32(sKV), kTile, 0);
    const uint64_t vd0 = umma_desc_mnmajor(smem_u32(sKV + TILE_BYTES), kTile, 0, 0);
    constexpr uint32_t STAGE_U = (2 * TILE_BYTES) >> 4, QBUF_U = TILE_BYTES >> 4;
    int use_s[2] = {0, 0};  // items whose first S was issued, per lane (query buffer and its phase)
    int use_p[2] = {0, 0};  // items whose P V products are all issued
    int ts[2] = {0, 0};     // S products issued per lane (phase of s_free)
    int tp[2] = {0, 0};     // P V products issued per lane (phase of p_ready)
    int kvt0 = 0;           // K/V tiles of all earlier items
    bool pre[2] = {false, false};  // first S of the current item was issued while the previous item ran

    // S of a lane's next tile: Q buffer qb, K/V ring index kv; last = the item's last S for the lane
    auto issue_s = [&](int l, int qb, int kv, bool last) {
      if (!Cfg::OVERLAY && ts[l] > 0 && alive) alive = mbar_wait(&cb.s_free[l], (ts[l] - 1) & 1, a.status);
      if (alive) alive = mbar_wait(&cb.kv_full[kv % STAGES], (kv / STAGES) & 1, a.status);
      tc_fence_after_sync();
      if (leader) {
        const uint32_t tS = tmem + Cfg::COL_S + l * 128;
        const uint64_t kd = kd0 + (uint64_t)((kv % STAGES) * STAGE_U);
        const uint64_t qd = qd0 + (uint64_t)((l * QBUFS + qb) * QBUF_U);
#pragma unroll
        for (int kk = 0; kk < DPAD; kk += 16) {  // K-major step: 16 elements = 32 bytes = 2 units; 64 elements per panel
          constexpr uint32_t PANEL_U = (kTile * 128) >> 4;
          const uint32_t off = (kk >> 6) * PANEL_U + ((kk & 63) >> 3);
          umma_ss(tS, qd + off, kd + off, idesc_s, kk > 0);
        }
        umma_commit(&cb.s_full[l]);
        if (last) umma_commit(&cb.q_free[l][qb]);
      }
      __syncwarp();
      ++ts[l];
    };

    FwdItem cur, nxt;
    bool has = fwd_decode_item<SELF>(a, fwd_item_index(0), cur);
    for (int k = 0; has; ++k) {
      const bool has_next = fwd_decode_item<SELF>(a, fwd_item_index(k + 1), nxt);
      const int n = max(cur.n[0], cur.n[1]);
      bool pre_next[2] = {false, false};
#pragma unroll
      for (int l = 0; l < 2; ++l) {
        if (cur.n[l] > 0 && !pre[l]) {
          const int qb = use_s[l] % QBUFS;
          if (alive) alive = mbar_wait(&cb.q_full[l][qb], (use_s[l] / QBUFS) & 1, a.status);
          issue_s(l, qb, kvt0, cur.n[l] == 1);
          ++use_s[l];
        }
      }
      for (int j = 0; j < n; ++j) {
#pragma unroll
        for (int l = 0; l < 2; ++l) {
          if (j >= cur.n[l]) continue;
          auto next_s = [&]() {
            if (j + 1 < cur.n[l]) {
              issue_s(l, (use_s[l] - 1) % QBUFS, kvt0 + j + 1, j + 2 == cur.n[l]);
            } else if (has_next && nxt.n[l] > 0 && j > n - STAGES) {
              // first S of the lane's next item; its K tile can only be in the ring once the tile that
              // used the stage before was released, which happened in an earlier iteration if j > n - STAGES
              const int qb = use_s[l] % QBUFS;
              if (alive) alive = mbar_wait(&cb.q_full[l][qb], (use_s[l] / QBUFS) & 1, a.status);
              issue_s(l, qb, kvt0 + n, nxt.n[l] == 1);
              ++use_s[l];
              pre_next[l] = true;
            }
          };
          if (!Cfg::OVERLAY) next_s();
          // O += P V: P of the tile is in tensor memory, V in its ring stage
          if (alive) alive = mbar_wait(&cb.p_ready[l], tp[l] & 1, a.status);
          if (j == 0 && use_p[l] > 0 && alive) alive = mbar_wait(&cb.o_free[l], (use_p[l] - 1) & 1, a.status);
          tc_fence_after_sync();
          if (leader) {
            const uint32_t tP = tmem + Cfg::COL_P + l * Cfg::P_STRIDE, tO = tmem + Cfg::COL_O + l * DPAD;
            const uint64_t vd = vd0 + (uint64_t)(((kvt0 + j) % STAGES) * STAGE_U);
#pragma unroll
            for (int kk = 0; kk < kTile; kk += 16)  // MN-major step: 16 rows = 2048 bytes = 128 units
              umma_ts(tO, tP + kk / 2, vd + kk * 8, idesc_o, (j > 0) | (kk > 0));
            umma_commit(&cb.o_full[l]);
          }
          __syncwarp();
          ++tp[l];
          if (Cfg::OVERLAY) next_s();  // P lives in S's columns: the next S may only follow this P V
        }
        if (leader) umma_commit(&cb.kv_free[(kvt0 + j) % STAGES]);  // every lane that walks the stage has issued its P V
        __syncwarp();
      }
#pragma unroll
      for (int l = 0; l < 2; ++l) {
        if (cur.n[l] > 0) ++use_p[l];
        pre[l] = pre_next[l];
      }
      kvt0 += n;
      cur = nxt;
      has = has_next;
    }
  }
  } else {
    // ================================================================== softmax + epilogue, one lane per warpgroup
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int l = warp >> 2;
    const int row = tid & 127;
    const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + Cfg::COL_S + l * 128;
    const uint32_t tO = tmem + lane_off + Cfg::COL_O + l * DPAD;
    const uint32_t tP = tmem + lane_off + Cfg::COL_P + l * Cfg::P_STRIDE;
    int tc = 0;  // tiles this lane has processed
    FwdItem it;
    for (int k = 0; fwd_decode_item<SELF>(a, fwd_item_index(k), it); ++k) {
      const int n = it.n[l];
      if (n == 0) continue;
      int row_id = -1;  // SELF: t*Hq+h of this thread's row; REMOTE: slot id
      const int tok = it.first[l] + row;
      if (row < it.rows[l]) {
        if (SELF) {
          row_id = tok * pv.Hq + it.h;
        } else {
          row_id = a.rowlist[it.first[l] + row];
          if (row_id < 0 || row_id / pv.R >= pv.T * pv.Hq) { atomicOr(a.status, kErrBadIndex); row_id = -1; }
        }
      }
      const int key_end = SELF ? it.first[l] + it.rows[l] : it.key_end;  // causal: nothing past the tile's last token
      float m_used = 0.f, l_run = 0.f;
      for (int j = 0; j < n; ++j, ++tc) {
        const int k0 = it.key_begin + j * kTile;
        int klimit = key_end - k0;                     // keys of the tile that exist
        if (SELF) klimit = min(klimit, tok - k0 + 1);  // causal inside the own chunk
        const bool need_mask = __any_sync(0xFFFFFFFFu, klimit < kTile);
        if (alive) alive = mbar_wait(&cb.s_full[l], tc & 1, a.status);
        tc_fence_after_sync();
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld32(tS, s0);
        tmem_ld32(tS + 32, s1);
        tmem_ld32(tS + 64, s2);
        tmem_ld32(tS + 96, s3);
        tmem_ld_wait();
        if (!Cfg::OVERLAY) {  // S is in registers: the tensor pipe may compute the lane's next S
          tc_fence_before_sync();
          __syncwarp();
          if (lane_id == 0) mbar_arrive(&cb.s_free[l]);
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i >= klimit) s0[i] = 0xFF800000u;
            if (32 + i >= klimit) s1[i] = 0xFF800000u;
            if (64 + i >= klimit) s2[i] = 0xFF800000u;
            if (96 + i >= klimit) s3[i] = 0xFF800000u;
          }
        }
        float mx0 = __uint_as_float(s0[0]), mx1 = __uint_as_float(s1[0]), mx2 = __uint_as_float(s2[0]), mx3 = __uint_as_float(s3[0]);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          mx0 = max3(mx0, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
          mx1 = max3(mx1, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
          mx2 = max3(mx2, __uint_as_float(s2[i]), __uint_as_float(s2[i + 1]));
          mx3 = max3(mx3, __uint_as_float(s3[i]), __uint_as_float(s3[i + 1]));
        }
        const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2;
        // The maximum in use is raised only when the row's maximum outgrew it by 2^8; P stays below 2^8.
        float alpha = 1.f;
        bool raise = false;
        if (j == 0) {
          m_used = m_tile;
        } else if (m_tile > m_used + 8.f) {
          alpha = fast_exp2(m_used - m_tile);
          m_used = m_tile;
          raise = true;
        }
        // P V of the previous tile must have landed before O is rescaled or its P is overwritten; on the usual
        // path (no rescale) the wait sits right before the first P store, under the first half of the exponentials
        const bool rescale = j > 0 && __any_sync(0xFFFFFFFFu, raise);
        if (rescale) {
          if (alive) alive = mbar_wait(&cb.o_full[l], (tc - 1) & 1, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int pc = 0; pc < DPAD / 32; ++pc) {
            uint32_t o[32];
            tmem_ld32(tO + pc * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + pc * 32, o);
          }
          l_run *= alpha;
        }
        // two elements per instruction where the hardware has a packed form (scale-and-shift, row sum)
        float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2), neg2 = make_float2(-m_used, -m_used);
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 xa = __ffma2_rn(make_float2(__uint_as_float(s0[i]), __uint_as_float(s0[i + 1])), sc2, neg2);
          const float2 xb = __ffma2_rn(make_float2(__uint_as_float(s1[i]), __uint_as_float(s1[i + 1])), sc2, neg2);
          const bool soft = MOBA_FWD_POLY_MASK != 0 && (i & MOBA_FWD_POLY_MASK) == MOBA_FWD_POLY_MASK;   // known at compile time: the loop is unrolled
          const float2 pa = soft ? poly_exp2x2(xa) : make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
          const float2 pb = soft ? poly_exp2x2(xb) : make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
          sum0 = __fadd2_rn(sum0, pa);
          sum1 = __fadd2_rn(sum1, pb);
          pk[i >> 1] = pack16<F16>(pa.x, pa.y);
          pk[16 + (i >> 1)] = pack16<F16>(pb.x, pb.y);
        }
        if (j > 0 && !rescale && alive) alive = mbar_wait(&cb.o_full[l], (tc - 1) & 1, a.status);
        tmem_st32(tP, pk);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 xa = __ffma2_rn(make_float2(__uint_as_float(s2[i]), __uint_as_float(s2[i + 1])), sc2, neg2);
          const float2 xb = __ffma2_rn(make_float2(__uint_as_float(s3[i]), __uint_as_float(s3[i + 1])), sc2, neg2);
          const bool soft = MOBA_FWD_POLY_MASK != 0 && (i & MOBA_FWD_POLY_MASK) == MOBA_FWD_POLY_MASK;   // known at compile time: the loop is unrolled
          const float2 pa = soft ? poly_exp2x2(xa) : make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
          const float2 pb = soft ? poly_exp2x2(xb) : make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
          sum0 = __fadd2_rn(sum0, pa);
          sum1 = __fadd2_rn(sum1, pb);
          pk[i >> 1] = pack16<F16>(pa.x, pa.y);
          pk[16 + (i >> 1)] = pack16<F16>(pb.x, pb.y);
        }
        tmem_st32(tP + 32, pk);
        l_run += (sum0.x + sum0.y) + (sum1.x + sum1.y);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane_id == 0) mbar_arrive(&cb.p_ready[l]);
      }

      // ---- epilogue: O of the row leaves tensor memory, then the lane's accumulator is free again
      if (alive) alive = mbar_wait(&cb.o_full[l], (tc - 1) & 1, a.status);
      tc_fence_after_sync();
      float o_acc[DPAD];
#pragma unroll
      for (int pc = 0; pc < DPAD / 32; ++pc) {
        uint32_t o[32];
        tmem_ld32(tO + pc * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[pc * 32 + i] = __uint_as_float(o[i]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane_id == 0) mbar_arrive(&cb.o_free[l]);
      if (row_id < 0 || !alive) continue;
      if (!SELF) {
        const float inv = 1.f / l_run;
        __nv_bfloat16* dst = a.part_o + (long long)row_id * D;
#pragma unroll
        for (int u = 0; u < UPR; ++u) {
          if (u * 8 < D)
            *reinterpret_cast<uint4*>(dst + u * 8) =
                make_uint4(pack16<F16>(o_acc[u * 8] * inv, o_acc[u * 8 + 1] * inv), pack16<F16>(o_acc[u * 8 + 2] * inv, o_acc[u * 8 + 3] * inv),
                           pack16<F16>(o_acc[u * 8 + 4] * inv, o_acc[u * 8 + 5] * inv), pack16<F16>(o_acc[u * 8 + 6] * inv, o_acc[u * 8 + 7] * inv));
        }
        a.part_lse[row_id] = m_used + log2f(l_run);
      } else {
        // global-softmax merge of the self branch with the row's remote partials (fixed slot order).  The loads are
        // issued in batches that do not depend on each other - the selection and the partial LSEs of four slots, then
        // the partial output rows of two slots - so that a row costs a few trips to memory, not three per slot.
        const int R = pv.R;
        const float l2_self = m_used + log2f(l_run);
        float big = l2_self;
        const int* mysel = a.sel + (long long)row_id * R;
        const float* mylse = a.part_lse + (long long)row_id * R;
        int nsel = 0;  // sel is ascending with -1 padding at the end: the chosen slots are the first nsel
        for (int s0 = 0; s0 < R; s0 += 4) {
          int c[4];
          float e[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            c[i] = s0 + i < R ? mysel[s0 + i] : -1;
            e[i] = s0 + i < R ? mylse[s0 + i] : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (c[i] >= 0) { big = fmaxf(big, e[i]); ++nsel; }
          }
        }
        const float w_self = fast_exp2(l2_self - big);
        float z = w_self;
        const float f_self = w_self / l_run;
#pragma unroll
        for (int d = 0; d < DPAD; ++d) o_acc[d] *= f_self;
        for (int s0 = 0; s0 < nsel; s0 += 2) {
          uint4 raw[2][UPR];
          float w[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const bool on = s0 + i < nsel;
            const long long slot = (long long)row_id * R + (on ? s0 + i : s0);
            w[i] = on ? mylse[on ? s0 + i : s0] : -INFINITY;
            const __nv_bfloat16* src = a.part_o + slot * D;
#pragma unroll
            for (int u = 0; u < UPR; ++u)
              raw[i][u] = (on && u * 8 < D) ? *reinterpret_cast<const uint4*>(src + u * 8) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float wi = fast_exp2(w[i] - big);   // 0 for the slot that is not there
            z += wi;
#pragma unroll
            for (int u = 0; u < UPR; ++u) {
              const uint32_t wv[4] = {raw[i][u].x, raw[i][u].y, raw[i][u].z, raw[i][u].w};
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                const float2 pv2 = unpack16<F16>(wv[x]);
                o_acc[u * 8 + 2 * x] = fmaf(wi, pv2.x, o_acc[u * 8 + 2 * x]);
                o_acc[u * 8 + 2 * x + 1] = fmaf(wi, pv2.y, o_acc[u * 8 + 2 * x + 1]);
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
                make_uint4(pack16<F16>(o_acc[u * 8] * inv, o_acc[u * 8 + 1] * inv), pack16<F16>(o_acc[u * 8 + 2] * inv, o_acc[u * 8 + 3] * inv),
                           pack16<F16>(o_acc[u * 8 + 4] * inv, o_acc[u * 8 + 5] * inv), pack16<F16>(o_acc[u * 8 + 6] * inv, o_acc[u * 8 + 7] * inv));
        }
        a.lse[row_id] = (big + log2f(z)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, Cfg::TMEM_COLS);
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

template <int DPAD, bool SELF, bool F16>
static cudaError_t launch_fwd_as(const FwdArgs& a, long long items, cudaStream_t st) {
  const int smem = FwdCfg<DPAD>::SMEM;
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<DPAD, SELF, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const int sms = sm_count();
  if (sms <= 0) return cudaErrorUnknown;
  const int grid = (int)(items < sms ? (items < 1 ? 1 : items) : sms);
  attn_fwd_kernel<DPAD, SELF, F16><<<grid, kFwdThreads, smem, st>>>(a);
  return cudaGetLastError();
}
template <int DPAD, bool SELF>
static cudaError_t launch_fwd(const FwdArgs& a, long long items, cudaStream_t st) {
  return a.pv.fp16 ? launch_fwd_as<DPAD, SELF, true>(a, items, st) : launch_fwd_as<DPAD, SELF, false>(a, items, st);
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
    // every expert has at most ceil(rows/128) + 1 tiles; half of the bound is the number of tile pairs
    const long long bound = ((long long)(slots / kTile) + 2ll * d->num_chunks * d->hkv + 1) / 2;
    prof_begin(kProfFwdRemote, st);
    e = wide ? launch_fwd<128, false>(a, bound, st) : launch_fwd<64, false>(a, bound, st);
    prof_end(kProfFwdRemote, st);
    if (e != cudaSuccess) return MOBA_ERR_CUDA;
  }
  const long long items = (long long)d->num_self_pairs * d->hq;
  prof_begin(kProfFwdSelf, st);
  e = wide ? launch_fwd<128, true>(a, items, st) : launch_fwd<64, true>(a, items, st);
  prof_end(kProfFwdSelf, st);
  return e == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
