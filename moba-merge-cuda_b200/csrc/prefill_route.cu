// Prefill routing: chunk mean-pool of K, FP32 gate q . mean, deterministic top-k, and the
// per-expert query lists.  Replaces the torch-op routing and packing of the reference
// (src/moba_opt/grouped_attention.py:48-94): nothing of size [F, Hq, T] is materialised, there
// is no host synchronisation, and every list is produced in a fixed order (head in group, token).
//
// Passes (all on one stream, four launches):
//   1. chunk_mean_kernel     partial sums of K over 256-token slices of a chunk (one CTA each, so the pass
//                            has enough loads in flight to run at memory speed); the CTA that finishes a
//                            (chunk, kv head) last adds the slices in slice order and writes the mean
//   2. gate_topk_kernel      per (token, q head): FP32 scores against the earlier chunks of the same
//                            sequence, top-R with "lowest chunk wins ties", sel[T,Hq,R] ascending;
//                            per (query tile, q head, chunk) selection counts
//   3. segment_scan_kernel   per (chunk, q head): exclusive scan of the counts over query tiles; the block
//                            that finishes last turns the totals into segment bases and per-expert tile bases
//   4. fill_kernel           writes slot ids into rowlist at base + tile offset + rank in tile
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

constexpr int kCandBatch = 32;   // candidate means staged in shared memory per pass
constexpr int kMeanRows = 256;   // tokens per CTA of the mean pass

// --------------------------------------------------------------------------- 1. chunk means
// grid (chunk, kv head, slice).  part [n_chunks*Hkv][splits][D] FP32, tickets [n_chunks*Hkv] zero on entry (and
// left zero).  Every sum has a fixed order - rows of a slice by (row mod rows-per-pass, then pass), slices
// ascending - so the means are bit-repeatable whichever CTA happens to finish last.
__global__ void __launch_bounds__(256) chunk_mean_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ k, float* part,
                                                         float* __restrict__ means, int* tickets, int round_bf16, int splits) {
  extern __shared__ float s_part[];  // [rows_per_iter][D]
  __shared__ int s_last;
  const int c = blockIdx.x, g = blockIdx.y, sl = blockIdx.z;
  const int c0 = pv.chunk_start[c], c1 = pv.chunk_start[c + 1];
  const int t0 = min(c1, c0 + sl * kMeanRows), t1 = min(c1, t0 + kMeanRows);
  const int upr = pv.D >> 3;
  const int rpi = 256 / upr;
  const int ri = threadIdx.x / upr, u = threadIdx.x - ri * upr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const bool f16 = pv.fp16 != 0;
  if (ri < rpi) {
    const __nv_bfloat16* base = k + (long long)g * pv.k_sh + u * 8;
    auto add = [&](const uint4& raw) {
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = f16 ? unpack16<true>(w[i]) : unpack16<false>(w[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    };
    int t = t0 + ri;
    for (; t + 3 * rpi < t1; t += 4 * rpi) {   // four rows in flight per thread
      uint4 raw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) raw[j] = *reinterpret_cast<const uint4*>(base + (long long)(t + j * rpi) * pv.k_st);
#pragma unroll
      for (int j = 0; j < 4; ++j) add(raw[j]);
    }
    for (; t < t1; t += rpi) add(*reinterpret_cast<const uint4*>(base + (long long)t * pv.k_st));
#pragma unroll
    for (int i = 0; i < 8; ++i) s_part[ri * pv.D + u * 8 + i] = acc[i];
  }
  __syncthreads();
  const long long seg = (long long)c * pv.Hkv + g;
  for (int d = threadIdx.x; d < pv.D; d += 256) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += s_part[r * pv.D + d];
    part[(seg * splits + sl) * pv.D + d] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&tickets[seg], 1) == splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int d = threadIdx.x; d < pv.D; d += 256) {
    float s = 0.f;
    for (int j = 0; j < splits; ++j) s += __ldcg(part + (seg * splits + j) * pv.D + d);
    float m = s / (float)(c1 - c0);
    if (round_bf16) m = round16(m, f16);   // to the format of the inputs
    means[seg * pv.D + d] = m;
  }
  if (threadIdx.x == 0) tickets[seg] = 0;
}

// --------------------------------------------------------------------------- 2. gate + top-k
// Two FP32 multiply-adds per instruction (packed pairs of lanes 2j, 2j+1 of the dot product).
__device__ __forceinline__ void fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
// A pair of FP32 values as one 64-bit register pair and back: register moves at most, no arithmetic.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float sum2(unsigned long long v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}

// grid (query tile, query head).  A group of LPR lanes shares four query rows: each lane keeps DD of the DD * LPR
// (padded) head dimensions of all four rows as FP32 in registers for the whole launch, converted from the 16-bit inputs once.  The
// candidate means sit in shared memory as FP32; one 16-byte broadcast load feeds eight packed FMAs (four rows), which
// is what keeps the shared-memory pipe below the FMA pipe - with one row per lane it is the limit.  The four partial
// sums of a lane are combined across the group by a butterfly of three (LPR = 4) or four (LPR = 8) shuffles that
// leaves every lane with the complete score of one row, for which it then keeps the running top-R.
//   LPR = 4: 128 threads, 32 rows per warp.  LPR = 8: 256 threads, 16 rows per warp.
template <int RT, int DD, int LPR>
__global__ void __launch_bounds__(32 * LPR) gate_topk_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ q,
                                                             const float* __restrict__ means, int* __restrict__ sel,
                                                             int* __restrict__ cnt) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int DP = DD * LPR;
  constexpr int NT = 32 * LPR;
  constexpr int RPW = 128 / LPR;           // rows per warp
  const int D = pv.D, R = pv.R;
  constexpr int qrow_bytes = DP * 2 + 16;  // padded so that the rows of a warp start in different banks
  float4* s_means = reinterpret_cast<float4*>(smem);                      // [kCandBatch][DP / 4], 16-byte units interleaved by lane of the group
  uint8_t* s_q = smem + (size_t)kCandBatch * DP * 4;                      // [128][qrow_bytes]
  int* s_cnt = reinterpret_cast<int*>(s_q + (size_t)kTile * qrow_bytes);  // [ncand]

  const int tile = blockIdx.x, h = blockIdx.y, g = h / pv.G;
  const int c = pv.qtile_chunk[tile];
  const int tok0 = pv.qtile_tok0[tile];
  const int ncand = pv.chunk_local[c];
  const int c0 = c - ncand;
  const int nrows = min(kTile, pv.chunk_start[c + 1] - tok0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = lane % LPR;
  const int row0 = warp * RPW + (lane / LPR) * 4;                         // first of the group's four rows
  const int row = row0 + (part & 1) * 2 + ((part >> 1) & 1);              // the row whose score this lane ends up with
  const bool owner = row < nrows && part < 4;
  int* out = sel + ((long long)(tok0 + row) * pv.Hq + h) * R;
  if (ncand == 0) {  // first chunk of a sequence: nothing to route to
    if (owner)
      for (int s = 0; s < R; ++s) out[s] = -1;
    return;
  }
  const int upr = D >> 3;
  for (int i = tid; i < nrows * (DP / 8); i += NT) {
    const int r = i / (DP / 8), u = i - r * (DP / 8);
    const __nv_bfloat16* src = q + (long long)(tok0 + r) * pv.q_st + (long long)h * pv.q_sh;
    cp_async16(smem_u32(s_q + (size_t)r * qrow_bytes + u * 16), u < upr ? src + u * 8 : src, u < upr);  // zero fill beyond D
  }
  cp_async_commit();
  for (int i = tid; i < ncand; i += NT) s_cnt[i] = 0;

  unsigned long long qp[4][DD / 2];
  float topv[RT];
  int topi[RT];
#pragma unroll
  for (int i = 0; i < RT; ++i) { topv[i] = -INFINITY; topi[i] = -1; }

  for (int cb = 0; cb < ncand; cb += kCandBatch) {
    const int nb = min(kCandBatch, ncand - cb);
    if (cb) __syncthreads();  // previous batch consumed
    for (int i = tid; i < nb * (DP / 4); i += NT) {
      const int ci = i / (DP / 4), f4 = i - ci * (DP / 4);
      const int d0 = f4 * 4;
      float4 mv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d0 < D) mv = *reinterpret_cast<const float4*>(means + ((long long)(c0 + cb + ci) * pv.Hkv + g) * D + d0);
      s_means[ci * (DP / 4) + ((d0 % DD) >> 2) * LPR + d0 / DD] = mv;
    }
    if (cb == 0) {
      cp_async_wait<0>();
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint8_t* qrow = s_q + (size_t)(row0 + j) * qrow_bytes + part * (DD * 2);
#pragma unroll
        for (int u = 0; u < DD / 8; ++u) {
          uint4 raw = make_uint4(0u, 0u, 0u, 0u);
          if (row0 + j < nrows) raw = *reinterpret_cast<const uint4*>(qrow + u * 16);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          if (pv.fp16) {   // one uniform branch per 16 bytes, not a select per value
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = unpack16<true>(w[i]); qp[j][u * 4 + i] = pack2(f.x, f.y); }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = unpack16<false>(w[i]); qp[j][u * 4 + i] = pack2(f.x, f.y); }
          }
        }
      }
    } else {
      __syncthreads();
    }
    for (int ci = 0; ci < nb; ++ci) {
      // a 16-byte shared load lands in two aligned register pairs, which are the packed operands as they are
      const ulonglong2* m = reinterpret_cast<const ulonglong2*>(s_means + ci * (DP / 4) + part);
      unsigned long long a0 = 0ull, a1 = 0ull, a2 = 0ull, a3 = 0ull;
#pragma unroll
      for (int jj = 0; jj < DD / 4; ++jj) {
        const ulonglong2 mv = m[jj * LPR];
        fma2(a0, qp[0][2 * jj], mv.x); fma2(a1, qp[1][2 * jj], mv.x); fma2(a2, qp[2][2 * jj], mv.x); fma2(a3, qp[3][2 * jj], mv.x);
        fma2(a0, qp[0][2 * jj + 1], mv.y); fma2(a1, qp[1][2 * jj + 1], mv.y); fma2(a2, qp[2][2 * jj + 1], mv.y);
        fma2(a3, qp[3][2 * jj + 1], mv.y);
      }
      const float s0 = sum2(a0), s1 = sum2(a1), s2 = sum2(a2), s3 = sum2(a3);
      // butterfly over the group: lanes with an odd index keep rows 2 and 3, then lanes 2, 3 (mod 4) the second of the pair
      const bool odd = part & 1, upper = part & 2;
      const float t0 = (odd ? s2 : s0) + __shfl_xor_sync(0xFFFFFFFFu, odd ? s0 : s2, 1);
      const float t1 = (odd ? s3 : s1) + __shfl_xor_sync(0xFFFFFFFFu, odd ? s1 : s3, 1);
      float score = (upper ? t1 : t0) + __shfl_xor_sync(0xFFFFFFFFu, upper ? t0 : t1, 2);
      if (LPR == 8) score += __shfl_xor_sync(0xFFFFFFFFu, score, 4);   // both lanes of the pair get the same bits
      // strict '>' keeps the earlier (lower) chunk on exact ties; infinities never enter
      if (score > topv[RT - 1] && score < INFINITY) {
        float v = score;
        int idx = cb + ci;
#pragma unroll
        for (int i = 0; i < RT; ++i) {
          if (v > topv[i]) {
            const float tv = topv[i]; const int ti = topi[i];
            topv[i] = v; topi[i] = idx; v = tv; idx = ti;
          }
        }
      }
    }
  }
  // keep the R best, emit them in ascending chunk order
  if (owner) {
    int last = -1;
    for (int s = 0; s < R; ++s) {
      int best = 0x7FFFFFFF;
#pragma unroll
      for (int i = 0; i < RT; ++i)
        if (i < R && topi[i] > last && topi[i] < best) best = topi[i];
      if (best == 0x7FFFFFFF) {
        out[s] = -1;
      } else {
        out[s] = c0 + best;
        last = best;
        atomicAdd(&s_cnt[best], 1);
      }
    }
  }
  __syncthreads();
  const int tile_local = pv.qtile_local[tile];
  for (int i = tid; i < ncand; i += NT)
    cnt[((long long)(c0 + i) * pv.Hq + h) * pv.max_tiles_per_seq + tile_local] = s_cnt[i];
}

// --------------------------------------------------------------------------- 3. scan over query tiles, then the bases
// Bases, by the block that finishes the scan last.  seg_base[i] = sum of seg_count[<i]; tile_base[e] = sum over
// experts < e of ceil(rows(e) / 128) rounded up to even, with expert e = chunk * Hkv + kv head.
__device__ void plan_bases(const PrefillView& pv, const int* seg_count, int* seg_base, int* tile_base, int* s_part, int* s_total) {
  const int tid = threadIdx.x;
  for (int pass = 0; pass < 2; ++pass) {
    const int n = pass == 0 ? pv.n_chunks * pv.Hq : pv.n_chunks * pv.Hkv;
    int* out = pass == 0 ? seg_base : tile_base;
    const int per = (n + 1023) / 1024;
    const int lo = min(n, tid * per), hi = min(n, lo + per);
    auto value = [&](int i) {
      if (pass == 0) return __ldcg(seg_count + i);
      const int cidx = i / pv.Hkv, g = i - cidx * pv.Hkv;
      const int rows = seg_base[cidx * pv.Hq + (g + 1) * pv.G] - seg_base[cidx * pv.Hq + g * pv.G];
      return ((rows + kTile - 1) / kTile + 1) & ~1;  // even: the forward pairs tiles
    };
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += value(i);
    s_part[tid] = sum;
    __syncthreads();
    if (tid == 0) {
      int run = 0;
      for (int i = 0; i < 1024; ++i) { const int v = s_part[i]; s_part[i] = run; run += v; }
      *s_total = run;
    }
    __syncthreads();
    int run = s_part[tid];
    for (int i = lo; i < hi; ++i) { out[i] = run; run += value(i); }
    if (tid == 0) out[n] = *s_total;
    __threadfence_block();
    __syncthreads();
  }
}

// One warp per (chunk, q head); 32 warps per block.  ticket: one zero int on entry (left zero).
__global__ void __launch_bounds__(1024) segment_scan_kernel(PrefillView pv, int* __restrict__ cnt, int* seg_count,
                                                            int* seg_base, int* tile_base, int* ticket) {
  __shared__ int s_part[1024];
  __shared__ int s_total;
  __shared__ int s_last;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp < pv.n_chunks * pv.Hq) {
    const int c = warp / pv.Hq;
    const int b = pv.chunk_seq[c];
    const int len = pv.cu_seqlens[b + 1] - pv.cu_seqlens[b];
    const int nb = (len + pv.C - 1) / pv.C;
    const int tpc = (pv.C + kTile - 1) / kTile;
    const int last = len - (nb - 1) * pv.C;
    const int ntl = (nb - 1) * tpc + (last + kTile - 1) / kTile;
    const int j = pv.chunk_local[c];
    int* row = cnt + (long long)warp * pv.max_tiles_per_seq;
    int carry = 0;
    if (j < nb - 1) {
      for (int base = (j + 1) * tpc; base < ntl; base += 32) {
        const int i = base + lane;
        const int v = i < ntl ? row[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += n;
        }
        if (i < ntl) row[i] = carry + incl - v;
        carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
      }
    }
    if (lane == 0) seg_count[warp] = carry;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  plan_bases(pv, seg_count, seg_base, tile_base, s_part, &s_total);
  if (threadIdx.x == 0) *ticket = 0;
}

// --------------------------------------------------------------------------- 5. fill
__global__ void __launch_bounds__(128) fill_kernel(PrefillView pv, const int* __restrict__ sel, const int* __restrict__ cnt,
                                                   const int* __restrict__ seg_base, int* __restrict__ rowlist) {
  extern __shared__ unsigned s_ballot[];  // [4][ncand]
  const int tile = blockIdx.x, g = blockIdx.y;
  const int c = pv.qtile_chunk[tile];
  const int ncand = pv.chunk_local[c];
  if (ncand == 0) return;
  const int c0 = c - ncand;
  const int tok0 = pv.qtile_tok0[tile];
  const int nrows = min(kTile, pv.chunk_start[c + 1] - tok0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = tok0 + tid;
  const bool valid = tid < nrows;
  const int tile_local = pv.qtile_local[tile];
  const int R = pv.R;
  for (int hl = 0; hl < pv.G; ++hl) {
    const int h = g * pv.G + hl;
    const int* mine = sel + ((long long)t * pv.Hq + h) * R;
    __syncthreads();
    // ballots per candidate: the row's list is ascending, so one cursor walks it
    int cur = 0;
    int next = (valid && R > 0) ? mine[0] : -1;
    for (int cl = 0; cl < ncand; ++cl) {
      const bool hit = next == c0 + cl;
      const unsigned bal = __ballot_sync(0xFFFFFFFFu, hit);
      if (lane == 0) s_ballot[warp * ncand + cl] = bal;
      if (hit) { ++cur; next = cur < R ? mine[cur] : -1; }
    }
    __syncthreads();
    if (valid) {
      for (int s = 0; s < R; ++s) {
        const int cc = mine[s];
        if (cc < 0) break;
        const int cl = cc - c0;
        int rank = __popc(s_ballot[warp * ncand + cl] & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w) rank += __popc(s_ballot[w * ncand + cl]);
        const long long seg = (long long)cc * pv.Hq + h;
        const int pos = seg_base[seg] + cnt[seg * pv.max_tiles_per_seq + tile_local] + rank;
        rowlist[pos] = (t * pv.Hq + h) * R + s;
      }
    }
  }
}

// --------------------------------------------------------------------------- host side
int validate_desc(const moba_prefill_desc* d) {
  if (!d) return MOBA_ERR_INVALID;
  if (d->total_tokens < 1 || d->num_seqs < 1 || d->hq < 1 || d->hkv < 1 || d->hq % d->hkv) return MOBA_ERR_INVALID;
  if (d->dim < 8 || d->dim > 256 || d->dim % 8) return MOBA_ERR_INVALID;
  if (d->chunk_size < 1 || d->remote_k < 0 || d->num_chunks < 1 || d->num_qtiles < 1) return MOBA_ERR_INVALID;
  if (d->remote_k > 16 || d->dim > 128) return MOBA_ERR_UNSUPPORTED;  // prefill kernels: head_dim up to 128
  if ((long long)d->total_tokens * d->hq * (d->remote_k > 0 ? d->remote_k : 1) >= (1ll << 31)) return MOBA_ERR_UNSUPPORTED;
  if (d->max_chunks_per_seq > 4096) return MOBA_ERR_UNSUPPORTED;
  if (!d->cu_seqlens || !d->chunk_start || !d->chunk_seq || !d->chunk_local || !d->qtile_chunk || !d->qtile_tok0 ||
      !d->qtile_local || !d->self_pairs || d->num_self_pairs < 1 || d->num_self_pairs > d->num_qtiles)
    return MOBA_ERR_INVALID;
  return MOBA_OK;
}

template <int RT, int DD, int LPR>
static cudaError_t launch_gate_as(const PrefillView& pv, const __nv_bfloat16* q, const float* means, int* sel, int* cnt,
                                  int max_chunks_per_seq, cudaStream_t st) {
  constexpr int DP = DD * LPR;
  const size_t smem = (size_t)kCandBatch * DP * 4 + (size_t)kTile * (DP * 2 + 16) + (size_t)max_chunks_per_seq * 4 + 16;
  cudaError_t e = cudaFuncSetAttribute(gate_topk_kernel<RT, DD, LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  gate_topk_kernel<RT, DD, LPR><<<dim3(pv.n_qtiles, pv.Hq), 32 * LPR, smem, st>>>(pv, q, means, sel, cnt);
  return cudaGetLastError();
}

template <int RT>
static cudaError_t launch_gate(const PrefillView& pv, const __nv_bfloat16* q, const float* means, int* sel, int* cnt,
                               int max_chunks_per_seq, cudaStream_t st) {
  if (pv.D <= 32) return launch_gate_as<RT, 8, 4>(pv, q, means, sel, cnt, max_chunks_per_seq, st);
  if (pv.D <= 64) return launch_gate_as<RT, 16, 4>(pv, q, means, sel, cnt, max_chunks_per_seq, st);
  return launch_gate_as<RT, 16, 8>(pv, q, means, sel, cnt, max_chunks_per_seq, st);
}

// Layout of the routing scratch.  Only `tickets` has to be zero when a call starts (route_impl clears it).
struct RouteScratch {
  float* means;     // [n_chunks][Hkv][D]
  float* part;      // [n_chunks][Hkv][splits][D] slice sums of the mean pass
  int* cnt;         // [n_chunks][Hq][max_tiles_per_seq]
  int* seg_count;   // [n_chunks][Hq]
  int* tickets;     // [n_chunks * Hkv + 1] arrival counters of the mean pass, then one for the scan pass
  size_t tickets_bytes, total;
};
static int mean_splits(const moba_prefill_desc& d) { return (d.chunk_size + kMeanRows - 1) / kMeanRows; }
static RouteScratch carve_route_scratch(const moba_prefill_desc& d, void* base) {
  RouteScratch r;
  char* p = static_cast<char*>(base);
  const size_t seg = (size_t)d.num_chunks * d.hkv;
  r.means = reinterpret_cast<float*>(p); p += align256(seg * d.dim * 4);
  r.part = reinterpret_cast<float*>(p); p += align256(seg * mean_splits(d) * d.dim * 4);
  r.cnt = reinterpret_cast<int*>(p); p += align256((size_t)d.num_chunks * d.hq * d.max_tiles_per_seq * 4);
  r.seg_count = reinterpret_cast<int*>(p); p += align256((size_t)d.num_chunks * d.hq * 4);
  r.tickets = reinterpret_cast<int*>(p);
  r.tickets_bytes = (seg + 1) * 4;
  p += align256(r.tickets_bytes);
  r.total = (size_t)(p - static_cast<char*>(base));
  return r;
}

}  // namespace moba

using namespace moba;

extern "C" size_t moba_prefill_route_state_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  return route_state_bytes(*d);
}

extern "C" size_t moba_prefill_route_scratch_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  return carve_route_scratch(*d, nullptr).total;
}

static int route_impl(const moba_prefill_desc* d, const void* q, const void* k, void* route_state, void* scratch,
                      cudaStream_t st) {
  if (d->remote_k == 0) return MOBA_OK;  // dense fallback: nothing to route
  const PrefillView pv = make_view(*d);
  RouteState rs = carve_route_state(*d, route_state);
  const RouteScratch sc = carve_route_scratch(*d, scratch);
  float* means = sc.means;
  int* cnt = sc.cnt;
  int* seg_count = sc.seg_count;
  // The arrival counters are the one part of the scratch that must start at zero; everything else is written before
  // it is read.  (The kernels leave the counters at zero, but a caller's scratch arrives with arbitrary contents.)
  if (cudaMemsetAsync(sc.tickets, 0, sc.tickets_bytes, st) != cudaSuccess) return MOBA_ERR_CUDA;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);

  const int rpi = 256 / (d->dim / 8);
  chunk_mean_kernel<<<dim3(d->num_chunks, d->hkv, mean_splits(*d)), 256, (size_t)rpi * d->dim * 4, st>>>(
      pv, kb, sc.part, means, sc.tickets, d->flags & MOBA_ROUTE_BF16_MEANS, mean_splits(*d));
  if (cudaGetLastError() != cudaSuccess) return MOBA_ERR_CUDA;
  cudaError_t e;
  const int R = d->remote_k;
  if (R <= 1) e = launch_gate<1>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  else if (R <= 2) e = launch_gate<2>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  else if (R <= 3) e = launch_gate<3>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  else if (R <= 4) e = launch_gate<4>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  else if (R <= 8) e = launch_gate<8>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  else e = launch_gate<16>(pv, qb, means, rs.sel, cnt, d->max_chunks_per_seq, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  const int segs = d->num_chunks * d->hq;
  segment_scan_kernel<<<(segs + 31) / 32, 1024, 0, st>>>(pv, cnt, seg_count, rs.seg_base, rs.tile_base,
                                                          sc.tickets + (size_t)d->num_chunks * d->hkv);
  fill_kernel<<<dim3(d->num_qtiles, d->hkv), 128, (size_t)4 * d->max_chunks_per_seq * 4 + 16, st>>>(pv, rs.sel, cnt, rs.seg_base,
                                                                                                 rs.rowlist);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_prefill_route(const moba_prefill_desc* d, const void* q, const void* k, void* route_state,
                                  void* scratch, size_t scratch_bytes, void* stream) {
  int rc = validate_desc(d);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !route_state || !scratch) return MOBA_ERR_INVALID;
  if (scratch_bytes < moba_prefill_route_scratch_bytes(d)) return MOBA_ERR_WORKSPACE;
  return route_impl(d, q, k, route_state, scratch, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Routing for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain the routing scratch: a serving loop whose device
// memory was handed out in full at start-up to one pool, code running under a runtime that forbids
// cudaMalloc on the request path because it stalls every stream of the device, or a foreign-language
// binding that only holds the tensors its framework passed in.  For them the scratch lives in the
// library itself: one fixed array in device memory, reserved on every GPU that loads the library for
// as long as the process lives.
constexpr size_t kRouteStaticScratchBytes = MOBA_ROUTE_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_route_scratch[kRouteStaticScratchBytes];

#include <mutex>
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_route_scratch_mutex;
void* g_route_scratch_addr[kMaxDevices];  // device address of g_route_scratch, per device ordinal
}  // namespace

extern "C" size_t moba_prefill_route_static_capacity(void) { return kRouteStaticScratchBytes; }

extern "C" int moba_prefill_route_static(const moba_prefill_desc* d, const void* q, const void* k, void* route_state,
                                         void* stream) {
  int rc = validate_desc(d);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !route_state) return MOBA_ERR_INVALID;
  if (moba_prefill_route_scratch_bytes(d) > kRouteStaticScratchBytes) return MOBA_ERR_WORKSPACE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MOBA_ERR_CUDA;
  void* scratch = nullptr;
  {
    // First call on a device: resolve the array's device address.  In host code the symbol is only
    // a handle; the kernels need the address cudaGetSymbolAddress returns for the current device.
    std::lock_guard<std::mutex> lock(g_route_scratch_mutex);
    if (!g_route_scratch_addr[dev]) {
      void* addr = nullptr;
      if (cudaGetSymbolAddress(&addr, g_route_scratch) != cudaSuccess || !addr) return MOBA_ERR_CUDA;
      g_route_scratch_addr[dev] = addr;
    }
    scratch = g_route_scratch_addr[dev];
  }
  // The previous call's contents stay in the array.  The arrival counters of the mean and scan passes are the
  // only words that must start at zero, and route_impl clears them on the stream before the first kernel; every
  // other word the later passes read is written by an earlier pass of the same call.
  return route_impl(d, q, k, route_state, scratch, (cudaStream_t)stream);
}
