// Paged KV-cache decode kernels (HBM-bound, CUDA cores): token append through the page table,
// chunk means, per-step metadata, block routing and split-K paged attention with in-kernel merge.
// They replace the Triton kernels of the reference (src/moba_opt/ops/paged_decode.py:11-144,
// src/moba_opt/ops/prepared_decode.py:7-94) and torch.topk in the routing step.
//
// Every kernel reads positions / lengths / the page table from device memory at fixed addresses and
// has a launch shape that depends only on sizes fixed at prepare time, so a decode step can be
// captured in a CUDA graph and replayed.
//
// Attention reads each needed K/V token once per KV head: the routing kernel turns the per-query-
// head selections of a GQA group into the union of chunks with a bitmask of the heads that attend
// each of them; one CTA handles one part of one chunk for all those heads.  Partial (max, sum,
// accumulator) triples go to a workspace and the last CTA of a (query, kv head) pair to finish -
// found with an atomic ticket, nobody waits - merges them in a fixed order.
#include "moba_b200.h"
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

struct CacheView {
  int slots, max_seq_len, page, num_pages, width, C, max_chunks, Hkv, D;
  __nv_bfloat16* kc;
  __nv_bfloat16* vc;
  int* table;
  int* lengths;
  __nv_bfloat16* means;
};

static CacheView make_cache_view(const moba_cache_desc& c) {
  CacheView v;
  v.slots = c.batch_slots; v.max_seq_len = c.max_seq_len; v.page = c.page_size; v.num_pages = c.num_pages;
  v.width = c.table_width; v.C = c.chunk_size; v.max_chunks = c.max_chunks; v.Hkv = c.hkv; v.D = c.dim;
  v.kc = static_cast<__nv_bfloat16*>(c.k_cache); v.vc = static_cast<__nv_bfloat16*>(c.v_cache);
  v.table = c.table; v.lengths = c.lengths; v.means = static_cast<__nv_bfloat16*>(c.means);
  return v;
}

static int validate_cache(const moba_cache_desc* c) {
  if (!c) return MOBA_ERR_INVALID;
  if (c->batch_slots < 1 || c->max_seq_len < 1 || c->page_size < 1 || c->num_pages < 1 || c->table_width < 1 ||
      c->chunk_size < 1 || c->max_chunks < 1 || c->hkv < 1)
    return MOBA_ERR_INVALID;
  if (c->dim < 8 || c->dim > 256 || c->dim % 8) return MOBA_ERR_UNSUPPORTED;
  if (!c->k_cache || !c->v_cache || !c->table || !c->lengths || !c->means) return MOBA_ERR_INVALID;
  return MOBA_OK;
}

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float dec_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// --------------------------------------------------------------------------- metadata (K15)
// Applies the page-table delta of this step (idempotent), publishes the query positions and, for an
// appending step, advances the lengths.  One CTA; rows are independent.
__global__ void decode_metadata_kernel(CacheView cv, const int* __restrict__ ids, int* __restrict__ positions,
                                       const int* __restrict__ delta, int b, int append) {
  for (int row = threadIdx.x; row < b; row += blockDim.x) {
    const int sid = ids[row];
    const int logical = delta[row], physical = delta[b + row];
    if (logical >= 0 && logical < cv.width) cv.table[(long long)sid * cv.width + logical] = physical;
    const int len = cv.lengths[sid];
    if (append) {
      positions[row] = len;
      cv.lengths[sid] = len + 1;
    } else {
      positions[row] = len - 1;
    }
  }
}

// --------------------------------------------------------------------------- append (K10)
__global__ void __launch_bounds__(256) decode_append_kernel(CacheView cv, const __nv_bfloat16* __restrict__ k,
                                                            const __nv_bfloat16* __restrict__ v, const int* __restrict__ tok_seq,
                                                            const int* __restrict__ tok_pos, long long units, unsigned* status) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= units) return;
  const int upr = cv.D >> 3;
  const int u = (int)(i % upr);
  const long long th = i / upr;  // token * Hkv + head
  const int head = (int)(th % cv.Hkv);
  const long long token = th / cv.Hkv;
  const int sid = tok_seq[token], pos = tok_pos[token];
  const int physical = cv.table[(long long)sid * cv.width + pos / cv.page];
  if (physical < 0 || physical >= cv.num_pages) {
    if (status) atomicOr(status, kErrBadIndex);
    return;
  }
  const long long dst = (((long long)physical * cv.page + pos % cv.page) * cv.Hkv + head) * cv.D + u * 8;
  const long long src = th * cv.D + u * 8;
  *reinterpret_cast<uint4*>(cv.kc + dst) = *reinterpret_cast<const uint4*>(k + src);
  *reinterpret_cast<uint4*>(cv.vc + dst) = *reinterpret_cast<const uint4*>(v + src);
}

// --------------------------------------------------------------------------- chunk means (K11, K16)
// One CTA per (item, kv head).  Explicit mode: item = (sequence, chunk).  Predicated mode: item =
// a decode row; the mean is computed only when the token just appended completes its chunk.
__global__ void __launch_bounds__(256) decode_means_kernel(CacheView cv, const int* __restrict__ seqs,
                                                           const int* __restrict__ chunk_or_pos, int predicated,
                                                           unsigned* status) {
  extern __shared__ float s_part[];
  const int item = blockIdx.x, g = blockIdx.y;
  const int sid = seqs[item];
  int chunk = chunk_or_pos[item];
  if (predicated) {
    const int pos = chunk;
    if ((pos + 1) % cv.C != 0) return;
    chunk = pos / cv.C;
  }
  if (chunk < 0 || chunk >= cv.max_chunks) return;
  const int upr = cv.D >> 3, rpi = 256 / upr;
  const int ri = threadIdx.x / upr, u = threadIdx.x - ri * upr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (ri < rpi) {
    for (int w = ri; w < cv.C; w += rpi) {
      const int t = chunk * cv.C + w;
      const int physical = cv.table[(long long)sid * cv.width + t / cv.page];
      if (physical < 0 || physical >= cv.num_pages) {
        if (status) atomicOr(status, kErrBadIndex);
        continue;
      }
      const uint4 raw =
          *reinterpret_cast<const uint4*>(cv.kc + (((long long)physical * cv.page + t % cv.page) * cv.Hkv + g) * cv.D + u * 8);
      const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[2 * i] += bf_lo(wv[i]); acc[2 * i + 1] += bf_hi(wv[i]); }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_part[ri * cv.D + u * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < cv.D; d += 256) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += s_part[r * cv.D + d];
    cv.means[(((long long)sid * cv.max_chunks + chunk) * cv.Hkv + g) * cv.D + d] = __float2bfloat16_rn(s / (float)cv.C);
  }
}

// --------------------------------------------------------------------------- routing (K12, K13, K17, K18)
// One CTA (128 threads) per (query row, kv head).  scores[row, h, c] = q . mean[c] in FP32 for the
// chunks completed before the query's own chunk, -inf elsewhere; top-`remote` per head in descending
// score order with the lowest chunk winning exact ties; selected[row, h, :] = (own chunk, picks...,
// -1 padding); and the group's union list (chunk ascending, bitmask of heads) for the attention kernel.
__global__ void __launch_bounds__(128) decode_route_kernel(CacheView cv, const __nv_bfloat16* __restrict__ q,
                                                           const int* __restrict__ ids, const int* __restrict__ positions,
                                                           int Hq, int remote, int width, float* __restrict__ scores,
                                                           int* __restrict__ selected, int* __restrict__ u_chunk,
                                                           unsigned* __restrict__ u_mask, int* __restrict__ u_count, int umax) {
  extern __shared__ float s_dyn[];
  const int G = Hq / cv.Hkv;
  float* s_scores = s_dyn;                                            // [G][width]
  unsigned* s_mask = reinterpret_cast<unsigned*>(s_dyn + G * width);  // [width + 1]
  const int row = blockIdx.x, g = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sid = ids[row], pos = positions[row];
  const int cur = pos / cv.C;
  const int nlegal = min(min(cur, width), cv.max_chunks);
  const int upr = cv.D >> 3;

  for (int i = tid; i <= width; i += 128) s_mask[i] = 0u;
  // scores: warp w takes (head, chunk) pairs round-robin, lanes split the head dimension
  for (int pair = warp; pair < G * width; pair += 4) {
    const int hl = pair / width, c = pair - hl * width;
    float s = -INFINITY;
    if (c < nlegal) {
      float part = 0.f;
      if (lane < upr) {
        const uint4 qa = *reinterpret_cast<const uint4*>(q + ((long long)row * Hq + g * G + hl) * cv.D + lane * 8);
        const uint4 ma = *reinterpret_cast<const uint4*>(cv.means + (((long long)sid * cv.max_chunks + c) * cv.Hkv + g) * cv.D + lane * 8);
        const uint32_t qw[4] = {qa.x, qa.y, qa.z, qa.w}, mw[4] = {ma.x, ma.y, ma.z, ma.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          part = fmaf(bf_lo(qw[i]), bf_lo(mw[i]), part);
          part = fmaf(bf_hi(qw[i]), bf_hi(mw[i]), part);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
      s = part;
    }
    if (lane == 0) {
      s_scores[pair] = s;
      if (scores) scores[((long long)row * Hq + g * G + hl) * width + c] = s;
    }
  }
  __syncthreads();
  // top-k: one warp per head, `remote` rounds of (max value, lowest index among equals)
  for (int hl = warp; hl < G; hl += 4) {
    float* sc = s_scores + hl * width;
    int* out = selected + ((long long)row * Hq + g * G + hl) * (remote + 1);
    if (lane == 0) out[0] = cur;
    for (int r = 0; r < remote; ++r) {
      float best = -INFINITY;
      int idx = 0x7FFFFFFF;
      for (int c = lane; c < nlegal; c += 32) {
        const float v = sc[c];
        if (v > best || (v == best && c < idx && v > -INFINITY)) { best = v; idx = c; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
      }
      const bool found = best > -INFINITY && idx != 0x7FFFFFFF;
      if (lane == 0) {
        out[1 + r] = found ? idx : -1;
        if (found) {
          sc[idx] = -INFINITY;
          atomicOr(&s_mask[idx], 1u << hl);
        }
      }
      __syncwarp();
    }
  }
  __syncthreads();
  // union list: routed chunks ascending, the own chunk (all heads) last
  if (warp == 0) {
    const long long base = ((long long)row * cv.Hkv + g) * umax;
    int count = 0;
    for (int c0 = 0; c0 < nlegal; c0 += 32) {
      const int c = c0 + lane;
      const unsigned m = c < nlegal ? s_mask[c] : 0u;
      const unsigned bal = __ballot_sync(0xFFFFFFFFu, m != 0u);
      if (m) {
        const int at = count + __popc(bal & ((1u << lane) - 1u));
        if (at < umax - 1) { u_chunk[base + at] = c; u_mask[base + at] = m; }
      }
      count += __popc(bal);
    }
    if (lane == 0) {
      count = min(count, umax - 1);
      u_chunk[base + count] = cur;
      u_mask[base + count] = G >= 32 ? 0xFFFFFFFFu : ((1u << G) - 1u);
      u_count[(long long)row * cv.Hkv + g] = count + 1;
    }
  }
}

// --------------------------------------------------------------------------- attention (K14)
struct AttendArgs {
  CacheView cv;
  const __nv_bfloat16* q;
  const int* ids;
  const int* positions;
  const int* selected;  // [nq, Hq, ns] or null for dense
  const int* u_chunk;
  const unsigned* u_mask;
  const int* u_count;
  int Hq, ns, umax, parts, part_tokens;
  int* counters;   // [nq * Hkv], zero between launches
  float* pm;       // [nq*Hq*ns*parts]
  float* pl;
  float* pacc;     // [.., D]
  __nv_bfloat16* out;
  float* lse;
  unsigned* status;
  float scale_log2;
};

constexpr int kHeadBatch = 8;

template <int LPR>
__global__ void __launch_bounds__(128) decode_attend_kernel(AttendArgs a) {
  constexpr int NRG = 128 / LPR;  // token rows in flight per CTA
  extern __shared__ float s_red[];  // [NRG][kHeadBatch][D + 2]
  __shared__ int s_last;
  const CacheView& cv = a.cv;
  const int D = cv.D, G = a.Hq / cv.Hkv;
  const int rowg = blockIdx.z, row = rowg / cv.Hkv, g = rowg - row * cv.Hkv;
  const int k = blockIdx.x, part = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31;
  const int rg = tid / LPR, li = tid - rg * LPR;
  const int sid = a.ids[row], pos = a.positions[row];
  const int visible = min(pos + 1, cv.lengths[sid]);  // tokens [0, visible) exist and are not in the future
  const int cur = pos / cv.C;
  const bool dense = a.selected == nullptr;
  const int ucount = dense ? cur + 1 : a.u_count[rowg];
  if (k >= ucount) return;
  const int chunk = dense ? k : a.u_chunk[(long long)rowg * a.umax + k];
  const unsigned mask = dense ? (G >= 32 ? 0xFFFFFFFFu : ((1u << G) - 1u)) : a.u_mask[(long long)rowg * a.umax + k];
  const int limit = min((chunk + 1) * cv.C, visible);
  const int t_begin = chunk * cv.C + part * a.part_tokens;
  const int t_end = min(t_begin + a.part_tokens, limit);
  if (t_begin >= t_end) return;
  const int cur_parts = (visible - cur * cv.C + a.part_tokens - 1) / a.part_tokens;
  const int expected = (ucount - 1) * a.parts + cur_parts;
  const bool dl = li * 8 < D;  // this lane holds 8 head-dim elements

  for (int hb = 0; hb < G; hb += kHeadBatch) {
    const unsigned active = (mask >> hb) & 0xFFu;
    if (!active) continue;
    float qv[kHeadBatch][8], acc[kHeadBatch][8], m[kHeadBatch], l[kHeadBatch];
#pragma unroll
    for (int hh = 0; hh < kHeadBatch; ++hh) {
      m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) { acc[hh][j] = 0.f; qv[hh][j] = 0.f; }
      if (((active >> hh) & 1u) && dl) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a.q + ((long long)row * a.Hq + g * G + hb + hh) * D + li * 8);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { qv[hh][2 * j] = bf_lo(w[j]) * a.scale_log2; qv[hh][2 * j + 1] = bf_hi(w[j]) * a.scale_log2; }
      }
    }
    for (int t0 = t_begin; t0 < t_end; t0 += 2 * NRG) {
      uint4 kr[2], vr[2];
      bool ok[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int t = t0 + x * NRG + rg;
        ok[x] = t < t_end;
        kr[x] = make_uint4(0, 0, 0, 0);
        vr[x] = make_uint4(0, 0, 0, 0);
        if (ok[x]) {
          const int physical = cv.table[(long long)sid * cv.width + t / cv.page];
          if (physical < 0 || physical >= cv.num_pages) {
            atomicOr(a.status, kErrBadIndex);
            ok[x] = false;
          } else if (dl) {
            const long long off = (((long long)physical * cv.page + t % cv.page) * cv.Hkv + g) * D + li * 8;
            kr[x] = __ldg(reinterpret_cast<const uint4*>(cv.kc + off));
            vr[x] = __ldg(reinterpret_cast<const uint4*>(cv.vc + off));
          }
        }
      }
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const uint32_t kw[4] = {kr[x].x, kr[x].y, kr[x].z, kr[x].w}, vw[4] = {vr[x].x, vr[x].y, vr[x].z, vr[x].w};
        float kf[8], vf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { kf[2 * j] = bf_lo(kw[j]); kf[2 * j + 1] = bf_hi(kw[j]); vf[2 * j] = bf_lo(vw[j]); vf[2 * j + 1] = bf_hi(vw[j]); }
#pragma unroll
        for (int hh = 0; hh < kHeadBatch; ++hh) {
          if (!((active >> hh) & 1u)) continue;
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) s = fmaf(qv[hh][j], kf[j], s);
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
          if (ok[x]) {
            const float mn = fmaxf(m[hh], s);
            const float alpha = dec_exp2(m[hh] - mn), p = dec_exp2(s - mn);
            l[hh] = l[hh] * alpha + p;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[hh][j] = fmaf(acc[hh][j], alpha, p * vf[j]);
            m[hh] = mn;
          }
        }
      }
    }
    // combine the NRG row groups of the CTA, then write one partial per head
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < kHeadBatch; ++hh) {
      if (!((active >> hh) & 1u)) continue;
      float* dst = s_red + ((size_t)rg * kHeadBatch + hh) * (D + 2);
      if (dl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[li * 8 + j] = acc[hh][j];
      }
      if (li == 0) { dst[D] = m[hh]; dst[D + 1] = l[hh]; }
    }
    __syncthreads();
    for (int hh = 0; hh < kHeadBatch; ++hh) {
      if (!((active >> hh) & 1u)) continue;
      const int h = g * G + hb + hh;
      int slot = dense ? chunk : -1;
      if (!dense) {
        for (int s = 0; s < a.ns; ++s)
          if (a.selected[((long long)row * a.Hq + h) * a.ns + s] == chunk) { slot = s; break; }
      }
      if (slot < 0) continue;
      const long long pidx = (((long long)row * a.Hq + h) * a.ns + slot) * a.parts + part;
      float big = -INFINITY;
      for (int r = 0; r < NRG; ++r) big = fmaxf(big, s_red[((size_t)r * kHeadBatch + hh) * (D + 2) + D]);
      float lsum = 0.f;
      for (int r = 0; r < NRG; ++r) {
        const float* src = s_red + ((size_t)r * kHeadBatch + hh) * (D + 2);
        lsum += src[D + 1] * dec_exp2(src[D] - big);
      }
      for (int d = tid; d < D; d += 128) {
        float v = 0.f;
        for (int r = 0; r < NRG; ++r) {
          const float* src = s_red + ((size_t)r * kHeadBatch + hh) * (D + 2);
          v += src[d] * dec_exp2(src[D] - big);
        }
        a.pacc[pidx * D + d] = v;
      }
      if (tid == 0) { a.pm[pidx] = big; a.pl[pidx] = lsum; }
    }
  }

  // ---- ticket: the last CTA of this (query, kv head) merges every partial of the group's heads
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&a.counters[rowg], 1);
    s_last = ticket == expected - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int hl = 0; hl < G; ++hl) {
    const int h = g * G + hl;
    const long long hbase = ((long long)row * a.Hq + h) * a.ns;
    const int nslots = dense ? cur + 1 : a.ns;
    float big = -INFINITY;
    for (int s = 0; s < nslots; ++s) {
      const int c = dense ? s : a.selected[hbase + s];
      if (c < 0) continue;
      const int np = c == cur ? cur_parts : a.parts;
      for (int p = 0; p < np; ++p) big = fmaxf(big, __ldcg(a.pm + (hbase + s) * a.parts + p));
    }
    float lsum = 0.f;
    for (int s = 0; s < nslots; ++s) {
      const int c = dense ? s : a.selected[hbase + s];
      if (c < 0) continue;
      const int np = c == cur ? cur_parts : a.parts;
      for (int p = 0; p < np; ++p) {
        const long long pidx = (hbase + s) * a.parts + p;
        lsum += __ldcg(a.pl + pidx) * dec_exp2(__ldcg(a.pm + pidx) - big);
      }
    }
    for (int d = tid; d < D; d += 128) {
      float v = 0.f;
      for (int s = 0; s < nslots; ++s) {
        const int c = dense ? s : a.selected[hbase + s];
        if (c < 0) continue;
        const int np = c == cur ? cur_parts : a.parts;
        for (int p = 0; p < np; ++p) {
          const long long pidx = (hbase + s) * a.parts + p;
          v += __ldcg(a.pacc + pidx * D + d) * dec_exp2(__ldcg(a.pm + pidx) - big);
        }
      }
      a.out[((long long)row * a.Hq + h) * D + d] = __float2bfloat16_rn(v / lsum);
    }
    if (tid == 0) a.lse[(long long)row * a.Hq + h] = (big + log2f(lsum)) * 0.6931471805599453f;
  }
  if (tid == 0) a.counters[rowg] = 0;  // ready for the next launch (graph replay included)
}

}  // namespace moba

using namespace moba;

extern "C" int moba_decode_metadata(const moba_cache_desc* c, const int32_t* ids, int32_t* positions, const int32_t* delta,
                                    int rows, int append, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!ids || !positions || !delta || rows < 1) return MOBA_ERR_INVALID;
  decode_metadata_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(make_cache_view(*c), ids, positions, delta, rows, append);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_append(const moba_cache_desc* c, const void* k, const void* v, const int32_t* token_seq,
                                  const int32_t* token_pos, int tokens, unsigned* status, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!k || !v || !token_seq || !token_pos || tokens < 1) return MOBA_ERR_INVALID;
  const long long units = (long long)tokens * c->hkv * (c->dim / 8);
  decode_append_kernel<<<(unsigned)((units + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      make_cache_view(*c), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), token_seq, token_pos, units,
      status);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_means(const moba_cache_desc* c, const int32_t* seqs, const int32_t* chunk_or_pos, int items,
                                 int predicated, unsigned* status, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (items == 0) return MOBA_OK;
  if (!seqs || !chunk_or_pos || items < 0) return MOBA_ERR_INVALID;
  const int rpi = 256 / (c->dim / 8);
  decode_means_kernel<<<dim3(items, c->hkv), 256, (size_t)rpi * c->dim * 4, (cudaStream_t)stream>>>(
      make_cache_view(*c), seqs, chunk_or_pos, predicated, status);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_union_capacity(int hq, int hkv, int remote, int width) {
  if (hq < 1 || hkv < 1 || hq % hkv || remote < 0 || width < 0) return 0;
  const long long routed = (long long)(hq / hkv) * remote;
  return (int)(routed < width ? routed : width) + 1;
}

extern "C" int moba_decode_route(const moba_cache_desc* c, const void* q, const int32_t* ids, const int32_t* positions,
                                 int rows, int hq, int remote, int width, float* scores, int32_t* selected, int32_t* u_chunk,
                                 uint32_t* u_mask, int32_t* u_count, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!q || !ids || !positions || !selected || !u_chunk || !u_mask || !u_count || rows < 1 || hq < 1 || hq % c->hkv ||
      remote < 0 || width < 1)
    return MOBA_ERR_INVALID;
  const int G = hq / c->hkv;
  if (G > 32 || remote > 16) return MOBA_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)G * width + width + 1) * 4;
  if (smem > 200 * 1024) return MOBA_ERR_UNSUPPORTED;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(decode_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return MOBA_ERR_CUDA;
  const int umax = moba_decode_union_capacity(hq, c->hkv, remote, width);
  decode_route_kernel<<<dim3(rows, c->hkv), 128, smem, (cudaStream_t)stream>>>(
      make_cache_view(*c), static_cast<const __nv_bfloat16*>(q), ids, positions, hq, remote, width, scores, selected, u_chunk, u_mask,
      u_count, umax);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

static int attend_parts(const moba_cache_desc* c) {
  const int part_tokens = c->chunk_size >= 256 ? 256 : c->chunk_size;
  return (c->chunk_size + part_tokens - 1) / part_tokens;
}

extern "C" size_t moba_decode_attend_workspace_bytes(const moba_cache_desc* c, int rows, int hq, int slots) {
  if (validate_cache(c) != MOBA_OK || rows < 1 || hq < 1 || slots < 1) return 0;
  const size_t n = (size_t)rows * hq * slots * attend_parts(c);
  return align256((size_t)rows * c->hkv * 4) + 2 * align256(n * 4) + align256(n * c->dim * 4);
}

extern "C" int moba_decode_attend(const moba_cache_desc* c, const void* q, const int32_t* ids, const int32_t* positions,
                                  int rows, int hq, const int32_t* selected, int slots, const int32_t* u_chunk,
                                  const uint32_t* u_mask, const int32_t* u_count, int umax, void* workspace,
                                  size_t workspace_bytes, void* out, float* lse, unsigned* status, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!q || !ids || !positions || !workspace || !out || !lse || !status || rows < 1 || hq < 1 || hq % c->hkv || slots < 1)
    return MOBA_ERR_INVALID;
  if (selected && (!u_chunk || !u_mask || !u_count || umax < 1)) return MOBA_ERR_INVALID;
  if (hq / c->hkv > 32) return MOBA_ERR_UNSUPPORTED;
  if (workspace_bytes < moba_decode_attend_workspace_bytes(c, rows, hq, slots)) return MOBA_ERR_WORKSPACE;
  AttendArgs a;
  a.cv = make_cache_view(*c);
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.ids = ids; a.positions = positions; a.selected = selected;
  a.u_chunk = u_chunk; a.u_mask = u_mask; a.u_count = u_count;
  a.Hq = hq; a.ns = slots; a.umax = selected ? umax : slots;
  a.parts = attend_parts(c);
  a.part_tokens = c->chunk_size >= 256 ? 256 : c->chunk_size;
  const size_t n = (size_t)rows * hq * slots * a.parts;
  char* p = static_cast<char*>(workspace);
  a.counters = reinterpret_cast<int*>(p); p += align256((size_t)rows * c->hkv * 4);
  a.pm = reinterpret_cast<float*>(p); p += align256(n * 4);
  a.pl = reinterpret_cast<float*>(p); p += align256(n * 4);
  a.pacc = reinterpret_cast<float*>(p);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.status = status;
  a.scale_log2 = (float)(1.4426950408889634 / sqrt((double)c->dim));
  const int lpr = c->dim <= 32 ? 4 : c->dim <= 64 ? 8 : c->dim <= 128 ? 16 : 32;
  const int nrg = 128 / lpr;
  const size_t smem = (size_t)nrg * kHeadBatch * (c->dim + 2) * 4;
  const dim3 grid(a.umax, a.parts, rows * c->hkv);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  prof_begin(kProfDecodeAttend, st);
#define MOBA_LAUNCH_ATTEND(L)                                                                                      \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      e = cudaFuncSetAttribute(decode_attend_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e == cudaSuccess) decode_attend_kernel<L><<<grid, 128, smem, st>>>(a);                                     \
  } while (0)
  if (lpr == 4) MOBA_LAUNCH_ATTEND(4);
  else if (lpr == 8) MOBA_LAUNCH_ATTEND(8);
  else if (lpr == 16) MOBA_LAUNCH_ATTEND(16);
  else MOBA_LAUNCH_ATTEND(32);
#undef MOBA_LAUNCH_ATTEND
  prof_end(kProfDecodeAttend, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
