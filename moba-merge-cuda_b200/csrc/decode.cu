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
#include "launch.cuh"
#include "moba_b200.h"
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

struct CacheView {
  int slots, max_seq_len, page, num_pages, width, C, max_chunks, Hkv, D;
  int fp16;  // pools, means, q and out are IEEE half (MOBA_CACHE_FP16), else bf16; the pointer types below only address 16-bit elements
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
  v.fp16 = (c.flags & MOBA_CACHE_FP16) ? 1 : 0;
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
// one 16-bit value to its bits in the cache's format
__device__ __forceinline__ uint16_t bits16(float x, bool f16) {
  return f16 ? __half_as_ushort(__float2half_rn(x)) : __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float value16(const __nv_bfloat16* p, bool f16) {
  const uint16_t w = *reinterpret_cast<const uint16_t*>(p);
  return f16 ? __half2float(__ushort_as_half(w)) : __uint_as_float((uint32_t)w << 16);
}
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

// Host-planned changes of the device page table and lengths, changed entries only: `edits` = n triples (sequence,
// logical page, physical page; physical -1 unmaps), then for the m sequences in ids: lengths[ids[j]] = lengths_new[j],
// and with clear_rows the whole table row of every listed sequence is unmapped first (a reset).
__global__ void __launch_bounds__(256) cache_update_kernel(CacheView cv, const int* __restrict__ edits, int n,
                                                           const int* __restrict__ ids, const int* __restrict__ lengths_new, int m,
                                                           int clear_rows) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (clear_rows) {
    for (long long e = i; e < (long long)m * cv.width; e += (long long)gridDim.x * 256) {
      const int sid = ids[e / cv.width];
      if (sid >= 0 && sid < cv.slots) cv.table[(long long)sid * cv.width + e % cv.width] = -1;
    }
  } else if (i < n) {
    const int sid = edits[3 * i], logical = edits[3 * i + 1];
    if (sid >= 0 && sid < cv.slots && logical >= 0 && logical < cv.width) cv.table[(long long)sid * cv.width + logical] = edits[3 * i + 2];
  }
  if (i < m) {
    const int sid = ids[i];
    if (sid >= 0 && sid < cv.slots) cv.lengths[sid] = lengths_new[i];
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

// Second half of a chunk mean: thread (ri, u) holds the sums of unit u over the rows w = ri, ri + rpi, ... of the chunk;
// the row groups are added in ascending order and the mean is rounded to the cache's format.  Every producer of a mean goes through
// here with the same assignment of rows to threads, so a mean has the same bits whichever call computed it.
__device__ __forceinline__ void chunk_mean_finish(const CacheView& cv, int sid, int chunk, int g, const float (&acc)[8], float* s_part) {
  const int upr = cv.D >> 3, rpi = 256 / upr;
  const int ri = threadIdx.x / upr, u = threadIdx.x - ri * upr;
  if (ri < rpi) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_part[ri * cv.D + u * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < cv.D; d += 256) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += s_part[r * cv.D + d];
    reinterpret_cast<uint16_t*>(cv.means)[(((long long)sid * cv.max_chunks + chunk) * cv.Hkv + g) * cv.D + d] =
        bits16(s / (float)cv.C, cv.fp16 != 0);
  }
}

// Mean of the keys of one (sequence, chunk, kv head) by one CTA of 256 threads; s_part holds (256 / (D / 8)) * D floats.
__device__ __forceinline__ void chunk_mean_cta(const CacheView& cv, int sid, int chunk, int g, float* s_part, unsigned* status) {
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
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack16(wv[i], cv.fp16 != 0);
        acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
      }
    }
  }
  chunk_mean_finish(cv, sid, chunk, g, acc, s_part);
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
  chunk_mean_cta(cv, sid, chunk, g, s_part, status);
}

// --------------------------------------------------------------------------- prefill hand-off
// Appends whole prompts and writes the means of the chunks they complete in one pass over K: one CTA per (chunk
// touched, kv head, sequence) stores the chunk's new K and V rows into their pages and adds the K rows up as it
// goes (rows of the chunk that were cached before are read back), instead of an append launch over per-token
// (sequence, position) arrays built on the host followed by a second pass over K for the means.
__global__ void __launch_bounds__(256) prefill_to_cache_kernel(CacheView cv, const __nv_bfloat16* __restrict__ k,
                                                               const __nv_bfloat16* __restrict__ v, const int* __restrict__ seqs,
                                                               const int* __restrict__ start, const int* __restrict__ cu,
                                                               unsigned* status) {
  extern __shared__ float s_part[];
  const int s = blockIdx.z, g = blockIdx.y;
  const int sid = seqs[s], first = start[s], src0 = cu[s], last = first + (cu[s + 1] - cu[s]);
  const int chunk = first / cv.C + blockIdx.x;
  const int lo = chunk * cv.C, hi = min(lo + cv.C, last);
  if (lo >= last) return;
  const int upr = cv.D >> 3, rpi = 256 / upr;
  const int ri = threadIdx.x / upr, u = threadIdx.x - ri * upr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (ri < rpi) {
    // four rows per round: table entries, then rows, then stores, so that a round costs three trips, not twelve
    for (int w0 = ri; lo + w0 < hi; w0 += 4 * rpi) {
      long long dst[4];
      bool fresh[4];
      uint4 kr[4], vr[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = lo + w0 + j * rpi;
        dst[j] = -1;
        fresh[j] = t >= first;
        if (t < hi) {
          const int physical = cv.table[(long long)sid * cv.width + t / cv.page];
          if (physical < 0 || physical >= cv.num_pages) {
            if (status) atomicOr(status, kErrBadIndex);
          } else {
            dst[j] = (((long long)physical * cv.page + t % cv.page) * cv.Hkv + g) * cv.D + u * 8;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kr[j] = vr[j] = make_uint4(0u, 0u, 0u, 0u);
        if (dst[j] < 0) continue;
        if (fresh[j]) {
          const long long src = (((long long)src0 + (lo + w0 + j * rpi - first)) * cv.Hkv + g) * cv.D + u * 8;
          kr[j] = *reinterpret_cast<const uint4*>(k + src);
          vr[j] = *reinterpret_cast<const uint4*>(v + src);
        } else {
          kr[j] = *reinterpret_cast<const uint4*>(cv.kc + dst[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // ascending rows: the order of chunk_mean_cta
        if (dst[j] < 0) continue;
        if (fresh[j]) {
          *reinterpret_cast<uint4*>(cv.kc + dst[j]) = kr[j];
          *reinterpret_cast<uint4*>(cv.vc + dst[j]) = vr[j];
        }
        const uint32_t wv[4] = {kr[j].x, kr[j].y, kr[j].z, kr[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack16(wv[i], cv.fp16 != 0);
          acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
        }
      }
    }
  }
  if (hi - lo < cv.C || chunk >= cv.max_chunks) return;  // the chunk is still open
  chunk_mean_finish(cv, sid, chunk, g, acc, s_part);
}

// --------------------------------------------------------------------------- staging of a step's inputs
// Copies the caller's q, k, v of a step into the fixed buffers a captured step reads, as one launch of 16-byte units.
__global__ void __launch_bounds__(256) stage_inputs_kernel(uint4* dq, const uint4* __restrict__ sq, long long nq, uint4* dk,
                                                           const uint4* __restrict__ sk, long long nk, uint4* dv,
                                                           const uint4* __restrict__ sv, long long nv) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < nq) dq[i] = sq[i];
  else if (i < nq + nk) dk[i - nq] = sk[i - nq];
  else if (i < nq + nk + nv) dv[i - nq - nk] = sv[i - nq - nk];
}

// --------------------------------------------------------------------------- first launch of an appending decode step
// Metadata, append and the predicated chunk mean of one request per CTA, and, when the caller hands over the fused
// q/k/v projection instead of separate k and v, the rotary embedding and the split as well: what were four
// launches whose only cost is the wait from one to the next.  rotate-half rotary embedding with cos, sin [rows, D],
// rounding to bf16 where the Hugging Face implementation does.
__global__ void __launch_bounds__(256) decode_step_begin_kernel(CacheView cv, const int* ids, int* positions, const int* delta, int b,
                                                                int Hq, const __nv_bfloat16* qkv, const __nv_bfloat16* cosv,
                                                                const __nv_bfloat16* sinv, __nv_bfloat16* q, __nv_bfloat16* k,
                                                                __nv_bfloat16* v, unsigned* status) {
  // No pointer here is __restrict__ and nothing is read through the read-only path: this grid may start before the
  // kernel that produces its inputs has finished, and a load the compiler may treat as invariant could be moved
  // above the wait below.
  extern __shared__ float s_part[];
  __shared__ int s_sid, s_pos, s_phys;
  const int row = blockIdx.x, tid = threadIdx.x;
  dependents_may_start();
  wait_for_predecessor();  // the projection of the new token
  if (tid == 0) {
    // two trips to memory, not three: the page of the new token is guessed from the previous step's position and
    // its table entry is read together with the length; the guess is checked against the length afterwards
    const int sid = ids[row];
    // positions is read before it is written: whatever it holds before the first step (any int) must not produce an
    // index, so the hint counts only when it is a position this cache can have
    const int hint = positions[row];
    const bool guessed = hint >= 0 && hint < cv.max_seq_len && (hint + 1) / cv.page < cv.width;
    const int guess_page = guessed ? (hint + 1) / cv.page : 0;
    const int logical = delta[row], physical = delta[b + row];
    const int len = cv.lengths[sid];
    const int spec = guessed ? cv.table[(long long)sid * cv.width + guess_page] : -1;
    if (logical >= 0 && logical < cv.width) cv.table[(long long)sid * cv.width + logical] = physical;
    positions[row] = len;
    cv.lengths[sid] = len + 1;
    s_sid = sid; s_pos = len;
    const int page = len / cv.page;
    int phys = -1;
    if (page < cv.width) {
      if (page == logical) phys = physical;                      // opened by this step's delta
      else if (guessed && page == guess_page) phys = spec;
      else phys = cv.table[(long long)sid * cv.width + page];
    }
    s_phys = phys;
  }
  // rotary embedding + split.  With head dimensions that are multiples of 16 a thread takes 8 dimensions of a head
  // (one trip for its four 16-byte loads) and the new K and V rows also stay in shared memory for the append below.
  const int upr = cv.D >> 3;
  const bool vec = qkv && (cv.D & 15) == 0 &&
                   !(((uintptr_t)qkv | (uintptr_t)cosv | (uintptr_t)sinv | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15);
  const bool staged = vec && cv.Hkv * cv.D <= 2048;  // 2 * Hkv * D bf16 fit the 8 KB of s_part
  uint4* s_kv = reinterpret_cast<uint4*>(s_part);    // [K, V][Hkv][D / 8]
  if (vec) {
    const int heads = Hq + 2 * cv.Hkv, D = cv.D;
    const __nv_bfloat16* src = qkv + (long long)row * heads * D;
    for (int item = tid; item < heads * upr; item += 256) {
      const int h = item / upr, c = item - h * upr;
      const uint4 own = *reinterpret_cast<const uint4*>(src + h * D + c * 8);
      if (h >= Hq + cv.Hkv) {
        *reinterpret_cast<uint4*>(v + ((long long)row * cv.Hkv + (h - Hq - cv.Hkv)) * D + c * 8) = own;
        if (staged) s_kv[(cv.Hkv + h - Hq - cv.Hkv) * upr + c] = own;
        continue;
      }
      const bool low = c < (upr >> 1);
      const uint4 oth = *reinterpret_cast<const uint4*>(src + h * D + (low ? c + (upr >> 1) : c - (upr >> 1)) * 8);
      const uint4 cs = *reinterpret_cast<const uint4*>(cosv + (long long)row * D + c * 8);
      const uint4 sn = *reinterpret_cast<const uint4*>(sinv + (long long)row * D + c * 8);
      const uint32_t xw[4] = {own.x, own.y, own.z, own.w}, ow[4] = {oth.x, oth.y, oth.z, oth.w};
      const uint32_t cw[4] = {cs.x, cs.y, cs.z, cs.w}, sw[4] = {sn.x, sn.y, sn.z, sn.w};
      uint32_t out[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __bfloat162float(__float2bfloat16_rn(bf_lo(xw[i]) * bf_lo(cw[i]))) +
                         __bfloat162float(__float2bfloat16_rn((low ? -bf_lo(ow[i]) : bf_lo(ow[i])) * bf_lo(sw[i])));
        const float hi = __bfloat162float(__float2bfloat16_rn(bf_hi(xw[i]) * bf_hi(cw[i]))) +
                         __bfloat162float(__float2bfloat16_rn((low ? -bf_hi(ow[i]) : bf_hi(ow[i])) * bf_hi(sw[i])));
        const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
        out[i] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      const uint4 res = make_uint4(out[0], out[1], out[2], out[3]);
      if (h < Hq) {
        *reinterpret_cast<uint4*>(q + ((long long)row * Hq + h) * D + c * 8) = res;
      } else {
        *reinterpret_cast<uint4*>(k + ((long long)row * cv.Hkv + (h - Hq)) * D + c * 8) = res;
        if (staged) s_kv[(h - Hq) * upr + c] = res;
      }
    }
  } else if (qkv) {
    const int heads = Hq + 2 * cv.Hkv, D = cv.D, half = D >> 1;
    const __nv_bfloat16* src = qkv + (long long)row * heads * D;
    for (int i = tid; i < heads * D; i += 256) {
      const int h = i / D, d = i - h * D;
      if (h >= Hq + cv.Hkv) { v[((long long)row * cv.Hkv + (h - Hq - cv.Hkv)) * D + d] = src[i]; continue; }
      const float x = __bfloat162float(src[i]);
      const float other = __bfloat162float(src[h * D + (d < half ? d + half : d - half)]);
      const float rot = d < half ? -other : other;
      const float c = __bfloat162float(cosv[(long long)row * D + d]), sn = __bfloat162float(sinv[(long long)row * D + d]);
      const __nv_bfloat16 out = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(x * c)) +
                                                    __bfloat162float(__float2bfloat16_rn(rot * sn)));
      if (h < Hq) q[((long long)row * Hq + h) * D + d] = out;
      else k[((long long)row * cv.Hkv + (h - Hq)) * D + d] = out;
    }
  }
  __syncthreads();  // position and page known; this CTA's k and v rows written
  const int sid = s_sid, pos = s_pos, physical = s_phys;
  if (physical < 0 || physical >= cv.num_pages) {
    if (tid == 0 && status) atomicOr(status, kErrBadIndex);
    return;
  }
  for (int i = tid; i < cv.Hkv * upr; i += 256) {
    const int head = i / upr, u = i - head * upr;
    const long long dst = (((long long)physical * cv.page + pos % cv.page) * cv.Hkv + head) * cv.D + u * 8;
    const long long src = ((long long)row * cv.Hkv + head) * cv.D + u * 8;
    *reinterpret_cast<uint4*>(cv.kc + dst) = staged ? s_kv[i] : *reinterpret_cast<const uint4*>(k + src);
    *reinterpret_cast<uint4*>(cv.vc + dst) = staged ? s_kv[cv.Hkv * upr + i] : *reinterpret_cast<const uint4*>(v + src);
  }
  if ((pos + 1) % cv.C != 0) return;  // the token does not complete its chunk
  const int chunk = pos / cv.C;
  if (chunk >= cv.max_chunks) return;
  for (int g = 0; g < cv.Hkv; ++g) {
    __syncthreads();  // the appended row is visible; the previous head is done with the partial sums
    chunk_mean_cta(cv, sid, chunk, g, s_part, status);
  }
}

constexpr int kRouteTile = 64;      // chunk means staged in shared memory per round of decode_route_kernel
constexpr int kRouteThreads = 256;  // eight warps: a group of up to eight heads is ranked in one round

// --------------------------------------------------------------------------- routing (K12, K13, K17, K18)
// One CTA (kRouteThreads threads) per (query row, kv head).  scores[row, h, c] = q . mean[c] in FP32 for the
// chunks completed before the query's own chunk, -inf elsewhere; top-`remote` per head in descending
// score order with the lowest chunk winning exact ties; selected[row, h, :] = (own chunk, picks...,
// -1 padding); and the group's union list (chunk ascending, bitmask of heads) for the attention kernel.
template <bool F16>
__global__ void __launch_bounds__(kRouteThreads) decode_route_kernel(CacheView cv, const __nv_bfloat16* q, const int* ids, const int* positions,
                                                           int Hq, int remote, int width, float* scores, int* selected, int* u_chunk,
                                                           unsigned* u_mask, int* u_count, int umax) {
  // As in decode_step_begin_kernel: no __restrict__, no read-only loads - positions, the query and the chunk means
  // come from kernels this grid may overlap with until the wait below.
  extern __shared__ float s_dyn[];
  dependents_may_start();
  wait_for_predecessor();  // positions, the query, a chunk mean the step's first launch may just have written
  const int G = Hq / cv.Hkv;
  float* s_scores = s_dyn;                                            // [G][width]
  unsigned* s_mask = reinterpret_cast<unsigned*>(s_dyn + G * width);  // [width + 1]
  const int row = blockIdx.x, g = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sid = ids[row], pos = positions[row];
  const int cur = pos / cv.C;
  const int nlegal = min(min(cur, width), cv.max_chunks);
  const int upr = cv.D >> 3;

  for (int i = tid; i <= width; i += kRouteThreads) s_mask[i] = 0u;
  // stage the group's query rows as FP32, then one thread per (head, chunk) pair: the loads of all
  // pairs are independent, so their latencies overlap instead of adding up
  float* s_q = reinterpret_cast<float*>(s_mask + width + 1);  // [G][D]
  // the query loads are issued here and stored after the first tile of means has been requested, so that the two
  // trips to L2 overlap (a store to shared memory would make the warp wait for its load first)
  const __nv_bfloat16* qsrc = q + ((long long)row * Hq + g * G) * cv.D;
  float qreg[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = tid + j * kRouteThreads;
    qreg[j] = i < G * cv.D ? value16(qsrc + i, F16) : 0.f;
  }
  auto store_q = [&]() {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + j * kRouteThreads;
      if (i < G * cv.D) s_q[i] = qreg[j];
    }
    for (int i = tid + 4 * kRouteThreads; i < G * cv.D; i += kRouteThreads) s_q[i] = value16(qsrc + i, F16);
  };
  // The mean rows of kRouteTile chunks at a time are brought into shared memory by all threads with loads that do not
  // depend on each other (one trip to L2 per tile); the (head, chunk) pairs are then scored from there.  Rows are
  // padded to an odd number of 16-byte units so that threads on consecutive chunks hit different banks.
  const int ustride = upr | 1;
  uint4* s_tile = reinterpret_cast<uint4*>(s_dyn + ((G * width + width + 1 + G * cv.D + 3) & ~3));
  for (int c0 = 0; c0 < nlegal; c0 += kRouteTile) {
    const int nt = min(kRouteTile, nlegal - c0);
#pragma unroll 4
    for (int idx = tid; idx < nt * upr; idx += kRouteThreads) {
      const int cl = idx / upr, u = idx - cl * upr;
      s_tile[cl * ustride + u] = __ldcg(
          reinterpret_cast<const uint4*>(cv.means + (((long long)sid * cv.max_chunks + c0 + cl) * cv.Hkv + g) * cv.D) + u);
    }
    if (c0 == 0) store_q();
    __syncthreads();
    for (int pair = tid; pair < G * nt; pair += kRouteThreads) {
      const int hl = pair / nt, cl = pair - hl * nt;
      const uint4* mrow = s_tile + cl * ustride;
      const float* qrow = s_q + hl * cv.D;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      for (int u = 0; u < upr; ++u) {
        const uint4 ma = mrow[u];
        const float* qq = qrow + u * 8;
        const float2 m0 = unpack16<F16>(ma.x), m1 = unpack16<F16>(ma.y), m2 = unpack16<F16>(ma.z), m3 = unpack16<F16>(ma.w);
        a0 = fmaf(qq[0], m0.x, a0); a1 = fmaf(qq[1], m0.y, a1);
        a2 = fmaf(qq[2], m1.x, a2); a3 = fmaf(qq[3], m1.y, a3);
        a0 = fmaf(qq[4], m2.x, a0); a1 = fmaf(qq[5], m2.y, a1);
        a2 = fmaf(qq[6], m3.x, a2); a3 = fmaf(qq[7], m3.y, a3);
      }
      const float sc = (a0 + a1) + (a2 + a3);
      s_scores[hl * width + c0 + cl] = sc;
      if (scores) scores[((long long)row * Hq + g * G + hl) * width + c0 + cl] = sc;
    }
    __syncthreads();
  }
  for (int pair = tid; pair < G * (width - nlegal); pair += kRouteThreads) {  // not a candidate
    const int hl = pair / (width - nlegal), c = nlegal + pair - hl * (width - nlegal);
    s_scores[hl * width + c] = -INFINITY;
    if (scores) scores[((long long)row * Hq + g * G + hl) * width + c] = -INFINITY;
  }
  __syncthreads();
  // top-k: one warp per head, `remote` rounds of (max value, lowest index among equals)
  for (int hl = warp; hl < G; hl += kRouteThreads / 32) {
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

constexpr int kHeadBlock = 16;    // query heads of a group processed together (MMA M dimension)
constexpr int kStageTokens = 64;  // tokens per pipeline stage: 16 per warp
// Two 32 KB stages (D <= 128) and 160 registers let three CTAs share an SM; measured faster than three
// stages with two CTAs when the grid fills the GPU.  A grid of at most one CTA per SM (a batch of one or two
// requests) is bound by latency instead: each stage then costs one trip to memory and one dependent chain of
// math, so that case runs two teams of four warps, each with a ring of its own over half of the part's stages,
// which together have up to a whole 512-token part in flight.
#ifndef MOBA_DEC_STAGES
#define MOBA_DEC_STAGES 2
#endif
#ifndef MOBA_DEC_MINBLOCKS
#define MOBA_DEC_MINBLOCKS 3
#endif
constexpr int kStages = MOBA_DEC_STAGES;  // cp.async stages in flight per CTA, throughput variant
constexpr int deep_stages(int dp) { return dp <= 64 ? 4 : dp <= 128 ? 2 : 3; }  // latency variant, per team (two teams up to D = 128)

// Shared-memory K/V stage: row = one token, DP bf16 values; the 16-byte units of a row are
// XOR-permuted by (token & 7) so that ldmatrix reads of 8 consecutive tokens are conflict-free.
template <int DP>
__device__ __forceinline__ uint32_t kv_unit_offset(int tok, int unit) {
  constexpr int UPR = DP / 8;
  const int sw = UPR >= 8 ? (unit ^ (tok & 7)) : unit;
  return (uint32_t)(tok * DP * 2 + sw * 16);
}

// Row base (element offset of the K/V row of kv head g, or -1) of the token at offset r of logical page pg.  The
// lookup goes through the page table; it is issued one stage ahead of the copy that needs it.  No branch depends
// on the table entry, so several lookups can be in flight; a bad entry is recorded in `bad` and reported later.
__device__ __forceinline__ long long attend_row_base(const CacheView& cv, int sid, int g, int pg, int r, bool exists,
                                                     bool& bad) {
  // an ordinary cached load (a page serves many tokens): not the read-only path, which a dependent launch must avoid
  const int physical = exists ? cv.table[(long long)sid * cv.width + pg] : 0;
  const bool wrong = physical < 0 || physical >= cv.num_pages;
  bad |= wrong;
  return exists && !wrong ? (((long long)physical * cv.page + r) * cv.Hkv + g) * cv.D : -1;
}

// Copies the K and V rows of one stage with cp.async.  Consecutive threads copy consecutive 16-byte
// units of a row, so every 32-byte sector fetched from L2 is used in full; rows that do not exist
// and head-dim padding are zero-filled.
template <int DP>
__device__ __forceinline__ void attend_load_stage(const CacheView& cv, uint8_t* stage, const long long* row_base, int ltid) {
  constexpr int UPR = DP / 8;
  constexpr int ROWS_PER_PASS = 128 / UPR;
  const int u = ltid % UPR, r0 = ltid / UPR;  // ltid: thread within its team of 128
  const uint32_t kdst = smem_u32(stage);
  const uint32_t vdst = kdst + kStageTokens * DP * 2;
  const bool uok = u * 8 < cv.D;
#pragma unroll
  for (int x = 0; x < kStageTokens / ROWS_PER_PASS; ++x) {
    const int tok = r0 + x * ROWS_PER_PASS;
    const long long base = row_base[tok];
    const bool ok = uok && base >= 0;
    const uint32_t off = kv_unit_offset<DP>(tok, u);
    cp_async16(kdst + off, ok ? cv.kc + base + u * 8 : cv.kc, ok);
    cp_async16(vdst + off, ok ? cv.vc + base + u * 8 : cv.vc, ok);
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (F16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- pieces of the merge that are needed only when a head has more partials than fit in shared memory; they
// are functions of their own so that the common path stays short.
struct MergeTail {
  const int* selected;  // null: dense, slot == chunk
  const float *pm, *pl, *pacc;
  int parts, cur, cur_parts, D;
  __device__ __forceinline__ bool valid(long long hbase, int j) const {
    const int sl = j / parts, pt = j - sl * parts;
    const int c = selected ? __ldcg(selected + hbase + sl) : sl;
    return c >= 0 && pt < (c == cur ? cur_parts : parts);
  }
};
// a select, not a branch: stale values where the weight is zero never count and the load stays unconditional
__device__ __forceinline__ void merge_add(float4& v, const float4& x, float w) {
  const bool use = w != 0.f;
  v.x = fmaf(use ? x.x : 0.f, w, v.x); v.y = fmaf(use ? x.y : 0.f, w, v.y);
  v.z = fmaf(use ? x.z : 0.f, w, v.z); v.w = fmaf(use ? x.w : 0.f, w, v.w);
}
__device__ __noinline__ float merge_tail_max(const MergeTail& t, long long hbase, int from, int total, float big) {
  for (int j = from; j < total; j += 16)
    if (t.valid(hbase, j)) big = fmaxf(big, __ldcg(t.pm + hbase * t.parts + j));
  return big;
}
__device__ __noinline__ float merge_tail_den(const MergeTail& t, long long hbase, int from, int total, float big, float lsum) {
  for (int j = from; j < total; j += 16)
    if (t.valid(hbase, j))
      lsum = fmaf(__ldcg(t.pl + hbase * t.parts + j), dec_exp2(__ldcg(t.pm + hbase * t.parts + j) - big), lsum);
  return lsum;
}
// partials [from, to) whose weights are in shared memory but whose sums are not
__device__ __noinline__ float4 merge_rest_acc(const MergeTail& t, long long hbase, int from, int to, int d, const float* wrow,
                                              float4 v) {
  const float4* src = reinterpret_cast<const float4*>(t.pacc + hbase * t.parts * t.D + d);
#pragma unroll 8
  for (int j = from; j < to; ++j) merge_add(v, __ldcg(src + (long long)j * (t.D >> 2)), wrow[j]);
  return v;
}
// partials [from, total) with nothing in shared memory
__device__ __noinline__ float4 merge_tail_acc(const MergeTail& t, long long hbase, int from, int total, int d, float big,
                                              float4 v) {
  const float4* src = reinterpret_cast<const float4*>(t.pacc + hbase * t.parts * t.D + d);
  for (int j = from; j < total; ++j)
    if (t.valid(hbase, j))
      merge_add(v, __ldcg(src + (long long)j * (t.D >> 2)), dec_exp2(__ldcg(t.pm + hbase * t.parts + j) - big));
  return v;
}

// Split-K paged attention for one (query row, kv head, union chunk, part).  The query heads of the
// GQA group are the 16 rows of m16n8k16 tensor-core tiles (unused rows are zero), so a K/V token read
// from HBM serves every head at no extra cost and the kernel stays memory bound for any group size.
// Each warp takes 16 tokens of every 64-token stage and keeps its own running (max, sum, O); the
// warps are combined through shared memory at the end.  A team is four warps with a copy ring and a barrier of its
// own; the latency variant runs two teams, each on half of the part's stages, because with one warp per scheduler
// nothing hides the dependent chain of a stage (ldmatrix, mma, shuffles, exp2, mma).
template <int DP, int NS, int TEAMS, bool F16>
__global__ void __launch_bounds__(128 * TEAMS, (TEAMS == 1 && DP <= 128 ? MOBA_DEC_MINBLOCKS : 1)) decode_attend_kernel(AttendArgs a) {
  constexpr int NT = 128 * TEAMS, NW = 4 * TEAMS;  // threads and warps of the CTA
  constexpr int KSTEPS = DP / 16;
  constexpr int DT = DP / 8;  // 8-column output tiles
  constexpr int STAGE_BYTES = 2 * kStageTokens * DP * 2;
  extern __shared__ __align__(128) uint8_t s_pipe[];  // NS stages per team; reused for the cross-warp reduction
  __shared__ int s_last, s_slot[kHeadBlock];
  __shared__ long long s_rowbase_all[TEAMS][NS][kStageTokens];
  dependents_may_start();   // e.g. the output projection, whose weight loads need nothing from here
  wait_for_predecessor();   // routes, positions, the appended row
  const CacheView& cv = a.cv;
  const int D = cv.D, G = a.Hq / cv.Hkv;
  const int rowg = blockIdx.z, row = rowg / cv.Hkv, g = rowg - row * cv.Hkv;
  const int k = blockIdx.x, part = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int team = warp >> 2, wt = warp & 3, ltid = tid & 127;  // team, warp in the team, thread in the team
  long long (*s_rowbase)[kStageTokens] = s_rowbase_all[team];
  uint8_t* const t_pipe = s_pipe + (size_t)team * NS * STAGE_BYTES;
  auto team_sync = [&]() {
    if (TEAMS == 1) __syncthreads();
    else asm volatile("bar.sync %0, 128;" ::"r"(team + 1) : "memory");
  };
  const int qr = lane >> 2, qc = lane & 3;  // fragment row within 8 and column pair
  const int sid = a.ids[row], pos = a.positions[row];
  const int visible = min(pos + 1, cv.lengths[sid]);  // tokens [0, visible) exist and are not in the future
  const int cur = pos / cv.C;
  const bool dense = a.selected == nullptr;
  // the union entry of this CTA is read together with the count (k < umax always), not after the test on the count
  const int listed = dense ? 0 : a.u_chunk[(long long)rowg * a.umax + k];
  const unsigned listed_mask = dense ? 0u : a.u_mask[(long long)rowg * a.umax + k];
  const int ucount = dense ? cur + 1 : a.u_count[rowg];
  if (k >= ucount) return;
  const int chunk = dense ? k : listed;
  const unsigned mask = dense ? (G >= 32 ? 0xFFFFFFFFu : ((1u << G) - 1u)) : listed_mask;
  const int limit = min((chunk + 1) * cv.C, visible);
  const int t_begin = chunk * cv.C + part * a.part_tokens;
  const int t_end = min(t_begin + a.part_tokens, limit);
  if (t_begin >= t_end) return;
  const int cur_parts = (visible - cur * cv.C + a.part_tokens - 1) / a.part_tokens;
  const int expected = (ucount - 1) * a.parts + cur_parts;
  const int all_tiles = (t_end - t_begin + kStageTokens - 1) / kStageTokens;
  const int first_tile = team * ((all_tiles + TEAMS - 1) / TEAMS);           // this team's stages: [first_tile, first_tile + ntiles)
  const int ntiles = max(0, min(all_tiles - first_tile, (all_tiles + TEAMS - 1) / TEAMS));
  const int tt_begin = t_begin + first_tile * kStageTokens;                  // first token of the team

  for (int hb = 0; hb < G; hb += kHeadBlock) {
    const unsigned active = (mask >> hb) & 0xFFFFu;
    if (!active) continue;
    // row bases of the tokens of the stages about to be copied (ring of NS slots).  A thread looks up one token
    // of every stage; from stage to stage the token advances by kStageTokens, so page and offset are stepped
    // instead of divided anew.
    int look_t = tt_begin + ltid, look_pg = 0, look_r = 0, step_pg = 0, step_r = 0;
    bool look_bad = false;
    if (ltid < kStageTokens) {
      look_pg = look_t / cv.page; look_r = look_t - look_pg * cv.page;
      step_pg = kStageTokens / cv.page; step_r = kStageTokens - step_pg * cv.page;
    }
    auto lookup = [&]() {
      const long long base = attend_row_base(cv, sid, g, look_pg, look_r, look_t < t_end, look_bad);
      look_t += kStageTokens; look_pg += step_pg; look_r += step_r;
      if (look_r >= cv.page) { look_r -= cv.page; ++look_pg; }
      return base;
    };
    long long first_base[NS];  // issued before the query loads below, stored after them
    if (ltid < kStageTokens) {
#pragma unroll
      for (int s = 0; s < NS; ++s) first_base[s] = lookup();
    }
    // Q fragments (A operand): rows qr and qr+8 of the head block, all k-steps
    uint32_t qf[KSTEPS][4];
    {
      const bool r0 = hb + qr < G && ((active >> qr) & 1u), r1 = hb + qr + 8 < G && ((active >> (qr + 8)) & 1u);
      const __nv_bfloat16* q0 = a.q + ((long long)row * a.Hq + g * G + hb + qr) * D;
      const __nv_bfloat16* q1 = q0 + 8 * D;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int c0 = ks * 16 + qc * 2, c1 = c0 + 8;
        qf[ks][0] = (r0 && c0 < D) ? *reinterpret_cast<const uint32_t*>(q0 + c0) : 0u;
        qf[ks][1] = (r1 && c0 < D) ? *reinterpret_cast<const uint32_t*>(q1 + c0) : 0u;
        qf[ks][2] = (r0 && c1 < D) ? *reinterpret_cast<const uint32_t*>(q0 + c1) : 0u;
        qf[ks][3] = (r1 && c1 < D) ? *reinterpret_cast<const uint32_t*>(q1 + c1) : 0u;
      }
    }
    float o[DT][4];
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows qr and qr+8; l: this thread's columns only

    __syncthreads();  // the previous head block is done with shared memory
    if (ltid < kStageTokens) {
#pragma unroll
      for (int s = 0; s < NS; ++s) s_rowbase[s][ltid] = first_base[s];
    }
    team_sync();
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
      if (s < ntiles) attend_load_stage<DP>(cv, t_pipe + s * STAGE_BYTES, s_rowbase[s], ltid);
      cp_async_commit();
    }
    for (int i = 0; i < ntiles; ++i) {
      cp_async_wait<NS - 2>();
      team_sync();  // tile i has landed; every warp of the team finished tile i-1, whose buffer is refilled next
      const int nx = i + NS - 1;
      if (nx < ntiles) attend_load_stage<DP>(cv, t_pipe + (nx % NS) * STAGE_BYTES, s_rowbase[nx % NS], ltid);
      cp_async_commit();
      // look up the rows of tile nx+1 now, publish them after this tile's math (slot i % NS is free)
      long long next_base = -1;
      if (ltid < kStageTokens && nx + 1 < ntiles) next_base = lookup();
      const int tok0 = wt * 16;                                   // this warp's tokens inside the stage
      const int nvalid = t_end - (tt_begin + i * kStageTokens + tok0);  // tokens of the warp tile that exist
      if (nvalid <= 0) {                                          // warp-uniform
        if (ltid < kStageTokens) s_rowbase[i % NS][ltid] = next_base;
        continue;
      }
      const uint32_t kbase = smem_u32(t_pipe + (i % NS) * STAGE_BYTES);
      const uint32_t vbase = kbase + kStageTokens * DP * 2;
      // ---- S = Q K^T for 16 tokens: two 8-token column tiles
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t b[4];
        const int mat = lane >> 3, r = lane & 7;
        ldmatrix_x4(kbase + kv_unit_offset<DP>(tok0 + (mat >> 1) * 8 + r, ks * 2 + (mat & 1)), b);
        mma_16816<F16>(sc[0], qf[ks], b[0], b[1]);
        mma_16816<F16>(sc[1], qf[ks], b[2], b[3]);
      }
      // ---- online softmax of rows qr / qr+8 (exp2 domain)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = nt * 8 + qc * 2 + (e & 1);
          sc[nt][e] = col < nvalid ? sc[nt][e] * a.scale_log2 : -INFINITY;
        }
      }
      float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);  // finite: column 0 of the warp tile always exists
      const float al0 = dec_exp2(m0 - n0), al1 = dec_exp2(m1 - n1);
      m0 = n0; m1 = n1;
      uint32_t pf[4];
      {
        const float p00 = dec_exp2(sc[0][0] - n0), p01 = dec_exp2(sc[0][1] - n0), p02 = dec_exp2(sc[0][2] - n1), p03 = dec_exp2(sc[0][3] - n1);
        const float p10 = dec_exp2(sc[1][0] - n0), p11 = dec_exp2(sc[1][1] - n0), p12 = dec_exp2(sc[1][2] - n1), p13 = dec_exp2(sc[1][3] - n1);
        l0 = l0 * al0 + (p00 + p01) + (p10 + p11);
        l1 = l1 * al1 + (p02 + p03) + (p12 + p13);
        pf[0] = pack16<F16>(p00, p01); pf[1] = pack16<F16>(p02, p03);
        pf[2] = pack16<F16>(p10, p11); pf[3] = pack16<F16>(p12, p13);
      }
      // ---- O = O * alpha + P V; the running maxima rarely move after the first tiles, and alpha == 1 needs no pass over O
      const bool rescale = __any_sync(0xFFFFFFFFu, al0 != 1.f || al1 != 1.f);
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        uint32_t b[4];
        const int mat = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(vbase + kv_unit_offset<DP>(tok0 + (mat & 1) * 8 + r, dp * 2 + (mat >> 1)), b);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float (&acc)[4] = o[dp * 2 + h2];
          if (rescale) { acc[0] *= al0; acc[1] *= al0; acc[2] *= al1; acc[3] *= al1; }
          mma_16816<F16>(acc, pf, b[h2 * 2], b[h2 * 2 + 1]);
        }
      }
      if (ltid < kStageTokens) s_rowbase[i % NS][ltid] = next_base;
    }
    if (look_bad) atomicOr(a.status, kErrBadIndex);
    // ---- combine the warps, then write one partial per active head
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 1); l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, 2);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 1); l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, 2);
    __syncthreads();
    float* s_o = reinterpret_cast<float*>(s_pipe);                   // [NW warps][16 rows][DP]
    float* s_ml = s_o + NW * 16 * DP;                                 // [NW warps][16 rows][2]
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      float* w0 = s_o + ((size_t)warp * 16 + qr) * DP + dt * 8 + qc * 2;
      float* w1 = w0 + 8 * DP;
      w0[0] = o[dt][0]; w0[1] = o[dt][1]; w1[0] = o[dt][2]; w1[1] = o[dt][3];
    }
    if (qc == 0) {
      s_ml[((size_t)warp * 16 + qr) * 2] = m0; s_ml[((size_t)warp * 16 + qr) * 2 + 1] = l0;
      s_ml[((size_t)warp * 16 + qr + 8) * 2] = m1; s_ml[((size_t)warp * 16 + qr + 8) * 2 + 1] = l1;
    }
    // slot of this chunk in each head's route (all candidate slots are read before any is compared)
    const int nh = min(kHeadBlock, G - hb);
    if (tid < kHeadBlock) {
      int slot = -1;
      if (tid < nh && ((active >> tid) & 1u)) {
        if (dense) {
          slot = chunk;
        } else {
          const int* sel = a.selected + ((long long)row * a.Hq + g * G + hb + tid) * a.ns;
#pragma unroll 4
          for (int s2 = a.ns - 1; s2 >= 0; --s2)
            if (__ldcg(sel + s2) == chunk) slot = s2;
        }
      }
      s_slot[tid] = slot;
    }
    __syncthreads();
    // every thread takes two dimensions of one head
    const int d2n = D >> 1;
    for (int item = tid; item < nh * d2n; item += NT) {
      const int hh = item / d2n, d = (item - hh * d2n) * 2;
      const int slot = s_slot[hh];
      if (slot < 0) continue;
      const int h = g * G + hb + hh;
      const long long pidx = (((long long)row * a.Hq + h) * a.ns + slot) * a.parts + part;
      float mw[NW], big = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) { mw[w] = s_ml[((size_t)w * 16 + hh) * 2]; big = fmaxf(big, mw[w]); }
      float lsum = 0.f, v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float wgt = mw[w] == -INFINITY ? 0.f : dec_exp2(mw[w] - big);  // a warp that saw no token adds nothing
        lsum += s_ml[((size_t)w * 16 + hh) * 2 + 1] * wgt;
        const float2 x = *reinterpret_cast<const float2*>(s_o + ((size_t)w * 16 + hh) * DP + d);
        v0 += x.x * wgt; v1 += x.y * wgt;
      }
      *reinterpret_cast<float2*>(a.pacc + pidx * D + d) = make_float2(v0, v1);
      if (d == 0) { a.pm[pidx] = big; a.pl[pidx] = lsum; }
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
  // The partials of a head are (slot, part) pairs, j = slot * parts + part, and lie one after the other.  All
  // threads first start asynchronous copies of the partial sums into shared memory, as many partials per head as
  // fit, and read the maxima and denominators of every head's partials, all with accesses that do not depend on
  // each other: one trip to L2 for the whole merge.  One warp per head then finds the maximum, the weights and the
  // denominator; finally every thread takes four dimensions of one head and sums over the partials.  What does not
  // fit in shared memory is read from global memory in the same fixed order, so the result is bit-repeatable.
  const int nslots = dense ? cur + 1 : a.ns;
  const int total = nslots * a.parts;
  const int pipe_floats = TEAMS * NS * STAGE_BYTES / 4;
  const int cap = min(min(1024, (total + 3) & ~3), (pipe_floats / (2 * G)) & ~3);  // maxima / weights kept per head
  const int tc = min(total, cap);
  const int pb = min(tc, (pipe_floats - 2 * G * cap) / (G * D));                   // partial sums kept per head
  float* s_w = reinterpret_cast<float*>(s_pipe);  // [G][cap] maxima, then weights
  float* s_l = s_w + G * cap;                       // [G][cap] denominators
  float* s_acc = s_l + G * cap;                     // [G][pb][D] partial sums
  __shared__ float s_big[32], s_inv[32];
  const int d4n = D >> 2;  // the head dimension is a multiple of 8
  const long long gbase = ((long long)row * a.Hq + g * G) * a.ns;  // first slot of the group's first head
  for (int hl = 0; hl < G; ++hl) {
    const float* src = a.pacc + (gbase + (long long)hl * a.ns) * a.parts * D;
    const uint32_t dst = smem_u32(s_acc + (size_t)hl * pb * D);
    for (int u = tid; u < pb * d4n; u += NT) cp_async16(dst + u * 16, src + u * 4, true);
  }
  cp_async_commit();
  // This code runs once per launch in one CTA per group, from a cold instruction cache: it is kept short (little
  // unrolling; the rarely needed paths sit in functions of their own) because fetching it costs more than running it.
  const MergeTail tail{a.selected, a.pm, a.pl, a.pacc, a.parts, cur, cur_parts, D};
#pragma unroll 2
  for (int idx = tid; idx < G * tc; idx += NT) {
    const int hl = idx / tc, j = idx - hl * tc;
    const long long hbase = gbase + (long long)hl * a.ns;
    const float m = __ldcg(a.pm + hbase * a.parts + j), l = __ldcg(a.pl + hbase * a.parts + j);
    const bool ok = tail.valid(hbase, j);
    s_w[hl * cap + j] = ok ? m : -INFINITY;
    s_l[hl * cap + j] = ok ? l : 0.f;
  }
  cp_async_wait<0>();
  __syncthreads();
  // half a warp per head
  const int sub = lane & 15;
#pragma unroll 1
  for (int hl = warp * 2 + (lane >> 4); hl < ((G + 2 * NW - 1) / (2 * NW)) * (2 * NW); hl += 2 * NW) {
    const bool live = hl < G;  // the shuffles below need every lane
    const int hc = live ? hl : 0;
    const int h = g * G + hc;
    const long long hbase = gbase + (long long)hc * a.ns;
    float big = -INFINITY;
    if (live) {
#pragma unroll 1
      for (int j = sub; j < tc; j += 16) big = fmaxf(big, s_w[hc * cap + j]);
      if (total > cap) big = merge_tail_max(tail, hbase, cap + sub, total, big);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xFFFFFFFFu, big, o));
    float lsum = 0.f;
    if (live) {
#pragma unroll 1
      for (int j = sub; j < tc; j += 16) {
        const float m = s_w[hc * cap + j];
        const float w = m == -INFINITY ? 0.f : dec_exp2(m - big);
        s_w[hc * cap + j] = w;
        lsum = fmaf(s_l[hc * cap + j], w, lsum);
      }
      if (total > cap) lsum = merge_tail_den(tail, hbase, cap + sub, total, big, lsum);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, o);
    if (live && sub == 0) {
      s_big[hc] = big;
      s_inv[hc] = 1.f / lsum;
      a.lse[(long long)row * a.Hq + h] = (big + log2f(lsum)) * 0.6931471805599453f;
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int item = tid; item < G * d4n; item += NT) {
    const int hl = item / d4n, d = (item - hl * d4n) * 4;
    const int h = g * G + hl;
    const long long hbase = gbase + (long long)hl * a.ns;
    const float* wrow = s_w + hl * cap;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* sacc = reinterpret_cast<const float4*>(s_acc + (size_t)hl * pb * D + d);
#pragma unroll 4
    for (int j = 0; j < pb; ++j) merge_add(v, sacc[(size_t)j * d4n], wrow[j]);
    if (tc > pb) v = merge_rest_acc(tail, hbase, pb, tc, d, wrow, v);
    if (total > cap) v = merge_tail_acc(tail, hbase, cap, total, d, s_big[hl], v);
    const float inv = s_inv[hl];
    uint2 pk;
    pk.x = pack16<F16>(v.x * inv, v.y * inv);
    pk.y = pack16<F16>(v.z * inv, v.w * inv);
    *reinterpret_cast<uint2*>(a.out + ((long long)row * a.Hq + h) * D + d) = pk;
  }
  __syncthreads();
  if (tid == 0) a.counters[rowg] = 0;  // ready for the next launch (graph replay included)
}

}  // namespace moba

using namespace moba;

static int decode_sm_count() {
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

extern "C" int moba_decode_metadata(const moba_cache_desc* c, const int32_t* ids, int32_t* positions, const int32_t* delta,
                                    int rows, int append, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!ids || !positions || !delta || rows < 1) return MOBA_ERR_INVALID;
  decode_metadata_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(make_cache_view(*c), ids, positions, delta, rows, append);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_cache_update(const moba_cache_desc* c, const int32_t* edits, int n, const int32_t* ids, const int32_t* lengths_new,
                                 int m, int clear_rows, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (n < 0 || m < 0 || (n > 0 && !edits) || (m > 0 && (!ids || !lengths_new)) || (clear_rows && n > 0)) return MOBA_ERR_INVALID;
  if (n == 0 && m == 0) return MOBA_OK;
  long long work = n > m ? n : m;
  if (clear_rows) work = (long long)m * c->table_width;
  const unsigned blocks = (unsigned)((work + 255) / 256 < 1024 ? (work + 255) / 256 : 1024);
  const unsigned min_blocks = (unsigned)(((n > m ? n : m) + 255) / 256);
  cache_update_kernel<<<blocks > min_blocks ? blocks : min_blocks, 256, 0, (cudaStream_t)stream>>>(make_cache_view(*c), edits, n, ids,
                                                                                                   lengths_new, m, clear_rows);
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

extern "C" int moba_prefill_to_cache(const moba_cache_desc* c, const void* k, const void* v, const int32_t* seqs, const int32_t* start,
                                     const int32_t* cu_seqlens, int num_seqs, int max_chunks_touched, unsigned* status,
                                     void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!k || !v || !seqs || !start || !cu_seqlens || num_seqs < 1 || num_seqs > 65535 || max_chunks_touched < 1)
    return MOBA_ERR_INVALID;
  const int rpi = 256 / (c->dim / 8);
  prefill_to_cache_kernel<<<dim3(max_chunks_touched, c->hkv, num_seqs), 256, (size_t)rpi * c->dim * 4, (cudaStream_t)stream>>>(
      make_cache_view(*c), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), seqs, start, cu_seqlens,
      status);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_stage_inputs(void* q_dst, const void* q_src, size_t q_bytes, void* k_dst, const void* k_src, size_t k_bytes,
                                        void* v_dst, const void* v_src, size_t v_bytes, void* stream) {
  if ((q_bytes && (!q_dst || !q_src)) || (k_bytes && (!k_dst || !k_src)) || (v_bytes && (!v_dst || !v_src)))
    return MOBA_ERR_INVALID;
  if ((q_bytes | k_bytes | v_bytes) & 15) return MOBA_ERR_UNSUPPORTED;
  if (((uintptr_t)q_dst | (uintptr_t)q_src | (uintptr_t)k_dst | (uintptr_t)k_src | (uintptr_t)v_dst | (uintptr_t)v_src) & 15)
    return MOBA_ERR_UNSUPPORTED;
  const long long nq = (long long)(q_bytes >> 4), nk = (long long)(k_bytes >> 4), nv = (long long)(v_bytes >> 4);
  const long long total = nq + nk + nv;
  if (total == 0) return MOBA_OK;
  stage_inputs_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      static_cast<uint4*>(q_dst), static_cast<const uint4*>(q_src), nq, static_cast<uint4*>(k_dst), static_cast<const uint4*>(k_src), nk,
      static_cast<uint4*>(v_dst), static_cast<const uint4*>(v_src), nv);
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

extern "C" int moba_decode_step_begin(const moba_cache_desc* c, const int32_t* ids, int32_t* positions, const int32_t* delta, int rows,
                                      int hq, const void* qkv, const void* cosv, const void* sinv, void* q, void* k, void* v,
                                      unsigned* status, void* stream) {
  int rc = validate_cache(c);
  if (rc != MOBA_OK) return rc;
  if (!ids || !positions || !delta || !k || !v || rows < 1) return MOBA_ERR_INVALID;
  if (qkv && (!cosv || !sinv || !q || hq < 1 || hq % c->hkv || (c->dim & 1))) return MOBA_ERR_INVALID;
  if (qkv && (c->flags & MOBA_CACHE_FP16)) return MOBA_ERR_UNSUPPORTED;  // the rotary step rounds as the bf16 modules do
  const int rpi = 256 / (c->dim / 8);
  if (launch_dependent(2u, decode_step_begin_kernel, dim3(rows), dim3(256), (size_t)rpi * c->dim * 4, (cudaStream_t)stream,
                       make_cache_view(*c), ids, positions, delta, rows, hq, static_cast<const __nv_bfloat16*>(qkv),
                       static_cast<const __nv_bfloat16*>(cosv), static_cast<const __nv_bfloat16*>(sinv),
                       static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
                       status) != cudaSuccess)
    return MOBA_ERR_CUDA;
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
  const size_t smem = ((((size_t)G * width + width + 1 + (size_t)G * c->dim + 3) & ~(size_t)3)) * 4 +
                      (size_t)kRouteTile * ((c->dim / 8) | 1) * 16;
  if (smem > 200 * 1024) return MOBA_ERR_UNSUPPORTED;
  const auto kernel = (c->flags & MOBA_CACHE_FP16) ? decode_route_kernel<true> : decode_route_kernel<false>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return MOBA_ERR_CUDA;
  const int umax = moba_decode_union_capacity(hq, c->hkv, remote, width);
  if (launch_dependent(4u, kernel, dim3(rows, c->hkv), dim3(kRouteThreads), smem, (cudaStream_t)stream, make_cache_view(*c),
                       static_cast<const __nv_bfloat16*>(q), ids, positions, hq, remote, width, scores, selected, u_chunk, u_mask,
                       u_count, umax) != cudaSuccess)
    return MOBA_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}

static int attend_part_tokens(const moba_cache_desc* c) {
  return c->chunk_size >= 2048 ? 1024 : c->chunk_size >= 512 ? 512 : c->chunk_size;
}
static int attend_parts(const moba_cache_desc* c) {
  const int part_tokens = attend_part_tokens(c);
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
  if (c->chunk_size >= 512 && attend_part_tokens(c) % kStageTokens) return MOBA_ERR_UNSUPPORTED;
  if (workspace_bytes < moba_decode_attend_workspace_bytes(c, rows, hq, slots)) return MOBA_ERR_WORKSPACE;
  AttendArgs a;
  a.cv = make_cache_view(*c);
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.ids = ids; a.positions = positions; a.selected = selected;
  a.u_chunk = u_chunk; a.u_mask = u_mask; a.u_count = u_count;
  a.Hq = hq; a.ns = slots; a.umax = selected ? umax : slots;
  a.parts = attend_parts(c);
  a.part_tokens = attend_part_tokens(c);
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
  const int dp = c->dim <= 32 ? 32 : c->dim <= 64 ? 64 : c->dim <= 128 ? 128 : 256;
  const dim3 grid(a.umax, a.parts, rows * c->hkv);
  const bool deep = (long long)grid.x * grid.y * grid.z <= decode_sm_count();
  const int teams = deep && dp <= 128 ? 2 : 1;
  const int stages = deep ? deep_stages(dp) : kStages;  // per team
  const size_t red_bytes = (size_t)4 * teams * 16 * (dp + 2) * 4;
  const size_t pipe_bytes = (size_t)teams * stages * 2 * kStageTokens * dp * 2;
  const size_t smem = red_bytes > pipe_bytes ? red_bytes : pipe_bytes;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  const bool half = (c->flags & MOBA_CACHE_FP16) != 0;
  prof_begin(kProfDecodeAttend, st);
#define MOBA_LAUNCH_ATTEND_F(L, NS, T, F)                                                                               \
  do {                                                                                                                  \
    e = cudaFuncSetAttribute(decode_attend_kernel<L, NS, T, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e == cudaSuccess) e = launch_dependent(8u, decode_attend_kernel<L, NS, T, F>, grid, dim3(128 * T), smem, st, a); \
  } while (0)
#define MOBA_LAUNCH_ATTEND_NS(L, NS, T)             \
  do {                                              \
    if (half) MOBA_LAUNCH_ATTEND_F(L, NS, T, true); \
    else MOBA_LAUNCH_ATTEND_F(L, NS, T, false);     \
  } while (0)
#define MOBA_LAUNCH_ATTEND(L)                                                                                      \
  do {                                                                                                             \
    if (deep) MOBA_LAUNCH_ATTEND_NS(L, deep_stages(L), (L <= 128 ? 2 : 1));                                        \
    else MOBA_LAUNCH_ATTEND_NS(L, kStages, 1);                                                                     \
  } while (0)
  if (dp == 32) MOBA_LAUNCH_ATTEND(32);
  else if (dp == 64) MOBA_LAUNCH_ATTEND(64);
  else if (dp == 128) MOBA_LAUNCH_ATTEND(128);
  else MOBA_LAUNCH_ATTEND(256);
#undef MOBA_LAUNCH_ATTEND_NS
#undef MOBA_LAUNCH_ATTEND_F
#undef MOBA_LAUNCH_ATTEND
  prof_end(kProfDecodeAttend, st);
  if (e != cudaSuccess) return MOBA_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? MOBA_OK : MOBA_ERR_CUDA;
}
