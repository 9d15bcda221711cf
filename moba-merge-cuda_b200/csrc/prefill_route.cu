// Prefill routing: chunk mean-pool of K, FP32 gate q . mean, deterministic top-k, and the
// per-expert query lists.  Replaces the torch-op routing and packing of the reference
// (src/moba_opt/grouped_attention.py:48-94): nothing of size [F, Hq, T] is materialised, there
// is no host synchronisation, and every list is produced in a fixed order (head in group, token).
//
// Passes (all on one stream):
//   1. chunk_mean_kernel     means[c, g, :] = mean over the tokens of chunk c (FP32 accumulation)
//   2. gate_topk_kernel      per (token, q head): scores against the earlier chunks of the same
//                            sequence, top-R with "lowest chunk wins ties", sel[T,Hq,R] ascending;
//                            per (query tile, q head, chunk) selection counts
//   3. segment_scan_kernel   per (chunk, q head): exclusive scan of the counts over query tiles
//   4. plan_kernel           segment bases and per-expert tile bases (exclusive scans)
//   5. fill_kernel           writes slot ids into rowlist at base + tile offset + rank in tile
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

constexpr int kCandBatch = 32;  // candidate means staged in shared memory per pass

// --------------------------------------------------------------------------- 1. chunk means
__global__ void __launch_bounds__(256) chunk_mean_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ k,
                                                         float* __restrict__ means, int round_bf16) {
  extern __shared__ float s_part[];  // [rows_per_iter][D]
  const int c = blockIdx.x, g = blockIdx.y;
  const int t0 = pv.chunk_start[c], t1 = pv.chunk_start[c + 1];
  const int upr = pv.D >> 3;
  const int rpi = 256 / upr;
  const int ri = threadIdx.x / upr, u = threadIdx.x - ri * upr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (ri < rpi) {
    for (int t = t0 + ri; t < t1; t += rpi) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + (long long)t * pv.k_st + (long long)g * pv.k_sh + u * 8);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(w[i] << 16);
        acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_part[ri * pv.D + u * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < pv.D; d += 256) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += s_part[r * pv.D + d];
    float m = s / (float)(t1 - t0);
    if (round_bf16) m = __bfloat162float(__float2bfloat16_rn(m));
    means[((long long)c * pv.Hkv + g) * pv.D + d] = m;
  }
}

// --------------------------------------------------------------------------- 2. gate + top-k
template <int RT>
__global__ void __launch_bounds__(128) gate_topk_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ q,
                                                        const float* __restrict__ means, int* __restrict__ sel,
                                                        int* __restrict__ cnt) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int D = pv.D, R = pv.R;
  const int qrow_bytes = D * 2 + 16;  // padded so that per-thread row reads are conflict-free
  float* s_means = reinterpret_cast<float*>(smem);                        // [kCandBatch][D]
  uint8_t* s_q = smem + (size_t)kCandBatch * D * 4;                       // [128][qrow_bytes]
  int* s_cnt = reinterpret_cast<int*>(s_q + (size_t)kTile * qrow_bytes);  // [ncand]

  const int tile = blockIdx.x, g = blockIdx.y;
  const int c = pv.qtile_chunk[tile];
  const int tok0 = pv.qtile_tok0[tile];
  const int ncand = pv.chunk_local[c];
  const int c0 = c - ncand;
  const int chunk_end = pv.chunk_start[c + 1];
  const int nrows = min(kTile, chunk_end - tok0);
  const int tid = threadIdx.x;
  const int t = tok0 + tid;
  const bool valid = tid < nrows;
  const int upr = D >> 3;
  const int tile_local = pv.qtile_local[tile];

  for (int hl = 0; hl < pv.G; ++hl) {
    const int h = g * pv.G + hl;
    float topv[RT];
    int topi[RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) { topv[i] = -INFINITY; topi[i] = -1; }

    if (ncand > 0) {
      __syncthreads();  // previous head's s_q / s_cnt readers are done
      for (int i = tid; i < nrows * upr; i += 128) {
        const int r = i / upr, u = i - r * upr;
        cp_async16(smem_u32(s_q + (size_t)r * qrow_bytes + u * 16),
                   q + (long long)(tok0 + r) * pv.q_st + (long long)h * pv.q_sh + u * 8, true);
      }
      cp_async_commit();
      for (int i = tid; i < ncand; i += 128) s_cnt[i] = 0;
      for (int cb = 0; cb < ncand; cb += kCandBatch) {
        const int nb = min(kCandBatch, ncand - cb);
        __syncthreads();  // previous batch consumed
        for (int i = tid; i < nb * (D >> 2); i += 128)
          reinterpret_cast<float4*>(s_means)[i] =
              *reinterpret_cast<const float4*>(means + ((long long)(c0 + cb + i / (D >> 2)) * pv.Hkv + g) * D + (i % (D >> 2)) * 4);
        cp_async_wait<0>();
        __syncthreads();
        if (valid) {
          const uint8_t* qrow = s_q + (size_t)tid * qrow_bytes;
          for (int ci = 0; ci < nb; ++ci) {
            const float* m = s_means + ci * D;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (int u = 0; u < upr; ++u) {
              const uint4 raw = *reinterpret_cast<const uint4*>(qrow + u * 16);
              const float4 m0 = *reinterpret_cast<const float4*>(m + u * 8);
              const float4 m1 = *reinterpret_cast<const float4*>(m + u * 8 + 4);
              a0 = fmaf(__uint_as_float(raw.x << 16), m0.x, a0);
              a1 = fmaf(__uint_as_float(raw.x & 0xFFFF0000u), m0.y, a1);
              a2 = fmaf(__uint_as_float(raw.y << 16), m0.z, a2);
              a3 = fmaf(__uint_as_float(raw.y & 0xFFFF0000u), m0.w, a3);
              a0 = fmaf(__uint_as_float(raw.z << 16), m1.x, a0);
              a1 = fmaf(__uint_as_float(raw.z & 0xFFFF0000u), m1.y, a1);
              a2 = fmaf(__uint_as_float(raw.w << 16), m1.z, a2);
              a3 = fmaf(__uint_as_float(raw.w & 0xFFFF0000u), m1.w, a3);
            }
            const float score = (a0 + a1) + (a2 + a3);
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
      }
    }
    // keep the R best, emit them in ascending chunk order
    if (valid) {
      int last = -1;
      int* out = sel + ((long long)t * pv.Hq + h) * R;
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
    if (ncand > 0) {
      __syncthreads();
      for (int i = tid; i < ncand; i += 128)
        cnt[((long long)(c0 + i) * pv.Hq + h) * pv.max_tiles_per_seq + tile_local] = s_cnt[i];
    }
  }
}

// --------------------------------------------------------------------------- 3. scan over query tiles
__global__ void __launch_bounds__(128) segment_scan_kernel(PrefillView pv, int* __restrict__ cnt, int* __restrict__ seg_count) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= pv.n_chunks * pv.Hq) return;
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

// --------------------------------------------------------------------------- 4. bases
// Single block.  seg_base[i] = sum of seg_count[<i]; tile_base[e] = sum over experts < e of
// ceil(rows(e) / 128) rounded up to even, with expert e = chunk * Hkv + kv head.
__global__ void __launch_bounds__(1024) plan_kernel(PrefillView pv, const int* __restrict__ seg_count,
                                                    int* __restrict__ seg_base, int* __restrict__ tile_base) {
  __shared__ int s_part[1024];
  __shared__ int s_total;
  const int tid = threadIdx.x;
  for (int pass = 0; pass < 2; ++pass) {
    const int n = pass == 0 ? pv.n_chunks * pv.Hq : pv.n_chunks * pv.Hkv;
    int* out = pass == 0 ? seg_base : tile_base;
    const int per = (n + 1023) / 1024;
    const int lo = min(n, tid * per), hi = min(n, lo + per);
    auto value = [&](int i) {
      if (pass == 0) return seg_count[i];
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
      s_total = run;
    }
    __syncthreads();
    int run = s_part[tid];
    for (int i = lo; i < hi; ++i) { out[i] = run; run += value(i); }
    if (tid == 0) out[n] = s_total;
    __threadfence_block();
    __syncthreads();
  }
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

template <int RT>
static cudaError_t launch_gate(const PrefillView& pv, const __nv_bfloat16* q, const float* means, int* sel, int* cnt,
                               int max_chunks_per_seq, cudaStream_t st) {
  size_t smem = (size_t)kCandBatch * pv.D * 4 + (size_t)kTile * (pv.D * 2 + 16) + (size_t)max_chunks_per_seq * 4 + 16;
  cudaError_t e = cudaFuncSetAttribute(gate_topk_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  gate_topk_kernel<RT><<<dim3(pv.n_qtiles, pv.Hkv), 128, smem, st>>>(pv, q, means, sel, cnt);
  return cudaGetLastError();
}

}  // namespace moba

using namespace moba;

extern "C" size_t moba_prefill_route_state_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  return route_state_bytes(*d);
}

extern "C" size_t moba_prefill_route_scratch_bytes(const moba_prefill_desc* d) {
  if (validate_desc(d) != MOBA_OK) return 0;
  return align256((size_t)d->num_chunks * d->hkv * d->dim * 4) +
         align256((size_t)d->num_chunks * d->hq * d->max_tiles_per_seq * 4) + align256((size_t)d->num_chunks * d->hq * 4);
}

static int route_impl(const moba_prefill_desc* d, const void* q, const void* k, void* route_state, void* scratch,
                      cudaStream_t st) {
  if (d->remote_k == 0) return MOBA_OK;  // dense fallback: nothing to route
  const PrefillView pv = make_view(*d);
  RouteState rs = carve_route_state(*d, route_state);
  char* p = static_cast<char*>(scratch);
  float* means = reinterpret_cast<float*>(p); p += align256((size_t)d->num_chunks * d->hkv * d->dim * 4);
  int* cnt = reinterpret_cast<int*>(p); p += align256((size_t)d->num_chunks * d->hq * d->max_tiles_per_seq * 4);
  int* seg_count = reinterpret_cast<int*>(p);
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(k);

  const int rpi = 256 / (d->dim / 8);
  chunk_mean_kernel<<<dim3(d->num_chunks, d->hkv), 256, (size_t)rpi * d->dim * 4, st>>>(pv, kb, means,
                                                                                           d->flags & MOBA_ROUTE_BF16_MEANS);
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
  segment_scan_kernel<<<(segs * 32 + 127) / 128, 128, 0, st>>>(pv, cnt, seg_count);
  plan_kernel<<<1, 1024, 0, st>>>(pv, seg_count, rs.seg_base, rs.tile_base);
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
  // Nothing in the scratch has to start at zero: every word the later passes read is written by an
  // earlier pass of the same call, so the previous call's contents are simply overwritten.
  return route_impl(d, q, k, route_state, scratch, (cudaStream_t)stream);
}
