// Packing pass of the prefill: gathers K/V key blocks and Q query tiles into contiguous, already
// swizzled shared-memory images (see PackState in prefill_common.cuh), so the attention kernels
// fetch a tile with one bulk copy instead of 128 per-thread row gathers.  HBM-bound: every Q row is
// read once per tile it belongs to (own chunk + each selected chunk), K and V once.
#include "prefill_common.cuh"
#include "sm100.cuh"

namespace moba {

// One CTA per (key block, kv head): rows are the block's tokens, missing tokens and head-dim padding are zero.
__global__ void __launch_bounds__(128) pack_kv_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ k,
                                                      const __nv_bfloat16* __restrict__ v, uint8_t* __restrict__ kpack,
                                                      uint8_t* __restrict__ vpack, int dpad) {
  const int blk = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;
  const int c = pv.qtile_chunk[blk];
  const int k0 = pv.qtile_tok0[blk];
  const int nkeys = min(kTile, pv.chunk_start[c + 1] - k0);
  const int upr = dpad >> 3;
  const size_t tile_bytes = (size_t)kTile * dpad * 2;
  uint8_t* kd = kpack + ((size_t)blk * pv.Hkv + g) * tile_bytes;
  uint8_t* vd = vpack + ((size_t)blk * pv.Hkv + g) * tile_bytes;
  for (int i = tid; i < kTile * upr; i += 128) {
    const int r = i / upr, u = i - r * upr;
    uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
    if (r < nkeys && u * 8 < pv.D) {
      kv = *reinterpret_cast<const uint4*>(k + (long long)(k0 + r) * pv.k_st + (long long)g * pv.k_sh + u * 8);
      vv = *reinterpret_cast<const uint4*>(v + (long long)(k0 + r) * pv.v_st + (long long)g * pv.v_sh + u * 8);
    }
    const uint32_t off = sw128_offset(kTile, r, u);
    *reinterpret_cast<uint4*>(kd + off) = kv;
    *reinterpret_cast<uint4*>(vd + off) = vv;
  }
}

// One CTA per query tile (own-chunk tiles first, then the expert tiles in list order).
__global__ void __launch_bounds__(128) pack_q_kernel(PrefillView pv, const __nv_bfloat16* __restrict__ q,
                                                     const int* __restrict__ rowlist, const int* __restrict__ seg_base,
                                                     const int* __restrict__ tile_base, uint8_t* __restrict__ qpack,
                                                     int* __restrict__ rowpack, int dpad, unsigned* status) {
  __shared__ int s_th[kTile];
  const int tid = threadIdx.x;
  const long long tile = blockIdx.x;
  const long long n_self = (long long)pv.n_qtiles * pv.Hq;
  int th = -1;
  if (tile < n_self) {
    const int qt = (int)(tile / pv.Hq), h = (int)(tile - (long long)qt * pv.Hq);
    const int c = pv.qtile_chunk[qt];
    const int tok = pv.qtile_tok0[qt] + tid;
    if (tok < pv.chunk_start[c + 1]) th = tok * pv.Hq + h;
  } else {
    const int E = pv.n_chunks * pv.Hkv;
    const long long w = tile - n_self;
    if (w >= tile_base[E]) return;
    int lo = 0, hi = E;  // largest e with tile_base[e] <= w
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_base[mid] <= w) lo = mid; else hi = mid;
    }
    const int e = lo, i = (int)(w - tile_base[e]);
    const int c = e / pv.Hkv, g = e - c * pv.Hkv;
    const int start = seg_base[c * pv.Hq + g * pv.G] + i * kTile;
    const int end = seg_base[c * pv.Hq + (g + 1) * pv.G];
    if (start + tid < end) {
      th = rowlist[start + tid] / pv.R;
      if (th < 0 || th >= pv.T * pv.Hq) { atomicOr(status, kErrBadIndex); th = -1; }
    }
  }
  s_th[tid] = th;
  rowpack[tile * kTile + tid] = th;
  __syncthreads();
  const int upr = dpad >> 3;
  uint8_t* dst = qpack + tile * ((size_t)kTile * dpad * 2);
  for (int i = tid; i < kTile * upr; i += 128) {
    const int r = i / upr, u = i - r * upr;
    const int rth = s_th[r];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (rth >= 0 && u * 8 < pv.D) {
      const int t = rth / pv.Hq, h = rth - t * pv.Hq;
      val = *reinterpret_cast<const uint4*>(q + (long long)t * pv.q_st + (long long)h * pv.q_sh + u * 8);
    }
    *reinterpret_cast<uint4*>(dst + sw128_offset(kTile, r, u)) = val;
  }
}

cudaError_t launch_prefill_pack(const moba_prefill_desc& d, const void* q, const void* k, const void* v, void* route_state,
                                unsigned* status, cudaStream_t st) {
  const PrefillView pv = make_view(d);
  const PackState ps = carve_pack_state(d, route_state);
  const int dpad = pack_dpad(d);
  pack_kv_kernel<<<dim3(d.num_qtiles, d.hkv), 128, 0, st>>>(pv, static_cast<const __nv_bfloat16*>(k),
                                                            static_cast<const __nv_bfloat16*>(v),
                                                            reinterpret_cast<uint8_t*>(ps.kpack),
                                                            reinterpret_cast<uint8_t*>(ps.vpack), dpad);
  const int* rowlist = nullptr;
  const int* seg_base = nullptr;
  const int* tile_base = nullptr;
  if (d.remote_k > 0) {
    const RouteState rs = carve_route_state(d, route_state);
    rowlist = rs.rowlist; seg_base = rs.seg_base; tile_base = rs.tile_base;
  }
  const long long tiles = d.remote_k > 0 ? pack_q_tiles(d) : (long long)d.num_qtiles * d.hq;
  pack_q_kernel<<<(unsigned)tiles, 128, 0, st>>>(pv, static_cast<const __nv_bfloat16*>(q), rowlist, seg_base, tile_base,
                                                 reinterpret_cast<uint8_t*>(ps.qpack), ps.rowpack, dpad, status);
  return cudaGetLastError();
}

}  // namespace moba
