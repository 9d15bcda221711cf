// Shared definitions of the prefill kernels: the device-side view of the packed batch and the
// layout of the route state that the routing pass produces and both attention passes consume.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moba_b200.h"

namespace moba {

constexpr int kTile = 128;  // query rows per tile and keys per tile

// Plain-value copy of moba_prefill_desc with typed pointers, passed to kernels by value.
struct PrefillView {
  int T, B, Hq, Hkv, G, D, C, R;
  int n_chunks, n_qtiles, max_tiles_per_seq, n_self_pairs;
  int fp16;  // q, k, v, out and the gradients are IEEE half (MOBA_INPUT_FP16), else bf16
  long long q_st, q_sh, k_st, k_sh, v_st, v_sh;  // element strides of token and head
  const int* cu_seqlens;   // [B+1]
  const int* chunk_start;  // [n_chunks+1] first packed token of every chunk
  const int* chunk_seq;    // [n_chunks]
  const int* chunk_local;  // [n_chunks] index of the chunk inside its sequence
  const int* qtile_chunk;  // [n_qtiles] chunk a 128-token query tile lies in
  const int* qtile_tok0;   // [n_qtiles] first packed token of the tile
  const int* qtile_local;  // [n_qtiles] index of the tile inside its sequence
  const int* self_pairs;   // [n_self_pairs] first tile of each pair of query tiles of a chunk, by decreasing causal work
  const int* kv_order;     // [n_qtiles] key blocks ordered by decreasing expected backward work
};

inline PrefillView make_view(const moba_prefill_desc& d) {
  PrefillView v;
  v.T = d.total_tokens; v.B = d.num_seqs; v.Hq = d.hq; v.Hkv = d.hkv; v.G = d.hq / d.hkv; v.D = d.dim;
  v.C = d.chunk_size; v.R = d.remote_k; v.n_chunks = d.num_chunks; v.n_qtiles = d.num_qtiles;
  v.max_tiles_per_seq = d.max_tiles_per_seq; v.n_self_pairs = d.num_self_pairs;
  v.fp16 = (d.flags & MOBA_INPUT_FP16) ? 1 : 0;
  v.q_st = d.q_stride_t; v.q_sh = d.q_stride_h; v.k_st = d.k_stride_t; v.k_sh = d.k_stride_h;
  v.v_st = d.v_stride_t; v.v_sh = d.v_stride_h;
  v.cu_seqlens = d.cu_seqlens; v.chunk_start = d.chunk_start; v.chunk_seq = d.chunk_seq;
  v.chunk_local = d.chunk_local; v.qtile_chunk = d.qtile_chunk; v.qtile_tok0 = d.qtile_tok0;
  v.qtile_local = d.qtile_local; v.self_pairs = d.self_pairs; v.kv_order = d.kv_order;
  return v;
}

// Route state (caller-owned, produced by moba_prefill_route, read by forward and backward).
//   sel        [T, Hq, R] int32   chunks chosen per (token, query head), ascending, -1 padded
//   rowlist    [T*Hq*R]   int32   for every expert (chunk, kv head) the slot ids (t*Hq+h)*R+s of
//                                 the rows that chose it, ordered by (head in group, token)
//   seg_base   [n_chunks*Hq + 1]  start of the (chunk, query head) segment inside rowlist
//   tile_base  [n_chunks*Hkv + 1] number of 128-row tiles of all experts before expert e; every expert's
//                                 count is rounded up to even (the forward works on pairs of tiles), the
//                                 padding tile has no rows
struct RouteState {
  int* sel;
  int* rowlist;
  int* seg_base;
  int* tile_base;
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

inline size_t route_lists_bytes(const moba_prefill_desc& d) {
  size_t rows = (size_t)d.total_tokens * d.hq * (d.remote_k > 0 ? d.remote_k : 1);
  return align256(rows * 4) * 2 + align256(((size_t)d.num_chunks * d.hq + 1) * 4) +
         align256(((size_t)d.num_chunks * d.hkv + 1) * 4);
}
inline RouteState carve_route_state(const moba_prefill_desc& d, void* base) {
  size_t rows = (size_t)d.total_tokens * d.hq * (d.remote_k > 0 ? d.remote_k : 1);
  char* p = static_cast<char*>(base);
  RouteState s;
  s.sel = reinterpret_cast<int*>(p); p += align256(rows * 4);
  s.rowlist = reinterpret_cast<int*>(p); p += align256(rows * 4);
  s.seg_base = reinterpret_cast<int*>(p); p += align256(((size_t)d.num_chunks * d.hq + 1) * 4);
  s.tile_base = reinterpret_cast<int*>(p);
  return s;
}

// Packed operand tiles (second part of the state kept from forward to backward).  Gathering 128
// scattered rows per tile with per-thread copies costs an attention kernel more issue time than the
// math of the tile, so rows are gathered once into ready-made shared-memory images - 128 rows x DPAD
// bf16 in the swizzled operand format, contiguous - which the kernels fetch with bulk copies.
//   kpack, vpack [num_qtiles * Hkv]  key block (128 tokens of a chunk) x kv head
//   qpack        [pack_q_tiles]      query tiles: (query tile qt, head h) -> qt*Hq + h, then the
//                                    expert tiles: num_qtiles*Hq + tile_base[e] + i
//   rowpack      [pack_q_tiles][128] t*Hq+h of every row, -1 = padding row
struct PackState {
  __nv_bfloat16* kpack;
  __nv_bfloat16* vpack;
  __nv_bfloat16* qpack;
  int* rowpack;
};
inline int pack_dpad(const moba_prefill_desc& d) { return d.dim <= 64 ? 64 : 128; }
inline long long pack_q_tiles(const moba_prefill_desc& d) {
  const long long slots = (long long)d.total_tokens * d.hq * d.remote_k;
  return (long long)d.num_qtiles * d.hq + slots / kTile + (d.remote_k > 0 ? 2ll * d.num_chunks * d.hkv : 0);
}
inline size_t pack_state_bytes(const moba_prefill_desc& d) {
  if (d.dim > 128) return 0;
  const size_t tile = (size_t)kTile * pack_dpad(d) * 2;
  return 2 * align256((size_t)d.num_qtiles * d.hkv * tile) + align256((size_t)pack_q_tiles(d) * tile) +
         align256((size_t)pack_q_tiles(d) * kTile * 4);
}
inline size_t route_state_bytes(const moba_prefill_desc& d) { return route_lists_bytes(d) + pack_state_bytes(d); }
inline PackState carve_pack_state(const moba_prefill_desc& d, void* base) {
  const size_t tile = (size_t)kTile * pack_dpad(d) * 2;
  char* p = static_cast<char*>(base) + route_lists_bytes(d);
  PackState s;
  s.kpack = reinterpret_cast<__nv_bfloat16*>(p); p += align256((size_t)d.num_qtiles * d.hkv * tile);
  s.vpack = reinterpret_cast<__nv_bfloat16*>(p); p += align256((size_t)d.num_qtiles * d.hkv * tile);
  s.qpack = reinterpret_cast<__nv_bfloat16*>(p); p += align256((size_t)pack_q_tiles(d) * tile);
  s.rowpack = reinterpret_cast<int*>(p);
  return s;
}
// Fills the pack state (prefill_pack.cu).
cudaError_t launch_prefill_pack(const moba_prefill_desc& d, const void* q, const void* k, const void* v, void* route_state,
                                unsigned* status, cudaStream_t st);

int validate_desc(const moba_prefill_desc* d);

// Optional CUDA events recorded right before / after one kernel (see moba_profile_events).
enum { kProfFwdRemote = 1, kProfFwdSelf = 2, kProfBwdMain = 3, kProfDecodeAttend = 4, kProfSlots = 8 };
void prof_begin(int which, cudaStream_t st);
void prof_end(int which, cudaStream_t st);

}  // namespace moba
