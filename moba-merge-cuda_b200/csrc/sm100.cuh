// Blackwell (sm_100a) device primitives used by the MoBA kernels: mbarriers with bounded
// waits, tensor-memory (TMEM) allocation, tcgen05.mma issue/commit, TMEM loads, and the
// 128-byte-swizzled shared-memory tile format that tcgen05 operand descriptors address.
//
// Shared-memory tile format ("SW128 tile")
//   A tile of R rows x W 16-bit elements is stored as W/64 panels; a panel holds 64 elements
//   (128 bytes) of every row, rows are 128 bytes apart, and the eight 16-byte units of a row
//   are XOR-permuted by (row & 7).  A panel is R*128 bytes and must start on a 1024-byte
//   boundary.  The same image serves as
//     * a K-major operand  (MN index = row,    K index = column): SBO = 1024, one K step of
//       16 elements advances the start address by 32 bytes inside a panel;
//     * an MN-major operand (MN index = column, K index = row):    SBO = 1024 (8 rows),
//       LBO = panel stride, one K step of 16 rows advances the start address by 2048 bytes.
//   This is also the image a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moba {

// Error bits a kernel may set in the caller-provided status word.
enum : unsigned {
  kErrBarrierTimeout = 1u,   // an mbarrier wait ran out of iterations
  kErrBadIndex = 2u,         // an index read from a table was out of range and was skipped
  kErrCapacity = 4u,         // a list would overflow its capacity
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and records kErrBarrierTimeout) after `limit_clocks` SM clocks instead
// of spinning forever, so a protocol bug cannot hang the GPU.  Kernels use mbar_wait (about a second).
constexpr long long kWaitLimitClocks = 2000000000ll;
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, unsigned* status, long long limit_clocks) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int it = 0; it < 64; ++it)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > limit_clocks) break;
  }
  if (status) atomicOr(status, kErrBarrierTimeout);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned* status) {
  return mbar_wait_for(bar, parity, status, kWaitLimitClocks);
}

// ----------------------------------------------------------------------------- fences
__device__ __forceinline__ void fence_async_smem() {
  // Makes generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma, TMA).
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------- TMEM
// One full warp allocates; the base address (lane 0, first column) lands in *slot (shared).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Store counterpart: thread i of the warp writes 32 consecutive 32-bit columns of lane (base+i).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16-column variant of tmem_st32.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- descriptors
// Shared-memory operand descriptor for an SW128 tile (see the header comment).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;  // layout type: 128-byte swizzle
  return d;
}
// K-major operand: element (mn, k) of a tile with `rows` rows; k0 = first K column of the step.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t tile_saddr, uint32_t rows, uint32_t k0) {
  uint32_t a = tile_saddr + (k0 >> 6) * rows * 128u + (k0 & 63u) * 2u;
  return umma_desc_sw128(a, 16u, 1024u);
}
// MN-major operand: K index = tile row; k0 = first row of the step (multiple of 16),
// mn0 = first MN column (multiple of 64).
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t tile_saddr, uint32_t rows, uint32_t k0, uint32_t mn0) {
  uint32_t a = tile_saddr + (mn0 >> 6) * rows * 128u + k0 * 128u;
  return umma_desc_sw128(a, rows * 128u, 1024u);
}

// Instruction descriptor: bf16 x bf16 -> fp32, M x N tile, operand majors (0 = K, 1 = MN).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t M, uint32_t N, uint32_t a_mn_major,
                                                       uint32_t b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((N >> 3) << 17) |
         ((M >> 4) << 24);
}
// The same for either 16-bit input format: the operand-format fields (bits 7-9 for A, 10-12 for B) hold 1 for
// bf16 and 0 for IEEE half.
template <bool F16>
__host__ __device__ constexpr uint32_t umma_idesc_16(uint32_t M, uint32_t N, uint32_t a_mn_major, uint32_t b_mn_major) {
  return umma_idesc_bf16(M, N, a_mn_major, b_mn_major) & (F16 ? ~((1u << 7) | (1u << 10)) : ~0u);
}

// ----------------------------------------------------------------------------- the two 16-bit input formats
// Kernels that convert inside their inner loops are compiled once per format (F16 = IEEE half, else bf16).
template <bool F16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {  // (lo, hi) -> two 16-bit values, lo in the low half
  uint32_t r;
  if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <bool F16>
__device__ __forceinline__ float2 unpack16(uint32_t w) {
  if (F16) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
// Run-time forms for kernels that convert a few values per thread (the flag is uniform over the launch).
__device__ __forceinline__ float2 unpack16(uint32_t w, bool f16) { return f16 ? unpack16<true>(w) : unpack16<false>(w); }
__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool f16) { return f16 ? pack16<true>(lo, hi) : pack16<false>(lo, hi); }
// x rounded to the 16-bit format and back (what storing and re-reading it would give)
__device__ __forceinline__ float round16(float x, bool f16) {
  return f16 ? __half2float(__float2half_rn(x)) : __bfloat162float(__float2bfloat16_rn(x));
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory, lane = M index, one 32-bit
// column holding the bf16 pair (k, k+1) with k in the low half; a K step of 16 is 8 columns.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------- SW128 tile access
// Byte offset of 16-byte unit `u` (0..W/8-1) of row `r` in an SW128 tile with `rows` rows.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t rows, uint32_t r, uint32_t u) {
  return (u >> 3) * rows * 128u + r * 128u + (((u & 7u) ^ (r & 7u)) << 4);
}

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* g, bool valid) {
  int sz = valid ? 16 : 0;  // zero-fill when not valid
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(saddr), "l"(g), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------- bulk (TMA) copies
// Linear global -> shared copy by the copy engine; completion is signalled as `bytes` of transaction
// count on the mbarrier.  Addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Adds `bytes` of FP32 values in shared memory to global memory through the copy engine (both addresses 16-byte
// aligned, bytes a multiple of 16); part of the calling thread's current bulk group.
__device__ __forceinline__ void bulk_reduce_add_f32(float* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
// The same for 64-bit integers (two's complement: order of the additions does not matter).
__device__ __forceinline__ void bulk_reduce_add_u64(unsigned long long* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u64 [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the calling thread's bulk groups have read their shared-memory sources / have completed.
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
}  // namespace moba
