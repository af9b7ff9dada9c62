// Shared device/host helpers for librelux_cuda (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#include "relux_cuda.h"

namespace relux {

// ---------------------------------------------------------------------------------------------
// bf16 <-> f32 with the reference's exact bit rule (internal/transformer/dtype_convert.go:15-24):
// u += 0x7FFF + ((u >> 16) & 1); u >>= 16.  No NaN special case, so results match the reference
// bit for bit on every input, unlike __float2bfloat16_rn which canonicalises NaN.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint16_t bf16_bits_from_f32(float x) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(x);
#else
  uint32_t u;
  memcpy(&u, &x, 4);
#endif
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float f32_from_bf16_bits(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)bf16_bits_from_f32(lo) | ((uint32_t)bf16_bits_from_f32(hi) << 16);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// fastexp32 of internal/transformer/mha.go:823-833 with its operations kept unfused.
__device__ __forceinline__ float fastexp32_ref(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 87.0f) return __uint_as_float(0x7F800000u);
  float t = __fmul_rn(12102203.0f, x);
  t = __fadd_rn(t, 1064948224.0f);
  return __uint_as_float((uint32_t)__float2int_rz(t));
}

// ---------------------------------------------------------------------------------------------
// Device status word: kernels record the first problem they meet and carry on without faulting.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void set_status(int32_t* status, int32_t code) {
  if (status) atomicCAS(status, 0, code);
}

// Resolves (sequence, token position) to the element offset of the row's page inside one layer.
// Returns false (and records RELUX_ERR_BAD_PAGE) when the table holds an id outside the pool.
__device__ __forceinline__ bool page_of(const int32_t* __restrict__ table, int32_t table_stride, int32_t seq,
                                        int32_t page_slot, int32_t num_pages, int32_t* status, int32_t* page_out) {
  int32_t pg = table[(size_t)seq * table_stride + page_slot];
  if (pg < 0 || pg >= num_pages) {
    set_status(status, RELUX_ERR_BAD_PAGE);
    return false;
  }
  *page_out = pg;
  return true;
}

// Element offset of (token-in-page, column) inside one MLA page.
//   blocked (page_tokens = 64 and row width a multiple of 64): the page is stored as
//     [row_width / 64 column blocks][64 tokens][64 columns], so each 64 x 64 tile a TMA box fetches is one
//     contiguous 8 KB run of HBM instead of 64 pieces of 128 bytes 1152 bytes apart;
//   otherwise token-major [page_tokens][row_width].
// A vector of 8 consecutive columns starting at a multiple of 8 never straddles a block.
__device__ __forceinline__ size_t mla_page_off(bool blocked, int page_tokens, int row_width, int tok, int col) {
  return blocked ? ((size_t)(col >> 6) * page_tokens + tok) * 64 + (col & 63) : (size_t)tok * row_width + col;
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers: shared-memory addresses, mbarrier with bounded waits, TMA, ldmatrix, mma.sync.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Every wait is bounded: after kSpinLimit failed polls the caller gets `false`, records
// RELUX_ERR_TIMEOUT and leaves its loop, so a protocol bug cannot hang the GPU.
constexpr uint32_t kSpinLimit = 4u * 1000u * 1000u;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 2-D tiled TMA load global -> shared (no multicast), completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Brings one box of a tiled tensor into L2 without touching shared memory (no mbarrier, fire and forget).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// 2-D tiled TMA store shared -> global of one box (bulk async-group completion).  The shared tile must have been made
// visible to the async proxy (fence_proxy_async) by the threads that wrote it.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int32_t x, int32_t y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All committed stores of this thread have finished READING their shared tiles (the tiles may be written again).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All committed stores of this thread are complete.
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Programmatic dependent launch.  A kernel launched with the stream-serialization attribute may be scheduled while the
// kernel before it in the stream still runs; chain_wait() returns once that kernel has completed and its writes are
// visible, so it stands before the first access to global memory.  chain_release() lets the kernel after this one be
// scheduled (it blocks in its own chain_wait() until this grid is complete).  Both are no-ops in a plain launch.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Untiled bulk copy global -> shared through the TMA unit (not the load/store unit): both addresses 16-byte aligned,
// `bytes` a multiple of 16; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(gsrc),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Byte offset of element (row, col16B chunk) inside a tile whose rows are 128 bytes and which was
// written by TMA with CU_TENSOR_MAP_SWIZZLE_128B: the 16-byte chunk index is XORed with (row & 7).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk16) { return row * 128u + ((chunk16 ^ (row & 7u)) << 4); }

}  // namespace relux
