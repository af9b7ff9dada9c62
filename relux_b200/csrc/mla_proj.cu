// The two small per-head GEMMs around the absorbed MLA decode, on tensor cores (mma.sync m16n8k16, bf16 in,
// f32 accumulate):
//   absorb:  q~[row][h][0:dC]  = q_nope[row][h][:] . W_UK[:, h*Dh:(h+1)*Dh]^T      M = rows, N = dC,  K = Dh
//            q~[row][h][dC: ]  = q_rope[row][h][:]
//   up-proj: out[row][h][:]    = O_lat[row][h][:] . W_UV[:, h*Dh:(h+1)*Dh]          M = rows, N = Dh,  K = dC
// Both are about 1 GFLOP per step at batch 64 (1.5 % of the decode's work) and move ~30 MB; they are written to stay
// out of the way of the decode kernel, not to chase the tensor peak: one CTA per (head, 128-wide slice, 64 rows),
// operands staged in padded shared memory (cp.async, every load of a CTA in flight at once), fragments through
// ldmatrix.  The up-projection also performs the split-KV merge while it builds its A operand.
// Shapes: Dh = 128, dC a multiple of 128.  Other shapes use the scalar kernels in mla_decode.cu.
#include "common.cuh"
#include "internal.h"
#include "prep_parts.cuh"

namespace relux {

namespace {

constexpr int kDh = 128;
constexpr int kStride = kDh + 8;  // bf16 elements per shared-memory row (272 B: conflict-free ldmatrix)
constexpr int kMaxChunks = 4;     // the fused merge + up-projection keeps at most 4 x 128 latent columns in shared memory

// 64 x 128 A tile (rows x k) and 128 x 128 B tile; warp w owns rows 16w..16w+15 and all 128 columns.
// kBTrans = false: Bs is [n][k] (k contiguous)  -> ldmatrix;  true: Bs is [k][n] (n contiguous) -> ldmatrix.trans
template <bool kBTrans>
__device__ __forceinline__ void tile_mma_64x128x128(const uint16_t* As, const uint16_t* Bs, float (&acc)[16][4], int warp, int lane) {
#pragma unroll
  for (int ks = 0; ks < 8; ks++) {
    uint32_t a[4];
    {
      const int m = lane >> 3;
      const int row = warp * 16 + (m & 1) * 8 + (lane & 7);
      const int col = ks * 16 + (m >> 1) * 8;
      ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(As + row * kStride + col));
    }
#pragma unroll
    for (int n2 = 0; n2 < 8; n2++) {
      uint32_t b0, b1, b2, b3;
      const int m = lane >> 3;
      if (!kBTrans) {
        const int nrow = n2 * 16 + (m >> 1) * 8 + (lane & 7);
        const int kcol = ks * 16 + (m & 1) * 8;
        ldmatrix_x4(b0, b1, b2, b3, smem_u32(Bs + nrow * kStride + kcol));
      } else {
        const int krow = ks * 16 + (m & 1) * 8 + (lane & 7);
        const int ncol = n2 * 16 + (m >> 1) * 8;
        ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(Bs + krow * kStride + ncol));
      }
      mma_bf16_16816(acc[2 * n2], a, b0, b1);
      mma_bf16_16816(acc[2 * n2 + 1], a, b2, b3);
    }
  }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (H, dC/128, ceil(rows/64)), 128 threads.  Every load of the CTA is in flight at once (cp.async for bf16
// sources), the result leaves through shared memory as 16-byte row-contiguous stores.
__device__ __forceinline__ void absorb_block(uint16_t* sm, const void* __restrict__ q_nope, const void* __restrict__ q_rope, int q_bf16,
                                             const uint16_t* __restrict__ W_UK, uint16_t* __restrict__ q_abs, int rows, int H, int dC,
                                             int dHR, int bx, int by, int bz) {
  uint16_t* As = sm;                  // [64][kStride]
  uint16_t* Bs = sm + 64 * kStride;   // [128][kStride]   rows = latent index c, cols = d
  const int h = bx, c0 = by * 128, r0 = bz * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 4
  for (int e = threadIdx.x; e < 128 * (kDh / 8); e += blockDim.x) {
    const int c = e / (kDh / 8), v = e % (kDh / 8);
    cp_async16(Bs + c * kStride + v * 8, W_UK + (size_t)(c0 + c) * H * kDh + (size_t)h * kDh + (size_t)v * 8);
  }
  // A: 64 rows x 128 d, 8 elements per thread per step
#pragma unroll 4
  for (int e = threadIdx.x; e < 64 * (kDh / 8); e += blockDim.x) {
    const int r = e / (kDh / 8), v = e % (kDh / 8);
    uint16_t* dst = As + r * kStride + v * 8;
    if (r0 + r >= rows) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const size_t off = ((size_t)(r0 + r) * H + h) * kDh + (size_t)v * 8;
    if (q_bf16) {
      cp_async16(dst, reinterpret_cast<const uint16_t*>(q_nope) + off);
    } else {
      const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q_nope) + off);
      const float4 x = s[0], y = s[1];
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w), pack_bf16x2(y.x, y.y), pack_bf16x2(y.z, y.w));
    }
  }
  cp_async_commit();
  const int roww = dC + dHR;
  if (by == 0) {   // the rope part of q~ is a copy (with the same rounding when the source is float32)
    const int vecs = dHR / 8;
    for (int e = threadIdx.x; e < 64 * vecs; e += blockDim.x) {
      const int r = e / vecs, v = e % vecs;
      if (r0 + r >= rows) continue;
      const size_t off = ((size_t)(r0 + r) * H + h) * dHR + (size_t)v * 8;
      uint4 w;
      if (q_bf16) w = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(q_rope) + off);
      else {
        const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q_rope) + off);
        const float4 x = s[0], y = s[1];
        w = make_uint4(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w), pack_bf16x2(y.x, y.y), pack_bf16x2(y.z, y.w));
      }
      *reinterpret_cast<uint4*>(q_abs + ((size_t)(r0 + r) * H + h) * roww + dC + (size_t)v * 8) = w;
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  float acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  tile_mma_64x128x128<false>(As, Bs, acc, warp, lane);
  __syncthreads();   // every warp is done with As / Bs: Bs becomes the 64 x 128 output staging tile
  uint16_t* Os = Bs;
#pragma unroll
  for (int hf = 0; hf < 2; hf++) {
    const int r = warp * 16 + hf * 8 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < 16; nt++)
      *reinterpret_cast<uint32_t*>(Os + r * kStride + nt * 8 + 2 * (lane & 3)) = pack_bf16x2(acc[nt][hf * 2], acc[nt][hf * 2 + 1]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 64 * 16; e += blockDim.x) {
    const int r = e / 16, v = e % 16;
    if (r0 + r >= rows) continue;
    *reinterpret_cast<uint4*>(q_abs + ((size_t)(r0 + r) * H + h) * roww + c0 + v * 8) = *reinterpret_cast<const uint4*>(Os + r * kStride + v * 8);
  }
}

__global__ void __launch_bounds__(128) mla_absorb_mma_kernel(const void* __restrict__ q_nope, const void* __restrict__ q_rope, int q_bf16,
                                                             const uint16_t* __restrict__ W_UK, uint16_t* __restrict__ q_abs, int rows,
                                                             int H, int dC, int dHR) {
  extern __shared__ __align__(16) uint16_t sm[];
  absorb_block(sm, q_nope, q_rope, q_bf16, W_UK, q_abs, rows, H, dC, dHR, blockIdx.x, blockIdx.y, blockIdx.z);
}

// The preparation of one MLA decode step in ONE launch: the absorb grid (H, dC/128, ceil(rows/64)) plus one extra z
// slice whose blocks append the step's new rows (block e < n_seqs: sequence e) and build the stream partition (block
// e == n_seqs).  The three jobs are independent of one another: the append reads the lengths before it writes, the
// partition counts every sequence's new rows itself, and the last of those blocks to finish advances the lengths.
__global__ void __launch_bounds__(128) mla_prep_kernel(const void* __restrict__ q_nope, const void* __restrict__ q_rope, int q_bf16,
                                                       const uint16_t* __restrict__ W_UK, uint16_t* __restrict__ q_abs, int rows, int H,
                                                       int dC, int dHR, int z_absorb, const PrepAppend ap, const PrepPlan pl) {
  extern __shared__ __align__(16) uint16_t sm[];
  chain_release();
  chain_wait();   // the kernel before this one in the stream may still be reading what this one overwrites
  if ((int)blockIdx.z < z_absorb) {
    absorb_block(sm, q_nope, q_rope, q_bf16, W_UK, q_abs, rows, H, dC, dHR, blockIdx.x, blockIdx.y, blockIdx.z);
    return;
  }
  const int e = blockIdx.y * gridDim.x + blockIdx.x;
  if (e > ap.n_seqs) return;
  if (e < ap.n_seqs) prep_append_seq(ap, e);
  else prep_build_stream(ap, pl);
  prep_arrive_and_advance(ap, (uint32_t)ap.n_seqs + 1u);
}

// grid (H, ceil(rows/64)), 128 threads.  o_lat bf16 [rows][H][dC]; out f32 [rows][H][128].
__global__ void __launch_bounds__(128) mla_vup_mma_kernel(const uint16_t* __restrict__ o_lat, const uint16_t* __restrict__ W_UV,
                                                          float* __restrict__ out, int rows, int H, int dC) {
  extern __shared__ __align__(16) uint16_t sm[];
  uint16_t* As = sm;                  // [64][kStride]   rows x 128 latent columns of this k chunk
  uint16_t* Bs = sm + 64 * kStride;   // [128][kStride]  rows = latent index c of the chunk, cols = d
  const int h = blockIdx.x, r0 = blockIdx.y * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int kc = 0; kc < dC; kc += 128) {
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * 16; e += blockDim.x) {
      const int r = e / 16, v = e % 16;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (r0 + r < rows) w = *reinterpret_cast<const uint4*>(o_lat + ((size_t)(r0 + r) * H + h) * dC + kc + (size_t)v * 8);
      *reinterpret_cast<uint4*>(As + r * kStride + v * 8) = w;
    }
    for (int e = threadIdx.x; e < 128 * 16; e += blockDim.x) {
      const int c = e / 16, v = e % 16;
      const uint4 w = *reinterpret_cast<const uint4*>(W_UV + (size_t)(kc + c) * H * kDh + (size_t)h * kDh + (size_t)v * 8);
      *reinterpret_cast<uint4*>(Bs + c * kStride + v * 8) = w;
    }
    __syncthreads();
    tile_mma_64x128x128<true>(As, Bs, acc, warp, lane);
  }
#pragma unroll
  for (int hf = 0; hf < 2; hf++) {
    const int r = r0 + warp * 16 + hf * 8 + (lane >> 2);
    if (r >= rows) continue;
    float* dst = out + ((size_t)r * H + h) * kDh;
#pragma unroll
    for (int nt = 0; nt < 16; nt++)
      *reinterpret_cast<float2*>(dst + nt * 8 + 2 * (lane & 3)) = make_float2(acc[nt][hf * 2], acc[nt][hf * 2 + 1]);
  }
}

// 64 x 128 x 128 tile for eight warps: warp w owns rows 16 (w & 3) .. +15 and the 64 columns of half (w >> 2).
// Bs is [k][n] (n contiguous) -> ldmatrix.trans.
__device__ __forceinline__ void tile_mma_64x64x128_bt(const uint16_t* As, const uint16_t* Bs, float (&acc)[8][4], int warp, int lane) {
  const int wr = warp & 3, wn = warp >> 2;
#pragma unroll
  for (int ks = 0; ks < 8; ks++) {
    uint32_t a[4];
    const int m = lane >> 3;
    {
      const int row = wr * 16 + (m & 1) * 8 + (lane & 7);
      const int col = ks * 16 + (m >> 1) * 8;
      ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(As + row * kStride + col));
    }
#pragma unroll
    for (int n2 = 0; n2 < 4; n2++) {
      uint32_t b0, b1, b2, b3;
      const int krow = ks * 16 + (m & 1) * 8 + (lane & 7);
      const int ncol = wn * 64 + n2 * 16 + (m >> 1) * 8;
      ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(Bs + krow * kStride + ncol));
      mma_bf16_16816(acc[2 * n2], a, b0, b1);
      mma_bf16_16816(acc[2 * n2 + 1], a, b2, b3);
    }
  }
}

// Merges the split-KV partials of the tile's rows into the bf16 A operand, one warp per row at a time: a lane owns the
// same 4 of every 128 latent columns, so every load instruction of a warp is 512 contiguous bytes of one partial row
// (four threads per row with 128 bytes each, the first layout, put 32 different cache lines into every load
// instruction: the kernel spent most of its time in the load unit's address stage).  The weights of a row's items come
// from one round trip: lane j reads (max, sum) of item j, the warp reduces.  Four items are in flight per lane.
// Rows past the batch are zero rows of the MMA tile.
constexpr int kMergeWarps = 16;
// `after_first_requests` runs once per thread, after the loads of the warp's first row have been issued: work that
// stalls the thread for its own reasons goes there, under the shadow of that round trip.
template <typename Hook>
__device__ __forceinline__ void merge_rows_warp(uint16_t* As, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                const int32_t* __restrict__ chunk_off, int r0, int rows, int S, int H, int h, int dC, int nk,
                                                int rows_total, Hook&& after_first_requests) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool hook_due = true;
  // The item range of a row is the first of two dependent round trips to L2, so it is requested one row ahead.
  int c0_next = 0, c1_next = 0;
  if (r0 + warp < rows) {
    const int i = (r0 + warp) / S;
    c0_next = __ldg(chunk_off + i);
    c1_next = __ldg(chunk_off + i + 1);
  }
  for (int row = warp; row < 64; row += kMergeWarps) {
    const int r = r0 + row;
    const int c0 = c0_next, c1 = c1_next;
    c0_next = c1_next = 0;
    if (row + kMergeWarps < 64 && r + kMergeWarps < rows) {
      const int i = (r + kMergeWarps) / S;
      c0_next = __ldg(chunk_off + i);
      c1_next = __ldg(chunk_off + i + 1);
    }
    float4 acc[kMaxChunks];
#pragma unroll
    for (int k = 0; k < kMaxChunks; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) {
      const size_t prow = (size_t)(r % S) * H + h;
      // (max, sum) of this lane's item of every group of 32, and at the same time the partial rows of the first four
      // items: one memory round trip serves the common case of a sequence cut into a handful of items
      const int n_items = c1 - c0;
      if (n_items <= 0) goto store_row;   // no partial to merge: a zero row
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < n_items) ml = __ldg(reinterpret_cast<const float2*>(part_ml + ((size_t)(c0 + lane) * rows_total + prow) * 2));
      float4 x[4][kMaxChunks];
      const int ng0 = min(32, n_items);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        // a slot past the group's last item stays zero (its weight is zero too): the load unit's data path, 128 bytes
        // per clock for all 16 warps, is what a row's requests queue on, so no load is spent on padding
        const float4* src = reinterpret_cast<const float4*>(part_o + ((size_t)(c0 + u) * rows_total + prow) * dC) + lane;
#pragma unroll
        for (int k = 0; k < kMaxChunks; k++)
          if (k < nk) x[u][k] = (u < ng0) ? __ldg(src + k * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (hook_due) {
        after_first_requests();
        hook_due = false;
      }
      // global maximum and normaliser over all items of the sequence
      float M = ml.x;
      for (int c = c0 + 32 + lane; c < c1; c += 32) M = fmaxf(M, __ldg(part_ml + ((size_t)c * rows_total + prow) * 2));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      float L = (ml.x != -INFINITY) ? ml.y * exp2f(ml.x - M) : 0.f;
      for (int c = c0 + 32 + lane; c < c1; c += 32) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(part_ml + ((size_t)c * rows_total + prow) * 2));
        if (t.x != -INFINITY) L += t.y * exp2f(t.x - M);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
      const float inv = (L > 0.f) ? 1.0f / L : 0.f;
      for (int cb = c0; cb < c1; cb += 32) {
        // this lane's item of the group of 32: its weight; then four items at a time, weights by shuffle
        float w_mine = 0.f;
        if (cb == c0) {
          w_mine = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - M) * inv;
        } else if (cb + lane < c1) {
          const float m = __ldg(part_ml + ((size_t)(cb + lane) * rows_total + prow) * 2);
          w_mine = (m == -INFINITY) ? 0.f : exp2f(m - M) * inv;
        }
        const int ng = min(32, c1 - cb);
        for (int j = 0; j < ng; j += 4) {
          if (cb != c0 || j != 0) {   // the first four items of the row are in flight already
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const float4* src = reinterpret_cast<const float4*>(part_o + ((size_t)(cb + j + u) * rows_total + prow) * dC) + lane;
#pragma unroll
              for (int k = 0; k < kMaxChunks; k++)
                if (k < nk) x[u][k] = (j + u < ng) ? __ldg(src + k * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; u++) {
            float w = __shfl_sync(0xffffffffu, w_mine, min(j + u, 31));
            if (j + u >= ng) w = 0.f;
#pragma unroll
            for (int k = 0; k < kMaxChunks; k++)
              if (k < nk) {
                acc[k].x = fmaf(x[u][k].x, w, acc[k].x);
                acc[k].y = fmaf(x[u][k].y, w, acc[k].y);
                acc[k].z = fmaf(x[u][k].z, w, acc[k].z);
                acc[k].w = fmaf(x[u][k].w, w, acc[k].w);
              }
          }
        }
      }
    }
  store_row:
    if (hook_due) {
      after_first_requests();
      hook_due = false;
    }
#pragma unroll
    for (int k = 0; k < kMaxChunks; k++)
      if (k < nk)
        *reinterpret_cast<uint2*>(As + ((size_t)k * 64 + row) * kStride + lane * 4) =
            make_uint2(pack_bf16x2(acc[k].x, acc[k].y), pack_bf16x2(acc[k].z, acc[k].w));
  }
}

// Split-KV merge fused into the value up-projection: the A operand (the merged, normalised latent output of
// 64 rows of one head, as bf16) is built straight from the per-item partials
//   part_o [item][S * H][dC] f32 (unnormalised), part_ml [item][S * H][2] = (max in the log2 domain, sum),
// items of sequence i = [chunk_off[i], chunk_off[i + 1]).  All of W_UV's slice for this head (dC x 128 bf16) streams
// into shared memory as bulk copies while the partials are combined by 16 warps (merge_rows_warp); the first 8 warps
// then run the MMAs, chunk by chunk as the copies land.
// grid (H, ceil(rows/64)), 512 threads, row = seq_index * S + query token.  dC = 128 * nk, nk <= 4.
__global__ void __launch_bounds__(32 * kMergeWarps) mla_merge_vup_mma_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                const int32_t* __restrict__ chunk_off, const uint16_t* __restrict__ W_UV,
                                                                float* __restrict__ out, int rows, int S, int H, int dC,
                                                                int32_t* __restrict__ status) {
  extern __shared__ __align__(16) uint16_t sm[];
  __shared__ __align__(8) uint64_t w_full[kMaxChunks];   // chunk k of W_UV has landed (bytes counted by the bulk copies)
  const int nk = dC / 128;
  uint16_t* As = sm;                             // [nk][64][kStride]
  uint16_t* Bs = sm + (size_t)nk * 64 * kStride;  // [nk][128][kStride]
  const int h = blockIdx.x, r0 = blockIdx.y * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_total = S * H;
  chain_release();
  chain_wait();   // the partial results come from the kernel before this one
  // W_UV's slice comes in as one 256-byte bulk copy per latent row, through the TMA unit: as 16-byte cp.async requests
  // the same 128 KB sat in the load/store unit's queue ahead of the merge's own loads, whose round trips then took
  // 1.0-1.6 us each.
  if (threadIdx.x == 0) {
    for (int k = 0; k < nk; k++) mbar_init(&w_full[k], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int k = 0; k < nk; k++) mbar_expect_tx(&w_full[k], 128u * kDh * 2u);
  // 512 bulk copies queue up in the TMA unit (2-3 us until the last is accepted), so each thread issues its own after the
  // loads of its first row are on their way
  merge_rows_warp(As, part_o, part_ml, chunk_off, r0, rows, S, H, h, dC, nk, rows_total, [&]() {
    for (int e = threadIdx.x; e < nk * 128; e += blockDim.x)
      bulk_load_1d(Bs + (size_t)e * kStride, W_UV + (size_t)e * H * kDh + (size_t)h * kDh, kDh * 2, &w_full[e >> 7]);
  });
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  __syncthreads();   // the merged A tiles are complete
  if (warp >= 8) return;
  for (int k = 0; k < nk; k++) {
    if (!mbar_wait(&w_full[k], 0)) set_status(status, RELUX_ERR_TIMEOUT);   // bounded: a copy that never lands is reported, not waited for
    tile_mma_64x64x128_bt(As + (size_t)k * 64 * kStride, Bs + (size_t)k * 128 * kStride, acc, warp, lane);
  }
#pragma unroll
  for (int hf = 0; hf < 2; hf++) {
    const int r = r0 + (warp & 3) * 16 + hf * 8 + (lane >> 2);
    if (r >= rows) continue;
    float* dst = out + ((size_t)r * H + h) * kDh + (warp >> 2) * 64;
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
      *reinterpret_cast<float2*>(dst + nt * 8 + 2 * (lane & 3)) = make_float2(acc[nt][hf * 2], acc[nt][hf * 2 + 1]);
  }
}

}  // namespace

bool mla_proj_mma_eligible(int Dh, int dC) { return Dh == kDh && dC % 128 == 0; }

int32_t launch_mla_absorb_mma(Device* dev, const void* q_nope, const void* q_rope, int q_bf16, const uint16_t* W_UK, uint16_t* q_abs,
                              int rows, int H, int dC, int dHR) {
  dim3 grid(H, dC / 128, (rows + 63) / 64);
  const size_t smem = (size_t)(64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_absorb_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mla_absorb_mma_kernel<<<grid, 128, smem, dev->stream>>>(q_nope, q_rope, q_bf16, W_UK, q_abs, rows, H, dC, dHR);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  return RELUX_OK;
}

// One launch: absorb + append of the step's rows + stream partition (see mla_prep_kernel).  n_seqs + 1 extra blocks
// must fit one z slice of the absorb grid.
bool mla_prep_fits(int n_seqs, int H, int dC) { return n_seqs + 1 <= H * (dC / 128); }
int32_t launch_mla_prep(Device* dev, const void* q_nope, const void* q_rope, int q_bf16, const uint16_t* W_UK, uint16_t* q_abs, int rows,
                        int H, int dC, int dHR, const PrepAppend& ap, const PrepPlan& pl, bool chained) {
  const int z_absorb = (rows + 63) / 64;
  dim3 grid(H, dC / 128, z_absorb + 1);
  const size_t smem = (size_t)(64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RELUX_CUDA_TRY(launch_chained(chained, mla_prep_kernel, grid, dim3(128), smem, dev->stream, q_nope, q_rope, q_bf16, W_UK, q_abs, rows, H, dC,
                                dHR, z_absorb, ap, pl));
  count_launch(dev);
  return RELUX_OK;
}

int32_t launch_mla_vup_mma(Device* dev, const uint16_t* o_lat, const uint16_t* W_UV, float* out, int rows, int H, int dC) {
  dim3 grid(H, (rows + 63) / 64);
  const size_t smem = (size_t)(64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_vup_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mla_vup_mma_kernel<<<grid, 128, smem, dev->stream>>>(o_lat, W_UV, out, rows, H, dC);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  return RELUX_OK;
}

int32_t launch_mla_merge_vup_mma(Device* dev, const float* part_o, const float* part_ml, const int32_t* chunk_off, const uint16_t* W_UV,
                                 float* out, int rows, int S, int H, int dC, int32_t* status, bool chained) {
  dim3 grid(H, (rows + 63) / 64);
  const size_t smem = (size_t)(dC / 128) * (64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_merge_vup_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RELUX_CUDA_TRY(launch_chained(chained, mla_merge_vup_mma_kernel, grid, dim3(32 * kMergeWarps), smem, dev->stream, part_o, part_ml, chunk_off,
                                W_UV, out, rows, S, H, dC, status));
  count_launch(dev);
  return RELUX_OK;
}

}  // namespace relux
