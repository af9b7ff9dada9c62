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

// Merges the split-KV partials of the tile's rows into the bf16 A operand.  COLS = columns of every 128-column chunk
// one thread owns; 128 / COLS threads share a row, 256 * COLS / 128 rows are covered (the rest of the 64-row tile is
// zeroed).  Two items are in flight per thread at a time: their loads do not depend on each other.
template <int COLS>
__device__ __forceinline__ void merge_rows(uint16_t* As, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           const int32_t* sC0, const int32_t* sC1, const float* sM, const float* sInv, int r0, int rows,
                                           int S, int H, int h, int dC, int nk, int rows_total) {
  constexpr int TPR = 128 / COLS, ROWS = 256 / TPR;
  const int row = threadIdx.x / TPR, qt = threadIdx.x % TPR;
  for (int e = threadIdx.x; e < (64 - ROWS) * 16 * nk; e += 256) {   // rows of the MMA tile nobody merges into
    const int k = e / ((64 - ROWS) * 16), rem = e % ((64 - ROWS) * 16);
    *reinterpret_cast<uint4*>(As + ((size_t)k * 64 + ROWS + rem / 16) * kStride + (rem % 16) * 8) = make_uint4(0, 0, 0, 0);
  }
  const int r = r0 + row;
  const int c0 = sC0[row], c1 = sC1[row];
  const float M = sM[row], inv = sInv[row];
  const size_t prow = (r < rows) ? (size_t)(r % S) * H + h : 0;
  float acc[kMaxChunks][COLS];
#pragma unroll
  for (int k = 0; k < kMaxChunks; k++)
#pragma unroll
    for (int j = 0; j < COLS; j++) acc[k][j] = 0.f;
  for (int c = c0; c < c1; c += 2) {
    const bool two = c + 1 < c1;
    const size_t pr0 = (size_t)c * rows_total + prow, pr1 = (size_t)(two ? c + 1 : c) * rows_total + prow;
    const float m0 = __ldg(part_ml + pr0 * 2), m1 = __ldg(part_ml + pr1 * 2);
    const float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M) * inv;
    const float w1 = (!two || m1 == -INFINITY) ? 0.f : exp2f(m1 - M) * inv;
    const float4* s0 = reinterpret_cast<const float4*>(part_o + pr0 * dC + qt * COLS);
    const float4* s1 = reinterpret_cast<const float4*>(part_o + pr1 * dC + qt * COLS);
#pragma unroll
    for (int k = 0; k < kMaxChunks; k++) {
      if (k < nk) {
        float4 x0[COLS / 4], x1[COLS / 4];
#pragma unroll
        for (int j = 0; j < COLS / 4; j++) {
          x0[j] = __ldg(s0 + k * 32 + j);
          x1[j] = __ldg(s1 + k * 32 + j);
        }
#pragma unroll
        for (int j = 0; j < COLS / 4; j++) {
          acc[k][4 * j] = fmaf(x1[j].x, w1, fmaf(x0[j].x, w0, acc[k][4 * j]));
          acc[k][4 * j + 1] = fmaf(x1[j].y, w1, fmaf(x0[j].y, w0, acc[k][4 * j + 1]));
          acc[k][4 * j + 2] = fmaf(x1[j].z, w1, fmaf(x0[j].z, w0, acc[k][4 * j + 2]));
          acc[k][4 * j + 3] = fmaf(x1[j].w, w1, fmaf(x0[j].w, w0, acc[k][4 * j + 3]));
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxChunks; k++) {
    if (k < nk) {
      uint16_t* dst = As + ((size_t)k * 64 + row) * kStride + qt * COLS;
      if constexpr (COLS >= 8) {
#pragma unroll
        for (int j = 0; j < COLS / 8; j++)
          *reinterpret_cast<uint4*>(dst + j * 8) =
              make_uint4(pack_bf16x2(acc[k][8 * j], acc[k][8 * j + 1]), pack_bf16x2(acc[k][8 * j + 2], acc[k][8 * j + 3]),
                         pack_bf16x2(acc[k][8 * j + 4], acc[k][8 * j + 5]), pack_bf16x2(acc[k][8 * j + 6], acc[k][8 * j + 7]));
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(acc[k][0], acc[k][1]), pack_bf16x2(acc[k][2], acc[k][3]));
      }
    }
  }
}

// Split-KV merge fused into the value up-projection: the A operand (the merged, normalised latent output of
// 64 rows of one head, as bf16) is built straight from the per-item partials
//   part_o [item][S * H][dC] f32 (unnormalised), part_ml [item][S * H][2] = (max in the log2 domain, sum),
// items of sequence i = [chunk_off[i], chunk_off[i + 1]).  All of W_UV's slice for this head (dC x 128 bf16) streams
// into shared memory with cp.async while the partials are combined; four threads per row keep 32 independent
// 16-byte loads in flight per item, so the merge costs about one memory round trip per item of a sequence.
// grid (H, ceil(rows/64)), 256 threads, row = seq_index * S + query token.  dC = 128 * nk, nk <= 4.
__global__ void __launch_bounds__(256) mla_merge_vup_mma_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                const int32_t* __restrict__ chunk_off, const uint16_t* __restrict__ W_UV,
                                                                float* __restrict__ out, int rows, int S, int H, int dC) {
  extern __shared__ __align__(16) uint16_t sm[];
  const int nk = dC / 128;
  uint16_t* As = sm;                             // [nk][64][kStride]
  uint16_t* Bs = sm + (size_t)nk * 64 * kStride;  // [nk][128][kStride]
  __shared__ float sM[64], sInv[64];
  __shared__ int32_t sC0[64], sC1[64];
  const int h = blockIdx.x, r0 = blockIdx.y * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_total = S * H;
  for (int k = 0; k < nk; k++) {
#pragma unroll 4
    for (int e = threadIdx.x; e < 128 * 16; e += blockDim.x) {
      const int c = e / 16, v = e % 16;
      cp_async16(Bs + ((size_t)k * 128 + c) * kStride + v * 8, W_UV + (size_t)(k * 128 + c) * H * kDh + (size_t)h * kDh + (size_t)v * 8);
    }
    cp_async_commit();
  }
  if (threadIdx.x < 64) {
    const int r = r0 + threadIdx.x;
    int c0 = 0, c1 = 0;
    float M = -INFINITY, L = 0.f;
    if (r < rows) {
      const int i = r / S, sq = r % S;
      c0 = chunk_off[i];
      c1 = chunk_off[i + 1];
      const size_t prow = (size_t)sq * H + h;
      for (int c = c0; c < c1; c++) M = fmaxf(M, part_ml[((size_t)c * rows_total + prow) * 2]);
      for (int c = c0; c < c1; c++) {
        const float* ml = part_ml + ((size_t)c * rows_total + prow) * 2;
        if (ml[0] != -INFINITY) L += ml[1] * exp2f(ml[0] - M);
      }
    }
    sM[threadIdx.x] = M;
    sInv[threadIdx.x] = (L > 0.f) ? 1.0f / L : 0.f;
    sC0[threadIdx.x] = c0;
    sC1[threadIdx.x] = c1;
  }
  __syncthreads();
  // fewer real rows in the tile -> more threads per row, so that a short batch still keeps every thread loading
  const int rows_here = min(64, rows - r0);
  if (rows_here > 32) merge_rows<32>(As, part_o, part_ml, sC0, sC1, sM, sInv, r0, rows, S, H, h, dC, nk, rows_total);
  else if (rows_here > 16) merge_rows<16>(As, part_o, part_ml, sC0, sC1, sM, sInv, r0, rows, S, H, h, dC, nk, rows_total);
  else if (rows_here > 8) merge_rows<8>(As, part_o, part_ml, sC0, sC1, sM, sInv, r0, rows, S, H, h, dC, nk, rows_total);
  else merge_rows<4>(As, part_o, part_ml, sC0, sC1, sM, sInv, r0, rows, S, H, h, dC, nk, rows_total);
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k = 0; k < nk; k++) {
    // chunk k of W_UV has landed once at most nk - 1 - k younger groups are still in flight
    switch (nk - 1 - k) {
      case 3: cp_async_wait<3>(); break;
      case 2: cp_async_wait<2>(); break;
      case 1: cp_async_wait<1>(); break;
      default: cp_async_wait<0>(); break;
    }
    __syncthreads();   // also publishes the merged A tiles (first iteration)
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
                        int H, int dC, int dHR, const PrepAppend& ap, const PrepPlan& pl) {
  const int z_absorb = (rows + 63) / 64;
  dim3 grid(H, dC / 128, z_absorb + 1);
  const size_t smem = (size_t)(64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mla_prep_kernel<<<grid, 128, smem, dev->stream>>>(q_nope, q_rope, q_bf16, W_UK, q_abs, rows, H, dC, dHR, z_absorb, ap, pl);
  RELUX_CUDA_TRY(cudaGetLastError());
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
                                 float* out, int rows, int S, int H, int dC) {
  dim3 grid(H, (rows + 63) / 64);
  const size_t smem = (size_t)(dC / 128) * (64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_merge_vup_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mla_merge_vup_mma_kernel<<<grid, 256, smem, dev->stream>>>(part_o, part_ml, chunk_off, W_UV, out, rows, S, H, dC);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  return RELUX_OK;
}

}  // namespace relux
