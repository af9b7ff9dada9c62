// The two small per-head GEMMs around the absorbed MLA decode, on tensor cores (mma.sync m16n8k16, bf16 in,
// f32 accumulate):
//   absorb:  q~[row][h][0:dC]  = q_nope[row][h][:] . W_UK[:, h*Dh:(h+1)*Dh]^T      M = rows, N = dC,  K = Dh
//            q~[row][h][dC: ]  = q_rope[row][h][:]
//   up-proj: out[row][h][:]    = O_lat[row][h][:] . W_UV[:, h*Dh:(h+1)*Dh]          M = rows, N = Dh,  K = dC
// Both are about 1 GFLOP per step at batch 64 (1.5 % of the decode's work) and move ~30 MB; they are written to stay
// out of the way of the decode kernel, not to chase the tensor peak: one CTA per (head, 128-wide slice, 64 rows),
// operands staged in padded shared memory, fragments through ldmatrix.
// Shapes: Dh = 128, dC a multiple of 128.  Other shapes use the scalar kernels in mla_decode.cu.
#include "common.cuh"
#include "internal.h"

namespace relux {

namespace {

constexpr int kDh = 128;
constexpr int kStride = kDh + 8;  // bf16 elements per shared-memory row (272 B: conflict-free ldmatrix)

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

// grid (H, dC/128, ceil(rows/64)), 128 threads.
__global__ void __launch_bounds__(128) mla_absorb_mma_kernel(const void* __restrict__ q_nope, const void* __restrict__ q_rope, int q_bf16,
                                                             const uint16_t* __restrict__ W_UK, uint16_t* __restrict__ q_abs, int rows,
                                                             int H, int dC, int dHR) {
  extern __shared__ __align__(16) uint16_t sm[];
  uint16_t* As = sm;                  // [64][kStride]
  uint16_t* Bs = sm + 64 * kStride;   // [128][kStride]   rows = latent index c, cols = d
  const int h = blockIdx.x, c0 = blockIdx.y * 128, r0 = blockIdx.z * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A: 64 rows x 128 d, 8 elements per thread per step
  for (int e = threadIdx.x; e < 64 * (kDh / 8); e += blockDim.x) {
    const int r = e / (kDh / 8), v = e % (kDh / 8);
    uint4 w = make_uint4(0, 0, 0, 0);
    if (r0 + r < rows) {
      const size_t off = ((size_t)(r0 + r) * H + h) * kDh + (size_t)v * 8;
      if (q_bf16) w = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(q_nope) + off);
      else {
        const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q_nope) + off);
        const float4 x = s[0], y = s[1];
        w = make_uint4(pack_bf16x2(x.x, x.y), pack_bf16x2(x.z, x.w), pack_bf16x2(y.x, y.y), pack_bf16x2(y.z, y.w));
      }
    }
    *reinterpret_cast<uint4*>(As + r * kStride + v * 8) = w;
  }
  for (int e = threadIdx.x; e < 128 * (kDh / 8); e += blockDim.x) {
    const int c = e / (kDh / 8), v = e % (kDh / 8);
    const uint4 w = *reinterpret_cast<const uint4*>(W_UK + (size_t)(c0 + c) * H * kDh + (size_t)h * kDh + (size_t)v * 8);
    *reinterpret_cast<uint4*>(Bs + c * kStride + v * 8) = w;
  }
  __syncthreads();
  float acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  tile_mma_64x128x128<false>(As, Bs, acc, warp, lane);
  const int roww = dC + dHR;
#pragma unroll
  for (int hf = 0; hf < 2; hf++) {
    const int r = r0 + warp * 16 + hf * 8 + (lane >> 2);
    if (r >= rows) continue;
    uint16_t* dst = q_abs + ((size_t)r * H + h) * roww + c0;
#pragma unroll
    for (int nt = 0; nt < 16; nt++)
      *reinterpret_cast<uint32_t*>(dst + nt * 8 + 2 * (lane & 3)) = pack_bf16x2(acc[nt][hf * 2], acc[nt][hf * 2 + 1]);
  }
  if (blockIdx.y == 0) {
    for (int e = threadIdx.x; e < 64 * dHR; e += blockDim.x) {
      const int r = e / dHR, d = e % dHR;
      if (r0 + r >= rows) continue;
      const size_t off = ((size_t)(r0 + r) * H + h) * dHR + d;
      const uint16_t b = q_bf16 ? reinterpret_cast<const uint16_t*>(q_rope)[off] : bf16_bits_from_f32(reinterpret_cast<const float*>(q_rope)[off]);
      q_abs[((size_t)(r0 + r) * H + h) * roww + dC + d] = b;
    }
  }
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

int32_t launch_mla_vup_mma(Device* dev, const uint16_t* o_lat, const uint16_t* W_UV, float* out, int rows, int H, int dC) {
  dim3 grid(H, (rows + 63) / 64);
  const size_t smem = (size_t)(64 + 128) * kStride * 2;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(mla_vup_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  mla_vup_mma_kernel<<<grid, 128, smem, dev->stream>>>(o_lat, W_UV, out, rows, H, dC);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(dev);
  return RELUX_OK;
}

}  // namespace relux
