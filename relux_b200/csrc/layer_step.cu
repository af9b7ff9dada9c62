// Whole attention layer steps on the device: the work of MLA.forwardCached (internal/transformer/mla.go:272-397) and
// MHA.forwardCached (mha.go:245-369) either side of the cached attention, so that a caller hands over the layer
// input x and gets the layer output back.  For MLA:
//   1. projections  q^C = x W_Q, q^R = x W_QR, c^KV = x W_DKV, k^R = x W_KR          mla.go:285-288
//   2. decoupled RoPE on q^R and k^R at position cacheLen + s                          mla.go:297-307, rope.go:130-180
//   3. append (c^KV, k^R) to the paged latent cache                                    mla.go:309-314
//   4. absorbed attention over the cache (the kernels of mla_decode.cu)                mla.go:317-377
//   5. output projection  out = o W_O                                                  mla.go:380-389
// and for GQA: q, k, v = x Wq, x Wk, x Wv (mha.go:251-258), RoPE on q and k (mha.go:272-282), append k / v
// (mha.go:284-289), attention (mha.go:292-348), Wo (mha.go:351-355).
// The projections are skinny GEMMs (M = sequences x new tokens, at most a few hundred rows) against bf16 weight
// matrices of up to 16384 x 16384: they are bound by streaming the weights from HBM once.  FAST mode runs them on
// tcgen05 (activations rounded to bf16, f32 accumulation in tensor memory, split along K so that every SM streams an
// equal share of the weights); REFERENCE mode runs them in the reference's own float32 operation order
// (matmulBatched3D, matmul.go: k ascending, multiply then add, never fused), bit for bit.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include "common.cuh"
#include "internal.h"
#include "umma.cuh"

namespace relux {

int32_t stage_in(Pool* p, GrowBuf& buf, const void* src, size_t bytes, int mem, const void** dptr);

namespace {

constexpr int kMaxWeights = 4;   // weight matrices that share one activation matrix in a launch
constexpr int kTileN = 128, kTileM = 128, kTileK = 64;
constexpr int kStages = 6;
constexpr int kStageA = kTileM * kTileK * 2;   // 16 KB: [128 rows][64 k] bf16, 128-byte swizzle, K-major
constexpr int kStageB = kTileK * kTileN * 2;   // 16 KB: two [64 k][64 n] blocks, 128-byte swizzle, MN-major
constexpr int kGemmSmem = kStages * (kStageA + kStageB) + 1024;

struct GemmMaps {
  CUtensorMap a;                 // activations [M][K] bf16
  CUtensorMap w[kMaxWeights];    // weights [K][N_j] bf16
};
struct GemmParams {
  int32_t n_weights;
  int32_t tile_first[kMaxWeights + 1];   // first 128-column tile of every weight
  int32_t n_cols[kMaxWeights];           // N_j
  int32_t col_first[kMaxWeights];        // first output column of weight j in the concatenated result
  int32_t M, K, n_total, split_k;
  float* part;                           // [split_k][M][n_total] f32
  int32_t* status;
};

struct GemmBars {
  uint64_t full[kStages], empty[kStages], done;
  uint32_t tmem_base;
  volatile int32_t abort_flag;
};

__device__ __noinline__ void gemm_wait_slow(uint64_t* bar, uint32_t parity, GemmBars* b, int32_t* status) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 255) == 255 && b->abort_flag) return;
    if (i > 512) __nanosleep(20);
  }
  b->abort_flag = 1;
  set_status(status, RELUX_ERR_TIMEOUT);
}
// Bounded wait: a wait that runs out records RELUX_ERR_TIMEOUT and raises the CTA's abort flag; nobody leaves a loop early.
__device__ __forceinline__ void gemm_wait(uint64_t* bar, uint32_t parity, GemmBars* b, int32_t* status) {
  if (!mbar_try_wait(bar, parity)) gemm_wait_slow(bar, parity, b, status);
}

// grid (tiles * split_k, ceil(M / 128)), 192 threads: warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer.
// Unit = (128-column tile of one weight, K split): D[128 x 128] f32 in tensor memory accumulates
// A[128 x 64] (K-major) x W[64 x 128] (MN-major: the row-major weight rows as they lie in HBM) per pipeline stage.
__global__ void __launch_bounds__(192, 1) skinny_gemm_sm100_kernel(const __grid_constant__ GemmMaps maps, const GemmParams prm) {
  extern __shared__ __align__(1024) uint8_t smem[];
  GemmBars* bars = reinterpret_cast<GemmBars*>(smem + kStages * (kStageA + kStageB));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / prm.split_k, split = blockIdx.x % prm.split_k;
  const int m0 = blockIdx.y * kTileM;
  int j = 0;
  while (j + 1 < prm.n_weights && tile >= prm.tile_first[j + 1]) j++;
  const int n0 = (tile - prm.tile_first[j]) * kTileN;
  const int steps_total = (prm.K + kTileK - 1) / kTileK;
  const int step0 = (int)((long long)steps_total * split / prm.split_k);
  const int step1 = (int)((long long)steps_total * (split + 1) / prm.split_k);
  const int nsteps = step1 - step0;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(prm.status, RELUX_ERR_UNSUPPORTED);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    mbar_init(&bars->done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<1>(&bars->tmem_base, 128);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 4) {
    const bool el = elect_one();
    const CUtensorMap* wmap = &maps.w[j];
    if (el) {
      tma_prefetch_desc(&maps.a);
      tma_prefetch_desc(wmap);
    }
    for (int i = 0; i < nsteps; i++) {
      const int s = i % kStages, use = i / kStages;
      if (use > 0) gemm_wait(&bars->empty[s], (use - 1) & 1, bars, prm.status);
      if (el) {
        uint8_t* sa = smem + s * (kStageA + kStageB);
        uint8_t* sb = sa + kStageA;
        const int k0 = (step0 + i) * kTileK;
        mbar_expect_tx(&bars->full[s], kStageA + kStageB);   // out-of-range parts of a box are zero-filled and still counted
        tma_load_2d(sa, &maps.a, k0, m0, &bars->full[s]);
        tma_load_2d(sb, wmap, n0, k0, &bars->full[s]);
        tma_load_2d(sb + kStageB / 2, wmap, n0 + 64, k0, &bars->full[s]);
      }
      __syncwarp();
    }
  } else if (warp == 5) {
    const bool el = elect_one();
    const uint32_t idesc = make_idesc_bf16(kTileM, kTileN, false, true);
    for (int i = 0; i < nsteps; i++) {
      const int s = i % kStages, use = i / kStages;
      gemm_wait(&bars->full[s], use & 1, bars, prm.status);
      tc_fence_after();
      if (el) {
        const uint32_t sa = smem_u32(smem + s * (kStageA + kStageB));
        const uint64_t dA = make_desc_kmajor_sw128(sa);
        const uint64_t dB = make_desc_mnmajor_sw128(sa + kStageA, kStageB / 2);
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; kk++)
          umma_ss<1>(tmem, dA + ((uint32_t)(kk * 32) >> 4), dB + ((uint32_t)(kk * 2048) >> 4), idesc, (i | kk) != 0);
        umma_commit<1>(&bars->empty[s]);
      }
      __syncwarp();
    }
    if (el) umma_commit<1>(&bars->done);
    __syncwarp();
  } else {
    // epilogue: thread = accumulator row
    gemm_wait(&bars->done, 0, bars, prm.status);
    tc_fence_after();
    const int row = m0 + warp * 32 + lane;
    const int ncols = min(kTileN, prm.n_cols[j] - n0);   // a multiple of 8
    const bool ok = !bars->abort_flag && nsteps > 0;
    float* dst = prm.part + ((size_t)split * prm.M + row) * prm.n_total + prm.col_first[j] + n0;
#pragma unroll 1
    for (int c = 0; c < kTileN; c += 32) {
      uint32_t v[32];
      if (ok) {
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(warp * 32) << 16) + c, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int q = 0; q < 32; q++) v[q] = 0u;
      }
      if (row < prm.M) {
#pragma unroll
        for (int q = 0; q < 32; q += 4)
          if (c + q < ncols)
            *reinterpret_cast<float4*>(dst + c + q) = make_float4(__uint_as_float(v[q]), __uint_as_float(v[q + 1]),
                                                                  __uint_as_float(v[q + 2]), __uint_as_float(v[q + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<1>(tmem, 128);
}

// The reference's matmulBatched3D in its own operation order: out[m][n] = sum over k ascending of x[m][k] * w[k][n],
// float32, multiply then add, never fused.  One thread per output element; threads of a warp read consecutive n.
__global__ void gemm_reference_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, float* __restrict__ out, int M, int K,
                                      int N, int out_stride, int col_first) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
  if (n >= N || m >= M) return;
  const float* xr = x + (size_t)m * K;
  float acc = 0.f;
  for (int k = 0; k < K; k++) acc = __fadd_rn(acc, __fmul_rn(xr[k], f32_from_bf16_bits(w[(size_t)k * N + n])));
  out[(size_t)m * out_stride + col_first + n] = acc;
}

__global__ void cast_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
  reinterpret_cast<uint4*>(dst)[i] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
}

// Sums the K splits of the projection result (fixed order, so the result does not depend on scheduling), applies
// RoPE (rope.go:168-176: pairs (2i, 2i+1) of a head, out0 = x0 c - x1 s, out1 = x1 c + x0 s, unfused) at position
// len[seq] + s to the segments that ask for it, and scatters every segment to its own buffer.
// One thread per pair of adjacent columns of the concatenated result.
struct ProjSeg {
  int32_t n;          // columns of this segment (= of its weight matrix)
  int32_t rope_dim;   // 0: no rotation; else the per-head width the rotation works on
  void* dst;          // [M][n], f32 or bf16
  int32_t bf16;
};
struct FinishParams {
  const float* part;
  int32_t split_k, M, n_total, S, n_segs;
  ProjSeg seg[kMaxWeights];
  const int32_t* len;              // this layer's lengths BEFORE the append
  const int32_t* seq_ids;
  const float* rope_cos;           // [positions][rope_dim / 2]
  const float* rope_sin;
  int32_t rope_positions;
  int32_t same_pos;                // the reference's own rule (rope.go:151-158): on a non-empty cache every new row takes position len
  int32_t* status;
};
__global__ void proj_finish_kernel(const FinishParams p) {
  const int pair = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
  const int col = 2 * pair;
  if (col >= p.n_total || m >= p.M) return;
  float v0 = 0.f, v1 = 0.f;
  for (int s = 0; s < p.split_k; s++) {
    const float2 t = *reinterpret_cast<const float2*>(p.part + ((size_t)s * p.M + m) * p.n_total + col);
    v0 += t.x;
    v1 += t.y;
  }
  int c = col, j = 0;
  while (j + 1 < p.n_segs && c >= p.seg[j].n) {
    c -= p.seg[j].n;
    j++;
  }
  const ProjSeg sg = p.seg[j];
  if (sg.rope_dim > 0) {
    const int i = m / p.S, s = m % p.S;
    const int seq = p.seq_ids ? p.seq_ids[i] : i;
    const int len0 = p.len[seq];
    const int pos = (p.same_pos && len0 > 0) ? len0 : len0 + s;
    if (pos >= p.rope_positions) {
      set_status(p.status, RELUX_ERR_OVERFLOW);   // the reference panics: position >= maxSeqLen (rope.go:160-162)
    } else {
      const int half = sg.rope_dim / 2, idx = (c % sg.rope_dim) >> 1;
      const float cs = p.rope_cos[(size_t)pos * half + idx], sn = p.rope_sin[(size_t)pos * half + idx];
      const float r0 = __fsub_rn(__fmul_rn(v0, cs), __fmul_rn(v1, sn));
      const float r1 = __fadd_rn(__fmul_rn(v1, cs), __fmul_rn(v0, sn));
      v0 = r0;
      v1 = r1;
    }
  }
  if (sg.bf16) reinterpret_cast<uint32_t*>(sg.dst)[((size_t)m * sg.n + c) >> 1] = pack_bf16x2(v0, v1);
  else *reinterpret_cast<float2*>(reinterpret_cast<float*>(sg.dst) + (size_t)m * sg.n + c) = make_float2(v0, v1);
}

__global__ void sum_splits_kernel(const float* __restrict__ part, int split_k, size_t n4, float* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 acc = reinterpret_cast<const float4*>(part)[i];
  for (int s = 1; s < split_k; s++) {
    const float4 t = reinterpret_cast<const float4*>(part)[(size_t)s * n4 + i];
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  reinterpret_cast<float4*>(out)[i] = acc;
}

struct WeightRef {
  const void* w;
  int n;
};

// part[split][M][n_total] = A[M][K] x [W_0 | W_1 | ...]; returns the number of splits used.
int32_t launch_skinny_gemm(Pool* p, const uint16_t* a_bf16, int M, int K, const WeightRef* ws, int nw, float* part, size_t part_cap_bytes,
                           int* split_out) {
  GemmMaps maps;
  GemmParams g;
  memset(&g, 0, sizeof(g));
  if (!make_tmap_2d(&maps.a, (void*)a_bf16, (uint64_t)M, (uint64_t)K, kTileK, kTileM)) {
    set_error("tensor map for the activations could not be encoded");
    return RELUX_ERR_CUDA;
  }
  int tiles = 0, cols = 0;
  for (int j = 0; j < nw; j++) {
    if (!make_tmap_2d(&maps.w[j], (void*)ws[j].w, (uint64_t)K, (uint64_t)ws[j].n, 64, kTileK)) {
      set_error("tensor map for a weight matrix could not be encoded");
      return RELUX_ERR_CUDA;
    }
    g.tile_first[j] = tiles;
    g.n_cols[j] = ws[j].n;
    g.col_first[j] = cols;
    tiles += (ws[j].n + kTileN - 1) / kTileN;
    cols += ws[j].n;
  }
  for (int j = nw; j < kMaxWeights; j++) maps.w[j] = maps.w[0];
  g.tile_first[nw] = tiles;
  g.n_weights = nw;
  g.M = M;
  g.K = K;
  g.n_total = cols;
  const int mblocks = (M + kTileM - 1) / kTileM;
  const int steps = (K + kTileK - 1) / kTileK;
  const int sms = std::max(1, p->dev->sm_count);
  // split K so that the units fill whole waves of SMs: cost = waves x (steps per unit + fixed cost per unit)
  int best = 1;
  double best_cost = 1e300;
  const int max_split = std::min(std::min(steps, 32), (int)std::max<size_t>(1, part_cap_bytes / ((size_t)M * cols * 4)));
  for (int s = 1; s <= max_split; s++) {
    const long units = (long)tiles * mblocks * s;
    const long waves = (units + sms - 1) / sms;
    const double cost = (double)waves * ((double)(steps + s - 1) / s + 6.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  if (const int ov = p->tune.get(RELUX_TUNE_GEMM_SPLIT)) best = std::max(1, std::min(max_split, ov));   // tuning knob
  g.split_k = best;
  g.part = part;
  g.status = p->d_status;
  RELUX_CUDA_TRY(cudaFuncSetAttribute(skinny_gemm_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
  dim3 grid(tiles * best, mblocks);
  skinny_gemm_sm100_kernel<<<grid, 192, kGemmSmem, p->dev->stream>>>(maps, g);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  *split_out = best;
  return RELUX_OK;
}

bool gemm_sm100_eligible(int K, const WeightRef* ws, int nw) {
  if (K % 8 != 0 || nw > kMaxWeights) return false;
  for (int j = 0; j < nw; j++)
    if (ws[j].n % 8 != 0 || ((uintptr_t)ws[j].w & 15) != 0) return false;
  return true;
}

int32_t launch_gemm_reference(Pool* p, const float* x, int M, int K, const WeightRef* ws, int nw, float* out, int out_stride) {
  int col = 0;
  for (int j = 0; j < nw; j++) {
    dim3 grid((ws[j].n + 127) / 128, M);
    gemm_reference_kernel<<<grid, 128, 0, p->dev->stream>>>(x, (const uint16_t*)ws[j].w, out, M, K, ws[j].n, out_stride, col);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
    col += ws[j].n;
  }
  return RELUX_OK;
}

// cos / sin tables of the decoupled RoPE exactly as NewRotaryEmbedding builds them (rope.go:59-68):
// theta = float32(1) / float32(pow(base, 2i / headDim)), angle = float32(pos * theta), cos / sin in float64, rounded.
int32_t ensure_rope_table(Pool* p, int dHR, float base, int positions) {
  if (p->rope_dim == dHR && p->rope_base == base && p->rope_positions >= positions) return RELUX_OK;
  const int half = dHR / 2;
  std::vector<float> tab((size_t)2 * positions * half);
  for (int pos = 0; pos < positions; pos++)
    for (int i = 0; i < half; i++) {
      const float theta = 1.0f / (float)std::pow((double)base, (double)(2 * i) / (double)dHR);
      const float angle = (float)((double)pos * (double)theta);
      tab[(size_t)pos * half + i] = (float)std::cos((double)angle);
      tab[(size_t)positions * half + (size_t)pos * half + i] = (float)std::sin((double)angle);
    }
  int32_t rc = grow(p->dev, p->rope_tab, tab.size() * 4);
  if (rc) return rc;
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->rope_tab.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, p->dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(p->dev->stream));   // `tab` goes out of scope
  p->rope_dim = dHR;
  p->rope_base = base;
  p->rope_positions = positions;
  return RELUX_OK;
}

// x [M][K] f32 -> every segment's buffer: cast + split-K tensor-core GEMM (or the reference-order GEMM), then the
// finish kernel.  `proj_timing` records the event pair of the GEMM launch in the pool's projection ring.
int32_t project_and_finish(Pool* p, const SeqBatch& sb, int layer, const float* dx, int M, int K, int S, const WeightRef* ws,
                           const ProjSeg* segs, int nw, bool mma, uint16_t* a_bf16, float* part, size_t part_cap, bool same_pos = false) {
  cudaStream_t st = p->dev->stream;
  int n_total = 0;
  for (int j = 0; j < nw; j++) n_total += ws[j].n;
  int split = 1;
  cudaEvent_t evs[2] = {Pool::ring_event(p->proj_ring, p->proj_calls, 0), Pool::ring_event(p->proj_ring, p->proj_calls, 1)};
  if (mma) {
    const size_t n8 = (size_t)M * K / 8;
    cast_bf16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(dx, a_bf16, n8);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
    if (evs[0]) RELUX_CUDA_TRY(cudaEventRecord(evs[0], st));
    int32_t rc = launch_skinny_gemm(p, a_bf16, M, K, ws, nw, part, part_cap, &split);
    if (rc) return rc;
  } else {
    if (evs[0]) RELUX_CUDA_TRY(cudaEventRecord(evs[0], st));
    int32_t rc = launch_gemm_reference(p, dx, M, K, ws, nw, part, n_total);
    if (rc) return rc;
  }
  if (evs[0]) {
    RELUX_CUDA_TRY(cudaEventRecord(evs[1], st));
    p->proj_calls++;
  }
  FinishParams f;
  memset(&f, 0, sizeof(f));
  f.part = part;
  f.split_k = split;
  f.M = M;
  f.n_total = n_total;
  f.S = S;
  f.n_segs = nw;
  int rope_dim = 0;
  for (int j = 0; j < nw; j++) {
    f.seg[j] = segs[j];
    if (segs[j].rope_dim) rope_dim = segs[j].rope_dim;
  }
  f.len = p->d_len + (size_t)layer * p->prm.max_seqs;
  f.seq_ids = sb.d_seq_ids;
  f.rope_cos = (const float*)p->rope_tab.p;
  f.rope_sin = f.rope_cos ? f.rope_cos + (size_t)p->rope_positions * (rope_dim / 2) : nullptr;
  f.rope_positions = p->rope_positions;
  f.same_pos = same_pos ? 1 : 0;
  f.status = p->d_status;
  dim3 grid((n_total / 2 + 255) / 256, M);
  proj_finish_kernel<<<grid, 256, 0, st>>>(f);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

// out [M][N] f32 = attn [M][K] f32 x W_O [K][N]; `out` is the caller's buffer (host or device).
int32_t output_projection(Pool* p, const float* d_attn, int M, int K, const void* w_o, int N, bool mma, uint16_t* a_bf16, float* part,
                          size_t part_cap, void* out, int out_mem) {
  cudaStream_t st = p->dev->stream;
  const bool direct = out_mem == RELUX_MEM_DEVICE;
  float* d_out = direct ? (float*)out : nullptr;
  if (!direct) {
    int32_t rc = grow(p->dev, p->out_buf, (size_t)M * N * 4);
    if (rc) return rc;
    d_out = (float*)p->out_buf.p;
  }
  const WeightRef outp[1] = {{w_o, N}};
  if (mma) {
    const size_t n8 = (size_t)M * K / 8;
    cast_bf16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(d_attn, a_bf16, n8);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
    int split = 1;
    int32_t rc = launch_skinny_gemm(p, a_bf16, M, K, outp, 1, part, part_cap, &split);
    if (rc) return rc;
    const size_t n4 = (size_t)M * N / 4;
    sum_splits_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(part, split, n4, d_out);
    RELUX_CUDA_TRY(cudaGetLastError());
    count_launch(p->dev);
  } else {
    int32_t rc = launch_gemm_reference(p, d_attn, M, K, outp, 1, d_out, N);
    if (rc) return rc;
  }
  if (!direct) {
    RELUX_CUDA_TRY(cudaMemcpyAsync(out, d_out, (size_t)M * N * 4, cudaMemcpyDeviceToHost, st));
    RELUX_CUDA_TRY(cudaStreamSynchronize(st));
  }
  return RELUX_OK;
}

// Validation shared by the two layer entry points; fills the batch with explicit rows per sequence (the append
// kernels read "no row offsets" as one row per sequence).
int32_t layer_batch(Pool* p, int layer, int n_seqs, const int32_t* seq_ids, int S, const char* what, SeqBatch* sb) {
  const relux_pool_params& prm = p->prm;
  if (layer < 0 || layer >= prm.num_layers) {
    set_error("layerIdx=%d out of range [0, %d)", layer, prm.num_layers);
    return RELUX_ERR_INVALID_ARG;
  }
  if (n_seqs <= 0 || n_seqs > prm.max_seqs) {
    set_error("n_seqs=%d outside [1, max_seqs=%d]", n_seqs, prm.max_seqs);
    return RELUX_ERR_INVALID_ARG;
  }
  const std::vector<int32_t> rows_per_seq((size_t)n_seqs, S);
  int32_t rc = stage_batch(p, n_seqs, seq_ids, rows_per_seq.data(), 1, sb);
  if (rc) return rc;
  for (int i = 0; i < sb->n_seqs; i++) {   // the reference panics on overflow (kvcache.go:282-285, mla_cache.go:160-164)
    const int s = sb->seq[i];
    const int len = p->h_len[(size_t)layer * prm.max_seqs + s], cap = p->seq_pages[s] * prm.page_tokens;
    if (len + S > cap) {
      set_error("%s: layer %d overflow: total=%d + newLen=%d > capacity=%d (sequence %d)", what, layer, len, S, cap, s);
      return RELUX_ERR_OVERFLOW;
    }
  }
  return RELUX_OK;
}

struct LayerScratch {
  uint16_t* a_bf16;
  float* part;
  size_t part_cap;
  char* rest;
};
// [activations as bf16 (M x max_k) | split partials | caller's buffers (rest_bytes)]
int32_t layer_scratch(Pool* p, int M, int max_k, int max_n, size_t rest_bytes, LayerScratch* out) {
  const size_t part_cap = std::max<size_t>((size_t)64 << 20, (size_t)M * max_n * 4 * 4);
  const size_t off_part = ((size_t)M * max_k * 2 + 255) & ~(size_t)255;
  const size_t off_rest = off_part + part_cap;
  int32_t rc = grow(p->dev, p->layer_buf, off_rest + rest_bytes);
  if (rc) return rc;
  char* base = (char*)p->layer_buf.p;
  out->a_bf16 = (uint16_t*)base;
  out->part = (float*)(base + off_part);
  out->part_cap = part_cap;
  out->rest = base + off_rest;
  return RELUX_OK;
}
inline size_t pad256(size_t b) { return (b + 255) & ~(size_t)255; }

}  // namespace

int32_t do_mla_layer(Pool* p, const relux_mla_layer_args* a) {
  if (!a || !a->w) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const relux_pool_params& prm = p->prm;
  if (prm.kind != RELUX_POOL_MLA) { set_error("pool kind does not match this call (MLA pool needed)"); return RELUX_ERR_INVALID_ARG; }
  const relux_mla_layer_weights& w = *a->w;
  if (!a->x || !a->out || !w.w_q || !w.w_qr || !w.w_dkv || !w.w_kr || !w.w_uk || !w.w_uv || !w.w_o) {
    set_error("nil input, output or weight pointer");
    return RELUX_ERR_INVALID_ARG;
  }
  const int H = a->num_heads, D = a->d_model, S = a->q_tokens, dC = prm.mla_dc, dHR = prm.mla_dhr;
  if (H <= 0 || D <= 0 || S <= 0 || D % H != 0) {   // NewMLA, mla.go:69-74
    set_error("NewMLA: dModel=%d not divisible by numHeads=%d (or non-positive sizes)", D, H);
    return RELUX_ERR_INVALID_ARG;
  }
  if (dHR % 2 != 0) { set_error("NewMLA: dHR=%d must be even for paired RoPE rotation", dHR); return RELUX_ERR_INVALID_ARG; }
  if (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE && a->mode != RELUX_ATTN_REFERENCE_FAITHFUL) { set_error("bad mode"); return RELUX_ERR_INVALID_ARG; }
  const bool faithful = a->mode == RELUX_ATTN_REFERENCE_FAITHFUL;
  if (faithful && !p->compat) { set_error("RELUX_ATTN_REFERENCE_FAITHFUL needs a pool created with RELUX_POOL_FLAG_REFERENCE_COMPAT"); return RELUX_ERR_INVALID_ARG; }
  if (a->x_dtype != RELUX_DTYPE_F32) { set_error("x must be float32"); return RELUX_ERR_UNSUPPORTED; }
  const int Dh = D / H;
  const float rope_base = a->rope_base == 0.f ? 10000.f : a->rope_base;   // NewMLA, mla.go:78-80
  SeqBatch sb;
  int32_t rc = layer_batch(p, a->layer, a->n_seqs, a->seq_ids, S, "MLACache.Append", &sb);
  if (rc) return rc;
  const int M = sb.n_seqs * S;
  rc = ensure_rope_table(p, dHR, rope_base, prm.max_pages_per_seq * prm.page_tokens);
  if (rc) return rc;
  const void* dx = nullptr;
  rc = stage_in(p, p->in_a, a->x, (size_t)M * D * 4, a->x_mem, &dx);
  if (rc) return rc;

  const WeightRef proj[4] = {{w.w_q, H * Dh}, {w.w_qr, H * dHR}, {w.w_dkv, dC}, {w.w_kr, dHR}};
  const WeightRef outp[1] = {{w.w_o, D}};
  const int n_total = H * Dh + H * dHR + dC + dHR;
  const bool fast = a->mode == RELUX_ATTN_FAST;
  const bool mma = fast && !p->tune.get(RELUX_TUNE_GEMM_GENERIC) && gemm_sm100_eligible(D, proj, 4) && gemm_sm100_eligible(H * Dh, outp, 1);
  const size_t q_es = fast ? 2 : 4;
  const size_t b_qc = pad256((size_t)M * H * Dh * q_es), b_qr = pad256((size_t)M * H * dHR * q_es), b_c = pad256((size_t)M * dC * 4),
               b_kr = pad256((size_t)M * dHR * 4);
  LayerScratch sc;
  rc = layer_scratch(p, M, std::max(D, H * Dh), std::max(n_total, D), b_qc + b_qr + b_c + b_kr + (size_t)M * H * Dh * 4, &sc);
  if (rc) return rc;
  void* d_qc = sc.rest;
  void* d_qr = sc.rest + b_qc;
  float* d_c = (float*)(sc.rest + b_qc + b_qr);
  float* d_kr = (float*)(sc.rest + b_qc + b_qr + b_c);
  float* d_attn = (float*)(sc.rest + b_qc + b_qr + b_c + b_kr);
  // 1 + 2. projections, RoPE on q^R and k^R
  const ProjSeg segs[4] = {{H * Dh, 0, d_qc, fast ? 1 : 0}, {H * dHR, dHR, d_qr, fast ? 1 : 0}, {dC, 0, d_c, 0}, {dHR, dHR, d_kr, 0}};
  rc = project_and_finish(p, sb, a->layer, (const float*)dx, M, D, S, proj, segs, 4, mma, sc.a_bf16, sc.part, sc.part_cap, faithful);
  if (rc) return rc;
  // 3. append (advances the cursors).  A one-token step on the tensor-core path leaves the append to the attention's
  //    preparation launch (absorb + append + stream partition in one kernel, as relux_mla_step does).
  relux_attn_args probe;
  memset(&probe, 0, sizeof(probe));
  probe.mode = a->mode;
  probe.num_heads = H;
  probe.head_dim = Dh;
  probe.q_tokens = S;
  const bool fused_append = fast && S == 1 && mla_step_fusable(p, probe, sb.n_seqs);
  if (!fused_append) {
    rc = launch_mla_append(p, sb, a->layer, d_c, d_kr, RELUX_DTYPE_F32, 1);
    if (rc) return rc;
  }
  for (int i = 0; i < sb.n_seqs; i++) {
    int32_t& len = p->h_len[(size_t)a->layer * prm.max_seqs + sb.seq[i]];
    note_append(p, a->layer, sb.seq[i], len, S);
    len += S;
  }
  // 4. attention over the cache, the S new rows included
  relux_attn_args aa;
  memset(&aa, 0, sizeof(aa));
  aa.layer = a->layer;
  aa.n_seqs = sb.n_seqs;
  aa.seq_ids = a->seq_ids;
  aa.q_tokens = S;
  aa.extra_tokens = 0;
  aa.causal = a->causal;
  aa.num_heads = H;
  aa.head_dim = Dh;
  aa.scale = (float)(1.0 / std::sqrt((double)(Dh + dHR)));   // mla.go:344-345
  aa.q_dtype = fast ? RELUX_DTYPE_BF16 : RELUX_DTYPE_F32;
  aa.q_layout = RELUX_LAYOUT_TOKEN_MAJOR;
  aa.w_uk = w.w_uk;
  aa.w_uv = w.w_uv;
  aa.mode = a->mode;
  const StepAppend step{d_c, d_kr, RELUX_DTYPE_F32, nullptr};   // one row per sequence
  rc = fast ? launch_mla_decode_fast(p, sb, aa, d_qc, d_qr, d_attn, fused_append ? &step : nullptr)
            : launch_attn_reference_mla(p, sb, aa, (const float*)d_qc, (const float*)d_qr, d_attn);
  if (rc) return rc;
  // 5. output projection
  return output_projection(p, d_attn, M, H * Dh, w.w_o, D, mma, sc.a_bf16, sc.part, sc.part_cap, a->out, a->out_mem);
}

// MHA.forwardCached (mha.go:245-369) for a batch of independent sequences: projections with Wq / Wk / Wv, RoPE on q
// and k at position cacheLen + s (when the layer has a rotary embedding), append of k / v, GQA attention, Wo.
int32_t do_gqa_layer(Pool* p, const relux_gqa_layer_args* a) {
  if (!a || !a->w) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const relux_pool_params& prm = p->prm;
  if (prm.kind != RELUX_POOL_GQA) { set_error("pool kind does not match this call (GQA pool needed)"); return RELUX_ERR_INVALID_ARG; }
  const relux_gqa_layer_weights& w = *a->w;
  if (!a->x || !a->out || !w.w_q || !w.w_k || !w.w_v || !w.w_o) {
    set_error("nil input, output or weight pointer");
    return RELUX_ERR_INVALID_ARG;
  }
  const int H = a->num_heads, D = a->d_model, S = a->q_tokens, Hkv = prm.gqa_num_kv_heads, hd = prm.gqa_head_dim;
  if (H <= 0 || D <= 0 || S <= 0 || D % H != 0 || D / H != hd || H % Hkv != 0) {   // NewMHAGQA, mha.go
    set_error("dModel=%d / numHeads=%d must equal the pool's head_dim=%d, numHeads a multiple of numKVHeads=%d", D, H, hd, Hkv);
    return RELUX_ERR_INVALID_ARG;
  }
  if (a->rope && hd % 2 != 0) { set_error("NewRotaryEmbedding: headDim=%d, must be even and > 0", hd); return RELUX_ERR_INVALID_ARG; }
  if (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE && a->mode != RELUX_ATTN_REFERENCE_FAITHFUL) { set_error("bad mode"); return RELUX_ERR_INVALID_ARG; }
  const bool faithful = a->mode == RELUX_ATTN_REFERENCE_FAITHFUL;
  if (faithful && (!p->compat || !a->advance)) { set_error("RELUX_ATTN_REFERENCE_FAITHFUL needs a pool created with RELUX_POOL_FLAG_REFERENCE_COMPAT and advance != 0"); return RELUX_ERR_INVALID_ARG; }
  if (a->x_dtype != RELUX_DTYPE_F32) { set_error("x must be float32"); return RELUX_ERR_UNSUPPORTED; }
  if (a->mode == RELUX_ATTN_FAST && (!p->has_tmap || prm.page_tokens != 64 || hd != 128 || H / Hkv > 32)) {
    // checked before anything is written to the cache
    set_error("GQA FAST kernels need page_tokens=64, head_dim=128 and num_heads/num_kv_heads <= 32 "
              "(got page_tokens=%d head_dim=%d group=%d); use RELUX_ATTN_REFERENCE for other shapes", prm.page_tokens, hd, H / Hkv);
    return RELUX_ERR_UNSUPPORTED;
  }
  const float rope_base = a->rope_base == 0.f ? 10000.f : a->rope_base;
  SeqBatch sb;
  int32_t rc = layer_batch(p, a->layer, a->n_seqs, a->seq_ids, S, "Append", &sb);
  if (rc) return rc;
  const int M = sb.n_seqs * S;
  if (a->rope) {
    rc = ensure_rope_table(p, hd, rope_base, prm.max_pages_per_seq * prm.page_tokens);
    if (rc) return rc;
  }
  const void* dx = nullptr;
  rc = stage_in(p, p->in_a, a->x, (size_t)M * D * 4, a->x_mem, &dx);
  if (rc) return rc;
  const WeightRef proj[3] = {{w.w_q, H * hd}, {w.w_k, Hkv * hd}, {w.w_v, Hkv * hd}};
  const WeightRef outp[1] = {{w.w_o, D}};
  const int n_total = (H + 2 * Hkv) * hd;
  const bool fast = a->mode == RELUX_ATTN_FAST;
  const bool mma = fast && !p->tune.get(RELUX_TUNE_GEMM_GENERIC) && gemm_sm100_eligible(D, proj, 3) && gemm_sm100_eligible(H * hd, outp, 1);
  const size_t q_es = fast ? 2 : 4;
  const size_t b_q = pad256((size_t)M * H * hd * q_es), b_kv = pad256((size_t)M * Hkv * hd * 4);
  LayerScratch sc;
  rc = layer_scratch(p, M, std::max(D, H * hd), std::max(n_total, D), b_q + 2 * b_kv + (size_t)M * H * hd * 4, &sc);
  if (rc) return rc;
  void* d_q = sc.rest;
  float* d_k = (float*)(sc.rest + b_q);
  float* d_v = (float*)(sc.rest + b_q + b_kv);
  float* d_attn = (float*)(sc.rest + b_q + 2 * b_kv);
  const int rd = a->rope ? hd : 0;
  const ProjSeg segs[3] = {{H * hd, rd, d_q, fast ? 1 : 0}, {Hkv * hd, rd, d_k, 0}, {Hkv * hd, 0, d_v, 0}};
  rc = project_and_finish(p, sb, a->layer, (const float*)dx, M, D, S, proj, segs, 3, mma, sc.a_bf16, sc.part, sc.part_cap, faithful);
  if (rc) return rc;
  // append: the GEMM rows are token-major [row][Hkv][hd]; advance = 0 leaves the rows past the cursor (verify)
  rc = launch_gqa_append(p, sb, a->layer, d_k, d_v, RELUX_DTYPE_F32, RELUX_LAYOUT_TOKEN_MAJOR, a->advance);
  if (rc) return rc;
  if (a->advance)
    for (int i = 0; i < sb.n_seqs; i++) {
      int32_t& len = p->h_len[(size_t)a->layer * prm.max_seqs + sb.seq[i]];
      note_append(p, a->layer, sb.seq[i], len, S);
      len += S;
    }
  relux_attn_args aa;
  memset(&aa, 0, sizeof(aa));
  aa.layer = a->layer;
  aa.n_seqs = sb.n_seqs;
  aa.seq_ids = a->seq_ids;
  aa.q_tokens = S;
  aa.extra_tokens = a->advance ? 0 : S;
  aa.causal = a->causal;
  aa.num_heads = H;
  aa.head_dim = hd;
  aa.scale = (float)(1.0 / std::sqrt((double)hd));   // mha.go:319
  aa.q_dtype = fast ? RELUX_DTYPE_BF16 : RELUX_DTYPE_F32;
  aa.q_layout = RELUX_LAYOUT_TOKEN_MAJOR;
  aa.mode = a->mode;
  rc = fast ? launch_gqa_decode_fast(p, sb, aa, d_q, d_attn) : launch_attn_reference_gqa(p, sb, aa, (const float*)d_q, d_attn);
  if (rc) return rc;
  return output_projection(p, d_attn, M, H * hd, w.w_o, D, mma, sc.a_bf16, sc.part, sc.part_cap, a->out, a->out_mem);
}

// ComputeBackend.MatMulFloat32 as matmulBatched3D uses it (interface.go:25-29, mha.go:759-785): C = A x B with A, C float32
// and B a bf16 weight matrix [K][N] on the device.
int32_t do_matmul(Pool* p, const relux_matmul_args* a) {
  if (!a || !a->a || !a->b || !a->c) { set_error("nil argument"); return RELUX_ERR_INVALID_ARG; }
  const int M = a->m, K = a->k, N = a->n;
  if (M <= 0 || K <= 0 || N <= 0) { set_error("MatMulFloat32: M=%d K=%d N=%d must be positive", M, K, N); return RELUX_ERR_INVALID_ARG; }
  if (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE) { set_error("bad mode"); return RELUX_ERR_INVALID_ARG; }
  for (int i = 0; i < 4; i++)
    if (a->reserved[i]) { set_error("reserved fields must be zero"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc;
  if ((rc = check_dev_align(a->b, "B"))) return rc;
  if (a->a_mem == RELUX_MEM_DEVICE && (rc = check_dev_align(a->a, "A"))) return rc;
  if (a->c_mem == RELUX_MEM_DEVICE && (rc = check_dev_align(a->c, "C"))) return rc;
  const WeightRef w[1] = {{a->b, N}};
  const bool fast = a->mode == RELUX_ATTN_FAST;
  if (fast && (p->tune.get(RELUX_TUNE_GEMM_GENERIC) || !gemm_sm100_eligible(K, w, 1) || N % 4 != 0)) {
    set_error("MatMulFloat32 FAST needs K and N multiples of 8 (got K=%d N=%d); use RELUX_ATTN_REFERENCE", K, N);
    return RELUX_ERR_UNSUPPORTED;
  }
  const void* dA = nullptr;
  rc = stage_in(p, p->in_a, a->a, (size_t)M * K * 4, a->a_mem, &dA);
  if (rc) return rc;
  LayerScratch sc;
  rc = layer_scratch(p, M, K, N, 0, &sc);
  if (rc) return rc;
  return output_projection(p, (const float*)dA, M, K, a->b, N, fast, sc.a_bf16, sc.part, sc.part_cap, a->c, a->c_mem);
}

}  // namespace relux
