// Weight import: checkpoint layout -> the device layout the layer calls take, and the bounded-wait self test.
//
// relux's DeepSeek mapper names the checkpoint tensors of an MLA layer and marks every one "Transpose: true"
// (internal/loader/mapper.go:139-180: checkpoints hold [out][in], relux holds [in][out]); its loader rounds each tensor
// to bf16 with BF16FromF32 (loader.go:239-281, 394-404).  The fused tensors are only named there (kv_b_proj ->
// "mla.W_UK_W_UV", mapper.go:163-173; loader.go:322-338 has slots for the separate matrices only).  The kernel below does
// the split and the transposes in one pass per tensor: a tiled transpose that sends each source row (one output feature)
// to the column of the destination matrix its feature belongs to.
#include "common.cuh"
#include "internal.h"

namespace relux {

namespace {

// One destination of a split: source rows whose index inside a group of `period` rows lies in [r0, r0 + rn) go to
// dst [in_dim][groups * rn] at column group * rn + (index - r0).
struct SplitDst {
  uint16_t* dst;
  int32_t r0, rn;
};

// src [rows][cols] (row = output feature, cols = input features) -> up to two destinations [cols][...].
// 32 x 32 tiles through shared memory so that both the reads and the writes are coalesced.
template <bool kF32>
__global__ void import_transpose_split_kernel(const void* __restrict__ src, int rows, int cols, int period, SplitDst d0, SplitDst d1) {
  __shared__ uint16_t tile[32][33];
  const int r_base = blockIdx.y * 32, c_base = blockIdx.x * 32;
  for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
    const int r = r_base + dy, c = c_base + threadIdx.x;
    uint16_t v = 0;
    if (r < rows && c < cols) {
      const size_t off = (size_t)r * cols + c;
      v = kF32 ? bf16_bits_from_f32(reinterpret_cast<const float*>(src)[off]) : reinterpret_cast<const uint16_t*>(src)[off];
    }
    tile[dy][threadIdx.x] = v;
  }
  __syncthreads();
  for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
    const int c = c_base + dy;            // destination row (input feature)
    const int r = r_base + threadIdx.x;   // source row (output feature)
    if (r >= rows || c >= cols) continue;
    const int grp = r / period, idx = r % period;
    const int ngroups = rows / period;
    if (d0.dst && idx >= d0.r0 && idx < d0.r0 + d0.rn)
      d0.dst[(size_t)c * ngroups * d0.rn + (size_t)grp * d0.rn + (idx - d0.r0)] = tile[threadIdx.x][dy];
    else if (d1.dst && idx >= d1.r0 && idx < d1.r0 + d1.rn)
      d1.dst[(size_t)c * ngroups * d1.rn + (size_t)grp * d1.rn + (idx - d1.r0)] = tile[threadIdx.x][dy];
  }
}

int32_t import_one(Pool* p, const void* src, int src_dtype, int src_mem, int rows, int cols, int period, SplitDst d0, SplitDst d1) {
  if (!src) return RELUX_OK;
  if (rows % period != 0) { set_error("import: %d source rows are not a multiple of the per-head group of %d", rows, period); return RELUX_ERR_INVALID_ARG; }
  int32_t rc;
  if (d0.dst && (rc = check_dev_align(d0.dst, "import destination"))) return rc;
  if (d1.dst && (rc = check_dev_align(d1.dst, "import destination"))) return rc;
  const size_t bytes = (size_t)rows * cols * (src_dtype == RELUX_DTYPE_BF16 ? 2 : 4);
  const void* d_src = src;
  if (src_mem == RELUX_MEM_HOST) {
    rc = grow(p->dev, p->layer_buf, bytes);
    if (rc) return rc;
    RELUX_CUDA_TRY(cudaMemcpyAsync(p->layer_buf.p, src, bytes, cudaMemcpyHostToDevice, p->dev->stream));
    d_src = p->layer_buf.p;
  } else if ((rc = check_dev_align(src, "import source"))) {
    return rc;
  }
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (src_dtype == RELUX_DTYPE_F32)
    import_transpose_split_kernel<true><<<grid, block, 0, p->dev->stream>>>(d_src, rows, cols, period, d0, d1);
  else
    import_transpose_split_kernel<false><<<grid, block, 0, p->dev->stream>>>(d_src, rows, cols, period, d0, d1);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  if (src_mem == RELUX_MEM_HOST) RELUX_CUDA_TRY(cudaStreamSynchronize(p->dev->stream));   // the staging block is reused by the next tensor
  return RELUX_OK;
}

// One warp waits on an mbarrier that nobody arrives at, with the same polling loop as the attention kernels' waits but
// a caller-chosen limit; when the limit runs out it records RELUX_ERR_TIMEOUT and returns.
__global__ void selftest_wait_kernel(int32_t* status, uint32_t polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  bool done = false;
  for (uint32_t i = 0; i < polls && !done; i++) {
    done = mbar_try_wait(&bar, 0);
    if (!done && i > 64) __nanosleep(32);
  }
  if (!done && threadIdx.x == 0) set_status(status, RELUX_ERR_TIMEOUT);
}

}  // namespace

int32_t do_import_mla(Pool* p, const relux_mla_import_args* a) {
  if (!a || !a->dst) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const int D = a->d_model, H = a->num_heads, dn = a->nope_dim, dr = a->rope_dim, dv = a->v_dim, dC = a->dc;
  if (D <= 0 || H <= 0 || dn <= 0 || dr < 0 || dv <= 0 || dC <= 0) { set_error("import: non-positive sizes"); return RELUX_ERR_INVALID_ARG; }
  if ((a->src_dtype != RELUX_DTYPE_F32 && a->src_dtype != RELUX_DTYPE_BF16) || (a->src_mem != RELUX_MEM_HOST && a->src_mem != RELUX_MEM_DEVICE)) {
    set_error("bad dtype/mem flag");
    return RELUX_ERR_INVALID_ARG;
  }
  for (int i = 0; i < 3; i++)
    if (a->reserved[i]) { set_error("reserved fields must be zero"); return RELUX_ERR_INVALID_ARG; }
  const relux_mla_layer_weights& w = *a->dst;
  const SplitDst none{nullptr, 0, 0};
  const bool fused = a->fused_rope != 0;
  if (fused && (a->q_pe_proj || a->k_pe_proj)) { set_error("import: q_pe_proj / k_pe_proj belong to fused_rope = 0"); return RELUX_ERR_INVALID_ARG; }
  if (fused && dr <= 0) { set_error("import: fused_rope needs rope_dim > 0"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc;
  // q_proj: per head the nope rows (then, fused, the rope rows)
  if (a->q_proj && (!w.w_q || (fused && !w.w_qr))) { set_error("import: q_proj needs the w_q (and, fused, w_qr) destinations"); return RELUX_ERR_INVALID_ARG; }
  const int q_period = fused ? dn + dr : dn;
  rc = import_one(p, a->q_proj, a->src_dtype, a->src_mem, H * q_period, D, q_period, SplitDst{(uint16_t*)w.w_q, 0, dn},
                  fused ? SplitDst{(uint16_t*)w.w_qr, dn, dr} : none);
  if (rc) return rc;
  // kv_a_proj_with_mqa: the latent rows (then, fused, the shared rope-key rows), one group
  if (a->kv_a_proj_with_mqa && (!w.w_dkv || (fused && !w.w_kr))) { set_error("import: kv_a_proj_with_mqa needs the w_dkv (and, fused, w_kr) destinations"); return RELUX_ERR_INVALID_ARG; }
  const int a_period = fused ? dC + dr : dC;
  rc = import_one(p, a->kv_a_proj_with_mqa, a->src_dtype, a->src_mem, a_period, D, a_period, SplitDst{(uint16_t*)w.w_dkv, 0, dC},
                  fused ? SplitDst{(uint16_t*)w.w_kr, dC, dr} : none);
  if (rc) return rc;
  // the separate rope tensors the reference's mapper names (mapper.go:142-145, 174-179): plain transposes
  if ((a->q_pe_proj && !w.w_qr) || (a->k_pe_proj && !w.w_kr) || ((a->q_pe_proj || a->k_pe_proj) && dr <= 0)) {
    set_error("import: q_pe_proj / k_pe_proj need rope_dim > 0 and the w_qr / w_kr destinations");
    return RELUX_ERR_INVALID_ARG;
  }
  if (dr > 0) {
    rc = import_one(p, a->q_pe_proj, a->src_dtype, a->src_mem, H * dr, D, H * dr, SplitDst{(uint16_t*)w.w_qr, 0, H * dr}, none);
    if (rc) return rc;
    rc = import_one(p, a->k_pe_proj, a->src_dtype, a->src_mem, dr, D, dr, SplitDst{(uint16_t*)w.w_kr, 0, dr}, none);
    if (rc) return rc;
  }
  // kv_b_proj [H * (nope + v)][dC]: per head the key up-projection rows, then the value up-projection rows
  if (a->kv_b_proj && (!w.w_uk || !w.w_uv)) { set_error("import: kv_b_proj needs the w_uk and w_uv destinations"); return RELUX_ERR_INVALID_ARG; }
  rc = import_one(p, a->kv_b_proj, a->src_dtype, a->src_mem, H * (dn + dv), dC, dn + dv, SplitDst{(uint16_t*)w.w_uk, 0, dn},
                  SplitDst{(uint16_t*)w.w_uv, dn, dv});
  if (rc) return rc;
  // o_proj [D][H * v] -> w_o [H * v][D]: a plain transpose
  if (a->o_proj && !w.w_o) { set_error("import: o_proj needs the w_o destination"); return RELUX_ERR_INVALID_ARG; }
  return import_one(p, a->o_proj, a->src_dtype, a->src_mem, D, H * dv, D, SplitDst{(uint16_t*)w.w_o, 0, D}, none);
}

int32_t do_selftest_wait(Pool* p, int32_t polls) {
  if (polls <= 0 || polls > 1000000) { set_error("selftest_wait: polls=%d outside [1, 1000000]", polls); return RELUX_ERR_INVALID_ARG; }
  selftest_wait_kernel<<<1, 32, 0, p->dev->stream>>>(p->d_status, (uint32_t)polls);
  RELUX_CUDA_TRY(cudaGetLastError());
  count_launch(p->dev);
  return RELUX_OK;
}

}  // namespace relux
