// Runtime half of librelux_cuda: handles, errors, memory, paged pools, page tables, and the
// C-ABI entry points that validate arguments and dispatch to the kernels.
#include <algorithm>
#include <cstdlib>
#include <new>

#include "internal.h"

namespace relux {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int32_t cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  if (e == cudaErrorMemoryAllocation) return RELUX_ERR_OUT_OF_MEMORY;
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) return RELUX_ERR_NO_DEVICE;
  return RELUX_ERR_CUDA;
}

int32_t grow(Device* dev, GrowBuf& b, size_t bytes) {
  if (bytes <= b.cap) return RELUX_OK;
  size_t want = std::max(bytes, b.cap + b.cap / 2);
  want = (want + 255) & ~(size_t)255;
  if (b.p) {
    RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    RELUX_CUDA_TRY(cudaFree(b.p));
    b.p = nullptr;
    b.cap = 0;
  }
  RELUX_CUDA_TRY(cudaMalloc(&b.p, want));
  b.cap = want;
  return RELUX_OK;
}

int32_t stage_acquire(Pool* p, int32_t** slot, int* slot_index) {
  const int i = (int)(p->stage_next++ % Pool::kStageSlots);
  if (p->stage_busy[i]) {
    RELUX_CUDA_TRY(cudaEventSynchronize(p->stage_ev[i]));
    p->stage_busy[i] = false;
  }
  *slot = p->h_stage + (size_t)i * p->stage_slot_ints();
  *slot_index = i;
  return RELUX_OK;
}
int32_t stage_release(Pool* p, int slot_index) {
  RELUX_CUDA_TRY(cudaEventRecord(p->stage_ev[slot_index], p->dev->stream));
  p->stage_busy[slot_index] = true;
  return RELUX_OK;
}

// Copies the call's sequence ids / rows-per-sequence to the device when they are not the
// trivial (identity, uniform) case, through one pinned staging block guarded by an event.
int32_t stage_batch(Pool* p, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_rows, int32_t uniform_rows,
                    SeqBatch* out) {
  const relux_pool_params& prm = p->prm;
  if (n_seqs <= 0 || n_seqs > prm.max_seqs) {
    set_error("n_seqs=%d outside [1, max_seqs=%d]", n_seqs, prm.max_seqs);
    return RELUX_ERR_INVALID_ARG;
  }
  out->n_seqs = n_seqs;
  out->seq.resize(n_seqs);
  out->rows.resize(n_seqs);
  out->total_rows = 0;
  out->max_rows = 0;
  bool uniform = true;
  for (int i = 0; i < n_seqs; i++) {
    int s = seq_ids ? seq_ids[i] : i;
    if (s < 0 || s >= prm.max_seqs || p->seq_pages[s] == 0) {
      set_error("sequence id %d is not live in this pool", s);
      return RELUX_ERR_INVALID_ARG;
    }
    int r = n_rows ? n_rows[i] : uniform_rows;
    if (r < 0) {
      set_error("negative row count for sequence %d", s);
      return RELUX_ERR_INVALID_ARG;
    }
    if (r != uniform_rows) uniform = false;
    out->seq[i] = s;
    out->rows[i] = r;
    out->total_rows += r;
    out->max_rows = std::max(out->max_rows, r);
  }
  if (seq_ids) {   // a sequence named twice would be written by two blocks and advanced twice
    if (++p->stamp == 0) {   // the call counter wrapped: forget every stamp
      std::fill(p->seq_stamp.begin(), p->seq_stamp.end(), 0u);
      p->stamp = 1;
    }
    for (int i = 0; i < n_seqs; i++) {
      if (p->seq_stamp[out->seq[i]] == p->stamp) {
        set_error("sequence id %d appears twice in one call", out->seq[i]);
        return RELUX_ERR_INVALID_ARG;
      }
      p->seq_stamp[out->seq[i]] = p->stamp;
    }
  }
  out->d_seq_ids = nullptr;
  out->d_row_off = nullptr;
  if (!seq_ids && uniform) return RELUX_OK;
  Device* dev = p->dev;
  int32_t* slot = nullptr;
  int slot_index = 0;
  int32_t rc_stage = stage_acquire(p, &slot, &slot_index);
  if (rc_stage) return rc_stage;
  int32_t* h_ids = slot;
  int32_t* h_off = slot + prm.max_seqs;
  if (seq_ids) {
    memcpy(h_ids, out->seq.data(), sizeof(int32_t) * n_seqs);
    RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_seq_ids, h_ids, sizeof(int32_t) * n_seqs, cudaMemcpyHostToDevice, dev->stream));
    out->d_seq_ids = p->d_seq_ids;
  }
  if (!uniform) {
    int32_t acc = 0;
    for (int i = 0; i < n_seqs; i++) {
      h_off[i] = acc;
      acc += out->rows[i];
    }
    h_off[n_seqs] = acc;
    RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_row_off, h_off, sizeof(int32_t) * (n_seqs + 1), cudaMemcpyHostToDevice, dev->stream));
    out->d_row_off = p->d_row_off;
  }
  return stage_release(p, slot_index);
}

struct DeviceGuard {
  std::unique_lock<std::mutex> lk;
  int32_t rc;
  explicit DeviceGuard(Device* d) : lk(d->mu) {
    cudaError_t e = cudaSetDevice(d->index);
    rc = (e == cudaSuccess) ? RELUX_OK : cuda_fail(e, "cudaSetDevice");
  }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  }
  return fn;
}
// 2-D bf16 tensor [rows][cols] (cols contiguous), box = box_cols x box_rows, 128-byte swizzle.
bool make_tmap_2d(CUtensorMap* m, void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
bool make_tmap_3d(CUtensorMap* m, void* base, uint64_t outer, uint64_t mid, uint64_t cols, uint32_t box_cols, uint32_t box_mid,
                  uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[3] = {cols, mid, outer};
  cuuint64_t strides[2] = {cols * 2, mid * cols * 2};
  cuuint32_t box[3] = {box_cols, box_mid, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

void tuning_defaults(Tuning* t);

static void pool_free_all(Pool* p) {
  auto fr = [](void* q) { if (q) cudaFree(q); };
  for (cudaStream_t st : {p->dev->h2d_stream, p->dev->d2h_stream})
    if (st) cudaStreamSynchronize(st);
  for (PipeSlots* ps : {&p->pipe_in_a, &p->pipe_in_b, &p->pipe_app_a, &p->pipe_app_b, &p->pipe_out})
    for (int i = 0; i < PipeSlots::kSlots; i++) {
      fr(ps->buf[i].p);
      if (ps->ready[i]) cudaEventDestroy(ps->ready[i]);
      if (ps->freed[i]) cudaEventDestroy(ps->freed[i]);
    }
  fr(p->storage); fr(p->d_table); fr(p->d_len); fr(p->d_status); fr(p->d_seq_ids); fr(p->d_row_off);
  fr(p->in_a.p); fr(p->in_b.p); fr(p->out_buf.p); fr(p->q_abs.p); fr(p->part_o.p); fr(p->part_ml.p); fr(p->work.p);
  fr(p->o_lat.p); fr(p->q_conv.p); fr(p->rope_tab.p); fr(p->layer_buf.p); fr(p->shadow_f32); fr(p->chunk_tab.p); fr(p->step_rows.p); fr(p->expand_buf.p);
  if (p->h_stage) cudaFreeHost(p->h_stage);
  for (cudaEvent_t ev : p->stage_ev)
    if (ev) cudaEventDestroy(ev);
  for (auto& pair : p->ev_ring)
    for (cudaEvent_t ev : pair)
      if (ev) cudaEventDestroy(ev);
  for (auto& pair : p->proj_ring)
    for (cudaEvent_t ev : pair)
      if (ev) cudaEventDestroy(ev);
  p->magic = 0;
  delete p;
}

static int32_t check_layer(Pool* p, int layer) {
  if (layer < 0 || layer >= p->prm.num_layers) {
    set_error("layerIdx=%d out of range [0, %d)", layer, p->prm.num_layers);
    return RELUX_ERR_INVALID_ARG;
  }
  return RELUX_OK;
}

// Moves an activation that arrives in host memory to the device staging block.
int32_t stage_in(Pool* p, GrowBuf& buf, const void* src, size_t bytes, int mem, const void** dptr) {
  if (mem == RELUX_MEM_DEVICE) {
    *dptr = src;
    return RELUX_OK;
  }
  int32_t rc = grow(p->dev, buf, bytes);
  if (rc) return rc;
  RELUX_CUDA_TRY(cudaMemcpyAsync(buf.p, src, bytes, cudaMemcpyHostToDevice, p->dev->stream));
  *dptr = buf.p;
  return RELUX_OK;
}

static size_t dtype_size(int dt) { return dt == RELUX_DTYPE_BF16 ? 2 : 4; }

static int32_t pipe_events(PipeSlots& ps, int slot) {
  if (!ps.ready[slot]) RELUX_CUDA_TRY(cudaEventCreateWithFlags(&ps.ready[slot], cudaEventDisableTiming));
  if (!ps.freed[slot]) RELUX_CUDA_TRY(cudaEventCreateWithFlags(&ps.freed[slot], cudaEventDisableTiming));
  return RELUX_OK;
}
// A slot's buffer may be replaced only when nothing queued on any stream still uses it.
static int32_t pipe_grow(Pool* p, GrowBuf& b, size_t bytes) {
  if (bytes <= b.cap) return RELUX_OK;
  Device* dev = p->dev;
  if (dev->h2d_stream) RELUX_CUDA_TRY(cudaStreamSynchronize(dev->h2d_stream));
  if (dev->d2h_stream) RELUX_CUDA_TRY(cudaStreamSynchronize(dev->d2h_stream));
  return grow(dev, b, bytes);
}
int32_t pipe_stage_in(Pool* p, PipeSlots& ps, const void* src, size_t bytes, const void** dptr, int* slot) {
  Device* dev = p->dev;
  const int s = (int)(ps.next++ % PipeSlots::kSlots);
  int32_t rc = pipe_events(ps, s);
  if (rc) return rc;
  rc = pipe_grow(p, ps.buf[s], bytes);
  if (rc) return rc;
  // the kernels that read this slot two calls ago must be done before the copy overwrites it
  if (ps.used[s]) RELUX_CUDA_TRY(cudaStreamWaitEvent(dev->h2d_stream, ps.freed[s], 0));
  RELUX_CUDA_TRY(cudaMemcpyAsync(ps.buf[s].p, src, bytes, cudaMemcpyHostToDevice, dev->h2d_stream));
  RELUX_CUDA_TRY(cudaEventRecord(ps.ready[s], dev->h2d_stream));
  RELUX_CUDA_TRY(cudaStreamWaitEvent(dev->stream, ps.ready[s], 0));
  dev->copies_in_flight = true;
  *dptr = ps.buf[s].p;
  *slot = s;
  return RELUX_OK;
}
int32_t pipe_release(Pool* p, PipeSlots& ps, int slot) {
  if (slot < 0) return RELUX_OK;
  RELUX_CUDA_TRY(cudaEventRecord(ps.freed[slot], p->dev->stream));
  ps.used[slot] = true;
  return RELUX_OK;
}
// Orders the compute stream after everything queued on the copy streams (used where a caller's event or a full
// synchronisation must cover the copies of pipelined calls).
static int32_t join_copy_streams(Device* dev) {
  if (!dev->copies_in_flight || !dev->ev_copy_join) return RELUX_OK;
  for (cudaStream_t st : {dev->h2d_stream, dev->d2h_stream}) {
    if (!st) continue;
    RELUX_CUDA_TRY(cudaEventRecord(dev->ev_copy_join, st));
    RELUX_CUDA_TRY(cudaStreamWaitEvent(dev->stream, dev->ev_copy_join, 0));
  }
  return RELUX_OK;
}

int32_t check_dev_align(const void* ptr, const char* what) {
  if (((uintptr_t)ptr & 15u) != 0) {
    set_error("%s: device pointer %p is not 16-byte aligned (the kernels read it with 16-byte vector loads)", what, ptr);
    return RELUX_ERR_INVALID_ARG;
  }
  return RELUX_OK;
}

void note_append(Pool* p, int layer, int seq, int old_len, int n) {
  if (!p->compat || n <= 0) return;
  p->chunks[(size_t)layer * p->prm.max_seqs + seq].push_back(old_len);
}
void note_set_len(Pool* p, int layer, int seq, int old_len, int new_len) {
  if (!p->compat || new_len == old_len) return;
  std::vector<int32_t>& c = p->chunks[(size_t)layer * p->prm.max_seqs + seq];
  if (new_len < old_len) {
    while (!c.empty() && c.back() >= new_len) c.pop_back();   // a chunk cut in the middle keeps its start
  } else {
    c.push_back(old_len);   // rows made visible without an Append of their own (a committed draft) form one chunk
  }
}

static int32_t do_append(Pool* p, const relux_append_args* a, int kind) {
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (p->prm.kind != kind) { set_error("pool kind does not match this append call"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc = check_layer(p, a->layer);
  if (rc) return rc;
  if (!a->a || !a->b) { set_error("nil input pointer"); return RELUX_ERR_INVALID_ARG; }
  if ((a->dtype != RELUX_DTYPE_F32 && a->dtype != RELUX_DTYPE_BF16) || (a->mem != RELUX_MEM_HOST && a->mem != RELUX_MEM_DEVICE)) {
    set_error("bad dtype/mem flag");
    return RELUX_ERR_INVALID_ARG;
  }
  if (a->flags & ~RELUX_CALL_PIPELINED) { set_error("unknown call flags 0x%x", a->flags); return RELUX_ERR_INVALID_ARG; }
  SeqBatch sb;
  rc = stage_batch(p, a->n_seqs, a->seq_ids, a->n_new, 1, &sb);
  if (rc) return rc;
  // capacity check on the host shadow: the reference panics on overflow (kvcache.go:282-285)
  const relux_pool_params& prm = p->prm;
  for (int i = 0; i < sb.n_seqs; i++) {
    int s = sb.seq[i];
    int len = p->h_len[(size_t)a->layer * prm.max_seqs + s];
    int cap = p->seq_pages[s] * prm.page_tokens;
    if (len + sb.rows[i] > cap) {
      set_error("Append: layer %d overflow: total=%d + newLen=%d > capacity=%d (sequence %d)", a->layer, len, sb.rows[i], cap, s);
      return RELUX_ERR_OVERFLOW;
    }
  }
  if (sb.total_rows == 0) return RELUX_OK;
  if (a->mem == RELUX_MEM_DEVICE) {
    if ((rc = check_dev_align(a->a, "append input a")) || (rc = check_dev_align(a->b, "append input b"))) return rc;
  }
  size_t es = dtype_size(a->dtype);
  const void *da = nullptr, *db = nullptr;
  const bool piped = (a->flags & RELUX_CALL_PIPELINED) && a->mem == RELUX_MEM_HOST && p->dev->h2d_stream;
  int slot_a = -1, slot_b = -1;
  const size_t bytes_a = (kind == RELUX_POOL_MLA) ? (size_t)sb.total_rows * prm.mla_dc * es
                                                  : (size_t)sb.total_rows * prm.gqa_num_kv_heads * prm.gqa_head_dim * es;
  const size_t bytes_b = (kind == RELUX_POOL_MLA) ? (size_t)sb.total_rows * prm.mla_dhr * es : bytes_a;
  if (piped) {
    if ((rc = pipe_stage_in(p, p->pipe_app_a, a->a, bytes_a, &da, &slot_a))) return rc;
    if ((rc = pipe_stage_in(p, p->pipe_app_b, a->b, bytes_b, &db, &slot_b))) return rc;
  } else {
    if ((rc = stage_in(p, p->in_a, a->a, bytes_a, a->mem, &da))) return rc;
    if ((rc = stage_in(p, p->in_b, a->b, bytes_b, a->mem, &db))) return rc;
  }
  if (kind == RELUX_POOL_MLA) rc = launch_mla_append(p, sb, a->layer, da, db, a->dtype, a->advance);
  else rc = launch_gqa_append(p, sb, a->layer, da, db, a->dtype, a->layout, a->advance);
  if (rc) return rc;
  if ((rc = pipe_release(p, p->pipe_app_a, slot_a)) || (rc = pipe_release(p, p->pipe_app_b, slot_b))) return rc;
  if (rc) return rc;
  if (a->advance)
    for (int i = 0; i < sb.n_seqs; i++) {
      int32_t& len = p->h_len[(size_t)a->layer * prm.max_seqs + sb.seq[i]];
      note_append(p, a->layer, sb.seq[i], len, sb.rows[i]);
      len += sb.rows[i];
    }
  return RELUX_OK;
}

// Converts q to the kernels' canonical device form and runs the attention, then delivers `out`.
int32_t convert_layout(Device* dev, const void* src, void* dst, int n, int S, int H, int D, int src_dtype, int dst_dtype,
                       int src_layout, int dst_layout);

static int32_t do_attention(Pool* p, const relux_attn_args* a, int kind, const StepAppend* step = nullptr) {
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (p->prm.kind != kind) { set_error("pool kind does not match this attention call"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc = check_layer(p, a->layer);
  if (rc) return rc;
  const relux_pool_params& prm = p->prm;
  if (!a->q || !a->out || a->q_tokens <= 0 || a->num_heads <= 0 || a->head_dim <= 0 || a->extra_tokens < 0) {
    set_error("bad attention arguments (nil q/out or non-positive sizes)");
    return RELUX_ERR_INVALID_ARG;
  }
  if (kind == RELUX_POOL_MLA && (!a->q_rope || !a->w_uk || !a->w_uv)) {
    set_error("MLA decode needs q_rope, w_uk and w_uv");
    return RELUX_ERR_INVALID_ARG;
  }
  if (kind == RELUX_POOL_GQA && (a->head_dim != prm.gqa_head_dim || a->num_heads % prm.gqa_num_kv_heads != 0)) {
    set_error("GQA decode: head_dim=%d (pool %d), num_heads=%d not a multiple of kv heads=%d", a->head_dim, prm.gqa_head_dim,
              a->num_heads, prm.gqa_num_kv_heads);
    return RELUX_ERR_INVALID_ARG;
  }
  if (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE && a->mode != RELUX_ATTN_REFERENCE_FAITHFUL) {
    set_error("bad mode");
    return RELUX_ERR_INVALID_ARG;
  }
  if (a->mode == RELUX_ATTN_REFERENCE_FAITHFUL && (!p->compat || a->extra_tokens != 0)) {
    set_error("RELUX_ATTN_REFERENCE_FAITHFUL needs a pool created with RELUX_POOL_FLAG_REFERENCE_COMPAT and extra_tokens = 0");
    return RELUX_ERR_INVALID_ARG;
  }
  if (!(a->scale > 0.f)) { set_error("scale=%g, must be > 0", (double)a->scale); return RELUX_ERR_INVALID_ARG; }
  if (a->flags & ~RELUX_CALL_PIPELINED) { set_error("unknown call flags 0x%x", a->flags); return RELUX_ERR_INVALID_ARG; }
  if (a->q_mem == RELUX_MEM_DEVICE) {
    if ((rc = check_dev_align(a->q, "q"))) return rc;
    if (kind == RELUX_POOL_MLA && (rc = check_dev_align(a->q_rope, "q_rope"))) return rc;
  }
  if (a->out_mem == RELUX_MEM_DEVICE && (rc = check_dev_align(a->out, "out"))) return rc;
  if (kind == RELUX_POOL_MLA && ((rc = check_dev_align(a->w_uk, "w_uk")) || (rc = check_dev_align(a->w_uv, "w_uv")))) return rc;
  SeqBatch sb;
  rc = stage_batch(p, a->n_seqs, a->seq_ids, nullptr, a->q_tokens, &sb);
  if (rc) return rc;
  for (int i = 0; i < sb.n_seqs; i++) {
    int s = sb.seq[i];
    int T = p->h_len[(size_t)a->layer * prm.max_seqs + s] + a->extra_tokens;
    if (T < a->q_tokens || T > p->seq_pages[s] * prm.page_tokens) {
      set_error("sequence %d: %d cached rows (with extra_tokens) cannot serve %d query tokens within capacity %d", s, T,
                a->q_tokens, p->seq_pages[s] * prm.page_tokens);
      return RELUX_ERR_INVALID_ARG;
    }
  }
  const int n = sb.n_seqs, S = a->q_tokens, H = a->num_heads, D = a->head_dim, R = prm.mla_dhr;
  const size_t q_elems = (size_t)n * S * H * D, qr_elems = (size_t)n * S * H * R;
  const void *dq = nullptr, *dqr = nullptr;
  const bool piped = (a->flags & RELUX_CALL_PIPELINED) != 0 && p->dev->h2d_stream && p->dev->d2h_stream;
  const bool piped_in = piped && a->q_mem == RELUX_MEM_HOST;
  int slot_q = -1, slot_qr = -1;
  if (piped_in) {
    if ((rc = pipe_stage_in(p, p->pipe_in_a, a->q, q_elems * dtype_size(a->q_dtype), &dq, &slot_q))) return rc;
    if (kind == RELUX_POOL_MLA && (rc = pipe_stage_in(p, p->pipe_in_b, a->q_rope, qr_elems * dtype_size(a->q_dtype), &dqr, &slot_qr))) return rc;
  } else {
    rc = stage_in(p, p->in_a, a->q, q_elems * dtype_size(a->q_dtype), a->q_mem, &dq);
    if (rc) return rc;
    if (kind == RELUX_POOL_MLA) {
      rc = stage_in(p, p->in_b, a->q_rope, qr_elems * dtype_size(a->q_dtype), a->q_mem, &dqr);
      if (rc) return rc;
    }
  }
  // canonical kernel input: token-major; f32 for REFERENCE, caller's dtype for FAST
  int want_dtype = (a->mode != RELUX_ATTN_FAST) ? RELUX_DTYPE_F32 : a->q_dtype;
  // a GQA prompt goes to the tcgen05 prefill kernel, whose Q tile is a TMA load of bf16 rows
  if (kind == RELUX_POOL_GQA && a->mode == RELUX_ATTN_FAST && gqa_prompt_wants_bf16(p, *a)) want_dtype = RELUX_DTYPE_BF16;
  // so does an MLA prompt (expanded keys / values + the same kernel)
  if (kind == RELUX_POOL_MLA && a->mode == RELUX_ATTN_FAST && mla_prefill_eligible(p, sb, *a)) want_dtype = RELUX_DTYPE_BF16;
  const bool relayout_q = (a->q_layout == RELUX_LAYOUT_HEAD_MAJOR && S > 1) || want_dtype != a->q_dtype;
  if (relayout_q) {
    size_t need = (q_elems + qr_elems) * dtype_size(want_dtype);
    rc = grow(p->dev, p->q_conv, need);
    if (rc) return rc;
    char* base = (char*)p->q_conv.p;
    rc = convert_layout(p->dev, dq, base, n, S, H, D, a->q_dtype, want_dtype, a->q_layout, RELUX_LAYOUT_TOKEN_MAJOR);
    if (rc) return rc;
    dq = base;
    if (kind == RELUX_POOL_MLA) {
      char* b2 = base + q_elems * dtype_size(want_dtype);
      rc = convert_layout(p->dev, dqr, b2, n, S, H, R, a->q_dtype, want_dtype, a->q_layout, RELUX_LAYOUT_TOKEN_MAJOR);
      if (rc) return rc;
      dqr = b2;
    }
  }
  // kernels write f32 token-major into `kout`; deliver converts if the caller wants otherwise
  const size_t out_elems = (size_t)n * S * H * D;
  const bool direct = a->out_mem == RELUX_MEM_DEVICE && a->out_dtype == RELUX_DTYPE_F32 &&
                      (a->out_layout == RELUX_LAYOUT_TOKEN_MAJOR || S == 1);
  float* kout;
  const bool piped_out = piped && a->out_mem == RELUX_MEM_HOST;
  int slot_out = -1;
  char* out_block = nullptr;   // [kernel output f32 | converted output]
  if (direct) kout = (float*)a->out;
  else if (piped_out) {
    PipeSlots& po = p->pipe_out;
    slot_out = (int)(po.next++ % PipeSlots::kSlots);
    if ((rc = pipe_events(po, slot_out))) return rc;
    if ((rc = pipe_grow(p, po.buf[slot_out], out_elems * 4 + out_elems * dtype_size(a->out_dtype)))) return rc;
    // the copy that last read this slot (two pipelined calls ago) must have finished before the kernels overwrite it
    if (po.used[slot_out]) RELUX_CUDA_TRY(cudaStreamWaitEvent(p->dev->stream, po.freed[slot_out], 0));
    out_block = (char*)po.buf[slot_out].p;
    kout = (float*)out_block;
  } else {
    rc = grow(p->dev, p->out_buf, out_elems * 4 + out_elems * dtype_size(a->out_dtype));
    if (rc) return rc;
    out_block = (char*)p->out_buf.p;
    kout = (float*)out_block;
  }
  relux_attn_args aa = *a;
  aa.q_dtype = want_dtype;
  aa.q_layout = RELUX_LAYOUT_TOKEN_MAJOR;
  if (a->mode != RELUX_ATTN_FAST) {
    rc = (kind == RELUX_POOL_MLA) ? launch_attn_reference_mla(p, sb, aa, (const float*)dq, (const float*)dqr, kout)
                                  : launch_attn_reference_gqa(p, sb, aa, (const float*)dq, kout);
  } else {
    rc = (kind == RELUX_POOL_MLA) ? launch_mla_decode_fast(p, sb, aa, dq, dqr, kout, step) : launch_gqa_decode_fast(p, sb, aa, dq, kout);
  }
  if (rc) return rc;
  if ((rc = pipe_release(p, p->pipe_in_a, slot_q)) || (rc = pipe_release(p, p->pipe_in_b, slot_qr))) return rc;
  if (!direct) {
    void* conv = out_block + out_elems * 4;
    const bool need_conv = a->out_dtype != RELUX_DTYPE_F32 || (a->out_layout == RELUX_LAYOUT_HEAD_MAJOR && S > 1);
    const void* src = kout;
    if (need_conv) {
      void* dst = (a->out_mem == RELUX_MEM_DEVICE) ? a->out : conv;
      rc = convert_layout(p->dev, kout, dst, n, S, H, D, RELUX_DTYPE_F32, a->out_dtype, RELUX_LAYOUT_TOKEN_MAJOR, a->out_layout);
      if (rc) return rc;
      src = dst;
    }
    if (piped_out) {
      PipeSlots& po = p->pipe_out;
      Device* dev = p->dev;
      RELUX_CUDA_TRY(cudaEventRecord(po.ready[slot_out], dev->stream));
      RELUX_CUDA_TRY(cudaStreamWaitEvent(dev->d2h_stream, po.ready[slot_out], 0));
      RELUX_CUDA_TRY(cudaMemcpyAsync(a->out, src, out_elems * dtype_size(a->out_dtype), cudaMemcpyDeviceToHost, dev->d2h_stream));
      RELUX_CUDA_TRY(cudaEventRecord(po.freed[slot_out], dev->d2h_stream));
      po.used[slot_out] = true;
      dev->copies_in_flight = true;
    } else if (a->out_mem == RELUX_MEM_HOST) {
      RELUX_CUDA_TRY(cudaMemcpyAsync(a->out, src, out_elems * dtype_size(a->out_dtype), cudaMemcpyDeviceToHost, p->dev->stream));
      RELUX_CUDA_TRY(cudaStreamSynchronize(p->dev->stream));
    }
  }
  return RELUX_OK;
}

// Built-in defaults of the tuning knobs, then the environment (read here, once per pool, never on a launch path).
static const int32_t kTuneDefault[RELUX_TUNE_COUNT] = {0, 0, 0, 0, 0, 256, 0, -1, -1, 0, 128, 16384, 1, 1};
static const char* const kTuneEnv[RELUX_TUNE_COUNT] = {"RELUX_MLA_GENERIC", "RELUX_MLA_WORKERS", "RELUX_CHUNK_PAGES", "RELUX_GEMM_GENERIC",
                                                       "RELUX_GEMM_SPLIT", "RELUX_GQA_PROMPT_PARTIAL_MB", "RELUX_SEL_CLUSTER",
                                                       "RELUX_SEL_LOOKAHEAD", "RELUX_SEL_BATCHED", "RELUX_GQA_PROMPT_SLICES",
                                                       "RELUX_MLA_PROMPT_MIN_TOKENS", "RELUX_MLA_PROMPT_SCRATCH_MB", "RELUX_KERNEL_TIMING_STRIDE",
                                                       "RELUX_CHAINED_LAUNCHES"};
void tuning_defaults(Tuning* t) {
  for (int i = 0; i < RELUX_TUNE_COUNT; i++) {
    t->v[i] = kTuneDefault[i];
    if (const char* e = getenv(kTuneEnv[i])) t->v[i] = atoi(e);
  }
}

}  // namespace relux

using namespace relux;

#define API extern "C" __attribute__((visibility("default")))
#define GET_DEV(h)                                               \
  Device* dev = as_device(h);                                    \
  if (!dev) { set_error("bad device handle"); return RELUX_ERR_BAD_HANDLE; } \
  DeviceGuard guard__(dev);                                      \
  if (guard__.rc) return guard__.rc;
#define GET_POOL(h)                                              \
  Pool* p = as_pool(h);                                          \
  if (!p) { set_error("bad pool handle"); return RELUX_ERR_BAD_HANDLE; } \
  Device* dev = p->dev;                                          \
  DeviceGuard guard__(dev);                                      \
  if (guard__.rc) return guard__.rc;

API int32_t relux_cuda_version(void) { return RELUX_CUDA_ABI_VERSION; }

API int32_t relux_cuda_last_error(char* buf, int32_t buf_len) {
  if (!buf || buf_len <= 0) return RELUX_ERR_INVALID_ARG;
  snprintf(buf, (size_t)buf_len, "%s", g_err);
  return RELUX_OK;
}

API int32_t relux_cuda_device_count(int32_t* count) {
  if (!count) return RELUX_ERR_INVALID_ARG;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *count = 0;
    return cuda_fail(e, "cudaGetDeviceCount");
  }
  *count = n;
  return RELUX_OK;
}

API int32_t relux_cuda_device_open(int32_t device_index, relux_device_t* out) {
  if (!out) return RELUX_ERR_INVALID_ARG;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
  if (n == 0) { set_error("no CUDA device"); return RELUX_ERR_NO_DEVICE; }
  if (device_index < 0 || device_index >= n) { set_error("device index %d outside [0,%d)", device_index, n); return RELUX_ERR_INVALID_ARG; }
  RELUX_CUDA_TRY(cudaSetDevice(device_index));
  cudaDeviceProp prop;
  RELUX_CUDA_TRY(cudaGetDeviceProperties(&prop, device_index));
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; this library holds sm_100a code only", device_index, prop.major, prop.minor);
    return RELUX_ERR_UNSUPPORTED;
  }
  Device* d = new (std::nothrow) Device();
  if (!d) return RELUX_ERR_OUT_OF_MEMORY;
  d->index = device_index;
  d->sm_count = prop.multiProcessorCount;
  d->total_mem = prop.totalGlobalMem;
  snprintf(d->name, sizeof(d->name), "%s", prop.name);
  e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { delete d; return cuda_fail(e, "cudaStreamCreate"); }
  if (cudaStreamCreateWithFlags(&d->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&d->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&d->ev_join, cudaEventDisableTiming) != cudaSuccess) {
    (void)cudaGetLastError();   // the side stream is an optimisation: without it the kernels stay on the main stream
    d->side_stream = nullptr;
  }
  if (cudaStreamCreateWithFlags(&d->h2d_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&d->d2h_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&d->ev_copy_join, cudaEventDisableTiming) != cudaSuccess) {
    (void)cudaGetLastError();   // without copy streams pipelined calls behave like ordinary ones
    d->h2d_stream = d->d2h_stream = nullptr;
  }
  *out = d;
  return RELUX_OK;
}

API int32_t relux_cuda_device_close(relux_device_t h) {
  Device* dev = as_device(h);
  if (!dev) { set_error("bad device handle"); return RELUX_ERR_BAD_HANDLE; }
  {
    DeviceGuard g(dev);
    if (g.rc) return g.rc;
    cudaStreamSynchronize(dev->stream);
    if (dev->flush_buf) cudaFree(dev->flush_buf);
    if (dev->side_stream) { cudaStreamSynchronize(dev->side_stream); cudaStreamDestroy(dev->side_stream); }
    if (dev->ev_fork) cudaEventDestroy(dev->ev_fork);
    if (dev->ev_join) cudaEventDestroy(dev->ev_join);
    for (cudaStream_t st : {dev->h2d_stream, dev->d2h_stream})
      if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
    if (dev->ev_copy_join) cudaEventDestroy(dev->ev_copy_join);
    cudaStreamDestroy(dev->stream);
    dev->magic = 0;
  }
  delete dev;
  return RELUX_OK;
}

API int32_t relux_cuda_sync(relux_device_t h) {
  GET_DEV(h);
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  if (dev->copies_in_flight) {
    if (dev->h2d_stream) RELUX_CUDA_TRY(cudaStreamSynchronize(dev->h2d_stream));
    if (dev->d2h_stream) RELUX_CUDA_TRY(cudaStreamSynchronize(dev->d2h_stream));
    RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
    dev->copies_in_flight = false;
  }
  return RELUX_OK;
}

API int32_t relux_cuda_device_info(relux_device_t h, char* name, int32_t name_len, int32_t* sm_count, int64_t* total_mem) {
  GET_DEV(h);
  if (name && name_len > 0) snprintf(name, (size_t)name_len, "%s", dev->name);
  if (sm_count) *sm_count = dev->sm_count;
  if (total_mem) *total_mem = (int64_t)dev->total_mem;
  return RELUX_OK;
}

API int32_t relux_cuda_launch_count(relux_device_t h, int64_t* count) {
  GET_DEV(h);
  if (!count) return RELUX_ERR_INVALID_ARG;
  *count = dev->launches;
  return RELUX_OK;
}

API int32_t relux_cuda_stream(relux_device_t h, void** stream) {
  GET_DEV(h);
  if (!stream) return RELUX_ERR_INVALID_ARG;
  *stream = (void*)dev->stream;
  return RELUX_OK;
}

API int32_t relux_cuda_dev_alloc(relux_device_t h, size_t bytes, void** dptr) {
  GET_DEV(h);
  if (!dptr) return RELUX_ERR_INVALID_ARG;
  *dptr = nullptr;
  if (bytes == 0) return RELUX_OK;
  RELUX_CUDA_TRY(cudaMalloc(dptr, bytes));
  return RELUX_OK;
}
API int32_t relux_cuda_dev_free(relux_device_t h, void* dptr) {
  GET_DEV(h);
  if (!dptr) return RELUX_OK;
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  RELUX_CUDA_TRY(cudaFree(dptr));
  return RELUX_OK;
}
API int32_t relux_cuda_host_alloc(relux_device_t h, size_t bytes, void** hptr) {
  GET_DEV(h);
  if (!hptr) return RELUX_ERR_INVALID_ARG;
  *hptr = nullptr;
  if (bytes == 0) return RELUX_OK;
  RELUX_CUDA_TRY(cudaMallocHost(hptr, bytes));
  return RELUX_OK;
}
API int32_t relux_cuda_host_free(relux_device_t h, void* hptr) {
  GET_DEV(h);
  if (!hptr) return RELUX_OK;
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  RELUX_CUDA_TRY(cudaFreeHost(hptr));
  return RELUX_OK;
}
API int32_t relux_cuda_h2d(relux_device_t h, void* dst, const void* src, size_t bytes) {
  GET_DEV(h);
  if (bytes == 0) return RELUX_OK;
  if (!dst || !src) return RELUX_ERR_INVALID_ARG;
  RELUX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, dev->stream));
  return RELUX_OK;
}
API int32_t relux_cuda_d2h(relux_device_t h, void* dst, const void* src, size_t bytes) {
  GET_DEV(h);
  if (bytes == 0) return RELUX_OK;
  if (!dst || !src) return RELUX_ERR_INVALID_ARG;
  RELUX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return RELUX_OK;
}
API int32_t relux_cuda_memset(relux_device_t h, void* dst, int32_t value, size_t bytes) {
  GET_DEV(h);
  if (bytes == 0) return RELUX_OK;
  if (!dst) return RELUX_ERR_INVALID_ARG;
  RELUX_CUDA_TRY(cudaMemsetAsync(dst, value, bytes, dev->stream));
  return RELUX_OK;
}

API int32_t relux_cuda_event_create(relux_device_t h, relux_event_t* ev) {
  GET_DEV(h);
  if (!ev) return RELUX_ERR_INVALID_ARG;
  cudaEvent_t e;
  RELUX_CUDA_TRY(cudaEventCreate(&e));
  *ev = (relux_event_t)e;
  return RELUX_OK;
}
API int32_t relux_cuda_event_record(relux_device_t h, relux_event_t ev) {
  GET_DEV(h);
  if (!ev) return RELUX_ERR_INVALID_ARG;
  int32_t rcj = join_copy_streams(dev);   // the event also covers the copies of pipelined calls
  if (rcj) return rcj;
  RELUX_CUDA_TRY(cudaEventRecord((cudaEvent_t)ev, dev->stream));
  return RELUX_OK;
}
API int32_t relux_cuda_event_elapsed_ms(relux_device_t h, relux_event_t a, relux_event_t b, float* ms) {
  GET_DEV(h);
  if (!a || !b || !ms) return RELUX_ERR_INVALID_ARG;
  RELUX_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)b));
  RELUX_CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)a, (cudaEvent_t)b));
  return RELUX_OK;
}
API int32_t relux_cuda_event_destroy(relux_device_t h, relux_event_t ev) {
  GET_DEV(h);
  if (!ev) return RELUX_OK;
  RELUX_CUDA_TRY(cudaEventDestroy((cudaEvent_t)ev));
  return RELUX_OK;
}
API int32_t relux_cuda_flush_l2(relux_device_t h) {
  GET_DEV(h);
  const size_t bytes = (size_t)256 << 20;  // twice the 126 MB L2
  if (!dev->flush_buf) {
    RELUX_CUDA_TRY(cudaMalloc(&dev->flush_buf, bytes));
    dev->flush_bytes = bytes;
  }
  RELUX_CUDA_TRY(cudaMemsetAsync(dev->flush_buf, 0, dev->flush_bytes, dev->stream));
  return RELUX_OK;
}

// ---------------------------------------------------------------------------------------------
// pools
// ---------------------------------------------------------------------------------------------
API int32_t relux_pool_create(relux_device_t h, const relux_pool_params* prm, relux_pool_t* out) {
  GET_DEV(h);
  if (!prm || !out) { set_error("nil argument"); return RELUX_ERR_INVALID_ARG; }
  *out = nullptr;
  if (prm->num_layers <= 0) { set_error("NewCache: numLayers=%d, must be > 0", prm->num_layers); return RELUX_ERR_INVALID_ARG; }
  if (prm->num_pages <= 0 || prm->page_tokens <= 0 || prm->max_seqs <= 0 || prm->max_pages_per_seq <= 0) {
    set_error("NewCache: num_pages, page_tokens, max_seqs, max_pages_per_seq must all be > 0");
    return RELUX_ERR_INVALID_ARG;
  }
  for (int i = 0; i < 5; i++)
    if (prm->reserved[i]) { set_error("reserved fields must be zero"); return RELUX_ERR_INVALID_ARG; }
  if (prm->flags & ~RELUX_POOL_FLAG_REFERENCE_COMPAT) { set_error("unknown pool flags 0x%x", prm->flags); return RELUX_ERR_INVALID_ARG; }
  Pool* p = new (std::nothrow) Pool();
  if (!p) return RELUX_ERR_OUT_OF_MEMORY;
  p->dev = dev;
  p->prm = *prm;
  if (prm->kind == RELUX_POOL_MLA) {
    if (prm->mla_dc <= 0 || prm->mla_dhr <= 0 || prm->mla_dhr % 2 || (prm->mla_dc % 8) || (prm->mla_dhr % 8)) {
      set_error("MLA pool: dC=%d and dHR=%d must be positive multiples of 8 (16-byte rows)", prm->mla_dc, prm->mla_dhr);
      delete p;
      return RELUX_ERR_INVALID_ARG;
    }
    p->row_elems_a = prm->mla_dc + prm->mla_dhr;
    p->page_elems = (size_t)prm->page_tokens * p->row_elems_a;
    p->layer_elems = p->page_elems * prm->num_pages;
  } else if (prm->kind == RELUX_POOL_GQA) {
    if (prm->gqa_num_kv_heads <= 0 || prm->gqa_head_dim <= 0 || prm->gqa_head_dim % 8) {
      set_error("GQA pool: num_kv_heads=%d, head_dim=%d (must be a positive multiple of 8)", prm->gqa_num_kv_heads, prm->gqa_head_dim);
      delete p;
      return RELUX_ERR_INVALID_ARG;
    }
    p->row_elems_a = prm->gqa_head_dim;
    p->page_elems = (size_t)prm->gqa_num_kv_heads * prm->page_tokens * prm->gqa_head_dim;
    p->layer_elems = 2 * p->page_elems * prm->num_pages;
  } else {
    set_error("unknown pool kind %d", prm->kind);
    delete p;
    return RELUX_ERR_INVALID_ARG;
  }
  const size_t storage_bytes = p->layer_elems * prm->num_layers * sizeof(uint16_t);
  const size_t table_n = (size_t)prm->max_seqs * prm->max_pages_per_seq, len_n = (size_t)prm->num_layers * prm->max_seqs;
  cudaError_t e = cudaSuccess;
  auto A = [&](void** q, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(q, bytes); };
  A((void**)&p->storage, storage_bytes);
  A((void**)&p->d_table, table_n * 4);
  A((void**)&p->d_len, len_n * 4);
  A((void**)&p->d_status, 8);   // [0] status word, [1] block counter of the append kernels
  A((void**)&p->d_seq_ids, (size_t)prm->max_seqs * 4);
  A((void**)&p->d_row_off, ((size_t)prm->max_seqs + 1) * 4);
  p->compat = (prm->flags & RELUX_POOL_FLAG_REFERENCE_COMPAT) != 0;
  if (p->compat && prm->kind == RELUX_POOL_MLA) {
    const size_t shadow_bytes = p->layer_elems * prm->num_layers * sizeof(float);
    A((void**)&p->shadow_f32, shadow_bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->shadow_f32, 0, shadow_bytes, dev->stream);
  }
  if (e == cudaSuccess) e = cudaMallocHost((void**)&p->h_stage, Pool::kStageSlots * (2 * (size_t)prm->max_seqs + 1) * 4);
  for (cudaEvent_t& ev : p->stage_ev)
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaMemsetAsync(p->d_table, 0xFF, table_n * 4, dev->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(p->d_len, 0, len_n * 4, dev->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(p->d_status, 0, 8, dev->stream);
  // The reference zero-fills new caches (kvcache.go:73-84, mla_cache.go:46-52).
  if (e == cudaSuccess) e = cudaMemsetAsync(p->storage, 0, storage_bytes, dev->stream);
  if (e != cudaSuccess) {
    int32_t rc = cuda_fail(e, "pool allocation");
    pool_free_all(p);
    return rc;
  }
  p->h_table.assign(table_n, -1);
  p->h_len.assign(len_n, 0);
  p->seq_pages.assign(prm->max_seqs, 0);
  p->seq_owned.assign(prm->max_seqs, 0);
  p->seq_stamp.assign(prm->max_seqs, 0u);
  if (p->compat) p->chunks.assign(len_n, std::vector<int32_t>());
  tuning_defaults(&p->tune);
  p->free_pages.resize(prm->num_pages);
  for (int i = 0; i < prm->num_pages; i++) p->free_pages[i] = prm->num_pages - 1 - i;
  // TMA views of the storage: all layers form one 2-D array of 64-row page slabs
  p->has_tmap = false;
  if (prm->page_tokens == 64) {
    if (prm->kind == RELUX_POOL_MLA && p->row_elems_a % 64 == 0) {
      // blocked page layout: the whole pool is one [blocks * 64][64] array, every TMA box is one contiguous 8 KB block
      p->mla_blocked = true;
      uint64_t rows = (uint64_t)prm->num_layers * prm->num_pages * (p->row_elems_a / 64) * prm->page_tokens;
      p->has_tmap = make_tmap_2d(&p->tmap_mla, p->storage, rows, 64, 64, 64);
    } else if (prm->kind == RELUX_POOL_GQA && prm->gqa_head_dim % 64 == 0) {
      uint64_t rows = (uint64_t)prm->num_layers * 2 * prm->num_pages * prm->gqa_num_kv_heads * prm->page_tokens;
      p->has_tmap = make_tmap_2d(&p->tmap_gqa, p->storage, rows, (uint64_t)prm->gqa_head_dim, 64, 64);
    }
  }
  *out = p;
  return RELUX_OK;
}

API int32_t relux_pool_destroy(relux_pool_t h) {
  GET_POOL(h);
  cudaStreamSynchronize(dev->stream);
  pool_free_all(p);
  return RELUX_OK;
}

API int32_t relux_pool_reset(relux_pool_t h) {
  GET_POOL(h);
  const relux_pool_params& prm = p->prm;
  std::fill(p->h_len.begin(), p->h_len.end(), 0);
  for (auto& c : p->chunks) c.clear();
  for (int s = 0; s < prm.max_seqs; s++)
    if (p->seq_owned[s]) {
      for (int i = 0; i < p->seq_pages[s]; i++) p->free_pages.push_back(p->h_table[(size_t)s * prm.max_pages_per_seq + i]);
      p->seq_pages[s] = 0;
      p->seq_owned[s] = 0;
    }
  RELUX_CUDA_TRY(cudaMemsetAsync(p->d_len, 0, p->h_len.size() * 4, dev->stream));
  RELUX_CUDA_TRY(cudaMemsetAsync(p->d_status, 0, 4, dev->stream));
  return RELUX_OK;
}

API int32_t relux_pool_set_tables(relux_pool_t h, const int32_t* table, int32_t n_seqs, int32_t stride, const int32_t* ctx_len) {
  GET_POOL(h);
  const relux_pool_params& prm = p->prm;
  if (!table || n_seqs <= 0 || n_seqs > prm.max_seqs || stride <= 0 || stride > prm.max_pages_per_seq) {
    set_error("set_tables: n_seqs=%d (max %d), stride=%d (max %d)", n_seqs, prm.max_seqs, stride, prm.max_pages_per_seq);
    return RELUX_ERR_INVALID_ARG;
  }
  // One pool has one owner of its pages: either the caller's tables or the library's free list.  Mixing them would
  // let relux_seq_alloc hand out a page that a caller-made table still maps.
  for (int s = 0; s < prm.max_seqs; s++)
    if (p->seq_owned[s]) { set_error("set_tables: sequence %d is owned by relux_seq_alloc; a pool uses either caller tables or the library's free list", s); return RELUX_ERR_INVALID_ARG; }
  std::vector<uint8_t> seen((size_t)prm.num_pages, 0);
  for (int s = 0; s < n_seqs; s++) {
    for (int i = 0; i < stride; i++) {
      int pg = table[(size_t)s * stride + i];
      if (pg < 0 || pg >= prm.num_pages) {
        set_error("page table entry [%d][%d]=%d outside [0,%d)", s, i, pg, prm.num_pages);
        return RELUX_ERR_BAD_PAGE;
      }
      if (seen[pg]) {
        set_error("page %d is mapped twice (second time at [%d][%d]): two sequences would share cache rows", pg, s, i);
        return RELUX_ERR_BAD_PAGE;
      }
      seen[pg] = 1;
    }
    if (ctx_len && (ctx_len[s] < 0 || ctx_len[s] > stride * prm.page_tokens)) {
      set_error("ctx_len[%d]=%d exceeds the %d tokens its pages hold", s, ctx_len[s], stride * prm.page_tokens);
      return RELUX_ERR_OVERFLOW;
    }
  }
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  for (int s = 0; s < n_seqs; s++) {
    for (int i = 0; i < stride; i++) p->h_table[(size_t)s * prm.max_pages_per_seq + i] = table[(size_t)s * stride + i];
    p->seq_pages[s] = stride;
    for (int l = 0; l < prm.num_layers; l++) {
      p->h_len[(size_t)l * prm.max_seqs + s] = ctx_len ? ctx_len[s] : 0;
      if (p->compat) {
        std::vector<int32_t>& c = p->chunks[(size_t)l * prm.max_seqs + s];
        c.clear();
        if (ctx_len && ctx_len[s] > 0) c.push_back(0);
      }
    }
  }
  // on the handle's stream (it does not synchronise with the legacy default stream), then waited for: the shadows are pageable
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_table, p->h_table.data(), p->h_table.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_len, p->h_len.data(), p->h_len.size() * 4, cudaMemcpyHostToDevice, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  p->caller_tables = true;
  return RELUX_OK;
}

API int32_t relux_seq_alloc(relux_pool_t h, int32_t max_tokens, int32_t* seq_id) {
  GET_POOL(h);
  const relux_pool_params& prm = p->prm;
  if (!seq_id || max_tokens <= 0) { set_error("seq_alloc: maxLen=%d, must be > 0", max_tokens); return RELUX_ERR_INVALID_ARG; }
  int need = (max_tokens + prm.page_tokens - 1) / prm.page_tokens;
  if (need > prm.max_pages_per_seq) { set_error("seq_alloc: %d tokens need %d pages, max_pages_per_seq=%d", max_tokens, need, prm.max_pages_per_seq); return RELUX_ERR_OVERFLOW; }
  if (p->caller_tables) { set_error("seq_alloc: this pool's page tables were set by relux_pool_set_tables; a pool uses either caller tables or the library's free list"); return RELUX_ERR_INVALID_ARG; }
  int s = -1;
  for (int i = 0; i < prm.max_seqs; i++)
    if (p->seq_pages[i] == 0) { s = i; break; }
  if (s < 0 || (int)p->free_pages.size() < need) { set_error("pool exhausted: %d free pages, %d needed", (int)p->free_pages.size(), need); return RELUX_ERR_POOL_EXHAUSTED; }
  for (int i = 0; i < need; i++) {
    p->h_table[(size_t)s * prm.max_pages_per_seq + i] = p->free_pages.back();
    p->free_pages.pop_back();
  }
  p->seq_pages[s] = need;
  p->seq_owned[s] = 1;
  for (int l = 0; l < prm.num_layers; l++) {
    p->h_len[(size_t)l * prm.max_seqs + s] = 0;
    if (p->compat) p->chunks[(size_t)l * prm.max_seqs + s].clear();
  }
  // every update goes through the handle's stream, so that it is ordered with the kernels queued there
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_table + (size_t)s * prm.max_pages_per_seq, &p->h_table[(size_t)s * prm.max_pages_per_seq], (size_t)need * 4,
                                 cudaMemcpyHostToDevice, dev->stream));
  for (int l = 0; l < prm.num_layers; l++) RELUX_CUDA_TRY(cudaMemsetAsync(p->d_len + (size_t)l * prm.max_seqs + s, 0, 4, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));   // h_table is pageable host memory
  *seq_id = s;
  return RELUX_OK;
}

API int32_t relux_seq_extend(relux_pool_t h, int32_t s, int32_t max_tokens) {
  GET_POOL(h);
  const relux_pool_params& prm = p->prm;
  if (s < 0 || s >= prm.max_seqs || p->seq_pages[s] == 0) { set_error("seq_extend: sequence %d is not live", s); return RELUX_ERR_INVALID_ARG; }
  if (!p->seq_owned[s]) { set_error("seq_extend: sequence %d uses a caller-supplied page table", s); return RELUX_ERR_INVALID_ARG; }
  const int need = (max_tokens + prm.page_tokens - 1) / prm.page_tokens, have = p->seq_pages[s];
  if (need <= have) return RELUX_OK;   // never shrinks: cached rows keep their pages
  if (need > prm.max_pages_per_seq) { set_error("seq_extend: %d tokens need %d pages, max_pages_per_seq=%d", max_tokens, need, prm.max_pages_per_seq); return RELUX_ERR_OVERFLOW; }
  if ((int)p->free_pages.size() < need - have) { set_error("pool exhausted: %d free pages, %d needed", (int)p->free_pages.size(), need - have); return RELUX_ERR_POOL_EXHAUSTED; }
  for (int i = have; i < need; i++) {
    p->h_table[(size_t)s * prm.max_pages_per_seq + i] = p->free_pages.back();
    p->free_pages.pop_back();
  }
  p->seq_pages[s] = need;
  // the new table entries lie past every page a queued kernel of this sequence can touch; the copy is ordered on the stream
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_table + (size_t)s * prm.max_pages_per_seq + have, &p->h_table[(size_t)s * prm.max_pages_per_seq + have],
                                 (size_t)(need - have) * 4, cudaMemcpyHostToDevice, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));   // h_table is pageable host memory
  return RELUX_OK;
}

API int32_t relux_seq_free(relux_pool_t h, int32_t s) {
  GET_POOL(h);
  const relux_pool_params& prm = p->prm;
  if (s < 0 || s >= prm.max_seqs || p->seq_pages[s] == 0) { set_error("seq_free: sequence %d is not live", s); return RELUX_ERR_INVALID_ARG; }
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  if (p->seq_owned[s])
    for (int i = 0; i < p->seq_pages[s]; i++) p->free_pages.push_back(p->h_table[(size_t)s * prm.max_pages_per_seq + i]);
  p->seq_pages[s] = 0;
  p->seq_owned[s] = 0;
  for (int l = 0; l < prm.num_layers; l++) {
    p->h_len[(size_t)l * prm.max_seqs + s] = 0;
    if (p->compat) p->chunks[(size_t)l * prm.max_seqs + s].clear();
    RELUX_CUDA_TRY(cudaMemsetAsync(p->d_len + (size_t)l * prm.max_seqs + s, 0, 4, dev->stream));
  }
  return RELUX_OK;
}

API int32_t relux_seq_len(relux_pool_t h, int32_t layer, int32_t s, int32_t* len) {
  GET_POOL(h);
  if (!len) return RELUX_ERR_INVALID_ARG;
  // TotalLen returns 0 for an out-of-range layer (kvcache.go:383-388)
  if (layer < 0 || layer >= p->prm.num_layers || s < 0 || s >= p->prm.max_seqs) { *len = 0; return RELUX_OK; }
  *len = p->h_len[(size_t)layer * p->prm.max_seqs + s];
  return RELUX_OK;
}

API int32_t relux_seq_set_len(relux_pool_t h, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const int32_t* new_len) {
  GET_POOL(h);
  return seq_set_len(p, layer, n_seqs, seq_ids, new_len);
}

// The caller holds the device guard.
int32_t relux::seq_set_len(Pool* p, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const int32_t* new_len) {
  Device* dev = p->dev;
  const relux_pool_params& prm = p->prm;
  if (!new_len || layer >= prm.num_layers) { set_error("set_len: bad arguments"); return RELUX_ERR_INVALID_ARG; }
  SeqBatch sb;
  int32_t rc = stage_batch(p, n_seqs, seq_ids, nullptr, 1, &sb);
  if (rc) return rc;
  for (int i = 0; i < n_seqs; i++)
    if (new_len[i] < 0 || new_len[i] > p->seq_pages[sb.seq[i]] * prm.page_tokens) {
      set_error("set_len: length %d outside the capacity of sequence %d", new_len[i], sb.seq[i]);
      return RELUX_ERR_OVERFLOW;
    }
  // lengths travel through the row-offset staging block
  int32_t* hs = nullptr;
  int slot_index = 0;
  rc = stage_acquire(p, &hs, &slot_index);
  if (rc) return rc;
  memcpy(hs, new_len, sizeof(int32_t) * n_seqs);
  RELUX_CUDA_TRY(cudaMemcpyAsync(p->d_row_off, hs, sizeof(int32_t) * n_seqs, cudaMemcpyHostToDevice, dev->stream));
  rc = stage_release(p, slot_index);
  if (rc) return rc;
  int l0 = layer < 0 ? 0 : layer, l1 = layer < 0 ? prm.num_layers : layer + 1;
  for (int l = l0; l < l1; l++) {
    rc = launch_set_len(p, sb, l, p->d_row_off);
    if (rc) return rc;
    for (int i = 0; i < n_seqs; i++) {
      int32_t& len = p->h_len[(size_t)l * prm.max_seqs + sb.seq[i]];
      note_set_len(p, l, sb.seq[i], len, new_len[i]);
      len = new_len[i];
    }
  }
  return RELUX_OK;
}

API int32_t relux_pool_status(relux_pool_t h, int32_t* status) {
  GET_POOL(h);
  if (!status) return RELUX_ERR_INVALID_ARG;
  RELUX_CUDA_TRY(cudaMemcpyAsync(status, p->d_status, 4, cudaMemcpyDeviceToHost, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  if (*status) RELUX_CUDA_TRY(cudaMemsetAsync(p->d_status, 0, 4, dev->stream));
  return RELUX_OK;
}

API int32_t relux_pool_read_rows(relux_pool_t h, const relux_read_rows_args* a) {
  GET_POOL(h);
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const relux_pool_params& prm = p->prm;
  const int32_t layer = a->layer, s = a->seq_id, tok0 = a->tok0, n = a->n_tokens;
  int32_t rc = check_layer(p, layer);
  if (rc) return rc;
  if (s < 0 || s >= prm.max_seqs || p->seq_pages[s] == 0 || tok0 < 0 || n < 0 || tok0 + n > p->seq_pages[s] * prm.page_tokens) {
    set_error("read_rows: sequence %d rows [%d,%d) outside its capacity", s, tok0, tok0 + n);
    return RELUX_ERR_INVALID_ARG;
  }
  if (n == 0) return RELUX_OK;
  size_t ea, eb;
  if (prm.kind == RELUX_POOL_MLA) { ea = (size_t)n * prm.mla_dc; eb = (size_t)n * prm.mla_dhr; }
  else { ea = eb = (size_t)n * prm.gqa_num_kv_heads * prm.gqa_head_dim; }
  rc = grow(dev, p->out_buf, (ea + eb) * 2);
  if (rc) return rc;
  uint16_t* da = (uint16_t*)p->out_buf.p;
  uint16_t* db = da + ea;
  rc = launch_gather_rows(p, layer, s, tok0, n, da, db);
  if (rc) return rc;
  if (a->dst_a) RELUX_CUDA_TRY(cudaMemcpyAsync(a->dst_a, da, ea * 2, cudaMemcpyDeviceToHost, dev->stream));
  if (a->dst_b) RELUX_CUDA_TRY(cudaMemcpyAsync(a->dst_b, db, eb * 2, cudaMemcpyDeviceToHost, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return RELUX_OK;
}

API int32_t relux_pool_wait_output(relux_pool_t h, int32_t calls_back) {
  GET_POOL(h);
  PipeSlots& po = p->pipe_out;
  if (calls_back < 0 || calls_back >= PipeSlots::kSlots || (uint64_t)calls_back >= po.next) {
    set_error("wait_output: calls_back=%d, but %llu pipelined outputs exist (two are kept)", calls_back, (unsigned long long)po.next);
    return RELUX_ERR_INVALID_ARG;
  }
  const int slot = (int)((po.next - 1 - (uint64_t)calls_back) % PipeSlots::kSlots);
  if (po.used[slot]) RELUX_CUDA_TRY(cudaEventSynchronize(po.freed[slot]));
  return RELUX_OK;
}

API int32_t relux_pool_tune(relux_pool_t h, int32_t knob, int32_t value) {
  GET_POOL(h);
  if (knob < 0 || knob >= RELUX_TUNE_COUNT) { set_error("unknown tuning knob %d", knob); return RELUX_ERR_INVALID_ARG; }
  p->tune.v[knob] = value < 0 ? kTuneDefault[knob] : value;
  return RELUX_OK;
}

API int32_t relux_mla_append(relux_pool_t h, const relux_append_args* a) {
  GET_POOL(h);
  return do_append(p, a, RELUX_POOL_MLA);
}
API int32_t relux_gqa_append(relux_pool_t h, const relux_append_args* a) {
  GET_POOL(h);
  return do_append(p, a, RELUX_POOL_GQA);
}
API int32_t relux_mla_decode(relux_pool_t h, const relux_attn_args* a) {
  GET_POOL(h);
  return do_attention(p, a, RELUX_POOL_MLA);
}
API int32_t relux_gqa_decode(relux_pool_t h, const relux_attn_args* a) {
  GET_POOL(h);
  return do_attention(p, a, RELUX_POOL_GQA);
}

static int32_t do_verify(Pool* p, const relux_attn_args* attn, const relux_append_args* kv, int kind) {
  if (!attn || !kv) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (kv->advance != 0) { set_error("verify: draft rows must be appended with advance=0"); return RELUX_ERR_INVALID_ARG; }
  if (kv->layer != attn->layer || kv->n_seqs != attn->n_seqs) { set_error("verify: append and attention arguments disagree"); return RELUX_ERR_INVALID_ARG; }
  if (attn->extra_tokens != attn->q_tokens) { set_error("verify: extra_tokens must equal q_tokens"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc = do_append(p, kv, kind);
  if (rc) return rc;
  return do_attention(p, attn, kind);
}
// One decode step: append the new rows (advance = 1), then attend over the cache that now includes them
// (MLA.forwardCached steps 4-6, mla.go:309-377; MHA.forwardCached steps 5-8, mha.go:283-348).  For the MLA tensor-core
// path the append rides in the attention call's preparation launch (absorb + append + stream partition: one kernel
// instead of three); every other case is the two calls one after the other.
static int32_t do_step(Pool* p, const relux_append_args* kv, const relux_attn_args* attn, int kind) {
  if (!attn || !kv) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (kv->advance != 1) { set_error("step: the new rows must be appended with advance=1 (use relux_*_verify for draft rows)"); return RELUX_ERR_INVALID_ARG; }
  if (kv->layer != attn->layer || kv->n_seqs != attn->n_seqs) { set_error("step: append and attention arguments disagree"); return RELUX_ERR_INVALID_ARG; }
  const bool same_ids = (!kv->seq_ids && !attn->seq_ids) ||
                        (kv->seq_ids && attn->seq_ids && memcmp(kv->seq_ids, attn->seq_ids, sizeof(int32_t) * (size_t)std::max(0, kv->n_seqs)) == 0);
  const bool fuse = kind == RELUX_POOL_MLA && p->prm.kind == RELUX_POOL_MLA && same_ids && kv->n_seqs > 0 && kv->n_seqs <= p->prm.max_seqs &&
                    kv->a && kv->b && attn->num_heads > 0 && attn->head_dim > 0 && mla_step_fusable(p, *attn, kv->n_seqs) &&
                    (kv->dtype == RELUX_DTYPE_F32 || kv->dtype == RELUX_DTYPE_BF16) && (kv->mem == RELUX_MEM_HOST || kv->mem == RELUX_MEM_DEVICE) &&
                    !(kv->flags & ~RELUX_CALL_PIPELINED) && kv->layer >= 0 && kv->layer < p->prm.num_layers;
  if (!fuse) {
    int32_t rc = do_append(p, kv, kind);
    if (rc) return rc;
    return do_attention(p, attn, kind);
  }
  // --- fused: validate and stage the append exactly as do_append does, but leave the launch to the attention call ---
  const relux_pool_params& prm = p->prm;
  SeqBatch sb;
  int32_t rc = stage_batch(p, kv->n_seqs, kv->seq_ids, kv->n_new, 1, &sb);
  if (rc) return rc;
  for (int i = 0; i < sb.n_seqs; i++) {
    const int s = sb.seq[i];
    const int len = p->h_len[(size_t)kv->layer * prm.max_seqs + s], cap = p->seq_pages[s] * prm.page_tokens;
    if (len + sb.rows[i] > cap) {
      set_error("Append: layer %d overflow: total=%d + newLen=%d > capacity=%d (sequence %d)", kv->layer, len, sb.rows[i], cap, s);
      return RELUX_ERR_OVERFLOW;
    }
  }
  if (sb.total_rows == 0) return do_attention(p, attn, kind);
  if (kv->mem == RELUX_MEM_DEVICE && ((rc = check_dev_align(kv->a, "append input a")) || (rc = check_dev_align(kv->b, "append input b")))) return rc;
  const size_t es = dtype_size(kv->dtype);
  const size_t bytes_a = (size_t)sb.total_rows * prm.mla_dc * es, bytes_b = (size_t)sb.total_rows * prm.mla_dhr * es;
  const bool piped = (kv->flags & RELUX_CALL_PIPELINED) && kv->mem == RELUX_MEM_HOST && p->dev->h2d_stream;
  const void *da = nullptr, *db = nullptr;
  int slot_a = -1, slot_b = -1;
  if (piped) {
    if ((rc = pipe_stage_in(p, p->pipe_app_a, kv->a, bytes_a, &da, &slot_a))) return rc;
    if ((rc = pipe_stage_in(p, p->pipe_app_b, kv->b, bytes_b, &db, &slot_b))) return rc;
  } else if (kv->mem == RELUX_MEM_HOST) {
    // the attention call stages q / q_rope in in_a / in_b: the step's rows get a block of their own
    if ((rc = grow(p->dev, p->step_rows, bytes_a + bytes_b + 256))) return rc;
    char* base = (char*)p->step_rows.p;
    const size_t off_b = (bytes_a + 255) & ~(size_t)255;
    RELUX_CUDA_TRY(cudaMemcpyAsync(base, kv->a, bytes_a, cudaMemcpyHostToDevice, p->dev->stream));
    RELUX_CUDA_TRY(cudaMemcpyAsync(base + off_b, kv->b, bytes_b, cudaMemcpyHostToDevice, p->dev->stream));
    da = base;
    db = base + off_b;
  } else {
    da = kv->a;
    db = kv->b;
  }
  // the host lengths count the new rows from here on: the attention call plans with them
  for (int i = 0; i < sb.n_seqs; i++) p->h_len[(size_t)kv->layer * prm.max_seqs + sb.seq[i]] += sb.rows[i];
  StepAppend step{da, db, kv->dtype, sb.d_row_off};
  rc = do_attention(p, attn, kind, &step);
  if (rc) {   // nothing was launched for the append: take the rows back
    for (int i = 0; i < sb.n_seqs; i++) p->h_len[(size_t)kv->layer * prm.max_seqs + sb.seq[i]] -= sb.rows[i];
    return rc;
  }
  if ((rc = pipe_release(p, p->pipe_app_a, slot_a)) || (rc = pipe_release(p, p->pipe_app_b, slot_b))) return rc;
  return RELUX_OK;
}
API int32_t relux_mla_step(relux_pool_t h, const relux_append_args* kv, const relux_attn_args* attn) {
  GET_POOL(h);
  return do_step(p, kv, attn, RELUX_POOL_MLA);
}
API int32_t relux_gqa_step(relux_pool_t h, const relux_append_args* kv, const relux_attn_args* attn) {
  GET_POOL(h);
  return do_step(p, kv, attn, RELUX_POOL_GQA);
}

API int32_t relux_mla_expand_kv(relux_pool_t h, const relux_mla_expand_args* a) {
  GET_POOL(h);
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  if (p->prm.kind != RELUX_POOL_MLA) { set_error("pool kind does not match this call (MLA pool needed)"); return RELUX_ERR_INVALID_ARG; }
  int32_t rc = check_layer(p, a->layer);
  if (rc) return rc;
  if (a->num_heads <= 0 || a->extra_tokens < 0) { set_error("bad expansion arguments"); return RELUX_ERR_INVALID_ARG; }
  if (p->compat || !mla_expand_eligible(p, a->num_heads, 128)) {
    set_error("the expansion kernel covers latent 512, 64-token pages and 128-wide heads on an ordinary pool");
    return RELUX_ERR_UNSUPPORTED;
  }
  SeqBatch sb;
  rc = stage_batch(p, a->n_seqs, a->seq_ids, nullptr, 1, &sb);
  if (rc) return rc;
  const int64_t rows = mla_expand_rows(p, sb, a->layer, a->extra_tokens);
  if (a->rows_total_out) *a->rows_total_out = rows;
  if (!a->kv_out) return RELUX_OK;
  if (!a->w_uk || !a->w_uv || !a->seq_base || a->rows_total != rows) {
    set_error("expansion: nil weights / seq_base, or rows_total=%lld does not match the cached lengths (%lld)", (long long)a->rows_total,
              (long long)rows);
    return RELUX_ERR_INVALID_ARG;
  }
  if (2 * (int64_t)a->num_heads * rows >= ((int64_t)1 << 31)) { set_error("expansion: more rows than one launch addresses"); return RELUX_ERR_UNSUPPORTED; }
  if ((rc = check_dev_align(a->w_uk, "w_uk")) || (rc = check_dev_align(a->w_uv, "w_uv")) || (rc = check_dev_align(a->kv_out, "kv_out"))) return rc;
  uint16_t* kx = (uint16_t*)a->kv_out;
  rc = launch_mla_expand_sm100(p, sb, a->layer, a->extra_tokens, a->num_heads, (const uint16_t*)a->w_uk, (const uint16_t*)a->w_uv, rows, kx,
                               kx + (size_t)a->num_heads * rows * 128, a->seq_base);
  if (rc) return rc;
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return RELUX_OK;
}

API int32_t relux_gqa_verify(relux_pool_t h, const relux_attn_args* attn, const relux_append_args* kv) {
  GET_POOL(h);
  return do_verify(p, attn, kv, RELUX_POOL_GQA);
}
API int32_t relux_mla_verify(relux_pool_t h, const relux_attn_args* attn, const relux_append_args* kv) {
  GET_POOL(h);
  return do_verify(p, attn, kv, RELUX_POOL_MLA);
}

API int32_t relux_mla_forward_cached(relux_pool_t h, const relux_mla_layer_args* a) {
  GET_POOL(h);
  return do_mla_layer(p, a);
}

API int32_t relux_gqa_forward_cached(relux_pool_t h, const relux_gqa_layer_args* a) {
  GET_POOL(h);
  return do_gqa_layer(p, a);
}

API int32_t relux_spec_accept(relux_pool_t h, const relux_spec_accept_args* a) {
  GET_POOL(h);
  return do_spec_accept(p, a);
}

API int32_t relux_sampler_sample(relux_pool_t h, const relux_sample_args* a) {
  GET_POOL(h);
  return do_sample(p, a);
}

API int32_t relux_matmul_f32_bf16(relux_pool_t h, const relux_matmul_args* a) {
  GET_POOL(h);
  return do_matmul(p, a);
}

API int32_t relux_mla_import_weights(relux_pool_t h, const relux_mla_import_args* a) {
  GET_POOL(h);
  return do_import_mla(p, a);
}

API int32_t relux_pool_selftest_wait(relux_pool_t h, int32_t polls) {
  GET_POOL(h);
  return do_selftest_wait(p, polls);
}

API int32_t relux_pool_last_kernel_ms(relux_pool_t h, float* ms) {
  GET_POOL(h);
  if (!ms) return RELUX_ERR_INVALID_ARG;
  if (!p->timed_calls) { set_error("no attention kernel has been timed on this pool yet"); return RELUX_ERR_INVALID_ARG; }
  const auto& pair = p->ev_ring[(p->timed_calls - 1) % Pool::kTimeRing];
  if (!pair[0] || !pair[1]) { set_error("the last call recorded no timing events"); return RELUX_ERR_CUDA; }
  RELUX_CUDA_TRY(cudaEventSynchronize(pair[1]));
  RELUX_CUDA_TRY(cudaEventElapsedTime(ms, pair[0], pair[1]));
  return RELUX_OK;
}

// Times of the last n calls of a ring, oldest first; slots whose events were never recorded are skipped.
static int32_t ring_list(cudaEvent_t (*ring)[2], uint64_t calls, int32_t last_n, float* out, int32_t* counted) {
  const uint64_t n = std::min<uint64_t>(std::min<uint64_t>((uint64_t)last_n, calls), Pool::kTimeRing);
  int32_t k = 0;
  for (uint64_t i = n; i-- > 0;) {
    cudaEvent_t* pair = ring[(calls - 1 - i) % Pool::kTimeRing];
    if (!pair[0] || !pair[1]) continue;
    float ms = 0.f;
    RELUX_CUDA_TRY(cudaEventSynchronize(pair[1]));
    RELUX_CUDA_TRY(cudaEventElapsedTime(&ms, pair[0], pair[1]));
    out[k++] = ms;
  }
  *counted = k;
  return RELUX_OK;
}
static int32_t ring_mean(cudaEvent_t (*ring)[2], uint64_t calls, int32_t last_n, float* mean_ms, int32_t* counted) {
  std::vector<float> ms((size_t)std::min<int64_t>(last_n, Pool::kTimeRing));
  int32_t n = 0;
  int32_t rc = ring_list(ring, calls, last_n, ms.data(), &n);
  if (rc) return rc;
  double sum = 0.0;
  for (int i = 0; i < n; i++) sum += ms[i];
  *mean_ms = n ? (float)(sum / (double)n) : 0.f;
  if (counted) *counted = n;
  return RELUX_OK;
}

API int32_t relux_pool_kernel_ms_list(relux_pool_t h, int32_t last_n, float* ms_out, int32_t* counted) {
  GET_POOL(h);
  if (!ms_out || !counted || last_n <= 0) return RELUX_ERR_INVALID_ARG;
  return ring_list(p->ev_ring, p->timed_calls, last_n, ms_out, counted);
}

API int32_t relux_pool_kernel_ms_mean(relux_pool_t h, int32_t last_n, float* mean_ms, int32_t* counted) {
  GET_POOL(h);
  if (!mean_ms || last_n <= 0) return RELUX_ERR_INVALID_ARG;
  if (!p->timed_calls) { set_error("no attention kernel has been timed on this pool yet"); return RELUX_ERR_INVALID_ARG; }
  return ring_mean(p->ev_ring, p->timed_calls, last_n, mean_ms, counted);
}

API int32_t relux_pool_projection_ms_mean(relux_pool_t h, int32_t last_n, float* mean_ms, int32_t* counted) {
  GET_POOL(h);
  if (!mean_ms || last_n <= 0) return RELUX_ERR_INVALID_ARG;
  if (!p->proj_calls) { set_error("no layer step has run on this pool yet"); return RELUX_ERR_INVALID_ARG; }
  return ring_mean(p->proj_ring, p->proj_calls, last_n, mean_ms, counted);
}
