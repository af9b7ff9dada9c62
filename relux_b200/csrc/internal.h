// Host-side structures of librelux_cuda: device handle, paged pool, per-call staging.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "relux_cuda.h"

namespace relux {

constexpr uint32_t kDeviceMagic = 0x52444556u;  // "RDEV"
constexpr uint32_t kPoolMagic = 0x52504F4Cu;    // "RPOL"

void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);

#define RELUX_CUDA_TRY(expr)                                  \
  do {                                                        \
    cudaError_t e__ = (expr);                                 \
    if (e__ != cudaSuccess) return ::relux::cuda_fail(e__, #expr); \
  } while (0)

struct Device {
  uint32_t magic = kDeviceMagic;
  int index = 0;
  int sm_count = 0;
  size_t total_mem = 0;
  char name[256] = {0};
  cudaStream_t stream = nullptr;
  // side stream for small kernels that do not depend on their predecessor (forked from / joined to `stream` by events)
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  // copy streams of pipelined calls (RELUX_CALL_PIPELINED): host -> device inputs, device -> host outputs
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  cudaEvent_t ev_copy_join = nullptr;
  bool copies_in_flight = false;
  std::mutex mu;
  int64_t launches = 0;
  void* flush_buf = nullptr;
  size_t flush_bytes = 0;
};

// A device buffer that grows on demand (never shrinks) for inputs that arrive in host memory
// and for kernel scratch.  Growth synchronises the stream before the old block is freed.
struct GrowBuf {
  void* p = nullptr;
  size_t cap = 0;
};

// Tuning knobs of a pool.  Defaults come from the environment ONCE, when the pool is created (RELUX_MLA_GENERIC,
// RELUX_MLA_WORKERS, RELUX_CHUNK_PAGES, RELUX_GEMM_GENERIC, RELUX_GEMM_SPLIT, RELUX_GQA_PROMPT_PARTIAL_MB,
// RELUX_SEL_CLUSTER, RELUX_SEL_LOOKAHEAD, RELUX_SEL_BATCHED, RELUX_GQA_PROMPT_SLICES); relux_pool_tune changes them
// afterwards.  No launch path reads the environment.
struct Tuning {
  int32_t v[RELUX_TUNE_COUNT];
  int32_t get(int knob) const { return v[knob]; }
};

// Two device buffers used in turn by pipelined calls.  `ready`: the copy into (inputs) or the kernels writing (outputs)
// the slot are done; `freed`: whoever read the slot is done with it, so it may be overwritten.
struct PipeSlots {
  static constexpr int kSlots = 2;
  GrowBuf buf[kSlots];
  cudaEvent_t ready[kSlots] = {}, freed[kSlots] = {};
  bool used[kSlots] = {};
  uint64_t next = 0;
};

struct Pool {
  uint32_t magic = kPoolMagic;
  Device* dev = nullptr;
  relux_pool_params prm{};
  Tuning tune{};
  int row_elems_a = 0;  // MLA: dC + dHR (one fused row); GQA: head_dim
  size_t page_elems = 0;    // elements per page per tensor (MLA: P*(dC+dHR); GQA: Hkv*P*D for K, same for V)
  size_t layer_elems = 0;   // elements per layer (GQA: K then V)
  uint16_t* storage = nullptr;  // bf16 bits
  int32_t* d_table = nullptr;   // [max_seqs][max_pages_per_seq]
  int32_t* d_len = nullptr;     // [num_layers][max_seqs]
  int32_t* d_status = nullptr;   // [0] status word, [1] block counter of the append kernels
  std::vector<int32_t> h_table, h_len;
  std::vector<int32_t> seq_pages;  // pages reserved per sequence (capacity), 0 = slot not live
  std::vector<uint8_t> seq_owned;  // 1 = table rows were filled by relux_seq_alloc
  bool caller_tables = false;      // relux_pool_set_tables filled the tables: the free list stays unused until a reset
  std::vector<int32_t> free_pages;
  std::vector<uint32_t> seq_stamp;  // duplicate-id detection of stage_batch: call number that last named the sequence
  uint32_t stamp = 0;
  // reference-compat pools (RELUX_POOL_FLAG_REFERENCE_COMPAT): what the quirk-faithful attention mode needs
  bool compat = false;
  float* shadow_f32 = nullptr;   // MLA: float32 copy of every appended row, [layer][page][token][dC + dHR] (the reference's cache
                                 // is float32, mla_cache.go:46-52)
  std::vector<std::vector<int32_t>> chunks;   // GQA: per (layer, sequence) the first row of every Append call (kvcache.go:407-438
                                              // writes chunk-linear; mha.go:299-312 reads head-major)
  GrowBuf chunk_tab;             // device staging of the chunk starts of one call's sequences
  // per-call staging of small host arrays (seq ids, row offsets)
  int32_t* d_seq_ids = nullptr;  // [max_seqs]
  int32_t* d_row_off = nullptr;  // [max_seqs + 1]
  // Pinned staging for per-call id / row-offset / length arrays: a ring of slots, each guarded by its own event, so
  // that a call waits for a copy issued kStageSlots calls ago (long finished) instead of for the previous step's kernels.
  static constexpr int kStageSlots = 8;
  int32_t* h_stage = nullptr;    // pinned [kStageSlots][2 * max_seqs + 1]
  cudaEvent_t stage_ev[kStageSlots] = {};
  bool stage_busy[kStageSlots] = {};
  uint32_t stage_next = 0;
  size_t stage_slot_ints() const { return 2 * (size_t)prm.max_seqs + 1; }
  // staging of activations that arrive in host memory, and outputs that leave to it
  GrowBuf in_a, in_b, out_buf, q_conv;
  GrowBuf expand_buf;  // expanded keys / values of an MLA prompt (+ the sequences' first rows)
  GrowBuf step_rows;   // host-resident new rows of a fused decode step (the attention call uses in_a / in_b for the queries)
  PipeSlots pipe_in_a, pipe_in_b, pipe_app_a, pipe_app_b, pipe_out;   // the same for pipelined calls
  // attention scratch
  GrowBuf q_abs;     // MLA absorbed queries, bf16 [n][S][H][dC+dHR]
  GrowBuf part_o;    // split-KV partial accumulators, f32
  GrowBuf part_ml;   // split-KV partial (max, sum), f32 pairs
  GrowBuf work;      // int32 work list + per-sequence chunk offsets
  GrowBuf o_lat;     // MLA merged latent output, f32/bf16
  // TMA descriptors over the pool storage (built at create when the shape allows it)
  CUtensorMap tmap_mla{};   // 2-D [rows][dC+dHR], box 64 x 64, 128-byte swizzle
  CUtensorMap tmap_gqa{};   // 2-D [rows][D],      box 64 x 64, 128-byte swizzle
  bool has_tmap = false;
  bool mla_blocked = false;   // MLA pages stored as 64-column blocks (see mla_page_off)
  // layer-level step (layer_step.cu): RoPE tables [cos | sin][positions][dHR / 2] and the step's scratch block
  GrowBuf rope_tab, layer_buf;
  int rope_dim = 0, rope_positions = 0;
  float rope_base = 0.f;
  // timing of the dominant kernel: a ring of event pairs, one pair per attention call, so that a caller can read
  // the device times of its last kTimeRing calls after the fact without a synchronisation between them.  The events
  // of a slot are created the first time the slot is used.
  static constexpr int kTimeRing = 8192;
  cudaEvent_t ev_ring[kTimeRing][2] = {};
  uint64_t timed_calls = 0;
  uint64_t attn_calls = 0;   // MLA decode calls, timed or not (RELUX_TUNE_KERNEL_TIMING_STRIDE)
  cudaEvent_t proj_ring[kTimeRing][2] = {};   // same, around the input-projection GEMM of the layer step
  uint64_t proj_calls = 0;
  static cudaEvent_t ring_event(cudaEvent_t (*ring)[2], uint64_t call, int which) {
    cudaEvent_t& e = ring[call % kTimeRing][which];
    if (!e && cudaEventCreate(&e) != cudaSuccess) { (void)cudaGetLastError(); e = nullptr; }
    return e;
  }
  cudaEvent_t ev_begin() { return ring_event(ev_ring, timed_calls, 0); }
  cudaEvent_t ev_end() { return ring_event(ev_ring, timed_calls, 1); }
};

inline Device* as_device(relux_device_t h) {
  Device* d = (Device*)h;
  return (d && d->magic == kDeviceMagic) ? d : nullptr;
}
inline Pool* as_pool(relux_pool_t h) {
  Pool* p = (Pool*)h;
  return (p && p->magic == kPoolMagic && p->dev && p->dev->magic == kDeviceMagic) ? p : nullptr;
}

int32_t grow(Device* dev, GrowBuf& b, size_t bytes);
// Pipelined staging: copies a host input into the next slot on the copy stream and makes the compute stream wait for it;
// pipe_release is called once the kernels that read the slot have been queued.
int32_t pipe_stage_in(Pool* p, PipeSlots& ps, const void* src, size_t bytes, const void** dptr, int* slot);
int32_t pipe_release(Pool* p, PipeSlots& ps, int slot);
// Next staging slot (waits for the copy that last used it); call stage_release after the copies are enqueued.
int32_t stage_acquire(Pool* p, int32_t** slot, int* slot_index);
int32_t stage_release(Pool* p, int slot_index);

// Resolved view of one call's sequences on the device.
struct SeqBatch {
  int32_t n_seqs = 0;
  const int32_t* d_seq_ids = nullptr;  // nullptr = identity
  const int32_t* d_row_off = nullptr;  // nullptr = one row per sequence
  int32_t total_rows = 0;
  int32_t max_rows = 0;
  std::vector<int32_t> seq;  // host copy of ids
  std::vector<int32_t> rows; // host copy of rows per sequence
};
int32_t stage_batch(Pool* p, int32_t n_seqs, const int32_t* seq_ids, const int32_t* n_rows, int32_t uniform_rows,
                    SeqBatch* out);

// kernels (defined in the .cu files of this directory)
int32_t launch_mla_append(Pool* p, const SeqBatch& sb, int layer, const void* ckv, const void* kr, int dtype, int advance);
int32_t launch_gqa_append(Pool* p, const SeqBatch& sb, int layer, const void* k, const void* v, int dtype, int layout,
                          int advance);
int32_t launch_set_len(Pool* p, const SeqBatch& sb, int layer, const int32_t* d_new_len);
int32_t launch_gather_rows(Pool* p, int layer, int seq, int tok0, int n, uint16_t* d_a, uint16_t* d_b);
int32_t launch_attn_reference_gqa(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const float* d_q, float* d_out);
int32_t launch_attn_reference_mla(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const float* d_q, const float* d_qr,
                                  float* d_out);
int32_t launch_gqa_decode_fast(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, void* d_out);
// True when this call is a multi-token call that the tcgen05 prefill kernel serves (it takes bf16 queries).
bool mla_expand_eligible(const Pool* p, int num_heads, int head_dim);
int64_t mla_expand_rows(const Pool* p, const SeqBatch& sb, int layer, int extra);
int32_t launch_mla_expand_sm100(Pool* p, const SeqBatch& sb, int layer, int extra, int H, const uint16_t* w_uk, const uint16_t* w_uv,
                                int64_t Ttot, uint16_t* kx, uint16_t* vx, int32_t* seq_base);
bool mla_prefill_eligible(const Pool* p, const SeqBatch& sb, const relux_attn_args& a);
bool gqa_prompt_wants_bf16(const Pool* p, const relux_attn_args& a);
// The new rows of a decode step handed to the attention call, for the fused preparation (one launch for absorb + append +
// stream partition); the host lengths already include them.
struct StepAppend {
  const void* ckv;
  const void* kr;
  int dtype;
  const int32_t* d_row_off;   // device row offsets of the append batch (nullptr = one row per sequence)
};
int32_t launch_mla_decode_fast(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const void* d_q, const void* d_qr,
                               void* d_out, const StepAppend* step = nullptr);
// True when launch_mla_decode_fast can take the step's append into its preparation launch.
bool mla_step_fusable(Pool* p, const relux_attn_args& a, int n_seqs);

int32_t do_mla_layer(Pool* p, const relux_mla_layer_args* a);
int32_t do_gqa_layer(Pool* p, const relux_gqa_layer_args* a);
int32_t do_spec_accept(Pool* p, const relux_spec_accept_args* a);
int32_t do_sample(Pool* p, const relux_sample_args* a);
int32_t do_matmul(Pool* p, const relux_matmul_args* a);
int32_t do_import_mla(Pool* p, const relux_mla_import_args* a);
int32_t do_selftest_wait(Pool* p, int32_t polls);
int32_t seq_set_len(Pool* p, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const int32_t* new_len);
// Chunk bookkeeping of reference-compat pools (no-ops otherwise): an append of n rows at old_len, a length change.
void note_append(Pool* p, int layer, int seq, int old_len, int n);
void note_set_len(Pool* p, int layer, int seq, int old_len, int new_len);
// Host pointers handed over as device memory must be 16-byte aligned: the kernels read them with vector loads.
int32_t check_dev_align(const void* ptr, const char* what);

// Tensor maps (runtime.cu).  bf16 elements, 128-byte swizzle, no out-of-bounds fill value (zeros); false when the driver
// entry point is missing or refuses the map.
//   2-D: [rows][cols], cols contiguous, box = box_cols x box_rows.
//   3-D: [outer][mid][cols], cols contiguous and mid rows adjacent, box = box_cols x box_mid x box_outer.
bool make_tmap_2d(CUtensorMap* m, void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows);
bool make_tmap_3d(CUtensorMap* m, void* base, uint64_t outer, uint64_t mid, uint64_t cols, uint32_t box_cols, uint32_t box_mid,
                  uint32_t box_outer);

inline void count_launch(Device* d, int n = 1) { d->launches += n; }

// Launches `kern`; with `chained` the launch carries the programmatic stream-serialization attribute, so the grid may be
// scheduled while the kernel before it in the stream still runs.  Such a kernel calls chain_wait() (common.cuh) before
// its first access to global memory, which is what keeps the stream's order of results.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(bool chained, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &at;
  cfg.numAttrs = chained ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

}  // namespace relux
