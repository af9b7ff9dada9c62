// Split-KV work list shared by the FAST attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace relux {

struct WorkItem {
  int32_t seq_index;   // position of the sequence inside this call (row block of q / out)
  int32_t seq;         // pool sequence id (page-table row)
  int32_t page_begin;  // first logical page of the chunk
  int32_t page_end;    // one past the last logical page
};

// Item of a stream plan (plan_stream): like WorkItem plus the sequence's token count, so that a persistent kernel
// needs a single load per item.
struct __align__(16) StreamItem {
  int32_t seq_index;
  int32_t seq;
  int32_t page_begin;
  int32_t page_end;
  int32_t tokens;      // cached length of the sequence + the call's extra tokens
  int32_t pad[3];
};

struct SplitPlan {
  int chunk_pages = 0;
  int num_items = 0;
  WorkItem* items = nullptr;    // device
  int32_t* chunk_off = nullptr; // device [n_seqs + 1]
  // stream plans only (plan_stream): worker w owns items [worker_first[w], worker_first[w + 1])
  int num_workers = 0;
  StreamItem* stream_items = nullptr;  // device [num_items]
  int32_t* worker_first = nullptr;     // device [num_workers + 1]
};

struct Pool;
struct SeqBatch;
int32_t plan_splitkv(Pool* p, const SeqBatch& sb, int layer, int extra, int ctas_per_item, int min_chunk_pages, int chunk_multiple,
                     int max_chunk_pages, SplitPlan* plan);
// Stream partition for persistent kernels: the pages of all sequences of the call, laid end to end, are cut into
// `workers` equal ranges of `chunk_pages` pages (a multiple of `page_multiple`); one item = the part of one sequence
// inside one range, so a worker meets an item boundary only where a sequence ends inside its range.
// `st`: the stream the builder kernel is launched on (the pool's main stream, or the device's side stream).
// launch_builder = false: only the host half (counts, buffers); the caller builds the lists itself (the fused decode-step
// preparation of mla_proj.cu does it inside its own launch).
int32_t plan_stream(Pool* p, const SeqBatch& sb, int layer, int extra, int workers, int page_multiple, SplitPlan* plan, cudaStream_t st,
                    bool launch_builder = true);
int32_t launch_build_worklist_raw(cudaStream_t st, const int32_t* len, const int32_t* seq_ids, int n_seqs, int extra, int page_tokens,
                                  int chunk_pages, WorkItem* items, int32_t* chunk_off);
int32_t launch_merge_raw(cudaStream_t st, const float* part_o, const float* part_ml, const int32_t* chunk_off, int n_seqs, int rows,
                         int width, float* out);
int32_t launch_merge(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, uint16_t* out_bf16);
// Same, for a launch that covers `rows` of the `out_rows` output rows of every sequence, starting at row out_row0.
int32_t launch_merge_rows(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, int out_rows, int out_row0,
                          int slices = 1, long long part_group_rows = 0);

}  // namespace relux
