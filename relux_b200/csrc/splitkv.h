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

struct SplitPlan {
  int chunk_pages = 0;
  int num_items = 0;
  WorkItem* items = nullptr;    // device
  int32_t* chunk_off = nullptr; // device [n_seqs + 1]
};

struct Pool;
struct SeqBatch;
int32_t plan_splitkv(Pool* p, const SeqBatch& sb, int layer, int extra, int ctas_per_item, int min_chunk_pages, int chunk_multiple,
                     int max_chunk_pages, SplitPlan* plan);
int32_t launch_build_worklist_raw(cudaStream_t st, const int32_t* len, const int32_t* seq_ids, int n_seqs, int extra, int page_tokens,
                                  int chunk_pages, WorkItem* items, int32_t* chunk_off);
int32_t launch_merge_raw(cudaStream_t st, const float* part_o, const float* part_ml, const int32_t* chunk_off, int n_seqs, int rows,
                         int width, float* out);
int32_t launch_merge(Pool* p, const SplitPlan& plan, int n_seqs, int rows, int width, float* out, uint16_t* out_bf16);

}  // namespace relux
