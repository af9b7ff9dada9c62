/*
 * relux_cuda.h -- C ABI of librelux_cuda.so, the B200 (sm_100a) KV-cache and cached-attention
 * path for the pure-Go framework relux.
 *
 * Design rules of this surface (so that Go can bind it with purego, without cgo):
 *   - every function is extern "C", returns an int32 status (0 = ok, negative = error), takes
 *     only integers, floats, pointers, or a pointer to a plain-old-data argument struct;
 *   - no callbacks, no struct by value, no C++ exceptions cross the boundary;
 *   - every call selects the handle's CUDA device itself (goroutines migrate between OS threads);
 *   - calls on one device handle are serialised internally; distinct handles are independent;
 *   - there is no CPU fallback: when a GPU cannot do the work the call fails with a status;
 *   - every pointer flagged RELUX_MEM_DEVICE (and every weight pointer) must be 16-byte aligned and every row of the
 *     array it names a multiple of 16 bytes long: the kernels read them with 16-byte vector loads.  A misaligned device
 *     pointer is refused with RELUX_ERR_INVALID_ARG before anything is launched.  Host pointers have no such rule.
 *
 * "Reference" below is the relux source tree; paths are relative to its root.
 */
#ifndef RELUX_CUDA_H_
#define RELUX_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RELUX_CUDA_ABI_VERSION 1

/* ---- status codes ------------------------------------------------------------------------ */
#define RELUX_OK 0
#define RELUX_ERR_INVALID_ARG (-1)    /* nil pointer, bad enum, mismatched dims                     */
#define RELUX_ERR_CUDA (-2)           /* a CUDA runtime/driver call failed; see relux_cuda_last_error */
#define RELUX_ERR_OUT_OF_MEMORY (-3)  /* device allocation failed                                  */
#define RELUX_ERR_POOL_EXHAUSTED (-4) /* no free page / sequence slot                              */
#define RELUX_ERR_OVERFLOW (-5)       /* append past a sequence's page capacity (the reference panics:
                                         internal/transformer/kvcache.go:282-285, mla_cache.go:164-167) */
#define RELUX_ERR_BAD_PAGE (-6)       /* a page table holds an id outside the pool (found on device) */
#define RELUX_ERR_TIMEOUT (-7)        /* a bounded device-side wait ran out                         */
#define RELUX_ERR_BAD_HANDLE (-8)
#define RELUX_ERR_UNSUPPORTED (-9)    /* shape outside what the kernels implement                   */
#define RELUX_ERR_NO_DEVICE (-10)     /* no CUDA device / library built without a usable GPU        */

/* ---- enums ------------------------------------------------------------------------------- */
#define RELUX_DTYPE_F32 0
#define RELUX_DTYPE_BF16 1
#define RELUX_MEM_HOST 0
#define RELUX_MEM_DEVICE 1
/* Activation layouts.  TOKEN_MAJOR: [seq][token][head][dim].  HEAD_MAJOR: [seq][head][token][dim],
 * the layout of the reference's tensors after rearrangeBSNH (internal/transformer/mha.go:789-803). */
#define RELUX_LAYOUT_TOKEN_MAJOR 0
#define RELUX_LAYOUT_HEAD_MAJOR 1
#define RELUX_POOL_MLA 0
#define RELUX_POOL_GQA 1
/* Attention arithmetic.
 * FAST: bf16 tensor-core contractions, online softmax with exp2, split-KV + merge.
 * REFERENCE: float32 CUDA-core arithmetic in the reference's own operation order
 *   (k-ascending unfused dot products, full-row softmax with the fastexp32 bit trick of
 *   internal/transformer/mha.go:823-861, decompress-then-attend for MLA as mla.go:323-377);
 *   meant for small models where token-id identity with the reference matters. */
#define RELUX_ATTN_FAST 0
#define RELUX_ATTN_REFERENCE 1
/* REFERENCE_FAITHFUL: the REFERENCE arithmetic with the reference's own indexing, for the small models on which greedy
 * token ids are compared with what relux itself emits.  Needs a pool created with RELUX_POOL_FLAG_REFERENCE_COMPAT.
 *   GQA: the cache is written chunk by chunk (one chunk per Append call, head-major inside the chunk:
 *        internal/transformer/kvcache.go:407-438) but read as one head-major [numKVHeads, T, headDim] array
 *        (mha.go:299-312): logical (kv head h, position j) reads stream row h*T + j.
 *   MLA: the decompressed keys / values are token-major [T, H, headDim] but indexed as head-major
 *        (mla.go:323-326 vs :348, 351): logical (head h, position j) reads token (h*T + j) / H, head (h*T + j) % H; the
 *        latent rows are read as float32, the reference's cache dtype (mla_cache.go:46-52).
 *   A causal mask is applied only when the call's q_tokens equal the cached length (mha.go:340, mla.go:368), and the
 *   layer-level calls give every row of a multi-token call on a non-empty cache the same RoPE position
 *   (rope.go:151-158).  extra_tokens must be 0. */
#define RELUX_ATTN_REFERENCE_FAITHFUL 2
/* relux_pool_params.flags */
#define RELUX_POOL_FLAG_REFERENCE_COMPAT 1   /* keep what RELUX_ATTN_REFERENCE_FAITHFUL needs: the chunk boundaries of every
                                                Append (GQA), a float32 copy of every appended row (MLA) */

typedef void* relux_device_t;
typedef void* relux_pool_t;
typedef void* relux_event_t;

/* ---- runtime ------------------------------------------------------------------------------
 * Replaces the backend discovery of internal/compute/factory.go:32-85 (NewComputeBackend) and the
 * Available()/DeviceInfo() methods of internal/compute/interface.go:13-41 for this path. */
int32_t relux_cuda_version(void);
int32_t relux_cuda_device_count(int32_t* count);
int32_t relux_cuda_device_open(int32_t device_index, relux_device_t* out);
int32_t relux_cuda_device_close(relux_device_t dev);
int32_t relux_cuda_sync(relux_device_t dev);
/* Copies the calling thread's last error message (NUL terminated) into buf.  The reference reports misuse by
 * panic(fmt.Sprintf(...)) (kvcache.go:241-249, 282-285; mla_cache.go:153-167); a C ABI cannot unwind through the
 * caller, so the same wording is fetched here after a non-zero status. */
int32_t relux_cuda_last_error(char* buf, int32_t buf_len);
/* Name, SM count, memory of the device (DeviceInfo() equivalent, interface.go:37-40). */
int32_t relux_cuda_device_info(relux_device_t dev, char* name, int32_t name_len, int32_t* sm_count,
                               int64_t* total_mem_bytes);
/* Number of kernels this library has launched on the handle since it was opened.  Measurement aid: no counterpart
 * in the reference. */
int32_t relux_cuda_launch_count(relux_device_t dev, int64_t* count);
/* The CUDA stream (cudaStream_t) all work of this handle is issued on, for callers that order their own device work
 * with it.  No counterpart in the reference. */
int32_t relux_cuda_stream(relux_device_t dev, void** stream);

/* ---- device memory ------------------------------------------------------------------------
 * Replaces internal/alloc/alloc.go:95-117,168-188,375-390 (alloc.Float32 / alloc.Uint16 / alloc.Free)
 * for buffers that must live on the GPU (weights, activations handed over as device pointers); host_alloc gives
 * page-locked host memory, like the reference's off-heap buffers "with stable addresses" (alloc.go:15-18). */
int32_t relux_cuda_dev_alloc(relux_device_t dev, size_t bytes, void** dptr);
int32_t relux_cuda_dev_free(relux_device_t dev, void* dptr);
int32_t relux_cuda_host_alloc(relux_device_t dev, size_t bytes, void** hptr);
int32_t relux_cuda_host_free(relux_device_t dev, void* hptr);
/* Host <-> device copies and fill; asynchronous on the handle's stream when the host side is pinned, ordered with
 * kernel calls.  No counterpart in the reference, whose buffers all live in host memory (alloc.go:15-18). */
int32_t relux_cuda_h2d(relux_device_t dev, void* dst_dev, const void* src_host, size_t bytes);
int32_t relux_cuda_d2h(relux_device_t dev, void* dst_host, const void* src_dev, size_t bytes);
int32_t relux_cuda_memset(relux_device_t dev, void* dst_dev, int32_t value, size_t bytes);

/* ---- timing helpers (CUDA events on the handle's stream) --------------------------------
 * Measurement aids: no counterpart in the reference. */
int32_t relux_cuda_event_create(relux_device_t dev, relux_event_t* ev);
int32_t relux_cuda_event_record(relux_device_t dev, relux_event_t ev);
int32_t relux_cuda_event_elapsed_ms(relux_device_t dev, relux_event_t start, relux_event_t stop, float* ms);
int32_t relux_cuda_event_destroy(relux_device_t dev, relux_event_t ev);
/* Overwrites a scratch buffer larger than L2 so the next kernel starts cold.  Measurement aid: no counterpart in
 * the reference. */
int32_t relux_cuda_flush_l2(relux_device_t dev);

/* ---- paged KV pools -----------------------------------------------------------------------
 * A pool replaces, on the device, both the cache objects and their backing arenas:
 *   GQA: KVCache / NewKVCacheSized   internal/transformer/kvcache.go:34-49, 66-93
 *   MLA: MLACache / NewMLACache      internal/transformer/mla_cache.go:21-59
 *   storage: internal/alloc/alloc.go:95-117,168-188 (64 MiB power-of-two freelist buckets)
 * Storage is bf16.  One pool serves num_layers layers and up to max_seqs sequences; a sequence
 * owns a page table of up to max_pages_per_seq physical page ids shared by all layers, and a
 * length per layer (the reference keeps one cursor per layer: kvcache.go:44-49).
 * MLA page  : [page_tokens][dC + dHR] (latent row followed by the rotated shared key).
 * GQA pages : K and V each [num_kv_heads][page_tokens][head_dim]. */
typedef struct relux_pool_params {
  int32_t kind;              /* RELUX_POOL_MLA | RELUX_POOL_GQA */
  int32_t num_layers;
  int32_t num_pages;         /* physical pages per layer */
  int32_t page_tokens;       /* tokens per page (64 enables the TMA/tensor-core kernels) */
  int32_t max_seqs;
  int32_t max_pages_per_seq;
  int32_t mla_dc;            /* MLA latent width (kv_lora_rank) */
  int32_t mla_dhr;           /* MLA decoupled RoPE key width */
  int32_t gqa_num_kv_heads;
  int32_t gqa_head_dim;
  int32_t flags;             /* RELUX_POOL_FLAG_* */
  int32_t reserved[5];       /* must be zero */
} relux_pool_params;

/* NewKVCacheSized (kvcache.go:66-93) / NewMLACache (mla_cache.go:38-59) for a whole batch of sequences; destroy
 * frees what the reference leaves to the garbage collector and alloc.Free. */
int32_t relux_pool_create(relux_device_t dev, const relux_pool_params* params, relux_pool_t* out);
int32_t relux_pool_destroy(relux_pool_t pool);
/* KVCache.Reset / MLACache.Reset (kvcache.go:174-202, mla_cache.go:118-133): every sequence length
 * becomes 0 and library-allocated sequences are released.  Page contents are left as they are. */
int32_t relux_pool_reset(relux_pool_t pool);
/* Caller-owned page tables: table is a host array [n_seqs][stride] of physical page ids, ctx_len a host
 * array [n_seqs] applied to every layer (NULL = 0).  Sequences 0..n_seqs-1 become live.  Ids are
 * validated on the host; a bad id is RELUX_ERR_BAD_PAGE.  No counterpart in the reference, whose caches are one
 * contiguous buffer per layer (kvcache.go:66-93): page tables are what the paged pool adds. */
int32_t relux_pool_set_tables(relux_pool_t pool, const int32_t* table, int32_t n_seqs, int32_t stride,
                              const int32_t* ctx_len);
/* Library-owned page tables: reserves pages for max_tokens tokens and returns a sequence id; per sequence what
 * NewKVCacheSized(numLayers, maxLen, ...) (kvcache.go:66-93) does for the reference's single sequence.  relux_seq_free
 * returns the pages (the reference: Reset + garbage collection, kvcache.go:174-202). */
int32_t relux_seq_alloc(relux_pool_t pool, int32_t max_tokens, int32_t* seq_id);
int32_t relux_seq_free(relux_pool_t pool, int32_t seq_id);
/* Grows a sequence created by relux_seq_alloc to hold max_tokens rows, taking the missing pages from the pool's free
 * list (never shrinks; cached rows stay where they are).  The reference's caches are sized once at construction
 * (NewKVCacheSized, kvcache.go:66-93); this is the paged pool's way to start small and grow. */
int32_t relux_seq_extend(relux_pool_t pool, int32_t seq_id, int32_t max_tokens);
/* KVCache.TotalLen / MLACache.TotalLen (kvcache.go:383-388, mla_cache.go:236-241). */
int32_t relux_seq_len(relux_pool_t pool, int32_t layer, int32_t seq_id, int32_t* len);
/* Sets the length of n_seqs sequences on one layer (layer < 0: on every layer).  Used to commit the accepted
 * prefix after a speculative verify, or to roll a sequence back.  seq_ids NULL = 0..n_seqs-1.  The reference has no
 * such call: its speculative decoder never removes rejected draft rows from the cache (speculative.go:136-156). */
int32_t relux_seq_set_len(relux_pool_t pool, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                          const int32_t* new_len);
/* Reads the device status word (0, or the first RELUX_ERR_BAD_PAGE / RELUX_ERR_TIMEOUT a kernel recorded)
 * and clears it.  Synchronises the stream.  No counterpart in the reference (its checks panic on the host). */
int32_t relux_pool_status(relux_pool_t pool, int32_t* status);
/* KVCache.View / MLACache.View equivalent used by the bit-exactness tests (kvcache.go:363-380,
 * mla_cache.go:222-233): copies n_tokens logical rows starting at token tok0 of one sequence to host memory
 * as bf16 bit patterns.  MLA: dst_a = latent rows [n][dC], dst_b = rope-key rows [n][dHR].
 * GQA: dst_a = K rows [n][Hkv][D], dst_b = V rows.  Either destination may be NULL.  Rows past the
 * sequence length are returned as stored (unspecified content). */
typedef struct relux_read_rows_args {
  int32_t layer;
  int32_t seq_id;
  int32_t tok0;
  int32_t n_tokens;
  void* dst_a;               /* host */
  void* dst_b;               /* host */
  int32_t reserved[4];
} relux_read_rows_args;
int32_t relux_pool_read_rows(relux_pool_t pool, const relux_read_rows_args* args);

/* Tuning knobs of relux_pool_tune. */
#define RELUX_TUNE_MLA_GENERIC 0        /* RELUX_MLA_GENERIC: 1 = MLA decode on the CUDA-core kernels                      */
#define RELUX_TUNE_MLA_WORKERS 1        /* RELUX_MLA_WORKERS: ranges the stream of pages is cut into (0 = resident pairs)   */
#define RELUX_TUNE_CHUNK_PAGES 2        /* RELUX_CHUNK_PAGES: chunk length of the split-KV planner (0 = chosen per call)    */
#define RELUX_TUNE_GEMM_GENERIC 3       /* RELUX_GEMM_GENERIC: 1 = projections on the plain kernel                          */
#define RELUX_TUNE_GEMM_SPLIT 4         /* RELUX_GEMM_SPLIT: split-K factor of the tcgen05 GEMM (0 = chosen per call)       */
#define RELUX_TUNE_GQA_PROMPT_PARTIAL_MB 5 /* RELUX_GQA_PROMPT_PARTIAL_MB: partial-buffer budget of a GQA prompt (256)      */
#define RELUX_TUNE_SEL_CLUSTER 6        /* RELUX_SEL_CLUSTER: cluster size of the selection kernel, 1/2/4/8 (0 = per call) */
#define RELUX_TUNE_SEL_LOOKAHEAD 7      /* RELUX_SEL_LOOKAHEAD: 0/1 (-1 = per call)                                         */
#define RELUX_TUNE_SEL_BATCHED 8        /* RELUX_SEL_BATCHED: 0/1 (-1 = per call)                                           */
#define RELUX_TUNE_GQA_PROMPT_SLICES 9  /* RELUX_GQA_PROMPT_SLICES: 1 = GQA prompts as grid slices of the decode kernel instead
                                           of the tcgen05 prefill kernel                                                  */
#define RELUX_TUNE_MLA_PROMPT_MIN_TOKENS 10 /* RELUX_MLA_PROMPT_MIN_TOKENS: query tokens per sequence from which an MLA call expands
                                           K / V and runs the tcgen05 prefill kernel (128; a huge value turns the path off) */
#define RELUX_TUNE_MLA_PROMPT_SCRATCH_MB 11 /* RELUX_MLA_PROMPT_SCRATCH_MB: most device memory the expanded K / V may take (16384) */
#define RELUX_TUNE_KERNEL_TIMING_STRIDE 12 /* RELUX_KERNEL_TIMING_STRIDE: the MLA decode kernel's event pair is recorded on every
                                           Nth call (1); the pairs are what relux_pool_kernel_ms_* read */
#define RELUX_TUNE_CHAINED_LAUNCHES 13 /* RELUX_CHAINED_LAUNCHES: 1 = the kernels of an MLA decode step are launched with
                                           programmatic stream serialization, so each is scheduled while the one before it
                                           still runs and waits on the device for its results (1); 0 = plain launches */
#define RELUX_TUNE_COUNT 14
/* Changes one tuning knob of a pool (see RELUX_TUNE_*).  A pool takes its defaults once, when it is created, from the
 * environment variables named beside the knobs; no call reads the environment afterwards.  value < 0 restores the
 * built-in default.  Tuning aid: no counterpart in the reference. */
int32_t relux_pool_tune(relux_pool_t pool, int32_t knob, int32_t value);

/* ---- call flags (relux_append_args.flags, relux_attn_args.flags) -----------------------------------
 * RELUX_CALL_PIPELINED: inputs and outputs that live in HOST memory travel on two copy streams of their own instead of
 * the handle's compute stream: inputs into one of two staging slots on the device, outputs from one of two result
 * slots, with events between the streams.  The call returns as soon as its work is queued, so the copies of the next
 * call overlap the kernels of this one.  Rules for the caller: pass page-locked buffers (relux_cuda_host_alloc) --
 * pageable ones make the copies synchronous --; leave an input buffer unchanged, and an output buffer unread, until
 * relux_pool_wait_output (or relux_cuda_sync) has returned for that call; give calls that may be in flight together
 * different output buffers.  relux_cuda_sync and relux_cuda_event_record cover the copy streams.  The reference has no
 * counterpart: its tensors never leave host memory (internal/alloc/alloc.go:15-18). */
#define RELUX_CALL_PIPELINED 1
/* Blocks until the host-memory output of a pipelined attention call has landed: calls_back = 0 the most recent such
 * call on this pool, 1 the one before it (two result slots exist; a third call in flight waits on the device for the
 * first one's copy).  No counterpart in the reference. */
int32_t relux_pool_wait_output(relux_pool_t pool, int32_t calls_back);

/* ---- append -------------------------------------------------------------------------------
 * MLACache.Append (mla_cache.go:152-182) fed by MLA.forwardCached step 4 (mla.go:309-312):
 * the latent c^KV and the already rotated shared key k^R of n_new[i] tokens per sequence.
 * KVCache.Append + copyInto (kvcache.go:240-291, 407-438) fed by MHA.forwardCached step 5
 * (mha.go:283-287): post-RoPE K and V.  float32 inputs are rounded with the reference's own
 * rule BF16FromF32 (dtype_convert.go:15-24); bf16 inputs are copied bit for bit.
 * Rows land at logical positions len .. len+n_new-1 of each sequence, i.e. the textbook per-head
 * placement (the reference's chunk-linear stream for Hkv > 1 is not reproduced). */
typedef struct relux_append_args {
  int32_t layer;
  int32_t n_seqs;
  const int32_t* seq_ids;   /* host [n_seqs]; NULL = 0..n_seqs-1 */
  const int32_t* n_new;     /* host [n_seqs]; NULL = 1 token each */
  const void* a;            /* MLA: c_kv [sum n_new][dC]     GQA: K */
  const void* b;            /* MLA: k_rope [sum n_new][dHR]  GQA: V */
  int32_t dtype;            /* RELUX_DTYPE_* of a and b */
  int32_t mem;              /* RELUX_MEM_* of a and b */
  int32_t layout;           /* GQA only: TOKEN_MAJOR [tok][Hkv][D] or HEAD_MAJOR [Hkv][n_new_i][D] per sequence */
  int32_t advance;          /* 1: lengths grow by n_new.  0: rows are written past the cursor, lengths unchanged
                               (draft rows of a speculative verify; commit with relux_seq_set_len) */
  int32_t flags;            /* RELUX_CALL_* */
  int32_t reserved[3];
} relux_append_args;
int32_t relux_mla_append(relux_pool_t pool, const relux_append_args* args);
int32_t relux_gqa_append(relux_pool_t pool, const relux_append_args* args);

/* ---- cached attention ---------------------------------------------------------------------
 * Each sequence attends over its first (len + extra_tokens) cached rows; its q_tokens query rows are the
 * LAST q_tokens of those rows.  causal != 0: query row i sees rows j <= T - q_tokens + i (causal inside
 * the new tokens); causal == 0: every query row sees all T rows (what the reference does for a
 * multi-token cached call, mha.go:340, mla.go:368).
 *
 * relux_mla_decode replaces MLA.forwardCached steps 5-6 (mla.go:317-377) in absorbed form:
 *   q~ = [W_UK_h q_nope | q_rope], scores over the latent rows, O_lat = P C, out = W_UV_h^T O_lat,
 * with w_uk / w_uv the reference's bf16 weight matrices [dC][H*head_dim] (mla.go:44-45) on the device.
 * relux_gqa_decode replaces MHA.forwardCached steps 6-8 (mha.go:292-348).  q_tokens > 1 with causal != 0
 * and extra_tokens = q_tokens is the verify step of SpeculativeDecoder.verifyPhase (speculative.go:189-207). */
typedef struct relux_attn_args {
  int32_t layer;
  int32_t n_seqs;
  const int32_t* seq_ids;   /* host [n_seqs]; NULL = 0..n_seqs-1 */
  int32_t q_tokens;
  int32_t extra_tokens;
  int32_t causal;
  int32_t num_heads;
  int32_t head_dim;         /* MLA: content (nope) and value head dim; GQA: must equal the pool's */
  float scale;              /* MLA 1/sqrt(head_dim + dHR) (mla.go:341), GQA 1/sqrt(head_dim) (mha.go:319) */
  const void* q;            /* MLA: q_nope [n][S][H][head_dim]; GQA: q [n][S][H][head_dim] (post-RoPE) */
  const void* q_rope;       /* MLA: [n][S][H][dHR] (post-RoPE); GQA: NULL */
  int32_t q_dtype, q_mem, q_layout;
  const void* w_uk;         /* MLA: device bf16 [dC][H*head_dim]; GQA: NULL */
  const void* w_uv;
  void* out;                /* [n][S][H][head_dim] */
  int32_t out_dtype, out_mem, out_layout;
  int32_t mode;             /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE | RELUX_ATTN_REFERENCE_FAITHFUL */
  int32_t flags;            /* RELUX_CALL_* */
  int32_t reserved[4];
} relux_attn_args;
int32_t relux_mla_decode(relux_pool_t pool, const relux_attn_args* args);
int32_t relux_gqa_decode(relux_pool_t pool, const relux_attn_args* args);

/* One decode step in one call: append the new rows (append->advance must be 1), then attend over the cache that now
 * includes them -- MLA.forwardCached steps 4-6 (mla.go:309-377), MHA.forwardCached steps 5-8 (mha.go:283-348).  Same
 * results as relux_*_append followed by relux_*_decode.  On the MLA tensor-core path the append and the stream partition
 * ride in the launch that absorbs W_UK into the queries (one kernel instead of three); other shapes and modes run the two
 * calls one after the other.  Both argument structs must name the same layer and sequences. */
int32_t relux_mla_step(relux_pool_t pool, const relux_append_args* append, const relux_attn_args* attn);
int32_t relux_gqa_step(relux_pool_t pool, const relux_append_args* append, const relux_attn_args* attn);

/* Speculative verify in one call (speculative.go:189-207 -> mha.go:245-369 with seqQ = k+1): writes the
 * q_tokens draft K/V rows of every sequence past its cursor (append with advance = 0), then attends with
 * extra_tokens = q_tokens.  Commit the accepted prefix with relux_seq_set_len afterwards. */
int32_t relux_gqa_verify(relux_pool_t pool, const relux_attn_args* attn, const relux_append_args* draft_kv);
int32_t relux_mla_verify(relux_pool_t pool, const relux_attn_args* attn, const relux_append_args* draft_kv);

/* One MLA attention layer step, device-resident end to end: MLA.forwardCached (mla.go:272-397) for a batch of
 * independent sequences.  x [n_seqs][q_tokens][d_model] float32 (host or device) is projected with the reference's
 * bf16 weight matrices (row-major [in][out] exactly as optim.Param.Data holds them, mla.go:41-47, on the device):
 *   q^C = x W_Q, q^R = x W_QR, c^KV = x W_DKV, k^R = x W_KR                      (mla.go:285-288)
 * q^R and k^R are rotated with the decoupled RoPE of NewMLA (mla.go:83, tables built as rope.go:59-68) at position
 * cached_len + s for the s-th new token of a sequence, (c^KV, k^R) are appended to this pool's layer `layer`
 * (cursors advance by q_tokens), the absorbed attention runs over the cache with scale 1/sqrt(head_dim + dHR)
 * (mla.go:344-345; causal != 0 masks inside the q_tokens new rows), and out = o W_O [n_seqs][q_tokens][d_model]
 * float32 (host or device).  head_dim = d_model / num_heads like NewMLA; dC and dHR are the pool's.
 * RELUX_ATTN_FAST runs the projections on the tensor cores with x rounded to bf16; RELUX_ATTN_REFERENCE runs every
 * step in the reference's float32 operation order.  Errors: RELUX_ERR_OVERFLOW when a sequence would pass its
 * capacity (the reference panics, mla_cache.go:160-164) or a position passes the RoPE table (rope.go:160-162). */
typedef struct relux_mla_layer_weights {
  const void* w_q;    /* device bf16 [d_model][num_heads*head_dim] */
  const void* w_qr;   /* device bf16 [d_model][num_heads*dHR] */
  const void* w_dkv;  /* device bf16 [d_model][dC] */
  const void* w_kr;   /* device bf16 [d_model][dHR] */
  const void* w_uk;   /* device bf16 [dC][num_heads*head_dim] */
  const void* w_uv;   /* device bf16 [dC][num_heads*head_dim] */
  const void* w_o;    /* device bf16 [num_heads*head_dim][d_model] */
} relux_mla_layer_weights;
typedef struct relux_mla_layer_args {
  int32_t layer;
  int32_t n_seqs;
  const int32_t* seq_ids;   /* host [n_seqs]; NULL = 0..n_seqs-1 */
  int32_t q_tokens;         /* new tokens per sequence (1 for decode) */
  int32_t causal;
  int32_t d_model;
  int32_t num_heads;
  float rope_base;          /* 0 = 10000 like NewMLA (mla.go:78-80) */
  int32_t mode;             /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE */
  const void* x;
  int32_t x_dtype, x_mem;   /* RELUX_DTYPE_F32; RELUX_MEM_HOST | RELUX_MEM_DEVICE */
  void* out;
  int32_t out_mem;
  int32_t reserved[3];
  const relux_mla_layer_weights* w;
} relux_mla_layer_args;
int32_t relux_mla_forward_cached(relux_pool_t pool, const relux_mla_layer_args* args);

/* One GQA attention layer step, device-resident end to end: MHA.forwardCached (mha.go:245-369) for a batch of
 * independent sequences.  x [n_seqs][q_tokens][d_model] float32 is projected with Wq [d_model][num_heads*head_dim],
 * Wk and Wv [d_model][num_kv_heads*head_dim] (mha.go:251-258; bf16, row-major [in][out], on the device); with
 * rope != 0 q and k are rotated at position cached_len + s (mha.go:272-282, tables as rope.go:59-68); k / v are
 * written to this pool's layer (advance != 0: cursors move by q_tokens, decode / prefill; advance = 0: the rows stay
 * past the cursor, the speculative verify step, commit the accepted prefix with relux_seq_set_len); attention with
 * scale 1/sqrt(head_dim) (mha.go:319), causal inside the q_tokens new rows; out = o Wo [n_seqs][q_tokens][d_model]
 * float32.  head_dim = d_model / num_heads must equal the pool's, num_kv_heads is the pool's. */
typedef struct relux_gqa_layer_weights {
  const void* w_q;   /* device bf16 [d_model][num_heads*head_dim] */
  const void* w_k;   /* device bf16 [d_model][num_kv_heads*head_dim] */
  const void* w_v;   /* device bf16 [d_model][num_kv_heads*head_dim] */
  const void* w_o;   /* device bf16 [num_heads*head_dim][d_model] */
} relux_gqa_layer_weights;
typedef struct relux_gqa_layer_args {
  int32_t layer;
  int32_t n_seqs;
  const int32_t* seq_ids;   /* host [n_seqs]; NULL = 0..n_seqs-1 */
  int32_t q_tokens;
  int32_t causal;
  int32_t d_model;
  int32_t num_heads;
  int32_t rope;             /* 0: the layer has no rotary embedding (m.rope == nil) */
  float rope_base;          /* 0 = 10000 */
  int32_t advance;
  int32_t mode;             /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE */
  const void* x;
  int32_t x_dtype, x_mem;
  void* out;
  int32_t out_mem;
  int32_t reserved[3];
  const relux_gqa_layer_weights* w;
} relux_gqa_layer_args;
int32_t relux_gqa_forward_cached(relux_pool_t pool, const relux_gqa_layer_args* args);

/* ---- token selection after a verify pass -----------------------------------------------------
 * relux_spec_accept replaces SpeculativeDecoder.acceptPhase with resampleRejected (speculative.go:211-295; softmaxAlloc
 * :346-368) for a batch of independent sequences, and the Sampler.Sample call it ends with when every draft token was
 * accepted (internal/transformer/sampler.go:73-218: temperature, top-k, nucleus, min-p, categorical draw; the
 * repetition penalties, which acceptPhase never uses, are left out).  The reference takes its uniform numbers from a
 * math/rand stream; here the caller supplies them: draws [n_seqs][k + 1], consumed per sequence in the reference's
 * order (one per examined draft token, then one for the resample or for the final sample).
 *   draft_tokens [n_seqs][k], draft_logits [n_seqs][k][vocab], target_logits [n_seqs][k + 1][vocab] (row i judges
 *   draft token i, row k gives the bonus token), all float32 / int32, in host or device memory (mem).
 *   n_accepted [n_seqs] and next_token [n_seqs] are written to HOST memory; the call synchronises the stream.
 * k = 0 is plain Sampler.Sample on target_logits [n_seqs][vocab] with draws [n_seqs] (n_accepted may be NULL).
 * commit != 0: afterwards every layer's length of sequence seq_ids[i] grows by n_accepted[i] + 1 -- the rows of the
 * token fed first and of the accepted draft tokens that a relux_*_verify call wrote past the cursor become part of
 * the sequence (the reference's startPos += nAccepted + 1, speculative.go:155).
 * RELUX_ATTN_FAST: one thread-block cluster per sequence, parallel float32 sums -- a decision can differ from the
 * reference's only when a draw lies within rounding distance of a boundary.  RELUX_ATTN_REFERENCE: the reference's
 * sequential float32 order, bit-exact, one thread per sequence (meant for parity checks: with the nucleus filter on it
 * is quadratic in the vocabulary like the reference's selection sort, and returns RELUX_ERR_UNSUPPORTED above 32768).
 * Errors: RELUX_ERR_INVALID_ARG for a draft token outside [0, vocab) (the reference would panic on the index). */
typedef struct relux_sampler_params {
  float temperature;        /* <= 0 is replaced by 1e-5 (sampler.go:90-93) */
  int32_t top_k;            /* <= 0 or >= vocab: off */
  float top_p;              /* <= 0 or >= 1: off */
  float min_p;              /* <= 0: off */
} relux_sampler_params;
typedef struct relux_spec_accept_args {
  int32_t n_seqs;
  int32_t k;
  int32_t vocab;
  int32_t mem;              /* RELUX_MEM_* of draft_tokens, draft_logits, target_logits and draws */
  const int32_t* draft_tokens;
  const float* draft_logits;
  const float* target_logits;
  const float* draws;
  relux_sampler_params sampler;
  int32_t mode;             /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE */
  int32_t commit;
  const int32_t* seq_ids;   /* host [n_seqs]; NULL = 0..n_seqs-1; only read when commit != 0 */
  int32_t* n_accepted;      /* host [n_seqs], out */
  int32_t* next_token;      /* host [n_seqs], out */
  int32_t reserved[4];
} relux_spec_accept_args;
int32_t relux_spec_accept(relux_pool_t pool, const relux_spec_accept_args* args);

/* Sampler.Sample (internal/transformer/sampler.go:73-218) for a batch of rows, repetition control included: the
 * logits of the tokens in a row's window of previous tokens are rewritten first (applyRepetitionPenalties,
 * sampler.go:221-266: repeat penalty -- divide a positive logit, multiply a negative one --, frequency penalty times
 * the count in the window, presence penalty; each once per distinct token; tokens outside [0, vocab) are ignored),
 * then temperature, top-k, softmax, nucleus, min-p and the categorical draw run as in relux_spec_accept with k = 0.
 * This is the call Transformer.Generate makes per step (transformer.go:955-962) and draftPhase per draft token
 * (speculative.go:178).  logits [n_rows][vocab] float32 and draws [n_rows] (the reference's rng.Float32() per call) in
 * host or device memory; prev_tokens host int32 [n_rows][prev_stride] with prev_len [n_rows] valid entries per row
 * (NULL: previousTokens == nil); repeat_window 0 = all previous tokens.  tokens [n_rows] is written to HOST memory;
 * the call synchronises the stream.  The input logits are never modified (the reference works on a copy too). */
typedef struct relux_sample_args {
  int32_t n_rows;
  int32_t vocab;
  int32_t mem;               /* RELUX_MEM_* of logits and draws */
  int32_t mode;              /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE */
  const float* logits;
  const float* draws;
  relux_sampler_params sampler;
  float repeat_penalty;      /* 0 or 1: off (sampler.go:246) */
  float frequency_penalty;
  float presence_penalty;
  int32_t repeat_window;
  const int32_t* prev_tokens;
  const int32_t* prev_len;
  int32_t prev_stride;
  int32_t reserved[3];
  int32_t* tokens;           /* host [n_rows], out */
} relux_sample_args;
int32_t relux_sampler_sample(relux_pool_t pool, const relux_sample_args* args);

/* GQA flash-decode / verify that allocates nothing.  It has no counterpart in the reference; it exists for callers
 * that may not allocate device memory at the moment they decode: a serving loop whose memory budget has been handed
 * out completely (so a late cudaMalloc can fail or stall the whole device while it synchronises), or code running
 * under rules that forbid allocator calls after start-up.  relux_gqa_decode grows its split-KV scratch with
 * cudaMalloc when a call needs more than any earlier one; this entry point never does.  Its work list and split-KV
 * partials live in one fixed 16 MiB array in device memory that every GPU holds from the moment the library is
 * loaded until the process exits.
 *   - Same arguments and results as relux_gqa_decode, restricted to what needs no staging: RELUX_ATTN_FAST, q and
 *     out in device memory, q token-major f32 or bf16, out token-major f32, page_tokens 64, head_dim 128,
 *     (num_heads / num_kv_heads) * q_tokens <= 32.
 *   - Limits of the fixed scratch: at most 4096 sequences per call, at most 4096 (sequence, chunk) work items, and
 *     work_items * q_tokens * num_heads * 520 bytes of partials within 16 MiB minus a 96 KiB header.  Chunks are
 *     lengthened to fit; a call that cannot fit even with one chunk per sequence returns RELUX_ERR_UNSUPPORTED and
 *     its message names the limit.
 *   - The first call on a device looks up the array's device address (one cudaGetSymbolAddress, checked); make that
 *     first call before starting any stream capture.  No call uses cudaMalloc, cudaFree or another allocating routine.
 *   - All calls share the array and it keeps whatever the last call left in it; nothing in it has to start at zero.
 *     Two calls whose kernels overlap on the GPU (different pools on different streams, or different processes'
 *     copies aside) would overwrite each other's partials: run calls of this entry point one after another. */
int32_t relux_gqa_decode_noalloc(relux_pool_t pool, const relux_attn_args* args);

/* One sequence's cache as a file in the layout of the reference's file-backed caches: NewKVCacheFile
 * (kvcache.go:104-166: per layer K [1, numKVHeads, maxLen, headDim] then V, bf16) or NewMLACacheFile
 * (mla_cache.go:63-113: per layer C_KV [1, maxLen, dC] then K_R [1, maxLen, dHR], float32).  Rows past a layer's
 * length are zeros.  Like the reference's files these hold no lengths: relux_seq_load_file takes the per-layer lengths
 * (host [num_layers]) from the caller, resets the sequence and appends the rows (MLA rows are rounded to bf16 with the
 * reference's rule).  max_len is the maxLen the file was / is to be made with (>= every layer's length). */
int32_t relux_seq_save_file(relux_pool_t pool, int32_t seq_id, const char* path, int32_t max_len);
int32_t relux_seq_load_file(relux_pool_t pool, int32_t seq_id, const char* path, int32_t max_len, const int32_t* layer_len);

/* The stream partition the persistent MLA decode kernel works on, computed on the host from page counts (no device
 * needed): the pages of all sequences, laid end to end, are cut into ranges of *range_pages_out pages (a multiple of
 * page_multiple), one range per worker; an item is the part of one sequence inside one range.
 * items_out: n x {seq_index, page_begin, page_end, worker} (cap items of room), worker_first [*workers_out + 1],
 * chunk_off [n_seqs + 1]; any of the three may be NULL.  Returns the number of items, -1 on bad arguments or when cap
 * is too small.  Scheduling aid: no counterpart in the reference. */
typedef struct relux_stream_partition_args {
  const int32_t* pages;      /* [n_seqs] pages per sequence */
  int32_t n_seqs;
  int32_t workers;
  int32_t page_multiple;
  int32_t cap;               /* room in items_out, in items */
  int32_t* range_pages_out;
  int32_t* workers_out;
  int32_t* items_out;
  int32_t* worker_first;
  int32_t* chunk_off;
} relux_stream_partition_args;
int32_t relux_stream_partition(const relux_stream_partition_args* args);

/* Device-time of the dominant attention kernel of the most recent relux_*_decode / verify call on this
 * pool, measured with CUDA events around that one launch.  Synchronises the stream.  Measurement aid: no counterpart
 * in the reference. */
int32_t relux_pool_last_kernel_ms(relux_pool_t pool, float* ms);

/* Mean device time of that kernel over the most recent `last_n` decode / verify calls on this pool (at most
 * 8192 are kept); `counted` receives how many calls went into the mean.  The event pairs are recorded by the
 * calls themselves, so reading them after a timed loop does not disturb the loop.  Synchronises the stream.
 * Measurement aid: no counterpart in the reference. */
int32_t relux_pool_kernel_ms_mean(relux_pool_t pool, int32_t last_n, float* mean_ms, int32_t* counted);
/* The same times one by one: ms_out [last_n] receives the device time of each of the most recent calls, oldest first;
 * `counted` how many were written.  Measurement aid: no counterpart in the reference. */
int32_t relux_pool_kernel_ms_list(relux_pool_t pool, int32_t last_n, float* ms_out, int32_t* counted);

/* Same for the input-projection launch (x . [W_Q | W_QR | W_DKV | W_KR]) of the most recent
 * relux_mla_forward_cached calls on this pool.  Measurement aid: no counterpart in the reference. */
int32_t relux_pool_projection_ms_mean(relux_pool_t pool, int32_t last_n, float* mean_ms, int32_t* counted);

/* ---- the matmul of the compute backend ---------------------------------------------------------
 * ComputeBackend.MatMulFloat32 (internal/compute/interface.go:25-29) as matmulBatched3D calls it for every projection
 * (internal/transformer/mha.go:759-785 -> nativeBackend.MatMulFloat32, internal/compute/native.go:175-187):
 *   C [M][N] float32 = A [M][K] float32 x B [K][N] bf16 (row-major, the layout of optim.Param.Data).
 * A and C in host or device memory, B on the device (weights are uploaded once).
 * RELUX_ATTN_FAST: A rounded to bf16, tcgen05 tensor-core GEMM with split-K (needs K and N multiples of 8);
 * RELUX_ATTN_REFERENCE: one k-ascending chain of unfused float32 multiply-then-add per output, the order of
 * internal/transformer/matmul.go:15-27 -- bit-identical to the reference.
 * An error is an error: the reference's caller falls back to Go when the backend fails (mha.go:768-772); this library has
 * no fallback, the binding must surface the status. */
typedef struct relux_matmul_args {
  int32_t m, k, n;
  int32_t mode;              /* RELUX_ATTN_FAST | RELUX_ATTN_REFERENCE */
  const float* a;
  int32_t a_mem;
  int32_t c_mem;
  const void* b;             /* device bf16 [k][n] */
  float* c;
  int32_t reserved[4];
} relux_matmul_args;
int32_t relux_matmul_f32_bf16(relux_pool_t pool, const relux_matmul_args* args);

/* ---- expansion of the cached MLA latents --------------------------------------------------------
 * What MLA.forwardCached does before it scores a multi-token call: every cached latent row times W_UK and W_UV
 * (internal/transformer/mla.go:323-326), here as one tensor-core GEMM with bf16 results.  The library's own prompt path
 * (relux_mla_decode with 128 or more query tokens) runs it into an internal scratch array; this entry point runs it
 * into the caller's memory.
 *   kv_out     device bf16 [2 * num_heads][rows_total][128]: keys of head h at block h, values at block num_heads + h;
 *              row = seq_base[i] + token for the i-th named sequence
 *   seq_base   device int32 [n_seqs + 1], written by the call: first row of every sequence (lengths rounded up to 256;
 *              rows past a sequence's end hold values computed from whatever its last page holds)
 *   rows_total as returned by a first call with kv_out == NULL (host value; nothing is launched then)
 * Shapes: latent 512, 64-token pages, head width 128, FAST arithmetic; other pools get RELUX_ERR_UNSUPPORTED. */
typedef struct relux_mla_expand_args {
  int32_t layer, n_seqs;
  const int32_t* seq_ids;      /* host, or NULL = 0..n_seqs-1 */
  int32_t extra_tokens, num_heads;
  const void* w_uk;            /* device bf16 [dC][num_heads * 128] */
  const void* w_uv;            /* device bf16 [dC][num_heads * 128] */
  void* kv_out;                /* device, or NULL to ask for rows_total only */
  int32_t* seq_base;           /* device */
  int64_t rows_total;          /* in (when kv_out != NULL) */
  int64_t* rows_total_out;     /* host, may be NULL */
  int32_t reserved[4];
} relux_mla_expand_args;
int32_t relux_mla_expand_kv(relux_pool_t pool, const relux_mla_expand_args* args);

/* ---- weight import -------------------------------------------------------------------------------
 * Brings the attention weights of one MLA layer from checkpoint layout into the device layout the layer calls take.
 * The reference's DeepSeek mapper names the checkpoint tensors (internal/loader/mapper.go:139-180): q_proj -> mla.W_Q,
 * kv_a_proj_with_mqa -> mla.W_DKV, kv_b_proj -> the fused "mla.W_UK_W_UV", o_proj -> mla.W_O, every one with
 * Transpose: true (checkpoints store [out][in], relux holds [in][out]); its loader converts each tensor to bf16 with
 * BF16FromF32 (loader.go:239-281, 394-404) and has a slot for the separate matrices only (loader.go:322-338): the fused
 * kind is named but never split.  This call does the split and the transposes on the device:
 *   kv_b_proj [H * (nope + v)][dC], per head nope rows then v rows (the shape rule of mapper.go:146-152)
 *                                                      -> w_uk [dC][H * nope], w_uv [dC][H * v]
 *   o_proj [d_model][H * v]                            -> w_o [H * v][d_model]
 *   fused_rope == 0, the tensors the reference's mapper names (mapper.go:139-180):
 *     q_proj [H * nope][d_model] -> w_q;  q_pe_proj [H * rope][d_model] -> w_qr;
 *     kv_a_proj_with_mqa [dC][d_model] -> w_dkv;  k_pe_proj [rope][d_model] -> w_kr
 *   fused_rope != 0, the layout of published DeepSeek-V2 checkpoints (the rope rows ride inside the two tensors):
 *     q_proj [H * (nope + rope)][d_model], per head nope rows then rope rows -> w_q, w_qr
 *     kv_a_proj_with_mqa [dC + rope][d_model], latent rows then the shared rope-key rows -> w_dkv, w_kr
 * Sources are float32 or bf16 in host or device memory (src_dtype, src_mem); destinations are device bf16 buffers of the
 * caller, the seven pointers of relux_mla_layer_weights.  A NULL source skips its destinations.  float32 values are
 * rounded with the reference's rule (dtype_convert.go:15-24); bf16 values are moved bit for bit. */
typedef struct relux_mla_import_args {
  int32_t d_model, num_heads, nope_dim, rope_dim, v_dim, dc;
  int32_t src_dtype, src_mem;
  int32_t fused_rope;
  int32_t reserved[3];
  const void* q_proj;
  const void* kv_a_proj_with_mqa;
  const void* kv_b_proj;
  const void* o_proj;
  const void* q_pe_proj;                /* fused_rope == 0 only */
  const void* k_pe_proj;                /* fused_rope == 0 only */
  const relux_mla_layer_weights* dst;   /* device buffers */
} relux_mla_import_args;
int32_t relux_mla_import_weights(relux_pool_t pool, const relux_mla_import_args* args);

/* Test aid for the bounded waits of the kernels: launches one warp that waits, through the same bounded mbarrier wait
 * the attention kernels use, on a barrier nobody arrives at, with a poll limit of `polls`.  The wait gives up, the kernel
 * records RELUX_ERR_TIMEOUT in the pool's status word and returns; relux_pool_status then reports it.  Nothing hangs and
 * nothing faults.  No counterpart in the reference. */
int32_t relux_pool_selftest_wait(relux_pool_t pool, int32_t polls);

#ifdef __cplusplus
}
#endif
#endif /* RELUX_CUDA_H_ */
