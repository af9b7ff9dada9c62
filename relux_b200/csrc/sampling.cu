// Token selection after a speculative verify pass, on the device: SpeculativeDecoder.acceptPhase and
// resampleRejected (speculative.go:211-295, softmaxAlloc :346-368) and Sampler.Sample without the repetition
// penalties (internal/transformer/sampler.go:73-218).  The uniform draws the reference takes from math/rand are
// arguments, consumed in the reference's order.
//
// FAST: one thread-block cluster per sequence.  The CTAs of a cluster split the vocabulary into contiguous slices;
// every step of the reference's chain (row maximum, sum of exponentials, the top-k threshold, the nucleus cut, the
// inverse-CDF search) is one pass over the row out of L2 with a reduction across the cluster through distributed shared
// memory, so a row is read from HBM once however many passes follow.  Exponentials use the reference's fastexp32 bit
// trick, which makes the distribution the reference's own; what differs is the order of the float32 sums (parallel
// instead of sequential), so a decision can only differ when a draw falls within rounding distance of a boundary.
// REFERENCE: one thread per sequence walks the reference's loops in the reference's order (bit-exact, slow).
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include <cstdint>
#include <cstdlib>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace cg = cooperative_groups;

namespace relux {

int32_t stage_in(Pool* p, GrowBuf& buf, const void* src, size_t bytes, int mem, const void** dptr);   // runtime.cu

namespace {

constexpr int kSelThreads = 512;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kMaxCluster = 8;
constexpr int kStatMax = 16;     // batched statistics: two rows for each of up to 8 draft positions

struct SelParams {
  const int32_t* draft_tokens;   // [n][k] or nullptr (plain sampling)
  const float* draft_logits;     // [n][k][V]
  const float* target_logits;    // [n][k+1][V]; plain sampling: [n][V] with k = 0
  const float* draws;            // [n][k+1]
  int32_t* n_accepted;           // [n]
  int32_t* next_token;           // [n]
  int32_t* status;
  int32_t k, vocab;
  float temperature;
  int32_t top_k;
  float top_p, min_p;
  int32_t lookahead;             // accept loop: take the next position's maxima in the pass that sums this one's
  int32_t batched;               // accept loop: maxima of all positions' rows in one stage, all sums in a second
};

// Shared memory of one CTA: exchange slots read by the other CTAs of the cluster.
struct SelShared {
  float red[2][4];            // double-buffered per-CTA partials of a cluster reduction (up to 4 values)
  float warp_part[kSelWarps][4];
  float hist_sum[256];
  uint32_t hist_cnt[256];
  float warp_seg[kSelWarps];  // per-warp segment sums of the search pass
  uint32_t warp_hist[kSelWarps][256];   // radix selection: one histogram per warp (counts, or float sums)
  uint32_t list_count;        // candidate list of the small-top-k path (the list itself reuses warp_hist)
  float red_n[2][kStatMax];   // cluster_reduce_n: per-CTA partials, double-buffered like red
  float warp_part_n[kSelWarps][kStatMax];
  float stat[2][kStatMax];    // [0] maxima, [1] sums of exponentials of all draft positions' rows (batched statistics)
};

__device__ __forceinline__ uint32_t order_key(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Everything the passes need to evaluate the reference's probability of one logit on the fly.
struct Dist {
  float temp;        // 1 = untouched
  uint32_t topk_key; // elements whose key is below are masked (0 = nothing masked)
  float m, inv1;     // maximum and 1 / sum of exponentials
  float tau, inv2;   // nucleus: probabilities below tau are dropped, the rest scaled by inv2
  float minp_thr, inv3;
  __device__ __forceinline__ float scaled(float v) const { return temp == 1.0f ? v : __fdiv_rn(v, temp); }
  __device__ __forceinline__ float p1(float v) const {
    float x = scaled(v);
    if (order_key(x) < topk_key) return 0.0f;
    return __fmul_rn(fastexp32_ref(__fsub_rn(x, m)), inv1);
  }
};

struct Ctx {
  SelShared* sh;
  int rank, csize;     // CTA rank in the cluster, cluster size
  int lo, hi;          // this CTA's slice of the vocabulary
  int wlo, whi;        // this warp's contiguous segment of the slice
  int warp, lane;
  bool vec;            // rows can be read as aligned float4s
  uint32_t round;      // reduction counter (selects the exchange buffer)
};

// Sum or maximum of up to four per-thread values over the whole cluster; every thread of every CTA gets the same result,
// combined in CTA order.  kMode 0: four sums; 1: four maxima; 2: values 0-1 summed, values 2-3 maximised (one barrier
// for the sums of one row pair and the maxima of the next).  One cluster barrier per call: the two exchange buffers
// alternate.
template <int kMode>
__device__ void cluster_reduce4(Ctx& c, float (&v)[4]) {
  cg::cluster_group cl = cg::this_cluster();
  auto is_max = [](int j) { return kMode == 1 || (kMode == 2 && j >= 2); };
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] = is_max(j) ? warp_max(v[j]) : warp_sum(v[j]);
  if (c.lane == 0) {
#pragma unroll
    for (int j = 0; j < 4; j++) c.sh->warp_part[c.warp][j] = v[j];
  }
  __syncthreads();
  const int buf = c.round & 1;
  if (threadIdx.x < 4) {
    const bool mx = is_max((int)threadIdx.x);
    float a = c.sh->warp_part[0][threadIdx.x];
    for (int w = 1; w < kSelWarps; w++) a = mx ? fmaxf(a, c.sh->warp_part[w][threadIdx.x]) : a + c.sh->warp_part[w][threadIdx.x];
    c.sh->red[buf][threadIdx.x] = a;
  }
  cl.sync();
#pragma unroll
  for (int j = 0; j < 4; j++) {
    float a = is_max(j) ? -INFINITY : 0.0f;
    for (int r = 0; r < c.csize; r++) {
      const float* remote = cl.map_shared_rank(&c.sh->red[buf][j], r);
      a = is_max(j) ? fmaxf(a, *remote) : a + *remote;
    }
    v[j] = a;
  }
  c.round++;
}

// The same for `count` <= kStatMax values per thread (acc[]); the results land in dst[] in this CTA's shared memory.
template <bool kMax>
__device__ void cluster_reduce_n(Ctx& c, const float* acc, int count, float* dst) {
  cg::cluster_group cl = cg::this_cluster();
  for (int j = 0; j < count; j++) {
    const float r = kMax ? warp_max(acc[j]) : warp_sum(acc[j]);
    if (c.lane == 0) c.sh->warp_part_n[c.warp][j] = r;
  }
  __syncthreads();
  const int buf = c.round & 1;
  if ((int)threadIdx.x < count) {
    float a = c.sh->warp_part_n[0][threadIdx.x];
    for (int w = 1; w < kSelWarps; w++) a = kMax ? fmaxf(a, c.sh->warp_part_n[w][threadIdx.x]) : a + c.sh->warp_part_n[w][threadIdx.x];
    c.sh->red_n[buf][threadIdx.x] = a;
  }
  cl.sync();
  if ((int)threadIdx.x < count) {
    float a = kMax ? -INFINITY : 0.0f;
    for (int r = 0; r < c.csize; r++) {
      const float x = *cl.map_shared_rank(&c.sh->red_n[buf][threadIdx.x], r);
      a = kMax ? fmaxf(a, x) : a + x;
    }
    dst[threadIdx.x] = a;
  }
  __syncthreads();
  c.round++;
}

// Every CTA learns every CTA's value (in rank order), through the same exchange buffers as cluster_reduce4.
__device__ void cluster_gather1(Ctx& c, float mine, float (&all)[kMaxCluster]) {
  cg::cluster_group cl = cg::this_cluster();
  const int buf = c.round & 1;
  if (threadIdx.x == 0) c.sh->red[buf][0] = mine;
  cl.sync();
#pragma unroll
  for (int r = 0; r < kMaxCluster; r++) all[r] = r < c.csize ? *cl.map_shared_rank(&c.sh->red[buf][0], r) : 0.0f;
  c.round++;
}

// Calls f(index, value) for every element of this warp's segment of `row`.  Segments start on multiples of 128
// elements, so when the vocabulary is a multiple of four and the rows are 16-byte aligned (c.vec) every lane reads
// float4s, four in flight; otherwise lanes interleave single floats.
template <class F>
__device__ __forceinline__ void for_segment(const Ctx& c, const float* __restrict__ row, F f) {
  if (c.vec) {
    int i = c.wlo + c.lane * 4;
    for (; i + 896 < c.whi; i += 1024) {   // eight float4 loads in flight per lane
      float4 t[8];
#pragma unroll
      for (int q = 0; q < 8; q++) t[q] = __ldg(reinterpret_cast<const float4*>(row + i + 128 * q));
#pragma unroll
      for (int q = 0; q < 8; q++) { f(i + 128 * q, t[q].x); f(i + 128 * q + 1, t[q].y); f(i + 128 * q + 2, t[q].z); f(i + 128 * q + 3, t[q].w); }
    }
    for (; i + 384 < c.whi; i += 512) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(row + i));
      const float4 b = __ldg(reinterpret_cast<const float4*>(row + i + 128));
      const float4 d = __ldg(reinterpret_cast<const float4*>(row + i + 256));
      const float4 e = __ldg(reinterpret_cast<const float4*>(row + i + 384));
      f(i, a.x); f(i + 1, a.y); f(i + 2, a.z); f(i + 3, a.w);
      f(i + 128, b.x); f(i + 129, b.y); f(i + 130, b.z); f(i + 131, b.w);
      f(i + 256, d.x); f(i + 257, d.y); f(i + 258, d.z); f(i + 259, d.w);
      f(i + 384, e.x); f(i + 385, e.y); f(i + 386, e.z); f(i + 387, e.w);
    }
    for (; i < c.whi; i += 128) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(row + i));
      f(i, a.x); f(i + 1, a.y); f(i + 2, a.z); f(i + 3, a.w);
    }
    return;
  }
  int i = c.wlo + c.lane;
  for (; i + 96 < c.whi; i += 128) {
    float a = __ldg(row + i), b = __ldg(row + i + 32), d = __ldg(row + i + 64), e = __ldg(row + i + 96);
    f(i, a); f(i + 32, b); f(i + 64, d); f(i + 96, e);
  }
  for (; i < c.whi; i += 32) f(i, __ldg(row + i));
}

// The same over two rows at once: f(index, value_a, value_b).
template <class F>
__device__ __forceinline__ void for_segment2(const Ctx& c, const float* __restrict__ ra, const float* __restrict__ rb, F f) {
  if (c.vec) {
    int i = c.wlo + c.lane * 4;
    for (; i + 384 < c.whi; i += 512) {   // four float4 loads per row in flight per lane
      float4 ta[4], tb[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        ta[q] = __ldg(reinterpret_cast<const float4*>(ra + i + 128 * q));
        tb[q] = __ldg(reinterpret_cast<const float4*>(rb + i + 128 * q));
      }
#pragma unroll
      for (int q = 0; q < 4; q++) {
        f(i + 128 * q, ta[q].x, tb[q].x); f(i + 128 * q + 1, ta[q].y, tb[q].y);
        f(i + 128 * q + 2, ta[q].z, tb[q].z); f(i + 128 * q + 3, ta[q].w, tb[q].w);
      }
    }
    for (; i < c.whi; i += 128) {
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(ra + i)), b0 = __ldg(reinterpret_cast<const float4*>(rb + i));
      f(i, a0.x, b0.x); f(i + 1, a0.y, b0.y); f(i + 2, a0.z, b0.z); f(i + 3, a0.w, b0.w);
    }
    return;
  }
  int i = c.wlo + c.lane;
  for (; i + 32 < c.whi; i += 64) {
    float a0 = __ldg(ra + i), b0 = __ldg(rb + i), a1 = __ldg(ra + i + 32), b1 = __ldg(rb + i + 32);
    f(i, a0, b0); f(i + 32, a1, b1);
  }
  for (; i < c.whi; i += 32) f(i, __ldg(ra + i), __ldg(rb + i));
}

// Radix selection, eight bits a round, over keys that order like the values.  kWeighted = false: the key of the
// `want`-th largest element (Sampler's kthLargest, sampler.go:283-300).  kWeighted = true: keys are probabilities and
// the walk stops at the largest probability tau for which the sum of all probabilities >= tau reaches `want_sum` (the
// nucleus cut of sampler.go:148-160; elements tied with tau are all kept).  Returns false when the total never
// reaches want_sum.
// stop_at (counting walk only): as soon as no more than stop_at elements have a key >= the lower bound of the chosen
// bin, the walk ends early; *key_out is then that lower bound and *n_ge_out the number of elements at or above it (a
// superset of the `want` largest that is small enough to finish on a list).
template <bool kWeighted, class KeyF>
__device__ bool radix_select(Ctx& c, const float* __restrict__ row, KeyF key_weight, uint32_t want, float want_sum, uint32_t* key_out,
                             uint32_t stop_at = 0, uint32_t* n_ge_out = nullptr) {
  const uint32_t want0 = want;
  cg::cluster_group cl = cg::this_cluster();
  uint32_t prefix = 0, mask = 0;
  float above = 0.0f;
  __shared__ uint32_t comb_cnt[256];
  __shared__ float comb_sum[256];
  __shared__ uint32_t pick[3];
  __shared__ float pick_above;
  for (int shift = 24; shift >= 0; shift -= 8) {
    // every warp fills a histogram of its own (no contention between warps); they are added up afterwards
    for (int t = threadIdx.x; t < kSelWarps * 256; t += kSelThreads) (&c.sh->warp_hist[0][0])[t] = 0u;
    __syncthreads();
    uint32_t* my_cnt = c.sh->warp_hist[c.warp];
    float* my_sum = reinterpret_cast<float*>(c.sh->warp_hist[c.warp]);
    // Most keys share their leading bits (the exponent of neighbouring logits or probabilities), so plain atomics
    // would pile onto two or three bins.  Every lane therefore keeps the bin it hit last in a register and only
    // touches shared memory when the bin changes.
    {
      uint32_t cur = 0xffffffffu, cur_n = 0;
      float cur_w = 0.0f;
      for_segment(c, row, [&](int, float v) {
        uint32_t key; float w;
        key_weight(v, key, w);
        if ((key & mask) != prefix) return;
        const uint32_t d = (key >> shift) & 255u;
        if (d != cur) {
          if (cur != 0xffffffffu) {
            if (kWeighted) atomicAdd(&my_sum[cur], cur_w);
            else atomicAdd(&my_cnt[cur], cur_n);
          }
          cur = d; cur_n = 0; cur_w = 0.0f;
        }
        cur_n++;
        cur_w += w;
      });
      if (cur != 0xffffffffu) {
        if (kWeighted) atomicAdd(&my_sum[cur], cur_w);
        else atomicAdd(&my_cnt[cur], cur_n);
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      uint32_t n = 0; float sacc = 0.0f;
      for (int wq = 0; wq < kSelWarps; wq++) {
        if (kWeighted) sacc += reinterpret_cast<const float*>(c.sh->warp_hist[wq])[threadIdx.x];
        else n += c.sh->warp_hist[wq][threadIdx.x];
      }
      c.sh->hist_cnt[threadIdx.x] = n; c.sh->hist_sum[threadIdx.x] = sacc;
    }
    cl.sync();
    if (threadIdx.x < 256) {
      uint32_t n = 0; float s = 0.0f;
      for (int r = 0; r < c.csize; r++) {
        if (kWeighted) s += *cl.map_shared_rank(&c.sh->hist_sum[threadIdx.x], r);
        else n += *cl.map_shared_rank(&c.sh->hist_cnt[threadIdx.x], r);
      }
      comb_cnt[threadIdx.x] = n; comb_sum[threadIdx.x] = s;
    }
    __syncthreads();
    // Walk the bins from the top until the running count (or sum) reaches the target: warp 0, eight bins a lane.
    if (threadIdx.x == 0) { pick[0] = 256; pick_above = above; }
    __syncthreads();
    if (c.warp == 0) {
      const int b_hi = 8 * c.lane + 7;
      if (kWeighted) {
        float mine = 0.0f;
        for (int q = 0; q < 8; q++) mine += comb_sum[b_hi - q];
        float upper = mine;      // inclusive sum over this lane and the lanes above it
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          float y = __shfl_down_sync(0xffffffffu, upper, o);
          if (c.lane + o < 32) upper += y;
        }
        const float higher = __shfl_down_sync(0xffffffffu, upper, 1);   // sum over the lanes above this one
        float acc = above + (c.lane < 31 ? higher : 0.0f);
        int hit = -1;
        float acc_hit = acc;
        for (int q = 0; q < 8 && hit < 0; q++) {
          float nxt = acc + comb_sum[b_hi - q];
          if (nxt >= want_sum) { hit = b_hi - q; acc_hit = acc; }
          acc = nxt;
        }
        const uint32_t any = __ballot_sync(0xffffffffu, hit >= 0);
        if (any && c.lane == 31 - __clz(any)) { pick[0] = (uint32_t)hit; pick_above = acc_hit; }
        if (!any && c.lane == 0) pick_above = acc;   // the whole row stays below the target
      } else {
        uint32_t mine = 0;
        for (int q = 0; q < 8; q++) mine += comb_cnt[b_hi - q];
        uint32_t upper = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          uint32_t y = __shfl_down_sync(0xffffffffu, upper, o);
          if (c.lane + o < 32) upper += y;
        }
        uint32_t acc = upper - mine;
        int hit = -1;
        uint32_t acc_hit = 0;
        for (int q = 0; q < 8 && hit < 0; q++) {
          if (acc + comb_cnt[b_hi - q] >= want) { hit = b_hi - q; acc_hit = acc; }
          acc += comb_cnt[b_hi - q];
        }
        const uint32_t any = __ballot_sync(0xffffffffu, hit >= 0);
        if (any && c.lane == 31 - __clz(any)) { pick[0] = (uint32_t)hit; pick[1] = want - acc_hit; pick[2] = comb_cnt[hit]; }
      }
    }
    __syncthreads();
    const uint32_t digit = pick[0];
    if (kWeighted) above = pick_above; else want = pick[1];
    const uint32_t n_ge = kWeighted ? 0u : (want0 - want) + pick[2];   // elements above the bin plus the bin itself
    cl.sync();   // remote readers are done with this round's histograms
    if (digit == 256) return false;
    prefix |= digit << shift;
    mask |= 255u << shift;
    if (n_ge_out) *n_ge_out = n_ge;
    if (!kWeighted && stop_at && n_ge <= stop_at) break;
  }
  *key_out = prefix;
  return true;
}

// Inverse-CDF search: the first index whose running sum of prob(index, value) exceeds r (Sampler.Sample step 8,
// sampler.go:200-209; resampleRejected, speculative.go:271-291), or `dflt` when the sum never does.  Sums run per
// warp segment, then in segment order; the segment that crosses is walked again in index order.
template <class ProbF>
__device__ void cdf_find(Ctx& c, const float* __restrict__ row, ProbF prob, float r, int dflt, int32_t* out) {
  float part = 0.0f;
  for_segment(c, row, [&](int i, float v) { part += prob(i, v); });
  part = warp_sum(part);
  if (c.lane == 0) c.sh->warp_seg[c.warp] = part;
  __syncthreads();
  float tot = 0.0f;
  for (int w = 0; w < kSelWarps; w++) tot += c.sh->warp_seg[w];
  float all[kMaxCluster];
  cluster_gather1(c, tot, all);
  float base = 0.0f;
  int cross = -1;
  float run = 0.0f;
  for (int q = 0; q < c.csize; q++) {
    if (q == c.rank) base = run;
    run += all[q];
    if (cross < 0 && run > r) cross = q;
  }
  // No path below leaves early with the cluster's exchange still in use: the caller ends with a cluster barrier.
  if (cross < 0) {
    if (c.rank == 0 && threadIdx.x == 0) *out = dflt;
  } else if (cross == c.rank) {
    // this CTA holds the crossing: pick the warp, then walk its segment in order
    int wsel = kSelWarps - 1;
    float wbase = base;
    float acc = base;
    for (int w = 0; w < kSelWarps; w++) {
      float nxt = acc + c.sh->warp_seg[w];
      wbase = acc;
      if (nxt > r) { wsel = w; break; }
      acc = nxt;
    }
    if (c.warp == wsel) {
      // Two levels, so that the walk costs two memory latencies instead of one per 32 elements: every lane sums a
      // contiguous chunk of the segment, a scan over the lanes finds the chunk that crosses, and that chunk alone is
      // walked in index order.
      const int seglen = c.whi - c.wlo;
      const int chunk = (((seglen + 31) >> 5) + 3) & ~3;
      const int l0 = min(c.whi, c.wlo + c.lane * chunk), l1 = min(c.whi, l0 + chunk);
      float mine = 0.0f;
#pragma unroll 4
      for (int i = l0; i < l1; i++) mine += prob(i, __ldg(row + i));
      float x = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        float y = __shfl_up_sync(0xffffffffu, x, o);
        if (c.lane >= o) x += y;
      }
      const uint32_t over = __ballot_sync(0xffffffffu, wbase + x > r);
      const uint32_t carry = __ballot_sync(0xffffffffu, mine > 0.0f);
      int hit_idx = -1;
      if (over || carry) {
        const int lsel = over ? __ffs(over) - 1 : 31 - __clz(carry);
        const float before = __shfl_up_sync(0xffffffffu, x, 1);
        float acc2 = wbase + __shfl_sync(0xffffffffu, c.lane > 0 ? before : 0.0f, lsel);
        const int c0 = __shfl_sync(0xffffffffu, l0, lsel), c1 = __shfl_sync(0xffffffffu, l1, lsel);
        int last_pos = -1;
        for (int j = c0; j < c1 && hit_idx < 0; j += 32) {
          const int i = j + c.lane;
          const float pv = i < c1 ? prob(i, __ldg(row + i)) : 0.0f;
          float z = pv;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            float y = __shfl_up_sync(0xffffffffu, z, o);
            if (c.lane >= o) z += y;
          }
          const uint32_t hit = __ballot_sync(0xffffffffu, i < c1 && acc2 + z > r);
          if (hit) hit_idx = j + __ffs(hit) - 1;
          const uint32_t pos = __ballot_sync(0xffffffffu, pv > 0.0f);
          if (pos) last_pos = j + 31 - __clz(pos);
          acc2 += __shfl_sync(0xffffffffu, z, 31);
        }
        // when rounding put the crossing past the end of the chunk: its last element that carries probability
        if (hit_idx < 0) hit_idx = last_pos;
      }
      if (hit_idx < 0) hit_idx = c.whi > c.wlo ? c.whi - 1 : dflt;
      if (c.lane == 0) *out = hit_idx;
    }
  }
}

// Sampler.Sample with a small top-k, finished on a list: after top-k only the k largest logits (and their ties) carry
// probability, so once the radix walk has narrowed the row down to at most kCandCap elements the CTAs collect them,
// CTA 0 sorts them by index and walks the rest of the reference's chain (softmax, nucleus, min-p, draw) over the list.
// Every float32 sum runs in index order over the kept elements -- the elements the reference adds zeros for are
// skipped -- so this path gives the reference's token bit for bit.  Returns false (nothing written) when the list
// would not fit; the caller then takes the pass-per-step path.
constexpr int kCandTopK = 128;   // largest top-k that takes this path
constexpr int kCandCap = 512;    // list capacity

__device__ bool sample_row_candidates(Ctx& c, const SelParams& prm, const float* __restrict__ row, const Dist& d, int topk, float r,
                                      int32_t* out) {
  cg::cluster_group cl = cg::this_cluster();
  const int V = prm.vocab;
  uint32_t key_lo = 0, n_ge = 0;
  radix_select<false>(c, row, [&](float v, uint32_t& k, float& w) { k = order_key(d.scaled(v)); w = 0.0f; }, (uint32_t)topk, 0.0f, &key_lo,
                      (uint32_t)kCandCap, &n_ge);
  if (n_ge > (uint32_t)kCandCap) return false;     // more ties at the threshold than the list holds (uniform over the cluster)
  // the list lives in the histogram block: words [0,512) values, [512,1024) indices
  float* l_val = reinterpret_cast<float*>(&c.sh->warp_hist[0][0]);
  int32_t* l_idx = reinterpret_cast<int32_t*>(&c.sh->warp_hist[0][0]) + kCandCap;
  uint32_t* l_cnt = &c.sh->list_count;
  if (threadIdx.x == 0) *l_cnt = 0;
  __syncthreads();
  for_segment(c, row, [&](int i, float v) {
    const float x = d.scaled(v);
    if (order_key(x) >= key_lo) {
      const uint32_t pos = atomicAdd(l_cnt, 1u);
      if (pos < (uint32_t)kCandCap) { l_val[pos] = x; l_idx[pos] = i; }
    }
  });
  __syncthreads();
  cl.sync();
  if (c.rank == 0) {
    float* a_val = l_val + 2 * kCandCap;            // all candidates, then (sorted by index) the kept ones and their probabilities
    int32_t* a_idx = l_idx + 2 * kCandCap;
    float* k_val = l_val + 4 * kCandCap;
    int32_t* k_idx = l_idx + 4 * kCandCap;
    float* k_p = l_val + 6 * kCandCap;
    int32_t* k_ord = l_idx + 6 * kCandCap;
    __shared__ int s_n, s_cut, s_tok;
    __shared__ float s_thr, s_scale;
    // gather the lists of all CTAs (rank order)
    int n_c = 0;
    for (int q = 0; q < c.csize; q++) {
      const uint32_t cnt = min(*cl.map_shared_rank(l_cnt, q), (uint32_t)kCandCap);
      const float* rv = cl.map_shared_rank(l_val, q);
      const int32_t* ri = cl.map_shared_rank(l_idx, q);
      for (int t = threadIdx.x; t < (int)cnt; t += kSelThreads)
        if (n_c + t < kCandCap) { a_val[n_c + t] = rv[t]; a_idx[n_c + t] = ri[t]; }
      n_c += (int)cnt;
    }
    n_c = min(n_c, kCandCap);
    __syncthreads();
    // kthLargest (sampler.go:283-300): the value with fewer than topk elements above it and at least topk at or above
    if (threadIdx.x < n_c) {
      const float v = a_val[threadIdx.x];
      int gt = 0, ge = 0;
      for (int j = 0; j < n_c; j++) { gt += a_val[j] > v; ge += a_val[j] >= v; }
      if (gt < topk && topk <= ge) s_thr = v;
    }
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    const float thr = s_thr;
    // keep what the mask leaves (not below the threshold), in index order
    if (threadIdx.x < n_c && !(a_val[threadIdx.x] < thr)) {
      int pos = 0;
      for (int j = 0; j < n_c; j++) pos += (!(a_val[j] < thr)) && a_idx[j] < a_idx[threadIdx.x];
      k_val[pos] = a_val[threadIdx.x];
      k_idx[pos] = a_idx[threadIdx.x];
      atomicAdd(&s_n, 1);
    }
    __syncthreads();
    const int n_k = s_n;
    // softmax over the kept logits (sampler.go:118-137)
    if (threadIdx.x == 0) {
      float maxV = k_val[0];
      for (int j = 1; j < n_k; j++) if (k_val[j] > maxV) maxV = k_val[j];
      float sum = 0.0f;
      for (int j = 0; j < n_k; j++) { k_p[j] = fastexp32_ref(__fsub_rn(k_val[j], maxV)); sum = __fadd_rn(sum, k_p[j]); }
      s_scale = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 1.0f;
    }
    __syncthreads();
    if (threadIdx.x < n_k) k_p[threadIdx.x] = __fmul_rn(k_p[threadIdx.x], s_scale);
    __syncthreads();
    float topP = prm.top_p;
    if (topP <= 0.0f || topP > 1.0f) topP = 1.0f;
    if (topP < 1.0f) {
      // argsortDescF32 (sampler.go:268-281) followed only as far as the cut: a selection sort over all indices whose
      // step i swaps the first largest remaining entry with whatever sits at position i.  Entries without probability
      // are interchangeable, so only the positions of the kept elements are tracked (k_ord: position in the reference's
      // index array, -1 once selected, -2 selected and kept); which of two equal probabilities comes first follows
      // from the swaps, exactly as in the reference.
      if (threadIdx.x < n_k) k_ord[threadIdx.x] = k_idx[threadIdx.x];
      __syncthreads();
      if (c.warp == 0) {   // one warp: the search of every step is spread over its lanes, the running sum stays sequential
        float cum = 0.0f;
        bool cut = false;
        for (int step = 0; step < n_k && !cut; step++) {
          float bp = -1.0f;
          int bpos = 0x7fffffff, bj = -1, at_i = -1;
          for (int j = c.lane; j < n_k; j += 32) {
            const int pj = k_ord[j];
            if (pj < 0) continue;
            if (pj == step) at_i = j;
            const float pv = k_p[j];
            if (pv > bp || (pv == bp && pj < bpos)) { bp = pv; bpos = pj; bj = j; }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float op = __shfl_xor_sync(0xffffffffu, bp, o);
            const int opos = __shfl_xor_sync(0xffffffffu, bpos, o), oj = __shfl_xor_sync(0xffffffffu, bj, o);
            at_i = max(at_i, __shfl_xor_sync(0xffffffffu, at_i, o));
            if (op > bp || (op == bp && opos < bpos)) { bp = op; bpos = opos; bj = oj; }
          }
          if (bj < 0 || !(bp > 0.0f)) break;      // only zeros are left: the running sum stays below top-p
          if (c.lane == 0) {
            if (at_i >= 0 && at_i != bj) k_ord[at_i] = bpos;   // what sat at position `step` moves to the winner's place
            k_ord[bj] = -2;
          }
          __syncwarp();
          cum = __fadd_rn(cum, bp);
          if (cum >= topP) cut = true;
        }
        if (c.lane == 0) s_cut = cut ? 1 : 0;
      }
      __syncthreads();
      if (s_cut && threadIdx.x < n_k && k_ord[threadIdx.x] != -2) k_p[threadIdx.x] = 0.0f;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s2 = 0.0f;
        for (int j = 0; j < n_k; j++) s2 = __fadd_rn(s2, k_p[j]);
        s_scale = s2 > 0.0f ? __fdiv_rn(1.0f, s2) : 1.0f;
      }
      __syncthreads();
      if (threadIdx.x < n_k) k_p[threadIdx.x] = __fmul_rn(k_p[threadIdx.x], s_scale);
      __syncthreads();
    }
    if (prm.min_p > 0.0f) {
      if (threadIdx.x == 0) {
        float maxProb = 0.0f;
        for (int j = 0; j < n_k; j++) if (k_p[j] > maxProb) maxProb = k_p[j];
        s_thr = __fmul_rn(maxProb, prm.min_p);
      }
      __syncthreads();
      if (threadIdx.x < n_k && k_p[threadIdx.x] < s_thr) k_p[threadIdx.x] = 0.0f;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s3 = 0.0f;
        for (int j = 0; j < n_k; j++) s3 = __fadd_rn(s3, k_p[j]);
        s_scale = s3 > 0.0f ? __fdiv_rn(1.0f, s3) : 1.0f;
      }
      __syncthreads();
      if (threadIdx.x < n_k) k_p[threadIdx.x] = __fmul_rn(k_p[threadIdx.x], s_scale);
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      float cum = 0.0f;
      int tok = V - 1;
      for (int j = 0; j < n_k; j++) {
        cum = __fadd_rn(cum, k_p[j]);
        if (r < cum) { tok = k_idx[j]; break; }
      }
      *out = tok;
    }
  }
  return true;
}

// Sampler.Sample on one row (sampler.go:73-218, steps 3-8; no repetition penalties), one cluster per row.
__device__ void sample_row(Ctx& c, const SelParams& prm, const float* __restrict__ row, float r, int32_t* out) {
  const int V = prm.vocab;
  Dist d;
  d.temp = prm.temperature <= 0.0f ? 1e-5f : prm.temperature;
  d.topk_key = 0; d.tau = 0.0f; d.inv2 = 1.0f; d.minp_thr = 0.0f; d.inv3 = 1.0f;
  bool nucleus = false, minp = false;
  int topk = prm.top_k;
  if (topk < 0 || topk >= V) topk = 0;
  d.m = 0.0f; d.inv1 = 1.0f;
  if (topk > 0 && topk <= kCandTopK && sample_row_candidates(c, prm, row, d, topk, r, out)) return;
  if (topk > 0) {
    uint32_t key = 0;
    radix_select<false>(c, row, [&](float v, uint32_t& k, float& w) { k = order_key(d.scaled(v)); w = 0.0f; }, (uint32_t)topk, 0.0f, &key);
    d.topk_key = key;
  }
  float v4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  for_segment(c, row, [&](int, float v) { v4[0] = fmaxf(v4[0], d.scaled(v)); });
  cluster_reduce4<1>(c, v4);
  d.m = v4[0];
  d.inv1 = 1.0f;
  v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
  for_segment(c, row, [&](int, float v) { v4[0] += d.p1(v); });
  cluster_reduce4<0>(c, v4);
  if (v4[0] > 0.0f) d.inv1 = __fdiv_rn(1.0f, v4[0]);
  float topP = prm.top_p;
  if (topP <= 0.0f || topP > 1.0f) topP = 1.0f;
  if (topP < 1.0f) {
    nucleus = true;
    uint32_t key = 0;
    bool cut = radix_select<true>(c, row, [&](float v, uint32_t& k, float& w) { w = d.p1(v); k = __float_as_uint(w); }, 0u, topP, &key);
    const float tau = cut ? __uint_as_float(key) : 0.0f;
    v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
    for_segment(c, row, [&](int, float v) { float p = d.p1(v); if (p >= tau) v4[0] += p; });
    cluster_reduce4<0>(c, v4);
    d.tau = tau;
    d.inv2 = v4[0] > 0.0f ? __fdiv_rn(1.0f, v4[0]) : 1.0f;
  }
  // Dist::p2 drops below tau only when tau > 0; the renormalisation applies whenever the nucleus step ran
  auto p2 = [&](float v) { float p = d.p1(v); if (nucleus) p = p < d.tau ? 0.0f : __fmul_rn(p, d.inv2); return p; };
  if (prm.min_p > 0.0f) {
    minp = true;
    // the largest probability belongs to the row maximum, which no filter removes
    v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
    for_segment(c, row, [&](int, float v) { v4[0] = fmaxf(v4[0], p2(v)); });
    cluster_reduce4<1>(c, v4);
    const float thr = __fmul_rn(v4[0], prm.min_p);
    v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
    for_segment(c, row, [&](int, float v) { float p = p2(v); if (!(p < thr)) v4[0] += p; });
    cluster_reduce4<0>(c, v4);
    d.minp_thr = thr;
    d.inv3 = v4[0] > 0.0f ? __fdiv_rn(1.0f, v4[0]) : 1.0f;
  }
  auto p3 = [&](int, float v) { float p = p2(v); if (minp) p = p < d.minp_thr ? 0.0f : __fmul_rn(p, d.inv3); return p; };
  cdf_find(c, row, p3, r, V - 1, out);
}

__global__ void __launch_bounds__(kSelThreads, 2) spec_accept_kernel(SelParams prm) {
  cg::cluster_group cl = cg::this_cluster();
  __shared__ SelShared sh;
  Ctx c;
  c.sh = &sh;
  c.csize = (int)cl.num_blocks();
  c.rank = (int)cl.block_rank();
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.round = 0;
  const int V = prm.vocab, k = prm.k;
  const int per = ((V + c.csize - 1) / c.csize + 127) & ~127;
  c.lo = min(V, c.rank * per);
  c.hi = min(V, c.lo + per);
  const int wper = ((c.hi - c.lo + kSelWarps - 1) / kSelWarps + 127) & ~127;
  c.vec = (V & 3) == 0 && (((uintptr_t)prm.target_logits | (uintptr_t)prm.draft_logits) & 15) == 0;
  c.wlo = min(c.hi, c.lo + c.warp * wper);
  c.whi = min(c.hi, c.wlo + wper);
  const int b = blockIdx.x / c.csize;
  const float* draws = prm.draws + (size_t)b * (k + 1);
  int32_t* out_tok = prm.next_token + b;
  const bool writer = c.rank == 0 && threadIdx.x == 0;
  int used = 0;
  int n_acc = k;
  bool done = false;
  // Few sequences: the chain's length is what costs, not the bytes.  The maxima of the rows of ALL draft positions are
  // taken in one stage and all sums of exponentials in a second, so the accept loop below runs without a pass of its own
  // per position (rows after a rejection are read in vain).
  const bool batched = prm.batched && k >= 2 && 2 * k <= kStatMax;
  if (batched) {
    float acc[kStatMax];
    for (int i = 0; i < k; i++) {
      float a = -INFINITY, t = -INFINITY;
      for_segment2(c, prm.draft_logits + ((size_t)b * k + i) * V, prm.target_logits + ((size_t)b * (k + 1) + i) * V,
                   [&](int, float dv, float tv) { a = fmaxf(a, dv); t = fmaxf(t, tv); });
      acc[2 * i] = a;
      acc[2 * i + 1] = t;
    }
    cluster_reduce_n<true>(c, acc, 2 * k, c.sh->stat[0]);
    for (int i = 0; i < k; i++) {
      const float md = c.sh->stat[0][2 * i], mt = c.sh->stat[0][2 * i + 1];
      float a = 0.0f, t = 0.0f;
      for_segment2(c, prm.draft_logits + ((size_t)b * k + i) * V, prm.target_logits + ((size_t)b * (k + 1) + i) * V,
                   [&](int, float dv, float tv) { a += fastexp32_ref(__fsub_rn(dv, md)); t += fastexp32_ref(__fsub_rn(tv, mt)); });
      acc[2 * i] = a;
      acc[2 * i + 1] = t;
    }
    cluster_reduce_n<false>(c, acc, 2 * k, c.sh->stat[1]);
  }
  float next_md = 0.0f, next_mt = 0.0f;
  if (k > 0 && prm.lookahead && !batched) {
    float v4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for_segment2(c, prm.draft_logits + (size_t)b * k * V, prm.target_logits + (size_t)b * (k + 1) * V,
                 [&](int, float dv, float tv) { v4[0] = fmaxf(v4[0], dv); v4[1] = fmaxf(v4[1], tv); });
    cluster_reduce4<1>(c, v4);
    next_md = v4[0];
    next_mt = v4[1];
  }
  for (int i = 0; i < k && !done; i++) {
    const float* drow = prm.draft_logits + ((size_t)b * k + i) * V;
    const float* trow = prm.target_logits + ((size_t)b * (k + 1) + i) * V;
    const int tok = prm.draft_tokens[(size_t)b * k + i];
    if (tok < 0 || tok >= V) {   // uniform over the cluster: every thread reads the same token
      if (writer) { set_status(prm.status, RELUX_ERR_INVALID_ARG); *out_tok = -1; }
      n_acc = -1;
      done = true;
      break;
    }
    // With look-ahead the maxima of this position's rows came with the previous position's sums (or from the pass
    // before the loop): the pass below adds up the exponentials and already takes the maxima of the next position's
    // rows, one barrier per draft position, at the price of two rows read in vain when this position rejects.  That
    // pays while the chain is bound by latency (few sequences); with many sequences the passes are bound by bytes and
    // the maxima get a pass of their own.
    float v4[4];
    float md, mt;
    if (batched) {
      md = c.sh->stat[0][2 * i];
      mt = c.sh->stat[0][2 * i + 1];
      v4[0] = c.sh->stat[1][2 * i];
      v4[1] = c.sh->stat[1][2 * i + 1];
    } else {
      if (!prm.lookahead) {
        v4[0] = v4[1] = v4[2] = v4[3] = -INFINITY;
        for_segment2(c, drow, trow, [&](int, float dv, float tv) { v4[0] = fmaxf(v4[0], dv); v4[1] = fmaxf(v4[1], tv); });
        cluster_reduce4<1>(c, v4);
        next_md = v4[0];
        next_mt = v4[1];
      }
      md = next_md;
      mt = next_mt;
      v4[0] = v4[1] = 0.0f;
      v4[2] = v4[3] = -INFINITY;
      for_segment2(c, drow, trow, [&](int, float dv, float tv) {
        v4[0] += fastexp32_ref(__fsub_rn(dv, md));
        v4[1] += fastexp32_ref(__fsub_rn(tv, mt));
      });
      if (prm.lookahead && i + 1 < k)
        for_segment2(c, drow + V, trow + V, [&](int, float dv, float tv) { v4[2] = fmaxf(v4[2], dv); v4[3] = fmaxf(v4[3], tv); });
      cluster_reduce4<2>(c, v4);
      next_md = v4[2];
      next_mt = v4[3];
    }
    const float invd = v4[0] > 0.0f ? __fdiv_rn(1.0f, v4[0]) : 1.0f;
    const float invt = v4[1] > 0.0f ? __fdiv_rn(1.0f, v4[1]) : 1.0f;
    const float dP = __fmul_rn(fastexp32_ref(__fsub_rn(__ldg(drow + tok), md)), invd);
    const float tP = __fmul_rn(fastexp32_ref(__fsub_rn(__ldg(trow + tok), mt)), invt);
    float ap = __fdiv_rn(tP, dP > 1e-10f ? dP : 1e-10f);
    if (ap > 1.0f) ap = 1.0f;
    const float u = draws[used++];
    if (u < ap) continue;
    // rejected at i: resample from norm(max(0, p_target - p_draft))   speculative.go:256-295
    auto adj = [&](int j, float tv) {
      float tp = __fmul_rn(fastexp32_ref(__fsub_rn(tv, mt)), invt);
      float dp = __fmul_rn(fastexp32_ref(__fsub_rn(__ldg(drow + j), md)), invd);
      float diff = __fsub_rn(tp, dp);
      return diff < 0.0f ? 0.0f : diff;
    };
    v4[0] = v4[1] = v4[2] = v4[3] = 0.0f;
    for_segment2(c, drow, trow, [&](int, float dv, float tv) {
      float diff = __fsub_rn(__fmul_rn(fastexp32_ref(__fsub_rn(tv, mt)), invt), __fmul_rn(fastexp32_ref(__fsub_rn(dv, md)), invd));
      v4[0] += diff < 0.0f ? 0.0f : diff;
    });
    cluster_reduce4<0>(c, v4);
    const float r = draws[used++];
    if (v4[0] > 0.0f) {
      const float inv = __fdiv_rn(1.0f, v4[0]);
      cdf_find(c, trow, [&](int j, float tv) { return __fmul_rn(adj(j, tv), inv); }, r, 0, out_tok);
    } else {
      cdf_find(c, trow, [&](int, float tv) { return __fmul_rn(fastexp32_ref(__fsub_rn(tv, mt)), invt); }, r, 0, out_tok);
    }
    n_acc = i;
    done = true;
  }
  if (!done) sample_row(c, prm, prm.target_logits + ((size_t)b * (k + 1) + k) * V, draws[used++], out_tok);
  if (writer && prm.n_accepted) prm.n_accepted[b] = n_acc;
  cl.sync();   // no CTA leaves while another may still read its exchange buffers
}

// ---- REFERENCE: one thread per sequence, the reference's loops in the reference's order ------------------------
__device__ void ref_softmax_alloc(const float* logits, int n, float* probs) {   // speculative.go:346-368
  float maxV = logits[0];
  for (int i = 1; i < n; i++)
    if (logits[i] > maxV) maxV = logits[i];
  float sum = 0.0f;
  for (int i = 0; i < n; i++) {
    probs[i] = fastexp32_ref(__fsub_rn(logits[i], maxV));
    sum = __fadd_rn(sum, probs[i]);
  }
  if (sum > 0.0f) {
    const float inv = __fdiv_rn(1.0f, sum);
    for (int i = 0; i < n; i++) probs[i] = __fmul_rn(probs[i], inv);
  }
}

__device__ void ref_renormalise(float* probs, int n) {
  float s = 0.0f;
  for (int i = 0; i < n; i++) s = __fadd_rn(s, probs[i]);
  if (s > 0.0f) {
    const float inv = __fdiv_rn(1.0f, s);
    for (int i = 0; i < n; i++) probs[i] = __fmul_rn(probs[i], inv);
  }
}

// Sampler.Sample steps 3-8 (sampler.go:89-209).  scratch, probs: [n] floats; idx: [n] ints.
__device__ int ref_sample(const SelParams& prm, const float* logits, int n, float r, float* scratch, float* probs, int32_t* idx) {
  float temp = prm.temperature <= 0.0f ? 1e-5f : prm.temperature;
  for (int i = 0; i < n; i++) scratch[i] = temp != 1.0f ? __fdiv_rn(logits[i], temp) : logits[i];
  int topK = prm.top_k;
  if (topK < 0 || topK >= n) topK = 0;
  if (topK > 0) {
    // value of the topK-th largest element, duplicates counted (kthLargest, sampler.go:283-300)
    float bound = INFINITY;
    int seen = 0;
    float threshold = scratch[0];
    while (true) {
      float best = -INFINITY;
      int cnt = 0;
      for (int i = 0; i < n; i++) {
        const float v = scratch[i];
        if (v < bound) {
          if (v > best) { best = v; cnt = 1; }
          else if (v == best) cnt++;
        }
      }
      if (cnt == 0) break;
      seen += cnt;
      threshold = best;
      if (seen >= topK) break;
      bound = best;
    }
    for (int i = 0; i < n; i++)
      if (scratch[i] < threshold) scratch[i] = -INFINITY;
  }
  float maxV = scratch[0];
  for (int i = 1; i < n; i++)
    if (scratch[i] > maxV) maxV = scratch[i];
  float sum = 0.0f;
  for (int i = 0; i < n; i++) {
    if (scratch[i] == -INFINITY) probs[i] = 0.0f;
    else { probs[i] = fastexp32_ref(__fsub_rn(scratch[i], maxV)); sum = __fadd_rn(sum, probs[i]); }
  }
  if (sum > 0.0f) {
    const float inv = __fdiv_rn(1.0f, sum);
    for (int i = 0; i < n; i++) probs[i] = __fmul_rn(probs[i], inv);
  }
  float topP = prm.top_p;
  if (topP <= 0.0f || topP > 1.0f) topP = 1.0f;
  if (topP < 1.0f) {
    // argsortDescF32's selection sort (sampler.go:268-281), stopped at the cut-off: later positions are all zeroed
    for (int i = 0; i < n; i++) idx[i] = i;
    float cum = 0.0f;
    int cutoff = n;
    for (int i = 0; i < n; i++) {
      int maxJ = i;
      for (int j = i + 1; j < n; j++)
        if (probs[idx[j]] > probs[idx[maxJ]]) maxJ = j;
      const int t = idx[i]; idx[i] = idx[maxJ]; idx[maxJ] = t;
      cum = __fadd_rn(cum, probs[idx[i]]);
      if (cum >= topP) { cutoff = i + 1; break; }
    }
    for (int j = cutoff; j < n; j++) probs[idx[j]] = 0.0f;
    ref_renormalise(probs, n);
  }
  if (prm.min_p > 0.0f) {
    float maxProb = 0.0f;
    for (int i = 0; i < n; i++)
      if (probs[i] > maxProb) maxProb = probs[i];
    const float threshold = __fmul_rn(maxProb, prm.min_p);
    for (int i = 0; i < n; i++)
      if (probs[i] < threshold) probs[i] = 0.0f;
    ref_renormalise(probs, n);
  }
  float cum = 0.0f;
  for (int i = 0; i < n; i++) {
    cum = __fadd_rn(cum, probs[i]);
    if (r < cum) return i;
  }
  return n - 1;
}

__global__ void spec_accept_reference_kernel(SelParams prm, int n_seqs, float* fscratch, int32_t* iscratch) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_seqs) return;
  const int V = prm.vocab, k = prm.k;
  float* dp = fscratch + (size_t)b * 2 * V;
  float* tp = dp + V;
  int32_t* idx = iscratch + (size_t)b * V;
  const float* draws = prm.draws + (size_t)b * (k + 1);
  int used = 0;
  for (int i = 0; i < k; i++) {
    const int tok = prm.draft_tokens[(size_t)b * k + i];
    if (tok < 0 || tok >= V) {
      set_status(prm.status, RELUX_ERR_INVALID_ARG);
      prm.next_token[b] = -1;
      if (prm.n_accepted) prm.n_accepted[b] = -1;
      return;
    }
    ref_softmax_alloc(prm.draft_logits + ((size_t)b * k + i) * V, V, dp);
    ref_softmax_alloc(prm.target_logits + ((size_t)b * (k + 1) + i) * V, V, tp);
    const float dP = dp[tok], tP = tp[tok];
    float ap = __fdiv_rn(tP, dP > 1e-10f ? dP : 1e-10f);
    if (ap > 1.0f) ap = 1.0f;
    if (draws[used++] < ap) continue;
    // resampleRejected (speculative.go:256-295); the adjusted row overwrites dp
    float sum = 0.0f;
    for (int j = 0; j < V; j++) {
      float diff = __fsub_rn(tp[j], dp[j]);
      if (diff < 0.0f) diff = 0.0f;
      dp[j] = diff;
      sum = __fadd_rn(sum, diff);
    }
    const float r = draws[used++];
    int result = 0;
    float cum = 0.0f;
    if (sum > 0.0f) {
      const float inv = __fdiv_rn(1.0f, sum);
      for (int j = 0; j < V; j++) {
        cum = __fadd_rn(cum, __fmul_rn(dp[j], inv));
        if (r < cum) { result = j; break; }
      }
    } else {
      for (int j = 0; j < V; j++) {
        cum = __fadd_rn(cum, tp[j]);
        if (r < cum) { result = j; break; }
      }
    }
    prm.next_token[b] = result;
    if (prm.n_accepted) prm.n_accepted[b] = i;
    return;
  }
  prm.next_token[b] = ref_sample(prm, prm.target_logits + ((size_t)b * (k + 1) + k) * V, V, draws[used++], dp, tp, idx);
  if (prm.n_accepted) prm.n_accepted[b] = k;
}


// Sampler.applyRepetitionPenalties (sampler.go:221-266): copies every row to `dst` and rewrites the logits of the tokens
// in the row's window of previous tokens -- repeat penalty (divide a positive logit, multiply a negative one), then
// frequency penalty times the token's count in the window, then presence penalty, each applied once per distinct
// token, in float32 like the reference.  One block per row; win_off [n + 1] delimits the rows' windows in win_tok.
__global__ void repetition_penalty_kernel(const float* __restrict__ src, float* __restrict__ dst, int vocab,
                                          const int32_t* __restrict__ win_tok, const int32_t* __restrict__ win_off,
                                          float rp, float fp, float pp) {
  const int b = blockIdx.x;
  const float* s = src + (size_t)b * vocab;
  float* d = dst + (size_t)b * vocab;
  if ((vocab & 3) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    for (int i = threadIdx.x * 4; i < vocab; i += blockDim.x * 4)
      *reinterpret_cast<float4*>(d + i) = __ldg(reinterpret_cast<const float4*>(s + i));
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) d[i] = s[i];
  }
  __syncthreads();
  const int w0 = win_off[b], w1 = win_off[b + 1];
  for (int j = w0 + threadIdx.x; j < w1; j += blockDim.x) {
    const int tok = win_tok[j];
    if (tok < 0 || tok >= vocab) continue;
    bool first = true;
    int freq = 0;
    for (int q = w0; q < w1; q++) {
      if (win_tok[q] == tok) { freq++; if (q < j) first = false; }
    }
    if (!first) continue;     // one thread per distinct token: the first occurrence owns the update
    float x = d[tok];
    if (rp != 1.0f && rp != 0.0f) x = x > 0.0f ? __fdiv_rn(x, rp) : __fmul_rn(x, rp);
    if (fp != 0.0f) x = __fsub_rn(x, __fmul_rn(fp, (float)freq));
    if (pp != 0.0f) x = __fsub_rn(x, pp);
    d[tok] = x;
  }
}

// Launches the selection kernel on device-resident inputs (prm holds the input pointers, k and vocab) and brings the
// 2 n result words (accepted counts, then tokens) to the host; synchronises the stream.
static int32_t launch_selection(Pool* p, SelParams& prm, int n, const relux_sampler_params& sp, int mode, std::vector<int32_t>& host) {
  Device* dev = p->dev;
  const int V = prm.vocab;
  int32_t rc;
  rc = grow(dev, p->out_buf, sizeof(int32_t) * 2 * (size_t)n);
  if (rc) return rc;
  prm.n_accepted = (int32_t*)p->out_buf.p;
  prm.next_token = prm.n_accepted + n;
  prm.status = p->d_status;
  prm.temperature = sp.temperature;
  prm.top_k = sp.top_k;
  prm.top_p = sp.top_p;
  prm.min_p = sp.min_p;
  prm.batched = n <= 16 ? 1 : 0;
  if (p->tune.get(RELUX_TUNE_SEL_BATCHED) >= 0) prm.batched = p->tune.get(RELUX_TUNE_SEL_BATCHED) ? 1 : 0;       // tuning knob
  prm.lookahead = n <= 32 ? 1 : 0;   // measured: 6 % faster at 4-16 sequences, even at 32, 1 % slower at 64
  if (p->tune.get(RELUX_TUNE_SEL_LOOKAHEAD) >= 0) prm.lookahead = p->tune.get(RELUX_TUNE_SEL_LOOKAHEAD) ? 1 : 0;   // tuning knob
  if (mode == RELUX_ATTN_REFERENCE) {
    // One thread per sequence repeats the reference's selection sorts: quadratic in the vocabulary for the nucleus cut,
    // top_k x vocabulary for kthLargest.  Refuse sizes that would keep the device busy for many seconds.
    const bool nucleus = sp.top_p > 0.0f && sp.top_p < 1.0f;
    const bool topk = sp.top_k > 0 && sp.top_k < V;
    if ((nucleus && V > 32768) || (topk && (double)sp.top_k * V > 1e9)) {
      set_error("RELUX_ATTN_REFERENCE repeats the reference's O(vocab^2) sorts on one thread per sequence: vocab %d with these "
                "filters is outside what it is meant for (parity checks); use RELUX_ATTN_FAST", V);
      return RELUX_ERR_UNSUPPORTED;
    }
    rc = grow(dev, p->part_o, sizeof(float) * 2 * (size_t)n * V);
    if (rc) return rc;
    rc = grow(dev, p->part_ml, sizeof(int32_t) * (size_t)n * V);
    if (rc) return rc;
  }
  // device time of the selection kernel, readable through relux_pool_kernel_ms_mean like the attention kernels'
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_begin(), dev->stream));
  if (mode == RELUX_ATTN_REFERENCE) {
    spec_accept_reference_kernel<<<(n + 31) / 32, 32, 0, dev->stream>>>(prm, n, (float*)p->part_o.p, (int32_t*)p->part_ml.p);
  } else {
    // Cluster size: slices should stay long enough to keep 512 threads busy, and all sequences should be resident at
    // once -- a second wave of clusters doubles the latency of the whole chain, which costs more than longer slices.
    const int by_vocab = V >= 32768 ? 8 : V >= 8192 ? 4 : V >= 2048 ? 2 : 1;
    static int resident[64][4] = {};   // [device][log2 cluster size]: clusters the device holds at once, 0 = not asked yet
    int csize = 1;
    double best = 1e30;
    for (int lg = 3; lg >= 0; lg--) {
      const int cs = 1 << lg;
      if (cs > by_vocab) continue;
      int& have = resident[dev->index & 63][lg];
      if (have == 0) {
        cudaLaunchConfig_t q{};
        q.gridDim = dim3((unsigned)(cs * 64));
        q.blockDim = dim3(kSelThreads);
        cudaLaunchAttribute qa{};
        qa.id = cudaLaunchAttributeClusterDimension;
        qa.val.clusterDim.x = (unsigned)cs;
        qa.val.clusterDim.y = qa.val.clusterDim.z = 1;
        q.attrs = &qa;
        q.numAttrs = 1;
        int nc = 0;
        if (cudaOccupancyMaxActiveClusters(&nc, spec_accept_kernel, &q) != cudaSuccess || nc <= 0) { cudaGetLastError(); nc = 1; }
        have = nc;
      }
      const double cost = (double)((n + have - 1) / have) / cs;   // waves x slice length
      if (cost <= best) { best = cost; csize = cs; }   // on a tie the smaller cluster: fewer waves, fewer remote reads
    }
    {   // tuning knob: 1, 2, 4 or 8
      const int v = p->tune.get(RELUX_TUNE_SEL_CLUSTER);
      if (v == 1 || v == 2 || v == 4 || v == 8) csize = v;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(n * csize));
    cfg.blockDim = dim3(kSelThreads);
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)csize;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    RELUX_CUDA_TRY(cudaLaunchKernelEx(&cfg, spec_accept_kernel, prm));
  }
  RELUX_CUDA_TRY(cudaGetLastError());
  RELUX_CUDA_TRY(cudaEventRecord(p->ev_end(), dev->stream));
  p->timed_calls++;
  count_launch(dev);
  host.resize((size_t)2 * n);
  RELUX_CUDA_TRY(cudaMemcpyAsync(host.data(), p->out_buf.p, sizeof(int32_t) * 2 * (size_t)n, cudaMemcpyDeviceToHost, dev->stream));
  RELUX_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return RELUX_OK;
}

}  // namespace

int32_t do_spec_accept(Pool* p, const relux_spec_accept_args* a) {
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const int n = a->n_seqs, k = a->k, V = a->vocab;
  if (n <= 0 || k < 0 || V <= 0 || !a->target_logits || !a->draws || !a->next_token ||
      (k > 0 && (!a->draft_tokens || !a->draft_logits || !a->n_accepted)) ||
      (a->mem != RELUX_MEM_HOST && a->mem != RELUX_MEM_DEVICE) ||
      (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE)) {
    set_error("spec_accept: bad arguments");
    return RELUX_ERR_INVALID_ARG;
  }
  if (a->commit) {
    // checked before anything is launched, so that a commit is all or nothing: every sequence live and named once, and
    // room on every layer for the longest possible result (k + 1 rows)
    if (n > p->prm.max_seqs) { set_error("spec_accept: more sequences than the pool holds"); return RELUX_ERR_INVALID_ARG; }
    SeqBatch chk;
    int32_t rc0 = stage_batch(p, n, a->seq_ids, nullptr, 1, &chk);
    if (rc0) return rc0;
    for (int l = 0; l < p->prm.num_layers; l++)
      for (int i = 0; i < n; i++) {
        const int s = chk.seq[i];
        const int len = p->h_len[(size_t)l * p->prm.max_seqs + s], cap = p->seq_pages[s] * p->prm.page_tokens;
        if (len + k + 1 > cap) {
          set_error("spec_accept: committing up to %d rows would pass the capacity %d of sequence %d on layer %d (length %d)", k + 1, cap, s, l, len);
          return RELUX_ERR_OVERFLOW;
        }
      }
  }
  if (a->mem == RELUX_MEM_HOST)
    for (size_t i = 0; i < (size_t)n * k; i++)
      if (a->draft_tokens[i] < 0 || a->draft_tokens[i] >= V) {
        set_error("spec_accept: draft token %d outside the vocabulary of %d", a->draft_tokens[i], V);
        return RELUX_ERR_INVALID_ARG;
      }
  Device* dev = p->dev;
  SelParams prm{};
  const void* d = nullptr;
  int32_t rc;
  if (k > 0) {
    rc = stage_in(p, p->in_a, a->draft_logits, sizeof(float) * (size_t)n * k * V, a->mem, &d);
    if (rc) return rc;
    prm.draft_logits = (const float*)d;
    rc = stage_in(p, p->q_conv, a->draft_tokens, sizeof(int32_t) * (size_t)n * k, a->mem, &d);
    if (rc) return rc;
    prm.draft_tokens = (const int32_t*)d;
  }
  rc = stage_in(p, p->in_b, a->target_logits, sizeof(float) * (size_t)n * (k + 1) * V, a->mem, &d);
  if (rc) return rc;
  prm.target_logits = (const float*)d;
  rc = stage_in(p, p->o_lat, a->draws, sizeof(float) * (size_t)n * (k + 1), a->mem, &d);
  if (rc) return rc;
  prm.draws = (const float*)d;
  prm.k = k;
  prm.vocab = V;
  std::vector<int32_t> host;
  rc = launch_selection(p, prm, n, a->sampler, a->mode, host);
  if (rc) return rc;
  for (int i = 0; i < n; i++) {
    if (a->n_accepted) a->n_accepted[i] = host[i];
    a->next_token[i] = host[(size_t)n + i];
    if (host[(size_t)n + i] < 0 || (k > 0 && host[i] < 0)) {
      set_error("spec_accept: a draft token of sequence %d lies outside the vocabulary of %d", i, V);
      return RELUX_ERR_INVALID_ARG;
    }
  }
  if (a->commit) {
    std::vector<int32_t> new_len((size_t)n);
    for (int l = 0; l < p->prm.num_layers; l++) {
      for (int i = 0; i < n; i++) {
        const int s = a->seq_ids ? a->seq_ids[i] : i;
        if (s < 0 || s >= p->prm.max_seqs) { set_error("spec_accept: bad sequence id %d", s); return RELUX_ERR_INVALID_ARG; }
        new_len[i] = p->h_len[(size_t)l * p->prm.max_seqs + s] + (k > 0 ? host[i] : 0) + 1;
      }
      rc = seq_set_len(p, l, n, a->seq_ids, new_len.data());
      if (rc) return rc;
    }
  }
  return RELUX_OK;
}

int32_t do_sample(Pool* p, const relux_sample_args* a) {
  if (!a) { set_error("nil argument struct"); return RELUX_ERR_INVALID_ARG; }
  const int n = a->n_rows, V = a->vocab;
  if (n <= 0 || V <= 0 || !a->logits || !a->draws || !a->tokens || (a->mem != RELUX_MEM_HOST && a->mem != RELUX_MEM_DEVICE) ||
      (a->mode != RELUX_ATTN_FAST && a->mode != RELUX_ATTN_REFERENCE) || (a->prev_tokens && (!a->prev_len || a->prev_stride < 0))) {
    set_error("sampler_sample: bad arguments");
    return RELUX_ERR_INVALID_ARG;
  }
  Device* dev = p->dev;
  SelParams prm{};
  const void* d = nullptr;
  int32_t rc = stage_in(p, p->in_b, a->logits, sizeof(float) * (size_t)n * V, a->mem, &d);
  if (rc) return rc;
  prm.target_logits = (const float*)d;
  rc = stage_in(p, p->o_lat, a->draws, sizeof(float) * (size_t)n, a->mem, &d);
  if (rc) return rc;
  prm.draws = (const float*)d;
  const bool penalties = a->prev_tokens && ((a->repeat_penalty != 1.0f && a->repeat_penalty != 0.0f) || a->frequency_penalty != 0.0f ||
                                            a->presence_penalty != 0.0f);
  if (penalties) {
    // the window of every row (sampler.go:225-228), flattened: offsets [n + 1] then tokens
    std::vector<int32_t> flat((size_t)n + 1, 0);
    for (int i = 0; i < n; i++) {
      int len = a->prev_len[i];
      if (len < 0 || len > a->prev_stride) { set_error("sampler_sample: prev_len[%d] = %d outside [0, %d]", i, len, a->prev_stride); return RELUX_ERR_INVALID_ARG; }
      int w0 = (a->repeat_window > 0 && len > a->repeat_window) ? len - a->repeat_window : 0;
      const int32_t* row = a->prev_tokens + (size_t)i * a->prev_stride;
      flat.insert(flat.end(), row + w0, row + len);
      flat[i + 1] = (int32_t)(flat.size() - (size_t)n - 1);
    }
    if (flat.size() > (size_t)n + 1) {
      rc = grow(dev, p->q_conv, sizeof(int32_t) * flat.size());
      if (rc) return rc;
      rc = grow(dev, p->layer_buf, sizeof(float) * (size_t)n * V);
      if (rc) return rc;
      // pageable source: the copy has left the vector when the call returns
      RELUX_CUDA_TRY(cudaMemcpyAsync(p->q_conv.p, flat.data(), sizeof(int32_t) * flat.size(), cudaMemcpyHostToDevice, dev->stream));
      const int32_t* d_off = (const int32_t*)p->q_conv.p;
      repetition_penalty_kernel<<<n, 256, 0, dev->stream>>>(prm.target_logits, (float*)p->layer_buf.p, V, d_off + n + 1, d_off,
                                                            a->repeat_penalty, a->frequency_penalty, a->presence_penalty);
      RELUX_CUDA_TRY(cudaGetLastError());
      count_launch(dev);
      prm.target_logits = (const float*)p->layer_buf.p;
    }
  }
  prm.k = 0;
  prm.vocab = V;
  std::vector<int32_t> host;
  rc = launch_selection(p, prm, n, a->sampler, a->mode, host);
  if (rc) return rc;
  for (int i = 0; i < n; i++) a->tokens[i] = host[(size_t)n + i];
  return RELUX_OK;
}

}  // namespace relux
