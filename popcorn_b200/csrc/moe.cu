// MoE token routing, permutation index, permute and weighted unpermute for sm_100a.
//
//   route      softmax over experts, top-k, renormalise        (momoe.py:47-49)
//   index      expert histogram, scan, stable permutation      (momoe_tl.py:1071-1161)
//   permute    rows[pos[t,k]] = x[t]    (one read, top_k writes per token row)
//   gather     out[p] = x[src[p]]
//   unpermute  y[t] = sum_k w[t,k] * rows[pos[t,k]], fp32, ascending expert order (momoe.py:52-53)
//
// Bound: HBM for permute / gather / unpermute (pure row traffic, 128-bit
// accesses, a warp moves 512 contiguous bytes per step); route and index move
// only a few MB and are latency-bound.
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTopK = 32;
constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------ route --

template <typename L>
__device__ __forceinline__ float logit_to_float(const L* p, int64_t i);
template <>
__device__ __forceinline__ float logit_to_float<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float logit_to_float<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <>
__device__ __forceinline__ float logit_to_float<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// Monotone map fp32 -> u32 (larger float, larger key); NaN maps to 0 and never wins.
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  if (v != v) return 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// One warp per token; lane l holds experts l, l + 32, ... (NPL of them) as
// order-preserving integer keys.  Each of the top_k rounds is two warp-wide
// integer reductions (redux.sync): the largest key, then the lowest expert index
// holding it.  Selection runs on the logits: exp and the shared softmax
// denominator are monotone, so this is the order of the probabilities, with ties
// going to the lower index.  The softmax denominator cancels in
// picked / sum(picked), so the weights are exp(l_k - l_top) / sum_j exp(l_j - l_top)
// over the picked logits.
template <typename L, int NPL>
__global__ void __launch_bounds__(256)
route_kernel(const L* __restrict__ logits, int32_t* __restrict__ indices, float* __restrict__ weights,
             int64_t tokens, int experts, int top_k, int64_t ld) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < tokens; t += warps) {
    uint32_t key[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      key[i] = e < experts ? order_key(logit_to_float<L>(logits, t * ld + e)) : 0u;
    }
    uint32_t taken = 0;  // bit i: my i-th expert is picked (or does not exist)
#pragma unroll
    for (int i = 0; i < NPL; ++i)
      if (lane + 32 * i >= experts) taken |= 1u << i;

    uint32_t my_key = 0;
    int my_idx = 0;
    for (int k = 0; k < top_k; ++k) {
      uint32_t best = 0;
      int best_i = -1;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const bool free_slot = !((taken >> i) & 1u);
        if (free_slot && (best_i < 0 || key[i] > best)) {
          best = key[i];
          best_i = i;
        }
      }
      const uint32_t top = __reduce_max_sync(kFull, best_i >= 0 ? best : 0u);
      const uint32_t cand = (best_i >= 0 && best == top) ? static_cast<uint32_t>(lane + 32 * best_i) : 0xffffffffu;
      const uint32_t who = __reduce_min_sync(kFull, cand);
      if (best_i >= 0 && cand == who) taken |= 1u << best_i;
      if (lane == k) {
        my_key = top;
        my_idx = static_cast<int>(who);
      }
    }
    const float top_logit = key_value(__shfl_sync(kFull, my_key, 0));
    const float p = lane < top_k ? expf(__fsub_rn(key_value(my_key), top_logit)) : 0.f;
    const float denom = warp_sum(p);
    if (lane < top_k) {
      indices[t * top_k + lane] = my_idx;
      weights[t * top_k + lane] = __fdiv_rn(p, denom);
    }
  }
}

// Up to 64 experts and top_k <= 8: FOUR lanes per token.  Each lane keeps a quarter of the token's logits as
// order-preserving integer keys in registers (expert 16 j + 4 q + c in slot 4 j + c of lane q, so that the four lanes
// of a token read 64 contiguous bytes with one 128-bit load each); a top-k round is a balanced tree of
// compare-and-select pairs over the lane's keys (no branches, left operand = lower index wins ties) and two butterfly
// shuffles over the quad, where equal keys go to the lower expert index.  Against the warp-per-token form above this
// is a quarter of the warp instructions per token and no warp-wide reduction; against one thread per token (tried:
// 25-61 us) the dependent chain per thread is a quarter as long and there are four times as many warps to hide it.
// Same arithmetic for the weights: exp(l_k - l_top) / sum_j exp(l_j - l_top) over the picked logits, in pick order.
constexpr int kQuadTopK = 8;

// The picks of token t as seen by lane q of its group of LPT lanes (a quad in the launched form): sel[k] / prob[k]
// (every lane of the group ends with the same values) and the sum of the picked probabilities.  Slot s of lane q holds
// expert 4 LPT (s / 4) + 4 q + s % 4.  All 32 lanes of the warp must call it together.
template <typename L, int KPL, int LPT>
__device__ __forceinline__ void route_quad_token(const L* __restrict__ logits, int64_t t, int q, int experts, int top_k,
                                                 int64_t ld, int vectorised, int (&sel)[kQuadTopK], float (&prob)[kQuadTopK],
                                                 float& denom) {
  uint32_t key[KPL];
  if (vectorised) {  // fp32 logits, rows and row pitch multiples of four: one 128-bit load per four slots
#pragma unroll
    for (int j = 0; j < KPL / 4; ++j) {
      const int e = 4 * LPT * j + 4 * q;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < experts) v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(logits) + t * ld + e));
      key[4 * j + 0] = e < experts ? order_key(v.x) : 0u;
      key[4 * j + 1] = e < experts ? order_key(v.y) : 0u;
      key[4 * j + 2] = e < experts ? order_key(v.z) : 0u;
      key[4 * j + 3] = e < experts ? order_key(v.w) : 0u;
    }
  } else {
#pragma unroll
    for (int s = 0; s < KPL; ++s) {
      const int e = 4 * LPT * (s >> 2) + 4 * q + (s & 3);
      key[s] = e < experts ? order_key(logit_to_float<L>(logits, t * ld + e)) : 0u;
    }
  }
  // NaN logits have key 0 and so has every expert already picked: a round whose best key is 0 has only those left
  // and takes the lowest index not picked yet (the bit mask), like the warp form.
  unsigned long long picked = 0;
  float top_logit = 0.f;
  denom = 0.f;
#pragma unroll
  for (int k = 0; k < kQuadTopK; ++k) {
    sel[k] = 0;
    prob[k] = 0.f;
    if (k < top_k) {
      uint32_t val[KPL / 2];
      int arg[KPL / 2];
#pragma unroll
      for (int i = 0; i < KPL / 2; ++i) {
        const bool right = key[2 * i + 1] > key[2 * i];
        val[i] = right ? key[2 * i + 1] : key[2 * i];
        arg[i] = right ? 2 * i + 1 : 2 * i;
      }
#pragma unroll
      for (int width = KPL / 4; width >= 1; width /= 2) {
#pragma unroll
        for (int i = 0; i < width; ++i) {
          const bool right = val[2 * i + 1] > val[2 * i];
          val[i] = right ? val[2 * i + 1] : val[2 * i];
          arg[i] = right ? arg[2 * i + 1] : arg[2 * i];
        }
      }
      uint32_t best = val[0];
      int who = 4 * LPT * (arg[0] >> 2) + 4 * q + (arg[0] & 3);
#pragma unroll
      for (int mask = 1; mask < LPT; mask <<= 1) {
        const uint32_t other = __shfl_xor_sync(kFull, best, mask);
        const int other_who = __shfl_xor_sync(kFull, who, mask);
        const bool take = other > best || (other == best && other_who < who);
        best = take ? other : best;
        who = take ? other_who : who;
      }
      if (best == 0) {
        who = 0;
        while (who < experts - 1 && ((picked >> who) & 1ull)) ++who;
      }
      picked |= 1ull << who;
      const int mine = who - 4 * q;  // slot s of this lane holds expert 16 (s / 4) + 4 q + s % 4
#pragma unroll
      for (int s = 0; s < KPL; ++s) key[s] = mine == 4 * LPT * (s >> 2) + (s & 3) ? 0u : key[s];
      const float logit = key_value(best);
      if (k == 0) top_logit = logit;
      const float p = expf(__fsub_rn(logit, top_logit));
      denom = k == 0 ? p : __fadd_rn(denom, p);
      sel[k] = who;
      prob[k] = p;
    }
  }
}

template <typename L, int KPL, int LPT>
__global__ void __launch_bounds__(256)
route_quad_kernel(const L* __restrict__ logits, int32_t* __restrict__ indices, float* __restrict__ weights,
                  int64_t tokens, int experts, int top_k, int64_t ld, int vectorised) {
  pdl_prologue();
  const int q = threadIdx.x & (LPT - 1);
  const int64_t token = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) / LPT;
  const bool live = token < tokens;  // whole quads; dead quads still take part in the shuffles
  const int64_t t = live ? token : tokens - 1;
  int sel[kQuadTopK];
  float prob[kQuadTopK];
  float denom;
  route_quad_token<L, KPL, LPT>(logits, t, q, experts, top_k, ld, vectorised, sel, prob, denom);
  if (live) {
#pragma unroll
    for (int k = 0; k < kQuadTopK; ++k) {
      if (k / (kQuadTopK / LPT) == q && k < top_k) {  // with four lanes, lane q stores picks 2 q and 2 q + 1
        indices[t * top_k + k] = sel[k];
        weights[t * top_k + k] = __fdiv_rn(prob[k], denom);
      }
    }
  }
}

// ------------------------------------------------------------------ index --

constexpr int kIndexThreads = 256;
constexpr int kPairsPerThread = 8;
constexpr int kPairsPerBlock = kIndexThreads * kPairsPerThread;  // 2048 (token, slot) pairs

// Step 1: per-block expert histogram -> block_hist[e * nblk + b].  Every warp counts its 256 consecutive pairs in a
// histogram of its own (with 64 experts a shared one sees 32 colliding updates per bin), read as two 128-bit words
// per lane where the block is complete; the eight histograms are added at the end.
__global__ void __launch_bounds__(kIndexThreads)
index_hist_kernel(const int32_t* __restrict__ idx, int64_t pairs, int experts, int nblk,
                  int32_t* __restrict__ block_hist) {
  pdl_prologue();
  extern __shared__ int hist[];  // [8 warps][experts]
  constexpr int kWarps = kIndexThreads / 32;
  for (int i = threadIdx.x; i < kWarps * experts; i += kIndexThreads) hist[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  int* mine = hist + (threadIdx.x >> 5) * experts;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kPairsPerBlock + (threadIdx.x >> 5) * (kPairsPerBlock / kWarps);
  if (base + kPairsPerBlock / kWarps <= pairs && (reinterpret_cast<uintptr_t>(idx) & 15) == 0) {
    const int4* words = reinterpret_cast<const int4*>(idx + base);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int4 v = words[r * 32 + lane];
      const int e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (e[j] >= 0 && e[j] < experts) atomicAdd(&mine[e[j]], 1);
    }
  } else {
#pragma unroll
    for (int r = 0; r < kPairsPerThread; ++r) {
      const int64_t i = base + r * 32 + lane;
      if (i < pairs) {
        const int e = idx[i];
        if (e >= 0 && e < experts) atomicAdd(&mine[e], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kIndexThreads) {
    int total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += hist[w * experts + e];
    block_hist[static_cast<int64_t>(e) * nblk + blockIdx.x] = total;
  }
}

// Step 2 (one CTA): per expert, exclusive scan of its block counts in place and
// its total; then the exclusive scan of the totals over experts.
__global__ void __launch_bounds__(1024)
index_scan_kernel(int32_t* __restrict__ block_hist, int experts, int nblk,
                  int32_t* __restrict__ counts, int32_t* __restrict__ offsets) {
  pdl_prologue();
  __shared__ int total[kMaxExperts];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int e = warp; e < experts; e += 32) {
    int32_t* h = block_hist + static_cast<int64_t>(e) * nblk;
    int running = 0;
    for (int b0 = 0; b0 < nblk; b0 += 32) {
      const int b = b0 + lane;
      const int c = b < nblk ? h[b] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += up;
      }
      if (b < nblk) h[b] = running + incl - c;
      running += __shfl_sync(kFull, incl, 31);
    }
    if (lane == 0) total[e] = running;
  }
  __syncthreads();
  // experts <= 1024: thread e owns expert e; scan 1024 slots through warp scans
  __shared__ int warp_tot[32];
  const int e = threadIdx.x;
  const int c = e < experts ? total[e] : 0;
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(kFull, wi, o);
      if (lane >= o) wi += up;
    }
    warp_tot[lane] = wi - w;  // exclusive
  }
  __syncthreads();
  const int excl = warp_tot[warp] + incl - c;
  if (e < experts) {
    counts[e] = c;
    offsets[e] = excl;
    if (e == experts - 1) offsets[experts] = excl + c;
  }
}

// Step 3: every pair gets offsets[e] + (pairs of e in earlier blocks) + (pairs of e
// earlier in this block).  A warp walks its 256 consecutive pairs 32 at a time;
// __match_any_sync ranks equal experts inside a step by lane, which is pair order.
__global__ void __launch_bounds__(kIndexThreads)
index_scatter_kernel(const int32_t* __restrict__ idx, int64_t pairs, int top_k, int experts, int nblk,
                     const int32_t* __restrict__ block_hist, const int32_t* __restrict__ offsets,
                     int32_t* __restrict__ perm_token, int32_t* __restrict__ pos) {
  pdl_prologue();
  extern __shared__ int whist[];  // [8 warps][experts]
  constexpr int kWarps = kIndexThreads / 32;
  constexpr int kPairsPerWarp = kPairsPerBlock / kWarps;  // 256
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kWarps * experts; i += kIndexThreads) whist[i] = 0;
  __syncthreads();
  const int64_t wbase = static_cast<int64_t>(blockIdx.x) * kPairsPerBlock + warp * kPairsPerWarp;
  int my_e[kPairsPerThread];
#pragma unroll
  for (int r = 0; r < kPairsPerThread; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    int e = -1;
    if (i < pairs) {
      e = idx[i];
      if (e < 0 || e >= experts) e = -1;
    }
    my_e[r] = e;
    if (e >= 0) atomicAdd(&whist[warp * experts + e], 1);
  }
  __syncthreads();
  // exclusive prefix over the warps of this block, seeded with the global base
  for (int e = threadIdx.x; e < experts; e += kIndexThreads) {
    int running = offsets[e] + block_hist[static_cast<int64_t>(e) * nblk + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = whist[w * experts + e];
      whist[w * experts + e] = running;
      running += c;
    }
  }
  __syncthreads();
  int* cursor = whist + warp * experts;
#pragma unroll
  for (int r = 0; r < kPairsPerThread; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    const int e = my_e[r];
    const unsigned same = __match_any_sync(kFull, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    const int leader = __ffs(same) - 1;  // advances the cursor for its group
    int base = 0;
    if (e >= 0 && lane == leader) base = atomicAdd(&cursor[e], __popc(same));
    base = __shfl_sync(kFull, base, leader);
    const int dst = e >= 0 ? base + rank : -1;
    if (i < pairs) {
      pos[i] = dst;
      if (dst >= 0 && perm_token != nullptr) perm_token[dst] = static_cast<int32_t>(static_cast<uint32_t>(i) / static_cast<uint32_t>(top_k));
    }
  }
}

// ------------------------------------------------ index in one launch --
//
// One cooperative launch of at most one CTA per SM replaces the three launches above, whose cost at MoE sizes is
// launch latency, not traffic.  CTA b owns a contiguous range of tokens and warp w of it a contiguous sub-range, so
// (CTA, warp, step, lane) order is pair order and the permutation stays stable:
//   1  each warp counts the experts of its pairs in a shared-memory histogram of its own;
//   2  the CTA turns the warp histograms into exclusive prefixes over its warps and publishes its per-expert totals;
//   3  grid rendezvous: every CTA stores a tag into a flag of its own; CTA 0 waits for all flags (one thread per
//      flag) and then stores the tag into one word that a single thread of every other CTA waits for.  All waits are
//      bounded.  The tag is a generation counter kept in the workspace and advanced by CTA 0 after the rendezvous,
//      so replaying the same launch (a CUDA graph) works and nothing has to be cleared between calls;
//   4  every CTA sums the published totals (pairs of each expert in earlier CTAs, and overall), scans the overall
//      counts over the experts, and ranks its own pairs with __match_any_sync like index_scatter_kernel.
// The cooperative launch attribute guarantees that all CTAs are resident together, which is what makes step 3 legal.
// If a wait runs out all the same, the kernel writes -1 into offsets[experts] and returns.
//
// Routing stays a launch of its own: fused in front of step 1 (tried) it runs at 32 warps per SM instead of 46 and
// the whole kernel took 33-35 us against 15 + 15 for the two launches; the routing is bound by the integer pipe
// (a compare-and-select tree per pick), not by its launch.
constexpr int kCoopThreads = 1024;
constexpr int kCoopWarps = kCoopThreads / 32;
constexpr int kCoopExperts = 256;
constexpr int kCoopMaxGrid = 256;   // CTAs (flags in the workspace header)
constexpr int kCoopGoWord = 1 + kCoopMaxGrid + 15;  // on a 128-byte line of its own behind the flags
constexpr size_t kCoopHeaderBytes = 8 * (kCoopMaxGrid + 64);  // generation word, one flag per CTA, the go word, spare
constexpr unsigned long long kCoopWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long coop_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Polls *word until it holds `tag`; false when `budget_ns` ran out first.
__device__ __forceinline__ bool coop_wait(const unsigned long long* word, unsigned long long tag, unsigned long long budget_ns) {
  const unsigned long long start = coop_timer();
  for (;;) {
    unsigned long long seen;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(word) : "memory");
    if (seen == tag) return true;
    if (coop_timer() - start > budget_ns) return false;
  }
}
__device__ __forceinline__ void coop_post(unsigned long long* word, unsigned long long tag) {
  __threadfence();
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(word), "l"(tag) : "memory");
}

// Exclusive scan of a[0 .. n) in place by ONE warp (n <= 32 * kPer); returns the total to every lane.
template <int kPer>
__device__ __forceinline__ int warp_exclusive_scan(int* a, int n, int lane) {
  const int per = (n + 31) / 32;  // lane l owns a[l * per .. l * per + per - 1]
  int c[kPer];
  int sum = 0;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane * per + i;
    c[i] = (i < per && e < n) ? a[e] : 0;
    sum += c[i];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += up;
  }
  int excl = incl - sum;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane * per + i;
    if (i < per && e < n) {
      a[e] = excl;
      excl += c[i];
    }
  }
  return __shfl_sync(kFull, incl, 31);
}

// Ranks the pairs [first, last) of one warp, 32 consecutive pairs per step: destination = base[e] + the warp's cursor
// + the number of lower lanes with the same expert.  The first lane of every group of equal experts advances the
// cursor with a shared-memory atomic and hands the old value to its group by shuffle.  pair numbers fit in 31 bits.
__device__ __forceinline__ void rank_pairs_by_match(const int32_t* __restrict__ indices, int first, int last, int experts, int top_k,
                                                    int lane, const int* base_of, int* cursor, int32_t* __restrict__ pos,
                                                    int32_t* __restrict__ perm_token) {
  const int shift = (top_k & (top_k - 1)) == 0 ? __ffs(top_k) - 1 : -1;
  int e_next = -1;
  if (first + lane < last) e_next = indices[first + lane];
#pragma unroll 1
  for (int i0 = first; i0 < last; i0 += 32) {
    const int i = i0 + lane;
    int e = e_next;
    if (e < 0 || e >= experts) e = -1;
    e_next = -1;
    if (i + 32 < last) e_next = indices[i + 32];
    const unsigned same = __match_any_sync(kFull, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    const int leader = __ffs(same) - 1;
    int base = 0;
    if (e >= 0 && lane == leader) base = atomicAdd(&cursor[e], __popc(same));
    base = __shfl_sync(kFull, base, leader);
    const int dst = e >= 0 ? base_of[e] + base + rank : -1;
    if (i < last) {
      pos[i] = dst;
      if (dst >= 0 && perm_token != nullptr)  // optional: one scattered 4-byte store per pair
        perm_token[dst] = shift >= 0 ? i >> shift : static_cast<int>(static_cast<unsigned>(i) / static_cast<unsigned>(top_k));
    }
  }
}

__global__ void __launch_bounds__(kCoopThreads, 1)
index_one_launch_kernel(const int32_t* __restrict__ indices, int64_t tokens, int experts, int top_k,
                        int64_t tokens_per_cta, int tokens_per_warp,
                        int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                        int32_t* __restrict__ perm_token, int32_t* __restrict__ pos,
                        unsigned long long* header, int32_t* grid_hist, unsigned long long budget_ns) {
  extern __shared__ int coop_smem[];
  int* whist = coop_smem;                            // [32 warps][experts]
  int* s_before = coop_smem + kCoopWarps * experts;  // [experts] pairs of the expert in earlier CTAs
  int* s_offset = s_before + experts;                // [experts] totals, then first destination of this CTA's pairs
  constexpr int kPer = kCoopExperts / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
#ifdef B200_COOP_STAMPS  // phase times of the last CTA into spare header words (a build for measuring only)
#define B200_STAMP(n) do { if (cta == grid - 1 && tid == 0) header[kCoopGoWord + 16 + (n)] = coop_timer(); } while (0)
#else
#define B200_STAMP(n) do { } while (0)
#endif
  B200_STAMP(0);
  for (int i = tid; i < kCoopWarps * experts; i += kCoopThreads) whist[i] = 0;
  // the generation this launch answers to; CTA 0 advances it only after every CTA has passed the rendezvous
  const unsigned long long tag = __ldcg(header) + 1ull;
  __syncthreads();

  const int64_t cta_begin = static_cast<int64_t>(cta) * tokens_per_cta;
  const int64_t cta_end = cta_begin + tokens_per_cta < tokens ? cta_begin + tokens_per_cta : tokens;
  int64_t warp_begin = cta_begin + static_cast<int64_t>(warp) * tokens_per_warp;
  if (warp_begin > cta_end) warp_begin = cta_end;
  const int64_t warp_end = warp_begin + tokens_per_warp < cta_end ? warp_begin + tokens_per_warp : cta_end;
  const int64_t pair_begin = warp_begin * top_k, pair_end = warp_end * top_k;
  int* mine = whist + warp * experts;

  for (int i = static_cast<int>(pair_begin) + lane; i < static_cast<int>(pair_end); i += 32) {  // tokens * top_k < 2^31
    const int e = indices[i];
    if (e >= 0 && e < experts) atomicAdd(&mine[e], 1);
  }
  __syncthreads();
  B200_STAMP(1);
  for (int e = tid; e < experts; e += kCoopThreads) {
    int running = 0;
#pragma unroll 4
    for (int w = 0; w < kCoopWarps; ++w) {
      const int c = whist[w * experts + e];
      whist[w * experts + e] = running;
      running += c;
    }
    __stcg(grid_hist + static_cast<int64_t>(e) * grid + cta, running);
  }
  __syncthreads();

  // ---- rendezvous of the whole grid
  B200_STAMP(2);
  unsigned long long* flags = header + 1;
  unsigned long long* go = header + kCoopGoWord;
  int gave_up = 0;
  if (cta != 0) {
    if (tid == 0) {
      coop_post(flags + cta, tag);
      gave_up = coop_wait(go, tag, budget_ns) ? 0 : 1;
    }
  } else if (tid > 0 && tid < grid) {
    gave_up = coop_wait(flags + tid, tag, budget_ns) ? 0 : 1;
  }
  if (__syncthreads_or(gave_up)) {  // CTA 0 never posts the go word then, so every CTA ends up here
    if (tid == 0) {
      offsets[experts] = -1;
      if (cta == 0) *header = tag;  // the flags of this launch must not satisfy the next one
    }
    return;
  }
  if (cta == 0 && tid == 0) coop_post(go, tag);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  B200_STAMP(3);

  // ---- pairs of every expert in earlier CTAs and overall; a warp takes experts w and w + 32 together
  for (int e0 = warp; e0 < experts; e0 += 2 * kCoopWarps) {
    const int e1 = e0 + kCoopWarps;
    int before0 = 0, total0 = 0, before1 = 0, total1 = 0;
    for (int g = lane; g < grid; g += 32) {
      const int c0 = __ldcg(grid_hist + static_cast<int64_t>(e0) * grid + g);
      const int c1 = e1 < experts ? __ldcg(grid_hist + static_cast<int64_t>(e1) * grid + g) : 0;
      total0 += c0;
      total1 += c1;
      before0 += g < cta ? c0 : 0;
      before1 += g < cta ? c1 : 0;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
      before0 += __shfl_xor_sync(kFull, before0, o);
      total0 += __shfl_xor_sync(kFull, total0, o);
      before1 += __shfl_xor_sync(kFull, before1, o);
      total1 += __shfl_xor_sync(kFull, total1, o);
    }
    if (lane == 0) {
      s_before[e0] = before0;
      s_offset[e0] = total0;
      if (e1 < experts) {
        s_before[e1] = before1;
        s_offset[e1] = total1;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    if (cta == 0)
      for (int e = lane; e < experts; e += 32) counts[e] = s_offset[e];
    __syncwarp();  // the scan's lanes own other entries than the loops around it
    const int all = warp_exclusive_scan<kPer>(s_offset, experts, lane);
    __syncwarp();
    if (cta == 0) {
      for (int e = lane; e < experts; e += 32) offsets[e] = s_offset[e];
      if (lane == 0) {
        offsets[experts] = all;
        *header = tag;  // every CTA read the old generation before it posted its flag
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < experts; e += kCoopThreads) s_offset[e] += s_before[e];
  __syncthreads();

  // ---- rank this warp's pairs: destination = first destination of this CTA's pairs of the expert + earlier warps of
  // this CTA (the cursor in `mine`) + rank inside the step
  B200_STAMP(4);
  // (Tried instead of the match: seven votes, one per bit of the expert number - the same time; one token per lane
  // with per-expert token masks built by shared-memory atomicOr - 2.7 instead of 3.8 us for this phase at 3544 pairs per
  // SM when the permutation is not stored, but 2 us slower on small inputs, whose time is the length of the dependent
  // chain; staging the permutation in shared memory to store it in runs - slower.)
  rank_pairs_by_match(indices, static_cast<int>(pair_begin), static_cast<int>(pair_end), experts, top_k, lane, s_offset, mine, pos, perm_token);
#ifdef B200_COOP_STAMPS
  __syncthreads();
  B200_STAMP(5);
#endif
#undef B200_STAMP
}

// ---------------------------------------------------- permute / gather --

// Word types for pure row copies: the widest one every address is aligned to.
template <typename W>
__device__ __forceinline__ W ld_word(const W* p) { return *p; }
template <>
__device__ __forceinline__ uint4 ld_word<uint4>(const uint4* p) { return ld_stream(p); }
template <typename W>
__device__ __forceinline__ void st_word(W* p, const W& v) { *p = v; }
template <>
__device__ __forceinline__ void st_word<uint4>(uint4* p, const uint4& v) { st_stream(p, v); }

// Destination / source buffers of the multi-buffer forms: buffer 0 is this GPU's
// own memory in the single-GPU entry points; in the expert-parallel ones entry r is
// rank r's exchange buffer, mapped into this process (peer memory over NVLink).
constexpr int kMaxBuffers = 16;
struct BufferTable {
  void* base[kMaxBuffers];
};
// base[i] for a run-time i.  A dynamically indexed kernel parameter would be copied to
// per-thread local memory (128 bytes per thread); a chain of selects on constant indices
// keeps the table in the parameter bank.
__device__ __forceinline__ void* table_entry(const BufferTable& table, int i) {
  void* p = table.base[0];
#pragma unroll
  for (int k = 1; k < kMaxBuffers; ++k)
    if (i == k) p = table.base[k];
  return p;
}

// One warp per token: read the row once (UNROLL words per lane at a time) and
// write it to each of its top_k destinations (buffer dst_buf[t,k], row pos[t,k];
// dst_buf == nullptr means buffer 0).  Loop bounds are the same for all lanes of
// a warp, because the destinations travel by shuffle.  With peer buffers in the
// table this kernel IS the dispatch half of the expert-parallel exchange: each row
// goes from local HBM straight into the owning rank's memory with ordinary
// 128-bit stores, with no staging copy and no separate collective.
template <typename W, int UNROLL>
__global__ void __launch_bounds__(256)
permute_kernel(const W* __restrict__ x, const int32_t* __restrict__ pos, const int32_t* __restrict__ dst_buf,
               const BufferTable bufs, int64_t tokens, int top_k, int words, int64_t ldx, int64_t ldrows) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (t >= tokens) return;  // whole warps leave together
  int my_dst = -1, my_buf = 0;
  if (lane < top_k) {
    my_dst = pos[t * top_k + lane];
    if (dst_buf != nullptr) my_buf = dst_buf[t * top_k + lane];
  }
  // destination row address of slot `lane`
  W* my_out = my_dst >= 0 ? static_cast<W*>(table_entry(bufs, my_buf)) + static_cast<int64_t>(my_dst) * ldrows : nullptr;
  const W* src = x + t * ldx;
  for (int w0 = 0; w0 < words; w0 += 32 * UNROLL) {
    W v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (w0 + lane + 32 * u < words) v[u] = ld_word<W>(src + w0 + lane + 32 * u);
    for (int k = 0; k < top_k; ++k) {
      W* out = reinterpret_cast<W*>(__shfl_sync(kFull, reinterpret_cast<unsigned long long>(my_out), k));
      if (out == nullptr) continue;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (w0 + lane + 32 * u < words) st_word<W>(out + w0 + lane + 32 * u, v[u]);
    }
  }
}

// The same for rows made of whole 8 KiB pieces that are 32-byte aligned: 256-bit accesses (half the memory
// instructions) and sixteen tokens per CTA.  On 8 KiB rows with eight destinations: 0.736 ms against 0.749 ms for the
// form above.  Neither form is limited by how it issues its accesses: a fan-out copy that reads one row per eight
// written tops out at 6.4-6.7 TB/s on this part even with ideal (sequential) destinations, while the same stores
// without the loads reach 7.4 TB/s; the reads interrupt the write drains of the memory controller.
__global__ void __launch_bounds__(512)
permute_wide_kernel(const Word256* __restrict__ x, const int32_t* __restrict__ pos, const int32_t* __restrict__ dst_buf,
                    const BufferTable bufs, int64_t tokens, int top_k, int words, int64_t ldx, int64_t ldrows) {
  pdl_prologue();
  constexpr int UNROLL = 8;
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 16 + (threadIdx.x >> 5);
  if (t >= tokens) return;  // whole warps leave together
  int my_dst = -1, my_buf = 0;
  if (lane < top_k) {
    my_dst = pos[t * top_k + lane];
    if (dst_buf != nullptr) my_buf = dst_buf[t * top_k + lane];
  }
  Word256* my_out = my_dst >= 0 ? static_cast<Word256*>(table_entry(bufs, my_buf)) + static_cast<int64_t>(my_dst) * ldrows : nullptr;
  const Word256* src = x + t * ldx;
  for (int w0 = 0; w0 < words; w0 += 32 * UNROLL) {
    Word256 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ld_stream256(src + w0 + lane + 32 * u);
    for (int k = 0; k < top_k; ++k) {
      Word256* out = reinterpret_cast<Word256*>(__shfl_sync(kFull, reinterpret_cast<unsigned long long>(my_out), k));
      if (out == nullptr) continue;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) st_stream256(out + w0 + lane + 32 * u, v[u]);
    }
  }
}

// One warp per output row.
template <typename W>
__global__ void __launch_bounds__(256)
gather_kernel(const W* __restrict__ x, const int32_t* __restrict__ src_row, W* __restrict__ out,
              int64_t n_rows, int words, int64_t ldx, int64_t ldo) {
  pdl_prologue();
  constexpr int UNROLL = 8;
  const int lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int s = src_row[r];
  if (s < 0) return;
  const W* src = x + static_cast<int64_t>(s) * ldx;
  W* dst = out + r * ldo;
  for (int w0 = lane; w0 < words; w0 += 32 * UNROLL) {
    W v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (w0 + 32 * u < words) v[u] = ld_word<W>(src + w0 + 32 * u);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (w0 + 32 * u < words) st_word<W>(dst + w0 + 32 * u, v[u]);
  }
}

// -------------------------------------------------------------- unpermute --

// One warp per token.  Lanes < top_k hold (buffer, pos, weight); the slots are
// visited in ascending (buffer, pos), which is ascending expert index.  The sorted
// row addresses and weights sit in shared memory (one line per warp).  With peer
// buffers in the table this kernel IS the combine half of the expert-parallel
// exchange: the token's owner reads the expert outputs straight out of the other
// ranks' memory with ordinary 128-bit loads while it accumulates.  Rows are fetched eight at a
// time, one 128-bit word per lane, and the NEXT batch of eight is already in
// flight while the current one is accumulated.  VEC: 128-bit words.
template <typename T, bool VEC, int WB>
__global__ void __launch_bounds__(256, 2)
unpermute_kernel(const BufferTable bufs, const int32_t* __restrict__ src_buf, const float* __restrict__ weights,
                 const int32_t* __restrict__ pos, T* __restrict__ y, int64_t tokens, int top_k, int hidden,
                 int64_t ldrows, int64_t ldy) {
  pdl_prologue();
  constexpr int V = VEC ? Num<T>::kVec : 1;
  constexpr int KB = 8;  // rows fetched together
  using Word = typename std::conditional<VEC, uint4, T>::type;
  __shared__ int64_t s_off[8][kMaxTopK];
  __shared__ float s_w[8][kMaxTopK];
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + wid;
  if (t >= tokens) return;  // whole warps leave together; no block-wide barrier below
  int my_pos = -1, my_buf = 0;
  float my_w = 0.f;
  if (lane < top_k) {
    my_pos = pos[t * top_k + lane];
    my_w = weights[t * top_k + lane];
    if (src_buf != nullptr) my_buf = src_buf[t * top_k + lane];
  }
  // rank of my slot among the valid ones, by (buffer, row); equal keys keep slot order.
  // Buffers hold contiguous expert blocks in rank order, so this is ascending expert index.
  int rank = 0;
  int valid = 0;
  for (int j = 0; j < top_k; ++j) {
    const int pj = __shfl_sync(kFull, my_pos, j);
    const int bj = __shfl_sync(kFull, my_buf, j);
    if (pj >= 0) {
      ++valid;
      if (bj < my_buf || (bj == my_buf && (pj < my_pos || (pj == my_pos && j < lane)))) ++rank;
    }
  }
  if (my_pos >= 0) {
    // absolute byte address of the row
    s_off[wid][rank] = reinterpret_cast<int64_t>(table_entry(bufs, my_buf)) + static_cast<int64_t>(my_pos) * ldrows * static_cast<int64_t>(sizeof(T));
    s_w[wid][rank] = my_w;
  }
  __syncwarp();

  // One batch = RB rows x WB words per lane (RB * WB = 8 loads in flight per lane per batch):
  // each row contributes WB * 512 contiguous bytes per warp, which keeps DRAM pages open longer
  // than eight 512-byte pieces of eight different rows.
  constexpr int RB = KB / WB;
  const int words = hidden / V;
  const int steps = (words + 32 * WB - 1) / (32 * WB);
  const int nb = (valid + RB - 1) / RB;
  const int total = steps * nb;
  T* out = y + t * ldy;
  float acc[WB][V];

  auto fetch = [&](Word (&buf)[KB], int item) {
    const int step = nb == 1 ? item : item / nb;
    const int b = item - step * nb;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int kk = b * RB + r;
#pragma unroll
      for (int j = 0; j < WB; ++j) {
        const int w = (step * WB + j) * 32 + lane;
        if (kk < valid && w < words) {
          const T* src = reinterpret_cast<const T*>(s_off[wid][kk]) + static_cast<int64_t>(w) * V;
          if constexpr (VEC) buf[r * WB + j] = ld_stream(src);
          else buf[r * WB + j] = *src;
        }
      }
    }
  };
  auto reduce = [&](const Word (&buf)[KB], int item) {
    const int step = nb == 1 ? item : item / nb;
    const int b = item - step * nb;
    if (b == 0) {
#pragma unroll
      for (int j = 0; j < WB; ++j)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[j][e] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int kk = b * RB + r;
      if (kk < valid) {
        const float ww = s_w[wid][kk];
#pragma unroll
        for (int j = 0; j < WB; ++j) {
          const int w = (step * WB + j) * 32 + lane;
          if (w < words) {
            if constexpr (VEC) {
              float f[V];
              Num<T>::unpack(buf[r * WB + j], f);
#pragma unroll
              for (int e = 0; e < V; ++e) acc[j][e] = __fadd_rn(acc[j][e], __fmul_rn(ww, f[e]));
            } else {
              acc[j][0] = __fadd_rn(acc[j][0], __fmul_rn(ww, Num<T>::up(buf[r * WB + j])));
            }
          }
        }
      }
    }
    if (b == nb - 1) {
#pragma unroll
      for (int j = 0; j < WB; ++j) {
        const int w = (step * WB + j) * 32 + lane;
        if (w < words) {
          if constexpr (VEC) st_stream(out + static_cast<int64_t>(w) * V, Num<T>::pack(acc[j]));
          else out[w] = Num<T>::down(acc[j][0]);
        }
      }
    }
  };

  if (valid == 0) {  // no valid slot: the row is zero
    for (int w = lane; w < words; w += 32) {
#pragma unroll
      for (int e = 0; e < V; ++e) acc[0][e] = 0.f;
      if constexpr (VEC) st_stream(out + static_cast<int64_t>(w) * V, Num<T>::pack(acc[0]));
      else out[w] = Num<T>::down(0.f);
    }
    return;
  }
  Word a[KB], b[KB];
  fetch(a, 0);
  for (int i = 0; i < total; i += 2) {
    if (i + 1 < total) fetch(b, i + 1);
    reduce(a, i);
    if (i + 1 < total) {
      if (i + 2 < total) fetch(a, i + 2);
      reduce(b, i + 1);
    }
  }
}

// The fast form of the kernel above for top_k <= 8 and rows made of whole 1 KiB pieces, everything 32-byte aligned:
// 256-bit loads, one batch = one 32-byte word of every slot's row (up to eight loads of 32 bytes in flight per lane,
// the next batch already issued), four tokens per CTA and three CTAs per SM.
// Same arithmetic in the same order: fp32 products and sums rounded separately, slots in ascending (buffer, row).
// On 8 KiB bf16 rows with eight slots: 0.674 ms = 7.17 TB/s against 0.762 ms for the general form (the slimmer loop
// alone is worth 0.706 ms; 256-bit loads at twelve resident warps the rest).
constexpr int kWideSlots = 8;
template <typename T>
__global__ void __launch_bounds__(128, 3)
unpermute_wide_kernel(const BufferTable bufs, const int32_t* __restrict__ src_buf, const float* __restrict__ weights,
                      const int32_t* __restrict__ pos, T* __restrict__ y, int64_t tokens, int top_k, int steps,
                      int64_t ldrows, int64_t ldy) {
  pdl_prologue();
  constexpr int V = Num<T>::kVec;  // elements per 128-bit half
  __shared__ int64_t s_off[4][kWideSlots];
  __shared__ float s_w[4][kWideSlots];
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 4 + wid;
  if (t >= tokens) return;  // whole warps leave together; no block-wide barrier below
  int my_pos = -1, my_buf = 0;
  float my_w = 0.f;
  if (lane < top_k) {
    my_pos = pos[t * top_k + lane];
    my_w = weights[t * top_k + lane];
    if (src_buf != nullptr) my_buf = src_buf[t * top_k + lane];
  }
  int rank = 0, valid = 0;
  for (int j = 0; j < top_k; ++j) {
    const int pj = __shfl_sync(kFull, my_pos, j);
    const int bj = __shfl_sync(kFull, my_buf, j);
    if (pj >= 0) {
      ++valid;
      if (bj < my_buf || (bj == my_buf && (pj < my_pos || (pj == my_pos && j < lane)))) ++rank;
    }
  }
  if (my_pos >= 0) {
    s_off[wid][rank] = reinterpret_cast<int64_t>(table_entry(bufs, my_buf)) + static_cast<int64_t>(my_pos) * ldrows * static_cast<int64_t>(sizeof(T));
    s_w[wid][rank] = my_w;
  }
  __syncwarp();
  float w[kWideSlots];
#pragma unroll
  for (int k = 0; k < kWideSlots; ++k) w[k] = k < valid ? s_w[wid][k] : 0.f;
  char* out = reinterpret_cast<char*>(y + t * ldy) + lane * 32;

  // the row addresses stay in shared memory (one broadcast read per load) rather than in sixteen registers
  auto fetch = [&](Word256 (&buf)[kWideSlots], int step) {
    const int64_t at = static_cast<int64_t>(step) * 1024 + lane * 32;
#pragma unroll
    for (int k = 0; k < kWideSlots; ++k)
      if (k < valid) buf[k] = ld_stream256(reinterpret_cast<const char*>(s_off[wid][k]) + at);
  };
  auto reduce = [&](const Word256 (&buf)[kWideSlots], int step) {
    float lo[V], hi[V];
#pragma unroll
    for (int e = 0; e < V; ++e) lo[e] = hi[e] = 0.f;
#pragma unroll
    for (int k = 0; k < kWideSlots; ++k) {
      if (k < valid) {
        float f[V];
        Num<T>::unpack(buf[k].lo, f);
#pragma unroll
        for (int e = 0; e < V; ++e) lo[e] = __fadd_rn(lo[e], __fmul_rn(w[k], f[e]));
        Num<T>::unpack(buf[k].hi, f);
#pragma unroll
        for (int e = 0; e < V; ++e) hi[e] = __fadd_rn(hi[e], __fmul_rn(w[k], f[e]));
      }
    }
    Word256 o;
    o.lo = Num<T>::pack(lo);
    o.hi = Num<T>::pack(hi);
    st_stream256(out + static_cast<int64_t>(step) * 1024, o);
  };
  Word256 a[kWideSlots], b[kWideSlots];
  fetch(a, 0);
  for (int i = 0; i < steps; i += 2) {
    if (i + 1 < steps) fetch(b, i + 1);
    reduce(a, i);
    if (i + 1 < steps) {
      if (i + 2 < steps) fetch(a, i + 2);
      reduce(b, i + 1);
    }
  }
}

template <typename W>
bool rows_aligned(const void* a, const void* b, int64_t row_bytes, int64_t lda_bytes, int64_t ldb_bytes) {
  return aligned(a, sizeof(W)) && aligned(b, sizeof(W)) && row_bytes % sizeof(W) == 0 && lda_bytes % sizeof(W) == 0 &&
         ldb_bytes % sizeof(W) == 0;
}

int nblk_for(int64_t pairs) { return static_cast<int>(ceil_div(pairs, kPairsPerBlock)); }

// Workspace of the index entry points: a header (generation word and per-CTA flags of the one-launch kernel), then the
// histogram table of whichever kernels run: [experts][CTAs] for the one-launch kernel, [experts][blocks of 2048 pairs]
// for the three-kernel chain.
int64_t coop_grid_bound(int64_t tokens) {
  const int64_t want = ceil_div(tokens, 64);
  return want < 1 ? 1 : (want > kCoopMaxGrid ? kCoopMaxGrid : want);
}
size_t index_scratch_need(int64_t tokens, int64_t top_k, int64_t experts) {
  const int64_t nblk = nblk_for(tokens * top_k);
  const int64_t floor_cols = experts <= kCoopExperts ? coop_grid_bound(tokens) : 1;
  const int64_t cols = nblk > floor_cols ? nblk : floor_cols;
  return kCoopHeaderBytes + static_cast<size_t>(cols * experts) * sizeof(int32_t);
}

// Whether the current device can run the one-launch kernel (cooperative launch, one CTA of 1024 threads per SM).
int g_coop_state[64] = {};  // per device: 0 not looked at yet, 1 usable, -1 not usable (or a launch did not fit once)
bool coop_supported() {
  int* cached = g_coop_state;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return false;
  }
  if (cached[dev] == 0) {
    int flag = 0;
    const bool ok = cudaDeviceGetAttribute(&flag, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && flag != 0;
    (void)cudaGetLastError();
    cached[dev] = ok ? 1 : -1;
  }
  return cached[dev] > 0;
}

template <typename... Params, typename... Args>
cudaError_t launch_cooperative(void (*kernel)(Params...), unsigned grid, unsigned block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(block);
  config.dynamicSmemBytes = smem;
  config.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// B200_INDEX_CHAIN=1 in the environment keeps the separate route / histogram / scan / scatter launches (read at every
// call: a getenv is a few tens of nanoseconds).
bool one_launch_index(int64_t experts) {
  const char* v = std::getenv("B200_INDEX_CHAIN");
  if (v != nullptr && v[0] == '1') return false;
  return experts <= kCoopExperts && coop_supported();
}

// The index as one cooperative launch.  The caller has checked shapes and pointers.  Returns kCoopDoesNotFit (and
// launches nothing) when the device cannot hold the grid at once, e.g. because part of its SMs is reserved for another
// client: the caller then runs the three-kernel chain, and so do later calls on that device.
constexpr int kCoopDoesNotFit = -1;
int launch_index_one(const int32_t* indices, int64_t tokens, int E, int K, int32_t* counts, int32_t* offsets,
                     int32_t* perm_token, int32_t* pos, void* scratch, cudaStream_t st) {
  int64_t grid = coop_grid_bound(tokens);
  if (grid > sm_count()) grid = sm_count();
  const int64_t tokens_per_cta = ceil_div(tokens > 0 ? tokens : 1, grid);
  const int tokens_per_warp = static_cast<int>(ceil_div(tokens_per_cta, kCoopWarps));
  unsigned long long* header = static_cast<unsigned long long*>(scratch);
  int32_t* grid_hist = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + kCoopHeaderBytes);
  const size_t smem = static_cast<size_t>(kCoopWarps + 2) * E * sizeof(int);  // at most 34 KiB
  const cudaError_t err = launch_cooperative(index_one_launch_kernel, static_cast<unsigned>(grid), kCoopThreads, smem, st, indices, tokens, E,
                                             K, tokens_per_cta, tokens_per_warp, counts, offsets, perm_token, pos, header, grid_hist, kCoopWaitNs);
  if (err == cudaErrorCooperativeLaunchTooLarge || err == cudaErrorLaunchOutOfResources || err == cudaErrorNotSupported) {
    (void)cudaGetLastError();
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) g_coop_state[dev] = -1;
    return kCoopDoesNotFit;
  }
  return after_launch("index_one_launch_kernel");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route(const void* logits, int32_t* indices, float* weights,
                              int64_t tokens, int64_t experts, int64_t top_k, int64_t ld_logits,
                              int logits_dtype, void* stream) {
  if (!dtype_ok(logits_dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported logits dtype %d", __func__, logits_dtype);
  if (tokens < 0 || experts < 1 || experts > kMaxExperts)
    return fail(B200_ERR_SHAPE, "%s: need tokens >= 0 and 1 <= experts <= %d (got %lld, %lld)", __func__, kMaxExperts, (long long)tokens, (long long)experts);
  if (top_k < 1 || top_k > experts || top_k > kMaxTopK)
    return fail(B200_ERR_SHAPE, "%s: need 1 <= top_k <= min(experts, %d) (got %lld)", __func__, kMaxTopK, (long long)top_k);
  if (ld_logits < experts) return fail(B200_ERR_SHAPE, "%s: ld_logits smaller than experts", __func__);
  if (tokens == 0) return B200_OK;
  B200_REQUIRE_PTR(logits);
  B200_REQUIRE_PTR(indices);
  B200_REQUIRE_PTR(weights);
  if (!aligned(logits, dtype_size(logits_dtype)) || !aligned(indices, 4) || !aligned(weights, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = static_cast<int>(experts), K = static_cast<int>(top_k);
  if (E <= 64 && K <= kQuadTopK) {
    // Four lanes per token.  (Two lanes with 16 / 32 keys each execute fewer instructions per token but run at 64
    // registers and 32 warps per SM: 14.9-15.2 us for 65536 tokens against 14.9, and 1-1.5 us slower below 16384 tokens.)
    const unsigned blocks = static_cast<unsigned>(ceil_div(tokens, 64));
    const int vec = logits_dtype == B200_F32 && E % 4 == 0 && ld_logits % 4 == 0 && aligned(logits, 16);
#define B200_ROUTE_QUAD(L)                                                                                             \
  do {                                                                                                                 \
    if (E <= 32) launch(route_quad_kernel<L, 8, 4>, blocks, 256, 0, st, static_cast<const L*>(logits), indices, weights, tokens, E, K, ld_logits, vec); \
    else launch(route_quad_kernel<L, 16, 4>, blocks, 256, 0, st, static_cast<const L*>(logits), indices, weights, tokens, E, K, ld_logits, vec);       \
  } while (0)
    if (logits_dtype == B200_F32) B200_ROUTE_QUAD(float);
    else if (logits_dtype == B200_F16) B200_ROUTE_QUAD(__half);
    else B200_ROUTE_QUAD(__nv_bfloat16);
#undef B200_ROUTE_QUAD
    return after_launch("route_quad_kernel");
  }
  const int64_t want = ceil_div(tokens, 8);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 64;
  const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
#define B200_ROUTE(L, NPL) \
  launch(route_kernel<L, NPL>, grid, 256, 0, st, static_cast<const L*>(logits), indices, weights, tokens, E, K, ld_logits)
#define B200_ROUTE_NPL(L)                  \
  do {                                     \
    if (E <= 32) B200_ROUTE(L, 1);         \
    else if (E <= 64) B200_ROUTE(L, 2);    \
    else if (E <= 128) B200_ROUTE(L, 4);   \
    else if (E <= 256) B200_ROUTE(L, 8);   \
    else if (E <= 512) B200_ROUTE(L, 16);  \
    else B200_ROUTE(L, 32);                \
  } while (0)
  if (logits_dtype == B200_F32) B200_ROUTE_NPL(float);
  else if (logits_dtype == B200_F16) B200_ROUTE_NPL(__half);
  else B200_ROUTE_NPL(__nv_bfloat16);
#undef B200_ROUTE_NPL
#undef B200_ROUTE
  return after_launch("route_kernel");
}

static int index_check(const char* fn, int64_t tokens, int64_t top_k, int64_t experts) {
  if (tokens < 0 || top_k < 1 || experts < 1 || experts > kMaxExperts)
    return fail(B200_ERR_SHAPE, "%s: need tokens >= 0, top_k >= 1, 1 <= experts <= %d", fn, kMaxExperts);
  if (tokens * top_k >= 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: tokens*top_k must be below 2^31", fn);
  return B200_OK;
}

extern "C" int b200_moe_index_scratch_bytes(int64_t tokens, int64_t top_k, int64_t experts, size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  if (int rc = index_check(__func__, tokens, top_k, experts)) return rc;
  *bytes = index_scratch_need(tokens, top_k, experts);
  return B200_OK;
}

extern "C" int b200_moe_index(const int32_t* indices, int64_t tokens, int64_t top_k, int64_t experts,
                              int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                              void* scratch, size_t scratch_bytes, void* stream) {
  if (int rc = index_check(__func__, tokens, top_k, experts)) return rc;
  B200_REQUIRE_PTR(counts);
  B200_REQUIRE_PTR(offsets);
  B200_REQUIRE_PTR(scratch);
  const int64_t pairs = tokens * top_k;
  if (pairs > 0) {
    B200_REQUIRE_PTR(indices);
    B200_REQUIRE_PTR(pos);
  }
  const int nblk = nblk_for(pairs);
  const size_t need = index_scratch_need(tokens, top_k, experts);
  if (scratch_bytes < need || !aligned(scratch, 16))
    return fail(B200_ERR_SCRATCH, "%s: scratch needs %zu bytes, 16-byte aligned (got %zu)", __func__, need, scratch_bytes);
  if (!aligned(indices, 4) || !aligned(counts, 4) || !aligned(offsets, 4) || !aligned(perm_token, 4) || !aligned(pos, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to 4 bytes", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = static_cast<int>(experts);
  if (one_launch_index(experts)) {
    const int rc = launch_index_one(indices, tokens, E, static_cast<int>(top_k), counts, offsets, perm_token, pos, scratch, st);
    if (rc != kCoopDoesNotFit) return rc;
  }
  int32_t* block_hist = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + kCoopHeaderBytes);
  if (nblk > 0) {
    launch(index_hist_kernel, nblk, kIndexThreads, 8 * E * sizeof(int), st, indices, pairs, E, nblk, block_hist);
    if (int rc = after_launch("index_hist_kernel")) return rc;
  }
  launch(index_scan_kernel, 1, 1024, 0, st, block_hist, E, nblk, counts, offsets);
  if (int rc = after_launch("index_scan_kernel")) return rc;
  if (nblk > 0) {
    launch(index_scatter_kernel, nblk, kIndexThreads, 8 * E * sizeof(int), st,
        indices, pairs, static_cast<int>(top_k), E, nblk, block_hist, offsets, perm_token, pos);
    if (int rc = after_launch("index_scatter_kernel")) return rc;
  }
  return B200_OK;
}

// Routing and the index in one call: b200_moe_route, then b200_moe_index on its picks (two or four kernel launches).
extern "C" int b200_moe_route_index(const void* logits, int32_t* indices, float* weights,
                                    int64_t tokens, int64_t experts, int64_t top_k, int64_t ld_logits, int logits_dtype,
                                    int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                                    void* scratch, size_t scratch_bytes, void* stream) {
  if (int rc = index_check(__func__, tokens, top_k, experts)) return rc;
  B200_REQUIRE_PTR(scratch);
  if (scratch_bytes < index_scratch_need(tokens, top_k, experts) || !aligned(scratch, 16))  // before anything is launched
    return fail(B200_ERR_SCRATCH, "%s: scratch needs %zu bytes, 16-byte aligned (got %zu)", __func__,
                index_scratch_need(tokens, top_k, experts), scratch_bytes);
  if (int rc = b200_moe_route(logits, indices, weights, tokens, experts, top_k, ld_logits, logits_dtype, stream)) return rc;
  return b200_moe_index(indices, tokens, top_k, experts, counts, offsets, perm_token, pos, scratch, scratch_bytes, stream);
}

// ------------------------------------------------- index without a workspace --

namespace b200 {
namespace {
// Scratch of b200_moe_index_static: the per-block expert histogram, kept in the
// library image instead of being passed in.  1 MiB per GPU that loads the library,
// held until the process exits.  On the host this name is only a stand-in for the
// symbol; the device address comes from cudaGetSymbolAddress, once per device.
constexpr size_t kStaticScratchBytes = size_t{1} << 20;
static __device__ __align__(256) unsigned char g_index_scratch[kCoopHeaderBytes + kStaticScratchBytes];

constexpr int kMaxDevicesStatic = 64;
std::mutex g_static_mutex;
void* g_static_address[kMaxDevicesStatic] = {};  // per device, filled on that device's first call

// Device address of g_index_scratch on the CURRENT device (looked up on the first call per device).
int static_scratch(void** address) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevicesStatic) {
    (void)cudaGetLastError();
    return fail(B200_ERR_DEVICE, "b200_moe_index_static: no usable CUDA device is current");
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_address[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_index_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return fail(B200_ERR_SCRATCH, "b200_moe_index_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
    }
    g_static_address[dev] = ptr;
  }
  *address = g_static_address[dev];
  return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_index_static_max_bytes(size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  *bytes = kStaticScratchBytes;
  return B200_OK;
}

extern "C" int b200_moe_index_static(const int32_t* indices, int64_t tokens, int64_t top_k, int64_t experts,
                                     int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                                     void* stream) {
  if (int rc = index_check(__func__, tokens, top_k, experts)) return rc;
  B200_REQUIRE_PTR(counts);
  B200_REQUIRE_PTR(offsets);
  const int64_t pairs = tokens * top_k;
  if (pairs > 0) {
    B200_REQUIRE_PTR(indices);
    B200_REQUIRE_PTR(pos);
  }
  const int nblk = nblk_for(pairs);
  const size_t need = index_scratch_need(tokens, top_k, experts);
  if (need - kCoopHeaderBytes > kStaticScratchBytes)
    return fail(B200_ERR_SCRATCH,
                "%s: tokens*top_k=%lld with %lld experts needs %zu bytes of scratch, over the built-in %zu; "
                "use b200_moe_index with a caller-provided workspace",
                __func__, (long long)pairs, (long long)experts, need - kCoopHeaderBytes, kStaticScratchBytes);
  if (!aligned(indices, 4) || !aligned(counts, 4) || !aligned(offsets, 4) || !aligned(perm_token, 4) || !aligned(pos, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to 4 bytes", __func__);
  if (int rc = check_device()) return rc;
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = static_cast<int>(experts);
  // The histogram kernels write every entry the later steps read, and the one-launch kernel's generation word only has
  // to differ from its flags' last value, so nothing left over from an earlier call has to be cleared first.
  if (one_launch_index(experts)) {
    const int rc = launch_index_one(indices, tokens, E, static_cast<int>(top_k), counts, offsets, perm_token, pos, scratch, st);
    if (rc != kCoopDoesNotFit) return rc;
  }
  int32_t* block_hist = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + kCoopHeaderBytes);
  if (nblk > 0) {
    launch(index_hist_kernel, nblk, kIndexThreads, 8 * E * sizeof(int), st, indices, pairs, E, nblk, block_hist);
    if (int rc = after_launch("index_hist_kernel")) return rc;
  }
  launch(index_scan_kernel, 1, 1024, 0, st, block_hist, E, nblk, counts, offsets);
  if (int rc = after_launch("index_scan_kernel")) return rc;
  if (nblk > 0) {
    launch(index_scatter_kernel, nblk, kIndexThreads, 8 * E * sizeof(int), st,
           indices, pairs, static_cast<int>(top_k), E, nblk, block_hist, offsets, perm_token, pos);
    if (int rc = after_launch("index_scatter_kernel")) return rc;
  }
  return B200_OK;
}

namespace b200 {
namespace {
template <typename W>
int launch_permute(const void* x, const int32_t* pos, const int32_t* dst_buf, const BufferTable& bufs, int64_t tokens,
                   int top_k, int64_t row_bytes, int64_t ldx_bytes, int64_t ldr_bytes, cudaStream_t st) {
  const int words = static_cast<int>(row_bytes / sizeof(W));
  const unsigned grid = static_cast<unsigned>(ceil_div(tokens, 8));
  const int64_t ldx = ldx_bytes / static_cast<int64_t>(sizeof(W)), ldr = ldr_bytes / static_cast<int64_t>(sizeof(W));
  // the more of a row one warp writes in one go, the better the DRAM pages are used
  // (measured on 8 KiB rows: 4 words per lane 6277 GB/s, 8: 6085+, 16 = the whole row: 6437)
  if (words >= 512)
    launch(permute_kernel<W, 16>, grid, 256, 0, st, static_cast<const W*>(x), pos, dst_buf, bufs, tokens, top_k, words, ldx, ldr);
  else if (words >= 256)
    launch(permute_kernel<W, 8>, grid, 256, 0, st, static_cast<const W*>(x), pos, dst_buf, bufs, tokens, top_k, words, ldx, ldr);
  else
    launch(permute_kernel<W, 4>, grid, 256, 0, st, static_cast<const W*>(x), pos, dst_buf, bufs, tokens, top_k, words, ldx, ldr);
  return after_launch("permute_kernel");
}
template <typename W>
int launch_gather(const void* x, const int32_t* src, void* out, int64_t n_rows, int64_t row_bytes,
                  int64_t ldx_bytes, int64_t ldo_bytes, cudaStream_t st) {
  launch(gather_kernel<W>, static_cast<unsigned>(ceil_div(n_rows, 8)), 256, 0, st,
      static_cast<const W*>(x), src, static_cast<W*>(out), n_rows, static_cast<int>(row_bytes / sizeof(W)),
      ldx_bytes / static_cast<int64_t>(sizeof(W)), ldo_bytes / static_cast<int64_t>(sizeof(W)));
  return after_launch("gather_kernel");
}
}  // namespace
}  // namespace b200

namespace b200 {
namespace {
// Shared body of b200_moe_permute and b200_moe_permute_multi.
int permute_impl(const char* fn, const void* x, const int32_t* dst_buf, const int32_t* pos, void* const* bufs, int64_t n_bufs,
                 int64_t tokens, int64_t top_k, int64_t hidden, int64_t ldx, int64_t ldrows, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (tokens < 0 || hidden < 0 || top_k < 1 || top_k > kMaxTopK)
    return fail(B200_ERR_SHAPE, "%s: need tokens, hidden >= 0 and 1 <= top_k <= %d", fn, kMaxTopK);
  if (n_bufs < 1 || n_bufs > kMaxBuffers) return fail(B200_ERR_SHAPE, "%s: need 1 <= n_bufs <= %d", fn, kMaxBuffers);
  if (ldx < hidden || ldrows < hidden) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than hidden", fn);
  if (tokens > 0x7fffffffLL * 8 || hidden > 0x7fffffffLL / 4) return fail(B200_ERR_SHAPE, "%s: problem too large", fn);
  if (tokens == 0 || hidden == 0) return B200_OK;
  B200_REQUIRE_PTR(x);
  B200_REQUIRE_PTR(pos);
  B200_REQUIRE_PTR(bufs);
  if (n_bufs > 1) B200_REQUIRE_PTR(dst_buf);
  const int64_t es = static_cast<int64_t>(dtype_size(dtype));
  BufferTable table{};
  bool all16 = true;
  for (int64_t i = 0; i < n_bufs; ++i) {
    if (bufs[i] == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: bufs[%lld] is NULL", fn, (long long)i);
    if (!aligned(bufs[i], es)) return fail(B200_ERR_ALIGNMENT, "%s: bufs[%lld] not aligned to the element size", fn, (long long)i);
    all16 = all16 && aligned(bufs[i], 16);
    table.base[i] = bufs[i];
  }
  if (!aligned(x, es) || !aligned(pos, 4) || (dst_buf && !aligned(dst_buf, 4)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int K = static_cast<int>(top_k);
  const int64_t rb = hidden * es, lxb = ldx * es, lrb = ldrows * es;
  bool all32 = aligned(x, 32) && rb % 8192 == 0 && lxb % 32 == 0 && lrb % 32 == 0;
  for (int64_t i = 0; i < n_bufs; ++i) all32 = all32 && aligned(bufs[i], 32);
  if (all32) {
    launch(permute_wide_kernel, static_cast<unsigned>(ceil_div(tokens, 16)), 512, 0, st, static_cast<const Word256*>(x), pos, dst_buf, table,
           tokens, K, static_cast<int>(rb / 32), lxb / 32, lrb / 32);
    return after_launch("permute_wide_kernel");
  }
  const void* probe = all16 ? x : static_cast<const char*>(x) + 4;  // a table entry that is only 4-byte aligned rules out 16-byte words
  if (rows_aligned<uint4>(probe, x, rb, lxb, lrb)) return launch_permute<uint4>(x, pos, dst_buf, table, tokens, K, rb, lxb, lrb, st);
  bool all4 = true;
  for (int64_t i = 0; i < n_bufs; ++i) all4 = all4 && aligned(bufs[i], 4);
  if (all4 && rows_aligned<uint32_t>(x, x, rb, lxb, lrb)) return launch_permute<uint32_t>(x, pos, dst_buf, table, tokens, K, rb, lxb, lrb, st);
  return launch_permute<uint16_t>(x, pos, dst_buf, table, tokens, K, rb, lxb, lrb, st);
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_permute(const void* x, const int32_t* pos, void* rows,
                                int64_t tokens, int64_t top_k, int64_t hidden,
                                int64_t ldx, int64_t ldrows, int dtype, void* stream) {
  void* const one[1] = {rows};
  if (rows == nullptr && tokens > 0 && hidden > 0) return fail(B200_ERR_NULL_POINTER, "%s: rows is NULL", __func__);
  return permute_impl(__func__, x, nullptr, pos, one, 1, tokens, top_k, hidden, ldx, ldrows, dtype, stream);
}

extern "C" int b200_moe_permute_multi(const void* x, const int32_t* dst_buf, const int32_t* dst_row,
                                      void* const* bufs, int64_t n_bufs,
                                      int64_t tokens, int64_t top_k, int64_t hidden,
                                      int64_t ldx, int64_t ldrows, int dtype, void* stream) {
  return permute_impl(__func__, x, dst_buf, dst_row, bufs, n_bufs, tokens, top_k, hidden, ldx, ldrows, dtype, stream);
}

extern "C" int b200_moe_gather(const void* x, const int32_t* src_row, void* out,
                               int64_t n_rows, int64_t hidden, int64_t ldx, int64_t ldo,
                               int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", __func__, dtype);
  if (n_rows < 0 || hidden < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (ldx < hidden || ldo < hidden) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than hidden", __func__);
  if (n_rows > 0x7fffffffLL * 8 || hidden > 0x7fffffffLL / 4) return fail(B200_ERR_SHAPE, "%s: problem too large", __func__);
  if (n_rows == 0 || hidden == 0) return B200_OK;
  B200_REQUIRE_PTR(x);
  B200_REQUIRE_PTR(src_row);
  B200_REQUIRE_PTR(out);
  const int64_t es = static_cast<int64_t>(dtype_size(dtype));
  if (!aligned(x, es) || !aligned(out, es) || !aligned(src_row, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rb = hidden * es, lxb = ldx * es, lob = ldo * es;
  if (rows_aligned<uint4>(x, out, rb, lxb, lob)) return launch_gather<uint4>(x, src_row, out, n_rows, rb, lxb, lob, st);
  if (rows_aligned<uint32_t>(x, out, rb, lxb, lob)) return launch_gather<uint32_t>(x, src_row, out, n_rows, rb, lxb, lob, st);
  return launch_gather<uint16_t>(x, src_row, out, n_rows, rb, lxb, lob, st);
}

namespace b200 {
namespace {
int unpermute_impl(const char* fn, void* const* bufs, int64_t n_bufs, const int32_t* src_buf, const int32_t* pos,
                   const float* weights, void* y, int64_t tokens, int64_t top_k, int64_t hidden,
                   int64_t ldrows, int64_t ldy, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (tokens < 0 || hidden < 0 || top_k < 1 || top_k > kMaxTopK)
    return fail(B200_ERR_SHAPE, "%s: need tokens, hidden >= 0 and 1 <= top_k <= %d", fn, kMaxTopK);
  if (n_bufs < 1 || n_bufs > kMaxBuffers) return fail(B200_ERR_SHAPE, "%s: need 1 <= n_bufs <= %d", fn, kMaxBuffers);
  if (ldrows < hidden || ldy < hidden) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than hidden", fn);
  if (tokens > 0x7fffffffLL * 8 || hidden > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: problem too large", fn);
  if (tokens == 0 || hidden == 0) return B200_OK;
  B200_REQUIRE_PTR(bufs);
  B200_REQUIRE_PTR(weights);
  B200_REQUIRE_PTR(pos);
  B200_REQUIRE_PTR(y);
  if (n_bufs > 1) B200_REQUIRE_PTR(src_buf);
  const size_t es = dtype_size(dtype);
  BufferTable table{};
  bool all16 = true;
  for (int64_t i = 0; i < n_bufs; ++i) {
    if (bufs[i] == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: bufs[%lld] is NULL", fn, (long long)i);
    if (!aligned(bufs[i], es)) return fail(B200_ERR_ALIGNMENT, "%s: bufs[%lld] not aligned to the element size", fn, (long long)i);
    all16 = all16 && aligned(bufs[i], 16);
    table.base[i] = bufs[i];
  }
  if (!aligned(y, es) || !aligned(weights, 4) || !aligned(pos, 4) || (src_buf && !aligned(src_buf, 4)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div(tokens, 8));
  const int K = static_cast<int>(top_k), H = static_cast<int>(hidden);
  bool all32 = aligned(y, 32) && top_k <= kWideSlots && (hidden * static_cast<int64_t>(es)) % 1024 == 0 &&
               (ldrows * static_cast<int64_t>(es)) % 32 == 0 && (ldy * static_cast<int64_t>(es)) % 32 == 0;
  for (int64_t i = 0; i < n_bufs; ++i) all32 = all32 && aligned(bufs[i], 32);
  if (all32) {
    const int steps = static_cast<int>(hidden * static_cast<int64_t>(es) / 1024);
    B200_DISPATCH_DTYPE(dtype, T, {
      launch(unpermute_wide_kernel<T>, static_cast<unsigned>(ceil_div(tokens, 4)), 128, 0, st, table, src_buf, weights, pos, static_cast<T*>(y),
             tokens, K, steps, ldrows, ldy);
    });
    return after_launch("unpermute_wide_kernel");
  }
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = Num<T>::kVec;
    const bool vec = hidden % V == 0 && ldrows % V == 0 && ldy % V == 0 && all16 && aligned(y, 16);
    // as many contiguous words per row as the row has (measured on 8 KiB rows: 6126, 6090 (2), 6327 GB/s (4))
    if (!vec)
      launch(unpermute_kernel<T, false, 1>, grid, 256, 0, st, table, src_buf, weights, pos, static_cast<T*>(y), tokens, K, H, ldrows, ldy);
    else if (hidden / V >= 128)
      launch(unpermute_kernel<T, true, 4>, grid, 256, 0, st, table, src_buf, weights, pos, static_cast<T*>(y), tokens, K, H, ldrows, ldy);
    else if (hidden / V >= 64)
      launch(unpermute_kernel<T, true, 2>, grid, 256, 0, st, table, src_buf, weights, pos, static_cast<T*>(y), tokens, K, H, ldrows, ldy);
    else
      launch(unpermute_kernel<T, true, 1>, grid, 256, 0, st, table, src_buf, weights, pos, static_cast<T*>(y), tokens, K, H, ldrows, ldy);
  });
  return after_launch("unpermute_kernel");
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_unpermute(const void* rows, const float* weights, const int32_t* pos, void* y,
                                  int64_t tokens, int64_t top_k, int64_t hidden,
                                  int64_t ldrows, int64_t ldy, int dtype, void* stream) {
  void* const one[1] = {const_cast<void*>(rows)};
  if (rows == nullptr && tokens > 0 && hidden > 0) return fail(B200_ERR_NULL_POINTER, "%s: rows is NULL", __func__);
  return unpermute_impl(__func__, one, 1, nullptr, pos, weights, y, tokens, top_k, hidden, ldrows, ldy, dtype, stream);
}

extern "C" int b200_moe_unpermute_multi(void* const* bufs, int64_t n_bufs, const int32_t* src_buf, const int32_t* src_row,
                                        const float* weights, void* y,
                                        int64_t tokens, int64_t top_k, int64_t hidden,
                                        int64_t ldrows, int64_t ldy, int dtype, void* stream) {
  return unpermute_impl(__func__, bufs, n_bufs, src_buf, src_row, weights, y, tokens, top_k, hidden, ldrows, ldy, dtype, stream);
}

// ------------------------------------------------------ unpermute backward --

namespace b200 {
namespace {
// y[t] = round_T(sum_k w[t,k] rows[pos[t,k]]) (fp32 inside), so
//   d_rows[pos[t,k]] = round_T(w[t,k] * dy[t]),   d_w[t,k] = <dy[t], rows[pos[t,k]]>   (fp32).
// One warp per token; for every slot the token's gradient row is re-read (it stays in L1), the expert row is
// streamed once for the dot product and the scaled gradient row is streamed out.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
unpermute_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ rows, const float* __restrict__ weights,
                     const int32_t* __restrict__ pos, T* __restrict__ d_rows, float* __restrict__ d_weights,
                     int64_t tokens, int top_k, int hidden, int64_t lddy, int64_t ldrows, int64_t lddrows) {
  pdl_prologue();
  constexpr int V = VEC ? Num<T>::kVec : 1;
  constexpr int UNROLL = 4;
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (t >= tokens) return;  // whole warps leave together
  const int words = hidden / V;
  const T* g = dy + t * lddy;
  for (int k = 0; k < top_k; ++k) {
    const int p = pos[t * top_k + k];  // the same for all lanes
    if (p < 0) {
      if (lane == 0) d_weights[t * top_k + k] = 0.f;
      continue;
    }
    const float w = weights[t * top_k + k];
    const T* src = rows + static_cast<int64_t>(p) * ldrows;
    T* dst = d_rows + static_cast<int64_t>(p) * lddrows;
    float dot = 0.f;
    for (int w0 = lane; w0 < words; w0 += 32 * UNROLL) {
      if constexpr (VEC) {
        uint4 vg[UNROLL], vr[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (w0 + 32 * u < words) {
            vg[u] = ld_reuse(g + static_cast<int64_t>(w0 + 32 * u) * V);
            vr[u] = ld_stream(src + static_cast<int64_t>(w0 + 32 * u) * V);
          }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (w0 + 32 * u < words) {
            float fg[Num<T>::kVec], fr[Num<T>::kVec];
            Num<T>::unpack(vg[u], fg);
            Num<T>::unpack(vr[u], fr);
#pragma unroll
            for (int j = 0; j < Num<T>::kVec; ++j) {
              dot = __fmaf_rn(fg[j], fr[j], dot);
              fg[j] = __fmul_rn(w, fg[j]);
            }
            st_stream(dst + static_cast<int64_t>(w0 + 32 * u) * V, Num<T>::pack(fg));
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int i = w0 + 32 * u;
          if (i < words) {
            const float fg = Num<T>::up(g[i]);
            dot = __fmaf_rn(fg, Num<T>::up(src[i]), dot);
            dst[i] = Num<T>::down(__fmul_rn(w, fg));
          }
        }
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) d_weights[t * top_k + k] = dot;
  }
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_unpermute_backward(const void* grad_y, const void* rows, const float* weights, const int32_t* pos,
                                           void* grad_rows, float* grad_weights, int64_t tokens, int64_t top_k, int64_t hidden,
                                           int64_t ld_grad_y, int64_t ldrows, int64_t ld_grad_rows, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", __func__, dtype);
  if (tokens < 0 || top_k < 0 || hidden < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (top_k > kMaxTopK) return fail(B200_ERR_SHAPE, "%s: top_k=%lld exceeds %d", __func__, (long long)top_k, kMaxTopK);
  if (tokens > 0x7fffffffLL * 8 || hidden > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: size out of range", __func__);
  if (tokens == 0 || top_k == 0) return B200_OK;
  B200_REQUIRE_PTR(weights);
  B200_REQUIRE_PTR(pos);
  B200_REQUIRE_PTR(grad_weights);
  if (hidden > 0) {
    B200_REQUIRE_PTR(grad_y);
    B200_REQUIRE_PTR(rows);
    B200_REQUIRE_PTR(grad_rows);
  }
  if (ld_grad_y < hidden || ldrows < hidden || ld_grad_rows < hidden) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than hidden", __func__);
  const size_t es = dtype_size(dtype);
  if (!aligned(grad_y, es) || !aligned(rows, es) || !aligned(grad_rows, es) || !aligned(weights, 4) || !aligned(pos, 4) || !aligned(grad_weights, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div(tokens, 8));
  const int K = static_cast<int>(top_k), H = static_cast<int>(hidden);
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = Num<T>::kVec;
    const bool vec = hidden % V == 0 && ld_grad_y % V == 0 && ldrows % V == 0 && ld_grad_rows % V == 0 && aligned(grad_y, 16) &&
                     aligned(rows, 16) && aligned(grad_rows, 16);
    if (vec)
      launch(unpermute_bwd_kernel<T, true>, grid, 256, 0, st, static_cast<const T*>(grad_y), static_cast<const T*>(rows), weights, pos,
             static_cast<T*>(grad_rows), grad_weights, tokens, K, H, ld_grad_y, ldrows, ld_grad_rows);
    else
      launch(unpermute_bwd_kernel<T, false>, grid, 256, 0, st, static_cast<const T*>(grad_y), static_cast<const T*>(rows), weights, pos,
             static_cast<T*>(grad_rows), grad_weights, tokens, K, H, ld_grad_y, ldrows, ld_grad_rows);
  });
  return after_launch("unpermute_bwd_kernel");
}

// --------------------------------------------------- expert-parallel plan --

namespace b200 {
namespace {
// For every (token, slot): the rank that owns its expert and the row it takes in that
// rank's exchange buffer.  dst_base[e] is where this rank's rows for expert e start there;
// the row inside that block is the pair's position among this rank's pairs of e.
__global__ void __launch_bounds__(256)
ep_destinations_kernel(const int32_t* __restrict__ indices, const int32_t* __restrict__ pos,
                       const int32_t* __restrict__ local_offsets, const int32_t* __restrict__ dst_base,
                       int64_t pairs, int experts, int experts_per_rank,
                       int32_t* __restrict__ dst_rank, int32_t* __restrict__ dst_row) {
  pdl_prologue();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= pairs) return;
  const int e = indices[i];
  const int p = pos[i];
  if (e < 0 || e >= experts || p < 0) {
    dst_rank[i] = 0;
    dst_row[i] = -1;
    return;
  }
  dst_rank[i] = e / experts_per_rank;
  dst_row[i] = dst_base[e] + (p - local_offsets[e]);
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_ep_destinations(const int32_t* indices, const int32_t* pos, const int32_t* local_offsets,
                                        const int32_t* dst_base, int64_t tokens, int64_t top_k, int64_t experts,
                                        int64_t experts_per_rank, int32_t* dst_rank, int32_t* dst_row, void* stream) {
  if (int rc = index_check(__func__, tokens, top_k, experts)) return rc;
  if (experts_per_rank < 1 || experts % experts_per_rank != 0)
    return fail(B200_ERR_SHAPE, "%s: experts_per_rank must divide experts", __func__);
  const int64_t pairs = tokens * top_k;
  if (pairs == 0) return B200_OK;
  B200_REQUIRE_PTR(indices);
  B200_REQUIRE_PTR(pos);
  B200_REQUIRE_PTR(local_offsets);
  B200_REQUIRE_PTR(dst_base);
  B200_REQUIRE_PTR(dst_rank);
  B200_REQUIRE_PTR(dst_row);
  if (!aligned(indices, 4) || !aligned(pos, 4) || !aligned(local_offsets, 4) || !aligned(dst_base, 4) || !aligned(dst_rank, 4) || !aligned(dst_row, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to 4 bytes", __func__);
  if (int rc = check_device()) return rc;
  launch(ep_destinations_kernel, static_cast<unsigned>(ceil_div(pairs, 256)), 256, 0, static_cast<cudaStream_t>(stream),
         indices, pos, local_offsets, dst_base, pairs, static_cast<int>(experts), static_cast<int>(experts_per_rank), dst_rank, dst_row);
  return after_launch("ep_destinations_kernel");
}
