// Expert-parallel exchange without the host in the loop: the count exchange, the addressing plan and the two
// rendezvous of a dispatch + combine step as kernels over peer-mapped memory (NVLink loads and stores).
//
// popcorn has no multi-GPU code (its momoe op is single-GPU, src/popcorn/kernels/momoe.py:34-53); these kernels are
// the plumbing around moe_permute_multi / moe_unpermute_multi, which move the rows themselves.
//
// Every rank owns one small "meta" buffer that all ranks map (symmetric memory).  Layout, in 32-bit words, the same on
// every rank:
//   [0, 2 * kMaxRanks * kMaxExperts)     two count tables (table = epoch & 1), row r = the per-expert counts of rank r
//   then kChannels * kMaxRanks flags     flag (channel, r) = the last epoch rank r has reached on that channel, each
//                                        flag alone in a 128-byte line
// A rank publishes by plain stores into every peer's copy, then a system-scope fence, then a release store of the
// epoch into its flag on every peer; a rank consumes after acquire loads of all its own flags have reached the epoch.
// Every wait is bounded by a time budget: when it runs out the kernel records where it gave up in a status word and
// returns (the plan is then written so that every destination is negative, which the row kernels skip); nothing
// traps and nothing spins for ever.  Only ordinary loads and stores touch peer memory: no multimem, no bulk copies.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxRanks = 16;
constexpr int kMaxExpertsEp = 1024;
constexpr int kChannels = 4;
constexpr int kFlagStride = 32;  // words: one flag per 128-byte line
constexpr int kTableWords = kMaxRanks * kMaxExpertsEp;
constexpr int kFlagBase = 2 * kTableWords;
constexpr int kMetaWords = kFlagBase + kChannels * kMaxRanks * kFlagStride;
constexpr int kBadRow = -(1 << 30);

struct MetaTable {
  int32_t* base[kMaxRanks];
};
__device__ __forceinline__ int32_t* meta_of(const MetaTable& table, int r) {
  int32_t* p = table.base[0];
#pragma unroll
  for (int k = 1; k < kMaxRanks; ++k)
    if (r == k) p = table.base[k];
  return p;
}
__device__ __forceinline__ int flag_word(int channel, int r) { return kFlagBase + (channel * kMaxRanks + r) * kFlagStride; }

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int32_t ld_relaxed_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait until *flag has reached `epoch` (epochs only grow; the comparison is wrap-safe).  Returns false when the budget
// ran out first.
__device__ __forceinline__ bool wait_flag(const int32_t* flag, int32_t epoch, unsigned long long budget_ns) {
  const unsigned long long start = now_ns();
  while (static_cast<int32_t>(static_cast<uint32_t>(ld_acquire_sys(flag)) - static_cast<uint32_t>(epoch)) < 0) {
    if (now_ns() - start > budget_ns) return false;
    __nanosleep(100);
  }
  return true;
}

// status[0]: 0 ok, else the first failure (1 count exchange timed out, 2 rendezvous timed out, 3 a rank would receive
// more rows than the exchange buffers hold); status[1]: the peer waited for, or the row count.
__device__ __forceinline__ void record(int32_t* status, int code, int detail) {
  if (atomicCAS(status, 0, code) == 0) status[1] = detail;
}

// One CTA.  Publishes this rank's per-expert counts, waits for everybody's, and derives this rank's addressing:
//   dst_base[e]        row in the buffer of e's owner at which THIS rank's rows for expert e start (the owner's buffer
//                      is expert-major; inside an expert the source ranks follow in rank order)
//   expert_offsets[j]  start of this rank's j-th own expert in its own buffer, j = 0 .. experts / world
//   info[0..3]         rows this rank receives, rows it sends to other ranks, the largest receive of any rank, world
__global__ void __launch_bounds__(1024)
ep_exchange_kernel(const int32_t* __restrict__ counts, const MetaTable meta, int world, int rank, int experts,
                   int64_t capacity_rows, int32_t epoch, unsigned long long budget_ns, int32_t* __restrict__ dst_base,
                   int32_t* __restrict__ expert_offsets, int32_t* __restrict__ info, int32_t* __restrict__ status) {
  pdl_prologue();
  __shared__ int total[kMaxExpertsEp];
  __shared__ int scanned[kMaxExpertsEp];
  __shared__ int warp_tot[32];
  __shared__ int rows_of_rank[kMaxRanks];
  __shared__ int failed;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int table = (epoch & 1) * kTableWords;
  if (tid == 0) failed = 0;
  for (int i = tid; i < world * experts; i += 1024) {
    const int r = i / experts, e = i - r * experts;
    meta_of(meta, r)[table + rank * kMaxExpertsEp + e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) st_release_sys(meta_of(meta, tid) + flag_word(0, rank), epoch);
  int32_t* mine = meta_of(meta, rank);
  if (tid < world && !wait_flag(mine + flag_word(0, tid), epoch, budget_ns)) {
    record(status, 1, tid);
    failed = 1;
  }
  __syncthreads();
  const int per_rank = experts / world;
  const int e = tid;
  int c_total = 0, c_before = 0, c_mine = 0;
  if (!failed && e < experts) {
    for (int r = 0; r < world; ++r) {
      const int c = ld_relaxed_sys(mine + table + r * kMaxExpertsEp + e);
      c_total += c;
      if (r < rank) c_before += c;
      if (r == rank) c_mine = c;
    }
  }
  if (e < kMaxExpertsEp) total[e] = c_total;
  // exclusive scan of the totals over all experts (warp scans, then a scan of the warp totals)
  int incl = c_total;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = warp_tot[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += up;
    }
    warp_tot[lane] = wi - w;
  }
  __syncthreads();
  scanned[e] = warp_tot[warp] + incl - c_total;
  __syncthreads();
  if (tid < world) {
    const int first = tid * per_rank;
    const int last = first + per_rank - 1;
    rows_of_rank[tid] = scanned[last] + total[last] - scanned[first];
  }
  __syncthreads();
  int largest = 0;
  for (int r = 0; r < world; ++r) largest = rows_of_rank[r] > largest ? rows_of_rank[r] : largest;
  const bool over = !failed && largest > capacity_rows;  // the same in every thread
  if (over && tid == 0) record(status, 3, largest);
  const bool bad = failed || over;
  if (e < experts) {
    const int owner_first = (e / per_rank) * per_rank;
    dst_base[e] = bad ? kBadRow : scanned[e] - scanned[owner_first] + c_before;
  }
  if (tid < per_rank) {
    const int first = rank * per_rank;
    expert_offsets[tid] = bad ? 0 : scanned[first + tid] - scanned[first];
  }
  if (tid == 0) expert_offsets[per_rank] = bad ? 0 : rows_of_rank[rank];
  // rows this rank sends away: its own counts for experts it does not own (a sum over the block, by thread 0 of it)
  __shared__ int sent_away;
  if (tid == 0) sent_away = 0;
  __syncthreads();
  if (e < experts && e / per_rank != rank) atomicAdd(&sent_away, c_mine);
  __syncthreads();
  if (tid == 0) {
    info[0] = bad ? 0 : rows_of_rank[rank];
    info[1] = sent_away;
    info[2] = largest;
    info[3] = world;
  }
}

// One CTA: tell every rank that this rank has reached `epoch` on `channel`, then wait until every rank has.  Placed
// after a kernel that wrote peer memory it makes those writes visible to the peers' following kernels; placed before
// a kernel that reads peer memory it guarantees the peers have finished writing.
__global__ void __launch_bounds__(32)
ep_barrier_kernel(const MetaTable meta, int world, int rank, int channel, int32_t epoch, unsigned long long budget_ns,
                  int32_t* __restrict__ status) {
  pdl_prologue();
  const int tid = threadIdx.x;
  __threadfence_system();
  if (tid < world) {
    st_release_sys(meta_of(meta, tid) + flag_word(channel, rank), epoch);
    if (!wait_flag(meta_of(meta, rank) + flag_word(channel, tid), epoch, budget_ns)) record(status, 2, tid);
  }
  __syncwarp();
  __threadfence_system();
}

int meta_table(const char* fn, void* const* meta, int64_t world, int64_t rank, MetaTable* table) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(B200_ERR_SHAPE, "%s: need 1 <= world <= %d and 0 <= rank < world", fn, kMaxRanks);
  if (meta == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: meta is NULL", fn);
  for (int64_t r = 0; r < world; ++r) {
    if (meta[r] == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: meta[%lld] is NULL", fn, (long long)r);
    if (!aligned(meta[r], 128)) return fail(B200_ERR_ALIGNMENT, "%s: meta[%lld] is not 128-byte aligned", fn, (long long)r);
    table->base[r] = static_cast<int32_t*>(meta[r]);
  }
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_moe_ep_meta_bytes(size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  *bytes = static_cast<size_t>(kMetaWords) * sizeof(int32_t);
  return B200_OK;
}

extern "C" int b200_moe_ep_exchange(const int32_t* counts, void* const* meta, int64_t world, int64_t rank, int64_t experts,
                                    int64_t capacity_rows, int32_t epoch, int64_t budget_ns, int32_t* dst_base,
                                    int32_t* expert_offsets, int32_t* info, int32_t* status, void* stream) {
  MetaTable table{};
  if (int rc = meta_table(__func__, meta, world, rank, &table)) return rc;
  if (experts < 1 || experts > kMaxExpertsEp || experts % world != 0)
    return fail(B200_ERR_SHAPE, "%s: need 1 <= experts <= %d, a multiple of world", __func__, kMaxExpertsEp);
  if (capacity_rows < 0 || budget_ns <= 0) return fail(B200_ERR_SHAPE, "%s: need capacity_rows >= 0 and budget_ns > 0", __func__);
  B200_REQUIRE_PTR(counts);
  B200_REQUIRE_PTR(dst_base);
  B200_REQUIRE_PTR(expert_offsets);
  B200_REQUIRE_PTR(info);
  B200_REQUIRE_PTR(status);
  if (!aligned(counts, 4) || !aligned(dst_base, 4) || !aligned(expert_offsets, 4) || !aligned(info, 4) || !aligned(status, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to 4 bytes", __func__);
  if (int rc = check_device()) return rc;
  launch(ep_exchange_kernel, 1, 1024, 0, static_cast<cudaStream_t>(stream), counts, table, static_cast<int>(world), static_cast<int>(rank),
         static_cast<int>(experts), capacity_rows, epoch, static_cast<unsigned long long>(budget_ns), dst_base, expert_offsets, info, status);
  return after_launch("ep_exchange_kernel");
}

extern "C" int b200_moe_ep_barrier(void* const* meta, int64_t world, int64_t rank, int64_t channel, int32_t epoch, int64_t budget_ns,
                                   int32_t* status, void* stream) {
  MetaTable table{};
  if (int rc = meta_table(__func__, meta, world, rank, &table)) return rc;
  if (channel < 1 || channel >= kChannels) return fail(B200_ERR_SHAPE, "%s: need 1 <= channel < %d (channel 0 belongs to the count exchange)", __func__, kChannels);
  if (budget_ns <= 0) return fail(B200_ERR_SHAPE, "%s: need budget_ns > 0", __func__);
  B200_REQUIRE_PTR(status);
  if (!aligned(status, 4)) return fail(B200_ERR_ALIGNMENT, "%s: status not aligned to 4 bytes", __func__);
  if (int rc = check_device()) return rc;
  launch(ep_barrier_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), table, static_cast<int>(world), static_cast<int>(rank),
         static_cast<int>(channel), epoch, static_cast<unsigned long long>(budget_ns), status);
  return after_launch("ep_barrier_kernel");
}
