// Grouped expert GEMM for sm_100a: the dense step either side of the MoE permutation.
//
//   out[p, :] = rows[p, :] @ weight[e(p)]            (one weight matrix per expert)
//   out[p, :] = (rows[p, :] @ up[e]) * silu(rows[p, :] @ gate[e])   (DUAL: both projections and SwiGLU in one pass)
//
// where e(p) is the expert whose segment offsets[e] <= p < offsets[e + 1] holds row p of the
// expert-major `rows` buffer that b200_moe_permute writes.  This is what the reference's
// lin1_kernel / lin2_kernel compute (src/popcorn/impls/momoe_tl.py:90-212 and 225-330) and what the
// registered reference states as two einsums over a dense [batch, seq, experts, .] tensor
// (src/popcorn/kernels/momoe.py:50-52); weights keep the reference's layout
// [experts, in_features, out_features] with out_features contiguous.
//
// Bound: tensor cores.  One CTA owns a 128 x 256 output tile (DUAL: 128 x 128 of each projection,
// side by side in one accumulator) of one expert:
//   warp 0     producer: one lane issues tiled bulk-tensor copies (TMA, 128-byte swizzle) of the
//              128 x 64 slice of `rows` and the 64 x 256 slice of the expert's weight into a
//              shared-memory ring, completion counted on a `full` mbarrier per slot
//   warp 1     one lane issues tcgen05.mma (M 128, N 256, K 16; A K-major, B N-major straight from
//              the reference's weight layout) into one of two 256-column fp32 accumulators in
//              tensor memory; tcgen05.commit releases the ring slot and, after the last K slice,
//              publishes the accumulator
//   warps 2-5  epilogue: tcgen05.ld of the finished accumulator (each warp its 32-lane quarter),
//              conversion (and SwiGLU) in registers, a transpose through a small shared-memory tile so
//              that every store instruction writes whole 128-byte row segments, and only the rows that
//              belong to the expert; overlaps the next tile's main loop through the second accumulator
// CTAs are persistent (one per SM) and walk the tile list (expert, m tile, n tile; n fastest) derived on
// the device from `offsets`, so the host never reads the routing result.
//
// Pair mode (the default): two CTAs of a cluster work as one (tcgen05 cta_group::2) on a 256 x 256
// tile.  Each loads its own 128 rows and only HALF of the weight slice (128 of the 256 columns), the
// leader's MMA reads both halves across the pair, so per SM the shared-memory fill drops from 48 to
// 32 KiB per 64 K values; a ring slot then holds two such K spans (3 slots of 64 KiB).  Copies of both
// CTAs complete on the leader's `full` barrier; the leader's tcgen05.commit reaches the `empty` and
// `acc_full` barriers of both CTAs; both epilogues arrive on the leader's `acc_empty`.
//
// Every wait is bounded (tma.cuh): a wait that runs out marks the CTA aborted, every role leaves
// its loop, the CTA waits (bounded again) for copies and MMAs it still has in flight, frees its
// tensor memory and returns; b200_wait_timeouts() reports it.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "activations.cuh"
#include "common.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kUmmaK = 16;  // kBK: K values per 128-byte swizzle span (one copy box)
constexpr int kASubBytes = kBM * kBK * 2;        // 16 KiB: 128 rows x 64 K values
constexpr int kMaxStages = 4;
// Per CTA, with CTAS = 1 (alone) or 2 (pair): the weight columns it loads, its ring slot and ring depth.
// A slot of a pair holds TWO 64-wide K spans: the single thread that issues the MMAs pays one barrier wait and
// one commit per slot, and with eight MMAs per slot instead of four that fixed cost no longer outlasts the
// tensor pipe (ncu sm__pipe_tensor_cycles_active went from 81 % to 97 % on the gate/up launch).
template <int CTAS>
struct Ring {
  static constexpr int kSub = CTAS;                          // 64-wide K spans per slot
  static constexpr int kSlotK = kBK * kSub;                  // K values per slot
  static constexpr int kChunks = kBN / 64 / CTAS;            // 64-column chunks of the weight slice this CTA loads
  static constexpr int kABytes = kSub * kASubBytes;
  static constexpr int kBChunkBytes = kSlotK * 128;          // one 64-column chunk: kSlotK rows of 128 bytes
  static constexpr int kStageBytes = kABytes + kChunks * kBChunkBytes;  // 48 KiB alone, 64 KiB in a pair
  static constexpr int kStages = CTAS == 2 ? 3 : 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // + slack to align the ring to the swizzle atom
};
constexpr int kTmemCols = 512;                   // two accumulators of kBN fp32 columns
constexpr int kMaxExperts = 1024;
constexpr int kThreads = 192;

// ---- tcgen05 / tensor-map wrappers; PAIR = the cta_group::2 forms.  No copy is addressed to more than one CTA. ----
//
// The producer and the MMA issuer are single threads whose instruction streams run beside a tensor pipe that
// finishes a K slice every ~512 cycles, so their inner loops work on raw 32-bit shared-memory addresses and
// counters that wrap (no division, no address conversion per copy).
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicAdd(&g_wait_timeouts, 1u);
  return false;
}
__device__ __forceinline__ void mbar_arrive_expect_addr(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Tiled bulk-tensor copies into THIS CTA's shared memory; in a pair the bytes are counted on a barrier of the leader.
template <bool PAIR>
__device__ __forceinline__ void tma_2d(uint32_t dst, uint64_t map, int x, int y, uint32_t bar) {
  if constexpr (PAIR)
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
  else
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tma_3d(uint32_t dst, uint64_t map, int x, int y, int z, uint32_t bar) {
  if constexpr (PAIR)
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
  else
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  if constexpr (PAIR) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
}
template <bool PAIR>
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on `bar` (in a pair: on the barrier at that offset in BOTH CTAs) when every tcgen05.mma this thread
// issued before has completed.
template <bool PAIR>
__device__ __forceinline__ void mma_commit_addr(uint32_t bar) {
  if constexpr (PAIR)
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem] with the descriptors given as (low word, shared high word); `accumulate` = 0
// overwrites D.  In a pair M is 256: each CTA contributes its 128 rows of A and its half of B and receives its
// 128 rows of D.
template <bool PAIR>
__device__ __forceinline__ void mma_issue(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t a_hi, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if constexpr (PAIR)
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// ---- cluster helpers for the pair ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of this CTA's shared-memory location `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive fp32 columns of tensor memory: lane l of the warp receives row (quarter * 32 + l).
__device__ __forceinline__ void tmem_load_32(uint32_t addr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (sm_100 format: start >> 4 in bits 0-13, leading byte offset >> 4
// in 16-29, stride byte offset >> 4 in 32-45, version 1 in 46-47, swizzle mode in 61-63; 2 = 128 bytes).
//  A, K-major, rows of 128 bytes (64 K values): 8-row groups 1024 bytes apart (stride offset); the
//     leading offset is not used by swizzled K-major layouts and is set to its canonical 1.
//  B, N-major, rows of 128 bytes (64 N values) per K index: 8-row K groups 1024 bytes apart (stride
//     offset), 64-column chunks one whole [64 x 128 B] block apart (leading offset).
constexpr uint64_t kDescFixed = (uint64_t(1) << 46) | (uint64_t(2) << 61);
constexpr uint64_t kDescA = kDescFixed | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32);
template <int CTAS>
constexpr uint64_t kDescB = kDescFixed | (uint64_t(Ring<CTAS>::kBChunkBytes >> 4) << 16) | (uint64_t(1024 >> 4) << 32);

// Instruction descriptor of kind::f16: fp32 accumulate (bit 4), A/B format (0 fp16, 1 bf16) at bits 7
// and 10, A K-major (bit 15 = 0), B N-major (bit 16 = 1), N >> 3 at bit 17, M >> 4 at bit 24 (M = 256 for a pair).
__host__ __device__ constexpr uint32_t instr_desc(uint32_t format, int ctas) {
  return (1u << 4) | (format << 7) | (format << 10) | (1u << 16) | (uint32_t(kBN >> 3) << 17) | (uint32_t((kBM * ctas) >> 4) << 24);
}

struct GemmArgs {
  const int32_t* offsets;  // [experts + 1], device
  void* out;
  int64_t ld_out;
  int experts;
  int n;        // output columns (per projection)
  int k;
  int total_rows;  // rows of `rows` and `out`: nothing is stored past them, whatever `offsets` says
  uint32_t idesc;
};

struct Tile {
  int expert, row0, row_end, n0;
};

// tile -> (expert, m tile, n tile): tiles of one expert are consecutive, n fastest, so that the CTAs running
// together work on a few row blocks of ONE expert against all of its weight columns: their working set (a few MB
// of rows plus the expert's weight matrix, 12-25 MB here) stays in L2 and every operand byte comes from DRAM once.
// (m fastest sweeps the expert's whole row segment, 64 MB here, once per column tile, which L2 does not hold.)
// (`offsets` is the CTA's shared-memory copy of the segment bounds: a tile switch costs no global-memory round trip.)
__device__ __forceinline__ Tile decode_tile(int tile, const int* tile_start, const int* offsets, int experts, int out_tile_n, int tile_rows, int tiles_n) {
  int lo = 0, hi = experts;  // last expert with tile_start[e] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_start[mid] <= tile) lo = mid;
    else hi = mid;
  }
  const int first = offsets[lo], end = offsets[lo + 1];
  const int local = tile - tile_start[lo];
  Tile t;
  t.expert = lo;
  t.row0 = first + (local / tiles_n) * tile_rows;
  t.row_end = end;
  t.n0 = (local % tiles_n) * out_tile_n;
  return t;
}

template <typename T, bool DUAL, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_w2, const GemmArgs p) {
  using R = Ring<CTAS>;
  constexpr bool PAIR = CTAS == 2;
  constexpr int OUT_N = DUAL ? kBN / 2 : kBN;  // output columns per tile
  constexpr int STAGES = R::kStages;
  constexpr int TILE_ROWS = kBM * CTAS;
  pdl_prologue();
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int aborted;
  __shared__ int tile_start[kMaxExperts + 1], seg[kMaxExperts + 1];
  __shared__ uint4 staging[4][32][8];  // per epilogue warp: 32 rows x 128 bytes of finished output

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_rank() : 0u;  // position in the pair; rank 0 leads
  const int first_tile = PAIR ? blockIdx.x / 2 : blockIdx.x;
  const int tile_step = PAIR ? gridDim.x / 2 : gridDim.x;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tiles_n = (p.n + OUT_N - 1) / OUT_N;

  if (threadIdx.x == 0) {
    aborted = 0;
    int total = 0, lo = max(p.offsets[0], 0);
    seg[0] = lo;
    for (int e = 0; e < p.experts; ++e) {
      tile_start[e] = total;
      const int hi = min(p.offsets[e + 1], p.total_rows);
      seg[e + 1] = hi;
      total += (hi > lo ? (hi - lo + TILE_ROWS - 1) / TILE_ROWS : 0) * tiles_n;
      lo = hi;
    }
    tile_start[p.experts] = total;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4 * CTAS);  // one arrival per epilogue warp (of both CTAs in a pair)
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc<PAIR>(&tmem_base_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();  // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total_tiles = tile_start[p.experts];
  volatile int* abort_flag = &aborted;
  const uint32_t ring_addr = smem_addr(ring), full_addr = smem_addr(&full[0]), empty_addr = smem_addr(&empty[0]);

  if (warp == 0) {
    // ------------------------------------------------------------- producer --
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      // the barrier the copies complete on: this CTA's own, or in a pair the leader's
      const uint32_t signal_addr = PAIR ? map_to_rank(full_addr, 0) : full_addr;
      const uint64_t rows_map = reinterpret_cast<uint64_t>(&map_rows), w2_map = reinterpret_cast<uint64_t>(&map_w2);
      // this CTA's share of the 256 accumulator columns: all of them alone, one half in a pair
      // (DUAL: columns 0-127 are the gate projection, 128-255 the up projection of the same output columns)
      const uint64_t b_map = (DUAL && PAIR && rank == 1) ? w2_map : reinterpret_cast<uint64_t>(&map_w);
      for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step) {
        const Tile t = decode_tile(tile, tile_start, seg, p.experts, OUT_N, TILE_ROWS, tiles_n);
        const int row0 = t.row0 + static_cast<int>(rank) * kBM;
        const int col0 = t.n0 + ((!DUAL && PAIR) ? static_cast<int>(rank) * (kBN / 2) : 0);
        for (int k0 = 0; k0 < p.k; k0 += R::kSlotK) {
          if (!mbar_wait_addr(empty_addr + stage * 8, phase ^ 1u)) {
            *abort_flag = 1;
            break;
          }
          const uint32_t a_dst = ring_addr + stage * R::kStageBytes, b_dst = a_dst + R::kABytes, bar = signal_addr + stage * 8;
          if (rank == 0) mbar_arrive_expect_addr(full_addr + stage * 8, CTAS * R::kStageBytes);  // in a pair both CTAs' bytes land here
#pragma unroll
          for (int j = 0; j < R::kSub; ++j) tma_2d<PAIR>(a_dst + j * kASubBytes, rows_map, k0 + j * kBK, row0, bar);  // past K: zero fill
#pragma unroll
          for (int c = 0; c < R::kChunks; ++c) {
            if (DUAL && !PAIR && c >= R::kChunks / 2) tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, w2_map, t.n0 + (c - R::kChunks / 2) * 64, k0, t.expert, bar);
            else tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, b_map, col0 + c * 64, k0, t.expert, bar);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag && rank == 0) {
        // copies already issued (by either CTA of a pair) still write shared memory: give each slot's last copy a bounded wait
        for (uint32_t k = issued > STAGES ? issued - STAGES : 0; k < issued; ++k) (void)mbar_wait(&full[k % STAGES], (k / STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer --
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, local = 0;
      bool pending = false;
      const uint32_t acc_full_addr = smem_addr(&acc_full[0]), acc_empty_addr = smem_addr(&acc_empty[0]);
      const uint32_t a_hi = static_cast<uint32_t>(kDescA >> 32), b_hi = static_cast<uint32_t>(kDescB<CTAS> >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(kDescA) | (ring_addr >> 4);
      const uint32_t b_lo0 = static_cast<uint32_t>(kDescB<CTAS>) | ((ring_addr + R::kABytes) >> 4);
      const uint32_t idesc = p.idesc;
      for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step, ++local) {
        const uint32_t acc = local & 1u;
        if (!mbar_wait_addr(acc_empty_addr + acc * 8, ((local >> 1) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        uint32_t accumulate = 0;
        for (int k0 = 0; k0 < p.k; k0 += R::kSlotK) {
          if (!mbar_wait_addr(full_addr + stage * 8, phase)) {
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          // descriptor start fields advance in 16-byte units: a ring slot, then per MMA 16 K values = 32 bytes along
          // A's swizzled 128-byte rows (a new 16 KiB block every 64 K values) and 16 K rows = 2048 bytes of B
          const uint32_t a_lo = a_lo0 + stage * (R::kStageBytes >> 4), b_lo = b_lo0 + stage * (R::kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < R::kSlotK / kUmmaK; ++k) {
            constexpr int kPerSpan = kBK / kUmmaK;
            mma_issue<PAIR>(d_tmem, a_lo + (k / kPerSpan) * (kASubBytes >> 4) + (k % kPerSpan) * (kUmmaK * 2 >> 4), b_lo + k * (kUmmaK * 128 >> 4),
                            a_hi, b_hi, idesc, accumulate);
            accumulate = 1;
          }
          mma_commit_addr<PAIR>(empty_addr + stage * 8);  // the slot (in both CTAs of a pair) is free once these MMAs have read it
          pending = true;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (*abort_flag) break;
        mma_commit_addr<PAIR>(acc_full_addr + acc * 8);
      }
      if (*abort_flag && pending) {
        // MMAs may still be running: a bounded wait on a fresh commit before tensor memory is freed
        mma_commit_addr<PAIR>(acc_full_addr);
        (void)mbar_wait(&acc_full[0], 0);
        (void)mbar_wait(&acc_full[0], 1);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue --
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    uint32_t local = 0;
    T* out = static_cast<T*>(p.out);
    for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step, ++local) {
      const Tile t = decode_tile(tile, tile_start, seg, p.experts, OUT_N, TILE_ROWS, tiles_n);
      const uint32_t acc = local & 1u;
      // one lane polls for the whole warp
      const int ready = __shfl_sync(0xffffffffu, lane == 0 ? static_cast<int>(mbar_wait(&acc_full[acc], (local >> 1) & 1u)) : 0, 0);
      if (!ready) {
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int warp_row0 = t.row0 + static_cast<int>(rank) * kBM + quarter * 32;
      uint4(*mine)[8] = staging[quarter];
#pragma unroll 1
      for (int c = 0; c < OUT_N / 32; ++c) {
        uint32_t v[32], u[32];
        tmem_load_32(taddr + c * 32, v);
        if constexpr (DUAL) tmem_load_32(taddr + OUT_N + c * 32, u);
        tmem_load_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float lo = __uint_as_float(v[2 * j]), hi = __uint_as_float(v[2 * j + 1]);
          if constexpr (DUAL) {
            // columns 0..127 of the accumulator hold rows @ gate, 128..255 rows @ up
            lo = __fmul_rn(silu_f32<1>(lo), __uint_as_float(u[2 * j]));
            hi = __fmul_rn(silu_f32<1>(hi), __uint_as_float(u[2 * j + 1]));
          }
          packed[j] = Num<T>::pack2(lo, hi);
        }
        // lane = row: its 32 columns are four 16-byte pieces of the 128-byte staging row (piece index
        // xor-ed with the row so that neither these writes nor the transposed reads conflict on banks)
#pragma unroll
        for (int q = 0; q < 4; ++q)
          mine[lane][((c & 1) * 4 + q) ^ (lane & 7)] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        if (c & 1) {
          // 64 finished columns of 32 rows: write them out as whole 128-byte row segments, four rows per instruction
          __syncwarp();
          const int piece = lane & 7;
          const int col = t.n0 + (c - 1) * 32 + piece * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3);
            const int row = warp_row0 + r;
            if (row < t.row_end && col < p.n)
              st_stream(out + static_cast<int64_t>(row) * p.ld_out + col, mine[r][piece ^ (r & 7)]);
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) remote_arrive(map_to_rank(smem_addr(&acc_empty[acc]), 0));  // the leader issues the MMAs
        else mbar_arrive(&acc_empty[acc]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) tmem_dealloc<PAIR>(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------ host side --

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library links against cudart only.
EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// rows [total_rows, k], row stride ld: box 64 (K) x 128 (rows), 128-byte swizzle, zero fill outside.
bool encode_rows(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t total_rows, int64_t k, int64_t ld) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(total_rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kBK, kBM}, elem[2] = {1, 1};
  return encoder()(map, type, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// weight [experts, k, n], n contiguous: box 64 (N) x slot_k (K) x 1 (expert).
bool encode_weight(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t experts, int64_t k, int64_t n, int slot_k) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(n) * 2, static_cast<cuuint64_t>(n) * static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(slot_k), 1}, elem[3] = {1, 1, 1};
  return encoder()(map, type, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// B200_GEMM_PAIR=0 in the environment runs every CTA on its own (cta_group::1); read at every call.
bool pair_enabled() {
  const char* v = std::getenv("B200_GEMM_PAIR");
  return !(v && v[0] == '0');
}

constexpr int kNoClusters = -1000;  // run_with<., ., 2>: no cluster of two CTAs can be resident; the caller runs single CTAs instead

// What the tensor maps of one call describe.
struct Operands {
  const void *rows, *weight, *weight2;
  int64_t total_rows, k, n, experts, ld_rows;
  CUtensorMapDataType type;
};

template <typename T, bool DUAL, int CTAS>
int run_with(const Operands& op, GemmArgs args, uint32_t format, cudaStream_t st) {
  alignas(64) CUtensorMap rows, w, w2;
  constexpr int slot_k = Ring<CTAS>::kSlotK;
  if (!encode_rows(&rows, op.type, op.rows, op.total_rows, op.k, op.ld_rows) ||
      !encode_weight(&w, op.type, op.weight, op.experts, op.k, op.n, slot_k) ||
      !encode_weight(&w2, op.type, op.weight2 ? op.weight2 : op.weight, op.experts, op.k, op.n, slot_k))
    return fail(B200_ERR_LAUNCH, "b200_moe_grouped_gemm: tensor map encoding failed");
  auto kernel = grouped_gemm_kernel<T, DUAL, CTAS>;
  constexpr int smem = Ring<CTAS>::kSmemBytes;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(B200_ERR_LAUNCH, "b200_moe_grouped_gemm: cannot reserve %d bytes of shared memory", smem);
  }
  args.idesc = instr_desc(format, CTAS);
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = st;
  cudaLaunchAttribute attrs[2];
  unsigned n_attrs = 0;
  if (CTAS == 2) {
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 2;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  config.attrs = attrs;
  config.numAttrs = n_attrs;
  int ctas = sm_count();
  if (CTAS == 2) {
    // persistent pairs: as many clusters as can be resident at once (an odd SM of a processing cluster has no partner)
    config.gridDim = dim3(static_cast<unsigned>(ctas & ~1));
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      return kNoClusters;
    }
    ctas = 2 * std::min(clusters, ctas / 2);
  }
  config.gridDim = dim3(static_cast<unsigned>(ctas));
  if (pdl_enabled()) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = ++n_attrs;
  }
  (void)cudaLaunchKernelEx(&config, kernel, rows, w, w2, args);
  return after_launch(CTAS == 2 ? "grouped_gemm_kernel (pairs)" : "grouped_gemm_kernel");
}

template <typename T, bool DUAL>
int run(const Operands& op, const GemmArgs& args, uint32_t format, cudaStream_t st) {
  if (pair_enabled()) {
    const int rc = run_with<T, DUAL, 2>(op, args, format, st);
    if (rc != kNoClusters) return rc;
  }
  return run_with<T, DUAL, 1>(op, args, format, st);
}

}  // namespace

unsigned int gemm_wait_timeouts() { return read_wait_timeouts(); }

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_grouped_gemm(const void* rows, const void* weight, const void* weight2, const int32_t* offsets, void* out,
                                     int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_out,
                                     int dtype, void* stream) {
  if (dtype != B200_BF16 && dtype != B200_F16)
    return fail(B200_ERR_DTYPE, "%s: dtype %d not supported (bf16 or fp16 operands, fp32 accumulation)", __func__, dtype);
  if (total_rows < 0 || k < 0 || n < 0 || experts < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (experts > kMaxExperts) return fail(B200_ERR_SHAPE, "%s: experts=%lld exceeds %d", __func__, (long long)experts, kMaxExperts);
  if (total_rows > 0x7fffffffLL - kBM || k > 0x7fffffffLL || n > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: size out of range", __func__);
  if (total_rows == 0 || n == 0 || experts == 0) return B200_OK;
  B200_REQUIRE_PTR(rows);
  B200_REQUIRE_PTR(weight);
  B200_REQUIRE_PTR(offsets);
  B200_REQUIRE_PTR(out);
  if (k == 0) return fail(B200_ERR_SHAPE, "%s: k must be positive", __func__);
  if (k % 8 != 0 || n % 8 != 0 || ld_rows % 8 != 0 || ld_out % 8 != 0)
    return fail(B200_ERR_SHAPE, "%s: k, n and the row strides must be multiples of 8 elements (16-byte rows for the tensor maps)", __func__);
  if (ld_rows < k || ld_out < n) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than the row", __func__);
  if (!aligned(rows, 16) || !aligned(weight, 16) || !aligned(out, 16) || (weight2 && !aligned(weight2, 16)) || !aligned(offsets, 4))
    return fail(B200_ERR_ALIGNMENT, "%s: rows, weights and out must be 16-byte aligned", __func__);
  if (int rc = check_device()) return rc;
  if (encoder() == nullptr) return fail(B200_ERR_LAUNCH, "%s: the driver does not provide cuTensorMapEncodeTiled", __func__);

  const CUtensorMapDataType type = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const Operands op{rows, weight, weight2, total_rows, k, n, experts, ld_rows, type};

  GemmArgs args{};
  args.offsets = offsets;
  args.out = out;
  args.ld_out = ld_out;
  args.experts = static_cast<int>(experts);
  args.n = static_cast<int>(n);
  args.k = static_cast<int>(k);
  args.total_rows = static_cast<int>(total_rows);
  const uint32_t format = dtype == B200_BF16 ? 1u : 0u;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200_BF16) return weight2 ? run<__nv_bfloat16, true>(op, args, format, st) : run<__nv_bfloat16, false>(op, args, format, st);
  return weight2 ? run<__half, true>(op, args, format, st) : run<__half, false>(op, args, format, st);
}
