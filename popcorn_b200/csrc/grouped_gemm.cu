// Grouped expert GEMM for sm_100a: the dense step either side of the MoE permutation.
//
//   out[p, :] = rows[p, :] @ weight[e(p)]            (one weight matrix per expert)
//   out[p, :] = (rows[p, :] @ up[e]) * silu(rows[p, :] @ gate[e])   (DUAL: both projections and SwiGLU in one pass)
//
//   grad_rows[p, :] = grad_out[p, :] @ weight[e(p)]^T (+ a second pair)   (the weight read along its rows, in place)
//   grad_weight[e]  = rows[segment e]^T @ grad_out[segment e]             (contraction over the expert's rows)
//
// where e(p) is the expert whose segment offsets[e] <= p < offsets[e + 1] holds row p of the
// expert-major `rows` buffer that b200_moe_permute writes.  The gradients differ from the forward only in how
// the operands lie in shared memory (enum Mode below); roles, ring and accumulators are the same.  This is what the reference's
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
// Four rows of a 2-D tensor, given by four row coordinates, x columns on: 4 x (box width) elements land as four
// consecutive rows of the swizzled tile at `dst` (sm_100 tile::gather4).  The map's box is (box width, 1).
template <bool PAIR>
__device__ __forceinline__ void tma_gather4(uint32_t dst, uint64_t map, int x, int r0, int r1, int r2, int r3, uint32_t bar) {
  if constexpr (PAIR)
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar) : "memory");
  else
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar) : "memory");
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
//  K-major operand (the contraction index is contiguous in memory): rows of 128 bytes (64 K values), 8-row
//     groups 1024 bytes apart (stride offset); the leading offset is not used by swizzled K-major layouts and
//     is set to its canonical 1.
//  MN-major operand (the M or N index is contiguous): per K index a 128-byte line of 64 M/N values, 8-line K
//     groups 1024 bytes apart (stride offset), 64-value chunks one whole [slot K x 128 B] block apart (leading
//     offset).
constexpr uint64_t kDescFixed = (uint64_t(1) << 46) | (uint64_t(2) << 61);
constexpr uint64_t kDescKMajor = kDescFixed | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32);
template <int CTAS>
constexpr uint64_t kDescMnMajor = kDescFixed | (uint64_t(Ring<CTAS>::kBChunkBytes >> 4) << 16) | (uint64_t(1024 >> 4) << 32);

// Instruction descriptor of kind::f16: fp32 accumulate (bit 4), A/B format (0 fp16, 1 bf16) at bits 7
// and 10, A / B MN-major at bits 15 / 16, N >> 3 at bit 17, M >> 4 at bit 24 (M = 256 for a pair).
__host__ __device__ constexpr uint32_t instr_desc(uint32_t format, int ctas, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (format << 7) | (format << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
         (uint32_t(kBN >> 3) << 17) | (uint32_t((kBM * ctas) >> 4) << 24);
}

// What one launch computes.  Operand layouts as staged in shared memory:
//   kPlain   out = rows @ w                              A K-major,  B N-major
//   kSwiglu  out = silu(rows @ w) * (rows @ w2)          same; the two projections share one accumulator
//   kGateUp  out = [rows @ w | rows @ w2]                same; both halves stored, no activation
//   kDgrad   out = g @ w^T (+ g2 @ w2^T)                 A K-major,  B K-major (the weight read along its rows)
//   kWgrad   out[e] = rows[segment e]^T @ g[segment e]   A MN-major, B N-major; the contraction runs over the segment
enum Mode : int { kPlain = 0, kSwiglu = 1, kGateUp = 2, kDgrad = 3, kWgrad = 4 };

struct GemmArgs {
  const int32_t* offsets;  // [experts + 1], device
  void* out;
  int64_t ld_out;
  int experts;
  int n;           // output columns (per projection)
  int k;           // contraction length (kWgrad: unused, the segment length)
  int m;           // kWgrad: output rows per expert (the features of `rows`)
  int sources;     // kDgrad: 1 or 2 (A, B) operand pairs summed into one result
  int total_rows;  // rows of the token-major operands: nothing is read or stored past them, whatever `offsets` says
  uint32_t idesc;
  // forward modes only: when set, row p of the A operand is row gather[p] of the tensor map_a describes (the token
  // rows, in token order), fetched four rows per copy, and no expert-major copy of the rows has to exist
  const int32_t* gather;
};

struct Tile {
  int expert, row0, row_end, n0;  // output rows [row0, row_end) x columns from n0
  int k_lo, k_hi;                 // kWgrad: the segment's rows
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
  t.k_lo = t.k_hi = 0;
  return t;
}

// kWgrad: every expert owns tiles_m x tiles_n tiles of its [m, n] gradient, n fastest; an expert without rows
// still gets its tiles (they are written as zeros).  The CTAs running together then stream the SAME rows of the
// segment (all feature and gradient columns of a few hundred rows), so the operands come from DRAM once.
__device__ __forceinline__ Tile decode_wgrad_tile(int tile, const int* offsets, int tiles_per_expert, int tiles_n, int tile_rows, int m) {
  Tile t;
  t.expert = tile / tiles_per_expert;
  const int local = tile - t.expert * tiles_per_expert;
  const int mt = local / tiles_n;
  t.n0 = (local - mt * tiles_n) * kBN;
  t.row0 = t.expert * m + mt * tile_rows;
  t.row_end = (t.expert + 1) * m;
  t.k_lo = offsets[t.expert];
  t.k_hi = offsets[t.expert + 1];
  return t;
}

template <typename T, int MODE, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2, const GemmArgs p) {
  using R = Ring<CTAS>;
  constexpr bool PAIR = CTAS == 2;
  constexpr bool DUAL = MODE == kSwiglu || MODE == kGateUp;  // two weight tensors, 128 columns of each per tile
  constexpr bool WGRAD = MODE == kWgrad;
  constexpr bool B_K_MAJOR = MODE == kDgrad;
  constexpr int OUT_N = DUAL ? kBN / 2 : kBN;  // output columns per tile (and per projection)
  constexpr int ACC_COLS = MODE == kSwiglu ? kBN / 2 : kBN;  // accumulator columns the epilogue walks
  constexpr int STAGES = R::kStages;
  constexpr int TILE_ROWS = kBM * CTAS;
  constexpr int B_ROWS = kBN / CTAS;                 // kDgrad: weight rows (= accumulator columns) this CTA stages
  constexpr int kBSpanBytes = B_ROWS * 128;          // kDgrad: one 64-wide K span of them
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
  const int tiles_per_expert = WGRAD ? ((p.m + TILE_ROWS - 1) / TILE_ROWS) * tiles_n : 0;
  const int fixed_slots = p.sources * ((p.k + R::kSlotK - 1) / R::kSlotK);  // ring slots per tile unless kWgrad

  if (threadIdx.x == 0) {
    aborted = 0;
    int total = 0, lo = max(p.offsets[0], 0);
    seg[0] = lo;
    for (int e = 0; e < p.experts; ++e) {
      tile_start[e] = total;
      const int hi = min(p.offsets[e + 1], p.total_rows);
      seg[e + 1] = hi;
      if constexpr (WGRAD) total += tiles_per_expert;
      else total += (hi > lo ? (hi - lo + TILE_ROWS - 1) / TILE_ROWS : 0) * tiles_n;
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
  auto tile_at = [&](int tile) {
    if constexpr (WGRAD) return decode_wgrad_tile(tile, seg, tiles_per_expert, tiles_n, TILE_ROWS, p.m);
    else return decode_tile(tile, tile_start, seg, p.experts, OUT_N, TILE_ROWS, tiles_n);
  };
  // ring slots of the tile's main loop; a kWgrad tile of an expert without rows has none and never touches an accumulator
  auto slots_of = [&](const Tile& t) {
    if constexpr (WGRAD) return t.k_hi > t.k_lo ? (t.k_hi - t.k_lo + R::kSlotK - 1) / R::kSlotK : 0;
    else return fixed_slots;
  };

  bool gathering = false;
  if constexpr (!WGRAD && !B_K_MAJOR) gathering = p.gather != nullptr;
  if (warp == 0 && gathering) {
    // ------------------------------------------- producer, A rows gathered --
    // What the reference's lin1_kernel does with idx_ptr_Msum (src/popcorn/impls/momoe_tl.py:156-158): the tile's rows
    // are addressed through the permutation.  Lane l owns rows 4 l .. 4 l + 3 of this CTA's 128: it reads their token
    // ids once per tile and issues one four-row copy per 64-wide K span, so a whole span is ONE warp instruction;
    // lane 0 claims the ring slots and issues the weight copies as in the plain producer.  Measured: the copy engine
    // completes about one four-row copy per 45 cycles per SM, a third of what this tile shape consumes (gate/up +
    // SwiGLU on 524288 x 4096 x 1536: 26.6 ms against 9.5 ms from materialised rows), so the layer keeps its permute
    // pass and this path serves callers that cannot afford the expert-major copy of the rows.
    if constexpr (!WGRAD && !B_K_MAJOR) {
      uint32_t stage = 0, phase = 0, issued = 0;
      const uint32_t signal_addr = PAIR ? map_to_rank(full_addr, 0) : full_addr;
      const uint64_t a_map = reinterpret_cast<uint64_t>(&map_a);
      const uint64_t b_map = reinterpret_cast<uint64_t>(&map_b), b2_map = reinterpret_cast<uint64_t>(&map_b2);
      const int last_row = seg[p.experts] - 1;  // rows past a tile's segment still need a valid token id (results unused)
      bool stop = false;
      for (int tile = first_tile; tile < total_tiles && !stop; tile += tile_step) {
        const Tile t = tile_at(tile);
        const int row0 = t.row0 + static_cast<int>(rank) * kBM;
        int token[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) token[q] = __ldg(p.gather + min(row0 + 4 * lane + q, last_row));
        const uint64_t bm = (DUAL && PAIR && rank == 1) ? b2_map : b_map;
        const int col0 = t.n0 + ((!DUAL && PAIR) ? static_cast<int>(rank) * (kBN / 2) : 0);
        for (int k0 = 0; k0 < p.k; k0 += R::kSlotK) {
          uint32_t a_dst = 0, bar = 0;
          int ok = 1;
          if (lane == 0) {
            if (*abort_flag || !mbar_wait_addr(empty_addr + stage * 8, phase ^ 1u)) {
              *abort_flag = 1;
              ok = 0;
            } else {
              a_dst = ring_addr + stage * R::kStageBytes;
              bar = signal_addr + stage * 8;
              if (rank == 0) mbar_arrive_expect_addr(full_addr + stage * 8, CTAS * R::kStageBytes);
              ++issued;
              if (++stage == STAGES) {
                stage = 0;
                phase ^= 1u;
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) {
            stop = true;
            break;
          }
          a_dst = __shfl_sync(0xffffffffu, a_dst, 0);
          bar = __shfl_sync(0xffffffffu, bar, 0);
#pragma unroll
          for (int j = 0; j < R::kSub; ++j)  // past K: zero fill
            tma_gather4<PAIR>(a_dst + j * kASubBytes + lane * 512, a_map, k0 + j * kBK, token[0], token[1], token[2], token[3], bar);
          if (lane == 0) {
            const uint32_t b_dst = a_dst + R::kABytes;
#pragma unroll
            for (int c = 0; c < R::kChunks; ++c) {
              if (DUAL && !PAIR && c >= R::kChunks / 2) tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, b2_map, t.n0 + (c - R::kChunks / 2) * 64, k0, t.expert, bar);
              else tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, bm, col0 + c * 64, k0, t.expert, bar);
            }
          }
        }
      }
      if (lane == 0 && *abort_flag && rank == 0) {
        for (uint32_t k = issued > STAGES ? issued - STAGES : 0; k < issued; ++k) (void)mbar_wait(&full[k % STAGES], (k / STAGES) & 1u);
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------- producer --
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      // the barrier the copies complete on: this CTA's own, or in a pair the leader's
      const uint32_t signal_addr = PAIR ? map_to_rank(full_addr, 0) : full_addr;
      const uint64_t a_map = reinterpret_cast<uint64_t>(&map_a), a2_map = reinterpret_cast<uint64_t>(&map_a2);
      const uint64_t b_map = reinterpret_cast<uint64_t>(&map_b), b2_map = reinterpret_cast<uint64_t>(&map_b2);
      // claims the next ring slot; false after a wait that ran out
      auto acquire = [&](uint32_t& a_dst, uint32_t& b_dst, uint32_t& bar) {
        if (!mbar_wait_addr(empty_addr + stage * 8, phase ^ 1u)) {
          *abort_flag = 1;
          return false;
        }
        a_dst = ring_addr + stage * R::kStageBytes;
        b_dst = a_dst + R::kABytes;
        bar = signal_addr + stage * 8;
        if (rank == 0) mbar_arrive_expect_addr(full_addr + stage * 8, CTAS * R::kStageBytes);  // in a pair both CTAs' bytes land here
        ++issued;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        return true;
      };
      for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step) {
        const Tile t = tile_at(tile);
        uint32_t a_dst, b_dst, bar;
        if constexpr (WGRAD) {
          // A: 64-feature chunks of rows^T, B: 64-column chunks of the gradient, both indexed by the segment's rows.
          // The maps see the buffers as [row][window line][feature] with the SAME stride for the two outer
          // dimensions, so a box placed at window line -(pad) reads zeros into its first `pad` lines and rows
          // row0 .. row0 + valid - 1 into the rest: the last slot of a segment is padded with zeros, not with the
          // next expert's rows.
          const int m0 = t.row0 - t.expert * p.m + static_cast<int>(rank) * kBM;
          const int col0 = t.n0 + (PAIR ? static_cast<int>(rank) * (kBN / 2) : 0);
          for (int r0 = t.k_lo; r0 < t.k_hi; r0 += R::kSlotK) {
            if (!acquire(a_dst, b_dst, bar)) break;
            const int line0 = min(t.k_hi - r0, R::kSlotK) - R::kSlotK;  // <= 0
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c) tma_3d<PAIR>(a_dst + c * R::kBChunkBytes, a_map, m0 + c * 64, line0, r0, bar);
#pragma unroll
            for (int c = 0; c < R::kChunks; ++c) tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, b_map, col0 + c * 64, line0, r0, bar);
          }
        } else if constexpr (B_K_MAJOR) {
          const int row0 = t.row0 + static_cast<int>(rank) * kBM;
          const int col0 = t.n0 + (PAIR ? static_cast<int>(rank) * (kBN / 2) : 0);
          for (int s = 0; s < p.sources && !*abort_flag; ++s) {
            const uint64_t am = s ? a2_map : a_map, bm = s ? b2_map : b_map;
            for (int k0 = 0; k0 < p.k; k0 += R::kSlotK) {
              if (!acquire(a_dst, b_dst, bar)) break;
#pragma unroll
              for (int j = 0; j < R::kSub; ++j) tma_2d<PAIR>(a_dst + j * kASubBytes, am, k0 + j * kBK, row0, bar);  // past K: zero fill
#pragma unroll
              for (int j = 0; j < R::kSub; ++j) tma_3d<PAIR>(b_dst + j * kBSpanBytes, bm, k0 + j * kBK, col0, t.expert, bar);
            }
          }
        } else {
          // this CTA's share of the 256 accumulator columns: all of them alone, one half in a pair
          // (DUAL: columns 0-127 are the first projection, 128-255 the second projection of the same output columns)
          const uint64_t bm = (DUAL && PAIR && rank == 1) ? b2_map : b_map;
          const int row0 = t.row0 + static_cast<int>(rank) * kBM;
          const int col0 = t.n0 + ((!DUAL && PAIR) ? static_cast<int>(rank) * (kBN / 2) : 0);
          for (int k0 = 0; k0 < p.k; k0 += R::kSlotK) {
            if (!acquire(a_dst, b_dst, bar)) break;
#pragma unroll
            for (int j = 0; j < R::kSub; ++j) tma_2d<PAIR>(a_dst + j * kASubBytes, a_map, k0 + j * kBK, row0, bar);  // past K: zero fill
#pragma unroll
            for (int c = 0; c < R::kChunks; ++c) {
              if (DUAL && !PAIR && c >= R::kChunks / 2) tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, b2_map, t.n0 + (c - R::kChunks / 2) * 64, k0, t.expert, bar);
              else tma_3d<PAIR>(b_dst + c * R::kBChunkBytes, bm, col0 + c * 64, k0, t.expert, bar);
            }
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
      constexpr uint64_t desc_a = WGRAD ? kDescMnMajor<CTAS> : kDescKMajor;
      constexpr uint64_t desc_b = B_K_MAJOR ? kDescKMajor : kDescMnMajor<CTAS>;
      const uint32_t a_hi = static_cast<uint32_t>(desc_a >> 32), b_hi = static_cast<uint32_t>(desc_b >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(desc_a) | (ring_addr >> 4);
      const uint32_t b_lo0 = static_cast<uint32_t>(desc_b) | ((ring_addr + R::kABytes) >> 4);
      const uint32_t idesc = p.idesc;
      for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step) {
        int slots = fixed_slots;
        if constexpr (WGRAD) {
          slots = slots_of(tile_at(tile));
          if (slots == 0) continue;
        }
        const uint32_t acc = local & 1u;
        if (!mbar_wait_addr(acc_empty_addr + acc * 8, ((local >> 1) & 1u) ^ 1u)) {
          *abort_flag = 1;
          break;
        }
        ++local;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        uint32_t accumulate = 0;
        for (int s = 0; s < slots; ++s) {
          if (!mbar_wait_addr(full_addr + stage * 8, phase)) {
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          // descriptor start fields advance in 16-byte units: a ring slot, then per MMA (16 K values) 32 bytes along a
          // K-major operand's swizzled 128-byte rows (a new block every 64 K values) or 16 lines = 2048 bytes of an
          // MN-major operand
          const uint32_t a_lo = a_lo0 + stage * (R::kStageBytes >> 4), b_lo = b_lo0 + stage * (R::kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < R::kSlotK / kUmmaK; ++k) {
            constexpr int kPerSpan = kBK / kUmmaK;
            const uint32_t a_step = WGRAD ? k * (kUmmaK * 128 >> 4) : (k / kPerSpan) * (kASubBytes >> 4) + (k % kPerSpan) * (kUmmaK * 2 >> 4);
            const uint32_t b_step = B_K_MAJOR ? (k / kPerSpan) * (kBSpanBytes >> 4) + (k % kPerSpan) * (kUmmaK * 2 >> 4) : k * (kUmmaK * 128 >> 4);
            mma_issue<PAIR>(d_tmem, a_lo + a_step, b_lo + b_step, a_hi, b_hi, idesc, accumulate);
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
    for (int tile = first_tile; tile < total_tiles && !*abort_flag; tile += tile_step) {
      const Tile t = tile_at(tile);
      const bool zeros = slots_of(t) == 0;  // kWgrad, expert without rows: no accumulator was produced
      const uint32_t acc = local & 1u;
      if (!zeros) {
        // one lane polls for the whole warp
        const int ready = __shfl_sync(0xffffffffu, lane == 0 ? static_cast<int>(mbar_wait(&acc_full[acc], (local >> 1) & 1u)) : 0, 0);
        if (!ready) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int warp_row0 = t.row0 + static_cast<int>(rank) * kBM + quarter * 32;
      uint4(*mine)[8] = staging[quarter];
      // 64 output columns per step (one 128-byte staging row per lane).  The tensor-memory loads of the NEXT step are
      // issued before this step's conversion, transpose and stores, so their latency hides behind them (the fused
      // SwiGLU form needs both projections' columns per step and does not prefetch: its main loop is long anyway).
      constexpr int STEPS = ACC_COLS / 64;
      constexpr bool PREFETCH = MODE != kSwiglu;
      uint32_t held[2][64], second[MODE == kSwiglu ? 64 : 1];
      auto fetch = [&](uint32_t (&v)[64], int step) {
        tmem_load_32(taddr + step * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_load_32(taddr + step * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      };
      if (!zeros) fetch(held[0], 0);
#pragma unroll
      for (int step = 0; step < STEPS; ++step) {
        uint32_t(&v)[64] = held[PREFETCH ? (step & 1) : 0];
        uint32_t packed[32];
        if (zeros) {
#pragma unroll
          for (int j = 0; j < 32; ++j) packed[j] = 0u;
        } else {
          if constexpr (MODE == kSwiglu) {
            tmem_load_32(taddr + OUT_N + step * 64, *reinterpret_cast<uint32_t(*)[32]>(&second[0]));
            tmem_load_32(taddr + OUT_N + step * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&second[32]));
          }
          tmem_load_wait();
          if constexpr (PREFETCH) {
            if (step + 1 < STEPS) fetch(held[(step + 1) & 1], step + 1);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float lo = __uint_as_float(v[2 * j]), hi = __uint_as_float(v[2 * j + 1]);
            if constexpr (MODE == kSwiglu) {
              // columns 0..127 of the accumulator hold rows @ gate, 128..255 rows @ up
              lo = __fmul_rn(silu_f32<1>(lo), __uint_as_float(second[2 * j]));
              hi = __fmul_rn(silu_f32<1>(hi), __uint_as_float(second[2 * j + 1]));
            }
            packed[j] = Num<T>::pack2(lo, hi);
          }
          if constexpr (!PREFETCH) {
            if (step + 1 < STEPS) fetch(held[0], step + 1);  // the registers are free again
          }
        }
        // lane = row: its 64 columns are eight 16-byte pieces of the 128-byte staging row (piece index xor-ed with
        // the row so that neither these writes nor the transposed reads conflict on banks)
#pragma unroll
        for (int q = 0; q < 8; ++q)
          mine[lane][q ^ (lane & 7)] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        // 64 finished columns of 32 rows: write them out as whole 128-byte row segments, four rows per instruction
        __syncwarp();
        const int piece = lane & 7;
        int tile_col = step * 64 + piece * 8, shift = 0;  // column within the tile; kGateUp: the second projection lies n columns further
        if (MODE == kGateUp && tile_col >= OUT_N) {
          tile_col -= OUT_N;
          shift = p.n;
        }
        const int col = t.n0 + tile_col;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          const int row = warp_row0 + r;
          if (row < t.row_end && col < p.n)
            st_stream(out + static_cast<int64_t>(row) * p.ld_out + col + shift, mine[r][piece ^ (r & 7)]);
        }
        __syncwarp();
      }
      if (!zeros) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) remote_arrive(map_to_rank(smem_addr(&acc_empty[acc]), 0));  // the leader issues the MMAs
          else mbar_arrive(&acc_empty[acc]);
        }
        ++local;
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

// A 2- or 3-dimensional map of 16-bit elements: 128-byte swizzle, zero fill outside; strides in elements.
bool encode(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const int64_t (&dims)[3], const int64_t (&strides)[2],
            const int (&box)[3]) {
  cuuint64_t d[3], s[2];
  cuuint32_t b[3], elem[3] = {1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    d[i] = static_cast<cuuint64_t>(dims[i]);
    b[i] = static_cast<cuuint32_t>(box[i]);
  }
  for (int i = 0; i < 2; ++i) s[i] = static_cast<cuuint64_t>(strides[i]) * 2;
  return encoder()(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// token-major operand [total_rows, width], row stride ld: box 64 (contraction values) x 128 (rows).
bool encode_rows(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t total_rows, int64_t width, int64_t ld) {
  return encode(map, type, 2, base, {width, total_rows, 1}, {ld, 0}, {kBK, kBM, 1});
}

// the same operand for four-row gathered copies (tile::gather4): the box is ONE row of 64 contraction values; the
// instruction names four row coordinates and copies the box once per row.  (A box of four rows makes the copy an
// illegal instruction.)
bool encode_gathered_rows(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t rows, int64_t width, int64_t ld) {
  return encode(map, type, 2, base, {width, rows, 1}, {ld, 0}, {kBK, 1, 1});
}

// weight [experts, k, n], n contiguous, read along n: box 64 (n) x slot_k (k) x 1 (expert).
bool encode_weight(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t experts, int64_t k, int64_t n, int slot_k) {
  return encode(map, type, 3, base, {n, k, experts}, {n, n * k}, {64, slot_k, 1});
}

// the same weight read along its rows (the contraction runs over n): box 64 (n) x rows (k) x 1 (expert).
bool encode_weight_rows(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t experts, int64_t k, int64_t n, int rows) {
  return encode(map, type, 3, base, {n, k, experts}, {n, n * k}, {64, rows, 1});
}

// token-major operand [total_rows, width] for a contraction over rows: seen as [row][window line][column] with the
// row stride for BOTH outer dimensions, element (row r, line j, column c) = buffer[r + j][c].  A box of slot_k lines
// placed at line -(pad) of row r0 reads `pad` lines of zeros and then rows r0 .. r0 + slot_k - pad - 1.
bool encode_window(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t total_rows, int64_t width, int64_t ld, int slot_k) {
  return encode(map, type, 3, base, {width, slot_k, total_rows}, {ld, ld}, {64, slot_k, 1});
}

// B200_GEMM_PAIR=0 in the environment runs every CTA on its own (cta_group::1); read at every call (a getenv is a
// short scan of the environment block; tests flip the switch between calls).
bool pair_enabled() {
  const char* v = std::getenv("B200_GEMM_PAIR");
  return !(v && v[0] == '0');
}

// Per (kernel instantiation, device): the dynamic shared-memory attribute has been raised, and how many CTAs a launch
// gets (for pairs: twice the number of clusters that can be resident, or kNoClusters).  Both are properties of the
// kernel and the device, so a call pays for them once instead of on every launch.
constexpr int kMaxDevicesGemm = 64;
struct LaunchPlan {
  std::mutex mutex;
  int ctas[kMaxDevicesGemm] = {};  // 0: not looked up yet
};

constexpr int kNoClusters = -1000;  // run_with<., ., 2>: no cluster of two CTAs can be resident; the caller runs single CTAs instead

// What the tensor maps of one call describe (widths and strides in elements).
struct Operands {
  const void *a, *b, *a2, *b2;  // a: token-major [total_rows, .]; b: weight (kWgrad: the token-major gradient)
  int64_t total_rows, experts;
  int64_t k, n;                 // the WEIGHT's shape [experts, k, n], whichever way the mode contracts
  int64_t ld_a, ld_b;           // row strides of the token-major operands (ld_b: kWgrad only)
  CUtensorMapDataType type;
  int64_t gather_rows = 0;      // forward modes: > 0 when `a` is the token-order tensor [gather_rows, k] read through an index
};

template <int MODE, int CTAS>
bool encode_operands(const Operands& op, CUtensorMap* a, CUtensorMap* b, CUtensorMap* a2, CUtensorMap* b2) {
  constexpr int slot_k = Ring<CTAS>::kSlotK;
  const void* second_a = op.a2 ? op.a2 : op.a;
  const void* second_b = op.b2 ? op.b2 : op.b;
  if constexpr (MODE == kWgrad) {
    return encode_window(a, op.type, op.a, op.total_rows, op.k, op.ld_a, slot_k) &&
           encode_window(b, op.type, op.b, op.total_rows, op.n, op.ld_b, slot_k) &&
           encode_window(a2, op.type, op.a, op.total_rows, op.k, op.ld_a, slot_k) &&
           encode_window(b2, op.type, op.b, op.total_rows, op.n, op.ld_b, slot_k);
  } else if constexpr (MODE == kDgrad) {
    return encode_rows(a, op.type, op.a, op.total_rows, op.n, op.ld_a) && encode_rows(a2, op.type, second_a, op.total_rows, op.n, op.ld_a) &&
           encode_weight_rows(b, op.type, op.b, op.experts, op.k, op.n, kBN / CTAS) &&
           encode_weight_rows(b2, op.type, second_b, op.experts, op.k, op.n, kBN / CTAS);
  } else {
    const bool rows_ok = op.gather_rows > 0
                             ? encode_gathered_rows(a, op.type, op.a, op.gather_rows, op.k, op.ld_a) &&
                                   encode_gathered_rows(a2, op.type, op.a, op.gather_rows, op.k, op.ld_a)
                             : encode_rows(a, op.type, op.a, op.total_rows, op.k, op.ld_a) && encode_rows(a2, op.type, op.a, op.total_rows, op.k, op.ld_a);
    return rows_ok && encode_weight(b, op.type, op.b, op.experts, op.k, op.n, slot_k) && encode_weight(b2, op.type, second_b, op.experts, op.k, op.n, slot_k);
  }
}

template <typename T, int MODE, int CTAS>
int run_with(const char* what, const Operands& op, GemmArgs args, uint32_t format, cudaStream_t st) {
  alignas(64) CUtensorMap a, b, a2, b2;
  if (!encode_operands<MODE, CTAS>(op, &a, &b, &a2, &b2)) return fail(B200_ERR_LAUNCH, "%s: tensor map encoding failed", what);
  auto kernel = grouped_gemm_kernel<T, MODE, CTAS>;
  constexpr int smem = Ring<CTAS>::kSmemBytes;
  static LaunchPlan plan;  // one per instantiation
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevicesGemm) {
    (void)cudaGetLastError();
    return fail(B200_ERR_DEVICE, "%s: no usable CUDA device is current", what);
  }
  args.idesc = instr_desc(format, CTAS, MODE == kWgrad, MODE != kDgrad);
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
  int ctas = 0;
  {
    std::lock_guard<std::mutex> lock(plan.mutex);
    if (plan.ctas[device] == 0) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(B200_ERR_LAUNCH, "%s: cannot reserve %d bytes of shared memory", what, smem);
      }
      int found = sm_count();
      if (CTAS == 2) {
        // persistent pairs: as many clusters as can be resident at once (an odd SM of a processing cluster has no partner)
        config.gridDim = dim3(static_cast<unsigned>(found & ~1));
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters < 1) {
          (void)cudaGetLastError();
          found = kNoClusters;
        } else {
          found = 2 * std::min(clusters, found / 2);
        }
      }
      plan.ctas[device] = found;
    }
    ctas = plan.ctas[device];
  }
  if (ctas == kNoClusters) return kNoClusters;
  config.gridDim = dim3(static_cast<unsigned>(ctas));
  if (pdl_enabled()) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = ++n_attrs;
  }
  (void)cudaLaunchKernelEx(&config, kernel, a, b, a2, b2, args);
  return after_launch(CTAS == 2 ? "grouped_gemm_kernel (pairs)" : "grouped_gemm_kernel");
}

template <typename T, int MODE>
int run(const char* what, const Operands& op, const GemmArgs& args, uint32_t format, cudaStream_t st) {
  if (pair_enabled()) {
    const int rc = run_with<T, MODE, 2>(what, op, args, format, st);
    if (rc != kNoClusters) return rc;
  }
  return run_with<T, MODE, 1>(what, op, args, format, st);
}

template <int MODE>
int run_typed(const char* what, int dtype, const Operands& op, const GemmArgs& args, cudaStream_t st) {
  if (dtype == B200_BF16) return run<__nv_bfloat16, MODE>(what, op, args, 1u, st);
  return run<__half, MODE>(what, op, args, 0u, st);
}

// Checks shared by the four entry points; B200_OK with *skip = true when there is nothing to compute.
int check_common(const char* what, int dtype, int64_t total_rows, int64_t k, int64_t n, int64_t experts, const int64_t (&lds)[2],
                 const int64_t (&ld_min)[2], const void* const (&ptrs)[6], const int32_t* offsets) {
  if (dtype != B200_BF16 && dtype != B200_F16)
    return fail(B200_ERR_DTYPE, "%s: dtype %d not supported (bf16 or fp16 operands, fp32 accumulation)", what, dtype);
  if (total_rows < 0 || k < 0 || n < 0 || experts < 0) return fail(B200_ERR_SHAPE, "%s: negative size", what);
  if (experts > kMaxExperts) return fail(B200_ERR_SHAPE, "%s: experts=%lld exceeds %d", what, (long long)experts, kMaxExperts);
  if (total_rows > 0x7fffffffLL - 2 * kBM || k > 0x3fffffffLL || n > 0x3fffffffLL) return fail(B200_ERR_SHAPE, "%s: size out of range", what);
  if (k % 8 != 0 || n % 8 != 0 || lds[0] % 8 != 0 || lds[1] % 8 != 0)
    return fail(B200_ERR_SHAPE, "%s: k, n and the row strides must be multiples of 8 elements (16-byte rows for the tensor maps)", what);
  if (lds[0] < ld_min[0] || lds[1] < ld_min[1]) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than the row", what);
  for (const void* ptr : ptrs)
    if (ptr && !aligned(ptr, 16)) return fail(B200_ERR_ALIGNMENT, "%s: operands and results must be 16-byte aligned", what);
  if (!aligned(offsets, 4)) return fail(B200_ERR_ALIGNMENT, "%s: offsets must be 4-byte aligned", what);
  return B200_OK;
}

CUtensorMapDataType map_type(int dtype) { return dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16; }

}  // namespace

unsigned int gemm_wait_timeouts() { return read_wait_timeouts(); }

}  // namespace b200

using namespace b200;

namespace {

// The three forward forms: out = rows @ weight, the fused SwiGLU of two projections, or both projections side by side.
int forward(const char* what, int mode, const void* rows, const void* weight, const void* weight2, const int32_t* offsets, void* out,
            int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_out, int dtype, void* stream,
            const int32_t* gather = nullptr, int64_t gather_rows = 0) {
  if (int rc = check_common(what, dtype, total_rows, k, n, experts, {ld_rows, ld_out}, {k, mode == kGateUp ? 2 * n : n},
                            {rows, weight, weight2, out, nullptr, nullptr}, offsets))
    return rc;
  if (total_rows == 0 || n == 0 || experts == 0) return B200_OK;
  if (!rows || !weight || !offsets || !out || (mode != kPlain && !weight2)) return fail(B200_ERR_NULL_POINTER, "%s: null pointer", what);
  if (k == 0) return fail(B200_ERR_SHAPE, "%s: k must be positive", what);
  if (int rc = check_device()) return rc;
  if (encoder() == nullptr) return fail(B200_ERR_LAUNCH, "%s: the driver does not provide cuTensorMapEncodeTiled", what);
  Operands op{rows, weight, nullptr, weight2, total_rows, experts, k, n, ld_rows, 0, map_type(dtype)};
  op.gather_rows = gather ? gather_rows : 0;
  GemmArgs args{};
  args.offsets = offsets;
  args.out = out;
  args.ld_out = ld_out;
  args.experts = static_cast<int>(experts);
  args.n = static_cast<int>(n);
  args.k = static_cast<int>(k);
  args.sources = 1;
  args.total_rows = static_cast<int>(total_rows);
  args.gather = gather;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode == kSwiglu) return run_typed<kSwiglu>(what, dtype, op, args, st);
  if (mode == kGateUp) return run_typed<kGateUp>(what, dtype, op, args, st);
  return run_typed<kPlain>(what, dtype, op, args, st);
}

}  // namespace

extern "C" int b200_moe_grouped_gemm(const void* rows, const void* weight, const void* weight2, const int32_t* offsets, void* out,
                                     int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_out,
                                     int dtype, void* stream) {
  return forward(__func__, weight2 ? kSwiglu : kPlain, rows, weight, weight2, offsets, out, total_rows, k, n, experts, ld_rows, ld_out, dtype, stream);
}

extern "C" int b200_moe_grouped_gemm_gathered(const void* x, const int32_t* perm, const void* weight, const void* weight2, const int32_t* offsets,
                                              void* out, int64_t tokens, int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ldx,
                                              int64_t ld_out, int dtype, void* stream) {
  if (tokens < 0 || tokens > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: tokens out of range", __func__);
  if (total_rows > 0 && n > 0 && experts > 0) {
    if (!perm) return fail(B200_ERR_NULL_POINTER, "%s: perm is NULL", __func__);
    if (!aligned(perm, 4)) return fail(B200_ERR_ALIGNMENT, "%s: perm must be 4-byte aligned", __func__);
    if (tokens == 0) return fail(B200_ERR_SHAPE, "%s: rows to gather but no tokens", __func__);
  }
  return forward(__func__, weight2 ? kSwiglu : kPlain, x, weight, weight2, offsets, out, total_rows, k, n, experts, ldx, ld_out, dtype, stream,
                 perm, tokens);
}

extern "C" int b200_moe_grouped_gemm_gate_up(const void* rows, const void* gate_weight, const void* up_weight, const int32_t* offsets, void* out,
                                             int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_out,
                                             int dtype, void* stream) {
  return forward(__func__, kGateUp, rows, gate_weight, up_weight, offsets, out, total_rows, k, n, experts, ld_rows, ld_out, dtype, stream);
}

extern "C" int b200_moe_grouped_gemm_dgrad(const void* grad_out, const void* weight, const void* grad_out2, const void* weight2,
                                           const int32_t* offsets, void* grad_rows, int64_t total_rows, int64_t k, int64_t n, int64_t experts,
                                           int64_t ld_grad, int64_t ld_out, int dtype, void* stream) {
  if (int rc = check_common(__func__, dtype, total_rows, k, n, experts, {ld_grad, ld_out}, {n, k},
                            {grad_out, weight, grad_out2, weight2, grad_rows, nullptr}, offsets))
    return rc;
  if ((grad_out2 == nullptr) != (weight2 == nullptr)) return fail(B200_ERR_NULL_POINTER, "%s: grad_out2 and weight2 go together", __func__);
  if (total_rows == 0 || k == 0 || experts == 0) return B200_OK;
  if (!grad_out || !weight || !offsets || !grad_rows) return fail(B200_ERR_NULL_POINTER, "%s: null pointer", __func__);
  if (n == 0) return fail(B200_ERR_SHAPE, "%s: n must be positive", __func__);
  if (int rc = check_device()) return rc;
  if (encoder() == nullptr) return fail(B200_ERR_LAUNCH, "%s: the driver does not provide cuTensorMapEncodeTiled", __func__);
  const Operands op{grad_out, weight, grad_out2, weight2, total_rows, experts, k, n, ld_grad, 0, map_type(dtype)};
  GemmArgs args{};
  args.offsets = offsets;
  args.out = grad_rows;
  args.ld_out = ld_out;
  args.experts = static_cast<int>(experts);
  args.n = static_cast<int>(k);  // the result has the weight's k columns, the contraction runs over its n
  args.k = static_cast<int>(n);
  args.sources = grad_out2 ? 2 : 1;
  args.total_rows = static_cast<int>(total_rows);
  return run_typed<kDgrad>(__func__, dtype, op, args, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_moe_grouped_gemm_wgrad(const void* rows, const void* grad_out, const int32_t* offsets, void* grad_weight,
                                           int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_grad,
                                           int dtype, void* stream) {
  if (int rc = check_common(__func__, dtype, total_rows, k, n, experts, {ld_rows, ld_grad}, {k, n},
                            {rows, grad_out, grad_weight, nullptr, nullptr, nullptr}, offsets))
    return rc;
  if (k == 0 || n == 0 || experts == 0) return B200_OK;
  if (experts * k > 0x7fffffffLL - 2 * kBM) return fail(B200_ERR_SHAPE, "%s: experts * k out of range", __func__);
  const int64_t tiles = experts * ((k + kBM - 1) / kBM) * ((n + kBN - 1) / kBN);
  if (tiles > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: too many output tiles", __func__);
  if (!offsets || !grad_weight || (total_rows > 0 && (!rows || !grad_out))) return fail(B200_ERR_NULL_POINTER, "%s: null pointer", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (total_rows == 0) {  // no rows at all: every expert's gradient is zero
    if (cudaMemsetAsync(grad_weight, 0, static_cast<size_t>(experts * k * n) * 2, st) != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(B200_ERR_LAUNCH, "%s: clearing the result failed", __func__);
    }
    return B200_OK;
  }
  if (encoder() == nullptr) return fail(B200_ERR_LAUNCH, "%s: the driver does not provide cuTensorMapEncodeTiled", __func__);
  const Operands op{rows, grad_out, nullptr, nullptr, total_rows, experts, k, n, ld_rows, ld_grad, map_type(dtype)};
  GemmArgs args{};
  args.offsets = offsets;
  args.out = grad_weight;
  args.ld_out = n;
  args.experts = static_cast<int>(experts);
  args.n = static_cast<int>(n);
  args.k = 0;
  args.m = static_cast<int>(k);
  args.sources = 1;
  args.total_rows = static_cast<int>(total_rows);
  return run_typed<kWgrad>(__func__, dtype, op, args, st);
}
