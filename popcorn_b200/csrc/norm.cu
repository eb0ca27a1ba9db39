// RMSNorm and residual-add + RMSNorm for sm_100a.
//
// Bound: HBM. Each input row is read from global memory exactly once and each
// output row written once: the row lives in registers between the sum-of-squares
// pass and the scaling pass (`rms_rows_kernel`).  Rows too long for registers,
// or not 16-byte aligned, go through `rms_stream_kernel`, which re-reads the row
// (served by L2 for any row that fits there).
//
// Arithmetic follows src/popcorn/kernels/_utils.py:14-16 (rms),
// src/popcorn/kernels/rms_norm.py:29-30 and src/popcorn/kernels/add_rms_norm.py:22-23
// of the reference, including its intermediate roundings to the storage type.
#include <algorithm>
#include <cstdlib>

#include <type_traits>

#include "common.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

// 1 / sqrt(sum / cols + eps), all IEEE-rounded fp32 steps (the reference computes
// mean = sum / n, then torch.rsqrt, which on the host is 1 / sqrt).
__device__ __forceinline__ float inv_rms(float sumsq, float cols, float eps) {
  return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, cols), eps)));
}

// y for one element: round_T(round_T(h * r) * w) [+ bias, rounded again]
template <typename T>
__device__ __forceinline__ float scale_one(float h, float r, float w, float b, bool has_bias) {
  float n = Num<T>::rt(__fmul_rn(h, r));
  float y = Num<T>::rt(__fmul_rn(n, w));
  if (has_bias) y = Num<T>::rt(__fadd_rn(y, b));
  return y;
}

// One row per group of TPR threads, ITEMS 128-bit words per thread, the row held
// in registers.  THREADS / TPR rows per CTA.  ADD selects add_rms_norm.
// Sum over the TPR consecutive lanes of a row group (TPR <= 32, a power of two).
template <int TPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T, int TPR, int ITEMS, bool ADD, int RU>
__global__ void __launch_bounds__(TPR < 256 ? 256 : TPR)
rms_rows_kernel(const T* x, const T* res, const T* __restrict__ weight,
                const T* __restrict__ bias, T* y, T* s_out,
                int64_t rows, int nvec, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                float cols_f, float eps, float offset) {
  constexpr int V = Num<T>::kVec;
  constexpr int THREADS = TPR < 256 ? 256 : TPR;
  constexpr int GROUPS = THREADS / TPR;  // row groups per CTA; each owns RU consecutive rows
  constexpr int WARPS_PER_ROW = TPR / 32;
  static_assert(RU == 1 || TPR <= 32, "several rows per group only for rows that fit a warp");
  pdl_prologue();

  const int tid = threadIdx.x;
  const int sub = tid / TPR;
  const int lane_in_row = tid % TPR;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * GROUPS + sub) * RU;

  uint4 data[RU][ITEMS];
  uint4 rdata[ADD ? RU : 1][ADD ? ITEMS : 1];
  bool ok[RU][ITEMS];
  // issue every load of every row before touching any of them
#pragma unroll
  for (int u = 0; u < RU; ++u) {
    const int64_t row = row0 + u;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int v = lane_in_row + i * TPR;
      ok[u][i] = row < rows && v < nvec;
      data[u][i] = make_uint4(0, 0, 0, 0);
      if (ok[u][i]) data[u][i] = ld_stream(x + row * ldx + static_cast<int64_t>(v) * V);
      if constexpr (ADD) {
        rdata[u][i] = make_uint4(0, 0, 0, 0);
        if (ok[u][i]) rdata[u][i] = ld_stream(res + row * ldr + static_cast<int64_t>(v) * V);
      }
    }
  }
  const bool has_bias = bias != nullptr;

#pragma unroll
  for (int u = 0; u < RU; ++u) {
    const int64_t row = row0 + u;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      float f[V];
      Num<T>::unpack(data[u][i], f);
      if constexpr (ADD) {
        float g[V];
        Num<T>::unpack(rdata[u][i], g);
#pragma unroll
        for (int j = 0; j < V; ++j) f[j] = __fadd_rn(f[j], g[j]);
        data[u][i] = Num<T>::pack(f);  // s = x + residual, rounded to T by the pack
        Num<T>::unpack(data[u][i], f);
        if (ok[u][i]) st_stream(s_out + row * lds + static_cast<int64_t>(lane_in_row + i * TPR) * V, data[u][i]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) acc = __fmaf_rn(f[j], f[j], acc);
    }

    acc = group_sum<TPR>(acc);
    if constexpr (WARPS_PER_ROW > 1) {
      __shared__ float partial[THREADS / 32];
      const int warp = tid / 32;
      if ((tid & 31) == 0) partial[warp] = acc;
      __syncthreads();
      float total = 0.f;
      const int first = sub * WARPS_PER_ROW;
#pragma unroll
      for (int w = 0; w < WARPS_PER_ROW; ++w) total = __fadd_rn(total, partial[first + w]);
      acc = total;
    }
    const float r = inv_rms(acc, cols_f, eps);

#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      if (!ok[u][i]) continue;
      const int64_t col = static_cast<int64_t>(lane_in_row + i * TPR) * V;
      if constexpr (sizeof(T) == 4) {
        float f[V], w[V], b[V];
        Num<T>::unpack(data[u][i], f);
        Num<T>::unpack(ld_reuse(weight + col), w);
        if (has_bias) Num<T>::unpack(ld_reuse(bias + col), b);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float wj = ADD ? __fadd_rn(w[j], offset) : w[j];
          f[j] = __fmul_rn(__fmul_rn(f[j], r), wj);
          if (has_bias) f[j] = __fadd_rn(f[j], b[j]);
        }
        st_stream(y + row * ldy + col, Num<T>::pack(f));
      } else {
        // 16-bit: h * r in fp32, one packed rounding to T, then the packed product with the weight
        // word (a product of two 16-bit values is rounded once, as in the reference)
        const uint4 wv = ld_reuse(weight + col);
        uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        if (ADD && offset != 0.f) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float lo, hi;
            Num<T>::unpack2(ww[j], lo, hi);
            ww[j] = Num<T>::pack2(__fadd_rn(lo, offset), __fadd_rn(hi, offset));
          }
        }
        const uint32_t wd[4] = {data[u][i].x, data[u][i].y, data[u][i].z, data[u][i].w};
        uint32_t wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          Num<T>::unpack2(wd[j], lo, hi);
          wo[j] = Num<T>::mul2(Num<T>::pack2(__fmul_rn(lo, r), __fmul_rn(hi, r)), ww[j]);
        }
        if (has_bias) {
          const uint4 bv = ld_reuse(bias + col);
          const uint32_t wb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float lo, hi, blo, bhi;
            Num<T>::unpack2(wo[j], lo, hi);
            Num<T>::unpack2(wb[j], blo, bhi);
            wo[j] = Num<T>::pack2(__fadd_rn(lo, blo), __fadd_rn(hi, bhi));
          }
        }
        st_stream(y + row * ldy + col, make_uint4(wo[0], wo[1], wo[2], wo[3]));
      }
    }
  }
}

// Any width, any alignment: one CTA per row, scalar accesses, two passes.
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
rms_stream_kernel(const T* x, const T* res, const T* __restrict__ weight,
                  const T* __restrict__ bias, T* y, T* s_out,
                  int64_t cols, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                  float cols_f, float eps, float offset) {
  pdl_prologue();
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  const T* rr = ADD ? res + row * ldr : nullptr;
  T* sr = ADD ? s_out + row * lds : nullptr;
  float acc = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float h = Num<T>::up(xr[c]);
    if (ADD) {
      h = Num<T>::rt(__fadd_rn(h, Num<T>::up(rr[c])));
      sr[c] = Num<T>::down(h);
    }
    acc = __fmaf_rn(h, h, acc);
  }
  __shared__ float partial[8];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x / 32] = acc;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total = __fadd_rn(total, partial[w]);
  const float r = inv_rms(total, cols_f, eps);
  const bool has_bias = bias != nullptr;
  // second pass: each thread re-reads exactly the elements it visited above
  // (for ADD, the values of s it stored itself)
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float h = ADD ? Num<T>::up(sr[c]) : Num<T>::up(xr[c]);
    float w = Num<T>::up(weight[c]);
    if (ADD) w = Num<T>::rt(__fadd_rn(w, offset));
    float b = has_bias ? Num<T>::up(bias[c]) : 0.f;
    y[row * ldy + c] = Num<T>::down(scale_one<T>(h, r, w, b, has_bias));
  }
}

template <typename T, int TPR, int ITEMS, bool ADD, int RU = 1>
void launch_rows(const void* x, const void* res, const void* w, const void* b, void* y, void* s,
                 int64_t rows, int nvec, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                 float cols_f, float eps, float offset, cudaStream_t st) {
  constexpr int THREADS = TPR < 256 ? 256 : TPR;
  constexpr int ROWS_PER_CTA = THREADS / TPR * RU;
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, ROWS_PER_CTA));
  launch(rms_rows_kernel<T, TPR, ITEMS, ADD, RU>, grid, THREADS, 0, st,
      static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(w), static_cast<const T*>(b),
      static_cast<T*>(y), static_cast<T*>(s), rows, nvec, ldx, ldr, ldy, lds, cols_f, eps, offset);
}

template <typename T, bool ADD>
int run(const void* x, const void* res, const void* w, const void* b, void* y, void* s,
        int64_t rows, int64_t cols, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
        float eps, float offset, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const float cols_f = static_cast<float>(cols);
  bool vec = cols % V == 0 && ldx % V == 0 && ldy % V == 0 && aligned(x, 16) && aligned(y, 16) && aligned(w, 16) &&
             (b == nullptr || aligned(b, 16));
  if (ADD) vec = vec && ldr % V == 0 && lds % V == 0 && aligned(res, 16) && aligned(s, 16);
  const int64_t nvec64 = cols / V;
  if (vec && nvec64 <= 8192) {
    const int nvec = static_cast<int>(nvec64);
#define B200_ROWS(TPR, ITEMS)                                                                                   \
  launch_rows<T, TPR, ITEMS, ADD>(x, res, w, b, y, s, rows, nvec, ldx, ldr, ldy, lds, cols_f, eps, offset, st); \
  return after_launch("rms_rows_kernel")
    // short rows (per-head norms): several rows per warp, four rows per lane group in flight
    if (nvec <= 8) {
      launch_rows<T, 8, 1, ADD, 4>(x, res, w, b, y, s, rows, nvec, ldx, ldr, ldy, lds, cols_f, eps, offset, st);
      return after_launch("rms_rows_kernel");
    }
    if (nvec <= 16) {
      launch_rows<T, 16, 1, ADD, 4>(x, res, w, b, y, s, rows, nvec, ldx, ldr, ldy, lds, cols_f, eps, offset, st);
      return after_launch("rms_rows_kernel");
    }
    if (nvec <= 32) {
      launch_rows<T, 32, 1, ADD, 4>(x, res, w, b, y, s, rows, nvec, ldx, ldr, ldy, lds, cols_f, eps, offset, st);
      return after_launch("rms_rows_kernel");
    }
    if (nvec <= 64) { B200_ROWS(32, 2); }
    if (nvec <= 128) { B200_ROWS(32, 4); }
    if (nvec <= 256) { B200_ROWS(32, 8); }
    if (nvec <= 512) { B200_ROWS(256, 2); }
    if (nvec <= 1024) { B200_ROWS(256, 4); }
    if (nvec <= 2048) { B200_ROWS(256, 8); }
    if (nvec <= 4096) { B200_ROWS(1024, 4); }
    B200_ROWS(1024, 8);
#undef B200_ROWS
  }
  launch(rms_stream_kernel<T, ADD>, static_cast<unsigned>(rows), 256, 0, st,
      static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(w), static_cast<const T*>(b),
      static_cast<T*>(y), static_cast<T*>(s), cols, ldx, ldr, ldy, lds, cols_f, eps, offset);
  return after_launch("rms_stream_kernel");
}

// ---------------------------------------------------------------- backward --
//
// y = round_T(round_T(h * r) * w) (+ b), h = fp32(x), r = rsqrt(mean(h^2) + eps).  What autograd
// derives from the reference (src/popcorn/kernels/_utils.py:14-16, rms_norm.py:29-30,
// add_rms_norm.py:22-23), tensor by tensor, with n = round_T(h * r):
//   grad_b = sum_rows g                         grad_w = sum_rows round_T(g * n)
//   gn = round_T(g * w)                         (fp32 from here on)
//   gr = sum_cols gn * h                        gv = gr * (-0.5 * r^3)
//   grad_h = gn * r + ((gv / cols) * 2) * h     grad_x = round_T(grad_h)
// add_rms_norm: w is round_T(weight + offset), x is the saved residual stream s, and the gradient
// arriving on s is added: grad_x = grad_residual = round_T(round_T(grad_h) + gs).
//
// Persistent CTAs: each walks over rows blockIdx.x, blockIdx.x + gridDim.x, ... with the row in
// registers, keeps fp32 partial column sums for grad_w / grad_b in registers, and writes them to
// its own line of the scratch buffer at the end; rms_bwd_reduce_kernel adds the lines up.
//
// RING: a persistent CTA finishes a row (two passes with a barrier between them) before it can
// ask for the next one, so with plain loads only about one row per CTA is in flight and the
// kernel is latency-bound.  With RING the rows of gy, x (and gs) arrive through a ring of `stages`
// shared-memory slots filled by bulk asynchronous copies that thread 0 issues `stages` rows
// ahead; a slot is refilled one iteration after its row was consumed (after the barrier that
// every thread reaches only when it is done with the previous row).  Waits on the copies are
// bounded: when one runs out, the CTA marks the ring broken, reads the remaining rows with plain
// loads (the data is the same) and thread 0 waits, bounded again, for copies still in flight
// before it leaves.
constexpr int kMaxRingStages = 8;

template <typename T, int ITEMS, bool ADD, bool HAS_BIAS, bool RING>
__global__ void __launch_bounds__(256)
rms_bwd_rows_kernel(const T* __restrict__ gy, const T* __restrict__ gs, const T* __restrict__ x,
                    const T* __restrict__ weight, T* __restrict__ dx, float* __restrict__ part_w,
                    float* __restrict__ part_b, int64_t rows, int nvec, int64_t ldg, int64_t ldgs, int64_t ldx,
                    int64_t lddx, float cols_f, float eps, float offset, int stages) {
  constexpr int V = Num<T>::kVec;
  pdl_prologue();
  const int cols_i = nvec * V;
  const float inv_cols = (cols_i & (cols_i - 1)) == 0 ? 1.0f / cols_f : 0.f;
  __shared__ float red[2][2][8];  // [parity][quantity][warp]
  __shared__ uint64_t full[RING ? kMaxRingStages : 1];
  __shared__ int ring_broken;
  extern __shared__ __align__(128) unsigned char ring[];  // [stages][gy, x, (gs)][row_bytes]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t row_bytes = static_cast<uint32_t>(nvec) * kVecBytes;
  const int nsrc = (ADD && gs != nullptr) ? 3 : 2;
  int64_t issued = 0;  // thread 0: rows of this CTA whose copies have been issued
  // copies of this CTA's `it`-th row into slot it % stages
  auto issue = [&](int64_t it) {
    const int64_t row = blockIdx.x + it * static_cast<int64_t>(gridDim.x);
    const int slot = static_cast<int>(it % stages);
    unsigned char* dst = ring + static_cast<size_t>(slot) * nsrc * row_bytes;
    mbar_arrive_expect(&full[slot], nsrc * row_bytes);
    bulk_load(dst, gy + row * ldg, row_bytes, &full[slot]);
    bulk_load(dst + row_bytes, x + row * ldx, row_bytes, &full[slot]);
    if (nsrc == 3) bulk_load(dst + 2 * row_bytes, gs + row * ldgs, row_bytes, &full[slot]);
  };
  const int64_t my_rows = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if constexpr (RING) {
    if (tid == 0) {
      ring_broken = 0;
      for (int k = 0; k < stages; ++k) mbar_init(&full[k], 1);
      mbar_init_fence();
      for (; issued < stages && issued < my_rows; ++issued) issue(issued);
    }
    __syncthreads();
  }
  float accw[ITEMS][V], accb[HAS_BIAS ? ITEMS : 1][V];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) {
      accw[i][j] = 0.f;
      if constexpr (HAS_BIAS) accb[i][j] = 0.f;
    }
  bool ok[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) ok[i] = tid + i * 256 < nvec;

  // 16-bit types: the effective weight round_T(w + offset) of this thread's columns, packed, for all rows
  // (with a bias gradient the second set of accumulators needs those registers, and the words are re-read per row)
  constexpr bool KEEP_W = sizeof(T) == 2 && !HAS_BIAS;
  uint32_t weff[KEEP_W ? ITEMS : 1][4];
  auto weight_words = [&](int i, uint32_t (&out)[4]) {
    if constexpr (KEEP_W) {
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = weff[i][j];
    } else {
      const uint4 wv = ld_reuse(weight + static_cast<int64_t>(tid + i * 256) * V);
      out[0] = wv.x, out[1] = wv.y, out[2] = wv.z, out[3] = wv.w;
    }
  };
  if constexpr (KEEP_W) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      uint4 wv = make_uint4(0, 0, 0, 0);
      if (ok[i]) wv = ld_reuse(weight + static_cast<int64_t>(tid + i * 256) * V);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        weff[i][j] = ww[j];
        if constexpr (ADD) {
          float w0, w1;
          Num<T>::unpack2(ww[j], w0, w1);
          weff[i][j] = Num<T>::pack2(__fadd_rn(w0, offset), __fadd_rn(w1, offset));
        }
      }
    }
  }

  int parity = 0;
  int64_t it = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1, ++it) {
    uint4 xv[ITEMS], gv[ITEMS];
    const unsigned char* slot = nullptr;  // this row in shared memory, when its copies have landed
    if constexpr (RING) {
      if (*static_cast<volatile int*>(&ring_broken) == 0) {
        if (mbar_wait(&full[it % stages], static_cast<uint32_t>(it / stages) & 1u)) {
          slot = ring + static_cast<size_t>(it % stages) * nsrc * row_bytes;
        } else {
          ring_broken = 1;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      xv[i] = gv[i] = make_uint4(0, 0, 0, 0);
      if (ok[i]) {
        const int64_t col = static_cast<int64_t>(tid + i * 256) * V;
        if (RING && slot != nullptr) {
          gv[i] = *reinterpret_cast<const uint4*>(slot + (tid + i * 256) * kVecBytes);
          xv[i] = *reinterpret_cast<const uint4*>(slot + row_bytes + (tid + i * 256) * kVecBytes);
        } else {
          xv[i] = ld_stream(x + row * ldx + col);
          gv[i] = ld_stream(gy + row * ldg + col);
        }
      }
    }
    float sumsq = 0.f, dot = 0.f;
    if constexpr (sizeof(T) == 2) {
      // 16-bit types: gn = round_T(g * w) is one packed product per pair; two running sums each, two elements per instruction
      Float2x sumsq2 = pack_f2(0.f, 0.f), dot2 = pack_f2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        if (!ok[i]) continue;
        const uint32_t wx[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, wg[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w};
        uint32_t ww[4];
        weight_words(i, ww);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float h0, h1, gn0, gn1;
          Num<T>::unpack2(wx[j], h0, h1);
          Num<T>::unpack2(Num<T>::mul2(wg[j], ww[j]), gn0, gn1);
          if constexpr (HAS_BIAS) {
            float g0, g1;
            Num<T>::unpack2(wg[j], g0, g1);
            accb[i][2 * j] = __fadd_rn(accb[i][2 * j], g0);
            accb[i][2 * j + 1] = __fadd_rn(accb[i][2 * j + 1], g1);
          }
          const Float2x h2 = pack_f2(h0, h1);
          sumsq2 = fma_f2(h2, h2, sumsq2);
          dot2 = fma_f2(pack_f2(gn0, gn1), h2, dot2);
        }
      }
      float a0, a1;
      unpack_f2(sumsq2, a0, a1);
      sumsq = __fadd_rn(a0, a1);
      unpack_f2(dot2, a0, a1);
      dot = __fadd_rn(a0, a1);
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        if (!ok[i]) continue;
        const int64_t col = static_cast<int64_t>(tid + i * 256) * V;
        float h[V], g[V], w[V];
        Num<T>::unpack(xv[i], h);
        Num<T>::unpack(gv[i], g);
        Num<T>::unpack(ld_reuse(weight + col), w);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          if constexpr (ADD) w[j] = __fadd_rn(w[j], offset);
          if constexpr (HAS_BIAS) accb[i][j] = __fadd_rn(accb[i][j], g[j]);
          const float gn = __fmul_rn(g[j], w[j]);
          sumsq = __fmaf_rn(h[j], h[j], sumsq);
          dot = __fmaf_rn(gn, h[j], dot);
        }
      }
    }
    sumsq = warp_sum(sumsq);
    dot = warp_sum(dot);
    if (lane == 0) {
      red[parity][0][warp] = sumsq;
      red[parity][1][warp] = dot;
    }
    __syncthreads();  // the other parity's slots are free again once everyone is past this point
    if constexpr (RING) {
      // every thread is done with the previous row, whose ring slot can take this CTA's next unissued row
      if (tid == 0 && it > 0 && issued < my_rows && *static_cast<volatile int*>(&ring_broken) == 0) issue(issued++);
    }
    // the eight warps' partial sums: one slot per lane, three shuffle steps
    float tot_sq = red[parity][0][lane & 7], tot_dot = red[parity][1][lane & 7];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      tot_sq = __fadd_rn(tot_sq, __shfl_xor_sync(0xffffffffu, tot_sq, o));
      tot_dot = __fadd_rn(tot_dot, __shfl_xor_sync(0xffffffffu, tot_dot, o));
    }
    const float r = inv_rms(tot_sq, cols_f, eps);
    const float gv_scalar = __fmul_rn(tot_dot, __fmul_rn(-0.5f, __fmul_rn(__fmul_rn(r, r), r)));
    // gv / cols: a product with 1 / cols is the same number when cols is a power of two
    const float coef = __fmul_rn(inv_cols > 0.f ? __fmul_rn(gv_scalar, inv_cols) : __fdiv_rn(gv_scalar, cols_f), 2.0f);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      if (!ok[i]) continue;
      const int64_t col = static_cast<int64_t>(tid + i * 256) * V;
      uint4 extra_word = make_uint4(0, 0, 0, 0);
      if (ADD && gs != nullptr) {
        if (RING && slot != nullptr) extra_word = *reinterpret_cast<const uint4*>(slot + 2 * row_bytes + (tid + i * 256) * kVecBytes);
        else extra_word = ld_stream(gs + row * ldgs + col);
      }
      if constexpr (sizeof(T) == 2) {
        // n = round_T(h * r), grad_w += round_T(g * n), grad_h = gn * r + coef * h (one fused multiply-add: the
        // result is rounded to T, and graded against fp64 like the reference's own gradient)
        const uint32_t wx[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, wg[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w};
        const uint32_t we[4] = {extra_word.x, extra_word.y, extra_word.z, extra_word.w};
        const Float2x r2 = pack_f2(r, r), coef2 = pack_f2(coef, coef);
        uint32_t wo[4], ww[4];
        weight_words(i, ww);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float h0, h1, n0, n1, gn0, gn1, gw0, gw1, o0, o1;
          Num<T>::unpack2(wx[j], h0, h1);
          unpack_f2(mul_f2(pack_f2(h0, h1), r2), n0, n1);
          const uint32_t n = Num<T>::pack2(n0, n1);
          Num<T>::unpack2(Num<T>::mul2(wg[j], n), gw0, gw1);
          accw[i][2 * j] = __fadd_rn(accw[i][2 * j], gw0);
          accw[i][2 * j + 1] = __fadd_rn(accw[i][2 * j + 1], gw1);
          Num<T>::unpack2(Num<T>::mul2(wg[j], ww[j]), gn0, gn1);
          const Float2x h2 = pack_f2(h0, h1);
          unpack_f2(fma_f2(pack_f2(gn0, gn1), r2, mul_f2(coef2, h2)), o0, o1);
          wo[j] = Num<T>::pack2(o0, o1);
          if (ADD && gs != nullptr) wo[j] = Num<T>::add2(wo[j], we[j]);
        }
        st_stream(dx + row * lddx + col, make_uint4(wo[0], wo[1], wo[2], wo[3]));
      } else {
        float h[V], g[V], w[V], out[V], extra[V];
        Num<T>::unpack(xv[i], h);
        Num<T>::unpack(gv[i], g);
        Num<T>::unpack(ld_reuse(weight + col), w);
        Num<T>::unpack(extra_word, extra);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          if constexpr (ADD) w[j] = __fadd_rn(w[j], offset);
          const float gn = __fmul_rn(g[j], w[j]);
          accw[i][j] = __fadd_rn(accw[i][j], __fmul_rn(g[j], __fmul_rn(h[j], r)));
          out[j] = __fadd_rn(__fmul_rn(gn, r), __fmul_rn(coef, h[j]));
          if (ADD && gs != nullptr) out[j] = __fadd_rn(out[j], extra[j]);
        }
        st_stream(dx + row * lddx + col, Num<T>::pack(out));
      }
    }
  }
  const int64_t cols = static_cast<int64_t>(nvec) * V;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    if (!ok[i]) continue;
    const int64_t col = static_cast<int64_t>(tid + i * 256) * V;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      part_w[blockIdx.x * cols + col + j] = accw[i][j];
      if constexpr (HAS_BIAS) part_b[blockIdx.x * cols + col + j] = accb[i][j];
    }
  }
  if constexpr (RING) {
    // a broken ring may still have copies in flight into this CTA's shared memory: thread 0 stays
    // (and with it the CTA's shared memory) until each slot's last issued copy has landed or a
    // bounded wait has run out
    __syncthreads();
    if (tid == 0 && ring_broken != 0) {
      for (int64_t k = issued > stages ? issued - stages : 0; k < issued; ++k)
        (void)mbar_wait(&full[k % stages], static_cast<uint32_t>(k / stages) & 1u);
    }
  }
}

// Any width, any alignment: the same arithmetic with scalar accesses; each CTA accumulates its
// partial column sums directly in its own scratch line (zeroed first by the CTA itself).
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
rms_bwd_stream_kernel(const T* __restrict__ gy, const T* __restrict__ gs, const T* __restrict__ x,
                      const T* __restrict__ weight, T* __restrict__ dx, float* __restrict__ part_w,
                      float* __restrict__ part_b, int64_t rows, int64_t cols, int64_t ldg, int64_t ldgs, int64_t ldx,
                      int64_t lddx, float cols_f, float eps, float offset) {
  pdl_prologue();
  __shared__ float red[2][8];
  float* my_w = part_w + blockIdx.x * cols;
  float* my_b = part_b ? part_b + blockIdx.x * cols : nullptr;
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    my_w[c] = 0.f;
    if (my_b) my_b[c] = 0.f;
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float sumsq = 0.f, dot = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float h = Num<T>::up(x[row * ldx + c]);
      float w = Num<T>::up(weight[c]);
      if (ADD) w = Num<T>::rt(__fadd_rn(w, offset));
      const float gn = Num<T>::rt(__fmul_rn(Num<T>::up(gy[row * ldg + c]), w));
      sumsq = __fmaf_rn(h, h, sumsq);
      dot = __fmaf_rn(gn, h, dot);
    }
    sumsq = warp_sum(sumsq);
    dot = warp_sum(dot);
    __syncthreads();  // the previous row's readers are done with `red`
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = sumsq;
      red[1][threadIdx.x >> 5] = dot;
    }
    __syncthreads();
    float tot_sq = 0.f, tot_dot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tot_sq = __fadd_rn(tot_sq, red[0][k]);
      tot_dot = __fadd_rn(tot_dot, red[1][k]);
    }
    const float r = inv_rms(tot_sq, cols_f, eps);
    const float coef = __fmul_rn(__fdiv_rn(__fmul_rn(tot_dot, __fmul_rn(-0.5f, __fmul_rn(__fmul_rn(r, r), r))), cols_f), 2.0f);
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float h = Num<T>::up(x[row * ldx + c]);
      const float g = Num<T>::up(gy[row * ldg + c]);
      float w = Num<T>::up(weight[c]);
      if (ADD) w = Num<T>::rt(__fadd_rn(w, offset));
      const float gn = Num<T>::rt(__fmul_rn(g, w));
      const float n = Num<T>::rt(__fmul_rn(h, r));
      my_w[c] = __fadd_rn(my_w[c], Num<T>::rt(__fmul_rn(g, n)));
      if (my_b) my_b[c] = __fadd_rn(my_b[c], g);
      float out = __fadd_rn(__fmul_rn(gn, r), __fmul_rn(coef, h));
      if (ADD && gs != nullptr) out = __fadd_rn(Num<T>::rt(out), Num<T>::up(gs[row * ldgs + c]));
      dx[row * lddx + c] = Num<T>::down(out);
    }
  }
}

// out[c] = round_T(sum over lines of part[line][c]).  A CTA owns 32 columns; its eight warps each add every eighth
// line (a warp load is one 128-byte segment of a line), then the eight partial sums are added in warp order, so the
// result does not depend on timing.
template <typename T>
__global__ void __launch_bounds__(256)
rms_bwd_reduce_kernel(const float* __restrict__ part, int lines, int64_t cols, T* __restrict__ out) {
  pdl_prologue();
  __shared__ float sums[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + lane;
  float acc = 0.f;
  if (c < cols)
    for (int l = warp; l < lines; l += 8) acc = __fadd_rn(acc, part[static_cast<int64_t>(l) * cols + c]);
  sums[warp][lane] = acc;
  __syncthreads();
  if (warp == 0 && c < cols) {
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) total = __fadd_rn(total, sums[k][lane]);
    out[c] = Num<T>::down(total);
  }
}

// Shared memory a backward CTA may use for its ring: two CTAs share an SM's 227 KB with their static buffers.
constexpr size_t kRingBytesPerCta = 108 * 1024;

// B200_BWD_RING=0 in the environment reads the rows with plain loads instead of the ring.
bool ring_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200_BWD_RING");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Which rows take the row-bucket kernel of norm_family.cu instead of the ring kernel below: rows of up to 512 words
// (measured on a B200, GB/s of the two paths, rms_norm / add_rms_norm backward without a bias gradient:
// bf16 [65536, 2048] 5701 / 5683 vs 2386 / 3485, bf16 [32768, 4096] 5607 / 5501 vs 4272 / 5122, fp32 [200000, 768]
// 5688 / 6643 vs 1829 / 2734); wider rows keep the ring (bf16 [32768, 5120] 4522 vs 4667, [16384, 8192] 5455 vs 5912).
// B200_BWD_FAMILY_WORDS=<n> in the environment replaces the rule by "rows of at most n words".
// With a bias gradient the row-bucket kernel also wins up to 1024 words (bf16 [32768, 5120] 3906 vs 3332,
// [16384, 8192] 4486 vs 4223): the ring kernel re-reads its weight words per row in that case.
bool takes_family_path(int64_t words, bool bias_gradient) {
  static const int forced = [] {
    const char* v = std::getenv("B200_BWD_FAMILY_WORDS");
    return v ? std::atoi(v) : -1;
  }();
  if (forced >= 0) return words <= forced;
  return words <= (bias_gradient ? 1024 : 512);
}

int bwd_lines(int64_t rows) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * 2;
  return static_cast<int>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

template <typename T, bool ADD>
int run_bwd(const void* gy, const void* gs, const void* x, const void* w, void* dx, void* dw, void* db,
            int64_t rows, int64_t cols, int64_t ldg, int64_t ldgs, int64_t ldx, int64_t lddx,
            float eps, float offset, void* scratch, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const int lines = bwd_lines(rows);
  float* part_w = static_cast<float*>(scratch);
  float* part_b = db ? part_w + static_cast<int64_t>(lines) * cols : nullptr;
  const float cols_f = static_cast<float>(cols);
  bool vec = cols % V == 0 && ldg % V == 0 && ldx % V == 0 && lddx % V == 0 && aligned(gy, 16) && aligned(x, 16) &&
             aligned(dx, 16) && aligned(w, 16) && cols / V <= 256 * 8;
  if (gs) vec = vec && ldgs % V == 0 && aligned(gs, 16);
  const T *tgy = static_cast<const T*>(gy), *tgs = static_cast<const T*>(gs), *tx = static_cast<const T*>(x), *tw = static_cast<const T*>(w);
  T* tdx = static_cast<T*>(dx);
  if (vec && takes_family_path(cols / V, db != nullptr)) {
    // short rows: a 256-thread CTA per row would leave lanes idle or spend its time at barriers; 8 to 128 threads per row instead
    const int dtype = sizeof(T) == 4 ? B200_F32 : (std::is_same<T, __half>::value ? B200_F16 : B200_BF16);
    return rms_backward_narrow_rows(dtype, gy, gs, x, w, dx, dw, db, static_cast<float*>(scratch), rows, cols, ldg, ldgs, ldx, lddx, eps,
                                    offset, ADD, st);
  }
  if (vec) {
    const int nvec = static_cast<int>(cols / V);
    // ring of bulk-copied rows: as many slots as fit twice into an SM's shared memory (two CTAs per SM), at least two
    const size_t slot_bytes = static_cast<size_t>(gs ? 3 : 2) * nvec * kVecBytes;
    const int stages = static_cast<int>(std::min<size_t>(kMaxRingStages, kRingBytesPerCta / slot_bytes));
    const bool use_ring = stages >= 2 && ring_enabled();
    const size_t ring_bytes = use_ring ? stages * slot_bytes : 0;
#define B200_BWD_KERNEL(ITEMS, BIAS, RING)                                                                               \
  do {                                                                                                                   \
    auto kernel = rms_bwd_rows_kernel<T, ITEMS, ADD, BIAS, RING>;                                                        \
    if (RING) (void)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring_bytes)); \
    launch(kernel, lines, 256, ring_bytes, st, tgy, tgs, tx, tw, tdx, part_w, part_b, rows, nvec, ldg, ldgs, ldx, lddx,    \
           cols_f, eps, offset, stages);                                                                                 \
  } while (0)
#define B200_BWD(ITEMS, BIAS)                     \
  do {                                            \
    if (use_ring) B200_BWD_KERNEL(ITEMS, BIAS, true); \
    else B200_BWD_KERNEL(ITEMS, BIAS, false);     \
  } while (0)
#define B200_BWD_ITEMS(BIAS)                 \
  do {                                       \
    if (nvec <= 256) B200_BWD(1, BIAS);      \
    else if (nvec <= 512) B200_BWD(2, BIAS); \
    else if (nvec <= 768) B200_BWD(3, BIAS); \
    else if (nvec <= 1024) B200_BWD(4, BIAS);\
    else B200_BWD(8, BIAS);                  \
  } while (0)
    if (db) B200_BWD_ITEMS(true);
    else B200_BWD_ITEMS(false);
#undef B200_BWD_ITEMS
#undef B200_BWD
#undef B200_BWD_KERNEL
    if (int rc = after_launch("rms_bwd_rows_kernel")) return rc;
  } else {
    launch(rms_bwd_stream_kernel<T, ADD>, lines, 256, 0, st, tgy, tgs, tx, tw, tdx, part_w, part_b, rows, cols, ldg, ldgs,
           ldx, lddx, cols_f, eps, offset);
    if (int rc = after_launch("rms_bwd_stream_kernel")) return rc;
  }
  const unsigned grid = static_cast<unsigned>(ceil_div(cols, 32));
  launch(rms_bwd_reduce_kernel<T>, grid, 256, 0, st, static_cast<const float*>(part_w), lines, cols, static_cast<T*>(dw));
  if (int rc = after_launch("rms_bwd_reduce_kernel")) return rc;
  if (db) {
    launch(rms_bwd_reduce_kernel<T>, grid, 256, 0, st, static_cast<const float*>(part_b), lines, cols, static_cast<T*>(db));
    if (int rc = after_launch("rms_bwd_reduce_kernel")) return rc;
  }
  return B200_OK;
}

int check_common(const char* fn, int64_t rows, int64_t cols, int dtype) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size (rows=%lld, cols=%lld)", fn, (long long)rows, (long long)cols);
  if (rows > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: rows=%lld exceeds 2^31-1", fn, (long long)rows);
  return B200_OK;
}

}  // namespace

unsigned int norm_wait_timeouts() { return read_wait_timeouts(); }

}  // namespace b200

using namespace b200;

extern "C" int b200_rms_norm(const void* x, const void* weight, const void* bias, void* y,
                             int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                             int dtype, double eps, void* stream) {
  if (int rc = check_common(__func__, rows, cols, dtype)) return rc;
  if (rows == 0 || cols == 0) return B200_OK;
  B200_REQUIRE_PTR(x);
  B200_REQUIRE_PTR(weight);
  B200_REQUIRE_PTR(y);
  if (ldx < cols || ldy < cols) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", __func__);
  const size_t es = dtype_size(dtype);
  if (!aligned(x, es) || !aligned(y, es) || !aligned(weight, es) || (bias && !aligned(bias, es)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return (run<T, false>(x, nullptr, weight, bias, y, nullptr, rows, cols, ldx, 0, ldy, 0,
                                                       static_cast<float>(eps), 0.f, st)));
  return B200_OK;
}

extern "C" int b200_add_rms_norm(const void* x, const void* residual, const void* weight, void* y, void* s,
                                 int64_t rows, int64_t cols, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                                 int dtype, double eps, double offset, void* stream) {
  if (int rc = check_common(__func__, rows, cols, dtype)) return rc;
  if (rows == 0 || cols == 0) return B200_OK;
  B200_REQUIRE_PTR(x);
  B200_REQUIRE_PTR(residual);
  B200_REQUIRE_PTR(weight);
  B200_REQUIRE_PTR(y);
  B200_REQUIRE_PTR(s);
  if (ldx < cols || ldr < cols || ldy < cols || lds < cols)
    return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", __func__);
  if (y == s) return fail(B200_ERR_SHAPE, "%s: y and s must be distinct buffers", __func__);
  const size_t es = dtype_size(dtype);
  if (!aligned(x, es) || !aligned(residual, es) || !aligned(y, es) || !aligned(s, es) || !aligned(weight, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return (run<T, true>(x, residual, weight, nullptr, y, s, rows, cols, ldx, ldr, ldy, lds,
                                                      static_cast<float>(eps), static_cast<float>(offset), st)));
  return B200_OK;
}

extern "C" int b200_rms_norm_backward_scratch_bytes(int64_t rows, int64_t cols, int with_bias, size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (int rc = check_device()) return rc;
  const size_t lines = static_cast<size_t>(bwd_lines(rows));
  *bytes = lines * static_cast<size_t>(cols > 0 ? cols : 1) * sizeof(float) * (with_bias ? 2 : 1);
  return B200_OK;
}

static int norm_backward(const char* fn, bool add, const void* gy, const void* gs, const void* x, const void* weight, void* dx,
                         void* dw, void* db, int64_t rows, int64_t cols, int64_t ldg, int64_t ldgs, int64_t ldx, int64_t lddx,
                         int dtype, double eps, double offset, void* scratch, size_t scratch_bytes, void* stream) {
  if (int rc = check_common(fn, rows, cols, dtype)) return rc;
  if (cols == 0) return B200_OK;
  if (gy == nullptr || x == nullptr || weight == nullptr || dx == nullptr || dw == nullptr || scratch == nullptr)
    return fail(B200_ERR_NULL_POINTER, "%s: a required pointer is NULL", fn);
  if (ldg < cols || ldx < cols || lddx < cols || (gs && ldgs < cols)) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", fn);
  const size_t es = dtype_size(dtype);
  if (!aligned(gy, es) || !aligned(x, es) || !aligned(weight, es) || !aligned(dx, es) || !aligned(dw, es) || (gs && !aligned(gs, es)) ||
      (db && !aligned(db, es)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  const size_t need = static_cast<size_t>(bwd_lines(rows)) * static_cast<size_t>(cols) * sizeof(float) * (db ? 2 : 1);
  if (scratch_bytes < need || !aligned(scratch, 16))
    return fail(B200_ERR_SCRATCH, "%s: scratch needs %zu bytes, 16-byte aligned (got %zu)", fn, need, scratch_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float e = static_cast<float>(eps), o = static_cast<float>(offset);
  if (add) {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, true>(gy, gs, x, weight, dx, dw, nullptr, rows, cols, ldg, ldgs, ldx, lddx, e, o, scratch, st)));
  } else {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, false>(gy, nullptr, x, weight, dx, dw, db, rows, cols, ldg, 0, ldx, lddx, e, 0.f, scratch, st)));
  }
  return B200_OK;
}

extern "C" int b200_rms_norm_backward(const void* grad_y, const void* x, const void* weight, void* grad_x, void* grad_weight,
                                      void* grad_bias, int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx,
                                      int dtype, double eps, void* scratch, size_t scratch_bytes, void* stream) {
  return norm_backward(__func__, false, grad_y, nullptr, x, weight, grad_x, grad_weight, grad_bias, rows, cols, ldg, 0, ldx, lddx,
                       dtype, eps, 0.0, scratch, scratch_bytes, stream);
}

extern "C" int b200_add_rms_norm_backward(const void* grad_y, const void* grad_s, const void* s, const void* weight, void* grad_x,
                                          void* grad_weight, int64_t rows, int64_t cols, int64_t ldgy, int64_t ldgs, int64_t lds,
                                          int64_t lddx, int dtype, double eps, double offset, void* scratch, size_t scratch_bytes,
                                          void* stream) {
  return norm_backward(__func__, true, grad_y, grad_s, s, weight, grad_x, grad_weight, nullptr, rows, cols, ldgy, ldgs, lds, lddx,
                       dtype, eps, offset, scratch, scratch_bytes, stream);
}
