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
#include "common.cuh"

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
template <typename T, int TPR, int ITEMS, bool ADD>
__global__ void __launch_bounds__(TPR < 256 ? 256 : TPR)
rms_rows_kernel(const T* x, const T* res, const T* __restrict__ weight,
                const T* __restrict__ bias, T* y, T* s_out,
                int64_t rows, int nvec, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                float cols_f, float eps, float offset) {
  constexpr int V = Num<T>::kVec;
  constexpr int THREADS = TPR < 256 ? 256 : TPR;
  constexpr int ROWS_PER_CTA = THREADS / TPR;
  constexpr int WARPS_PER_ROW = TPR / 32;
  pdl_prologue();

  const int tid = threadIdx.x;
  const int sub = tid / TPR;        // which row of this CTA
  const int lane_in_row = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * ROWS_PER_CTA + sub;
  const bool row_ok = row < rows;

  uint4 data[ITEMS];
  bool ok[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) ok[i] = row_ok && (lane_in_row + i * TPR) < nvec;

  // issue every load of the row before touching any of them
  uint4 rdata[ADD ? ITEMS : 1];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int v = lane_in_row + i * TPR;
    data[i] = make_uint4(0, 0, 0, 0);
    if (ok[i]) data[i] = ld_stream(x + row * ldx + static_cast<int64_t>(v) * V);
    if constexpr (ADD) {
      rdata[i] = make_uint4(0, 0, 0, 0);
      if (ok[i]) rdata[i] = ld_stream(res + row * ldr + static_cast<int64_t>(v) * V);
    }
  }

  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    float f[V];
    Num<T>::unpack(data[i], f);
    if constexpr (ADD) {
      float g[V];
      Num<T>::unpack(rdata[i], g);
#pragma unroll
      for (int j = 0; j < V; ++j) f[j] = __fadd_rn(f[j], g[j]);
      data[i] = Num<T>::pack(f);  // s = x + residual, rounded to T by the pack
      Num<T>::unpack(data[i], f);
      if (ok[i]) st_stream(s_out + row * lds + static_cast<int64_t>(lane_in_row + i * TPR) * V, data[i]);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) acc = __fmaf_rn(f[j], f[j], acc);
  }

  acc = warp_sum(acc);
  if (WARPS_PER_ROW > 1) {
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
  const bool has_bias = bias != nullptr;

#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    if (!ok[i]) continue;
    const int64_t col = static_cast<int64_t>(lane_in_row + i * TPR) * V;
    if constexpr (sizeof(T) == 4) {
      float f[V], w[V], b[V];
      Num<T>::unpack(data[i], f);
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
      const uint32_t wd[4] = {data[i].x, data[i].y, data[i].z, data[i].w};
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

template <typename T, int TPR, int ITEMS, bool ADD>
void launch_rows(const void* x, const void* res, const void* w, const void* b, void* y, void* s,
                 int64_t rows, int nvec, int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                 float cols_f, float eps, float offset, cudaStream_t st) {
  constexpr int THREADS = TPR < 256 ? 256 : TPR;
  constexpr int ROWS_PER_CTA = THREADS / TPR;
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, ROWS_PER_CTA));
  launch(rms_rows_kernel<T, TPR, ITEMS, ADD>, grid, THREADS, 0, st,
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
    if (nvec <= 32) { B200_ROWS(32, 1); }
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

int check_common(const char* fn, int64_t rows, int64_t cols, int dtype) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size (rows=%lld, cols=%lld)", fn, (long long)rows, (long long)cols);
  if (rows > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: rows=%lld exceeds 2^31-1", fn, (long long)rows);
  return B200_OK;
}

}  // namespace
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
