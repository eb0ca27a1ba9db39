// Row-normalisation siblings of RMSNorm for sm_100a: gated RMSNorm, L2 norm, LayerNorm.
//
// Same shape as the RMSNorm kernel: one row per warp (rows up to 256 128-bit words) or per
// 256-thread CTA (up to 2048 words), the row held in registers, one HBM read and one write per
// element; anything wider or unaligned goes through the scalar two/three-pass kernel.
//
// Arithmetic follows the references tensor by tensor, including their roundings to T:
//   rms_norm_gated  src/popcorn/kernels/rms_norm_gated.py:27-29
//       y = round_T( round_T(round_T(round_T(h*r) * w) [+ b]) * round_T(act(g)) ),  act = silu | sigmoid
//   l2_norm         src/popcorn/kernels/l2_norm.py:14   (everything in T)
//       y = round_T( x * round_T(rsqrt(round_T(round_T(sum round_T(x^2)) + eps))) )
//   layer_norm      src/popcorn/kernels/layer_norm.py:20 (F.layer_norm: fp32 statistics, one rounding)
//       y = round_T( (x*rstd - mean*rstd) * w + b ),  rstd = 1/sqrt(var + eps), biased variance
#include "activations.cuh"
#include "common.cuh"

namespace b200 {
namespace {

enum Mode { kGatedSwish = 0, kGatedSigmoid = 1, kL2 = 2, kLayer = 3, kRms = 4, kRmsAdd = 5 };  // kRms / kRmsAdd: backward only (rms_norm, add_rms_norm on short rows)

// Gate of the gated RMSNorm in fp32: the reference's operation sequence for fp32 tensors, the
// corrected-ex2 / Newton forms (activations.cuh) for 16-bit ones, whose result is rounded to T anyway.
template <typename T, int MODE>
__device__ __forceinline__ float gate_act(float g) {
  constexpr int MATH = sizeof(T) == 4 ? 0 : 1;
  if constexpr (MODE == 0) return silu_f32<MATH>(g);
  else return sigmoid_f32<MATH>(g);
}

// Sum over the TPR threads of a row.  TPR <= 32: shuffles only (TPR consecutive lanes).  TPR == 256: one row per CTA, the
// caller passes a distinct smem slot per reduction so that one barrier per reduction is enough.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* slot) {
#pragma unroll
  for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (TPR > 32) {
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < TPR / 32; ++k) total = __fadd_rn(total, slot[k]);
    v = total;
  }
  return v;
}

template <typename T, int TPR, int ITEMS, int MODE, int RU>
__global__ void __launch_bounds__(256)
family_rows_kernel(const T* x, const T* gate, const T* __restrict__ weight, const T* __restrict__ bias, T* y,
                   int64_t rows, int nvec, int64_t ldx, int64_t ldg, int64_t ldy, float cols_f, float eps) {
  constexpr int V = Num<T>::kVec;
  constexpr int GROUPS = 256 / TPR;  // row groups per CTA; each owns RU consecutive rows
  static_assert(RU == 1 || TPR <= 32, "several rows per group only for rows that fit a warp");
  constexpr bool GATED = MODE == kGatedSwish || MODE == kGatedSigmoid;
  pdl_prologue();
  __shared__ float slots[2][8];
  const int tid = threadIdx.x;
  const int sub = tid / TPR, lane_in_row = tid % TPR;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * GROUPS + sub) * RU;

  uint4 all_data[RU][ITEMS], all_gdata[GATED ? RU : 1][GATED ? ITEMS : 1];
  bool all_ok[RU][ITEMS];
#pragma unroll
  for (int u = 0; u < RU; ++u) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int64_t row = row0 + u;
      all_ok[u][i] = row < rows && (lane_in_row + i * TPR) < nvec;
      all_data[u][i] = make_uint4(0, 0, 0, 0);
      const int64_t col = static_cast<int64_t>(lane_in_row + i * TPR) * V;
      if (all_ok[u][i]) all_data[u][i] = ld_stream(x + row * ldx + col);
      if constexpr (GATED) {
        all_gdata[u][i] = make_uint4(0, 0, 0, 0);
        if (all_ok[u][i]) all_gdata[u][i] = ld_stream(gate + row * ldg + col);
      }
    }
  }
  const bool has_bias = bias != nullptr;

#pragma unroll
  for (int u = 0; u < RU; ++u) {
  const int64_t row = row0 + u;
  uint4(&data)[ITEMS] = all_data[u];
  uint4(&gdata)[GATED ? ITEMS : 1] = all_gdata[GATED ? u : 0];
  bool(&ok)[ITEMS] = all_ok[u];

  // first moment (LayerNorm) or sum of squares
  constexpr bool HALF = sizeof(T) == 2;
  float acc = 0.f;
  if constexpr (MODE == kLayer) {
    Float2x acc2 = pack_f2(0.f, 0.f);  // two running sums, two elements per instruction
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      float f[V];
      Num<T>::unpack(data[i], f);
#pragma unroll
      for (int j = 0; j < V; j += 2) acc2 = add_f2(acc2, pack_f2(f[j], f[j + 1]));
    }
    float a0, a1;
    unpack_f2(acc2, a0, a1);
    acc = __fadd_rn(a0, a1);
  } else {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      if constexpr (MODE == kL2 && HALF) {
        // x.pow(2) is a tensor of dtype T: packed product, one rounding per element
        const uint32_t wx[4] = {data[i].x, data[i].y, data[i].z, data[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float s0, s1;
          Num<T>::unpack2(Num<T>::mul2(wx[j], wx[j]), s0, s1);
          acc = __fadd_rn(acc, __fadd_rn(s0, s1));
        }
      } else {
        float f[V];
        Num<T>::unpack(data[i], f);
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          if constexpr (MODE == kL2) {
            acc = __fadd_rn(acc, __fadd_rn(__fmul_rn(f[j], f[j]), __fmul_rn(f[j + 1], f[j + 1])));
          } else {
            acc = __fmaf_rn(f[j], f[j], acc);
            acc = __fmaf_rn(f[j + 1], f[j + 1], acc);
          }
        }
      }
    }
  }
  acc = row_sum<TPR>(acc, slots[0]);

  float scale, shift = 0.f;  // y_pre = x * scale + shift
  if constexpr (MODE == kLayer) {
    const float mean = __fdiv_rn(acc, cols_f);
    const Float2x neg_mean = pack_f2(-mean, -mean);
    Float2x var2 = pack_f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      if (!ok[i]) continue;
      float f[V];
      Num<T>::unpack(data[i], f);
#pragma unroll
      for (int j = 0; j < V; j += 2) {
        const Float2x d = add_f2(pack_f2(f[j], f[j + 1]), neg_mean);
        var2 = fma_f2(d, d, var2);
      }
    }
    float v0, v1;
    unpack_f2(var2, v0, v1);
    const float var = __fdiv_rn(row_sum<TPR>(__fadd_rn(v0, v1), slots[1]), cols_f);
    scale = __frcp_rn(__fsqrt_rn(__fadd_rn(fmaxf(var, 0.f), eps)));
    shift = -__fmul_rn(scale, mean);
  } else if constexpr (MODE == kL2) {
    const float total = Num<T>::rt(acc);                   // .sum(-1) returns dtype T
    const float v = Num<T>::rt(__fadd_rn(total, eps));     // + eps, dtype T
    // torch.rsqrt of a T tensor: 1/sqrt in fp32, one rounding.  (PyTorch's vectorised CPU loop rounds sqrt(v)
    // to T before the reciprocal for 16-bit dtypes, its scalar tail does not; this is the tail's arithmetic.)
    scale = Num<T>::rt(__frcp_rn(__fsqrt_rn(v)));
  } else {
    scale = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(acc, cols_f), eps)));
  }

#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    if (!ok[i]) continue;
    const int64_t col = static_cast<int64_t>(lane_in_row + i * TPR) * V;
    if constexpr (MODE == kLayer) {
      // (x * scale + shift) * w + b in fp32 with two fused multiply-adds, two elements per instruction; the
      // result is rounded to T once (F.layer_norm keeps fp32 until its output)
      float f[V], w[V], b[V];
      Num<T>::unpack(data[i], f);
      Num<T>::unpack(ld_reuse(weight + col), w);
      if (has_bias) Num<T>::unpack(ld_reuse(bias + col), b);
      const Float2x scale2 = pack_f2(scale, scale), shift2 = pack_f2(shift, shift);
#pragma unroll
      for (int j = 0; j < V; j += 2) {
        const Float2x t = fma_f2(pack_f2(f[j], f[j + 1]), scale2, shift2);
        const Float2x o = has_bias ? fma_f2(t, pack_f2(w[j], w[j + 1]), pack_f2(b[j], b[j + 1])) : mul_f2(t, pack_f2(w[j], w[j + 1]));
        unpack_f2(o, f[j], f[j + 1]);
      }
      st_stream(y + row * ldy + col, Num<T>::pack(f));
    } else if constexpr (HALF) {
      // 16-bit types: every product and sum of two T tensors is one packed instruction with the reference's rounding
      const uint32_t wx[4] = {data[i].x, data[i].y, data[i].z, data[i].w};
      uint32_t wo[4];
      if constexpr (MODE == kL2) {
        const uint32_t scale2 = Num<T>::pack2(scale, scale);
#pragma unroll
        for (int j = 0; j < 4; ++j) wo[j] = Num<T>::mul2(wx[j], scale2);
      } else {
        const uint4 wv = ld_reuse(weight + col);
        uint4 bv = make_uint4(0, 0, 0, 0);
        if (has_bias) bv = ld_reuse(bias + col);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, wb[4] = {bv.x, bv.y, bv.z, bv.w};
        const uint32_t wg[4] = {gdata[i].x, gdata[i].y, gdata[i].z, gdata[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float h0, h1, g0, g1;
          Num<T>::unpack2(wx[j], h0, h1);
          Num<T>::unpack2(wg[j], g0, g1);
          uint32_t t = Num<T>::mul2(Num<T>::pack2(__fmul_rn(h0, scale), __fmul_rn(h1, scale)), ww[j]);
          if (has_bias) t = Num<T>::add2(t, wb[j]);
          const uint32_t a = Num<T>::pack2(gate_act<T, MODE == kGatedSwish ? 0 : 1>(g0), gate_act<T, MODE == kGatedSwish ? 0 : 1>(g1));
          wo[j] = Num<T>::mul2(t, a);
        }
      }
      st_stream(y + row * ldy + col, make_uint4(wo[0], wo[1], wo[2], wo[3]));
    } else {
      float f[V], w[V], b[V], g[V];
      Num<T>::unpack(data[i], f);
      if constexpr (MODE != kL2) Num<T>::unpack(ld_reuse(weight + col), w);
      if (MODE != kL2 && has_bias) Num<T>::unpack(ld_reuse(bias + col), b);
      if constexpr (GATED) Num<T>::unpack(gdata[i], g);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float o = __fmul_rn(f[j], scale);
        if constexpr (MODE != kL2) {
          o = __fmul_rn(o, w[j]);
          if (has_bias) o = __fadd_rn(o, b[j]);
          o = __fmul_rn(o, gate_act<T, MODE == kGatedSwish ? 0 : 1>(g[j]));
        }
        f[j] = o;
      }
      st_stream(y + row * ldy + col, Num<T>::pack(f));
    }
  }
  }  // rows of this group
}

// Any width, any alignment: one CTA per row, scalar accesses, the row re-read for every pass.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
family_stream_kernel(const T* x, const T* gate, const T* __restrict__ weight, const T* __restrict__ bias, T* y,
                     int64_t cols, int64_t ldx, int64_t ldg, int64_t ldy, float cols_f, float eps) {
  constexpr bool GATED = MODE == kGatedSwish || MODE == kGatedSigmoid;
  pdl_prologue();
  __shared__ float slots[2][8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  float acc = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    const float h = Num<T>::up(xr[c]);
    if (MODE == kLayer) acc = __fadd_rn(acc, h);
    else if (MODE == kL2) acc = __fadd_rn(acc, Num<T>::rt(__fmul_rn(h, h)));
    else acc = __fmaf_rn(h, h, acc);
  }
  acc = row_sum<256>(acc, slots[0]);
  float scale, shift = 0.f;
  if (MODE == kLayer) {
    const float mean = __fdiv_rn(acc, cols_f);
    float var = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float d = __fsub_rn(Num<T>::up(xr[c]), mean);
      var = __fmaf_rn(d, d, var);
    }
    var = __fdiv_rn(row_sum<256>(var, slots[1]), cols_f);
    scale = __frcp_rn(__fsqrt_rn(__fadd_rn(fmaxf(var, 0.f), eps)));
    shift = -__fmul_rn(scale, mean);
  } else if (MODE == kL2) {
    scale = Num<T>::rt(__frcp_rn(__fsqrt_rn(Num<T>::rt(__fadd_rn(Num<T>::rt(acc), eps)))));
  } else {
    scale = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(acc, cols_f), eps)));
  }
  const bool has_bias = bias != nullptr;
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    const float h = Num<T>::up(xr[c]);
    float o;
    if (MODE == kLayer) {
      o = __fmul_rn(__fadd_rn(__fmul_rn(h, scale), shift), Num<T>::up(weight[c]));
      if (has_bias) o = __fadd_rn(o, Num<T>::up(bias[c]));
    } else if (MODE == kL2) {
      o = __fmul_rn(h, scale);
    } else {
      o = Num<T>::rt(__fmul_rn(Num<T>::rt(__fmul_rn(h, scale)), Num<T>::up(weight[c])));
      if (has_bias) o = Num<T>::rt(__fadd_rn(o, Num<T>::up(bias[c])));
      const float g = GATED ? Num<T>::up(gate[row * ldg + c]) : 0.f;
      o = __fmul_rn(o, Num<T>::rt(MODE == kGatedSwish ? silu_f32<0>(g) : sigmoid_f32<0>(g)));
    }
    y[row * ldy + c] = Num<T>::down(o);
  }
}

template <typename T, int MODE>
int run(const void* x, const void* gate, const void* w, const void* b, void* y, int64_t rows, int64_t cols,
        int64_t ldx, int64_t ldg, int64_t ldy, float eps, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  constexpr bool GATED = MODE == kGatedSwish || MODE == kGatedSigmoid;
  const float cols_f = static_cast<float>(cols);
  bool vec = cols % V == 0 && ldx % V == 0 && ldy % V == 0 && aligned(x, 16) && aligned(y, 16) &&
             (w == nullptr || aligned(w, 16)) && (b == nullptr || aligned(b, 16));
  if (GATED) vec = vec && ldg % V == 0 && aligned(gate, 16);
  const T *tx = static_cast<const T*>(x), *tg = static_cast<const T*>(gate), *tw = static_cast<const T*>(w), *tb = static_cast<const T*>(b);
  T* ty = static_cast<T*>(y);
  const int64_t nvec64 = cols / V;
  if (vec && nvec64 <= 2048) {
    const int nvec = static_cast<int>(nvec64);
#define B200_FAMILY_RU(TPR, ITEMS, RU)                                                                                        \
  launch(family_rows_kernel<T, TPR, ITEMS, MODE, RU>, static_cast<unsigned>(ceil_div(rows, 256 / TPR * RU)), 256, 0, st, tx, tg, \
         tw, tb, ty, rows, nvec, ldx, ldg, ldy, cols_f, eps)
#define B200_FAMILY(TPR, ITEMS) B200_FAMILY_RU(TPR, ITEMS, 1)
    // short rows (per-head norms): several rows per warp, four rows per lane group in flight
    if (nvec <= 8) B200_FAMILY_RU(8, 1, 4);
    else if (nvec <= 16) B200_FAMILY_RU(16, 1, 4);
    else if (nvec <= 32) B200_FAMILY_RU(32, 1, 4);
    else if (nvec <= 64) B200_FAMILY(32, 2);
    else if (nvec <= 128) B200_FAMILY(32, 4);
    else if (nvec <= 256) B200_FAMILY(32, 8);
    else if (nvec <= 512) B200_FAMILY(256, 2);
    else if (nvec <= 1024) B200_FAMILY(256, 4);
    else B200_FAMILY(256, 8);
#undef B200_FAMILY
#undef B200_FAMILY_RU
    return after_launch("family_rows_kernel");
  }
  launch(family_stream_kernel<T, MODE>, static_cast<unsigned>(rows), 256, 0, st, tx, tg, tw, tb, ty, cols, ldx, ldg, ldy, cols_f, eps);
  return after_launch("family_stream_kernel");
}

int entry(const char* fn, int mode, const void* x, const void* gate, const void* weight, const void* bias, void* y,
          int64_t rows, int64_t cols, int64_t ldx, int64_t ldg, int64_t ldy, int dtype, double eps, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (rows > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: rows=%lld exceeds 2^31-1", fn, (long long)rows);
  if (rows == 0 || cols == 0) return B200_OK;
  const bool gated = mode == kGatedSwish || mode == kGatedSigmoid;
  if (x == nullptr || y == nullptr || (mode != kL2 && weight == nullptr) || (gated && gate == nullptr))
    return fail(B200_ERR_NULL_POINTER, "%s: a required pointer is NULL", fn);
  if (ldx < cols || ldy < cols || (gated && ldg < cols)) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", fn);
  const size_t es = dtype_size(dtype);
  if (!aligned(x, es) || !aligned(y, es) || !aligned(gate, es) || !aligned(weight, es) || !aligned(bias, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float e = static_cast<float>(eps);
  switch (mode) {
    case kGatedSwish: B200_DISPATCH_DTYPE(dtype, T, return (run<T, kGatedSwish>(x, gate, weight, bias, y, rows, cols, ldx, ldg, ldy, e, st))); break;
    case kGatedSigmoid: B200_DISPATCH_DTYPE(dtype, T, return (run<T, kGatedSigmoid>(x, gate, weight, bias, y, rows, cols, ldx, ldg, ldy, e, st))); break;
    case kL2: B200_DISPATCH_DTYPE(dtype, T, return (run<T, kL2>(x, nullptr, nullptr, nullptr, y, rows, cols, ldx, 0, ldy, e, st))); break;
    default: B200_DISPATCH_DTYPE(dtype, T, return (run<T, kLayer>(x, nullptr, weight, bias, y, rows, cols, ldx, 0, ldy, e, st))); break;
  }
  return B200_OK;
}


// ---------------------------------------------------------------- backward --
//
// l2_norm:    y = x s, s = rsqrt(sum x^2 + eps)          dx = g s - x s^3 <g, x>
// layer_norm: y = xhat w + b, xhat = (x - mean) rstd     dx = rstd (gw - mean(gw) - xhat mean(gw xhat)), gw = g w
//                                                        dw = sum_rows g xhat,  db = sum_rows g
// in fp32 from the stored 16-bit (or fp32) values, one rounding per output; gradients are graded against an fp64
// evaluation like the reference's own (src/popcorn/bench/compare.py:243-277).
//
// Two kernels.  family_bwd_rows_kernel (further down) is the fast path for aligned rows of up to 1024 words.  The
// kernel right below is the general one for everything else (wider rows, widths or pointers that are not a multiple
// of the 128-bit word): persistent CTAs walk the rows, a row is read once from HBM and re-read from L1/L2 for the
// later passes, and each thread adds its columns' contributions to dw / db in the CTA's own line of `partial`
// ([lines][2][cols] fp32, in global memory), which family_sum_lines_kernel adds up.
// VEC: 128-bit accesses (cols, strides and pointers aligned), else element by element.
template <typename T, bool VEC>
__device__ __forceinline__ void load_elems(const T* p, float (&f)[Num<T>::kVec]) {
  if constexpr (VEC) Num<T>::unpack(ld_plain(p), f);
  else f[0] = Num<T>::up(*p);
}
template <typename T, bool VEC>
__device__ __forceinline__ void store_elems(T* p, const float (&f)[Num<T>::kVec]) {
  if constexpr (VEC) st_stream(p, Num<T>::pack(f));
  else *p = Num<T>::down(f[0]);
}

template <typename T, int MODE, bool VEC>
__global__ void __launch_bounds__(256)
family_bwd_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ dx,
                  float* __restrict__ partial, int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx,
                  float cols_f, float eps, int has_bias) {
  constexpr int V = Num<T>::kVec;
  constexpr int E = VEC ? V : 1;  // elements per thread per step
  pdl_prologue();
  __shared__ float slots[4][8];
  float* my_w = nullptr;
  float* my_b = nullptr;
  if constexpr (MODE == kLayer) {
    my_w = partial + static_cast<int64_t>(blockIdx.x) * 2 * cols;
    my_b = my_w + cols;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      my_w[c] = 0.f;
      my_b[c] = 0.f;
    }
  }
  const int64_t step = 256 * E;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ldx;
    const T* gr = gy + row * ldg;
    T* dr = dx + row * lddx;
    __syncthreads();  // the previous row is done with `slots`
    if constexpr (MODE == kL2) {
      float ss = 0.f, dot = 0.f;
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V], fg[V];
        load_elems<T, VEC>(xr + c, fx);
        load_elems<T, VEC>(gr + c, fg);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          ss = __fmaf_rn(fx[j], fx[j], ss);
          dot = __fmaf_rn(fg[j], fx[j], dot);
        }
      }
      ss = row_sum<256>(ss, slots[0]);
      dot = row_sum<256>(dot, slots[1]);
      const float s = __frcp_rn(__fsqrt_rn(__fadd_rn(ss, eps)));
      const float coef = -__fmul_rn(__fmul_rn(__fmul_rn(s, s), s), dot);
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V], fg[V];
        load_elems<T, VEC>(xr + c, fx);
        load_elems<T, VEC>(gr + c, fg);
#pragma unroll
        for (int j = 0; j < E; ++j) fg[j] = __fmaf_rn(fg[j], s, __fmul_rn(fx[j], coef));
        store_elems<T, VEC>(dr + c, fg);
      }
    } else {
      float sum = 0.f;
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V];
        load_elems<T, VEC>(xr + c, fx);
#pragma unroll
        for (int j = 0; j < E; ++j) sum = __fadd_rn(sum, fx[j]);
      }
      const float mean = __fdiv_rn(row_sum<256>(sum, slots[0]), cols_f);
      float var = 0.f;
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V];
        load_elems<T, VEC>(xr + c, fx);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float d = __fsub_rn(fx[j], mean);
          var = __fmaf_rn(d, d, var);
        }
      }
      var = __fdiv_rn(row_sum<256>(var, slots[1]), cols_f);
      const float rstd = __frcp_rn(__fsqrt_rn(__fadd_rn(fmaxf(var, 0.f), eps)));
      float s1 = 0.f, s2 = 0.f;
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V], fg[V], fw[V];
        load_elems<T, VEC>(xr + c, fx);
        load_elems<T, VEC>(gr + c, fg);
        load_elems<T, VEC>(weight + c, fw);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float gw = __fmul_rn(fg[j], fw[j]);
          s1 = __fadd_rn(s1, gw);
          s2 = __fmaf_rn(gw, __fmul_rn(__fsub_rn(fx[j], mean), rstd), s2);
        }
      }
      s1 = __fdiv_rn(row_sum<256>(s1, slots[2]), cols_f);
      s2 = __fdiv_rn(row_sum<256>(s2, slots[3]), cols_f);
      for (int64_t c = static_cast<int64_t>(threadIdx.x) * E; c < cols; c += step) {
        float fx[V], fg[V], fw[V];
        load_elems<T, VEC>(xr + c, fx);
        load_elems<T, VEC>(gr + c, fg);
        load_elems<T, VEC>(weight + c, fw);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float xhat = __fmul_rn(__fsub_rn(fx[j], mean), rstd);
          my_w[c + j] = __fmaf_rn(fg[j], xhat, my_w[c + j]);  // this thread owns these columns of the CTA's line
          if (has_bias) my_b[c + j] = __fadd_rn(my_b[c + j], fg[j]);
          fx[j] = __fmul_rn(rstd, __fsub_rn(__fsub_rn(__fmul_rn(fg[j], fw[j]), s1), __fmul_rn(xhat, s2)));
        }
        store_elems<T, VEC>(dr + c, fx);
      }
    }
  }
}

// N sums over the TPR threads of a row: shuffles only (TPR <= 32), or one barrier per call: the CTA-wide one when the
// row owns the CTA (TPR == 256), a named barrier of the row's TPR threads when several rows share it (TPR 64 or 128;
// `group` is the row's index in the CTA).  `slot` is this row's [N][8] piece of shared memory.
template <int TPR, int N>
__device__ __forceinline__ void row_sums(float (&v)[N], float (*slot)[8], int group) {
#pragma unroll
  for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1) {
#pragma unroll
    for (int n = 0; n < N; ++n) v[n] = __fadd_rn(v[n], __shfl_xor_sync(0xffffffffu, v[n], o));
  }
  if constexpr (TPR > 32) {
    constexpr int WARPS = TPR / 32;
    const int warp_in_row = (threadIdx.x >> 5) % WARPS;
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
      for (int n = 0; n < N; ++n) slot[n][warp_in_row] = v[n];
    }
    if constexpr (TPR == 256) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(TPR) : "memory");
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float total = 0.f;
#pragma unroll
      for (int k = 0; k < WARPS; ++k) total = __fadd_rn(total, slot[n][k]);
      v[n] = total;
    }
  }
}

// A 128-bit word of T as V / 2 pairs of fp32 (the operands of the two-element fp32 instructions).
template <typename T>
__device__ __forceinline__ void unpack_pairs(const uint4& word, Float2x (&out)[Num<T>::kVec / 2]) {
  float f[Num<T>::kVec];
  Num<T>::unpack(word, f);
#pragma unroll
  for (int j = 0; j < Num<T>::kVec / 2; ++j) out[j] = pack_f2(f[2 * j], f[2 * j + 1]);
}
__device__ __forceinline__ float pair_total(Float2x v) {
  float lo, hi;
  unpack_f2(v, lo, hi);
  return __fadd_rn(lo, hi);
}

// The fast path of the backward: rows of up to 1024 128-bit words, held in registers.  TPR threads share a row
// (TPR <= 32: several rows per warp, RU of them in flight per group; 256: one row per CTA), each thread keeps its
// ITEMS words of x and of the incoming gradient, so both are read from HBM once and nothing is re-read.  Persistent
// CTAs walk the rows; for LayerNorm every thread adds its columns' contributions to dw (and db) in registers, the
// CTA folds its row groups in a fixed order through shared memory and writes ONE line of partial sums, which
// family_sum_lines_kernel adds up, so the result does not depend on timing.  The arithmetic is fp32 with two
// elements per instruction; gradients are compared within a tolerance, so products and sums may be fused:
//   LayerNorm, per row:  mean = sum x / n;  var = sum (x - mean)^2 / n;  rstd = 1 / sqrt(var + eps)
//                        m1 = sum gw / n;  m2 = rstd (sum gw x - mean sum gw) / n            (gw = g w)
//                        xhat = x rstd - mean rstd;  dx = gw rstd - m1 rstd - xhat m2 rstd;  dw += g xhat;  db += g
template <typename T, int TPR, int ITEMS, int MODE, int RU, bool BIAS>
__global__ void __launch_bounds__(256, 2)
family_bwd_rows_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ dx,
                       float* __restrict__ partial, int64_t rows, int nvec, int64_t ldg, int64_t ldx, int64_t lddx,
                       float cols_f, float eps, int line_arrays, const T* __restrict__ gs, int64_t ldgs, float offset) {
  constexpr int V = Num<T>::kVec;
  constexpr int P = V / 2;  // fp32 pairs per word
  constexpr int GROUPS = 256 / TPR;
  constexpr bool LAYER = MODE == kLayer || MODE == kRms || MODE == kRmsAdd;  // modes with a weight: dw (and db) partials per thread
  constexpr bool KEEP_W = ITEMS < 4 || !BIAS;  // wide rows with a bias gradient re-read their weight words (L1 hits): no registers left
  static_assert(RU == 1 || TPR <= 32, "several rows per group only for rows that fit a warp");
  pdl_prologue();
  constexpr int SLOT_GROUPS = (TPR > 32 && TPR < 256) ? GROUPS : 1;  // rows that meet at a barrier of their own
  __shared__ float slot_store[SLOT_GROUPS][8][8];
  __shared__ float fold[LAYER && GROUPS > 1 ? 2 * TPR * ITEMS * V : 1];
  const int tid = threadIdx.x;
  const int sub = tid / TPR, lane_in_row = tid % TPR;
  float(*slots)[8] = slot_store[SLOT_GROUPS > 1 ? sub : 0];
  bool col_ok[ITEMS];
  uint4 wv[LAYER && KEEP_W ? ITEMS : 1];
  auto weight_word = [&](int i) { return KEEP_W ? wv[KEEP_W ? i : 0] : ld_reuse(weight + static_cast<int64_t>(lane_in_row + i * TPR) * V); };
  Float2x dw[LAYER ? ITEMS : 1][P], db[LAYER && BIAS ? ITEMS : 1][P];  // BIAS: the op has a bias, so db is wanted
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    col_ok[i] = lane_in_row + i * TPR < nvec;
    if constexpr (LAYER) {
      if constexpr (KEEP_W) {
        wv[i] = make_uint4(0, 0, 0, 0);
        if (col_ok[i]) wv[i] = ld_reuse(weight + static_cast<int64_t>(lane_in_row + i * TPR) * V);
      }
#pragma unroll
      for (int j = 0; j < P; ++j) {
        dw[i][j] = pack_f2(0.f, 0.f);
        if constexpr (BIAS) db[i][j] = pack_f2(0.f, 0.f);
      }
    }
  }
  const int64_t stride = static_cast<int64_t>(gridDim.x) * GROUPS * RU;
  int parity = 0;  // the L2 mode has one barrier per row: consecutive rows alternate between two slot pairs
  // every thread of the CTA runs the same number of iterations (barriers and full-warp shuffles inside)
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * GROUPS * RU; base < rows; base += stride, parity ^= 1) {
    uint4 xv[RU][ITEMS], gv[RU][ITEMS];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int64_t row = base + static_cast<int64_t>(sub) * RU + u;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        xv[u][i] = gv[u][i] = make_uint4(0, 0, 0, 0);
        if (row < rows && col_ok[i]) {
          const int64_t col = static_cast<int64_t>(lane_in_row + i * TPR) * V;
          xv[u][i] = ld_stream(x + row * ldx + col);
          gv[u][i] = ld_stream(gy + row * ldg + col);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int64_t row = base + static_cast<int64_t>(sub) * RU + u;
      const bool live = row < rows;
      if constexpr (MODE == kL2) {
        Float2x ss2 = pack_f2(0.f, 0.f), dot2 = ss2;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          Float2x fx[P], fg[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
#pragma unroll
          for (int j = 0; j < P; ++j) {
            ss2 = fma_f2(fx[j], fx[j], ss2);
            dot2 = fma_f2(fg[j], fx[j], dot2);
          }
        }
        float sums[2] = {pair_total(ss2), pair_total(dot2)};
        row_sums<TPR, 2>(sums, &slots[parity * 2], sub);
        const float sc = __frcp_rn(__fsqrt_rn(__fadd_rn(sums[0], eps)));
        const float coef = -__fmul_rn(__fmul_rn(__fmul_rn(sc, sc), sc), sums[1]);
        const Float2x sc2 = pack_f2(sc, sc), coef2 = pack_f2(coef, coef);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          Float2x fx[P], fg[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
          float out[V];
#pragma unroll
          for (int j = 0; j < P; ++j) unpack_f2(fma_f2(fg[j], sc2, mul_f2(fx[j], coef2)), out[2 * j], out[2 * j + 1]);
          if (live && col_ok[i]) st_stream(dx + row * lddx + static_cast<int64_t>(lane_in_row + i * TPR) * V, Num<T>::pack(out));
        }
      } else if constexpr (MODE == kRms || MODE == kRmsAdd) {
        // y = x r w (+ b), r = 1 / sqrt(mean x^2 + eps):  dx = gw r - x r^3 <gw, x> / n,  dw += g x r,  db += g.
        // add_rms_norm's backward is the same on s = x + residual with w = round_T(weight + offset), plus the
        // gradient that arrived for s itself (gs): dx = round_T(dx) + gs.
        const Float2x offset2 = pack_f2(offset, offset);
        auto effective_weight = [&](int i, Float2x (&fw)[P]) {
          unpack_pairs<T>(weight_word(i), fw);
          if constexpr (MODE == kRmsAdd) {
#pragma unroll
            for (int j = 0; j < P; ++j) {
              float lo, hi;
              unpack_f2(add_f2(fw[j], offset2), lo, hi);
              if constexpr (sizeof(T) == 2) Num<T>::round2(lo, hi);
              fw[j] = pack_f2(lo, hi);
            }
          }
        };
        Float2x ss2 = pack_f2(0.f, 0.f), dot2 = ss2;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          if (!col_ok[i]) continue;
          Float2x fx[P], fg[P], fw[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
          effective_weight(i, fw);
#pragma unroll
          for (int j = 0; j < P; ++j) {
            ss2 = fma_f2(fx[j], fx[j], ss2);
            dot2 = fma_f2(mul_f2(fg[j], fw[j]), fx[j], dot2);
          }
        }
        float sums[2] = {pair_total(ss2), pair_total(dot2)};
        row_sums<TPR, 2>(sums, &slots[parity * 2], sub);
        const float r = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sums[0], cols_f), eps)));
        const float coef = -__fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(r, r), r), sums[1]), cols_f);
        const Float2x r2 = pack_f2(r, r), coef2 = pack_f2(coef, coef);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          if (!col_ok[i]) continue;
          Float2x fx[P], fg[P], fw[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
          effective_weight(i, fw);
          float out[V];
#pragma unroll
          for (int j = 0; j < P; ++j) {
            dw[i][j] = fma_f2(fg[j], mul_f2(fx[j], r2), dw[i][j]);
            if constexpr (BIAS) db[i][j] = add_f2(db[i][j], fg[j]);
            unpack_f2(fma_f2(mul_f2(fg[j], fw[j]), r2, mul_f2(fx[j], coef2)), out[2 * j], out[2 * j + 1]);
          }
          if (MODE == kRmsAdd && gs != nullptr && live) {
            float extra[V];
            Num<T>::unpack(ld_stream(gs + row * ldgs + static_cast<int64_t>(lane_in_row + i * TPR) * V), extra);
#pragma unroll
            for (int j = 0; j < V; j += 2) {
              if constexpr (sizeof(T) == 2) Num<T>::round2(out[j], out[j + 1]);
              out[j] = __fadd_rn(out[j], extra[j]);
              out[j + 1] = __fadd_rn(out[j + 1], extra[j + 1]);
            }
          }
          if (live) st_stream(dx + row * lddx + static_cast<int64_t>(lane_in_row + i * TPR) * V, Num<T>::pack(out));
        }
      } else {
        // 16-bit rows: the variance comes from the same pass as the mean, as E[x^2] - mean^2 in fp32 (its error, about
        // 1e-6 (1 + mean^2 / var), is far below the 2^-9 rounding of the outputs; one barrier and one unpacking of the
        // row less per row).  fp32 rows keep the two-pass form sum (x - mean)^2, whose gradients are graded to 2e-5.
        constexpr bool ONE_PASS = sizeof(T) == 2;
        Float2x sx2 = pack_f2(0.f, 0.f), s12 = sx2, sgx2 = sx2, sxx2 = sx2;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          if (!col_ok[i]) continue;
          Float2x fx[P], fg[P], fw[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
          unpack_pairs<T>(weight_word(i), fw);
#pragma unroll
          for (int j = 0; j < P; ++j) {
            const Float2x gw = mul_f2(fg[j], fw[j]);
            sx2 = add_f2(sx2, fx[j]);
            s12 = add_f2(s12, gw);
            sgx2 = fma_f2(gw, fx[j], sgx2);
            if constexpr (ONE_PASS) sxx2 = fma_f2(fx[j], fx[j], sxx2);
          }
        }
        float first[ONE_PASS ? 4 : 3];
        first[0] = pair_total(sx2), first[1] = pair_total(s12), first[2] = pair_total(sgx2);
        if constexpr (ONE_PASS) first[3] = pair_total(sxx2);
        // one barrier per row in the one-pass form: consecutive rows alternate between two sets of slots
        row_sums<TPR, ONE_PASS ? 4 : 3>(first, &slots[ONE_PASS ? parity * 4 : 0], sub);
        const float mean = __fdiv_rn(first[0], cols_f);
        const Float2x mean2 = pack_f2(mean, mean);
        float variance;
        if constexpr (ONE_PASS) {
          variance = __fsub_rn(__fdiv_rn(first[3], cols_f), __fmul_rn(mean, mean));
        } else {
          Float2x var2 = pack_f2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < ITEMS; ++i) {
            if (!col_ok[i]) continue;  // padding columns must not see -mean
            Float2x fx[P];
            unpack_pairs<T>(xv[u][i], fx);
#pragma unroll
            for (int j = 0; j < P; ++j) {
              const Float2x d = sub_f2(fx[j], mean2);
              var2 = fma_f2(d, d, var2);
            }
          }
          float second[1] = {pair_total(var2)};
          row_sums<TPR, 1>(second, &slots[3], sub);
          variance = __fdiv_rn(second[0], cols_f);
        }
        const float rstd = __frcp_rn(__fsqrt_rn(__fadd_rn(fmaxf(variance, 0.f), eps)));
        const float m1 = __fdiv_rn(first[1], cols_f);                                                     // mean of g w
        const float m2 = __fdiv_rn(__fmul_rn(__fsub_rn(first[2], __fmul_rn(mean, first[1])), rstd), cols_f);  // mean of g w xhat
        const float shift = -__fmul_rn(mean, rstd), c1 = -__fmul_rn(m1, rstd), c2 = -__fmul_rn(m2, rstd);
        const Float2x rstd2 = pack_f2(rstd, rstd), shift2 = pack_f2(shift, shift), c12 = pack_f2(c1, c1), c22 = pack_f2(c2, c2);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          if (!col_ok[i]) continue;
          Float2x fx[P], fg[P], fw[P];
          unpack_pairs<T>(xv[u][i], fx);
          unpack_pairs<T>(gv[u][i], fg);
          unpack_pairs<T>(weight_word(i), fw);
          float out[V];
#pragma unroll
          for (int j = 0; j < P; ++j) {
            const Float2x xhat = fma_f2(fx[j], rstd2, shift2);  // a row past the end is all zeros: mean, shift and xhat are 0
            dw[i][j] = fma_f2(fg[j], xhat, dw[i][j]);
            if constexpr (BIAS) db[i][j] = add_f2(db[i][j], fg[j]);
            unpack_f2(fma_f2(xhat, c22, fma_f2(mul_f2(fg[j], fw[j]), rstd2, c12)), out[2 * j], out[2 * j + 1]);
          }
          if (live) st_stream(dx + row * lddx + static_cast<int64_t>(lane_in_row + i * TPR) * V, Num<T>::pack(out));
        }
      }
    }
  }
  if constexpr (LAYER) {
    // this CTA's line of the partial sums: [0][cols] for dw, [1][cols] for db (line_arrays = 1: dw only)
    float* line = partial + static_cast<int64_t>(blockIdx.x) * line_arrays * nvec * V;
    if constexpr (GROUPS > 1) {
      // fold the row groups in group order: group 0 stores, every later group adds, one barrier per group
      for (int g = 0; g < GROUPS; ++g) {
        if (sub == g) {
#pragma unroll
          for (int i = 0; i < ITEMS; ++i)
#pragma unroll
            for (int j = 0; j < P; ++j) {
              const int c = (lane_in_row + i * TPR) * V + 2 * j;
              float w0, w1;
              unpack_f2(dw[i][j], w0, w1);
              float* fw = fold + c;
              fw[0] = g == 0 ? w0 : __fadd_rn(fw[0], w0);
              fw[1] = g == 0 ? w1 : __fadd_rn(fw[1], w1);
              if constexpr (BIAS) {
                float b0, b1;
                unpack_f2(db[i][j], b0, b1);
                float* fb = fold + TPR * ITEMS * V + c;
                fb[0] = g == 0 ? b0 : __fadd_rn(fb[0], b0);
                fb[1] = g == 0 ? b1 : __fadd_rn(fb[1], b1);
              }
            }
        }
        __syncthreads();
      }
      for (int c = tid; c < nvec * V; c += 256) {
        line[c] = fold[c];
        if constexpr (BIAS) line[nvec * V + c] = fold[TPR * ITEMS * V + c];
      }
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        if (!col_ok[i]) continue;
        const int64_t c = static_cast<int64_t>(lane_in_row + i * TPR) * V;
#pragma unroll
        for (int j = 0; j < P; j += 2) {
          float a0, a1, a2, a3;
          unpack_f2(dw[i][j], a0, a1);
          unpack_f2(dw[i][j + 1], a2, a3);
          *reinterpret_cast<float4*>(line + c + 2 * j) = make_float4(a0, a1, a2, a3);
          if constexpr (BIAS) {
            unpack_f2(db[i][j], a0, a1);
            unpack_f2(db[i][j + 1], a2, a3);
            *reinterpret_cast<float4*>(line + nvec * V + c + 2 * j) = make_float4(a0, a1, a2, a3);
          }
        }
      }
    }
  }
}

// dw[c] = round_T(sum over lines of partial[line][0][c]), db likewise from partial[line][1][c].  A CTA owns 32
// columns; its eight warps each add every eighth line (a warp load is one 128-byte segment of a line), then the
// eight partial sums are added in warp order, so the result does not depend on timing.
template <typename T>
__global__ void __launch_bounds__(256)
family_sum_lines_kernel(const float* __restrict__ partial, int lines, int line_arrays, int64_t cols, T* __restrict__ dw, T* __restrict__ db) {
  pdl_prologue();
  __shared__ float part[2][8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + lane;
  float aw = 0.f, ab = 0.f;
  if (c < cols) {
    for (int l = warp; l < lines; l += 8) {
      aw = __fadd_rn(aw, partial[(static_cast<int64_t>(l) * line_arrays) * cols + c]);
      if (db != nullptr) ab = __fadd_rn(ab, partial[(static_cast<int64_t>(l) * line_arrays + 1) * cols + c]);
    }
  }
  part[0][warp][lane] = aw;
  part[1][warp][lane] = ab;
  __syncthreads();
  if (warp == 0 && c < cols) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tw = __fadd_rn(tw, part[0][k][lane]);
      tb = __fadd_rn(tb, part[1][k][lane]);
    }
    dw[c] = Num<T>::down(tw);
    if (db != nullptr) db[c] = Num<T>::down(tb);
  }
}

int family_bwd_lines(int64_t rows) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * 2;  // the row kernels run two CTAs per SM
  return static_cast<int>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

// CTAs of the persistent backward launch for `groups` rows per CTA pass; also the number of partial lines.
int family_bwd_ctas(int64_t rows, int groups) {
  const int64_t want = ceil_div(rows > 0 ? rows : 1, static_cast<int64_t>(groups));
  const int64_t cap = family_bwd_lines(rows);
  return static_cast<int>(want < cap ? want : cap);
}

template <typename T, int MODE>
int run_bwd(const void* gy, const void* x, const void* w, void* dx, void* dw, void* db, float* scratch, int64_t rows, int64_t cols,
            int64_t ldg, int64_t ldx, int64_t lddx, float eps, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const bool vec = cols % V == 0 && ldg % V == 0 && ldx % V == 0 && lddx % V == 0 && aligned(gy, 16) && aligned(x, 16) && aligned(dx, 16) &&
                   (w == nullptr || aligned(w, 16));
  const T *tg = static_cast<const T*>(gy), *tx = static_cast<const T*>(x), *tw = static_cast<const T*>(w);
  T* tdx = static_cast<T*>(dx);
  const float cols_f = static_cast<float>(cols);
  const int bias = db != nullptr ? 1 : 0;
  const int64_t nvec64 = cols / V;
  int lines = 0;
  if (vec && nvec64 <= 1024) {
    const int nvec = static_cast<int>(nvec64);
#define B200_FAMILY_BWD(TPR, ITEMS, RU)                                                                                          \
  do {                                                                                                                           \
    lines = family_bwd_ctas(rows, 256 / TPR * RU);                                                                               \
    if (bias)                                                                                                                    \
      launch(family_bwd_rows_kernel<T, TPR, ITEMS, MODE, RU, true>, static_cast<unsigned>(lines), 256, 0, st, tg, tx, tw, tdx,   \
             scratch, rows, nvec, ldg, ldx, lddx, cols_f, eps, 2, static_cast<const T*>(nullptr), 0, 0.f);                       \
    else                                                                                                                         \
      launch(family_bwd_rows_kernel<T, TPR, ITEMS, MODE, RU, false>, static_cast<unsigned>(lines), 256, 0, st, tg, tx, tw, tdx,  \
             scratch, rows, nvec, ldg, ldx, lddx, cols_f, eps, 2, static_cast<const T*>(nullptr), 0, 0.f);                       \
  } while (0)
    if (nvec <= 8) B200_FAMILY_BWD(8, 1, 4);
    else if (nvec <= 16) B200_FAMILY_BWD(16, 1, 4);
    else if (nvec <= 32) B200_FAMILY_BWD(32, 1, 4);
    else if (nvec <= 64) B200_FAMILY_BWD(32, 2, 1);
    else if (nvec <= 128) B200_FAMILY_BWD(32, 4, 1);
    else if (nvec <= 256) B200_FAMILY_BWD(64, 4, 1);
    else if (nvec <= 384) B200_FAMILY_BWD(128, 3, 1);
    else if (nvec <= 512) B200_FAMILY_BWD(128, 4, 1);
    else if (nvec <= 768) B200_FAMILY_BWD(256, 3, 1);
    else B200_FAMILY_BWD(256, 4, 1);
#undef B200_FAMILY_BWD
    if (int rc = after_launch("family_bwd_rows_kernel")) return rc;
  } else {
    lines = family_bwd_lines(rows);
    if (vec) launch(family_bwd_kernel<T, MODE, true>, lines, 256, 0, st, tg, tx, tw, tdx, scratch, rows, cols, ldg, ldx, lddx, cols_f, eps, bias);
    else launch(family_bwd_kernel<T, MODE, false>, lines, 256, 0, st, tg, tx, tw, tdx, scratch, rows, cols, ldg, ldx, lddx, cols_f, eps, bias);
    if (int rc = after_launch("family_bwd_kernel")) return rc;
  }
  if (MODE == kLayer) {
    launch(family_sum_lines_kernel<T>, static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, st, static_cast<const float*>(scratch), lines, 2, cols,
           static_cast<T*>(dw), static_cast<T*>(db));
    return after_launch("family_sum_lines_kernel");
  }
  return B200_OK;
}

template <typename T, int MODE>
int run_rms_narrow(const void* gy, const void* gs, const void* x, const void* w, void* dx, void* dw, void* db, float* scratch, int64_t rows,
                   int nvec, int64_t ldg, int64_t ldgs, int64_t ldx, int64_t lddx, float eps, float offset, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const T *tg = static_cast<const T*>(gy), *tx = static_cast<const T*>(x), *tw = static_cast<const T*>(w);
  T* tdx = static_cast<T*>(dx);
  const int64_t cols = static_cast<int64_t>(nvec) * V;
  const float cols_f = static_cast<float>(cols);
  const int bias = db != nullptr ? 1 : 0, arrays = bias ? 2 : 1;
  int lines = 0;
#define B200_RMS_NARROW(TPR, ITEMS, RU)                                                                                       \
  do {                                                                                                                        \
    lines = family_bwd_ctas(rows, 256 / TPR * RU);                                                                            \
    if (bias)                                                                                                                 \
      launch(family_bwd_rows_kernel<T, TPR, ITEMS, MODE, RU, true>, static_cast<unsigned>(lines), 256, 0, st, tg, tx, tw, tdx, \
             scratch, rows, nvec, ldg, ldx, lddx, cols_f, eps, arrays, static_cast<const T*>(gs), ldgs, offset);              \
    else                                                                                                                      \
      launch(family_bwd_rows_kernel<T, TPR, ITEMS, MODE, RU, false>, static_cast<unsigned>(lines), 256, 0, st, tg, tx, tw, tdx, \
             scratch, rows, nvec, ldg, ldx, lddx, cols_f, eps, arrays, static_cast<const T*>(gs), ldgs, offset);              \
  } while (0)
  if (nvec <= 8) B200_RMS_NARROW(8, 1, 4);
  else if (nvec <= 16) B200_RMS_NARROW(16, 1, 4);
  else if (nvec <= 32) B200_RMS_NARROW(32, 1, 4);
  else if (nvec <= 64) B200_RMS_NARROW(32, 2, 1);
  else if (nvec <= 128) B200_RMS_NARROW(32, 4, 1);
  else if (nvec <= 256) B200_RMS_NARROW(64, 4, 1);
  else if (nvec <= 384) B200_RMS_NARROW(128, 3, 1);
  else if (nvec <= 512) B200_RMS_NARROW(128, 4, 1);
  else if (nvec <= 768) B200_RMS_NARROW(256, 3, 1);
  else B200_RMS_NARROW(256, 4, 1);
#undef B200_RMS_NARROW
  if (int rc = after_launch("family_bwd_rows_kernel")) return rc;
  launch(family_sum_lines_kernel<T>, static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, st, static_cast<const float*>(scratch), lines, arrays, cols,
         static_cast<T*>(dw), static_cast<T*>(db));
  return after_launch("family_sum_lines_kernel");
}

int bwd_entry(const char* fn, int mode, const void* gy, const void* x, const void* weight, void* dx, void* dw, void* db,
              int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx, int dtype, double eps, void* scratch, size_t scratch_bytes,
              void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (rows > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "%s: rows=%lld exceeds 2^31-1", fn, (long long)rows);
  if (cols == 0) return B200_OK;
  if (gy == nullptr || x == nullptr || dx == nullptr || (mode == kLayer && (weight == nullptr || dw == nullptr || scratch == nullptr)))
    return fail(B200_ERR_NULL_POINTER, "%s: a required pointer is NULL", fn);
  if (ldg < cols || ldx < cols || lddx < cols) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", fn);
  const size_t es = dtype_size(dtype);
  if (!aligned(gy, es) || !aligned(x, es) || !aligned(dx, es) || !aligned(weight, es) || !aligned(dw, es) || !aligned(db, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  if (mode == kLayer) {
    const size_t need = static_cast<size_t>(family_bwd_lines(rows)) * 2 * static_cast<size_t>(cols) * sizeof(float);
    if (scratch_bytes < need || !aligned(scratch, 16))
      return fail(B200_ERR_SCRATCH, "%s: scratch needs %zu bytes, 16-byte aligned (got %zu)", fn, need, scratch_bytes);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float e = static_cast<float>(eps);
  float* sc = static_cast<float*>(scratch);
  if (mode == kL2) {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, kL2>(gy, x, nullptr, dx, nullptr, nullptr, sc, rows, cols, ldg, ldx, lddx, e, st)));
  } else {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, kLayer>(gy, x, weight, dx, dw, db, sc, rows, cols, ldg, ldx, lddx, e, st)));
  }
  return B200_OK;
}

}  // namespace

int rms_backward_narrow_rows(int dtype, const void* gy, const void* gs, const void* x, const void* w, void* dx, void* dw, void* db,
                             float* scratch, int64_t rows, int64_t cols, int64_t ldg, int64_t ldgs, int64_t ldx, int64_t lddx, float eps,
                             float offset, bool add, cudaStream_t st) {
  B200_DISPATCH_DTYPE(dtype, T, {
    if (add) return run_rms_narrow<T, kRmsAdd>(gy, gs, x, w, dx, dw, db, scratch, rows, static_cast<int>(cols / Num<T>::kVec), ldg, ldgs, ldx, lddx, eps, offset, st);
    return run_rms_narrow<T, kRms>(gy, nullptr, x, w, dx, dw, db, scratch, rows, static_cast<int>(cols / Num<T>::kVec), ldg, 0, ldx, lddx, eps, 0.f, st);
  });
  return B200_ERR_DTYPE;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rms_norm_gated(const void* x, const void* gate, const void* weight, const void* bias, void* y,
                                   int64_t rows, int64_t cols, int64_t ldx, int64_t ldg, int64_t ldy,
                                   int dtype, int sigmoid_gate, double eps, void* stream) {
  return entry(__func__, sigmoid_gate ? kGatedSigmoid : kGatedSwish, x, gate, weight, bias, y, rows, cols, ldx, ldg, ldy, dtype, eps, stream);
}

extern "C" int b200_l2_norm(const void* x, void* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                            int dtype, double eps, void* stream) {
  return entry(__func__, kL2, x, nullptr, nullptr, nullptr, y, rows, cols, ldx, 0, ldy, dtype, eps, stream);
}

extern "C" int b200_layer_norm(const void* x, const void* weight, const void* bias, void* y,
                               int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                               int dtype, double eps, void* stream) {
  return entry(__func__, kLayer, x, nullptr, weight, bias, y, rows, cols, ldx, 0, ldy, dtype, eps, stream);
}

extern "C" int b200_l2_norm_backward(const void* grad_y, const void* x, void* grad_x, int64_t rows, int64_t cols,
                                     int64_t ldg, int64_t ldx, int64_t lddx, int dtype, double eps, void* stream) {
  return bwd_entry(__func__, kL2, grad_y, x, nullptr, grad_x, nullptr, nullptr, rows, cols, ldg, ldx, lddx, dtype, eps, nullptr, 0, stream);
}

extern "C" int b200_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols, size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (int rc = check_device()) return rc;
  *bytes = static_cast<size_t>(family_bwd_lines(rows)) * 2 * static_cast<size_t>(cols > 0 ? cols : 1) * sizeof(float);
  return B200_OK;
}

extern "C" int b200_layer_norm_backward(const void* grad_y, const void* x, const void* weight, void* grad_x, void* grad_weight,
                                        void* grad_bias, int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx,
                                        int dtype, double eps, void* scratch, size_t scratch_bytes, void* stream) {
  return bwd_entry(__func__, kLayer, grad_y, x, weight, grad_x, grad_weight, grad_bias, rows, cols, ldg, ldx, lddx, dtype, eps, scratch,
                   scratch_bytes, stream);
}

