// SwiGLU forward for sm_100a:  out = round_T(round_T(silu(a)) * b).
//
// Bound: HBM (2 reads + 1 write per element, ~20 fp32 instructions).  `a` and `b`
// are addressed through their own leading dimensions, so the two column halves
// of a fused [rows, 2*cols] gate_up buffer are consumed in place; the
// incumbent (src/popcorn/impls/swiglu.cu:80-81) copies them to contiguous
// buffers first.
//
// Arithmetic follows F.silu(a) * b of src/popcorn/kernels/swiglu.py:18 as PyTorch
// evaluates it for a 16-bit dtype: silu = a / (1 + exp(-a)) in fp32, rounded to
// T, then the product computed in fp32 and rounded to T again.
#include "activations.cuh"
#include "common.cuh"

namespace b200 {
namespace {

template <typename T, int ACT>
__device__ __forceinline__ float swiglu_one(float a, float b) {
  return Num<T>::rt(__fmul_rn(Num<T>::rt(silu_f32<0, ACT>(a)), b));
}

// Each thread owns UNROLL 128-bit words, THREADS words apart, so a warp always
// touches 512 contiguous bytes of one row.  (row, word) of the first word comes
// from one division; the rest follow by carry.
template <typename T, int UNROLL, typename Index, int MATH, int ACT>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const T* a, const T* b, T* out, Index total_words, Index words_per_row,
                  int64_t lda, int64_t ldb, int64_t ldo) {
  constexpr int V = Num<T>::kVec;
  constexpr int THREADS = 256;
  pdl_prologue();
  const Index first = static_cast<Index>(blockIdx.x) * (THREADS * UNROLL) + threadIdx.x;
  Index row = first / words_per_row;
  Index word = first - row * words_per_row;

  uint4 va[UNROLL], vb[UNROLL];
  int64_t off_o[UNROLL];
  bool ok[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    ok[u] = first + static_cast<Index>(u) * THREADS < total_words;
    va[u] = make_uint4(0, 0, 0, 0);
    vb[u] = make_uint4(0, 0, 0, 0);
    if (ok[u]) {
      va[u] = ld_stream(a + static_cast<int64_t>(row) * lda + static_cast<int64_t>(word) * V);
      vb[u] = ld_stream(b + static_cast<int64_t>(row) * ldb + static_cast<int64_t>(word) * V);
    }
    off_o[u] = static_cast<int64_t>(row) * ldo + static_cast<int64_t>(word) * V;
    word += THREADS;
    if (word >= words_per_row) {
      if (words_per_row >= THREADS) {  // at most one row boundary crossed
        word -= words_per_row;
        ++row;
      } else {
        const Index next = first + static_cast<Index>(u + 1) * THREADS;
        row = next / words_per_row;
        word = next - row * words_per_row;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    if constexpr (sizeof(T) == 4) {
      float fa[V], fb[V];
      Num<T>::unpack(va[u], fa);
      Num<T>::unpack(vb[u], fb);
#pragma unroll
      for (int j = 0; j < V; ++j) fa[j] = __fmul_rn(silu_f32<MATH, ACT>(fa[j]), fb[j]);
      if (ok[u]) st_stream(out + off_o[u], Num<T>::pack(fa));
    } else {
      // 16-bit: silu of a pair in fp32, one packed rounding to T, then the packed product with
      // the untouched word of b (rounded once, as the reference's 16-bit multiply is)
      const uint32_t wa[4] = {va[u].x, va[u].y, va[u].z, va[u].w};
      const uint32_t wb[4] = {vb[u].x, vb[u].y, vb[u].z, vb[u].w};
      uint32_t wo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo, hi;
        Num<T>::unpack2(wa[j], lo, hi);
        wo[j] = Num<T>::mul2(Num<T>::pack2(silu_f32<MATH, ACT>(lo), silu_f32<MATH, ACT>(hi)), wb[j]);
      }
      if (ok[u]) st_stream(out + off_o[u], make_uint4(wo[0], wo[1], wo[2], wo[3]));
    }
  }
}

// ---------------------------------------------------------------- backward --
//
// out = round_T(silu(a)) * b.  PyTorch's autograd of the reference evaluates, tensor by tensor,
//   db = round_T(g * round_T(silu(a)))
//   gs = round_T(g * b)                                  (gradient reaching silu)
//   da = round_T(gs * (s * (1 + a * (1 - s)))),  s = 1 / (1 + exp(-a)) in fp32
// and this kernel does the same in one pass (3 reads, 2 writes per element).
// GEGLU (tanh approximation): with s = 1 / (1 + exp(-2u)) = 0.5 * (1 + tanh u), u = sqrt(2/pi) * (a + 0.044715 a^3),
//   gelu'(a) = s + a * (1 - tanh^2 u) / 2 * u' = s * (1 + 2 a (1 - s) u'),  u' = sqrt(2/pi) * (1 + 3 * 0.044715 a^2),
// the derivative PyTorch's gelu backward evaluates (0.5 (1 + tanh u) + 0.5 a (1 - tanh^2 u) u') in another arrangement.
template <int MATH, int ACT = kSilu>
__device__ __forceinline__ float dsilu_f32(float a) {
  const float d = __fadd_rn(1.0f, exp_neg<MATH>(gate_argument<ACT>(a)));
  const float s = MATH == 0 ? __fdiv_rn(1.0f, d) : rcp_approx(d);
  if constexpr (ACT == kSilu) {
    return __fmul_rn(s, __fmaf_rn(a, __fsub_rn(1.0f, s), 1.0f));
  } else {
    const float du = __fmul_rn(0.7978845608028654f, __fmaf_rn(__fmul_rn(3.0f * 0.044715f, a), a, 1.0f));
    return __fmul_rn(s, __fmaf_rn(__fmul_rn(__fmul_rn(2.0f, a), __fsub_rn(1.0f, s)), du, 1.0f));
  }
}

// The gate's value as the forward computes it, and the gradient of out = gate(a) * b with respect to a, given
// gs = grad * b rounded to T and s = gate(a) rounded to T (what autograd keeps).  For the sigmoid gate PyTorch's
// sigmoid backward evaluates (gs * (1 - s)) * s on the ROUNDED s; the other gates differentiate the fp32 value.
template <int MATH, int ACT>
__device__ __forceinline__ float gate_value(float a) {
  if constexpr (ACT == kSigmoidGate) return sigmoid_f32<MATH>(a);
  else return silu_f32<MATH, ACT>(a);
}
template <int MATH, int ACT>
__device__ __forceinline__ float gate_grad(float gs, float s, float a) {
  if constexpr (ACT == kSigmoidGate) return __fmul_rn(__fmul_rn(gs, __fsub_rn(1.0f, s)), s);
  else return __fmul_rn(gs, dsilu_f32<MATH, ACT>(a));
}

template <typename T, int UNROLL, typename Index, int MATH, int ACT>
__global__ void __launch_bounds__(256)
swiglu_bwd_vec_kernel(const T* g, const T* a, const T* b, T* da, T* db, Index total_words, Index words_per_row,
                      int64_t ldg, int64_t lda, int64_t ldb, int64_t ldda, int64_t lddb) {
  constexpr int V = Num<T>::kVec;
  constexpr int THREADS = 256;
  pdl_prologue();
  const Index first = static_cast<Index>(blockIdx.x) * (THREADS * UNROLL) + threadIdx.x;
  uint4 vg[UNROLL], va[UNROLL], vb[UNROLL];
  int64_t off_da[UNROLL], off_db[UNROLL];
  bool ok[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const Index idx = first + static_cast<Index>(u) * THREADS;
    ok[u] = idx < total_words;
    const Index row = idx / words_per_row;
    const int64_t word = static_cast<int64_t>(idx - row * words_per_row) * V;
    const int64_t r = static_cast<int64_t>(row);
    vg[u] = va[u] = vb[u] = make_uint4(0, 0, 0, 0);
    if (ok[u]) {
      vg[u] = ld_stream(g + r * ldg + word);
      va[u] = ld_stream(a + r * lda + word);
      vb[u] = ld_stream(b + r * ldb + word);
    }
    off_da[u] = r * ldda + word;
    off_db[u] = r * lddb + word;
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    float fg[V], fa[V], fb[V], ra[V], rb[V];
    Num<T>::unpack(vg[u], fg);
    Num<T>::unpack(va[u], fa);
    Num<T>::unpack(vb[u], fb);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float s = Num<T>::rt(gate_value<MATH, ACT>(fa[j]));
      rb[j] = __fmul_rn(fg[j], s);
      const float gs = Num<T>::rt(__fmul_rn(fg[j], fb[j]));
      ra[j] = gate_grad<MATH, ACT>(gs, s, fa[j]);
    }
    if (ok[u]) {
      st_stream(da + off_da[u], Num<T>::pack(ra));
      st_stream(db + off_db[u], Num<T>::pack(rb));
    }
  }
}

template <typename T, int ACT>
__global__ void __launch_bounds__(256)
swiglu_bwd_scalar_kernel(const T* g, const T* a, const T* b, T* da, T* db, int64_t rows, int64_t cols,
                         int64_t ldg, int64_t lda, int64_t ldb, int64_t ldda, int64_t lddb) {
  pdl_prologue();
  const int64_t total = rows * cols;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const float fg = Num<T>::up(g[r * ldg + c]), fa = Num<T>::up(a[r * lda + c]), fb = Num<T>::up(b[r * ldb + c]);
    const float s = Num<T>::rt(gate_value<0, ACT>(fa));
    db[r * lddb + c] = Num<T>::down(__fmul_rn(fg, s));
    da[r * ldda + c] = Num<T>::down(gate_grad<0, ACT>(Num<T>::rt(__fmul_rn(fg, fb)), s, fa));
  }
}

template <typename T, int ACT>
int run_bwd(const void* g, const void* a, const void* b, void* da, void* db, int64_t rows, int64_t cols,
            int64_t ldg, int64_t lda, int64_t ldb, int64_t ldda, int64_t lddb, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  constexpr int UNROLL = 2;
  constexpr int MATH = sizeof(T) == 4 ? 0 : 1;
  const bool vec = cols % V == 0 && ldg % V == 0 && lda % V == 0 && ldb % V == 0 && ldda % V == 0 && lddb % V == 0 &&
                   aligned(g, 16) && aligned(a, 16) && aligned(b, 16) && aligned(da, 16) && aligned(db, 16);
  const int64_t wpr = cols / V;
  const int64_t total = rows * wpr;
  if (vec && total < 0x7fffffffLL) {
    launch(swiglu_bwd_vec_kernel<T, UNROLL, uint32_t, MATH, ACT>, static_cast<unsigned>(ceil_div(total, 256 * UNROLL)), 256, 0, st,
           static_cast<const T*>(g), static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(da), static_cast<T*>(db),
           static_cast<uint32_t>(total), static_cast<uint32_t>(wpr), ldg, lda, ldb, ldda, lddb);
    return after_launch("swiglu_bwd_vec_kernel");
  }
  const int64_t want = ceil_div(rows * cols, 256);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  launch(swiglu_bwd_scalar_kernel<T, ACT>, static_cast<unsigned>(want < cap ? want : cap), 256, 0, st,
         static_cast<const T*>(g), static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(da), static_cast<T*>(db),
         rows, cols, ldg, lda, ldb, ldda, lddb);
  return after_launch("swiglu_bwd_scalar_kernel");
}

// Any width, any alignment.
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
swiglu_scalar_kernel(const T* a, const T* b, T* out, int64_t rows, int64_t cols,
                     int64_t lda, int64_t ldb, int64_t ldo) {
  pdl_prologue();
  const int64_t total = rows * cols;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    out[r * ldo + c] = Num<T>::down(swiglu_one<T, ACT>(Num<T>::up(a[r * lda + c]), Num<T>::up(b[r * ldb + c])));
  }
}

template <typename T, int ACT>
int run(const void* a, const void* b, void* out, int64_t rows, int64_t cols,
        int64_t lda, int64_t ldb, int64_t ldo, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  constexpr int UNROLL = 4;
  const bool vec = cols % V == 0 && lda % V == 0 && ldb % V == 0 && ldo % V == 0 && aligned(a, 16) &&
                   aligned(b, 16) && aligned(out, 16);
  if (vec) {
    int64_t wpr = cols / V;
    int64_t n_rows = rows;
    if (lda == cols && ldb == cols && ldo == cols) {  // fully contiguous: one long row
      wpr = rows * wpr;
      n_rows = 1;
    }
    const int64_t total = n_rows * wpr;
    const int64_t grid = ceil_div(total, 256 * UNROLL);
    if (grid > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "b200_swiglu: problem too large for one launch");
    constexpr int MATH = sizeof(T) == 4 ? 0 : 1;
    if (total < 0x7fffffffLL) {
      launch(swiglu_vec_kernel<T, UNROLL, uint32_t, MATH, ACT>, static_cast<unsigned>(grid), 256, 0, st,
             static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), static_cast<uint32_t>(total),
             static_cast<uint32_t>(wpr), lda, ldb, ldo);
    } else {
      launch(swiglu_vec_kernel<T, UNROLL, uint64_t, MATH, ACT>, static_cast<unsigned>(grid), 256, 0, st,
             static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), static_cast<uint64_t>(total),
             static_cast<uint64_t>(wpr), lda, ldb, ldo);
    }
    return after_launch("swiglu_vec_kernel");
  }
  const int64_t want = ceil_div(rows * cols, 256);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  launch(swiglu_scalar_kernel<T, ACT>, static_cast<unsigned>(want < cap ? want : cap), 256, 0, st,
      static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), rows, cols, lda, ldb, ldo);
  return after_launch("swiglu_scalar_kernel");
}

}  // namespace
}  // namespace b200

using namespace b200;

namespace b200 {
namespace {
template <int ACT>
int gated_forward(const char* fn, const void* a, const void* b, void* out, int64_t rows, int64_t cols,
                  int64_t lda, int64_t ldb, int64_t ldo, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (rows == 0 || cols == 0) return B200_OK;
  if (a == nullptr || b == nullptr || out == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: a, b or out is NULL", fn);
  if (lda < cols || ldb < cols || ldo < cols) return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", fn);
  const size_t es = dtype_size(dtype);
  if (!aligned(a, es) || !aligned(b, es) || !aligned(out, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return (run<T, ACT>(a, b, out, rows, cols, lda, ldb, ldo, st)));
  return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" int b200_swiglu(const void* a, const void* b, void* out, int64_t rows, int64_t cols,
                           int64_t lda, int64_t ldb, int64_t ldo, int dtype, void* stream) {
  return gated_forward<kSilu>(__func__, a, b, out, rows, cols, lda, ldb, ldo, dtype, stream);
}

extern "C" int b200_geglu(const void* a, const void* b, void* out, int64_t rows, int64_t cols,
                          int64_t lda, int64_t ldb, int64_t ldo, int dtype, void* stream) {
  return gated_forward<kGeluTanh>(__func__, a, b, out, rows, cols, lda, ldb, ldo, dtype, stream);
}

namespace {

int gate_backward(const char* fn, int act, const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                  int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb, int64_t ldda, int64_t lddb, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (rows < 0 || cols < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (rows == 0 || cols == 0) return B200_OK;
  if (grad_out == nullptr || a == nullptr || b == nullptr || grad_a == nullptr || grad_b == nullptr)
    return fail(B200_ERR_NULL_POINTER, "%s: a required pointer is NULL", fn);
  if (ldg < cols || lda < cols || ldb < cols || ldda < cols || lddb < cols)
    return fail(B200_ERR_SHAPE, "%s: leading dimension smaller than cols", fn);
  const size_t es = dtype_size(dtype);
  if (!aligned(grad_out, es) || !aligned(a, es) || !aligned(b, es) || !aligned(grad_a, es) || !aligned(grad_b, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == kSilu) {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, kSilu>(grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, st)));
  } else if (act == kSigmoidGate) {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, kSigmoidGate>(grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, st)));
  } else {
    B200_DISPATCH_DTYPE(dtype, T, return (run_bwd<T, kGeluTanh>(grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, st)));
  }
  return B200_OK;
}

}  // namespace

extern "C" int b200_swiglu_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                                    int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                                    int64_t ldda, int64_t lddb, int dtype, void* stream) {
  return gate_backward(__func__, kSilu, grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, dtype, stream);
}

extern "C" int b200_geglu_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                                   int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                                   int64_t ldda, int64_t lddb, int dtype, void* stream) {
  return gate_backward(__func__, kGeluTanh, grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, dtype, stream);
}

extern "C" int b200_sigmoid_gate_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                                          int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                                          int64_t ldda, int64_t lddb, int dtype, void* stream) {
  return gate_backward(__func__, kSigmoidGate, grad_out, a, b, grad_a, grad_b, rows, cols, ldg, lda, ldb, ldda, lddb, dtype, stream);
}
