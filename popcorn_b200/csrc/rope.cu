// Rotary position embedding (GPT-NeoX halves or GPT-J pairs) for sm_100a.
//
// Bound: HBM (each element of q / k read once and written once; the fp32
// cos/sin table is small and stays in L2).  One warp owns one sequence
// position: it keeps that position's cos/sin values in registers and walks
// over the heads of q and, in the fused entry point, k, for one or more batch
// entries.  The eight warps of a CTA share a position and differ in batch, so
// the cos/sin row is pulled into L1 once per CTA.
//
// Arithmetic follows src/popcorn/kernels/rotary_embedding.py:28-40 of the
// reference: fp32 products and sums rounded one by one, one final rounding.
#include "common.cuh"

namespace b200 {
namespace {

struct RopeTensor {
  const void* x;
  void* out;
  int64_t xs_b, xs_s, xs_h;
  int64_t os_b, os_s, os_h;
  int heads;
};

struct RopeArgs {
  RopeTensor t[2];
  int n_tensors;
  const void* cos;
  const void* sin;
  int64_t seq;
  int batch;
  int batch_split;  // warps per position; warp w of a position takes batches w, w + split, ...
  int half;
  int head_dim;
};

// N consecutive cos (or sin) values -> fp32 registers.
template <typename CS, int N>
__device__ __forceinline__ void load_cs(const CS* p, float (&f)[N]) {
  if constexpr (sizeof(CS) == 4) {
    if constexpr (N == 2) {
      const float2 v = __ldg(reinterpret_cast<const float2*>(p));
      f[0] = v.x;
      f[1] = v.y;
    } else {
#pragma unroll
      for (int i = 0; i < N / 4; ++i) {
        float g[4];
        Num<float>::unpack(ld_reuse(p + 4 * i), g);
#pragma unroll
        for (int j = 0; j < 4; ++j) f[4 * i + j] = g[j];
      }
    }
  } else {
    if constexpr (N == 4) {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
      Num<CS>::unpack2(v.x, f[0], f[1]);
      Num<CS>::unpack2(v.y, f[2], f[3]);
    } else {
      static_assert(N == 8, "16-bit cos/sin come in groups of 4 or 8");
      Num<CS>::unpack(ld_reuse(p), f);
    }
  }
}

__device__ __forceinline__ void rotate(float x1, float x2, float c, float s, float& y1, float& y2) {
  y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  y2 = __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
}

// A "unit" is the smallest piece one lane rotates on its own:
//   NeoX:        one 128-bit word of the first half plus its partner in the second half
//   interleaved: one 128-bit word (V/2 adjacent pairs)
// FIXED: 32 is a multiple of the units per head, so a lane meets the same
// channel group at every step and loads its cos/sin once.
template <typename T, typename CS, bool INTERLEAVED, bool FIXED>
__global__ void __launch_bounds__(256) rope_warp_kernel(const RopeArgs p) {
  constexpr int V = Num<T>::kVec;
  constexpr int NCS = INTERLEAVED ? V / 2 : V;  // cos values per unit
  constexpr int UNROLL = 4;
  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t pos = warp / p.batch_split;
  const int split = static_cast<int>(warp - pos * p.batch_split);
  if (pos >= p.seq) return;

  const int uph = (INTERLEAVED ? 2 * p.half : p.half) / V;  // units per head
  const CS* cos_row = static_cast<const CS*>(p.cos) + pos * p.half;
  const CS* sin_row = static_cast<const CS*>(p.sin) + pos * p.half;
  float c[NCS], s[NCS];
  if (FIXED) {
    const int g = lane % uph;
    load_cs<CS, NCS>(cos_row + g * NCS, c);
    load_cs<CS, NCS>(sin_row + g * NCS, s);
  }
  const int tail_words = (p.head_dim - 2 * p.half) / V;

  for (int b = split; b < p.batch; b += p.batch_split) {
    for (int ti = 0; ti < p.n_tensors; ++ti) {
      const RopeTensor& t = p.t[ti];
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s;
      T* xout = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s;
      const int units = t.heads * uph;
      for (int u0 = lane; u0 < units; u0 += 32 * UNROLL) {
        uint4 v1[UNROLL], v2[INTERLEAVED ? 1 : UNROLL];
        int64_t off_o[UNROLL];
        int grp[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
          const int u = u0 + 32 * k;
          const int h = u / uph;
          grp[k] = u - h * uph;
          const int64_t off_i = h * t.xs_h + static_cast<int64_t>(grp[k]) * V;
          off_o[k] = h * t.os_h + static_cast<int64_t>(grp[k]) * V;
          if (u < units) {
            v1[k] = ld_stream(xin + off_i);
            if constexpr (!INTERLEAVED) v2[k] = ld_stream(xin + off_i + p.half);
          }
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
          if (u0 + 32 * k >= units) continue;
          if (!FIXED) {
            load_cs<CS, NCS>(cos_row + grp[k] * NCS, c);
            load_cs<CS, NCS>(sin_row + grp[k] * NCS, s);
          }
          float a[V];
          Num<T>::unpack(v1[k], a);
          if constexpr (INTERLEAVED) {
#pragma unroll
            for (int j = 0; j < V / 2; ++j) {
              float y1, y2;
              rotate(a[2 * j], a[2 * j + 1], c[j], s[j], y1, y2);
              a[2 * j] = y1;
              a[2 * j + 1] = y2;
            }
            st_stream(xout + off_o[k], Num<T>::pack(a));
          } else {
            float d[V];
            Num<T>::unpack(v2[k], d);
#pragma unroll
            for (int j = 0; j < V; ++j) {
              float y1, y2;
              rotate(a[j], d[j], c[j], s[j], y1, y2);
              a[j] = y1;
              d[j] = y2;
            }
            st_stream(xout + off_o[k], Num<T>::pack(a));
            st_stream(xout + off_o[k] + p.half, Num<T>::pack(d));
          }
        }
      }
      // channels past the rotated ones pass through (nothing to do in place)
      if (tail_words > 0 && t.x != t.out) {
        const int words = t.heads * tail_words;
        for (int w = lane; w < words; w += 32) {
          const int h = w / tail_words;
          const int64_t j = 2 * p.half + static_cast<int64_t>(w - h * tail_words) * V;
          st_stream(xout + h * t.os_h + j, ld_stream(xin + h * t.xs_h + j));
        }
      }
    }
  }
}

// Any shape, any alignment: one thread per (batch, position, head, channel pair or tail channel).
template <typename T, typename CS, bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_scalar_kernel(const RopeArgs p) {
  const int per_head = p.half + (p.head_dim - 2 * p.half);  // pairs, then pass-through channels
  for (int ti = 0; ti < p.n_tensors; ++ti) {
    const RopeTensor& t = p.t[ti];
    const int64_t total = static_cast<int64_t>(p.batch) * p.seq * t.heads * per_head;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int j = static_cast<int>(i % per_head);
      int64_t r = i / per_head;
      const int h = static_cast<int>(r % t.heads);
      r /= t.heads;
      const int64_t pos = r % p.seq;
      const int64_t b = r / p.seq;
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + h * t.xs_h;
      T* xout = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s + h * t.os_h;
      if (j >= p.half) {
        const int ch = 2 * p.half + (j - p.half);
        if (t.x != t.out) xout[ch] = xin[ch];
        continue;
      }
      const int i1 = INTERLEAVED ? 2 * j : j;
      const int i2 = INTERLEAVED ? 2 * j + 1 : j + p.half;
      const float c = Num<CS>::up(static_cast<const CS*>(p.cos)[pos * p.half + j]);
      const float s = Num<CS>::up(static_cast<const CS*>(p.sin)[pos * p.half + j]);
      float y1, y2;
      rotate(Num<T>::up(xin[i1]), Num<T>::up(xin[i2]), c, s, y1, y2);
      xout[i1] = Num<T>::down(y1);
      xout[i2] = Num<T>::down(y2);
    }
  }
}

template <typename T, typename CS, bool INTERLEAVED>
int run(RopeArgs& p, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  constexpr int NCS = INTERLEAVED ? V / 2 : V;
  // cos/sin are fetched in pieces of at most 16 bytes; every row must start on such a piece
  constexpr size_t kPiece = NCS * sizeof(CS) < 16 ? NCS * sizeof(CS) : 16;
  bool vec = p.half > 0 && p.half % V == 0 && p.head_dim % V == 0 && aligned(p.cos, kPiece) && aligned(p.sin, kPiece) &&
             (static_cast<size_t>(p.half) * sizeof(CS)) % kPiece == 0;
  for (int i = 0; i < p.n_tensors; ++i) {
    const RopeTensor& t = p.t[i];
    vec = vec && aligned(t.x, 16) && aligned(t.out, 16) && t.xs_b % V == 0 && t.xs_s % V == 0 && t.xs_h % V == 0 &&
          t.os_b % V == 0 && t.os_s % V == 0 && t.os_h % V == 0;
  }
  if (vec) {
    // enough warps to fill the machine several times over, else split the batch
    const int64_t want = static_cast<int64_t>(sm_count()) * 64 * 4;
    int split = p.batch;
    while (split > 1 && p.seq * split > want && split % 2 == 0) split /= 2;
    p.batch_split = split;
    const int64_t warps = p.seq * split;
    const int64_t grid = ceil_div(warps, 8);
    if (grid > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "b200_rope: problem too large for one launch");
    const int uph = (INTERLEAVED ? 2 * p.half : p.half) / V;
    if (32 % uph == 0)
      rope_warp_kernel<T, CS, INTERLEAVED, true><<<static_cast<unsigned>(grid), 256, 0, st>>>(p);
    else
      rope_warp_kernel<T, CS, INTERLEAVED, false><<<static_cast<unsigned>(grid), 256, 0, st>>>(p);
    return after_launch("rope_warp_kernel");
  }
  p.batch_split = 1;
  rope_scalar_kernel<T, CS, INTERLEAVED><<<static_cast<unsigned>(sm_count()) * 8, 256, 0, st>>>(p);
  return after_launch("rope_scalar_kernel");
}

template <typename T>
int run_cs(RopeArgs& p, int cs_dtype, int interleaved, cudaStream_t st) {
  if (cs_dtype == B200_F32) {
    return interleaved ? run<T, float, true>(p, st) : run<T, float, false>(p, st);
  }
  return interleaved ? run<T, T, true>(p, st) : run<T, T, false>(p, st);
}

int validate(const char* fn, int64_t batch, int64_t seq, int64_t head_dim, int64_t half, int dtype, int cs_dtype) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (cs_dtype != B200_F32 && cs_dtype != dtype)
    return fail(B200_ERR_DTYPE, "%s: cos/sin must be fp32 or the dtype of x (got %d vs %d)", fn, cs_dtype, dtype);
  if (batch < 0 || seq < 0 || head_dim < 0 || half < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (2 * half > head_dim) return fail(B200_ERR_SHAPE, "%s: 2*half=%lld exceeds head_dim=%lld", fn, (long long)(2 * half), (long long)head_dim);
  if (batch > 0x7fffffffLL || head_dim > (1 << 20)) return fail(B200_ERR_SHAPE, "%s: batch or head_dim out of range", fn);
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_rope(const void* x, const void* cos, const void* sin, void* out,
                         int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, int64_t half,
                         int64_t x_stride_b, int64_t x_stride_s, int64_t x_stride_h,
                         int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h,
                         int dtype, int cs_dtype, int interleaved, void* stream) {
  if (int rc = validate(__func__, batch, seq, head_dim, half, dtype, cs_dtype)) return rc;
  if (heads < 0 || heads > (1 << 20)) return fail(B200_ERR_SHAPE, "%s: heads out of range", __func__);
  if (batch == 0 || seq == 0 || heads == 0 || head_dim == 0) return B200_OK;
  B200_REQUIRE_PTR(x);
  B200_REQUIRE_PTR(out);
  if (half > 0) {
    B200_REQUIRE_PTR(cos);
    B200_REQUIRE_PTR(sin);
  }
  const size_t es = dtype_size(dtype);
  if (!aligned(x, es) || !aligned(out, es) || !aligned(cos, dtype_size(cs_dtype)) || !aligned(sin, dtype_size(cs_dtype)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  RopeArgs p{};
  p.t[0] = RopeTensor{x, out, x_stride_b, x_stride_s, x_stride_h, o_stride_b, o_stride_s, o_stride_h, static_cast<int>(heads)};
  p.n_tensors = 1;
  p.cos = cos;
  p.sin = sin;
  p.seq = seq;
  p.batch = static_cast<int>(batch);
  p.half = static_cast<int>(half);
  p.head_dim = static_cast<int>(head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return run_cs<T>(p, cs_dtype, interleaved, st));
  return B200_OK;
}

extern "C" int b200_rope_qk(void* q, void* k, const void* cos, const void* sin,
                            int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads,
                            int64_t head_dim, int64_t half,
                            int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                            int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                            int dtype, int cs_dtype, int interleaved, void* stream) {
  if (int rc = validate(__func__, batch, seq, head_dim, half, dtype, cs_dtype)) return rc;
  if (q_heads < 0 || k_heads < 0 || q_heads > (1 << 20) || k_heads > (1 << 20))
    return fail(B200_ERR_SHAPE, "%s: heads out of range", __func__);
  if (batch == 0 || seq == 0 || head_dim == 0 || (q_heads == 0 && k_heads == 0)) return B200_OK;
  if (q_heads > 0) B200_REQUIRE_PTR(q);
  if (k_heads > 0) B200_REQUIRE_PTR(k);
  if (half > 0) {
    B200_REQUIRE_PTR(cos);
    B200_REQUIRE_PTR(sin);
  }
  const size_t es = dtype_size(dtype);
  if (!aligned(q, es) || !aligned(k, es) || !aligned(cos, dtype_size(cs_dtype)) || !aligned(sin, dtype_size(cs_dtype)))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  RopeArgs p{};
  int n = 0;
  if (q_heads > 0) p.t[n++] = RopeTensor{q, q, q_stride_b, q_stride_s, q_stride_h, q_stride_b, q_stride_s, q_stride_h, static_cast<int>(q_heads)};
  if (k_heads > 0) p.t[n++] = RopeTensor{k, k, k_stride_b, k_stride_s, k_stride_h, k_stride_b, k_stride_s, k_stride_h, static_cast<int>(k_heads)};
  p.n_tensors = n;
  p.cos = cos;
  p.sin = sin;
  p.seq = seq;
  p.batch = static_cast<int>(batch);
  p.half = static_cast<int>(half);
  p.head_dim = static_cast<int>(head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return run_cs<T>(p, cs_dtype, interleaved, st));
  return B200_OK;
}
