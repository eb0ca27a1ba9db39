// Rotary position embedding (GPT-NeoX halves or GPT-J pairs) for sm_100a.
//
// Bound: HBM (each element of q / k read once and written once; the fp32
// cos/sin table is small and stays in L2).  A CTA owns a tile of consecutive
// sequence positions: the tile's cos/sin rows are staged in shared memory by
// bulk asynchronous copies, and each thread rotates one fixed (head, channel
// group) of q or k over the tile's positions, for one or more batch entries.
//
// Arithmetic follows src/popcorn/kernels/rotary_embedding.py:28-40 of the
// reference: fp32 products and sums rounded one by one, one final rounding.
#include "common.cuh"
#include "tma.cuh"

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

// The same from shared memory.
template <typename CS, int N>
__device__ __forceinline__ void load_cs_shared(const CS* p, float (&f)[N]) {
  if constexpr (sizeof(CS) == 4) {
    if constexpr (N == 2) {
      const float2 v = *reinterpret_cast<const float2*>(p);
      f[0] = v.x;
      f[1] = v.y;
    } else {
#pragma unroll
      for (int i = 0; i < N / 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(p + 4 * i);
        f[4 * i] = v.x;
        f[4 * i + 1] = v.y;
        f[4 * i + 2] = v.z;
        f[4 * i + 3] = v.w;
      }
    }
  } else {
    if constexpr (N == 4) {
      const uint2 v = *reinterpret_cast<const uint2*>(p);
      Num<CS>::unpack2(v.x, f[0], f[1]);
      Num<CS>::unpack2(v.y, f[2], f[3]);
    } else {
      static_assert(N == 8, "16-bit cos/sin come in groups of 4 or 8");
      Num<CS>::unpack(*reinterpret_cast<const uint4*>(p), f);
    }
  }
}

__device__ __forceinline__ void rotate(float x1, float x2, float c, float s, float& y1, float& y2) {
  y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  y2 = __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
}

// A "unit" is the smallest piece one thread rotates on its own:
//   NeoX:        one 128-bit word of the first half plus its partner in the second half
//   interleaved: one 128-bit word (V/2 adjacent pairs)
// A position of q and k together holds units_per_pos = (q_heads + k_heads) * units_per_head
// of them.  A CTA is laid out as `groups` x `tpp` threads: thread (g, r) owns unit r
// (and r + tpp, ... if a position has more units than tpp) of the TS consecutive
// positions of group g, so its head, channel group and tensor are fixed and found
// once.  The CTA's cos/sin rows (groups * TS positions, contiguous in the table)
// are staged in shared memory by two bulk asynchronous copies while the first
// loads of x are already in flight.
constexpr int kRopeTS = 4;

template <typename T, typename CS, bool INTERLEAVED>
__global__ void __launch_bounds__(512, 2) rope_tile_kernel(const RopeArgs p, int tpp, int groups) {
  constexpr int V = Num<T>::kVec;
  constexpr int NCS = INTERLEAVED ? V / 2 : V;  // cos values per unit
  constexpr int TS = kRopeTS;
  extern __shared__ __align__(16) unsigned char rope_smem[];
  __shared__ __align__(8) uint64_t bar;

  pdl_prologue();
  const int tile_positions = groups * TS;
  const int64_t tiles = (p.seq + tile_positions - 1) / tile_positions;
  const int64_t tile = blockIdx.x % tiles;
  const int split = static_cast<int>(blockIdx.x / tiles);
  const int64_t pos0 = tile * tile_positions;
  const int n_pos = static_cast<int>(p.seq - pos0 < tile_positions ? p.seq - pos0 : tile_positions);

  CS* cos_s = reinterpret_cast<CS*>(rope_smem);
  CS* sin_s = cos_s + static_cast<size_t>(tile_positions) * p.half;
  const uint32_t table_bytes = static_cast<uint32_t>(n_pos) * p.half * sizeof(CS);
  const CS* cos_g = static_cast<const CS*>(p.cos) + pos0 * p.half;
  const CS* sin_g = static_cast<const CS*>(p.sin) + pos0 * p.half;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    mbar_arrive_expect(&bar, 2 * table_bytes);
    bulk_load(cos_s, cos_g, table_bytes, &bar);
    bulk_load(sin_s, sin_g, table_bytes, &bar);
  }
  __syncthreads();  // the barrier is initialised before anyone polls it

  const int grp = threadIdx.x / tpp;
  const int r0 = threadIdx.x - grp * tpp;
  const int uph = (INTERLEAVED ? 2 * p.half : p.half) / V;  // units per head
  const int heads0 = p.t[0].heads;
  const int upp = (heads0 + (p.n_tensors > 1 ? p.t[1].heads : 0)) * uph;
  const int gpos = grp * TS;  // first position of my group inside the tile
  const int tail_words = (p.head_dim - 2 * p.half) / V;

  uint4 v1[TS], v2[INTERLEAVED ? 1 : TS];
  // the loads of one (batch, unit) item: TS positions, one or two words each
  auto issue_loads = [&](int b, int r) {
    int hh = r / uph;
    const int g = r - hh * uph;
    const int ti = hh >= heads0 ? 1 : 0;
    if (ti) hh -= heads0;
    const RopeTensor& t = p.t[ti];
    const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + (pos0 + gpos) * t.xs_s + hh * t.xs_h + static_cast<int64_t>(g) * V;
#pragma unroll
    for (int k = 0; k < TS; ++k) {
      if (gpos + k < n_pos) {
        v1[k] = ld_stream(xin + k * t.xs_s);
        if constexpr (!INTERLEAVED) v2[k] = ld_stream(xin + k * t.xs_s + p.half);
      }
    }
  };

  // The first item's loads go out before anyone waits for the tables.
  bool first = true;
  if (split < p.batch && r0 < upp) issue_loads(split, r0);

  // Wait for the tables (every thread, at this one place).  If the bounded wait
  // runs out anywhere in the CTA, all threads fill the tables with ordinary loads.
  {
    const bool ok = mbar_wait(&bar, 0);
    if (__syncthreads_or(!ok)) {
      const int n = n_pos * p.half;
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        cos_s[i] = cos_g[i];
        sin_s[i] = sin_g[i];
      }
      __syncthreads();
    }
  }

  for (int b = split; b < p.batch; b += p.batch_split) {
    for (int r = r0; r < upp; r += tpp) {
      if (!first) issue_loads(b, r);
      first = false;
      int hh = r / uph;
      const int g = r - hh * uph;
      const int ti = hh >= heads0 ? 1 : 0;
      if (ti) hh -= heads0;
      const RopeTensor& t = p.t[ti];
      T* xout = static_cast<T*>(t.out) + b * t.os_b + (pos0 + gpos) * t.os_s + hh * t.os_h + static_cast<int64_t>(g) * V;
#pragma unroll
      for (int k = 0; k < TS; ++k) {
        if (gpos + k >= n_pos) continue;
        float c[NCS], sn[NCS];
        load_cs_shared<CS, NCS>(cos_s + (gpos + k) * p.half + g * NCS, c);
        load_cs_shared<CS, NCS>(sin_s + (gpos + k) * p.half + g * NCS, sn);
        float a[V];
        Num<T>::unpack(v1[k], a);
        if constexpr (INTERLEAVED) {
#pragma unroll
          for (int j = 0; j < V / 2; ++j) {
            float y1, y2;
            rotate(a[2 * j], a[2 * j + 1], c[j], sn[j], y1, y2);
            a[2 * j] = y1;
            a[2 * j + 1] = y2;
          }
          st_stream(xout + k * t.os_s, Num<T>::pack(a));
        } else {
          float d[V];
          Num<T>::unpack(v2[k], d);
          // The four products of two channels come from packed fp32x2 multiplies (each half rounded
          // on its own, identical to __fmul_rn); the difference and the sum stay scalar, because the
          // assembler turns a packed product followed by a packed add/sub into one fused
          // multiply-add (measured), which would change the rounding.
#pragma unroll
          for (int j = 0; j < V; j += 2) {
            const Float2x x1 = pack_f2(a[j], a[j + 1]), x2 = pack_f2(d[j], d[j + 1]);
            const Float2x cc = pack_f2(c[j], c[j + 1]), ss = pack_f2(sn[j], sn[j + 1]);
            float ac0, ac1, ds0, ds1, as0, as1, dc0, dc1;
            unpack_f2(mul_f2(x1, cc), ac0, ac1);
            unpack_f2(mul_f2(x2, ss), ds0, ds1);
            unpack_f2(mul_f2(x1, ss), as0, as1);
            unpack_f2(mul_f2(x2, cc), dc0, dc1);
            a[j] = __fsub_rn(ac0, ds0);
            a[j + 1] = __fsub_rn(ac1, ds1);
            d[j] = __fadd_rn(as0, dc0);
            d[j + 1] = __fadd_rn(as1, dc1);
          }
          st_stream(xout + k * t.os_s, Num<T>::pack(a));
          st_stream(xout + k * t.os_s + p.half, Num<T>::pack(d));
        }
      }
    }
    // channels past the rotated ones pass through (nothing to do in place)
    if (tail_words > 0) {
      for (int ti = 0; ti < p.n_tensors; ++ti) {
        const RopeTensor& t = p.t[ti];
        if (t.x == t.out) continue;
        const int words = t.heads * tail_words;
        for (int k = 0; k < TS; ++k) {
          if (gpos + k >= n_pos) break;
          const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + (pos0 + gpos + k) * t.xs_s;
          T* xout = static_cast<T*>(t.out) + b * t.os_b + (pos0 + gpos + k) * t.os_s;
          for (int w = r0; w < words; w += tpp) {
            const int h = w / tail_words;
            const int64_t j = 2 * p.half + static_cast<int64_t>(w - h * tail_words) * V;
            st_stream(xout + h * t.os_h + j, ld_stream(xin + h * t.xs_h + j));
          }
        }
      }
    }
  }
}

// Any shape, any alignment: one thread per (batch, position, head, channel pair or tail channel).
template <typename T, typename CS, bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_scalar_kernel(const RopeArgs p) {
  pdl_prologue();
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
  // bulk copies need 16-byte aligned table rows
  vec = vec && (static_cast<size_t>(p.half) * sizeof(CS)) % 16 == 0 && aligned(p.cos, 16) && aligned(p.sin, 16);
  if (vec) {
    const int uph = (INTERLEAVED ? 2 * p.half : p.half) / V;
    int64_t upp = static_cast<int64_t>(p.t[0].heads + (p.n_tensors > 1 ? p.t[1].heads : 0)) * uph;
    // threads per position: all its units if they fit in a CTA, in whole warps
    int tpp = static_cast<int>(upp < 512 ? (upp + 31) / 32 * 32 : 512);
    int groups = 256 / tpp > 0 ? 256 / tpp : 1;
    const int threads = tpp * groups;
    const int tile_positions = groups * kRopeTS;
    const int64_t tiles = ceil_div(p.seq, tile_positions);
    // one CTA per (tile, batch entry) unless that is far more CTAs than the machine needs
    const int64_t want = static_cast<int64_t>(sm_count()) * 64;
    int split = p.batch;
    while (split > 1 && tiles * split > want && split % 2 == 0) split /= 2;
    p.batch_split = split;
    const int64_t grid = tiles * split;
    if (grid > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "b200_rope: problem too large for one launch");
    const size_t smem = 2 * static_cast<size_t>(tile_positions) * p.half * sizeof(CS);
    if (smem <= 48 * 1024) {
      launch(rope_tile_kernel<T, CS, INTERLEAVED>, static_cast<unsigned>(grid), threads, smem, st, p, tpp, groups);
      return after_launch("rope_tile_kernel");
    }
  }
  p.batch_split = 1;
  launch(rope_scalar_kernel<T, CS, INTERLEAVED>, static_cast<unsigned>(sm_count()) * 8, 256, 0, st, p);
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

unsigned int rope_wait_timeouts() { return read_wait_timeouts(); }

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
