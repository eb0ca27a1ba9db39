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
#include <algorithm>

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
  int tail_elsewhere;  // the channels past the rotated ones are copied by rope_tail_kernel, not by the rotation kernel
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
// TS positions per thread.  Eight for the interleaved form (whose unit is one word, so four positions keep only 64
// bytes per thread in flight) was measured again and again at 0.83-0.85 of the copy peak, like four: no gain, a few
// spilled registers; both forms use four.
template <bool INTERLEAVED>
constexpr int rope_ts() { return 4; }

template <typename T, typename CS, bool INTERLEAVED>
__global__ void __launch_bounds__(512, 2) rope_tile_kernel(const RopeArgs p, int tpp, int groups) {
  constexpr int V = Num<T>::kVec;
  constexpr int NCS = INTERLEAVED ? V / 2 : V;  // cos values per unit
  constexpr int TS = rope_ts<INTERLEAVED>();
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
  bool tables_late = false;  // the same in every thread of the CTA
  {
    const bool ok = mbar_wait(&bar, 0);
    tables_late = __syncthreads_or(!ok);
    if (tables_late) {
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
    if (tail_words > 0 && !p.tail_elsewhere) {
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
  if (tables_late) {
    // the two bulk copies may still be in flight into this CTA's shared memory (they bring the same bytes the plain
    // loads wrote): thread 0 gives them one more bounded wait and the CTA stays resident until it returns, so that
    // a late copy cannot land in shared memory that already belongs to another CTA
    if (threadIdx.x == 0) (void)mbar_wait(&bar, 0);
    __syncthreads();
  }
}

// Any shape, any alignment: one thread per (batch, position, head, channel pair or tail channel).
// Out-of-place partial rotary: the channels past the rotated ones are a strided copy, four 128-bit words in flight
// per thread (inside rope_tile_kernel, which has no registers to spare, the same copy ran one word at a time).
template <typename T>
__global__ void __launch_bounds__(256) rope_tail_kernel(const RopeArgs p) {
  constexpr int V = Num<T>::kVec;
  constexpr int U = 4;
  pdl_prologue();
  const int tail_words = (p.head_dim - 2 * p.half) / V;
  for (int ti = 0; ti < p.n_tensors; ++ti) {
    const RopeTensor& t = p.t[ti];
    if (t.x == t.out || t.heads == 0) continue;
    const int64_t per_pos = static_cast<int64_t>(t.heads) * tail_words;
    const int64_t total = static_cast<int64_t>(p.batch) * p.seq * per_pos;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i0 < total; i0 += stride * U) {
      uint4 held[U];
      int64_t dst[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + u * stride;
        if (i < total) {
          const int64_t bp = i / per_pos;
          const int rem = static_cast<int>(i - bp * per_pos);
          const int h = rem / tail_words, w = rem - h * tail_words;
          const int64_t b = bp / p.seq, pos = bp - b * p.seq;
          const int64_t j = 2 * p.half + static_cast<int64_t>(w) * V;
          held[u] = ld_stream(static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + h * t.xs_h + j);
          dst[u] = b * t.os_b + pos * t.os_s + h * t.os_h + j;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < total) st_stream(static_cast<T*>(t.out) + dst[u], held[u]);
    }
  }
}

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
    const int tile_positions = groups * rope_ts<INTERLEAVED>();
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
      bool out_of_place = false;
      for (int i = 0; i < p.n_tensors; ++i) out_of_place = out_of_place || p.t[i].x != p.t[i].out;
      p.tail_elsewhere = (p.head_dim > 2 * p.half && out_of_place) ? 1 : 0;
      if (p.tail_elsewhere) {
        launch(rope_tail_kernel<T>, static_cast<unsigned>(sm_count()) * 8, 256, 0, st, p);
        if (int rc = after_launch("rope_tail_kernel")) return rc;
      }
      launch(rope_tile_kernel<T, CS, INTERLEAVED>, static_cast<unsigned>(grid), threads, smem, st, p, tpp, groups);
      return after_launch("rope_tile_kernel");
    }
  }
  p.batch_split = 1;
  launch(rope_scalar_kernel<T, CS, INTERLEAVED>, static_cast<unsigned>(sm_count()) * 8, 256, 0, st, p);
  return after_launch("rope_scalar_kernel");
}

// ------------------------------------------------------------ paired rope --
//
// rope(q, k, cos, sin) of the reference (src/popcorn/kernels/rope.py:24-36): layout
// (batch, heads, seq, head_dim), tables [cos_batch, seq, head_dim] in the dtype of q, and the
// arithmetic done tensor by tensor in that dtype:
//   y = round_T(round_T(x * cos) + round_T(rot(x) * sin)),  rot(x) = (-x[half:], x[:half])
struct PairedTensor {
  const void* x;
  void* out;
  int64_t xs_b, xs_h, xs_s;
  int64_t os_b, os_h, os_s;
  int heads;
};
struct PairedArgs {
  PairedTensor t[2];
  const void* cos;
  const void* sin;
  int64_t cs_stride_b;  // 0 when the tables have one batch entry
  int64_t seq;
  int batch;
  int head_dim;
  // fused per-head RMS normalisation (qk_norm_rope): one weight row of head_dim per tensor
  const void* weight[2];
  float eps;
};

// 1 / sqrt(sum / n + eps) for the per-head norm, where it is evaluated once per 2 x head_dim elements and
// the IEEE division, square root and reciprocal (about 25 instructions) would be a tenth of the kernel.
// `inv_n` > 0 says n is a power of two: sum * inv_n is then exact and one fused multiply-add gives the
// reference's round(round(sum / n) + eps).  The reciprocal square root is the hardware approximation
// polished by one Newton step, i.e. the true value rounded to within about half a unit in the last place;
// the reference's 1 / sqrt (two roundings) differs from it in the last bit about as often as a different
// summation order of the squares does.  Arguments of 0 / inf (and denormal ones, flushed to 0) give the
// approximation's own inf / 0, like the reference.
__device__ __forceinline__ float inv_rms(float sumsq, float n, float inv_n, float eps) {
  const float v = inv_n > 0.f ? __fmaf_rn(sumsq, inv_n, eps) : __fadd_rn(__fdiv_rn(sumsq, n), eps);
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(v));
  const float e = __fmaf_rn(-__fmul_rn(v, y), y, 1.0f);  // 1 - v*y^2
  const float y1 = __fmaf_rn(__fmul_rn(0.5f, y), e, y);
  return e == e ? y1 : y;
}

// One unit = a 128-bit word of the first half of a row and its partner in the second half.
// A thread owns one (position, unit): it keeps the four table words it needs in registers and
// walks over all heads of q and k of one batch entry, four heads in flight at a time.
//
// NORM fuses the per-head RMS normalisation of qk_norm_rope in front of the rotation
// (examples/03_write_a_kernel.ipynb, cell 3): x <- round_T(round_T(x * r) * w) with
// r = 1/sqrt(mean(x^2) + eps) in fp32.  The row's units sit in adjacent lanes (units per row is
// a power of two <= 32 on this path), so the sum of squares is a few shuffles; lanes whose
// position is past the end compute on the last position and store nothing, which keeps every
// shuffle full-width.
template <typename T, bool NORM>
__global__ void __launch_bounds__(256, NORM ? 2 : 3) rope_paired_kernel(const PairedArgs p) {
  constexpr int V = Num<T>::kVec;
  // heads in flight per thread; the fused norm keeps fewer CTAs resident (more registers), so each asks for more
  constexpr int UNROLL = NORM ? 8 : 4;
  pdl_prologue();
  const int half = p.head_dim / 2;
  const int upr = half / V;  // units per row
  const int tile_pos = 256 / upr;
  const int64_t tiles = (p.seq + tile_pos - 1) / tile_pos;
  const int64_t tile = blockIdx.x % tiles;
  const int b = static_cast<int>(blockIdx.x / tiles);
  const int unit = threadIdx.x % upr;
  int64_t pos = tile * tile_pos + threadIdx.x / upr;
  bool active = threadIdx.x / upr < tile_pos && pos < p.seq;
  if constexpr (NORM) {
    if (!active) pos = p.seq - 1;
  } else {
    if (!active) return;
  }

  const T* cos = static_cast<const T*>(p.cos) + b * p.cs_stride_b + pos * p.head_dim + unit * V;
  const T* sin = static_cast<const T*>(p.sin) + b * p.cs_stride_b + pos * p.head_dim + unit * V;
  const uint4 c1 = ld_reuse(cos), c2 = ld_reuse(cos + half), s1 = ld_reuse(sin), s2 = ld_reuse(sin + half);

  auto combine = [](uint4 x, uint4 c, uint4 r, uint4 sn, bool negate_r) {
    if constexpr (sizeof(T) == 4) {
      float fx[4], fc[4], fr[4], fs[4];
      Num<T>::unpack(x, fx);
      Num<T>::unpack(c, fc);
      Num<T>::unpack(r, fr);
      Num<T>::unpack(sn, fs);
#pragma unroll
      for (int j = 0; j < 4; ++j) fx[j] = __fadd_rn(__fmul_rn(fx[j], fc[j]), __fmul_rn(negate_r ? -fr[j] : fr[j], fs[j]));
      return Num<T>::pack(fx);
    } else {
      const uint32_t flip = negate_r ? 0x80008000u : 0u;  // sign bits of both 16-bit halves
      const uint32_t wx[4] = {x.x, x.y, x.z, x.w}, wc[4] = {c.x, c.y, c.z, c.w};
      const uint32_t wr[4] = {r.x, r.y, r.z, r.w}, ws[4] = {sn.x, sn.y, sn.z, sn.w};
      uint32_t wo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)  // round_T(round_T(x * cos) + round_T(rot(x) * sin)), all three packed
        wo[j] = Num<T>::add2(Num<T>::mul2(wx[j], wc[j]), Num<T>::mul2(wr[j] ^ flip, ws[j]));
      return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
  };

  // x <- round_T(round_T(x * r) * w) on one 128-bit word
  auto normalise = [](uint4 x, float r, uint4 w) {
    float f[V];
    Num<T>::unpack(x, f);
    if constexpr (sizeof(T) == 4) {
      float fw[V];
      Num<T>::unpack(w, fw);
#pragma unroll
      for (int j = 0; j < V; ++j) f[j] = __fmul_rn(__fmul_rn(f[j], r), fw[j]);
      return Num<T>::pack(f);
    } else {
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
      const Float2x r2 = pack_f2(r, r);
      uint32_t wo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float n0, n1;
        unpack_f2(mul_f2(pack_f2(f[2 * j], f[2 * j + 1]), r2), n0, n1);
        wo[j] = Num<T>::mul2(Num<T>::pack2(n0, n1), ww[j]);
      }
      return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
  };
  // two running sums of squares, two elements per instruction
  auto sum_squares = [](uint4 x, Float2x acc) {
    float f[V];
    Num<T>::unpack(x, f);
#pragma unroll
    for (int j = 0; j < V; j += 2) {
      const Float2x v = pack_f2(f[j], f[j + 1]);
      acc = fma_f2(v, v, acc);
    }
    return acc;
  };
  const float cols_f = static_cast<float>(p.head_dim);
  const float inv_cols = (p.head_dim & (p.head_dim - 1)) == 0 ? 1.0f / cols_f : 0.f;

  for (int ti = 0; ti < 2; ++ti) {
    const PairedTensor& t = p.t[ti];
    const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + unit * V;
    T* xout = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s + unit * V;
    uint4 w1 = {}, w2 = {};
    if constexpr (NORM) {
      if (t.heads > 0) {
        w1 = ld_reuse(static_cast<const T*>(p.weight[ti]) + unit * V);
        w2 = ld_reuse(static_cast<const T*>(p.weight[ti]) + unit * V + half);
      }
    }
    for (int h0 = 0; h0 < t.heads; h0 += UNROLL) {
      uint4 lo[UNROLL], hi[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (h0 + u < t.heads) {
          lo[u] = ld_stream(xin + (h0 + u) * t.xs_h);
          hi[u] = ld_stream(xin + (h0 + u) * t.xs_h + half);
        }
      }
      if constexpr (NORM) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (h0 + u < t.heads) {  // uniform over the CTA
            float a0, a1;
            unpack_f2(sum_squares(hi[u], sum_squares(lo[u], pack_f2(0.f, 0.f))), a0, a1);
            float acc = __fadd_rn(a0, a1);
            for (int o = upr >> 1; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
            const float r = inv_rms(acc, cols_f, inv_cols, p.eps);
            lo[u] = normalise(lo[u], r, w1);
            hi[u] = normalise(hi[u], r, w2);
          }
        }
        if (!active) continue;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (h0 + u < t.heads) {
          st_stream(xout + (h0 + u) * t.os_h, combine(lo[u], c1, hi[u], s1, true));
          st_stream(xout + (h0 + u) * t.os_h + half, combine(hi[u], c2, lo[u], s2, false));
        }
      }
    }
  }
}

// Any head_dim (even), any alignment.
template <typename T>
__global__ void __launch_bounds__(256) rope_paired_scalar_kernel(const PairedArgs p) {
  pdl_prologue();
  const int half = p.head_dim / 2;
  for (int ti = 0; ti < 2; ++ti) {
    const PairedTensor& t = p.t[ti];
    const int64_t total = static_cast<int64_t>(p.batch) * t.heads * p.seq * p.head_dim;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int j = static_cast<int>(i % p.head_dim);
      int64_t r = i / p.head_dim;
      const int64_t pos = r % p.seq;
      r /= p.seq;
      const int h = static_cast<int>(r % t.heads);
      const int64_t b = r / t.heads;
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + h * t.xs_h + pos * t.xs_s;
      const float x = Num<T>::up(xin[j]);
      const float rot = j < half ? -Num<T>::up(xin[j + half]) : Num<T>::up(xin[j - half]);
      const int64_t ci = b * p.cs_stride_b + pos * p.head_dim + j;
      const float c = Num<T>::up(static_cast<const T*>(p.cos)[ci]), sn = Num<T>::up(static_cast<const T*>(p.sin)[ci]);
      const float y = __fadd_rn(Num<T>::rt(__fmul_rn(x, c)), Num<T>::rt(__fmul_rn(rot, sn)));
      static_cast<T*>(t.out)[b * t.os_b + h * t.os_h + pos * t.os_s + j] = Num<T>::down(y);
    }
  }
}

// Fused norm + paired rope for any even head_dim and any alignment: one warp per (batch, head,
// position) row, two passes over the row (the second one served by L1/L2).
template <typename T>
__global__ void __launch_bounds__(256) norm_rope_scalar_kernel(const PairedArgs p) {
  pdl_prologue();
  const int half = p.head_dim / 2;
  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * 8;
  const float cols_f = static_cast<float>(p.head_dim);
  for (int ti = 0; ti < 2; ++ti) {
    const PairedTensor& t = p.t[ti];
    const T* weight = static_cast<const T*>(p.weight[ti]);
    const int64_t rows = static_cast<int64_t>(p.batch) * t.heads * p.seq;
    for (int64_t row = warp; row < rows; row += n_warps) {
      const int64_t pos = row % p.seq;
      const int h = static_cast<int>((row / p.seq) % t.heads);
      const int64_t b = row / p.seq / t.heads;
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + h * t.xs_h + pos * t.xs_s;
      T* xout = static_cast<T*>(t.out) + b * t.os_b + h * t.os_h + pos * t.os_s;
      float acc = 0.f;
      for (int j = lane; j < p.head_dim; j += 32) {
        const float v = Num<T>::up(xin[j]);
        acc = __fadd_rn(acc, __fmul_rn(v, v));
      }
      const float r = inv_rms(warp_sum(acc), cols_f, 0.f, p.eps);
      auto normed = [&](int j) {
        return Num<T>::rt(__fmul_rn(Num<T>::rt(__fmul_rn(Num<T>::up(xin[j]), r)), Num<T>::up(weight[j])));
      };
      const T* cos = static_cast<const T*>(p.cos) + b * p.cs_stride_b + pos * p.head_dim;
      const T* sin = static_cast<const T*>(p.sin) + b * p.cs_stride_b + pos * p.head_dim;
      // out may alias x: a lane reads both partners of its channels before any lane stores them,
      // because the loop below keeps the (j, j + half) pair in one lane
      for (int j = lane; j < half; j += 32) {
        const float a = normed(j), c = normed(j + half);
        const float y1 = __fadd_rn(Num<T>::rt(__fmul_rn(a, Num<T>::up(cos[j]))), Num<T>::rt(__fmul_rn(-c, Num<T>::up(sin[j]))));
        const float y2 = __fadd_rn(Num<T>::rt(__fmul_rn(c, Num<T>::up(cos[j + half]))), Num<T>::rt(__fmul_rn(a, Num<T>::up(sin[j + half]))));
        xout[j] = Num<T>::down(y1);
        xout[j + half] = Num<T>::down(y2);
      }
    }
  }
}

template <typename T, bool NORM>
int run_paired(const PairedArgs& p, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const int half = p.head_dim / 2;
  bool vec = half % V == 0 && half / V <= 256 && aligned(p.cos, 16) && aligned(p.sin, 16) && p.cs_stride_b % V == 0;
  if (NORM) {
    const int upr = half / V;
    vec = vec && upr <= 32 && (upr & (upr - 1)) == 0 && upr > 0;
    for (int i = 0; i < 2; ++i) vec = vec && (p.t[i].heads == 0 || aligned(p.weight[i], 16));
  }
  for (int i = 0; i < 2; ++i) {
    const PairedTensor& t = p.t[i];
    if (t.heads == 0) continue;
    vec = vec && aligned(t.x, 16) && aligned(t.out, 16) && t.xs_b % V == 0 && t.xs_h % V == 0 && t.xs_s % V == 0 &&
          t.os_b % V == 0 && t.os_h % V == 0 && t.os_s % V == 0;
  }
  if (vec) {
    const int tile_pos = 256 / (half / V);
    const int64_t grid = ceil_div(p.seq, tile_pos) * p.batch;
    if (grid > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "b200_rope_paired: problem too large for one launch");
    launch(rope_paired_kernel<T, NORM>, static_cast<unsigned>(grid), 256, 0, st, p);
    return after_launch("rope_paired_kernel");
  }
  if (NORM) {
    int64_t rows = 0;
    for (int i = 0; i < 2; ++i) rows += static_cast<int64_t>(p.batch) * p.t[i].heads * p.seq;
    const int64_t grid = std::min<int64_t>(ceil_div(rows, 8), static_cast<int64_t>(sm_count()) * 16);
    launch(norm_rope_scalar_kernel<T>, static_cast<unsigned>(grid), 256, 0, st, p);
    return after_launch("norm_rope_scalar_kernel");
  }
  launch(rope_paired_scalar_kernel<T>, static_cast<unsigned>(sm_count()) * 8, 256, 0, st, p);
  return after_launch("rope_paired_scalar_kernel");
}


// ------------------------------------------------------------ llama4 rope --
//
// llama4_rope(q, k, freqs) of the reference (src/popcorn/kernels/llama4_rope.py:14-39): layout
// (batch, seq, heads, head_dim), channels taken as (real, imaginary) pairs, freqs
// [seq, head_dim/2, 2] = (cos, sin) per pair in the dtype of q, arithmetic tensor by tensor in
// that dtype:
//   y_re = round_T(round_T(re * f_re) - round_T(im * f_im))
//   y_im = round_T(round_T(re * f_im) + round_T(im * f_re))
struct Llama4Tensor {
  const void* x;
  void* out;
  int64_t xs_b, xs_s, xs_h;
  int64_t os_b, os_s, os_h;
  int heads;
};
struct Llama4Args {
  Llama4Tensor t[2];
  const void* freqs;
  int64_t seq;
  int batch;
  int head_dim;
};

// A 128-bit word of x lines up with the 128-bit word of the freqs row at the same offset (both
// hold whole pairs).  A thread owns one (position, word): the freqs word stays in registers
// while it walks over the batch entries of its CTA and all heads of q and k.
template <typename T>
__global__ void __launch_bounds__(256) llama4_rope_kernel(const Llama4Args p, const int batch_per_cta) {
  constexpr int V = Num<T>::kVec;
  constexpr int UNROLL = 8;
  pdl_prologue();
  const int wpr = p.head_dim / V;  // words per row
  const int tile_pos = 256 / wpr;
  const int64_t tiles = (p.seq + tile_pos - 1) / tile_pos;
  const int64_t tile = blockIdx.x % tiles;
  const int b0 = static_cast<int>(blockIdx.x / tiles) * batch_per_cta;
  const int word = threadIdx.x % wpr;
  const int64_t pos = tile * tile_pos + threadIdx.x / wpr;
  if (threadIdx.x / wpr >= tile_pos || pos >= p.seq) return;

  const uint4 f = ld_reuse(static_cast<const T*>(p.freqs) + pos * p.head_dim + word * V);
  // 16-bit types: (-f_im, f_re) per pair, so that the whole rotation is two packed products and one packed sum
  //   (re, re) * (f_re, f_im) + (im, im) * (-f_im, f_re) = (re*f_re - im*f_im, re*f_im + im*f_re)
  // (negating an operand negates the rounded product exactly)
  uint32_t fs[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) fs[j] = __byte_perm(fs[j], 0, 0x1032) ^ 0x00008000u;

  auto rotate = [&f, &fs](uint4 x) {
    if constexpr (sizeof(T) == 4) {
      float v[4], w[4];
      Num<T>::unpack(x, v);
      Num<T>::unpack(f, w);
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        o[j] = __fsub_rn(__fmul_rn(v[j], w[j]), __fmul_rn(v[j + 1], w[j + 1]));
        o[j + 1] = __fadd_rn(__fmul_rn(v[j], w[j + 1]), __fmul_rn(v[j + 1], w[j]));
      }
      return Num<T>::pack(o);
    } else {
      const uint32_t wx[4] = {x.x, x.y, x.z, x.w}, wf[4] = {f.x, f.y, f.z, f.w};
      uint32_t wo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        wo[j] = Num<T>::add2(Num<T>::mul2(__byte_perm(wx[j], 0, 0x1010), wf[j]), Num<T>::mul2(__byte_perm(wx[j], 0, 0x3232), fs[j]));
      return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
  };

  const int b1 = min(b0 + batch_per_cta, p.batch);
  for (int b = b0; b < b1; ++b) {
    for (int ti = 0; ti < 2; ++ti) {
      const Llama4Tensor& t = p.t[ti];
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + word * V;
      T* xout = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s + word * V;
      for (int h0 = 0; h0 < t.heads; h0 += UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (h0 + u < t.heads) v[u] = ld_stream(xin + (h0 + u) * t.xs_h);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (h0 + u < t.heads) st_stream(xout + (h0 + u) * t.os_h, rotate(v[u]));
      }
    }
  }
}

// Any even head_dim, any alignment: one thread per pair.
template <typename T>
__global__ void __launch_bounds__(256) llama4_rope_scalar_kernel(const Llama4Args p) {
  pdl_prologue();
  const int half = p.head_dim / 2;
  for (int ti = 0; ti < 2; ++ti) {
    const Llama4Tensor& t = p.t[ti];
    const int64_t total = static_cast<int64_t>(p.batch) * p.seq * t.heads * half;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int j = static_cast<int>(i % half);
      int64_t r = i / half;
      const int h = static_cast<int>(r % t.heads);
      r /= t.heads;
      const int64_t pos = r % p.seq;
      const int64_t b = r / p.seq;
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + h * t.xs_h + 2 * j;
      T* xout = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s + h * t.os_h + 2 * j;
      const T* fr = static_cast<const T*>(p.freqs) + pos * p.head_dim + 2 * j;
      const float re = Num<T>::up(xin[0]), im = Num<T>::up(xin[1]);
      const float f_re = Num<T>::up(fr[0]), f_im = Num<T>::up(fr[1]);
      const float y_re = __fsub_rn(Num<T>::rt(__fmul_rn(re, f_re)), Num<T>::rt(__fmul_rn(im, f_im)));
      const float y_im = __fadd_rn(Num<T>::rt(__fmul_rn(re, f_im)), Num<T>::rt(__fmul_rn(im, f_re)));
      xout[0] = Num<T>::down(y_re);
      xout[1] = Num<T>::down(y_im);
    }
  }
}

template <typename T>
int run_llama4(const Llama4Args& p, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  bool vec = p.head_dim % V == 0 && p.head_dim / V <= 256 && aligned(p.freqs, 16);
  for (int i = 0; i < 2; ++i) {
    const Llama4Tensor& t = p.t[i];
    if (t.heads == 0) continue;
    vec = vec && aligned(t.x, 16) && aligned(t.out, 16) && t.xs_b % V == 0 && t.xs_s % V == 0 && t.xs_h % V == 0 &&
          t.os_b % V == 0 && t.os_s % V == 0 && t.os_h % V == 0;
  }
  if (vec) {
    const int tile_pos = 256 / (p.head_dim / V);
    const int64_t tiles = ceil_div(p.seq, tile_pos);
    // one CTA per (tile, batch entry) unless that is far more CTAs than the machine needs
    const int64_t want = static_cast<int64_t>(sm_count()) * 32;
    int per_cta = 1;
    while (tiles * ceil_div(p.batch, per_cta) > want && per_cta < p.batch) per_cta *= 2;
    const int64_t grid = tiles * ceil_div(p.batch, per_cta);
    if (grid > 0x7fffffffLL) return fail(B200_ERR_SHAPE, "b200_llama4_rope: problem too large for one launch");
    launch(llama4_rope_kernel<T>, static_cast<unsigned>(grid), 256, 0, st, p, per_cta);
    return after_launch("llama4_rope_kernel");
  }
  launch(llama4_rope_scalar_kernel<T>, static_cast<unsigned>(sm_count()) * 8, 256, 0, st, p);
  return after_launch("llama4_rope_scalar_kernel");
}


// ------------------------------------------------- qk_norm_rope backward --
//
// What autograd derives from the fused op's reference (examples/03_write_a_kernel.ipynb, cell 3; the
// notebook's own hand-written backward is cells 8-9), per head row x with n = round_T(x r), r = 1/rms(x):
//   g   = transpose of the rotation applied to dy, in T:  g1 = dy1 c1 + dy2 s2,  g2 = dy2 c2 - dy1 s1
//   dw += round_T(g * n)                       (summed over every row of the tensor)
//   u   = round_T(g * w),  dx = round_T(u r - x r^3 <u, x> / head_dim)      (fp32 inside)
// r is recomputed from x (no saved statistics).  Thread mapping as in rope_paired_kernel; the per-thread
// column sums of dw are reduced over the positions of a warp by shuffles, over the warps of the CTA through
// shared memory, and written to this CTA's line of `partial` ([gridDim.x][2][head_dim] fp32), which
// sum_lines_kernel adds up.
struct NormRopeBwdArgs {
  PairedArgs fwd;        // q / k (inputs of the forward), tables, weights, eps; t[i].out = grad of the input
  const void* dy[2];     // gradients of the outputs, contiguous [batch, heads, seq, head_dim]
};

template <typename T>
__global__ void __launch_bounds__(256, 2) norm_rope_bwd_kernel(const NormRopeBwdArgs a, float* __restrict__ partial) {
  constexpr int V = Num<T>::kVec;
  const PairedArgs& p = a.fwd;
  pdl_prologue();
  __shared__ float red[8][32 * 2 * 8];  // [warp][unit][lo|hi][element]: at most 32 units of 2 x 8 columns
  const int half = p.head_dim / 2;
  const int upr = half / V;  // units per row: a power of two <= 32 on this path
  const int tile_pos = 256 / upr;
  const int64_t tiles = (p.seq + tile_pos - 1) / tile_pos;
  const int64_t tile = blockIdx.x % tiles;
  const int b = static_cast<int>(blockIdx.x / tiles);
  const int unit = threadIdx.x % upr, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t pos = tile * tile_pos + threadIdx.x / upr;
  const bool active = pos < p.seq;
  if (!active) pos = p.seq - 1;  // keeps the shuffles full-width; contributes nothing
  const float cols_f = static_cast<float>(p.head_dim);
  const float inv_cols = (p.head_dim & (p.head_dim - 1)) == 0 ? 1.0f / cols_f : 0.f;

  const T* cos = static_cast<const T*>(p.cos) + b * p.cs_stride_b + pos * p.head_dim + unit * V;
  const T* sin = static_cast<const T*>(p.sin) + b * p.cs_stride_b + pos * p.head_dim + unit * V;
  const uint4 c1w = ld_reuse(cos), c2w = ld_reuse(cos + half), s1w = ld_reuse(sin), s2w = ld_reuse(sin + half);

  // g = round_T(round_T(d * c) + round_T(+-e * s)) on one 128-bit word: the transpose of the rotation, in T
  auto rotate_back = [](uint4 d, uint4 c, uint4 e, uint4 sn, bool negate_e) {
    if constexpr (sizeof(T) == 4) {
      float fd[4], fc[4], fe[4], fs[4];
      Num<T>::unpack(d, fd);
      Num<T>::unpack(c, fc);
      Num<T>::unpack(e, fe);
      Num<T>::unpack(sn, fs);
#pragma unroll
      for (int j = 0; j < 4; ++j) fd[j] = __fadd_rn(__fmul_rn(fd[j], fc[j]), __fmul_rn(negate_e ? -fe[j] : fe[j], fs[j]));
      return Num<T>::pack(fd);
    } else {
      const uint32_t flip = negate_e ? 0x80008000u : 0u;
      const uint32_t wd[4] = {d.x, d.y, d.z, d.w}, wc[4] = {c.x, c.y, c.z, c.w};
      const uint32_t we[4] = {e.x, e.y, e.z, e.w}, ws[4] = {sn.x, sn.y, sn.z, sn.w};
      uint32_t wo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wo[j] = Num<T>::add2(Num<T>::mul2(wd[j], wc[j]), Num<T>::mul2(we[j] ^ flip, ws[j]));
      return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
  };
  // One half row (a 128-bit word x, the matching word g of the rotated-back gradient, the weight word w):
  // adds round_T(g * round_T(x r)) to the column sums, leaves u = round_T(g * w) and x as fp32 pairs and returns the
  // two partial sums of <u, x>.  fp32 arithmetic two elements per instruction, every element rounded on its own.
  constexpr int P = V / 2;
  auto half_row = [](uint4 xw, uint4 gw, uint4 ww, Float2x r2, bool active, Float2x (&acc)[P], Float2x (&x)[P], Float2x (&u)[P], Float2x dot) {
    float fx[V];
    Num<T>::unpack(xw, fx);
#pragma unroll
    for (int j = 0; j < P; ++j) x[j] = pack_f2(fx[2 * j], fx[2 * j + 1]);
    if constexpr (sizeof(T) == 4) {
      float g[V], w[V];
      Num<T>::unpack(gw, g);
      Num<T>::unpack(ww, w);
#pragma unroll
      for (int j = 0; j < P; ++j) {
        const Float2x g2 = pack_f2(g[2 * j], g[2 * j + 1]);
        const Float2x term = mul_f2(g2, mul_f2(x[j], r2));
        float t0, t1, a0, a1;
        unpack_f2(term, t0, t1);
        unpack_f2(acc[j], a0, a1);
        if (active) acc[j] = pack_f2(__fadd_rn(a0, t0), __fadd_rn(a1, t1));  // separate product and sum, as in the reference
        u[j] = mul_f2(g2, pack_f2(w[2 * j], w[2 * j + 1]));
        dot = fma_f2(u[j], x[j], dot);
      }
    } else {
      const uint32_t wg[4] = {gw.x, gw.y, gw.z, gw.w}, wwt[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float n0, n1, a0, a1, u0, u1;
        unpack_f2(mul_f2(x[j], r2), n0, n1);
        Num<T>::unpack2(Num<T>::mul2(wg[j], Num<T>::pack2(n0, n1)), a0, a1);
        if (active) acc[j] = add_f2(acc[j], pack_f2(a0, a1));
        Num<T>::unpack2(Num<T>::mul2(wg[j], wwt[j]), u0, u1);
        u[j] = pack_f2(u0, u1);
        dot = fma_f2(u[j], x[j], dot);
      }
    }
    return dot;
  };

  constexpr int UNROLL = 2;  // heads in flight per thread
  for (int ti = 0; ti < 2; ++ti) {
    const PairedTensor& t = p.t[ti];
    Float2x acc_lo2[P], acc_hi2[P];
#pragma unroll
    for (int j = 0; j < P; ++j) acc_lo2[j] = acc_hi2[j] = pack_f2(0.f, 0.f);
    if (t.heads > 0) {
      const uint4 w1 = ld_reuse(static_cast<const T*>(p.weight[ti]) + unit * V);
      const uint4 w2 = ld_reuse(static_cast<const T*>(p.weight[ti]) + unit * V + half);
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + pos * t.xs_s + unit * V;
      T* dx = static_cast<T*>(t.out) + b * t.os_b + pos * t.os_s + unit * V;
      const T* dy = static_cast<const T*>(a.dy[ti]) + (static_cast<int64_t>(b) * t.heads * p.seq + pos) * p.head_dim + unit * V;
      const int64_t dy_h = static_cast<int64_t>(p.seq) * p.head_dim;
      for (int h0 = 0; h0 < t.heads; h0 += UNROLL) {
        uint4 x_lo[UNROLL], x_hi[UNROLL], d_lo[UNROLL], d_hi[UNROLL];
#pragma unroll
        for (int q = 0; q < UNROLL; ++q) {
          if (h0 + q < t.heads) {
            x_lo[q] = ld_stream(xin + (h0 + q) * t.xs_h);
            x_hi[q] = ld_stream(xin + (h0 + q) * t.xs_h + half);
            d_lo[q] = ld_stream(dy + (h0 + q) * dy_h);
            d_hi[q] = ld_stream(dy + (h0 + q) * dy_h + half);
          }
        }
#pragma unroll
        for (int q = 0; q < UNROLL; ++q) {
          if (h0 + q < t.heads) {  // uniform over the CTA
            Float2x x1[P], x2[P], u1[P], u2[P];
            float ss;
            {
              float f1[V], f2[V];
              Num<T>::unpack(x_lo[q], f1);
              Num<T>::unpack(x_hi[q], f2);
              Float2x ss2 = pack_f2(0.f, 0.f);
#pragma unroll
              for (int j = 0; j < P; ++j) {
                const Float2x p1 = pack_f2(f1[2 * j], f1[2 * j + 1]), p2 = pack_f2(f2[2 * j], f2[2 * j + 1]);
                ss2 = fma_f2(p2, p2, fma_f2(p1, p1, ss2));
              }
              float s0, s1;
              unpack_f2(ss2, s0, s1);
              ss = __fadd_rn(s0, s1);
            }
            for (int o = upr >> 1; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
            const float r = inv_rms(ss, cols_f, inv_cols, p.eps);
            const Float2x r2 = pack_f2(r, r);
            const uint4 g1 = rotate_back(d_lo[q], c1w, d_hi[q], s2w, false);  // g1 = dy1 c1 + dy2 s2
            const uint4 g2 = rotate_back(d_hi[q], c2w, d_lo[q], s1w, true);   // g2 = dy2 c2 - dy1 s1
            Float2x dot2 = half_row(x_lo[q], g1, w1, r2, active, acc_lo2, x1, u1, pack_f2(0.f, 0.f));
            dot2 = half_row(x_hi[q], g2, w2, r2, active, acc_hi2, x2, u2, dot2);
            float dot, dot_hi;
            unpack_f2(dot2, dot, dot_hi);
            dot = __fadd_rn(dot, dot_hi);
            for (int o = upr >> 1; o > 0; o >>= 1) dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, o));
            const float dot_over_n = inv_cols > 0.f ? __fmul_rn(dot, inv_cols) : __fdiv_rn(dot, cols_f);
            const float coef = -__fmul_rn(__fmul_rn(__fmul_rn(r, r), r), dot_over_n);
            const Float2x coef2 = pack_f2(coef, coef);
            float o1[V], o2[V];
#pragma unroll
            for (int j = 0; j < P; ++j) {
              unpack_f2(fma_f2(u1[j], r2, mul_f2(x1[j], coef2)), o1[2 * j], o1[2 * j + 1]);
              unpack_f2(fma_f2(u2[j], r2, mul_f2(x2[j], coef2)), o2[2 * j], o2[2 * j + 1]);
            }
            if (active) {
              st_stream(dx + (h0 + q) * t.os_h, Num<T>::pack(o1));
              st_stream(dx + (h0 + q) * t.os_h + half, Num<T>::pack(o2));
            }
          }
        }
      }
    }
    float acc_lo[V], acc_hi[V];
#pragma unroll
    for (int j = 0; j < P; ++j) {
      unpack_f2(acc_lo2[j], acc_lo[2 * j], acc_lo[2 * j + 1]);
      unpack_f2(acc_hi2[j], acc_hi[2 * j], acc_hi[2 * j + 1]);
    }
    // column sums of this CTA: lanes with the same unit sit `upr` apart inside a warp
#pragma unroll
    for (int j = 0; j < V; ++j) {
      for (int o = upr; o < 32; o <<= 1) {
        acc_lo[j] = __fadd_rn(acc_lo[j], __shfl_xor_sync(0xffffffffu, acc_lo[j], o));
        acc_hi[j] = __fadd_rn(acc_hi[j], __shfl_xor_sync(0xffffffffu, acc_hi[j], o));
      }
    }
    __syncthreads();  // `red` is free again (second tensor)
    if (lane < upr) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        red[warp][(unit * 2 + 0) * 8 + j] = acc_lo[j];
        red[warp][(unit * 2 + 1) * 8 + j] = acc_hi[j];
      }
    }
    __syncthreads();
    // when a position group spans several warps' worth of lanes (upr = 32) every warp holds other units' sums too:
    // with upr <= 32 and 256 threads each warp covers 32 / upr positions of all units, so the eight warps add up
    for (int idx = threadIdx.x; idx < upr * 2 * V; idx += 256) {
      const int u = idx / (2 * V), part = (idx / V) & 1, j = idx % V;
      float total = 0.f;
#pragma unroll
      for (int wv = 0; wv < 8; ++wv) total = __fadd_rn(total, red[wv][(u * 2 + part) * 8 + j]);
      partial[(static_cast<int64_t>(blockIdx.x) * 2 + ti) * p.head_dim + part * half + u * V + j] = total;
    }
  }
}

// out[ti][c] = round_T(sum over lines of partial[line][ti][c]), lines added in order.
template <typename T>
__global__ void __launch_bounds__(1024) sum_lines_kernel(const float* __restrict__ partial, int lines, int head_dim, T* __restrict__ dw0, T* __restrict__ dw1) {
  // A CTA owns 32 of the 2 x head_dim columns; each of its 32 warps adds every 32nd line (one 128-byte segment per
  // load), then the 32 partial sums are added in warp order: the result does not depend on timing.
  pdl_prologue();
  __shared__ float part[32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int idx = blockIdx.x * 32 + lane;
  const bool in_range = idx < 2 * head_dim;
  const int ti = in_range ? idx / head_dim : 0, c = in_range ? idx % head_dim : 0;
  float acc = 0.f;
  if (in_range)
    for (int l = warp; l < lines; l += 32) acc = __fadd_rn(acc, partial[(static_cast<int64_t>(l) * 2 + ti) * head_dim + c]);
  part[warp][lane] = acc;
  __syncthreads();
  T* out = ti == 0 ? dw0 : dw1;
  if (warp == 0 && in_range && out != nullptr) {
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) total = __fadd_rn(total, part[k][lane]);
    out[c] = Num<T>::down(total);
  }
}

// Any even head_dim, any alignment: one warp per (batch, head, position) row, column sums by atomic adds into
// line 0 of `partial` (zeroed by the caller).
template <typename T>
__global__ void __launch_bounds__(256) norm_rope_bwd_scalar_kernel(const NormRopeBwdArgs a, float* __restrict__ partial) {
  const PairedArgs& p = a.fwd;
  pdl_prologue();
  const int half = p.head_dim / 2;
  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * 8;
  const float cols_f = static_cast<float>(p.head_dim);
  for (int ti = 0; ti < 2; ++ti) {
    const PairedTensor& t = p.t[ti];
    const T* weight = static_cast<const T*>(p.weight[ti]);
    const int64_t rows = static_cast<int64_t>(p.batch) * t.heads * p.seq;
    for (int64_t row = warp; row < rows; row += n_warps) {
      const int64_t pos = row % p.seq;
      const int h = static_cast<int>((row / p.seq) % t.heads);
      const int64_t b = row / p.seq / t.heads;
      const T* xin = static_cast<const T*>(t.x) + b * t.xs_b + h * t.xs_h + pos * t.xs_s;
      T* dx = static_cast<T*>(t.out) + b * t.os_b + h * t.os_h + pos * t.os_s;
      const T* dy = static_cast<const T*>(a.dy[ti]) + row * p.head_dim;
      const T* cos = static_cast<const T*>(p.cos) + b * p.cs_stride_b + pos * p.head_dim;
      const T* sin = static_cast<const T*>(p.sin) + b * p.cs_stride_b + pos * p.head_dim;
      float ss = 0.f;
      for (int j = lane; j < p.head_dim; j += 32) {
        const float v = Num<T>::up(xin[j]);
        ss = __fmaf_rn(v, v, ss);
      }
      const float r = inv_rms(warp_sum(ss), cols_f, 0.f, p.eps);
      auto g_of = [&](int j) {  // transpose of the rotation at column j
        if (j < half)
          return Num<T>::rt(__fadd_rn(Num<T>::rt(__fmul_rn(Num<T>::up(dy[j]), Num<T>::up(cos[j]))),
                                      Num<T>::rt(__fmul_rn(Num<T>::up(dy[j + half]), Num<T>::up(sin[j + half])))));
        return Num<T>::rt(__fsub_rn(Num<T>::rt(__fmul_rn(Num<T>::up(dy[j]), Num<T>::up(cos[j]))),
                                    Num<T>::rt(__fmul_rn(Num<T>::up(dy[j - half]), Num<T>::up(sin[j - half])))));
      };
      float dot = 0.f;
      for (int j = lane; j < p.head_dim; j += 32) {
        const float x = Num<T>::up(xin[j]), g = g_of(j);
        atomicAdd(&partial[ti * p.head_dim + j], Num<T>::rt(__fmul_rn(g, Num<T>::rt(__fmul_rn(x, r)))));
        dot = __fmaf_rn(Num<T>::rt(__fmul_rn(g, Num<T>::up(weight[j]))), x, dot);
      }
      dot = warp_sum(dot);
      const float coef = -__fmul_rn(__fmul_rn(__fmul_rn(r, r), r), __fdiv_rn(dot, cols_f));
      for (int j = lane; j < p.head_dim; j += 32) {
        const float x = Num<T>::up(xin[j]);
        const float u = Num<T>::rt(__fmul_rn(g_of(j), Num<T>::up(weight[j])));
        dx[j] = Num<T>::down(__fmaf_rn(u, r, __fmul_rn(x, coef)));
      }
    }
  }
}

int norm_rope_bwd_lines(int64_t batch, int64_t seq, int64_t head_dim, int elem_size) {
  const int v = 16 / elem_size, half = static_cast<int>(head_dim / 2);
  if (half % v != 0) return 1;
  const int upr = half / v;
  if (upr <= 0 || upr > 32 || (upr & (upr - 1)) != 0) return 1;
  const int64_t lines = ceil_div(seq, 256 / upr) * batch;
  return lines > 0x7fffffffLL ? 1 : static_cast<int>(lines);
}

template <typename T>
int run_norm_rope_bwd(const NormRopeBwdArgs& a, void* dw0, void* dw1, float* scratch, cudaStream_t st) {
  constexpr int V = Num<T>::kVec;
  const PairedArgs& p = a.fwd;
  const int half = p.head_dim / 2;
  const int upr = half % V == 0 ? half / V : 0;
  bool vec = upr > 0 && upr <= 32 && (upr & (upr - 1)) == 0 && aligned(p.cos, 16) && aligned(p.sin, 16) && p.cs_stride_b % V == 0;
  for (int i = 0; i < 2; ++i) {
    const PairedTensor& t = p.t[i];
    if (t.heads == 0) continue;
    vec = vec && aligned(t.x, 16) && aligned(t.out, 16) && aligned(a.dy[i], 16) && aligned(p.weight[i], 16) && t.xs_b % V == 0 &&
          t.xs_h % V == 0 && t.xs_s % V == 0 && t.os_b % V == 0 && t.os_h % V == 0 && t.os_s % V == 0;
  }
  int lines = 1;
  if (vec) {
    lines = norm_rope_bwd_lines(p.batch, p.seq, p.head_dim, sizeof(T));
    launch(norm_rope_bwd_kernel<T>, static_cast<unsigned>(lines), 256, 0, st, a, scratch);
    if (int rc = after_launch("norm_rope_bwd_kernel")) return rc;
  } else {
    if (cudaMemsetAsync(scratch, 0, sizeof(float) * 2 * p.head_dim, st) != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(B200_ERR_LAUNCH, "b200_qk_norm_rope_backward: cannot clear the scratch buffer");
    }
    int64_t rows = 0;
    for (int i = 0; i < 2; ++i) rows += static_cast<int64_t>(p.batch) * p.t[i].heads * p.seq;
    const int64_t grid = std::max<int64_t>(1, std::min<int64_t>(ceil_div(rows, 8), static_cast<int64_t>(sm_count()) * 16));
    launch(norm_rope_bwd_scalar_kernel<T>, static_cast<unsigned>(grid), 256, 0, st, a, scratch);
    if (int rc = after_launch("norm_rope_bwd_scalar_kernel")) return rc;
  }
  launch(sum_lines_kernel<T>, static_cast<unsigned>(ceil_div(2 * p.head_dim, 32)), 1024, 0, st, static_cast<const float*>(scratch), lines,
         p.head_dim, static_cast<T*>(dw0), static_cast<T*>(dw1));
  return after_launch("sum_lines_kernel");
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

namespace {

int paired_common(const char* fn, bool norm, const void* q, const void* k, const void* q_weight, const void* k_weight,
                  const void* cos, const void* sin, void* q_out, void* k_out,
                  int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                  const int64_t (&qs)[3], const int64_t (&ks)[3], const int64_t (&qos)[3], const int64_t (&kos)[3],
                  float eps, int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", fn, dtype);
  if (batch < 0 || q_heads < 0 || k_heads < 0 || seq < 0 || head_dim < 0) return fail(B200_ERR_SHAPE, "%s: negative size", fn);
  if (head_dim % 2 != 0) return fail(B200_ERR_SHAPE, "%s: head_dim=%lld must be even", fn, (long long)head_dim);
  if (cos_batch != 1 && cos_batch != batch) return fail(B200_ERR_SHAPE, "%s: cos_batch must be 1 or batch", fn);
  if (batch > 0x7fffffffLL || q_heads > (1 << 20) || k_heads > (1 << 20) || head_dim > (1 << 20))
    return fail(B200_ERR_SHAPE, "%s: size out of range", fn);
  if (batch == 0 || seq == 0 || head_dim == 0 || (q_heads == 0 && k_heads == 0)) return B200_OK;
  const size_t es = dtype_size(dtype);
  if (q_heads > 0) {
    if (q == nullptr || q_out == nullptr || (norm && q_weight == nullptr)) return fail(B200_ERR_NULL_POINTER, "%s: q, q_out or q_weight is NULL", fn);
  }
  if (k_heads > 0) {
    if (k == nullptr || k_out == nullptr || (norm && k_weight == nullptr)) return fail(B200_ERR_NULL_POINTER, "%s: k, k_out or k_weight is NULL", fn);
  }
  if (cos == nullptr || sin == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: cos or sin is NULL", fn);
  if (!aligned(q, es) || !aligned(k, es) || !aligned(q_out, es) || !aligned(k_out, es) || !aligned(cos, es) || !aligned(sin, es) ||
      !aligned(q_weight, es) || !aligned(k_weight, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", fn);
  if (int rc = check_device()) return rc;
  PairedArgs p{};
  p.t[0] = PairedTensor{q, q_out, qs[0], qs[1], qs[2], qos[0], qos[1], qos[2], static_cast<int>(q_heads)};
  p.t[1] = PairedTensor{k, k_out, ks[0], ks[1], ks[2], kos[0], kos[1], kos[2], static_cast<int>(k_heads)};
  p.cos = cos;
  p.sin = sin;
  p.cs_stride_b = cos_batch == 1 ? 0 : seq * head_dim;
  p.seq = seq;
  p.batch = static_cast<int>(batch);
  p.head_dim = static_cast<int>(head_dim);
  p.weight[0] = q_weight;
  p.weight[1] = k_weight;
  p.eps = eps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (norm) {
    B200_DISPATCH_DTYPE(dtype, T, return (run_paired<T, true>(p, st)));
  } else {
    B200_DISPATCH_DTYPE(dtype, T, return (run_paired<T, false>(p, st)));
  }
  return B200_OK;
}

}  // namespace

extern "C" int b200_rope_paired(const void* q, const void* k, const void* cos, const void* sin, void* q_out, void* k_out,
                                int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                                int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                int64_t qo_stride_b, int64_t qo_stride_h, int64_t qo_stride_s,
                                int64_t ko_stride_b, int64_t ko_stride_h, int64_t ko_stride_s,
                                int dtype, void* stream) {
  const int64_t qs[3] = {q_stride_b, q_stride_h, q_stride_s}, ks[3] = {k_stride_b, k_stride_h, k_stride_s};
  const int64_t qos[3] = {qo_stride_b, qo_stride_h, qo_stride_s}, kos[3] = {ko_stride_b, ko_stride_h, ko_stride_s};
  return paired_common(__func__, false, q, k, nullptr, nullptr, cos, sin, q_out, k_out, batch, q_heads, k_heads, seq, head_dim,
                       cos_batch, qs, ks, qos, kos, 0.f, dtype, stream);
}

extern "C" int b200_qk_norm_rope(const void* q, const void* k, const void* q_weight, const void* k_weight,
                                 const void* cos, const void* sin, void* q_out, void* k_out,
                                 int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                                 int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                 int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                 int64_t qo_stride_b, int64_t qo_stride_h, int64_t qo_stride_s,
                                 int64_t ko_stride_b, int64_t ko_stride_h, int64_t ko_stride_s,
                                 double eps, int dtype, void* stream) {
  const int64_t qs[3] = {q_stride_b, q_stride_h, q_stride_s}, ks[3] = {k_stride_b, k_stride_h, k_stride_s};
  const int64_t qos[3] = {qo_stride_b, qo_stride_h, qo_stride_s}, kos[3] = {ko_stride_b, ko_stride_h, ko_stride_s};
  return paired_common(__func__, true, q, k, q_weight, k_weight, cos, sin, q_out, k_out, batch, q_heads, k_heads, seq, head_dim,
                       cos_batch, qs, ks, qos, kos, static_cast<float>(eps), dtype, stream);
}

extern "C" int b200_llama4_rope(const void* q, const void* k, const void* freqs, void* q_out, void* k_out,
                                int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim,
                                int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                                int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                                int64_t qo_stride_b, int64_t qo_stride_s, int64_t qo_stride_h,
                                int64_t ko_stride_b, int64_t ko_stride_s, int64_t ko_stride_h,
                                int dtype, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", __func__, dtype);
  if (batch < 0 || q_heads < 0 || k_heads < 0 || seq < 0 || head_dim < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (head_dim % 2 != 0) return fail(B200_ERR_SHAPE, "%s: head_dim=%lld must be even", __func__, (long long)head_dim);
  if (batch > 0x7fffffffLL || q_heads > (1 << 20) || k_heads > (1 << 20) || head_dim > (1 << 20))
    return fail(B200_ERR_SHAPE, "%s: size out of range", __func__);
  if (batch == 0 || seq == 0 || head_dim == 0 || (q_heads == 0 && k_heads == 0)) return B200_OK;
  if (q_heads > 0) {
    B200_REQUIRE_PTR(q);
    B200_REQUIRE_PTR(q_out);
  }
  if (k_heads > 0) {
    B200_REQUIRE_PTR(k);
    B200_REQUIRE_PTR(k_out);
  }
  B200_REQUIRE_PTR(freqs);
  const size_t es = dtype_size(dtype);
  if (!aligned(q, es) || !aligned(k, es) || !aligned(q_out, es) || !aligned(k_out, es) || !aligned(freqs, es))
    return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  Llama4Args p{};
  p.t[0] = Llama4Tensor{q, q_out, q_stride_b, q_stride_s, q_stride_h, qo_stride_b, qo_stride_s, qo_stride_h, static_cast<int>(q_heads)};
  p.t[1] = Llama4Tensor{k, k_out, k_stride_b, k_stride_s, k_stride_h, ko_stride_b, ko_stride_s, ko_stride_h, static_cast<int>(k_heads)};
  p.freqs = freqs;
  p.seq = seq;
  p.batch = static_cast<int>(batch);
  p.head_dim = static_cast<int>(head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_DTYPE(dtype, T, return run_llama4<T>(p, st));
  return B200_OK;
}

extern "C" int b200_qk_norm_rope_backward_scratch_bytes(int64_t batch, int64_t seq, int64_t head_dim, int dtype, size_t* bytes) {
  B200_REQUIRE_PTR(bytes);
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", __func__, dtype);
  if (batch < 0 || seq < 0 || head_dim < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  const int lines = norm_rope_bwd_lines(batch, seq, head_dim, static_cast<int>(dtype_size(dtype)));
  *bytes = static_cast<size_t>(lines > 0 ? lines : 1) * 2 * static_cast<size_t>(head_dim > 0 ? head_dim : 1) * sizeof(float);
  return B200_OK;
}

extern "C" int b200_qk_norm_rope_backward(const void* grad_q_out, const void* grad_k_out, const void* q, const void* k,
                                          const void* q_weight, const void* k_weight, const void* cos, const void* sin,
                                          void* grad_q, void* grad_k, void* grad_q_weight, void* grad_k_weight,
                                          int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                                          int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                          int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                          double eps, int dtype, void* scratch, size_t scratch_bytes, void* stream) {
  if (!dtype_ok(dtype)) return fail(B200_ERR_DTYPE, "%s: unsupported dtype %d", __func__, dtype);
  if (batch < 0 || q_heads < 0 || k_heads < 0 || seq < 0 || head_dim < 0) return fail(B200_ERR_SHAPE, "%s: negative size", __func__);
  if (head_dim % 2 != 0) return fail(B200_ERR_SHAPE, "%s: head_dim=%lld must be even", __func__, (long long)head_dim);
  if (cos_batch != 1 && cos_batch != batch) return fail(B200_ERR_SHAPE, "%s: cos_batch must be 1 or batch", __func__);
  if (batch > 0x7fffffffLL || q_heads > (1 << 20) || k_heads > (1 << 20) || head_dim > (1 << 20))
    return fail(B200_ERR_SHAPE, "%s: size out of range", __func__);
  if (head_dim == 0) return B200_OK;
  if (scratch == nullptr) return fail(B200_ERR_NULL_POINTER, "%s: scratch is NULL", __func__);
  if (q_heads > 0 && (grad_q_out == nullptr || q == nullptr || q_weight == nullptr || grad_q == nullptr || grad_q_weight == nullptr))
    return fail(B200_ERR_NULL_POINTER, "%s: a query pointer is NULL", __func__);
  if (k_heads > 0 && (grad_k_out == nullptr || k == nullptr || k_weight == nullptr || grad_k == nullptr || grad_k_weight == nullptr))
    return fail(B200_ERR_NULL_POINTER, "%s: a key pointer is NULL", __func__);
  if ((q_heads > 0 || k_heads > 0) && batch > 0 && seq > 0 && (cos == nullptr || sin == nullptr))
    return fail(B200_ERR_NULL_POINTER, "%s: cos or sin is NULL", __func__);
  const size_t es = dtype_size(dtype);
  for (const void* ptr : {grad_q_out, grad_k_out, q, k, q_weight, k_weight, cos, sin, static_cast<const void*>(grad_q),
                          static_cast<const void*>(grad_k), static_cast<const void*>(grad_q_weight), static_cast<const void*>(grad_k_weight)})
    if (!aligned(ptr, es)) return fail(B200_ERR_ALIGNMENT, "%s: pointer not aligned to the element size", __func__);
  if (int rc = check_device()) return rc;
  const size_t need = static_cast<size_t>(norm_rope_bwd_lines(batch, seq, head_dim, static_cast<int>(es))) * 2 * head_dim * sizeof(float);
  if (scratch_bytes < need || !aligned(scratch, 16))
    return fail(B200_ERR_SCRATCH, "%s: scratch needs %zu bytes, 16-byte aligned (got %zu)", __func__, need, scratch_bytes);
  NormRopeBwdArgs a{};
  PairedArgs& p = a.fwd;
  // gradients of the inputs are written contiguously, [batch, heads, seq, head_dim]
  p.t[0] = PairedTensor{q, grad_q, q_stride_b, q_stride_h, q_stride_s, q_heads * seq * head_dim, seq * head_dim, head_dim, static_cast<int>(q_heads)};
  p.t[1] = PairedTensor{k, grad_k, k_stride_b, k_stride_h, k_stride_s, k_heads * seq * head_dim, seq * head_dim, head_dim, static_cast<int>(k_heads)};
  p.cos = cos;
  p.sin = sin;
  p.cs_stride_b = cos_batch == 1 ? 0 : seq * head_dim;
  p.seq = seq;
  p.batch = static_cast<int>(batch);
  p.head_dim = static_cast<int>(head_dim);
  p.weight[0] = q_weight;
  p.weight[1] = k_weight;
  p.eps = static_cast<float>(eps);
  a.dy[0] = grad_q_out;
  a.dy[1] = grad_k_out;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (batch == 0 || seq == 0 || (q_heads == 0 && k_heads == 0)) {
    // no rows: the weight gradients are zero
    if (q_heads >= 0 && grad_q_weight) (void)cudaMemsetAsync(grad_q_weight, 0, head_dim * es, st);
    if (k_heads >= 0 && grad_k_weight) (void)cudaMemsetAsync(grad_k_weight, 0, head_dim * es, st);
    return B200_OK;
  }
  B200_DISPATCH_DTYPE(dtype, T, return run_norm_rope_bwd<T>(a, q_heads > 0 ? grad_q_weight : nullptr, k_heads > 0 ? grad_k_weight : nullptr,
                                                             static_cast<float*>(scratch), st));
  return B200_OK;
}
