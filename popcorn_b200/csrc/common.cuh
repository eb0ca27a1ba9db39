// Shared device/host helpers for the sm_100a kernels of libpopcorn_b200.
//
// Numeric rule used throughout: a value is rounded to the storage type T at
// every point where the PyTorch reference materialises a tensor of that type,
// and every fp32 product / sum is rounded on its own (explicit *_rn intrinsics,
// which the compiler never contracts into a fused multiply-add).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/popcorn_b200.h"

namespace b200 {

// ---------------------------------------------------------------- host side --

// Records a failure reason for the calling thread and returns `status`.
int fail(int status, const char* fmt, ...);
// cudaGetLastError() -> status, counting the launch when it succeeded.
int after_launch(const char* kernel);
// B200_OK when the current device is compute capability 10.x.
int check_device();
// Number of SMs of the current device (cached per device).
int sm_count();
// Bounded waits that ran out, per source file that uses bulk asynchronous copies.
unsigned int rope_wait_timeouts();
unsigned int norm_wait_timeouts();
unsigned int gemm_wait_timeouts();
// rms_norm / add_rms_norm backward through the row-bucket kernel of norm_family.cu (rows of at most 1024 128-bit
// words held in registers; narrow rows several per warp).  gs: the gradient that arrived for the sum s of
// add_rms_norm, or nullptr; offset: added to the weight; add = false ignores both (rms_norm).  All pointers 16-byte aligned, cols and
// the strides multiples of the word; scratch as for b200_rms_norm_backward.  Called from norm.cu, which decides
// which shapes take this path.
int rms_backward_narrow_rows(int dtype, const void* gy, const void* gs, const void* x, const void* w, void* dx, void* dw, void* db,
                             float* scratch, int64_t rows, int64_t cols, int64_t ldg, int64_t ldgs, int64_t ldx, int64_t lddx, float eps,
                             float offset, bool add, cudaStream_t st);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline size_t dtype_size(int dtype) { return dtype == B200_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == B200_F32 || dtype == B200_F16 || dtype == B200_BF16; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Whether kernels are launched with programmatic dependent launch (see launch()).
bool pdl_enabled();

// Launch `kernel` on `st`.  With programmatic dependent launch the grid may be
// scheduled while the previous kernel of the stream is still draining; every
// kernel of this library calls pdl_prologue() before its first global access,
// which blocks until that previous kernel has completed and its writes are
// visible, so stream order is preserved and only launch latency overlaps.
template <typename... Params, typename... Args>
inline void launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  (void)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

#define B200_REQUIRE_PTR(p)                                                        \
  do {                                                                             \
    if ((p) == nullptr) return ::b200::fail(B200_ERR_NULL_POINTER, "%s: %s is NULL", __func__, #p); \
  } while (0)

// -------------------------------------------------------------- device side --

constexpr int kVecBytes = 16;  // every fast path moves 128-bit words

// First statement of every kernel: let the next kernel of the stream begin its
// launch, then wait until the previous one has completed (a no-op for a grid
// that was launched without programmatic dependent launch).
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename T>
struct Num;

template <>
struct Num<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ float up(float v) { return v; }
  static __device__ __forceinline__ float down(float v) { return v; }
  // round-trip through the storage type: identity for fp32
  static __device__ __forceinline__ float rt(float v) { return v; }
  static __device__ __forceinline__ void round2(float&, float&) {}
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

template <>
struct Num<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float rt(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  // bf16 -> fp32 is a 16-bit shift of the bit pattern
  static __device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  // Round two fp32 values to bf16 and back with ONE packed conversion. The scalar
  // cvt.rn.bf16.f32 issues on the quarter-rate conversion pipe and made kernels
  // that round per element pipe-bound; the packed form does not.
  static __device__ __forceinline__ void round2(float& a, float& b) { unpack2(pack2(a, b), a, b); }
  // Product of two packed pairs, each rounded once to bf16.  A bf16 x bf16 product is exact in
  // fp32, so this equals round(fp32(a) * fp32(b)), the way the reference multiplies two bf16 tensors.
  static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2_rn(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  // Sum of two packed pairs, each rounded once to bf16.  The reference adds two bf16 tensors as
  // round_bf16(round_fp32(a + b)); the two roundings can only differ from one when the exact sum
  // does not fit fp32 (exponents more than 16 apart) AND lies next to a bf16 tie (exponents about 8
  // apart), which cannot both hold, so the packed add gives the reference's bits.
  static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hadd2_rn(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    unpack2(v.x, f[0], f[1]);
    unpack2(v.y, f[2], f[3]);
    unpack2(v.z, f[4], f[5]);
    unpack2(v.w, f[6], f[7]);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};

template <>
struct Num<__half> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float rt(float v) { return __half2float(__float2half_rn(v)); }
  static __device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  static __device__ __forceinline__ void round2(float& a, float& b) { unpack2(pack2(a, b), a, b); }
  // fp16 x fp16 is exact in fp32 as well (22 significant bits): one rounding, like the reference.
  static __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    __half2 r = __hmul2_rn(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  // Packed sum, one rounding per half; equal to round_fp16(round_fp32(a + b)) for the same reason as
  // in the bf16 case (inexact in fp32 needs exponents more than 13 apart, a near-tie about 11).
  static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    __half2 r = __hadd2_rn(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    unpack2(v.x, f[0], f[1]);
    unpack2(v.y, f[2], f[3]);
    unpack2(v.z, f[4], f[5]);
    unpack2(v.w, f[6], f[7]);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};

// 128-bit global accesses. Inputs are read once: bypass L1 allocation (a
// coherent load, not .nc, because several entry points allow out == in).
// Outputs are written once: streaming store.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Plain (cacheable) 128-bit load for data another thread of this kernel may have written.
__device__ __forceinline__ uint4 ld_plain(const void* p) { return *reinterpret_cast<const uint4*>(p); }
// Read-only 128-bit load that may stay in L1 (weights, cos/sin rows: reused by many warps).
__device__ __forceinline__ uint4 ld_reuse(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 256-bit global accesses (sm_100: ld/st.global.v8.b32): half as many memory instructions per byte as the 128-bit
// forms.  The address must be 32-byte aligned.
struct alignas(32) Word256 {
  uint4 lo, hi;
};
__device__ __forceinline__ Word256 ld_stream256(const void* p) {
  Word256 v;
  asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream256(void* p, const Word256& v) {
  asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.lo.x), "r"(v.lo.y), "r"(v.lo.z), "r"(v.lo.w),
               "r"(v.hi.x), "r"(v.hi.y), "r"(v.hi.z), "r"(v.hi.w)
               : "memory");
}

// Two fp32 operations per instruction (Blackwell packed fp32).  Each half is rounded to
// nearest-even on its own, exactly like the scalar __fmul_rn / __fadd_rn / __fsub_rn.
struct Float2x {
  unsigned long long bits;
};
__device__ __forceinline__ Float2x pack_f2(float lo, float hi) {
  Float2x r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.bits) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(Float2x v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v.bits));
}
__device__ __forceinline__ Float2x mul_f2(Float2x a, Float2x b) {
  Float2x r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}
// NOTE: the assembler fuses a packed product with a following packed add or sub into one fused
// multiply-add when the product has no other use (measured: the result then equals
// fma(-d, s, a*c) in every case; --fmad=false and adding through fma(p, +-1, q) do not stop it).
// Where the reference rounds product and sum separately, take the products packed and add them
// with the scalar __fadd_rn / __fsub_rn.
__device__ __forceinline__ Float2x add_f2(Float2x a, Float2x b) {
  Float2x r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}
// a * b + c with one rounding per half; only for places where the reference's own result is rounded
// to a 16-bit type afterwards or is compared within a tolerance.
__device__ __forceinline__ Float2x fma_f2(Float2x a, Float2x b, Float2x c) {
  Float2x r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits), "l"(c.bits));
  return r;
}
__device__ __forceinline__ Float2x sub_f2(Float2x a, Float2x b) {
  Float2x r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dispatch a runtime dtype enum to a template parameter.
#define B200_DISPATCH_DTYPE(dtype, T, ...)              \
  do {                                                  \
    switch (dtype) {                                    \
      case B200_F32: {                                  \
        using T = float;                                \
        __VA_ARGS__;                                    \
      } break;                                          \
      case B200_F16: {                                  \
        using T = __half;                               \
        __VA_ARGS__;                                    \
      } break;                                          \
      default: {                                        \
        using T = __nv_bfloat16;                        \
        __VA_ARGS__;                                    \
      } break;                                          \
    }                                                   \
  } while (0)

}  // namespace b200
