// Device helpers shared by the kernels of the M-to-N redistribution (sm_100a): streaming loads, multicast
// stores, box index arithmetic, typed 8-element vectors, the reduce step, completion signalling and the
// tile -> op lookup.  Everything is `static`/inline so that each translation unit gets its own copy.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "m2n.h"

namespace {

// ---------------------------------------------------------------------------------------------
// memory access helpers
// ---------------------------------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ V ld_stream(const void* p);

template <>
__device__ __forceinline__ uint4 ld_stream<uint4>(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
template <>
__device__ __forceinline__ uint2 ld_stream<uint2>(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
template <>
__device__ __forceinline__ uint32_t ld_stream<uint32_t>(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
template <>
__device__ __forceinline__ uint16_t ld_stream<uint16_t>(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
template <>
__device__ __forceinline__ uint8_t ld_stream<uint8_t>(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return (uint8_t)v;
}

// a thread that reads 32 contiguous bytes with two 16-byte loads touches every 32-byte sector twice: let the
// first load allocate the sector in L1 so that the second one does not go back to L2
__device__ __forceinline__ uint4 ld_keep(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <typename V>
__device__ __forceinline__ void st_plain(void* p, V v) {
  *reinterpret_cast<V*>(p) = v;
}

// one 16-byte store delivered by NVSwitch to every GPU bound to the multicast object
__device__ __forceinline__ void st_multimem16(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t shr) {
  return mul ? (__umulhi(n, mul) >> shr) : n;  // mul == 0 encodes "divide by one"
}

// byte offsets of unit `unit` of the op inside the source and the destination box
template <int ND = -1>
__device__ __forceinline__ void unit_offsets(const M2NOp& op, uint32_t unit, int64_t& so, int64_t& dof) {
  if constexpr (ND == 0) {  // one contiguous run on both sides
    so = (int64_t)unit * op.unit_bytes_src;
    dof = (int64_t)unit * op.unit_bytes_dst;
    return;
  }
  uint32_t q = fast_div(unit, op.div_mul[M2N_MAX_DIMS], op.div_shr[M2N_MAX_DIMS]);
  uint32_t col = unit - q * op.inner_units;
  so = (int64_t)col * op.unit_bytes_src;
  dof = (int64_t)col * op.unit_bytes_dst;
  if constexpr (ND == 1) {  // rows of a matrix
    so += (int64_t)q * op.src_stride[0];
    dof += (int64_t)q * op.dst_stride[0];
    return;
  }
  const int nd = op.ndim;
#pragma unroll
  for (int d = M2N_MAX_DIMS - 1; d >= 0; --d) {
    if (d < nd) {
      uint32_t q2 = (d == 0) ? 0u : fast_div(q, op.div_mul[d], op.div_shr[d]);
      uint32_t i = q - q2 * op.extent[d];
      so += (int64_t)i * op.src_stride[d];
      dof += (int64_t)i * op.dst_stride[d];
      q = q2;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// typed element vectors (8 elements) for conversion and reduction
// ---------------------------------------------------------------------------------------------
template <int DT>
struct Elem;

template <>
struct Elem<M2N_F32> {
  static constexpr int W = 2;  // 16-byte words per 8 elements
  static __device__ __forceinline__ void load_raw(const char* p, uint4 (&r)[2]) {
    r[0] = ld_keep(p);
    r[1] = ld_keep(p + 16);
  }
  static __device__ __forceinline__ void decode(const uint4 (&r)[2], float (&f)[8]) {
    const uint4 a = r[0], b = r[1];
    f[0] = __uint_as_float(a.x), f[1] = __uint_as_float(a.y), f[2] = __uint_as_float(a.z), f[3] = __uint_as_float(a.w);
    f[4] = __uint_as_float(b.x), f[5] = __uint_as_float(b.y), f[6] = __uint_as_float(b.z), f[7] = __uint_as_float(b.w);
  }
  static __device__ __forceinline__ void load8(const char* p, float (&f)[8]) {
    uint4 r[2];
    load_raw(p, r);
    decode(r, f);
  }
  static __device__ __forceinline__ void store8(char* p, const float (&f)[8]) {
    st_plain<uint4>(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
    st_plain<uint4>(p + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
  }
  static __device__ __forceinline__ float load1(const char* p) { return __uint_as_float(ld_stream<uint32_t>(p)); }
  static __device__ __forceinline__ void store1(char* p, float f) { *reinterpret_cast<float*>(p) = f; }
};

template <>
struct Elem<M2N_BF16> {
  static __device__ __forceinline__ float up(uint32_t w, int hi) { return __uint_as_float(hi ? (w & 0xffff0000u) : (w << 16)); }
  static constexpr int W = 1;
  static __device__ __forceinline__ void load_raw(const char* p, uint4 (&r)[1]) { r[0] = ld_stream<uint4>(p); }
  static __device__ __forceinline__ void decode(const uint4 (&r)[1], float (&f)[8]) {
    const uint4 a = r[0];
    f[0] = up(a.x, 0), f[1] = up(a.x, 1), f[2] = up(a.y, 0), f[3] = up(a.y, 1);
    f[4] = up(a.z, 0), f[5] = up(a.z, 1), f[6] = up(a.w, 0), f[7] = up(a.w, 1);
  }
  static __device__ __forceinline__ void load8(const char* p, float (&f)[8]) {
    uint4 r[1];
    load_raw(p, r);
    decode(r, f);
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void store8(char* p, const float (&f)[8]) {
    st_plain<uint4>(p, make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7])));
  }
  static __device__ __forceinline__ float load1(const char* p) { return __uint_as_float((uint32_t)ld_stream<uint16_t>(p) << 16); }
  static __device__ __forceinline__ void store1(char* p, float f) { *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(f); }
};

template <>
struct Elem<M2N_F16> {
  static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    float2 f = __half22float2(h);
    lo = f.x, hi = f.y;
  }
  static constexpr int W = 1;
  static __device__ __forceinline__ void load_raw(const char* p, uint4 (&r)[1]) { r[0] = ld_stream<uint4>(p); }
  static __device__ __forceinline__ void decode(const uint4 (&r)[1], float (&f)[8]) {
    const uint4 a = r[0];
    unpack(a.x, f[0], f[1]), unpack(a.y, f[2], f[3]), unpack(a.z, f[4], f[5]), unpack(a.w, f[6], f[7]);
  }
  static __device__ __forceinline__ void load8(const char* p, float (&f)[8]) {
    uint4 r[1];
    load_raw(p, r);
    decode(r, f);
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void store8(char* p, const float (&f)[8]) {
    st_plain<uint4>(p, make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7])));
  }
  static __device__ __forceinline__ float load1(const char* p) {
    uint16_t b = ld_stream<uint16_t>(p);
    return __half2float(*reinterpret_cast<__half*>(&b));
  }
  static __device__ __forceinline__ void store1(char* p, float f) { *reinterpret_cast<__half*>(p) = __float2half_rn(f); }
};

// store 8 converted elements either with plain stores or, for an NVLS destination, with multicast stores
template <int DDT>
__device__ __forceinline__ void store8_to(char* p, const float (&f)[8], bool multicast) {
  if (!multicast) {
    Elem<DDT>::store8(p, f);
    return;
  }
  if constexpr (DDT == M2N_F32) {
    st_multimem16(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
    st_multimem16(p + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
  } else {
    st_multimem16(p, make_uint4(Elem<DDT>::pack(f[0], f[1]), Elem<DDT>::pack(f[2], f[3]), Elem<DDT>::pack(f[4], f[5]),
                                Elem<DDT>::pack(f[6], f[7])));
  }
}

__device__ __forceinline__ float reduce2(float a, float b, int op) {
  switch (op) {
    case M2N_MAX: return (a != a) ? a : ((b != b) ? b : fmaxf(a, b));  // NaN propagates, like torch.maximum
    case M2N_MIN: return (a != a) ? a : ((b != b) ? b : fminf(a, b));
    case M2N_PROD: return a * b;
    default: return a + b;  // SUM and AVG
  }
}

template <int DT>
__device__ __forceinline__ float round_through(float x) {
  if constexpr (DT == M2N_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  if constexpr (DT == M2N_F16) return __half2float(__float2half_rn(x));
  return x;
}

// after the last CTA: publish `epoch` to every flag with system-scope release ordering
__device__ __forceinline__ void finish_and_signal(uint32_t* sync, const uint64_t* signals, uint32_t n_signals,
                                                  uint32_t epoch) {
  __shared__ uint32_t s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t prev = atomicAdd(&sync[0], 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) sync[0] = 0;  // ready for the next launch on this stream
    __threadfence_system();
    for (uint32_t i = threadIdx.x; i < n_signals; i += blockDim.x) {
      uint32_t* flag = reinterpret_cast<uint32_t*>(signals[i]);
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
    }
  }
}

// binary search of the op that owns `tile`, and (re)load of that op into shared memory
__device__ __forceinline__ uint32_t locate_op(const M2NOp* __restrict__ ops, const uint32_t* __restrict__ tile_start,
                                              uint32_t n_ops, uint32_t tile, uint32_t& cur, M2NOp* s_op) {
  uint32_t lo = 0, hi = n_ops;
  while (hi - lo > 1) {
    uint32_t mid = (lo + hi) >> 1;
    if (tile_start[mid] <= tile) lo = mid; else hi = mid;
  }
  if (lo != cur) {
    __syncthreads();
    const uint4* g = reinterpret_cast<const uint4*>(ops + lo);
    uint4* s = reinterpret_cast<uint4*>(s_op);
    for (uint32_t i = threadIdx.x; i < sizeof(M2NOp) / 16; i += blockDim.x) s[i] = g[i];
    __syncthreads();
    cur = lo;
  }
  return lo;
}

}  // namespace
