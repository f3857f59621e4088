// sm_100a kernels of the M-to-N redistribution: strided gather -> (convert | reduce) -> strided
// scatter into local, peer or multicast memory, plus the release/acquire flag kernels.
//
// One persistent launch walks a device-resident table of `M2NOp`s (see m2n.h).  The table is built
// once per registered batch and launched once per transfer, so a transfer costs no host work per
// chunk and no staging buffer: the producer GPU reads its own memory and stores straight into the
// consumers' slices over NVLink.  This replaces the reference's per-chunk slice/contiguous/cast/
// pack kernels and its NCCL send/recv/broadcast/all-reduce calls (src/etha/comm/ir.py:101-141,
// 229-310; src/etha/comm/transfer.py:20-41).
#include "m2n.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <type_traits>

#include "common.h"
#include "m2n_device.cuh"

namespace {

// ---------------------------------------------------------------------------------------------
// tile bodies
// ---------------------------------------------------------------------------------------------
template <typename V, int UNROLL, int ND>
__device__ __forceinline__ void tile_raw(const M2NOp& op, uint32_t base, uint32_t limit) {
  V v[UNROLL];
  int64_t doff[UNROLL];
  bool ok[UNROLL];
  const char* src = reinterpret_cast<const char*>(op.src[0]);
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    uint32_t unit = base + u * blockDim.x + threadIdx.x;
    ok[u] = unit < limit;
    if (ok[u]) {
      int64_t so;
      unit_offsets<ND>(op, unit, so, doff[u]);
      v[u] = ld_stream<V>(src + so);
    }
  }
  const int nd = op.ndst;
  if constexpr (std::is_same<V, uint4>::value) {
    if (op.flags & M2N_FLAG_MULTIMEM) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (ok[u]) st_multimem16(reinterpret_cast<char*>(op.dst[0]) + doff[u], v[u]);
      return;
    }
  }
  for (int j = 0; j < nd; ++j) {
    char* dst = reinterpret_cast<char*>(op.dst[j]);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (ok[u]) st_plain<V>(dst + doff[u], v[u]);
  }
}

template <int SDT, int DDT, int UNROLL, int ND = -1>
__device__ __forceinline__ void tile_cvt8(const M2NOp& op, uint32_t base, uint32_t limit) {
  // all loads of the thread are issued before the first store, so UNROLL * 16..32 bytes are in flight per thread
  const char* src = reinterpret_cast<const char*>(op.src[0]);
  uint4 raw[UNROLL][Elem<SDT>::W];
  int64_t doff[UNROLL];
  bool ok[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    uint32_t unit = base + u * blockDim.x + threadIdx.x;
    ok[u] = unit < limit;
    if (ok[u]) {
      int64_t so;
      unit_offsets<ND>(op, unit, so, doff[u]);
      Elem<SDT>::load_raw(src + so, raw[u]);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    if (ok[u]) {
      float f[8];
      Elem<SDT>::decode(raw[u], f);
      const bool mc = op.flags & M2N_FLAG_MULTIMEM;
      for (int j = 0; j < op.ndst; ++j) store8_to<DDT>(reinterpret_cast<char*>(op.dst[j]) + doff[u], f, mc);
    }
  }
}

// Single-level Partial collapse of exactly NSRC sources, 8 elements per unit: every source word of the unit is
// requested before the first one is used.
template <int SDT, int DDT, int NSRC, int ND = -1>
__device__ __forceinline__ void tile_reduce_flat(const M2NOp& op, uint32_t base, uint32_t limit, int unroll) {
  const int rop = op.red_op[0];
  for (int u = 0; u < unroll; ++u) {
    uint32_t unit = base + u * blockDim.x + threadIdx.x;
    if (unit >= limit) continue;
    int64_t so, dof;
    unit_offsets<ND>(op, unit, so, dof);
    uint4 raw[NSRC][Elem<SDT>::W];
#pragma unroll
    for (int i = 0; i < NSRC; ++i) Elem<SDT>::load_raw(reinterpret_cast<const char*>(op.src[i]) + so, raw[i]);
    float acc[8];
    Elem<SDT>::decode(raw[0], acc);
#pragma unroll
    for (int i = 1; i < NSRC; ++i) {
      float f[8];
      Elem<SDT>::decode(raw[i], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = reduce2(acc[k], f[k], rop);
    }
    if (rop == M2N_AVG) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = __fdiv_rn(acc[k], (float)NSRC);
    }
    if constexpr (SDT != DDT) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = round_through<SDT>(acc[k]);
    }
    const bool mc = op.flags & M2N_FLAG_MULTIMEM;
    for (int j = 0; j < op.ndst; ++j) store8_to<DDT>(reinterpret_cast<char*>(op.dst[j]) + dof, acc, mc);
  }
}

template <int SDT, int DDT, int UNROLL>
__device__ __forceinline__ void tile_cvt1(const M2NOp& op, uint32_t base, uint32_t limit) {
  const char* src = reinterpret_cast<const char*>(op.src[0]);
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    uint32_t unit = base + u * blockDim.x + threadIdx.x;
    if (unit < limit) {
      int64_t so, dof;
      unit_offsets(op, unit, so, dof);
      float f = Elem<SDT>::load1(src + so);
      for (int j = 0; j < op.ndst; ++j) Elem<DDT>::store1(reinterpret_cast<char*>(op.dst[j]) + dof, f);
    }
  }
}

// Partial collapse: level 0 groups of red_size[0] consecutive sources, then level 1 over the group results;
// fp32 accumulation in ascending source order, "avg" divides by the group size.  The collapsed value is
// rounded once to the SOURCE dtype (the dtype a Partial -> Replicate redistribution yields) and then converted
// to the destination dtype, so a two-way sum is bit-identical to an all-reduce in the source dtype.
template <int SDT, int DDT, int N>
__device__ __forceinline__ void tile_reduce(const M2NOp& op, uint32_t base, uint32_t limit, int unroll) {
  const int s0 = op.red_size[0], s1 = op.red_size[1];
  const int op0 = op.red_op[0], op1 = op.red_op[1];
  for (int u = 0; u < unroll; ++u) {
    uint32_t unit = base + u * blockDim.x + threadIdx.x;
    if (unit >= limit) continue;
    int64_t so, dof;
    unit_offsets(op, unit, so, dof);
    float acc[N];
    for (int g = 0; g < s1; ++g) {
      float a[N];
      for (int i = 0; i < s0; ++i) {
        const char* p = reinterpret_cast<const char*>(op.src[g * s0 + i]) + so;
        float f[N];
        if constexpr (N == 8) {
          Elem<SDT>::load8(p, f);
        } else {
          f[0] = Elem<SDT>::load1(p);
        }
#pragma unroll
        for (int k = 0; k < N; ++k) a[k] = (i == 0) ? f[k] : reduce2(a[k], f[k], op0);
      }
      if (op0 == M2N_AVG) {
#pragma unroll
        for (int k = 0; k < N; ++k) a[k] = __fdiv_rn(a[k], (float)s0);
      }
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = (g == 0) ? a[k] : reduce2(acc[k], a[k], op1);
    }
    if (op1 == M2N_AVG && s1 > 1) {
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = __fdiv_rn(acc[k], (float)s1);
    }
    if constexpr (SDT != DDT) {
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = round_through<SDT>(acc[k]);
    }
    for (int j = 0; j < op.ndst; ++j) {
      char* d = reinterpret_cast<char*>(op.dst[j]) + dof;
      if constexpr (N == 8) {
        store8_to<DDT>(d, acc, op.flags & M2N_FLAG_MULTIMEM);
      } else {
        Elem<DDT>::store1(d, acc[0]);
      }
    }
  }
}

// One out-of-line walker per (source dtype, destination dtype): each gets its own register allocation.
#ifndef ETHA_TYPED_UNROLL
#define ETHA_TYPED_UNROLL 4
#endif
#ifndef ETHA_GENERAL_CTAS
#define ETHA_GENERAL_CTAS 4
#endif
constexpr int kTypedUnroll = ETHA_TYPED_UNROLL;

template <int S, int D>
__device__ __noinline__ void walk_cvt(const M2NOp& op, uint32_t base, uint32_t limit) {
  const uint32_t step = blockDim.x * kTypedUnroll;
  if (op.unit_elems == 8) {
    // boxes that are one run or rows of a matrix (almost every weight) skip the generic index arithmetic
    if (op.ndim == 0) {
      for (uint32_t b = base; b < limit; b += step) tile_cvt8<S, D, kTypedUnroll, 0>(op, b, limit);
    } else if (op.ndim == 1) {
      for (uint32_t b = base; b < limit; b += step) tile_cvt8<S, D, kTypedUnroll, 1>(op, b, limit);
    } else {
      for (uint32_t b = base; b < limit; b += step) tile_cvt8<S, D, kTypedUnroll>(op, b, limit);
    }
  } else {
    for (uint32_t b = base; b < limit; b += step) tile_cvt1<S, D, kTypedUnroll>(op, b, limit);
  }
}

template <int S, int D>
__device__ __noinline__ void walk_red(const M2NOp& op, uint32_t base, uint32_t limit) {
  const bool vec = op.unit_elems == 8;
  const bool flat = vec && op.red_size[1] == 1;
  const uint32_t step = blockDim.x * 2;
  for (uint32_t b = base; b < limit; b += step) {
    if (flat && op.nsrc == 2 && op.ndim == 0) tile_reduce_flat<S, D, 2, 0>(op, b, limit, 2);
    else if (flat && op.nsrc == 2 && op.ndim == 1) tile_reduce_flat<S, D, 2, 1>(op, b, limit, 2);
    else if (flat && op.nsrc == 2) tile_reduce_flat<S, D, 2>(op, b, limit, 2);
    else if (flat && op.nsrc == 4) tile_reduce_flat<S, D, 4>(op, b, limit, 2);
    else if (flat && op.nsrc == 8) tile_reduce_flat<S, D, 8>(op, b, limit, 2);
    else if (vec) tile_reduce<S, D, 8>(op, b, limit, 2);
    else tile_reduce<S, D, 1>(op, b, limit, 2);
  }
}

__device__ __forceinline__ bool dispatch_typed(const M2NOp& op, uint32_t base, uint32_t limit) {
  const int key = (op.mode << 8) | (op.src_dtype << 4) | op.dst_dtype;
#define CASE_CVT(S, D) case (M2N_MODE_CVT << 8) | (S << 4) | D: walk_cvt<S, D>(op, base, limit); return true;
#define CASE_RED(S, D) case (M2N_MODE_REDUCE << 8) | (S << 4) | D: walk_red<S, D>(op, base, limit); return true;
  switch (key) {
    CASE_CVT(M2N_F32, M2N_BF16) CASE_CVT(M2N_F32, M2N_F16) CASE_CVT(M2N_BF16, M2N_F32) CASE_CVT(M2N_F16, M2N_F32)
    CASE_CVT(M2N_BF16, M2N_F16) CASE_CVT(M2N_F16, M2N_BF16)
    CASE_RED(M2N_F32, M2N_F32) CASE_RED(M2N_F32, M2N_BF16) CASE_RED(M2N_F32, M2N_F16) CASE_RED(M2N_BF16, M2N_BF16)
    CASE_RED(M2N_BF16, M2N_F32) CASE_RED(M2N_BF16, M2N_F16) CASE_RED(M2N_F16, M2N_F16) CASE_RED(M2N_F16, M2N_F32)
    CASE_RED(M2N_F16, M2N_BF16)
    default: return false;
  }
#undef CASE_CVT
#undef CASE_RED
}

#ifndef ETHA_FAST_UNROLL
#define ETHA_FAST_UNROLL 4
#endif
constexpr int kUnroll = ETHA_FAST_UNROLL;

// Fast class: 16-byte bit copies whose box is one run or rows of a matrix (the bulk of a weight sync).
__global__ void __launch_bounds__(512, 2)
m2n_fast_kernel(const M2NOp* __restrict__ ops, const uint32_t* __restrict__ tile_start, uint32_t n_ops, uint32_t* sync,
                const uint64_t* __restrict__ signals, uint32_t n_signals, uint32_t epoch, int do_signal) {
  __shared__ M2NOp s_op;
  const uint32_t total_tiles = n_ops ? tile_start[n_ops] : 0;
  uint32_t cur = 0xffffffffu;
  for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const uint32_t lo = locate_op(ops, tile_start, n_ops, tile, cur, &s_op);
    const M2NOp& op = s_op;
    const uint32_t base = (tile - tile_start[lo]) * op.tile_units;
    const uint32_t limit = min(op.total_units, base + op.tile_units);
    const uint32_t step = blockDim.x * kUnroll;
    if (op.ndim == 0) {
      for (uint32_t b = base; b < limit; b += step) tile_raw<uint4, kUnroll, 0>(op, b, limit);
    } else {
      for (uint32_t b = base; b < limit; b += step) tile_raw<uint4, kUnroll, 1>(op, b, limit);
    }
  }
  if (do_signal) finish_and_signal(sync, signals, n_signals, epoch);
}

// General class: any other bit copy, converting copies and Partial collapses.
constexpr int kGenUnroll = 2;
template <typename V>
__device__ __noinline__ void walk_raw(const M2NOp& op, uint32_t base, uint32_t limit) {
  for (uint32_t b = base; b < limit; b += blockDim.x * kGenUnroll) tile_raw<V, kGenUnroll, -1>(op, b, limit);
}

__global__ void __launch_bounds__(256, ETHA_GENERAL_CTAS)
m2n_general_kernel(const M2NOp* __restrict__ ops, const uint32_t* __restrict__ tile_start, uint32_t n_ops,
                   uint32_t* sync, const uint64_t* __restrict__ signals, uint32_t n_signals, uint32_t epoch,
                   int do_signal) {
  __shared__ M2NOp s_op;
  const uint32_t total_tiles = n_ops ? tile_start[n_ops] : 0;
  uint32_t cur = 0xffffffffu;
  for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const uint32_t lo = locate_op(ops, tile_start, n_ops, tile, cur, &s_op);
    const M2NOp& op = s_op;
    const uint32_t base = (tile - tile_start[lo]) * op.tile_units;
    const uint32_t limit = min(op.total_units, base + op.tile_units);
    if (op.mode == M2N_MODE_RAW) {
      switch (op.unit_bytes_src) {
        case 16: walk_raw<uint4>(op, base, limit); break;
        case 8: walk_raw<uint2>(op, base, limit); break;
        case 4: walk_raw<uint32_t>(op, base, limit); break;
        case 2: walk_raw<uint16_t>(op, base, limit); break;
        default: walk_raw<uint8_t>(op, base, limit); break;
      }
    } else if (!dispatch_typed(op, base, limit)) {
      if (threadIdx.x == 0) sync[1] = M2N_BAD_OP;
    }
  }
  if (do_signal) finish_and_signal(sync, signals, n_signals, epoch);
}

__global__ void set_flags_kernel(const uint64_t* __restrict__ signals, uint32_t n_signals, uint32_t epoch) {
  __threadfence_system();
  for (uint32_t i = threadIdx.x; i < n_signals; i += blockDim.x) {
    uint32_t* flag = reinterpret_cast<uint32_t*>(signals[i]);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
  }
}

// Bounded acquire-wait.  A flag counts as set once it reached `epoch` (wrap-safe compare).  On timeout the
// kernel reports which flag was missing and returns; it never traps and never spins without a limit.
__global__ void wait_flags_kernel(const uint32_t* __restrict__ flags, const uint32_t* __restrict__ which, uint32_t n,
                                  uint32_t epoch, uint64_t timeout_ns, uint32_t* status) {
  __shared__ uint32_t s_fail, s_who;
  if (threadIdx.x == 0) { s_fail = 0; s_who = 0xffffffffu; }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t* flag = flags + which[i];
    uint64_t t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    bool ok = false;
    for (uint64_t it = 0; it < (1ull << 34); ++it) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if ((int32_t)(v - epoch) >= 0) { ok = true; break; }
      if ((it & 63) == 63) {
        uint64_t t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (t - t0 > timeout_ns) break;
        __nanosleep(200);
      }
    }
    if (!ok) { atomicExch(&s_fail, 1u); atomicMin(&s_who, i); }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    status[1] = s_who;
    __threadfence_system();
    status[0] = s_fail ? M2N_TIMEOUT : M2N_OK;
  }
}

inline int fail(cudaError_t e, const char* what) {
  snprintf(etha_err_buf(), ETHA_ERR_LEN, "%s: %s", what, cudaGetErrorString(e));
  return -(int)e - 1000;
}

}  // namespace

extern "C" {

// resident 256-thread CTAs per SM the general kernel was compiled for (the launcher sizes its grid with it)
int etha_general_ctas_per_sm(void) { return ETHA_GENERAL_CTAS; }

int etha_m2n_launch(const M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int typed, int grid, int block,
                    uint32_t* sync_scratch, const uint64_t* signals, uint32_t n_signals, uint32_t epoch,
                    int do_signal, void* stream) {
  if (grid < 1) grid = 1;
  if (typed) {
    if (block < 32 || block > 256 || (block & 31)) block = 256;
    m2n_general_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(ops, tile_start, n_ops, sync_scratch, signals, n_signals,
                                                               epoch, do_signal);
  } else {
    if (block < 32 || block > 512 || (block & 31)) block = 512;
    m2n_fast_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(ops, tile_start, n_ops, sync_scratch, signals, n_signals,
                                                             epoch, do_signal);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail(e, "m2n kernel launch");
}

int etha_set_flags(const uint64_t* signals, uint32_t n_signals, uint32_t epoch, void* stream) {
  set_flags_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(signals, n_signals, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail(e, "set_flags launch");
}

int etha_wait_flags(const uint32_t* flags, const uint32_t* which, uint32_t n, uint32_t epoch, uint64_t timeout_ns,
                    uint32_t* status, void* stream) {
  int block = n < 32 ? 32 : (n > 256 ? 256 : (int)((n + 31) & ~31u));
  wait_flags_kernel<<<1, block, 0, (cudaStream_t)stream>>>(flags, which, n, epoch, timeout_ns, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail(e, "wait_flags launch");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in no_alloc.h).  Same kernels as above; the op table, the tile
// prefix sums and the counters live in a resident array instead of caller-allocated device buffers.
// ---------------------------------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

namespace {

static_assert(sizeof(M2NOp) <= 320, "scratch layout assumes ops of at most 320 bytes");

// layout: [0,256) counters of the fast launch, [256,512) counters of the general launch,
//         [512,1280) tile_start of the fast class, [1280,2048) tile_start of the general class,
//         [2048, ...) ops: fast class first, general class after it
static __device__ __align__(256) unsigned char g_noalloc_scratch[ETHA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};
int g_noalloc_sms[kMaxDevices] = {0};

// Host code must not use `g_noalloc_scratch` as an address: there it is only a stand-in for the symbol.
// The device address is queried once per device, with that device current.
int noalloc_setup(int dev, unsigned char** out, int* sms) {
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "device index %d out of range", dev);
    return -101;
  }
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return fail(e, "cudaGetSymbolAddress(scratch)");
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(e, "cudaDeviceGetAttribute(sm count)");
    g_noalloc_sms[dev] = n;
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_noalloc_ptr[dev];
  *sms = g_noalloc_sms[dev];
  return 0;
}

}  // namespace

extern "C" int etha_pack_op(const M2NOpSpec* spec, M2NOp* out, char* err, int err_len);
extern "C" uint32_t etha_op_tiles(const M2NOp* op);
extern "C" int etha_op_class(const M2NOp* op);

extern "C" int etha_m2n_run_noalloc(const M2NOpSpec* specs, uint32_t n_specs, int ctas_per_sm, void* stream) {
  if (!specs && n_specs) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "null spec array");
    return -101;
  }
  if (n_specs > ETHA_NOALLOC_MAX_OPS) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "%u ops requested, the allocation-free entry point takes at most %d per call",
             n_specs, ETHA_NOALLOC_MAX_OPS);
    return -100;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(e, "cudaGetDevice");
  // every call stages its tables from host arrays of the calling thread with asynchronous copies: recorded into a
  // stream capture they would be replayed later from whatever those arrays hold then, so a capturing stream is refused
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  e = cudaStreamIsCapturing((cudaStream_t)stream, &cap);
  if (e != cudaSuccess) return fail(e, "cudaStreamIsCapturing");
  if (cap != cudaStreamCaptureStatusNone) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "the allocation-free entry point cannot be recorded into a stream capture");
    return -101;
  }
  unsigned char* scratch = nullptr;
  int sms = 0;
  int rc = noalloc_setup(dev, &scratch, &sms);
  if (rc != 0) return rc;

  // host staging lives in thread-local storage: no heap allocation per call
  static thread_local M2NOp packed[2][ETHA_NOALLOC_MAX_OPS];
  static thread_local uint32_t tile_start[2][ETHA_NOALLOC_MAX_OPS + 1];
  uint32_t count[2] = {0, 0};
  tile_start[0][0] = tile_start[1][0] = 0;
  for (uint32_t i = 0; i < n_specs; ++i) {
    M2NOp op;
    rc = etha_pack_op(&specs[i], &op, etha_err_buf(), ETHA_ERR_LEN);
    if (rc != 0) return rc;
    const uint32_t tiles = etha_op_tiles(&op);
    if (!tiles) continue;
    const int c = etha_op_class(&op);
    const uint64_t next = (uint64_t)tile_start[c][count[c]] + tiles;
    if (next >= (1ull << 32)) {
      snprintf(etha_err_buf(), ETHA_ERR_LEN, "too many tiles in one call");
      return -101;
    }
    packed[c][count[c]] = op;
    tile_start[c][++count[c]] = (uint32_t)next;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // counters must start at zero whatever the previous call left there
  e = cudaMemsetAsync(scratch, 0, 512, s);
  if (e != cudaSuccess) return fail(e, "cudaMemsetAsync(scratch counters)");
  if (ctas_per_sm <= 0) ctas_per_sm = 2;
  M2NOp* ops_dev = reinterpret_cast<M2NOp*>(scratch + 2048);
  for (int c = 0; c < 2; ++c) {
    if (!count[c]) continue;
    uint32_t* tiles_dev = reinterpret_cast<uint32_t*>(scratch + 512 + 768 * c);
    M2NOp* class_ops = ops_dev + (c == 0 ? 0 : count[0]);
    e = cudaMemcpyAsync(tiles_dev, tile_start[c], (count[c] + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return fail(e, "cudaMemcpyAsync(tile table)");
    e = cudaMemcpyAsync(class_ops, packed[c], count[c] * sizeof(M2NOp), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return fail(e, "cudaMemcpyAsync(op table)");
    const uint32_t total = tile_start[c][count[c]];
    int grid = (int)(total < (uint32_t)(sms * ctas_per_sm) ? total : (uint32_t)(sms * ctas_per_sm));
    if (grid < 1) grid = 1;
    uint32_t* sync = reinterpret_cast<uint32_t*>(scratch + 256 * c);
    if (c == 0)
      m2n_fast_kernel<<<grid, 512, 0, s>>>(class_ops, tiles_dev, count[c], sync, nullptr, 0, 0, 0);
    else
      m2n_general_kernel<<<grid, 256, 0, s>>>(class_ops, tiles_dev, count[c], sync, nullptr, 0, 0, 0);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(e, "allocation-free launch");
  }
  return 0;
}

extern "C" int etha_m2n_noalloc_status(uint32_t* status, void* stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(e, "cudaGetDevice");
  unsigned char* scratch = nullptr;
  int sms = 0;
  int rc = noalloc_setup(dev, &scratch, &sms);
  if (rc != 0) return rc;
  uint32_t words[2] = {0, 0};
  e = cudaMemcpyAsync(&words[0], scratch + 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(&words[1], scratch + 256 + 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(e, "read scratch status");
  *status = words[0] ? words[0] : words[1];
  return 0;
}
