// Streaming class of the typed ops: dtype conversion and single-level Partial collapse of 2 or 4 sources over
// boxes that are one run or the rows of a matrix, in 8-element units (16-byte aligned on every side).
//
// One kernel instance per (source dtype, destination dtype, number of sources): no dtype or source-count
// branch is left inside the loop, the box arithmetic is the one-run / matrix-row form, and every load a thread
// needs for its `kUnits` units (all sources of all units, 128 bytes per thread) is issued before the first value
// is used, so that a Partial collapse whose other contributors live on peer GPUs keeps enough bytes in flight to
// cover the NVLink round trip.  Two 256-thread CTAs per SM (up to 128 registers per thread: no spills).
// Arithmetic is the same as the general kernel's: fp32 accumulation in source order, "avg" divides by the
// number of sources, one rounding to the source dtype when the destination dtype differs, then conversion.
//
// Replaces, for these shapes, the reference's contiguous()/clone()/all_reduce/to() chain per chunk
// (src/etha/comm/ir.py:101-132).
#include <cuda_runtime.h>

#include <cstdio>

#include "common.h"
#include "m2n.h"
#include "m2n_device.cuh"

namespace {

#ifndef ETHA_STREAM_THREADS
#define ETHA_STREAM_THREADS 256
#endif
#ifndef ETHA_STREAM_CTAS
#define ETHA_STREAM_CTAS 2
#endif
constexpr int kTypedThreads = ETHA_STREAM_THREADS;
constexpr int kTypedCtasPerSm = ETHA_STREAM_CTAS;

template <int SDT, int NSRC>
struct Plan {
  static constexpr int W = Elem<SDT>::W;                       // 16-byte words per unit and source
  static constexpr int kRaw = 8;                               // 16-byte words in flight per thread
  static constexpr int kUnits = (kRaw / (W * NSRC)) > 4 ? 4 : ((kRaw / (W * NSRC)) < 1 ? 1 : kRaw / (W * NSRC));
};

template <int SDT, int DDT, int NSRC, int ND>
__device__ __forceinline__ void stream_tile(const M2NOp& op, uint32_t base, uint32_t limit) {
  constexpr int W = Elem<SDT>::W;
  constexpr int U = Plan<SDT, NSRC>::kUnits;
  const int rop = op.red_op[0];
  const bool mc = op.flags & M2N_FLAG_MULTIMEM;
  const uint32_t step = blockDim.x * U;
  for (uint32_t b = base; b < limit; b += step) {
    uint4 raw[U][NSRC][W];
    int64_t dof[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t unit = b + u * blockDim.x + threadIdx.x;
      ok[u] = unit < limit;
      if (ok[u]) {
        int64_t so;
        unit_offsets<ND>(op, unit, so, dof[u]);
#pragma unroll
        for (int i = 0; i < NSRC; ++i) Elem<SDT>::load_raw(reinterpret_cast<const char*>(op.src[i]) + so, raw[u][i]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!ok[u]) continue;
      float acc[8];
      Elem<SDT>::decode(raw[u][0], acc);
      if constexpr (NSRC > 1) {
#pragma unroll
        for (int i = 1; i < NSRC; ++i) {
          float f[8];
          Elem<SDT>::decode(raw[u][i], f);
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
      }
      for (int j = 0; j < op.ndst; ++j) store8_to<DDT>(reinterpret_cast<char*>(op.dst[j]) + dof[u], acc, mc);
    }
  }
}

template <int SDT, int DDT, int NSRC>
__global__ void __launch_bounds__(kTypedThreads, kTypedCtasPerSm)
m2n_typed_kernel(const M2NOp* __restrict__ ops, const uint32_t* __restrict__ tile_start, uint32_t n_ops, uint32_t* sync,
                 const uint64_t* __restrict__ signals, uint32_t n_signals, uint32_t epoch, int do_signal) {
  __shared__ M2NOp s_op;
  const uint32_t total_tiles = n_ops ? tile_start[n_ops] : 0;
  uint32_t cur = 0xffffffffu;
  for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const uint32_t lo = locate_op(ops, tile_start, n_ops, tile, cur, &s_op);
    const M2NOp& op = s_op;
    const uint32_t base = (tile - tile_start[lo]) * op.tile_units;
    const uint32_t limit = min(op.total_units, base + op.tile_units);
    // the host only puts ops of this instance's key into the table; anything else is reported, not executed
    if (op.src_dtype != SDT || op.dst_dtype != DDT || op.nsrc != NSRC || op.unit_elems != 8 || op.ndim > 1) {
      if (threadIdx.x == 0) sync[1] = M2N_BAD_OP;
      continue;
    }
    if (op.ndim == 0) stream_tile<SDT, DDT, NSRC, 0>(op, base, limit);
    else stream_tile<SDT, DDT, NSRC, 1>(op, base, limit);
  }
  if (do_signal) finish_and_signal(sync, signals, n_signals, epoch);
}

constexpr bool typed(int dt) { return dt == M2N_F32 || dt == M2N_BF16 || dt == M2N_F16; }

// combinations with a kernel instance: conversions between any two of fp32/bf16/fp16; collapses of 2 or 4
// sources whose destination dtype equals the source dtype or where one of the two is fp32
constexpr bool has_instance(int s, int d, int n) {
  if (!typed(s) || !typed(d)) return false;
  if (n == 1) return s != d;
  if (n != 2 && n != 4) return false;
  return s == d || s == M2N_F32 || d == M2N_F32;
}

template <int S, int D, int N>
int launch(const M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int grid, uint32_t* sync, const uint64_t* signals,
           uint32_t n_signals, uint32_t epoch, int do_signal, cudaStream_t stream) {
  if constexpr (has_instance(S, D, N)) {
    m2n_typed_kernel<S, D, N><<<grid, kTypedThreads, 0, stream>>>(ops, tile_start, n_ops, sync, signals, n_signals, epoch, do_signal);
    return 0;
  } else {
    return -1;
  }
}

template <int S, int D>
int by_nsrc(int n, const M2NOp* ops, const uint32_t* ts, uint32_t n_ops, int grid, uint32_t* sync, const uint64_t* sig,
            uint32_t n_sig, uint32_t epoch, int do_signal, cudaStream_t st) {
  switch (n) {
    case 1: return launch<S, D, 1>(ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    case 2: return launch<S, D, 2>(ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    case 4: return launch<S, D, 4>(ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    default: return -1;
  }
}

template <int S>
int by_dst(int d, int n, const M2NOp* ops, const uint32_t* ts, uint32_t n_ops, int grid, uint32_t* sync, const uint64_t* sig,
           uint32_t n_sig, uint32_t epoch, int do_signal, cudaStream_t st) {
  switch (d) {
    case M2N_F32: return by_nsrc<S, M2N_F32>(n, ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    case M2N_BF16: return by_nsrc<S, M2N_BF16>(n, ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    case M2N_F16: return by_nsrc<S, M2N_F16>(n, ops, ts, n_ops, grid, sync, sig, n_sig, epoch, do_signal, st);
    default: return -1;
  }
}

}  // namespace

extern "C" {

int etha_stream_ctas_per_sm(void) { return kTypedCtasPerSm; }

// Key of the streaming instance that can run `op`: (src dtype << 8) | (dst dtype << 4) | sources, or 0 when the
// op has to stay in the general kernel.
int etha_op_stream_key(const M2NOp* op) {
  if (op->unit_elems != 8 || op->ndim > 1 || op->total_units == 0) return 0;
  if (op->mode == M2N_MODE_CVT) {
    if (op->nsrc != 1 || !has_instance(op->src_dtype, op->dst_dtype, 1)) return 0;
  } else if (op->mode == M2N_MODE_REDUCE) {
    if (op->red_size[1] != 1 || op->red_size[0] != op->nsrc || !has_instance(op->src_dtype, op->dst_dtype, op->nsrc)) return 0;
  } else {
    return 0;
  }
  return (op->src_dtype << 8) | (op->dst_dtype << 4) | op->nsrc;
}

int etha_m2n_typed_launch(const M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int key, int grid, uint32_t* sync_scratch,
                          const uint64_t* signals, uint32_t n_signals, uint32_t epoch, int do_signal, void* stream) {
  const int s = (key >> 8) & 0xf, d = (key >> 4) & 0xf, n = key & 0xf;
  if (grid < 1) grid = 1;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  switch (s) {
    case M2N_F32: rc = by_dst<M2N_F32>(d, n, ops, tile_start, n_ops, grid, sync_scratch, signals, n_signals, epoch, do_signal, st); break;
    case M2N_BF16: rc = by_dst<M2N_BF16>(d, n, ops, tile_start, n_ops, grid, sync_scratch, signals, n_signals, epoch, do_signal, st); break;
    case M2N_F16: rc = by_dst<M2N_F16>(d, n, ops, tile_start, n_ops, grid, sync_scratch, signals, n_signals, epoch, do_signal, st); break;
    default: rc = -1;
  }
  if (rc != 0) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "no streaming kernel instance for key 0x%x", key);
    return -102;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "typed kernel launch: %s", cudaGetErrorString(e));
    return -(int)e - 1000;
  }
  return 0;
}

}  // extern "C"
