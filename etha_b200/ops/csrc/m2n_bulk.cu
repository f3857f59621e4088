// TMA variant of the fast copy class: cp.async.bulk global -> shared -> global through a ring of stages.
//
// One warp per CTA drives the copy engine: for every 32 KiB stage the lanes compute the (at most one per
// matrix row) contiguous pieces of the stage in parallel, one lane arms the stage's mbarrier with the byte
// count and every lane issues its pieces as untiled bulk loads; when the barrier completes the same pieces
// are written out with bulk stores from shared memory.  Loads run several stages ahead of the stores, so
// well over 100 KiB per SM are in flight with almost no instruction issue.  No cluster, no multicast.
//
// Loads always read this GPU's own memory; the stores go to local memory, to a peer's memory over NVLink
// (plain non-multicast bulk stores to the mapped peer address) or to several replicas one after the other
// (a Replicate fan-out: the stage is read from HBM once and stored once per destination).  Every address
// and size handed to the copy engine is a multiple of 16 bytes: the table packer admits only 16-byte units
// with 16-byte aligned bases and strides into this class.  A side that is contiguous over the whole fill is
// moved with ONE bulk copy per stage instead of one per matrix row.
// Waits on the barriers are bounded: after the limit the CTA records an error word, drains its own stores
// and returns.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "common.h"
#include "m2n.h"

namespace {

#ifndef ETHA_BULK_STAGES
#define ETHA_BULK_STAGES 6
#endif
#ifndef ETHA_BULK_STAGE_KB
#define ETHA_BULK_STAGE_KB 32
#endif
constexpr int kStages = ETHA_BULK_STAGES;
constexpr uint32_t kStageBytes = ETHA_BULK_STAGE_KB * 1024;
constexpr uint32_t kMinRowBytes = 512;  // shortest matrix row the packer admits into this class
// store pieces (row fragments) per stage: a fill that starts and ends inside a row touches one row more than
// stage bytes / row bytes; the kernel still checks every fill against this bound before it issues anything
constexpr int kMaxPieces = kStageBytes / kMinRowBytes + 2;

struct StageMeta {
  int64_t dof[kMaxPieces];  // byte offset of the piece inside every destination slice
  uint32_t off[kMaxPieces];
  uint32_t bytes[kMaxPieces];
  uint32_t npieces;
  uint32_t op;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

// where fill `f` of this CTA lives: (tile, first unit, one-past-last unit)
struct FillPos {
  uint32_t op, u0, u1;
};

__device__ __forceinline__ uint32_t find_op(const uint32_t* __restrict__ tile_start, uint32_t n_ops, uint32_t tile) {
  uint32_t lo = 0, hi = n_ops;
  while (hi - lo > 1) {
    uint32_t mid = (lo + hi) >> 1;
    if (tile_start[mid] <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(32, 1)
m2n_bulk_kernel(const M2NOp* __restrict__ ops, const uint32_t* __restrict__ tile_start, uint32_t n_ops, uint32_t* sync,
                const uint64_t* __restrict__ signals, uint32_t n_signals, uint32_t epoch, int do_signal) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* stage_buf = smem;  // kStages * kStageBytes
  StageMeta* meta = reinterpret_cast<StageMeta*>(smem + kStages * kStageBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(meta + kStages);
  const uint32_t lane = threadIdx.x;
  const uint32_t total_tiles = n_ops ? tile_start[n_ops] : 0;

  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // ---- iterator over this CTA's fills (a tile is cut into stage-sized fills) ------------------------
  uint32_t it_tile = blockIdx.x, it_op = 0, it_u = 0, it_limit = 0;
  bool it_open = false;
  auto next_fill = [&](FillPos& out) -> bool {
    while (true) {
      if (!it_open) {
        if (it_tile >= total_tiles) return false;
        it_op = find_op(tile_start, n_ops, it_tile);
        const M2NOp& op = ops[it_op];
        it_u = (it_tile - tile_start[it_op]) * op.tile_units;
        it_limit = min(op.total_units, it_u + op.tile_units);
        it_open = true;
      }
      if (it_u < it_limit) {
        out.op = it_op;
        out.u0 = it_u;
        out.u1 = min(it_limit, it_u + kStageBytes / 16);
        it_u = out.u1;
        return true;
      }
      it_open = false;
      it_tile += gridDim.x;
    }
  };

  // issue the loads of one fill into stage s (all lanes), record the matching stores; returns false (nothing
  // issued, error word set) if the fill would need more store pieces than the stage's table holds
  auto issue_loads = [&](const FillPos& f, int s) -> bool {
    const M2NOp& op = ops[f.op];
    const bool rows = op.ndim != 0;
    const uint32_t inner = rows ? op.inner_units : 0xffffffffu;
    const uint32_t r0 = rows ? f.u0 / inner : 0;
    const uint32_t r1 = rows ? (f.u1 - 1) / inner : 0;
    const uint32_t nrows = r1 - r0 + 1;
    const bool src_flat = !rows || op.src_stride[0] == (int64_t)inner * 16;
    const bool dst_flat = !rows || op.dst_stride[0] == (int64_t)inner * 16;
    const uint32_t n_store = dst_flat ? 1u : nrows;
    if (n_store > (uint32_t)kMaxPieces) {
      if (lane == 0) sync[1] = M2N_BAD_OP;
      return false;
    }
    StageMeta& m = meta[s];
    unsigned char* buf = stage_buf + (size_t)s * kStageBytes;
    if (lane == 0) {
      m.npieces = n_store;
      m.op = f.op;
      mbar_expect_tx(&full[s], (f.u1 - f.u0) * 16);
    }
    __syncwarp();
    if (dst_flat) {
      if (lane == 0) { m.dof[0] = (int64_t)f.u0 * 16; m.off[0] = 0; m.bytes[0] = (f.u1 - f.u0) * 16; }
    }
    if (src_flat) {
      if (lane == 0) bulk_load(buf, reinterpret_cast<const char*>(op.src[0]) + (int64_t)f.u0 * 16, (f.u1 - f.u0) * 16, &full[s]);
    }
    if (!(src_flat && dst_flat)) {
      for (uint32_t k = lane; k < nrows; k += 32) {
        const uint32_t row = r0 + k;
        const uint32_t a = max(f.u0, row * inner);
        const uint32_t b = min(f.u1, (row + 1) * inner);
        const uint32_t col = a - row * inner;
        const uint32_t off = (a - f.u0) * 16, bytes = (b - a) * 16;
        if (!dst_flat) {
          m.dof[k] = (int64_t)col * 16 + (int64_t)row * op.dst_stride[0];
          m.off[k] = off;
          m.bytes[k] = bytes;
        }
        if (!src_flat)
          bulk_load(buf + off, reinterpret_cast<const char*>(op.src[0]) + (int64_t)col * 16 + (int64_t)row * op.src_stride[0],
                    bytes, &full[s]);
      }
    }
    __syncwarp();
    return true;
  };

  FillPos pos;
  uint32_t issued = 0, consumed = 0;
  bool more = true;
  bool failed = false;
  // prologue: run kStages-1 fills ahead
  while (issued < kStages - 1 && (more = next_fill(pos))) {
    if (!issue_loads(pos, issued % kStages)) { more = false; break; }
    ++issued;
  }
  while (consumed < issued) {
    const int s = consumed % kStages;
    const uint32_t parity = (consumed / kStages) & 1;
    // bounded wait for the stage's loads
    bool ready = false;
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
      if (mbar_try_wait(&full[s], parity)) { ready = true; break; }
      if (spin > 64) __nanosleep(64);
    }
    ready = __all_sync(0xffffffffu, ready);
    if (!ready) { failed = true; break; }
    const StageMeta& m = meta[s];
    const uint32_t np = m.npieces;
    const M2NOp& sop = ops[m.op];
    const uint32_t nd = sop.ndst;
    // piece k of destination j: the lanes walk the (destination, piece) pairs
    for (uint32_t i = lane; i < np * nd; i += 32) {
      const uint32_t j = i / np, k = i - j * np;
      bulk_store(reinterpret_cast<char*>(sop.dst[j]) + m.dof[k], stage_buf + (size_t)s * kStageBytes + m.off[k], m.bytes[k]);
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    ++consumed;
    // the stage used one fill earlier may be refilled once its stores have read shared memory
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
    if (more && (more = next_fill(pos))) {
      if (issue_loads(pos, issued % kStages)) ++issued; else more = false;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
  if (failed && lane == 0) sync[1] = M2N_TIMEOUT;

  // ---- completion: same protocol as the LD/ST kernels -------------------------------------------------
  if (do_signal) {
    __syncwarp();
    uint32_t last = 0;
    if (lane == 0) {
      __threadfence_system();
      last = (atomicAdd(&sync[0], 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      if (lane == 0) sync[0] = 0;
      __threadfence_system();
      for (uint32_t i = lane; i < n_signals; i += 32) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(signals[i]);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
      }
    }
  }
}

}  // namespace

extern "C" int etha_m2n_bulk_launch(const M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int grid,
                                    uint32_t* sync_scratch, const uint64_t* signals, uint32_t n_signals, uint32_t epoch,
                                    int do_signal, void* stream) {
  static bool configured[64] = {false};
  const size_t smem = (size_t)kStages * kStageBytes + kStages * sizeof(StageMeta) + kStages * sizeof(uint64_t) + 128;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(m2n_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      snprintf(etha_err_buf(), ETHA_ERR_LEN, "bulk kernel shared memory opt-in: %s", cudaGetErrorString(e));
      return -(int)e - 1000;
    }
    configured[dev] = true;
  }
  if (grid < 1) grid = 1;
  m2n_bulk_kernel<<<grid, 32, smem, (cudaStream_t)stream>>>(ops, tile_start, n_ops, sync_scratch, signals, n_signals, epoch,
                                                            do_signal);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(etha_err_buf(), ETHA_ERR_LEN, "bulk kernel launch: %s", cudaGetErrorString(e));
    return -(int)e - 1000;
  }
  return 0;
}
