// Copy-engine lowering of the copy table: the large bit copies of a transfer (one contiguous run, or rows of a
// matrix with a pitch on either side) become memcpy nodes of one CUDA graph that is built when a batch is
// registered and launched once per transfer.  The DMA engines write NVLink packets of twice the payload an SM
// store or a TMA bulk store can produce, so on the same bytes they deliver about 10 % more than the copy
// kernels; the kernels keep everything a DMA engine cannot do (conversion, Partial collapse, boxes with more
// strided dims, multicast stores, the many small messages) and publish the completion flags afterwards.
// Nodes have no edges between them, so the driver spreads them over the device's copy engines.
//
// The reference moves the same chunks one NCCL send/recv at a time (src/etha/comm/transfer.py:20-30,
// src/etha/comm/comm_methods.py:81-117).
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <vector>

#include "common.h"
#include "m2n.h"

namespace {

int fail(cudaError_t e, const char* what) {
  snprintf(etha_err_buf(), ETHA_ERR_LEN, "%s: %s", what, cudaGetErrorString(e));
  return -(int)e - 1000;
}

struct DmaPlan {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  std::vector<EthaDmaCopy> copies;    // kept for the stream fallback
  std::vector<cudaStream_t> streams;  // stream fallback: copies are dealt round-robin over these
  std::vector<cudaEvent_t> done;
  cudaEvent_t fork = nullptr;
  cudaStream_t branch = nullptr;  // the graph runs here so that kernels on the caller's stream overlap with it
  cudaEvent_t joined = nullptr;
};

void destroy(DmaPlan* p) {
  if (!p) return;
  if (p->exec) cudaGraphExecDestroy(p->exec);
  if (p->graph) cudaGraphDestroy(p->graph);
  for (auto e : p->done) cudaEventDestroy(e);
  for (auto s : p->streams) cudaStreamDestroy(s);
  if (p->fork) cudaEventDestroy(p->fork);
  if (p->joined) cudaEventDestroy(p->joined);
  if (p->branch) cudaStreamDestroy(p->branch);
  delete p;
}

}  // namespace

extern "C" {

// Copies an op can be lowered to: one per destination, or 0 if the op needs a kernel (conversion, reduction,
// more than one strided dim, negative or overlapping pitches, multicast destination).  `out` has room for
// M2N_MAX_DST entries.
int etha_op_dma_copies(const M2NOp* op, EthaDmaCopy* out) {
  if (op->mode != M2N_MODE_RAW || op->nsrc != 1 || op->ndim > 1 || (op->flags & M2N_FLAG_MULTIMEM) || op->total_units == 0)
    return 0;
  const uint64_t width = (uint64_t)op->inner_units * op->unit_bytes_src;
  uint64_t height = 1, spitch = width, dpitch = width;
  if (op->ndim == 1) {
    if (op->src_stride[0] < (int64_t)width || op->dst_stride[0] < (int64_t)width) return 0;
    height = op->extent[0];
    spitch = (uint64_t)op->src_stride[0];
    dpitch = (uint64_t)op->dst_stride[0];
  }
  for (int j = 0; j < op->ndst; ++j) out[j] = EthaDmaCopy{op->dst[j], op->src[0], width, height, dpitch, spitch};
  return op->ndst;
}

// Builds the plan.  `use_graph` != 0: one graph of independent memcpy nodes; 0: the same copies issued as
// asynchronous copies over `n_streams` internal streams at every launch.
int etha_dma_plan_create(const EthaDmaCopy* copies, uint32_t n, int use_graph, int n_streams, void** out) {
  *out = nullptr;
  DmaPlan* p = new DmaPlan();
  p->copies.assign(copies, copies + n);
  cudaError_t e = cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->joined, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->branch, cudaStreamNonBlocking);
  if (e != cudaSuccess) { destroy(p); return fail(e, "branch stream of the copy plan"); }
  if (use_graph) {
    e = cudaGraphCreate(&p->graph, 0);
    if (e != cudaSuccess) { destroy(p); return fail(e, "cudaGraphCreate"); }
    for (uint32_t i = 0; i < n; ++i) {
      const EthaDmaCopy& c = copies[i];
      cudaGraphNode_t node;
      if (c.height == 1) {
        e = cudaGraphAddMemcpyNode1D(&node, p->graph, nullptr, 0, reinterpret_cast<void*>(c.dst),
                                     reinterpret_cast<const void*>(c.src), c.width, cudaMemcpyDeviceToDevice);
      } else {
        cudaMemcpy3DParms m = {};
        m.srcPtr = make_cudaPitchedPtr(reinterpret_cast<void*>(c.src), c.spitch, c.width, c.height);
        m.dstPtr = make_cudaPitchedPtr(reinterpret_cast<void*>(c.dst), c.dpitch, c.width, c.height);
        m.extent = make_cudaExtent(c.width, c.height, 1);
        m.kind = cudaMemcpyDeviceToDevice;
        e = cudaGraphAddMemcpyNode(&node, p->graph, nullptr, 0, &m);
      }
      if (e != cudaSuccess) { destroy(p); return fail(e, "cudaGraphAddMemcpyNode"); }
    }
    e = cudaGraphInstantiate(&p->exec, p->graph, 0);
    if (e != cudaSuccess) { destroy(p); return fail(e, "cudaGraphInstantiate"); }
  } else {
    if (n_streams < 1) n_streams = 1;
    if (n_streams > 32) n_streams = 32;
    for (int k = 0; k < n_streams; ++k) {
      cudaStream_t s;
      cudaEvent_t ev;
      e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
      if (e != cudaSuccess) { destroy(p); return fail(e, "cudaStreamCreate"); }
      p->streams.push_back(s);
      e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
      if (e != cudaSuccess) { destroy(p); return fail(e, "cudaEventCreate"); }
      p->done.push_back(ev);
    }
  }
  *out = p;
  return 0;
}

// Starts every copy of the plan after the work already on `stream`, on side streams: what the caller enqueues on
// `stream` next (the copy kernels) runs concurrently with the DMA engines.  `etha_dma_plan_join` makes `stream`
// wait for the copies; the completion flags are published after it.
int etha_dma_plan_launch(void* plan, void* stream) {
  DmaPlan* p = static_cast<DmaPlan*>(plan);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaEventRecord(p->fork, s);
  if (e != cudaSuccess) return fail(e, "cudaEventRecord");
  if (p->exec) {
    e = cudaStreamWaitEvent(p->branch, p->fork, 0);
    if (e == cudaSuccess) e = cudaGraphLaunch(p->exec, p->branch);
    if (e == cudaSuccess) e = cudaEventRecord(p->joined, p->branch);
    return e == cudaSuccess ? 0 : fail(e, "cudaGraphLaunch");
  }
  const size_t ns = p->streams.size();
  for (size_t k = 0; k < ns; ++k) {
    e = cudaStreamWaitEvent(p->streams[k], p->fork, 0);
    if (e != cudaSuccess) return fail(e, "cudaStreamWaitEvent");
  }
  for (size_t i = 0; i < p->copies.size(); ++i) {
    const EthaDmaCopy& c = p->copies[i];
    cudaStream_t cs = p->streams[i % ns];
    if (c.height == 1)
      e = cudaMemcpyAsync(reinterpret_cast<void*>(c.dst), reinterpret_cast<const void*>(c.src), c.width,
                          cudaMemcpyDeviceToDevice, cs);
    else
      e = cudaMemcpy2DAsync(reinterpret_cast<void*>(c.dst), c.dpitch, reinterpret_cast<const void*>(c.src), c.spitch, c.width,
                            c.height, cudaMemcpyDeviceToDevice, cs);
    if (e != cudaSuccess) return fail(e, "cudaMemcpy(2D)Async");
  }
  for (size_t k = 0; k < ns; ++k) {
    e = cudaEventRecord(p->done[k], p->streams[k]);
    if (e != cudaSuccess) return fail(e, "cudaEventRecord");
  }
  return 0;
}

int etha_dma_plan_join(void* plan, void* stream) {
  DmaPlan* p = static_cast<DmaPlan*>(plan);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (p->exec) {
    e = cudaStreamWaitEvent(s, p->joined, 0);
  } else {
    for (size_t k = 0; k < p->done.size() && e == cudaSuccess; ++k) e = cudaStreamWaitEvent(s, p->done[k], 0);
  }
  return e == cudaSuccess ? 0 : fail(e, "join of the copy streams");
}

int etha_dma_plan_destroy(void* plan) {
  destroy(static_cast<DmaPlan*>(plan));
  return 0;
}

}  // extern "C"
