// Device copy table and C entry points of the M-to-N redistribution kernels (sm_100a).
//
// One `M2NOp` describes the delivery of one cell: up to `M2N_MAX_SRC` source slices (one for a plain
// copy, several when a Partial source is collapsed on the fly) and up to `M2N_MAX_DST` destination
// slices (one for a point-to-point route, several for a Replicate fan-out).  Pointers may be local,
// peer (CUDA IPC / VMM mappings of another GPU) or an NVLS multicast address.  The slice is a
// strided box of at most `M2N_MAX_DIMS` outer dims times one contiguous inner run, expressed in
// "units" (a unit is `unit_elems` elements, sized so that every access is one aligned vector).
//
// The reference moves the same data with ATen gather/cast/pack kernels plus NCCL send/recv/
// broadcast/all-reduce (src/etha/comm/ir.py:101-141,229-284, src/etha/comm/transfer.py:20-41).
#pragma once
#include <stdint.h>

#define M2N_MAX_SRC 8
#define M2N_MAX_DST 8
#define M2N_MAX_DIMS 4

// element types the kernels can convert between / reduce over
enum M2NDtype : uint8_t { M2N_RAW = 0, M2N_F32 = 1, M2N_BF16 = 2, M2N_F16 = 3 };
// per-level reduce ops of a Partial source
enum M2NReduce : uint8_t { M2N_SUM = 0, M2N_AVG = 1, M2N_MAX = 2, M2N_MIN = 3, M2N_PROD = 4 };
// how a tile of the op is executed
enum M2NMode : uint8_t {
  M2N_MODE_RAW = 0,     // bit copy, unit = `unit_bytes_src` bytes (16, 8, 4, 2 or 1)
  M2N_MODE_CVT = 1,     // typed copy with conversion, unit = `unit_elems` elements (8 or 1)
  M2N_MODE_REDUCE = 2,  // several typed sources, fp32 accumulation, one rounding
};
enum M2NFlags : uint8_t { M2N_FLAG_MULTIMEM = 1 };  // dst[0] is an NVLS multicast address

struct __attribute__((aligned(16))) M2NOp {
  uint64_t src[M2N_MAX_SRC];
  uint64_t dst[M2N_MAX_DST];
  int64_t src_stride[M2N_MAX_DIMS];  // bytes, outer dims, slowest first
  int64_t dst_stride[M2N_MAX_DIMS];  // bytes
  uint32_t extent[M2N_MAX_DIMS];     // outer extents
  uint32_t div_mul[M2N_MAX_DIMS + 1];  // magic numbers: [0..3] outer extents, [4] inner units
  uint32_t div_shr[M2N_MAX_DIMS + 1];
  uint32_t inner_units;  // units per contiguous inner run
  uint32_t total_units;  // < 2^31
  uint32_t tile_units;   // units per tile
  uint32_t unit_bytes_src;
  uint32_t unit_bytes_dst;
  uint8_t ndim;  // number of outer dims in use
  uint8_t nsrc, ndst;
  uint8_t mode;
  uint8_t src_dtype, dst_dtype;
  uint8_t unit_elems;
  uint8_t flags;
  uint8_t red_size[2];  // Partial levels: group sizes (level 0 varies fastest); red_size[1] == 1 if one level
  uint8_t red_op[2];
  uint32_t pad_[5];
};

// status codes written by the kernels (never a trap)
enum M2NStatus : uint32_t { M2N_OK = 0, M2N_TIMEOUT = 1, M2N_BAD_OP = 2 };

#ifdef __cplusplus
extern "C" {
#endif

// ---- table packer (host) --------------------------------------------------------------------
// Describes one op before collapsing: element strides, full shapes. Returns 0 or a negative error code and
// fills `out` (host memory). `err` receives a message (may be null).
struct M2NOpSpec {
  int32_t ndim;
  int64_t shape[8];
  int64_t src_stride[8];  // elements
  int64_t dst_stride[8];  // elements
  int32_t src_itemsize, dst_itemsize;
  int32_t src_dtype, dst_dtype;  // M2NDtype
  int32_t nsrc, ndst;
  uint64_t src[M2N_MAX_SRC];
  uint64_t dst[M2N_MAX_DST];
  // allocation bounds of every pointer, for validation: [lo, hi)
  uint64_t src_lo[M2N_MAX_SRC], src_hi[M2N_MAX_SRC];
  uint64_t dst_lo[M2N_MAX_DST], dst_hi[M2N_MAX_DST];
  int32_t red_size[2];
  int32_t red_op[2];
  int32_t flags;
  int32_t tile_bytes;  // target bytes (destination side) per tile
};
int etha_pack_op(const struct M2NOpSpec* spec, struct M2NOp* out, char* err, int err_len);
uint32_t etha_op_tiles(const struct M2NOp* op);
int etha_sizeof_op(void);
int etha_op_class(const struct M2NOp* op);  // 0 = fast kernel, 1 = general kernel

// ---- launches ---------------------------------------------------------------------------------
// `ops`/`tile_start` are device arrays (`tile_start` has n_ops+1 entries) holding ops of ONE class
// (see etha_op_class): `general == 0` 16-byte bit copies of a run or of matrix rows, `general == 1` everything
// else (narrower bit copies, boxes with more strided dims, conversions, reductions). With `do_signal`, after
// the last CTA finishes every address in `signals` (device array of `n_signals` pointers to uint32 flags,
// local or peer) is set to `epoch` with system-scope release semantics. `sync_scratch` is a zero-initialised
// device uint32[2] owned by this table (CTA arrival counter + error word).
int etha_m2n_launch(const struct M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int general, int grid,
                    int block, uint32_t* sync_scratch, const uint64_t* signals, uint32_t n_signals, uint32_t epoch,
                    int do_signal, void* stream);
// Bounded wait: one thread per flag polls until `*flag >= epoch` or `timeout_ns` passed; writes
// M2N_OK/M2N_TIMEOUT and the index of the first missing flag to `status[0..1]` (device or mapped host memory).
int etha_wait_flags(const uint32_t* flags, const uint32_t* which, uint32_t n, uint32_t epoch, uint64_t timeout_ns,
                    uint32_t* status, void* stream);
int etha_set_flags(const uint64_t* signals, uint32_t n_signals, uint32_t epoch, void* stream);

// TMA (cp.async.bulk) variant of the fast class: bulk loads from this GPU's own memory into a shared-memory
// ring, bulk stores (never multicast) to local or peer destinations. Every op of the table must satisfy
// etha_op_bulk_ok (16-byte bit copy, one source, one or more plain destinations, at most one strided dim whose
// rows are at least 512 bytes). One warp per CTA; `grid` is normally the SM count.
int etha_op_bulk_ok(const struct M2NOp* op);
int etha_m2n_bulk_launch(const struct M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int grid,
                         uint32_t* sync_scratch, const uint64_t* signals, uint32_t n_signals, uint32_t epoch,
                         int do_signal, void* stream);

// Streaming class of the typed ops (m2n_typed.cu): conversions and single-level collapses of 2 or 4 sources over
// one-run / matrix-row boxes in 8-element units, one kernel instance per key. `etha_op_stream_key` returns the key
// of the instance that can run `op` ((src dtype << 8) | (dst dtype << 4) | sources) or 0; every op of a table
// handed to `etha_m2n_typed_launch` must have that key. Other arguments as etha_m2n_launch.
int etha_op_stream_key(const struct M2NOp* op);
int etha_stream_ctas_per_sm(void);
int etha_m2n_typed_launch(const struct M2NOp* ops, const uint32_t* tile_start, uint32_t n_ops, int key, int grid,
                          uint32_t* sync_scratch, const uint64_t* signals, uint32_t n_signals, uint32_t epoch, int do_signal,
                          void* stream);

// ---- copy-engine lowering (dma_graph.cu) -------------------------------------------------------
// One DMA copy: `height` rows of `width` bytes, `spitch` / `dpitch` bytes between rows (height 1: one run).
struct EthaDmaCopy {
  uint64_t dst, src, width, height, dpitch, spitch;
};
int etha_op_dma_copies(const struct M2NOp* op, struct EthaDmaCopy* out);  // copies written (0: needs a kernel)
int etha_dma_plan_create(const struct EthaDmaCopy* copies, uint32_t n, int use_graph, int n_streams, void** out);
int etha_dma_plan_launch(void* plan, void* stream);  // copies start after the work on `stream`, on side streams
int etha_dma_plan_join(void* plan, void* stream);    // `stream` waits for them
int etha_dma_plan_destroy(void* plan);

// ---- IPC / device helpers ---------------------------------------------------------------------
int etha_ipc_export(uint64_t ptr, unsigned char* handle64, uint64_t* base, uint64_t* size);
int etha_ipc_open(const unsigned char* handle64, uint64_t* mapped_base);
int etha_ipc_close(uint64_t mapped_base);
int etha_copy_engine_d2d(uint64_t dst, uint64_t src, uint64_t bytes, void* stream);
int etha_enable_peer_access(int peer_device);
int etha_device_info(int* sm_count, int* cc_major, int* cc_minor, int* multicast_supported);
const char* etha_last_error(void);

#ifdef __cplusplus
}
#endif
