// Host-side packer of the device copy table: collapses a strided box, picks the widest aligned access
// unit, validates every pointer range against its registered allocation and emits one `M2NOp`.
// (The reference has no counterpart: it slices tensors in Python and lets ATen choose kernels per chunk,
// src/etha/comm/get_chunks.py:12-19, src/etha/comm/ir.py:101-141.)
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.h"
#include "m2n.h"

namespace {

thread_local char g_err[ETHA_ERR_LEN] = {0};

int error(char* err, int err_len, int code, const char* fmt, ...) {
  char buf[ETHA_ERR_LEN];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  snprintf(g_err, sizeof(g_err), "%s", buf);
  if (err && err_len > 0) snprintf(err, err_len, "%s", buf);
  return code;
}

void magic(uint32_t d, uint32_t* mul, uint32_t* shr) {
  if (d <= 1) { *mul = 0; *shr = 0; return; }
  uint32_t k = 0;
  while ((1ull << k) < d) ++k;  // ceil(log2(d))
  const unsigned p = 31 + k;
  *mul = (uint32_t)((((unsigned __int128)1 << p) + d - 1) / d);
  *shr = p - 32;
}

bool dtype_typed(int dt) { return dt == M2N_F32 || dt == M2N_BF16 || dt == M2N_F16; }

}  // namespace

extern "C" {

char* etha_err_buf(void) { return g_err; }
const char* etha_last_error(void) { return g_err; }
int etha_sizeof_op(void) { return (int)sizeof(M2NOp); }

int etha_op_class(const M2NOp* op) {
  return (op->mode == M2N_MODE_RAW && op->unit_bytes_src == 16 && op->ndim <= 1) ? 0 : 1;
}

int etha_op_bulk_ok(const M2NOp* op) {
  if (etha_op_class(op) != 0 || op->nsrc != 1 || op->ndst < 1 || (op->flags & M2N_FLAG_MULTIMEM)) return 0;
  if (op->ndim == 1 && (uint64_t)op->inner_units * 16 < 512) return 0;  // kMinRowBytes of the TMA kernel
  return 1;
}

uint32_t etha_op_tiles(const M2NOp* op) {
  if (op->total_units == 0) return 0;
  return (op->total_units + op->tile_units - 1) / op->tile_units;
}

int etha_pack_op(const M2NOpSpec* s, M2NOp* o, char* err, int err_len) {
  memset(o, 0, sizeof(*o));
  if (s->ndim < 0 || s->ndim > 8) return error(err, err_len, -1, "ndim %d out of range", s->ndim);
  if (s->nsrc < 1 || s->nsrc > M2N_MAX_SRC) return error(err, err_len, -2, "nsrc %d out of range [1,%d]", s->nsrc, M2N_MAX_SRC);
  if (s->ndst < 1 || s->ndst > M2N_MAX_DST) return error(err, err_len, -3, "ndst %d out of range [1,%d]", s->ndst, M2N_MAX_DST);
  const int es = s->src_itemsize, ed = s->dst_itemsize;
  if (es < 1 || ed < 1) return error(err, err_len, -4, "bad itemsize");

  // 1. drop unit dims, 2. merge neighbours that are contiguous on both sides
  struct Dim { int64_t n, ss, ds; };
  std::vector<Dim> dims;
  bool empty = false;
  for (int i = 0; i < s->ndim; ++i) {
    if (s->shape[i] < 0) return error(err, err_len, -5, "negative extent");
    if (s->shape[i] == 0) empty = true;
    if (s->shape[i] != 1) dims.push_back({s->shape[i], s->src_stride[i], s->dst_stride[i]});
  }
  if (empty) { o->tile_units = 2048; o->nsrc = (uint8_t)s->nsrc; o->ndst = (uint8_t)s->ndst; return 0; }
  for (size_t i = 0; i + 1 < dims.size();) {
    Dim& a = dims[i];
    Dim& b = dims[i + 1];
    if (a.ss == b.ss * b.n && a.ds == b.ds * b.n) {
      b.n *= a.n;
      dims.erase(dims.begin() + i);
      if (i > 0) --i;
    } else {
      ++i;
    }
  }
  int64_t inner_elems = 1;
  if (!dims.empty() && dims.back().ss == 1 && dims.back().ds == 1) {
    inner_elems = dims.back().n;
    dims.pop_back();
  }
  if (dims.size() > M2N_MAX_DIMS)
    return error(err, err_len, -6, "slice needs %zu strided dims, at most %d are supported", dims.size(), M2N_MAX_DIMS);

  // mode
  int mode;
  if (s->nsrc > 1) {
    if (!dtype_typed(s->src_dtype) || !dtype_typed(s->dst_dtype))
      return error(err, err_len, -7, "reduction needs fp32/bf16/fp16 on both sides");
    if ((int64_t)s->red_size[0] * std::max(1, s->red_size[1]) != s->nsrc)
      return error(err, err_len, -8, "reduce levels %d x %d do not cover %d sources", s->red_size[0], s->red_size[1], s->nsrc);
    mode = M2N_MODE_REDUCE;
  } else if (s->src_dtype == s->dst_dtype && es == ed) {
    mode = M2N_MODE_RAW;
  } else {
    if (!dtype_typed(s->src_dtype) || !dtype_typed(s->dst_dtype))
      return error(err, err_len, -9, "conversion between dtype codes %d and %d is not supported", s->src_dtype, s->dst_dtype);
    mode = M2N_MODE_CVT;
  }

  auto aligned_all = [&](uint64_t a_src, uint64_t a_dst) {
    for (int i = 0; i < s->nsrc; ++i) if (s->src[i] % a_src) return false;
    for (int i = 0; i < s->ndst; ++i) if (s->dst[i] % a_dst) return false;
    for (auto& d : dims) {
      if ((uint64_t)std::llabs(d.ss * es) % a_src) return false;
      if ((uint64_t)std::llabs(d.ds * ed) % a_dst) return false;
    }
    return true;
  };

  uint32_t unit_elems = 1, ubs = es, ubd = ed;
  int64_t inner_units;
  if (mode == M2N_MODE_RAW) {
    const int64_t inner_bytes = inner_elems * es;
    uint32_t ub = 16;
    while (ub > 1 && !(inner_bytes % ub == 0 && aligned_all(ub, ub))) ub >>= 1;
    ubs = ubd = ub;
    inner_units = inner_bytes / ub;
    unit_elems = (uint32_t)std::max<int64_t>(1, ub / es);
  } else {
    if (inner_elems % 8 == 0 && aligned_all(16, 16)) unit_elems = 8;
    ubs = unit_elems * es;
    ubd = unit_elems * ed;
    inner_units = inner_elems / unit_elems;
  }
  // a multicast destination is written 16 bytes at a time: bit copies in 16-byte units, typed ops in 8-element units
  if ((s->flags & M2N_FLAG_MULTIMEM) &&
      !(s->ndst == 1 && ((mode == M2N_MODE_RAW && ubs == 16) || (mode != M2N_MODE_RAW && unit_elems == 8))))
    return error(err, err_len, -10, "multicast store needs 16-byte aligned units and one (multicast) destination");

  int64_t total = inner_units;
  for (auto& d : dims) {
    total *= d.n;
    if (total >= (1ll << 31)) return error(err, err_len, -11, "op has too many units; split it");
    if (d.n >= (1ll << 31)) return error(err, err_len, -11, "extent too large");
  }
  if (inner_units >= (1ll << 31) || total >= (1ll << 31)) return error(err, err_len, -11, "op has too many units; split it");

  // bounds: every byte touched must lie inside the registered allocation of its pointer
  int64_t s_lo = 0, s_hi = inner_elems * es, d_lo = 0, d_hi = inner_elems * ed;
  for (auto& d : dims) {
    const int64_t ss = d.ss * es * (d.n - 1), ds = d.ds * ed * (d.n - 1);
    (ss < 0 ? s_lo : s_hi) += ss;
    (ds < 0 ? d_lo : d_hi) += ds;
  }
  for (int i = 0; i < s->nsrc; ++i) {
    if (!s->src[i]) return error(err, err_len, -12, "null source pointer %d", i);
    if (s->src_hi[i] && ((int64_t)s->src[i] + s_lo < (int64_t)s->src_lo[i] || s->src[i] + (uint64_t)s_hi > s->src_hi[i]))
      return error(err, err_len, -13, "source %d reads [%lld,%lld) outside its allocation", i, (long long)s_lo, (long long)s_hi);
  }
  for (int i = 0; i < s->ndst; ++i) {
    if (!s->dst[i]) return error(err, err_len, -12, "null destination pointer %d", i);
    if (s->dst_hi[i] && ((int64_t)s->dst[i] + d_lo < (int64_t)s->dst_lo[i] || s->dst[i] + (uint64_t)d_hi > s->dst_hi[i]))
      return error(err, err_len, -14, "destination %d writes [%lld,%lld) outside its allocation", i, (long long)d_lo, (long long)d_hi);
  }

  for (int i = 0; i < s->nsrc; ++i) o->src[i] = s->src[i];
  for (int i = 0; i < s->ndst; ++i) o->dst[i] = s->dst[i];
  o->ndim = (uint8_t)dims.size();
  for (size_t i = 0; i < dims.size(); ++i) {
    o->extent[i] = (uint32_t)dims[i].n;
    o->src_stride[i] = dims[i].ss * es;
    o->dst_stride[i] = dims[i].ds * ed;
    magic((uint32_t)dims[i].n, &o->div_mul[i], &o->div_shr[i]);
  }
  magic((uint32_t)inner_units, &o->div_mul[M2N_MAX_DIMS], &o->div_shr[M2N_MAX_DIMS]);
  o->inner_units = (uint32_t)inner_units;
  o->total_units = (uint32_t)total;
  o->unit_bytes_src = ubs;
  o->unit_bytes_dst = ubd;
  o->unit_elems = (uint8_t)unit_elems;
  o->nsrc = (uint8_t)s->nsrc;
  o->ndst = (uint8_t)s->ndst;
  o->mode = (uint8_t)mode;
  o->src_dtype = (uint8_t)s->src_dtype;
  o->dst_dtype = (uint8_t)s->dst_dtype;
  o->flags = (uint8_t)s->flags;
  o->red_size[0] = (uint8_t)std::max(1, s->red_size[0]);
  o->red_size[1] = (uint8_t)std::max(1, s->red_size[1]);
  o->red_op[0] = (uint8_t)s->red_op[0];
  o->red_op[1] = (uint8_t)s->red_op[1];
  const int64_t tile_bytes = s->tile_bytes > 0 ? s->tile_bytes : 65536;
  int64_t tu = (tile_bytes + ubd - 1) / ubd;
  tu = ((tu + 2047) / 2048) * 2048;
  o->tile_units = (uint32_t)std::min<int64_t>(tu, 1ll << 30);
  return 0;
}

}  // extern "C"
