// C ABI of libnvnorms (include/nvnorms.h): argument checking, the dispatch
// table that maps a problem (dtype, N, C, D, layout, alignment) to a kernel
// variant, workspace carving and the launches.
//
// Takes the place of the host halves of the reference functors
// (atex/nv_norms/cc/kernels/fused_layer_norm_op.cu:805-1030,
//  atex/nv_norms/cc/kernels/fused_instance_norm_op.cu:820-906, 1203-1561) and of
// the shape bookkeeping in the OpKernels (fused_layer_norm_op.cc:252-282,
// fused_instance_norm_op.cc:25-34, 333-376).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/nvnorms.h"
#include "nvn_host.h"
#include "twophase.h"

namespace nvn {

namespace {
std::atomic<uint64_t> g_launches{0};
thread_local int t_last_cuda_error = 0;
std::atomic<int> g_sm_count{0};

struct Shape {
  int tpr, vpt, cs, pf;
};
#define X(I, TPR, VPT, CS, RB, PR, MINB, PF) {TPR, VPT, CS, PF},
const Shape kLightShapes[] = {NVN_ROW_SHAPES_LIGHT(X)};
const Shape kHeavyShapes[] = {NVN_ROW_SHAPES_HEAVY(X)};
const Shape kScalarShapes[] = {NVN_ROW_SHAPES_SCALAR(X)};
const Shape kAffineWideShapes[] = {NVN_ROW_SHAPES_AFFINE_WIDE(X)};
#undef X
constexpr int kNumLight = sizeof(kLightShapes) / sizeof(Shape);
constexpr int kNumHeavy = sizeof(kHeavyShapes) / sizeof(Shape);
constexpr int kNumScalar = sizeof(kScalarShapes) / sizeof(Shape);
constexpr int kNumAffineWide = sizeof(kAffineWideShapes) / sizeof(Shape);

inline int64_t cap(const Shape& s) { return static_cast<int64_t>(s.tpr) * s.vpt * s.cs; }

// Bytes per tensor from which a held-ring shape is preferred over its register-prefetch
// twin (between [4096, 1024] fp32, 17 MB, where the twin is 25 % faster, and
// [65536, 2048] bf16, 268 MB, where the held ring is 15 % faster).
constexpr int64_t kHeldRingMinBytes = 64ll << 20;

// The one experiment switch of the library, off by default: the environment variable
// NVN_FORCE_VARIANT, read once when the library is first used, holds comma-separated
// key=value pairs that override the dispatcher for profiler and tuning runs:
//   wide=twophase|cluster   path of contiguous rows that need a thread-block cluster
//   nlc=twophase|onchip|stream   channels-last InstanceNorm: skip the on-chip and / or
//                           the warp-per-item kernels; `stream` sends every eligible
//                           shape, whatever its size, to the persistent kernel
//   fwd_shape=I bwd_shape=I affine_shape=I   index into the shape tables of nvn_host.h
//                           (used when that shape is large enough for the row)
//   wide_fwd=I wide_bwd=I   index into the shape tables of rows_wide.cu (used when the row
//                           fills that shape)
//   stream_block=256|512    persistent channels-last kernels: threads per CTA
//   stream_groups=K         persistent channels-last kernels: CTA groups (1 to 8)
//   pdl=0                   launch the row kernels without programmatic stream serialization
struct Variant {
  int wide = 0;  // 0 default, 1 two-phase, 2 cluster
  int nlc = 0;   // 0 default, 1 two-phase, 2 on-chip but no warp-per-item, 3 persistent
  int fwd_shape = -1, bwd_shape = -1, affine_shape = -1;
  int wide_fwd = -1, wide_bwd = -1;
  int stream_block = 0;  // persistent channels-last kernels: threads per CTA (256 or 512)
  int stream_groups = 0; // persistent channels-last kernels: CTA groups (0: by item size)
  int pdl = 1;           // programmatic dependent launch of the row kernels
};

const Variant& variant() {
  static const Variant v = [] {
    Variant r;
    const char* env = getenv("NVN_FORCE_VARIANT");
    if (env == nullptr) return r;
    std::string text(env);
    size_t pos = 0;
    while (pos < text.size()) {
      size_t end = text.find(',', pos);
      if (end == std::string::npos) end = text.size();
      const std::string item = text.substr(pos, end - pos);
      pos = end + 1;
      const size_t eq = item.find('=');
      if (eq == std::string::npos) continue;
      const std::string key = item.substr(0, eq), val = item.substr(eq + 1);
      if (key == "wide") r.wide = val == "twophase" ? 1 : (val == "cluster" ? 2 : 0);
      if (key == "nlc")
        r.nlc = val == "twophase" ? 1 : (val == "onchip" ? 2 : (val == "stream" ? 3 : 0));
      if (key == "fwd_shape") r.fwd_shape = atoi(val.c_str());
      if (key == "bwd_shape") r.bwd_shape = atoi(val.c_str());
      if (key == "affine_shape") r.affine_shape = atoi(val.c_str());
      if (key == "wide_fwd") r.wide_fwd = atoi(val.c_str());
      if (key == "wide_bwd") r.wide_bwd = atoi(val.c_str());
      if (key == "stream_block") r.stream_block = atoi(val.c_str());
      if (key == "stream_groups") r.stream_groups = atoi(val.c_str());
      if (key == "pdl") r.pdl = atoi(val.c_str());
    }
    return r;
  }();
  return v;
}

// Smallest capacity that holds `nvec` vectors; among equals the first listed, skipping
// held-ring entries for problems of less than kHeldRingMinBytes per tensor.  `forced` (a
// table index from NVN_FORCE_VARIANT, or -1) wins when that shape is large enough.
int pick_shape(const Shape* table, int n, int64_t nvec, int64_t tensor_bytes, int forced) {
  if (forced >= 0 && forced < n && cap(table[forced]) >= nvec) return forced;
  int best = -1;
  for (int pass = 0; pass < 2 && best < 0; ++pass) {
    for (int i = 0; i < n; ++i) {
      if (cap(table[i]) < nvec) continue;
      // first pass: leave held rings out for small problems; second pass: anything
      if (pass == 0 && table[i].pf >= 10 && tensor_bytes < kHeldRingMinBytes) continue;
      if (best < 0 || cap(table[i]) < cap(table[best])) best = i;
    }
  }
  return best;
}

inline bool aligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
// Scratch the column reduction may use to split very many partial rows of F features into
// slabs (colreduce.cu); only InstanceNorm over thousands of items gets there.
inline size_t colreduce_scratch_bytes(int64_t partial_rows, int64_t F) {
  return partial_rows >= 4096
             ? align_up(static_cast<size_t>(kColreduceScratchRows) * 2 * F * 4, 256)
             : 0;
}
inline size_t dtype_size(int dtype) { return dtype == NVN_F32 ? 4 : 2; }
inline int full_epv(int dtype) { return dtype == NVN_F32 ? 4 : 8; }

typedef cudaError_t (*RowsFn)(bool, int, int, const RowsArgs&, cudaStream_t, bool, RowsPlan*);

// Largest power-of-two alignment (capped at 16) shared by all the pointers given.
inline size_t common_alignment(std::initializer_list<const void*> ptrs) {
  uintptr_t bits = 0;
  for (const void* p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
  size_t a = 16;
  while (a > 1 && (bits & (a - 1)) != 0) a >>= 1;
  return a;
}

// Elements per access for rows of width D: the widest of (full, full/2, full/4) that
// divides D and fits the alignment, else single elements.
// `align` is the activations' alignment, `par_align` that of the fp32 parameters, which are
// read e floats at a time in accesses of at most 16 bytes.
inline int pick_epv(int dtype, int64_t D, size_t align, size_t par_align) {
  const int V = full_epv(dtype);
  const size_t es = dtype_size(dtype);
  for (int e = V; e >= 2; e >>= 1)
    if (D % e == 0 && e * es <= align && std::min<size_t>(16, e * 4) <= par_align) return e;
  return 1;
}
RowsFn rows_fn(int dtype, bool bwd) {
  switch (dtype) {
    case NVN_F32:
      return bwd ? rows_f32_bwd : rows_f32_fwd;
    case NVN_F16:
      return bwd ? rows_f16_bwd : rows_f16_fwd;
    default:
      return bwd ? rows_bf16_bwd : rows_bf16_fwd;
  }
}

int fail_cuda(cudaError_t e) {
  t_last_cuda_error = static_cast<int>(e);
  (void)cudaGetLastError();
  return NVN_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Plan for a contiguous-row problem ([rows, D], LayerNorm or "NC..." InstanceNorm)
// ---------------------------------------------------------------------------
constexpr int kStreamBlock = 512;  // threads per CTA of the persistent kernels (nlc_stream.cu)
int stream_groups(int dtype, bool bwd, int64_t N, int64_t C, int64_t D);

struct RowProblemPlan {
  bool two_phase;
  bool stream_rows;   // channel-first rows too wide for the row-cached kernels: persistent kernels in row mode
  int stream_groups;
  bool wide;       // LayerNorm rows that fill a shape of the split-barrier cluster kernels
  WidePlan wp;
  size_t off_colscratch;  // slab scratch of the column reduction (0 bytes: none)
  bool has_colscratch;
  bool scalar;     // two-phase variant runs element-wise
  int epv;         // elements per access of the row-cached variant
  int shape;       // row-cached variant
  RowsPlan rows;   // filled by a dry run
  R2Plan r2;       // two-phase variant
  // workspace carving (byte offsets)
  size_t off_part, off_coef, off_colpart, bytes;
  int64_t colpart_rows;  // P of the column reduction (LayerNorm backward / IN backward)
};

// align: alignment shared by every pointer (16 is assumed for size queries).
int plan_rows_uncached(int dtype, bool bwd, bool row_affine, int64_t rows, int64_t D, int64_t N,
                       int64_t C, size_t align, size_t par_align, RowProblemPlan* p) {
  memset(p, 0, sizeof(*p));
  const Variant& var = variant();
  const int V = full_epv(dtype);
  int epv = pick_epv(dtype, D, align, par_align);
  p->epv = epv;
  const bool full = epv == V;
  const int64_t nvec = D / epv;
  const bool heavy = bwd && !row_affine;
  // InstanceNorm backward on rows of more than 2048 vectors has a table of its own
  const bool affine_wide = bwd && row_affine && full && nvec > 2048;
  const Shape* table = !full ? kScalarShapes
                             : (heavy ? kHeavyShapes : (affine_wide ? kAffineWideShapes : kLightShapes));
  const int ntab =
      !full ? kNumScalar : (heavy ? kNumHeavy : (affine_wide ? kNumAffineWide : kNumLight));
  const int forced = !full ? -1
                           : (affine_wide ? var.affine_shape : (bwd ? var.bwd_shape : var.fwd_shape));
  const int64_t tensor_bytes = rows * D * static_cast<int64_t>(dtype_size(dtype));
  p->shape = pick_shape(table, ntab, nvec, tensor_bytes, forced);
  p->two_phase = p->shape < 0;
  const int table_index = p->shape;  // `table[table_index]` below; p->shape is what the launcher gets
  if (affine_wide && p->shape >= 0) p->shape += kAffineWideBase;
  // Rows of thousands of vectors that fill a shape of rows_wide.cu take those kernels.
  if (!row_affine && full && var.wide == 0 && wide_ok(nvec, bwd)) {
    RowsArgs a = {};
    a.N = rows;
    a.D = D;
    cudaError_t e =
        wide_launch(dtype, bwd, bwd ? var.wide_bwd : var.wide_fwd, a, nullptr, true, &p->wp);
    if (e != cudaSuccess) return fail_cuda(e);
    p->wide = true;
    p->two_phase = false;
    size_t woff = 0;
    if (bwd) {
      p->colpart_rows = p->wp.partial_rows;
      p->off_colpart = 0;
      woff = align_up(static_cast<size_t>(p->colpart_rows) * 2 * D * 4, 256);
      const size_t sb = colreduce_scratch_bytes(p->colpart_rows, D);
      p->has_colscratch = sb > 0;
      p->off_colscratch = woff;
      woff += sb;
    }
    p->bytes = woff;
    return NVN_OK;
  }
  const bool clustered = !p->two_phase && table[table_index].cs > 1;
  // Rows that need a cluster but do not fill its shape lose the ring (equal slices) and run
  // with idle lanes; measured on B200 (bf16 widths 20000 ... 200000, fp32 20000 / 50000) the
  // two-phase kernels are 10-40 % faster there, so they take those.
  if (clustered && full && cap(table[table_index]) != nvec && rows <= 0x7fffffffLL && var.wide != 2)
    p->two_phase = true;
  // Forward over cluster shapes pays two cluster barriers per row; once the problem is large
  // (>= 64 MB per tensor) the three-pass two-phase kernels are faster (fp16 [1024, 65536]:
  // 3.6 against 2.6 TB/s), while few rows ([256, 65536]: 25 against 29 us) stay on clusters.
  if (clustered && !bwd && full && rows <= 0x7fffffffLL && tensor_bytes >= kHeldRingMinBytes &&
      var.wide != 2)
    p->two_phase = true;
  if (clustered && var.wide == 1) p->two_phase = true;
  size_t off = 0;
  if (!p->two_phase) {
    RowsArgs a = {};
    a.N = rows;
    a.D = D;
    a.C = C;
    cudaError_t e = rows_fn(dtype, bwd)(row_affine, p->epv, p->shape, a, nullptr, true,
                                        &p->rows);
    if (e != cudaSuccess) return fail_cuda(e);
    if (bwd) {
      p->colpart_rows = row_affine ? N : p->rows.partial_rows;
      p->off_colpart = off;
      off += align_up(static_cast<size_t>(p->colpart_rows) * 2 * (row_affine ? C : D) * 4, 256);
    }
  } else if (row_affine && full && var.nlc != 1 && rows <= 0x7fffffffLL &&
             (var.nlc == 3 || tensor_bytes / rows >= (384 << 10)) &&
             stream_groups(dtype, bwd, rows, V, D / V) > 0) {
    // InstanceNorm "NC..." rows of 384 KB and more (512 KB rows measured 8 % faster than
    // the two-phase kernels, 4 MB rows 17 %; the per-row barrier and merge would dominate
    // shorter ones): the persistent kernels in row mode (a row is read as D / V voxels of
    // one channel vector), in CTA groups
    p->stream_rows = true;
    p->stream_groups = stream_groups(dtype, bwd, rows, V, D / V);
    off = nlc_stream_workspace_bytes(bwd, rows, V);
    if (bwd) {
      p->colpart_rows = N;
      p->off_colpart = off;
      off += align_up(static_cast<size_t>(N) * 2 * C * 4, 256);
    }
  } else {
    if (rows > 0x7fffffffLL) return NVN_ERR_UNSUPPORTED;
    p->scalar = !full;
    epv = full ? V : 1;
    p->r2 = r2_plan(rows, D, epv, bwd && !row_affine);
    p->off_part = off;
    off += align_up(static_cast<size_t>(rows) * p->r2.nchunks * (bwd ? 2 : 3) * 4, 256);
    if (bwd) {
      p->off_coef = off;
      off += align_up(static_cast<size_t>(rows) * 2 * 4, 256);
      p->colpart_rows = row_affine ? N : p->r2.slices;
      p->off_colpart = off;
      off += align_up(static_cast<size_t>(p->colpart_rows) * 2 * (row_affine ? C : D) * 4, 256);
    }
  }
  if (bwd) {
    const size_t sb = colreduce_scratch_bytes(p->colpart_rows, row_affine ? C : D);
    p->has_colscratch = sb > 0;
    p->off_colscratch = off;
    off += sb;
  }
  p->bytes = off;
  return NVN_OK;
}

// Plans are pure functions of the problem (every device this library runs on is the same
// part), and a training step asks for the same few over and over: once for the workspace
// size and once per launch.  A small table keyed by the problem keeps the dispatcher out of
// the per-call cost.
struct PlanKey {
  int64_t rows, D, N, C;
  int dtype, flags, align, par_align;
  bool operator==(const PlanKey& o) const {
    return rows == o.rows && D == o.D && N == o.N && C == o.C && dtype == o.dtype &&
           flags == o.flags && align == o.align && par_align == o.par_align;
  }
};
struct PlanKeyHash {
  size_t operator()(const PlanKey& k) const {
    uint64_t h = 0x9e3779b97f4a7c15ull;
    for (uint64_t v : {static_cast<uint64_t>(k.rows), static_cast<uint64_t>(k.D),
                       static_cast<uint64_t>(k.N), static_cast<uint64_t>(k.C),
                       static_cast<uint64_t>(k.dtype * 64 + k.flags),
                       static_cast<uint64_t>(k.align * 32 + k.par_align)})
      h = (h ^ v) * 0xff51afd7ed558ccdull + (h >> 29);
    return static_cast<size_t>(h);
  }
};
template <typename Plan>
struct PlanCache {
  std::mutex mu;
  std::unordered_map<PlanKey, Plan, PlanKeyHash> map;
  bool find(const PlanKey& k, Plan* out) {
    std::lock_guard<std::mutex> lock(mu);
    auto it = map.find(k);
    if (it == map.end()) return false;
    *out = it->second;
    return true;
  }
  void put(const PlanKey& k, const Plan& p) {
    std::lock_guard<std::mutex> lock(mu);
    if (map.size() >= 1024) map.clear();  // a bound, not a policy: real jobs use a handful
    map[k] = p;
  }
};
PlanCache<RowProblemPlan> g_row_plans;
PlanCache<size_t> g_ws_bytes;

int plan_rows(int dtype, bool bwd, bool row_affine, int64_t rows, int64_t D, int64_t N,
              int64_t C, size_t align, size_t par_align, RowProblemPlan* p) {
  const PlanKey key = {rows, D, N, C, dtype, (bwd ? 1 : 0) | (row_affine ? 2 : 0),
                       static_cast<int>(align), static_cast<int>(par_align)};
  if (g_row_plans.find(key, p)) return NVN_OK;
  const int st = plan_rows_uncached(dtype, bwd, row_affine, rows, D, N, C, align, par_align, p);
  if (st == NVN_OK) g_row_plans.put(key, *p);
  return st;
}

size_t rows_workspace_bytes(int dtype, bool bwd, bool row_affine, int64_t rows, int64_t D,
                            int64_t N, int64_t C) {
  if (rows <= 0 || D <= 0) return 0;
  const PlanKey key = {rows, D, N, C, dtype, (bwd ? 1 : 0) | (row_affine ? 2 : 0) | 4, 0, 0};
  size_t b = 0;
  if (g_ws_bytes.find(key, &b)) return b;
  RowProblemPlan pv;
  // the workspace can depend on the access width, which depends on the caller's alignment
  for (size_t al : {size_t(16), size_t(8), size_t(4), size_t(2)}) {
    if (plan_rows(dtype, bwd, row_affine, rows, D, N, C, al, 16, &pv) == NVN_OK)
      b = std::max(b, pv.bytes);
  }
  g_ws_bytes.put(key, b);
  return b;
}

int run_rows(int dtype, bool bwd, bool row_affine, const void* dy, const void* x,
             const float* gamma, const float* beta, const float* mean_in, const float* ivar_in,
             int64_t rows, int64_t D, int64_t N, int64_t C, float eps, void* out, float* mean,
             float* ivar, float* dgamma, float* dbeta, void* ws, size_t ws_bytes,
             cudaStream_t stream, const nvn_dp_comm* comm = nullptr) {
  const size_t align = bwd ? common_alignment({x, out, dy}) : common_alignment({x, out});
  const size_t par_align = bwd ? common_alignment({gamma}) : common_alignment({gamma, beta});
  RowProblemPlan p;
  int st = plan_rows(dtype, bwd, row_affine, rows, D, N, C, align, par_align, &p);
  if (st != NVN_OK) return st;
  if (p.bytes > 0 && (ws == nullptr || !aligned(ws, 256) || ws_bytes < p.bytes))
    return NVN_ERR_WORKSPACE;
  char* wsb = static_cast<char*>(ws);
  const int64_t F = row_affine ? C : D;

  if (!p.two_phase) {
    RowsArgs a = {};
    a.x = x;
    a.dy = dy;
    a.gamma = gamma;
    a.beta = beta;
    a.mean_in = mean_in;
    a.ivar_in = ivar_in;
    a.out = out;
    a.mean = mean;
    a.ivar = ivar;
    a.ws = bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr;
    a.N = rows;
    a.D = D;
    a.C = C;
    a.eps = eps;
    a.status = device_status_word();
    cudaError_t e;
    if (p.wide) {
      WidePlan wp;
      e = wide_launch(dtype, bwd, bwd ? variant().wide_bwd : variant().wide_fwd, a, stream, false,
                      &wp);
    } else {
      RowsPlan rp;
      e = rows_fn(dtype, bwd)(row_affine, p.epv, p.shape, a, stream, false, &rp);
    }
    if (e != cudaSuccess) return fail_cuda(e);
  } else if (p.stream_rows) {
    const int V = full_epv(dtype);
    cudaError_t e = nlc_stream_launch(
        dtype, bwd, dy, x, gamma, beta, mean_in, ivar_in, rows, V, D / V, eps, out, mean, ivar, wsb,
        bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr, device_status_word(),
        kStreamBlock, p.stream_groups, C, stream);
    if (e != cudaSuccess) return fail_cuda(e);
  } else {
    R2Args a = {};
    a.x = x;
    a.dy = dy;
    a.gamma = gamma;
    a.beta = beta;
    a.mean = bwd ? const_cast<float*>(mean_in) : mean;
    a.ivar = bwd ? const_cast<float*>(ivar_in) : ivar;
    a.out = out;
    a.ws_part = reinterpret_cast<float*>(wsb + p.off_part);
    a.ws_coef = bwd ? reinterpret_cast<float*>(wsb + p.off_coef) : nullptr;
    a.ws_colpart = bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr;
    a.rows = rows;
    a.D = D;
    a.C = C;
    a.eps = eps;
    a.row_affine = row_affine;
    cudaError_t e = r2_launch(dtype, bwd, p.scalar, a, p.r2, stream);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  if (bwd) {
    const float* partials = reinterpret_cast<const float*>(wsb + p.off_colpart);
    cudaError_t e = comm != nullptr ? colreduce_allreduce_launch(partials, p.colpart_rows, F, comm,
                                                                 dgamma, dbeta, stream)
                                    : colreduce_launch(
                                          partials, p.colpart_rows, F, dgamma, dbeta, stream,
                                          p.has_colscratch
                                              ? reinterpret_cast<float*>(wsb + p.off_colscratch)
                                              : nullptr,
                                          p.has_colscratch ? kColreduceScratchRows : 0);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  return NVN_OK;
}

// ---------------------------------------------------------------------------
// Plan for channels-last InstanceNorm (x[n, d, c])
// ---------------------------------------------------------------------------

// CTA groups of the persistent kernels, or 0 when the two-phase kernels are the better
// choice.  One group for items that keep every SM busy for tens of microseconds; smaller
// items share the GPU, so that one group's barrier and merge hide under another group's
// streaming: about 96 MB in flight forward, 32 MB backward (whose first phase reads twice
// as much per item), at most one group per item.  Group counts: powers of two up to 16,
// then a quarter, a half and all of the SMs (37, 74, 148 groups of 4, 2, 1 CTAs on B200).
// Measured on B200, fp16, forward + backward: 8 items of 16.8 MB (C = 32), two-phase 217 us,
// 1 / 2 / 4 / 8 groups 229 / 170 / 166 / 176 us; 16 items of 7 MB, 183 us against 310 / 197 /
// 152 / 141 us; 32 items of 2 MB, 119 us against 110 / 88 / 83 us with 8 / 16 / 32 groups;
// 64 items of 256 KB, 53 us against 100 / 57 / 39 / 30 us with 8 / 16 / 37 / 64 groups.
int stream_groups(int dtype, bool bwd, int64_t N, int64_t C, int64_t D) {
  const double item_bytes = static_cast<double>(D) * C * (dtype == 0 ? 4 : 2);
  int g = 1;
  if (variant().stream_groups > 0) {
    g = variant().stream_groups;
  } else {
    const double want = (bwd ? 32.0 : 96.0) * 1048576.0 / item_bytes;
    const int sm = device_sm_count();
    const int cand[] = {1, 2, 4, 8, 16, sm / 4, sm / 2, sm};
    for (int c : cand)   // the candidate nearest to `want` on a log scale (ascending list)
      if (c > g && static_cast<double>(c) * g < want * want) g = c;
  }
  if (g > N) g = static_cast<int>(N);
  if (variant().nlc == 3) return g;
  const double in_flight = g * item_bytes;
  return (item_bytes >= 32.0 * 1048576.0 || in_flight >= 24.0 * 1048576.0 ||
          (g >= 16 && in_flight >= 8.0 * 1048576.0))
             ? g
             : 0;
}

struct NlcPlan {
  bool stream;  // persistent kernel: one cooperative launch, item tails kept on chip
  bool scalar;
  bool onchip;  // a batch item fits in shared memory: one launch, one pass over HBM
  bool small;   // small items: one warp per item
  S2Plan s2;
  size_t off_part, off_coef, off_colpart, off_colscratch, bytes;
  bool has_colscratch;
};

int plan_nlc(int dtype, bool bwd, int64_t N, int64_t C, int64_t D, bool vec_ok, NlcPlan* p,
             bool allow_onchip = true) {
  memset(p, 0, sizeof(*p));
  const int V = full_epv(dtype);
  p->scalar = !(vec_ok && C % V == 0);
  // Small items: a warp per item beats a CTA per item below 2048 elements, and is the only
  // one-launch path for channel counts or alignments the vector kernels cannot take.
  // (items that fit in one CTA's shared memory keep their single-pass kernel)
  if (vec_ok && allow_onchip && variant().nlc != 1 && nlc_stream_ok(dtype, N, C, D) &&
      (variant().nlc == 3 || !nlc_onchip_ok(dtype, bwd, C, D)) &&
      stream_groups(dtype, bwd, N, C, D) > 0) {
    p->stream = true;
    size_t off = nlc_stream_workspace_bytes(bwd, N, C);
    if (bwd) {
      p->off_colpart = off;
      off += align_up(static_cast<size_t>(N) * 2 * C * 4, 256);
      const size_t sb = colreduce_scratch_bytes(N, C);
      p->has_colscratch = sb > 0;
      p->off_colscratch = off;
      off += sb;
    }
    p->bytes = off;
    return NVN_OK;
  }
  const bool onchip_ok = vec_ok && allow_onchip && nlc_onchip_ok(dtype, bwd, C, D);
  if (nlc_small_ok(C, D) && (D * C <= 2048 || !onchip_ok)) {
    if (variant().nlc == 0) {
      p->small = true;
      p->off_colpart = 0;
      p->bytes = bwd ? align_up(static_cast<size_t>(N) * 2 * C * 4, 256) : 0;
      if (bwd) {
        const size_t sb = colreduce_scratch_bytes(N, C);
        p->has_colscratch = sb > 0;
        p->off_colscratch = p->bytes;
        p->bytes += sb;
      }
      return NVN_OK;
    }
  }
  if (onchip_ok) {
    if (variant().nlc != 1) {
      p->onchip = true;
      p->off_colpart = 0;
      p->bytes = bwd ? align_up(static_cast<size_t>(N) * 2 * C * 4, 256) : 0;
      if (bwd) {
        const size_t sb = colreduce_scratch_bytes(N, C);
        p->has_colscratch = sb > 0;
        p->off_colscratch = p->bytes;
        p->bytes += sb;
      }
      return NVN_OK;
    }
  }
  const int epv = p->scalar ? 1 : V;
  p->s2 = s2_plan(dtype, bwd, N, C, D, epv);
  if (p->s2.ctiles > 65535) return NVN_ERR_UNSUPPORTED;
  size_t off = 0;
  p->off_part = off;
  off += align_up(static_cast<size_t>(N) * p->s2.nchunks * (bwd ? 2 : 3) * C * 4, 256);
  if (bwd) {
    p->off_coef = off;
    off += align_up(static_cast<size_t>(N) * 3 * C * 4, 256);
    p->off_colpart = off;
    off += align_up(static_cast<size_t>(N) * 2 * C * 4, 256);
    const size_t sb = colreduce_scratch_bytes(N, C);
    p->has_colscratch = sb > 0;
    p->off_colscratch = off;
    off += sb;
  }
  p->bytes = off;
  return NVN_OK;
}

int run_nlc(int dtype, bool bwd, const void* dy, const void* x, const float* gamma,
            const float* beta, const float* mean_in, const float* ivar_in, int64_t N, int64_t C,
            int64_t D, float eps, void* out, float* mean, float* ivar, float* dgamma,
            float* dbeta, void* ws, size_t ws_bytes, cudaStream_t stream,
            const nvn_dp_comm* comm = nullptr) {
  bool vec_ok = aligned(x, 16) && aligned(out, 16) && (!bwd || aligned(dy, 16));
  // the on-chip kernels also read the parameters and the saved statistics as vectors
  const bool par_ok = aligned(gamma, 16) && (bwd ? aligned(mean_in, 16) && aligned(ivar_in, 16)
                                                 : aligned(beta, 16));
  NlcPlan p;
  int st = plan_nlc(dtype, bwd, N, C, D, vec_ok, &p, par_ok);
  if (st != NVN_OK) return st;
  if (p.bytes > 0 && (ws == nullptr || !aligned(ws, 256) || ws_bytes < p.bytes))
    return NVN_ERR_WORKSPACE;
  char* wsb = static_cast<char*>(ws);
  if (p.stream) {
    float* colpart = bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr;
    cudaError_t e = nlc_stream_launch(dtype, bwd, dy, x, gamma, beta, mean_in, ivar_in, N, C, D,
                                      eps, out, mean, ivar, wsb, colpart, device_status_word(),
                                      variant().stream_block > 0 ? variant().stream_block : kStreamBlock,
                                      stream_groups(dtype, bwd, N, C, D), 0, stream);
    if (e != cudaSuccess) return fail_cuda(e);
    if (bwd) {
      e = comm != nullptr ? colreduce_allreduce_launch(colpart, N, C, comm, dgamma, dbeta, stream)
                          : colreduce_launch(colpart, N, C, dgamma, dbeta, stream,
                                             p.has_colscratch
                                                 ? reinterpret_cast<float*>(wsb + p.off_colscratch)
                                                 : nullptr,
                                             p.has_colscratch ? kColreduceScratchRows : 0);
      if (e != cudaSuccess) return fail_cuda(e);
    }
    return NVN_OK;
  }
  if (p.onchip || p.small) {
    float* colpart = bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr;
    cudaError_t e = p.small
                        ? nlc_small_launch(dtype, bwd, dy, x, gamma, beta, mean_in, ivar_in, N, C,
                                           D, eps, out, mean, ivar, colpart, stream)
                        : nlc_onchip_launch(dtype, bwd, dy, x, gamma, beta, mean_in, ivar_in, N, C, D,
                                      eps, out, mean, ivar, colpart, device_status_word(), stream);
    if (e != cudaSuccess) return fail_cuda(e);
    if (bwd) {
      e = comm != nullptr ? colreduce_allreduce_launch(colpart, N, C, comm, dgamma, dbeta, stream)
                          : colreduce_launch(colpart, N, C, dgamma, dbeta, stream,
                                             p.has_colscratch
                                                 ? reinterpret_cast<float*>(wsb + p.off_colscratch)
                                                 : nullptr,
                                             p.has_colscratch ? kColreduceScratchRows : 0);
      if (e != cudaSuccess) return fail_cuda(e);
    }
    return NVN_OK;
  }
  S2Args a = {};
  a.x = x;
  a.dy = dy;
  a.gamma = gamma;
  a.beta = beta;
  a.mean = bwd ? const_cast<float*>(mean_in) : mean;
  a.ivar = bwd ? const_cast<float*>(ivar_in) : ivar;
  a.out = out;
  a.ws_part = reinterpret_cast<float*>(wsb + p.off_part);
  a.ws_coef = bwd ? reinterpret_cast<float*>(wsb + p.off_coef) : nullptr;
  a.ws_colpart = bwd ? reinterpret_cast<float*>(wsb + p.off_colpart) : nullptr;
  a.N = N;
  a.C = C;
  a.D = D;
  a.eps = eps;
  cudaError_t e = s2_launch(dtype, bwd, p.scalar, a, p.s2, stream);
  if (e != cudaSuccess) return fail_cuda(e);
  if (bwd) {
    e = comm != nullptr
            ? colreduce_allreduce_launch(a.ws_colpart, N, C, comm, dgamma, dbeta, stream)
            : colreduce_launch(a.ws_colpart, N, C, dgamma, dbeta, stream,
                               p.has_colscratch ? reinterpret_cast<float*>(wsb + p.off_colscratch)
                                                : nullptr,
                               p.has_colscratch ? kColreduceScratchRows : 0);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  return NVN_OK;
}

int zero_grads(float* dgamma, float* dbeta, int64_t F, cudaStream_t stream) {
  if (F <= 0) return NVN_OK;
  cudaError_t e = cudaMemsetAsync(dgamma, 0, static_cast<size_t>(F) * 4, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(dbeta, 0, static_cast<size_t>(F) * 4, stream);
  return e == cudaSuccess ? NVN_OK : fail_cuda(e);
}

inline bool valid_dtype(int d) { return d == NVN_F32 || d == NVN_F16 || d == NVN_BF16; }

}  // namespace

int device_sm_count() {
  int v = g_sm_count.load(std::memory_order_relaxed);
  if (v > 0) return v;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
    (void)cudaGetLastError();
    return 148;  // B200; only reached when no device is usable
  }
  g_sm_count.store(v, std::memory_order_relaxed);
  return v;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

bool use_dependent_launch() { return variant().pdl != 0; }

namespace {
// Raised by a kernel whose bounded wait on an asynchronous copy gave up.
__device__ int g_status_word = 0;
std::mutex g_status_mutex;
int* g_status_ptr[64] = {};
}  // namespace

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

bool rows_res_ok(int dtype, int64_t D, size_t align, size_t par_align) {
  const int V = full_epv(dtype);
  return D % V == 0 && D / V <= 4096 && align >= 16 && par_align >= 16;
}

cudaError_t rows_res_launch(int dtype, const RowsResArgs& a, cudaStream_t s) {
  return dtype == NVN_F32 ? rows_res_f32(a, s) : (dtype == NVN_F16 ? rows_res_f16(a, s) : rows_res_bf16(a, s));
}

cudaError_t residual_add_launch(int dtype, const void* x, const void* res, void* sum_out,
                                int64_t count, cudaStream_t s) {
  return dtype == NVN_F32 ? residual_add_f32(x, res, sum_out, count, s)
                          : (dtype == NVN_F16 ? residual_add_f16(x, res, sum_out, count, s)
                                              : residual_add_bf16(x, res, sum_out, count, s));
}

}  // namespace nvn

using namespace nvn;

extern "C" {

int nvn_version(void) { return 100; }

const char* nvn_status_string(int status) {
  switch (status) {
    case NVN_OK:
      return "ok";
    case NVN_ERR_INVALID_ARGUMENT:
      return "invalid argument";
    case NVN_ERR_AXIS_RANGE:
      return "axis contains invalid value";
    case NVN_ERR_AXIS_NOT_PACKED:
      return "axis is not packed from last dim.";
    case NVN_ERR_DATA_FORMAT:
      return "We only accept 'NC...' or 'N...C' data format";
    case NVN_ERR_RANK:
      return "input rank too small";
    case NVN_ERR_WORKSPACE:
      return "workspace missing, misaligned or too small";
    case NVN_ERR_CUDA:
      return "CUDA runtime error";
    case NVN_ERR_UNSUPPORTED:
      return "problem size not supported";
    case NVN_ERR_LIMIT:
      return "problem size exceeds a built-in capacity";
    case NVN_ERR_TIMEOUT:
      return "a kernel gave up waiting for an asynchronous copy";
    default:
      return "unknown status";
  }
}

int nvn_last_cuda_error(void) { return t_last_cuda_error; }

uint64_t nvn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int nvn_device_status(void) {
  int* p = device_status_word();
  if (p == nullptr) return NVN_ERR_CUDA;
  int v = 0;
  // synchronous on purpose: a diagnostic, not part of the asynchronous call path
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVN_ERR_CUDA;
  }
  return v == 0 ? NVN_OK : NVN_ERR_TIMEOUT;
}

int nvn_ln_dims(int rank, const int64_t* dims, int n_axis, const int* axis, int64_t* N,
                int64_t* D) {
  if (dims == nullptr || N == nullptr || D == nullptr || n_axis < 0 ||
      (n_axis > 0 && axis == nullptr))
    return NVN_ERR_INVALID_ARGUMENT;
  if (rank < 1) return NVN_ERR_RANK;
  if (n_axis == 0) return NVN_ERR_AXIS_NOT_PACKED;
  std::vector<int> ax;
  ax.reserve(n_axis);
  for (int i = 0; i < n_axis; ++i) {
    const int a = axis[i] < 0 ? rank + axis[i] : axis[i];
    if (a < 0 || a >= rank) return NVN_ERR_AXIS_RANGE;
    ax.push_back(a);
  }
  std::sort(ax.begin(), ax.end());
  ax.erase(std::unique(ax.begin(), ax.end()), ax.end());
  if (ax[0] != rank - static_cast<int>(ax.size())) return NVN_ERR_AXIS_NOT_PACKED;
  int64_t n = 1, d = 1;
  for (int i = 0; i < rank; ++i) {
    if (dims[i] < 0) return NVN_ERR_INVALID_ARGUMENT;
    if (i >= ax[0]) {
      d *= dims[i];
    } else {
      n *= dims[i];
    }
  }
  *N = n;
  *D = d;
  return NVN_OK;
}

int nvn_in_dims(int rank, const int64_t* dims, const char* data_format, int64_t* N, int64_t* C,
                int64_t* D, int* channel_first) {
  if (dims == nullptr || data_format == nullptr || N == nullptr || C == nullptr ||
      D == nullptr || channel_first == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  const size_t len = strlen(data_format);
  if (!(len > 2 && data_format[0] == 'N' &&
        (data_format[1] == 'C' || data_format[len - 1] == 'C')))
    return NVN_ERR_DATA_FORMAT;
  if (rank < 4) return NVN_ERR_RANK;
  const bool cf = data_format[1] == 'C';
  for (int i = 0; i < rank; ++i)
    if (dims[i] < 0) return NVN_ERR_INVALID_ARGUMENT;
  *N = dims[0];
  *C = cf ? dims[1] : dims[rank - 1];
  int64_t d = 1;
  const int lo = cf ? 2 : 1, hi = cf ? rank : rank - 1;
  for (int i = lo; i < hi; ++i) d *= dims[i];
  *D = d;
  *channel_first = cf ? 1 : 0;
  return NVN_OK;
}

size_t nvn_ln_fwd_workspace_bytes(int dtype, int64_t N, int64_t D) {
  if (!valid_dtype(dtype)) return 0;
  return rows_workspace_bytes(dtype, false, false, N, D, N, 1);
}

size_t nvn_ln_bwd_workspace_bytes(int dtype, int64_t N, int64_t D) {
  if (!valid_dtype(dtype)) return 0;
  return rows_workspace_bytes(dtype, true, false, N, D, N, 1);
}

static size_t in_workspace_bytes(int dtype, bool bwd, int64_t N, int64_t C, int64_t D,
                                 int channel_first) {
  if (!valid_dtype(dtype) || N <= 0 || C <= 0 || D <= 0) return 0;
  if (channel_first || C == 1)
    return rows_workspace_bytes(dtype, bwd, true, N * C, D, N, C);
  NlcPlan pv, ps;
  size_t b = 0;
  // whichever path alignment lets the call take, the workspace must be large enough
  for (const bool vec_ok : {true, false})
    for (const bool onchip : {true, false})
      if (plan_nlc(dtype, bwd, N, C, D, vec_ok, &pv, onchip) == NVN_OK) b = std::max(b, pv.bytes);
  (void)ps;
  return b;
}

size_t nvn_in_fwd_workspace_bytes(int dtype, int64_t N, int64_t C, int64_t D,
                                  int channel_first) {
  return in_workspace_bytes(dtype, false, N, C, D, channel_first);
}

size_t nvn_in_bwd_workspace_bytes(int dtype, int64_t N, int64_t C, int64_t D,
                                  int channel_first) {
  return in_workspace_bytes(dtype, true, N, C, D, channel_first);
}

int nvn_ln_fwd(int dtype, const void* x, const float* gamma, const float* beta, int64_t N,
               int64_t D, float epsilon, void* y, float* mean, float* inv_std, void* workspace,
               size_t workspace_bytes, void* stream) {
  if (!valid_dtype(dtype) || N < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  if (N == 0 || D == 0) return NVN_OK;
  if (x == nullptr || gamma == nullptr || beta == nullptr || y == nullptr || mean == nullptr ||
      inv_std == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  return run_rows(dtype, false, false, nullptr, x, gamma, beta, nullptr, nullptr, N, D, N, 1,
                  epsilon, y, mean, inv_std, nullptr, nullptr, workspace, workspace_bytes,
                  static_cast<cudaStream_t>(stream));
}

int nvn_ln_fwd_residual(int dtype, const void* x, const void* residual, const float* gamma,
                        const float* beta, int64_t N, int64_t D, float epsilon, void* sum_out,
                        void* y, float* mean, float* inv_std, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (!valid_dtype(dtype) || N < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  if (N == 0 || D == 0) return NVN_OK;
  if (x == nullptr || residual == nullptr || gamma == nullptr || beta == nullptr ||
      sum_out == nullptr || y == nullptr || mean == nullptr || inv_std == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t align = common_alignment({x, residual, sum_out, y});
  const size_t par_align = common_alignment({gamma, beta});
  if (rows_res_ok(dtype, D, align, par_align)) {
    RowsResArgs a = {};
    a.x = x;
    a.res = residual;
    a.sum_out = sum_out;
    a.gamma = gamma;
    a.beta = beta;
    a.out = y;
    a.mean = mean;
    a.ivar = inv_std;
    a.N = N;
    a.D = D;
    a.C = 1;
    a.eps = epsilon;
    a.status = device_status_word();
    const cudaError_t e = rows_res_launch(dtype, a, s);
    return e == cudaSuccess ? NVN_OK : fail_cuda(e);
  }
  // any other width or alignment: the sum as a kernel of its own, then the plain forward
  const cudaError_t e = residual_add_launch(dtype, x, residual, sum_out, N * D, s);
  if (e != cudaSuccess) return fail_cuda(e);
  return nvn_ln_fwd(dtype, sum_out, gamma, beta, N, D, epsilon, y, mean, inv_std, workspace,
                    workspace_bytes, stream);
}

static int ln_bwd_impl(int dtype, const void* dy, const void* x, const float* gamma,
                       const float* mean, const float* inv_std, int64_t N, int64_t D, void* dx,
                       float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
                       const nvn_dp_comm* comm, void* stream) {
  if (!valid_dtype(dtype) || N < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  if (D > 0 && (dgamma == nullptr || dbeta == nullptr)) return NVN_ERR_INVALID_ARGUMENT;
  if (N == 0 || D == 0) return zero_grads(dgamma, dbeta, D, static_cast<cudaStream_t>(stream));
  if (dy == nullptr || x == nullptr || gamma == nullptr || mean == nullptr ||
      inv_std == nullptr || dx == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  return run_rows(dtype, true, false, dy, x, gamma, nullptr, mean, inv_std, N, D, N, 1, 0.f, dx,
                  nullptr, nullptr, dgamma, dbeta, workspace, workspace_bytes,
                  static_cast<cudaStream_t>(stream), comm);
}

int nvn_ln_bwd(int dtype, const void* dy, const void* x, const float* gamma, const float* mean,
               const float* inv_std, int64_t N, int64_t D, void* dx, float* dgamma,
               float* dbeta, void* workspace, size_t workspace_bytes, void* stream) {
  return ln_bwd_impl(dtype, dy, x, gamma, mean, inv_std, N, D, dx, dgamma, dbeta, workspace,
                     workspace_bytes, nullptr, stream);
}

// Every rank must take part in the exchange, also with an empty local shard, so the
// data-parallel variants reject empty problems instead of silently skipping the kernel.
static int check_comm(const nvn_dp_comm* c, int64_t F) {
  if (c == nullptr || c->world < 1 || c->world > NVN_DP_MAX_RANKS || c->rank < 0 ||
      c->rank >= c->world || (c->epoch == 0 && c->device_epochs == nullptr) || F % 2 != 0)
    return NVN_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < c->world; ++i)
    if (c->recv[i] == nullptr || !aligned(c->recv[i], 16))
      return NVN_ERR_INVALID_ARGUMENT;
  return NVN_OK;
}

int nvn_dp_finish(int64_t F, const nvn_dp_comm* comm, float* dgamma, float* dbeta,
                  void* stream) {
  if (F <= 0 || dgamma == nullptr || dbeta == nullptr) return NVN_ERR_INVALID_ARGUMENT;
  const int st = check_comm(comm, F);
  if (st != NVN_OK) return st;
  cudaError_t e = dp_finish_launch(F, comm, dgamma, dbeta, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVN_OK : fail_cuda(e);
}

size_t nvn_dp_recv_bytes(int64_t F, int world) {
  if (F <= 0 || world < 1) return 0;
  // [4 slots][world][2F] pairs of (value, epoch)
  return static_cast<size_t>(4) * world * 2 * F * 2 * sizeof(uint32_t);
}

int nvn_ln_bwd_dp(int dtype, const void* dy, const void* x, const float* gamma,
                  const float* mean, const float* inv_std, int64_t N, int64_t D, void* dx,
                  float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
                  const nvn_dp_comm* comm, void* stream) {
  if (N <= 0 || D <= 0) return NVN_ERR_INVALID_ARGUMENT;
  const int st = check_comm(comm, D);
  if (st != NVN_OK) return st;
  return ln_bwd_impl(dtype, dy, x, gamma, mean, inv_std, N, D, dx, dgamma, dbeta, workspace,
                     workspace_bytes, comm, stream);
}

int nvn_in_fwd(int dtype, const void* x, const float* gamma, const float* beta, int64_t N,
               int64_t C, int64_t D, int channel_first, float epsilon, void* y, float* mean,
               float* inv_std, void* workspace, size_t workspace_bytes, void* stream) {
  if (!valid_dtype(dtype) || N < 0 || C < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  if (N == 0 || C == 0 || D == 0) return NVN_OK;
  if (x == nullptr || gamma == nullptr || beta == nullptr || y == nullptr || mean == nullptr ||
      inv_std == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (channel_first || C == 1)
    return run_rows(dtype, false, true, nullptr, x, gamma, beta, nullptr, nullptr, N * C, D, N,
                    C, epsilon, y, mean, inv_std, nullptr, nullptr, workspace, workspace_bytes,
                    s);
  return run_nlc(dtype, false, nullptr, x, gamma, beta, nullptr, nullptr, N, C, D, epsilon, y,
                 mean, inv_std, nullptr, nullptr, workspace, workspace_bytes, s);
}

static int in_bwd_impl(int dtype, const void* dy, const void* x, const float* gamma,
                       const float* mean, const float* inv_std, int64_t N, int64_t C, int64_t D,
                       int channel_first, void* dx, float* dgamma, float* dbeta, void* workspace,
                       size_t workspace_bytes, const nvn_dp_comm* comm, void* stream) {
  if (!valid_dtype(dtype) || N < 0 || C < 0 || D < 0) return NVN_ERR_INVALID_ARGUMENT;
  if (C > 0 && (dgamma == nullptr || dbeta == nullptr)) return NVN_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N == 0 || C == 0 || D == 0) return zero_grads(dgamma, dbeta, C, s);
  if (dy == nullptr || x == nullptr || gamma == nullptr || mean == nullptr ||
      inv_std == nullptr || dx == nullptr)
    return NVN_ERR_INVALID_ARGUMENT;
  if (channel_first || C == 1)
    return run_rows(dtype, true, true, dy, x, gamma, nullptr, mean, inv_std, N * C, D, N, C,
                    0.f, dx, nullptr, nullptr, dgamma, dbeta, workspace, workspace_bytes, s,
                    comm);
  return run_nlc(dtype, true, dy, x, gamma, nullptr, mean, inv_std, N, C, D, 0.f, dx, nullptr,
                 nullptr, dgamma, dbeta, workspace, workspace_bytes, s, comm);
}

int nvn_in_bwd(int dtype, const void* dy, const void* x, const float* gamma, const float* mean,
               const float* inv_std, int64_t N, int64_t C, int64_t D, int channel_first,
               void* dx, float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
               void* stream) {
  return in_bwd_impl(dtype, dy, x, gamma, mean, inv_std, N, C, D, channel_first, dx, dgamma,
                     dbeta, workspace, workspace_bytes, nullptr, stream);
}

int nvn_in_bwd_dp(int dtype, const void* dy, const void* x, const float* gamma,
                  const float* mean, const float* inv_std, int64_t N, int64_t C, int64_t D,
                  int channel_first, void* dx, float* dgamma, float* dbeta, void* workspace,
                  size_t workspace_bytes, const nvn_dp_comm* comm, void* stream) {
  if (N <= 0 || C <= 0 || D <= 0) return NVN_ERR_INVALID_ARGUMENT;
  const int st = check_comm(comm, C);
  if (st != NVN_OK) return st;
  return in_bwd_impl(dtype, dy, x, gamma, mean, inv_std, N, C, D, channel_first, dx, dgamma,
                     dbeta, workspace, workspace_bytes, comm, stream);
}

int nvn_describe_plan(int op, int dtype, int64_t N, int64_t C, int64_t D, int channel_first,
                      char* out, size_t out_bytes) {
  if (out == nullptr || out_bytes == 0 || !valid_dtype(dtype) || op < 0 || op > 3)
    return NVN_ERR_INVALID_ARGUMENT;
  const bool bwd = (op & 1) != 0;
  const bool is_in = op >= 2;
  if (N <= 0 || D <= 0 || (is_in && C <= 0)) {
    snprintf(out, out_bytes, "empty");
    return NVN_OK;
  }
  if (is_in && !channel_first && C != 1) {
    NlcPlan p;
    int st = plan_nlc(dtype, bwd, N, C, D, true, &p);
    if (st != NVN_OK) return st;
    if (p.stream) {
      snprintf(out, out_bytes, "nlc persistent epv=%d consumers=%d ring=6x%dKB groups=%d",
               full_epv(dtype), variant().stream_block == 256 ? 256 : kStreamBlock,
               (variant().stream_block == 256 ? 256 : kStreamBlock) / 16,
               stream_groups(dtype, bwd, N, C, D));
      return NVN_OK;
    }
    if (p.small) {
      snprintf(out, out_bytes, "nlc warp-per-item block=256");
      return NVN_OK;
    }
    if (p.onchip) {
      snprintf(out, out_bytes, "nlc on-chip epv=%d block=256", full_epv(dtype));
      return NVN_OK;
    }
    snprintf(out, out_bytes,
             "nlc two-phase epv=%d cvt=%d lanes=%d ctiles=%d chunk=%lld nchunks=%d group=%d",
             p.scalar ? 1 : full_epv(dtype), p.s2.cvt, p.s2.lanes, p.s2.ctiles,
             static_cast<long long>(p.s2.chunk), p.s2.nchunks, p.s2.group);
    return NVN_OK;
  }
  const int64_t rows = is_in ? N * C : N;
  RowProblemPlan p;
  int st = plan_rows(dtype, bwd, is_in, rows, D, N, is_in ? C : 1, 16, 16, &p);
  if (st != NVN_OK) return st;
  if (p.wide) {
    snprintf(out, out_bytes, "rows wide block=%d vpt=%d cluster=%d stages=%d epv=%d grid=%d",
             p.wp.block, p.wp.vpt, p.wp.cluster, p.wp.stages, full_epv(dtype), p.wp.grid);
  } else if (p.stream_rows) {
    snprintf(out, out_bytes, "rows persistent epv=%d consumers=%d ring=6x32KB groups=%d",
             full_epv(dtype), kStreamBlock, p.stream_groups);
  } else if (p.two_phase) {
    snprintf(out, out_bytes, "rows two-phase epv=%d chunk=%lld nchunks=%d slices=%d",
             p.scalar ? 1 : full_epv(dtype), static_cast<long long>(p.r2.chunk), p.r2.nchunks,
             p.r2.slices);
  } else {
    snprintf(out, out_bytes, "rows tpr=%d vpt=%d cluster=%d rb=%d load=%s%d epv=%d block=%d grid=%d",
             p.rows.tpr, p.rows.vpt, p.rows.cluster, p.rows.rb,
             p.rows.load_mode >= 10 ? "tma-held"
                                    : (p.rows.load_mode >= 2
                                           ? "tma"
                                           : (p.rows.load_mode == 1 ? "prefetch" : "plain")),
             p.rows.load_mode >= 10 ? p.rows.load_mode - 10
                                    : (p.rows.load_mode >= 2 ? p.rows.load_mode : 0),
             p.rows.epv, p.rows.block, p.rows.grid);
  }
  return NVN_OK;
}

}  // extern "C"
