// C ABI of the kernel library (see include/tbk.h): packed-forest upload, launch-shape
// selection, kernel dispatch, the second pass, and the host-buffer pipeline.
#include "../../include/tbk.h"
#include "pack.h"
#include "quant_pack.h"
#include "deep_pack.h"
#include "schedule.h"
#include "walk_kernels.cuh"
#include "walk_quant.cuh"
#include "walk_quant_batch.cuh"
#include "walk_deep.cuh"
#include "packed_image.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define CUDA_TRY(expr)                                                                     \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return fail(TBK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),   \
                  __FILE__, __LINE__);                                                     \
  } while (0)

} // namespace

struct tbk_image {
  tb::PackedImage im;
};

struct tbk_forest {
  tb::PackedForest packed; // host copy (orig_node kept for lazy upload)
  int device = 0;
  tbk_schedule user{};     // what the caller asked for (zeros = auto)
  tb::LaunchPlan last_plan{};
  int64_t batch_hint = 0;
  int max_smem_optin = 0;
  int num_sms = 0;
  // device buffers
  uint8_t *d_blob = nullptr;
  tb::DevGroupMeta *d_groups = nullptr;
  int16_t *d_tree_class = nullptr;
  int32_t *d_tree_index = nullptr;
  int32_t *d_orig_node = nullptr;
  unsigned long long *d_orig_off = nullptr;
  int8_t *d_lut = nullptr;
  int32_t *d_status = nullptr;
  float *d_scratch = nullptr; // tree-chunk partials, two slots
  size_t scratch_bytes = 0;
  // a slot's last user: a call on another stream waits for it before reusing the slot
  cudaEvent_t scratch_done[2] = {nullptr, nullptr};
  cudaStream_t scratch_stream[2] = {nullptr, nullptr};
  bool scratch_used[2] = {false, false};
  // 16-bit-key layout (wide rows)
  bool quant = false;
  tb::QuantForest qf;
  uint32_t *d_qnode = nullptr;
  float *d_qleaf = nullptr, *d_qexact = nullptr, *d_qlo = nullptr, *d_qscale = nullptr;
  tb::DevQuantGroup *d_qgroups = nullptr;
  int32_t *d_qtree_index = nullptr, *d_qorig = nullptr;
  int32_t *d_qset_groups = nullptr, *d_qgroup_class = nullptr; // multiclass key layout
  int32_t qset_count[2] = {0, 0};
  unsigned long long *d_ties = nullptr;
  // one-tree-per-stage layout (deep trees); shares the device buffers of the key layout
  bool deep = false;
  tb::DeepForest df;
  int deep_row_warps = 0, deep_slots = 0;
  int uniform_depth = 0; // key layouts: depth shared by all groups / pairs, 0 = mixed
  // host pipeline
  float *d_in[2] = {nullptr, nullptr};
  unsigned char *d_res[2] = {nullptr, nullptr};
  float *h_pin[2] = {nullptr, nullptr};
  unsigned char *h_res = nullptr;
  size_t pipe_rows = 0, pipe_ld = 0, h_res_bytes = 0;
  cudaStream_t streams[2] = {nullptr, nullptr};
  cudaEvent_t in_free[2] = {nullptr, nullptr};
  // timing
  bool timing = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  bool ev_pending = false;
  int64_t launches = 0;
  bool expire_next_wait = false; // failure drill (tbk_debug_expire_next_wait)
  std::mutex mu;
};

namespace {

using KernelFn = void (*)(const tb::WalkParams);

template <int REP, int TS> KernelFn pick3(int rpl, bool staged, bool cached) {
  if (!cached) return staged ? tb::tb_walk_kernel<REP, TS, 1, true, false> : tb::tb_walk_kernel<REP, TS, 1, false, false>;
  if (rpl == 2) return staged ? tb::tb_walk_kernel<REP, TS, 2, true, true> : tb::tb_walk_kernel<REP, TS, 2, false, true>;
  return staged ? tb::tb_walk_kernel<REP, TS, 1, true, true> : tb::tb_walk_kernel<REP, TS, 1, false, true>;
}

KernelFn pick_kernel(int rep, int ts, int rpl, bool staged, bool cached) {
  if (rep == tb::kReorg) return pick3<2, 1>(rpl, staged, cached);
  if (rep == tb::kSparse) {
    switch (ts) {
    case 1: return pick3<0, 1>(rpl, staged, cached);
    case 2: return pick3<0, 2>(rpl, staged, cached);
    case 3: return pick3<0, 3>(rpl, staged, cached);
    default: return pick3<0, 4>(rpl, staged, cached);
    }
  }
  switch (ts) {
  case 1: return pick3<1, 1>(rpl, staged, cached);
  case 2: return pick3<1, 2>(rpl, staged, cached);
  case 3: return pick3<1, 3>(rpl, staged, cached);
  default: return pick3<1, 4>(rpl, staged, cached);
  }
}

int ensure_scratch(tbk_forest *f, size_t bytes) {
  if (bytes <= f->scratch_bytes) return TBK_OK;
  if (f->d_scratch) CUDA_TRY(cudaFree(f->d_scratch));
  f->d_scratch = nullptr;
  f->scratch_bytes = 0;
  CUDA_TRY(cudaMalloc(&f->d_scratch, bytes));
  f->scratch_bytes = bytes;
  return TBK_OK;
}

// The tree-chunk partial sums of a call live in a slot of the forest's scratch buffer from the
// walk until the second pass has read them.  Calls on one stream are ordered anyway; a call on
// another stream first waits (on the device) for the slot's previous user.
int scratch_acquire(tbk_forest *f, int slot, cudaStream_t stream) {
  if (f->scratch_used[slot] && f->scratch_stream[slot] != stream)
    CUDA_TRY(cudaStreamWaitEvent(stream, f->scratch_done[slot], 0));
  return TBK_OK;
}
int scratch_release(tbk_forest *f, int slot, cudaStream_t stream) {
  if (!f->scratch_done[slot]) CUDA_TRY(cudaEventCreateWithFlags(&f->scratch_done[slot], cudaEventDisableTiming));
  CUDA_TRY(cudaEventRecord(f->scratch_done[slot], stream));
  f->scratch_stream[slot] = stream;
  f->scratch_used[slot] = true;
  return TBK_OK;
}

int ensure_orig(tbk_forest *f) {
  if (f->d_orig_node) return TBK_OK;
  const auto &p = f->packed;
  CUDA_TRY(cudaMalloc(&f->d_orig_node, std::max<size_t>(4, p.orig_node.size() * 4)));
  CUDA_TRY(cudaMemcpy(f->d_orig_node, p.orig_node.data(), p.orig_node.size() * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMalloc(&f->d_orig_off, std::max<size_t>(8, p.orig_off.size() * 8)));
  CUDA_TRY(cudaMemcpy(f->d_orig_off, p.orig_off.data(), p.orig_off.size() * 8, cudaMemcpyHostToDevice));
  return TBK_OK;
}

enum Mode { kPredict, kPartial, kLeafIds };

int quant_smem_bytes(int num_features) {
  return tb::kQBarBytes + tb::kQRingBytes + tb::kQLeafTableBytes + tb::quant_key_tile_bytes(num_features);
}

// Tiles of 32 rows that the narrow-row kernel can stage together (0: the rows are too wide for it).
int quant_batch_tiles(const tbk_forest *f, int num_features) {
  const int room = f->max_smem_optin - tb::kQBBarBytes - tb::kQBRingBytes;
  const int fit = room / tb::quant_batch_tile_bytes(num_features);
  return fit >= 4 ? std::min(fit, tb::kQBMaxTiles) : 0;
}

// One prediction with a 15-bit-key kernel: rows whose key tiles fit shared memory several at a
// time go to the batch kernel (persistent blocks of 22 warps over batches of up to 16 tiles),
// wide rows to the kernel that holds one tile (persistent blocks of 24 warps over tiles of 32 rows).
int run_quant(tbk_forest *f, Mode mode, const float *d_rows, int64_t n_rows, int64_t ld, void *d_out, int32_t out_kind,
              float *d_partial, int32_t *d_leaf_ids, cudaStream_t stream, int slot) {
  const auto &q = f->qf;
  const int64_t G = (int64_t)q.groups.size();
  const int64_t tiles = (n_rows + 31) / 32;
  const int max_batch = quant_batch_tiles(f, q.num_features);
  const bool batched = max_batch > 0;
  const bool multi = q.num_classes > 0;
  if (multi && !batched) return fail(TBK_ERR_UNSUPPORTED, "multiclass forests in the key layout need rows narrow enough for the batch kernel");
  // batch kernel: as many tiles per batch as still give every SM a batch
  int R = 1;
  if (batched) {
    R = max_batch;
    while (R > 1 && (tiles + R - 1) / R < (int64_t)f->num_sms) R = (R + 1) / 2;
  }
  const int64_t units = batched ? (tiles + R - 1) / R : tiles; // blocks' units of work along x
  int64_t chunks = 1;
  if (multi) chunks = 1; // a class must stay within one leaf warp's sequence of groups
  else if (f->user.tree_chunks > 0) chunks = f->user.tree_chunks;
  else if (batched) {
    if (units < (int64_t)f->num_sms) chunks = ((int64_t)f->num_sms + units - 1) / units;
  } else if (tiles < 2 * (int64_t)f->num_sms) chunks = (2 * (int64_t)f->num_sms + tiles - 1) / tiles;
  // (batch kernel: a second pass over partial sums costs about ten microseconds, more than the
  // walk of a small forest: trees are split only into chunks of at least 32 groups -- measured
  // on 4 096 rows x 32 groups: 38 us in one chunk, 47 us in two -- unless the caller asks)
  const int64_t max_chunks = !batched ? G : f->user.tree_chunks > 0 ? std::max<int64_t>(1, G / 2) : std::max<int64_t>(1, G / 32);
  chunks = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(chunks, max_chunks), 65535));
  const int gpc = (int)((G + chunks - 1) / chunks);
  chunks = (G + gpc - 1) / gpc;
  const bool vec4 = q.num_features % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(d_rows) & 15) == 0;
  // One block per SM (shared memory allows no more).  With more units than blocks a block is
  // persistent; the one-tile kernel then stages its next tile in tensor memory while it walks
  // the current one, a path that reads rows with 16-byte loads.
  const int64_t blocks_x = std::max<int64_t>(1, (int64_t)f->num_sms / chunks);
  const int64_t grid_x = batched ? std::min(units, blocks_x) : (vec4 && tiles > blocks_x) ? blocks_x : tiles;
  tb::LaunchPlan plan;
  plan.row_warps = batched ? R : 1;
  plan.tree_threads = tb::kQWalkers;
  plan.rows_per_lane = 1;
  plan.chunks = (int32_t)chunks;
  plan.groups_per_chunk = gpc;
  plan.staged = 1;
  plan.cache_rows = 1;
  plan.stage_bytes = tb::kQPiece;
  plan.smem_bytes = batched ? tb::quant_batch_smem_bytes(q.num_features, R) : quant_smem_bytes(q.num_features);
  plan.threads = batched ? tb::kQBThreads : tb::kQThreads;
  plan.grid_x = grid_x;
  f->last_plan = plan;

  const bool need_partials = mode == kPartial || (mode == kPredict && chunks > 1);
  float *partial_dst = nullptr;
  bool uses_scratch = false;
  if (need_partials) {
    if (mode == kPartial && chunks == 1) {
      partial_dst = d_partial;
    } else {
      const size_t need = ((size_t)chunks * n_rows * sizeof(float) + 255) & ~(size_t)255;
      int rc = ensure_scratch(f, 2 * need);
      if (rc) return rc;
      partial_dst = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(f->d_scratch) + (size_t)slot * (f->scratch_bytes / 2));
      rc = scratch_acquire(f, slot, stream);
      if (rc) return rc;
      uses_scratch = true;
    }
  }
  tb::QuantParams p{};
  p.node_plane = f->d_qnode;
  p.leaf_plane = f->d_qleaf;
  p.exact_plane = f->d_qexact;
  p.groups = f->d_qgroups;
  p.tree_index = f->d_qtree_index;
  p.orig_leaf = f->d_qorig;
  p.lo = f->d_qlo;
  p.scale = f->d_qscale;
  p.rows = d_rows;
  p.n_rows = n_rows;
  p.ld = ld;
  p.partial = partial_dst;
  p.out = d_out;
  p.write_partial = need_partials ? 1 : 0;
  p.leaf_ids = mode == kLeafIds ? d_leaf_ids : nullptr;
  p.num_trees = q.num_trees;
  p.num_groups = (int32_t)G;
  p.groups_per_chunk = gpc;
  p.num_features = q.num_features;
  p.transform = q.transform;
  p.initial_value = (float)q.initial_value;
  p.vec4_ok = vec4 ? 1 : 0;
  p.tiles_per_batch = R;
  p.set_groups = f->d_qset_groups;
  p.set_count[0] = f->qset_count[0];
  p.set_count[1] = f->qset_count[1];
  p.group_class = f->d_qgroup_class;
  p.num_classes = q.num_classes;
  p.out_kind = out_kind == TBK_OUT_I8 ? 1 : 0;
  p.status = f->d_status;
  p.tie_count = f->d_ties;
  p.skip_first_copy = f->expire_next_wait ? 1 : 0;
  p.wait_tries = f->expire_next_wait ? 2000u : 0u;
  f->expire_next_wait = false;
  // kernels specialised for forests whose groups all have 8 (or 6) levels; generic otherwise
  using QuantKernel = void (*)(const tb::QuantParams);
  const bool ids = mode == kLeafIds;
  const int ud = (f->uniform_depth == 8 || f->uniform_depth == 6) ? f->uniform_depth : 0;
  const QuantKernel qkernel =
      multi ? (ud == 8 ? (ids ? tb::tb_walk_quant_batch_kernel<8, true, true> : tb::tb_walk_quant_batch_kernel<8, false, true>)
                       : (ids ? tb::tb_walk_quant_batch_kernel<0, true, true> : tb::tb_walk_quant_batch_kernel<0, false, true>))
      : batched
          ? (ud == 8   ? (ids ? tb::tb_walk_quant_batch_kernel<8, true, false> : tb::tb_walk_quant_batch_kernel<8, false, false>)
             : ud == 6 ? (ids ? tb::tb_walk_quant_batch_kernel<6, true, false> : tb::tb_walk_quant_batch_kernel<6, false, false>)
                       : (ids ? tb::tb_walk_quant_batch_kernel<0, true, false> : tb::tb_walk_quant_batch_kernel<0, false, false>))
      : ud == 8 ? (ids ? tb::tb_walk_quant_kernel<8, true> : tb::tb_walk_quant_kernel<8, false>)
      : ud == 6 ? (ids ? tb::tb_walk_quant_kernel<6, true> : tb::tb_walk_quant_kernel<6, false>)
                : (ids ? tb::tb_walk_quant_kernel<0, true> : tb::tb_walk_quant_kernel<0, false>);
  CUDA_TRY(cudaFuncSetAttribute((const void *)qkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));
  if (f->timing) CUDA_TRY(cudaEventRecord(f->ev0, stream));
  dim3 grid((unsigned)grid_x, (unsigned)chunks);
  qkernel<<<grid, plan.threads, plan.smem_bytes, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
  ++f->launches;
  const int tpb = 256;
  if (mode == kPredict && chunks > 1) {
    tb::tb_finalize_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(
        partial_dst, (int)chunks, n_rows, 1, 0, (float)q.initial_value, q.transform, d_out, TBK_OUT_F32);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  } else if (mode == kPartial && chunks > 1) {
    tb::tb_sum_partials_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(partial_dst, (int)chunks, n_rows, d_partial);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  }
  if (f->timing) {
    CUDA_TRY(cudaEventRecord(f->ev1, stream));
    f->ev_pending = true;
  }
  if (uses_scratch) return scratch_release(f, slot, stream);
  return TBK_OK;
}

// Shared-memory plan of the deep-tree kernel: the most row warps (even -- one block per SM
// either way, and more rows per tile mean fewer passes over the forest and more walks in
// flight) whose key tile leaves room for a ring of at least 4 whole-tree pieces.
bool deep_plan(int num_features, int max_depth, int smem_limit, int *row_warps, int *slots) {
  const int64_t slot = 4ll << std::max(max_depth, tb::kDeepMinDepth);
  // four slots hold the node planes of the pair being walked and of the next one
  for (int rw = 30; rw >= 4; rw -= 2) { // (the block has one more warp, the ring producer)
    const int64_t keys = (int64_t)(num_features + 1) * 64 * rw;
    const int64_t room = (int64_t)smem_limit - 128 - keys;
    const int64_t s = std::min<int64_t>(tb::kDeepMaxSlots, room / slot);
    if (s >= 4) {
      *row_warps = rw;
      *slots = (int)s;
      return true;
    }
  }
  return false;
}
int deep_smem_bytes(const tbk_forest *f) {
  return 128 + f->deep_slots * (4 << std::max(f->df.max_depth, tb::kDeepMinDepth)) +
         (f->df.num_features + 1) * 64 * f->deep_row_warps;
}

// One prediction with the deep-tree kernel (one block per 32 x row_warps rows).
int run_deep(tbk_forest *f, Mode mode, const float *d_rows, int64_t n_rows, int64_t ld, void *d_out,
             float *d_partial, int32_t *d_leaf_ids, cudaStream_t stream, int slot) {
  const auto &q = f->df;
  const int64_t G = (int64_t)q.pairs.size();
  // small batches: fewer row warps per block, so that the tiles still cover the SMs
  int rw = f->deep_row_warps;
  while (rw > 4 && (n_rows + 32 * rw - 1) / (32 * rw) < f->num_sms) rw -= 2;
  const int64_t rows_per_block = 32 * rw;
  const int64_t grid_x = (n_rows + rows_per_block - 1) / rows_per_block;
  int64_t chunks = 1;
  if (f->user.tree_chunks > 0) chunks = f->user.tree_chunks;
  else if (grid_x < (int64_t)f->num_sms) chunks = ((int64_t)f->num_sms + grid_x - 1) / grid_x;
  chunks = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(chunks, G), 65535));
  const int gpc = (int)((G + chunks - 1) / chunks);
  chunks = (G + gpc - 1) / gpc;
  tb::LaunchPlan plan;
  plan.row_warps = rw;
  plan.tree_threads = 1;
  plan.rows_per_lane = 1;
  plan.chunks = (int32_t)chunks;
  plan.groups_per_chunk = gpc;
  plan.staged = 1;
  plan.cache_rows = 1;
  plan.stage_bytes = 4u << std::max(q.max_depth, tb::kDeepMinDepth);
  plan.smem_bytes = deep_smem_bytes(f);
  plan.threads = 32 * (rw + 1); // row warps + the ring producer
  plan.grid_x = grid_x;
  f->last_plan = plan;

  const bool need_partials = mode == kPartial || (mode == kPredict && chunks > 1);
  float *partial_dst = nullptr;
  bool uses_scratch = false;
  if (need_partials) {
    if (mode == kPartial && chunks == 1) {
      partial_dst = d_partial;
    } else {
      const size_t need = ((size_t)chunks * n_rows * sizeof(float) + 255) & ~(size_t)255;
      int rc = ensure_scratch(f, 2 * need);
      if (rc) return rc;
      partial_dst = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(f->d_scratch) + (size_t)slot * (f->scratch_bytes / 2));
      rc = scratch_acquire(f, slot, stream);
      if (rc) return rc;
      uses_scratch = true;
    }
  }
  tb::DeepParams p{};
  p.node_plane = f->d_qnode;
  p.leaf_plane = f->d_qleaf;
  p.exact_plane = f->d_qexact;
  p.pairs = f->d_qgroups;
  p.tree_index = f->d_qtree_index;
  p.orig_leaf = f->d_qorig;
  p.lo = f->d_qlo;
  p.scale = f->d_qscale;
  p.rows = d_rows;
  p.n_rows = n_rows;
  p.ld = ld;
  p.partial = partial_dst;
  p.out = d_out;
  p.write_partial = need_partials ? 1 : 0;
  p.leaf_ids = mode == kLeafIds ? d_leaf_ids : nullptr;
  p.num_trees = q.num_trees;
  p.num_pairs = (int32_t)G;
  p.pairs_per_chunk = gpc;
  p.num_features = q.num_features;
  p.transform = q.transform;
  p.initial_value = (float)q.initial_value;
  p.ring_slots = f->deep_slots;
  p.slot_bytes = plan.stage_bytes;
  p.key_stride = 64u * (uint32_t)f->deep_row_warps; // the tile keeps its full width whatever rw is
  p.status = f->d_status;
  p.tie_count = f->d_ties;
  p.skip_first_copy = f->expire_next_wait ? 1 : 0;
  p.wait_tries = f->expire_next_wait ? 2000u : 0u;
  f->expire_next_wait = false;
  // up to 24 warps (row warps + producer) the compiler may use 80 registers per thread, beyond that 64
  // specialised for forests whose pairs all have 12 levels; generic otherwise
  using DeepKernel = void (*)(const tb::DeepParams);
  const bool d12 = f->uniform_depth == 12, ids = mode == kLeafIds, small = plan.threads <= 768;
  const DeepKernel kernel =
      small ? (d12 ? (ids ? tb::tb_walk_deep_kernel<768, 12, true> : tb::tb_walk_deep_kernel<768, 12, false>)
                   : (ids ? tb::tb_walk_deep_kernel<768, 0, true> : tb::tb_walk_deep_kernel<768, 0, false>))
            : (d12 ? (ids ? tb::tb_walk_deep_kernel<1024, 12, true> : tb::tb_walk_deep_kernel<1024, 12, false>)
                   : (ids ? tb::tb_walk_deep_kernel<1024, 0, true> : tb::tb_walk_deep_kernel<1024, 0, false>));
  CUDA_TRY(cudaFuncSetAttribute((const void *)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));
  if (f->timing) CUDA_TRY(cudaEventRecord(f->ev0, stream));
  dim3 grid((unsigned)grid_x, (unsigned)chunks);
  kernel<<<grid, plan.threads, plan.smem_bytes, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
  ++f->launches;
  const int tpb = 256;
  if (mode == kPredict && chunks > 1) {
    tb::tb_finalize_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(
        partial_dst, (int)chunks, n_rows, 1, 0, (float)q.initial_value, q.transform, d_out, TBK_OUT_F32);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  } else if (mode == kPartial && chunks > 1) {
    tb::tb_sum_partials_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(partial_dst, (int)chunks, n_rows, d_partial);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  }
  if (f->timing) {
    CUDA_TRY(cudaEventRecord(f->ev1, stream));
    f->ev_pending = true;
  }
  if (uses_scratch) return scratch_release(f, slot, stream);
  return TBK_OK;
}

// One prediction over device-resident rows.
int run(tbk_forest *f, Mode mode, const float *d_rows, int64_t n_rows, int64_t ld, void *d_out,
        int32_t out_kind, float *d_partial, int32_t *d_leaf_ids, cudaStream_t stream, int slot = 0) {
  const auto &pk = f->packed;
  if (n_rows < 0 || ld < pk.num_features) return fail(TBK_ERR_INVALID, "ld (%lld) is smaller than the row size (%d)", (long long)ld, pk.num_features);
  if (n_rows == 0) return TBK_OK;
  if (!d_rows) return fail(TBK_ERR_INVALID, "null input pointer");
  if (mode == kPredict) {
    if (!d_out) return fail(TBK_ERR_INVALID, "null output pointer");
    if (out_kind == TBK_OUT_I8 && pk.num_classes == 0) return fail(TBK_ERR_INVALID, "int8 output needs a multiclass forest");
    if (out_kind != TBK_OUT_F32 && out_kind != TBK_OUT_I8) return fail(TBK_ERR_INVALID, "unknown output kind %d", out_kind);
  }
  CUDA_TRY(cudaSetDevice(f->device));
  if (f->quant) return run_quant(f, mode, d_rows, n_rows, ld, d_out, out_kind, d_partial, d_leaf_ids, stream, slot);
  if (f->deep) return run_deep(f, mode, d_rows, n_rows, ld, d_out, d_partial, d_leaf_ids, stream, slot);

  tb::ForestShape shape{pk.num_features, pk.num_classes, (int64_t)pk.groups.size(), pk.max_group_bytes,
                        (int32_t)pk.lut.size(), pk.representation, pk.tile_size};
  tb::LaunchPlan plan;
  std::string why = tb::select_launch(shape, f->user, n_rows, f->max_smem_optin, f->num_sms, mode == kLeafIds, &plan,
                                      mode == kPartial);
  if (!why.empty()) return fail(TBK_ERR_UNSUPPORTED, "%s", why.c_str());
  f->last_plan = plan;

  const int W = std::max(1, pk.num_classes);
  const bool need_partials = mode == kPartial || (mode == kPredict && plan.chunks > 1);
  float *partial_dst = nullptr;
  bool uses_scratch = false;
  if (mode == kLeafIds) {
    int rc = ensure_orig(f);
    if (rc) return rc;
  } else if (need_partials) {
    if (mode == kPartial && plan.chunks == 1) {
      partial_dst = d_partial;
    } else {
      // two slots, so that the two streams of the host pipeline never share partials
      const size_t need = ((size_t)plan.chunks * n_rows * W * sizeof(float) + 255) & ~(size_t)255;
      int rc = ensure_scratch(f, 2 * need);
      if (rc) return rc;
      partial_dst = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(f->d_scratch) + (size_t)slot * (f->scratch_bytes / 2));
      rc = scratch_acquire(f, slot, stream);
      if (rc) return rc;
      uses_scratch = true;
    }
  }

  tb::WalkParams p{};
  p.blob = f->d_blob;
  p.groups = f->d_groups;
  p.tree_class = f->d_tree_class;
  p.tree_index = f->d_tree_index;
  p.orig_node = f->d_orig_node;
  p.orig_off = f->d_orig_off;
  p.lut = f->d_lut;
  p.lut_bytes = (int32_t)pk.lut.size();
  p.rows = d_rows;
  p.n_rows = n_rows;
  p.ld = ld;
  p.partial = partial_dst;
  p.out = d_out;
  p.out_kind = out_kind;
  p.write_partial = need_partials ? 1 : 0;
  p.leaf_ids = mode == kLeafIds ? d_leaf_ids : nullptr;
  p.num_trees = pk.num_trees;
  p.num_groups = (int32_t)pk.groups.size();
  p.groups_per_chunk = plan.groups_per_chunk;
  p.num_features = pk.num_features;
  p.num_classes = pk.num_classes;
  p.transform = pk.transform;
  p.initial_value = (float)pk.initial_value;
  p.row_warps = plan.row_warps;
  p.tree_threads = plan.tree_threads;
  p.stage_bytes = plan.staged ? plan.stage_bytes : 0;
  p.vec4_ok = (pk.num_features % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(d_rows) & 15) == 0) ? 1 : 0;
  p.status = f->d_status;
  p.skip_first_copy = (f->expire_next_wait && plan.staged) ? 1 : 0;
  p.wait_limit = f->expire_next_wait ? 2000u : 0u;
  f->expire_next_wait = false;
  // the plan's shared-memory size has no class table when class sums live in registers
  if (plan.class_regs && (plan.chunks != 1 || mode == kPartial))
    return fail(TBK_ERR_UNSUPPORTED, "launch plan with register class sums needs a single tree chunk");
  p.class_regs = plan.class_regs;

  KernelFn fn = pick_kernel(pk.representation, pk.tile_size, plan.rows_per_lane, plan.staged, plan.cache_rows);
  CUDA_TRY(cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));
  if (f->timing) CUDA_TRY(cudaEventRecord(f->ev0, stream));
  dim3 grid((unsigned)plan.grid_x, (unsigned)plan.chunks), block((unsigned)plan.threads);
  fn<<<grid, block, plan.smem_bytes, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
  ++f->launches;
  if (mode == kPredict && plan.chunks > 1) {
    const int tpb = 256;
    tb::tb_finalize_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(
        partial_dst, plan.chunks, n_rows, W, pk.num_classes, (float)pk.initial_value, pk.transform, d_out, out_kind);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  } else if (mode == kPartial && plan.chunks > 1) {
    const int tpb = 256;
    const long long total = n_rows * W;
    tb::tb_sum_partials_kernel<<<(unsigned)((total + tpb - 1) / tpb), tpb, 0, stream>>>(partial_dst, plan.chunks, total, d_partial);
    CUDA_TRY(cudaGetLastError());
    ++f->launches;
  }
  if (f->timing) {
    CUDA_TRY(cudaEventRecord(f->ev1, stream));
    f->ev_pending = true;
  }
  if (uses_scratch) return scratch_release(f, slot, stream);
  return TBK_OK;
}

int check_status(tbk_forest *f) {
  int32_t st = 0;
  CUDA_TRY(cudaMemcpy(&st, f->d_status, 4, cudaMemcpyDeviceToHost));
  if (st != 0) {
    int32_t zero = 0;
    cudaMemcpy(f->d_status, &zero, 4, cudaMemcpyHostToDevice);
    return fail(TBK_ERR_DEVICE_WAIT, "a bounded wait on a bulk copy expired inside the walk kernel (status %d)", st);
  }
  return TBK_OK;
}

// Uploads the planes of a 16-bit-key layout (quant_pack.h / deep_pack.h) and fills the
// threshold keys on the device, so that thresholds and row values are quantised by the
// very same arithmetic.
int upload_key_planes(tbk_forest *f, const std::vector<uint32_t> &node, const std::vector<float> &leaf,
                      const std::vector<float> &exact, const std::vector<int32_t> &orig,
                      const std::vector<tb::QuantGroup> &groups, const std::vector<int32_t> &tree_index,
                      const std::vector<float> &lo, const std::vector<float> &scale, int num_features, bool wide) {
  const size_t n = node.size();
  static_assert(sizeof(tb::QuantGroup) == sizeof(tb::DevQuantGroup), "group metadata layout");
  uint32_t dmin = 0xffffffffu, dmax = 0;
  for (const auto &g : groups) {
    dmin = std::min(dmin, g.depth);
    dmax = std::max(dmax, g.depth);
  }
  f->uniform_depth = dmin == dmax ? (int)dmin : 0;
  CUDA_TRY(cudaMalloc(&f->d_qnode, n * 4));
  CUDA_TRY(cudaMalloc(&f->d_qleaf, n * 4));
  CUDA_TRY(cudaMalloc(&f->d_qexact, n * 4));
  CUDA_TRY(cudaMalloc(&f->d_qorig, n * 4));
  CUDA_TRY(cudaMalloc(&f->d_qgroups, groups.size() * sizeof(tb::QuantGroup)));
  CUDA_TRY(cudaMalloc(&f->d_qtree_index, tree_index.size() * 4));
  // lo / scale are read with 16-byte loads: pad to a multiple of 4 entries
  const size_t nf = ((size_t)num_features + 1 + 3) / 4 * 4;
  CUDA_TRY(cudaMalloc(&f->d_qlo, nf * 4));
  CUDA_TRY(cudaMalloc(&f->d_qscale, nf * 4));
  CUDA_TRY(cudaMemset(f->d_qlo, 0, nf * 4));
  CUDA_TRY(cudaMemset(f->d_qscale, 0, nf * 4));
  CUDA_TRY(cudaMalloc(&f->d_ties, 128));
  CUDA_TRY(cudaMemset(f->d_ties, 0, 128));
  CUDA_TRY(cudaMemcpy(f->d_qnode, node.data(), n * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qleaf, leaf.data(), n * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qexact, exact.data(), n * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qorig, orig.data(), n * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qgroups, groups.data(), groups.size() * sizeof(tb::QuantGroup), cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qtree_index, tree_index.data(), tree_index.size() * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qlo, lo.data(), lo.size() * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(f->d_qscale, scale.data(), scale.size() * 4, cudaMemcpyHostToDevice));
  tb::tb_quant_fill_keys<<<(unsigned)((n + 255) / 256), 256>>>(f->d_qnode, f->d_qexact, f->d_qlo, f->d_qscale,
                                                             (unsigned long long)n, num_features, wide ? 1 : 0);
  CUDA_TRY(cudaGetLastError());
  CUDA_TRY(cudaDeviceSynchronize());
  ++f->launches;
  return TBK_OK;
}

void free_pipeline(tbk_forest *f) {
  for (int i = 0; i < 2; ++i) {
    if (f->d_in[i]) cudaFree(f->d_in[i]);
    if (f->d_res[i]) cudaFree(f->d_res[i]);
    if (f->h_pin[i]) cudaFreeHost(f->h_pin[i]);
    f->d_in[i] = nullptr; f->d_res[i] = nullptr; f->h_pin[i] = nullptr;
  }
  if (f->h_res) cudaFreeHost(f->h_res);
  f->h_res = nullptr;
  f->pipe_rows = f->pipe_ld = f->h_res_bytes = 0;
}

} // namespace

extern "C" {

const char *tbk_last_error(void) { return g_last_error.c_str(); }

int tbk_forest_create(const tbk_forest_arrays *fa, const tbk_schedule *schedule, int32_t device,
                      int64_t batch_hint, tbk_forest **out) {
  if (!out) return fail(TBK_ERR_INVALID, "null argument");
  *out = nullptr;
  int smem_limit = 0;
  CUDA_TRY(cudaSetDevice(device));
  CUDA_TRY(cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  tbk_image *img = nullptr;
  int rc = tbk_image_create(fa, schedule, smem_limit, &img);
  if (rc != TBK_OK) return rc;
  rc = tbk_forest_create_from_image(img, schedule, device, batch_hint, out);
  tbk_image_free(img);
  return rc;
}

int tbk_image_create(const tbk_forest_arrays *fa, const tbk_schedule *schedule, int32_t smem_limit, tbk_image **out) {
  if (!fa || !out) return fail(TBK_ERR_INVALID, "null argument");
  *out = nullptr;
  if (fa->num_trees <= 0 || !fa->tree_off || !fa->left || !fa->right || !fa->feat || !fa->thr)
    return fail(TBK_ERR_INVALID, "forest arrays are incomplete");
  tb::Forest host;
  const int64_t T = fa->num_trees, N = fa->tree_off[T];
  if (N <= 0) return fail(TBK_ERR_INVALID, "forest has no nodes");
  host.tree_off.assign(fa->tree_off, fa->tree_off + T + 1);
  host.left.assign(fa->left, fa->left + N);
  host.right.assign(fa->right, fa->right + N);
  host.feat.assign(fa->feat, fa->feat + N);
  host.thr.assign(fa->thr, fa->thr + N);
  if (fa->num_classes > 0) {
    if (!fa->class_id) return fail(TBK_ERR_INVALID, "multiclass forest without class ids");
    host.class_id.assign(fa->class_id, fa->class_id + T);
  }
  host.num_classes = fa->num_classes;
  host.transform = fa->transform;
  host.initial_value = fa->initial_value;
  host.num_features = fa->num_features;
  if (fa->num_classes > 0 && fa->num_classes > 127) return fail(TBK_ERR_UNSUPPORTED, "more than 127 classes");
  if (smem_limit <= 0) smem_limit = 227 * 1024;

  std::unique_ptr<tbk_image> img(new tbk_image());
  tb::PackedImage &im = img->im;
  if (schedule) im.user = *schedule;
  im.smem_limit = smem_limit;

  // ---- choose the layout
  const int bits = im.user.feature_bits;
  if (bits != 0 && bits != 16 && bits != 32) return fail(TBK_ERR_INVALID, "feature_bits must be 0, 16 or 32");
  int rep = im.user.representation;
  const int ts = im.user.tile_size <= 0 ? 1 : im.user.tile_size;
  im.requested_representation = rep;
  im.requested_tile_size = ts;
  im.requested_feature_bits = bits;
  // an fp32 tile of 32 rows (plus the sentinel column) must fit beside a little metadata
  const bool fp32_tile_fits = (int64_t)(host.num_features + 1) * 128 + 1024 <= smem_limit;
  {
    const std::string verr = tb::validate(host);
    if (!verr.empty()) return fail(TBK_ERR_INVALID, "%s", verr.c_str());
  }
  int max_depth = 0;
#pragma omp parallel for reduction(max : max_depth) schedule(dynamic, 64) num_threads(tb::pack_threads())
  for (int64_t t = 0; t < T; ++t) max_depth = std::max(max_depth, (int)tb::tree_depth(host, t));
  // narrow rows: the key tiles of at least four 32-row tiles fit beside the ring, so the batch
  // kernel applies; measured faster than the fp32 walk on single-output forests of up to 8 levels
  const bool batch_fits =
      (smem_limit - tb::kQBBarBytes - tb::kQBRingBytes) / tb::quant_batch_tile_bytes(host.num_features) >= 4;
  // (multiclass forests too: one walker set per class, arg-max or per-class sums in the leaf warps)
  bool want_quant = (bits == 16 && max_depth <= tb::kQuantMaxDepth && (host.num_classes == 0 || batch_fits)) ||
                    (bits == 0 && (rep == TBK_REP_AUTO || rep == TBK_REP_REORG) && ts == 1 && !fp32_tile_fits &&
                     host.num_classes == 0) ||
                    (bits == 0 && rep == TBK_REP_AUTO && ts == 1 && batch_fits && max_depth <= tb::kQuantMaxDepth);
  if (want_quant) {
    // narrow rows (batch kernel): features with whole-number thresholds become lattice features
    std::string qerr = tb::pack_quant(host, &im.qf, batch_fits);
    // Whole-number thresholds that could not be put on a lattice (a feature with other
    // thresholds too, or wide rows) mean integer-valued features whose rows tie with thresholds
    // all the time (measured: one comparison in 16 on 4-bit features, the key walk then runs at
    // a quarter of the fp32 walk's rate): such forests keep fp32 tiles unless keys were asked for.
    if (qerr.empty() && bits == 0 && fp32_tile_fits && 2 * im.qf.whole_number_splits > im.qf.num_splits)
      qerr = "integer-valued features";
    if (qerr.empty() && !batch_fits && quant_smem_bytes(host.num_features) > smem_limit)
      qerr = "rows are too wide for the 16-bit key tile";
    if (qerr.empty() && im.qf.node_plane.size() >= (1ull << 32))
      qerr = "forest too large for the 16-bit key layout (2^32 plane elements)";
    if (!qerr.empty()) {
      if (bits == 16) return fail(TBK_ERR_UNSUPPORTED, "%s", qerr.c_str());
      want_quant = false;
      im.qf = tb::QuantForest();
    }
  }
  // ---- deep trees: whole-tree stages over a key tile (deep_pack.h); not chosen for forests
  // whose thresholds are mostly whole numbers on features that cannot be lattice features
  // (integer-valued features then tie on every equality)
  bool deep_ok = !want_quant && host.num_classes == 0 && ts == 1 && bits != 32 &&
                 (bits == 16 || im.user.representation == TBK_REP_AUTO);
  if (deep_ok && bits == 0 && max_depth > tb::kQuantMaxDepth) {
    std::vector<float> lo, scale; // a negative scale marks a lattice feature
    if (tb::quant_feature_ranges(host, tb::kKey15Span, &lo, &scale, true).empty()) {
      int64_t splits = 0, whole = 0;
#pragma omp parallel for reduction(+ : splits, whole) schedule(static) num_threads(tb::pack_threads())
      for (int64_t g = 0; g < host.num_nodes(); ++g)
        if (!host.is_leaf(g)) {
          ++splits;
          whole += host.thr[g] == std::floor(host.thr[g]) && !(scale[host.feat[g]] < 0.f) ? 1 : 0;
        }
      deep_ok = 2 * whole <= splits;
    }
  }
  if (deep_ok) {
    int rw = 0, slots = 0;
    const bool fits = max_depth > tb::kQuantMaxDepth && max_depth <= tb::kDeepMaxDepth &&
                      deep_plan(host.num_features, max_depth, smem_limit, &rw, &slots);
    if (fits) {
      std::string derr = tb::pack_deep(host, &im.df);
      if (derr.empty()) {
        im.kind = tb::PackedImage::kDeep;
        im.deep_row_warps = rw;
        im.deep_slots = slots;
        im.user.representation = TBK_REP_REORG;
        *out = img.release();
        return TBK_OK;
      }
      if (bits == 16) return fail(TBK_ERR_UNSUPPORTED, "%s", derr.c_str());
      im.df = tb::DeepForest();
    } else if (bits == 16) {
      return fail(TBK_ERR_UNSUPPORTED, "16-bit feature keys: neither key layout fits this forest (depth %d, %d features)",
                  max_depth, host.num_features);
    }
  }
  if (bits == 16 && !want_quant)
    return fail(TBK_ERR_UNSUPPORTED, "16-bit feature keys cover single-output forests of at most %d levels and multiclass "
                                     "forests of at most %d levels over narrow rows, tile size 1 "
                                     "(this forest: %d levels, %d classes, %d features, tile size %d)",
                tb::kDeepMaxDepth, tb::kQuantMaxDepth, max_depth, host.num_classes, host.num_features, ts);
  if (rep == TBK_REP_AUTO) rep = TBK_REP_SPARSE;
  if (want_quant) {
    im.kind = tb::PackedImage::kQuant;
    im.user.representation = TBK_REP_REORG;
    *out = img.release();
    return TBK_OK;
  }
  tb::PackOptions opt;
  opt.representation = rep;
  opt.tile_size = ts;
  im.user.representation = rep;
  std::string err = tb::pack_forest(host, opt, &im.packed);
  if (!err.empty()) return fail(TBK_ERR_INVALID, "%s", err.c_str());
  im.kind = tb::PackedImage::kGeneral;
  *out = img.release();
  return TBK_OK;
}

int tbk_image_free(tbk_image *img) {
  delete img;
  return TBK_OK;
}

int tbk_image_serialize(const tbk_image *img, void *buffer, uint64_t capacity, uint64_t *size) {
  if (!img || !size) return fail(TBK_ERR_INVALID, "null argument");
  *size = tb::serialized_image_size(img->im);
  if (!buffer) return TBK_OK;
  if (capacity < *size) return fail(TBK_ERR_INVALID, "buffer of %llu bytes, the image needs %llu",
                                    (unsigned long long)capacity, (unsigned long long)*size);
  std::vector<uint8_t> bytes;
  tb::serialize_image(img->im, &bytes);
  std::memcpy(buffer, bytes.data(), bytes.size());
  return TBK_OK;
}

int tbk_image_deserialize(const void *buffer, uint64_t size, tbk_image **out) {
  if (!buffer || !out) return fail(TBK_ERR_INVALID, "null argument");
  *out = nullptr;
  std::unique_ptr<tbk_image> img(new tbk_image());
  const std::string err = tb::deserialize_image(static_cast<const uint8_t *>(buffer), size, &img->im);
  if (!err.empty()) return fail(TBK_ERR_IO, "%s", err.c_str());
  *out = img.release();
  return TBK_OK;
}

int tbk_image_matches(const tbk_image *img, const tbk_schedule *schedule, int32_t smem_limit) {
  if (!img) return 0;
  tbk_schedule want{};
  if (schedule) want = *schedule;
  const tb::PackedImage &im = img->im;
  const int ts = want.tile_size <= 0 ? 1 : want.tile_size;
  if (smem_limit <= 0) smem_limit = 227 * 1024;
  return im.requested_representation == want.representation && im.requested_tile_size == ts &&
         im.requested_feature_bits == want.feature_bits && im.smem_limit == smem_limit;
}

int tbk_forest_create_from_image(const tbk_image *img, const tbk_schedule *schedule, int32_t device,
                                 int64_t batch_hint, tbk_forest **out) {
  if (!img || !out) return fail(TBK_ERR_INVALID, "null argument");
  *out = nullptr;
  const tb::PackedImage &im = img->im;
  auto *f = new tbk_forest();
  f->user = im.user;
  if (schedule) { // launch-shape requests of the caller; the layout is the image's
    f->user.rows_per_block = schedule->rows_per_block;
    f->user.rows_per_thread = schedule->rows_per_thread;
    f->user.tree_threads = schedule->tree_threads;
    f->user.tree_chunks = schedule->tree_chunks;
    f->user.cache_trees = schedule->cache_trees;
  }
  f->batch_hint = batch_hint;
  f->device = device;
  auto bail = [&](int rc) {
    tbk_forest_free(f);
    return rc;
  };
#define CUDA_TRY_F(expr)                                                                   \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return bail(fail(TBK_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)));    \
  } while (0)
  CUDA_TRY_F(cudaSetDevice(device));
  CUDA_TRY_F(cudaDeviceGetAttribute(&f->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  CUDA_TRY_F(cudaDeviceGetAttribute(&f->num_sms, cudaDevAttrMultiProcessorCount, device));
  if (im.smem_limit > f->max_smem_optin)
    return bail(fail(TBK_ERR_UNSUPPORTED, "the packed image was laid out for %d bytes of shared memory per block, this device has %d",
                     im.smem_limit, f->max_smem_optin));
  CUDA_TRY_F(cudaMalloc(&f->d_status, 4));
  CUDA_TRY_F(cudaMemset(f->d_status, 0, 4));
  CUDA_TRY_F(cudaEventCreate(&f->ev0));
  CUDA_TRY_F(cudaEventCreate(&f->ev1));

  if (im.kind == tb::PackedImage::kDeep) {
    f->df = im.df; // (metadata and planes; the planes' host copies are dropped after the upload)
    auto &q = f->df;
    f->deep = true;
    f->deep_row_warps = im.deep_row_warps;
    f->deep_slots = im.deep_slots;
    f->packed.representation = tb::kReorg;
    f->packed.tile_size = 1;
    f->packed.num_features = q.num_features;
    f->packed.transform = q.transform;
    f->packed.initial_value = q.initial_value;
    f->packed.num_trees = q.num_trees;
    f->packed.num_nodes = q.num_nodes;
    f->packed.max_depth = q.max_depth;
    int urc = upload_key_planes(f, q.node_plane, q.leaf_plane, q.exact_plane, q.orig_leaf, q.pairs, q.tree_index,
                                q.lo, q.scale, q.num_features, false);
    if (urc != TBK_OK) return bail(urc);
    std::vector<uint32_t>().swap(q.node_plane);
    std::vector<float>().swap(q.leaf_plane);
    std::vector<float>().swap(q.exact_plane);
    std::vector<int32_t>().swap(q.orig_leaf);
    tb::LaunchPlan &pl = f->last_plan;
    pl.row_warps = f->deep_row_warps; pl.tree_threads = 1; pl.rows_per_lane = 1; pl.chunks = 1; pl.staged = 1; pl.cache_rows = 1;
    pl.stage_bytes = 4u << std::max(q.max_depth, tb::kDeepMinDepth); pl.smem_bytes = deep_smem_bytes(f); pl.threads = 32 * (f->deep_row_warps + 1);
    *out = f;
    return TBK_OK;
  }
  if (im.kind == tb::PackedImage::kQuant) {
    f->qf = im.qf;
    const auto &q = f->qf;
    f->quant = true;
    // metadata shared with the generic entry points
    f->packed.representation = tb::kReorg;
    f->packed.tile_size = 1;
    f->packed.num_features = q.num_features;
    f->packed.num_classes = q.num_classes;
    f->packed.transform = q.transform;
    f->packed.initial_value = q.initial_value;
    f->packed.num_trees = q.num_trees;
    f->packed.num_nodes = q.num_nodes;
    f->packed.max_depth = q.max_depth;
    int urc = upload_key_planes(f, q.node_plane, q.leaf_plane, q.exact_plane, q.orig_leaf, q.groups, q.tree_index,
                                q.lo, q.scale, q.num_features, true);
    if (urc != TBK_OK) return bail(urc);
    if (q.num_classes > 0) {
      // every class goes to one of the two walker sets, whichever has fewer groups so far;
      // within a set the groups keep their order, so its classes come in increasing order
      const size_t G = q.groups.size();
      std::vector<int32_t> lists(2 * G, 0);
      int32_t count[2] = {0, 0};
      for (size_t g = 0; g < G;) {
        size_t e = g;
        while (e < G && q.group_class[e] == q.group_class[g]) ++e;
        const int s = count[1] < count[0] ? 1 : 0;
        for (; g < e; ++g) lists[(size_t)s * G + count[s]++] = (int32_t)g;
      }
      f->qset_count[0] = count[0];
      f->qset_count[1] = count[1];
      CUDA_TRY_F(cudaMalloc(&f->d_qset_groups, lists.size() * 4));
      CUDA_TRY_F(cudaMemcpy(f->d_qset_groups, lists.data(), lists.size() * 4, cudaMemcpyHostToDevice));
      CUDA_TRY_F(cudaMalloc(&f->d_qgroup_class, G * 4));
      CUDA_TRY_F(cudaMemcpy(f->d_qgroup_class, q.group_class.data(), G * 4, cudaMemcpyHostToDevice));
    }
    // host copies of the big planes are no longer needed
    std::vector<uint32_t>().swap(f->qf.node_plane);
    std::vector<float>().swap(f->qf.leaf_plane);
    std::vector<float>().swap(f->qf.exact_plane);
    std::vector<int32_t>().swap(f->qf.orig_leaf);
    tb::LaunchPlan &pl = f->last_plan;
    pl.row_warps = 1; pl.tree_threads = tb::kQWalkers; pl.rows_per_lane = 1; pl.chunks = 1; pl.staged = 1; pl.cache_rows = 1;
    pl.stage_bytes = tb::kQPiece; pl.smem_bytes = quant_smem_bytes(q.num_features); pl.threads = tb::kQThreads;
    if (const int batch = quant_batch_tiles(f, q.num_features)) { // narrow rows: the batch kernel
      pl.row_warps = batch;
      pl.smem_bytes = tb::quant_batch_smem_bytes(q.num_features, batch);
      pl.threads = tb::kQBThreads;
    }
    *out = f;
    return TBK_OK;
  }

  f->packed = im.packed;
  const auto &p = f->packed;
  CUDA_TRY_F(cudaMalloc(&f->d_blob, std::max<size_t>(16, p.blob.size())));
  CUDA_TRY_F(cudaMemcpy(f->d_blob, p.blob.data(), p.blob.size(), cudaMemcpyHostToDevice));
  static_assert(sizeof(tb::GroupMeta) == sizeof(tb::DevGroupMeta), "group metadata layout");
  CUDA_TRY_F(cudaMalloc(&f->d_groups, p.groups.size() * sizeof(tb::GroupMeta)));
  CUDA_TRY_F(cudaMemcpy(f->d_groups, p.groups.data(), p.groups.size() * sizeof(tb::GroupMeta), cudaMemcpyHostToDevice));
  CUDA_TRY_F(cudaMalloc(&f->d_tree_class, p.tree_class.size() * 2));
  CUDA_TRY_F(cudaMemcpy(f->d_tree_class, p.tree_class.data(), p.tree_class.size() * 2, cudaMemcpyHostToDevice));
  CUDA_TRY_F(cudaMalloc(&f->d_tree_index, p.tree_index.size() * 4));
  CUDA_TRY_F(cudaMemcpy(f->d_tree_index, p.tree_index.data(), p.tree_index.size() * 4, cudaMemcpyHostToDevice));
  CUDA_TRY_F(cudaMalloc(&f->d_lut, std::max<size_t>(16, p.lut.size())));
  CUDA_TRY_F(cudaMemcpy(f->d_lut, p.lut.data(), p.lut.size(), cudaMemcpyHostToDevice));
  // the packed blob is only needed on the device from here on
  std::vector<uint8_t>().swap(f->packed.blob);
  // settle the plan for the hinted batch so that get_info can report it
  tb::ForestShape shape{p.num_features, p.num_classes, (int64_t)p.groups.size(), p.max_group_bytes,
                        (int32_t)p.lut.size(), p.representation, p.tile_size};
  std::string why = tb::select_launch(shape, f->user, batch_hint > 0 ? batch_hint : 65536, f->max_smem_optin,
                                      f->num_sms, false, &f->last_plan);
  if (!why.empty()) return bail(fail(TBK_ERR_UNSUPPORTED, "%s", why.c_str()));
  *out = f;
  return TBK_OK;
}

int tbk_forest_free(tbk_forest *f) {
  if (!f) return TBK_OK;
  cudaSetDevice(f->device);
  free_pipeline(f);
  for (int i = 0; i < 2; ++i) {
    if (f->streams[i]) cudaStreamDestroy(f->streams[i]);
    if (f->in_free[i]) cudaEventDestroy(f->in_free[i]);
  }
  cudaFree(f->d_blob);
  cudaFree(f->d_groups);
  cudaFree(f->d_tree_class);
  cudaFree(f->d_tree_index);
  cudaFree(f->d_orig_node);
  cudaFree(f->d_orig_off);
  cudaFree(f->d_lut);
  cudaFree(f->d_status);
  cudaFree(f->d_scratch);
  cudaFree(f->d_qnode);
  cudaFree(f->d_qleaf);
  cudaFree(f->d_qexact);
  cudaFree(f->d_qorig);
  cudaFree(f->d_qgroups);
  cudaFree(f->d_qtree_index);
  cudaFree(f->d_qset_groups);
  cudaFree(f->d_qgroup_class);
  cudaFree(f->d_qlo);
  cudaFree(f->d_qscale);
  cudaFree(f->d_ties);
  for (int i = 0; i < 2; ++i)
    if (f->scratch_done[i]) cudaEventDestroy(f->scratch_done[i]);
  if (f->ev0) cudaEventDestroy(f->ev0);
  if (f->ev1) cudaEventDestroy(f->ev1);
  delete f;
  return TBK_OK;
}

int tbk_forest_get_info(const tbk_forest *f, tbk_forest_info *info) {
  if (!f || !info) return fail(TBK_ERR_INVALID, "null argument");
  std::memset(info, 0, sizeof *info);
  const auto &p = f->packed;
  info->num_trees = p.num_trees;
  info->num_nodes = p.num_nodes;
  info->num_groups = f->quant ? (int64_t)f->qf.groups.size() : f->deep ? (int64_t)f->df.pairs.size() : (int64_t)p.groups.size();
  info->packed_bytes = f->deep ? (int64_t)(f->df.pairs.empty() ? 0 : 8 * (f->df.pairs.back().elem_off + 2ull * f->df.pairs.back().slots)) :
                       f->quant ? (int64_t)(f->qf.groups.empty() ? 0 : 8 * (f->qf.groups.back().elem_off + (uint64_t)f->qf.groups.back().slots * tb::kQuantCols)) :
                       p.groups.empty() ? 0 : (int64_t)(p.groups.back().byte_off +
      (((uint64_t)p.groups.back().slots * tb::kGroupTrees * p.tile_bytes + 15) & ~15ull));
  info->max_depth = p.max_depth;
  info->num_features = p.num_features;
  info->num_classes = p.num_classes;
  info->transform = p.transform;
  info->device = f->device;
  const tb::LaunchPlan &pl = f->last_plan;
  info->schedule.representation = p.representation;
  info->schedule.tile_size = p.tile_size;
  info->schedule.rows_per_block = pl.row_warps * 32 * pl.rows_per_lane;
  info->schedule.rows_per_thread = pl.rows_per_lane;
  info->schedule.tree_threads = pl.tree_threads;
  info->schedule.tree_chunks = pl.chunks;
  info->schedule.cache_trees = pl.staged ? 1 : 2;
  info->schedule.feature_bits = (f->quant || f->deep) ? 16 : 32;
  info->staged = pl.staged;
  info->smem_bytes = pl.smem_bytes;
  info->threads_per_block = pl.threads;
  if ((f->quant || f->deep) && f->d_ties) {
    // key ties resolved on exact values so far (statistics; synchronises with the device)
    unsigned long long ties = 0;
    if (cudaMemcpy(&ties, f->d_ties, 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
      info->reserved[0] = (int32_t)(ties & 0x7fffffff);
      info->reserved[1] = (int32_t)(ties >> 31);
    }
  }
  return TBK_OK;
}

int tbk_predict(tbk_forest *f, const float *d_rows, int64_t n_rows, int64_t ld, void *d_out,
                int32_t out_kind, void *stream) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  std::lock_guard<std::mutex> lock(f->mu);
  return run(f, kPredict, d_rows, n_rows, ld, d_out, out_kind, nullptr, nullptr, (cudaStream_t)stream);
}

int tbk_predict_partial(tbk_forest *f, const float *d_rows, int64_t n_rows, int64_t ld, float *d_partial,
                        void *stream) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  if (!d_partial && n_rows > 0) return fail(TBK_ERR_INVALID, "null output pointer");
  std::lock_guard<std::mutex> lock(f->mu);
  return run(f, kPartial, d_rows, n_rows, ld, nullptr, TBK_OUT_F32, d_partial, nullptr, (cudaStream_t)stream);
}

int tbk_finalize(tbk_forest *f, const float *d_partial, int64_t n_rows, void *d_out, int32_t out_kind,
                 void *stream) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  if (n_rows == 0) return TBK_OK;
  if (!d_partial || !d_out) return fail(TBK_ERR_INVALID, "null pointer");
  const auto &p = f->packed;
  if (out_kind == TBK_OUT_I8 && p.num_classes == 0) return fail(TBK_ERR_INVALID, "int8 output needs a multiclass forest");
  std::lock_guard<std::mutex> lock(f->mu);
  CUDA_TRY(cudaSetDevice(f->device));
  const int tpb = 256;
  tb::tb_finalize_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, (cudaStream_t)stream>>>(
      d_partial, 1, n_rows, std::max(1, p.num_classes), p.num_classes, (float)p.initial_value, p.transform, d_out, out_kind);
  CUDA_TRY(cudaGetLastError());
  ++f->launches;
  return TBK_OK;
}

int tbk_predict_leaf_ids(tbk_forest *f, const float *d_rows, int64_t n_rows, int64_t ld,
                         int32_t *d_leaf_ids, void *stream) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  if (!d_leaf_ids && n_rows > 0) return fail(TBK_ERR_INVALID, "null output pointer");
  std::lock_guard<std::mutex> lock(f->mu);
  return run(f, kLeafIds, d_rows, n_rows, ld, nullptr, TBK_OUT_F32, nullptr, d_leaf_ids, (cudaStream_t)stream);
}

int tbk_predict_host(tbk_forest *f, const float *h_rows, int64_t n_rows, int64_t ld, void *h_out,
                     int32_t out_kind) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  if (n_rows == 0) return TBK_OK;
  if (!h_rows || !h_out) return fail(TBK_ERR_INVALID, "null pointer");
  std::lock_guard<std::mutex> lock(f->mu);
  CUDA_TRY(cudaSetDevice(f->device));
  const size_t out_elt = out_kind == TBK_OUT_I8 ? 1 : 4;
  // chunk size: about 64 MiB of features, a multiple of 1024 rows
  size_t chunk = std::max<size_t>(1024, ((size_t)64 << 20) / ((size_t)ld * 4) / 1024 * 1024);
  chunk = std::min<size_t>(chunk, ((size_t)n_rows + 1023) / 1024 * 1024);
  if (!f->streams[0]) {
    for (int i = 0; i < 2; ++i) {
      CUDA_TRY(cudaStreamCreateWithFlags(&f->streams[i], cudaStreamNonBlocking));
      CUDA_TRY(cudaEventCreateWithFlags(&f->in_free[i], cudaEventDisableTiming));
    }
  }
  cudaPointerAttributes attr{};
  const bool in_pinned = cudaPointerGetAttributes(&attr, h_rows) == cudaSuccess && attr.type == cudaMemoryTypeHost;
  cudaGetLastError();
  cudaPointerAttributes oattr{};
  const bool out_pinned = cudaPointerGetAttributes(&oattr, h_out) == cudaSuccess && oattr.type == cudaMemoryTypeHost;
  cudaGetLastError();
  if (f->pipe_rows < chunk || f->pipe_ld != (size_t)ld) {
    free_pipeline(f);
    for (int i = 0; i < 2; ++i) {
      CUDA_TRY(cudaMalloc(&f->d_in[i], chunk * ld * 4));
      CUDA_TRY(cudaMalloc(&f->d_res[i], chunk * 4));
    }
    f->pipe_rows = chunk;
    f->pipe_ld = (size_t)ld;
  }
  if (!in_pinned && !f->h_pin[0])
    for (int i = 0; i < 2; ++i) CUDA_TRY(cudaMallocHost(&f->h_pin[i], f->pipe_rows * ld * 4));
  if (!out_pinned && f->h_res_bytes < (size_t)n_rows * out_elt) {
    if (f->h_res) CUDA_TRY(cudaFreeHost(f->h_res));
    f->h_res = nullptr;
    CUDA_TRY(cudaMallocHost(&f->h_res, (size_t)n_rows * out_elt));
    f->h_res_bytes = (size_t)n_rows * out_elt;
  }
  unsigned char *res_dst = out_pinned ? static_cast<unsigned char *>(h_out) : f->h_res;
  const bool was_timing = f->timing;
  f->timing = false; // per-chunk launches overlap on two streams; event timing does not apply
  int rc = TBK_OK;
  int64_t done = 0;
  for (int it = 0; done < n_rows && rc == TBK_OK; ++it) {
    const int s = it & 1;
    const int64_t n = std::min<int64_t>((int64_t)chunk, n_rows - done);
    const float *src = h_rows + done * ld;
    if (!in_pinned) {
      // the staging buffer is free once the copy that last read it has finished
      cudaError_t e = cudaEventSynchronize(f->in_free[s]);
      if (e != cudaSuccess) { rc = fail(TBK_ERR_CUDA, "cudaEventSynchronize: %s", cudaGetErrorString(e)); break; }
      std::memcpy(f->h_pin[s], src, (size_t)n * ld * 4);
      src = f->h_pin[s];
    }
    cudaError_t e = cudaMemcpyAsync(f->d_in[s], src, (size_t)n * ld * 4, cudaMemcpyHostToDevice, f->streams[s]);
    if (e == cudaSuccess) e = cudaEventRecord(f->in_free[s], f->streams[s]);
    if (e != cudaSuccess) { rc = fail(TBK_ERR_CUDA, "host-to-device copy: %s", cudaGetErrorString(e)); break; }
    rc = run(f, kPredict, f->d_in[s], n, ld, f->d_res[s], out_kind, nullptr, nullptr, f->streams[s], s);
    if (rc != TBK_OK) break;
    e = cudaMemcpyAsync(res_dst + done * out_elt, f->d_res[s], (size_t)n * out_elt, cudaMemcpyDeviceToHost, f->streams[s]);
    if (e != cudaSuccess) { rc = fail(TBK_ERR_CUDA, "device-to-host copy: %s", cudaGetErrorString(e)); break; }
    done += n;
  }
  for (int i = 0; i < 2; ++i) {
    cudaError_t e = cudaStreamSynchronize(f->streams[i]);
    if (e != cudaSuccess && rc == TBK_OK) rc = fail(TBK_ERR_CUDA, "cudaStreamSynchronize: %s", cudaGetErrorString(e));
  }
  f->timing = was_timing;
  if (rc != TBK_OK) return rc;
  if (!out_pinned) std::memcpy(h_out, f->h_res, (size_t)n_rows * out_elt);
  return check_status(f);
}

int tbk_set_timing(tbk_forest *f, int32_t enable) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  f->timing = enable != 0;
  f->ev_pending = false;
  return TBK_OK;
}

int64_t tbk_last_kernel_time_us(tbk_forest *f) {
  if (!f || !f->ev_pending) return -1;
  if (cudaEventSynchronize(f->ev1) != cudaSuccess) return -1;
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, f->ev0, f->ev1) != cudaSuccess) return -1;
  return (int64_t)(ms * 1000.0f + 0.5f);
}

int64_t tbk_launch_count(const tbk_forest *f) { return f ? f->launches : 0; }

int tbk_check_status(tbk_forest *f) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  return check_status(f);
}

int tbk_debug_expire_next_wait(tbk_forest *f) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  std::lock_guard<std::mutex> lock(f->mu);
  f->expire_next_wait = true;
  return TBK_OK;
}

} // extern "C"

// ---------------------------------------------------------------------------
// Prediction for callers that must not allocate.
//
// Some hosts of this library may not call cudaMalloc on the prediction path: a serving
// loop whose memory is fixed at start-up (a pool carved once, with nothing left over for
// the driver to hand out later), a latency-critical thread that cannot afford the implicit
// device synchronisation an allocation may bring, or an embedding runtime whose policy
// forbids device allocations outside its own allocator.  tbk_predict sizes its tree-chunk
// partial sums at run time and grows a cudaMalloc'ed buffer when a larger batch arrives;
// this variant runs the same two kernels (walk into per-chunk partials, then the
// atomic-free second pass) with the partials in a fixed array that is part of the loaded
// library image, so it never allocates or frees anything.
//
// The array lives on every GPU that loads the library, from load until the process exits
// (kNoAllocScratchFloats * 4 bytes = 8 MiB per GPU).  In host code its name is only a
// stand-in for the device object; the device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that address is what the kernels
// receive.

namespace {

constexpr size_t kNoAllocScratchFloats = size_t(1) << 21; // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
float *g_noalloc_addr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

// Device address of the scratch array on `device` (which must be current).
int noalloc_scratch_address(int device, float **out) {
  if (device < 0 || device >= kMaxDevices) return fail(TBK_ERR_INVALID, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_addr[device]) {
    float *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(TBK_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", device, cudaGetErrorString(e));
    g_noalloc_addr[device] = ptr;
  }
  *out = g_noalloc_addr[device];
  return TBK_OK;
}

} // namespace

extern "C" int tbk_predict_noalloc(tbk_forest *f, const float *d_rows, int64_t n_rows, int64_t ld, void *d_out,
                                   int32_t out_kind, void *stream_) {
  if (!f) return fail(TBK_ERR_INVALID, "null forest");
  std::lock_guard<std::mutex> lock(f->mu);
  const auto &pk = f->packed;
  if (f->quant || f->deep) return fail(TBK_ERR_UNSUPPORTED, "tbk_predict_noalloc does not cover the 16-bit key layouts");
  if (n_rows < 0 || ld < pk.num_features) return fail(TBK_ERR_INVALID, "ld (%lld) is smaller than the row size (%d)", (long long)ld, pk.num_features);
  if (n_rows == 0) return TBK_OK;
  if (!d_rows || !d_out) return fail(TBK_ERR_INVALID, "null pointer");
  if (out_kind != TBK_OUT_F32 && out_kind != TBK_OUT_I8) return fail(TBK_ERR_INVALID, "unknown output kind %d", out_kind);
  if (out_kind == TBK_OUT_I8 && pk.num_classes == 0) return fail(TBK_ERR_INVALID, "int8 output needs a multiclass forest");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  CUDA_TRY(cudaSetDevice(f->device));
  float *scratch = nullptr;
  int rc = noalloc_scratch_address(f->device, &scratch);
  if (rc != TBK_OK) return rc;

  tb::ForestShape shape{pk.num_features, pk.num_classes, (int64_t)pk.groups.size(), pk.max_group_bytes,
                        (int32_t)pk.lut.size(), pk.representation, pk.tile_size};
  tb::LaunchPlan plan;
  // this call always writes partial sums, so the plan must be one for partial output: its
  // shared memory then includes the per-warp class table of a multiclass forest
  std::string why = tb::select_launch(shape, f->user, n_rows, f->max_smem_optin, f->num_sms, false, &plan, true);
  if (!why.empty()) return fail(TBK_ERR_UNSUPPORTED, "%s", why.c_str());
  if (plan.class_regs)
    return fail(TBK_ERR_UNSUPPORTED, "tbk_predict_noalloc: launch plan keeps class sums in registers and cannot write partial sums");
  const int W = std::max(1, pk.num_classes);
  const size_t need = (size_t)plan.chunks * (size_t)n_rows * (size_t)W;
  if (need > kNoAllocScratchFloats)
    return fail(TBK_ERR_UNSUPPORTED,
                "tbk_predict_noalloc: %lld rows x %d tree chunks x %d outputs need %zu partial sums, the fixed scratch "
                "holds %zu; split the batch or use tbk_predict",
                (long long)n_rows, plan.chunks, W, need, kNoAllocScratchFloats);

  tb::WalkParams p{};
  p.blob = f->d_blob;
  p.groups = f->d_groups;
  p.tree_class = f->d_tree_class;
  p.tree_index = f->d_tree_index;
  p.lut = f->d_lut;
  p.lut_bytes = (int32_t)pk.lut.size();
  p.rows = d_rows;
  p.n_rows = n_rows;
  p.ld = ld;
  p.partial = scratch; // every (chunk, row, output) element is written by the walk: nothing to clear
  p.out = d_out;
  p.out_kind = out_kind;
  p.write_partial = 1;
  p.num_trees = pk.num_trees;
  p.num_groups = (int32_t)pk.groups.size();
  p.groups_per_chunk = plan.groups_per_chunk;
  p.num_features = pk.num_features;
  p.num_classes = pk.num_classes;
  p.transform = pk.transform;
  p.initial_value = (float)pk.initial_value;
  p.row_warps = plan.row_warps;
  p.tree_threads = plan.tree_threads;
  p.stage_bytes = plan.staged ? plan.stage_bytes : 0;
  p.vec4_ok = (pk.num_features % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(d_rows) & 15) == 0) ? 1 : 0;
  p.status = f->d_status;
  p.class_regs = 0; // class sums go through the shared-memory table the plan has sized
  KernelFn fn = pick_kernel(pk.representation, pk.tile_size, plan.rows_per_lane, plan.staged, plan.cache_rows);
  CUDA_TRY(cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));
  dim3 grid((unsigned)plan.grid_x, (unsigned)plan.chunks), block((unsigned)plan.threads);
  fn<<<grid, block, plan.smem_bytes, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
  const int tpb = 256;
  tb::tb_finalize_kernel<<<(unsigned)((n_rows + tpb - 1) / tpb), tpb, 0, stream>>>(
      scratch, plan.chunks, n_rows, W, pk.num_classes, (float)pk.initial_value, pk.transform, d_out, out_kind);
  CUDA_TRY(cudaGetLastError());
  f->launches += 2;
  return TBK_OK;
}

// ---------------------------------------------------------------------------
// Host-only utilities (no device is touched).

extern "C" {

int tbk_host_layout_check(const tbk_forest_arrays *fa, const tbk_schedule *schedule, const float *rows,
                          int64_t n_rows, int64_t ld, int32_t *leaf_ids, float *sums,
                          tbk_forest_info *info) {
  if (!fa || fa->num_trees <= 0) return fail(TBK_ERR_INVALID, "null or empty forest");
  tb::Forest host;
  const int64_t T = fa->num_trees, N = fa->tree_off[T];
  host.tree_off.assign(fa->tree_off, fa->tree_off + T + 1);
  host.left.assign(fa->left, fa->left + N);
  host.right.assign(fa->right, fa->right + N);
  host.feat.assign(fa->feat, fa->feat + N);
  host.thr.assign(fa->thr, fa->thr + N);
  if (fa->num_classes > 0 && fa->class_id) host.class_id.assign(fa->class_id, fa->class_id + T);
  host.num_classes = fa->num_classes;
  host.transform = fa->transform;
  host.initial_value = fa->initial_value;
  host.num_features = fa->num_features;
  if (schedule && schedule->feature_bits == 16) {
    // the key layouts: groups of 32 trees up to 8 levels, whole-tree stages beyond
    int max_depth = 0;
    {
      const std::string verr = tb::validate(host);
      if (!verr.empty()) return fail(TBK_ERR_INVALID, "%s", verr.c_str());
      for (int64_t t = 0; t < T; ++t) max_depth = std::max(max_depth, (int)tb::tree_depth(host, t));
    }
    int64_t ties = 0, groups = 0, elems = 0;
    if (max_depth <= tb::kQuantMaxDepth) {
      tb::QuantForest q;
      // (lattice features where the rows are narrow enough for the batch kernel, as at upload)
      const bool narrow = (227 * 1024 - tb::kQBBarBytes - tb::kQBRingBytes) / tb::quant_batch_tile_bytes(host.num_features) >= 4;
      std::string qerr = tb::pack_quant(host, &q, narrow);
      if (!qerr.empty()) return fail(TBK_ERR_UNSUPPORTED, "%s", qerr.c_str());
      if (rows && n_rows > 0) tb::walk_quant_on_host(q, rows, n_rows, ld, leaf_ids, sums, &ties);
      groups = (int64_t)q.groups.size();
      elems = (int64_t)q.node_plane.size();
    } else {
      tb::DeepForest q;
      std::string qerr = tb::pack_deep(host, &q);
      if (!qerr.empty()) return fail(TBK_ERR_UNSUPPORTED, "%s", qerr.c_str());
      if (rows && n_rows > 0) tb::walk_deep_on_host(q, rows, n_rows, ld, leaf_ids, sums, &ties);
      groups = (int64_t)q.pairs.size();
      elems = (int64_t)q.node_plane.size();
    }
    if (info) {
      std::memset(info, 0, sizeof *info);
      info->num_trees = T;
      info->num_nodes = N;
      info->num_groups = groups;
      info->packed_bytes = elems * 8;
      info->max_depth = max_depth;
      info->num_features = host.num_features;
      info->transform = host.transform;
      info->schedule.representation = TBK_REP_REORG;
      info->schedule.tile_size = 1;
      info->schedule.feature_bits = 16;
      info->reserved[0] = (int32_t)std::min<int64_t>(ties, 0x7fffffff);
    }
    return TBK_OK;
  }
  tb::PackOptions opt;
  opt.representation = schedule && schedule->representation >= 0 ? schedule->representation : 0;
  opt.tile_size = schedule && schedule->tile_size > 0 ? schedule->tile_size : 1;
  tb::PackedForest packed;
  std::string err = tb::pack_forest(host, opt, &packed);
  if (!err.empty()) return fail(TBK_ERR_INVALID, "%s", err.c_str());
  if (info) {
    std::memset(info, 0, sizeof *info);
    info->num_trees = packed.num_trees;
    info->num_nodes = packed.num_nodes;
    info->num_groups = (int64_t)packed.groups.size();
    info->packed_bytes = (int64_t)packed.blob.size();
    info->max_depth = packed.max_depth;
    info->num_features = packed.num_features;
    info->num_classes = packed.num_classes;
    info->transform = packed.transform;
    info->schedule.representation = packed.representation;
    info->schedule.tile_size = packed.tile_size;
    info->reserved[0] = packed.num_shapes;
    info->reserved[1] = (int32_t)packed.lut.size();
    info->reserved[2] = (int32_t)std::min<uint64_t>(packed.max_group_bytes, 0x7fffffff);
  }
  if (rows && n_rows > 0) tb::walk_packed_on_host(packed, rows, n_rows, ld, leaf_ids, sums);
  return TBK_OK;
}

int tbk_plan_launch(int32_t num_features, int32_t num_classes, int64_t num_groups, int64_t max_group_bytes,
                    int32_t lut_bytes, const tbk_schedule *schedule, int64_t n_rows, int32_t smem_limit,
                    int32_t num_sms, int32_t partial_sums, tbk_forest_info *info) {
  if (!info) return fail(TBK_ERR_INVALID, "null argument");
  tbk_schedule user{};
  if (schedule) user = *schedule;
  tb::ForestShape shape{num_features, num_classes, num_groups, (uint64_t)max_group_bytes, lut_bytes,
                        user.representation, user.tile_size > 0 ? user.tile_size : 1};
  tb::LaunchPlan pl;
  std::string why = tb::select_launch(shape, user, n_rows, smem_limit, num_sms, false, &pl, partial_sums != 0);
  if (!why.empty()) return fail(TBK_ERR_UNSUPPORTED, "%s", why.c_str());
  std::memset(info, 0, sizeof *info);
  info->schedule = user;
  info->schedule.rows_per_block = pl.row_warps * 32 * pl.rows_per_lane;
  info->schedule.rows_per_thread = pl.rows_per_lane;
  info->schedule.tree_threads = pl.tree_threads;
  info->schedule.tree_chunks = pl.chunks;
  info->schedule.cache_trees = pl.staged ? 1 : 2;
  info->staged = pl.staged;
  info->smem_bytes = pl.smem_bytes;
  info->threads_per_block = pl.threads;
  info->reserved[0] = pl.cache_rows;
  info->reserved[1] = (int32_t)std::min<int64_t>(pl.grid_x, 0x7fffffff);
  info->reserved[2] = pl.groups_per_chunk;
  info->reserved[3] = pl.class_regs;
  return TBK_OK;
}

} // extern "C"
