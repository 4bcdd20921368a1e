// Tree-walk kernels for sm_100a.
//
// Work decomposition (what the reference expresses as a schedule over the (row, tree)
// iteration space, src/mlir/GPUAutoSchedule.cpp:355-403):
//   grid.x  -> row tiles of (row_warps * 32 * RPL) rows
//   grid.y  -> tree chunks (ranges of 16-tree groups); partial sums of the chunks are
//              combined by a second, atomic-free pass
//   block   -> row_warps * tree_threads warps.  A warp owns 32*RPL rows (lane = row,
//              RPL rows per lane walked in lock-step for instruction-level
//              parallelism); the tree_threads warps that share a row tile split the 16
//              columns of every group between them.
//
// The walk (reference: src/mlir/CodeGenStateMachine.cpp:149-243 scalar step,
// :284-507 tile step with look-up table, src/mlir/WalkDecisionTreeLoweringPass.cpp:24-53
// fixed-depth walk of padded trees) is branch-free: every tree of a group is walked
// for exactly the group's depth; leaves route back to themselves through the sentinel
// feature (see pack.h).  At shift s lane j walks column (j + s) mod 16, so the 32
// lanes of a warp always address 16 distinct tile columns (bank-conflict free in the
// slot-major interleaved layout) and, in the transposed row tile xs[feature][row],
// 32 distinct banks.
//
// Tree groups are staged into shared memory with cp.async.bulk (the TMA unit's
// untiled bulk copy) into a two-stage ring guarded by mbarriers; feature rows are
// read with 16-byte loads and transposed through shared memory.  The reference's
// counterparts are the cooperative row cache (src/gpu/GPURepresentations.cpp:279-399)
// and tree cache (:630-715).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tb {

struct DevGroupMeta {
  unsigned long long byte_off;
  uint32_t slots;
  uint32_t depth;
};

struct WalkParams {
  const uint8_t *blob;
  const DevGroupMeta *groups;
  const int16_t *tree_class;
  const int32_t *tree_index;
  const int32_t *orig_node;
  const unsigned long long *orig_off;
  const int8_t *lut;
  int32_t lut_bytes;
  const float *rows;
  long long n_rows;
  long long ld;
  float *partial;      // [chunks][n_rows][W]; used when write_partial != 0
  void *out;
  int32_t out_kind;
  int32_t write_partial;
  int32_t *leaf_ids;   // [n_rows][num_trees] or null
  long long num_trees;
  int32_t num_groups;
  int32_t groups_per_chunk;
  int32_t num_features;
  int32_t num_classes;
  int32_t transform;
  float initial_value;
  int32_t row_warps;
  int32_t tree_threads;
  uint32_t stage_bytes; // capacity of one stage (0 when not staged)
  int32_t vec4_ok;      // rows can be read with 16-byte loads
  int32_t class_regs;   // multiclass: class sums in registers, arg-max decided on the fly
  int32_t *status;      // device status word, 0 = ok
  uint32_t wait_limit;  // polls before a wait on a stage gives up (0 = kWaitLimit)
  int32_t skip_first_copy; // failure drill: the first stage's copy is never issued, so its wait expires
};

constexpr int kCols = 16;
constexpr uint32_t kWaitLimit = 1u << 22;

// --------------------------------------------------------------------------
// mbarrier / bulk-copy primitives

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               " selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = kWaitLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_test(bar, parity)) return true;
    if (it > 64) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------------
// tile decode: loads the tile at (slot n, column col) and returns the next slot.

template <bool SMEM> __device__ __forceinline__ uint2 ld2(const void *p) {
  if (SMEM) return *reinterpret_cast<const uint2 *>(p);
  return __ldg(reinterpret_cast<const uint2 *>(p));
}
template <bool SMEM> __device__ __forceinline__ uint4 ld4(const void *p) {
  if (SMEM) return *reinterpret_cast<const uint4 *>(p);
  return __ldg(reinterpret_cast<const uint4 *>(p));
}

struct RowAccess {
  const float *xs;      // cached: transposed tile base (+ lane offset applied)
  const float *grow;    // uncached: row base in global memory
  int32_t num_features;
};

// RT = floats between consecutive features of the transposed row tile.
template <bool CACHED, int RT> __device__ __forceinline__ float feature(const RowAccess &ra, uint32_t f) {
  if (CACHED) return ra.xs[f * RT];
  return f == (uint32_t)ra.num_features ? __int_as_float(0xff800000) : __ldg(ra.grow + f);
}

// REP: 0 sparse, 1 array, 2 reorg.  Returns the leaf value after `depth` steps and
// the final slot in *slot_out.
template <int REP, int TS, bool SMEM, bool CACHED, int RT>
__device__ __forceinline__ float walk_one(const uint8_t *gbase, uint32_t slots, uint32_t depth, uint32_t col,
                                          const RowAccess &ra, const int8_t *lut, uint32_t *slot_out) {
  uint32_t n = 0;
  if (REP == 2) {
    const float *thr = reinterpret_cast<const float *>(gbase);
    const uint16_t *feat = reinterpret_cast<const uint16_t *>(gbase + (size_t)slots * kCols * 4);
    for (uint32_t d = 0; d < depth; ++d) {
      const uint32_t i = n * kCols + col;
      const float t = SMEM ? thr[i] : __ldg(thr + i);
      const uint32_t f = SMEM ? feat[i] : __ldg(feat + i);
      const float x = feature<CACHED, RT>(ra, f);
      n = 2 * n + 1 + !(x < t);
    }
    *slot_out = n;
    const uint32_t i = n * kCols + col;
    return SMEM ? thr[i] : __ldg(thr + i);
  }
  constexpr int TB = TS == 1 ? 8 : TS == 2 ? 16 : TS == 3 ? 24 : 32;
  for (uint32_t d = 0; d < depth; ++d) {
    const uint8_t *tp = gbase + (size_t)(n * kCols + col) * TB;
    uint32_t k, child;
    if (TS == 1) {
      const uint2 t = ld2<SMEM>(tp);
      const float x = feature<CACHED, RT>(ra, t.y & 0xffffu);
      child = t.y >> 16;
      k = !(x < __uint_as_float(t.x));
    } else {
      float thr[TS];
      uint32_t f[TS], shape;
      if (TS == 2) {
        const uint4 t = ld4<SMEM>(tp);
        thr[0] = __uint_as_float(t.x); thr[1] = __uint_as_float(t.y);
        f[0] = t.z & 0xffffu; f[1] = t.z >> 16;
        shape = t.w & 0xffffu; child = t.w >> 16;
      } else if (TS == 3) {
        const uint2 a = ld2<SMEM>(tp), b = ld2<SMEM>(tp + 8), c = ld2<SMEM>(tp + 16);
        thr[0] = __uint_as_float(a.x); thr[1] = __uint_as_float(a.y); thr[2] = __uint_as_float(b.x);
        f[0] = b.y & 0xffffu; f[1] = b.y >> 16; f[2] = c.x & 0xffffu;
        shape = c.x >> 16; child = c.y & 0xffffu;
      } else {
        const uint4 a = ld4<SMEM>(tp), b = ld4<SMEM>(tp + 16);
        thr[0] = __uint_as_float(a.x); thr[1] = __uint_as_float(a.y);
        thr[2] = __uint_as_float(a.z); thr[3] = __uint_as_float(a.w);
        f[0] = b.x & 0xffffu; f[1] = b.x >> 16; f[2] = b.y & 0xffffu; f[3] = b.y >> 16;
        shape = b.z & 0xffffu; child = b.z >> 16;
      }
      uint32_t bits = 0;
#pragma unroll
      for (int i = 0; i < TS; ++i) bits |= (uint32_t)(feature<CACHED, RT>(ra, f[i]) < thr[i]) << i;
      k = (uint32_t)lut[(shape << TS) + bits];
    }
    n = REP == 0 ? child + k : n * (TS + 1) + 1 + k;
  }
  *slot_out = n;
  const uint8_t *tp = gbase + (size_t)(n * kCols + col) * TB;
  return SMEM ? *reinterpret_cast<const float *>(tp) : __ldg(reinterpret_cast<const float *>(tp));
}

__device__ __forceinline__ float apply_transform(float v, int transform) {
  return transform == 1 ? 1.0f / (1.0f + expf(-v)) : v;
}

// argmax with the reference generated code's tie rule
// (src/reduction/LowerReduceOps.cpp:148-189): "if (max > v) keep else take".
template <typename Load> __device__ __forceinline__ int argmax_last(int C, Load load) {
  float best = __int_as_float(0xff800000);
  int arg = 0;
  for (int c = 0; c < C; ++c) {
    const float v = load(c);
    if (!(best > v)) { best = v; arg = c; }
  }
  return arg;
}

// --------------------------------------------------------------------------

template <int REP, int TS, int RPL, bool STAGED, bool CACHED>
__global__ void __launch_bounds__(1024, 1) tb_walk_kernel(const WalkParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int RW = p.row_warps, TT = p.tree_threads;
  const int rw = warp % RW, tt = warp / RW;
  const int F = p.num_features;
  const int W = p.num_classes > 0 ? p.num_classes : 1;
  constexpr int RT = 32 * RPL; // rows per warp tile

  // shared memory carve-up
  uint64_t *mbar = reinterpret_cast<uint64_t *>(smem_raw);                 // 2 barriers
  int8_t *lut_s = reinterpret_cast<int8_t *>(smem_raw + 16);               // look-up table
  size_t off = (16 + (size_t)p.lut_bytes + 127) & ~(size_t)127;
  unsigned char *stage0 = smem_raw + off;
  off += STAGED ? 2 * (size_t)p.stage_bytes : 0;
  float *xs_all = reinterpret_cast<float *>(smem_raw + off);
  const size_t xs_floats = CACHED ? (size_t)(F + 1) * RT : 0;
  off += (size_t)RW * xs_floats * 4;
  // per-warp class sums (multiclass) or cross-tree-thread partials
  float *acc_s = reinterpret_cast<float *>(smem_raw + off);

  const long long row_base = (long long)blockIdx.x * RW * RT + (long long)rw * RT;
  const int g0 = blockIdx.y * p.groups_per_chunk;
  const int g1 = min(p.num_groups, g0 + p.groups_per_chunk);

  if (STAGED && tid == 0) {
    mbar_init(&mbar[0], 1);
    mbar_init(&mbar[1], 1);
    fence_barrier_init();
  }
  for (int i = tid; i < p.lut_bytes; i += blockDim.x) lut_s[i] = p.lut[i];

  // ---- stage the row tile: 16-byte loads, transposed store xs[f][row]
  if (CACHED) {
    float *xs = xs_all + (size_t)rw * xs_floats;
#pragma unroll
    for (int q = 0; q < RPL; ++q) {
      const long long row = row_base + q * 32 + lane;
      const bool live = row < p.n_rows;
      const float *src = p.rows + (live ? row : 0) * p.ld;
      float *dst = xs + q * 32 + lane;
      if (p.vec4_ok) {
        for (int k = tt; k < F / 4; k += TT) {
          float4 v = live ? __ldg(reinterpret_cast<const float4 *>(src) + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          dst[(4 * k + 0) * RT] = v.x; dst[(4 * k + 1) * RT] = v.y;
          dst[(4 * k + 2) * RT] = v.z; dst[(4 * k + 3) * RT] = v.w;
        }
      } else {
        for (int k = tt; k < F; k += TT) dst[k * RT] = live ? __ldg(src + k) : 0.f;
      }
      if (tt == 0) dst[F * RT] = __int_as_float(0xff800000); // sentinel feature: -inf
    }
  }
  __syncthreads();

  if (STAGED && tid == 0) {
    for (int s = p.skip_first_copy ? 1 : 0; s < 2 && g0 + s < g1; ++s) {
      const DevGroupMeta gm = p.groups[g0 + s];
      const uint32_t bytes = (gm.slots * kCols * (REP == 2 ? 6u : (uint32_t)(TS == 1 ? 8 : TS == 2 ? 16 : TS == 3 ? 24 : 32)) + 15u) & ~15u;
      mbar_expect_tx(&mbar[s], bytes);
      bulk_g2s(stage0 + (size_t)s * p.stage_bytes, p.blob + gm.byte_off, bytes, &mbar[s]);
    }
  }

  RowAccess ra[RPL];
#pragma unroll
  for (int q = 0; q < RPL; ++q) {
    ra[q].xs = xs_all + (size_t)rw * xs_floats + q * 32 + lane;
    const long long row = row_base + q * 32 + lane;
    ra[q].grow = p.rows + (row < p.n_rows ? row : 0) * p.ld;
    ra[q].num_features = F;
  }

  float acc[RPL];
#pragma unroll
  for (int q = 0; q < RPL; ++q) acc[q] = 0.f;
  float *cacc = acc_s + (size_t)warp * W * RT; // multiclass: [class][row in tile]
  if (p.num_classes > 0 && !p.class_regs)
    for (int i = lane; i < W * RT; i += 32) cacc[i] = 0.f;
  __syncwarp();
  // Multiclass with class sums in registers: the packer lays a multiclass forest out class
  // by class (every group belongs to one class, classes in increasing order, every class
  // present), so one register per row holds the running sum of the current class and the
  // arg-max is updated whenever the class changes -- no shared-memory class table, which
  // leaves room for a full block of row warps.
  int cur_cls = -1;
  float best[RPL];
  int arg[RPL];
#pragma unroll
  for (int q = 0; q < RPL; ++q) {
    best[q] = __int_as_float(0xff800000);
    arg[q] = 0;
  }
  auto close_class = [&]() {
    if (cur_cls < 0) return;
#pragma unroll
    for (int q = 0; q < RPL; ++q) {
      const float v = p.initial_value + acc[q];
      if (!(best[q] > v)) { // the reference's tie rule: the later class wins
        best[q] = v;
        arg[q] = cur_cls;
      }
      acc[q] = 0.f;
    }
  };

  for (int g = g0; g < g1; ++g) {
    const DevGroupMeta gm = p.groups[g];
    if (p.class_regs) {
      const int cls = p.tree_class[g * kCols];
      if (cls != cur_cls) {
        close_class();
        cur_cls = cls;
      }
    }
    const uint8_t *gbase;
    if (STAGED) {
      const int s = (g - g0) & 1;
      const uint32_t parity = ((g - g0) >> 1) & 1;
      const bool ok = mbar_wait_bounded(&mbar[s], parity, p.wait_limit ? p.wait_limit : kWaitLimit);
      if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicExch(p.status, 4);
        return;
      }
      gbase = stage0 + (size_t)s * p.stage_bytes;
    } else {
      gbase = p.blob + gm.byte_off;
    }
    for (int s = tt; s < kCols; s += TT) {
      const uint32_t col = (lane + s) & (kCols - 1);
      const int k = g * kCols + (int)col;
      uint32_t slot[RPL];
      float v[RPL];
#pragma unroll
      for (int q = 0; q < RPL; ++q)
        v[q] = walk_one<REP, TS, STAGED, CACHED, RT>(gbase, gm.slots, gm.depth, col, ra[q], lut_s, &slot[q]);
      if (p.leaf_ids != nullptr) {
        const int t = p.tree_index[k];
        if (t >= 0) {
#pragma unroll
          for (int q = 0; q < RPL; ++q) {
            const long long row = row_base + q * 32 + lane;
            if (row < p.n_rows)
              p.leaf_ids[row * p.num_trees + t] = p.orig_node[p.orig_off[g] + (size_t)slot[q] * kCols + col];
          }
        }
      } else if (p.num_classes > 0 && !p.class_regs) {
        const int cls = p.tree_class[k];
#pragma unroll
        for (int q = 0; q < RPL; ++q) cacc[cls * RT + q * 32 + lane] += v[q];
      } else {
#pragma unroll
        for (int q = 0; q < RPL; ++q) acc[q] += v[q];
      }
    }
    if (STAGED) {
      __syncthreads(); // every warp is done with this stage
      if (tid == 0 && g + 2 < g1) {
        const int s = (g - g0) & 1;
        const DevGroupMeta nx = p.groups[g + 2];
        const uint32_t bytes = (nx.slots * kCols * (REP == 2 ? 6u : (uint32_t)(TS == 1 ? 8 : TS == 2 ? 16 : TS == 3 ? 24 : 32)) + 15u) & ~15u;
        mbar_expect_tx(&mbar[s], bytes);
        bulk_g2s(stage0 + (size_t)s * p.stage_bytes, p.blob + nx.byte_off, bytes, &mbar[s]);
      }
    }
  }
  if (p.leaf_ids != nullptr) return;

  // ---- combine the tree-thread warps that share a row tile (block-level pass)
  if (p.num_classes == 0) {
    if (TT > 1) {
      __syncthreads();
#pragma unroll
      for (int q = 0; q < RPL; ++q) acc_s[(size_t)warp * RT + q * 32 + lane] = acc[q];
      __syncthreads();
      if (tt == 0) {
        for (int o = 1; o < TT; ++o)
#pragma unroll
          for (int q = 0; q < RPL; ++q) acc[q] += acc_s[(size_t)(o * RW + rw) * RT + q * 32 + lane];
      }
    }
    if (tt != 0) return;
#pragma unroll
    for (int q = 0; q < RPL; ++q) {
      const long long row = row_base + q * 32 + lane;
      if (row >= p.n_rows) continue;
      if (p.write_partial)
        p.partial[(long long)blockIdx.y * p.n_rows + row] = acc[q];
      else
        reinterpret_cast<float *>(p.out)[row] = apply_transform(p.initial_value + acc[q], p.transform);
    }
  } else if (p.class_regs) {
    close_class();
#pragma unroll
    for (int q = 0; q < RPL; ++q) {
      const long long row = row_base + q * 32 + lane;
      if (row >= p.n_rows) continue;
      if (p.out_kind == 1) reinterpret_cast<int8_t *>(p.out)[row] = (int8_t)arg[q];
      else reinterpret_cast<float *>(p.out)[row] = (float)arg[q];
    }
  } else {
    __syncthreads();
    if (tt != 0) return;
    for (int o = 1; o < TT; ++o) {
      const float *other = acc_s + (size_t)(o * RW + rw) * W * RT;
      for (int i = lane; i < W * RT; i += 32) cacc[i] += other[i];
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < RPL; ++q) {
      const long long row = row_base + q * 32 + lane;
      if (row >= p.n_rows) continue;
      const float *mine = cacc + q * 32 + lane;
      if (p.write_partial) {
        float *dst = p.partial + ((long long)blockIdx.y * p.n_rows + row) * W;
        for (int c = 0; c < W; ++c) dst[c] = mine[c * RT];
      } else {
        const float init = p.initial_value;
        const int arg = argmax_last(W, [&](int c) { return init + mine[c * RT]; });
        if (p.out_kind == 1) reinterpret_cast<int8_t *>(p.out)[row] = (int8_t)arg;
        else reinterpret_cast<float *>(p.out)[row] = (float)arg;
      }
    }
  }
}

// Second pass: sums the partials of all tree chunks for a row (fixed order, no
// atomics), adds the initial value and applies the transformation / class argmax.
// Reference: the per-column serial sum plus initial value of
// src/reduction/LowerReduceOps.cpp:921-1003.
__global__ void tb_finalize_kernel(const float *__restrict__ partial, int chunks, long long n_rows, int W,
                                   int num_classes, float initial_value, int transform, void *out,
                                   int out_kind) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows) return;
  if (num_classes == 0) {
    float s = 0.f;
    for (int c = 0; c < chunks; ++c) s += partial[(long long)c * n_rows + row];
    reinterpret_cast<float *>(out)[row] = apply_transform(initial_value + s, transform);
  } else {
    const int arg = argmax_last(W, [&](int k) {
      float s = 0.f;
      for (int c = 0; c < chunks; ++c) s += partial[((long long)c * n_rows + row) * W + k];
      return initial_value + s;
    });
    if (out_kind == 1) reinterpret_cast<int8_t *>(out)[row] = (int8_t)arg;
    else reinterpret_cast<float *>(out)[row] = (float)arg;
  }
}

// Sums tree-chunk partials into one partial per row (tree-sharded use: the result is
// what crosses the NVLink reduction).
__global__ void tb_sum_partials_kernel(const float *__restrict__ partial, int chunks, long long total,
                                       float *__restrict__ dst) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += partial[(long long)c * total + i];
  dst[i] = s;
}

} // namespace tb
