// Walk kernel for the 16-bit-key layout (quant_pack.h): forests over rows too wide for
// an fp32 row tile.
//
// One block = 32 warps = one tile of 32 rows.  Lane = row; warp w walks, in every group
// of 32 trees, column (lane + w) mod 32, so the 32 lanes of a warp read 32 distinct
// columns of the node plane (one shared-memory wavefront) and the block covers every
// (row, tree) pair of the group exactly once.  The row tile is staged ONCE per block as
// 16-bit keys, transposed (keys[feature][row]); the node and leaf planes of every group
// stream through a three-slot ring of 32 KB stages filled by cp.async.bulk copies, each
// issued by a different warp so that two copies are always in flight.  Per-row sums live
// in registers and are combined across the 32 warps once, at the end.
//
// Reference counterparts: the walk of src/mlir/CodeGenStateMachine.cpp:149-243 over the
// reorg layout (src/gpu/ReorgForestRepresentation.cpp:495-571), the row cache
// (src/gpu/GPURepresentations.cpp:279-399) and the per-thread-column reduction
// (src/reduction/LowerReduceOps.cpp:921-1003).
#pragma once
#include "walk_kernels.cuh"

namespace tb {

struct DevQuantGroup {
  unsigned long long elem_off;
  uint32_t depth;
  uint32_t slots;
};

struct QuantParams {
  const uint32_t *node_plane;
  const float *leaf_plane;
  const float *exact_plane;
  const DevQuantGroup *groups;
  const int32_t *tree_index;
  const int32_t *orig_leaf;
  const float *lo;
  const float *scale;
  const float *rows;
  long long n_rows, ld;
  float *partial;
  void *out;
  int32_t write_partial;
  int32_t *leaf_ids;
  long long num_trees;
  int32_t num_groups, groups_per_chunk, num_features, transform;
  float initial_value;
  int32_t vec4_ok;
  int32_t *status;
  unsigned long long *tie_count; // optional statistics
};

constexpr int kQStage = 32768;
constexpr uint32_t kQWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t quant_key_dev(float v, float lo, float sc) {
  const float y = __fmaf_rn(__fsub_rn(v, lo), -sc, 65533.0f);
  unsigned short h;
  asm("cvt.rmi.u16.f32 %0, %1;" : "=h"(h) : "f"(y)); // floor, clamp to [0, 65535], NaN -> 0
  return h;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait_q(uint64_t *bar, uint32_t parity) {
  for (uint32_t it = 0; it < kQWaitLimit; ++it) {
    if (mbar_test(bar, parity)) return true;
    if (it > 32) __nanosleep(40);
  }
  return false;
}

// Fills the key field of every split node from its exact threshold (run once at upload,
// so that thresholds and row values are quantised by the very same device arithmetic).
__global__ void tb_quant_fill_keys(uint32_t *node_plane, const float *exact_plane, const float *lo,
                                   const float *scale, unsigned long long n, int num_features) {
  const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t node = node_plane[i], f = node >> 16;
  if (f < (uint32_t)num_features) node_plane[i] = (f << 16) | quant_key_dev(exact_plane[i], lo[f], scale[f]);
}

__global__ void __launch_bounds__(1024, 1) tb_walk_quant_kernel(const QuantParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int F = p.num_features;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);      // [3]
  uint64_t *empty = full + 3;                                   // [3]
  unsigned char *ring = smem_raw + 128;
  const uint32_t ring_s = smem_u32(ring);
  const uint32_t keys_s = ring_s + 3 * kQStage;                 // u16 [F+1][32]
  const uint32_t keys_lane = keys_s + lane * 2;

  const long long row = (long long)blockIdx.x * 32 + lane;
  const bool live = row < p.n_rows;
  const float *rowp = p.rows + (live ? row : 0) * p.ld;
  const int g0 = blockIdx.y * p.groups_per_chunk;
  const int g1 = min(p.num_groups, g0 + p.groups_per_chunk);
  const int P = 2 * (g1 - g0); // pieces: node plane, leaf plane of each group

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 32);
    }
    fence_barrier_init();
  }
  __syncthreads();

  auto issue = [&](int piece) {
    const DevQuantGroup gm = p.groups[g0 + (piece >> 1)];
    const uint32_t bytes = gm.slots * 128u;
    const void *src = (piece & 1) ? static_cast<const void *>(p.leaf_plane + gm.elem_off)
                                  : static_cast<const void *>(p.node_plane + gm.elem_off);
    uint64_t *bar = &full[piece % 3];
    mbar_expect_tx(bar, bytes);
    bulk_g2s(ring + (size_t)(piece % 3) * kQStage, src, bytes, bar);
  };
  if (lane == 0 && warp < 3 && warp < P) issue(warp);

  // ---- stage the row tile as keys: keys[f][row]
  if (p.vec4_ok) {
    for (int k = warp; k < F / 4; k += 32) {
      const float4 v = live ? __ldg(reinterpret_cast<const float4 *>(rowp) + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 lo = __ldg(reinterpret_cast<const float4 *>(p.lo) + k);
      const float4 sc = __ldg(reinterpret_cast<const float4 *>(p.scale) + k);
      const uint32_t a = keys_lane + (uint32_t)k * 256u;
      sts_u16(a, quant_key_dev(v.x, lo.x, sc.x));
      sts_u16(a + 64, quant_key_dev(v.y, lo.y, sc.y));
      sts_u16(a + 128, quant_key_dev(v.z, lo.z, sc.z));
      sts_u16(a + 192, quant_key_dev(v.w, lo.w, sc.w));
    }
  } else {
    for (int k = warp; k < F; k += 32)
      sts_u16(keys_lane + (uint32_t)k * 64u, quant_key_dev(live ? __ldg(rowp + k) : 0.f, __ldg(p.lo + k), __ldg(p.scale + k)));
  }
  if (warp == 0) sts_u16(keys_lane + (uint32_t)F * 64u, 65535u); // sentinel feature
  __syncthreads();

  const uint32_t col = (uint32_t)(lane + warp) & 31u;
  float acc = 0.f;
  bool ok = true;
  unsigned ties = 0;

  // after a piece is consumed: release its stage and, if it is this warp's turn, refill it
  auto release = [&](int piece) {
    __syncwarp();
    if (lane == 0) {
      uint64_t *e = &empty[piece % 3];
      mbar_arrive(e);
      const int next = piece + 3;
      if (next < P && (next & 31) == warp) {
        if (mbar_wait_q(e, (uint32_t)(piece / 3) & 1u)) issue(next);
        else ok = false;
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
  };

  for (int gi = 0; gi < g1 - g0 && ok; ++gi) {
    const DevQuantGroup gm = p.groups[g0 + gi];
    int piece = 2 * gi;
    if (!mbar_wait_q(&full[piece % 3], (uint32_t)(piece / 3) & 1u)) { ok = false; break; }
    const uint32_t colbase = ring_s + (uint32_t)(piece % 3) * kQStage + col * 4u;
    const uint32_t cL = 128u - colbase, cR = 256u - colbase;
    uint32_t A = colbase;
#pragma unroll 2
    for (uint32_t d = 0; d < gm.depth; ++d) {
      const uint32_t node = lds_u32(A);
      const uint32_t f = node >> 16, kt = node & 0xffffu;
      const uint32_t kx = lds_u16(keys_lane + f * 64u);
      bool right = kx < kt;
      if (kx == kt) {
        // keys tie: decide on the exact fp32 values
        const uint32_t slot = (A - colbase) >> 7;
        const float thr = __ldg(p.exact_plane + gm.elem_off + (unsigned long long)slot * 32u + col);
        right = !(__ldg(rowp + f) < thr);
        ++ties;
      }
      A = 2u * A + (right ? cR : cL);
    }
    const uint32_t leaf = ((A - colbase) >> 7) - (gm.slots - 1u);
    release(piece);
    if (!ok) break;
    ++piece;
    if (!mbar_wait_q(&full[piece % 3], (uint32_t)(piece / 3) & 1u)) { ok = false; break; }
    acc += lds_f32(ring_s + (uint32_t)(piece % 3) * kQStage + leaf * 128u + col * 4u);
    if (p.leaf_ids != nullptr && live) {
      const int t = p.tree_index[(g0 + gi) * 32 + (int)col];
      if (t >= 0) p.leaf_ids[row * p.num_trees + t] = p.orig_leaf[gm.elem_off + (unsigned long long)leaf * 32u + col];
    }
    release(piece);
  }
  if (__syncthreads_or(!ok)) {
    if (tid == 0) atomicExch(p.status, 4);
    return;
  }
  if (p.tie_count != nullptr && ties) atomicAdd(p.tie_count, (unsigned long long)ties);
  if (p.leaf_ids != nullptr) return;

  // ---- combine the 32 warps (one partial per row each)
  float *red = reinterpret_cast<float *>(ring);
  red[warp * 32 + lane] = acc;
  __syncthreads();
  if (warp != 0 || !live) return;
  float s = 0.f;
#pragma unroll 8
  for (int w = 0; w < 32; ++w) s += red[w * 32 + lane];
  if (p.write_partial)
    p.partial[(long long)blockIdx.y * p.n_rows + row] = s;
  else
    reinterpret_cast<float *>(p.out)[row] = apply_transform(p.initial_value + s, p.transform);
}

} // namespace tb
