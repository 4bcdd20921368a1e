// Walk kernel for the 16-bit-key layout (quant_pack.h): forests over rows too wide for
// an fp32 row tile.
//
// One block = 32 warps = one tile of 32 rows, staged ONCE per block as 16-bit keys,
// transposed (keys[feature][row]).  Lane = row.  The block works as TWO independent halves
// of 16 warps: half h takes the groups h, h+2, ... of the chunk for all 32 rows; warp w of
// a half walks, in every group of 32 trees, the columns (lane + w) mod 32 and
// (lane + w + 16) mod 32 in lock-step, so the 32 lanes of a warp read 32 distinct columns
// of the node plane (one shared-memory wavefront per load) and the half covers every
// (row, tree) pair of the group exactly once.  While one half waits for a piece or sits in
// its barrier, the other keeps the issue slots and the shared-memory pipe busy; the forest
// is still streamed only once per 32-row tile.
//
// Only the NODE planes stream through shared memory: two 16 KB pieces per group (upper
// levels, bottom level) through a three-slot ring per half, filled by cp.async.bulk copies
// that rotating warps issue; one named barrier per group frees the group's two slots.  The
// leaf values are read straight from L2 (staging the leaf plane would move as many bytes
// and take ring slots) and consumed one group later; the walkers first exchange their leaf
// numbers through a small shared-memory table, so that a warp loads ONE tree's leaves for
// all 32 rows (see fetch_leaves).  Per-row sums live in registers and are combined across
// the 32 warps once, at the end.
//
// The walk is fully unrolled per depth: one key load, one compare, one node load per level.
// Key ties are only flagged on the fast path; a flagged (row, tree)
// pair is then re-walked on the exact fp32 values from global memory.  Every lane polls
// the stage barrier itself (mbarrier.try_wait, bounded).
//
// Reference counterparts: the walk of src/mlir/CodeGenStateMachine.cpp:149-243 over the
// reorg layout (src/gpu/ReorgForestRepresentation.cpp:495-571), the unrolled walk of
// padded trees (src/mlir/WalkDecisionTreeLoweringPass.cpp:24-53), the row cache
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
  int32_t meta_bytes;            // shared-memory bytes reserved for the group table
  int32_t *status;
  unsigned long long *tie_count; // optional statistics
};

constexpr int kQRingBytes = 6 * 16384; // two half-blocks x three 16 KB pieces
constexpr int kQMaxGroupsPerChunk = 160;
constexpr int kQLeafTableBytes = 4096; // [2 halves][2 buffers][32 columns][32 rows] leaf numbers
constexpr uint32_t kQWaitTries = 1u << 20;

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
  uint32_t v; // a 16-bit load into a 32-bit register zero-extends: no conversion afterwards
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v));
}
// Bounded wait executed by every lane of the calling warp (no election, no shuffle).
__device__ __forceinline__ bool mbar_wait_all_lanes(uint32_t bar_addr, uint32_t parity) {
  for (uint32_t it = 0; it < kQWaitTries; ++it) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
                 " selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(bar_addr), "r"(parity), "r"(200u)
                 : "memory");
    if (ok) return true;
  }
  return false;
}

// Fast walk of DEPTH levels of one column of a staged node plane.  Returns the byte
// address of the slot reached (colbase + 128 * slot); *tie is set when any key
// comparison on the path tied (the result is then not to be trusted).
template <int DEPTH>
__device__ __forceinline__ uint32_t quant_walk(uint32_t colbase, uint32_t keys_lane, bool *tie) {
  uint32_t A = colbase;
  bool t = false;
  if (DEPTH > 0) {
    uint32_t node = lds_u32(A);
    const uint32_t cL = 128u - colbase;
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      // one key load and one node load per level: the kernel is bound by the SM's load/store
      // path, so fetching both children ahead of the comparison costs more than it hides
      const uint32_t kx = lds_u16(keys_lane + (node >> 16) * 64u);
      const uint32_t kt = node & 0xffffu;
      t |= (kx == kt);
      A = 2u * A + cL + (kx < kt ? 128u : 0u);
      if (d + 1 < DEPTH) node = lds_u32(A);
    }
  }
  *tie = t;
  return A;
}

__device__ __forceinline__ uint32_t quant_walk_any(uint32_t depth, uint32_t colbase, uint32_t keys_lane, bool *tie) {
  switch (depth) {
  case 0: return quant_walk<0>(colbase, keys_lane, tie);
  case 1: return quant_walk<1>(colbase, keys_lane, tie);
  case 2: return quant_walk<2>(colbase, keys_lane, tie);
  case 3: return quant_walk<3>(colbase, keys_lane, tie);
  case 4: return quant_walk<4>(colbase, keys_lane, tie);
  case 5: return quant_walk<5>(colbase, keys_lane, tie);
  case 6: return quant_walk<6>(colbase, keys_lane, tie);
  case 7: return quant_walk<7>(colbase, keys_lane, tie);
  default: return quant_walk<8>(colbase, keys_lane, tie);
  }
}

// Re-walk of one (row, tree) pair behind a key tie: the staged keys decide wherever they
// can, and only the tied comparisons read the exact fp32 values from global memory.
// Returns the slot reached (level-order numbering of the planes).
__device__ __noinline__ uint32_t quant_walk_exact(uint32_t colbase, uint32_t keys_lane, const float *exact_plane,
                                                  size_t plane_row, uint32_t depth, uint32_t col,
                                                  const float *rowp) {
  uint32_t s = 0;
  for (uint32_t d = 0; d < depth; ++d) {
    const uint32_t node = lds_u32(colbase + s * 128u);
    const uint32_t f = node >> 16, kt = node & 0xffffu;
    const uint32_t kx = lds_u16(keys_lane + f * 64u);
    bool right = kx < kt;
    if (kx == kt) right = !(__ldg(rowp + f) < __ldg(exact_plane + (plane_row + s) * 32u + col));
    s = 2u * s + 1u + (right ? 1u : 0u);
  }
  return s;
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

constexpr int kQPiece = 16384;  // one ring slot: half a plane of a group of 8 levels
constexpr int kQHalfWarps = 16; // warps per half-block

// Barrier over the 512 threads of one half-block that also ORs a predicate across them.
__device__ __forceinline__ bool half_barrier_or(int id, bool pred) {
  uint32_t r;
  asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.or.pred p, %2, 512, q;\n"
               " selp.u32 %0, 1, 0, p;\n}"
               : "=r"(r)
               : "r"((uint32_t)pred), "r"(id)
               : "memory");
  return r != 0;
}

// UD: depth shared by every group of the forest (0 = mixed depths, decided per group at run
// time; with a constant depth the walk is called directly and piece sizes fold).
// LEAF_IDS: the launch records leaf ids instead of predictions.
template <int UD, bool LEAF_IDS>
__global__ void __launch_bounds__(1024, 1) tb_walk_quant_kernel(const QuantParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = warp / kQHalfWarps, hw = warp % kQHalfWarps;
  const int F = p.num_features;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw) + half * 3; // [2 halves][3 slots]
  // group table of this chunk: {plane offset in 32-element rows, depth}
  uint2 *gtab = reinterpret_cast<uint2 *>(smem_raw + 128);
  unsigned char *ring = smem_raw + 128 + p.meta_bytes + (size_t)half * 3 * kQPiece;
  const uint32_t ring_s = smem_u32(ring);
  // leaf numbers of a group, exchanged between the warps of a half (see below)
  const uint32_t ltab_s = smem_u32(smem_raw + 128 + p.meta_bytes) + 6 * kQPiece + (uint32_t)half * 2048u;
  const uint32_t keys_s = smem_u32(smem_raw + 128 + p.meta_bytes) + 6 * kQPiece + kQLeafTableBytes; // u16 [F+1][32]
  const uint32_t keys_lane = keys_s + lane * 2;

  const long long row = (long long)blockIdx.x * 32 + lane;
  const bool live = row < p.n_rows;
  const float *rowp = p.rows + (live ? row : 0) * p.ld;
  const int g0 = blockIdx.y * p.groups_per_chunk;
  const int g1 = min(p.num_groups, g0 + p.groups_per_chunk);
  const int NG = g1 - g0;
  const int NGh = (NG - half + 1) / 2; // groups half, half + 2, ... of the chunk
  const int P = 2 * NGh;               // pieces of this half: upper levels and bottom level of the node planes

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) mbar_init(reinterpret_cast<uint64_t *>(smem_raw) + i, 1);
    fence_barrier_init();
  }
  for (int i = tid; i < NG; i += blockDim.x) {
    const DevQuantGroup gm = p.groups[g0 + i];
    gtab[i] = make_uint2((uint32_t)(gm.elem_off >> 5), gm.depth);
  }
  __syncthreads();

  auto issue = [&](int piece, int slot) { // slot = piece % 3
    const uint2 gm = gtab[2 * (piece >> 1) + half];
    const uint32_t hs = UD ? (1u << (UD ? UD - 1 : 0)) : 1u << (gm.y - 1); // slots per piece
    const size_t off = ((size_t)gm.x + ((piece & 1) ? hs : 0u)) * 32;
    uint64_t *bar = &full[slot];
    mbar_expect_tx(bar, hs * 128u);
    bulk_g2s(ring + (size_t)slot * kQPiece, p.node_plane + off, hs * 128u, bar);
  };
  if (lane == 0 && hw < 3 && hw < P) issue(hw, hw);

  // ---- stage the row tile as keys: keys[f][row]
  {
    // A warp takes a block of 32 consecutive features: every load instruction reads 128
    // contiguous bytes of ONE row (lane = feature), so DRAM sees whole lines and adjacent
    // warps continue the same rows.  A lane thus collects its feature for all 32 rows,
    // packs the 32 keys into 64 bytes and writes them with four 16-byte stores.  Loads
    // go to L2 only (the unified L1 is almost entirely shared memory here); sixteen are
    // in flight per thread.
    const long long row0 = (long long)blockIdx.x * 32;
    const int live_rows = (int)min((long long)32, p.n_rows - row0);
    const float *tile = p.rows + row0 * p.ld;
    for (int f0 = warp * 32; f0 < F; f0 += 32 * 32) {
      const int f = f0 + lane;
      const bool fok = f < F;
      const float lo = fok ? __ldg(p.lo + f) : 0.f, sc = fok ? __ldg(p.scale + f) : 0.f;
      uint32_t packed[16];
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        float x[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const int rr = part * 16 + r;
          x[r] = (fok && rr < live_rows) ? __ldcg(tile + (long long)rr * p.ld + f) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 16; r += 2)
          packed[part * 8 + r / 2] = quant_key_dev(x[r], lo, sc) | (quant_key_dev(x[r + 1], lo, sc) << 16);
      }
      if (fok) {
        const uint32_t dst = keys_s + (uint32_t)f * 64u;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 16u * c), "r"(packed[4 * c]),
                       "r"(packed[4 * c + 1]), "r"(packed[4 * c + 2]), "r"(packed[4 * c + 3]));
      }
    }
  }
  if (warp == 0) sts_u16(keys_lane + (uint32_t)F * 64u, 65535u); // sentinel feature
  __syncthreads();

  // the two columns this lane walks in every group of its half
  const uint32_t col[2] = {(uint32_t)(lane + hw) & 31u, (uint32_t)(lane + hw + 16) & 31u};
  float acc = 0.f;
  float pend[2] = {0.f, 0.f}; // leaf values of the previous group, on their way from L2
  bool ok = true, failed = false;
  unsigned ties = 0;

  // One barrier per group over the half-block (it also carries any wait failure to its 512
  // threads, so that their exit is uniform) frees the group's two slots; the refills are
  // issued by two rotating warps.
  // Two pieces per group through three slots: the slots of a group's pieces rotate with period
  // three -- (0,1), (2,0), (1,2) -- and so do the phases of their barriers -- (0,0), (0,1),
  // (1,1) -- whatever the group number; both follow from two counters, without divisions.
  int su = 0, sb = 1; // ring slots of the current group's upper-level and bottom-level pieces
  auto release = [&](int first) {
    failed = half_barrier_or(1 + half, !ok);
    if (!failed && lane == 0) {
      // pieces first+3 and first+4 land in the two slots just freed, in the same order
      if (first + 3 < P && ((first + 3) % kQHalfWarps) == hw) issue(first + 3, su);
      if (first + 4 < P && ((first + 4) % kQHalfWarps) == hw) issue(first + 4, sb);
    }
    su = su == 0 ? 2 : su - 1;
    sb = sb == 0 ? 2 : sb - 1;
  };
  const uint32_t full_s = smem_u32(full);
  auto upper_ready = [&]() { return mbar_wait_all_lanes(full_s + 8u * (uint32_t)su, su == 1 ? 1u : 0u); };
  auto bottom_ready = [&]() { return mbar_wait_all_lanes(full_s + 8u * (uint32_t)sb, sb != 1 ? 1u : 0u); };

  // Leaf values come straight from L2, but not in the walk's lane assignment: there the 32
  // lanes of a warp sit in 32 different trees, i.e. 32 different lines of the leaf plane
  // whatever its layout.  The walkers therefore drop their leaf NUMBERS (one byte each) into
  // a [column][row] table in shared memory; after the group's barrier warp w of the half
  // picks up columns 2w and 2w+1 for all 32 rows and loads those leaves from the
  // column-major leaf plane, where one tree's 256 leaves span 1 KB: at most 8 lines per
  // warp load instead of 32.  Lane = row on both sides, so the sum stays in the lane's
  // register; the loads are consumed one group later.
  // (element offsets fit 32 bits: the host refuses planes of 2^32 elements or more)
  const uint32_t my_cols_s = ltab_s + (2u * (uint32_t)hw) * 32u + (uint32_t)lane;
  auto fetch_leaves = [&](int gi_prev, uint2 gprev, uint32_t buf) {
    const uint32_t slots = UD ? (1u << UD) : 2u << (gprev.y - 1);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const uint32_t c = 2u * (uint32_t)hw + (uint32_t)w;
      uint32_t leaf;
      asm volatile("ld.shared.u8 %0, [%1];" : "=r"(leaf) : "r"(my_cols_s + buf * 1024u + (uint32_t)w * 32u));
      const uint32_t e = gprev.x * 32u + c * slots + leaf;
      if (LEAF_IDS) {
        if (live) {
          const int t = p.tree_index[(g0 + gi_prev) * 32 + (int)c];
          if (t >= 0) p.leaf_ids[row * p.num_trees + t] = p.orig_leaf[e];
        }
      } else {
        pend[w] = __ldg(p.leaf_plane + e);
      }
    }
  };
  uint2 gprev = make_uint2(0, 0);
  int gi_prev = -1;
  // where this lane drops the leaf numbers of its two walks (buffer 0)
  const uint32_t drop_s[2] = {ltab_s + col[0] * 32u + (uint32_t)lane, ltab_s + col[1] * 32u + (uint32_t)lane};

  for (int k = 0; k < NGh; ++k) {
    const int gi = 2 * k + half;
    const uint2 gm = gtab[gi];
    const uint32_t depth = UD ? (uint32_t)UD : gm.y, hs = 1u << (depth - 1);
    const int q = 2 * k;
    uint32_t idx[2] = {0, 0};

    // leaves of the previous group (its table is complete: the barrier has been passed)
    if (gi_prev >= 0) fetch_leaves(gi_prev, gprev, (uint32_t)(k - 1) & 1u);

    // upper levels 0 .. depth-2
    ok = upper_ready();
    if (ok) {
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const uint32_t colbase = ring_s + (uint32_t)su * kQPiece + col[w] * 4u;
        bool tie;
        uint32_t s;
        if constexpr (UD > 0)
          s = (quant_walk<UD - 1>(colbase, keys_lane, &tie) - colbase) >> 7;
        else
          s = (quant_walk_any(depth - 1, colbase, keys_lane, &tie) - colbase) >> 7;
        if (tie) {
          s = quant_walk_exact(colbase, keys_lane, p.exact_plane, gm.x, depth - 1, col[w], rowp);
          ++ties;
        }
        idx[w] = s - (hs - 1u); // position inside the bottom decision level
      }
    }

    // bottom decision level; the leaf number goes into the table
    if (ok) ok = bottom_ready();
    if (ok) {
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const uint32_t node = lds_u32(ring_s + (uint32_t)sb * kQPiece + idx[w] * 128u + col[w] * 4u);
        const uint32_t f = node >> 16, kt = node & 0xffffu;
        const uint32_t kx = lds_u16(keys_lane + f * 64u);
        bool right = kx < kt;
        if (kx == kt) {
          right = !(__ldg(rowp + f) < __ldg(p.exact_plane + ((size_t)gm.x + hs + idx[w]) * 32u + col[w]));
          ++ties;
        }
        const uint32_t leaf = 2u * idx[w] + (right ? 1u : 0u);
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(drop_s[w] + ((uint32_t)k & 1u) * 1024u), "r"(leaf));
      }
      acc += pend[0] + pend[1]; // previous group's leaves have had a whole walk to arrive
      pend[0] = pend[1] = 0.f;
    }
    release(q);
    if (failed) break;
    gprev = gm;
    gi_prev = gi;
  }
  if (!failed && gi_prev >= 0) {
    fetch_leaves(gi_prev, gprev, (uint32_t)(NGh - 1) & 1u);
    acc += pend[0] + pend[1];
  }
  if (__syncthreads_or(failed)) {
    if (tid == 0) atomicExch(p.status, 4);
    return;
  }
  if (p.tie_count != nullptr && ties) atomicAdd(p.tie_count, (unsigned long long)ties);
  if (LEAF_IDS) return;

  // ---- combine the 32 warps (one partial per row each)
  float *red = reinterpret_cast<float *>(smem_raw + 128 + p.meta_bytes);
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
