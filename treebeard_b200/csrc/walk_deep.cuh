// Walk kernel for the one-tree-per-stage layout (deep_pack.h): forests of deep trees.
//
// One block = RW warps = one tile of 32*RW rows, staged ONCE as 15-bit keys and kept for
// the whole forest.  Lane = row: every thread walks its own row through BOTH trees of a
// pair in lock-step (two independent dependence chains per thread), so all threads of the
// block read the same two node planes.  The node planes stream through a ring of whole-tree
// pieces (16 KB each at 12 levels) filled by cp.async.bulk copies that one extra PRODUCER warp
// issues, the next pair's always in flight while a pair is walked; a row warp frees a slot
// with one arrival on the slot's "empty" mbarrier and the producer refills it when all row
// warps have arrived, so the row warps never meet at a block barrier and may drift apart by a
// pair.  Leaf values are read straight from L2 (32 scattered
// sectors per warp whatever the layout) and consumed one pair later.  Sums stay in the
// owning thread's register: there is no cross-thread reduction.
//
// Keys of two row warps are interleaved (feature-major, 128 bytes per warp pair: word j =
// row j of the even warp | row j of the odd warp << 16), so a warp's key load touches 32
// distinct banks.  A key tie is only flagged on the fast path; the flagged (row, tree) is
// re-walked with exact fp32 comparisons at the tied steps.
//
// Reference counterparts: src/mlir/CodeGenStateMachine.cpp:149-243 (scalar walk),
// src/mlir/WalkDecisionTreeLoweringPass.cpp:24-53 (fixed-depth walk of padded trees),
// src/gpu/GPURepresentations.cpp:279-399 (row cache) and :630-715 (tree cache).
#pragma once
#include "walk_quant.cuh"

namespace tb {

struct DeepParams {
  const uint32_t *node_plane;
  const float *leaf_plane;
  const float *exact_plane;
  const DevQuantGroup *pairs;
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
  int32_t num_pairs, pairs_per_chunk, num_features, transform;
  float initial_value;
  int32_t ring_slots;  // 4 .. 8
  uint32_t slot_bytes; // 4 << max depth of the forest
  uint32_t key_stride; // bytes per feature in the key tile: 64 * (row warps rounded up to even)
  int32_t *status;
  unsigned long long *tie_count;
  int32_t skip_first_copy; // failure drill: the first piece's copy is never issued, so its wait expires
  uint32_t wait_tries;     // polls before a wait gives up (0 = kQWaitTries)
};

constexpr int kDeepMaxSlots = 8;

// Fast walk of DEPTH levels of two trees in lock-step, in PTX (the step of walk_quant.cuh: keys
// are 15-bit integers that compare as fp16 numbers, so one half2 comparison of (key, node word)
// picks the child and a second one accumulates the tie flag; the node's address itself is
// tracked: the children of the node at address A = base + 4 i sit at 2A - base and 2A - base + 4).
// base0 / base1: shared-memory addresses of the node planes; returns the heap indices reached
// (in [2^DEPTH, 2^(DEPTH+1))) and whether any key comparison on either path tied.
//   %0, %1  node addresses (updated)   %2, %3  node words (scratch)   %4  tie flags (out)
//   %5  the thread's base in the key tile   %6  key-tile bytes per feature   %7, %8  -base
#define TBD_DECL ".reg .b32 ka0, ka1, kx0, kx1;\n .reg .pred p0, p1, t0, t1, q;\n"
#define TBD_LOAD "ld.shared.u32 %2, [%0];\n ld.shared.u32 %3, [%1];\n"
#define TBD_KEY(i, n) "shr.u32 ka" #i ", " n ", 16;\n mad.lo.u32 ka" #i ", ka" #i ", %6, %5;\n ld.shared.u16 kx" #i ", [ka" #i "];\n"
#define TBD_CMP0(i, n) "setp.lt.f16x2 p" #i "|q, kx" #i ", " n ";\n setp.eq.f16x2 t" #i "|q, kx" #i ", " n ";\n"
#define TBD_CMP(i, n) "setp.lt.f16x2 p" #i "|q, kx" #i ", " n ";\n setp.eq.or.f16x2 t" #i "|q, kx" #i ", " n ", t" #i ";\n"
#define TBD_ADV(i, a, c) "shl.b32 " a ", " a ", 1;\n add.u32 " a ", " a ", " c ";\n @p" #i " add.u32 " a ", " a ", 4;\n"
#define TBD_KEYS TBD_KEY(0, "%2") TBD_KEY(1, "%3")
#define TBD_ADVS TBD_ADV(0, "%0", "%7") TBD_ADV(1, "%1", "%8")
#define TBD_FIRST TBD_KEYS TBD_CMP0(0, "%2") TBD_CMP0(1, "%3") TBD_ADVS
#define TBD_NEXT TBD_LOAD TBD_KEYS TBD_CMP(0, "%2") TBD_CMP(1, "%3") TBD_ADVS
#define TBD_TIES "selp.u32 %4, 1, 0, t0;\n @t1 or.b32 %4, %4, 2;\n"
#define TBD_N2 TBD_NEXT TBD_NEXT
#define TBD_N4 TBD_N2 TBD_N2
#define TBD_N8 TBD_N4 TBD_N4
template <int DEPTH>
__device__ __forceinline__ void deep_walk(uint32_t base0, uint32_t base1, uint32_t key_lane, uint32_t ks,
                                          uint32_t *i0_out, uint32_t *i1_out, bool *tie0, bool *tie1) {
  static_assert(DEPTH >= 2 && DEPTH <= 12, "two to twelve levels");
  uint32_t a0 = base0 + 4u, a1 = base1 + 4u, tb; // the root is heap node 1
  [[maybe_unused]] uint32_t n0, n1;
#define TBD_OPERANDS : "+r"(a0), "+r"(a1), "=&r"(n0), "=&r"(n1), "=&r"(tb) : "r"(key_lane), "r"(ks), "r"(0u - base0), "r"(0u - base1)
  // DEPTH levels = the first one and DEPTH - 1 more, each of which loads its node first
  if constexpr (DEPTH == 2) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 3) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N2 TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 4) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N2 TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 5) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N4 TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 6) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N4 TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 7) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N4 TBD_N2 TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 8) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N4 TBD_N2 TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 9) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N8 TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 10) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N8 TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
  else if constexpr (DEPTH == 11) asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N8 TBD_N2 TBD_TIES "}" TBD_OPERANDS);
  else asm volatile("{\n" TBD_DECL TBD_LOAD TBD_FIRST TBD_N8 TBD_N2 TBD_NEXT TBD_TIES "}" TBD_OPERANDS);
#undef TBD_OPERANDS
  *i0_out = (a0 - base0) >> 2;
  *i1_out = (a1 - base1) >> 2;
  *tie0 = tb & 1u;
  *tie1 = tb & 2u;
}

__device__ __forceinline__ void deep_walk_any(uint32_t depth, uint32_t base0, uint32_t base1, uint32_t key_lane,
                                              uint32_t ks, uint32_t *i0, uint32_t *i1, bool *t0, bool *t1) {
  switch (depth) {
  case 2: return deep_walk<2>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 3: return deep_walk<3>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 4: return deep_walk<4>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 5: return deep_walk<5>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 6: return deep_walk<6>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 7: return deep_walk<7>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 8: return deep_walk<8>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 9: return deep_walk<9>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 10: return deep_walk<10>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  case 11: return deep_walk<11>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  default: return deep_walk<12>(base0, base1, key_lane, ks, i0, i1, t0, t1);
  }
}

// Re-walk of one (row, tree) behind a key tie: the staged keys decide wherever they can,
// the tied comparisons read the exact fp32 values from global memory.
__device__ __noinline__ uint32_t deep_walk_exact(uint32_t base, uint32_t key_lane, uint32_t ks, uint32_t depth,
                                                 const float *exact_tree, const float *rowp) {
  uint32_t i = 1;
  for (uint32_t d = 0; d < depth; ++d) {
    const uint32_t node = lds_u32(base + i * 4u);
    const uint32_t f = node >> 16, kt = node & 0xffffu;
    const uint32_t kx = lds_u16(key_lane + f * ks);
    bool right = kx < kt;
    if (kx == kt) right = !(__ldg(rowp + f) < __ldg(exact_tree + i));
    i = 2u * i + (right ? 1u : 0u);
  }
  return i;
}

// UD: depth shared by every pair of the forest (0 = mixed, decided per pair at run time).
// LEAF_IDS: the launch records leaf ids instead of predictions.
template <int MAX_THREADS, int UD, bool LEAF_IDS>
__global__ void __launch_bounds__(MAX_THREADS, 1) tb_walk_deep_kernel(const DeepParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int RW = (blockDim.x >> 5) - 1; // row warps; the last warp is the ring producer
  const int F = p.num_features;
  const int S = p.ring_slots;
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw); // [S], then empty[S]
  unsigned char *ring = smem_raw + 128;
  const uint32_t ring_s = smem_u32(ring);
  const uint32_t keys_s = ring_s + (uint32_t)S * p.slot_bytes;
  const uint32_t ks = p.key_stride;
  const uint32_t key_lane = keys_s + (uint32_t)(warp >> 1) * 128u + (uint32_t)lane * 4u + (uint32_t)(warp & 1) * 2u;

  const long long row = ((long long)blockIdx.x * RW + warp) * 32 + lane;
  const bool live = row < p.n_rows;
  const float *rowp = p.rows + (live ? row : 0) * p.ld;
  const int g0 = blockIdx.y * p.pairs_per_chunk;
  const int g1 = min(p.num_pairs, g0 + p.pairs_per_chunk);
  const int P = 2 * (g1 - g0); // pieces of this block: the node planes of every tree

  if (tid == 0) {
    for (int i = 0; i < S; ++i) mbar_init(&full[i], 1);
    for (int i = 0; i < S; ++i) mbar_init(&full[S + i], RW); // empty: one arrival per row warp
    fence_barrier_init();
  }
  __syncthreads();
  const uint32_t full_s = smem_u32(full), empty_s = full_s + 8u * (uint32_t)S;
  const uint32_t tries = p.wait_tries ? p.wait_tries : kQWaitTries;

  // piece 2k + j of the block: node plane of tree j of pair k.  Pieces are consumed in order,
  // so slots and barrier phases advance by counters (S and RW are run-time values: no
  // division on the hot path).
  auto issue = [&](int piece, int slot) {
    const DevQuantGroup gm = p.pairs[g0 + (piece >> 1)];
    const size_t off = (size_t)gm.elem_off + ((piece & 1) ? gm.slots : 0u);
    uint64_t *bar = &full[slot];
    mbar_expect_tx(bar, gm.slots * 4u);
    bulk_g2s(ring + (size_t)slot * p.slot_bytes, p.node_plane + off, gm.slots * 4u, bar);
  };
  if (warp == RW) {
    // ---- the producer: piece q goes to slot q mod S, once every row warp has released
    // the piece that was there
    bool ok = true;
    int slot = 0;
    uint32_t round = 0;
    for (int piece = 0; piece < P && ok; ++piece) {
      if (round > 0) ok = mbar_wait_all_lanes(empty_s + 8u * (uint32_t)slot, (round - 1u) & 1u, tries);
      if (ok && lane == 0 && !(p.skip_first_copy && piece == 0)) issue(piece, slot);
      if (++slot == S) {
        slot = 0;
        ++round;
      }
    }
    if (__syncthreads_or(!ok) && lane == 0) atomicExch(p.status, 4);
    return;
  }

  // ---- stage this thread's row as keys
  {
    const bool vec = (F % 4 == 0) && (p.ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.rows) & 15) == 0);
    if (vec) {
      for (int f = 0; f < F; f += 4) {
        const float4 x = live ? __ldg(reinterpret_cast<const float4 *>(rowp + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 lo = __ldg(reinterpret_cast<const float4 *>(p.lo + f));
        const float4 sc = __ldg(reinterpret_cast<const float4 *>(p.scale + f));
        sts_u16(key_lane + (uint32_t)f * ks, quant_key15_lattice_dev(x.x, lo.x, sc.x));
        sts_u16(key_lane + (uint32_t)(f + 1) * ks, quant_key15_lattice_dev(x.y, lo.y, sc.y));
        sts_u16(key_lane + (uint32_t)(f + 2) * ks, quant_key15_lattice_dev(x.z, lo.z, sc.z));
        sts_u16(key_lane + (uint32_t)(f + 3) * ks, quant_key15_lattice_dev(x.w, lo.w, sc.w));
      }
    } else {
      for (int f = 0; f < F; ++f)
        sts_u16(key_lane + (uint32_t)f * ks, quant_key15_lattice_dev(live ? __ldg(rowp + f) : 0.f, __ldg(p.lo + f), __ldg(p.scale + f)));
    }
    sts_u16(key_lane + (uint32_t)F * ks, 0x7bffu); // sentinel feature: the largest key
  }
  // (each thread reads back only the keys it wrote: no barrier is needed for the tile)

  // thousands of leaf values per row: a double accumulator keeps the sum within the
  // fp32 rounding of the exact result (one conversion and one add per tree)
  double acc = 0.0;
  float pend0 = 0.f, pend1 = 0.f; // leaf values of the previous pair, on their way from L2
  bool ok = true;
  unsigned ties = 0;
  int slot = 0;          // ring slot of the next piece to consume
  uint32_t parity = 0;   // phase of that slot's barrier

  // Takes the next piece: waits for it and returns its shared-memory address.
  auto take = [&](int *slot_out) -> uint32_t {
    const int s = slot;
    if (ok) ok = mbar_wait_all_lanes(full_s + 8u * (uint32_t)s, parity, tries);
    *slot_out = s;
    if (++slot == S) {
      slot = 0;
      parity ^= 1u;
    }
    return ring_s + (uint32_t)s * p.slot_bytes;
  };

  for (int k = 0; k < g1 - g0 && ok; ++k) {
    const DevQuantGroup gm = p.pairs[g0 + k];
    const uint32_t depth = UD ? (uint32_t)UD : gm.depth;
    uint32_t i0 = gm.slots, i1 = gm.slots;
    int sl[2];

    const uint32_t n0 = take(&sl[0]), n1 = take(&sl[1]);
    if (ok) {
      bool t0, t1;
      if constexpr (UD > 0)
        deep_walk<UD>(n0, n1, key_lane, ks, &i0, &i1, &t0, &t1);
      else
        deep_walk_any(depth, n0, n1, key_lane, ks, &i0, &i1, &t0, &t1);
      if (t0) {
        i0 = deep_walk_exact(n0, key_lane, ks, depth, p.exact_plane + gm.elem_off, rowp);
        ++ties;
      }
      if (t1) {
        i1 = deep_walk_exact(n1, key_lane, ks, depth, p.exact_plane + gm.elem_off + gm.slots, rowp);
        ++ties;
      }
    }
    // The two leaf values come straight from L2 and are consumed one pair later: a warp's
    // 32 leaves are scattered over the leaf plane (one sector each), which moves the same
    // bytes as staging the plane would, without taking ring slots.
    if (ok) {
      const uint32_t j0 = i0 - gm.slots, j1 = i1 - gm.slots;
      if (!LEAF_IDS) {
        acc += (double)pend0 + (double)pend1;
        pend0 = __ldg(p.leaf_plane + gm.elem_off + j0);
        pend1 = __ldg(p.leaf_plane + gm.elem_off + gm.slots + j1);
      }
      if (LEAF_IDS && live) {
        const int t0 = p.tree_index[(g0 + k) * 2], t1 = p.tree_index[(g0 + k) * 2 + 1];
        if (t0 >= 0) p.leaf_ids[row * p.num_trees + t0] = p.orig_leaf[gm.elem_off + j0];
        if (t1 >= 0) p.leaf_ids[row * p.num_trees + t1] = p.orig_leaf[gm.elem_off + gm.slots + j1];
      }
    }
    // this warp is done with the pair's two node planes
    __syncwarp();
    if (ok && lane == 0) {
      mbar_arrive(empty_s + 8u * (uint32_t)sl[0]);
      mbar_arrive(empty_s + 8u * (uint32_t)sl[1]);
    }
  }
  // every wait above is bounded: a wait that gave up ends the launch with a status word
  const bool failed = __syncthreads_or(!ok) != 0;
  if (failed) {
    if (tid == 0) atomicExch(p.status, 4);
    return;
  }
  acc += (double)pend0 + (double)pend1;
  if (p.tie_count != nullptr && ties) atomicAdd(p.tie_count, (unsigned long long)ties);
  if (LEAF_IDS || !live) return;
  if (p.write_partial)
    p.partial[(long long)blockIdx.y * p.n_rows + row] = (float)acc;
  else
    reinterpret_cast<float *>(p.out)[row] = apply_transform((float)((double)p.initial_value + acc), p.transform);
}

} // namespace tb
