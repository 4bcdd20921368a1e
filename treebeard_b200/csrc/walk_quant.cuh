// Walk kernel for the 15-bit-key layout (quant_pack.h): forests over rows too wide for
// an fp32 row tile.
//
// A PERSISTENT block of 24 warps takes the 32-row tiles blockIdx.x, blockIdx.x + gridDim.x,
// ... one after another and streams its tree chunk through shared memory once per tile.  A
// tile is held as 15-bit keys, transposed and paired: line m of the key tile (128 bytes)
// holds, for row j in word j, the keys of features 2m (low half) and 2m+1 (high half).
// Lane = row, so a key load of a warp touches 32 distinct banks whatever the features are.
//
// The warps are specialised; they meet only at mbarriers, never at a block barrier:
//  * 16 walkers in TWO independent sets of 8.  Set s takes the groups s, s+2, ... of the
//    chunk for all 32 rows; warp w of a set walks, in every group of 32 trees, the four
//    columns (lane + w + 8c) mod 32 in lock-step, so the 32 lanes of a warp read 32 distinct
//    columns of the node plane (one shared-memory wavefront per load) and the set covers
//    every (row, tree) pair of the group exactly once.  While one set waits for a piece, the
//    other keeps the issue slots and the shared-memory pipe busy.
//  * 2 ring producers, one per set.  Only the NODE planes stream through shared memory: two
//    16 KB pieces per group (upper levels, bottom level) through the set's three-slot ring,
//    filled by cp.async.bulk copies ("full" barriers); a walker warp releases a slot with one
//    arrive on its "empty" barrier.
//  * 2 leaf warps, one per set.  The walkers drop their leaf numbers into a small
//    shared-memory table (two per set, alternating); the leaf warp turns a finished table
//    into leaf-plane addresses, gathers the values straight from L2 one group ahead of their
//    use, and keeps the per-row sums.  Leaf warp 1 hands its sums to leaf warp 0, which
//    writes the tile's results.
//  * 4 stagers, one per quarter of tensor memory.  While the walkers are busy with tile i
//    they read the rows of tile i+1 (eight rows x 64 bytes per load instruction), turn
//    them into paired keys and park them in tensor memory (tcgen05.st); at the end of a
//    tile the walkers copy the parked keys into the key tile (tcgen05.ld, about a
//    microsecond), so the walk never waits for row data.  The first tile of a block
//    is staged by the walkers themselves; the rows of tile i+2 are prefetched into L2.
//
// The walk is fully unrolled per depth and written in PTX, the four columns of a lane
// interleaved.  A level costs one key load, two half2 comparisons on the low halves of
// (key, node word) -- "less than" picks the child, "equal" accumulates the tie flag -- one
// shift-add, one predicated add and one node load; the key's address is the node word
// shifted right by 15 plus the lane's base (bit 15 of a node word is 0, the feature code in
// the upper half is the key's byte offset halved).  Key ties are only flagged on the fast
// path; a flagged (row, tree) pair is then re-walked on the exact fp32 values from global
// memory.  Every lane polls its barrier itself (mbarrier.try_wait, bounded); a wait that
// gives up ends the launch with status 4 after tensor memory has been released.
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
  int32_t tiles_per_batch;       // narrow-row kernel (walk_quant_batch.cuh): 32-row tiles staged together
  // multiclass forests (narrow-row kernel only): the groups each walker set takes, in walking
  // order ([2][num_groups], set_count of them used; null = groups set, set + 2, ...), the class
  // of every group, and the output type (0 = fp32 class id, 1 = int8 class id)
  const int32_t *set_groups;
  int32_t set_count[2];
  const int32_t *group_class;
  int32_t num_classes, out_kind;
  int32_t skip_first_copy;       // failure drill: the first piece's copy is never issued, so its wait expires
  uint32_t wait_tries;           // polls before a wait gives up (0 = kQWaitTries)
  int32_t *status;
  unsigned long long *tie_count; // optional statistics
};

constexpr int kQRingBytes = 6 * 16384; // two walker sets x three 16 KB pieces
constexpr int kQLeafTableBytes = 4096; // [2 sets][2 tables][32 columns][32 rows] leaf numbers
constexpr uint32_t kQWaitTries = 1u << 20;

// 15-bit keys of this layout and of the deep-tree layout (walk_deep.cuh): integers in
// [1024, 31743] (quant_pack.h); NaN -> 1024.
__device__ __forceinline__ uint32_t quant_key15_dev(float v, float lo, float sc) {
  float y = __fmaf_rn(__fsub_rn(v, lo), -sc, 31741.0f);
  y = fminf(fmaxf(y, 1024.0f), 31743.0f);
  unsigned short h;
  asm("cvt.rmi.u16.f32 %0, %1;" : "=h"(h) : "f"(y));
  return h;
}

// The same with lattice features (negative scale, quant_pack.h): whole-number values land
// exactly on their key, other values get floor + 1.  Used where staging is cheap (the kernel
// for narrow rows) and for the node keys.
__device__ __forceinline__ uint32_t quant_key15_lattice_dev(float v, float lo, float sc) {
  if (sc < 0.f) {
    float y = __fmaf_rn(__fsub_rn(v, lo), sc, 31741.0f);
    y = fminf(fmaxf(y, 1024.0f), 31743.0f);
    return (uint32_t)(v == floorf(v) ? y : fminf(floorf(y) + 1.0f, 31743.0f));
  }
  return quant_key15_dev(v, lo, sc);
}
__device__ __forceinline__ uint32_t quant_threshold_key15_dev(float t, float lo, float sc) {
  return quant_key15_lattice_dev(t, lo, sc) + (sc < 0.f ? 1u : 0u);
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
__device__ __forceinline__ bool mbar_wait_all_lanes(uint32_t bar_addr, uint32_t parity, uint32_t tries = kQWaitTries) {
  for (uint32_t it = 0; it < tries; ++it) {
    uint32_t ok;
    // (no suspend-time hint: the hardware's own limit per try measured a little faster)
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 " selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(bar_addr), "r"(parity)
                 : "memory");
    if (ok) return true;
  }
  return false;
}

// ---------------------------------------------------------------------------
// The walk of four columns in lock-step, in PTX.  Operands of every block:
//   %0..%3    byte addresses of the current nodes of columns 0..3 (updated)
//   %4..%7    node words (updated)
//   %8        tie flags of the block, bit i = column i (out)
//   %9        the lane's base in the key tile
//   %10..%13  address constants of the step per column, %14..%17 those of the crossing into
//             the bottom-level piece, see quant_upper4
// A node at address A has its children at 2A + c (left) and 2A + c + 128 (right).
#define TBQ_DECL                                                                          \
  ".reg .b32 ka0, ka1, ka2, ka3, kx0, kx1, kx2, kx3;\n"                                   \
  ".reg .pred p0, p1, p2, p3, t0, t1, t2, t3, q;\n"
#define TBQ_KEY(i, n) "shr.u32 ka" #i ", " n ", 15;\n add.u32 ka" #i ", ka" #i ", %9;\n ld.shared.u16 kx" #i ", [ka" #i "];\n"
#define TBQ_CMP(i, n) "setp.lt.f16x2 p" #i "|q, kx" #i ", " n ";\n setp.eq.or.f16x2 t" #i "|q, kx" #i ", " n ", t" #i ";\n"
// the first comparison of a block starts the block's tie flags
#define TBQ_CMP0(i, n) "setp.lt.f16x2 p" #i "|q, kx" #i ", " n ";\n setp.eq.f16x2 t" #i "|q, kx" #i ", " n ";\n"
#define TBQ_ADV(i, a, c) "shl.b32 " a ", " a ", 1;\n add.u32 " a ", " a ", " c ";\n @p" #i " add.u32 " a ", " a ", 128;\n"
#define TBQ_LD(a, n) "ld.shared.u32 " n ", [" a "];\n"
#define TBQ_LEAF(i, a, c) "sub.u32 " a ", " a ", " c ";\n shr.u32 " a ", " a ", 6;\n @p" #i " add.u32 " a ", " a ", 1;\n"
#define TBQ_COMPARE                                                                       \
  TBQ_KEY(0, "%4") TBQ_KEY(1, "%5") TBQ_KEY(2, "%6") TBQ_KEY(3, "%7")                     \
  TBQ_CMP(0, "%4") TBQ_CMP(1, "%5") TBQ_CMP(2, "%6") TBQ_CMP(3, "%7")
#define TBQ_COMPARE0                                                                      \
  TBQ_KEY(0, "%4") TBQ_KEY(1, "%5") TBQ_KEY(2, "%6") TBQ_KEY(3, "%7")                     \
  TBQ_CMP0(0, "%4") TBQ_CMP0(1, "%5") TBQ_CMP0(2, "%6") TBQ_CMP0(3, "%7")
#define TBQ_ADVANCE TBQ_ADV(0, "%0", "%10") TBQ_ADV(1, "%1", "%11") TBQ_ADV(2, "%2", "%12") TBQ_ADV(3, "%3", "%13")
#define TBQ_LOAD TBQ_LD("%0", "%4") TBQ_LD("%1", "%5") TBQ_LD("%2", "%6") TBQ_LD("%3", "%7")
#define TBQ_LEAVES TBQ_LEAF(0, "%0", "%10") TBQ_LEAF(1, "%1", "%11") TBQ_LEAF(2, "%2", "%12") TBQ_LEAF(3, "%3", "%13")
#define TBQ_TIES "selp.u32 %8, 1, 0, t0;\n @t1 or.b32 %8, %8, 2;\n @t2 or.b32 %8, %8, 4;\n @t3 or.b32 %8, %8, 8;\n"
#define TBQ_ADVANCE_X TBQ_ADV(0, "%0", "%14") TBQ_ADV(1, "%1", "%15") TBQ_ADV(2, "%2", "%16") TBQ_ADV(3, "%3", "%17")
#define TBQ_STEP TBQ_COMPARE TBQ_ADVANCE TBQ_LOAD
#define TBQ_STEP0 TBQ_COMPARE0 TBQ_ADVANCE TBQ_LOAD
// the last upper level: compare and compute the address in the bottom-level piece (the
// constants %14..%17 carry the change of piece); nothing is loaded, the piece may not have arrived
#define TBQ_CROSS TBQ_COMPARE TBQ_ADVANCE_X
#define TBQ_CROSS0 TBQ_COMPARE0 TBQ_ADVANCE_X
#define TBQ_OPERANDS_UP                                                                   \
  : "+r"(A[0]), "+r"(A[1]), "+r"(A[2]), "+r"(A[3]), "=&r"(n[0]), "=&r"(n[1]), "=&r"(n[2]), "=&r"(n[3]), "=&r"(tb)   \
  : "r"(keys_lane), "r"(cu[0]), "r"(cu[1]), "r"(cu[2]), "r"(cu[3]), "r"(cx[0]), "r"(cx[1]), "r"(cx[2]), "r"(cx[3])
#define TBQ_OPERANDS_BOTTOM                                                               \
  : "+r"(A[0]), "+r"(A[1]), "+r"(A[2]), "+r"(A[3]), "=&r"(n[0]), "=&r"(n[1]), "=&r"(n[2]), "=&r"(n[3]), "=&r"(tb)   \
  : "r"(keys_lane), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3])

// Upper levels 0 .. DEPTH-2 of four columns of a group of DEPTH levels (2 <= DEPTH <= 8), one
// block of PTX: load the roots, DEPTH-2 steps inside the upper-level piece (compare, move to
// the child, load it), then the crossing into the bottom-level piece.
// In: A[i] = address of the root in the upper-level piece.  Out: the address of the
// bottom-level node reached; bit i of `ties` is set if column i met a key tie.
// cu = 128 - (root address), cx = cu + (first bottom-level node's address) - (root address)
// - 128 * (2^(DEPTH-1) - 1), per column.
template <int DEPTH>
__device__ __forceinline__ void quant_upper4(uint32_t (&A)[4], uint32_t &ties, uint32_t keys_lane,
                                             const uint32_t (&cu)[4], const uint32_t (&cx)[4]) {
  static_assert(DEPTH >= 2 && DEPTH <= 8, "the upper-level piece holds at most seven levels");
  [[maybe_unused]] uint32_t n[4];
  uint32_t tb;
  if constexpr (DEPTH == 2)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_CROSS0 TBQ_TIES "}" TBQ_OPERANDS_UP);
  else if constexpr (DEPTH == 3)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_CROSS TBQ_TIES "}" TBQ_OPERANDS_UP);
  else if constexpr (DEPTH == 4)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_CROSS TBQ_TIES "}" TBQ_OPERANDS_UP);
  else if constexpr (DEPTH == 5)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_TIES "}" TBQ_OPERANDS_UP);
  else if constexpr (DEPTH == 6)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_TIES "}" TBQ_OPERANDS_UP);
  else if constexpr (DEPTH == 7)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_TIES "}" TBQ_OPERANDS_UP);
  else
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_TIES "}"
                 TBQ_OPERANDS_UP);
  ties |= tb;
}
// The bottom level: load the node, compare; A[i] becomes the leaf number
// ((A - c) >> 6) + went right, c = address of the column's first bottom-level node.
__device__ __forceinline__ void quant_bottom4(uint32_t (&A)[4], uint32_t &ties, uint32_t keys_lane,
                                              const uint32_t (&c)[4]) {
  [[maybe_unused]] uint32_t n[4];
  uint32_t tb;
  asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_COMPARE0 TBQ_LEAVES TBQ_TIES "}" TBQ_OPERANDS_BOTTOM);
  ties |= tb;
}
__device__ __forceinline__ void quant_upper4_any(uint32_t depth, uint32_t (&A)[4], uint32_t &ties, uint32_t keys_lane,
                                                 const uint32_t (&cu)[4], const uint32_t (&cx)[4]) {
  switch (depth) {
  case 2: return quant_upper4<2>(A, ties, keys_lane, cu, cx);
  case 3: return quant_upper4<3>(A, ties, keys_lane, cu, cx);
  case 4: return quant_upper4<4>(A, ties, keys_lane, cu, cx);
  case 5: return quant_upper4<5>(A, ties, keys_lane, cu, cx);
  case 6: return quant_upper4<6>(A, ties, keys_lane, cu, cx);
  case 7: return quant_upper4<7>(A, ties, keys_lane, cu, cx);
  default: return quant_upper4<8>(A, ties, keys_lane, cu, cx);
  }
}

// Re-walks behind a key tie: the staged keys decide wherever they can, and only the tied
// comparisons read the exact fp32 values from global memory.
// Upper levels 0 .. depth-2 of the column at address `up` of the upper-level piece; returns
// the number of the bottom-level node reached (0 .. 2^(depth-1) - 1).
__device__ __noinline__ uint32_t quant_upper_exact(uint32_t up, uint32_t keys_lane, const float *exact_plane,
                                                   size_t plane_row, uint32_t depth, uint32_t col,
                                                   const float *rowp) {
  uint32_t s = 0; // level-order number of the node
  for (uint32_t d = 0; d + 1 < depth; ++d) {
    const uint32_t node = lds_u32(up + s * 128u);
    const uint32_t code = node >> 16, kt = node & 0x7fffu;
    const uint32_t kx = lds_u16(keys_lane + 2u * code);
    bool right = kx < kt;
    if (kx == kt) {
      const uint32_t f = (code >> 6) * 2u + (code & 1u);
      right = !(__ldg(rowp + f) < __ldg(exact_plane + (plane_row + s) * 32u + col));
    }
    s = 2u * s + 1u + (right ? 1u : 0u);
  }
  return s - ((1u << (depth - 1)) - 1u);
}
// The bottom level: node j of the column at address `bot` of the bottom-level piece;
// returns the leaf number.
__device__ __noinline__ uint32_t quant_bottom_exact(uint32_t bot, uint32_t j, uint32_t keys_lane,
                                                    const float *exact_plane, size_t plane_row, uint32_t depth,
                                                    uint32_t col, const float *rowp) {
  const uint32_t node = lds_u32(bot + j * 128u);
  const uint32_t code = node >> 16, kt = node & 0x7fffu;
  const uint32_t kx = lds_u16(keys_lane + 2u * code);
  bool right = kx < kt;
  if (kx == kt) {
    const uint32_t f = (code >> 6) * 2u + (code & 1u);
    // the bottom level fills the second half of the planes (quant_plane_slot)
    right = !(__ldg(rowp + f) < __ldg(exact_plane + (plane_row + (1u << (depth - 1)) + j) * 32u + col));
  }
  return 2u * j + (right ? 1u : 0u);
}

// Fills the key field of every split node from its exact threshold (run once at upload,
// so that thresholds and row values are quantised by the very same device arithmetic).
// wide = 1: the 15-bit keys and feature codes of the wide-row layout (quant_pack.h);
// 0: the same keys with plain feature indices, the deep-tree layout (deep_pack.h).
__global__ void tb_quant_fill_keys(uint32_t *node_plane, const float *exact_plane, const float *lo,
                                   const float *scale, unsigned long long n, int num_features, int wide) {
  const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t node = node_plane[i];
  if (wide) {
    const uint32_t code = node >> 16, f = (code >> 6) * 2u + (code & 1u);
    if (f < (uint32_t)num_features) node_plane[i] = (code << 16) | quant_threshold_key15_dev(exact_plane[i], lo[f], scale[f]);
  } else {
    const uint32_t f = node >> 16;
    if (f < (uint32_t)num_features) node_plane[i] = (f << 16) | quant_threshold_key15_dev(exact_plane[i], lo[f], scale[f]);
  }
}

constexpr int kQPiece = 16384;  // one ring slot: half a plane of a group of 8 levels
constexpr int kQSetWarps = 8;   // walker warps per set
constexpr int kQWalkers = 2 * kQSetWarps;
constexpr int kQStagers = 4;             // warps 16..19: one per lane quarter of tensor memory
constexpr int kQLeafWarps = 2;           // warps 20, 21: leaf gathers and row sums of set 0 / set 1
constexpr int kQProducers = 2;           // warps 22, 23: ring producers of set 0 / set 1
constexpr int kQThreads = 32 * (kQWalkers + kQStagers + kQLeafWarps + kQProducers);
constexpr int kQBarBytes = 512;          // mbarriers, a few control words, one row of partial sums
constexpr uint32_t kQTmemCols = 256;     // 128 lanes x 256 columns x 4 bytes = the 128 KB of a key tile
constexpr int kQStagerPairs = 256;       // feature pairs per stager = columns of its lane quarter
constexpr int kQUnitPairs = 8;           // pairs per staging unit: 16 features of all 32 rows

// L2 eviction policies: the forest (2 MB, re-read by every tile of every block) should stay
// in L2 while the rows (gigabytes, read once) stream through it.
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
               : "memory");
}
__device__ __forceinline__ float4 ldg_f4_hint(const float *ptr, uint64_t pol) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr), "l"(pol));
  return v;
}
__device__ __forceinline__ float ldg_f32_hint(const float *ptr, uint64_t pol) {
  float v;
  asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(ptr), "l"(pol));
  return v;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void tmem_store8(uint32_t taddr, const uint32_t (&w)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&w)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
               "%14, %15}, [%16];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
                 "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory bytes of the key tile: one 128-byte line per pair of features, the
// sentinel feature (index num_features) included.
__host__ __device__ constexpr int quant_key_tile_bytes(int num_features) { return (num_features + 2) / 2 * 128; }

// UD: depth shared by every group of the forest (0 = mixed depths, read per group at run
// time; with a constant depth the walk is called directly and plane offsets are computed).
// LEAF_IDS: the launch records leaf ids instead of predictions.
//
// A block is persistent: it takes the 32-row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// and is specialised by warp:
//   warps 0..15   walkers, two sets of eight (set s takes the groups s, s+2, ... of the chunk).
//                 A walker ends a group by dropping its four leaf NUMBERS (one byte each) into
//                 the set's [column][row] table: walkers touch shared memory only.
//   warps 16..19  stagers: while a tile is walked they turn the NEXT tile's rows into keys and
//                 park the finished key words in tensor memory -- the only on-chip space left
//                 beside the 128 KB key tile -- stager s in lane quarter s (feature pairs
//                 256 s ...).  At the end of the tile the sixteen walker warps copy
//                 the words from tensor memory into the key tile with conflict-free stores.
//   warps 20, 21  leaf warps, one per set: pick up each finished table, gather the leaf values
//                 from the column-major leaf plane in L2 (lane = row; the leaves that the 32
//                 rows need of ONE tree lie within 1 KB, at most 8 lines per warp load -- in
//                 the walk's own lane assignment the 32 lanes sit in 32 different trees), keep
//                 the row sums of their set and write the tile's results.  The long-latency
//                 loads -- rows and leaves -- thus never sit in a walker's instruction stream.
//   warps 22, 23  ring producers, one per set: the node planes stream through three 16 KB slots
//                 per set; a producer issues the bulk copy of the piece that comes three later
//                 as soon as the set's eight walkers have arrived on the slot's barrier.
// The first tile of a block is staged by the walkers themselves, straight into the key tile.
// All hand-offs go through mbarriers with bounded waits; a wait that gives up ends the
// launch with a status word instead of a hang.
//
// Shared memory: [0,512) mbarriers -- full[set][3], empty[set][3], table_full[set][2],
// table_free[set][2], tile_done, keys_ready, sum_ready, sum_free --, the tensor-memory address
// and the row sums that leaf warp 1 hands to leaf warp 0; the ring of six 16 KB pieces (three
// per set); the leaf-number tables (two per set, 1 KB each); the key tile.
// (24 warps x 32 x 80 registers fill the register file)
template <int UD, bool LEAF_IDS>
__global__ void __launch_bounds__(kQThreads, 1) tb_walk_quant_kernel(const QuantParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31;
  // the warp's number through a shuffle: the compiler then knows that it -- and every role, set,
  // slot and feature index derived from it -- is the same for all lanes (uniform registers and
  // uniform constant loads instead of per-lane ones)
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const bool stager = warp >= kQWalkers && warp < kQWalkers + kQStagers;
  const bool leafer = warp >= kQWalkers + kQStagers && warp < kQWalkers + kQStagers + kQLeafWarps;
  const bool producer = warp >= kQWalkers + kQStagers + kQLeafWarps;
  // the set this warp works for (walkers: warps 0..7 / 8..15; leaf warps and producers: one per set)
  const int set = (warp >= kQWalkers + kQStagers ? warp - kQWalkers - kQStagers : warp / kQSetWarps) & 1;
  const int sw = warp % kQSetWarps;
  const int F = p.num_features;
  const uint32_t bars_s = smem_u32(smem_raw);
  const uint32_t full_s = bars_s + (uint32_t)set * 24u, empty_s = bars_s + 48u + (uint32_t)set * 24u;
  const uint32_t table_s = bars_s + 96u + (uint32_t)set * 16u;
  const uint32_t tile_done_s = bars_s + 128u, keys_ready_s = bars_s + 144u;
  const uint32_t sum_ready_s = bars_s + 184u, sum_free_s = bars_s + 192u, sums1_s = bars_s + 256u;
  const uint32_t table_free_s = bars_s + 152u + (uint32_t)set * 16u;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_raw + 240);
  unsigned char *ring = smem_raw + kQBarBytes + (size_t)set * 3 * kQPiece;
  const uint32_t ring_s = smem_u32(ring);
  // leaf numbers of a group, exchanged between the warps of a set (see below)
  const uint32_t ltab0_s = smem_u32(smem_raw + kQBarBytes) + 6 * kQPiece;
  const uint32_t ltab_s = ltab0_s + (uint32_t)set * 2048u;
  // key tile: line m = features 2m | 2m+1 << 16 for the 32 rows
  const uint32_t keys_s = ltab0_s + kQLeafTableBytes;
  const uint32_t keys_lane = keys_s + lane * 4;

  const long long num_tiles = (p.n_rows + 31) / 32;
  const int my_tiles = (int)((num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const bool use_tmem = my_tiles > 1; // the host launches fewer blocks than tiles only for rows that 16-byte loads can read
  const int g0 = blockIdx.y * p.groups_per_chunk;
  const int g1 = min(p.num_groups, g0 + p.groups_per_chunk);
  const int NG = g1 - g0;
  const int NGs = (NG - set + 1) / 2; // groups set, set + 2, ... of the chunk
  const int P = 2 * NGs;              // pieces of this set per tile: upper levels and bottom level of the node planes
  const int NP = (F + 2) / 2;         // feature pairs = lines of the key tile

  if (tid == 0) {
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
    for (int i = 0; i < 6; ++i) mbar_init(bars + i, 1);            // full: the copy's bytes
    for (int i = 6; i < 12; ++i) mbar_init(bars + i, kQSetWarps);  // empty: one arrival per walker warp of the set
    for (int i = 12; i < 16; ++i) mbar_init(bars + i, kQSetWarps); // table_full: every walker of the set has written
    mbar_init(bars + 16, kQWalkers + kQStagers);                   // tile_done: the tile is walked, the next one's keys are staged
    mbar_init(bars + 18, kQWalkers + kQStagers);                   // keys_ready: every walker has copied its share of the keys, the stagers know of it
    for (int i = 19; i < 23; ++i) mbar_init(bars + i, 1);          // table_free: the leaf warp has read the table
    mbar_init(bars + 23, 1);                                       // sum_ready: leaf warp 1 has written its row sums
    mbar_init(bars + 24, 1);                                       // sum_free: leaf warp 0 has read them
    fence_barrier_init();
  }
  if (warp == 0 && use_tmem) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bars_s + 240u), "r"(kQTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = use_tmem ? *tmem_slot : 0u;

  // plane offset (in rows of 32 elements) and depth of group gi of the chunk
  auto group_of = [&](int gi) -> uint2 {
    if constexpr (UD > 0) return make_uint2((uint32_t)(g0 + gi) << UD, (uint32_t)UD);
    const DevQuantGroup gm = p.groups[g0 + gi];
    return make_uint2((uint32_t)(gm.elem_off >> 5), gm.depth);
  };

  bool ok = true;
  unsigned tie_count = 0;
  const uint64_t keep = l2_policy_keep(), stream = l2_policy_stream();
  const uint32_t wait_tries = p.wait_tries ? p.wait_tries : kQWaitTries;
  auto mbar_wait_all_lanes = [wait_tries](uint32_t bar_addr, uint32_t parity) {
    return tb::mbar_wait_all_lanes(bar_addr, parity, wait_tries);
  };
  // Copy of piece `piece` of a tile (upper levels of group piece/2 of the set for even
  // numbers, its bottom level for odd ones) into ring slot `slot` of the set.
  auto issue = [&](int piece, int slot) {
    const uint2 gm = group_of(2 * (piece >> 1) + set);
    const uint32_t hs = 1u << (gm.y - 1); // slots per piece
    const size_t off = ((size_t)gm.x + ((piece & 1) ? hs : 0u)) * 32;
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem_raw) + set * 3 + slot;
    mbar_expect_tx(bar, hs * 128u);
    bulk_g2s_hint(ring + (size_t)slot * kQPiece, p.node_plane + off, hs * 128u, bar, keep);
  };
  // Staging of a tile's keys through tensor memory.  Lane quarter q (= warp mod 4) belongs to
  // stager q and holds the feature pairs [256 q, 256 q + 256), in units of eight pairs (16
  // features) of all 32 rows.  Within a unit lane 4a + j loads 16 bytes -- features 4j .. 4j+3
  // of the unit -- of the rows a, a+8, a+16, a+24: four neighbouring lanes read 64 contiguous
  // bytes of a row (8 lines per load instruction instead of the 32 of a lane = row pattern),
  // and the lane's key parameters are one 16-byte load each.  A lane thus finishes the words of
  // pairs 2j, 2j+1 for four rows; it stores them rotated by j (slot s holds row
  // a + 8 ((s + j) mod 4)), so that when the columns are copied into the key tile the 32 lanes
  // of a store hit 32 different rows, i.e. banks.
  const int pair0 = (warp & 3) * kQStagerPairs;
  const uint32_t taddr = tmem_base + ((uint32_t)(warp & 3) * 32u << 16);
  const int sa = lane >> 2, sj = lane & 3;
  struct Unit { // a staging unit in flight
    float4 x[4], lo, sc;
  };
  // loads of unit u of the tile whose first row is at `base`, `live_rows` of them real
  auto unit_load = [&](const float *base, int live_rows, int u, Unit &un) {
    const int f = 2 * (pair0 + kQUnitPairs * u) + 4 * sj; // a multiple of 4, like F: f < F covers f + 3
    const bool in = f < F;                                // p.lo / p.scale are padded to a multiple of four entries
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = sa + 8 * q;
      un.x[q] = (in && r < live_rows) ? ldg_f4_hint(base + (long long)r * p.ld + f, stream) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    un.lo = in ? __ldg(reinterpret_cast<const float4 *>(p.lo + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
    un.sc = in ? __ldg(reinterpret_cast<const float4 *>(p.scale + f)) : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  // keys of unit u into the quarter's columns of tensor memory
  auto unit_store = [&](int u, const Unit &un) {
    const int f = 2 * (pair0 + kQUnitPairs * u) + 4 * sj;
    uint32_t w[4][2];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t k0 = quant_key15_dev(un.x[q].x, un.lo.x, un.sc.x), k1 = quant_key15_dev(un.x[q].y, un.lo.y, un.sc.y);
      uint32_t k2 = quant_key15_dev(un.x[q].z, un.lo.z, un.sc.z), k3 = quant_key15_dev(un.x[q].w, un.lo.w, un.sc.w);
      if (f >= F) k0 = k1 = k2 = k3 = 0x7bffu; // the sentinel feature (and padding): the largest key
      w[q][0] = k0 | (k1 << 16);
      w[q][1] = k2 | (k3 << 16);
    }
    // rotate the four rows left by j: slot s <- row index (s + j) mod 4
    uint32_t t[4][2], o[8];
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4)
#pragma unroll
      for (int e = 0; e < 2; ++e) t[s4][e] = (sj & 1) ? w[(s4 + 1) & 3][e] : w[s4][e];
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4)
#pragma unroll
      for (int e = 0; e < 2; ++e) o[2 * s4 + e] = (sj & 2) ? t[(s4 + 2) & 3][e] : t[s4][e];
    tmem_store8(taddr + (uint32_t)(kQUnitPairs * u), o);
  };
  // This warp's share of the copy from tensor memory into the key tile: the quarter's columns
  // in chunks of 16 (two units), dealt to the quarter's four walker warps (rank = warp / 4; a warp reaches only
  // the lane quarter warp mod 4; the stagers stay out of it and finish their tile switch at once).  Column
  // 8u + 2s + e of lane 4a + j is the word of pair 256 q + 8u + 2j + e for row a + 8 ((s + j) mod 4).
  auto copy_keys_out = [&]() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t rowoff[4];
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4) rowoff[s4] = (uint32_t)(sa + 8 * ((s4 + sj) & 3)) * 4u;
#pragma unroll 1
    for (int c0 = 16 * (warp >> 2); c0 < kQStagerPairs && pair0 + c0 < NP; c0 += 16 * 4) {
      uint32_t w[16];
      tmem_load16(taddr + (uint32_t)c0, w);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int m = pair0 + c0 + 8 * (i >> 3) + 2 * sj + (i & 1);
        if (m < NP)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(keys_s + (uint32_t)m * 128u + rowoff[(i >> 1) & 3]), "r"(w[i]) : "memory");
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  };

  if (stager) {
    // ---- stagers: keys of the next tile into tensor memory
    const int NU = max(0, (min(NP, pair0 + kQStagerPairs) - pair0 + kQUnitPairs - 1) / kQUnitPairs);
    for (int it = 0; it < my_tiles && ok; ++it) {
      const bool has_next = it + 1 < my_tiles;
      if (has_next) {
        const long long tile = blockIdx.x + (long long)it * gridDim.x;
        const long long row0_next = (tile + gridDim.x) * 32;
        const float *base = p.rows + row0_next * p.ld;
        const int live_rows = (int)min((long long)32, p.n_rows - row0_next);
        if (it + 2 < my_tiles && warp == kQWalkers) { // the rows of the tile after that are pulled into L2
          const long long row_after = (tile + 2ll * gridDim.x) * 32 + lane;
          if (row_after < p.n_rows)
            asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(p.rows + row_after * p.ld),
                         "r"((uint32_t)F * 4u), "l"(stream)
                         : "memory");
        }
        Unit ua, ub; // two units in flight
        if (0 < NU) unit_load(base, live_rows, 0, ua);
        if (1 < NU) unit_load(base, live_rows, 1, ub);
#pragma unroll 1
        for (int u = 0; u < NU; u += 2) {
          unit_store(u, ua);
          if (u + 2 < NU) unit_load(base, live_rows, u + 2, ua);
          if (u + 1 < NU) {
            unit_store(u + 1, ub);
            if (u + 3 < NU) unit_load(base, live_rows, u + 3, ub);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(tile_done_s);
      ok = mbar_wait_all_lanes(tile_done_s, (uint32_t)it & 1u);
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(keys_ready_s);
      ok = mbar_wait_all_lanes(keys_ready_s, (uint32_t)it & 1u); // the copy is complete: tensor memory may be rewritten
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
  } else if (producer) {
    // ---- the set's ring producer.  The q-th piece (upper levels of a group for even q, its
    // bottom level for odd q) goes to slot q mod 3 as soon as every walker warp of the set has
    // released the piece that was there.
    int slot = 0;
    uint32_t round = 0; // how often the slots have wrapped
    for (int it = 0; it < my_tiles && ok; ++it) {
      for (int piece = 0; piece < P && ok; ++piece) {
        if (round > 0) ok = mbar_wait_all_lanes(empty_s + 8u * (uint32_t)slot, (round - 1u) & 1u);
        if (ok && lane == 0 && !(p.skip_first_copy && it == 0 && piece == 0)) issue(piece, slot);
        if (++slot == 3) {
          slot = 0;
          ++round;
        }
      }
    }
  } else if (leafer) {
    // ---- leaf warps: gather the leaf values of every finished table of the set, keep its row
    // sums; leaf warp 0 adds the two sets' sums and writes the results
    uint32_t kk = 0; // groups of the set seen so far (tables alternate, their barriers change phase)
    const uint32_t ltab_lane = ltab_s + (uint32_t)lane;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const long long tile = blockIdx.x + (long long)it * gridDim.x;
      const long long row = tile * 32 + lane;
      const bool live = row < p.n_rows;
      // Leaf values are consumed one group after their loads were issued (a ring of 32), and
      // summed in eight independent accumulators that are combined pairwise at the end: a single
      // running fp32 sum over a thousand leaves would carry several times the rounding error.
      float pend[32], acc8[8];
#pragma unroll
      for (int i = 0; i < 32; ++i) pend[i] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc8[i] = 0.f;
      for (int k = 0; k < NGs && ok; ++k, ++kk) {
        const int gi = 2 * k + set;
        const uint2 gm = group_of(gi);
        const uint32_t slots = 2u << (gm.y - 1);
        ok = mbar_wait_all_lanes(table_s + 8u * (kk & 1u), (kk >> 1) & 1u);
        if (!ok) break;
        const uint32_t tab = ltab_lane + (kk & 1u) * 1024u;
        // (element offsets fit 32 bits: the host refuses planes of 2^32 elements or more)
#pragma unroll
        for (int oct = 0; oct < 4; ++oct) {
          uint32_t e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t c = (uint32_t)(8 * oct + i);
            uint32_t leaf;
            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(leaf) : "r"(tab + c * 32u) : "memory");
            e[i] = gm.x * 32u + c * slots + leaf;
          }
          if (oct == 3) { // every column has been read: the table may be rewritten
            __syncwarp();
            if (lane == 0) mbar_arrive(table_free_s + 8u * (kk & 1u));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = 8 * oct + i;
            if (LEAF_IDS) {
              if (live) {
                const int t = p.tree_index[(g0 + gi) * 32 + c];
                if (t >= 0) p.leaf_ids[row * p.num_trees + t] = p.orig_leaf[e[i]];
              }
            } else {
              acc8[i] += pend[c]; // loaded a group ago
              pend[c] = ldg_f32_hint(p.leaf_plane + e[i], keep);
            }
          }
        }
      }
      if (!ok) break;
      if constexpr (!LEAF_IDS) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc8[i & 7] += pend[i];
        const float acc = ((acc8[0] + acc8[1]) + (acc8[2] + acc8[3])) + ((acc8[4] + acc8[5]) + (acc8[6] + acc8[7]));
        // the row's result: leaf warp 1 hands its sums to leaf warp 0 (well off the walkers' path)
        if (set == 1) {
          if (it > 0) ok = mbar_wait_all_lanes(sum_free_s, (uint32_t)(it - 1) & 1u);
          if (!ok) break;
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(sums1_s + (uint32_t)lane * 4u), "f"(acc) : "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_ready_s);
        } else {
          ok = mbar_wait_all_lanes(sum_ready_s, (uint32_t)it & 1u);
          if (!ok) break;
          const float s = acc + lds_f32(sums1_s + (uint32_t)lane * 4u);
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_free_s);
          if (live) {
            if (p.write_partial)
              p.partial[(long long)blockIdx.y * p.n_rows + row] = s;
            else
              reinterpret_cast<float *>(p.out)[row] = apply_transform(p.initial_value + s, p.transform);
          }
        }
      }
    }
  } else {
    // ---- the walk
    // the four columns this lane walks in every group of its set: warp w takes the columns
    // (lane + w + 8c) mod 32, so a load of the warp touches 32 distinct columns (banks) and
    // the eight warps of the set cover every (row, tree) pair of the group exactly once
    uint32_t col[4], colb[4], drop_s[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      col[c] = (uint32_t)(lane + sw + 8 * c) & 31u;
      colb[c] = ring_s + col[c] * 4u;                     // the column's address in slot 0
      drop_s[c] = ltab_s + col[c] * 32u + (uint32_t)lane; // where its leaf number goes (table 0)
    }
    // pieces are consumed in order, tile after tile: slot and phase of the next piece, and the
    // phase of the leaf-number tables, follow from counters
    int slot = 0;
    uint32_t parity = 0, kk = 0; // kk: groups this warp has walked so far
    const bool elected = lane == 0;
    // ---- the first tile: the walkers stage the rows themselves
    {
      // A warp takes a block of 32 consecutive features: every load instruction reads 128
      // contiguous bytes of ONE row (lane = feature), so DRAM sees whole lines and adjacent
      // warps continue the same rows.  A lane thus collects its feature for all 32 rows and
      // packs the keys two to a register; neighbouring lanes (features 2m, 2m+1) then swap
      // halves through a shuffle, so that the even lane holds the finished words of rows
      // 0..15 and the odd lane those of rows 16..31, 64 contiguous bytes each, written with
      // four 16-byte stores.  Loads go to L2 only; sixteen are in flight per thread.
      const long long row0 = (long long)blockIdx.x * 32;
      const int live_rows = (int)min((long long)32, p.n_rows - row0);
      const float *tile = p.rows + row0 * p.ld;
      const bool odd = lane & 1;
      // byte selectors: the even feature's packed keys are operand a on even lanes, b on odd
      const uint32_t sel_lo = odd ? 0x1054u : 0x5410u, sel_hi = odd ? 0x3276u : 0x7632u;
      for (int f0 = warp * 32; f0 <= F; f0 += kQWalkers * 32) {
        const int f = f0 + lane;
        const bool fok = f < F;
        const float lo = fok ? __ldg(p.lo + f) : 0.f, sc = fok ? __ldg(p.scale + f) : 0.f;
        uint32_t packed[16]; // keys of rows 2i | 2i+1 << 16 of this lane's feature
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
            packed[part * 8 + r / 2] = quant_key15_dev(x[r], lo, sc) | (quant_key15_dev(x[r + 1], lo, sc) << 16);
        }
        if (f == F) { // the sentinel feature: the largest key for every row
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[i] = 0x7bff7bffu;
        }
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t own = odd ? packed[8 + i] : packed[i];
          const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? packed[i] : packed[8 + i], 1);
          w[2 * i] = __byte_perm(own, got, sel_lo);
          w[2 * i + 1] = __byte_perm(own, got, sel_hi);
        }
        if (f <= F + (odd ? 1 : 0)) { // lanes of a pair that holds at least one real feature
          const uint32_t dst = keys_s + (uint32_t)(f >> 1) * 128u + (odd ? 64u : 0u);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 16u * c), "r"(w[4 * c]),
                         "r"(w[4 * c + 1]), "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                         : "memory");
        }
      }
      // only the walkers take part, and nothing can have failed yet
      asm volatile("bar.sync 1, %0;" ::"r"(32 * kQWalkers) : "memory");
    }

    for (int it = 0; it < my_tiles && ok; ++it) {
      const long long tile = blockIdx.x + (long long)it * gridDim.x;
      const long long row = tile * 32 + lane;
      const bool live = row < p.n_rows;
      const float *rowp = p.rows + (live ? row : 0) * p.ld;
      const bool has_next = it + 1 < my_tiles;
      for (int k = 0; k < NGs && ok; ++k, ++kk) {
        const int gi = 2 * k + set;
        const uint2 gm = group_of(gi);
        const uint32_t depth = UD ? (uint32_t)UD : gm.y, hs = 1u << (depth - 1);

        // the two pieces of this group
        const uint32_t su = (uint32_t)slot, pu = parity;
        if (++slot == 3) { slot = 0; parity ^= 1u; }
        const uint32_t sb = (uint32_t)slot, pb = parity;
        if (++slot == 3) { slot = 0; parity ^= 1u; }
        uint32_t A[4], bot[4], ties = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          bot[c] = colb[c] + sb * kQPiece;
          A[c] = bot[c];
        }

        // upper levels 0 .. depth-2: ends at the addresses of the bottom-level nodes
        ok = mbar_wait_all_lanes(full_s + 8u * su, pu);
        if (!ok) break;
        if (depth >= 2) {
          uint32_t cu[4], cx[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            A[c] = colb[c] + su * kQPiece;
            cu[c] = 128u - A[c];
            cx[c] = cu[c] + bot[c] - A[c] - 128u * (hs - 1u);
          }
          if constexpr (UD >= 2)
            quant_upper4<UD>(A, ties, keys_lane, cu, cx);
          else
            quant_upper4_any(depth, A, ties, keys_lane, cu, cx);
          if (ties) { // rare: the tied column is walked again on exact values
#pragma unroll
            for (int c = 0; c < 4; ++c)
              if (ties & (1u << c)) {
                A[c] = bot[c] + 128u * quant_upper_exact(colb[c] + su * kQPiece, keys_lane, p.exact_plane, gm.x, depth,
                                                         col[c], rowp);
                ++tie_count;
              }
            ties = 0;
          }
        }
        __syncwarp();
        if (elected) mbar_arrive(empty_s + 8u * su);

        // bottom decision level; the leaf numbers go into the table
        ok = mbar_wait_all_lanes(full_s + 8u * sb, pb);
        if (!ok) break;
        quant_bottom4(A, ties, keys_lane, bot);
        if (ties) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (ties & (1u << c)) {
              A[c] = quant_bottom_exact(bot[c], A[c] >> 1, keys_lane, p.exact_plane, gm.x, depth, col[c], rowp);
              ++tie_count;
            }
        }
        // the leaf numbers go into table kk mod 2, once the leaf warp has read what group kk - 2 left there
        if (kk >= 2) {
          ok = mbar_wait_all_lanes(table_free_s + 8u * (kk & 1u), ((kk >> 1) - 1u) & 1u);
          if (!ok) break;
        }
        const uint32_t buf = (kk & 1u) * 1024u;
#pragma unroll
        for (int c = 0; c < 4; ++c) asm volatile("st.shared.u8 [%0], %1;" ::"r"(drop_s[c] + buf), "r"(A[c]) : "memory");
        __syncwarp();
        if (elected) {
          mbar_arrive(empty_s + 8u * sb);
          mbar_arrive(table_s + 8u * (kk & 1u));
        }
      }
      if (!ok) break;

      // ---- end of the tile.  Every walker and stager arrives; past this barrier the key tile and
      // the leaf-number tables are free and the next tile's keys are complete in tensor memory.
      __syncwarp();
      if (elected) mbar_arrive(tile_done_s);
      ok = mbar_wait_all_lanes(tile_done_s, (uint32_t)it & 1u);
      if (!ok) break;
      if (has_next) copy_keys_out();
      __syncwarp();
      if (elected) mbar_arrive(keys_ready_s);
      ok = mbar_wait_all_lanes(keys_ready_s, (uint32_t)it & 1u);
    }
  }
  // every wait above is bounded: a wait that gave up ends the launch with a status word
  const bool failed = __syncthreads_or(!ok) != 0;
  if (warp == 0 && use_tmem) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kQTmemCols) : "memory");
  }
  if (failed) {
    if (tid == 0) atomicExch(p.status, 4);
    return;
  }
  if (p.tie_count != nullptr && tie_count) atomicAdd(p.tie_count, (unsigned long long)tie_count);
}

} // namespace tb
