// Walk kernel for the 15-bit-key layout (quant_pack.h) over NARROW rows: the key tiles of
// several 32-row tiles fit shared memory together, so a block stages a BATCH of up to 16
// tiles (512 rows) and streams its tree chunk through shared memory once per batch instead
// of once per tile (walk_quant.cuh, the kernel for rows so wide that one key tile fills
// shared memory, has to re-stream the forest for every 32 rows).
//
// A persistent block of 22 warps takes the batches blockIdx.x, blockIdx.x + gridDim.x, ...:
//  * 16 walkers in two sets of 8, as in walk_quant.cuh: set s takes the groups s, s+2, ... of
//    the chunk; warp w of a set walks the four columns (lane + w + 8c) mod 32 of every group in
//    lock-step, lane = row.  For a group the warp waits once for the two 16 KB pieces of the
//    node planes, then walks the group for EVERY tile of the batch, so the per-group hand-offs
//    (three barrier waits, three arrivals, the address set-up) are paid once per batch.  The
//    walkers also stage the batch: thread = row, keys written as paired lines
//    (word j of line m = keys of features 2m | 2m+1 << 16 for row j).
//  * 4 leaf warps, two per set (one takes the even tiles of the batch, one the odd tiles; one
//    leaf warp per scheduler): the walkers drop their leaf numbers into [tile][column][row]
//    byte tables (two per set, alternating by group); a leaf warp gathers the leaf values
//    from L2, sums a group pairwise and keeps one running sum per tile.  The leaf warps of set 1
//    hand their sums to those of set 0, which write the batch's results.  Multiclass forests: a group
//    belongs to one class and every class to one set, whose leaf warp meets the classes in
//    increasing order; it keeps the running sum of the current class and, when the class
//    changes, updates the best class so far (ties go to the higher class index, the rule of
//    the reference's generated arg-max, src/reduction/LowerReduceOps.cpp:148-189); leaf warp 0
//    merges the two sets' winners and writes the class id (or each leaf warp writes its
//    classes' sums, where per-class partial sums are asked for).
//  * 2 ring producers, one per set: four 16 KB slots per set (the two pieces of the group
//    being walked and both pieces of the next one), cp.async.bulk + mbarrier.
// Ties between 15-bit keys are flagged by the walk and re-walked on the exact fp32 values, as
// in walk_quant.cuh.  Every wait is bounded; a wait that gives up ends the launch with status 4.
//
// Reference counterparts: as for walk_quant.cuh; the batch is the reference's row tile of a
// thread block (src/gpu/GPURepresentations.cpp:279-399) with its trees cached stage by stage.
#pragma once
#include "walk_quant.cuh"

namespace tb {

constexpr int kQBWalkers = 16, kQBLeafWarps = 4, kQBProducers = 2;
constexpr int kQBThreads = 32 * (kQBWalkers + kQBLeafWarps + kQBProducers);
constexpr int kQBMaxThreads = 768; // 22 warps are allocated as 24: 80 registers per thread
constexpr int kQBMaxTiles = 16;   // tiles per batch: one per walker warp when the batch is staged
constexpr int kQBBarBytes = 512;
constexpr int kQBSlots = 4;       // ring slots per set
constexpr int kQBRingBytes = 2 * kQBSlots * 16384;
// shared memory: barriers, the ring, then per tile of the batch its leaf-number tables
// (2 sets x 2 tables x 1 KB), what leaf warp 1 hands over (row sums, or best class sums and
// their classes: 256 B) and its key tile
__host__ __device__ constexpr int quant_batch_tile_bytes(int num_features) {
  return 4 * 1024 + 256 + quant_key_tile_bytes(num_features);
}
__host__ __device__ constexpr int quant_batch_smem_bytes(int num_features, int tiles) {
  return kQBBarBytes + kQBRingBytes + tiles * quant_batch_tile_bytes(num_features);
}

// All DEPTH levels of four columns in ONE block of PTX, for callers that hold both pieces of
// the group (walk_quant_batch.cuh): the upper levels as in quant_upper4, then the bottom level
// as in quant_bottom4 (cb = address of the column's first bottom-level node).  In: A[i] =
// address of the root.  Out: A[i] = leaf number; bit i of `ties` is set if column i met a key
// tie on any level.
#define TBQ_LEAVES_B TBQ_LEAF(0, "%0", "%18") TBQ_LEAF(1, "%1", "%19") TBQ_LEAF(2, "%2", "%20") TBQ_LEAF(3, "%3", "%21")
#define TBQ_BOTTOM TBQ_LOAD TBQ_COMPARE TBQ_LEAVES_B TBQ_TIES
#define TBQ_OPERANDS_FULL TBQ_OPERANDS_UP, "r"(cb[0]), "r"(cb[1]), "r"(cb[2]), "r"(cb[3])
template <int DEPTH>
__device__ __forceinline__ void quant_full4(uint32_t (&A)[4], uint32_t &ties, uint32_t keys_lane, const uint32_t (&cu)[4],
                                            const uint32_t (&cx)[4], const uint32_t (&cb)[4]) {
  static_assert(DEPTH >= 2 && DEPTH <= 8, "two to eight levels");
  [[maybe_unused]] uint32_t n[4];
  uint32_t tb;
  if constexpr (DEPTH == 2)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_CROSS0 TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else if constexpr (DEPTH == 3)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_CROSS TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else if constexpr (DEPTH == 4)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_CROSS TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else if constexpr (DEPTH == 5)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else if constexpr (DEPTH == 6)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else if constexpr (DEPTH == 7)
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_BOTTOM "}" TBQ_OPERANDS_FULL);
  else
    asm volatile("{\n" TBQ_DECL TBQ_LOAD TBQ_STEP0 TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_STEP TBQ_CROSS TBQ_BOTTOM "}"
                 TBQ_OPERANDS_FULL);
  ties |= tb;
}
__device__ __forceinline__ void quant_full4_any(uint32_t depth, uint32_t (&A)[4], uint32_t &ties, uint32_t keys_lane,
                                                const uint32_t (&cu)[4], const uint32_t (&cx)[4], const uint32_t (&cb)[4]) {
  switch (depth) {
  case 2: return quant_full4<2>(A, ties, keys_lane, cu, cx, cb);
  case 3: return quant_full4<3>(A, ties, keys_lane, cu, cx, cb);
  case 4: return quant_full4<4>(A, ties, keys_lane, cu, cx, cb);
  case 5: return quant_full4<5>(A, ties, keys_lane, cu, cx, cb);
  case 6: return quant_full4<6>(A, ties, keys_lane, cu, cx, cb);
  case 7: return quant_full4<7>(A, ties, keys_lane, cu, cx, cb);
  default: return quant_full4<8>(A, ties, keys_lane, cu, cx, cb);
  }
}
template <int UD, bool LEAF_IDS, bool MULTI>
__global__ void __launch_bounds__(kQBMaxThreads, 1) tb_walk_quant_batch_kernel(const QuantParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0); // uniform by construction
  const bool leafer = warp >= kQBWalkers && warp < kQBWalkers + kQBLeafWarps;
  const bool producer = warp >= kQBWalkers + kQBLeafWarps;
  const int set = (warp >= kQBWalkers ? warp - kQBWalkers : warp / kQSetWarps) & 1; // (leaf warps 16..19, producers 20, 21)
  const int half = (warp - kQBWalkers) >> 1 & 1; // leaf warps: tiles half, half + 2, ... of the batch
  const int sw = warp % kQSetWarps;
  const int F = p.num_features, R = p.tiles_per_batch;
  const int KT = quant_key_tile_bytes(F);
  const uint32_t bars_s = smem_u32(smem_raw);
  // barriers: full[set][4] @0, empty[set][4] @64, table_full[set][2] @128, table_free[set][2] @160,
  // keys_free @192, keys_ready @200, sum_ready[half] @208, sum_free[half] @224
  const uint32_t full_s = bars_s + (uint32_t)set * 32u, empty_s = bars_s + 64u + (uint32_t)set * 32u;
  const uint32_t table_s = bars_s + 128u + (uint32_t)set * 16u, table_free_s = bars_s + 160u + (uint32_t)set * 16u;
  const uint32_t keys_free_s = bars_s + 192u, keys_ready_s = bars_s + 200u;
  const uint32_t sum_ready_s = bars_s + 208u + (uint32_t)half * 8u, sum_free_s = bars_s + 224u + (uint32_t)half * 8u;
  unsigned char *ring = smem_raw + kQBBarBytes + (size_t)set * kQBSlots * kQPiece;
  const uint32_t ring_s = smem_u32(ring);
  const uint32_t ltab0_s = bars_s + kQBBarBytes + (uint32_t)kQBRingBytes;   // [set][table][tile][column][row] bytes
  const uint32_t ltab_s = ltab0_s + (uint32_t)set * 2u * (uint32_t)R * 1024u;
  const uint32_t sums1_s = ltab0_s + 4u * (uint32_t)R * 1024u;   // [tile][row] floats
  const uint32_t keys_s = sums1_s + (uint32_t)R * 256u;          // [tile] key tiles

  const long long num_tiles = (p.n_rows + 31) / 32;
  const long long num_batches = (num_tiles + R - 1) / R;
  const int my_batches = (int)((num_batches - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const int g0 = blockIdx.y * p.groups_per_chunk;
  const int g1 = min(p.num_groups, g0 + p.groups_per_chunk);
  const int NG = g1 - g0;
  // the set's groups: set, set + 2, ... of the chunk; whole classes of a multiclass forest
  const int NGs = MULTI ? p.set_count[set] : (NG - set + 1) / 2;
  auto group_index = [&](int k) { return MULTI ? p.set_groups[set * p.num_groups + k] : 2 * k + set; };
  const int P = 2 * NGs;              // pieces of this set per batch
  const int NP = (F + 2) / 2;         // feature pairs = lines of a key tile

  if (tid == 0) {
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
    for (int i = 0; i < 8; ++i) mbar_init(bars + i, 1);             // full: the copy's bytes
    for (int i = 8; i < 16; ++i) mbar_init(bars + i, kQSetWarps);   // empty: one arrival per walker warp of the set
    for (int i = 16; i < 20; ++i) mbar_init(bars + i, kQSetWarps);  // table_full: every walker of the set has written
    for (int i = 20; i < 24; ++i) mbar_init(bars + i, 2);           // table_free: both leaf warps of the set have read the table
    mbar_init(bars + 24, kQBWalkers);                               // keys_free: the previous batch is walked
    mbar_init(bars + 25, kQBWalkers);                               // keys_ready: the batch's keys are staged
    for (int i = 26; i < 28; ++i) mbar_init(bars + i, 1);           // sum_ready[half]: set 1's leaf warp has written its sums
    for (int i = 28; i < 30; ++i) mbar_init(bars + i, 1);           // sum_free[half]: set 0's leaf warp has read them
    fence_barrier_init();
  }
  __syncthreads();

  auto group_of = [&](int gi) -> uint2 { // plane offset (in rows of 32 elements) and depth of group gi of the chunk
    if constexpr (UD > 0) return make_uint2((uint32_t)(g0 + gi) << UD, (uint32_t)UD);
    const DevQuantGroup gm = p.groups[g0 + gi];
    return make_uint2((uint32_t)(gm.elem_off >> 5), gm.depth);
  };

  bool ok = true;
  unsigned tie_count = 0;
  const uint64_t keep = l2_policy_keep();
  const uint32_t wait_tries = p.wait_tries ? p.wait_tries : kQWaitTries;
  auto wait = [wait_tries](uint32_t bar_addr, uint32_t parity) { return tb::mbar_wait_all_lanes(bar_addr, parity, wait_tries); };

  if (producer) {
    // ---- the set's ring producer: piece q (upper levels of a group for even q, its bottom
    // level for odd q) goes to slot q mod 4 once every walker of the set has released the slot
    int slot = 0;
    uint32_t round = 0;
    for (int it = 0; it < my_batches && ok; ++it) {
      for (int piece = 0; piece < P && ok; ++piece) {
        if (round > 0) ok = wait(empty_s + 8u * (uint32_t)slot, (round - 1u) & 1u);
        if (ok && lane == 0 && !(p.skip_first_copy && it == 0 && piece == 0)) {
          const uint2 gm = group_of(group_index(piece >> 1));
          const uint32_t hs = 1u << (gm.y - 1); // slots per piece
          const size_t off = ((size_t)gm.x + ((piece & 1) ? hs : 0u)) * 32;
          uint64_t *bar = reinterpret_cast<uint64_t *>(smem_raw) + set * kQBSlots + slot;
          mbar_expect_tx(bar, hs * 128u);
          bulk_g2s_hint(ring + (size_t)slot * kQPiece, p.node_plane + off, hs * 128u, bar, keep);
        }
        if (++slot == kQBSlots) {
          slot = 0;
          ++round;
        }
      }
    }
  } else if (leafer) {
    // ---- leaf warps: for every finished table of the set, gather the leaf values of this
    // warp's tiles of the batch (every other one), add the group's 32 values pairwise and keep
    // one running sum per tile
    uint32_t kk = 0; // groups of the set seen so far (tables alternate, their barriers change phase)
    for (int it = 0; it < my_batches && ok; ++it) {
      const long long batch = blockIdx.x + (long long)it * gridDim.x;
      const long long row0 = batch * R * 32 + lane;
      float sums[kQBMaxTiles / 2];
      [[maybe_unused]] float best[kQBMaxTiles / 2];  // multiclass: the largest class sum so far and its class
      [[maybe_unused]] int best_class[kQBMaxTiles / 2];
      [[maybe_unused]] int cur_class = -1;
#pragma unroll
      for (int q = 0; q < kQBMaxTiles / 2; ++q) {
        sums[q] = 0.f;
        if constexpr (MULTI) {
          best[q] = -INFINITY;
          best_class[q] = 0;
        }
      }
      // the class whose sum has been running is complete: it is written out where per-class
      // partial sums are wanted ([rows][classes]; every class belongs to one set, so every
      // element is written once), and it wins against a smaller or equal best
      auto fold = [&]() {
#pragma unroll
        for (int q = 0; q < kQBMaxTiles / 2; ++q) {
          const int r = 2 * q + half;
          if (p.write_partial) {
            const long long row = row0 + r * 32;
            if (r < R && row < p.n_rows) p.partial[row * p.num_classes + cur_class] = sums[q];
          }
          if (sums[q] >= best[q]) {
            best[q] = sums[q];
            best_class[q] = cur_class;
          }
          sums[q] = 0.f;
        }
      };
      for (int k = 0; k < NGs && ok; ++k, ++kk) {
        const int gi = group_index(k);
        const uint2 gm = group_of(gi);
        if constexpr (MULTI && !LEAF_IDS) {
          const int cls = p.group_class[g0 + gi];
          if (cls != cur_class) {
            if (cur_class >= 0) fold();
            cur_class = cls;
          }
        }
        const uint32_t slots = 2u << (gm.y - 1);
        ok = wait(table_s + 8u * (kk & 1u), (kk >> 1) & 1u);
        if (!ok) break;
        const uint32_t tab0 = ltab_s + (kk & 1u) * (uint32_t)R * 1024u + (uint32_t)lane;
        // (element offsets fit 32 bits: the host refuses planes of 2^32 elements or more)
#pragma unroll
        for (int q = 0; q < kQBMaxTiles / 2; ++q) {
          const int r = 2 * q + half;
          if (r < R) {
            const uint32_t tab = tab0 + (uint32_t)r * 1024u;
            uint32_t e[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              uint32_t leaf;
              asm volatile("ld.shared.u8 %0, [%1];" : "=r"(leaf) : "r"(tab + (uint32_t)c * 32u) : "memory");
              e[c] = gm.x * 32u + (uint32_t)c * slots + leaf;
            }
            if constexpr (LEAF_IDS) {
              const long long row = row0 + r * 32;
              if (row < p.n_rows) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                  const int t = p.tree_index[(g0 + gi) * 32 + c];
                  if (t >= 0) p.leaf_ids[row * p.num_trees + t] = p.orig_leaf[e[c]];
                }
              }
            } else {
              float v[32];
#pragma unroll
              for (int c = 0; c < 32; ++c) v[c] = ldg_f32_hint(p.leaf_plane + e[c], keep);
#pragma unroll
              for (int w = 16; w >= 1; w >>= 1)
#pragma unroll
                for (int c = 0; c < w; ++c) v[c] += v[c + w];
              sums[q] += v[0];
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(table_free_s + 8u * (kk & 1u)); // every tile's table has been read
      }
      if (!ok) break;
      if constexpr (MULTI && !LEAF_IDS) {
        if (cur_class >= 0) fold();
        if (p.write_partial) continue; // the per-class sums are the result
        // the batch's results: leaf warp 1 hands its best class to leaf warp 0
        if (set == 1) {
          if (it > 0) ok = wait(sum_free_s, (uint32_t)(it - 1) & 1u);
          if (!ok) break;
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q)
            if (const int r = 2 * q + half; r < R) {
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(sums1_s + (uint32_t)(r * 64 + lane) * 4u), "f"(best[q]) : "memory");
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(sums1_s + (uint32_t)(r * 64 + 32 + lane) * 4u), "r"(best_class[q]) : "memory");
            }
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_ready_s);
        } else {
          ok = wait(sum_ready_s, (uint32_t)it & 1u);
          if (!ok) break;
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q)
            if (const int r = 2 * q + half; r < R) {
              const float b1 = lds_f32(sums1_s + (uint32_t)(r * 64 + lane) * 4u);
              const int c1 = (int)lds_u32(sums1_s + (uint32_t)(r * 64 + 32 + lane) * 4u);
              if (b1 > best[q] || (b1 == best[q] && c1 > best_class[q])) best_class[q] = c1;
            }
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_free_s);
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q) {
            const int r = 2 * q + half;
            const long long row = row0 + r * 32;
            if (r < R && row < p.n_rows) {
              if (p.out_kind == 1)
                reinterpret_cast<int8_t *>(p.out)[row] = (int8_t)best_class[q];
              else
                reinterpret_cast<float *>(p.out)[row] = (float)best_class[q];
            }
          }
        }
      } else if constexpr (!LEAF_IDS) {
        // the batch's results: leaf warp 1 hands its sums to leaf warp 0
        if (set == 1) {
          if (it > 0) ok = wait(sum_free_s, (uint32_t)(it - 1) & 1u);
          if (!ok) break;
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q)
            if (const int r = 2 * q + half; r < R)
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(sums1_s + (uint32_t)(r * 32 + lane) * 4u), "f"(sums[q]) : "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_ready_s);
        } else {
          ok = wait(sum_ready_s, (uint32_t)it & 1u);
          if (!ok) break;
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q)
            if (const int r = 2 * q + half; r < R) sums[q] += lds_f32(sums1_s + (uint32_t)(r * 32 + lane) * 4u);
          __syncwarp();
          if (lane == 0) mbar_arrive(sum_free_s);
#pragma unroll
          for (int q = 0; q < kQBMaxTiles / 2; ++q) {
            const int r = 2 * q + half;
            const long long row = row0 + r * 32;
            if (r < R && row < p.n_rows) {
              if (p.write_partial)
                p.partial[(long long)blockIdx.y * p.n_rows + row] = sums[q];
              else
                reinterpret_cast<float *>(p.out)[row] = apply_transform(p.initial_value + sums[q], p.transform);
            }
          }
        }
      }
    }
  } else {
    // ---- the walkers
    uint32_t col[4], colb[4], drop0[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      col[c] = (uint32_t)(lane + sw + 8 * c) & 31u;
      colb[c] = ring_s + col[c] * 4u;                     // the column's address in slot 0
      drop0[c] = ltab_s + col[c] * 32u + (uint32_t)lane;  // where its leaf number goes (table 0, tile 0)
    }
    int slot = 0;
    uint32_t parity = 0, kk = 0; // kk: groups this warp has walked so far
    const bool elected = lane == 0;
    for (int it = 0; it < my_batches && ok; ++it) {
      const long long batch = blockIdx.x + (long long)it * gridDim.x;
      const long long row0 = batch * R * 32;
      // ---- stage the batch: warp = tile, lane = row; first every walker must be done with
      // the previous batch's keys
      if (it > 0) {
        __syncwarp();
        if (elected) mbar_arrive(keys_free_s);
        ok = wait(keys_free_s, (uint32_t)(it - 1) & 1u);
        if (!ok) break;
      }
      if (warp < R) {
        const long long row = row0 + warp * 32 + lane;
        const bool live = row < p.n_rows;
        const float *src = p.rows + (live ? row : 0) * p.ld;
        const uint32_t dst = keys_s + (uint32_t)warp * (uint32_t)KT + (uint32_t)lane * 4u;
        for (int m = 0; m < NP; ++m) {
          uint32_t k2[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int f = 2 * m + h;
            k2[h] = f < F ? quant_key15_lattice_dev(live ? __ldg(src + f) : 0.f, __ldg(p.lo + f), __ldg(p.scale + f)) : 0x7bffu;
          }
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + (uint32_t)m * 128u), "r"(k2[0] | (k2[1] << 16)) : "memory");
        }
      }
      __syncwarp();
      if (elected) mbar_arrive(keys_ready_s);
      ok = wait(keys_ready_s, (uint32_t)it & 1u);
      if (!ok) break;

      for (int k = 0; k < NGs && ok; ++k, ++kk) {
        const int gi = group_index(k);
        const uint2 gm = group_of(gi);
        const uint32_t depth = UD ? (uint32_t)UD : gm.y, hs = 1u << (depth - 1);
        // the two pieces of this group
        const uint32_t su = (uint32_t)slot, pu = parity;
        if (++slot == kQBSlots) { slot = 0; parity ^= 1u; }
        const uint32_t sb = (uint32_t)slot, pb = parity;
        if (++slot == kQBSlots) { slot = 0; parity ^= 1u; }
        uint32_t root[4], bot[4], cu[4], cx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          root[c] = colb[c] + su * kQPiece;
          bot[c] = colb[c] + sb * kQPiece;
          cu[c] = 128u - root[c];
          cx[c] = cu[c] + bot[c] - root[c] - 128u * (hs - 1u);
        }
        ok = wait(full_s + 8u * su, pu);
        if (!ok) break;
        ok = wait(full_s + 8u * sb, pb);
        if (!ok) break;
        // the leaf numbers go into table kk mod 2, once the leaf warp has read what group kk - 2 left there
        if (kk >= 2) {
          ok = wait(table_free_s + 8u * (kk & 1u), ((kk >> 1) - 1u) & 1u);
          if (!ok) break;
        }
        uint32_t keys_lane = keys_s + (uint32_t)lane * 4u, drop[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) drop[c] = drop0[c] + (kk & 1u) * (uint32_t)R * 1024u;
#pragma unroll 1
        for (int r = 0; r < R; ++r) {
          uint32_t A[4], ties = 0;
          if (depth >= 2) {
#pragma unroll
            for (int c = 0; c < 4; ++c) A[c] = root[c];
            if constexpr (UD >= 2)
              quant_full4<UD>(A, ties, keys_lane, cu, cx, bot);
            else
              quant_full4_any(depth, A, ties, keys_lane, cu, cx, bot);
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) A[c] = bot[c];
            quant_bottom4(A, ties, keys_lane, bot);
          }
          if (ties) { // rare: a tied column is walked again, exact values deciding the tied comparisons
            const long long row = row0 + r * 32 + lane;
            const float *rowp = p.rows + (row < p.n_rows ? row : 0) * p.ld;
#pragma unroll
            for (int c = 0; c < 4; ++c)
              if (ties & (1u << c)) {
                const uint32_t j = depth >= 2 ? quant_upper_exact(root[c], keys_lane, p.exact_plane, gm.x, depth, col[c], rowp) : 0u;
                A[c] = quant_bottom_exact(bot[c], j, keys_lane, p.exact_plane, gm.x, depth, col[c], rowp);
                ++tie_count;
              }
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) asm volatile("st.shared.u8 [%0], %1;" ::"r"(drop[c]), "r"(A[c]) : "memory");
          keys_lane += (uint32_t)KT;
#pragma unroll
          for (int c = 0; c < 4; ++c) drop[c] += 1024u;
        }
        __syncwarp();
        if (elected) {
          mbar_arrive(empty_s + 8u * su);
          mbar_arrive(empty_s + 8u * sb);
          mbar_arrive(table_s + 8u * (kk & 1u));
        }
      }
    }
  }
  // every wait above is bounded: a wait that gave up ends the launch with a status word
  const bool failed = __syncthreads_or(!ok) != 0;
  if (failed) {
    if (tid == 0) atomicExch(p.status, 4);
    return;
  }
  if (p.tie_count != nullptr && tie_count) atomicAdd(p.tie_count, (unsigned long long)tie_count);
}

} // namespace tb
