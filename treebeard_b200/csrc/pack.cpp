// Forest -> packed node tiles.  See pack.h for the layout and the reference files
// whose ground this covers.
#include "pack.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <limits>
#include <map>
#include <numeric>
#include <queue>
#include <cstdlib>
#include <thread>

namespace tb {

std::string validate(const Forest &f) {
  const int64_t T = f.num_trees();
  if (T < 0 || f.tree_off.empty() || f.tree_off[0] != 0) return "tree_off must start at 0";
  const int64_t N = f.num_nodes();
  if ((int64_t)f.left.size() != N || (int64_t)f.right.size() != N ||
      (int64_t)f.feat.size() != N || (int64_t)f.thr.size() != N)
    return "node arrays do not match tree_off";
  if (f.num_features <= 0) return "num_features must be positive";
  if (f.num_classes < 0) return "num_classes must be >= 0";
  if (f.num_classes > 0 && (int64_t)f.class_id.size() != T) return "class_id must have one entry per tree";
  for (int64_t t = 0; t < T; ++t) {
    const int64_t a = f.tree_off[t], n = f.tree_off[t + 1] - a;
    if (n <= 0) return "tree " + std::to_string(t) + " has no nodes";
    if (f.num_classes > 0 && (f.class_id[t] < 0 || f.class_id[t] >= f.num_classes))
      return "class id out of range in tree " + std::to_string(t);
    std::vector<int32_t> parents(n, 0);
    for (int64_t i = 0; i < n; ++i) {
      const int32_t l = f.left[a + i], r = f.right[a + i];
      if ((l < 0) != (r < 0)) return "node with a single child in tree " + std::to_string(t);
      if (l < 0) continue;
      if (l >= n || r >= n || l == 0 || r == 0 || l == r)
        return "child index out of range in tree " + std::to_string(t);
      if (f.feat[a + i] < 0 || f.feat[a + i] >= f.num_features)
        return "feature index out of range in tree " + std::to_string(t);
      ++parents[l];
      ++parents[r];
    }
    for (int64_t i = 1; i < n; ++i)
      if (parents[i] > 1) return "node with two parents in tree " + std::to_string(t);
    // reachability from the root without revisits rules out cycles
    int64_t seen = 0;
    std::vector<int32_t> stack{0};
    while (!stack.empty()) {
      int32_t i = stack.back();
      stack.pop_back();
      if (++seen > n) return "cycle in tree " + std::to_string(t);
      if (f.left[a + i] >= 0) {
        stack.push_back(f.left[a + i]);
        stack.push_back(f.right[a + i]);
      }
    }
  }
  return "";
}

int pack_threads() {
  if (const char *env = std::getenv("TBK_PACK_THREADS")) {
    const int n = std::atoi(env);
    if (n > 0) return n;
  }
  const unsigned hw = std::thread::hardware_concurrency();
  return (int)std::min(32u, std::max(1u, hw));
}

int32_t tree_depth(const Forest &f, int64_t t) {
  const int64_t a = f.tree_off[t];
  int32_t best = 0;
  std::vector<std::pair<int32_t, int32_t>> stack{{0, 0}};
  while (!stack.empty()) {
    auto [i, d] = stack.back();
    stack.pop_back();
    if (f.left[a + i] < 0) {
      best = std::max(best, d);
    } else {
      stack.push_back({f.left[a + i], d + 1});
      stack.push_back({f.right[a + i], d + 1});
    }
  }
  return best;
}

// ---------------------------------------------------------------------------
// tile shapes and the look-up table

namespace {

// A shape is the in-tile structure of up to ts nodes listed in level order; for node
// i, bit 2i says "left child is in the tile", bit 2i+1 the same for the right child.
struct ShapeTable {
  int ts = 1;
  std::map<uint32_t, int> id_of; // key = code | (nodes << 24)
  std::vector<int8_t> lut;       // [(num_shapes) << ts]
  int num_shapes = 0;
};

uint32_t shape_key(uint32_t code, int nodes) { return code | ((uint32_t)nodes << 24); }

void enumerate_shapes(int nodes_left, std::vector<std::pair<int, int>> &links, size_t cursor,
                      std::vector<uint32_t> &out) {
  // links[i] = (left in tile, right in tile) for the nodes created so far, in level
  // order; cursor = next node whose children are to be decided.
  if (cursor == links.size()) {
    {
      uint32_t code = 0;
      for (size_t i = 0; i < links.size(); ++i)
        code |= (uint32_t)(links[i].first | (links[i].second << 1)) << (2 * i);
      out.push_back(shape_key(code, (int)links.size()));
    }
    return;
  }
  for (int l = 0; l <= 1; ++l)
    for (int r = 0; r <= 1; ++r) {
      if (l + r > nodes_left) continue;
      links[cursor] = {l, r};
      for (int k = 0; k < l + r; ++k) links.push_back({0, 0});
      enumerate_shapes(nodes_left - l - r, links, cursor + 1, out);
      for (int k = 0; k < l + r; ++k) links.pop_back();
    }
  links[cursor] = {0, 0};
}

ShapeTable build_shape_table(int ts) {
  ShapeTable st;
  st.ts = ts;
  std::vector<uint32_t> keys;
  for (int m = 1; m <= ts; ++m) {
    std::vector<std::pair<int, int>> links{{0, 0}};
    std::vector<uint32_t> all;
    enumerate_shapes(m - 1, links, 0, all);
    for (uint32_t k : all)
      if ((int)(k >> 24) == m) keys.push_back(k);
  }
  std::sort(keys.begin(), keys.end());
  keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
  // shape 0 is the leaf tile: every outcome stays on child 0
  st.num_shapes = (int)keys.size() + 1;
  st.lut.assign((size_t)st.num_shapes << ts, 0);
  for (size_t s = 0; s < keys.size(); ++s) {
    const int id = (int)s + 1;
    st.id_of[keys[s]] = id;
    const int m = (int)(keys[s] >> 24);
    const uint32_t code = keys[s] & 0xFFFFFF;
    // level-order index of the in-tile children of each node
    std::vector<int> lc(m, -1), rc(m, -1);
    int next = 1;
    for (int i = 0; i < m; ++i) {
      if (code >> (2 * i) & 1) lc[i] = next++;
      if (code >> (2 * i + 1) & 1) rc[i] = next++;
    }
    // exits numbered left to right
    std::vector<int> lexit(m, -1), rexit(m, -1);
    int exits = 0;
    std::function<void(int)> number = [&](int i) {
      if (lc[i] >= 0) number(lc[i]); else lexit[i] = exits++;
      if (rc[i] >= 0) number(rc[i]); else rexit[i] = exits++;
    };
    number(0);
    for (uint32_t bits = 0; bits < (1u << ts); ++bits) {
      int i = 0, out = -1;
      while (out < 0) {
        const bool go_left = bits >> i & 1; // bit set: x < threshold
        if (go_left) { if (lc[i] >= 0) i = lc[i]; else out = lexit[i]; }
        else         { if (rc[i] >= 0) i = rc[i]; else out = rexit[i]; }
      }
      st.lut[((size_t)id << ts) + bits] = (int8_t)out;
    }
  }
  return st;
}

// One tile of one tree: up to ts internal nodes in level order, or a single leaf.
struct Tile {
  int n = 0;                 // internal nodes in the tile (0 = leaf tile)
  int32_t nodes[kMaxTileSize] = {-1, -1, -1, -1};
  int32_t leaf = -1;         // original node id when n == 0
  int shape = 0;
  int num_exits = 0;
  int32_t exits[kMaxTileSize + 1] = {};       // original node ids, left to right
  int32_t child_tiles[kMaxTileSize + 1] = {}; // tile ids of the exits
};

struct TiledTree {
  std::vector<Tile> tiles; // tiles[0] holds the root
  int depth = 0;           // internal-tile levels on the longest path
};

// Uniform tiling: walk the tree in pre-order; every node not yet in a tile starts
// one, which grabs up to ts internal nodes in level order below it.
void tile_tree(const Forest &f, int64_t t, int ts, const ShapeTable &st, TiledTree *out) {
  const int64_t a = f.tree_off[t];
  TiledTree &tt = *out;
  tt.tiles.clear();
  tt.tiles.reserve((size_t)(f.tree_off[t + 1] - a));
  const int shape1 = ts == 1 ? st.id_of.at(shape_key(0, 1)) : 0;
  std::function<int(int32_t, int)> build = [&](int32_t root, int level) -> int {
    const int id = (int)tt.tiles.size();
    tt.tiles.emplace_back();
    if (f.left[a + root] < 0) {
      tt.tiles[id].leaf = root;
      return id;
    }
    tt.depth = std::max(tt.depth, level + 1);
    Tile tile;
    if (ts == 1) {
      tile.n = 1;
      tile.nodes[0] = root;
      tile.shape = shape1;
      tile.num_exits = 2;
      tile.exits[0] = f.left[a + root];
      tile.exits[1] = f.right[a + root];
    } else {
      int32_t q[2 * kMaxTileSize + 2];
      int head = 0, tail = 0;
      q[tail++] = root;
      while (head < tail && tile.n < ts) {
        const int32_t v = q[head++];
        tile.nodes[tile.n++] = v;
        const int32_t l = f.left[a + v], r = f.right[a + v];
        if (f.left[a + l] >= 0) q[tail++] = l;
        if (f.left[a + r] >= 0) q[tail++] = r;
      }
      auto pos = [&](int32_t v) {
        for (int i = 0; i < tile.n; ++i)
          if (tile.nodes[i] == v) return i;
        return -1;
      };
      uint32_t code = 0;
      for (int i = 0; i < tile.n; ++i) {
        if (pos(f.left[a + tile.nodes[i]]) >= 0) code |= 1u << (2 * i);
        if (pos(f.right[a + tile.nodes[i]]) >= 0) code |= 1u << (2 * i + 1);
      }
      tile.shape = st.id_of.at(shape_key(code, tile.n));
      std::function<void(int32_t)> collect = [&](int32_t v) {
        const int32_t l = f.left[a + v], r = f.right[a + v];
        if (pos(l) >= 0) collect(l); else tile.exits[tile.num_exits++] = l;
        if (pos(r) >= 0) collect(r); else tile.exits[tile.num_exits++] = r;
      };
      collect(root);
    }
    for (int k = 0; k < tile.num_exits; ++k) tile.child_tiles[k] = -1;
    tt.tiles[id] = tile;
    for (int k = 0; k < tile.num_exits; ++k) {
      const int c = build(tile.exits[k], level + 1);
      tt.tiles[id].child_tiles[k] = c;
    }
    return id;
  };
  tt.depth = 0;
  build(0, 0);
}

struct TileWriter {
  int ts, tile_bytes;
  uint16_t sentinel;
  void write(uint8_t *dst, const Forest &f, int64_t a, const Tile &tile, float leaf_value,
             uint16_t child) const {
    float thr[kMaxTileSize];
    uint16_t feat[kMaxTileSize];
    for (int i = 0; i < ts; ++i) {
      if (i < tile.n) {
        thr[i] = f.thr[a + tile.nodes[i]];
        feat[i] = (uint16_t)f.feat[a + tile.nodes[i]];
      } else {
        thr[i] = tile.n == 0 ? leaf_value : std::numeric_limits<float>::infinity();
        feat[i] = sentinel;
      }
    }
    std::memcpy(dst, thr, 4 * ts);
    std::memcpy(dst + 4 * ts, feat, 2 * ts);
    if (ts == 1) {
      std::memcpy(dst + 6, &child, 2);
    } else {
      const uint16_t shape = (uint16_t)tile.shape;
      std::memcpy(dst + 6 * ts, &shape, 2);
      std::memcpy(dst + 6 * ts + 2, &child, 2);
    }
  }
};

} // namespace

std::string pack_forest(const Forest &f, const PackOptions &opt, PackedForest *out) {
  std::string err = validate(f);
  if (!err.empty()) return err;
  const int ts = opt.tile_size <= 0 ? 1 : opt.tile_size;
  if (ts > kMaxTileSize) return "tile size above " + std::to_string(kMaxTileSize) + " is not supported";
  if (opt.representation == kReorg && ts != 1) return "the reorg representation is scalar (tile size 1) only";
  if (opt.representation < kSparse || opt.representation > kReorg) return "unknown representation";
  if (f.num_features > 65534) return "more than 65534 features";
  for (float v : f.thr)
    if (std::isnan(v)) return "NaN threshold or leaf value";
  for (int64_t g = 0; g < f.num_nodes(); ++g)
    if (f.is_leaf(g) && f.thr[g] == -std::numeric_limits<float>::infinity())
      return "-inf leaf value";

  PackedForest &p = *out;
  p = PackedForest();
  p.representation = opt.representation;
  p.tile_size = ts;
  p.tile_bytes = opt.representation == kReorg ? 6 : (ts == 1 ? 8 : ts == 2 ? 16 : ts == 3 ? 24 : 32);
  p.num_features = f.num_features;
  p.num_classes = f.num_classes;
  p.transform = f.transform;
  p.initial_value = f.initial_value;
  p.num_trees = f.num_trees();
  p.num_nodes = f.num_nodes();

  ShapeTable st = build_shape_table(ts);
  p.lut = st.lut;
  p.num_shapes = st.num_shapes;

  const int64_t T = f.num_trees();
  std::vector<int32_t> tdepth(T);   // tile levels of each tree
  std::vector<int64_t> tcount(T);   // tiles of each tree
  int32_t max_depth = 0;
#pragma omp parallel for schedule(dynamic, 16) reduction(max : max_depth) num_threads(pack_threads())
  for (int64_t t = 0; t < T; ++t) {
    if (ts == 1) {
      tdepth[t] = tree_depth(f, t);
      tcount[t] = f.tree_off[t + 1] - f.tree_off[t];
      max_depth = std::max(max_depth, tdepth[t]);
    } else {
      TiledTree tt;
      tile_tree(f, t, ts, st, &tt);
      tdepth[t] = tt.depth;
      tcount[t] = (int64_t)tt.tiles.size();
      max_depth = std::max(max_depth, tree_depth(f, t));
    }
  }
  p.max_depth = max_depth;
  // trees of similar shape share a group: order by (tile depth, tile count)
  std::vector<int64_t> order(T);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int64_t x, int64_t y) {
    if (tdepth[x] != tdepth[y]) return tdepth[x] < tdepth[y];
    return tcount[x] < tcount[y];
  });

  // columns of the groups: tree index or -1 (filler).  A multiclass forest is laid out
  // class by class, every class padded to whole groups, so that a group belongs to ONE
  // class and the classes appear in increasing order: the kernel can then keep a class
  // sum in a register and decide the arg-max on the fly.
  std::vector<int64_t> cols;
  std::vector<int16_t> col_class; // class of every column, fillers included
  if (f.num_classes > 0) {
    std::vector<std::vector<int64_t>> by_class(f.num_classes);
    for (int64_t k = 0; k < T; ++k) by_class[f.class_id[order[k]]].push_back(order[k]);
    for (int32_t cls = 0; cls < f.num_classes; ++cls) {
      const auto &list = by_class[cls];
      cols.insert(cols.end(), list.begin(), list.end());
      if (list.empty()) cols.push_back(-1); // a class without trees still gets a (filler) group
      while (cols.size() % kGroupTrees) cols.push_back(-1);
      col_class.resize(cols.size(), (int16_t)cls);
    }
  } else {
    cols.assign(order.begin(), order.end());
    while (cols.size() % kGroupTrees) cols.push_back(-1);
  }
  const int64_t G = (int64_t)cols.size() / kGroupTrees;
  p.groups.resize(G);
  p.tree_class.assign(G * kGroupTrees, 0);
  if (f.num_classes > 0) p.tree_class = col_class;
  p.tree_index.assign(G * kGroupTrees, -1);
  p.orig_off.resize(G);
  const bool implicit = opt.representation != kSparse;
  const TileWriter writer{ts, p.tile_bytes, (uint16_t)f.num_features};

  uint64_t blob_bytes = 0, orig_elems = 0;
  for (int64_t g = 0; g < G; ++g) {
    uint32_t gdepth = 0;
    uint64_t slots = 1;
    for (int c = 0; c < kGroupTrees; ++c) {
      const int64_t t = cols[g * kGroupTrees + c];
      if (t < 0) continue;
      gdepth = std::max<uint32_t>(gdepth, tdepth[t]);
      if (!implicit) slots = std::max<uint64_t>(slots, tcount[t]);
    }
    if (implicit) {
      // complete (ts+1)-ary array down to level gdepth
      slots = 0;
      uint64_t level = 1;
      for (uint32_t l = 0; l <= gdepth; ++l) {
        slots += level;
        level *= (uint64_t)(ts + 1);
        if (slots > (1ull << 26)) return "array layout of this forest is too large (deep unbalanced trees); use the sparse representation";
      }
    } else if (slots > 65536) {
      return "a tree has more than 65536 tiles";
    }
    p.groups[g] = GroupMeta{blob_bytes, (uint32_t)slots, gdepth};
    p.orig_off[g] = orig_elems;
    uint64_t gbytes = slots * kGroupTrees * (uint64_t)p.tile_bytes;
    gbytes = (gbytes + 15) & ~15ull;
    p.max_group_bytes = std::max(p.max_group_bytes, gbytes);
    blob_bytes += gbytes;
    orig_elems += slots * kGroupTrees;
    if (blob_bytes > (48ull << 30)) return "packed forest exceeds 48 GiB";
  }
  p.blob.assign(blob_bytes, 0);
  p.orig_node.assign(orig_elems, -1);

#pragma omp parallel for schedule(dynamic, 4) num_threads(pack_threads())
  for (int64_t g = 0; g < G; ++g) {
    const GroupMeta &gm = p.groups[g];
    TiledTree tt;
    uint8_t *base = p.blob.data() + gm.byte_off;
    int32_t *orig = p.orig_node.data() + p.orig_off[g];
    const uint64_t S = gm.slots;
    // reorg planes
    float *thr_plane = reinterpret_cast<float *>(base);
    uint16_t *feat_plane = reinterpret_cast<uint16_t *>(base + S * kGroupTrees * 4);
    auto put = [&](uint64_t slot, int c, const Tile &tile, int64_t a, float leaf_value,
                   uint16_t child, int32_t orig_id) {
      if (opt.representation == kReorg) {
        thr_plane[slot * kGroupTrees + c] = tile.n ? f.thr[a + tile.nodes[0]] : leaf_value;
        feat_plane[slot * kGroupTrees + c] = tile.n ? (uint16_t)f.feat[a + tile.nodes[0]] : writer.sentinel;
      } else {
        writer.write(base + (slot * kGroupTrees + c) * (uint64_t)p.tile_bytes, f, a, tile, leaf_value, child);
      }
      orig[slot * kGroupTrees + c] = orig_id;
    };
    const Tile filler; // leaf tile with value 0
    for (int c = 0; c < kGroupTrees; ++c) {
      const int64_t k = g * kGroupTrees + c;
      const int64_t t = cols[k];
      const bool real = t >= 0;
      const int64_t a = real ? f.tree_off[t] : 0;
      if (real) {
        p.tree_index[k] = (int32_t)t;
      }
      if (!implicit) {
        // level-order numbering of tiles, children of a tile adjacent
        for (uint64_t s = 0; s < S; ++s) put(s, c, filler, 0, 0.f, (uint16_t)s, -1);
        if (!real) continue;
        tile_tree(f, t, ts, st, &tt);
        std::vector<int> slot_of(tt.tiles.size(), -1), bfs;
        bfs.push_back(0);
        slot_of[0] = 0;
        int next = 1;
        for (size_t h = 0; h < bfs.size(); ++h) {
          const Tile &tile = tt.tiles[bfs[h]];
          for (int e = 0; e < tile.num_exits; ++e) { slot_of[tile.child_tiles[e]] = next++; bfs.push_back(tile.child_tiles[e]); }
        }
        for (size_t h = 0; h < bfs.size(); ++h) {
          const Tile &tile = tt.tiles[bfs[h]];
          const int s = slot_of[bfs[h]];
          if (tile.n == 0)
            put(s, c, tile, a, f.thr[a + tile.leaf], (uint16_t)s, tile.leaf);
          else
            put(s, c, tile, a, 0.f, (uint16_t)slot_of[tile.child_tiles[0]], -1);
        }
      } else {
        for (uint64_t s = 0; s < S; ++s) put(s, c, filler, 0, 0.f, 0, -1);
        if (!real) continue;
        tile_tree(f, t, ts, st, &tt);
        std::function<void(int, uint64_t, uint32_t)> place = [&](int id, uint64_t slot, uint32_t level) {
          const Tile &tile = tt.tiles[id];
          if (tile.n == 0) {
            // the leaf and its chain of copies down the first-child spine
            uint64_t s = slot;
            for (uint32_t l = level;; ++l) {
              put(s, c, tile, a, f.thr[a + tile.leaf], 0, tile.leaf);
              if (l == gm.depth) break;
              s = s * (uint64_t)(ts + 1) + 1;
            }
            return;
          }
          put(slot, c, tile, a, 0.f, 0, -1);
          for (int k2 = 0; k2 < tile.num_exits; ++k2)
            place(tile.child_tiles[k2], slot * (uint64_t)(ts + 1) + 1 + k2, level + 1);
        };
        place(0, 0, 0);
      }
    }
  }
  return "";
}

// ---------------------------------------------------------------------------

void walk_packed_on_host(const PackedForest &p, const float *rows, int64_t n_rows, int64_t ld,
                         int32_t *leaf_ids, float *sums) {
  const int ts = p.tile_size;
  const int W = std::max(1, p.num_classes);
  const float ninf = -std::numeric_limits<float>::infinity();
  for (int64_t r = 0; r < n_rows; ++r) {
    const float *row = rows + r * ld;
    if (sums) for (int c = 0; c < W; ++c) sums[r * W + c] = 0.f;
    for (size_t g = 0; g < p.groups.size(); ++g) {
      const GroupMeta &gm = p.groups[g];
      const uint8_t *base = p.blob.data() + gm.byte_off;
      const uint64_t S = gm.slots;
      for (int c = 0; c < kGroupTrees; ++c) {
        const int64_t k = (int64_t)g * kGroupTrees + c;
        if (p.tree_index[k] < 0) continue;
        uint64_t n = 0;
        float value = 0.f;
        for (uint32_t step = 0; step <= gm.depth; ++step) {
          float thr[kMaxTileSize];
          uint16_t feat[kMaxTileSize], shape = 0, child = 0;
          if (p.representation == kReorg) {
            thr[0] = reinterpret_cast<const float *>(base)[n * kGroupTrees + c];
            feat[0] = reinterpret_cast<const uint16_t *>(base + S * kGroupTrees * 4)[n * kGroupTrees + c];
          } else {
            const uint8_t *tile = base + (n * kGroupTrees + c) * (uint64_t)p.tile_bytes;
            std::memcpy(thr, tile, 4 * ts);
            std::memcpy(feat, tile + 4 * ts, 2 * ts);
            if (ts == 1) std::memcpy(&child, tile + 6, 2);
            else { std::memcpy(&shape, tile + 6 * ts, 2); std::memcpy(&child, tile + 6 * ts + 2, 2); }
          }
          value = thr[0];
          if (step == gm.depth) break;
          uint32_t bits = 0;
          for (int i = 0; i < ts; ++i) {
            const float x = feat[i] == p.num_features ? ninf : row[feat[i]];
            bits |= (uint32_t)(x < thr[i]) << i;
          }
          const int kk = ts == 1 ? !(bits & 1) : p.lut[((size_t)shape << ts) + bits];
          n = p.representation == kSparse ? (uint64_t)child + kk : n * (uint64_t)(ts + 1) + 1 + kk;
        }
        if (leaf_ids) leaf_ids[r * p.num_trees + p.tree_index[k]] = p.orig_node[p.orig_off[g] + n * kGroupTrees + c];
        if (sums) sums[r * W + (p.num_classes > 0 ? p.tree_class[k] : 0)] += value;
      }
    }
  }
}

} // namespace tb
