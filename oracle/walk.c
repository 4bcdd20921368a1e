/*
 * TEST INFRASTRUCTURE -- CPU oracle for tree-ensemble inference.
 *
 * This file is a plain-C restatement of the reference's ground-truth walker
 * and of its parallel CPU schedule.  It is the checker for the CUDA kernels and
 * the timed CPU baseline; it is never linked into, imported by or called from
 * the product library.
 *
 * Parity status: PINNED.  tbo_predict() is checked (a) against the reference's
 * own golden CSV predictions for the higgs, airline, year_prediction_msd and
 * Random_{1,2,4}Tree models and (b) against the reference's unmodified
 * DecisionForest.h compiled into oracle/_ref (see ref_shim.cpp).
 *
 * Reference lines followed (paths inside the reference project):
 *   walk            src/include/DecisionForest.h:366-379  (PredictTree_Float:
 *                   "x[f] < (float)threshold -> left, else right"; NaN -> right)
 *   reduce          src/include/DecisionForest.h:504-536  (Predict_Float: leaf
 *                   values grouped by class id, std::accumulate seeded with the
 *                   double initial value => double accumulator, float addends)
 *   sigmoid         src/include/DecisionForest.h:442-444
 *   argmax          src/include/DecisionForest.h:446-468  (std::max_element:
 *                   first maximum wins) and, as tie rule 1, the generated code's
 *                   loop src/reduction/LowerReduceOps.cpp:148-189 (last maximum
 *                   wins: "if (max > v) keep else take")
 *   CPU schedule    src/mlir/ReorderTiledTreesByDepth.cpp:387-399 (batch split
 *                   into one contiguous row block per core, blocks in parallel),
 *                   src/schedule/schedule.cpp:464-469 (one tree at a time: tree
 *                   loop outside the row loop), sparse node layout
 *                   src/include/DecisionForest.h:595-629, fp32 accumulation
 *                   src/mlir/LowerToMidLevelIR.cpp:596-614, 698-708.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Flat forest: tree t owns nodes [tree_off[t], tree_off[t+1]).  left/right are
 * node indices relative to the tree (-1/-1 marks a leaf); for a leaf, thr holds
 * the leaf value; feat is ignored for leaves. */
typedef struct {
  int64_t num_trees;
  const int64_t *tree_off;
  const int32_t *left;
  const int32_t *right;
  const int32_t *feat;
  const float *thr;
  const int32_t *class_id; /* per tree */
  int32_t num_classes;     /* 0 => single output */
  int32_t transform;       /* 0 identity, 1 sigmoid, 2 softmax (argmax of sums) */
  double initial_value;
  int32_t num_features;
} tbo_forest;

static inline int32_t walk_one(const tbo_forest *f, int64_t t, const float *row) {
  const int64_t base = f->tree_off[t];
  int32_t n = 0;
  while (f->left[base + n] != -1 || f->right[base + n] != -1) {
    if (row[f->feat[base + n]] < f->thr[base + n])
      n = f->left[base + n];
    else
      n = f->right[base + n];
  }
  return n;
}

/* Ground truth.  out: n_rows floats (prediction, or class index as a float for a
 * multiclass forest).  leaf_ids (optional): n_rows x num_trees int32, the node
 * index of the selected leaf in the tree's own numbering.  class_sums
 * (optional): n_rows x num_classes floats.  tie_rule 0 = first max, 1 = last max. */
int tbo_predict(const tbo_forest *f, const float *rows, int64_t n_rows,
                int64_t ld, float *out, int32_t *leaf_ids, float *class_sums,
                int32_t tie_rule) {
  const int64_t T = f->num_trees;
  const int32_t C = f->num_classes;
#pragma omp parallel
  {
    double *sums = (double *)malloc(sizeof(double) * (C > 0 ? C : 1));
    char *seen = (char *)malloc(C > 0 ? C : 1);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
      const float *row = rows + r * ld;
      if (C == 0) {
        double acc = f->initial_value;
        for (int64_t t = 0; t < T; ++t) {
          int32_t n = walk_one(f, t, row);
          if (leaf_ids) leaf_ids[r * T + t] = n;
          acc += (double)f->thr[f->tree_off[t] + n];
        }
        if (f->transform == 1) acc = 1.0 / (1.0 + exp(-acc));
        out[r] = (float)acc;
      } else {
        for (int32_t c = 0; c < C; ++c) { sums[c] = f->initial_value; seen[c] = 0; }
        for (int64_t t = 0; t < T; ++t) {
          int32_t n = walk_one(f, t, row);
          if (leaf_ids) leaf_ids[r * T + t] = n;
          sums[f->class_id[t]] += (double)f->thr[f->tree_off[t] + n];
          seen[f->class_id[t]] = 1;
        }
        int32_t best = 0;
        float bestv = 0.f;
        for (int32_t c = 0; c < C; ++c) {
          /* a class without trees keeps 0, as in the reference's vector init */
          float v = seen[c] ? (float)sums[c] : 0.f;
          if (class_sums) class_sums[r * C + c] = v;
          if (c == 0 || (tie_rule == 0 ? v > bestv : !(bestv > v))) { best = c; bestv = v; }
        }
        out[r] = (float)best;
      }
    }
    free(sums);
    free(seen);
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Timed CPU baseline: the reference's parallel CPU schedule, restated.        */

typedef struct { float thr; int16_t feat; int16_t child; } sparse_node; /* 8 B */

typedef struct {
  int64_t num_trees;
  int64_t *off;       /* per tree offset into nodes */
  sparse_node *nodes; /* level order, children adjacent, leaf: feat == -1 */
  int32_t *class_id;
  int32_t num_classes, transform;
  float initial_value;
} tbo_sparse;

/* Level-order renumbering with adjacent children (childIndex = left child). */
tbo_sparse *tbo_sparse_build(const tbo_forest *f) {
  tbo_sparse *s = (tbo_sparse *)calloc(1, sizeof(tbo_sparse));
  const int64_t T = f->num_trees;
  s->num_trees = T;
  s->off = (int64_t *)malloc(sizeof(int64_t) * (T + 1));
  s->nodes = (sparse_node *)malloc(sizeof(sparse_node) * (size_t)f->tree_off[T]);
  s->class_id = (int32_t *)malloc(sizeof(int32_t) * T);
  s->num_classes = f->num_classes;
  s->transform = f->transform;
  s->initial_value = (float)f->initial_value;
  int64_t maxn = 0;
  for (int64_t t = 0; t < T; ++t) {
    int64_t n = f->tree_off[t + 1] - f->tree_off[t];
    if (n > maxn) maxn = n;
  }
  int32_t *queue = (int32_t *)malloc(sizeof(int32_t) * maxn);
  for (int64_t t = 0; t < T; ++t) {
    const int64_t base = f->tree_off[t];
    s->off[t] = base;
    s->class_id[t] = f->class_id ? f->class_id[t] : 0;
    int64_t head = 0, tail = 0;
    queue[tail++] = 0;
    while (head < tail) {
      int32_t o = queue[head];
      sparse_node *d = &s->nodes[base + head];
      d->thr = f->thr[base + o];
      if (f->left[base + o] == -1 && f->right[base + o] == -1) {
        d->feat = -1;
        d->child = -1;
      } else {
        d->feat = (int16_t)f->feat[base + o];
        d->child = (int16_t)tail;
        queue[tail++] = f->left[base + o];
        queue[tail++] = f->right[base + o];
      }
      ++head;
    }
  }
  s->off[T] = f->tree_off[T];
  free(queue);
  return s;
}

void tbo_sparse_free(tbo_sparse *s) {
  if (!s) return;
  free(s->off); free(s->nodes); free(s->class_id); free(s);
}

/* One row block per thread, tree loop outside the row loop, fp32 sums. */
int tbo_cpu_baseline(const tbo_sparse *s, const float *rows, int64_t n_rows,
                     int64_t ld, float *out, int32_t num_threads) {
  const int32_t C = s->num_classes;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
  const int nblocks = num_threads > 0 ? num_threads : omp_get_max_threads();
#else
  const int nblocks = 1;
#endif
  const int64_t per = (n_rows + nblocks - 1) / nblocks;
#pragma omp parallel for schedule(static, 1)
  for (int b = 0; b < nblocks; ++b) {
    const int64_t r0 = b * per, r1 = (r0 + per < n_rows) ? r0 + per : n_rows;
    if (r0 >= r1) continue;
    const int64_t nr = r1 - r0;
    const int32_t W = C > 0 ? C : 1;
    float *acc = (float *)malloc(sizeof(float) * nr * W);
    for (int64_t i = 0; i < nr * W; ++i) acc[i] = s->initial_value;
    for (int64_t t = 0; t < s->num_trees; ++t) {
      const sparse_node *nodes = s->nodes + s->off[t];
      const int32_t cls = C > 0 ? s->class_id[t] : 0;
      for (int64_t r = 0; r < nr; ++r) {
        const float *row = rows + (r0 + r) * ld;
        int32_t n = 0;
        while (nodes[n].feat != -1)
          n = nodes[n].child + !(row[nodes[n].feat] < nodes[n].thr);
        acc[r * W + cls] += nodes[n].thr;
      }
    }
    for (int64_t r = 0; r < nr; ++r) {
      if (C == 0) {
        float v = acc[r];
        if (s->transform == 1) v = 1.0f / (1.0f + expf(-v));
        out[r0 + r] = v;
      } else {
        int32_t best = 0;
        float bestv = acc[r * W];
        for (int32_t c = 1; c < C; ++c)
          if (!(bestv > acc[r * W + c])) { best = c; bestv = acc[r * W + c]; }
        out[r0 + r] = (float)best;
      }
    }
    free(acc);
  }
  return 0;
}

int tbo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
