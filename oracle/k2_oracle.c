/* TEST INFRASTRUCTURE ONLY - never linked into or loaded by the product path.
 *
 * Plain-C, single-threaded CPU restatement of the k2 reference algorithms on the
 * dense-intersection / total-score hot path.  It is the checker the CUDA path is
 * compared with in tests, in the smoke test and as the "port" CPU baseline.
 *
 * Restated: CtcGraphs, IntersectDense, IntersectDensePruned (batch mode), forward and
 * backward scores in both semirings, total scores, arc posteriors, ShortestPath, the
 * basic properties.
 *
 * Parity of this restatement is PINNED: tests/test_oracle_vs_reference.py
 * compares every function here with the reference's own CPU code (compiled by
 * oracle/Makefile into oracle/_ref/libk2ref.so) on seeded random inputs, and
 * tests/test_oracle_golden.py checks it against fixtures produced by that
 * reference build plus the literal answers of the reference's Python tests.
 *
 * Differences from the reference, all deliberate:
 *  - state ids are 32-bit (the reference packs them into uint16,
 *    k2/csrc/intersect_dense.cu:631-633,985-987, which silently breaks graphs
 *    with more than 65535 states);
 *  - an arc whose label is >= the number of classes scores -inf everywhere
 *    (the reference does so in the recursion, intersect_dense.cu:817-832, but
 *    reads past the row in FormatOutput, :426-428);
 *  - FSAs are processed one at a time, so the grid of state copies is
 *    (T_i+1)*S_i per FSA rather than (T_max+1)*S_total; the enumeration order
 *    of kept states and arcs is the same.
 *
 * Conventions (k2/csrc/fsa.h:31-63, :138-185; k2/csrc/utils.h:107-140):
 *  Arc = {int32 src, int32 dest, int32 label, float score}, src/dest relative
 *  to their FSA.  An FsaVec is row_splits1[N+1] (fsa -> state), row_splits2[S+1]
 *  (state -> arc) and arcs[A].  A DenseFsaVec is scores[rows][cols] with
 *  cols = C+1, column = label+1, and b_row_splits[K+1] giving the rows of each
 *  sequence (T_i frames plus one final row [0,-inf,...]).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  int32_t src, dest, label;
  float score;
} Arc;

typedef struct {
  int32_t num_fsas, num_states, num_arcs;
  int32_t *row_splits1; /* [num_fsas+1] */
  int32_t *row_splits2; /* [num_states+1] */
  Arc *arcs;            /* [num_arcs] */
  int32_t *aux;         /* [num_arcs] or NULL: aux_labels (ctc_graphs) */
  int32_t *arc_map_a;   /* [num_arcs] or NULL */
  int32_t *arc_map_b;   /* [num_arcs] or NULL */
  float final_beam;     /* output_beam actually used (after any reduction) */
} K2oFsaVec;

static const char *g_err = "";
const char *k2o_last_error(void) { return g_err; }

void k2o_free(K2oFsaVec *f) {
  if (!f) return;
  free(f->row_splits1);
  free(f->row_splits2);
  free(f->arcs);
  free(f->aux);
  free(f->arc_map_a);
  free(f->arc_map_b);
  free(f);
}

void k2o_dims(const K2oFsaVec *f, int32_t *nf, int32_t *ns, int32_t *na) {
  *nf = f->num_fsas;
  *ns = f->num_states;
  *na = f->num_arcs;
}

float k2o_final_beam(const K2oFsaVec *f) { return f->final_beam; }

void k2o_copy(const K2oFsaVec *f, int32_t *rs1, int32_t *rs2, void *arcs,
              int32_t *aux, int32_t *map_a, int32_t *map_b) {
  memcpy(rs1, f->row_splits1, sizeof(int32_t) * (f->num_fsas + 1));
  memcpy(rs2, f->row_splits2, sizeof(int32_t) * (f->num_states + 1));
  size_t n = (size_t)f->num_arcs;
  if (n) {
    memcpy(arcs, f->arcs, sizeof(Arc) * n);
    if (aux && f->aux) memcpy(aux, f->aux, 4 * n);
    if (map_a && f->arc_map_a) memcpy(map_a, f->arc_map_a, 4 * n);
    if (map_b && f->arc_map_b) memcpy(map_b, f->arc_map_b, 4 * n);
  }
}

/* ------------------------------------------------------------------------
 * CtcGraphs: k2/csrc/fsa_algo.cu:577-730.  For a transcript of L symbols the
 * graph has 2L+2 states: even state 2k is the blank state in front of symbol k
 * (k == L: the trailing blank state), odd state 2k+1 is the state of symbol k,
 * and 2L+1 is the final state.  Scores are all zero.
 * ---------------------------------------------------------------------- */
K2oFsaVec *k2o_ctc_graphs(const int32_t *sym_row_splits, int32_t num_seqs,
                          const int32_t *symbols, int32_t modified) {
  K2oFsaVec *g = (K2oFsaVec *)calloc(1, sizeof(K2oFsaVec));
  g->num_fsas = num_seqs;
  g->row_splits1 = (int32_t *)malloc(4 * (num_seqs + 1));
  int32_t ns = 0;
  for (int32_t i = 0; i < num_seqs; ++i) {
    g->row_splits1[i] = ns;
    ns += 2 * (sym_row_splits[i + 1] - sym_row_splits[i]) + 2; /* :596 */
  }
  g->row_splits1[num_seqs] = ns;
  g->num_states = ns;
  g->row_splits2 = (int32_t *)malloc(4 * (ns + 1));
  int32_t na = 0;
  for (int32_t i = 0; i < num_seqs; ++i) {
    int32_t s0 = g->row_splits1[i], L = sym_row_splits[i + 1] - sym_row_splits[i];
    const int32_t *sym = symbols + sym_row_splits[i];
    for (int32_t s = 0; s < 2 * L + 2; ++s) {
      g->row_splits2[s0 + s] = na;
      int32_t k = s / 2, n = 2; /* :614-645 */
      if (s % 2) {
        if (k == L) {
          n = 0;
        } else if (modified) {
          n = 3;
        } else {
          int32_t next = (k + 1 == L) ? -1 : sym[k + 1];
          if (sym[k] != next) n = 3;
        }
      }
      na += n;
    }
  }
  g->row_splits2[ns] = na;
  g->num_arcs = na;
  g->arcs = (Arc *)malloc(sizeof(Arc) * (na ? na : 1));
  g->aux = (int32_t *)malloc(4 * (na ? na : 1));
  for (int32_t i = 0; i < num_seqs; ++i) {
    int32_t s0 = g->row_splits1[i], L = sym_row_splits[i + 1] - sym_row_splits[i];
    const int32_t *sym = symbols + sym_row_splits[i];
    for (int32_t s = 0; s < 2 * L + 2; ++s) {
      int32_t k = s / 2, is_final = (k == L);
      int32_t cur = is_final ? -1 : sym[k];
      int32_t a0 = g->row_splits2[s0 + s], n = g->row_splits2[s0 + s + 1] - a0;
      for (int32_t j = 0; j < n; ++j) { /* :672-727 */
        Arc arc;
        int32_t aux = 0;
        arc.score = 0;
        arc.src = s;
        if (s % 2) {
          int32_t next = (k + 1 == L) ? -1 : sym[k + 1];
          if (cur == next && !modified) {
            arc.label = j == 0 ? 0 : cur;
            arc.dest = j == 0 ? s + 1 : s;
          } else if (j == 0) {
            arc.label = 0;
            arc.dest = s + 1;
          } else if (j == 1) {
            arc.label = cur;
            arc.dest = s;
          } else {
            arc.label = next;
            aux = (k + 1 == L) ? -1 : next;
            arc.dest = s + 2;
          }
        } else {
          arc.label = j == 0 ? 0 : cur;
          arc.dest = j == 0 ? s : s + 1;
          aux = j == 0 ? 0 : cur;
          if (is_final && j != 0) aux = -1;
        }
        g->arcs[a0 + j] = arc;
        g->aux[a0 + j] = aux;
      }
    }
  }
  return g;
}

/* ------------------------------------------------------------------------
 * IntersectDense: k2/csrc/intersect_dense.cu.
 * ---------------------------------------------------------------------- */
static inline float dense_score(const float *scores, int64_t row, int32_t cols,
                                int32_t label) {
  int32_t c = label + 1;
  if (c < 0 || c >= cols) return -INFINITY;
  return scores[row * cols + c];
}

/* Viterbi forward and backward grids of one FSA: DoStep0 (:745-774) and DoStep
 * (:778-847).  fwd and bwd are [(Tk+1)*S]; bwd[t] is the backward score after t
 * steps, i.e. at time position Tk - t. */
static void viterbi_grids(const Arc *arcs, int32_t num_arcs, int32_t S, int32_t Tk,
                          const float *scores, int64_t row0, int32_t cols,
                          float *fwd, float *bwd) {
  for (int64_t i = 0; i < (int64_t)(Tk + 1) * S; ++i) fwd[i] = bwd[i] = -INFINITY;
  if (S == 0) return;
  fwd[0] = 0.0f;
  bwd[S - 1] = 0.0f;
  for (int32_t t = 1; t <= Tk; ++t) {
    const float *fp = fwd + (int64_t)(t - 1) * S, *bp = bwd + (int64_t)(t - 1) * S;
    float *fn = fwd + (int64_t)t * S, *bn = bwd + (int64_t)t * S;
    for (int32_t a = 0; a < num_arcs; ++a) {
      Arc arc = arcs[a];
      float bf = dense_score(scores, row0 + (t - 1), cols, arc.label),
            bb = dense_score(scores, row0 + (Tk - t), cols, arc.label);
      float f = fp[arc.src] + arc.score + bf; /* :833-836, left to right */
      float b = bp[arc.dest] + arc.score + bb;
      if (f > fn[arc.dest]) fn[arc.dest] = f;
      if (b > bn[arc.src]) bn[arc.src] = b;
    }
  }
}

K2oFsaVec *k2o_intersect_dense(const int32_t *a_rs1, int32_t num_fsas,
                               const int32_t *a_rs2, const void *a_arcs_v,
                               const float *scores, int32_t rows, int32_t cols,
                               const int32_t *b_row_splits, int32_t num_seqs,
                               const int32_t *a_to_b_map, float output_beam,
                               int32_t max_states, int32_t max_arcs) {
  const Arc *a_arcs = (const Arc *)a_arcs_v;
  (void)rows;
  if (num_fsas <= 0) { g_err = "num_fsas must be > 0"; return NULL; }   /* :136 */
  if (!(output_beam > 0)) { g_err = "output_beam must be > 0"; return NULL; } /* :137 */
  if (!a_to_b_map && num_fsas != num_seqs) {                              /* :1054 */
    g_err = "a_fsas.Dim0() != b_fsas.Dim0() and no a_to_b_map";
    return NULL;
  }
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t j = a_to_b_map ? a_to_b_map[i] : i;
    if (j < 0 || j >= num_seqs) { g_err = "a_to_b_map out of range"; return NULL; }
    if (i > 0 && a_to_b_map && a_to_b_map[i] < a_to_b_map[i - 1]) {       /* :1058 */
      g_err = "a_to_b_map should be monotonically increasing";
      return NULL;
    }
  }
  for (int32_t j = 1; j < num_seqs; ++j) {                                /* :168-177 */
    if (b_row_splits[j + 1] - b_row_splits[j] > b_row_splits[j] - b_row_splits[j - 1]) {
      g_err = "Sequences (DenseFsaVec) must be in sorted order from greatest to least length";
      return NULL;
    }
  }

  /* Viterbi grids for every FSA. */
  float **fwd = (float **)calloc(num_fsas, sizeof(float *)),
        **bwd = (float **)calloc(num_fsas, sizeof(float *));
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t j = a_to_b_map ? a_to_b_map[i] : i;
    int32_t Tk = b_row_splits[j + 1] - b_row_splits[j];
    int32_t s0 = a_rs1[i], S = a_rs1[i + 1] - s0;
    int32_t arc0 = a_rs2[s0], narcs = a_rs2[s0 + S] - arc0;
    size_t n = (size_t)(Tk + 1) * (size_t)S;
    fwd[i] = (float *)malloc(4 * (n ? n : 1));
    bwd[i] = (float *)malloc(4 * (n ? n : 1));
    viterbi_grids(a_arcs + arc0, narcs, S, Tk, scores, b_row_splits[j], cols, fwd[i],
                  bwd[i]);
  }

  float *cutoff = (float *)malloc(4 * num_fsas);
  int64_t tot_states, tot_arcs;
  for (;;) { /* :240-320 */
    tot_states = 0;
    tot_arcs = 0;
    for (int32_t i = 0; i < num_fsas; ++i) {
      int32_t j = a_to_b_map ? a_to_b_map[i] : i;
      int32_t Tk = b_row_splits[j + 1] - b_row_splits[j];
      int32_t s0 = a_rs1[i], S = a_rs1[i + 1] - s0;
      /* GetScoreCutoffs :870-924 */
      float start = S == 0 ? -INFINITY : bwd[i][(int64_t)Tk * S + 0],
            end = S == 0 ? -INFINITY : fwd[i][(int64_t)Tk * S + (S - 1)];
      float mn = start < end ? start : end;
      cutoff[i] = mn - output_beam;
      for (int32_t t = 0; t <= Tk; ++t)
        for (int32_t s = 0; s < S; ++s)
          if (fwd[i][(int64_t)t * S + s] + bwd[i][(int64_t)(Tk - t) * S + s] > cutoff[i]) {
            tot_states++;
            tot_arcs += a_rs2[s0 + s + 1] - a_rs2[s0 + s]; /* :298 (last frame included) */
          }
    }
    int64_t limit = 0, total = 0;
    if (tot_states > max_states) { limit = max_states; total = tot_states; }
    else if (tot_arcs > max_arcs) { limit = max_arcs; total = tot_arcs; }
    else break;
    /* DecreaseBeam :854-862 */
    float cur = output_beam, next = cur * sqrt(limit * 1.0 / total);
    if (next < cur * 0.25) next = cur * 0.25;
    if (next > cur * 0.75) next = cur * 0.75;
    output_beam = next;
  }

  K2oFsaVec *out = (K2oFsaVec *)calloc(1, sizeof(K2oFsaVec));
  out->final_beam = output_beam;
  out->num_fsas = num_fsas;
  out->num_states = (int32_t)tot_states;
  out->row_splits1 = (int32_t *)malloc(4 * (num_fsas + 1));
  out->row_splits2 = (int32_t *)malloc(4 * (tot_states + 1));
  /* tot_arcs is an upper bound on the kept arcs */
  size_t cap = (size_t)(tot_arcs ? tot_arcs : 1);
  out->arcs = (Arc *)malloc(sizeof(Arc) * cap);
  out->arc_map_a = (int32_t *)malloc(4 * cap);
  out->arc_map_b = (int32_t *)malloc(4 * cap);

  int32_t ns_out = 0, na_out = 0;
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t j = a_to_b_map ? a_to_b_map[i] : i;
    int32_t Tk = b_row_splits[j + 1] - b_row_splits[j];
    int64_t row0 = b_row_splits[j];
    int32_t s0 = a_rs1[i], S = a_rs1[i + 1] - s0;
    out->row_splits1[i] = ns_out;
    int32_t fsa_first_state = ns_out;
    /* new ids of the kept states of frames t and t+1 (-1 = pruned) */
    int32_t *id_cur = (int32_t *)malloc(4 * (S ? S : 1)),
            *id_next = (int32_t *)malloc(4 * (S ? S : 1));
    int32_t next_id = ns_out;
    for (int32_t s = 0; s < S; ++s) /* frame 0 */
      id_cur[s] = (fwd[i][s] + bwd[i][(int64_t)Tk * S + s] > cutoff[i]) ? next_id++ : -1;
    for (int32_t t = 0; t <= Tk; ++t) {
      if (t < Tk) {
        for (int32_t s = 0; s < S; ++s)
          id_next[s] = (fwd[i][(int64_t)(t + 1) * S + s] +
                            bwd[i][(int64_t)(Tk - t - 1) * S + s] > cutoff[i])
                           ? next_id++ : -1;
      }
      for (int32_t s = 0; s < S; ++s) {
        if (id_cur[s] < 0) continue;
        out->row_splits2[id_cur[s]] = na_out;
        if (t == Tk) continue; /* :385-387 */
        for (int32_t a = a_rs2[s0 + s]; a < a_rs2[s0 + s + 1]; ++a) {
          Arc arc = a_arcs[a];
          if (id_next[arc.dest] < 0) continue; /* :456 */
          float arc_score = arc.score + dense_score(scores, row0 + t, cols, arc.label);
          float fb = fwd[i][(int64_t)t * S + s] + arc_score +
                     bwd[i][(int64_t)(Tk - t - 1) * S + arc.dest]; /* :465-467 */
          if (!(fb > cutoff[i])) continue;
          Arc o;
          o.src = id_cur[s] - fsa_first_state;
          o.dest = id_next[arc.dest] - fsa_first_state;
          o.label = arc.label;
          o.score = arc_score;
          out->arcs[na_out] = o;
          out->arc_map_a[na_out] = a;
          out->arc_map_b[na_out] =
              (int32_t)((row0 + t) * cols + (arc.label + 1)); /* :531-535 */
          na_out++;
        }
      }
      int32_t *tmp = id_cur; id_cur = id_next; id_next = tmp;
    }
    ns_out = next_id;
    free(id_cur);
    free(id_next);
  }
  out->row_splits1[num_fsas] = ns_out;
  out->row_splits2[ns_out] = na_out;
  out->num_arcs = na_out;
  for (int32_t i = 0; i < num_fsas; ++i) { free(fwd[i]); free(bwd[i]); }
  free(fwd); free(bwd); free(cutoff);
  return out;
}

/* ------------------------------------------------------------------------
 * IntersectDensePruned, batch mode: k2/csrc/intersect_dense_pruned.cu:41-1694 as its
 * CPU build runs it, one sequence at a time (beam, cutoffs, state numbering and
 * pruning windows are all per sequence).  Frames hold their states and arcs in
 * growable arrays; the windows compact them in place.
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t ns, na;     /* states and arcs of the frame */
  int32_t *astate;    /* [ns] state in the graph (idx01) */
  float *fwd, *bwd;   /* [ns] */
  int32_t *arc0;      /* [ns+1] first arc of every state */
  int32_t *aidx;      /* [na] arc in the graph (idx012) */
  float *ll;          /* [na] arc.score + dense score */
  int32_t *dest;      /* [na] state of the next frame, -1 if it was pruned */
} PFrame;

static void pframe_free(PFrame *f) {
  free(f->astate); free(f->fwd); free(f->bwd); free(f->arc0); free(f->aidx); free(f->ll);
  free(f->dest);
  memset(f, 0, sizeof(*f));
}

/* GetPruningCutoffs, :687-767: the mixed float / double arithmetic is the reference's. */
static float next_beam(float dyn, float best, int32_t active, int32_t t, int32_t final_t,
                       float default_beam, float min_active, float max_active,
                       float *cutoff) {
  float cur_min = min_active;
  if (t + 5 >= final_t) cur_min = fmaxf(min_active, max_active / 2);
  if (active <= max_active) {
    if (active >= cur_min || active == 0) {
      dyn = 0.8 * dyn + 0.2 * default_beam;
    } else {
      if (dyn < default_beam) dyn = default_beam;
      dyn *= 1.25;
    }
  } else if (t + 5 < final_t) {
    if (dyn > default_beam) dyn = default_beam;
    dyn *= 0.8;
  }
  if (t == final_t - 1) dyn = 1.0e+10;
  *cutoff = best - dyn;
  return dyn;
}

/* PruneTimeRange, :1373-1634 (SetBackwardProbsFinal :1170-1193, PropagateBackward
 * :1239-1346), frames [begin, end) of one sequence. */
static void prune_window(PFrame *fr, int32_t begin, int32_t end, int32_t g_final,
                         float output_beam) {
  PFrame *last = &fr[end];
  for (int32_t k = 0; k < last->ns; ++k) {
    float f = last->fwd[k];
    last->bwd[k] = (f - f == 0) ? -f : -INFINITY;
  }
  int32_t *new_next = NULL; /* new numbers of the states of frame t + 1 */
  for (int32_t t = end - 1; t >= begin; --t) {
    PFrame *c = &fr[t], *n = &fr[t + 1];
    int32_t *new_cur = (int32_t *)malloc(4 * (c->ns + 1));
    uint8_t *keep_arc = (uint8_t *)malloc(c->na + 1);
    int32_t kept_states = 0;
    for (int32_t k = 0; k < c->ns; ++k) {
      float best = -INFINITY;
      for (int32_t p = c->arc0[k]; p < c->arc0[k + 1]; ++p) {
        keep_arc[p] = 0;
        if (c->dest[p] < 0) continue;
        /* frame t + 1 has been compacted already: find the state under its new number
         * (a state that was dropped there had a backward score of -inf) */
        int32_t d = new_next ? new_next[c->dest[p]] : c->dest[p];
        if (d < 0) continue;
        float bl = c->ll[p] + n->bwd[d];
        if (bl + c->fwd[k] >= -output_beam) {
          keep_arc[p] = 1;
          if (bl > best) best = bl;
        }
      }
      c->bwd[k] = (c->astate[k] == g_final) ? -c->fwd[k] : best;
      int32_t keep = (c->bwd[k] != -INFINITY) || t == begin;
      new_cur[k] = keep ? kept_states++ : -1;
    }
    /* compaction of frame t: arcs first (their dest moves to the new numbering of
     * frame t + 1, which was fixed in the previous iteration), then states */
    int32_t wa = 0, ws = 0;
    for (int32_t k = 0; k < c->ns; ++k) {
      int32_t first = wa;
      for (int32_t p = c->arc0[k]; p < c->arc0[k + 1]; ++p) {
        if (!keep_arc[p]) continue;
        c->aidx[wa] = c->aidx[p];
        c->ll[wa] = c->ll[p];
        c->dest[wa] = new_next ? new_next[c->dest[p]] : c->dest[p];
        ++wa;
      }
      if (new_cur[k] >= 0) {
        c->astate[ws] = c->astate[k];
        c->fwd[ws] = c->fwd[k];
        c->bwd[ws] = c->bwd[k];
        c->arc0[ws] = first;
        ++ws;
      }
    }
    c->arc0[ws] = wa;
    c->ns = ws;
    c->na = wa;
    free(keep_arc);
    free(new_next);
    new_next = new_cur;
  }
  free(new_next);
}

K2oFsaVec *k2o_intersect_dense_pruned(const int32_t *a_rs1, int32_t a_num_fsas,
                                      const int32_t *a_rs2, const void *a_arcs_v,
                                      const float *scores, int32_t rows, int32_t cols,
                                      const int32_t *b_rs, int32_t num_seqs, float search_beam,
                                      float output_beam, int32_t min_active,
                                      int32_t max_active, int32_t allow_partial) {
  const Arc *a_arcs = (const Arc *)a_arcs_v;
  if (!(search_beam > 0) || !(output_beam > 0)) { g_err = "beams must be > 0"; return NULL; }
  if (min_active < 0 || max_active <= min_active) { g_err = "bad active limits"; return NULL; }
  if (a_num_fsas != num_seqs && a_num_fsas != 1) { g_err = "a_fsas.Dim0() mismatch"; return NULL; }
  int32_t T = 0;
  for (int32_t i = 0; i < num_seqs; ++i)
    if (b_rs[i + 1] - b_rs[i] > T) T = b_rs[i + 1] - b_rs[i];

  K2oFsaVec *out = (K2oFsaVec *)calloc(1, sizeof(K2oFsaVec));
  out->num_fsas = num_seqs;
  out->row_splits1 = (int32_t *)calloc(num_seqs + 1, 4);
  int64_t cap_s = 1024, cap_a = 1024, tot_s = 0, tot_a = 0;
  out->row_splits2 = (int32_t *)malloc(4 * (cap_s + 1));
  out->arcs = (Arc *)malloc(sizeof(Arc) * cap_a);
  out->arc_map_a = (int32_t *)malloc(4 * cap_a);
  out->arc_map_b = (int32_t *)malloc(4 * cap_a);

  for (int32_t i = 0; i < num_seqs; ++i) {
    const int32_t gi = a_num_fsas == 1 ? 0 : i, g_start = a_rs1[gi],
                  g_states = a_rs1[gi + 1] - g_start, g_final = a_rs1[gi + 1] - 1;
    const int32_t row0 = b_rs[i], final_t = b_rs[i + 1] - row0;
    PFrame *fr = (PFrame *)calloc(T + 2, sizeof(PFrame));
    int32_t *slot = (int32_t *)malloc(4 * (g_states + 1)); /* graph state -> next-frame state */
    for (int32_t s = 0; s < g_states; ++s) slot[s] = -1;
    /* frame 0: InitialFrameInfo, :435-472 */
    fr[0].ns = g_states > 0;
    fr[0].astate = (int32_t *)malloc(4 * 2);
    fr[0].fwd = (float *)malloc(4 * 2);
    fr[0].bwd = (float *)malloc(4 * 2);
    fr[0].astate[0] = g_start;
    fr[0].fwd[0] = 0;
    float beam = search_beam;
    int32_t next_end = 20; /* :164-199: windows of 30 frames every 20 */
    for (int32_t t = 0; t < T; ++t) {
      PFrame *c = &fr[t], *n = &fr[t + 1];
      /* GetArcs, :778-908 */
      c->arc0 = (int32_t *)malloc(4 * (c->ns + 1));
      int32_t na = 0;
      for (int32_t k = 0; k < c->ns; ++k) {
        c->arc0[k] = na;
        na += a_rs2[c->astate[k] + 1] - a_rs2[c->astate[k]];
      }
      c->arc0[c->ns] = na;
      c->na = na;
      c->aidx = (int32_t *)malloc(4 * (na + 1));
      c->ll = (float *)malloc(4 * (na + 1));
      c->dest = (int32_t *)malloc(4 * (na + 1));
      float *end = (float *)malloc(4 * (na + 1));
      int32_t redirect = 0;
      if (allow_partial && t == final_t - 1) {
        redirect = 1;
        for (int32_t k = 0; k < c->ns; ++k)
          for (int32_t a = a_rs2[c->astate[k]]; a < a_rs2[c->astate[k] + 1]; ++a)
            if (a_arcs[a].label == -1) redirect = 0;
      }
      float best = -INFINITY;
      for (int32_t k = 0; k < c->ns; ++k) {
        int32_t p = c->arc0[k];
        for (int32_t a = a_rs2[c->astate[k]]; a < a_rs2[c->astate[k] + 1]; ++a, ++p) {
          float acoustic = row0 + t < rows
                               ? dense_score(scores, (int64_t)row0 + t, cols, a_arcs[a].label)
                               : -INFINITY;
          int32_t dest = c->astate[k] + a_arcs[a].dest - a_arcs[a].src;
          if (redirect) {
            dest = g_final;
            acoustic = 0;
          }
          c->aidx[p] = a;
          c->ll[p] = acoustic + a_arcs[a].score;
          c->dest[p] = dest;
          end[p] = c->fwd[k] + c->ll[p];
          if (end[p] > best) best = end[p];
        }
      }
      /* PropagateForward, :925-1153: the first arc above the cutoff creates a state */
      float cutoff;
      beam = next_beam(beam, best, c->ns, t, final_t, search_beam, (float)min_active,
                       (float)max_active, &cutoff);
      n->astate = (int32_t *)malloc(4 * (na + 2));
      n->fwd = (float *)malloc(4 * (na + 2));
      n->bwd = (float *)malloc(4 * (na + 2));
      int32_t nn = 0;
      for (int32_t p = 0; p < na; ++p) {
        int32_t d = c->dest[p] - g_start;
        if (end[p] > cutoff && slot[d] < 0) {
          slot[d] = nn;
          n->astate[nn] = c->dest[p];
          n->fwd[nn] = -INFINITY;
          ++nn;
        }
      }
      for (int32_t p = 0; p < na; ++p) {
        int32_t j = slot[c->dest[p] - g_start];
        c->dest[p] = j;
        if (j >= 0 && end[p] > n->fwd[j]) n->fwd[j] = end[p];
      }
      for (int32_t j = 0; j < nn; ++j) slot[n->astate[j] - g_start] = -1;
      n->ns = nn;
      free(end);
      int32_t this_end = next_end >= T ? T : next_end;
      if (t == this_end - 1) {
        int32_t begin = next_end - 30 > 0 ? next_end - 30 : 0;
        prune_window(fr, begin, this_end, g_final, output_beam);
        next_end += 20;
      }
    }
    fr[T].arc0 = (int32_t *)calloc(fr[T].ns + 1, 4); /* the last frame has no arcs */
    /* FormatOutput, :474-657 */
    int32_t seq_states = 0;
    for (int32_t t = 0; t <= T; ++t) seq_states += fr[t].ns;
    int32_t extra = (g_states > 0) && fr[final_t].ns == 0; /* :519-547 */
    int32_t state_base = 0;
    for (int32_t t = 0; t <= T; ++t) {
      PFrame *c = &fr[t];
      for (int32_t k = 0; k < c->ns; ++k) {
        if (tot_s + 2 > cap_s) {
          cap_s *= 2;
          out->row_splits2 = (int32_t *)realloc(out->row_splits2, 4 * (cap_s + 1));
        }
        out->row_splits2[tot_s++] = (int32_t)tot_a;
        for (int32_t p = c->arc0[k]; p < c->arc0[k + 1]; ++p) {
          if (tot_a + 1 > cap_a) {
            cap_a *= 2;
            out->arcs = (Arc *)realloc(out->arcs, sizeof(Arc) * cap_a);
            out->arc_map_a = (int32_t *)realloc(out->arc_map_a, 4 * cap_a);
            out->arc_map_b = (int32_t *)realloc(out->arc_map_b, 4 * cap_a);
          }
          int32_t label = a_arcs[c->aidx[p]].label, map_a = c->aidx[p];
          Arc arc;
          arc.src = state_base + k;
          arc.dest = state_base + c->ns + c->dest[p];
          arc.label = label;
          arc.score = c->ll[p];
          if (t == final_t - 1 && label != -1) { /* allow_partial, :625-634 */
            arc.label = -1;
            map_a = -1;
          }
          out->arcs[tot_a] = arc;
          out->arc_map_a[tot_a] = map_a;
          out->arc_map_b[tot_a] = (row0 + t) * cols + label + 1;
          ++tot_a;
        }
      }
      state_base += c->ns;
    }
    if (extra) {
      if (tot_s + 2 > cap_s) {
        cap_s *= 2;
        out->row_splits2 = (int32_t *)realloc(out->row_splits2, 4 * (cap_s + 1));
      }
      out->row_splits2[tot_s++] = (int32_t)tot_a;
    }
    (void)seq_states;
    out->row_splits1[i + 1] = (int32_t)tot_s;
    for (int32_t t = 0; t <= T + 1; ++t) pframe_free(&fr[t]);
    free(fr);
    free(slot);
  }
  out->row_splits2[tot_s] = (int32_t)tot_a;
  out->num_states = (int32_t)tot_s;
  out->num_arcs = (int32_t)tot_a;
  return out;
}

/* ------------------------------------------------------------------------
 * LogAdd: k2/csrc/utils.h:511-563.
 * ---------------------------------------------------------------------- */
#define MIN_LOG_DIFF_FLOAT -15.9423847198486328125f
#define MIN_LOG_DIFF_DOUBLE -36.0436533891171535515240975655615329742431640625

static inline double log_add_d(double x, double y) {
  double diff;
  if (x < y) { diff = x - y; x = y; } else { diff = y - x; }
  if (diff >= MIN_LOG_DIFF_DOUBLE) return x + log1p(exp(diff));
  return x;
}
static inline float log_add_f(float x, float y) {
  float diff;
  if (x < y) { diff = x - y; x = y; } else { diff = y - x; }
  if (diff >= MIN_LOG_DIFF_FLOAT) return x + log1pf(expf(diff));
  return x;
}

/* Incoming arcs bucketed by destination state, stable in arc index:
 * GetIncomingArcs, k2/csrc/fsa_utils.cu:901-928 (ragged_ops.cu:1482-1501). */
static void incoming_index(const int32_t *rs1, int32_t num_fsas, const int32_t *rs2,
                           const Arc *arcs, int32_t ns, int32_t na, int32_t *in_splits,
                           int32_t *in_arcs) {
  memset(in_splits, 0, 4 * (size_t)(ns + 1));
  for (int32_t i = 0; i < num_fsas; ++i)
    for (int32_t a = rs2[rs1[i]]; a < rs2[rs1[i + 1]]; ++a)
      in_splits[rs1[i] + arcs[a].dest + 1]++;
  for (int32_t s = 0; s < ns; ++s) in_splits[s + 1] += in_splits[s];
  int32_t *fill = (int32_t *)malloc(4 * (size_t)(ns + 1));
  memcpy(fill, in_splits, 4 * (size_t)(ns + 1));
  for (int32_t i = 0; i < num_fsas; ++i)
    for (int32_t a = rs2[rs1[i]]; a < rs2[rs1[i + 1]]; ++a)
      in_arcs[fill[rs1[i] + arcs[a].dest]++] = a;
  (void)na;
  free(fill);
}

/* GetForwardScores: k2/csrc/fsa_utils.cu:1124-1278 on a top-sorted acyclic
 * FsaVec.  States are visited in index order, which yields the same values as
 * the reference's state batches; each state folds its incoming arcs in arc order
 * starting from -inf (ragged_ops_inl.h:63-73; ArgMax ties go to the later arc,
 * :649-655).  Results are written as double; with use_double == 0 all
 * arithmetic is done in float exactly as the reference's float instantiation. */
int32_t k2o_forward_scores(const int32_t *rs1, int32_t num_fsas, const int32_t *rs2,
                           const void *arcs_v, int32_t log_semiring, int32_t use_double,
                           double *out, int32_t *entering_arcs) {
  const Arc *arcs = (const Arc *)arcs_v;
  int32_t ns = rs1[num_fsas], na = rs2[ns];
  int32_t *in_splits = (int32_t *)malloc(4 * (size_t)(ns + 1)),
          *in_arcs = (int32_t *)malloc(4 * (size_t)(na ? na : 1));
  incoming_index(rs1, num_fsas, rs2, arcs, ns, na, in_splits, in_arcs);
  /* arc -> src state idx01 */
  int32_t *src01 = (int32_t *)malloc(4 * (size_t)(na ? na : 1));
  for (int32_t s = 0; s < ns; ++s)
    for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a) src01[a] = s;
  for (int32_t i = 0; i < num_fsas; ++i) {
    for (int32_t s = rs1[i]; s < rs1[i + 1]; ++s) {
      int32_t best = -1;
      if (use_double) {
        double val = -INFINITY;
        for (int32_t k = in_splits[s]; k < in_splits[s + 1]; ++k) {
          int32_t a = in_arcs[k];
          float w = arcs[a].score;
          double e = out[src01[a]] + w;
          if (log_semiring) val = log_add_d(e, val);
          else if (e >= val) { val = e; best = a; }
        }
        if (s == rs1[i] && val == -INFINITY) val = 0; /* :1155-1165, :1268-1272 */
        out[s] = val;
      } else {
        float val = -INFINITY;
        for (int32_t k = in_splits[s]; k < in_splits[s + 1]; ++k) {
          int32_t a = in_arcs[k];
          float e = (float)out[src01[a]] + arcs[a].score;
          if (log_semiring) val = log_add_f(e, val);
          else if (e >= val) { val = e; best = a; }
        }
        if (s == rs1[i] && val == -INFINITY) val = 0;
        out[s] = val;
      }
      if (entering_arcs) entering_arcs[s] = best;
    }
  }
  free(in_splits); free(in_arcs); free(src01);
  return 0;
}

/* GetBackwardScores: k2/csrc/fsa_utils.cu:1345-1454. */
int32_t k2o_backward_scores(const int32_t *rs1, int32_t num_fsas, const int32_t *rs2,
                            const void *arcs_v, int32_t log_semiring, int32_t use_double,
                            double *out) {
  const Arc *arcs = (const Arc *)arcs_v;
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t s0 = rs1[i];
    for (int32_t s = rs1[i + 1] - 1; s >= s0; --s) {
      if (use_double) {
        double val = -INFINITY;
        for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a) {
          float w = arcs[a].score;
          double e = out[s0 + arcs[a].dest] + w;
          if (log_semiring) val = log_add_d(e, val);
          else if (e > val) val = e;
        }
        if (s == rs1[i + 1] - 1 && val == -INFINITY) val = 0;
        out[s] = val;
      } else {
        float val = -INFINITY;
        for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a) {
          float e = (float)out[s0 + arcs[a].dest] + arcs[a].score;
          if (log_semiring) val = log_add_f(e, val);
          else if (e > val) val = e;
        }
        if (s == rs1[i + 1] - 1 && val == -INFINITY) val = 0;
        out[s] = val;
      }
    }
  }
  return 0;
}

/* GetTotScores (fsa_utils.cu:1809-1837) and GetArcPost (:1839-1901). */
int32_t k2o_tot_scores_and_arc_post(const int32_t *rs1, int32_t num_fsas,
                                    const int32_t *rs2, const void *arcs_v,
                                    int32_t use_double, const double *fwd,
                                    const double *bwd, double *tot, double *post) {
  const Arc *arcs = (const Arc *)arcs_v;
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t b = rs1[i], e = rs1[i + 1];
    tot[i] = (e > b) ? fwd[e - 1] : -INFINITY;
    if (!post) continue;
    if (use_double) {
      double t = 0;
      if (b != e) t = 0.5 * (fwd[e - 1] + bwd[b]);
      double neg = (t != -INFINITY) ? -t : -INFINITY;
      for (int32_t s = b; s < e; ++s)
        for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a) {
          float w = arcs[a].score;
          post[a] = w + fwd[s] + bwd[b + arcs[a].dest] + neg;
        }
    } else {
      float t = 0;
      if (b != e) t = 0.5f * ((float)fwd[e - 1] + (float)bwd[b]);
      float neg = (t != -INFINITY) ? -t : -INFINITY;
      for (int32_t s = b; s < e; ++s)
        for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a)
          post[a] = arcs[a].score + (float)fwd[s] + (float)bwd[b + arcs[a].dest] + neg;
    }
  }
  return 0;
}

/* ShortestPath: k2/csrc/fsa_algo.cu:869-1144 (semantics of its "simple
 * version", :892-926): trace entering_arcs back from the final state; a path
 * that does not reach state 0 counts as no path. */
int32_t k2o_shortest_path(const int32_t *rs1, int32_t num_fsas, const void *arcs_v,
                          const int32_t *entering_arcs, int32_t *path_row_splits,
                          int32_t *best_arcs) {
  const Arc *arcs = (const Arc *)arcs_v;
  int32_t n = 0;
  for (int32_t i = 0; i < num_fsas; ++i) {
    path_row_splits[i] = n;
    int32_t b = rs1[i], e = rs1[i + 1];
    if (e == b) continue;
    int32_t cur = e - 1, len = 0, idx = entering_arcs[cur];
    while (idx != -1) {
      best_arcs[n + len++] = idx;
      cur = b + arcs[idx].src;
      idx = entering_arcs[cur];
    }
    if (cur != b) len = 0;
    for (int32_t k = 0; k < len / 2; ++k) { /* reverse into path order */
      int32_t tmp = best_arcs[n + k];
      best_arcs[n + k] = best_arcs[n + len - 1 - k];
      best_arcs[n + len - 1 - k] = tmp;
    }
    n += len;
  }
  path_row_splits[num_fsas] = n;
  return n;
}

/* GetFsaVecBasicProperties: k2/csrc/fsa.cu:54-217. */
int32_t k2o_properties(const int32_t *rs1, int32_t num_fsas, const int32_t *rs2,
                       const void *arcs_v, int32_t *props_out) {
  const Arc *arcs = (const Arc *)arcs_v;
  int32_t tot = 0x1FF;
  int32_t ns = rs1[num_fsas];
  char *reach = (char *)calloc((size_t)(2 * ns + 2), 1);
  for (int32_t i = 0; i < num_fsas; ++i) {
    int32_t b = rs1[i], e = rs1[i + 1], n = e - b;
    int32_t neg = 0;
    int32_t first_arc = rs2[b];
    for (int32_t s = b; s < e; ++s) {
      for (int32_t a = rs2[s]; a < rs2[s + 1]; ++a) {
        Arc arc = arcs[a];
        if (arc.src != s - b) neg |= 0x01;
        if (arc.dest <= arc.src) {
          neg |= 0x08;
          if (arc.dest < arc.src) neg |= 0x04;
        }
        if (arc.label == 0) neg |= 0x40;
        if (arc.label < 0) {
          if (arc.label != -1) neg |= 0x01;
          else if (arc.dest != n - 1) neg |= 0x01;
        }
        if (arc.label != -1 && arc.dest == n - 1) neg |= 0x01;
        if (arc.dest < 0 || arc.dest >= n) neg |= 0x01;
        else if (arc.dest != arc.src) reach[b + arc.dest] = 1;
        if (a == first_arc) {
          reach[b] = 1;
          reach[ns + e - 1] = 1;
        }
        if (arc.dest != arc.src) reach[ns + s] = 1;
        if (a != rs2[s]) {
          Arc p = arcs[a - 1];
          if ((uint32_t)arc.label <= (uint32_t)p.label) neg |= 0x20;
          if ((uint32_t)arc.label < (uint32_t)p.label) neg |= 0x10;
          if (arc.label == p.label && arc.dest < p.dest) neg |= 0x10;
        }
      }
    }
    char r = 1, cr = 1;
    for (int32_t s = b; s < e; ++s) { r &= reach[s]; cr &= reach[ns + s]; }
    int32_t no_arcs = (rs2[b] == rs2[e]);
    neg |= (!r * 0x80) | (!cr * 0x100) | (no_arcs * 0x02);
    int32_t p = (~neg) & 0x1FF;
    if (props_out) props_out[i] = p;
    tot &= p;
  }
  free(reach);
  return tot;
}
