/*
 * csr_oracle.c - CPU restatement of AutoSAGE's sparse hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the GPU kernels are compared with; it is never part of the product
 * path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load it.
 *
 * The reference computes this path on the CPU with PyTorch:
 *   SpMM      torch.sparse.mm(torch.sparse_csr_tensor(crow, col, val), x)   autosage/ops.py:124-143
 *   SDDMM     (q[rows] * k[col]).sum(1)                                      autosage/_auto.py:79-92
 *   softmax   exp(s - rowmax) / rowsum(exp(s - rowmax)) per CSR row          autosage/_auto.py:744-759
 *   attention SDDMM -> softmax -> SpMM                                       autosage/_auto.py:762-780
 *   row split nonzero(degree >= T) and its complement, ascending row id      csrc/launcher_spmm.cu:49-59
 *   COO->CSR  stable sort of edges by destination + counts + cumsum          autosage/utils/csr.py:6-26
 * The arithmetic of torch.sparse.mm lives in PyTorch (a dependency, not part of the reference
 * tree; the reference pins torch>=2.7); its definition is Y[i,:] = sum_e val[e] * X[col[e],:] over
 * the edges e of row i in storage order, which is what is restated here.  The functions are
 * pinned against outputs of the reference itself (tests/golden/, produced by
 * tests/golden/generate.py) and against the known answers in the reference's tests/test_cpu.py.
 *
 * "f64" functions accumulate in double (the accuracy oracle); "f32" functions accumulate in float
 * in storage order (what the reference's CPU path does; used as the timed CPU port).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ---- a minimal parallel-for over rows (pthreads; the image has no OpenMP runtime) ------------- */
static int g_threads = 0;

int orc_threads(void) {
  if (g_threads > 0) return g_threads;
  const char* env = getenv("ORC_THREADS");
  long n = env ? atol(env) : sysconf(_SC_NPROCESSORS_ONLN);
  if (n < 1) n = 1;
  if (n > 256) n = 256;
  return (int)n;
}

void orc_set_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*orc_row_fn)(int64_t row, void* ctx);

typedef struct {
  orc_row_fn fn;
  void* ctx;
  int64_t n;
  int64_t chunk;
  volatile int64_t* next;
} orc_job;

static void* orc_worker(void* arg) {
  orc_job* job = (orc_job*)arg;
  for (;;) {
    const int64_t begin = __sync_fetch_and_add(job->next, job->chunk);
    if (begin >= job->n) break;
    const int64_t end = begin + job->chunk < job->n ? begin + job->chunk : job->n;
    for (int64_t i = begin; i < end; ++i) job->fn(i, job->ctx);
  }
  return NULL;
}

static void orc_parallel_rows(orc_row_fn fn, void* ctx, int64_t n) {
  int threads = orc_threads();
  if (n < 256 || threads <= 1) {
    for (int64_t i = 0; i < n; ++i) fn(i, ctx);
    return;
  }
  volatile int64_t next = 0;
  orc_job job = {fn, ctx, n, 64, &next};
  pthread_t ids[256];
  int started = 0;
  for (int t = 0; t < threads - 1; ++t) {
    if (pthread_create(&ids[started], NULL, orc_worker, &job) == 0) ++started;
  }
  orc_worker(&job);
  for (int t = 0; t < started; ++t) pthread_join(ids[t], NULL);
}

typedef struct {
  const int64_t* crow;
  const int64_t* col;
  const float* val;
  const float* a;   /* x or q */
  const float* b;   /* k */
  const float* c;   /* v */
  void* out;
  const double* scores;
  int64_t f;
  double scale;
} orc_ctx;

/* Y[i,:] = sum over edges of row i of w * X[col,:], double accumulation. */
static void spmm_f64_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const int64_t f = c->f;
  double* out = (double*)c->out + i * f;
  for (int64_t j = 0; j < f; ++j) out[j] = 0.0;
  for (int64_t e = c->crow[i]; e < c->crow[i + 1]; ++e) {
    const double w = c->val ? (double)c->val[e] : 1.0;
    const float* row = c->a + c->col[e] * f;
    for (int64_t j = 0; j < f; ++j) out[j] += w * (double)row[j];
  }
}
void orc_spmm_f64(const int64_t* crow, const int64_t* col, const float* val, const float* x, double* y,
                  int64_t n, int64_t f) {
  orc_ctx c = {crow, col, val, x, NULL, NULL, y, NULL, f, 1.0};
  orc_parallel_rows(spmm_f64_row, &c, n);
}

/* Same in float, storage order: the reference's CPU arithmetic (timed CPU port). */
static void spmm_f32_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const int64_t f = c->f;
  float* out = (float*)c->out + i * f;
  for (int64_t j = 0; j < f; ++j) out[j] = 0.0f;
  for (int64_t e = c->crow[i]; e < c->crow[i + 1]; ++e) {
    const float w = c->val ? c->val[e] : 1.0f;
    const float* row = c->a + c->col[e] * f;
    for (int64_t j = 0; j < f; ++j) out[j] += w * row[j];
  }
}
void orc_spmm_f32(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                  int64_t n, int64_t f) {
  orc_ctx c = {crow, col, val, x, NULL, NULL, y, NULL, f, 1.0};
  orc_parallel_rows(spmm_f32_row, &c, n);
}

/* out[e] = <q[row(e),:], k[col[e],:]>, double accumulation. */
static void sddmm_f64_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const int64_t f = c->f;
  const float* qi = c->a + i * f;
  for (int64_t e = c->crow[i]; e < c->crow[i + 1]; ++e) {
    const float* kc = c->b + c->col[e] * f;
    double s = 0.0;
    for (int64_t j = 0; j < f; ++j) s += (double)qi[j] * (double)kc[j];
    ((double*)c->out)[e] = s;
  }
}
void orc_sddmm_f64(const int64_t* crow, const int64_t* col, const float* q, const float* k, double* out,
                   int64_t n, int64_t f) {
  orc_ctx c = {crow, col, NULL, q, k, NULL, out, NULL, f, 1.0};
  orc_parallel_rows(sddmm_f64_row, &c, n);
}

static void sddmm_f32_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const int64_t f = c->f;
  const float* qi = c->a + i * f;
  for (int64_t e = c->crow[i]; e < c->crow[i + 1]; ++e) {
    const float* kc = c->b + c->col[e] * f;
    float s = 0.0f;
    for (int64_t j = 0; j < f; ++j) s += qi[j] * kc[j];
    ((float*)c->out)[e] = s;
  }
}
void orc_sddmm_f32(const int64_t* crow, const int64_t* col, const float* q, const float* k, float* out,
                   int64_t n, int64_t f) {
  orc_ctx c = {crow, col, NULL, q, k, NULL, out, NULL, f, 1.0};
  orc_parallel_rows(sddmm_f32_row, &c, n);
}

/* Per-row softmax over CSR segments, double. Empty rows write nothing. */
static void softmax_f64_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const double* scores = c->scores;
  double* probs = (double*)c->out;
  const int64_t s = c->crow[i], e = c->crow[i + 1];
  if (e <= s) return;
  double m = scores[s];
  for (int64_t q = s + 1; q < e; ++q) m = scores[q] > m ? scores[q] : m;
  double sum = 0.0;
  for (int64_t q = s; q < e; ++q) sum += exp(scores[q] - m);
  for (int64_t q = s; q < e; ++q) probs[q] = exp(scores[q] - m) / sum;
}
void orc_row_softmax_f64(const int64_t* crow, const double* scores, double* probs, int64_t n) {
  orc_ctx c = {crow, NULL, NULL, NULL, NULL, NULL, probs, scores, 0, 1.0};
  orc_parallel_rows(softmax_f64_row, &c, n);
}

/* SDDMM (scaled) -> row softmax -> SpMM with V, all in double; rows without edges give zeros. */
static void attention_f64_row(int64_t i, void* p) {
  const orc_ctx* c = (const orc_ctx*)p;
  const int64_t f = c->f;
  const int64_t b = c->crow[i], e = c->crow[i + 1], d = e - b;
  double* o = (double*)c->out + i * f;
  for (int64_t j = 0; j < f; ++j) o[j] = 0.0;
  if (d <= 0) return;
  double* s = (double*)malloc(sizeof(double) * (size_t)d);
  const float* qi = c->a + i * f;
  double m = -INFINITY;
  for (int64_t t = 0; t < d; ++t) {
    const float* kc = c->b + c->col[b + t] * f;
    double acc = 0.0;
    for (int64_t j = 0; j < f; ++j) acc += (double)qi[j] * (double)kc[j];
    s[t] = acc * c->scale;
    if (s[t] > m) m = s[t];
  }
  double sum = 0.0;
  for (int64_t t = 0; t < d; ++t) {
    s[t] = exp(s[t] - m);
    sum += s[t];
  }
  for (int64_t t = 0; t < d; ++t) {
    const double w = s[t] / sum;
    const float* vc = c->c + c->col[b + t] * f;
    for (int64_t j = 0; j < f; ++j) o[j] += w * (double)vc[j];
  }
  free(s);
}
void orc_attention_f64(const int64_t* crow, const int64_t* col, const float* q, const float* k, const float* v,
                       double scale, double* out, int64_t n, int64_t f) {
  orc_ctx c = {crow, col, NULL, q, k, v, out, NULL, f, scale};
  orc_parallel_rows(attention_f64_row, &c, n);
}

/* hubs = rows with degree >= threshold (ascending), lights = the rest (ascending).
 * counts[0] = number of hubs, counts[1] = number of light rows. threshold <= 0: no hubs. */
void orc_hub_split(const int64_t* crow, int64_t n, int64_t threshold, int32_t* hubs, int32_t* lights,
                   int64_t* counts) {
  int64_t h = 0, l = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t d = crow[i + 1] - crow[i];
    if (threshold > 0 && d >= threshold) hubs[h++] = (int32_t)i;
    else lights[l++] = (int32_t)i;
  }
  counts[0] = h;
  counts[1] = l;
}

/* Processing order of the degree-binned plan: hubs first, then light rows; inside a class by
 * descending 1+floor(log2(degree)) capped at 23 (degree 0 -> 0), ties by ascending row id. */
static int orc_bucket(int64_t d, int64_t threshold) {
  int lg = 0;
  for (int64_t t = d; t > 0; t >>= 1) ++lg;
  if (lg > 23) lg = 23;
  const int desc = 23 - lg;
  return (threshold > 0 && d >= threshold) ? desc : 24 + desc;
}

void orc_plan_order(const int64_t* crow, int64_t n, int64_t threshold, int32_t* order, int64_t* counts) {
  int64_t start[49];
  memset(start, 0, sizeof(start));
  for (int64_t i = 0; i < n; ++i) start[orc_bucket(crow[i + 1] - crow[i], threshold) + 1]++;
  for (int b = 0; b < 48; ++b) start[b + 1] += start[b];
  counts[0] = start[24];
  counts[1] = n - start[24];
  for (int64_t i = 0; i < n; ++i) order[start[orc_bucket(crow[i + 1] - crow[i], threshold)]++] = (int32_t)i;
}

/* Row partition balanced by nnz: bounds[k] = first row r with crow[r] >= k*nnz/parts
 * (searchsorted left on crow), bounds[0] = 0, bounds[parts] = n. */
void orc_partition_rows(const int64_t* crow, int64_t n, int64_t parts, int64_t* bounds) {
  const int64_t nnz = crow[n] - crow[0];
  bounds[0] = 0;
  for (int64_t k = 1; k < parts; ++k) {
    const int64_t target = crow[0] + (k * nnz) / parts;
    int64_t lo = 0, hi = n + 1; /* search in crow[0..n] */
    while (lo < hi) {
      const int64_t mid = (lo + hi) / 2;
      if (crow[mid] < target) lo = mid + 1;
      else hi = mid;
    }
    if (lo > n) lo = n;
    if (lo < bounds[k - 1]) lo = bounds[k - 1];
    bounds[k] = lo;
  }
  bounds[parts] = n;
}

/* COO -> CSR keyed by `row_of_edge`, stable: edges of a row keep their input order.
 * perm[i] = input position of the edge stored at CSR position i. */
void orc_coo_to_csr(const int64_t* row_of_edge, const int64_t* col_of_edge, int64_t n_edges, int64_t n,
                    int64_t* crow, int64_t* col, int64_t* perm) {
  for (int64_t i = 0; i <= n; ++i) crow[i] = 0;
  for (int64_t e = 0; e < n_edges; ++e) crow[row_of_edge[e] + 1]++;
  for (int64_t i = 0; i < n; ++i) crow[i + 1] += crow[i];
  int64_t* cursor = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  for (int64_t i = 0; i < n; ++i) cursor[i] = crow[i];
  for (int64_t e = 0; e < n_edges; ++e) {
    const int64_t at = cursor[row_of_edge[e]]++;
    col[at] = col_of_edge[e];
    if (perm) perm[at] = e;
  }
  free(cursor);
}
