/*
 * CPU oracle for the dense-reduction path - TEST INFRASTRUCTURE, not product code.
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may load this file's
 * library; nothing under raft_b200/ or include/ does.
 *
 * It restates, as sequential fp64 host loops, what the reference computes:
 *   oracle_reduce          raft::linalg::reduce semantics - the naive kernels the reference's
 *                          own tests compare against: cpp/tests/linalg/reduce.cuh:21-147
 *                          (coalesced / strided, incl. the inplace rule :40-44, :93-97),
 *                          main_op index = position along the reduced axis
 *                          (linalg/detail/coalesced_reduction-inl.cuh:96,
 *                          linalg/detail/strided_reduction.cuh:42,103)
 *   norms                  functor choice of linalg/detail/norm.cuh:26-37, 49-60, checked in
 *                          the reference by cpp/tests/linalg/norm.cu:43-66, 144-158
 *   argmin / argmax        raft::argmin_op / argmax_op, core/operators.hpp:183-199
 *                          (ties -> lower key for both)
 *   oracle_rows_by_key     cpp/tests/linalg/reduce_rows_by_key.cu:21-44 (+ weights :46-72)
 *   oracle_cols_by_key     cpp/tests/linalg/reduce_cols_by_key.cu:20-42
 *   oracle_compare_approx  the reference's hybrid tolerance, cpp/tests/test_utils.h:31-45
 *   synth_fill             the counter-based generator of include/raft_b200/detail/synth.cuh,
 *                          same integer hash and the same three double operations
 *
 * Parity pin: tests/test_oracle_golden.py checks these functions against the known-answer
 * vectors of the reference's tests (3x4 max reduce, argmin/argmax operator cases, 3x4 argmin
 * matrices, constant-matrix sums) and tests/golden/ holds outputs of the reference's own
 * kernels (built by oracle/build_ref.sh) on seeded inputs.
 *
 * The omp_* functions are the same loops with OpenMP over the outputs; bench.py times them as
 * the host baseline.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define EXPORT __attribute__((visibility("default")))

/* dtype codes - same values as b2r_dtype in include/raft_b200.h */
enum { DT_F32 = 0, DT_F64 = 1, DT_F16 = 2, DT_I32 = 3, DT_I64 = 4, DT_I16 = 5, DT_U32 = 6 };
enum { MAIN_IDENTITY = 0, MAIN_SQ = 1, MAIN_ABS = 2, MAIN_NZ = 3, MAIN_TO_KVP = 4 };
enum { RED_ADD = 0, RED_MIN = 1, RED_MAX = 2, RED_ARGMIN = 3, RED_ARGMAX = 4 };
enum { FIN_IDENTITY = 0, FIN_SQRT = 1, FIN_MUL = 2, FIN_DIV = 3, FIN_ABS = 4 };

/* ------------------------------------------------------------------------------------ */
/* synthetic data                                                                         */
/* ------------------------------------------------------------------------------------ */
static uint64_t mix64(uint64_t x)
{
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

static uint16_t float_to_half_bits(float f);
static float half_bits_to_float(uint16_t h);

/* returns the value as double plus (for kind 2) the exact integer */
static double synth_value(uint64_t seed_mixed, uint64_t index, int kind, double lo, double hi, int wide,
                          long long* as_int)
{
  const uint64_t h = mix64(seed_mixed ^ mix64(index));
  if (kind == 2) {
    const long long ilo  = (long long)lo;
    const long long span = (long long)hi - ilo;
    const long long v    = ilo + (long long)((h >> 32) % (uint64_t)(span > 0 ? span : 1));
    if (as_int) *as_int = v;
    return (double)v;
  }
  if (kind == 1) {
    const uint64_t h2 = mix64(h);
    long long s       = 0;
    for (int k = 0; k < 4; ++k) {
      s += (long long)((h >> (16 * k)) & 0xffffull);
      s += (long long)((h2 >> (16 * k)) & 0xffffull);
    }
    s -= 4ll * 65535ll;
    volatile double r = (double)s * (1.0 / 53509.91992145008);
    return r;
  }
  volatile double u = wide ? (double)(h >> 11) * (1.0 / 9007199254740992.0) : (double)(h >> 40) * (1.0 / 16777216.0);
  volatile double p = (hi - lo) * u; /* volatile: keep mul and add as two rounded operations */
  volatile double r = lo + p;
  return r;
}

EXPORT int synth_fill(void* dst, int dtype, int64_t n, int64_t first_index, uint64_t seed, int kind, double lo,
                      double hi)
{
  const uint64_t sm = mix64(seed);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    long long iv   = 0;
    const double v = synth_value(sm, (uint64_t)(first_index + i), kind, lo, hi, dtype == DT_F64, &iv);
    switch (dtype) {
      case DT_F32: ((float*)dst)[i] = (float)v; break;
      case DT_F64: ((double*)dst)[i] = v; break;
      case DT_F16: ((uint16_t*)dst)[i] = float_to_half_bits((float)v); break;
      case DT_I32: ((int32_t*)dst)[i] = (int32_t)iv; break;
      case DT_U32: ((uint32_t*)dst)[i] = (uint32_t)iv; break;
      case DT_I64: ((int64_t*)dst)[i] = (int64_t)iv; break;
      case DT_I16: ((int16_t*)dst)[i] = (int16_t)iv; break;
      default: break;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------ */
/* element access                                                                         */
/* ------------------------------------------------------------------------------------ */
static float half_bits_to_float(uint16_t h)
{
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp        = (h >> 10) & 0x1fu;
  uint32_t man        = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      exp = 127 - 15 + 1;
      while ((man & 0x400u) == 0) {
        man <<= 1;
        --exp;
      }
      man &= 0x3ffu;
      bits = sign | (exp << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t float_to_half_bits(float f)
{
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp   = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man        = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift    = 14 - exp;
    uint32_t half_man  = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1);
    const uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half_man & 1u))) ++half_man;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half       = sign | ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem  = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
  return (uint16_t)half;
}

static inline double load_elem(const void* p, int dtype, int64_t i)
{
  switch (dtype) {
    case DT_F32: return (double)((const float*)p)[i];
    case DT_F64: return ((const double*)p)[i];
    case DT_F16: return (double)half_bits_to_float(((const uint16_t*)p)[i]);
    case DT_I32: return (double)((const int32_t*)p)[i];
    case DT_I64: return (double)((const int64_t*)p)[i];
    case DT_I16: return (double)((const int16_t*)p)[i];
    case DT_U32: return (double)((const uint32_t*)p)[i];
    default: return 0.0;
  }
}

/* main_op runs in the INPUT element type, as in the reference (raft::sq_op on a float returns
 * a float, core/operators.hpp:93-100; a half is squared in float, :102-106). */
static inline double apply_main(double x, int main_op, int in_dtype)
{
  switch (main_op) {
    case MAIN_SQ: {
      if (in_dtype == DT_F32 || in_dtype == DT_F16) {
        const volatile float f = (float)x;
        const volatile float p = f * f;
        return (double)p;
      }
      return x * x;
    }
    case MAIN_ABS: return fabs(x);
    case MAIN_NZ: return x != 0.0 ? 1.0 : 0.0;
    default: return x;
  }
}

static inline double apply_final(double x, int final_op, double scalar)
{
  switch (final_op) {
    case FIN_SQRT: return sqrt(x);
    case FIN_MUL: return x * scalar;
    case FIN_DIV: return x / scalar;
    case FIN_ABS: return fabs(x);
    default: return x;
  }
}

/* ------------------------------------------------------------------------------------ */
/* reduce                                                                                 */
/*   in: [n_rows x n_cols] in `layout` (0 row-major, 1 col-major); apply 0 = one output  */
/*   per row, 1 = one per column. Scalar outputs go to out_val (double); key/value        */
/*   outputs to out_key (int64) + out_val. When inplace, out_* hold the previous outputs. */
/*   Sums use a Neumaier-compensated fp64 accumulator, so fp64 inputs are also covered.   */
/* ------------------------------------------------------------------------------------ */
EXPORT int oracle_reduce(const void* in, int in_dtype, int layout, int apply, int64_t n_rows, int64_t n_cols,
                         int main_op, int reduce_op, int final_op, double final_scalar, double init,
                         int64_t init_key, int inplace, double* out_val, int64_t* out_key)
{
  const int64_t n_out = apply == 0 ? n_rows : n_cols;
  const int64_t n_red = apply == 0 ? n_cols : n_rows;
  const int kvp       = reduce_op == RED_ARGMIN || reduce_op == RED_ARGMAX;
  if (kvp && out_key == NULL) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < n_out; ++o) {
    double acc   = init, comp = 0.0;
    int64_t akey = init_key;
    for (int64_t j = 0; j < n_red; ++j) {
      const int64_t r   = apply == 0 ? o : j;
      const int64_t c   = apply == 0 ? j : o;
      const int64_t idx = layout == 0 ? r * n_cols + c : c * n_rows + r;
      const double x    = load_elem(in, in_dtype, idx);
      if (kvp) {
        /* main_op = {j, x}; argmin_op / argmax_op of core/operators.hpp:183-199 */
        const int better = reduce_op == RED_ARGMIN ? (x < acc) : (x > acc);
        if (better || (x == acc && j < akey)) {
          acc  = x;
          akey = j;
        }
      } else {
        const double v = apply_main(x, main_op, in_dtype);
        if (reduce_op == RED_ADD) {
          const double t = acc + v;
          comp += fabs(acc) >= fabs(v) ? (acc - t) + v : (v - t) + acc;
          acc = t;
        } else if (reduce_op == RED_MIN) {
          acc = fmin(acc, v);
        } else {
          acc = fmax(acc, v);
        }
      }
    }
    if (kvp) {
      if (inplace) {
        const double ov  = out_val[o];
        const int64_t ok = out_key[o];
        /* reduce_op(old, acc) */
        const int better = reduce_op == RED_ARGMIN ? (acc < ov) : (acc > ov);
        if (!(better || (acc == ov && akey < ok))) {
          acc  = ov;
          akey = ok;
        }
      }
      out_val[o] = acc;
      out_key[o] = akey;
    } else {
      double v = acc + comp;
      if (inplace) {
        const double ov = out_val[o];
        if (reduce_op == RED_ADD) {
          v = ov + v;
        } else if (reduce_op == RED_MIN) {
          v = fmin(ov, v);
        } else {
          v = fmax(ov, v);
        }
      }
      out_val[o] = apply_final(v, final_op, final_scalar);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------ */
/* row_normalize (linalg/normalize.cuh:46-107, kernels linalg/detail/normalize.cuh:26-56)*/
/*   norm_i = final(reduce_j main(in[i][j])) evaluated in fp64 and rounded ONCE to the    */
/*   element type; `if (norm <= eps) return;` leaves the row of `out` untouched; the      */
/*   division runs in the element type. norm_type 1 = L1, 2 = L2 (with root), 3 = Linf.   */
/* ------------------------------------------------------------------------------------ */
EXPORT int oracle_row_normalize(const void* in, void* out, int dtype, int64_t n_rows, int64_t n_cols, int norm_type,
                                double eps)
{
  if (dtype != DT_F32 && dtype != DT_F64) return 1;
  if (norm_type < 1 || norm_type > 3) return 1;
  const int main_op = norm_type == 2 ? MAIN_SQ : MAIN_ABS;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n_rows; ++i) {
    double acc = 0.0, comp = 0.0;
    for (int64_t j = 0; j < n_cols; ++j) {
      const double v = apply_main(load_elem(in, dtype, i * n_cols + j), main_op, dtype);
      if (norm_type == 3) {
        acc = fmax(acc, v);
      } else {
        const double t = acc + v;
        comp += fabs(acc) >= fabs(v) ? (acc - t) + v : (v - t) + acc;
        acc = t;
      }
    }
    double norm = acc + comp;
    if (norm_type == 2) norm = sqrt(norm);
    if (dtype == DT_F32) {
      const float nf = (float)norm;
      if (nf <= (float)eps) continue;
      for (int64_t j = 0; j < n_cols; ++j)
        ((float*)out)[i * n_cols + j] = ((const float*)in)[i * n_cols + j] / nf;
    } else {
      if (norm <= eps) continue;
      for (int64_t j = 0; j < n_cols; ++j)
        ((double*)out)[i * n_cols + j] = ((const double*)in)[i * n_cols + j] / norm;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------ */
/* by-key sums                                                                            */
/* ------------------------------------------------------------------------------------ */
static inline int64_t load_key(const void* keys, int key_dtype, int64_t i)
{
  switch (key_dtype) {
    case DT_I32: return ((const int32_t*)keys)[i];
    case DT_U32: return ((const uint32_t*)keys)[i];
    case DT_I64: return ((const int64_t*)keys)[i];
    default: return 0;
  }
}

/* sums[k][c] (+)= sum_i w[i] * A[i][c] over rows with key k; counts[k] (+)= rows with key k.
 * Each thread owns whole output rows (keys), so the row order of the additions is the
 * sequential one for any thread count. */
EXPORT int oracle_rows_by_key(const void* A, int dtype, int64_t lda, const void* keys, int key_dtype,
                              const void* weights, int64_t nrows, int64_t ncols, int64_t nkeys, int reset,
                              double* sums, int64_t* counts)
{
  if (reset) {
    memset(sums, 0, sizeof(double) * (size_t)(nkeys * ncols));
    if (counts) memset(counts, 0, sizeof(int64_t) * (size_t)nkeys);
  }
  double* comp = (double*)calloc((size_t)(nkeys * ncols), sizeof(double));
  if (!comp) return 2;
  /* bucket the rows by key first so that threads can work on disjoint keys */
  int64_t* start = (int64_t*)calloc((size_t)nkeys + 1, sizeof(int64_t));
  int64_t* order = (int64_t*)malloc(sizeof(int64_t) * (size_t)(nrows > 0 ? nrows : 1));
  if (!start || !order) return 2;
  for (int64_t i = 0; i < nrows; ++i) {
    const int64_t k = load_key(keys, key_dtype, i);
    if (k < 0 || k >= nkeys) return 3;
    start[k + 1]++;
  }
  for (int64_t k = 0; k < nkeys; ++k)
    start[k + 1] += start[k];
  int64_t* fill = (int64_t*)malloc(sizeof(int64_t) * (size_t)(nkeys > 0 ? nkeys : 1));
  memcpy(fill, start, sizeof(int64_t) * (size_t)nkeys);
  for (int64_t i = 0; i < nrows; ++i)
    order[fill[load_key(keys, key_dtype, i)]++] = i;
  free(fill);
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t k = 0; k < nkeys; ++k) {
    double* s = sums + k * ncols;
    double* c = comp + k * ncols;
    for (int64_t q = start[k]; q < start[k + 1]; ++q) {
      const int64_t i = order[q];
      const double w  = weights ? load_elem(weights, dtype, i) : 1.0;
      for (int64_t j = 0; j < ncols; ++j) {
        const double v = load_elem(A, dtype, i * lda + j) * w;
        const double t = s[j] + v;
        c[j] += fabs(s[j]) >= fabs(v) ? (s[j] - t) + v : (v - t) + s[j];
        s[j] = t;
      }
    }
    for (int64_t j = 0; j < ncols; ++j)
      s[j] += c[j];
    if (counts) counts[k] += start[k + 1] - start[k];
  }
  free(comp);
  free(start);
  free(order);
  return 0;
}

/* out[r][keys[c]] (+)= data[r][c] */
EXPORT int oracle_cols_by_key(const void* data, int dtype, const void* keys, int key_dtype, int64_t nrows,
                              int64_t ncols, int64_t nkeys, int reset, double* out)
{
  if (reset) memset(out, 0, sizeof(double) * (size_t)(nrows * nkeys));
  int bad = 0;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrows; ++r) {
    double* comp = (double*)calloc((size_t)(nkeys > 0 ? nkeys : 1), sizeof(double));
    double* s    = out + r * nkeys;
    for (int64_t c = 0; c < ncols; ++c) {
      const int64_t k = load_key(keys, key_dtype, c);
      if (k < 0 || k >= nkeys) {
        bad = 1;
        continue;
      }
      const double v = load_elem(data, dtype, r * ncols + c);
      const double t = s[k] + v;
      comp[k] += fabs(s[k]) >= fabs(v) ? (s[k] - t) + v : (v - t) + s[k];
      s[k] = t;
    }
    for (int64_t k = 0; k < nkeys; ++k)
      s[k] += comp[k];
    free(comp);
  }
  return bad ? 3 : 0;
}

/* ------------------------------------------------------------------------------------ */
/* comparison: passes when |a-b| <= eps, else when |a-b| / max(|a|,|b|) <= eps            */
/* returns the number of mismatches; worst_* describe the largest violation               */
/* ------------------------------------------------------------------------------------ */
EXPORT int64_t oracle_compare_approx(const double* expect, const double* actual, int64_t n, double eps,
                                     double* worst_abs, double* worst_rel, int64_t* worst_idx)
{
  int64_t bad = 0;
  double wa = 0.0, wr = 0.0;
  int64_t wi = -1;
  for (int64_t i = 0; i < n; ++i) {
    const double a = expect[i], b = actual[i];
    if (isnan(a) && isnan(b)) continue;
    const double diff  = fabs(a - b);
    const double m     = fmax(fabs(a), fabs(b));
    const double ratio = diff > eps ? diff / m : diff;
    if (!(ratio <= eps)) {
      ++bad;
      if (diff > wa || wi < 0) {
        wa = diff;
        wr = m > 0 ? diff / m : 0.0;
        wi = i;
      }
    }
  }
  if (worst_abs) *worst_abs = wa;
  if (worst_rel) *worst_rel = wr;
  if (worst_idx) *worst_idx = wi;
  return bad;
}

/* ------------------------------------------------------------------------------------ */
/* host baseline: the five benchmark reductions as tight fp32-load / fp64-accumulate loops */
/* ------------------------------------------------------------------------------------ */
EXPORT int omp_threads(void)
{
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

EXPORT void omp_row_sum_f32(const float* in, int64_t n_rows, int64_t n_cols, int square, int root, float* out)
{
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n_rows; ++r) {
    const float* p = in + r * n_cols;
    double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    int64_t j = 0;
    if (square) {
      for (; j + 4 <= n_cols; j += 4) {
        a0 += (double)p[j] * p[j];
        a1 += (double)p[j + 1] * p[j + 1];
        a2 += (double)p[j + 2] * p[j + 2];
        a3 += (double)p[j + 3] * p[j + 3];
      }
      for (; j < n_cols; ++j)
        a0 += (double)p[j] * p[j];
    } else {
      for (; j + 4 <= n_cols; j += 4) {
        a0 += p[j];
        a1 += p[j + 1];
        a2 += p[j + 2];
        a3 += p[j + 3];
      }
      for (; j < n_cols; ++j)
        a0 += p[j];
    }
    const double s = (a0 + a1) + (a2 + a3);
    out[r]         = (float)(root ? sqrt(s) : s);
  }
}

/* column sums of a row-major matrix; n_cols <= 4096 */
EXPORT int omp_col_sum_f32(const float* in, int64_t n_rows, int64_t n_cols, double scale, float* out)
{
  if (n_cols > 4096) return 1;
  double total[4096];
  memset(total, 0, sizeof(double) * (size_t)n_cols);
#pragma omp parallel
  {
    double local[4096];
    memset(local, 0, sizeof(double) * (size_t)n_cols);
#pragma omp for schedule(static) nowait
    for (int64_t r = 0; r < n_rows; ++r) {
      const float* p = in + r * n_cols;
      for (int64_t j = 0; j < n_cols; ++j)
        local[j] += p[j];
    }
#pragma omp critical
    for (int64_t j = 0; j < n_cols; ++j)
      total[j] += local[j];
  }
  for (int64_t j = 0; j < n_cols; ++j)
    out[j] = (float)(total[j] * scale);
  return 0;
}

EXPORT void omp_row_argmin_f32(const float* in, int64_t n_rows, int64_t n_cols, int32_t* out_key, float* out_val)
{
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n_rows; ++r) {
    const float* p = in + r * n_cols;
    float best     = p[0];
    int32_t bk     = 0;
    for (int64_t j = 1; j < n_cols; ++j) {
      if (p[j] < best) { /* strict: the first (lowest) index wins ties */
        best = p[j];
        bk   = (int32_t)j;
      }
    }
    out_key[r] = bk;
    out_val[r] = best;
  }
}

/* thread-private [nkeys x ncols] fp64 tables merged at the end */
EXPORT int omp_rows_by_key_f32(const float* A, const int32_t* keys, int64_t nrows, int64_t ncols, int64_t nkeys,
                               float* sums, int64_t* counts)
{
  const size_t tbl = (size_t)(nkeys * ncols);
  double* total    = (double*)calloc(tbl, sizeof(double));
  int64_t* tcount  = (int64_t*)calloc((size_t)nkeys, sizeof(int64_t));
  if (!total || !tcount) return 2;
#pragma omp parallel
  {
    double* local   = (double*)calloc(tbl, sizeof(double));
    int64_t* lcount = (int64_t*)calloc((size_t)nkeys, sizeof(int64_t));
#pragma omp for schedule(static) nowait
    for (int64_t i = 0; i < nrows; ++i) {
      const float* p = A + i * ncols;
      double* s      = local + (int64_t)keys[i] * ncols;
      for (int64_t j = 0; j < ncols; ++j)
        s[j] += p[j];
      lcount[keys[i]]++;
    }
#pragma omp critical
    {
      for (size_t q = 0; q < tbl; ++q)
        total[q] += local[q];
      for (int64_t k = 0; k < nkeys; ++k)
        tcount[k] += lcount[k];
    }
    free(local);
    free(lcount);
  }
  for (size_t q = 0; q < tbl; ++q)
    sums[q] = (float)total[q];
  if (counts) memcpy(counts, tcount, sizeof(int64_t) * (size_t)nkeys);
  free(total);
  free(tcount);
  return 0;
}
