/* CPU restatement in C (fp32, OpenMP) of the attention hot path, used as the TIMED CPU BASELINE and checked
 * against oracle/attn_oracle.py in tests/test_oracle_c.py.  TEST INFRASTRUCTURE ONLY: the product path never
 * links or calls this file.  Parity status: pinned through attn_oracle.py (which is pinned by the golden
 * vectors generated from the reference's ref/prefill_ref.py and ref/oracle.py).
 *
 * Built by crucible_strix_halo_b200/build.py: gcc -O3 -fopenmp -shared -> oracle/_ref/liboracle.so
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define EPS 1e-6f

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Overrides OMP_NUM_THREADS (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

static inline float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
static inline float siluf_(float x) { return x / (1.f + expf(-x)); }

/* One GDN layer over n rows from a carried state (ref/oracle.py:101-130 with the serial recurrence of
 * ref/prefill_ref.py:5-13; engine/layers/ops.h:296-375).
 * qkv [n][2*Hk*128+Hv*128], z [n][Hv*128], ab [n][2*Hv] (a then b logits), conv [C][4], hist3 [3][C] (rows
 * pos0-3..pos0-1, zeros at the start) or NULL, state [Hv][128][128] in/out, out [n][Hv*128] gated. */
void oracle_gdn_layer(const float* qkv, const float* z, const float* ab, const float* conv, const float* A_log,
                      const float* dt_bias, const float* gamma, const float* hist3, float* state, float* out, int n,
                      int Hv, int Hk) {
  const int KW = Hk * 128, C = 2 * KW + Hv * 128, VW = Hv * 128, rep = Hv / Hk;
  float* act = (float*)malloc((size_t)n * C * sizeof(float));   /* conv + SiLU, then normalised q/k */
#pragma omp parallel for schedule(static)
  for (int t = 0; t < n; ++t) {
    for (int ch = 0; ch < C; ++ch) {
      float acc = 0.f;
      for (int u = 0; u < 4; ++u) {
        const int r = t - (3 - u);
        float x = 0.f;
        if (r >= 0) x = qkv[(size_t)r * C + ch];
        else if (hist3) x = hist3[(size_t)(3 + r) * C + ch];
        acc += conv[(size_t)ch * 4 + u] * x;
      }
      act[(size_t)t * C + ch] = siluf_(acc);
    }
    for (int h = 0; h < 2 * Hk; ++h) {       /* q heads then k heads */
      float* v = act + (size_t)t * C + h * 128;
      float ss = 0.f;
      for (int j = 0; j < 128; ++j) ss += v[j] * v[j];
      const float sc = 1.f / sqrtf(ss + EPS) * (h < Hk ? 0.08838834764831845f : 1.f);
      for (int j = 0; j < 128; ++j) v[j] *= sc;
    }
  }
#pragma omp parallel for schedule(dynamic, 1)
  for (int h = 0; h < Hv; ++h) {
    float* S = state + (size_t)h * 16384;
    const int kh = h / rep;
    const float A = -expf(A_log[h]);
    float y[128], delta[128];
    for (int t = 0; t < n; ++t) {
      const float* q = act + (size_t)t * C + kh * 128;
      const float* k = act + (size_t)t * C + KW + kh * 128;
      const float* v = act + (size_t)t * C + 2 * KW + h * 128;
      const float sp = ab[(size_t)t * 2 * Hv + h] + dt_bias[h];
      const float decay = expf(A * (sp > 20.f ? sp : log1pf(expf(sp))));
      const float beta = sigmoidf_(ab[(size_t)t * 2 * Hv + Hv + h]);
      for (int j = 0; j < 128; ++j) delta[j] = 0.f;
      for (int i = 0; i < 128; ++i) {
        float* Si = S + i * 128;
        const float ki = k[i];
        for (int j = 0; j < 128; ++j) { Si[j] *= decay; delta[j] += Si[j] * ki; }
      }
      for (int j = 0; j < 128; ++j) { delta[j] = beta * (v[j] - delta[j]); y[j] = 0.f; }
      for (int i = 0; i < 128; ++i) {
        float* Si = S + i * 128;
        const float ki = k[i], qi = q[i];
        for (int j = 0; j < 128; ++j) { Si[j] += ki * delta[j]; y[j] += Si[j] * qi; }
      }
      float ss = 0.f;
      for (int j = 0; j < 128; ++j) ss += y[j] * y[j];
      const float rs = 1.f / sqrtf(ss / 128.f + EPS);
      const float* zr = z + (size_t)t * VW + h * 128;
      float* o = out + (size_t)t * VW + h * 128;
      for (int j = 0; j < 128; ++j) o[j] = y[j] * rs * gamma[j] * sigmoidf_(zr[j]);
    }
  }
  free(act);
}

static inline float half_to_float(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023;
  uint32_t u;
  if (e == 0) {
    if (m == 0) u = s;
    else {
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 1024)) { mm <<= 1; ++sh; }
      u = s | ((uint32_t)(113 - sh) << 23) | ((mm & 1023) << 13);
    }
  } else if (e == 31) u = s | 0x7f800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

typedef struct { float s; int id; } scored;
static int by_score_then_id(const void* a, const void* b) {
  const scored *x = (const scored*)a, *y = (const scored*)b;
  if (x->s != y->s) return x->s > y->s ? -1 : 1;
  return x->id - y->id;
}
static int by_int(const void* a, const void* b) { return *(const int*)a - *(const int*)b; }

/* One decode row of QSA against a full cache, after prep (engine/layers/qsa_long.h:9-43, :202-221, :399-499):
 * qn [Hq][256] normed+roped queries, gate [Hq][256], iq [4][128] prepared indexer queries, position p;
 * kc/vc fp16 bits [ctx][Hkv][256], pool tiled fp32 (offset(b,d) = (b/32)*4096 + d*32 + b%32).
 * Writes the gated context out [Hq][256] and the selected ids sel[512] (nsel = -1 when dense). */
void oracle_qsa_decode_row(const float* qn, const float* gate, const float* iq, int p, const uint16_t* kc,
                           const uint16_t* vc, const float* pool, float* out, int* sel, int* nsel, int Hq, int Hkv) {
  const int nb = (p + 1) / 4, gqa = Hq / Hkv;
  int n;
  int* pos = (int*)malloc((size_t)(p + 1 > 2052 ? 2052 : p + 1) * sizeof(int) + 64);
  if (nb <= 512) {
    *nsel = -1;
    n = p + 1;
    for (int t = 0; t < n; ++t) pos[t] = t;
  } else {
    scored* sc = (scored*)malloc((size_t)nb * sizeof(scored));
#pragma omp parallel for schedule(static)
    for (int b = 0; b < nb; ++b) {
      const float* key = pool + (size_t)(b / 32) * 4096 + b % 32;
      float s = 0.f;
      for (int h = 0; h < 4; ++h) {
        float d = 0.f;
        for (int j = 0; j < 128; ++j) d += iq[h * 128 + j] * key[j * 32];
        s += d > 0.f ? d : 0.f;
      }
      sc[b].s = s * 0.08838834764831845f;
      sc[b].id = b;
    }
    qsort(sc, nb, sizeof(scored), by_score_then_id);
    for (int i = 0; i < 512; ++i) sel[i] = sc[i].id;
    qsort(sel, 512, sizeof(int), by_int);
    free(sc);
    *nsel = 512;
    n = 0;
    for (int i = 0; i < 512; ++i)
      for (int t = 0; t < 4; ++t) pos[n++] = sel[i] * 4 + t;
    for (int t = nb * 4; t <= p; ++t) pos[n++] = t;
  }
#pragma omp parallel for schedule(static)
  for (int h = 0; h < Hq; ++h) {
    const int g = h / gqa;
    const float* q = qn + h * 256;
    float* lg = (float*)malloc((size_t)n * sizeof(float));
    float m = -INFINITY;
    for (int t = 0; t < n; ++t) {
      const uint16_t* k = kc + ((size_t)pos[t] * Hkv + g) * 256;
      float d = 0.f;
      for (int j = 0; j < 256; ++j) d += q[j] * half_to_float(k[j]);
      lg[t] = d * 0.0625f;
      m = lg[t] > m ? lg[t] : m;
    }
    float l = 0.f, acc[256];
    for (int j = 0; j < 256; ++j) acc[j] = 0.f;
    for (int t = 0; t < n; ++t) {
      const float e = expf(lg[t] - m);
      const uint16_t* v = vc + ((size_t)pos[t] * Hkv + g) * 256;
      l += e;
      for (int j = 0; j < 256; ++j) acc[j] += e * half_to_float(v[j]);
    }
    for (int j = 0; j < 256; ++j) out[h * 256 + j] = acc[j] / l * sigmoidf_(gate[h * 256 + j]);
    free(lg);
  }
  free(pos);
}
