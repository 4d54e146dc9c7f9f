/*
 * Scalar C restatement of the compressed-KV hot path (TEST INFRASTRUCTURE, not product
 * code).  It states, loop by loop, the arithmetic order the CUDA kernels must reproduce
 * and doubles as the multi-threaded CPU baseline that bench.py times.  Only tests/,
 * __graft_entry__.smoke() and bench.py's CPU legs may load the library built from it.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -pthread -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference's numpy path never fuses multiply and add.
 *
 * Parity is pinned by tests/test_oracle_c.py against fixtures produced by the reference.
 *
 * Reference locations restated (paths inside the reference project):
 *   key encoder      turboquant_pro/per_channel_kv.py:269-283, 324-353, 377-383
 *   key decoder      turboquant_pro/per_channel_kv.py:503-539
 *   value encoder    turboquant_pro/core.py:562-593   (norm, unit vector, rotation, bins)
 *   value decoder    turboquant_pro/core.py:645-652
 *   attention        tests/test_kv_fused_pck.py:202-208 (softmax(qK^T/sqrt d)V in fp32)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

static const float NF4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

/* ---- minimal pthread parallel-for (the image has no OpenMP runtime) ---------------- */
typedef void (*tqo_body)(int i, void* ctx);
typedef struct { tqo_body fn; void* ctx; int lo, hi; } tqo_span;

static void* tqo_worker(void* p) {
  tqo_span* s = (tqo_span*)p;
  for (int i = s->lo; i < s->hi; ++i) s->fn(i, s->ctx);
  return NULL;
}

/* Worker threads used: TQO_THREADS if set, else the online core count. */
int tqo_num_threads(void) {
  const char* e = getenv("TQO_THREADS");
  long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
  if (n < 1) n = 1;
  if (n > 256) n = 256;
  return (int)n;
}

static void parallel_for(int n, tqo_body fn, void* ctx) {
  int nt = tqo_num_threads();
  if (nt > n) nt = n;
  if (nt <= 1) {
    for (int i = 0; i < n; ++i) fn(i, ctx);
    return;
  }
  pthread_t th[256];
  tqo_span sp[256];
  for (int t = 0; t < nt; ++t) {
    sp[t].fn = fn;
    sp[t].ctx = ctx;
    sp[t].lo = (int)((long)n * t / nt);
    sp[t].hi = (int)((long)n * (t + 1) / nt);
    pthread_create(&th[t], NULL, tqo_worker, &sp[t]);
  }
  for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
}

static uint16_t f32_to_f16_bits(float f) {
  _Float16 h = (_Float16)f; /* round-to-nearest-even */
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

static float f16_bits_to_f32(uint16_t b) {
  _Float16 h;
  memcpy(&h, &b, 2);
  return (float)h;
}

static int cmp_float(const void* a, const void* b) {
  float x = *(const float*)a, y = *(const float*)b;
  return (x > y) - (x < y);
}

/* ---- keys ---------------------------------------------------------------------------- */
typedef struct {
  const float* x;
  int H, S, D, k_out;
  uint8_t* codes;
  float *scale, *mean, *kth;
} key_ctx;

/* One (head, channel) column of a key block.
 * mean   = (((x0 + x1) + x2) + ...) / S            sequential float32 sum over tokens
 * scale  = max(max_s |x - mean|, 1e-8)
 * level  = fl(mean + fl(scale * NF4[l]));  code = first l minimising |fl(x - level_l)|
 * kth    = k-th largest |x| of the column (the outlier threshold)                      */
static void key_channel(int hd, void* p) {
  key_ctx* c = (key_ctx*)p;
  int S = c->S, D = c->D;
  int h = hd / D, d = hd % D;
  const float* col = c->x + (size_t)h * S * D + d;
  float acc = col[0];
  for (int s = 1; s < S; ++s) acc = acc + col[(size_t)s * D];
  float mu = acc / (float)S;
  float amax = 0.0f;
  for (int s = 0; s < S; ++s) {
    float a = fabsf(col[(size_t)s * D] - mu);
    if (a > amax) amax = a;
  }
  if (amax < 1e-8f) amax = 1e-8f;
  float lev[16];
  for (int l = 0; l < 16; ++l) {
    float t = amax * NF4[l];
    lev[l] = mu + t;
  }
  for (int s = 0; s < S; ++s) {
    float v = col[(size_t)s * D];
    int best = 0;
    float bd = fabsf(v - lev[0]);
    for (int l = 1; l < 16; ++l) {
      float dd = fabsf(v - lev[l]);
      if (dd < bd) { bd = dd; best = l; }
    }
    c->codes[((size_t)h * S + s) * D + d] = (uint8_t)best;
  }
  c->scale[hd] = amax;
  c->mean[hd] = mu;
  if (c->k_out > 0) {
    if (c->k_out >= S) {
      c->kth[hd] = -1.0f; /* everything is kept */
    } else {
      float* tmp = (float*)malloc(sizeof(float) * S);
      for (int s = 0; s < S; ++s) tmp[s] = fabsf(col[(size_t)s * D]);
      qsort(tmp, S, sizeof(float), cmp_float);
      c->kth[hd] = tmp[S - c->k_out];
      free(tmp);
    }
  }
}

/* Per-channel asymmetric NF4 encoder for one block x[H][S][D].  Outliers: k_out entries
 * per channel by magnitude plus everything tied with the k-th, listed in ascending flat
 * index ((h*S + s)*D + d) with the fp16-rounded value.  Returns the number of outliers,
 * or -1 if out_cap is too small.                                                        */
int tqo_encode_keys(const float* x, int H, int S, int D, int k_out, uint8_t* codes,
                    float* scale, float* mean, int32_t* out_idx, uint16_t* out_val,
                    int out_cap) {
  float* kth = (float*)malloc(sizeof(float) * (size_t)H * D);
  key_ctx kc = {x, H, S, D, k_out, codes, scale, mean, kth};
  parallel_for(H * D, key_channel, &kc);
  int n = 0;
  if (k_out > 0) {
    for (int h = 0; h < H; ++h)
      for (int s = 0; s < S; ++s)
        for (int d = 0; d < D; ++d) {
          size_t i = ((size_t)h * S + s) * D + d;
          if (fabsf(x[i]) >= kth[h * D + d]) {
            if (n >= out_cap) { free(kth); return -1; }
            out_idx[n] = (int32_t)i;
            out_val[n] = f32_to_f16_bits(x[i]);
            ++n;
          }
        }
  }
  free(kth);
  return n;
}

typedef struct {
  const uint8_t* codes;
  const float *scale, *mean;
  int S, D;
  float* out;
} kdq_ctx;

static void kdq_row(int t, void* p) {
  kdq_ctx* c = (kdq_ctx*)p;
  int h = t / c->S;
  for (int d = 0; d < c->D; ++d) {
    size_t i = (size_t)t * c->D + d;
    float a = c->scale[h * c->D + d] * NF4[c->codes[i]];
    c->out[i] = a + c->mean[h * c->D + d];
  }
}

/* Key block decoder: level = fl(fl(scale*NF4[l]) + mean); outliers overwrite. */
void tqo_dequant_keys(const uint8_t* codes, const float* scale, const float* mean, int H, int S,
                      int D, const int32_t* out_idx, const uint16_t* out_val, int n_out,
                      float* out) {
  kdq_ctx c = {codes, scale, mean, S, D, out};
  parallel_for(H * S, kdq_row, &c);
  for (int e = 0; e < n_out; ++e) out[out_idx[e]] = f16_bits_to_f32(out_val[e]);
}

/* ---- values -------------------------------------------------------------------------- */

/* numpy's pairwise float32 sum. */
static float pairwise_sum(const float* a, int n) {
  if (n < 8) {
    float r = a[0];
    for (int i = 1; i < n; ++i) r = r + a[i];
    return r;
  }
  if (n <= 128) {
    float r[8];
    for (int j = 0; j < 8; ++j) r[j] = a[j];
    int full = n - (n % 8);
    for (int i = 8; i < full; i += 8)
      for (int j = 0; j < 8; ++j) r[j] = r[j] + a[i + j];
    float res = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
    for (int i = full; i < n; ++i) res = res + a[i];
    return res;
  }
  int n2 = n / 2;
  n2 -= n2 % 8;
  return pairwise_sum(a, n2) + pairwise_sum(a + n2, n - n2);
}

typedef struct {
  const float *x, *mat, *bnd, *cent, *norms_in;
  const uint8_t* codes_in;
  int D, n_bnd;
  uint8_t* codes;
  float *norms, *out;
} val_ctx;

/* One token of the PolarQuant value encoder (D <= 512).
 * norm = sqrt(pairwise sum of fl(x*x)); u = x / max(norm, 1e-30);
 * y[e] = ((fl(u0*P[0][e]) + fl(u1*P[1][e])) + ...) sequential over d, unfused;
 * code = #{ j : bnd[j] < y[e] }.                                                       */
static void venc_row(int t, void* p) {
  val_ctx* c = (val_ctx*)p;
  int D = c->D;
  const float* row = c->x + (size_t)t * D;
  float sq[512], u[512], y[512];
  for (int d = 0; d < D; ++d) sq[d] = row[d] * row[d];
  float nrm = sqrtf(pairwise_sum(sq, D));
  c->norms[t] = nrm;
  float safe = nrm > 1e-30f ? nrm : 1e-30f;
  for (int d = 0; d < D; ++d) u[d] = row[d] / safe;
  for (int e = 0; e < D; ++e) y[e] = u[0] * c->mat[e];
  for (int d = 1; d < D; ++d) {
    const float* prow = c->mat + (size_t)d * D;
    float ud = u[d];
    for (int e = 0; e < D; ++e) {
      float pr = ud * prow[e];
      y[e] = y[e] + pr;
    }
  }
  for (int e = 0; e < D; ++e) {
    int k = 0;
    for (int j = 0; j < c->n_bnd; ++j) k += (c->bnd[j] < y[e]);
    c->codes[(size_t)t * D + e] = (uint8_t)k;
  }
}

void tqo_encode_values(const float* x, int H, int S, int D, const float* pit, const float* bnd,
                       int n_bnd, uint8_t* codes, float* norms) {
  val_ctx c;
  memset(&c, 0, sizeof(c));
  c.x = x; c.mat = pit; c.bnd = bnd; c.n_bnd = n_bnd; c.D = D; c.codes = codes; c.norms = norms;
  parallel_for(H * S, venc_row, &c);
}

/* One token of the value decoder: x = (cent[code] @ Pi) * norm, sequential and unfused. */
static void vdq_row(int t, void* p) {
  val_ctx* c = (val_ctx*)p;
  int D = c->D;
  const uint8_t* cd = c->codes_in + (size_t)t * D;
  float y[512];
  float c0 = c->cent[cd[0]];
  for (int e = 0; e < D; ++e) y[e] = c0 * c->mat[e];
  for (int d = 1; d < D; ++d) {
    const float* prow = c->mat + (size_t)d * D;
    float v = c->cent[cd[d]];
    for (int e = 0; e < D; ++e) {
      float pr = v * prow[e];
      y[e] = y[e] + pr;
    }
  }
  for (int e = 0; e < D; ++e) c->out[(size_t)t * D + e] = y[e] * c->norms_in[t];
}

void tqo_dequant_values(const uint8_t* codes, const float* norms, int H, int S, int D,
                        const float* cent, const float* pi, float* out) {
  val_ctx c;
  memset(&c, 0, sizeof(c));
  c.codes_in = codes; c.norms_in = norms; c.cent = cent; c.mat = pi; c.D = D; c.out = out;
  parallel_for(H * S, vdq_row, &c);
}

/* ---- attention ----------------------------------------------------------------------- */
typedef struct {
  const float *q, *k, *v;
  int G, S, D;
  float* out;
} att_ctx;

static void att_head(int h, void* p) {
  att_ctx* c = (att_ctx*)p;
  int S = c->S, D = c->D;
  const float* kk = c->k + (size_t)(h / c->G) * S * D;
  const float* vv = c->v + (size_t)(h / c->G) * S * D;
  const float* qq = c->q + (size_t)h * D;
  float inv = 1.0f / sqrtf((float)D);
  float* sc = (float*)malloc(sizeof(float) * (S > 0 ? S : 1));
  float m = -INFINITY;
  for (int s = 0; s < S; ++s) {
    float a = 0.0f;
    for (int d = 0; d < D; ++d) a += qq[d] * kk[(size_t)s * D + d];
    sc[s] = a * inv;
    if (sc[s] > m) m = sc[s];
  }
  double den = 0.0;
  double acc[512];
  for (int d = 0; d < D; ++d) acc[d] = 0.0;
  for (int s = 0; s < S; ++s) {
    float e = expf(sc[s] - m);
    den += e;
    for (int d = 0; d < D; ++d) acc[d] += (double)e * vv[(size_t)s * D + d];
  }
  for (int d = 0; d < D; ++d) c->out[(size_t)h * D + d] = (float)(acc[d] / den);
  free(sc);
}

/* One decode step of attention: q[Hq][D], k/v[Hkv][S][D]; query head i reads KV head
 * i / (Hq/Hkv).  out[Hq][D].                                                          */
void tqo_attention(const float* q, const float* k, const float* v, int Hq, int Hkv, int S, int D,
                   float* out) {
  att_ctx c = {q, k, v, Hq / Hkv, S, D, out};
  parallel_for(Hq, att_head, &c);
}
