/* CPU oracle of the fused weight-gradient + optimizer path.  TEST INFRASTRUCTURE ONLY: it is the
 * checker for tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg; nothing in the
 * product (forge_b200/) links, imports or executes it.
 *
 * It restates, in scalar C with one IEEE fp32 rounding per operation (build with
 * -ffp-contract=off, no fast-math), the arithmetic of the reference's kernels:
 *   gradient      g[v,h] = sum_bt dY[bt,v] X[bt,h], fp32 accumulation, ascending bt
 *                 (src/fused_grad_optimizer/kernel.py:267-290)
 *   AdamW         src/fused_grad_optimizer/kernel.py:300-317
 *   SGD           src/fused_grad_optimizer/kernel.py:203-205
 *   int8 moments  src/fused_grad_optimizer/kernel.py:410-478 (dequantise, v floor 1e-8, per-(row,
 *                 64-column) absmax scale = absmax/127 + 1e-12, code = clamp(rint(x/scale), +-127)),
 *                 and the quantiser restated in tests/test_correctness.py:170-180
 *   fp8 moments   src/fused_grad_optimizer/kernel_fp8_state.py:272-295 (e4m3 m, e5m2 v, one scale
 *                 per tensor, clamp then round-to-nearest-even cast, running absmax of the
 *                 unquantised values), scale promotion src/fused_grad_optimizer/state.py:132-157
 * Scalars are fp32 kernel arguments in the reference; bias corrections are evaluated in double
 * (kernel.py:1367-1368) and narrowed.  Pinned by tests/golden (see tests/golden/make_golden.py).
 *
 * Not in the reference (parity unpinned by it, defined here): SGD with momentum (buffer semantics of
 * torch.optim.SGD with dampening 0, decoupled decay as in the reference's SGD), Lion (published
 * rule), e4m3 moments with per-block scales (the int8 scheme with scale = absmax/448 + 1e-12).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* Every scalar is what the reference's kernel receives: an fp32 narrowing of a Python double.
 * one_m_beta1/2 and decay are 1-beta and 1-lr*wd evaluated in double FIRST and then narrowed, as in
 * the reference's PyTorch checker (tests/test_correctness.py:43-44,52: `alpha=1 - beta1`,
 * `mul_(1.0 - lr * weight_decay)`) and as the Triton interpreter evaluates kernel.py:303-311. */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, momentum;
  float one_m_beta1, one_m_beta2, decay;
  int nesterov;
} OracleHyper;

/* ---- storage formats ------------------------------------------------------------------------ */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16 (round to nearest even) -> fp32 */
float oracle_round_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7F800000u) == 0x7F800000u) return u2f((u & 0xFFFF0000u) | ((u & 0xFFFFu) ? 0x00400000u : 0u));
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u2f(u & 0xFFFF0000u);
}

/* generic small-float decode: `eb` exponent bits, `mb` mantissa bits, bias, finite-only top (e4m3fn) */
static float fp8_decode(uint8_t c, int eb, int mb, int bias, int fn) {
  const int sign = c >> 7;
  const int e = (c >> mb) & ((1 << eb) - 1);
  const int m = c & ((1 << mb) - 1);
  float v;
  if (e == 0) {
    v = ldexpf((float)m, 1 - bias - mb);
  } else if (!fn && e == (1 << eb) - 1) {
    v = m ? NAN : INFINITY;
  } else if (fn && e == (1 << eb) - 1 && m == (1 << mb) - 1) {
    v = NAN;
  } else {
    v = ldexpf((float)((1 << mb) + m), e - bias - mb);
  }
  return sign ? -v : v;
}

float oracle_e4m3_to_float(uint8_t c) { return fp8_decode(c, 4, 3, 7, 1); }
float oracle_e5m2_to_float(uint8_t c) { return fp8_decode(c, 5, 2, 15, 0); }

/* encode a FINITE value already clamped to the format's range; round to nearest even */
static uint8_t fp8_encode(float x, int eb, int mb, int bias, float maxv) {
  const uint8_t sign = signbit(x) ? 0x80u : 0u;
  float a = fabsf(x);
  if (isnan(a)) return (uint8_t)(sign | 0x7Fu);
  if (a > maxv) a = maxv;
  if (a == 0.0f) return sign;
  int e;
  (void)frexpf(a, &e);          /* a = f * 2^e, f in [0.5,1)  -> unbiased exponent e-1 */
  int ue = e - 1;
  if (ue < 1 - bias) ue = 1 - bias; /* subnormal range shares the minimum exponent */
  /* quantum of this binade */
  const float q = ldexpf(1.0f, ue - mb);
  float n = rintf(a / q);       /* exact: a/q is a/2^k; rintf = half-to-even */
  int mant = (int)n;            /* in [0, 2^(mb+1)] */
  int be = ue + bias;           /* biased exponent, 1.. for normals */
  if (ue == 1 - bias && mant < (1 << mb)) {
    be = 0;                     /* subnormal */
  } else {
    if (mant >= (2 << mb)) { mant >>= 1; be += 1; }
    mant -= (1 << mb);
  }
  uint8_t code = (uint8_t)(sign | (be << mb) | mant);
  (void)eb;
  return code;
}

uint8_t oracle_float_to_e4m3(float x) {
  float c = fminf(fmaxf(x, -448.0f), 448.0f);
  return fp8_encode(c, 4, 3, 7, 448.0f);
}
uint8_t oracle_float_to_e5m2(float x) {
  float c = fminf(fmaxf(x, -57344.0f), 57344.0f);
  return fp8_encode(c, 5, 2, 15, 57344.0f);
}

/* ---- gradient ------------------------------------------------------------------------------- */
void oracle_wgrad(const float* dy, const float* x, long BT, long V, long H, float* g) {
#pragma omp parallel for schedule(static)
  for (long v = 0; v < V; ++v) {
    float* row = g + v * H;
    for (long h = 0; h < H; ++h) row[h] = 0.0f;
    for (long bt = 0; bt < BT; ++bt) {
      const float a = dy[bt * V + v];
      const float* xr = x + bt * H;
      for (long h = 0; h < H; ++h) {
        const float prod = a * xr[h];
        row[h] = row[h] + prod;
      }
    }
  }
}

/* ---- per-element updates --------------------------------------------------------------------- */
static inline float adamw_elem(float w, float g, float* m, float* v, const OracleHyper* h) {
  const float one_m_b1 = h->one_m_beta1;
  const float one_m_b2 = h->one_m_beta2;
  const float mn = h->beta1 * (*m) + one_m_b1 * g;
  const float t = one_m_b2 * g;
  const float vn = h->beta2 * (*v) + t * g;
  const float m_hat = mn / h->bc1;
  const float v_hat = vn / h->bc2;
  const float w1 = w * h->decay;
  const float num = h->lr * m_hat;
  const float den = sqrtf(v_hat) + h->eps;
  *m = mn;
  *v = vn;
  return w1 - num / den;
}

static inline float store_round(float x, int is_bf16) { return is_bf16 ? oracle_round_bf16(x) : x; }

/* AdamW with fp32 or bf16 moments; arrays hold the stored values widened to fp32 */
void oracle_adamw(float* w, float* m, float* v, const float* g, long n, const OracleHyper* h,
                  int w_bf16, int s_bf16) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    float mm = m[i], vv = v[i];
    const float wn = adamw_elem(w[i], g[i], &mm, &vv, h);
    w[i] = store_round(wn, w_bf16);
    m[i] = store_round(mm, s_bf16);
    v[i] = store_round(vv, s_bf16);
  }
}

void oracle_sgd(float* w, const float* g, long n, const OracleHyper* h, int w_bf16) {
  const float decay = h->decay;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const float a = w[i] * decay;
    const float b = h->lr * g[i];
    w[i] = store_round(a - b, w_bf16);
  }
}

void oracle_sgdm(float* w, float* buf, const float* g, long n, const OracleHyper* h, int w_bf16, int s_bf16) {
  const float decay = h->decay;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const float t = h->momentum * buf[i];
    const float b = t + g[i];
    float u = b;
    if (h->nesterov) {
      const float t2 = h->momentum * b;
      u = g[i] + t2;
    }
    const float a = w[i] * decay;
    const float s = h->lr * u;
    w[i] = store_round(a - s, w_bf16);
    buf[i] = store_round(b, s_bf16);
  }
}

void oracle_lion(float* w, float* m, const float* g, long n, const OracleHyper* h, int w_bf16, int s_bf16) {
  const float decay = h->decay;
  const float one_m_b1 = h->one_m_beta1;
  const float one_m_b2 = h->one_m_beta2;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const float c1 = h->beta1 * m[i];
    const float c2 = one_m_b1 * g[i];
    const float c = c1 + c2;
    const float u = (c > 0.0f) ? 1.0f : ((c < 0.0f) ? -1.0f : 0.0f);
    const float m1 = h->beta2 * m[i];
    const float m2 = one_m_b2 * g[i];
    const float a = w[i] * decay;
    const float s = h->lr * u;
    w[i] = store_round(a - s, w_bf16);
    m[i] = store_round(m1 + m2, s_bf16);
  }
}

/* AdamW with block-quantised moments.  code_kind 0: int8 (scale = absmax/127 + 1e-12,
 * code = clamp(rint(x/scale), +-127)); 1: e4m3 (scale = absmax/448 + 1e-12, code = e4m3(x/scale)). */
void oracle_adamw_blockq(float* w, uint8_t* mq, uint8_t* vq, float* ms, float* vs, const float* g,
                         long V, long H, long qblock, const OracleHyper* h, int w_bf16, int code_kind) {
  const long nb = H / qblock;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < V; ++r) {
    float mbuf[256], vbuf[256];
    for (long b = 0; b < nb; ++b) {
      const float sm = ms[r * nb + b], sv = vs[r * nb + b];
      float am = 0.0f, av = 0.0f;
      for (long k = 0; k < qblock; ++k) {
        const long i = r * H + b * qblock + k;
        float m, v;
        if (code_kind == 0) {
          m = (float)(int8_t)mq[i] * sm;
          v = fmaxf((float)(int8_t)vq[i] * sv, 1e-8f);
        } else {
          m = oracle_e4m3_to_float(mq[i]) * sm;
          v = fmaxf(oracle_e4m3_to_float(vq[i]) * sv, 1e-8f);
        }
        const float wn = adamw_elem(w[i], g[i], &m, &v, h);
        w[i] = store_round(wn, w_bf16);
        mbuf[k] = m;
        vbuf[k] = v;
        am = fmaxf(am, fabsf(m));
        av = fmaxf(av, fabsf(v));
      }
      const float div = code_kind == 0 ? 127.0f : 448.0f;
      const float smn = am / div + 1e-12f;
      const float svn = av / div + 1e-12f;
      ms[r * nb + b] = smn;
      vs[r * nb + b] = svn;
      for (long k = 0; k < qblock; ++k) {
        const long i = r * H + b * qblock + k;
        if (code_kind == 0) {
          float qm = rintf(mbuf[k] / smn), qv = rintf(vbuf[k] / svn);
          qm = fminf(fmaxf(qm, -127.0f), 127.0f);
          qv = fminf(fmaxf(qv, -127.0f), 127.0f);
          mq[i] = (uint8_t)(int8_t)(int)qm;
          vq[i] = (uint8_t)(int8_t)(int)qv;
        } else {
          mq[i] = oracle_float_to_e4m3(mbuf[k] / smn);
          vq[i] = oracle_float_to_e4m3(vbuf[k] / svn);
        }
      }
    }
  }
}

/* AdamW with e4m3 m / e5m2 v and one scale per tensor; amax_* accumulate max|m'|, max|v'| */
void oracle_adamw_fp8tensor(float* w, uint8_t* m8, uint8_t* v8, float s_m, float s_v, float* amax_m,
                            float* amax_v, const float* g, long n, const OracleHyper* h, int w_bf16) {
  const float inv_m = 1.0f / s_m, inv_v = 1.0f / s_v;
  float am = *amax_m, av = *amax_v;
  for (long i = 0; i < n; ++i) {
    float m = oracle_e4m3_to_float(m8[i]) * s_m;
    float v = oracle_e5m2_to_float(v8[i]) * s_v;
    const float wn = adamw_elem(w[i], g[i], &m, &v, h);
    w[i] = store_round(wn, w_bf16);
    am = fmaxf(am, fabsf(m));
    av = fmaxf(av, fabsf(v));
    m8[i] = oracle_float_to_e4m3(m * inv_m);
    v8[i] = oracle_float_to_e5m2(v * inv_v);
  }
  *amax_m = am;
  *amax_v = av;
}

/* state.py:132-157: scale <- clamp(absmax_next, 1e-8)/MAX, capped at 2x the previous scale */
void oracle_fp8_prestep(float* s_m, float* s_v, float* amax_m, float* amax_v) {
  float mn = fmaxf(*amax_m, 1e-8f) / 448.0f;
  float vn = fmaxf(*amax_v, 1e-8f) / 57344.0f;
  if (*s_m > 0.0f) mn = fminf(mn, *s_m * 2.0f);
  if (*s_v > 0.0f) vn = fminf(vn, *s_v * 2.0f);
  *s_m = mn;
  *s_v = vn;
  *amax_m = 0.0f;
  *amax_v = 0.0f;
}

/* int8 quantiser on its own (tests/test_correctness.py:170-180) */
void oracle_int8_quantise(const float* x, long V, long H, long qblock, uint8_t* q, float* scale) {
  const long nb = H / qblock;
  for (long r = 0; r < V; ++r)
    for (long b = 0; b < nb; ++b) {
      float am = 0.0f;
      for (long k = 0; k < qblock; ++k) am = fmaxf(am, fabsf(x[r * H + b * qblock + k]));
      const float s = am / 127.0f + 1e-12f;
      scale[r * nb + b] = s;
      for (long k = 0; k < qblock; ++k) {
        float c = rintf(x[r * H + b * qblock + k] / s);
        c = fminf(fmaxf(c, -127.0f), 127.0f);
        q[r * H + b * qblock + k] = (uint8_t)(int8_t)(int)c;
      }
    }
}
