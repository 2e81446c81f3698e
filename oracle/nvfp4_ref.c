/*
 * CPU restatement in C (pthreads) of the reference's NVFP4 weight quantisation — TEST / BASELINE
 * INFRASTRUCTURE, never linked into the product.  It follows the torch path of
 * NVFP4QTensor.quantize (modelopt/torch/quantization/qtensor/nvfp4_tensor.py:62-97,119-232) step
 * by step in IEEE float arithmetic, fused into one pass per 16-element block, and is checked
 * against the numpy oracle (and through it against the reference's golden vectors) by
 * tests/test_oracle_golden.py.  bench.py times it on the host cores as the CPU baseline.
 *
 * Build: make -C oracle   (gcc -O2 -pthread, no fast-math)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* torch's float32 -> float8_e4m3fn cast for a >= 0: round-to-nearest-even, 448 up to 464,
 * above that (and NaN) the NaN code (nvfp4_tensor.py:91) */
static inline uint8_t e4m3_from_f32_torch(float a) {
  if (!(a <= 464.0f)) return 0x7F;
  if (a < 0.015625f) return (uint8_t)nearbyintf(a * 512.0f); /* subnormals: multiples of 2^-9 */
  uint32_t u;
  memcpy(&u, &a, 4);
  uint32_t r = u + 0x7FFFFu + ((u >> 20) & 1u);
  uint32_t code = (r >> 20) - ((127u - 7u) << 3);
  return (uint8_t)(code > 0x7Eu ? 0x7Eu : code);
}

static inline float e4m3_to_f32(uint8_t c) {
  if ((c & 0x7F) == 0x7F) return NAN;
  int e = (c >> 3) & 0xF, m = c & 7;
  float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (c & 0x80) ? -v : v;
}

/* _cast_fp4 (nvfp4_tensor.py:119-140): sign from v < 0, ordinal = bounds below |v|, +1 on the
 * ties 0.75 / 1.75 / 3.5; NaN sorts past every bound */
static inline uint8_t e2m1_code(float v) {
  static const float b[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  uint8_t sign = v < 0.0f ? 8 : 0;
  float a = fabsf(v);
  uint8_t ord = 0;
  if (a != a) ord = 7;
  else
    for (int i = 0; i < 7; ++i) ord += (b[i] < a);
  if (a == 0.75f || a == 1.75f || a == 3.5f) ord += 1;
  return (uint8_t)(sign + ord);
}

/* ---- a minimal parallel-for over [0, n) with POSIX threads ---------------------------------- */
typedef void (*range_fn)(int64_t lo, int64_t hi, int tid, void* ctx);
typedef struct { range_fn fn; int64_t lo, hi; int tid; void* ctx; } job_t;
static void* job_main(void* p) {
  job_t* j = (job_t*)p;
  j->fn(j->lo, j->hi, j->tid, j->ctx);
  return 0;
}
#define MAX_THREADS 256
static void parallel_for(int64_t n, int nthreads, range_fn fn, void* ctx) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > MAX_THREADS) nthreads = MAX_THREADS;
  pthread_t th[MAX_THREADS];
  job_t jobs[MAX_THREADS];
  int64_t per = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    int64_t lo = t * per, hi = lo + per > n ? n : lo + per;
    if (lo > n) lo = n;
    jobs[t] = (job_t){fn, lo, hi, t, ctx};
    if (t > 0) pthread_create(&th[t], 0, job_main, &jobs[t]);
  }
  job_main(&jobs[0]);
  for (int t = 1; t < nthreads; ++t) pthread_join(th[t], 0);
}

/* abs-max of n bf16 values as float (reduce_amax, utils.py:155-188) */
typedef struct { const uint16_t* x; float part[MAX_THREADS]; } amax_ctx;
static void amax_range(int64_t lo, int64_t hi, int tid, void* p) {
  amax_ctx* c = (amax_ctx*)p;
  float m = 0.0f;
  for (int64_t i = lo; i < hi; ++i) {
    float a = fabsf(bf16_to_f32(c->x[i]));
    if (a > m) m = a;
  }
  c->part[tid] = m;
}
float nvfp4_ref_amax_bf16(const uint16_t* x, int64_t n, int nthreads) {
  amax_ctx c;
  c.x = x;
  for (int t = 0; t < MAX_THREADS; ++t) c.part[t] = 0.0f;
  parallel_for(n, nthreads, amax_range, &c);
  float m = 0.0f;
  for (int t = 0; t < MAX_THREADS; ++t)
    if (c.part[t] > m) m = c.part[t];
  return m;
}

typedef struct { const uint16_t* x; uint8_t* packed; uint8_t* scales; float s2, c; } quant_ctx;
static void quant_range(int64_t lo, int64_t hi, int tid, void* ptr) {
  (void)tid;
  quant_ctx* q = (quant_ctx*)ptr;
  for (int64_t b = lo; b < hi; ++b) {
    const uint16_t* p = q->x + 16 * b;
    float f[16], bamax = 0.0f;
    for (int i = 0; i < 16; ++i) {
      f[i] = bf16_to_f32(p[i]);
      float a = fabsf(f[i]);
      if (a > bamax) bamax = a;
    }
    float t = bamax / q->c;
    if (t == 0.0f) t = 1.0f;
    const uint8_t sc = e4m3_from_f32_torch(t);
    q->scales[b] = sc;
    const float d = e4m3_to_f32(sc) * q->s2;
    for (int j = 0; j < 8; ++j) {
      uint8_t l = e2m1_code(f[2 * j] / d), h = e2m1_code(f[2 * j + 1] / d);
      q->packed[8 * b + j] = (uint8_t)((h << 4) | l);
    }
  }
}

/* x: nblocks*16 bf16 values; packed: nblocks*8 bytes; scales: nblocks E4M3 codes.
 * amax < 0 means "take the tensor's own abs-max".  Returns weights_scaling_factor_2. */
float nvfp4_ref_quantize_bf16(const uint16_t* x, int64_t nblocks, float amax, uint8_t* packed,
                              uint8_t* scales, int nthreads) {
  if (amax < 0.0f) amax = nvfp4_ref_amax_bf16(x, nblocks * 16, nthreads);
  quant_ctx q = {x, packed, scales, amax / 2688.0f, 0.0f};
  q.c = 6.0f * q.s2;
  parallel_for(nblocks, nthreads, quant_range, &q);
  return q.s2;
}
