/*
 * CPU oracle for the UltraQuant FP4 paged verify-attention path.  TEST INFRASTRUCTURE ONLY:
 * the tests, the smoke check and the CPU-baseline leg of the benchmark link this file; the
 * product library never does.
 *
 * It restates, in plain C, the reference's CPU algorithm (reference file:line given at each
 * function).  Parity is pinned: this file reproduces the reference's frozen vectors
 * (cuda/vectors, sycl/vectors: attention outputs; cuda/vectors cache bytes: encoder) and the
 * fixtures generated from the reference's own Python functions (see tests/golden/).
 *
 * Build: make -C oracle      ->  oracle/libuq_oracle.so
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* e2m1 magnitudes, code & 7 -> value (uqmt/attn.py:46) */
static const float kGrid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

int uqo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of threads the parallel loops below use from now on (n < 1: every processor of the machine).  A launcher may
 * have set OMP_NUM_THREADS=1 for its workers (torch.distributed.run does): the benchmark's CPU arm calls this so that its
 * figure is for all host cores whoever started it.  Returns the count in effect. */
int uqo_set_threads(int n) {
#ifdef _OPENMP
  if (n < 1) n = omp_get_num_procs();
  omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/*
 * Encoder for one group of 32 values (uqmt/attn.py:52-66, frozen twin tools/gen_vectors.py:18-30).
 *   amax  = max |x| clamped below at 1e-30
 *   e     = clamp(ceil(log2(amax / 6)), -127, 127), all in fp32.  log2 is evaluated as the
 *           correctly rounded fp32 value (double log2 rounded to float), which is what the
 *           reference's torch CPU kernel returns on every probed point.
 *   y     = clamp(x / 2^e, -6, 6)
 *   code  = FIRST index minimising | |y| - grid[i] |  (ties go to the smaller magnitude),
 *           OR-ed with 8 when y < 0 (so -0.0 has no sign bit, but a negative value that
 *           rounds to magnitude 0 keeps it: nibble 0x8)
 *   byte  = e + 127
 * Packing: low nibble = even element.
 */
static void encode_group_rule(const float* x, uint8_t* packed16, uint8_t* scale, int rule, float c) {
  float amax = 0.0f;
  for (int i = 0; i < 32; i++) {
    float a = fabsf(x[i]);
    if (a > amax) amax = a;
  }
  if (!(amax >= 1e-30f)) amax = 1e-30f;
  float e;
  if (rule == 0) {
    float r = amax / 6.0f;
    e = ceilf((float)log2((double)r));
  } else {
    /* 'paper' rule (uqmt/quant.py:52-60): round(log2(c * amax)), torch.round = half to even; values then clip at +-6 */
    float r = c * amax;
    e = rintf((float)log2((double)r));
  }
  if (e < -127.0f) e = -127.0f;
  if (e > 127.0f) e = 127.0f;
  float sc = (float)ldexp(1.0, (int)e); /* exp2(e) in fp32; 2^-127 is a representable denormal */
  uint8_t codes[32];
  for (int i = 0; i < 32; i++) {
    float y = x[i] / sc;
    if (y < -6.0f) y = -6.0f;
    if (y > 6.0f) y = 6.0f;
    float a = fabsf(y);
    int best = 0;
    float bd = fabsf(a - kGrid[0]);
    for (int c = 1; c < 8; c++) {
      float d = fabsf(a - kGrid[c]);
      if (d < bd) { bd = d; best = c; }
    }
    codes[i] = (uint8_t)(best | ((y < 0.0f) ? 8 : 0));
  }
  for (int i = 0; i < 16; i++) packed16[i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
  *scale = (uint8_t)((int)e + 127);
}

static void encode_group(const float* x, uint8_t* packed16, uint8_t* scale) { encode_group_rule(x, packed16, scale, 0, 0.0f); }

/* The configurable quantiser (uqmt/quant.py:63-70 quantize): rule 0 = 'ceil' (the cache's own encoder), 1 = 'paper' with constant c. */
void uqo_quantize_rule(const float* x, size_t n_groups, int rule, float c, uint8_t* packed, uint8_t* scales) {
#pragma omp parallel for schedule(static)
  for (long long g = 0; g < (long long)n_groups; g++) encode_group_rule(x + g * 32, packed + g * 16, scales + g, rule, c);
}

/* Orthonormal fast Walsh-Hadamard transform of each row of n values, n a power of two (uqmt/quant.py:84-98 fwht): stages
 * h = 1, 2, 4, ...: within blocks of 2h, (a, b) = (x[i], x[i + h]) -> (a + b, a - b); then every value divided by
 * (float)sqrt(n), all in fp32. */
void uqo_fwht(const float* x, size_t rows, int n, float* out) {
  const float div = (float)sqrt((double)n);
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < (long long)rows; r++) {
    float* y = out + r * n;
    memcpy(y, x + r * n, sizeof(float) * (size_t)n);
    for (int h = 1; h < n; h *= 2)
      for (int b0 = 0; b0 < n; b0 += 2 * h)
        for (int i = b0; i < b0 + h; i++) {
          const float a = y[i], b = y[i + h];
          y[i] = a + b;
          y[i + h] = a - b;
        }
    for (int i = 0; i < n; i++) y[i] = y[i] / div;
  }
}

/* x: n_groups*32 floats -> packed n_groups*16 bytes, scales n_groups bytes. */
void uqo_quantize_fp4(const float* x, size_t n_groups, uint8_t* packed, uint8_t* scales) {
#pragma omp parallel for schedule(static)
  for (long long g = 0; g < (long long)n_groups; g++) encode_group(x + g * 32, packed + g * 16, scales + g);
}

/* Decoder (uqmt/attn.py:69-78): +-grid[c & 7] * 2^(s - 127); sign-bit-on-zero decodes to (-)0. */
static inline float decode_one(uint8_t nib, float sc) {
  float v = kGrid[nib & 7];
  return ((nib & 8) ? -v : v) * sc;
}
static inline float scale_of(uint8_t s) { return (float)ldexp(1.0, (int)s - 127); }

void uqo_dequantize_fp4(const uint8_t* packed, const uint8_t* scales, size_t n_groups, float* out) {
#pragma omp parallel for schedule(static)
  for (long long g = 0; g < (long long)n_groups; g++) {
    float sc = scale_of(scales[g]);
    for (int i = 0; i < 16; i++) {
      uint8_t b = packed[g * 16 + i];
      out[g * 32 + 2 * i] = decode_one(b & 0xF, sc);
      out[g * 32 + 2 * i + 1] = decode_one(b >> 4, sc);
    }
  }
}

/*
 * Append (uqmt/vllm_adapter.py:48-59): encode key/value [T,Hkv,D] and write token t at flat
 * slot = page * PAGE + offset, i.e. row ((page*Hkv + h)*PAGE + offset) of the four cache arrays.
 */
void uqo_append_kv(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const float* key, const float* value,
                   const int64_t* slots, int T, int HKV, int D, int PAGE) {
  const int ng = D / 32;
  for (int t = 0; t < T; t++) {
    int64_t pg = slots[t] / PAGE, off = slots[t] % PAGE;
    for (int h = 0; h < HKV; h++) {
      size_t row = ((size_t)pg * HKV + h) * PAGE + off;
      for (int g = 0; g < ng; g++) {
        encode_group(key + ((size_t)t * HKV + h) * D + g * 32, kc + row * (D / 2) + g * 16, ks + row * ng + g);
        encode_group(value + ((size_t)t * HKV + h) * D + g * 32, vc + row * (D / 2) + g * 16, vs + row * ng + g);
      }
    }
  }
}

static float e4m3fn_to_f32(uint8_t b);

/*
 * NVFP4 quantiser (uqmt/quant.py:125-136 quantize_nvfp4, tensor_scale given): per block of 16 values
 *   s    = e4m3fn(clamp(amax / 6 / ts, 2^-9, 448))      two fp32 divisions, round to nearest even
 *   y    = clamp(x / (float(s) * ts), -6, 6)
 *   code = nearest e2m1 value, ties to the smaller magnitude, sign bit from y < 0 (the same _encode as the UE8M0 format)
 */
static uint8_t f32_to_e4m3fn(float x) { /* 2^-9 <= x <= 448, round to nearest even */
  if (x < 0.015625f) {                  /* below the smallest normal 2^-6: multiples of 2^-9 */
    int q = (int)rintf(x * 512.0f);
    return (uint8_t)q;                  /* q = 8 is 0x08 = 2^-6 itself */
  }
  int e;
  float m = frexpf(x, &e);              /* x = m * 2^e, m in [0.5, 1) */
  int q = (int)rintf(m * 16.0f);        /* 8 .. 16 */
  e -= 1;
  if (q == 16) { q = 8; e += 1; }
  return (uint8_t)(((e + 7) << 3) | (q - 8));
}

void uqo_quantize_nvfp4(const float* x, size_t n_blocks, float ts, uint8_t* packed, uint8_t* scales) {
#pragma omp parallel for schedule(static)
  for (long long g = 0; g < (long long)n_blocks; g++) {
    const float* xb = x + g * 16;
    float amax = 0.0f;
    for (int i = 0; i < 16; i++) {
      float a = fabsf(xb[i]);
      if (a > amax) amax = a;
    }
    float r = amax / 6.0f / ts;
    if (!(r >= 0.001953125f)) r = 0.001953125f;
    if (r > 448.0f) r = 448.0f;
    const uint8_t sb = f32_to_e4m3fn(r);
    const float sf = e4m3fn_to_f32(sb) * ts;
    uint8_t codes[16];
    for (int i = 0; i < 16; i++) {
      float y = xb[i] / sf;
      if (y < -6.0f) y = -6.0f;
      if (y > 6.0f) y = 6.0f;
      float a = fabsf(y);
      int best = 0;
      float bd = fabsf(a - kGrid[0]);
      for (int c = 1; c < 8; c++) {
        float d = fabsf(a - kGrid[c]);
        if (d < bd) { bd = d; best = c; }
      }
      codes[i] = (uint8_t)(best | ((y < 0.0f) ? 8 : 0));
    }
    for (int i = 0; i < 8; i++) packed[g * 8 + i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
    scales[g] = sb;
  }
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static void decode_row(const uint8_t* codes, const uint8_t* scales, int D, float* out) {
  for (int g = 0; g < D / 32; g++) {
    float sc = scale_of(scales[g]);
    for (int i = 0; i < 16; i++) {
      uint8_t b = codes[g * 16 + i];
      out[g * 32 + 2 * i] = decode_one(b & 0xF, sc);
      out[g * 32 + 2 * i + 1] = decode_one(b >> 4, sc);
    }
  }
}

/* NVFP4 row (uqmt/quant.py:139-147 dequantize_nvfp4, uqmt/nvfp4.py:206-208): e2m1 value times
 * (e4m3fn scale of its 16-channel block, as fp32, times the per-tensor fp32 scale). */
static float e4m3fn_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
  if (e == 15 && m == 7) v = NAN;
  return (b & 0x80) ? -v : v;
}
/* All 256 e4m3fn bytes as fp32 (for the test that compares the table with torch.float8_e4m3fn). */
void uqo_e4m3fn_table(float* out256) {
  for (int b = 0; b < 256; b++) out256[b] = e4m3fn_to_f32((uint8_t)b);
}

static void decode_row_nvfp4(const uint8_t* codes, const uint8_t* scales, int D, float ts, float* out) {
  static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  for (int g = 0; g < D / 16; g++) {
    const float sc = e4m3fn_to_f32(scales[g]) * ts;
    for (int i = 0; i < 8; i++) {
      const uint8_t b = codes[g * 8 + i];
      const float lo = grid[b & 7], hi = grid[(b >> 4) & 7];
      out[g * 16 + 2 * i] = ((b & 8) ? -lo : lo) * sc;
      out[g * 16 + 2 * i + 1] = ((b & 0x80) ? -hi : hi) * sc;
    }
  }
}

/*
 * Attention oracle (uqmt/attn.py:402-422, frozen twin tools/gen_vectors.py:45-65).
 *   q bf16 bits [B,K,HQ,D]; caches as in cuda/uq_decode.h:3-6; out fp32 [B,K,HQ,D].
 *   Query j of sequence b sees lim = seq_len - K + j + 1 keys; lim <= 0 -> zero row.
 * Extension used only by the context-split tests: the sequence may be a shard that starts at
 * global position pos_offset (keys [0, n_local) of this cache are global positions
 * pos_offset .. pos_offset + n_local), in which case lim is clamped to the shard, and when
 * lse_out != NULL the natural-log sum-exp of the scaled scores over the shard is written per
 * row [B,K,HQ] (-inf for an empty row).  pos_offset = NULL, lse_out = NULL is the reference op.
 * seq_lens are always GLOBAL lengths (they include the K draft tokens).
 * n_local[b] (NULL = whole sequence) is the number of keys this cache holds for sequence b.
 */
static void reference_impl(const uint16_t* q, const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs,
                           const int32_t* block_table, const int32_t* seq_lens, const int32_t* pos_offset,
                           const int32_t* n_local, int B, int K, int HQ, int HKV, int D, int PAGE, int max_pages,
                           float sm_scale, float* out, float* lse_out, int fmt, float k_ts, float v_ts) {
  const int G = HQ / HKV, ng = fmt ? D / 16 : D / 32;
  memset(out, 0, sizeof(float) * (size_t)B * K * HQ * D);
  if (lse_out)
    for (size_t i = 0; i < (size_t)B * K * HQ; i++) lse_out[i] = -INFINITY;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; b++) {
    for (int hk = 0; hk < HKV; hk++) {
      const int n_glob = seq_lens[b];
      const int off = pos_offset ? pos_offset[b] : 0;
      int n = n_local ? n_local[b] : n_glob;
      if (n_glob <= 0 || n <= 0) continue;
      float* kd = (float*)malloc(sizeof(float) * (size_t)n * D);
      float* vd = (float*)malloc(sizeof(float) * (size_t)n * D);
      float* sc = (float*)malloc(sizeof(float) * (size_t)n);
      for (int t = 0; t < n; t++) {
        size_t row = ((size_t)block_table[(size_t)b * max_pages + t / PAGE] * HKV + hk) * PAGE + t % PAGE;
        if (fmt) {
          decode_row_nvfp4(kc + row * (D / 2), ks + row * ng, D, k_ts, kd + (size_t)t * D);
          decode_row_nvfp4(vc + row * (D / 2), vs + row * ng, D, v_ts, vd + (size_t)t * D);
        } else {
          decode_row(kc + row * (D / 2), ks + row * ng, D, kd + (size_t)t * D);
          decode_row(vc + row * (D / 2), vs + row * ng, D, vd + (size_t)t * D);
        }
      }
      for (int j = 0; j < K; j++) {
        int lim = n_glob - K + j + 1 - off;
        if (lim > n) lim = n;
        if (lim <= 0) continue;
        for (int g = 0; g < G; g++) {
          const int h = hk * G + g;
          const uint16_t* qr = q + (((size_t)b * K + j) * HQ + h) * D;
          float qf[512];
          for (int d = 0; d < D; d++) qf[d] = bf16_to_f32(qr[d]);
          float mx = -INFINITY;
          for (int t = 0; t < lim; t++) {
            double acc = 0.0;
            const float* kr = kd + (size_t)t * D;
            for (int d = 0; d < D; d++) acc += (double)qf[d] * (double)kr[d];
            float s = (float)acc * sm_scale;
            sc[t] = s;
            if (s > mx) mx = s;
          }
          double l = 0.0;
          for (int t = 0; t < lim; t++) {
            float p = expf(sc[t] - mx);
            sc[t] = p;
            l += p;
          }
          float* o = out + (((size_t)b * K + j) * HQ + h) * D;
          double od[512];
          for (int d = 0; d < D; d++) od[d] = 0.0;
          for (int t = 0; t < lim; t++) {
            const float* vr = vd + (size_t)t * D;
            const double p = sc[t];
            for (int d = 0; d < D; d++) od[d] += p * (double)vr[d];
          }
          for (int d = 0; d < D; d++) o[d] = (float)(od[d] / l);
          if (lse_out) lse_out[((size_t)b * K + j) * HQ + h] = mx + (float)log(l);
        }
      }
      free(kd);
      free(vd);
      free(sc);
    }
  }
}

void uqo_reference(const uint16_t* q, const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs,
                   const int32_t* block_table, const int32_t* seq_lens, const int32_t* pos_offset,
                   const int32_t* n_local, int B, int K, int HQ, int HKV, int D, int PAGE, int max_pages,
                   float sm_scale, float* out, float* lse_out) {
  reference_impl(q, kc, ks, vc, vs, block_table, seq_lens, pos_offset, n_local, B, K, HQ, HKV, D, PAGE, max_pages, sm_scale, out,
                 lse_out, 0, 1.0f, 1.0f);
}

/* NVFP4 attention oracle (uqmt/nvfp4.py:257-278 reference_nvfp4): scale bytes e4m3fn [pages,Hkv,PAGE,D/16], per-tensor
 * fp32 scales k_ts / v_ts; dequantise, then the same attention as above. */
void uqo_reference_nvfp4(const uint16_t* q, const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs,
                         const int32_t* block_table, const int32_t* seq_lens, int B, int K, int HQ, int HKV, int D, int PAGE,
                         int max_pages, float sm_scale, float k_ts, float v_ts, float* out) {
  reference_impl(q, kc, ks, vc, vs, block_table, seq_lens, NULL, NULL, B, K, HQ, HKV, D, PAGE, max_pages, sm_scale, out, NULL, 1,
                 k_ts, v_ts);
}

/*
 * Tree-masked attention oracle (uqmt/tree.py:169-201).  Same caches and conventions as uqo_reference; the
 * K draft tokens of sequence b sit at positions seq_len-K .. seq_len-1.  Query j sees every position
 * below seq_len-K, and draft token t (position seq_len-K+t) iff bit t of tree_mask[b*K+j] is set.
 * tree_mask = NULL is the chain mask (bit t set for t <= j): the ordinary causal op.  A row that sees
 * nothing is zeros.
 */
void uqo_tree_reference(const uint16_t* q, const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs,
                        const int32_t* block_table, const int32_t* seq_lens, const int32_t* tree_mask, int B, int K,
                        int HQ, int HKV, int D, int PAGE, int max_pages, float sm_scale, float* out) {
  const int G = HQ / HKV, ng = D / 32;
  memset(out, 0, sizeof(float) * (size_t)B * K * HQ * D);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; b++) {
    for (int hk = 0; hk < HKV; hk++) {
      const int n = seq_lens[b];
      if (n <= 0) continue;
      float* kd = (float*)malloc(sizeof(float) * (size_t)n * D);
      float* vd = (float*)malloc(sizeof(float) * (size_t)n * D);
      float* sc = (float*)malloc(sizeof(float) * (size_t)n);
      unsigned char* vis = (unsigned char*)malloc((size_t)n);
      for (int t = 0; t < n; t++) {
        size_t row = ((size_t)block_table[(size_t)b * max_pages + t / PAGE] * HKV + hk) * PAGE + t % PAGE;
        decode_row(kc + row * (D / 2), ks + row * ng, D, kd + (size_t)t * D);
        decode_row(vc + row * (D / 2), vs + row * ng, D, vd + (size_t)t * D);
      }
      const int prefix = n - K;
      for (int j = 0; j < K; j++) {
        const uint32_t m = tree_mask ? (uint32_t)tree_mask[(size_t)b * K + j] : ((2u << j) - 1u);
        int any = 0;
        for (int t = 0; t < n; t++) {
          vis[t] = t < prefix || (t >= prefix && ((m >> (t - prefix)) & 1u));
          any |= vis[t];
        }
        if (!any) continue;
        for (int g = 0; g < G; g++) {
          const int h = hk * G + g;
          const uint16_t* qr = q + (((size_t)b * K + j) * HQ + h) * D;
          float qf[512];
          for (int d = 0; d < D; d++) qf[d] = bf16_to_f32(qr[d]);
          float mx = -INFINITY;
          for (int t = 0; t < n; t++) {
            if (!vis[t]) continue;
            double acc = 0.0;
            const float* kr = kd + (size_t)t * D;
            for (int d = 0; d < D; d++) acc += (double)qf[d] * (double)kr[d];
            float sv = (float)acc * sm_scale;
            sc[t] = sv;
            if (sv > mx) mx = sv;
          }
          double l = 0.0;
          double od[512];
          for (int d = 0; d < D; d++) od[d] = 0.0;
          for (int t = 0; t < n; t++) {
            if (!vis[t]) continue;
            const double p = expf(sc[t] - mx);
            l += p;
            const float* vr = vd + (size_t)t * D;
            for (int d = 0; d < D; d++) od[d] += p * (double)vr[d];
          }
          float* o = out + (((size_t)b * K + j) * HQ + h) * D;
          for (int d = 0; d < D; d++) o[d] = (float)(od[d] / l);
        }
      }
      free(kd);
      free(vd);
      free(sc);
      free(vis);
    }
  }
}

/*
 * Merge of context-split partials (no reference twin; same math as the reference's in-GPU
 * split-KV combine, cuda/uq_decode.cu:353-388, in natural-log domain):
 *   out = sum_r exp(lse_r - max) * o_r / sum_r exp(lse_r - max);  all-(-inf) row -> 0.
 * o [R,rows,D], lse [R,rows] -> out [rows,D].
 */
void uqo_merge(const float* o, const float* lse, int R, size_t rows, int D, float* out) {
  for (size_t i = 0; i < rows; i++) {
    float mx = -INFINITY;
    for (int r = 0; r < R; r++)
      if (lse[(size_t)r * rows + i] > mx) mx = lse[(size_t)r * rows + i];
    for (int d = 0; d < D; d++) out[i * D + d] = 0.0f;
    if (mx == -INFINITY) continue;
    double den = 0.0;
    for (int r = 0; r < R; r++) den += exp((double)lse[(size_t)r * rows + i] - mx);
    for (int r = 0; r < R; r++) {
      double w = exp((double)lse[(size_t)r * rows + i] - mx) / den;
      if (w == 0.0) continue;
      for (int d = 0; d < D; d++) out[i * D + d] += (float)(w * o[((size_t)r * rows + i) * D + d]);
    }
  }
}
