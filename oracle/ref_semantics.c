/* TEST INFRASTRUCTURE - not part of the product.
 *
 * CPU restatement of the reference's dot_product_attention_impl<T>
 * (src/csrc/dot_product_attention.cpp:25-198 of HPC-SJTU/af3_kernels), written from its
 * semantics, with every rounding point of the T = bfloat16 instantiation kept.  Only tests,
 * the smoke check and the CPU-baseline legs of the benchmark may call it.
 *
 * The reference's arithmetic lives in libxsmm JIT kernels (un-vendored submodule, version not
 * recoverable); the element-level behaviour restated here follows the plain-C `.ref()` bodies
 * next to each functor in src/csrc/xsmm_functors.h:
 *   ScaleTPP::ref        :1608-1613   out = (float)in * (float)(T)scale
 *   BrgemmTPP::ref       :2399-2444   fp32 accumulate, store as T
 *   AddTPP::ref          :1207-1227   out = (T)((float)a + (float)b)
 *   AddBiasTPP::ref      :1079-1085   out[r][c] += (T)in[c]
 *   SoftMaxFwdTPP::ref   :2920-2951   max, expf(x - max), sum, * (1/sum), store as T
 *   VarSoftMaxFwdTPP::ref:3314-3361   flash: carried max, un-normalised exp out
 *   SoftMaxFixUpTPP::ref :3449-3460   flash: out = exp(omax-nmax)*out + cur ; osum likewise
 *   SoftMaxFlashScaleTPP::ref :3571-3581  out *= 1/osum
 * bf16 conversion is round-to-nearest-even (:142-145).  The JIT kernels use libxsmm's own exp
 * approximation, which cannot be restated without its source: expf() stands in, so agreement
 * with the real TPP kernel is NOT pinned bit-for-bit ("parity unpinned" at that boundary).
 *
 * Interface: all tensors are fp32 arrays (bf16 inputs are widened exactly by the caller).
 *   q, k, v : [B1][B2][S][K]      bias : [B2][S][S]      keep : [B1][S] bytes, non-zero = attend
 *   out     : [B1][B2][S][K]
 * round_bf16 != 0 selects the bf16 instantiation (results are bf16-representable floats),
 * 0 selects the float instantiation (no intermediate rounding).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

int af3k_oracle_num_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

static inline float bf16_round(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return f; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&f, &u, 4);
  return f;
}
static inline float rnd(float f, int round_bf16) { return round_bf16 ? bf16_round(f) : f; }

/* One (batch i, head j, query block kb) task of the non-flash loop (:91-120). */
static void task_plain(const float* q, const float* kT, const float* v, const float* bias,
                       const float* maskadd, float* out, int S, int K, int M, int BLK, int kb,
                       int rb, float* L, float* qs) {
  const float alpha = rnd(1.0f / sqrtf((float)K), rb); /* ScaleTPP: scalar becomes T first */
  const int r0 = kb * BLK;
  for (int r = 0; r < BLK; ++r) {
    const int qr = r0 + r;
    for (int d = 0; d < K; ++d) qs[r * K + d] = qr < S ? rnd(q[qr * K + d] * alpha, rb) : 0.f;
  }
  for (int r = 0; r < BLK; ++r) {
    const int qr = r0 + r;
    float* Lr = L + (size_t)r * M;
    /* logits GEMM: fp32 accumulation over d in index order for every key; kT is K transposed
     * ([d][key]) so that the loop over keys is the contiguous, vectorisable one */
    for (int c = 0; c < M; ++c) Lr[c] = 0.f;
    for (int d = 0; d < K; ++d) {
      const float qd = qs[r * K + d];
      const float* kd = kT + (size_t)d * S;
      for (int c = 0; c < S; ++c) Lr[c] += qd * kd[c];
    }
    const float* brow = (qr < S) ? bias + (size_t)qr * S : NULL;
    for (int c = 0; c < M; ++c) {
      float x = rnd(Lr[c], rb);                                            /* logits GEMM   */
      const float b = (brow && c < S) ? brow[c] : 0.f;                     /* padded bias=0 */
      x = rnd(x + b, rb);                                                  /* AddTPP        */
      x = rnd(x + maskadd[c], rb);                                         /* AddBiasTPP    */
      Lr[c] = x;
    }
    float mx = Lr[0];
    for (int c = 1; c < M; ++c) mx = Lr[c] > mx ? Lr[c] : mx;
    float sum = 0.f;
    for (int c = 0; c < M; ++c) { Lr[c] = expf(Lr[c] - mx); sum += Lr[c]; }
    const float inv = 1.0f / sum;
    for (int c = 0; c < M; ++c) Lr[c] = rnd(Lr[c] * inv, rb);              /* SoftMaxFwdTPP */
    if (qr < S) {
      /* P V: accumulation over keys in index order for every d (padded v = 0) */
      float acc[256];
      for (int d = 0; d < K; ++d) acc[d] = 0.f;
      for (int c = 0; c < S; ++c) {
        const float pc = Lr[c];
        const float* vc = v + (size_t)c * K;
        for (int d = 0; d < K; ++d) acc[d] += pc * vc[d];
      }
      for (int d = 0; d < K; ++d) out[qr * K + d] = rnd(acc[d], rb);
    }
  }
}

/* Flash task (:148-190): keys in chunks of FLASH, running max / sum, running output kept in T. */
static void task_flash(const float* q, const float* k, const float* v, const float* bias,
                       const float* maskadd, float* out, int S, int K, int M, int BLK, int FLASH,
                       int kb, int rb, float* E, float* qs) {
  const float alpha = rnd(1.0f / sqrtf((float)K), rb);
  const int r0 = kb * BLK;
  float* acc_out = (float*)malloc(sizeof(float) * (size_t)BLK * K);
  float* cur = (float*)malloc(sizeof(float) * (size_t)K);
  for (int r = 0; r < BLK; ++r) {
    const int qr = r0 + r;
    for (int d = 0; d < K; ++d) qs[r * K + d] = qr < S ? rnd(q[qr * K + d] * alpha, rb) : 0.f;
  }
  for (int r = 0; r < BLK; ++r) {
    const int qr = r0 + r;
    float omax = 0.f, osum = 0.f;
    for (int l = 0; l < M; l += FLASH) {
      const int n = (M - l) < FLASH ? (M - l) : FLASH;
      for (int cc = 0; cc < n; ++cc) {
        const int c = l + cc;
        float a = 0.f;
        if (c < S)
          for (int d = 0; d < K; ++d) a += qs[r * K + d] * k[c * K + d];
        float x = rnd(a, rb);
        const float b = (qr < S && c < S) ? bias[(size_t)qr * S + c] : 0.f;
        x = rnd(x + b, rb);
        x = rnd(x + maskadd[c], rb);
        E[cc] = x;
      }
      float cmax = (l == 0) ? E[0] : omax; /* later chunks seed the max with the carried one */
      for (int cc = 0; cc < n; ++cc) cmax = E[cc] > cmax ? E[cc] : cmax;
      float csum = 0.f;
      for (int cc = 0; cc < n; ++cc) {
        const float z = expf(E[cc] - cmax);
        csum += z;
        E[cc] = rnd(z, rb);
      }
      for (int d = 0; d < K; ++d) {
        float a = 0.f;
        for (int cc = 0; cc < n; ++cc)
          if (l + cc < S) a += E[cc] * v[(l + cc) * K + d];
        cur[d] = rnd(a, rb);
      }
      if (l == 0) {
        for (int d = 0; d < K; ++d) acc_out[r * K + d] = cur[d];
        omax = cmax;
        osum = csum;
      } else {
        const float oexp = expf(omax - cmax);
        for (int d = 0; d < K; ++d) acc_out[r * K + d] = rnd(oexp * acc_out[r * K + d] + cur[d], rb);
        osum = csum + oexp * osum;
        omax = cmax;
      }
    }
    if (qr < S) {
      const float isum = 1.0f / osum;
      for (int d = 0; d < K; ++d) out[qr * K + d] = rnd(acc_out[r * K + d] * isum, rb);
    }
  }
  free(acc_out);
  free(cur);
}

/* ---- task pool: the reference runs "#pragma omp parallel for collapse(3)" over (batch, head,
 * query block) (:88); gcc's OpenMP runtime is not installed in this image, so the same task
 * list is handed out to pthreads through an atomic counter. */
typedef struct {
  const float *q, *k, *v, *bias;
  const uint8_t* keep;
  long mask_row_stride;
  float* out;
  int B1, B2, S, K, M, Mb, BLK, FLASH, flash, rb;
  int next_task; /* atomic */
  int failed;
} job_t;

static void* worker(void* arg) {
  job_t* J = (job_t*)arg;
  float* L = (float*)malloc(sizeof(float) * (size_t)J->BLK * (J->flash ? J->FLASH : J->M));
  float* qs = (float*)malloc(sizeof(float) * (size_t)J->BLK * J->K);
  float* maskadd = (float*)malloc(sizeof(float) * (size_t)J->M);
  float* kT = (float*)malloc(sizeof(float) * (size_t)J->S * J->K);   /* K of one (batch, head), [d][key] */
  int kT_owner = -1;
  if (!L || !qs || !maskadd || !kT || J->K > 256) {
    __atomic_store_n(&J->failed, 1, __ATOMIC_RELAXED);
  } else {
    const float neg = rnd(-1e9f, J->rb);
    const int ntasks = J->B1 * J->B2 * J->Mb;
    for (;;) {
      const int t = __atomic_fetch_add(&J->next_task, 1, __ATOMIC_RELAXED);
      if (t >= ntasks) break;
      const int kb = t % J->Mb, j = (t / J->Mb) % J->B2, i = t / (J->Mb * J->B2);
      /* mask: 1.0 = masked, padded keys are masked (:54), times T(-1e9) (:63-74) */
      for (int c = 0; c < J->M; ++c) {
        const int masked =
            (c >= J->S) || (J->keep && !J->keep[(size_t)i * J->mask_row_stride + c]);
        maskadd[c] = rnd((masked ? 1.0f : 0.0f) * neg, J->rb);
      }
      const size_t off = ((size_t)i * J->B2 + j) * (size_t)J->S * J->K;
      const float* bj = J->bias + (size_t)j * J->S * J->S;
      if (J->flash)
        task_flash(J->q + off, J->k + off, J->v + off, bj, maskadd, J->out + off, J->S, J->K,
                   J->M, J->BLK, J->FLASH, kb, J->rb, L, qs);
      else {
        if (kT_owner != t / J->Mb) {
          const float* ksrc = J->k + off;
          for (int c = 0; c < J->S; ++c)
            for (int d = 0; d < J->K; ++d) kT[(size_t)d * J->S + c] = ksrc[(size_t)c * J->K + d];
          kT_owner = t / J->Mb;
        }
        task_plain(J->q + off, kT, J->v + off, bj, maskadd, J->out + off, J->S, J->K,
                   J->M, J->BLK, kb, J->rb, L, qs);
      }
    }
  }
  free(L);
  free(qs);
  free(maskadd);
  free(kT);
  return NULL;
}

/* Returns 0 on success.  mask_row_stride = 0 broadcasts one mask row over B1.
 * num_threads <= 0 uses every online CPU. */
int af3k_oracle_dot_product_attention(const float* q, const float* k, const float* v,
                                      const float* bias, const uint8_t* keep,
                                      long mask_row_stride, float* out, int B1, int B2, int S,
                                      int K, int BLK_SZ, int use_flash, int FLASH_SZ,
                                      int round_bf16, int num_threads) {
  if (B1 <= 0 || B2 <= 0 || S <= 0 || K <= 0 || BLK_SZ <= 0 || FLASH_SZ <= 0) return 1;
  job_t J;
  J.q = q; J.k = k; J.v = v; J.bias = bias; J.keep = keep;
  J.mask_row_stride = mask_row_stride;
  J.out = out;
  J.B1 = B1; J.B2 = B2; J.S = S; J.K = K;
  J.M = (S + BLK_SZ - 1) / BLK_SZ * BLK_SZ; /* :45 keys padded to a block multiple */
  J.Mb = J.M / BLK_SZ;
  J.BLK = BLK_SZ; J.FLASH = FLASH_SZ;
  J.flash = use_flash && J.M > FLASH_SZ;    /* :76 */
  J.rb = round_bf16;
  J.next_task = 0;
  J.failed = 0;
  int nt = num_threads > 0 ? num_threads : af3k_oracle_num_threads();
  if (nt > 256) nt = 256;
  pthread_t th[256];
  int started = 0;
  for (int t = 0; t < nt - 1; ++t)
    if (pthread_create(&th[started], NULL, worker, &J) == 0) ++started;
  worker(&J);
  for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
  return J.failed;
}
