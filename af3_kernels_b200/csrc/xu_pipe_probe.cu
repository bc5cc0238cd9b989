// Instruction-pipe probe behind the design of the attention kernel's softmax loop (sm_100a).
// Stand-alone program, registers and shared memory only; prints SM clock cycles.
//
//   part 1  cycles per warp instruction of the exponential forms (f32, f16x2, bf16x2) alone
//   part 2  which instruction classes run under a warp's ex2.approx.f32: one ex2 per step plus
//           2 / 4 / 6 / 8 instructions of one other kind, with one and with two warps per scheduler
//   part 3  ex2 in one warp, other work in the second warp of the same scheduler
//   part 4  the softmax loop of one 128 x 128 logits tile (one row per thread) in several
//           formulations, from shared memory and from registers only
//
// Build and run:  python -m af3_kernels_b200.build --probe && af3_kernels_b200/xu_pipe_probe
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

#define DI __device__ __forceinline__
DI float ex2f(float x) { float y; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
DI uint32_t ex2h2(uint32_t x) { uint32_t y; asm volatile("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x)); return y; }
DI uint32_t ex2h2ftz(uint32_t x) { uint32_t y; asm volatile("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x)); return y; }
DI uint32_t ex2b2(uint32_t x) { uint32_t y; asm volatile("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(y) : "r"(x)); return y; }
DI uint16_t ex2h1(uint16_t x) { uint16_t y; asm volatile("ex2.approx.f16 %0, %1;" : "=h"(y) : "h"(x)); return y; }
DI float fma1(float a, float b, float c) { float d; asm volatile("fma.rn.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
DI uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
DI uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm volatile("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
DI uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm volatile("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
DI float max3f(float a, float b, float c) { float d; asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
DI uint32_t cvtbf(float lo, float hi) { uint32_t d; asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
DI uint32_t cvth(float lo, float hi) { uint32_t d; asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
DI uint32_t lea23(uint32_t a, uint32_t b) { uint32_t d; asm volatile("{ .reg .u32 t; shl.b32 t, %1, 23; add.u32 %0, t, %2; }" : "=r"(d) : "r"(a), "r"(b)); return d; }
DI uint32_t iadd(uint32_t a, uint32_t b) { uint32_t d; asm volatile("add.u32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
DI uint64_t pk(float lo, float hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
DI void upk(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }


DI float add1(float a, float b) { float d; asm volatile("add.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
DI float mul1(float a, float b) { float d; asm volatile("mul.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
DI uint32_t lop(uint32_t a, uint32_t b) { uint32_t d; asm volatile("xor.b32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
DI uint32_t shl1(uint32_t a) { uint32_t d; asm volatile("shl.b32 %0, %1, 1;" : "=r"(d) : "r"(a)); return d; }
DI uint32_t mad1(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm volatile("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
DI uint32_t prmt1(uint32_t a, uint32_t b) { uint32_t d; asm volatile("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(d) : "r"(a), "r"(b)); return d; }
DI float max2f(float a, float b) { float d; asm volatile("max.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
DI uint64_t mul2(uint64_t a, uint64_t b) { uint64_t d; asm volatile("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// ---------------------------------------------------------------- parts 1-3
// OP: 1 ex2.f32, 4 FFMA, 5 FFMA2 (3 distinct operands), 6 max3, 7 cvt.bf16x2, 8 add.u32, 10 HFMA2, 11 FADD2,
//     13 FADD, 14 FMUL, 15 xor, 16 shl, 17 mad.lo, 18 prmt, 19 max (2-input), 20 FFMA2 with two loop-constant operands,
//     21 FMUL2, 22 lea-style shl+add
template <int OP>
DI void do_op(float (&x)[16], uint32_t (&u)[16], uint64_t (&w)[16], int i) {
  const int r = i & 15;
  if (OP == 1) x[r] = ex2f(x[r]);
  if (OP == 2) u[r] = ex2h2(u[r]);
  if (OP == 3) u[r] = ex2b2(u[r]);
  if (OP == 4) x[r] = fma1(x[r], 0.999f, 0.001f);
  if (OP == 13) x[r] = add1(x[r], 0.001f);
  if (OP == 14) x[r] = mul1(x[r], 0.999f);
  if (OP == 5) w[r] = fma2(w[r], w[(r + 1) & 15], w[(r + 2) & 15]);
  if (OP == 20) w[r] = fma2(w[r], w[14], w[15]);
  if (OP == 11) w[r] = add2(w[r], w[(r + 1) & 15]);
  if (OP == 21) w[r] = mul2(w[r], w[15]);
  if (OP == 6) x[r] = max3f(x[r], x[(r + 1) & 15], x[(r + 3) & 15]);
  if (OP == 19) x[r] = max2f(x[r], x[(r + 1) & 15]);
  if (OP == 7) x[r] = __uint_as_float(cvtbf(x[r], x[(r + 1) & 15]));
  if (OP == 8) u[r] = iadd(u[r], u[(r + 1) & 15]);
  if (OP == 15) u[r] = lop(u[r], u[(r + 1) & 15]);
  if (OP == 16) u[r] = shl1(u[r]) | 1u;
  if (OP == 17) u[r] = mad1(u[r], u[(r + 1) & 15], u[(r + 2) & 15]);
  if (OP == 18) u[r] = prmt1(u[r], u[(r + 1) & 15]);
  if (OP == 22) u[r] = lea23(u[r], u[(r + 1) & 15]);
  if (OP == 10) u[r] = hfma2(u[r], u[(r + 1) & 15], u[(r + 2) & 15]);
}

// part 3: warps 0-3 run (NA x OPA), warps 4-7 (same schedulers) run (NB x OPB)
template <int OPA, int NA, int OPB, int NB>
__global__ void __launch_bounds__(256, 1) two_roles(const float* in, float* out, long long* cyc, int iters) {
  float xa[16]; uint32_t ua[16]; uint64_t wa[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { xa[i] = in[(threadIdx.x * 16 + i) % 4096]; ua[i] = 0xB800B800u + i; wa[i] = pk(xa[i], xa[i] * 0.5f); }
  const bool second = (threadIdx.x >> 5) >= 4;
  __syncthreads();
  const long long t0 = clock64();
  if (!second) {
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
#pragma unroll
        for (int j = 0; j < NA; ++j) do_op<OPA>(xa, ua, wa, i * NA + j);
      }
    }
  } else {
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
#pragma unroll
        for (int j = 0; j < NB; ++j) do_op<OPB>(xa, ua, wa, i * NB + j);
      }
    }
  }
  const long long t1 = clock64();
  if ((threadIdx.x & 31) == 0 && blockIdx.x == 0) cyc[threadIdx.x >> 5] = t1 - t0;
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { float a, b; upk(wa[i], a, b); r += xa[i] + __uint_as_float(ua[i]) + a + b; }
  out[blockIdx.x * blockDim.x + threadIdx.x] = r;
}

template <int OPA, int NA, int OPB, int NB>
__global__ void __launch_bounds__(256, 1) pipes(const float* in, float* out, long long* cyc, int iters) {
  float xa[16], xb[16]; uint32_t ua[16], ub[16]; uint64_t wa[16], wb[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    xa[i] = in[(threadIdx.x * 16 + i) % 4096]; xb[i] = xa[i] * 0.5f;
    ua[i] = 0xB800B800u + i; ub[i] = 0xBF00BF00u + i;
    wa[i] = pk(xa[i], xb[i]); wb[i] = pk(xb[i], xa[i]);
  }
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
#pragma unroll
      for (int j = 0; j < NA; ++j) do_op<OPA>(xa, ua, wa, i * NA + j);
#pragma unroll
      for (int j = 0; j < NB; ++j) do_op<OPB>(xb, ub, wb, i * NB + j);
    }
  }
  const long long t1 = clock64();
  if ((threadIdx.x & 31) == 0 && blockIdx.x == 0) cyc[threadIdx.x >> 5] = t1 - t0;
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { float a, b; upk(wa[i], a, b); float c, d; upk(wb[i], c, d); r += xa[i] + xb[i] + __uint_as_float(ua[i]) + __uint_as_float(ub[i]) + a + b + c + d; }
  out[blockIdx.x * blockDim.x + threadIdx.x] = r;
}

static float* g_in; static float* g_out; static long long* g_cyc;
constexpr int kIters = 100;

template <int OPA, int NA, int OPB, int NB>
double time_pipes(int warps) {
  for (int rep = 0; rep < 2; ++rep) {
    pipes<OPA, NA, OPB, NB><<<148, warps * 32>>>(g_in, g_out, g_cyc, kIters);
    cudaDeviceSynchronize();
  }
  long long h[8]; cudaMemcpy(h, g_cyc, sizeof(h), cudaMemcpyDeviceToHost);
  return (double)h[0] / kIters / 32;
}
template <int OPA, int NA, int OPB, int NB>
void cross(const char* name) {
  for (int rep = 0; rep < 2; ++rep) {
    two_roles<OPA, NA, OPB, NB><<<148, 256>>>(g_in, g_out, g_cyc, kIters);
    cudaDeviceSynchronize();
  }
  long long h[8]; cudaMemcpy(h, g_cyc, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-36s | warp A %6.2f, warp B %6.2f cyc/step\n", name, (double)h[0] / kIters / 32, (double)h[4] / kIters / 32);
}
// one line per op: alone (4 per step), then with one ex2 per step and 2 / 4 / 6 / 8 of the op, 1 warp and 2 warps per scheduler
template <int OP>
void row(const char* name) {
  const double alone = time_pipes<OP, 4, 0, 0>(4) / 4;
  const double a2 = time_pipes<1, 1, OP, 2>(4), a4 = time_pipes<1, 1, OP, 4>(4), a6 = time_pipes<1, 1, OP, 6>(4), a8 = time_pipes<1, 1, OP, 8>(4);
  const double b2 = time_pipes<1, 1, OP, 2>(8), b4 = time_pipes<1, 1, OP, 4>(8), b6 = time_pipes<1, 1, OP, 6>(8);
  printf("%-28s | alone %5.2f cyc/instr | ex2 + 2/4/6/8 of it, 1 warp/sched: %6.2f %6.2f %6.2f %6.2f | 2 warps/sched (per warp): %6.2f %6.2f %6.2f\n",
         name, alone, a2, a4, a6, a8, b2, b4, b6);
}

// ---------------------------------------------------------------- part 4: softmax tile proxies
// MODE bits: 1 = scalar FFMA for the exponent argument (else FFMA2), 2 = scalar FADD row sum (else FADD2), 4 = no row sum,
//            8 = no exponent-argument instruction at all (ex2 of the raw value), 16 = no max pass, 32 = no bf16 pack (store p0 only),
//            64 = no ex2 (copy), 128 = values stay in registers between tiles (no shared-memory loads / stores)
template <int MODE>
DI void tile_body(const float* __restrict__ sx, uint32_t* __restrict__ sp, int tid, float& m_run, float& l_run, float (&x)[128]) {
  if (!(MODE & 128)) {
#pragma unroll
    for (int i = 0; i < 128; ++i) x[i] = sx[i * 128 + tid];
  }
  float ma = -INFINITY, mb = -INFINITY;
  if (!(MODE & 16)) {
#pragma unroll
    for (int i = 0; i < 128; i += 4) { ma = max3f(ma, x[i], x[i + 1]); mb = max3f(mb, x[i + 2], x[i + 3]); }
  } else { ma = x[0]; mb = x[1]; }
  const float mt = fmaxf(fmaxf(ma, mb), m_run);
  const float ef = 1.4426950408889634f;
  const float nml = -mt * ef;
  const uint64_t l2e2 = pk(ef, ef), nml2 = pk(nml, nml);
  uint64_t suma = pk(0.f, 0.f), sumb = suma;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  uint32_t keep = 0;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = g * 16 + 2 * i;
      float y0, y1;
      if (MODE & 8) { y0 = x[col]; y1 = x[col + 1]; }
      else if (MODE & 1) {
        asm("fma.rn.f32 %0, %1, %2, %3;" : "=f"(y0) : "f"(x[col]), "f"(ef), "f"(nml));
        asm("fma.rn.f32 %0, %1, %2, %3;" : "=f"(y1) : "f"(x[col + 1]), "f"(ef), "f"(nml));
      } else {
        uint64_t y2; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(y2) : "l"(pk(x[col], x[col + 1])), "l"(l2e2), "l"(nml2));
        upk(y2, y0, y1);
      }
      float p0, p1;
      if (MODE & 64) { p0 = y0; p1 = y1; }
      else { asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(y0)); asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(y1)); }
      if (!(MODE & 4)) {
        if (MODE & 2) {
          if (i & 1) { asm("add.rn.f32 %0, %1, %2;" : "=f"(s2) : "f"(s2), "f"(p0)); asm("add.rn.f32 %0, %1, %2;" : "=f"(s3) : "f"(s3), "f"(p1)); }
          else       { asm("add.rn.f32 %0, %1, %2;" : "=f"(s0) : "f"(s0), "f"(p0)); asm("add.rn.f32 %0, %1, %2;" : "=f"(s1) : "f"(s1), "f"(p1)); }
        } else {
          uint64_t& acc = (i & 1) ? sumb : suma;
          asm("add.rn.f32x2 %0, %1, %2;" : "=l"(acc) : "l"(acc), "l"(pk(p0, p1)));
        }
      }
      uint32_t word;
      if (MODE & 32) word = __float_as_uint(p0) ^ __float_as_uint(p1);
      else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(word) : "f"(p1), "f"(p0));
      if (MODE & 128) { keep ^= word; x[col] = p0 - 1.0f; x[col + 1] = p1 - 1.0f; }
      else sp[(g * 8 + i) * 128 + tid] = word;
    }
  }
  float a0, a1, a2, a3; upk(suma, a0, a1); upk(sumb, a2, a3);
  l_run = l_run + ((a0 + a1) + (a2 + a3)) + ((s0 + s1) + (s2 + s3)) + __uint_as_float(keep & 1u);
  m_run = mt;
}

template <int MODE>
__global__ void __launch_bounds__(256, 1) tiles(const float* in, float* out, long long* cyc, int ntiles) {
  extern __shared__ float smem[];
  const int wg = threadIdx.x >> 7, tid = threadIdx.x & 127;
  float* sx = smem + wg * (128 * 128 + 64 * 128);
  uint32_t* sp = reinterpret_cast<uint32_t*>(sx + 128 * 128);
  for (int i = tid; i < 128 * 128; i += 128) sx[i] = in[i % 4096] * 3.0f;
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;
  float x[128];
#pragma unroll
  for (int i = 0; i < 128; ++i) x[i] = sx[i * 128 + tid];
  const long long t0 = clock64();
  for (int t = 0; t < ntiles; ++t) {
    tile_body<MODE>(sx, sp, tid, m_run, l_run, x);
    asm volatile("" ::: "memory");
  }
  const long long t1 = clock64();
  if ((threadIdx.x & 31) == 0 && blockIdx.x == 0) cyc[threadIdx.x >> 5] = t1 - t0;
  float r = m_run + l_run + __uint_as_float(sp[tid]);
  if (MODE & 128) {
#pragma unroll
    for (int i = 0; i < 128; ++i) r += x[i];
  }
  out[blockIdx.x * blockDim.x + threadIdx.x] = r;
}

template <int MODE>
void run_tiles(const char* name) {
  const int smem = 2 * (128 * 128 + 64 * 128) * 4;
  cudaFuncSetAttribute(tiles<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  double r[2];
  int k = 0;
  for (int warps : {4, 8}) {
    for (int rep = 0; rep < 2; ++rep) {
      tiles<MODE><<<148, warps * 32, smem>>>(g_in, g_out, g_cyc, 64);
      cudaDeviceSynchronize();
    }
    long long h[8]; cudaMemcpy(h, g_cyc, sizeof(h), cudaMemcpyDeviceToHost);
    r[k++] = (double)h[0] / 64;
  }
  cudaError_t e = cudaGetLastError();
  printf("%-62s | 1 warp/sched %6.0f cyc/tile | 2 warps/sched %6.0f cyc/tile/warp = %5.0f cyc/tile/SM %s\n", name, r[0], r[1], r[1] / 2, e ? cudaGetErrorString(e) : "");
}

int main() {
  cudaMalloc(&g_in, 4096 * 4); cudaMalloc(&g_out, 148 * 256 * 4); cudaMalloc(&g_cyc, 64);
  float h[4096]; for (int i = 0; i < 4096; ++i) h[i] = -0.001f * (i % 977) - 0.5f;
  cudaMemcpy(g_in, h, sizeof(h), cudaMemcpyHostToDevice);
  printf("== exponential forms alone: cycles per warp instruction, 1 warp / 2 warps per scheduler\n");
  printf("ex2.approx.ftz.f32     %6.2f %6.2f\n", time_pipes<1, 1, 0, 0>(4), time_pipes<1, 1, 0, 0>(8));
  printf("ex2.approx.f16x2       %6.2f %6.2f   (two results per instruction)\n", time_pipes<2, 1, 0, 0>(4), time_pipes<2, 1, 0, 0>(8));
  printf("ex2.approx.ftz.bf16x2  %6.2f %6.2f   (two results per instruction)\n", time_pipes<3, 1, 0, 0>(4), time_pipes<3, 1, 0, 0>(8));
  printf("== which instructions run under a warp's ex2.approx.f32 (8 cycles each on the XU)\n");
  printf("ex2.approx.ftz.f32 alone: %.2f cyc/instr (1 warp/sched), %.2f per warp with 2 warps/sched\n", time_pipes<1, 1, 0, 0>(4), time_pipes<1, 1, 0, 0>(8));
  row<4>("fma.rn.f32");
  row<13>("add.rn.f32");
  row<14>("mul.rn.f32");
  row<20>("fma.rn.f32x2 (2 const operands)");
  row<5>("fma.rn.f32x2 (3 operands)");
  row<11>("add.rn.f32x2");
  row<21>("mul.rn.f32x2");
  row<6>("max.f32 (3-input)");
  row<19>("max.f32 (2-input)");
  row<7>("cvt.rn.bf16x2.f32");
  row<8>("add.u32");
  row<15>("xor.b32");
  row<16>("shl + or");
  row<22>("shl + add");
  row<17>("mad.lo.u32");
  row<18>("prmt.b32");
  row<10>("fma.rn.f16x2");
  printf("== ex2 in warps 0-3, other work in warps 4-7 of the same schedulers: cycles per step of each\n");
  cross<1, 1, 4, 4>("A: 1 ex2 | B: 4 fma.rn.f32");
  cross<1, 1, 4, 8>("A: 1 ex2 | B: 8 fma.rn.f32");
  cross<1, 1, 6, 4>("A: 1 ex2 | B: 4 max.f32 (3-input)");
  cross<1, 1, 1, 1>("A: 1 ex2 | B: 1 ex2");
  printf("== softmax tile proxies (128 x 128 tile, one row per thread)\n");
  run_tiles<0>("packed arg, packed sum (the kernel's loop)");
  run_tiles<1>("scalar arg, packed sum");
  run_tiles<2>("packed arg, scalar sum");
  run_tiles<3>("scalar arg, scalar sum");
  run_tiles<4>("packed arg, no sum");
  run_tiles<5>("scalar arg, no sum");
  run_tiles<12>("no arg, no sum");
  run_tiles<12 + 16>("no arg, no sum, no max");
  run_tiles<12 + 16 + 32>("no arg, no sum, no max, no pack (ex2 + ld/st only)");
  run_tiles<64 + 3>("scalar everything, exponential replaced by a copy");
  run_tiles<128 + 0>("registers only: packed arg, packed sum");
  run_tiles<128 + 3>("registers only: scalar arg, scalar sum");
  run_tiles<128 + 5>("registers only: scalar arg, no sum");
  run_tiles<128 + 12>("registers only: no arg, no sum");
  run_tiles<128 + 12 + 16 + 32>("registers only: ex2 alone");
  return 0;
}
