// The four input projections of the grid / triangle attention block as ONE pass over the
// (layer-normed) pair representation, for sm_100a:
//
//     [q | k | v | gate] = x [M, 128] * W4^T,     W4 = [Wq; Wk; Wv; Wg]  ([512, 128], rows = output channels)
//
// Stands in for the per-(row, head) K/V projection BRGEMMs and the per-query-block Q and gate
// projection BRGEMMs of the reference's fused block (src/csrc/dot_product_attention.cpp:285-298
// and :300-338).  x is read once (the reference, and four separate GEMMs, read it four times);
// q, k and v leave in the head-major layout [R, H, N, D] the attention kernel's TMA reads with
// unit-stride rows, q already multiplied by the softmax scale (in fp32, rounded once); the gate
// leaves as [M, 128].  HBM-bound: 256 bytes read and 1024 written per row of x.
//
//   warp 0      TMA producer: W4 once (128 KB, stays in shared memory), then x tiles of 128 rows
//   warp 1      allocates TMEM, issues tcgen05.mma: per x tile two groups of 8 (N = 256, K = 16),
//               columns [0, 256) = q | k and [256, 512) = v | gate
//   warps 4-7   epilogue of columns [0, 256): TMEM -> registers -> bf16 -> shared -> global
//   warps 8-11  epilogue of columns [256, 512)
// A TMEM lane is a row of x, so a thread holds 64 consecutive output columns of ONE row; stored
// from there, a warp's 16-byte pieces would land 64 or 256 bytes apart.  Each epilogue warp
// therefore passes its 32 rows x 128 bytes through a private, XOR-swizzled patch of shared memory
// and stores with consecutive lanes on consecutive 16-byte pieces (full 64 / 128-byte runs).
// The two column halves have their own full / empty barriers, so the MMAs of one half run while
// the other half is being drained.
//
// Second instantiation (kLn): x is the RAW pair representation and a fourth warpgroup stands
// between the TMA and the MMAs,
//   warps 12-19 two LayerNorm warpgroups, one per stage of the x ring (a tile's two walks are a
//               chain of about a thousand dependent instructions per thread, twice the tile's share
//               of the HBM time, so two tiles are normalised at a time): thread t owns row t -
//               moments, normalise in place, round to bf16 - and, from the rounded values, the
//               per-head logit bias of the row (up to four heads), stored straight into [H, R, N];
// which takes the normalised pair's round trip through HBM (one write and one read of M x 256
// bytes) out of the block.  Measured at N = 768: 0.232 ms against 0.073 + 0.140 ms for the stand-alone
// producer followed by the first instantiation - the row walks are latency-bound and only two tiles
// per SM are in them at a time (the stand-alone producer has five CTAs per SM) -, so the modules do
// not use this instantiation by default.  Reference: src/af3_kernels/Attention.py:51-52 and :152-153 in front of
// the projections above.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace af3k {

constexpr int kProjC = 128;                 // input channels (c_pair)
constexpr int kProjOut = 4 * kProjC;        // q | k | v | gate
constexpr int kProjThreads = 384;
constexpr int kProjLnThreads = 640;         // + the two LayerNorm warpgroups
// Registers of the kLn variant: launched with 96 per thread (61440, the pool setmaxnreg works in),
// then 128 x 72 (producer, MMA issuer) + 256 x 128 (epilogue) + 256 x 72 (LayerNorm) = 60416.
constexpr int kProjLnRegsMisc = 72, kProjLnRegsEpi = 128, kProjLnRegsNorm = 72;
static_assert(128 * kProjLnRegsMisc + 256 * kProjLnRegsEpi + 256 * kProjLnRegsNorm <= 96 * kProjLnThreads,
              "setmaxnreg totals exceed the launch allocation");
constexpr int kProjStages = 2;              // x tiles in flight
constexpr uint32_t kProjXTileBytes = 128 * kProjC * 2;          // 32 KB: two 128B-swizzled panels of 64 channels
constexpr uint32_t kProjWBytes = kProjOut * kProjC * 2;         // 128 KB: two panels of 64 channels x 512 rows
constexpr uint32_t kProjStagingBytes = 8 * 32 * 128;            // per epilogue warp: 32 rows x 64 bf16 columns
constexpr uint32_t kProjSmemBytes = kProjWBytes + kProjStages * kProjXTileBytes + 256 /*barriers*/ +
                                    kProjStagingBytes + 1024 /*alignment*/;

struct ProjParams {
  long long M;           // rows of x (= R * N)
  int N;                 // tokens per pair row
  int H, D;              // heads and head width, H * D == 128
  float q_scale;         // applied to the q columns before rounding
  __nv_bfloat16* q;      // [R, H, N, D]
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  __nv_bfloat16* g;      // [M, 128]
  int* status;           // same status word as the attention kernel
  long long wait_limit;
  // kLn only: LayerNorm weight / bias [128], bias projection [Hb, 128] (all fp32), output [Hb, R, bias_pitch]
  const float* gamma;
  const float* beta;
  const float* bias_w;
  __nv_bfloat16* bias;
  long long bias_pitch;
  int Hb, R;
  float eps;
};

struct ProjBar {
  static constexpr int w_full = 0;
  static constexpr int x_full = 1;                       // [kProjStages]
  static constexpr int x_empty = 1 + kProjStages;        // [kProjStages]
  static constexpr int acc_full = 1 + 2 * kProjStages;   // [2] column halves
  static constexpr int acc_empty = 3 + 2 * kProjStages;  // [2]
  static constexpr int x_ready = 5 + 2 * kProjStages;    // [kProjStages]  tile normalised in place (kLn)
  static constexpr int count = 5 + 3 * kProjStages;
};

__device__ __forceinline__ void proj_timeout(const ProjParams& p, volatile int* abort_flag, int bar) {
  *abort_flag = 1;
  if (p.status != nullptr) {
    atomicOr(p.status, 1 /* wait timeout */);
    if (atomicCAS(p.status + 1, 0, 1000 + bar + 1) == 0) {
      p.status[2] = blockIdx.x;
      p.status[3] = threadIdx.x >> 5;
    }
  }
}

#define AF3K_PROJ_WAIT(idx, parity)                                                              \
  do {                                                                                           \
    const bool ok_ = mbar_wait_bounded(bars + 8u * (idx), (parity), p.wait_limit, &abort_flag);   \
    if (!__all_sync(0xffffffffu, ok_)) {                                                         \
      proj_timeout(p, &abort_flag, (idx));                                                       \
      goto done;                                                                                 \
    }                                                                                            \
  } while (0)

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

template <bool kLn>
__global__ void __launch_bounds__(kLn ? kProjLnThreads : kProjThreads, 1)
qkvg_projection_kernel(const __grid_constant__ ProjParams p, const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t proj_smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem = (smem_u32(proj_smem_raw) + 1023u) & ~1023u;
  const uint32_t w_smem = smem;                                   // [2 panels][512 rows][128 B]
  const uint32_t x_smem = smem + kProjWBytes;                     // [stages][2 panels][128 rows][128 B]
  const uint32_t bars = x_smem + kProjStages * kProjXTileBytes;
  const long long n_tiles = (p.M + 127) / 128;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    mbar_init(bars + 8u * ProjBar::w_full, 1);
    for (int i = 0; i < kProjStages; ++i) {
      mbar_init(bars + 8u * (ProjBar::x_full + i), 1);
      mbar_init(bars + 8u * (ProjBar::x_empty + i), 1);
      mbar_init(bars + 8u * (ProjBar::x_ready + i), 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8u * (ProjBar::acc_full + i), 1);
      mbar_init(bars + 8u * (ProjBar::acc_empty + i), 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  if (kLn) {
    if (warp < 4) setmaxnreg_dec<kProjLnRegsMisc>();
    else if (warp < 12) setmaxnreg_inc<kProjLnRegsEpi>();
    else setmaxnreg_dec<kProjLnRegsNorm>();
  }
  if (warp == 0) {
    // ---- producer (whole warp runs the control flow, one lane issues)
    const bool leader = elect_one();
    if (leader) {
      mbar_arrive_expect_tx(bars + 8u * ProjBar::w_full, kProjWBytes);
      for (int kb = 0; kb < 2; ++kb)
        for (int nb = 0; nb < 2; ++nb)
          tma_load_2d(w_smem + kb * (kProjWBytes / 2) + nb * 256 * 128, &tm_w, bars + 8u * ProjBar::w_full, kb * 64, nb * 256);
    }
    uint32_t n = 0;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n) {
      const uint32_t st = n % kProjStages;
      if (n >= kProjStages) AF3K_PROJ_WAIT(ProjBar::x_empty + st, ((n / kProjStages) - 1) & 1);
      if (leader) {
        const uint32_t full = bars + 8u * (ProjBar::x_full + st);
        const uint32_t dst = x_smem + st * kProjXTileBytes;
        mbar_arrive_expect_tx(full, kProjXTileBytes);
        tma_load_2d(dst, &tm_x, full, 0, (int)(tile * 128));
        tma_load_2d(dst + kProjXTileBytes / 2, &tm_x, full, 64, (int)(tile * 128));
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc(1u, 1u, 0u, 0u, 256);
    const uint64_t ad0 = make_smem_desc(x_smem, 16, 8 * 128, 2);
    const uint64_t bd0 = make_smem_desc(w_smem, 16, 8 * 128, 2);
    const uint32_t ad_lo = (uint32_t)ad0, ad_hi = (uint32_t)(ad0 >> 32);
    const uint32_t bd_lo = (uint32_t)bd0, bd_hi = (uint32_t)(bd0 >> 32);
    AF3K_PROJ_WAIT(ProjBar::w_full, 0);
    uint32_t n = 0;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n) {
      const uint32_t st = n % kProjStages;
      AF3K_PROJ_WAIT((kLn ? ProjBar::x_ready : ProjBar::x_full) + st, (n / kProjStages) & 1);
      for (int nh = 0; nh < 2; ++nh) {
        // the epilogue warps of this half must have read the previous tile's columns
        if (n >= 1) AF3K_PROJ_WAIT(ProjBar::acc_empty + nh, (n - 1) & 1);
        tc_fence_after();
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < kProjC / 16; ++ks) {
            // 16 channels = 32 bytes of a 128-byte panel row; panel ks / 4
            const uint32_t a = ad_lo + ((st * kProjXTileBytes + (ks >> 2) * (kProjXTileBytes / 2)) >> 4) + 2 * (ks & 3);
            const uint32_t b = bd_lo + (((ks >> 2) * (kProjWBytes / 2) + nh * 256 * 128) >> 4) + 2 * (ks & 3);
            mma_ss_f16(tmem + nh * 256, a, ad_hi, b, bd_hi, idesc, ks > 0 ? 1u : 0u);
          }
          tc_commit(bars + 8u * (ProjBar::acc_full + nh));
          if (nh == 1) tc_commit(bars + 8u * (ProjBar::x_empty + st));
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---- epilogue: warp quarter (TMEM lanes) x column half
    const int quarter = warp & 3, half = (warp - 4) >> 2;
    const uint32_t t_base = tmem + ((uint32_t)(quarter * 32) << 16) + half * 256;
    const uint32_t patch = bars + 256 + (uint32_t)(warp - 4) * (32 * 128);
    const int log2d = 31 - __clz(p.D);
    uint32_t n = 0;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n) {
      AF3K_PROJ_WAIT(ProjBar::acc_full + half, n & 1);
      tc_fence_after();
      const long long m0 = tile * 128 + quarter * 32;                 // the warp's first row of x
      const long long r0 = m0 / p.N;
      const int tok0 = (int)(m0 - r0 * p.N);
      // Element offsets of the eight rows this lane stores in every 64-column piece (rows
      // (lane >> 3) + 4 i), worked out once per tile: into [R, H, N, D] at head 0 and into [M, 128].
      uint32_t off_qkv[8], off_g[8];
      uint32_t row_ok = 0;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int row = it * 4 + (lane >> 3);
        long long r = r0;
        int tok = tok0 + row;
        while (tok >= p.N) { tok -= p.N; ++r; }
        off_qkv[it] = (uint32_t)((r * p.H * p.N + tok) << log2d);
        off_g[it] = (uint32_t)((m0 + row) * kProjC);
        if (m0 + row < p.M) row_ok |= 1u << it;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 64) {
        uint32_t acc[64];
        tmem_ld_x32(t_base + c0, &acc[0]);
        tmem_ld_x32(t_base + c0 + 32, &acc[32]);
        tc_wait_ld();
        if (c0 == 192) {
          // the last columns are in registers: the MMAs of the next tile may overwrite this half
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + 8u * (ProjBar::acc_empty + half));
        }
        const int col0 = half * 256 + c0;                             // 64 columns of one output tensor
        const int which = col0 >> 7, within = col0 & 127;             // 0 q, 1 k, 2 v, 3 gate
        if (which == 0) {
#pragma unroll
          for (int e = 0; e < 64; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * p.q_scale);
        }
        // own row -> shared, piece j at position j ^ (row & 7): conflict-free both ways
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t w0 = pack_bf16x2(__uint_as_float(acc[8 * j + 0]), __uint_as_float(acc[8 * j + 1]));
          const uint32_t w1 = pack_bf16x2(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
          const uint32_t w2 = pack_bf16x2(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
          const uint32_t w3 = pack_bf16x2(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(patch + lane * 128 + ((j ^ (lane & 7)) << 4)),
                       "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
        }
        __syncwarp();
        // shared -> global: lane l takes piece l & 7 of rows (l >> 3) + 4 i
        const int ch = within + 8 * (lane & 7);
        __nv_bfloat16* dst;
        if (which == 3) {
          dst = p.g + ch;
        } else {
          const int head = ch >> log2d;
          dst = (which == 0 ? p.q : (which == 1 ? p.k : p.v)) + (((long long)head * p.N) << log2d) + (ch & (p.D - 1));
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          uint4 o;
          const int row = it * 4 + (lane >> 3);
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                       : "r"(patch + row * 128 + (((lane & 7) ^ (row & 7)) << 4)));
          if ((row_ok >> it) & 1u) *reinterpret_cast<uint4*>(dst + (which == 3 ? off_g[it] : off_qkv[it])) = o;
        }
        __syncwarp();      // the patch is rewritten by the next 64 columns
      }
    }
  }
  else if (kLn && warp >= 12) {
    // ---- LayerNorm in place + bias projection: warpgroup wg takes the tiles of ring stage wg,
    // thread t owns row t of the tile
    static_assert(kProjStages == 2, "one LayerNorm warpgroup per ring stage");
    const int wg = (warp - 12) >> 2;
    const int t = ((warp - 12) & 3) * 32 + lane;
    uint32_t n = (uint32_t)wg;
    for (long long tile = blockIdx.x + (long long)wg * gridDim.x; tile < n_tiles; tile += 2LL * gridDim.x, n += 2) {
      const uint32_t st = n % kProjStages;
      AF3K_PROJ_WAIT(ProjBar::x_full + st, (n / kProjStages) & 1);
      const uint32_t tile_s = x_smem + st * kProjXTileBytes;
      // 16-byte piece c8 of the row: panel c8 / 8, position (c8 % 8) ^ (row % 8) inside the 128-byte row
      auto piece = [&](int c8) { return tile_s + (uint32_t)((c8 >> 3) * (kProjXTileBytes / 2) + t * 128 + (((c8 & 7) ^ (t & 7)) << 4)); };
      auto load8 = [&](int c8, float (&x)[8]) {
        uint32_t w[4];
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(piece(c8)));
#pragma unroll
        for (int e = 0; e < 4; ++e) { x[2 * e] = __uint_as_float(w[e] << 16); x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
      };
      // mean and (biased) variance in one walk, as moments about the row's first element
      float pivot;
      {
        float x[8];
        load8(0, x);
        pivot = x[0];
      }
      const uint64_t npivot2 = pack_f32x2(-pivot, -pivot);
      uint64_t s1a = pack_f32x2(0.f, 0.f), s1b = s1a, s2a = s1a, s2b = s1a;
#pragma unroll 4
      for (int c8 = 0; c8 < 16; ++c8) {
        float x[8];
        load8(c8, x);
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
          const uint64_t da = add_f32x2(pack_f32x2(x[e], x[e + 1]), npivot2);
          const uint64_t db = add_f32x2(pack_f32x2(x[e + 2], x[e + 3]), npivot2);
          s1a = add_f32x2(s1a, da); s1b = add_f32x2(s1b, db);
          s2a = fma_f32x2(da, da, s2a); s2b = fma_f32x2(db, db, s2b);
        }
      }
      float s1lo, s1hi, s2lo, s2hi;
      unpack_f32x2(add_f32x2(s1a, s1b), s1lo, s1hi);
      unpack_f32x2(add_f32x2(s2a, s2b), s2lo, s2hi);
      const float m1 = (s1lo + s1hi) * (1.0f / kProjC);
      const float mean = pivot + m1;
      const float var = fmaxf((s2lo + s2hi) * (1.0f / kProjC) - m1 * m1, 0.f);
      const float rstd = rsqrtf(var + p.eps);
      const uint64_t rstd2 = pack_f32x2(rstd, rstd);
      const float nmr = -mean * rstd;
      const uint64_t nmr2 = pack_f32x2(nmr, nmr);
      uint64_t acc2[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) acc2[h] = pack_f32x2(0.f, 0.f);
#pragma unroll 4
      for (int c8 = 0; c8 < 16; ++c8) {
        float x[8];
        load8(c8, x);
        uint32_t yw[4];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          // the constants are the same for every thread: warp-wide broadcasts out of L1
          const ulonglong2 g4 = __ldg(reinterpret_cast<const ulonglong2*>(p.gamma + c8 * 8 + 4 * q));
          const ulonglong2 b4 = __ldg(reinterpret_cast<const ulonglong2*>(p.beta + c8 * 8 + 4 * q));
          const uint64_t z01 = fma_f32x2(pack_f32x2(x[4 * q], x[4 * q + 1]), rstd2, nmr2);
          const uint64_t z23 = fma_f32x2(pack_f32x2(x[4 * q + 2], x[4 * q + 3]), rstd2, nmr2);
          float y0, y1, y2, y3;
          unpack_f32x2(fma_f32x2(z01, g4.x, b4.x), y0, y1);
          unpack_f32x2(fma_f32x2(z23, g4.y, b4.y), y2, y3);
          yw[2 * q] = pack_bf16x2(y0, y1);
          yw[2 * q + 1] = pack_bf16x2(y2, y3);
          // the bias projection sees the rounded values
          const uint64_t r01 = pack_f32x2(__uint_as_float(yw[2 * q] << 16), __uint_as_float(yw[2 * q] & 0xffff0000u));
          const uint64_t r23 = pack_f32x2(__uint_as_float(yw[2 * q + 1] << 16), __uint_as_float(yw[2 * q + 1] & 0xffff0000u));
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            if (h < p.Hb) {
              const ulonglong2 w4 = __ldg(reinterpret_cast<const ulonglong2*>(p.bias_w + h * kProjC + c8 * 8 + 4 * q));
              acc2[h] = fma_f32x2(r23, w4.y, fma_f32x2(r01, w4.x, acc2[h]));
            }
          }
        }
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(piece(c8)), "r"(yw[0]), "r"(yw[1]), "r"(yw[2]), "r"(yw[3]) : "memory");
      }
      fence_proxy_async_smem();     // the tile was rewritten through the generic proxy; the tensor core reads it
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8u * (ProjBar::x_ready + st));
      // the row's bias values: consecutive threads are consecutive j of one pair row i (or the next one)
      const long long m = tile * 128 + t;
      if (m < p.M) {
        const long long i = m / p.N;
        const int j = (int)(m - i * p.N);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          if (h < p.Hb) {
            float lo, hi;
            unpack_f32x2(acc2[h], lo, hi);
            p.bias[((long long)h * p.R + i) * p.bias_pitch + j] = __float2bfloat16_rn(lo + hi);
          }
        }
      }
    }
  }

done:
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace af3k
