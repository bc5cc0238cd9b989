// Pair-bias producer for sm_100a: LayerNorm over the channels of the pair representation, the
// per-head bias projection and the [N, N, H] -> [H, N, N] permute, in one pass over the pair.
//
// Stands in for the two lines in front of the attention core in the reference's modules
// (src/af3_kernels/Attention.py:51-52 and :152-153):
//     pair = self.act_norm(pair)
//     bias = self.pair_bias_projection(pair).permute(2, 0, 1)
// which in PyTorch cost three passes over the pair tensor (LayerNorm read + write, Linear read)
// plus a strided-to-contiguous copy of the bias.  Here the pair is read once; the normalised
// pair (bf16, the operand of the q / k / v / gate projections) and the bias (bf16, [H, N, N],
// rows 16-byte aligned so that the attention kernel's TMA reads it in place) are written once.
//
// HBM traffic: 2 or 4 bytes read and 2 bytes written per pair element, plus H * 2 bytes per
// (i, j).  Two kernels.  Up to four heads (the grid / triangle attention of AlphaFold3): one thread
// per vector, tiles transposed through shared memory, no cross-lane reductions.  Five to sixteen
// heads: one warp per vector (4 channels per lane, statistics by shuffles in fp32).  Both run as
// persistent CTAs over tiles of consecutive j of one row i and stage each tile's bias values in
// shared memory so that they leave as full 16-byte pieces.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace af3k {

constexpr int kPbChannels = 128;   // c_pair
constexpr int kPbMaxHeads = 16;
constexpr int kPbTileJ = 128;      // vectors per CTA
constexpr int kPbThreads = 256;

struct PairBiasParams {
  const void* pair;            // [R, N, 128], bf16 or fp32, contiguous
  __nv_bfloat16* normed;       // [R, N, 128] bf16
  __nv_bfloat16* bias;         // [H, R, bias_pitch] bf16
  const float* gamma;          // [128] LayerNorm weight
  const float* beta;           // [128] LayerNorm bias
  const float* proj;           // [H, 128] projection weight (nn.Linear layout: out x in)
  int R, N, H;
  long long bias_pitch;        // elements between consecutive rows i of one head (multiple of 8)
  float eps;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums each of the kN values over the 32 lanes with a reduce-scatter butterfly: after the first
// log2(kN) exchange steps a lane holds one value's partial sum, the remaining steps finish it.
// Costs kN - 1 + (5 - log2 kN) shuffles instead of 5 * kN.  On return a[0] of lane l is the full
// sum of value number l / (32 / kN).
template <int kN>
__device__ __forceinline__ void warp_sum_scatter(float (&a)[kN], int lane) {
  static_assert(kN == 1 || kN == 2 || kN == 4 || kN == 8 || kN == 16, "power of two up to 16");
  int off = 16;
#pragma unroll
  for (int n = kN; n > 1; n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int k = 0; k < n / 2; ++k) {
      const float send = upper ? a[k] : a[k + n / 2];
      const float keep = upper ? a[k + n / 2] : a[k];
      a[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
  for (; off > 0; off >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], off);
}

__device__ __forceinline__ uint32_t pb_pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <typename T, int kHeads>
__global__ void __launch_bounds__(kPbThreads) pair_bias_kernel(const PairBiasParams p) {
  __shared__ __nv_bfloat16 s_bias[kHeads][kPbTileJ];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = lane * 4;

  // per-lane constants: 4 channels of the LayerNorm parameters and of every head's weights
  // (loaded once: the CTA is persistent and walks over the tiles of 128 vectors)
  float g[4], b[4], w[kHeads][4];
#pragma unroll
  for (int e = 0; e < 4; ++e) { g[e] = p.gamma[c0 + e]; b[e] = p.beta[c0 + e]; }
#pragma unroll
  for (int h = 0; h < kHeads; ++h)
#pragma unroll
    for (int e = 0; e < 4; ++e) w[h][e] = h < p.H ? p.proj[h * kPbChannels + c0 + e] : 0.f;

  constexpr int kWarps = kPbThreads / 32;
  constexpr int kUnroll = 4;   // vectors in flight per warp
  const int tiles_j = (p.N + kPbTileJ - 1) / kPbTileJ;
  const long long n_tiles = (long long)p.R * tiles_j;
  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
  const int i = (int)(tile / tiles_j);
  const int j0 = (int)(tile % tiles_j) * kPbTileJ;
  const long long row_base = (long long)i * p.N;
  for (int jj = warp * kUnroll; jj < kPbTileJ; jj += kWarps * kUnroll) {
    float x[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int j = j0 + jj + u;
      if (j < p.N) {
        const long long off = (row_base + j) * kPbChannels + c0;
        if (sizeof(T) == 4) {
          const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.pair) + off);
          x[u][0] = v.x; x[u][1] = v.y; x[u][2] = v.z; x[u][3] = v.w;
        } else {
          const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.pair) + off);
          x[u][0] = __uint_as_float(v.x << 16); x[u][1] = __uint_as_float(v.x & 0xffff0000u);
          x[u][2] = __uint_as_float(v.y << 16); x[u][3] = __uint_as_float(v.y & 0xffff0000u);
        }
      } else {
        x[u][0] = x[u][1] = x[u][2] = x[u][3] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int j = j0 + jj + u;
      // mean and (biased) variance over the 128 channels, two-pass in registers
      const float mean = warp_sum((x[u][0] + x[u][1]) + (x[u][2] + x[u][3])) * (1.0f / kPbChannels);
      float d[4], sq = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) { d[e] = x[u][e] - mean; sq += d[e] * d[e]; }
      const float rstd = rsqrtf(warp_sum(sq) * (1.0f / kPbChannels) + p.eps);
      // y = bf16(d * rstd * gamma + beta): written as the normalised pair and, as those same
      // rounded values, the operand of the bias projection (what a bf16 LayerNorm followed by a
      // bf16 Linear sees)
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = d[e] * rstd * g[e] + b[e];
      const uint32_t lo = pb_pack_bf16x2(y[0], y[1]), hi = pb_pack_bf16x2(y[2], y[3]);
      y[0] = __uint_as_float(lo << 16); y[1] = __uint_as_float(lo & 0xffff0000u);
      y[2] = __uint_as_float(hi << 16); y[3] = __uint_as_float(hi & 0xffff0000u);
      if (j < p.N)
        *reinterpret_cast<uint2*>(p.normed + (row_base + j) * kPbChannels + c0) = make_uint2(lo, hi);
      float acc[kHeads];
#pragma unroll
      for (int h = 0; h < kHeads; ++h)
        acc[h] = (y[0] * w[h][0] + y[1] * w[h][1]) + (y[2] * w[h][2] + y[3] * w[h][3]);
      warp_sum_scatter<kHeads>(acc, lane);
      // lanes 0, 32 / kHeads, ... hold heads 0, 1, ...
      if ((lane & (32 / kHeads - 1)) == 0) s_bias[lane / (32 / kHeads)][jj + u] = __float2bfloat16_rn(acc[0]);
    }
  }
  __syncthreads();
  // H rows of 128 bf16 = 256 bytes each: 16 threads x 16 bytes per head
  const int h = threadIdx.x >> 4, seg = threadIdx.x & 15;
  if (h < p.H) {
    const int j = j0 + seg * 8;
    __nv_bfloat16* dst = p.bias + ((long long)h * p.R + i) * p.bias_pitch + j;
    if (j + 8 <= p.N) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_bias[h][seg * 8]);
    } else {
      for (int e = 0; e < 8 && j + e < p.N; ++e) dst[e] = s_bias[h][seg * 8 + e];
    }
  }
  __syncthreads();   // s_bias is reused by the next tile
  }
}

// ---------------------------------------------------------------- up to 4 heads: one thread per vector
// The reductions are what held the kernels above back (chains of dependent shuffles), so here a
// vector is not shared between lanes at all: a tile of vectors is copied to shared memory with
// coalesced 16-byte loads (rows padded by 16 bytes, so that the 8 lanes of a 128-bit access
// phase hit different banks), then thread t walks over row t twice (moments; normalise, round,
// project), writes the bf16 result back over the row, and the
// tile leaves again with coalesced stores.  The constants are read from shared memory as
// warp-wide broadcasts.
template <typename T>
struct PbTile {
  static constexpr int kRows = sizeof(T) == 2 ? 128 : 64;           // vectors per tile = threads per CTA
  static constexpr int kRowBytes = kPbChannels * (int)sizeof(T);
  static constexpr int kStride = kRowBytes + 16;                    // bytes between rows in shared memory
  static constexpr int kPieces = kRowBytes / 16;                    // 16-byte pieces per row
  static constexpr int kSmemBytes = kRows * kStride + 6 * kPbChannels * 4 + 4 * kRows * 2;
};

template <typename T>
__device__ __forceinline__ void pb_unpack8(const uint4& v, const uint4& v2, float (&x)[8]) {
  if (sizeof(T) == 4) {
    x[0] = __uint_as_float(v.x); x[1] = __uint_as_float(v.y); x[2] = __uint_as_float(v.z); x[3] = __uint_as_float(v.w);
    x[4] = __uint_as_float(v2.x); x[5] = __uint_as_float(v2.y); x[6] = __uint_as_float(v2.z); x[7] = __uint_as_float(v2.w);
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { x[2 * e] = __uint_as_float(w[e] << 16); x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
  }
}

template <typename T>
__global__ void __launch_bounds__(PbTile<T>::kRows, 640 / PbTile<T>::kRows) pair_bias_kernel_t(const PairBiasParams p) {
  using Tl = PbTile<T>;
  extern __shared__ __align__(16) uint8_t pb_smem[];
  float* s_c = reinterpret_cast<float*>(pb_smem + Tl::kRows * Tl::kStride);   // g, b, w0..w3: [6][128]
  __nv_bfloat16* s_bias = reinterpret_cast<__nv_bfloat16*>(s_c + 6 * kPbChannels);   // [4][kRows]
  const int t = threadIdx.x;
  for (int c = t; c < kPbChannels; c += Tl::kRows) {
    s_c[c] = p.gamma[c];
    s_c[kPbChannels + c] = p.beta[c];
#pragma unroll
    for (int h = 0; h < 4; ++h) s_c[(2 + h) * kPbChannels + c] = h < p.H ? p.proj[h * kPbChannels + c] : 0.f;
  }
  const int tiles_j = (p.N + Tl::kRows - 1) / Tl::kRows;
  const long long n_tiles = (long long)p.R * tiles_j;
  // global -> shared, coalesced (the tile's vectors are contiguous in memory), as asynchronous
  // 16-byte copies: the whole tile is in flight at once and no registers are held.  (A second
  // row buffer that prefetches the next tile was slower: it costs two of the five resident CTAs.)
  auto request_tile = [&](long long tile, uint8_t* buf) {
    const int j0 = (int)(tile % tiles_j) * Tl::kRows;
    const int rows = min(Tl::kRows, p.N - j0);
    const long long vec0 = (tile / tiles_j) * p.N + j0;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.pair) + vec0 * Tl::kRowBytes);
    for (int k = t; k < rows * Tl::kPieces; k += Tl::kRows) {
      const uint32_t dst_s = (uint32_t)__cvta_generic_to_shared(buf + (k / Tl::kPieces) * Tl::kStride +
                                                                (k % Tl::kPieces) * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_s), "l"(src + k) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  uint8_t* s_rows = pb_smem;
  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int i = (int)(tile / tiles_j);
    const int j0 = (int)(tile % tiles_j) * Tl::kRows;
    const int rows = min(Tl::kRows, p.N - j0);
    const long long vec0 = (long long)i * p.N + j0;                 // first vector of the tile
    request_tile(tile, s_rows);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (t < rows) {
      const uint8_t* row = s_rows + t * Tl::kStride;
      constexpr int kStep = sizeof(T) == 2 ? 16 : 32;               // bytes per 8 channels
      // mean and (biased) variance in one walk over the row, as moments about the row's first
      // element (a sample of the distribution, so the subtraction of the squared mean loses at
      // most a bit or two)
      float pivot;
      {
        float x[8];
        pb_unpack8<T>(*reinterpret_cast<const uint4*>(row), *reinterpret_cast<const uint4*>(row + (sizeof(T) == 2 ? 0 : 16)), x);
        pivot = x[0];
      }
      const uint64_t npivot2 = pack_f32x2(-pivot, -pivot);
      uint64_t s1a = pack_f32x2(0.f, 0.f), s1b = s1a, s2a = s1a, s2b = s1a;
#pragma unroll 2
      for (int c8 = 0; c8 < kPbChannels / 8; ++c8) {
        float x[8];
        pb_unpack8<T>(*reinterpret_cast<const uint4*>(row + c8 * kStep),
                      *reinterpret_cast<const uint4*>(row + c8 * kStep + (sizeof(T) == 2 ? 0 : 16)), x);
        // packed f32x2 arithmetic: two channels per FMA-pipe instruction
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
      const float m1 = (s1lo + s1hi) * (1.0f / kPbChannels);
      const float mean = pivot + m1;
      const float var = fmaxf((s2lo + s2hi) * (1.0f / kPbChannels) - m1 * m1, 0.f);
      const float rstd = rsqrtf(var + p.eps);
      // y = x * A + B per channel with A = rstd * gamma, B = beta - mean * A
      const uint64_t rstd2 = pack_f32x2(rstd, rstd), nmean2 = pack_f32x2(-mean, -mean);
      uint64_t acc2[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) acc2[h] = pack_f32x2(0.f, 0.f);
#pragma unroll 2
      for (int c8 = 0; c8 < kPbChannels / 8; ++c8) {
        float x[8];
        pb_unpack8<T>(*reinterpret_cast<const uint4*>(row + c8 * kStep),
                      *reinterpret_cast<const uint4*>(row + c8 * kStep + (sizeof(T) == 2 ? 0 : 16)), x);
        uint32_t yw[4];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const ulonglong2 g4 = *reinterpret_cast<const ulonglong2*>(&s_c[c8 * 8 + 4 * q]);
          const ulonglong2 b4 = *reinterpret_cast<const ulonglong2*>(&s_c[kPbChannels + c8 * 8 + 4 * q]);
          const uint64_t a01 = mul_f32x2(g4.x, rstd2), a23 = mul_f32x2(g4.y, rstd2);
          const uint64_t y01 = fma_f32x2(pack_f32x2(x[4 * q], x[4 * q + 1]), a01, fma_f32x2(a01, nmean2, b4.x));
          const uint64_t y23 = fma_f32x2(pack_f32x2(x[4 * q + 2], x[4 * q + 3]), a23, fma_f32x2(a23, nmean2, b4.y));
          float y0, y1, y2, y3;
          unpack_f32x2(y01, y0, y1);
          unpack_f32x2(y23, y2, y3);
          yw[2 * q] = pb_pack_bf16x2(y0, y1);
          yw[2 * q + 1] = pb_pack_bf16x2(y2, y3);
          // the projection sees the rounded values
          const uint64_t r01 = pack_f32x2(__uint_as_float(yw[2 * q] << 16), __uint_as_float(yw[2 * q] & 0xffff0000u));
          const uint64_t r23 = pack_f32x2(__uint_as_float(yw[2 * q + 1] << 16), __uint_as_float(yw[2 * q + 1] & 0xffff0000u));
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const ulonglong2 w4 = *reinterpret_cast<const ulonglong2*>(&s_c[(2 + h) * kPbChannels + c8 * 8 + 4 * q]);
            acc2[h] = fma_f32x2(r23, w4.y, fma_f32x2(r01, w4.x, acc2[h]));
          }
        }
        // the bf16 result goes back over the part of the row that has been consumed
        *reinterpret_cast<uint4*>(s_rows + t * Tl::kStride + c8 * 16) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
      }
      float acc[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float lo, hi;
        unpack_f32x2(acc2[h], lo, hi);
        acc[h] = lo + hi;
      }
#pragma unroll
      for (int h = 0; h < 4; ++h) s_bias[h * Tl::kRows + t] = __float2bfloat16_rn(acc[h]);
    }
    __syncthreads();
    // ---- shared -> global, coalesced: normalised rows (256 bytes each), then the bias rows
    uint4* dst = reinterpret_cast<uint4*>(p.normed + vec0 * kPbChannels);
#pragma unroll 4
    for (int k = t; k < rows * 16; k += Tl::kRows)
      dst[k] = *reinterpret_cast<const uint4*>(s_rows + (k / 16) * Tl::kStride + (k % 16) * 16);
    for (int k = t; k < p.H * (Tl::kRows / 8); k += Tl::kRows) {
      const int h = k / (Tl::kRows / 8), seg = k % (Tl::kRows / 8);
      const int j = j0 + seg * 8;
      __nv_bfloat16* bd = p.bias + ((long long)h * p.R + i) * p.bias_pitch + j;
      if (j + 8 <= p.N) {
        *reinterpret_cast<uint4*>(bd) = *reinterpret_cast<const uint4*>(&s_bias[h * Tl::kRows + seg * 8]);
      } else {
        for (int e = 0; e < 8 && j + e < p.N; ++e) bd[e] = s_bias[h * Tl::kRows + seg * 8 + e];
      }
    }
    __syncthreads();   // the row buffer and s_bias are reused by the next tile
  }
}

// ---------------------------------------------------------------- bf16 pair, up to 16 heads: projection on the tensor core
// The thread-per-vector kernel above is bound by instruction issue, and a third of its
// instructions are the head projection (per channel and head one FMA and a share of a
// shared-memory read, on values unpacked again from their bf16 rounding).  That projection is a
// small GEMM, [128 vectors, 128 channels] x [128 channels, 16 heads], so here the tensor core does
// it: the tile sits in shared memory in the layout a tcgen05.mma A operand wants (K-major rows
// of 128 bytes, 128-byte swizzle, the two 64-channel halves 16 KB apart), thread t still walks
// over row t twice (moments; normalise and round, written back in place), one thread then issues
// eight MMAs (M 128, N 32, K 16) against the projection weights - each fp32 weight as a bf16 high
// part (B rows 0-15) plus a bf16 low part (rows 16-31), so that fp32 weights are not rounded to
// bf16 -, and while they run all threads copy the normalised tile out.  The accumulator (32 fp32
// columns of TMEM, lane = vector) comes back with one tcgen05.ld per thread; head h is column h
// plus column 16 + h.  The swizzle also keeps both the per-thread row walks
// and the coalesced copies free of bank conflicts, like the padding of the kernel above.
constexpr int kPbmRows = 128;                       // vectors per tile = threads per CTA
constexpr int kPbmHalfBytes = kPbmRows * 128;       // one 64-channel half of the tile
constexpr uint32_t kPbmTmemCols = 32;
// dynamic shared memory from a 1024-aligned base: tile, weights (same layout, 16 rows), gamma / beta,
// bias staging [16][128] bf16, mbarrier + TMEM address slot
constexpr int kPbmOffW = 2 * kPbmHalfBytes;
constexpr int kPbmWRows = 32;                       // B operand rows: 16 heads x {high, low} part
constexpr int kPbmOffC = kPbmOffW + 2 * kPbmWRows * 128;
constexpr int kPbmOffBias = kPbmOffC + 2 * kPbChannels * 4;
constexpr int kPbmOffBar = kPbmOffBias + kPbMaxHeads * kPbmRows * 2;
constexpr int kPbmSmemBytes = kPbmOffBar + 16 + 1024;

__device__ int g_pair_bias_status[4];   // {1 = a bounded wait ran out, block, tile (low word), 0}

__device__ __forceinline__ uint32_t pbm_swz(int row, int piece) {   // byte offset of 16-byte piece 0..15 of a row
  return (uint32_t)((piece >> 3) * kPbmHalfBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(kPbmRows, 5) pair_bias_mma_kernel(const PairBiasParams p, long long wait_limit) {
  extern __shared__ uint8_t pbm_raw[];
  const uint32_t base = (smem_u32(pbm_raw) + 1023u) & ~1023u;
  uint8_t* gbase = pbm_raw + (base - smem_u32(pbm_raw));
  float* s_c = reinterpret_cast<float*>(gbase + kPbmOffC);                       // gamma, beta
  __nv_bfloat16* s_bias = reinterpret_cast<__nv_bfloat16*>(gbase + kPbmOffBias);  // [16][128]
  const uint32_t bar = base + kPbmOffBar;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kPbmOffBar + 8);
  __shared__ int abort_flag;
  const int t = threadIdx.x, warp = t >> 5;

  if (t == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  s_c[t] = p.gamma[t];
  s_c[kPbChannels + t] = p.beta[t];
  // projection weights as the B operand: row = head (+ 16 for the low parts; absent heads zero), K = channel
  for (int k = t; k < kPbmWRows * 16; k += kPbmRows) {
    const int r = k >> 4, piece = k & 15, h = r & 15;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (h < p.H) {
      const float* src = p.proj + h * kPbChannels + piece * 8;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = src[2 * e], b = src[2 * e + 1];
        if (r >= 16) {   // what the bf16 high part leaves over
          a -= __bfloat162float(__float2bfloat16_rn(a));
          b -= __bfloat162float(__float2bfloat16_rn(b));
        }
        w[e] = pb_pack_bf16x2(a, b);
      }
    }
    const uint32_t off = (uint32_t)((piece >> 3) * (kPbmWRows * 128) + r * 128 + (((piece & 7) ^ (r & 7)) << 4));
    *reinterpret_cast<uint4*>(gbase + kPbmOffW + off) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(base + kPbmOffBar + 8, kPbmTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t idesc = make_idesc(1u, 1u, 0u, 0u, kPbmWRows);
  const uint64_t adesc = make_smem_desc(base, 16, 8 * 128, 2);
  const uint64_t bdesc = make_smem_desc(base + kPbmOffW, 16, 8 * 128, 2);

  const int tiles_j = (p.N + kPbmRows - 1) / kPbmRows;
  const long long n_tiles = (long long)p.R * tiles_j;
  uint32_t phase = 0;
  bool ok = true;
  for (long long tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
    const int i = (int)(tile / tiles_j);
    const int j0 = (int)(tile % tiles_j) * kPbmRows;
    const int rows = min(kPbmRows, p.N - j0);
    const long long vec0 = (long long)i * p.N + j0;
    // global -> shared, coalesced, as asynchronous 16-byte copies into the swizzled positions
    {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.pair) + vec0 * kPbChannels);
      for (int k = t; k < rows * 16; k += kPbmRows)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + pbm_swz(k >> 4, k & 15)), "l"(src + k) : "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    {
      // rows beyond the sequence are normalised too (whatever the buffer holds; finite after the
      // clamp below) so that the MMA reads defined values; they are never stored
      const bool live = t < rows;
      float pivot;
      {
        float x[8];
        pb_unpack8<__nv_bfloat16>(*reinterpret_cast<const uint4*>(gbase + pbm_swz(t, 0)), make_uint4(0, 0, 0, 0), x);
        pivot = live ? x[0] : 0.f;
      }
      const uint64_t npivot2 = pack_f32x2(-pivot, -pivot);
      uint64_t s1a = pack_f32x2(0.f, 0.f), s1b = s1a, s2a = s1a, s2b = s1a;
#pragma unroll 4
      for (int c8 = 0; c8 < 16; ++c8) {
        float x[8];
        pb_unpack8<__nv_bfloat16>(*reinterpret_cast<const uint4*>(gbase + pbm_swz(t, c8)), make_uint4(0, 0, 0, 0), x);
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
      const float m1 = (s1lo + s1hi) * (1.0f / kPbChannels);
      const float mean = live ? pivot + m1 : 0.f;
      const float var = fmaxf((s2lo + s2hi) * (1.0f / kPbChannels) - m1 * m1, 0.f);
      const float rstd = live ? rsqrtf(var + p.eps) : 0.f;
      // z = (x - mean) * rstd as one FMA, y = z * gamma + beta as another
      const uint64_t rstd2 = pack_f32x2(rstd, rstd);
      const float nmr = -mean * rstd;
      const uint64_t nmr2 = pack_f32x2(nmr, nmr);
#pragma unroll 4
      for (int c8 = 0; c8 < 16; ++c8) {
        const uint32_t off = pbm_swz(t, c8);
        float x[8];
        pb_unpack8<__nv_bfloat16>(*reinterpret_cast<const uint4*>(gbase + off), make_uint4(0, 0, 0, 0), x);
        uint32_t yw[4];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const ulonglong2 g4 = *reinterpret_cast<const ulonglong2*>(&s_c[c8 * 8 + 4 * q]);
          const ulonglong2 b4 = *reinterpret_cast<const ulonglong2*>(&s_c[kPbChannels + c8 * 8 + 4 * q]);
          const uint64_t z01 = fma_f32x2(pack_f32x2(x[4 * q], x[4 * q + 1]), rstd2, nmr2);
          const uint64_t z23 = fma_f32x2(pack_f32x2(x[4 * q + 2], x[4 * q + 3]), rstd2, nmr2);
          float y0, y1, y2, y3;
          unpack_f32x2(fma_f32x2(z01, g4.x, b4.x), y0, y1);
          unpack_f32x2(fma_f32x2(z23, g4.y, b4.y), y2, y3);
          yw[2 * q] = pb_pack_bf16x2(y0, y1);
          yw[2 * q + 1] = pb_pack_bf16x2(y2, y3);
        }
        *reinterpret_cast<uint4*>(gbase + off) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
      }
    }
    fence_proxy_async_smem();     // the tile was written through the generic proxy; the tensor core reads it
    __syncthreads();
    if (t == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 8; ++k) {   // 16 channels per step: 32 bytes inside a half, halves 16 KB / 4 KB apart
        const uint32_t a_off = (uint32_t)(((k >> 2) * kPbmHalfBytes + (k & 3) * 32) >> 4);
        const uint32_t b_off = (uint32_t)(((k >> 2) * (kPbmWRows * 128) + (k & 3) * 32) >> 4);
        mma_ss_f16(tmem, (uint32_t)adesc + a_off, (uint32_t)(adesc >> 32), (uint32_t)bdesc + b_off,
                   (uint32_t)(bdesc >> 32), idesc, k > 0 ? 1u : 0u);
      }
      tc_commit(bar);
    }
    // while the MMAs run: shared -> global, coalesced, the normalised rows (256 bytes each)
    {
      uint4* dst = reinterpret_cast<uint4*>(p.normed + vec0 * kPbChannels);
#pragma unroll 4
      for (int k = t; k < rows * 16; k += kPbmRows)
        dst[k] = *reinterpret_cast<const uint4*>(gbase + pbm_swz(k >> 4, k & 15));
    }
    ok = mbar_wait_bounded(bar, phase, wait_limit, &abort_flag);
    phase ^= 1;
    if (!__all_sync(0xffffffffu, ok)) {
      abort_flag = 1;
      if (atomicCAS(&g_pair_bias_status[0], 0, 1) == 0) {
        g_pair_bias_status[1] = blockIdx.x;
        g_pair_bias_status[2] = (int)tile;
      }
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      uint32_t acc[32];
      tmem_ld_x32(tmem + ((uint32_t)(warp * 32) << 16), acc);
      tc_wait_ld();
      tc_fence_before();
#pragma unroll
      for (int h = 0; h < kPbMaxHeads; ++h)
        if (h < p.H) s_bias[h * kPbmRows + t] = __float2bfloat16_rn(__uint_as_float(acc[h]) + __uint_as_float(acc[16 + h]));
    }
    __syncthreads();    // s_bias complete; every thread is past its reads of the tile and of TMEM
    if (abort_flag != 0) break;
    for (int k = t; k < p.H * (kPbmRows / 8); k += kPbmRows) {
      const int h = k / (kPbmRows / 8), seg = k % (kPbmRows / 8);
      const int j = j0 + seg * 8;
      __nv_bfloat16* bd = p.bias + ((long long)h * p.R + i) * p.bias_pitch + j;
      if (j + 8 <= p.N) {
        *reinterpret_cast<uint4*>(bd) = *reinterpret_cast<const uint4*>(&s_bias[h * kPbmRows + seg * 8]);
      } else {
        for (int e = 0; e < 8 && j + e < p.N; ++e) bd[e] = s_bias[h * kPbmRows + seg * 8 + e];
      }
    }
    __syncthreads();   // the tile buffer and s_bias are reused by the next tile
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    for (int k = 0; k < 100; ++k) __nanosleep(10000);   // let MMAs still in flight finish before TMEM goes away
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kPbmTmemCols);
  }
}

// ---------------------------------------------------------------- sigmoid gate
// out = weighted * sigmoid(gate), elementwise over bf16 tensors of n elements (n a multiple of 8,
// pointers 16-byte aligned).  Stands in for the SigmoidFwdTPP + MulTPP pair behind the core in the
// reference's fused blocks (src/csrc/dot_product_attention.cpp:339-345 and :522-528).  The
// sigmoid is taken in fp32 and only the product is rounded (the reference rounds the sigmoid to
// bf16 first).  HBM-bound: 4 bytes read and 2 written per element.
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const uint4* __restrict__ weighted,
                                                           const uint4* __restrict__ gate,
                                                           uint4* __restrict__ out, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 a = weighted[i], g = gate[i];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a0 = __uint_as_float(aw[e] << 16), a1 = __uint_as_float(aw[e] & 0xffff0000u);
      const float g0 = __uint_as_float(gw[e] << 16), g1 = __uint_as_float(gw[e] & 0xffff0000u);
      // sigmoid(x) = 1 / (1 + 2^(-x log2 e))
      const float s0 = __frcp_rn(1.0f + ex2_approx(-1.4426950408889634f * g0));
      const float s1 = __frcp_rn(1.0f + ex2_approx(-1.4426950408889634f * g1));
      r[e] = pb_pack_bf16x2(a0 * s0, a1 * s1);
    }
    out[i] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

}  // namespace af3k
