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
// HBM-bound: 2 or 4 bytes read and 2 bytes written per pair element, plus H * 2 bytes per
// (i, j).  One warp normalises one 128-channel vector (4 channels per lane, statistics by
// shuffles in fp32; with up to four heads 8 lanes share a vector); persistent CTAs walk over tiles
// of 128 consecutive j of one row i and stage each tile's H x 128 bias values in shared memory so
// that they leave as 256-byte rows.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

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

// ---------------------------------------------------------------- up to 4 heads: 8 lanes per vector
// The kernel above spends most of its instructions on 32-lane reductions (about 150 warp
// instructions per vector against 44 of arithmetic), which makes it issue-bound at under half of
// the HBM rate.  With at most four heads the weights of 16 channels fit a lane's registers, so
// here 8 lanes share a vector (16 channels each, as two 16-byte pieces 128 bytes apart, so that
// the 8 lanes of a load cover 128 contiguous bytes) and a warp works on 4 vectors at once:
// reductions take 3 steps, and all control is amortised over 4 vectors.
template <int kN>
__device__ __forceinline__ void octet_sum_scatter(float (&a)[kN], int lane) {
  static_assert(kN == 1 || kN == 2 || kN == 4, "power of two up to 4");
  int off = 4;
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
__device__ __forceinline__ float octet_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kPbThreads, 2) pair_bias_kernel_h4(const PairBiasParams p) {
  __shared__ __nv_bfloat16 s_bias[4][kPbTileJ];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sl = lane & 7;          // vector within the warp's four, lane within the vector
  // this lane's channels: [ca, ca + 8) and [cb, cb + 8)
  const int ca = sl * 8, cb = 64 + sl * 8;

  // LayerNorm parameters and projection weights live in shared memory (3 KB): held in registers
  // they cost 96 per thread, which left too few resident warps to cover the latencies
  __shared__ __align__(16) float s_g[kPbChannels], s_b[kPbChannels], s_w[4][kPbChannels];
  for (int c = threadIdx.x; c < kPbChannels; c += kPbThreads) {
    s_g[c] = p.gamma[c];
    s_b[c] = p.beta[c];
#pragma unroll
    for (int h = 0; h < 4; ++h) s_w[h][c] = h < p.H ? p.proj[h * kPbChannels + c] : 0.f;
  }
  __syncthreads();

  constexpr int kWarps = kPbThreads / 32;
  const int tiles_j = (p.N + kPbTileJ - 1) / kPbTileJ;
  const long long n_tiles = (long long)p.R * tiles_j;
  for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {   // persistent: constants loaded once
  const int i = (int)(tile / tiles_j);
  const int j0 = (int)(tile % tiles_j) * kPbTileJ;
  const long long row_base = (long long)i * p.N;
  // The warp's four passes over the tile: the raw loads of kDepth passes are issued before the
  // first is worked on, so that enough bytes are in flight per SM to cover the HBM latency.
  constexpr int kPasses = kPbTileJ / (kWarps * 4);
  constexpr int kDepth = 2;
  static_assert(kPasses % kDepth == 0, "passes per tile must be a multiple of the prefetch depth");
#pragma unroll 1
  for (int pass0 = 0; pass0 < kPasses; pass0 += kDepth) {
  uint4 raw[kDepth][sizeof(T) == 2 ? 2 : 4];
#pragma unroll
  for (int dpt = 0; dpt < kDepth; ++dpt) {
    const int j = j0 + (pass0 + dpt) * kWarps * 4 + warp * 4 + grp;
    if (j < p.N) {
      const long long off = (row_base + j) * kPbChannels;
      if (sizeof(T) == 4) {
        const float* src = static_cast<const float*>(p.pair) + off;
        raw[dpt][0] = *reinterpret_cast<const uint4*>(src + ca);
        raw[dpt][1] = *reinterpret_cast<const uint4*>(src + ca + 4);
        raw[dpt][2] = *reinterpret_cast<const uint4*>(src + cb);
        raw[dpt][3] = *reinterpret_cast<const uint4*>(src + cb + 4);
      } else {
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.pair) + off;
        raw[dpt][0] = *reinterpret_cast<const uint4*>(src + ca);
        raw[dpt][1] = *reinterpret_cast<const uint4*>(src + cb);
      }
    } else {
#pragma unroll
      for (int r = 0; r < (sizeof(T) == 2 ? 2 : 4); ++r) raw[dpt][r] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int dpt = 0; dpt < kDepth; ++dpt) {
    const int jl = (pass0 + dpt) * kWarps * 4 + warp * 4 + grp;   // vector within the CTA's tile
    const int j = j0 + jl;
    const bool live = j < p.N;
    float x[16];
    if (sizeof(T) == 4) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        x[4 * r + 0] = __uint_as_float(raw[dpt][r].x); x[4 * r + 1] = __uint_as_float(raw[dpt][r].y);
        x[4 * r + 2] = __uint_as_float(raw[dpt][r].z); x[4 * r + 3] = __uint_as_float(raw[dpt][r].w);
      }
    } else {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t ww[4] = {raw[dpt][r].x, raw[dpt][r].y, raw[dpt][r].z, raw[dpt][r].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x[8 * r + 2 * e] = __uint_as_float(ww[e] << 16);
          x[8 * r + 2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
        }
      }
    }
    // mean and (biased) variance over the 128 channels, two-pass in registers
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) sum += x[e];
    const float mean = octet_sum(sum) * (1.0f / kPbChannels);
    float sq = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) { x[e] -= mean; sq += x[e] * x[e]; }
    const float rstd = rsqrtf(octet_sum(sq) * (1.0f / kPbChannels) + p.eps);
    // y = bf16(d * rstd * gamma + beta): written as the normalised pair and, as those same rounded
    // values, the operand of the bias projection
    uint32_t yw[8];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {       // four channels at a time: x[4 q4 ..] are channels cq ..
      const int cq = (q4 < 2 ? ca : cb) + 4 * (q4 & 1);
      const float4 g4 = *reinterpret_cast<const float4*>(&s_g[cq]);
      const float4 b4 = *reinterpret_cast<const float4*>(&s_b[cq]);
      yw[2 * q4] = pb_pack_bf16x2(x[4 * q4] * rstd * g4.x + b4.x, x[4 * q4 + 1] * rstd * g4.y + b4.y);
      yw[2 * q4 + 1] = pb_pack_bf16x2(x[4 * q4 + 2] * rstd * g4.z + b4.z, x[4 * q4 + 3] * rstd * g4.w + b4.w);
    }
    if (live) {
      __nv_bfloat16* dst = p.normed + (row_base + j) * kPbChannels;
      *reinterpret_cast<uint4*>(dst + ca) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
      *reinterpret_cast<uint4*>(dst + cb) = make_uint4(yw[4], yw[5], yw[6], yw[7]);
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const int cq = (q4 < 2 ? ca : cb) + 4 * (q4 & 1);
      const float y0 = __uint_as_float(yw[2 * q4] << 16), y1 = __uint_as_float(yw[2 * q4] & 0xffff0000u);
      const float y2 = __uint_as_float(yw[2 * q4 + 1] << 16), y3 = __uint_as_float(yw[2 * q4 + 1] & 0xffff0000u);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float4 w4 = *reinterpret_cast<const float4*>(&s_w[h][cq]);
        acc[h] = fmaf(y3, w4.w, fmaf(y2, w4.z, fmaf(y1, w4.y, fmaf(y0, w4.x, acc[h]))));
      }
    }
    octet_sum_scatter<4>(acc, lane);
    // lanes 0, 2, 4, 6 of the octet hold heads 0, 1, 2, 3
    if ((sl & 1) == 0) s_bias[sl >> 1][jl] = __float2bfloat16_rn(acc[0]);
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

}  // namespace af3k
