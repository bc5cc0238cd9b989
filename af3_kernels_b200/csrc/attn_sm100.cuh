// Biased, key-masked flash attention for sm_100a:  out = softmax(scale * Q K^T + bias, masked) V
//
// Replaces the per-(batch, head, 128-query block) TPP sequence of the reference
// (src/csrc/dot_product_attention.cpp:88-122: scale -> BRGEMM -> add bias -> add mask ->
// softmax -> BRGEMM) with one persistent warp-specialised kernel:
//
//   warp 0      TMA producer: Q tiles, K/V ring, bias ring (cp.async.bulk.tensor, each CTA loads its own tiles)
//   warp 1      tcgen05.mma issuer for the logits (smem x smem -> TMEM)
//   warp 2      TMEM allocator, then tcgen05.mma issuer for O += P V (TMEM x smem -> TMEM); Q scaler
//   warp 3      key-mask writer (see below)
//   warps 4-7   softmax warpgroup 0 (owns S / P buffer 0 and the even streams of a work item)
//   warps 8-11  softmax warpgroup 1 (owns S / P buffer 1 and the odd streams)
//
// A work item is (head, 128-query tile, group of G pair rows).  The G "streams" of an item use
// the same bias tiles, so one staged bias tile serves G logits tiles; each stream has its own
// Q tile, K/V tiles, fp32 running max / sum and O accumulator in TMEM.  One softmax thread owns
// one query row (TMEM lane), so row max / row sum need no cross-thread traffic.
//
// The softmax threads are the bottleneck of this operator (one exponential per logit on the
// 16-lane XU, every other instruction competing for the same issue slots), so everything that
// can be an MMA is one.  With bf16 q/k the whole logit comes out of the tensor core:
//
//   * scale: warp 2 multiplies each Q tile by the softmax scale in shared memory and rounds it
//     back to bf16 - the reference's own first step (q = q * scaling, in bf16);
//   * bias: eight small MMAs per tile (M = 128, N = 16, K = 16) whose A operand is a 16-key
//     slice of the staged bf16 bias tile and whose B operand is a 16 x 16 identity, each adding
//     its slice into 16 columns of the accumulator - exact, the products are bias x 1;
//   * key mask: one more K step whose A operand is a column of ones and whose B operand holds,
//     per key, 0 (attend), -2^47 (masked) or -inf (beyond the sequence).  A masked key ends up
//     with weight exactly 0, a row whose keys are all masked with uniform weights over its real
//     keys (what "fill with -1e9, then softmax" gives), a key that does not exist with weight 0.
//
// What is left per logit is a maximum, one fused multiply-add, the exponential, the row sum and
// the bf16 rounding of P.  With fp8 q/k the logit scale t = softmax scale x the two
// de-quantisation factors cannot be folded into Q; there the bias staging pass divides the bias
// by t, the tensor core adds it to the raw fp8 products, the masked-key value is enlarged by 1/t,
// and t rides on the fused multiply-add.  When the caller gives no room for that staging copy
// the second instantiation of the kernel runs, in which the softmax threads apply t and add the
// bias in fp32 from the staged tile in shared memory; the mask column is used either way.
//
// Logits stay fp32 from the tensor core to the exponential; P is rounded to bf16 once, when it
// is written to TMEM as the A operand of the second GEMM.  S and P live in separate TMEM columns:
// a warpgroup releases its S buffer as soon as the logits are in registers, so the next logits
// tile of that buffer is computed under the softmax of the current one.  O is rescaled lazily:
// only when a row maximum grows by more than 2^8 (exact, because l is scaled with it).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace af3k {

constexpr int kTile = 128;         // query rows per tile == keys per tile
constexpr int kThreads = 384;      // 12 warps
// 65536 registers per SM: launched at 168 per thread, then 128 x 56 + 256 x 224 = 64512
constexpr int kRegsMisc = 56, kRegsSoftmax = 224;
constexpr int kMaxStreams = 4;     // pair rows per work item (two per softmax warpgroup; TMEM: kOCol + G * nv <= 512 columns)
// TMEM columns: two fp32 logits buffers, two bf16 P buffers (two keys per column), then O.
constexpr uint32_t kSCol = 0, kPCol = 2 * 128, kOCol = 2 * 128 + 2 * 64;
constexpr float kLazyRescaleLog2 = 8.0f;   // keep a stale row max while exp2 arguments stay <= 8
constexpr int kBiasStages = 2;
constexpr int kBiasTileBytes = kTile * kTile * 2;  // bf16, two 128B-swizzled boxes of 64 columns
constexpr int kMaxKvStages = 6;
constexpr uint32_t kTmemCols = 512;
// bf16 bit patterns of the mask column.  -2^47 stands in for the reference's "-1e9" fill: added
// in fp32 to any logit below 2^23 in magnitude it gives exactly -2^47, so all masked keys of a
// row are equal (uniform weights when nothing else is left) and vanish next to any real key.
constexpr uint16_t kMaskColKeep = 0x0000, kMaskColMasked = 0xD700, kMaskColAbsent = 0xFF80;
constexpr uint32_t kMaskPanelBytes = 2048;   // 128 keys x one 16-byte core-matrix row
constexpr uint32_t kBarrierBlockBytes = 512;
constexpr uint32_t kIdentBytes = 512;        // 16 x 16 bf16 identity, K-major core matrices
constexpr float kLog2e = 1.4426950408889634f;

// Exponentials: every weight is one ex2.approx.f32 on the XU (16 lanes per SM and clock: 4 results per
// clock and scheduler).  Measured alternatives that do not beat it here: ex2.approx.f16x2 / .bf16x2 take
// 16 XU cycles per warp instruction (the same 4 results per clock), kind::f16 MMAs take no f16 A with a
// bf16 B, and a degree-3 polynomial on the FMA pipe costs more issue slots than the ex2 it replaces.

enum StatusBits : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,   // a bounded mbarrier wait ran out
};

struct AttnParams {
  int B1, B2, Sq, Sk, D;
  int n_qt, n_kt;
  int G;                 // pair rows per work item
  int q_split;           // 1: the streams of an item are two neighbouring query tiles of ONE pair row (G == 1)
  int n_streams;         // streams per work item: G, or 2 with q_split
  int n_items;
  int qk_row_bytes;      // smem bytes per Q / K tile row: 32, 64 or 128 (= swizzle span)
  int v_row_bytes;       // same for V
  int qk_ksteps;         // number of 32-byte K steps of the first GEMM
  int nv;                // N of the second GEMM: D rounded up to 16
  int kv_stages;
  int q_buffers;         // 2: Q tiles double-buffered by item (the next item's land while this one runs); 1: single
  int qk_is_fp8;
  int scale_q;           // 1: bf16 q/k, the Q tiles are multiplied by `scale` in shared memory
  float scale;           // softmax scale; multiplied by q_scale[h] * k_scale[h] when those are set
  const float* q_scale;
  const float* k_scale;
  const uint8_t* mask;   // 1 = attend; nullptr = no mask
  long long mask_row_stride;
  __nv_bfloat16* out;
  long long out_stride_b1, out_stride_b2, out_stride_s;
  int* status;           // int[4]: {status bits, 1 + first barrier slot that timed out, block, warp}
  long long wait_limit;  // SM clocks a single wait may take before the kernel gives up
  float* debug;          // diagnostic dump of block 0's first logits tile (debug build of the kernel)
  uint32_t q_tile_bytes, k_tile_bytes, v_tile_bytes;
  uint32_t off_q, off_kv, off_bias, off_bar;   // from the 1024-aligned smem base
  // mask-column operands of the extra K step (all no-swizzle, K-major, 16-byte rows):
  //   off_ones: A operand, element (row, 0) = 1;  off_mcol: ring of per-tile B operands, element
  //   (key, 0) = mask value;  off_zero: the all-zero second half of K shared by both.
  uint32_t off_ones, off_mcol, off_zero;
  uint32_t off_ident;    // 16 x 16 identity (B operand of the bias MMAs)
  int mask_col;          // 1: the extra K step runs (a mask was given or Sk is not a tile multiple)
};

// Barrier slots inside the barrier block (8 bytes each, kBarrierBlockBytes in all).
struct BarIdx {
  static constexpr int s_full = 0;      // [2]  logits of a tile finished
  static constexpr int s_free = 2;      // [2]  softmax warpgroup has the logits in registers
  static constexpr int p_ready = 4;     // [2]  P written (and O rescaled if needed)
  static constexpr int epi_done = 6;    // [2]  warpgroup has read its O accumulators of the item
  static constexpr int bias_full = 8;   // [kBiasStages]
  static constexpr int bias_empty = 10; // [kBiasStages]
  static constexpr int kv_full = 12;    // [kMaxKvStages]
  static constexpr int kv_empty = 12 + kMaxKvStages;       // P V of the stage's tile finished
  // Q tiles: slot = (Q buffer) * kMaxStreams + stream
  static constexpr int q_full = 12 + 2 * kMaxKvStages;       // [2 * kMaxStreams]  Q tile landed
  static constexpr int q_empty = q_full + 2 * kMaxStreams;   // [2 * kMaxStreams]  last Q K^T of the stream finished
  static constexpr int q_scaled = q_empty + 2 * kMaxStreams; // [2 * kMaxStreams]  the P V warp has scaled the Q tile
  static constexpr int count = q_scaled + 2 * kMaxStreams;
};
static_assert(BarIdx::count * 8 <= (int)kBarrierBlockBytes, "barrier block too small");

// Diagnostic dump: four [128][128] float sections, row = query row of block 0's first tile:
// raw logits, packed P words (64 used), un-normalised O (nv used), {running max, running sum}.
constexpr int kDbgTimelineTiles = 256;   // per warpgroup; 8 clock values each, after kDbgFloats floats
constexpr int kDbgS = 0, kDbgP = kTile * kTile, kDbgO = 2 * kTile * kTile, kDbgML = 3 * kTile * kTile,
              kDbgFloats = 4 * kTile * kTile;

struct Ctx {
  const AttnParams* p;
  uint32_t smem;       // 1024-aligned shared base (shared-window address)
  uint32_t bars;       // shared address of barrier block
  volatile int* abort_flag;
  uint32_t tmem;       // TMEM base address
};

__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int idx) { return c.bars + 8u * idx; }

__device__ __noinline__ void report_timeout(const Ctx& c, int bar_idx) {
  *c.abort_flag = 1;
  if (c.p->status != nullptr) {
    atomicOr(c.p->status, kStatusWaitTimeout);
    if (atomicCAS(c.p->status + 1, 0, bar_idx + 1) == 0) {
      c.p->status[2] = blockIdx.x;
      c.p->status[3] = threadIdx.x >> 5;
    }
  }
}

#define AF3K_WAIT(ctx, idx, parity)                                                          \
  do {                                                                                       \
    if (!mbar_wait_bounded(bar_addr(ctx, idx), (parity), (ctx).p->wait_limit,                \
                           (ctx).abort_flag)) {                                              \
      report_timeout(ctx, idx);                                                              \
      return;                                                                                \
    }                                                                                        \
  } while (0)

// Form for helpers that report failure through their return value.
#define AF3K_WAIT_NORET(ctx, idx, parity)                                                    \
  do {                                                                                       \
    if (!mbar_wait_bounded(bar_addr(ctx, idx), (parity), (ctx).p->wait_limit,                \
                           (ctx).abort_flag)) {                                              \
      report_timeout(ctx, idx);                                                              \
      return false;                                                                          \
    }                                                                                        \
  } while (0)

// Warp-collective form: every lane leaves together, so no .sync.aligned instruction is ever
// executed by part of a warp after a timeout.
// The same for the single-warp roles, with the waiting loop out of line: these warps run their
// per-tile loops rarely, next to warps that stream through long unrolled loops, and one pass of
// such a loop costs 700 - 1 500 cycles whatever it does, so the path taken when nothing has to be
// waited for is kept short.
#define AF3K_WAIT_WARP_C(ctx, idx, parity)                                                   \
  do {                                                                                       \
    const bool ok_ = mbar_wait_bounded_compact(bar_addr(ctx, idx), (parity), (ctx).p->wait_limit, \
                                               (ctx).abort_flag);                            \
    if (!__all_sync(0xffffffffu, ok_)) {                                                     \
      report_timeout(ctx, idx);                                                              \
      return;                                                                                \
    }                                                                                        \
  } while (0)

#define AF3K_WAIT_WARP(ctx, idx, parity)                                                     \
  do {                                                                                       \
    const bool ok_ = mbar_wait_bounded(bar_addr(ctx, idx), (parity), (ctx).p->wait_limit,    \
                                       (ctx).abort_flag);                                    \
    if (!__all_sync(0xffffffffu, ok_)) {                                                     \
      report_timeout(ctx, idx);                                                                \
      return;                                                                                \
    }                                                                                        \
  } while (0)

__device__ __forceinline__ uint32_t swizzle_layout_code(int row_bytes) {
  return row_bytes == 128 ? 2u : (row_bytes == 64 ? 4u : 6u);
}

// A work item: head h, first query tile qt, first pair row r0, gv streams.  Normally the streams
// are gv pair rows sharing one query tile index (and therefore one bias tile per key tile).  With
// q_split (chosen when there is a single pair row per item, so that the second softmax warpgroup
// is not left idle) they are gv neighbouring query tiles of pair row r0, each with its own bias
// tiles.
struct Item {
  int qt, h, r0, gv;
};
__device__ __forceinline__ Item decode_item(const AttnParams& p, int item) {
  Item it;
  const int nq = p.q_split ? (p.n_qt + 1) >> 1 : p.n_qt;
  it.qt = (item % nq) << p.q_split;
  int t = item / nq;
  it.h = t % p.B2;
  int rg = t / p.B2;
  it.r0 = rg * p.G;
  it.gv = p.q_split ? min(2, p.n_qt - it.qt) : min(p.G, p.B1 - it.r0);
  return it;
}
__device__ __forceinline__ int stream_row(const AttnParams& p, const Item& it, int s) { return p.q_split ? it.r0 : it.r0 + s; }
__device__ __forceinline__ int stream_qt(const AttnParams& p, const Item& it, int s) { return p.q_split ? it.qt + s : it.qt; }

// Q buffer of the CTA's j-th item and how often that buffer was used before.
__device__ __forceinline__ uint32_t q_buf(const AttnParams& p, uint32_t j) { return p.q_buffers == 2 ? (j & 1u) : 0u; }
__device__ __forceinline__ uint32_t q_use(const AttnParams& p, uint32_t j) { return p.q_buffers == 2 ? (j >> 1) : j; }

// ------------------------------------------------------------------ producer (one thread)
__device__ void producer_role(const Ctx& c, const CUtensorMap* tm_q, const CUtensorMap* tm_k,
                              const CUtensorMap* tm_v, const CUtensorMap* tm_bias) {
  const AttnParams& p = *c.p;
  uint32_t ucount = 0, bcount = 0, icount = 0;
  const uint32_t nkv = p.kv_stages;
  // With two Q buffers the tiles of the next item are requested while the current item runs, so
  // that they are in place (and scaled) when it ends; with one (tiles too large for two), as
  // soon as the current item's K/V loads are all issued.
  auto load_q = [&](const Item& it, uint32_t j) {
    const uint32_t buf = q_buf(p, j), use = q_use(p, j);
    for (int s = 0; s < it.gv; ++s) {
      const int slot = (int)buf * kMaxStreams + s;
      // the buffer's previous user must have finished its last Q K^T of this stream
      if (use >= 1) AF3K_WAIT_NORET(c, BarIdx::q_empty + slot, (use - 1) & 1);
      mbar_arrive_expect_tx(bar_addr(c, BarIdx::q_full + slot), p.q_tile_bytes);
      tma_load_4d(c.smem + p.off_q + (buf * p.n_streams + s) * p.q_tile_bytes, tm_q, bar_addr(c, BarIdx::q_full + slot),
                  0, stream_qt(p, it, s) * kTile, it.h, stream_row(p, it, s));
    }
    return true;
  };
  if ((int)blockIdx.x < p.n_items) {
    if (!load_q(decode_item(p, blockIdx.x), 0)) return;
  }
  for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++icount) {
    const Item it = decode_item(p, item);
    for (int kt = 0; kt < p.n_kt; ++kt) {
      for (int s = 0; s < it.gv; ++s) {
        if (s == 0 || p.q_split) {   // one bias tile per key tile, or per stream when the streams are query tiles
          const uint32_t bst = bcount % kBiasStages;
          if (bcount >= kBiasStages)
            AF3K_WAIT(c, BarIdx::bias_empty + bst, ((bcount / kBiasStages) - 1) & 1);
          const uint32_t bfull = bar_addr(c, BarIdx::bias_full + bst);
          const uint32_t bdst = c.smem + p.off_bias + bst * kBiasTileBytes;
          mbar_arrive_expect_tx(bfull, kBiasTileBytes);
          tma_load_3d(bdst, tm_bias, bfull, kt * kTile, stream_qt(p, it, s) * kTile, it.h);
          tma_load_3d(bdst + kBiasTileBytes / 2, tm_bias, bfull, kt * kTile + 64, stream_qt(p, it, s) * kTile, it.h);
          ++bcount;
        }
        const uint32_t st = ucount % nkv;
        if (ucount >= nkv) AF3K_WAIT(c, BarIdx::kv_empty + st, ((ucount / nkv) - 1) & 1);
        const uint32_t full = bar_addr(c, BarIdx::kv_full + st);
        const uint32_t kdst = c.smem + p.off_kv + st * (p.k_tile_bytes + p.v_tile_bytes);
        mbar_arrive_expect_tx(full, p.k_tile_bytes + p.v_tile_bytes);
        tma_load_4d(kdst, tm_k, full, 0, kt * kTile, it.h, stream_row(p, it, s));
        tma_load_4d(kdst + p.k_tile_bytes, tm_v, full, 0, kt * kTile, it.h, stream_row(p, it, s));
        ++ucount;
      }
      if (kt == (p.q_buffers == 2 ? 0 : p.n_kt - 1) && item + (int)gridDim.x < p.n_items) {
        if (!load_q(decode_item(p, item + gridDim.x), icount + 1)) return;
      }
    }
  }
}

// ------------------------------------------------------------------ Q scaling and key-mask column
// q <- bf16(q * scale) for 1 KB of a Q tile in shared memory, 32 bytes per lane (any swizzle: the
// operation is elementwise).
__device__ __forceinline__ void scale_q_chunk(uint32_t addr, float scale, int lane) {
  uint32_t w[8];
  const uint32_t a = addr + lane * 16;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(a));
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(a + 512));
#pragma unroll
  for (int e = 0; e < 8; ++e)
    w[e] = pack_bf16x2(__uint_as_float(w[e] << 16) * scale, __uint_as_float(w[e] & 0xffff0000u) * scale);
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]) : "memory");
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a + 512), "r"(w[4]), "r"(w[5]),
               "r"(w[6]), "r"(w[7]) : "memory");
}

// The 128 mask-column values (bf16) of one logits tile, four per lane.
__device__ __forceinline__ void mask_values(const AttnParams& p, const Item& it, int kt, int s, int lane,
                                            uint16_t masked, uint16_t (&val)[4]) {
  const uint8_t* mrow = p.mask != nullptr ? p.mask + (long long)stream_row(p, it, s) * p.mask_row_stride : nullptr;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int key = kt * kTile + 32 * g + lane;
    val[g] = key >= p.Sk ? kMaskColAbsent : ((mrow == nullptr || mrow[key] != 0) ? kMaskColKeep : masked);
  }
}

// bf16 bits of the value a masked key gets for head h.  The tensor core's logits are multiplied
// by the head's logit scale t afterwards when that scale is not folded into Q (fp8 q/k), so the
// value is -2^(47 + ceil(-log2 t)) there: still -2^47 or beyond after the multiplication.
__device__ __forceinline__ uint16_t masked_value_bits(const AttnParams& p, int h) {
  if (p.q_scale == nullptr) return kMaskColMasked;
  const float t = p.scale * p.q_scale[h] * p.k_scale[h];
  int e = 47 - min(0, ilogbf(t));
  e = min(e, 120);
  return (uint16_t)(0x8000u | ((uint32_t)(e + 127) << 7));
}

// Scaling of Q tiles, cut into 1 KB pieces so that the warp doing it (the P V issuer, which
// mostly waits) can fit the pieces into its waiting time.
struct QScaler {
  uint32_t item = 0, chunk = 0;   // item index (per CTA) of the tiles being scaled, next piece
  int gv = 0, tile = 0;           // tiles that item has, next tile
  __device__ __forceinline__ void start(uint32_t j, int n) { item = j; gv = n; tile = 0; chunk = 0; }
  __device__ __forceinline__ bool pending() const { return tile < gv; }
  // One piece.  block: wait (bounded) for the tile to land, else give up if it has not.
  // Returns 1 = did a piece, 0 = nothing to do (now), -1 = a wait ran out.
  __device__ __forceinline__ int step(const Ctx& c, int lane, bool block) {
    const AttnParams& p = *c.p;
    if (tile >= gv) return 0;
    const uint32_t buf = q_buf(p, item);
    const int slot = (int)buf * kMaxStreams + tile;
    if (chunk == 0) {
      const uint32_t par = q_use(p, item) & 1;
      bool ok = mbar_test_wait(bar_addr(c, BarIdx::q_full + slot), par);
      if (!__all_sync(0xffffffffu, ok)) {
        if (!block) return 0;
        ok = mbar_wait_bounded(bar_addr(c, BarIdx::q_full + slot), par, p.wait_limit, c.abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          report_timeout(c, BarIdx::q_full + slot);
          return -1;
        }
      }
    }
    scale_q_chunk(c.smem + p.off_q + (buf * p.n_streams + tile) * p.q_tile_bytes + (chunk << 10), p.scale, lane);
    if (++chunk == (p.q_tile_bytes >> 10)) {
      fence_proxy_async_smem();    // make the generic-proxy stores visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::q_scaled + slot));
      chunk = 0;
      ++tile;
    }
    return 1;
  }
};

// Waits for a barrier phase; while it is pending, does Q scaling pieces (if any are left).
#define AF3K_WAIT_WARP_OR_SCALE(ctx, idx, parity, scaler, lane)                              \
  do {                                                                                       \
    while (true) {                                                                           \
      const bool done_ = mbar_test_wait(bar_addr(ctx, idx), (parity));                       \
      if (__all_sync(0xffffffffu, done_)) break;                                             \
      const int r_ = (scaler).step(ctx, lane, false);                                        \
      if (r_ < 0) return;                                                                    \
      if (r_ == 0) {                                                                         \
        AF3K_WAIT_WARP_C(ctx, idx, parity);                                                  \
        break;                                                                               \
      }                                                                                      \
    }                                                                                        \
  } while (0)

// Key-mask writer (one warp).  For every logits tile, in the producer's order: write the tile's
// 128 mask values into its slot of the mask-column ring.  The slot is the B operand of the extra
// K step; only element 0 of each key's 16-byte row changes, the rest stays zero.  Arrives on the
// tile's kv_full barrier (which then counts two arrivals: this one and the producer's).  The mask
// bytes of a tile are requested one tile ahead, so their latency is not on the path.
__device__ void mask_writer_role(const Ctx& c, int lane) {
  const AttnParams& p = *c.p;
  const uint32_t nkv = p.kv_stages;
  uint32_t st = 0, round = 0;      // ring slot, how many times the ring wrapped
  for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
    const Item it = decode_item(p, item);
    uint16_t val[4];
    const uint16_t masked = masked_value_bits(p, it.h);
    mask_values(p, it, 0, 0, lane, masked, val);
    for (int kt = 0; kt < p.n_kt; ++kt) {
      for (int s = 0; s < it.gv; ++s) {
        const uint16_t cur[4] = {val[0], val[1], val[2], val[3]};
        {
          const int ns = s + 1 < it.gv ? s + 1 : 0;
          const int nkt = s + 1 < it.gv ? kt : kt + 1;
          if (nkt < p.n_kt) mask_values(p, it, nkt, ns, lane, masked, val);
        }
        if (round > 0) AF3K_WAIT_WARP_C(c, BarIdx::kv_empty + st, (round - 1) & 1);
        const uint32_t slot = c.smem + p.off_mcol + st * kMaskPanelBytes;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(slot + (32 * g + lane) * 16), "h"(cur[g]) : "memory");
        fence_proxy_async_smem();    // make the generic-proxy stores visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::kv_full + st));
        if (++st == nkv) { st = 0; ++round; }
      }
    }
  }
}

// ------------------------------------------------------------------ MMA issuers (two warps)
// The tiles here are small (N = 128, K = 16 and N = D, K = 16), so the cost of issuing an MMA
// matters: one thread issuing both GEMMs of every tile was the limiter of the whole kernel, and
// so was issuing from one lane of a diverged warp (about 150 cycles per tcgen05.mma, because the
// descriptors then travel through per-lane registers).  The two GEMMs are therefore issued by two
// warps, each running its control flow and its waits as a whole warp so that addresses and
// descriptors stay warp-uniform; one elected lane issues.  The two warps touch different TMEM
// columns and every hand-over between them goes through an mbarrier, so no ordering between the
// two instruction streams is assumed.

// Logits of every tile, in order: Q K^T, then the mask column, then (bf16 q/k) the bias slices.
// (The MMA loops are real loops and the fp8 / bf16 choice is a template argument: the warp pays an
// instruction-cache miss for most lines of this loop on every pass, so the loop is kept small.)
template <bool kTcBias, bool kFp8>
__device__ void qk_issuer_role(const Ctx& c) {
  const AttnParams& p = *c.p;
  const bool leader = elect_one();
  const uint32_t nkv = p.kv_stages;
  const uint32_t qk_layout = swizzle_layout_code(p.qk_row_bytes);
  constexpr bool fp8 = kFp8;
  const uint32_t idesc_qk = make_idesc(fp8 ? 0u : 1u, fp8 ? 0u : 1u, 0u, 0u, kTile);
  const uint32_t kv_stage_bytes = p.k_tile_bytes + p.v_tile_bytes;
  // descriptor words for tile 0 / stage 0; later tiles only move the start-address field
  const uint64_t qd0 = make_smem_desc(c.smem + p.off_q, 16, 8 * p.qk_row_bytes, qk_layout);
  const uint64_t kd0 = make_smem_desc(c.smem + p.off_kv, 16, 8 * p.qk_row_bytes, qk_layout);
  const uint32_t qd_lo = (uint32_t)qd0, qd_hi = (uint32_t)(qd0 >> 32);
  const uint32_t kd_lo = (uint32_t)kd0, kd_hi = (uint32_t)(kd0 >> 32);
  const uint32_t q_step = p.q_tile_bytes >> 4, stage_step = kv_stage_bytes >> 4;
  const int ksteps = p.qk_ksteps;
  // extra K step: ones column x mask column, both K-major without swizzle (8-row groups 128 bytes
  // apart, the second 16-byte half of K in the shared zero block)
  const uint64_t od0 = make_smem_desc(c.smem + p.off_ones, p.off_zero - p.off_ones, 128, 0);
  const uint64_t md0 = make_smem_desc(c.smem + p.off_mcol, p.off_zero - p.off_mcol, 128, 0);
  const uint32_t od_lo = (uint32_t)od0, od_hi = (uint32_t)(od0 >> 32);
  const uint32_t md_lo = (uint32_t)md0, md_hi = (uint32_t)(md0 >> 32);
  const uint32_t idesc_mask = make_idesc(1u, 1u, 0u, 0u, kTile);
  const bool mask_col = p.mask_col != 0;
  // bias slices: A = 16 keys of the staged bias tile (K-major, 128-byte swizzled rows, two boxes
  // of 64 keys), B = the 16 x 16 identity (K-major, no swizzle: 8-key halves 256 bytes apart,
  // 8-row groups 128 bytes apart), D = 16 columns of the logits tile
  const uint64_t bd0 = make_smem_desc(c.smem + p.off_bias, 16, 8 * 128, 2);
  const uint64_t id0 = make_smem_desc(c.smem + p.off_ident, 256, 128, 0);
  const uint32_t bd_lo = (uint32_t)bd0, bd_hi = (uint32_t)(bd0 >> 32);
  const uint32_t id_lo = (uint32_t)id0, id_hi = (uint32_t)(id0 >> 32);
  const uint32_t idesc_bias = make_idesc(1u, 1u, 0u, 0u, 16);
  long long* tl = (p.debug != nullptr && blockIdx.x == 0)
                      ? reinterpret_cast<long long*>(p.debug + kDbgFloats) + 2 * kDbgTimelineTiles * 8
                      : nullptr;
  uint32_t tl_n = 0;
  // ring positions / barrier parities are carried incrementally: no division on this warp
  uint32_t st = 0, kv_par = 0, icount = 0, bst = 0, b_par = 0;
  uint32_t sfree_par[2] = {0, 0}, first[2] = {1, 1};
  for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++icount) {
    const Item it = decode_item(p, item);
    const int gv = it.gv;
    for (int kt = 0; kt < p.n_kt; ++kt) {
      for (int s = 0; s < gv; ++s) {
        const int b = s & 1;
        const int qslot = (int)q_buf(p, icount) * kMaxStreams + s;
        const int q_bar = (p.scale_q ? BarIdx::q_scaled : BarIdx::q_full) + qslot;
        const bool need_bias = kTcBias && (s == 0 || p.q_split);
        const bool need_sfree = !first[b];
        {
          // everything the tile needs is normally there already: test all its barriers, vote once
          bool ok = mbar_test_wait(bar_addr(c, BarIdx::kv_full + st), kv_par);
          if (need_sfree) ok = mbar_test_wait(bar_addr(c, BarIdx::s_free + b), sfree_par[b]) && ok;
          if (need_bias) ok = mbar_test_wait(bar_addr(c, BarIdx::bias_full + bst), b_par) && ok;
          if (kt == 0) ok = mbar_test_wait(bar_addr(c, q_bar), q_use(p, icount) & 1) && ok;
          if (!__all_sync(0xffffffffu, ok)) {
            if (need_bias) AF3K_WAIT_WARP_C(c, BarIdx::bias_full + bst, b_par);
            // the softmax warpgroup of this buffer must have read the previous logits tile
            if (need_sfree) AF3K_WAIT_WARP_C(c, BarIdx::s_free + b, sfree_par[b]);
            if (kt == 0) AF3K_WAIT_WARP_C(c, q_bar, q_use(p, icount) & 1);
            AF3K_WAIT_WARP_C(c, BarIdx::kv_full + st, kv_par);
          }
        }
        if (need_sfree) sfree_par[b] ^= 1;
        first[b] = 0;
        tc_fence_after();
        const uint32_t a_lo = qd_lo + (q_buf(p, icount) * p.n_streams + s) * q_step;
        const uint32_t b_lo = kd_lo + st * stage_step;
        const uint32_t s_tmem = c.tmem + kSCol + b * kTile;
        const uint32_t slot16 = st * (kMaskPanelBytes >> 4);
        const uint32_t bias_lo = bd_lo + bst * (kBiasTileBytes >> 4);
        if (leader) {
          const long long t0 = tl != nullptr ? clock64() : 0;
#pragma unroll 1
          for (int k = 0; k < ksteps; ++k) {     // one K step = 32 bytes of a tile row
            if (fp8) mma_ss_f8(s_tmem, a_lo + 2 * k, qd_hi, b_lo + 2 * k, kd_hi, idesc_qk, k > 0 ? 1u : 0u);
            else     mma_ss_f16(s_tmem, a_lo + 2 * k, qd_hi, b_lo + 2 * k, kd_hi, idesc_qk, k > 0 ? 1u : 0u);
          }
          // mask column: start address and leading offset both move with the ring slot (the
          // zero block stays put)
          if (mask_col)
            mma_ss_f16(s_tmem, od_lo, od_hi, md_lo + slot16 - (slot16 << 16), md_hi, idesc_mask, 1u);
          if (kTcBias) {
#pragma unroll 1
            for (int k = 0; k < kTile / 16; ++k)   // keys 16k .. 16k + 15: box k / 4, 32 bytes per step
              mma_ss_f16(s_tmem + 16 * k, bias_lo + (k >> 2) * (kBiasTileBytes >> 5) + 2 * (k & 3), bd_hi,
                         id_lo, id_hi, idesc_bias, 1u);
          }
          tc_commit(bar_addr(c, BarIdx::s_full + b));
          if (kt == p.n_kt - 1) tc_commit(bar_addr(c, BarIdx::q_empty + qslot));
          if (tl != nullptr && tl_n + 2 <= 2 * kDbgTimelineTiles) { tl[tl_n++] = t0; tl[tl_n++] = clock64(); }
        }
        __syncwarp();
        if (++st == nkv) { st = 0; kv_par ^= 1; }
        if (kTcBias && (s == gv - 1 || p.q_split)) {
          // every bias MMA that reads this stage is issued: the stage is free when they finish
          if (leader) tc_commit(bar_addr(c, BarIdx::bias_empty + bst));
          __syncwarp();
          if (++bst == kBiasStages) { bst = 0; b_par ^= 1; }
        }
      }
    }
  }
}

// O += P V for every tile, in order.  This warp mostly waits for the softmax warpgroups, so (bf16
// q/k) it also scales the Q tiles: the first item's up front, the next item's in 1 KB pieces
// while it waits, what is left when the item's last P V has been issued.
template <bool kTcBias>
__device__ void pv_issuer_role(const Ctx& c, int lane) {
  const AttnParams& p = *c.p;
  const bool leader = elect_one();
  QScaler scaler;
  if (kTcBias && p.scale_q && (int)blockIdx.x < p.n_items) {
    scaler.start(0, decode_item(p, blockIdx.x).gv);
    while (scaler.pending())
      if (scaler.step(c, lane, true) < 0) return;
  }
  const uint32_t nkv = p.kv_stages;
  const uint32_t v_layout = swizzle_layout_code(p.v_row_bytes);
  const uint32_t idesc_pv = make_idesc(1u, 1u, 0u, 1u, (uint32_t)p.nv);   // A = P and B = V, both bf16 (kind::f16 takes no mixed pair)
  const uint32_t kv_stage_bytes = p.k_tile_bytes + p.v_tile_bytes;
  const uint64_t vd0 = make_smem_desc(c.smem + p.off_kv + p.k_tile_bytes, p.v_tile_bytes,
                                      8 * p.v_row_bytes, v_layout);
  const uint32_t vd_lo = (uint32_t)vd0, vd_hi = (uint32_t)(vd0 >> 32);
  const uint32_t stage_step = kv_stage_bytes >> 4;
  const uint32_t v_kstep = (16u * p.v_row_bytes) >> 4;
  long long* tl = (p.debug != nullptr && blockIdx.x == 0)
                      ? reinterpret_cast<long long*>(p.debug + kDbgFloats) + 2 * kDbgTimelineTiles * 8 +
                            2 * kDbgTimelineTiles
                      : nullptr;
  uint32_t tl_n = 0;
  uint32_t st = 0, icount = 0;
  uint32_t pready_par[2] = {0, 0};
  for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++icount) {
    const Item it = decode_item(p, item);
    const int gv = it.gv;
    scaler.start(icount + 1, (kTcBias && p.scale_q && item + (int)gridDim.x < p.n_items) ? decode_item(p, item + gridDim.x).gv : 0);
    for (int kt = 0; kt < p.n_kt; ++kt) {
      for (int s = 0; s < gv; ++s) {
        const int b = s & 1;
        if (b) { AF3K_WAIT_WARP_OR_SCALE(c, BarIdx::p_ready + 1, pready_par[1], scaler, lane); pready_par[1] ^= 1; }
        else   { AF3K_WAIT_WARP_OR_SCALE(c, BarIdx::p_ready + 0, pready_par[0], scaler, lane); pready_par[0] ^= 1; }
        // the warpgroup's epilogue of the previous item must have read its O accumulators before
        // its first P V of this item overwrites one
        if (kt == 0 && s < 2 && icount > 0) AF3K_WAIT_WARP_C(c, BarIdx::epi_done + b, (icount - 1) & 1);
        tc_fence_after();
        const uint32_t b_lo = vd_lo + st * stage_step;
        const uint32_t o_tmem = c.tmem + kOCol + s * p.nv;
        const uint32_t p_tmem = c.tmem + kPCol + b * 64;
        if (leader) {
          const long long t0 = tl != nullptr ? clock64() : 0;
          mma_ts_f16(o_tmem, p_tmem, b_lo, vd_hi, idesc_pv, kt > 0 ? 1u : 0u);
#pragma unroll 1
          for (int k = 1; k < kTile / 16; ++k)   // 16 keys per step: 8 TMEM columns of P
            mma_ts_f16(o_tmem, p_tmem + k * 8, b_lo + k * v_kstep, vd_hi, idesc_pv, 1u);
          // one completion signal: the K/V stage is free, and so are this tile's P buffer and O
          tc_commit(bar_addr(c, BarIdx::kv_empty + st));
          if (tl != nullptr && tl_n + 2 <= 2 * kDbgTimelineTiles) { tl[tl_n++] = t0; tl[tl_n++] = clock64(); }
        }
        __syncwarp();
        if (++st == nkv) st = 0;
      }
    }
    while (scaler.pending())
      if (scaler.step(c, lane, true) < 0) return;
  }
}

// ------------------------------------------------------------------ softmax
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}



// x = s * scale + bias for the 64 columns [kCol0, kCol0 + 64) of the thread's row, row maximum
// updated.  xr holds the raw logits on entry and x on exit.  Masked and absent keys arrive from
// the tensor core as -2^47 and -inf and need no handling here.
template <int kCol0>
__device__ __forceinline__ void logits_half(uint32_t (&xr)[kTile], uint32_t bias_row, uint32_t row7,
                                            uint64_t scale2, float& mxa, float& mxb) {
#pragma unroll
  for (int j = kCol0 / 8; j < kCol0 / 8 + 8; ++j) {
    const uint4 bv = lds128(bias_row + (j >> 3) * (kBiasTileBytes / 2) + (((j & 7) ^ row7) << 4));
    const uint32_t w[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = j * 8 + 2 * e;
      // bf16 pair -> two fp32: low half shifted up, high half masked in place
      const uint64_t b2 = pack_f32x2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
      const uint64_t s2 = pack_f32x2(__uint_as_float(xr[col]), __uint_as_float(xr[col + 1]));
      float x0, x1;
      unpack_f32x2(fma_f32x2(s2, scale2, b2), x0, x1);
      xr[col] = __float_as_uint(x0);
      xr[col + 1] = __float_as_uint(x1);
      if (e & 1) mxb = max3(mxb, x0, x1); else mxa = max3(mxa, x0, x1);
    }
  }
}

// Row maximum over 64 finished logits (bf16 q/k: the tensor core has already applied scale, bias
// and mask).
template <int kCol0>
__device__ __forceinline__ void max_half(const uint32_t (&xr)[kTile], float& mxa, float& mxb) {
#pragma unroll
  for (int i = kCol0; i < kCol0 + 64; i += 4) {
    mxa = max3(mxa, __uint_as_float(xr[i]), __uint_as_float(xr[i + 1]));
    mxb = max3(mxb, __uint_as_float(xr[i + 2]), __uint_as_float(xr[i + 3]));
  }
}

// One 128 x 128 logits tile of one stream; the thread owns row `row` (TMEM lane).
// m_run is the reference maximum the running sums are scaled by (it may lag the true maximum by
// up to kLazyRescaleLog2 bits), l_run the running sum of the fp32 weights.
template <bool kTcBias>
__device__ __forceinline__ bool softmax_tile(const Ctx& c, float* dbg, int wg, int lane,
                                             uint32_t s_taddr, uint32_t p_taddr, uint32_t o_taddr,
                                             int nv, uint32_t bias_row, uint32_t row7, float scale,
                                             bool first_kt, bool wait_prev_pv, int prev_pv_bar,
                                             uint32_t prev_pv_parity, float& m_run, float& l_run,
                                             int next_s_bar, uint32_t next_s_parity, bool& next_ready,
                                             long long* ts = nullptr) {
  uint32_t xr[kTile];
  float mt;
  {
    tmem_ld_x32(s_taddr + 0, &xr[0]);
    tmem_ld_x32(s_taddr + 32, &xr[32]);
    tc_wait_ld();
    tmem_ld_x32(s_taddr + 64, &xr[64]);
    tmem_ld_x32(s_taddr + 96, &xr[96]);
    if (dbg != nullptr) {
#pragma unroll
      for (int i = 0; i < 64; ++i) dbg[kDbgS + i] = __uint_as_float(xr[i]);
    }
    const uint64_t scale2 = pack_f32x2(scale, scale);
    float mxa = -INFINITY, mxb = -INFINITY;
    if (kTcBias) max_half<0>(xr, mxa, mxb);
    else         logits_half<0>(xr, bias_row, row7, scale2, mxa, mxb);
    tc_wait_ld();
    // the logits are in registers: hand the S buffer back so that the next Q K^T can start
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::s_free + wg));
    if (dbg != nullptr) {
#pragma unroll
      for (int i = 64; i < kTile; ++i) dbg[kDbgS + i] = __uint_as_float(xr[i]);
    }
    if (kTcBias) max_half<64>(xr, mxa, mxb);
    else         logits_half<64>(xr, bias_row, row7, scale2, mxa, mxb);
    mt = fmaxf(mxa, mxb);
  }
  if (ts != nullptr) ts[2] = clock64() + (long long)(mt == 123.456f);   // logits and row maximum in registers
  // factor between a logit difference and the exponent of 2: log2(e), times the logit scale when
  // the tensor core's logits still lack it (fp8 q/k with tensor-core bias: `scale` carries it)
  const float ef = kTcBias ? scale : kLog2e;
  float m_use = m_run;
  float alpha = 1.0f;
  bool need = false;
  if (first_kt) {
    m_use = mt;
  } else {
    need = (mt - m_run) * ef > kLazyRescaleLog2;
    if (need) {
      m_use = mt;
      alpha = ex2_approx((m_run - mt) * ef);
    }
  }
  if (ts != nullptr) ts[3] = clock64();   // exponential pass starts
  // p = exp2((x - m) * log2e).  fp8 path: the subtraction comes first so that x == m gives
  // exactly 0 even for the huge negative values of masked keys (a row with no attended key: all
  // weights 1).  bf16 path: one fused multiply-add, x * log2e - m * log2e; for such a row x and
  // m are the same power of two, both products are exact and the result is 0 as well.
  // The pass is one ex2 per logit on the XU (a warp-wide ex2 every 8 cycles per scheduler, shared
  // by the scheduler's two softmax warps) with one packed FMA, one packed add and one bf16 pack per
  // pair of logits around it.  The two warpgroups run their passes in step (2 000 - 2 500 cycles per
  // pass against 2 048 for the XU alone); what keeps the kernel above that is the time between
  // passes, when both read logits, search the maximum and hand P over and the XU idles.
  const uint64_t l2e2 = pack_f32x2(ef, ef);
  const uint64_t nm2 = pack_f32x2(-m_use, -m_use);
  const float nml = -m_use * ef;
  const uint64_t nml2 = pack_f32x2(nml, nml);
  uint64_t suma = pack_f32x2(0.f, 0.f), sumb = suma;
  // The first kHeld column groups are computed before anything is written: the P buffer and the
  // O accumulator only become free when the previous P V of this warpgroup has finished, and that
  // wait is taken as late as the registers allow.
  constexpr int kHeld = 3;
  uint32_t pk[8][8];
#pragma unroll
  for (int cidx = 0; cidx < 8; ++cidx) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = cidx * 16 + 2 * i;
      float y0, y1;
      const uint64_t x2 = pack_f32x2(__uint_as_float(xr[col]), __uint_as_float(xr[col + 1]));
      if (kTcBias) unpack_f32x2(fma_f32x2(x2, l2e2, nml2), y0, y1);
      else         unpack_f32x2(mul_f32x2(add_f32x2(x2, nm2), l2e2), y0, y1);
      const float p0 = ex2_approx(y0);
      const float p1 = ex2_approx(y1);
      if (i & 1) sumb = add_f32x2(sumb, pack_f32x2(p0, p1));
      else       suma = add_f32x2(suma, pack_f32x2(p0, p1));
      pk[cidx][i] = pack_bf16x2(p0, p1);
    }
    if (dbg != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) dbg[kDbgP + cidx * 8 + i] = __uint_as_float(pk[cidx][i]);
    }
    if (cidx == kHeld - 1) {
      // the completion that frees P and O is the one that also frees the previous tile's K/V stage
      if (wait_prev_pv) {
        const bool ok = mbar_wait_bounded(bar_addr(c, prev_pv_bar), prev_pv_parity, c.p->wait_limit,
                                          c.abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          report_timeout(c, prev_pv_bar);
          return false;
        }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, need)) {
        for (int c0 = 0; c0 < nv; c0 += 16) {
          uint32_t o[16];
          tmem_ld_x16(o_taddr + c0, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x16(o_taddr + c0, o);
        }
      }
      if (ts != nullptr) ts[5] = clock64();   // previous P V awaited
    }
    if (cidx >= kHeld - 1) {
      // P as bf16, two keys per 32-bit TMEM column: the A operand of the second GEMM
#pragma unroll
      for (int cc = (cidx == kHeld - 1 ? 0 : cidx); cc <= cidx; ++cc)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
                     ::"r"(pk[cc][0]), "r"(pk[cc][1]), "r"(pk[cc][2]), "r"(pk[cc][3]), "r"(pk[cc][4]),
                     "r"(pk[cc][5]), "r"(pk[cc][6]), "r"(pk[cc][7]), "r"(p_taddr + cc * 8)
                     : "memory");
    }
  }
  if (ts != nullptr) ts[6] = clock64();     // last exponential issued
  // The next tile's logits are normally finished by now: ask while the P stores drain, so that the
  // barrier's round trip (about two hundred cycles even when the phase is complete) is not paid
  // between two tiles.
  next_ready = __all_sync(0xffffffffu, mbar_test_wait(bar_addr(c, next_s_bar), next_s_parity));
  tc_wait_st();
  if (ts != nullptr) ts[4] = clock64();   // P stored
  float s0, s1, s2, s3;
  unpack_f32x2(suma, s0, s1);
  unpack_f32x2(sumb, s2, s3);
  m_run = m_use;
  l_run = l_run * alpha + ((s0 + s1) + (s2 + s3));
  return true;
}

template <bool kDebug, bool kTcBias>
__device__ void softmax_role(const Ctx& c, int wg, int wq, int lane) {
  const AttnParams& p = *c.p;
  const int row = wq * 32 + lane;                    // row of the 128-query tile == TMEM lane
  const uint32_t lane_sel = (uint32_t)(wq * 32) << 16;
  const uint32_t s_taddr = c.tmem + lane_sel + kSCol + wg * kTile;
  const uint32_t p_taddr = c.tmem + lane_sel + kPCol + wg * 64;
  // running statistics of the warpgroup's (at most two) streams, kept in registers
  float m_st[2] = {-INFINITY, -INFINITY}, l_st[2] = {0.f, 0.f};
  uint32_t ucnt = 0, bcount = 0, icount = 0;         // tiles done by this warpgroup, bias tiles, items
  bool s_ready = false;                              // the next tile's s_full phase was seen complete already
  // position of tiles in the CTA-wide order (all streams): gives the K/V stage a tile used
  uint32_t kt_stage = 0, kt_round = 0;                // ring stage / lap of stream 0's tile at the current key tile
  uint32_t prev_stage = 0, prev_round = 0;            // the same for this warpgroup's last tile
  const uint32_t nkv = p.kv_stages;

  for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++icount) {
    const Item it = decode_item(p, item);
    // fp32 path: the logit scale the softmax threads apply themselves.  Tensor-core path: the
    // factor from logit differences to exponents of 2 (the scale is in Q already for bf16 q/k)
    float scale = p.scale;
    if (p.q_scale != nullptr) scale *= p.q_scale[it.h] * p.k_scale[it.h];
    if (kTcBias) scale = (p.scale_q ? 1.0f : scale) * kLog2e;

    long long* last_ts = nullptr;     // debug build: timeline slot of the warpgroup's last tile
    for (int kt = 0; kt < p.n_kt; ++kt) {
      // fp8 q/k: this thread adds the bias itself, from its row of the staged tile
      const uint32_t bst = bcount % kBiasStages;
      if (!kTcBias) AF3K_WAIT_WARP(c, BarIdx::bias_full + bst, (bcount / kBiasStages) & 1);
      const uint32_t bias_row = c.smem + p.off_bias + bst * kBiasTileBytes + row * 128;

      for (int s = wg; s < it.gv; s += 2) {
        float m_run = -INFINITY, l_run = 0.f;
        const int si = (s - wg) >> 1;
        if (kt > 0) { m_run = si ? m_st[1] : m_st[0]; l_run = si ? l_st[1] : l_st[0]; }

        // diagnostic timeline (debug build only): SM clock at the phase boundaries of every tile
        // this warp processes, 8 slots per tile, behind the tile dump
        long long* ts = nullptr;
        if (kDebug && p.debug != nullptr && blockIdx.x == 0 && wq == 0 && lane == 0 && ucnt < kDbgTimelineTiles)
          ts = reinterpret_cast<long long*>(p.debug + kDbgFloats) + ((size_t)wg * kDbgTimelineTiles + ucnt) * 8;
        if (ts != nullptr) ts[0] = clock64();
        if (kDebug) last_ts = ts;
        if (!s_ready) AF3K_WAIT_WARP(c, BarIdx::s_full + wg, ucnt & 1);
        tc_fence_after();
        if (ts != nullptr) ts[1] = clock64();
        const uint32_t o_taddr = c.tmem + lane_sel + kOCol + s * p.nv;
        float* dbg = nullptr;
        if (kDebug && p.debug != nullptr && blockIdx.x == 0 && icount == 0 && s == 0 && kt == 0)
          dbg = p.debug + (size_t)row * kTile;
        if (!softmax_tile<kTcBias>(c, dbg, wg, lane, s_taddr, p_taddr, o_taddr, p.nv, bias_row, row & 7, scale,
                                   kt == 0, ucnt > 0, BarIdx::kv_empty + (int)prev_stage, prev_round & 1, m_run,
                                   l_run, BarIdx::s_full + wg, (ucnt + 1) & 1, s_ready, ts))
          return;
        ++ucnt;
        {
          // tiles are numbered in the producer's order; the numbers are carried without a division
          prev_stage = kt_stage + (uint32_t)s;
          prev_round = kt_round;
          while (prev_stage >= nkv) { prev_stage -= nkv; ++prev_round; }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::p_ready + wg));
        if (si) { m_st[1] = m_run; l_st[1] = l_run; } else { m_st[0] = m_run; l_st[0] = l_run; }
      }
      if (!kTcBias) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::bias_empty + bst));
      }
      ++bcount;
      kt_stage += (uint32_t)it.gv;
      while (kt_stage >= nkv) { kt_stage -= nkv; ++kt_round; }
    }


    // ---- epilogue: O / l -> bf16 -> global, once this warpgroup's last P V has finished (the
    // other warpgroup may still be working on its own streams)
    if (kDebug && last_ts != nullptr) last_ts[5] = clock64();
    // only a warpgroup that had a stream in this item has a P V of this item to wait for (with an
    // odd row count the last item leaves warpgroup 1 without one: its record of a previous tile
    // may be a whole number of ring laps old, and the parity test would then wait for ever)
    if (wg < it.gv) AF3K_WAIT_WARP(c, BarIdx::kv_empty + (int)prev_stage, prev_round & 1);
    tc_fence_after();
    if (kDebug && last_ts != nullptr) last_ts[6] = clock64();
    for (int s = wg; s < it.gv; s += 2) {
      const int qrow = stream_qt(p, it, s) * kTile + row;
      const float inv = __frcp_rn(s == wg ? l_st[0] : l_st[1]);
      const uint32_t o_taddr = c.tmem + lane_sel + kOCol + s * p.nv;
      __nv_bfloat16* orow = p.out + (long long)stream_row(p, it, s) * p.out_stride_b1 +
                            (long long)it.h * p.out_stride_b2 + (long long)qrow * p.out_stride_s;
      for (int c0 = 0; c0 < p.nv; c0 += 16) {
        uint32_t o[16];
        tmem_ld_x16(o_taddr + c0, o);
        tc_wait_ld();
        if (kDebug && p.debug != nullptr && blockIdx.x == 0 && icount == 0 && s == 0) {
          float* dbg = p.debug + (size_t)row * kTile;
#pragma unroll
          for (int i = 0; i < 16; ++i) dbg[kDbgO + c0 + i] = __uint_as_float(o[i]);
          dbg[kDbgML + 0] = m_st[0];
          dbg[kDbgML + 1] = l_st[0];
        }
        if (qrow < p.Sq) {
#pragma unroll
          for (int hseg = 0; hseg < 2; ++hseg) {
            if (c0 + hseg * 8 + 8 <= p.D) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[hseg * 8 + 0]) * inv, __uint_as_float(o[hseg * 8 + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[hseg * 8 + 2]) * inv, __uint_as_float(o[hseg * 8 + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[hseg * 8 + 4]) * inv, __uint_as_float(o[hseg * 8 + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[hseg * 8 + 6]) * inv, __uint_as_float(o[hseg * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c0 + hseg * 8) = v;
            }
          }
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_addr(c, BarIdx::epi_done + wg));
    if (kDebug && last_ts != nullptr) last_ts[7] = clock64();
  }
}

// ------------------------------------------------------------------ kernel
template <bool kDebug, bool kTcBias>
__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_bias) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  Ctx c;
  c.p = &p;
  c.smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  c.bars = c.smem + p.off_bar;
  c.abort_flag = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_bias);
    for (int i = 0; i < 2 * kMaxStreams; ++i) {
      mbar_init(bar_addr(c, BarIdx::q_full + i), 1);
      mbar_init(bar_addr(c, BarIdx::q_empty + i), 1);
      mbar_init(bar_addr(c, BarIdx::q_scaled + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_addr(c, BarIdx::epi_done + i), 4);
      mbar_init(bar_addr(c, BarIdx::s_full + i), 1);
      mbar_init(bar_addr(c, BarIdx::s_free + i), 4);
      mbar_init(bar_addr(c, BarIdx::p_ready + i), 4);
    }
    for (int i = 0; i < kBiasStages; ++i) {
      mbar_init(bar_addr(c, BarIdx::bias_full + i), 1);
      // freed by the bias MMAs' completion (bf16 q/k) or by the eight softmax warps (fp8 q/k)
      mbar_init(bar_addr(c, BarIdx::bias_empty + i), kTcBias ? 1 : 8);
    }
    for (int i = 0; i < kMaxKvStages; ++i) {
      mbar_init(bar_addr(c, BarIdx::kv_full + i), p.mask_col ? 2 : 1);
      mbar_init(bar_addr(c, BarIdx::kv_empty + i), 1);
    }
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 3) {
    // ones column, mask-column ring, zero block and identity are contiguous: clear them, then set
    // element (row, 0) of the ones operand and the identity's diagonal to bf16 1.0
    const uint32_t base = c.smem + p.off_ones;
    const uint32_t bytes = p.off_ident + kIdentBytes - p.off_ones;
    for (uint32_t o = lane * 16; o < bytes; o += 32 * 16)
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(base + o), "r"(0u) : "memory");
    __syncwarp();
    for (int r = lane; r < kTile; r += 32)
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(base + r * 16), "h"((uint16_t)0x3F80) : "memory");
    // identity element (i, i): 8-row group i / 8 (128 bytes apart), 8-key half i / 8 (256 bytes
    // apart), row i % 8 (16 bytes), key i % 8 (2 bytes)
    if (lane < 16)
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(c.smem + p.off_ident + (lane >> 3) * 384 + (lane & 7) * 18),
                   "h"((uint16_t)0x3F80) : "memory");
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = tmem_base_slot;

  if (warp < 4) {
    // warps 0-3 need few registers; the two softmax warpgroups take what they give up
    setmaxnreg_dec<kRegsMisc>();
    if (warp == 0) {
      if (lane == 0) producer_role(c, &tm_q, &tm_k, &tm_v, &tm_bias);
    } else if (warp == 1) {
      if (p.qk_is_fp8) qk_issuer_role<kTcBias, true>(c);
      else             qk_issuer_role<kTcBias, false>(c);
    } else if (warp == 2) {
      pv_issuer_role<kTcBias>(c, lane);
    } else if (warp == 3) {
      if (p.mask_col) mask_writer_role(c, lane);
    }
  } else {
    setmaxnreg_inc<kRegsSoftmax>();
    softmax_role<kDebug, kTcBias>(c, (warp - 4) >> 2, warp & 3, lane);
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // a wait ran out: give loads and MMAs still in flight time to land before smem / TMEM go away
    for (int i = 0; i < 200; ++i) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(c.tmem, kTmemCols);
  }
}

// ------------------------------------------------------------------ bias staging pre-pass
// bias (fp32 or bf16, arbitrary row pitch) -> bf16 [B2, Sq, pitch] with a TMA-legal pitch.
// With fp8 q/k (q_scale / k_scale given) every value is divided by the head's logit scale
// softmax_scale * q_scale[h] * k_scale[h]: the tensor core then adds it to the raw fp8 products
// and the softmax threads apply that scale to the sum.
template <typename T>
__global__ void bias_to_bf16_kernel(const T* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                    int B2, int Sq, int Sk, long long src_stride_h,
                                    long long src_stride_r, int pitch, const float* __restrict__ q_scale,
                                    const float* __restrict__ k_scale, float softmax_scale) {
  const long long total = (long long)B2 * Sq * (pitch / 2);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cp = (int)(i % (pitch / 2));
    const long long t = i / (pitch / 2);
    const int r = (int)(t % Sq);
    const int h = (int)(t / Sq);
    const T* s = src + h * src_stride_h + r * src_stride_r;
    const float mul = q_scale != nullptr ? 1.0f / (softmax_scale * q_scale[h] * k_scale[h]) : 1.0f;
    const int col = cp * 2;
    const float a = col < Sk ? (float)s[col] * mul : 0.f;
    const float b = col + 1 < Sk ? (float)s[col + 1] * mul : 0.f;
    reinterpret_cast<uint32_t*>(dst)[i] = pack_bf16x2(a, b);
  }
}

}  // namespace af3k
