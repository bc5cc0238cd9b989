// C ABI of libaf3k.so (declared in include/af3k.h): argument validation, launch planning,
// TMA descriptor encoding and kernel launches.  No torch types cross this boundary.
#include "../../include/af3k.h"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include "attn_sm100.cuh"
#include "pair_bias_sm100.cuh"
#include "proj_sm100.cuh"

namespace {

using namespace af3k;

std::atomic<long long> g_wait_limit{-1};
thread_local int t_last_launches = 0;
std::atomic<float*> g_debug_dump{nullptr};
thread_local char t_detail[256] = "";

// Records which CUDA call failed (text returned by af3k_last_error_detail) and clears the
// runtime's sticky-until-read error so that it does not surface in the caller's next CUDA call.
int cuda_fail(const char* what, cudaError_t e) {
  std::snprintf(t_detail, sizeof(t_detail), "%s: %s", what, cudaGetErrorString(e));
  (void)cudaGetLastError();
  return AF3K_ERR_CUDA;
}
int driver_fail(const char* what, int r) {
  std::snprintf(t_detail, sizeof(t_detail), "%s: CUresult %d", what, r);
  return AF3K_ERR_CUDA;
}

long long wait_limit_cycles() {
  long long v = g_wait_limit.load();
  if (v > 0) return v;
  const char* e = std::getenv("AF3K_WAIT_LIMIT_CYCLES");
  v = e ? std::atoll(e) : 0;
  if (v <= 0) v = 2000000000LL;
  g_wait_limit.store(v);
  return v;
}

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

constexpr int kStaticSmemReserve = 256;

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  int max_smem_optin = 0;
  bool attr_set = false;
};

int device_info(DeviceInfo** out) {
  static DeviceInfo infos[64];
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return cuda_fail("cudaGetDevice", e);
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = infos[dev];
  if (d.sm_count == 0) {
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess)
      return cuda_fail("cudaGetDeviceProperties", e);
    d.sm_count = prop.multiProcessorCount;
    d.cc_major = prop.major;
    d.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  }
  if (d.cc_major != 10) return AF3K_ERR_UNSUPPORTED_DEVICE;
  if (!d.attr_set) {
    // the opt-in limit covers static + dynamic shared memory; the kernel has a few static bytes
    const int dyn = d.max_smem_optin - kStaticSmemReserve;
    const cudaFuncAttribute attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    const void* kernels[] = {
        (const void*)attention_kernel<false, false>, (const void*)attention_kernel<true, false>,
        (const void*)attention_kernel<false, true>,  (const void*)attention_kernel<true, true>,
    };
    e = cudaSuccess;
    for (const void* kfn : kernels)
      if (e == cudaSuccess) e = cudaFuncSetAttribute(kfn, attr, dyn);
    if (e != cudaSuccess)
      return cuda_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize)", e);
    if ((e = cudaFuncSetAttribute(pair_bias_kernel_t<float>, attr, PbTile<float>::kSmemBytes)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(pair_bias_kernel_t<__nv_bfloat16>, attr, PbTile<__nv_bfloat16>::kSmemBytes)) !=
            cudaSuccess)
      return cuda_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize, pair_bias)", e);
    if ((e = cudaFuncSetAttribute(pair_bias_mma_kernel, attr, kPbmSmemBytes)) != cudaSuccess)
      return cuda_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize, pair_bias_mma)", e);
    if ((e = cudaFuncSetAttribute(qkvg_projection_kernel<false>, attr, (int)kProjSmemBytes)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(qkvg_projection_kernel<true>, attr, (int)kProjSmemBytes)) != cudaSuccess)
      return cuda_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize, qkvg_projection)", e);
    d.attr_set = true;
  }
  *out = &d;
  return AF3K_OK;
}

int row_bytes_for(int64_t bytes) { return bytes <= 32 ? 32 : (bytes <= 64 ? 64 : 128); }
CUtensorMapSwizzle swizzle_for(int row_bytes) {
  return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Does the bias need the bf16 staging copy?
bool bias_needs_staging(const af3k_attention_desc& d, const void* bias) {
  if (d.bias_dtype != AF3K_BF16) return true;
  if ((d.bias_stride[0] * 2) % 16 != 0 || (d.bias_stride[1] * 2) % 16 != 0) return true;
  if (bias != nullptr && !aligned16(bias)) return true;
  return false;
}
int64_t staged_bias_pitch(int64_t Sk) { return (Sk + 7) / 8 * 8; }

int validate(const af3k_attention_desc& d) {
  if (d.qk_dtype != AF3K_BF16 && d.qk_dtype != AF3K_FP8_E4M3) return AF3K_ERR_BAD_DTYPE;
  if (d.bias_dtype != AF3K_BF16 && d.bias_dtype != AF3K_F32) return AF3K_ERR_BAD_DTYPE;
  if (d.B1 < 0 || d.B2 < 0 || d.Sq < 0 || d.Sk <= 0 || d.D <= 0) return AF3K_ERR_BAD_SHAPE;
  if (d.D % 8 != 0 || d.D > 64) return AF3K_ERR_BAD_SHAPE;
  if (d.qk_dtype == AF3K_FP8_E4M3 && d.D % 16 != 0) return AF3K_ERR_BAD_SHAPE;
  if (d.B1 > 0x7fffffff || d.B2 > 0x7fffffff || d.Sq > 0x7fffff00 || d.Sk > 0x7fffff00)
    return AF3K_ERR_BAD_SHAPE;
  if (d.rows_per_item < 0 || d.rows_per_item > 8) return AF3K_ERR_BAD_SHAPE;   // a request, clamped by the plan
  if (d.bias_prescaled != 0 && (d.bias_prescaled != 1 || d.qk_dtype != AF3K_FP8_E4M3 || d.bias_dtype != AF3K_BF16))
    return AF3K_ERR_BAD_DTYPE;
  if (d.max_ctas < 0) return AF3K_ERR_BAD_SHAPE;
  const int64_t es = d.qk_dtype == AF3K_FP8_E4M3 ? 1 : 2;
  for (int i = 0; i < 3; ++i) {
    if (d.q_stride[i] < 0 || d.k_stride[i] < 0 || d.v_stride[i] < 0 || d.out_stride[i] < 0)
      return AF3K_ERR_BAD_STRIDE;
    if ((d.q_stride[i] * es) % 16 || (d.k_stride[i] * es) % 16 || (d.v_stride[i] * 2) % 16 ||
        (d.out_stride[i] * 2) % 16)
      return AF3K_ERR_BAD_STRIDE;
  }
  if (d.q_stride[2] < d.D || d.k_stride[2] < d.D || d.v_stride[2] < d.D || d.out_stride[2] < d.D)
    return AF3K_ERR_BAD_STRIDE;
  if (d.bias_stride[0] < 0 || d.bias_stride[1] < d.Sk || d.mask_row_stride < 0)
    return AF3K_ERR_BAD_STRIDE;
  // A zero stride (a broadcast view) is only meaningful on a dimension of extent 1: TMA cannot
  // express it, and a zero output stride would make rows overwrite each other.
  const int64_t ext_q[3] = {d.B1, d.B2, d.Sq}, ext_k[3] = {d.B1, d.B2, d.Sk};
  for (int i = 0; i < 3; ++i) {
    if (ext_q[i] > 1 && (d.q_stride[i] == 0 || d.out_stride[i] == 0)) return AF3K_ERR_BAD_STRIDE;
    if (ext_k[i] > 1 && (d.k_stride[i] == 0 || d.v_stride[i] == 0)) return AF3K_ERR_BAD_STRIDE;
  }
  if (d.B2 > 1 && d.bias_stride[0] == 0) return AF3K_ERR_BAD_STRIDE;
  return AF3K_OK;
}

struct Plan {
  AttnParams p;
  size_t smem_bytes;
  int grid;
};

// Picks rows-per-item G and the K/V ring depth from a cost model of one CTA's time (below).
// allow_q_split: the kernel variant that will run supports query-tile streams (every variant in
// which the tensor core adds the bias).
int make_plan(const af3k_attention_desc& d, const DeviceInfo& dev, Plan* plan, bool allow_q_split = true) {
  AttnParams& p = plan->p;
  std::memset(&p, 0, sizeof(p));
  const int es = d.qk_dtype == AF3K_FP8_E4M3 ? 1 : 2;
  p.B1 = (int)d.B1; p.B2 = (int)d.B2; p.Sq = (int)d.Sq; p.Sk = (int)d.Sk; p.D = (int)d.D;
  p.n_qt = (p.Sq + kTile - 1) / kTile;
  p.n_kt = (p.Sk + kTile - 1) / kTile;
  p.qk_is_fp8 = es == 1;
  p.qk_row_bytes = row_bytes_for(d.D * es);
  p.v_row_bytes = row_bytes_for(d.D * 2);
  p.qk_ksteps = (int)((d.D * es + 31) / 32);
  p.nv = (int)((d.D + 15) / 16 * 16);
  p.q_tile_bytes = kTile * p.qk_row_bytes;
  p.k_tile_bytes = kTile * p.qk_row_bytes;
  p.v_tile_bytes = kTile * p.v_row_bytes;
  p.scale = d.softmax_scale;

  const int budget = dev.max_smem_optin - 1024 /*alignment slack*/ - kStaticSmemReserve;
  p.mask_col = 1;   // set for real in the launch path once the mask pointer is known
  const int fixed = kBiasStages * kBiasTileBytes + (int)kBarrierBlockBytes +
                    (kMaxKvStages + 2) * (int)kMaskPanelBytes /*ones column, mask ring, zero block*/ +
                    (int)kIdentBytes;
  const int kv_stage = (int)(p.k_tile_bytes + p.v_tile_bytes);
  const int g_tmem = (int)((kTmemCols - kOCol) / p.nv);
  int g_max = kMaxStreams < g_tmem ? kMaxStreams : g_tmem;
  if (g_max > p.B1) g_max = p.B1 > 0 ? p.B1 : 1;

  int best_g = 0, best_stages = 0, best_qbuf = 0;
  double best_cost = 0;
  // rows_per_item is a request: it is honoured up to what TMEM and the batch allow
  const int g_req = d.rows_per_item > g_max ? g_max : d.rows_per_item;
  for (int g = 1; g <= g_max; ++g) {
    if (g_req != 0 && g != g_req) continue;
    for (int qbuf = 2; qbuf >= 1; --qbuf) {
      // one pair row per item: the two softmax warpgroups take two neighbouring query tiles
      const bool split = g == 1 && allow_q_split && p.n_qt >= 2;
      const int streams = split ? 2 : g;
      int stages = (budget - fixed - qbuf * streams * (int)p.q_tile_bytes) / kv_stage;
      if (stages > kMaxKvStages) stages = kMaxKvStages;
      if (stages < 2) continue;
      const long long groups = (p.B1 + g - 1) / g;
      const long long items = groups * p.B2 * (split ? (p.n_qt + 1) / 2 : p.n_qt);
      const int ctas_avail = (d.max_ctas > 0 && d.max_ctas < dev.sm_count) ? d.max_ctas : dev.sm_count;
      const long long rounds = (items + ctas_avail - 1) / ctas_avail;
      // streams alternate between the two softmax warpgroups: an odd count leaves one idle slot.
      // A CTA's time, in logits-tile times of one warpgroup: per item n_kt tiles for each of its
      // slots / 2 streams plus about 0.8 for the epilogue and the hand-over to the next item; with
      // a single Q buffer the next item's Q tiles are loaded and scaled at the hand-over (about 0.5:
      // each stream's tile is replaced as soon as its last Q K^T has finished).
      const int slots = split ? 2 : ((g & 1) ? g + 1 : g);
      double cost = (double)rounds * (p.n_kt * (slots / 2) + 0.8 + (qbuf == 1 ? 0.5 : 0.0));
      // a K/V tile takes about two thousand cycles to arrive, most of a logits tile's time: with a
      // short ring the MMAs wait for their operands (measured: 4 stages cost about 3 %)
      static const double kRingPenalty[7] = {0, 0, 1.4, 1.15, 1.03, 1.0, 1.0};
      cost *= kRingPenalty[stages];
      if (split) cost *= 1.02;   // query-tile streams share no bias tile: pair rows win a tie
      if (best_g == 0 || cost < best_cost) { best_g = g; best_cost = cost; best_stages = stages; best_qbuf = qbuf; }
    }
  }
  if (best_g == 0) return AF3K_ERR_BAD_SHAPE;
  p.G = best_g;
  p.q_split = (best_g == 1 && allow_q_split && p.n_qt >= 2) ? 1 : 0;
  p.n_streams = p.q_split ? 2 : p.G;
  p.kv_stages = best_stages;
  p.q_buffers = best_qbuf;
  const long long groups = (p.B1 + p.G - 1) / p.G;
  const long long items = groups * p.B2 * (p.q_split ? (p.n_qt + 1) / 2 : p.n_qt);
  if (items > 0x7fffffff) return AF3K_ERR_BAD_SHAPE;
  p.n_items = (int)items;

  uint32_t off = 0;
  p.off_q = off;      off += p.q_buffers * p.n_streams * p.q_tile_bytes;
  p.off_kv = off;     off += p.kv_stages * kv_stage;
  p.off_bias = off;   off += kBiasStages * kBiasTileBytes;
  p.off_bar = off;    off += kBarrierBlockBytes;
  p.off_ones = off;   off += kMaskPanelBytes;
  p.off_mcol = off;   off += kMaxKvStages * kMaskPanelBytes;
  p.off_zero = off;   off += kMaskPanelBytes;
  p.off_ident = off;  off += kIdentBytes;
  size_t smem = off + 1024;
  // One CTA per SM is required (each CTA allocates all of TMEM): ask for more than half the SM's
  // shared memory even when the tiles need less.
  if (smem < 120 * 1024) smem = 120 * 1024;
  plan->smem_bytes = smem;
  const int ctas = (d.max_ctas > 0 && d.max_ctas < dev.sm_count) ? d.max_ctas : dev.sm_count;
  plan->grid = p.n_items < ctas ? p.n_items : ctas;
  return AF3K_OK;
}

int encode_qkv_map(CUtensorMap* tm, const void* base, bool fp8, int64_t D, int64_t S, int64_t B2,
                   int64_t B1, const int64_t* stride, int row_bytes) {
  auto enc = tensor_map_encoder();
  if (!enc) return driver_fail("cuTensorMapEncodeTiled entry point", -1);
  const uint64_t es = fp8 ? 1 : 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)B2, (cuuint64_t)B1};
  cuuint64_t strides[3] = {(cuuint64_t)stride[2] * es, (cuuint64_t)stride[1] * es,
                           (cuuint64_t)stride[0] * es};
  // a dimension of extent 1 may carry any stride; TMA still wants it non-zero and 16-aligned
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0) strides[i] = 16;
  cuuint32_t box[4] = {(cuuint32_t)(row_bytes / es), (cuuint32_t)kTile, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_for(row_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AF3K_OK : driver_fail("cuTensorMapEncodeTiled(q/k/v)", (int)r);
}

int encode_bias_map(CUtensorMap* tm, const void* base, int64_t Sk, int64_t Sq, int64_t B2,
                    int64_t stride_h, int64_t stride_r) {
  auto enc = tensor_map_encoder();
  if (!enc) return driver_fail("cuTensorMapEncodeTiled entry point", -1);
  cuuint64_t dims[3] = {(cuuint64_t)Sk, (cuuint64_t)Sq, (cuuint64_t)B2};
  cuuint64_t strides[2] = {(cuuint64_t)stride_r * 2, (cuuint64_t)stride_h * 2};
  for (int i = 0; i < 2; ++i)
    if (strides[i] == 0) strides[i] = 16;
  cuuint32_t box[3] = {64, (cuuint32_t)kTile, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AF3K_OK : driver_fail("cuTensorMapEncodeTiled(bias)", (int)r);
}

__global__ void wait_timeout_selftest_kernel(long long limit, int* status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    af3k::mbar_init(af3k::smem_u32(&bar), 1);
    af3k::fence_barrier_init();
    // nothing ever arrives on `bar`: the bounded wait must give up and report
    const bool ok = af3k::mbar_wait_bounded(af3k::smem_u32(&bar), 0, limit, &abort_flag);
    if (!ok && status != nullptr) atomicOr(status, (int)af3k::kStatusWaitTimeout);
    af3k::mbar_inval(af3k::smem_u32(&bar));
  }
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that have no way to hand us scratch memory.
//
// The bf16 staging copy of the bias normally lives in a caller-provided workspace.  Some hosts
// cannot provide one: a serving process that gave every byte of device memory to its own arena
// at start-up, a plug-in interface that only passes inputs and outputs through, or a
// latency-critical loop in which cudaMalloc (which synchronises the device) is forbidden.  For
// them the staging copy goes into a fixed array that is part of this library's device image.
// The array is reserved on every GPU that loads the library, for the life of the process, so
// its size is kept modest.
constexpr size_t kStaticScratchBytes = 16u << 20;   // 16 MiB: B2 * Sq * round_up(Sk, 8) <= 8 Mi entries
static __device__ __align__(256) unsigned char g_static_bias_scratch[kStaticScratchBytes];

// In host code the name of a __device__ array is only a handle for the runtime, not an address
// the GPU can use; the real device address has to be asked for, per device.
int static_scratch_address(void** out) {
  static void* addr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return cuda_fail("cudaGetDevice", e);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_bias_scratch);   // resolves for the current device
    if (e != cudaSuccess || p == nullptr) return cuda_fail("cudaGetSymbolAddress(static scratch)", e);
    addr[dev] = p;
  }
  *out = addr[dev];
  return AF3K_OK;
}

}  // namespace

extern "C" {

int af3k_version(void) { return 1002; }

const char* af3k_strerror(int code) {
  switch (code) {
    case AF3K_OK: return "ok";
    case AF3K_ERR_BAD_DTYPE: return "unsupported element type";
    case AF3K_ERR_BAD_SHAPE: return "unsupported shape (D must be a multiple of 8 and <= 64; Sk > 0)";
    case AF3K_ERR_BAD_STRIDE: return "unsupported stride (innermost must be 1, others 16-byte multiples)";
    case AF3K_ERR_BAD_ALIGNMENT: return "pointer is not 16-byte aligned";
    case AF3K_ERR_WORKSPACE: return "workspace missing or too small";
    case AF3K_ERR_NULL_POINTER: return "null pointer";
    case AF3K_ERR_CUDA: return "CUDA runtime or driver call failed";
    case AF3K_ERR_UNSUPPORTED_DEVICE: return "device is not compute capability 10.x (B200)";
    case AF3K_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the built-in array holds";
    default: return "unknown error code";
  }
}

size_t af3k_dot_product_attention_workspace(const af3k_attention_desc* desc, const void* bias) {
  if (desc == nullptr || validate(*desc) != AF3K_OK) return 0;
  // fp8 q/k: the staging copy is what lets the tensor core add the bias (optional, see the entry)
  if (!bias_needs_staging(*desc, bias) && (desc->qk_dtype != AF3K_FP8_E4M3 || desc->bias_prescaled)) return 0;
  return (size_t)desc->B2 * desc->Sq * staged_bias_pitch(desc->Sk) * 2;
}

int af3k_last_launch_count(void) { return t_last_launches; }

const char* af3k_last_error_detail(void) { return t_detail; }

void af3k_set_wait_limit_cycles(long long cycles) { g_wait_limit.store(cycles > 0 ? cycles : -1); }

namespace {
int launch_bias_staging(const af3k_attention_desc& d, const DeviceInfo& dev, const void* bias, const float* sq,
                        const float* sk, void* staged, cudaStream_t stream) {
  const int64_t pitch = staged_bias_pitch(d.Sk);
  const long long total = (long long)d.B2 * d.Sq * (pitch / 2);
  int blocks = (int)((total + 255) / 256);
  if (blocks > dev.sm_count * 16) blocks = dev.sm_count * 16;
  if (d.bias_dtype == AF3K_F32)
    bias_to_bf16_kernel<float><<<blocks, 256, 0, stream>>>(
        static_cast<const float*>(bias), static_cast<__nv_bfloat16*>(staged), (int)d.B2, (int)d.Sq,
        (int)d.Sk, d.bias_stride[0], d.bias_stride[1], (int)pitch, sq, sk, d.softmax_scale);
  else
    bias_to_bf16_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(staged), (int)d.B2,
        (int)d.Sq, (int)d.Sk, d.bias_stride[0], d.bias_stride[1], (int)pitch, sq, sk, d.softmax_scale);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AF3K_OK : cuda_fail("launch bias_to_bf16_kernel", e);
}
}  // namespace

int af3k_stage_bias(const af3k_attention_desc* desc, const void* bias, const float* q_scale,
                    const float* k_scale, void* staged, size_t staged_bytes, void* stream_v) {
  t_last_launches = 0;
  if (desc == nullptr) return AF3K_ERR_NULL_POINTER;
  af3k_attention_desc d = *desc;
  d.bias_prescaled = 0;      // describes the input bias here
  int rc = validate(d);
  if (rc != AF3K_OK) return rc;
  if (d.B2 == 0 || d.Sq == 0) return AF3K_OK;
  if (!bias || !staged) return AF3K_ERR_NULL_POINTER;
  if ((q_scale != nullptr) != (k_scale != nullptr)) return AF3K_ERR_BAD_DTYPE;
  if (q_scale != nullptr && d.qk_dtype != AF3K_FP8_E4M3) return AF3K_ERR_BAD_DTYPE;
  if (!aligned16(staged)) return AF3K_ERR_BAD_ALIGNMENT;
  if (staged_bytes < (size_t)d.B2 * d.Sq * staged_bias_pitch(d.Sk) * 2) return AF3K_ERR_WORKSPACE;
  DeviceInfo* dev = nullptr;
  if ((rc = device_info(&dev)) != AF3K_OK) return rc;
  rc = launch_bias_staging(d, *dev, bias, q_scale, k_scale, staged, reinterpret_cast<cudaStream_t>(stream_v));
  if (rc == AF3K_OK) t_last_launches = 1;
  return rc;
}

int af3k_dot_product_attention(const af3k_attention_desc* desc, const void* q, const void* k,
                               const void* v, const void* bias, const uint8_t* mask, void* out,
                               const float* q_scale, const float* k_scale, void* workspace,
                               size_t workspace_bytes, int* status_dev, void* stream_v) {
  t_last_launches = 0;
  if (desc == nullptr) return AF3K_ERR_NULL_POINTER;
  const af3k_attention_desc& d = *desc;
  int rc = validate(d);
  if (rc != AF3K_OK) return rc;
  if (d.B1 == 0 || d.B2 == 0 || d.Sq == 0) return AF3K_OK;  // empty output
  if (!q || !k || !v || !bias || !out) return AF3K_ERR_NULL_POINTER;
  const bool fp8 = d.qk_dtype == AF3K_FP8_E4M3;
  if (fp8 != (q_scale != nullptr) || fp8 != (k_scale != nullptr)) return AF3K_ERR_BAD_DTYPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return AF3K_ERR_BAD_ALIGNMENT;

  DeviceInfo* dev = nullptr;
  rc = device_info(&dev);
  if (rc != AF3K_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);

  // fp8 q/k run the tensor-core-bias kernel when the bias is (or can be) staged pre-divided by
  // the logit scale; bf16 q/k always do
  const bool fp8_with_tc_bias = fp8 && (d.bias_prescaled ||
      (workspace != nullptr && aligned16(workspace) &&
       workspace_bytes >= (size_t)d.B2 * d.Sq * staged_bias_pitch(d.Sk) * 2));
  Plan plan;
  rc = make_plan(d, *dev, &plan, !fp8 || fp8_with_tc_bias);
  if (rc != AF3K_OK) return rc;
  AttnParams& p = plan.p;
  if (plan.smem_bytes > (size_t)(dev->max_smem_optin - kStaticSmemReserve)) return AF3K_ERR_BAD_SHAPE;

  // bias: use in place when TMA can address it, else stage a bf16 copy in the workspace
  const void* bias_base = bias;
  int64_t bias_sh = d.bias_stride[0], bias_sr = d.bias_stride[1];
  int launches = 0;
  // fp8 q/k: with a staging copy divided by the head's logit scale the tensor core adds the bias
  // to the raw fp8 products (the fast kernel); without room for one the softmax threads add the
  // bias in fp32 as before
  const size_t stage_bytes = (size_t)d.B2 * d.Sq * staged_bias_pitch(d.Sk) * 2;
  const bool must_stage = bias_needs_staging(d, bias);
  if (d.bias_prescaled && must_stage) return AF3K_ERR_BAD_STRIDE;   // a staged copy is TMA-addressable by construction
  const bool stage_fp8 = fp8 && !d.bias_prescaled && workspace != nullptr && workspace_bytes >= stage_bytes &&
                         aligned16(workspace);
  const bool fp8_tc = fp8 && (d.bias_prescaled || stage_fp8);
  if (must_stage || stage_fp8) {
    if (workspace == nullptr || workspace_bytes < stage_bytes) return AF3K_ERR_WORKSPACE;
    if (!aligned16(workspace)) return AF3K_ERR_BAD_ALIGNMENT;
    const int64_t pitch = staged_bias_pitch(d.Sk);
    if ((rc = launch_bias_staging(d, *dev, bias, stage_fp8 ? q_scale : nullptr, stage_fp8 ? k_scale : nullptr,
                                  workspace, stream)) != AF3K_OK)
      return rc;
    ++launches;
    bias_base = workspace;
    bias_sr = pitch;
    bias_sh = pitch * d.Sq;
  }

  CUtensorMap tm_q, tm_k, tm_v, tm_b;
  if ((rc = encode_qkv_map(&tm_q, q, fp8, d.D, d.Sq, d.B2, d.B1, d.q_stride, p.qk_row_bytes))) return rc;
  if ((rc = encode_qkv_map(&tm_k, k, fp8, d.D, d.Sk, d.B2, d.B1, d.k_stride, p.qk_row_bytes))) return rc;
  if ((rc = encode_qkv_map(&tm_v, v, false, d.D, d.Sk, d.B2, d.B1, d.v_stride, p.v_row_bytes))) return rc;
  if ((rc = encode_bias_map(&tm_b, bias_base, d.Sk, d.Sq, d.B2, bias_sh, bias_sr))) return rc;

  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.mask = mask;
  p.mask_row_stride = d.mask_row_stride;
  p.mask_col = (mask != nullptr || d.Sk % kTile != 0) ? 1 : 0;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride_b1 = d.out_stride[0];
  p.out_stride_b2 = d.out_stride[1];
  p.out_stride_s = d.out_stride[2];
  p.status = status_dev;
  p.wait_limit = wait_limit_cycles();

  p.debug = g_debug_dump.load();
  // scale, bias and mask all come out of the tensor core, except for fp8 q/k without a staging
  // copy of the bias: there the softmax threads apply scale and bias in fp32
  const bool tc_bias = !fp8 || fp8_tc;
  p.scale_q = (fp8 || d.softmax_scale == 1.0f) ? 0 : 1;   // a scale of exactly 1 (q already scaled by its producer) needs no pass over Q
  const bool dbg = p.debug != nullptr;
#define AF3K_LAUNCH(...) attention_kernel<__VA_ARGS__><<<plan.grid, kThreads, plan.smem_bytes, stream>>>(p, tm_q, tm_k, tm_v, tm_b)
  if (!tc_bias) {
    if (dbg) AF3K_LAUNCH(true, false); else AF3K_LAUNCH(false, false);
  } else {
    if (dbg) AF3K_LAUNCH(true, true); else AF3K_LAUNCH(false, true);
  }
#undef AF3K_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("launch attention_kernel", e);
  ++launches;
  t_last_launches = launches;
  return AF3K_OK;
}

void af3k_debug_set_dump(float* dump_dev) { g_debug_dump.store(dump_dev); }

int af3k_describe_plan(const af3k_attention_desc* desc, int32_t* out6) {
  if (desc == nullptr || out6 == nullptr) return AF3K_ERR_NULL_POINTER;
  int rc = validate(*desc);
  if (rc != AF3K_OK) return rc;
  DeviceInfo dev;
  dev.sm_count = 148;
  dev.cc_major = 10;
  dev.max_smem_optin = 232448;
  int cur = 0;
  cudaDeviceProp prop;
  if (cudaGetDevice(&cur) == cudaSuccess && cudaGetDeviceProperties(&prop, cur) == cudaSuccess &&
      prop.major == 10) {
    dev.sm_count = prop.multiProcessorCount;
    dev.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  }
  Plan plan;
  rc = make_plan(*desc, dev, &plan);
  if (rc != AF3K_OK) return rc;
  out6[0] = plan.p.G;
  out6[1] = plan.p.kv_stages;
  out6[2] = plan.p.n_items;
  out6[3] = plan.grid;
  out6[4] = (int32_t)plan.smem_bytes;
  out6[5] = (int32_t)kOCol + plan.p.n_streams * plan.p.nv;
  return AF3K_OK;
}

size_t af3k_static_scratch_bytes(void) { return kStaticScratchBytes; }

int af3k_dot_product_attention_noalloc(const af3k_attention_desc* desc, const void* q,
                                       const void* k, const void* v, const void* bias,
                                       const uint8_t* mask, void* out, const float* q_scale,
                                       const float* k_scale, int* status_dev, void* stream) {
  if (desc == nullptr) return AF3K_ERR_NULL_POINTER;
  int rc = validate(*desc);
  if (rc != AF3K_OK) return rc;
  // the staging copy is required for a bias TMA cannot read in place, optional (faster kernel)
  // for fp8 q/k: an optional copy that does not fit is simply not made
  size_t need = af3k_dot_product_attention_workspace(desc, bias);
  if (need > kStaticScratchBytes && !bias_needs_staging(*desc, bias)) need = 0;
  if (need > kStaticScratchBytes) {
    std::snprintf(t_detail, sizeof(t_detail),
                  "bias staging copy needs %zu bytes, the built-in scratch holds %zu", need,
                  kStaticScratchBytes);
    return AF3K_ERR_SCRATCH_LIMIT;
  }
  // the device check comes first, so that a GPU this library has no code for is reported as
  // such and not as a failed symbol lookup
  DeviceInfo* dev = nullptr;
  if ((rc = device_info(&dev)) != AF3K_OK) return rc;
  void* scratch = nullptr;
  if (need != 0 && (rc = static_scratch_address(&scratch)) != AF3K_OK) return rc;
  // From here on this is the ordinary call with the built-in array as its workspace.  The
  // staging pre-pass rewrites every entry it later reads (pad columns included), so nothing of a
  // previous call's contents needs clearing.
  return af3k_dot_product_attention(desc, q, k, v, bias, mask, out, q_scale, k_scale, scratch,
                                    need != 0 ? kStaticScratchBytes : 0, status_dev, stream);
}

int af3k_pair_bias(const void* pair, int32_t pair_dtype, int64_t R, int64_t N, int64_t C, int64_t H,
                   const float* gamma, const float* beta, const float* proj, float eps, void* normed,
                   void* bias, int64_t bias_pitch, void* stream_v) {
  t_last_launches = 0;
  if (pair_dtype != AF3K_BF16 && pair_dtype != AF3K_F32) return AF3K_ERR_BAD_DTYPE;
  if (C != kPbChannels || H < 1 || H > kPbMaxHeads || R < 0 || N < 0 || R > 0x7fffffff || N > 0x7fffffff)
    return AF3K_ERR_BAD_SHAPE;
  if (bias_pitch < N || (bias_pitch & 7) != 0) return AF3K_ERR_BAD_STRIDE;
  if (R == 0 || N == 0) return AF3K_OK;
  if (!pair || !gamma || !beta || !proj || !normed || !bias) return AF3K_ERR_NULL_POINTER;
  if (!aligned16(pair) || !aligned16(normed) || !aligned16(bias)) return AF3K_ERR_BAD_ALIGNMENT;
  DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != AF3K_OK) return rc;
  PairBiasParams p;
  p.pair = pair; p.normed = static_cast<__nv_bfloat16*>(normed); p.bias = static_cast<__nv_bfloat16*>(bias);
  p.gamma = gamma; p.beta = beta; p.proj = proj;
  p.R = (int)R; p.N = (int)N; p.H = (int)H; p.bias_pitch = bias_pitch; p.eps = eps;
  // persistent CTAs (two per SM for the 4-head kernel, one for the wide ones) over R * ceil(N / 128) tiles
  const long long n_tiles = R * ((N + kPbTileJ - 1) / kPbTileJ);
  const long long max_ctas = (long long)dev->sm_count * (H <= 4 ? 2 : 1);
  const unsigned grid = (unsigned)(n_tiles < max_ctas ? n_tiles : max_ctas);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const bool f32 = pair_dtype == AF3K_F32;
#ifndef AF3K_PB_MMA_MIN_HEADS
#define AF3K_PB_MMA_MIN_HEADS 5
#endif
  if (!f32 && H >= AF3K_PB_MMA_MIN_HEADS) {
    // bf16 pair, more than four heads: moments and normalisation per thread, the head projection on
    // the tensor core (its time does not depend on the head count)
    const long long cap = (long long)dev->sm_count * 5;
    const unsigned grid_m = (unsigned)(n_tiles < cap ? n_tiles : cap);
    pair_bias_mma_kernel<<<grid_m, kPbmRows, kPbmSmemBytes, stream>>>(p, wait_limit_cycles());
  } else if (H <= 4) {
    // one thread per vector, tiles transposed through shared memory; five CTAs fit an SM
    const long long tiles_t = R * ((N + (f32 ? 64 : 128) - 1) / (f32 ? 64 : 128));
    const long long cap = (long long)dev->sm_count * 5;
    const unsigned grid_t = (unsigned)(tiles_t < cap ? tiles_t : cap);
    if (f32) pair_bias_kernel_t<float><<<grid_t, PbTile<float>::kRows, PbTile<float>::kSmemBytes, stream>>>(p);
    else     pair_bias_kernel_t<__nv_bfloat16><<<grid_t, PbTile<__nv_bfloat16>::kRows,
                                                PbTile<__nv_bfloat16>::kSmemBytes, stream>>>(p);
  } else if (H <= 8) {
    if (f32) pair_bias_kernel<float, 8><<<grid, kPbThreads, 0, stream>>>(p);
    else     pair_bias_kernel<__nv_bfloat16, 8><<<grid, kPbThreads, 0, stream>>>(p);
  } else {
    if (f32) pair_bias_kernel<float, 16><<<grid, kPbThreads, 0, stream>>>(p);
    else     pair_bias_kernel<__nv_bfloat16, 16><<<grid, kPbThreads, 0, stream>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("launch pair_bias_kernel", e);
  t_last_launches = 1;
  return AF3K_OK;
}

int af3k_pair_bias_status(int32_t* out4) {
  if (out4 == nullptr) return AF3K_ERR_NULL_POINTER;
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, g_pair_bias_status, sizeof(host));
  if (e != cudaSuccess) return cuda_fail("cudaMemcpyFromSymbol(pair-bias status)", e);
  for (int i = 0; i < 4; ++i) out4[i] = host[i];
  if (host[0] != 0) {
    const int zero[4] = {0, 0, 0, 0};
    if ((e = cudaMemcpyToSymbol(g_pair_bias_status, zero, sizeof(zero))) != cudaSuccess)
      return cuda_fail("cudaMemcpyToSymbol(pair-bias status)", e);
  }
  return AF3K_OK;
}

}  // extern "C"

namespace {
// Shared by af3k_qkvg_projection (x already layer-normed) and af3k_pair_front (x is the raw pair:
// the kernel's LayerNorm warpgroup normalises every tile in shared memory and writes the bias).
int launch_projection(const void* x, const void* w4, int64_t R, int64_t N, int64_t H, float q_scale, void* q,
                      void* k, void* v, void* gate, int* status_dev, void* stream_v, bool with_ln,
                      const float* gamma, const float* beta, const float* bias_w, int64_t Hb, float eps,
                      void* bias, int64_t bias_pitch) {
  t_last_launches = 0;
  if (R < 0 || N < 0 || H < 1 || kProjC % H != 0 || (kProjC / H) % 8 != 0) return AF3K_ERR_BAD_SHAPE;
  if (R > 0x7fffffff || N > 0x7fffffff || R * N > 0x7fffff00LL * 128) return AF3K_ERR_BAD_SHAPE;
  if (with_ln && (Hb < 1 || Hb > 4)) return AF3K_ERR_BAD_SHAPE;
  if (with_ln && (bias_pitch < N || (bias_pitch & 7) != 0)) return AF3K_ERR_BAD_STRIDE;
  if (R == 0 || N == 0) return AF3K_OK;
  if (!x || !w4 || !q || !k || !v || !gate) return AF3K_ERR_NULL_POINTER;
  if (with_ln && (!gamma || !beta || !bias_w || !bias)) return AF3K_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(w4) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(gate))
    return AF3K_ERR_BAD_ALIGNMENT;
  if (with_ln && (!aligned16(gamma) || !aligned16(beta) || !aligned16(bias_w) || !aligned16(bias)))
    return AF3K_ERR_BAD_ALIGNMENT;
  DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != AF3K_OK) return rc;
  auto enc = tensor_map_encoder();
  if (!enc) return driver_fail("cuTensorMapEncodeTiled entry point", -1);
  const long long M = R * N;
  if (M * kProjC > 0x7fffffffLL) return AF3K_ERR_BAD_SHAPE;    // 32-bit element offsets in the epilogue, 32-bit TMA coordinates
  CUtensorMap tm_x, tm_w;
  {
    cuuint64_t dims[2] = {(cuuint64_t)kProjC, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)kProjC * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return driver_fail("cuTensorMapEncodeTiled(x)", (int)r);
    cuuint64_t wdims[2] = {(cuuint64_t)kProjC, (cuuint64_t)kProjOut};
    cuuint32_t wbox[2] = {64, 256};
    r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w4), wdims, strides, wbox, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return driver_fail("cuTensorMapEncodeTiled(w4)", (int)r);
  }
  ProjParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = M; p.N = (int)N; p.H = (int)H; p.D = kProjC / (int)H; p.q_scale = q_scale;
  p.q = static_cast<__nv_bfloat16*>(q); p.k = static_cast<__nv_bfloat16*>(k);
  p.v = static_cast<__nv_bfloat16*>(v); p.g = static_cast<__nv_bfloat16*>(gate);
  p.status = status_dev;
  p.wait_limit = wait_limit_cycles();
  p.gamma = gamma; p.beta = beta; p.bias_w = bias_w; p.bias = static_cast<__nv_bfloat16*>(bias);
  p.bias_pitch = bias_pitch; p.Hb = (int)Hb; p.R = (int)R; p.eps = eps;
  const long long n_tiles = (M + 127) / 128;
  const unsigned grid = (unsigned)(n_tiles < dev->sm_count ? n_tiles : dev->sm_count);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (with_ln) qkvg_projection_kernel<true><<<grid, kProjLnThreads, kProjSmemBytes, stream>>>(p, tm_x, tm_w);
  else         qkvg_projection_kernel<false><<<grid, kProjThreads, kProjSmemBytes, stream>>>(p, tm_x, tm_w);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("launch qkvg_projection_kernel", e);
  t_last_launches = 1;
  return AF3K_OK;
}
}  // namespace

extern "C" {

int af3k_qkvg_projection(const void* x, const void* w4, int64_t R, int64_t N, int64_t H, float q_scale,
                         void* q, void* k, void* v, void* gate, int* status_dev, void* stream_v) {
  return launch_projection(x, w4, R, N, H, q_scale, q, k, v, gate, status_dev, stream_v, false, nullptr, nullptr,
                           nullptr, 0, 0.f, nullptr, 0);
}

int af3k_pair_front(const void* pair, const float* gamma, const float* beta, float eps, const float* bias_w,
                    int64_t Hb, const void* w4, int64_t R, int64_t N, int64_t H, float q_scale, void* bias,
                    int64_t bias_pitch, void* q, void* k, void* v, void* gate, int* status_dev, void* stream_v) {
  return launch_projection(pair, w4, R, N, H, q_scale, q, k, v, gate, status_dev, stream_v, true, gamma, beta,
                           bias_w, Hb, eps, bias, bias_pitch);
}

int af3k_sigmoid_gate(const void* weighted, const void* gate, void* out, int64_t n, void* stream_v) {
  t_last_launches = 0;
  if (n < 0 || (n & 7) != 0) return AF3K_ERR_BAD_SHAPE;
  if (n == 0) return AF3K_OK;
  if (!weighted || !gate || !out) return AF3K_ERR_NULL_POINTER;
  if (!aligned16(weighted) || !aligned16(gate) || !aligned16(out)) return AF3K_ERR_BAD_ALIGNMENT;
  DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != AF3K_OK) return rc;
  const long long n8 = n / 8;
  long long blocks = (n8 + 255) / 256;
  const long long cap = (long long)dev->sm_count * 8;
  if (blocks > cap) blocks = cap;
  sigmoid_gate_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const uint4*>(weighted), static_cast<const uint4*>(gate), static_cast<uint4*>(out), n8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("launch sigmoid_gate_kernel", e);
  t_last_launches = 1;
  return AF3K_OK;
}

int af3k_selftest_wait_timeout(long long limit_cycles, int* status_dev, void* stream_v) {
  if (limit_cycles <= 0) return AF3K_ERR_BAD_SHAPE;
  wait_timeout_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(limit_cycles,
                                                                                      status_dev);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AF3K_OK : cuda_fail("launch wait_timeout_selftest_kernel", e);
}

}  // extern "C"
