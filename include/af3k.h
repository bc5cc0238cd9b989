/* C ABI of the B200 (sm_100a) attention library  libaf3k.so.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless stated otherwise.  The
 * library borrows all buffers, owns nothing, writes only `out`, `workspace` and `status_dev`,
 * and launches on the stream it is given without synchronising.
 *
 * Each entry point names the reference interface it stands in for (paths are those of the
 * HPC-SJTU/af3_kernels source tree).
 */
#ifndef AF3K_H_
#define AF3K_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* return codes (0 = ok).  af3k_strerror() gives the text. */
enum {
  AF3K_OK = 0,
  AF3K_ERR_BAD_DTYPE = 1,
  AF3K_ERR_BAD_SHAPE = 2,
  AF3K_ERR_BAD_STRIDE = 3,
  AF3K_ERR_BAD_ALIGNMENT = 4,
  AF3K_ERR_WORKSPACE = 5,
  AF3K_ERR_NULL_POINTER = 6,
  AF3K_ERR_CUDA = 7,
  AF3K_ERR_UNSUPPORTED_DEVICE = 8,
  AF3K_ERR_SCRATCH_LIMIT = 9
};

/* element types */
enum {
  AF3K_BF16 = 0,
  AF3K_F32 = 1,
  AF3K_FP8_E4M3 = 2
};

/* bits of the device status word written by the kernels (0 = clean run) */
enum {
  AF3K_STATUS_WAIT_TIMEOUT = 1 /* a bounded on-device wait ran out; output is not valid */
};

/* Shapes, strides (in ELEMENTS) and types of one attention call.
 *   q, k, v, out : [B1, B2, S, D]   innermost (D) stride must be 1
 *   bias         : [B2, Sq, Sk]     shared by every b1; innermost stride must be 1
 *   mask         : [B1, Sk] bytes, non-zero = attend; row stride 0 broadcasts one row
 * D must be a multiple of 8 and at most 64.  q/k may be bf16 or fp8-e4m3 (then q_scale/k_scale
 * hold one fp32 de-quantisation factor per head); v and out are bf16; bias is bf16 or fp32.
 */
typedef struct af3k_attention_desc {
  int64_t B1, B2, Sq, Sk, D;
  int64_t q_stride[3];    /* b1, b2, s */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t out_stride[3];
  int64_t bias_stride[2]; /* head, query row */
  int64_t mask_row_stride;
  int32_t qk_dtype;       /* AF3K_BF16 or AF3K_FP8_E4M3 */
  int32_t bias_dtype;     /* AF3K_BF16 or AF3K_F32 */
  float softmax_scale;    /* the reference uses 1/sqrt(D) */
  int32_t rows_per_item;  /* 0 = choose; else requested pair rows per staged bias tile (1..8, clamped to what fits, at most 4) */
  int32_t bias_prescaled; /* fp8 q/k only: 1 = `bias` is the output of af3k_stage_bias for these scales (already divided
                             by the head's logit scale); the tensor core adds it and no staging pass runs.  0 otherwise. */
  int32_t max_ctas;       /* 0 = one CTA per SM; > 0: at most this many CTAs, leaving the other SMs to
                             kernels that run beside this one (the collective that gathers a
                             row-sharded output while the next piece is computed) */
} af3k_attention_desc;

/* Library / ABI version (major * 1000 + minor). */
int af3k_version(void);

/* Text for a return code.  Never NULL. */
const char* af3k_strerror(int code);

/* For AF3K_ERR_CUDA: which CUDA call failed on this thread and the runtime's text for it
 * ("" if none failed yet).  Never NULL. */
const char* af3k_last_error_detail(void);

/* Bytes of device scratch af3k_dot_product_attention can use for this problem (0 if none): the
 * bf16 staging copy of the bias.  It is required for a bias that is fp32 or whose row pitch TMA
 * cannot address (AF3K_ERR_WORKSPACE without it); with fp8 q/k it is optional and selects the
 * faster kernel, in which the tensor core adds the (pre-scaled) bias. */
size_t af3k_dot_product_attention_workspace(const af3k_attention_desc* desc, const void* bias);

/* The bias staging pass on its own, for callers that use one bias in many attention calls (the
 * diffusion transformer applies the same pair bias in every denoising step): converts `bias`
 * (bf16 or fp32, any row pitch) into `staged`, a bf16 [B2, Sq, round_up(Sk, 8)] array that
 * af3k_dot_product_attention reads in place, so that later calls launch one kernel instead of
 * two.  Pass `staged` as the bias of those calls with bias_dtype = AF3K_BF16 and bias_stride =
 * {Sq * round_up(Sk, 8), round_up(Sk, 8)}.  With fp8 q/k (q_scale / k_scale non-NULL) every value
 * is also divided by softmax_scale * q_scale[h] * k_scale[h]; set desc.bias_prescaled = 1 in the
 * calls that use such a copy.  staged_bytes must be at least
 * af3k_dot_product_attention_workspace()'s figure for an fp32 bias of this shape (B2 * Sq *
 * round_up(Sk, 8) * 2).  Stands in for the cast the reference's wrapper makes on every call
 * (`bias = bias.to(q.dtype)`, src/af3_kernels/__init__.py:48). */
int af3k_stage_bias(const af3k_attention_desc* desc, const void* bias, const float* q_scale,
                    const float* k_scale, void* staged, size_t staged_bytes, void* stream);

/* out = softmax(scale * q k^T + bias, key-masked) v
 *
 * Stands in for  at::Tensor dot_product_attention(q, k, v, mask, bias, use_flash_attention,
 * BLK_SZ, FLASH_SZ)  (src/csrc/dot_product_attention.h:25-32, bound at src/csrc/init.cpp:349-351)
 * and the work its Python wrapper does before it (src/af3_kernels/__init__.py:41-50).
 * Differences a caller sees: inputs are never written (the reference overwrites q), the result
 * goes to a caller-provided `out`, masked keys are a byte predicate instead of an additive
 * -1e9 tensor, and errors come back as codes instead of exit(1).
 * Rounding points with bf16 q/k: q * softmax_scale is rounded to bf16 before the first GEMM (as
 * in the reference); logits, bias add and softmax are fp32 (the reference rounds the logits to
 * bf16); the weights are rounded to bf16 for the second GEMM (as in the reference).
 *
 * mask may be NULL (no key is masked).  q_scale / k_scale must be NULL for bf16 q/k.
 * status_dev may be NULL; otherwise it must point at int[4] the caller zeroed: [0] is OR-ed
 * with AF3K_STATUS_* bits by the device, [1..3] identify the first wait that gave up
 * (1 + barrier slot, block, warp).  stream is a cudaStream_t.
 */
int af3k_dot_product_attention(const af3k_attention_desc* desc, const void* q, const void* k,
                               const void* v, const void* bias, const uint8_t* mask, void* out,
                               const float* q_scale, const float* k_scale, void* workspace,
                               size_t workspace_bytes, int* status_dev, void* stream);

/* The same operation for callers that cannot supply a workspace and cannot allocate one: a
 * host that handed all device memory to its own arena at start-up, a plug-in boundary that only
 * carries inputs and outputs, or a serving loop where cudaMalloc (which synchronises the whole
 * device) is not allowed.  This entry point has no counterpart in the reference.
 *
 * It makes no cudaMalloc / cudaFree call and uses no allocating library routine.  The bias
 * staging copy goes into an array of af3k_static_scratch_bytes() (16 MiB) that is built into the
 * library's device image, so every GPU that loads the library gives up that much memory until
 * the process exits.  A problem whose staging copy is larger (B2 * Sq * round_up(Sk, 8) * 2
 * bytes; none is needed for a bf16 bias with 16-byte-aligned rows) is refused with
 * AF3K_ERR_SCRATCH_LIMIT and nothing is launched.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call outside any stream capture.  The address is kept
 * for the life of the process: after a cudaDeviceReset of that device it is stale and this entry
 * point must not be used again in the process.  With fp8 q/k the staging copy is optional; when
 * it does not fit the array it is left out and the slower kernel variant runs (no error).  All calls on a device
 * share the one array: two calls whose kernels can overlap on the GPU (different streams) race
 * on it, so keep them on one stream or order them with events.  Nothing in the array has to be
 * cleared between calls; each call rewrites every entry it reads.
 * Arguments are those of af3k_dot_product_attention without the workspace pair. */
int af3k_dot_product_attention_noalloc(const af3k_attention_desc* desc, const void* q,
                                       const void* k, const void* v, const void* bias,
                                       const uint8_t* mask, void* out, const float* q_scale,
                                       const float* k_scale, int* status_dev, void* stream);

/* Size in bytes of the built-in scratch array used by af3k_dot_product_attention_noalloc. */
size_t af3k_static_scratch_bytes(void);

/* Number of kernels the last successful af3k_dot_product_attention call on this thread
 * launched (1, or 2 when the bias staging pre-pass ran). */
int af3k_last_launch_count(void);

/* Upper bound, in SM clock cycles, for any single on-device wait (default 2e9, about a second).
 * A kernel whose wait runs out sets AF3K_STATUS_WAIT_TIMEOUT and returns. */
void af3k_set_wait_limit_cycles(long long cycles);

/* Launch plan the library would use for `desc` on the current device (a B200 with 148 SMs and
 * 227 KB of shared memory per block is assumed when no such device is present, so this also
 * works on a CPU-only host): out6 = {pair rows per work item, K/V ring stages, work items,
 * grid size, dynamic shared memory bytes, TMEM columns used}.  Diagnostic; no counterpart in
 * the reference. */
int af3k_describe_plan(const af3k_attention_desc* desc, int32_t* out6);

/* Diagnostic: when dump_dev is non-NULL, later attention calls run a debug build of the kernel
 * that writes block 0's first logits tile to dump_dev (4 * 128 * 128 floats: logits as the
 * tensor core delivers them - with bf16 q/k that is scale * q k^T + bias + mask value -, packed
 * P words, un-normalised O, {max, sum}), followed by 2 * (2 * 256 * 8 + 4 * 256) floats of
 * SM-clock stamps.  Pass NULL to switch it off.  No counterpart in the reference. */
void af3k_debug_set_dump(float* dump_dev);

/* Pair-bias producer: LayerNorm over the 128 channels of the pair representation, the per-head
 * bias projection and the [N, N, H] -> [H, N, N] permute, in one pass.
 *
 * Stands in for the two statements in front of the attention core in the reference's modules,
 *     pair = self.act_norm(pair); bias = self.pair_bias_projection(pair).permute(2, 0, 1)
 * (src/af3_kernels/Attention.py:51-52 and :152-153).
 *
 *   pair    [R, N, 128] contiguous, pair_dtype AF3K_BF16 or AF3K_F32
 *   gamma, beta [128] fp32 (LayerNorm weight and bias), proj [H, 128] fp32 (nn.Linear weight)
 *   normed  [R, N, 128] bf16: the normalised pair (operand of the q / k / v / gate projections)
 *   bias    [H, R, bias_pitch] bf16, bias_pitch >= N and a multiple of 8: element (h, i, j) is the
 *           logit bias of head h between positions i and j, bias[h][i][j] =
 *           sum_c bf16(normed[i][j][c]) * proj[h][c]; pad columns are not written
 * 1 <= H <= 16.  All pointers 16-byte aligned.  stream is a cudaStream_t.
 * A bf16 pair with more than four heads runs the projection on the tensor core (each fp32 weight as
 * a bf16 high part plus a bf16 low part, fp32 accumulation); its waits are bounded and report
 * through af3k_pair_bias_status. */
int af3k_pair_bias(const void* pair, int32_t pair_dtype, int64_t R, int64_t N, int64_t C, int64_t H,
                   const float* gamma, const float* beta, const float* proj, float eps, void* normed,
                   void* bias, int64_t bias_pitch, void* stream);

/* Status of the pair-bias producer on the current device: out4 = {1 when a bounded wait of the
 * kernel ran out (its MMAs did not complete within the wait limit), block, tile, 0}; reading a
 * non-zero status clears it.  Synchronises the device.  No counterpart in the reference. */
int af3k_pair_bias_status(int32_t* out4);

/* The four input projections of the grid / triangle attention block in one pass over the
 * layer-normed pair representation (c_pair = 128):  [q | k | v | gate] = x * W4^T.
 *
 * Stands in for the K / V projection BRGEMMs per (pair row, head) and the Q and gate projection
 * BRGEMMs per query block inside the reference's fused block
 * (src/csrc/dot_product_attention.cpp:285-298 and :300-338).
 *
 *   x     [R, N, 128] bf16, contiguous
 *   w4    [512, 128] bf16: the four nn.Linear weights (out x in) stacked in the order q, k, v, gate
 *   q,k,v [R, H, N, 128 / H] bf16, contiguous (what af3k_dot_product_attention reads with unit-stride
 *         rows); q is multiplied by q_scale in fp32 before it is rounded, so the attention call
 *         that follows passes softmax_scale = 1
 *   gate  [R, N, 128] bf16
 * H must divide 128 with 128 / H a multiple of 8.  All pointers 16-byte aligned.  status_dev as in
 * af3k_dot_product_attention (may be NULL).  stream is a cudaStream_t. */
int af3k_qkvg_projection(const void* x, const void* w4, int64_t R, int64_t N, int64_t H, float q_scale,
                         void* q, void* k, void* v, void* gate, int* status_dev, void* stream);

/* The whole front of the grid / triangle attention block in one pass over the RAW pair
 * representation (bf16, c_pair = 128):
 *     x = LayerNorm(pair);  bias = (x W_b^T).permute(2, 0, 1);  [q | k | v | gate] = x W4^T
 * i.e. af3k_pair_bias followed by af3k_qkvg_projection without the normalised pair's round trip
 * through HBM (src/af3_kernels/Attention.py:51-52, :152-153 and
 * src/csrc/dot_product_attention.cpp:285-338).  x is rounded to bf16 before both projections, as
 * the stand-alone entry points do.
 *
 *   pair   [R, N, 128] bf16, contiguous;  gamma, beta [128] fp32;  bias_w [Hb, 128] fp32, 1 <= Hb <= 4
 *   bias   [Hb, R, bias_pitch] bf16, bias_pitch >= N and a multiple of 8 (pad columns not written)
 *   w4, q, k, v, gate, H, q_scale, status_dev: as in af3k_qkvg_projection
 * All pointers 16-byte aligned.  stream is a cudaStream_t. */
int af3k_pair_front(const void* pair, const float* gamma, const float* beta, float eps, const float* bias_w,
                    int64_t Hb, const void* w4, int64_t R, int64_t N, int64_t H, float q_scale, void* bias,
                    int64_t bias_pitch, void* q, void* k, void* v, void* gate, int* status_dev, void* stream);

/* out = weighted * sigmoid(gate), elementwise over n bf16 elements (n a multiple of 8; all three
 * pointers 16-byte aligned; out may be weighted).  Stands in for the SigmoidFwdTPP + MulTPP pair
 * behind the attention core in the reference's fused blocks
 * (src/csrc/dot_product_attention.cpp:339-345 and :522-528). */
int af3k_sigmoid_gate(const void* weighted, const void* gate, void* out, int64_t n, void* stream);

/* Self-test of the bounded wait: launches one block that waits, with the given limit, on a
 * barrier nothing ever arrives at, and writes AF3K_STATUS_WAIT_TIMEOUT to status_dev when the
 * wait gives up.  No counterpart in the reference (it has no device code). */
int af3k_selftest_wait_timeout(long long limit_cycles, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AF3K_H_ */
