/*
 * llnvfp4 - C ABI of the B200 (sm_100a) NVFP4 inference path.
 *
 * Every entry point takes plain device pointers, extents and a CUDA stream handle, returns
 * 0 on success or a negative LLNV_E_* code, never throws and never aborts.  After a failure
 * llnv_last_error() returns a thread-local, human readable message.  The caller owns and
 * allocates every buffer; unless an entry point says otherwise the library allocates nothing.
 *
 * Each declaration cites the interface of the reference implementation (NVlabs/LongLive,
 * paths relative to its repository root) that it stands in for.
 */
#ifndef LLNVFP4_H_
#define LLNVFP4_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* llnv_stream_t; /* a cudaStream_t */

enum {
  LLNV_OK = 0,
  LLNV_E_INVALID = -1,   /* bad argument: null pointer, shape, alignment, unsupported option */
  LLNV_E_CUDA = -2,      /* a CUDA runtime / driver call failed */
  LLNV_E_TIMEOUT = -3,   /* a bounded device-side wait gave up (reported by llnv_check_status) */
  LLNV_E_UNSUPPORTED = -4
};

/* Scale-selection rule ids; same numbering as ScaleRule.cuda_id() in
 * fouroversix/src/fouroversix/utils.py:113-122. */
enum {
  LLNV_RULE_STATIC_6 = 0,
  LLNV_RULE_STATIC_4 = 1,
  LLNV_RULE_MAE = 2,
  LLNV_RULE_MSE = 3,
  LLNV_RULE_ABS_MAX = 4
};

/* Output element type codes; same numbering as utils/kernel/kv_dequant.py:18-25. */
enum { LLNV_DTYPE_BF16 = 0, LLNV_DTYPE_FP16 = 1, LLNV_DTYPE_FP32 = 2 };

/* Which of the reference's dequantize roundings to follow (they can differ in the last bit):
 *  FUSED   (v*s) * (amax * fp32(1/(e2m1_max*e4m3_max)))   utils/kernel/kv_dequant_cuda.cu:95-101,216
 *  PYTORCH ((v*s) * amax) / (e2m1_max*e4m3_max)           fouroversix/src/fouroversix/quantize/quantized_tensor.py:187-209
 *  TRITON  (v*s) * (amax / (e2m1_max*e4m3_max))           utils/quant.py:756-766 */
enum { LLNV_DEQ_FUSED = 0, LLNV_DEQ_PYTORCH = 1, LLNV_DEQ_TRITON = 2 };

int llnv_version(void);
const char* llnv_last_error(void);

/* One-time set-up for the current device: allocates the 16-byte device status word (the only device
 * memory the library itself owns besides the fixed scratch array of llnv_adaln_quantize_nvfp4_static).
 * Every entry point does this lazily on its first use on a device; call it at start-up when the first
 * use could otherwise fall inside a stream capture, where an allocation is not allowed. */
int llnv_init_device(void);

/* Reads and clears the device-side status word that kernels with bounded waits write when a
 * wait gives up.  Synchronises `stream`.  Returns LLNV_OK or LLNV_E_TIMEOUT. */
int llnv_check_status(llnv_stream_t stream);

/* max|x| of a bf16 matrix [M, K] with row stride ldx (elements) into *amax (device fp32).
 * Stands in for the tensor-amax half of fp4_quant_prologue_kernel
 * (fouroversix/src/fouroversix/csrc/include/fp4_quant_kernel.h:31-229).  *amax is overwritten. */
int llnv_amax_bf16(const void* x, int64_t M, int64_t K, int64_t ldx, float* amax, llnv_stream_t stream);

/* bf16 [M, K] -> NVFP4.  Stands in for torch.ops.fouroversix.quantize_to_fp4 with
 * is_nvfp4=1, is_rtn=1, no RHT, 1-D blocks, no transpose
 * (fouroversix/src/fouroversix/csrc/bindings.cpp:28, csrc/quantize/fp4_quant.cu:99-239);
 * results follow the reference's PyTorch quantizer bit for bit
 * (fouroversix/src/fouroversix/quantize/pytorch/reference.py:242-368).
 *   K % 64 == 0.  Mp = M rounded up to 128.
 *   codes: uint8 [Mp, K/2], low nibble = even column.  Rows M..Mp-1 are written as zeros.
 *   sf:    e4m3 bytes, Mp*K/16 of them, in the 128x4 swizzled layout
 *          (fouroversix/src/fouroversix/quantize/utils.py:88-96).
 *   amax:  device fp32 scalar.  amax_given == 0: computed here (overwritten);
 *          amax_given == 1: read as the tensor scale (reference.py:244 `x_amax`).
 *   rule:  LLNV_RULE_*. */
int llnv_quantize_nvfp4(const void* x, int64_t M, int64_t K, int64_t ldx, int rule,
                        void* codes, void* sf, float* amax, int amax_given, llnv_stream_t stream);

/* The same quantizer reading a column-sharded activation: x is [shards][M][K / shards] (row stride
 * ldx inside a shard, shards M * ldx elements apart), which is how the head -> token exchange of
 * sequence parallelism delivers the attention output (ulysses_head_to_seq,
 * wan_5b/distributed/sp_ulysses_inference.py:139-154, then permutes it into [M, K]; here the
 * quantizer reads the received layout directly).  Codes and scales are those of the [M, K] matrix.
 * shards = 1 is llnv_quantize_nvfp4. */
int llnv_quantize_nvfp4_ex(const void* x, int64_t M, int64_t K, int64_t ldx, int rule,
                           void* codes, void* sf, float* amax, int amax_given, int shards, llnv_stream_t stream);

/* Two tensors of the same shape and row stride in one launch, each with its own outputs and tensor
 * scale: the K and the V block of a KV-cache write (wan_5b/modules/causal_model.py:1420-1470 quantizes
 * them one after the other). */
int llnv_quantize_nvfp4_pair(const void* x0, const void* x1, int64_t M, int64_t K, int64_t ldx, int rule, void* codes0,
                             void* sf0, float* amax0, void* codes1, void* sf1, float* amax1, int amax_given,
                             llnv_stream_t stream);

/* adaLN modulation fused into the quantizer: y = LayerNorm(x) (no affine, eps) -> bf16 ->
 * * bf16(1 + scale[f]) -> bf16 -> + shift[f] -> bf16, f = row / frame_rows, then y is quantized as by
 * llnv_quantize_nvfp4 (amax computed here).  Stands in for adaln_modulate_triton
 * (utils/adaln_triton.py:36-126; call sites wan_5b/modules/causal_model.py:867-873, 908-914)
 * followed by the activation quantize of the next Linear
 * (fouroversix/src/fouroversix/model/modules/linear.py:45-46); y itself is written only when
 * y_out != NULL.  With codes == NULL and sf == NULL only y is produced (the modulated LayerNorm in front of a
 * bf16 Linear: CausalHead.forward, wan_5b/modules/causal_model.py:950-959).
 *   x: bf16 [M, C], C % 64 == 0, C <= 4096.  scale/shift: bf16 [frames, mod_stride].
 *   add_one: 1 -> multiply by (1 + scale) (adaln_triton.py:74-78), 0 -> by scale.
 *   row_stats: caller-provided scratch of 2*M floats (mean and 1/std of every row). */
int llnv_adaln_quantize_nvfp4(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                              int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes,
                              void* sf, float* amax, void* y_out, int64_t ldy, float* row_stats, llnv_stream_t stream);

/* Extended forms for token-sharded (sequence-parallel) use: `row_offset` is added to the row index
 * before the frame lookup, and `phase` splits the call so that the tensor amax can be max-reduced
 * across ranks in between: 0 = everything, 1 = row statistics + amax only, 2 = quantize only
 * (reads amax and row_stats as phase 1 left them). */
int llnv_adaln_quantize_nvfp4_ex(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                                 int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes,
                                 void* sf, float* amax, void* y_out, int64_t ldy, float* row_stats, int64_t row_offset,
                                 int phase, llnv_stream_t stream);
int llnv_layernorm_quantize_nvfp4_ex(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight, const void* bias,
                                     float eps, int rule, void* codes, void* sf, float* amax, void* y_out, int64_t ldy,
                                     float* row_stats, int phase, llnv_stream_t stream);

/* Same operation and results as llnv_adaln_quantize_nvfp4 for callers that cannot allocate device
 * memory where they call it (a server that owns all device memory through its own arena, a
 * latency-critical loop that must not take cudaMalloc's device-wide synchronisation).  It has no
 * counterpart in the reference.  The row-statistics scratch is a fixed array inside the library
 * image, so the call performs no cudaMalloc / cudaFree and uses no allocating library routine;
 * inputs and outputs are still the caller's buffers.
 *   - M must not exceed llnv_static_max_rows() (16384 rows, 128 KiB per GPU, held until exit);
 *     larger M fails with LLNV_E_INVALID and a message naming the limit.
 *   - All calls on a GPU share the array and it keeps the previous call's contents; nothing in it
 *     needs to start at zero.  Calls that can overlap on the same GPU race: issue them on one stream.
 *   - The array's device address is looked up on every call and never cached, so the entry point keeps
 *     working after cudaDeviceReset() or a rebuilt primary context (the contents are lost then, which is
 *     harmless).  The first call on a device may load the library's device code: make it at start-up,
 *     before any stream capture begins. */
int llnv_adaln_quantize_nvfp4_static(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale,
                                     const void* shift, int64_t mod_stride, int frame_rows, float eps, int add_one,
                                     int rule, void* codes, void* sf, float* amax, void* y_out, int64_t ldy,
                                     llnv_stream_t stream);
int64_t llnv_static_max_rows(void);

/* LayerNorm with affine weight/bias (bf16 [C]) fused into the quantizer: y = bf16(LN(x)*w + b).
 * Stands in for the cross-attention input norm (`norm3`, wan_5b/modules/causal_model.py:817-819, 906;
 * wan_5b/modules/model.py:101-111) followed by the quantize of cross_attn.q.  Same buffers as above. */
int llnv_layernorm_quantize_nvfp4(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight, const void* bias,
                                  float eps, int rule, void* codes, void* sf, float* amax, void* y_out, int64_t ldy,
                                  float* row_stats, llnv_stream_t stream);

/* Q / K prologue of the chunk attention: RMSNorm over all C channels (weight != NULL), 3-D RoPE on
 * interleaved pairs of every 128-channel head (cos/sin != NULL, fp32 [S, 64] per token), and
 * optionally the smoothed copy `out - mean over the head` plus max|out|.
 * Stands in for WanRMSNorm (wan_5b/modules/model.py:82-98; call site
 * wan_5b/modules/causal_model.py:363-365), rope_apply_triton (utils/rope_triton.py:94-135; call
 * site causal_model.py:479-486) and k_smooth (utils/quant.py:797-798; call sites
 * causal_model.py:568, 631).  x, out, out_smooth: bf16 [S, C] with row strides ldx/ldo/lds;
 * amax_out: fp32 scalar that is overwritten (the tensor scale for the KV-cache write of `out`). */
int llnv_rmsnorm_rope(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                      const float* cos, const float* sin, void* out, int64_t ldo, void* out_smooth, int64_t lds,
                      float* amax_out, llnv_stream_t stream);

/* The same prologue writing head-sharded outputs: out and out_smooth are [shards][S][C / shards]
 * (row strides ldo / lds inside a shard, shards S * ldo / S * lds elements apart), the send layout
 * of the token -> head exchange (ulysses_seq_to_head, sp_ulysses_inference.py:122-137), so that no
 * pack copy is needed before the all-to-all.  shards = 1 is llnv_rmsnorm_rope. */
int llnv_rmsnorm_rope_ex(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                         const float* cos, const float* sin, void* out, int64_t ldo, void* out_smooth, int64_t lds,
                         float* amax_out, int shards, llnv_stream_t stream);

/* The same prologue with one base pointer per head shard (shard r of out / out_smooth is a
 * [S, C / shards] matrix at out_ptrs[r] / smooth_ptrs[r] with row stride ldo / lds).  The pointers
 * may address other GPUs of the node (peer-mapped symmetric memory): the kernel stores every shard
 * at its final place on the rank that owns those heads, which is the token -> head all-to-all of
 * sequence parallelism (ulysses_seq_to_head, sp_ulysses_inference.py:122-137) fused into the
 * producer.  Follow it with llnv_peer_barrier before the consumers run.  smooth_ptrs may be NULL. */
int llnv_rmsnorm_rope_scatter(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                              const float* cos, const float* sin, void* const* out_ptrs, int64_t ldo,
                              void* const* smooth_ptrs, int64_t lds, float* amax_out, int shards, llnv_stream_t stream);

/* The q and the k prologue of one block in a single launch (they share tokens, channels and rotary
 * tables; causal_model.py:363-365, 479-486, 568): q gets RMSNorm(wq) + RoPE, k gets RMSNorm(wk) +
 * RoPE plus, optionally, the smoothed copy and its amax.  Outputs are pointer tables as in
 * llnv_rmsnorm_rope_scatter (one entry per head shard; shards = 1 for plain [S, C] outputs). */
int llnv_rmsnorm_rope_qk(const void* xq, int64_t ldxq, const void* wq, void* const* q_ptrs, int64_t ldq, const void* xk,
                         int64_t ldxk, const void* wk, void* const* k_ptrs, int64_t ldk, void* const* k_smooth_ptrs,
                         int64_t lds, float* k_amax, int64_t S, int64_t C, float eps, const float* cos, const float* sin,
                         int shards, llnv_stream_t stream);

/* Pushes a matrix to `shards` destinations with plain 16-byte stores (the destinations may be peer
 * memory): destination r receives `rows` rows of `row_bytes` bytes read from
 * src + r * src_shard_bytes with row pitch src_pitch, written with row pitch dst_pitch.
 * Column blocks (src_shard_bytes = row_bytes) give the token -> head exchange of a [tokens, C]
 * matrix, row blocks (src_shard_bytes = rows * src_pitch) the head -> token exchange
 * (ulysses_head_to_seq, sp_ulysses_inference.py:139-154). */
int llnv_scatter_2d(const void* src, int64_t src_shard_bytes, int64_t src_pitch, void* const* dst_ptrs, int64_t dst_pitch,
                    int64_t rows, int64_t row_bytes, int shards, llnv_stream_t stream);

/* Barrier over the `world` GPUs of a sequence-parallel group, on the stream: signal_ptrs[r] is rank
 * r's signal area (>= 4 * world bytes of zero-initialised symmetric memory, peer-mapped), epoch a
 * zero-initialised device uint32 of this rank.  Everything enqueued before the barrier on every
 * rank (peer stores included) is visible to everything enqueued after it on every rank.  The wait
 * is bounded; a rank that gives up records LLNV_E_TIMEOUT for llnv_check_status and returns. */
int llnv_peer_barrier(void* const* signal_ptrs, int rank, int world, void* epoch, llnv_stream_t stream);

/* Number of polls after which llnv_peer_barrier / llnv_peer_allreduce_max give up (process-wide, read at
 * launch; 0 restores the default of about four million polls, a few seconds).  Returns the previous
 * value.  After a timeout the kernel returns normally, llnv_check_status reports LLNV_E_TIMEOUT and
 * whatever the consumers of that barrier read is undefined. */
int llnv_set_peer_poll_limit(unsigned int max_polls);

/* MAX all-reduce of n <= 32 device floats over the group, in place, fused with that barrier (same
 * signal areas and epoch; counts as one barrier).  slot_ptrs[r] is rank r's slot area: 2 * 8 * 32
 * floats of symmetric memory.  Used for the per-tensor amax values of the quantizers, so that a
 * sequence-parallel group produces the codes and scales of the single-GPU run. */
int llnv_peer_allreduce_max(float* vals, int n, void* const* slot_ptrs, void* const* signal_ptrs, int rank, int world,
                            void* epoch, llnv_stream_t stream);

/* Quantizers of a sequence-parallel group that reduce their tensor amax themselves.  Bit-identity with the single-GPU
 * run needs the MAX of every tensor amax over the ranks before the first block is quantized.  These forms take this
 * rank's amax in *amax (llnv_quantize_nvfp4_group: written by the producer's epilogue; the adaLN / LayerNorm forms
 * compute it in their statistics pass) and do the exchange inside the quantize kernel - its first CTA publishes the
 * value into every rank's slot area and raises this rank's flag, one thread of every CTA waits (bounded by
 * llnv_set_peer_poll_limit) for all flags and takes the maximum - instead of a separate all-reduce launch in front
 * of it.  On return *amax holds the group maximum.  slot_ptrs / signal_ptrs / rank / world as in
 * llnv_peer_allreduce_max; epoch points to TWO zero-initialised device uint32 of this rank (the epoch that
 * llnv_peer_barrier and llnv_peer_allreduce_max also use, and a counter of finished CTAs).  Every call counts as one
 * barrier of the group's sequence, so all ranks must issue the same sequence of barrier / all-reduce / group calls.
 * M must be positive on every rank.  A wait that gives up records LLNV_E_TIMEOUT for llnv_check_status. */
int llnv_quantize_nvfp4_group(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf, float* amax,
                              int shards, const void* const* slot_ptrs, const void* const* signal_ptrs, int rank, int world,
                              void* epoch, llnv_stream_t stream);
int llnv_adaln_quantize_nvfp4_group(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                                    int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes, void* sf,
                                    float* amax, float* row_stats, int64_t row_offset, const void* const* slot_ptrs,
                                    const void* const* signal_ptrs, int rank, int world, void* epoch, llnv_stream_t stream);
int llnv_layernorm_quantize_nvfp4_group(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight, const void* bias,
                                        float eps, int rule, void* codes, void* sf, float* amax, float* row_stats,
                                        const void* const* slot_ptrs, const void* const* signal_ptrs, int rank, int world,
                                        void* epoch, llnv_stream_t stream);

/* Dequantize `num_blocks` KV-cache blocks, each an NVFP4 matrix [rows_padded, 128] holding
 * block_token_size*num_heads logical rows (token-major, head-minor), into one contiguous
 * tensor [1, num_blocks*block_token_size, num_heads, 128] of dtype_code.
 * Stands in for torch.ops.longlive_kernels.dequantize_kv_cache_fp4
 * (utils/kernel/kv_dequant.cpp:14, utils/kernel/kv_dequant_cuda.cu:148-244).
 * codes/sf/amax are HOST arrays of `num_blocks` DEVICE pointers (passed to the kernel as
 * launch parameters: no pointer-table upload, no synchronisation). */
int llnv_kv_dequant(const void* const* codes, const void* const* sf, const float* const* amax,
                    int num_blocks, int num_heads, int block_token_size, int dtype_code,
                    float e2m1_max, float e4m3_max, int rounding, void* out, llnv_stream_t stream);

/* General NVFP4 -> bf16/fp16/fp32 matrix dequantize ([rows, cols] logical, codes [rows_padded, cols_padded/2]).
 * Stands in for QuantizedTensor.dequantize (fouroversix/src/fouroversix/quantize/quantized_tensor.py:184-214). */
int llnv_dequantize_nvfp4(const void* codes, const void* sf, const float* amax, int64_t rows, int64_t cols,
                          int64_t cols_padded, int dtype_code, float e2m1_max, float e4m3_max, int rounding,
                          void* out, int64_t ldo, llnv_stream_t stream);

/* Non-causal attention of a query chunk over a key/value window: out[q,h,:] =
 * softmax_k(q[q,h,:].k[k,h,:] * scale) v[k,h,:], head_dim 128, bf16 tensors laid out
 * [tokens, heads*128] with row strides ldq/ldk/ldv/ldo (elements), fp32 softmax, bf16 P.V on
 * tcgen05 tensor cores.  Stands in for attention() -> flash_attn_varlen_func as called on the
 * sink + local window (wan_5b/modules/attention.py:241-254, 260-290; call site
 * wan_5b/modules/causal_model.py:781) and on the text context (causal_model.py:197-295).
 * The window is one contiguous K and one contiguous V tensor: dequantized cache blocks followed by
 * the current chunk (llnv_kv_dequant and llnv_rmsnorm_rope / the V GEMM write straight into it). */
int llnv_attention_bf16(const void* q, int64_t Lq, int64_t ldq, const void* k, const void* v, int64_t Lk,
                        int64_t ldk, int64_t ldv, int heads, float scale, void* out, int64_t ldo,
                        llnv_stream_t stream);

/* The same attention with the key window split over `key_splits` CTAs per (256-query tile, head),
 * for calls whose tiles alone cannot fill the device: a head shard of a sequence-parallel rank
 * (wan_5b/distributed/sp_ulysses_inference.py:122-154 leaves heads / P heads per rank) has only
 * ceil(Lq / 256) * heads / P tiles.  Every split attends to a contiguous range of 128-key tiles
 * and writes unnormalised fp32 partial outputs plus (row maximum, row sum) to `workspace`; a
 * second small kernel merges them.  key_splits = 1 is llnv_attention_bf16 (no workspace).
 * out_amax (optional, device fp32) receives max |out| over the written elements: the tensor scale
 * of the quantizer that follows (utils/quant.py quantize_to_fp4 on the attention output) without
 * a separate reduction pass.
 * key_splits = LLNV_ATTN_SPLIT_TAIL balances the other case, more tiles than SMs with a last partial
 * wave (264 tiles on 148 SMs run two waves with 32 SMs idle in the second): the tiles of the last wave
 * are each cut once, into a long and a short CTA sized so that the short ones fill the SMs the long
 * ones leave free, and only those tiles go through the workspace (sized as for 2 splits) and the merge
 * kernel.  Where it would save under 5 % it runs as key_splits = 1.  Partial results are merged in fp32, so
 * a split or balanced call agrees with key_splits = 1 to fp32 rounding of the softmax sums, not bit for bit.
 * llnv_attention_key_splits() proposes a value for the current device (1 when the tiles fill it evenly,
 * LLNV_ATTN_SPLIT_TAIL or a count otherwise); llnv_attention_workspace_bytes() is the workspace for it. */
enum { LLNV_ATTN_SPLIT_TAIL = -1 };
int llnv_attention_bf16_ex(const void* q, int64_t Lq, int64_t ldq, const void* k, const void* v, int64_t Lk,
                           int64_t ldk, int64_t ldv, int heads, float scale, void* out, int64_t ldo,
                           int key_splits, void* workspace, int64_t workspace_bytes, float* out_amax,
                           llnv_stream_t stream);
int llnv_attention_key_splits(int64_t Lq, int64_t Lk, int heads);

/* The chunk attention reading the NVFP4 KV cache directly: the window is `num_blocks` cached blocks
 * (oldest first; block b holds block_token_size tokens x heads rows of 128 channels, token-major /
 * head-minor, as an NVFP4 matrix [rows_padded, 128] with swizzled scales and one fp32 amax) followed by
 * the current chunk in bf16 (k_cur / v_cur: [L_cur, heads*128], row strides ldk / ldv; L_cur may be 0).
 * Stands in for the reference's dequantize-every-block-then-attend sequence: dequantize_kv_cache on all
 * max_blocks blocks of K and of V (utils/quant.py:731-768, utils/kernel/kv_dequant_cuda.cu:59-107; call
 * sites wan_5b/modules/causal_model.py:557-600, 628-652), window assembly with torch.cat (:673-724) and
 * attention() (:781, wan_5b/modules/attention.py:241-254).  Here the cached keys and values are decoded
 * inside the attention kernel's load stage, with the rounding of the fused dequantize kernel
 * (LLNV_DEQ_FUSED), so no bf16 copy of the cache exists and the result equals llnv_kv_dequant followed
 * by llnv_attention_bf16_ex on the concatenated window bit for bit.
 *   k_codes / k_sf / k_amax / v_*: HOST arrays of num_blocks (<= 16) DEVICE pointers, passed to the kernel
 *   as launch parameters.  Codes must be 16-byte aligned, block_token_size >= 128 (a 128-key tile then
 *   touches at most two blocks) and heads * 64 a multiple of 16.  num_blocks == 0 is llnv_attention_bf16_ex on
 *   the current chunk.  key_splits / workspace / out_amax as in llnv_attention_bf16_ex, with
 *   Lk = num_blocks * block_token_size + L_cur. */
int llnv_attention_nvfp4kv(const void* q, int64_t Lq, int64_t ldq, const void* const* k_codes, const void* const* k_sf,
                           const float* const* k_amax, const void* const* v_codes, const void* const* v_sf,
                           const float* const* v_amax, int num_blocks, int block_token_size, float e2m1_max,
                           float e4m3_max, const void* k_cur, const void* v_cur, int64_t L_cur, int64_t ldk, int64_t ldv,
                           int heads, float scale, void* out, int64_t ldo, int key_splits, void* workspace,
                           int64_t workspace_bytes, float* out_amax, llnv_stream_t stream);
int64_t llnv_attention_workspace_bytes(int64_t Lq, int heads, int key_splits);

/* Fused epilogue of the W4A4 GEMM.  All pointers are device pointers and optional (NULL = skip).
 * With everything NULL/0 the GEMM writes bf16(alpha * acc), which is what the reference's
 * CUTLASS kernel produces.  The chain follows the reference's rounding points
 * (fouroversix/src/fouroversix/model/modules/linear.py:73-74, wan_5b/modules/causal_model.py:889,919):
 *   y  = bf16(alpha * acc)
 *   y  = bf16(y + bias[n])                         if bias
 *   y  = bf16(gelu_tanh(y))                        if act == 1
 *   y  = bf16(residual[m,n] + bf16(y * gate[f,n])) if residual (gate NULL -> y added as is),
 *        f = (m + row_offset) / frame_rows
 *   out_amax = max(out_amax, |y|)                  if out_amax (atomic, caller zeroes it)
 *   (q_codes, q_sf) = quantize_nvfp4(y, amax = *q_amax)   if q_codes: the NVFP4 form of y, so that the Linear that
 *        consumes y needs no separate quantize pass (the reference quantizes the input of every Linear in its own
 *        kernels, fouroversix/src/fouroversix/model/modules/linear.py:45-46, and its GEMM has no epilogue at all,
 *        fouroversix/src/fouroversix/csrc/fp4_gemm.cu:64-86).  The tensor amax must be known before the GEMM runs
 *        (the reference's quantizer accepts a given amax: quantize/pytorch/reference.py:244, 262); codes and scales
 *        are then bit for bit those of llnv_quantize_nvfp4(y, amax_given = 1).  Rule: LLNV_RULE_MSE.  Not combinable
 *        with residual.  With q_codes set, d may be NULL: the bf16 result is then not written at all.
 */
typedef struct {
  const float* alpha;     /* device scalar; NULL -> amax_a*amax_b/(6*Ea*6*Eb) from the rules */
  const void* bias;       /* bf16 [N] */
  int32_t act;            /* 0 none, 1 GELU(tanh) */
  const void* residual;   /* bf16 [M, ldr] */
  int64_t ldr;
  const void* gate;       /* bf16 [frames, gate_stride] */
  int64_t gate_stride;
  int32_t frame_rows;     /* rows per frame for the gate lookup */
  float* out_amax;        /* fp32 scalar, atomic max of |out| */
  int32_t row_offset;     /* added to m before the gate's frame lookup (token shards) */
  void* q_codes;          /* uint8 [Mp, N/2], Mp = M rounded up to 128 (rows M..Mp-1 are written as zeros) */
  void* q_sf;             /* e4m3 bytes, Mp*N/16, 128x4 swizzled */
  const float* q_amax;    /* device fp32: the tensor amax the codes are scaled with (read, not computed) */
  int32_t q_rule;         /* LLNV_RULE_MSE */
} llnv_epilogue_t;

/* D[M, N] = epilogue(alpha * A[M, K] * B[N, K]^T), A and B NVFP4 (codes [rows_padded, K/2],
 * swizzled e4m3 scales), fp32 accumulation on tcgen05 block-scaled tensor cores, bf16 output
 * with row stride ldd.  Stands in for
 * torch.ops.fouroversix.gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt
 * (fouroversix/src/fouroversix/csrc/bindings.cpp:31, csrc/fp4_gemm.cu:40-154) together with the
 * alpha computation of fouroversix/src/fouroversix/matmul/cutlass/backend.py:81-90.
 *   M: logical rows written (A holds ceil(M/128)*128 rows); N % 128 == 0; K % 256 == 0. */
int llnv_gemm_nvfp4(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule,
                    const void* b_codes, const void* b_sf, const float* b_amax, int b_rule,
                    int64_t M, int64_t N, int64_t K, const llnv_epilogue_t* epilogue,
                    void* d, int64_t ldd, llnv_stream_t stream);

/* llnv_gemm_nvfp4 with the tiling chosen by the caller instead of by shape (all tilings give the same
 * bits: same products, same accumulation order along K): LLNV_GEMM_TILE_AUTO, 128 / 192 / 256 = one
 * CTA per 128 x tile output tile (a width that does not divide N falls back to the automatic choice),
 * LLNV_GEMM_TILE_PAIR = one 256 x 256 tile per pair of SMs (cta_group::2; needs N % 256 == 0).  The
 * reference fixes one CUTLASS tile shape at compile time (fouroversix/src/fouroversix/csrc/fp4_gemm.cu:67-84). */
enum { LLNV_GEMM_TILE_AUTO = 0, LLNV_GEMM_TILE_PAIR = 2 };
int llnv_gemm_nvfp4_ex(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule,
                       const void* b_codes, const void* b_sf, const float* b_amax, int b_rule,
                       int64_t M, int64_t N, int64_t K, const llnv_epilogue_t* epilogue,
                       void* d, int64_t ldd, int tile, llnv_stream_t stream);

/* Entry points that produce a tensor amax normally overwrite it: the call clears the scalar with a 4-byte memset before
 * its kernels max-accumulate into it.  A caller that runs hundreds of such calls per step can clear all its scalars with
 * ONE fill and switch the per-call memsets off.  llnv_set_amax_accumulate(mask) (per calling thread; returns the previous
 * mask; default 0): bit 1 = llnv_attention_bf16_ex / llnv_attention_nvfp4kv (out_amax) and the adaLN / LayerNorm
 * quantizers (amax, phases 0 and 1); bit 2 = llnv_gemm_nvfp4_grouped (out_amax[]) and llnv_rmsnorm_rope* (amax_out).
 * With a bit set those entry points accumulate into whatever the scalar holds: the caller clears every scalar before
 * the first call that writes it and does not let two producers share one without a clear in between.  A 30-layer
 * chunk of five forwards saves about 1200 memset and fill nodes this way (about 3 % of its time on a B200).
 * llnv_gemm_nvfp4's epilogue out_amax is never cleared by the library in either mode (see llnv_epilogue_t);
 * llnv_amax_bf16 and llnv_quantize_nvfp4 (amax_given = 0) always clear theirs. */
int llnv_set_amax_accumulate(int on);

/* llnv_quantize_nvfp4 for fp16 input (x: IEEE half, row stride ldx elements): the reference's CUDA backend takes fp16
 * activations beside bf16 (fouroversix/src/fouroversix/quantize/cuda/backend.py:45-51, csrc/quantize/fp4_quant.cu:205-227).
 * Same outputs, layouts and bit-exactness against the reference's PyTorch quantizer on the values widened to fp32; every
 * block is evaluated with the reference's fp32 arithmetic one operation at a time (no packed fast path), so it is the
 * slower of the two.  The DiT path is bf16 throughout. */
int llnv_quantize_nvfp4_f16(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf,
                            float* amax, int amax_given, llnv_stream_t stream);

/* Measurement aid, not part of the reference's interface: one CTA per SM issues k_blocks x 4 block-scaled FP4
 * MMAs (128 x 256 x 64, the GEMM's instruction shape) on operands that stay in shared memory, with no loads,
 * scale refills or epilogue.  *flop_out (may be NULL) receives the flop of the launch; time the launch with
 * events on `stream`: flop / time is the tensor-core rate a W4A4 main loop can at most reach on this device,
 * the denominator the GEMM's tensor roofline is quoted against. */
int llnv_fp4_mma_rate(int k_blocks, double* flop_out, llnv_stream_t stream);

/* Two or three Linears that share their input in one launch: B is the concatenation along N of
 * `groups` weight matrices of N_each rows (codes and swizzled scales concatenated, b_amax one fp32
 * per matrix), matrix g is written to d[g] (row stride ldd[g]) and, if out_amax[g] is not NULL, its
 * output amax to out_amax[g] (overwritten).  The q, k and v projections of a block
 * (wan_5b/modules/causal_model.py:363-366) are such a group: one grid of 3x the tiles fills the SMs
 * better than three grids, and two launches are saved.  The epilogue may carry bias (N_each * groups
 * values, concatenated) and act; residual / gate / alpha / out_amax belong to llnv_gemm_nvfp4. */
int llnv_gemm_nvfp4_grouped(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule, const void* b_codes,
                            const void* b_sf, const float* b_amax, int b_rule, int64_t M, int64_t N_each, int64_t K, int groups,
                            const llnv_epilogue_t* epilogue, void* const* d, const int64_t* ldd, float* const* out_amax,
                            llnv_stream_t stream);

/* ---- bf16 Linear of the unquantized edge layers ------------------------------------------------ */

/* d[M, N] = act(a[M, K] . w[N, K]^T + bias), bf16 in and out, fp32 accumulation on tcgen05
 * (kind::f16): torch.nn.functional.linear for the layers the reference's NVFP4 filter leaves in
 * bf16 -- patch embedding (the Conv3d of wan_5b/modules/causal_model.py:1052-1056 applied to
 * patchified tokens), text_embedding, time_embedding, time_projection (:1057-1066) and head.head
 * (wan_5b/modules/model.py Head, called at causal_model.py:1648-1651).  bias (N values) may be NULL.
 * act: 0 none, 1 GELU(tanh), 2 SiLU, applied to the bf16-rounded sum as the reference's separate
 * activation module does.  lda / ldw / ldd: row strides in elements.  K, N and the strides must be
 * multiples of 8; a, w, d 16-byte aligned. */
int llnv_linear_bf16(const void* a, int64_t lda, const void* w, int64_t ldw, const void* bias, int act, int64_t M, int64_t N,
                     int64_t K, void* d, int64_t ldd, llnv_stream_t stream);

/* ---- latent <-> token layout ----------------------------------------------------------------- */

/* bf16 latent [C, F, 2h, 2w] (element strides stride_c and stride_f, image axes contiguous) to
 * tokens [F*h*w, 4*C] with features ordered (c, kh, kw) -- the view of the input the patch-embedding
 * Conv3d with kernel and stride (1, 2, 2) takes (wan_5b/modules/causal_model.py:1052-1056, 1535-1540) --
 * and back, which is the reference's unpatchify (causal_model.py:1835-1858) for a head whose rows
 * are stored in that feature order.  ldt: token row stride in elements.  h, w: token grid. */
int llnv_patchify(const void* latent, int64_t stride_c, int64_t stride_f, void* tokens, int64_t ldt, int C, int F, int h, int w,
                  llnv_stream_t stream);
int llnv_unpatchify(const void* tokens, int64_t ldt, void* latent, int64_t stride_c, int64_t stride_f, int C, int F, int h, int w,
                    llnv_stream_t stream);

/* ---- flow-matching UniPC scheduler step ------------------------------------------------------ */

/* Scalars of one scheduler step, computed on the host in fp32 exactly as the reference computes
 * them as 0-dim tensors (wan_5b/utils/fm_solvers_unipc.py:407-455 for the predictor, :550-605 for
 * the corrector): with sigma_t / sigma_s0 the sigmas the update goes to / starts from,
 * lambda = log(1 - sigma) - log(sigma), h = lambda_t - lambda_s0,
 *   c1 = sigma_t / sigma_s0, c2 = (1 - sigma_t) * expm1(-h), c3 = (1 - sigma_t) * B(h) with B(h) = expm1(-h),
 *   inv_rk = 1 / r_1 (r_1 = (lambda_older - lambda_s0) / h, order 2 only),
 *   rho: the UniC weights (0.5 for order 1, the 2 x 2 solve for order 2), already rounded to the
 *   latents' dtype; the UniP weight of order 2 is the constant 0.5.
 * p_zero is c3 * 0 of the predictor (the term an order-1 predictor subtracts; it is -0 or +0). */
typedef struct {
  float sigma;               /* sigma of this step: x0 = sample - sigma * model_output (:320-323) */
  int use_corrector;         /* 0 on the first step (:689-693) */
  int corrector_order;       /* 1 or 2: the order the previous step's predictor used */
  float cc1, cc2, cc3, c_inv_rk, c_rho0, c_rho1;
  int predictor_order;       /* 1 or 2 (:714-722) */
  float pc1, pc2, pc3, p_inv_rk, p_zero;
} llnv_unipc_coef;

/* scheduler.step of FlowUniPCMultistepScheduler (wan_5b/utils/fm_solvers_unipc.py:657-741, called
 * once per denoising step by the chunk loop, pipeline/causal_diffusion_inference.py:604-609) for
 * solver order <= 2, `bh2`, x0 prediction from a flow prediction, as one elementwise pass over n
 * values of dtype 0 (bf16) or 1 (fp32):
 *   x0_out     = sample - sigma * model_output                    (convert_model_output, :320-323)
 *   sample_out = UniC(last_sample, x0_prev, x0_older, x0_out)     (:599-627) or sample without corrector
 *   next_out   = UniP(sample_out, x0_out, x0_prev)                (:457-485)
 * with every intermediate rounded to the dtype as the reference's PyTorch calls round it on a GPU.
 * x0_prev / x0_older are the x0_out of the previous two steps, last_sample the previous step's
 * sample_out; pointers a step does not need may be NULL.  Outputs may alias inputs (x0_out =
 * x0_older rotates the history in place).  All pointers are device memory. */
int llnv_unipc_step(const void* model_output, const void* sample, const void* x0_prev, const void* x0_older,
                    const void* last_sample, void* x0_out, void* sample_out, void* next_out, int64_t n, int dtype,
                    const llnv_unipc_coef* coef, llnv_stream_t stream);

/* Test / benchmark hooks (no counterpart in the reference). */
/* Number of kernels the library has launched in this process (every launch, captured ones included, is counted
 * when it is issued; a replayed graph is not re-counted). */
unsigned long long llnv_launch_count(void);
/* 1: launch kernels with programmatic stream serialization (the next kernel of a stream is
 * scheduled while the previous one drains and waits for it on the device); 0 (default): plain
 * launches.  Returns the previous setting.  The environment variable LLNV_PDL=1 switches it on at
 * load time.  Results do not depend on it; on a B200 it measured no gain for graph-replayed chunks. */
int llnv_set_pdl(int on);
int llnv_selftest_div_const(int divisor, uint32_t first_bits, uint64_t count, unsigned long long* mismatches,
                            llnv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LLNVFP4_H_ */
