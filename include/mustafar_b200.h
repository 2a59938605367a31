/*
 * mustafar_b200 -- C ABI of the B200 (sm_100a) sparse KV-cache hot path.
 *
 * Plain pointers and sizes only; every pointer named "device" must point into
 * memory reachable from the current CUDA device.  All entry points are
 * asynchronous on `stream` (a cudaStream_t passed as void*), never allocate
 * device memory and return an `mfar_status` (0 = ok) for host-side argument
 * errors or a failed launch.  Device-side problems (capacity overflow, a bounded
 * wait that gave up) are reported through the optional `dev_status` word.
 *
 * Each function names the reference interface (Haozon/mustafar, path inside
 * that project) it replaces.
 *
 * Fixed by the format: head_dim D = 128, a "tile" = 64 logical elements with
 * one 64-bit bitmap (bit 63-i = element i), a "block" = 64 tokens = 128 tiles.
 */
#ifndef MUSTAFAR_B200_H_
#define MUSTAFAR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MFAR_HEAD_DIM 128
#define MFAR_TILE 64
#define MFAR_BLOCK_TOKENS 64
#define MFAR_TILES_PER_BLOCK 128

typedef enum {
    MFAR_OK = 0,
    MFAR_ERR_ARG = 1,          /* bad size / null pointer / unsupported shape     */
    MFAR_ERR_ALIGN = 2,        /* pointer or stride not aligned as documented     */
    MFAR_ERR_WORKSPACE = 3,    /* scratch / workspace too small                   */
    MFAR_ERR_LAUNCH = 4,       /* cudaGetLastError() != success after a launch    */
    MFAR_ERR_DEVICE = 5,       /* dev_status non-zero (see MFAR_DEV_* bits)       */
    MFAR_ERR_LIMIT = 6         /* size beyond a fixed limit of the entry point    */
} mfar_status;

/* bits OR-ed into *dev_status by kernels */
#define MFAR_DEV_CAPACITY 1u   /* packed values would not fit nz_capacity         */
#define MFAR_DEV_TIMEOUT 2u    /* a bounded wait gave up (look-back or mbarrier)  */
#define MFAR_DEV_BADMETA 4u    /* offsets in the cache are inconsistent           */

enum { MFAR_KIND_KEY = 0, MFAR_KIND_VALUE = 1 };

int mfar_version(void);
const char* mfar_status_string(int status);

/* ------------------------------------------------------------------------- *
 * Compression: fused per-token magnitude prune + bitmap/packed-value encoding.
 *
 * Replaces  kernel/compression.py:249-342  convert_key_batched   (kind = KEY)
 *           kernel/compression.py:344-435  convert_value_batched (kind = VALUE)
 *  and, when prune_rank > 0, the pruning in front of them,
 *           models/llama_mustafar_kernel.py:194-232 / :236-274 (dh_prune_key/value):
 *           thr = prune_rank-th SMALLEST |x| of the 128 channels of a token,
 *           keep |x| >= thr (ties kept).  prune_rank = 0: input is taken as is.
 *
 * x            device, fp16, element (h, t, c) at x[h*x_head_stride + t*x_token_stride + c];
 *              strides in elements, multiples of 8; x 16-byte aligned.  heads_per_group > 0
 *              addresses a two-level layout instead: head h = (g, j), g = h / heads_per_group,
 *              at x[g*x_group_stride + j*x_head_stride + ...] - e.g. the [batch, token, kv head, 128]
 *              output of a fused q|k|v projection read in place (group = sequence).
 * n_tokens     multiple of 64.  Tiles are appended at tile index tile_start
 *              (= tokens already in the cache * 2); tile_start = 0 starts a cache.
 * bitmaps      device int64, head h at bitmaps + h*bmp_head_stride.
 * accum        device int32 prefix of padded counts in uint32 units
 *              (reference `accum_counts`), head h at accum + h*acc_head_stride,
 *              entry tile_start must already hold the head's current tail when
 *              tile_start > 0; entry 0 is written as 0 when tile_start == 0.
 * nz           device fp16 packed values; head h starts at
 *              nz + 8*nz_offset[h] halves (nz_offset device int32, uint4 units,
 *              the reference's NZ_Offset) or, when nz_offset is NULL, at
 *              nz + h*nz_head_stride halves (multiple of 8).
 * nz_capacity  halves available per head (bounds check; a 64-token block that would not fit
 *              sets MFAR_DEV_CAPACITY and its values are dropped: bitmaps and accum are
 *              still written and later blocks carry on, so the cache is unusable and the
 *              caller has to look at dev_status).
 * scratch      device, mfar_compress_scratch_bytes() bytes, 16-byte aligned;
 *              cleared by this call (no need to pre-zero).
 * dev_status   device uint32 or NULL.
 * max_block_halves  device uint32 or NULL: atomicMax'ed with the packed halves of
 *              every block written (a safe `stage_halves` for the decode calls).
 * ------------------------------------------------------------------------- */
size_t mfar_compress_scratch_bytes(int n_heads, int n_tokens);

int mfar_compress_fp16(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                       int heads_per_group, int64_t x_group_stride,
                       int n_heads, int n_tokens, int kind, int prune_rank,
                       int64_t* bitmaps, int64_t bmp_head_stride,
                       int32_t* accum, int64_t acc_head_stride, int64_t tile_start,
                       void* nz, const int32_t* nz_offset, int64_t nz_head_stride,
                       int64_t nz_capacity,
                       void* scratch, size_t scratch_bytes,
                       uint32_t* dev_status, uint32_t* max_block_halves, void* stream);

/* Gathers the packed values of all heads of an arena back to back: head h (at nz + h*nz_head_stride, length
 * 2 * accum[h*acc_head_stride + n_tiles] halves) goes behind the heads before it in `out` (out_capacity halves; a
 * head that would not fit is skipped).  Replaces the per-head `.item()` + `clone()` loop and the model's
 * `torch.cat` of the per-head buffers (kernel/compression.py:334-338, models/llama_mustafar_kernel.py:395).
 * nz, out 16-byte aligned. */
int mfar_compact_heads_fp16(const void* nz, int64_t nz_head_stride, const int32_t* accum, int64_t acc_head_stride,
                            int64_t n_tiles, int n_heads, void* out, int64_t out_capacity, void* stream);

/* The same compression for callers that cannot provide a scratch buffer because they may not
 * allocate device memory while running (a server that hands out all GPU memory from its own arena at
 * start-up, a plugin inside another runtime's budget).  No counterpart in the reference.
 * The look-back scratch is a fixed array inside the library (64 KiB + 16 B per GPU, held until the
 * process exits), which limits one call to n_heads * (n_tokens / 64) <= MFAR_NOALLOC_MAX_BLOCKS;
 * larger jobs return MFAR_ERR_LIMIT without launching.  Calls on one device share that array: each call
 * clears what it uses, but calls that could overlap on the GPU race and must be ordered by the caller.
 * The first call on a device resolves the array's address; issue it before any stream capture. */
#define MFAR_NOALLOC_MAX_BLOCKS 8192
int mfar_compress_fp16_noalloc(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                               int n_heads, int n_tokens, int kind, int prune_rank,
                               int64_t* bitmaps, int64_t bmp_head_stride,
                               int32_t* accum, int64_t acc_head_stride, int64_t tile_start,
                               void* nz, const int32_t* nz_offset, int64_t nz_head_stride,
                               int64_t nz_capacity, uint32_t* dev_status, uint32_t* max_block_halves,
                               void* stream);

/* Prune only (writes x * (|x| >= thr) with the reference's signed zeros).
 * Replaces models/llama_mustafar_kernel.py:194-232.  In place allowed (y == x). */
int mfar_prune_fp16(const void* x, void* y, int64_t n_rows, int64_t row_stride,
                    int prune_rank, void* stream);

/* ------------------------------------------------------------------------- *
 * Quantised compression: prune + bitmap + per-group asymmetric `bits`-bit codes.
 *
 * Replaces  kernel_quant/compression_quant.py:159-264  convert_key_batched_quant   (kind = KEY)
 *           kernel_quant/compression_quant.py:425-529  convert_value_batched_quant (kind = VALUE)
 * with bits = 2, group = 64 (bit-exact: scale = (max-min)/3 and zero = floor(-min/scale+0.5) in
 * fp32, stored fp16; codes from the stored fp16 parameters with IEEE division).  bits = 4 and
 * group = 32 (a fresh scale/zero every 32 nonzeros of a tile) have no reference counterpart.
 *
 * x, strides, heads_per_group, n_tokens, kind, prune_rank, bitmaps, tile_start: as mfar_compress_fp16.
 * tile_offsets/counts/units  device int32, head h at + h*meta_head_stride (counts, units may be NULL);
 *              tile_offsets[t] = uint32 offset of tile t in the flat `packed` buffer.
 * scales/zeros device fp16, (64/group) entries per tile: index (h*meta_head_stride + t)*(64/group) + g.
 * packed       device uint32 codes, 32/bits per word, least significant first.
 *   packed_head_stride == 0 : compact, heads back to back from offset 0 (the reference's
 *              layout); packed_capacity = words available in total; head_tail (NULL or device
 *              int32[n_heads]) receives the end offset of every head.
 *   packed_head_stride  > 0 : arena, head h owns [h*stride, h*stride + packed_capacity);
 *              head_tail[h] (required) = words already used, updated by the call.
 * scratch      mfar_compress_scratch_bytes() bytes, cleared by the call.
 * ------------------------------------------------------------------------- */
int mfar_compress_quant(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                        int heads_per_group, int64_t x_group_stride, int n_heads,
                        int n_tokens, int kind, int prune_rank, int bits, int group,
                        int64_t* bitmaps, int64_t bmp_head_stride, int32_t* tile_offsets,
                        int32_t* counts, int32_t* units, void* scales, void* zeros,
                        int64_t meta_head_stride, int64_t tile_start, int32_t* packed,
                        int64_t packed_head_stride, int64_t packed_capacity, int32_t* head_tail,
                        void* scratch, size_t scratch_bytes, uint32_t* dev_status, void* stream);

/* ------------------------------------------------------------------------- *
 * Decode over the fp16 compressed cache.  Common arguments:
 *
 * q             device fp16, query of q-head i at q + i*q_stride (128 halves), 4-byte aligned, q_stride even;
 *               q-head i uses kv head i / group  (kernel/csrc/SpMM_Kernel.cuh:258-265).
 * n_kv_heads    B * Hkv;  group = Hq / Hkv in {1, 2, 4, 8}.
 * bitmaps/accum/nz/nz_offset/..._head_stride   the cache as written by
 *               mfar_compress_fp16 (bmp_head_stride even; bitmaps and nz 16-byte
 *               aligned); n_tokens = compressed tokens, multiple of 64.
 * nz_extent     halves addressable from nz (the whole buffer, all heads), or 0 when unknown.  The
 *               kernels check every 64-token block's packed range before copying it: start and
 *               size 16-byte aligned, size within the stage, end within nz_extent; a block that
 *               fails sets MFAR_DEV_BADMETA and its values are not read (no fault).
 * stage_halves  upper bound on the packed halves of any 64-token block of one
 *               tensor (sizes the shared-memory ring); 0 = worst case 8192.  A
 *               block larger than the bound sets MFAR_DEV_BADMETA.
 * ------------------------------------------------------------------------- */

/* Split count and workspace size the decode entry points will use.  The first 64 KiB of a workspace are arrival
 * counters of the fused attention (one per kv head; the split records of every entry point start behind them):
 * they must be ZERO before the first call that uses the buffer; every call leaves them zero again (also after a
 * bounded wait gave up).  Calls that could overlap on the GPU need workspaces of their own. */
int mfar_decode_plan(int n_kv_heads, int n_tokens, int window, int nsplit_hint, int* nsplit_out,
                     size_t* workspace_bytes, int group);

/* Fused decode attention: softmax(q.[K~;Kwin]^T * softmax_scale).[V~;Vwin] for one
 * query token per q-head, fp32 accumulation, fp16 result out[i*out_stride + c].
 * Replaces the whole decode-step sequence models/llama_mustafar_kernel.py:394-438
 * (key op, window matmul, softmax, value op, window matmul, add) in one call.
 * k_window/v_window: dense fp16 [n_kv_heads][window][128] with the given strides
 * (elements, multiples of 8); window may be 0.  workspace: mfar_decode_plan bytes.
 * window_len_dev: NULL, or a device int32 holding the current window length (<= window, which is then the
 * capacity): lets a launch captured in a CUDA graph be replayed while the window grows.
 * nsplit 0 = automatic.  One kernel launch: the CTA that finishes a kv head last merges its split records. */
int mfar_decode_attention_fp16(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride, int64_t k_nz_extent,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride, int64_t v_nz_extent,
    int n_tokens, const void* k_window, const void* v_window, int64_t win_head_stride, int64_t win_token_stride,
    int window, const int32_t* window_len_dev, float softmax_scale, void* out, int64_t out_stride, void* workspace,
    size_t workspace_bytes, int nsplit, int stage_halves, uint32_t* dev_status, void* stream);

/* scores[i*scores_stride + t] = sum_c K~[i/group][t][c] * q[i][c]  (fp32 accumulate, fp16 store).
 * Replaces mustafar_key_formulation -> Key_SplitK_API -> Key_Kernel
 * (kernel/kernel_wrapper/mustafar_wrapper.cu:19-133, kernel/csrc/SpMM_API.cu:179-240,
 *  kernel/csrc/SpMM_Kernel.cuh:240-520); only row 0 of the reference's 8-row output is real. */
int mfar_key_scores_fp16(const void* q, int64_t q_stride, int n_kv_heads, int group,
                         const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                         int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                         int64_t nz_head_stride, int64_t nz_extent, int n_tokens, void* scores,
                         int64_t scores_stride, int stage_halves, uint32_t* dev_status, void* stream);

/* out[i*out_stride + c] = sum_t V~[i/group][t][c] * probs[i*probs_stride + t].
 * Replaces mustafar_value_formulation -> Value_SplitK_API -> Value_Kernel (+SplitK_Reduction)
 * (kernel/kernel_wrapper/mustafar_wrapper.cu:139-263, kernel/csrc/SpMM_API.cu:331-400,
 *  kernel/csrc/SpMM_Kernel.cuh:535-796, kernel/csrc/Reduction_Kernel.cuh:26-48). */
int mfar_value_output_fp16(const void* probs, int64_t probs_stride, int n_kv_heads, int group,
                           const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                           int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                           int64_t nz_head_stride, int64_t nz_extent, int n_tokens, void* out,
                           int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit,
                           int stage_halves, uint32_t* dev_status, void* stream);

/* ------------------------------------------------------------------------- *
 * Decode over the quantised cache written by mfar_compress_quant (bits in {2,4},
 * qgroup in {64, 32}); dequantisation is fused into the SpMV.  The two single-product entries keep
 * (code - zero) * scale in fp32 (no fp16 rounding of the dequantised value, which the reference applies: the
 * outputs differ by less than 5e-4 relative L2, a test bounds it); the fused attention entry rounds like the reference.
 * Arguments as their fp16 counterparts; tile_offsets / scales / zeros share
 * meta_head_stride (tiles per head), packed_words bounds every access to `packed`.
 * ------------------------------------------------------------------------- */

/* Replaces mustafar_key_formulation_quant[_meta] -> Key_SplitK_API_Quant -> Key_Kernel_Quant
 * (kernel_quant/kernel_wrapper/mustafar_wrapper_quant.cu:14-215, kernel_quant/csrc/SpMM_API_Quant.cu:263-340,
 *  kernel_quant/csrc/SpMM_Kernel_Quant.cuh:273-503). */
int mfar_key_scores_quant(const void* q, int64_t q_stride, int n_kv_heads, int group,
                          const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* tile_offsets,
                          const void* scales, const void* zeros, int64_t meta_head_stride,
                          const int32_t* packed, int64_t packed_words, int n_tokens, int bits, int qgroup,
                          void* scores, int64_t scores_stride, uint32_t* dev_status, void* stream);

/* Replaces mustafar_value_formulation_quant and ..._decode_n1 -> Value_SplitK_API_Quant -> Value_Kernel_Quant
 * (kernel_quant/kernel_wrapper/mustafar_wrapper_quant.cu:217-457, kernel_quant/csrc/SpMM_API_Quant.cu:342-573,
 *  kernel_quant/csrc/SpMM_Kernel_Quant.cuh:510-735).  workspace: the 64 KiB of counters described at mfar_decode_plan
 *  (left untouched) + n_kv_heads * splits * group * 132 floats, splits <= max(1, n_tokens / 128) unless nsplit is given. */
int mfar_value_output_quant(const void* probs, int64_t probs_stride, int n_kv_heads, int group,
                            const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* tile_offsets,
                            const void* scales, const void* zeros, int64_t meta_head_stride,
                            const int32_t* packed, int64_t packed_words, int n_tokens, int bits, int qgroup,
                            void* out, int64_t out_stride, void* workspace, size_t workspace_bytes,
                            int nsplit, uint32_t* dev_status, void* stream);

/* Fused decode attention over the quantised cache + dense fp16 window (the quantised model's decode step,
 * models/llama_mustafar_quant_kernel.py:426-662, in one call and one launch).  Every dequantised value is
 * fp16((code - zero) * scale) with the subtraction and the product in fp32, the reference's default arithmetic
 * (kernel_quant/csrc/SpMM_Kernel_Quant.cuh:235-240); the products with q / p accumulate in fp32.
 * n_tokens_dev / window_len_dev: NULL, or device int32 holding the current compressed length (a multiple of 64,
 * at most n_tokens, which then sizes the grid) / window length (at most window), read when the kernel runs, so that a
 * captured launch can be replayed while the cache grows.  workspace as mfar_decode_plan. */
int mfar_decode_attention_quant(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, const int32_t* k_tile_offsets, const void* k_scales, const void* k_zeros,
    const int32_t* k_packed, int64_t k_packed_words,
    const int64_t* v_bitmaps, const int32_t* v_tile_offsets, const void* v_scales, const void* v_zeros,
    const int32_t* v_packed, int64_t v_packed_words,
    int64_t bmp_head_stride, int64_t meta_head_stride, int n_tokens, const int32_t* n_tokens_dev, int bits, int qgroup,
    const void* k_window, const void* v_window, int64_t win_head_stride, int64_t win_token_stride, int window,
    const int32_t* window_len_dev, float softmax_scale, void* out, int64_t out_stride, void* workspace,
    size_t workspace_bytes, int nsplit, uint32_t* dev_status, void* stream);

/* mfar_decode_attention_fp16 for callers that replay a captured launch while the cache grows: the number of
 * compressed tokens is read from n_tokens_dev (int32 on the device, a multiple of 64) when the kernel runs;
 * max_tokens (a multiple of 64) bounds it and sizes the grid, the plan (mfar_decode_plan with max_tokens) and
 * the workspace.  stage_halves must cover the largest 64-token block that will ever be appended
 * (64 * kept values per token + 7 * 128 of padding is enough unless tokens have more than three ties at the
 * pruning threshold; a larger block sets MFAR_DEV_BADMETA when it is decoded).  No reference counterpart (the reference re-launches with host-side lengths,
 * models/llama_mustafar_kernel.py:391-438). */
int mfar_decode_attention_fp16_dyn(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride, int64_t k_nz_extent,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride, int64_t v_nz_extent,
    int max_tokens, const int32_t* n_tokens_dev, const void* k_window, const void* v_window, int64_t win_head_stride,
    int64_t win_token_stride, int window, const int32_t* window_len_dev, float softmax_scale, void* out,
    int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit, int stage_halves,
    uint32_t* dev_status, void* stream);

/* ---- decode-step glue (no counterpart in the reference's extensions: its model file does these with torch ops) ----
 * Three small fused kernels for the one-token decode step around the sparse attention, so that a layer is a
 * handful of launches.  All tensors fp16, contiguous rows; rounding follows the torch expressions they replace
 * (each elementwise op in fp32, rounded to fp16 once; RMS statistics in fp32). */

/* x[r] += delta[r] (skipped when delta is NULL), then out[r] = fp16(x[r] * rsqrt(mean(x[r]^2) + eps)) * weight:
 * the residual add and the RMSNorm that follows it (HF LlamaRMSNorm as called at models/llama_mustafar_kernel.py:744,760).
 * hidden % 8 == 0, pointers 16-byte aligned. */
int mfar_add_rmsnorm_f16(void* x, const void* delta, const void* weight, void* out, int64_t rows, int hidden,
                         float eps, void* stream);

/* qkv [batch, n_q_heads + 2*n_kv_heads, 128]: the fused q|k|v projection of one new token per sequence.
 * Rotary embedding (rotate-half, inv_freq[64] fp32, cos/sin rounded to fp16) on q and k
 * (models/llama_mustafar_kernel.py:373-374); q goes to q_out [batch*n_q_heads, 128]; k and v go into the dense
 * windows [batch*n_kv_heads][slot] (the torch.cat of :391 and :430 without the copy).  Position and slot are read from
 * pos_dev / slot_dev (int32 on the device) when those are not NULL, so that a captured CUDA graph can be replayed
 * while they advance; else from pos / slot.  window_capacity = token slots per window head: a slot outside
 * [0, window_capacity) writes nothing to the windows and sets MFAR_DEV_BADMETA in *dev_status (device uint32 or NULL).
 * prune_rank > 0 selects per-step pruning: the same launch prunes in place (rule of mfar_prune_fp16) the window token
 * at slot - prune_back - 1 of every K and V head, i.e. the token that has just left the prune_back most recent ones
 * (what the reference's torch path does at the end of every decode step,
 * models/llama_mustafar_Kt_Mag_Vt_Mag.py:917-926, :1015-1024); windows 16-byte aligned, strides multiples of 8. */
int mfar_rope_append_f16(const void* qkv, const float* inv_freq, const int32_t* pos_dev, int pos,
                         const int32_t* slot_dev, int slot, int batch, int n_q_heads, int n_kv_heads,
                         void* q_out, void* k_window, void* v_window, int64_t win_head_stride,
                         int64_t win_token_stride, int window_capacity, int prune_rank, int prune_back,
                         uint32_t* dev_status, void* stream);

/* out[r, j] = fp16(silu(gate_up[r, j])) * gate_up[r, width + j], gate_up [rows, 2*width] (HF LlamaMLP). */
int mfar_silu_mul_f16(const void* gate_up, void* out, int64_t rows, int width, void* stream);

/* One-shot all-reduce over peer-mapped buffers fused with the residual add and the RMSNorm behind it, for the
 * tensor-parallel decode step (no counterpart in the reference, which has no distributed code; replaces an NCCL
 * all-reduce + mfar_add_rmsnorm_f16):  x[r] += sum over ranks of partial_rank[r];  out[r] = rmsnorm(x[r]) * weight.
 * Every rank calls it with the same arguments but its own `rank`.
 * partials[world]  HOST array of device pointers: each rank's partial [rows, hidden] fp16 for THIS call, as mapped
 *                  into this process (CUDA IPC or any peer mapping; partials[rank] is local).  Callers alternate
 *                  between two buffers from call to call.
 * flags[world]     HOST array of device pointers: each rank's flag array (8 uint32, zero at start-up).
 * epoch of a call = step * calls_per_step + call + 1, step read from step_dev (device int32) when not NULL; it must
 *                  grow from call to call, the same on every rank.
 * wait_ns          bound on the wait for the peers' flags; when it runs out MFAR_DEV_TIMEOUT is set in *dev_status and
 *                  x / out are left untouched.  Plain loads and stores over NVLink only: no TMA, no multicast. */
int mfar_peer_reduce_add_rmsnorm_f16(void* x, const void* const* partials, void* const* flags, int world, int rank,
                                     const int32_t* step_dev, int step, int calls_per_step, int call,
                                     const void* weight, void* out, int64_t rows, int hidden, float eps,
                                     int64_t wait_ns, uint32_t* dev_status, void* stream);

/* Arg-max over a vocabulary split across the ranks (vocabulary-parallel lm_head of the tensor-parallel step; no
 * counterpart in the reference): logits [rows, n_local] fp16 are this rank's slice, columns vocab_offset.. of the whole
 * vocabulary; n_local a multiple of 8, rows 16-byte aligned.  Two launches: the row-wise local arg-max into
 * pairs[rank] (8 bytes per row: float value, int32 global index), then the exchange - announce, bounded wait on the
 * flags (same flag arrays and epoch rule as mfar_peer_reduce_add_rmsnorm_f16, of whose calls this one takes a `call`
 * index of its own), read all ranks' pairs - which writes tokens[rows] (int64): the largest value, the smallest index
 * among equal values, identical on every rank.  pairs[world]: HOST array of device pointers, one pair buffer per rank
 * as mapped into this process.  A wait that runs out sets MFAR_DEV_TIMEOUT and leaves tokens untouched. */
int mfar_peer_argmax_f16(const void* logits, int64_t row_stride, int64_t rows, int n_local, int vocab_offset,
                         void* const* pairs, void* const* flags, int world, int rank, const int32_t* step_dev,
                         int step, int calls_per_step, int call, int64_t* tokens, int64_t wait_ns,
                         uint32_t* dev_status, void* stream);

/* Set-up of the buffers mfar_peer_reduce_add_rmsnorm_f16 reads across GPUs (one-off, not on the hot path).
 * mfar_peer_alloc: cudaMalloc of `bytes` zeroed bytes on the current device, *ptr = the allocation, handle64 (64 host
 *                  bytes) = its CUDA IPC handle, to be sent to the other ranks' processes by any host channel.
 * mfar_peer_open:  maps a peer's handle with THIS process's GPU current, so that its kernels can read and write the
 *                  memory over NVLink (a mapping opened with the owner's device current is only good for copies).
 * mfar_peer_close / mfar_peer_free undo the two; close every mapping before its owner frees the allocation. */
int mfar_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int mfar_peer_open(const void* handle64, void** ptr);
int mfar_peer_close(void* ptr);
int mfar_peer_free(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* MUSTAFAR_B200_H_ */
