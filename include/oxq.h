/*
 * oxq -- B200 (sm_100a) kernels for oxydLLM's quantized-weight matrix product.
 *
 * C ABI of liboxq.so. Every entry point takes raw DEVICE pointers to the
 * reference's packed layouts (unchanged), explicit sizes, dtype enums and a
 * cudaStream_t passed as void*. The library never allocates or frees caller
 * memory, never synchronises the device and never aborts: it returns an
 * oxq_status and records a message retrievable with oxq_last_error().
 * All work is enqueued on the given stream. Results are deterministic: no
 * floating-point atomics, fixed-order reductions (the reference's
 * bit-reproducibility contract, metal_ops.rs:4562-4625).
 *
 * Each declaration cites the reference interface it stands in for
 * (file:line inside the oxydllm source tree).
 */
#ifndef OXQ_H
#define OXQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    OXQ_OK = 0,
    OXQ_ERR_BAD_SHAPE = -1,   /* a shape/divisibility rule of the reference is violated */
    OXQ_ERR_BAD_ALIGN = -2,   /* a pointer is not aligned as the kernel requires */
    OXQ_ERR_UNSUPPORTED = -3, /* dtype / bits / format combination not implemented */
    OXQ_ERR_NULL = -4,        /* a required pointer is NULL */
    OXQ_ERR_WORKSPACE = -5,   /* workspace missing or too small */
    OXQ_ERR_CUDA = -6,        /* a CUDA runtime/driver call failed */
    OXQ_ERR_DEVICE_FLAG = -7  /* a kernel reported a bounded wait that ran out */
} oxq_status;

/* Element types of activations, scales, biases and outputs. */
typedef enum { OXQ_F32 = 0, OXQ_F16 = 1, OXQ_BF16 = 2 } oxq_dtype;

/* GGML block types, numbered as in GGUF files (candle GgmlDType; linear.rs:199-211). */
typedef enum {
    OXQ_GGML_Q4_0 = 2, OXQ_GGML_Q4_1 = 3, OXQ_GGML_Q5_0 = 6, OXQ_GGML_Q5_1 = 7, OXQ_GGML_Q8_0 = 8,
    OXQ_GGML_Q2_K = 10, OXQ_GGML_Q3_K = 11, OXQ_GGML_Q4_K = 12, OXQ_GGML_Q5_K = 13, OXQ_GGML_Q6_K = 14
} oxq_ggml_type;

const char *oxq_status_string(int status);
/* Message of the last failing call on this thread ("" if none). */
const char *oxq_last_error(void);
int oxq_version(void);

/* ------------------------------------------------------------------ AWQ
 * qweight u32 [k, n/8] (slot s of a word = out column 8j + {0,2,4,6,1,3,5,7}[s]),
 * qzeros u32 [k/g, n/8], scales [k/g, n] of `scales_dtype` (awq.rs:23-24,45-70).
 */

/* dequantize_awq / fill_awq_weight (awq.rs:325-440,612-633):
 * w_out[o][i] = convert((nibble - zero) as f32 * f32(scale)), dense [n, k], bit-exact. */
int oxq_awq_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                    void *w_out, int out_dtype, int k, int n, int group_size, void *stream);

/* PackedQuantLinear::forward, decode and continuous-batching sizes (linear.rs:450-505: the
 * w4a16_matmul / batched-GEMV branch, metal_ops.rs:1821-1867,2326): y[m, n] = x[m, k] . deq(W) (+ bias[n])
 * for 1 <= m <= oxq_decode_max_m() on the tcgen05 tensor cores. The packed words are read once and
 * become one E4M3 byte per weight in shared memory (a nibble q read as E4M3 is q * 2^-9 exactly); each
 * bf16 activation is split into three E5M2 values that add up to it exactly; scale and zero point are
 * applied in f32 once per (out feature, 128-wide k group). Needs n % 32 == 0, k % 128 == 0 and
 * group_size % 128 == 0 (other shapes: oxq_awq_gemv / oxq_awq_gemm). `workspace`: device memory of
 * oxq_decode_workspace_bytes(m, k, n) bytes, 256-byte aligned, zero-filled once before its first use
 * (only the first word, the bounded-wait flag read by oxq_gemm_check, has to start at zero); it
 * holds the token pieces and the partial sums of out-feature tiles shared by several CTAs, and is
 * rewritten by every call, so calls sharing it must be stream-ordered. Deterministic. */
int oxq_decode_max_m(void);
size_t oxq_decode_workspace_bytes(int m, int k, int n);
int oxq_awq_decode_matmul(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                          const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                          int y_dtype, int m, int k, int n, int group_size, void *workspace,
                          size_t workspace_bytes, void *stream);

/* PackedQuantLinear::forward decode branch -> w4a16_matmul (linear.rs:450-480,
 * metal_ops.rs:1821-1867): y[m, n] = x[m, k] . deq(W) (+ bias[n]), 1 <= m <= 32,
 * x bf16, f32 accumulation, y in `y_dtype`. No workspace: the split along k is
 * reduced inside a thread-block cluster. */
int oxq_awq_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                 int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                 int group_size, void *stream);

/* oxq_awq_gemv streams weight boxes into shared memory with the TMA unit and waits for each with a
 * bounded wait. Synchronises `stream`; returns OXQ_ERR_DEVICE_FLAG (once) if such a wait ran out on
 * the current device in any oxq_awq_gemv call since the last check. No counterpart in the reference. */
int oxq_awq_gemv_check(void *stream);

/* Gated FFN projection on a fused AWQ [gate | up] weight (concat_awq_along_out of gate_proj and
 * up_proj, ffn.rs:235-254): y[m, inter] = act(x . W_gate^T) * (x . W_up^T), act = 1 SiLU, 2 GeLU-tanh
 * (FeedForward::forward, ffn.rs:385-470; gated_silu_fused / gated_gelu_tanh_fused, metal_ops.rs:1243-1277).
 * x, y bf16. qweight u32 [k, 2*inter/8], qzeros u32 [k/g, 2*inter/8], scales [k/g, 2*inter].
 * m <= 16 runs the GEMV and a small activation kernel; 17 .. 256 tokens run the kernel that unpacks inside
 * the tensor-core loop (on the shapes oxq_awq_gemm takes it for; the GEMV up to 32 tokens elsewhere) and the
 * same activation kernel; larger m dequantizes the weight with gate row j and up row j side by side and applies the activation in the tensor-core GEMM's epilogue (no
 * [m, 2*inter] round trip). Workspace as for oxq_awq_gemm with n = 2*inter; oxq_gemm_check applies. */
int oxq_awq_ffn_gate_up(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                        int scales_dtype, int activation, void *y, int m, int k, int inter, int group_size,
                        void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------ GPTQ
 * qweight u32 [k/pf, n] sequential LSB-first along k, qzeros u32 [k/g, n/pf]
 * storing zero-1 (NULL or sym != 0: zero = 2^(bits-1) - 1), pf = 32/bits. */

/* dequantize_gptq / fill_gptq_weight (awq.rs:442-590), dense [n, k], bit-exact. */
int oxq_gptq_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                     void *w_out, int out_dtype, int k, int n, int group_size, int bits, int sym, void *stream);

/* ------------------------------------------------------------------ GGUF
 * weight = raw GGML blocks, rows [n] contiguous, blocks along k
 * (metal_ops.rs:5228-5241, linear.rs:220-236). */

/* QTensor::dequantize as restated by the reference's per-element strips
 * (quant_kernels.metal:2342-2384,2438-2482,2518-2554; Q5_0/Q4_1/Q5_1: 2315-2341,2386-2437; Q5_K: block
 * layout 1438-1445), dense [n, k], bit-exact. Types: Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K. */
int oxq_gguf_dequant(int ggml_type, const void *blocks, void *w_out, int out_dtype, int n, int k, void *stream);

/* QLinear::forward (linear.rs:324-393) / gguf_quant_matmul (metal_ops.rs:5819):
 * y[m, n] = x[m, k] . deq(W)^T (+ bias), 1 <= m <= 32, x bf16. */
int oxq_gguf_gemv(int ggml_type, const void *x, int x_dtype, const void *blocks, const void *bias, int bias_dtype,
                  void *y, int y_dtype, int m, int k, int n, void *stream);

/* ------------------------------------------------------------------- FP8
 * weight = E4M3fn bytes [n, k]; scale_inv f32 grid [s_out, s_in] tiling the
 * weight evenly (128x128 blocks: s_out = n/128, s_in = k/128; per-row: s_in = 1;
 * scalar: 1x1; none: NULL) (linear.rs:96-141, weights.rs:207-234). */

/* f8_block_dequant_bf16 / Fp8Linear's dequant (metal_ops.rs:5788, linear.rs:96-141):
 * w_out = convert(f32(e4m3) * scale), bit-exact. */
int oxq_fp8_dequant(const uint8_t *weight, const float *scale_inv, int s_out, int s_in, void *w_out, int out_dtype,
                    int n, int k, void *stream);

/* Fp8Linear::forward (linear.rs:96-145) / f8_gemv (metal_ops.rs:5788-5796), 1 <= m <= 32. */
int oxq_fp8_gemv(const void *x, int x_dtype, const uint8_t *weight, const float *scale_inv, int s_out, int s_in,
                 const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *stream);

/* ----------------------------------------------------------------- MXFP4
 * blocks u8 [n, k/32, 16] two E2M1 codes per byte low nibble first, scales u8
 * [n, k/32] E8M0 (mxfp4.rs:3-6). */

/* dequantize_mxfp4_f32 (mxfp4.rs:35-64), dense [n, k], bit-exact. */
int oxq_mxfp4_dequant(const uint8_t *blocks, const uint8_t *scales, void *w_out, int out_dtype, int n, int k,
                      void *stream);

/* Mxfp4Linear::forward (mxfp4.rs:119-154) / mxfp4_matmul gemv branch
 * (metal_ops.rs:6197-6222), 1 <= m <= 32. */
int oxq_mxfp4_gemv(const void *x, int x_dtype, const uint8_t *blocks, const uint8_t *scales, const void *bias,
                   int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *stream);

/* ------------------------------------------------------------------ GPTQ / W8A16 decode
 * PackedQuantLinear::chunked_batch_gemv for the layouts next to 4-bit AWQ (linear.rs:450-480):
 * gptq_matmul (PackDim::In, bits 4 or 8; metal_ops.rs:1960-2316, quant_kernels.metal:360-545,3501-3648) and
 * w8a16_matmul (PackDim::Out at 8 bits; metal_ops.rs:1835, quant_kernels.metal:3349-3499,3650-3728).
 * y[m, n] = x[m, k] . deq(W) (+ bias[n]), 1 <= m <= 32 (tokens are taken up to four per launch), x bf16,
 * f32 accumulation, on the packed tensors as stored; no workspace; deterministic (fixed-order k split).
 * GPTQ: qweight u32 [k / pf, n], qzeros u32 [k / g, n / pf] or NULL, w = (q - (zero + 1)) * scale, `sym`
 * (or NULL qzeros) = the symmetric zero 2^(bits-1) - 1 (awq.rs:561-590).
 * W8A16: qweight u32 [k, n / 4] (byte c of word j = out column 4 j + c), qzeros u32 [k / g, n / 4],
 * w = (q - zero) * scale (quant_kernels.metal:1-16,40-48). in_features <= 40960. */
int oxq_gptq_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                  int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                  int group_size, int bits, int sym, void *stream);
int oxq_w8a16_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                   int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                   int group_size, void *stream);
/* dequantize_w8 (metal_ops.rs, quant_kernels.metal:335-356): dense [n, k] weight of the 8-bit AWQ layout, bit-exact. */
int oxq_w8a16_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                      void *w_out, int out_dtype, int k, int n, int group_size, void *stream);

/* ------------------------------------------------- prefill-sized matmuls
 * m > 32 (any m >= 1 is accepted): weight rows are dequantized in slabs into
 * `workspace` by the bit-exact kernels above and contracted on the tensor
 * cores (tcgen05, TMEM accumulators, TMA-fed operands), bf16 x bf16 -> f32.
 * `workspace` is caller-owned DEVICE memory, 256-byte aligned, of at least
 * oxq_gemm_workspace_bytes(n, k) bytes; its first word is a flag that a
 * kernel sets if one of its bounded waits ran out. The flag is sticky: no
 * call clears it, it keeps the code of the FIRST wait that ran out in any call
 * on this workspace until oxq_gemm_check reports and clears it. The rest of
 * the 256-byte header holds arrival tickets of the fused kernel's k splits
 * (zero between calls). Fresh workspace memory must start with a zeroed
 * header: allocate it zero-filled or call oxq_gemm_workspace_init once. Calls sharing a workspace must be
 * stream-ordered. The same holds for the workspaces of
 * oxq_awq_decode_matmul and oxq_gptoss_moe_forward. */

size_t oxq_gemm_workspace_bytes(int n, int k);

/* Self-test of the bounded waits (no counterpart in the reference): one thread waits, with a 50 ms limit, on a
 * barrier that nothing arrives on; the wait gives up, stores `code` (> 0) in the flag word of `workspace`
 * and the kernel ends normally, so the next oxq_gemm_check reports OXQ_ERR_DEVICE_FLAG and the workspace
 * stays usable. */
int oxq_selftest_wait_expiry(void *workspace, int code, void *stream);

/* The same through the dense tensor-core GEMM itself (one-CTA kernel for m <= 128, two-CTA kernel above, m <= 256): its
 * TMA producer issues no loads, the MMA issuer's wait for tile data runs out after the regular 2 s limit, every role
 * falls through, tensor memory is freed and the kernel ends with code 2 in the flag word. Operands and output are
 * scratch inside `workspace` (256-byte aligned, at least 1 MiB). */
int oxq_selftest_gemm_wait_expiry(void *workspace, size_t workspace_bytes, int m, void *stream);

/* The same for the grouped kernel of the MoE expert layer (the one that unpacks MXFP4 inside its tensor-core
 * loop): one unit of work whose weight producer never loads, so every other role gives up on its bounded
 * wait (about two seconds), the flag word takes a code, tensor memory is freed and the kernel returns.
 * workspace: at least 1 MiB, 256-byte aligned; oxq_gemm_check(workspace) afterwards returns
 * OXQ_ERR_DEVICE_FLAG once. No counterpart in the reference. */
int oxq_selftest_moe_wait_expiry(void *workspace, size_t workspace_bytes, void *stream);

/* Zeroes the 256-byte header (flag word) of a fresh workspace on `stream`. */
int oxq_gemm_workspace_init(void *workspace, void *stream);

/* Synchronises `stream`, reads the flag word of `workspace`; if a tensor-core
 * kernel gave up on a wait in any call since the last check it clears the
 * flag and returns OXQ_ERR_DEVICE_FLAG (the outputs of those calls are not
 * to be trusted). */
int oxq_gemm_check(const void *workspace, void *stream);

/* PackedQuantLinear::forward beyond the decode GEMV: maybe_mpp_quant_matmul, else
 * dequantize_w4 + matmul (linear.rs:494-524, metal_ops.rs:2771-2797). Up to 256
 * tokens, when n % 128 == 0, k % 128 == 0, group_size is a power of two >= 64 and
 * the scales are f16 or bf16, one kernel unpacks the words into its shared-memory
 * operand and multiplies on tcgen05 (same bf16 weights, no slab written); all
 * other calls dequantize slabs into the workspace. The workspace is required
 * (and its flag word used) either way. */
int oxq_awq_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                 int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                 int group_size, void *workspace, size_t workspace_bytes, void *stream);

/* Tensor-parallel column shard of the same matmul (no counterpart in the reference, which runs on one device; the
 * sharding rule is the column-slice property concat_awq_along_out relies on, awq.rs:256-323). The packed tensors are
 * this rank's columns [col_base, col_base + n_local) of a layer with n_full out features; the result is written into
 * y[:, col_base : col_base + n_local] (y has n_full columns) and then copied by a small kernel of this library, with the
 * same offsets, into the n_peers (<= 7) buffers y_peers[i]: device pointers into the OTHER ranks' output buffers
 * (peer-mapped or symmetric memory), given as a HOST array. Only plain stores cross NVLink; nothing is read from a peer
 * and no tensor map covers peer memory. `bias`, if given, has n_full entries. The column block and the rows of y must
 * be 16-byte aligned. The caller orders the ranks (a barrier after the call before anyone reads y, and before
 * the next call overwrites it). */
int oxq_awq_gemm_tp(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                    int scales_dtype, const void *bias, int bias_dtype, void *y, void *const *y_peers, int n_peers,
                    int y_dtype, int m, int k, int n_local, int col_base, int n_full, int group_size, void *workspace,
                    size_t workspace_bytes, void *stream);

/* Same branch for the 8-bit AWQ layout (dequantize_w8 + matmul, linear.rs:506-508). */
int oxq_w8a16_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                   int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                   int group_size, void *workspace, size_t workspace_bytes, void *stream);

/* Same branch for GPTQ-packed weights (dequantize_gptq_packed + matmul, linear.rs:509-520). 4-bit weights of
 * the shapes named above take the fused unpack + tcgen05 kernel up to 256 tokens (K-major operand: a GPTQ
 * word is eight input rows of one out feature); qzeros, where given, must then be 16-byte aligned. */
int oxq_gptq_gemm(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                  int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                  int group_size, int bits, int sym, void *workspace, size_t workspace_bytes, void *stream);

/* QLinear::forward prefill branch: gguf_quant_mul_mm (linear.rs:268-285, metal_ops.rs:5973). */
int oxq_gguf_gemm(int ggml_type, const void *x, int x_dtype, const void *blocks, const void *bias, int bias_dtype,
                  void *y, int y_dtype, int m, int k, int n, void *workspace, size_t workspace_bytes, void *stream);

/* Fp8Linear::forward for m beyond the GEMV range (linear.rs:96-145). Up to 256 tokens, when n % 128 == 0,
 * k % 128 == 0 and the scale blocks are multiples of 128 rows and 64 columns, the bytes are widened inside the
 * tensor-core kernel (same bf16 weights as the dequantization kernel); otherwise slabs are dequantized. */
int oxq_fp8_gemm(const void *x, int x_dtype, const uint8_t *weight, const float *scale_inv, int s_out, int s_in,
                 const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *workspace,
                 size_t workspace_bytes, void *stream);

/* Mxfp4Linear::forward mul_mm branch (metal_ops.rs:6204-6222). */
int oxq_mxfp4_gemm(const void *x, int x_dtype, const uint8_t *blocks, const uint8_t *scales, const void *bias,
                   int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *workspace, size_t workspace_bytes,
                   void *stream);

/* ------------------------------------------------------- GPT-OSS MoE layer
 * MoeFeedForward::forward for GptOss experts (moe.rs:466-499 routing, 563-607
 * dispatch_sparse, 152-173 expert math; tensor layout of load_gpt_oss,
 * moe.rs:407-434): gu_blocks u8 [E, 2*inter, hidden/32, 16], gu_scales u8
 * [E, 2*inter, hidden/32], gu_bias [E, 2*inter] (gate = even, up = odd rows),
 * dn_blocks u8 [E, hidden, inter/32, 16], dn_scales, dn_bias [E, hidden].
 * router_logits f32 [tokens, E] are the router linear's output. Only experts
 * in [expert_lo, expert_hi) are evaluated (expert parallelism: the outputs of
 * the ranks add up to the full layer); pass 0, E for the whole layer.
 * Everything runs on `stream` without a host round trip. `workspace`: device
 * memory of oxq_gptoss_moe_workspace_bytes(tokens, top_k, expert_hi -
 * expert_lo, hidden, inter) bytes, 256-byte aligned; oxq_gemm_check applies. */
size_t oxq_gptoss_moe_workspace_bytes(int tokens, int top_k, int num_local_experts, int hidden, int inter);
int oxq_gptoss_moe_forward(const void *x, int x_dtype, const float *router_logits, int tokens, int num_experts,
                           int top_k, int norm_topk, int hidden, int inter, const uint8_t *gu_blocks,
                           const uint8_t *gu_scales, const void *gu_bias, const uint8_t *dn_blocks,
                           const uint8_t *dn_scales, const void *dn_bias, int bias_dtype, float limit, int expert_lo,
                           int expert_hi, void *out, int out_dtype, void *workspace, size_t workspace_bytes,
                           void *stream);

/* The owner side of expert parallelism (no counterpart in the reference, which dispatches on one device,
 * moe.rs:563-607): rows that already carry their expert id go through that expert with weight one,
 * out[r] = MoeExpert::GptOss(expert_ids[r]).forward(rows[r]) (moe.rs:152-173). Only experts in
 * [expert_lo, expert_hi) may occur. Workspace: oxq_gptoss_moe_workspace_bytes(n_rows, 1, expert_hi - expert_lo, ...). */
int oxq_gptoss_experts_forward(const void *rows, int x_dtype, const int32_t *expert_ids, int n_rows, int num_experts,
                               int hidden, int inter, const uint8_t *gu_blocks, const uint8_t *gu_scales,
                               const void *gu_bias, const uint8_t *dn_blocks, const uint8_t *dn_scales, const void *dn_bias,
                               int bias_dtype, float limit, int expert_lo, int expert_hi, void *out, int out_dtype,
                               void *workspace, size_t workspace_bytes, void *stream);

/* The combine of dispatch_sparse (moe.rs:593-605: expert outputs times routing weight, added in ascending expert order):
 * out[t] = sum_s top_w[t, s] * rows[pos[t * top_k + s]], rows bf16 [*, hidden], f32 accumulation, one rounding. */
int oxq_moe_combine(const void *rows, const int32_t *top_idx, const float *top_w, const int32_t *pos, int tokens,
                    int top_k, int hidden, int num_experts, void *out, int out_dtype, void *stream);

/* Expert parallelism, sender and owner side bookkeeping on the device (no counterpart in the reference, whose
 * dispatch_sparse, moe.rs:563-607, keeps all experts local): pairs (token, slot) sorted by expert id with the
 * pair order kept inside an expert. counts i32 [num_experts], offsets i32 [num_experts + 1], perm i32 [pairs]
 * (perm[i] = the pair sent i-th), inv i32 [pairs] (inv[pair] = its position; the `pos` of oxq_moe_combine).
 * top_idx i32 [pairs], 16-byte aligned. */
int oxq_moe_dispatch_plan(const int32_t *top_idx, int pairs, int num_experts, int32_t *counts, int32_t *offsets,
                          int32_t *perm, int32_t *inv, void *stream);

/* out[i, :] = x[perm[i] / top_k, :], i < rows: the rows of a dispatch in send order. bf16, hidden % 8 == 0. */
int oxq_moe_gather_rows(const void *x, const int32_t *perm, int rows, int top_k, int hidden, void *out, void *stream);

/* Expert ids of rows received in groups, source rank major and local expert minor: group g holds counts[g] rows
 * of expert lo + g % n_local. counts i32 [groups], ids i32 [sum of counts]. */
int oxq_moe_expand_ids(const int32_t *counts, int groups, int n_local, int lo, int32_t *ids, void *stream);

/* Routing alone: softmax over all experts, top-k (ties: lower index), optional
 * renormalisation (moe.rs:472-487). top_idx i32 [tokens, top_k], top_w f32. */
int oxq_moe_route(const float *router_logits, int tokens, int num_experts, int top_k, int norm_topk, int32_t *top_idx,
                  float *top_w, void *stream);

/* No counterpart in the reference. oxq_awq_gemm for callers that cannot
 * allocate device memory: code running inside a host runtime that owns the
 * only allocator and does not lend it out, a plugin loaded after the process
 * has handed all free memory to a pool, or a call made while allocation is
 * forbidden (for instance between the start and end of a stream capture).
 * The dequantization slab and the flag word live in a fixed 8 MiB (+256 B)
 * device array inside the library image, held by every GPU that loads the
 * library until the process exits. Limits and rules:
 *   - in_features <= oxq_awq_gemm_noalloc_max_k() (16384), otherwise
 *     OXQ_ERR_WORKSPACE is returned and nothing is launched;
 *   - the first call on each device is a set-up step: it looks up the array's
 *     device address (cudaGetSymbolAddress), which under lazy module loading is
 *     also where the driver loads the module and reserves the array; make that
 *     first call outside any stream capture;
 *   - all calls share the one array: the slab is overwritten by each call, the
 *     flag word is sticky until oxq_awq_gemm_noalloc_check reads and clears
 *     it; calls that may overlap on the GPU (different
 *     streams without ordering) race on it and give wrong results;
 *   - it calls no cudaMalloc/cudaFree and no allocating library routine.
 * oxq_awq_gemm_noalloc_check is oxq_gemm_check on that built-in array. */
size_t oxq_awq_gemm_noalloc_max_k(void);
int oxq_awq_gemm_noalloc(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                         const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype,
                         int m, int k, int n, int group_size, void *stream);
int oxq_awq_gemm_noalloc_check(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* OXQ_H */
