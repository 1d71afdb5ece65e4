/*
 * dqmoe.h — C ABI of the B200 (sm_100a) dynamic-quantization MoE layer library.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its kernels
 * on the CUDA stream it is given (a cudaStream_t passed as void*), never
 * synchronises with the host and never allocates device memory: the caller
 * owns all tensors and passes one workspace buffer, exactly as the reference
 * operator does (csrc/pybind11_register.h:99-151).
 *
 * Return value: 0 on success, a DQMOE_ERR_* code otherwise; the message of the
 * last failure on the calling thread is returned by dqmoe_last_error() and has
 * the reference's "[ASSERT FAILED] file:line  Condition: ..." form
 * (csrc/util.h:143-152) for argument checks.
 *
 * Layout conventions (all row-major, innermost dimension contiguous):
 *   a        [T, H]        activations          (e4m3 bytes or bf16)
 *   b        [E, 2I, H]    fc1 weights, rows 0..I-1 of an expert are the gate
 *                          half, rows I..2I-1 the value half
 *   b1       [E, H, I]     fc2 weights
 *   d        [T, k, H]     bf16 output, slot j of token t holds the output of
 *                          expert m_indices[t, j] (unweighted)
 *   m_indices[T, k]        int32 expert ids; an id outside [0, E) drops the row
 * Scale tensors are fp32; their shapes depend on the quantisation mode:
 *   tensor  (256):  a_scale [1],             b_scale [E],                    b1_scale [E]
 *   channel (512):  a_scale [T],             b_scale [E, 2I],                b1_scale [E, H]
 *   block   (1024): a_scale [T, ceil(H/128)], b_scale [E, ceil(2I/128), ceil(H/128)],
 *                   b1_scale [E, ceil(H/128), ceil(I/128)]
 *   MXFP8   (2048): the scale pointers address UE8M0 bytes (value 2^(byte - 127)), not floats:
 *                   a_scale [T, H/32] row-major; b_scale (E * 2I rows, H columns) and b1_scale (E * H rows,
 *                   I columns) in the tiled layout of dqmoe_mx_tile_scales (same byte count as row-major)
 */
#ifndef DQMOE_H_
#define DQMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DQMOE_ABI_VERSION 1

/* error codes */
#define DQMOE_OK 0
#define DQMOE_ERR_INVALID 1   /* argument check failed (shape, alignment, mode) */
#define DQMOE_ERR_CUDA 2      /* a CUDA runtime/driver call failed */
#define DQMOE_ERR_WORKSPACE 3 /* workspace too small or misaligned */
#define DQMOE_ERR_DEVICE 4    /* a kernel's bounded wait gave up (see dqmoe_device_status) */

/* quantisation modes: the reference's QuantMode bit values (csrc/quantization.h:10-28) */
#define DQMOE_QUANT_NONE 0          /* bf16 activations and weights */
#define DQMOE_QUANT_FP8_TENSOR 256  /* FP8_QDQ      : per-tensor act scale, per-expert weight scale */
#define DQMOE_QUANT_FP8_CHANNEL 512 /* FP8_ROWWISE  : per-token act scale, per-output-channel weight scale */
#define DQMOE_QUANT_FP8_BLOCK 1024  /* FP8_BLOCKWISE: 1x128 act scales, 128x128 weight scales */
/* MXFP8: e4m3 with one UE8M0 (power-of-two) scale byte per row and 32 K elements, activations and weights
 * alike; the bit between FP8_BLOCKWISE (1 << 10) and FP4 (1 << 12), which the reference leaves unused
 * (csrc/quantization.h:25-38). Needs H and I to be multiples of 128. */
#define DQMOE_QUANT_FP8_MX 2048
/* NVFP4: e2m1 values, two per byte, with one UE4M3 scale byte per row and 16 K elements and an fp32 global scale
 * per tensor (per expert for the weights): the bit the reference names FP4 / nvfp4() and reserves without a
 * kernel behind it (csrc/quantization.h:30-33, 81-84, 116-119). Served by dqmoe_moe_forward_nvfp4 (the global
 * scales do not fit dqmoe_moe_forward's argument list); dqmoe_moe_workspace_bytes accepts the value. Needs H and
 * I to be multiples of 256. */
#define DQMOE_QUANT_NVFP4 4096

/* router scoring functions */
#define DQMOE_SCORE_SOFTMAX 0 /* softmax over experts, top-k, renormalised to sum 1 */
#define DQMOE_SCORE_SIGMOID 1 /* sigmoid per expert, top-k, normalised by their sum */

typedef void* dqmoe_stream_t; /* a cudaStream_t */

/* Message of the last error raised on the calling thread ("" if none). */
const char* dqmoe_last_error(void);
int dqmoe_abi_version(void);

/*
 * Sticky device status. Kernels that wait on barriers bound every wait; one that
 * gives up writes a code into a host-mapped word instead of trapping. This call
 * synchronises the current device, returns the word through *code (0 = clean)
 * and clears it. No counterpart in the reference, whose CUDA_CHECK exits the
 * process (csrc/util.h:61-80).
 */
int dqmoe_device_status(int* code);

/* ------------------------------------------------------------------ layer */

/*
 * Workspace bytes needed by dqmoe_moe_forward for a problem size.
 * Replaces MoeFCRunner::getWorkspaceSize (csrc/moe_kernels.h:713-722).
 */
size_t dqmoe_moe_workspace_bytes(int T, int H, int I, int E, int k, int quant_mode);

/*
 * One MoE layer: expert sort -> row gather -> grouped fc1 + SwiGLU (+ dynamic
 * FP8 re-quantisation of the intermediate) -> grouped fc2 -> scatter into d.
 * Replaces m_grouped_moe_nt_contiguous<T,W,O> / MoeFCRunner::runMoe
 * (csrc/pybind11_register.h:99-151, csrc/moe_kernels.h:770-892).
 * quant_mode selects the element type: NONE = bf16 data (scale pointers are
 * ignored and may be anything), the FP8 modes = e4m3 data.
 * `fused` is accepted for signature compatibility; the dequantisation is always
 * fused into the GEMM epilogue (csrc/moe_gemm_template.h:1111-1118 selects
 * between two kernels with equal results).
 * workspace must be 256-byte aligned (checked, as pybind11_register.h:141-142)
 * and at least dqmoe_moe_workspace_bytes() long (checked; pass
 * workspace_bytes = 0 to skip the size check as the reference does).
 */
int dqmoe_moe_forward(const void* a, const float* a_scale, const void* b, const float* b_scale,
                      const void* b1, const float* b1_scale, void* d, const int32_t* m_indices,
                      void* workspace, size_t workspace_bytes, int T, int H, int I, int E, int k,
                      int quant_mode, int fused, dqmoe_stream_t stream);

/*
 * The unquantised layer on IEEE half operands: a [T,H], b [E,2I,H], b1 [E,H,I] and
 * d [T,k,H] are fp16, accumulation is fp32, every intermediate rounding is to fp16. The
 * T = half instantiation of the reference's runner (csrc/pybind11_register.h:104-151
 * is templated on the activation type; its Python module exports only the bf16 one). Same
 * workspace size as quant_mode DQMOE_QUANT_NONE.
 */
int dqmoe_moe_forward_f16(const void* a, const void* b, const void* b1, void* d,
                          const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T,
                          int H, int I, int E, int k, dqmoe_stream_t stream);

/*
 * The layer with expert biases: bias1 [E, 2I] and bias2 [E, H], fp32, are added to the dequantised fc1 and
 * fc2 products before their rounding (out = A W^T + bias, as torch's F.linear); either may be NULL. Other
 * arguments as dqmoe_moe_forward / dqmoe_moe_forward_f16. The reference's runner carries expert_bias1 /
 * expert_bias2 and its plugin a use_bias field (csrc/moe_kernels.h:72-78, test/trt_test.py:82-89, :121), but
 * its GEMMs are launched with C = nullptr (csrc/moe_kernels.h:908), so it defines no bias arithmetic.
 */
int dqmoe_moe_forward_bias(const void* a, const float* a_scale, const void* b, const float* b_scale,
                           const void* b1, const float* b1_scale, const float* bias1, const float* bias2,
                           void* d, const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T,
                           int H, int I, int E, int k, int quant_mode, dqmoe_stream_t stream);

/*
 * The layer in the NVFP4 mode: a [T, H/2] packed e2m1 with a_sf [T, H/16] UE4M3 bytes row-major and a_gscale
 * (1 float); b [E, 2I, H/2] and b1 [E, H, I/2] with tiled scale bytes (dqmoe_mx_tile_scales over cols = 2H / 2I)
 * and per-expert global scales [E]; act_gscale (1 float) the global scale the intermediate is re-quantised
 * with (a calibrated constant, as NVFP4 inference stacks keep one per layer); bias1 / bias2 fp32 or NULL; d
 * [T, k, H] bf16. Workspace: dqmoe_moe_workspace_bytes(..., DQMOE_QUANT_NVFP4). No counterpart in the reference.
 */
int dqmoe_moe_forward_nvfp4(const void* a, const uint8_t* a_sf, const float* a_gscale, const void* b, const uint8_t* b_sf,
                            const float* b_gscale, const void* b1, const uint8_t* b1_sf, const float* b1_gscale,
                            const float* act_gscale, const float* bias1, const float* bias2, void* d,
                            const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T, int H, int I, int E,
                            int k, dqmoe_stream_t stream);
int dqmoe_moe_forward_f16_bias(const void* a, const void* b, const void* b1, const float* bias1,
                               const float* bias2, void* d, const int32_t* m_indices, void* workspace,
                               size_t workspace_bytes, int T, int H, int I, int E, int k,
                               dqmoe_stream_t stream);

/*
 * The unquantised layer on fp32 operands: a [T,H], b [E,2I,H], b1 [E,H,I] and d [T,k,H] are fp32, the
 * intermediate stays fp32. The products run on the tensor cores as TF32 (operands read with a 10-bit
 * mantissa, fp32 accumulation), which is also what the reference's T = float instantiation does on its
 * tensor-op GEMM (csrc/moe_gemm_template.h:487-528, README.md:7); results agree with an fp32 reference to
 * about 1e-3 relative, not bit for bit. H and I must be multiples of 4. bias1 / bias2 as above, or NULL.
 */
size_t dqmoe_moe_workspace_bytes_f32(int T, int H, int I, int E, int k);
int dqmoe_moe_forward_f32(const void* a, const void* b, const void* b1, const float* bias1,
                          const float* bias2, void* d, const int32_t* m_indices, void* workspace,
                          size_t workspace_bytes, int T, int H, int I, int E, int k, dqmoe_stream_t stream);

/*
 * Addresses of intermediates inside a workspace laid out by dqmoe_moe_forward
 * for the same problem size (debug/testing aid; the reference has the unused
 * extractIntermediateResultsforTorch, csrc/moe_kernels.h:739-767).
 * which: 0 offsets[E+1] int32, 1 dest_to_src[n] int32, 2 permuted activations,
 *        3 permuted activation scales, 4 intermediate (fc2 input),
 *        5 intermediate scales, 6 counts[E] int32, 7 m-tile prefix[E+1] int32.
 * Returns NULL for an unknown id.
 */
void* dqmoe_moe_workspace_ptr(void* workspace, int which, int T, int H, int I, int E, int k,
                              int quant_mode);

/*
 * The whole MoE block from bf16 activations x [T, H] and fp32 router logits [T, E] to
 * out [T, H] bf16: top-k router, expert sort, gather fused with the dynamic 1x128 FP8
 * quantisation of the activations (block mode) or plain gather (bf16 mode), grouped fc1 +
 * SwiGLU (+ re-quantisation), grouped fc2, weighted combine of the k slots. quant_mode is
 * DQMOE_QUANT_NONE (bf16 weights), DQMOE_QUANT_FP8_BLOCK (e4m3 weights with 128x128
 * scales), or DQMOE_QUANT_FP8_TENSOR / _CHANNEL (x is quantised per tensor / per token
 * into the workspace first, then the layer runs as dqmoe_moe_forward does; weight
 * scales). The natural caller of the reference's layer (its tests do routing and input
 * quantisation in torch, test/torch_test.py:60-80, test/util.py:162-184); no single
 * counterpart in the reference.
 */
size_t dqmoe_moe_block_workspace_bytes(int T, int H, int I, int E, int k, int quant_mode);
int dqmoe_moe_block(const void* x_bf16, const float* logits, const void* b, const float* b_scale,
                    const void* b1, const float* b1_scale, void* out_bf16, void* workspace,
                    size_t workspace_bytes, int T, int H, int I, int E, int k, int scoring,
                    int quant_mode, dqmoe_stream_t stream);

/*
 * The same block with n_shared shared experts (DeepSeek-style: every token also runs
 * through them, weight 1). b / b1 and their scales hold E routed experts followed by the
 * n_shared shared ones (E + n_shared in all, same H and I); logits stay [T, E]. The
 * shared experts occupy k..k+n_shared-1 of each token's slots and go through the same
 * sort, gather, grouped GEMMs and weighted sum. Size the workspace with
 * dqmoe_moe_block_workspace_bytes(T, H, I, E + n_shared, k + n_shared, quant_mode).
 * No counterpart in the reference.
 */
int dqmoe_moe_block_shared(const void* x_bf16, const float* logits, const void* b, const float* b_scale,
                           const void* b1, const float* b1_scale, void* out_bf16, void* workspace,
                           size_t workspace_bytes, int T, int H, int I, int E, int k, int n_shared,
                           int scoring, int quant_mode, dqmoe_stream_t stream);

/* ------------------------------------------------------------------ plugin-shaped front end */

/*
 * The layer behind the interface of the reference's "mixture_of_experts" TensorRT plugin
 * as its test drives it (test/trt_test.py): the nine creation fields (:97-135), the input
 * list in the plugin's order (:140-150) and one output [num_tokens, top_k, hidden]. A
 * TensorRT build wraps these calls in IPluginV2DynamicExt (create -> the creator's
 * createPlugin, workspace_size -> getWorkspaceSize, enqueue -> enqueue, serialize /
 * deserialize -> serialize / deserializePlugin). The plugin's own source is not part of the
 * reference; its kernels are the ones dqmoe_moe_forward replaces.
 *
 * type / output_type use the nvinfer1::DataType codes below. Built: FP8 operands with
 * quant_mode 256 / 512 / 1024 (and the added 2048, whose scale inputs hold UE8M0 bytes: actscale row-major,
 * scale_a / scale_b tiled, see DQMOE_QUANT_FP8_MX) and BF16 operands with quant_mode 0, with outputs BF16
 * (written directly), HALF or FLOAT (converted from the layer's bf16 result through
 * workspace); HALF operands with quant_mode 0 and HALF output (dqmoe_moe_forward_f16);
 * FLOAT operands with quant_mode 0 and FLOAT output (dqmoe_moe_forward_f32).
 * enqueue inputs: 0 input [T,H], 1 weight1 [E,2I,H], 2 weight2 [E,H,I], 3 index [T,k] int32,
 * 4 bias1 [E,2I] fp32, 5 bias2 [E,H] fp32 (read only when use_bias != 0; the reference's test
 * passes weight-shaped dummies with use_bias = 0), 6 actscale, 7 scale_a (fc1 weight scales),
 * 8 scale_b (fc2 weight scales); entries 6-8 are read only for FP8 operands. Scale shapes per
 * mode as listed at the top of this file.
 */
#define DQMOE_DT_FLOAT 0
#define DQMOE_DT_HALF 1
#define DQMOE_DT_FP8 6
#define DQMOE_DT_BF16 7

typedef struct dqmoe_plugin_fields {
    int32_t number_of_experts;
    int32_t top_k;
    int32_t expert_hidden_size;
    int32_t expert_inter_size;
    int32_t max_num_tokens;
    int32_t use_bias;
    int32_t type;
    int32_t output_type;
    int32_t quant_mode;
} dqmoe_plugin_fields;

typedef struct dqmoe_plugin dqmoe_plugin; /* opaque, host memory only */

int dqmoe_plugin_create(const dqmoe_plugin_fields* fields, dqmoe_plugin** out);
void dqmoe_plugin_destroy(dqmoe_plugin* plugin);
int dqmoe_plugin_get_fields(const dqmoe_plugin* plugin, dqmoe_plugin_fields* out);
/* 0 for a null plugin or num_tokens outside [0, max_num_tokens] */
size_t dqmoe_plugin_workspace_size(const dqmoe_plugin* plugin, int num_tokens);
int dqmoe_plugin_enqueue(const dqmoe_plugin* plugin, int num_tokens, const void* const* inputs,
                         void* const* outputs, void* workspace, dqmoe_stream_t stream);
size_t dqmoe_plugin_serialization_size(void);
int dqmoe_plugin_serialize(const dqmoe_plugin* plugin, void* buffer, size_t bytes);
int dqmoe_plugin_deserialize(const void* buffer, size_t bytes, dqmoe_plugin** out);

/* ------------------------------------------------------------------ routing */

/*
 * Top-k router over fp32 logits [T, E]: indices [T, k] int32 in descending score
 * order (ties: lower expert id first), weights [T, k] fp32 normalised to sum 1.
 * The reference has no router kernel; its tests use torch.randn + torch.topk
 * (test/torch_test.py:78-80). E <= 1024, k <= 32.
 * An expert is chosen at most once per token, also when fewer than k logits are above -inf
 * (masked experts then fill the last slots in id order with weight 0 under softmax). A NaN logit is
 * never chosen; a row with fewer than k non-NaN logits gets the id 0x7fffffff in the slots that are
 * left, which the expert sort drops like any id outside [0, E).
 */
int dqmoe_route_topk(const float* logits, int T, int E, int k, int scoring, int32_t* indices,
                     float* weights, dqmoe_stream_t stream);

/*
 * Expert sort of n = T*k expanded rows: counts[E], exclusive offsets[E+1], the
 * permutation dest_to_src[n] (dest row -> t*k+j) and, if not NULL, its inverse
 * src_to_dest[n]. Order inside an expert is ascending source row (stable), which
 * is the order torch.where gives (test/util.py:80). Rows whose id is outside
 * [0, E) are dropped: src_to_dest = -1 and the tail of dest_to_src is -1.
 * Replaces cubHistogramAndScan + GetGroupIndex (csrc/moe_kernels.h:108-127,
 * 452-471), whose atomic slot assignment is not deterministic.
 */
size_t dqmoe_route_sort_workspace_bytes(int n, int E);
int dqmoe_route_sort(const int32_t* expert_ids, int n, int E, int32_t* counts, int32_t* offsets,
                     int32_t* dest_to_src, int32_t* src_to_dest, void* workspace,
                     size_t workspace_bytes, dqmoe_stream_t stream);

/*
 * Expand run lengths: out[r] = values[s] for the counts[s] consecutive rows of segment s
 * (S <= 1024 segments, n rows in all; rows beyond the sum of counts get -1). Used by the
 * expert-parallel layer to label received rows with their local expert id. No counterpart in
 * the reference, which has no multi-GPU path.
 */
int dqmoe_segment_ids(const int32_t* counts, const int32_t* values, int S, int32_t* out, int n,
                      dqmoe_stream_t stream);

/* ------------------------------------------------------------------ permute / finalize */

/*
 * Row gather dst[r, :] = src[dest_to_src[r] / k, :] for r < n (rows with a
 * negative map entry are skipped), row_bytes a multiple of 16; optionally the
 * same gather over an fp32 scale matrix with scale_cols columns (0 = none).
 * Replaces expandInputRowsGatherKernel and expandInputScale{,Block}GatherKernel
 * (csrc/moe_kernels.h:487-576).
 */
int dqmoe_permute_rows(const void* src, size_t row_bytes, int k, const int32_t* dest_to_src, int n,
                       void* dst, const float* src_scale, int scale_cols, float* dst_scale,
                       dqmoe_stream_t stream);

/*
 * Fused gather + dynamic 1x128 FP8 quantisation of bf16 activations:
 * q[r, :], scale[r, :] = quant_1x128(x[dest_to_src[r] / k, :]).
 * The reference quantises in torch (test/util.py:34-45) and gathers afterwards.
 */
int dqmoe_permute_quant_block_1x128(const void* x_bf16, int H, int k, const int32_t* dest_to_src,
                                    int n, void* q, float* scale, dqmoe_stream_t stream);

/*
 * Scatter of permuted rows back to slot order: d[dest_to_src[r], :] = rows[r, :].
 * Replaces finalizeScatterKernel (csrc/moe_kernels.h:581-620).
 */
int dqmoe_finalize_scatter(const void* rows, size_t row_bytes, const int32_t* dest_to_src, int n,
                           void* d, dqmoe_stream_t stream);

/*
 * Weighted combine out[t, :] = sum_j weights[t, j] * d[t, j, :] (bf16 in, fp32
 * accumulate in slot order, bf16 out). Slots whose weight is exactly 0 are not
 * read. No counterpart in the reference (its output stays [T, k, H]).
 */
int dqmoe_finalize_weighted(const void* d_bf16, const float* weights, void* out_bf16, int T, int k,
                            int H, dqmoe_stream_t stream);

/* ------------------------------------------------------------------ quantisers */

/*
 * Dynamic FP8 E4M3 quantisers over bf16 input, bit-exact to the torch
 * expressions of the reference: sf = max(amax, 1e-4) / 448, q = e4m3(x * (1 / sf))
 * with IEEE fp32 division and round-to-nearest-even (test/util.py:18-68).
 */
/* per row of a [rows, cols] matrix: per_token_cast_to_fp8 / per_channel_cast_to_fp8 (test/util.py:18-30) */
int dqmoe_quant_fp8_rowwise(const void* x_bf16, int64_t rows, int cols, void* q, float* scale,
                            dqmoe_stream_t stream);
/* per 1x128 group of a row: per_token_block_cast_to_fp8 (test/util.py:34-45); scale [rows, ceil(cols/128)] */
int dqmoe_quant_fp8_block_1x128(const void* x_bf16, int64_t rows, int cols, void* q, float* scale,
                                dqmoe_stream_t stream);
/* per 128x128 block of each of e matrices [rows, cols]: per_block_cast_to_fp8 (test/util.py:48-68) */
int dqmoe_quant_fp8_block_128x128(const void* w_bf16, int e, int rows, int cols, void* q,
                                  float* scale, dqmoe_stream_t stream);
/*
 * One scale per tensor (or per expert when e > 1: x is [e, numel_per] and scale [e]).
 * amax_scratch is e floats of caller-owned device memory, overwritten.
 * The reference has this mode only for the intermediate (csrc/moe_kernels.h:136-221).
 */
int dqmoe_quant_fp8_tensor(const void* x_bf16, int e, int64_t numel_per, void* q, float* scale,
                           float* amax_scratch, dqmoe_stream_t stream);

/*
 * dqmoe_quant_fp8_tensor without the amax_scratch argument, for callers that must not
 * allocate device memory and own no spare buffer: code running between fixed, pre-planned
 * buffers (an inference-engine plugin's enqueue step, a step being recorded for replay, a
 * host with a locked memory budget). It has no counterpart in the reference. The scratch
 * is a 4 KiB static device array inside the library (held by every GPU that loads it), so
 * e is limited to 1024 slices; a larger e returns DQMOE_ERR_INVALID. The first call on a
 * device queries the array's address from the runtime and should happen before any stream
 * capture begins. All calls on a device share the array (it is zeroed per call): calls that
 * overlap on the GPU race. Results are identical to dqmoe_quant_fp8_tensor.
 */
int dqmoe_quant_fp8_tensor_static(const void* x_bf16, int e, int64_t numel_per, void* q, float* scale,
                                  dqmoe_stream_t stream);

/*
 * MXFP8 (see DQMOE_QUANT_FP8_MX; no counterpart in the reference). Quantiser over bf16 input: q e4m3
 * [rows, cols], scale UE8M0 bytes [rows, cols/32] row-major, s = 2^ceil(log2(max(amax, 1e-4) / 448)) per
 * 32-element group (cols a multiple of 32).
 */
int dqmoe_quant_mxfp8(const void* x_bf16, int64_t rows, int cols, void* q, uint8_t* scale, dqmoe_stream_t stream);
/*
 * The grouped GEMM reads scales in a tiled layout: one 512-byte block per 128 rows and 128 columns, row r of
 * the block at byte (r % 32) * 16 + (r / 32) * 4 with its four scale bytes in column order (the order the
 * tensor core's scale copy wants in shared memory), blocks indexed [row block][column block]. Rows form row
 * blocks by their index (weights: offsets == NULL, rows a multiple of 128) or, for expert-sorted activation
 * rows, by tile: block mtile_prefix[e] + (r - offsets[e]) / 128, row (r - offsets[e]) % 128 (offsets and
 * mtile_prefix [E+1] as dqmoe_route_sort / dqmoe_mtile_prefix give them), so that every 128-row tile of a
 * ragged expert owns whole blocks. dqmoe_mx_tile_scales converts row-major scales [*, cols/32] (cols a multiple
 * of 128); with dest_to_src != NULL output row r takes the scales of input row dest_to_src[r] / k (the
 * expert-sort gather; negative entries are skipped). With offsets, rows at or beyond offsets[E] are skipped, so
 * `rows` may be an upper bound of a row count that exists only on the device. dqmoe_mx_tiled_scale_bytes: size of the tiled buffer for
 * `rows` rows (E_sorted = number of experts for expert-sorted rows, 0 for rows that form blocks by index).
 */
size_t dqmoe_mx_tiled_scale_bytes(int64_t rows, int E_sorted, int cols);
int dqmoe_mx_tile_scales(const uint8_t* scale_rows, int64_t rows, int cols, const int32_t* dest_to_src, int k,
                         const int32_t* offsets, const int32_t* mtile_prefix, int E, uint8_t* scale_tiled,
                         dqmoe_stream_t stream);
/* Gather fused with the quantiser: q[r] = quant(x[dest_to_src[r] / k]), scales written tiled (H a multiple of 128). */
int dqmoe_permute_quant_mxfp8(const void* x_bf16, int H, int k, const int32_t* dest_to_src, int n,
                              const int32_t* offsets, const int32_t* mtile_prefix, int E, void* q,
                              uint8_t* scale_tiled, dqmoe_stream_t stream);

/*
 * NVFP4 quantiser over bf16 input (see DQMOE_QUANT_NVFP4; no counterpart in the reference): q [rows, cols/2]
 * bytes, element 2i of a row in the low nibble of byte i; scale [rows, cols/16] UE4M3 bytes row-major; gscale
 * one fp32 global scale per rows_per_gscale rows (rows for a whole tensor, rows of one expert for weights), given
 * by the caller - amax / (448 * 6) of the rows it covers is the usual choice. Per 16-element group:
 * scale byte = e4m3_rne((amax / 6) / g) saturating at 448, nibbles = e2m1_rne(x * (1 / (e4m3 * g))) saturating
 * at 6 (all divisions IEEE fp32; a group whose scale byte is zero stores zeros). cols a multiple of 16.
 * dqmoe_mx_tile_scales called with cols = 2 * (row length) turns the scale bytes into the tiled layout the
 * grouped GEMM reads: one 512-byte block per 128 rows and 64 elements.
 */
int dqmoe_quant_nvfp4(const void* x_bf16, int64_t rows, int cols, const float* gscale, int64_t rows_per_gscale, void* q,
                      uint8_t* scale, dqmoe_stream_t stream);

/* ------------------------------------------------------------------ grouped GEMM */

/*
 * Grouped GEMM over expert-sorted rows, the MoeGemmRunner::runGemm step
 * (csrc/moe_gemm_template.h:43-70, 1099-1103) with the epilogues fused:
 *   stage 1 (gated != 0): act = silu(A_e B_e[0:I]^T) * (A_e B_e[I:2I]^T), written as bf16
 *       (NONE), as bf16 plus per-row/per-tensor amax (CHANNEL/TENSOR), or as
 *       e4m3 with 1x128 scales (BLOCK);
 *   stage 2 (gated == 0): out[map[r], :] = dequant(A_e B_e^T) as bf16, map = dest_to_src
 *       or identity when NULL.
 * a: [n, K] expert-sorted rows; w: [E, gated ? 2*N : N, K]; offsets [E+1] and
 * mtile_prefix [E+1] (cumulative ceil(M_e/128)) as produced by dqmoe_route_sort's
 * workspace. N is the number of output columns.
 */
int dqmoe_grouped_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale,
                       const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K,
                       int E, int quant_mode, int gated, void* out, float* out_scale, float* amax,
                       const int32_t* dest_to_src, dqmoe_stream_t stream);

/*
 * Stage-2 grouped GEMM whose epilogue stores row r to the address row_dst[r] (uint64 device
 * addresses, 16-byte aligned rows of N bf16; 0 skips the row). The addresses may lie in another
 * GPU's memory that this GPU can reach over NVLink: the expert-parallel layer uses this to write
 * each result row directly into its home rank's output. Same GEMM as dqmoe_grouped_gemm.
 */
int dqmoe_grouped_gemm_rows(const void* a, const float* a_scale, const void* w, const float* w_scale,
                            const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K,
                            int E, int quant_mode, const void* row_dst, dqmoe_stream_t stream);

/*
 * The grouped GEMM in the MXFP8 mode (block-scaled tensor-core instruction, scales in TMEM): a [n, K] e4m3
 * expert-sorted rows, w [E, gated ? 2N : N, K] e4m3; a_sf and w_sf in the tiled layout above (a_sf by tiles of
 * the expert sort, w_sf by row index). Stage 1 writes e4m3 [n, N] and out_sf, tiled like a_sf, ready to be the
 * next GEMM's a_sf; stage 2 writes bf16 rows through dest_to_src (identity when NULL). K and N multiples of
 * 128. No counterpart in the reference.
 */
int dqmoe_grouped_gemm_mx(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf,
                          const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                          int gated, void* out, uint8_t* out_sf, const int32_t* dest_to_src,
                          dqmoe_stream_t stream);

/* Stage 2 of the MXFP8 grouped GEMM with explicit row addresses, as dqmoe_grouped_gemm_rows. */
int dqmoe_grouped_gemm_mx_rows(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf,
                               const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                               const void* row_dst, dqmoe_stream_t stream);

/*
 * The grouped GEMM in the NVFP4 mode (tcgen05.mma.kind::mxf4nvf4, 16-element UE4M3 scales in TMEM): a [n, K/2]
 * and w [E, gated ? 2N : N, K/2] packed e2m1; a_sf / w_sf tiled with one 512-byte block per 128 rows and 64 K
 * elements; a_gscale (1 float) and w_gscale [E] the global scales, whose product multiplies the accumulator.
 * Stage 1 re-quantises silu(gate) * value to NVFP4 with out_gscale (1 float, the caller's global scale of the
 * intermediate) and writes [n, N/2] bytes plus out_sf, tiled like a_sf; stage 2 writes bf16 rows through
 * dest_to_src. K a multiple of 256, N of 128. No counterpart in the reference.
 */
int dqmoe_grouped_gemm_nvfp4(const void* a, const uint8_t* a_sf, const float* a_gscale, const void* w,
                             const uint8_t* w_sf, const float* w_gscale, const int32_t* offsets,
                             const int32_t* mtile_prefix, int n, int N, int K, int E, int gated, void* out,
                             uint8_t* out_sf, const float* out_gscale, const int32_t* dest_to_src,
                             dqmoe_stream_t stream);

/* cumulative 128-row tile counts per expert from offsets[E+1] (device to device) */
int dqmoe_mtile_prefix(const int32_t* offsets, int E, int32_t* mtile_prefix, dqmoe_stream_t stream);

/*
 * Re-quantise the bf16 intermediate [n, I] written by a TENSOR/CHANNEL stage-1
 * GEMM using the amax it accumulated: per row (CHANNEL: scale [n]) or one value
 * (TENSOR: scale [1]). Replaces perTokendynamicFp8QuantKernel /
 * perTensorDynamicFp8QuantKernel (csrc/moe_kernels.h:136-282).
 */
int dqmoe_requant_from_amax(const void* act_bf16, int64_t n, int I, const float* amax,
                            int per_row, void* q, float* scale, dqmoe_stream_t stream);
/* The same over at most n_max rows when the row count exists only on the device
 * (*n_rows_device, e.g. the rows an expert-parallel rank received); NULL means n_max rows. */
int dqmoe_requant_from_amax_dev(const void* act_bf16, int64_t n_max, int I, const float* amax,
                                int per_row, void* q, float* scale, const int32_t* n_rows_device,
                                dqmoe_stream_t stream);

/* ------------------------------------------------------------------ expert parallel over peer memory */

/*
 * Building blocks of the expert-parallel layer that exchanges rows through peer-mapped
 * ("symmetric") buffers instead of a collective library. W <= 8 ranks of one node; rank `me`
 * owns experts [me*E/W, (me+1)*E/W). The *_ptrs arguments are host arrays of W device addresses,
 * entry r being rank r's copy of the same buffer (this rank's own copy included). Flags are
 * int32[3][8] per rank and carry a per-call `epoch` (any value different from the previous
 * call's), so nothing is cleared between calls. Waits are bounded (about 10 s unless
 * dqmoe_ep_set_wait_limit says otherwise) and report through dqmoe_device_status() instead of
 * hanging: 201 = plan never saw every rank's counts, 202 = some rank would receive more than `cap`
 * rows (every rank then sends and computes nothing in this call), 211 / 212 = wait on phase 1 / 2
 * ran out. The status word is sticky; a caller that must know whether a call's output is complete
 * reads it after the call. The reference has no multi-GPU path.
 *
 *   publish_counts  counts[E] of the local expert sort -> row `me` of every rank's cnt[W][E]; flag 0
 *   plan            waits flag 0 of all ranks; send_base[E] = row in the owner's receive buffer where
 *                   this rank's rows of expert e start (the receive buffer is grouped by expert, then
 *                   by source rank; send_base has E + 1 words, the last one is set to 1 when the plan
 *                   is void: counts missing, or a receive buffer of `cap` rows too small);
 *                   rx_offsets / rx_mtiles [E/W + 1] describe this rank's own receive buffer for
 *                   dqmoe_grouped_gemm
 *   dispatch        a[dest_to_src[i] / k] (+ scale row, + home slot) of every kept sorted row i ->
 *                   the owner's rx_rows / rx_scale / rx_home; flag 1 when all rows are written
 *   wait / signal   flag `phase` (1: rows landed, 2: results landed)
 *   row_ptrs        row_dst[r] = address of received row r's result in its home rank's d_out
 */
int dqmoe_ep_publish_counts(const int32_t* counts, int E, int me, int W, const void* const* cnt_ptrs,
                            const void* const* flag_ptrs, int epoch, dqmoe_stream_t stream);
int dqmoe_ep_plan(const int32_t* cnt, const int32_t* my_flags, int E, int me, int W, int epoch, int cap,
                  int32_t* send_base, int32_t* rx_offsets, int32_t* rx_mtiles, dqmoe_stream_t stream);
/* Clock cycles a flag wait of the kernels above may spin before it gives up (process-wide, applies to
 * launches made afterwards); 0 restores the default of about 10 s. */
int dqmoe_ep_set_wait_limit(int64_t cycles);
/* publish_counts followed by plan, and signal followed by wait, each as one launch (a launch less on the path
 * every call waits on); same arguments and status codes as the separate calls. */
int dqmoe_ep_publish_plan(const int32_t* counts, int E, int me, int W, const void* const* cnt_ptrs,
                          const void* const* flag_ptrs, int epoch, int cap, int32_t* send_base,
                          int32_t* rx_offsets, int32_t* rx_mtiles, dqmoe_stream_t stream);
int dqmoe_ep_signal_wait(const void* const* flag_ptrs, int phase, int me, int W, int epoch, dqmoe_stream_t stream);
int dqmoe_ep_dispatch(const void* a, const float* a_scale, size_t row_bytes, int scale_cols, int k, int n,
                      const int32_t* offsets, const int32_t* dest_to_src, const int32_t* send_base,
                      int E, int me, int W, const void* const* rx_rows, const void* const* rx_scale,
                      const void* const* rx_home, const void* const* flag_ptrs, int32_t* done_counter,
                      int epoch, dqmoe_stream_t stream);
int dqmoe_ep_wait(const int32_t* my_flags, int phase, int W, int epoch, dqmoe_stream_t stream);
int dqmoe_ep_signal(const void* const* flag_ptrs, int phase, int me, int W, int epoch, dqmoe_stream_t stream);
int dqmoe_ep_row_ptrs(const int32_t* rx_home, const int32_t* rx_offsets, int E_local,
                      const void* const* d_out_ptrs, int W, size_t out_row_bytes, int cap, void* row_dst,
                      dqmoe_stream_t stream);
/* dqmoe_ep_wait on phase 1 and dqmoe_ep_row_ptrs as one launch (every block waits for the W flags itself). */
int dqmoe_ep_wait_row_ptrs(const int32_t* my_flags, int epoch, const int32_t* rx_home, const int32_t* rx_offsets, int E_local,
                           const void* const* d_out_ptrs, int W, size_t out_row_bytes, int cap, void* row_dst,
                           dqmoe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DQMOE_H_ */
