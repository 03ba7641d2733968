/* kquant_b200 - C ABI of the B200 (sm_100a) quantized-weight path.
 *
 * A drop-in for the quantized-weight ops of asher/mlx-kquant: the entry points
 * below are what the reference's op layer (src/kquant_ops.cpp) hands to its
 * Primitive::eval_* implementations, flattened to plain pointers and sizes. File
 * and line citations are paths inside the reference repository.
 *
 * Conventions
 *  - Every function returns 0 on success or a KQ_ERR_* code and records a
 *    message retrievable with kq_last_error() (thread-local). Argument errors
 *    carry the reference's message text, prefixed "[mlx_kquant.<op>]".
 *  - All data pointers are DEVICE pointers owned by the caller unless a name
 *    ends in _host. Nothing is allocated internally; the one kernel family that
 *    needs scratch (gather) takes a caller-provided workspace whose size is
 *    given by kq_gather_qmm_workspace_bytes().
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *    Calls are asynchronous; ordering is stream order.
 *  - dtype codes: KQ_F32 = 0, KQ_F16 = 1, KQ_BF16 = 2.
 *  - Codecs are named as in the reference registry (src/kquant_codec.cpp:12-37);
 *    this library implements all 21 of them: q2_k q3_k q4_k q5_k q6_k q4_0 q8_0 iq4_nl iq4_xs
 *    iq2_xxs q4_1 q5_0 q5_1 iq3_xxs iq3_s iq2_xs iq2_s iq1_s iq1_m mxfp4 nvfp4 (registry indices in that
 *    order; the ten the benchmark names come first). Any other name is reported as unknown.
 */
#ifndef KQUANT_B200_H
#define KQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KQ_API __attribute__((visibility("default")))
#else
#define KQ_API
#endif

#define KQ_F32 0
#define KQ_F16 1
#define KQ_BF16 2

#define KQ_OK 0
#define KQ_ERR_INVALID_ARGUMENT 1 /* the reference throws std::invalid_argument here */
#define KQ_ERR_RUNTIME 2          /* the reference throws std::runtime_error here */
#define KQ_ERR_CUDA 3             /* a CUDA call failed; message holds cudaGetErrorString */
#define KQ_ERR_UNSUPPORTED 4      /* valid in the reference, not built here yet */

/* Message of the last failing call on this thread ("" if none). */
KQ_API const char* kq_last_error(void);

/* Library version string. */
KQ_API const char* kq_version(void);

/* ---- codec registry: replaces codec_by_name / codec_names,
 * src/kquant_codec.h:10-25, src/kquant_codec.cpp:12-55 ---- */
KQ_API int kq_codec_count(void);
/* Fills the geometry of codec `index` (0 <= index < kq_codec_count()); any
 * out-pointer may be NULL. *name points at a static string. */
KQ_API int kq_codec_info(int index, const char** name, int* weights_per_block, int* bytes_per_block, int* bits,
                  int* requires_imatrix);
/* Index of a codec name, or -1. */
KQ_API int kq_codec_find(const char* name);

/* ---- dequantize: replaces KQuantDequantize::eval_cpu / eval_gpu,
 * src/kquant_dequantize.cpp:59-130 (op: src/kquant_ops.cpp:55-110) ----
 * w: w_bytes of wire data, a whole number of blocks. out: w_bytes /
 * bytes_per_block * weights_per_block elements of out_dtype. Bit-exact with the
 * reference's CPU decoders for f32; f16/bf16 are the IEEE round-to-nearest-even
 * of that f32 value. */
KQ_API int kq_dequantize(const void* w, size_t w_bytes, const char* kquant_type, int out_dtype, void* out, void* stream);

/* ---- quantize: replaces KQuantQuantize::eval_cpu, src/kquant_encode.cpp:48-98 ->
 * kquant_quantize_dispatch, src/kquant_cpu_encode.cpp:824-859 (op: src/kquant_ops.cpp:550-631) ----
 * HOST pointers: the reference's encoder is a CPU-only op as well. w: n_weights values of w_dtype
 * (rows of K), out: n_weights / weights_per_block * bytes_per_block bytes, imatrix: K floats or NULL.
 * Byte-identical with the reference for the thirteen codecs that have a host encoder here - q2_k .. q6_k, q4_0, q4_1,
 * q5_0, q5_1, q8_0, iq4_nl, iq4_xs, iq2_xxs; the other eight of the registry are decode-only in this library and
 * return KQ_ERR_UNSUPPORTED - (the IQ ones: src/kquant_iq_encode.cpp:2099-2176);
 * iq2_xxs requires an imatrix, as in the reference.
 * threads: 0 = all host threads (blocks are independent: the bytes do not depend on it). */
KQ_API int kq_quantize_cpu(const void* w, int w_dtype, long long n_weights, long long K, const char* kquant_type,
                           const float* imatrix, void* out, int threads);

/* ---- quantized_matmul: replaces KQuantMatmul::eval_cpu / eval_gpu,
 * src/kquant_matmul.cpp:1104-1164, 1199-1488 (op: src/kquant_ops.cpp:112-183) ----
 * y[rows, N] = x[rows, K] . dequant(w)^T with fp32 accumulation, w laid out
 * [N, K / weights_per_block * bytes_per_block] (transpose != 0).
 *  - x_dtype KQ_F16 / KQ_BF16: y has the same dtype. KQ_F32: x is rounded to
 *    bf16 and y is bf16, as the reference's op does (src/kquant_ops.cpp:159).
 *  - x rows: `rows` of them (all leading dims of the reference's x flattened),
 *    x_row_stride elements apart, each row contiguous and 16-byte aligned.
 *  - y rows are y_row_stride elements apart.
 *  - transpose == 0: w is [K, N / weights_per_block * bytes_per_block] (every row a quantized vector of N
 *    weights), y = x . dequant(w); served by a plain streaming kernel (any M, tuned for small M); x needs
 *    element alignment only.
 *  - workspace: kq_quantized_matmul_workspace_bytes(x_dtype, rows, K) bytes of
 *    device memory, 256-byte aligned (0 bytes, and NULL allowed, for fp16
 *    activations or a single row). Calls with more than 16 rows run on the tensor
 *    cores in fp16; bf16 / f32 activations are converted there first, exactly, with
 *    a per-row power-of-two factor. With 2-16 rows the workspace is optional: q4_k
 *    uses it for the same conversion (several times faster), and a call without it
 *    still works. */
KQ_API size_t kq_quantized_matmul_workspace_bytes(int x_dtype, long long rows, int K);
KQ_API int kq_quantized_matmul(const void* x, int x_dtype, long long rows, int K, long long x_row_stride, const void* w,
                        size_t w_row_bytes, int N, const char* kquant_type, int transpose, void* y,
                        long long y_row_stride, void* workspace, size_t workspace_bytes, void* stream);

/* Diagnostic: kernels never spin forever - a wait that does not complete within
 * two seconds makes the kernel stop, raise a bit here and return (results of that
 * call are then undefined). *flags = 0 means no kernel ever gave up. Synchronises
 * the device; clear != 0 resets the flags. No counterpart in the reference. */
KQ_API int kq_device_error_flags(int* flags, int clear);

/* ---- gather_qmm: replaces KQuantGatherQMM::eval_cpu / eval_gpu,
 * src/kquant_gather.cpp:470-746, 819-956 (op: src/kquant_ops.cpp:293-420) ----
 * For every index entry b in [0, n_entries):
 *     y[b] [M, N] = x[lhs[b]] [M, K] . dequant(w[rhs[b]])^T
 * x: [x_batch, M, K] dense (x_dtype as above); w: n_experts matrices, matrix e
 * at w + e * w_expert_stride_bytes (64-bit, so strided views and stacks above
 * 2 GiB work, cf. src/kquant_gather.cpp:548-563); lhs / rhs: uint32 device
 * arrays of n_entries, already broadcast together; y: [n_entries, M, N] dense.
 * rhs_sorted != 0 promises rhs is non-decreasing (the reference's right_sorted
 * flag); it is a hint only, results do not depend on it.
 * workspace: at least kq_gather_qmm_workspace_bytes(n_entries, M, n_experts, K)
 * bytes of device memory, 256-byte aligned, private to this call until it
 * completes on the stream. Decode-sized calls need a few hundred KB; prefill-sized
 * ones (16 or more rows per expert on average) also hold an expert-sorted fp16 copy
 * of the routed activations (n_entries * M * K * 2 bytes) for the tensor-core kernel.
 * The size depends on K (the fp16 copy): pass the call's own K. K = 0 returns the size of the grouping
 * scratch alone, which is what kq_gather_qmm_noalloc needs; kq_gather_qmm rejects a workspace of that size.
 * Entries whose rhs index is >= n_experts or whose lhs index is >= x_batch are skipped: their rows of y stay
 * unwritten (the reference checks neither). n_entries * M must stay below 2^31. */
KQ_API size_t kq_gather_qmm_workspace_bytes(long long n_entries, int M, int n_experts, int K);
KQ_API int kq_gather_qmm(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w, int n_experts,
                  long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                  const uint32_t* lhs_indices, const uint32_t* rhs_indices, long long n_entries, int transpose,
                  int rhs_sorted, void* y, void* workspace, size_t workspace_bytes, void* stream);

/* ---- the elementwise stages of a mixture-of-experts SwiGLU block ----
 * Not among the reference's three ops: they are the stages its fused Metal MoE op (moe_glu_gather_kq,
 * src/kquant.h:335-357; no CPU evaluation) performs between the three gathered products, offered here so that
 * a block composed of kq_gather_qmm calls needs no generic elementwise passes. Device pointers, dtype KQ_F16
 * or KQ_BF16, fp32 arithmetic, one rounding.
 *  kq_swiglu:      out[r, c] = silu(gate[r * in_row_stride + c]) * up[r * in_row_stride + c], c < F; out is
 *                  [rows, F] dense. A fused [rows, 2F] gate|up product passes up = gate + F, stride 2F.
 *  kq_moe_combine: y[t, :] = sum_j probs[t * k + j] * d[(t * k + j), :], d [tokens * k, H], probs float32.
 *                  A row whose weight is exactly 0 is not read.
 * The two variants below serve a rank that holds only some of the experts (every rank sees every routed row,
 * and rows of other ranks' experts carry an out-of-range index, which kq_gather_qmm leaves unwritten):
 *  kq_swiglu_routed:   kq_swiglu that skips rows with row_expert[r] >= n_experts (uint32 compare).
 *  kq_moe_combine_f32: kq_moe_combine with a float32 y, the partial sum a reduce-scatter then completes. */
KQ_API int kq_swiglu(const void* gate, const void* up, long long in_row_stride, long long rows, int F, int dtype,
                     void* out, void* stream);
KQ_API int kq_moe_combine(const void* d, const float* probs, long long tokens, int k, int H, int dtype, void* y,
                          void* stream);
KQ_API int kq_swiglu_routed(const void* gate, const void* up, long long in_row_stride, long long rows, int F, int dtype,
                            void* out, const uint32_t* row_expert, int n_experts, void* stream);
KQ_API int kq_moe_combine_f32(const void* d, const float* probs, long long tokens, int k, int H, int dtype, float* y,
                              void* stream);

/* ---- fused mixture-of-experts decode ops: replace the reference's Metal-only moe_glu_gather_kq,
 * gather_qmv_mix_ns_kq and moe_router_topk (src/kquant.h:335-357, 549-558, 560-585; no CPU eval exists there,
 * src/kquant_moe_glu.cpp:1-8, so their oracle is the composition of gather_qmm calls) ----
 * kq_codec_has_moe_glu: 1 when the codec has these kernels (q4_k), else 0 (codec_has_moe_glu, src/kquant.h:359).
 * kq_moe_glu_gather: x [T, K]; gate_w / up_w: n_experts matrices [N, w_row_bytes] each, matrix e at
 *   base + e * expert_stride_bytes; indices uint32 [T, R]; y [T, R, N] in x's dtype:
 *   y[t, r] = act(x[t] . Wg[e]^T) * (x[t] . Wu[e]^T), e = indices[t, r], float32 sums, the activation in float32,
 *   ONE rounding. act: "silu", "gelu" (tanh form), "silu_limit" (gate clamped from above and up to +-limit first;
 *   limit > 0). Entries with e >= n_experts are skipped (their rows of y stay unwritten).
 * kq_gather_qmv_mix: x [T, S, K] (one row per routed slot); w as above; indices uint32 [T, S]; scores float32
 *   [T, S]; y [T, N] in x's dtype: y[t] = sum_s scores[t, s] * (x[t, s] . W[e_s]^T), accumulated in float32 in slot
 *   order, ONE rounding.
 * Both: q4_k, float16 / bfloat16 rows, K % 256 == 0, dense 16-byte aligned rows; anything else returns
 *   KQ_ERR_UNSUPPORTED and the caller composes the op from kq_gather_qmm. Up to KQ_MOE_DIRECT_MAX_ENTRIES (token,
 *   slot) entries every entry streams its expert's rows by itself and no scratch is needed (workspace may be
 *   NULL). Beyond that, with a workspace of kq_moe_decode_workspace_bytes(T * R, n_experts, N_mix) bytes (N_mix =
 *   N for kq_gather_qmv_mix, 0 for kq_moe_glu_gather; 256-byte aligned, private to the call until it completes),
 *   the entries are grouped by expert on the device and one read of an expert's rows serves up to sixteen entries; the
 *   mix then rounds each slot's product once before the weighted sum, as the unfused ops do. reuse_grouping != 0
 *   tells kq_gather_qmv_mix that `workspace` still holds the grouping kq_moe_glu_gather made from the SAME indices
 *   (same T * S, same n_experts; a workspace of the mix size was given to both calls): it is not rebuilt. Without a workspace
 *   the per-entry form runs at any size. These are decode kernels: for prefill-sized calls (dozens of rows per
 *   expert) compose the block from kq_gather_qmm, which uses the tensor-core tile kernel.
 * kq_moe_router_topk: logits [T, E (+ 1 with shared_gate)] of `dtype`; scores the E columns in float32
 *   ("softmax", or "sqrtsoftplus" = sqrt(softplus(x)), which requires norm_topk_prob), picks the top_k largest of
 *   score (+ bias [E] if given: it ranks only), lowest index first among equals, optionally renormalises the picked
 *   scores (sqrtsoftplus with a 1e-20 guard), multiplies by per_expert_scale [E] (if given) and by `scale`; with
 *   shared_gate the sigmoid of column E lands in scores[:, top_k]. indices uint32 [T, top_k], scores float32
 *   [T, top_k (+ 1)]. E <= 1024, top_k <= 16. */
#define KQ_MOE_DIRECT_MAX_ENTRIES 152
KQ_API int kq_codec_has_moe_glu(const char* kquant_type);
KQ_API size_t kq_moe_decode_workspace_bytes(long long n_entries, int n_experts, int N_mix);
KQ_API int kq_moe_glu_gather(const void* x, int x_dtype, long long T, int K, const void* gate_w,
                             long long gate_expert_stride_bytes, const void* up_w, long long up_expert_stride_bytes,
                             size_t w_row_bytes, int N, int n_experts, const char* kquant_type, const uint32_t* indices,
                             int R, const char* act, float limit, void* y, void* workspace, size_t workspace_bytes,
                             void* stream);
KQ_API int kq_gather_qmv_mix(const void* x, int x_dtype, long long T, int S, int K, const void* w,
                             long long w_expert_stride_bytes, size_t w_row_bytes, int N, int n_experts,
                             const char* kquant_type, const uint32_t* indices, const float* scores, void* y,
                             void* workspace, size_t workspace_bytes, int reuse_grouping, void* stream);
/* One mixture-of-experts SwiGLU block for prefill-sized calls, y[t] = sum_j scores[t, j] * down_e( silu(gate_e x_t) *
 * up_e x_t ) with e = indices[t, j]: what a reference caller composes from gather_qmm(gate), gather_qmm(up), the
 * activation, gather_qmm(down) and the weighted sum (mlx_kquant/nn.py SwitchGLU + src/kquant_ops.cpp:292-420), with the
 * same roundings to x's dtype after each product and after the activation - so the same bits as that composition -
 * but ONE grouping by expert, no scatter / re-gather between the products and the activation computed inside the
 * pre-pass of the down product. x [T, H] (row stride x_row_stride elements, float16 / bfloat16, 16-byte aligned rows);
 * token_rows NULL, or [T] uint32: token t's activation is row token_rows[t] of x (tokens scattered in a larger
 * buffer); w_gate_up [n_experts, 2 F, gate_up_row_bytes] = every expert's gate rows then its up rows (H weights per
 * row); w_down [n_experts, H, down_row_bytes] (F weights per row); indices / scores [T, top_k] (uint32 / float32); an
 * index outside [0, n_experts) contributes nothing (an expert-parallel rank passes the other ranks' experts that
 * way). y [T, H] of y_dtype = x_dtype or KQ_F32 (partial sums for a later reduction). Any codec. Sizes: at least 512
 * routed rows and 16 per expert on average, H % 8 == F % 8 == 0; otherwise KQ_ERR_UNSUPPORTED.
 * kq_moe_block_workspace_bytes(T, top_k, n_experts, H, F): bytes of device scratch the call needs (0 = sizes not
 * supported); 256-byte aligned, private to the call until it completes. */
KQ_API size_t kq_moe_block_workspace_bytes(long long T, int top_k, int n_experts, int H, int F);
KQ_API int kq_moe_swiglu_block(const void* x, int x_dtype, long long T, int H, long long x_row_stride,
                               const uint32_t* token_rows, const void* w_gate_up, long long gate_up_expert_stride_bytes,
                               size_t gate_up_row_bytes, int F, const void* w_down, long long down_expert_stride_bytes,
                               size_t down_row_bytes, int n_experts, const char* kquant_type, const uint32_t* indices,
                               const float* scores, int top_k, void* y, int y_dtype, void* workspace,
                               size_t workspace_bytes, void* stream);
/* Expert parallelism over peer memory (one process per GPU; the buffers are mapped into each other's address space
 * by the host, e.g. with CUDA IPC handles; plain stores, no multicast). kq_moe_swiglu_block_scatter is
 * kq_moe_swiglu_block for a rank that owns n_experts of the experts and sees the tokens of ALL ranks (T = world *
 * tokens_per_rank, token g = w * tokens_per_rank + t belongs to rank w): instead of a [T, H] output it writes the
 * partial row of token g to slot_ptrs[w] + (my_rank * tokens_per_rank + t) * H elements - slot_ptrs being a DEVICE
 * array of `world` pointers to the ranks' [world, tokens_per_rank, H] slot buffers of slot_dtype (x_dtype or
 * KQ_F32) - and writes nothing for a token none of whose experts it owns. After every rank's call has completed
 * (the host orders that, e.g. with a collective on the same streams), the owner adds its tokens' slots with
 * kq_moe_sum_slots: slots [world, T, H] (T tokens of this rank), ids [T, top_k] GLOBAL expert indices, rank_lo
 * [world + 1] (device) the first expert of each rank's contiguous share: y[t] = sum, in rank order, of slots[r][t]
 * over the ranks r that own at least one of token t's experts (float32 accumulation, one rounding to y_dtype).
 * Together they replace "partial sums + reduce-scatter": only non-empty partial rows cross the link, once. */
KQ_API int kq_moe_swiglu_block_scatter(const void* x, int x_dtype, long long T, int H, long long x_row_stride,
                                       const uint32_t* token_rows, const void* w_gate_up,
                                       long long gate_up_expert_stride_bytes, size_t gate_up_row_bytes, int F,
                                       const void* w_down, long long down_expert_stride_bytes, size_t down_row_bytes,
                                       int n_experts, const char* kquant_type, const uint32_t* indices,
                                       const float* scores, int top_k, void* const* slot_ptrs, int slot_dtype,
                                       int my_rank, long long tokens_per_rank, void* workspace, size_t workspace_bytes,
                                       void* stream);
KQ_API int kq_moe_sum_slots(const void* slots, int slot_dtype, const uint32_t* ids, const int* rank_lo, int world,
                            long long T, int top_k, int H, void* y, int y_dtype, void* stream);
/* Device buffers shared between the processes of one node, for the peer-memory forms above: the owner creates
 * (cudaMalloc + CUDA IPC; handle64 receives the 64-byte handle, to be sent to the peers over any host channel), a
 * peer opens the handle on ITS current device (lazy peer access) and gets a pointer its kernels may store to, closes
 * it when done; the owner destroys the buffer after every peer has closed it. */
KQ_API int kq_peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle64);
KQ_API int kq_peer_buffer_open(const unsigned char* handle64, void** ptr);
KQ_API int kq_peer_buffer_close(void* ptr);
KQ_API int kq_peer_buffer_destroy(void* ptr);
/* One asynchronous device-to-device copy on `stream` (copy engines, no SM); dst may be a peer's buffer. */
KQ_API int kq_peer_copy_async(void* dst, const void* src, size_t bytes, void* stream);
KQ_API int kq_moe_router_topk(const void* logits, int dtype, long long T, int E, int top_k, int norm_topk_prob,
                              int shared_gate, const float* per_expert_scale, const float* bias, const char* scoring,
                              float scale, uint32_t* indices, float* scores, void* stream);

/* ---- gather_qmm without a workspace (no counterpart in the reference) ----
 * Same computation and arguments as kq_gather_qmm, minus the workspace: the
 * grouping scratch lives in a fixed KQ_GATHER_STATIC_WS_BYTES array that is part
 * of the library image on every GPU that loads it. Meant for callers that are
 * not allowed to allocate device memory at all: a plugin inside a host process
 * that has handed every byte of HBM to its own arena and forbids driver
 * allocations afterwards, or a serving loop that must never pay cudaMalloc's
 * device-wide synchronisation. Nothing here calls cudaMalloc, cudaFree or an
 * allocating library routine.
 *  - Always runs the decode regime, whatever the size of the call, and without the fp16 copy of the rows
 *    that kq_gather_qmm makes for q4_k with bfloat16 / float32 activations: those calls take the slower
 *    kernels that read such rows directly.
 *  - Limit (transpose != 0 only; the [K, N] orientation needs no scratch): the grouping scratch of the call -
 *    counters per expert, an index per entry and a 144-byte task per 16 rows of every expert, about
 *    14 bytes per entry plus 0.4 KB per expert at M = 1 - must fit KQ_GATHER_STATIC_WS_BYTES, else the call is
 *    rejected with KQ_ERR_INVALID_ARGUMENT after the ordinary argument checks (for M = 1 and 128 experts that
 *    is about 75 000 index entries per call). kq_gather_qmm_workspace_bytes(n_entries, M, n_experts, 0) is the
 *    number compared with the limit.
 *  - The first call on each device looks up the array's device address; make
 *    that first call outside any stream capture.
 *  - All calls on a device share the one array (it keeps the previous call's
 *    contents; what has to start from zero is cleared on the stream first), so
 *    two calls that can overlap on the GPU - different streams, no dependency -
 *    race. Serialise them or use kq_gather_qmm with separate workspaces. */
#define KQ_GATHER_STATIC_WS_BYTES (1u << 20)
KQ_API int kq_gather_qmm_noalloc(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w,
                                 int n_experts, long long w_expert_stride_bytes, size_t w_row_bytes, int N,
                                 const char* kquant_type, const uint32_t* lhs_indices, const uint32_t* rhs_indices,
                                 long long n_entries, int transpose, int rhs_sorted, void* y, void* stream);

/* Decode product with the bias add fused: y = round(x @ dequant(w).T + bias), one row of x, the sum and the add
 * in float32 and ONE rounding to the output dtype (x's dtype, bfloat16 for float32 x). bias: N values in that
 * output dtype. Replaces mlx_kquant::quantized_matmul_qmv_bias (src/kquant_ops.cpp:185-283): q8_0 only, any other
 * codec is KQ_ERR_INVALID_ARGUMENT, as there. */
KQ_API int kq_quantized_matmul_qmv_bias(const void* x, int x_dtype, int K, const void* w, size_t w_row_bytes, int N,
                                        const char* kquant_type, const void* bias, void* y, void* stream);

/* ---- expert tile map + segment product (the MoE prefill pair of the reference) ----
 * Replaces: mlx_kquant::expert_tile_map (src/kquant_ops.cpp:422-447) and mlx_kquant::gather_qmm_seg
 * (src/kquant_ops.cpp:466-548; Metal-only in the reference, "no CPU implementation",
 * src/kquant_gather.cpp:983-1006).
 *  kq_expert_tile_map: indices uint32 [rows], the expert of every row, rows sorted by expert. Writes
 *    map uint32 [capacity, 3] = (expert, row_start, num_rows <= 64) for the first *count entries (entry order
 *    unspecified beyond that, as in the reference) and count uint32 [1]. capacity =
 *    kq_expert_tile_map_capacity(rows, n_experts) = max(rows / 64 + min(n_experts, rows), 1). Entries whose
 *    expert is >= n_experts belong to no tile. Device pointers; no host read.
 *  kq_gather_qmm_seg: x [rows, K] dense (rows grouped by expert), w [n_experts, N, w_row_bytes] with
 *    w_expert_stride_bytes between matrices, y [rows, N] dense in x's dtype (bfloat16 for float32 x):
 *    y[r] = x[r] @ dequant(w[expert of the map entry that covers r]).T for the first *count entries of
 *    map [map_tiles, 3]; rows no entry covers are left unwritten. The pieces of one expert should form
 *    one run of consecutive rows (both builders above do that); then they are re-cut into 256-row tiles.
 *    Any other map is taken piece by piece. Pieces must not overlap. */
KQ_API long long kq_expert_tile_map_capacity(long long rows, int n_experts);
KQ_API size_t kq_expert_tile_map_workspace_bytes(int n_experts);
KQ_API int kq_expert_tile_map(const uint32_t* indices, long long rows, int n_experts, uint32_t* map, uint32_t* count,
                              void* workspace, size_t workspace_bytes, void* stream);
KQ_API size_t kq_gather_qmm_seg_workspace_bytes(int x_dtype, long long rows, int K, int n_experts, long long map_tiles);
KQ_API int kq_gather_qmm_seg(const void* x, int x_dtype, long long rows, int K, const void* w, int n_experts,
                             long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                             const uint32_t* map, const uint32_t* count, long long map_tiles, void* y, void* workspace,
                             size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KQUANT_B200_H */
