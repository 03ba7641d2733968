// Internal launch interface between the C-ABI layer (kq_abi.cu) and the kernel
// translation units. Not installed; the public surface is include/kquant_b200.h.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kq {

// dequantize n_blocks blocks of `codec` wire bytes to `dtype` (0 f32, 1 f16, 2 bf16).
cudaError_t launch_dequantize(int codec, const uint8_t* w, long long n_blocks, int dtype, void* out,
                              cudaStream_t st);

// One group of at most 16 activation rows that all multiply the same weight
// matrix: the unit of work of the skinny-M kernel. Built on the device by the
// gather path (one per expert and 16-row slice); the dense path needs none.
struct GemvTask {
  const uint8_t* w;   // wire bytes of the [N, K] matrix
  int m;              // valid rows, 1..16
  int pad;
  int xrow[16];       // row index into x (units of x_row_stride)
  int yrow[16];       // row index into y (units of y_row_stride)
};

struct GemvArgs {
  const void* x;
  long long x_row_stride;   // elements between consecutive x rows
  void* y;
  long long y_row_stride;   // elements between consecutive y rows
  const uint8_t* w;         // used when tasks == nullptr
  int w_align16;            // every weight matrix (w, or each task's w) starts 16-byte aligned
  long long row_bytes;      // wire bytes per weight row
  int N, K;
  int M;                    // total rows when tasks == nullptr (split in 16-row slices)
  const GemvTask* tasks;    // device array or nullptr
  const int* n_tasks_dev;   // device count of valid tasks (may be < grid.y), or nullptr
  int n_tasks;              // grid.y when tasks != nullptr
  int task_offset;          // index of tasks[0] in the whole task list (for n_tasks_dev)
  int max_m;                // upper bound on any task's m (picks the 8- or 16-row B tile)
  int avg_rows;             // task lists: average rows per weight matrix (0 = unknown), a dispatch hint
  // fp16 kernels only: write bfloat16 instead (y = bf16(sum * row_scale[x row])), for callers that
  // converted bf16 / f32 activations to fp16 with a per-row power-of-two factor
  int out_bf16;
  const float* row_scale;   // indexed like the rows of x, or nullptr
  // one dense row only: N values in the output dtype added to the float sum before its single rounding
  // (quantized_matmul_qmv_bias), or nullptr. Honoured by gemv_kernel<> and gemv_dp4a_kernel<>.
  const void* bias;
};

// y = x . dequant(w)^T for skinny row groups. x_dtype: 0 f32 (rounded to bf16
// on load, output bf16), 1 f16, 2 bf16.
cudaError_t launch_gemv(int codec, int x_dtype, const GemvArgs& a, cudaStream_t st);

// Up to four activation rows per pass (dense, or task lists in slices of four): products on the
// integer dot-product pipe over 16-bit quantized activations (kq_gemv_dp4a.cu).
bool gemv_dp4a_supported(int codec, int x_dtype, const GemvArgs& a);
cudaError_t launch_gemv_dp4a(int codec, int x_dtype, const GemvArgs& a, cudaStream_t st);

// Prefill (M > 16) tile kernel on tcgen05 tensor cores with TMEM accumulators.
// bf16 / f32 activations need gemm_workspace_bytes() of scratch for their fp16 copy.
size_t gemm_workspace_bytes(int x_dtype, long long rows, int K);
cudaError_t launch_gemm(int codec, int x_dtype, const void* x, long long x_row_stride, void* y, long long y_row_stride,
                        const uint8_t* w, long long row_bytes, int M, int N, int K, void* workspace, cudaStream_t st);
// Grouped (mixture-of-experts) prefill: 256-row tiles of expert-sorted rows, see kq_gather.cu.
constexpr int kGroupedTileRows = 256;
constexpr int kSegMapTileRows = 64;  // rows per entry of an expert tile map (the reference kernel's tile height)
// expert_tile_map / gather_qmm_seg (kq_gather.cu)
size_t tile_map_workspace_bytes(int n_experts);
cudaError_t launch_tile_map(const uint32_t* indices, long long rows, int n_experts, uint32_t* map, uint32_t* count,
                            void* workspace, cudaStream_t st);
size_t gather_seg_workspace_bytes(int x_dtype, long long rows, int K, int n_experts, long long cap);
cudaError_t launch_gather_seg(int codec, int x_dtype, const void* x, long long rows, int K, const uint8_t* w,
                              int n_experts, long long expert_stride, long long row_bytes, int N, const uint32_t* map,
                              const uint32_t* count, long long cap, void* y, void* workspace, cudaStream_t st);
cudaError_t launch_gemm_grouped(int codec, int x_dtype, const void* x, int M, int K, const uint8_t* w,
                                long long expert_stride, long long row_bytes, int N, const uint32_t* lhs,
                                const int* order, long long rows_total, void* y, __half* xh, float* row_scale,
                                int* yrow, const void* tiles, const int* n_tiles_dev, int max_tiles,
                                const int* n_valid_dev, cudaStream_t st);
cudaError_t launch_gemm_tiles(int codec, bool out_half, const void* xh, long long rows_total, int K, const uint8_t* w,
                              long long expert_stride, long long row_bytes, int N, void* y, const float* row_scale,
                              const int* yrow, const void* tiles, const int* n_tiles_dev, int max_tiles,
                              cudaStream_t st);
// Flags raised by kernels that gave up on a bounded wait (0 = none); synchronises the device.
cudaError_t read_device_error(int* out, bool clear);
int* device_error_word();  // device address of that flag word on the current device (nullptr on failure)

// Fused mixture-of-experts decode kernels (kq_moe_decode.cu): q4_k expert stacks, fp16 / bf16 rows.
// act: 0 silu, 1 gelu (tanh form), 2 silu with limit. scoring: 0 softmax, 1 sqrt(softplus).
bool moe_decode_supported(int codec, int x_dtype, int K, long long row_bytes, const void* x, const void* w0,
                          long long stride0, const void* w1, long long stride1);
cudaError_t launch_moe_glu(int x_dtype, const void* x, int K, const uint8_t* wg, long long stride_g, const uint8_t* wu,
                           long long stride_u, long long row_bytes, int F, int n_experts, const uint32_t* idx,
                           long long n_entries, int R, int act, float limit, void* y, cudaStream_t st);
cudaError_t launch_moe_mix(int x_dtype, const void* x, int K, const uint8_t* w, long long stride_w, long long row_bytes,
                           int N, int n_experts, const uint32_t* idx, const float* scores, long long T, int S, void* y,
                           cudaStream_t st);
// grouped forms for more entries (tasks of up to four entries per expert); scratch from moe_grouped_workspace_bytes
size_t moe_grouped_workspace_bytes(long long n_entries, int n_experts, long long d_bytes);
bool moe_grouped_supported(int K, long long row_bytes, bool rows_kernel);
cudaError_t launch_moe_grouping_only(const uint32_t* idx, long long n_entries, int n_experts, void* workspace,
                                     cudaStream_t st);
cudaError_t launch_moe_glu_grouped(int x_dtype, const void* x, int K, const uint8_t* wg, long long stride_g,
                                   const uint8_t* wu, long long stride_u, long long row_bytes, int F, int n_experts,
                                   const uint32_t* idx, long long n_entries, int R, int act, float limit, void* y,
                                   void* workspace, cudaStream_t st);
cudaError_t launch_moe_mix_grouped(int x_dtype, const void* x, int K, const uint8_t* w, long long stride_w,
                                   long long row_bytes, int N, int n_experts, const uint32_t* idx, const float* scores,
                                   long long T, int S, void* y, void* workspace, bool reuse_grouping, cudaStream_t st);
cudaError_t launch_router_topk(const void* logits, int dtype, int T, int E, int top_k, int norm, int shared, int scoring,
                               const float* pes, const float* bias, float scale, uint32_t* indices, float* scores,
                               cudaStream_t st);

// q4_k, one dense fp16 / bf16 activation row, matrices of about one wave of CTAs (kq_gemv_stream.cu)
bool gemv_stream_supported(int codec, int x_dtype, const GemvArgs& a);
cudaError_t launch_gemv_stream(int x_dtype, const GemvArgs& a, cudaStream_t st);
// Exact fp16 copy of `rows` activation rows (x_dtype 0 f32 / 1 f16 / 2 bf16) with a per-row power-of-two
// factor in row_scale (kq_gemm.cu). lhs != nullptr: output row r is x row lhs[r / M] * M + r % M.
cudaError_t launch_convert_rows(int x_dtype, const void* x, long long x_row_stride, int K, long long rows,
                                const uint32_t* lhs, int M, void* xh, float* row_scale, cudaStream_t st);

// The general form of that pre-pass: optional expert order (output row r is entry order[r / M]), optional
// index array over units of lhs_div entries, optional fused h = silu(gate) * up over gate | up rows (glu).
cudaError_t launch_convert(int x_dtype, const void* x, long long x_row_stride, int K, long long rows, const int* order,
                           const uint32_t* lhs, int lhs_div, int M, void* xh, float* row_scale, int* yrow,
                           const int* n_valid, bool glu, cudaStream_t st);

// A whole mixture-of-experts SwiGLU block on the tile kernel (kq_gather.cu): one grouping, an expert-sorted fp16
// copy of the routed rows, gate | up product left in expert order, activation fused into the pre-pass of the
// down product, weighted sum per token. wgu: [E, 2F, rb_h] (gate rows then up rows); y: x dtype or float32.
bool moe_block_supported(int x_dtype, long long T, int k, int n_experts, int H, int F);
size_t moe_block_workspace_bytes(long long T, int k, int n_experts, int H, int F);
// scatter != nullptr (expert parallel over peer memory): instead of y, token g = w * tokens_per_rank + t leaves its
// partial row in slots[w][my_rank][t] - slots: device array of `world` pointers to the ranks' [world,
// tokens_per_rank, H] buffers (peer mappings) - unless none of its experts is local.
struct MoeScatter {
  void* const* slots;
  int my_rank;
  long long tokens_per_rank;
  bool slot_f32;
};
cudaError_t launch_moe_block(int codec, int x_dtype, const void* x, long long x_row_stride, const uint32_t* token_rows,
                             long long T, int H, const uint8_t* wgu, long long stride_gu, long long rb_h, int F,
                             const uint8_t* wd, long long stride_d, long long rb_f, int n_experts, const uint32_t* idx,
                             const float* scores, int k, void* y, bool y_f32, void* workspace, cudaStream_t st,
                             const MoeScatter* scatter = nullptr);
cudaError_t launch_moe_combine_scatter(int dtype, const void* d, const float* probs, const uint32_t* idx,
                                       uint32_t n_experts, long long tokens, int k, int H, long long tokens_per_rank,
                                       int my_rank, void* const* slots, bool slot_f32, cudaStream_t st);
cudaError_t launch_moe_slot_sum(int slot_dtype, const void* slots, const uint32_t* ids, const int* rank_lo, int world,
                                long long T, int k, int H, int y_dtype, void* y, cudaStream_t st);

// gather_qmm: device-side grouping by expert + the skinny-M kernel per group.
struct GatherLayout {
  size_t counts, offsets, task_base, cursor, n_tasks, order, tasks, total;
  long long max_tasks;
  // grouped tile-kernel regime only (grouped == true): fp16 copy of the sorted rows etc.
  bool grouped;
  size_t xh, row_scale, yrow, tiles;
  long long max_tiles;
};
// K > 0 lets the layout include the grouped regime's buffers when that regime would be chosen;
// K == 0 is the decode-only layout (the skinny kernel over task lists).
GatherLayout gather_layout(long long n_entries, int M, int n_experts, int K);
// Entries with rhs >= n_experts or lhs >= x_batch are skipped: their output rows stay unwritten.
cudaError_t launch_gather(int codec, int x_dtype, const void* x, long long x_batch, int M, int K, const uint8_t* w,
                          int n_experts, long long expert_stride, long long row_bytes, int N, const uint32_t* lhs,
                          const uint32_t* rhs, long long n_entries, void* y, void* workspace, bool allow_grouped,
                          cudaStream_t st);

// memset + histogram + scan + scatter of kq_gather.cu for other callers: see the definition.
cudaError_t launch_group_by_expert(const uint32_t* rhs, long long n, int n_experts, int unit, int* counts, int* cursor,
                                   int* offsets, int* unit_base, int* n_units, int* order, cudaStream_t st);

// The body of kq_gather_qmm; allow_grouped = false pins the decode regime (fixed-size scratch);
// builtin_scratch = true words a too-small workspace as the limit of the library's fixed array.
int gather_qmm_entry(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w, int n_experts,
                     long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                     const uint32_t* lhs_indices, const uint32_t* rhs_indices, long long n_entries, int transpose,
                     int rhs_sorted, void* y, void* workspace, size_t workspace_bytes, void* stream,
                     bool allow_grouped, bool builtin_scratch);

// Record `msg` as this thread's last error (what kq_last_error() returns) and
// hand back `code`; lets entry points that live outside kq_abi.cu report errors.
int set_error(int code, const char* msg);

// Host-side encoder (kq_quantize.cu): float weights -> wire bytes, byte-identical with the
// reference's CPU encoder for the thirteen codecs that have one here (quantize_supported).
bool quantize_supported(int codec);
void quantize_host(int codec, const void* w, int dtype, long long n_weights, long long K, const float* imatrix,
                   uint8_t* out, int threads);

// Elementwise stages of a mixture-of-experts SwiGLU block (kq_moe.cu). dtype 1 f16 / 2 bf16.
// q4_k, one or two dense activation rows, on the integer tensor pipe (kq_gemv_imma.cu).
bool gemv_imma_supported(int codec, int x_dtype, const GemvArgs& a);
cudaError_t launch_gemv_imma(int x_dtype, const GemvArgs& a, cudaStream_t st);

// row_expert != nullptr: rows with row_expert[r] >= n_experts are skipped. y_f32: y is float32.
cudaError_t launch_swiglu(int dtype, const void* gate, const void* up, long long in_row_stride, long long rows, int F,
                          void* out, const uint32_t* row_expert, uint32_t n_experts, cudaStream_t st);
cudaError_t launch_moe_combine(int dtype, const void* d, const float* probs, long long tokens, int k, int H, void* y,
                               bool y_f32, cudaStream_t st, const uint32_t* idx = nullptr, uint32_t n_experts = 0);

cudaError_t launch_qvm_gather(int codec, int x_dtype, const void* x, long long x_batch, void* y, const uint8_t* w,
                              int n_experts, long long expert_stride, long long row_bytes, int M, int N, int K,
                              const uint32_t* lhs, const uint32_t* rhs, long long n_entries, cudaStream_t st);
// transpose == 0 ([K, N] weights, rows quantized along N): streaming CUDA-core kernel (kq_qvm.cu).
cudaError_t launch_qvm(int codec, int x_dtype, const void* x, long long x_row_stride, void* y, long long y_row_stride,
                       const uint8_t* w, long long row_bytes, int M, int N, int K, cudaStream_t st);

}  // namespace kq
