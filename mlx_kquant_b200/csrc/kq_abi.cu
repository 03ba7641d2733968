// The extern "C" surface declared in include/kquant_b200.h: argument validation
// with the reference op layer's rules and message texts (src/kquant_ops.cpp),
// regime selection, and kernel launches. No allocation happens here.
#include <cstdarg>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/kquant_b200.h"
#include "kq_common.cuh"
#include "kq_launch.h"

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

int cuda_fail(const char* what, cudaError_t e) {
  return fail(KQ_ERR_CUDA, "[mlx_kquant] %s: CUDA error: %s", what, cudaGetErrorString(e));
}

int find_codec(const char* name) {
  if (name == nullptr) return -1;
  for (int i = 0; i < kq::NUM_CODECS; i++)
    if (std::strcmp(kq::kCodecs[i].name, name) == 0) return i;
  return -1;
}

bool dtype_ok(int d) { return d == KQ_F32 || d == KQ_F16 || d == KQ_BF16; }

}  // namespace

namespace kq {
int set_error(int code, const char* msg) {
  g_err = msg ? msg : "";
  return code;
}
}  // namespace kq

extern "C" {

const char* kq_last_error(void) { return g_err.c_str(); }

const char* kq_version(void) { return "kquant_b200 0.1 (sm_100a)"; }

int kq_codec_count(void) { return kq::NUM_CODECS; }

int kq_codec_info(int index, const char** name, int* wpb, int* bpb, int* bits, int* requires_imatrix) {
  if (index < 0 || index >= kq::NUM_CODECS) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant] codec index out of range");
  const kq::CodecInfo& c = kq::kCodecs[index];
  if (name) *name = c.name;
  if (wpb) *wpb = c.wpb;
  if (bpb) *bpb = c.bpb;
  if (bits) *bits = c.bits;
  if (requires_imatrix) *requires_imatrix = c.requires_imatrix;
  return KQ_OK;
}

int kq_codec_find(const char* name) { return find_codec(name); }

int kq_dequantize(const void* w, size_t w_bytes, const char* kquant_type, int out_dtype, void* out, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.dequantize] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_bytes % (size_t)c.bpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.dequantize] Last dim (%zu) must be a multiple of bytes_per_block (%d) for codec '%s'.",
                w_bytes, c.bpb, c.name);
  if (!dtype_ok(out_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.dequantize] Only real floating output dtypes are supported.");
  if (w_bytes == 0) return KQ_OK;
  if (w == nullptr || out == nullptr) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.dequantize] null pointer.");
  cudaError_t e = kq::launch_dequantize(ci, static_cast<const uint8_t*>(w), (long long)(w_bytes / c.bpb), out_dtype,
                                        out, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("dequantize", e);
  return KQ_OK;
}

int kq_quantize_cpu(const void* w, int w_dtype, long long n_weights, long long K, const char* kquant_type,
                    const float* imatrix, void* out, int threads) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantize] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (!dtype_ok(w_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantize] w must be a real floating tensor (float32, float16, or bfloat16).");
  if (K <= 0 || n_weights < 0 || n_weights % K != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantize] w must have at least 1 dimension.");
  if (K % c.wpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantize] Last dim (%lld) must be a multiple of weights_per_block (%d) for codec '%s'.", K,
                c.wpb, c.name);
  if (c.requires_imatrix && imatrix == nullptr)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantize] codec '%s' requires an importance matrix (imatrix); ggml rejects encoding it "
                "without one.",
                c.name);
  if (!kq::quantize_supported(ci))
    return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.quantize] the host encoder of codec '%s' is not built in this library.",
                c.name);
  if (n_weights == 0) return KQ_OK;
  if (w == nullptr || out == nullptr) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantize] null pointer.");
  kq::quantize_host(ci, w, w_dtype, n_weights, K, imatrix, static_cast<uint8_t*>(out), threads);
  return KQ_OK;
}

size_t kq_quantized_matmul_workspace_bytes(int x_dtype, long long rows, int K) {
  if (!dtype_ok(x_dtype) || rows <= 0 || K <= 0) return 0;
  return kq::gemm_workspace_bytes(x_dtype, rows, K);
}

int kq_quantized_matmul(const void* x, int x_dtype, long long rows, int K, long long x_row_stride, const void* w,
                        size_t w_row_bytes, int N, const char* kquant_type, int transpose, void* y,
                        long long y_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_row_bytes % (size_t)c.bpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul] KQuant weight last dim (%zu bytes) is not a whole number of %d-byte %s "
                "blocks.",
                w_row_bytes, c.bpb, c.name);
  if (!dtype_ok(x_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] Only real floating x dtypes are supported.");
  const long long wpr = (long long)(w_row_bytes / c.bpb) * c.wpb;
  // transpose: w is [N, bytes(K)]; otherwise w is [K, bytes(N)] and its row count is x's last dim by construction
  if (transpose ? wpr != K : wpr != N)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul] x last dim (%d) does not match the expanded quantized matrix inner dim "
                "(%lld) for codec '%s' with transpose=%s.",
                K, transpose ? wpr : (long long)K, c.name, transpose ? "true" : "false");
  if (rows < 0 || N < 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] negative size.");
  if (rows == 0 || N == 0) return KQ_OK;
  if (!x || !w || !y) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] null pointer.");
  const size_t xe = x_dtype == KQ_F32 ? 4 : 2;
  // the [N, K] kernels read activations sixteen bytes at a time; the [K, N] one reads them one by one
  if (transpose && ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((size_t)x_row_stride * xe) % 16 != 0))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] x rows must be 16-byte aligned.");
  if (rows > 16LL * 65535)
    return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.quantized_matmul] more than 1048560 rows in one call.");

  // Regimes: at most 16 rows -> the HBM-bound skinny kernel; more -> the tcgen05 tile kernel
  // (KQ_FORCE_SKINNY=1 keeps everything on the skinny kernel, an A/B lever).
  static const bool force_skinny = std::getenv("KQ_FORCE_SKINNY") != nullptr;
  cudaError_t e;
  if (!transpose) {
    if (rows > 0x7fffffffLL) return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.quantized_matmul] too many rows.");
    e = kq::launch_qvm(ci, x_dtype, x, x_row_stride, y, y_row_stride, static_cast<const uint8_t*>(w),
                       (long long)w_row_bytes, (int)rows, N, K, static_cast<cudaStream_t>(stream));
  } else if (rows > 16 && !force_skinny) {
    const size_t need = kq::gemm_workspace_bytes(x_dtype, rows, K);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
      return fail(KQ_ERR_INVALID_ARGUMENT,
                  "[mlx_kquant.quantized_matmul] workspace too small: %zu bytes given, %zu needed.", workspace_bytes,
                  need);
    if (need > 0 && (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
      return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul] workspace must be 256-byte aligned.");
    e = kq::launch_gemm(ci, x_dtype, x, x_row_stride, y, y_row_stride, static_cast<const uint8_t*>(w),
                        (long long)w_row_bytes, (int)rows, N, K, workspace, static_cast<cudaStream_t>(stream));
  } else {
    kq::GemvArgs a{};
    a.x = x;
    a.x_row_stride = x_row_stride;
    a.y = y;
    a.y_row_stride = y_row_stride;
    a.w = static_cast<const uint8_t*>(w);
    a.w_align16 = (reinterpret_cast<uintptr_t>(w) & 15) == 0 ? 1 : 0;
    a.row_bytes = (long long)w_row_bytes;
    a.N = N;
    a.K = K;
    a.M = (int)rows;
    // q4_k, 2-16 rows of bf16 / f32 activations, scratch at hand: exact fp16 copy of the rows (per-row
    // power-of-two factor), then the fp16 tensor-core decode kernel writing bf16(sum * factor) - several
    // times faster than the path that takes bf16 rows directly. Without scratch that path still serves.
    const size_t need = kq::gemm_workspace_bytes(x_dtype, rows, K);
    int eff_dtype = x_dtype;
    if (ci == kq::Q4_K && x_dtype != KQ_F16 && rows >= 2 && a.w_align16 && (w_row_bytes & 15) == 0 &&
        workspace != nullptr && workspace_bytes >= need && need > 0 &&
        (reinterpret_cast<uintptr_t>(workspace) & 255) == 0) {
      float* rs = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                           (((size_t)rows * (size_t)K * 2 + 255) & ~(size_t)255));
      e = kq::launch_convert_rows(x_dtype, x, x_row_stride, K, rows, nullptr, 1, workspace, rs,
                                  static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return cuda_fail("quantized_matmul", e);
      a.x = workspace;
      a.x_row_stride = K;
      a.out_bf16 = 1;
      a.row_scale = rs;
      eff_dtype = KQ_F16;
    }
    e = kq::launch_gemv(ci, eff_dtype, a, static_cast<cudaStream_t>(stream));
  }
  if (e != cudaSuccess) return cuda_fail("quantized_matmul", e);
  return KQ_OK;
}

static int swiglu_impl(const void* gate, const void* up, long long in_row_stride, long long rows, int F, int dtype,
                       void* out, const uint32_t* row_expert, int n_experts, void* stream) {
  if (dtype != KQ_F16 && dtype != KQ_BF16)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.swiglu] activations must be float16 or bfloat16.");
  if (rows < 0 || F < 0 || F % 8 != 0 || in_row_stride % 8 != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.swiglu] F and the row stride must be multiples of 8.");
  if (rows == 0 || F == 0) return KQ_OK;
  if (!gate || !up || !out || ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                                reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.swiglu] pointers must be non-null and 16-byte aligned.");
  cudaError_t e = kq::launch_swiglu(dtype, gate, up, in_row_stride, rows, F, out, row_expert,
                                    (uint32_t)(n_experts < 0 ? 0 : n_experts), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("swiglu", e);
  return KQ_OK;
}

int kq_swiglu(const void* gate, const void* up, long long in_row_stride, long long rows, int F, int dtype, void* out,
              void* stream) {
  return swiglu_impl(gate, up, in_row_stride, rows, F, dtype, out, nullptr, 0, stream);
}

int kq_swiglu_routed(const void* gate, const void* up, long long in_row_stride, long long rows, int F, int dtype,
                     void* out, const uint32_t* row_expert, int n_experts, void* stream) {
  if (!row_expert && rows > 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.swiglu] row_expert must be non-null.");
  return swiglu_impl(gate, up, in_row_stride, rows, F, dtype, out, row_expert, n_experts, stream);
}

static int combine_impl(const void* d, const float* probs, long long tokens, int k, int H, int dtype, void* y,
                        bool y_f32, void* stream) {
  if (dtype != KQ_F16 && dtype != KQ_BF16)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_combine] activations must be float16 or bfloat16.");
  if (tokens < 0 || k <= 0 || H < 0 || H % 8 != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_combine] H must be a multiple of 8 and k positive.");
  if (tokens == 0 || H == 0) return KQ_OK;
  if (!d || !probs || !y || ((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_combine] pointers must be non-null and 16-byte aligned.");
  cudaError_t e = kq::launch_moe_combine(dtype, d, probs, tokens, k, H, y, y_f32, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("moe_combine", e);
  return KQ_OK;
}

int kq_moe_combine(const void* d, const float* probs, long long tokens, int k, int H, int dtype, void* y,
                   void* stream) {
  return combine_impl(d, probs, tokens, k, H, dtype, y, false, stream);
}

int kq_moe_combine_f32(const void* d, const float* probs, long long tokens, int k, int H, int dtype, float* y,
                       void* stream) {
  return combine_impl(d, probs, tokens, k, H, dtype, y, true, stream);
}

int kq_quantized_matmul_qmv_bias(const void* x, int x_dtype, int K, const void* w, size_t w_row_bytes, int N,
                                 const char* kquant_type, const void* bias, void* y, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci != kq::Q8_0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul_qmv_bias] only kquant_type 'q8_0' is wired so far, got '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_row_bytes % (size_t)c.bpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul_qmv_bias] KQuant weight last dim (%zu bytes) is not a whole number of "
                "%d-byte %s blocks.",
                w_row_bytes, c.bpb, c.name);
  if ((long long)(w_row_bytes / c.bpb) * c.wpb != K)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul_qmv_bias] x last dim (%d) does not match the expanded quantized matrix "
                "inner dim (%lld) for codec '%s'.",
                K, (long long)(w_row_bytes / c.bpb) * c.wpb, c.name);
  if (!dtype_ok(x_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.quantized_matmul_qmv_bias] Only real floating x dtypes are supported.");
  if (N < 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul_qmv_bias] negative size.");
  if (N == 0) return KQ_OK;
  if (!x || !w || !y || !bias) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul_qmv_bias] null pointer.");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.quantized_matmul_qmv_bias] x must be 16-byte aligned.");
  kq::GemvArgs a{};
  a.x = x;
  a.x_row_stride = K;
  a.y = y;
  a.y_row_stride = N;
  a.w = static_cast<const uint8_t*>(w);
  a.w_align16 = (reinterpret_cast<uintptr_t>(w) & 15) == 0 ? 1 : 0;
  a.row_bytes = (long long)w_row_bytes;
  a.N = N;
  a.K = K;
  a.M = 1;
  a.bias = bias;
  cudaError_t e = kq::launch_gemv(ci, x_dtype, a, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("quantized_matmul_qmv_bias", e);
  return KQ_OK;
}

long long kq_expert_tile_map_capacity(long long rows, int n_experts) {
  if (rows < 1 || n_experts < 1) return 0;
  const long long present = rows < n_experts ? rows : n_experts;
  const long long cap = rows / 64 + present;
  return cap < 1 ? 1 : cap;
}

size_t kq_expert_tile_map_workspace_bytes(int n_experts) {
  return n_experts < 1 ? 0 : kq::tile_map_workspace_bytes(n_experts);
}

int kq_expert_tile_map(const uint32_t* indices, long long rows, int n_experts, uint32_t* map, uint32_t* count,
                       void* workspace, size_t workspace_bytes, void* stream) {
  if (rows < 1 || n_experts < 1)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.expert_tile_map] indices must be non-empty and n_experts positive.");
  if (rows >= (1LL << 31)) return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.expert_tile_map] too many rows.");
  if (!indices || !map || !count) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.expert_tile_map] null pointer.");
  const size_t need = kq::tile_map_workspace_bytes(n_experts);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 3) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.expert_tile_map] workspace too small: %zu bytes given, %zu needed.",
                workspace_bytes, need);
  cudaError_t e = kq::launch_tile_map(indices, rows, n_experts, map, count, workspace, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("expert_tile_map", e);
  return KQ_OK;
}

size_t kq_gather_qmm_seg_workspace_bytes(int x_dtype, long long rows, int K, int n_experts, long long map_tiles) {
  if (!dtype_ok(x_dtype) || rows <= 0 || K <= 0 || n_experts <= 0 || map_tiles <= 0) return 0;
  return kq::gather_seg_workspace_bytes(x_dtype, rows, K, n_experts, map_tiles);
}

int kq_gather_qmm_seg(const void* x, int x_dtype, long long rows, int K, const void* w, int n_experts,
                      long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                      const uint32_t* map, const uint32_t* count, long long map_tiles, void* y, void* workspace,
                      size_t workspace_bytes, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm_seg] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_row_bytes % (size_t)c.bpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm_seg] KQuant weight last dim (%zu bytes) is not a whole number of %d-byte %s "
                "blocks.",
                w_row_bytes, c.bpb, c.name);
  const long long wpr = (long long)(w_row_bytes / c.bpb) * c.wpb;
  if (wpr != K)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm_seg] x last dim (%d) does not match the expanded quantized row width (%lld) for "
                "codec '%s'.",
                K, wpr, c.name);
  if (!dtype_ok(x_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm_seg] Only real floating x dtypes are supported.");
  if (rows < 0 || N < 0 || n_experts < 1 || map_tiles < 1)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm_seg] map must be uint32 [n_tiles >= 1, 3] (expert, row_start, num_rows).");
  if (rows == 0 || N == 0) return KQ_OK;
  if (!x || !w || !y || !map || !count) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm_seg] null pointer.");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((size_t)K * (x_dtype == KQ_F32 ? 4 : 2)) % 16 != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm_seg] x rows must be 16-byte aligned.");
  if (rows >= (1LL << 31) || map_tiles + rows / 256 + 1 > 65535)
    return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.gather_qmm_seg] too many rows or map entries for one call.");
  const size_t need = kq::gather_seg_workspace_bytes(x_dtype, rows, K, n_experts, map_tiles);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm_seg] workspace too small or not 256-byte aligned: %zu bytes given, %zu needed.",
                workspace_bytes, need);
  cudaError_t e = kq::launch_gather_seg(ci, x_dtype, x, rows, K, static_cast<const uint8_t*>(w), n_experts,
                                        w_expert_stride_bytes, (long long)w_row_bytes, N, map, count, map_tiles, y,
                                        workspace, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("gather_qmm_seg", e);
  return KQ_OK;
}

size_t kq_moe_decode_workspace_bytes(long long n_entries, int n_experts, int N_mix) {
  if (n_entries <= KQ_MOE_DIRECT_MAX_ENTRIES || n_experts <= 0) return 0;
  return kq::moe_grouped_workspace_bytes(n_entries, n_experts, N_mix > 0 ? n_entries * (long long)N_mix * 2 : 0);
}

int kq_codec_has_moe_glu(const char* kquant_type) {
  const int ci = find_codec(kquant_type);
  return ci == kq::Q4_K ? 1 : 0;
}

static int moe_act_code(const char* act) {
  if (act == nullptr || std::strcmp(act, "silu") == 0) return 0;
  if (std::strcmp(act, "gelu") == 0) return 1;
  if (std::strcmp(act, "silu_limit") == 0) return 2;
  return -1;
}

int kq_moe_glu_gather(const void* x, int x_dtype, long long T, int K, const void* gate_w,
                      long long gate_expert_stride_bytes, const void* up_w, long long up_expert_stride_bytes,
                      size_t w_row_bytes, int N, int n_experts, const char* kquant_type, const uint32_t* indices, int R,
                      const char* act, float limit, void* y, void* workspace, size_t workspace_bytes, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_glu_gather_kq] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  const int a = moe_act_code(act);
  if (a < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_glu_gather_kq] act must be 'silu', 'gelu' or 'silu_limit' but got '%s'.", act);
  if (a == 2 && !(limit > 0.f))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_glu_gather_kq] act 'silu_limit' requires limit > 0.");
  if (w_row_bytes % (size_t)c.bpb != 0 || (long long)(w_row_bytes / c.bpb) * c.wpb != K)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_glu_gather_kq] x last dim (%d) does not match the expanded expert row (%lld weights).", K,
                (long long)(w_row_bytes / c.bpb) * c.wpb);
  if (K % 256 != 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_glu_gather_kq] requires K %% 256 == 0.");
  if (T < 0 || R < 0 || N < 0 || n_experts < 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_glu_gather_kq] negative size.");
  if (T == 0 || R == 0 || N == 0) return KQ_OK;
  if (!x || !gate_w || !up_w || !indices || !y)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_glu_gather_kq] null pointer.");
  if (T * (long long)R > 65535 ||
      !kq::moe_decode_supported(ci, x_dtype, K, (long long)w_row_bytes, x, gate_w, gate_expert_stride_bytes, up_w,
                                up_expert_stride_bytes))
    return fail(KQ_ERR_UNSUPPORTED,
                "[mlx_kquant.moe_glu_gather_kq] no fused kernel for this call (q4_k, float16 / bfloat16 rows, 16-byte "
                "aligned operands, at most 65535 entries): compose it from gather_qmm.");
  cudaError_t e;
  const long long n_entries = T * (long long)R;
  if (n_entries > KQ_MOE_DIRECT_MAX_ENTRIES && workspace != nullptr) {
    const size_t need = kq::moe_grouped_workspace_bytes(n_entries, n_experts, 0);
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
      return fail(KQ_ERR_INVALID_ARGUMENT,
                  "[mlx_kquant.moe_glu_gather_kq] workspace too small or not 256-byte aligned: %zu bytes given, %zu needed.",
                  workspace_bytes, need);
    if (kq::moe_grouped_supported(K, (long long)w_row_bytes, false)) {
      e = kq::launch_moe_glu_grouped(x_dtype, x, K, static_cast<const uint8_t*>(gate_w), gate_expert_stride_bytes,
                                     static_cast<const uint8_t*>(up_w), up_expert_stride_bytes, (long long)w_row_bytes, N,
                                     n_experts, indices, n_entries, R, a, limit, y, workspace,
                                     static_cast<cudaStream_t>(stream));
    } else {
      // rows too long for the grouped kernel's shared memory: per-entry kernel; the grouping is still left in
      // the workspace for a kq_gather_qmv_mix call that was told to reuse it
      e = kq::launch_moe_grouping_only(indices, n_entries, n_experts, workspace, static_cast<cudaStream_t>(stream));
      if (e == cudaSuccess)
        e = kq::launch_moe_glu(x_dtype, x, K, static_cast<const uint8_t*>(gate_w), gate_expert_stride_bytes,
                               static_cast<const uint8_t*>(up_w), up_expert_stride_bytes, (long long)w_row_bytes, N,
                               n_experts, indices, n_entries, R, a, limit, y, static_cast<cudaStream_t>(stream));
    }
  } else {
    e = kq::launch_moe_glu(x_dtype, x, K, static_cast<const uint8_t*>(gate_w), gate_expert_stride_bytes,
                           static_cast<const uint8_t*>(up_w), up_expert_stride_bytes, (long long)w_row_bytes, N,
                           n_experts, indices, n_entries, R, a, limit, y, static_cast<cudaStream_t>(stream));
  }
  if (e != cudaSuccess) return cuda_fail("moe_glu_gather_kq", e);
  return KQ_OK;
}

int kq_gather_qmv_mix(const void* x, int x_dtype, long long T, int S, int K, const void* w,
                      long long w_expert_stride_bytes, size_t w_row_bytes, int N, int n_experts, const char* kquant_type,
                      const uint32_t* indices, const float* scores, void* y, void* workspace, size_t workspace_bytes,
                      int reuse_grouping, void* stream) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmv_mix_ns_kq] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_row_bytes % (size_t)c.bpb != 0 || (long long)(w_row_bytes / c.bpb) * c.wpb != K)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmv_mix_ns_kq] x last dim (%d) does not match the expanded expert row (%lld weights).",
                K, (long long)(w_row_bytes / c.bpb) * c.wpb);
  if (T < 0 || S < 0 || N < 0 || n_experts < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmv_mix_ns_kq] negative size.");
  if (T == 0 || N == 0) return KQ_OK;
  if (!x || !w || !indices || !scores || !y)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmv_mix_ns_kq] null pointer.");
  if (T > 65535 || S == 0 || K % 256 != 0 ||
      !kq::moe_decode_supported(ci, x_dtype, K, (long long)w_row_bytes, x, w, w_expert_stride_bytes, nullptr, 0))
    return fail(KQ_ERR_UNSUPPORTED,
                "[mlx_kquant.gather_qmv_mix_ns_kq] no fused kernel for this call (q4_k, float16 / bfloat16 rows, "
                "K %% 256 == 0, 16-byte aligned operands, at most 65535 tokens): compose it from gather_qmm.");
  cudaError_t e;
  const long long n_entries = T * (long long)S;
  if (n_entries > KQ_MOE_DIRECT_MAX_ENTRIES && workspace != nullptr && N % 8 == 0 &&
      kq::moe_grouped_supported(K, (long long)w_row_bytes, true)) {
    const size_t need = kq::moe_grouped_workspace_bytes(n_entries, n_experts, n_entries * (long long)N * 2);
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
      return fail(KQ_ERR_INVALID_ARGUMENT,
                  "[mlx_kquant.gather_qmv_mix_ns_kq] workspace too small or not 256-byte aligned: %zu bytes given, %zu needed.",
                  workspace_bytes, need);
    e = kq::launch_moe_mix_grouped(x_dtype, x, K, static_cast<const uint8_t*>(w), w_expert_stride_bytes,
                                   (long long)w_row_bytes, N, n_experts, indices, scores, T, S, y, workspace,
                                   reuse_grouping != 0, static_cast<cudaStream_t>(stream));
  } else {
    e = kq::launch_moe_mix(x_dtype, x, K, static_cast<const uint8_t*>(w), w_expert_stride_bytes, (long long)w_row_bytes,
                           N, n_experts, indices, scores, T, S, y, static_cast<cudaStream_t>(stream));
  }
  if (e != cudaSuccess) return cuda_fail("gather_qmv_mix_ns_kq", e);
  return KQ_OK;
}

size_t kq_moe_block_workspace_bytes(long long T, int top_k, int n_experts, int H, int F) {
  return kq::moe_block_workspace_bytes(T, top_k, n_experts, H, F);
}

static int moe_block_entry(const void* x, int x_dtype, long long T, int H, long long x_row_stride,
                           const uint32_t* token_rows, const void* w_gate_up, long long gate_up_expert_stride_bytes,
                           size_t gate_up_row_bytes, int F, const void* w_down, long long down_expert_stride_bytes,
                           size_t down_row_bytes, int n_experts, const char* kquant_type, const uint32_t* indices,
                           const float* scores, int top_k, void* y, int y_dtype, void* workspace,
                           size_t workspace_bytes, void* stream, const kq::MoeScatter* scatter) {
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_swiglu_block] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (T < 0 || H < 0 || F < 0 || top_k < 0 || n_experts < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_swiglu_block] negative size.");
  if (gate_up_row_bytes % (size_t)c.bpb != 0 || (long long)(gate_up_row_bytes / c.bpb) * c.wpb != H)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_swiglu_block] x last dim (%d) does not match the expanded gate / up row (%lld weights).", H,
                (long long)(gate_up_row_bytes / c.bpb) * c.wpb);
  if (down_row_bytes % (size_t)c.bpb != 0 || (long long)(down_row_bytes / c.bpb) * c.wpb != F)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_swiglu_block] expert FFN width (%d) does not match the expanded down row (%lld weights).", F,
                (long long)(down_row_bytes / c.bpb) * c.wpb);
  if (y_dtype != x_dtype && y_dtype != KQ_F32)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_swiglu_block] y must have x's dtype or float32.");
  if (T == 0 || H == 0) return KQ_OK;
  if (!x || !w_gate_up || !w_down || !indices || !scores || (!y && !scatter))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_swiglu_block] null pointer.");
  const size_t xe = 2;
  if (!kq::moe_block_supported(x_dtype, T, top_k, n_experts, H, F) || (reinterpret_cast<uintptr_t>(x) & 15) != 0 ||
      ((size_t)x_row_stride * xe) % 16 != 0)
    return fail(KQ_ERR_UNSUPPORTED,
                "[mlx_kquant.moe_swiglu_block] the tile-kernel block takes float16 / bfloat16 rows (16-byte aligned), "
                "H and F multiples of 8 and at least 512 routed rows with 16 or more per expert on average: compose "
                "smaller calls from kq_moe_glu_gather + kq_gather_qmv_mix or kq_gather_qmm.");
  const size_t need = kq::moe_block_workspace_bytes(T, top_k, n_experts, H, F);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_swiglu_block] workspace too small or not 256-byte aligned: %zu bytes given, %zu needed.",
                workspace_bytes, need);
  cudaError_t e = kq::launch_moe_block(ci, x_dtype, x, x_row_stride, token_rows, T, H, static_cast<const uint8_t*>(w_gate_up),
                                       gate_up_expert_stride_bytes, (long long)gate_up_row_bytes, F,
                                       static_cast<const uint8_t*>(w_down), down_expert_stride_bytes,
                                       (long long)down_row_bytes, n_experts, indices, scores, top_k, y, y_dtype == KQ_F32,
                                       workspace, static_cast<cudaStream_t>(stream), scatter);
  if (e != cudaSuccess) return cuda_fail("moe_swiglu_block", e);
  return KQ_OK;
}

int kq_moe_swiglu_block(const void* x, int x_dtype, long long T, int H, long long x_row_stride,
                        const uint32_t* token_rows, const void* w_gate_up, long long gate_up_expert_stride_bytes,
                        size_t gate_up_row_bytes, int F, const void* w_down, long long down_expert_stride_bytes,
                        size_t down_row_bytes, int n_experts, const char* kquant_type, const uint32_t* indices,
                        const float* scores, int top_k, void* y, int y_dtype, void* workspace, size_t workspace_bytes,
                        void* stream) {
  return moe_block_entry(x, x_dtype, T, H, x_row_stride, token_rows, w_gate_up, gate_up_expert_stride_bytes,
                         gate_up_row_bytes, F, w_down, down_expert_stride_bytes, down_row_bytes, n_experts, kquant_type,
                         indices, scores, top_k, y, y_dtype, workspace, workspace_bytes, stream, nullptr);
}

int kq_moe_swiglu_block_scatter(const void* x, int x_dtype, long long T, int H, long long x_row_stride,
                                const uint32_t* token_rows, const void* w_gate_up, long long gate_up_expert_stride_bytes,
                                size_t gate_up_row_bytes, int F, const void* w_down, long long down_expert_stride_bytes,
                                size_t down_row_bytes, int n_experts, const char* kquant_type, const uint32_t* indices,
                                const float* scores, int top_k, void* const* slot_ptrs, int slot_dtype, int my_rank,
                                long long tokens_per_rank, void* workspace, size_t workspace_bytes, void* stream) {
  if (slot_ptrs == nullptr || tokens_per_rank <= 0 || my_rank < 0 || T % (tokens_per_rank > 0 ? tokens_per_rank : 1) != 0 ||
      (long long)my_rank >= T / (tokens_per_rank > 0 ? tokens_per_rank : 1))
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_swiglu_block_scatter] slot_ptrs must be a device array of one buffer per rank, T a "
                "whole number of tokens_per_rank and my_rank one of the T / tokens_per_rank ranks.");
  if (slot_dtype != x_dtype && slot_dtype != KQ_F32)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_swiglu_block_scatter] slots must have x's dtype or float32.");
  const kq::MoeScatter sc{slot_ptrs, my_rank, tokens_per_rank, slot_dtype == KQ_F32};
  return moe_block_entry(x, x_dtype, T, H, x_row_stride, token_rows, w_gate_up, gate_up_expert_stride_bytes,
                         gate_up_row_bytes, F, w_down, down_expert_stride_bytes, down_row_bytes, n_experts, kquant_type,
                         indices, scores, top_k, nullptr, slot_dtype, workspace, workspace_bytes, stream, &sc);
}

int kq_moe_sum_slots(const void* slots, int slot_dtype, const uint32_t* ids, const int* rank_lo, int world, long long T,
                     int top_k, int H, void* y, int y_dtype, void* stream) {
  if (!dtype_ok(slot_dtype) || !dtype_ok(y_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_sum_slots] Only real floating dtypes are supported.");
  if (T < 0 || top_k < 0 || H < 0 || world <= 0 || world > 32 || top_k > 256 || (H % 8) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_sum_slots] sizes: world 1..32, top_k <= 256, H a multiple of 8.");
  if (T == 0 || H == 0 || top_k == 0) return KQ_OK;
  if (!slots || !ids || !rank_lo || !y) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_sum_slots] null pointer.");
  cudaError_t e = kq::launch_moe_slot_sum(slot_dtype, slots, ids, rank_lo, world, T, top_k, H, y_dtype, y,
                                          static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("moe_sum_slots", e);
  return KQ_OK;
}

// ---- buffers shared between the processes of one node (one process per GPU) ---------------------------------
// Plain cudaMalloc + CUDA IPC: the owner creates the buffer and hands the 64-byte handle to its peers (any host
// channel); a peer opens it ON ITS OWN DEVICE with lazy peer access, so its kernels can store into the owner's
// memory over NVLink without a context on the owner's GPU.
int kq_peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr || bytes == 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.peer_buffer_create] null pointer or zero size.");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_fail("peer_buffer_create", e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail("peer_buffer_create", e);
  }
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return KQ_OK;
}

int kq_peer_buffer_open(const unsigned char* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.peer_buffer_open] null pointer.");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail("peer_buffer_open", e);
  *ptr = p;
  return KQ_OK;
}

int kq_peer_buffer_close(void* ptr) {
  if (ptr == nullptr) return KQ_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return cuda_fail("peer_buffer_close", e);
  return KQ_OK;
}

int kq_peer_buffer_destroy(void* ptr) {
  if (ptr == nullptr) return KQ_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return cuda_fail("peer_buffer_destroy", e);
  return KQ_OK;
}

int kq_peer_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return KQ_OK;
  if (dst == nullptr || src == nullptr) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.peer_copy_async] null pointer.");
  // one copy per call, device to device (the destination may be another GPU's memory opened with
  // kq_peer_buffer_open): the copy engines move it, no SM is involved
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("peer_copy_async", e);
  return KQ_OK;
}

int kq_moe_router_topk(const void* logits, int dtype, long long T, int E, int top_k, int norm_topk_prob, int shared_gate,
                       const float* per_expert_scale, const float* bias, const char* scoring, float scale,
                       uint32_t* indices, float* scores, void* stream) {
  int sc = -1;
  if (scoring == nullptr || std::strcmp(scoring, "softmax") == 0) sc = 0;
  else if (std::strcmp(scoring, "sqrtsoftplus") == 0) sc = 1;
  if (sc < 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_router_topk] unknown scoring '%s'.", scoring);
  if (!dtype_ok(dtype)) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_router_topk] logits must be floating.");
  if (E < 1 || E > 1024 || top_k < 1 || top_k > 16 || top_k > E)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_router_topk] needs 1 <= top_k <= min(E, 16) and E <= 1024.");
  if (sc == 1 && !norm_topk_prob)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.moe_router_topk] sqrtsoftplus has no global normaliser: norm_topk_prob is required.");
  if (T < 0 || T > 0x7fffffff) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_router_topk] bad token count.");
  if (T == 0) return KQ_OK;
  if (!logits || !indices || !scores) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.moe_router_topk] null pointer.");
  cudaError_t e = kq::launch_router_topk(logits, dtype, (int)T, E, top_k, norm_topk_prob ? 1 : 0, shared_gate ? 1 : 0, sc,
                                         per_expert_scale, bias, scale, indices, scores,
                                         static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("moe_router_topk", e);
  return KQ_OK;
}

int kq_device_error_flags(int* flags, int clear) {
  if (flags == nullptr) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant] kq_device_error_flags: null pointer.");
  cudaError_t e = kq::read_device_error(flags, clear != 0);
  if (e != cudaSuccess) return cuda_fail("device_error_flags", e);
  return KQ_OK;
}

size_t kq_gather_qmm_workspace_bytes(long long n_entries, int M, int n_experts, int K) {
  if (n_entries < 0 || M <= 0 || n_experts <= 0 || K < 0) return 0;
  return kq::gather_layout(n_entries, M, n_experts, K).total;
}

int kq_gather_qmm(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w, int n_experts,
                  long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                  const uint32_t* lhs_indices, const uint32_t* rhs_indices, long long n_entries, int transpose,
                  int rhs_sorted, void* y, void* workspace, size_t workspace_bytes, void* stream) {
  return kq::gather_qmm_entry(x, x_dtype, x_batch, M, K, w, n_experts, w_expert_stride_bytes, w_row_bytes, N,
                              kquant_type, lhs_indices, rhs_indices, n_entries, transpose, rhs_sorted, y, workspace,
                              workspace_bytes, stream, /*allow_grouped=*/true, /*builtin_scratch=*/false);
}

}  // extern "C"

namespace kq {
int gather_qmm_entry(const void* x, int x_dtype, long long x_batch, int M, int K, const void* w, int n_experts,
                     long long w_expert_stride_bytes, size_t w_row_bytes, int N, const char* kquant_type,
                     const uint32_t* lhs_indices, const uint32_t* rhs_indices, long long n_entries, int transpose,
                     int rhs_sorted, void* y, void* workspace, size_t workspace_bytes, void* stream,
                     bool allow_grouped, bool builtin_scratch) {
  (void)rhs_sorted;
  const int ci = find_codec(kquant_type);
  if (ci < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] Unknown kquant_type: '%s'.",
                kquant_type ? kquant_type : "(null)");
  const kq::CodecInfo& c = kq::kCodecs[ci];
  if (w_row_bytes % (size_t)c.bpb != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm] KQuant weight last dim (%zu bytes) is not a whole number of %d-byte %s blocks.",
                w_row_bytes, c.bpb, c.name);
  if (!dtype_ok(x_dtype))
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] Only real floating x dtypes are supported.");
  const long long wpr = (long long)(w_row_bytes / c.bpb) * c.wpb;
  if (!transpose) {
    // [K, N] expert matrices (rows quantized along N): the streaming kernel of kq_qvm.cu over the entries
    if (wpr != N)
      return fail(KQ_ERR_INVALID_ARGUMENT,
                  "[mlx_kquant.gather_qmm] x last dim (%d) does not match the expanded quantized matrix inner dim (%d) "
                  "for codec '%s' with transpose=false.",
                  K, K, c.name);
    if (n_entries < 0 || M < 0 || N < 0 || K < 0 || n_experts < 0)
      return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] negative size.");
    if (n_entries == 0 || M == 0 || N == 0) return KQ_OK;
    if (n_experts == 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] no expert matrices.");
    if (!x || !w || !y || !lhs_indices || !rhs_indices)
      return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] null pointer.");
    cudaError_t et = kq::launch_qvm_gather(ci, x_dtype, x, x_batch, y, static_cast<const uint8_t*>(w), n_experts,
                                           w_expert_stride_bytes, (long long)w_row_bytes, M, N, K, lhs_indices,
                                           rhs_indices, n_entries, static_cast<cudaStream_t>(stream));
    if (et != cudaSuccess) return cuda_fail("gather_qmm", et);
    return KQ_OK;
  }
  if (wpr != K)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm] x last dim (%d) does not match the expanded quantized matrix inner dim (%lld) "
                "for codec '%s' with transpose=true.",
                K, wpr, c.name);
  if (n_entries < 0 || M < 0 || N < 0 || n_experts < 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] negative size.");
  if (n_entries == 0 || M == 0 || N == 0) return KQ_OK;
  if (n_experts == 0) return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] no expert matrices.");
  if (!x || !w || !y || !lhs_indices || !rhs_indices)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] null pointer.");
  const size_t xe = x_dtype == KQ_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((size_t)K * xe) % 16 != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] x rows must be 16-byte aligned.");
  // rows are numbered with 32-bit integers on the device
  if (n_entries > (long long)INT_MAX / (M > 0 ? M : 1))
    return fail(KQ_ERR_UNSUPPORTED, "[mlx_kquant.gather_qmm] n_entries * M = %lld rows exceed 2^31 - 1; split the call.",
                n_entries * (long long)M);
  const size_t need = kq::gather_layout(n_entries, M, n_experts, allow_grouped ? K : 0).total;
  if (builtin_scratch && need > workspace_bytes)
    return fail(KQ_ERR_INVALID_ARGUMENT,
                "[mlx_kquant.gather_qmm] problem too large for the built-in scratch: needs %zu bytes, the fixed array "
                "holds %zu; use kq_gather_qmm with a caller-provided workspace.",
                need, workspace_bytes);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] workspace too small: %zu bytes given, %zu needed.",
                workspace_bytes, need);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(KQ_ERR_INVALID_ARGUMENT, "[mlx_kquant.gather_qmm] workspace must be 256-byte aligned.");
  cudaError_t e = kq::launch_gather(ci, x_dtype, x, x_batch, M, K, static_cast<const uint8_t*>(w), n_experts,
                                    w_expert_stride_bytes, (long long)w_row_bytes, N, lhs_indices, rhs_indices,
                                    n_entries, y, workspace, allow_grouped, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("gather_qmm", e);
  return KQ_OK;
}
}  // namespace kq
