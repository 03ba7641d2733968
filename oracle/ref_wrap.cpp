// TEST INFRASTRUCTURE - not part of the shipped library.
//
// Flat C entry points over the reference's own CPU codec library, which is
// compiled in place from the reference checkout (src/kquant_codec.cpp,
// src/kquant_cpu_decode.cpp, src/kquant_cpu_encode.cpp,
// src/kquant_iq_encode.cpp) next to this file into oracle/_ref/libkqref.so.
// Nothing here re-implements codec math: every function forwards to the
// reference template it names. Only tests, the smoke check and the benchmark's
// CPU-baseline leg load this library.
//
// dtype codes everywhere: 0 = float32, 1 = float16, 2 = bfloat16.
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "kquant_codec.h"
#include "kquant_cpu_decode.h"
#include "kquant_cpu_encode.h"
#include "mlx/types/half_types.h"

namespace mx = mlx::core;
using namespace mlx_kquant;

static thread_local std::string g_err;

static int fail(const std::exception& e) {
  g_err = e.what();
  return 1;
}

extern "C" {

const char* kqref_last_error() {
  return g_err.c_str();
}

// src/kquant_cpu_decode.cpp:912-914 (kq_cpu_threads)
int kqref_threads() {
  return kq_cpu_threads();
}

// src/kquant_codec.cpp:12-55 (registry, codec_names)
int kqref_codec_count() {
  return static_cast<int>(codec_names().size());
}

int kqref_codec_info(
    int idx,
    char* name,
    int name_cap,
    int* weights_per_block,
    int* bytes_per_block,
    int* bits,
    int* has_encode,
    int* requires_imatrix) {
  auto names = codec_names();
  if (idx < 0 || idx >= static_cast<int>(names.size())) {
    return 1;
  }
  const KQuantCodec* c = codec_by_name(names[idx]);
  std::strncpy(name, c->name.c_str(), name_cap - 1);
  name[name_cap - 1] = 0;
  *weights_per_block = c->weights_per_block;
  *bytes_per_block = c->bytes_per_block;
  *bits = c->bits;
  *has_encode = c->has_encode ? 1 : 0;
  *requires_imatrix = c->requires_imatrix ? 1 : 0;
  return 0;
}

// src/kquant_cpu_encode.cpp:824-859 (kquant_quantize_dispatch), float32 input.
int kqref_quantize_f32(
    const float* w,
    uint8_t* out,
    size_t num_weights,
    const char* codec,
    const float* imatrix,
    size_t K) {
  try {
    kquant_quantize_dispatch<float>(w, out, num_weights, codec, imatrix, K);
  } catch (const std::exception& e) {
    return fail(e);
  }
  return 0;
}

// src/kquant_cpu_decode.cpp:1190-1207 (kquant_dequantize_parallel)
int kqref_dequantize(
    const uint8_t* w,
    void* out,
    size_t num_weights,
    const char* codec,
    int dtype) {
  try {
    if (dtype == 0) {
      kquant_dequantize_parallel<float>(
          w, static_cast<float*>(out), num_weights, codec);
    } else if (dtype == 1) {
      kquant_dequantize_parallel<mx::float16_t>(
          w, static_cast<mx::float16_t*>(out), num_weights, codec);
    } else if (dtype == 2) {
      kquant_dequantize_parallel<mx::bfloat16_t>(
          w, static_cast<mx::bfloat16_t*>(out), num_weights, codec);
    } else {
      g_err = "bad dtype";
      return 1;
    }
  } catch (const std::exception& e) {
    return fail(e);
  }
  return 0;
}

// src/kquant_cpu_decode.cpp:1210-1359 (kquant_qmm_cpu)
int kqref_qmm(
    void* result,
    const void* x,
    const uint8_t* w,
    int M,
    int N,
    int K,
    int transpose_w,
    const char* codec,
    int dtype) {
  try {
    if (dtype == 0) {
      kquant_qmm_cpu<float>(
          static_cast<float*>(result),
          static_cast<const float*>(x),
          w, M, N, K, transpose_w != 0, codec);
    } else if (dtype == 1) {
      kquant_qmm_cpu<mx::float16_t>(
          static_cast<mx::float16_t*>(result),
          static_cast<const mx::float16_t*>(x),
          w, M, N, K, transpose_w != 0, codec);
    } else if (dtype == 2) {
      kquant_qmm_cpu<mx::bfloat16_t>(
          static_cast<mx::bfloat16_t*>(result),
          static_cast<const mx::bfloat16_t*>(x),
          w, M, N, K, transpose_w != 0, codec);
    } else {
      g_err = "bad dtype";
      return 1;
    }
  } catch (const std::exception& e) {
    return fail(e);
  }
  return 0;
}

// src/kquant_cpu_decode.cpp:1362-1527 (kquant_qmm_cpu_batch): n_tasks fused
// GEMVs, task t = { out[t] [m[t], N], x[t] [m[t], K], w[t] wire [N, K] }.
int kqref_qmm_batch(
    void* const* outs,
    const void* const* xs,
    const uint8_t* const* ws,
    const int* ms,
    int n_tasks,
    int N,
    int K,
    const char* codec,
    int dtype) {
  try {
    auto run = [&](auto* tag) {
      using T = std::remove_pointer_t<decltype(tag)>;
      std::vector<KQmvTask<T>> tasks(n_tasks);
      for (int t = 0; t < n_tasks; t++) {
        tasks[t].out = static_cast<T*>(outs[t]);
        tasks[t].x = static_cast<const T*>(xs[t]);
        tasks[t].w = ws[t];
        tasks[t].m = ms[t];
      }
      kquant_qmm_cpu_batch<T>(tasks.data(), n_tasks, N, K, codec);
    };
    if (dtype == 0) {
      run(static_cast<float*>(nullptr));
    } else if (dtype == 1) {
      run(static_cast<mx::float16_t*>(nullptr));
    } else if (dtype == 2) {
      run(static_cast<mx::bfloat16_t*>(nullptr));
    } else {
      g_err = "bad dtype";
      return 1;
    }
  } catch (const std::exception& e) {
    return fail(e);
  }
  return 0;
}

} // extern "C"
