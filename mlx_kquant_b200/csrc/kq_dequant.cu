// dequantize: GGUF wire bytes -> f32 / f16 / bf16, bit-exact with the
// reference's CPU decoders (src/kquant_dequantize.cpp:59-91 ->
// src/kquant_cpu_decode.cpp:1136-1207).
//
// HBM-bound streaming kernel. One CTA handles a tile of kTileW consecutive
// weights: the tile's wire bytes (tile_blocks * bytes_per_block, not a multiple
// of 16 for most codecs) are brought into shared memory with 16-byte loads that
// start at the 16-byte boundary below the tile, so global reads are fully
// coalesced whatever the block size; every thread then decodes eight
// consecutive weights at a time from shared memory and writes them with one or
// two 16-byte stores, consecutive threads writing consecutive chunks.
// Algorithmic bytes per weight: bytes_per_block / weights_per_block read plus
// sizeof(out type) written.
#include "kq_common.cuh"
#include "kq_launch.h"

namespace kq {

constexpr int kDqThreads = 256;
constexpr int kTileW = 8192;  // weights per CTA tile

template <typename T>
struct Pack8;
template <>
struct Pack8<float> {
  static __device__ __forceinline__ void store(float* o, const float (&v)[8], bool vec) {
    if (vec) {
      reinterpret_cast<float4*>(o)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(o)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) o[i] = v[i];
    }
  }
};
template <>
struct Pack8<__half> {
  static __device__ __forceinline__ void store(__half* o, const float (&v)[8], bool vec) {
    if (vec) {
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      *reinterpret_cast<uint4*>(o) = *reinterpret_cast<uint4*>(h);
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) o[i] = __float2half_rn(v[i]);
    }
  }
};
template <>
struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void store(__nv_bfloat16* o, const float (&v)[8], bool vec) {
    if (vec) {
      __nv_bfloat162 h[4];
#pragma unroll
      for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      *reinterpret_cast<uint4*>(o) = *reinterpret_cast<uint4*>(h);
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) o[i] = __float2bfloat16_rn(v[i]);
    }
  }
};

// A = alignment of every block start in SHARED memory, which equals the
// alignment of block starts in global memory because the staging copy keeps
// the address phase modulo 16.
template <int C, int A, typename T>
__global__ void __launch_bounds__(kDqThreads)
dequant_kernel(const uint8_t* __restrict__ w, T* __restrict__ out, long long n_blocks, int out_vec) {
  constexpr int WPB = wpb_of(C), BPB = bpb_of(C);
  constexpr int TB = kTileW / WPB;            // blocks per tile
  constexpr int OPB = WPB / 8;                // octets per block
  constexpr int kStage = TB * BPB + 32;       // tile bytes + phase + round-up
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* stage = smem;
  IqTables tabs = global_iq_tables();
  if constexpr (C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS) {
    tabs = stage_iq_tables(smem + ((kStage + 15) & ~15), threadIdx.x, kDqThreads);
  }

  const long long tile = blockIdx.x;
  const long long b0 = tile * TB;
  const int nb = (int)min((long long)TB, n_blocks - b0);
  if (nb <= 0) return;
  const uint8_t* src = w + b0 * BPB;
  const int bytes = nb * BPB;
  const uint8_t* w_end = w + n_blocks * BPB;

  int phase;
  if constexpr (A >= 2) {
    // 16-byte loads from the boundary at or below src; a chunk that would run
    // past the end of the wire buffer is copied byte by byte instead.
    phase = (int)(reinterpret_cast<uintptr_t>(src) & 15);
    const uint8_t* a0 = src - phase;
    const int nchunks = (phase + bytes + 15) >> 4;
    for (int c = threadIdx.x; c < nchunks; c += kDqThreads) {
      const uint8_t* g = a0 + 16 * c;
      if (g + 16 <= w_end) {
        reinterpret_cast<uint4*>(stage)[c] = *reinterpret_cast<const uint4*>(g);
      } else {
        for (int i = 0; i < 16; i++)
          if (g + i < w_end) stage[16 * c + i] = g[i];
      }
    }
  } else {
    phase = 0;
    for (int i = threadIdx.x; i < bytes; i += kDqThreads) stage[i] = src[i];
  }
  __syncthreads();

  const uint8_t* tile_s = stage + phase;
  T* out_t = out + b0 * WPB;
  const int n_oct = nb * OPB;
  if constexpr ((C == Q4_K || C == Q5_K) && A >= 4) {
    // The 6-bit scale / min pair of a sub-block serves 32 weights: unpack each pair once per tile
    // (one per thread: TB * 8 = 256 of them) instead of once per eight weights. Same arithmetic as
    // decode8<>: sc = d * scale, mn = dmin * min in fp32, v = sc * q - mn (sc * q is exact).
    float2* scmn = reinterpret_cast<float2*>(smem + ((kStage + 15) & ~15));
    for (int i = threadIdx.x; i < nb * 8; i += kDqThreads) {
      const uint8_t* blk = tile_s + (i >> 3) * BPB;
      const uint32_t h = ld32<A>(blk);
      const float d = __half2float(__ushort_as_half((unsigned short)(h & 0xffff)));
      const float dmin = __half2float(__ushort_as_half((unsigned short)(h >> 16)));
      uint32_t rsc, rmn;
      k4_scale_min(ld32<A>(blk + 4), ld32<A>(blk + 8), ld32<A>(blk + 12), i & 7, rsc, rmn);
      scmn[i] = make_float2(d * u2f(rsc), dmin * u2f(rmn));
    }
    __syncthreads();
    for (int o = threadIdx.x; o < n_oct; o += kDqThreads) {
      const int blk = o / OPB, j = o % OPB;
      const int sb = j >> 2, i0 = (j & 3) * 8;
      const float2 sm = scmn[blk * 8 + sb];
      const uint8_t* bp = tile_s + blk * BPB;
      const uint8_t* qs = bp + (C == Q4_K ? 16 : 48) + (sb >> 1) * 32 + i0;
      const int sh = (sb & 1) * 4;
      // four nibbles per word in the low halves of its bytes, then one conversion per byte
      uint32_t n0 = (ld32<A>(qs) >> sh) & 0x0f0f0f0fu, n1 = (ld32<A>(qs + 4) >> sh) & 0x0f0f0f0fu;
      if constexpr (C == Q5_K) {
        n0 |= ((ld32<A>(bp + 16 + i0) >> sb) & 0x01010101u) << 4;
        n1 |= ((ld32<A>(bp + 20 + i0) >> sb) & 0x01010101u) << 4;
      }
      float v[8];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        v[c] = sm.x * u2f((n0 >> (8 * c)) & 0xffu) - sm.y;
        v[c + 4] = sm.x * u2f((n1 >> (8 * c)) & 0xffu) - sm.y;
      }
      Pack8<T>::store(out_t + (size_t)o * 8, v, out_vec != 0);
    }
    return;
  }
  for (int o = threadIdx.x; o < n_oct; o += kDqThreads) {
    const int blk = o / OPB, j = o % OPB;
    float v[8];
    decode8<C, A>(tile_s + blk * BPB, j, v, tabs);
    Pack8<T>::store(out_t + (size_t)o * 8, v, out_vec != 0);
  }
}

template <int C, int A, typename T>
static cudaError_t launch_one(const uint8_t* w, void* out, long long n_blocks, cudaStream_t st) {
  constexpr int WPB = wpb_of(C), BPB = bpb_of(C), TB = kTileW / WPB;
  const long long tiles = (n_blocks + TB - 1) / TB;
  if (tiles == 0) return cudaSuccess;
  static_assert(kIqSmemBytes >= (kTileW / 256) * 8 * 8, "the k-quant scale table shares the IQ table area");
  const int smem = ((TB * BPB + 32 + 15) & ~15) + kIqSmemBytes;
  const int out_vec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  dequant_kernel<C, A, T><<<(unsigned)tiles, kDqThreads, smem, st>>>(w, static_cast<T*>(out), n_blocks, out_vec);
  return cudaGetLastError();
}

template <int C, int NAT>
static cudaError_t launch_codec(const uint8_t* w, void* out, long long n_blocks, int dtype, cudaStream_t st) {
  // Natural block alignment holds when the wire base is 16-byte aligned
  // (cudaMalloc / torch allocations are); otherwise take the byte-wise variant.
  const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0;
#define KQ_DQ(T)                                                   \
  return aligned ? launch_one<C, NAT, T>(w, out, n_blocks, st)     \
                 : launch_one<C, 1, T>(w, out, n_blocks, st)
  switch (dtype) {
    case F32: KQ_DQ(float);
    case F16: KQ_DQ(__half);
    case BF16: KQ_DQ(__nv_bfloat16);
  }
#undef KQ_DQ
  return cudaErrorInvalidValue;
}

cudaError_t launch_dequantize(int codec, const uint8_t* w, long long n_blocks, int dtype, void* out,
                              cudaStream_t st) {
  switch (codec) {
    case Q2_K: return launch_codec<Q2_K, 4>(w, out, n_blocks, dtype, st);
    case Q3_K: return launch_codec<Q3_K, 2>(w, out, n_blocks, dtype, st);
    case Q4_K: return launch_codec<Q4_K, 16>(w, out, n_blocks, dtype, st);
    case Q5_K: return launch_codec<Q5_K, 16>(w, out, n_blocks, dtype, st);
    case Q6_K: return launch_codec<Q6_K, 2>(w, out, n_blocks, dtype, st);
    case Q4_0: return launch_codec<Q4_0, 2>(w, out, n_blocks, dtype, st);
    case Q8_0: return launch_codec<Q8_0, 2>(w, out, n_blocks, dtype, st);
    case IQ4_NL: return launch_codec<IQ4_NL, 2>(w, out, n_blocks, dtype, st);
    case IQ4_XS: return launch_codec<IQ4_XS, 8>(w, out, n_blocks, dtype, st);
    case IQ2_XXS: return launch_codec<IQ2_XXS, 2>(w, out, n_blocks, dtype, st);
    case Q4_1: return launch_codec<Q4_1, 4>(w, out, n_blocks, dtype, st);
    case Q5_0: return launch_codec<Q5_0, 2>(w, out, n_blocks, dtype, st);
    case Q5_1: return launch_codec<Q5_1, 8>(w, out, n_blocks, dtype, st);
    case IQ3_XXS: return launch_codec<IQ3_XXS, 2>(w, out, n_blocks, dtype, st);
    case IQ3_S: return launch_codec<IQ3_S, 2>(w, out, n_blocks, dtype, st);
    case IQ2_XS: return launch_codec<IQ2_XS, 2>(w, out, n_blocks, dtype, st);
    case IQ2_S: return launch_codec<IQ2_S, 2>(w, out, n_blocks, dtype, st);
    case IQ1_S: return launch_codec<IQ1_S, 2>(w, out, n_blocks, dtype, st);
    case IQ1_M: return launch_codec<IQ1_M, 8>(w, out, n_blocks, dtype, st);
    case MXFP4: return launch_codec<MXFP4, 1>(w, out, n_blocks, dtype, st);
    case NVFP4: return launch_codec<NVFP4, 4>(w, out, n_blocks, dtype, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace kq
