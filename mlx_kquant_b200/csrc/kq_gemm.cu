// Prefill quantized matmul (M > 16): y[M, N] = x[M, K] . dequant(W)^T on the
// 5th-generation tensor cores, replacing the reference's dequantize-then-GEMM CPU
// path (src/kquant_cpu_decode.cpp:1299-1352) and its Metal tile kernels
// (src/kquant_matmul.cpp:313-527).
//
// One CTA computes a (128*MT) x 128 output tile, MT in {1, 2, 4}. A weight tile
// costs CUDA-core work to make, an activation tile costs nothing (TMA), so the
// dequantized weight tile of each K-step (64 wide: one 128-byte swizzle row of
// fp16) is multiplied against MT activation tiles: at MT = 4 the tensor pipe has
// 1024 cycles of work per weight tile and the producers keep up.
//   warps 0-7  weight producers: wire bytes -> fp16 in registers -> the
//              128B-swizzled K-major tile of a 3-deep ring; fence.proxy.async +
//              mbarrier arrive. Two threads per weight row, 32 weights each.
//   warp 8     one thread issues tcgen05.mma (M=128, N=128, K=16, kind::f16, fp32
//              accumulators in tensor memory: MT x 128 columns); tcgen05.commit
//              hands activation slots and weight stages back.
//   warp 9     one thread streams activation tiles [128 rows x 64] with TMA
//              (cp.async.bulk.tensor.2d, 128B swizzle, zero fill past M and K)
//              into an 8-slot ring, two K-steps ahead of the MMAs.
//   warps 0-7  epilogue: tcgen05.ld the accumulators (thread = output row, warps
//              4-7 take the upper half of the columns), round once, 32-byte stores.
// Both operands are fp16: rounding a dequantized weight to bf16 alone would cost
// 1.6e-3 relative error and break the 2e-3 budget together with a bf16 output
// (fp16 costs 3e-4), and kind::f16 rejects a bf16 A operand next to an fp16 B
// operand (illegal instruction on sm_100a), so bf16 / f32 activations are first
// converted to fp16 by convert_x_kernel - exactly, with a per-row power-of-two
// factor that the epilogue undoes.
// q4_k weights are built exactly up to one rounding: sc*q is an exact integer in
// fp16, d is an fp16 value already, so w = fma(sc*q, d, -fp16(dmin*mn)).
//
// Every mbarrier wait is bounded (2 s of %globaltimer): on expiry the CTA raises
// a flag in g_kq_device_error, stops issuing work, frees its tensor memory and
// returns, so a logic error can never leave the GPU spinning.
#include <cooperative_groups.h>
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_launch.h"
#include "kq_tcgen05.cuh"

namespace cg = cooperative_groups;

namespace kq {

constexpr int kBN = 128;
constexpr int kBK = 64;
// weight-tile ring: three stages (two next to a raw-block ring of a 256-column tile, which fills shared memory;
// that combination was measured slower than per-thread loads and is not dispatched)
// KS: 64-deep K-steps per stage. KS = 2 (the 128 x 128 tile of small M): a stage is 128 deep, so every wait, fence,
// arrive and commit is paid once per two K-steps - at small M those handshakes, not the tensor pipe, set the pace.
__host__ __device__ constexpr int b_stages(int NB, bool RAW, int KS = 1) { return ((RAW && NB == 2) || KS == 2) ? 2 : 3; }
// Eight producer warps, then the MMA issuer warp(s) and one TMA warp. A 128-row weight tile has two producer
// threads per row (32 weights each per K-step), a 256-row tile one (sixteen producer warps were measured
// slower: 0.55 against 0.71 of the tensor peak at M = 8192).
__host__ __device__ constexpr int producer_threads(int) { return 256; }
// One thread issues the MMAs of an accumulator row block; a tcgen05.mma costs its issuing thread ~75 cycles
// (measured) against 128 cycles of tensor-pipe time, and every K-step adds barrier waits and commits, so ONE
// issuer for two or four row blocks leaves the pipe idle half of the time: tiles with two or more row blocks
// have two issuer warps (row blocks h = 0, 2 and h = 1, 3).
__host__ __device__ constexpr int mma_warps(int MT) { return MT >= 2 ? 2 : 1; }
__host__ __device__ constexpr int gemm_threads(int MT, int NB) { return producer_threads(NB) + 32 * (mma_warps(MT) + 1); }
// activation-tile ring; the raw-block ring of the small-M kernels takes the room of four slots
__host__ __device__ constexpr int a_slots(int MT, int NB, bool RAW = false, int KS = 1) {
  return KS == 2 ? 2 : (NB == 2 ? (RAW ? 5 : 6) : (MT == 1 || RAW ? 4 : 8));
}
constexpr int kTileBytes = 128 * 128;  // 128 rows x 64 16-bit elements

__device__ int g_kq_device_error = 0;
#ifdef KQ_GEMM_TRACE
// cycles summed over CTAs: [0] MMA warp waiting for weight tiles, [1] for activation tiles, [2] MMA loop,
// [3] loader waiting for free slots, [4] producer (thread 0) waiting for free stages, [5] producing, [6] CTAs,
// [7] epilogue
__device__ unsigned long long g_gemm_trace[12];  // [8] CTA lifetime per tile, [9] start of the tile to the first K-step
#define KQ_TR(...) __VA_ARGS__
#else
#define KQ_TR(...)
#endif

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  return mbar_wait_err(bar, parity, abort_flag, code, &g_kq_device_error);
}

__device__ __forceinline__ uint32_t pack_h2f(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, __half2 b, __half2 c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), b, c);
  return *reinterpret_cast<uint32_t*>(&r);
}

constexpr int kTileGridCap = 256;  // grid.y of the grouped kernel, see launch_gemm_tiles
struct GemmTile {
  int expert, row_start, rows, pad;
};

struct GemmArgs {
  const void* x;
  long long x_row_stride;
  void* y;
  long long y_row_stride;
  const uint8_t* w;
  long long row_bytes;
  int M, N, K;
  const float* row_scale;  // per-row factor applied in the epilogue, or nullptr
  // grouped (mixture-of-experts) mode: CTA row tiles come from a device-built list
  const GemmTile* tiles;       // nullptr = dense
  const int* n_tiles_dev;      // valid entries of `tiles`
  long long w_expert_stride;   // bytes between expert matrices
  const int* yrow;             // output row of each (expert-sorted) activation row
};

// ---- weight producers: 64 consecutive weights of one row -> eight swizzled 16-byte chunks
// hh = 0 / 1: which 32 of the 64 weights this thread makes (chunks 4hh .. 4hh+3)
template <int C, int A>
__device__ __forceinline__ void produce_w_generic(const uint8_t* row, int kb, int K, uint8_t* dst_row, int r, int hh,
                                                  const IqTables& tabs) {
  constexpr int BPB = bpb_of(C);
#pragma unroll 2
  for (int c = 4 * hh; c < 4 * hh + 4; c++) {
    const int k = kb * kBK + c * 8;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (k < K) {
      float v[8];
      decode8<C, A>(row + block_of<C>(k) * BPB, octet_of<C>(k), v, tabs);
      out = make_uint4(pack_h2f(v[0], v[1]), pack_h2f(v[2], v[3]), pack_h2f(v[4], v[5]), pack_h2f(v[6], v[7]));
    }
    *reinterpret_cast<uint4*>(dst_row + ((c ^ (r & 7)) << 4)) = out;
  }
}

// q6_k (src/kquant_cpu_decode.cpp:238-280): K-chunk kb is weights 64 p .. 64 p + 63 of superblock kb >> 2,
// p = kb & 3: half hf = p >> 1, quarters qd = 2 (p & 1) + hh for the row's two threads. Thread hh makes the 32
// weights l = 0..31 of its quarter: q = nibble of ql[64 hf + 32 hh + l] (high nibbles for the upper two
// quarters) | two bits 2 qd of qh[32 hf + l] << 4. The six-bit value becomes fp16 through the 1024 + q bit
// pattern, q - 32 is exact, and the weight is (q - 32) * fp16(d * scale): two roundings (scale, product)
// instead of the generic path's one, 2^-10 at worst, for a third of the instructions.
template <int A>
__device__ __forceinline__ void produce_w_q6k(const uint8_t* row, int kb, uint8_t* dst_row, int r, int hh) {
  const uint8_t* blk = row + (long long)(kb >> 2) * 210;
  const int p = kb & 3, hf = p >> 1, qd = 2 * (p & 1) + hh;
  const float d = ldf16<A>(blk + 208);
  const int is = 8 * hf + 2 * qd;
  const uint32_t sc2 = (uint32_t)blk[192 + is] | ((uint32_t)blk[193 + is] << 8);
  const __half2 sA = __float2half2_rn(d * (float)(int)(int8_t)(sc2 & 0xffu));
  const __half2 sB = __float2half2_rn(d * (float)(int)(int8_t)(sc2 >> 8));
  const __half2 k1056 = __float2half2_rn(1056.f);
  const uint8_t* ql = blk + 64 * hf + 32 * hh;
  const uint8_t* qh = blk + 128 + 32 * hf;
  const int nsh = (qd & 2) ? 4 : 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t L = ld32<A>(ql + 8 * c + 4 * h), H = ld32<A>(qh + 8 * c + 4 * h);
      const uint32_t hb = (qd < 2) ? (H << (4 - 2 * (qd & 1))) : (H >> (2 * (qd & 1)));
      const uint32_t q4 = ((L >> nsh) & 0x0f0f0f0fu) | (hb & 0x30303030u);
      const __half2 s = c < 2 ? sA : sB;
      const uint32_t m0 = __byte_perm(q4, 0x64646464u, 0x4140), m1 = __byte_perm(q4, 0x64646464u, 0x4342);
      const __half2 w0 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&m0), k1056), s);
      const __half2 w1 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&m1), k1056), s);
      o[2 * h] = *reinterpret_cast<const uint32_t*>(&w0);
      o[2 * h + 1] = *reinterpret_cast<const uint32_t*>(&w1);
    }
    *reinterpret_cast<uint4*>(dst_row + (((c + 4 * hh) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The same producer with its bytes requested one K-step ahead (as the q4_k producer does): rows that start on
// 8-byte boundaries (base pointer and row bytes multiples of 8, i.e. K a multiple of 1024) read the 32 ql bytes
// and the 32 qh bytes of a thread's quarter as five aligned 8-byte loads each - the quarter starts 0, 2, 4 or 6
// bytes into its window, the same for every row of the tile - and funnel-shift them into place. The version
// above issues 35 two-byte loads per K-step and uses each at once, so every K-step waits out a load latency.
struct Q6kTileLoad {
  uint2 ql[5], qh[5];
  uint32_t sc2, dbits;
};
__device__ __forceinline__ Q6kTileLoad q6k_tile_load(const uint8_t* row, int kb, int hh) {
  const uint8_t* blk = row + (long long)(kb >> 2) * 210;
  const int p = kb & 3, hf = p >> 1, qd = 2 * (p & 1) + hh;
  const uint8_t* ql = blk + 64 * hf + 32 * hh;
  const uint8_t* qh = blk + 128 + 32 * hf;
  const uint2* al = reinterpret_cast<const uint2*>(reinterpret_cast<uintptr_t>(ql) & ~(uintptr_t)7);
  const uint2* ah = reinterpret_cast<const uint2*>(reinterpret_cast<uintptr_t>(qh) & ~(uintptr_t)7);
  Q6kTileLoad l;
#pragma unroll
  for (int i = 0; i < 5; i++) {
    l.ql[i] = __ldg(al + i);
    l.qh[i] = __ldg(ah + i);
  }
  l.sc2 = __ldg(reinterpret_cast<const unsigned short*>(blk + 192 + 8 * hf + 2 * qd));
  l.dbits = __ldg(reinterpret_cast<const unsigned short*>(blk + 208));
  return l;
}
// eight consecutive 32-bit words starting `phase` bytes (0, 2, 4, 6) into a 40-byte window
__device__ __forceinline__ void q6k_window(const uint2 (&win)[5], int phase, uint32_t (&out)[8]) {
  const uint32_t w[10] = {win[0].x, win[0].y, win[1].x, win[1].y, win[2].x, win[2].y, win[3].x, win[3].y, win[4].x, win[4].y};
  const bool up = (phase & 4) != 0;
  const uint32_t sh = (phase & 2) * 8;
  uint32_t v[9];
#pragma unroll
  for (int i = 0; i < 9; i++) v[i] = up ? w[i + 1] : w[i];
#pragma unroll
  for (int i = 0; i < 8; i++) out[i] = __funnelshift_r(v[i], v[i + 1], sh);
}
__device__ __forceinline__ void produce_w_q6k_pre(const Q6kTileLoad& l, const uint8_t* row, int kb, uint8_t* dst_row,
                                                  int r, int hh) {
  const int p = kb & 3, hf = p >> 1, qd = 2 * (p & 1) + hh;
  // phases of the two windows: the row base is 8-byte aligned, so they follow from the offsets alone
  const int off = (kb >> 2) * 210;
  const int phl = (int)((reinterpret_cast<uintptr_t>(row) + off + 64 * hf + 32 * hh) & 7);
  const int phh = (int)((reinterpret_cast<uintptr_t>(row) + off + 128 + 32 * hf) & 7);
  uint32_t L[8], H[8];
  q6k_window(l.ql, phl, L);
  q6k_window(l.qh, phh, H);
  const float d = __half2float(__ushort_as_half((unsigned short)l.dbits));
  const __half2 sA = __float2half2_rn(d * (float)(int)(int8_t)(l.sc2 & 0xffu));
  const __half2 sB = __float2half2_rn(d * (float)(int)(int8_t)((l.sc2 >> 8) & 0xffu));
  const __half2 k1056 = __float2half2_rn(1056.f);
  const int nsh = (qd & 2) ? 4 : 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t Lw = L[2 * c + h], Hw = H[2 * c + h];
      const uint32_t hb = (qd < 2) ? (Hw << (4 - 2 * (qd & 1))) : (Hw >> (2 * (qd & 1)));
      const uint32_t q4 = ((Lw >> nsh) & 0x0f0f0f0fu) | (hb & 0x30303030u);
      const __half2 s = c < 2 ? sA : sB;
      const uint32_t m0 = __byte_perm(q4, 0x64646464u, 0x4140), m1 = __byte_perm(q4, 0x64646464u, 0x4342);
      const __half2 w0 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&m0), k1056), s);
      const __half2 w1 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&m1), k1056), s);
      o[2 * h] = *reinterpret_cast<const uint32_t*>(&w0);
      o[2 * h + 1] = *reinterpret_cast<const uint32_t*>(&w1);
    }
    *reinterpret_cast<uint4*>(dst_row + (((c + 4 * hh) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__device__ __forceinline__ uint32_t two_bytes_to_h2(uint32_t two_bytes) {
  const uint32_t m = (two_bytes & 0xffu) | ((two_bytes & 0xff00u) << 8) | 0x64006400u;
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&m), __float2half2_rn(1024.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// q4_k: K-chunk kb is sub-block pair p = kb & 3 of superblock kb >> 2
// (src/kquant_cpu_decode.cpp:177-202); thread hh of the row makes sub-block 2p + hh,
// i.e. the low (hh = 0) or high (hh = 1) nibbles of the pair's 32 quant bytes.
struct Q4kTileLoad {
  uint4 hdr, q0, q1;
};
__device__ __forceinline__ Q4kTileLoad q4k_tile_load(const uint8_t* row, int kb) {
  const uint4* blk = reinterpret_cast<const uint4*>(row + (long long)(kb >> 2) * 144);
  const int p = kb & 3;
  Q4kTileLoad l;
  l.hdr = __ldg(blk);
  l.q0 = __ldg(blk + 1 + 2 * p);
  l.q1 = __ldg(blk + 2 + 2 * p);
  return l;
}
__device__ __forceinline__ void produce_w_q4k(const Q4kTileLoad& l, int kb, uint8_t* dst_row, int r, int hh) {
  const int p = kb & 3;
  const uint4 hdr = l.hdr;
  const int sh = 16 * (p & 1);
  const uint32_t u0 = (hdr.y >> sh) & 0xffffu, u1 = (hdr.z >> sh) & 0xffffu, u2 = (hdr.w >> sh) & 0xffffu;
  uint32_t sc2, mn2;
  if (p < 2) {
    sc2 = u0 & 0x3f3fu;
    mn2 = u1 & 0x3f3fu;
  } else {
    sc2 = (u2 & 0x0f0fu) | ((u0 >> 2) & 0x3030u);
    mn2 = ((u2 >> 4) & 0x0f0fu) | ((u1 >> 2) & 0x3030u);
  }
  const uint32_t scb = (sc2 >> (8 * hh)) & 0xffu, mnb = (mn2 >> (8 * hh)) & 0xffu;
  const uint32_t scm = scb | (scb << 16) | 0x64006400u;  // half2(1024 + sc, 1024 + sc)
  const __half2 sc = __hsub2(*reinterpret_cast<const __half2*>(&scm), __float2half2_rn(1024.f));
  const __half2 off = __hmul2(sc, __float2half2_rn(-1024.f));
  const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
  const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
  const __half2 ndm = __float2half2_rn(-(dmin * (float)mnb));
  const uint32_t w[8] = {l.q0.x, l.q0.y, l.q0.z, l.q0.w, l.q1.x, l.q1.y, l.q1.z, l.q1.w};
  const int shn = 4 * hh;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t n4 = (w[2 * c + h] >> shn) & 0x0f0f0f0fu;
      // (1024 + q) pairs in natural order, then sc*q exactly, then one rounding: fma(sc*q, d, -dmin*mn)
      o[2 * h] = hfma2_bits(hfma2_bits(__byte_perm(n4, 0x64646464u, 0x4140), sc, off), d2, ndm);
      o[2 * h + 1] = hfma2_bits(hfma2_bits(__byte_perm(n4, 0x64646464u, 0x4342), sc, off), d2, ndm);
    }
    *reinterpret_cast<uint4*>(dst_row + (((c + 4 * hh) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------ the kernel
// Activations are always fp16 here (bf16 / f32 callers go through
// convert_x_kernel first) and arrive through the tensor map. OT: output type.
// NB: 128-row halves of the weight tile (UMMA N = 128 * NB); MT * NB <= 4 (512 TMEM columns).
// RAW (q4_k fast producer, NB = 1, K-steps a multiple of 4): the wire blocks of the tile's 128 rows
// stream through a four-superblock cp.async ring in shared memory instead of per-thread register
// loads - at small M a CTA is alone on its SM and needs ~70 KB in flight to hide HBM latency.
// The ring holds whole superblocks of the tile's rows: four of 128 rows (18 KB each), or two of 256 rows (36 KB
// each) - the next superblock is then requested one superblock (four K-steps) before its first use.
__host__ __device__ constexpr int raw_depth(int NB) { return NB == 2 ? 2 : 4; }
__host__ __device__ constexpr int raw_slot(int NB) { return 128 * NB * 144; }
template <int C, int A, typename OT, int MT, int NB, bool FASTQ4, bool RAW = false, int KS = 1>
__global__ void __launch_bounds__(gemm_threads(MT, NB), 1)
gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tmap_x) {
  constexpr int kProducerThreads = producer_threads(NB), kGemmThreads = gemm_threads(MT, NB);
  constexpr int kMmaWarp = kProducerThreads / 32, kMmaWarps = mma_warps(MT);
  static_assert(!RAW || FASTQ4, "raw ring: q4_k fast producer");
  static_assert(KS == 1 || (KS == 2 && MT == 1 && NB == 1), "128-deep stages: the 128 x 128 tile only");
  constexpr int kBStages = b_stages(NB, RAW, KS), kRawDepth = raw_depth(NB), kRawSlot = raw_slot(NB);
  constexpr int kRawPieces = 128 * NB * 9;  // 16-byte pieces of one superblock of the tile's rows
  constexpr bool kHalf = std::is_same<OT, __half>::value;
  constexpr int NA = a_slots(MT, NB, RAW, KS);
  constexpr int BN = kBN * NB;
  constexpr int kBTile = NB * kTileBytes;       // one 64-deep weight tile; a stage holds KS of them
  constexpr int kBStage = KS * kBTile, kASlot = KS * kTileBytes;
  constexpr bool kIq = (C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS);
  extern __shared__ __align__(1024) uint8_t gemm_smem[];
  // 1024-byte alignment of the tiles is what the 128B swizzle pattern assumes
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* b_ring = tiles;                          // kBStages weight tiles
  uint8_t* a_ring = tiles + kBStages * kBStage;     // NA activation slots
  __shared__ uint64_t b_full[kBStages], b_empty[kBStages], a_full[NA], a_empty[NA], accum_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ __align__(16) uint8_t s_tabs[kIq ? kIqSmemBytes : 16];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  // Grouped mode: the CTA takes tile blockIdx.y of the device-built list, then every gridDim.y-th after it (the
  // grid is sized on the host for the largest list the call could produce, capped; the list is usually far
  // shorter, and a CTA with no tile leaves before it allocates anything).
  const int n_list = a.tiles != nullptr ? *a.n_tiles_dev : 0;
  if (a.tiles != nullptr && (int)blockIdx.y >= n_list) return;
  // K-steps of this CTA: all of them, or slice blockIdx.z of gridDim.z equal slices (split K, below)
  const int KB = (a.K + kBK - 1) / kBK / (int)gridDim.z;
  const int kb0 = (int)blockIdx.z * KB;
  constexpr uint32_t kTmemCols = MT * BN;               // 128, 256 or 512: a power of two >= 32

  IqTables tabs = global_iq_tables();
  if constexpr (kIq) tabs = stage_iq_tables(s_tabs, threadIdx.x, kGemmThreads);
  if (threadIdx.x == 0) abort_s = 0;
  if (warp == kMmaWarp) tmem_alloc(&tmem_base_s, kTmemCols);
  volatile int* abort_flag = &abort_s;
  uint32_t tmem_base = 0;

  for (int tile = (int)blockIdx.y;; tile += (int)gridDim.y) {
    int m0 = tile * (128 * MT), m_end = a.M;
    const uint8_t* wbase = a.w;
    if (a.tiles != nullptr) {
      const GemmTile t = a.tiles[tile];
      m0 = t.row_start;
      m_end = t.row_start + t.rows;
      wbase += (long long)t.expert * a.w_expert_stride;
    }
    const int mt_live = min(MT, (m_end - m0 + 127) / 128);  // activation tiles of this CTA that hold rows
    KQ_TR(const long long c_tile = clock64();)
    // Every tile starts from freshly initialised barriers (phase 0): nothing is in flight between tiles - the
    // loader has waited for its last loads, the issuers' MMAs have completed, the epilogue has stored.
    if (threadIdx.x == 0) {
      const bool again = tile != (int)blockIdx.y;
      for (int s = 0; s < kBStages; s++) {
        if (again) mbar_inval(&b_full[s]), mbar_inval(&b_empty[s]);
        mbar_init(&b_full[s], kProducerThreads / 32);
        mbar_init(&b_empty[s], kMmaWarps);
      }
      for (int s = 0; s < NA; s++) {
        if (again) mbar_inval(&a_full[s]), mbar_inval(&a_empty[s]);
        mbar_init(&a_full[s], 1);
        mbar_init(&a_empty[s], 1);
      }
      if (again) mbar_inval(&accum_bar);
      mbar_init(&accum_bar, kMmaWarps);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = tmem_base_s;

    if (warp < kMmaWarp) {
      // ================= weight producers =================
      const int tid = threadIdx.x;
      // NB = 1: two threads per weight row (hh = which 32 of its 64 weights); NB = 2: one thread per row
      const int wr = tid % (128 * NB);   // weight row of the tile
      const int hh0 = tid / (128 * NB);  // first 32-weight half of its 64 weights per K-step this thread makes
      constexpr int kHalves = 256 * NB / kProducerThreads;  // and how many of them
      const uint8_t* wrow = wbase + (long long)min(n0 + wr, a.N - 1) * a.row_bytes;
      bool ok = true;
      uint8_t* raw = a_ring + NA * kASlot;
      const int nsb = KB >> 2;
      auto issue_sb = [&](int sbl) {  // one copy group per superblock, an empty one past the end
        if (sbl < nsb) {
          uint8_t* slot = raw + (sbl % kRawDepth) * kRawSlot;
  #pragma unroll
          for (int i = 0; i < (kRawPieces + kProducerThreads - 1) / kProducerThreads; i++) {
            const int piece = tid + kProducerThreads * i;  // contiguous in the slot
            if (piece < kRawPieces) {
              const int row = piece / 9, pc = piece % 9;
              const uint8_t* src = wbase + (long long)min(n0 + row, a.N - 1) * a.row_bytes +
                                   (long long)((kb0 >> 2) + sbl) * 144 + pc * 16;
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(slot + piece * 16)), "l"(src)
                           : "memory");
            }
          }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
      };
      if constexpr (RAW) {
        for (int d = 0; d < kRawDepth; d++) issue_sb(d);
      }
      Q4kTileLoad cur{};
      if constexpr (FASTQ4 && !RAW) cur = q4k_tile_load(wrow, kb0);
      constexpr bool kQ6Pre = (C == Q6_K && A == 8 && NB == 1);  // 8-byte aligned rows, two threads per row
      Q6kTileLoad cur6{};
      if constexpr (kQ6Pre) cur6 = q6k_tile_load(wrow, kb0, hh0);
      KQ_TR(long long tr_wait = 0; long long tr_prod = 0; const long long c_loop = clock64();)
      {
      for (int it = 0; it < KB && (ok || RAW); it++) {
        const int kb = kb0 + it;
        const int sti = it / KS, sub = it % KS;  // stage number and 64-deep part of it
        const int s = sti % kBStages;
        if constexpr (RAW) {
          // Every producer passes every superblock barrier, also after a failed wait: nobody is left behind.
          if ((it & 3) == 0) {
            asm volatile("cp.async.wait_group %0;\n" ::"n"(kRawDepth - 2) : "memory");
            asm volatile("bar.sync 1, %0;\n" ::"n"(kProducerThreads) : "memory");  // data landed, previous slot read
            if (it > 0) issue_sb((it >> 2) - 1 + kRawDepth);
          }
          KQ_TR(const long long c0 = clock64();)
          if (ok && sub == 0 && sti >= kBStages) ok = mbar_wait(&b_empty[s], ((sti / kBStages) & 1) ^ 1, abort_flag, 1);
          KQ_TR(tr_wait += clock64() - c0;)
          if (!ok) continue;
        } else {
          KQ_TR(const long long c0 = clock64();)
          if (sub == 0 && sti >= kBStages) ok = mbar_wait(&b_empty[s], ((sti / kBStages) & 1) ^ 1, abort_flag, 1);
          KQ_TR(tr_wait += clock64() - c0;)
          if (!ok) break;
        }
        KQ_TR(const long long c1 = clock64();)
        uint8_t* wdst = b_ring + s * kBStage + sub * kBTile + wr * 128;
        if constexpr (RAW) {
          const uint8_t* blk = raw + ((it >> 2) % kRawDepth) * kRawSlot + wr * 144;
          Q4kTileLoad l;
          l.hdr = *reinterpret_cast<const uint4*>(blk);
          l.q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * (it & 3));
          l.q1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * (it & 3));
  #pragma unroll
          for (int hh = hh0; hh < hh0 + kHalves; hh++) produce_w_q4k(l, kb, wdst, wr, hh);
        } else if constexpr (FASTQ4) {
          Q4kTileLoad nxt = cur;
          if (it + 1 < KB) nxt = q4k_tile_load(wrow, kb + 1);  // next K-step's bytes are requested first
  #pragma unroll
          for (int hh = hh0; hh < hh0 + kHalves; hh++)
            produce_w_q4k(cur, kb, wdst, wr, hh);
          cur = nxt;
        } else if constexpr (kQ6Pre) {
          Q6kTileLoad nxt6 = cur6;
          if (it + 1 < KB) nxt6 = q6k_tile_load(wrow, kb + 1, hh0);  // next K-step's bytes are requested first
          produce_w_q6k_pre(cur6, wrow, kb, wdst, wr, hh0);
          cur6 = nxt6;
        } else {
  #pragma unroll
          for (int hh = hh0; hh < hh0 + kHalves; hh++) {
            if constexpr (C == Q6_K && A >= 2) produce_w_q6k<2>(wrow, kb, wdst, wr, hh);  // blocks are 2-byte aligned
            else produce_w_generic<C, A>(wrow, kb, a.K, wdst, wr, hh, tabs);
          }
        }
        if (sub == KS - 1) {
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&b_full[s]);
        }
        KQ_TR(tr_prod += clock64() - c1;)
      }
      }
      KQ_TR(if (tid == 0) { atomicAdd(&g_gemm_trace[4], (unsigned long long)tr_wait); atomicAdd(&g_gemm_trace[5], (unsigned long long)tr_prod); atomicAdd(&g_gemm_trace[6], 1ull); atomicAdd(&g_gemm_trace[9], (unsigned long long)(c_loop - c_tile)); })
      // ================= epilogue =================
      KQ_TR(const long long ce = clock64();)
      if (ok) ok = mbar_wait(&accum_bar, 0, abort_flag, 4);
      KQ_TR(if (tid == 0) atomicAdd(&g_gemm_trace[10], (unsigned long long)(clock64() - ce));)
      if (ok) {
        tc_fence_after();
        const int lq = warp & 3;                   // TMEM lane quarter this warp may read
        constexpr int kColSpan = BN / (kProducerThreads / 128);  // four warps (one per lane quarter) per column span
        const int cbeg = (warp >> 2) * kColSpan;
        if (gridDim.z > 1) {
          // split K: this CTA's partial tile goes to shared memory (the rings are idle now) as fp32
          // [rows][BN], 16-byte chunks XOR-swizzled by the row so that a warp's stores spread over the banks
          if constexpr (MT * NB <= 2) {  // 128 x 128, 256 x 128 and 128 x 256 tiles: the partial tile fits the rings
  #pragma unroll 1
            for (int h = 0; h < mt_live; h++) {
              const int rl = h * 128 + lq * 32 + lane;
              const float rs = (a.row_scale && m0 + rl < m_end) ? a.row_scale[m0 + rl] : 1.f;
              float* srow = reinterpret_cast<float*>(tiles) + rl * BN;
  #pragma unroll 1
              for (int c0 = cbeg; c0 < cbeg + kColSpan; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(h * BN + c0), v);
                tmem_ld_wait();
  #pragma unroll
                for (int i = 0; i < 4; i++)
                  *reinterpret_cast<float4*>(srow + 4 * (((c0 >> 2) + i) ^ (rl & 31))) =
                      make_float4(__uint_as_float(v[4 * i]) * rs, __uint_as_float(v[4 * i + 1]) * rs,
                                  __uint_as_float(v[4 * i + 2]) * rs, __uint_as_float(v[4 * i + 3]) * rs);
              }
            }
          }
        } else {
          // A thread owns one accumulator row (a TMEM lane): storing from here would write 32 rows x 32 bytes per
          // instruction, one memory transaction per lane. The rounded tile goes through shared memory instead (the
          // rings are idle: every MMA has completed), rows of BN outputs with their 16-byte chunks XOR-swizzled by
          // the row, and leaves as whole rows, 16 bytes per lane.
          constexpr int kRowBytes = BN * 2, kChunks = BN / 8;
          uint8_t* stage = tiles;
  #pragma unroll 1
          for (int h = 0; h < mt_live; h++) {
            const int rl = h * 128 + lq * 32 + lane;
            const float rs = (a.row_scale && m0 + rl < m_end) ? a.row_scale[m0 + rl] : 1.f;
            uint8_t* srow = stage + rl * kRowBytes;
  #pragma unroll 1
            for (int c0 = cbeg; c0 < cbeg + kColSpan; c0 += 32) {
              uint32_t va[16], vb[16];
              tmem_ld16(tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(h * BN + c0), va);
              tmem_ld16(tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(h * BN + c0 + 16), vb);
              tmem_ld_wait();
              uint32_t o[16];
  #pragma unroll
              for (int i = 0; i < 16; i++) {
                const uint32_t u0 = i < 8 ? va[2 * i] : vb[2 * i - 16], u1 = i < 8 ? va[2 * i + 1] : vb[2 * i - 15];
                const float f0 = __uint_as_float(u0) * rs, f1 = __uint_as_float(u1) * rs;
                if constexpr (kHalf) {
                  o[i] = pack_h2f(f0, f1);
                } else {
                  __nv_bfloat162 bb = __floats2bfloat162_rn(f0, f1);
                  o[i] = *reinterpret_cast<uint32_t*>(&bb);
                }
              }
  #pragma unroll
              for (int q = 0; q < 4; q++)
                *reinterpret_cast<uint4*>(srow + ((((c0 >> 3) + q) ^ (rl & (kChunks - 1))) << 4)) =
                    make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
            }
          }
          asm volatile("bar.sync 2, %0;\n" ::"n"(kProducerThreads) : "memory");
          KQ_TR(if (tid == 0) atomicAdd(&g_gemm_trace[11], (unsigned long long)(clock64() - ce));)
          const int rows_live = min(m_end - m0, mt_live * 128);
          constexpr int kRowsPerPass = 32 / kChunks;  // 1 (256 columns) or 2 (128 columns) rows per warp instruction
          const int chunk = lane % kChunks;
          const int col = n0 + chunk * 8;
          OT* ybase = static_cast<OT*>(a.y);
          // Output rows come from a table in grouped mode. A load per row inside the loop would put a global-memory
          // round trip before every store (measured: 12 k of a tile's 18 k epilogue cycles), so lane i fetches the
          // rows of pass i up front (at most 32 passes for every tile shape) and the passes read them by shuffle.
          constexpr int kPassRows = (kProducerThreads / 32) * kRowsPerPass;
          const int passes = (rows_live + kPassRows - 1) / kPassRows;
          const int sub = lane / kChunks;  // which of the pass's rows of this warp (kRowsPerPass = 2) the lane stores
          long long mine0 = 0, mine1 = 0;
          {
            const int r0 = warp * kRowsPerPass + lane * kPassRows;
            if (r0 < rows_live) mine0 = a.yrow ? (long long)a.yrow[m0 + r0] : (long long)(m0 + r0);
            if (kRowsPerPass == 2 && r0 + 1 < rows_live) mine1 = a.yrow ? (long long)a.yrow[m0 + r0 + 1] : (long long)(m0 + r0 + 1);
          }
          for (int i = 0; i < passes; i++) {
            const long long o0 = __shfl_sync(0xffffffffu, mine0, i), o1 = __shfl_sync(0xffffffffu, mine1, i);
            const int r = warp * kRowsPerPass + sub + i * kPassRows;
            if (r >= rows_live) continue;
            const long long orow = sub ? o1 : o0;
            const uint4 q = *reinterpret_cast<const uint4*>(stage + r * kRowBytes + ((chunk ^ (r & (kChunks - 1))) << 4));
            OT* yp = ybase + orow * a.y_row_stride + col;
            if (col + 8 <= a.N && (reinterpret_cast<uintptr_t>(yp) & 15) == 0) {
              *reinterpret_cast<uint4*>(yp) = q;
            } else {
              const OT* qe = reinterpret_cast<const OT*>(&q);
              for (int e = 0; e < 8; e++)
                if (col + e < a.N) yp[e] = qe[e];
            }
          }
        }
      }
      KQ_TR(if (tid == 0) atomicAdd(&g_gemm_trace[7], (unsigned long long)(clock64() - ce));)
    } else if (warp < kMmaWarp + kMmaWarps) {
      // ================= MMA issuers =================
      // Issuer w takes the row blocks h = w, w + kMmaWarps, ...; the activation tile of (K-step kb, row block h)
      // is tile number kb * mt_live + h of the loader's sequence. Every issuer arrives on every stage barrier
      // (a commit with no MMA of its own completes at once), so the counts do not depend on mt_live.
      constexpr uint32_t idesc = umma_idesc(0u, BN);
      const int w = warp - kMmaWarp;
      bool ok = true;
      KQ_TR(long long tr_b = 0; long long tr_a = 0; const long long cm = clock64();)
      for (int kb = 0; kb < KB && ok; kb++) {  // kb counts this CTA's own K-steps
        const int sti = kb / KS, sub = kb % KS;
        const int s = sti % kBStages;
        KQ_TR(const long long c0 = clock64();)
        if (sub == 0) ok = mbar_wait(&b_full[s], (sti / kBStages) & 1, abort_flag, 2);
        KQ_TR(tr_b += clock64() - c0;)
        if (!ok) break;
        const uint32_t bt = smem_u32(b_ring + s * kBStage + sub * kBTile);
        for (int h = w; h < mt_live && ok; h += kMmaWarps) {
          const int t = sti * mt_live + h;
          const int slot = t % NA;
          KQ_TR(const long long c2 = clock64();)
          if (sub == 0) ok = mbar_wait(&a_full[slot], (t / NA) & 1, abort_flag, 16);
          KQ_TR(tr_a += clock64() - c2;)
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t at = smem_u32(a_ring + slot * kASlot + sub * kTileBytes);
  #pragma unroll
            for (int j = 0; j < kBK / 16; j++)
              umma_f16(tmem_base + h * BN, umma_desc_sw128(at + j * 32), umma_desc_sw128(bt + j * 32), idesc,
                       (kb > 0 || j > 0) ? 1u : 0u);
            if (sub == KS - 1) umma_commit(&a_empty[slot]);  // the slot is free once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok && sub == KS - 1 && lane == 0) umma_commit(&b_empty[s]);
        __syncwarp();
      }
      KQ_TR(if (lane == 0 && w == 0) { atomicAdd(&g_gemm_trace[0], (unsigned long long)tr_b); atomicAdd(&g_gemm_trace[1], (unsigned long long)tr_a); atomicAdd(&g_gemm_trace[2], (unsigned long long)(clock64() - cm)); })
      if (lane == 0) umma_commit(&accum_bar);  // also on the abort path: lets the wait below see the MMAs drain
      __syncwarp();
      if (!ok) mbar_wait(&accum_bar, 0, abort_flag, 8);
    } else {
      // ================= activation loader (TMA) =================
      bool ok = true;
      int t = 0;
      KQ_TR(long long tr_e = 0;)
      for (int sti = 0; sti < KB / KS && ok; sti++) {  // one slot = the KS 64-deep boxes of a stage
        for (int h = 0; h < mt_live && ok; h++, t++) {
          const int slot = t % NA;
          KQ_TR(const long long c0 = clock64();)
          if (t >= NA) ok = mbar_wait(&a_empty[slot], ((t / NA) & 1) ^ 1, abort_flag, 32);
          KQ_TR(tr_e += clock64() - c0;)
          if (!ok) break;
          if (lane == 0) {
            mbar_expect_tx(&a_full[slot], kASlot);
  #pragma unroll
            for (int sub = 0; sub < KS; sub++)
              tma_load_2d(a_ring + slot * kASlot + sub * kTileBytes, &tmap_x, (kb0 + sti * KS + sub) * kBK, m0 + h * 128,
                          &a_full[slot]);
          }
          __syncwarp();
        }
      }
      KQ_TR(if (lane == 0) atomicAdd(&g_gemm_trace[3], (unsigned long long)tr_e);)
      // In-flight loads must have landed before the CTA may exit: wait (bounded) for the last ones.
      if (ok && t > 0) {
        const int first = t > NA ? t - NA : 0;
        for (int u = first; u < t; u++)
          if (!mbar_wait(&a_full[u % NA], (u / NA) & 1, abort_flag, 64)) break;
      }
    }

    // ================= split K: the slices of a cluster meet through distributed shared memory =================
    if (gridDim.z > 1) {
      if constexpr (MT * NB <= 2) {
        cg::cluster_group cluster = cg::this_cluster();
        tc_fence_before();
        cluster.sync();  // every slice's partial tile is in its shared memory
        const int S = (int)gridDim.z, z = (int)blockIdx.z;
        if (warp < kMmaWarp) {
          const float* peer[8];
  #pragma unroll
          for (int q = 0; q < 8; q++)
            peer[q] = q < S ? cluster.map_shared_rank(reinterpret_cast<float*>(tiles), q) : nullptr;
          for (int rl = z + S * (threadIdx.x >> 5); rl < mt_live * 128; rl += S * (kProducerThreads / 32)) {
            const int row = m0 + rl;
            if (row >= m_end) continue;
  #pragma unroll
            for (int part = 0; part < NB; part++) {
              const int c = 32 * part + (threadIdx.x & 31);  // 16-byte chunk = four columns
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  #pragma unroll
              for (int q = 0; q < 8; q++) {
                if (q < S) {
                  const float4 v = *reinterpret_cast<const float4*>(peer[q] + rl * BN + 4 * (c ^ (rl & 31)));
                  acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
                }
              }
              OT* yp = static_cast<OT*>(a.y) + (long long)row * a.y_row_stride + n0 + 4 * c;
              const float f[4] = {acc.x, acc.y, acc.z, acc.w};
  #pragma unroll
              for (int i = 0; i < 4; i++) {
                if (n0 + 4 * c + i < a.N) {
                  if constexpr (kHalf) yp[i] = __float2half_rn(f[i]);
                  else yp[i] = __float2bfloat16_rn(f[i]);
                }
              }
            }
          }
        }
        cluster.sync();  // peers may still be reading this CTA's partial tile
      }
    }

    // ================= end of the tile =================
    tc_fence_before();
    __syncthreads();
    KQ_TR(if (threadIdx.x == 0) atomicAdd(&g_gemm_trace[8], (unsigned long long)(clock64() - c_tile));)
    if (a.tiles == nullptr || tile + (int)gridDim.y >= n_list || abort_s != 0) break;
  }  // tile loop

  // ================= teardown =================
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ activation pre-pass
// bf16 / f32 activations -> fp16 for the tensor-core tile kernel (kind::f16 does
// not accept a bf16 A operand next to an fp16 B operand). float input is first
// rounded to bf16, as the reference's op does (src/kquant_ops.cpp:159-168). A
// bf16 value converts to fp16 exactly unless it is out of fp16's range, so each
// row is divided by a power of two 2^e (e = 0 for every row whose largest
// magnitude is below 32768, i.e. practically always) and the factor is handed to
// the epilogue: nothing saturates, nothing is rounded twice.
// Gather mode (order != nullptr): output row r is activation row
// lhs[order[r / M]] * M + r % M of x, and yrow[r] = order[r / M] * M + r % M says where
// its result goes; this is the expert-sorted copy the grouped kernel streams with TMA.
template <typename XT>
__global__ void __launch_bounds__(256)
convert_x_scalar_kernel(const XT* __restrict__ x, long long x_row_stride, int K, __half* __restrict__ xh,
                 float* __restrict__ row_scale, const int* __restrict__ order, const uint32_t* __restrict__ lhs, int M,
                 int* __restrict__ yrow, const int* __restrict__ n_valid) {
  const long long row = blockIdx.x;
  long long src_row = row;
  // gather mode: entries whose expert index is out of range were never placed in `order`; its tail is unset
  if (n_valid != nullptr && row >= (long long)(*n_valid) * M) return;
  if (order != nullptr) {
    const int entry = order[row / M], i = (int)(row % M);
    src_row = (long long)lhs[entry] * M + i;
    if (threadIdx.x == 0) yrow[row] = entry * M + i;
  } else if (lhs != nullptr) {
    src_row = (long long)lhs[row / M] * M + row % M;  // entry order, no sort
  }
  const XT* xr = x + src_row * x_row_stride;
  __half* o = xh + row * (long long)K;
  if constexpr (std::is_same<XT, __half>::value) {
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8)
      *reinterpret_cast<uint4*>(o + k) = __ldg(reinterpret_cast<const uint4*>(xr + k));
    if (threadIdx.x == 0) row_scale[row] = 1.f;
    return;
  } else {
    __shared__ float s_max[8];
    float mx = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) {
      float v;
      if constexpr (sizeof(XT) == 2) v = __bfloat162float(xr[k]);
      else v = __bfloat162float(__float2bfloat16_rn(xr[k]));
      v = fabsf(v);
      if (v < INFINITY) mx = fmaxf(mx, v);  // inf / nan propagate on their own
    }
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = s_max[0];
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, s_max[i]);
    // Every row is normalised: its largest magnitude lands in [16384, 32768), so small rows keep their
    // mantissas instead of turning into fp16 subnormals. The factor 2^-e is applied in two exact halves
    // (2^-e alone overflows float32 for the smallest bf16 magnitudes).
    int e = 0;
    if (mx > 0.f) e = ilogbf(mx) - 14;
    const int eh = (-e) / 2;
    const float down1 = ldexpf(1.f, eh), down2 = ldexpf(1.f, -e - eh);
    if (threadIdx.x == 0) row_scale[row] = ldexpf(1.f, e);
    for (int k = threadIdx.x; k < K; k += 256) {
      float v;
      if constexpr (sizeof(XT) == 2) v = __bfloat162float(xr[k]);
      else v = __bfloat162float(__float2bfloat16_rn(xr[k]));
      o[k] = __float2half_rn(v * down1 * down2);
    }
  }
}


// ---- the same pre-pass, eight activations per access: one warp per row, the first 2048 activations of a row
// stay in registers between the two passes (largest magnitude, then the scaled copy). Rows and K must be whole
// numbers of 16 bytes (callers fall back to the scalar kernel above otherwise).
// GLU: the source row holds gate | up (2 K values); the activation is h = silu(gate) * up, rounded to XT first -
// the value a separate activation kernel would have stored - so the fused form changes no bit of the product.
// Eight consecutive activations as four bf16 pairs (float input rounded to bf16 as the reference's op does).
template <typename XT>
__device__ __forceinline__ uint4 cvt_load8_bf16(const XT* p) {
  if constexpr (sizeof(XT) == 4) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    const __nv_bfloat162 q0 = __floats2bfloat162_rn(a.x, a.y), q1 = __floats2bfloat162_rn(a.z, a.w),
                         q2 = __floats2bfloat162_rn(b.x, b.y), q3 = __floats2bfloat162_rn(b.z, b.w);
    return make_uint4(*reinterpret_cast<const uint32_t*>(&q0), *reinterpret_cast<const uint32_t*>(&q1),
                      *reinterpret_cast<const uint32_t*>(&q2), *reinterpret_cast<const uint32_t*>(&q3));
  } else {
    return __ldg(reinterpret_cast<const uint4*>(p));
  }
}
// The fused activation over eight gate / up pairs of 16-bit type XT: h = silu(gate) * up rounded to XT, returned
// as XT pairs.
template <typename XT>
__device__ __forceinline__ uint4 cvt_glu8(const XT* xr, int K, int c) {
  const uint4 g = __ldg(reinterpret_cast<const uint4*>(xr + 8 * c));
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(xr + K + 8 * c));
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    if constexpr (std::is_same<XT, __half>::value) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&gw[i]));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&uw[i]));
      o[i] = pack_h2f(silu_f(a.x) * b.x, silu_f(a.y) * b.y);
    } else {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
      const __nv_bfloat162 h = __floats2bfloat162_rn(silu_f(a.x) * b.x, silu_f(a.y) * b.y);
      o[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}
template <typename XT, bool GLU>
__device__ __forceinline__ uint4 cvt_fetch8(const XT* xr, int K, int c) {
  if constexpr (GLU) return cvt_glu8<XT>(xr, K, c);
  else return cvt_load8_bf16<XT>(xr + 8 * c);
}
__device__ __forceinline__ __nv_bfloat162 cvt_absmax(__nv_bfloat162 m, const uint4& q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i])));  // skips NaNs
  return m;
}
__device__ __forceinline__ float cvt_finite_absmax(float m, const uint4& q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    if (fabsf(f.x) < INFINITY) m = fmaxf(m, fabsf(f.x));
    if (fabsf(f.y) < INFINITY) m = fmaxf(m, fabsf(f.y));
  }
  return m;
}
// bf16 pairs times s1 * s2 (powers of two: exact) -> fp16 pairs
__device__ __forceinline__ uint4 cvt_scale8(const uint4& q, float s1, float s2) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    o[i] = pack_h2f(f.x * s1 * s2, f.y * s1 * s2);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}
constexpr int kCvtChunks = 8;
template <typename XT, bool GLU>
__global__ void __launch_bounds__(256, 3)
convert_x_kernel(const XT* __restrict__ x, long long x_row_stride, int K, __half* __restrict__ xh,
                 float* __restrict__ row_scale, const int* __restrict__ order, const uint32_t* __restrict__ lhs,
                 int lhs_div, int M, int* __restrict__ yrow, const int* __restrict__ n_valid, long long rows) {
  static_assert(!GLU || sizeof(XT) == 2, "the fused activation takes fp16 / bf16 gate | up rows");
  const int lane = threadIdx.x & 31;
  // rows that exist: all, or the first *n_valid * M in gather mode (see the scalar kernel). The grid is capped on
  // the host and the warps stride over the rows, so a list sized for many more rows than it holds costs nothing.
  const long long limit = n_valid != nullptr ? min(rows, (long long)(*n_valid) * M) : rows;
  for (long long row = blockIdx.x * 8LL + (threadIdx.x >> 5); row < limit; row += gridDim.x * 8LL) {
    long long src_row = row;
    if (order != nullptr) {
      const int entry = order[row / M], i = (int)(row % M);
      // the activation row of an entry: that of unit u = entry / lhs_div (lhs_div = k routed rows per token when
      // the entries are a [tokens, k] routing table, else 1), through lhs when there is an index array
      const int u = entry / lhs_div;
      src_row = (lhs != nullptr ? (long long)lhs[u] : (long long)u) * M + i;
      if (lane == 0 && yrow != nullptr) yrow[row] = entry * M + i;
    } else if (lhs != nullptr) {
      src_row = (long long)lhs[row / M] * M + row % M;
    }
    const XT* xr = x + src_row * x_row_stride;
    __half* o = xh + row * (long long)K;
    const int nch = K >> 3;
    if constexpr (std::is_same<XT, __half>::value) {
      for (int c = lane; c < nch; c += 32) *reinterpret_cast<uint4*>(o + 8 * c) = cvt_fetch8<XT, GLU>(xr, K, c);
      if (lane == 0) row_scale[row] = 1.f;
    } else {
      uint4 keep[kCvtChunks];  // the row's values as bf16 pairs (they are bf16 values: nothing is lost)
      __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
  #pragma unroll
      for (int j = 0; j < kCvtChunks; j++) {
        const int c = lane + 32 * j;
        if (c < nch) {
          keep[j] = cvt_fetch8<XT, GLU>(xr, K, c);
          m2 = cvt_absmax(m2, keep[j]);
        }
      }
      for (int c = lane + 32 * kCvtChunks; c < nch; c += 32) m2 = cvt_absmax(m2, cvt_fetch8<XT, GLU>(xr, K, c));
      float mx = fmaxf(__low2float(m2), __high2float(m2));
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      if (!(mx < INFINITY)) {
        // a row with infinities: they propagate on their own, the factor comes from the finite values
        mx = 0.f;
  #pragma unroll
        for (int j = 0; j < kCvtChunks; j++)
          if (lane + 32 * j < nch) mx = cvt_finite_absmax(mx, keep[j]);
        for (int c = lane + 32 * kCvtChunks; c < nch; c += 32) mx = cvt_finite_absmax(mx, cvt_fetch8<XT, GLU>(xr, K, c));
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      }
      // Every row is normalised (see the scalar kernel); 2^-e in two exact halves, since it can overflow float32.
      int e = 0;
      if (mx > 0.f) e = ilogbf(mx) - 14;
      const int eh = (-e) / 2;
      const float down1 = ldexpf(1.f, eh), down2 = ldexpf(1.f, -e - eh);
      if (lane == 0) row_scale[row] = ldexpf(1.f, e);
  #pragma unroll
      for (int j = 0; j < kCvtChunks; j++) {
        const int c = lane + 32 * j;
        if (c < nch) *reinterpret_cast<uint4*>(o + 8 * c) = cvt_scale8(keep[j], down1, down2);
      }
      for (int c = lane + 32 * kCvtChunks; c < nch; c += 32)
        *reinterpret_cast<uint4*>(o + 8 * c) = cvt_scale8(cvt_fetch8<XT, GLU>(xr, K, c), down1, down2);
    }
  }
}

template <typename XT>
static void launch_convert_t(const void* x, long long x_row_stride, int K, long long rows, const int* order,
                             const uint32_t* lhs, int lhs_div, int M, __half* o, float* row_scale, int* yrow,
                             const int* n_valid, bool glu, bool vec, cudaStream_t st) {
  const XT* xp = static_cast<const XT*>(x);
  const unsigned gv = (unsigned)std::min<long long>((rows + 7) / 8, 148 * 64);  // strided beyond; a lower cap left a thin second pass
  if (glu) {
    if constexpr (sizeof(XT) == 2)
      convert_x_kernel<XT, true><<<gv, 256, 0, st>>>(xp, x_row_stride, K, o, row_scale, order, lhs, lhs_div, M, yrow,
                                                     n_valid, rows);
  } else if (vec) {
    convert_x_kernel<XT, false><<<gv, 256, 0, st>>>(xp, x_row_stride, K, o, row_scale, order, lhs, lhs_div, M, yrow,
                                                    n_valid, rows);
  } else {
    convert_x_scalar_kernel<XT><<<(unsigned)rows, 256, 0, st>>>(xp, x_row_stride, K, o, row_scale, order, lhs, M, yrow,
                                                                n_valid);
  }
}

// One launch of the pre-pass: rows [rows, K] of x (dtype x_dtype, row stride in elements) -> xh, row_scale.
// order / lhs / lhs_div / M / yrow / n_valid as in the kernels; glu: x rows hold gate | up (2 K values).
cudaError_t launch_convert(int x_dtype, const void* x, long long x_row_stride, int K, long long rows, const int* order,
                           const uint32_t* lhs, int lhs_div, int M, void* xh, float* row_scale, int* yrow,
                           const int* n_valid, bool glu, cudaStream_t st) {
  if (rows <= 0 || K <= 0) return cudaSuccess;
  __half* o = static_cast<__half*>(xh);
  const size_t es = x_dtype == F32 ? 4 : 2;
  const bool vec = (K % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ((size_t)x_row_stride * es) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(xh) & 15) == 0;
  if (glu && (!vec || x_dtype == F32)) return cudaErrorInvalidValue;
  if (!vec && order != nullptr && (lhs == nullptr || lhs_div != 1)) return cudaErrorInvalidValue;  // vector kernel only
  if (x_dtype == F16)
    launch_convert_t<__half>(x, x_row_stride, K, rows, order, lhs, lhs_div, M, o, row_scale, yrow, n_valid, glu, vec, st);
  else if (x_dtype == BF16)
    launch_convert_t<__nv_bfloat16>(x, x_row_stride, K, rows, order, lhs, lhs_div, M, o, row_scale, yrow, n_valid, glu,
                                    vec, st);
  else
    launch_convert_t<float>(x, x_row_stride, K, rows, order, lhs, lhs_div, M, o, row_scale, yrow, n_valid, glu, vec, st);
  return cudaGetLastError();
}

cudaError_t launch_convert_rows(int x_dtype, const void* x, long long x_row_stride, int K, long long rows,
                                const uint32_t* lhs, int M, void* xh, float* row_scale, cudaStream_t st) {
  return launch_convert(x_dtype, x, x_row_stride, K, rows, nullptr, lhs, 1, M, xh, row_scale, nullptr, nullptr, false, st);
}

size_t gemm_workspace_bytes(int x_dtype, long long rows, int K) {
  // rows 2..16 of bf16 / f32 activations use the same fp16 copy (q4_k decode kernel); one row never does
  if (x_dtype == F16 || rows <= 1) return 0;
  const size_t xh = ((size_t)rows * (size_t)K * 2 + 255) & ~(size_t)255;
  return xh + (((size_t)rows * 4 + 255) & ~(size_t)255);
}

// ------------------------------------------------------------------ launch
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of the fp16 activations [M, K] (row stride in elements): boxes of 64 x 128, 128B swizzle.
static cudaError_t make_x_map(CUtensorMap* map, const void* x, long long x_row_stride, int M, int K) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)x_row_stride * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int C, int A, typename OT, int MT, int NB, bool FASTQ4, bool RAW = false, int KS = 1>
static cudaError_t launch_g(const GemmArgs& a, cudaStream_t st, int grid_y = 0, int ksplit = 1) {
  auto kern = gemm_kernel<C, A, OT, MT, NB, FASTQ4, RAW, KS>;
  const size_t dyn = (size_t)(b_stages(NB, RAW, KS) * NB + a_slots(MT, NB, RAW, KS)) * KS * kTileBytes + 1024 +
                     (RAW ? raw_depth(NB) * raw_slot(NB) : 0);
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  alignas(64) CUtensorMap map;
  cudaError_t e = make_x_map(&map, a.x, a.x_row_stride, a.M, a.K);
  if (e != cudaSuccess) return e;
  if (MT * NB > 2) ksplit = 1;  // split K needs the fp32 partial tile in shared memory
  const dim3 grid((a.N + kBN * NB - 1) / (kBN * NB), grid_y > 0 ? grid_y : (a.M + 128 * MT - 1) / (128 * MT), ksplit);
  if (ksplit == 1) {
    kern<<<grid, gemm_threads(MT, NB), dyn, st>>>(a, map);
    return cudaGetLastError();
  }
  // split K: the ksplit CTAs of one output tile form a cluster
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(gemm_threads(MT, NB));
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = ksplit;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a, map);
}

template <int C, int A, bool FASTQ4>
static cudaError_t launch_shape(bool out_half, const GemmArgs& a, cudaStream_t st) {
  // Tile shapes (rows x columns): 512 x 128 amortises the weight dequantization best,
  // 256 x 256 halves the activation traffic out of L2; smaller ones fill the GPU at small M.
  // KQ_GEMM_TILE=1|2|4|22|12 forces 128x128 / 256x128 / 512x128 / 256x256 / 128x256 (an A/B lever).
  const long long n_tiles = (a.N + kBN - 1) / kBN;
  int mt = a.M > 256 ? 4 : (a.M > 128 ? 2 : 1);
  if (mt == 4 && n_tiles * ((a.M + 511) / 512) < 148) mt = 2;
  // the q4_k producer is cheap enough to feed a 256-column tile; decode8-based producers are not
  if (FASTQ4 && a.M > 256) mt = 22;
  static const char* const tile_env = std::getenv("KQ_GEMM_TILE");  // A/B lever, read once per process
  bool forced = false;
  if (const char* env = tile_env) {
    const int v = std::atoi(env);
    if (v == 1 || v == 2 || v == 4 || v == 22 || (v == 12 && FASTQ4 && a.M <= 128)) mt = v, forced = true;
  }
  // Few output tiles (small M on a matrix with few 128-row groups): split K over a cluster so that
  // the weights stream through more SMs. The slices must be equal: K-steps % ksplit == 0.
  const int kb_total = (a.K + kBK - 1) / kBK;
  auto pick_ksplit = [&](long long ctas) {
    int ks = 1;
    while (ks < 8 && ctas * ks * 2 <= 160 && kb_total % (ks * 2) == 0 && kb_total / (ks * 2) >= 4) ks *= 2;
    if (FASTQ4)
      while (ks > 1 && ((a.K / 256) % ks) != 0) ks >>= 1;  // q4_k producers work in whole superblocks
    return ks;
  };
  int ksplit = 1;
  if (mt == 1 || mt == 2) ksplit = pick_ksplit(n_tiles * ((a.M + 128 * mt - 1) / (128 * mt)));
  // Up to 128 rows, q4_k: a 128 x 256 tile makes a K-step's weights with one thread per weight row (64 weights,
  // one scale decode) where the 128 x 128 tile uses two (32 each): measured ~1450 cycles per K-step against
  // ~1250 for half the weights, plus ~12 k cycles per CTA and ~3 k per extra K slice. It is taken when the waves
  // it needs, times that, come out shorter - and only with at most two K slices: clusters of four or eight
  // 256-column CTAs were measured slower than the model says ([4096, 4096]: 24 us against 17 us).
  if (FASTQ4 && a.M <= 128 && ((mt == 1 && !forced) || mt == 12)) {
    const long long ctas12 = (a.N + 2 * kBN - 1) / (2 * kBN);
    const int ks12 = pick_ksplit(ctas12);
    auto cost = [&](long long ctas, int ks, double per_step) {
      return (double)((ctas * ks + 147) / 148) * ((kb_total / ks) * per_step + 12000.0 + 3000.0 * (ks - 1));
    };
    if (mt == 12 || (ks12 <= 2 && cost(ctas12, ks12, 1450.0) < cost(n_tiles, ksplit, 1250.0))) {
      mt = 12;
      ksplit = ks12;
    }
  }
  // 129 to 256 rows, q4_k: the same trade between the 256 x 128 tile (two producer threads per weight row, K may
  // be split; ~1300 cycles per K-step) and the 256 x 256 tile (one thread per row, ~1620 cycles for twice the
  // weights, no split): [28672, 8192] 184 -> 115 us.
  if (FASTQ4 && a.M > 128 && a.M <= 256 && mt == 2 && !forced) {
    auto cost = [&](long long ctas, int ks, double per_step) {
      return (double)((ctas * ks + 147) / 148) * ((kb_total / ks) * per_step + 12000.0 + 3000.0 * (ks - 1));
    };
    if (cost((a.N + 2 * kBN - 1) / (2 * kBN), 1, 1620.0) < cost(n_tiles, ksplit, 1300.0)) {
      mt = 22;
      ksplit = 1;
    }
  }
  static const char* const ksplit_env = std::getenv("KQ_GEMM_KSPLIT");  // A/B lever, read once per process
  if (const char* env = ksplit_env) {
    const int v = std::atoi(env);
    if ((v == 1 || v == 2 || v == 4 || v == 8) && kb_total % v == 0 && (!FASTQ4 || (a.K / 256) % v == 0)) ksplit = v;
  }
  // raw-block ring: whole superblocks per slice and rows that are whole numbers of 16 bytes
  static const bool no_raw = std::getenv("KQ_GEMM_NO_RAW") != nullptr;  // A/B lever
  const bool raw_ok = FASTQ4 && !no_raw && (a.K % 256) == 0 && ((a.K / 256) % ksplit) == 0 && (a.row_bytes % 16) == 0;
  // 128-deep stages for the 128 x 128 tile: every CTA's K-steps must pair up
  static const bool no_deep = std::getenv("KQ_GEMM_NO_DEEP") != nullptr;  // A/B lever
  const bool deep_ok = !no_deep && (((a.K + kBK - 1) / kBK / ksplit) % 2) == 0;
#define KQ_TILE(OT)                                                          \
  do {                                                                       \
    if (mt == 22) return launch_g<C, A, OT, 2, 2, FASTQ4>(a, st);             \
    if (mt == 4) return launch_g<C, A, OT, 4, 1, FASTQ4>(a, st);              \
    if constexpr (FASTQ4) {                                                  \
      if (mt == 12) return launch_g<C, A, OT, 1, 2, true>(a, st, 0, ksplit);  \
      if (raw_ok && mt == 2) return launch_g<C, A, OT, 2, 1, true, true>(a, st, 0, ksplit); \
      if (raw_ok && deep_ok) return launch_g<C, A, OT, 1, 1, true, true, 2>(a, st, 0, ksplit); \
      if (raw_ok) return launch_g<C, A, OT, 1, 1, true, true>(a, st, 0, ksplit);            \
    }                                                                        \
    if (mt == 2) return launch_g<C, A, OT, 2, 1, FASTQ4>(a, st, 0, ksplit);   \
    return launch_g<C, A, OT, 1, 1, FASTQ4>(a, st, 0, ksplit);                \
  } while (0)
  if (out_half) KQ_TILE(__half);
  KQ_TILE(__nv_bfloat16);
#undef KQ_TILE
}

template <int C, int NAT>
static cudaError_t launch_codec(bool out_half, const GemmArgs& a, bool aligned, cudaStream_t st) {
  return aligned ? launch_shape<C, NAT, false>(out_half, a, st) : launch_shape<C, 1, false>(out_half, a, st);
}

cudaError_t launch_gemm(int codec, int x_dtype, const void* x, long long x_row_stride, void* y, long long y_row_stride,
                        const uint8_t* w, long long row_bytes, int M, int N, int K, void* workspace, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaSuccess;
  GemmArgs a;
  a.x = x;
  a.x_row_stride = x_row_stride;
  a.y = y;
  a.y_row_stride = y_row_stride;
  a.w = w;
  a.row_bytes = row_bytes;
  a.M = M;
  a.N = N;
  a.K = K;
  a.row_scale = nullptr;
  a.tiles = nullptr;
  a.n_tiles_dev = nullptr;
  a.w_expert_stride = 0;
  a.yrow = nullptr;
  if (x_dtype != F16) {
    __half* xh = static_cast<__half*>(workspace);
    float* rs = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + (((size_t)M * K * 2 + 255) & ~(size_t)255));
    cudaError_t e = launch_convert(x_dtype, x, x_row_stride, K, M, nullptr, nullptr, 1, 1, xh, rs, nullptr, nullptr, false, st);
    if (e != cudaSuccess) return e;
    a.x = xh;
    a.x_row_stride = K;
    a.row_scale = rs;
  }
  const bool out_half = x_dtype == F16;
  const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  if (codec == Q4_K && aligned) return launch_shape<Q4_K, 16, true>(out_half, a, st);
  // q6_k rows on 8-byte boundaries (K a multiple of 1024): the producer that requests its bytes a K-step ahead
  if (codec == Q6_K && aligned && (row_bytes % 8) == 0) return launch_shape<Q6_K, 8, false>(out_half, a, st);
  switch (codec) {
    case Q2_K: return launch_codec<Q2_K, 4>(out_half, a, aligned, st);
    case Q3_K: return launch_codec<Q3_K, 2>(out_half, a, aligned, st);
    case Q4_K: return launch_codec<Q4_K, 16>(out_half, a, aligned, st);
    case Q5_K: return launch_codec<Q5_K, 16>(out_half, a, aligned, st);
    case Q6_K: return launch_codec<Q6_K, 2>(out_half, a, aligned, st);
    case Q4_0: return launch_codec<Q4_0, 2>(out_half, a, aligned, st);
    case Q8_0: return launch_codec<Q8_0, 2>(out_half, a, aligned, st);
    case IQ4_NL: return launch_codec<IQ4_NL, 2>(out_half, a, aligned, st);
    case IQ4_XS: return launch_codec<IQ4_XS, 8>(out_half, a, aligned, st);
    case IQ2_XXS: return launch_codec<IQ2_XXS, 2>(out_half, a, aligned, st);
    case Q4_1: return launch_codec<Q4_1, 4>(out_half, a, aligned, st);
    case Q5_0: return launch_codec<Q5_0, 2>(out_half, a, aligned, st);
    case Q5_1: return launch_codec<Q5_1, 8>(out_half, a, aligned, st);
    case IQ3_XXS: return launch_codec<IQ3_XXS, 2>(out_half, a, aligned, st);
    case IQ3_S: return launch_codec<IQ3_S, 2>(out_half, a, aligned, st);
    case IQ2_XS: return launch_codec<IQ2_XS, 2>(out_half, a, aligned, st);
    case IQ2_S: return launch_codec<IQ2_S, 2>(out_half, a, aligned, st);
    case IQ1_S: return launch_codec<IQ1_S, 2>(out_half, a, aligned, st);
    case IQ1_M: return launch_codec<IQ1_M, 8>(out_half, a, aligned, st);
    case MXFP4: return launch_codec<MXFP4, 1>(out_half, a, aligned, st);
    case NVFP4: return launch_codec<NVFP4, 4>(out_half, a, aligned, st);
  }
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------ grouped (MoE prefill)
// Row tiles of 256 expert-sorted rows; workspace pieces are laid out by the caller (kq_gather.cu).
template <int C, int NAT>
static cudaError_t launch_grouped_codec(bool out_half, const GemmArgs& a, bool aligned, int grid_y, cudaStream_t st) {
  if (out_half)
    return aligned ? launch_g<C, NAT, __half, 2, 1, false>(a, st, grid_y) : launch_g<C, 1, __half, 2, 1, false>(a, st, grid_y);
  return aligned ? launch_g<C, NAT, __nv_bfloat16, 2, 1, false>(a, st, grid_y)
                 : launch_g<C, 1, __nv_bfloat16, 2, 1, false>(a, st, grid_y);
}

cudaError_t launch_gemm_grouped(int codec, int x_dtype, const void* x, int M, int K, const uint8_t* w,
                                long long expert_stride, long long row_bytes, int N, const uint32_t* lhs,
                                const int* order, long long rows_total, void* y, __half* xh, float* row_scale,
                                int* yrow, const void* tiles, const int* n_tiles_dev, int max_tiles,
                                const int* n_valid_dev, cudaStream_t st) {
  if (rows_total <= 0 || N <= 0 || K <= 0) return cudaSuccess;
  cudaError_t e = launch_convert(x_dtype, x, K, K, rows_total, order, lhs, 1, M, xh, row_scale, yrow, n_valid_dev, false, st);
  if (e != cudaSuccess) return e;
  return launch_gemm_tiles(codec, x_dtype == F16, xh, rows_total, K, w, expert_stride, row_bytes, N, y,
                           x_dtype == F16 ? nullptr : row_scale, yrow, tiles, n_tiles_dev, max_tiles, st);
}

// The tile kernel over a device-built list of (expert, row_start, rows <= 256) tiles: fp16 activations xh
// [rows_total, K] (dense), output row yrow[r] (or r when yrow == nullptr), y = out_half ? fp16 : bf16.
cudaError_t launch_gemm_tiles(int codec, bool out_half, const void* xh, long long rows_total, int K, const uint8_t* w,
                              long long expert_stride, long long row_bytes, int N, void* y, const float* row_scale,
                              const int* yrow, const void* tiles, const int* n_tiles_dev, int max_tiles,
                              cudaStream_t st) {
  if (rows_total <= 0 || N <= 0 || K <= 0 || max_tiles <= 0) return cudaSuccess;
  if (max_tiles > 65535) return cudaErrorInvalidConfiguration;
  // The list may hold up to max_tiles tiles but usually holds far fewer (an expert-parallel rank sizes it for all
  // ranks' rows and owns an eighth of them): a CTA without a tile still costs about 2 us of an SM (one CTA per
  // SM by shared memory), so the grid is capped and CTAs loop over the list when it is longer.
  if (max_tiles > kTileGridCap) max_tiles = kTileGridCap;
  GemmArgs a;
  a.x = xh;
  a.x_row_stride = K;
  a.y = y;
  a.y_row_stride = N;
  a.w = w;
  a.row_bytes = row_bytes;
  a.M = (int)rows_total;
  a.N = N;
  a.K = K;
  a.row_scale = row_scale;
  a.tiles = static_cast<const GemmTile*>(tiles);
  a.n_tiles_dev = n_tiles_dev;
  a.w_expert_stride = expert_stride;
  a.yrow = yrow;
  const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (expert_stride & 15) == 0;
  if (codec == Q4_K && aligned) {
    if (out_half) return launch_g<Q4_K, 16, __half, 2, 2, true>(a, st, max_tiles);
    return launch_g<Q4_K, 16, __nv_bfloat16, 2, 2, true>(a, st, max_tiles);
  }
  if (codec == Q6_K && aligned && (row_bytes % 8) == 0 && (expert_stride % 8) == 0) {
    if (out_half) return launch_g<Q6_K, 8, __half, 2, 1, false>(a, st, max_tiles);
    return launch_g<Q6_K, 8, __nv_bfloat16, 2, 1, false>(a, st, max_tiles);
  }
  switch (codec) {
    case Q2_K: return launch_grouped_codec<Q2_K, 4>(out_half, a, aligned, max_tiles, st);
    case Q3_K: return launch_grouped_codec<Q3_K, 2>(out_half, a, aligned, max_tiles, st);
    case Q4_K: return launch_grouped_codec<Q4_K, 16>(out_half, a, aligned, max_tiles, st);
    case Q5_K: return launch_grouped_codec<Q5_K, 16>(out_half, a, aligned, max_tiles, st);
    case Q6_K: return launch_grouped_codec<Q6_K, 2>(out_half, a, aligned, max_tiles, st);
    case Q4_0: return launch_grouped_codec<Q4_0, 2>(out_half, a, aligned, max_tiles, st);
    case Q8_0: return launch_grouped_codec<Q8_0, 2>(out_half, a, aligned, max_tiles, st);
    case IQ4_NL: return launch_grouped_codec<IQ4_NL, 2>(out_half, a, aligned, max_tiles, st);
    case IQ4_XS: return launch_grouped_codec<IQ4_XS, 8>(out_half, a, aligned, max_tiles, st);
    case IQ2_XXS: return launch_grouped_codec<IQ2_XXS, 2>(out_half, a, aligned, max_tiles, st);
    case Q4_1: return launch_grouped_codec<Q4_1, 4>(out_half, a, aligned, max_tiles, st);
    case Q5_0: return launch_grouped_codec<Q5_0, 2>(out_half, a, aligned, max_tiles, st);
    case Q5_1: return launch_grouped_codec<Q5_1, 8>(out_half, a, aligned, max_tiles, st);
    case IQ3_XXS: return launch_grouped_codec<IQ3_XXS, 2>(out_half, a, aligned, max_tiles, st);
    case IQ3_S: return launch_grouped_codec<IQ3_S, 2>(out_half, a, aligned, max_tiles, st);
    case IQ2_XS: return launch_grouped_codec<IQ2_XS, 2>(out_half, a, aligned, max_tiles, st);
    case IQ2_S: return launch_grouped_codec<IQ2_S, 2>(out_half, a, aligned, max_tiles, st);
    case IQ1_S: return launch_grouped_codec<IQ1_S, 2>(out_half, a, aligned, max_tiles, st);
    case IQ1_M: return launch_grouped_codec<IQ1_M, 8>(out_half, a, aligned, max_tiles, st);
    case MXFP4: return launch_grouped_codec<MXFP4, 1>(out_half, a, aligned, max_tiles, st);
    case NVFP4: return launch_grouped_codec<NVFP4, 4>(out_half, a, aligned, max_tiles, st);
  }
  return cudaErrorInvalidValue;
}

// Device address of the error word of the current device, for kernels of other translation units.
int* device_error_word() {
  static int* addr[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kq_device_error) != cudaSuccess) return nullptr;
    addr[dev] = static_cast<int*>(p);
  }
  return addr[dev];
}

#ifdef KQ_GEMM_TRACE
extern "C" __attribute__((visibility("default"))) int kq_debug_gemm_trace(unsigned long long* out, int clear) {
  cudaMemcpyFromSymbol(out, g_gemm_trace, sizeof(g_gemm_trace));
  if (clear) {
    const unsigned long long z[12] = {};
    cudaMemcpyToSymbol(g_gemm_trace, z, sizeof(z));
  }
  return 0;
}
#endif

// Flags raised by kernels that gave up on a bounded wait (0 = none). Synchronises the device.
cudaError_t read_device_error(int* out, bool clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_kq_device_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_kq_device_error, &zero, sizeof(int));
  }
  return e;
}

}  // namespace kq
