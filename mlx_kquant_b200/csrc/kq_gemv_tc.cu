// q4_k decode product for one or two activation rows on the 5th-generation tensor cores.
//
// The mma.sync decode kernels (kq_gemv.cu) spend their time in the legacy tensor pipe: with one
// activation row seven of its eight columns are idle, and on sm_100a that pipe is slow enough to
// bound the kernel before HBM does. Here the same arithmetic runs on tcgen05:
//   * A operand = the weights of 128 rows, written by their own threads straight into TENSOR
//     MEMORY (tcgen05.st, thread = row = lane) as fp16 1024 + q (low nibbles) / 64 + q (high
//     nibbles): one three-input logic op per weight pair, no multiply, no shared-memory round trip
//     of the 4x larger fp16 tile;
//   * B operand = the activations in shared memory, laid out so that column n of the product is
//     sub-block n of the superblock: row n of a 64-wide K stage holds x only in the K slots whose
//     weights belong to sub-block n and zeros elsewhere (columns 8-15: the second activation row);
//   * D = [128 rows x 16] fp32 in tensor memory per superblock, D[r][n] = sum_k (off + q_rk) x_k
//     over sub-block n. The thread that owns row r reads it back (tcgen05.ld), removes the offsets
//     with the fp32 group sums of x and applies the 6-bit scales and d / dmin in fp32
//     (src/kquant_cpu_decode.cpp:155-174, 214-247):
//       y += d * sum_n sc_n (D_n - off_n xs_n) - dmin * sum_n mn_n xs_n.
// All products are exact in fp32 (11-bit x 11-bit significands); rounding happens only in the
// fp32 accumulation, as in the other decode kernels.
//
// grid = (ceil(N / 128), S, 1), cluster = (1, S, 1): the S CTAs of a cluster split K (at most 8
// superblocks each) and meet through distributed shared memory. Warps 0-7: weight stream
// (cp.async ring of raw blocks), A producers (two threads per row, two of a superblock's four
// 64-wide K stages each), epilogue (alternate superblocks). Warp 8: activation staging, MMA issue.
// Every mbarrier wait is bounded (2 s); on expiry the CTA raises a flag, stops issuing work,
// still passes every barrier, frees its tensor memory and returns.
//
// Status: correct (same results as the mma.sync kernels to fp16 rounding) but NOT the default.
// Measured on B200 it is slower than them (8.7 vs 5.4 us on [4096, 4096], 2.1 vs 3.9 TB/s on
// [28672, 8192]): an in-kernel clock trace shows ~65 cycles per M128 x N16 x K16 product with the
// A operand in tensor memory - sixteen of them per superblock serialise behind one issuing thread -
// and ~1.9 us from kernel entry to the first useful instruction (tensor-memory allocation, barrier
// setup). It runs only with KQ_GEMV_TC=1 in the environment and is kept as the measured record of
// that design.
#include <cooperative_groups.h>

#include <cstdlib>

#include "kq_common.cuh"
#include "kq_launch.h"
#include "kq_tcgen05.cuh"

namespace cg = cooperative_groups;

namespace kq {

__device__ int g_kq_tc_error = 0;

constexpr int kTcRows = 128;
constexpr int kTcProducers = 256;  // two threads per weight row
constexpr int kTcThreads = kTcProducers + 32;
constexpr int kTcCtlWarp = kTcProducers / 32;
constexpr int kTcMaxSb = 8;               // superblocks per CTA: 8 x 16 accumulator columns
constexpr int kTcDCols = 16;              // accumulator columns per superblock
constexpr int kTcACol0 = kTcMaxSb * kTcDCols;  // A stages start behind the accumulators
constexpr int kTcACols = 32;              // one 64-wide K stage of fp16 pairs
constexpr int kTcTmemCols = 256;          // 128 accumulator + 4 x 32 A-stage columns
constexpr int kTcSlotBytes = kTcRows * 144;  // raw ring slot: one superblock of 128 rows
constexpr int kTcBTile = 2048;            // 16 rows x 128 B, two 8-row swizzle atoms
constexpr int kTcBPerSb = 4 * kTcBTile;
constexpr int kTcMaxSplit = 8;
constexpr int kTcMaxRing = 4;

__device__ __forceinline__ void tc_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void tc_pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void tc_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void tc_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void tc_cp_async_wait(int n) {  // at most n groups still pending
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
  }
}
__device__ __forceinline__ void producer_bar() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }
// (a & mask) | magic as one three-input logic op
__device__ __forceinline__ uint32_t tc_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));
  return r;
}
__device__ __forceinline__ float tc_byte_to_float(uint32_t v, int byte) {
  // 0x4B0000bb is 2^23 + bb exactly
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 + byte)) - 8388608.f;
}
__device__ __forceinline__ void tc_cluster_sync_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
}

__global__ void __launch_bounds__(kTcThreads, 2) gemv_q4k_tc_kernel(const GemvArgs a, const int R) {
  __shared__ __align__(8) uint64_t a_full, a_free, d_ready[kTcMaxSb], x_ready;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float red[2 * 2 * kTcRows];  // [producer half][row of x][weight row]
  __shared__ __align__(16) float xs[kTcMaxSb * 16], xo[kTcMaxSb * 16];  // [superblock][row of x][sub-block]
  extern __shared__ uint8_t dyn_raw[];
  uint8_t* dyn = dyn_raw + ((1024u - (smem_u32(dyn_raw) & 1023u)) & 1023u);  // B tiles need 1024-byte alignment

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = gridDim.y, slice = blockIdx.y;
  const int nchunks = a.K >> 8;
  const int per = (nchunks + S - 1) / S;
  const int ch0 = min(slice * per, nchunks), ch1 = min(ch0 + per, nchunks);
  const int nsb = ch1 - ch0;
  const int m = min(a.M, 2);
  const int row0 = blockIdx.x * kTcRows;
  uint8_t* btiles = dyn;
  uint8_t* ring = dyn + per * kTcBPerSb;

  if (tid == 0) {
    mbar_init(&a_full, kTcProducers / 32);  // one arrival per producer warp
    mbar_init(&a_free, 1);
    for (int i = 0; i < kTcMaxSb; i++) mbar_init(&d_ready[i], 1);
    mbar_init(&x_ready, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == kTcCtlWarp) tmem_alloc(&tmem_base_s, kTcTmemCols);

  // The weight stream starts first: it depends on nothing. 1152 16-byte pieces per superblock,
  // contiguous in the slot (row * 144 + piece * 16 = 16 * piece index), four or five per thread.
  const uint8_t* src[5];
  int issued = 0;
  auto issue = [&]() {
    if (issued < nsb) {
      uint8_t* slot = ring + (issued % R) * kTcSlotBytes;
#pragma unroll
      for (int i = 0; i < 5; i++) {
        if (i < 4 || tid < 1152 - 4 * kTcProducers) tc_cp_async16(slot + 16 * (tid + kTcProducers * i), src[i]);
        src[i] += 144;
      }
      issued++;
    }
    tc_cp_async_commit();
  };
  if (warp < kTcCtlWarp) {
#pragma unroll
    for (int i = 0; i < 5; i++) {
      const int j = min(tid + kTcProducers * i, 1151);
      const int row = j / 9, piece = j % 9;
      src[i] = a.w + (long long)min(row0 + row, a.N - 1) * a.row_bytes + (long long)ch0 * 144 + piece * 16;
    }
    for (int d = 0; d < R; d++) issue();
  }
  // zeros everywhere in the B tiles; the activations land on top of them later
  for (int i = tid; i < nsb * (kTcBPerSb / 16); i += kTcThreads)
    reinterpret_cast<uint4*>(btiles)[i] = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;
  tc_pdl_launch_dependents();

  if (warp < kTcCtlWarp) {
    // ===== weight producers + epilogue: thread = (row, half of the superblock's four K stages) =====
    const int hw = warp >> 2;              // stages 2 hw, 2 hw + 1; epilogue of superblocks with j % 2 == hw
    const int r = 32 * (warp & 3) + lane;  // row of the tile = lane of tensor memory
    const uint32_t lane_field = (uint32_t)(32 * (warp & 3)) << 16;
    const uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u, kM1024 = 0x64006400u, kM64 = 0x54005400u;
    float y0 = 0.f, y1 = 0.f;
    bool ok = true;
    bool x_seen = false;
    // One lane polls, the warp follows: a whole CTA hammering one barrier word serialises.
    auto warp_wait = [&](uint64_t* bar, uint32_t parity, int code) {
      int rr = 1;
      if (lane == 0) rr = mbar_wait_err(bar, parity, abort_flag, code, &g_kq_tc_error) ? 1 : 0;
      rr = __shfl_sync(0xffffffffu, rr, 0);
      __syncwarp();
      return rr != 0;
    };
    auto epilogue = [&](int j, const uint4 hdr) {
      if (!x_seen) {
        ok = warp_wait(&x_ready, 0, 8) && ok;
        x_seen = true;
      }
      ok = warp_wait(&d_ready[j], 0, 2) && ok;
      tc_fence_after();
      uint32_t d[16];
#pragma unroll
      for (int i = 0; i < 16; i++) d[i] = 0u;
      if (ok) {
        tmem_ld16(tmem_base + lane_field + kTcDCols * j, d);
        tmem_ld_wait();
      }
      // eight 6-bit (scale, min) pairs from twelve bytes, four at a time
      const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
      const uint32_t scl = u0 & 0x3f3f3f3fu, mnl = u1 & 0x3f3f3f3fu;
      const uint32_t sch = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
      const uint32_t mnh = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
      float sc[8], mn[8];
#pragma unroll
      for (int n = 0; n < 4; n++) {
        sc[n] = tc_byte_to_float(scl, n);
        sc[4 + n] = tc_byte_to_float(sch, n);
        mn[n] = tc_byte_to_float(mnl, n);
        mn[4 + n] = tc_byte_to_float(mnh, n);
      }
      const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // (d, dmin)
#pragma unroll
      for (int tk = 0; tk < 2; tk++) {
        if (tk < m) {
          const float4* xsp = reinterpret_cast<const float4*>(xs + (j * 2 + tk) * 8);
          const float4* xop = reinterpret_cast<const float4*>(xo + (j * 2 + tk) * 8);
          const float4 s0 = xsp[0], s1 = xsp[1], o0 = xop[0], o1 = xop[1];
          const float xsv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          const float xov[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
          float a1 = 0.f, a2 = 0.f;
#pragma unroll
          for (int n = 0; n < 8; n++) {
            a1 = fmaf(sc[n], __uint_as_float(d[8 * tk + n]) - xov[n], a1);
            a2 = fmaf(mn[n], xsv[n], a2);
          }
          float& y = tk ? y1 : y0;
          y = fmaf(dd.x, a1, y);
          y = fmaf(-dd.y, a2, y);
        }
      }
    };

    uint4 hdr_mine = make_uint4(0u, 0u, 0u, 0u);
    for (int j = 0; j < nsb; j++) {
      tc_cp_async_wait(R - 1);
      producer_bar();  // every producer's pieces of this superblock have landed
      const uint8_t* blk = ring + (j % R) * kTcSlotBytes + r * 144;
      const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
      const uint4* qp = reinterpret_cast<const uint4*>(blk + 16 + 64 * hw);
      const uint4 q0 = qp[0], q1 = qp[1], q2 = qp[2], q3 = qp[3];
      producer_bar();  // every row of this slot is in registers: refill it
      issue();
      // the previous superblock's products must be done with the A stages
      ok = warp_wait(&a_free, (uint32_t)((j & 1) ^ 1), 1) && ok;
      tc_fence_after();
#pragma unroll
      for (int pp = 0; pp < 2; pp++) {
        const uint4 qa = pp ? q2 : q0, qb = pp ? q3 : q1;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t v[32];
#pragma unroll
        for (int q = 0; q < 8; q++) {
          const uint32_t W = w[q], W8 = W >> 8;
          v[4 * q + 0] = tc_and_or(W, kLo, kM1024);   // bytes 0, 2: low nibbles  -> weights 4q, 4q+2
          v[4 * q + 1] = tc_and_or(W8, kLo, kM1024);  // bytes 1, 3: low nibbles  -> weights 4q+1, 4q+3
          v[4 * q + 2] = tc_and_or(W, kHi, kM64);     // bytes 0, 2: high nibbles -> weights 32+4q, 32+4q+2
          v[4 * q + 3] = tc_and_or(W8, kHi, kM64);    // bytes 1, 3: high nibbles
        }
        if (ok) tmem_st32(tmem_base + lane_field + kTcACol0 + kTcACols * (2 * hw + pp), v);
      }
      if (ok) tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full);
      // epilogue of the previous superblock, if it is this half's, while the products run
      if (j > 0 && ((j - 1) & 1) == hw) epilogue(j - 1, hdr_mine);
      if ((j & 1) == hw) hdr_mine = hdr;
    }
    if (nsb > 0 && ((nsb - 1) & 1) == hw) epilogue(nsb - 1, hdr_mine);
    red[(hw * 2 + 0) * kTcRows + r] = y0;
    red[(hw * 2 + 1) * kTcRows + r] = y1;
  } else {
    // ================= activation staging + MMA issue =================
    if (a.tasks == nullptr) tc_pdl_wait();  // activations may come from the kernel before this one
    const int n = lane >> 2;                // sub-block of this lane's eight activations
    const int p = n >> 1, h = n & 1;
    const int q = 2 * (lane & 3);           // first of the two 16-byte K chunks they fall into
    for (int tk = 0; tk < m; tk++) {
      const __half* xrow = static_cast<const __half*>(a.x) + (long long)tk * a.x_row_stride;
      for (int j = 0; j < nsb; j++) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(xrow + (long long)(ch0 + j) * 256 + 8 * lane));
        const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        float sum = ((p0.x + p0.y) + (p1.x + p1.y)) + ((p2.x + p2.y) + (p3.x + p3.y));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) {
          xs[(j * 2 + tk) * 8 + n] = sum;
          xo[(j * 2 + tk) * 8 + n] = sum * (h ? 64.f : 1024.f);
        }
        // K slots of a chunk: weights (4c, 4c+2, 4c+1, 4c+3) of the low nibbles, then of the high ones
        uint8_t* rowp = btiles + (j * 4 + p) * kTcBTile + tk * 1024 + n * 128 + 8 * h;
        *reinterpret_cast<uint2*>(rowp + ((q ^ n) & 7) * 16) =
            make_uint2(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632));
        *reinterpret_cast<uint2*>(rowp + (((q + 1) ^ n) & 7) * 16) =
            make_uint2(__byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
      }
    }
    fence_proxy_async();  // the tensor core reads these tiles through the async proxy
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&x_ready);  // the group sums are in place for the epilogue
      constexpr uint32_t idesc = umma_idesc(0, 16);
      bool ok = true;
      for (int j = 0; j < nsb; j++) {
        ok = ok && mbar_wait_err(&a_full, (uint32_t)(j & 1), abort_flag, 4, &g_kq_tc_error);
        tc_fence_after();
        if (ok) {
#pragma unroll
          for (int pp = 0; pp < 4; pp++) {
            const uint32_t b0 = smem_u32(btiles + (j * 4 + pp) * kTcBTile);
#pragma unroll
            for (int i = 0; i < 4; i++)
              umma_f16_ts(tmem_base + kTcDCols * j, tmem_base + kTcACol0 + kTcACols * pp + 8 * i,
                          umma_desc_sw128(b0 + 32 * i), idesc, (uint32_t)((pp | i) != 0));
          }
          umma_commit(&a_free);
          umma_commit(&d_ready[j]);
        }
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  cluster.sync();  // partial sums are in place; all tensor-memory reads of this CTA are done
  if (warp == kTcCtlWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTcTmemCols);
  }
  const float* peer[kTcMaxSplit];
#pragma unroll
  for (int s = 0; s < kTcMaxSplit; s++) peer[s] = s < S ? cluster.map_shared_rank(red, s) : red;
  for (int idx = slice + S * tid; idx < kTcRows * m; idx += S * kTcThreads) {
    const int tk = idx / kTcRows, row = idx % kTcRows;
    if (row0 + row < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kTcMaxSplit; s++)
        if (s < S) sum += peer[s][tk * kTcRows + row] + peer[s][(2 + tk) * kTcRows + row];
      static_cast<__half*>(a.y)[(long long)tk * a.y_row_stride + row0 + row] = __float2half_rn(sum);
    }
  }
  tc_cluster_sync_relaxed();  // peers may still be reading this CTA's partial sums
}

// ---- host side ------------------------------------------------------------------
// Never less than 80 KB: at most two CTAs then fit on an SM, so their 2 x 256 tensor-memory columns
// always can be allocated. A third CTA would block in tcgen05.alloc while its cluster peers wait for it.
static inline int tc_dyn_smem(int per, int R) {
  const int need = 1024 + per * kTcBPerSb + R * kTcSlotBytes;
  return need < 80 * 1024 ? 80 * 1024 : need;
}

bool gemv_tc_supported(int codec, int x_dtype, const GemvArgs& a) {
  if (codec != Q4_K || x_dtype != F16 || a.tasks != nullptr || a.M < 1 || a.M > 2) return false;
  if (!a.w_align16 || (a.row_bytes & 15) != 0 || (a.K & 255) != 0) return false;
  return (a.K >> 8) <= kTcMaxSb * kTcMaxSplit;
}

cudaError_t launch_gemv_tc(const GemvArgs& a, cudaStream_t st) {
  const int nchunks = a.K >> 8;
  const int row_tiles = (a.N + kTcRows - 1) / kTcRows;
  int S = 1;
  while ((nchunks + S - 1) / S > kTcMaxSb) S *= 2;
  // few row tiles: split K further, as long as both this launch and the next one fit on the chip
  while (S < kTcMaxSplit && S * 2 <= nchunks && row_tiles * S * 2 <= 160) S *= 2;
  if (const char* env = std::getenv("KQ_TC_SPLIT")) {  // A/B lever
    const int v = std::atoi(env);
    if ((v == 1 || v == 2 || v == 4 || v == 8) && v <= nchunks && (nchunks + v - 1) / v <= kTcMaxSb) S = v;
  }
  const int per = (nchunks + S - 1) / S;
  int R = per < kTcMaxRing ? per : kTcMaxRing;
  while (R > 1 && tc_dyn_smem(per, R) > 110 * 1024) R--;  // two CTAs per SM
  if (const char* env = std::getenv("KQ_TC_RING")) {  // A/B lever
    const int v = std::atoi(env);
    if (v >= 1 && v <= kTcMaxRing) R = v;
  }
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tc_dyn_smem(kTcMaxSb, kTcMaxRing));
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(row_tiles, S, 1);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = tc_dyn_smem(per, R);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 1 : 2;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_tc_kernel, a, R);
}

cudaError_t read_device_error_tc(int* out, bool clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_kq_tc_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_kq_tc_error, &zero, sizeof(int));
  }
  return e;
}

}  // namespace kq
